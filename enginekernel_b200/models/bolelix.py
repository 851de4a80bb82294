"""Bolelix decoder: configuration -> model description.

x = embed[id] * s.  Every layer is parallel: with u = rms(x) w, x += ls1 * mixer(u) + ls2 * ff(u), one norm
read by both sublayers and a learned scale per channel on each result (``parts/block.py``, ``parallel``).
Mixers: grouped-query attention with a partial rotation whose frequencies are divided by a factor, unit
queries and keys after the rotation, a sliding window that also keeps a sequence's first tokens, a sigmoid
gate per head, value heads of a size of their own, and optionally the keys and values of an earlier layer
instead of its own (``parts/attention.py``); a state-space layer (``state_space``) or a matrix memory with
exponential gates (``matrix_memory``), both in ``parts/recurrent.py``.  Feed-forward: routed experts with a
SiLU gate, the largest logits chosen and weighted by the softmax over the chosen ones (``parts/moe.py``).
Output: RMS norm, then logits against ``head``.

Tensor names: ``embed``, ``final.norm``, ``head``, per layer i ``l<i>.norm1``, ``l<i>.ls1``, ``l<i>.ls2``,
``l<i>.mix.*`` and ``l<i>.mlp.*``.  This module only names parts and sizes; the parts know nothing of Bolelix.
"""

from __future__ import annotations

from ..config.bolelix import BolelixConfig, Mamba2Config, MlstmConfig, WindowAttentionConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunSpec, TensorSpec
from ..registry import register_architecture

MAX_POSITIONS = 1 << 30      # the design sets no limit; positions are 32-bit on the device


def _mixer(cfg: BolelixConfig, m, p: str) -> PartSpec:
    if isinstance(m, WindowAttentionConfig):
        position = None
        if m.rot_dims > 0:
            position = PartSpec("rope_stretched", {"rotary_dim": m.rot_dims, "theta": m.rot_base,
                                                   "divide": m.rot_factor})
        weights = {"q": p + "q", "gate": p + "g", "o": p + "o"}
        if m.kv_from is None:
            weights.update(k=p + "k", v=p + "v")
        return PartSpec(
            "attention",
            {"hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
             "value_dim": m.vdim, "scale": m.scale, "window": m.window, "keep_first": m.keep_first,
             "unit_norm_after_rotation": cfg.norm_eps, "head_gate": True, "kv_projection": m.kv_from is None,
             "keep_all_keys": True, "position": position},
            weights)
    if isinstance(m, Mamba2Config):
        return PartSpec(
            "state_space",
            {"hidden_size": cfg.width, "num_heads": m.heads, "v_dim": m.vdim, "state": m.state, "groups": m.groups,
             "conv": m.conv, "norm_groups": m.norm_groups, "eps": cfg.norm_eps},
            {"in": p + "in", "conv": p + "conv", "conv_bias": p + "conv.b", "dt_bias": p + "dt_bias",
             "A_log": p + "A_log", "D": p + "D", "norm": p + "norm", "o": p + "o"})
    assert isinstance(m, MlstmConfig)
    return PartSpec(
        "matrix_memory",
        {"hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "v_dim": m.vdim, "gate_cap": m.gate_cap,
         "eps": cfg.norm_eps},
        {"q": p + "q", "k": p + "k", "v": p + "v", "g": p + "g", "i": p + "i", "f": p + "f", "i_bias": p + "i.b",
         "f_bias": p + "f.b", "norm": p + "norm", "o": p + "o"})


def _feed_forward(cfg: BolelixConfig, mlp, p: str) -> PartSpec:
    weights = {"router": p + "router"}
    for e in range(mlp.experts):
        weights[f"gate_{e}"] = f"{p}e{e}.gate"
        weights[f"up_{e}"] = f"{p}e{e}.up"
        weights[f"down_{e}"] = f"{p}e{e}.down"
    return PartSpec("routed_experts",
                    {"hidden_size": cfg.width, "intermediate_size": mlp.ff, "experts": mlp.experts, "top": mlp.top,
                     "activation": "silu", "gated": True, "weights": "softmax_of_chosen"}, weights)


def build_bolelix(cfg: BolelixConfig) -> ModelSpec:
    layers, schedule, ignorable, entry_of = [], [], [], {}
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        norms = {"pre_mixer": PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps}, {"gain": p + "norm1"})}
        scales = {"mixer_scale": p + "ls1"}
        ffn = None
        if layer.mlp is not None:
            ffn = _feed_forward(cfg, layer.mlp, p + "mlp.")
            scales["feed_forward_scale"] = p + "ls2"
        else:                                   # a file may keep the unused sublayer's scale
            ignorable.append(p + "ls2")
        block = PartSpec("parallel", {"hidden_size": cfg.width}, scales)
        layers.append(LayerSpec(block, _mixer(cfg, layer.mixer, p + "mix."), ffn, norms))
        src = getattr(layer.mixer, "kv_from", None)
        if src is None:
            entry_of[i] = len(entry_of)
            schedule.append(RunSpec(i, entry_of[i]))
        else:                                   # reads what layer `src` stored in this step and before
            schedule.append(RunSpec(i, entry_of[src], writes_cache=False))

    spec = ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding=TensorSpec("embed", (cfg.vocab, cfg.width), "embedding"), layers=layers, schedule=schedule,
        final_norm=PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps}, {"gain": "final.norm"}),
        lm_head=TensorSpec("head", (cfg.vocab, cfg.width), "linear"),
        embedding_multiplier=cfg.embedding_scale, ignorable=tuple(ignorable))
    spec.check()
    return spec


register_architecture(BolelixConfig.architecture, BolelixConfig, build_bolelix)
