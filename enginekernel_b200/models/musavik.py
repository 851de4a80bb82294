"""Musavik decoder: configuration -> model description.

x = embed[id] * s + pairs[hash(previous id, id)] (the last row of ``pairs`` for a sequence's first token).
Every layer has a norm before and a norm behind each sublayer (``parts/block.py``, ``sandwich``), all norms with
a weight stored around zero (factor 1 + w): x += n1b(mixer(n1(x))), x += n2b(ff(n2(x))).  Mixers: a gated linear
recurrence (``gated_linear_recurrence`` in ``parts/recurrent.py``), or two mixers side by side whose results are
summed with two constants (``parts/pair.py``): attention whose heads share their softmax weights, with biases,
a gained norm of queries and keys before a rotation of neighbouring pairs, unit values, a window that keeps a
sequence's first tokens and an element-wise output gate (``parts/mixed_attention.py``), and the delta rule with
one decay per head (``head_delta`` in ``parts/delta.py``).  Feed-forward: down(gelu_tanh(up(h))) with biases
(``dense_mlp`` in ``parts/mlp.py``).  A stretch of layers may run several times with the same weights, each pass
with cache entries of its own; right before the first layer of every pass x <- W_in [x ; x0] with x0 the
embedding output (``RunSpec.mix_input``).  Output: the same kind of norm, then logits against ``head``.

Tensor names: ``embed``, ``bigram``, ``loop.in``, ``final.norm``, ``head``, per layer i ``l<i>.norm1``, ``norm1b``,
``norm2``, ``norm2b``, ``l<i>.mix.*`` and ``l<i>.mlp.*``.  This module only names parts and sizes; the parts know
nothing of Musavik.
"""

from __future__ import annotations

from ..config.musavik import MusavikConfig, RglruConfig, SideBySideConfig
from ..parts.spec import LayerSpec, ModelSpec, PairTableSpec, PartSpec, RunSpec, TensorSpec
from ..registry import register_architecture

MAX_POSITIONS = 1 << 30      # the design sets no limit; positions are 32-bit on the device
LRU_RATE = 8.0               # log a = -8 r softplus(lam): fixed by the design


def _mixer(cfg: MusavikConfig, m, p: str) -> PartSpec:
    if isinstance(m, RglruConfig):
        return PartSpec(
            "gated_linear_recurrence",
            {"hidden_size": cfg.width, "width": m.width, "blocks": m.blocks, "conv": m.conv, "rate": LRU_RATE},
            {"y": p + "y", "y_bias": p + "y.b", "x": p + "x", "x_bias": p + "x.b", "conv": p + "conv",
             "conv_bias": p + "conv.b", "a_gate": p + "ra", "a_gate_bias": p + "ra.b", "i_gate": p + "ri",
             "i_gate_bias": p + "ri.b", "lam": p + "lam", "o": p + "o"})
    assert isinstance(m, SideBySideConfig)
    a, d = m.left, m.right
    lp, rp = p + "left.", p + "right."
    position = None
    if a.rot_dims > 0:
        position = PartSpec("rope_stretched", {"rotary_dim": a.rot_dims, "theta": a.rot_base})
    left = PartSpec(
        "mixed_head_attention",
        {"hidden_size": cfg.width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
         "value_dim": a.vdim, "scale": a.scale, "eps": cfg.norm_eps, "window": a.window, "keep_first": a.keep_first,
         "position": position},
        {"q": lp + "q", "q_bias": lp + "q.b", "k": lp + "k", "k_bias": lp + "k.b", "v": lp + "v", "v_bias": lp + "v.b",
         "q_norm": lp + "q.norm", "k_norm": lp + "k.norm", "mix": lp + "talk", "gate": lp + "g", "o": lp + "o"})
    right = PartSpec(
        "head_delta",
        {"hidden_size": cfg.width, "num_heads": d.heads, "num_kv_heads": d.kv_heads, "head_dim": d.dim,
         "v_dim": d.vdim, "conv": d.conv, "eps": cfg.norm_eps},
        {"q": rp + "q", "k": rp + "k", "v": rp + "v", "q_conv": rp + "q.conv", "k_conv": rp + "k.conv",
         "v_conv": rp + "v.conv", "b": rp + "b", "a": rp + "a", "A_log": rp + "A_log", "dt_bias": rp + "dt_bias",
         "g": rp + "g", "norm": rp + "norm", "o": rp + "o"})
    return PartSpec("mixer_pair", {"first": left, "second": right, "weight_first": m.left_scale,
                                   "weight_second": m.right_scale})


def build_musavik(cfg: MusavikConfig) -> ModelSpec:
    def norm(name):
        return PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps, "one_plus": True}, {"gain": name})

    layers, ignorable = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        norms = {"pre_mixer": norm(p + "norm1"), "post_mixer": norm(p + "norm1b")}
        ffn = None
        if layer.mlp is not None:
            norms.update(pre_feed_forward=norm(p + "norm2"), post_feed_forward=norm(p + "norm2b"))
            m = p + "mlp."
            ffn = PartSpec("dense_mlp", {"hidden_size": cfg.width, "intermediate_size": layer.mlp.ff,
                                         "activation": "gelu_tanh", "bias": True},
                           {"up": m + "up", "up_bias": m + "up.b", "down": m + "down", "down_bias": m + "down.b"})
        else:                                   # a file may keep the unused sublayer's norms
            ignorable += [p + "norm2", p + "norm2b"]
        layers.append(LayerSpec(PartSpec("sandwich", {"hidden_size": cfg.width}), _mixer(cfg, layer.mixer, p + "mix."),
                                ffn, norms))

    # every run of a layer has cache entries of its own: one, or two for a pair of mixers
    schedule, entries = [], 0
    for i, _, starts_pass in cfg.runs():
        pair = isinstance(cfg.layers[i].mixer, SideBySideConfig)
        schedule.append(RunSpec(i, entries, mix_input=starts_pass, more_caches=(entries + 1,) if pair else ()))
        entries += 2 if pair else 1
    # (a file may keep the tensors of an input mix or a pair table that its configuration does not use)
    if cfg.loop is None:
        ignorable.append("loop.in")
    if cfg.pair_table is None:
        ignorable.append("bigram")
    pairs = None
    if cfg.pair_table is not None:
        t = cfg.pair_table
        pairs = PairTableSpec(TensorSpec("bigram", (t.buckets + 1, cfg.width), "embedding"), t.buckets, t.mul_prev,
                              t.mul_cur, cache=entries)
    spec = ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding=TensorSpec("embed", (cfg.vocab, cfg.width), "embedding"), layers=layers, schedule=schedule,
        final_norm=norm("final.norm"), lm_head=TensorSpec("head", (cfg.vocab, cfg.width), "linear"),
        embedding_multiplier=cfg.embedding_scale, ignorable=tuple(ignorable), pair_table=pairs,
        input_mix=TensorSpec("loop.in", (cfg.width, 2 * cfg.width), "linear") if cfg.loop is not None else None)
    spec.check()
    return spec


register_architecture(MusavikConfig.architecture, MusavikConfig, build_musavik)
