"""Bolelix without a GPU: reading the configuration, the schedule with shared cache entries, the tensors
the model asks for, the divided rotation's tables, and the plain implementation against itself."""

import copy
import json
import math

import pytest
import torch

from enginekernel_b200 import registry
from enginekernel_b200.config.base import ConfigError
from enginekernel_b200.config.bolelix import BolelixConfig
from enginekernel_b200.engine.model import expected_tensors, ignorable_tensors
from enginekernel_b200.parts.spec import PartSpec
from tests.plain import bolelix_models as models
from tests.plain import bolelix_plain as plain

F64 = torch.float64


def test_registered_and_chosen_by_the_architecture_key(tmp_path):
    assert "Bolelix" in registry.architectures()
    for tag, raw in models.SHAPES.items():
        folder = models.write_folder(str(tmp_path / tag), raw, {})
        cfg = registry.config_from_folder(folder)
        assert isinstance(cfg, BolelixConfig)
        assert cfg.to_dict() == raw
        assert BolelixConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg


@pytest.mark.parametrize("tag", list(models.SHAPES))
def test_schedule_parts_and_tensors_follow_the_configuration(tag):
    raw = models.SHAPES[tag]
    spec = registry.model_spec_for(BolelixConfig.from_dict(raw))
    assert [r.layer for r in spec.schedule] == list(range(len(raw["layers"])))
    want = models.tensor_shapes(raw)
    got = expected_tensors(spec)
    assert set(got) == set(want)
    for name, shape in want.items():
        assert got[name].fits(shape), (name, got[name].shape, shape)
    assert spec.embedding_multiplier == raw["embedding"]["scale"]
    assert spec.lm_head.optional_alias is None                       # the head is a tensor of its own
    entries = {}
    for i, (layer, run) in enumerate(zip(raw["layers"], spec.schedule)):
        ls = spec.layers[i]
        assert ls.block.kind == "parallel" and list(ls.norms) == ["pre_mixer"]
        assert ls.mixer.kind == {"attention": "attention", "mamba2": "state_space", "mlstm": "matrix_memory"}[layer["type"]]
        assert (ls.feed_forward is None) == (layer["mlp"] is None)
        assert (f"l{i}.ls2" in ignorable_tensors(spec)) == (layer["mlp"] is None)
        src = layer["mixer"].get("kv_from")
        if src is None:                                              # an entry of its own, in order
            assert run.writes_cache and run.cache == len(entries)
            entries[i] = run.cache
        else:                                                        # reads the entry of the layer it names
            assert not run.writes_cache and run.cache == entries[src]
            assert not ls.mixer.params["kv_projection"]
    assert spec.num_cache_entries() == len(entries)


@pytest.mark.parametrize("change,match", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_heads"), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["rot"].pop("base"), "base"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), "groups"),
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][2]["mixer"].update(gate_cap=0.0), "gate_cap"),
    (lambda c: c["layers"][0].update(type="window"), "not a Bolelix mixer"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not a Bolelix feed-forward"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=24), "equal those of layer 0"),
])
def test_bad_configurations_are_refused_by_name(change, match):
    raw = copy.deepcopy(models.MIXED)
    change(raw)
    with pytest.raises(ConfigError, match=match):
        BolelixConfig.from_dict(raw)


@pytest.mark.parametrize("dims,base,factor", [(16, 10000.0, 2.0), (10, 1e6, 8.0), (32, 500.0, None), (4, 10.0, 1.5)])
def test_divided_rotation_tables(dims, base, factor):
    from enginekernel_b200.parts.rope import RopeStretched
    params = {"rotary_dim": dims, "theta": base}
    if factor is not None:
        params["divide"] = factor
    part = RopeStretched(PartSpec("rope_stretched", params), torch.float32, "cpu")
    part.prepare(300)
    f = plain.rotation_frequencies(dims, base, factor or 1.0)
    assert abs(float(f[1]) - base ** (-2.0 / dims) / (factor or 1.0)) < 1e-15
    ang = torch.arange(300, dtype=F64)[:, None] * f[None, :]
    assert part.cos.shape == (300, dims // 2) and part.rotary_dim == dims
    assert (part.cos.double() - torch.cos(ang)).abs().max() < 1e-6
    assert (part.sin.double() - torch.sin(ang)).abs().max() < 1e-6


def test_plain_visibility_and_rotation():
    see = lambda i, j: plain.visible(i, j, 5, 2)
    assert see(10, 10) and see(10, 6) and not see(10, 5) and see(10, 1) and see(10, 0) and not see(10, 2)
    assert not see(3, 4) and plain.visible(900, 0, None, 0)
    x = torch.randn(3, 2, 12, dtype=F64, generator=torch.Generator().manual_seed(0))
    y = plain.rotate(x, torch.tensor([0, 5, 9]), 8, 100.0, 2.0)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 8:], x[..., 8:])         # position 0 and the tail pass
    assert (y.norm(dim=-1) - x.norm(dim=-1)).abs().max() < 1e-12
    a = 5 * 100.0 ** (-2.0 / 8) / 2.0                                               # dimension 1 turns with 5
    assert abs(float(y[1, 0, 1]) - float(x[1, 0, 1] * math.cos(a) - x[1, 0, 5] * math.sin(a))) < 1e-12
    assert abs(float(y[1, 0, 5]) - float(x[1, 0, 5] * math.cos(a) + x[1, 0, 1] * math.sin(a))) < 1e-12


def test_plain_recurrences_against_closed_forms():
    g = torch.Generator().manual_seed(1)
    # one token through the matrix memory from nothing: m = max(f, i) with m_0 = 0, S = exp(i - m) k v^T, n likewise
    w = {"q": torch.randn(4, 6, generator=g), "k": torch.randn(4, 6, generator=g), "v": torch.randn(3, 6, generator=g),
         "g": torch.zeros(3, 6), "i": torch.randn(1, 6, generator=g), "i.b": torch.randn(1, generator=g),
         "f": torch.randn(1, 6, generator=g), "f.b": torch.randn(1, generator=g), "norm": torch.ones(3), "o": torch.eye(3)}
    m = {"heads": 1, "dim": 4, "vdim": 3, "gate_cap": 2.0}
    h = torch.randn(1, 6, generator=g, dtype=F64)
    q, k, v = (w[n].double() @ h[0] for n in "qkv")
    q = q / 2.0
    i = 2.0 * math.tanh(float(w["i"].double() @ h[0] + w["i.b"].double()) / 2.0)
    f = -math.log1p(math.exp(-2.0 * math.tanh(float(w["f"].double() @ h[0] + w["f.b"].double()) / 2.0)))
    mx = max(f, i)
    put = math.exp(i - mx)
    o = put * float(k @ q) * v / (max(abs(put * float(k @ q)), math.exp(-mx)) + 1e-6)
    want = 0.5 * plain.rms_unit(o, 1e-5)                          # the gate projection is zero: sigmoid = 1/2
    assert (plain.mlstm(h, w, "", m, 1e-5)[0] - want).abs().max() < 1e-12
    # the convolution's last column multiplies the current token, and what came before can be handed in
    x = torch.randn(7, 3, generator=g, dtype=F64)
    cw, cb = torch.randn(3, 4, generator=g, dtype=F64), torch.randn(3, generator=g, dtype=F64)
    full = plain.causal_conv(x, cw, cb)
    assert (full[0] - (x[0] * cw[:, 3] + cb)).abs().max() < 1e-12
    assert (plain.causal_conv(x[4:], cw, cb, before=x[1:4]) - full[4:]).abs().max() < 1e-12


def test_plain_router_weights_are_the_softmax_of_the_chosen_logits():
    g = torch.Generator().manual_seed(2)
    h, wr = torch.randn(50, 12, generator=g, dtype=F64), torch.randn(8, 12, generator=g)
    idx, wt = plain.route(h, wr, 3)
    z = h @ wr.double().T
    assert (idx == z.topk(3, -1).indices).all() and (wt.sum(-1) - 1).abs().max() < 1e-12
    assert (wt[:, 0] / wt[:, 1] - torch.exp(z.gather(1, idx)[:, 0] - z.gather(1, idx)[:, 1])).abs().max() < 1e-9


def test_plain_model_is_causal_and_shared_keys_are_the_source_layers():
    cfg = models.MIXED
    w = models.make_tensors(cfg, 3)
    ids = models.random_prompts(cfg, [40], seed=1)[0]
    full = plain.forward(cfg, w, ids)
    assert (plain.forward(cfg, w, ids[:17]) - full[:17]).abs().max() < 1e-9
    # the last layer has no keys of its own: changing layer 0's key projection moves the model through both
    w2 = dict(w)
    w2["l0.mix.k"] = w["l0.mix.k"].flip(0)
    assert (plain.forward(cfg, w2, ids) - full).abs().max() > 1e-3
    assert "l3.mix.k" not in models.tensor_shapes(cfg)
