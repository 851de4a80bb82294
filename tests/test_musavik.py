"""Musavik without a GPU: reading the configuration, the schedule of a looped stretch with its cache entries,
the tensors the model asks for, the reordering that turns neighbouring rotation pairs into half-split ones,
and the plain implementation against closed forms."""

import copy
import json
import math

import pytest
import torch

from enginekernel_b200 import registry
from enginekernel_b200.config.base import ConfigError
from enginekernel_b200.config.musavik import MusavikConfig
from enginekernel_b200.engine.model import expected_tensors, ignorable_tensors
from enginekernel_b200.parts.mixed_attention import neighbours_to_halves
from tests.plain import musavik_models as models
from tests.plain import musavik_plain as plain

F64 = torch.float64


def test_registered_and_chosen_by_the_architecture_key(tmp_path):
    assert "Musavik" in registry.architectures()
    for tag, raw in models.SHAPES.items():
        folder = models.write_folder(str(tmp_path / tag), raw, {})
        cfg = registry.config_from_folder(folder)
        assert isinstance(cfg, MusavikConfig)
        assert cfg.to_dict() == raw
        assert MusavikConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg


@pytest.mark.parametrize("tag", list(models.SHAPES))
def test_schedule_parts_and_tensors_follow_the_configuration(tag):
    raw = models.SHAPES[tag]
    spec = registry.model_spec_for(MusavikConfig.from_dict(raw))
    runs = plain.layer_runs(raw)
    assert [(r.layer, r.mix_input) for r in spec.schedule] == runs
    want = models.tensor_shapes(raw)
    got = expected_tensors(spec)
    assert set(got) == set(want)
    for name, shape in want.items():
        assert got[name].fits(shape), (name, got[name].shape, shape)
    assert spec.embedding_multiplier == raw["embedding"]["scale"]
    assert (spec.pair_table is None) == ("bigram" not in raw["embedding"])
    assert (spec.input_mix is None) == ("loop" not in raw)
    used = []
    for run in spec.schedule:                                        # every run has entries of its own
        layer = raw["layers"][run.layer]
        ls = spec.layers[run.layer]
        assert ls.block.kind == "sandwich"
        assert ls.mixer.kind == {"rglru": "gated_linear_recurrence", "parallel": "mixer_pair"}[layer["type"]]
        assert len(run.more_caches) == (1 if layer["type"] == "parallel" else 0)
        assert (ls.feed_forward is None) == (layer["mlp"] is None)
        assert set(ls.norms) == {"pre_mixer", "post_mixer"} | ({"pre_feed_forward", "post_feed_forward"} if layer["mlp"] else set())
        assert (f"l{run.layer}.norm2" in ignorable_tensors(spec)) == (layer["mlp"] is None)
        used += [run.cache, *run.more_caches]
    if spec.pair_table is not None:
        used.append(spec.pair_table.cache)
    assert sorted(used) == list(range(spec.num_cache_entries()))


def test_what_the_configuration_refuses():
    base = models.SHAPES["early"]

    def broken(change):
        raw = copy.deepcopy(base)
        change(raw)
        return raw

    cases = {
        "vocab": lambda r: r.pop("vocab"),
        "norm": lambda r: r.pop("norm"),
        "embedding": lambda r: r.pop("embedding"),
        "layers": lambda r: r.update(layers=[]),
        "type": lambda r: r["layers"][1].update(type="attention"),
        "blocks": lambda r: r["layers"][2]["mixer"].update(blocks=3),
        "left": lambda r: r["layers"][0]["mixer"].pop("left"),
        "kv_heads": lambda r: r["layers"][0]["mixer"]["left"].update(kv_heads=3),
        "rot.dims": lambda r: r["layers"][0]["mixer"]["left"]["rot"].update(dims=26),
        "keep_first": lambda r: r["layers"][0]["mixer"]["left"].update(mask={"keep_first": 2}),
        "left_scale": lambda r: r["layers"][0]["mixer"].pop("left_scale"),
        "conv": lambda r: r["layers"][0]["mixer"]["right"].update(conv=0),
        "kind": lambda r: r["layers"][0]["mlp"].update(kind="moe"),
        "loop": lambda r: r["loop"].update(stop=4),
        "buckets": lambda r: r["embedding"]["bigram"].update(buckets=0),
        "width": lambda r: r.update(width=96.5),
    }
    for word, change in cases.items():
        with pytest.raises(ConfigError, match=word.replace(".", r"\.")):
            MusavikConfig.from_dict(broken(change))


def test_a_model_description_must_be_consistent():
    from enginekernel_b200.parts.spec import RunSpec
    import dataclasses
    spec = registry.model_spec_for(MusavikConfig.from_dict(models.SHAPES["flat"]))
    with pytest.raises(ValueError, match="input_mix"):
        dataclasses.replace(spec, schedule=[RunSpec(0, 0, mix_input=True)] + spec.schedule[1:]).check()
    with pytest.raises(ValueError, match="further cache entry"):
        dataclasses.replace(spec, schedule=[spec.schedule[0], RunSpec(1, 1, more_caches=(0,))] + spec.schedule[2:]).check()


# ------------------------------------------------------------------ the plain implementation against closed forms
def test_pair_rows_and_the_first_token():
    assert plain.pair_rows([5, 9, 9, 0], 7, 3, 2) == [7, (5 * 3 + 9 * 2) % 7, (9 * 3 + 9 * 2) % 7, (9 * 3) % 7]
    assert plain.pair_rows([4], 11, 1000, 999) == [11]


@pytest.mark.parametrize("dim,rot", [(8, 8), (12, 6), (20, 0), (6, 2)])
def test_neighbouring_pairs_become_half_split_pairs_without_changing_scores(dim, rot):
    """Reordering queries and keys alike and turning (i, i + rot/2) gives the scores of turning (2i, 2i + 1)."""
    g = torch.Generator().manual_seed(dim)
    q, k = torch.randn(5, 2, dim, generator=g, dtype=F64), torch.randn(5, 2, dim, generator=g, dtype=F64)
    pos = torch.tensor([0, 1, 7, 300, 301])
    want = torch.einsum("thd,shd->hts", plain.rotate_pairs(q, pos, rot, 100.0), plain.rotate_pairs(k, pos, rot, 100.0))
    order = neighbours_to_halves(dim, rot)
    assert sorted(order.tolist()) == list(range(dim))

    def half_split(x):
        x = x[..., order]
        if not rot:
            return x
        half = rot // 2
        ang = pos.to(F64)[:, None] * 100.0 ** (-2.0 * torch.arange(half, dtype=F64) / rot)[None, :]
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
        a, b = x[..., :half], x[..., half:rot]
        return torch.cat([a * c - b * s, b * c + a * s, x[..., rot:]], -1)

    got = torch.einsum("thd,shd->hts", half_split(q), half_split(k))
    assert torch.allclose(got, want, atol=1e-12)


def test_recurrence_with_constant_gates_is_a_geometric_sum():
    """r and i constant: S_t = sum_j a^(t-j) sqrt(1 - a^2) i u_j."""
    t, width = 9, 4
    u = torch.arange(t * width, dtype=F64).view(t, width) / 10 - 1
    r, i = torch.full((t, width), 0.3, dtype=F64), torch.full((t, width), 0.6, dtype=F64)
    lam = torch.tensor([-1.0, 0.0, 0.5, 2.0], dtype=F64)
    a = torch.exp(-8 * 0.3 * torch.log1p(torch.exp(lam)))
    s, last = plain.rglru_scan(u, r, i, lam)
    want = torch.stack([sum(a ** (n - j) * torch.sqrt(1 - a * a) * 0.6 * u[j] for j in range(n + 1)) for n in range(t)])
    assert torch.allclose(s, want, atol=1e-12) and torch.equal(last, s[-1])
    s2, _ = plain.rglru_scan(u[5:], r[5:], i[5:], lam, state=s[4])           # carried on from a state
    assert torch.allclose(s2, s[5:], atol=1e-12)


def test_delta_rule_stores_a_value_under_a_key_and_overwrites_it():
    """beta = 1, no decay, unit keys: after writing (k, v) the read-out with q = k gives v; writing (k, v2) replaces it,
    and an orthogonal key is left alone."""
    k1, k2 = torch.tensor([1.0, 0, 0], dtype=F64), torch.tensor([0, 1.0, 0], dtype=F64)
    v = torch.tensor([[2.0, -1.0], [0.5, 4.0], [7.0, 7.0]], dtype=F64)
    keys = torch.stack([k1, k2, k1])[:, None]
    out, s = plain.delta_scan(keys, keys, v[:, None], torch.ones(3, 1, dtype=F64), torch.ones(3, 1, dtype=F64))
    assert torch.allclose(out[:, 0], v)
    assert torch.allclose(s[0].T @ k2, v[1]) and torch.allclose(s[0].T @ k1, v[2])
    out2, _ = plain.delta_scan(keys, keys, v[:, None], torch.ones(3, 1, dtype=F64), torch.full((3, 1), 0.5, dtype=F64))
    assert torch.allclose(out2[2, 0], v[2])                                  # beta = 1 overwrites whatever decayed


def test_mixing_with_the_identity_is_ordinary_attention_and_windows_hide_keys():
    g = torch.Generator().manual_seed(3)
    q, k = torch.randn(12, 4, 6, generator=g, dtype=F64), torch.randn(12, 2, 6, generator=g, dtype=F64)
    w = plain.softmax_weights(q, k, 0.5, 4, 2)
    assert torch.allclose(w.sum(-1), torch.ones(4, 12, dtype=F64))
    assert torch.equal(plain.mix_heads(w, torch.eye(4)), w)
    for i in range(12):
        for j in range(12):
            assert (w[0, i, j] > 0) == plain.sees(i, j, 4, 2)
    assert plain.sees(11, 1, 4, 2) and not plain.sees(11, 2, 4, 2) and plain.sees(11, 8, 4, 2) and not plain.sees(11, 7, 4, 2)
    mix = torch.tensor([[0.5, 0.5, 0, 0], [0, 1, 0, 0], [0, 0, 2.0, -1.0], [0, 0, 0, 1]], dtype=F64)
    mixed = plain.mix_heads(w, mix)
    assert torch.allclose(mixed[0], 0.5 * (w[0] + w[1])) and torch.allclose(mixed[2], 2 * w[2] - w[3])


@pytest.mark.parametrize("tag", ["early", "odd"])
def test_the_plain_model_is_causal_and_a_pass_sees_the_tokens_through_the_input_mix_only(tag):
    cfg = models.SHAPES[tag]
    w = models.make_tensors(cfg, 4)
    a = models.random_prompts(cfg, [30], seed=1)[0]
    b = list(a)
    b[20] = (a[20] + 1) % cfg["vocab"]
    la, lb = plain.forward(cfg, w, a), plain.forward(cfg, w, b)
    assert torch.equal(la[:20], lb[:20]) and (la[20:] - lb[20:]).abs().max() > 1e-6
    # with a zero input mix nothing of the tokens gets past the start of a pass
    w2 = dict(w)
    w2["loop.in"] = torch.zeros_like(w["loop.in"])
    assert torch.equal(plain.forward(cfg, w2, a), plain.forward(cfg, w2, b))
