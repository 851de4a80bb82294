"""The Musavik decoder in the engine against the plain implementation, mechanism by mechanism and then
whole models under every way of cutting the work.

Part one drives the new kernels alone: the hashed pair table with the token carried from step to step, the
norm of a result on its way into the stream with the next norm behind it, bias and activation on a product's
rows, the convolution with a bias on its input, the gates and the scan of the gated linear recurrence from a
carried state, norms of padded heads with the value norm and the cache write, attention whose heads share
their weights (one key made to stand out at every edge), and the delta scan with one decay per head.  Part
two runs one-mixer models, and part three four small models of unlike shapes (tests/plain/musavik_models.py)
through ``Engine``: whole prompts, prompts in portions down to two tokens, token-by-token decoding, unequal
batches, slots, pages and states used again, long decoding, and greedy generation through the scheduler.
"""

import json
import math

import pytest
import torch

from tests import helpers
from tests.plain import musavik_models as models
from tests.plain import musavik_plain as plain
from tests.test_kernels_gpu import DEV, DTYPES, TOL, K, Pages, rel, rnd

pytestmark = pytest.mark.gpu
F32, F64 = torch.float32, torch.float64


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ===================================================================== mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_pair_table_with_the_token_carried_between_steps(dtype):
    """Two sequences in unlike portions: the row follows (previous, current), the first token takes the last
    row, and the token before a portion comes from the slot's state; multipliers beyond 32 bits' comfort."""
    k = K()
    buckets, mp, mc, width = 13, 100003, 99991, 24
    table = rnd(buckets + 1, width, dtype=dtype, seed=1)
    a, b = [5, 70000, 3, 3, 9, 11, 2], [8, 8, 1]
    before = torch.full((4, 1), 12345, dtype=torch.int32, device=DEV)        # stale values of earlier users
    want = {0: table.double()[plain.pair_rows(a, buckets, mp, mc)], 2: table.double()[plain.pair_rows(b, buckets, mp, mc)]}
    got = {0: [], 2: []}
    steps = [[(0, 0, 3), (2, 0, 1)], [(2, 1, 1), (0, 3, 1)], [(0, 4, 3), (2, 2, 1)]]        # (slot, first place, count)
    for step in steps:
        ids, pos, slots = [], [], []
        for slot, at, n in step:
            seq = a if slot == 0 else b
            ids += seq[at:at + n]
            pos += list(range(at, at + n))
            slots += [slot] * n
        stream = torch.ones(len(ids), width, device=DEV)
        k.embed_pair(stream, table, i32(ids), i32(pos), i32(slots), before, len(ids), buckets, mp, mc)
        k.keep_last_token(before, i32(ids), i32(pos), i32(slots), len(ids))
        r = 0
        for slot, at, n in step:
            got[slot].append(stream[r:r + n] - 1)
            r += n
    for slot in (0, 2):
        assert rel(torch.cat(got[slot]), want[slot]) <= 1e-6
    assert before[:, 0].tolist() == [a[-1], 12345, b[-1], 12345]
    # rows of finished sequences (negative positions) neither add nor store
    stream = torch.ones(2, width, device=DEV)
    k.embed_pair(stream, table, i32([1, 2]), i32([-1, -1]), i32([0, 2]), before, 2, buckets, mp, mc)
    k.keep_last_token(before, i32([1, 2]), i32([-1, -1]), i32([0, 2]), 2)
    assert torch.equal(stream, torch.ones(2, width, device=DEV)) and before[:, 0].tolist() == [a[-1], 12345, b[-1], 12345]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width", [(1, 40), (17, 100), (5, 96), (33, 2560)])
def test_norm_of_a_result_into_the_stream_and_the_next_norm(dtype, rows, width):
    k = K()
    stream = rnd(rows, width, seed=1, scale=3.0)
    a, b = rnd(rows, width, dtype=dtype, seed=2), rnd(rows, width, dtype=dtype, seed=3, scale=2.0)
    bias = rnd(width, seed=4, scale=0.3)
    g_post, g_next = 1 + 0.2 * rnd(width, seed=5), 1 + 0.2 * rnd(width, seed=6)
    unit = lambda x, eps: x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    for wa, wb, use_b, use_bias in ((1.0, 1.0, False, False), (0.8, 0.5, True, False), (1.0, 1.0, False, True),
                                    (-1.5, 0.25, True, True)):
        u = a.double() * wa + (b.double() * wb if use_b else 0) + (bias.double() if use_bias else 0)
        new = stream.double() + unit(u, 1e-5) * g_post.double()
        s, y = stream.clone(), torch.empty(rows, width, dtype=dtype, device=DEV)
        k.rmsnorm_post_add(y, s, a, g_post, 1e-5, g_next, 1e-6, weight_a=wa, b=b if use_b else None, weight_b=wb,
                           bias=bias if use_bias else None)
        assert rel(s, new) <= 1e-6
        assert rel(y, unit(new, 1e-6) * g_next.double()) <= TOL[dtype]
        s2 = stream.clone()
        k.rmsnorm_post_add(None, s2, a, g_post, 1e-5, weight_a=wa, b=b if use_b else None, weight_b=wb,
                           bias=bias if use_bias else None)
        assert torch.equal(s2, s)


@pytest.mark.parametrize("dtype", DTYPES)
def test_bias_with_activation_and_cast_into_columns(dtype):
    k = K()
    x32, bias = rnd(7, 50, seed=1, scale=2.0), rnd(30, seed=2)
    for src in (x32, x32.to(dtype)):
        for act, f in ((None, lambda z: z), ("gelu_tanh", plain.gelu_tanh), ("silu", plain.silu)):
            out = torch.empty(7, 30, dtype=dtype, device=DEV)
            k.bias_act(out, src, bias, act, col0=11)
            assert rel(out, f(src.double()[:, 11:41] + bias.double())) <= TOL[dtype]
    wide, bias4 = rnd(5, 96, seed=3, scale=2.0), rnd(64, seed=4)             # sizes the four-values-a-thread form takes
    for src in (wide, wide.to(dtype)):
        out = torch.empty(5, 64, dtype=dtype, device=DEV)
        k.bias_act(out, src, bias4, "gelu_tanh", col0=16)
        assert rel(out, plain.gelu_tanh(src.double()[:, 16:80] + bias4.double())) <= TOL[dtype]
    dst = torch.zeros(7, 64, dtype=dtype, device=DEV)
    k.cast_columns(dst, 9, x32, 7)
    assert torch.equal(dst[:, 9:59], x32.to(dtype)) and dst[:, :9].abs().sum() == 0 and dst[:, 59:].abs().sum() == 0
    dst = torch.zeros(5, 128, dtype=dtype, device=DEV)
    k.cast_columns(dst, 24, wide, 5)
    assert torch.equal(dst[:, 24:120], wide.to(dtype)) and dst[:, :24].abs().sum() == 0 and dst[:, 120:].abs().sum() == 0


@pytest.mark.parametrize("channels,taps", [(30, 4), (7, 1), (300, 2), (64, 3)])
def test_convolution_with_a_bias_on_its_input(channels, taps):
    """The projection's own bias belongs to every token that exists and to nothing before the start; a sequence
    run whole and cut 1 + 2 + 8 + rest (portions shorter than the taps) with the inputs carried in the state."""
    k = K()
    n, col0, width = 25, 3, channels + 9
    x = rnd(n, width, seed=1)
    w, b, xb = rnd(channels, taps, seed=2, scale=0.6), rnd(channels, seed=3, scale=0.2), rnd(channels, seed=4)
    want = plain.causal_conv(x[:, col0:col0 + channels].double().cpu() + xb.double().cpu(), w.double().cpu(), b.double().cpu())
    state = torch.zeros(2, 8 + channels * (taps - 1), device=DEV)
    out = torch.empty(n, channels, device=DEV)
    k.conv_act(out, x, col0, w, b, state, 8, i32(list(range(n))), i32([1] * n), n, channels, taps, in_bias=xb, activation=None)
    assert rel(out, want) <= 1e-6
    k.conv_act(out, x, col0, w, b, state, 8, i32(list(range(n))), i32([1] * n), n, channels, taps, in_bias=xb)
    assert rel(out, plain.silu(want)) <= 1e-6
    at = 0
    for size in (1, 2, 8, n):
        part = x[at:at + size].contiguous()
        m = part.shape[0]
        if m == 0:
            break
        pos, slots = i32(list(range(at, at + m))), i32([0] * m)
        o = torch.empty(m, channels, device=DEV)
        k.conv_act(o, part, col0, w, b, state, 8, pos, slots, m, channels, taps, in_bias=xb, activation=None)
        k.conv_tail(state, 8, part, col0, i32([0, m]), pos, slots, 1, channels, taps)
        assert rel(o, want[at:at + m]) <= 1e-6, (size, at)
        at += m


@pytest.mark.parametrize("parts,size", [(1, 64), (5, 16), (2, 30), (3, 200), (4, 129), (2, 300)])
def test_gates_of_the_linear_recurrence(parts, size):
    k = K()
    n, width = 237, parts * size
    u = rnd(n, width + 5, seed=1)
    wa, wi = rnd(parts, size, size, seed=2, scale=2 / math.sqrt(size)), rnd(parts, size, size, seed=3, scale=2 / math.sqrt(size))
    ba, bi, lam = rnd(parts, size, seed=4, scale=0.3), rnd(parts, size, seed=5, scale=0.3), rnd(width, seed=6, scale=1.5) - 2
    w = {"ra": wa.cpu(), "ri": wi.cpu(), "ra.b": ba.cpu(), "ri.b": bi.cpu()}
    uu = u[:, :width].double().cpu()
    r, i = plain.rglru_gates(uu, w, "", parts)
    log_a = -8.0 * r * plain.softplus(lam.double().cpu())
    wat, wit = wa.transpose(1, 2).contiguous(), wi.transpose(1, 2).contiguous()
    # a tile of tokens a block (prompts), and a warp an output channel (steps of few tokens, weights as stored)
    for rows in ({}, {"w_a_rows": wa.contiguous(), "w_i_rows": wi.contiguous()}):
        for m in (n, 37, 3, 1):
            a, x = torch.empty(m, width, device=DEV), torch.empty(m, width, device=DEV)
            k.lru_gates(a, x, u[:m], wat, ba.reshape(-1), wit, bi.reshape(-1), lam, 8.0, m, parts, size, **rows)
            assert rel(a, torch.exp(log_a)[:m]) <= 1e-5
            assert rel(x, (torch.sqrt(1 - torch.exp(2 * log_a)) * i * uu)[:m]) <= 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("channels", [5, 128, 300])
def test_scan_of_the_linear_recurrence_from_a_carried_state(dtype, channels):
    """Three unequal sequences at once, then each continued from its state in slots that others used before."""
    k = K()
    lens, slots = [9, 1, 30 if channels != 128 else 700], [2, 0, 3]        # (700: several passes of eight stretches)
    n = sum(lens)
    a = torch.rand(2 * n, channels, generator=torch.Generator().manual_seed(1)).to(DEV) * 0.6 + 0.4
    x, side = rnd(2 * n, channels, seed=2), rnd(2 * n, channels + 4, seed=3)
    sb = rnd(channels, seed=4, scale=0.3)
    state = rnd(4, channels + 6, seed=5)                                      # stale: a slot is zeroed when taken
    for s in slots:
        state[s].zero_()
    want, at = [], 0
    for ln in lens:                                                          # first and second half of each sequence
        rows = list(range(at, at + ln)) + list(range(n + at, n + at + ln))
        s = torch.zeros(channels, dtype=F64)
        o = []
        for r_ in rows:
            s = a[r_].double().cpu() * s + x[r_].double().cpu()
            o.append(s * plain.gelu_tanh(side[r_, 2:2 + channels].double().cpu() + sb.double().cpu()))
        want.append(torch.stack(o))
        at += ln
    cu = [0]
    for ln in lens:
        cu.append(cu[-1] + ln)
    tok_slots = [s for s, ln in zip(slots, lens) for _ in range(ln)]
    for half in (0, 1):
        pos = [half * ln + j for ln in lens for j in range(ln)]
        out = torch.empty(n, channels, dtype=dtype, device=DEV)
        k.lru_scan(out, a[half * n:(half + 1) * n].contiguous(), x[half * n:(half + 1) * n].contiguous(),
                   side[half * n:(half + 1) * n], 2, sb, state, i32(cu), i32(pos), i32(tok_slots), 3, channels,
                   max_new=max(lens))
        for j, ln in enumerate(lens):
            assert rel(out[cu[j]:cu[j + 1]], want[j][half * ln:(half + 1) * ln]) <= TOL[dtype], (half, j)
    assert torch.equal(state[1], rnd(4, channels + 6, seed=5)[1])             # a slot nobody holds is not touched
    # a finished sequence's row: zeros out, state as it was
    keep = state.clone()
    out = torch.ones(1, channels, dtype=dtype, device=DEV)
    k.lru_scan(out, a[:1].contiguous(), x[:1].contiguous(), side[:1], 2, sb, state, i32([0, 1]), i32([-1]), i32([2]), 1, channels)
    assert out.abs().sum() == 0 and torch.equal(state, keep)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,e,rot", [(4, 2, 24, 16, 12), (3, 3, 32, 32, 32), (6, 1, 20, 28, 0), (8, 4, 128, 64, 64)])
def test_norms_of_padded_heads_rotation_and_cache_write(dtype, nq, nkv, d, e, rot):
    """Queries and keys with bias, gained norm over the true size and the rotation of neighbouring pairs (through
    reordered rows); values with bias over their root mean square; on both sides of a page border."""
    from enginekernel_b200.parts.mixed_attention import neighbours_to_halves
    k = K()
    big, eps, base = -(-max(d, e) // 8) * 8, 1e-5, 300.0
    positions = [0, 1, 63, 64, 65, 130]
    n = len(positions)
    order = neighbours_to_halves(d, rot)
    q, kk, v = rnd(n, nq, d, seed=1), rnd(n, nkv, d, seed=2), rnd(n, nkv, e, seed=3)
    qb, kb, vb = rnd(nq, d, seed=4, scale=0.3), rnd(nkv, d, seed=5, scale=0.3), rnd(nkv, e, seed=6, scale=0.3)
    qg, kg = 1 + 0.2 * rnd(d, seed=7), 1 + 0.2 * rnd(d, seed=8)

    def padded(t, reorder):
        t = t[..., order.to(t.device)] if reorder else t
        out = torch.zeros(*t.shape[:-1], big, dtype=t.dtype, device=t.device)
        out[..., :t.shape[-1]] = t
        return out

    rows = torch.cat([padded(q, True).reshape(n, -1), padded(kk, True).reshape(n, -1), padded(v, False).reshape(n, -1),
                      rnd(n, 10, seed=9)], 1).to(dtype).contiguous()
    src = rows.double().cpu()
    pages = Pages(2, 200, nkv, big, dtype, seed=nq)
    half = rot // 2
    ang = torch.outer(torch.tensor(positions, dtype=F64), base ** (-2.0 * torch.arange(half, dtype=F64) / max(rot, 1)))
    cos, sin = torch.zeros(200, half), torch.zeros(200, half)
    cos[positions], sin[positions] = ang.cos().float(), ang.sin().float()
    k.qk_prepare_padded_kv(rows, n, padded(qg, True).contiguous(), padded(kg, True).contiguous(), cos.to(DEV).contiguous(),
                           sin.to(DEV).contiguous(), rot, i32(positions), i32([1] * n), pages.k, pages.v, pages.table, nq, nkv,
                           big, eps, d, q_bias=padded(qb, True).reshape(-1).contiguous(),
                           k_bias=padded(kb, True).reshape(-1).contiguous(), v_bias=padded(vb, False).reshape(-1).contiguous(),
                           value_unit_eps=eps, value_dim=e)
    pos_t = torch.tensor(positions)
    inv = torch.argsort(order)
    # what the plain functions give from the rounded projections, in the design's own order of values
    q_in = src[:, :nq * big].view(n, nq, big)[..., :d][..., inv]
    k_in = src[:, nq * big:(nq + nkv) * big].view(n, nkv, big)[..., :d][..., inv]
    v_in = src[:, (nq + nkv) * big:(nq + 2 * nkv) * big].view(n, nkv, big)[..., :e]
    want_q = plain.rotate_pairs(plain.rms_unit(q_in + qb.double().cpu(), eps) * qg.double().cpu(), pos_t, rot, base)
    want_k = plain.rotate_pairs(plain.rms_unit(k_in + kb.double().cpu(), eps) * kg.double().cpu(), pos_t, rot, base)
    want_v = plain.rms_unit(v_in + vb.double().cpu(), eps)
    got_q = rows[:, :nq * big].view(n, nq, big).double().cpu()
    assert rel(got_q[..., :d][..., inv], want_q) <= TOL[dtype] and got_q[..., d:].abs().sum() == 0
    keys, values = pages.dense(1, 131)
    got_k, got_v = keys[positions].double().cpu(), values[positions].double().cpu()
    assert rel(got_k[..., :d][..., inv], want_k) <= TOL[dtype] and got_k[..., d:].abs().sum() == 0
    assert rel(got_v[..., :e], want_v) <= TOL[dtype] and got_v[..., e:].abs().sum() == 0
    assert rows[:, (nq + 2 * nkv) * big:].equal(rnd(n, 10, seed=9).to(dtype))       # what lies behind the heads is left alone


def _mixed_reference(q, keys, values, pos, scale, window, keep, mix, gate):
    """q [NH, D] at ``pos``; keys, values [len, NKV, D]: mixed weights on the head's own values, float64."""
    nh, nkv = q.shape[0], keys.shape[1]
    js = [j for j in range(pos + 1) if plain.sees(pos, j, window, keep)]
    wts = torch.stack([torch.softmax((keys[js, h // (nh // nkv)].double() @ q[h].double()) * scale, 0) for h in range(nh)])
    wts = mix.double() @ wts
    out = torch.stack([wts[h] @ values[js, h // (nh // nkv)].double() for h in range(nh)])
    return out * torch.sigmoid(gate.double()) if gate is not None else out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,keep,length", [(9, 3, 40), (70, 5, 300), (64, 64, 200), (3, 1, 700), (None, 0, 150)])
def test_heads_that_share_their_weights_behind_a_window_with_kept_first_tokens(dtype, window, keep, length):
    """Single queries at the end and every query of a prompt; the keys cut into splits; then one key made to fit
    the last query far better than any other, put just inside and just outside the window and the kept first
    tokens and on both sides of page borders: every head's result is its mixed share of that key's values
    exactly when the plain rule sees the key."""
    k = K()
    nq, nkv, d, e, scale = 4, 2, 40, 24, 0.3
    pages = Pages(1, length, nkv, d, dtype, seed=length)
    keys, values = rnd(length, nkv, d, dtype=dtype, seed=1), rnd(length, nkv, d, dtype=dtype, seed=2)
    pages.fill(0, keys, values)
    q = rnd(length, nq * d + nq * e, dtype=dtype, seed=3)                   # the gate sits behind the heads in the row
    gate = q[:, nq * d:]
    mix = (torch.eye(nq) + 0.4 * torch.randn(nq, nq, generator=torch.Generator().manual_seed(4))).to(DEV)
    parts = torch.empty(length, nq, nkv, d, device=DEV)
    out = torch.empty(length, nq * e, dtype=dtype, device=DEV)

    def run(rows, pos, n, g, **kw):
        k.attention_generic_cross(parts, rows, n, pos, i32([0] * n), pages.k, pages.v, pages.table, nq, nkv, d, scale,
                                  window, keep_first=keep, **kw)
        k.mix_heads(out, parts, mix, pos, n, nq, nkv, d, e, gate=g)

    run(q, i32(list(range(length))), length, gate)
    kc, vc, qc, mc = keys.cpu(), values.cpu(), q.cpu(), mix.cpu()
    w0 = window or 10 ** 9
    for pos in sorted({0, 1, keep, keep + 1, w0 - 1, w0, w0 + keep, 63, 64, 65, length - 1} & set(range(length))):
        want = _mixed_reference(qc[pos, :nq * d].view(nq, d), kc, vc[..., :e], pos, scale, window, keep, mc,
                                qc[pos, nq * d:].view(nq, e))
        assert rel(out[pos].view(nq, e), want) <= TOL[dtype], pos
    last = length - 1
    acc, ml = torch.empty(1, nq * nkv, 4, d, device=DEV), torch.empty(1, nq * nkv, 4, 2, device=DEV)
    run(q[last:], i32([last]), 1, gate[last:], n_splits=4, keys_per_split=-(-length // 4), part_acc=acc, part_ml=ml)
    want = _mixed_reference(qc[last, :nq * d].view(nq, d), kc, vc[..., :e], last, scale, window, keep, mc, qc[last, nq * d:].view(nq, e))
    assert rel(out[0].view(nq, e), want) <= TOL[dtype]
    sharp_q = torch.zeros(1, nq * d, dtype=dtype, device=DEV)
    sharp_q.view(nq, d)[:, 0] = 30.0
    for j in sorted({0, keep - 1, keep, last - w0, last - w0 + 1, 63, 64, last} & set(range(length))):
        k2 = (keys.float() * 0.1).to(dtype)
        k2[j, :, 0] = 30.0
        pages.fill(0, k2, values)
        run(sharp_q, i32([last]), 1, None)
        seen = plain.sees(last, j, window, keep)
        # every head's weights sit on key j alone: head h gets (sum_g mix[h, g]) times its own value head's row
        want = mc.sum(1, keepdim=True).double() * vc[j, :, :e].double().repeat_interleave(nq // nkv, 0)
        hit = rel(out[0].view(nq, e), want) <= 2e-2
        assert hit == seen, (j, seen)


@pytest.mark.parametrize("d,nq,nkv", [(64, 4, 2), (96, 6, 1), (128, 8, 4)])
@pytest.mark.parametrize("window,keep,length", [(9, 3, 40), (70, 5, 300), (64, 64, 200), (3, 1, 700), (130, 70, 400)])
def test_the_16_bit_prompt_and_decode_kernels_apply_every_heads_weights_to_every_value_head(d, nq, nkv, window, keep, length):
    """Both 16-bit kernels against the general one, which the test above holds against the plain rule: a prompt
    whole and cut behind a cached prefix, single tokens with the keys whole and split."""
    k = K()
    dtype, scale = torch.bfloat16, 0.3
    pages = Pages(2, length, nkv, d, dtype, seed=length)
    keys, values = rnd(length, nkv, d, dtype=dtype, seed=1), rnd(length, nkv, d, dtype=dtype, seed=2)
    pages.fill(1, keys, values)
    q = rnd(length, nq * d + 8, dtype=dtype, seed=3)
    pos, slots = i32(list(range(length))), i32([1] * length)
    want = torch.empty(length, nq, nkv, d, device=DEV)
    k.attention_generic_cross(want, q, length, pos, slots, pages.k, pages.v, pages.table, nq, nkv, d, scale, window,
                              keep_first=keep)
    got = torch.full((length, nq, nkv, d), 7.0, device=DEV)
    k.attention_prefill_cross_bf16(got, q, length, pos, slots, i32([0, length]), 1, pages.k, pages.v, pages.table, nq, nkv,
                                   d, scale, window, keep_first=keep)
    assert rel(got, want) <= 2e-2
    cut = length // 3 + 1                                                   # the rest of the prompt behind a cached part
    got2 = torch.full((length - cut, nq, nkv, d), 7.0, device=DEV)
    k.attention_prefill_cross_bf16(got2, q[cut:], length - cut, pos[cut:].contiguous(), slots[cut:].contiguous(),
                                   i32([0, length - cut]), 1, pages.k, pages.v, pages.table, nq, nkv, d, scale, window,
                                   keep_first=keep)
    assert rel(got2, want[cut:]) <= 2e-2
    picks = sorted({0, 1, keep, window - 1, window, window + keep, 63, 64, length - 1} & set(range(length)))
    rows = q[picks].contiguous()
    for splits in (1, 3):
        acc = torch.empty(len(picks), nq * nkv, splits, d, device=DEV) if splits > 1 else None
        ml = torch.empty(len(picks), nq * nkv, splits, 2, device=DEV) if splits > 1 else None
        got3 = torch.full((len(picks), nq, nkv, d), 7.0, device=DEV)
        k.attention_decode_cross_bf16(got3, rows, len(picks), i32(picks), i32([1] * len(picks)), pages.k, pages.v, pages.table,
                                      nq, nkv, d, scale, window, splits, 0, acc, ml, keep_first=keep)
        assert rel(got3, want[picks]) <= 2e-2, splits
    dead = torch.full((2, nq, nkv, d), 7.0, device=DEV)                     # rows of finished sequences give zeros
    k.attention_decode_cross_bf16(dead, rows[:2], 2, i32([-1, -1]), i32([1, 1]), pages.k, pages.v, pages.table, nq, nkv, d,
                                  scale, window, keep_first=keep)
    assert dead.abs().sum() == 0


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 16, 24), (2, 2, 64, 32), (6, 1, 12, 20), (3, 3, 128, 64)])
def test_delta_scan_with_one_decay_per_head_and_the_gated_norm(heads, kv_heads, dim, vdim):
    """Unequal sequences at once, then continued from their states; the read-out through the norm per head
    with a weight and the SiLU of a raw gate."""
    k = K()
    lens, slots = [7, 1, 20], [1, 3, 0]
    n = sum(lens)
    rows_s = k.delta_state_rows(dim)
    q = torch.nn.functional.normalize(rnd(2 * n, kv_heads, dim, seed=1), dim=-1) * dim ** -0.5
    kk = torch.nn.functional.normalize(rnd(2 * n, kv_heads, dim, seed=2), dim=-1)
    v, beta = rnd(2 * n, heads, vdim, seed=3), torch.sigmoid(rnd(2 * n, heads, seed=4))
    g = torch.rand(2 * n, heads, generator=torch.Generator().manual_seed(5)).to(DEV) * 0.5 + 0.5
    state = torch.zeros(4, heads * vdim * rows_s + 8, device=DEV)
    per = heads // kv_heads
    idx = [h // per for h in range(heads)]
    cu = [0]
    for ln in lens:
        cu.append(cu[-1] + ln)
    tok_slots = [s for s, ln in zip(slots, lens) for _ in range(ln)]
    want, at = [], 0
    for ln in lens:
        r_ = list(range(at, at + ln)) + list(range(n + at, n + at + ln))
        o, _ = plain.delta_scan(q[r_].double().cpu()[:, idx], kk[r_].double().cpu()[:, idx], v[r_].double().cpu(),
                                beta[r_].double().cpu(), g[r_].double().cpu())
        want.append(o)
        at += ln
    gate = rnd(n, heads * vdim + 3, seed=6)
    wn = 1 + 0.2 * rnd(vdim, seed=7)
    for half in (0, 1):
        pos = [half * ln + j for ln in lens for j in range(ln)]
        sl = slice(half * n, (half + 1) * n)
        out = torch.empty(n, heads * vdim, device=DEV)
        k.delta_scan(out, q[sl].reshape(n, -1).contiguous(), kk[sl].reshape(n, -1).contiguous(), v[sl].reshape(n, -1).contiguous(),
                     beta[sl].contiguous(), g[sl].contiguous(), state, i32(cu), i32(pos), i32(tok_slots), 3, heads, kv_heads,
                     dim, vdim, n_tokens=n, decay_per_head=True)
        for j, ln in enumerate(lens):
            assert rel(out[cu[j]:cu[j + 1]].view(ln, heads, vdim), want[j][half * ln:(half + 1) * ln]) <= 2e-5, (half, j)
        for dtype in DTYPES:
            y = torch.empty(n, heads * vdim, dtype=dtype, device=DEV)
            k.delta_out_norm(y, out, gate[:, 3:], wn, 1e-5, i32(pos), n, (heads, kv_heads, dim, vdim, 2, heads, heads * vdim),
                             gate_activation="silu")
            o = out.double().cpu().view(n, heads, vdim)
            ref = plain.rms_unit(o, 1e-5) * wn.double().cpu() * plain.silu(gate[:, 3:].double().cpu().view(n, heads, vdim))
            assert rel(y.view(n, heads, vdim), ref) <= TOL[dtype]


# ===================================================================== one-mixer models
def _one_layer(mixer_entry, width, vocab, **kw):
    return models.config(width, vocab, [(mixer_entry, None)], embedding_scale=1.3, **kw)


_QUIET_RIGHT = models.right(2, 1, 16, 16, 2)
ONE_LAYER = {
    # sharp attentions: scores spread over tens, so one key can hold nearly all the weight
    "window": _one_layer(models.parallel(models.left(4, 2, 24, 40, 16, 50, keep_first=4, scale=20.0 / 24), _QUIET_RIGHT, 1.0, 0.1), 96, 600),
    "window_wide": _one_layer(models.parallel(models.left(8, 4, 128, 64, 64, 100, keep_first=70, base=1e6, scale=0.4), _QUIET_RIGHT, 1.0, 0.1), 128, 600),
    "window_small_values": _one_layer(models.parallel(models.left(6, 1, 40, 12, 10, 64, keep_first=1, scale=0.5), _QUIET_RIGHT, 1.0, 0.1), 100, 600),
    "delta": _one_layer(models.parallel(models.left(2, 1, 16, 16, 0, 8), models.right(4, 2, 24, 16, 3), 0.1, 1.0), 96, 83),
    "delta_wide": _one_layer(models.parallel(models.left(2, 1, 16, 16, 0, 8), models.right(4, 4, 128, 64, 4), 0.1, 1.0), 128, 83),
    "recurrence": _one_layer(models.rglru(80, 5, 3), 96, 83, pairs=(31, 5, 3)),
    "recurrence_wide": _one_layer(models.rglru(256, 1, 4), 128, 83, loop=(0, 1, 2)),
}


@pytest.fixture(scope="module")
def one_layer_engines(tmp_path_factory):
    from enginekernel_b200 import Engine
    made = {}

    def get(tag, dtype):
        if (tag, dtype) not in made:
            cfg = ONE_LAYER[tag]
            w = models.make_tensors(cfg, 5)
            folder = models.write_folder(str(tmp_path_factory.mktemp("one_" + tag)), cfg, w)
            made[(tag, dtype)] = (Engine(folder, dtype, max_tokens=2048, max_batch=4), cfg, w)
        return made[(tag, dtype)]
    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", list(ONE_LAYER))
def test_one_mixer_whole_then_token_by_token(one_layer_engines, tag, dtype):
    eng, cfg, w = one_layer_engines(tag, dtype)
    ids = models.random_prompts(cfg, [330], seed=2)[0]
    want = plain.forward(cfg, w, ids)
    assert helpers.rel_err(helpers.whole(eng, ids), want) <= helpers.TOL[dtype]
    got = helpers.tail_one_by_one(eng, ids, 140)              # across three page borders, the window passing over decoded tokens
    assert helpers.rel_err(got, want) <= helpers.TOL[dtype]


def _best_key_token(cfg, w, last_token, last_pos, key_pos):
    """The vocabulary token whose key at ``key_pos`` scores highest against the query of ``last_token`` at
    ``last_pos`` in some head of layer 0's attention (from the plain pieces); no pair table in these models."""
    m, eps, p = cfg["layers"][0]["mixer"]["left"], cfg["norm"]["eps"], "l0.mix.left."
    x = w["embed"].double() * cfg["embedding"]["scale"]
    h = plain.norm_one_plus(x, w["l0.norm1"], eps)
    v = cfg["vocab"]
    rot = m.get("rot") or {}
    dims, base = int(rot.get("dims", 0)), float(rot.get("base", 1e4))
    keys = (h @ w[p + "k"].double().T + w[p + "k.b"].double()).view(v, m["kv_heads"], m["dim"])
    keys = plain.rotate_pairs(plain.rms_unit(keys, eps) * w[p + "k.norm"].double(), torch.full((v,), key_pos), dims, base)
    q = (h[last_token:last_token + 1] @ w[p + "q"].double().T + w[p + "q.b"].double()).view(1, m["heads"], m["dim"])
    q = plain.rotate_pairs(plain.rms_unit(q, eps) * w[p + "q.norm"].double(), torch.tensor([last_pos]), dims, base)[0]
    per = m["heads"] // m["kv_heads"]
    s = torch.einsum("hd,vhd->vh", q, keys.repeat_interleave(per, 1)) * m["scale"]
    s[:v // 2] = -1e9                                       # the prompts are drawn from the lower half
    return int(s.amax(-1).argmax())


@pytest.mark.parametrize("tag", ["window", "window_wide", "window_small_values"])
def test_one_key_at_every_edge_decides_or_is_not_seen(one_layer_engines, tag):
    """The token whose key fits the last query best is put at the first places, just inside and just outside
    the kept first tokens and the window, and on both sides of page borders, among 320 others: the last
    logits follow it where the plain rule sees it, in a prompt and when the last tokens are decoded alone.
    (Where the attention does not see it, the delta rule beside it still carries a trace of it.)"""
    eng, cfg, w = one_layer_engines(tag, "float32")
    mask = cfg["layers"][0]["mixer"]["left"]["mask"]
    window, keep, n = mask["size"], mask["keep_first"], 320
    a = [t % (cfg["vocab"] // 2) for t in models.random_prompts(cfg, [n], seed=3)[0]]
    wa = plain.forward(cfg, w, a)[-1]
    runs = (helpers.whole, lambda e, ids: helpers.tail_one_by_one(e, ids, 3))
    ga = [run(eng, a)[-1] for run in runs]
    moved = {}
    for key_pos in sorted({0, 1, keep - 1, keep, 63, 64, 255, 256, n - window - 1, n - window, n - 2}):
        b = list(a)
        b[key_pos] = _best_key_token(cfg, w, a[-1], n - 1, key_pos)         # a token that is nowhere else
        wb = plain.forward(cfg, w, b)[-1]
        seen = plain.sees(n - 1, key_pos, window, keep)
        moved[key_pos] = (float((wa - wb).abs().max() / wa.abs().max()), seen)
        for run, base in zip(runs, ga):
            gb = run(eng, b)[-1]
            assert helpers.rel_err(gb, wb) <= helpers.TOL["float32"], key_pos
            assert (base - gb - (wa - wb).float()).abs().max().item() <= 1e-3 * float((wa - wb).abs().max()) + 2e-5 * float(wa.abs().max()), key_pos
    # the test's weights do what they are made for: a seen key moves the logits far more than an unseen one
    assert min(m for m, seen in moved.values() if seen) > 5 * max(m for m, seen in moved.values() if not seen), moved


@pytest.mark.parametrize("tag", ["delta", "delta_wide", "recurrence", "recurrence_wide"])
@pytest.mark.parametrize("changed", [0, 63, 64, 300, 318])
def test_one_changed_token_moves_the_last_logits(one_layer_engines, tag, changed):
    """The same prompt with one token changed: what the state carries of it moves the logits at the end in
    the engine as in the plain model, in a prompt and when the last tokens are decoded alone."""
    eng, cfg, w = one_layer_engines(tag, "float32")
    a = models.random_prompts(cfg, [320], seed=3)[0]
    b = list(a)
    b[changed] = (a[changed] + 1) % cfg["vocab"]
    wa, wb = plain.forward(cfg, w, a)[-1], plain.forward(cfg, w, b)[-1]
    if changed >= 300:
        assert (wa - wb).abs().max() > 1e-4 * wa.abs().max()
    for run in (helpers.whole, lambda e, ids: helpers.tail_one_by_one(e, ids, 3)):
        ga, gb = run(eng, a)[-1], run(eng, b)[-1]
        assert (ga - gb - (wa - wb).float()).abs().max().item() <= 2e-2 * float((wa - wb).abs().max()) + 2e-5 * float(wa.abs().max())


# ===================================================================== whole models
TAGS = list(models.SHAPES)
SEEDS = {"early": 11, "flat": 12, "odd": 13, "wide": 14}


@pytest.fixture(scope="module")
def weights():
    return {tag: models.make_tensors(cfg, SEEDS[tag]) for tag, cfg in models.SHAPES.items()}


@pytest.fixture(scope="module")
def engines(tmp_path_factory, weights):
    from enginekernel_b200 import Engine
    made = {}

    def get(tag, dtype):
        if (tag, dtype) not in made:
            folder = models.write_folder(str(tmp_path_factory.mktemp("musavik_" + tag)), models.SHAPES[tag], weights[tag])
            made[(tag, dtype)] = Engine(folder, dtype, max_tokens=4096, max_batch=8)
        return made[(tag, dtype)]
    return get


def close(got, want, dtype, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs().amax(-1) / want.abs().max()
    limit = helpers.TOL[dtype] * (3 if dtype == "bfloat16" else 1)
    assert err.max().item() <= limit, f"{what} {dtype}: worst row {err.max():.3e} (limit {limit})"
    if dtype == "bfloat16" and err.numel() >= 3:
        assert err.median().item() <= helpers.TOL[dtype], f"{what}: median {err.median():.3e}"


_WANT = {}


def want_logits(weights, tag, ids):
    key = (tag, tuple(ids))
    if key not in _WANT:
        _WANT[key] = plain.forward(models.SHAPES[tag], weights[tag], ids)
    return _WANT[key]


def in_portions(engine, tokens, sizes):
    slot = engine.open_sequence()
    try:
        rows, at = [], 0
        for n in list(sizes) + [len(tokens)]:
            part = tokens[at:at + n]
            if not part:
                break
            rows.append(engine.step([(slot, part, list(range(len(part))))]).cpu())
            at += len(part)
        return torch.cat(rows, 0)
    finally:
        engine.close_sequence(slot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", TAGS)
def test_whole_prompts(engines, weights, tag, dtype):
    eng = engines(tag, dtype)
    for j, n in enumerate((1, 2, 7, 33, 64, 65, 130, 260)):
        ids = models.random_prompts(models.SHAPES[tag], [n], seed=40 + j)[0]
        close(helpers.whole(eng, ids), want_logits(weights, tag, ids), dtype, f"{tag} length {n}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", TAGS)
def test_prompt_then_token_by_token(engines, weights, tag, dtype):
    eng = engines(tag, dtype)
    ids = models.random_prompts(models.SHAPES[tag], [150], seed=77)[0]
    got = helpers.tail_one_by_one(eng, ids, 80)               # every window of the shapes passes over decoded tokens
    close(got, want_logits(weights, tag, ids), dtype, tag)
    if dtype == "float32":
        assert helpers.rel_err(got, helpers.whole(eng, ids)) <= 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", TAGS)
def test_prompts_in_portions(engines, weights, tag, dtype):
    eng = engines(tag, dtype)
    ids = models.random_prompts(models.SHAPES[tag], [210], seed=78)[0]
    want = want_logits(weights, tag, ids)
    for sizes in ((2, 2, 2, 3, 17), (64, 64, 2), (63, 2, 65), (1, 127, 2), (129,)):
        close(in_portions(eng, ids, sizes), want, dtype, f"{tag} portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", TAGS)
def test_unequal_batches_and_reuse(engines, weights, tag, dtype):
    """Requests of unequal lengths start together and end at different steps; three such batches in a row
    through the same few slots, pages and states, then everything is free again."""
    eng = engines(tag, dtype)
    shapes = [((5, 9, 13), (3, 9, 1)), ((1, 70, 31, 16), (1, 64, 20, 16)), ((66, 2, 140), (65, 1, 100))]
    for j, (lens, heads) in enumerate(shapes):
        seqs = models.random_prompts(models.SHAPES[tag], lens, seed=200 + j)
        got = helpers.batch_then_steps(eng, seqs, heads)
        for ids, g in zip(seqs, got):
            close(g, want_logits(weights, tag, ids), dtype, f"{tag} batch {j} length {len(ids)}")
            if dtype == "float32":                       # what else is in the batch does not matter beyond rounding
                assert helpers.rel_err(g, helpers.whole(eng, ids)) <= 1e-5
    assert eng.cache.book.open_slots() == []
    assert eng.cache.free_tokens() == eng.cache.num_pages * 64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["odd", "early"])
def test_first_tokens_one_by_one(engines, weights, tag, dtype):
    eng = engines(tag, dtype)
    ids = models.random_prompts(models.SHAPES[tag], [7], seed=5)[0]
    close(helpers.tail_one_by_one(eng, ids, tail=6), want_logits(weights, tag, ids), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["early", "flat"])
def test_long_decoding(engines, weights, tag, dtype):
    eng = engines(tag, dtype)
    ids = models.random_prompts(models.SHAPES[tag], [300], seed=9)[0]
    close(helpers.tail_one_by_one(eng, ids, tail=290), want_logits(weights, tag, ids), dtype, tag)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["early", "wide"])
def test_greedy_generation_through_the_scheduler(tmp_path, tag, dtype):
    """``Engine.generate_all``: five requests of unequal lengths through two slots, so the scheduler forms
    several batches and the captured decode step runs on slots, states and carried tokens used before."""
    from enginekernel_b200 import Engine
    cfg = models.SHAPES[tag]
    w = models.make_tensors(cfg, 21)
    folder = models.write_folder(str(tmp_path / "m"), cfg, w)
    eng = Engine(folder, dtype, max_tokens=2048, max_batch=2)
    prompts = models.random_prompts(cfg, [3, 70, 17, 64, 1], seed=8)
    got = eng.generate_all(prompts, 12)
    distinct = set()
    for ids, out in zip(prompts, got):
        assert len(out) == 12
        want = plain.greedy(cfg, w, ids, 12)
        distinct.update(want)
        if dtype == "float32":
            assert out == want
        else:
            assert out[:1] == want[:1]
    assert len(distinct) > 3
    assert eng.cache.book.open_slots() == []
    if dtype == "float32":                                   # without the captured graph: the same tokens
        eager = Engine(folder, dtype, max_tokens=2048, max_batch=2, use_graph=False)
        assert eager.generate_all(prompts, 12) == got


def test_unused_tensors_and_missing_ones(tmp_path):
    """A layer without feed-forward may still carry its second pair of norms; a file that lacks a tensor is
    refused by name."""
    from enginekernel_b200 import Engine
    from enginekernel_b200.weights.checkpoint import WeightsError
    cfg = models.SHAPES["early"]
    w = models.make_tensors(cfg, 2)
    w["l1.norm2"] = torch.zeros(cfg["width"], dtype=torch.bfloat16)
    eng = Engine(models.write_folder(str(tmp_path / "a"), cfg, w), "float32", max_tokens=256, max_batch=2)
    ids = models.random_prompts(cfg, [20], seed=1)[0]
    assert helpers.rel_err(helpers.whole(eng, ids), plain.forward(cfg, w, ids)) <= helpers.TOL["float32"]
    for name in ("loop.in", "bigram", "l0.mix.left.talk", "l2.mix.ra.b"):
        less = dict(w)
        del less[name]
        with pytest.raises(WeightsError, match=name):
            Engine(models.write_folder(str(tmp_path / ("b" + name)), cfg, less), "float32", max_tokens=256, max_batch=2)


def test_command_line_and_trace_replay(tmp_path):
    """``random-model`` writes a Musavik folder from a configuration file, ``generate`` prints the plain model's
    greedy tokens for it, and ``bin/trace_run`` replays steps over the same folder."""
    import os
    import subprocess
    import sys

    import numpy as np
    from safetensors import safe_open
    from tests.test_cli_gpu import ROOT, run_cli
    cfg = models.SHAPES["flat"]
    config_file = tmp_path / "config.json"
    config_file.write_text(json.dumps(cfg))
    folder = tmp_path / "model"
    run_cli("random-model", "--config", str(config_file), "--seed", "5", "--out", str(folder))
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as f:
        w = {name: f.get_tensor(name) for name in f.keys()}
    assert {n: tuple(t.shape) for n, t in w.items()} == models.tensor_shapes(cfg)
    prompts = models.random_prompts(cfg, (3, 40), seed=4)
    ids = ";".join(",".join(str(t) for t in p) for p in prompts)
    out = run_cli("generate", "--model", str(folder), "--dtype", "float32", "--prompt-ids", ids, "--out-len", "5")
    rows = [json.loads(line) for line in out.strip().splitlines()]
    assert [r["tokens"] for r in rows] == [plain.greedy(cfg, w, p, 5) for p in prompts]

    steps = [{"step": 0, "entries": [{"id": "a", "tokens": prompts[1][:30], "want": [0, 29]},
                                     {"id": "b", "tokens": prompts[0][:1], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": prompts[1][30:31], "want": [0]},
                                     {"id": "b", "tokens": prompts[0][1:2], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": prompts[1][31:32], "want": [0]}], "end": ["a"]}]
    out_dir = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(folder), "--dtype",
                        "float32", "--out", str(out_dir), "--max-tokens", "128"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                       timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    a, b = plain.forward(cfg, w, prompts[1][:32]), plain.forward(cfg, w, prompts[0][:2])
    want = {0: torch.stack([a[0], a[29]]), 1: torch.stack([a[30], b[1]]), 2: a[31:32]}
    for n, rows_wanted in want.items():
        got = torch.from_numpy(np.fromfile(str(out_dir / f"{n}.f32"), dtype="<f4").reshape(rows_wanted.shape))
        assert helpers.rel_err(got, rows_wanted) <= helpers.TOL["float32"], n
