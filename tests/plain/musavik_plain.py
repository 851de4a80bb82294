"""A plain, slow implementation of the Musavik decoder in 64-bit, one function per mechanism.

Written from the design's equations, token by token where the design is a recurrence; it shares
no code with ``enginekernel_b200``.  ``weights`` is a dict name -> tensor (any float dtype; the
hashed table of token pairs is float too), ``config`` the parsed ``config.json``.  Everything is
computed in float64 on the CPU, for ONE sequence whose positions count from 0.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- small pieces
def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """The layers' norm: the weight is stored around zero, the factor is 1 + w."""
    return rms_unit(x, eps) * (1.0 + w.to(F64))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def causal_conv(x, taps_w, bias=None):
    """x [T, C]; taps_w [C, K] with the last column the current token's; zeros before the start."""
    t, c = x.shape
    k = taps_w.shape[1]
    out = torch.zeros_like(x)
    for j in range(k):                       # column j reaches back k - 1 - j tokens
        back = k - 1 - j
        if back < t:
            out[back:] += x[:t - back] * taps_w[:, j].to(F64)
    if bias is not None:
        out = out + bias.to(F64)
    return out


# ----------------------------------------------------------------------------- embedding
def pair_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the hashed pair table for every token: (prev * mul_prev + cur * mul_cur) mod buckets, and
    row number ``buckets`` for the first token."""
    rows = []
    for i, tok in enumerate(tokens):
        rows.append(buckets if i == 0 else (tokens[i - 1] * mul_prev + tok * mul_cur) % buckets)
    return rows


def embedding(config, w, tokens):
    e = config["embedding"]
    x = w["embed"].to(F64)[list(tokens)] * float(e["scale"])
    big = e.get("bigram")
    if big:
        rows = pair_rows(list(tokens), int(big["buckets"]), int(big["mul_prev"]), int(big["mul_cur"]))
        x = x + w["bigram"].to(F64)[rows]
    return x


# ----------------------------------------------------------------------------- gated linear recurrence
def rglru_gates(u, w, p, blocks):
    """Both gates of the recurrence from block-diagonal products: u [T, R] -> r, i [T, R]."""
    t, width = u.shape
    size = width // blocks
    ub = u.view(t, blocks, size)
    r = torch.einsum("tbi,boi->tbo", ub, w[p + "ra"].to(F64)) + w[p + "ra.b"].to(F64)
    i = torch.einsum("tbi,boi->tbo", ub, w[p + "ri"].to(F64)) + w[p + "ri.b"].to(F64)
    return torch.sigmoid(r).reshape(t, width), torch.sigmoid(i).reshape(t, width)


def rglru_scan(u, r, i, lam, state=None):
    """S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t with a_t = exp(-8 r_t softplus(lam)); S starts at zero."""
    t, width = u.shape
    s = torch.zeros(width, dtype=F64) if state is None else state.clone()
    log_a = -8.0 * r * softplus(lam.to(F64))
    a = torch.exp(log_a)
    out = torch.zeros_like(u)
    for n in range(t):
        s = a[n] * s + torch.sqrt(1.0 - a[n] ** 2) * i[n] * u[n]
        out[n] = s
    return out, s


def rglru_mixer(h, w, p, m):
    y = gelu_tanh(h @ w[p + "y"].to(F64).T + w[p + "y.b"].to(F64))
    u = causal_conv(h @ w[p + "x"].to(F64).T + w[p + "x.b"].to(F64), w[p + "conv"], w[p + "conv.b"])
    r, i = rglru_gates(u, w, p, int(m["blocks"]))
    s, _ = rglru_scan(u, r, i, w[p + "lam"])
    return (s * y) @ w[p + "o"].to(F64).T


# ----------------------------------------------------------------------------- attention with mixed heads
def rotate_pairs(x, positions, dims, base):
    """x [T, heads, d]; values 2i and 2i+1 of the first ``dims`` turn together by position * base^(-2i/dims)."""
    if not dims:
        return x
    out = x.clone()
    i = torch.arange(dims // 2, dtype=F64)
    ang = positions.to(F64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def sees(i, j, size, keep_first):
    if j > i:
        return False
    if size is None:
        return True
    return i - j < size or j < keep_first


def softmax_weights(q, k, scale, size, keep_first):
    """q [T, H, d], k [T, G, d] -> weights [H, T, T] (rows: queries), zero where a key is not seen."""
    t, nh, _ = q.shape
    g = k.shape[1]
    per = nh // g
    out = torch.zeros(nh, t, t, dtype=F64)
    for h in range(nh):
        s = (q[:, h] @ k[:, h // per].T) * scale
        for i in range(t):
            vis = [j for j in range(t) if sees(i, j, size, keep_first)]
            out[h, i, vis] = torch.softmax(s[i, vis], -1)
    return out


def mix_heads(weights, talk):
    """weight_h <- sum_g talk[h, g] weight_g."""
    return torch.einsum("hg,gij->hij", talk.to(F64), weights)


def mixed_attention(h, w, p, m, eps, positions):
    t = h.shape[0]
    nh, g, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].to(F64).T + w[p + "q.b"].to(F64)).view(t, nh, d)
    k = (h @ w[p + "k"].to(F64).T + w[p + "k.b"].to(F64)).view(t, g, d)
    v = (h @ w[p + "v"].to(F64).T + w[p + "v.b"].to(F64)).view(t, g, e)
    q = rms_unit(q, eps) * w[p + "q.norm"].to(F64)
    k = rms_unit(k, eps) * w[p + "k.norm"].to(F64)
    rot = m.get("rot") or {}
    dims, base = int(rot.get("dims", 0)), float(rot.get("base", 10000.0))
    q, k = rotate_pairs(q, positions, dims, base), rotate_pairs(k, positions, dims, base)
    v = rms_unit(v, eps)
    mask = m.get("mask") or {}
    size = mask.get("size")
    keep = int(mask.get("keep_first", 0) or 0)
    wts = softmax_weights(q, k, float(m["scale"]), size, keep)
    wts = mix_heads(wts, w[p + "talk"])
    per = nh // g
    heads = torch.stack([wts[a] @ v[:, a // per] for a in range(nh)], 1)          # [T, H, e]
    gate = torch.sigmoid(h @ w[p + "g"].to(F64).T)
    return (heads.reshape(t, nh * e) * gate) @ w[p + "o"].to(F64).T


# ----------------------------------------------------------------------------- gated delta rule
def unit_vector(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_scan(q, k, v, beta, g, state=None):
    """Per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  q, k [T, H, d]; v [T, H, e];
    beta, g [T, H].  S [H, d, e] starts at zero."""
    t, nh, d = q.shape
    e = v.shape[-1]
    s = torch.zeros(nh, d, e, dtype=F64) if state is None else state.clone()
    out = torch.zeros(t, nh, e, dtype=F64)
    for n in range(t):
        for a in range(nh):
            s[a] = g[n, a] * s[a]
            u = beta[n, a] * (v[n, a] - s[a].T @ k[n, a])
            s[a] = s[a] + torch.outer(k[n, a], u)
            out[n, a] = s[a].T @ q[n, a]
    return out, s


def delta_mixer(h, w, p, m, eps):
    t = h.shape[0]
    nh, g, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(causal_conv(h @ w[p + "q"].to(F64).T, w[p + "q.conv"])).view(t, g, d)
    k = silu(causal_conv(h @ w[p + "k"].to(F64).T, w[p + "k.conv"])).view(t, g, d)
    v = silu(causal_conv(h @ w[p + "v"].to(F64).T, w[p + "v.conv"])).view(t, nh, e)
    q = unit_vector(q) * d ** -0.5
    k = unit_vector(k)
    per = nh // g
    idx = [a // per for a in range(nh)]
    beta = torch.sigmoid(h @ w[p + "b"].to(F64).T)
    decay = torch.exp(-torch.exp(w[p + "A_log"].to(F64)) * softplus(h @ w[p + "a"].to(F64).T + w[p + "dt_bias"].to(F64)))
    o, _ = delta_scan(q[:, idx], k[:, idx], v, beta, decay)
    o = rms_unit(o, eps) * w[p + "norm"].to(F64)
    o = o.reshape(t, nh * e) * silu(h @ w[p + "g"].to(F64).T)
    return o @ w[p + "o"].to(F64).T


def side_by_side(h, w, p, m, eps, positions):
    left = mixed_attention(h, w, p + "left.", m["left"], eps, positions)
    right = delta_mixer(h, w, p + "right.", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# ----------------------------------------------------------------------------- feed-forward, layer, model
def dense_ff(h, w, p):
    up = gelu_tanh(h @ w[p + "up"].to(F64).T + w[p + "up.b"].to(F64))
    return up @ w[p + "down"].to(F64).T + w[p + "down.b"].to(F64)


def layer(x, config, w, i, positions):
    spec = config["layers"][i]
    eps = float(config["norm"]["eps"])
    p = f"l{i}."
    h = norm_one_plus(x, w[p + "norm1"], eps)
    if spec["type"] == "rglru":
        y = rglru_mixer(h, w, p + "mix.", spec["mixer"])
    elif spec["type"] == "parallel":
        y = side_by_side(h, w, p + "mix.", spec["mixer"], eps, positions)
    else:
        raise ValueError(spec["type"])
    x = x + norm_one_plus(y, w[p + "norm1b"], eps)
    if spec.get("mlp") is not None:
        h = norm_one_plus(x, w[p + "norm2"], eps)
        x = x + norm_one_plus(dense_ff(h, w, p + "mlp."), w[p + "norm2b"], eps)
    return x


def layer_runs(config):
    """(layer, starts a pass) in execution order: layers start .. stop-1 run ``times`` times in a row."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(a)]
    for _ in range(times):
        runs += [(i, i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def model_forward(config, w, tokens, return_layers=False, final_one_plus=True):
    tokens = list(tokens)
    positions = torch.arange(len(tokens))
    x0 = embedding(config, w, tokens)
    x = x0
    eps = float(config["norm"]["eps"])
    after = []
    for i, starts_pass in layer_runs(config):
        if starts_pass:
            x = torch.cat([x, x0], -1) @ w["loop.in"].to(F64).T
        x = layer(x, config, w, i, positions)
        after.append(x.clone())
    fw = w["final.norm"].to(F64)
    x = rms_unit(x, eps) * ((1.0 + fw) if final_one_plus else fw)
    logits = x @ w["head"].to(F64).T
    return (logits, after) if return_layers else logits


def forward(config, w, tokens):
    """Logits [T, vocab] of one sequence."""
    return model_forward(config, w, tokens)


def greedy(config, w, tokens, n_new):
    """``n_new`` tokens by arg-max, the whole sequence run again for each (slow and plain)."""
    seq, out = list(tokens), []
    for _ in range(n_new):
        nxt = int(model_forward(config, w, seq)[-1].argmax())
        out.append(nxt)
        seq.append(nxt)
    return out
