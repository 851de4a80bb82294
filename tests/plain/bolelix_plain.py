"""A plain, slow implementation of the Bolelix decoder in 64-bit, one function per mechanism.

Written from the design's equations, token by token where the design is a recurrence; it shares
no code with ``enginekernel_b200``.  ``weights`` is a dict name -> tensor (any float dtype),
``config`` the parsed ``config.json``.  Everything is computed in float64 on the CPU.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- small pieces
def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def log_sigmoid(z):
    return -softplus(-z)


# ----------------------------------------------------------------------------- rotation
def rotation_frequencies(dims, base, factor=1.0):
    i = torch.arange(dims // 2, dtype=F64)
    return base ** (-2.0 * i / dims) / factor


def rotate(x, positions, dims, base, factor=1.0):
    """x [T, heads, d]; the first ``dims`` values of each head turn, i with i + dims/2."""
    if dims == 0:
        return x
    half = dims // 2
    ang = positions.to(F64)[:, None] * rotation_frequencies(dims, base, factor)[None, :]     # [T, half]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


# ----------------------------------------------------------------------------- attention
def visible(i, j, size, keep_first):
    """Whether the query at position i sees the key at position j: a window of ``size`` (None:
    everything before) and the first ``keep_first`` positions."""
    if j > i:
        return False
    if size is None:
        return True
    return i - j < size or j < keep_first


def attention_keys_values(h, w, p, m, eps, positions):
    """Keys as a cache holds them (rotated, then unit rms per head) and values: [T, G, d], [T, G, e]."""
    t = h.shape[0]
    g, d, e = m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {}
    dims, base = int(rot.get("dims", 0)), float(rot.get("base", 10000.0))
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    k = (h @ w[p + "k"].to(F64).T).view(t, g, d)
    v = (h @ w[p + "v"].to(F64).T).view(t, g, e)
    k = rms_unit(rotate(k, positions, dims, base, factor), eps)
    return k, v


def attention(h, w, p, m, eps, positions, keys, values):
    """h [T, width] at ``positions``; ``keys`` / ``values`` [T, G, .] of the same tokens (this
    layer's own or another layer's)."""
    t = h.shape[0]
    nh, g, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {}
    dims, base = int(rot.get("dims", 0)), float(rot.get("base", 10000.0))
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    mask = m.get("mask") or {}
    size, keep = mask.get("size"), int(mask.get("keep_first", 0))
    q = (h @ w[p + "q"].to(F64).T).view(t, nh, d)
    q = rms_unit(rotate(q, positions, dims, base, factor), eps)
    gate = torch.sigmoid(h @ w[p + "g"].to(F64).T)                     # [T, heads]
    out = torch.zeros(t, nh, e, dtype=F64)
    pos = positions.tolist()
    for a in range(nh):
        kv = a // (nh // g)
        for i in range(t):
            js = [j for j in range(t) if visible(pos[i], pos[j], size, keep)]
            s = (keys[js, kv] @ q[i, a]) * m["scale"]
            pw = torch.softmax(s, 0)
            out[i, a] = pw @ values[js, kv]
    out = out * gate[:, :, None]
    return out.reshape(t, nh * e) @ w[p + "o"].to(F64).T


# ----------------------------------------------------------------------------- mamba2
def causal_conv(x, weight, bias, before=None):
    """x [T, C]; weight [C, K] whose last column multiplies the current token; zeros (or
    ``before`` [K-1, C]) ahead of the first token."""
    t, c = x.shape
    k = weight.shape[1]
    pad = torch.zeros(k - 1, c, dtype=F64) if before is None else before
    xx = torch.cat([pad, x], 0)
    out = torch.zeros(t, c, dtype=F64)
    for j in range(k):
        out += xx[j:j + t] * weight[:, j][None, :]
    return out + bias[None, :]


def mamba2(h, w, p, m, eps):
    """State-space duality mixer over one whole sequence, state zero at the start."""
    t = h.shape[0]
    nh, e, n, g = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = nh * e
    proj = h @ w[p + "in"].to(F64).T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * g * n], proj[:, 2 * inner + 2 * g * n:]
    xbc = silu(causal_conv(xbc, w[p + "conv"].to(F64), w[p + "conv.b"].to(F64)))
    x = xbc[:, :inner].view(t, nh, e)
    b = xbc[:, inner:inner + g * n].view(t, g, n)
    c = xbc[:, inner + g * n:].view(t, g, n)
    dt = softplus(dt + w[p + "dt_bias"].to(F64)[None, :])              # [T, heads]
    a = torch.exp(w[p + "A_log"].to(F64))
    dskip = w[p + "D"].to(F64)
    y = torch.zeros(t, nh, e, dtype=F64)
    for head in range(nh):
        grp = head // (nh // g)
        s = torch.zeros(n, e, dtype=F64)
        for i in range(t):
            s = math.exp(-a[head].item() * dt[i, head].item()) * s \
                + dt[i, head] * torch.outer(b[i, grp], x[i, head])
            y[i, head] = s.T @ c[i, grp] + dskip[head] * x[i, head]
    y = y.reshape(t, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.view(t, parts, inner // parts), eps).reshape(t, inner) * w[p + "norm"].to(F64)
    return y @ w[p + "o"].to(F64).T


# ----------------------------------------------------------------------------- mlstm
def mlstm(h, w, p, m, eps):
    """Matrix memory with exponential gates kept stable by a running maximum that starts at 0."""
    t = h.shape[0]
    nh, d, e, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w[p + "q"].to(F64).T).view(t, nh, d) * d ** -0.5
    k = (h @ w[p + "k"].to(F64).T).view(t, nh, d)
    v = (h @ w[p + "v"].to(F64).T).view(t, nh, e)
    ig = cap * torch.tanh((h @ w[p + "i"].to(F64).T + w[p + "i.b"].to(F64)) / cap)
    fg = log_sigmoid(cap * torch.tanh((h @ w[p + "f"].to(F64).T + w[p + "f.b"].to(F64)) / cap))
    o = torch.zeros(t, nh, e, dtype=F64)
    for head in range(nh):
        s = torch.zeros(d, e, dtype=F64)
        n = torch.zeros(d, dtype=F64)
        mx = 0.0
        for i in range(t):
            f, ii = fg[i, head].item(), ig[i, head].item()
            m_new = max(f + mx, ii)
            keep, put = math.exp(f + mx - m_new), math.exp(ii - m_new)
            s = keep * s + put * torch.outer(k[i, head], v[i, head])
            n = keep * n + put * k[i, head]
            mx = m_new
            den = max(abs(float(n @ q[i, head])), math.exp(-mx)) + 1e-6
            o[i, head] = (s.T @ q[i, head]) / den
    o = rms_unit(o, eps).reshape(t, nh * e) * w[p + "norm"].to(F64)
    o = o * torch.sigmoid(h @ w[p + "g"].to(F64).T)
    return o @ w[p + "o"].to(F64).T


# ----------------------------------------------------------------------------- feed-forward
def route(h, router_w, top):
    """The ``top`` largest router logits of every token and the softmax over those alone."""
    z = h @ router_w.to(F64).T
    vals, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(vals, -1)


def moe(h, w, p, mlp):
    top, n = mlp["router"]["top"], mlp["router"]["experts"]
    idx, weight = route(h, w[p + "router"], top)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(idx[t, c])
            assert 0 <= e < n
            a = silu(w[f"{p}e{e}.gate"].to(F64) @ h[t]) * (w[f"{p}e{e}.up"].to(F64) @ h[t])
            out[t] += weight[t, c] * (w[f"{p}e{e}.down"].to(F64) @ a)
    return out


# ----------------------------------------------------------------------------- the model
def forward(config, w, tokens, layer_outputs=None):
    """Logits [T, vocab] of one whole sequence from position 0.  ``layer_outputs``: a list that
    receives the residual stream after every layer."""
    eps = float(config["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    x = w["embed"].to(F64)[tokens] * float(config["embedding"]["scale"])
    held = {}                                             # layer -> (keys, values) as its cache holds them
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = rms_norm(x, w[p + "norm1"].to(F64), eps)
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                held[i] = attention_keys_values(h, w, p + "mix.", m, eps, positions)
                src = i
            mix = attention(h, w, p + "mix.", m, eps, positions, *held[src])
        elif layer["type"] == "mamba2":
            mix = mamba2(h, w, p + "mix.", m, eps)
        elif layer["type"] == "mlstm":
            mix = mlstm(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        y = mix * w[p + "ls1"].to(F64)
        if layer.get("mlp") is not None:
            y = y + moe(h, w, p + "mlp.", layer["mlp"]) * w[p + "ls2"].to(F64)
        x = x + y
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    x = rms_norm(x, w["final.norm"].to(F64), eps)
    return x @ w["head"].to(F64).T


def greedy(config, w, prompt, n_new):
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = int(forward(config, w, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out
