"""Two recurrent mixers with a decay per head and token, over one scan kernel, and one with a decay per
channel and no matrix state (``gated_linear_recurrence``, described at its class).

Both keep a matrix S [key size, value size] per head and sequence in 32-bit and update it token by token,

    S_t = a_t S_(t-1) + b_t k_t v_t^T        o_t = S_t^T q_t

with scalars a_t, b_t per head; they differ in where q, k, v, a and b come from and in what follows o.
The state of a sequence is one ``state`` cache entry, zero for a new sequence; prompts, portions of
prompts and single tokens all read it, run the tokens they bring and write it back.  Everything between
the input projection and the output projection is computed in 32-bit.

``state_space`` (state-space duality, the Mamba-2 layer).  With H heads of value size e, state size N,
G groups (head h reads group h // (H / G)), inner = H e, and a causal convolution of K taps:

    [z | x | B | C | dt] = W_in h                    (inner, inner, G N, G N, H values)
    [x | B | C] <- silu(conv([x | B | C]) + bias)    per channel, the last column is the current token's
    dt <- softplus(dt + dt_bias);  a = exp(-exp(A_log) dt);  b = dt;  k = B, q = C, v = x
    y = o + D x (D per head);  y <- y silu(z);  y <- y / rms(y) w over each of ``norm_groups`` equal parts
    out = W_o y

The state also holds the convolution's last K - 1 inputs.  Parameters: ``hidden_size``, ``num_heads``,
``v_dim``, ``state``, ``groups``, ``conv``, ``norm_groups``, ``eps``.  Tensors: ``in`` [2 inner + 2 G N +
H, hidden], ``conv`` [inner + 2 G N, K], ``conv_bias``, ``dt_bias`` [H], ``A_log`` [H], ``D`` [H], ``norm``
[inner], ``o`` [hidden, inner].

``matrix_memory`` (the mLSTM cell of xLSTM).  H heads, key size d, value size e, gate cap c:

    q = W_q h d^-1/2, k = W_k h, v = W_v h
    i = c tanh((W_i h + b_i) / c);  f = logsigmoid(c tanh((W_f h + b_f) / c))        per head
    m_t = max(f + m_(t-1), i), m_0 = 0;  a = exp(f + m_(t-1) - m_t);  b = exp(i - m_t)
    n_t = a n_(t-1) + b k;  o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)
    y = o / rms(o) per head * w * sigmoid(W_g h);  out = W_o y

n rides in the scan as one more column of S whose v is 1; the state also holds m per head.
Parameters: ``hidden_size``, ``num_heads``, ``head_dim``, ``v_dim``, ``gate_cap``, ``eps``.  Tensors: ``q``,
``k`` [H d, hidden], ``v``, ``g`` [H e, hidden], ``i``, ``f`` [H, hidden], ``i_bias``, ``f_bias`` [H], ``norm``
[H e], ``o`` [hidden, H e].
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import linear
from ..registry import register_part
from .base import Mixer
from .spec import CacheSpec, TensorSpec


def _padded_rows(rows, hidden, multiple=64):
    """The projection's weight with zero rows up to a multiple of ``multiple`` (the library's product of
    many rows is much slower on a ragged count)."""
    n = sum(r.shape[0] for r in rows)
    if n % multiple:
        rows = list(rows) + [torch.zeros((-n % multiple, hidden), dtype=rows[0].dtype, device=rows[0].device)]
    return torch.cat(rows, 0)


@register_part("mixer", "state_space")
class StateSpace(Mixer):
    @classmethod
    def tensors(cls, spec):
        p, w = spec.params, spec.weights
        hid, nh, e, n, g, k = (p["hidden_size"], p["num_heads"], p["v_dim"], p["state"], p["groups"], p["conv"])
        inner, ch = nh * e, nh * e + 2 * g * n
        return [TensorSpec(w["in"], (2 * inner + 2 * g * n + nh, hid)), TensorSpec(w["conv"], (ch, k)),
                TensorSpec(w["conv_bias"], (ch,)), TensorSpec(w["dt_bias"], (nh,)), TensorSpec(w["A_log"], (nh,)),
                TensorSpec(w["D"], (nh,), "gain"), TensorSpec(w["norm"], (inner,), "gain"),
                TensorSpec(w["o"], (hid, inner))]

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        g = lambda n: int(self.param(n))
        self.hidden, self.num_heads, self.v_dim, self.n_state = g("hidden_size"), g("num_heads"), g("v_dim"), g("state")
        self.groups, self.taps, self.norm_groups = g("groups"), g("conv"), g("norm_groups")
        self.eps = float(self.param("eps"))
        self.inner = self.num_heads * self.v_dim
        if self.num_heads % self.groups:
            raise ValueError("state_space: groups must divide the heads")
        if self.inner % self.norm_groups:
            raise ValueError("state_space: norm_groups must divide heads * v_dim")
        if self.taps < 1:
            raise ValueError("state_space: the convolution has at least one tap")
        self.rows = kernels.decay_scan_rows(self.n_state)
        self.channels = self.inner + 2 * self.groups * self.n_state
        self.s_values = self.num_heads * self.v_dim * self.rows
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d_skip = self.norm_w = None

    def cache_spec(self):
        # (a multiple of four values, so that every slot's S starts on a 16-byte boundary)
        return CacheSpec("state", shape=(-(-(self.s_values + self.channels * (self.taps - 1)) // 4) * 4,))

    def load(self, tensors):
        w, f32 = self.spec.weights, torch.float32
        self.w_in = _padded_rows([tensors[w["in"]]], self.hidden).to(self.dtype).contiguous()
        self.conv_w = tensors[w["conv"]].to(f32).contiguous()
        self.conv_b = tensors[w["conv_bias"]].to(f32).contiguous()
        self.dt_bias = tensors[w["dt_bias"]].to(f32).contiguous()
        self.a_log = tensors[w["A_log"]].to(f32).contiguous()
        self.d_skip = tensors[w["D"]].to(f32).contiguous()
        self.norm_w = tensors[w["norm"]].to(f32).contiguous()
        self.w_o = tensors[w["o"]].to(self.dtype).contiguous()

    def forward(self, x, ctx, entry, writes_cache=True):
        t, ws, f32 = ctx.n_tokens, ctx.workspace, torch.float32
        nh, e, n, g, inner, ch = self.num_heads, self.v_dim, self.n_state, self.groups, self.inner, self.channels
        state = entry.state                                  # [slots, values] 32-bit
        proj = linear(x, self.w_in, ctx, "ssm_in", n_rows=t, out_dtype=f32, wide_f32="library")
        xbc = ws.get("ssm_xbc", (t, ch), f32)
        kernels.conv_silu(xbc, proj, inner, self.conv_w, self.conv_b, state, self.s_values, ctx.positions,
                          ctx.token_slot, t, ch, self.taps)
        if writes_cache:
            kernels.conv_tail(state, self.s_values, proj, inner, ctx.cu_seqlens, ctx.positions, ctx.token_slot,
                              ctx.n_seqs, ch, self.taps)
        a = ws.get("scan_a", (t, nh), f32)
        b = ws.get("scan_b", (t, nh), f32)
        kernels.ssm_gates(a, b, proj, inner + ch, self.dt_bias, self.a_log, t, nh)
        o = ws.get("scan_o", (t, inner), f32)
        kernels.decay_scan(o, xbc[:, inner + g * n:], xbc[:, inner:inner + g * n], xbc, a, b, state,
                           ctx.cu_seqlens, ctx.positions, ctx.token_slot, ctx.n_seqs, nh, g, n, e,
                           write_state=writes_cache, n_tokens=t)
        y = ws.get("attn_out", (t, inner), self.dtype)
        kernels.ssm_out(y, o, xbc, proj, 0, self.d_skip, self.norm_w, self.eps, ctx.positions, t, inner, e,
                        self.norm_groups)
        return linear(y, self.w_o, ctx, "attn_proj", n_rows=t)


@register_part("mixer", "matrix_memory")
class MatrixMemory(Mixer):
    @classmethod
    def tensors(cls, spec):
        p, w = spec.params, spec.weights
        hid, nh, d, e = p["hidden_size"], p["num_heads"], p["head_dim"], p["v_dim"]
        return [TensorSpec(w["q"], (nh * d, hid)), TensorSpec(w["k"], (nh * d, hid)), TensorSpec(w["v"], (nh * e, hid)),
                TensorSpec(w["g"], (nh * e, hid)), TensorSpec(w["i"], (nh, hid)), TensorSpec(w["f"], (nh, hid)),
                TensorSpec(w["i_bias"], (nh,)), TensorSpec(w["f_bias"], (nh,)),
                TensorSpec(w["norm"], (nh * e,), "gain"), TensorSpec(w["o"], (hid, nh * e))]

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        g = lambda n: int(self.param(n))
        self.hidden, self.num_heads, self.head_dim, self.v_dim = g("hidden_size"), g("num_heads"), g("head_dim"), g("v_dim")
        self.cap, self.eps = float(self.param("gate_cap")), float(self.param("eps"))
        if not self.cap > 0:
            raise ValueError("matrix_memory: the gate cap must be positive")
        self.rows = kernels.decay_scan_rows(self.head_dim)
        self.s_values = self.num_heads * (self.v_dim + 1) * self.rows
        self.w_in = self.w_o = self.bias_i = self.bias_f = self.norm_w = None

    def cache_spec(self):
        return CacheSpec("state", shape=(-(-(self.s_values + self.num_heads) // 4) * 4,))

    def load(self, tensors):
        w, f32 = self.spec.weights, torch.float32
        # one product for everything that reads the input: [q | k | v | g | i | f]
        rows = [tensors[w[n]] for n in ("q", "k", "v", "g", "i", "f")]
        self.w_in = _padded_rows(rows, self.hidden).to(self.dtype).contiguous()
        self.bias_i = tensors[w["i_bias"]].to(f32).contiguous()
        self.bias_f = tensors[w["f_bias"]].to(f32).contiguous()
        self.norm_w = tensors[w["norm"]].to(f32).contiguous()
        self.w_o = tensors[w["o"]].to(self.dtype).contiguous()

    def forward(self, x, ctx, entry, writes_cache=True):
        t, ws, f32 = ctx.n_tokens, ctx.workspace, torch.float32
        nh, d, e = self.num_heads, self.head_dim, self.v_dim
        state = entry.state
        proj = linear(x, self.w_in, ctx, "xlstm_in", n_rows=t, out_dtype=f32, wide_f32="library")
        col_k, col_v = nh * d, 2 * nh * d
        col_g = col_v + nh * e
        col_i = col_g + nh * e
        a = ws.get("scan_a", (t, nh), f32)
        b = ws.get("scan_b", (t, nh), f32)
        m_run = ws.get("scan_m", (t, nh), f32)
        kernels.xgate_scan(a, b, m_run, proj, col_i, col_i + nh, self.bias_i, self.bias_f, self.cap, state,
                           self.s_values, ctx.cu_seqlens, ctx.positions, ctx.token_slot, ctx.n_seqs, nh,
                           write_state=writes_cache)
        o = ws.get("scan_o", (t, nh * (e + 1)), f32)
        kernels.decay_scan(o, proj, proj[:, col_k:], proj[:, col_v:], a, b, state, ctx.cu_seqlens, ctx.positions,
                           ctx.token_slot, ctx.n_seqs, nh, nh, d, e, ones_column=True, write_state=writes_cache,
                           n_tokens=t)
        y = ws.get("attn_out", (t, nh * e), self.dtype)
        kernels.xlstm_out(y, o, m_run, proj, col_g, self.norm_w, self.eps, d ** -0.5, ctx.positions, t, nh, e)
        return linear(y, self.w_o, ctx, "attn_proj", n_rows=t)


@register_part("mixer", "gated_linear_recurrence")
class GatedLinearRecurrence(Mixer):
    """The recurrent block of Griffin around a real-gated linear recurrent unit.  With R = ``width`` channels
    in ``blocks`` equal parts and a causal convolution of K taps per channel (bias, no activation):

        y = gelu_tanh(W_y h + b_y)                      u = conv(W_x h + b_x)
        r = sigmoid(A[p] u_p + a_bias),  i = sigmoid(I[p] u_p + i_bias)        per part p, square matrices
        a = exp(-rate * r * softplus(lam))              S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t
        out = W_o (S * y)

    S starts at zero for a new sequence, first token included.  The state of a sequence - S and the
    convolution's last K - 1 inputs, 32-bit - is one ``state`` cache entry.  The projections' results, the
    convolution, the gates and S are 32-bit; S * y is rounded once to the activation type.

    Parameters: ``hidden_size``, ``width``, ``blocks``, ``conv``, optional ``rate`` (8, the unit's constant).
    Tensors: ``y``, ``x`` [R, hidden] with ``y_bias``, ``x_bias`` [R]; ``conv`` [R, K] (last column: the
    current token), ``conv_bias`` [R]; ``a_gate``, ``i_gate`` [blocks, R / blocks, R / blocks] ([out, in])
    with ``a_gate_bias``, ``i_gate_bias`` [blocks, R / blocks]; ``lam`` [R]; ``o`` [hidden, R].
    """

    @classmethod
    def tensors(cls, spec):
        p, w = spec.params, spec.weights
        hid, r, nb, k = p["hidden_size"], p["width"], p["blocks"], p["conv"]
        size = r // nb
        return [TensorSpec(w["y"], (r, hid)), TensorSpec(w["y_bias"], (r,)), TensorSpec(w["x"], (r, hid)),
                TensorSpec(w["x_bias"], (r,)), TensorSpec(w["conv"], (r, k)), TensorSpec(w["conv_bias"], (r,)),
                TensorSpec(w["a_gate"], (nb, size, size)), TensorSpec(w["a_gate_bias"], (nb, size)),
                TensorSpec(w["i_gate"], (nb, size, size)), TensorSpec(w["i_gate_bias"], (nb, size)),
                TensorSpec(w["lam"], (r,)), TensorSpec(w["o"], (hid, r))]

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        g = lambda n: int(self.param(n))
        self.hidden, self.width, self.blocks, self.taps = g("hidden_size"), g("width"), g("blocks"), g("conv")
        self.rate = float(spec.params.get("rate", 8.0))
        if self.width % self.blocks:
            raise ValueError("gated_linear_recurrence: blocks must divide the width")
        if self.taps < 1:
            raise ValueError("gated_linear_recurrence: the convolution has at least one tap")
        self.size = self.width // self.blocks
        self.w_in = self.w_o = self.y_bias = self.x_bias = self.conv_w = self.conv_b = None
        self.w_a = self.w_i = self.w_a_rows = self.w_i_rows = self.b_a = self.b_i = self.lam = None

    def cache_spec(self):
        return CacheSpec("state", shape=(-(-(self.width * self.taps) // 4) * 4,))

    def load(self, tensors):
        w, f32 = self.spec.weights, torch.float32
        # one product for both branches: [y | x]
        self.w_in = _padded_rows([tensors[w["y"]], tensors[w["x"]]], self.hidden).to(self.dtype).contiguous()
        self.y_bias = tensors[w["y_bias"]].to(f32).contiguous()
        self.x_bias = tensors[w["x_bias"]].to(f32).contiguous()
        self.conv_w = tensors[w["conv"]].to(f32).contiguous()
        self.conv_b = tensors[w["conv_bias"]].to(f32).contiguous()
        # [part][in][out]: neighbouring threads of the gate kernel own neighbouring outputs
        self.w_a = tensors[w["a_gate"]].to(f32).transpose(1, 2).contiguous()
        self.w_i = tensors[w["i_gate"]].to(f32).transpose(1, 2).contiguous()
        # and as stored, [part][out][in], for steps of few tokens (a warp reads an output's row)
        self.w_a_rows = tensors[w["a_gate"]].to(f32).contiguous()
        self.w_i_rows = tensors[w["i_gate"]].to(f32).contiguous()
        self.b_a = tensors[w["a_gate_bias"]].to(f32).reshape(-1).contiguous()
        self.b_i = tensors[w["i_gate_bias"]].to(f32).reshape(-1).contiguous()
        self.lam = tensors[w["lam"]].to(f32).contiguous()
        self.w_o = tensors[w["o"]].to(self.dtype).contiguous()

    def forward(self, x, ctx, entry, writes_cache=True):
        t, ws, f32, r = ctx.n_tokens, ctx.workspace, torch.float32, self.width
        state = entry.state                                  # [slots, S | conv tail] 32-bit
        proj = linear(x, self.w_in, ctx, "lru_in", n_rows=t, out_dtype=f32, wide_f32="library")
        u = ws.get("lru_u", (t, r), f32)
        kernels.conv_act(u, proj, r, self.conv_w, self.conv_b, state, r, ctx.positions, ctx.token_slot, t, r,
                         self.taps, in_bias=self.x_bias, activation=None)
        if writes_cache:
            kernels.conv_tail(state, r, proj, r, ctx.cu_seqlens, ctx.positions, ctx.token_slot, ctx.n_seqs, r,
                              self.taps)
        a = ws.get("lru_a", (t, r), f32)
        xin = ws.get("lru_x", (t, r), f32)
        kernels.lru_gates(a, xin, u, self.w_a, self.b_a, self.w_i, self.b_i, self.lam, self.rate, t, self.blocks,
                          self.size, w_a_rows=self.w_a_rows, w_i_rows=self.w_i_rows)
        y = ws.get("attn_out", (t, r), self.dtype)
        kernels.lru_scan(y, a, xin, proj, 0, self.y_bias, state, ctx.cu_seqlens, ctx.positions, ctx.token_slot,
                         ctx.n_seqs, r, write_state=writes_cache, n_tokens=t, max_new=ctx.max_new)
        return linear(y, self.w_o, ctx, "attn_proj", n_rows=t)

    def bytes_read_per_step(self, n_tokens):
        # (the gates' matrices are held in two layouts; a step reads one of them)
        read = (self.w_in, self.w_o, self.w_a, self.w_i, self.y_bias, self.x_bias, self.conv_w, self.conv_b, self.b_a,
                self.b_i, self.lam)
        return sum(t.numel() * t.element_size() for t in read)
