"""Gated delta rule with a decay per key channel: a recurrent mixer with fixed-size state.

Per token, with h the normalised input, H value heads of size e, G key heads of size d (value head
a reads key head a // (H / G)) and a causal convolution of K taps per channel:

    q, k = silu(conv(W_q h)), silu(conv(W_k h))      made unit vectors per head; q also times d^-1/2
    v    = silu(conv(W_v h))
    beta = sigmoid(W_b h)                            one per head
    g    = exp(-exp(A_log) * softplus(W_a2 (W_a1 h) + dt_bias))     one per head and key channel
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q        (S is [d, e] per head)
    y    = W_o [ o / rms(o) * w_norm * sigmoid(W_g2 (W_g1 h)) ]               (rms per head over e)

The state of a sequence - S of every head in 32-bit and the convolution's last K - 1 inputs - is one
``state`` cache entry, zero for a new sequence; prompts, portions of prompts and single tokens all
read it, run the tokens they bring and write it back.  Everything between the projections and W_o is
computed in 32-bit.  The inner sizes of the two low-rank pairs (a1/a2, g1/g2) are read off the
tensors.

Parameters: ``hidden_size``, ``num_heads`` (H), ``num_kv_heads`` (G), ``head_dim`` (d), ``v_dim`` (e),
``conv`` (K), ``eps``, optional ``rank`` (inner size of both low-rank pairs when weights are drawn at
random).  Tensors: ``q``, ``k`` [G d, hidden], ``v`` [H e, hidden], ``q_conv``, ``k_conv``, ``v_conv``
[channels, K] (last column: the current token), ``b`` [H, hidden], ``A_log`` [H], ``dt_bias`` [H d],
``a1`` [ra, hidden], ``a2`` [H d, ra], ``g1`` [rg, hidden], ``g2`` [H e, rg], ``norm`` [e], ``o`` [hidden, H e].
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import linear
from ..registry import register_part
from .base import Mixer
from .spec import CacheSpec, TensorSpec


@register_part("mixer", "channel_delta")
class ChannelDelta(Mixer):
    @classmethod
    def tensors(cls, spec):
        p, w = spec.params, spec.weights
        hid, nh, g, d, e, k = (p["hidden_size"], p["num_heads"], p["num_kv_heads"], p["head_dim"], p["v_dim"],
                               p["conv"])
        free = dict(free_size=int(p.get("rank") or 16))
        return [TensorSpec(w["q"], (g * d, hid)), TensorSpec(w["k"], (g * d, hid)), TensorSpec(w["v"], (nh * e, hid)),
                TensorSpec(w["q_conv"], (g * d, k)), TensorSpec(w["k_conv"], (g * d, k)),
                TensorSpec(w["v_conv"], (nh * e, k)), TensorSpec(w["b"], (nh, hid)),
                TensorSpec(w["A_log"], (nh,)), TensorSpec(w["dt_bias"], (nh * d,)),
                TensorSpec(w["a1"], (-1, hid), **free), TensorSpec(w["a2"], (nh * d, -1), **free),
                TensorSpec(w["g1"], (-1, hid), **free), TensorSpec(w["g2"], (nh * e, -1), **free),
                TensorSpec(w["norm"], (e,), "gain"), TensorSpec(w["o"], (hid, nh * e))]

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        g = lambda n: int(self.param(n))
        self.hidden, self.num_heads, self.num_kv_heads = g("hidden_size"), g("num_heads"), g("num_kv_heads")
        self.head_dim, self.v_dim, self.taps = g("head_dim"), g("v_dim"), g("conv")
        self.eps = float(self.param("eps"))
        if self.num_heads % self.num_kv_heads:
            raise ValueError("channel_delta: num_heads must be a multiple of num_kv_heads")
        if self.taps < 1:
            raise ValueError("channel_delta: the convolution has at least one tap")
        self.rows = kernels.delta_state_rows(self.head_dim)
        self.channels = 2 * self.num_kv_heads * self.head_dim + self.num_heads * self.v_dim
        self.s_values = self.num_heads * self.v_dim * self.rows
        self.rank_a = self.rank_g = 0
        self.w_in = self.w_o = self.conv_w = self.a2t = self.g2t = None
        self.dt_bias = self.a_log = self.norm_w = None

    def cache_spec(self):
        # (a multiple of four values, so that every slot's S starts on a 16-byte boundary)
        return CacheSpec("state", shape=(-(-(self.s_values + self.channels * (self.taps - 1)) // 4) * 4,))

    def load(self, tensors):
        w, f32 = self.spec.weights, torch.float32
        a1, a2, g1, g2 = (tensors[w[n]] for n in ("a1", "a2", "g1", "g2"))
        if a1.shape[0] != a2.shape[1] or g1.shape[0] != g2.shape[1]:
            raise ValueError("channel_delta: the inner sizes of a1/a2 or g1/g2 disagree")
        self.rank_a, self.rank_g = a1.shape[0], g1.shape[0]
        # one product for everything that reads the input: [q | k | v | beta | a1 | g1]
        # (zero rows up to a multiple of 64: the library's product of many rows is much slower on a ragged count)
        rows = [tensors[w["q"]], tensors[w["k"]], tensors[w["v"]], tensors[w["b"]], a1, g1]
        n = sum(r.shape[0] for r in rows)
        rows.append(torch.zeros((-n % 64, self.hidden), dtype=a1.dtype, device=a1.device))
        self.w_in = torch.cat(rows, 0).to(self.dtype).contiguous()
        self.conv_w = torch.cat([tensors[w["q_conv"]], tensors[w["k_conv"]], tensors[w["v_conv"]]], 0) \
            .to(f32).contiguous()
        self.a2t = a2.to(f32).t().contiguous()              # [ra, H d]: neighbouring channels side by side
        self.g2t = g2.to(f32).t().contiguous()
        self.dt_bias = tensors[w["dt_bias"]].to(f32).contiguous()
        self.a_log = tensors[w["A_log"]].to(f32).contiguous()
        self.norm_w = tensors[w["norm"]].to(f32).contiguous()
        self.w_o = tensors[w["o"]].to(self.dtype).contiguous()

    def shape(self):
        return (self.num_heads, self.num_kv_heads, self.head_dim, self.v_dim, self.taps, self.rank_a, self.rank_g)

    def forward(self, x, ctx, entry, writes_cache=True):
        t, ws, f32 = ctx.n_tokens, ctx.workspace, torch.float32
        nh, g, d, e = self.num_heads, self.num_kv_heads, self.head_dim, self.v_dim
        state = entry.state                                  # [slots, values] 32-bit
        proj = linear(x, self.w_in, ctx, "delta_in", n_rows=t, out_dtype=f32, wide_f32="library")
        qn = ws.get("delta_q", (t, g * d), f32)
        kn = ws.get("delta_k", (t, g * d), f32)
        vc = ws.get("delta_v", (t, nh * e), f32)
        beta = ws.get("delta_beta", (t, nh), f32)
        decay = ws.get("delta_decay", (t, nh * d), f32)
        gate = ws.get("delta_gate", (t, nh * e), f32)
        off_a = self.channels + nh
        kernels.delta_low_rank(decay, proj, t, off_a, self.a2t, bias=self.dt_bias, a_log=self.a_log, dim=d)
        kernels.delta_low_rank(gate, proj, t, off_a + self.rank_a, self.g2t)
        kernels.delta_prepare(qn, kn, vc, beta, proj, t, self.conv_w, state, self.s_values, ctx.positions,
                              ctx.token_slot, self.shape())
        if writes_cache:
            kernels.delta_conv_tail(state, self.s_values, proj, ctx.cu_seqlens, ctx.positions, ctx.token_slot,
                                    ctx.n_seqs, self.channels, self.taps)
        o = ws.get("delta_o", (t, nh * e), f32)
        kernels.delta_scan(o, qn, kn, vc, beta, decay, state, ctx.cu_seqlens, ctx.positions, ctx.token_slot,
                           ctx.n_seqs, nh, g, d, e, n_tokens=t)
        y = ws.get("attn_out", (t, nh * e), self.dtype)
        kernels.delta_out_norm(y, o, gate, self.norm_w, self.eps, ctx.positions, t, self.shape())
        return linear(y, self.w_o, ctx, "attn_proj", n_rows=t)


@register_part("mixer", "head_delta")
class HeadDelta(Mixer):
    """Gated delta rule with ONE decay per head (the gated delta network): the recurrence of
    :class:`ChannelDelta` with a scalar in place of the decay vector, plain projections in place of its
    low-rank pairs, and a SiLU output gate.

        q, k = silu(conv(W_q h)), silu(conv(W_k h))      unit vectors per head; q also times d^-1/2
        v    = silu(conv(W_v h));   beta = sigmoid(W_b h)
        g    = exp(-exp(A_log) * softplus(W_a h + dt_bias))                     one per head
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q             (S is [d, e] per head)
        y    = W_o [ o / rms(o) * w_norm * silu(W_g h) ]                         (rms per head over e)

    The state of a sequence - S of every head in 32-bit and the convolution's last K - 1 inputs - is one
    ``state`` cache entry.  Everything between the projections and W_o is computed in 32-bit, with the
    kernels of the per-channel form.  Parameters: ``hidden_size``, ``num_heads`` (H), ``num_kv_heads``
    (G), ``head_dim`` (d), ``v_dim`` (e), ``conv`` (K), ``eps``.  Tensors: ``q``, ``k`` [G d, hidden],
    ``v`` [H e, hidden], ``q_conv``, ``k_conv``, ``v_conv`` [channels, K], ``b``, ``a`` [H, hidden],
    ``A_log``, ``dt_bias`` [H], ``g`` [H e, hidden], ``norm`` [e], ``o`` [hidden, H e].
    """

    @classmethod
    def tensors(cls, spec):
        p, w = spec.params, spec.weights
        hid, nh, g, d, e, k = (p["hidden_size"], p["num_heads"], p["num_kv_heads"], p["head_dim"], p["v_dim"],
                               p["conv"])
        return [TensorSpec(w["q"], (g * d, hid)), TensorSpec(w["k"], (g * d, hid)), TensorSpec(w["v"], (nh * e, hid)),
                TensorSpec(w["q_conv"], (g * d, k)), TensorSpec(w["k_conv"], (g * d, k)),
                TensorSpec(w["v_conv"], (nh * e, k)), TensorSpec(w["b"], (nh, hid)), TensorSpec(w["a"], (nh, hid)),
                TensorSpec(w["A_log"], (nh,)), TensorSpec(w["dt_bias"], (nh,)), TensorSpec(w["g"], (nh * e, hid)),
                TensorSpec(w["norm"], (e,), "gain"), TensorSpec(w["o"], (hid, nh * e))]

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        g = lambda n: int(self.param(n))
        self.hidden, self.num_heads, self.num_kv_heads = g("hidden_size"), g("num_heads"), g("num_kv_heads")
        self.head_dim, self.v_dim, self.taps = g("head_dim"), g("v_dim"), g("conv")
        self.eps = float(self.param("eps"))
        if self.num_heads % self.num_kv_heads:
            raise ValueError("head_delta: num_heads must be a multiple of num_kv_heads")
        if self.taps < 1:
            raise ValueError("head_delta: the convolution has at least one tap")
        self.rows = kernels.delta_state_rows(self.head_dim)
        self.channels = 2 * self.num_kv_heads * self.head_dim + self.num_heads * self.v_dim
        self.s_values = self.num_heads * self.v_dim * self.rows
        self.w_in = self.w_o = self.conv_w = self.dt_bias = self.a_log = self.norm_w = None

    def cache_spec(self):
        # (a multiple of four values, so that every slot's S starts on a 16-byte boundary)
        return CacheSpec("state", shape=(-(-(self.s_values + self.channels * (self.taps - 1)) // 4) * 4,))

    def load(self, tensors):
        w, f32 = self.spec.weights, torch.float32
        # one product for everything that reads the input: [q | k | v | beta | a | g] (zero rows up to a
        # multiple of 64, as the per-channel form has them)
        rows = [tensors[w[n]] for n in ("q", "k", "v", "b", "a", "g")]
        n = sum(r.shape[0] for r in rows)
        rows.append(torch.zeros((-n % 64, self.hidden), dtype=rows[0].dtype, device=rows[0].device))
        self.w_in = torch.cat(rows, 0).to(self.dtype).contiguous()
        self.conv_w = torch.cat([tensors[w["q_conv"]], tensors[w["k_conv"]], tensors[w["v_conv"]]], 0) \
            .to(f32).contiguous()
        self.dt_bias = tensors[w["dt_bias"]].to(f32).contiguous()
        self.a_log = tensors[w["A_log"]].to(f32).contiguous()
        self.norm_w = tensors[w["norm"]].to(f32).contiguous()
        self.w_o = tensors[w["o"]].to(self.dtype).contiguous()

    def shape(self):
        """The per-channel kernels' shape: the decay logits and the gate stand where its two low-rank
        first halves do."""
        return (self.num_heads, self.num_kv_heads, self.head_dim, self.v_dim, self.taps, self.num_heads,
                self.num_heads * self.v_dim)

    def forward(self, x, ctx, entry, writes_cache=True):
        t, ws, f32 = ctx.n_tokens, ctx.workspace, torch.float32
        nh, g, d, e = self.num_heads, self.num_kv_heads, self.head_dim, self.v_dim
        state = entry.state                                  # [slots, values] 32-bit
        proj = linear(x, self.w_in, ctx, "delta_in", n_rows=t, out_dtype=f32, wide_f32="library")
        qn = ws.get("delta_q", (t, g * d), f32)
        kn = ws.get("delta_k", (t, g * d), f32)
        vc = ws.get("delta_v", (t, nh * e), f32)
        beta = ws.get("delta_beta", (t, nh), f32)
        decay = ws.get("delta_head_decay", (t, nh), f32)
        unused = ws.get("delta_head_dt", (t, nh), f32)
        col_a = self.channels + nh
        kernels.ssm_gates(decay, unused, proj, col_a, self.dt_bias, self.a_log, t, nh)
        kernels.delta_prepare(qn, kn, vc, beta, proj, t, self.conv_w, state, self.s_values, ctx.positions,
                              ctx.token_slot, self.shape())
        if writes_cache:
            kernels.delta_conv_tail(state, self.s_values, proj, ctx.cu_seqlens, ctx.positions, ctx.token_slot,
                                    ctx.n_seqs, self.channels, self.taps)
        o = ws.get("delta_o", (t, nh * e), f32)
        kernels.delta_scan(o, qn, kn, vc, beta, decay, state, ctx.cu_seqlens, ctx.positions, ctx.token_slot,
                           ctx.n_seqs, nh, g, d, e, n_tokens=t, decay_per_head=True)
        y = ws.get("attn_out", (t, nh * e), self.dtype)
        kernels.delta_out_norm(y, o, proj[:, col_a + nh:], self.norm_w, self.eps, ctx.positions, t, self.shape(),
                               gate_activation="silu")
        return linear(y, self.w_o, ctx, "attn_proj", n_rows=t)
