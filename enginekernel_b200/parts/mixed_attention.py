"""Grouped-query attention whose heads share their softmax weights ("talking heads" behind the softmax).

Per token, with h the normalised input, H query heads on G key/value heads (query head a reads key/value
head c(a) = a // (H / G)), key size d, value size e:

    q = W_q h + b_q,  k = W_k h + b_k,  v = W_v h + b_v
    q, k <- gain * x / rms(x) per head over d (one gain vector for all heads), then rotated: the first
            ``rotary_dim`` values of a head turn in neighbouring pairs (2i, 2i + 1) by position * theta^(-2i/rot)
    v <- v / rms(v) per head over e (no gain); keys and values are cached in this form
    w_a(i, j) = softmax_j(scale q_a(i) . k_c(a)(j))   over j <= i with i - j < window or j < keep_first
    w_a <- sum_b mix[a, b] w_b                        (the heads' weights are mixed)
    o_a(i) = sum_j w_a(i, j) v_c(a)(j);   y = W_o [ o * sigmoid(W_g h) ]      (the gate element by element)

Because the mix is linear, o_a = sum_b mix[a, b] A[b, c(a)] with A[b, c] = head b's own weights applied to
the values of key/value head c; the attention kernel writes A (32-bit) and a second kernel forms the sums,
applies the gate and rounds.  Scores, softmax, A and the sums are 32-bit.

The kernels and the cache see heads of one size, max(d, e) rounded up to 8 values (32 in bfloat16), the shorter
ones padded with zeros (zero weight rows); the norms take their means over the true sizes.  The pairing of neighbours is
turned into the half-split pairing the rotation kernels use by reordering the rows of W_q and W_k (and their
biases and gains) once at load: scores do not change when queries and keys are permuted alike.

Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``value_dim``, ``scale``, ``eps``
(of all three norms), ``window`` (None: all keys), ``keep_first``, ``position`` (a position PartSpec or None).
Tensors: ``q`` [H d, hidden], ``k`` [G d, hidden], ``v`` [G e, hidden] with ``q_bias``, ``k_bias``, ``v_bias``;
``q_norm``, ``k_norm`` [d]; ``mix`` [H, H]; ``gate`` [H e, hidden]; ``o`` [hidden, H e].
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import linear
from ..registry import lookup_part, register_part
from .attention import _no_table
from .base import Mixer
from .spec import CacheSpec, TensorSpec


def neighbours_to_halves(dim: int, rotary_dim: int) -> torch.Tensor:
    """Order of a head's values that turns the pairs (2i, 2i + 1) of its first ``rotary_dim`` values into
    the pairs (i, i + rotary_dim / 2): new[i] = old[order[i]]."""
    even = list(range(0, rotary_dim, 2))
    odd = list(range(1, rotary_dim, 2))
    return torch.tensor(even + odd + list(range(rotary_dim, dim)), dtype=torch.long)


@register_part("mixer", "mixed_head_attention")
class MixedHeadAttention(Mixer):
    @classmethod
    def tensors(cls, spec):
        p, w = spec.params, spec.weights
        h, nh, g, d, e = p["hidden_size"], p["num_heads"], p["num_kv_heads"], p["head_dim"], p["value_dim"]
        return [TensorSpec(w["q"], (nh * d, h)), TensorSpec(w["q_bias"], (nh * d,)),
                TensorSpec(w["k"], (g * d, h)), TensorSpec(w["k_bias"], (g * d,)),
                TensorSpec(w["v"], (g * e, h)), TensorSpec(w["v_bias"], (g * e,)),
                TensorSpec(w["q_norm"], (d,), "gain"), TensorSpec(w["k_norm"], (d,), "gain"),
                TensorSpec(w["mix"], (nh, nh)), TensorSpec(w["gate"], (nh * e, h)), TensorSpec(w["o"], (h, nh * e))]

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        g = lambda n: int(self.param(n))
        self.hidden, self.num_heads, self.num_kv_heads = g("hidden_size"), g("num_heads"), g("num_kv_heads")
        self.head_dim, self.value_dim = g("head_dim"), g("value_dim")
        self.scale, self.eps = float(self.param("scale")), float(self.param("eps"))
        self.window = spec.params.get("window")
        self.keep_first = int(spec.params.get("keep_first") or 0)
        if self.num_heads % self.num_kv_heads:
            raise ValueError("mixed_head_attention: num_heads must be a multiple of num_kv_heads")
        if self.keep_first and not self.window:
            raise ValueError("mixed_head_attention: keep_first needs a window")
        # (in bfloat16 a multiple of 32, which both 16-bit attention kernels take)
        unit = 32 if dtype == torch.bfloat16 else 8
        self.padded_dim = -(-max(self.head_dim, self.value_dim) // unit) * unit
        kernels.check_head_dim(self.padded_dim)
        pos = spec.params.get("position")
        self.position = lookup_part("position", pos.kind)(pos, dtype, device) if pos else None
        self.rotary_dim = int(getattr(self.position, "rotary_dim", 0)) if self.position is not None else 0
        if self.rotary_dim > self.head_dim:
            raise ValueError("mixed_head_attention: the rotation covers more values than a head has")
        self.w_in = self.w_o = self.q_gain = self.k_gain = self.mix = None
        self.q_bias = self.k_bias = self.v_bias = None
        self.gate_col = (self.num_heads + 2 * self.num_kv_heads) * self.padded_dim

    def cache_spec(self):
        return CacheSpec("kv", heads=self.num_kv_heads, head_dim=self.padded_dim,
                         window=None if self.keep_first else self.window)

    def prepare(self, max_positions):
        if self.position is not None:
            self.position.prepare(max_positions)

    def load(self, tensors):
        w, f32, big = self.spec.weights, torch.float32, self.padded_dim
        order = neighbours_to_halves(self.head_dim, self.rotary_dim).to(self.device)

        def heads(t, n, size, reorder):
            """[n * size, ...] -> [n * big, ...]: values of a head reordered, zeros behind them."""
            t = t.reshape(n, size, *t.shape[1:])
            if reorder:
                t = t.index_select(1, order)
            out = torch.zeros((n, big) + tuple(t.shape[2:]), dtype=t.dtype, device=t.device)
            out[:, :size] = t
            return out.reshape(n * big, *t.shape[2:])

        nh, g, d, e = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        rows = [heads(tensors[w["q"]], nh, d, True), heads(tensors[w["k"]], g, d, True),
                heads(tensors[w["v"]], g, e, False), tensors[w["gate"]]]
        n = sum(r.shape[0] for r in rows)
        if n % 64:
            rows.append(torch.zeros((-n % 64, self.hidden), dtype=rows[0].dtype, device=rows[0].device))
        self.w_in = torch.cat(rows, 0).to(self.dtype).contiguous()
        self.q_bias = heads(tensors[w["q_bias"]].to(f32), nh, d, True).contiguous()
        self.k_bias = heads(tensors[w["k_bias"]].to(f32), g, d, True).contiguous()
        self.v_bias = heads(tensors[w["v_bias"]].to(f32), g, e, False).contiguous()
        self.q_gain = heads(tensors[w["q_norm"]].to(f32), 1, d, True).contiguous()
        self.k_gain = heads(tensors[w["k_norm"]].to(f32), 1, d, True).contiguous()
        self.mix = tensors[w["mix"]].to(f32).contiguous()
        self.w_o = tensors[w["o"]].to(self.dtype).contiguous()

    def bytes_read_per_step(self, n_tokens):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o, self.q_gain, self.k_gain, self.mix,
                                                          self.q_bias, self.k_bias, self.v_bias))

    def forward(self, x, ctx, entry, writes_cache=True):
        t, big, nh, g = ctx.n_tokens, self.padded_dim, self.num_heads, self.num_kv_heads
        pos = self.position
        rows = linear(x, self.w_in, ctx, "qkv", n_rows=t)
        kernels.qk_prepare_padded_kv(
            rows, t, self.q_gain, self.k_gain, pos.cos if pos else _no_table(self.device),
            pos.sin if pos else _no_table(self.device), self.rotary_dim, ctx.positions, ctx.token_slot,
            entry.k_pages, entry.v_pages, entry.block_table, nh, g, big, self.eps, self.head_dim,
            write_kv=writes_cache, q_bias=self.q_bias, k_bias=self.k_bias, v_bias=self.v_bias,
            value_unit_eps=self.eps, value_dim=self.value_dim)
        parts = ctx.workspace.get("mixed_parts", (t, nh, g, big), torch.float32)
        out = ctx.workspace.get("attn_out", (t, nh * self.value_dim), self.dtype)
        if not ctx.is_decode and kernels.attention_prefill_supported(self.dtype, big, nh, g):
            kernels.attention_prefill_cross_bf16(parts, rows, t, ctx.positions, ctx.token_slot, ctx.cu_seqlens,
                                                 ctx.n_seqs, entry.k_pages, entry.v_pages, entry.block_table, nh, g,
                                                 big, self.scale, self.window, keep_first=self.keep_first)
            kernels.mix_heads(out, parts, self.mix, ctx.positions, t, nh, g, big, self.value_dim,
                              gate=rows[:, self.gate_col:])
            return linear(out, self.w_o, ctx, "attn_proj", n_rows=t)
        visible = min(ctx.max_context, self.window + self.keep_first) if self.window else ctx.max_context
        if ctx.is_decode and kernels.attention_decode_supported(self.dtype, big):
            # blocks = tokens x key heads (x 16-row blocks of the group) x value heads, three fit an SM: every
            # token's own window is cut so that the blocks about fill the machine, never finer than two pages a split
            blocks = t * g * -(-(nh // g) // 16) * g
            splits = max(1, min(3 * kernels.sm_count(self.device) // blocks, -(-visible // 128)))
            acc = ml = None
            if splits > 1:
                acc = ctx.workspace.get("attn_part_acc", (t, nh * g, splits, big), torch.float32)
                ml = ctx.workspace.get("attn_part_ml", (t, nh * g, splits, 2), torch.float32)
            kernels.attention_decode_cross_bf16(parts, rows, t, ctx.positions, ctx.token_slot, entry.k_pages,
                                                entry.v_pages, entry.block_table, nh, g, big, self.scale, self.window,
                                                splits, 0, acc, ml, keep_first=self.keep_first)
            kernels.mix_heads(out, parts, self.mix, ctx.positions, t, nh, g, big, self.value_dim,
                              gate=rows[:, self.gate_col:])
            return linear(out, self.w_o, ctx, "attn_proj", n_rows=t)
        splits, per_split, acc, ml = 1, 0, None, None
        blocks = t * nh * g
        if blocks < 2 * kernels.sm_count(self.device) and visible > 512:
            splits = max(1, min(-(-visible // 256), -(-4 * kernels.sm_count(self.device) // blocks), 64))
        if splits > 1:
            per_split = -(-(-(-ctx.max_context // splits)) // 128) * 128
            splits = -(-ctx.max_context // per_split)
        if splits > 1:
            acc = ctx.workspace.get("attn_part_acc", (t, nh * g, splits, big), torch.float32)
            ml = ctx.workspace.get("attn_part_ml", (t, nh * g, splits, 2), torch.float32)
        kernels.attention_generic_cross(parts, rows, t, ctx.positions, ctx.token_slot, entry.k_pages, entry.v_pages,
                                        entry.block_table, nh, g, big, self.scale, self.window, splits, per_split,
                                        acc, ml, keep_first=self.keep_first)
        kernels.mix_heads(out, parts, self.mix, ctx.positions, t, nh, g, big, self.value_dim,
                          gate=rows[:, self.gate_col:])
        return linear(out, self.w_o, ctx, "attn_proj", n_rows=t)
