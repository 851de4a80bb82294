"""Grouped-query attention over the paged cache.

Per token: q/k/v projections without bias (one fused product), optional RMSNorm of each
query and key head over the head dimension, position encoding of queries and keys, keys
and values stored in the cache entry, softmax(scale * q.K^T) V over the keys the token may
see (all earlier ones, or the last ``window``), output projection
(engine/ek_model.py:298-325 for prompts, 380-403 for decode; formula 475-488).
Query head h reads KV head h // (num_heads // num_kv_heads).

Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``,
``qk_norm_eps`` (None: no q/k norm), ``window`` (None: all keys), ``position`` (a
position PartSpec or None).  Tensors: ``q`` [NH*D, H], ``k``, ``v`` [NKV*D, H], ``o``
[H, NH*D], and with q/k norm ``q_norm``, ``k_norm`` [D].  q, k and v are concatenated at
load as the reference does (engine/ek_model.py:140-144).

Optional parameters, all off by default, for designs that differ there:

``bias``               which of ``"q"``, ``"k"``, ``"v"`` carry a bias (tensors ``q_bias`` ...
                       [heads * D]); it is added in 32-bit before the head norm.
``values``             ``"keys"``: there is no value projection - a token's value is its key as
                       projected (with bias, before the key's norm and rotation).
``query_temperature``  ``(coef, every)``: the query of the token at position p is multiplied by
                       1 + coef * ln(floor((p + 1) / every) + 1).
``sink``               the score of one more key without a value that every query sees: its
                       exponential is one more term of the softmax denominator (0.0: "+ 1").
``value_dim``          size of a value head when it differs from ``head_dim`` (``v`` is then [NKV * E, H]
                       and ``o`` [H, NH * E]); the cache and the kernels see heads of the larger of the
                       two sizes (rounded up to 8 values), the shorter ones padded with zeros.
``unit_norm_after_rotation``  an eps: queries and keys are rotated first and then divided by their root
                       mean square over the head (no gain), instead of the gained norm before rotation.
``keep_first``         with a window: the first ``keep_first`` positions of a sequence stay visible to every
                       later token, at their true positions.  The cache then keeps all keys.
``head_gate``          every head's output is multiplied by the sigmoid of one number per token and head,
                       a projection of the mixer's input (tensor ``gate`` [NH, H]), before ``o``.
``kv_projection``      False: the layer has no ``k`` and ``v``; it reads the keys and values another run
                       stored in the cache entry it shares (a run with ``writes_cache=False``).
``keep_all_keys``      the cache keeps every key although this layer sees a window (layers that share an
                       entry may see different windows).
Any of these sends the layer down one path: a single product for everything that reads the input,
the rotate-and-norm kernel, and the general attention kernel.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import linear, pair_product_wins, row_scale_of, tc_takes
from ..registry import lookup_part, register_part
from .base import DeferredNorm, Mixer
from .spec import CacheSpec, TensorSpec

FUSE_ROPE_ROWS = 64       # the q/k/v product does norm, rotation and cache write itself up to here
WIDE_CLUSTER_PAGES = 64     # clusters of more than 8 key splits only from this many pages of context


@register_part("mixer", "attention")
class Attention(Mixer):
    @classmethod
    def tensors(cls, spec):
        p, w = spec.params, spec.weights
        h, nh, nkv, d = p["hidden_size"], p["num_heads"], p["num_kv_heads"], p["head_dim"]
        e = int(p.get("value_dim") or d)
        out = [TensorSpec(w["q"], (nh * d, h))]
        if p.get("kv_projection", True):
            out.append(TensorSpec(w["k"], (nkv * d, h)))
            if p.get("values", "projection") != "keys":
                out.append(TensorSpec(w["v"], (nkv * e, h)))
        if p.get("head_gate"):
            out.append(TensorSpec(w["gate"], (nh, h)))
        out.append(TensorSpec(w["o"], (h, nh * e)))
        if p.get("qk_norm_eps") is not None:
            out += [TensorSpec(w["q_norm"], (d,), "gain"), TensorSpec(w["k_norm"], (d,), "gain")]
        for which in p.get("bias") or ():
            out.append(TensorSpec(w[which + "_bias"], ((nh if which == "q" else nkv) * d,)))
        return out

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.hidden = int(self.param("hidden_size"))
        self.num_heads = int(self.param("num_heads"))
        self.num_kv_heads = int(self.param("num_kv_heads"))
        self.head_dim = int(self.param("head_dim"))
        self.scale = float(self.param("scale"))
        self.qk_norm_eps = spec.params.get("qk_norm_eps")
        self.window = spec.params.get("window")
        self.biased = tuple(spec.params.get("bias") or ())
        self.values_from_keys = spec.params.get("values", "projection") == "keys"
        self.query_temperature = spec.params.get("query_temperature")
        self.sink = spec.params.get("sink")
        if spec.params.get("values", "projection") not in ("projection", "keys"):
            raise ValueError("attention: values are 'projection' or 'keys'")
        if any(b not in ("q", "k", "v") for b in self.biased) or (self.values_from_keys and "v" in self.biased):
            raise ValueError("attention: bias names q, k, v (v only with a value projection)")
        if self.query_temperature is not None and int(self.query_temperature[1]) < 1:
            raise ValueError("attention: the query temperature steps every >= 1 positions")
        self.bias = {"q": None, "k": None, "v": None}
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        kernels.check_head_dim(self.head_dim)
        self.value_dim = int(spec.params.get("value_dim") or self.head_dim)
        self.unit_norm_eps = spec.params.get("unit_norm_after_rotation")
        self.keep_first = int(spec.params.get("keep_first") or 0)
        self.head_gate = bool(spec.params.get("head_gate"))
        self.kv_projection = bool(spec.params.get("kv_projection", True))
        self.keep_all_keys = bool(spec.params.get("keep_all_keys")) or self.keep_first > 0
        self.general = (self.value_dim != self.head_dim or self.unit_norm_eps is not None or self.keep_first > 0
                        or self.head_gate or not self.kv_projection)
        #: the head size the cache and the kernels see
        self.padded_dim = self.head_dim
        if self.general:
            if not self._plain or self.qk_norm_eps is not None or self.sink is not None:
                raise ValueError("attention: value_dim, unit_norm_after_rotation, keep_first, head_gate and "
                                 "kv_projection do not combine with biases, values from keys, a query "
                                 "temperature, the gained q/k norm or a sink")
            if self.keep_first and not self.window:
                raise ValueError("attention: keep_first needs a window")
            # (a multiple of 32 where the 16-bit attention kernels can take it: at most a quarter more)
            widest = max(self.head_dim, self.value_dim)
            self.padded_dim = -(-widest // 32) * 32 if dtype == torch.bfloat16 and widest >= 64 else -(-widest // 8) * 8
            if self.padded_dim > kernels.MAX_HEAD_DIM:
                self.padded_dim = -(-widest // 8) * 8
            kernels.check_head_dim(self.padded_dim)
            # (this path takes normalised activations and returns a plain tensor)
            self.takes_deferred_norm = self.defers_norm = False
        pos = spec.params.get("position")
        self.position = lookup_part("position", pos.kind)(pos, dtype, device) if pos else None
        self.w_qkv = self.w_o = self.q_gain = self.k_gain = None

    def cache_spec(self):
        return CacheSpec("kv", heads=self.num_kv_heads, head_dim=self.padded_dim,
                         window=None if self.keep_all_keys else self.window)

    def prepare(self, max_positions):
        if self.position is not None:
            self.position.prepare(max_positions)

    def _tiles_key(self):
        return ("prefill_tc_tiles", self.num_heads // self.num_kv_heads, self.num_kv_heads * self.head_dim)

    def begin_step(self, ctx):
        """The table of tiles of the tcgen05 prompt attention, once per step and shape of the heads."""
        if self.general or ctx.is_decode or ctx.n_seqs > kernels.PREFILL_TC_MAX_SEQS or not self.scale > 0 or \
                not kernels.attention_prefill_tc_supported(self.dtype, self.head_dim, self.num_heads,
                                                           self.num_kv_heads):
            return
        key = self._tiles_key()
        if key in ctx.shared:
            return
        per_tile = kernels.PREFILL_TC_ROWS // (self.num_heads // self.num_kv_heads)
        rows = -(-ctx.n_tokens // per_tile) + ctx.n_seqs
        tiles = ctx.workspace.get(f"prefill_tc_tiles_{key[1]}_{key[2]}", (rows, 4), torch.int32)
        n = kernels.attention_prefill_tiles(tiles, ctx.n_tokens, ctx.positions, ctx.token_slot, ctx.cu_seqlens,
                                            ctx.n_seqs, self.num_heads, self.num_kv_heads, self.head_dim)
        ctx.shared[key] = (tiles, n)

    def _load_general(self, tensors):
        """[q | k | v | gate] as one weight, every head padded with zero rows to ``padded_dim``, zero rows
        up to a multiple of 64; ``o`` with zero columns where the value heads are padded."""
        w, big = self.spec.weights, self.padded_dim

        def heads(t, n, size):
            t = t.view(n, size, self.hidden)
            if size == big:
                return t.reshape(n * big, self.hidden)
            out = torch.zeros((n, big, self.hidden), dtype=t.dtype, device=t.device)
            out[:, :size] = t
            return out.view(n * big, self.hidden)

        rows = [heads(tensors[w["q"]], self.num_heads, self.head_dim)]
        if self.kv_projection:
            rows += [heads(tensors[w["k"]], self.num_kv_heads, self.head_dim),
                     heads(tensors[w["v"]], self.num_kv_heads, self.value_dim)]
        if self.head_gate:
            rows.append(tensors[w["gate"]])
        n = sum(r.shape[0] for r in rows)
        if n % 64:
            rows.append(torch.zeros((-n % 64, self.hidden), dtype=rows[0].dtype, device=rows[0].device))
        self.w_qkv = torch.cat(rows, dim=0).to(self.dtype).contiguous()
        o = tensors[w["o"]].view(self.hidden, self.num_heads, self.value_dim)
        if self.value_dim != big:
            wide = torch.zeros((self.hidden, self.num_heads, big), dtype=o.dtype, device=o.device)
            wide[:, :, :self.value_dim] = o
            o = wide
        self.w_o = o.reshape(self.hidden, self.num_heads * big).to(self.dtype).contiguous()

    def _forward_general(self, x, ctx, entry, writes_cache):
        t, big, nh, nkv = ctx.n_tokens, self.padded_dim, self.num_heads, self.num_kv_heads
        pos = self.position
        rows = linear(x, self.w_qkv, ctx, "qkv", n_rows=t)
        k_col = nh * big
        gate_col = k_col + (2 * nkv * big if self.kv_projection else 0)
        kernels.qk_rope_unit_kv(
            rows, t, k_col, k_col + nkv * big, pos.cos if pos else _no_table(self.device),
            pos.sin if pos else _no_table(self.device), pos.rotary_dim if pos else 0, ctx.positions,
            ctx.token_slot, entry.k_pages, entry.v_pages, entry.block_table, nh, nkv, big, self.head_dim,
            self.unit_norm_eps or 0.0, unit=self.unit_norm_eps is not None,
            write_kv=writes_cache and self.kv_projection)
        out = ctx.workspace.get("attn_out", (t, nh * big), self.dtype)
        visible = min(ctx.max_context, self.window + self.keep_first) if self.window else ctx.max_context
        gate = rows[:, gate_col:] if self.head_gate else None
        if not ctx.is_decode and kernels.attention_prefill_supported(self.dtype, big, nh, nkv):
            kernels.attention_prefill_bf16(out, rows, t, ctx.positions, ctx.token_slot, ctx.cu_seqlens, ctx.n_seqs,
                                           entry.k_pages, entry.v_pages, entry.block_table, nh, nkv, big, self.scale,
                                           self.window, keep_first=self.keep_first, gate=gate)
            return linear(out, self.w_o, ctx, "attn_proj", n_rows=t)
        if ctx.is_decode and kernels.attention_decode_supported(self.dtype, big):
            # blocks = tokens x KV heads (x 16-row blocks of the group), three fit an SM: every token's own
            # window is cut so that the blocks about fill the machine, never finer than two pages a split
            blocks = t * nkv * -(-(nh // nkv) // 16)
            splits = max(1, min(3 * kernels.sm_count(self.device) // blocks, -(-visible // 128)))
            acc = ml = None
            if splits > 1:
                acc = ctx.workspace.get("attn_part_acc", (t, nh, splits, big), torch.float32)
                ml = ctx.workspace.get("attn_part_ml", (t, nh, splits, 2), torch.float32)
            kernels.attention_decode_bf16(out, rows, t, ctx.positions, ctx.token_slot, entry.k_pages, entry.v_pages,
                                          entry.block_table, nh, nkv, big, self.scale, self.window, splits, 0, acc, ml,
                                          keep_first=self.keep_first, gate=gate)
            return linear(out, self.w_o, ctx, "attn_proj", n_rows=t)
        splits, per_split, acc, ml = 1, 0, None, None
        blocks = t * nh
        if blocks < 2 * kernels.sm_count(self.device) and visible > 512:
            splits = max(1, min(-(-visible // 256), -(-4 * kernels.sm_count(self.device) // blocks), 64))
        if splits > 1:
            per_split = -(-(-(-ctx.max_context // splits)) // 128) * 128
            splits = -(-ctx.max_context // per_split)
        if splits > 1:
            acc = ctx.workspace.get("attn_part_acc", (t, nh, splits, big), torch.float32)
            ml = ctx.workspace.get("attn_part_ml", (t, nh, splits, 2), torch.float32)
        kernels.attention_generic(out, rows, t, ctx.positions, ctx.token_slot, entry.k_pages, entry.v_pages,
                                  entry.block_table, nh, nkv, big, self.scale, self.window, splits, per_split,
                                  acc, ml, keep_first=self.keep_first, gate=gate)
        return linear(out, self.w_o, ctx, "attn_proj", n_rows=t)

    def load(self, tensors):
        if self.general:
            return self._load_general(tensors)
        w = self.spec.weights
        rows = [tensors[w["q"]], tensors[w["k"]]] + ([] if self.values_from_keys else [tensors[w["v"]]])
        self.w_qkv = torch.cat(rows, dim=0).to(self.dtype).contiguous()
        for which in self.biased:
            self.bias[which] = tensors[w[which + "_bias"]].to(torch.float32).contiguous()
        self.w_o = tensors[w["o"]].to(self.dtype).contiguous()
        if self.qk_norm_eps is not None:
            self.q_gain = tensors[w["q_norm"]].to(torch.float32).contiguous()
            self.k_gain = tensors[w["k_norm"]].to(torch.float32).contiguous()

    def bytes_read_per_step(self, n_tokens):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o, self.q_gain, self.k_gain,
                                                          *self.bias.values()) if t is not None)

    # ------------------------------------------------------------------
    takes_deferred_norm = True
    defers_norm = True

    def forward(self, x, ctx, entry, writes_cache=True, defer=None):
        t = ctx.n_tokens
        pos = self.position
        if self.general:
            if isinstance(x, DeferredNorm):
                raise kernels.KernelError("this attention layer takes normalised activations, not a deferred norm")
            return self._forward_general(x, ctx, entry, writes_cache)
        if self._fuses_rope(x, ctx):
            # few rows, heads of 128: norm, rotation and cache write ride on the product's epilogue
            row_scale, xin = (row_scale_of(x), x.scaled) if isinstance(x, DeferredNorm) else (None, x)
            qkv = ctx.workspace.get("qkv", (t, self.w_qkv.shape[0]), self.dtype)
            kernels.gemm_tc_qkv_rope(
                qkv, xin, self.w_qkv, t, self.q_gain, self.k_gain,
                self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, pos.cos, pos.sin,
                ctx.positions, ctx.token_slot, entry.k_pages, entry.v_pages, entry.block_table,
                self.num_heads, self.num_kv_heads, write_kv=writes_cache, row_scale=row_scale)
            out = ctx.workspace.get("attn_out", (t, self.num_heads * self.head_dim), self.dtype)
            self._attend(out, qkv, ctx, entry)
            return linear(out, self.w_o, ctx, "attn_proj", n_rows=t, defer=defer, image=self.product_image())
        if self._fuses_prepare(x, ctx):
            # the same for designs with biases, a query temperature, values taken from the keys,
            # or no rotation at all
            row_scale, xin = (row_scale_of(x), x.scaled) if isinstance(x, DeferredNorm) else (None, x)
            qkv = ctx.workspace.get("qkv", (t, self.w_qkv.shape[0]), self.dtype)
            kernels.gemm_tc_qkv_prepare(
                qkv, xin, self.w_qkv, t, self.q_gain, self.k_gain,
                self.qk_norm_eps if self.qk_norm_eps is not None else 0.0,
                pos.cos if pos else None, pos.sin if pos else None,
                ctx.positions, ctx.token_slot, entry.k_pages, entry.v_pages, entry.block_table,
                self.num_heads, self.num_kv_heads, write_kv=writes_cache, row_scale=row_scale,
                q_bias=self.bias["q"], k_bias=self.bias["k"], v_bias=self.bias["v"],
                q_temperature=self.query_temperature, values_from_keys=self.values_from_keys)
            out = ctx.workspace.get("attn_out", (t, self.num_heads * self.head_dim), self.dtype)
            self._attend(out, qkv, ctx, entry)
            return linear(out, self.w_o, ctx, "attn_proj", n_rows=t, defer=defer, image=self.product_image())
        if self._fuses_rope_of_many_rows(x, ctx):
            # many rows, heads of 128: the same on the epilogue of the product on pairs of SMs
            qkv = ctx.workspace.get("qkv", (t, self.w_qkv.shape[0]), self.dtype)
            kernels.gemm_pair_qkv_rope(
                qkv, x, self.w_qkv, t, self.q_gain, self.k_gain,
                self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, pos.cos, pos.sin,
                ctx.positions, ctx.token_slot, entry.k_pages, entry.v_pages, entry.block_table,
                self.num_heads, self.num_kv_heads, write_kv=writes_cache)
            out = ctx.workspace.get("attn_out", (t, self.num_heads * self.head_dim), self.dtype)
            self._attend(out, qkv, ctx, entry)
            return linear(out, self.w_o, ctx, "attn_proj", n_rows=t, defer=defer, image=self.product_image())
        qkv = linear(x, self.w_qkv, ctx, "qkv", n_rows=t)
        prepare = (qkv, t, self.q_gain, self.k_gain,
                   pos.cos if pos else _no_table(self.device), pos.sin if pos else _no_table(self.device),
                   pos.rotary_dim if pos else 0, ctx.positions, ctx.token_slot, entry.k_pages,
                   entry.v_pages, entry.block_table, self.num_heads, self.num_kv_heads, self.head_dim,
                   self.qk_norm_eps if self.qk_norm_eps is not None else 0.0)
        if self._plain:
            kernels.qk_norm_rope_kv(*prepare, write_kv=writes_cache)
        else:
            kernels.qk_prepare_kv(*prepare, write_kv=writes_cache, q_bias=self.bias["q"],
                                  k_bias=self.bias["k"], v_bias=self.bias["v"],
                                  q_temperature=self.query_temperature,
                                  values_from_keys=self.values_from_keys)
        out = ctx.workspace.get("attn_out", (t, self.num_heads * self.head_dim), self.dtype)
        self._attend(out, qkv, ctx, entry)
        return linear(out, self.w_o, ctx, "attn_proj", n_rows=t, defer=defer, image=self.product_image())

    @property
    def _plain(self):
        """None of the optional parameters that change what happens between the projection and
        the cache is on (the sink only changes the softmax)."""
        return not self.biased and not self.values_from_keys and self.query_temperature is None

    def _fuses_rope(self, x, ctx):
        xin = x.scaled if isinstance(x, DeferredNorm) else x
        pos = self.position
        return (self._plain and self.dtype == torch.bfloat16 and ctx.n_tokens <= FUSE_ROPE_ROWS
                and self.head_dim == kernels.QKV_ROPE_HEAD_DIM and pos is not None
                and getattr(pos, "rotary_dim", 0) == self.head_dim and tc_takes(xin, self.w_qkv))

    def product_image(self):
        """``"extended"`` when this layer's q/k/v product of few rows runs the extended epilogue."""
        pos = self.position
        if ((not self._plain or pos is None) and self.dtype == torch.bfloat16
                and self.head_dim == kernels.QKV_ROPE_HEAD_DIM
                and (pos is None or getattr(pos, "rotary_dim", 0) == self.head_dim)):
            return "extended"
        return None

    def _fuses_prepare(self, x, ctx):
        xin = x.scaled if isinstance(x, DeferredNorm) else x
        return (self.product_image() == "extended" and ctx.n_tokens <= FUSE_ROPE_ROWS
                and tc_takes(xin, self.w_qkv))

    def _fuses_rope_of_many_rows(self, x, ctx):
        pos = self.position
        if (not self._plain or isinstance(x, DeferredNorm) or self.dtype != torch.bfloat16
                or self.head_dim != kernels.QKV_ROPE_HEAD_DIM or pos is None
                or getattr(pos, "rotary_dim", 0) != self.head_dim):
            return False
        qkv = ctx.workspace.get("qkv", (ctx.n_tokens, self.w_qkv.shape[0]), self.dtype)
        return pair_product_wins(qkv, x, self.w_qkv, ctx.n_tokens, kernels.PAIR_EPI_BF16)

    def _attend(self, out, qkv, ctx, entry):
        t = ctx.n_tokens
        visible = min(ctx.max_context, self.window) if self.window else ctx.max_context
        fast_decode = ctx.is_decode and kernels.attention_decode_supported(self.dtype, self.head_dim)
        if not ctx.is_decode and kernels.attention_prefill_supported(
                self.dtype, self.head_dim, self.num_heads, self.num_kv_heads):
            prefill = kernels.attention_prefill_bf16
            if ctx.n_seqs <= kernels.PREFILL_TC_MAX_SEQS and self.scale > 0 and \
                    kernels.attention_prefill_tc_supported(self.dtype, self.head_dim, self.num_heads,
                                                           self.num_kv_heads):
                prefill = kernels.attention_prefill_tc      # tcgen05: head sizes 64 and 128
            extra = {}
            if prefill is kernels.attention_prefill_tc:
                made = ctx.shared.get(self._tiles_key())
                if made is not None:                 # (made in begin_step; a part driven alone has none)
                    extra = dict(tiles=made[0], n_tiles=made[1])
            prefill(
                out, qkv, t, ctx.positions, ctx.token_slot, ctx.cu_seqlens, ctx.n_seqs,
                entry.k_pages, entry.v_pages, entry.block_table, self.num_heads, self.num_kv_heads,
                self.head_dim, self.scale, self.window, sink=self.sink, **extra)
            return
        if ctx.is_decode and t <= 65535 and kernels.attention_decode_tma_supported(
                self.dtype, self.head_dim, self.num_heads, self.num_kv_heads):
            # blocks = tokens x KV heads x splits, two fit an SM; a split takes whole pages and the
            # splits of a token are one cluster
            blocks = t * self.num_kv_heads
            pages = -(-visible // kernels.PAGE)
            # (more than 8 blocks a token only pay with many pages each: long contexts, few sequences)
            limit = kernels.decode_tma_max_splits(self.head_dim, self.device) if pages >= WIDE_CLUSTER_PAGES else \
                kernels.DECODE_TMA_PORTABLE_SPLITS
            splits = max(1, min(2 * kernels.sm_count(self.device) // blocks, pages, limit))
            splits = 1 << (splits.bit_length() - 1)      # clusters of 3, 5, 6, 7 pack the GPCs badly
            kernels.attention_decode_tma(
                out, qkv, t, ctx.positions, ctx.token_slot, entry.k_pages, entry.v_pages,
                entry.block_table, self.num_heads, self.num_kv_heads, self.head_dim, self.scale,
                self.window, splits, sink=self.sink)
            return
        if fast_decode:
            # blocks = tokens x KV heads (x 16-row blocks of the group); three fit an SM.  Split
            # the keys so that the blocks just fill the machine once, or about twice when one
            # filling cannot be approached; never finer than two pages a split.
            blocks = t * self.num_kv_heads * -(-(self.num_heads // self.num_kv_heads) // 16)
            resident = 3 * kernels.sm_count(self.device)
            splits = resident // blocks
            if blocks * splits < 0.7 * resident:
                splits = int(1.8 * resident / blocks + 0.5)
            splits = max(1, min(splits, -(-visible // 128)))
            unit = 64
        else:
            blocks = t * self.num_heads
            splits = 1
            if blocks < 2 * kernels.sm_count(self.device) and ctx.max_context > 512:
                splits = max(1, min(-(-visible // 256), -(-4 * kernels.sm_count(self.device) // blocks), 64))
            unit = 128
        per_split, acc, ml = 0, None, None
        if splits > 1 and not fast_decode:      # the decode kernel cuts each token's own range
            per_split = -(-(-(-ctx.max_context // splits)) // unit) * unit
            splits = -(-ctx.max_context // per_split)
        if splits > 1:
            acc = ctx.workspace.get("attn_part_acc", (t, self.num_heads, splits, self.head_dim),
                                    torch.float32)
            ml = ctx.workspace.get("attn_part_ml", (t, self.num_heads, splits, 2), torch.float32)
        args = (out, qkv, t, ctx.positions, ctx.token_slot, entry.k_pages, entry.v_pages,
                entry.block_table, self.num_heads, self.num_kv_heads, self.head_dim, self.scale,
                self.window, splits, per_split, acc, ml)
        fn = kernels.attention_decode_bf16 if fast_decode else kernels.attention_generic
        fn(*args, sink=self.sink)


_EMPTY = {}


def _no_table(device):
    key = str(device)
    if key not in _EMPTY:
        _EMPTY[key] = torch.zeros((1, 0), dtype=torch.float32, device=device)
    return _EMPTY[key]
