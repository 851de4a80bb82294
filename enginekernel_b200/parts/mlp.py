"""Gated feed-forward: down(act(gate(x)) * up(x)), no biases; act is SiLU (SwiGLU) or the
tanh form of GELU, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).

engine/ek_model.py:205-209 with engine/ek_kernels.py:125-143; gate and up are
concatenated at load (gate rows first, engine/ek_model.py:145-147).  Parameters:
``hidden_size``, ``intermediate_size``, ``activation`` ("silu", the default, or "gelu_tanh").  Tensors: ``gate``,
``up`` [I, H], ``down`` [H, I].
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import linear, pair_product_wins, row_scale_of, tc_takes
from ..registry import register_part
from .base import DeferredNorm, FeedForward
from .spec import TensorSpec


@register_part("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    @classmethod
    def tensors(cls, spec):
        p, w = spec.params, spec.weights
        h, i = p["hidden_size"], p["intermediate_size"]
        return [TensorSpec(w["gate"], (i, h)), TensorSpec(w["up"], (i, h)),
                TensorSpec(w["down"], (h, i))]

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        self.activation = spec.params.get("activation", "silu")
        if self.activation not in kernels.GATE_ACTIVATIONS:
            raise ValueError(f"gated_mlp has no activation {self.activation!r} "
                             f"({', '.join(kernels.GATE_ACTIVATIONS)})")
        self.w_gate_up = self.w_down = None

    def load(self, tensors):
        w = self.spec.weights
        self.w_gate_up = torch.cat([tensors[w["gate"]], tensors[w["up"]]], dim=0) \
            .to(self.dtype).contiguous()
        self.w_down = tensors[w["down"]].to(self.dtype).contiguous()

    def bytes_read_per_step(self, n_tokens):
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    takes_deferred_norm = True
    defers_norm = True

    def forward(self, x, ctx, defer=None):
        t = ctx.n_tokens
        row_scale = None
        if isinstance(x, DeferredNorm):
            row_scale, x = row_scale_of(x), x.scaled
        if self.dtype == torch.bfloat16 and t <= kernels.TC_SWAP_MAX_ROWS and tc_takes(x, self.w_gate_up):
            # gate and up rows share a tile, so act(gate) * up is formed in the epilogue
            act = ctx.workspace.get("mlp_act", (t, self.inter), self.dtype)
            kernels.gemm_tc_bf16(act, x, self.w_gate_up, kernels.GATED_EPILOGUES[self.activation], n_rows=t,
                                 swap=True, row_scale=row_scale)
        elif row_scale is not None:
            raise kernels.KernelError("a deferred norm reached a product that cannot scale its rows")
        elif self.dtype == torch.bfloat16 and pair_product_wins(
                ctx.workspace.get("mlp_act", (t, self.inter), self.dtype), x, self.w_gate_up, t,
                kernels.PAIR_GATED_EPILOGUES[self.activation]):
            # many rows: the pair of blocks that shares a tile stages gate rows in one block and the
            # matching up rows in the other, and the epilogue forms act(gate) * up from the 32-bit sums
            act = ctx.workspace.get("mlp_act", (t, self.inter), self.dtype)
            kernels.gemm_pair_bf16(act, x, self.w_gate_up, kernels.PAIR_GATED_EPILOGUES[self.activation],
                                   n_rows=t)
        else:
            gu = linear(x, self.w_gate_up, ctx, "mlp_gate_up", n_rows=t)
            act = ctx.workspace.get("mlp_act", (t, self.inter), self.dtype)
            kernels.act_mul(act, gu, self.activation, n_rows=t)
        return linear(act, self.w_down, ctx, "mlp_down", n_rows=t, defer=defer, image=self.product_image)


@register_part("feed_forward", "dense_mlp")
class DenseMLP(FeedForward):
    """Feed-forward without a gate: down(act(up(x) + b_up)) + b_down; act is the tanh form of GELU or SiLU.
    Parameters: ``hidden_size``, ``intermediate_size``, ``activation`` ("gelu_tanh", the default, or "silu"),
    ``bias`` (True: both products have one).  Tensors: ``up`` [I, H], ``down`` [H, I], and with biases
    ``up_bias`` [I], ``down_bias`` [H].  The first bias and the activation are one pass over the up
    product's rows; the last bias is added here, or - ``forward(..., leave_bias=True)`` - left to the
    consumer as ``output_bias`` (a block whose norm kernel reads the result anyway)."""

    @classmethod
    def tensors(cls, spec):
        p, w = spec.params, spec.weights
        h, i = p["hidden_size"], p["intermediate_size"]
        out = [TensorSpec(w["up"], (i, h)), TensorSpec(w["down"], (h, i))]
        if p.get("bias"):
            out += [TensorSpec(w["up_bias"], (i,)), TensorSpec(w["down_bias"], (h,))]
        return out

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        self.activation = spec.params.get("activation", "gelu_tanh")
        if self.activation not in ("gelu_tanh", "silu"):
            raise ValueError(f"dense_mlp has no activation {self.activation!r} (gelu_tanh, silu)")
        self.biased = bool(spec.params.get("bias"))
        self.w_up = self.w_down = self.up_bias = self.output_bias = None

    def load(self, tensors):
        w = self.spec.weights
        self.w_up = tensors[w["up"]].to(self.dtype).contiguous()
        self.w_down = tensors[w["down"]].to(self.dtype).contiguous()
        if self.biased:
            self.up_bias = tensors[w["up_bias"]].to(torch.float32).contiguous()
            self.output_bias = tensors[w["down_bias"]].to(torch.float32).contiguous()

    def forward(self, x, ctx, leave_bias=False):
        t = ctx.n_tokens
        up = linear(x, self.w_up, ctx, "mlp_up", n_rows=t)
        act = ctx.workspace.get("mlp_act", (t, self.inter), self.dtype)
        kernels.bias_act(act, up, self.up_bias, self.activation, n_rows=t)
        down = linear(act, self.w_down, ctx, "mlp_down", n_rows=t)
        if self.output_bias is not None and not leave_bias:
            out = ctx.workspace.get("mlp_down_biased", (t, self.hidden), self.dtype)
            kernels.bias_act(out, down, self.output_bias, None, n_rows=t)
            return out
        return down
