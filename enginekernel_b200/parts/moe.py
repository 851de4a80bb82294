"""Routed experts: every token goes through ``top`` of E small feed-forwards.

    z = W_router h (32-bit);   s = softmax(z) over all experts
    experts form ``groups`` equal groups of neighbours; a group's score is its best expert's; only
    experts of the ``keep`` best groups can be chosen; the ``top`` largest scores among those are;
    weight = chosen score / (sum of the chosen scores + 1e-20) * ``scale``
    out = sum over the chosen experts of weight * W_down,e act(W_up,e h)

With ``weights="softmax_of_chosen"`` the ``top`` largest logits (of the kept groups) are chosen and the
weights are the softmax over those chosen logits alone, times ``scale``.  With ``gated`` an expert is
W_down,e (act(W_gate,e h) * (W_up,e h)) (tensors ``gate_<e>`` [I, hidden] beside ``up_<e>``; gate and up rows
are interleaved at load, so that one product gives both and its epilogue their 32-bit product).

Experts have no biases; ``activation`` is ``"relu2"`` (the square of relu), ``"silu"``,
``"gelu_tanh"`` or ``"none"``.  The choice is made and used on the device: a kernel sorts the (token,
choice) pairs by expert and cuts every expert's stretch into row tiles, and the two expert products
walk those tiles, so nothing here waits for the device and the step can be captured in a graph.

Parameters: ``hidden_size``, ``intermediate_size`` (of one expert), ``experts``, ``top``, ``groups``
(default 1), ``keep`` (default: all groups), ``scale``, ``activation``, ``gated`` (default False), ``weights``
(``"scores_of_chosen"``, the default, or ``"softmax_of_chosen"``).  Tensors: ``router`` [E, hidden]
and per expert ``up_<e>`` [I, hidden], ``down_<e>`` [hidden, I].
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import linear
from ..registry import register_part
from .base import FeedForward
from .spec import TensorSpec


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    @classmethod
    def tensors(cls, spec):
        p, w = spec.params, spec.weights
        h, i, n = p["hidden_size"], p["intermediate_size"], p["experts"]
        out = [TensorSpec(w["router"], (n, h))]
        for e in range(n):
            if p.get("gated"):
                out.append(TensorSpec(w[f"gate_{e}"], (i, h)))
            out += [TensorSpec(w[f"up_{e}"], (i, h)), TensorSpec(w[f"down_{e}"], (h, i))]
        return out

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        g = lambda n: int(self.param(n))
        self.hidden, self.inter, self.experts, self.top = g("hidden_size"), g("intermediate_size"), g("experts"), g("top")
        self.groups = int(spec.params.get("groups") or 1)
        self.keep = int(spec.params.get("keep") or self.groups)
        self.scale = float(spec.params.get("scale", 1.0))
        self.activation = spec.params.get("activation", "relu2")
        self.gated = bool(spec.params.get("gated"))
        self.weights = spec.params.get("weights", "scores_of_chosen")
        if self.weights not in ("scores_of_chosen", "softmax_of_chosen"):
            raise ValueError(f"routed_experts has no weights {self.weights!r}")
        if self.activation not in kernels.EXPERT_ACTIVATIONS:
            raise ValueError(f"routed_experts has no activation {self.activation!r}")
        if self.experts % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError("routed_experts: groups must divide experts, 1 <= keep <= groups")
        if not 1 <= self.top <= self.keep * (self.experts // self.groups):
            raise ValueError("routed_experts: top exceeds the experts of the kept groups")
        self.w_router = self.w_up = self.w_down = None

    def load(self, tensors):
        w = self.spec.weights
        self.w_router = tensors[w["router"]].to(self.dtype).contiguous()
        ups = [tensors[w[f"up_{e}"]] for e in range(self.experts)]
        if self.gated:               # rows gate_0, up_0, gate_1, up_1, ... of every expert
            ups = [torch.stack([tensors[w[f"gate_{e}"]], up], 1).reshape(2 * self.inter, self.hidden)
                   for e, up in enumerate(ups)]
        self.w_up = torch.stack(ups).to(self.dtype).contiguous()
        self.w_down = torch.stack([tensors[w[f"down_{e}"]] for e in range(self.experts)]).to(self.dtype).contiguous()

    def bytes_read_per_step(self, n_tokens):
        """The router and the experts that ``n_tokens`` tokens can reach at most."""
        touched = min(self.experts, n_tokens * self.top)
        per_expert = (self.w_up[0].numel() + self.w_down[0].numel()) * self.w_up.element_size()
        return self.w_router.numel() * self.w_router.element_size() + touched * per_expert

    def forward(self, x, ctx):
        t, ws, top = ctx.n_tokens, ctx.workspace, self.top
        pairs = t * top
        logits = linear(x, self.w_router, ctx, "router_logits", n_rows=t, out_dtype=torch.float32, wide_f32="library")
        chosen = ws.get("moe_chosen", (t, top), torch.int32)
        weight = ws.get("moe_weight", (t, top), torch.float32)
        kernels.moe_route(chosen, weight, logits, t, self.groups, self.keep, top, self.scale,
                          among_chosen=self.weights == "softmax_of_chosen")
        sorted_pair = ws.get("moe_sorted", (pairs,), torch.int32)
        tiles = ws.get("moe_tiles", (kernels.moe_max_tiles(pairs, self.experts), 3), torch.int32)
        n_tiles = ws.get("moe_n_tiles", (1,), torch.int32)
        kernels.moe_plan(sorted_pair, tiles, n_tiles, chosen, pairs, self.experts)
        act = ws.get("moe_act", (pairs, self.inter), self.dtype)
        kernels.moe_expert_up(act, x, self.w_up, tiles, n_tiles, sorted_pair, pairs, top, self.activation,
                              gated=self.gated)
        pair_out = ws.get("moe_pair_out", (pairs, self.hidden), torch.float32)
        kernels.moe_expert_down(pair_out, act, self.w_down, tiles, n_tiles, sorted_pair, weight, pairs)
        out = ws.get("mlp_down", (t, self.hidden), self.dtype)
        kernels.moe_combine(out, pair_out, t, top)
        return out
