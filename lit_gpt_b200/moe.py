"""Sparse mixtures of experts.

``GroupLimitedRouter``: scores s = sigmoid(W x) in fp32.  Experts are CHOSEN by s + correction (a per-expert selection bias
that does not enter the output), among the experts of the ``keep`` best of ``groups`` equal groups of neighbouring experts --
a group is ranked by the sum of its two largest corrected scores -- and the chosen experts are WEIGHTED by s itself, without
renormalisation.  ``SparseExperts``: out = sum_k weight_k * W_down[e_k] relu(W_up[e_k] x)^2 over stacked expert weights, as a
grouped matrix product for many tokens (the vendor's grouped GEMM for bf16, this library's any-size fp32-accumulating kernel
otherwise) and as weight-streaming GEMVs for a few (``K.moe_experts``).

``GroupLimitedRouter(softmax=True, group_max=True)`` scores with a softmax over all experts and ranks a group by its largest
score; ``GatedSparseExperts`` uses it with gated experts, out = sum_k s_k * W_down[e_k] (silu(W_gate[e_k] x) * (W_up[e_k] x)), gate
and up rows stacked into one (experts, 2 ff, width) tensor so that both are one (grouped) product.

``ClampedSparseExperts``: the router adds a bias to its logits, takes the `top` largest and weights them by a softmax among
those few; experts are gated with clamped branches, W_down (g sigmoid(alpha g) (u + 1)), g = min(W_gate x, limit), u = clamp(W_up x,
-limit, limit); ``ClampedGLU`` is one such expert for every token (a shared expert).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import kernels as K
from .config import ClampedMoESpec, GatedMoESpec, MoESpec


VENDOR_GROUPED_GEMM = True   # tests switch it off to run the library's own grouped kernel on the same input


class GroupLimitedRouter(nn.Module):
    def __init__(self, width: int, experts: int, top: int, groups: int = 1, keep: int = 1, *, softmax: bool = False, group_max: bool = False,
                 correction: bool = True, topk_softmax: bool = False, bias: bool = False) -> None:
        """topk_softmax: raw logits choose, weights = softmax among those few; bias: `correction` is a bias inside the logit."""
        super().__init__()
        self.top, self.groups, self.keep, self.softmax, self.group_max = top, groups, keep, softmax, group_max
        self.topk_softmax, self.bias = topk_softmax, bias
        self.weight = nn.Parameter(torch.empty(experts, width), requires_grad=False)
        self.correction = nn.Parameter(torch.zeros(experts), requires_grad=False) if correction else None

    def forward(self, x: torch.Tensor):
        """x (n, width) -> (expert ids int32 (n, top), weights fp32 (n, top))"""
        return K.moe_route(x, self.weight, self.correction, self.top, self.groups, self.keep, softmax=self.softmax, group_max=self.group_max,
                           topk_softmax=self.topk_softmax, bias=self.bias)


class SparseExperts(nn.Module):
    def __init__(self, width: int, spec: MoESpec) -> None:
        super().__init__()
        self.spec = spec
        self.router = GroupLimitedRouter(width, spec.experts, spec.top, spec.groups, spec.keep)
        self.w_up = nn.Parameter(torch.empty(spec.experts, spec.ff, width), requires_grad=False)
        self.w_down = nn.Parameter(torch.empty(spec.experts, width, spec.ff), requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ids, weights = self.router(x)
        n, d = x.shape
        if (n * self.spec.top <= K.MOE_GEMV_MAX_PAIRS or x.dtype != torch.bfloat16 or d % 8 or self.spec.ff % 8
                or not VENDOR_GROUPED_GEMM or not hasattr(torch, "_grouped_mm")):
            return K.moe_experts(x, ids, weights, self.w_up, self.w_down)   # this library's kernels only (always so in fp32)
        # many bf16 tokens: the two products go to the vendor's grouped GEMM (as the dense products go to its GEMM), over the
        # rows this library sorted by expert on the device -- no host round trip for the per-expert counts
        plan = K.moe_plan(ids, self.spec.experts)
        ends = plan.expert_off[1:]
        hidden = torch._grouped_mm(K.gather_rows(x, plan.slot_token), self.w_up.transpose(1, 2), offs=ends)
        y = torch._grouped_mm(K.sqrelu_(hidden), self.w_down.transpose(1, 2), offs=ends)
        return K.moe_combine(y, plan, weights)


class GatedSparseExperts(nn.Module):
    def __init__(self, width: int, spec: GatedMoESpec) -> None:
        super().__init__()
        self.spec = spec
        self.router = GroupLimitedRouter(width, spec.experts, spec.top, spec.groups, spec.keep, softmax=True, group_max=True, correction=False)
        self.w_up = nn.Parameter(torch.empty(spec.experts, 2 * spec.ff, width), requires_grad=False)   # per expert: ff gate rows, then ff up rows
        self.w_down = nn.Parameter(torch.empty(spec.experts, width, spec.ff), requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ids, weights = self.router(x)
        n, d = x.shape
        if (n * self.spec.top <= K.MOE_GEMV_MAX_PAIRS or x.dtype != torch.bfloat16 or d % 8 or self.spec.ff % 8
                or not VENDOR_GROUPED_GEMM or not hasattr(torch, "_grouped_mm")):
            return K.moe_experts(x, ids, weights, self.w_up, self.w_down, gated=True)
        plan = K.moe_plan(ids, self.spec.experts)
        ends = plan.expert_off[1:]
        both = torch._grouped_mm(K.gather_rows(x, plan.slot_token), self.w_up.transpose(1, 2), offs=ends)
        y = torch._grouped_mm(K.glu(both, K.ACT_SILU), self.w_down.transpose(1, 2), offs=ends)
        return K.moe_combine(y, plan, weights)


class ClampedGLU(nn.Module):
    """W_down (g sigmoid(alpha g) (u + 1)) with g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit); gate and up rows stacked."""

    def __init__(self, width: int, ff: int, limit: float, alpha: float) -> None:
        super().__init__()
        self.limit, self.alpha = limit, alpha
        self.w_up = nn.Parameter(torch.empty(2 * ff, width), requires_grad=False)   # ff gate rows, then ff up rows
        self.w_down = nn.Parameter(torch.empty(width, ff), requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.linear(K.glu_clamped(torch.nn.functional.linear(x, self.w_up), self.limit, self.alpha), self.w_down)


class ClampedSparseExperts(nn.Module):
    def __init__(self, width: int, spec: ClampedMoESpec) -> None:
        super().__init__()
        self.spec = spec
        self.router = GroupLimitedRouter(width, spec.experts, spec.top, softmax=False, topk_softmax=True, bias=True)
        self.w_up = nn.Parameter(torch.empty(spec.experts, 2 * spec.ff, width), requires_grad=False)   # per expert: ff gate rows, then ff up rows
        self.w_down = nn.Parameter(torch.empty(spec.experts, width, spec.ff), requires_grad=False)
        self.shared = ClampedGLU(width, spec.shared_ff, spec.shared_limit, spec.alpha) if spec.shared_ff else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """The routed experts' weighted sum; the shared expert is the caller's to add (``self.shared(x)``)."""
        ids, weights = self.router(x)
        n, d = x.shape
        sp = self.spec
        if (n * sp.top <= K.MOE_GEMV_MAX_PAIRS or x.dtype != torch.bfloat16 or d % 8 or sp.ff % 8
                or not VENDOR_GROUPED_GEMM or not hasattr(torch, "_grouped_mm")):
            return K.moe_experts(x, ids, weights, self.w_up, self.w_down, gated=True, limit=sp.limit, alpha=sp.alpha)
        plan = K.moe_plan(ids, sp.experts)
        ends = plan.expert_off[1:]
        both = torch._grouped_mm(K.gather_rows(x, plan.slot_token), self.w_up.transpose(1, 2), offs=ends)
        y = torch._grouped_mm(K.glu_clamped(both, sp.limit, sp.alpha), self.w_down.transpose(1, 2), offs=ends)
        return K.moe_combine(y, plan, weights)


class DenseMLP(nn.Module):
    """W_down act(W_up x), act = the exact (erf) gelu unless another of ``K.ACT_*`` is named, or xIELU with its two learned numbers
    (``xielu=True``); the products are vendor GEMMs, the activation this library's kernel."""

    def __init__(self, width: int, ff: int, activation: int = K.ACT_GELU, xielu: bool = False) -> None:
        super().__init__()
        self.activation = activation
        self.w_up = nn.Parameter(torch.empty(ff, width), requires_grad=False)
        self.w_down = nn.Parameter(torch.empty(width, ff), requires_grad=False)
        self.act = nn.Parameter(torch.zeros(2), requires_grad=False) if xielu else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        hidden = torch.nn.functional.linear(x, self.w_up)
        hidden = K.xielu_(hidden, self.act) if self.act is not None else K.activation_(hidden, self.activation)
        return torch.nn.functional.linear(hidden, self.w_down)
