"""A feed-forward of routed experts: each token runs `top` of `n_experts` small feed-forwards (gated, or
down(relu(up x)^2) without a gate; the router may add a correction to the scores for the choice only, restrict the choice
to the best groups of experts, and scale the weights: parts/spec.py: RoutedFeedForwardSpec).

  z = W_router h (32-bit sums), s = sigmoid(z) or softmax(z); the `top` largest scores choose the experts
  w_j = s[e_j], or s[e_j] / sum_j s[e_j] with `renormalize`
  expert(x) = W_down (g * sigmoid(act_alpha g) * (u + up_shift)),  g = min(W_gate x, gate_limit),
              u = clamp(W_up x, -up_limit, up_limit)
  result = sum_j expert_{e_j}(w_j h)  (weight_on_input)   or   sum_j w_j expert_{e_j}(h)

The experts' matrices are kept stacked, [E, 2 ff, hidden] (gate rows, then up rows) and [E, hidden, ff], in the type
they are stored in.  A step routes on the device (no read on the host: the part is graph-safe) and then takes one of
two forms: in a 16-bit engine the (token, expert) pairs are sorted by expert and run as grouped products on the tensor
cores (csrc/moe_grouped.cu, csrc/gemm_tc.cu); the 32-bit engine, and sizes the tensor-core product refuses, stream the
chosen experts' matrices through the multiply-add units (csrc/moe.cu).
"""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import FeedForward, to_device, weight_to_device
from .registry import register_feed_forward
from .spec import RoutedFeedForwardSpec


class RoutedExperts(FeedForward):
    graph_safe = True
    can_overwrite = True
    libraries = ("moe", "moe_grouped", "gemm_tc")
    # Rows from which the grouped tensor-core form runs in a 16-bit engine.  Measured at width 2048 (8 experts of inner
    # width 2816, 2 a token): a decode step of 1 / 8 / 32 requests takes 0.48 / 0.75 / 1.03 ms with it and 0.52 / 1.10 /
    # 2.54 ms with the kernels that stream the matrices through the multiply-add units, so it always runs.
    GROUPED_FROM = 1

    def __init__(self, spec: RoutedFeedForwardSpec):
        s = self.spec = spec
        if not (1 <= s.top <= s.n_experts) or len(s.experts) != s.n_experts:
            raise ValueError(f"{s.top} of {s.n_experts} experts ({len(s.experts)} listed) is not a choice")
        if s.top > 16 or s.n_experts > 1024:
            raise ValueError("the routing kernel takes up to 16 chosen of up to 1024 experts")
        if s.scores not in ("sigmoid", "softmax"):
            raise ValueError(f"unknown scores {s.scores!r}: sigmoid or softmax")
        if s.expert_form not in ops.EXPERT_FORMS:
            raise ValueError(f"unknown expert form {s.expert_form!r}: {sorted(ops.EXPERT_FORMS)}")
        self.gated = s.expert_form == "gated_swish"
        if any((e.gate is None) == self.gated for e in s.experts):
            raise ValueError(f"experts of form {s.expert_form!r} {'need' if self.gated else 'have no'} gate matrices")
        if s.n_groups < 1 or s.n_experts % s.n_groups or not (1 <= s.keep_groups <= s.n_groups) or s.group_top < 1:
            raise ValueError(f"{s.n_experts} experts in {s.n_groups} groups of which {s.keep_groups} are kept is not a choice")
        if s.keep_groups * (s.n_experts // s.n_groups) < s.top:
            raise ValueError(f"the {s.keep_groups} kept groups hold fewer than {s.top} experts")
        if (s.correction or s.n_groups > 1) and s.scores != "sigmoid":
            raise ValueError("a correction of the choice and groups of experts go with sigmoid scores")
        self.router = self.gate_up = self.down = self.correction = None

    def tensor_specs(self):
        s = self.spec
        out = [TensorSpec(s.router, (s.n_experts, s.hidden), "matrix")]
        if s.correction:
            out.append(TensorSpec(s.correction, (s.n_experts,), "bias"))
        for e in s.experts:
            if self.gated:
                out.append(TensorSpec(e.gate, (s.ff, s.hidden), "matrix"))
            out += [TensorSpec(e.up, (s.ff, s.hidden), "matrix"), TensorSpec(e.down, (s.hidden, s.ff), "matrix")]
        return out

    def load(self, tensors, device, act_dtype):
        s = self.spec
        self.router = weight_to_device(tensors[s.router], device, act_dtype, s.router)
        if s.correction:
            self.correction = to_device(tensors[s.correction], device, torch.float32)
        first = weight_to_device(tensors[s.experts[0].up], device, act_dtype, s.experts[0].up)
        # gate rows, then up rows; experts without a gate: the up rows alone
        self.gate_up = torch.empty((s.n_experts, (2 if self.gated else 1) * s.ff, s.hidden), dtype=first.dtype, device=device)
        self.down = torch.empty((s.n_experts, s.hidden, s.ff), dtype=first.dtype, device=device)
        for i, e in enumerate(s.experts):
            mats = ((e.gate, self.gate_up[i, :s.ff]), (e.up, self.gate_up[i, s.ff:]), (e.down, self.down[i])) if self.gated \
                else ((e.up, self.gate_up[i]), (e.down, self.down[i]))
            for name, dst in mats:
                w = weight_to_device(tensors[name], device, act_dtype, name)
                if w.dtype != first.dtype:
                    raise ValueError(f"{name} is stored as {w.dtype}, the other experts' matrices as {first.dtype}")
                dst.copy_(w)

    def parameter_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.router, self.gate_up, self.down, self.correction)
                   if t is not None)

    def step_bytes(self, n_tokens: int) -> int:
        """Bytes of weights a step of n_tokens is expected to read: every expert once that some token chooses, with
        tokens that choose independently and evenly."""
        s = self.spec
        used = s.n_experts * (1.0 - (1.0 - s.top / s.n_experts) ** n_tokens)
        per = (self.gate_up[0].numel() + self.down[0].numel()) * self.gate_up.element_size()
        return int(self.router.numel() * self.router.element_size() + used * per)

    def forward(self, ctx, h, out, accumulate=True):
        s, N = self.spec, h.shape[0]
        ids = ctx.scratch(N, s.top, torch.int32)
        weights = ctx.scratch(N, s.top, torch.float32)
        ops.moe_route(h, self.router, ctx.token_request, ids, weights, s.top, softmax_scores=s.scores == "softmax",
                      renormalize=s.renormalize, correction=self.correction, n_groups=s.n_groups, keep_groups=s.keep_groups,
                      group_top=s.group_top, renorm_eps=s.renorm_eps, weight_scale=s.weight_scale)
        inf = math.inf
        limits = (s.gate_limit if s.gate_limit is not None else inf, -s.up_limit if s.up_limit is not None else -inf,
                  s.up_limit if s.up_limit is not None else inf)
        if N >= self.GROUPED_FROM and ops.moe_grouped_supported(h, self.gate_up, self.down):
            ops.moe_grouped(ctx, h, self.gate_up, self.down, ids, weights, out, *limits, s.act_alpha, s.up_shift,
                            weight_on_input=s.weight_on_input, accumulate=accumulate, form=s.expert_form)
            return
        y = ctx.scratch(N * s.top, s.ff)
        ops.moe_experts(h, self.gate_up, self.down, ids, weights, y, out, *limits, s.act_alpha, s.up_shift,
                        weight_on_input=s.weight_on_input, accumulate=accumulate,
                        per_pair=ctx.scratch(N * s.top, s.hidden, torch.float32), form=s.expert_form)


register_feed_forward("routed_experts", RoutedExperts)
