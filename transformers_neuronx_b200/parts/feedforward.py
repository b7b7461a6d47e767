"""Dense feed-forward: residual += fc2(act(fc1(h))) with biases
(src/transformers_neuronx/hlo.py:504-577); the activation is named by the configuration
(hlo.py:485-501).  The activation and the residual add run in the epilogues of the two products."""
from __future__ import annotations

from ..kernels import ops
from ..kernels.ops import activation_code
from .base import FeedForward
from .linear import Linear, fuse_linears
from .registry import register_feed_forward
from .spec import DenseFeedForwardSpec, GatedFeedForwardSpec


class DenseFeedForward(FeedForward):
    graph_safe = True
    takes_normed_input = True       # `h` only feeds fc1
    can_overwrite = True
    libraries = ("gemm_simt", "gemm_tc", "gemv")

    def __init__(self, spec: DenseFeedForwardSpec):
        self.spec = spec
        activation_code(spec.activation)          # raises on a name the epilogues do not know
        self.fc1, self.fc2 = Linear(spec.fc1), Linear(spec.fc2)

    def tensor_specs(self):
        return self.fc1.tensor_specs() + self.fc2.tensor_specs()

    def load(self, tensors, device, act_dtype):
        self.fc1.load(tensors, device, act_dtype)
        self.fc2.load(tensors, device, act_dtype)

    def parameter_bytes(self):
        return self.fc1.parameter_bytes() + self.fc2.parameter_bytes()

    def forward(self, ctx, h, residual, accumulate=True):
        a = ctx.scratch(h.shape[0], self.spec.fc1.out_features)
        self.fc1.forward(h, a, activation=self.spec.activation)
        self.fc2.forward(a, residual, residual=residual if accumulate else None)


class GatedDenseFeedForward(FeedForward):
    """down(act(gate(h)) * up(h)), all three with optional biases: gate and up are one product, the
    activation and the multiplication one elementwise kernel in 32-bit on its output."""
    graph_safe = True
    can_overwrite = True
    libraries = ("gemm_simt", "gemm_tc", "gemv", "gated_act")

    def __init__(self, spec: GatedFeedForwardSpec):
        self.spec = spec
        activation_code(spec.activation)
        if spec.gate.out_features != spec.up.out_features or spec.down.in_features != spec.up.out_features:
            raise ValueError("gate, up and down of a gated feed-forward must agree on the inner width")
        self.gate, self.up, self.down = Linear(spec.gate), Linear(spec.up), Linear(spec.down)
        self.gate_up = None

    def tensor_specs(self):
        return self.gate.tensor_specs() + self.up.tensor_specs() + self.down.tensor_specs()

    def load(self, tensors, device, act_dtype):
        for p in (self.gate, self.up, self.down):
            p.load(tensors, device, act_dtype)
        self.gate_up = fuse_linears([self.gate, self.up], device)
        for p in (self.gate, self.up):
            p.weight = p.bias = None

    def parameter_bytes(self):
        return self.gate_up.parameter_bytes() + self.down.parameter_bytes()

    def forward(self, ctx, h, out, accumulate=True):
        N, F = h.shape[0], self.spec.up.out_features
        gu = ctx.scratch(N, 2 * F)
        self.gate_up.forward(h, gu)
        a = ctx.scratch(N, F)
        ops.gated_activation(gu, a, self.spec.activation)
        self.down.forward(a, out, residual=out if accumulate else None)


register_feed_forward("dense", DenseFeedForward)
register_feed_forward("gated_dense", GatedDenseFeedForward)
