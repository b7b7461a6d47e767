"""Norms over the hidden axis.

RMS norm: y / sqrt(mean(y^2) + eps) * (weight + weight_offset), in 32-bit; it can normalise a sum
y = x_scale * x + delta in the same kernel, which is what a post-norm block with a scaled residual asks for,
or normalise a sublayer's output alone and add it to the stream (x + add_scale * norm(delta)).

LayerNorm as the reference computes it: statistics and affine in 32-bit over the hidden axis
(src/transformers_neuronx/hlo.py:84-105), with eps, scale and shift as parameters of the part."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Norm, to_device
from .registry import register_norm
from .spec import NormSpec


class LayerNorm(Norm):
    graph_safe = True
    libraries = ("layernorm",)

    def __init__(self, spec: NormSpec):
        self.spec = spec
        self.weight = None
        self.bias = None

    def tensor_specs(self):
        s, out = self.spec, []
        if s.weight:
            out.append(TensorSpec(s.weight, (s.size,), "norm_weight"))
        if s.bias:
            out.append(TensorSpec(s.bias, (s.size,), "norm_bias"))
        return out

    def load(self, tensors, device, act_dtype):
        s = self.spec
        self.weight = to_device(tensors[s.weight], device, torch.float32) if s.weight else None
        self.bias = to_device(tensors[s.bias], device, torch.float32) if s.bias else None

    def parameter_bytes(self):
        return sum(t.numel() * 4 for t in (self.weight, self.bias) if t is not None)

    def fused_params(self):
        return self.weight, self.bias, self.spec.eps

    def forward(self, ctx, x, out_f32=None, out_act=None, rows=None):
        ops.layer_norm(x, self.weight, self.bias, self.spec.eps, out_f32=out_f32, out_act=out_act, rows=rows)


class RMSNorm(Norm):
    graph_safe = True
    takes_out_scale = True            # forward(..., out_scale=c) multiplies the result by a constant in the same kernel
    libraries = ("rmsnorm",)

    def __init__(self, spec: NormSpec):
        if spec.bias:
            raise ValueError("an RMS norm has no shift")
        self.spec = spec
        self.weight = None

    def tensor_specs(self):
        s = self.spec
        return [TensorSpec(s.weight, (s.size,), "norm_weight")] if s.weight else []

    def load(self, tensors, device, act_dtype):
        s = self.spec
        self.weight = to_device(tensors[s.weight], device, torch.float32) if s.weight else None

    def parameter_bytes(self):
        return self.weight.numel() * 4 if self.weight is not None else 0

    def forward(self, ctx, x, out_f32=None, out_act=None, rows=None, out_scale=1.0):
        ops.rms_norm(x, self.weight, self.spec.eps, out_f32=out_f32, out_act=out_act, rows=rows,
                     weight_offset=self.spec.weight_offset, out_scale=out_scale)

    def forward_pair(self, ctx, x, out1, other=None, out2=None):
        """This norm and `other` (an RMSNorm) of the same rows in one kernel: the inputs of two sublayers side by side."""
        if other is not None and not isinstance(other, RMSNorm):
            raise ValueError(f"only RMS norms share a kernel, not {type(other).__name__}")
        o = other.spec if other is not None else None
        ops.rms_norm_pair(x, self.weight, self.spec.weight_offset, self.spec.eps, out1,
                          other.weight if other is not None else None, o.weight_offset if o else 0.0,
                          o.eps if o else 0.0, out2 if other is not None else None)

    def forward_sum(self, ctx, x, x_scale, delta, out_f32=None, out_act=None):
        """norm(x_scale * x + delta) in one kernel; out_f32 may be x."""
        ops.rms_norm(x, self.weight, self.spec.eps, out_f32=out_f32, out_act=out_act, x_scale=x_scale, delta=delta,
                     weight_offset=self.spec.weight_offset)

    def forward_add(self, ctx, x, add_scale, delta, out_f32=None, out_act=None, then=None):
        """x + add_scale * norm(delta) in one kernel (the norm on a sublayer's output alone); out_f32 may be x.
        `then` (another RMSNorm): out_act receives that norm of the new row instead of the row's copy."""
        nxt = None
        if then is not None:
            if not isinstance(then, RMSNorm):
                raise ValueError(f"only an RMS norm can follow inside the same kernel, not {type(then).__name__}")
            nxt = (then.weight, then.spec.weight_offset, then.spec.eps)
        ops.rms_norm_add(x, add_scale, delta, self.weight, self.spec.eps, out_f32=out_f32, out_act=out_act,
                         weight_offset=self.spec.weight_offset, then=nxt)


register_norm("layer_norm", LayerNorm)
register_norm("rms_norm", RMSNorm)
