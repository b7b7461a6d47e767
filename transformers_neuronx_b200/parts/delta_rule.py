"""A recurrent mixer with an error-correcting write ("delta rule") and a decay per head and key channel.

  q = W_q h, k = W_k h (n_kv_heads x k_dim; head i uses q/k head i / (n_heads / n_kv_heads)), v = W_v h (n_heads x v_dim)
  each channel of q, k and v through a short causal convolution over time, then an activation (silu)
  q, k per head: x / sqrt(sum(x^2) + unit_eps); q times q_scale
  beta = sigmoid(W_b h) per head;  g = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 h) + dt_bias)) per head and key channel
  per head:  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
  each head's o divided by its root mean square, times a weight vector of v_dim, times sigmoid(W_g2 (W_g1 h)); output projection

What the mixer keeps per request, both state of fixed size in the request's slot (zeroed when a request takes it): S
(n_heads x v_dim x k_dim, a column's rows side by side) in 32-bit, and the last taps - 1 projected values of every
convolved channel in the activation type, exactly what a longer step would have read from its own rows.  Everything
that enters the recurrence is 32-bit from the projections' output on: the convolution's sums, the unit norms, beta and g
(their logits leave the second low-rank product in 32-bit).  A step's tokens of one request are walked in order by one
kernel, portions of prompts and single tokens alike, so the state after a token does not depend on how the prompt was cut.

All projections of h (q, k, v, the two low-rank first halves, beta) are one product.
"""
from __future__ import annotations

import torch

from ..cache.manager import FixedStateNeed
from ..kernels import ops
from ..kernels.ops import activation_code
from ..weights.loader import TensorSpec
from .base import Mixer, to_device
from .linear import Linear, fuse_linears
from .registry import register_mixer
from .spec import DeltaRuleSpec

MAX_TAPS = 8           # csrc/delta_rule.cu
MAX_K_DIM = 256


class DeltaRule(Mixer):
    graph_safe = True
    can_overwrite = True
    libraries = ("gemm_simt", "gemm_tc", "gemv", "delta_rule", "conv_qkv", "retention")

    def __init__(self, spec: DeltaRuleSpec):
        s = self.spec = spec
        if s.n_heads % s.n_kv_heads:
            raise ValueError(f"{s.n_heads} heads cannot share {s.n_kv_heads} query/key heads")
        if not (1 <= s.conv_taps <= MAX_TAPS):
            raise ValueError(f"a convolution of {s.conv_taps} taps is not supported (1 to {MAX_TAPS})")
        if s.k_dim > MAX_K_DIM:
            raise ValueError(f"key size {s.k_dim} is not supported: the scan keeps up to {MAX_K_DIM} rows of a column in a warp")
        activation_code(s.conv_activation)
        self.q, self.k, self.v, self.beta = Linear(s.q), Linear(s.k), Linear(s.v), Linear(s.beta)
        self.a1, self.a2, self.g1, self.g2, self.out = Linear(s.a1), Linear(s.a2), Linear(s.g1), Linear(s.g2), Linear(s.out)
        self.keep = s.conv_taps - 1
        self.channels = 2 * s.n_kv_heads * s.k_dim + s.n_heads * s.v_dim
        self.fused_in = self.conv_w = self.a_log = self.dt_bias = self.norm_w = None
        self.rank_a = self.rank_g = 0

    def _conv_names(self):
        s = self.spec
        return [(s.q_conv, s.n_kv_heads * s.k_dim), (s.k_conv, s.n_kv_heads * s.k_dim), (s.v_conv, s.n_heads * s.v_dim)]

    def tensor_specs(self):
        s, out = self.spec, []
        for p in (self.q, self.k, self.v, self.beta, self.a1, self.a2, self.g1, self.g2, self.out):
            out += p.tensor_specs()
        for name, ch in self._conv_names():
            out.append(TensorSpec(name, (ch, s.conv_taps), "matrix"))
        out += [TensorSpec(s.a_log, (s.n_heads,), "bias"), TensorSpec(s.dt_bias, (s.n_heads * s.k_dim,), "bias")]
        if s.out_norm:
            out.append(TensorSpec(s.out_norm, (s.v_dim,), "norm_weight"))
        return out

    def load(self, tensors, device, act_dtype):
        s = self.spec
        for p in (self.q, self.k, self.v, self.beta, self.a1, self.a2, self.g1, self.g2, self.out):
            p.load(tensors, device, act_dtype)
        self.rank_a, self.rank_g = self.a1.weight.shape[0], self.g1.weight.shape[0]
        if self.a2.weight.shape[1] != self.rank_a or self.g2.weight.shape[1] != self.rank_g:
            raise ValueError(f"{s.a1.weight} / {s.a2.weight} or {s.g1.weight} / {s.g2.weight}: the two halves of a low-rank "
                             "projection do not agree on its inner size")
        # q, k, v first (the convolved channels, side by side), the write strengths' few columns last
        ins = [self.q, self.k, self.v, self.a1, self.g1, self.beta]
        self.fused_in = fuse_linears(ins, device)
        for p in ins:
            p.weight = p.bias = None
        f32 = lambda name: to_device(tensors[name], device, torch.float32)
        # [taps, channels]: the kernel reads a tap's weights of consecutive channels together
        self.conv_w = torch.cat([f32(name) for name, _ in self._conv_names()], dim=0).t().contiguous()
        self.a_log, self.dt_bias = f32(s.a_log), f32(s.dt_bias)
        self.norm_w = f32(s.out_norm) if s.out_norm else None

    def parameter_bytes(self):
        n = sum(p.parameter_bytes() for p in (self.fused_in, self.a2, self.g2, self.out))
        return n + sum(t.numel() * 4 for t in (self.conv_w, self.a_log, self.dt_bias, self.norm_w) if t is not None)

    def cache_need(self):
        s = self.spec
        state = FixedStateNeed((s.n_heads, s.v_dim, s.k_dim), "float32")
        if not self.keep:
            return (state,)
        return (state, FixedStateNeed((self.keep, self.channels), "activation"))

    def forward(self, ctx, h, out, accumulate=True):
        s, N = self.spec, h.shape[0]
        H, G, dk, dv = s.n_heads, s.n_kv_heads, s.k_dim, s.v_dim
        C, ra, rg = self.channels, self.rank_a, self.rank_g
        width = C + ra + rg + H
        proj = ctx.scratch(N, -(-width // 8) * 8)[:, :width]
        self.fused_in.forward(h, proj)
        f32 = torch.float32
        a = ctx.scratch(N, H * dk, f32)                       # the decays' logits stay 32-bit
        self.a2.forward(proj[:, C:C + ra], a)
        gate = ctx.scratch(N, H * dv)
        self.g2.forward(proj[:, C + ra:C + ra + rg], gate)
        q, k = ctx.scratch(N, G * dk, f32), ctx.scratch(N, G * dk, f32)
        v, beta, g = ctx.scratch(N, H * dv, f32), ctx.scratch(N, H, f32), ctx.scratch(N, H * dk, f32)
        ops.delta_prep(proj, 0, C + ra + rg, a, self.conv_w, s.conv_taps, ctx.cache(1) if self.keep else None, ctx,
                       self.a_log, self.dt_bias, s.unit_eps, s.q_scale, s.conv_activation, q, k, v, beta, g, H, G, dk, dv)
        o = ctx.scratch(N, H * dv, f32)
        ops.delta_scan(q, k, v, beta, g, ctx.cache(0), ctx.q_start, ctx.q_len, ctx.state_slots, o, H, G, dk, dv)
        inner = ctx.scratch(N, H * dv)
        ops.headwise_gated_rms_norm(o, gate, ctx.token_request, self.norm_w, s.norm_eps, 1.0, inner, H, dv,
                                    gate_activation="sigmoid")
        self.out.forward(inner, out, residual=out if accumulate else None)


register_mixer("delta_rule", DeltaRule)
