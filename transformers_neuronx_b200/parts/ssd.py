"""A selective state-space mixer with one decay per head and token ("state-space duality").

  W_in h = [z: inner | x: inner | B: groups * state | C: groups * state | dt: heads],  inner = heads * v_dim
  x, B, C: one short causal convolution per channel over time (with bias), then an activation (silu)
  dt = softplus(dt + dt_bias);  per head h (group h / (heads / groups)), S of state x v_dim:
      S <- exp(-exp(A_log_h) dt) S + dt B x^T;   y = S^T C + D_h x
  y * act(z), divided by its root mean square in `norm_groups` equal parts of the inner width, times a weight; output projection

The recurrence is retention's (parts/retention.py: S <- decay S + k v^T, o = S^T q) with k = B, q = C, v = x, a decay and
a key scale (dt) that change from token to token, and keys and queries shared by the heads of a group; it runs on
retention's scan kernel with those options.  What the mixer keeps per request, both state of fixed size in the
request's slot (zeroed when a request takes it): S (heads x v_dim x state, a column's rows side by side) in 32-bit, and
the last taps - 1 projected values of every convolved channel in the activation type, exactly what a longer step would
have read from its own rows.  Everything behind the convolution's activation is 32-bit: x, B, C, dt, the decays, the
state and y.  A step's tokens of one request are walked in order by one kernel, portions of prompts and single tokens
alike, so the state after a token does not depend on how the prompt was cut.
"""
from __future__ import annotations

import torch

from ..cache.manager import FixedStateNeed
from ..kernels import ops
from ..kernels.ops import activation_code
from ..weights.loader import TensorSpec
from .base import Mixer, to_device
from .linear import Linear
from .registry import register_mixer
from .spec import SSDSpec

MAX_TAPS = 8           # csrc/ssd.cu
MAX_STATE = 256        # the scan keeps up to 256 rows of a column in a warp


class SSD(Mixer):
    graph_safe = True
    can_overwrite = True
    libraries = ("gemm_simt", "gemm_tc", "gemv", "ssd", "conv_qkv", "retention")

    def __init__(self, spec: SSDSpec):
        s = self.spec = spec
        if s.n_heads % s.groups:
            raise ValueError(f"{s.n_heads} heads cannot share {s.groups} groups of B and C")
        if not (1 <= s.conv_taps <= MAX_TAPS):
            raise ValueError(f"a convolution of {s.conv_taps} taps is not supported (1 to {MAX_TAPS})")
        if s.state > MAX_STATE:
            raise ValueError(f"state size {s.state} is not supported: the scan keeps up to {MAX_STATE} rows of a column in a warp")
        self.inner = s.n_heads * s.v_dim
        if self.inner % s.norm_groups:
            raise ValueError(f"{self.inner} inner channels do not form {s.norm_groups} equal parts")
        activation_code(s.activation)
        self.channels = self.inner + 2 * s.groups * s.state
        self.keep = s.conv_taps - 1
        self.in_proj, self.out = Linear(s.in_proj), Linear(s.out)
        self.conv_w = self.conv_b = self.a_log = self.dt_bias = self.skip = self.norm_w = None

    def tensor_specs(self):
        s = self.spec
        out = self.in_proj.tensor_specs() + self.out.tensor_specs()
        out.append(TensorSpec(s.conv, (self.channels, s.conv_taps), "matrix"))
        if s.conv_bias:
            out.append(TensorSpec(s.conv_bias, (self.channels,), "bias"))
        out += [TensorSpec(s.dt_bias, (s.n_heads,), "bias"), TensorSpec(s.a_log, (s.n_heads,), "bias")]
        if s.skip:
            out.append(TensorSpec(s.skip, (s.n_heads,), "bias"))
        if s.out_norm:
            out.append(TensorSpec(s.out_norm, (self.inner,), "norm_weight"))
        return out

    def load(self, tensors, device, act_dtype):
        s = self.spec
        self.in_proj.load(tensors, device, act_dtype)
        self.out.load(tensors, device, act_dtype)
        f32 = lambda name: to_device(tensors[name], device, torch.float32) if name else None
        self.conv_w = f32(s.conv).t().contiguous()            # [taps, channels]: a tap's weights of consecutive channels together
        self.conv_b, self.a_log, self.dt_bias = f32(s.conv_bias), f32(s.a_log), f32(s.dt_bias)
        self.skip, self.norm_w = f32(s.skip), f32(s.out_norm)

    def parameter_bytes(self):
        n = self.in_proj.parameter_bytes() + self.out.parameter_bytes()
        return n + sum(t.numel() * 4 for t in (self.conv_w, self.conv_b, self.a_log, self.dt_bias, self.skip, self.norm_w)
                       if t is not None)

    def cache_need(self):
        s = self.spec
        state = FixedStateNeed((s.n_heads, s.v_dim, s.state), "float32")      # a column's rows side by side
        if not self.keep:
            return (state,)
        return (state, FixedStateNeed((self.keep, self.channels), "activation"))

    def forward(self, ctx, h, out, accumulate=True):
        s, N = self.spec, h.shape[0]
        H, P, Ns, G, inner = s.n_heads, s.v_dim, s.state, s.groups, self.inner
        width = inner + self.channels + H
        proj = ctx.scratch(N, -(-width // 8) * 8)[:, :width]
        self.in_proj.forward(h, proj)
        f32 = torch.float32
        x, b, c = ctx.scratch(N, inner, f32), ctx.scratch(N, G * Ns, f32), ctx.scratch(N, G * Ns, f32)
        dt, decay = ctx.scratch(N, H, f32), ctx.scratch(N, H, f32)
        ops.ssd_prep(proj, 0, self.conv_w, self.conv_b, s.conv_taps, ctx.cache(1) if self.keep else None, ctx, self.a_log,
                     self.dt_bias, s.activation, x, b, c, dt, decay, H, P, G, Ns)
        y = ctx.scratch(N, inner, f32)
        ops.retention_scan(c, b, x, None, ctx.cache(0), ctx.q_start, ctx.q_len, ctx.state_slots, y, H, Ns, P,
                           most_tokens=1 if ctx.decode_only else N, decay_tok=decay, kscale_tok=dt, qk_heads=G)
        act = ctx.scratch(N, inner)
        ops.ssd_gate_norm(y, x, self.skip, proj[:, :inner], ctx.token_request, self.norm_w, s.norm_eps, s.activation, act, P,
                          s.norm_groups)
        self.out.forward(act, out, residual=out if accumulate else None)


register_mixer("ssd", SSD)
