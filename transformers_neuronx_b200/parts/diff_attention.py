"""Differential softmax attention over the paged cache.

  q = W_q h (heads x [map 1, map 2] x k_dim), k = W_k h (kv_heads x [map 1, map 2] x k_dim), v = W_v h (kv_heads x v_dim)
  every (head, map) of q and k: RMS norm with one weight vector of k_dim; q times 1 + c ln(floor((p + 1) / every) + 1)
  a_m = softmax(scale q_m k_m^T, causal) v        for the two maps m of a head, over the same values
  lambda = exp(<lq1, lk1>) - exp(<lq2, lk2>) + diff                 one number for the layer
  o = (a_1 - lambda a_2) / rms(a_1 - lambda a_2) * out_mult * sigmoid(W_g h)_head;   output projection

The two maps run as 2 heads query heads on the kv_heads key/value heads of ONE call of the paged attention kernels that
every other attention part uses, with rows of D = max(2 k_dim, v_dim) (rounded up to 16) dims: a key row holds both maps
side by side, the query of map 1 is zero on map 2's columns and the other way round, so a score is the map's own product,
and a key/value head's pages are read once for both maps and hold every value once (csrc/diff_attention.cu).  With
2 k_dim = v_dim a multiple of 16 nothing is padded.

cache_need() is the tuple (pages,); a mixer whose spec names `kv_source` keeps nothing: it projects queries and gates only
and reads the pages of the schedule entry with that cache number, which ran earlier in the same step, so that the pages
already hold this step's tokens (keys as they are kept: after the norm).
"""
from __future__ import annotations

import math

import torch

from ..cache.manager import PagedKVNeed
from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import to_device
from .fusable import FusableMixer
from .linear import Linear
from .registry import register_mixer
from .spec import DiffAttentionSpec


class DiffAttention(FusableMixer):
    @property
    def extra_libraries(self):
        prefill = "attention_prefill_tc" if self.pad_dim in (64, 80, 96, 112, 128) else "attention_prefill"
        return ("diff_attention", "kv_cache", "attention_simt", prefill, "attention_decode")

    def __init__(self, spec: DiffAttentionSpec):
        s = self.spec = spec
        if s.n_heads % s.n_kv_heads:
            raise ValueError(f"{s.n_heads} heads cannot share {s.n_kv_heads} key/value heads")
        self.pad_dim = -(-max(2 * s.k_dim, s.v_dim) // 16) * 16
        if self.pad_dim > 768:
            raise ValueError(f"head sizes 2 x {s.k_dim} / {s.v_dim} are not supported: the attention kernels take rows of up to 768")
        if not (s.scale > 0):
            raise ValueError(f"the scale of the scores must be positive, got {s.scale}")
        if s.temp_every < 0:
            raise ValueError("the query temperature's period must be positive (0: no temperature)")
        self.own_kv = s.kv_source is None
        if self.own_kv and (s.k is None or s.v is None):
            raise ValueError("an attention mixer without kv_source needs key and value projections")
        self.inputs = [Linear(s.q)] + ([Linear(s.k), Linear(s.v)] if self.own_kv else []) + \
                      ([Linear(s.gate)] if s.gate is not None else [])
        self.output = Linear(s.out)
        self.q_weight = self.k_weight = None
        self.lam = 0.0

    @property
    def inner_width(self):
        return self.spec.n_heads * self.spec.v_dim

    def extra_tensor_specs(self):
        s = self.spec
        out = [TensorSpec(n, (s.k_dim,), "norm_weight") for n in (s.q_norm, s.k_norm if self.own_kv else None) if n]
        return out + [TensorSpec(n, (s.k_dim,), "bias") for n in (s.lambda_q1, s.lambda_k1, s.lambda_q2, s.lambda_k2)]

    def load_extras(self, tensors, device, act_dtype):
        s = self.spec
        f32 = lambda name: to_device(tensors[name], device, torch.float32) if name else None
        self.q_weight, self.k_weight = f32(s.q_norm), (f32(s.k_norm) if self.own_kv else None)
        dot = lambda a, b: float((tensors[a].to(torch.float32) * tensors[b].to(torch.float32)).sum())
        # one number for the layer, in 32-bit like the norms
        lam = torch.tensor(math.exp(dot(s.lambda_q1, s.lambda_k1)) - math.exp(dot(s.lambda_q2, s.lambda_k2)) + s.diff,
                           dtype=torch.float32)
        self.lam = float(lam)

    def extra_parameter_bytes(self):
        return sum(t.numel() * 4 for t in (self.q_weight, self.k_weight) if t is not None)

    def cache_need(self):
        s = self.spec
        if not self.own_kv:
            return ()
        return (PagedKVNeed(s.n_kv_heads, self.pad_dim, s.window, None),)

    def forward(self, ctx, h, out, accumulate=True):
        N, width = h.shape[0], self.projection_width
        proj = ctx.scratch(N, -(-width // 8) * 8)[:, :width]   # the gates' few columns leave the row pitch a multiple of 16 bytes
        self._fused_in.forward(h, proj)
        inner = ctx.scratch(N, self.inner_width)
        self.mix(ctx, proj, 0, inner, 1.0)
        self.output.forward(inner, out, residual=out if accumulate else None)

    def mix(self, ctx, proj, col0, inner_out, out_scale, sub=None):
        if sub is not None:
            raise NotImplementedError("this mixer's caches are a tuple of its own and it cannot be a branch of another")
        s, D, N = self.spec, self.pad_dim, proj.shape[0]
        H, G, dk, dv = s.n_heads, s.n_kv_heads, s.k_dim, s.v_dim
        q = ctx.scratch(N, 2 * H * D)
        k = v = None
        if self.own_kv:
            k, v = ctx.scratch(N, G * D), ctx.scratch(N, G * D)
        ops.diff_qkv_prep(proj, col0, ctx.token_request, ctx.positions, self.q_weight, self.k_weight, s.norm_eps,
                          s.temp_coef, s.temp_every, q, k, v, H, G if self.own_kv else 0, dk, dv, D)
        if self.own_kv:
            cache, g = ctx.cache(0), ctx.cache_group(0)
            new_kv = (k, v, ctx.slot_mapping[g])
        else:
            cache, g = ctx.cache_of(s.kv_source, 0), ctx.cache_group_of(s.kv_source, 0)
            new_kv = None
            if cache.dim() != 5 or cache.shape[2] != G or cache.shape[4] != D:
                raise ValueError(f"cache {s.kv_source} does not hold pages of {G} key/value heads of {D} dims")
        att = ctx.scratch(N, 2 * H * D)
        ops.attention(ctx, g, q, cache, att, 2 * H, s.scale, s.window or 0, new_kv=new_kv)
        gate = None
        if s.gate is not None:
            g0 = col0 + 2 * H * dk + (G * (2 * dk + dv) if self.own_kv else 0)
            gate = proj[:, g0:g0 + H]
        ops.diff_combine(att, gate, ctx.token_request, self.lam, s.norm_eps, s.out_mult, out_scale, inner_out, H, dv, D)


register_mixer("diff_attention", DiffAttention)
