"""Softmax attention over the paged cache with rotated queries, keys and (optionally) values.

  q = W_q h + b, k = W_k h + b, v = W_v h + b
  q, k: RMS norm over the WHOLE projection (all heads at once) where the spec names a weight, before rotation
  q, k: rotated by position on the first rotary.dims dims of each head (dim i with dim i + dims/2)
  score(i, j) = scale * head_scale[h] * <q_i, k_j>, causal (and windowed where the spec says), softmax in 32-bit
  rotate_values: v_j is turned by its position j over all v_dim dims before it is cached, and each head's
      output at position i is turned back by i: the sum then holds the values turned by j - i
  output projection with bias
  a spec without a value projection: the values are the keys as projected (bias included), before their norm and
      rotation; nothing more is computed for them, the same columns of the product are read twice

Queries/keys (k_dim) and values (v_dim) may differ in size.  The cache's pages and the attention kernels take
one head size, so q, k and v are written with D = max(k_dim, v_dim) rounded up to 16 dims a head, the rest zero:
zeros in q and k add nothing to a score, zeros in v give output columns that are dropped.  With k_dim = v_dim a
multiple of 16 (the usual case) nothing is padded, and the kernels are those of every other attention part:
tcgen05 prefill, split-KV decode with its own cache append, the 32-bit kernel in a 32-bit engine.  head_scale
is folded into q in 32-bit before q is rounded.
"""
from __future__ import annotations

import torch

from ..cache.manager import PagedKVNeed
from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import to_device
from .fusable import FusableMixer
from .linear import Linear
from .registry import register_mixer
from .rotary import inverse_frequencies
from .spec import RotaryAttentionSpec


class RotaryAttention(FusableMixer):
    @property
    def extra_libraries(self):
        # the prefill kernel of this head size only: tcgen05 for 64 .. 128, mma.sync for the others
        prefill = "attention_prefill_tc" if self.pad_dim in (64, 80, 96, 112, 128) else "attention_prefill"
        return ("rotary_qkv", "kv_cache", "attention_simt", prefill, "attention_decode")

    def __init__(self, spec: RotaryAttentionSpec):
        s = self.spec = spec
        if s.n_heads % s.n_kv_heads:
            raise ValueError(f"{s.n_heads} heads cannot share {s.n_kv_heads} key/value heads")
        self.pad_dim = -(-max(s.k_dim, s.v_dim) // 16) * 16
        if self.pad_dim > 768:                       # up to 256 on the 16-bit kernels, beyond that on the CUDA cores
            raise ValueError(f"head sizes {s.k_dim}/{s.v_dim} are not supported: the attention kernels take up to 768")
        if s.rotary is not None and (s.rotary.dims > s.k_dim or s.rotary.dims % 2):
            raise ValueError(f"{s.rotary.dims} rotated dims do not fit heads of {s.k_dim}")
        if s.rotate_values and (s.rotary is None or s.v_dim % 2):
            raise ValueError("rotated values need a rotation and an even value size")
        self.values_are_keys = s.v is None
        if self.values_are_keys and (s.v_dim != s.k_dim or s.rotate_values):
            raise ValueError("values that are the keys have the keys' size and are not rotated")
        self.inputs = [Linear(s.q), Linear(s.k)] + ([] if self.values_are_keys else [Linear(s.v)])
        self.output = Linear(s.out)
        self.q_weight = self.k_weight = self.head_scale = self.inv_freq_qk = self.inv_freq_v = None

    @property
    def inner_width(self):
        return self.spec.n_heads * self.spec.v_dim

    def extra_tensor_specs(self):
        s, out = self.spec, []
        if s.q_norm:
            out.append(TensorSpec(s.q_norm, (s.n_heads * s.k_dim,), "norm_weight"))
        if s.k_norm:
            out.append(TensorSpec(s.k_norm, (s.n_kv_heads * s.k_dim,), "norm_weight"))
        if s.head_scale:
            out.append(TensorSpec(s.head_scale, (s.n_heads,), "norm_weight"))
        return out

    def load_extras(self, tensors, device, act_dtype):
        s = self.spec
        f32 = lambda name: to_device(tensors[name], device, torch.float32) if name else None
        self.q_weight, self.k_weight, self.head_scale = f32(s.q_norm), f32(s.k_norm), f32(s.head_scale)
        if s.rotary is not None and s.rotary.dims:
            self.inv_freq_qk = inverse_frequencies(s.rotary.dims, s.rotary.base, device)
        if s.rotate_values:
            self.inv_freq_v = inverse_frequencies(s.v_dim, s.rotary.base, device)

    def extra_parameter_bytes(self):
        return sum(t.numel() * 4 for t in (self.q_weight, self.k_weight, self.head_scale) if t is not None)

    def cache_need(self):
        return PagedKVNeed(self.spec.n_kv_heads, self.pad_dim, self.spec.window)

    def mix(self, ctx, proj, col0, inner_out, out_scale, sub=None):
        s, D, N = self.spec, self.pad_dim, proj.shape[0]
        H, G = s.n_heads, s.n_kv_heads
        q, k, v = ctx.scratch(N, H * D), ctx.scratch(N, G * D), ctx.scratch(N, G * D)
        k_off = col0 + H * s.k_dim
        v_off = k_off if self.values_are_keys else k_off + G * s.k_dim
        ops.rotary_qkv_prep(proj, col0, k_off, v_off, ctx.token_request, ctx.positions, self.q_weight,
                            self.k_weight, s.norm_eps, self.head_scale, self.inv_freq_qk,
                            s.rotary.dims if s.rotary is not None else 0, self.inv_freq_v, q, k, v, H, G, s.k_dim,
                            s.v_dim, D)
        cache, g = ctx.cache(sub), ctx.cache_group(sub)
        # heads that are neither padded, turned back nor scaled go from the attention kernel straight to their place
        direct = (D == s.v_dim and self.inv_freq_v is None and out_scale == 1.0 and inner_out.dtype == q.dtype
                  and inner_out.stride(0) % 8 == 0 and inner_out.data_ptr() % 16 == 0)
        att = inner_out if direct else ctx.scratch(N, H * D)
        ops.attention(ctx, g, q, cache, att, H, s.scale, s.window or 0, new_kv=(k, v, ctx.slot_mapping[g]))
        if not direct:
            ops.rotary_unrotate(att, ctx.token_request, ctx.positions, self.inv_freq_v, out_scale, inner_out, H, s.v_dim, D)


register_mixer("rotary_attention", RotaryAttention)
