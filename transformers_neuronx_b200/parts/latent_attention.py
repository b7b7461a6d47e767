"""Softmax attention whose queries and whose keys and values pass through low-rank latents.

  c_q = rms(W_dq h) * g_q,   q = W_uq c_q, per head [k_dim unrotated | rot_dim rotated]
  W_dkv h = [x | r]:  c = rms(x) * g_kv  (kv_rank numbers, the latent),  r (rot_dim numbers) one key part for all heads
  per head:  k = [W_uk c | turn(r)],  v = W_uv c,  score(i, j) = scale * <q_i, k_j> over the window, softmax in 32-bit
  output projection on the concatenated heads

What the mixer keeps per position is c and the turned r only, as the pages of ONE key/value head of
D = kv_rank + rot_dim dims (rounded up to 16): the key row is [c | turn(r) | 0], the value row [c | 0].  The per-head
expansion moves to the queries' side, q'_h = [W_uk,h^T q_h | turn(q_rot,h) | 0], whose product with the key row is the
score above, and to the output's side, v_h-weighted sum = W_uv,h (sum_j p_j c_j).  Between the two sits the same paged
attention every other attention part uses (tcgen05 prefill, split decode with its own append, the 32-bit kernel), with
all query heads on the one key/value head.

The down projections of queries and of keys/values are one product; the two norms, the rotation of r and the rows'
layout are one kernel; the per-head products run as ONE batched tensor-core product (a launch for all heads) where
there are enough tokens and the sizes allow 16-byte accesses, else in one kernel that reads a head's matrix once for
eight tokens.
"""
from __future__ import annotations

import torch

from ..cache.manager import PagedKVNeed
from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Mixer, to_device, weight_to_device
from .linear import Linear, fuse_linears
from .registry import register_mixer
from .rotary import inverse_frequencies
from .spec import LatentAttentionSpec

MAX_ROW_DIMS = 768               # a position's row: up to 256 dims on the 16-bit attention kernels, beyond that on the CUDA cores
TENSOR_CORE_TOKENS = 64          # from this many tokens on the per-head products run as one batched tensor-core product


class LatentAttention(Mixer):
    graph_safe = True
    can_overwrite = True

    @property
    def libraries(self):
        prefill = "attention_prefill_tc" if self.pad_dim in (64, 80, 96, 112, 128) else "attention_prefill"
        return ("gemm_simt", "gemm_tc", "gemv", "latent_attention", "kv_cache", "attention_simt", prefill,
                "attention_decode")

    def __init__(self, spec: LatentAttentionSpec):
        s = self.spec = spec
        self.pad_dim = -(-(s.kv_rank + s.rot_dim) // 16) * 16
        if self.pad_dim > MAX_ROW_DIMS:
            raise ValueError(f"a latent of {s.kv_rank} and a rotated part of {s.rot_dim} dims are not supported: the "
                             f"attention kernels take up to {MAX_ROW_DIMS} dims a position")
        if s.rot_dim % 2 or (s.rot_dim and (s.rotary is None or s.rotary.dims != s.rot_dim)):
            raise ValueError(f"the rotated part of {s.rot_dim} dims needs a rotation over exactly those dims")
        if not (s.scale > 0):
            raise ValueError(f"the scale of the scores must be positive, got {s.scale}")
        self.dq, self.dkv, self.uq, self.out = Linear(s.dq), Linear(s.dkv), Linear(s.uq), Linear(s.out)
        self.down = None
        self.uk = self.uk_t = self.uv = self.uv_t = self.q_weight = self.kv_weight = self.inv_freq = None

    def tensor_specs(self):
        s = self.spec
        out = []
        for p in (self.dq, self.dkv, self.uq, self.out):
            out += p.tensor_specs()
        out += [TensorSpec(s.uk, (s.n_heads * s.k_dim, s.kv_rank), "matrix"),
                TensorSpec(s.uv, (s.n_heads * s.v_dim, s.kv_rank), "matrix")]
        if s.q_norm:
            out.append(TensorSpec(s.q_norm, (s.q_rank,), "norm_weight"))
        if s.kv_norm:
            out.append(TensorSpec(s.kv_norm, (s.kv_rank,), "norm_weight"))
        return out

    def load(self, tensors, device, act_dtype):
        s = self.spec
        for p in (self.dq, self.dkv, self.uq, self.out):
            p.load(tensors, device, act_dtype)
        self.down = fuse_linears([self.dq, self.dkv], device)
        self.dq.weight = self.dkv.weight = None
        H = s.n_heads
        uk = weight_to_device(tensors[s.uk], device, act_dtype, s.uk).to(act_dtype)
        uv = weight_to_device(tensors[s.uv], device, act_dtype, s.uv).to(act_dtype)
        # [head, inputs, outputs] for the kernel that walks a head's matrix once for eight tokens; [head, outputs, inputs]
        # (the layout of every product's weights) for the tensor-core products, in a 16-bit engine only
        self.uk = uk.view(H, s.k_dim, s.kv_rank).contiguous()
        self.uv = uv.view(H, s.v_dim, s.kv_rank).transpose(1, 2).contiguous()
        if act_dtype != torch.float32:
            self.uk_t = self.uk.transpose(1, 2).contiguous()
            self.uv_t = uv.view(H, s.v_dim, s.kv_rank).contiguous()
        f32 = lambda name: to_device(tensors[name], device, torch.float32) if name else None
        self.q_weight, self.kv_weight = f32(s.q_norm), f32(s.kv_norm)
        if s.rot_dim:
            self.inv_freq = inverse_frequencies(s.rot_dim, s.rotary.base, device)

    def parameter_bytes(self):
        n = self.down.parameter_bytes() + self.uq.parameter_bytes() + self.out.parameter_bytes()
        n += sum(t.numel() * t.element_size() for t in (self.uk, self.uv))
        return n + sum(t.numel() * 4 for t in (self.q_weight, self.kv_weight) if t is not None)

    def cache_need(self):
        return PagedKVNeed(1, self.pad_dim, self.spec.window)

    def _per_head(self, ctx, x, x_head, w, w_t, out, out_head, k, n_out, **tail):
        """out[:, h] = x[:, h, :k] W_h for every head: one batched tensor-core product for many tokens (where the sizes
        allow; it reads x up to k rounded up to 64 within a head, which the callers' buffers hold as finite numbers), else
        one kernel; the rotated tail and the padding, if any, by that kernel either way."""
        H, N = self.spec.n_heads, x.shape[0]
        if w_t is not None and N >= TENSOR_CORE_TOKENS and ops.gemm_tc_batched_supported(x, x_head, w_t, out, out_head):
            ops.gemm_tc_batched(x, x_head, w_t, out, out_head)       # all heads in one launch
            if tail:
                ops.headwise_product(x, x_head, None, out, out_head, ctx.token_request, H, k, n_out, do_product=False, **tail)
            return
        ops.headwise_product(x, x_head, w, out, out_head, ctx.token_request, H, k, n_out, **tail)

    def forward(self, ctx, h, out, accumulate=True):
        s, D, N = self.spec, self.pad_dim, h.shape[0]
        H, d, dr, dv, rq, rkv = s.n_heads, s.k_dim, s.rot_dim, s.v_dim, s.q_rank, s.kv_rank
        width = rq + rkv + dr
        proj = ctx.scratch(N, -(-width // 8) * 8)[:, :width]
        self.down.forward(h, proj)
        cq, k_new, v_new = ctx.scratch(N, rq), ctx.scratch(N, D), ctx.scratch(N, D)
        interleaved = bool(s.rotary is not None and s.rotary.interleaved)
        ops.latent_prep(proj, 0, ctx.token_request, ctx.positions, self.q_weight, self.kv_weight, s.norm_eps, self.inv_freq,
                        interleaved, cq, k_new, v_new, rq, rkv, dr)
        q = ctx.scratch(N, H * (d + dr))
        self.uq.forward(cq, q)
        qa = ctx.scratch(N, H * D)
        tail = dict(positions=ctx.positions, inv_freq=self.inv_freq, rot_dims=dr, interleaved=interleaved, pad_to=D) \
            if D > rkv else {}
        self._per_head(ctx, q, d + dr, self.uk, self.uk_t, qa, D, d, rkv, **tail)
        cache, g = ctx.cache(), ctx.cache_group()
        att = ctx.scratch(N, H * D)
        ops.attention(ctx, g, qa, cache, att, H, s.scale, s.window or 0, new_kv=(k_new, v_new, ctx.slot_mapping[g]))
        inner = ctx.scratch(N, H * dv)
        self._per_head(ctx, att, D, self.uv, self.uv_t, inner, dv, rkv, dv)
        self.out.forward(inner, out, residual=out if accumulate else None)


register_mixer("latent_attention", LatentAttention)
