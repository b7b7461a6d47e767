"""Shared by the Tutelix tests: small configurations that differ from one another in every size and constant (head
counts and shared key heads, windows that are and are not multiples of a page, partly and fully rotated heads, latents
narrower and wider than a head, convolutions of 1 to 5 taps, inner sizes of the low-rank projections, loops over one
layer, over several and none, layers without a feed-forward), and a model folder with seeded random weights beside the
plain implementation's answers (tests/plain/tutelix_plain.py)."""
from __future__ import annotations

import torch

from plain import tutelix_plain as TP
from vononex_helpers import VononexModel, compare, cut_steps, mixed_steps, whole_steps  # noqa: F401  (architecture-neutral)


def attention(heads, kv, dim, scale, window, rot_dims, base):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    return m


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window, base):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"dims": rot_dim, "base": base}}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def delta(heads, kv, dim, vdim, conv, decay_rank, gate_rank):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": decay_rank,
            "gate_rank": gate_rank}


def layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


# Odd sizes everywhere: 6 heads on 2 key heads of 24 dims with 16 rotated and a window of 21 (no multiple of a page); a
# latent layer whose latent (40) is wider than its heads (12 + 6 rotated; values of 20), without feed-forward; a
# recurrence whose 6 heads share 2 query/key heads of 18 dims with values of 10, five taps; a loop of three passes over
# two layers; widths the tensor-core product refuses in places.
CONFIG_A = {"architecture": "Tutelix", "vocab": 211, "width": 72, "embedding": {"scale": 3.7}, "norm": {"eps": 1e-4},
            "init_std": 0.2, "loop": {"start": 1, "stop": 3, "times": 3}, "layers": [
                layer("attention", attention(6, 2, 24, 0.3, 21, 16, 500.0), 88),
                layer("latent_attention", latent(5, 12, 6, 20, 28, 40, 0.25, 33, 77.0), None),
                layer("channel_delta", delta(6, 2, 18, 10, 5, 7, 12), 50),
                layer("attention", attention(2, 1, 64, 0.125, None, 64, 10000.0), None)]}
# Sizes the tensor-core kernels take: head sizes 128 and 64, latents of 48 + 16 and 96 + 32 dims a position, windows of
# 64 and 48, a layer without mask, recurrences with 128 and 32 rows a column, a single looped layer, one tap.
CONFIG_B = {"architecture": "Tutelix", "vocab": 1003, "width": 256, "embedding": {"scale": 16.0}, "norm": {"eps": 1e-6},
            "init_std": 0.1, "loop": {"start": 2, "stop": 3, "times": 2}, "layers": [
                layer("channel_delta", delta(2, 2, 128, 64, 4, 16, 24), 320),
                layer("latent_attention", latent(6, 64, 16, 32, 72, 48, 0.11, 64, 20000.0), 128),
                layer("attention", attention(6, 3, 128, 0.09, 48, 32, 100000.0), 384),
                layer("latent_attention", latent(4, 32, 32, 96, 48, 96, 0.12, None, 3e4), None),
                layer("channel_delta", delta(4, 2, 32, 64, 1, 8, 8), 192)]}
# A width and a vocabulary that are no multiples of 8 (the 16-bit engine falls back to the CUDA-core product and to
# scalar loads), as many key heads as heads, head sizes of 20, no loop, a window of one page and a window of a single
# position, an unrotated attention layer, a latent without rotated part, a recurrence of one head.
CONFIG_C = {"architecture": "Tutelix", "vocab": 333, "width": 100, "embedding": {"scale": 0.5}, "norm": {"eps": 1e-5},
            "init_std": 0.2, "layers": [
                layer("attention", attention(5, 5, 20, 0.22, 16, 20, 2000.0), 36),
                layer("channel_delta", delta(1, 1, 50, 30, 2, 5, 3), None),
                layer("latent_attention", latent(3, 10, 0, 14, 9, 22, 0.3, 1, 50.0), 70),
                layer("attention", attention(2, 1, 50, 0.14, 40, 0, 1.0), 44)]}
# Rows wider than the 16-bit attention kernels take (256 dims a position): a latent of 272 with 16 rotated dims, heads of
# 288 whose values are their keys.
CONFIG_D = {"architecture": "Tutelix", "vocab": 120, "width": 96, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
            "init_std": 0.1, "layers": [
                layer("latent_attention", latent(3, 24, 16, 40, 20, 272, 0.2, 37, 300.0), 64),
                layer("attention", attention(2, 1, 288, 0.06, 50, 32, 1e4), None)]}
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D}


class TutelixModel(VononexModel):
    def plain_logits(self, ids):
        key = tuple(int(i) for i in ids)
        if key not in self._cache:
            self._cache[key] = TP.forward_logits(key, self.plain_tensors, self.cfg_dict).float()
        return self._cache[key]

    def plain_hidden(self, ids):
        return TP.forward_hidden(tuple(int(i) for i in ids), self.plain_tensors, self.cfg_dict)[0].float()
