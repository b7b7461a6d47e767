"""The arrangement of a layer's parts.

pre_norm  (src/transformers_neuronx/opt/model.py:336-376):  x += mixer(norm1(x)); x += ff(norm2(x))
post_norm (the reference rejects it, opt/config.py:23-24; this is the usual order):
                                                          x = norm1(x + mixer(x)); x = norm2(x + ff(x))

post_norm_scaled:                                         x = norm1(a x + mixer(x)); x = norm2(a x + ff(x))
    with a = the layer's residual_scale; a layer may have no feed-forward (then no second norm).  The
    sublayer's result goes into a 32-bit buffer of its own and the norm's kernel forms the sum
    (Norm.forward_sum), so the stream is read and written once per sublayer.

output_norm:                                              x = x + m norm1(mixer(x)); x = x + m norm2(ff(x))
    with m = the layer's residual_scale: the norm sits on the sublayer's output only and the sublayers read x
    itself.  The sublayer's result goes into a 32-bit buffer and the norm's kernel adds it to the stream
    (Norm.forward_add); a layer may have no feed-forward.

sandwich_norm:                                            x = x + norm1_post(mixer(norm1(x))); x = x + norm2_post(ff(norm2(x)))
    a norm before and after each sublayer (the layer's spec names the two further norms).  The sublayer's result
    goes into a 32-bit buffer; one kernel normalises it, adds it to the stream and, where the next sublayer of the
    same layer follows, applies that sublayer's input norm to the new row (Norm.forward_add(..., then=norm2)).

parallel_residual:                                        x = x + s1 * mixer(norm1(x)) + s2 * ff(norm2(x))
    both sublayers read the same x, each behind a norm of its own (one kernel forms both norms: the mean square of a row
    is the same for both), and their results, multiplied channel by channel by learned vectors s1 and s2 (the layer's
    spec names the tensors; absent: 1), enter the stream in one pass.  A layer may have no feed-forward.

`x` is the 32-bit residual stream and is updated in place; `x_act` is its copy in the activation
type, which a block that feeds x itself into a matrix product needs on entry
(``needs_act_input``) and keeps current (``keeps_act_current``).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import NormedInput, Part, to_device
from .registry import register_block


class PreNormBlock:
    needs_act_input = False
    keeps_act_current = False

    def __init__(self, norm1, mixer, norm2, feed_forward):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    @staticmethod
    def _normed(ctx, x, norm, part):
        """norm(x) as the part's input: for one token and a part that takes it, the norm is handed on
        to be applied inside the part's first product; otherwise its own kernel runs here."""
        fused = getattr(norm, "fused_params", None)
        if (x.shape[0] == 1 and ctx.act_dtype != x.dtype and getattr(part, "takes_normed_input", False)
                and fused is not None and fused() is not None):
            return NormedInput(ctx, x, norm)
        h = ctx.scratch(x.shape[0], x.shape[1])
        norm.forward(ctx, x, out_act=h)
        return h

    def forward(self, ctx, x, x_act):
        self.mixer.forward(ctx, self._normed(ctx, x, self.norm1, self.mixer), x)
        self.feed_forward.forward(ctx, self._normed(ctx, x, self.norm2, self.feed_forward), x)


class PostNormBlock:
    needs_act_input = True
    keeps_act_current = True

    def __init__(self, norm1, mixer, norm2, feed_forward):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    def forward(self, ctx, x, x_act):
        self.mixer.forward(ctx, x_act, x)
        self.norm1.forward(ctx, x, out_f32=x, out_act=x_act)      # in place: a row is read whole first
        self.feed_forward.forward(ctx, x_act, x)
        self.norm2.forward(ctx, x, out_f32=x, out_act=x_act)


class ScaledPostNormBlock:
    """x <- norm(residual_scale * x + sublayer(x)).  A sublayer that can write its result instead of adding it
    (``can_overwrite``: forward(ctx, h, out, accumulate=False)) is asked to; any other adds into a zeroed buffer."""
    needs_act_input = True
    keeps_act_current = True
    takes_layer_spec = True

    def __init__(self, norm1, mixer, norm2, feed_forward, layer_spec=None):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward
        self.residual_scale = float(getattr(layer_spec, "residual_scale", 1.0))
        for n in (norm1, norm2 if feed_forward is not None else None):
            if n is not None and not hasattr(n, "forward_sum"):
                raise ValueError(f"a post_norm_scaled block needs norms that normalise a sum; {type(n).__name__} does not")

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    @staticmethod
    def _run(ctx, part, h, out):
        if getattr(part, "can_overwrite", False):
            part.forward(ctx, h, out, accumulate=False)
        else:
            out.zero_()
            part.forward(ctx, h, out)

    def forward(self, ctx, x, x_act):
        out = ctx.scratch(x.shape[0], x.shape[1], x.dtype)
        self._run(ctx, self.mixer, x_act, out)
        self.norm1.forward_sum(ctx, x, self.residual_scale, out, out_f32=x, out_act=x_act)
        if self.feed_forward is not None:
            self._run(ctx, self.feed_forward, x_act, out)
            self.norm2.forward_sum(ctx, x, self.residual_scale, out, out_f32=x, out_act=x_act)


class OutputNormBlock(ScaledPostNormBlock):
    """x <- x + residual_scale * norm(sublayer(x)): the sublayers read the stream itself (its copy in the
    activation type), only what they produce is normalised."""

    def __init__(self, norm1, mixer, norm2, feed_forward, layer_spec=None):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward
        self.residual_scale = float(getattr(layer_spec, "residual_scale", 1.0))
        for n in (norm1,) + ((norm2,) if feed_forward is not None else ()):
            if n is None or not hasattr(n, "forward_add"):
                raise ValueError(f"an output_norm block needs norms that add a normalised sublayer output to the stream; "
                                 f"{type(n).__name__} does not")

    def forward(self, ctx, x, x_act):
        out = ctx.scratch(x.shape[0], x.shape[1], x.dtype)
        self._run(ctx, self.mixer, x_act, out)
        self.norm1.forward_add(ctx, x, self.residual_scale, out, out_f32=x, out_act=x_act)
        if self.feed_forward is not None:
            self._run(ctx, self.feed_forward, x_act, out)
            self.norm2.forward_add(ctx, x, self.residual_scale, out, out_f32=x, out_act=x_act)


class SandwichNormBlock(ScaledPostNormBlock):
    """x <- x + norm1_post(mixer(norm1(x))), then x <- x + norm2_post(ff(norm2(x))); a layer may have no feed-forward."""
    needs_act_input = False
    keeps_act_current = False

    def __init__(self, norm1, mixer, norm2, feed_forward, layer_spec=None):
        from .registry import build_part
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward
        self.norm1_post = build_part("norm", getattr(layer_spec, "norm1_post", None))
        self.norm2_post = build_part("norm", getattr(layer_spec, "norm2_post", None)) if feed_forward is not None else None
        need = [(norm1, "forward"), (self.norm1_post, "forward_add")]
        if feed_forward is not None:
            need += [(norm2, "forward"), (self.norm2_post, "forward_add")]
        for n, method in need:
            if n is None or not hasattr(n, method):
                raise ValueError("a sandwich_norm block needs a norm before each sublayer and one that adds a normalised "
                                 f"sublayer output to the stream behind it; {type(n).__name__} does not fit")

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm1_post, self.norm2, self.feed_forward, self.norm2_post)
                if p is not None]

    def forward(self, ctx, x, x_act):
        N, W = x.shape
        h = ctx.scratch(N, W)
        self.norm1.forward(ctx, x, out_act=h)
        out = ctx.scratch(N, W, x.dtype)
        self._run(ctx, self.mixer, h, out)
        if self.feed_forward is None:
            self.norm1_post.forward_add(ctx, x, 1.0, out, out_f32=x)
            return
        # one kernel: the stream takes the normalised mixer output, and the new row is normalised for the feed-forward
        self.norm1_post.forward_add(ctx, x, 1.0, out, out_f32=x, out_act=h, then=self.norm2)
        self._run(ctx, self.feed_forward, h, out)
        self.norm2_post.forward_add(ctx, x, 1.0, out, out_f32=x)


class ChannelScale(Part):
    """A learned vector over the hidden axis that multiplies a sublayer's result (kept in 32-bit)."""
    graph_safe = True

    def __init__(self, name: str, size: int):
        self.name, self.size = name, size
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.size,), "norm_weight")]

    def load(self, tensors, device, act_dtype):
        self.weight = to_device(tensors[self.name], device, torch.float32)

    def parameter_bytes(self):
        return self.weight.numel() * 4 if self.weight is not None else 0


class ParallelResidualBlock(ScaledPostNormBlock):
    """x <- x + s1 * mixer(norm1(x)) + s2 * ff(norm2(x)), both sublayers on the same x."""
    needs_act_input = False
    keeps_act_current = False
    takes_layer_spec = True

    def __init__(self, norm1, mixer, norm2, feed_forward, layer_spec=None):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward
        need = [norm1] + ([norm2] if feed_forward is not None else [])
        for n in need:
            if n is None or not hasattr(n, "forward_pair"):
                raise ValueError("a parallel_residual block needs a norm before each sublayer that can share a kernel with "
                                 f"the other; {type(n).__name__} does not")
        size = norm1.spec.size
        s1, s2 = getattr(layer_spec, "scale1", None), getattr(layer_spec, "scale2", None)
        self.scale1 = ChannelScale(s1, size) if s1 else None
        self.scale2 = ChannelScale(s2, size) if (s2 and feed_forward is not None) else None

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.scale1, self.norm2, self.feed_forward, self.scale2)
                if p is not None]

    def forward(self, ctx, x, x_act):
        N, W = x.shape
        two = self.feed_forward is not None
        handed, ctx.handed_on = getattr(ctx, "handed_on", None), None
        if handed is not None and handed[0] == ctx.entry_index and handed[1] is self:
            h1, h2 = handed[2], handed[3]          # the block before formed them in the kernel that closed its layer
        else:
            h1 = ctx.scratch(N, W)
            h2 = ctx.scratch(N, W) if two else None
            self.norm1.forward_pair(ctx, x, h1, self.norm2 if two else None, h2)
        a = ctx.scratch(N, W, x.dtype)
        self._run(ctx, self.mixer, h1, a)
        b = None
        if two:
            b = ctx.scratch(N, W, x.dtype)
            self._run(ctx, self.feed_forward, h2, b)
        # the layer that follows, if it is of this kind, gets its two norms from the kernel that closes this one
        nxt, then = getattr(ctx, "next_block", None), None
        if isinstance(nxt, ParallelResidualBlock):
            par = (ctx.entry_index + 1) & 1
            n1, n2 = nxt.norm1, (nxt.norm2 if nxt.feed_forward is not None else None)
            o1 = ctx.carry(("pair", par, 0), N, W)
            o2 = ctx.carry(("pair", par, 1), N, W) if n2 is not None else None
            then = (n1.weight, n1.spec.weight_offset, n1.spec.eps, o1, n2.weight if n2 is not None else None,
                    n2.spec.weight_offset if n2 is not None else 0.0, n2.spec.eps if n2 is not None else 0.0, o2)
            ctx.handed_on = (ctx.entry_index + 1, nxt, o1, o2)
        ops.scaled_residual_add(x, a, self.scale1.weight if self.scale1 else None, b,
                                self.scale2.weight if self.scale2 else None, then=then)


register_block("pre_norm", PreNormBlock)
register_block("parallel_residual", ParallelResidualBlock)
register_block("sandwich_norm", SandwichNormBlock)
register_block("output_norm", OutputNormBlock)
register_block("post_norm_scaled", ScaledPostNormBlock)
register_block("post_norm", PostNormBlock)
