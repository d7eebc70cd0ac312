"""Arrangements of a layer's parts around the residual stream.

"prenorm": h <- h + mixer(norm(h)); h <- h + feed_forward(norm(h)), carried as the pair
(x = the last sublayer's output, residual = the float32 stream) so that every "add, then
normalise" is one kernel (12vivi/tandem python/tandem/models/llama_family.py:11-16,59-67).

"parallel": n = norm(h); h <- h + (mixer(n) + feed_forward(n)): one norm, both sublayers read
its output, and their outputs (with their biases) are added into the float32 stream together.
The feed-forward may be absent.

"connected": pre-norm sublayers on a residual of one or several streams, each sublayer tied to it
by a link of its own (``parts/connection.py``): u = norm(read of the streams); y = sublayer(u);
the streams are rewritten from themselves and y.  The write is left pending and done by the next
norm's kernel, so every "write, read, normalise" is one launch.  The feed-forward may be absent.

"postnorm": the norms sit on the sublayers' OUTPUT, x <- x + norm(mixer(x)); x <- x + norm(feed_forward(x)), all
on one float32 stream.  Optional parts: a short convolution in front of either sublayer (the sublayer reads
x + conv(x)), and a depth average behind the layer (what is handed on is a weighted sum of the results of all
layers so far).  One kernel per boundary does "norm, add, [average,] convolution"; the feed-forward may be absent.

"sandwich": a norm in front of and behind each sublayer, h <- h + norm_b(mixer(norm_a(h))); h <- h + norm_d(feed_forward(
norm_c(h))), on one float32 stream.  A sublayer's output is handed on un-normed (``deferred.Normed``), so that "norm the
output, add it, norm the stream for the next sublayer" is one kernel; the feed-forward may be absent.

An arrangement declares the parts it works with as ``slots`` (slot name -> family; all needed)
and ``optional_slots``; the decoder builds what the layer's spec lists under those names and
hands the arrangement a layer whose attributes they are.  ``forward(layer, x, residual, ctx)``
gets the last sublayer's output ``x`` (None in front of the first layer) and the float32
residual stream, and returns its own last sublayer's output, not yet added to the stream.

Values between parts may be *pending* (``tandem_b200.kernels.deferred``): a product that its
norm will have added into the residual by the product's own kernel, a norm whose rows' scale the
product behind it applies.  Only parts that declare ``takes_deferred = True`` are handed such
values or asked for them (``forward(..., defer=True)``); an arrangement that declares it may get a
pending ``x`` and return one.
"""

from __future__ import annotations

from typing import Optional

import torch

from tandem_b200.kernels import deferred
from tandem_b200.parts.base import StepContext


def lazy(part) -> bool:
    return getattr(part, "takes_deferred", False)


def normed(norm, x, residual: torch.Tensor, ctx: StepContext, reader):
    """``norm`` applied to residual + x for the part ``reader``; pending where both can deal with it."""
    if lazy(norm):
        return norm.forward(x, residual, ctx.dtype, defer=lazy(reader))
    return norm.forward(deferred.tensor(x), residual, ctx.dtype)


def run(part, h, ctx: StepContext):
    """A mixer or feed-forward on ``h``; its last product may come back pending if the part knows how."""
    return part.forward(h, ctx, defer=True) if lazy(part) else part.forward(deferred.tensor(h), ctx)


class PreNormBlock:
    slots = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}
    takes_deferred = True

    def forward(self, layer, x, residual: torch.Tensor, ctx: StepContext):
        h = normed(layer.mixer_norm, x, residual, ctx, layer.mixer)
        a = run(layer.mixer, h, ctx)
        h = normed(layer.feed_forward_norm, a, residual, ctx, layer.feed_forward)
        return run(layer.feed_forward, h, ctx)


class ParallelBlock:
    slots = {"norm": "norm", "mixer": "mixer"}
    optional_slots = {"feed_forward": "feed_forward"}
    takes_deferred = True

    @staticmethod
    def _terms(value, ctx: StepContext):
        """(float32 tensor, bias or None) of a sublayer's output."""
        if isinstance(value, deferred.Unsummed):
            return value.product, value.bias
        t = deferred.tensor(value)
        return (t if t.dtype == torch.float32 else t.float()), None

    def forward(self, layer, x, residual: torch.Tensor, ctx: StepContext):
        from tandem_b200.kernels import ops

        h = layer.norm.forward(deferred.tensor(x), residual, ctx.dtype)  # two readers: the norm is made whole
        a, a_bias = self._terms(run(layer.mixer, h, ctx), ctx)
        f, f_bias = (None, None)
        if getattr(layer, "feed_forward", None) is not None:
            f, f_bias = self._terms(run(layer.feed_forward, h, ctx), ctx)
        ops.add_pair(residual, a, a_bias, f, f_bias)
        return None  # everything is in the stream already


class ConnectedBlock:
    slots = {"mixer_norm": "norm", "mixer": "mixer", "mixer_link": "connection"}
    optional_slots = {"feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_link": "connection"}
    takes_deferred = True  # x is None or the write that the layer in front left pending

    def forward(self, layer, x, residual: torch.Tensor, ctx: StepContext):
        if x is not None and not isinstance(x, deferred.StreamWrite):
            raise TypeError("a connected layer follows only layers of its kind: what comes in must be a pending write "
                            "into the streams")
        h = layer.mixer_norm.forward(x, residual, ctx.dtype, read=layer.mixer_link.read)
        x = layer.mixer_link.write(deferred.tensor(layer.mixer.forward(h, ctx)))
        if getattr(layer, "feed_forward", None) is not None:
            h = layer.feed_forward_norm.forward(x, residual, ctx.dtype, read=layer.feed_forward_link.read)
            x = layer.feed_forward_link.write(deferred.tensor(layer.feed_forward.forward(h, ctx)))
        return x


class PostNormBlock:
    """Norms behind the sublayers.  Everything is in the stream when the layer returns (it returns None)."""

    slots = {"mixer": "mixer", "mixer_norm": "norm"}
    optional_slots = {"feed_forward": "feed_forward", "feed_forward_norm": "norm", "mixer_conv": "mixer",
                      "feed_forward_conv": "mixer", "average": "connection"}
    BUFFER = "postnorm.second_stream"

    @staticmethod
    def _float32(y) -> torch.Tensor:
        y = deferred.tensor(y)
        return y if y.dtype == torch.float32 else y.float()

    def forward(self, layer, x, residual: torch.Tensor, ctx: StepContext):
        from tandem_b200.kernels import ops, post_norm

        if x is not None:  # an arrangement of another kind in front left its last output outside the stream
            ops.add_pair(residual, self._float32(x))
        conv1, conv2 = getattr(layer, "mixer_conv", None), getattr(layer, "feed_forward_conv", None)
        average, ff = getattr(layer, "average", None), getattr(layer, "feed_forward", None)
        planes = average.results(ctx, residual) if average is not None else None
        tail = dict(planes=planes, coeff=average.coeff, n_planes=average.count - 1) if average is not None else {}
        if conv1 is not None:
            h = conv1.forward(residual, ctx)
        else:
            h = residual if ctx.dtype == torch.float32 else post_norm.short_conv(residual, None, None, ctx, ctx.dtype)
        y = deferred.tensor(layer.mixer.forward(h, ctx))  # float32 or the step's type: the link reads either
        n1 = layer.mixer_norm
        if ff is None:
            post_norm.link(residual, y, n1.weight, n1.groups, n1.eps, residual, **tail)
            return None
        second = ctx.scratch.get(self.BUFFER)
        if second is None or second.shape != residual.shape:
            second = ctx.scratch[self.BUFFER] = torch.empty_like(residual)
        if conv2 is not None and conv2.fusable:
            h = post_norm.link(residual, y, n1.weight, n1.groups, n1.eps, second, taps=conv2.taps, state=conv2.state(ctx), ctx=ctx,
                               out_dtype=ctx.dtype)
            conv2.keep(second, ctx)
        elif conv2 is not None:  # more taps than the fused kernel keeps in registers
            post_norm.link(residual, y, n1.weight, n1.groups, n1.eps, second)
            h = conv2.forward(second, ctx)
        else:
            post_norm.link(residual, y, n1.weight, n1.groups, n1.eps, second)
            h = second if ctx.dtype == torch.float32 else post_norm.short_conv(second, None, None, ctx, ctx.dtype)
        y = deferred.tensor(ff.forward(h, ctx))
        n2 = layer.feed_forward_norm
        post_norm.link(second, y, n2.weight, n2.groups, n2.eps, residual, **tail)
        return None


class SandwichBlock:
    """Norms on both sides of the sublayers.  What the layer returns is its last sublayer's output with the norm
    behind it still to do (``deferred.Normed``): the next norm in line (the next layer's first, or the model's last)
    norms it, adds it into the stream and norms the stream in one launch."""

    slots = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm"}
    optional_slots = {"feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_post_norm": "norm"}
    takes_deferred = True

    @staticmethod
    def _output(value) -> torch.Tensor:
        """A sublayer's output as a tensor, unrounded where the sublayer left it so."""
        if isinstance(value, deferred.Unsummed) and value.bias is None:
            return value.product
        return deferred.tensor(value)

    @staticmethod
    def _behind(norm, y: torch.Tensor) -> deferred.Normed:
        if getattr(norm, "groups", 1) != 1 or not hasattr(norm, "weight"):
            raise TypeError("the norm behind a sublayer of a sandwich layer is an RMS norm over the whole row")
        return deferred.Normed(y, norm.weight, norm.eps)

    def forward(self, layer, x, residual: torch.Tensor, ctx: StepContext):
        h = normed(layer.mixer_norm, x, residual, ctx, layer.mixer)
        x = self._behind(layer.mixer_post_norm, self._output(run(layer.mixer, h, ctx)))
        ff = getattr(layer, "feed_forward", None)
        if ff is None:
            return x
        if getattr(layer, "feed_forward_norm", None) is None or getattr(layer, "feed_forward_post_norm", None) is None:
            raise TypeError("a sandwich layer with a feed-forward has a norm in front of it and one behind it")
        h = normed(layer.feed_forward_norm, x, residual, ctx, ff)
        return self._behind(layer.feed_forward_post_norm, self._output(run(ff, h, ctx)))
