"""How a sublayer hangs on the residual: the link between the two.

``StreamLink`` keeps the coefficients of one sublayer on a residual of S parallel streams
("hyper-connections"): the sublayer reads u = sum_s in[s] X_s and its output y rewrites every
stream, X_t <- sum_s mix[s, t] X_s + mult * out[t] * y.  Without learned coefficients (one stream,
in = out = mix = 1) it is the plain residual sum with a factor on the sublayer's output.  The
arithmetic runs in the norm's kernel (``ops.stream_norm``): the link only says which numbers.

``DepthAverage`` keeps the coefficients with which a layer hands on a weighted sum of the results of all layers
so far, and the room in which a step keeps those results.
"""

from __future__ import annotations

import torch

from tandem_b200.config.model_config import ConfigError
from tandem_b200.config.plan import DepthAverageSpec, ParamSpec, StreamLinkSpec, WeightSource
from tandem_b200.kernels import deferred


class StreamLink:
    @staticmethod
    def params(spec: StreamLinkSpec) -> dict:
        if spec.prefix is None:
            return {}
        s = spec.streams
        return {"read": ParamSpec((s,), (WeightSource(f"{spec.prefix}.in"),), role="vector"),
                "out": ParamSpec((s,), (WeightSource(f"{spec.prefix}.out"),), role="vector"),
                "mix": ParamSpec((s, s), (WeightSource(f"{spec.prefix}.mix"),), role="vector")}

    def __init__(self, spec: StreamLinkSpec, weights: dict, dtype: torch.dtype, device) -> None:
        if spec.prefix is None and spec.streams != 1:
            raise ConfigError(f"{spec.streams} streams need learned coefficients (a checkpoint prefix)")
        if not 1 <= spec.streams <= 8:
            raise ConfigError(f"a residual of {spec.streams} streams: the kernel takes 1 to 8")
        self.streams, self.mult = spec.streams, float(spec.mult)
        if spec.prefix is None:
            one = torch.ones(1, dtype=torch.float32, device=device)
            self.read, self.out, self.mix = one, one, one.view(1, 1)
        else:
            self.read, self.out, self.mix = weights["read"], weights["out"], weights["mix"]

    def write(self, y: torch.Tensor) -> deferred.StreamWrite:
        """The sublayer's output on its way into the streams."""
        return deferred.StreamWrite(y, self.mix, self.out, self.mult)


class DepthAverage:
    """x <- sum_(j <= n) a[j] Y_j (see :class:`~tandem_b200.config.plan.DepthAverageSpec`).  The results of a step
    live in one float32 tensor [total, T, W] that the first layer of the step makes (Y_0 = the stream as that layer
    receives it) and every later layer finds in the step's scratch; the sum itself runs in the kernel that makes Y_n."""

    KEY = "depth_average.results"

    @staticmethod
    def params(spec: DepthAverageSpec) -> dict:
        return {"coeff": ParamSpec((spec.count,), (WeightSource(spec.weight),), role="vector")}

    def __init__(self, spec: DepthAverageSpec, weights: dict, dtype: torch.dtype, device) -> None:
        if spec.count < 2 or spec.count > spec.total:
            raise ConfigError(f"a depth average over {spec.count} of {spec.total} results")
        self.count, self.total = spec.count, spec.total
        self.coeff = weights["coeff"]

    def results(self, ctx, stream: torch.Tensor) -> torch.Tensor:
        """The step's results so far; the first layer starts them with the stream it was given."""
        if self.count == 2:
            planes = torch.empty((self.total,) + tuple(stream.shape), dtype=torch.float32, device=stream.device)
            planes[0].copy_(stream)
            ctx.scratch[self.KEY] = planes
            return planes
        planes = ctx.scratch.get(self.KEY)
        if planes is None or planes.shape[0] < self.count or tuple(planes.shape[1:]) != tuple(stream.shape):
            raise RuntimeError(f"a depth average over {self.count} results follows layers that kept them")
        return planes
