"""RMSNorm with the residual add fused in front of it, and the RMS norm in equal groups of a row.

y = weight * x * rsqrt(mean(x^2) + eps), all in float32
(12vivi/tandem python/tandem/layers/norm.py:15-19, python/tandem/layers/ops.py:29-42); the
residual stream it adds into is float32 in both modes.
"""

from __future__ import annotations

from typing import Optional

import torch

from tandem_b200.config.plan import NormSpec, ParamSpec, WeightSource
from tandem_b200.kernels import ops
from tandem_b200.parts.base import Norm


class RMSNorm(Norm):
    takes_deferred = True  # x may be a product that is still pending; the result may stay pending (kernels/deferred.py)

    @staticmethod
    def params(spec: NormSpec) -> dict:
        return {"weight": ParamSpec((spec.size,), (WeightSource(spec.weight),), role="vector")}

    def __init__(self, spec: NormSpec, weights: dict, dtype: torch.dtype, device) -> None:
        self.eps = spec.eps
        self.weight = weights["weight"]
        if spec.offset:  # a weight stored around zero: the sum is made once, in float32
            self.weight = self.weight + float(spec.offset)
        self.groups = 1  # one run: the whole row (what an arrangement with norms on the sublayers' output reads)

    def forward(self, x, residual: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                defer: bool = False, read: Optional[torch.Tensor] = None):
        """``read``: the residual is several streams side by side and the norm's input is their sum weighted by
        these coefficients; ``x`` is then None or the write into the streams that is still pending."""
        if read is not None:
            return ops.stream_norm(residual, x, read, self.weight, self.eps, out_dtype, rows)
        return ops.add_rmsnorm(x, residual, self.weight, self.eps, out_dtype, rows, defer=defer)


class GroupRMSNorm(Norm):
    """The row in ``groups`` equal consecutive runs, each divided by its own sqrt(mean(run^2) + eps), the whole times
    the weight; float32 arithmetic.  As a norm in FRONT of a sublayer it adds ``x`` into the stream and norms the
    stream's rows; an arrangement whose norms sit on the sublayers' output reads ``weight``, ``groups`` and ``eps`` and
    has the norm done inside the kernel that adds the output into the stream (``kernels/post_norm.py``)."""

    @staticmethod
    def params(spec: NormSpec) -> dict:
        return {"weight": ParamSpec((spec.size,), (WeightSource(spec.weight),), role="vector")}

    def __init__(self, spec: NormSpec, weights: dict, dtype: torch.dtype, device) -> None:
        from tandem_b200.config.model_config import ConfigError

        if spec.groups <= 0 or spec.size % spec.groups:
            raise ConfigError(f"a norm over {spec.size} numbers in {spec.groups} groups: the groups must be equal")
        self.eps, self.groups = spec.eps, spec.groups
        self.weight = weights["weight"]

    def forward(self, x, residual: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None):
        from tandem_b200.kernels import post_norm

        if x is not None:
            ops.add_pair(residual, x if x.dtype == torch.float32 else x.float())
        return post_norm.group_norm(residual, self.weight, self.groups, self.eps, out_dtype, rows=rows)

    def in_place(self, stream: torch.Tensor) -> torch.Tensor:
        """The rows of a float32 stream replaced by their norm."""
        from tandem_b200.kernels import post_norm

        return post_norm.group_norm(stream, self.weight, self.groups, self.eps, torch.float32, out=stream)
