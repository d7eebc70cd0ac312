"""A short causal convolution over time on every channel of the stream, in front of a sublayer.

h_t = x_t + sum_j w[c, j] x_(t - taps + 1 + j) with zeros in front of a sequence (see
:class:`~tandem_b200.config.plan.ShortConvolutionSpec`).  A request's last ``taps`` - 1 inputs are its state: the
part belongs to the mixer family so that the cache manager gives it a state row per request like any other
part with state, zeroed at admission.  The arithmetic is float32; the result is rounded to the model's type.
The arrangement that uses it may have the convolution done by the kernel that makes its input (``post_norm.link``)
and then only calls :meth:`keep`.
"""

from __future__ import annotations

import torch

from tandem_b200.config.model_config import ConfigError
from tandem_b200.config.plan import ParamSpec, ShortConvolutionSpec, WeightSource
from tandem_b200.kernels import post_norm
from tandem_b200.parts.base import Mixer, StateNeed, StepContext


class ShortConvolution(Mixer):
    capturable = True  # only launches kernels and reads the batch from the context's device arrays
    capturable_portions = True

    @staticmethod
    def params(spec: ShortConvolutionSpec) -> dict:
        return {"taps": ParamSpec((spec.hidden_size, spec.taps), (WeightSource(spec.weight),), role="vector")}

    @staticmethod
    def state_need(spec: ShortConvolutionSpec):
        return StateNeed((spec.taps - 1, spec.hidden_size), torch.float32) if spec.taps > 1 else None

    def __init__(self, spec: ShortConvolutionSpec, weights: dict, dtype: torch.dtype, device) -> None:
        if spec.taps < 1:
            raise ConfigError(f"a convolution of {spec.taps} taps")
        if not spec.skip:
            raise ConfigError("the convolution without its skip term is not built")
        self.num_taps = spec.taps
        self.taps = weights["taps"]
        self.fusable = spec.taps <= post_norm.MAX_TAPS  # the kernel that makes this part's input can run the convolution too

    def state(self, ctx: StepContext):
        return ctx.state(self) if self.num_taps > 1 else None

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """x float32 [T, W] -> x + conv(x) in the model's type, and the state moved on."""
        h = post_norm.short_conv(x, self.taps, self.state(ctx), ctx, ctx.dtype)
        self.keep(x, ctx)
        return h

    def keep(self, x: torch.Tensor, ctx: StepContext) -> None:
        """The requests' newest inputs into their state rows (after the kernel that read the old ones)."""
        post_norm.short_conv_state(x, self.state(ctx), ctx, self.num_taps)
