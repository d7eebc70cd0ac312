"""Grouped-query attention over a sliding window with prepared queries and keys: projection biases, a short
causal convolution over time, a weighted norm per head or over all heads, a partial rotation with optional
slowed frequencies; values of their own or the keys as projected; capped scores, a constant softmax sink, a
sigmoid gate per head; keys and values of its own or another run's.  Every option is a field of
:class:`~tandem_b200.config.plan.WindowAttentionSpec`; the mixer does not know which model it serves.

One fused projection (rows [q | k | v | gate]) with a float32 result; one kernel does bias, convolution, norm
and rotation and stores k and v (``sink_attention.prepare_rows``); the attention itself is the package's windowed
attention over the paged cache (``kernels/sink_attention.py``: one warp per token and head in float32 and wherever
the others do not take the shape, query tiles on the tensor cores for bfloat16 steps that bring prompt portions,
a token's keys cut over several blocks for bfloat16 steps of single tokens), which multiplies each head by its
gate on the way out.  The output projection comes back in float32: the arrangement norms it before it is added.
"""

from __future__ import annotations

import torch

from tandem_b200.cache.manager import KVNeed
from tandem_b200.config.model_config import ConfigError
from tandem_b200.config.plan import ParamSpec, WeightSource, WindowAttentionSpec, rotary_band_table
from tandem_b200.kernels import deferred, ops, post_norm
from tandem_b200.kernels import sink_attention as kernels
from tandem_b200.parts.base import Mixer, StateNeed, StepContext


def _columns(spec: WindowAttentionSpec) -> tuple:
    """(q, k, v, gate) columns of the fused projection."""
    q = spec.num_heads * spec.head_dim
    k = 0 if spec.borrows_kv else spec.num_kv_heads * spec.head_dim
    v = 0 if spec.borrows_kv or spec.values == "keys" else spec.num_kv_heads * spec.value_dim
    g = spec.num_heads if spec.gate == "sigmoid_head" else 0
    return q, k, v, g


class WindowAttention(Mixer):
    capturable = True  # forward only launches kernels and reads the batch from device arrays
    takes_deferred = True

    @staticmethod
    def params(spec: WindowAttentionSpec) -> dict:
        p, H = spec.prefix, spec.hidden_size
        q, k, v, g = _columns(spec)
        sources, at = [], 0
        for name, rows in (("q", q), ("k", k), ("v", v), ("g", g)):
            if rows:
                sources.append(WeightSource(f"{p}.{name}", at, rows))
                at += rows
        out = {"in": ParamSpec((at, H), tuple(sources)),
               "o": ParamSpec((H, spec.num_heads * spec.value_dim), (WeightSource(f"{p}.o"),))}
        if spec.bias:
            b = [WeightSource(f"{p}.q.b", 0, q)] + ([WeightSource(f"{p}.k.b", q, k)] if k else [])
            out["bias"] = ParamSpec((q + k,), tuple(b), role="vector")
        if spec.conv_taps >= 1:
            t, at = [], 0
            for name, rows in (("q", q), ("k", k), ("v", v)):
                if rows:
                    t.append(WeightSource(f"{p}.{name}.conv", at, rows))
                    at += rows
            out["taps"] = ParamSpec((at, spec.conv_taps), tuple(t), role="vector")
        if spec.qk_norm in ("head", "whole"):
            out["q_norm"] = ParamSpec((spec.head_dim if spec.qk_norm == "head" else q,), (WeightSource(f"{p}.q.norm"),), role="vector")
            if k:
                out["k_norm"] = ParamSpec((spec.head_dim if spec.qk_norm == "head" else k,), (WeightSource(f"{p}.k.norm"),), role="vector")
        return out

    @staticmethod
    def kv_need(spec: WindowAttentionSpec) -> KVNeed:
        window = spec.window
        if spec.cache_window is not None and window is not None:  # other runs read this cache through their own windows
            window = None if spec.cache_window == 0 else max(window, spec.cache_window)
        return KVNeed(spec.num_kv_heads, spec.head_dim, window, value_dim=spec.value_dim)

    @staticmethod
    def state_need(spec: WindowAttentionSpec):
        q, k, v, _ = _columns(spec)
        return StateNeed((spec.conv_taps - 1, q + k + v), torch.float32) if spec.conv_taps > 1 else None

    def __init__(self, spec: WindowAttentionSpec, weights: dict, dtype: torch.dtype, device) -> None:
        if spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads:
            raise ConfigError(f"{spec.num_heads} query heads cannot share {spec.num_kv_heads} kv heads")
        if spec.window is not None and spec.window <= 0:
            raise ConfigError(f"a window of {spec.window} keys shows a token nothing")
        if spec.qk_norm not in kernels.QK_NORMS:
            raise ConfigError(f"no norm {spec.qk_norm!r} of queries and keys (have {sorted(kernels.QK_NORMS)})")
        if spec.values not in ("projection", "keys") or (spec.values == "keys" and spec.value_dim != spec.head_dim):
            raise ConfigError(f"values {spec.values!r} of size {spec.value_dim} beside keys of {spec.head_dim}: values are a "
                              "projection of their own, or the keys (then of the keys' size)")
        if spec.gate not in ("none", "sigmoid_head"):
            raise ConfigError(f"no gate {spec.gate!r} (sigmoid_head or none)")
        if spec.rotary_dim % 2 or not 0 <= spec.rotary_dim <= spec.head_dim:
            raise ConfigError(f"{spec.rotary_dim} rotated numbers must be even and at most the head's {spec.head_dim}")
        if spec.conv_taps < 0:
            raise ConfigError(f"a convolution of {spec.conv_taps} taps")
        self.spec = spec
        self.w_in, self.o = weights["in"], weights["o"]
        self.bias = weights.get("bias")
        q, k, v, _ = _columns(spec)
        if self.bias is not None and v:  # the value columns have no bias: the kernel takes one number per column
            self.bias = torch.cat([self.bias, torch.zeros(v, dtype=torch.float32, device=self.bias.device)])
        self.taps = weights.get("taps")
        if self.taps is not None:  # [columns, taps] in the checkpoint; the kernel reads a tap of neighbouring columns side by side
            self.taps = self.taps.t().contiguous()
        self.q_norm, self.k_norm = weights.get("q_norm"), weights.get("k_norm")
        self.freq = None
        if spec.rotary_dim:
            freq = rotary_band_table(spec.rotary_dim, spec.rotary_base, spec.rotary_scaling)
            self.freq = torch.tensor(freq, dtype=torch.float64).to(torch.float32).to(device)
        self.sink = None
        if spec.sink is not None:
            self.sink = torch.full((spec.num_heads,), float(spec.sink), dtype=torch.float32, device=device)

    def _tiles_key(self):
        return ("sink_attention_tiles", self.spec.num_heads // self.spec.num_kv_heads)

    def step_arrays(self, ctx: StepContext, out: dict) -> None:
        """Steps that bring prompt portions run the tensor-core kernel where it takes the shape: its query tiles
        are cut here, once per step for all layers with as many query heads per kv head."""
        s, key = self.spec, self._tiles_key()
        if key in out or ctx.max_new < 2 or \
                not kernels.tiles_apply(ctx.dtype, s.head_dim, s.value_dim, s.num_heads // s.num_kv_heads, s.num_heads * s.head_dim):
            return
        out[key] = kernels.plan_tiles(ctx.host_starts, ctx.host_lens, s.num_heads // s.num_kv_heads)

    def step_array_capacity(self, bucket: int, max_model_len: int, page_size: int, out: dict) -> None:
        """Steps of single tokens (the ones CUDA graphs capture) need no arrays."""

    def forward(self, x, ctx: StepContext, defer: bool = False):
        s = self.spec
        x = deferred.tensor(x)
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
        kv = ctx.kv(self)
        q_cols, k_cols, v_cols, g_cols = _columns(s)
        state = ctx.state(self) if s.conv_taps > 1 else None
        q = kernels.prepare_rows(proj, kv, ctx, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, bias=self.bias,
                                 taps=self.taps, state=state, qk_norm=s.qk_norm, q_weight=self.q_norm, k_weight=self.k_norm,
                                 eps=s.norm_eps, freq=self.freq, has_kv=not s.borrows_kv, values_from_keys=s.values == "keys")
        if state is not None:  # after the kernel that read the old rows
            post_norm.short_conv_state(proj, state, ctx, s.conv_taps, width=q_cols + k_cols + v_cols)
        gate = proj[:, q_cols + k_cols + v_cols:] if g_cols else None
        groups, cols = s.num_heads // s.num_kv_heads, q.shape[1]
        args = (s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, s.window, 0, s.scale, s.softcap, None, self.sink)
        tiles = ctx.extras.get(self._tiles_key())
        if tiles is not None and kernels.tiles_apply(kv.k.dtype, s.head_dim, s.value_dim, groups, cols):
            o = kernels.attend_tiles(q, kv, tiles, *args, gate=gate)
        elif ctx.max_new == 1 and kernels.split_applies(kv.k.dtype, s.head_dim, s.value_dim, groups, cols):
            o = kernels.attend_split(q, kv, ctx, *args, gate=gate)
        else:
            o = kernels.attend(q, kv, ctx, *args, gate=gate)
        return ops.linear(o, self.o, out_dtype=torch.float32)
