"""Causal softmax attention whose keys and values are expanded from a cached latent.

A token stores c = RMSNorm(latent) * w (``latent_dim`` numbers) and one rotated key part shared by
all heads; head h's key is [W_uk[h] c | rotated part], its value W_uv[h] c.  The expansion is
never carried out for a cached token: W_uk[h]^T is folded into the query (a small product per
head) and W_uv[h] is applied to the attention output, so the attention kernel sees H query heads
of latent_dim + rotary_dim numbers over one key head whose values are the latents themselves.  It
is the package's attention kernel for keys and values of different sizes (one warp per token and
head in float32, query tiles on the tensor cores for prompt portions and split keys for single
tokens in bfloat16), with no window, cap, bias or sink.  One fused projection (rows [q | down-projection
| gate]) with a float32 result; the gate multiplies the concatenated heads (or every head by one number)
by sigmoid of its own projection of the mixer's input.  Where the queries come through a latent of their
own, the fused projection's first rows make that latent, which is normed and expanded by a second product.
"""

from __future__ import annotations

import torch

from tandem_b200.cache.manager import KVNeed
from tandem_b200.config.model_config import ConfigError
from tandem_b200.config.plan import LatentAttentionSpec, ParamSpec, WeightSource, rotary_table
from tandem_b200.kernels import deferred, ops
from tandem_b200.kernels import latent_attention as kernels
from tandem_b200.kernels import post_norm
from tandem_b200.kernels import sink_attention as attention
from tandem_b200.parts.base import Mixer, StepContext

_SUFFIX = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "g": "g", "o": "o", "dq": "dq",
           "dq_norm": "dq.norm", "uq": "uq"}


def _name(spec, local: str) -> str:
    return f"{spec.prefix}.{dict(spec.names).get(local, _SUFFIX[local])}"


class LatentAttention(Mixer):
    capturable = True  # forward only launches kernels and reads the batch from device arrays

    @staticmethod
    def gate_rows(spec: LatentAttentionSpec) -> int:
        return {"sigmoid": spec.num_heads * spec.value_dim, "sigmoid_head": spec.num_heads}.get(spec.gate, 0)

    @classmethod
    def params(cls, spec: LatentAttentionSpec) -> dict:
        H, W = spec.num_heads, spec.hidden_size
        q, kv, g = H * (spec.head_dim + spec.rotary_dim), spec.latent_dim + spec.rotary_dim, cls.gate_rows(spec)
        first = spec.query_latent_dim or q  # the fused projection's first rows: the queries, or their latent
        sources = [WeightSource(_name(spec, "dq" if spec.query_latent_dim else "q"), 0, first), WeightSource(_name(spec, "dkv"), first, kv)]
        if g:
            sources.append(WeightSource(_name(spec, "g"), first + kv, g))
        out = {
            "in": ParamSpec((first + kv + g, W), tuple(sources)),
            "dkv_norm": ParamSpec((spec.latent_dim,), (WeightSource(_name(spec, "dkv_norm")),), role="vector"),
            "uk": ParamSpec((H * spec.head_dim, spec.latent_dim), (WeightSource(_name(spec, "uk")),)),
            "uv": ParamSpec((H * spec.value_dim, spec.latent_dim), (WeightSource(_name(spec, "uv")),)),
            "o": ParamSpec((W, H * spec.value_dim), (WeightSource(_name(spec, "o")),)),
        }
        if spec.query_latent_dim:
            out["dq_norm"] = ParamSpec((spec.query_latent_dim,), (WeightSource(_name(spec, "dq_norm")),), role="vector")
            out["uq"] = ParamSpec((q, spec.query_latent_dim), (WeightSource(_name(spec, "uq")),))
        return out

    @staticmethod
    def kv_need(spec: LatentAttentionSpec) -> KVNeed:
        return KVNeed(1, spec.latent_dim + spec.rotary_dim, None, value_dim=spec.latent_dim)

    def __init__(self, spec: LatentAttentionSpec, weights: dict, dtype: torch.dtype, device) -> None:
        rd = spec.rotated_dims or spec.rotary_dim
        if rd % 2 or rd > spec.rotary_dim:
            raise ConfigError(f"{rd} rotated dims must be even and at most the rotated part of {spec.rotary_dim}")
        if spec.gate not in ("sigmoid", "sigmoid_head", "none"):
            raise ConfigError(f"no gate {spec.gate!r} (sigmoid, sigmoid_head or none)")
        if spec.rotary_pairing not in ("half", "interleaved"):
            raise ConfigError(f"no rotary pairing {spec.rotary_pairing!r} (half or interleaved)")
        self.spec, self.w = spec, weights
        self.freq, self.magnitude = None, 1.0
        if rd:
            freq, self.magnitude = rotary_table(rd, spec.rotary_base, spec.rotary_scaling)
            self.freq = torch.tensor(freq, dtype=torch.float64).to(torch.float32).to(device)

    def _shape(self) -> tuple:
        """(query heads per key head, key size, value size, floats in a query row) as the attention kernels see them."""
        s = self.spec
        dk = s.latent_dim + s.rotary_dim
        return s.num_heads, dk, s.latent_dim, s.num_heads * dk

    def _tiles_key(self):
        return ("sink_attention_tiles", self.spec.num_heads)

    def step_arrays(self, ctx: StepContext, out: dict) -> None:
        """Steps that bring prompt portions run the tensor-core kernel where it takes the shape; its query
        tiles are cut here, once per step for all layers with as many query heads per key head."""
        groups, dk, dv, cols = self._shape()
        key = self._tiles_key()
        if key in out or ctx.max_new < 2 or not attention.tiles_apply(ctx.dtype, dk, dv, groups, cols):
            return
        out[key] = attention.plan_tiles(ctx.host_starts, ctx.host_lens, groups)

    def step_array_capacity(self, bucket: int, max_model_len: int, page_size: int, out: dict) -> None:
        """Steps of single tokens need no arrays."""

    def forward(self, x, ctx: StepContext, defer: bool = False):
        s, w = self.spec, self.w
        H, d, r, R, dv = s.num_heads, s.head_dim, s.rotary_dim, s.latent_dim, s.value_dim
        x = deferred.tensor(x)
        proj = ops.linear(x, w["in"], out_dtype=torch.float32)
        kv = ctx.kv(self)
        first = s.query_latent_dim or H * (d + r)
        queries = None
        if s.query_latent_dim:
            latent = post_norm.group_norm(proj[:, :first], w["dq_norm"], 1, s.norm_eps, ctx.dtype)
            queries = ops.linear(latent, w["uq"], out_dtype=torch.float32)
        q = kernels.prepare(proj, first, w["dkv_norm"], self.freq, ctx.positions, kv, H, d, r, R, s.norm_eps, queries=queries,
                            interleaved=s.rotary_pairing == "interleaved", magnitude=self.magnitude)
        q_in = proj if queries is None else queries
        kernels.head_linear(q_in, d + r, w["uk"], q.view(-1, H * (R + r)), R + r, H, R, d, transposed=True)
        groups, dk, dvl, cols = self._shape()
        q2 = q.view(-1, cols)
        tiles = ctx.extras.get(self._tiles_key())
        if tiles is not None and attention.tiles_apply(kv.k.dtype, dk, dvl, groups, cols):
            o = attention.attend_tiles(q2, kv, tiles, H, 1, dk, dvl, None, 0, s.scale, None, None, None)
        elif ctx.max_new == 1 and attention.split_applies(kv.k.dtype, dk, dvl, groups, cols):
            o = attention.attend_split(q2, kv, ctx, H, 1, dk, dvl, None, 0, s.scale, None, None, None)
        else:
            o = attention.attend(q2, kv, ctx, H, 1, dk, dvl, None, 0, s.scale, None, None, None)
        heads = torch.empty((o.shape[0], H * dv), dtype=torch.float32, device=o.device)
        kernels.head_linear(o, R, w["uv"], heads, dv, H, dv, R, transposed=False)
        gate = proj[:, first + R + r:] if s.gate != "none" else None
        y = kernels.sigmoid_gate(heads, gate, ctx.dtype, per=dv if s.gate == "sigmoid_head" else 1)
        return ops.linear(y, w["o"], out_dtype=torch.float32)
