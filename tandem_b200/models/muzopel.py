"""Muzopel: configuration -> model plan, and its random-weight recipe.

Every layer is a "postnorm" arrangement: a short convolution in front of the mixer (``l<i>.canon1``), the mixer
(``l<i>.mix.*``), the norm on its output (``l<i>.norm1``), and the same for the feed-forward where the layer has one
(``l<i>.canon2``, ``l<i>.mlp.*``, ``l<i>.norm2``); behind the layer the depth average (``l<i>.dwa``, i + 2 numbers).
Both kinds of mixer are the package's ``latent_attention`` part: "latent_attention" with a latent for the queries
(``.dq``, ``.dq.norm``, ``.uq``), frequencies stretched as the file says and a sigmoid gate per head (``.g``);
"latent_attention_2" with plain queries (``.q``), no gate.  Both rotate interleaved pairs.  The feed-forward is
``routed_mlp`` with softmax scores that are not renormalised, a bias on the choice (``.correction``), experts
down(gelu(up x)) and identity experts behind them.  The embedded rows are normed (``embed.norm``), all norms are RMS
norms in ``norm.groups`` equal runs of the row, the logits are soft-capped, and there is no table of positions.
"""

from __future__ import annotations

from typing import Iterator

import torch

from tandem_b200.config.muzopel_config import NO_POSITION_LIMIT, MuzopelConfig
from tandem_b200.config.plan import (
    DepthAverageSpec,
    EmbeddingSpec,
    HeadSpec,
    LatentAttentionSpec,
    LayerSpec,
    ModelPlan,
    NormSpec,
    RotaryScalingSpec,
    RoutedMLPSpec,
    RunStep,
    ShortConvolutionSpec,
)
from tandem_b200.registry import Architecture, register_architecture


def mixer_spec(cfg: MuzopelConfig, i: int) -> LatentAttentionSpec:
    L, m = cfg.layers[i], cfg.layers[i].mixer
    sc = m.scaling
    return LatentAttentionSpec(
        "latent_attention", prefix=f"l{i}.mix", hidden_size=cfg.width, num_heads=m.heads, head_dim=m.dim, rotary_dim=m.rot_dim,
        rotated_dims=m.rot_dims, rotary_base=m.rot_base, value_dim=m.vdim, latent_dim=m.kv_rank, scale=m.scale,
        norm_eps=cfg.norm_eps, gate="sigmoid_head" if L.type == "latent_attention" else "none", rotary_pairing="interleaved",
        rotary_scaling=None if sc is None else RotaryScalingSpec(sc.factor, sc.original, sc.fast, sc.slow),
        query_latent_dim=m.q_rank)


def feed_forward_spec(cfg: MuzopelConfig, i: int) -> RoutedMLPSpec:
    mlp = cfg.layers[i].mlp
    return RoutedMLPSpec("routed_mlp", prefix=f"l{i}.mlp", hidden_size=cfg.width, intermediate_size=mlp.ff, num_experts=mlp.experts,
                         top_k=mlp.top, score="softmax", normalize=False, route_scale=1.0, activation="gelu", gated=False,
                         identity_experts=mlp.identity, choice_bias="correction")


def build_plan(cfg: MuzopelConfig) -> ModelPlan:
    n = len(cfg.layers)

    def norm(name: str) -> NormSpec:
        return NormSpec("group_rmsnorm", cfg.width, cfg.norm_eps, name, groups=cfg.norm_groups)

    def conv(name: str) -> ShortConvolutionSpec:
        return ShortConvolutionSpec("short_convolution", hidden_size=cfg.width, taps=cfg.taps, weight=name)

    layers = []
    for i, L in enumerate(cfg.layers):
        slots = dict(mixer_conv=conv(f"l{i}.canon1"), mixer=mixer_spec(cfg, i), mixer_norm=norm(f"l{i}.norm1"))
        if L.mlp is not None:
            slots.update(feed_forward_conv=conv(f"l{i}.canon2"), feed_forward=feed_forward_spec(cfg, i),
                         feed_forward_norm=norm(f"l{i}.norm2"))
        slots["average"] = DepthAverageSpec("depth_average", count=i + 2, weight=f"l{i}.dwa", total=n + 1)
        layers.append(LayerSpec.of("postnorm", **slots))
    return ModelPlan(
        embedding=EmbeddingSpec(cfg.vocab, cfg.width, "embed", norm=norm("embed.norm")),
        layers=tuple(layers),
        order=tuple(RunStep(i) for i in range(n)),
        final_norm=norm("final.norm"),
        head=HeadSpec(cfg.vocab, cfg.width, "head", softcap=cfg.logit_softcap),
        max_position=NO_POSITION_LIMIT,
        eos_token_ids=tuple(cfg.eos_token_ids),
    )


def tensor_shapes(cfg: MuzopelConfig) -> dict:
    """Checkpoint tensor name -> shape, in file order."""
    W = cfg.width
    shapes: dict = {"embed": (cfg.vocab, W), "embed.norm": (W,)}
    for i, L in enumerate(cfg.layers):
        m, p = L.mixer, f"l{i}.mix"
        shapes[f"l{i}.norm1"] = (W,)
        if L.mlp is not None:
            shapes[f"l{i}.norm2"] = (W,)
        q = m.heads * (m.dim + m.rot_dim)
        if m.q_rank:
            shapes[f"{p}.dq"] = (m.q_rank, W)
            shapes[f"{p}.dq.norm"] = (m.q_rank,)
            shapes[f"{p}.uq"] = (q, m.q_rank)
        else:
            shapes[f"{p}.q"] = (q, W)
        shapes[f"{p}.dkv"] = (m.kv_rank + m.rot_dim, W)
        shapes[f"{p}.dkv.norm"] = (m.kv_rank,)
        shapes[f"{p}.uk"] = (m.heads * m.dim, m.kv_rank)
        shapes[f"{p}.uv"] = (m.heads * m.vdim, m.kv_rank)
        if L.type == "latent_attention":
            shapes[f"{p}.g"] = (m.heads, W)
        shapes[f"{p}.o"] = (W, m.heads * m.vdim)
        if L.mlp is not None:
            for e in range(L.mlp.experts):
                shapes[f"l{i}.mlp.e{e}.up"] = (L.mlp.ff, W)
                shapes[f"l{i}.mlp.e{e}.down"] = (W, L.mlp.ff)
            shapes[f"l{i}.mlp.router"] = (L.mlp.experts + L.mlp.identity, W)
            shapes[f"l{i}.mlp.correction"] = (L.mlp.experts + L.mlp.identity,)
        shapes[f"l{i}.canon1"] = (W, cfg.taps)
        if L.mlp is not None:
            shapes[f"l{i}.canon2"] = (W, cfg.taps)
        shapes[f"l{i}.dwa"] = (i + 2,)
    shapes["final.norm"] = (W,)
    shapes["head"] = (cfg.vocab, W)
    return shapes


def random_weights(cfg: MuzopelConfig, seed: int, device: str = "cpu", dtype: torch.dtype = torch.bfloat16,
                   std: float = 0.02, norm_spread: float = 0.1) -> Iterator[tuple]:
    """Seeded random tensors by checkpoint name, each from a generator of its own: matrices N(0, std) (the embedding
    N(0, 1); the router N(0, 1.5 / sqrt(width)), so that scores spread without saturating), norm weights 1 + U(-spread,
    spread) (those on a sublayer's output 0.5 + U: the stream grows slowly with depth), the choice bias N(0, 0.05),
    convolution taps N(0, 0.3), the depth average's coefficients the newest result 0.7 + N(0, 0.05) and the rest
    sharing 0.3 + N(0, 0.05)."""
    for index, (name, shape) in enumerate(tensor_shapes(cfg).items()):
        g = torch.Generator(device=device).manual_seed((seed * 1_000_003 + index) % (2**63 - 1))

        def normal(mean: float, sd: float) -> torch.Tensor:
            return torch.empty(shape, device=device, dtype=torch.float32).normal_(mean, sd, generator=g)

        def uniform(lo: float, hi: float) -> torch.Tensor:
            return lo + (hi - lo) * torch.rand(shape, generator=g, device=device, dtype=torch.float32)

        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2"):
            t = uniform(0.5 - norm_spread, 0.5 + norm_spread)
        elif leaf == "norm":
            t = uniform(1.0 - norm_spread, 1.0 + norm_spread)
        elif leaf in ("canon1", "canon2"):
            t = normal(0.0, 0.3)
        elif leaf == "dwa":
            t = normal(0.3 / (shape[0] - 1), 0.05 / (shape[0] - 1))
            t[-1] = 0.7 + 0.05 * float(torch.randn((), generator=g, device=device))
        elif leaf == "router":
            t = normal(0.0, 1.5 / cfg.width ** 0.5)
        elif leaf == "correction":
            t = normal(0.0, 0.05)
        elif name == "embed":
            t = normal(0.0, 1.0)
        else:
            t = normal(0.0, std)
        yield name, t.to(dtype)


register_architecture(Architecture("Muzopel", MuzopelConfig, build_plan, random_weights))
