"""Deletar: configuration -> model plan, and its random-weight recipe.

Every layer is a "sandwich" arrangement: a norm in front of the mixer (``l<i>.norm1``), the mixer (``l<i>.mix.*``), a
norm behind it (``l<i>.norm1b``), and the same for the feed-forward where the layer has one (``l<i>.norm2``,
``l<i>.mlp.*``, ``l<i>.norm2b``); all norms are RMS norms whose stored weight w stands for 1 + w.  The three mixers are
the package's ``window_attention`` part with three sets of options:

  "attention"    a convolution over time on q, k and v (``.q.conv`` ...), no norm of q and k, no cap, no gate;
  "attention_2"  biases on q and k, one norm over all heads of q (of k), the keys as projected for values (no ``.v``),
                 capped scores, a sigmoid gate per head (``.g``);
  "attention_3"  a norm per head with one weight for all heads, rotation frequencies slowed by wavelength where the file
                 says so, capped scores, one added to the softmax denominator, a gate per head; with ``kv_from`` the
                 layer has no key and value tensors and its run reads the named layer's cache.

The feed-forward is ``dense_mlp`` or ``routed_mlp`` with the relu2 activation, no gate and no biases; the experts of a
token are named by ``.table`` [vocab, top] and weigh 1 / top each; ``.shared`` is the expert every token passes.  The
embedding is scaled, the logits are soft-capped, and there is no table of positions.
"""

from __future__ import annotations

from typing import Iterator

import torch

from tandem_b200.config.deletar_config import NO_POSITION_LIMIT, DeletarConfig
from tandem_b200.config.plan import (
    DenseMLPSpec,
    EmbeddingSpec,
    HeadSpec,
    LayerSpec,
    ModelPlan,
    NormSpec,
    RotaryBandSpec,
    RoutedMLPSpec,
    RunStep,
    WindowAttentionSpec,
)
from tandem_b200.registry import Architecture, register_architecture


def cache_window(cfg: DeletarConfig, i: int):
    """How many keys layer i's cache must keep where layers that read it look further back than layer i itself:
    None where nobody reads it, 0 where a reader sees all keys."""
    readers = [L.mixer for L in cfg.layers if L.mixer.kv_from == i]
    if not readers:
        return None
    if any(m.window is None for m in readers):
        return 0
    return max(m.window for m in readers)


def mixer_spec(cfg: DeletarConfig, i: int) -> WindowAttentionSpec:
    L, m = cfg.layers[i], cfg.layers[i].mixer
    sc = m.scaling
    common = dict(prefix=f"l{i}.mix", hidden_size=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim,
                  value_dim=m.vdim, scale=m.scale, norm_eps=cfg.norm_eps, rotary_dim=m.rot_dims, rotary_base=m.rot_base,
                  rotary_scaling=None if sc is None else RotaryBandSpec(sc.factor, sc.low, sc.high, sc.original),
                  softcap=m.softcap, window=m.window, cache_window=cache_window(cfg, i))
    if L.type == "attention":
        return WindowAttentionSpec("window_attention", conv_taps=m.conv, **common)
    if L.type == "attention_2":
        return WindowAttentionSpec("window_attention", bias=True, qk_norm="whole", values="keys", gate="sigmoid_head", **common)
    return WindowAttentionSpec("window_attention", qk_norm="head", sink=0.0, gate="sigmoid_head", borrows_kv=m.kv_from is not None,
                               **common)


def feed_forward_spec(cfg: DeletarConfig, i: int):
    mlp = cfg.layers[i].mlp
    if mlp.kind == "dense":
        return DenseMLPSpec("dense_mlp", prefix=f"l{i}.mlp", hidden_size=cfg.width, intermediate_size=mlp.ff, activation="relu2",
                            bias=False)
    return RoutedMLPSpec("routed_mlp", prefix=f"l{i}.mlp", hidden_size=cfg.width, intermediate_size=mlp.ff, num_experts=mlp.experts,
                         top_k=mlp.top, activation="relu2", gated=False, router="token_table", table="table", vocab_size=cfg.vocab,
                         shared_intermediate_size=mlp.shared_ff)


def build_plan(cfg: DeletarConfig) -> ModelPlan:
    def norm(name: str) -> NormSpec:
        return NormSpec("rmsnorm", cfg.width, cfg.norm_eps, name, offset=1.0)

    layers = []
    for i, L in enumerate(cfg.layers):
        slots = dict(mixer_norm=norm(f"l{i}.norm1"), mixer=mixer_spec(cfg, i), mixer_post_norm=norm(f"l{i}.norm1b"))
        if L.mlp is not None:
            slots.update(feed_forward_norm=norm(f"l{i}.norm2"), feed_forward=feed_forward_spec(cfg, i),
                         feed_forward_post_norm=norm(f"l{i}.norm2b"))
        layers.append(LayerSpec.of("sandwich", **slots))
    return ModelPlan(
        embedding=EmbeddingSpec(cfg.vocab, cfg.width, "embed", scale=cfg.embedding_scale),
        layers=tuple(layers),
        order=tuple(RunStep(i, cache_of=L.mixer.kv_from) for i, L in enumerate(cfg.layers)),
        final_norm=norm("final.norm"),
        head=HeadSpec(cfg.vocab, cfg.width, "head", softcap=cfg.logit_softcap),
        max_position=NO_POSITION_LIMIT,
        eos_token_ids=tuple(cfg.eos_token_ids),
    )


def tensor_shapes(cfg: DeletarConfig) -> dict:
    """Checkpoint tensor name -> shape, in file order."""
    W = cfg.width
    shapes: dict = {"embed": (cfg.vocab, W)}
    for i, L in enumerate(cfg.layers):
        m, p = L.mixer, f"l{i}.mix"
        for n in ("norm1", "norm2", "norm1b", "norm2b"):
            if L.mlp is not None or n.startswith("norm1"):
                shapes[f"l{i}.{n}"] = (W,)
        q, k, v = m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim
        own = m.kv_from is None
        shapes[f"{p}.q"] = (q, W)
        if L.type == "attention_2":
            shapes[f"{p}.q.b"] = (q,)
        if own:
            shapes[f"{p}.k"] = (k, W)
            if L.type == "attention_2":
                shapes[f"{p}.k.b"] = (k,)
            else:
                shapes[f"{p}.v"] = (v, W)
        if L.type == "attention" and m.conv:
            shapes[f"{p}.q.conv"] = (q, m.conv)
            shapes[f"{p}.k.conv"] = (k, m.conv)
            shapes[f"{p}.v.conv"] = (v, m.conv)
        if L.type in ("attention_2", "attention_3"):
            shapes[f"{p}.q.norm"] = (q,) if L.type == "attention_2" else (m.dim,)
            if own:
                shapes[f"{p}.k.norm"] = (k,) if L.type == "attention_2" else (m.dim,)
            shapes[f"{p}.g"] = (m.heads, W)
        shapes[f"{p}.o"] = (W, m.heads * m.vdim)
        if L.mlp is not None and L.mlp.kind == "dense":
            shapes[f"l{i}.mlp.up"] = (L.mlp.ff, W)
            shapes[f"l{i}.mlp.down"] = (W, L.mlp.ff)
        elif L.mlp is not None:
            for e in range(L.mlp.experts):
                shapes[f"l{i}.mlp.e{e}.up"] = (L.mlp.ff, W)
                shapes[f"l{i}.mlp.e{e}.down"] = (W, L.mlp.ff)
            shapes[f"l{i}.mlp.table"] = (cfg.vocab, L.mlp.top)
            if L.mlp.shared_ff:
                shapes[f"l{i}.mlp.shared.up"] = (L.mlp.shared_ff, W)
                shapes[f"l{i}.mlp.shared.down"] = (W, L.mlp.shared_ff)
    shapes["final.norm"] = (W,)
    shapes["head"] = (cfg.vocab, W)
    return shapes


def random_weights(cfg: DeletarConfig, seed: int, device: str = "cpu", dtype: torch.dtype = torch.bfloat16,
                   std: float = 0.02, norm_spread: float = 0.1) -> Iterator[tuple]:
    """Seeded random tensors by checkpoint name, each from a generator of its own: matrices N(0, std) (the embedding
    N(0, 1 / scale), the projections of q and k N(0, 4 std) so that scores spread), stored norm weights U(-spread,
    spread) (those behind a sublayer -0.5 + U: the stream grows slowly with depth; those of q and k 1 + U), biases
    N(0, 0.1), convolution taps N(0, 0.5), and per token id ``top`` different experts drawn from a permutation (int32)."""
    for index, (name, shape) in enumerate(tensor_shapes(cfg).items()):
        g = torch.Generator(device=device).manual_seed((seed * 1_000_003 + index) % (2**63 - 1))

        def normal(mean: float, sd: float) -> torch.Tensor:
            return torch.empty(shape, device=device, dtype=torch.float32).normal_(mean, sd, generator=g)

        def uniform(lo: float, hi: float) -> torch.Tensor:
            return lo + (hi - lo) * torch.rand(shape, generator=g, device=device, dtype=torch.float32)

        parts = name.split(".")
        leaf = parts[-1]
        if leaf == "table":
            experts = next(L.mlp.experts for i, L in enumerate(cfg.layers) if name == f"l{i}.mlp.table")
            order = torch.rand((shape[0], experts), generator=g, device=device).argsort(dim=1)
            yield name, order[:, :shape[1]].to(torch.int32).contiguous()
            continue
        if leaf in ("norm1b", "norm2b"):
            t = uniform(-0.5 - norm_spread, -0.5 + norm_spread)
        elif leaf in ("norm1", "norm2") or name == "final.norm":
            t = uniform(-norm_spread, norm_spread)
        elif leaf == "norm":
            t = uniform(1.0 - norm_spread, 1.0 + norm_spread)
        elif leaf == "conv":
            t = normal(0.0, 0.5)
        elif leaf == "b":
            t = normal(0.0, 0.1)
        elif name == "embed":
            t = normal(0.0, 1.0 / cfg.embedding_scale)
        elif leaf in ("q", "k"):
            t = normal(0.0, 4.0 * std)
        else:
            t = normal(0.0, std)
        yield name, t.to(dtype)


register_architecture(Architecture("Deletar", DeletarConfig, build_plan, random_weights))
