"""Typed view of a Muzopel ``config.json``.

Muzopel is a decoder whose norms sit on the sublayers' OUTPUT: x <- x + norm(sublayer(x + conv(x))), the norm an RMS
norm in equal groups of the row, conv a short causal convolution per channel.  Its layers are listed one by one; a
layer's mixer is softmax attention over a cached latent, with the queries through a latent of their own, stretched
rotary frequencies and a gate per head ("latent_attention"), or with plain queries, plain frequencies and no gate
("latent_attention_2"); its feed-forward is routed experts without a gate (some router outputs may stand for experts
that return their input) or absent.  What a layer hands on is a learned weighted sum of the results of all layers so
far.  The logits are soft-capped.  Every size and every constant that may differ between models is a key of the
file; nothing here has a default that stands in for a missing size.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from tandem_b200.config.fumanex_config import NO_POSITION_LIMIT, _number
from tandem_b200.config.model_config import ConfigError, _positive_int, _require

MIXER_TYPES = ("latent_attention", "latent_attention_2")
MLP_KINDS = ("moe",)

__all__ = ["MuzopelConfig", "MuzopelLayer", "MuzopelLatent", "MuzopelScaling", "MuzopelExperts", "NO_POSITION_LIMIT"]


def _int(d: dict, key: str, where: str) -> int:
    return _positive_int(d, where + key, _require(d, key))


def _count(d: dict, key: str, where: str) -> int:
    """A count that may be zero or absent."""
    v = d.get(key) or 0
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"config.json: {where}{key!r} must be a non-negative integer, got {v!r}")
    return v


@dataclass(frozen=True)
class MuzopelScaling:
    factor: float
    original: float
    fast: float
    slow: float

    @classmethod
    def from_dict(cls, s: dict, where: str) -> "MuzopelScaling":
        c = cls(*(_number(s, k, where) for k in ("factor", "original", "fast", "slow")))
        if c.factor <= 0 or c.original <= 0 or c.fast <= 0 or c.slow <= 0:
            raise ConfigError(f"config.json: {where}factor, original, fast and slow must be positive")
        return c

    def to_dict(self) -> dict:
        original = int(self.original) if float(self.original).is_integer() else self.original
        return {"factor": self.factor, "original": original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class MuzopelLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float
    q_rank: int = 0  # 0: the queries are one projection of the mixer's input
    scaling: Optional[MuzopelScaling] = None

    @classmethod
    def from_dict(cls, m: dict, where: str, query_latent: bool) -> "MuzopelLatent":
        rot = _require(m, "rot")
        sc = rot.get("scaling")
        c = cls(heads=_int(m, "heads", where), dim=_int(m, "dim", where), rot_dim=_int(m, "rot_dim", where),
                vdim=_int(m, "vdim", where), kv_rank=_int(m, "kv_rank", where), scale=_number(m, "scale", where),
                rot_dims=_int(rot, "dims", where + "rot."), rot_base=_number(rot, "base", where + "rot."),
                q_rank=_int(m, "q_rank", where) if query_latent else 0,
                scaling=None if not sc else MuzopelScaling.from_dict(sc, where + "rot.scaling."))
        if c.rot_dims > c.rot_dim or c.rot_dims % 2:
            raise ConfigError(f"config.json: {where}rot.dims ({c.rot_dims}) must be even and at most rot_dim ({c.rot_dim})")
        if c.rot_base <= 1.0:
            raise ConfigError(f"config.json: {where}rot.base ({c.rot_base}) must exceed 1")
        return c

    def to_dict(self) -> dict:
        rot: dict = {"base": self.rot_base, "dims": self.rot_dims}
        if self.scaling is not None:
            rot["scaling"] = self.scaling.to_dict()
        d = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "rot": rot, "rot_dim": self.rot_dim,
             "scale": self.scale, "vdim": self.vdim}
        if self.q_rank:
            d["q_rank"] = self.q_rank
        return d


@dataclass(frozen=True)
class MuzopelExperts:
    ff: int  # width of one expert
    experts: int  # experts that have tensors
    identity: int  # router outputs behind them that stand for experts returning their input
    top: int

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "MuzopelExperts":
        kind = _require(m, "kind")
        if kind not in MLP_KINDS:
            raise ConfigError(f"config.json: {where}kind {kind!r} is not supported (supported: {list(MLP_KINDS)})")
        router, expert = _require(m, "router"), _require(m, "expert")
        c = cls(ff=_int(expert, "ff", where + "expert."), experts=_int(router, "experts", where + "router."),
                identity=_count(router, "identity", where + "router."), top=_int(router, "top", where + "router."))
        if c.top > c.experts + c.identity:
            raise ConfigError(f"config.json: {where}router.top ({c.top}) exceeds the router's {c.experts + c.identity} outputs")
        return c

    def to_dict(self) -> dict:
        return {"expert": {"ff": self.ff}, "kind": "moe",
                "router": {"experts": self.experts, "identity": self.identity, "top": self.top}}


@dataclass(frozen=True)
class MuzopelLayer:
    type: str
    mixer: MuzopelLatent
    mlp: Optional[MuzopelExperts]

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(), "type": self.type}


@dataclass(frozen=True)
class MuzopelConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    taps: int  # of the convolution in front of every sublayer
    logit_softcap: Optional[float]
    layers: tuple  # of MuzopelLayer
    eos_token_ids: tuple = ()
    extra: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, d: dict) -> "MuzopelConfig":
        entries = _require(d, "layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]."
            kind = _require(e, "type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}type {kind!r} is not supported (supported: {list(MIXER_TYPES)})")
            mixer = MuzopelLatent.from_dict(_require(e, "mixer"), where + "mixer.", query_latent=kind == "latent_attention")
            mlp = e.get("mlp")
            layers.append(MuzopelLayer(kind, mixer, None if mlp is None else MuzopelExperts.from_dict(mlp, where + "mlp.")))
        norm = _require(d, "norm")
        width = _positive_int(d, "width", _require(d, "width"))
        groups = _positive_int(norm, "norm.groups", norm.get("groups") or 1)
        if width % groups:
            raise ConfigError(f"config.json: norm.groups ({groups}) must divide width ({width})")
        cap = d.get("logit_softcap")
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or cap < 0):
            raise ConfigError(f"config.json: 'logit_softcap' must be a positive number, got {cap!r}")
        eos = d.get("eos_token_id")
        known = {"architecture", "vocab", "width", "norm", "canon", "logit_softcap", "layers", "eos_token_id"}
        return cls(
            architecture=d.get("architecture", "Muzopel"),
            vocab=_positive_int(d, "vocab", _require(d, "vocab")),
            width=width,
            norm_eps=_number(norm, "eps", "norm."),
            norm_groups=groups,
            taps=_int(_require(d, "canon"), "taps", "canon."),
            logit_softcap=float(cap) if cap else None,
            layers=tuple(layers),
            eos_token_ids=() if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos)),
            extra={k: v for k, v in d.items() if k not in known},
        )

    def to_dict(self) -> dict:
        d: dict = dict(self.extra)
        d.update(architecture=self.architecture, canon={"taps": self.taps}, layers=[l.to_dict() for l in self.layers],
                 norm={"eps": self.norm_eps, "groups": self.norm_groups}, vocab=self.vocab, width=self.width)
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d
