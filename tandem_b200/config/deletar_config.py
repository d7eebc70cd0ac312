"""Typed view of a Deletar ``config.json``.

Deletar is a decoder whose layers are listed one by one, each with a norm in front of and behind every sublayer:
x <- x + norm(mixer(norm(x))), then x <- x + norm(feed_forward(norm(x))), the norms RMS norms whose weight is stored
around zero.  All three mixers are grouped-query softmax attention over a sliding window with partly rotated heads:
"attention" passes q, k and v through a short causal convolution; "attention_2" has biases on q and k, a norm over
the whole of q and of k, the keys as projected for values, capped scores and a sigmoid gate per head; "attention_3"
norms every head with one shared weight, may slow its rotation's frequencies by wavelength, caps scores, adds one to the
softmax denominator, gates every head, and may read another layer's keys and values instead of making its own
(``kv_from``).  The feed-forward is down(relu(up h)^2), dense, or as experts that a table of token ids names, plus an
optional shared expert, or absent.  The embedding is scaled and the logits are soft-capped.  Every size and every
constant that may differ between models is a key of the file; nothing here has a default that stands in for a missing
size.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from tandem_b200.config.fumanex_config import NO_POSITION_LIMIT, _number
from tandem_b200.config.model_config import ConfigError, _positive_int, _require

MIXER_TYPES = ("attention", "attention_2", "attention_3")
MLP_KINDS = ("dense", "moe")

__all__ = ["DeletarConfig", "DeletarLayer", "DeletarMixer", "DeletarScaling", "DeletarMLP", "NO_POSITION_LIMIT"]


def _int(d: dict, key: str, where: str) -> int:
    return _positive_int(d, where + key, _require(d, key))


def _optional_number(d: dict, key: str, where: str) -> Optional[float]:
    if d.get(key) is None:
        return None
    v = _number(d, key, where)
    if v <= 0:
        raise ConfigError(f"config.json: {where}{key!r} must be positive, got {v!r}")
    return v


@dataclass(frozen=True)
class DeletarScaling:
    factor: float
    low: float
    high: float
    original: float

    @classmethod
    def from_dict(cls, s: dict, where: str) -> "DeletarScaling":
        c = cls(*(_number(s, k, where) for k in ("factor", "low", "high", "original")))
        if c.factor <= 0 or c.original <= 0 or c.low <= 0 or c.high <= c.low:
            raise ConfigError(f"config.json: {where}factor, original and low must be positive and high above low")
        return c

    def to_dict(self) -> dict:
        original = int(self.original) if float(self.original).is_integer() else self.original
        return {"factor": self.factor, "high": self.high, "low": self.low, "original": original}


@dataclass(frozen=True)
class DeletarMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float
    scaling: Optional[DeletarScaling] = None
    window: Optional[int] = None  # keys a position sees, itself included
    softcap: Optional[float] = None
    conv: int = 0  # taps of the convolution on q, k and v
    kv_from: Optional[int] = None  # the layer whose keys and values this one reads

    @classmethod
    def from_dict(cls, m: dict, where: str, kind: str) -> "DeletarMixer":
        rot = _require(m, "rot")
        sc, mask = rot.get("scaling"), m.get("mask")
        kv_from = m.get("kv_from")
        if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or kv_from < 0):
            raise ConfigError(f"config.json: {where}kv_from must be a layer's index, got {kv_from!r}")
        c = cls(heads=_int(m, "heads", where), kv_heads=_int(m, "kv_heads", where), dim=_int(m, "dim", where),
                vdim=_int(m, "vdim", where), scale=_number(m, "scale", where), rot_dims=_int(rot, "dims", where + "rot."),
                rot_base=_number(rot, "base", where + "rot."),
                scaling=None if not sc else DeletarScaling.from_dict(sc, where + "rot.scaling."),
                window=None if not mask else _int(mask, "size", where + "mask."),
                softcap=_optional_number(m, "softcap", where),
                conv=_int(m, "conv", where) if m.get("conv") else 0, kv_from=kv_from)
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}heads ({c.heads}) must be a multiple of kv_heads ({c.kv_heads})")
        if c.rot_dims > c.dim or c.rot_dims % 2:
            raise ConfigError(f"config.json: {where}rot.dims ({c.rot_dims}) must be even and at most dim ({c.dim})")
        if c.rot_base <= 1.0:
            raise ConfigError(f"config.json: {where}rot.base ({c.rot_base}) must exceed 1")
        if kind == "attention_2" and c.vdim != c.dim:
            raise ConfigError(f"config.json: {where}vdim ({c.vdim}) must equal dim ({c.dim}): this mixer's values are its keys")
        if kind != "attention" and c.conv:
            raise ConfigError(f"config.json: {where}conv belongs to the mixer 'attention' only")
        if kind != "attention_3" and c.kv_from is not None:
            raise ConfigError(f"config.json: {where}kv_from belongs to the mixer 'attention_3' only")
        return c

    def to_dict(self) -> dict:
        rot: dict = {"base": self.rot_base, "dims": self.rot_dims}
        if self.scaling is not None:
            rot["scaling"] = self.scaling.to_dict()
        d: dict = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "rot": rot, "scale": self.scale, "vdim": self.vdim}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        if self.conv:
            d["conv"] = self.conv
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class DeletarMLP:
    kind: str  # "dense" | "moe"
    ff: int  # width of the dense feed-forward, or of one expert
    experts: int = 0
    top: int = 0
    shared_ff: int = 0  # width of the expert that every token passes; 0: none

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "DeletarMLP":
        kind = _require(m, "kind")
        if kind not in MLP_KINDS:
            raise ConfigError(f"config.json: {where}kind {kind!r} is not supported (supported: {list(MLP_KINDS)})")
        if kind == "dense":
            return cls("dense", _int(m, "ff", where))
        router, expert, shared = _require(m, "router"), _require(m, "expert"), m.get("shared")
        c = cls("moe", _int(expert, "ff", where + "expert."), experts=_int(router, "experts", where + "router."),
                top=_int(router, "top", where + "router."), shared_ff=_int(shared, "ff", where + "shared.") if shared else 0)
        if c.top > c.experts:
            raise ConfigError(f"config.json: {where}router.top ({c.top}) exceeds the {c.experts} experts")
        return c

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        d: dict = {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class DeletarLayer:
    type: str
    mixer: DeletarMixer
    mlp: Optional[DeletarMLP]

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(), "type": self.type}


@dataclass(frozen=True)
class DeletarConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_softcap: Optional[float]
    layers: tuple  # of DeletarLayer
    eos_token_ids: tuple = ()
    extra: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, d: dict) -> "DeletarConfig":
        entries = _require(d, "layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]."
            kind = _require(e, "type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}type {kind!r} is not supported (supported: {list(MIXER_TYPES)})")
            mixer = DeletarMixer.from_dict(_require(e, "mixer"), where + "mixer.", kind)
            mlp = e.get("mlp")
            layers.append(DeletarLayer(kind, mixer, None if mlp is None else DeletarMLP.from_dict(mlp, where + "mlp.")))
        for i, L in enumerate(layers):
            j = L.mixer.kv_from
            if j is None:
                continue
            where = f"layers[{i}].mixer."
            if j >= i:
                raise ConfigError(f"config.json: {where}kv_from ({j}) must name an earlier layer")
            src = layers[j]
            if src.mixer.kv_from is not None:
                raise ConfigError(f"config.json: {where}kv_from names layer {j}, which itself reads another layer's keys")
            a, b = L.mixer, src.mixer
            if (a.kv_heads, a.dim, a.vdim) != (b.kv_heads, b.dim, b.vdim):
                raise ConfigError(f"config.json: {where}kv_from names layer {j}, whose keys and values have other sizes "
                                  f"({b.kv_heads} heads of {b.dim} / {b.vdim} against {a.kv_heads} of {a.dim} / {a.vdim})")
        embedding = d.get("embedding") or {}
        scale = _number(embedding, "scale", "embedding.") if embedding.get("scale") is not None else 1.0
        eos = d.get("eos_token_id")
        known = {"architecture", "vocab", "width", "norm", "embedding", "logit_softcap", "layers", "eos_token_id"}
        return cls(
            architecture=d.get("architecture", "Deletar"),
            vocab=_positive_int(d, "vocab", _require(d, "vocab")),
            width=_positive_int(d, "width", _require(d, "width")),
            norm_eps=_number(_require(d, "norm"), "eps", "norm."),
            embedding_scale=scale,
            logit_softcap=_optional_number(d, "logit_softcap", ""),
            layers=tuple(layers),
            eos_token_ids=() if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos)),
            extra={k: v for k, v in d.items() if k not in known},
        )

    def to_dict(self) -> dict:
        d: dict = dict(self.extra)
        d.update(architecture=self.architecture, embedding={"scale": self.embedding_scale}, layers=[l.to_dict() for l in self.layers],
                 norm={"eps": self.norm_eps}, vocab=self.vocab, width=self.width)
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d
