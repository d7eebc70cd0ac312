"""The model plan: what an architecture hands to the generic decoder.

A plan is data.  It lists the layers (each a block arrangement and the parts it arranges under
slot names of its own: norms, mixers, feed-forwards, every one a *spec*, a kind name plus the
sizes and constants that part takes), and the order in which the layers run.  The order is a list of :class:`RunStep`: it may name a
layer twice (the second run gets a cache of its own) or let a run read the cache that an
earlier run wrote (``cache_of``), in which case it writes none.

A spec never says which model it belongs to; parts are looked up by ``kind`` in
``tandem_b200.registry``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class WeightSource:
    """One checkpoint tensor copied into rows [row_start, row_start + rows) of a parameter."""

    name: str
    row_start: int = 0
    rows: Optional[int] = None  # None: the whole parameter


@dataclass(frozen=True)
class ParamSpec:
    """A parameter a part owns.

    role "matrix": a GEMM operand or embedding table, held in the model dtype.
    role "vector": a small tensor (norm weight), always held in float32.
    role "table_int": integers, held as int32.
    """

    shape: tuple
    sources: tuple  # of WeightSource
    role: str = "matrix"


@dataclass(frozen=True)
class PartSpec:
    """Base of every spec: ``kind`` picks the implementation in the registry, within the spec's
    ``family`` ("mixer", "feed_forward", "norm", "position", "connection")."""

    kind: str
    family = None  # set by the base class of each family


@dataclass(frozen=True)
class NormSpec(PartSpec):
    """kind "rmsnorm": the row divided by its root mean square, times a weight.  kind "group_rmsnorm": the row in
    ``groups`` equal consecutive runs, each divided by its own root mean square, the whole times the weight."""

    family = "norm"
    size: int = 0
    eps: float = 1e-6
    weight: str = ""  # checkpoint tensor name
    groups: int = 1
    offset: float = 0.0  # added to the stored weight: 1.0 for checkpoints that keep the weight around zero


@dataclass(frozen=True)
class PositionSpec(PartSpec):
    """kind "rope": rotate_half rotary encoding over the first ``rotary_dim`` dims of a head.
    kind "none": no position encoding."""

    family = "position"
    rotary_dim: int = 0
    theta: float = 10000.0
    max_position: int = 0


@dataclass(frozen=True)
class MixerSpec(PartSpec):
    family = "mixer"
    prefix: str = ""  # checkpoint name prefix, e.g. "model.layers.3.self_attn"


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 1.0
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    window: Optional[int] = None  # keys a query sees, itself included; None: all
    position: PositionSpec = PositionSpec("none")


@dataclass(frozen=True)
class DistanceBiasSpec:
    """A learned bias on attention scores by distance: ``table[bucket(i - j), head]`` with
    ``buckets`` rows.  Distances below ``buckets // 2`` have a row each; from there on the rows
    are spaced evenly in the logarithm of the distance up to ``max_distance``, and the last row
    takes everything beyond: bucket(n) = min(buckets - 1, half + floor(ln(n / half) / ln(max_distance
    / half) * (buckets - half))) with half = buckets // 2."""

    buckets: int
    max_distance: int

    def bucket(self, n: int) -> int:
        import math

        half = self.buckets // 2
        if n < half:
            return n
        return min(self.buckets - 1,
                   half + int(math.floor(math.log(n / half) / math.log(self.max_distance / half) * (self.buckets - half))))


@dataclass(frozen=True)
class SinkAttentionSpec(MixerSpec):
    """Grouped-query attention whose keys and values may differ in size, with these options, each
    off where its field says so: projection biases; q and k divided by their root mean square per
    head (no weight); scores capped by ``softcap * tanh(score / softcap)``; a learned bias by
    distance; a window with ``keep_first`` tokens at the front of the sequence that stay visible;
    a learned sink per head in the softmax denominator; values mixed with those that the first
    layer of ``value_mix`` (a name shared by the layers that mix) made for the same token.
    Checkpoint tensors: ``<prefix>.q``, ``.k``, ``.v``, ``.o`` (biases ``.q.b`` ...), ``.rel``
    [buckets, heads], ``.sink`` [heads], ``.vmix`` []; ``names`` renames them (local -> suffix)."""

    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0  # of queries and keys
    value_dim: int = 0
    scale: float = 1.0
    bias: bool = False
    unit_norm: bool = False
    norm_eps: float = 1e-6
    softcap: Optional[float] = None
    distance_bias: Optional[DistanceBiasSpec] = None
    window: Optional[int] = None  # keys a query sees behind itself, itself included; None: all
    keep_first: int = 0
    sink: bool = False
    value_mix: Optional[str] = None
    value_mix_first: bool = False  # this layer's values are the ones the others mix in
    names: tuple = ()


@dataclass(frozen=True)
class DecayRecurrenceSpec(MixerSpec):
    """Linear attention with a fixed decay per head, kept as a float32 state per request:
    S <- decay_h S + k v^T, o = S^T q.  ``activation``: on q, k and v ("none" | "silu");
    ``rotary_dim`` / ``rotary_base``: rotate_half encoding of the first dims of q and k (0: none);
    ``key_scale``: factor on k behind the rotation; ``output_norm``: "per_head" (each head divided by
    its root mean square) or "all_heads" (one RMSNorm over the concatenated heads with the weight
    ``<prefix>.norm``); ``gate``: activation of the output gate's own projection ("silu" | "sigmoid").
    Checkpoint tensors: ``<prefix>.q``, ``.k``, ``.v``, ``.g``, ``.o``, ``.norm``."""

    hidden_size: int = 0
    num_heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    decay: tuple = ()
    activation: str = "none"
    rotary_dim: int = 0
    rotary_base: float = 10000.0
    key_scale: float = 1.0
    output_norm: str = "per_head"
    gate: str = "silu"
    norm_eps: float = 1e-6
    names: tuple = ()


@dataclass(frozen=True)
class SelectiveRecurrenceSpec(MixerSpec):
    """A state-space recurrence whose decay and step size are made from the token (the "state-space
    duality" form): one projection laid out [z: H P | x: H P | B: G N | C: G N | dt: H] (H heads of P
    values, G groups of N state rows; head h reads group h // (H / G)); x, B and C pass a causal
    convolution of ``conv_taps`` taps per channel (with bias) and SiLU; dt <- softplus(dt + dt_bias);
    S <- exp(-exp(A_log_h) dt) S + dt B x^T, y = S^T C + D_h x per head, S [N, P] in float32; y times
    SiLU(z), divided by its root mean square in ``norm_groups`` equal parts, times a weight, then the
    output projection.  The state of a request is S of every head and the last ``conv_taps - 1`` inputs
    of the convolution.  Checkpoint tensors ``<prefix>.in``, ``.conv`` [channels, taps], ``.conv.b``,
    ``.dt_bias``, ``.A_log``, ``.D``, ``.norm``, ``.o``; ``names`` renames them (local -> suffix)."""

    hidden_size: int = 0
    num_heads: int = 0
    value_dim: int = 0  # P
    state_dim: int = 0  # N
    groups: int = 1  # G
    conv_taps: int = 1
    norm_groups: int = 1
    norm_eps: float = 1e-6
    names: tuple = ()


@dataclass(frozen=True)
class RotaryScalingSpec:
    """Frequencies stretched for sequences longer than ``original`` tokens, pair by pair.  With n(t) =
    dims ln(original / (2 pi t)) / (2 ln base) the pair index whose wave makes t turns in ``original`` tokens,
    lo = max(floor(n(fast)), 0) and hi = min(ceil(n(slow)), dims - 1): pair i keeps the share 1 - ramp_i of its
    frequency and takes the share ramp_i of frequency / ``factor``, ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1);
    cos and sin are multiplied by 0.1 ln(factor) + 1."""

    factor: float
    original: float
    fast: float
    slow: float


def rotary_table(dims: int, base: float, scaling: Optional["RotaryScalingSpec"] = None) -> tuple:
    """(frequency of every pair, factor on cos and sin) in double precision for a rotation of ``dims`` numbers."""
    import math

    freq = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling is None:
        return freq, 1.0

    def pair_of(turns: float) -> float:
        return dims * math.log(scaling.original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(scaling.fast)), 0)
    hi = min(math.ceil(pair_of(scaling.slow)), dims - 1)
    out = []
    for i, f in enumerate(freq):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(f / scaling.factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(scaling.factor) + 1.0


@dataclass(frozen=True)
class RotaryBandSpec:
    """Frequencies slowed by wavelength, for sequences longer than ``original`` tokens.  A pair whose wave
    (2 pi / frequency tokens long) is shorter than ``original / high`` keeps its frequency; one whose wave is
    longer than ``original / low`` gets frequency / ``factor``; between the two, with s = (original / wave - low) /
    (high - low), the pair gets (1 - s) frequency / factor + s frequency."""

    factor: float
    low: float
    high: float
    original: float


def rotary_band_table(dims: int, base: float, scaling: Optional["RotaryBandSpec"] = None) -> list:
    """The frequency base^(-2 i / dims) of every pair i < dims / 2 of a rotation of ``dims`` numbers, in double
    precision, slowed where ``scaling`` says so."""
    import math

    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling is not None:
            wave = 2.0 * math.pi / f
            if wave > scaling.original / scaling.low:
                f /= scaling.factor
            elif wave >= scaling.original / scaling.high:
                share = (scaling.original / wave - scaling.low) / (scaling.high - scaling.low)
                f = (1.0 - share) * f / scaling.factor + share * f
        out.append(f)
    return out


@dataclass(frozen=True)
class WindowAttentionSpec(MixerSpec):
    """Grouped-query softmax attention over a sliding window whose queries and keys are prepared between the
    projection and the scores by any of: projection biases on q and k (``bias``); a causal convolution over time
    on every column of q, k and v (``conv_taps`` > 1 taps, no bias, no skip term; a request's last taps - 1
    projected rows are its state); a norm of q and k, ``qk_norm`` = "none" | "unit" (each head divided by its root
    mean square) | "head" (the same times one weight of ``head_dim`` numbers that all heads share) | "whole" (q, and
    k, divided by the root mean square over all their heads, times a weight of that size); a rotation of the first
    ``rotary_dim`` numbers of every head, number i paired with i + rotary_dim / 2, by position * frequency_i
    (``rotary_base``, ``rotary_scaling``).  ``values`` = "projection" (a projection of their own) or "keys" (the keys
    as projected, with their bias and convolution, before norm and rotation; no value tensor).  Scores are
    ``scale`` q . k, capped by ``softcap * tanh(score / softcap)`` where a cap is given; position i sees j with
    0 <= i - j < ``window`` (None: all j <= i).  ``sink``: a number whose exponential joins the softmax denominator
    (0.0: one is added to it), None: none.  ``gate`` "sigmoid_head": every head's output times the sigmoid of one
    number, a projection of the mixer's input.  ``borrows_kv``: the mixer has no key or value tensors; its run reads
    the cache of another run (``RunStep.cache_of``).  ``cache_window``: how many keys the cache keeps behind the
    newest where that is more than ``window`` (a run whose cache is also read through a wider window; 0: all keys).
    Checkpoint tensors ``<prefix>.q``, ``.k``, ``.v``, ``.o``, ``.g`` [heads, hidden]; biases ``.q.b``, ``.k.b``;
    norm weights ``.q.norm``, ``.k.norm``; taps ``.q.conv``, ``.k.conv``, ``.v.conv`` [columns, taps]."""

    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0  # of queries and keys
    value_dim: int = 0
    scale: float = 1.0
    bias: bool = False
    conv_taps: int = 0
    qk_norm: str = "none"
    norm_eps: float = 1e-6
    rotary_dim: int = 0
    rotary_base: float = 10000.0
    rotary_scaling: Optional[RotaryBandSpec] = None
    values: str = "projection"
    softcap: Optional[float] = None
    window: Optional[int] = None
    sink: Optional[float] = None
    gate: str = "none"
    borrows_kv: bool = False
    cache_window: Optional[int] = None


@dataclass(frozen=True)
class LatentAttentionSpec(MixerSpec):
    """Causal softmax attention whose keys and values are expanded from a latent of ``latent_dim``
    numbers per token (RMS-normed with a weight), plus one rotated key part of ``rotary_dim``
    numbers that all heads share; a query head is [``head_dim`` unrotated | ``rotary_dim`` rotated].
    The rotation (angle = position * base^(-2 i / rotated_dims), frequencies stretched where
    ``rotary_scaling`` says so) turns the first ``rotated_dims`` numbers of the rotated part, paired
    (i, i + rotated_dims / 2) (``rotary_pairing`` "half") or (2 i, 2 i + 1) ("interleaved").
    Only the latent and the rotated key part are cached.  ``query_latent_dim`` > 0: the queries come
    through a latent of their own, q = W_uq RMSNorm(W_dq x) (tensors ``.dq``, ``.dq.norm``, ``.uq``
    instead of ``.q``).  ``gate``: "sigmoid" multiplies the concatenated heads by sigmoid of a
    projection of the mixer's input (``.g`` [heads * value_dim, hidden]), "sigmoid_head" each head by one
    such number (``.g`` [heads, hidden]), "none" leaves them.
    Checkpoint tensors ``<prefix>.q``, ``.dkv``, ``.dkv.norm``, ``.uk``, ``.uv``, ``.g``, ``.o``."""

    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0  # unrotated query/key dimensions per head
    rotary_dim: int = 0
    rotated_dims: int = 0
    rotary_base: float = 10000.0
    value_dim: int = 0
    latent_dim: int = 0
    scale: float = 1.0
    norm_eps: float = 1e-6
    gate: str = "sigmoid"
    names: tuple = ()
    rotary_pairing: str = "half"
    rotary_scaling: Optional[RotaryScalingSpec] = None
    query_latent_dim: int = 0


@dataclass(frozen=True)
class ShortConvolutionSpec(MixerSpec):
    """A causal convolution over time on every channel of the stream, in front of a sublayer:
    h_t = x_t + sum_j w[c, j] x_(t - taps + 1 + j) (``skip`` False: without x_t), zeros in front of a
    sequence.  A request's last ``taps`` - 1 inputs are its state.  Checkpoint tensor ``weight`` [hidden, taps]."""

    hidden_size: int = 0
    taps: int = 1
    weight: str = ""
    skip: bool = True


@dataclass(frozen=True)
class FeedForwardSpec(PartSpec):
    family = "feed_forward"
    prefix: str = ""


@dataclass(frozen=True)
class GatedMLPSpec(FeedForwardSpec):
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"
    names: tuple = ()  # (local, checkpoint suffix) for "gate", "up", "down" where they are not <x>_proj.weight
    float32_output: bool = False  # the down projection comes back unrounded


@dataclass(frozen=True)
class RoutedMLPSpec(FeedForwardSpec):
    """``num_experts`` gated feed-forwards (down(act(gate x) * up x), no biases) of which a token uses
    ``top_k``: router logits W_router x in float32, scores by ``score`` ("sigmoid" | "softmax"), the
    ``top_k`` largest scores chosen, their scores divided by their sum (+ 1e-20) where ``normalize``,
    times ``route_scale``; the output is the weighted sum of the chosen experts' outputs.  Checkpoint
    tensors ``<prefix>.router`` [experts, hidden], ``<prefix>.e<i>.gate``, ``.up``, ``.down``.
    ``gated`` False: an expert is down(act(up x)) (no ``.gate`` tensors; ``activation`` "gelu", the exact
    one).  ``identity_experts`` n: the router has n outputs more, behind the experts'; a token that
    chooses one of them gets its own input back for it (times the weight).  ``choice_bias``: a tensor
    ``<prefix>.<choice_bias>`` [router outputs] is added to the scores for the choice only.
    ``router`` "token_table": there is no router; an integer tensor ``<prefix>.<table>`` [vocab, top_k] names every
    token id's experts, each with the weight 1 / top_k (``score``, ``normalize``, ``route_scale`` and the identity
    experts do not apply).  ``activation`` "relu2" (without a gate): the square of max(z, 0).
    ``shared_intermediate_size`` > 0: one more expert of that width, of the same form (``<prefix>.shared.up``,
    ``.down``), runs for every token and is added with weight one."""

    hidden_size: int = 0
    intermediate_size: int = 0  # of one expert
    num_experts: int = 0
    top_k: int = 1
    score: str = "sigmoid"
    normalize: bool = True
    route_scale: float = 1.0
    activation: str = "silu"
    gated: bool = True
    identity_experts: int = 0
    choice_bias: Optional[str] = None
    router: str = "learned"
    table: str = "table"
    vocab_size: int = 0  # rows of the table
    shared_intermediate_size: int = 0


@dataclass(frozen=True)
class DenseMLPSpec(FeedForwardSpec):
    """down(act(up(x))) with optional biases; ``activation``: "gelu_tanh" | "silu" | "relu2" (the square of max(z, 0)) | "none".
    Checkpoint tensors ``<prefix>.up``, ``.down`` (biases ``.up.b``, ``.down.b``)."""

    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "gelu_tanh"
    bias: bool = True
    names: tuple = ()


@dataclass(frozen=True)
class ConnectionSpec(PartSpec):
    family = "connection"


@dataclass(frozen=True)
class StreamLinkSpec(ConnectionSpec):
    """How one sublayer hangs on a residual of ``streams`` parallel streams X_1 .. X_s: it reads
    u = sum_s in[s] X_s and, with its output y, every stream becomes (all from the old ones)
    X_t <- sum_s mix[s, t] X_s + mult * out[t] * y.  ``prefix`` names the checkpoint tensors
    ``<prefix>.in`` [s], ``.out`` [s], ``.mix`` [s, s] (indexed [from, to]); None: one stream with
    in = out = mix = 1, which is the plain residual sum x <- x + mult * y."""

    streams: int = 1
    mult: float = 1.0
    prefix: Optional[str] = None


@dataclass(frozen=True)
class DepthAverageSpec(ConnectionSpec):
    """What a layer hands on is a learned weighted sum of the results of all layers so far:
    x <- sum_(j <= n) a[j] Y_j with Y_0 the start of the stream and Y_n this layer's own result (``count`` =
    n + 1 coefficients in the checkpoint tensor ``weight``).  The layer with two coefficients is the first: what it
    receives is Y_0.  ``total``: how many results the model makes in all, Y_0 included (the room kept for them)."""

    count: int = 1
    weight: str = ""
    total: int = 1


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the kind of its block arrangement and the parts that arrangement works with, as
    (slot name, family, spec).  Which slots there are is the arrangement's business: "prenorm" has
    ``mixer_norm``, ``mixer``, ``feed_forward_norm`` and ``feed_forward``; another arrangement may
    have four norms, no feed-forward, or two mixers side by side."""

    block: str
    parts: tuple

    @classmethod
    def of(cls, block: str, **slots: PartSpec) -> "LayerSpec":
        """``LayerSpec.of("prenorm", mixer=..., feed_forward=..., mixer_norm=..., feed_forward_norm=...)``:
        the family of each part is the one its spec class belongs to."""
        for name, spec in slots.items():
            if getattr(spec, "family", None) is None:
                raise TypeError(f"slot {name!r}: {type(spec).__name__} belongs to no part family "
                                "(derive it from MixerSpec, FeedForwardSpec, NormSpec or PositionSpec)")
        return cls(block, tuple((name, spec.family, spec) for name, spec in slots.items()))

    def slot(self, name: str) -> PartSpec:
        for slot, _, spec in self.parts:
            if slot == name:
                return spec
        raise KeyError(f"the layer has no slot {name!r} (it has {[s for s, _, _ in self.parts]})")

    def with_slot(self, name: str, spec: PartSpec) -> "LayerSpec":
        """A copy in which the slot holds ``spec`` (put behind the others if the slot is new)."""
        entry = (name, spec.family, spec)
        if any(slot == name for slot, _, _ in self.parts):
            return LayerSpec(self.block, tuple(entry if slot == name else (slot, fam, sp) for slot, fam, sp in self.parts))
        return LayerSpec(self.block, self.parts + (entry,))

    def of_family(self, family: str) -> list:
        """(slot name, spec) of the layer's parts of one family, in the order they were given."""
        return [(slot, spec) for slot, fam, spec in self.parts if fam == family]


@dataclass(frozen=True)
class RunStep:
    layer: int
    cache_of: Optional[int] = None  # index into ModelPlan.order of the run whose cache is read


@dataclass(frozen=True)
class EmbeddingSpec:
    """Start of the residual stream: ``scale * table[token]``, plus ``positions[position]`` where
    the model has a learned table of absolute positions (a checkpoint tensor [max_position, hidden]);
    written ``copies`` times side by side for arrangements that keep several streams."""

    vocab_size: int
    hidden_size: int
    weight: str
    scale: float = 1.0
    positions: Optional[str] = None
    copies: int = 1  # the residual starts as so many equal streams side by side, [T, copies * hidden]
    norm: Optional[NormSpec] = None  # applied to the embedded rows before the first layer


@dataclass(frozen=True)
class HeadSpec:
    """Logits = ``scale * (h @ weight^T)``, then ``softcap * tanh(logits / softcap)`` where a cap is given."""

    vocab_size: int
    hidden_size: int
    weight: Optional[str]  # None: tied to the embedding table
    scale: float = 1.0
    softcap: Optional[float] = None


@dataclass(frozen=True)
class ModelPlan:
    embedding: EmbeddingSpec
    layers: tuple  # of LayerSpec
    order: tuple  # of RunStep
    final_norm: NormSpec
    head: HeadSpec
    max_position: int
    ignored_weights: tuple = ()  # regex patterns of checkpoint names that may be present and unused
    eos_token_ids: tuple = ()

    def __post_init__(self) -> None:
        for i, run in enumerate(self.order):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {run.layer}, the plan has {len(self.layers)}")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < i:
                    raise ValueError(f"order[{i}].cache_of must name an earlier run, got {run.cache_of}")
                if self.order[run.cache_of].cache_of is not None:
                    raise ValueError(f"order[{i}].cache_of names a run that itself reads another run's cache")
