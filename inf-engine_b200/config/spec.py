"""Descriptions of a model as data: parts, blocks, and the order they run in.

A ``ModelSpec`` is what an architecture's ``config.json`` is turned into.  It
names every size and constant and every weight tensor, layer by layer, so that
two layers of one model may use different mixers, feed-forwards, norms or
position encodings.  Nothing here computes; the classes under ``parts`` are
built from these records through the registries in ``parts.registry``.

A new kind of part adds a frozen dataclass with a ``kind`` string here or in its
own module (tests define toy ones) and registers a class for that ``kind``.
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class RopeScaling:
    """Frequency scaling of rotary embeddings, read from ``rope_scaling``."""

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last axis."""

    kind: str          # "rmsnorm" | "layernorm"
    size: int
    eps: float
    weight: str        # tensor name of the gain
    bias: str | None = None   # tensor name of the additive term ("layernorm")


@dataclass(frozen=True)
class PositionSpec:
    """How positions enter a mixer."""

    kind: str                     # "rotary" | "none" | "bucketed_bias"
    head_dim: int = 0
    theta: float = 0.0
    max_positions: int = 0
    scaling: RopeScaling | None = None
    # "bucketed_bias": a learned table [n_buckets, n_heads] added to the scores by distance; distances below half
    # the buckets have a row each, the rest share rows on a logarithmic scale that ends at ``max_distance``
    table: str = ""
    n_buckets: int = 0
    n_heads: int = 0
    max_distance: int = 0


@dataclass(frozen=True)
class HeadNormSpec:
    """RMS norm of every query head and key head before the scores, with gains of the head's size that all heads
    share (a name of None leaves that side alone)."""

    eps: float
    q_weight: str | None = None
    k_weight: str | None = None


@dataclass(frozen=True)
class MixerSpec:
    """Base of token mixers; ``kind`` selects the registered class."""

    kind: str


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    """Causal grouped-query attention over a paged key/value cache."""

    hidden: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    window: int | None = None      # None: every earlier key; n: the last n keys, itself included
    position: PositionSpec = PositionSpec(kind="none")
    q_proj: str = ""
    k_proj: str = ""
    v_proj: str = ""
    o_proj: str = ""
    v_head_dim: int | None = None  # head size of values and output when it is not ``head_dim``
    scale: float | None = None     # multiplier of q . k; None: head_dim ** -0.5
    qk_norm: HeadNormSpec | None = None
    head_scale: str | None = None  # tensor [n_heads]: a learned multiplier of each head's scores beside ``scale``

    @property
    def value_dim(self) -> int:
        return self.v_head_dim if self.v_head_dim is not None else self.head_dim


@dataclass(frozen=True)
class GeneralDeltaSpec(MixerSpec):
    """The generalized delta rule: a recurrent mixer with a head_dim x head_dim float32 state per head.

    Per token and head, with projections r, k, v, a gate g, a removal rate a = sigmoid(a_proj x + a_bias) and a
    decay w = exp(-decay_rate * sigmoid(w2 tanh(w1 x) + w0)) per key channel, and the unit key
    u = k / sqrt(sum(k^2) + key_eps):  S <- diag(w) S - (a * u)(u^T S) + k v^T,  o = S^T r.  Each head's o is
    divided by its root mean square (norm_eps), multiplied by ``out_gain`` and sigmoid(g), then projected by o_proj.
    """

    hidden: int = 0
    n_heads: int = 0
    head_dim: int = 0
    decay_rank: int = 0            # inner size of the low-rank pair w1, w2
    decay_rate: float = 0.0
    key_eps: float = 1e-6
    norm_eps: float = 1e-6
    r_proj: str = ""
    k_proj: str = ""
    v_proj: str = ""
    g_proj: str = ""
    a_proj: str = ""
    a_bias: str = ""
    w1: str = ""
    w2: str = ""
    w0: str = ""
    out_gain: str = ""
    o_proj: str = ""


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str


@dataclass(frozen=True)
class GatedMLPSpec(FeedForwardSpec):
    """``down(act(gate(x)) * up(x))``."""

    hidden: int = 0
    intermediate: int = 0
    activation: str = "silu"
    gate_proj: str = ""
    up_proj: str = ""
    down_proj: str = ""


@dataclass(frozen=True)
class PolyNormMLPSpec(FeedForwardSpec):
    """``down(act(up(x) + up_bias)) + down_bias`` with the PolyNorm activation: c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3,
    powers element by element, N(x) = x / sqrt(mean(x^2) + eps) over a token's ``intermediate`` values; ``coef`` names
    the tensor of the four numbers."""

    hidden: int = 0
    intermediate: int = 0
    eps: float = 1e-6
    up_proj: str = ""
    up_bias: str | None = None
    down_proj: str = ""
    down_bias: str | None = None
    coef: str = ""


@dataclass(frozen=True)
class BlockSpec:
    """One residual block: which norm, mixer and feed-forward, and how arranged.  A block without a feed-forward
    (``feedforward`` and ``ff_norm`` None) is its mixer half alone."""

    kind: str                      # "prenorm"
    mixer_norm: NormSpec
    mixer: MixerSpec
    ff_norm: NormSpec | None
    feedforward: FeedForwardSpec | None


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.

    ``layer`` indexes ``ModelSpec.layers`` and may occur in several entries
    (shared weights).  ``cache_from`` names an EARLIER entry of the schedule whose
    cache this run reads instead of writing one of its own.
    """

    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, layers, their order, final norm and head."""

    architecture: str
    vocab_size: int
    hidden: int
    max_positions: int
    embedding: str                           # tensor name of the token table
    layers: tuple[BlockSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    head: str | None                         # tensor name, or None: tied to the embedding
    optional_tensors: tuple[str, ...] = field(default_factory=tuple)  # present-but-unused names tolerated
    kind: str = "decoder"                    # which registered top level puts the parts together


@dataclass(frozen=True)
class BigramDecoderSpec(ModelSpec):
    """A decoder whose first residual is the token embedding plus a hashed bigram embedding: row
    ``(previous token * mul_prev + token * mul_cur) mod buckets`` of the tensor ``bigram`` ([buckets + 1, hidden]),
    and its last row for a sequence's first token."""

    bigram: str = ""
    bigram_buckets: int = 0
    bigram_mul_prev: int = 0
    bigram_mul_cur: int = 0
    kind: str = "bigram_decoder"
