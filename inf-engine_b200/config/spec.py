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
    unit_offset: bool = False  # "rmsnorm": the tensor is stored around zero and the multiplier is 1 + weight


@dataclass(frozen=True)
class PositionSpec:
    """How positions enter a mixer."""

    kind: str                     # "rotary" | "none" | "bucketed_bias" | "rotary_pairs"
    head_dim: int = 0
    theta: float = 0.0
    max_positions: int = 0
    scaling: RopeScaling | None = None
    # "rotary_pairs": neighbouring dimensions (2i, 2i + 1) of the first ``rot_dims`` dimensions of a head turn by
    # position * theta^(-2i / rot_dims); the rest of the head passes unchanged.  Angles are worked out from the
    # position inside the kernel, so there is no table and no limit on positions.
    rot_dims: int = 0
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
    # beside a window: keys at positions below ``keep_first`` stay visible to every later query (and stay in the
    # cache), at their true positions
    keep_first: int = 0
    q_bias: str | None = None      # biases of the three projections ([heads * head size] each)
    k_bias: str | None = None
    v_bias: str | None = None
    # RMS norm over the WHOLE projection of q (and of k), all heads at once, with gains of that size, before the
    # heads are split and rotated (``HeadNormSpec`` above norms each head by itself)
    q_row_norm: str | None = None
    k_row_norm: str | None = None
    row_norm_eps: float = 1e-6
    out_scale: float = 1.0         # multiplier of the heads' outputs before the output projection

    @property
    def value_dim(self) -> int:
        return self.v_head_dim if self.v_head_dim is not None else self.head_dim


@dataclass(frozen=True)
class ShortConvSpec:
    """A causal convolution over time, one filter per channel: ``weight`` [channels, taps], whose last column
    multiplies the current token's input; zeros stand before a sequence's start.  The last ``taps - 1`` inputs of a
    sequence are state that a mixer carries from step to step."""

    taps: int
    weight: str
    bias: str | None = None


@dataclass(frozen=True)
class GatedDeltaSpec(MixerSpec):
    """The gated delta rule: a recurrent mixer with a ``head_dim x v_head_dim`` float32 state per head.

    q and k have ``n_kv_heads`` heads of ``head_dim`` (head h of the state reads q/k head h // (n_heads / n_kv_heads)),
    v has ``n_heads`` heads of ``v_head_dim``.  Each passes a short convolution and SiLU; q and k become unit vectors
    (``key_eps`` inside the root) and q takes head_dim^-1/2.  Per token and head, with beta = sigmoid(b x) and the
    decay g = exp(-exp(A_log) * softplus(a x + dt_bias)):
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
    o is divided by its root mean square over ``v_head_dim`` (norm_eps), multiplied by ``out_gain`` ([v_head_dim],
    shared by the heads) and by silu(gate x), and projected by ``o_proj``."""

    hidden: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    v_head_dim: int = 0
    key_eps: float = 1e-6
    norm_eps: float = 1e-6
    q_proj: str = ""
    k_proj: str = ""
    v_proj: str = ""
    q_conv: ShortConvSpec | None = None
    k_conv: ShortConvSpec | None = None
    v_conv: ShortConvSpec | None = None
    beta_proj: str = ""
    decay_proj: str = ""
    decay_log: str = ""            # A_log, [n_heads]
    decay_bias: str = ""           # dt_bias, [n_heads]
    gate_proj: str = ""
    out_gain: str = ""
    o_proj: str = ""


@dataclass(frozen=True)
class GatedLinearRecurrenceSpec(MixerSpec):
    """A recurrent block around a real-gated linear recurrent unit, ``width`` channels:
        y = gelu_tanh(y_proj x + y_bias);  u = conv(x_proj x + x_bias)
        r = sigmoid(A_b u_b + a_b), i = sigmoid(I_b u_b + i_b)     per block b of ``n_blocks`` equal parts of u
        a = exp(-decay_scale * r * softplus(lam));  S <- a S + sqrt(1 - a^2) (i * u);  out = o_proj (S * y)
    with S a float32 vector per request that starts at zero."""

    hidden: int = 0
    width: int = 0
    n_blocks: int = 1
    decay_scale: float = 8.0
    y_proj: str = ""
    y_bias: str = ""
    x_proj: str = ""
    x_bias: str = ""
    conv: ShortConvSpec | None = None
    a_gate: str = ""               # [n_blocks, width / n_blocks, width / n_blocks], rows are outputs
    a_gate_bias: str = ""          # [n_blocks, width / n_blocks]
    i_gate: str = ""
    i_gate_bias: str = ""
    lam: str = ""                  # [width]
    o_proj: str = ""
    out_scale: float = 1.0         # multiplier of S * y before the output projection


@dataclass(frozen=True)
class ParallelMixerSpec(MixerSpec):
    """Several mixers side by side that read the same input; the result is the sum of their outputs, each times its
    weight (a branch folds the weight into what it hands its output projection)."""

    hidden: int = 0
    branches: tuple[MixerSpec, ...] = ()


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
class RoutedExpertsSpec(FeedForwardSpec):
    """A mixture of gated feed-forward experts with a sigmoid router.

    Router scores s = sigmoid(router x) in float32; an expert's choice score is s + ``correction``.  The experts
    form ``n_groups`` groups of neighbours; a group's score is the sum of its two largest choice scores, and only
    experts of the ``keep_groups`` best groups can be chosen.  The ``top`` largest choice scores among them are
    taken; their weights are their s divided by the sum of those (+ ``weight_eps``), times ``route_scale``.  The
    output is the weighted sum of the chosen experts' ``down(silu(gate x) * up x)``.  ``shared`` (optional) is a
    dense expert that every token runs; it is added times sigmoid(shared_gate x), one number a token."""

    hidden: int = 0
    intermediate: int = 0
    n_experts: int = 0
    top: int = 1
    n_groups: int = 1
    keep_groups: int = 1
    route_scale: float = 1.0
    weight_eps: float = 1e-20
    router: str = ""
    correction: str | None = None
    expert_prefix: str = ""        # expert e's tensors are <prefix><e>.gate / .up / .down
    shared: GatedMLPSpec | None = None
    shared_gate: str | None = None


@dataclass(frozen=True)
class BlockSpec:
    """One residual block: which norm, mixer and feed-forward, and how arranged.  A block without a feed-forward
    (``feedforward`` and ``ff_norm`` None) is its mixer half alone."""

    kind: str                      # "prenorm": x += part(norm(x)) | "outnorm": x += norm(part(x))
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
