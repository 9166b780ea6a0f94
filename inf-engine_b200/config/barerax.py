"""Typed configuration of the Barerax decoder, read from ``config.json``.

A Barerax model is a list of pre-norm layers, each with LayerNorm (weight and bias), one of two mixers and an
optional dense feed-forward with the PolyNorm activation; the token embedding takes a hashed bigram embedding
beside it and the head is the embedding table again.  The two mixers:

* ``attention``: grouped-query softmax attention without rotation; queries and keys take an RMS norm per head,
  scores are ``scale * temp[head] * (q . k) + rel[bucket(distance), head]`` with buckets that are one distance
  wide up to half the table and logarithmic up to ``bias_max`` beyond; values may have another head size.
* ``general_delta``: the generalized delta rule, a recurrent layer with a matrix state per head.

``config.json`` gives every size and every constant that differs between models of the family:

    {"architecture": "Barerax", "vocab": V, "width": d, "norm": {"eps": e},
     "embedding": {"bigram": {"buckets": n, "mul_prev": a, "mul_cur": b}},
     "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "bias_max"},
                 "mlp": {"kind": "dense", "ff": f} | null},
                {"type": "general_delta", "mixer": {"heads", "dim"}, "mlp": ...}, ...]}

Sizes that the file does not state (rows of the distance table, inner size of the decay's low-rank pair) are
read from the checkpoint's tensor shapes when a model folder is given; ``tensor_shapes`` carries them.
Tensor names: ``embed``, ``bigram``, ``l<i>.norm1[.b]``, ``l<i>.norm2[.b]``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm[.b]``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

from .llama import ConfigError
from .spec import (
    AttentionSpec,
    BigramDecoderSpec,
    BlockSpec,
    GeneralDeltaSpec,
    HeadNormSpec,
    NormSpec,
    PolyNormMLPSpec,
    PositionSpec,
    ScheduleEntry,
)

# The design fixes these: the decay of the delta rule is exp(-DECAY_RATE * sigmoid(.)), the unit key has
# KEY_EPS inside its root.  Positions have no limit of the model's own.
DECAY_RATE = math.exp(-0.5)
KEY_EPS = 1e-6
NO_POSITION_LIMIT = 1 << 30
DEFAULT_REL_BUCKETS = 16
DEFAULT_DECAY_RANK = 16


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    return d[key]


def _positive_int(v, what: str) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {what} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class BareraxLayer:
    type: str                       # "attention" | "general_delta"
    heads: int
    dim: int
    kv_heads: int = 0               # attention
    vdim: int = 0
    scale: float = 0.0
    bias_max: int = 0
    rel_buckets: int = DEFAULT_REL_BUCKETS      # rows of the distance table (from the checkpoint)
    decay_rank: int = DEFAULT_DECAY_RANK        # general_delta: inner size of w1, w2 (from the checkpoint)
    ff: int | None = None           # None: the layer has no feed-forward


@dataclass(frozen=True)
class BareraxConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    bigram_buckets: int
    bigram_mul_prev: int
    bigram_mul_cur: int
    layers: tuple[BareraxLayer, ...] = field(default_factory=tuple)
    eos_token_id: int | None = None

    # names other parts of the package ask a configuration for
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        return NO_POSITION_LIMIT

    # ---- reading and writing config.json
    @classmethod
    def from_dict(cls, d: dict, tensor_shapes: dict | None = None) -> "BareraxConfig":
        """``tensor_shapes`` (name -> shape of the checkpoint beside the file) settles the sizes that
        ``config.json`` leaves to the tensors."""
        shapes = tensor_shapes or d.get("_tensor_shapes") or {}
        vocab = _positive_int(_need(d, "vocab", "the top level"), "vocab")
        width = _positive_int(_need(d, "width", "the top level"), "width")
        eps = float(_need(_need(d, "norm", "the top level"), "eps", "'norm'"))
        if not eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        bg = _need(_need(d, "embedding", "the top level"), "bigram", "'embedding'")
        buckets = _positive_int(_need(bg, "buckets", "'embedding.bigram'"), "embedding.bigram.buckets")
        mul_prev, mul_cur = _need(bg, "mul_prev", "'embedding.bigram'"), _need(bg, "mul_cur", "'embedding.bigram'")
        for name, v in (("mul_prev", mul_prev), ("mul_cur", mul_cur)):
            if isinstance(v, bool) or not isinstance(v, int) or abs(v) >= 1 << 31:
                raise ConfigError(f"config.json: embedding.bigram.{name} must be an integer below 2^31, got {v!r}")
        raw = _need(d, "layers", "the top level")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(raw):
            where = f"layers[{i}]"
            kind = _need(e, "type", where)
            m = _need(e, "mixer", where)
            mlp = e.get("mlp")
            ff = None
            if mlp is not None:
                if _need(mlp, "kind", where + ".mlp") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not built (known: dense)")
                ff = _positive_int(_need(mlp, "ff", where + ".mlp"), where + ".mlp.ff")
            heads = _positive_int(_need(m, "heads", where + ".mixer"), where + ".mixer.heads")
            dim = _positive_int(_need(m, "dim", where + ".mixer"), where + ".mixer.dim")
            if kind == "attention":
                kv = _positive_int(m.get("kv_heads", heads), where + ".mixer.kv_heads")
                if heads % kv:
                    raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv} kv_heads")
                rel = shapes.get(f"l{i}.mix.rel")
                n_rel = int(rel[0]) if rel else int(m.get("rel_buckets", DEFAULT_REL_BUCKETS))
                bias_max = _need(m, "bias_max", where + ".mixer")
                if isinstance(bias_max, float) and bias_max.is_integer():
                    bias_max = int(bias_max)
                bias_max = _positive_int(bias_max, where + ".mixer.bias_max")
                if n_rel < 2 or bias_max <= n_rel // 2:
                    raise ConfigError(f"config.json: {where}: a distance table of {n_rel} rows needs bias_max above "
                                      f"{n_rel // 2}, got {bias_max}")
                layers.append(BareraxLayer("attention", heads, dim, kv_heads=kv,
                                           vdim=_positive_int(m.get("vdim", dim), where + ".mixer.vdim"),
                                           scale=float(_need(m, "scale", where + ".mixer")), bias_max=bias_max,
                                           rel_buckets=n_rel, ff=ff))
            elif kind == "general_delta":
                w1 = shapes.get(f"l{i}.mix.w1")
                rank = int(w1[0]) if w1 else int(m.get("decay_rank", DEFAULT_DECAY_RANK))
                layers.append(BareraxLayer("general_delta", heads, dim, decay_rank=_positive_int(rank, "decay rank"), ff=ff))
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not built (known: attention, general_delta)")
        return cls(architecture=str(d.get("architecture") or (d.get("architectures") or ["Barerax"])[0]), vocab=vocab,
                   width=width, norm_eps=eps, bigram_buckets=buckets, bigram_mul_prev=mul_prev, bigram_mul_cur=mul_cur,
                   layers=tuple(layers), eos_token_id=d.get("eos_token_id"))

    def to_hf_dict(self) -> dict:
        """The ``config.json`` dictionary; sizes that the file leaves to tensor shapes are written as well
        (``rel_buckets``, ``decay_rank``), so that the dictionary alone gives the same model back."""
        layers = []
        for L in self.layers:
            if L.type == "attention":
                mixer = {"heads": L.heads, "kv_heads": L.kv_heads, "dim": L.dim, "vdim": L.vdim, "scale": L.scale,
                         "bias_max": L.bias_max, "rel_buckets": L.rel_buckets}
            else:
                mixer = {"heads": L.heads, "dim": L.dim, "decay_rank": L.decay_rank}
            layers.append({"type": L.type, "mixer": mixer,
                           "mlp": None if L.ff is None else {"kind": "dense", "ff": L.ff}})
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps},
               "embedding": {"bigram": {"buckets": self.bigram_buckets, "mul_prev": self.bigram_mul_prev,
                                        "mul_cur": self.bigram_mul_cur}},
               "layers": layers}
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out

    to_dict = to_hf_dict

    # ---- the model as data
    def _norm(self, name: str) -> NormSpec:
        return NormSpec("layernorm", self.width, self.norm_eps, name, name + ".b")

    def model_spec(self) -> BigramDecoderSpec:
        layers, optional = [], []
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            m = p + "mix."
            if L.type == "attention":
                mixer = AttentionSpec(
                    kind="attention", hidden=self.width, n_heads=L.heads, n_kv_heads=L.kv_heads, head_dim=L.dim,
                    v_head_dim=L.vdim, window=None, scale=L.scale,
                    position=PositionSpec(kind="bucketed_bias", table=m + "rel", n_buckets=L.rel_buckets,
                                          n_heads=L.heads, max_distance=L.bias_max),
                    qk_norm=HeadNormSpec(self.norm_eps, m + "q.norm", m + "k.norm"), head_scale=m + "temp",
                    q_proj=m + "q", k_proj=m + "k", v_proj=m + "v", o_proj=m + "o")
            else:
                mixer = GeneralDeltaSpec(
                    kind="general_delta", hidden=self.width, n_heads=L.heads, head_dim=L.dim, decay_rank=L.decay_rank,
                    decay_rate=DECAY_RATE, key_eps=KEY_EPS, norm_eps=self.norm_eps, r_proj=m + "r", k_proj=m + "k",
                    v_proj=m + "v", g_proj=m + "g", a_proj=m + "a", a_bias=m + "a.b", w1=m + "w1", w2=m + "w2",
                    w0=m + "w0", out_gain=m + "norm", o_proj=m + "o")
            if L.ff is None:
                ff_norm, ff = None, None
                optional += [p + "norm2", p + "norm2.b"]      # a layer without a feed-forward has no use for them
            else:
                ff_norm = self._norm(p + "norm2")
                f = p + "mlp."
                ff = PolyNormMLPSpec(kind="polynorm_mlp", hidden=self.width, intermediate=L.ff, eps=self.norm_eps,
                                     up_proj=f + "up", up_bias=f + "up.b", down_proj=f + "down",
                                     down_bias=f + "down.b", coef=f + "act")
            layers.append(BlockSpec(kind="prenorm", mixer_norm=self._norm(p + "norm1"), mixer=mixer, ff_norm=ff_norm,
                                    feedforward=ff))
        return BigramDecoderSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden=self.width, max_positions=NO_POSITION_LIMIT,
            embedding="embed", layers=tuple(layers), schedule=tuple(ScheduleEntry(layer=i) for i in range(len(layers))),
            final_norm=self._norm("final.norm"), head=None, optional_tensors=tuple(optional),
            bigram="bigram", bigram_buckets=self.bigram_buckets, bigram_mul_prev=self.bigram_mul_prev,
            bigram_mul_cur=self.bigram_mul_cur)
