"""Typed configuration of the Kipezen decoder, read from ``config.json``.

A Kipezen model is a list of layers that put their norm on a sublayer's OUTPUT: ``x += norm1(mixer(x))`` and then
``x += norm2(ff(x))``, both reading the residual stream itself; the norm is an RMS norm whose weight is stored around
zero (multiplier ``1 + w``).  Two kinds of layer, in whatever order the file lists them:

* ``delta``: the gated delta rule, a recurrent mixer with a matrix state per head, short causal convolutions on q, k
  and v, a decay and a write strength per head and token.
* ``parallel``: two mixers side by side on the same input, their outputs added with a weight each: grouped-query
  softmax attention (biases, an RMS norm over the whole q and k projections, a rotation of neighbouring pairs of the
  first dimensions of each head, a sliding window that also keeps the first tokens of the sequence) and a recurrent
  block around a real-gated linear recurrent unit with block-diagonal gates.

The feed-forward is a mixture of experts: sigmoid router, a correction added to the scores for the choice only,
groups of experts of which the best are kept, and a shared expert with a gate of its own.  The head is the embedding
table again.

    {"architecture": "Kipezen", "vocab": V, "width": d, "norm": {"eps": e},
     "layers": [{"type": "delta", "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"}, "mlp": M | null},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "rot": {"base", "dims"},
                                    "mask": {"size", "keep_first"}},
                           "right": {"width", "blocks", "conv"}, "left_scale": a, "right_scale": b}, "mlp": M | null}]}
    M = {"kind": "moe", "expert": {"ff"}, "shared": {"ff"} | null,
         "router": {"experts", "top", "scale", "groups": {"count", "keep"}}}

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from .llama import ConfigError
from .spec import (
    AttentionSpec,
    BlockSpec,
    GatedDeltaSpec,
    GatedLinearRecurrenceSpec,
    GatedMLPSpec,
    ModelSpec,
    NormSpec,
    ParallelMixerSpec,
    PositionSpec,
    RoutedExpertsSpec,
    ScheduleEntry,
    ShortConvSpec,
)

# The design fixes these.
UNIT_VECTOR_EPS = 1e-6          # inside the root that makes q and k of the delta rule unit vectors
RECURRENCE_DECAY_SCALE = 8.0    # log a = -8 r softplus(lam) in the linear recurrent unit
ROUTE_WEIGHT_EPS = 1e-20        # added to the sum that the chosen experts' scores are divided by
NO_POSITION_LIMIT = 1 << 30


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    return d[key]


def _pos_int(v, what: str) -> int:
    if isinstance(v, float) and v.is_integer():
        v = int(v)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {what} must be a positive integer, got {v!r}")
    return v


def _nonneg_int(v, what: str) -> int:
    if isinstance(v, float) and v.is_integer():
        v = int(v)
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"config.json: {what} must be an integer of zero or more, got {v!r}")
    return v


@dataclass(frozen=True)
class KipezenMoE:
    ff: int
    experts: int
    top: int
    groups: int
    keep_groups: int
    scale: float
    shared_ff: int | None = None


@dataclass(frozen=True)
class KipezenDelta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class KipezenAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float
    window: int | None
    keep_first: int


@dataclass(frozen=True)
class KipezenRecurrence:
    width: int
    blocks: int
    conv: int


@dataclass(frozen=True)
class KipezenLayer:
    type: str                                   # "delta" | "parallel"
    delta: KipezenDelta | None = None
    left: KipezenAttention | None = None
    right: KipezenRecurrence | None = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    mlp: KipezenMoE | None = None


def _parse_mlp(mlp, where: str) -> KipezenMoE | None:
    if mlp is None:
        return None
    kind = _need(mlp, "kind", where)
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not built (known: moe)")
    r = _need(mlp, "router", where)
    ff = _pos_int(_need(_need(mlp, "expert", where), "ff", where + ".expert"), where + ".expert.ff")
    experts = _pos_int(_need(r, "experts", where + ".router"), where + ".router.experts")
    top = _pos_int(_need(r, "top", where + ".router"), where + ".router.top")
    g = r.get("groups") or {}
    groups = _pos_int(g.get("count", 1), where + ".router.groups.count")
    keep = _pos_int(g.get("keep", groups), where + ".router.groups.keep")
    if experts % groups:
        raise ConfigError(f"config.json: {where}: {experts} experts do not form {groups} equal groups")
    if keep > groups:
        raise ConfigError(f"config.json: {where}: {keep} groups cannot be kept out of {groups}")
    if top > keep * (experts // groups):
        raise ConfigError(f"config.json: {where}: {top} experts cannot be chosen from {keep} groups of {experts // groups}")
    shared = mlp.get("shared")
    shared_ff = _pos_int(_need(shared, "ff", where + ".shared"), where + ".shared.ff") if shared is not None else None
    return KipezenMoE(ff=ff, experts=experts, top=top, groups=groups, keep_groups=keep,
                      scale=float(r.get("scale", 1.0)), shared_ff=shared_ff)


def _heads(m, where: str) -> tuple[int, int, int, int]:
    heads = _pos_int(_need(m, "heads", where), where + ".heads")
    kv = _pos_int(m.get("kv_heads", heads), where + ".kv_heads")
    if heads % kv:
        raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv} kv_heads")
    dim = _pos_int(_need(m, "dim", where), where + ".dim")
    return heads, kv, dim, _pos_int(m.get("vdim", dim), where + ".vdim")


@dataclass(frozen=True)
class KipezenConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[KipezenLayer, ...] = field(default_factory=tuple)
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
    def from_dict(cls, d: dict) -> "KipezenConfig":
        vocab = _pos_int(_need(d, "vocab", "the top level"), "vocab")
        width = _pos_int(_need(d, "width", "the top level"), "width")
        eps = float(_need(_need(d, "norm", "the top level"), "eps", "'norm'"))
        if not eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        raw = _need(d, "layers", "the top level")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(raw):
            where = f"layers[{i}]"
            kind = _need(e, "type", where)
            m = _need(e, "mixer", where)
            mlp = _parse_mlp(e.get("mlp"), where + ".mlp")
            if kind == "delta":
                heads, kv, dim, vdim = _heads(m, where + ".mixer")
                conv = _pos_int(_need(m, "conv", where + ".mixer"), where + ".mixer.conv")
                layers.append(KipezenLayer("delta", delta=KipezenDelta(heads, kv, dim, vdim, conv), mlp=mlp))
            elif kind == "parallel":
                lw, rw = where + ".mixer.left", where + ".mixer.right"
                L, R = _need(m, "left", where + ".mixer"), _need(m, "right", where + ".mixer")
                heads, kv, dim, vdim = _heads(L, lw)
                rot = L.get("rot")
                rot_dims = _nonneg_int(rot.get("dims", 0), lw + ".rot.dims") if rot else 0
                if rot_dims % 2 or rot_dims > dim:
                    raise ConfigError(f"config.json: {lw}.rot.dims must be even and at most dim={dim}, got {rot_dims}")
                rot_base = float(_need(rot, "base", lw + ".rot")) if rot_dims else 0.0
                if rot_dims and not rot_base > 0:
                    raise ConfigError(f"config.json: {lw}.rot.base must be positive")
                mask = L.get("mask")
                window = _pos_int(_need(mask, "size", lw + ".mask"), lw + ".mask.size") if mask else None
                keep = _nonneg_int(mask.get("keep_first", 0), lw + ".mask.keep_first") if mask else 0
                left = KipezenAttention(heads, kv, dim, vdim, float(L.get("scale", dim ** -0.5)), rot_dims, rot_base,
                                        window, keep)
                rwidth = _pos_int(_need(R, "width", rw), rw + ".width")
                blocks = _pos_int(R.get("blocks", 1), rw + ".blocks")
                if rwidth % blocks:
                    raise ConfigError(f"config.json: {rw}: a width of {rwidth} does not split into {blocks} equal blocks")
                right = KipezenRecurrence(rwidth, blocks, _pos_int(_need(R, "conv", rw), rw + ".conv"))
                layers.append(KipezenLayer("parallel", left=left, right=right, left_scale=float(m.get("left_scale", 1.0)),
                                           right_scale=float(m.get("right_scale", 1.0)), mlp=mlp))
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not built (known: delta, parallel)")
        return cls(architecture=str(d.get("architecture") or (d.get("architectures") or ["Kipezen"])[0]), vocab=vocab,
                   width=width, norm_eps=eps, layers=tuple(layers), eos_token_id=d.get("eos_token_id"))

    def to_hf_dict(self) -> dict:
        layers = []
        for L in self.layers:
            if L.type == "delta":
                x = L.delta
                mixer = {"heads": x.heads, "kv_heads": x.kv_heads, "dim": x.dim, "vdim": x.vdim, "conv": x.conv}
            else:
                a, r = L.left, L.right
                left = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
                if a.rot_dims:
                    left["rot"] = {"base": a.rot_base, "dims": a.rot_dims}
                if a.window is not None:
                    left["mask"] = {"size": a.window, "keep_first": a.keep_first}
                mixer = {"left": left, "right": {"width": r.width, "blocks": r.blocks, "conv": r.conv},
                         "left_scale": L.left_scale, "right_scale": L.right_scale}
            mlp = None
            if L.mlp is not None:
                f = L.mlp
                mlp = {"kind": "moe", "expert": {"ff": f.ff},
                       "router": {"experts": f.experts, "top": f.top, "scale": f.scale,
                                  "groups": {"count": f.groups, "keep": f.keep_groups}},
                       "shared": None if f.shared_ff is None else {"ff": f.shared_ff}}
            layers.append({"type": L.type, "mixer": mixer, "mlp": mlp})
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out

    to_dict = to_hf_dict

    # ---- the model as data
    def _norm(self, name: str) -> NormSpec:
        return NormSpec("rmsnorm", self.width, self.norm_eps, name, unit_offset=True)

    def _delta_spec(self, m: str, x: KipezenDelta) -> GatedDeltaSpec:
        return GatedDeltaSpec(
            kind="gated_delta", hidden=self.width, n_heads=x.heads, n_kv_heads=x.kv_heads, head_dim=x.dim,
            v_head_dim=x.vdim, key_eps=UNIT_VECTOR_EPS, norm_eps=self.norm_eps, q_proj=m + "q", k_proj=m + "k",
            v_proj=m + "v", q_conv=ShortConvSpec(x.conv, m + "q.conv"), k_conv=ShortConvSpec(x.conv, m + "k.conv"),
            v_conv=ShortConvSpec(x.conv, m + "v.conv"), beta_proj=m + "b", decay_proj=m + "a", decay_log=m + "A_log",
            decay_bias=m + "dt_bias", gate_proj=m + "g", out_gain=m + "norm", o_proj=m + "o")

    def _attention_spec(self, m: str, a: KipezenAttention, out_scale: float) -> AttentionSpec:
        position = PositionSpec(kind="rotary_pairs", head_dim=a.dim, theta=a.rot_base, rot_dims=a.rot_dims) \
            if a.rot_dims else PositionSpec(kind="none")
        return AttentionSpec(
            kind="attention", hidden=self.width, n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim,
            v_head_dim=a.vdim, window=a.window, keep_first=a.keep_first if a.window is not None else 0, scale=a.scale,
            position=position, q_proj=m + "q", k_proj=m + "k", v_proj=m + "v", o_proj=m + "o", q_bias=m + "q.b",
            k_bias=m + "k.b", v_bias=m + "v.b", q_row_norm=m + "q.norm", k_row_norm=m + "k.norm",
            row_norm_eps=self.norm_eps, out_scale=out_scale)

    def _recurrence_spec(self, m: str, r: KipezenRecurrence, out_scale: float) -> GatedLinearRecurrenceSpec:
        return GatedLinearRecurrenceSpec(
            kind="gated_linear_recurrence", hidden=self.width, width=r.width, n_blocks=r.blocks,
            decay_scale=RECURRENCE_DECAY_SCALE, y_proj=m + "y", y_bias=m + "y.b", x_proj=m + "x", x_bias=m + "x.b",
            conv=ShortConvSpec(r.conv, m + "conv", m + "conv.b"), a_gate=m + "ra", a_gate_bias=m + "ra.b",
            i_gate=m + "ri", i_gate_bias=m + "ri.b", lam=m + "lam", o_proj=m + "o", out_scale=out_scale)

    def _moe_spec(self, f: str, x: KipezenMoE) -> RoutedExpertsSpec:
        shared = None
        if x.shared_ff is not None:
            shared = GatedMLPSpec(kind="gated_mlp", hidden=self.width, intermediate=x.shared_ff,
                                  gate_proj=f + "shared.gate", up_proj=f + "shared.up", down_proj=f + "shared.down")
        return RoutedExpertsSpec(
            kind="routed_experts", hidden=self.width, intermediate=x.ff, n_experts=x.experts, top=x.top,
            n_groups=x.groups, keep_groups=x.keep_groups, route_scale=x.scale, weight_eps=ROUTE_WEIGHT_EPS,
            router=f + "router", correction=f + "correction", expert_prefix=f + "e", shared=shared,
            shared_gate=f + "shared.sg" if shared is not None else None)

    def model_spec(self) -> ModelSpec:
        layers, optional = [], []
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            m = p + "mix."
            if L.type == "delta":
                mixer = self._delta_spec(m, L.delta)
            else:
                mixer = ParallelMixerSpec(kind="parallel", hidden=self.width, branches=(
                    self._attention_spec(m + "left.", L.left, L.left_scale),
                    self._recurrence_spec(m + "right.", L.right, L.right_scale)))
            if L.mlp is None:
                ff_norm, ff = None, None
                optional.append(p + "norm2")                 # a layer without a feed-forward has no use for it
            else:
                ff_norm, ff = self._norm(p + "norm2"), self._moe_spec(p + "mlp.", L.mlp)
            layers.append(BlockSpec(kind="outnorm", mixer_norm=self._norm(p + "norm1"), mixer=mixer, ff_norm=ff_norm,
                                    feedforward=ff))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden=self.width, max_positions=NO_POSITION_LIMIT,
            embedding="embed", layers=tuple(layers), schedule=tuple(ScheduleEntry(layer=i) for i in range(len(layers))),
            final_norm=self._norm("final.norm"), head=None, optional_tensors=tuple(optional))
