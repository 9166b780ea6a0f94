"""Small Kipezen configurations for the tests, and model folders made from them.

They differ from one another in every size and constant: width, vocabulary, order and number of layers, head counts
and groups of both mixers, key and value head sizes (equal and unequal, no powers of two among them), convolution
lengths (2 to 5), the rotated share of a head (all of it, a part, none), windows and kept first tokens (none, a few,
more than a page), the recurrent block's width and number of gate blocks (one to five), the two branch weights,
experts (groups of one, of several, all groups kept, one kept, two of three kept; one to three experts a token), a
shared expert of its own size or none, layers without a feed-forward.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch


def _moe(ff, experts, top, groups, keep, scale, shared):
    return {"kind": "moe", "expert": {"ff": ff}, "shared": None if shared is None else {"ff": shared},
            "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}}


def _delta(heads, kv, dim, vdim, conv, mlp):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def _par(heads, kv, dim, vdim, scale, rot, window, keep, width, blocks, conv, ls, rs, mlp):
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        left["rot"] = {"base": rot[0], "dims": rot[1]}
    if window is not None:
        left["mask"] = {"size": window, "keep_first": keep}
    return {"type": "parallel", "mixer": {"left": left, "right": {"width": width, "blocks": blocks, "conv": conv},
                                          "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def _model(vocab, width, eps, layers):
    return {"architecture": "Kipezen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# parallel first; values narrower than keys; three experts a token from two of three groups; a delta layer without mlp
KPZ_A = _model(211, 64, 1e-5, [
    _par(4, 2, 16, 8, 0.31, (10000.0, 8), 21, 3, 48, 3, 3, 0.7, 1.3, _moe(40, 12, 3, 3, 2, 1.7, 24)),
    _delta(4, 2, 16, 24, 3, None),
    _delta(2, 2, 24, 16, 2, _moe(56, 6, 1, 1, 1, 1.0, None)),
])
# one kv head under three query heads, the whole head rotated, a window shorter than a page, no kept tokens,
# one gate block, groups of one expert each, a shared expert larger than the routed ones
KPZ_B = _model(157, 96, 1e-6, [
    _delta(3, 1, 20, 12, 5, _moe(24, 5, 2, 5, 3, 2.5, 72)),
    _par(3, 1, 24, 40, 0.2, (500.0, 24), 7, 0, 40, 1, 2, 1.0, 0.5, None),
    _delta(1, 1, 32, 32, 4, _moe(32, 8, 2, 2, 1, 0.9, 32)),
])
# heads of 64 with values of 64, five gate blocks, more kept tokens than a page of 8 holds, no rotation at all in
# the second parallel layer and no window in it either (every key visible)
KPZ_C = _model(300, 128, 1e-5, [
    _par(2, 2, 64, 64, 0.125, (30000.0, 16), 33, 11, 80, 5, 4, 1.1, 0.9, _moe(48, 4, 2, 2, 2, 2.0, 16)),
    _delta(2, 1, 64, 64, 4, _moe(16, 16, 2, 4, 1, 1.5, 48)),
    _par(2, 1, 32, 48, 0.18, None, None, 0, 64, 2, 3, 0.6, 0.6, None),
])
# sizes that are multiples of nothing: width 100, heads of 10 and 6, a recurrent width of 35 in 5 blocks of 7
KPZ_D = _model(131, 100, 1e-5, [
    _delta(5, 5, 10, 6, 3, _moe(20, 9, 2, 3, 1, 3.0, 10)),
    _par(5, 5, 10, 6, 0.4, (100.0, 6), 13, 2, 35, 5, 5, 1.5, 0.8, _moe(12, 3, 3, 1, 1, 1.0, None)),
])
# one mechanism each
KPZ_DELTA = _model(120, 48, 1e-5, [_delta(3, 1, 16, 24, 4, None)])
KPZ_ATT = _model(120, 48, 1e-5, [_par(6, 3, 16, 8, 0.35, (1000.0, 12), 19, 4, 16, 2, 2, 1.0, 0.0, None)])
KPZ_REC = _model(120, 48, 1e-5, [_par(1, 1, 8, 8, 0.35, None, 5, 0, 56, 4, 4, 0.0, 1.0, None)])
KPZ_MOE = _model(120, 48, 1e-6, [_delta(1, 1, 8, 8, 2, _moe(28, 10, 2, 5, 2, 2.2, 20))])

MODELS = {"kpz_a": KPZ_A, "kpz_b": KPZ_B, "kpz_c": KPZ_C, "kpz_d": KPZ_D, "kpz_delta": KPZ_DELTA, "kpz_att": KPZ_ATT,
          "kpz_rec": KPZ_REC, "kpz_moe": KPZ_MOE}
SEEDS = {"kpz_a": 31, "kpz_b": 32, "kpz_c": 33, "kpz_d": 34, "kpz_delta": 35, "kpz_att": 36, "kpz_rec": 37, "kpz_moe": 38}


def lively(tensors: dict) -> None:
    """Random tensors drawn N(0, std) leave some mechanisms almost idle; give them values that matter: norm weights
    around zero of some size, biases of order one tenth, decays that reach close to one and well below it, router
    corrections that change the choice, row-norm gains that make the attention sharp."""
    g = torch.Generator().manual_seed(77)
    for name, t in tensors.items():
        f = t.float()
        if name.endswith((".norm1", ".norm2")) or name == "final.norm":
            f = torch.randn(f.shape, generator=g) * 0.2            # stored around zero: the multiplier is 1 + w
        elif name.endswith((".q.norm", ".k.norm")):
            f = 1.5 + torch.rand(f.shape, generator=g)
        elif name.endswith(".mix.norm"):
            f = 0.7 + 0.6 * torch.rand(f.shape, generator=g)
        elif name.endswith((".q.b", ".k.b", ".v.b", ".y.b", ".x.b", ".conv.b", ".ra.b", ".ri.b")):
            f = torch.randn(f.shape, generator=g) * 0.3
        elif name.endswith(".lam"):
            f = torch.linspace(-6.0, 0.5, f.numel()).reshape(f.shape)      # decays from 1 - 1e-5 to almost nothing
        elif name.endswith(".A_log"):
            f = torch.linspace(-4.0, 0.5, f.numel()).reshape(f.shape)
        elif name.endswith(".dt_bias"):
            f = torch.linspace(-3.0, 1.0, f.numel()).reshape(f.shape)
        elif name.endswith(".correction"):
            f = torch.randn(f.shape, generator=g) * 0.3
        elif name.endswith((".ra", ".ri", ".mix.b", ".mix.a", ".router", ".shared.sg")):
            f = f * 6
        elif name.endswith(".conv"):
            f = torch.randn(f.shape, generator=g) * 0.5
        else:
            continue
        tensors[name] = f.to(t.dtype)


def decisive_routers(tensors: dict) -> None:
    """Corrections two apart, in an order that differs from layer to layer: which experts a token takes is then
    settled by the corrections alone (scores lie between 0 and 1), while the weights of the chosen ones still follow
    the token.  For comparisons in bfloat16, where rounding would otherwise flip a close choice now and then and a
    flipped expert is no rounding error; the 32-bit comparisons keep routers whose choice follows the token."""
    g = torch.Generator().manual_seed(5)
    for name, t in tensors.items():
        if name.endswith(".correction"):
            tensors[name] = (2.0 * torch.randperm(t.numel(), generator=g).float()).to(t.dtype)


def make_kipezen_dir(tmp, name: str, store_dtype: str = "bfloat16", std: float = 0.08, fix=None, config: dict | None = None,
                     seed: int | None = None, decisive: bool = False) -> Path:
    """A model folder with random weights for ``MODELS[name]`` (or ``config``); ``fix(tensors)`` may change them;
    ``decisive``: see ``decisive_routers``."""
    from inf_engine_b200.config import parse_config_dict
    from inf_engine_b200.parts import expected_tensors
    from inf_engine_b200.weights import random_tensors, write_safetensors

    d = config if config is not None else MODELS[name]
    out = Path(tmp) / f"{name}_{store_dtype}{'_decisive' if decisive else ''}"
    out.mkdir(parents=True, exist_ok=True)
    cfg = parse_config_dict(d)
    tensors = random_tensors(expected_tensors(cfg.model_spec()), SEEDS.get(name, 7) if seed is None else seed, std=std,
                             store_dtype=store_dtype)
    lively(tensors)
    if decisive:
        decisive_routers(tensors)
    if fix is not None:
        fix(tensors)
    (out / "config.json").write_text(json.dumps(d, indent=1))
    write_safetensors(out / "model.safetensors", tensors, metadata={"format": "pt"})
    return out
