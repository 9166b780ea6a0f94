"""Small Barerax configurations for the tests, and model folders made from them.

The configurations differ from one another in every size and constant: width, vocabulary, bigram constants, order
and number of layers, head counts and groups, key and value head sizes (equal in one model, different in the others),
rows of the distance table (even and odd), its far end, the scale, the size of the delta rule's heads (16 to 128, one
that is no power of two) and of its low-rank pair, layers with and without a feed-forward.  ``rel_buckets`` and
``decay_rank`` are only used to draw the random tensors; the ``config.json`` that is written leaves them out, as
checkpoints of the family do, and the loader reads them from the tensor shapes.
"""

from __future__ import annotations

import copy
import json
from pathlib import Path

import torch


def _att(heads, kv, dim, vdim, scale, far, rows, ff):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": far,
                      "rel_buckets": rows},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _delta(heads, dim, rank, ff):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _model(vocab, width, eps, buckets, mul_prev, mul_cur, layers):
    return {"architecture": "Barerax", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}, "layers": layers}


# attention first, values wider than keys, a delta layer without a feed-forward, kv heads equal to heads at the end
BRX_A = _model(301, 64, 1e-5, 211, 31, 5, [
    _att(4, 2, 16, 24, 0.3, 40, 12, 96),
    _delta(2, 32, 8, 80),
    _delta(3, 16, 4, None),
    _att(2, 2, 32, 16, 0.21, 64, 16, 72),
])
# one query group over one kv head, an odd number of table rows, heads of 48 (no power of two), one delta head
BRX_B = _model(389, 96, 1e-6, 97, 1, 13, [
    _delta(2, 48, 12, 136),
    _att(3, 1, 24, 40, 0.17, 30, 9, None),
    _delta(1, 32, 5, 64),
])
# keys and values of one size, heads of 64 and of 128 in the delta layers, one attention head
BRX_C = _model(270, 128, 1e-5, 401, 1000, 3, [
    _delta(1, 128, 16, 160),
    _att(1, 1, 64, 64, 0.125, 100, 20, 144),
    _delta(2, 64, 6, None),
])
# sizes that are multiples of nothing: width 100, a vocabulary of 257, heads of 24 and 40 with values of 20, five heads
# with five kv heads, a feed-forward of 100, seven table rows, one bigram bucket and a multiplier of zero
BRX_D = _model(257, 100, 1e-5, 1, 0, 3, [
    _att(5, 5, 40, 20, 0.15, 11, 7, 100),
    _delta(3, 24, 3, 52),
    _att(2, 1, 8, 4, 0.5, 50, 3, None),
])
# one layer each, for a mechanism alone
BRX_ATT = _model(200, 48, 1e-5, 50, 7, 11, [_att(6, 3, 16, 8, 0.4, 24, 10, None)])
BRX_DELTA = _model(200, 48, 1e-5, 50, 7, 11, [_delta(3, 16, 7, None)])
BRX_FF = _model(200, 48, 1e-6, 50, 7, 11, [_delta(1, 16, 3, 104)])

MODELS = {"brx_a": BRX_A, "brx_b": BRX_B, "brx_c": BRX_C, "brx_d": BRX_D, "brx_att": BRX_ATT, "brx_delta": BRX_DELTA, "brx_ff": BRX_FF}
SEEDS = {"brx_a": 11, "brx_b": 12, "brx_c": 13, "brx_d": 17, "brx_att": 14, "brx_delta": 15, "brx_ff": 16}


def stated_config(d: dict) -> dict:
    """The dictionary as a checkpoint's ``config.json`` states it: without the sizes that tensor shapes carry."""
    out = copy.deepcopy(d)
    for layer in out["layers"]:
        layer["mixer"].pop("rel_buckets", None)
        layer["mixer"].pop("decay_rank", None)
    return out


def lively(tensors: dict) -> None:
    """Random tensors drawn N(0, std) leave some mechanisms almost idle; give them values that matter: distance
    biases of order one, temperatures that differ between heads, decays and removal rates away from their middle, a
    PolyNorm with four different coefficients, norm biases of some size."""
    g = torch.Generator().manual_seed(99)
    for name, t in tensors.items():
        f = t.float()
        if name.endswith(".mix.rel"):
            f = torch.randn(f.shape, generator=g) * 1.5
        elif name.endswith(".mix.temp"):
            f = 0.5 + 1.5 * torch.rand(f.shape, generator=g)
        elif name.endswith((".mix.w0", ".mix.a.b")):
            f = torch.randn(f.shape, generator=g) * 1.5
        elif name.endswith(".mlp.act"):
            f = torch.tensor([0.9, -0.4, 0.25, 0.1])
        elif name.endswith((".norm1.b", ".norm2.b", "final.norm.b", ".up.b", ".down.b")):
            f = torch.randn(f.shape, generator=g) * 0.2
        else:
            continue
        tensors[name] = f.to(t.dtype)


def make_barerax_dir(tmp, name: str, store_dtype: str = "bfloat16", std: float = 0.08, fix=None, config: dict | None = None,
                     seed: int | None = None) -> Path:
    """A model folder with random weights for ``MODELS[name]`` (or ``config``); ``fix(tensors)`` may change them."""
    from inf_engine_b200.config import parse_config_dict
    from inf_engine_b200.parts import expected_tensors
    from inf_engine_b200.weights import random_tensors, write_safetensors

    d = config if config is not None else MODELS[name]
    out = Path(tmp) / f"{name}_{store_dtype}"
    out.mkdir(parents=True, exist_ok=True)
    cfg = parse_config_dict(d)
    tensors = random_tensors(expected_tensors(cfg.model_spec()), SEEDS.get(name, 7) if seed is None else seed, std=std,
                             store_dtype=store_dtype)
    lively(tensors)
    if fix is not None:
        fix(tensors)
    (out / "config.json").write_text(json.dumps(stated_config(d), indent=1))
    write_safetensors(out / "model.safetensors", tensors, metadata={"format": "pt"})
    return out
