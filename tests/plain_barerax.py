"""Plain, slow, whole-sequence implementation of the Barerax decoder: the oracle
of the tests for that family.

Written from the design's equations, one function per mechanism, and sharing no
code with the product package: it takes the ``config.json`` dictionary and a
``{tensor name: tensor}`` dictionary, keeps no cache and no state between
calls, and recomputes every position of a sequence on the CPU in float64.
Sizes that the configuration leaves out (rows of the distance table, inner
size of the decay's low-rank pair) are taken from tensor shapes.

Notation: x is a [T, d] sequence, W y means ``y @ W.T`` for a weight stored
[out, in], ``sig`` is the logistic function.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def sig(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-x))


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * weight + bias."""
    mu = x.mean(dim=-1, keepdim=True)
    var = (x - mu).pow(2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * weight + bias


def bigram_rows(tokens: list[int], buckets: int, mul_prev: int, mul_cur: int) -> list[int]:
    """Row of the bigram table for every token: a hash of (previous, current), the extra last row at the start."""
    return [buckets if i == 0 else (tokens[i - 1] * mul_prev + tokens[i] * mul_cur) % buckets for i in range(len(tokens))]


def embed(tokens: list[int], w: dict, cfg: dict) -> torch.Tensor:
    bg = cfg["embedding"]["bigram"]
    rows = bigram_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"])
    return w["embed"][torch.tensor(tokens)] + w["bigram"][torch.tensor(rows)]


def distance_row(n: int, n_rows: int, far: int) -> int:
    """Which row of a distance table of ``n_rows`` rows serves a key n positions back: the first half of the rows
    is one distance each, the second half is spread evenly over the logarithm of the distance up to ``far``."""
    half = n_rows // 2
    if n < half:
        return n
    step = math.log(n / half) / math.log(far / half) * (n_rows - half)
    return min(n_rows - 1, half + int(math.floor(step)))


def attention(x: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Causal softmax attention with grouped keys, normed q and k, a temperature per head and a bias by distance."""
    T = x.shape[0]
    H, G, d = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    dv = m.get("vdim", d)
    q = (x @ w[p + "q"].T).view(T, H, d)
    k = (x @ w[p + "k"].T).view(T, G, d)
    v = (x @ w[p + "v"].T).view(T, G, dv)
    q = unit_rms(q, eps) * w[p + "q.norm"]
    k = unit_rms(k, eps) * w[p + "k.norm"]
    rel = w[p + "rel"]
    rows = torch.tensor([distance_row(n, rel.shape[0], m["bias_max"]) for n in range(T)])
    back = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).clamp_min(0)        # i - j where j <= i
    visible = torch.arange(T)[:, None] >= torch.arange(T)[None, :]
    out = torch.zeros(T, H, dv, dtype=x.dtype)
    for h in range(H):
        g = h // (H // G)
        score = (q[:, h] @ k[:, g].T) * m["scale"] * w[p + "temp"][h] + rel[rows[back], h]
        score = score.masked_fill(~visible, float("-inf"))
        out[:, h] = torch.softmax(score, dim=-1) @ v[:, g]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def delta_rule_states(r, k, v, decay, rate, key_eps: float = 1e-6, state=None):
    """The recurrence alone, for one head: r, k, v, decay, rate are [T, D]; returns (outputs [T, D], last state).
    S <- diag(decay) S - (rate * u)(u^T S) + k v^T with u the unit key; o = S^T r."""
    T, D = k.shape
    S = torch.zeros(D, D, dtype=k.dtype) if state is None else state.clone()
    out = []
    for t in range(T):
        u = k[t] / torch.sqrt(k[t].pow(2).sum() + key_eps)
        seen = u @ S                                       # what the state holds along the key's direction
        S = decay[t][:, None] * S - (rate[t] * u)[:, None] * seen[None, :] + k[t][:, None] * v[t][None, :]
        out.append(S.T @ r[t])
    return torch.stack(out), S


def general_delta(x: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    T = x.shape[0]
    H, D = m["heads"], m["dim"]
    r, k, v = ((x @ w[p + n].T).view(T, H, D) for n in ("r", "k", "v"))
    decay = torch.exp(-math.exp(-0.5) * sig(torch.tanh(x @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, D)
    rate = sig(x @ w[p + "a"].T + w[p + "a.b"]).view(T, H, D)
    o = torch.stack([delta_rule_states(r[:, h], k[:, h], v[:, h], decay[:, h], rate[:, h])[0] for h in range(H)], dim=1)
    o = unit_rms(o, eps).reshape(T, H * D) * w[p + "norm"] * sig(x @ w[p + "g"].T)
    return o @ w[p + "o"].T


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    return coef[0] * unit_rms(z, eps) + coef[1] * unit_rms(z * z, eps) + coef[2] * unit_rms(z * z * z, eps) + coef[3]


def feed_forward(x: torch.Tensor, w: dict, p: str, eps: float) -> torch.Tensor:
    z = x @ w[p + "up"].T + w[p + "up.b"]
    return polynorm(z, w[p + "act"], eps) @ w[p + "down"].T + w[p + "down.b"]


def forward_logits(weights: dict, cfg: dict, tokens: list[int], residuals: list | None = None, dtype=F) -> torch.Tensor:
    """Logits [T, vocab] (float32) of a whole sequence; ``residuals`` collects the stream after every layer.
    ``dtype``: the arithmetic (float64; float32 shows how much of a difference is the conditioning of the input)."""
    w = {n: (t.to(dtype) if t.is_floating_point() else t) for n, t in weights.items()}
    eps = cfg["norm"]["eps"]
    x = embed(tokens, w, cfg)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer["type"] == "attention":
            x = x + attention(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "general_delta":
            x = x + general_delta(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + feed_forward(layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps), w, p + "mlp.", eps)
        if residuals is not None:
            residuals.append(x.float())
    return (layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["embed"].T).float()
