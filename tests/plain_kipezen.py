"""Plain implementation of the Kipezen decoder for the tests: whole sequences, no cache, float64 unless told otherwise,
one function per mechanism, no code shared with the package.

Layers norm their sublayers' OUTPUTS: x += N1(mixer(x)), x += N2(ff(x)), N(y) = y / sqrt(mean(y^2) + eps) * (1 + w).
Mixers: the gated delta rule with short convolutions (``delta_mixer``), and softmax attention over a sliding window
that also keeps the first tokens (``window_attention``) side by side with a recurrent block around a real-gated
linear recurrent unit (``rglru_block``).  The feed-forward is a routed mixture of experts (``route``, ``moe``).
"""
import math

import torch


# ``forward_logits(..., round_to=torch.bfloat16)`` rounds where an engine that keeps activations in bfloat16 rounds: a
# sublayer's input, every projection's output, a convolution's output, what enters an output projection, an expert's
# hidden vector.  Everything else stays in the working precision.  The difference from the unrounded run is "the error
# that rounding alone causes" at each position, which the tests use as the yardstick for bfloat16 comparisons.
_ROUND = None


def _r(x):
    return x if _ROUND is None else x.to(_ROUND).to(x.dtype)


def lin(h, W, b=None):
    y = h @ W.T
    return _r(y if b is None else y + b)


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms_unit(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(x, w, bias=None):
    """x [T, C], w [C, taps]; last column multiplies the current token; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    out = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j          # column j looks `back` tokens back
        if back < T:
            out[back:] += x[:T - back] * w[:, j]
    if bias is not None:
        out = out + bias
    return out


def delta_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = _r(silu(causal_conv(lin(h, w[p + "q"]), w[p + "q.conv"]))).view(T, G, dk)
    k = _r(silu(causal_conv(lin(h, w[p + "k"]), w[p + "k.conv"]))).view(T, G, dk)
    v = _r(silu(causal_conv(lin(h, w[p + "v"]), w[p + "v.conv"]))).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(lin(h, w[p + "b"]))                                   # [T, H]
    g = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(lin(h, w[p + "a"]) + w[p + "dt_bias"]))
    gate = silu(lin(h, w[p + "g"])).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    rep = H // G
    for hh in range(H):
        S = torch.zeros(dk, dv, dtype=h.dtype)
        c = hh // rep
        for t in range(T):
            S = g[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, c])
            S = S + torch.outer(k[t, c], u)
            out[t, hh] = S.T @ q[t, c]
    out = rms_unit(out, eps) * w[p + "norm"] * gate
    return lin(_r(out.reshape(T, H * dv)), w[p + "o"])


def rotate_interleaved(x, pos, dims, base):
    """x [T, heads, dim]; the first `dims` dimensions rotate in pairs (2i, 2i+1)."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=x.dtype) / dims)
    a = pos.to(x.dtype)[:, None] * f[None, :]                                 # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def window_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = lin(h, w[p + "q"]) + w[p + "q.b"]
    k = lin(h, w[p + "k"]) + w[p + "k.b"]
    v = _r(lin(h, w[p + "v"]) + w[p + "v.b"]).view(T, G, dv)
    q = _r(rms_unit(q, eps) * w[p + "q.norm"]).view(T, H, d)
    k = _r(rms_unit(k, eps) * w[p + "k.norm"]).view(T, G, d)
    pos = torch.arange(T)
    if m.get("rot"):
        q = rotate_interleaved(q, pos, m["rot"]["dims"], m["rot"]["base"])
        k = rotate_interleaved(k, pos, m["rot"]["dims"], m["rot"]["base"])
    i, j = pos[:, None], pos[None, :]
    visible = j <= i
    if m.get("mask"):
        visible = visible & ((i - j < m["mask"]["size"]) | (j < m["mask"].get("keep_first", 0)))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    rep = H // G
    for hh in range(H):
        s = (q[:, hh] @ k[:, hh // rep].T) * m["scale"]
        s = s.masked_fill(~visible, float("-inf"))
        out[:, hh] = torch.softmax(s, -1) @ v[:, hh // rep]
    return lin(_r(out.reshape(T, H * dv)), w[p + "o"])


def rglru_block(h, w, p, m):
    T = h.shape[0]
    W, nb = m["width"], m["blocks"]
    y = gelu_tanh(lin(h, w[p + "y"], w[p + "y.b"]))
    u = _r(causal_conv(lin(h, w[p + "x"], w[p + "x.b"]), w[p + "conv"], w[p + "conv.b"]))
    bs = W // nb
    ub = u.view(T, nb, bs)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[p + "ra"], ub) + w[p + "ra.b"]).reshape(T, W)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[p + "ri"], ub) + w[p + "ri.b"]).reshape(T, W)
    log_a = -8.0 * r * torch.nn.functional.softplus(w[p + "lam"])
    a = torch.exp(log_a)
    mult = torch.sqrt(1.0 - a * a)
    S = torch.zeros(W, dtype=h.dtype)
    out = torch.zeros(T, W, dtype=h.dtype)
    for t in range(T):
        S = a[t] * S + mult[t] * i[t] * u[t]
        out[t] = S
    return lin(_r(out * y), w[p + "o"])


def parallel_mixer(h, w, p, m, eps):
    left = window_attention(h, w, p + "left.", m["left"], eps)
    right = rglru_block(h, w, p + "right.", m["right"])
    return m["left_scale"] * left + m["right_scale"] * right


def expert(h, w, p):
    return lin(_r(silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)), w[p + "down"])


def route(h, w, p, r):
    """(chosen expert ids [T, top], their weights [T, top])."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    n_g, keep = r["groups"]["count"], r["groups"]["keep"]
    per = E // n_g
    grouped = choice.view(-1, n_g, per)
    score = grouped.topk(min(2, per), dim=-1).values.sum(-1)                  # [T, groups]
    best = score.topk(keep, dim=-1).indices
    allowed = torch.zeros_like(score, dtype=torch.bool).scatter_(1, best, True)
    masked = choice.masked_fill(~allowed[:, :, None].expand(-1, -1, per).reshape(-1, E), float("-inf"))
    ids = masked.topk(top, dim=-1).indices
    wts = s.gather(1, ids)
    wts = wts / (wts.sum(-1, keepdim=True) + 1e-20) * r["scale"]
    return ids, wts


def moe(h, w, p, m):
    ids, wts = route(h, w, p, m["router"])
    out = torch.zeros_like(h)
    for e in range(m["router"]["experts"]):
        tok, slot = (ids == e).nonzero(as_tuple=True)
        if tok.numel():
            out[tok] += wts[tok, slot][:, None] * expert(h[tok], w, f"{p}e{e}.")
    if m.get("shared") is not None:
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * expert(h, w, p + "shared.")
    return out


def forward_logits(w, cfg, tokens, dtype=torch.float64, layers_out=None, round_to=None):
    global _ROUND
    _ROUND = round_to
    try:
        return _forward_logits(w, cfg, tokens, dtype, layers_out)
    finally:
        _ROUND = None


def _forward_logits(w, cfg, tokens, dtype, layers_out):
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        if L["type"] == "delta":
            y = delta_mixer(_r(x), w, p + "mix.", L["mixer"], eps)
        elif L["type"] == "parallel":
            y = parallel_mixer(_r(x), w, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + norm_one_plus(y, w[p + "norm1"], eps)
        if L.get("mlp") is not None:
            x = x + norm_one_plus(moe(_r(x), w, p + "mlp.", L["mlp"]), w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return _r(norm_one_plus(x, w["final.norm"], eps)) @ w["embed"].T
