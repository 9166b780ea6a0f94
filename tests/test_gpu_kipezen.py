"""The Kipezen family on the GPU against the plain implementation: each new kernel alone, each mechanism alone in a
one-layer model, whole prompts against token-by-token decoding and portions down to two tokens, batches of unequal
requests with pages and state slots used again, the first tokens of a sequence, keys just inside and just outside the
window and the kept first tokens in prompts and in decoding, a far key that must stand out, long decoding, greedy
generation through the engine and its scheduler, the command line and the trace replay.  Every test runs in 32-bit
and in bfloat16."""

import math
import os
import subprocess
import sys

import pytest
import torch

import plain_kipezen as plain
from kipezen_models import MODELS, make_kipezen_dir
import helpers
from helpers import BF16_NEAR_TIE, plain_inputs, random_tokens, run_trace

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# bfloat16: every sublayer's output is divided by its own root mean square before it joins the residual, each
# delta-rule head by its own; where such an output happens to be small (the first tokens of a sequence, above all) the
# rounding of its inputs enters at full size, and no fixed bound tells that from a fault.  So a row's bound is three
# times the error that rounding alone causes there (the plain model with bfloat16 rounding at the places where the
# engine rounds, ``plain.forward_logits(round_to=...)``, against itself without) plus a floor.  Measured on a B200:
# worst row 0.04 to 0.07 of the row's norm on well-conditioned rows, means 0.015 to 0.036.  32-bit: the same division
# lets rounding that is small against a sublayer's inputs through at full size where the output is small; measured
# worst difference 1.2 times the shared bound, on one row of some 3,000.
F32_NOISE = 2.0
BF16_FLOOR = 0.03
NEAR_TIE_NOISE = 4.0


class Ref:
    """Plain logits of a sequence and, for bfloat16 comparisons, the relative error per row that rounding alone causes."""

    def __init__(self, logits, noise=None):
        self.logits, self.noise = logits, noise

    def __getitem__(self, idx):
        return Ref(self.logits[idx], None if self.noise is None else self.noise[idx])


def reference(w, cfg, toks, dtype):
    logits = plain.forward_logits(w, cfg, toks)
    if dtype == "float32":
        return Ref(logits)
    rounded = plain.forward_logits(w, cfg, toks, round_to=torch.bfloat16)
    return Ref(logits, (rounded - logits).norm(dim=-1) / logits.norm(dim=-1).clamp_min(1e-6))


def assert_close(got, ref, dtype, what="", noise=1.0):
    if not isinstance(ref, Ref):
        ref = Ref(ref, torch.zeros(ref.shape[0], dtype=torch.float64) if dtype != "float32" else None)
    got, want = got.double().cpu(), ref.logits.double().cpu()
    assert got.shape == want.shape and torch.isfinite(got).all(), what
    if dtype == "float32":
        tol = F32_NOISE * helpers.tolerance(dtype, want)
        worst = float((got - want).abs().max())
        helpers.STATS.append({"what": what, "dtype": dtype, "max_abs": worst, "tol": tol})
        assert worst <= tol, f"{what}: max |diff| {worst:.3e} > {tol:.3e}; worst row {int((got - want).abs().max(dim=-1).values.argmax())}"
        return
    rel = (got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-6)
    bound = noise * (3.0 * ref.noise + BF16_FLOOR)
    helpers.STATS.append({"what": what, "dtype": dtype, "rows": int(rel.numel()), "row_max": float(rel.max()),
                          "row_mean": float(rel.mean()), "worst_of_bound": float((rel / bound).max()),
                          "rounding_alone_mean": float(ref.noise.mean())})
    bad = (rel > bound).nonzero().flatten().tolist()
    assert not bad, (f"{what}: relative error of row {bad[0]} is {float(rel[bad[0]]):.3e} > {float(bound[bad[0]]):.3e} "
                     f"(rounding alone: {float(ref.noise[bad[0]]):.3e}; rows over their bound: {bad[:20]})")
    if rel.numel() >= 8:
        assert float(rel.mean()) <= noise * (2.0 * float(ref.noise.mean()) + BF16_FLOOR / 2), \
            f"{what}: mean relative row error {float(rel.mean()):.3e}, rounding alone {float(ref.noise.mean()):.3e}"


def model_dir(tmp_path, name, dtype, **kw):
    """bfloat16 comparisons run on routers whose choice rounding cannot flip (``kipezen_models.decisive_routers``)."""
    return make_kipezen_dir(tmp_path, name, decisive=dtype == "bfloat16", **kw)


def k():
    from inf_engine_b200 import kernels
    return kernels


def dev_i32(x):
    return torch.as_tensor(x, dtype=torch.int32).to(DEV)


def close(got, want, dtype, rel=2e-2, atol=2e-5):
    """float32: element by element against the float64 oracle; bfloat16: against the largest value of the tensor."""
    got, want = got.double().cpu(), want.double().cpu()
    if dtype == "float32":
        return torch.allclose(got, want, atol=atol, rtol=2e-5)
    return float((got - want).abs().max()) <= rel * max(1.0, float(want.abs().max()))


# =============================================================== kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_outnorm_accumulate_kernel(dtype):
    torch.manual_seed(1)
    act = TORCH[dtype]
    n, d = 6, 100
    res = torch.randn(n, d)
    y = (torch.randn(n, d) * 3).to(act)
    gain = 1.0 + 0.2 * torch.randn(d)
    want = res.double() + plain.rms_unit(y.double(), 1e-5) * gain.double()
    wide = torch.zeros(n, d + 28, device=DEV, dtype=act)             # a row-strided input
    wide[:, :d] = y.to(DEV)
    r = res.to(DEV)
    nxt = torch.empty(n, d, device=DEV, dtype=act)
    k().outnorm_accumulate(r, wide[:, :d], gain.to(DEV), 1e-5, nxt)
    assert close(r, want, "float32") and close(nxt, want, dtype)
    r2 = res.to(DEV)
    k().outnorm_accumulate(r2, y.float().to(DEV), gain.to(act).to(DEV), 1e-5, None)       # float32 rows, gain as stored
    assert close(r2, res.double() + plain.rms_unit(y.double(), 1e-5) * gain.to(act).double(), "float32")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps, channels, bias, act_fn", [(4, 70, False, "silu"), (2, 33, True, None), (5, 8, True, "silu"),
                                                           (1, 40, False, None)])
def test_causal_conv_kernel_carries_its_inputs_over_any_cut(dtype, taps, channels, bias, act_fn):
    """Two requests in one batch, cut into steps of unequal sizes (also shorter than the filter), in slots that are
    not their order; a third slot holds another sequence's inputs and must stay as it is."""
    torch.manual_seed(2)
    act = TORCH[dtype]
    lens = [23, 9]
    xs = [torch.randn(n, channels).to(act) for n in lens]
    w = (torch.randn(channels, taps) * 0.5).to(act)
    b = torch.randn(channels).to(act) if bias else None
    want = []
    for x in xs:
        y = plain.causal_conv(x.double(), w.double(), b.double() if bias else None)
        want.append(plain.silu(y) if act_fn == "silu" else y)
    state = torch.zeros(3, max(taps - 1, 0), channels, device=DEV, dtype=act)
    state[1] = 7.0
    slots = [2, 0]
    cuts = [[1, 2, 1, 5, 3, 11], [2, 1, 1, 5]]
    got = [[], []]
    at = [0, 0]
    for step in range(6):
        rows, q_start, sl, who = [], [0], [], []
        for r in range(2):
            if step < len(cuts[r]):
                n = cuts[r][step]
                rows.append(xs[r][at[r]:at[r] + n])
                at[r] += n
                q_start.append(q_start[-1] + n)
                sl.append(slots[r])
                who.append((r, n))
        x = torch.zeros(q_start[-1], channels + 16, device=DEV, dtype=act)
        x[:, :channels] = torch.cat(rows).to(DEV)
        out = torch.empty(q_start[-1], channels, device=DEV, dtype=act)
        k().causal_conv(x[:, :channels], w.to(DEV), b.to(DEV) if bias else None, state, out, dev_i32(q_start), dev_i32(sl),
                        len(sl), activation=act_fn)
        o = 0
        for r, n in who:
            got[r].append(out[o:o + n].cpu())
            o += n
    for r in range(2):
        assert close(torch.cat(got[r]), want[r], dtype), f"request {r}"
    assert bool((state[1] == 7.0).all())
    if taps > 1:      # what is left behind is the last inputs, oldest first
        assert torch.equal(state[2].cpu(), xs[0][-(taps - 1):]) and torch.equal(state[0].cpu(), xs[1][-(taps - 1):])


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_recurrence_kernel_with_decays_next_to_one(dtype):
    """Channels whose decay runs from 1 - 1e-6 to almost nothing, 300 tokens in portions, from a state that is not
    zero; a padding row; a run that may not write."""
    torch.manual_seed(3)
    act = TORCH[dtype]
    T, W = 300, 72
    u, y_pre = torch.randn(T, W).to(act), torch.randn(T, W).to(act)
    r_pre, i_pre = torch.randn(T, W) * 2, torch.randn(T, W) * 2
    rb, ib = torch.randn(W).to(act), torch.randn(W).to(act)
    lam = torch.linspace(-9.0, 1.0, W).to(act)
    S0 = torch.randn(W)
    r = torch.sigmoid(r_pre.double() + rb.double())
    i = torch.sigmoid(i_pre.double() + ib.double())
    log_a = -8.0 * r * torch.nn.functional.softplus(lam.double())
    a, mult = torch.exp(log_a), torch.sqrt(-torch.expm1(2 * log_a))
    S, want = S0.double(), []
    for t in range(T):
        S = a[t] * S + mult[t] * i[t] * u[t].double()
        want.append(0.8 * S * plain.gelu_tanh(y_pre[t].double()))
    want = torch.stack(want)
    state = torch.zeros(3, W, device=DEV)
    state[1] = S0.to(DEV)
    gates = torch.cat([r_pre, i_pre], dim=1).to(DEV)
    out = torch.empty(T + 1, W, device=DEV, dtype=act)
    ud, yd = torch.cat([u, u[:1]]).to(DEV), torch.cat([y_pre, y_pre[:1]]).to(DEV)
    p = 0
    for n in [1, 2, 5, 64, 3, 225]:
        q_start, sl = dev_i32([0, n, n + 1]), dev_i32([1, -1])          # the request, then a padding row
        rows = torch.cat([gates[p:p + n], gates[:1]])
        o = torch.empty(n + 1, W, device=DEV, dtype=act)
        k().linear_recurrence(torch.cat([ud[p:p + n], ud[:1]]), torch.cat([yd[p:p + n], yd[:1]]), rows[:, :W], rows[:, W:],
                              rb.to(DEV), ib.to(DEV), lam.to(DEV), state, o, q_start, sl, 2, 8.0, 0.8)
        out[p:p + n] = o[:n]
        assert bool((o[n] == 0).all())
        p += n
    assert close(out[:T], want, dtype, atol=5e-5)
    assert close(state[1], S, "float32", atol=5e-5) and bool((state[0] == 0).all()) and bool((state[2] == 0).all())
    before = state.clone()
    k().linear_recurrence(ud[:4], yd[:4], gates[:4, :W], gates[:4, W:], rb.to(DEV), ib.to(DEV), lam.to(DEV), state,
                          out[:4], dev_i32([0, 4]), dev_i32([1]), 1, 8.0, 0.8, write_state=False)
    assert torch.equal(state, before)


def plain_gated_delta(q, kk, v, b_pre, a_pre, gate, a_log, dt_bias, gain, S0, H, G, dk, dv, eps):
    T = q.shape[0]
    q, kk, v = q.double().view(T, G, dk), kk.double().view(T, G, dk), v.double().view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    kk = kk / torch.sqrt((kk * kk).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(b_pre.double())
    g = torch.exp(-torch.exp(a_log.double()) * torch.nn.functional.softplus(a_pre.double() + dt_bias.double()))
    out = torch.zeros(T, H, dv, dtype=torch.float64)
    S_end = []
    for h in range(H):
        S = S0[h].double().clone()
        c = h // (H // G)
        for t in range(T):
            S = g[t, h] * S
            u = beta[t, h] * (v[t, h] - S.T @ kk[t, c])
            S = S + torch.outer(kk[t, c], u)
            out[t, h] = S.T @ q[t, c]
        S_end.append(S)
    out = plain.rms_unit(out, eps) * gain.double() * plain.silu(gate.double().view(T, H, dv))
    return out.reshape(T, H * dv), torch.stack(S_end)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dk, dv, heads, kv", [(16, 24, 4, 2), (20, 12, 3, 1), (64, 64, 2, 2), (10, 6, 5, 5), (128, 48, 2, 1)])
def test_gated_delta_kernel(dtype, dk, dv, heads, kv):
    """Key and value heads of unequal sizes, heads that share q and k, 45 tokens in portions from a state that is not
    zero, decays from almost one to a tenth, a padding row, a run that may not write."""
    torch.manual_seed(4)
    act = TORCH[dtype]
    T, H, G = 45, heads, kv
    q, kk, v = (torch.randn(T, G * dk).to(act), torch.randn(T, G * dk).to(act), torch.randn(T, H * dv).to(act))
    b_pre, a_pre, gate = torch.randn(T, H).to(act) * 2, torch.randn(T, H).to(act) * 2, torch.randn(T, H * dv).to(act)
    a_log, dt_bias = torch.linspace(-5.0, 0.8, H).to(act), torch.linspace(-2.0, 1.0, H).to(act)
    gain = (1 + 0.3 * torch.randn(dv)).to(act)
    S0 = torch.randn(H, dk, dv) * 0.3
    want, S_end = plain_gated_delta(q, kk, v, b_pre, a_pre, gate, a_log, dt_bias, gain, S0, H, G, dk, dv, 1e-5)
    state = torch.zeros(3, H, dk, dv, device=DEV)
    state[2] = S0.to(DEV)
    buf = torch.zeros(T, 2 * G * dk + 2 * H * dv + 2 * H + 8, device=DEV, dtype=act)       # columns of one buffer
    c = [0, G * dk, 2 * G * dk, 2 * G * dk + H * dv, 2 * G * dk + 2 * H * dv, 2 * G * dk + 2 * H * dv + H]
    for t_, c0 in zip((q, kk, v, gate, b_pre, a_pre), c):
        buf[:, c0:c0 + t_.shape[1]] = t_.to(DEV)
    out = torch.empty(T, H * dv, device=DEV, dtype=act)
    p = 0
    for n in [1, 2, 17, 1, 24]:
        rows = torch.cat([buf[p:p + n], buf[:1]])
        o = torch.empty(n + 1, H * dv, device=DEV, dtype=act)
        k().gated_delta(rows[:, c[0]:c[1]], rows[:, c[1]:c[2]], rows[:, c[2]:c[3]], rows[:, c[4]:c[4] + H],
                        rows[:, c[5]:c[5] + H], rows[:, c[3]:c[4]], a_log.to(DEV), dt_bias.to(DEV), gain.to(DEV), state, o,
                        dev_i32([0, n, n + 1]), dev_i32([2, -1]), 2, H, G, dk, dv, 1e-6, 1e-5)
        out[p:p + n] = o[:n]
        assert bool((o[n] == 0).all())
        p += n
    assert close(out, want, dtype, rel=3e-2, atol=1e-4)
    assert close(state[2], S_end, "float32", atol=1e-4) and bool((state[:2] == 0).all())
    before = state.clone()
    k().gated_delta(buf[:3, c[0]:c[1]], buf[:3, c[1]:c[2]], buf[:3, c[2]:c[3]], buf[:3, c[4]:c[4] + H], buf[:3, c[5]:c[5] + H],
                    buf[:3, c[3]:c[4]], a_log.to(DEV), dt_bias.to(DEV), gain.to(DEV), state, out[:3], dev_i32([0, 3]),
                    dev_i32([2]), 1, H, G, dk, dv, 1e-6, 1e-5, write_state=False)
    assert torch.equal(state, before)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd, hdv, rot", [(16, 8, 12), (24, 40, 24), (10, 6, 0)])
def test_rownorm_rotate_write_kernel(dtype, hd, hdv, rot):
    """Positions up to a million: the angle must come out of the position and the frequency without losing digits."""
    torch.manual_seed(5)
    act = TORCH[dtype]
    n, H, G, ps = 6, 4, 2, 8
    q, kk, v = torch.randn(n, H * hd).to(act), torch.randn(n, G * hd).to(act), torch.randn(n, G * hdv).to(act)
    qb, kb, vb = torch.randn(H * hd).to(act), torch.randn(G * hd).to(act), torch.randn(G * hdv).to(act)
    qg, kg = (1.5 + torch.rand(H * hd)).to(act), (1.5 + torch.rand(G * hd)).to(act)
    pos = torch.tensor([0, 1, 7, 137, 4095, 1000003])
    base = 50000.0
    wq = plain.rms_unit(q.double() + qb.double(), 1e-5) * qg.double()
    wk = plain.rms_unit(kk.double() + kb.double(), 1e-5) * kg.double()
    wq, wk = wq.view(n, H, hd), wk.view(n, G, hd)
    if rot:
        wq, wk = plain.rotate_interleaved(wq, pos, rot, base), plain.rotate_interleaved(wk, pos, rot, base)
    wv = (v.double() + vb.double()).view(n, G, hdv)
    inv_freq = (base ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1))).to(DEV) if rot else None
    slots = [5, 0, 9, 23, 14, 8]
    kpool = torch.full((3, G, ps, hd), float("nan"), device=DEV, dtype=act)
    vpool = torch.full((3, G, ps, hdv), float("nan"), device=DEV, dtype=act)
    buf = torch.zeros(n, (H + G) * hd + G * hdv, device=DEV, dtype=act)
    buf[:, :H * hd], buf[:, H * hd:(H + G) * hd], buf[:, (H + G) * hd:] = q.to(DEV), kk.to(DEV), v.to(DEV)
    k().rownorm_rotate_write(buf[:, :H * hd], buf[:, H * hd:(H + G) * hd], buf[:, (H + G) * hd:], qb.to(DEV), kb.to(DEV),
                             vb.to(DEV), qg.to(DEV), kg.to(DEV), 1e-5, inv_freq, rot, dev_i32(pos.tolist()), dev_i32(slots),
                             kpool, vpool, H, G, hd, hdv, ps)
    assert close(buf[:, :H * hd].view(n, H, hd), wq, dtype, atol=1e-5)
    for i, s in enumerate(slots):
        assert close(kpool[s // ps, :, s % ps], wk[i], dtype, atol=1e-5) and close(vpool[s // ps, :, s % ps], wv[i], dtype)
    written = torch.zeros(3 * ps, dtype=torch.bool)
    written[slots] = True
    assert bool(torch.isnan(kpool.float()).all(dim=-1).all(dim=1).view(-1).cpu()[~written].all())     # nothing else was touched


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, "tiles", "rows"])
def test_a_key_stands_out_only_where_the_window_and_the_kept_tokens_allow(dtype, decode):
    """One key is made to stand out (its key and the last query share a large component); the last query must return
    that key's value when the key is the last one inside the window, the last kept first token, or at a page border
    inside, and must not when it is the first one outside the window or the first token that is not kept."""
    torch.manual_seed(6)
    act = TORCH[dtype]
    H, G, hd, hdv, ps, window, keep, scale = 4, 2, 16, 8, 8, 21, 5, 0.3
    T = 75
    for target, seen in [(T - window, True), (T - window - 1, False), (keep - 1, True), (keep, False), (0, True),
                         (T - 1, True), (T - 1 - ps, True), (56, True), (55, True), (40, False), (7, False), (8, False)]:
        q, kx, v = torch.randn(T, H * hd), torch.randn(T, G * hd), torch.randn(T, G * hdv)
        kx.view(T, G, hd)[target, :, 3] += 14.0
        q.view(T, H, hd)[T - 1, :, 3] += 14.0
        q, kx, v = q.to(act), kx.to(act), v.to(act)
        qq, kk, vv = q.double().view(T, H, hd), kx.double().view(T, G, hd), v.double().view(T, G, hdv)
        j = torch.arange(T)
        visible = (T - 1 - j < window) | (j < keep)
        want = torch.zeros(H, hdv, dtype=torch.float64)
        for h in range(H):
            s = ((kk[:, h // 2] @ qq[T - 1, h]) * scale).masked_fill(~visible, float("-inf"))
            want[h] = 0.7 * torch.softmax(s, 0) @ vv[:, h // 2]
        n_pages = -(-T // ps)
        order = list(reversed(range(n_pages)))
        kpool = torch.full((n_pages, G, ps, hd), float("nan"), device=DEV, dtype=act)
        vpool = torch.full((n_pages, G, ps, hdv), float("nan"), device=DEV, dtype=act)
        table = [order[p] for p in range(n_pages)]
        # pages wholly behind the window that hold no kept token are given back (as the cache manager does)
        for p in range(n_pages):
            if (p + 1) * ps <= T - window and p * ps >= keep:
                table[p] = -1
        slot_map = dev_i32([order[p // ps] * ps + p % ps for p in range(T)])
        qd = q.to(DEV).clone()
        k().rownorm_rotate_write(qd, kx.to(DEV), v.to(DEV), None, None, None, None, None, 0.0, None, 0,
                                 dev_i32(list(range(T))), slot_map, kpool, vpool, H, G, hd, hdv, ps)
        for p in range(n_pages):
            if table[p] < 0:
                kpool[order[p]] = float("nan")
                vpool[order[p]] = float("nan")
        out = torch.empty(T, H * hdv, device=DEV, dtype=act)
        table_dev = dev_i32([table]).view(1, n_pages)
        if decode == "rows":        # the kernel of decode steps: a block per (token, head), the keys split over its warps
            k().attention_rows(qd[T - 1:], out[T - 1:], kpool, vpool, table_dev, dev_i32([0, 1]), dev_i32([T - 1]), 1, 16,
                               H, G, hd, ps, window, scale, None, None, hdv, keep, 0.7)
        elif decode:
            k().attention_general(qd[T - 1:], out[T - 1:], kpool, vpool, table_dev, dev_i32([0, 1]), dev_i32([T - 1]),
                                  dev_i32([0]), dev_i32([0]), 1, H, G, hd, ps, window, scale, None, None, hdv, keep, 0.7)
        else:
            n_tiles = -(-T * (H // G) // 32)
            k().attention_general(qd, out, kpool, vpool, table_dev, dev_i32([0, T]), dev_i32([0]), dev_i32([0] * n_tiles),
                                  dev_i32([32 * i for i in range(n_tiles)]), n_tiles, H, G, hd, ps, window, scale, None,
                                  None, hdv, keep, 0.7)
        got = out[T - 1].view(H, hdv)
        assert close(got, want, dtype), f"key {target}"
        stood_out = float((want[0] / 0.7 - vv[target, 0]).abs().max()) < 0.3
        assert stood_out == seen, f"key {target}: the plain weights say {stood_out}"


@pytest.mark.parametrize("experts, top, groups, keep", [(12, 3, 3, 2), (5, 2, 5, 3), (16, 2, 4, 1), (6, 1, 1, 1), (40, 4, 8, 3),
                                                         (9, 2, 3, 1)])
def test_route_kernel_chooses_what_the_plain_rule_chooses(experts, top, groups, keep):
    """Corrections of the scores' own size (some negative enough to make choice scores negative), so that the choice
    differs from the plain top of the scores; the weights come from the scores without the correction."""
    torch.manual_seed(7)
    n = 200
    logits = torch.randn(n, experts + 3) * 2
    corr = torch.randn(experts) * 0.4 - 0.6
    w = {"r.router": torch.eye(experts, dtype=torch.float64), "r.correction": corr.double()}
    r = {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": groups, "keep": keep}}
    ids_want, wts_want = plain.route(logits[:, :experts].double(), w, "r.", r)
    ids = torch.empty(n, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(n, top, device=DEV)
    gate = torch.empty(n, device=DEV)
    k().moe_route(logits.to(DEV), corr.to(DEV), ids, wts, gate, experts, top, groups, keep, 2.5, 1e-20, gate_col=experts + 1)
    assert torch.equal(ids.cpu().long().sort(-1).values, ids_want.sort(-1).values)
    got = torch.zeros(n, experts, dtype=torch.float64).scatter_(1, ids.cpu().long(), wts.cpu().double())
    want = torch.zeros(n, experts, dtype=torch.float64).scatter_(1, ids_want, wts_want)
    assert torch.allclose(got, want, atol=1e-5)
    assert torch.allclose(gate.cpu().double(), torch.sigmoid(logits[:, experts + 1].double()), atol=1e-6)
    assert len(set(ids.cpu().flatten().tolist())) >= min(experts, 3)             # the correction did not settle everything


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, ff", [(40, 52), (64, 200), (136, 72)])
def test_grouped_products_of_the_experts(dtype, d, ff):
    """Sort, both grouped products and the combine against the plain mixture, with an expert nobody chooses, one that
    more than a tile of tokens choose, and widths that are no multiple of a tile (in bfloat16 the first pair of sizes
    takes the CUDA-core kernel for the way back, the others the tensor-core kernel both ways)."""
    torch.manual_seed(8)
    act = TORCH[dtype]
    n, E, top = 150, 7, 2
    x = torch.randn(n, d).to(act)
    ids = torch.stack([torch.randperm(E - 1)[:top] for _ in range(n)])          # expert 6 stays idle
    ids[:100, 0] = 3
    ids[:100, 1] = torch.where(ids[:100, 1] == 3, 5, ids[:100, 1])
    wts = torch.rand(n, top)
    gate_w, up_w, down_w = (torch.randn(E, ff, d) * 0.2).to(act), (torch.randn(E, ff, d) * 0.2).to(act), (torch.randn(E, d, ff) * 0.2).to(act)
    shared, sg = torch.randn(n, d).to(act), torch.rand(n)
    want = torch.zeros(n, d, dtype=torch.float64)
    for t in range(n):
        for r in range(top):
            e = int(ids[t, r])
            h = plain.silu(gate_w[e].double() @ x[t].double()) * (up_w[e].double() @ x[t].double())
            if dtype == "bfloat16":
                h = h.to(act).double()
            want[t] += wts[t, r].double() * (down_w[e].double() @ h)
        want[t] += sg[t].double() * shared[t].double()
    gate_up = torch.stack([gate_w, up_w], dim=2).reshape(E, 2 * ff, d).contiguous().to(DEV)
    ids_d = ids.to(torch.int32).to(DEV)
    sorted_pairs = torch.empty(n * top, dtype=torch.int32, device=DEV)
    tiles = torch.empty(k().moe_max_tiles(n * top, E), 4, dtype=torch.int32, device=DEV)
    k().moe_sort(ids_d, E, sorted_pairs, tiles)
    sp = sorted_pairs.cpu().long()
    assert sorted(sp.tolist()) == list(range(n * top))
    experts_in_order = ids.flatten()[sp]
    assert bool((experts_in_order[1:] >= experts_in_order[:-1]).all())
    tl = tiles.cpu()
    assert int(tl[:, 2].sum()) == n * top and int(tl[:, 2].max()) <= k().moe_tile_rows()
    hidden = torch.empty(n * top, ff, device=DEV, dtype=act)
    k().moe_gemm(x.to(DEV), gate_up, hidden, sorted_pairs, tiles, top, gather=True, scatter=False, epi="silu_mul")
    y = torch.full((n * top, d), float("nan"), device=DEV)
    k().moe_gemm(hidden, down_w.to(DEV), y, sorted_pairs, tiles, top, gather=False, scatter=True)
    out = torch.empty(n, d, device=DEV)
    k().moe_combine(y, wts.to(DEV), sg.to(DEV), shared.to(DEV), out)
    assert close(out, want, dtype, atol=5e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_diagonal_product(dtype):
    torch.manual_seed(9)
    act = TORCH[dtype]
    n, blocks, bs = 70, 5, 7
    a = torch.randn(n, blocks * bs).to(act)
    w = torch.randn(blocks, bs, bs).to(act)
    want = torch.einsum("boi,tbi->tbo", w.double(), a.double().view(n, blocks, bs)).reshape(n, blocks * bs)
    out = torch.zeros(n, 2 * blocks * bs, device=DEV)
    k().gemm_simt_batched(a.to(DEV), w.to(DEV), out[:, blocks * bs:])
    assert close(out[:, blocks * bs:], want, "float32") and bool((out[:, :blocks * bs] == 0).all())


# =============================================================== models
def load(folder, dtype, page_size=16, n_pages=64, max_requests=4, **kw):
    from inf_engine_b200 import ModelRunner
    return ModelRunner.from_dir(folder, dtype=dtype, page_size=page_size, n_pages=n_pages, max_requests=max_requests, **kw)


def stepped(r, rid, tokens, sizes, end=True):
    """Logits of every position of ``tokens``, fed in portions of ``sizes`` (repeated as needed)."""
    from inf_engine_b200 import StepEntry
    r.open(rid)
    out, p, i = [], 0, 0
    while p < len(tokens):
        n = min(sizes[i % len(sizes)], len(tokens) - p)
        out.append(r.step([StepEntry(rid, tokens[p:p + n], list(range(n)))]).cpu().clone())
        p += n
        i += 1
    if end:
        r.close(rid)
    return torch.cat(out)


def steady_tokens(cfg, w, n: int, seed: int) -> list[int]:
    """``n`` random tokens whose first ones are well conditioned.  After one token the state of a delta-rule head is
    one outer product and its output (q . k) beta v; when q . k nearly cancels, the head's norm divides by almost
    nothing and the sum's rounding shows in the logits whatever computes them.  Such a start says nothing about the
    product, so the next seed is taken: the plain model in 32-bit must agree with itself in 64-bit on the first rows."""
    for s in range(seed, seed + 50):
        toks = random_tokens(cfg["vocab"], n, s)
        m = min(n, 3)
        a, b = plain.forward_logits(w, cfg, toks[:m]), plain.forward_logits(w, cfg, toks[:m], dtype=torch.float32)
        if float((a - b).abs().max()) <= 2e-6 * max(1.0, float(a.abs().max())):
            return toks
    raise AssertionError("no well-conditioned first tokens in 50 seeds")


LENGTH = {"kpz_a": 97, "kpz_b": 70, "kpz_c": 131, "kpz_d": 75, "kpz_delta": 50, "kpz_att": 60, "kpz_rec": 60, "kpz_moe": 41}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(MODELS))
def test_whole_prompt_decoding_and_portions_agree_with_the_plain_model(tmp_path, name, dtype):
    folder = model_dir(tmp_path, name, dtype)
    cfg, w = plain_inputs(folder)
    toks = steady_tokens(cfg, w, LENGTH[name], 21)
    ref = reference(w, cfg, toks, dtype)
    r = load(folder, dtype, page_size=8)
    T = len(toks)
    assert_close(stepped(r, "whole", toks, [T]), ref, dtype, f"{name}: whole")
    assert_close(stepped(r, "decode", toks, [T - 40] + [1] * 40), ref, dtype, f"{name}: decoded one by one")
    assert_close(stepped(r, "one", toks[:30], [1]), ref[:30], dtype, f"{name}: token by token from the start")
    assert_close(stepped(r, "cut", toks, [7, 2, 16, 3, 2, 17, 2, 31, 1, 5]), ref, dtype, f"{name}: portions")
    assert_close(stepped(r, "pairs", toks[:40], [2]), ref[:40], dtype, f"{name}: portions of two")
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["kpz_a", "kpz_b", "kpz_c", "kpz_d"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(tmp_path, name, dtype):
    """Seven requests, at most three live, portions of some beside decoded tokens of others, some left out of a step;
    the pool holds exactly what the fullest moment needs and free pages are filled with NaN."""
    import random
    from inf_engine_b200 import StepEntry

    folder = model_dir(tmp_path, name, dtype)
    cfg, w = plain_inputs(folder)
    lengths = [45, 17, 80, 3, 33, 64, 1]
    reqs = {f"q{i}": steady_tokens(cfg, w, n, 40 + 100 * i) for i, n in enumerate(lengths)}
    refs = {rid: reference(w, cfg, t, dtype) for rid, t in reqs.items()}
    rng = random.Random(7)
    plan, waiting, live = [], list(reqs), {}
    while waiting or live:
        while waiting and len(live) < 3:
            rid = waiting.pop(0)
            live[rid] = [0, max(1, len(reqs[rid]) - rng.choice([2, 6, 12]))]
        step, ended = [], []
        for rid, st in list(live.items()):
            if rng.random() < 0.25 and len(live) > 1:
                continue
            n = 1 if st[0] >= st[1] else min(rng.choice([2, 3, 5, 11, 24]), st[1] - st[0])
            step.append((rid, st[0], n))
            st[0] += n
            if st[0] == len(reqs[rid]):
                ended.append(rid)
                del live[rid]
        if step:
            plan.append((step, ended))
    ps = 8
    held, most = {}, 0
    for step, ended in plan:
        for rid, p, n in step:
            held[rid] = -(-(p + n) // ps)
        most = max(most, sum(held.values()))
        for rid in ended:
            held.pop(rid)
    r = load(folder, dtype, page_size=ps, n_pages=max(most, 1), max_requests=3, poison_free_pages=True)
    got = {rid: [] for rid in reqs}
    slots_seen = {}
    for step, ended in plan:
        for rid, p, n in step:
            if not r.is_open(rid):
                assert r.open(rid)
                slots_seen[rid] = r.cache.slots[rid]
        lg = r.step([StepEntry(rid, reqs[rid][p:p + n], list(range(n))) for rid, p, n in step]).cpu()
        at = 0
        for rid, p, n in step:
            got[rid].append(lg[at:at + n].clone())
            at += n
        for rid in ended:
            r.close(rid)
        r.cache.check()
    assert len(set(slots_seen.values())) <= 3 < len(slots_seen)              # slots were used again
    for rid in reqs:
        assert_close(torch.cat(got[rid]), refs[rid], dtype, f"{name}: {rid} in mixed batches")


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence_and_a_slot_that_another_request_held(tmp_path, dtype):
    """Sequences of one, two and three tokens in one batch; then new requests in the slots they held: what the old
    requests left there (the inputs of their convolutions, their recurrent states) must not reach the new ones."""
    from inf_engine_b200 import StepEntry

    folder = model_dir(tmp_path, "kpz_a", dtype)
    cfg, w = plain_inputs(folder)
    r = load(folder, dtype, max_requests=3)
    first = {"a": steady_tokens(cfg, w, 1, 1), "b": steady_tokens(cfg, w, 2, 100), "c": steady_tokens(cfg, w, 3, 200)}
    for rid in first:
        r.open(rid)
    lg = r.step([StepEntry(rid, t, list(range(len(t)))) for rid, t in first.items()]).cpu()
    at = 0
    for rid, t in first.items():
        assert_close(lg[at:at + len(t)], reference(w, cfg, t, dtype), dtype, f"first tokens of {rid}")
        at += len(t)
    more = [9, 9, 120]
    for i, tok in enumerate(more):
        lg = r.step([StepEntry("b", [tok], [0])]).cpu()
        assert_close(lg, reference(w, cfg, first["b"] + more[:i + 1], dtype)[-1:], dtype, "second and later tokens")
    for rid in first:
        r.close(rid)
    second = {"d": steady_tokens(cfg, w, 9, 300), "e": steady_tokens(cfg, w, 1, 400), "f": steady_tokens(cfg, w, 2, 500)}
    for rid in second:
        r.open(rid)
    lg = r.step([StepEntry(rid, t, list(range(len(t)))) for rid, t in second.items()]).cpu()
    at = 0
    for rid, t in second.items():
        assert_close(lg[at:at + len(t)], reference(w, cfg, t, dtype), dtype, f"{rid} in a slot used before")
        at += len(t)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["kpz_att", "kpz_c"])
def test_edges_of_the_window_and_of_the_kept_tokens_in_prompts_and_in_decoding(tmp_path, name, dtype):
    """The attention is made sharp (row-norm gains of five) so that one key more or less changes the logits far beyond
    rounding; the sequence runs to three windows, in pages of 8, so that pages behind the window are given back while
    those of the kept tokens stay."""
    def fix(t):
        for n in list(t):
            if n.endswith((".q.norm", ".k.norm")):
                t[n] = (t[n].float() * 2.5).to(t[n].dtype)
    folder = model_dir(tmp_path, name, dtype, fix=fix)
    cfg, w = plain_inputs(folder)
    mask = [L["mixer"]["left"]["mask"] for L in cfg["layers"] if L["type"] == "parallel" and "mask" in L["mixer"]["left"]][0]
    toks = steady_tokens(cfg, w, 3 * mask["size"] + 9, 8)
    ref = reference(w, cfg, toks, dtype)
    # the faults this must catch: a window one key longer, one kept token more, one less
    for key, delta in (("size", 1), ("keep_first", 1), ("keep_first", -1)):
        other = {**cfg, "layers": [dict(L) for L in cfg["layers"]]}
        for L in other["layers"]:
            if L["type"] == "parallel" and "mask" in L["mixer"]["left"]:
                left = {**L["mixer"]["left"], "mask": {**L["mixer"]["left"]["mask"]}}
                left["mask"][key] += delta
                L["mixer"] = {**L["mixer"], "left": left}
        wrong = plain.forward_logits(w, other, toks)
        tail = slice(mask["size"] + mask["keep_first"] + 2, None)
        moved = (wrong - ref.logits).norm(dim=-1).div(ref.logits.norm(dim=-1))[tail]
        # (a key more or less matters where it would take, or takes, much of a sharp row's weight: some rows, not all;
        # such a row moves a thousand times the 32-bit bound)
        assert float(moved.max()) > 0.02, (key, delta, float(moved.max()))
    r = load(folder, dtype, page_size=8)
    noise = 1.5
    assert_close(stepped(r, "whole", toks, [len(toks)]), ref, dtype, f"{name}: window edges in a prompt", noise=noise)
    assert_close(stepped(r, "decode", toks, [3] + [1] * (len(toks) - 3)), ref, dtype, f"{name}: window edges in decoding", noise=noise)
    assert_close(stepped(r, "cut", toks, [mask["size"] - 1, 2, 1, 1, 5, 11]), ref, dtype, f"{name}: portions around the window's edge", noise=noise)
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(tmp_path, dtype):
    """Four tokens of prompt and 200 decoded one by one through the decode graphs: the recurrent states, the inputs of
    the convolutions and the cache are carried over 200 steps."""
    folder = model_dir(tmp_path, "kpz_b", dtype)
    cfg, w = plain_inputs(folder)
    toks = steady_tokens(cfg, w, 204, 77)
    ref = reference(w, cfg, toks, dtype)
    r = load(folder, dtype, page_size=8)
    got = stepped(r, "long", toks, [4] + [1] * 200)
    assert r.graphs.replays >= 150
    assert_close(got, ref, dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["kpz_a", "kpz_c"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype):
    """``Engine.run_offline``: scheduler, portions of prompts under a token budget, decode graphs, device sampling.
    Every generated token must be the plain model's choice (or tie with it within bfloat16's noise)."""
    from inf_engine_b200 import Engine, Request

    folder = model_dir(tmp_path, name, dtype)
    cfg, w = plain_inputs(folder)
    prompts = [steady_tokens(cfg, w, n, 60 + 100 * n) for n in (3, 41, 18, 1, 70)]
    outs = []
    for pipeline in (True, False):
        engine = Engine.from_dir(folder, dtype=dtype, n_total_blocks=24, block_size=8, max_requests=3,
                                 max_tokens_per_step=32, chunk=13, pipeline=pipeline)
        out = engine.run_offline([Request(i, p, max_new_tokens=10) for i, p in enumerate(prompts)])
        engine.runner.cache.check()
        assert engine.runner.cache.n_open == 0 and engine.runner.graphs.replays > 0
        outs.append(out)
        for i, p in enumerate(prompts):
            assert len(out[i]) == 10
            logits = plain.forward_logits(w, cfg, p + out[i])
            for j, tok in enumerate(out[i]):
                row = logits[len(p) + j - 1]
                slack = 0.0 if dtype == "float32" else BF16_NEAR_TIE * NEAR_TIE_NOISE * max(1.0, float(row.abs().max()))
                assert float(row.max() - row[tok]) <= slack, f"{name} {dtype}: request {i}, token {j}"
    if dtype == "float32":
        assert outs[0] == outs[1]


def test_command_line_and_trace_replay(tmp_path):
    folder = make_kipezen_dir(tmp_path, "kpz_b")
    cfg, w = plain_inputs(folder)
    prompt = random_tokens(cfg["vocab"], 12, 5)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate_llama"), "--model-dir", str(folder),
                           "--prompt-ids", ",".join(map(str, prompt)), "--n", "6", "--dtype", "float32"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    ids = [int(t) for t in proc.stdout.strip().splitlines()[-1].split(": ")[1].split(",")]
    logits = plain.forward_logits(w, cfg, prompt + ids)
    assert ids == [int(logits[len(prompt) + j - 1].argmax()) for j in range(6)]
    from test_gpu_replay import schedules
    for dtype in DTYPES:
        folder = model_dir(tmp_path, "kpz_b", dtype)
        cfg, w = plain_inputs(folder)
        requests = {str(i): steady_tokens(cfg, w, n, 300 + 50 * i) for i, n in enumerate([70, 45, 130, 20, 97, 33])}
        trace = schedules("kpz", requests, seed=3)
        got = run_trace(folder, dtype, trace, tmp_path / f"out_{dtype}", cfg["vocab"], page_size=8)
        refs = {rid: reference(w, cfg, t, dtype) for rid, t in requests.items()}
        for prefix in "wdpm":
            for rid, t in requests.items():
                rows = [got.get((prefix + rid, p)) for p in range(len(t))]
                if rows[0] is None:
                    continue
                assert_close(torch.stack(rows), refs[rid], dtype, f"replay {prefix}{rid}")
