"""The Barerax family on the GPU against the plain implementation: each new kernel alone, each mechanism alone in a
one-layer model, whole prompts against token-by-token decoding and portions down to two tokens, batches of unequal
requests with pages and state slots used again, the first tokens of a sequence, the edges of the distance table in
prompts and in decoding, a far key that must stand out, long decoding, greedy generation through the engine and
its scheduler, the command line and the trace replay.  Every test runs in 32-bit and in bfloat16."""

import os
import subprocess
import sys

import pytest
import torch

import plain_barerax as plain
from barerax_models import MODELS, make_barerax_dir
import helpers
from helpers import BF16_NEAR_TIE, plain_inputs, random_tokens, run_trace

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# bfloat16 rows of this family carry more rounding than the Llama rows that the shared bounds were measured on: each
# head of the delta rule is divided by its own root mean square, which for the first tokens of a sequence (a state
# made of one or two outer products) is small, and the PolyNorm divides cubes by theirs.  Measured worst row 0.023
# (widths up to 128); the 32-bit comparisons keep the shared bound and are the sharp ones.
BF16_NOISE = 1.5


def assert_close(got, ref, dtype, what=""):
    helpers.assert_close(got, ref, dtype, what, noise=BF16_NOISE)


def k():
    from inf_engine_b200 import kernels
    return kernels


def dev_i32(x):
    return torch.as_tensor(x, dtype=torch.int32).to(DEV)


def close(got, want, dtype, rel=2e-2):
    """float32: element by element against the float64 oracle; bfloat16: against the largest value of the tensor."""
    got, want = got.double().cpu(), want.double().cpu()
    if dtype == "float32":
        return torch.allclose(got, want, atol=2e-5, rtol=2e-5)
    return float((got - want).abs().max()) <= rel * max(1.0, float(want.abs().max()))


# =============================================================== kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_layernorm_kernel(dtype):
    torch.manual_seed(1)
    act = TORCH[dtype]
    n, d = 7, 200
    res = (torch.randn(n, d) * 2 + 30.0)                       # a mean far from zero: the variance must not cancel
    delta = torch.randn(n, d).to(act)
    w, b = (1 + 0.3 * torch.randn(d)).to(act), torch.randn(d).to(act)
    want = plain.layer_norm(res.double() + delta.double(), w.double(), b.double(), 1e-5)
    r = res.to(DEV)
    out = torch.empty(n, d, device=DEV, dtype=act)
    k().layernorm(r, delta.to(DEV), w.to(DEV), b.to(DEV), out, 1e-5)
    assert close(out, want, dtype) and torch.allclose(r.cpu(), res + delta.float(), atol=1e-6)     # the sum is kept
    rows = dev_i32([5, 0, 5])
    out3 = torch.empty(3, d, device=DEV, dtype=act)
    k().layernorm(r, None, w.to(DEV), b.to(DEV), out3, 1e-5, row_index=rows)
    assert close(out3, want[[5, 0, 5]], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_polynorm_kernel(dtype):
    torch.manual_seed(2)
    act = TORCH[dtype]
    n, f = 5, 136
    z = (torch.randn(n, f) * 1.7).to(act)
    bias = torch.randn(f).to(act)
    coef = torch.tensor([0.9, -0.4, 0.25, 0.1]).to(act)
    want = plain.polynorm(z.double() + bias.double(), coef.double(), 1e-6)
    wide = torch.zeros(n, f + 24, device=DEV, dtype=act)       # a row-strided input
    wide[:, :f] = z.to(DEV)
    out = torch.empty(n, f, device=DEV, dtype=act)
    k().polynorm(wide[:, :f], bias.to(DEV), coef.to(DEV), out, 1e-6)
    assert close(out, want, dtype)
    k().polynorm(wide[:, :f], None, coef.to(DEV), out, 1e-6)
    assert close(out, plain.polynorm(z.double(), coef.double(), 1e-6), dtype)


@pytest.mark.parametrize("dtype, d", [("float32", 24), ("bfloat16", 24), ("bfloat16", 20)])
def test_bigram_embedding_kernel_keeps_the_last_token_of_every_request(dtype, d):
    torch.manual_seed(3)
    vocab, buckets, mp, mc = 50, 13, 1000003, 7
    table, bigram = torch.randn(vocab, d).to(TORCH[dtype]), torch.randn(buckets + 1, d).to(TORCH[dtype])
    # request 0 starts (3 tokens), request 1 goes on from position 9 after token 41 (1 token), request 2 is padding
    ids = [4, 4, 17, 30, 0]
    state = dev_i32([0, 41, 99, 0])
    res = torch.empty(5, d, device=DEV)
    k().embed_bigram(dev_i32(ids), dev_i32([0, 1, 2, 9, 0]), dev_i32([0, 3, 4, 5]), dev_i32([2, 1, -1]), 3,
                     table.to(DEV), bigram.to(DEV), state, res, buckets, mp, mc)
    rows = [buckets, (4 * mp + 4 * mc) % buckets, (4 * mp + 17 * mc) % buckets, (41 * mp + 30 * mc) % buckets, buckets]
    want = table[ids].float() + bigram[rows].float()
    assert torch.equal(res.cpu(), want)
    assert state.tolist() == [0, 30, 17, 0]
    # the next step of request 0 takes its previous token from the slot
    k().embed_bigram(dev_i32([9, 2]), dev_i32([3, 4]), dev_i32([0, 2]), dev_i32([2]), 1, table.to(DEV), bigram.to(DEV),
                     state, res[:2], buckets, mp, mc)
    assert torch.equal(res[:2].cpu(), table[[9, 2]].float() + bigram[[(17 * mp + 9 * mc) % buckets, (9 * mp + 2 * mc) % buckets]].float())
    assert state.tolist() == [0, 30, 2, 0]
    # a negative multiplier: the remainder is the mathematical one, never negative
    k().embed_bigram(dev_i32([9, 2]), dev_i32([3, 4]), dev_i32([0, 2]), dev_i32([2]), 1, table.to(DEV), bigram.to(DEV),
                     state, res[:2], buckets, -5, 3)
    assert torch.equal(res[:2].cpu(), table[[9, 2]].float() + bigram[[(2 * -5 + 9 * 3) % buckets, (9 * -5 + 2 * 3) % buckets]].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim, heads", [(16, 3), (48, 2), (128, 1)])
def test_delta_rule_kernel(dtype, dim, heads):
    """Three requests of 1, 19 and 40 tokens and a padding row; the first goes on from a state that is not zero."""
    torch.manual_seed(dim)
    act = TORCH[dtype]
    W = heads * dim
    q_lens = [1, 19, 40, 1]
    n = sum(q_lens)
    q_start = [0, 1, 20, 60, 61]
    slots = [3, 0, 2, -1]
    proj = (torch.randn(n, 5 * W + 8) * 1.2).to(act)                       # r k v g a_pre, and 8 columns that are not ours
    w_pre = torch.randn(n, W) * 1.5
    a_bias, w_bias, gain = (torch.randn(W).to(act), torch.randn(W).to(act), (1 + 0.2 * torch.randn(W)).to(act))
    state0 = torch.zeros(4, heads, dim, dim)
    state0[3] = torch.randn(heads, dim, dim) * 0.3
    state0[1] = 7.0                                                          # nobody's slot: must stay as it is
    r, kk, v, g, a_pre = (proj[:, i * W:(i + 1) * W].double() for i in range(5))
    decay = torch.exp(-0.6 * plain.sig(w_pre.double() + w_bias.double()))
    rate = plain.sig(a_pre + a_bias.double())
    want = torch.zeros(n, W, dtype=torch.float64)
    want_state = state0.double().clone()
    for i in range(3):
        a, b = q_start[i], q_start[i + 1]
        for h in range(heads):
            c = slice(h * dim, (h + 1) * dim)
            o, S = plain.delta_rule_states(r[a:b, c], kk[a:b, c], v[a:b, c], decay[a:b, c], rate[a:b, c], 1e-6,
                                           want_state[slots[i], h])
            want[a:b, c] = plain.unit_rms(o, 1e-5) * gain.double()[c] * plain.sig(g[a:b, c])
            want_state[slots[i], h] = S
    p = proj.to(DEV)
    state = state0.to(DEV)
    out = torch.full((n, W), 5.0, device=DEV, dtype=act)
    views = [p[:, i * W:(i + 1) * W] for i in range(5)]
    k().delta_rule(views[0], views[1], views[2], views[4], views[3], w_pre.to(DEV), a_bias.to(DEV), w_bias.to(DEV),
                   gain.to(DEV), state, out, dev_i32(q_start), dev_i32(slots), 4, heads, dim, 0.6, 1e-6, 1e-5)
    assert close(out[:60], want[:60], dtype, rel=1e-2) and float(out[60:].abs().max()) == 0.0
    assert torch.allclose(state.cpu().double(), want_state, atol=1e-4, rtol=1e-4)
    # a run that may not write leaves the state alone
    before = state.clone()
    k().delta_rule(views[0], views[1], views[2], views[4], views[3], w_pre.to(DEV), a_bias.to(DEV), w_bias.to(DEV),
                   gain.to(DEV), state, out, dev_i32(q_start), dev_i32(slots), 4, heads, dim, 0.6, 1e-6, 1e-5,
                   write_state=False)
    assert torch.equal(state, before)


@pytest.mark.parametrize("dtype, tensor_cores", [("float32", 0), ("bfloat16", 0), ("bfloat16", 64), ("bfloat16", 128)])
@pytest.mark.parametrize("decode", [False, True])
def test_a_far_key_stands_out_at_every_edge_of_the_distance_table(dtype, tensor_cores, decode):
    """One key carries the direction that a query asks for, scaled so that its score beats all others by far; the
    value that comes back must be that key's.  The key is placed at every distance around the edges of the table's
    rows and around its far end, on both sides of page borders, and the table holds a different large value in every
    row for every head, so that a distance that falls into the neighbouring row moves the weights visibly.
    ``tensor_cores``: the bias build of the mma.sync kernels (heads of that size) instead of the general kernel."""
    from inf_engine_b200.parts import distance_bucket

    torch.manual_seed(5)
    act = TORCH[dtype]
    H, G, hd, hdv, ps, rows, far = (4, 2, tensor_cores, tensor_cores, 16, 10, 37) if tensor_cores else (4, 2, 16, 24, 8, 10, 37)
    T = 150 if tensor_cores else 90
    table = torch.tensor([[(-1.0) ** (r + h) * (1.0 + 0.7 * r) for h in range(H)] for r in range(rows)])
    bias = table[[distance_bucket(n, rows, far) for n in range(far + 1)]].t().contiguous()      # [H, far + 1]
    temp = torch.tensor([0.7, 1.0, 1.6, 1.2])
    scale = 0.2
    edges = sorted({d for r in range(rows) for d in range(far + 3) if distance_bucket(d, rows, far) == r
                    and (d == 0 or distance_bucket(d - 1, rows, far) != r or distance_bucket(d + 1, rows, far) != r)}
                   | {far - 1, far, far + 1, far + 20, 7, 8, 9, 15, 16, 17})
    for dist in edges:
        q = torch.randn(T, H * hd) * 0.3
        kx = torch.randn(T, G * hd) * 0.3
        v = torch.randn(T, G * hdv)
        target = T - 1 - dist
        direction = torch.zeros(hd)
        direction[3] = 1.0
        kx.view(T, G, hd)[target] += 12.0 * direction
        q.view(T, H, hd)[T - 1] += 12.0 * direction
        q, kx, v = q.to(act), kx.to(act), v.to(act)
        # plain: scores of the last query over all keys, float64
        qq, kk, vv = q.double().view(T, H, hd), kx.double().view(T, G, hd), v.double().view(T, G, hdv)
        want = torch.zeros(H, hdv, dtype=torch.float64)
        for h in range(H):
            s = (kk[:, h // 2] @ qq[T - 1, h]) * scale * temp[h].double()
            s = s + table[[distance_bucket(T - 1 - j, rows, far) for j in range(T)], h].double()
            want[h] = torch.softmax(s, 0) @ vv[:, h // 2]
        # product: keys and values into pages (in an order that is not the pages' own), then the kernel
        n_pages = -(-T // ps)
        order = list(reversed(range(n_pages)))
        kpool = torch.full((n_pages, G, ps, hd), float("nan"), device=DEV, dtype=act)
        vpool = torch.full((n_pages, G, ps, hdv), float("nan"), device=DEV, dtype=act)
        slot_map = dev_i32([order[p // ps] * ps + p % ps for p in range(T)])
        qd = q.to(DEV).clone()
        k().headnorm_kv_write(qd, kx.to(DEV), v.to(DEV), None, None, 0.0, slot_map, kpool, vpool, H, G, hd, hdv, ps)
        out = torch.empty(T, H * hdv, device=DEV, dtype=act)
        table_dev = dev_i32([order]).view(1, n_pages)
        if tensor_cores and decode:
            from inf_engine_b200.parts.attention import decode_splits
            n_splits, split_keys = decode_splits(T, G, *k().attention_decode_geometry(hd))
            scratch = torch.zeros(k().attention_decode_scratch_floats(1, H, n_splits, hd), device=DEV)
            k().attention_decode_mma(qd[T - 1:], out[T - 1:], kpool, vpool, table_dev, dev_i32([0, 1]), dev_i32([T - 1]),
                                     scratch, 1, 1, H, G, hd, ps, None, scale, n_splits, split_keys,
                                     score_bias_log2e=(bias * k().LOG2E).to(DEV), head_scale=temp.to(DEV))
        elif tensor_cores:
            n_tiles = -(-T * (H // G) // 64)
            k().attention_prefill_mma(qd, out, kpool, vpool, table_dev, dev_i32([0, T]), dev_i32([0]), dev_i32([0] * n_tiles),
                                      dev_i32([64 * i for i in range(n_tiles)]), n_tiles, H, G, hd, ps, None, scale, 64,
                                      score_bias_log2e=(bias * k().LOG2E).to(DEV), head_scale=temp.to(DEV))
        elif decode:      # the last token alone against the cache
            k().attention_general(qd[T - 1:], out[T - 1:], kpool, vpool, table_dev, dev_i32([0, 1]), dev_i32([T - 1]),
                                  dev_i32([0]), dev_i32([0]), 1, H, G, hd, ps, None, scale, bias.to(DEV), temp.to(DEV), hdv)
        else:
            n_tiles = -(-T * (H // G) // 32)
            k().attention_general(qd, out, kpool, vpool, table_dev, dev_i32([0, T]), dev_i32([0]), dev_i32([0] * n_tiles),
                                  dev_i32([32 * i for i in range(n_tiles)]), n_tiles, H, G, hd, ps, None, scale,
                                  bias.to(DEV), temp.to(DEV), hdv)
        got = out[T - 1].view(H, hdv)
        assert close(got, want, dtype), f"distance {dist}"
        # and the key did stand out for the head whose row of the table does not push it down
        best = max(range(H), key=lambda h: float(table[distance_bucket(dist, rows, far), h]))
        assert float((want[best] - vv[target, best // 2]).abs().max()) < 0.35, dist


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
    """``n`` random tokens whose first one is well conditioned.  After a single token the state of a delta-rule head
    is one outer product and its output (r . k) v; when r . k nearly cancels, the head's norm divides by almost
    nothing and the sum's rounding shows in the logits whatever computes them.  Such a first token (about one in a
    hundred) says nothing about the product, so the next seed is taken: the plain model in 32-bit must agree with
    itself in 64-bit on the first row."""
    for s in range(seed, seed + 50):
        toks = random_tokens(cfg["vocab"], n, s)
        a, b = plain.forward_logits(w, cfg, toks[:1]), plain.forward_logits(w, cfg, toks[:1], dtype=torch.float32)
        if float((a - b).abs().max()) <= 2e-6 * max(1.0, float(a.abs().max())):
            return toks
    raise AssertionError("no well-conditioned first token in 50 seeds")


LENGTH = {"brx_a": 97, "brx_b": 70, "brx_c": 131, "brx_d": 75, "brx_att": 60, "brx_delta": 50, "brx_ff": 41}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(MODELS))
def test_whole_prompt_decoding_and_portions_agree_with_the_plain_model(tmp_path, name, dtype):
    folder = make_barerax_dir(tmp_path, name)
    cfg, w = plain_inputs(folder)
    toks = steady_tokens(cfg, w, LENGTH[name], 21)
    ref = plain.forward_logits(w, cfg, toks)
    r = load(folder, dtype)
    T = len(toks)
    assert_close(stepped(r, "whole", toks, [T]), ref, dtype, f"{name}: whole")
    assert_close(stepped(r, "decode", toks, [T - 24] + [1] * 24), ref, dtype, f"{name}: decoded one by one")
    assert_close(stepped(r, "one", toks[:30], [1]), ref[:30], dtype, f"{name}: token by token from the start")
    assert_close(stepped(r, "cut", toks, [7, 2, 16, 3, 2, 17, 2, 31, 1, 5]), ref, dtype, f"{name}: portions")
    assert_close(stepped(r, "pairs", toks[:40], [2]), ref[:40], dtype, f"{name}: portions of two")
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["brx_a", "brx_b", "brx_c", "brx_d"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(tmp_path, name, dtype):
    """Seven requests, at most three live, portions of some beside decoded tokens of others, some left out of a step;
    the pool holds exactly what the fullest moment needs and free pages are filled with NaN."""
    import random
    from inf_engine_b200 import StepEntry

    folder = make_barerax_dir(tmp_path, name)
    cfg, w = plain_inputs(folder)
    lengths = [45, 17, 80, 3, 33, 64, 1]
    reqs = {f"q{i}": steady_tokens(cfg, w, n, 40 + 100 * i) for i, n in enumerate(lengths)}
    refs = {rid: plain.forward_logits(w, cfg, t) for rid, t in reqs.items()}
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
    requests left there (their last token, their recurrent state) must not reach the new ones.  The bigram table is
    made large so that a wrong row shows."""
    from inf_engine_b200 import StepEntry

    def fix(t):
        t["bigram"] = (t["bigram"].float() * 6).to(t["bigram"].dtype)
    folder = make_barerax_dir(tmp_path, "brx_a", fix=fix)
    cfg, w = plain_inputs(folder)
    r = load(folder, dtype, max_requests=3)
    first = {"a": steady_tokens(cfg, w, 1, 1), "b": steady_tokens(cfg, w, 1, 100) * 2, "c": steady_tokens(cfg, w, 1, 200) + [3, 3]}
    for rid in first:
        r.open(rid)
    lg = r.step([StepEntry(rid, t, list(range(len(t)))) for rid, t in first.items()]).cpu()
    at = 0
    for rid, t in first.items():
        assert_close(lg[at:at + len(t)], plain.forward_logits(w, cfg, t), dtype, f"first tokens of {rid}")
        at += len(t)
    # go on with one of them, one token at a time
    more = [9, 9, 120]
    for i, tok in enumerate(more):
        lg = r.step([StepEntry("b", [tok], [0])]).cpu()
        assert_close(lg, plain.forward_logits(w, cfg, first["b"] + more[:i + 1])[-1:], dtype, "second and later tokens")
    for rid in first:
        r.close(rid)
    second = {"d": steady_tokens(cfg, w, 9, 300), "e": steady_tokens(cfg, w, 1, 400), "f": steady_tokens(cfg, w, 2, 500)}
    for rid in second:
        r.open(rid)
    lg = r.step([StepEntry(rid, t, list(range(len(t)))) for rid, t in second.items()]).cpu()
    at = 0
    for rid, t in second.items():
        assert_close(lg[at:at + len(t)], plain.forward_logits(w, cfg, t), dtype, f"{rid} in a slot used before")
        at += len(t)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["brx_att", "brx_a"])
def test_edges_of_the_distance_table_in_prompts_and_in_decoding(tmp_path, name, dtype):
    """The distance table holds large values that differ from row to row, so that a key counted into the row beside
    its own changes the logits far beyond rounding; sequences reach well past the table's far end."""
    def fix(t):
        for n in list(t):
            if n.endswith(".mix.rel"):
                rows, heads = t[n].shape
                t[n] = torch.tensor([[(-1.0) ** (r + h) * (0.5 + 0.6 * r) for h in range(heads)] for r in range(rows)]).to(t[n].dtype)
    folder = make_barerax_dir(tmp_path, name, fix=fix)
    cfg, w = plain_inputs(folder)
    far = max(L["mixer"]["bias_max"] for L in cfg["layers"] if L["type"] == "attention")
    toks = steady_tokens(cfg, w, far + 40, 8)
    ref = plain.forward_logits(w, cfg, toks)
    # the fault this must catch: the same model with every distance one row too late
    shifted = dict(w)
    for n in w:
        if n.endswith(".mix.rel"):
            shifted[n] = torch.cat([w[n][:1], w[n][:-1]])
    wrong = plain.forward_logits(shifted, cfg, toks)
    assert float((wrong - ref).norm(dim=-1).div(ref.norm(dim=-1))[1:].min()) > 0.05          # (a single key has all the weight)
    r = load(folder, dtype, page_size=8)
    assert_close(stepped(r, "whole", toks, [len(toks)]), ref, dtype, f"{name}: table edges in a prompt")
    assert_close(stepped(r, "decode", toks, [3] + [1] * (len(toks) - 3)), ref, dtype, f"{name}: table edges in decoding")
    assert_close(stepped(r, "cut", toks, [far - 1, 2, 1, 1, 5]), ref, dtype, f"{name}: portions around the far end")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(tmp_path, dtype):
    """Four tokens of prompt and 200 decoded one by one through the decode graphs: the recurrent state and the cache
    are carried over 200 steps."""
    folder = make_barerax_dir(tmp_path, "brx_b")
    cfg, w = plain_inputs(folder)
    toks = steady_tokens(cfg, w, 204, 77)
    ref = plain.forward_logits(w, cfg, toks)
    r = load(folder, dtype, page_size=8)
    got = stepped(r, "long", toks, [4] + [1] * 200)
    assert r.graphs.replays >= 150
    assert_close(got, ref, dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["brx_a", "brx_c"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype):
    """``Engine.run_offline``: scheduler, portions of prompts under a token budget, decode graphs, device sampling.
    Every generated token must be the plain model's choice (or tie with it within bfloat16's noise)."""
    from inf_engine_b200 import Engine, Request

    folder = make_barerax_dir(tmp_path, name)
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
                slack = 0.0 if dtype == "float32" else BF16_NEAR_TIE * max(1.0, float(row.abs().max()))
                assert float(row.max() - row[tok]) <= slack, f"{name} {dtype}: request {i}, token {j}"
    if dtype == "float32":
        assert outs[0] == outs[1]


def test_command_line_and_trace_replay(tmp_path):
    folder = make_barerax_dir(tmp_path, "brx_b")
    cfg, w = plain_inputs(folder)
    prompt = random_tokens(cfg["vocab"], 12, 5)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate_llama"), "--model-dir", str(folder),
                           "--prompt-ids", ",".join(map(str, prompt)), "--n", "6", "--dtype", "float32"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    ids = [int(t) for t in proc.stdout.strip().splitlines()[-1].split(": ")[1].split(",")]
    logits = plain.forward_logits(w, cfg, prompt + ids)
    assert ids == [int(logits[len(prompt) + j - 1].argmax()) for j in range(6)]
    # the replay program: four live requests at most, a pool of what the trace holds at its fullest
    from test_gpu_replay import schedules
    requests = {str(i): random_tokens(cfg["vocab"], n, 300 + i) for i, n in enumerate([70, 45, 130, 20, 97, 33])}
    trace = schedules("brx", requests, seed=3)
    for dtype in DTYPES:
        got = run_trace(folder, dtype, trace, tmp_path / f"out_{dtype}", cfg["vocab"], page_size=8)
        refs = {rid: plain.forward_logits(w, cfg, t) for rid, t in requests.items()}
        for prefix in "wdpm":
            for rid, t in requests.items():
                rows = [got.get((prefix + rid, p)) for p in range(len(t))]
                if rows[0] is None:
                    continue
                assert_close(torch.stack(rows), refs[rid], dtype, f"replay {prefix}{rid}")
