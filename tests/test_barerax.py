"""Host-side tests of the Barerax family: configuration, tensor table, the distance buckets, the cache manager's
groups for it, the scheduler over a model without pages, and the plain implementation's own consistency."""

import copy
import json

import pytest
import torch

import plain_barerax as plain
from barerax_models import BRX_A, BRX_B, BRX_C, MODELS, make_barerax_dir, stated_config


def test_config_reads_every_size_and_constant():
    from inf_engine_b200.config import BareraxConfig, parse_config_dict

    cfg = parse_config_dict(BRX_A)
    assert isinstance(cfg, BareraxConfig)
    assert (cfg.vocab, cfg.width, cfg.norm_eps) == (301, 64, 1e-5)
    assert (cfg.bigram_buckets, cfg.bigram_mul_prev, cfg.bigram_mul_cur) == (211, 31, 5)
    assert [L.type for L in cfg.layers] == ["attention", "general_delta", "general_delta", "attention"]
    a = cfg.layers[0]
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.bias_max, a.rel_buckets, a.ff) == (4, 2, 16, 24, 0.3, 40, 12, 96)
    assert cfg.layers[2].ff is None and cfg.layers[1].decay_rank == 8
    assert parse_config_dict(cfg.to_hf_dict()) == cfg
    spec = cfg.model_spec()
    assert spec.kind == "bigram_decoder" and spec.head is None and spec.vocab_size == 301
    assert spec.layers[2].feedforward is None and spec.layers[2].ff_norm is None
    m = spec.layers[0].mixer
    assert m.value_dim == 24 and m.scale == 0.3 and m.position.kind == "bucketed_bias" and m.position.max_distance == 40
    assert spec.layers[1].mixer.decay_rate == pytest.approx(0.6065306597126334)


@pytest.mark.parametrize("damage, word", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d["embedding"]["bigram"].pop("mul_cur"), "mul_cur"),
    (lambda d: d["layers"][0].__setitem__("type", "conv"), "conv"),
    (lambda d: d["layers"][0]["mlp"].__setitem__("kind", "routed"), "routed"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("bias_max", 6), "bias_max"),
    (lambda d: d["layers"][1]["mixer"].pop("dim"), "dim"),
    (lambda d: d.__setitem__("layers", []), "layers"),
])
def test_config_errors_name_what_is_wrong(damage, word):
    from inf_engine_b200.config import ConfigError, parse_config_dict

    d = copy.deepcopy(BRX_A)
    damage(d)
    with pytest.raises(ConfigError, match=word):
        parse_config_dict(d)


def test_unknown_architecture_lists_the_known_ones():
    from inf_engine_b200.config import ConfigError, parse_config_dict

    with pytest.raises(ConfigError, match="Barerax"):
        parse_config_dict({"architecture": "Nothing"})


def test_sizes_that_the_file_leaves_out_come_from_tensor_shapes(tmp_path):
    from inf_engine_b200.config import detect_config, parse_config_dict
    from inf_engine_b200.parts import expected_tensors
    from inf_engine_b200.weights import check_names_and_shapes, open_checkpoint

    for name in ("brx_a", "brx_b"):
        folder = make_barerax_dir(tmp_path, name)
        stated = json.loads((folder / "config.json").read_text())
        assert all("rel_buckets" not in L["mixer"] and "decay_rank" not in L["mixer"] for L in stated["layers"])
        cfg = detect_config(folder)
        assert cfg == parse_config_dict(MODELS[name])
        found = {n: t.shape for n, t in open_checkpoint(folder).items()}
        check_names_and_shapes(found, expected_tensors(cfg.model_spec()))


def test_tensor_table():
    from inf_engine_b200.config import parse_config_dict
    from inf_engine_b200.parts import expected_tensors

    exp = expected_tensors(parse_config_dict(BRX_B).model_spec())
    shapes = {n: tuple(e.shape) for n, e in exp.items()}
    assert list(shapes)[:2] == ["embed", "bigram"] and shapes["bigram"] == (98, 96)
    assert shapes["l0.mix.w1"] == (12, 96) and shapes["l0.mix.w2"] == (96, 12) and shapes["l0.mix.a.b"] == (96,)
    assert shapes["l1.mix.q"] == (72, 96) and shapes["l1.mix.k"] == (24, 96) and shapes["l1.mix.v"] == (40, 96)
    assert shapes["l1.mix.o"] == (96, 120) and shapes["l1.mix.rel"] == (9, 3) and shapes["l1.mix.temp"] == (3,)
    assert shapes["l1.mix.q.norm"] == (24,) and "l1.norm2" not in shapes and "l1.mlp.up" not in shapes
    assert shapes["l2.mlp.act"] == (4,) and shapes["l2.mlp.up.b"] == (64,) and shapes["final.norm.b"] == (96,)


@pytest.mark.parametrize("rows, far", [(12, 40), (9, 30), (16, 64), (20, 100), (32, 256), (2, 5), (7, 1000)])
def test_distance_buckets(rows, far):
    from inf_engine_b200.parts import distance_bucket

    got = [distance_bucket(n, rows, far) for n in range(far + 50)]
    assert got == [plain.distance_row(n, rows, far) for n in range(far + 50)]
    half = rows // 2
    assert got[:half] == list(range(half))                         # one row per distance at first
    assert all(a <= b for a, b in zip(got, got[1:]))               # never back to an earlier row
    assert all(g == rows - 1 for g in got[far:]) and max(got) == rows - 1
    if far > half + 1:
        assert got[half] == half                                   # the logarithmic part starts in its own first row
    # the edge of every row, from exact integer arithmetic: row half + k starts where (n / half)^(rows - half) >= (far / half)^k
    m = rows - half
    for n in range(max(half, 1), far + 1):
        k = max(j for j in range(m + 1) if n ** m * half ** j >= far ** j * half ** m)
        assert got[n] == min(rows - 1, half + k), n


def test_plain_pieces_are_consistent():
    torch.manual_seed(0)
    T, D = 23, 8
    r, k, v = (torch.randn(T, D, dtype=torch.float64) for _ in range(3))
    decay = torch.rand(T, D, dtype=torch.float64) * 0.4 + 0.6
    rate = torch.rand(T, D, dtype=torch.float64)
    whole, S = plain.delta_rule_states(r, k, v, decay, rate)
    first, S1 = plain.delta_rule_states(r[:9], k[:9], v[:9], decay[:9], rate[:9])
    rest, S2 = plain.delta_rule_states(r[9:], k[9:], v[9:], decay[9:], rate[9:], state=S1)
    assert torch.allclose(torch.cat([first, rest]), whole, atol=1e-12) and torch.allclose(S2, S, atol=1e-12)
    # a rate of one and no decay: the old content along the key's direction is gone, the new pair is stored
    u = k[0] / k[0].norm()
    _, S = plain.delta_rule_states(r[:1], k[:1], v[:1], torch.ones(1, D, dtype=torch.float64), torch.ones(1, D, dtype=torch.float64),
                                   state=torch.randn(D, D, dtype=torch.float64))
    assert torch.allclose(u @ S, (u @ k[0]) * v[0], atol=1e-5)
    assert plain.bigram_rows([4, 9, 9], 7, 3, 5) == [7, (4 * 3 + 9 * 5) % 7, (9 * 3 + 9 * 5) % 7]
    z = torch.randn(3, 40, dtype=torch.float64)
    assert torch.allclose(plain.polynorm(z, torch.tensor([0.0, 0.0, 0.0, 2.5]), 1e-6), torch.full_like(z, 2.5))
    assert torch.allclose(plain.polynorm(z, torch.tensor([1.0, 0.0, 0.0, 0.0]), 0.0).pow(2).mean(-1), torch.ones(3, dtype=torch.float64))


def test_plain_model_is_causal(tmp_path):
    from helpers import plain_inputs, random_tokens

    cfg, w = plain_inputs(make_barerax_dir(tmp_path, "brx_a"))
    a = random_tokens(cfg["vocab"], 30, 1)
    b = a[:20] + random_tokens(cfg["vocab"], 10, 2)
    la, lb = plain.forward_logits(w, cfg, a), plain.forward_logits(w, cfg, b)
    assert torch.allclose(la[:20], lb[:20], atol=1e-6) and not torch.allclose(la[20:], lb[20:], atol=1e-3)


def test_cache_groups_of_the_family():
    from inf_engine_b200.cache import CacheManager, CacheRequirement

    kv = lambda d, dv: CacheRequirement(kind="kv", n_kv_heads=2, head_dim=d, dtype=torch.float32, v_head_dim=dv)
    state = CacheRequirement(kind="state", state_shape=(2, 8, 8), state_dtype=torch.float32)
    last = CacheRequirement(kind="state", state_shape=(1,), state_dtype=torch.int32)
    m = CacheManager([kv(16, 24), state, kv(16, None), kv(16, 24), state, last], page_size=4, n_pages=6, max_requests=2)
    assert len(m.kv_groups) == 2 and len(m.state_groups) == 2          # values of 24 and of 16 do not share pages
    assert m.bindings[0].group == m.bindings[3].group != m.bindings[2].group
    m.allocate_storage("cpu")
    g = m.kv_groups[0]
    assert g.k.shape == (2, 6, 2, 4, 16) and g.v.shape == (2, 6, 2, 4, 24)
    assert m.storage_bytes() == 4 * (2 * 6 * 2 * 4 * (16 + 24) + 6 * 2 * 4 * 32) + 2 * 2 * 128 * 4 + 2 * 4
    a = m.open("a")
    m.state_groups[0].data[:, a] = 3.0
    m.state_groups[1].data[:, a] = 77
    assert m.reserve("a", 9) and m.kv_groups[0].pool.n_free == m.kv_groups[1].pool.n_free == 3
    m.advance("a", 9)
    m.close("a")
    assert m.open("b") == a                                             # the slot is used again, and it is clean
    assert float(m.state_groups[0].data[:, a].abs().max()) == 0.0 and int(m.state_groups[1].data[:, a].abs().max()) == 0
    m.check()


def test_scheduler_over_a_model_without_pages():
    """A model of recurrent layers only has state slots and no page pool; admission is bounded by slots."""
    from inf_engine_b200 import Request, Scheduler
    from inf_engine_b200.cache import CacheManager, CacheRequirement

    state = CacheRequirement(kind="state", state_shape=(4,), state_dtype=torch.float32)
    m = CacheManager([state, state], page_size=16, n_pages=4, max_requests=2)
    s = Scheduler(m, max_positions=1 << 30, max_batch=8, max_tokens_per_step=16, chunk=7)
    reqs = [Request(i, list(range(1, 12 + i)), max_new_tokens=2) for i in range(3)]
    assert all(s.submit(r) for r in reqs)
    steps = 0
    while s.has_work and steps < 50:
        plan = s.plan()
        assert plan.entries and len(s.running) <= 2 and plan.n_tokens <= 16
        for e in plan.entries:
            m.advance(e.request.req_id, m.lengths[e.request.req_id] + len(e.tokens))
        s.commit(plan, {e.request.req_id: 5 for e in plan.entries if e.wants_logits})
        steps += 1
    assert not s.has_work and sorted(r.req_id for r in s.completed) == [0, 1, 2]
    assert all(r.generated == [5, 5] for r in reqs) and m.n_open == 0
    m.check()
