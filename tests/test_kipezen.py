"""The Kipezen family without a GPU: configuration and its errors, the tensor table, the cache groups that its mixers
ask for (several caches a layer, kept first keys beside a window), and the plain implementation's own consistency."""

import copy
import json

import pytest
import torch

import plain_kipezen as plain
from kipezen_models import MODELS, make_kipezen_dir
from helpers import plain_inputs, random_tokens


def parse(d):
    from inf_engine_b200.config import parse_config_dict
    return parse_config_dict(d)


def test_configuration_round_trip_and_specs():
    from inf_engine_b200.config import KipezenConfig
    for name, d in MODELS.items():
        cfg = parse(d)
        assert isinstance(cfg, KipezenConfig) and cfg.vocab_size == d["vocab"] and cfg.num_hidden_layers == len(d["layers"])
        assert parse(cfg.to_hf_dict()) == cfg, name
        spec = cfg.model_spec()
        assert spec.head is None and spec.final_norm.unit_offset and len(spec.schedule) == len(d["layers"])
        for blk, L in zip(spec.layers, d["layers"]):
            assert blk.kind == "outnorm" and (blk.feedforward is None) == (L["mlp"] is None)
            if L["type"] == "parallel":
                att, rec = blk.mixer.branches
                left = L["mixer"]["left"]
                assert att.out_scale == L["mixer"]["left_scale"] and rec.out_scale == L["mixer"]["right_scale"]
                assert att.window == (left["mask"]["size"] if "mask" in left else None)
                assert att.keep_first == (left["mask"]["keep_first"] if "mask" in left else 0)
                assert att.position.kind == ("rotary_pairs" if "rot" in left else "none")
            else:
                assert blk.mixer.kind == "gated_delta" and blk.mixer.q_conv.taps == L["mixer"]["conv"]


@pytest.mark.parametrize("path, value, needle", [
    (("layers", 0, "type"), "mamba", "not built"),
    (("layers", 0, "mlp", "kind"), "dense", "not built"),
    (("layers", 0, "mlp", "router", "groups", "count"), 5, "equal groups"),
    (("layers", 0, "mlp", "router", "groups", "keep"), 4, "cannot be kept"),
    (("layers", 0, "mlp", "router", "top"), 9, "cannot be chosen"),
    (("layers", 0, "mixer", "left", "kv_heads"), 3, "multiple"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 7, "even"),
    (("layers", 0, "mixer", "right", "blocks"), 5, "equal blocks"),
    (("layers", 1, "mixer", "conv"), 0, "positive"),
    (("norm", "eps"), 0.0, "positive"),
])
def test_configuration_errors_name_the_place(path, value, needle):
    from inf_engine_b200.config import ConfigError
    d = copy.deepcopy(MODELS["kpz_a"])
    at = d
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        parse(d)
    assert needle in str(e.value)


def test_tensor_table_and_a_folder_that_loads_back(tmp_path):
    from inf_engine_b200.config import detect_config
    from inf_engine_b200.parts import expected_tensors
    folder = make_kipezen_dir(tmp_path, "kpz_a")
    cfg = detect_config(folder)
    exp = expected_tensors(cfg.model_spec())
    _, w = plain_inputs(folder)
    assert set(exp) == set(w) and all(tuple(exp[n].shape) == tuple(w[n].shape) for n in exp)
    assert exp["l0.mix.left.q.norm"].shape == (4 * 16,) and exp["l0.mix.right.ra"].shape == (3, 16, 16)
    assert exp["l1.mix.v.conv"].shape == (4 * 24, 3) and exp["l0.mlp.shared.sg"].shape == (1, 64)
    assert "l1.norm2" not in exp and "l0.mlp.e11.down" in exp and "l2.mlp.shared.gate" not in exp


def test_a_layer_may_keep_several_caches_and_a_window_keeps_its_first_pages():
    from inf_engine_b200.cache.manager import CacheManager, CacheRequirement
    kv = CacheRequirement(kind="kv", n_kv_heads=2, head_dim=16, window=20, dtype=torch.float32, keep_first=9)
    s1 = CacheRequirement(kind="state", state_shape=(4, 16, 24), state_dtype=torch.float32)
    s2 = CacheRequirement(kind="state", state_shape=(2, 96), state_dtype=torch.float32)
    several = CacheRequirement(kind="several", parts=(kv, CacheRequirement(kind="several", parts=(s1, s2))))
    m = CacheManager([several, CacheRequirement(kind="several", parts=(s1, s2)), several], page_size=8, n_pages=32, max_requests=2)
    assert len(m.kv_groups) == 1 and len(m.state_groups) == 2 and m.kv_groups[0].keep_first == 9
    b0, b1, b2 = m.bindings
    assert b0.kind == "several" and b0.parts[0].kind == "kv" and b0.parts[1].parts[0].kind == "state"
    assert (b0.parts[0].row, b2.parts[0].row) == (0, 1) and (b0.parts[1].parts[0].row, b1.parts[0].row, b2.parts[1].parts[0].row) == (0, 1, 2)
    # kept keys 0..8 live on pages 0 and 1; at length 100 the window holds keys 81.. : pages 2..9 go back, 0 and 1 stay
    assert m.open("a") is not None and m.reserve("a", 100)
    m.advance("a", 100)
    table = m.table(0, "a")
    assert [p >= 0 for p in table] == [True, True] + [False] * 8 + [True] * 3
    m.check()
    assert m.kv_groups[0].pool.n_held == 5
    assert m.reserve("a", 130)
    m.advance("a", 130)
    assert [p >= 0 for p in m.table(0, "a")][:3] == [True, True, False]
    m.close("a")
    m.check()
    assert m.kv_groups[0].pool.n_held == 0
    # without kept keys the same window gives its first pages back too
    plain_window = CacheManager([CacheRequirement(kind="kv", n_kv_heads=2, head_dim=16, window=20, dtype=torch.float32)], 8, 32, 2)
    plain_window.open("a")
    plain_window.reserve("a", 100)
    plain_window.advance("a", 100)
    assert [p >= 0 for p in plain_window.table(0, "a")] == [False] * 10 + [True] * 3


def test_plain_model_a_prefix_gives_the_same_logits(tmp_path):
    for name in ("kpz_a", "kpz_d"):
        folder = make_kipezen_dir(tmp_path, name)
        cfg, w = plain_inputs(folder)
        toks = random_tokens(cfg["vocab"], 50, 4)
        full = plain.forward_logits(w, cfg, toks)
        assert torch.allclose(plain.forward_logits(w, cfg, toks[:23]), full[:23], atol=1e-10)


def test_plain_route_keeps_to_the_best_groups_and_weights_without_the_correction():
    torch.manual_seed(0)
    E, top, groups, keep = 12, 3, 3, 2
    z = torch.randn(40, E, dtype=torch.float64) * 2
    corr = torch.randn(E, dtype=torch.float64) - 0.5
    w = {"r.router": torch.eye(E, dtype=torch.float64), "r.correction": corr}
    ids, wts = plain.route(z, w, "r.", {"experts": E, "top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}})
    s = torch.sigmoid(z)
    choice = s + corr
    for t in range(40):
        score = [sorted(choice[t, g * 4:(g + 1) * 4].tolist())[-2:] for g in range(groups)]
        best = sorted(range(groups), key=lambda g: -sum(score[g]))[:keep]
        allowed = [e for e in range(E) if e // 4 in best]
        want = sorted(allowed, key=lambda e: -float(choice[t, e]))[:top]
        assert sorted(ids[t].tolist()) == sorted(want)
        picked = s[t, ids[t]]
        assert torch.allclose(wts[t], picked / picked.sum() * 1.7)


def test_plain_convolution_looks_back_only():
    torch.manual_seed(1)
    x, w = torch.randn(9, 5, dtype=torch.float64), torch.randn(5, 4, dtype=torch.float64)
    y = plain.causal_conv(x, w)
    want = torch.zeros_like(x)
    for t in range(9):
        for j in range(4):
            src = t - (3 - j)
            if src >= 0:
                want[t] += w[:, j] * x[src]
    assert torch.allclose(y, want)
    x2 = x.clone()
    x2[6:] += 1.0
    assert torch.equal(plain.causal_conv(x2, w)[:6], y[:6])


def test_plain_window_keeps_the_first_tokens_at_their_positions(tmp_path):
    """A sequence that is shorter than the window sees every key; rotating by pairs leaves the part of a head beyond
    the rotated dimensions alone and turns a pair by its position's angle."""
    x = torch.arange(24, dtype=torch.float64).reshape(2, 1, 12) + 1
    y = plain.rotate_interleaved(x, torch.tensor([0, 3]), 8, 100.0)
    assert torch.equal(y[0], x[0]) and torch.equal(y[1, 0, 8:], x[1, 0, 8:])
    a = 3 * 100.0 ** (-2.0 * 1 / 8)
    u, v = x[1, 0, 2], x[1, 0, 3]
    assert torch.allclose(y[1, 0, 2:4], torch.stack([u * torch.cos(torch.tensor(a)) - v * torch.sin(torch.tensor(a)),
                                                     v * torch.cos(torch.tensor(a)) + u * torch.sin(torch.tensor(a))]))
