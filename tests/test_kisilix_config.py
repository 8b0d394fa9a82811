"""The Kisilix configuration, plan, tensor list and cache layout, and the plain implementation's own
mechanisms against closed forms (no GPU)."""
import copy
import os

import numpy as np
import pytest
import torch

import plain_kisilix as P
from kisilix_configs import ALL, K_A, K_B, K_C, att


def plan_of(cfg):
    from lastengine_b200.registry import plan_from_config
    return plan_from_config(cfg)


def test_plan_follows_the_layer_list():
    plan = plan_of(K_A)
    assert [l.mixer.kind for l in plan.layers] == ["pooled_window_attention", "gated_delta_rule", "state_space",
                                                   "pooled_window_attention"]
    assert [None if l.ffn is None else l.ffn.kind for l in plan.layers] == ["gated_dense", "topk_moe", None, "topk_moe"]
    assert all(l.block == "post_norm_residual" and l.block_params == {"alpha": 1.5} for l in plan.layers)
    assert plan.max_positions == 512 and plan.vocab_size == 200 and plan.hidden_size == 64
    a = plan.layers[0].mixer.params
    assert (a["window"], a["pool"], a["scale"], a["v_head_dim"], a["value_rotation_base"]) == (20, 6, 0.2, 16, 10000.0)
    m = plan.layers[1].ffn.params
    assert m["groups"] == (4, 2) and m["top_k"] == 2 and m["shared_size"] == 48
    plan = plan_of(K_C)
    assert plan.layers[1].mixer.params["position"].kind == "none"           # no rotated dimensions of q and k
    assert plan.layers[1].mixer.params["value_rotation_base"] == 10000.0     # the values still turn


@pytest.mark.parametrize("edit,needle", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c.pop("postln_alpha"), "postln_alpha"),
    (lambda c: c.pop("max_positions"), "max_positions"),
    (lambda c: c["layers"][0].__setitem__("type", "retention"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "does not divide"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 64), "more than dim"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("vdim", 15), "odd"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("groups", 3), "does not divide"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("norm_groups", 5), "does not divide"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "experts"), "unknown mlp kind"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9), "top 9 of 8"),
    (lambda c: c["layers"][3]["mlp"]["router"]["groups"].update(count=3, keep=1), "cannot give"),
    (lambda c: c.__setitem__("norm", 1e-5), "must be an object"),
])
def test_config_errors_name_the_key(edit, needle):
    from lastengine_b200.config import ConfigError
    cfg = copy.deepcopy(K_A)
    edit(cfg)
    with pytest.raises(ConfigError, match=needle):
        plan_of(cfg)


def test_written_folder_reads_back_with_the_design_s_tensor_names(tmp_path):
    from lastengine_b200.weights import write_model_dir
    from lastengine_b200.weights.safetensors_io import SafetensorsFile
    d = write_model_dir(K_A, str(tmp_path / "m"), seed=3, norm_init="random")
    names = set(SafetensorsFile(os.path.join(d, "model.safetensors")).names())
    assert {"embed", "pos", "head", "final.norm", "final.norm.b", "l0.norm1", "l0.norm2.b", "l0.mix.q.b", "l0.mix.k.norm",
            "l0.mix.temp", "l0.mlp.gate", "l1.mix.q.conv", "l1.mix.a1", "l1.mix.g2", "l1.mix.dt_bias", "l1.mix.b",
            "l1.mlp.router", "l1.mlp.correction", "l1.mlp.e7.down", "l1.mlp.shared.up", "l2.mix.in", "l2.mix.conv.b",
            "l2.mix.D", "l2.mix.norm", "l3.mlp.e5.gate"} <= names
    assert "l2.norm2" not in names and "l2.mlp.gate" not in names          # a layer without a feed-forward
    t = P.read_safetensors(os.path.join(d, "model.safetensors"))
    assert t["pos"].shape == (512, 64) and t["l2.mix.in"].shape == (2 * 64 + 2 * 2 * 24 + 4, 64)
    assert t["l1.mix.k.conv"].shape == (2 * 16, 4) and t["l1.mix.a2"].shape[0] == 4 * 16
    lg, streams = P.forward(K_A, t, [1, 2, 3, 4, 5], want_layers=True)
    assert lg.shape == (5, 200) and np.isfinite(lg).all() and streams.shape == (4, 5, 64)


def test_the_low_ranks_are_the_checkpoint_s(tmp_path):
    """The two low-rank pairs of the delta mixer have whatever inner size the stored tensors have."""
    from lastengine_b200.engine.model import Model
    from lastengine_b200.parts.base import BuildEnv
    m = Model(plan_of(K_A), BuildEnv(device=torch.device("cpu"), dtype=torch.float32))
    specs = m.tensor_specs()
    a1, a2 = specs["l1.mix.a1"], specs["l1.mix.a2"]
    assert a1.fits((5, 64)) and a1.fits((31, 64)) and not a1.fits((5, 63))
    assert a2.fits((64, 5)) and not a2.fits((63, 5))


def test_cache_keeps_pooled_rows_in_pages_of_their_own_and_gives_window_pages_back():
    from lastengine_b200.cache import Cache
    from lastengine_b200.parts.base import KVSpec, StateSpec
    spec = KVSpec(2, 16, window=20, v_head_dim=8, pool=6)
    cache = Cache({0: spec, 1: (StateSpec((2, 4, 8), torch.float32), StateSpec((12, 2), torch.float32))},
                  max_tokens=1024, max_seqs=3, dtype=torch.float32, device=torch.device("cpu"), page_size=32)
    g = cache.kv_groups[0]
    s = cache.alloc_seq()
    cache.reserve({s: 100})
    cache.commit({s: 100})
    assert len(g.seq_pages[s]) == 4 and len(g.seq_pooled_pages[s]) == 1          # 16 pooled rows in one page
    # the next query, at 100, reaches back to 81; block 16 (96..101) is still filling
    assert [p >= 0 for p in g.seq_pages[s]] == [False, False, True, True]
    cache.reserve({s: 98})
    cache.commit({s: 98})
    assert len(g.seq_pooled_pages[s]) == 2                                       # block 32 ended at position 197
    assert [p >= 0 for p in g.seq_pages[s]] == [False] * 5 + [True] * 2
    view = cache.view(1, True, {})
    assert [tuple(t.shape[1:]) for t in view.states] == [(2, 4, 8), (12, 2)] and view.state is view.states[0]
    held = g.pages.n_held
    cache.free_seq(s)
    assert g.pages.n_held == 0 and g.pooled_pages.n_held == 0 and held == 2
    cache.check()


def test_a_block_larger_than_the_window_keeps_its_positions_until_it_is_pooled():
    from lastengine_b200.cache import Cache
    from lastengine_b200.parts.base import KVSpec
    cache = Cache({0: KVSpec(1, 8, window=4, pool=40)}, max_tokens=512, max_seqs=2, dtype=torch.float32,
                  device=torch.device("cpu"), page_size=32)
    g = cache.kv_groups[0]
    s = cache.alloc_seq()
    cache.reserve({s: 39})
    cache.commit({s: 39})
    assert all(p >= 0 for p in g.seq_pages[s])          # block 0 is not complete: its 39 positions stay
    cache.reserve({s: 2})
    cache.commit({s: 2})
    assert [p >= 0 for p in g.seq_pages[s]] == [False, True]      # pooled at 39; the window is 38..41


# ---- the plain implementation's mechanisms against closed forms ------------------------------------
def test_plain_conv_sees_zeros_before_the_start_and_nothing_ahead():
    u = np.arange(1.0, 7.0)[:, None].repeat(2, 1)
    w = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    y = P.causal_conv(u, w, bias=np.array([0.5, 0.0]))
    assert y[:, 0].tolist() == [100.5, 210.5, 321.5, 432.5, 543.5, 654.5]      # the last column meets the current row
    assert y[:, 1].tolist() == u[:, 1].tolist()


def test_plain_rotation_keeps_norms_turns_back_and_depends_on_distance_only():
    rng = np.random.default_rng(1)
    a, b = rng.standard_normal((1, 1, 12)), rng.standard_normal((1, 1, 12))
    ra = P.rotate_halves(a.repeat(3, 0), np.array([5, 105, 7]), 100.0, 8)
    rb = P.rotate_halves(b.repeat(3, 0), np.array([2, 102, 7]), 100.0, 8)
    assert np.allclose(np.linalg.norm(ra, axis=-1), np.linalg.norm(a))
    assert np.array_equal(ra[..., 8:], a.repeat(3, 0)[..., 8:])                  # the rest of the head passes unchanged
    assert np.allclose((ra[0] * rb[0]).sum(), (ra[1] * rb[1]).sum(), atol=1e-5)
    assert np.allclose(P.rotate_halves(ra, -np.array([5, 105, 7]), 100.0, 8), a.repeat(3, 0), atol=1e-12)
    # pair (i, i + dims/2): a unit vector on dimension 1 lands on dimensions 1 and 5
    e1 = np.zeros((1, 1, 12)); e1[0, 0, 1] = 1.0
    r = P.rotate_halves(e1, np.array([3]), 100.0, 8)[0, 0]
    ang = np.float32(3) * np.float32(100.0) ** np.float32(-2 * 1 / 8)
    assert np.allclose(r[[1, 5]], [np.cos(ang), np.sin(ang)], atol=1e-6) and np.count_nonzero(r) == 2


def test_plain_delta_rule_writes_a_value_and_reads_it_back():
    """One head, no decay (A_log far below zero), beta one: after writing v at a unit key, that key reads v back;
    writing another value at the same key replaces it."""
    d, e = 4, 3
    S = np.zeros((d, e))
    k = np.array([0.0, 1.0, 0.0, 0.0])
    for v in (np.array([1.0, 2.0, 3.0]), np.array([-4.0, 0.5, 9.0])):
        u = 1.0 * (v - S.T @ k)
        S = S + np.outer(k, u)
        assert np.allclose(S.T @ k, v)


def test_plain_window_and_blocks_by_the_definition():
    """Which positions and blocks a query sees, against the definition written out: j with 0 <= i - j < size,
    block b if its last position b P + P - 1 <= i - size."""
    T, size, Pn = 40, 7, 3
    m = att(1, 1, 4, 2, 1.0, 0, 10.0, size, Pn)
    rng = np.random.default_rng(2)
    D = 6
    w = {"q": rng.standard_normal((4, D)), "k": rng.standard_normal((4, D)), "v": rng.standard_normal((2, D)),
         "q.b": np.zeros(4), "k.b": np.zeros(4), "v.b": np.zeros(2), "q.norm": np.ones(4), "k.norm": np.ones(4),
         "temp": np.ones(1), "o": np.eye(2)}
    x = rng.standard_normal((T, D))
    got = P.pooled_window_attention(x, w, m, 1e-6)
    q = P.unit_rms(x @ w["q"].T, 1e-6)
    k = P.unit_rms(x @ w["k"].T, 1e-6)
    v = P.rotate_halves((x @ w["v"].T)[:, None, :], np.arange(T), 10.0, 2)[:, 0]
    for i in (0, 6, 7, 9, 10, 39):
        keys, vals = [], []
        for b in range(T // Pn):
            if b * Pn + Pn - 1 <= i - size:
                keys.append(k[b * Pn:(b + 1) * Pn].mean(0)); vals.append(v[b * Pn:(b + 1) * Pn].mean(0))
        for j in range(T):
            if 0 <= i - j < size:
                keys.append(k[j]); vals.append(v[j])
        s = np.exp(np.array(keys) @ q[i]); s /= s.sum()
        o = P.rotate_halves((s @ np.array(vals))[None, None, :], -np.array([i]), 10.0, 2)[0, 0]
        assert np.allclose(got[i], o, atol=1e-9), i
    assert (6 - size + 1) // Pn == 0 and sum(b * Pn + Pn - 1 <= 9 - size for b in range(13)) == 1


def test_plain_router_keeps_the_best_groups_and_weights_without_the_correction():
    f = {"router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}}
    x = np.eye(6)[:1]
    logits = np.array([2.0, 0.0, 1.9, 1.8, -1.0, -1.0])
    w = {"router": np.eye(6) * logits, "correction": np.array([0.0, 0.0, 0.0, 0.0, 0.9, 0.0])}
    # x = e0: only expert 0's logit is non-zero -> z = [2, 0, 0, 0, 0, 0]; the correction lifts expert 4
    ids, wts, _ = P.route(x, w, f)
    s = np.exp([2.0, 0, 0, 0, 0, 0]); s /= s.sum()
    assert set(ids[0]) == {4, 5}                              # group 2 wins by the corrected score of expert 4
    assert np.allclose(wts[0], s[ids[0]] / s[ids[0]].sum())   # weights from the scores without it
    w["correction"] = np.array([0.0, -5.0, 0.0, 0.0, 0.0, 0.0])
    ids, _, _ = P.route(x, w, f)
    assert set(ids[0]) == {0, 1}                              # a negative choice score still beats an excluded expert
