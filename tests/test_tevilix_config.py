"""The Tevilix decoder on the CPU: reading of config.json, the plan, cache needs, random weights and the loader's
names, and the plain implementation's own pieces."""
import copy
import os

import numpy as np
import pytest
import torch

import harness  # noqa: F401  (puts the repository and tests/ on the path)
import plain_tevilix as P
from tevilix_configs import ALL, T_A, T_B, T_C


def plan_of(cfg):
    from lastengine_b200.registry import plan_from_config
    return plan_from_config(cfg)


def test_every_size_and_constant_comes_from_the_file():
    from lastengine_b200.config import TevilixConfig
    c = TevilixConfig.from_dict(T_A)
    assert (c.vocab, c.width, c.eps, c.embedding_scale) == (200, 64, 1e-5, 3.0)
    assert [l.type for l in c.layers] == ["mlstm", "parallel", "mlstm", "parallel"]
    a = c.layers[1].mixer
    assert (a.left.heads, a.left.kv_heads, a.left.dim, a.left.vdim, a.left.scale, a.left.window) == (6, 2, 32, 16, 0.2, 20)
    assert (a.left.rot.dims, a.left.rot.base, a.left.rot.factor) == (16, 10000.0, 4.0)
    assert (a.left_scale, a.right_width, a.right_scale) == (0.7, 48, 1.3)
    m = c.layers[0].mixer
    assert (m.heads, m.dim, m.vdim, m.gate_cap) == (4, 16, 24, 8.0)
    f = c.layers[1].mlp
    assert (f.experts, f.top, f.groups, f.keep, f.scale, f.ff) == (8, 2, 4, 2, 1.5, 32)
    assert c.layers[2].mlp is None and c.layers[0].mlp.ff == 96
    assert c.runs() == [0, 1, 2, 1, 2, 3]


def test_what_may_be_absent_has_the_design_s_defaults():
    from lastengine_b200.config import TevilixConfig
    c = TevilixConfig.from_dict(T_C)
    assert c.embedding_scale == 1.0 and c.loop is None and c.runs() == [0, 1, 2, 3, 4]
    assert c.layers[0].mixer.left.rot.dims == 0 and c.layers[0].mixer.left.window == 1
    assert c.layers[2].mixer.left.window == 0 and c.layers[2].mixer.left.rot.dims == 0
    assert c.layers[4].mixer.left.rot.factor == 1.5
    a = TevilixConfig.from_dict(T_A)
    assert a.layers[3].mixer.left.rot.factor == 1.0 and (a.layers[3].mlp.groups, a.layers[3].mlp.keep) == (1, 1)
    assert TevilixConfig.from_dict(T_B).runs() == [0, 1, 2, 0, 1, 2]


@pytest.mark.parametrize("path,value,word", [
    (("layers", 1, "mixer", "left", "kv_heads"), 4, "kv_heads"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 15, "even"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 64, "rot.dims"),
    (("layers", 1, "mixer", "left", "rot", "scaling", "factor"), 0.0, "positive"),
    (("layers", 0, "mixer", "gate_cap"), -1.0, "gate_cap"),
    (("layers", 1, "mlp", "router", "top"), 9, "top"),
    (("layers", 1, "mlp", "router", "groups", "count"), 3, "groups"),
    (("layers", 0, "type"), "conv", "unknown layer type"),
    (("layers", 0, "mlp", "kind"), "gated", "unknown mlp kind"),
    (("loop", "stop"), 7, "loop"),
])
def test_errors_name_the_key(path, value, word):
    from lastengine_b200.config import ConfigError, TevilixConfig
    cfg = copy.deepcopy(T_A)
    at = cfg
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        TevilixConfig.from_dict(cfg)


def test_a_missing_key_is_named():
    from lastengine_b200.config import ConfigError, TevilixConfig
    cfg = copy.deepcopy(T_A)
    del cfg["layers"][1]["mixer"]["left"]["scale"]
    with pytest.raises(ConfigError, match="scale"):
        TevilixConfig.from_dict(cfg)
    cfg = copy.deepcopy(T_A)
    del cfg["layers"][0]["mixer"]["gate_cap"]
    with pytest.raises(ConfigError, match="gate_cap"):
        TevilixConfig.from_dict(cfg)


def test_plan_schedule_cache_needs_and_names():
    from lastengine_b200.engine.model import Model
    from lastengine_b200.parts.base import BuildEnv, KVSpec, StateSpec
    plan = plan_of(T_A)
    assert plan.architecture == "Tevilix" and [e.layer for e in plan.schedule] == [0, 1, 2, 1, 2, 3]
    model = Model(plan, BuildEnv(torch.device("cpu"), torch.float32))
    specs = model.cache_specs()
    assert len(specs) == 6                                        # every layer run keeps its own
    assert specs[0] == (StateSpec((4, 25, 16)), StateSpec((4,)))
    assert specs[1] == specs[3] == (KVSpec(2, 32, 20, 16), StateSpec((48,)))
    assert specs[5] == (KVSpec(1, 16, 33, 48), StateSpec((80,)))
    names = {plan.checkpoint_names(n) for n in model.tensor_specs()}
    for n in ("embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.i.b", "l0.mix.norm", "l0.mlp.up",
              "l1.mix.left.q.b", "l1.mix.left.talk", "l1.mix.left.q.norm", "l1.mix.left.o.b", "l1.mix.left.g",
              "l1.mix.right.z.b", "l1.mix.right.o", "l1.mlp.router", "l1.mlp.correction", "l1.mlp.e7.down", "l2.norm1"):
        assert n in names, n
    assert "l2.norm2" not in names and "l1.mlp.e0.gate" not in names and "l1.mlp.e8.up" not in names


def test_random_folder_goes_through_the_loader(tmp_path):
    from lastengine_b200.weights import write_model_dir
    from lastengine_b200.weights.safetensors_io import SafetensorsFile
    d = write_model_dir(T_C, str(tmp_path / "m"), seed=3, norm_init="random")
    sf = SafetensorsFile(os.path.join(d, "model.safetensors"))
    w = P.read_safetensors(os.path.join(d, "model.safetensors"))
    assert set(sf.names()) == set(w)
    assert w["l0.mix.left.talk"].shape == (5, 5) and w["l3.mix.norm"].shape == (40,) and w["l2.mlp.e8.up"].shape == (14, 40)
    lg = P.forward(T_C, w, [1, 2, 3, 4])
    assert lg.shape == (4, 97) and np.all(np.isfinite(lg))


def test_plain_group_choice_takes_the_sum_of_the_two_best_and_minus_infinity_outside():
    """Group 0 holds the single best expert, group 1 the best pair: the pair wins, and a negative choice score
    inside the kept group beats every score outside it."""
    D = 4
    w = {"router": np.zeros((6, D)), "correction": np.array([0.9, -0.9, -0.9, 0.3, 0.35, -0.8])}
    h = np.ones((1, D))
    r = {"experts": 6, "top": 3, "scale": 2.0, "groups": {"count": 2, "keep": 1}}
    ids, wts, c = P.route(h, w, r)
    assert sorted(ids[0].tolist()) == [3, 4, 5]                    # s = 1/2 everywhere: c = 1.4, -0.4, -0.4 | 0.8, 0.85, -0.3
    assert np.all(np.isinf(c[0, :3])) and np.allclose(wts.sum(), 2.0)
    r["groups"]["keep"] = 2
    assert sorted(P.route(h, w, r)[0][0].tolist()) == [0, 3, 4]


def test_plain_minimal_unit_candidate_and_memory_gates():
    w = {"z": np.zeros((1, 1)), "z.b": np.array([0.0]), "x": np.ones((1, 1)), "x.b": np.array([0.0]),
         "g": np.zeros((1, 1)), "o": np.ones((1, 1))}
    out = P.min_gru(np.array([[2.0], [-1.0]]), dict(w, g=np.ones((1, 1))))
    s1 = 0.5 * 2.5                              # z = 1/2; u = 2 >= 0: candidate u + 1/2
    s2 = 0.5 * s1 + 0.5 / (1 + np.e)           # u = -1 < 0: candidate sigmoid(-1)
    silu = lambda v: v / (1 + np.exp(-v))      # noqa: E731
    assert np.allclose(out[:, 0], [s1 * silu(2.0), s2 * silu(-1.0)])
    for n, cfg in ALL.items():
        assert P.layer_order(cfg)[0] == 0 and len(P.layer_order(cfg)) >= len(cfg["layers"])
