"""The Tevilix decoder on the GPU against the plain implementation (tests/plain_tevilix.py): every mechanism
alone, then whole models: prompts whole, in portions and token by token, unequal batches, slots and pages used
again, keys far away, at page borders and at the window's edges, states carried from far back, long decoding,
and greedy generation through the entry point."""
import os

import numpy as np
import pytest
import torch

import harness as H
import plain_tevilix as P
from harness import MixerRig, max_err as err, random_rows as inputs, whole_portions_and_batches
from tevilix_configs import ALL, att, dense, mls, moe, random_config

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": H.TOL_F32, "bfloat16": H.TOL_BF16}


def K():
    from lastengine_b200.ops import kernels
    return kernels


def rope(dims, base, factor):
    from lastengine_b200.parts.base import PartSpec
    return PartSpec("rope", {"rope_dim": dims, "theta": base, "style": "neox", "scaling_factor": factor}) if dims \
        else PartSpec("none")


# ---- attention with mixed heads ---------------------------------------------------------------------
def att_params(D, heads, kv, dim, vdim, scale, rot, base, factor, size, eps=1e-5):
    return dict(hidden_size=D, num_heads=heads, num_kv_heads=kv, head_dim=dim, v_head_dim=vdim, norm_eps=eps, scale=scale,
                window=size, position=rope(rot, base, factor))


ATT_CASES = [  # heads, kv heads, dim, vdim, scale, rotated, base, factor, window
    (6, 2, 32, 16, 0.2, 16, 10000.0, 4.0, 20),
    (3, 3, 64, 64, 0.125, 64, 200000.0, 1.0, 70),
    (4, 1, 128, 128, 0.09, 32, 1e6, 8.0, 9),
    (5, 5, 12, 20, 0.25, 0, 1.0, 1.0, 1),             # sizes off the 16-byte grid, a window of one position
    (2, 2, 24, 10, 0.4, 0, 1.0, 1.0, 0),              # no window
    (3, 1, 40, 24, 0.1, 40, 20000.0, 1.5, 64),
    (8, 4, 64, 32, 0.15, 32, 50000.0, 2.0, 128),
    (16, 2, 16, 40, 0.3, 8, 100.0, 1.0, 150),         # more pairs than a warp each: several pairs per warp
    (1, 1, 8, 8, 0.5, 8, 10000.0, 3.0, 5),
    (40, 8, 16, 8, 0.2, 16, 10000.0, 1.0, 100),       # more heads than a row of the block's pairs takes at once
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv,dim,vdim,scale,rot,base,factor,size", ATT_CASES)
def test_attention_alone_whole_in_portions_and_batched(heads, kv, dim, vdim, scale, rot, base, factor, size, dtype):
    D = 48
    rig = MixerRig("mixed_heads_attention", att_params(D, heads, kv, dim, vdim, scale, rot, base, factor, size), dtype, seed=3)
    m = att(heads, kv, dim, vdim, scale, rot if rot else None, base, factor, size)
    whole_portions_and_batches(rig, lambda h: P.mixed_heads_attention(h, rig.plain, m, 1e-5), (150, 1, 67), 21,
                               [0, 2, 3, 8, 9, 21], TOL[dtype], dtype == "bfloat16")


MMA_CASES = [  # heads, kv heads, dim, vdim, window: sizes the tensor-core kernel takes
    (4, 2, 128, 64, 75), (6, 2, 32, 16, 20), (32, 8, 64, 64, 200), (16, 4, 64, 32, 0), (3, 3, 64, 64, 70), (8, 1, 16, 8, 33),
    (32, 2, 16, 64, 100), (2, 2, 256, 24, 150),
]


@pytest.mark.parametrize("heads,kv,dim,vdim,size", MMA_CASES)
def test_tensor_core_attention_against_the_general_kernel_and_the_plain_one(heads, kv, dim, vdim, size):
    """bfloat16 prompts of 8 rows and more run the tensor-core kernel: whole, in portions that start and end off the
    tile grid, batched with unequal lengths; the same steps through the general kernel give the same numbers up to the
    rounding of the two kernels' different orders of summation."""
    assert K().lib().leb_attention_mixed_mma_supported(heads, kv, dim, vdim, 64)
    D = 48
    m = att(heads, kv, dim, vdim, 0.2, 16, 10000.0, 2.0, size)
    outs = {}
    for mma in (True, False):
        K().set_mixed_attention_mma(mma)
        try:
            rig = MixerRig("mixed_heads_attention", att_params(D, heads, kv, dim, vdim, 0.2, 16, 10000.0, 2.0, size), "bfloat16", seed=3)
            hs = [inputs(n, D, 70 + n, True) for n in (300, 9, 77)]
            slots = [rig.cache.alloc_seq() for _ in hs]
            got = [rig.step(slots, [h[:n] for h, n in zip(hs, (131, 8, 40))]), rig.step(slots, [h[n:] for h, n in zip(hs, (131, 8, 40))])]
            outs[mma] = [np.concatenate([a, b]) for a, b in zip(*got)]
            for s_ in slots:
                rig.cache.free_seq(s_)
        finally:
            K().set_mixed_attention_mma(True)
    for h, a, b in zip(hs, outs[True], outs[False]):
        want = P.mixed_heads_attention(h, rig.plain, m, 1e-5)
        assert err(a, want) < H.TOL_BF16 and err(b, want) < H.TOL_BF16
        assert err(a, b) < H.TOL_BF16 / 2


def test_the_mixing_matrix_matters_and_is_applied_before_the_softmax():
    """With the identity in its place the result is plain attention and far from the mixed one; a matrix that
    copies head 1's scores into head 0 makes head 0 weigh its own values by head 1's weights."""
    D, heads, kv, dim, vdim = 32, 2, 2, 16, 8
    params = att_params(D, heads, kv, dim, vdim, 0.5, 0, 1.0, 1.0, 0)
    m = att(heads, kv, dim, vdim, 0.5, None, None, None, 0)
    rig = MixerRig("mixed_heads_attention", params, "float32", seed=4)
    h = inputs(40, D, 1, False)
    mixed = P.mixed_heads_attention(h, rig.plain, m, 1e-5)
    plain_w = dict(rig.plain, talk=np.eye(2))
    assert err(P.mixed_heads_attention(h, plain_w, m, 1e-5), mixed) > 0.05
    assert err(rig.alone(h), mixed) < H.TOL_F32

    def edit(t):
        t["talk"][:] = [[0.0, 1.0], [0.0, 1.0]]
    rig2 = MixerRig("mixed_heads_attention", params, "float32", seed=4, edit=edit)
    want = P.mixed_heads_attention(h, rig2.plain, m, 1e-5)
    assert err(rig2.alone(h), want) < H.TOL_F32


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds_is_found_in_a_prompt_and_while_decoding(dtype):
    """No window.  Position 3 carries a key that only the last rows' queries match (one input channel drives a
    large component of q and k), so those rows put nearly all their weight 600 positions back: a key lost at a page
    border, or a split of the key range merged wrongly, changes their result."""
    D, heads, kv, dim, vdim = 32, 4, 2, 16, 16
    params = att_params(D, heads, kv, dim, vdim, 1.0, 0, 1.0, 1.0, 0)
    m = att(heads, kv, dim, vdim, 1.0, None, None, None, 0)

    def edit(t):
        for n in ("q", "k"):
            t[n][:, :2] = 0.0
        t["q"][::dim, 0] = 6.0              # channel 0 drives the first number of every q head, channel 1 of every k head
        t["k"][::dim, 1] = 6.0
        t["q.norm"][:] = 1.0
        t["k.norm"][:] = 1.0
        t["talk"][:] = np.eye(heads) + 0.1
    rig = MixerRig("mixed_heads_attention", params, dtype, seed=6, edit=edit, max_tokens=4096)
    bf = dtype == "bfloat16"
    h = inputs(640, D, 2, bf, 0.3)
    h[:, :2] = 0.0
    h[3, 1] = 30.0                      # the key the last rows look for
    h[600:, 0] = 30.0
    want = P.mixed_heads_attention(h, rig.plain, m, 1e-5)
    lost = P.mixed_heads_attention(h[4:], rig.plain, m, 1e-5)
    assert err(lost[600 - 4: 605 - 4], want[600:605]) > 0.1          # the far key matters
    assert err(rig.alone(h), want) < TOL[dtype]
    s = rig.cache.alloc_seq()
    a = rig.step([s], [h[:598]])[0]
    tail = np.concatenate([rig.step([s], [h[i:i + 1]])[0] for i in range(598, 640)])
    rig.cache.free_seq(s)
    assert err(np.concatenate([a, tail]), want) < TOL[dtype]


@pytest.mark.parametrize("size,at", [(5, 70), (64, 64), (65, 100), (33, 127), (128, 200), (72, 191)])
def test_a_key_just_inside_and_just_outside_the_window_in_prompts_and_in_decoding(size, at):
    """A flagged key at position `at` holds nearly all the weight of every later row while the window keeps it:
    the row `size - 1` positions later still sees it, the next one does not.  Both in a whole prompt and
    token by token (where the cache gives pages back as the window moves on)."""
    D, heads, kv, dim, vdim = 24, 2, 1, 8, 8
    params = att_params(D, heads, kv, dim, vdim, 1.0, 0, 1.0, 1.0, size)
    m = att(heads, kv, dim, vdim, 1.0, None, None, None, size)

    def edit(t):
        for n in ("q", "k"):
            t[n][:, :2] = 0.0
        t["q"][::dim, 0] = 6.0              # channel 0 drives the first number of every q head, channel 1 of the k head
        t["k"][::dim, 1] = 6.0
        t["q.norm"][:] = 1.0
        t["k.norm"][:] = 1.0
    rig = MixerRig("mixed_heads_attention", params, "float32", seed=7, edit=edit)
    T = at + size + 6
    h = inputs(T, D, 5, False, 0.3)
    h[:, 0] = 30.0                      # every query looks for the flag
    h[:, 1] = 0.0
    h[at, 1] = 30.0                     # the flagged key
    want = P.mixed_heads_attention(h, rig.plain, m, 1e-5)
    last_in, first_out = at + size - 1, at + size
    moved = h.copy()
    moved[at, 2:] += 3.0                # another value under the flag: rows that see it change, the others do not
    other = P.mixed_heads_attention(moved, rig.plain, m, 1e-5)
    assert np.abs(other[last_in] - want[last_in]).max() > 5e-3 * np.abs(want).max()
    assert np.abs(other[first_out] - want[first_out]).max() < 1e-9
    got = rig.alone(h)
    assert err(got, want) < H.TOL_F32
    assert err(got[[last_in, first_out]], want[[last_in, first_out]]) < H.TOL_F32
    s = rig.cache.alloc_seq()
    first = rig.step([s], [h[:at + 2]])[0]
    tail = np.concatenate([rig.step([s], [h[i:i + 1]])[0] for i in range(at + 2, T)])
    rig.cache.free_seq(s)
    rig.cache.check()
    assert err(np.concatenate([first, tail]), want) < H.TOL_F32


# ---- the minimal gated recurrent unit ---------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [48, 25, 300, 1])
def test_min_gru_alone_whole_in_portions_and_batched(width, dtype):
    D = 40
    rig = MixerRig("min_gru", dict(hidden_size=D, width=width), dtype, seed=9)
    whole_portions_and_batches(rig, lambda h: P.min_gru(h, rig.plain), (150, 1, 37), 21, [0, 2, 3, 8, 9, 21], TOL[dtype],
                               dtype == "bfloat16")


def test_min_gru_keeps_what_was_written_far_back_and_a_freed_slot_starts_from_zero():
    """Channel 0 of the input drives the update gate alone: open at row 2, shut for hundreds of rows after it.
    The last rows still hold what row 2 wrote; a sequence in the slot just given back holds nothing of it."""
    D, W = 16, 12

    def edit(t):
        t["z"][:, :] = 0.0
        t["z"][:, 0] = 8.0
        t["z.b"][:] = 0.0
        t["x"][:, 0] = 0.0
        t["g"][:, 0] = 0.0
    rig = MixerRig("min_gru", dict(hidden_size=D, width=W), "float32", seed=11, edit=edit, max_seqs=1)
    h = inputs(500, D, 4, False)
    h[:, 0] = -3.0
    h[2, 0] = 3.0
    want = P.min_gru(h, rig.plain)
    gone = P.min_gru(h[3:], rig.plain)
    assert err(gone[-5:], want[-5:]) > 0.2
    s = rig.cache.alloc_seq()
    a = rig.step([s], [h[:470]])[0]
    tail = np.concatenate([rig.step([s], [h[i:i + 1]])[0] for i in range(470, 500)])
    rig.cache.free_seq(s)
    assert err(np.concatenate([a, tail]), want) < H.TOL_F32
    assert err(rig.alone(h[3:]), gone) < H.TOL_F32          # the same slot again: zero state


# ---- the matrix memory with exponential gates -------------------------------------------------------
MLSTM_CASES = [  # heads, dim, vdim, cap
    (4, 16, 24, 8.0),
    (2, 64, 32, 15.0),
    (3, 32, 64, 10.0),
    (5, 10, 6, 12.0),            # rows of a head that are no multiple of four numbers
    (1, 40, 40, 5.0),
    (3, 128, 64, 12.0),
    (6, 32, 16, 20.0),
    (2, 256, 15, 3.0),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,vdim,cap", MLSTM_CASES)
def test_mlstm_alone_whole_in_portions_and_batched(heads, dim, vdim, cap, dtype):
    D = 48
    rig = MixerRig("mlstm", dict(hidden_size=D, num_heads=heads, head_dim=dim, v_head_dim=vdim, gate_cap=cap, norm_eps=1e-5),
                   dtype, seed=12)
    m = mls(heads, dim, vdim, cap)
    # bfloat16: the unit norm of a head's read-out amplifies the rounding of the projections where the read-out is small
    tol = TOL[dtype] if dtype == "float32" else 2 * TOL[dtype]
    whole_portions_and_batches(rig, lambda h: P.mlstm(h, rig.plain, m, 1e-5), (150, 1, 37), 21, [0, 2, 3, 8, 9, 21], tol,
                               dtype == "bfloat16")


def test_mlstm_gates_reach_their_cap_and_the_running_maximum_is_carried():
    """Large gate inputs: the input gate sits at +cap for one row, at -cap for a few rows and low afterwards while
    the forget gate stays open, so the running maximum stays high for hundreds of rows, exp(-m) is tiny and the
    normaliser decides the read-out; then the same sequence token by token, and a fresh one in the slot given back
    (m from zero again, where exp(-m) = 1 decides)."""
    D, heads, dim, vdim, cap = 16, 2, 8, 8, 6.0

    def edit(t):
        t["i"][:, :] = 0.0
        t["i"][:, 0] = 5.0
        t["i.b"][:] = 0.0
        t["f"][:, :] = 0.0
        t["f.b"][:] = 9.0
        for n in ("q", "k", "v", "g"):
            t[n][:, 0] = 0.0
    rig = MixerRig("mlstm", dict(hidden_size=D, num_heads=heads, head_dim=dim, v_head_dim=vdim, gate_cap=cap, norm_eps=1e-5),
                   "float32", seed=13, edit=edit, max_seqs=1)
    m = mls(heads, dim, vdim, cap)
    h = inputs(400, D, 6, False)
    h[:, 0] = -0.4
    h[1, 0] = 20.0
    h[5:10, 0] = -20.0
    want = P.mlstm(h, rig.plain, m, 1e-5)
    gone = P.mlstm(h[2:], rig.plain, m, 1e-5)
    assert err(gone[-5:], want[-5:]) > 0.2               # what row 1 wrote still decides the last rows
    s = rig.cache.alloc_seq()
    a = rig.step([s], [h[:380]])[0]
    tail = np.concatenate([rig.step([s], [h[i:i + 1]])[0] for i in range(380, 400)])
    rig.cache.free_seq(s)
    assert err(np.concatenate([a, tail]), want) < H.TOL_F32
    assert err(rig.alone(h[2:]), gone) < H.TOL_F32


# ---- two mixers side by side -------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("a,b", [(0.7, 1.3), (1.0, 1.0), (0.0, 2.0)])
def test_mixers_side_by_side(a, b, dtype):
    from lastengine_b200.parts.base import PartSpec
    D = 40
    left = att_params(D, 4, 2, 16, 24, 0.3, 8, 1000.0, 2.0, 30)
    params = dict(left=PartSpec("mixed_heads_attention", left), right=PartSpec("min_gru", dict(hidden_size=D, width=56)),
                  left_scale=a, right_scale=b)
    rig = MixerRig("parallel_mixers", params, dtype, seed=14, hidden_size=D)
    m = {"left": att(4, 2, 16, 24, 0.3, 8, 1000.0, 2.0, 30), "left_scale": a, "right": {"width": 56}, "right_scale": b}
    whole_portions_and_batches(rig, lambda h: P.parallel_mixer(h, rig.plain, m, 1e-5), (100, 1, 37), 21, [0, 2, 3, 8, 9, 21],
                               TOL[dtype], dtype == "bfloat16")


# ---- feed-forwards ---------------------------------------------------------------------------------
def ffn_out(kind, params, dtype, h, seed=21, edit=None, std=0.3):
    """A feed-forward part alone: random weights by its own declaration; returns (output, plain tensors)."""
    from lastengine_b200.engine.workspace import Workspace
    from lastengine_b200.parts.base import BuildEnv
    from lastengine_b200.registry import FEED_FORWARDS
    from lastengine_b200.weights.loader import kept_dtype
    from lastengine_b200.weights.random_init import random_tensor
    dev = torch.device(DEV)
    env = BuildEnv(device=dev, dtype=DT[dtype], workspace=Workspace(dev))
    part = FEED_FORWARDS.get(kind)(**params)
    specs = part.tensors()
    plain = {n: random_tensor(n, s, seed, std, norm_init="random").to(torch.bfloat16).double().numpy().copy()
             for n, s in specs.items()}
    if edit:
        edit(plain)
        plain = {n: H.bf16_round_np(v) for n, v in plain.items()}
    part.load({n: torch.from_numpy(v).float().to(dev, kept_dtype(specs[n], torch.bfloat16, DT[dtype])) for n, v in plain.items()}, env)
    x = torch.from_numpy(h).to(DEV, DT[dtype])
    out = torch.zeros(h.shape[0], params["hidden_size"], dtype=torch.float32, device=DEV)
    part.forward(x, out, False, None, env)
    K().check_device_status()
    return out.double().cpu().numpy(), plain


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D,F,rows", [(48, 96, 70), (72, 48, 1), (40, 56, 200), (64, 320, 17), (42, 30, 5)])
def test_dense_feed_forward_with_the_erf_gelu(D, F, rows, dtype):
    h = inputs(rows, D, 3, dtype == "bfloat16")
    got, w = ffn_out("dense", dict(hidden_size=D, intermediate_size=F, activation="gelu"), dtype, h)
    want = P.dense_ff(h, w)
    assert err(got, want) < TOL[dtype]
    tanh_form = (lambda z: 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3))))(h @ w["up"].T) @ w["down"].T
    if dtype == "float32":
        assert err(tanh_form, want) > 4 * H.TOL_F32         # the two forms of gelu are told apart


MOE_CASES = [  # experts, top, groups, kept, scale, expert width
    (8, 2, 4, 2, 1.5, 32),
    (12, 1, 3, 1, 2.0, 16),
    (4, 2, 4, 3, 0.5, 40),         # groups of one expert
    (9, 2, 3, 2, 2.5, 14),
    (5, 5, 1, 1, 1.0, 8),          # every expert chosen
    (16, 4, 4, 1, 2.5, 24),
    (16, 3, 2, 1, 1.5, 80),
    (6, 3, None, None, 1.0, 24),   # no groups
]


def moe_params(D, E, top, count, keep, scale, F):
    return dict(hidden_size=D, num_experts=E, top_k=top, expert_size=F, router="sigmoid_grouped",
                groups=(count or 1, keep or 1), group_top=2, use_bias=True, scaling=scale, gated=False,
                activation="relu_squared",
                names={"router": "router", "bias": "correction", "up": "e{e}.up", "down": "e{e}.down"})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,count,keep,scale,F", MOE_CASES)
def test_grouped_experts_with_squared_relu(E, top, count, keep, scale, F, dtype):
    D = 48
    bf = dtype == "bfloat16"
    for rows in (1, 9, 300):
        h = inputs(rows, D, 30 + rows, bf)

        def edit(t):
            t["router"] *= 4.0               # scores well apart: the arithmetic is compared, not a coin toss
            t["correction"][:] = np.linspace(-0.4, 0.4, E)[np.random.default_rng(1).permutation(E)]
        got, w = ffn_out("topk_moe", moe_params(D, E, top, count, keep, scale, F), dtype, h, edit=edit)
        mlp = moe(E, top, count, keep, scale, F)
        want = P.experts_ff(h, w, mlp)
        gap = P.route_gap(h, w, mlp["router"])
        ok = gap > (1e-5 if not bf else 2e-2)
        assert ok.mean() > 0.5
        assert err(got[ok], want[ok]) < TOL[dtype], f"{rows} rows"


def test_a_group_ranks_by_its_two_best_and_an_excluded_group_loses_to_a_negative_choice_score():
    """Router rows of zero: every score is 1/2 and the corrections alone choose.  Group 0 holds the single best
    expert, group 1 the best pair, so group 1 is kept (ranking by the best alone would keep group 0), and its third
    expert, whose choice score is negative, is chosen before everything in group 0."""
    D, E = 16, 6
    h = inputs(5, D, 2, False)

    def edit(t):
        t["router"][:] = 0.0
        t["correction"][:] = [0.9, -0.9, -0.9, 0.3, 0.35, -0.8]
    got, w = ffn_out("topk_moe", moe_params(D, E, 3, 2, 1, 2.0, 8), "float32", h, edit=edit)
    mlp = moe(E, 3, 2, 1, 2.0, 8)
    ids, wts, _ = P.route(h, w, mlp["router"])
    assert sorted(ids[0].tolist()) == [3, 4, 5] and np.allclose(wts, 2.0 / 3.0)
    assert err(got, P.experts_ff(h, w, mlp)) < H.TOL_F32
    by_best = sum((2.0 / 3.0) * ((np.maximum(h @ w[f"e{e}.up"].T, 0) ** 2) @ w[f"e{e}.down"].T) for e in (0, 1, 2))
    assert err(by_best, got) > 0.1


@pytest.mark.parametrize("D", [40, 42, 64, 256, 1000, 2048])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_layer_norms_of_one_row_with_and_without_the_sum(D, dtype):
    rng = np.random.default_rng(D)
    x = rng.standard_normal((7, D)) * 3 + 1.5
    y = rng.standard_normal((7, D))
    w1, w2 = 1 + 0.1 * rng.standard_normal(D), 1 + 0.1 * rng.standard_normal(D)
    xd = torch.from_numpy(x).float().to(DEV)
    h1 = torch.empty(7, D, dtype=DT[dtype], device=DEV)
    h2 = torch.empty_like(h1)
    t1, t2 = (torch.from_numpy(w).float().to(DEV) for w in (w1, w2))
    K().layernorm_pair(h1, h2, xd, t1, t2, 1e-5)
    x32 = xd.double().cpu().numpy()
    assert err(h1.double().cpu().numpy(), P.layer_norm(x32, w1, 1e-5)) < TOL[dtype] / 2
    assert err(h2.double().cpu().numpy(), P.layer_norm(x32, w2, 1e-5)) < TOL[dtype] / 2
    K().layernorm_pair(h1, h2, xd, t1, t2, 1e-5, y=torch.from_numpy(y).float().to(DEV), mult=0.75)
    new = x32 + 0.75 * torch.from_numpy(y).float().double().numpy()
    assert err(xd.double().cpu().numpy(), new) < 1e-6
    assert err(h2.double().cpu().numpy(), P.layer_norm(new, w2, 1e-5)) < TOL[dtype] / 2


# ---- whole models --------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    from lastengine_b200.weights import write_model_dir
    return {n: write_model_dir(cfg, str(tmp_path_factory.mktemp("t" + n)), seed=51 + i, norm_init="random")
            for i, (n, cfg) in enumerate(ALL.items())}


_tensors, _plain = {}, {}


def tensors_of(name, dirs):
    if name not in _tensors:
        _tensors[name] = P.read_safetensors(os.path.join(dirs[name], "model.safetensors"))
    return _tensors[name]


def plain(name, dirs, tokens):
    """(logits [T, V], per position the smallest gap of a routing decision)."""
    key = (name, tuple(tokens))
    if key not in _plain:
        t = tensors_of(name, dirs)
        _plain[key] = (P.forward(ALL[name], t, tokens), P.router_gaps(ALL[name], t, tokens))
    return _plain[key]


def close(got, want_gaps, dtype) -> bool:
    """32-bit: every position whose routing does not hang on rounding, within the tolerance.  bfloat16: the plain
    implementation does not round, and the unit norms of queries, keys and the memory's read-outs amplify rounding
    where their input is small, so the positions are compared as a whole: half of them within a third of the
    tolerance, nine in ten within it.  What a single position must hold is tested in 32-bit, and in bfloat16 on
    each mechanism alone."""
    want, gaps = want_gaps
    got = got.double().cpu().numpy() if isinstance(got, torch.Tensor) else np.asarray(got)
    e = np.abs(got - want).max(-1) / np.abs(want).max()
    if dtype == "float32":
        return bool(np.all(e[gaps > 1e-5] < H.TOL_F32))
    e = e[gaps > 2e-2]
    if e.size < 8:
        return bool(e.size == 0 or e.max() < 3 * H.TOL_BF16)
    return bool(np.median(e) < H.TOL_BF16 / 3 and np.quantile(e, 0.9) < H.TOL_BF16)


def reqs_for(name, lengths, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, ALL[name]["vocab"], size=n).tolist() for n in lengths]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALL))
def test_model_whole_tail_portions_and_batches(name, dtype, dirs):
    from lastengine_b200 import Engine
    eng = Engine.from_pretrained(dirs[name], dtype=dtype, max_tokens=1024, max_seqs=6)
    reqs = reqs_for(name, [150, 3, 70, 1], 40)
    want = [plain(name, dirs, r) for r in reqs]
    for r, w in zip(reqs, want):
        assert close(H.run_whole(eng, r), w, dtype), f"whole, {len(r)} tokens"
    assert close(H.run_tail(eng, reqs[0], tail=90), want[0], dtype)          # decoding across a page border
    assert close(H.run_tail(eng, reqs[2], tail=69), want[2], dtype)          # from the first token on
    # a prompt in portions of several sizes, down to two tokens and one
    s = eng.new_sequence()
    outs, at = [], 0
    for n in (2, 1, 2, 59, 1, 64, 3, 18):
        outs.append(H.to_host(eng.step([s], [reqs[0][at:at + n]], [list(range(n))], check=True)))
        at += n
    eng.release(s)
    assert at == 150 and close(torch.cat(outs), want[0], dtype)
    # unequal requests in one batch (prompts of different lengths, then token by token, leaving one by one)
    got = H.run_batch(eng, reqs, [100, 1, 64, 1])
    for g, w, r in zip(got, want, reqs):
        assert close(g, w, dtype), f"batched, {len(r)} tokens"
    # the same again in the slots and pages that were just given back, in another order
    got = H.run_batch(eng, reqs[::-1], [1, 7, 2, 149])
    for g, w in zip(got, want[::-1]):
        assert close(g, w, dtype)
    assert eng.cache.slots.n_held == 0
    eng.cache.check()


@pytest.mark.parametrize("name", ["A", "C"])
def test_stream_after_every_layer_run(name, dirs):
    """The stream after the first 1, 2, ... layers, seen through the final norm and the head: models whose later
    layers are cut off (a looped range as far as the shorter model reaches) against the plain implementation."""
    import json
    from lastengine_b200 import Engine
    from lastengine_b200.weights.safetensors_io import SafetensorsFile, save_file
    cfg = ALL[name]
    toks = reqs_for(name, [40], 47)[0]
    src = dirs[name]
    sf = SafetensorsFile(os.path.join(src, "model.safetensors"))
    for n_layers in range(1, len(cfg["layers"])):
        cut = dict(cfg, layers=cfg["layers"][:n_layers])
        lp = cfg.get("loop")
        if lp:       # the looped range as far as the shorter model reaches
            cut.pop("loop")
            if lp["start"] < n_layers:
                cut["loop"] = dict(lp, stop=min(lp["stop"], n_layers))
        d = os.path.join(src, f"cut{n_layers}")
        os.makedirs(d, exist_ok=True)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cut, f)
        keep = {n: sf.tensor(n).clone() for n in sf.names()
                if not n.startswith("l") or int(n.split(".")[0][1:]) < n_layers}
        save_file(keep, os.path.join(d, "model.safetensors"))
        eng = Engine.from_pretrained(d, dtype="float32", max_tokens=256, max_seqs=2)
        w = P.read_safetensors(os.path.join(d, "model.safetensors"))
        want = (P.forward(cut, w, toks), P.router_gaps(cut, w, toks))
        assert close(H.run_whole(eng, toks), want, "float32"), f"after {n_layers} layers"


@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_logits_do_not_depend_on_the_cut_or_the_batch_beyond_rounding(name, dirs):
    from lastengine_b200 import Engine
    eng = Engine.from_pretrained(dirs[name], dtype="float32", max_tokens=1024, max_seqs=6)
    reqs = reqs_for(name, [140, 9], 41)
    gaps = plain(name, dirs, reqs[0])[1]
    keep = torch.from_numpy(gaps > 1e-5)
    whole = H.run_whole(eng, reqs[0])[keep]
    tail = H.run_tail(eng, reqs[0], tail=80)[keep]
    batched = H.run_batch(eng, reqs, [61, 4])[0][keep]
    assert H.rel_err(tail, whole) < 5e-6 and H.rel_err(batched, whole) < 5e-6


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("D", "float32"), ("B", "bfloat16"), ("C", "float32")])
def test_long_decoding_from_a_short_prompt(name, dtype, dirs):
    """Several windows pass while decoding; window pages are given back on the way; the states are carried."""
    from lastengine_b200 import Engine
    eng = Engine.from_pretrained(dirs[name], dtype=dtype, max_tokens=512, max_seqs=2)
    r = reqs_for(name, [330], 42)[0]
    got = H.run_tail(eng, r, tail=326)
    assert close(got, plain(name, dirs, r), dtype)
    eng.cache.check()


@pytest.mark.parametrize("seed", [201, 202, 203, 204, 205, 206, 207, 208])
def test_configurations_drawn_at_random(seed, tmp_path):
    """Layer order, sizes, windows, loops and feed-forwards drawn at random: whole prompts, a tail token by token and an
    unequal batch in 32-bit against the plain implementation, every position held; bfloat16 over the positions."""
    from lastengine_b200 import Engine
    from lastengine_b200.weights import write_model_dir
    rng = np.random.default_rng(seed)
    cfg = random_config(rng)
    d = write_model_dir(cfg, str(tmp_path / "m"), seed=seed, norm_init="random")
    w = P.read_safetensors(os.path.join(d, "model.safetensors"))
    reqs = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in (170, 40)]
    want = [(P.forward(cfg, w, r), P.router_gaps(cfg, w, r)) for r in reqs]
    eng = Engine.from_pretrained(d, dtype="float32", max_tokens=1024, max_seqs=4)
    for r, wv in zip(reqs, want):
        assert close(H.run_whole(eng, r), wv, "float32"), cfg
    assert close(H.run_tail(eng, reqs[0], tail=70), want[0], "float32"), cfg
    for g, wv in zip(H.run_batch(eng, reqs, [130, 9]), want):
        assert close(g, wv, "float32"), cfg
    eng.cache.check()
    eng16 = Engine.from_pretrained(d, dtype="bfloat16", max_tokens=1024, max_seqs=4)
    e = np.abs(H.run_whole(eng16, reqs[0]).double().numpy() - want[0][0]).max(-1) / np.abs(want[0][0]).max()
    e = e[want[0][1] > 2e-2]
    assert e.size == 0 or np.median(e) < H.TOL_BF16, cfg


def plain_greedy(name, dirs, prompt, n, gap=2e-2):
    """Greedy tokens of the plain implementation, and per token how far the choice is from falling the other way
    (0 where a routing decision of the position is closer than `gap`)."""
    toks, out, margins = list(prompt), [], []
    for _ in range(n):
        lg, gaps = plain(name, dirs, toks)
        row = lg[-1]
        top = np.sort(row)[-2:]
        margins.append(float((top[1] - top[0]) / np.abs(row).max()) if gaps[-1] > gap else 0.0)
        out.append(int(np.argmax(row)))
        toks.append(out[-1])
    return out, margins


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "bfloat16"), ("C", "float32"), ("D", "float32")])
def test_greedy_generation_through_the_entry_point(name, dtype, graphs, dirs):
    from lastengine_b200 import Engine, SamplingParams
    eng = Engine.from_pretrained(dirs[name], dtype=dtype, max_tokens=1024, use_graphs=graphs)
    prompts = reqs_for(name, [5, 1, 23, 66], 43)
    steps = 10
    res = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=steps, stop_token_ids=[])
    compared = 0
    for p, got in zip(prompts, res.tokens):
        want, margins = plain_greedy(name, dirs, p, steps, gap=1e-5 if dtype == "float32" else 2e-2)
        assert len(got) == steps
        for i in range(steps):
            if margins[i] < TOL[dtype]:
                break
            assert got[i] == want[i], f"{name} {dtype}: prompt of {len(p)}, token {i}"
            compared += 1
    # bfloat16 stops a request at its first close call (of the logits or of a routing decision), which comes early
    assert compared >= (steps * len(prompts) // 3 if dtype == "float32" else 1)
    assert eng.cache.slots.n_held == 0
    eng.cache.check()


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16")])
def test_a_sequence_written_out_and_read_back_goes_on_where_it_stood(name, dtype, dirs):
    """Keys, values, the recurrent unit's state, the matrix memory and its running maximum go out as bytes and come
    back into other slots and pages."""
    from lastengine_b200 import Engine
    eng = Engine.from_pretrained(dirs[name], dtype=dtype, max_tokens=512, max_seqs=4)
    r = reqs_for(name, [120], 44)[0]
    s = eng.new_sequence()
    eng.step([s], [r[:100]], None)
    data = eng.export_sequence(s)
    a = H.to_host(eng.step([s], [r[100:]], [list(range(20))]))
    other = eng.new_sequence()
    eng.step([other], [r[:5]], None)
    t = eng.import_sequence(data)
    assert t != s and eng.length(t) == 100
    b = H.to_host(eng.step([t], [r[100:]], [list(range(20))]))
    eng.release([s, other, t])
    assert H.rel_err(b, a) < 1e-6
    eng.cache.check()


def test_replay_program_with_a_cache_sized_to_the_tokens_alone(dirs, tmp_path):
    """bin/trace_run with --max-tokens equal to the tokens the live requests hold: three unequal requests start
    together (the shortest with one token), go on token by token and leave one by one."""
    import json
    import subprocess
    import sys
    name = "A"
    reqs = dict(zip("xyz", reqs_for(name, [12, 95, 3], 45)))
    first = {"x": 9, "y": 70, "z": 1}
    steps = [{"step": 0, "entries": [{"id": r, "tokens": reqs[r][:first[r]], "want": list(range(first[r]))} for r in "xyz"],
              "end": []}]
    fed, live, n = dict(first), ["x", "y", "z"], 1
    while live:
        ent = [{"id": r, "tokens": [reqs[r][fed[r]]], "want": [0]} for r in live]
        for r in live:
            fed[r] += 1
        ended = [r for r in live if fed[r] >= len(reqs[r])]
        steps.append({"step": n, "entries": ent, "end": ended})
        live = [r for r in live if r not in ended]
        n += 1
    out = str(tmp_path / "out")
    p = subprocess.run([sys.executable, os.path.join(H.ROOT, "bin", "trace_run"), "--model", dirs[name], "--dtype", "float32",
                        "--out", out, "--max-tokens", str(sum(len(t) for t in reqs.values()))],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(n)]
    V = ALL[name]["vocab"]
    got = {r: [] for r in reqs}
    for st in steps:
        lg = np.fromfile(os.path.join(out, f"{st['step']}.f32"), dtype="<f4").reshape(-1, V)
        at = 0
        for e in st["entries"]:
            got[e["id"]].append(lg[at:at + len(e["want"])])
            at += len(e["want"])
        assert at == lg.shape[0]
    for r, t in reqs.items():
        assert close(np.concatenate(got[r]), plain(name, dirs, t), "float32"), r


def test_command_line_generates_and_inspects(dirs):
    import json
    import subprocess
    import sys
    exe = os.path.join(H.ROOT, "bin", "lastengine")
    d = dirs["A"]
    base = [sys.executable, exe, "generate", "--model", d, "--prompt-ids", "1,2,3", "--prompt-ids", "9 8 7 6 5", "--max-new-tokens", "6",
            "--stop-token-id", "199"]
    p = subprocess.run(base + ["--dtype", "float32", "--temperature", "0"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-1500:]
    rows = [json.loads(l) for l in p.stdout.splitlines()]
    assert len(rows) == 2 and all(1 <= len(r["tokens"]) <= 6 for r in rows)
    want, margins = plain_greedy("A", dirs, [1, 2, 3], 1)
    if margins[0] > 1e-4:
        assert rows[0]["tokens"][0] == want[0]
    sampled = [subprocess.run(base + ["--temperature", "0.9", "--top-k", "20", "--seed", "5"], capture_output=True, text=True, timeout=600)
               for _ in range(2)]
    assert sampled[0].returncode == 0, sampled[0].stderr[-1500:]
    assert sampled[0].stdout == sampled[1].stdout
    p2 = subprocess.run([sys.executable, exe, "inspect", d], capture_output=True, text=True, timeout=600)
    assert p2.returncode == 0, p2.stderr[-1500:]
    assert "parallel_mixers" in p2.stdout and "mlstm" in p2.stdout
