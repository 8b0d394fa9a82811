"""The Kisilix decoder on the GPU against the plain implementation (tests/plain_kisilix.py): every mechanism
alone, then whole models: prompts whole, in portions and token by token, unequal batches, slots and pages
used again, windows and pooled blocks at their edges, long decoding, and greedy generation through the
entry point."""
import os

import numpy as np
import pytest
import torch

import harness as H
import plain_kisilix as P
from kisilix_configs import ALL, att, delta, dense, moe, ssm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": H.TOL_F32, "bfloat16": H.TOL_BF16}


def K():
    from lastengine_b200.ops import kernels
    return kernels


def bf16_round(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.asarray(a, dtype=np.float64)).to(torch.bfloat16).double().numpy()


def err(got, want) -> float:
    """max |got - want| / max |want|."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return float(np.abs(got - want).max() / np.abs(want).max())


# ---- a mixer alone: its own cache, steps laid out as the engine lays them out ----------------------
class MixerRig:
    def __init__(self, kind, params, dtype, seed=0, std=0.3, max_tokens=2048, max_seqs=6, edit=None):
        from lastengine_b200.cache import Cache
        from lastengine_b200.engine.batch import BatchBuilder
        from lastengine_b200.engine.workspace import Workspace
        from lastengine_b200.parts.base import BuildEnv
        from lastengine_b200.registry import MIXERS
        from lastengine_b200.weights.loader import kept_dtype
        from lastengine_b200.weights.random_init import random_tensor
        dev = torch.device(DEV)
        self.env = BuildEnv(device=dev, dtype=DT[dtype], workspace=Workspace(dev))
        self.mixer = MIXERS.get(kind)(**params)
        specs = self.mixer.tensors()
        self.plain = {}
        for name, spec in specs.items():
            t = random_tensor(name, spec, seed, std, norm_init="random").to(torch.bfloat16).double()
            self.plain[name] = t.numpy().copy()
        if edit:
            edit(self.plain)
            self.plain = {n: bf16_round(v) for n, v in self.plain.items()}
        self.mixer.load({n: torch.from_numpy(v).float().to(dev, kept_dtype(specs[n], torch.bfloat16, DT[dtype]))
                         for n, v in self.plain.items()}, self.env)
        self.cache = Cache({0: self.mixer.cache_spec()}, max_tokens=max_tokens, max_seqs=max_seqs, dtype=DT[dtype], device=dev)
        self.builder = BatchBuilder(dev)
        self.D = params["hidden_size"]

    def step(self, slots, hs):
        """hs: per sequence a [n, D] array of mixer inputs; returns the mixer's outputs per sequence."""
        from lastengine_b200.cache import pooled_table_key
        slots = list(slots)
        grow = {s: h.shape[0] for s, h in zip(slots, hs)}
        pos0 = [self.cache.length(s) for s in slots]
        self.cache.reserve(grow)
        tables = {}
        for gi, g in enumerate(self.cache.kv_groups):
            tables[gi] = g.table(slots, max(1, max(len(g.seq_pages.get(s, ())) for s in slots)))
            if g.pool > 0:
                tables[pooled_table_key(gi)] = g.table(
                    slots, max(1, max(len(g.seq_pooled_pages.get(s, ())) for s in slots)), pooled=True)
        batch = self.builder.build(slots, [[0] * h.shape[0] for h in hs], pos0, [], tables)
        h = torch.from_numpy(np.concatenate(hs, 0)).to(DEV, self.env.dtype)
        out = torch.zeros(h.shape[0], self.D, dtype=torch.float32, device=DEV)
        self.mixer.forward(h, out, False, batch, self.cache.view(0, True, batch.tables), self.env)
        K().check_device_status()
        self.cache.commit(grow)
        out = out.double().cpu().numpy()
        return np.split(out, np.cumsum([x.shape[0] for x in hs])[:-1])

    def alone(self, h):
        s = self.cache.alloc_seq()
        try:
            return self.step([s], [h])[0]
        finally:
            self.cache.free_seq(s)


def inputs(T, D, seed, bf16, scale=1.0):
    h = np.random.default_rng(seed).standard_normal((T, D)) * scale
    return bf16_round(h) if bf16 else h


def whole_portions_and_batches(rig, plain_fn, lengths, more_n, cuts, dtype, seed=10):
    """Each sequence alone and whole; then all together in the slots and pages just given back; then every
    one goes on in portions (rows cut at `cuts`) beside the others."""
    bf16 = dtype == "bfloat16"
    tol = TOL[dtype]
    hs = [inputs(n, rig.D, seed + n, bf16) for n in lengths]
    want = [plain_fn(h) for h in hs]
    for h, w in zip(hs, want):
        assert err(rig.alone(h), w) < tol, f"alone, {h.shape[0]} rows"
    more = [inputs(more_n, rig.D, seed + 50 + i, bf16) for i in range(len(hs))]
    want2 = [plain_fn(np.concatenate([h, x])) for h, x in zip(hs, more)]
    slots = [rig.cache.alloc_seq() for _ in hs]
    for g, w in zip(rig.step(slots, hs), want):
        assert err(g, w) < tol, "batched"
    outs = [[] for _ in hs]
    for a, b in zip(cuts[:-1], cuts[1:]):
        for i, g in enumerate(rig.step(slots, [x[a:b] for x in more])):
            outs[i].append(g)
    for i, w in enumerate(want2):
        assert err(np.concatenate(outs[i]), w[hs[i].shape[0]:]) < tol, f"sequence {i} after portions"
    for s in slots:
        rig.cache.free_seq(s)
    rig.cache.check()


# ---- the gated delta rule ---------------------------------------------------------------------------
def delta_params(D, heads, kv, dim, vdim, taps, eps=1e-5):
    return dict(hidden_size=D, num_heads=heads, num_kv_heads=kv, head_dim=dim, v_head_dim=vdim, conv_taps=taps,
                norm_eps=eps)


DELTA_CASES = [  # heads, kv heads, dim, vdim, taps
    (4, 2, 16, 24, 4),
    (3, 3, 64, 32, 2),
    (3, 1, 24, 40, 1),
    (2, 2, 128, 64, 5),
    (1, 1, 40, 8, 3),
    (2, 1, 256, 16, 2),
    (2, 1, 18, 10, 3),           # rows of a head that are no multiple of four numbers: the narrow copies
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv,dim,vdim,taps", DELTA_CASES)
def test_delta_rule_alone_whole_in_portions_and_batched(heads, kv, dim, vdim, taps, dtype):
    D = 48
    rig = MixerRig("gated_delta_rule", delta_params(D, heads, kv, dim, vdim, taps), dtype, seed=5)
    m = delta(heads, kv, dim, vdim, taps)
    whole_portions_and_batches(rig, lambda h: P.channel_delta(h, rig.plain, m, 1e-5), (150, 1, 37), 21,
                               [0, 2, 3, 8, 9, 21], dtype)


def test_delta_rule_keeps_a_write_from_far_back():
    """A head that hardly decays (A_log far below zero) reads at position 600 what position 2 wrote under the same
    key.  Queries and keys share their weights here, input channel 0 drives the values alone (another value at
    600 than at 2) and channel 1 the write strength alone: about a half at the two rows, nothing between them
    (every write also erases along its key, so hundreds of them would wipe a state of 16 rows).  The result at
    600 then mixes both values; a state lost, reset or decayed on the way leaves the second alone."""
    D, d, e = 32, 16, 16

    def edit(t):
        t["A_log"][:] = [-12.0, 1.0]
        t["k"][:] = t["q"]
        t["k.conv"][:] = t["q.conv"]
        for n in ("q", "k", "b", "a1", "g1"):
            t[n][:, 0] = 0.0
        for n in ("q", "k", "v", "a1", "g1"):
            t[n][:, 1] = 0.0
        t["b"][:, 1] = 20.0
    rig = MixerRig("gated_delta_rule", delta_params(D, 2, 2, d, e, 2, 1e-6), "float32", seed=8, edit=edit)
    m = delta(2, 2, d, e, 2)
    h = inputs(601, D, 3, False, 0.05)
    h[:, 0] = 0.0
    h[2] *= 40
    h[600], h[599] = h[2], h[1]          # the same key again (two taps: the row before it too)
    h[2, 0], h[600, 0] = 25.0, -25.0
    h[:, 1] = -1.0
    h[[2, 600], 1] = 0.0
    want = P.channel_delta(h, rig.plain, m, 1e-6)
    gone = P.channel_delta(h[3:], rig.plain, m, 1e-6)
    assert err(gone[-1:], want[-1:]) > 0.2             # the far write matters to the last row
    s = rig.cache.alloc_seq()
    a = rig.step([s], [h[:590]])[0]
    tail = np.concatenate([rig.step([s], [h[i:i + 1]])[0] for i in range(590, 601)])
    rig.cache.free_seq(s)
    assert err(np.concatenate([a, tail]), want) < H.TOL_F32
    assert err(tail[-1:], want[-1:]) < H.TOL_F32


# ---- the state-space layer --------------------------------------------------------------------------
def ssm_params(D, heads, vdim, state, groups, parts, taps, eps=1e-5):
    return dict(hidden_size=D, num_heads=heads, v_head_dim=vdim, state_size=state, num_groups=groups,
                norm_groups=parts, conv_taps=taps, norm_eps=eps)


SSM_CASES = [  # heads, vdim, state, groups, norm parts, taps
    (4, 16, 24, 2, 2, 3),
    (3, 64, 64, 1, 3, 2),
    (5, 8, 40, 5, 1, 5),
    (2, 48, 16, 1, 4, 4),
    (4, 32, 256, 2, 1, 4),
    (6, 24, 128, 3, 6, 1),
    (3, 6, 10, 1, 1, 2),         # B and C start off a 16-byte boundary in the convolved row
    (6, 64, 32, 2, 1, 4),        # one norm group of 384 numbers: a whole block takes it
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,vdim,state,groups,parts,taps", SSM_CASES)
def test_state_space_alone_whole_in_portions_and_batched(heads, vdim, state, groups, parts, taps, dtype):
    D = 40
    rig = MixerRig("state_space", ssm_params(D, heads, vdim, state, groups, parts, taps), dtype, seed=6)
    m = ssm(heads, vdim, state, groups, parts, taps)
    whole_portions_and_batches(rig, lambda h: P.mamba2(h, rig.plain, m, 1e-5), (131, 2, 64), 12,
                               [0, 1, 3, 4, 10, 12], dtype)


def test_state_space_keeps_an_input_from_far_back():
    """A head whose state hardly decays carries position 1's input to position 500; the skip term and the
    fast head alone would not."""
    D = 24

    def edit(t):
        t["A_log"][:] = [-14.0, 2.0]
        t["dt_bias"][:] = [0.5, 0.5]
        t["D"][:] = [0.1, 0.1]
    rig = MixerRig("state_space", ssm_params(D, 2, 16, 16, 1, 1, 3, 1e-6), "float32", seed=9, edit=edit)
    m = ssm(2, 16, 16, 1, 1, 3)
    h = inputs(501, D, 4, False, 0.02)
    h[1] *= 60
    want = P.mamba2(h, rig.plain, m, 1e-6)
    gone = P.mamba2(h[4:], rig.plain, m, 1e-6)
    assert err(gone[-1:], want[-1:]) > 0.05
    s = rig.cache.alloc_seq()
    a = rig.step([s], [h[:470]])[0]
    tail = np.concatenate([rig.step([s], [h[i:i + 1]])[0] for i in range(470, 501)])
    rig.cache.free_seq(s)
    assert err(np.concatenate([a, tail]), want) < H.TOL_F32


@pytest.mark.parametrize("kind", ["gated_delta_rule", "state_space"])
def test_a_freed_slot_starts_from_zero_state_and_zero_convolution_memory(kind):
    """The same rows in a slot that another sequence just left give the same result as in a fresh one."""
    D = 32
    if kind == "gated_delta_rule":
        rig = MixerRig(kind, delta_params(D, 2, 1, 32, 16, 4), "float32", seed=3, max_seqs=1)
        fn = lambda h: P.channel_delta(h, rig.plain, delta(2, 1, 32, 16, 4), 1e-5)
    else:
        rig = MixerRig(kind, ssm_params(D, 2, 16, 32, 1, 2, 4), "float32", seed=3, max_seqs=1)
        fn = lambda h: P.mamba2(h, rig.plain, ssm(2, 16, 32, 1, 2, 4), 1e-5)
    a, b = inputs(40, D, 1, False, 3.0), inputs(5, D, 2, False)
    rig.alone(a)
    assert err(rig.alone(b), fn(b)) < H.TOL_F32


# ---- windowed attention with pooled blocks ------------------------------------------------------------
def att_params(D, heads, kv, dim, vdim, scale, rot, base, size, pool, eps=1e-5):
    from lastengine_b200.parts.base import PartSpec
    return dict(hidden_size=D, num_heads=heads, num_kv_heads=kv, head_dim=dim, v_head_dim=vdim, norm_eps=eps,
                scale=scale, window=size, pool=pool, value_rotation_base=base,
                position=PartSpec("rope", {"rope_dim": rot, "theta": base, "style": "neox"}) if rot else PartSpec("none"))


ATT_CASES = [  # heads, kv heads, dim, vdim, scale, rot dims, base, window, block
    (4, 2, 32, 16, 0.2, 16, 1e4, 20, 6),
    (2, 1, 16, 48, 0.3, 16, 1e3, 33, 5),
    (3, 3, 64, 64, 0.125, 64, 2e5, 70, 72),       # a block larger than the window and than a cache page
    (4, 1, 128, 128, 0.09, 32, 1e6, 9, 1),         # blocks of one position: every earlier position is seen
    (5, 5, 24, 40, 0.25, 0, 1e4, 1, 4),            # a window of the position itself, no rotation of q and k
    (2, 2, 96, 32, 0.1, 48, 2e4, 64, 64),          # window and block of a cache page
    (6, 2, 64, 32, 0.15, 64, 5e4, 128, 64),
    (2, 2, 256, 256, 0.06, 128, 1e4, 40, 8),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv,dim,vdim,scale,rot,base,size,pool", ATT_CASES)
def test_attention_alone_whole_in_portions_and_batched(heads, kv, dim, vdim, scale, rot, base, size, pool, dtype):
    D = 48
    rig = MixerRig("pooled_window_attention", att_params(D, heads, kv, dim, vdim, scale, rot, base, size, pool), dtype, seed=7)
    m = att(heads, kv, dim, vdim, scale, rot, base, size, pool)
    # over two page borders, a single row, a row count below most windows; then 30 more rows in portions
    whole_portions_and_batches(rig, lambda h: P.pooled_window_attention(h, rig.plain, m, 1e-5), (150, 1, 37), 30,
                               [0, 1, 3, 4, 10, 12, 30], dtype)


ATT_TENSOR_CORE_CASES = [  # sizes the tensor-core prompt kernel takes: key heads of 64, 1/2/4/8 query heads per kv head
    # heads, kv heads, vdim, scale, rot dims, base, window, block
    (8, 2, 64, 0.13, 64, 1e4, 96, 4),        # 151 pooled blocks at the end of 700 rows: three pages of them
    (8, 1, 64, 0.1, 32, 5e5, 64, 64),        # window and block of a cache page
    (4, 2, 64, 0.2, 64, 1e3, 200, 7),        # a block that divides neither the window nor a page
    (3, 3, 64, 0.125, 0, 2e4, 33, 1),        # blocks of one position: every earlier position is seen, 667 pooled rows
    (4, 1, 32, 0.15, 64, 1e4, 130, 5),       # value heads half as wide as the key heads
    (2, 2, 32, 0.11, 16, 3e4, 64, 16),
]


@pytest.mark.parametrize("heads,kv,vdim,scale,rot,base,size,pool", ATT_TENSOR_CORE_CASES)
def test_attention_on_the_tensor_cores_whole_in_portions_and_batched(heads, kv, vdim, scale, rot, base, size, pool):
    D = 64
    rig = MixerRig("pooled_window_attention", att_params(D, heads, kv, 64, vdim, scale, rot, base, size, pool), "bfloat16",
                   seed=11, max_tokens=4096)
    m = att(heads, kv, 64, vdim, scale, rot, base, size, pool)
    whole_portions_and_batches(rig, lambda h: P.pooled_window_attention(h, rig.plain, m, 1e-5), (700, 9, 130), 40,
                               [0, 8, 9, 17, 40], "bfloat16")


def flagged(D, heads, kv, dim, c, strength=30.0):
    """Weights in which input channel 0 alone drives number `c` of every query head and input channel 1 that of
    every key head, so strongly that after the head's norm a flagged query meets a flagged key with a score far
    above all others."""
    def edit(t):
        for name, n, col in (("q", heads, 0), ("k", kv, 1)):
            for h in range(n):
                t[name][h * dim + c, :] = 0.0
                t[name][h * dim + c, col] = strength
            t[name][:, col] *= (np.arange(t[name].shape[0]) % dim == c)      # the flag channel drives nothing else
            t[name + ".b"][:] *= 0.1
        t["q.norm"][c] = t["k.norm"][c] = 1.0
        t["temp"][:] = 1.0
    return edit


EDGE_CASES = [  # window, block, position of the flagged key
    (20, 6, 3), (33, 5, 62), (9, 1, 60), (64, 64, 1), (70, 72, 5), (1, 4, 66), (12, 8, 0), (17, 4, 127),
]


@pytest.mark.parametrize("size,pool,at", EDGE_CASES)
def test_a_key_passes_the_window_s_edge_waits_unseen_and_comes_back_in_its_block(size, pool, at):
    """Every query after position `at` asks for the key at `at` (a score that stands out).  It is seen while
    0 <= i - at < window, by nobody until its block is wholly behind the window, and from then on as a
    `pool`-th of the block's mean.  Whole, token by token from before the first edge, and in portions."""
    D, heads, kv, dim, vdim, rot = 24, 2, 1, 32, 16, 16
    p = att_params(D, heads, kv, dim, vdim, 1.0, rot, 1e4, size, pool, 1e-6)
    rig = MixerRig("pooled_window_attention", p, "float32", seed=11, edit=flagged(D, heads, kv, dim, 20))
    T = at + size + 2 * pool + 6
    h = inputs(T, D, 5, False)
    h[:, 0] = (np.arange(T) >= at) * 1.0
    h[:, 1] = (np.arange(T) == at) * 1.0
    m = att(heads, kv, dim, vdim, 1.0, rot, 1e4, size, pool)
    want = P.pooled_window_attention(h, rig.plain, m, 1e-6)
    # the plain implementation itself: without the flag on that key, the result changes where the key is seen
    # (much inside the window, by the block's share behind it) and nowhere between
    first_out = at + size
    block_end = (at // pool) * pool + pool - 1
    first_pooled = max(block_end + size, first_out)
    unflagged = h.copy()
    unflagged[at, 1] = 0.0
    other = P.pooled_window_attention(unflagged, rig.plain, m, 1e-6)
    diff = np.abs(other - want).max(-1) / np.abs(want).max()
    assert diff[first_out - 1] > 0.2
    assert np.all(diff[first_out:first_pooled] == 0.0)
    assert diff[first_pooled] > 0.02 / pool
    assert err(rig.alone(h), want) < H.TOL_F32
    start = max(1, at - 1)
    s = rig.cache.alloc_seq()
    got = [rig.step([s], [h[:start]])[0]] + [rig.step([s], [h[i:i + 1]])[0] for i in range(start, T)]
    rig.cache.free_seq(s)
    got = np.concatenate(got)
    bad = np.nonzero(np.abs(got - want).max(-1) / np.abs(want).max() > H.TOL_F32)[0]
    assert bad.size == 0, f"token by token: first wrong position {bad[0]} (edge {first_out}, pooled from {first_pooled})"
    s = rig.cache.alloc_seq()
    cuts = [0, 2, max(3, first_out - 1), first_out + 1, min(T - 1, first_pooled), T]
    cuts = sorted(set(c for c in cuts if 0 <= c <= T))
    got = np.concatenate([rig.step([s], [h[a:b]])[0] for a, b in zip(cuts[:-1], cuts[1:])])
    rig.cache.free_seq(s)
    assert err(got, want) < H.TOL_F32, f"portions cut at {cuts}"
    rig.cache.check()


def test_a_far_block_among_hundreds_is_found_while_decoding():
    """The flagged key sits in block 1 of 150; the query 600 positions later still finds it in the block's mean
    (the only flagged key: its score, a quarter of a lone key's, stands above the other blocks')."""
    D, heads, kv, dim, vdim, rot, size, pool = 24, 2, 2, 32, 32, 16, 16, 4
    p = att_params(D, heads, kv, dim, vdim, 2.0, rot, 1e4, size, pool, 1e-6)
    rig = MixerRig("pooled_window_attention", p, "float32", seed=12, edit=flagged(D, heads, kv, dim, 24))
    T, at = 606, 5
    h = inputs(T, D, 6, False, 0.3)
    h[:, 0] = (np.arange(T) >= 600) * 1.0
    h[:, 1] = (np.arange(T) == at) * 1.0
    m = att(heads, kv, dim, vdim, 2.0, rot, 1e4, size, pool)
    want = P.pooled_window_attention(h, rig.plain, m, 1e-6)
    other = h.copy()
    other[at, 1] = 0.0
    assert err(P.pooled_window_attention(other, rig.plain, m, 1e-6)[600:], want[600:]) > 0.1
    s = rig.cache.alloc_seq()
    got = [rig.step([s], [h[:590]])[0]] + [rig.step([s], [h[i:i + 1]])[0] for i in range(590, T)]
    rig.cache.free_seq(s)
    assert err(np.concatenate(got), want) < H.TOL_F32


# ---- feed-forwards, the layer's sums and norms, the embedding -----------------------------------------
class PartRig:
    """A feed-forward alone with random weights (rounded to bfloat16, kept as doubles by their short names)."""

    def __init__(self, part, dtype, seed, std=0.3, edit=None):
        from lastengine_b200.engine.batch import BatchBuilder
        from lastengine_b200.engine.workspace import Workspace
        from lastengine_b200.parts.base import BuildEnv
        from lastengine_b200.weights.loader import kept_dtype
        from lastengine_b200.weights.random_init import random_tensor
        dev = torch.device(DEV)
        self.env = BuildEnv(device=dev, dtype=DT[dtype], workspace=Workspace(dev))
        self.part = part
        specs = part.tensors()
        self.plain = {n: random_tensor(n, sp, seed, std, norm_init="random").to(torch.bfloat16).double().numpy().copy()
                      for n, sp in specs.items()}
        if edit:
            edit(self.plain)
            self.plain = {n: bf16_round(v) for n, v in self.plain.items()}
        part.load({n: torch.from_numpy(v).float().to(dev, kept_dtype(specs[n], torch.bfloat16, DT[dtype]))
                   for n, v in self.plain.items()}, self.env)
        self.builder = BatchBuilder(dev)

    def run(self, h):
        batch = self.builder.build([0], [[0] * h.shape[0]], [0], [], {})
        out = torch.zeros(h.shape[0], h.shape[1], dtype=torch.float32, device=DEV)
        self.part.forward(torch.from_numpy(h).to(DEV, self.env.dtype), out, False, batch, self.env)
        K().check_device_status()
        return out.double().cpu().numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D,F,limit", [(48, 96, 1.5), (72, 48, 7.0), (40, 56, 0.5), (64, 320, 2.5)])
def test_clamped_dense_feed_forward(D, F, limit, dtype):
    """Inputs large enough that the gate meets its upper limit and the other half both of its limits."""
    from lastengine_b200.registry import FEED_FORWARDS
    part = FEED_FORWARDS.get("gated_dense")(hidden_size=D, intermediate_size=F, activation="clamped_sigmoid", limit=limit,
                                             alpha=1.702, names=("gate", "up", "down"))
    rig = PartRig(part, dtype, seed=21)
    h = inputs(70, D, 1, dtype == "bfloat16", 1.5)
    f = dense(F, limit)
    g, u = h @ rig.plain["gate"].T, h @ rig.plain["up"].T
    assert (g > limit).mean() > 0.02 and (u > limit).mean() > 0.02 and (u < -limit).mean() > 0.02 and (g < -limit).any()
    assert err(rig.run(h), P.clamped_dense(h, rig.plain, f)) < TOL[dtype]


MOE_CASES = [  # experts, top, groups, kept, expert width, shared width
    (8, 2, 4, 2, 32, 48), (6, 3, 1, 1, 24, 16), (12, 1, 3, 1, 16, 40), (4, 4, 2, 2, 40, 8), (9, 2, 3, 2, 16, 24),
    (5, 5, 1, 1, 8, 32), (16, 4, 4, 1, 24, 56), (10, 3, 5, 3, 16, 16), (32, 6, 8, 3, 16, 64),
]


def moe_part(D, E, top, count, keep, F, Fs):
    from lastengine_b200.registry import FEED_FORWARDS
    return FEED_FORWARDS.get("topk_moe")(
        hidden_size=D, num_experts=E, top_k=top, expert_size=F, router="softmax_grouped", groups=(count, keep),
        use_bias=True, activation="silu", shared_size=Fs,
        names={"router": "router", "bias": "correction", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down"})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,count,keep,F,Fs", MOE_CASES)
def test_grouped_experts_with_a_correction_that_only_chooses(E, top, count, keep, F, Fs, dtype):
    """The correction is made as large as the scores differ, and partly negative, so that it changes the
    choice; rows whose choice hangs on rounding are left out in bfloat16."""
    D = 48

    def edit(t):
        t["router"] *= 3.0
        t["correction"][:] = np.random.default_rng(E).uniform(-0.6, 0.3, E) / E
    rig = PartRig(moe_part(D, E, top, count, keep, F, Fs), dtype, seed=22, edit=edit)
    bf16 = dtype == "bfloat16"
    h = inputs(90, D, 2, bf16)
    f = moe(E, top, count, keep, F, Fs)
    ids, _, gap = P.route(h, rig.plain, f)
    plain_ids, _, _ = P.route(h, {**rig.plain, "correction": np.zeros(E)}, f)
    if top < E:
        assert (np.sort(ids, -1) != np.sort(plain_ids, -1)).any()           # the correction does change choices
    want = P.expert_mixture(h, rig.plain, f)
    got = rig.run(h)
    keep_rows = gap > (2e-3 if bf16 else 1e-6) / max(1.0, E / 8)      # scores shrink as 1/E
    assert keep_rows.mean() > 0.5
    assert err(got[keep_rows], want[keep_rows]) < TOL[dtype]


def test_an_excluded_group_loses_to_a_negative_choice_score():
    """Two groups, one kept: every choice score of the kept group but one is negative; the excluded group's
    scores are positive.  Experts of the excluded group must not be chosen (minus infinity, not zero)."""
    D, E = 32, 8

    def edit(t):
        t["router"][:] = 0.0                      # equal scores 1/8 ...
        t["correction"][:] = [0.5, -1.0, -1.0, -1.0, 0.2, 0.2, 0.2, 0.2]       # ... so the correction alone chooses
    rig = PartRig(moe_part(D, E, 3, 2, 1, 16, 8), "float32", seed=23, edit=edit)
    h = inputs(20, D, 3, False)
    f = moe(E, 3, 2, 1, 16, 8)
    ids, wts, _ = P.route(h, rig.plain, f)
    assert all(set(r) <= {0, 1, 2, 3} for r in ids) and np.allclose(wts, 1 / 3)
    assert err(rig.run(h), P.expert_mixture(h, rig.plain, f)) < H.TOL_F32


@pytest.mark.parametrize("D", [40, 42, 64, 256, 1000, 2048])
@pytest.mark.parametrize("alpha", [1.0, 2.5])
def test_sum_and_layer_norm_with_bias(D, alpha):
    rng = np.random.default_rng(D)
    x, y = rng.standard_normal((33, D)) * 2 + 0.7, rng.standard_normal((33, D))
    w, b = 1 + 0.1 * rng.standard_normal(D), 0.3 * rng.standard_normal(D)
    t = lambda a: torch.from_numpy(a).float().to(DEV)
    xd, h = t(x), torch.zeros(33, D, dtype=torch.bfloat16, device=DEV)
    K().postnorm_residual(xd, t(y), alpha, t(w), t(b), 1e-5, h=h)
    want = P.layer_norm(alpha * t(x).double().cpu().numpy() + t(y).double().cpu().numpy(), t(w).double().cpu().numpy(),
                        t(b).double().cpu().numpy(), 1e-5)
    assert err(xd.double().cpu().numpy(), want) < 1e-5
    assert torch.equal(h, xd.to(torch.bfloat16))            # the stream once more, in the activation type


def test_embedding_adds_the_position_s_own_vector():
    from lastengine_b200.engine.batch import BatchBuilder
    from lastengine_b200.registry import EMBEDDINGS
    from lastengine_b200.parts.base import BuildEnv
    emb = EMBEDDINGS.get("token_position_embedding")(vocab_size=50, hidden_size=24, max_positions=90, position_tensor="pos")
    rng = np.random.default_rng(0)
    table, pos = bf16_round(rng.standard_normal((50, 24))), bf16_round(rng.standard_normal((90, 24)))
    env = BuildEnv(device=torch.device(DEV), dtype=torch.float32)
    names = list(emb.tensors())
    emb.load({names[0]: torch.from_numpy(table).float().to(DEV), "positions": torch.from_numpy(pos).float().to(DEV)}, env)
    toks = [[3, 4, 5, 6], [7], [8, 9]]
    batch = BatchBuilder(torch.device(DEV)).build([0, 1, 2], toks, [0, 88, 40], [], {})     # positions 0.., 88, 40..
    x = torch.zeros(7, 24, dtype=torch.float32, device=DEV)
    emb.forward(x, batch.tokens, batch=batch)
    want = table[[3, 4, 5, 6, 7, 8, 9]] + pos[[0, 1, 2, 3, 88, 40, 41]]
    assert err(x.double().cpu().numpy(), want) < 1e-6


# ---- whole models --------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    from lastengine_b200.weights import write_model_dir
    return {n: write_model_dir(cfg, str(tmp_path_factory.mktemp("k" + n)), seed=31 + i, norm_init="random")
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
    """32-bit: every position whose routing does not hang on rounding, within the tolerance.  bfloat16: the
    plain implementation does not round, and the norm after every sum, the unit norms of queries and keys and
    the root mean squares of the recurrent read-outs amplify rounding where their input is small; so the
    positions are compared as a whole: half of them within a third of the tolerance, nine in ten within it.
    What a single position must hold is tested in 32-bit, and in bfloat16 on each mechanism alone."""
    want, gaps = want_gaps
    got = got.double().cpu().numpy() if isinstance(got, torch.Tensor) else np.asarray(got)
    e = np.abs(got - want).max(-1) / np.abs(want).max()
    if dtype == "float32":
        return bool(np.all(e[gaps > 1e-5] < H.TOL_F32))
    e = e[gaps > 2e-3]
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


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("D", "float32"), ("B", "bfloat16")])
def test_long_decoding_from_a_short_prompt(name, dtype, dirs):
    """Several windows and many blocks pass while decoding; window pages are given back on the way."""
    from lastengine_b200 import Engine
    eng = Engine.from_pretrained(dirs[name], dtype=dtype, max_tokens=512, max_seqs=2)
    r = reqs_for(name, [330], 42)[0]
    got = H.run_tail(eng, r, tail=326)
    assert close(got, plain(name, dirs, r), dtype)
    eng.cache.check()


def test_a_sequence_may_fill_the_position_table_and_not_go_beyond(dirs):
    from lastengine_b200 import Engine
    from lastengine_b200.engine.engine import StepError
    eng = Engine.from_pretrained(dirs["C"], dtype="float32", max_tokens=1024, max_seqs=2)
    r = reqs_for("C", [400], 46)[0]
    s = eng.new_sequence()
    got = [H.to_host(eng.step([s], [r[:398]], [list(range(398))])), H.to_host(eng.step([s], [r[398:]], [[0, 1]]))]
    assert close(torch.cat(got), plain("C", dirs, r), "float32")
    with pytest.raises(StepError, match="positions"):
        eng.step([s], [[1]], [[0]])
    eng.release(s)


def plain_greedy(name, dirs, prompt, n):
    toks, out, margins = list(prompt), [], []
    for _ in range(n):
        lg, gaps = plain(name, dirs, toks)
        row = lg[-1]
        top = np.sort(row)[-2:]
        margins.append(float((top[1] - top[0]) / np.abs(row).max()) if gaps[-1] > 2e-3 else 0.0)
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
        want, margins = plain_greedy(name, dirs, p, steps)
        assert len(got) == steps
        for i in range(steps):
            if margins[i] < TOL[dtype]:
                break
            assert got[i] == want[i], f"{name} {dtype}: prompt of {len(p)}, token {i}"
            compared += 1
    # bfloat16 stops a request at its first close call, which comes early in a vocabulary of random logits
    assert compared >= (steps * len(prompts) // 3 if dtype == "float32" else len(prompts))
    assert eng.cache.slots.n_held == 0
    eng.cache.check()


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16")])
def test_a_sequence_written_out_and_read_back_goes_on_where_it_stood(name, dtype, dirs):
    """Keys, values, pooled rows, the convolutions' memory and the recurrent states go out as bytes and come back
    into other slots and pages."""
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


def test_command_line_generates_samples_and_compares_the_two_number_formats(dirs):
    """bin/lastengine on a folder of this design: greedy and sampled generation (the same seed gives the same
    tokens), the dump of a greedy run, and bfloat16 against the 32-bit path step by step."""
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
    p2 = subprocess.run([sys.executable, exe, "tf-dump", d, "1,2,3", "6", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert p2.returncode == 0, p2.stderr[-1500:]
    dump = json.loads(p2.stdout.splitlines()[-1])
    if len(rows[0]["tokens"]) == 6:
        assert dump["gen_ids"] == rows[0]["tokens"]
    p3 = subprocess.run([sys.executable, exe, "dense-cmp", d, "1,2,3", "6"], capture_output=True, text=True, timeout=600)
    assert p3.returncode == 0, p3.stderr[-1500:]
    assert "/6 argmax agree, mean |dlogprob|" in p3.stdout.splitlines()[-1]
