"""Helpers shared by the tests: tiny model folders, request sets, replay through the engine,
and the error measure."""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)

import plain_lfm3 as P  # noqa: E402

# tolerances: max |engine - plain| over max |plain|, per request.  Fixed; never widened to pass.
TOL_F32 = 2e-5
TOL_BF16 = 1.5e-2


def make_model_dir(cfg: dict, seed: int, path: str, router_scale: float = 1.0, freq_factors: bool = False,
                   expert_bias_scale: float = 1.0) -> str:
    """Random model folder; norm weights random around 1 (all-ones would hide a swapped norm);
    router rows scaled so that the experts' scores are well apart (a near-tie would make the
    choice of expert, not the arithmetic, decide the comparison), the experts' selection biases
    scaled to the same end; convolution biases (written as
    zeros) made random; with `freq_factors` the model's optional rotary factors are added."""
    from lastengine_b200.weights import write_model_dir
    from lastengine_b200.weights.safetensors_io import SafetensorsFile, save_file
    write_model_dir(cfg, path, seed=seed, dtype="bfloat16", norm_init="random")
    if router_scale != 1.0 or expert_bias_scale != 1.0 or freq_factors or cfg.get("conv_bias", False):
        f = os.path.join(path, "model.safetensors")
        sf = SafetensorsFile(f)
        t = {n: sf.tensor(n).clone() for n in sf.names()}
        g = torch.Generator().manual_seed(1000 + seed)
        for n in sorted(t):
            if n.endswith("feed_forward.gate.weight"):
                t[n] = (t[n].float() * router_scale).to(t[n].dtype)
            if n.endswith("feed_forward.expert_bias"):
                t[n] = t[n] * expert_bias_scale
            if n.endswith("conv.conv.bias"):
                t[n] = (0.004 * torch.randn(t[n].shape, generator=g)).to(t[n].dtype)
        if freq_factors:
            hd = cfg.get("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
            half = cfg.get("rope_dim", hd) // 2
            t["model.rope_freqs.weight"] = 1.0 + 7.0 * torch.rand(half, generator=g)      # 32-bit, as a norm weight would be
        del sf
        save_file(t, f)
    return path


def requests_for(cfg: dict, lengths, seed: int) -> list[list[int]]:
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in lengths]


_tensors_on: dict = {}


def plain_tensors(model_dir: str, device: str = "cpu") -> dict:
    """The folder's tensors in double precision as the plain implementation reads them, kept per
    (folder, device).  `device` other than the CPU only moves the same arithmetic to where a model
    of real layer sizes takes seconds instead of minutes."""
    key = (model_dir, device)
    if key not in _tensors_on:
        t = P.read_safetensors(os.path.join(model_dir, "model.safetensors"), torch.float64)
        _tensors_on[key] = t if device == "cpu" else {k: v.to(device) for k, v in t.items()}
    return _tensors_on[key]


def plain_logits(cfg: dict, model_dir: str, tokens, bf16: bool, device: str | None = None) -> torch.Tensor:
    t = plain_tensors(model_dir, device) if device else \
        P.read_safetensors(os.path.join(model_dir, "model.safetensors"), torch.float64)
    return P.forward(cfg, t, tokens, rnd=P.round_bf16 if bf16 else P.identity)


# A router near-tie is a discontinuity: when the chosen and the first rejected expert score
# closer than bfloat16 rounding moves them, rounding decides which expert runs, and the logits
# of that position jump.  Such positions (found by the plain implementation alone) are left
# out of bfloat16 comparisons; in 32-bit every position is compared.
ROUTER_GAP_BF16 = 1e-3
ROUTER_GAP_F32 = 1e-5


def router_gap(bf16: bool, hidden_size: int = 96) -> float:
    """The gap below which a routing decision counts as a near-tie.  A router score is a sum over
    the hidden size of terms that each carry bfloat16 rounding noise, so its noise grows with the
    root of the width: the gap set at a width of 96 is scaled accordingly for wider models."""
    if not bf16:
        return ROUTER_GAP_F32
    return ROUTER_GAP_BF16 * max(1.0, (hidden_size / 96) ** 0.5)


def plain_logits_and_margins(cfg: dict, model_dir: str, tokens, bf16: bool, device: str | None = None):
    """Plain logits [T, V] and, per position, the smallest gap between the last chosen and the
    first rejected expert score over the model's routed layers (inf without experts)."""
    margins = []
    orig = P.moe_route

    def spy(h, wr, bias, k, norm_topk, scaling):
        ids, w, c = orig(h, wr, bias, k, norm_topk, scaling)
        cs = torch.sort(c, dim=-1, descending=True).values
        margins.append(cs[:, k - 1] - cs[:, k] if cs.shape[1] > k
                       else torch.full((cs.shape[0],), float("inf"), dtype=cs.dtype, device=cs.device))
        return ids, w, c
    P.moe_route = spy
    try:
        lg = plain_logits(cfg, model_dir, tokens, bf16, device)
    finally:
        P.moe_route = orig
    m = torch.stack(margins).amin(0) if margins else \
        torch.full((len(tokens),), float("inf"), dtype=torch.float64, device=lg.device)
    return lg, m


def decided(margins: torch.Tensor, bf16: bool, hidden_size: int = 96) -> torch.Tensor:
    """Positions whose routing does not hang on rounding."""
    return margins > router_gap(bf16, hidden_size)


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """max |got - want| / max |want|, computed where `want` lives."""
    got, want = got.to(want.device).double(), want.double()
    return float((got - want).abs().max() / want.abs().max())


def first_bad_position(got: torch.Tensor, want: torch.Tensor, tol: float) -> int | None:
    got, want = got.to(want.device).double(), want.double()
    e = (got - want).abs().amax(dim=-1) / want.abs().max()
    bad = torch.nonzero(e > tol)
    return int(bad[0]) if bad.numel() else None


# ---- replay through the engine -----------------------------------------------------------------
def to_host(t: torch.Tensor) -> torch.Tensor:
    return t.float().cpu().clone()


def on_device(t: torch.Tensor) -> torch.Tensor:
    """Keeps a step's logits where they are (large vocabularies); the step's buffer is reused."""
    return t.float().clone()


def run_whole(eng, tokens, keep=to_host) -> torch.Tensor:
    s = eng.new_sequence()
    try:
        return keep(eng.step([s], [tokens], [list(range(len(tokens)))]))
    finally:
        eng.release(s)


def run_tail(eng, tokens, tail: int = 32, keep=to_host) -> torch.Tensor:
    """The prompt whole, then the last `tail` tokens one by one."""
    n = len(tokens)
    head = max(1, n - tail)
    s = eng.new_sequence()
    try:
        out = [keep(eng.step([s], [tokens[:head]], [list(range(head))]))]
        for i in range(head, n):
            out.append(keep(eng.step([s], [[tokens[i]]], [[0]])))
        return torch.cat(out, dim=0)
    finally:
        eng.release(s)


def run_batch(eng, requests, prompt_lens, keep=to_host) -> list[torch.Tensor]:
    """All requests start together with prompts of unequal lengths, then one token each per
    step; a request leaves when its tokens are used up.  Returns logits [len, vocab] per request."""
    seqs = [eng.new_sequence() for _ in requests]
    got = [[] for _ in requests]
    live = list(range(len(requests)))
    try:
        lg = keep(eng.step([seqs[i] for i in live], [requests[i][:prompt_lens[i]] for i in live],
                           [list(range(prompt_lens[i])) for i in live]))
        r0 = 0
        for i in live:
            got[i].append(lg[r0:r0 + prompt_lens[i]])
            r0 += prompt_lens[i]
        fed = list(prompt_lens)
        while True:
            done = [i for i in live if fed[i] >= len(requests[i])]
            for i in done:
                eng.release(seqs[i])
                seqs[i] = None
            live = [i for i in live if i not in done]
            if not live:
                break
            lg = keep(eng.step([seqs[i] for i in live], [[requests[i][fed[i]]] for i in live],
                               [[0] for _ in live]))
            for j, i in enumerate(live):
                got[i].append(lg[j:j + 1])
                fed[i] += 1
        return [torch.cat(g, dim=0) for g in got]
    finally:
        for s in seqs:
            if s is not None:
                eng.release(s)


# ---- a part alone on the GPU: its own cache, steps laid out as the engine lays them out -------------------
def bf16_round_np(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.asarray(a, dtype=np.float64)).to(torch.bfloat16).double().numpy()


def max_err(got, want) -> float:
    """max |got - want| / max |want|."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return float(np.abs(got - want).max() / np.abs(want).max())


def random_rows(T: int, D: int, seed: int, bf16: bool, scale: float = 1.0) -> np.ndarray:
    h = np.random.default_rng(seed).standard_normal((T, D)) * scale
    return bf16_round_np(h) if bf16 else h


class MixerRig:
    """A mixer of the registry with random weights (kept in double precision in `plain`, by the part's tensor
    names) and a cache of its own."""

    def __init__(self, kind, params, dtype: str, seed=0, std=0.3, max_tokens=2048, max_seqs=6, edit=None, device="cuda:0",
                 hidden_size=None):
        from lastengine_b200.cache import Cache
        from lastengine_b200.engine.batch import BatchBuilder
        from lastengine_b200.engine.workspace import Workspace
        from lastengine_b200.parts.base import BuildEnv
        from lastengine_b200.registry import MIXERS
        from lastengine_b200.weights.loader import kept_dtype
        from lastengine_b200.weights.random_init import random_tensor
        dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
        dev = torch.device(device)
        self.device = device
        self.env = BuildEnv(device=dev, dtype=dt, workspace=Workspace(dev))
        self.mixer = MIXERS.get(kind)(**params)
        specs = self.mixer.tensors()
        self.plain = {}
        for name, spec in specs.items():
            t = random_tensor(name, spec, seed, std, norm_init="random").to(torch.bfloat16).double()
            self.plain[name] = t.numpy().copy()
        if edit:
            edit(self.plain)
            self.plain = {n: bf16_round_np(v) for n, v in self.plain.items()}
        self.mixer.load({n: torch.from_numpy(v).float().to(dev, kept_dtype(specs[n], torch.bfloat16, dt))
                         for n, v in self.plain.items()}, self.env)
        self.cache = Cache({0: self.mixer.cache_spec()}, max_tokens=max_tokens, max_seqs=max_seqs, dtype=dt, device=dev)
        self.builder = BatchBuilder(dev)
        self.D = params["hidden_size"] if hidden_size is None else hidden_size

    def step(self, slots, hs):
        """hs: per sequence a [n, D] array of mixer inputs; returns the mixer's outputs per sequence."""
        from lastengine_b200.cache import pooled_table_key
        from lastengine_b200.ops import kernels
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
        h = torch.from_numpy(np.concatenate(hs, 0)).to(self.device, self.env.dtype)
        out = torch.zeros(h.shape[0], self.D, dtype=torch.float32, device=self.device)
        self.mixer.forward(h, out, False, batch, self.cache.view(0, True, batch.tables), self.env)
        kernels.check_device_status()
        self.cache.commit(grow)
        out = out.double().cpu().numpy()
        return np.split(out, np.cumsum([x.shape[0] for x in hs])[:-1])

    def alone(self, h):
        s = self.cache.alloc_seq()
        try:
            return self.step([s], [h])[0]
        finally:
            self.cache.free_seq(s)


def whole_portions_and_batches(rig: MixerRig, plain_fn, lengths, more_n, cuts, tol: float, bf16: bool, seed=10, scale=1.0):
    """Each sequence alone and whole; then all together in the slots and pages just given back; then every
    one goes on in portions (rows cut at `cuts`) beside the others."""
    hs = [random_rows(n, rig.D, seed + n, bf16, scale) for n in lengths]
    want = [plain_fn(h) for h in hs]
    for h, w in zip(hs, want):
        assert max_err(rig.alone(h), w) < tol, f"alone, {h.shape[0]} rows"
    more = [random_rows(more_n, rig.D, seed + 50 + i, bf16, scale) for i in range(len(hs))]
    want2 = [plain_fn(np.concatenate([h, x])) for h, x in zip(hs, more)]
    slots = [rig.cache.alloc_seq() for _ in hs]
    for g, w in zip(rig.step(slots, hs), want):
        assert max_err(g, w) < tol, "batched"
    outs = [[] for _ in hs]
    for a, b in zip(cuts[:-1], cuts[1:]):
        for i, g in enumerate(rig.step(slots, [x[a:b] for x in more])):
            outs[i].append(g)
    for i, w in enumerate(want2):
        assert max_err(np.concatenate(outs[i]), w[hs[i].shape[0]:]) < tol, f"sequence {i} after portions"
    for s in slots:
        rig.cache.free_seq(s)
    rig.cache.check()
