"""Two mixers side by side: out = a * Left(h) + b * Right(h), both reading the same rows.

The children are mixers of the registry, named by `PartSpec`; their tensors live under `left.` and `right.`
of this part's prefix.  What they keep per sequence is kept together in one cache entry: at most one of them
may hold keys and values, and their states must differ in shape (the cache files states by their shape).  A
child whose output projection has an additive term (`output_bias()`) gets it added here, in float, before
the weights a and b are applied.  Where both children form one product over their input rows with float results
(`input_projection()`), the two products are one here: the matrices are stacked once at load (the children keep
views of their rows), and each child's `forward` gets its columns of the result.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import MIXERS
from .base import BuildEnv, KVSpec, LatentSpec, Mixer, PartSpec, StateSpec, TensorSpec


def _as_list(spec) -> list:
    if spec is None:
        return []
    return list(spec) if isinstance(spec, (tuple, list)) else [spec]


@MIXERS.register("parallel_mixers")
class ParallelMixers(Mixer):
    def __init__(self, left: PartSpec, right: PartSpec, left_scale: float = 1.0, right_scale: float = 1.0,
                 names: tuple[str, str] = ("left", "right")):
        self.left = MIXERS.get(left.kind)(**left.params)
        self.right = MIXERS.get(right.kind)(**right.params)
        self.a, self.b = float(left_scale), float(right_scale)
        self.names = (str(names[0]), str(names[1]))
        specs = [_as_list(self.left.cache_spec()), _as_list(self.right.cache_spec())]
        kv = [s for side in specs for s in side if isinstance(s, (KVSpec, LatentSpec))]
        states = [s for side in specs for s in side if isinstance(s, StateSpec)]
        if len(kv) > 1 or len(set(states)) != len(states):
            raise ValueError("mixers side by side: at most one may keep keys and values, and their states must differ in shape")
        self._specs = specs

    def children(self):
        return ((self.names[0], self.left), (self.names[1], self.right))

    def tensors(self) -> dict[str, TensorSpec]:
        t = {}
        for name, part in self.children():
            for rel, spec in part.tensors().items():
                t[f"{name}.{rel}" if rel else name] = spec
        return t

    def load(self, tensors, env: BuildEnv) -> None:
        for name, part in self.children():
            own = {}
            for rel in part.tensors():
                full = f"{name}.{rel}" if rel else name
                if full in tensors:
                    own[rel] = tensors[full]
            part.load(own, env)
        self.w_in, self.n_left = None, 0
        wa = getattr(self.left, "input_projection", lambda: None)()
        wb = getattr(self.right, "input_projection", lambda: None)()
        if wa is not None and wb is not None and wa.dtype == wb.dtype and wa.shape[1] == wb.shape[1]:
            self.w_in = torch.cat([wa, wb], dim=0).contiguous()
            self.n_left = int(wa.shape[0])
            self.left.w_in, self.right.w_in = self.w_in[: self.n_left], self.w_in[self.n_left:]      # views: one copy of the weights

    def cache_spec(self):
        flat = [s for side in self._specs for s in side]
        return None if not flat else (flat[0] if len(flat) == 1 else tuple(flat))

    def flops_per_row(self) -> int:
        return self.left.flops_per_row() + self.right.flops_per_row()

    def flops_per_query_key(self) -> int:
        return self.left.flops_per_query_key() + self.right.flops_per_query_key()

    def unread_weight_bytes(self, rows: int) -> float:
        return self.left.unread_weight_bytes(rows) + self.right.unread_weight_bytes(rows)

    def _view(self, cache, side: int):
        """The cache entry as one child sees it: the keys and values if they are its own, and its states in its order."""
        from ..cache.cache import CacheView      # here: the cache module itself imports the parts' base
        mine = self._specs[side]
        before = sum(1 for s in self._specs[0] if isinstance(s, StateSpec)) if side == 1 else 0
        n_states = sum(1 for s in mine if isinstance(s, StateSpec))
        view = CacheView(writable=cache.writable, page_size=cache.page_size)
        if any(isinstance(s, (KVSpec, LatentSpec)) for s in mine):
            view.k, view.v, view.block_table = cache.k, cache.v, cache.block_table
            view.pooled_k, view.pooled_v, view.pooled_table = cache.pooled_k, cache.pooled_v, cache.pooled_table
        view.states = list(cache.states[before: before + n_states])
        view.state = view.states[0] if view.states else None
        return view

    def forward(self, h, out, accumulate, batch, cache, env) -> None:
        M, D = out.shape
        ws = env.workspace
        y1 = ws.get("pair.left", (M, D), torch.float32)
        y2 = ws.get("pair.right", (M, D), torch.float32)
        bias = getattr(self.left, "output_bias", lambda: None)()
        kl, kr = {}, {}
        if self.w_in is not None:
            proj = ws.get("pair.proj", (M, self.w_in.shape[0]), torch.float32)
            kernels.linear(proj, h, self.w_in)
            kl["proj"], kr["proj"] = proj[:, : self.n_left], proj[:, self.n_left:]
        if bias is not None:
            kl["add_output_bias"] = False
        self.left.forward(h, y1, False, batch, self._view(cache, 0), env, **kl)
        self.right.forward(h, y2, False, batch, self._view(cache, 1), env, **kr)
        if getattr(self.right, "output_bias", lambda: None)() is not None:
            raise NotImplementedError("an output bias on the right-hand mixer")
        kernels.weighted_pair_sum(out, y1, self.a, y2, self.b, bias1=bias, accumulate=accumulate)
