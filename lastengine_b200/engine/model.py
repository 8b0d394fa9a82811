"""A model: the parts a plan names, built through the registries, with their weights.

`forward` runs the schedule over the rows of a step and returns the logits of the wanted
rows.  It is the only forward pass in the library: generation, the replay program and the
benchmark all go through it.
"""
from __future__ import annotations

import torch

from .. import parts as _parts  # noqa: F401  (registers the built-in parts)
from ..parts.base import BuildEnv, ModelPlan, TensorSpec
from ..ops import kernels
from ..parts.base import VECTOR
from ..registry import BLOCKS, EMBEDDINGS, FEED_FORWARDS, GATES, HEADS, MIXERS, NORMS


class Model:
    def __init__(self, plan: ModelPlan, env: BuildEnv):
        self.plan, self.env = plan, env
        self.embedding = EMBEDDINGS.get(plan.embedding.kind)(**plan.embedding.params)
        self.final_norm = NORMS.get(plan.final_norm.kind)(**plan.final_norm.params)
        self.head = HEADS.get(plan.head.kind)(**plan.head.params)
        self.blocks = []
        for ls in plan.layers:
            mixer = MIXERS.get(ls.mixer.kind)(**ls.mixer.params)
            ffn = None if ls.ffn is None else FEED_FORWARDS.get(ls.ffn.kind)(**ls.ffn.params)
            norm = lambda s: None if s is None else NORMS.get(s.kind)(**s.params)  # noqa: E731
            gates = {role: GATES.get(g.kind)(**g.params) for role, g in ls.gates.items()}
            self.blocks.append(BLOCKS.get(ls.block)(
                mixer=mixer, ffn=ffn, mixer_norm=norm(ls.mixer_norm), ffn_norm=norm(ls.ffn_norm),
                post_mixer_norm=norm(ls.post_mixer_norm), post_ffn_norm=norm(ls.post_ffn_norm), **gates, **ls.block_params))
        self.hidden_size, self.vocab_size = plan.hidden_size, plan.vocab_size
        # additions to the residual stream between schedule entries, and the tables they take rows from
        self.stream_adds: dict[int, list] = {}
        for a in plan.stream_adds:
            self.stream_adds.setdefault(a.before, []).append(a)
        self.keeps_embedding = any(a.embedding for a in plan.stream_adds)
        self.stream_tables: dict[str, torch.Tensor] = {}

    # ---- tensors ------------------------------------------------------------------------
    def named_parts(self) -> list[tuple[str, object]]:
        """(tensor-name prefix, part) for every part that may own tensors."""
        n = self.plan.names
        out = [(n.get("embedding", "embedding"), self.embedding),
               (n.get("final_norm", "final_norm"), self.final_norm),
               (n.get("head", "head"), self.head)]
        for ls, blk in zip(self.plan.layers, self.blocks):
            for role, part in blk.parts().items():
                out.append((f"{ls.prefix}.{ls.names.get(role, role)}", part))
        return out

    @staticmethod
    def _name(prefix: str, rel: str, spec: TensorSpec) -> str:
        """A part's tensor under its prefix; the relative name "" is the prefix itself."""
        return spec.shared_name or (f"{prefix}.{rel}" if rel else prefix)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs: dict[str, TensorSpec] = {}
        for prefix, part in self.named_parts():
            for rel, spec in part.tensors().items():
                name = self._name(prefix, rel, spec)
                if name in specs and specs[name] != spec:
                    raise ValueError(f"tensor '{name}' is declared twice, as {specs[name]} and as {spec}")
                specs[name] = spec
        for name, shape in self.plan.stream_tables.items():
            specs[name] = TensorSpec(tuple(shape), VECTOR)
        return specs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        """`tensors`: canonical name -> tensor on the device in the dtype of its role."""
        for prefix, part in self.named_parts():
            own = {}
            for rel, spec in part.tensors().items():
                name = self._name(prefix, rel, spec)
                if name in tensors:
                    own[rel] = tensors[name]
            part.load(own, self.env)
        self.stream_tables = {n: tensors[n].contiguous() for n in self.plan.stream_tables if n in tensors}
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding)

    def cache_specs(self) -> dict[int, object]:
        """cache entry id -> spec, for the entries that own storage."""
        specs = {}
        for i, e in enumerate(self.plan.schedule):
            if e.cache is None or e.cache == i:
                specs[i] = self.blocks[e.layer].mixer.cache_spec()
        return specs

    # ---- the forward pass ---------------------------------------------------------------
    def forward(self, batch, cache) -> torch.Tensor:
        """Runs the step's rows through every scheduled layer; returns float logits
        [batch.n_logit_rows, vocab] (a view of workspace memory, valid until the next step)."""
        env, ws = self.env, self.env.workspace
        M, D = batch.n_rows, self.hidden_size
        x = ws.get("model.x", (M, D), torch.float32)
        self.embedding.forward(x, batch.tokens, batch=batch)
        x0 = None
        if self.keeps_embedding:      # the embedding output is added to the stream again later
            x0 = ws.get("model.x0", (M, D), torch.float32)
            self.embedding.forward(x0, batch.tokens, batch=batch)
        sched = self.plan.schedule
        pending = None      # the half of the next block's first norm that the last block left (decode steps)
        for i, e in enumerate(sched):
            entry = i if e.cache is None else e.cache
            view = cache.view(entry, e.writes_cache and entry == i, batch.tables)
            block = self.blocks[e.layer]
            for a in self.stream_adds.get(i, ()):
                kernels.stream_add(x, x0 if a.embedding else None,
                                   self.stream_tables[a.table][a.row] if a.table is not None else None)
                pending = None      # a norm half left for this block was taken from the stream as it was before
            after = self.blocks[sched[i + 1].layer] if i + 1 < len(sched) else None
            # (norm, part that reads it) of the block that runs next, for blocks that can split a norm
            # (nothing is offered across an addition to the stream: the norm would be of the stream before it)
            env.next_block_norm = after.first_reader() if hasattr(after, "first_reader") and (i + 1) not in self.stream_adds \
                else None
            if pending is not None:
                pending = block.forward(x, batch, view, env, pending=pending)
            else:
                pending = block.forward(x, batch, view, env)
        env.next_block_norm = None
        R = batch.n_logit_rows
        logits = ws.get("model.logits", (R, self.vocab_size), torch.float32)
        if R:
            xn = ws.get("model.xn", (R, D), env.dtype)
            self.final_norm.forward(xn, x, rows=batch.logit_rows)
            self.head.forward(logits, xn)
        return logits
