"""Configuration of the Tevilix decoder, read from its config.json.

    {"architecture": "Tevilix", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "layers": [{"type": "parallel" | "mlstm", "mixer": {...}, "mlp": {...} | null}, ...],
     "loop": {"start": a, "stop": b, "times": n}}

parallel mixer: {"left": {heads, kv_heads, dim, vdim, scale, rot {dims, base, scaling {factor}}, mask {size}},
                 "left_scale": a, "right": {"width": w}, "right_scale": b}
mlstm mixer: heads, dim, vdim, gate_cap.
mlp: {"kind": "dense", "ff": F}, or
     {"kind": "moe", "router": {"experts": E, "top": k, "scale": c, "groups": {"count": g, "keep": n}},
      "expert": {"ff": F}}.
Every size and constant comes from the file.  Objects the design allows to be absent: `mlp` (a layer without a
feed-forward), `loop` (every layer runs once), `embedding` (scale 1), `mask` (every earlier position is seen),
`rot` (no rotation) and its `scaling` (factor 1), `router.groups` (no limit to groups), `router.scale` (1), and
the two scales of the parallel mixer (1).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import ConfigError, KeyReader
from .zekivik import Loop, _obj

PARALLEL = "parallel"
MLSTM = "mlstm"


@dataclass(frozen=True)
class ScaledRotation:
    dims: int              # 0: no rotation
    base: float
    factor: float          # every frequency is divided by it


@dataclass(frozen=True)
class MixedAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: ScaledRotation
    window: int            # 0: every earlier position is seen


@dataclass(frozen=True)
class ParallelSizes:
    left: MixedAttentionSizes
    left_scale: float
    right_width: int
    right_scale: float


@dataclass(frozen=True)
class MlstmSizes:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class DenseSizes:
    ff: int


@dataclass(frozen=True)
class MoeSizes:
    experts: int
    top: int
    groups: int            # 1 and keep 1: no limit to groups
    keep: int
    scale: float
    ff: int


@dataclass(frozen=True)
class TevilixLayer:
    type: str
    mixer: Any             # ParallelSizes | MlstmSizes
    mlp: Any               # DenseSizes | MoeSizes | None


@dataclass(frozen=True)
class TevilixConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: tuple[TevilixLayer, ...]
    loop: Loop | None

    @staticmethod
    def from_dict(raw: dict[str, Any]) -> "TevilixConfig":
        r = KeyReader(raw)
        norm = _obj(r, "norm", "config.json")
        layers = r.array("layers", item=lambda e: isinstance(e, dict))
        if not layers:
            raise ConfigError("config.json: 'layers' is empty")
        out = []
        for i, e in enumerate(layers):
            where = f"config.json: layers[{i}]"
            lr = KeyReader(e, where)
            kind = lr.string("type")
            mr = _obj(lr, "mixer", where)
            if kind == PARALLEL:
                mixer = ParallelSizes(
                    left=_attention(_obj(mr, "left", where), f"{where}: mixer: left"),
                    left_scale=mr.number("left_scale", default=1.0),
                    right_width=_obj(mr, "right", where).integer("width", minimum=1),
                    right_scale=mr.number("right_scale", default=1.0))
            elif kind == MLSTM:
                mixer = MlstmSizes(heads=mr.integer("heads", minimum=1), dim=mr.integer("dim", minimum=1),
                                   vdim=mr.integer("vdim", minimum=1), gate_cap=mr.number("gate_cap"))
                if not mixer.gate_cap > 0:
                    raise ConfigError(f"{where}: gate_cap must be positive, got {mixer.gate_cap}")
            else:
                raise ConfigError(f"{where}: unknown layer type '{kind}' ({MLSTM}, {PARALLEL})")
            out.append(TevilixLayer(kind, mixer, _mlp(lr, where)))
        loop = None
        if r.has("loop"):
            lp = _obj(r, "loop", "config.json")
            loop = Loop(lp.integer("start", minimum=0), lp.integer("stop", minimum=0), lp.integer("times", minimum=1))
            if not loop.start <= loop.stop <= len(out):
                raise ConfigError(f"config.json: loop {loop.start}..{loop.stop} does not fit {len(out)} layers")
        scale = _obj(r, "embedding", "config.json").number("scale", default=1.0) if r.has("embedding") else 1.0
        return TevilixConfig(
            architecture=r.string("architecture"), vocab=r.integer("vocab", minimum=1),
            width=r.integer("width", minimum=1), eps=norm.number("eps"), embedding_scale=scale,
            layers=tuple(out), loop=loop)

    def runs(self) -> list[int]:
        """The layers in running order: those before the loop once, the looped range `times` times as a whole
        (start .. stop-1, then again), the rest once."""
        n = len(self.layers)
        if self.loop is None or self.loop.stop == self.loop.start:
            return list(range(n))
        a, b, times = self.loop.start, self.loop.stop, self.loop.times
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def _attention(ar: KeyReader, where: str) -> MixedAttentionSizes:
    rot = ScaledRotation(0, 10000.0, 1.0)
    if ar.has("rot"):
        rr = _obj(ar, "rot", where)
        dims = rr.integer("dims", minimum=0)
        if dims % 2:
            raise ConfigError(f"{where}: rot.dims must be even, got {dims}")
        factor = _obj(rr, "scaling", where).number("factor", default=1.0) if rr.has("scaling") else 1.0
        if not factor > 0:
            raise ConfigError(f"{where}: rot.scaling.factor must be positive, got {factor}")
        rot = ScaledRotation(dims, rr.number("base"), factor)
    window = _obj(ar, "mask", where).integer("size", minimum=1) if ar.has("mask") else 0
    a = MixedAttentionSizes(
        heads=ar.integer("heads", minimum=1), kv_heads=ar.integer("kv_heads", minimum=1),
        dim=ar.integer("dim", minimum=1), vdim=ar.integer("vdim", minimum=1), scale=ar.number("scale"),
        rot=rot, window=window)
    if a.heads % a.kv_heads:
        raise ConfigError(f"{where}: {a.heads} heads do not divide into {a.kv_heads} kv_heads")
    if a.rot.dims > a.dim:
        raise ConfigError(f"{where}: rot.dims {a.rot.dims} is more than dim {a.dim}")
    return a


def _mlp(lr: KeyReader, where: str):
    if not lr.has("mlp"):
        return None
    fr = _obj(lr, "mlp", where)
    kind = fr.string("kind")
    if kind == "dense":
        return DenseSizes(ff=fr.integer("ff", minimum=1))
    if kind != "moe":
        raise ConfigError(f"{where}: unknown mlp kind '{kind}' (dense, moe)")
    rr = _obj(fr, "router", where)
    experts, top = rr.integer("experts", minimum=1), rr.integer("top", minimum=1)
    groups = keep = 1
    if rr.has("groups"):
        gr = _obj(rr, "groups", where)
        groups, keep = gr.integer("count", minimum=1), gr.integer("keep", minimum=1)
    if top > experts:
        raise ConfigError(f"{where}: top {top} of {experts} experts")
    if experts % groups or keep > groups or keep * (experts // groups) < top:
        raise ConfigError(f"{where}: {keep} of {groups} groups over {experts} experts cannot give {top} choices")
    return MoeSizes(experts=experts, top=top, groups=groups, keep=keep, scale=rr.number("scale", default=1.0),
                    ff=_obj(fr, "expert", where).integer("ff", minimum=1))
