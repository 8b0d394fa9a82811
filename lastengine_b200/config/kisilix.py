"""Configuration of the Kisilix decoder, read from its config.json.

    {"architecture": "Kisilix", "vocab": V, "width": W, "max_positions": P, "norm": {"eps": e}, "postln_alpha": a,
     "layers": [{"type": "channel_delta" | "mamba2" | "attention", "mixer": {...}, "mlp": {...} | null}, ...]}

channel_delta mixer: heads, kv_heads, dim, vdim, conv (taps).
mamba2 mixer: heads, vdim, state, groups, norm_groups, conv (taps).
attention mixer: heads, kv_heads, dim, vdim, scale, rot {dims, base}, mask {size, pool}.
mlp: {"kind": "dense", "ff": F, "limit": L}, or
     {"kind": "moe", "router": {"experts": E, "top": k, "groups": {"count": c, "keep": n}},
      "expert": {"ff": F}, "shared": {"ff": Fs}}.
Every size and constant comes from the file.  Objects the design defines as optional: `mlp` (a layer without a
feed-forward), `router.groups` (no limit to groups), `shared` (no shared expert), `mask` (plain causal attention)
and `rot` (no rotation of queries, keys or values).  The low ranks of the delta mixer's decay and gate
projections are read off the tensors' shapes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import ConfigError, KeyReader
from .zekivik import Rotation, _obj, _rotation

CHANNEL_DELTA = "channel_delta"
MAMBA2 = "mamba2"
ATTENTION = "attention"


@dataclass(frozen=True)
class DeltaSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class StateSpaceSizes:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int


@dataclass(frozen=True)
class PooledAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Rotation | None
    window: int            # 0: every earlier position is seen
    pool: int              # 0: nothing is seen behind the window


@dataclass(frozen=True)
class DenseSizes:
    ff: int
    limit: float


@dataclass(frozen=True)
class MoeSizes:
    experts: int
    top: int
    groups: int            # 1 and keep 1: no limit to groups
    keep: int
    ff: int
    shared_ff: int         # 0: no shared expert


@dataclass(frozen=True)
class KisilixLayer:
    type: str
    mixer: Any             # DeltaSizes | StateSpaceSizes | PooledAttentionSizes
    mlp: Any               # DenseSizes | MoeSizes | None


@dataclass(frozen=True)
class KisilixConfig:
    architecture: str
    vocab: int
    width: int
    max_positions: int
    eps: float
    alpha: float
    layers: tuple[KisilixLayer, ...]

    @staticmethod
    def from_dict(raw: dict[str, Any]) -> "KisilixConfig":
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
            if kind == CHANNEL_DELTA:
                mixer = DeltaSizes(
                    heads=mr.integer("heads", minimum=1), kv_heads=mr.integer("kv_heads", minimum=1),
                    dim=mr.integer("dim", minimum=1), vdim=mr.integer("vdim", minimum=1), conv=mr.integer("conv", minimum=1))
                _divides(where, mixer.heads, mixer.kv_heads, "kv_heads")
            elif kind == MAMBA2:
                mixer = StateSpaceSizes(
                    heads=mr.integer("heads", minimum=1), vdim=mr.integer("vdim", minimum=1),
                    state=mr.integer("state", minimum=1), groups=mr.integer("groups", minimum=1),
                    norm_groups=mr.integer("norm_groups", minimum=1), conv=mr.integer("conv", minimum=1))
                _divides(where, mixer.heads, mixer.groups, "groups")
                _divides(where, mixer.heads * mixer.vdim, mixer.norm_groups, "norm_groups")
            elif kind == ATTENTION:
                window = pool = 0
                if mr.has("mask"):
                    mk = _obj(mr, "mask", where)
                    window = mk.integer("size", minimum=1)
                    pool = mk.integer("pool", default=0, minimum=0)
                mixer = PooledAttentionSizes(
                    heads=mr.integer("heads", minimum=1), kv_heads=mr.integer("kv_heads", minimum=1),
                    dim=mr.integer("dim", minimum=1), vdim=mr.integer("vdim", minimum=1), scale=mr.number("scale"),
                    rot=_rotation(mr, where) if mr.has("rot") else None, window=window, pool=pool)
                _divides(where, mixer.heads, mixer.kv_heads, "kv_heads")
                if mixer.rot is not None:
                    if mixer.rot.dims > mixer.dim:
                        raise ConfigError(f"{where}: rot.dims {mixer.rot.dims} is more than dim {mixer.dim}")
                    if mixer.vdim % 2:
                        raise ConfigError(f"{where}: values are rotated in pairs, vdim {mixer.vdim} is odd")
            else:
                raise ConfigError(f"{where}: unknown layer type '{kind}' ({ATTENTION}, {CHANNEL_DELTA}, {MAMBA2})")
            out.append(KisilixLayer(kind, mixer, _mlp(lr, where)))
        return KisilixConfig(
            architecture=r.string("architecture"), vocab=r.integer("vocab", minimum=1),
            width=r.integer("width", minimum=1), max_positions=r.integer("max_positions", minimum=1),
            eps=norm.number("eps"), alpha=r.number("postln_alpha"), layers=tuple(out))


def _divides(where: str, n: int, by: int, what: str) -> None:
    if n % by:
        raise ConfigError(f"{where}: {n} does not divide into {by} {what}")


def _mlp(lr: KeyReader, where: str):
    if not lr.has("mlp"):
        return None
    fr = _obj(lr, "mlp", where)
    kind = fr.string("kind")
    if kind == "dense":
        return DenseSizes(ff=fr.integer("ff", minimum=1), limit=fr.number("limit"))
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
    shared_ff = 0
    if fr.has("shared"):
        shared_ff = _obj(fr, "shared", where).integer("ff", minimum=1)
    return MoeSizes(experts=experts, top=top, groups=groups, keep=keep,
                    ff=_obj(fr, "expert", where).integer("ff", minimum=1), shared_ff=shared_ff)
