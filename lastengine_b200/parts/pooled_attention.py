"""Windowed attention with pooled blocks behind the window and rotated values, over the paged cache.

q = Wq h + bq, k = Wk h + bk, v = Wv h + bv (grouped key/value heads; value heads of their own width).  Every
q and k head is divided by its root mean square (eps of the norm) and multiplied by a weight over the head
shared by all heads, then rotated by its position on the first rope_dim numbers (split-half pairs).  The
value of position j is rotated by j over its whole width (split-half pairs, pair m by j * base^(-2m/vdim))
and cached so; a head's result at position i is turned back by -i before the output projection.
score = (q . k) * scale * temperature[head].  Position i sees the positions j with 0 <= i - j < window and,
beside them, one key and one value for every block of `pool` positions that lies wholly before the window:
the means of the block's cached keys and of its cached values.  Positions that have left the window and
whose block is not complete are seen by nobody.  One softmax over positions and blocks; out = Wo o.

The pooled rows live in pages of their own beside the positions' (parts.base.KVSpec.pool); the step that
brings a block's last position forms them from the cache, so they do not depend on how a sequence was cut
into steps.  Norms, rotations, scores, the softmax and the pooling sums are float.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import MIXERS, POSITION_ENCODINGS
from .base import BIAS, MATRIX, NORM, VECTOR, BuildEnv, KVSpec, Mixer, PartSpec, TensorSpec


@MIXERS.register("pooled_window_attention")
class PooledWindowAttentionMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int,
                 norm_eps: float, scale: float, window: int = 0, pool: int = 0, position: PartSpec | None = None,
                 value_rotation_base: float | None = None, bias: bool = True, qk_norm: bool = True,
                 head_temperature: bool = True, names: dict[str, str] | None = None):
        """`window` 0: every earlier position is seen (and nothing is pooled).  `value_rotation_base` None:
        values are cached as projected.  `position`: a split-half rotation of q and k, or none."""
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads do not divide into {num_kv_heads} kv heads")
        if not (1 <= head_dim <= 256 and 2 <= v_head_dim <= 256):
            raise ValueError(f"head sizes {head_dim} / {v_head_dim} outside what the kernels take (up to 256)")
        if pool and not window:
            raise ValueError("blocks are pooled behind a window: pool needs window > 0")
        if value_rotation_base is not None and v_head_dim % 2:
            raise ValueError(f"values are rotated in pairs, v_head_dim {v_head_dim} is odd")
        self.D, self.nh, self.nkv, self.hd, self.vd = (int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim),
                                                        int(v_head_dim))
        self.eps, self.scale = float(norm_eps), float(scale)
        self.window, self.pool = int(window), int(pool)
        self.v_base = None if value_rotation_base is None else float(value_rotation_base)
        self.has_bias, self.qk_norm, self.has_temp = bool(bias), bool(qk_norm), bool(head_temperature)
        pos = position or PartSpec("none")
        self.position = POSITION_ENCODINGS.get(pos.kind)(**pos.params)
        self.n = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                  "q_norm": "q.norm", "k_norm": "k.norm", "temperature": "temp"}
        self.n.update(names or {})
        self.w_in = self.w_out = self.b_in = self.q_norm_w = self.k_norm_w = self.head_scale = self.freq_v = None

    def tensors(self) -> dict[str, TensorSpec]:
        D, nh, nkv, hd, vd, n = self.D, self.nh, self.nkv, self.hd, self.vd, self.n
        t = {n["q"]: TensorSpec((nh * hd, D), MATRIX), n["k"]: TensorSpec((nkv * hd, D), MATRIX),
             n["v"]: TensorSpec((nkv * vd, D), MATRIX), n["o"]: TensorSpec((D, nh * vd), MATRIX)}
        if self.has_bias:
            t[n["q_bias"]] = TensorSpec((nh * hd,), BIAS, std=0.1)
            t[n["k_bias"]] = TensorSpec((nkv * hd,), BIAS, std=0.1)
            t[n["v_bias"]] = TensorSpec((nkv * vd,), BIAS, std=0.1)
        if self.qk_norm:
            t[n["q_norm"]] = TensorSpec((hd,), NORM)
            t[n["k_norm"]] = TensorSpec((hd,), NORM)
        if self.has_temp:
            t[n["temperature"]] = TensorSpec((nh,), NORM)       # a factor around one
        for name, spec in self.position.tensors().items():
            t[f"position.{name}"] = spec
        return t

    def cache_spec(self):
        return KVSpec(self.nkv, self.hd, self.window, None if self.vd == self.hd else self.vd, self.pool)

    def load(self, tensors, env: BuildEnv) -> None:
        n = self.n
        self.w_in = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous()
        self.w_out = tensors[n["o"]].contiguous()
        if self.has_bias:
            self.b_in = torch.cat([tensors[n[x]].to(torch.float32).reshape(-1) for x in ("q_bias", "k_bias", "v_bias")]).contiguous()
        if self.qk_norm:
            self.q_norm_w = tensors[n["q_norm"]].to(torch.float32).contiguous()
            self.k_norm_w = tensors[n["k_norm"]].to(torch.float32).contiguous()
        temp = tensors[n["temperature"]].to(torch.float32).reshape(-1) if self.has_temp \
            else torch.ones(self.nh, dtype=torch.float32, device=env.device)
        self.head_scale = (temp * self.scale).contiguous()       # what a head's scores are multiplied by
        self.position.load({k[len("position."):]: v for k, v in tensors.items() if k.startswith("position.")}, env)
        rotary = self.position.fused_rotary()
        if rotary is None or not rotary[2]:
            raise ValueError("this attention takes a split-half rotation (or none) as its position encoding")
        self.freq_qk, self.rot = rotary[0], (int(rotary[1]) if rotary[0] is not None else 0)
        if self.rot > self.hd:
            raise ValueError(f"{self.rot} rotated dimensions do not fit a head of {self.hd}")
        if self.v_base is not None:
            m = torch.arange(self.vd // 2, dtype=torch.float64)
            self.freq_v = torch.pow(torch.tensor(self.v_base, dtype=torch.float64), -2.0 * m / self.vd) \
                .to(torch.float32).to(env.device)

    def flops_per_query_key(self) -> int:
        return 2 * self.nh * (self.hd + self.vd)

    def forward(self, h, out, accumulate, batch, cache, env) -> None:
        nh, nkv, hd, vd = self.nh, self.nkv, self.hd, self.vd
        M = h.shape[0]
        ws = env.workspace
        if not cache.writable:
            raise NotImplementedError("this attention keeps its own keys and values")
        proj = ws.get("pattn.proj", (M, self.w_in.shape[0]), torch.float32)
        kernels.linear(proj, h, self.w_in)
        q = ws.get("pattn.q", (M, nh * hd), env.dtype)
        kernels.pooled_attn_prep(q, cache.k, cache.v, proj, self.b_in, self.q_norm_w, self.k_norm_w, self.eps,
                                 self.freq_qk, self.rot, self.freq_v, cache.block_table, batch, nh, nkv, hd, vd,
                                 cache.page_size)
        if self.pool > 0:      # the blocks this step completes, from the rows the launch above cached
            kernels.pool_blocks(cache.pooled_k, cache.pooled_v, cache.k, cache.v, cache.block_table, cache.pooled_table,
                                batch, nkv, hd, vd, cache.page_size, self.pool)
        o = ws.get("pattn.o", (M, nh * vd), env.dtype)
        n_splits = kernels.pooled_attention_splits(batch, nkv, nh // nkv, self.window, self.pool)
        scratch = ws.get("pattn.part", (M * nh * n_splits * (vd + 2),), torch.float32) if n_splits > 1 else None
        kernels.attention_pooled(o, q, cache.k, cache.v, cache.block_table, cache.pooled_k, cache.pooled_v,
                                 cache.pooled_table, batch, self.head_scale, self.freq_v, nh, nkv, hd, vd, cache.page_size,
                                 self.window, self.pool, n_splits=n_splits, scratch=scratch)
        kernels.linear(out, o, self.w_out, kernels.ACCUMULATE if accumulate else kernels.STORE)
