"""Grouped-query attention whose scores are mixed across the heads before the softmax, over the paged cache.

q = Wq h + bq, k = Wk h + bk, v = Wv h + bv (grouped key/value heads: query head g reads key/value head
g // (heads / kv_heads); value heads of their own width).  Every q and k head is divided by its root mean
square (eps of the norm) and multiplied by a weight over the head shared by all heads, then rotated by its
position on the first rope_dim numbers (split-half pairs).  Raw scores s_g(i, j) = scale * q_g(i) . k(j); the
heads' scores are then mixed with a learned [heads, heads] matrix, t_h = sum_g talk[h, g] s_g, and each head
runs an ordinary softmax over the positions it sees: j <= i, and i - j < window where there is a window.
The heads' results side by side are multiplied element by element with sigmoid(Wg h) where the layer has an
output gate (the gate reads the mixer's input), and out = Wo o + bo.

The projections (and the gate) are one product with float results; bias, norms, rotation and the cache write
are one launch; scores, mixing, softmax and the sums over the values are float.  Biases, norms, the gate and
the mixing matrix are each optional, so the part also serves as plain windowed attention with biases.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import MIXERS, POSITION_ENCODINGS
from .base import BIAS, MATRIX, NORM, VECTOR, BuildEnv, KVSpec, Mixer, PartSpec, TensorSpec


@MIXERS.register("mixed_heads_attention")
class MixedHeadsAttentionMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int,
                 norm_eps: float, scale: float, window: int = 0, position: PartSpec | None = None,
                 bias: bool = True, qk_norm: bool = True, mix_heads: bool = True, output_gate: bool = True,
                 output_bias: bool | None = None, names: dict[str, str] | None = None):
        """`window` 0: every earlier position is seen.  `position`: a split-half rotation of q and k, or none.
        `output_bias` None: as `bias`."""
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads do not divide into {num_kv_heads} kv heads")
        if not qk_norm:
            raise NotImplementedError("the launch that prepares q and k norms every head: qk_norm=False is not built")
        if num_heads > 128:
            raise ValueError(f"{num_heads} heads: the kernel mixes up to 128 heads")
        if not (1 <= head_dim <= 512 and 1 <= v_head_dim <= 256):
            raise ValueError(f"head sizes {head_dim} / {v_head_dim} outside what the kernel takes (up to 512 / 256)")
        self.D, self.nh, self.nkv, self.hd, self.vd = (int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim),
                                                        int(v_head_dim))
        self.eps, self.scale, self.window = float(norm_eps), float(scale), int(window)
        self.has_bias, self.qk_norm, self.mix, self.gated = bool(bias), bool(qk_norm), bool(mix_heads), bool(output_gate)
        self.out_bias = self.has_bias if output_bias is None else bool(output_bias)
        pos = position or PartSpec("none")
        self.position = POSITION_ENCODINGS.get(pos.kind)(**pos.params)
        self.n = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b",
                  "q_norm": "q.norm", "k_norm": "k.norm", "talk": "talk", "gate": "g"}
        self.n.update(names or {})
        self.w_in = self.w_out = self.b_in = self.b_out = self.q_norm_w = self.k_norm_w = self.talk = None

    def tensors(self) -> dict[str, TensorSpec]:
        D, nh, nkv, hd, vd, n = self.D, self.nh, self.nkv, self.hd, self.vd, self.n
        t = {n["q"]: TensorSpec((nh * hd, D), MATRIX), n["k"]: TensorSpec((nkv * hd, D), MATRIX),
             n["v"]: TensorSpec((nkv * vd, D), MATRIX), n["o"]: TensorSpec((D, nh * vd), MATRIX)}
        if self.has_bias:
            t[n["q_bias"]] = TensorSpec((nh * hd,), BIAS, std=0.1)
            t[n["k_bias"]] = TensorSpec((nkv * hd,), BIAS, std=0.1)
            t[n["v_bias"]] = TensorSpec((nkv * vd,), BIAS, std=0.1)
        if self.out_bias:
            t[n["o_bias"]] = TensorSpec((D,), BIAS, std=0.1)
        if self.qk_norm:
            t[n["q_norm"]] = TensorSpec((hd,), NORM)
            t[n["k_norm"]] = TensorSpec((hd,), NORM)
        if self.mix:
            t[n["talk"]] = TensorSpec((nh, nh), VECTOR, std=0.5)
        if self.gated:
            t[n["gate"]] = TensorSpec((nh * vd, D), MATRIX)
        for name, spec in self.position.tensors().items():
            t[f"position.{name}"] = spec
        return t

    def cache_spec(self):
        return KVSpec(self.nkv, self.hd, self.window, None if self.vd == self.hd else self.vd)

    def load(self, tensors, env: BuildEnv) -> None:
        n = self.n
        parts = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]] + ([tensors[n["gate"]]] if self.gated else [])
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.w_out = tensors[n["o"]].contiguous()
        if self.has_bias:
            self.b_in = torch.cat([tensors[n[x]].to(torch.float32).reshape(-1) for x in ("q_bias", "k_bias", "v_bias")]).contiguous()
        self.b_out = tensors[n["o_bias"]].to(torch.float32).contiguous() if self.out_bias else None
        if self.qk_norm:
            self.q_norm_w = tensors[n["q_norm"]].to(torch.float32).contiguous()
            self.k_norm_w = tensors[n["k_norm"]].to(torch.float32).contiguous()
        self.talk = tensors[n["talk"]].to(torch.float32).contiguous() if self.mix \
            else torch.eye(self.nh, dtype=torch.float32, device=env.device)
        self.position.load({k[len("position."):]: v for k, v in tensors.items() if k.startswith("position.")}, env)
        rotary = self.position.fused_rotary()
        if rotary is None or not rotary[2]:
            raise ValueError("this attention takes a split-half rotation (or none) as its position encoding")
        self.freq_qk, self.rot = rotary[0], (int(rotary[1]) if rotary[0] is not None else 0)
        if self.rot > self.hd:
            raise ValueError(f"{self.rot} rotated dimensions do not fit a head of {self.hd}")

    def input_projection(self):
        """The matrix of this mixer's one product over its input rows (q | k | v | gate), for whoever forms it
        together with another mixer's; `forward(proj=...)` then takes the float results instead of forming them."""
        return self.w_in

    def output_bias(self):
        """The additive term of the output projection, which whoever takes this mixer's float result adds."""
        return self.b_out

    def flops_per_query_key(self) -> int:
        return 2 * self.nh * (self.hd + self.vd + self.nh)

    def forward(self, h, out, accumulate, batch, cache, env, add_output_bias: bool = True, proj=None) -> None:
        nh, nkv, hd, vd = self.nh, self.nkv, self.hd, self.vd
        M = h.shape[0]
        ws = env.workspace
        if not cache.writable:
            raise NotImplementedError("this attention keeps its own keys and values")
        if proj is None:
            proj = ws.get("mattn.proj", (M, self.w_in.shape[0]), torch.float32)
            kernels.linear(proj, h, self.w_in)
        n_qkv = (nh + nkv) * hd + nkv * vd
        q = ws.get("mattn.q", (M, nh * hd), env.dtype)
        kernels.pooled_attn_prep(q, cache.k, cache.v, proj[:, :n_qkv], self.b_in, self.q_norm_w, self.k_norm_w, self.eps,
                                 self.freq_qk, self.rot, None, cache.block_table, batch, nh, nkv, hd, vd, cache.page_size)
        o = ws.get("mattn.o", (M, nh * vd), env.dtype)
        n_splits = kernels.mixed_attention_splits(batch, nh, self.window)
        scratch = ws.get("mattn.part", (M * nh * n_splits * (vd + 2),), torch.float32) if n_splits > 1 else None
        kernels.attention_mixed(o, q, cache.k, cache.v, cache.block_table, batch, self.talk,
                                proj[:, n_qkv:] if self.gated else None, nh, nkv, hd, vd, cache.page_size, self.window,
                                self.scale, n_splits=n_splits, scratch=scratch)
        kernels.linear(out, o, self.w_out, kernels.ACCUMULATE if accumulate else kernels.STORE)
        if add_output_bias and self.b_out is not None:
            kernels.add_row_vector(out, self.b_out)
