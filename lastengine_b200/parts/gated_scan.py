"""Recurrent mixers whose gates read only the current token: the minimal gated recurrent unit and the matrix
memory with exponential gates (mLSTM).  Both keep float state per sequence that is zero when the sequence starts;
the projections run in the activation type with float results, and everything between them and the output
projection (biases, gates, their logarithms and exponentials, the running maximum, the state, the read-out, its
norm and gate) is float.

min_gru: z = sigmoid(Wz h + bz), u = Wx h + bx, candidate c = u + 1/2 where u >= 0 and sigmoid(u) below;
per channel S <- (1 - z) S + z c; out = Wo (S * silu(Wg h)).  State: `width` numbers.

mlstm: q = Wq h * dim^-1/2, k = Wk h (heads x dim), v = Wv h (heads x vdim); per head a log input gate
i = cap tanh((Wi h + bi) / cap) and a log forget gate f = logsigmoid(cap tanh((Wf h + bf) / cap)); with a running
maximum m (zero at the start) m' = max(f + m, i), S <- exp(f + m - m') S + exp(i - m') k v^T and n likewise with k
alone; o = S^T q / (max(|n . q|, exp(-m')) + 1e-6); every head's o is divided by its root mean square (eps of the
norm), the heads side by side times a weight over all of them, times sigmoid(Wg h); out = Wo o.  The normaliser n
rides in the state as one more column (the recurrence kernel writes it with a value of one), so the state is
[heads, vdim + 1, dim] and one number m per head.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import MIXERS
from .base import BIAS, MATRIX, NORM, VECTOR, BuildEnv, Mixer, StateSpec, TensorSpec


@MIXERS.register("min_gru")
class MinGRUMixer(Mixer):
    def __init__(self, hidden_size: int, width: int, bias: bool = True, names: dict[str, str] | None = None):
        self.D, self.W = int(hidden_size), int(width)
        self.has_bias = bool(bias)
        self.n = {"z": "z", "x": "x", "g": "g", "o": "o", "z_bias": "z.b", "x_bias": "x.b"}
        self.n.update(names or {})
        self.w_in = self.w_out = self.bz = self.bx = None

    def tensors(self) -> dict[str, TensorSpec]:
        n, D, W = self.n, self.D, self.W
        t = {n["z"]: TensorSpec((W, D), MATRIX), n["x"]: TensorSpec((W, D), MATRIX), n["g"]: TensorSpec((W, D), MATRIX),
             n["o"]: TensorSpec((D, W), MATRIX)}
        if self.has_bias:
            t[n["z_bias"]] = TensorSpec((W,), BIAS, std=0.5)
            t[n["x_bias"]] = TensorSpec((W,), BIAS, std=0.5)
        return t

    def cache_spec(self):
        return StateSpec((self.W,), torch.float32)

    def load(self, tensors, env: BuildEnv) -> None:
        n = self.n
        self.w_in = torch.cat([tensors[n["z"]], tensors[n["x"]], tensors[n["g"]]], dim=0).contiguous()
        self.w_out = tensors[n["o"]].contiguous()
        if self.has_bias:
            self.bz = tensors[n["z_bias"]].to(torch.float32).contiguous()
            self.bx = tensors[n["x_bias"]].to(torch.float32).contiguous()

    def flops_per_row(self) -> int:
        return super().flops_per_row() + 8 * self.W

    def input_projection(self):
        """The matrix of this mixer's one product over its input rows (z | x | g); see `forward(proj=...)`."""
        return self.w_in

    def forward(self, h, out, accumulate, batch, cache, env, proj=None) -> None:
        W = self.W
        M = h.shape[0]
        ws = env.workspace
        if proj is None:
            proj = ws.get("gru.proj", (M, 3 * W), torch.float32)
            kernels.linear(proj, h, self.w_in)
        s = ws.get("gru.s", (M, W), env.dtype)
        n = kernels.min_gru_scratch(batch, W)
        scratch = ws.get("gru.pieces", (n,), torch.float32) if n else None
        kernels.min_gru(s, proj[:, :W], proj[:, W: 2 * W], proj[:, 2 * W:], self.bz, self.bx, cache.state, batch,
                        scratch=scratch)
        kernels.linear(out, s, self.w_out, kernels.ACCUMULATE if accumulate else kernels.STORE)


@MIXERS.register("mlstm")
class MLSTMMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, gate_cap: float, norm_eps: float,
                 gate_bias: bool = True, names: dict[str, str] | None = None):
        if head_dim > kernels.RECURRENCE_MAX_ROWS:
            raise ValueError(f"head_dim {head_dim} is larger than the recurrence kernel takes ({kernels.RECURRENCE_MAX_ROWS})")
        if not gate_cap > 0:
            raise ValueError(f"the gates' cap must be positive, got {gate_cap}")
        self.D, self.H, self.d, self.e = int(hidden_size), int(num_heads), int(head_dim), int(v_head_dim)
        self.cap, self.eps = float(gate_cap), float(norm_eps)
        self.has_bias = bool(gate_bias)
        self.n = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "i": "i", "f": "f", "i_bias": "i.b",
                  "f_bias": "f.b"}
        self.n.update(names or {})
        self.w_in = self.w_gates = self.w_out = self.bi = self.bf = self.norm_w = None

    def tensors(self) -> dict[str, TensorSpec]:
        n, D, H, d, e = self.n, self.D, self.H, self.d, self.e
        t = {n["q"]: TensorSpec((H * d, D), MATRIX), n["k"]: TensorSpec((H * d, D), MATRIX),
             n["v"]: TensorSpec((H * e, D), MATRIX), n["g"]: TensorSpec((H * e, D), MATRIX),
             n["o"]: TensorSpec((D, H * e), MATRIX), n["norm"]: TensorSpec((H * e,), NORM),
             n["i"]: TensorSpec((H, D), MATRIX), n["f"]: TensorSpec((H, D), MATRIX)}
        if self.has_bias:
            t[n["i_bias"]] = TensorSpec((H,), BIAS, std=0.5)
            t[n["f_bias"]] = TensorSpec((H,), BIAS, std=0.5)
        return t

    def cache_spec(self):
        # the matrix memory with the normaliser as one more column (a column of the state is contiguous), and m
        return StateSpec((self.H, self.e + 1, self.d), torch.float32), StateSpec((self.H,), torch.float32)

    def load(self, tensors, env: BuildEnv) -> None:
        n = self.n
        # one product for q | k | v | g | i | f: everything reads the same rows
        self.w_in = torch.cat([tensors[n[x]] for x in ("q", "k", "v", "g", "i", "f")], dim=0).contiguous()
        self.w_out = tensors[n["o"]].contiguous()
        if self.has_bias:
            self.bi = tensors[n["i_bias"]].to(torch.float32).contiguous()
            self.bf = tensors[n["f_bias"]].to(torch.float32).contiguous()
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous()

    def flops_per_row(self) -> int:
        return super().flops_per_row() + 6 * self.H * self.d * (self.e + 1)

    def forward(self, h, out, accumulate, batch, cache, env) -> None:
        H, d, e = self.H, self.d, self.e
        M = h.shape[0]
        ws = env.workspace
        f32 = torch.float32
        nq, nv = H * d, H * e
        proj = ws.get("mlstm.proj", (M, 2 * nq + 2 * nv + 2 * H), f32)
        kernels.linear(proj, h, self.w_in)
        q, k = proj[:, :nq], proj[:, nq: 2 * nq]
        v, g = proj[:, 2 * nq: 2 * nq + nv], proj[:, 2 * nq + nv: 2 * nq + 2 * nv]
        gi, gf = proj[:, 2 * nq + 2 * nv: 2 * nq + 2 * nv + H], proj[:, 2 * nq + 2 * nv + H:]
        decay = ws.get("mlstm.decay", (M, H), f32)
        write = ws.get("mlstm.write", (M, H), f32)
        mrow = ws.get("mlstm.m", (M, H), f32)
        kernels.exp_gates(decay, write, mrow, gi, gf, self.bi, self.bf, self.cap, cache.states[1], batch)
        y = ws.get("mlstm.y", (M, H * (e + 1)), f32)
        kernels.gated_recurrence(y, k, q, v, write, decay, cache.states[0], batch, H, H, d, e + 1, delta=False,
                                 ones_columns=1)
        o = ws.get("mlstm.o", (M, nv), env.dtype)
        kernels.exp_gates_finish(o, y, mrow, g, self.norm_w, d ** -0.5, self.eps, H, e)
        kernels.linear(out, o, self.w_out, kernels.ACCUMULATE if accumulate else kernels.STORE)
