"""Recurrent mixers with a matrix state per head: the gated delta rule and the state-space (SSD) layer.

Both keep, per sequence and head, a float state S [dim, vdim] that one kernel (ops.kernels.gated_recurrence)
walks over the step's rows, and the last taps-1 inputs of a short causal convolution; both are zero when a
sequence starts.  The projections and the convolutions run in the activation type with float results;
everything between them and the output projection (activations, unit norms, decays, step sizes, write
strengths, the recurrence, the norm and the gate of its result) is float.

gated_delta_rule: q = Wq h, k = Wk h (kv_heads x dim), v = Wv h (heads x vdim); each through its own causal
convolution over time per channel (`<tensor>.conv` [channels, taps], last column on the current row, no
bias) and silu; q and k become unit vectors per head, x / sqrt(sum x^2 + unit_eps), q times dim^-1/2; write
strength beta = sigmoid(Wb h) per head; decay per head and key channel g = exp(-exp(A_log_h) softplus(Wa2 Wa1 h
+ dt_bias)); per head (head h reads q/k head h // (heads / kv_heads))
    S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
so the read-out sees the row's own write; o is divided by its root mean square per head (eps of the norm), times
a weight over vdim shared by the heads, times sigmoid(Wg2 Wg1 h); out = Wo o.  The ranks of the two low-rank
pairs are whatever the checkpoint's tensors have.

state_space (SSD): Win h = [z: inner | x: inner | B: G N | C: G N | dt: heads], inner = heads x vdim; x, B and C
together through a causal convolution per channel with a bias, and silu; dt = softplus(dt + dt_bias), no clamp;
per head (head h reads group h // (heads / groups))
    S <- exp(-exp(A_log_h) dt) S + dt B x^T;   y = S^T C + D_h x
y silu(z) is divided by its root mean square in `norm_groups` equal parts of the row, times a weight over
inner; out = Wo y.  The gate comes before the norm.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import MIXERS
from .base import BIAS, MATRIX, NORM, VECTOR, BuildEnv, Mixer, StateSpec, TensorSpec

_MAX_TAPS = 16


def _check_taps(taps: int) -> int:
    if not 1 <= int(taps) <= _MAX_TAPS:
        raise ValueError(f"a convolution of {taps} taps: the kernel takes 1..{_MAX_TAPS}")
    return int(taps)


@MIXERS.register("gated_delta_rule")
class GatedDeltaRuleMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int,
                 conv_taps: int, norm_eps: float, unit_eps: float = 1e-6, decay_rank: int | None = None,
                 gate_rank: int | None = None, names: dict[str, str] | None = None):
        """`decay_rank`, `gate_rank`: the inner sizes of the two low-rank pairs; None: the checkpoint's
        (random weights then take a quarter of head_dim, at least 8)."""
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads do not divide into {num_kv_heads} key heads")
        if head_dim > kernels.RECURRENCE_MAX_ROWS:
            raise ValueError(f"head_dim {head_dim} is larger than the recurrence kernel takes ({kernels.RECURRENCE_MAX_ROWS})")
        self.D, self.H, self.G, self.d, self.e = (int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim),
                                                   int(v_head_dim))
        self.taps = _check_taps(conv_taps)
        self.eps, self.unit_eps = float(norm_eps), float(unit_eps)
        self.ra, self.rg = decay_rank, gate_rank
        self.n = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "write": "b",
                  "A_log": "A_log", "norm": "norm", "decay_down": "a1", "decay_up": "a2", "dt_bias": "dt_bias",
                  "gate_down": "g1", "gate_up": "g2", "o": "o"}
        self.n.update(names or {})
        self.C = 2 * self.G * self.d + self.H * self.e      # convolved channels: q | k | v
        self.w_in = self.w_low = self.w_a2 = self.w_g2 = self.w_out = None

    def tensors(self) -> dict[str, TensorSpec]:
        D, H, G, d, e, n, taps = self.D, self.H, self.G, self.d, self.e, self.n, self.taps
        free = max(8, d // 4)
        ra, rg = (-1 if self.ra is None else self.ra), (-1 if self.rg is None else self.rg)
        return {
            n["q"]: TensorSpec((G * d, D), MATRIX), n["k"]: TensorSpec((G * d, D), MATRIX),
            n["v"]: TensorSpec((H * e, D), MATRIX),
            n["q_conv"]: TensorSpec((G * d, taps), VECTOR, std=0.5), n["k_conv"]: TensorSpec((G * d, taps), VECTOR, std=0.5),
            n["v_conv"]: TensorSpec((H * e, taps), VECTOR, std=0.5),
            n["write"]: TensorSpec((H, D), MATRIX), n["A_log"]: TensorSpec((H,), VECTOR, std=0.5),
            n["norm"]: TensorSpec((e,), NORM),
            n["decay_down"]: TensorSpec((ra, D), MATRIX, free=free), n["decay_up"]: TensorSpec((H * d, ra), MATRIX, free=free),
            n["dt_bias"]: TensorSpec((H * d,), VECTOR, std=0.5),
            n["gate_down"]: TensorSpec((rg, D), MATRIX, free=free), n["gate_up"]: TensorSpec((H * e, rg), MATRIX, free=free),
            n["o"]: TensorSpec((D, H * e), MATRIX)}

    def cache_spec(self):
        state = StateSpec((self.H, self.e, self.d), torch.float32)      # a column of S is contiguous
        if self.taps <= 1:
            return state
        return state, StateSpec((self.C, self.taps - 1), torch.float32)

    def load(self, tensors, env: BuildEnv) -> None:
        n = self.n
        a1, a2, g1, g2 = (tensors[n[x]] for x in ("decay_down", "decay_up", "gate_down", "gate_up"))
        if a1.shape[0] != a2.shape[1] or g1.shape[0] != g2.shape[1]:
            raise ValueError(f"low-rank pairs do not fit: {tuple(a1.shape)} with {tuple(a2.shape)}, "
                             f"{tuple(g1.shape)} with {tuple(g2.shape)}")
        self.ra, self.rg = int(a1.shape[0]), int(g1.shape[0])
        # one product for q | k | v | write, one for the two low ranks (their results feed products again)
        self.w_in = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["write"]]], dim=0).contiguous()
        self.w_low = torch.cat([a1, g1], dim=0).contiguous()
        self.w_a2, self.w_g2 = a2.contiguous(), g2.contiguous()
        self.w_out = tensors[n["o"]].contiguous()
        self.w_conv = torch.cat([tensors[n["q_conv"]], tensors[n["k_conv"]], tensors[n["v_conv"]]], dim=0) \
            .to(torch.float32).contiguous()
        self.A_log = tensors[n["A_log"]].to(torch.float32).contiguous()
        self.dt_bias = tensors[n["dt_bias"]].to(torch.float32).contiguous()
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous()

    def flops_per_row(self) -> int:
        # the products, and per head the state's decay, read, write and read-out
        return super().flops_per_row() + 8 * self.H * self.d * self.e

    def forward(self, h, out, accumulate, batch, cache, env) -> None:
        H, G, d, e, C = self.H, self.G, self.d, self.e, self.C
        M = h.shape[0]
        ws = env.workspace
        f32 = torch.float32
        proj = ws.get("delta.proj", (M, C + H), f32)
        kernels.linear(proj, h, self.w_in)
        low = ws.get("delta.low", (M, self.ra + self.rg), env.dtype)
        kernels.linear(low, h, self.w_low)
        a = ws.get("delta.a", (M, H * d), f32)
        kernels.linear(a, low[:, : self.ra], self.w_a2)
        gate = ws.get("delta.gate", (M, H * e), f32)
        kernels.linear(gate, low[:, self.ra:], self.w_g2)
        conv = ws.get("delta.conv", (M, C), f32)
        kernels.causal_conv(conv, proj[:, :C], self.w_conv, cache.states[1] if self.taps > 1 else None, batch)
        qn = ws.get("delta.q", (M, G * d), f32)
        kn = ws.get("delta.k", (M, G * d), f32)
        vs = ws.get("delta.v", (M, H * e), f32)
        g = ws.get("delta.g", (M, H * d), f32)
        wr = ws.get("delta.w", (M, H), f32)
        kernels.delta_prep(qn, kn, vs, g, wr, conv, a, proj[:, C:], self.dt_bias, self.A_log, H, G, d, e,
                           self.unit_eps, d ** -0.5)
        o = ws.get("delta.o", (M, H * e), f32)
        kernels.gated_recurrence(o, kn, qn, vs, wr, g, cache.states[0], batch, H, G, d, e, delta=True)
        on = ws.get("delta.on", (M, H * e), env.dtype)
        kernels.group_norm_gate(on, o, gate, self.norm_w, e, self.eps, gate_first=False)
        kernels.linear(out, on, self.w_out, kernels.ACCUMULATE if accumulate else kernels.STORE)


@MIXERS.register("state_space")
class StateSpaceMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, v_head_dim: int, state_size: int, num_groups: int,
                 norm_groups: int, conv_taps: int, norm_eps: float, names: dict[str, str] | None = None):
        if num_heads % num_groups:
            raise ValueError(f"{num_heads} heads do not divide into {num_groups} groups")
        if (num_heads * v_head_dim) % norm_groups:
            raise ValueError(f"{num_heads * v_head_dim} inner channels do not divide into {norm_groups} norm groups")
        if state_size > kernels.RECURRENCE_MAX_ROWS:
            raise ValueError(f"a state of {state_size} rows is larger than the recurrence kernel takes "
                             f"({kernels.RECURRENCE_MAX_ROWS})")
        self.D, self.H, self.e, self.N, self.G = int(hidden_size), int(num_heads), int(v_head_dim), int(state_size), int(num_groups)
        self.parts_ = int(norm_groups)
        self.taps = _check_taps(conv_taps)
        self.eps = float(norm_eps)
        self.inner = self.H * self.e
        self.C = self.inner + 2 * self.G * self.N          # convolved channels: x | B | C
        self.n = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "A_log": "A_log", "D": "D",
                  "norm": "norm", "o": "o"}
        self.n.update(names or {})
        self.w_in = self.w_out = None

    def tensors(self) -> dict[str, TensorSpec]:
        n, D, H = self.n, self.D, self.H
        return {n["in"]: TensorSpec((self.inner + self.C + H, D), MATRIX),
                n["conv"]: TensorSpec((self.C, self.taps), VECTOR, std=0.5),
                n["conv_bias"]: TensorSpec((self.C,), BIAS, std=0.1),
                n["dt_bias"]: TensorSpec((H,), VECTOR, std=0.5), n["A_log"]: TensorSpec((H,), VECTOR, std=0.5),
                n["D"]: TensorSpec((H,), VECTOR, std=0.5), n["norm"]: TensorSpec((self.inner,), NORM),
                n["o"]: TensorSpec((D, self.inner), MATRIX)}

    def cache_spec(self):
        state = StateSpec((self.H, self.e, self.N), torch.float32)
        if self.taps <= 1:
            return state
        return state, StateSpec((self.C, self.taps - 1), torch.float32)

    def load(self, tensors, env: BuildEnv) -> None:
        n = self.n
        self.w_in = tensors[n["in"]].contiguous()
        self.w_out = tensors[n["o"]].contiguous()
        self.w_conv = tensors[n["conv"]].to(torch.float32).contiguous()
        self.b_conv = tensors[n["conv_bias"]].to(torch.float32).contiguous()
        self.dt_bias = tensors[n["dt_bias"]].to(torch.float32).contiguous()
        self.A_log = tensors[n["A_log"]].to(torch.float32).contiguous()
        self.skip = tensors[n["D"]].to(torch.float32).contiguous()
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous()

    def flops_per_row(self) -> int:
        return super().flops_per_row() + 6 * self.H * self.N * self.e

    def forward(self, h, out, accumulate, batch, cache, env) -> None:
        H, e, N, G, inner, C = self.H, self.e, self.N, self.G, self.inner, self.C
        M = h.shape[0]
        ws = env.workspace
        f32 = torch.float32
        proj = ws.get("ssm.proj", (M, inner + C + H), f32)
        kernels.linear(proj, h, self.w_in)
        z, dt_raw = proj[:, :inner], proj[:, inner + C:]
        xbc = ws.get("ssm.conv", (M, C), f32)
        kernels.causal_conv(xbc, proj[:, inner: inner + C], self.w_conv, cache.states[1] if self.taps > 1 else None, batch)
        dt = ws.get("ssm.dt", (M, H), f32)
        decay = ws.get("ssm.decay", (M, H), f32)
        kernels.ssm_prep(xbc, self.b_conv, dt, decay, dt_raw, self.dt_bias, self.A_log)
        y = ws.get("ssm.y", (M, inner), f32)
        # keys are B, queries C (one row stride: both are slices of xbc), values x, write strength dt
        kernels.gated_recurrence(y, xbc[:, inner: inner + G * N], xbc[:, inner + G * N:], xbc[:, :inner], dt, decay,
                                 cache.states[0], batch, H, G, N, e, delta=False, skip=self.skip)
        yn = ws.get("ssm.yn", (M, inner), env.dtype)
        kernels.group_norm_gate(yn, y, z, self.norm_w, inner // self.parts_, self.eps, gate_first=True)
        kernels.linear(out, yn, self.w_out, kernels.ACCUMULATE if accumulate else kernels.STORE)
