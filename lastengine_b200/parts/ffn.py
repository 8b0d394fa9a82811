"""Feed-forward parts: dense SwiGLU, and sigmoid-routed top-k experts of the same shape.

Dense (src/dense.rs:188-191): f = W2 (silu(W1 h) * W3 h).  Gate and up weights are one
matrix, as in the reference's GPU path (src/gpu/dense.rs:67-74).  In bfloat16 their rows are
interleaved in blocks of 16 so that the matrix product's epilogue holds a gate value and its
up value together and applies SwiGLU before anything is written; gate and up are never
rounded.

Experts: z = Wr h (float), s = sigmoid(z); the k experts with the largest s + bias (ties to
the lower index; the bias chooses, it does not weigh); weight s_e, divided by the sum over the
chosen when norm_topk, times the scaling factor; f = sum_e weight_e * expert_e(h).  The
reference's own lfm3 has no experts (src/dense.rs:187-191); its other architecture routes by
softmax and adds a shared expert (src/cpu_ref.rs:239-263), which this is not.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import FEED_FORWARDS
from .base import BIAS, MATRIX, VECTOR, BuildEnv, FeedForward, TensorSpec


def fuse_gate_up(w1: torch.Tensor, w3: torch.Tensor, interleave: bool) -> torch.Tensor:
    """[F, D] x 2 -> [2F, D]: gate rows then up rows, or blocks of 16 gate / 16 up alternating."""
    F_, D = w1.shape
    if not interleave:
        return torch.cat([w1, w3], dim=0).contiguous()
    g = w1.reshape(F_ // 16, 16, D)
    u = w3.reshape(F_ // 16, 16, D)
    return torch.stack([g, u], dim=1).reshape(2 * F_, D).contiguous()


_ACTIVATIONS = {"silu": kernels.SILU, "gelu_tanh": kernels.GELU_TANH, "clamped_sigmoid": kernels.CLAMPED_SIGMOID}


@FEED_FORWARDS.register("swiglu", "gated_dense")
class SwiGLU(FeedForward):
    """f = W_down (act(W_gate h) * (W_up h)); act is silu (SwiGLU) unless `activation` names another
    ("gelu_tanh": z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))); "clamped_sigmoid" with `limit` and `alpha`:
    g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit), y = g * sigmoid(alpha * g) * (u + 1)).
    `names`: the three tensors' names under the part's prefix, (gate, up, down)."""
    split_norm = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 names: tuple[str, str, str] = ("w1.weight", "w3.weight", "w2.weight"),
                 limit: float = 0.0, alpha: float = 1.0):
        self.D, self.F = int(hidden_size), int(intermediate_size)
        if activation not in _ACTIVATIONS:
            raise ValueError(f"unknown feed-forward activation '{activation}' ({', '.join(sorted(_ACTIVATIONS))})")
        if activation == "clamped_sigmoid" and not limit > 0:
            raise ValueError(f"the clamped activation needs a positive limit, got {limit}")
        self.activation = activation
        self.act = _ACTIVATIONS[activation]
        self.limit, self.alpha = float(limit), float(alpha)
        self.n_gate, self.n_up, self.n_down = (str(n) for n in names)
        self.w13 = self.w2 = None
        self.fused = False

    def tensors(self) -> dict[str, TensorSpec]:
        return {self.n_gate: TensorSpec((self.F, self.D), MATRIX),
                self.n_up: TensorSpec((self.F, self.D), MATRIX),
                self.n_down: TensorSpec((self.D, self.F), MATRIX)}

    def load(self, tensors, env: BuildEnv) -> None:
        # the gated epilogue with this part's activation (None: the activation has no fused form)
        self.epilogue = kernels.gated_epilogue(self.act, self.limit, self.alpha)
        self.fused = (not env.is_float32) and self.F % 16 == 0 and self.D % 8 == 0 and self.epilogue is not None
        self.w13 = fuse_gate_up(tensors[self.n_gate], tensors[self.n_up], self.fused)
        self.w2 = tensors[self.n_down].contiguous()

    def split_reader_weight(self):
        return self.w13

    def forward(self, h, out, accumulate, batch, env) -> None:
        M = h.shape[0]
        ws = env.workspace
        scale, emit = env.take_split_in(), env.take_split_out()
        a = ws.get("ffn.a", (M, self.F), env.dtype)
        if self.fused:
            kernels.linear(a, h, self.w13, self.epilogue, scale=scale)
        else:
            gu = ws.get("ffn.gu", (M, 2 * self.F), torch.float32)
            kernels.linear(gu, h, self.w13, scale=scale)
            if self.act == kernels.SILU:
                kernels.swiglu(a, gu)
            else:
                kernels.gated_act(a, gu, self.act, self.limit, self.alpha)
        kernels.linear(out, a, self.w2, kernels.ACCUMULATE if accumulate else kernels.STORE,
                       emit=emit if accumulate else None)


@FEED_FORWARDS.register("dense")
class DenseFeedForward(FeedForward):
    """f = W_down act(W_up h) without a gate; act is the erf form of gelu unless `activation` names another
    ("relu_squared": max(z, 0)^2; "gelu_tanh"; "silu").  The up projection's float sums go through the
    activation in float: in the product's epilogue in a decode step, in a launch of its own otherwise.
    `names`: (up, down)."""

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "gelu",
                 names: tuple[str, str] = ("up", "down")):
        if activation not in kernels.PLAIN_ACTIVATIONS:
            raise ValueError(f"unknown feed-forward activation '{activation}' ({', '.join(sorted(kernels.PLAIN_ACTIVATIONS))})")
        self.D, self.F = int(hidden_size), int(intermediate_size)
        self.act = kernels.PLAIN_ACTIVATIONS[activation]
        self.n_up, self.n_down = (str(n) for n in names)
        self.w1 = self.w2 = None

    def tensors(self) -> dict[str, TensorSpec]:
        return {self.n_up: TensorSpec((self.F, self.D), MATRIX), self.n_down: TensorSpec((self.D, self.F), MATRIX)}

    def load(self, tensors, env: BuildEnv) -> None:
        self.w1 = tensors[self.n_up].contiguous()
        self.w2 = tensors[self.n_down].contiguous()

    def forward(self, h, out, accumulate, batch, env) -> None:
        M = h.shape[0]
        ws = env.workspace
        a = ws.get("ffn.a", (M, self.F), env.dtype)
        if kernels.stream_takes_plain_act(h, self.w1, M):
            # a decode step: the weight stream applies the activation to its float sums before it stores
            kernels.linear(a, h, self.w1, kernels.plain_act_epilogue(self.act))
        else:
            u = ws.get("ffn.u", (M, self.F), torch.float32)
            kernels.linear(u, h, self.w1)
            kernels.activation(a, u, self.act)
        kernels.linear(out, a, self.w2, kernels.ACCUMULATE if accumulate else kernels.STORE)


@FEED_FORWARDS.register("sigmoid_topk_moe", "topk_moe")
class SigmoidTopKMoE(FeedForward):
    """Top-k experts of the gated shape.  Defaults: the sigmoid router described at the top of this file and
    SwiGLU experts under the names `gate.weight`, `expert_bias`, `experts.<e>.w1/w3/w2.weight`.

    `router="softmax_chosen"`: logits z = Wr h + bias (the bias is part of the logit), the k largest are
    chosen (ties to the lower index) and weighted by the softmax over the chosen logits alone.
    `activation="clamped_sigmoid"` with `limit` and `alpha`: g = min(W_gate h, limit),
    u = clamp(W_up h, -limit, limit), y = g * sigmoid(alpha * g) * (u + 1).
    `router="softmax_grouped"` with `groups=(count, keep)`: scores s = softmax(Wr h) over all experts; choice
    scores s + bias (the bias chooses, it does not weigh); the experts form `count` equal groups of neighbours,
    a group's score is its largest choice score, and only experts of the `keep` best groups can be chosen (the
    others' choice scores count as minus infinity); weights are the chosen s over their sum (+ 1e-20).
    `router="sigmoid_grouped"` with `groups=(count, keep)` and `group_top`: sigmoid scores, the bias only chooses,
    groups as above but a group's score is the sum of its `group_top` largest choice scores; weights are the
    chosen s over their sum (+ 1e-20), times `scaling`.
    `gated=False`: experts of the plain shape W_down act(W_up h) (no gate tensors) with `activation` one of
    "gelu" (erf form), "relu_squared", "gelu_tanh", "silu".
    `shared_size` > 0: one more expert of that width and the same activation runs for every row and is added
    (tensors "shared_gate"/"shared_up"/"shared_down").
    `names`: "router", "bias", and "gate"/"up"/"down" with `{e}` standing for the expert's number."""

    def __init__(self, hidden_size: int, num_experts: int, top_k: int, expert_size: int,
                 norm_topk: bool = True, use_bias: bool = True, scaling: float = 1.0,
                 bias_std: float = 0.1, router: str = "sigmoid", activation: str = "silu",
                 limit: float = 0.0, alpha: float = 1.0, names: dict[str, str] | None = None,
                 groups: tuple[int, int] | None = None, shared_size: int = 0, gated: bool = True,
                 group_top: int = 1):
        if not 1 <= top_k <= min(num_experts, 16):
            raise ValueError(f"top-{top_k} of {num_experts} experts: the router takes 1..min(experts, 16)")
        if num_experts > 256:
            raise ValueError(f"{num_experts} experts: the router takes at most 256")
        if router not in ("sigmoid", "softmax_chosen", "softmax_grouped", "sigmoid_grouped"):
            raise ValueError(f"unknown router '{router}' (sigmoid, softmax_chosen, softmax_grouped, sigmoid_grouped)")
        self.groups = None
        self.group_top = int(group_top)
        if not 1 <= self.group_top <= 15:
            raise ValueError(f"a group is ranked by its 1..15 best scores, got {group_top}")
        self.gated = bool(gated)
        if router in ("softmax_grouped", "sigmoid_grouped"):
            count, keep = (int(groups[0]), int(groups[1])) if groups is not None else (1, 1)
            if not (1 <= keep <= count <= 255 and num_experts % count == 0 and keep * (num_experts // count) >= top_k):
                raise ValueError(f"{keep} of {count} groups over {num_experts} experts cannot give {top_k} choices")
            self.groups = (count, keep)
        elif groups is not None:
            raise ValueError("groups of experts go with the softmax_grouped and sigmoid_grouped routers")
        known = _ACTIVATIONS if self.gated else kernels.PLAIN_ACTIVATIONS
        if activation not in known:
            raise ValueError(f"unknown expert activation '{activation}' ({', '.join(sorted(known))})")
        if not self.gated and shared_size:
            raise NotImplementedError("a shared expert beside experts without a gate")
        if activation == "clamped_sigmoid" and not limit > 0:
            raise ValueError(f"the clamped activation needs a positive limit, got {limit}")
        self.D, self.E, self.k, self.Fe = int(hidden_size), int(num_experts), int(top_k), int(expert_size)
        self.norm_topk, self.use_bias, self.scaling = bool(norm_topk), bool(use_bias), float(scaling)
        self.bias_std = float(bias_std)
        self.router, self.act = router, known[activation]
        self.limit, self.alpha = float(limit), float(alpha)
        self.n = {"router": "gate.weight", "bias": "expert_bias", "gate": "experts.{e}.w1.weight",
                  "up": "experts.{e}.w3.weight", "down": "experts.{e}.w2.weight"}
        self.n.update({"shared_gate": "shared.gate", "shared_up": "shared.up", "shared_down": "shared.down"})
        self.n.update(names or {})
        self.router_w = self.router_b = self.w13 = self.w2 = None
        self.fused = False
        self.shared = None
        if shared_size:
            self.shared = SwiGLU(hidden_size, shared_size, activation,
                                 (self.n["shared_gate"], self.n["shared_up"], self.n["shared_down"]), limit, alpha)

    def tensors(self) -> dict[str, TensorSpec]:
        n = self.n
        t = {n["router"]: TensorSpec((self.E, self.D), VECTOR)}
        if self.shared is not None:
            t.update(self.shared.tensors())
        if self.use_bias:
            t[n["bias"]] = TensorSpec((self.E,), BIAS, std=self.bias_std)
        for e in range(self.E):
            if self.gated:
                t[n["gate"].format(e=e)] = TensorSpec((self.Fe, self.D), MATRIX)
            t[n["up"].format(e=e)] = TensorSpec((self.Fe, self.D), MATRIX)
            t[n["down"].format(e=e)] = TensorSpec((self.D, self.Fe), MATRIX)
        return t

    def load(self, tensors, env: BuildEnv) -> None:
        n = self.n
        # the products' gated epilogue knows silu, gelu and the clamped form with the slope 1.702 and a limit
        # that bfloat16 holds exactly; anything else runs as a kernel of its own on the float gate and up values
        self.router_w = tensors[n["router"]].contiguous()
        self.router_b = tensors[n["bias"]].contiguous() if self.use_bias else None
        if not self.gated:
            self.epilogue, self.fused = None, False
            self.w13 = torch.stack([tensors[n["up"].format(e=e)] for e in range(self.E)]).contiguous()
            self.w2 = torch.stack([tensors[n["down"].format(e=e)] for e in range(self.E)]).contiguous()
            return
        self.epilogue = kernels.gated_epilogue(self.act, self.limit, self.alpha)
        self.fused = (not env.is_float32) and self.Fe % 16 == 0 and self.D % 8 == 0 and self.epilogue is not None
        self.w13 = torch.stack([fuse_gate_up(tensors[n["gate"].format(e=e)], tensors[n["up"].format(e=e)],
                                             self.fused) for e in range(self.E)]).contiguous()
        self.w2 = torch.stack([tensors[n["down"].format(e=e)] for e in range(self.E)]).contiguous()
        if self.shared is not None:
            self.shared.load(tensors, env)

    def flops_per_row(self) -> int:
        # the router, k experts of three matrices, and the shared expert
        return 2 * self.D * self.E + self.k * (6 if self.gated else 4) * self.D * self.Fe \
            + (self.shared.flops_per_row() if self.shared else 0)

    def unread_weight_bytes(self, rows: int) -> float:
        """With uniform routing an expert is chosen by none of `rows` rows with probability (1 - k/E)^rows."""
        if self.w13 is None:
            return 0.0
        per_expert = (self.w13[0].numel() + self.w2[0].numel()) * self.w13.element_size()
        return self.E * per_expert * (1.0 - self.k / self.E) ** rows

    def forward(self, h, out, accumulate, batch, env) -> None:
        M = h.shape[0]
        P = M * self.k
        ws = env.workspace
        ids = ws.get("moe.ids", (M, self.k), torch.int32)
        wts = ws.get("moe.w", (M, self.k), torch.float32)
        kernels.moe_router(ids, wts, h, self.router_w, self.router_b, self.norm_topk, self.scaling,
                           softmax_chosen=self.router == "softmax_chosen",
                           softmax_groups=self.groups if self.router == "softmax_grouped" else None,
                           sigmoid_groups=(*self.groups, self.group_top) if self.router == "sigmoid_grouped" else None)
        offsets = ws.get("moe.offsets", (self.E + 1,), torch.int32)
        sorted_pair = ws.get("moe.sorted", (P,), torch.int32)
        pair_row = ws.get("moe.rows", (P,), torch.int32)
        kernels.moe_align(offsets, sorted_pair, pair_row, ids, self.E)
        xs = ws.get("moe.xs", (P, self.D), env.dtype)
        kernels.gather_rows(xs, h, sorted_pair, div=self.k)
        a = ws.get("moe.a", (P, self.Fe), env.dtype)
        if not self.gated and kernels.stream_takes_plain_act(xs, self.w13, P, n_groups=self.E):
            kernels.linear(a, xs, self.w13, kernels.plain_act_epilogue(self.act), group_offsets=offsets, rows_hint=P)
        elif not self.gated:
            u = ws.get("moe.gu", (P, self.Fe), torch.float32)
            kernels.linear(u, xs, self.w13, group_offsets=offsets, rows_hint=P)
            kernels.activation(a, u, self.act)
        elif self.fused:
            kernels.linear(a, xs, self.w13, self.epilogue, group_offsets=offsets, rows_hint=P)
        else:
            gu = ws.get("moe.gu", (P, 2 * self.Fe), torch.float32)
            kernels.linear(gu, xs, self.w13, group_offsets=offsets, rows_hint=P)
            if self.act == kernels.SILU:
                kernels.swiglu(a, gu)
            else:
                kernels.gated_act(a, gu, self.act, self.limit, self.alpha)
        ys = ws.get("moe.ys", (P, self.D), torch.float32)
        kernels.linear(ys, a, self.w2, group_offsets=offsets, rows_hint=P)
        kernels.moe_combine(out, ys, pair_row, wts, accumulate)
        if self.shared is not None:
            self.shared.forward(h, out, True, batch, env)
