"""The Kisilix decoder as a plan.

x = embed[token] + pos[p] with a learned vector per position p (counted from 0 in each sequence).  A layer is
the post-norm arrangement (parts.block): x <- LN1(alpha x + mixer(x)) and, where the layer has a feed-forward,
x <- LN2(alpha x + ff(x)); the sublayers read the stream itself, the norms are layer norms with weight and bias.
Mixers, chosen layer by layer: the gated delta rule with a decay per key channel and the state-space (SSD)
layer (parts.recurrent), or windowed attention with pooled blocks behind the window, biases, weighted RMS
norms on q and k, a partial split-half rotation, rotated values and a temperature per head
(parts.pooled_attention).  Feed-forwards: the dense clamped form y = g sigmoid(1.702 g) (u + 1) with
g = min(gate, limit), u = clamp(up, -limit, limit); or a mixture of silu-gated experts chosen by a softmax
router with a correction that only chooses, limited to the best groups of neighbouring experts, plus a shared
expert.  The model's layer norm, then logits against the head's own matrix.

Tensor names: embed, pos, head, final.norm(.b), and per layer l<i>.norm1(.b), l<i>.norm2(.b), l<i>.mix.*
(the mixers' own names) and l<i>.mlp.{gate,up,down} or l<i>.mlp.{router, correction, e<j>.gate/up/down,
shared.gate/up/down}.
"""
from __future__ import annotations

import re

from ..config.kisilix import ATTENTION, CHANNEL_DELTA, MAMBA2, DenseSizes, KisilixConfig
from ..parts.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from ..registry import ARCHITECTURES

NAMES = ("Kisilix", "kisilix")
POSITION_TABLE = "pos"

DENSE_SIGMOID_SLOPE = 1.702      # the design's constant in g * sigmoid(1.702 g)
UNIT_NORM_EPS = 1e-6             # inside the root of the delta mixer's unit norms

# names that are a part's prefix in the plan and a tensor in the checkpoint
_BARE = re.compile(r"^(embed|head)$")


def _alias(name: str) -> str:
    return name + ".weight" if _BARE.match(name) else name


def _checkpoint_name(canonical: str) -> str:
    return canonical[: -len(".weight")] if canonical.endswith(".weight") and _BARE.match(canonical[: -len(".weight")]) \
        else canonical


def kisilix_plan(cfg: KisilixConfig) -> ModelPlan:
    W = cfg.width
    norm = PartSpec("layernorm", {"size": W, "eps": cfg.eps, "tensor": "", "bias": True, "bias_tensor": "b"})
    layers: list[LayerSpec] = []
    for i, lay in enumerate(cfg.layers):
        m = lay.mixer
        if lay.type == CHANNEL_DELTA:
            mixer = PartSpec("gated_delta_rule", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "v_head_dim": m.vdim, "conv_taps": m.conv, "norm_eps": cfg.eps, "unit_eps": UNIT_NORM_EPS})
        elif lay.type == MAMBA2:
            mixer = PartSpec("state_space", {
                "hidden_size": W, "num_heads": m.heads, "v_head_dim": m.vdim, "state_size": m.state,
                "num_groups": m.groups, "norm_groups": m.norm_groups, "conv_taps": m.conv, "norm_eps": cfg.eps})
        else:
            assert lay.type == ATTENTION
            position = PartSpec("rope", {"rope_dim": m.rot.dims, "theta": m.rot.base, "style": "neox"}) \
                if m.rot is not None and m.rot.dims else PartSpec("none")
            mixer = PartSpec("pooled_window_attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "v_head_dim": m.vdim, "norm_eps": cfg.eps, "scale": m.scale, "window": m.window, "pool": m.pool,
                "position": position, "value_rotation_base": None if m.rot is None else m.rot.base})
        ffn = None
        f = lay.mlp
        if isinstance(f, DenseSizes):
            ffn = PartSpec("gated_dense", {
                "hidden_size": W, "intermediate_size": f.ff, "activation": "clamped_sigmoid", "limit": f.limit,
                "alpha": DENSE_SIGMOID_SLOPE, "names": ("gate", "up", "down")})
        elif f is not None:
            ffn = PartSpec("topk_moe", {
                "hidden_size": W, "num_experts": f.experts, "top_k": f.top, "expert_size": f.ff,
                "router": "softmax_grouped", "groups": (f.groups, f.keep), "use_bias": True, "activation": "silu",
                "shared_size": f.shared_ff,
                "names": {"router": "router", "bias": "correction", "gate": "e{e}.gate", "up": "e{e}.up",
                          "down": "e{e}.down"}})
        layers.append(LayerSpec(
            prefix=f"l{i}", mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=None if ffn is None else norm,
            block="post_norm_residual", block_params={"alpha": cfg.alpha},
            names={"mixer": "mix", "ffn": "mlp", "mixer_norm": "norm1", "ffn_norm": "norm2"}))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=W, vocab_size=cfg.vocab,
        embedding=PartSpec("token_position_embedding", {"vocab_size": cfg.vocab, "hidden_size": W,
                                                        "max_positions": cfg.max_positions,
                                                        "position_tensor": POSITION_TABLE}),
        final_norm=norm,
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": False}),
        layers=layers, schedule=[ScheduleEntry(i) for i in range(len(layers))],
        names={"embedding": "embed", "final_norm": "final.norm", "head": "head"},
        tensor_aliases=_alias, checkpoint_names=_checkpoint_name, max_positions=cfg.max_positions,
        # sizes that keep the signal of random weights alive through the norms after every sum
        init_std=0.05, init_stds={".router": 0.3, ".correction": 0.02, POSITION_TABLE: 0.5})


@ARCHITECTURES.register(*NAMES)
def build_kisilix(raw: dict) -> ModelPlan:
    return kisilix_plan(KisilixConfig.from_dict(raw))
