"""The Tevilix decoder as a plan.

x = embed[token] * scale.  A layer is the parallel arrangement with a norm per sublayer (parts.block):
x <- x + mixer(LN1(x)) + ff(LN2(x)), both norms of the same x, layer norms with a weight and no bias.  Mixers,
chosen layer by layer: two mixers side by side (parts.composite), a * attention + b * minimal gated recurrent
unit, where the attention (parts.mixed_attention) has biases, weighted RMS norms on q and k, a partial
split-half rotation with linear position scaling, scores mixed across heads before the softmax, a sliding
window and an output gate; or the matrix memory with exponential gates (parts.gated_scan, mlstm).
Feed-forwards: dense down(gelu(up h)) with the erf form, or a mixture of experts down(relu(up h)^2) chosen by a
sigmoid router with a correction that only chooses, limited to the best groups of neighbouring experts (a
group ranks by the sum of its two best choice scores), weights over their sum times a constant.  A range of
layers may run several times in a row with the same weights, every run with a cache entry of its own.  The
model's layer norm, then logits against the head's own matrix.

Tensor names: embed, head, final.norm, and per layer l<i>.norm1, l<i>.norm2, l<i>.mix.* (left.* and right.* of
the parallel mixer; the mlstm's own names) and l<i>.mlp.{up,down} or l<i>.mlp.{router, correction, e<j>.up/down}.
"""
from __future__ import annotations

import re

from ..config.tevilix import MLSTM, PARALLEL, DenseSizes, TevilixConfig
from ..parts.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from ..registry import ARCHITECTURES

NAMES = ("Tevilix", "tevilix")

GROUP_RANK_TOP = 2       # a group of experts ranks by the sum of this many of its best choice scores

# names that are a part's prefix in the plan and a tensor in the checkpoint
_BARE = re.compile(r"^(embed|head)$")


def _alias(name: str) -> str:
    return name + ".weight" if _BARE.match(name) else name


def _checkpoint_name(canonical: str) -> str:
    return canonical[: -len(".weight")] if canonical.endswith(".weight") and _BARE.match(canonical[: -len(".weight")]) \
        else canonical


def tevilix_plan(cfg: TevilixConfig) -> ModelPlan:
    W = cfg.width
    norm = PartSpec("layernorm", {"size": W, "eps": cfg.eps, "tensor": ""})
    layers: list[LayerSpec] = []
    for i, lay in enumerate(cfg.layers):
        m = lay.mixer
        if lay.type == PARALLEL:
            a = m.left
            position = PartSpec("rope", {"rope_dim": a.rot.dims, "theta": a.rot.base, "style": "neox",
                                         "scaling_factor": a.rot.factor}) if a.rot.dims else PartSpec("none")
            mixer = PartSpec("parallel_mixers", {
                "left": PartSpec("mixed_heads_attention", {
                    "hidden_size": W, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
                    "v_head_dim": a.vdim, "norm_eps": cfg.eps, "scale": a.scale, "window": a.window,
                    "position": position}),
                "right": PartSpec("min_gru", {"hidden_size": W, "width": m.right_width}),
                "left_scale": m.left_scale, "right_scale": m.right_scale})
        else:
            assert lay.type == MLSTM
            mixer = PartSpec("mlstm", {"hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                                       "gate_cap": m.gate_cap, "norm_eps": cfg.eps})
        ffn = None
        f = lay.mlp
        if isinstance(f, DenseSizes):
            ffn = PartSpec("dense", {"hidden_size": W, "intermediate_size": f.ff, "activation": "gelu"})
        elif f is not None:
            ffn = PartSpec("topk_moe", {
                "hidden_size": W, "num_experts": f.experts, "top_k": f.top, "expert_size": f.ff,
                "router": "sigmoid_grouped", "groups": (f.groups, f.keep), "group_top": GROUP_RANK_TOP,
                "use_bias": True, "scaling": f.scale, "gated": False, "activation": "relu_squared",
                "names": {"router": "router", "bias": "correction", "up": "e{e}.up", "down": "e{e}.down"}})
        layers.append(LayerSpec(
            prefix=f"l{i}", mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=None if ffn is None else norm,
            block="parallel_residual",
            names={"mixer": "mix", "ffn": "mlp", "mixer_norm": "norm1", "ffn_norm": "norm2"}))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=W, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "scale": cfg.embedding_scale}),
        final_norm=norm,
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": False}),
        layers=layers, schedule=[ScheduleEntry(layer) for layer in cfg.runs()],
        names={"embedding": "embed", "final_norm": "final.norm", "head": "head"},
        tensor_aliases=_alias, checkpoint_names=_checkpoint_name,
        # sizes that keep the signal of random weights alive through the sums of a looped model
        init_std=0.05, init_stds={".router": 0.3, ".correction": 0.02, ".talk": 0.5})


@ARCHITECTURES.register(*NAMES)
def build_tevilix(raw: dict) -> ModelPlan:
    return tevilix_plan(TevilixConfig.from_dict(raw))
