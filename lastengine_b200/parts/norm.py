"""Norms.  RMSNorm: y = x / sqrt(mean(x^2) + eps) * w  (src/dense.rs:27-30); layer norm with a weight
and no bias below it.

`offset`: the weight is stored around zero and the factor is offset + w (1 + w in the designs that
store it so); it is added once, in float, when the weights are loaded.  `tensor`: the weight's name
under the part's prefix ("" where the prefix itself names it)."""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import NORMS
from .base import BIAS, NORM, NORM_AROUND_ZERO, BuildEnv, Part, TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Part):
    # y = x * r * w with one factor r per row: a block may leave bfloat16(x * w) to the product
    # before it and r to the product after it (a norm with a mean or a bias could not be split so)
    splittable = True

    def __init__(self, size: int, eps: float, offset: float = 0.0, tensor: str = "weight"):
        self.size = int(size)
        self.eps = float(eps)
        self.offset = float(offset)
        self.tensor = str(tensor)
        self.weight: torch.Tensor | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        # a weight stored around zero starts at zero (the factor is then 1), not at one
        return {self.tensor: TensorSpec((self.size,), NORM if self.offset == 0.0 else NORM_AROUND_ZERO)}

    def load(self, tensors: dict[str, torch.Tensor], env: BuildEnv) -> None:
        w = tensors[self.tensor].to(torch.float32)
        self.weight = (w + self.offset if self.offset != 0.0 else w).contiguous()

    def forward(self, out: torch.Tensor, x: torch.Tensor, rows: torch.Tensor | None = None,
                add: bool = False) -> None:
        """out = norm(x[rows]) (or out += norm(x) with add); x is the float residual or a float buffer."""
        kernels.rmsnorm(out, x, self.weight, self.eps, rows=rows, add=add)


@NORMS.register("layernorm")
class LayerNorm(Part):
    """y = (x - mean(x)) / sqrt(var(x) + eps) * w (+ b) with var the mean of the squared deviations; a weight
    and, with `bias`, an additive term under the name `bias_tensor`.  It takes a mean off the row, so it cannot
    be split between two products as the RMS norm is."""
    splittable = False

    def __init__(self, size: int, eps: float, tensor: str = "weight", bias: bool = False, bias_tensor: str = "bias"):
        self.size = int(size)
        self.eps = float(eps)
        self.tensor = str(tensor)
        self.has_bias, self.bias_tensor = bool(bias), str(bias_tensor)
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        t = {self.tensor: TensorSpec((self.size,), NORM)}
        if self.has_bias:
            t[self.bias_tensor] = TensorSpec((self.size,), BIAS, std=0.1)
        return t

    def load(self, tensors: dict[str, torch.Tensor], env: BuildEnv) -> None:
        self.weight = tensors[self.tensor].to(torch.float32).contiguous()
        self.bias = tensors[self.bias_tensor].to(torch.float32).contiguous() if self.has_bias else None

    def forward(self, out: torch.Tensor, x: torch.Tensor, rows: torch.Tensor | None = None,
                add: bool = False) -> None:
        if add:
            raise NotImplementedError("a layer norm added into the residual stream")
        kernels.layernorm(out, x, self.weight, self.eps, rows=rows, bias=self.bias)
