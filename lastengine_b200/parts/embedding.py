"""Token embedding and output head.

x = embed[token] (src/dense.rs:172-177), times a constant where the design has one; logits = W_out . norm(x) with W_out the head's own
matrix, or the embedding when the model ties them (src/dense.rs:195-196).  Logits are float.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import EMBEDDINGS, HEADS
from .base import EMBEDDING, MATRIX, VECTOR, BuildEnv, Part, TensorSpec


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0):
        """`scale` multiplies the row on its way into the residual stream; the table itself (which a
        tied output head multiplies with) stays as stored."""
        self.V, self.D = int(vocab_size), int(hidden_size)
        self.scale = float(scale)
        self.weight: torch.Tensor | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.V, self.D), EMBEDDING)}

    def load(self, tensors, env: BuildEnv) -> None:
        self.weight = tensors["weight"].contiguous()

    def forward(self, x: torch.Tensor, tokens: torch.Tensor, batch=None) -> None:
        kernels.embed(x, self.weight, tokens, self.scale)


@EMBEDDINGS.register("token_position_embedding")
class TokenPositionEmbedding(TokenEmbedding):
    """x = embed[token] * scale + positions[p]: a learned vector per position p (counted from 0 in each
    sequence, not scaled) beside the token's row.  The table of `max_positions` rows is the tensor
    `position_tensor` of the model (not under the part's prefix); the plan's `max_positions` makes the engine
    refuse a step that would go beyond it."""

    def __init__(self, vocab_size: int, hidden_size: int, max_positions: int, position_tensor: str = "positions",
                 scale: float = 1.0):
        super().__init__(vocab_size, hidden_size, scale)
        self.P = int(max_positions)
        self.position_tensor = str(position_tensor)
        self.positions: torch.Tensor | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        t = super().tensors()
        t["positions"] = TensorSpec((self.P, self.D), VECTOR, shared_name=self.position_tensor)
        return t

    def load(self, tensors, env: BuildEnv) -> None:
        super().load(tensors, env)
        self.positions = tensors["positions"].to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, tokens: torch.Tensor, batch=None) -> None:
        if batch is None:
            raise ValueError("an embedding with learned positions needs the step's positions")
        kernels.embed_positions(x, None, self.weight, tokens, self.positions, batch.row_pos, self.scale)


@HEADS.register("linear_head")
class LinearHead(Part):
    def __init__(self, vocab_size: int, hidden_size: int, tied: bool):
        self.V, self.D, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.weight: torch.Tensor | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        return {} if self.tied else {"weight": TensorSpec((self.V, self.D), MATRIX)}

    def load(self, tensors, env: BuildEnv) -> None:
        if not self.tied:
            self.weight = tensors["weight"].contiguous()

    def tie(self, embedding: TokenEmbedding) -> None:
        self.weight = embedding.weight

    def flops_per_row(self) -> int:
        return 2 * self.V * self.D

    def forward(self, logits: torch.Tensor, xn: torch.Tensor) -> None:
        kernels.linear(logits, xn, self.weight)
