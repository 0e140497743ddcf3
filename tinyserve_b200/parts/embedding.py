"""Token embedding (a row gather with no scaling, upstream src/tinyserve/model.py:192) and
the output head (``logits = float32(x W^T)`` with ``W`` the embedding table when tied,
src/tinyserve/model.py:129-130,208).
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from .base import EMBEDDINGS, EVERY_STEP, HEADS, Part, StepContext, TensorSpec


class TokenEmbedding(Part):
    recordable = EVERY_STEP

    def __init__(self, name: str, vocab_size: int, hidden_size: int, scale: float = 1.0) -> None:
        # scale: the gathered row is multiplied by it on its way into the 32-bit stream
        self.name, self.vocab_size, self.hidden_size = name, int(vocab_size), int(hidden_size)
        self.scale = float(scale)
        self.table: torch.Tensor | None = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(prefix + self.name, (self.vocab_size, self.hidden_size))]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[prefix + self.name]

    def forward(self, ctx: StepContext) -> torch.Tensor:
        """The 32-bit residual stream ``[T, hidden]`` of this step's tokens."""
        out = ctx.arena.take((ctx.num_tokens, self.hidden_size), torch.float32)
        ops.embed(ctx.tokens, self.table, out, self.scale)
        return out


class PositionedEmbedding(Part):
    """Token embedding plus a learned position row, optionally followed by an RMS norm with a plain
    weight: ``x = table[token] * scale + positions[p]``, then ``x / sqrt(mean(x^2) + eps) * w``. One
    kernel writes the result into the 32-bit stream. Positions count from 0 in each request; a
    position beyond the table gives a row of NaN."""

    recordable = EVERY_STEP

    def __init__(self, name: str, vocab_size: int, hidden_size: int, position_name: str, max_positions: int,
                 norm_name: str | None = None, eps: float = 1e-6, scale: float = 1.0) -> None:
        self.name, self.vocab_size, self.hidden_size = name, int(vocab_size), int(hidden_size)
        self.position_name, self.max_positions = position_name, int(max_positions)
        self.norm_name, self.eps, self.scale = norm_name, float(eps), float(scale)
        self.table = self.positions = self.norm_w = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        specs = [TensorSpec(prefix + self.name, (self.vocab_size, self.hidden_size)),
                 TensorSpec(prefix + self.position_name, (self.max_positions, self.hidden_size))]
        if self.norm_name is not None:
            specs.append(TensorSpec(prefix + self.norm_name, (self.hidden_size,), init="one_plus_normal"))
        return specs

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table, self.positions = tensors[prefix + self.name], tensors[prefix + self.position_name]
        self.norm_w = None if self.norm_name is None else tensors[prefix + self.norm_name]

    def forward(self, ctx: StepContext) -> torch.Tensor:
        out = ctx.arena.take((ctx.num_tokens, self.hidden_size), torch.float32)
        ops.embed_pos_norm(ctx.tokens, ctx.positions, self.table, self.positions, self.norm_w, self.eps, out, self.scale)
        return out


class LMHead(Part):
    recordable = EVERY_STEP

    def __init__(self, name: str, tied: bool, vocab_size: int, hidden_size: int,
                 ignored_when_tied: str | None = None, softcap: float | None = None) -> None:
        # softcap: logits <- softcap * tanh(logits / softcap) after the product (None: no cap)
        if softcap is not None and not softcap > 0:
            raise ValueError(f"softcap must be positive or None, got {softcap}")
        self.softcap = None if softcap is None else float(softcap)
        self.name, self.tied = name, bool(tied)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.ignored_when_tied = ignored_when_tied
        self.weight: torch.Tensor | None = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        # When tied this names the embedding table, which the embedding declares as well;
        # equal declarations are one tensor.
        return [TensorSpec(prefix + self.name, (self.vocab_size, self.hidden_size))]

    def ignorable_tensors(self, prefix: str) -> set[str]:
        # A tied checkpoint may still ship a copy of the table under the head's name.
        return {prefix + self.ignored_when_tied} if self.tied and self.ignored_when_tied else set()

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[prefix + self.name]

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``x [R, hidden]`` in the model dtype -> ``out [R, vocab]`` float32."""
        ops.gemm(x, self.weight, out)
        if self.softcap is not None:
            ops.softcap(out, self.softcap)
        return out


EMBEDDINGS.register("token_embedding", TokenEmbedding)
EMBEDDINGS.register("positioned_embedding", PositionedEmbedding)
HEADS.register("lm_head", LMHead)
