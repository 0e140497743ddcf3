"""A per-layer input looked up by token id: every layer owns a slice of one wide table.

``e = table[token][col0 : col0 + dim]``; ``g = act(W_gate x) * e`` with ``x`` the stream's current
value; the result is ``W_proj g`` (``[T, hidden]``), which the block adds to the stream (usually
through a norm of its own). The table is one tensor shared by all layers, named without the layer's
prefix; layer ``i`` of ``n`` reads columns ``[i * dim, (i + 1) * dim)``.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from .base import EVERY_STEP, TOKEN_INPUTS, StepContext, TensorSpec, TokenInput


class GatedTokenTable(TokenInput):
    recordable = EVERY_STEP

    def __init__(self, prefix: str, table_name: str, vocab_size: int, hidden_size: int, dim: int, index: int, count: int,
                 activation: str = "gelu_tanh", names: "Mapping[str, str] | None" = None) -> None:
        if not 0 <= index < count or dim <= 0:
            raise ValueError(f"slice {index} of {count} with {dim} columns")
        if activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"activation {activation!r}: 'silu' or 'gelu_tanh'")
        self.prefix, self.table_name = prefix, table_name
        self.vocab_size, self.h, self.dim = int(vocab_size), int(hidden_size), int(dim)
        self.index, self.count, self.activation = int(index), int(count), activation
        self.names = {"gate": "gate", "proj": "proj", **(names or {})}

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p, n = prefix + self.prefix, self.names
        return [TensorSpec(self.table_name, (self.vocab_size, self.count * self.dim)),
                TensorSpec(p + n["gate"], (self.dim, self.h)),
                TensorSpec(p + n["proj"], (self.h, self.dim))]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = prefix + self.prefix, self.names
        self.table = tensors[self.table_name]
        self.w_gate, self.w_proj = tensors[p + n["gate"]], tensors[p + n["proj"]]

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        t, arena = x.shape[0], ctx.arena
        pre = arena.take((t, self.dim), ctx.dtype)
        ops.gemm(x, self.w_gate, pre)
        gated = arena.take((t, self.dim), ctx.dtype)
        ops.act_mul_gather(pre, ctx.tokens, self.table, self.index * self.dim, gated, self.activation)
        out = arena.take((t, self.h), ctx.dtype)
        ops.gemm(gated, self.w_proj, out)
        return out


TOKEN_INPUTS.register("gated_token_table", GatedTokenTable)
