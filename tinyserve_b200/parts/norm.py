"""RMSNorm over the last dimension, fused with the residual sum that precedes it.

Formula (upstream src/tinyserve/layers.py:35-38): in 32-bit ``y = x * rsqrt(mean(x^2) +
eps)``; ``y`` is cast to the model dtype and THEN multiplied by the weight (a plain weight,
not ``1 + w``). Here ``x`` is the 32-bit residual stream plus the pending sub-layer output,
which the same kernel adds and writes back.

Options serve designs that norm differently: ``round_once`` (the weight is applied in 32-bit too and
the result rounded once), ``unit_offset`` (the weight is stored around
zero and the gain is ``1 + weight``; the whole norm is then 32-bit with one rounding), and
``PostRMSNorm``, a norm on a sub-layer's OUTPUT with an optional per-column layer scale, which
is left pending on the stream and applied by the next norm's kernel in the same pass as the
residual sum: ``x <- x + scale * norm(y)``, then ``norm(x)``; and ``LayerScale``, the per-column scale
alone (``x <- x + scale * y``), pending in the same way.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from .base import EVERY_STEP, LazyNormed, Norm, ResidualStream, StepContext, TensorSpec, register_norm


class RMSNorm(Norm):
    recordable = EVERY_STEP

    def __init__(self, name: str, size: int, eps: float, unit_offset: bool = False, round_once: bool = False) -> None:
        self.name, self.size, self.eps = name, int(size), float(eps)
        self.unit_offset = bool(unit_offset)
        self.round_once = bool(round_once) or self.unit_offset
        self.weight: torch.Tensor | None = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(prefix + self.name, (self.size,), init="normal" if self.unit_offset else "one_plus_normal")]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[prefix + self.name]

    def _run(self, stream: ResidualStream, out: torch.Tensor, rows: torch.Tensor | None) -> None:
        if stream.post is None and not self.round_once:
            ops.add_rms_norm(stream.resid, stream.delta, self.weight, self.eps, out, rows=rows)
            return
        post_w, post_scale, post_eps, post_offset, post_mult, *rest = \
            stream.post if stream.post is not None else (None, None, 0.0, False, 1.0)
        ops.post_norm_add_rms_norm(stream.resid, stream.delta, post_w, post_scale, post_eps, post_offset, self.weight,
                                   self.unit_offset, self.eps, out, rows=rows, post_mult=post_mult,
                                   delta_bias=rest[0] if rest else None)

    def forward(self, stream: ResidualStream, ctx: StepContext) -> torch.Tensor:
        out = ctx.arena.take((stream.resid.shape[0], self.size), ctx.dtype)
        self._run(stream, out, None)
        if stream.delta is not None:
            stream.delta = None
            stream.post = None
            stream.sumsq = None          # the stream has changed
        return out

    def lazy(self, stream: ResidualStream, ctx: StepContext) -> "torch.Tensor | LazyNormed":
        if stream.delta is None and stream.sumsq is not None and not self.round_once:
            return LazyNormed(stream, self.weight, self.eps, lambda: self.forward(stream, ctx))
        return self.forward(stream, ctx)

    def forward_rows(self, stream: ResidualStream, rows: torch.Tensor, num_rows: int,
                     ctx: StepContext) -> torch.Tensor:
        out = ctx.arena.take((num_rows, self.size), ctx.dtype)
        self._run(stream, out, rows)
        return out


class PostRMSNorm(Norm):
    """The norm on a sub-layer's output, with an optional layer scale (one factor per column,
    tensor ``scale_name``) and an optional constant ``mult``: ``leave(stream, y)`` leaves ``y`` pending
    together with this norm, and the next norm's kernel adds ``mult * layer_scale * norm(y)`` to the stream."""

    recordable = EVERY_STEP

    def __init__(self, name: str, size: int, eps: float, unit_offset: bool = False, scale_name: str | None = None,
                 mult: float = 1.0) -> None:
        self.name, self.size, self.eps = name, int(size), float(eps)
        self.unit_offset, self.scale_name, self.mult = bool(unit_offset), scale_name, float(mult)
        self.weight: torch.Tensor | None = None
        self.scale: torch.Tensor | None = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        specs = [TensorSpec(prefix + self.name, (self.size,), init="normal" if self.unit_offset else "one_plus_normal")]
        if self.scale_name is not None:
            specs.append(TensorSpec(prefix + self.scale_name, (self.size,), init="one_plus_normal", std=0.1))
        return specs

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[prefix + self.name]
        self.scale = None if self.scale_name is None else tensors[prefix + self.scale_name]

    def leave(self, stream: ResidualStream, y: torch.Tensor) -> None:
        if stream.delta is not None:
            raise RuntimeError("a sub-layer output is already pending on the stream")
        stream.delta = y
        stream.post = (self.weight, self.scale, self.eps, self.unit_offset, self.mult)
        stream.sumsq = None

    def forward(self, stream: ResidualStream, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError("a post norm is applied by the norm that follows it; use leave()")

    def forward_rows(self, stream, rows, num_rows, ctx):
        raise NotImplementedError("a post norm is applied by the norm that follows it; use leave()")


class LayerScale(Norm):
    """No norm at all on a sub-layer's output, only a learned factor per column (tensor ``name``) and an
    optional constant ``mult``: ``leave(stream, y)`` leaves ``y`` pending with the factor, and the next norm's
    kernel adds ``mult * scale * y`` to the 32-bit stream in the same pass as its own norm. ``leave(stream, y,
    bias)`` takes over the sub-layer's output bias too (``accepts_bias``): the kernel adds ``scale * (y + bias)``."""

    accepts_bias = True

    recordable = EVERY_STEP

    def __init__(self, name: str, size: int, mult: float = 1.0) -> None:
        self.name, self.size, self.mult = name, int(size), float(mult)
        if self.mult != 1.0:
            raise NotImplementedError("a layer scale with a constant beside it")
        self.scale: torch.Tensor | None = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(prefix + self.name, (self.size,), init="one_plus_normal", std=0.1)]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        self.scale = tensors[prefix + self.name]

    def leave(self, stream: ResidualStream, y: torch.Tensor, bias: torch.Tensor | None = None) -> None:
        if stream.delta is not None:
            raise RuntimeError("a sub-layer output is already pending on the stream")
        stream.delta = y
        stream.post = (None, self.scale, 0.0, False, 1.0, bias)
        stream.sumsq = None

    def forward(self, stream: ResidualStream, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError("a layer scale is applied by the norm that follows it; use leave()")

    def forward_rows(self, stream, rows, num_rows, ctx):
        raise NotImplementedError("a layer scale is applied by the norm that follows it; use leave()")


register_norm("layer_scale", LayerScale)
register_norm("rms_norm", RMSNorm)
register_norm("post_rms_norm", PostRMSNorm)
