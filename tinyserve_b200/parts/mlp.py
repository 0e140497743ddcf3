"""Dense gated feed-forward (SwiGLU).

``y = (silu(x Wgate^T) * (x Wup^T)) Wdown^T`` with ``silu(z) = z * sigmoid(z)`` and no
biases (upstream src/tinyserve/layers.py:94-115); gate and up come from one product with
the merged ``[2 * intermediate, hidden]`` matrix, gate rows first
(src/tinyserve/model.py:178-179, src/tinyserve/weights.py:104-129).
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from .base import (EVERY_STEP, FeedForward, LazyNormed, ResidualStream, StepContext, TensorSpec, project, project_to_stream,
                   register_feed_forward)


class SwiGLU(FeedForward):
    recordable = EVERY_STEP

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int) -> None:
        self.prefix = prefix
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p, h, i = prefix + self.prefix, self.hidden_size, self.intermediate_size
        return [
            TensorSpec(p + "gate_up_proj.weight", (2 * i, h),
                       merged_from=(p + "gate_proj.weight", p + "up_proj.weight"),
                       merged_rows=(i, i)),
            TensorSpec(p + "down_proj.weight", (h, i)),
        ]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p = prefix + self.prefix
        self.w_gate_up = tensors[p + "gate_up_proj.weight"]
        self.w_down = tensors[p + "down_proj.weight"]

    takes_lazy_input = True
    adds_to_stream = True

    def streamed_weights(self) -> list[torch.Tensor]:
        return [self.w_gate_up, self.w_down]

    def forward(self, x: "torch.Tensor | LazyNormed", ctx: StepContext,
                stream: ResidualStream | None = None) -> torch.Tensor | None:
        t = x.shape[0]
        act = ctx.arena.take((t, self.intermediate_size), ctx.dtype)
        project(x, self.w_gate_up, act, ctx, swiglu=True)
        return project_to_stream(act, self.w_down, stream, ctx)


class GatedMLP(FeedForward):
    """``y = (act(x Wgate^T) * (x Wup^T)) Wdown^T`` with a choice of activation ("silu",
    "gelu_tanh": ``0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))``; "clamped_swish" with its
    ``limit``: ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``, ``g sigmoid(1.702 g) (u + 1)``
    in place of ``act(gate) * up``) and of tensor names
    (``names``: role "gate" / "up" / "down" -> name after the prefix). Gate and up come from one
    product with the merged matrix, with the activation in the same kernel where the framework
    has one for the step's shape (``ops.gemm_gated``). With ``bias`` every projection has a bias
    (the projection's name with ``.b`` added): those of gate and up are added where the activation is
    applied (inside the product where the framework has such a kernel for the step's shape, ``ops.gemm_biased_swiglu``); the output's is ``output_bias``, which a block that sums the output into the stream
    itself may take over (``forward(..., add_output_bias=False)``)."""

    recordable = EVERY_STEP

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 names: "Mapping[str, str] | None" = None, limit: float | None = None, bias: bool = False) -> None:
        self.bias = bool(bias)
        self.b_gate_up = self.output_bias = None
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not one of {sorted(ops.ACTIVATIONS)}")
        if (activation == "clamped_swish") != (limit is not None) or (limit is not None and not limit > 0):
            raise ValueError("'clamped_swish' takes a positive limit, the other activations none")
        self.prefix, self.activation, self.limit = prefix, activation, 0.0 if limit is None else float(limit)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight", **(names or {})}
        self.w_gate_up = self.w_down = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p, h, i, n = prefix + self.prefix, self.hidden_size, self.intermediate_size, self.names
        specs = [TensorSpec(p + n["gate"] + "+" + n["up"], (2 * i, h), merged_from=(p + n["gate"], p + n["up"]),
                            merged_rows=(i, i)),
                 TensorSpec(p + n["down"], (h, i))]
        if self.bias:
            specs += [TensorSpec(p + n["gate"] + ".b+" + n["up"] + ".b", (2 * i,), merged_from=(p + n["gate"] + ".b", p + n["up"] + ".b"),
                                 merged_rows=(i, i)),
                      TensorSpec(p + n["down"] + ".b", (h,))]
        return specs

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = prefix + self.prefix, self.names
        self.w_gate_up = tensors[p + n["gate"] + "+" + n["up"]]
        self.w_down = tensors[p + n["down"]]
        if self.bias:
            self.b_gate_up = tensors[p + n["gate"] + ".b+" + n["up"] + ".b"]
            self.output_bias = tensors[p + n["down"] + ".b"]

    def streamed_weights(self) -> list[torch.Tensor]:
        return [self.w_gate_up, self.w_down]

    def forward(self, x: torch.Tensor, ctx: StepContext, add_output_bias: bool = True) -> torch.Tensor:
        t = x.shape[0]
        act = ctx.arena.take((t, self.intermediate_size), ctx.dtype)
        if self.bias and self.activation == "silu":
            ops.gemm_biased_swiglu(x, self.w_gate_up, self.b_gate_up, act, ctx.arena)
        elif self.bias:
            gate_up = ctx.arena.take((t, 2 * self.intermediate_size), ctx.dtype)
            ops.gemm(x, self.w_gate_up, gate_up)
            ops.act_mul(gate_up, act, self.activation, self.limit, bias=self.b_gate_up)
        else:
            ops.gemm_gated(x, self.w_gate_up, act, ctx.arena, self.activation, self.limit)
        out = ctx.arena.take((t, self.hidden_size), ctx.dtype)
        ops.gemm(act, self.w_down, out)
        if self.bias and add_output_bias:
            ops.add_bias(out, self.output_bias)
        return out


class RoutedExperts(FeedForward):
    """A mixture of ``num_experts`` small SwiGLU feed-forwards of which each token uses ``top``.

    Router logits ``z = W_router x`` are 32-bit; the ``top`` experts with the largest logits are
    chosen (ties to the lower index) and weighted by the softmax over the chosen logits only; the
    output is the weighted sum of ``W_down,e (silu(W_gate,e x) * (W_up,e x))`` over the chosen
    experts, plus, with ``shared_size``, a SwiGLU expert of that inner size that every token uses.
    Experts have no biases. Tensor names after the prefix: ``router``, ``e<i>.gate|up|down``,
    ``shared.gate|up|down`` (``names`` renames "router", "expert" (a format of the index), "shared",
    "gate", "up", "down", "correction", "shared_gate").

    ``routing="scored"`` chooses differently: the scores are the softmax over ALL router outputs; the
    choice takes the ``top`` largest of ``score + correction`` (``correction=True``: a tensor with one value
    per output) and looks only inside the ``group_keep`` best of ``groups`` equal groups of neighbouring
    outputs (a group's value is its largest choice score); the weights are the chosen scores (without the
    correction) over their sum, times ``route_scale``. ``identity``: that many further router outputs after
    the experts' are identity experts, whose output is the token's input itself; they take part in the
    softmax, the groups and the choice, and have no tensors. ``shared_gate``: the shared expert's output is
    multiplied by ``sigmoid(w_sg . x)``, one value per token (a ``[1, hidden]`` tensor, which rides along
    in the router's product so that it is 32-bit like the router).

    The experts' matrices are stacked (``[E, 2 ff, hidden]`` gate rows then up rows, ``[E, hidden,
    ff]``); tokens are sorted by expert on the device and the products run tile by tile over that
    order (``ops.moe_route`` / ``moe_gemm`` / ``moe_combine``), so a step is the same launches
    whatever the routing and can be recorded."""

    recordable = EVERY_STEP
    _NAMES = {"router": "router", "expert": "e{}.", "shared": "shared.", "gate": "gate", "up": "up", "down": "down",
              "correction": "correction", "shared_gate": "sg"}

    def __init__(self, prefix: str, hidden_size: int, num_experts: int, top: int, expert_size: int,
                 shared_size: int | None = None, names: "Mapping[str, str] | None" = None, routing: str = "top_logits",
                 correction: bool = False, groups: int = 1, group_keep: int = 1, route_scale: float = 1.0,
                 identity: int = 0, shared_gate: bool = False) -> None:
        outputs = int(num_experts) + int(identity)
        if not 0 < top <= min(outputs, 32):
            raise ValueError(f"top={top} must be between 1 and min(router outputs={outputs}, 32)")
        if routing not in ("top_logits", "scored"):
            raise ValueError(f"routing={routing!r}: 'top_logits' or 'scored'")
        if routing != "scored" and (correction or groups != 1 or identity or route_scale != 1.0):
            raise ValueError("a correction, groups, identity experts and a constant on the weights come with routing='scored'")
        if identity < 0 or not 1 <= groups <= 32 or outputs % groups or not 1 <= group_keep <= groups:
            raise ValueError(f"groups={groups} (at most 32) must divide the {outputs} router outputs, and 1 <= group_keep <= groups")
        if outputs // groups * group_keep < top:
            raise ValueError(f"the {group_keep} kept groups of {outputs // groups} outputs hold fewer than top={top}")
        if shared_gate and shared_size is None:
            raise ValueError("a gate on the shared expert needs a shared expert")
        self.scored, self.has_correction, self.groups, self.group_keep = routing == "scored", bool(correction), int(groups), int(group_keep)
        self.route_scale, self.identity, self.shared_gate, self.outputs = float(route_scale), int(identity), bool(shared_gate), outputs
        self.rule = ops.PLAIN_ROUTE
        if expert_size <= 0 or (shared_size is not None and shared_size <= 0):
            raise ValueError("expert sizes must be positive")
        self.prefix, self.h = prefix, int(hidden_size)
        self.experts, self.top, self.ff = int(num_experts), int(top), int(expert_size)
        self.shared_ff = None if shared_size is None else int(shared_size)
        self.names = {**self._NAMES, **(names or {})}
        self.counts: torch.Tensor | None = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p, n, h, ff, e = prefix + self.prefix, self.names, self.h, self.ff, self.experts
        each = [p + n["expert"].format(i) for i in range(e)]
        if self.shared_gate:
            sg = p + n["shared"] + n["shared_gate"]
            router = TensorSpec(p + n["router"] + "+" + n["shared"] + n["shared_gate"], (self.outputs + 1, h),
                                merged_from=(p + n["router"], sg), merged_rows=(self.outputs, 1))
        else:
            router = TensorSpec(p + n["router"], (self.outputs, h))
        specs = [router,
                 TensorSpec(p + "experts.gate+up", (e * 2 * ff, h),
                            merged_from=tuple(x + n[r] for x in each for r in ("gate", "up")), merged_rows=(ff,) * (2 * e)),
                 TensorSpec(p + "experts.down", (e * h, ff), merged_from=tuple(x + n["down"] for x in each),
                            merged_rows=(h,) * e)]
        if self.shared_ff is not None:
            sp, sf = p + n["shared"], self.shared_ff
            specs += [TensorSpec(sp + n["gate"] + "+" + n["up"], (2 * sf, h), merged_from=(sp + n["gate"], sp + n["up"]),
                                 merged_rows=(sf, sf)),
                      TensorSpec(sp + n["down"], (h, sf))]
        if self.has_correction:
            specs.append(TensorSpec(p + n["correction"], (self.outputs,), std=0.05))
        return specs

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = prefix + self.prefix, self.names
        self.w_router = tensors[p + n["router"] + ("+" + n["shared"] + n["shared_gate"] if self.shared_gate else "")]
        if self.scored and self.w_router.shape[0] % 16:
            # zero rows up to a multiple of 16: the few-row product of decode steps takes such matrices
            padded = torch.zeros((-(-self.w_router.shape[0] // 16) * 16, self.h), dtype=self.w_router.dtype, device=self.w_router.device)
            padded[: self.w_router.shape[0]] = self.w_router
            self.w_router = padded
        if self.scored:
            corr = tensors[p + n["correction"]].float().contiguous() if self.has_correction else None
            self.rule = ops.RouteRule(scored=True, groups=self.groups, keep=self.group_keep, scale=self.route_scale,
                                      identity=self.identity, correction=corr)
        self.w_gate_up = tensors[p + "experts.gate+up"].view(self.experts, 2 * self.ff, self.h)
        self.w_down = tensors[p + "experts.down"].view(self.experts, self.h, self.ff)
        if self.shared_ff is not None:
            sp = p + n["shared"]
            self.ws_gate_up = tensors[sp + n["gate"] + "+" + n["up"]]
            self.ws_down = tensors[sp + n["down"]]
        # the experts' queue counters: zero between steps (the planning kernel clears them)
        self.counts = torch.zeros(self.experts, dtype=torch.int32, device=self.w_router.device)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        t, arena = x.shape[0], ctx.arena
        tile_rows = ops.moe_tile_rows(t, self.top, self.experts, ctx.dtype, (self.h, self.ff))
        plan = ops.moe_route_from(x, self.w_router, self.top, self.counts, arena, tile_rows, self.rule, self.outputs)
        act = arena.take((t * self.top, self.ff), ctx.dtype)
        ops.moe_gemm(x, self.w_gate_up, act, plan, gated=True, gather=True, arena=arena)
        y = arena.take((t * self.top, self.h), ctx.dtype)
        ops.moe_gemm(act, self.w_down, y, plan, gated=False, gather=False, arena=arena)
        shared = None
        if self.shared_ff is not None:
            sact = arena.take((t, self.shared_ff), ctx.dtype)
            ops.gemm_gated(x, self.ws_gate_up, sact, arena, "silu")
            shared = arena.take((t, self.h), ctx.dtype)
            ops.gemm(sact, self.ws_down, shared)
        out = arena.take((t, self.h), ctx.dtype)
        ops.moe_combine(y, plan, shared, out, x=x if self.identity else None,
                        shared_gate=plan["logits"][:, self.outputs] if self.shared_gate else None)
        return out


register_feed_forward("routed_experts", RoutedExperts)
register_feed_forward("swiglu", SwiGLU)
register_feed_forward("gated_mlp", GatedMLP)
