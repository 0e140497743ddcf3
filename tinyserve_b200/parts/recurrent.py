"""Recurrent mixers whose memory is a matrix per head, kept in a state slot per request.

``MLSTMMixer``: the matrix memory of xLSTM. Per head, with log gates
``i = cap tanh((W_i h + b_i) / cap)`` and ``f = logsigmoid(cap tanh((W_f h + b_f) / cap))`` and a
stabiliser ``m`` (a running maximum, 0 for a fresh state): ``m' = max(f + m, i)``;
``S <- e^(f + m - m') S + e^(i - m') k v^T``; ``n`` likewise with ``k``;
``o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)`` with ``q`` scaled by ``dim^-1/2``. Each head's ``o``
is divided by its root mean square, the heads are concatenated, multiplied by a weight and by
``sigmoid(W_g h)``, and projected by ``W_o``.

``ChannelDeltaMixer``: the gated delta rule with one decay per head and key channel. q, k (``kv_heads``
heads) and v (``heads`` heads) pass a short causal convolution per channel and SiLU; q and k are
scaled to unit length (q also by ``dim^-1/2``); ``beta = sigmoid(W_b h)``;
``g = exp(-exp(A_log) softplus(W_a2 W_a1 h + dt_bias))`` per key channel. Per head:
``S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q``. Each head's ``o`` is divided by
its root mean square, multiplied by a weight shared by the heads and by ``sigmoid(W_g2 W_g1 h)``,
and projected by ``W_o``. The convolution's last ``taps - 1`` inputs are state too.

``GatedDeltaMixer``: the gated delta rule with ONE decay per head and token,
``g = exp(-exp(A_log_h) softplus(W_a h + dt_bias_h))``, full-rank projections for the step size and
the output gate, and ``z sigmoid(z)`` of ``W_g h`` as the gate; otherwise as above.

``TimeMixMixer``: time mixing in the manner of RWKV-6. With ``h'`` the previous token's input (zero
before the first token; it is state), each of r, k, v, g, w reads ``h + (h' - h) mu_s``; ``r, k, v``
are projections (``heads x dim``), the gate is ``silu(W_g .)``, the decay per head and key channel
``w = exp(-exp(W_w2 tanh(W_w1 .) + w0))``. Per head ``o = (S + diag(u) k v^T)^T r`` with a bonus ``u``
for the current token, then ``S <- diag(w) S + k v^T``. Each head's ``o`` is divided by its root mean
square, multiplied by a weight (one value per head and column) and by the gate, and projected by ``W_o``.

``DecayLinearAttention``: linear attention with a constant decay per head (the constants are
arguments): ``q, k, v = silu(W_q h), silu(W_k h), silu(W_v h)``; per head ``S <- decay_h S + k v^T``,
``o = S^T q``; the concatenated heads are RMS-normed together with a plain weight, multiplied by
``sigmoid(W_g h)`` and projected by ``W_o``.

``GatedLinearAttention``: linear attention with a decay per head, key channel and token:
``q = W_q h * dim^-1/2``, ``k = W_k h``, ``v = W_v h``; ``alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau)`` with a
constant ``tau``; per head ``S <- diag(alpha) S + k v^T``, ``o = S^T q`` (the read-out sees the current
token's write). Each head's ``o`` is RMS-normed with a weight shared by the heads, multiplied by
``silu(W_g h)`` and projected by ``W_o``.

Gates, decays, step sizes, unit scalings and the state are 32-bit; the projections and the
convolution's inputs are in the model dtype. Nothing of a step is read on the host: requests are
found through ``cu_query_lens`` and ``state_slots`` on the device, so every kind of step can be
recorded.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..kernels import ops
from .base import EVERY_STEP, Mixer, StateCacheEntry, StateNeed, StepContext, TensorSpec, register_mixer

_MLSTM_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "norm": "norm", "input_gate": "i",
                "forget_gate": "f", "input_bias": "i.b", "forget_bias": "f.b"}
_DELTA_NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta": "b",
                "a_log": "A_log", "norm": "norm", "step_down": "a1", "step_up": "a2", "step_bias": "dt_bias",
                "gate_down": "g1", "gate_up": "g2", "out": "o"}


def _check_key_dim(kind: str, d: int) -> None:
    if not 0 < d <= ops.SCAN_MAX_KEY_DIM:
        raise ValueError(f"{kind}: key size {d} is outside 1..{ops.SCAN_MAX_KEY_DIM}, what the scan kernel keeps in registers")


class MLSTMMixer(Mixer):
    recordable = EVERY_STEP

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, gate_cap: float,
                 norm_eps: float, names: Mapping[str, str] | None = None) -> None:
        _check_key_dim("mlstm", key_dim)
        if not gate_cap > 0:
            raise ValueError(f"gate_cap must be positive, got {gate_cap}")
        self.prefix, self.h = prefix, int(hidden_size)
        self.heads, self.d, self.dv = int(num_heads), int(key_dim), int(value_dim)
        self.cap, self.eps = float(gate_cap), float(norm_eps)
        self.names = {**_MLSTM_NAMES, **(names or {})}

    def cache_need(self) -> StateNeed:
        return StateNeed((ops.mlstm_state_size(self.heads, self.d, self.dv),), torch.float32)

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p, n, h = prefix + self.prefix, self.names, self.h
        qk, vv = self.heads * self.d, self.heads * self.dv
        return [
            TensorSpec(p + "qkvg", (2 * qk + 2 * vv, h), merged_from=tuple(p + n[r] for r in ("q", "k", "v", "gate")),
                       merged_rows=(qk, qk, vv, vv)),
            TensorSpec(p + "if", (2 * self.heads, h), merged_from=(p + n["input_gate"], p + n["forget_gate"]),
                       merged_rows=(self.heads, self.heads)),
            TensorSpec(p + "if.b", (2 * self.heads,), std=1.0, merged_from=(p + n["input_bias"], p + n["forget_bias"]),
                       merged_rows=(self.heads, self.heads)),
            TensorSpec(p + n["norm"], (vv,), init="one_plus_normal"),
            TensorSpec(p + n["out"], (h, vv)),
        ]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = prefix + self.prefix, self.names
        self.w_qkvg, self.w_if = tensors[p + "qkvg"], tensors[p + "if"]
        self.bias = tensors[p + "if.b"].float().contiguous()
        self.norm_w, self.w_o = tensors[p + n["norm"]], tensors[p + n["out"]]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: StateCacheEntry, writes_cache: bool, position: Any) -> torch.Tensor:
        t, arena = x.shape[0], ctx.arena
        qk, vv = self.heads * self.d, self.heads * self.dv
        proj = arena.take((t, 2 * qk + 2 * vv), ctx.dtype)
        ops.gemm(x, self.w_qkvg, proj)
        gates = arena.take((t, 2 * self.heads), torch.float32)
        ops.gemm(x, self.w_if, gates)
        read = arena.take((t, self.heads, self.dv), torch.float32)
        ops.mlstm_scan(proj, 0, qk, 2 * qk, gates, self.bias, self.cap, self.d ** -0.5, cache.state, ctx,
                       self.heads, self.d, self.dv, read)
        gated = arena.take((t, vv), ctx.dtype)
        ops.head_norm_gate(read, self.norm_w, True, proj[:, 2 * qk + vv:], True, self.eps, gated)
        out = arena.take((t, self.h), ctx.dtype)
        ops.gemm(gated, self.w_o, out)
        return out


class ChannelDeltaMixer(Mixer):
    recordable = EVERY_STEP

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                 conv_taps: int, norm_eps: float, step_rank: int = -1, gate_rank: int = -1,
                 names: Mapping[str, str] | None = None) -> None:
        """``step_rank`` / ``gate_rank``: inner sizes of the two low-rank pairs; ``-1`` takes them
        from the checkpoint (then the model cannot be drawn at random)."""
        _check_key_dim("channel_delta", key_dim)
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        if not 1 <= conv_taps <= ops.SCAN_MAX_TAPS:
            raise ValueError(f"conv_taps={conv_taps} is outside 1..{ops.SCAN_MAX_TAPS}")
        self.prefix, self.h = prefix, int(hidden_size)
        self.heads, self.groups, self.d, self.dv = int(num_heads), int(num_kv_heads), int(key_dim), int(value_dim)
        self.taps, self.eps = int(conv_taps), float(norm_eps)
        self.step_rank, self.gate_rank = int(step_rank), int(gate_rank)
        self.names = {**_DELTA_NAMES, **(names or {})}
        self.channels = 2 * self.groups * self.d + self.heads * self.dv
        self.state_floats = self.heads * self.d * self.dv

    def cache_need(self) -> StateNeed:
        # the matrix memory of every head, then the convolution's last taps - 1 inputs of every channel
        return StateNeed((self.state_floats + (self.taps - 1) * self.channels,), torch.float32)

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p, n, h = prefix + self.prefix, self.names, self.h
        qk, vv = self.groups * self.d, self.heads * self.dv
        return [
            TensorSpec(p + "qkv", (self.channels, h), merged_from=tuple(p + n[r] for r in ("q", "k", "v")),
                       merged_rows=(qk, qk, vv)),
            TensorSpec(p + "qkv.conv", (self.channels, self.taps), std=0.3,
                       merged_from=tuple(p + n[r] for r in ("q_conv", "k_conv", "v_conv")), merged_rows=(qk, qk, vv)),
            TensorSpec(p + n["beta"], (self.heads, h)),
            TensorSpec(p + n["a_log"], (self.heads,), std=0.5),
            TensorSpec(p + n["norm"], (self.dv,), init="one_plus_normal"),
            TensorSpec(p + n["step_down"], (self.step_rank, h)),
            TensorSpec(p + n["step_up"], (self.heads * self.d, self.step_rank)),
            TensorSpec(p + n["step_bias"], (self.heads * self.d,), std=1.0),
            TensorSpec(p + n["gate_down"], (self.gate_rank, h)),
            TensorSpec(p + n["gate_up"], (vv, self.gate_rank)),
            TensorSpec(p + n["out"], (h, vv)),
        ]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = prefix + self.prefix, self.names
        self.w_qkv, self.w_conv = tensors[p + "qkv"], tensors[p + "qkv.conv"]
        self.w_beta, self.norm_w, self.w_o = tensors[p + n["beta"]], tensors[p + n["norm"]], tensors[p + n["out"]]
        self.a_log = tensors[p + n["a_log"]].float().contiguous()
        self.step_bias = tensors[p + n["step_bias"]].float().contiguous()
        self.w_a1, self.w_a2 = tensors[p + n["step_down"]], tensors[p + n["step_up"]]
        self.w_g1, self.w_g2 = tensors[p + n["gate_down"]], tensors[p + n["gate_up"]]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: StateCacheEntry, writes_cache: bool, position: Any) -> torch.Tensor:
        t, arena = x.shape[0], ctx.arena
        qk, vv = self.groups * self.d, self.heads * self.dv
        proj = arena.take((t, self.channels), ctx.dtype)
        ops.gemm(x, self.w_qkv, proj)
        conved = arena.take((t, self.channels), torch.float32)
        ops.causal_conv_silu(proj, self.w_conv, cache.state[:, self.state_floats:], ctx, conved)
        low = arena.take((t, self.w_a1.shape[0]), ctx.dtype)
        ops.gemm(x, self.w_a1, low)
        step = arena.take((t, self.heads * self.d), torch.float32)
        ops.gemm(low, self.w_a2, step)
        beta = arena.take((t, self.heads), torch.float32)
        ops.gemm(x, self.w_beta, beta)
        low = arena.take((t, self.w_g1.shape[0]), ctx.dtype)
        ops.gemm(x, self.w_g1, low)
        gate = arena.take((t, vv), ctx.dtype)
        ops.gemm(low, self.w_g2, gate)
        read = arena.take((t, self.heads, self.dv), torch.float32)
        ops.delta_scan(conved, 0, qk, 2 * qk, step, self.step_bias, self.a_log, beta, self.d ** -0.5,
                       cache.state[:, : self.state_floats], ctx, self.heads, self.groups, self.d, self.dv, read)
        gated = arena.take((t, vv), ctx.dtype)
        ops.head_norm_gate(read, self.norm_w, False, gate, True, self.eps, gated)
        out = arena.take((t, self.h), ctx.dtype)
        ops.gemm(gated, self.w_o, out)
        return out


class GatedDeltaMixer(Mixer):
    recordable = EVERY_STEP
    _NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta": "b",
              "step": "a", "a_log": "A_log", "step_bias": "dt_bias", "norm": "norm", "gate": "g", "out": "o"}

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                 conv_taps: int, norm_eps: float, names: Mapping[str, str] | None = None) -> None:
        _check_key_dim("gated_delta", key_dim)
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        if not 1 <= conv_taps <= ops.SCAN_MAX_TAPS:
            raise ValueError(f"conv_taps={conv_taps} is outside 1..{ops.SCAN_MAX_TAPS}")
        self.prefix, self.h = prefix, int(hidden_size)
        self.heads, self.groups, self.d, self.dv = int(num_heads), int(num_kv_heads), int(key_dim), int(value_dim)
        self.taps, self.eps = int(conv_taps), float(norm_eps)
        self.names = {**self._NAMES, **(names or {})}
        self.channels = 2 * self.groups * self.d + self.heads * self.dv
        self.state_floats = self.heads * self.d * self.dv

    def cache_need(self) -> StateNeed:
        # the matrix memory of every head, then the convolution's last taps - 1 inputs of every channel
        return StateNeed((self.state_floats + (self.taps - 1) * self.channels,), torch.float32)

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p, n, h = prefix + self.prefix, self.names, self.h
        qk, vv = self.groups * self.d, self.heads * self.dv
        return [
            TensorSpec(p + "qkvg", (self.channels + vv, h), merged_from=tuple(p + n[r] for r in ("q", "k", "v", "gate")),
                       merged_rows=(qk, qk, vv, vv)),
            TensorSpec(p + "qkv.conv", (self.channels, self.taps), std=0.3,
                       merged_from=tuple(p + n[r] for r in ("q_conv", "k_conv", "v_conv")), merged_rows=(qk, qk, vv)),
            TensorSpec(p + "beta+step", (2 * self.heads, h), merged_from=(p + n["beta"], p + n["step"]),
                       merged_rows=(self.heads, self.heads)),
            TensorSpec(p + n["a_log"], (self.heads,), std=0.5),
            TensorSpec(p + n["step_bias"], (self.heads,), std=1.0),
            TensorSpec(p + n["norm"], (self.dv,), init="one_plus_normal"),
            TensorSpec(p + n["out"], (h, vv)),
        ]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = prefix + self.prefix, self.names
        self.w_in, self.w_conv = tensors[p + "qkvg"], tensors[p + "qkv.conv"]
        self.w_bs, self.norm_w, self.w_o = tensors[p + "beta+step"], tensors[p + n["norm"]], tensors[p + n["out"]]
        self.a_log = tensors[p + n["a_log"]].float().contiguous()
        self.step_bias = tensors[p + n["step_bias"]].float().contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: StateCacheEntry, writes_cache: bool, position: Any) -> torch.Tensor:
        t, arena = x.shape[0], ctx.arena
        qk, vv, ch = self.groups * self.d, self.heads * self.dv, self.channels
        proj = arena.take((t, ch + vv), ctx.dtype)
        ops.gemm(x, self.w_in, proj)
        conved = arena.take((t, ch), torch.float32)
        ops.causal_conv_silu(proj[:, :ch], self.w_conv, cache.state[:, self.state_floats:], ctx, conved)
        bs = arena.take((t, 2 * self.heads), torch.float32)      # beta and step-size pre-activations, 32-bit
        ops.gemm(x, self.w_bs, bs)
        read = arena.take((t, self.heads, self.dv), torch.float32)
        ops.delta_scan(conved, 0, qk, 2 * qk, bs[:, self.heads:], self.step_bias, self.a_log, bs[:, : self.heads],
                       self.d ** -0.5, cache.state[:, : self.state_floats], ctx, self.heads, self.groups, self.d, self.dv, read)
        gated = arena.take((t, vv), ctx.dtype)
        ops.head_norm_gate(read, self.norm_w, False, proj[:, ch:], True, self.eps, gated, gate_silu=True)
        out = arena.take((t, self.h), ctx.dtype)
        ops.gemm(gated, self.w_o, out)
        return out


class TimeMixMixer(Mixer):
    recordable = EVERY_STEP
    _NAMES = {"mu_r": "mu.r", "mu_k": "mu.k", "mu_v": "mu.v", "mu_g": "mu.g", "mu_w": "mu.w", "r": "r", "k": "k", "v": "v",
              "gate": "g", "decay_down": "w1", "decay_up": "w2", "decay_bias": "w0", "bonus": "u", "norm": "norm", "out": "o"}

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, head_dim: int, norm_eps: float, decay_rank: int = -1,
                 names: Mapping[str, str] | None = None) -> None:
        """``decay_rank``: the inner size of the decay's low-rank pair; ``-1`` takes it from the
        checkpoint (then the model cannot be drawn at random)."""
        _check_key_dim("time_mix", head_dim)
        self.prefix, self.h = prefix, int(hidden_size)
        self.heads, self.d, self.eps, self.rank = int(num_heads), int(head_dim), float(norm_eps), int(decay_rank)
        self.names = {**self._NAMES, **(names or {})}
        self.state_floats = self.heads * self.d * self.d

    def cache_need(self) -> StateNeed:
        # the matrix memory of every head, then the previous token's input
        return StateNeed((self.state_floats + self.h,), torch.float32)

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p, n, h, hd = prefix + self.prefix, self.names, self.h, self.heads * self.d
        return [
            TensorSpec(p + "mu", (5 * h,), std=0.3, merged_from=tuple(p + n[r] for r in ("mu_r", "mu_k", "mu_v", "mu_g", "mu_w")),
                       merged_rows=(h,) * 5),
            TensorSpec(p + "rkvg", (4 * hd, h), merged_from=tuple(p + n[r] for r in ("r", "k", "v", "gate")), merged_rows=(hd,) * 4),
            TensorSpec(p + n["decay_down"], (self.rank, h)),
            TensorSpec(p + n["decay_up"], (hd, self.rank)),
            TensorSpec(p + n["decay_bias"], (hd,), std=1.0),
            TensorSpec(p + n["bonus"], (self.heads, self.d), std=0.5),
            TensorSpec(p + n["norm"], (hd,), init="one_plus_normal"),
            TensorSpec(p + n["out"], (h, hd)),
        ]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n, hd = prefix + self.prefix, self.names, self.heads * self.d
        self.mu = tensors[p + "mu"].view(5, self.h)
        self.w_rkvg_t = tensors[p + "rkvg"].view(4, hd, self.h).transpose(1, 2)      # [4, hidden, heads * dim] (a view)
        self.w_down, self.w_up = tensors[p + n["decay_down"]], tensors[p + n["decay_up"]]
        self.decay_bias = tensors[p + n["decay_bias"]].float().contiguous()
        self.bonus = tensors[p + n["bonus"]].float().contiguous().view(hd)
        self.norm_w, self.w_o = tensors[p + n["norm"]], tensors[p + n["out"]]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: StateCacheEntry, writes_cache: bool, position: Any) -> torch.Tensor:
        t, arena, hd = x.shape[0], ctx.arena, self.heads * self.d
        mixes = arena.take((5, t, self.h), ctx.dtype)
        ops.token_shift_mix(x, self.mu, cache.state[:, self.state_floats:], ctx, mixes)
        rkvg = arena.take((4, t, hd), ctx.dtype)
        ops.bmm(mixes[:4], self.w_rkvg_t, rkvg)
        low = arena.take((t, self.w_down.shape[0]), ctx.dtype)
        ops.gemm(mixes[4], self.w_down, low)
        ops.tanh_(low)
        w_pre = arena.take((t, hd), torch.float32)
        ops.gemm(low, self.w_up, w_pre)
        read = arena.take((t, self.heads, self.d), torch.float32)
        ops.linear_scan_bonus(rkvg[0], rkvg[1], rkvg[2], w_pre, self.decay_bias, self.bonus,
                              cache.state[:, : self.state_floats], ctx, self.heads, self.d, self.d, read)
        gated = arena.take((t, hd), ctx.dtype)
        ops.head_norm_gate(read, self.norm_w, True, rkvg[3], True, self.eps, gated, gate_silu=True)
        out = arena.take((t, self.h), ctx.dtype)
        ops.gemm(gated, self.w_o, out)
        return out


class DecayLinearAttention(Mixer):
    recordable = EVERY_STEP
    _NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "norm": "norm", "out": "o"}

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, decay: "list[float]",
                 norm_eps: float, names: Mapping[str, str] | None = None) -> None:
        _check_key_dim("decay_linear_attention", key_dim)
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decay constants for {num_heads} heads")
        self.prefix, self.h = prefix, int(hidden_size)
        self.heads, self.d, self.dv, self.eps = int(num_heads), int(key_dim), int(value_dim), float(norm_eps)
        self.decay_values = [float(x) for x in decay]
        self.names = {**self._NAMES, **(names or {})}

    def cache_need(self) -> StateNeed:
        return StateNeed((self.heads * self.d * self.dv,), torch.float32)

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p, n, h = prefix + self.prefix, self.names, self.h
        qk, vv = self.heads * self.d, self.heads * self.dv
        return [TensorSpec(p + "qkvg", (2 * qk + 2 * vv, h), merged_from=tuple(p + n[r] for r in ("q", "k", "v", "gate")),
                           merged_rows=(qk, qk, vv, vv)),
                TensorSpec(p + n["norm"], (vv,), init="one_plus_normal"),
                TensorSpec(p + n["out"], (h, vv))]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = prefix + self.prefix, self.names
        self.w_in, self.norm_w, self.w_o = tensors[p + "qkvg"], tensors[p + n["norm"]], tensors[p + n["out"]]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_o.device)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: StateCacheEntry, writes_cache: bool, position: Any) -> torch.Tensor:
        t, arena = x.shape[0], ctx.arena
        qk, vv = self.heads * self.d, self.heads * self.dv
        proj = arena.take((t, 2 * qk + 2 * vv), ctx.dtype)
        ops.gemm(x, self.w_in, proj)
        read = arena.take((t, self.heads, self.dv), torch.float32)
        ops.linear_scan_decay(proj[:, :qk], proj[:, qk: 2 * qk], proj[:, 2 * qk: 2 * qk + vv], self.decay, cache.state, ctx,
                              self.heads, self.d, self.dv, read)
        gated = arena.take((t, vv), ctx.dtype)
        # one norm over all heads together: a single "head" as wide as their concatenation
        ops.head_norm_gate(read.view(t, 1, vv), self.norm_w, False, proj[:, 2 * qk + vv:], True, self.eps, gated)
        out = arena.take((t, self.h), ctx.dtype)
        ops.gemm(gated, self.w_o, out)
        return out


class GatedLinearAttention(Mixer):
    recordable = EVERY_STEP
    _NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "decay_down": "a1", "decay_up": "a2", "decay_bias": "a2.b",
              "norm": "norm", "out": "o"}

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, tau: float,
                 norm_eps: float, decay_rank: int = -1, names: Mapping[str, str] | None = None) -> None:
        """``decay_rank``: the inner size of the decay's low-rank pair; ``-1`` takes it from the
        checkpoint (then the model cannot be drawn at random)."""
        _check_key_dim("gated_linear_attention", key_dim)
        if not tau > 0:
            raise ValueError(f"tau={tau} must be positive")
        self.prefix, self.h = prefix, int(hidden_size)
        self.heads, self.d, self.dv = int(num_heads), int(key_dim), int(value_dim)
        self.tau, self.eps, self.rank = float(tau), float(norm_eps), int(decay_rank)
        self.names = {**self._NAMES, **(names or {})}

    def cache_need(self) -> StateNeed:
        return StateNeed((self.heads * self.d * self.dv,), torch.float32)

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p, n, h = prefix + self.prefix, self.names, self.h
        qk, vv = self.heads * self.d, self.heads * self.dv
        return [TensorSpec(p + "qkvg", (2 * qk + 2 * vv, h), merged_from=tuple(p + n[r] for r in ("q", "k", "v", "gate")),
                           merged_rows=(qk, qk, vv, vv)),
                TensorSpec(p + n["decay_down"], (self.rank, h)),
                TensorSpec(p + n["decay_up"], (qk, self.rank)),
                TensorSpec(p + n["decay_bias"], (qk,), std=1.0),
                TensorSpec(p + n["norm"], (self.dv,), init="one_plus_normal"),
                TensorSpec(p + n["out"], (h, vv))]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = prefix + self.prefix, self.names
        self.w_in, self.norm_w, self.w_o = tensors[p + "qkvg"], tensors[p + n["norm"]], tensors[p + n["out"]]
        self.w_a1, self.w_a2 = tensors[p + n["decay_down"]], tensors[p + n["decay_up"]]
        self.decay_bias = tensors[p + n["decay_bias"]].float().contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: StateCacheEntry, writes_cache: bool, position: Any) -> torch.Tensor:
        t, arena = x.shape[0], ctx.arena
        qk, vv = self.heads * self.d, self.heads * self.dv
        proj = arena.take((t, 2 * qk + 2 * vv), ctx.dtype)
        ops.gemm(x, self.w_in, proj)
        low = arena.take((t, self.w_a1.shape[0]), ctx.dtype)
        ops.gemm(x, self.w_a1, low)
        z = arena.take((t, qk), torch.float32)            # the decay's pre-activation leaves its product as 32-bit
        ops.gemm(low, self.w_a2, z)
        read = arena.take((t, self.heads, self.dv), torch.float32)
        ops.linear_scan_gated(proj[:, :qk], proj[:, qk: 2 * qk], proj[:, 2 * qk: 2 * qk + vv], z, self.decay_bias, self.tau,
                              self.d ** -0.5, cache.state, ctx, self.heads, self.d, self.dv, read)
        gated = arena.take((t, vv), ctx.dtype)
        ops.head_norm_gate(read, self.norm_w, False, proj[:, 2 * qk + vv:], True, self.eps, gated, gate_silu=True)
        out = arena.take((t, self.h), ctx.dtype)
        ops.gemm(gated, self.w_o, out)
        return out


register_mixer("gated_linear_attention", GatedLinearAttention)
register_mixer("gated_delta", GatedDeltaMixer)
register_mixer("time_mix", TimeMixMixer)
register_mixer("decay_linear_attention", DecayLinearAttention)
register_mixer("mlstm", MLSTMMixer)
register_mixer("channel_delta", ChannelDeltaMixer)
