"""A plain, slow implementation of the Gasavik decoder, one function per mechanism, written from
the design's equations and sharing no code with the product path. Everything runs token by
token or with full matrices on the CPU in one floating type (float64 for an oracle, float32
otherwise); nothing is cached between calls.

Notation: ``h`` is a sub-layer's input ``[T, width]``; weights are ``[out, in]``; ``w`` maps
tensor names to tensors already converted to the working type; ``p`` is a tensor-name prefix.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path
from typing import Any, Mapping

import torch


# ------------------------------------------------------------------------ files
def read_config(folder: str | Path) -> dict[str, Any]:
    return json.loads((Path(folder) / "config.json").read_text())


def read_weights(folder: str | Path, dtype: torch.dtype = torch.float64) -> dict[str, torch.Tensor]:
    """Parse ``model.safetensors`` by hand: 8-byte length, JSON header, raw data."""
    raw = (Path(folder) / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8: 8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + a: 8 + n + b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        out[name] = t if info["dtype"] == "I32" else t.to(dtype)
    return out


# -------------------------------------------------------------------- mechanisms
def rms_norm(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    y = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def embed(tokens: list[int], w: Mapping[str, torch.Tensor], eps: float) -> torch.Tensor:
    """Token row plus the learned row of the position, then the model's norm."""
    t = len(tokens)
    x = w["embed"][tokens] + w["pos"][:t]
    return rms_norm(x, w["embed.norm"], eps)


def biased_swiglu(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    gate = h @ w[p + "gate"].T + w[p + "gate.b"]
    up = h @ w[p + "up"].T + w[p + "up.b"]
    return (silu(gate) * up) @ w[p + "down"].T + w[p + "down.b"]


def token_side(x: torch.Tensor, tokens: list[int], table_part: torch.Tensor, w: Mapping[str, torch.Tensor], p: str,
               eps: float) -> torch.Tensor:
    """The per-layer token input: the layer's stretch of the side table, gated by the stream,
    projected to the width and RMS-normed with a plain weight."""
    e = table_part[tokens]
    g = gelu_tanh(x @ w[p + "gate"].T) * e
    return rms_norm(g @ w[p + "proj"].T, w[p + "norm"], eps)


def visible(i: int, j: int, window: int | None, keep_first: int) -> bool:
    """Whether the query at position i sees the key at position j."""
    if j > i:
        return False
    return window is None or i - j < window or j < keep_first


def windowed_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any], eps: float) -> torch.Tensor:
    """Grouped-query attention without rotation: biased projections, RMS norm of queries and keys
    per head, a sliding window that also keeps the first tokens, ordinary softmax, one sigmoid
    gate per head."""
    t = h.shape[0]
    heads, groups, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    mask = m.get("mask") or {}
    window, keep = mask.get("size"), int(mask.get("keep_first", 0))
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(t, heads, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(t, groups, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(t, groups, dv)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    gate = torch.sigmoid(h @ w[p + "g"].T)                      # [T, heads]
    see = torch.tensor([[visible(i, j, window, keep) for j in range(t)] for i in range(t)])
    out = torch.zeros(t, heads, dv, dtype=h.dtype)
    per = heads // groups
    for a in range(heads):
        g = a // per
        s = (q[:, a] @ k[:, g].T) * float(m["scale"])
        pr = torch.softmax(s.masked_fill(~see, -math.inf), -1)
        out[:, a] = (pr @ v[:, g]) * gate[:, a: a + 1]
    return out.reshape(t, heads * dv) @ w[p + "o"].T


def lightning_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any], eps: float) -> torch.Tensor:
    """Linear attention with a fixed decay per head: ``S <- decay S + k v^T; o = S^T q``."""
    t = h.shape[0]
    heads, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ w[p + "q"].T).view(t, heads, d)
    k = silu(h @ w[p + "k"].T).view(t, heads, d)
    v = silu(h @ w[p + "v"].T).view(t, heads, dv)
    out = torch.zeros(t, heads, dv, dtype=h.dtype)
    for a in range(heads):
        state = torch.zeros(d, dv, dtype=h.dtype)
        for i in range(t):
            state = float(m["decay"][a]) * state + torch.outer(k[i, a], v[i, a])
            out[i, a] = state.T @ q[i, a]
    y = rms_norm(out.reshape(t, heads * dv), w[p + "norm"], eps) * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def side_by_side(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any], eps: float) -> torch.Tensor:
    left = windowed_attention(h, w, p + "left.", m["left"], eps)
    right = lightning_attention(h, w, p + "right.", m["right"], eps)
    return float(m.get("left_scale", 1.0)) * left + float(m.get("right_scale", 1.0)) * right


def wkv(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any], eps: float) -> torch.Tensor:
    """Time mixing with a data-dependent decay per key channel and a bonus for the current token."""
    t = h.shape[0]
    heads, d = int(m["heads"]), int(m["dim"])
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]])

    def mix(s: str) -> torch.Tensor:
        return h + (before - h) * w[p + "mu." + s]

    r = (mix("r") @ w[p + "r"].T).view(t, heads, d)
    k = (mix("k") @ w[p + "k"].T).view(t, heads, d)
    v = (mix("v") @ w[p + "v"].T).view(t, heads, d)
    gate = silu(mix("g") @ w[p + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix("w") @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(t, heads, d)
    u = w[p + "u"]
    out = torch.zeros(t, heads, d, dtype=h.dtype)
    for a in range(heads):
        state = torch.zeros(d, d, dtype=h.dtype)
        for i in range(t):
            kv = torch.outer(k[i, a], v[i, a])
            out[i, a] = (state + u[a][:, None] * kv).T @ r[i, a]
            state = decay[i, a][:, None] * state + kv
    y = rms_norm(out, None, eps).reshape(t, heads * d) * w[p + "norm"] * gate
    return y @ w[p + "o"].T


def causal_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x ``[T, C]``, taps ``[C, K]``; the last tap multiplies the current token's input; zeros before the start."""
    t, k = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(k - 1, x.shape[1], dtype=x.dtype), x])
    return sum(padded[j: j + t] * taps[:, j] for j in range(k))


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).sum(-1, keepdim=True) + 1e-6)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def head_delta(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any], eps: float) -> torch.Tensor:
    """The gated delta rule with one decay per head."""
    t = h.shape[0]
    heads, groups, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = unit(silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(t, groups, d)) * d ** -0.5
    k = unit(silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(t, groups, d))
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(t, heads, dv)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))   # [T, heads]
    out = torch.zeros(t, heads, dv, dtype=h.dtype)
    per = heads // groups
    for a in range(heads):
        g = a // per
        state = torch.zeros(d, dv, dtype=h.dtype)
        for i in range(t):
            state = decay[i, a] * state
            write = beta[i, a] * (v[i, a] - state.T @ k[i, g])
            state = state + torch.outer(k[i, g], write)
            out[i, a] = state.T @ q[i, g]
    y = rms_norm(out, w[p + "norm"], eps) * silu(h @ w[p + "g"].T).view(t, heads, dv)
    return y.reshape(t, heads * dv) @ w[p + "o"].T


MIXERS = {"parallel": side_by_side, "wkv": wkv, "delta": head_delta}


# ------------------------------------------------------------------------ model
def forward(config: Mapping[str, Any], w: Mapping[str, torch.Tensor], tokens: list[int],
            after_layers: list[torch.Tensor] | None = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence from its start. ``after_layers`` collects the
    residual stream after every layer."""
    eps = float(config["norm"]["eps"])
    mult = float(config.get("residual_mult", 1.0))
    side = config.get("token_side")
    x = embed(tokens, w, eps)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        y = MIXERS[layer["type"]](h, w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            y = y + biased_swiglu(h, w, p + "mlp.")
        x = x + mult * y
        if side is not None:
            dim = int(side["dim"])
            x = x + mult * token_side(x, tokens, w["side.embed"][:, i * dim: (i + 1) * dim], w, p + "side.", eps)
        if after_layers is not None:
            after_layers.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(config: Mapping[str, Any], w: Mapping[str, torch.Tensor], prompt: list[int], new_tokens: int) -> list[int]:
    """The ``new_tokens`` most likely next tokens, one after the other (the whole sequence is run again each time)."""
    seq = list(prompt)
    for _ in range(new_tokens):
        seq.append(int(forward(config, w, seq)[-1].argmax()))
    return seq[len(prompt):]
