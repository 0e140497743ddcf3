"""A plain, slow implementation of the Diderax decoder, one function per mechanism, written from
the design's equations and sharing no code with the product path. Everything runs token by
token or with full matrices on the CPU in one floating type (float64 for an oracle, float32
otherwise); nothing is cached between calls.

Notation: ``h`` is a sub-layer's input ``[T, width]``; weights are ``[out, in]``; ``w`` maps
tensor names to tensors already converted to the working type; ``p`` is a tensor-name prefix;
``m`` is the layer's ``mixer`` dictionary of the configuration.
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


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate_half(x: torch.Tensor, dims: int, base: float, factor: float = 1.0, first_position: int = 0) -> torch.Tensor:
    """``x [T, heads, d]``: the first ``dims`` elements of every head turn, element i with element
    ``i + dims / 2``, by ``position * base^(-2i/dims) / factor``; the rest stays."""
    t, half = x.shape[0], dims // 2
    out = x.clone()
    for n in range(t):
        pos = first_position + n
        for i in range(half):
            a = pos * (base ** (-2.0 * i / dims)) / factor
            c, s = math.cos(a), math.sin(a)
            u, v = x[n, :, i], x[n, :, i + half]
            out[n, :, i] = u * c - v * s
            out[n, :, i + half] = v * c + u * s
    return out


def softmax_with_sink(scores: torch.Tensor, sink: float | None) -> torch.Tensor:
    """Weights of one query over its visible keys; with a sink the denominator has the extra
    term ``exp(sink)``, to which no value belongs."""
    top = float(scores.max()) if sink is None else max(float(scores.max()), float(sink))
    e = torch.exp(scores - top)
    den = e.sum() + (0.0 if sink is None else math.exp(float(sink) - top))
    return e / den


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, sinks: "list[float | None]") -> torch.Tensor:
    """``q [T, H, d]``, ``k [T, H, d]``, ``v [T, H, dv]`` (already one key/value head per query
    head); position i sees every j <= i."""
    t, heads, _ = q.shape
    out = torch.zeros(t, heads, v.shape[-1], dtype=q.dtype)
    for a in range(heads):
        for i in range(t):
            s = (k[: i + 1, a] @ q[i, a]) * scale
            out[i, a] = softmax_with_sink(s, sinks[a]) @ v[: i + 1, a]
    return out


def attention_mixer(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any], eps: float) -> torch.Tensor:
    """Grouped-query attention whose values are the keys as projected; q and k are RMS-normed over
    the whole projection, partly rotated with scaled frequencies; one is added to the softmax's
    denominator; the heads are gated per element by ``sigmoid(W_g h)``."""
    t = h.shape[0]
    heads, groups, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    rot = m["rot"]
    q_raw, k_raw = h @ w[p + "q"].T, h @ w[p + "k"].T
    values = k_raw.view(t, groups, d)
    q = rms_norm(q_raw, w[p + "q.norm"], eps).view(t, heads, d)
    k = rms_norm(k_raw, w[p + "k.norm"], eps).view(t, groups, d)
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    q = rotate_half(q, int(rot["dims"]), float(rot["base"]), factor)
    k = rotate_half(k, int(rot["dims"]), float(rot["base"]), factor)
    per = heads // groups
    k_full = k.repeat_interleave(per, dim=1)
    v_full = values.repeat_interleave(per, dim=1)
    o = causal_attention(q, k_full, v_full, float(m["scale"]), [0.0] * heads)
    gated = o.reshape(t, -1) * torch.sigmoid(h @ w[p + "g"].T)
    return gated @ w[p + "o"].T


def latent_attention_mixer(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any], eps: float) -> torch.Tensor:
    """Queries through a normed latent; keys and values from a normed latent per token plus one
    rotated key part shared by the heads; a learned sink per head."""
    t = h.shape[0]
    heads, dn, dr, dv, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    rot = m["rot"]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(t, heads, dn + dr)
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    shared = down[:, rank:].view(t, 1, dr)
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    q_rot = rotate_half(q[:, :, dn:], int(rot["dims"]), float(rot["base"]), factor)
    k_rot = rotate_half(shared, int(rot["dims"]), float(rot["base"]), factor)
    k_plain = (c @ w[p + "uk"].T).view(t, heads, dn)
    v = (c @ w[p + "uv"].T).view(t, heads, dv)
    q_all = torch.cat([q[:, :, :dn], q_rot], dim=-1)
    k_all = torch.cat([k_plain, k_rot.expand(t, heads, dr)], dim=-1)
    sinks = [float(x) for x in w[p + "sink"]]
    o = causal_attention(q_all, k_all, v, float(m["scale"]), sinks)
    return o.reshape(t, -1) @ w[p + "o"].T


def gla_mixer(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any], eps: float,
              state: "torch.Tensor | None" = None) -> torch.Tensor:
    """Gated linear attention, token by token: ``S <- diag(alpha) S + k v^T``, ``o = S^T q`` with a
    decay per key channel ``alpha = sigmoid(z)^(1/tau)``."""
    t = h.shape[0]
    heads, d, dv, tau = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["tau"])
    q = (h @ w[p + "q"].T).view(t, heads, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(t, heads, d)
    v = (h @ w[p + "v"].T).view(t, heads, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / tau).view(t, heads, d)
    s = torch.zeros(heads, d, dv, dtype=h.dtype) if state is None else state
    o = torch.zeros(t, heads, dv, dtype=h.dtype)
    for n in range(t):
        for a in range(heads):
            s[a] = alpha[n, a][:, None] * s[a] + torch.outer(k[n, a], v[n, a])
            o[n, a] = s[a].T @ q[n, a]
    o = rms_norm(o, w[p + "norm"], eps)
    return (o.reshape(t, -1) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def dense_ff(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    gate = h @ w[p + "gate"].T + w[p + "gate.b"]
    up = h @ w[p + "up"].T + w[p + "up.b"]
    return (silu(gate) * up) @ w[p + "down"].T + w[p + "down.b"]


def expert(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, router: Mapping[str, Any]) -> list[list[tuple[int, float]]]:
    """Per token the chosen (expert, weight) pairs. The choice uses the softmax scores plus the
    correction and looks only inside the best groups; the weights use the scores alone."""
    real, ident, top = int(router["experts"]), int(router.get("identity", 0)), int(router["top"])
    total = real + ident
    groups = router.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(groups["count"]), int(groups["keep"])
    size = total // count
    scale = float(router.get("scale", 1.0))
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    choice = s + w[p + "correction"] if p + "correction" in w else s.clone()
    picks = []
    for n in range(h.shape[0]):
        best = [max(float(choice[n, e]) for e in range(g * size, (g + 1) * size)) for g in range(count)]
        kept = sorted(range(count), key=lambda g: (-best[g], g))[:keep]
        allowed = [e for g in kept for e in range(g * size, (g + 1) * size)]
        chosen = sorted(allowed, key=lambda e: (-float(choice[n, e]), e))[:top]
        den = sum(float(s[n, e]) for e in chosen) + 1e-20
        picks.append([(e, float(s[n, e]) / den * scale) for e in chosen])
    return picks


def moe_ff(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, mlp: Mapping[str, Any]) -> torch.Tensor:
    real = int(mlp["router"]["experts"])
    out = torch.zeros_like(h)
    for n, chosen in enumerate(route(h, w, p, mlp["router"])):
        for e, weight in chosen:
            y = h[n] if e >= real else expert(h[n: n + 1], w, f"{p}e{e}.")[0]
            out[n] = out[n] + weight * y
    if mlp.get("shared") is not None:
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * expert(h, w, p + "shared.")
    return out


MIXERS = {"attention": attention_mixer, "latent_attention": latent_attention_mixer, "gla": gla_mixer}


def layer(x: torch.Tensor, w: Mapping[str, torch.Tensor], i: int, spec: Mapping[str, Any], eps: float) -> torch.Tensor:
    p = f"l{i}."
    x = x + w[p + "ls1"] * MIXERS[spec["type"]](rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", spec["mixer"], eps)
    mlp = spec.get("mlp")
    if mlp is not None:
        hn = rms_norm(x, w[p + "norm2"], eps)
        y = dense_ff(hn, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(hn, w, p + "mlp.", mlp)
        x = x + w[p + "ls2"] * y
    return x


def forward(cfg: Mapping[str, Any], w: Mapping[str, torch.Tensor], tokens: list[int], streams: "list | None" = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence from its first token; ``streams`` collects the
    residual stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][tokens]
    for i, spec in enumerate(cfg["layers"]):
        x = layer(x, w, i, spec, eps)
        if streams is not None:
            streams.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(cfg: Mapping[str, Any], w: Mapping[str, torch.Tensor], prompt: list[int], new_tokens: int) -> list[int]:
    """Greedy continuation, recomputing the whole sequence for every token."""
    toks = list(prompt)
    for _ in range(new_tokens):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]
