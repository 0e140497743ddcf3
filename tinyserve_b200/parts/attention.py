"""Grouped-query attention over the paged cache, with optional per-head q/k RMSNorm,
rotary position encoding and an optional sliding window.

Per token (upstream src/tinyserve/model.py:154-173, src/tinyserve/attention.py:89-111):
``qkv = x Wqkv^T`` (rows q, then k, then v; no bias); q and k are normalised per head over
``head_dim`` before the rotation; k (rotated) and v go to the cache at the token's slot;
query head ``h`` reads kv head ``h // (num_heads / num_kv_heads)``; scores are scaled by
``scale``, masked causally (and to the last ``window`` positions if a window is set),
soft-maxed in 32-bit and applied to v; the heads are concatenated and projected by ``Wo``.
The residual add happens in the next norm.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..kernels import ops
from .base import (EVERY_STEP, KVCacheEntry, KVNeed, LatentNeed, LazyNormed, Mixer, ResidualStream, SplitKVNeed,
                   StepContext, TensorSpec, project, project_to_stream, register_mixer)


class GQAAttention(Mixer):
    recordable = EVERY_STEP

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, scale: float, qk_norm: bool = False, qk_norm_eps: float = 1e-6,
                 window: int | None = None) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        if window is not None and window <= 0:
            raise ValueError(f"window must be positive or None, got {window}")
        if head_dim <= 0 or head_dim % 16 or head_dim > 256:
            raise ValueError(f"head_dim={head_dim}: the attention kernels take head sizes in steps of 16 up to 256")
        self.prefix = prefix
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.scale = int(head_dim), float(scale)
        self.qk_norm, self.qk_norm_eps = bool(qk_norm), float(qk_norm_eps)
        self.window = None if window is None else int(window)
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.w_qkv = self.w_q = self.w_o = self.q_norm_w = self.k_norm_w = None

    def cache_need(self) -> KVNeed:
        return KVNeed(self.num_kv_heads, self.head_dim, self.window)

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p, h = prefix + self.prefix, self.hidden_size
        specs = [
            TensorSpec(p + "qkv_proj.weight", (self.q_size + 2 * self.kv_size, h),
                       merged_from=(p + "q_proj.weight", p + "k_proj.weight", p + "v_proj.weight"),
                       merged_rows=(self.q_size, self.kv_size, self.kv_size)),
            TensorSpec(p + "o_proj.weight", (h, self.q_size)),
        ]
        if self.qk_norm:
            specs += [TensorSpec(p + "q_norm.weight", (self.head_dim,), init="one_plus_normal"),
                      TensorSpec(p + "k_norm.weight", (self.head_dim,), init="one_plus_normal")]
        return specs

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p = prefix + self.prefix
        self.w_qkv = tensors[p + "qkv_proj.weight"]
        self.w_q = self.w_qkv[: self.q_size]          # a view: rows of q only
        self.w_o = tensors[p + "o_proj.weight"]
        if self.qk_norm:
            self.q_norm_w = tensors[p + "q_norm.weight"]
            self.k_norm_w = tensors[p + "k_norm.weight"]

    takes_lazy_input = True
    adds_to_stream = True

    def forward(self, x: "torch.Tensor | LazyNormed", ctx: StepContext, cache: KVCacheEntry, writes_cache: bool,
                position: Any, stream: ResidualStream | None = None) -> torch.Tensor | None:
        t = x.shape[0]
        x_device = cache.k.device
        arena = ctx.arena
        group = ctx.kv[cache.group]
        width = self.q_size + 2 * self.kv_size if writes_cache else self.q_size
        qkv = arena.take((t, width), ctx.dtype)
        project(x, self.w_qkv if writes_cache else self.w_q, qkv, ctx)
        # what the layer's position encoding asks to be done to q and k: a rotation, or nothing
        rot = None if position is None else position.qk_rotation()
        cos = None if rot is None else rot.cos
        sin = None if rot is None else rot.sin
        rotary_dim = 0 if rot is None else rot.rotary_dim
        interleaved = False if rot is None else rot.interleaved
        attn = arena.take((t, self.q_size), ctx.dtype)
        join = None
        if ops.PREFETCH_WEIGHTS and ctx.num_prefill == 0 and ctx.num_decode <= ops.PREFETCH_MAX_ROWS and x_device.type == "cuda":
            # decode: attention streams the cache and leaves bandwidth idle; the weights of the
            # products after it (output projection, feed-forward) come into L2 meanwhile
            ahead = [w for w in [self.w_o, *ctx.upcoming_weights] if w is not None][:8]
            nbytes = sum(w.numel() * w.element_size() for w in ahead)
            if ahead and nbytes <= ops.PREFETCH_MAX_BYTES:
                # at the rate that makes it last as long as the attention kernel is expected to: that
                # kernel's fixed part and the cache it streams
                cache_bytes = 2.0 * ctx.num_decode * min(ctx.max_context_len, ops.PREFETCH_TYPICAL_CONTEXT) \
                    * self.kv_size * self.w_o.element_size()
                beside_us = ops.PREFETCH_ATTENTION_FIXED_US + cache_bytes / (ops.PREFETCH_ATTENTION_GBS * 1e3)
                join = ops.prefetch_l2_beside(ahead, ops.prefetch_threads(nbytes, beside_us))
        if writes_cache and ops.can_fuse_decode(ctx, ctx.dtype, self.num_heads, self.num_kv_heads, self.head_dim,
                                                cache.page_size, cache.k.shape[0], rotary_dim, interleaved,
                                                cache.k.device):
            # decode tokens only: norm, rotation, cache write and attention in one kernel
            ops.decode_attention_fused(qkv, self.q_norm_w, self.k_norm_w, self.qk_norm_eps, cos, sin, group.slots,
                                       cache.k, cache.v, cache.page_size, group.block_tables, ctx, self.scale,
                                       self.window or 0, self.num_heads, attn)
        else:
            q = arena.take((t, self.num_heads, self.head_dim), ctx.dtype)
            ops.qk_norm_rope_write(qkv, q, self.q_norm_w, self.k_norm_w, self.qk_norm_eps, cos, sin, rotary_dim,
                                   interleaved, group.slots, cache.k, cache.v, cache.page_size,
                                   self.num_heads, self.num_kv_heads, self.head_dim, writes_cache)
            ops.paged_attention(q, cache.k, cache.v, cache.page_size, group.block_tables, ctx,
                                self.scale, self.window or 0, attn)
        if join is not None:
            join()
        nxt = ctx.upcoming_caches.get("mixer")
        if (ops.PREFETCH_NEXT_CACHE and join is not None and isinstance(nxt, KVCacheEntry) and nxt.k is not cache.k
                and nxt.group in ctx.kv):
            # the products that follow read their weights from L2 and leave the memory idle: the next
            # layer's pages of these requests come into L2 meanwhile (nothing waits for them)
            later = ops.prefetch_pages_later(nxt.k, nxt.v, ctx.kv[nxt.group].block_tables, ctx, nxt.page_size)
            if not ctx.at_step_end:
                ctx.at_step_end.append(later)
        return project_to_stream(attn, self.w_o, stream, ctx)


class GatedSinkAttention(Mixer):
    """Grouped-query attention with a sink logit per head and a sigmoid output gate.

    ``q = W_q h`` (``num_heads x key_dim``), ``k = W_k h`` (``num_kv_heads x key_dim``),
    ``v = W_v h`` (``num_kv_heads x value_dim``: values may have a head size of their own), no
    biases; optional RMSNorm of q and k per head (plain weights shared by the heads) before the
    rotation that the layer's position encoding asks for; scores ``scale * q . k``, causal; the
    softmax's denominator gets one more term per head, ``exp(sink_h)``, to which no value belongs; the
    concatenated heads are multiplied by ``sigmoid(W_g h)`` and projected by ``W_o``. ``sink="zero"``
    fixes every head's sink logit at 0 (one is added to the denominator; no tensor); ``gate="head"``
    makes ``W_g`` ``[num_heads, hidden]``, one gate value for a whole head; ``window`` limits every
    query to the last ``window`` positions, itself included, and ``keep_first`` (with a window) leaves
    the first ``keep_first`` positions visible to every later query all the same; ``qkv_bias`` adds a
    bias to q, k and v (the projection's name with ``.b`` added) before the norms. ``qk_norm="all"``
    norms q (and k) over the whole projection, all heads together, with weights of that size, instead of
    head by head. ``values="keys"``: there is no ``W_v``; the values are the keys as projected, before norm
    and rotation (``value_dim`` must equal ``key_dim``). With
    ``own_kv=False`` the layer has no key/value tensors and only ever runs as a call that reads
    another call's cache. ``names`` maps the roles "q", "k", "v", "gate", "out", "q_norm",
    "k_norm", "sink" to tensor names after the prefix.

    One product makes q, k, v and the gate's pre-activation; norm, rotation and the cache write are
    one kernel; attention runs over the pages; the gate is applied in 32-bit and rounded once.
    """

    recordable = EVERY_STEP
    _NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink"}

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                 scale: float, qk_norm: bool = True, qk_norm_eps: float = 1e-6, sink: "bool | str" = True,
                 own_kv: bool = True, names: Mapping[str, str] | None = None, window: int | None = None,
                 gate: str = "element", keep_first: int = 0, qkv_bias: bool = False, values: str = "own") -> None:
        if qk_norm not in (True, False, "head", "all"):
            raise ValueError(f"qk_norm={qk_norm!r}: True / 'head' (per head), 'all' (over the whole projection) or False")
        if values not in ("own", "keys") or (values == "keys" and value_dim != key_dim):
            raise ValueError(f"values={values!r}: 'own' (a projection of their own) or 'keys' (then value_dim must equal key_dim)")
        self.norm_whole, self.values_are_keys = qk_norm == "all", values == "keys"
        if self.values_are_keys and qkv_bias:
            raise NotImplementedError("biases on q, k, v together with values that are the keys")
        if keep_first < 0 or (keep_first and window is None):
            raise ValueError(f"keep_first={keep_first} must not be negative and needs a window")
        self.keep_first, self.qkv_bias = int(keep_first), bool(qkv_bias)
        self.b_in = None
        if sink not in (True, False, "zero"):
            raise ValueError(f"sink={sink!r}: True (a learned logit per head), 'zero' (a fixed logit of 0) or False")
        if gate not in ("element", "head"):
            raise ValueError(f"gate={gate!r}: 'element' (a value per output element) or 'head' (one per head)")
        if window is not None and window <= 0:
            raise ValueError(f"window must be positive or None, got {window}")
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        for what, size in (("key_dim", key_dim), ("value_dim", value_dim)):
            if not 0 < size <= 256:
                raise ValueError(f"{what}={size}: the attention kernels take head sizes up to 256")
        self.prefix, self.h = prefix, int(hidden_size)
        self.heads, self.groups, self.d, self.dv = int(num_heads), int(num_kv_heads), int(key_dim), int(value_dim)
        self.scale, self.qk_norm, self.eps = float(scale), bool(qk_norm), float(qk_norm_eps)
        self.has_sink, self.learned_sink, self.own_kv = bool(sink), sink is True, bool(own_kv)
        self.window = None if window is None else int(window)
        self.gate_per_head = gate == "head"
        self.names = {**self._NAMES, **(names or {})}
        self.q_norm_w = self.k_norm_w = self.sink = None

    def cache_need(self) -> "KVNeed | SplitKVNeed":
        if self.d == self.dv:
            return KVNeed(self.groups, self.d, self.window, self.keep_first)
        return SplitKVNeed(self.groups, self.d, self.dv, self.window, self.keep_first)

    def _widths(self) -> tuple[int, int, int, int]:
        """Rows of the q, k, v and gate products."""
        return (self.heads * self.d, self.groups * self.d, 0 if self.values_are_keys else self.groups * self.dv,
                self.heads if self.gate_per_head else self.heads * self.dv)

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p, n, h = prefix + self.prefix, self.names, self.h
        q, k, v, g = self._widths()
        if self.own_kv and self.values_are_keys:
            specs = [TensorSpec(p + "qkg", (q + k + g, h), merged_from=tuple(p + n[r] for r in ("q", "k", "gate")),
                                merged_rows=(q, k, g))]
        elif self.own_kv:
            specs = [TensorSpec(p + "qkvg", (q + k + v + g, h), merged_from=tuple(p + n[r] for r in ("q", "k", "v", "gate")),
                                merged_rows=(q, k, v, g))]
        else:
            specs = [TensorSpec(p + "qg", (q + g, h), merged_from=(p + n["q"], p + n["gate"]), merged_rows=(q, g))]
        specs.append(TensorSpec(p + n["out"], (h, self.heads * self.dv)))
        if self.qkv_bias:
            if self.own_kv:
                specs.append(TensorSpec(p + "qkv.b", (q + k + v,), merged_from=tuple(p + n[r] + ".b" for r in ("q", "k", "v")),
                                        merged_rows=(q, k, v)))
            else:
                specs.append(TensorSpec(p + n["q"] + ".b", (q,)))
        if self.qk_norm:
            specs.append(TensorSpec(p + n["q_norm"], (q if self.norm_whole else self.d,), init="one_plus_normal"))
            if self.own_kv:
                specs.append(TensorSpec(p + n["k_norm"], (k if self.norm_whole else self.d,), init="one_plus_normal"))
        if self.learned_sink:
            specs.append(TensorSpec(p + n["sink"], (self.heads,), std=1.0))
        return specs

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = prefix + self.prefix, self.names
        self.w_in = tensors[p + (("qkg" if self.values_are_keys else "qkvg") if self.own_kv else "qg")]
        self.w_o = tensors[p + n["out"]]
        if self.qkv_bias:
            self.b_in = tensors[p + ("qkv.b" if self.own_kv else n["q"] + ".b")]
        if self.qk_norm:
            self.q_norm_w = tensors[p + n["q_norm"]]
            self.k_norm_w = tensors[p + n["k_norm"]] if self.own_kv else None
        if self.learned_sink:
            self.sink = tensors[p + n["sink"]].float().contiguous()
        elif self.has_sink:
            self.sink = torch.zeros(self.heads, dtype=torch.float32, device=self.w_o.device)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: KVCacheEntry, writes_cache: bool, position: Any) -> torch.Tensor:
        if writes_cache != self.own_kv:
            raise RuntimeError("a layer without key/value tensors must read another call's cache, and one with them writes its own")
        t, arena = x.shape[0], ctx.arena
        group = ctx.kv[cache.group]
        q, k, v, g = self._widths()
        proj = arena.take((t, self.w_in.shape[0]), ctx.dtype)
        ops.gemm(x, self.w_in, proj)
        rot = None if position is None else position.qk_rotation()
        if rot is not None and rot.interleaved:
            raise NotImplementedError("this mixer rotates pairs (i, i + rotary_dim / 2) only")
        queries = arena.take((t, self.heads, self.d), ctx.dtype)
        values = proj[:, q: q + k] if self.values_are_keys else proj[:, q + k: q + k + v]
        ops.qkv_prepare(proj[:, :q], proj[:, q: q + k] if writes_cache else None,
                        values if writes_cache else None, self.q_norm_w, self.k_norm_w, self.eps,
                        None if rot is None else rot.cos, None if rot is None else rot.sin,
                        0 if rot is None else rot.rotary_dim, group.slots if writes_cache else None,
                        cache.k if writes_cache else None, cache.v if writes_cache else None, cache.page_size,
                        self.heads, self.groups, self.d, self.dv, queries,
                        q_bias=None if self.b_in is None else self.b_in[:q],
                        k_bias=None if self.b_in is None or not writes_cache else self.b_in[q: q + k],
                        v_bias=None if self.b_in is None or not writes_cache else self.b_in[q + k: q + k + v],
                        norm_whole=self.norm_whole)
        width = self.heads * self.dv
        attn = arena.take((t, width), ctx.dtype)
        ops.paged_attention(queries, cache.k, cache.v, cache.page_size, group.block_tables, ctx, self.scale,
                            self.window or 0, attn, sinks=self.sink, keep_first=self.keep_first)
        gated = arena.take((t, width), ctx.dtype)
        ops.head_norm_gate(attn.view(t, self.heads, self.dv), None, False, proj[:, proj.shape[1] - g:], False, 0.0, gated,
                           gate_per_head=self.gate_per_head)
        out = arena.take((t, self.h), ctx.dtype)
        ops.gemm(gated, self.w_o, out)
        return out


class LatentAttention(Mixer):
    """Attention whose keys and values are made from one low-rank latent vector per token.

    ``q = W_q h``, per head ``nope_dim`` unrotated then ``rope_dim`` rotated elements. ``W_dkv h`` has
    ``rank + rope_dim`` rows: the first ``rank``, RMS-normed with a plain weight, are the latent ``c``;
    the last ``rope_dim`` are a key part shared by all heads, rotated like the queries' (the layer's
    position encoding; its first ``rotary_dim`` elements turn). Head a's unrotated keys are
    ``W_uk,a c`` and its values ``W_uv,a c``; scores ``scale * (q_nope . k_nope + q_rope . k_rope)``,
    causal (optionally only the last ``window`` positions), ordinary softmax; ``W_o`` on the heads.

    Only ``[c, k_rope]`` is cached, one row per token for all heads (``LatentNeed``). The keys'
    up-projection is folded into the queries (``q'_a = W_uk,a^T q_nope,a``, a product per head) so
    that every head scores against the cached row itself, and the values' up-projection is applied
    to the weighted sum of latents (another product per head): attention with one shared key/value
    head whose values are the first ``rank`` elements of its keys.

    ``q_rank``: the queries go through a latent of their own, ``q = W_uq RMSnorm(W_dq h)`` (plain weight, the
    same eps), instead of ``W_q h``. ``sink``: a learned logit per head joins the softmax's denominator
    (unscaled, without a value). ``names`` maps the roles "q", "down", "down_norm", "up_k", "up_v", "out",
    "q_down", "q_down_norm", "q_up", "sink" to tensor names after the prefix."""

    recordable = EVERY_STEP
    _NAMES = {"q": "q", "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "out": "o",
              "q_down": "dq", "q_down_norm": "dq.norm", "q_up": "uq", "sink": "sink"}

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, nope_dim: int, rope_dim: int, value_dim: int,
                 rank: int, scale: float, norm_eps: float, window: int | None = None,
                 names: Mapping[str, str] | None = None, q_rank: int | None = None, sink: bool = False) -> None:
        if q_rank is not None and q_rank <= 0:
            raise ValueError(f"q_rank={q_rank} must be positive or None")
        self.q_rank, self.has_sink = None if q_rank is None else int(q_rank), bool(sink)
        self.sink = None
        if min(num_heads, nope_dim, value_dim, rank) <= 0 or rope_dim < 0:
            raise ValueError("latent attention: heads, head sizes and the latent size must be positive")
        if rank > ops.LATENT_MAX_RANK:
            raise ValueError(f"rank={rank}: the latent attention kernel takes latents up to {ops.LATENT_MAX_RANK}")
        if window is not None and window <= 0:
            raise ValueError(f"window must be positive or None, got {window}")
        self.prefix, self.h = prefix, int(hidden_size)
        self.heads, self.dn, self.dr, self.dv, self.rank = int(num_heads), int(nope_dim), int(rope_dim), int(value_dim), int(rank)
        self.scale, self.eps = float(scale), float(norm_eps)
        self.window = None if window is None else int(window)
        self.names = {**self._NAMES, **(names or {})}

    def cache_need(self) -> LatentNeed:
        return LatentNeed(self.rank + self.dr, self.window)

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p, n, h = prefix + self.prefix, self.names, self.h
        q, down = self.heads * (self.dn + self.dr), self.rank + self.dr
        if self.q_rank is None:
            first = [TensorSpec(p + "q+down", (q + down, h), merged_from=(p + n["q"], p + n["down"]), merged_rows=(q, down))]
        else:
            first = [TensorSpec(p + n["q_down"] + "+" + n["down"], (self.q_rank + down, h), merged_from=(p + n["q_down"], p + n["down"]),
                                merged_rows=(self.q_rank, down)),
                     TensorSpec(p + n["q_down_norm"], (self.q_rank,), init="one_plus_normal"),
                     TensorSpec(p + n["q_up"], (q, self.q_rank))]
        if self.has_sink:
            first.append(TensorSpec(p + n["sink"], (self.heads,), std=1.0))
        return first + [
                TensorSpec(p + n["down_norm"], (self.rank,), init="one_plus_normal"),
                TensorSpec(p + n["up_k"], (self.heads * self.dn, self.rank)),
                TensorSpec(p + n["up_v"], (self.heads * self.dv, self.rank)),
                TensorSpec(p + n["out"], (h, self.heads * self.dv))]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = prefix + self.prefix, self.names
        if self.q_rank is None:
            self.w_in = tensors[p + "q+down"]
        else:
            self.w_in = tensors[p + n["q_down"] + "+" + n["down"]]
            self.q_norm_w, self.w_uq = tensors[p + n["q_down_norm"]], tensors[p + n["q_up"]]
        if self.has_sink:
            self.sink = tensors[p + n["sink"]].float().contiguous()
        self.norm_w = tensors[p + n["down_norm"]]
        self.w_uk = tensors[p + n["up_k"]].view(self.heads, self.dn, self.rank)                    # [H, nope, rank]
        self.w_uv_t = tensors[p + n["up_v"]].view(self.heads, self.dv, self.rank).transpose(1, 2)  # [H, rank, dv] (a view)
        self.w_o = tensors[p + n["out"]]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: KVCacheEntry, writes_cache: bool, position: Any) -> torch.Tensor:
        if not writes_cache:
            raise RuntimeError("a latent attention layer keeps a cache of its own")
        t, arena, hd = x.shape[0], ctx.arena, self.heads
        group = ctx.kv[cache.group]
        qw = hd * (self.dn + self.dr)
        proj = arena.take((t, self.w_in.shape[0]), ctx.dtype)
        ops.gemm(x, self.w_in, proj)
        if self.q_rank is None:
            q_rows, ckr = proj[:, :qw], proj[:, qw:]
        else:
            # the queries' latent: normed in 32-bit (rounded once), then up-projected
            cq = arena.take((t, self.q_rank), ctx.dtype)
            ops.rms_norm_rows(proj[:, : self.q_rank], self.q_norm_w, self.eps, cq)
            q_rows, ckr = arena.take((t, qw), ctx.dtype), proj[:, self.q_rank:]
            ops.gemm(cq, self.w_uq, q_rows)
        # the keys' up-projection folded into the queries, head by head: [H, T, nope] x [H, nope, rank]
        q_nope = q_rows.view(t, hd, self.dn + self.dr)[:, :, : self.dn].transpose(0, 1)
        folded = arena.take((hd, t, self.rank), ctx.dtype)
        ops.bmm(q_nope, self.w_uk, folded)
        rot = None if position is None else position.qk_rotation()
        queries = arena.take((t, hd, self.rank + self.dr), ctx.dtype)
        rows = cache.k.view(-1, self.rank + self.dr)
        ops.latent_prepare(q_rows, folded, ckr, self.norm_w, self.eps,
                           None if rot is None else rot.cos, None if rot is None else rot.sin,
                           0 if rot is None else rot.rotary_dim, False if rot is None else rot.interleaved,
                           group.slots, rows, hd, self.dn, self.rank, self.dr, queries)
        mixed = arena.take((t, hd, self.rank), ctx.dtype)
        ops.latent_attention(queries, rows, cache.page_size, group.block_tables, ctx, self.rank, self.scale,
                             self.window or 0, mixed, sinks=self.sink)
        # the values' up-projection, head by head: [H, T, rank] x [H, rank, dv], then back to token-major
        by_head = arena.take((hd, t, self.dv), ctx.dtype)
        ops.bmm(mixed.transpose(0, 1), self.w_uv_t, by_head)
        heads_out = arena.take((t, hd, self.dv), ctx.dtype)
        ops.transpose01(by_head, heads_out)
        out = arena.take((t, self.h), ctx.dtype)
        ops.gemm(heads_out.view(t, hd * self.dv), self.w_o, out)
        return out


register_mixer("gqa_attention", GQAAttention)
register_mixer("latent_attention", LatentAttention)
register_mixer("gated_sink_attention", GatedSinkAttention)
