"""Plain PyTorch references of the kernels in ``tinyserve_b200.kernels.ops``, one per kernel,
with the same signatures. They run on any device. The GPU tests compare every kernel with its
reference; the host-only tests put them in the kernels' place (``use_references``) to check
the step function, the cache and the scheduler without a GPU.

Formulas: upstream src/tinyserve/layers.py (norm, rotation), src/tinyserve/attention.py
(paged attention), src/tinyserve/sampling.py (sampling).
"""

from __future__ import annotations

import math
from contextlib import contextmanager
from typing import Any

import numpy as np
import torch


def _round(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return x.to(dtype).float()


def embed(tokens, table, out, scale=1.0) -> None:
    out.copy_(table[tokens.long()].float() * scale)


def add_rms_norm(resid, delta, weight, eps, out, rows=None) -> None:
    x = resid if rows is None else resid[rows.long()]
    if delta is not None:
        x = x + (delta if rows is None else delta[rows.long()]).float()
        if rows is None:
            resid.copy_(x)
    n = _round(x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps), out.dtype)
    out.copy_((n * weight.float()).to(out.dtype))


def post_norm_add_rms_norm(resid, delta, post_weight, layer_scale, post_eps, post_offset, weight, offset, eps, out,
                           rows=None, post_mult=1.0, delta_bias=None) -> None:
    x = resid if rows is None else resid[rows.long()]
    if delta is not None:
        y = (delta if rows is None else delta[rows.long()]).float()
        if delta_bias is not None:
            y = y + delta_bias.float()
        if post_weight is not None:
            g = post_weight.float()
            y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + post_eps) * (1 + g if post_offset else g) * post_mult
        if layer_scale is not None:
            y = y * layer_scale.float()
        x = x + y
        if rows is None:
            resid.copy_(x)
    g = weight.float()
    out.copy_((x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (1 + g if offset else g)).to(out.dtype))


def rope_tables(positions, inv_freq, cos, sin) -> None:
    a = positions.double()[:, None] * inv_freq[None, :]
    cos.copy_(a.cos().float())
    sin.copy_(a.sin().float())


def silu_mul(gate_up, out) -> None:
    inter = out.shape[1]
    g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    out.copy_((_round(g / (1 + torch.exp(-g)), out.dtype) * u).to(out.dtype))


def _head_norm(x: torch.Tensor, w: torch.Tensor | None, eps: float, dtype: torch.dtype) -> torch.Tensor:
    xf = x.float()
    if w is None:
        return xf
    n = _round(xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps), dtype)
    return _round(n * w.float(), dtype)


def _rotate(x: torch.Tensor, cos, sin, rotary_dim: int, interleaved: bool) -> torch.Tensor:
    if not rotary_dim:
        return x
    rot, rest = x[..., :rotary_dim], x[..., rotary_dim:]
    c, s = cos[:, None, :], sin[:, None, :]
    if interleaved:
        a, b = rot[..., 0::2], rot[..., 1::2]
        o = torch.stack([a * c - b * s, b * c + a * s], dim=-1).flatten(-2)
    else:
        half = rotary_dim // 2
        a, b = rot[..., :half], rot[..., half:]
        o = torch.cat([a * c - b * s, b * c + a * s], dim=-1)
    return torch.cat([o, rest], dim=-1)


def qk_norm_rope_write(qkv, q_out, q_weight, k_weight, eps, cos, sin, rotary_dim, interleaved, slots,
                       k_cache, v_cache, page_size, num_heads, num_kv_heads, head_dim, write_kv) -> None:
    t = q_out.shape[0]
    dt = q_out.dtype
    qs = num_heads * head_dim
    q = qkv[:, :qs].view(t, num_heads, head_dim)
    q = _rotate(_head_norm(q, q_weight, eps, dt), cos, sin, rotary_dim, interleaved)
    q_out.copy_(q.to(dt))
    if not write_kv:
        return
    ks = num_kv_heads * head_dim
    k = qkv[:, qs: qs + ks].view(t, num_kv_heads, head_dim)
    v = qkv[:, qs + ks:].view(t, num_kv_heads, head_dim)
    k = _rotate(_head_norm(k, k_weight, eps, dt), cos, sin, rotary_dim, interleaved).to(dt)
    page, off = slots.long() // page_size, slots.long() % page_size
    k_cache[page, :, off] = k
    v_cache[page, :, off] = v


def paged_attention(q, k_cache, v_cache, page_size, block_tables, ctx: Any, scale, window, out, sinks=None,
                    keep_first=0) -> None:
    """Per request: gather its keys and values from the pages in position order, then plain
    causal (windowed) attention for its new tokens (upstream src/tinyserve/attention.py:62-111)."""
    t, hq, d = q.shape
    hkv = k_cache.shape[1]
    group = hq // hkv
    dv = v_cache.shape[3]
    res = torch.zeros(t, hq, dv, dtype=torch.float32, device=q.device)
    cu = ctx.cu_query_lens.tolist()
    lens = ctx.context_lens_dev.tolist()
    for b in range(ctx.num_seqs):
        r0, n, total = cu[b], cu[b + 1] - cu[b], lens[b]
        pos = torch.arange(total, device=q.device)
        lo = 0
        if window:
            lo = max(0, (total - n) - window + 1)      # pages before this may be gone
        kept = min(int(keep_first), lo) if window else 0    # first positions that stay visible below the window
        pos = torch.cat([pos[:kept], pos[lo:]])
        pages = block_tables[b].long()[pos // page_size]
        k = k_cache[pages, :, pos % page_size].float().repeat_interleave(group, dim=1)   # [keys, Hq, D]
        v = v_cache[pages, :, pos % page_size].float().repeat_interleave(group, dim=1)
        qpos = torch.arange(total - n, total, device=q.device)
        hidden = pos[None, :] > qpos[:, None]
        if window:
            hidden = hidden | ((pos[None, :] <= qpos[:, None] - window) & (pos[None, :] >= int(keep_first)))
        s = torch.einsum("ihd,jhd->hij", q[r0: r0 + n].float(), k) * scale
        s = s.masked_fill(hidden, float("-inf"))
        if sinks is not None:
            # one more column that holds the head's sink logit and carries no value
            s = torch.cat([s, sinks.float()[:, None, None].expand(hq, n, 1)], dim=-1)
            p = torch.softmax(s, -1)[..., :-1]
        else:
            p = torch.softmax(s, -1)
        res[r0: r0 + n] = torch.einsum("hij,jhd->ihd", p, v)
    out.copy_(res.view(t, hq * dv).to(out.dtype))


def gemm(x, w, out) -> None:
    out.copy_((x.float() @ w.float().t()).to(out.dtype))


gemm_simt = gemm


def gemm_swiglu(x, w_gate_up, out, arena=None) -> None:
    inter = out.shape[1]
    gu = torch.empty(x.shape[0], 2 * inter, dtype=x.dtype, device=x.device)
    gemm(x, w_gate_up, gu)
    silu_mul(gu, out)


# ------------------------------------------------------------- hyper-connections
def _hc_rebuilt(lanes, fresh, delta, mix_prev, out_prev):
    if fresh is not None:
        return fresh[None].expand(lanes.shape[0], -1, -1).clone()
    if delta is None:
        return lanes.clone()
    return torch.einsum("st,sih->tih", mix_prev, lanes) + out_prev[:, None, None] * delta.float()[None]


def hc_mix_norm(lanes, fresh, delta, mix_prev, out_prev, in_next, norm_weight, eps, out) -> None:
    new = _hc_rebuilt(lanes, fresh, delta, mix_prev, out_prev)
    lanes.copy_(new)
    u = torch.einsum("s,sih->ih", in_next, new)
    out.copy_((u * torch.rsqrt(u.pow(2).mean(-1, keepdim=True) + eps) * norm_weight.float()).to(out.dtype))


def hc_collapse(lanes, fresh, delta, mix_prev, out_prev, rows, out) -> None:
    total = _hc_rebuilt(lanes, fresh, delta, mix_prev, out_prev).sum(0)
    out.copy_(total if rows is None else total[rows.long()])


# ---------------------------------------------------------------------------- gates
def act_mul(gate_up, out, activation, limit=0.0, bias=None) -> None:
    inter = out.shape[1]
    g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    if bias is not None:
        g, u = g + bias[:inter].float(), u + bias[inter:].float()
    if activation == "clamped_swish":
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
        out.copy_((g * torch.sigmoid(1.702 * g) * (u + 1)).to(out.dtype))
        return
    if activation == "silu":
        a = g * torch.sigmoid(g)
    else:
        a = 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3)))
    out.copy_((a * u).to(out.dtype))


def gemm_biased_swiglu(x, w_gate_up, bias, out, arena=None) -> None:
    act_mul(x.float() @ w_gate_up.float().t(), out, "silu", bias=bias)


def gemm_gated(x, w_gate_up, out, arena, activation, limit=0.0) -> None:
    if activation == "silu":
        gemm_swiglu(x, w_gate_up, out, arena)
        return
    gu = (x.float() @ w_gate_up.float().t())
    act_mul(gu, out, activation, limit)


def softcap(logits, cap) -> None:
    logits.copy_(cap * torch.tanh(logits / cap))


def head_norm_gate(x, weight, weight_per_head, gate, normalise, eps, out, gate_per_head=False, gate_silu=False) -> None:
    t, heads, w = x.shape
    y = x.float()
    if normalise:
        y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * (weight.float().view(heads, w) if weight_per_head else weight.float().view(1, w))
    if gate is not None:
        z = gate.float().reshape(t, heads, 1 if gate_per_head else w)
        y = y * (z * torch.sigmoid(z) if gate_silu else torch.sigmoid(z))
    out.copy_(y.reshape(out.shape).to(out.dtype))


# ----------------------------------------------------------------- latent attention
def latent_prepare(q_in, q_folded, ckr, norm_weight, eps, cos, sin, rotary_dim, interleaved, slots, cache, heads, nope,
                   rank, rot, q_out) -> None:
    t = q_out.shape[0]
    if slots is not None:
        c = ckr[:, :rank].float()
        c = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * norm_weight.float()
        kr = _rotate(ckr[:, rank:].float().reshape(t, 1, rot), cos, sin, rotary_dim, interleaved).reshape(t, rot)
        cache[slots.long()] = torch.cat([c, kr], -1).to(cache.dtype)
    qr = _rotate(q_in.float().reshape(t, heads, nope + rot)[:, :, nope:], cos, sin, rotary_dim, interleaved)
    q_out.copy_(torch.cat([q_folded.float().transpose(0, 1), qr], -1).to(q_out.dtype))


def latent_attention(q, cache, page_size, block_tables, ctx: Any, rank, scale, window, out, sinks=None) -> None:
    t, heads, d = q.shape
    res = torch.zeros(t, heads, rank, dtype=torch.float32, device=q.device)
    cu = ctx.cu_query_lens.tolist()
    lens = ctx.context_lens_dev.tolist()
    for b in range(ctx.num_seqs):
        r0, n, total = cu[b], cu[b + 1] - cu[b], lens[b]
        lo = max(0, (total - n) - window + 1) if window else 0      # pages before this may be gone
        pos = torch.arange(lo, total, device=q.device)
        rows = cache[block_tables[b].long()[pos // page_size] * page_size + pos % page_size].float()    # [keys, D]
        qpos = torch.arange(total - n, total, device=q.device)
        hidden = pos[None, :] > qpos[:, None]
        if window:
            hidden = hidden | (pos[None, :] <= qpos[:, None] - window)
        s = torch.einsum("ihd,jd->hij", q[r0: r0 + n].float(), rows) * scale
        s = s.masked_fill(hidden, float("-inf"))
        if sinks is not None:        # one more column per head whose value is zero
            s = torch.cat([s, sinks.float().view(heads, 1, 1).expand(heads, n, 1)], -1)
        p = torch.softmax(s, -1)[:, :, : rows.shape[0]]
        res[r0: r0 + n] = torch.einsum("hij,jd->ihd", p, rows[:, :rank])
    out.copy_(res.to(out.dtype))


def bmm(x, w, out) -> None:
    out.copy_(torch.bmm(x.float(), w.float()).to(out.dtype))


def transpose01(x, out) -> None:
    out.copy_(x.transpose(0, 1))


# -------------------------------------------------------------------------- experts
def moe_max_tiles(num_tokens, top, experts, tile_rows=64) -> int:
    picks = num_tokens * top
    return max(1, min(picks, picks // tile_rows + experts))


def moe_tile_rows(num_tokens, top, experts, dtype, widths) -> int:
    return 64


def moe_route_from(x, w_router, top, counts, arena=None, tile_rows=64, rule=None, outputs=None) -> dict:
    return moe_route(x.float() @ w_router.float().t(), top, counts, arena, tile_rows, rule, outputs)


def moe_route(logits, top, counts, arena=None, tile_rows=64, rule=None, outputs=None) -> dict:
    """The same plan as the kernels make, with the rows of an expert in token order. ``rule``: an object with
    ``scored, groups, keep, scale, identity, correction`` (None: the largest logits, soft-maxed alone)."""
    t = logits.shape[0]
    e = logits.shape[1] if outputs is None else outputs
    z = logits[:, :e].float()
    identity = 0
    if rule is None or not rule.scored:
        # value down, index up: a stable sort of the negated logits
        order = torch.sort(-z, dim=-1, stable=True).indices[:, :top]
        weights = torch.softmax(torch.gather(z, 1, order), -1)
    else:
        identity = rule.identity
        scores = torch.exp(z - z.max(-1, keepdim=True).values)
        scores = scores / scores.sum(-1, keepdim=True)
        choice = scores if rule.correction is None else scores + rule.correction.float()
        if rule.groups > 1:
            best = choice.view(t, rule.groups, -1).max(-1).values
            kept = torch.sort(-best, dim=-1, stable=True).indices[:, : rule.keep]
            allowed = torch.zeros(t, rule.groups, dtype=torch.bool, device=z.device).scatter_(1, kept, True)
            choice = choice.masked_fill(~allowed.repeat_interleave(e // rule.groups, dim=1), float("-inf"))
        order = torch.sort(-choice, dim=-1, stable=True).indices[:, :top]
        picked = torch.gather(scores, 1, order)
        weights = picked / (picked.sum(-1, keepdim=True) + 1e-20) * rule.scale
    real = e - identity
    ids = order.reshape(-1)
    queued = torch.nonzero(ids < real).reshape(-1)                     # picks of experts with matrices
    by_expert = queued[torch.sort(ids[queued], stable=True).indices]   # sorted row -> pick
    row_of = torch.full_like(ids, -1)
    row_of[by_expert] = torch.arange(by_expert.numel(), device=ids.device)
    token_of = torch.zeros_like(ids)
    token_of[: by_expert.numel()] = by_expert // top
    sizes = torch.bincount(ids[queued], minlength=real)
    offsets = torch.cat([sizes.new_zeros(1), sizes.cumsum(0)])
    return {"top": top, "experts": real, "picks": ids.numel(), "ids": ids.int(), "weights": weights.reshape(-1),
            "row_of": row_of.int(), "token_of": token_of.int(), "offsets": offsets.int(), "logits": logits, "identity": identity,
            "max_tiles": moe_max_tiles(t, top, real, tile_rows), "tile_rows": tile_rows}


def moe_gemm(x, w, out, plan, gated, gather, arena=None) -> None:
    off = plan["offsets"].tolist()
    src = x[plan["token_of"].long()] if gather else x
    n = out.shape[1]
    for e in range(plan["experts"]):
        if off[e + 1] > off[e]:
            z = src[off[e]: off[e + 1]].float() @ w[e].float().t()
            if gated:
                z = z[:, :n] * torch.sigmoid(z[:, :n]) * z[:, n:]
            out[off[e]: off[e + 1]] = z.to(out.dtype)


def moe_combine(y, plan, shared_out, out, x=None, shared_gate=None) -> None:
    t, top = out.shape[0], plan["top"]
    rows = plan["row_of"].long()
    picked = y[rows.clamp(min=0)].float().reshape(t, top, -1)
    if x is not None:                       # an identity pick's output is the token's input
        picked = torch.where((rows < 0).reshape(t, top, 1), x.float().reshape(t, 1, -1), picked)
    total = (picked * plan["weights"].reshape(t, top, 1)).sum(1)
    if shared_out is not None:
        g = 1.0 if shared_gate is None else torch.sigmoid(shared_gate.float()).reshape(t, 1)
        total = total + g * shared_out.float()
    out.copy_(total.to(out.dtype))


# ----------------------------------------------------------------- recurrent mixers
def mlstm_state_size(heads, d, dv) -> int:
    return heads * (d * dv + -(-dv // 32) * (d + 1))


def mlstm_scan(qkv, q_off, k_off, v_off, gates, gate_bias, cap, q_scale, state, ctx, heads, d, dv, out) -> None:
    cu, slots = ctx.cu_query_lens.tolist(), ctx.state_slots.tolist()
    nblk = -(-dv // 32)
    per_head = d * dv + nblk * (d + 1)
    x = qkv.float()
    for b in range(ctx.num_seqs):
        st = state[slots[b]].view(heads, per_head)
        for h in range(heads):
            S = st[h, : d * dv].view(d, dv).clone()
            n = st[h, d * dv: d * dv + d].clone()
            m = st[h, d * dv + d].clone()
            for t in range(cu[b], cu[b + 1]):
                q = x[t, q_off + h * d: q_off + (h + 1) * d] * q_scale
                k = x[t, k_off + h * d: k_off + (h + 1) * d]
                v = x[t, v_off + h * dv: v_off + (h + 1) * dv]
                li = cap * torch.tanh((gates[t, h] + gate_bias[h]) / cap)
                lf = torch.nn.functional.logsigmoid(cap * torch.tanh((gates[t, heads + h] + gate_bias[heads + h]) / cap))
                m_new = torch.maximum(lf + m, li)
                keep, take = torch.exp(lf + m - m_new), torch.exp(li - m_new)
                S = keep * S + take * torch.outer(k, v)
                n = keep * n + take * k
                m = m_new
                out[t, h] = (S.t() @ q) / (torch.maximum((n @ q).abs(), torch.exp(-m)) + 1e-6)
            st[h, : d * dv] = S.reshape(-1)
            for blk in range(nblk):
                base = d * dv + blk * (d + 1)
                st[h, base: base + d] = n
                st[h, base + d] = m


def delta_scan(qkv, q_off, k_off, v_off, a, dt_bias, a_log, beta_pre, q_scale, state, ctx, heads, kv_heads, d, dv, out) -> None:
    cu, slots = ctx.cu_query_lens.tolist(), ctx.state_slots.tolist()
    rep = heads // kv_heads
    per_head = a.shape[1] == heads and d != 1
    for b in range(ctx.num_seqs):
        st = state[slots[b]].view(heads, d, dv)
        for h in range(heads):
            g = h // rep
            S = st[h].clone()
            rate = torch.exp(a_log[h])
            for t in range(cu[b], cu[b + 1]):
                q = qkv[t, q_off + g * d: q_off + (g + 1) * d]
                k = qkv[t, k_off + g * d: k_off + (g + 1) * d]
                v = qkv[t, v_off + h * dv: v_off + (h + 1) * dv]
                q = q / torch.sqrt(q.pow(2).sum() + 1e-6) * q_scale
                k = k / torch.sqrt(k.pow(2).sum() + 1e-6)
                cols = slice(h, h + 1) if per_head else slice(h * d, (h + 1) * d)
                decay = torch.exp(-rate * torch.nn.functional.softplus(a[t, cols] + dt_bias[cols]))
                S = decay[:, None] * S
                u = torch.sigmoid(beta_pre[t, h]) * (v - S.t() @ k)
                S = S + torch.outer(k, u)
                out[t, h] = S.t() @ q
            st[h] = S


def causal_conv_silu(x, taps, state, ctx, out) -> None:
    cu, slots = ctx.cu_query_lens.tolist(), ctx.state_slots.tolist()
    c, k = taps.shape
    for b in range(ctx.num_seqs):
        lo, hi = cu[b], cu[b + 1]
        seq = torch.cat([state[slots[b]].view(k - 1, c), x[lo:hi].float()])
        y = sum(seq[j: j + hi - lo] * taps[:, j].float()[None, :] for j in range(k))
        out[lo:hi] = y * torch.sigmoid(y)
        if k > 1:
            state[slots[b]] = seq[-(k - 1):].reshape(-1)


def qkv_prepare(q_in, k_in, v_in, q_weight, k_weight, eps, cos, sin, rotary_dim, slots, k_cache, v_cache, page_size,
                heads, kv_heads, d, dv, q_out, q_bias=None, k_bias=None, v_bias=None, norm_whole=False) -> None:
    t = q_out.shape[0]

    def prep(x, w, n, bias=None):
        y = x.float().reshape(t, n, d)
        if bias is not None:
            y = y + bias.float().view(n, d)
        if w is not None and norm_whole:        # one root mean square over all heads, a weight per element
            y = y * torch.rsqrt(y.pow(2).mean((-2, -1), keepdim=True) + eps) * w.float().view(n, d)
        elif w is not None:
            y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps) * w.float()
        return _rotate(y, cos, sin, rotary_dim, False)

    q_out.copy_(prep(q_in, q_weight, heads, q_bias).to(q_out.dtype))
    if k_in is None:
        return
    page, off = slots.long() // page_size, slots.long() % page_size
    k_cache[page, :, off] = prep(k_in, k_weight, kv_heads, k_bias).to(k_cache.dtype)
    v = v_in.reshape(t, kv_heads, dv)
    if v_bias is not None:
        v = (v.float() + v_bias.float().view(kv_heads, dv)).to(v_cache.dtype)
    v_cache[page, :, off] = v


# ------------------------------------------------- linear attention without a correction term
def _silu(z):
    return z * torch.sigmoid(z)


def linear_scan_bonus(r, k, v, w_pre, w_bias, bonus, state, ctx, heads, d, dv, out) -> None:
    cu, slots = ctx.cu_query_lens.tolist(), ctx.state_slots.tolist()
    for b in range(ctx.num_seqs):
        st = state[slots[b]].view(heads, d, dv)
        for h in range(heads):
            S = st[h].clone()
            u = bonus[h * d: (h + 1) * d].to(state.dtype)
            for t in range(cu[b], cu[b + 1]):
                rr, kk = r[t, h * d: (h + 1) * d].to(state.dtype), k[t, h * d: (h + 1) * d].to(state.dtype)
                vv = v[t, h * dv: (h + 1) * dv].to(state.dtype)
                kv = torch.outer(kk, vv)
                out[t, h] = (S + u[:, None] * kv).t() @ rr
                w = torch.exp(-torch.exp(w_pre[t, h * d: (h + 1) * d] + w_bias[h * d: (h + 1) * d]))
                S = w[:, None] * S + kv
            st[h] = S


def linear_scan_decay(q, k, v, decay, state, ctx, heads, d, dv, out) -> None:
    cu, slots = ctx.cu_query_lens.tolist(), ctx.state_slots.tolist()
    for b in range(ctx.num_seqs):
        st = state[slots[b]].view(heads, d, dv)
        for h in range(heads):
            S = st[h].clone()
            for t in range(cu[b], cu[b + 1]):
                qq, kk = _silu(q[t, h * d: (h + 1) * d].to(state.dtype)), _silu(k[t, h * d: (h + 1) * d].to(state.dtype))
                vv = _silu(v[t, h * dv: (h + 1) * dv].to(state.dtype))
                S = decay[h] * S + torch.outer(kk, vv)
                out[t, h] = S.t() @ qq
            st[h] = S


def linear_scan_gated(q, k, v, w_pre, w_bias, tau, q_scale, state, ctx, heads, d, dv, out) -> None:
    cu, slots = ctx.cu_query_lens.tolist(), ctx.state_slots.tolist()
    for b in range(ctx.num_seqs):
        st = state[slots[b]].view(heads, d, dv)
        for h in range(heads):
            S = st[h].clone()
            for t in range(cu[b], cu[b + 1]):
                qq, kk = q[t, h * d: (h + 1) * d].to(state.dtype) * q_scale, k[t, h * d: (h + 1) * d].to(state.dtype)
                vv = v[t, h * dv: (h + 1) * dv].to(state.dtype)
                z = w_pre[t, h * d: (h + 1) * d] + w_bias[h * d: (h + 1) * d]
                alpha = torch.exp(torch.nn.functional.logsigmoid(z.to(state.dtype)) / tau)
                S = alpha[:, None] * S + torch.outer(kk, vv)
                out[t, h] = S.t() @ qq
            st[h] = S


def rms_norm_rows(x, weight, eps, out) -> None:
    y = x.float()
    out.copy_((y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(out.dtype))


def token_shift_mix(x, mu, state, ctx, out) -> None:
    cu, slots = ctx.cu_query_lens.tolist(), ctx.state_slots.tolist()
    for b in range(ctx.num_seqs):
        lo, hi = cu[b], cu[b + 1]
        if hi <= lo:
            continue
        cur = x[lo:hi].to(state.dtype)
        before = torch.cat([state[slots[b]].view(1, -1), cur[:-1]])
        out[:, lo:hi] = (cur[None] + (before - cur)[None] * mu.to(state.dtype)[:, None, :]).to(out.dtype)
        state[slots[b]] = cur[-1]


# ------------------------------------------------------- around the residual stream
def embed_pos_norm(tokens, positions, table, pos_table, norm_weight, eps, out, scale=1.0) -> None:
    x = table[tokens.long()].float() * scale
    if pos_table is not None:
        x = x + pos_table[positions.long()].float()
    if norm_weight is not None:
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * norm_weight.float()
    out.copy_(x)


def stream_sum(resid, terms, scales, bias=None, bias_scale=1.0, copy=None) -> None:
    x = resid.clone()
    for y, s in zip(terms, scales):
        x = x + float(s) * y.float()
    if bias is not None:
        x = x + float(bias_scale) * bias.float()
    resid.copy_(x)
    if copy is not None:
        copy.copy_(x.to(copy.dtype))


def add_bias(y, bias) -> None:
    y.copy_((y.float() + bias.float()).to(y.dtype))


def tanh_(x) -> None:
    x.copy_(torch.tanh(x.float()).to(x.dtype))


def act_mul_gather(x, rows, table, col0, out, activation) -> None:
    n = out.shape[1]
    z = x.float()
    a = _silu(z) if activation == "silu" else 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
    out.copy_((a * table[rows.long(), col0: col0 + n].float()).to(out.dtype))


# ---------------------------------------------------------------------- sampling
def _philox4x32_10(c: np.ndarray, k0: int, k1: int) -> np.ndarray:
    """c: [N, 4] uint32 counters -> [N, 4] uint32 (Philox4x32 with 10 rounds)."""
    c = c.astype(np.uint64)
    k0, k1 = np.uint64(k0), np.uint64(k1)
    m0, m1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
    mask = np.uint64(0xFFFFFFFF)
    c0, c1, c2, c3 = c[:, 0], c[:, 1], c[:, 2], c[:, 3]
    for _ in range(10):
        p0, p1 = m0 * c0, m1 * c2
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & mask, p1 >> np.uint64(32), p1 & mask
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & mask, lo1, (hi0 ^ c3 ^ k1) & mask, lo0
        k0 = (k0 + np.uint64(0x9E3779B9)) & mask
        k1 = (k1 + np.uint64(0xBB67AE85)) & mask
    return np.stack([c0, c1, c2, c3], axis=1).astype(np.uint32)


def exponential_noise(vocab: int, seed: int, draw: int) -> torch.Tensor:
    """E_i = -log(u_i): u_i from Philox keyed by the seed, counter (i // 4, draw), word i % 4,
    mapped to the 24-bit grid ((x >> 8) + 0.5) / 2^24."""
    n4 = (vocab + 3) // 4
    c = np.zeros((n4, 4), dtype=np.uint32)
    c[:, 0] = np.arange(n4, dtype=np.uint32)
    c[:, 1] = draw & 0xFFFFFFFF
    c[:, 2] = (draw >> 32) & 0xFFFFFFFF
    bits = _philox4x32_10(c, seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF).reshape(-1)[:vocab]
    u = ((bits >> 8).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
    return -torch.log(torch.from_numpy(u))


def sample(logits, out, temperature=None, top_p=None, seeds=None, draws=None, status_out=None) -> None:
    """Greedy rows: first argmax. Others (upstream src/tinyserve/sampling.py:56-102, with
    this framework's noise): p = softmax(logits / T); with top_p < 1 keep tokens whose strictly
    more likely tokens hold less than top_p; pick argmax of log p - log E."""
    r, v = logits.shape
    res = []
    for b in range(r):
        row = logits[b].float().cpu()
        temp = 0.0 if temperature is None else float(temperature[b])
        if not temp > 0:
            res.append(int(row.argmax()))
            continue
        z = row * (np.float32(1.0) / np.float32(temp))
        e = torch.exp(z - z.max())
        keep = torch.ones(v, dtype=torch.bool)
        tp = 1.0 if top_p is None else float(top_p[b])
        if tp < 1:
            total = e.sum()
            order = torch.argsort(e, descending=True, stable=True)
            es = e[order]
            above = torch.cumsum(es, 0) - es
            # tokens of equal probability share the mass above the first of them
            first = torch.searchsorted(-es, -es, right=False)
            above = above[first]
            keep_sorted = above < tp * total
            keep = torch.zeros(v, dtype=torch.bool)
            keep[order] = keep_sorted
        noise = exponential_noise(v, int(seeds[b]), int(draws[b]))
        score = torch.where(keep, z - torch.log(noise), torch.full_like(z, -math.inf))
        res.append(int(score.argmax()))
    out.copy_(torch.tensor(res, dtype=torch.int32, device=out.device))
    if status_out is not None:
        status_out.zero_()


_NAMES = ["embed", "add_rms_norm", "rope_tables", "silu_mul", "qk_norm_rope_write", "paged_attention",
          "gemm", "gemm_simt", "gemm_swiglu", "sample", "hc_mix_norm", "hc_collapse", "act_mul", "softcap",
          "head_norm_gate", "mlstm_scan", "delta_scan", "causal_conv_silu", "qkv_prepare", "gemm_gated",
          "post_norm_add_rms_norm", "latent_prepare", "latent_attention", "bmm", "transpose01", "moe_max_tiles", "moe_tile_rows", "moe_route_from",
          "moe_route", "moe_gemm", "moe_combine", "linear_scan_bonus", "linear_scan_decay", "token_shift_mix",
          "embed_pos_norm", "stream_sum", "add_bias", "tanh_", "act_mul_gather", "gemm_biased_swiglu", "linear_scan_gated",
          "rms_norm_rows"]


@contextmanager
def use_references():
    """Put the references in the kernels' place (host-only tests of the engine's logic)."""
    from tinyserve_b200.kernels import ops

    saved = {n: getattr(ops, n) for n in _NAMES}
    try:
        for n in _NAMES:
            setattr(ops, n, globals()[n])
        yield
    finally:
        for n, f in saved.items():
            setattr(ops, n, f)
