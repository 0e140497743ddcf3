"""The operations of the product path, each one a hand-written sm_100a kernel (or, for the
plain bf16 matrix products, the vendor library, as the upstream engine uses one there).

Every function checks its arguments on the host, then launches on the current CUDA stream.
There is no CPU implementation and no alternative backend: without a CUDA device or the
compiled library these functions raise. Tensors are contiguous; ``dt`` below is the model
dtype (bfloat16 or float32) and selects the kernel instantiation.
"""

from __future__ import annotations

import ctypes
import math
import os
from dataclasses import dataclass
from typing import Any, Callable, Sequence

import torch

from . import build

_F32, _BF16 = 0, 1
_c = ctypes
_vp, _i, _f = _c.c_void_p, _c.c_int, _c.c_float


class KernelError(RuntimeError):
    """A kernel refused its arguments or the launch failed."""


_SIGNATURES: dict[str, list[Any]] = {
    "ts_embed": [_vp, _vp, _vp, _i, _i, _i, _i, _f, _vp],
    "ts_add_rms_norm": [_vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp],
    "ts_rope_tables": [_vp, _vp, _vp, _vp, _i, _i, _vp],
    "ts_silu_mul": [_vp, _vp, _i, _i, _i, _vp],
    "ts_qk_norm_rope_write": [_vp, _vp, _vp, _vp, _f, _vp, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "ts_paged_attention_simt": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i,
                                _f, _i, _i, _vp, _vp, _vp, _i, _i, _i, _vp],
    "ts_hc_mix_norm": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _vp],
    "ts_hc_collapse": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "ts_act_mul": [_vp, _vp, _vp, _i, _i, _i, _f, _i, _vp],
    "ts_act_mul_gather": [_vp, _i, _vp, _vp, _i, _i, _i, _vp, _i, _i, _i, _i, _vp],
    "ts_embed_pos_norm": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f, _i, _vp],
    "ts_stream_sum": [_vp, _vp, _vp, _vp, _vp, _f, _f, _f, _f, _i, _vp, _f, _vp, _i, _i, _i, _vp],
    "ts_add_bias": [_vp, _vp, _i, _i, _i, _vp],
    "ts_tanh": [_vp, _c.c_size_t, _i, _vp],
    "ts_linear_scan": [_i, _vp, _i, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _i, _i, _i, _i, _vp, _vp,
                       _f, _f, _vp],
    "ts_token_shift_mix": [_vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _vp, _i, _vp],
    "ts_softcap": [_vp, _c.c_size_t, _f, _vp],
    "ts_rms_norm_rows": [_vp, _c.c_longlong, _vp, _f, _vp, _i, _i, _i, _vp],
    "ts_head_norm_gate": [_vp, _i, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _f, _i, _i, _i, _vp],
    "ts_post_norm_add_rms_norm": [_vp, _vp, _vp, _vp, _f, _i, _f, _vp, _i, _f, _vp, _vp, _i, _i, _vp, _i, _vp],
    "ts_mlstm_scan": [_vp, _i, _i, _i, _i, _vp, _vp, _f, _f, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp],
    "ts_delta_scan": [_vp, _i, _i, _i, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _f, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp],
    "ts_causal_conv_silu": [_vp, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp],
    "ts_qkv_prepare": [_vp, _i, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _f, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i,
                       _i, _i, _vp, _i, _i, _vp],
    "ts_prefill_attention_mma": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _vp],
    "ts_decode_attention_mma": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _vp, _vp,
                                _vp, _vp],
    "ts_decode_attention_mma_slots": [_i],
    "ts_decode_attention_tma": [_vp, _vp, _vp, _vp, _c.c_longlong, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i,
                                _i, _vp, _vp, _vp, _vp, _vp],
    "ts_decode_attention_tma_fused": [_vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _c.c_longlong, _vp, _i, _vp,
                                      _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _vp, _vp, _vp, _vp],
    "ts_decode_attention_tma_slots": [_i],
    "ts_prefill_attention_tma": [_vp, _vp, _vp, _vp, _c.c_longlong, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f,
                                 _i, _vp, _vp],
    "ts_prefill_attention_tcgen05": [_vp, _vp, _vp, _vp, _c.c_longlong, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                                     _f, _i, _i, _vp, _vp, _i, _vp],
    "ts_gemm_skinny_normed": [_vp, _vp, _i, _vp, _f, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "ts_gemm_skinny_to_stream": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "ts_gemm_skinny_to_stream_parts": [_i, _i, _i],
    "ts_prefetch_l2": [_vp, _vp, _i, _i, _vp],
    "ts_prefetch_pages": [_vp, _vp, _c.c_ulonglong, _vp, _i, _vp, _i, _i, _i, _vp],
    "ts_gemm_simt": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "ts_gemm_skinny": [_vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "ts_gemm_skinny_swiglu": [_vp, _vp, _vp, _i, _i, _i, _vp],
    "ts_gemm_tcgen05": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp],
    "ts_gemm_tcgen05_swiglu": [_vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "ts_gemm_tcgen05_gated": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp, _vp],
    "ts_gemm_tcgen05_biased_swiglu": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "ts_gemm_skinny_biased_swiglu": [_vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "ts_gemm_skinny_gated": [_vp, _vp, _vp, _i, _i, _i, _i, _f, _vp],
    "ts_latent_prepare": [_vp, _c.c_longlong, _vp, _vp, _c.c_longlong, _vp, _f, _vp, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i,
                          _i, _i, _i, _vp],
    "ts_latent_attention": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _i, _vp, _vp, _i, _vp, _vp],
    "ts_latent_attention_mma_takes": [_i, _i],
    "ts_moe_route": [_vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _vp],
    "ts_moe_route_fused": [_vp, _vp, _i, _i, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _vp],
    "ts_moe_gather": [_vp, _vp, _vp, _i, _i, _vp, _vp],
    "ts_moe_gemm_tcgen05": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp],
    "ts_moe_gemm": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "ts_moe_combine": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _i, _i, _vp],
    "ts_sample": [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
}
_fns: dict[str, Any] = {}

# Kernel classes launched with programmatic dependent launch in decode steps. Up to 16 rows: all
# classes (the L2 prefetch kernel then starts beside the product before it, and nothing small is
# left that loses from starting early); beyond: the skinny product and the attention kernels.
# Measured on B200 in the recorded decode step of Qwen3-0.6B, all classes against those two:
# batch 8 1.046 / 1.112 ms, 16 1.736 / 1.776 ms, 32 1.839 / 1.796 ms, 64 2.719 / 2.690 ms.
DEFAULT_PDL_MASK = 2 | 4
SMALL_DECODE_PDL_MASK = -1
SMALL_DECODE_ROWS = 16


def decode_pdl_mask(rows: int) -> int:
    return SMALL_DECODE_PDL_MASK if rows <= SMALL_DECODE_ROWS else DEFAULT_PDL_MASK


# Steps that carry prompt portions run large kernels, where starting early costs nothing and
# hides the launch: all classes (2,048-token prefill of Qwen3-0.6B: 7.7 ms against 8.1 ms).
PREFILL_PDL_MASK = -1
_pdl_mask = DEFAULT_PDL_MASK


def use_pdl_mask(mask: int) -> None:
    """Switch the launch-overlap mask if it differs from the current one (cheap to call per step)."""
    global _pdl_mask
    if mask != _pdl_mask:
        set_programmatic_launch(mask)

# Kernels of this library launched so far (library matrix products are not counted).
launch_count = 0


def _fn(name: str) -> Any:
    f = _fns.get(name)
    if f is None:
        lib = build.library()
        if not _fns:
            # first use of the library: overlap the launches of the kernel classes that gain from it
            lib.ts_set_programmatic_launch.argtypes = [_i]
            lib.ts_set_programmatic_launch.restype = None
            lib.ts_set_programmatic_launch(_pdl_mask)      # the default, or what the caller has set already
        f = getattr(lib, name)
        f.argtypes = _SIGNATURES[name]
        f.restype = _i
        _fns[name] = f
    return f


def _check(status: int, name: str, kernels: int = 1) -> None:
    global launch_count
    if status == 0:
        launch_count += kernels
        return
    if status == -1:
        raise KernelError(f"{name}: bad argument")
    if status == -2:
        raise KernelError(f"{name}: size not supported by this kernel")
    if status == -3:
        raise KernelError(f"{name}: the job needs more scratch than the library's fixed array holds")
    raise KernelError(f"{name}: CUDA error {status}")


_stream_stack: list[int] = []


def _stream() -> int:
    if _stream_stack:
        return _stream_stack[-1]
    return torch.cuda.current_stream().cuda_stream


class stream_scope:
    """While it is open, this library's kernels go to the stream that was current when it was
    opened, without asking for the current stream at every launch (that query costs several
    microseconds, as much as the launch). Open it around a step's launches; inside it, change
    the stream only through another ``stream_scope`` opened under the new stream."""

    def __enter__(self) -> "stream_scope":
        _stream_stack.append(torch.cuda.current_stream().cuda_stream if torch.cuda.is_available() else 0)
        return self

    def __exit__(self, *exc: Any) -> None:
        _stream_stack.pop()


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"dtype {dtype} is not supported (float32 or bfloat16)")


def _dev(t: torch.Tensor, name: str, dtype: torch.dtype | None = None) -> int:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


def _opt(t: torch.Tensor | None, name: str, dtype: torch.dtype | None = None) -> int | None:
    return None if t is None else _dev(t, name, dtype)


# ------------------------------------------------------------------ elementwise
def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """``out[t] = float32(table[tokens[t]]) * scale``; tokens int32 ``[T]``, table ``[V, h]`` dt."""
    t, h = out.shape
    if tokens.shape != (t,) or table.shape[1] != h:
        raise KernelError(f"embed: shapes {tuple(tokens.shape)}, {tuple(table.shape)}, {tuple(out.shape)}")
    _check(_fn("ts_embed")(_dev(tokens, "tokens", torch.int32), _dev(table, "table"),
                           _dev(out, "out", torch.float32), t, h, table.shape[0], _code(table.dtype),
                           float(scale), _stream()), "embed")


def add_rms_norm(resid: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                 out: torch.Tensor, rows: torch.Tensor | None = None) -> None:
    """``x = resid (+ delta)``; ``out = dt(x * rsqrt(mean(x^2) + eps)) * weight``.

    Without ``rows`` every row is processed and the sum is written back to ``resid``
    (float32). With ``rows`` (int32) only those rows are read, ``out`` has one row per entry
    and ``resid`` is left unchanged."""
    h = resid.shape[1]
    n = out.shape[0]
    dt = out.dtype
    if weight.shape != (h,) or out.shape[1] != h or (delta is not None and delta.shape != resid.shape):
        raise KernelError("add_rms_norm: shape mismatch")
    if rows is None and n != resid.shape[0]:
        raise KernelError("add_rms_norm: out must have one row per row of resid")
    if rows is not None and rows.shape != (n,):
        raise KernelError("add_rms_norm: rows must have one entry per row of out")
    _check(_fn("ts_add_rms_norm")(_dev(resid, "resid", torch.float32), _opt(delta, "delta", dt),
                                  _dev(weight, "weight", dt), _dev(out, "out"),
                                  _opt(rows, "rows", torch.int32), n, h, float(eps), _code(dt), _stream()),
           "add_rms_norm")


def post_norm_add_rms_norm(resid: torch.Tensor, delta: torch.Tensor | None, post_weight: torch.Tensor | None,
                           layer_scale: torch.Tensor | None, post_eps: float, post_offset: bool, weight: torch.Tensor,
                           offset: bool, eps: float, out: torch.Tensor, rows: torch.Tensor | None = None,
                           post_mult: float = 1.0, delta_bias: torch.Tensor | None = None) -> None:
    """The residual sum with a norm on the pending sub-layer output, and the next norm, in one pass,
    all in 32-bit: ``y = post_mult * delta / sqrt(mean(delta^2) + post_eps) * gain(post_weight) * layer_scale``
    (``post_weight`` / ``layer_scale`` ``None``: that factor is left out; without a ``post_weight``, ``delta_bias``
    (one value per column, dt) is added to ``delta`` first: ``y = (delta + delta_bias) * layer_scale``), ``x = resid + y``,
    ``out = dt(x / sqrt(mean(x^2) + eps) * gain(weight))`` with ``gain(w) = 1 + w`` when the matching
    ``offset`` flag is set, else ``w``. Without ``rows`` the sum is written back to ``resid``; with
    ``rows`` (int32) only those rows are read and ``resid`` stays."""
    h = resid.shape[1]
    n = out.shape[0]
    dt = out.dtype
    if weight.shape != (h,) or out.shape[1] != h or (delta is not None and delta.shape != resid.shape):
        raise KernelError("post_norm_add_rms_norm: shape mismatch")
    if delta_bias is not None and post_weight is not None:
        raise KernelError("post_norm_add_rms_norm: a bias on the pending output goes without a norm on it")
    for name, v in (("post_weight", post_weight), ("layer_scale", layer_scale), ("delta_bias", delta_bias)):
        if v is not None and (delta is None or v.shape != (h,)):
            raise KernelError(f"post_norm_add_rms_norm: {name} needs a pending output and one value per column")
    if (rows is None and n != resid.shape[0]) or (rows is not None and rows.shape != (n,)):
        raise KernelError("post_norm_add_rms_norm: out must have one row per row of resid, or per entry of rows")
    _check(_fn("ts_post_norm_add_rms_norm")(
        _dev(resid, "resid", torch.float32), _opt(delta, "delta", dt), _opt(post_weight, "post_weight", dt),
        _opt(layer_scale, "layer_scale", dt), float(post_eps), int(bool(post_offset)), float(post_mult), _dev(weight, "weight", dt),
        int(bool(offset)), float(eps), _dev(out, "out"), _opt(rows, "rows", torch.int32), n, h, _opt(delta_bias, "delta_bias", dt),
        _code(dt), _stream()), "post_norm_add_rms_norm")


def rope_tables(positions: torch.Tensor, inv_freq: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> None:
    """``cos/sin[t, i] = float32(cos/sin(float64(positions[t]) * inv_freq[i]))``."""
    t, half = cos.shape
    if positions.shape != (t,) or inv_freq.shape != (half,) or sin.shape != cos.shape:
        raise KernelError("rope_tables: shape mismatch")
    _check(_fn("ts_rope_tables")(_dev(positions, "positions", torch.int32), _dev(inv_freq, "inv_freq", torch.float64),
                                 _dev(cos, "cos", torch.float32), _dev(sin, "sin", torch.float32), t, half,
                                 _stream()), "rope_tables")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """``out[t, j] = dt(silu(gate_up[t, j])) * gate_up[t, I + j]``."""
    t, inter = out.shape
    if gate_up.shape != (t, 2 * inter) or gate_up.dtype != out.dtype:
        raise KernelError("silu_mul: shape or dtype mismatch")
    _check(_fn("ts_silu_mul")(_dev(gate_up, "gate_up"), _dev(out, "out"), t, inter, _code(out.dtype), _stream()),
           "silu_mul")


def qk_norm_rope_write(qkv: torch.Tensor, q_out: torch.Tensor, q_weight: torch.Tensor | None,
                       k_weight: torch.Tensor | None, eps: float, cos: torch.Tensor | None,
                       sin: torch.Tensor | None, rotary_dim: int, interleaved: bool, slots: torch.Tensor,
                       k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int, num_heads: int,
                       num_kv_heads: int, head_dim: int, write_kv: bool) -> None:
    """Per (token, head): optional RMSNorm over ``head_dim``, optional rotation of the first
    ``rotary_dim`` elements; q heads go to ``q_out``, k and v heads to the cache at the token's
    slot (only when ``write_kv``; then ``qkv`` rows hold q, k and v, else q alone)."""
    t = q_out.shape[0]
    dt = q_out.dtype
    width = (num_heads + 2 * num_kv_heads) * head_dim if write_kv else num_heads * head_dim
    if qkv.shape != (t, width) or qkv.dtype != dt or tuple(q_out.shape) != (t, num_heads, head_dim):
        raise KernelError("qk_norm_rope_write: qkv/q_out shape or dtype mismatch")
    if k_cache.dtype != dt or v_cache.dtype != dt or k_cache.shape != v_cache.shape:
        raise KernelError("qk_norm_rope_write: cache dtype/shape mismatch")
    if tuple(k_cache.shape[1:]) != (num_kv_heads, page_size, head_dim):
        raise KernelError("qk_norm_rope_write: cache layout must be [pages, kv_heads, page_size, head_dim]")
    if rotary_dim and (cos is None or sin is None or tuple(cos.shape) != (t, rotary_dim // 2)):
        raise KernelError("qk_norm_rope_write: rotary tables missing or of the wrong shape")
    if slots.shape != (t,):
        raise KernelError("qk_norm_rope_write: one slot per token")
    if write_kv:
        _check_indices("qk_norm_rope_write", None, None, page_size, k_cache.shape[0], slots)
    _check(_fn("ts_qk_norm_rope_write")(
        _dev(qkv, "qkv"), _dev(q_out, "q_out"), _opt(q_weight, "q_weight", dt), _opt(k_weight, "k_weight", dt),
        float(eps), _opt(cos, "cos", torch.float32), _opt(sin, "sin", torch.float32), int(rotary_dim),
        int(bool(interleaved)), _dev(slots, "slots", torch.int32), _dev(k_cache, "k_cache"),
        _dev(v_cache, "v_cache"), page_size, t, num_heads, num_kv_heads, head_dim, int(bool(write_kv)),
        _code(dt), _stream()), "qk_norm_rope_write")


# ------------------------------------------------------------------ index checks
# TINYSERVE_B200_CHECK_INDICES=1 (or ``ops.CHECK_INDICES = True``): before a kernel that follows
# block tables or cache slots is launched, the step's indices are read back and checked on the
# host: every block-table entry that the launch can reach names a page of the cache, every slot
# lies inside it. A violation raises ``KernelError`` and nothing is launched, so a corrupted table
# never becomes a read outside the cache. Each check waits for the device: a debugging aid, off in
# serving (the launchers' own host checks of shapes, sizes and alignment are always on). It plays
# the part that device-side index asserts play in a debug build, without a device trap.
CHECK_INDICES = os.environ.get("TINYSERVE_B200_CHECK_INDICES", "") not in ("", "0")


def _check_indices(name: str, block_tables: torch.Tensor | None, ctx: Any, page_size: int, num_pages: int,
                   slots: torch.Tensor | None = None) -> None:
    if not CHECK_INDICES:
        return
    if torch.cuda.is_current_stream_capturing():
        return                       # nothing can be read back while a step is being recorded
    if block_tables is not None:
        lens = ctx.context_lens_dev[: ctx.num_seqs].to(torch.int64)
        if int(lens.min()) < 1:
            raise KernelError(f"{name}: a request of the step holds no token")
        need = (lens + page_size - 1) // page_size
        if int(need.max()) > block_tables.shape[1]:
            raise KernelError(f"{name}: a request needs {int(need.max())} pages, its block table holds {block_tables.shape[1]}")
        cols = torch.arange(block_tables.shape[1], device=block_tables.device)[None, :]
        used = cols < need[:, None]
        bad = used & ((block_tables < 0) | (block_tables >= num_pages))
        if bool(bad.any()):
            row, col = [int(v) for v in bad.nonzero()[0]]
            raise KernelError(f"{name}: block table of request {row}, entry {col} is page {int(block_tables[row, col])}; "
                              f"the cache has pages 0..{num_pages - 1}")
    if slots is not None and slots.numel():
        lo, hi = int(slots.min()), int(slots.max())
        if lo < 0 or hi >= num_pages * page_size:
            raise KernelError(f"{name}: cache slot {lo if lo < 0 else hi} is outside 0..{num_pages * page_size - 1}")


# -------------------------------------------------------------------- attention
# The bf16 prefill kernel for head sizes 64 / 128: "tcgen05" (tensor memory accumulators) or "mma"
# (mma.sync with TMA tiles); and how many query heads of a kv group share a CTA of the former and
# its key / value tiles (0: chosen by the size of the grid, see ``_prefill_heads_per_cta``).
PREFILL_ATTENTION = "tcgen05"
PREFILL_HEADS_PER_CTA = 0
TARGET_DECODE_CTAS = 148 * 4
MIN_KEYS_PER_SPLIT = 64
MAX_SPLITS = 32


def _prefill_heads_per_cta(ctx: Any, num_heads: int, num_kv_heads: int) -> int:
    """Two query heads of a kv group in a CTA share its key and value tiles, which is worth more
    than anything once the pairs alone give every SM a CTA (measured on B200, 16 / 8 heads of 128:
    2,048 tokens 39 us with one head, 46 us with two; 3,072 tokens 79 / 64 us; 8,192 tokens
    428 / 292 us)."""
    if (num_heads // num_kv_heads) % 2:
        return 1
    if PREFILL_HEADS_PER_CTA:
        return PREFILL_HEADS_PER_CTA
    tiles = sum(-(-n // 128) for n in ctx.query_lens if n > 1)
    return 2 if tiles * (num_heads // 2) > 148 else 1


def decode_splits(num_decode: int, num_kv_heads: int, group: int, max_context_len: int) -> int:
    """How many ranges the keys of each decoding request are cut into. Depends only on the
    shape of the step (after upstream src/tinyserve/triton_attention.py:499-510)."""
    passes = (group + 7) // 8 if group > 8 else 1
    ctas = max(1, num_decode * num_kv_heads * passes)
    want = -(-TARGET_DECODE_CTAS // ctas)
    most = max(1, max_context_len // MIN_KEYS_PER_SPLIT)
    return max(1, min(want, most, MAX_SPLITS))


CLUSTER_MERGE = True       # the TMA decode kernel merges 2 to 8 key ranges inside a thread-block cluster
CLUSTER_MAX = 8            # the portable cluster size
CLUSTER_ROOM = 18          # CTA slots left free per CTA of a cluster
CLUSTER_FILL = 0.82        # and clusters of three or more fill at most this much of the machine


def choose_splits(ctas: int, slots: int, most: int, cluster: bool = False) -> int:
    """Key ranges per request for a kernel of which ``slots`` CTAs run at once and that would
    launch ``ctas`` CTAs unsplit. A step that already gives most of the machine a CTA is not cut
    (the merge of the ranges costs more than a partly filled last round of CTAs); fewer CTAs are
    cut until they fill the machine, up to 12 ranges (measured on B200 at batch 1 to 64). Depends
    only on the shape of the step, so a recorded step always replays the same grid.

    ``cluster``: the kernel merges the ranges of a request inside a thread-block cluster, which is
    cheaper but needs all CTAs of a cluster to find room on one GPC at the same moment, while the
    kernel before it is still leaving. The more CTAs a cluster has, the more of the machine must
    stay free for that: measured at batch 1 to 24 (16 / 8 heads of 128), the best number of ranges
    was each time the largest s <= 8 with ``s * ctas <= slots - 18 s`` (batch 8: 5 ranges, 0.95 ms
    a step; 6 ranges, which fill 86% of the slots, 1.04 ms; without clusters 1.02 ms; batch 9: 5 ranges
    fill 81%, 0.97 ms, 4 ranges 0.93 ms; batch 7: 6 ranges, 76%, are the best), except at
    batch 16, where 3 ranges pass that rule and fill 86%: 1.31 ms a step, with now and then a layer
    whose attention takes twice as long, against 1.21 ms with 2 ranges. Hence the second bound on
    what clusters of three or more may fill."""
    if 2 * ctas > slots:
        return 1
    if cluster and CLUSTER_MERGE:
        for s in range(min(CLUSTER_MAX, most, MAX_SPLITS), 1, -1):
            if s * ctas <= slots - CLUSTER_ROOM * s and (s == 2 or s * ctas <= CLUSTER_FILL * slots):
                return s
        return 1
    return max(1, min(slots // ctas, most, 12, MAX_SPLITS))


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int,
                    block_tables: torch.Tensor, ctx: Any, scale: float, window: int, out: torch.Tensor,
                    sinks: torch.Tensor | None = None, keep_first: int = 0) -> None:
    """Causal attention of this step's queries over each request's cached keys and values.

    ``q`` ``[T, Hq, D]`` dt; key cache ``[pages, Hkv, page_size, D]`` dt, value cache the same
    with a head size ``Dv`` of its own; ``block_tables`` ``[B, W]`` int32; ``ctx`` supplies
    ``cu_query_lens``, ``context_lens_dev``, the lists of decoding and prefilling requests and the
    step's maxima. ``window`` 0 means all earlier positions. ``sinks`` (float32 ``[Hq]``,
    optional): a logit per head that joins the softmax's denominator, unscaled, without a value.
    ``keep_first`` (with a window): positions below it stay visible to every later query, whatever
    the window. ``out`` ``[T, Hq * Dv]`` dt."""
    t, hq, d = q.shape
    hkv = k_cache.shape[1]
    dv = v_cache.shape[3]
    dt = q.dtype
    if k_cache.dtype != dt or v_cache.dtype != dt or out.dtype != dt:
        raise KernelError("paged_attention: dtype mismatch")
    if tuple(k_cache.shape[1:]) != (hkv, page_size, d) or tuple(v_cache.shape[:3]) != tuple(k_cache.shape[:3]):
        raise KernelError("paged_attention: cache layout must be [pages, kv_heads, page_size, head_dim]")
    if out.numel() != t * hq * dv or hq % hkv:
        raise KernelError("paged_attention: out shape or head grouping")
    tma_ok = (dt == torch.bfloat16 and d in (64, 128) and dv == d and (page_size == 8 or page_size % 16 == 0)
              and k_cache.shape[0] * hkv * page_size < 2 ** 31)
    # sink logits are known to the tcgen05 prompt kernel, the TMA decode kernel and the CUDA-core
    # kernels; a value head size of its own and odd head sizes to the CUDA-core kernels only
    keep_first = int(keep_first) if window > 0 else 0
    if keep_first < 0:
        raise KernelError("paged_attention: keep_first must not be negative")
    # kept first positions are known to the tcgen05 prompt kernel and the CUDA-core kernels
    simt_only = (dv != d or d % 16 != 0
                 or ((sinks is not None or keep_first > 0) and not (tma_ok and PREFILL_ATTENTION == "tcgen05")))
    if d > 256 or dv > 256:
        raise KernelError(f"paged_attention: head sizes {d}/{dv} must be at most 256")
    if block_tables.dim() != 2 or block_tables.shape[0] != ctx.num_seqs:
        raise KernelError("paged_attention: block_tables must be [requests, width]")
    if sinks is not None and (sinks.shape != (hq,) or sinks.dtype != torch.float32):
        raise KernelError("paged_attention: sinks must be float32, one per query head")
    _check_indices("paged_attention", block_tables, ctx, page_size, k_cache.shape[0])
    num_prefill = ctx.num_prefill
    if simt_only:
        # the CUDA-core kernels know sink logits, a value head size of its own and odd head sizes
        _paged_attention_simt(q, k_cache, v_cache, page_size, block_tables, ctx, scale, window, out, sinks, num_prefill,
                              keep_first)
        return
    if num_prefill and dt == torch.bfloat16 and d <= 128:
        # prefill rows on the tensor cores; the decode rows follow below
        if tma_ok and PREFILL_ATTENTION == "tcgen05":
            # both products as tcgen05.mma with the accumulators in tensor memory
            _check(_fn("ts_prefill_attention_tcgen05")(
                _dev(q, "q"), _dev(out, "out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), k_cache.shape[0],
                _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1],
                _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32),
                _dev(ctx.context_lens_dev, "context_lens", torch.int32),
                _dev(ctx.prefill_seqs, "prefill_seqs", torch.int32), num_prefill, ctx.max_query_len,
                hq, hkv, d, page_size, float(scale), int(window),
                _prefill_heads_per_cta(ctx, hq, hkv),
                _error_word(q.device).data_ptr(), _opt(sinks, "sinks", torch.float32), keep_first, _stream()),
                "prefill_attention_tcgen05")
        elif tma_ok:
            _check(_fn("ts_prefill_attention_tma")(
                _dev(q, "q"), _dev(out, "out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), k_cache.shape[0],
                _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1],
                _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32),
                _dev(ctx.context_lens_dev, "context_lens", torch.int32),
                _dev(ctx.prefill_seqs, "prefill_seqs", torch.int32), num_prefill, ctx.max_query_len,
                hq, hkv, d, page_size, float(scale), int(window), _error_word(q.device).data_ptr(), _stream()),
                "prefill_attention_tma")
        else:
            _check(_fn("ts_prefill_attention_mma")(
                _dev(q, "q"), _dev(out, "out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
                _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1],
                _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32),
                _dev(ctx.context_lens_dev, "context_lens", torch.int32),
                _dev(ctx.prefill_seqs, "prefill_seqs", torch.int32), num_prefill, ctx.max_query_len,
                hq, hkv, d, page_size, float(scale), int(window), _stream()), "prefill_attention_mma")
        num_prefill = 0
        if not ctx.num_decode:
            return
    if keep_first > 0:
        # single tokens over a window and the kept first positions: the CUDA-core kernel, which walks the two
        # runs of keys as one and splits them over CTAs
        _paged_attention_simt(q, k_cache, v_cache, page_size, block_tables, ctx, scale, window, out, sinks, num_prefill, keep_first)
        return
    if dt == torch.bfloat16 and d <= 128:
        # decode rows on the tensor cores too: one CTA per (request, kv group, key range)
        ctas = ctx.num_decode * hkv * (-(-(hq // hkv) // 16))
        tma = tma_ok
        slots = _decode_slots(d, tma)
        splits = choose_splits(ctas, slots, ctx.max_context_len // 64, cluster=tma)
        part_acc = part_ml = None
        if splits > 1:
            part_acc = ctx.arena.take((ctx.num_decode, hq, splits, d), torch.float32)
            part_ml = ctx.arena.take((ctx.num_decode, hq, splits, 2), torch.float32)
        common = (_dev(block_tables, "block_tables", torch.int32), block_tables.shape[1],
                  _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32),
                  _dev(ctx.context_lens_dev, "context_lens", torch.int32),
                  _dev(ctx.decode_seqs, "decode_seqs", torch.int32), ctx.num_decode,
                  hq, hkv, d, page_size, float(scale), int(window), splits,
                  _opt(part_acc, "part_acc"), _opt(part_ml, "part_ml"), _error_word(q.device).data_ptr(), _stream())
        if tma:
            # tiles fetched by the TMA unit (tensor copies, 128-byte swizzle)
            _check(_fn("ts_decode_attention_tma")(
                _dev(q, "q"), _dev(out, "out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
                k_cache.shape[0], *common[:-1], _opt(sinks, "sinks", torch.float32), common[-1]), "decode_attention_tma")
        else:
            # tiles fetched row by row with bulk copies
            _check(_fn("ts_decode_attention_mma")(
                _dev(q, "q"), _dev(out, "out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), *common),
                "decode_attention_mma")
        return
    _paged_attention_simt(q, k_cache, v_cache, page_size, block_tables, ctx, scale, window, out, None, num_prefill)


def _paged_attention_simt(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int,
                          block_tables: torch.Tensor, ctx: Any, scale: float, window: int, out: torch.Tensor,
                          sinks: torch.Tensor | None, num_prefill: int, keep_first: int = 0) -> None:
    t, hq, d = q.shape
    hkv, dv, dt = k_cache.shape[1], v_cache.shape[3], q.dtype
    splits, part_acc, part_ml = 1, None, None
    if ctx.num_decode and dv == d and d % 16 == 0:
        splits = decode_splits(ctx.num_decode, hkv, hq // hkv, ctx.max_context_len)
        if splits > 1:
            part_acc = ctx.arena.take((ctx.num_decode, hq, splits, d), torch.float32)
            part_ml = ctx.arena.take((ctx.num_decode, hq, splits, 2), torch.float32)
    _check(_fn("ts_paged_attention_simt")(
        _dev(q, "q"), _dev(out, "out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
        _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1],
        _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32),
        _dev(ctx.context_lens_dev, "context_lens", torch.int32),
        _dev(ctx.decode_seqs, "decode_seqs", torch.int32), ctx.num_decode,
        _dev(ctx.prefill_seqs, "prefill_seqs", torch.int32), num_prefill, ctx.max_query_len,
        hq, hkv, d, page_size, float(scale), int(window), splits,
        _opt(part_acc, "part_acc"), _opt(part_ml, "part_ml"), _opt(sinks, "sinks", torch.float32), dv,
        int(keep_first), _code(dt), _stream()), "paged_attention",
        kernels=(1 if num_prefill else 0) + (1 if ctx.num_decode else 0))


# The fused decode kernel takes steps of up to this many decode tokens (0 turns it off), and
# only grids that fit the machine at once (and have at least FUSED_DECODE_MIN_CTAS CTAs). Measured
# on B200 (Qwen3-0.6B sizes, 1,024-token contexts): batches 1 to 48 gain 1 to 5 % of the step;
# larger ones (batch 56, 64) repeat the extra work in a second round of CTAs and lose 1 to 4 %.
FUSED_DECODE_MAX_ROWS = 1 << 30
FUSED_DECODE_MIN_CTAS = 0


def can_fuse_decode(ctx: Any, dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                    pages: int, rotary_dim: int, interleaved: bool, device: torch.device) -> bool:
    """Whether :func:`decode_attention_fused` takes this step and gains from it: decode tokens
    only, bf16, a head of 64 or 128, pages of 8 or a multiple of 16 positions, the whole head
    rotated with the rotate-half pairing (or no rotation at all), and a grid that fills the machine
    once. Depends only on the shape of the step, as the choice of the key ranges does."""
    if not (device.type == "cuda" and ctx.num_prefill == 0 and 0 < ctx.num_decode <= FUSED_DECODE_MAX_ROWS
            and dtype == torch.bfloat16 and head_dim in (64, 128) and (page_size == 8 or page_size % 16 == 0)
            and pages * num_kv_heads * page_size < 2 ** 31
            and (rotary_dim == 0 or (rotary_dim == head_dim and not interleaved))):
        return False
    ctas = ctx.num_decode * num_kv_heads * (-(-(num_heads // num_kv_heads) // 16))
    slots = _decode_slots(head_dim, True)
    grid = ctas * choose_splits(ctas, slots, ctx.max_context_len // 64, cluster=True)
    return min(FUSED_DECODE_MIN_CTAS, slots) <= grid <= slots


def decode_attention_fused(qkv: torch.Tensor, q_weight: torch.Tensor | None, k_weight: torch.Tensor | None,
                           eps: float, cos: torch.Tensor | None, sin: torch.Tensor | None, slots: torch.Tensor,
                           k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int,
                           block_tables: torch.Tensor, ctx: Any, scale: float, window: int, num_heads: int,
                           out: torch.Tensor) -> None:
    """:func:`qk_norm_rope_write` and :func:`paged_attention` of a step of decode tokens in one
    kernel: ``qkv`` ``[T, (Hq + 2 Hkv) * D]`` bf16 is the raw output of the qkv product; the new
    keys and values go to the cache at ``slots``; ``out`` ``[T, Hq * D]``. One query per request,
    no intermediate query tensor. Call only when :func:`can_fuse_decode` says so."""
    t = qkv.shape[0]
    hkv, d = k_cache.shape[1], k_cache.shape[3]
    dt = torch.bfloat16
    if qkv.dtype != dt or k_cache.dtype != dt or v_cache.dtype != dt or out.dtype != dt:
        raise KernelError("decode_attention_fused: bfloat16 only")
    if tuple(k_cache.shape[1:]) != (hkv, page_size, d) or k_cache.shape != v_cache.shape:
        raise KernelError("decode_attention_fused: cache layout must be [pages, kv_heads, page_size, head_dim]")
    if num_heads % hkv or qkv.shape != (t, (num_heads + 2 * hkv) * d) or out.numel() != t * num_heads * d:
        raise KernelError("decode_attention_fused: qkv/out shape or head grouping")
    if ctx.num_prefill or ctx.num_decode != t or block_tables.shape[0] != ctx.num_seqs or slots.shape != (t,):
        raise KernelError("decode_attention_fused: a step of decode tokens only, one token per request")
    if (cos is None) != (sin is None) or (cos is not None and tuple(cos.shape) != (t, d // 2)):
        raise KernelError("decode_attention_fused: rotary tables must be [tokens, head_dim / 2]")
    _check_indices("decode_attention_fused", block_tables, ctx, page_size, k_cache.shape[0], slots)
    ctas = t * hkv * (-(-(num_heads // hkv) // 16))
    splits = choose_splits(ctas, _decode_slots(d, True), ctx.max_context_len // 64, cluster=True)
    part_acc = part_ml = None
    if splits > 1:
        part_acc = ctx.arena.take((t, num_heads, splits, d), torch.float32)
        part_ml = ctx.arena.take((t, num_heads, splits, 2), torch.float32)
    _check(_fn("ts_decode_attention_tma_fused")(
        _dev(qkv, "qkv"), _opt(q_weight, "q_weight", dt), _opt(k_weight, "k_weight", dt), float(eps),
        _opt(cos, "cos", torch.float32), _opt(sin, "sin", torch.float32), _dev(slots, "slots", torch.int32),
        _dev(out, "out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), k_cache.shape[0],
        _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1],
        _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32),
        _dev(ctx.context_lens_dev, "context_lens", torch.int32),
        _dev(ctx.decode_seqs, "decode_seqs", torch.int32), t, num_heads, hkv, d, page_size, float(scale),
        int(window), splits, _opt(part_acc, "part_acc"), _opt(part_ml, "part_ml"),
        _error_word(qkv.device).data_ptr(), _stream()), "decode_attention_tma_fused")


_slots_cache: dict[tuple[int, bool], int] = {}


def _decode_slots(head_dim: int, tma: bool) -> int:
    n = _slots_cache.get((head_dim, tma))
    if n is None:
        name = "ts_decode_attention_tma_slots" if tma else "ts_decode_attention_mma_slots"
        n = _slots_cache[(head_dim, tma)] = int(_fn(name)(head_dim))
    return n


# ------------------------------------------------------------------------- gemm
def gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out[M, N] = x[M, K] @ w[N, K]^T`` with 32-bit accumulation. ``x`` and ``w`` share a
    dtype; ``out`` has it too, or is float32 (the logits). float32 inputs run on CUDA cores in
    true 32-bit; bfloat16 inputs use the tensor cores."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or tuple(out.shape) != (m, n) or x.dtype != w.dtype:
        raise KernelError(f"gemm: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)}")
    if out.dtype not in (x.dtype, torch.float32):
        raise KernelError(f"gemm: out dtype {out.dtype} for inputs {x.dtype}")
    if m == 0:
        return
    if x.dtype == torch.float32:
        _check(_fn("ts_gemm_simt")(_dev(x, "x"), _dev(w, "w"), _dev(out, "out"), m, n, k, _F32, _F32, _stream()),
               "gemm")
        return
    if m <= SKINNY_MAX_ROWS and k % 32 == 0 and n % 16 == 0 and (n * k <= SKINNY_MAX_WEIGHTS or out.dtype != x.dtype):
        gemm_skinny(x, w, out)
        return
    if m >= TCGEN05_MIN_ROWS and n >= TCGEN05_MIN_COLS and k % 8 == 0:
        tiles = tcgen05_tiles(m, n, 256)
        if tiles:
            gemm_tcgen05(x, w, out, TCGEN05_PAIR_TILE if tiles == "pairs" else 256)
            return
    _dev(x, "x"), _dev(w, "w"), _dev(out, "out")
    if out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)                       # vendor library matrix product
    else:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)


# Up to this many rows a bf16 product streams the weights through the skinny kernel ...
SKINNY_MAX_ROWS = 16
# ... if the matrix is not larger than this (measured on B200: at the Qwen3-8B and 32B layer
# shapes the vendor library streams 15-35% faster; at the 0.6B shapes and for the output head
# the skinny kernel is level or ahead).
SKINNY_MAX_WEIGHTS = 1 << 24


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """bf16 ``out[M, N] = x[M, K] @ w[N, K]^T`` for M <= 64, K % 32 == 0, N % 16 == 0: weights
    streamed once from HBM into tensor-core fragments (``csrc/gemm_skinny.cu``)."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or tuple(out.shape) != (m, n) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_skinny: shape or dtype mismatch")
    _check(_fn("ts_gemm_skinny")(_dev(x, "x"), _dev(w, "w"), _dev(out, "out"), m, n, k, _code(out.dtype), _stream()),
           "gemm_skinny")


_error_words: dict[torch.device, torch.Tensor] = {}


def _error_word(device: torch.device) -> torch.Tensor:
    """A device int32 that kernels with bounded waits set when a wait ran out."""
    w = _error_words.get(device)
    if w is None:
        w = _error_words[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return w


# What a non-zero error word says (csrc/bounded_wait.cuh).
WAIT_FAILURES = {1: "gemm_tcgen05", 2: "prefill_attention_tcgen05", 3: "prefill_attention_tma",
                 4: "decode_attention_tma", 5: "decode_attention_mma"}


def raise_for_status(code: int, device: torch.device | str | None = None) -> None:
    """Raise ``KernelError`` for a non-zero error word read from the device (and clear the word, so
    that the next step starts clean)."""
    if code == 0:
        return
    for dev, w in _error_words.items():
        if device is None or torch.device(device) == dev:
            w.zero_()
    raise KernelError(f"kernel {WAIT_FAILURES.get(code, code)!r} gave up waiting on its pipeline (a bounded wait "
                      f"ran out): this step's results are not valid")


def check_device_errors() -> None:
    """Raise if a kernel gave up on a bounded wait since the last check (synchronises)."""
    for dev, w in _error_words.items():
        raise_for_status(int(w.item()), dev)


def set_wait_control(cycles: int | None = None, unarmed: bool = False) -> None:
    """How long the kernels' mbarrier waits may last, in clock cycles (``None``: the default, about a
    second), and the test switch ``unarmed`` that makes every kernel skip its copies so that its
    waits run out (``csrc/bounded_wait.cuh``). For the current device; call it with nothing in
    flight, and never with ``unarmed`` outside a test."""
    lib = build.library()
    lib.ts_set_wait_control.argtypes = [_c.c_longlong, _i]
    lib.ts_set_wait_control.restype = _i
    status = lib.ts_set_wait_control(int(cycles or 0), int(bool(unarmed)))
    if status != 0:
        raise KernelError(f"set_wait_control: CUDA error {status}")


# Default output-tile width of the tcgen05 product.
TCGEN05_TILE_N = 256
# 256-row tiles by pairs of CTAs (tcgen05 cta_group::2) where they fill the machine: a CTA then fetches a
# third less from L2 per flop. Measured on B200 (``python bench.py --profile gemm``), 2,048 rows, library /
# one CTA a tile / pairs: Qwen3-8B gate-up 267 / 291 / 275 us, Qwen3-32B gate-up 651 / 739 / 694 us;
# 8,192 rows of the Qwen3-8B o shape 221 / 228 / 194 us; level at the Qwen3-0.6B shapes.
TCGEN05_PAIR = True
TCGEN05_PAIR_TILE = 512      # the value of ``tile_n`` that asks for them
# The tcgen05 kernel takes the bf16 products with at least this many rows and output columns
# (measured on B200 at 2,048 rows: 17.9 / 26.6 / 564 us against the vendor library's 15.3 / 21.5 /
# 473 us for the qkv, gate-up and head shapes of Qwen3-0.6B; narrower outputs leave most SMs
# without a tile and stay with the library until the kernel learns to split K).
TCGEN05_MIN_ROWS = 128
TCGEN05_MIN_COLS = 2048
TCGEN05_MIN_FILL = 0.85
SM_COUNT = 148


def tcgen05_fills_the_machine(m: int, n: int, tile_cols: int) -> bool:
    """Whether the 128 x ``tile_cols`` output tiles of an ``m`` x ``n`` product keep the persistent
    CTAs of the tcgen05 kernel busy: the tiles fill at least 85 % of the rounds they take (one tile
    per SM and round). The kernel does not split K, so fewer tiles than SMs, or a nearly empty last
    round, leave SMs idle for a whole tile's time; those shapes go to the vendor library, which
    cuts them differently. Measured on B200, kernel by kernel (``python bench.py --profile gemm``):
    512 rows of the Qwen3-8B shapes (64 to 96 tiles) 27 / 76 / 30 us against the library's 17 / 42 /
    24 us for o / down / qkv; 2,048 x 5,120 outputs with K = 25,600 (320 tiles, 2.2 rounds) 604
    against 438 us; where the rounds are full the two are within a tenth of each other. (Cutting
    the last round's k blocks over all SMs, with the last CTA to arrive adding a tile's parts in
    the order of K, was written and passed its tests, but the reducing CTA's 128 epilogue threads
    read a tile's 128 to 384 KB of partial sums with 16 KB in flight, which cost 20 us a launch;
    the reduction has to go through bulk copies into the then idle operand buffers first.)"""
    tiles = -(-m // 128) * -(-n // tile_cols)
    rounds = -(-tiles // SM_COUNT)
    return tiles >= TCGEN05_MIN_FILL * rounds * SM_COUNT


def tcgen05_pairs_fill_the_machine(m: int, n: int, tile_cols: int) -> bool:
    """The same for tiles of 256 rows, each computed by a pair of CTAs (one tile per pair of SMs and round)."""
    tiles = -(-m // 256) * -(-n // tile_cols)
    rounds = -(-tiles // (SM_COUNT // 2))
    return tiles >= TCGEN05_MIN_FILL * rounds * (SM_COUNT // 2)


def tcgen05_tiles(m: int, n: int, tile_cols: int) -> str:
    """How the tcgen05 product cuts an ``m`` x ``n`` output: "pairs" (256-row tiles by pairs of CTAs),
    "single" (128-row tiles), or "" when neither fills the machine and the vendor library takes it."""
    if TCGEN05_PAIR and tcgen05_pairs_fill_the_machine(m, n, tile_cols):
        return "pairs"
    return "single" if tcgen05_fills_the_machine(m, n, tile_cols) else ""


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_n: int | None = None) -> None:
    """bf16 ``out[M, N] = x[M, K] @ w[N, K]^T`` with tcgen05.mma, TMA and TMEM
    (``csrc/gemm_tcgen05.cu``); K % 8 == 0, any M and N; out bf16 or float32."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or tuple(out.shape) != (m, n) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tcgen05: shape or dtype mismatch")
    _check(_fn("ts_gemm_tcgen05")(_dev(x, "x"), _dev(w, "w"), _dev(out, "out"), m, n, k, _code(out.dtype),
                                  tile_n or TCGEN05_TILE_N, _error_word(x.device).data_ptr(), _stream()),
           "gemm_tcgen05")


def gemm_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, arena: Any) -> None:
    """``out[M, I] = silu(x Wgate^T) * (x Wup^T)`` with ``w_gate_up`` = gate rows then up rows,
    ``[2 I, K]``. For a few bf16 rows the product and the activation are one kernel (the gate
    and up rows of an output column are computed by the same CTA); otherwise a product into
    scratch from ``arena`` followed by the SiLU-multiply kernel; many bf16 rows of a wide matrix
    take the tcgen05 product with the activation in its epilogue."""
    m, k = x.shape
    inter = out.shape[1]
    if tuple(w_gate_up.shape) != (2 * inter, k) or out.shape[0] != m or out.dtype != x.dtype:
        raise KernelError("gemm_swiglu: shape or dtype mismatch")
    if (x.dtype == torch.bfloat16 and m <= SKINNY_MAX_ROWS and k % 32 == 0 and inter % 16 == 0
            and 2 * inter * k <= SKINNY_MAX_WEIGHTS):
        _check(_fn("ts_gemm_skinny_swiglu")(_dev(x, "x"), _dev(w_gate_up, "w_gate_up"), _dev(out, "out"), m, inter, k,
                                            _stream()), "gemm_swiglu")
        return
    tiles = tcgen05_tiles(m, inter, 128)
    if x.dtype == torch.bfloat16 and m >= TCGEN05_MIN_ROWS and 2 * inter >= TCGEN05_MIN_COLS and k % 8 == 0 and tiles:
        # many rows: the tcgen05 product with the activation in its epilogue
        _check(_fn("ts_gemm_tcgen05_swiglu")(_dev(x, "x"), _dev(w_gate_up, "w_gate_up"), _dev(out, "out"), m, inter, k,
                                             int(tiles == "pairs"), _error_word(x.device).data_ptr(), _stream()),
               "gemm_tcgen05_swiglu")
        return
    gate_up = arena.take((m, 2 * inter), x.dtype)
    gemm(x, w_gate_up, gate_up)
    silu_mul(gate_up, out)


def gemm_biased_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, bias: torch.Tensor, out: torch.Tensor, arena: Any) -> None:
    """``out[M, I] = silu(x Wgate^T + b_gate) * (x Wup^T + b_up)`` with ``bias [2 I]`` (gate, then up) in the model
    dtype; the sums with the biases, the activation and the product of the halves are 32-bit, rounded once. The same
    three routes as :func:`gemm_swiglu`: a few bf16 rows the skinny product, many bf16 rows of a wide matrix the tcgen05
    product, each with the biases and the activation in its epilogue; anything else a product into scratch and the
    activation kernel."""
    m, k = x.shape
    inter = out.shape[1]
    if (tuple(w_gate_up.shape) != (2 * inter, k) or out.shape[0] != m or out.dtype != x.dtype or bias.shape != (2 * inter,)
            or bias.dtype != x.dtype):
        raise KernelError("gemm_biased_swiglu: shape or dtype mismatch")
    if (x.dtype == torch.bfloat16 and m <= SKINNY_MAX_ROWS and k % 32 == 0 and inter % 16 == 0
            and 2 * inter * k <= SKINNY_MAX_WEIGHTS):
        _check(_fn("ts_gemm_skinny_biased_swiglu")(_dev(x, "x"), _dev(w_gate_up, "w_gate_up"), _dev(bias, "bias"), _dev(out, "out"),
                                                   m, inter, k, _stream()), "gemm_biased_swiglu")
        return
    tiles = tcgen05_tiles(m, inter, 128)
    if x.dtype == torch.bfloat16 and m >= TCGEN05_MIN_ROWS and 2 * inter >= TCGEN05_MIN_COLS and k % 8 == 0 and tiles:
        _check(_fn("ts_gemm_tcgen05_biased_swiglu")(_dev(x, "x"), _dev(w_gate_up, "w_gate_up"), _dev(bias, "bias"), _dev(out, "out"),
                                                    m, inter, k, int(tiles == "pairs"), _error_word(x.device).data_ptr(),
                                                    _stream()), "gemm_tcgen05_biased_swiglu")
        return
    gate_up = arena.take((m, 2 * inter), x.dtype)
    gemm(x, w_gate_up, gate_up)
    act_mul(gate_up, out, "silu", bias=bias)


def gemm_gated(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, arena: Any, activation: str,
               limit: float = 0.0) -> None:
    """``out[M, I] = act(x Wgate^T) * (x Wup^T)`` with a choice of activation (``ACTIVATIONS``). "silu"
    is :func:`gemm_swiglu`. "gelu_tanh" and "clamped_swish" (with its ``limit``) take the same three routes: a few bf16 rows the skinny product
    with the activation in the same pass, many bf16 rows of a wide matrix the tcgen05 product with the
    activation in its epilogue, anything else a product into scratch and the activation kernel. The
    activation and the product of the halves are 32-bit, rounded once."""
    if activation == "silu":
        gemm_swiglu(x, w_gate_up, out, arena)
        return
    if activation not in ACTIVATIONS:
        raise KernelError(f"gemm_gated: unknown activation {activation!r}")
    m, k = x.shape
    inter = out.shape[1]
    if tuple(w_gate_up.shape) != (2 * inter, k) or out.shape[0] != m or out.dtype != x.dtype:
        raise KernelError("gemm_gated: shape or dtype mismatch")
    code = ACTIVATIONS[activation]
    if activation == "clamped_swish" and not limit > 0:
        raise KernelError("gemm_gated: the clamped activation needs a positive limit")
    if (x.dtype == torch.bfloat16 and m <= SKINNY_MAX_ROWS and k % 32 == 0 and inter % 16 == 0
            and 2 * inter * k <= SKINNY_MAX_WEIGHTS):
        _check(_fn("ts_gemm_skinny_gated")(_dev(x, "x"), _dev(w_gate_up, "w_gate_up"), _dev(out, "out"), m, inter, k,
                                           code, float(limit), _stream()), "gemm_gated")
        return
    tiles = tcgen05_tiles(m, inter, 128)
    if x.dtype == torch.bfloat16 and m >= TCGEN05_MIN_ROWS and 2 * inter >= TCGEN05_MIN_COLS and k % 8 == 0 and tiles:
        _check(_fn("ts_gemm_tcgen05_gated")(_dev(x, "x"), _dev(w_gate_up, "w_gate_up"), _dev(out, "out"), m, inter, k,
                                            int(tiles == "pairs"), code, float(limit), _error_word(x.device).data_ptr(),
                                            _stream()),
               "gemm_tcgen05_gated")
        return
    gate_up = arena.take((m, 2 * inter), x.dtype)
    gemm(x, w_gate_up, gate_up)
    act_mul(gate_up, out, activation, limit)


# Steps of a few rows (decode) fold the RMSNorm into the products around it: the product that
# writes a sub-layer's output adds it to the residual stream itself and leaves a bf16 copy and the
# rows' sums of squares, and the next product normalises that copy while it loads it. It saves two
# of seven launches per layer. Measured on B200 (Qwen3-0.6B sizes, 1,024-token contexts, with the
# weights prefetched into L2): the decode step gains 6.7 % at batch 1, 6.3 % at 2, 1.3 % at 4,
# 0.9 % at 8. With the 16-row forms of the products in tiles of 16 weight rows it lost 2 % at 16 rows
# (they ran out of registers); with those in tiles of 8 weight rows it gains 1.3 % at 9 rows and is
# level at 12 and 16, hence up to 16 rows, the most the skinny kernels take. (Before the weights were
# prefetched the norm kernels hid behind the next product's weight stream and the fusion gained nothing.)
FUSE_STREAM_NORM = True
STREAM_FUSE_MAX_ROWS = 16


STREAM_FUSE_MAX_WIDTH = 2048      # 128 parts of 16 columns: what a warp of the consumer adds up


def can_stream_fuse(m: int, n: int, k: int, width: int, dtype: torch.dtype, device: torch.device) -> bool:
    """Whether a product of ``m`` rows with an ``[n, k]`` weight matrix can take part in the
    norm fusion (:func:`gemm_to_stream`, :func:`gemm_normed`) on a stream ``width`` wide: what
    the skinny kernel takes."""
    return (FUSE_STREAM_NORM and device.type == "cuda" and dtype == torch.bfloat16 and 0 < m <= STREAM_FUSE_MAX_ROWS
            and k % 32 == 0 and n % 16 == 0 and n * k <= SKINNY_MAX_WEIGHTS
            and width <= STREAM_FUSE_MAX_WIDTH)


def gemm_to_stream(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, resid16: torch.Tensor,
                   sumsq: torch.Tensor) -> torch.Tensor:
    """``resid[M, N] += bf16(x[M, K] @ w[N, K]^T)`` in place (float32 stream); ``resid16`` gets
    the new stream in bf16 and ``sumsq`` (at least ``2 N`` floats of scratch) the rows' sums of squares in
    parts: returned as a view ``[M, parts]`` with ``parts`` = ``N / 16`` or, where the kernel cuts the
    output into tiles of 8 columns, ``N / 8``; both for the product that normalises the stream next
    (:func:`gemm_normed`). bf16, ``M <= 16``."""
    m, k = x.shape
    n = w.shape[0]
    if (w.shape[1] != k or tuple(resid.shape) != (m, n) or resid.dtype != torch.float32 or sumsq.dtype != torch.float32
            or sumsq.numel() < 2 * n or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16
            or tuple(resid16.shape) != (m, n) or resid16.dtype != torch.bfloat16):
        raise KernelError("gemm_to_stream: shape or dtype mismatch")
    _check(_fn("ts_gemm_skinny_to_stream")(_dev(x, "x"), _dev(w, "w"), _dev(resid, "resid"), _dev(resid16, "resid16"),
                                           _dev(sumsq, "sumsq"), m, n, k, _stream()), "gemm_to_stream")
    parts = int(_fn("ts_gemm_skinny_to_stream_parts")(m, n, k))
    return sumsq[: m * parts].view(m, parts)


def gemm_normed(resid16: torch.Tensor, sumsq: torch.Tensor, norm_weight: torch.Tensor, eps: float, w: torch.Tensor,
                out: torch.Tensor, swiglu: bool = False) -> None:
    """``out = rms_norm(resid) @ w^T`` (or its SwiGLU form, ``w`` = gate rows then up rows) where
    the norm is applied inside the product: ``resid16`` ``[M, K]`` bf16 and ``sumsq`` ``[M, parts]`` as
    :func:`gemm_to_stream` returned it (at most 128 parts per row), ``norm_weight`` ``[K]`` bf16."""
    m, k = resid16.shape
    n = out.shape[1]
    if (tuple(w.shape) != ((2 * n if swiglu else n), k) or out.shape[0] != m or resid16.dtype != torch.bfloat16
            or sumsq.dtype != torch.float32 or sumsq.dim() != 2 or sumsq.shape[0] != m or not sumsq.is_contiguous()
            or norm_weight.shape != (k,) or w.dtype != torch.bfloat16 or norm_weight.dtype != torch.bfloat16):
        raise KernelError("gemm_normed: shape or dtype mismatch")
    _check(_fn("ts_gemm_skinny_normed")(_dev(resid16, "resid16"), _dev(sumsq, "sumsq"), int(sumsq.shape[1]),
                                        _dev(norm_weight, "norm_weight"), float(eps), _dev(w, "w"), _dev(out, "out"), m, n,
                                        k, _code(out.dtype), int(bool(swiglu)), _stream()), "gemm_normed")


# -------------------------------------------------------------------- L2 prefetch
# Decode steps of a few requests fetch the weights of the products that follow the attention
# kernel into L2 while that kernel runs (it leaves memory bandwidth idle), from a kernel of their
# own on a side stream (other placements were measured and are worse: csrc/prefetch.cu). Measured on B200 at the
# Qwen3-0.6B sizes with 1,024-token contexts: with their weights in L2 the products take 2.6-3.8 us
# instead of 3.4-5.4 us each; the decode step gains 1.5 % at batch 1 and 4.7 % at batch 8, nothing
# at 16, and loses 3 % from batch 32 on, where attention needs the bandwidth itself. Fetching the
# next layer's first weights as well changed nothing.
PREFETCH_WEIGHTS = True
PREFETCH_MAX_ROWS = 16
PREFETCH_MAX_BYTES = 48 << 20          # per call: well under L2's size
_side_streams: dict[int, "torch.cuda.Stream"] = {}


# The attention kernel of a decode step lasts about this long: a fixed part and its cache at the rate
# it reaches beside the prefetch. A recorded step is recorded for the longest context it may carry,
# so the typical context is assumed for anything longer.
PREFETCH_ATTENTION_FIXED_US = 3.0
PREFETCH_ATTENTION_GBS = 4000.0
PREFETCH_TYPICAL_CONTEXT = 1024
PREFETCH_THREADS = 0             # non-zero: requests per CTA, whatever the step (measurements)
PREFETCH_SM_GBS = 150.0          # what one SM passes on of such requests (measured on B200)
PREFETCH_PIECE = 16 * 1024


def prefetch_threads(total_bytes: int, beside_us: float) -> int:
    """Requests per CTA of the prefetch kernel so that it lasts about ``beside_us`` microseconds (the
    kernel lasts until its requests are served, and it is joined again after the kernel it runs
    beside, so it should end with that one: slower and the step waits for it, faster and it takes
    bandwidth the other kernel could use)."""
    if PREFETCH_THREADS:
        return PREFETCH_THREADS
    ctas = max(1.0, total_bytes / (PREFETCH_SM_GBS * 1e3 * max(beside_us, 1.0)))
    pieces = max(1, total_bytes // PREFETCH_PIECE)
    per_cta = pieces / ctas
    return int(min(128, max(16, 16 * round(per_cta / 16))))


def prefetch_l2(tensors: Sequence[torch.Tensor], threads: int = 128) -> None:
    """Ask for the memory of ``tensors`` (contiguous, on the device; at most 8) to be brought
    into L2. Returns at once; nothing waits for the data. ``threads``: requests of 16 KB per CTA
    (16 to 128 in steps of 16; fewer means more CTAs and a higher rate, see ``prefetch_threads``)."""
    tensors = [t for t in tensors if t is not None and t.numel()]
    if not tensors:
        return
    if len(tensors) > 8:
        raise KernelError("prefetch_l2: at most 8 tensors per call")
    bases = (_c.c_void_p * len(tensors))(*[_dev(t, "tensor") for t in tensors])
    sizes = (_c.c_ulonglong * len(tensors))(*[t.numel() * t.element_size() for t in tensors])
    _check(_fn("ts_prefetch_l2")(bases, sizes, len(tensors), int(threads), _stream()), "prefetch_l2")


def prefetch_l2_beside(tensors: Sequence[torch.Tensor], threads: int = 128) -> "Callable[[], None]":
    """:func:`prefetch_l2` on a stream of its own that starts where the current stream stands,
    so that it runs beside the kernels launched next. Returns the function that makes the
    current stream wait for it again (call it after those kernels; a recording of the step
    needs every side branch joined)."""
    cur = torch.cuda.current_stream()
    side = _side_streams.get(cur.device.index)
    if side is None:
        side = _side_streams[cur.device.index] = torch.cuda.Stream(device=cur.device)
    side.wait_stream(cur)
    with torch.cuda.stream(side), stream_scope():
        prefetch_l2(tensors, threads)
    return lambda: cur.wait_stream(side)


# While the products after the attention kernel read their weights from L2, memory idles: the pages
# that the step's requests hold in the NEXT layer's cache are asked for meanwhile, on a second side
# stream that nothing waits for until the end of the step. Measured on B200 in the recorded decode
# step (Qwen3-0.6B sizes, 1,024-token contexts): batch 1 / 4 / 8 / 16: 0.792 -> 0.775, 0.804 ->
# 0.793, 0.892 -> 0.876, 1.555 -> 1.540 ms. The gain is small because the attention kernel is bound
# by its own chain of latencies more than by where its keys come from (batch 8, kernel alone: 9.7 us
# with the cache in HBM, 8.7 us with it in L2), and it needs the slow rate of 128 requests per CTA:
# at 16 to 32 per CTA the requests disturb the products and the step loses 4 to 7 %.
PREFETCH_NEXT_CACHE = True
PREFETCH_NEXT_CACHE_THREADS = 128
_cache_streams: dict[int, "torch.cuda.Stream"] = {}


def prefetch_pages_later(k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor, ctx: Any,
                         page_size: int) -> "Callable[[], None]":
    """Ask for the cache pages that the step's requests hold in ``k_cache`` / ``v_cache`` to be
    brought into L2, on a stream of its own that starts where the current stream stands and that
    nothing of the step waits for; returns the function that joins it (call it once, at the end of
    the step: a recording needs every side branch joined)."""
    cur = torch.cuda.current_stream()
    side = _cache_streams.get(cur.device.index)
    if side is None:
        side = _cache_streams[cur.device.index] = torch.cuda.Stream(device=cur.device)
    side.wait_stream(cur)
    page_bytes = k_cache[0].numel() * k_cache.element_size()
    with torch.cuda.stream(side), stream_scope():
        _check(_fn("ts_prefetch_pages")(_dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), page_bytes,
                                        _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1],
                                        _dev(ctx.context_lens_dev, "context_lens", torch.int32), ctx.num_seqs,
                                        page_size, PREFETCH_NEXT_CACHE_THREADS, _stream()), "prefetch_pages")
    return lambda: cur.wait_stream(side)


PDL_ELEMENTWISE, PDL_SKINNY, PDL_ATTENTION, PDL_TCGEN05, PDL_SAMPLING, PDL_OTHER = 1, 2, 4, 8, 16, 32


def set_decode_cluster_merge(on: bool) -> None:
    """Whether decode attention merges 2 to 8 key ranges of a request inside a thread-block cluster
    (the default) or through global memory, as it does for more ranges. Same bits either way."""
    lib = build.library()
    lib.ts_set_decode_cluster_merge.argtypes = [_i]
    lib.ts_set_decode_cluster_merge.restype = None
    lib.ts_set_decode_cluster_merge(1 if on else 0)
    global CLUSTER_MERGE
    CLUSTER_MERGE = bool(on)


_TIMELINE_CLASSES = {1: "elementwise", 2: "skinny", 4: "attention", 8: "tcgen05", 16: "sampling", 32: "other"}


def timeline(capacity: int = 1 << 16) -> list[dict[str, Any]]:
    """The kernels launched since the last call, in the order they started on the device: for each
    its class, grid and block size, ``start`` (ns on the device clock when its first CTA began) and
    ``waited`` (ns when that CTA's wait for the kernels before it returned; 0 if its first thread
    never waits). Synchronises the device. Empty unless the library was built with
    ``TINYSERVE_B200_TIMELINE=1`` in the environment (a second, slower build kept apart)."""
    lib = build.library()
    lib.ts_timeline_read.argtypes = [ctypes.c_void_p, _i]
    lib.ts_timeline_read.restype = _i
    buf = (ctypes.c_uint64 * (3 * capacity))()
    n = lib.ts_timeline_read(buf, capacity)
    if n < 0:
        raise KernelError("timeline: CUDA error while reading the records")
    out = []
    for i in range(n):
        tag, start, waited = buf[3 * i], buf[3 * i + 1], buf[3 * i + 2]
        out.append({"class": _TIMELINE_CLASSES.get(tag & 0xFF, str(tag & 0xFF)), "grid": ((tag >> 8) & 0xFFFFF, (tag >> 28) & 0xFFFF),
                    "block": tag >> 44, "start": int(start), "waited": int(waited)})
    out.sort(key=lambda r: r["start"])
    return out


def set_programmatic_launch(on: bool | int) -> None:
    """Launch this library's kernels so that each may start while its predecessor on the stream
    is draining (programmatic dependent launch); every kernel waits for its predecessor before
    it touches data. ``True`` / ``False`` turn it on / off for all kernels; an int is a mask of
    the ``PDL_*`` kernel classes. Off by default."""
    lib = build.library()
    lib.ts_set_programmatic_launch.argtypes = [_i]
    lib.ts_set_programmatic_launch.restype = None
    global _pdl_mask
    mask = (-1 if on else 0) if isinstance(on, bool) else int(on)
    lib.ts_set_programmatic_launch(mask)
    _pdl_mask = mask


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """The CUDA-core product for any dtype pairing ``gemm`` allows (slow; any size)."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or tuple(out.shape) != (m, n) or x.dtype != w.dtype:
        raise KernelError("gemm_simt: shape or dtype mismatch")
    _check(_fn("ts_gemm_simt")(_dev(x, "x"), _dev(w, "w"), _dev(out, "out"), m, n, k, _code(x.dtype),
                               _code(out.dtype), _stream()), "gemm_simt")


# ------------------------------------------------------------- hyper-connections
def hc_mix_norm(lanes: torch.Tensor, fresh: torch.Tensor | None, delta: torch.Tensor | None,
                mix_prev: torch.Tensor | None, out_prev: torch.Tensor | None, in_next: torch.Tensor,
                norm_weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """The residual stream as ``S`` lanes ``lanes [S, T, h]`` float32. In one pass per row: with
    ``fresh`` ``[T, h]`` every lane becomes that row; else with a pending sub-layer output
    ``delta`` ``[T, h]`` dt the lanes are rebuilt, ``x_t <- sum_s mix_prev[s, t] x_s + out_prev[t] delta``;
    then ``u = sum_s in_next[s] x_s`` and ``out = dt(u / sqrt(mean(u^2) + eps) * norm_weight)``."""
    s_, t, h = lanes.shape
    dt = out.dtype
    if tuple(out.shape) != (t, h) or norm_weight.shape != (h,) or in_next.shape != (s_,):
        raise KernelError("hc_mix_norm: shape mismatch")
    if delta is not None and (mix_prev is None or out_prev is None or tuple(mix_prev.shape) != (s_, s_)
                              or out_prev.shape != (s_,) or tuple(delta.shape) != (t, h)):
        raise KernelError("hc_mix_norm: a pending output needs its mix [S, S] and out [S]")
    if fresh is not None and (delta is not None or tuple(fresh.shape) != (t, h)):
        raise KernelError("hc_mix_norm: fresh lanes take no pending output")
    _check(_fn("ts_hc_mix_norm")(
        _dev(lanes, "lanes", torch.float32), _opt(fresh, "fresh", torch.float32), _opt(delta, "delta", dt),
        _opt(mix_prev, "mix_prev", torch.float32), _opt(out_prev, "out_prev", torch.float32),
        _dev(in_next, "in_next", torch.float32), _dev(norm_weight, "norm_weight", dt), _dev(out, "out"),
        s_, t, h, float(eps), _code(dt), _stream()), "hc_mix_norm")


def hc_collapse(lanes: torch.Tensor, fresh: torch.Tensor | None, delta: torch.Tensor | None,
                mix_prev: torch.Tensor | None, out_prev: torch.Tensor | None, rows: torch.Tensor | None,
                out: torch.Tensor) -> None:
    """``out[r] = sum_t x_t`` (float32 ``[R, h]``) at the rows ``rows`` (int32; all rows if
    ``None``), after the pending rebuild of ``hc_mix_norm``; the lanes are left as they are."""
    s_, t, h = lanes.shape
    r = out.shape[0]
    dt = delta.dtype if delta is not None else torch.float32
    if out.shape[1] != h or (rows is None and r != t) or (rows is not None and rows.shape != (r,)):
        raise KernelError("hc_collapse: shape mismatch")
    if delta is not None and (mix_prev is None or out_prev is None):
        raise KernelError("hc_collapse: a pending output needs its mix and out")
    _check(_fn("ts_hc_collapse")(
        _dev(lanes, "lanes", torch.float32), _opt(fresh, "fresh", torch.float32), _opt(delta, "delta"),
        _opt(mix_prev, "mix_prev", torch.float32), _opt(out_prev, "out_prev", torch.float32),
        _opt(rows, "rows", torch.int32), _dev(out, "out", torch.float32), s_, t, r, h, _code(dt), _stream()),
        "hc_collapse")


# --------------------------------------------------------------------------- gates
ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}


def act_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str, limit: float = 0.0,
            bias: torch.Tensor | None = None) -> None:
    """``out[t, j] = dt(act(gate_up[t, j]) * gate_up[t, I + j])`` in 32-bit, rounded once (with
    ``bias [2 I]`` dt, ``bias[j]`` and ``bias[I + j]`` are added to the two factors first);
    ``activation``: "silu", "gelu_tanh" (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))) or
    "clamped_swish": with ``g = min(gate, limit)`` and ``u = clamp(up, -limit, limit)`` the result is
    ``g sigmoid(1.702 g) (u + 1)``."""
    t, inter = out.shape
    if gate_up.shape != (t, 2 * inter) or gate_up.dtype != out.dtype or activation not in ACTIVATIONS:
        raise KernelError("act_mul: shape, dtype or activation")
    if activation == "clamped_swish" and not limit > 0:
        raise KernelError("act_mul: the clamped activation needs a positive limit")
    if bias is not None and (bias.shape != (2 * inter,) or bias.dtype != out.dtype):
        raise KernelError("act_mul: bias must have one value per column of gate_up")
    _check(_fn("ts_act_mul")(_dev(gate_up, "gate_up"), _opt(bias, "bias"), _dev(out, "out"), t, inter, ACTIVATIONS[activation],
                             float(limit), _code(out.dtype), _stream()), "act_mul")


def softcap(logits: torch.Tensor, cap: float) -> None:
    """In place on float32: ``x <- cap * tanh(x / cap)``."""
    _check(_fn("ts_softcap")(_dev(logits, "logits", torch.float32), logits.numel(), float(cap), _stream()), "softcap")


def head_norm_gate(x: torch.Tensor, weight: torch.Tensor | None, weight_per_head: bool, gate: torch.Tensor | None,
                   normalise: bool, eps: float, out: torch.Tensor, gate_per_head: bool = False,
                   gate_silu: bool = False) -> None:
    """Per (token, head) of ``x [T, H, w]`` (float32 or dt): divide by the root mean square over
    ``w`` (``normalise``), multiply by ``weight`` (``[H * w]`` when ``weight_per_head`` else ``[w]``
    shared by the heads) and by ``sigmoid(gate[t, h, :])`` (``gate`` dt, rows of ``H * w`` values,
    possibly a column slice of a wider matrix; with ``gate_per_head`` the gate has ``H`` values a row
    and head ``h`` is multiplied by ``sigmoid(gate[t, h])``; with ``gate_silu`` the gate's value is
    ``z sigmoid(z)`` instead of ``sigmoid(z)``); ``out [T, H * w]`` dt."""
    t, heads, w = x.shape
    dt = out.dtype
    if out.numel() != t * heads * w or x.dtype not in (torch.float32, dt):
        raise KernelError("head_norm_gate: shape or dtype mismatch")
    if weight is not None and weight.numel() != (heads * w if weight_per_head else w):
        raise KernelError("head_norm_gate: weight size")
    gate_stride = 0
    if gate is not None:
        if gate.dtype != dt or gate.shape[0] != t or gate.shape[1] != (heads if gate_per_head else heads * w) or gate.stride(1) != 1:
            raise KernelError("head_norm_gate: gate must be [T, H * w] (or [T, H]) dt with unit column stride")
        gate_stride = gate.stride(0)
    _check(_fn("ts_head_norm_gate")(
        _dev(x, "x"), int(x.dtype == torch.float32), _opt(weight, "weight", dt), w if weight_per_head else 0,
        None if gate is None else gate.data_ptr(), gate_stride, _dev(out, "out"), t, heads, w, int(bool(normalise)),
        float(eps), int(bool(gate_per_head)), int(bool(gate_silu)), _code(dt), _stream()), "head_norm_gate")


def rms_norm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """``out[r] = dt(x[r] / sqrt(mean(x[r]^2) + eps) * weight)`` in 32-bit, rounded once; ``x [R, w]`` dt with unit
    column stride (a column slice of a wider product is fine), ``weight [w]`` dt, ``out [R, w]`` dt contiguous."""
    r, w = out.shape
    dt = out.dtype
    if tuple(x.shape) != (r, w) or x.dtype != dt or x.stride(1) != 1 or not x.is_cuda or weight.shape != (w,):
        raise KernelError("rms_norm_rows: shapes, dtypes or the column stride")
    _check(_fn("ts_rms_norm_rows")(x.data_ptr(), x.stride(0), _dev(weight, "weight", dt), float(eps), _dev(out, "out"), r, w,
                                   _code(dt), _stream()), "rms_norm_rows")


# ---------------------------------------------------------------- recurrent mixers
SCAN_MAX_KEY_DIM = 256
SCAN_MAX_TAPS = 8


def _state_rows(state: torch.Tensor, width: int, name: str) -> tuple[int, int]:
    """Address and row stride of per-slot state ``[slots, width]`` float32: whole rows of the
    slot storage or a column range of them."""
    if (not state.is_cuda or state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != width
            or (width > 1 and state.stride(1) != 1)):
        raise KernelError(f"{name}: state must be float32 [slots, {width}] on the device with unit column stride")
    return state.data_ptr(), state.stride(0)


def mlstm_state_size(heads: int, d: int, dv: int) -> int:
    """Floats of one request's state: per head ``S [d, dv]`` and, per block of 32 value columns,
    a copy of the normaliser ``n [d]`` and the running maximum ``m``."""
    return heads * (d * dv + -(-dv // 32) * (d + 1))


def mlstm_scan(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, gates: torch.Tensor, gate_bias: torch.Tensor,
               cap: float, q_scale: float, state: torch.Tensor, ctx: Any, heads: int, d: int, dv: int,
               out: torch.Tensor) -> None:
    """The mLSTM recurrence over this step's tokens of every request, from and to its state slot.
    ``qkv [T, *]`` dt holds q, k (``heads * d`` each) and v (``heads * dv``) at the given column
    offsets; ``gates [T, 2 * heads]`` float32 the pre-activations of the input and forget gates
    (bias not yet added, ``gate_bias [2 * heads]`` float32); ``state [slots, mlstm_state_size]``
    float32; ``out [T, heads, dv]`` float32 (before the head norm)."""
    t = qkv.shape[0]
    if gates.shape != (t, 2 * heads) or gate_bias.shape != (2 * heads,) or tuple(out.shape) != (t, heads, dv):
        raise KernelError("mlstm_scan: shape mismatch")
    if d > SCAN_MAX_KEY_DIM:
        raise KernelError("mlstm_scan: key size")
    state_ptr, state_stride = _state_rows(state, mlstm_state_size(heads, d, dv), "mlstm_scan")
    _check(_fn("ts_mlstm_scan")(
        _dev(qkv, "qkv"), qkv.shape[1], q_off, k_off, v_off, _dev(gates, "gates", torch.float32),
        _dev(gate_bias, "gate_bias", torch.float32), float(cap), float(q_scale), state_ptr, state_stride,
        _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32), _dev(ctx.state_slots, "state_slots", torch.int32),
        ctx.num_seqs, heads, d, dv, _dev(out, "out", torch.float32), _code(qkv.dtype), _stream()), "mlstm_scan")


def delta_scan(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, a: torch.Tensor, dt_bias: torch.Tensor,
               a_log: torch.Tensor, beta_pre: torch.Tensor, q_scale: float, state: torch.Tensor, ctx: Any,
               heads: int, kv_heads: int, d: int, dv: int, out: torch.Tensor) -> None:
    """The gated delta rule with a decay per key channel (or, when ``a`` has one column per head, one
    decay per head: then ``dt_bias`` is ``[heads]`` too) over this step's tokens, from and to the
    state slot. ``qkv [T, *]`` float32 holds q, k (``kv_heads * d``) and v (``heads * dv``) after
    their convolutions; ``a [T, heads * d]`` float32 the step-size pre-activations, ``dt_bias
    [heads * d]``, ``a_log [heads]``, ``beta_pre [T, heads]`` float32; ``state [slots, heads * d * dv]``
    float32; ``out [T, heads, dv]`` float32. q and k are scaled to unit length inside (q also by
    ``q_scale``); head h reads q/k head ``h // (heads / kv_heads)``."""
    t = qkv.shape[0]
    per_head = a.shape[1] == heads and d != 1
    if a.shape not in ((t, heads * d), (t, heads)) or beta_pre.shape != (t, heads) or tuple(out.shape) != (t, heads, dv):
        raise KernelError("delta_scan: shape mismatch")
    if a.stride(1) != 1 or beta_pre.stride(1) != 1 or a.dtype != torch.float32 or beta_pre.dtype != torch.float32:
        raise KernelError("delta_scan: a and beta_pre must be float32 with unit column stride")
    if dt_bias.shape != (a.shape[1],) or a_log.shape != (heads,) or d > SCAN_MAX_KEY_DIM:
        raise KernelError("delta_scan: parameter or key size")
    state_ptr, state_stride = _state_rows(state, heads * d * dv, "delta_scan")
    _check(_fn("ts_delta_scan")(
        _dev(qkv, "qkv", torch.float32), qkv.shape[1], q_off, k_off, v_off, a.data_ptr(), a.stride(0), int(per_head),
        _dev(dt_bias, "dt_bias", torch.float32), _dev(a_log, "a_log", torch.float32),
        beta_pre.data_ptr(), beta_pre.stride(0), float(q_scale), state_ptr, state_stride,
        _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32), _dev(ctx.state_slots, "state_slots", torch.int32),
        ctx.num_seqs, heads, kv_heads, d, dv, _dev(out, "out", torch.float32), _stream()), "delta_scan")


def causal_conv_silu(x: torch.Tensor, taps: torch.Tensor, state: torch.Tensor, ctx: Any, out: torch.Tensor) -> None:
    """``out[t, c] = silu(sum_k taps[c, k] * in[t - (K - 1 - k), c])`` (float32) per request, where
    tokens before this step come from ``state [slots, (K - 1) * C]`` float32 (zero at a request's
    start); afterwards the state holds the request's last ``K - 1`` inputs. ``x [T, C]`` dt, ``taps [C, K]`` dt."""
    t, c = x.shape
    k = taps.shape[1]
    if taps.shape[0] != c or tuple(out.shape) != (t, c) or taps.dtype != x.dtype or not x.is_cuda or x.stride(1) != 1:
        raise KernelError("causal_conv_silu: shape or dtype mismatch (x may be a column slice with unit column stride)")
    state_ptr, state_stride = _state_rows(state, (k - 1) * c, "causal_conv_silu")
    _check(_fn("ts_causal_conv_silu")(
        x.data_ptr(), x.stride(0), _dev(taps, "taps"), state_ptr, state_stride,
        _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32), _dev(ctx.state_slots, "state_slots", torch.int32),
        ctx.num_seqs, t, c, k, _dev(out, "out", torch.float32), _code(x.dtype), _stream()), "causal_conv_silu",
        kernels=2 if k > 1 else 1)


def linear_scan_bonus(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w_pre: torch.Tensor, w_bias: torch.Tensor,
                      bonus: torch.Tensor, state: torch.Tensor, ctx: Any, heads: int, d: int, dv: int,
                      out: torch.Tensor) -> None:
    """Time mixing with a decay per key channel and a bonus for the current token, over this step's
    tokens of every request, from and to its state slot. Per head: ``o = (S + diag(u) k v^T)^T r``,
    then ``S <- diag(w) S + k v^T`` with ``w = exp(-exp(w_pre + w_bias))``. ``r``, ``k`` ``[T, heads * d]``
    and ``v`` ``[T, heads * dv]`` dt with unit column stride (column slices are fine); ``w_pre``
    ``[T, heads * d]`` float32; ``w_bias``, ``bonus`` ``[heads * d]`` float32; ``state``
    ``[slots, heads * d * dv]`` float32; ``out [T, heads, dv]`` float32."""
    _linear_scan(0, r, k, v, w_pre, w_bias, bonus, None, state, ctx, heads, d, dv, out)


def linear_scan_decay(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
                      ctx: Any, heads: int, d: int, dv: int, out: torch.Tensor) -> None:
    """Linear attention with a constant decay per head: q, k and v pass SiLU (32-bit); per head
    ``S <- decay_h S + k v^T``, ``o = S^T q``. Shapes as for ``linear_scan_bonus``; ``decay [heads]`` float32."""
    _linear_scan(1, q, k, v, None, None, None, decay, state, ctx, heads, d, dv, out)


def linear_scan_gated(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w_pre: torch.Tensor, w_bias: torch.Tensor,
                      tau: float, q_scale: float, state: torch.Tensor, ctx: Any, heads: int, d: int, dv: int,
                      out: torch.Tensor) -> None:
    """Gated linear attention with a decay per key channel and token, ``alpha = sigmoid(w_pre + w_bias)^(1/tau)``
    (formed in 32-bit as ``exp(logsigmoid(.) / tau)``): per head ``S <- diag(alpha) S + k v^T``, ``o = S^T (q_scale q)``
    (the read-out sees the current token's write). Shapes as for ``linear_scan_bonus``."""
    if not tau > 0:
        raise KernelError("linear_scan_gated: tau must be positive")
    _linear_scan(2, q, k, v, w_pre, w_bias, None, None, state, ctx, heads, d, dv, out, inv_tau=1.0 / tau, q_scale=q_scale)


def _linear_scan(mode: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w_pre: torch.Tensor | None,
                 w_bias: torch.Tensor | None, bonus: torch.Tensor | None, decay: torch.Tensor | None,
                 state: torch.Tensor, ctx: Any, heads: int, d: int, dv: int, out: torch.Tensor,
                 inv_tau: float = 0.0, q_scale: float = 1.0) -> None:
    t, dt = q.shape[0], q.dtype
    for name, x, width in (("q", q, heads * d), ("k", k, heads * d), ("v", v, heads * dv)):
        if not x.is_cuda or x.dtype != dt or x.shape != (t, width) or x.stride(1) != 1:
            raise KernelError(f"linear_scan: {name} must be [T, {width}] {dt} with unit column stride on the device")
    if tuple(out.shape) != (t, heads, dv) or d > SCAN_MAX_KEY_DIM:
        raise KernelError("linear_scan: out shape or key size")
    if mode in (0, 2):
        if (w_pre.shape != (t, heads * d) or w_pre.dtype != torch.float32 or w_pre.stride(1) != 1
                or w_bias.shape != (heads * d,) or (mode == 0 and bonus.shape != (heads * d,))):
            raise KernelError("linear_scan: decay pre-activations, their bias or the bonus")
    elif decay.shape != (heads,):
        raise KernelError("linear_scan: one decay per head")
    state_ptr, state_stride = _state_rows(state, heads * d * dv, "linear_scan")
    seg_len, max_segs = linear_scan_segments(ctx.max_query_len, ctx.num_seqs, heads, d, dv)
    seg_state = seg_decay = None
    if max_segs > 1:
        seg_state = ctx.arena.take((ctx.num_seqs * max_segs, heads * d * dv), torch.float32)
        if mode in (0, 2):
            seg_decay = ctx.arena.take((ctx.num_seqs * max_segs, heads * d), torch.float32)
    _check(_fn("ts_linear_scan")(
        mode, q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
        None if w_pre is None else w_pre.data_ptr(), 0 if w_pre is None else w_pre.stride(0),
        _opt(w_bias, "w_bias", torch.float32), _opt(bonus, "bonus", torch.float32), _opt(decay, "decay", torch.float32),
        state_ptr, state_stride, _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32),
        _dev(ctx.state_slots, "state_slots", torch.int32), ctx.num_seqs, heads, d, dv,
        _dev(out, "out", torch.float32), _code(dt), int(ctx.max_query_len), seg_len, max_segs,
        None if seg_state is None else seg_state.data_ptr(), None if seg_decay is None else seg_decay.data_ptr(),
        float(inv_tau), float(q_scale), _stream()),
        "linear_scan", kernels=1 if max_segs <= 1 else (4 if mode in (0, 2) else 3))


# A portion of this many tokens or more is cut into segments that run side by side.
LINEAR_SCAN_SEGMENT_MIN_TOKENS = 256
LINEAR_SCAN_SEGMENT_SCRATCH_BYTES = 256 << 20
LINEAR_SCAN_SEGMENT_TOKENS: int | None = None    # a fixed segment length instead of the choice below (tests)


def linear_scan_segments(max_query_len: int, num_seqs: int, heads: int, d: int, dv: int) -> tuple[int, int]:
    """``(tokens per segment, segments per request)`` for a step whose longest portion has ``max_query_len`` tokens;
    one segment = the plain scan. Segments of 64 tokens while the machine has room for more CTAs than the
    requests, heads and column blocks give, of 128 beyond; longer ones when the segments' states would not fit
    the scratch bound."""
    if max_query_len < LINEAR_SCAN_SEGMENT_MIN_TOKENS:
        return 0, 1
    ctas = num_seqs * heads * ((dv + 31) // 32)
    seg_len = LINEAR_SCAN_SEGMENT_TOKENS or (64 if ctas * ((max_query_len + 127) // 128) < 2 * 148 else 128)
    most = max(1, LINEAR_SCAN_SEGMENT_SCRATCH_BYTES // (4 * heads * d * dv * max(1, num_seqs)))
    if (max_query_len + seg_len - 1) // seg_len > most:
        seg_len = ((max_query_len + most - 1) // most + 15) // 16 * 16
    max_segs = (max_query_len + seg_len - 1) // seg_len
    return (seg_len, max_segs) if max_segs > 1 else (0, 1)


def token_shift_mix(x: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, ctx: Any, out: torch.Tensor) -> None:
    """``out[m, t] = x[t] + (x[t - 1] - x[t]) * mu[m]`` for every mix m, where the row before a
    request's first token of the step comes from ``state [slots, C]`` float32 (zero at the request's
    start); afterwards the state holds the request's last row. ``x [T, C]`` dt, ``mu [M, C]`` dt,
    ``out [M, T, C]`` dt."""
    t, c = x.shape
    m = mu.shape[0]
    if mu.shape != (m, c) or tuple(out.shape) != (m, t, c) or mu.dtype != x.dtype or out.dtype != x.dtype:
        raise KernelError("token_shift_mix: shape or dtype mismatch")
    state_ptr, state_stride = _state_rows(state, c, "token_shift_mix")
    _check(_fn("ts_token_shift_mix")(
        _dev(x, "x"), c, _dev(mu, "mu"), m, state_ptr, state_stride,
        _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32), _dev(ctx.state_slots, "state_slots", torch.int32),
        ctx.num_seqs, t, c, _dev(out, "out"), _code(x.dtype), _stream()), "token_shift_mix")


# ------------------------------------------------------- around the residual stream
def embed_pos_norm(tokens: torch.Tensor, positions: torch.Tensor | None, table: torch.Tensor,
                   pos_table: torch.Tensor | None, norm_weight: torch.Tensor | None, eps: float, out: torch.Tensor,
                   scale: float = 1.0) -> None:
    """``x = float32(table[tokens[t]]) * scale (+ pos_table[positions[t]])``, then, with a norm weight,
    ``x / sqrt(mean(x^2) + eps) * weight``; ``out [T, h]`` float32. An id or a position outside its
    table gives a row of NaN."""
    t, h = out.shape
    dt = table.dtype
    if tokens.shape != (t,) or table.shape[1] != h or (pos_table is not None and (pos_table.shape[1] != h or positions is None)):
        raise KernelError("embed_pos_norm: shape mismatch")
    if norm_weight is not None and norm_weight.shape != (h,):
        raise KernelError("embed_pos_norm: norm weight size")
    _check(_fn("ts_embed_pos_norm")(
        _dev(tokens, "tokens", torch.int32), _opt(positions, "positions", torch.int32), _dev(table, "table"),
        _opt(pos_table, "pos_table", dt), _opt(norm_weight, "norm_weight", dt), _dev(out, "out", torch.float32), t, h,
        table.shape[0], 0 if pos_table is None else pos_table.shape[0], float(scale), float(eps), _code(dt), _stream()),
        "embed_pos_norm")


STREAM_SUM_MAX_TERMS = 4


def stream_sum(resid: torch.Tensor, terms: Sequence[torch.Tensor], scales: Sequence[float],
               bias: torch.Tensor | None = None, bias_scale: float = 1.0, copy: torch.Tensor | None = None) -> None:
    """``resid <- resid + sum_i scales[i] * terms[i] (+ bias_scale * bias)`` in 32-bit; ``copy`` (dt,
    optional) receives the new stream rounded once. ``terms [T, h]`` dt, up to four; ``bias [h]`` dt."""
    t, h = resid.shape
    if len(terms) != len(scales) or len(terms) > STREAM_SUM_MAX_TERMS:
        raise KernelError(f"stream_sum: {len(terms)} terms, {len(scales)} scales (up to {STREAM_SUM_MAX_TERMS})")
    dts = {x.dtype for x in terms} | ({bias.dtype} if bias is not None else set()) | ({copy.dtype} if copy is not None else set())
    if len(dts) > 1:
        raise KernelError("stream_sum: terms, bias and copy share the model dtype")
    dt = dts.pop() if dts else torch.float32
    for x in terms:
        if tuple(x.shape) != (t, h):
            raise KernelError("stream_sum: a term's shape")
    if (bias is not None and bias.shape != (h,)) or (copy is not None and tuple(copy.shape) != (t, h)):
        raise KernelError("stream_sum: bias or copy shape")
    ptrs = [_dev(x, "term") for x in terms] + [None] * (STREAM_SUM_MAX_TERMS - len(terms))
    sc = [float(x) for x in scales] + [0.0] * (STREAM_SUM_MAX_TERMS - len(scales))
    _check(_fn("ts_stream_sum")(_dev(resid, "resid", torch.float32), *ptrs, *sc, len(terms), _opt(bias, "bias"),
                                float(bias_scale), _opt(copy, "copy"), t, h, _code(dt), _stream()), "stream_sum")


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> None:
    """In place: ``y[t, j] += bias[j]`` (32-bit sum, rounded once); ``y [T, n]`` dt, ``bias [n]`` dt."""
    if y.dim() != 2 or bias.shape != (y.shape[1],) or bias.dtype != y.dtype:
        raise KernelError("add_bias: shape or dtype mismatch")
    _check(_fn("ts_add_bias")(_dev(y, "y"), _dev(bias, "bias"), y.shape[0], y.shape[1], _code(y.dtype), _stream()), "add_bias")


def tanh_(x: torch.Tensor) -> None:
    """In place: ``x <- tanh(x)`` (32-bit, rounded once)."""
    _check(_fn("ts_tanh")(_dev(x, "x"), x.numel(), _code(x.dtype), _stream()), "tanh")


def act_mul_gather(x: torch.Tensor, rows: torch.Tensor, table: torch.Tensor, col0: int, out: torch.Tensor,
                   activation: str) -> None:
    """``out[t, j] = dt(act(x[t, j]) * table[rows[t], col0 + j])``: a gate on a row looked up per token
    (``rows`` int32 ``[T]``; a row outside the table gives NaN). ``x [T, n]`` dt with unit column stride."""
    t, n = out.shape
    if (x.shape != (t, n) or x.stride(1) != 1 or x.dtype != out.dtype or table.dtype != out.dtype or rows.shape != (t,)
            or activation not in ("silu", "gelu_tanh") or not 0 <= col0 <= table.shape[1] - n):
        raise KernelError("act_mul_gather: shape, dtype, activation or column range")
    _check(_fn("ts_act_mul_gather")(x.data_ptr(), x.stride(0), _dev(rows, "rows", torch.int32), _dev(table, "table"),
                                    table.shape[0], table.shape[1], int(col0), _dev(out, "out"), t, n,
                                    ACTIVATIONS[activation], _code(out.dtype), _stream()), "act_mul_gather")


def _bias(b: torch.Tensor | None, n: int, name: str, dt: torch.dtype) -> int | None:
    """Address of an optional bias ``[n]`` dt (a slice of a longer vector is fine)."""
    if b is None:
        return None
    if not b.is_cuda or b.dtype != dt or b.shape != (n,) or b.stride(0) != 1:
        raise KernelError(f"{name} must be [{n}] {dt} on the device")
    return b.data_ptr()


def qkv_prepare(q_in: torch.Tensor, k_in: torch.Tensor | None, v_in: torch.Tensor | None, q_weight: torch.Tensor | None,
                k_weight: torch.Tensor | None, eps: float, cos: torch.Tensor | None, sin: torch.Tensor | None,
                rotary_dim: int, slots: torch.Tensor | None, k_cache: torch.Tensor | None, v_cache: torch.Tensor | None,
                page_size: int, heads: int, kv_heads: int, d: int, dv: int, q_out: torch.Tensor,
                q_bias: torch.Tensor | None = None, k_bias: torch.Tensor | None = None,
                v_bias: torch.Tensor | None = None, norm_whole: bool = False) -> None:
    """Per (token, head): optional bias (one value per projection row, dt), optional RMSNorm over the head with a plain weight
    (``norm_whole``: over all heads of q, or of k, together, with weights of ``heads * d`` and ``kv_heads * d`` values), rotation of the first
    ``rotary_dim`` elements (i pairs with i + rotary_dim / 2); queries to ``q_out [T, heads, d]``,
    keys and (unchanged) values to the caches at the tokens' slots (when ``k_in`` is given).
    ``q_in``/``k_in``/``v_in`` are 2-D dt with unit column stride (column slices of a merged
    projection are fine); the value head size ``dv`` may differ from ``d``."""
    t = q_out.shape[0]
    dt = q_out.dtype
    for name, x, width in (("q_in", q_in, heads * d), ("k_in", k_in, kv_heads * d), ("v_in", v_in, kv_heads * dv)):
        if x is not None and (x.dtype != dt or x.shape != (t, width) or x.stride(1) != 1 or not x.is_cuda):
            raise KernelError(f"qkv_prepare: {name} must be [T, {width}] {dt} with unit column stride on the device")
    if tuple(q_out.shape) != (t, heads, d) or (k_in is None) != (v_in is None):
        raise KernelError("qkv_prepare: q_out shape, or keys without values")
    if k_in is not None:
        if tuple(k_cache.shape[1:]) != (kv_heads, page_size, d) or tuple(v_cache.shape[1:]) != (kv_heads, page_size, dv):
            raise KernelError("qkv_prepare: cache layout")
        _check_indices("qkv_prepare", None, None, page_size, k_cache.shape[0], slots)
    if rotary_dim and (cos is None or tuple(cos.shape) != (t, rotary_dim // 2) or tuple(sin.shape) != tuple(cos.shape)):
        raise KernelError("qkv_prepare: rotary tables missing or of the wrong shape")
    for name, w, width in (("q_weight", q_weight, heads * d), ("k_weight", k_weight, kv_heads * d)):
        if w is not None and w.numel() != (width if norm_whole else d):
            raise KernelError(f"qkv_prepare: {name} must have {width if norm_whole else d} values")
    _check(_fn("ts_qkv_prepare")(
        q_in.data_ptr(), q_in.stride(0), None if k_in is None else k_in.data_ptr(), 0 if k_in is None else k_in.stride(0),
        None if v_in is None else v_in.data_ptr(), 0 if v_in is None else v_in.stride(0),
        _bias(q_bias, heads * d, "q_bias", dt), _bias(k_bias if k_in is not None else None, kv_heads * d, "k_bias", dt),
        _bias(v_bias if v_in is not None else None, kv_heads * dv, "v_bias", dt),
        _opt(q_weight, "q_weight", dt), _opt(k_weight, "k_weight", dt), float(eps),
        _opt(cos, "cos", torch.float32), _opt(sin, "sin", torch.float32), int(rotary_dim),
        _opt(slots, "slots", torch.int32), _opt(k_cache, "k_cache", dt), _opt(v_cache, "v_cache", dt), page_size, t,
        heads, kv_heads, d, dv, _dev(q_out, "q_out"), int(bool(norm_whole)), _code(dt), _stream()), "qkv_prepare")


# ------------------------------------------------------------- latent attention
LATENT_MAX_RANK = 512
LATENT_TENSOR_CORES = True        # bf16 at sizes the mma.sync form takes; False: CUDA cores always
LATENT_MAX_SPLITS = 16
LATENT_MIN_KEYS_PER_SPLIT = 64


def latent_splits(num_seqs: int, heads: int, keys: int) -> int:
    """Key ranges per request for a step of single tokens: enough CTAs (one per request, 64 heads and
    range) to give every SM one, no range shorter than 64 keys. Depends only on the step's shape."""
    ctas = max(1, num_seqs * -(-heads // 64))
    return max(1, min(SM_COUNT // ctas, keys // LATENT_MIN_KEYS_PER_SPLIT, LATENT_MAX_SPLITS))


def latent_prepare(q_in: torch.Tensor, q_folded: torch.Tensor, ckr: torch.Tensor | None, norm_weight: torch.Tensor | None,
                   eps: float, cos: torch.Tensor | None, sin: torch.Tensor | None, rotary_dim: int, interleaved: bool,
                   slots: torch.Tensor | None, cache: torch.Tensor | None, heads: int, nope: int, rank: int, rot: int,
                   q_out: torch.Tensor) -> None:
    """Per token: the latent part ``ckr[:, :rank]`` is RMS-normed with a plain weight and the shared
    key part ``ckr[:, rank:]`` rotated (its first ``rotary_dim`` elements), both into the cache row
    of the token's slot (``cache [rows, rank + rot]``; nothing is written without ``slots``); the
    query rows ``q_out [T, heads, rank + rot]`` are the folded queries ``q_folded [heads, T, rank]``
    followed by the rotated last ``rot`` elements of each head of ``q_in [T, heads * (nope + rot)]``.
    ``q_in`` and ``ckr`` are 2-D dt with unit column stride (column slices of a merged product)."""
    t = q_out.shape[0]
    dt = q_out.dtype
    if tuple(q_out.shape) != (t, heads, rank + rot) or tuple(q_folded.shape) != (heads, t, rank) or q_folded.dtype != dt:
        raise KernelError("latent_prepare: query shapes")
    if q_in.dtype != dt or tuple(q_in.shape) != (t, heads * (nope + rot)) or q_in.stride(1) != 1 or not q_in.is_cuda:
        raise KernelError("latent_prepare: q_in must be [T, heads * (nope + rot)] dt with unit column stride on the device")
    if slots is not None:
        if ckr is None or ckr.dtype != dt or tuple(ckr.shape) != (t, rank + rot) or ckr.stride(1) != 1 or norm_weight is None:
            raise KernelError("latent_prepare: ckr must be [T, rank + rot] dt with unit column stride, with its norm weight")
        if cache is None or cache.dim() != 2 or cache.shape[1] != rank + rot or cache.dtype != dt:
            raise KernelError("latent_prepare: cache must be [rows, rank + rot] dt")
        _check_indices("latent_prepare", None, None, 1, cache.shape[0], slots)
    if rotary_dim and (cos is None or tuple(cos.shape) != (t, rotary_dim // 2) or tuple(sin.shape) != tuple(cos.shape)):
        raise KernelError("latent_prepare: rotary tables missing or of the wrong shape")
    _check(_fn("ts_latent_prepare")(
        q_in.data_ptr(), q_in.stride(0), _dev(q_folded, "q_folded"), None if ckr is None else ckr.data_ptr(),
        0 if ckr is None else ckr.stride(0), _opt(norm_weight, "norm_weight", dt), float(eps),
        _opt(cos, "cos", torch.float32), _opt(sin, "sin", torch.float32), int(rotary_dim), int(bool(interleaved)),
        _opt(slots, "slots", torch.int32), _opt(cache, "cache", dt), _dev(q_out, "q_out"), t, heads, nope, rank, rot,
        _code(dt), _stream()), "latent_prepare")


def latent_attention(q: torch.Tensor, cache: torch.Tensor, page_size: int, block_tables: torch.Tensor, ctx: Any,
                     rank: int, scale: float, window: int, out: torch.Tensor, sinks: torch.Tensor | None = None) -> None:
    """Causal attention of the query rows ``q [T, H, rank + rot]`` over each request's cached rows
    (``cache [pages * page_size, rank + rot]``: one row per position, shared by all heads); the
    values are the first ``rank`` elements of the keys. ``window`` 0 means all earlier positions.
    ``sinks`` (float32 ``[H]``, optional): a logit per head that joins the softmax's denominator, unscaled,
    without a value. ``out [T, H, rank]`` dt."""
    t, heads, d = q.shape
    dt = q.dtype
    if cache.dtype != dt or out.dtype != dt or cache.dim() != 2 or cache.shape[1] != d or tuple(out.shape) != (t, heads, rank):
        raise KernelError("latent_attention: shapes or dtypes")
    if not 0 < rank <= min(d, LATENT_MAX_RANK):
        raise KernelError(f"latent_attention: latent size {rank} must be at most {LATENT_MAX_RANK}")
    if block_tables.dim() != 2 or block_tables.shape[0] != ctx.num_seqs:
        raise KernelError("latent_attention: block_tables must be [requests, width]")
    if sinks is not None and (sinks.shape != (heads,) or sinks.dtype != torch.float32):
        raise KernelError("latent_attention: sinks must be float32, one per head")
    _check_indices("latent_attention", block_tables, ctx, page_size, cache.shape[0] // page_size)
    mma = bool(LATENT_TENSOR_CORES and dt == torch.bfloat16 and _fn("ts_latent_attention_mma_takes")(rank, d - rank))
    splits, part_acc, part_ml = 1, None, None
    if mma and ctx.max_query_len == 1:
        keys = min(ctx.max_context_len, window) if window else ctx.max_context_len
        splits = latent_splits(ctx.num_seqs, heads, keys)
        if splits > 1:
            part_acc = ctx.arena.take((t, heads, splits, rank), torch.float32)
            part_ml = ctx.arena.take((t, heads, splits, 2), torch.float32)
    _check(_fn("ts_latent_attention")(
        _dev(q, "q"), _dev(out, "out"), _dev(cache, "cache"), _dev(block_tables, "block_tables", torch.int32),
        block_tables.shape[1], _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32),
        _dev(ctx.context_lens_dev, "context_lens", torch.int32), ctx.num_seqs, ctx.max_query_len, heads, rank, d - rank,
        page_size, float(scale), int(window), _code(dt), int(mma), splits, _opt(part_acc, "part_acc"),
        _opt(part_ml, "part_ml"), t, _opt(sinks, "sinks", torch.float32), _stream()), "latent_attention",
        kernels=2 if splits > 1 else 1)


def bmm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out[b] = x[b] @ w[b]`` for ``x [B, M, K]`` (any strides), ``w [B, K, N]``, ``out [B, M, N]``
    contiguous: the per-head products of a latent attention layer, on the vendor library as the
    plain products of middle sizes are. float32 is true 32-bit: the reduced-precision matrix mode
    of the library is refused."""
    b, m, k = x.shape
    n = w.shape[2]
    if tuple(w.shape) != (b, k, n) or tuple(out.shape) != (b, m, n) or x.dtype != w.dtype or out.dtype != x.dtype:
        raise KernelError("bmm: shapes or dtypes")
    if m == 0:
        return
    _dev(out, "out")
    if x.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        raise KernelError("bmm: float32 products must not run in the library's TF32 mode")
    torch.bmm(x, w, out=out)


def transpose01(x: torch.Tensor, out: torch.Tensor) -> None:
    """``out[j, i, :] = x[i, j, :]`` (both contiguous, 3-D)."""
    a, b, c = x.shape
    if tuple(out.shape) != (b, a, c) or out.dtype != x.dtype:
        raise KernelError("transpose01: shapes or dtypes")
    _dev(x, "x"), _dev(out, "out")
    out.copy_(x.transpose(0, 1))


# ------------------------------------------------------------------------- experts
MOE_TILE_ROWS = 64
MOE_TENSOR_CORES = True          # bf16: False sends every product of the experts to the CUDA-core form
# From this many sorted rows a step (and at least an average tile's worth of rows per expert), bf16 products
# of experts whose matrices are wide enough run on the tcgen05 product over tiles of 128 rows; smaller steps
# run mma.sync tiles of 64 rows (a few rows per expert waste less of a tile, and no gather is needed).
MOE_TCGEN05 = True
MOE_TCGEN05_MIN_ROWS = 1024
MOE_TCGEN05_MIN_COLS = 256


def moe_max_tiles(num_tokens: int, top: int, experts: int, tile_rows: int = MOE_TILE_ROWS) -> int:
    """The most row tiles a step's sorted order can have: every tile holds a row, and an expert at
    most one ragged tile beyond its full ones."""
    picks = num_tokens * top
    return max(1, min(picks, picks // tile_rows + experts))


def moe_tile_rows(num_tokens: int, top: int, experts: int, dtype: torch.dtype, widths: Sequence[int]) -> int:
    """128 when the experts' products of this step go to the tcgen05 product (``widths``: the inner sizes
    K and output sizes N of the two products), else 64. Depends only on the step's shape."""
    picks = num_tokens * top
    big = (MOE_TCGEN05 and MOE_TENSOR_CORES and dtype == torch.bfloat16 and picks >= MOE_TCGEN05_MIN_ROWS
           and picks >= 64 * experts and all(w % 8 == 0 and w >= MOE_TCGEN05_MIN_COLS for w in widths))
    return 128 if big else MOE_TILE_ROWS


# Multiply-adds up to which the one routing CTA of a small step forms the router's logits itself instead of a
# product launched before it. Off (0): measured on B200 at 8 tokens, 16 experts, width 1,024 the recorded decode
# step of six layers went from 0.606 to 0.640 ms with it (84 to 79 kernels): one SM's 16 warps take about 8 us
# over the 128 dot products that the few-row product spreads over the machine in 3.
MOE_ROUTE_FUSED_MAX_WORK = 0


def _moe_plan(t: int, e: int, top: int, arena: Any, tile_rows: int) -> dict[str, Any]:
    picks, tiles = t * top, moe_max_tiles(t, top, e, tile_rows)
    ints = arena.take((4 * picks + e + 1 + 2 * tiles + 1,), torch.int32)
    plan = {"top": top, "experts": e, "max_tiles": tiles, "picks": picks, "tile_rows": tile_rows,
            "ids": ints[:picks], "place": ints[picks: 2 * picks], "row_of": ints[2 * picks: 3 * picks],
            "token_of": ints[3 * picks: 4 * picks], "offsets": ints[4 * picks: 4 * picks + e + 1]}
    at = 4 * picks + e + 1
    plan["tile_expert"], plan["tile_row0"], plan["num_tiles"] = ints[at: at + tiles], ints[at + tiles: at + 2 * tiles], ints[at + 2 * tiles:]
    plan["weights"] = arena.take((picks,), torch.float32)
    return plan


@dataclass(frozen=True)
class RouteRule:
    """How a token's experts and their weights follow from its router outputs. ``scored=False``: the ``top``
    largest logits, weighted by the softmax over the picked logits alone. ``scored=True``: scores are the
    softmax over ALL outputs; the choice looks at ``score + correction`` (``correction`` float32, one per output,
    or None) and only inside the ``keep`` best of ``groups`` equal groups of neighbouring outputs (a group's
    value is its largest choice score; the others' count as minus infinity); the weights are the picks' scores
    over their sum (+ 1e-20), times ``scale``. ``identity``: the last outputs are experts without matrices
    whose output is their input; their picks take no row of the sorted order."""

    scored: bool = False
    groups: int = 1
    keep: int = 1
    scale: float = 1.0
    identity: int = 0
    correction: torch.Tensor | None = None


PLAIN_ROUTE = RouteRule()


def moe_route_from(x: torch.Tensor, w_router: torch.Tensor, top: int, counts: torch.Tensor, arena: Any,
                   tile_rows: int = MOE_TILE_ROWS, rule: RouteRule = PLAIN_ROUTE, outputs: int | None = None) -> dict[str, Any]:
    """Router logits ``x W_router^T`` (32-bit sums and output) and :func:`moe_route` on them. ``outputs``: how
    many of the first rows of ``w_router`` are router outputs (all by default); rows beyond ride along in the
    same product (a gate of a shared expert) and are found in ``plan["logits"]``. A step of few
    tokens can do both in the one CTA that routes (no launch for the router's product); its sums run in
    another order than the product's, so a token's logits differ in the last bits between the two;
    switched by ``MOE_ROUTE_FUSED_MAX_WORK``, off by default, plain rule only)."""
    t, k = x.shape
    e = w_router.shape[0]
    if w_router.shape[1] != k or x.dtype != w_router.dtype:
        raise KernelError("moe_route_from: shapes or dtypes")
    logits = arena.take((t, e), torch.float32)
    if (rule is PLAIN_ROUTE and outputs in (None, e) and t <= 64 and e <= 1024 and t * e * k <= MOE_ROUTE_FUSED_MAX_WORK
            and 0 < top <= min(e, 32)):
        plan = _moe_plan(t, e, top, arena, tile_rows)
        _check(_fn("ts_moe_route_fused")(
            _dev(x, "x"), _dev(w_router, "w_router"), k, _code(x.dtype), _dev(logits, "logits", torch.float32), t, e, top,
            plan["ids"].data_ptr(), plan["weights"].data_ptr(), plan["place"].data_ptr(), plan["offsets"].data_ptr(),
            plan["tile_expert"].data_ptr(), plan["tile_row0"].data_ptr(), plan["num_tiles"].data_ptr(), plan["max_tiles"],
            plan["row_of"].data_ptr(), plan["token_of"].data_ptr(), tile_rows, _stream()), "moe_route_fused")
        plan["logits"] = logits
        return plan
    gemm(x, w_router, logits)
    return moe_route(logits, top, counts, arena, tile_rows, rule, outputs)


def moe_route(logits: torch.Tensor, top: int, counts: torch.Tensor, arena: Any, tile_rows: int = MOE_TILE_ROWS,
              rule: RouteRule = PLAIN_ROUTE, outputs: int | None = None) -> dict[str, Any]:
    """From router logits ``[T, >= outputs]`` float32 (the first ``outputs`` columns; all by default): every
    token's ``top`` experts and their weights by ``rule`` (ties to the lower index), and the sorted order in
    which the products run: rows grouped by expert, cut into tiles. ``counts`` is int32, one per expert with
    matrices (``outputs - rule.identity``), zero before the call and zero again after it. Returns the plan's
    device arrays; ``plan["experts"]`` counts the experts with matrices."""
    t, ld = logits.shape
    e = ld if outputs is None else int(outputs)
    real = e - rule.identity
    if not 0 < e <= ld or real <= 0 or logits.stride(1) != 1:
        raise KernelError("moe_route: outputs, identity experts or the logits' layout")
    if not 0 < top <= min(e, 32) or counts.shape != (real,):
        raise KernelError("moe_route: top must be between 1 and min(outputs, 32); counts one per expert with matrices")
    if not rule.scored and (rule.identity or rule.groups > 1 or rule.correction is not None):
        raise KernelError("moe_route: groups, a correction and identity experts come with the scored rule")
    if rule.groups < 1 or rule.groups > 32 or e % rule.groups or not 1 <= rule.keep <= rule.groups or e // rule.groups * rule.keep < top:
        raise KernelError("moe_route: up to 32 equal groups, of which the kept ones must hold at least `top` outputs")
    if rule.correction is not None and (rule.correction.shape != (e,) or rule.correction.dtype != torch.float32):
        raise KernelError("moe_route: the correction must be float32, one value per output")
    tiles = moe_max_tiles(t, top, real, tile_rows)
    plan = _moe_plan(t, real, top, arena, tile_rows)
    _check(_fn("ts_moe_route")(
        _dev(logits, "logits", torch.float32), logits.stride(0), t, e, real, top, int(rule.scored), rule.groups, rule.keep,
        float(rule.scale), _opt(rule.correction, "correction", torch.float32), plan["ids"].data_ptr(),
        plan["weights"].data_ptr(), plan["place"].data_ptr(), _dev(counts, "counts", torch.int32), plan["offsets"].data_ptr(),
        plan["tile_expert"].data_ptr(), plan["tile_row0"].data_ptr(), plan["num_tiles"].data_ptr(), tiles,
        plan["row_of"].data_ptr(), plan["token_of"].data_ptr(), tile_rows, _stream()), "moe_route",
        kernels=1 if t <= 64 else 3)
    plan["logits"] = logits
    plan["identity"] = rule.identity
    return plan


def moe_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, plan: dict[str, Any], gated: bool, gather: bool,
             arena: Any = None) -> None:
    """The experts' products over the sorted order of ``plan``: for every sorted row r of expert e,
    ``out[r] = x_r W_e^T`` (``gated``: ``silu(x_r Wgate_e^T) * (x_r Wup_e^T)`` with ``w [E, 2 N, K]``,
    gate rows first; else ``w [E, N, K]``). ``gather``: ``x`` is ``[T, K]`` and row r reads its
    token's row; else ``x`` is ``[picks, K]`` in the sorted order. ``out [picks, N]`` dt."""
    picks, n = out.shape
    e, rows, k = w.shape
    if picks != plan["picks"] or e != plan["experts"] or rows != (2 * n if gated else n) or x.shape[1] != k:
        raise KernelError("moe_gemm: shapes")
    if x.dtype != w.dtype or out.dtype != x.dtype or (not gather and x.shape[0] != picks):
        raise KernelError("moe_gemm: dtypes, or rows of x")
    if plan["tile_rows"] == 128:
        # tiles of 128 rows: the tcgen05 product over the sorted rows (gathered first where x is by token)
        if x.dtype != torch.bfloat16 or (gather and arena is None):
            raise KernelError("moe_gemm: tiles of 128 rows are for bfloat16, with scratch for the gathered rows")
        if gather:
            xs = arena.take((picks, k), x.dtype)
            total_rows = plan["offsets"][e:]          # the rows of the sorted order that exist: identity picks take none
            _check(_fn("ts_moe_gather")(_dev(x, "x"), plan["token_of"].data_ptr(), _dev(xs, "xs"), picks, k * x.element_size(),
                                        total_rows.data_ptr(), _stream()), "moe_gather")
            x = xs
        _check(_fn("ts_moe_gemm_tcgen05")(
            _dev(x, "x"), _dev(w, "w"), _dev(out, "out"), picks, n, k, e, int(bool(gated)), plan["offsets"].data_ptr(),
            plan["tile_expert"].data_ptr(), plan["tile_row0"].data_ptr(), plan["num_tiles"].data_ptr(), plan["max_tiles"],
            _error_word(x.device).data_ptr(), _stream()), "moe_gemm_tcgen05")
        return
    _check(_fn("ts_moe_gemm")(
        _dev(x, "x"), plan["token_of"].data_ptr() if gather else None, _dev(w, "w"), _dev(out, "out"),
        plan["offsets"].data_ptr(), plan["tile_expert"].data_ptr(), plan["tile_row0"].data_ptr(),
        plan["num_tiles"].data_ptr(), plan["max_tiles"], n, k, int(bool(gated)), _code(x.dtype), int(MOE_TENSOR_CORES),
        _stream()), "moe_gemm")


def moe_combine(y: torch.Tensor, plan: dict[str, Any], shared_out: torch.Tensor | None, out: torch.Tensor,
                x: torch.Tensor | None = None, shared_gate: torch.Tensor | None = None) -> None:
    """``out[t] = dt(sum_j weight[t, j] * y[row_of[t, j]] (+ g[t] * shared_out[t]))`` in 32-bit. A pick of an
    identity expert contributes ``weight * x[t]`` (``x [T, hidden]`` dt: the experts' input; needed when the plan
    has identity experts). ``shared_gate`` (float32 ``[T]``, possibly a column of a wider matrix): ``g =
    sigmoid(shared_gate)``; without it ``g = 1``."""
    t, h = out.shape
    if tuple(y.shape) != (plan["picks"], h) or t * plan["top"] != plan["picks"] or y.dtype != out.dtype:
        raise KernelError("moe_combine: shapes or dtypes")
    if shared_out is not None and (tuple(shared_out.shape) != (t, h) or shared_out.dtype != out.dtype):
        raise KernelError("moe_combine: the shared output must be [T, hidden] dt")
    if plan.get("identity", 0) and x is None:
        raise KernelError("moe_combine: identity experts need the experts' input")
    if x is not None and (tuple(x.shape) != (t, h) or x.dtype != out.dtype or not x.is_contiguous()):
        raise KernelError("moe_combine: x must be [T, hidden] dt")
    if shared_gate is not None and (shared_out is None or shared_gate.shape != (t,) or shared_gate.dtype != torch.float32):
        raise KernelError("moe_combine: the shared gate is one float32 logit per token and needs a shared output")
    _check(_fn("ts_moe_combine")(_dev(y, "y"), plan["row_of"].data_ptr(), plan["weights"].data_ptr(),
                                 _opt(shared_out, "shared_out"), _dev(out, "out"), t, plan["top"], h, _opt(x, "x"),
                                 None if shared_gate is None else shared_gate.data_ptr(),
                                 0 if shared_gate is None else shared_gate.stride(0), _code(out.dtype), _stream()),
           "moe_combine")


# --------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, out: torch.Tensor, temperature: torch.Tensor | None = None,
           top_p: torch.Tensor | None = None, seeds: torch.Tensor | None = None,
           draws: torch.Tensor | None = None, status_out: torch.Tensor | None = None) -> None:
    """One token per row of ``logits`` ``[R, V]`` float32 into ``out`` ``[R]`` int32. With no
    ``temperature`` every row is greedy; else rows with temperature 0 are greedy and the others
    are drawn (``seeds``/``draws`` int64 ``[R]``: the request's seed and how many tokens it
    has drawn so far; ``top_p`` float32 ``[R]`` optional). ``status_out`` (int32, one element):
    receives the device's error word, which kernels with bounded waits set when a wait ran out,
    so that it reaches the host in the same copy as the tokens."""
    r, v = logits.shape
    if out.shape != (r,):
        raise KernelError("sample: one output per row")
    _check(_fn("ts_sample")(_dev(logits, "logits", torch.float32), r, v, _opt(temperature, "temperature", torch.float32),
                            _opt(top_p, "top_p", torch.float32), _opt(seeds, "seeds", torch.int64),
                            _opt(draws, "draws", torch.int64), _dev(out, "out", torch.int32),
                            None if status_out is None else _error_word(logits.device).data_ptr(),
                            _opt(status_out, "status_out", torch.int32), _stream()), "sample")
