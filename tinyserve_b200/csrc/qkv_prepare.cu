// Queries, keys and values on their way to attention when keys and values may have different
// head sizes: per (token, head) an optional RMSNorm over the head (plain weight), an optional
// rotation of the first `rotary_dim` elements (element i pairs with i + rotary_dim / 2), then
// queries go to q_out [T, heads, d], keys to k_cache [pages, kv_heads, page_size, d] and values,
// unchanged, to v_cache [pages, kv_heads, page_size, dv] at the token's slot. q, k and v are read
// from rows with strides of their own, so they may be parts of one merged projection. Optional
// biases (one value per projection row) are added first. With `norm_whole` the RMSNorm runs over the
// whole projection row (all heads of q, or of k, together; the weight then has one value per row
// element) instead of head by head. All arithmetic is 32-bit and the result is rounded once.
#define TS_PDL_CLASS PDL_ELEMENTWISE
#include "common.cuh"

namespace ts {

constexpr int QP_WARPS = 4;          // warps (heads in flight) per CTA
constexpr int QP_MAX_DIM = 256;      // largest head the staging rows hold

// Two neighbouring elements in one access.
template <typename T> struct Pair;
template <> struct Pair<float> {
  static __device__ __forceinline__ void load(const float* p, float& a, float& b) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x; b = v.y;
  }
  static __device__ __forceinline__ void store(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
  static constexpr uintptr_t MASK = 7;
};
template <> struct Pair<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float& a, float& b) {
    const uint32_t v = *reinterpret_cast<const uint32_t*>(p);
    a = __uint_as_float(v << 16); b = __uint_as_float(v & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(bf16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
  }
  static constexpr uintptr_t MASK = 3;
};

// The sum of squares of a whole projection row of n elements (bias added first), by all threads of the CTA.
template <typename T>
__device__ __forceinline__ float row_sumsq(const T* __restrict__ x, const T* __restrict__ bias, int n, float* scratch) {
  float ss = 0.f;
  if ((n & 1) == 0 && ((((uintptr_t)x) | ((uintptr_t)bias)) & Pair<T>::MASK) == 0) {
    for (int i = 2 * threadIdx.x; i < n; i += 2 * blockDim.x) {
      float a, b;
      Pair<T>::load(x + i, a, b);
      if (bias) {
        float ba, bb;
        Pair<T>::load(bias + i, ba, bb);
        a += ba;
        b += bb;
      }
      ss = fmaf(a, a, fmaf(b, b, ss));
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float v = to_float(x[i]) + (bias ? to_float(bias[i]) : 0.f);
      ss = fmaf(v, v, ss);
    }
  }
  return block_sum(ss, scratch);
}

// One head by one warp: the head is read once from global memory into the warp's row of shared
// memory (as 32-bit values), the sum of squares is formed on the way, and every element is then
// written with its rotation partner taken from that row. Heads of an even size at an aligned
// address move two elements per access.
template <typename T>
__device__ __forceinline__ void norm_rotate_head(const T* __restrict__ x, const T* __restrict__ bias,
                                                 const T* __restrict__ w, float eps,
                                                 const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                 int rotary_dim, int d, T* __restrict__ dst, int lane,
                                                 float* __restrict__ row, float given_rstd = -1.f) {
  const bool pairs = (d & 1) == 0 &&
      ((((uintptr_t)x) | ((uintptr_t)dst) | ((uintptr_t)w) | ((uintptr_t)bias)) & Pair<T>::MASK) == 0;
  const int half = rotary_dim >> 1;
  float ss = 0.f;
  if (pairs) {
    // everything this lane needs from global memory is asked for before anything is used: its pairs of
    // the head, of the weight, and the angles of its elements (QP_MAX_DIM / 64 pairs at most)
    constexpr int J = QP_MAX_DIM / 64;
    float a[J], b[J], wa[J], wb[J], c0[J], s0[J], c1[J], s1[J];
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int i = 2 * lane + 64 * j;
      a[j] = b[j] = 0.f;
      wa[j] = wb[j] = c0[j] = c1[j] = 1.f;
      s0[j] = s1[j] = 0.f;
      if (i < d) {
        Pair<T>::load(x + i, a[j], b[j]);
        if (bias) {
          float ba, bb;
          Pair<T>::load(bias + i, ba, bb);
          a[j] += ba;
          b[j] += bb;
        }
        if (w) Pair<T>::load(w + i, wa[j], wb[j]);
        if (i < rotary_dim) {
          const int f = i < half ? i : i - half;
          c0[j] = cos_t[f];
          s0[j] = sin_t[f];
        }
        if (i + 1 < rotary_dim) {
          const int f = i + 1 < half ? i + 1 : i + 1 - half;
          c1[j] = cos_t[f];
          s1[j] = sin_t[f];
        }
      }
    }
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int i = 2 * lane + 64 * j;
      if (i < d) {
        row[i] = a[j] * wa[j];
        row[i + 1] = b[j] * wb[j];
        ss = fmaf(a[j], a[j], fmaf(b[j], b[j], ss));
      }
    }
    const float rstd = !w ? 1.f : given_rstd >= 0.f ? given_rstd : rsqrtf(warp_sum(ss) / (float)d + eps);
    __syncwarp();
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int i = 2 * lane + 64 * j;
      if (i < d) {
        float y0 = row[i] * rstd, y1 = row[i + 1] * rstd;
        if (i < rotary_dim) {
          const float p = row[i < half ? i + half : i - half] * rstd;
          y0 = i < half ? y0 * c0[j] - p * s0[j] : y0 * c0[j] + p * s0[j];
        }
        if (i + 1 < rotary_dim) {
          const float p = row[i + 1 < half ? i + 1 + half : i + 1 - half] * rstd;
          y1 = i + 1 < half ? y1 * c1[j] - p * s1[j] : y1 * c1[j] + p * s1[j];
        }
        Pair<T>::store(dst + i, y0, y1);
      }
    }
    return;
  }
  for (int i = lane; i < d; i += 32) {
    const float v = to_float(x[i]) + (bias ? to_float(bias[i]) : 0.f);
    row[i] = w ? v * to_float(w[i]) : v;
    ss = fmaf(v, v, ss);
  }
  const float rstd = !w ? 1.f : given_rstd >= 0.f ? given_rstd : rsqrtf(warp_sum(ss) / (float)d + eps);
  __syncwarp();
  for (int i = lane; i < d; i += 32) {
    float y = row[i] * rstd;
    if (i < rotary_dim) {
      const float yp = row[i < half ? i + half : i - half] * rstd;
      const int f = i < half ? i : i - half;
      const float c = cos_t[f], s = sin_t[f];
      y = i < half ? y * c - yp * s : y * c + yp * s;
    }
    dst[i] = from_float<T>(y);
  }
}

template <typename T>
__global__ void qkv_prepare_kernel(const T* __restrict__ q_in, int q_stride, const T* __restrict__ k_in, int k_stride,
                                   const T* __restrict__ v_in, int v_stride, const T* __restrict__ q_b,
                                   const T* __restrict__ k_b, const T* __restrict__ v_b, const T* __restrict__ q_w,
                                   const T* __restrict__ k_w, float eps, const float* __restrict__ cos_tab,
                                   const float* __restrict__ sin_tab, int rotary_dim, const int* __restrict__ slots,
                                   T* __restrict__ k_cache, T* __restrict__ v_cache, int page_size, int num_tokens,
                                   int heads, int kv_heads, int d, int dv, T* __restrict__ q_out) {
  __shared__ float rows[QP_WARPS][QP_MAX_DIM];
  float* row = rows[threadIdx.x >> 5];
  pdl_trigger();
  pdl_wait();
  const int jobs = heads + (k_in ? 2 * kv_heads : 0);
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)num_tokens * jobs) return;
  const int t = (int)(warp / jobs), job = (int)(warp - (long long)t * jobs);
  const float* cos_t = rotary_dim ? cos_tab + (size_t)t * (rotary_dim >> 1) : nullptr;
  const float* sin_t = rotary_dim ? sin_tab + (size_t)t * (rotary_dim >> 1) : nullptr;
  if (job < heads) {
    norm_rotate_head(q_in + (size_t)t * q_stride + job * d, q_b ? q_b + job * d : nullptr, q_w, eps, cos_t, sin_t, rotary_dim, d,
                     q_out + ((size_t)t * heads + job) * d, lane, row);
    return;
  }
  const int slot = slots[t];
  const int page = slot / page_size, off = slot - page * page_size;
  if (job < heads + kv_heads) {
    const int g = job - heads;
    norm_rotate_head(k_in + (size_t)t * k_stride + g * d, k_b ? k_b + g * d : nullptr, k_w, eps, cos_t, sin_t, rotary_dim, d,
                     k_cache + (((size_t)page * kv_heads + g) * page_size + off) * d, lane, row);
    return;
  }
  const int g = job - heads - kv_heads;
  const T* src = v_in + (size_t)t * v_stride + g * dv;
  T* dst = v_cache + (((size_t)page * kv_heads + g) * page_size + off) * dv;
  const T* vb = v_b ? v_b + g * dv : nullptr;
  if ((dv & 1) == 0 && ((((uintptr_t)src) | ((uintptr_t)dst) | ((uintptr_t)vb)) & Pair<T>::MASK) == 0) {
    for (int i = 2 * lane; i < dv; i += 64) {
      float a, b;
      Pair<T>::load(src + i, a, b);
      if (vb) {
        float ba, bb;
        Pair<T>::load(vb + i, ba, bb);
        a += ba;
        b += bb;
      }
      Pair<T>::store(dst + i, a, b);
    }
  } else if (vb) {
    for (int i = lane; i < dv; i += 32) dst[i] = from_float<T>(to_float(src[i]) + to_float(vb[i]));
  } else {
    for (int i = lane; i < dv; i += 32) dst[i] = src[i];
  }
}

// The norm over the whole projection: a CTA per token. All its threads form the sums of squares of the token's q row
// and k row once; then its warps take the heads in turn, each with the row's 1 / rms and its own stretch of the weight.
constexpr int QW_WARPS = 8;
template <typename T>
__global__ void __launch_bounds__(QW_WARPS * 32) qkv_prepare_whole_kernel(
    const T* __restrict__ q_in, int q_stride, const T* __restrict__ k_in, int k_stride, const T* __restrict__ v_in, int v_stride,
    const T* __restrict__ q_b, const T* __restrict__ k_b, const T* __restrict__ v_b, const T* __restrict__ q_w,
    const T* __restrict__ k_w, float eps, const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int rotary_dim,
    const int* __restrict__ slots, T* __restrict__ k_cache, T* __restrict__ v_cache, int page_size, int heads, int kv_heads,
    int d, int dv, T* __restrict__ q_out) {
  __shared__ float rows[QW_WARPS][QP_MAX_DIM];
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* row = rows[warp];
  float rstd_q = 1.f, rstd_k = 1.f;
  if (q_w) rstd_q = rsqrtf(row_sumsq(q_in + (size_t)t * q_stride, q_b, heads * d, scratch) / (float)(heads * d) + eps);
  if (k_in && k_w) rstd_k = rsqrtf(row_sumsq(k_in + (size_t)t * k_stride, k_b, kv_heads * d, scratch) / (float)(kv_heads * d) + eps);
  const float* cos_t = rotary_dim ? cos_tab + (size_t)t * (rotary_dim >> 1) : nullptr;
  const float* sin_t = rotary_dim ? sin_tab + (size_t)t * (rotary_dim >> 1) : nullptr;
  const int jobs = heads + (k_in ? 2 * kv_heads : 0);
  int page = 0, off = 0;
  if (k_in) {
    const int slot = slots[t];
    page = slot / page_size;
    off = slot - page * page_size;
  }
  for (int job = warp; job < jobs; job += QW_WARPS) {
    if (job < heads) {
      norm_rotate_head(q_in + (size_t)t * q_stride + job * d, q_b ? q_b + job * d : nullptr, q_w ? q_w + job * d : nullptr, eps,
                       cos_t, sin_t, rotary_dim, d, q_out + ((size_t)t * heads + job) * d, lane, row, rstd_q);
    } else if (job < heads + kv_heads) {
      const int g = job - heads;
      norm_rotate_head(k_in + (size_t)t * k_stride + g * d, k_b ? k_b + g * d : nullptr, k_w ? k_w + g * d : nullptr, eps, cos_t,
                       sin_t, rotary_dim, d, k_cache + (((size_t)page * kv_heads + g) * page_size + off) * d, lane, row, rstd_k);
    } else {
      const int g = job - heads - kv_heads;
      const T* src = v_in + (size_t)t * v_stride + g * dv;
      T* dst = v_cache + (((size_t)page * kv_heads + g) * page_size + off) * dv;
      const T* vb = v_b ? v_b + g * dv : nullptr;
      if ((dv & 1) == 0 && ((((uintptr_t)src) | ((uintptr_t)dst) | ((uintptr_t)vb)) & Pair<T>::MASK) == 0) {
        for (int i = 2 * lane; i < dv; i += 64) {
          float a, b;
          Pair<T>::load(src + i, a, b);
          if (vb) {
            float ba, bb;
            Pair<T>::load(vb + i, ba, bb);
            a += ba;
            b += bb;
          }
          Pair<T>::store(dst + i, a, b);
        }
      } else {
        for (int i = lane; i < dv; i += 32) dst[i] = vb ? from_float<T>(to_float(src[i]) + to_float(vb[i])) : src[i];
      }
    }
    __syncwarp();          // the warp's staging row is free for its next head
  }
}

}  // namespace ts

using namespace ts;

extern "C" int ts_qkv_prepare(const void* q_in, int q_stride, const void* k_in, int k_stride, const void* v_in,
                              int v_stride, const void* q_b, const void* k_b, const void* v_b, const void* q_w, const void* k_w, float eps, const float* cos_tab,
                              const float* sin_tab, int rotary_dim, const int* slots, void* k_cache, void* v_cache,
                              int page_size, int num_tokens, int heads, int kv_heads, int d, int dv, void* q_out,
                              int norm_whole, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (d > QP_MAX_DIM) return TS_ERR_UNSUPPORTED;
  if (rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1) || (rotary_dim && (!cos_tab || !sin_tab))) return TS_ERR_BAD_ARGUMENT;
  if (k_in && (!v_in || !slots || !k_cache || !v_cache || page_size <= 0)) return TS_ERR_BAD_ARGUMENT;
  if (norm_whole) {
    if (dtype == TS_DTYPE_F32)
      return launch(qkv_prepare_whole_kernel<float>, num_tokens, QW_WARPS * 32, 0, stream, (const float*)q_in, q_stride,
                    (const float*)k_in, k_stride, (const float*)v_in, v_stride, (const float*)q_b, (const float*)k_b, (const float*)v_b,
                    (const float*)q_w, (const float*)k_w, eps, cos_tab, sin_tab, rotary_dim, slots, (float*)k_cache, (float*)v_cache,
                    page_size, heads, kv_heads, d, dv, (float*)q_out);
    if (dtype == TS_DTYPE_BF16)
      return launch(qkv_prepare_whole_kernel<bf16>, num_tokens, QW_WARPS * 32, 0, stream, (const bf16*)q_in, q_stride,
                    (const bf16*)k_in, k_stride, (const bf16*)v_in, v_stride, (const bf16*)q_b, (const bf16*)k_b, (const bf16*)v_b,
                    (const bf16*)q_w, (const bf16*)k_w, eps, cos_tab, sin_tab, rotary_dim, slots, (bf16*)k_cache, (bf16*)v_cache,
                    page_size, heads, kv_heads, d, dv, (bf16*)q_out);
    return TS_ERR_BAD_ARGUMENT;
  }
  const long long warps = (long long)num_tokens * (heads + (k_in ? 2 * kv_heads : 0));
  const int threads = QP_WARPS * 32;
  const int blocks = (int)((warps * 32 + threads - 1) / threads);
  if (dtype == TS_DTYPE_F32)
    return launch(qkv_prepare_kernel<float>, blocks, threads, 0, stream, (const float*)q_in, q_stride, (const float*)k_in,
                  k_stride, (const float*)v_in, v_stride, (const float*)q_b, (const float*)k_b, (const float*)v_b, (const float*)q_w, (const float*)k_w, eps, cos_tab, sin_tab,
                  rotary_dim, slots, (float*)k_cache, (float*)v_cache, page_size, num_tokens, heads, kv_heads, d, dv,
                  (float*)q_out);
  if (dtype == TS_DTYPE_BF16)
    return launch(qkv_prepare_kernel<bf16>, blocks, threads, 0, stream, (const bf16*)q_in, q_stride, (const bf16*)k_in,
                  k_stride, (const bf16*)v_in, v_stride, (const bf16*)q_b, (const bf16*)k_b, (const bf16*)v_b, (const bf16*)q_w, (const bf16*)k_w, eps, cos_tab, sin_tab,
                  rotary_dim, slots, (bf16*)k_cache, (bf16*)v_cache, page_size, num_tokens, heads, kv_heads, d, dv,
                  (bf16*)q_out);
  return TS_ERR_BAD_ARGUMENT;
}
