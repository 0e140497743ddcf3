// Residual sum with a norm on the sub-layer's output, fused with the norm in front of the next
// sub-layer. For a row x of the 32-bit stream and the pending sub-layer output d (model dtype):
//
//   y   = d / sqrt(mean(d^2) + eps_post) * gain(post_weight) * layer_scale * m  (when a post norm is pending;
//                                                                                  m a constant multiplier)
//   y   = (d + bias) * layer_scale                                               (a layer scale alone, with the
//                                                                                  sub-layer's output bias, if any)
//   x  <- x + y                                                                   (written back unless `rows`)
//   out = x / sqrt(mean(x^2) + eps) * gain(weight)
//
// gain(w) = 1 + w when the weight is stored around zero (`unit_offset`), else w. Everything is
// 32-bit; `out` is rounded once to the model dtype. Without a post norm y = d (the plain residual
// sum), so the kernel is also the norm with an offset weight alone. With `rows` only those rows
// are read, `out` has one row per entry and the stream is left as it is.
#define TS_PDL_CLASS PDL_ELEMENTWISE
#include "common.cuh"

namespace ts {

struct PostNormArgs {
  float* resid;
  const void* delta;        // may be null: nothing pending
  const void* post_weight;  // may be null: the pending output is added as it is
  const void* layer_scale;  // may be null
  const void* delta_bias;   // may be null: one value per column added to the pending output (only without a post norm)
  const void* weight;
  void* out;
  const int* rows;
  int num_rows, hidden;
  float post_eps, eps;
  float post_mult;          // a constant on the normed pending output
  int post_offset, offset;  // 1: the gain is 1 + weight
};

// A CTA per row; the row lives in shared memory (32-bit) between the passes. VEC: 4 elements per
// access (needs hidden % 4 == 0 and 16-byte aligned rows), else 1.
template <typename T, int VEC>
__global__ void post_norm_add_rms_norm_kernel(PostNormArgs a) {
  extern __shared__ float xs[];
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, hidden = a.hidden;
  const int row = a.rows ? a.rows[r] : r;
  float* x = a.resid + (size_t)row * hidden;
  const T* d = a.delta ? (const T*)a.delta + (size_t)row * hidden : nullptr;
  const T* pw = (const T*)a.post_weight;
  const T* ls = (const T*)a.layer_scale;
  const T* db = (const T*)a.delta_bias;
  const T* w = (const T*)a.weight;
  const bool write_back = (a.rows == nullptr) && (d != nullptr);
  float post_rstd = 1.f;
  if (d && pw) {
    float ss = 0.f;
    for (int i = threadIdx.x * VEC; i < hidden; i += blockDim.x * VEC) {
      float f[VEC];
      if constexpr (VEC == 4) Quad<T>::load(d + i, f); else f[0] = to_float(d[i]);
#pragma unroll
      for (int e = 0; e < VEC; ++e) { xs[i + e] = f[e]; ss = fmaf(f[e], f[e], ss); }
    }
    ss = block_sum(ss, scratch);
    post_rstd = rsqrtf(ss / (float)hidden + a.post_eps);
  }
  float ss = 0.f;
  for (int i = threadIdx.x * VEC; i < hidden; i += blockDim.x * VEC) {
    float v[VEC];
    if constexpr (VEC == 4) Quad<float>::load(x + i, v); else v[0] = x[i];
    if (d) {
      float y[VEC];
      if (pw) {
        float g[VEC];
        if constexpr (VEC == 4) Quad<T>::load(pw + i, g); else g[0] = to_float(pw[i]);
#pragma unroll
        for (int e = 0; e < VEC; ++e) y[e] = xs[i + e] * post_rstd * (a.post_offset ? 1.f + g[e] : g[e]) * a.post_mult;
      } else {
        if constexpr (VEC == 4) Quad<T>::load(d + i, y); else y[0] = to_float(d[i]);
        if (db) {
          float b[VEC];
          if constexpr (VEC == 4) Quad<T>::load(db + i, b); else b[0] = to_float(db[i]);
#pragma unroll
          for (int e = 0; e < VEC; ++e) y[e] += b[e];
        }
      }
      if (ls) {
        float s[VEC];
        if constexpr (VEC == 4) Quad<T>::load(ls + i, s); else s[0] = to_float(ls[i]);
#pragma unroll
        for (int e = 0; e < VEC; ++e) y[e] *= s[e];
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) v[e] += y[e];
      if (write_back) {
        if constexpr (VEC == 4) Quad<float>::store(x + i, v); else x[i] = v[0];
      }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) { xs[i + e] = v[e]; ss = fmaf(v[e], v[e], ss); }
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)hidden + a.eps);
  T* o = (T*)a.out + (size_t)r * hidden;
  for (int i = threadIdx.x * VEC; i < hidden; i += blockDim.x * VEC) {
    float g[VEC], res[VEC];
    if constexpr (VEC == 4) Quad<T>::load(w + i, g); else g[0] = to_float(w[i]);
#pragma unroll
    for (int e = 0; e < VEC; ++e) res[e] = xs[i + e] * rstd * (a.offset ? 1.f + g[e] : g[e]);
    if constexpr (VEC == 4) Quad<T>::store(o + i, res); else o[i] = from_float<T>(res[0]);
  }
}

}  // namespace ts

using namespace ts;

extern "C" int ts_post_norm_add_rms_norm(float* resid, const void* delta, const void* post_weight, const void* layer_scale,
                                         float post_eps, int post_offset, float post_mult, const void* weight, int offset,
                                         float eps, void* out, const int* rows, int num_rows, int hidden, const void* delta_bias,
                                         int dtype, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (hidden <= 0 || hidden > 12288 || !weight || !out || !resid) return TS_ERR_BAD_ARGUMENT;
  if (dtype != TS_DTYPE_F32 && dtype != TS_DTYPE_BF16) return TS_ERR_BAD_ARGUMENT;
  if ((post_weight || layer_scale || delta_bias) && !delta) return TS_ERR_BAD_ARGUMENT;
  if (delta_bias && post_weight) return TS_ERR_UNSUPPORTED;
  PostNormArgs a;
  a.resid = resid; a.delta = delta; a.post_weight = post_weight; a.layer_scale = layer_scale; a.delta_bias = delta_bias; a.weight = weight;
  a.out = out; a.rows = rows; a.num_rows = num_rows; a.hidden = hidden; a.post_eps = post_eps; a.eps = eps;
  a.post_offset = post_offset; a.offset = offset; a.post_mult = post_mult;
  const size_t smem = sizeof(float) * (size_t)hidden;
  const bool aligned = hidden % 4 == 0 &&
      (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)post_weight | (uintptr_t)layer_scale | (uintptr_t)delta_bias | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
  const int per = aligned ? 4 : 1;
  int threads = 64;
  while (threads < 512 && threads * per * 2 <= hidden) threads <<= 1;
#define TS_PN_CASE(T_, V_)                                                                          \
  do {                                                                                              \
    auto kern = post_norm_add_rms_norm_kernel<T_, V_>;                                              \
    if (smem > 48 * 1024) {                                                                         \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return (int)e;                                                          \
    }                                                                                               \
    return launch(kern, num_rows, threads, smem, stream, a);                                        \
  } while (0)
  if (dtype == TS_DTYPE_F32) { if (aligned) TS_PN_CASE(float, 4); TS_PN_CASE(float, 1); }
  if (aligned) TS_PN_CASE(bf16, 4);
  TS_PN_CASE(bf16, 1);
#undef TS_PN_CASE
}
