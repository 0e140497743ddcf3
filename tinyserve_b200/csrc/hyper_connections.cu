// Hyper-connections: the residual stream as S parallel lanes, lanes [S, T, hidden] in 32-bit.
//
// A sub-layer q reads u = sum_s in_q[s] x_s, and when its output y is known every lane is
// rebuilt from the old ones: x_t <- sum_s mix_q[s][t] x_s + out_q[t] y. The rebuild of the
// sub-layer before (its y still pending, as the single-stream norm kernel keeps its delta
// pending) and the read of the next one are one pass here, fused with the RMSNorm that follows
// the read: one load and one store of the lanes per sub-layer. The very first sub-layer of a
// step finds no lanes yet and takes every lane from the embedding output.
// The collapse kernel applies a pending rebuild and sums the lanes for chosen rows.
// All arithmetic is 32-bit; the normalised output is rounded once to the model dtype.
#define TS_PDL_CLASS PDL_ELEMENTWISE
#include "common.cuh"

namespace ts {

constexpr int HC_MAX_LANES = 8;

struct HcWeights {
  float mix[HC_MAX_LANES * HC_MAX_LANES];   // [from][to] of the pending sub-layer
  float out[HC_MAX_LANES];
  float in[HC_MAX_LANES];                   // of the sub-layer about to run
};

__device__ __forceinline__ void hc_load(HcWeights& w, const float* mix, const float* out, const float* in, int S) {
  for (int s = 0; s < S; ++s) {
    if (mix)
      for (int t = 0; t < S; ++t) w.mix[s * HC_MAX_LANES + t] = mix[s * S + t];
    if (out) w.out[s] = out[s];
    if (in) w.in[s] = in[s];
  }
}

template <typename T>
__global__ void hc_mix_norm_kernel(float* __restrict__ lanes, const float* __restrict__ fresh,
                                   const T* __restrict__ delta, const float* __restrict__ mix_prev,
                                   const float* __restrict__ out_prev, const float* __restrict__ in_next,
                                   const T* __restrict__ norm_w, T* __restrict__ out, int S, int num_tokens,
                                   int hidden, float eps) {
  extern __shared__ float us[];             // the row of u
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  HcWeights w;
  hc_load(w, delta ? mix_prev : nullptr, delta ? out_prev : nullptr, in_next, S);
  const int row = blockIdx.x;
  const size_t lane_stride = (size_t)num_tokens * hidden;
  float* x = lanes + (size_t)row * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float nx[HC_MAX_LANES];
    if (fresh) {
      const float v = fresh[(size_t)row * hidden + i];
#pragma unroll
      for (int t = 0; t < HC_MAX_LANES; ++t) nx[t] = v;
    } else {
      float ox[HC_MAX_LANES];
#pragma unroll
      for (int s = 0; s < HC_MAX_LANES; ++s) ox[s] = s < S ? x[s * lane_stride + i] : 0.f;
      if (delta) {
        const float y = to_float(delta[(size_t)row * hidden + i]);
#pragma unroll
        for (int t = 0; t < HC_MAX_LANES; ++t) {
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < HC_MAX_LANES; ++s)
            if (s < S) acc = fmaf(w.mix[s * HC_MAX_LANES + t], ox[s], acc);
          nx[t] = t < S ? fmaf(w.out[t], y, acc) : 0.f;
        }
      } else {
#pragma unroll
        for (int t = 0; t < HC_MAX_LANES; ++t) nx[t] = ox[t];
      }
    }
    float u = 0.f;
#pragma unroll
    for (int t = 0; t < HC_MAX_LANES; ++t)
      if (t < S) {
        if (fresh || delta) x[t * lane_stride + i] = nx[t];
        u = fmaf(w.in[t], nx[t], u);
      }
    us[i] = u;
    ss = fmaf(u, u, ss);
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)row * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<T>(us[i] * rstd * to_float(norm_w[i]));
}

// The same for a lane count known at compile time and rows of a multiple of four 16-byte-aligned
// values: the connection weights sit in registers and every access is 16 bytes wide (8 for bf16).
// (Quad: four neighbouring elements in one access, common.cuh.)
template <typename T, int S>
__global__ void hc_mix_norm_vec_kernel(float* __restrict__ lanes, const float* __restrict__ fresh,
                                       const T* __restrict__ delta, const float* __restrict__ mix_prev,
                                       const float* __restrict__ out_prev, const float* __restrict__ in_next,
                                       const T* __restrict__ norm_w, T* __restrict__ out, int num_tokens, int hidden,
                                       float eps) {
  extern __shared__ __align__(16) float us[];
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  float mix[S][S], wo[S], wi[S];
#pragma unroll
  for (int a = 0; a < S; ++a) {
    wi[a] = in_next[a];
    wo[a] = delta ? out_prev[a] : 0.f;
#pragma unroll
    for (int b = 0; b < S; ++b) mix[a][b] = delta ? mix_prev[a * S + b] : (a == b ? 1.f : 0.f);
  }
  const int row = blockIdx.x;
  const size_t lane_stride = (size_t)num_tokens * hidden;
  float* x = lanes + (size_t)row * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
    float nx[S][4];
    if (fresh) {
      float v[4];
      Quad<float>::load(fresh + (size_t)row * hidden + i, v);
#pragma unroll
      for (int t = 0; t < S; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) nx[t][e] = v[e];
    } else {
      float ox[S][4];
#pragma unroll
      for (int a = 0; a < S; ++a) Quad<float>::load(x + a * lane_stride + i, ox[a]);
      if (delta) {
        float y[4];
        Quad<T>::load(delta + (size_t)row * hidden + i, y);
#pragma unroll
        for (int t = 0; t < S; ++t)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float acc = 0.f;
#pragma unroll
            for (int a = 0; a < S; ++a) acc = fmaf(mix[a][t], ox[a][e], acc);
            nx[t][e] = fmaf(wo[t], y[e], acc);
          }
      } else {
#pragma unroll
        for (int t = 0; t < S; ++t)
#pragma unroll
          for (int e = 0; e < 4; ++e) nx[t][e] = ox[t][e];
      }
    }
    float u[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int t = 0; t < S; ++t) {
      if (fresh || delta) Quad<float>::store(x + t * lane_stride + i, nx[t]);
#pragma unroll
      for (int e = 0; e < 4; ++e) u[e] = fmaf(wi[t], nx[t][e], u[e]);
    }
    Quad<float>::store(us + i, u);
#pragma unroll
    for (int e = 0; e < 4; ++e) ss = fmaf(u[e], u[e], ss);
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)row * hidden;
  for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
    float u[4], w[4];
    Quad<float>::load(us + i, u);
    Quad<T>::load(norm_w + i, w);
#pragma unroll
    for (int e = 0; e < 4; ++e) u[e] = u[e] * rstd * w[e];
    Quad<T>::store(o + i, u);
  }
}

// sum_out[r] = sum_t (sum_s mix[s][t] x_s + out[t] y) at row rows[r] (or r); lanes stay as they are.
template <typename T>
__global__ void hc_collapse_kernel(const float* __restrict__ lanes, const float* __restrict__ fresh,
                                   const T* __restrict__ delta, const float* __restrict__ mix_prev,
                                   const float* __restrict__ out_prev, const int* __restrict__ rows,
                                   float* __restrict__ sum_out, int S, int num_tokens, int hidden) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  const size_t lane_stride = (size_t)num_tokens * hidden;
  // the sum over the new lanes only needs, per old lane, the sum of its row of mix, and the sum of out
  float colsum[HC_MAX_LANES], outsum = 0.f;
  for (int s = 0; s < S; ++s) {
    float c = 0.f;
    if (delta)
      for (int t = 0; t < S; ++t) c += mix_prev[s * S + t];
    colsum[s] = delta ? c : 1.f;
    if (delta) outsum += out_prev[s];
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float acc;
    if (fresh) {
      acc = (float)S * fresh[(size_t)row * hidden + i];
    } else {
      acc = 0.f;
      for (int s = 0; s < S; ++s) acc = fmaf(colsum[s], lanes[s * lane_stride + (size_t)row * hidden + i], acc);
      if (delta) acc = fmaf(outsum, to_float(delta[(size_t)row * hidden + i]), acc);
    }
    sum_out[(size_t)r * hidden + i] = acc;
  }
}

}  // namespace ts

using namespace ts;

extern "C" int ts_hc_mix_norm(float* lanes, const float* fresh, const void* delta, const float* mix_prev,
                              const float* out_prev, const float* in_next, const void* norm_w, void* out,
                              int num_lanes, int num_tokens, int hidden, float eps, int dtype,
                              cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (num_lanes < 1 || num_lanes > HC_MAX_LANES) return TS_ERR_UNSUPPORTED;
  if (delta && (!mix_prev || !out_prev)) return TS_ERR_BAD_ARGUMENT;
  if (hidden > 48 * 1024 / 4) return TS_ERR_UNSUPPORTED;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  const size_t smem = sizeof(float) * hidden;
  const bool aligned = ((((uintptr_t)lanes) | ((uintptr_t)fresh) | ((uintptr_t)delta) | ((uintptr_t)norm_w) | ((uintptr_t)out)) & 15) == 0;
  if (aligned && hidden % 4 == 0 && num_lanes <= 4 && (dtype == TS_DTYPE_F32 || dtype == TS_DTYPE_BF16)) {
    const int vthreads = hidden >= 2048 ? 256 : 128;
#define TS_HC_CASE(T_, S_)                                                                                              \
  return launch(hc_mix_norm_vec_kernel<T_, S_>, num_tokens, vthreads, smem, stream, lanes, fresh, (const T_*)delta,      \
                mix_prev, out_prev, in_next, (const T_*)norm_w, (T_*)out, num_tokens, hidden, eps)
#define TS_HC_LANES(T_)                       \
  if (num_lanes == 1) { TS_HC_CASE(T_, 1); }  \
  if (num_lanes == 2) { TS_HC_CASE(T_, 2); }  \
  if (num_lanes == 3) { TS_HC_CASE(T_, 3); }  \
  TS_HC_CASE(T_, 4)
    if (dtype == TS_DTYPE_F32) { TS_HC_LANES(float); }
    TS_HC_LANES(bf16);
#undef TS_HC_LANES
#undef TS_HC_CASE
  }
  if (dtype == TS_DTYPE_F32)
    return launch(hc_mix_norm_kernel<float>, num_tokens, threads, smem, stream, lanes, fresh, (const float*)delta,
                  mix_prev, out_prev, in_next, (const float*)norm_w, (float*)out, num_lanes, num_tokens, hidden, eps);
  if (dtype == TS_DTYPE_BF16)
    return launch(hc_mix_norm_kernel<bf16>, num_tokens, threads, smem, stream, lanes, fresh, (const bf16*)delta,
                  mix_prev, out_prev, in_next, (const bf16*)norm_w, (bf16*)out, num_lanes, num_tokens, hidden, eps);
  return TS_ERR_BAD_ARGUMENT;
}

extern "C" int ts_hc_collapse(const float* lanes, const float* fresh, const void* delta, const float* mix_prev,
                              const float* out_prev, const int* rows, float* sum_out, int num_lanes,
                              int num_tokens, int num_rows, int hidden, int dtype, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (num_lanes < 1 || num_lanes > HC_MAX_LANES) return TS_ERR_UNSUPPORTED;
  if (delta && (!mix_prev || !out_prev)) return TS_ERR_BAD_ARGUMENT;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == TS_DTYPE_F32)
    return launch(hc_collapse_kernel<float>, num_rows, threads, 0, stream, lanes, fresh, (const float*)delta, mix_prev,
                  out_prev, rows, sum_out, num_lanes, num_tokens, hidden);
  if (dtype == TS_DTYPE_BF16)
    return launch(hc_collapse_kernel<bf16>, num_rows, threads, 0, stream, lanes, fresh, (const bf16*)delta, mix_prev,
                  out_prev, rows, sum_out, num_lanes, num_tokens, hidden);
  return TS_ERR_BAD_ARGUMENT;
}
