// Kernels around the 32-bit residual stream for layers that are not a plain pre-norm chain:
//
//  * embedding with a learned position row and a norm: x = table[token] * scale + pos[position],
//    optionally x / sqrt(mean(x^2) + eps) * weight, written to the 32-bit stream;
//  * the weighted sum of several sub-layer outputs into the stream,
//    x <- x + sum_i s_i y_i + s_b bias, with a copy of the new stream in the model dtype
//    (for a product that reads the stream itself rather than a norm of it).
//
// All arithmetic is 32-bit; the copy is rounded once.
#define TS_PDL_CLASS PDL_ELEMENTWISE
#include "common.cuh"

namespace ts {

// ---------------------------------------------------- embedding + position row + norm
// A CTA per token; the row waits in shared memory between the two passes.
template <typename T>
__global__ void embed_pos_norm_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
                                      const T* __restrict__ table, const T* __restrict__ pos_table,
                                      const T* __restrict__ norm_w, float* __restrict__ out, int hidden, int vocab,
                                      int max_pos, float scale, float eps) {
  extern __shared__ float xs[];
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = tokens[t];
  const int p = pos_table ? positions[t] : 0;
  float* o = out + (size_t)t * hidden;
  if (id < 0 || id >= vocab || p < 0 || (pos_table && p >= max_pos)) {
    // an id or a position outside its table: a row of NaN, never a read out of bounds
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = __int_as_float(0x7fc00000);
    return;
  }
  const T* row = table + (size_t)id * hidden;
  const T* prow = pos_table ? pos_table + (size_t)p * hidden : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = to_float(row[i]) * scale;
    if (prow) v += to_float(prow[i]);
    xs[i] = v;
    ss = fmaf(v, v, ss);
  }
  if (!norm_w) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = xs[i];
    return;
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = xs[i] * rstd * to_float(norm_w[i]);
}

// ------------------------------------------------- weighted sum of outputs into the stream
constexpr int SUM_MAX_TERMS = 4;
struct StreamSumArgs {
  float* resid;                 // [T, hidden]
  const void* term[SUM_MAX_TERMS];
  float scale[SUM_MAX_TERMS];
  int num_terms;
  const void* bias;             // [hidden] or null
  float bias_scale;
  void* copy;                   // [T, hidden] model dtype, or null
  int hidden;
  size_t total;
};

template <typename T, int VEC>
__global__ void stream_sum_kernel(StreamSumArgs a) {
  pdl_trigger();
  pdl_wait();
  const size_t n = a.total / VEC;
  for (size_t q = (size_t)blockIdx.x * blockDim.x + threadIdx.x; q < n; q += (size_t)gridDim.x * blockDim.x) {
    const size_t idx = q * VEC;
    const int c = (int)(idx % a.hidden);
    float x[VEC];
    if constexpr (VEC == 4) Quad<float>::load(a.resid + idx, x); else x[0] = a.resid[idx];
#pragma unroll
    for (int i = 0; i < SUM_MAX_TERMS; ++i) {
      if (i < a.num_terms) {
        float y[VEC];
        if constexpr (VEC == 4) Quad<T>::load((const T*)a.term[i] + idx, y); else y[0] = to_float(((const T*)a.term[i])[idx]);
#pragma unroll
        for (int e = 0; e < VEC; ++e) x[e] = fmaf(a.scale[i], y[e], x[e]);
      }
    }
    if (a.bias) {
      float b[VEC];
      if constexpr (VEC == 4) Quad<T>::load((const T*)a.bias + c, b); else b[0] = to_float(((const T*)a.bias)[c]);
#pragma unroll
      for (int e = 0; e < VEC; ++e) x[e] = fmaf(a.bias_scale, b[e], x[e]);
    }
    if constexpr (VEC == 4) Quad<float>::store(a.resid + idx, x); else a.resid[idx] = x[0];
    if (a.copy) {
      if constexpr (VEC == 4) Quad<T>::store((T*)a.copy + idx, x); else ((T*)a.copy)[idx] = from_float<T>(x[0]);
    }
  }
}

// ------------------------------------------------------------- a bias on every row
// y[t, j] <- y[t, j] + bias[j], in 32-bit, rounded once
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ y, const T* __restrict__ bias, int n, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
    y[idx] = from_float<T>(to_float(y[idx]) + to_float(bias[idx % n]));
}

// x <- tanh(x), in 32-bit, rounded once
template <typename T>
__global__ void tanh_kernel(T* __restrict__ x, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
    x[idx] = from_float<T>(tanhf(to_float(x[idx])));
}

}  // namespace ts

using namespace ts;

extern "C" int ts_tanh(void* x, size_t total, int dtype, cudaStream_t stream) {
  if (total == 0) return 0;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == TS_DTYPE_F32) return launch(tanh_kernel<float>, (int)blocks, 256, 0, stream, (float*)x, total);
  if (dtype == TS_DTYPE_BF16) return launch(tanh_kernel<bf16>, (int)blocks, 256, 0, stream, (bf16*)x, total);
  return TS_ERR_BAD_ARGUMENT;
}

extern "C" int ts_add_bias(void* y, const void* bias, int num_rows, int n, int dtype, cudaStream_t stream) {
  const size_t total = (size_t)num_rows * n;
  if (total == 0) return 0;
  if (!y || !bias) return TS_ERR_BAD_ARGUMENT;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == TS_DTYPE_F32) return launch(add_bias_kernel<float>, (int)blocks, 256, 0, stream, (float*)y, (const float*)bias, n, total);
  if (dtype == TS_DTYPE_BF16) return launch(add_bias_kernel<bf16>, (int)blocks, 256, 0, stream, (bf16*)y, (const bf16*)bias, n, total);
  return TS_ERR_BAD_ARGUMENT;
}

extern "C" int ts_embed_pos_norm(const int* tokens, const int* positions, const void* table, const void* pos_table,
                                 const void* norm_w, float* out, int num_tokens, int hidden, int vocab, int max_pos,
                                 float scale, float eps, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (hidden <= 0 || hidden > 12288 || (pos_table && !positions)) return TS_ERR_BAD_ARGUMENT;
  const int threads = hidden >= 1024 ? 256 : 128;
  const size_t smem = sizeof(float) * (size_t)hidden;
  if (dtype == TS_DTYPE_F32)
    return launch(embed_pos_norm_kernel<float>, num_tokens, threads, smem, stream, tokens, positions, (const float*)table,
                  (const float*)pos_table, (const float*)norm_w, out, hidden, vocab, max_pos, scale, eps);
  if (dtype == TS_DTYPE_BF16)
    return launch(embed_pos_norm_kernel<bf16>, num_tokens, threads, smem, stream, tokens, positions, (const bf16*)table,
                  (const bf16*)pos_table, (const bf16*)norm_w, out, hidden, vocab, max_pos, scale, eps);
  return TS_ERR_BAD_ARGUMENT;
}

extern "C" int ts_stream_sum(float* resid, const void* t0, const void* t1, const void* t2, const void* t3, float s0, float s1,
                             float s2, float s3, int num_terms, const void* bias, float bias_scale, void* copy,
                             int num_tokens, int hidden, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (hidden <= 0 || num_terms < 0 || num_terms > SUM_MAX_TERMS || !resid) return TS_ERR_BAD_ARGUMENT;
  if (dtype != TS_DTYPE_F32 && dtype != TS_DTYPE_BF16) return TS_ERR_BAD_ARGUMENT;
  StreamSumArgs a;
  a.resid = resid;
  a.term[0] = t0; a.term[1] = t1; a.term[2] = t2; a.term[3] = t3;
  a.scale[0] = s0; a.scale[1] = s1; a.scale[2] = s2; a.scale[3] = s3;
  a.num_terms = num_terms; a.bias = bias; a.bias_scale = bias_scale; a.copy = copy; a.hidden = hidden;
  a.total = (size_t)num_tokens * hidden;
  uintptr_t all = (uintptr_t)resid | (uintptr_t)bias | (uintptr_t)copy;
  for (int i = 0; i < num_terms; ++i) {
    if (!a.term[i]) return TS_ERR_BAD_ARGUMENT;
    all |= (uintptr_t)a.term[i];
  }
  const bool vec = hidden % 4 == 0 && (all & 15) == 0;
  const size_t work = vec ? a.total / 4 : a.total;
  size_t blocks = (work + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == TS_DTYPE_F32)
    return vec ? launch(stream_sum_kernel<float, 4>, (int)blocks, 256, 0, stream, a)
               : launch(stream_sum_kernel<float, 1>, (int)blocks, 256, 0, stream, a);
  return vec ? launch(stream_sum_kernel<bf16, 4>, (int)blocks, 256, 0, stream, a)
             : launch(stream_sum_kernel<bf16, 1>, (int)blocks, 256, 0, stream, a);
}
