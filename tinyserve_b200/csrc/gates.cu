// Gating and squashing kernels: a gated feed-forward's activation with a choice of activation,
// the per-head RMSNorm and sigmoid output gate that follows a mixer's read-out, and the tanh
// soft cap of the logits. All arithmetic is 32-bit with one rounding to the output type.
#define TS_PDL_CLASS PDL_ELEMENTWISE
#include "common.cuh"

namespace ts {

constexpr int ACT_SILU = 0, ACT_GELU_TANH = 1, ACT_CLAMPED_SWISH = 2;

__device__ __forceinline__ float sigmoidf(float z) { return 1.f / (1.f + expf(-z)); }

template <int ACT>
__device__ __forceinline__ float activate(float z) {
  if (ACT == ACT_SILU || ACT == ACT_CLAMPED_SWISH) return z / (1.f + expf(-z));
  // 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
  const float inner = 0.7978845608028654f * fmaf(0.044715f * z * z, z, z);
  return 0.5f * z * (1.f + tanhf(inner));
}

// out[t, j] = act(gate_up[t, j] + bias[j]) * (gate_up[t, I + j] + bias[I + j])   (bias optional)
// ACT_CLAMPED_SWISH: g = min(gate, limit), u = clamp(up, -limit, limit), out = g sigmoid(1.702 g) (u + 1)
template <typename T, int ACT>
__global__ void act_mul_kernel(const T* __restrict__ gate_up, const T* __restrict__ bias, T* __restrict__ out, int inter,
                               size_t total, float limit) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter;
    const int j = (int)(idx - t * inter);
    const T* row = gate_up + t * 2 * (size_t)inter;
    float gate = to_float(row[j]), up = to_float(row[inter + j]);
    if (bias) {
      gate += to_float(bias[j]);
      up += to_float(bias[inter + j]);
    }
    if (ACT == ACT_CLAMPED_SWISH) {
      const float g = fminf(gate, limit);
      const float u = fminf(fmaxf(up, -limit), limit);
      out[idx] = from_float<T>(g * sigmoidf(1.702f * g) * (u + 1.f));
    } else {
      out[idx] = from_float<T>(activate<ACT>(gate) * up);
    }
  }
}

// out[t, j] = act(x[t, j]) * table[rows[t], col0 + j]: a gate on a row that is looked up per token
// (x rows are `x_stride` apart, table rows `table_width`); a row index outside the table gives NaN.
template <typename T, int ACT>
__global__ void act_mul_gather_kernel(const T* __restrict__ x, int x_stride, const int* __restrict__ rows,
                                      const T* __restrict__ table, int table_rows, int table_width, int col0,
                                      T* __restrict__ out, int n, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / n;
    const int j = (int)(idx - t * n);
    const int r = rows[t];
    const float e = (r >= 0 && r < table_rows) ? to_float(table[(size_t)r * table_width + col0 + j]) : __int_as_float(0x7fc00000);
    out[idx] = from_float<T>(activate<ACT>(to_float(x[t * x_stride + j])) * e);
  }
}

// logits <- cap * tanh(logits / cap), in place
__global__ void softcap_kernel(float* __restrict__ x, float cap, float inv_cap, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
    x[idx] = cap * tanhf(x[idx] * inv_cap);
}

// One warp per (token, head): y = x / sqrt(mean(x^2) + eps) when `normalise`, times
// weight[head * weight_head_stride + c] when a weight is given, times sigmoid(gate[t, head, c])
// when a gate is given (`gate_per_head`: sigmoid(gate[t, head]), one value for the whole head;
// `gate_silu`: the gate's value is z sigmoid(z) instead of sigmoid(z)).
// x is [T, heads, width] of type IN; gate rows are `gate_stride` apart.
template <typename IN, typename T>
__global__ void head_norm_gate_kernel(const IN* __restrict__ x, const T* __restrict__ weight, int weight_head_stride,
                                      const T* __restrict__ gate, int gate_stride, T* __restrict__ out,
                                      int num_tokens, int heads, int width, int normalise, float eps,
                                      int gate_per_head, int gate_silu) {
  pdl_trigger();
  pdl_wait();
  const int warp = (int)(((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (warp >= num_tokens * heads) return;
  const int t = warp / heads, h = warp - t * heads;
  const IN* xr = x + (size_t)warp * width;
  float rstd = 1.f;
  if (normalise) {
    float ss = 0.f;
    for (int c = lane; c < width; c += 32) {
      const float v = to_float(xr[c]);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / (float)width + eps);
  }
  float head_gate = 1.f;
  if (gate && gate_per_head) {
    const float z = to_float(gate[(size_t)t * gate_stride + h]);
    head_gate = gate_silu ? z * sigmoidf(z) : sigmoidf(z);
  }
  for (int c = lane; c < width; c += 32) {
    float v = to_float(xr[c]) * rstd * head_gate;
    if (weight) v *= to_float(weight[h * weight_head_stride + c]);
    if (gate && !gate_per_head) {
      const float z = to_float(gate[(size_t)t * gate_stride + h * width + c]);
      v *= gate_silu ? z * sigmoidf(z) : sigmoidf(z);
    }
    out[(size_t)warp * width + c] = from_float<T>(v);
  }
}

// The same for wide rows (all heads normed together, say): a CTA per (token, head), the row's sum of squares
// through shared memory.
template <typename IN, typename T>
__global__ void __launch_bounds__(256) head_norm_gate_wide_kernel(const IN* __restrict__ x, const T* __restrict__ weight,
                                                                  int weight_head_stride, const T* __restrict__ gate,
                                                                  int gate_stride, T* __restrict__ out, int heads, int width,
                                                                  int normalise, float eps, int gate_per_head, int gate_silu) {
  __shared__ float parts[8];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x, t = row / heads, h = row - t * heads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const IN* xr = x + (size_t)row * width;
  float rstd = 1.f;
  if (normalise) {
    float ss = 0.f;
    for (int c = tid; c < width; c += 256) {
      const float v = to_float(xr[c]);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) parts[warp] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) ss += parts[w];
    rstd = rsqrtf(ss / (float)width + eps);
  }
  float head_gate = 1.f;
  if (gate && gate_per_head) {
    const float z = to_float(gate[(size_t)t * gate_stride + h]);
    head_gate = gate_silu ? z * sigmoidf(z) : sigmoidf(z);
  }
  for (int c = tid; c < width; c += 256) {
    float v = to_float(xr[c]) * rstd * head_gate;
    if (weight) v *= to_float(weight[h * weight_head_stride + c]);
    if (gate && !gate_per_head) {
      const float z = to_float(gate[(size_t)t * gate_stride + h * width + c]);
      v *= gate_silu ? z * sigmoidf(z) : sigmoidf(z);
    }
    out[(size_t)row * width + c] = from_float<T>(v);
  }
}

// RMSNorm of rows that lie `x_stride` elements apart (a column slice of a wider product): out[r] =
// dt(x[r] / sqrt(mean(x[r]^2) + eps) * weight), 32-bit and rounded once. A CTA per row.
template <typename T>
__global__ void rms_norm_rows_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ weight, float eps,
                                     T* __restrict__ out, int width) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const T* xr = x + (size_t)blockIdx.x * x_stride;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = to_float(xr[c]);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[(size_t)blockIdx.x * width + c] = from_float<T>(to_float(xr[c]) * rstd * to_float(weight[c]));
}

}  // namespace ts

using namespace ts;

static int blocks_for(size_t total, int threads) {
  size_t b = (total + threads - 1) / threads;
  if (b > 148 * 16) b = 148 * 16;
  return (int)b;
}

extern "C" int ts_act_mul(const void* gate_up, const void* bias, void* out, int num_tokens, int inter, int activation,
                          float limit, int dtype, cudaStream_t stream) {
  const size_t total = (size_t)num_tokens * inter;
  if (total == 0) return 0;
  if (activation != ACT_SILU && activation != ACT_GELU_TANH && activation != ACT_CLAMPED_SWISH) return TS_ERR_BAD_ARGUMENT;
  if (activation == ACT_CLAMPED_SWISH && !(limit > 0.f)) return TS_ERR_BAD_ARGUMENT;
  const int b = blocks_for(total, 256);
#define TS_ACT_CASE(T_, ACT_) \
  return launch(act_mul_kernel<T_, ACT_>, b, 256, 0, stream, (const T_*)gate_up, (const T_*)bias, (T_*)out, inter, total, limit)
  if (dtype == TS_DTYPE_F32) {
    if (activation == ACT_SILU) TS_ACT_CASE(float, ACT_SILU);
    if (activation == ACT_CLAMPED_SWISH) TS_ACT_CASE(float, ACT_CLAMPED_SWISH);
    TS_ACT_CASE(float, ACT_GELU_TANH);
  }
  if (dtype == TS_DTYPE_BF16) {
    if (activation == ACT_SILU) TS_ACT_CASE(bf16, ACT_SILU);
    if (activation == ACT_CLAMPED_SWISH) TS_ACT_CASE(bf16, ACT_CLAMPED_SWISH);
    TS_ACT_CASE(bf16, ACT_GELU_TANH);
  }
#undef TS_ACT_CASE
  return TS_ERR_BAD_ARGUMENT;
}

extern "C" int ts_act_mul_gather(const void* x, int x_stride, const int* rows, const void* table, int table_rows,
                                 int table_width, int col0, void* out, int num_tokens, int n, int activation, int dtype,
                                 cudaStream_t stream) {
  const size_t total = (size_t)num_tokens * n;
  if (total == 0) return 0;
  if (activation != ACT_SILU && activation != ACT_GELU_TANH) return TS_ERR_BAD_ARGUMENT;
  if (col0 < 0 || col0 + n > table_width || x_stride < n) return TS_ERR_BAD_ARGUMENT;
  const int b = blocks_for(total, 256);
#define TS_GATHER_CASE(T_, ACT_)                                                                                      \
  return launch(act_mul_gather_kernel<T_, ACT_>, b, 256, 0, stream, (const T_*)x, x_stride, rows, (const T_*)table, \
                table_rows, table_width, col0, (T_*)out, n, total)
  if (dtype == TS_DTYPE_F32) {
    if (activation == ACT_SILU) TS_GATHER_CASE(float, ACT_SILU);
    TS_GATHER_CASE(float, ACT_GELU_TANH);
  }
  if (dtype == TS_DTYPE_BF16) {
    if (activation == ACT_SILU) TS_GATHER_CASE(bf16, ACT_SILU);
    TS_GATHER_CASE(bf16, ACT_GELU_TANH);
  }
#undef TS_GATHER_CASE
  return TS_ERR_BAD_ARGUMENT;
}

extern "C" int ts_softcap(float* x, size_t total, float cap, cudaStream_t stream) {
  if (total == 0) return 0;
  if (!(cap > 0.f)) return TS_ERR_BAD_ARGUMENT;
  return launch(softcap_kernel, blocks_for(total, 256), 256, 0, stream, x, cap, 1.f / cap, total);
}

extern "C" int ts_head_norm_gate(const void* x, int x_is_f32, const void* weight, int weight_head_stride,
                                 const void* gate, int gate_stride, void* out, int num_tokens, int heads, int width,
                                 int normalise, float eps, int gate_per_head, int gate_silu, int dtype,
                                 cudaStream_t stream) {
  const size_t warps = (size_t)num_tokens * heads;
  if (warps == 0) return 0;
  if (width >= 512) {      // a CTA per row
    const int rows = (int)warps;
    if (dtype == TS_DTYPE_F32)
      return launch(head_norm_gate_wide_kernel<float, float>, rows, 256, 0, stream, (const float*)x, (const float*)weight,
                    weight_head_stride, (const float*)gate, gate_stride, (float*)out, heads, width, normalise, eps, gate_per_head, gate_silu);
    if (dtype != TS_DTYPE_BF16) return TS_ERR_BAD_ARGUMENT;
    if (x_is_f32)
      return launch(head_norm_gate_wide_kernel<float, bf16>, rows, 256, 0, stream, (const float*)x, (const bf16*)weight,
                    weight_head_stride, (const bf16*)gate, gate_stride, (bf16*)out, heads, width, normalise, eps, gate_per_head, gate_silu);
    return launch(head_norm_gate_wide_kernel<bf16, bf16>, rows, 256, 0, stream, (const bf16*)x, (const bf16*)weight,
                  weight_head_stride, (const bf16*)gate, gate_stride, (bf16*)out, heads, width, normalise, eps, gate_per_head, gate_silu);
  }
  const int threads = 128;
  const int b = (int)((warps * 32 + threads - 1) / threads);
  if (dtype == TS_DTYPE_F32)
    return launch(head_norm_gate_kernel<float, float>, b, threads, 0, stream, (const float*)x, (const float*)weight,
                  weight_head_stride, (const float*)gate, gate_stride, (float*)out, num_tokens, heads, width, normalise, eps, gate_per_head, gate_silu);
  if (dtype != TS_DTYPE_BF16) return TS_ERR_BAD_ARGUMENT;
  if (x_is_f32)
    return launch(head_norm_gate_kernel<float, bf16>, b, threads, 0, stream, (const float*)x, (const bf16*)weight,
                  weight_head_stride, (const bf16*)gate, gate_stride, (bf16*)out, num_tokens, heads, width, normalise, eps, gate_per_head, gate_silu);
  return launch(head_norm_gate_kernel<bf16, bf16>, b, threads, 0, stream, (const bf16*)x, (const bf16*)weight,
                weight_head_stride, (const bf16*)gate, gate_stride, (bf16*)out, num_tokens, heads, width, normalise, eps, gate_per_head, gate_silu);
}

extern "C" int ts_rms_norm_rows(const void* x, long long x_stride, const void* weight, float eps, void* out, int num_rows,
                                int width, int dtype, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (width <= 0 || x_stride < width || !weight) return TS_ERR_BAD_ARGUMENT;
  const int threads = width >= 512 ? 256 : width >= 128 ? 128 : 32;
  if (dtype == TS_DTYPE_F32)
    return launch(rms_norm_rows_kernel<float>, num_rows, threads, 0, stream, (const float*)x, x_stride, (const float*)weight, eps,
                  (float*)out, width);
  if (dtype == TS_DTYPE_BF16)
    return launch(rms_norm_rows_kernel<bf16>, num_rows, threads, 0, stream, (const bf16*)x, x_stride, (const bf16*)weight, eps,
                  (bf16*)out, width);
  return TS_ERR_BAD_ARGUMENT;
}
