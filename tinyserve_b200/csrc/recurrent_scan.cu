// Recurrent mixers with a matrix state per (request, head): the state S [d x dv] lives in a
// slot of 32-bit floats, is loaded once per step into registers, advanced token by token over
// the request's new tokens, and stored back. Prompt portions and single decoded tokens are the
// same kernel; what a request brings is read from cu_q on the device.
//
// Work split: a CTA owns (request, head, block of 32 value columns). Its compute warps split the
// key rows into contiguous runs of RPT rows (one warp up to 128 key rows, two up to 256); lane c
// owns column c of the block, so a thread keeps RPT elements of S in registers and a read-out
// sum over the key rows is a sum over the thread's own registers (plus one exchange through
// shared memory when there are two compute warps). Four loader warps stage the operands of the
// next chunk of tokens in shared memory (two buffers) while the compute warps walk the current
// one: they convert to 32-bit, and compute everything that does not depend on the state (log
// gates, decays, sigmoid, the unit scalings), so that the token-by-token chain holds only the
// state update itself. One block barrier per chunk.
//
//  * mLSTM: m' = max(f + m, i); S <- e^(f + m - m') S + e^(i - m') k v^T; n likewise with k;
//    o = S^T q / (max(|n.q|, e^(-m')) + 1e-6), with log gates i = cap tanh(a_i / cap) and
//    f = logsigmoid(cap tanh(a_f / cap)). A lane keeps RPT / 32 rows of the normaliser n.
//  * gated delta rule with a decay per key channel: S <- diag(g) S; u = beta (v - S^T k);
//    S <- S + k u^T; o = S^T q, with q and k scaled to unit length (q also by q_scale) and
//    g = exp(-exp(A_log) softplus(a + dt_bias)). The unit scalings are applied to the sums,
//    not to the vectors: S^T (k/|k|) = (S^T k)/|k|.
//  * the short causal convolution with SiLU in front of it, whose last taps-1 inputs are state too.
#define TS_PDL_CLASS PDL_OTHER
#include "common.cuh"

namespace ts {

constexpr int SCAN_MAX_TAPS = 8;
constexpr int SCAN_MAX_KEY_DIM = 256;   // eight compute warps of 32 key rows, or two of 128
constexpr int SCAN_LOADER_WARPS = 4;
constexpr int SCAN_LOADS = 8;           // elements a loader thread has in flight

__device__ __forceinline__ float softplusf(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float logsigmoidf(float z) { return z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z)); }
__device__ __forceinline__ void compute_warps_sync(int threads) { asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory"); }

// ------------------------------------------------------------------------ mLSTM
// Shared memory per buffer: q [CH][dpad] (scaled), k [CH][dpad], v [CH][32], log gates [CH][2].
template <typename T, int RPT>
__global__ void mlstm_scan_kernel(const T* __restrict__ qkv, int stride, int q_off, int k_off, int v_off,
                                  const float* __restrict__ gates, const float* __restrict__ gate_bias, float cap,
                                  float q_scale, float* __restrict__ state, int state_stride,
                                  const int* __restrict__ cu_q, const int* __restrict__ state_slots, int H, int d,
                                  int dv, float* __restrict__ out, int W, int CH) {
  extern __shared__ __align__(16) float sm[];
  constexpr int NPL = RPT / 32;
  const int dpad = W * RPT;
  const int buf_floats = CH * (2 * dpad + 32 + 2);
  float* part = sm + 2 * buf_floats;            // [CH][W][32] read-out parts of the chunk's tokens
  float* nqp = part + CH * W * 32;              // [CH][W] parts of n . q
  float* mcs = nqp + CH * W;                    // [CH] the running maximum after each token
  const int b = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_trigger();
  pdl_wait();
  const int start = cu_q[b], end = cu_q[b + 1];
  if (end <= start) return;
  const int chunks = (end - start + CH - 1) / CH;
  const bool loader = warp >= W;

  auto load_chunk = [&](int c) {
    float* q_s = sm + (c & 1) * buf_floats;
    float* k_s = q_s + CH * dpad;
    float* v_s = k_s + CH * dpad;
    float* g_s = v_s + CH * 32;
    const int t0 = start + c * CH, nt = min(CH, end - t0);
    const int lt = tid - W * 32, ln = SCAN_LOADER_WARPS * 32;
    // eight elements a thread and round: all their loads are in flight before the first is stored
    for (int base = lt; base < nt * dpad; base += ln * SCAN_LOADS) {
      float qv[SCAN_LOADS], kv[SCAN_LOADS];
#pragma unroll
      for (int u = 0; u < SCAN_LOADS; ++u) {
        const int idx = base + u * ln;
        const int tok = idx / dpad, r = idx - tok * dpad;
        const bool ok = idx < nt * dpad && r < d;
        const T* row = qkv + (size_t)(t0 + tok) * stride;
        qv[u] = ok ? to_float(row[q_off + h * d + r]) * q_scale : 0.f;
        kv[u] = ok ? to_float(row[k_off + h * d + r]) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < SCAN_LOADS; ++u) {
        const int idx = base + u * ln;
        if (idx < nt * dpad) {
          q_s[idx] = qv[u];
          k_s[idx] = kv[u];
        }
      }
    }
    for (int idx = lt; idx < nt * 32; idx += ln) {
      const int tok = idx >> 5, c2 = idx & 31;
      v_s[idx] = (c0 + c2 < dv) ? to_float(qkv[(size_t)(t0 + tok) * stride + v_off + h * dv + c0 + c2]) : 0.f;
    }
    for (int tok = lt; tok < nt; tok += ln) {
      const float ai = gates[(size_t)(t0 + tok) * 2 * H + h] + gate_bias[h];
      const float af = gates[(size_t)(t0 + tok) * 2 * H + H + h] + gate_bias[H + h];
      g_s[2 * tok] = cap * tanhf(ai / cap);
      g_s[2 * tok + 1] = logsigmoidf(cap * tanhf(af / cap));
    }
  };

  // ---- the state of this thread: RPT rows of its column, NPL rows of n, the running maximum
  const int slot = state_slots[b];
  const int col = c0 + lane;
  const bool col_ok = col < dv;
  // per head: S [d][dv], then one copy of (n [d], m) per column block, so that the CTAs of a
  // head share nothing that one of them writes
  float* S = state + (size_t)slot * state_stride + (size_t)h * ((size_t)d * dv + (size_t)gridDim.z * (d + 1));
  float* nvec = S + (size_t)d * dv + (size_t)blockIdx.z * (d + 1);
  float* mptr = nvec + d;
  const int r0 = warp * RPT;
  float s[RPT], n[NPL], m = 0.f;
  if (!loader) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) s[i] = (r0 + i < d && col_ok) ? S[(size_t)(r0 + i) * dv + col] : 0.f;
#pragma unroll
    for (int u = 0; u < NPL; ++u) n[u] = (r0 + lane + 32 * u < d) ? nvec[r0 + lane + 32 * u] : 0.f;
    m = *mptr;
  } else {
    load_chunk(0);
  }
  __syncthreads();
  for (int c = 0; c < chunks; ++c) {
    if (loader) {
      if (c + 1 < chunks) load_chunk(c + 1);
    } else {
      const float* q_s = sm + (c & 1) * buf_floats;
      const float* k_s = q_s + CH * dpad;
      const float* v_s = k_s + CH * dpad;
      const float* g_s = v_s + CH * 32;
      const int t0 = start + c * CH, nt = min(CH, end - t0);
      for (int tok = 0; tok < nt; ++tok) {
        const float li = g_s[2 * tok], lf = g_s[2 * tok + 1];
        const float m_new = fmaxf(lf + m, li);
        const float keep = expf(lf + m - m_new), take = expf(li - m_new);
        m = m_new;
        const float4* q4 = reinterpret_cast<const float4*>(q_s + tok * dpad + r0);
        const float4* k4 = reinterpret_cast<const float4*>(k_s + tok * dpad + r0);
        const float tv = take * v_s[tok * 32 + lane];
        float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
        for (int i = 0; i < RPT / 4; ++i) {
          const float4 kk = k4[i], qq = q4[i];
          s[4 * i] = fmaf(keep, s[4 * i], kk.x * tv);
          s[4 * i + 1] = fmaf(keep, s[4 * i + 1], kk.y * tv);
          s[4 * i + 2] = fmaf(keep, s[4 * i + 2], kk.z * tv);
          s[4 * i + 3] = fmaf(keep, s[4 * i + 3], kk.w * tv);
          acc0 = fmaf(s[4 * i], qq.x, acc0);
          acc1 = fmaf(s[4 * i + 1], qq.y, acc1);
          acc0 = fmaf(s[4 * i + 2], qq.z, acc0);
          acc1 = fmaf(s[4 * i + 3], qq.w, acc1);
        }
        float nq = 0.f;
#pragma unroll
        for (int u = 0; u < NPL; ++u) {
          const int r = r0 + lane + 32 * u;
          n[u] = fmaf(keep, n[u], take * k_s[tok * dpad + r]);
          nq = fmaf(n[u], q_s[tok * dpad + r], nq);
        }
        // the parts of this token's read-out wait in shared memory until the chunk is done: the next
        // token's update needs none of them, so no warp waits for another inside a chunk
        nq = warp_sum(nq);
        part[(tok * W + warp) * 32 + lane] = acc0 + acc1;
        if (lane == 0) {
          nqp[tok * W + warp] = nq;
          if (warp == 0) mcs[tok] = m;
        }
      }
      if (W > 1) compute_warps_sync(W * 32); else __syncwarp();
      for (int tok = warp; tok < nt; tok += W) {
        float acc = 0.f, nq = 0.f;
        for (int w = 0; w < W; ++w) {
          acc += part[(tok * W + w) * 32 + lane];
          nq += nqp[tok * W + w];
        }
        if (col_ok) out[((size_t)(t0 + tok) * H + h) * dv + col] = acc / (fmaxf(fabsf(nq), expf(-mcs[tok])) + 1e-6f);
      }
    }
    __syncthreads();
  }
  if (loader) return;
#pragma unroll
  for (int i = 0; i < RPT; ++i)
    if (r0 + i < d && col_ok) S[(size_t)(r0 + i) * dv + col] = s[i];
#pragma unroll
  for (int u = 0; u < NPL; ++u)
    if (r0 + lane + 32 * u < d) nvec[r0 + lane + 32 * u] = n[u];
  if (tid == 0) *mptr = m;
}

// ------------------------------------------------------------------- delta rule
// Shared memory per buffer: q [CH][dpad], k [CH][dpad], g [CH][dpad], v [CH][32], and per token
// beta, 1/|k|, q_scale/|q|.
template <int RPT>
__global__ void delta_scan_kernel(const float* __restrict__ qkv, int stride, int q_off, int k_off, int v_off,
                                  const float* __restrict__ a, int a_stride, int a_per_head,
                                  const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                  const float* __restrict__ beta_pre, int beta_stride,
                                  float q_scale, float* __restrict__ state, int state_stride,
                                  const int* __restrict__ cu_q, const int* __restrict__ state_slots, int H, int G,
                                  int d, int dv, float* __restrict__ out, int W, int CH) {
  extern __shared__ __align__(16) float sm[];
  const int dpad = W * RPT;
  const int buf_floats = CH * (3 * dpad + 32 + 4);
  float* part = sm + 2 * buf_floats;            // [2][W][32] parts of S^T k, exchanged token by token
  float* outp = part + 2 * W * 32;              // [CH][W][32] read-out parts of the chunk's tokens
  const int b = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * 32;
  const int g = h / (H / G);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_trigger();
  pdl_wait();
  const int start = cu_q[b], end = cu_q[b + 1];
  if (end <= start) return;
  const int chunks = (end - start + CH - 1) / CH;
  const bool loader = warp >= W;
  const float A = expf(a_log[h]);

  auto load_chunk = [&](int c) {
    float* q_s = sm + (c & 1) * buf_floats;
    float* k_s = q_s + CH * dpad;
    float* g_s = k_s + CH * dpad;
    float* v_s = g_s + CH * dpad;
    float* t_s = v_s + CH * 32;
    const int t0 = start + c * CH, nt = min(CH, end - t0);
    const int lt = tid - W * 32, ln = SCAN_LOADER_WARPS * 32, lw = warp - W;
    // eight elements a thread and round: all their loads are in flight before the first is stored
    for (int base = lt; base < nt * dpad; base += ln * SCAN_LOADS) {
      float qv[SCAN_LOADS], kv[SCAN_LOADS], av[SCAN_LOADS];
#pragma unroll
      for (int u = 0; u < SCAN_LOADS; ++u) {
        const int idx = base + u * ln;
        const int tok = idx / dpad, r = idx - tok * dpad;
        const bool ok = idx < nt * dpad && r < d;
        const float* row = qkv + (size_t)(t0 + tok) * stride;
        qv[u] = ok ? row[q_off + g * d + r] : 0.f;
        kv[u] = ok ? row[k_off + g * d + r] : 0.f;
        const int ac = a_per_head ? h : h * d + r;   // one step size per head, or per head and key channel
        av[u] = ok ? a[(size_t)(t0 + tok) * a_stride + ac] + dt_bias[ac] : -INFINITY;
      }
#pragma unroll
      for (int u = 0; u < SCAN_LOADS; ++u) {
        const int idx = base + u * ln;
        if (idx < nt * dpad) {
          q_s[idx] = qv[u];
          k_s[idx] = kv[u];
          g_s[idx] = av[u] == -INFINITY ? 1.f : expf(-A * softplusf(av[u]));
        }
      }
    }
    for (int idx = lt; idx < nt * 32; idx += ln) {
      const int tok = idx >> 5, c2 = idx & 31;
      v_s[idx] = (c0 + c2 < dv) ? qkv[(size_t)(t0 + tok) * stride + v_off + h * dv + c0 + c2] : 0.f;
    }
    // the unit scalings: once the loader warps have stored the chunk, a loader warp per token
    asm volatile("bar.sync 2, %0;" ::"r"(SCAN_LOADER_WARPS * 32) : "memory");
    for (int tok = lw; tok < nt; tok += SCAN_LOADER_WARPS) {
      float qq = 0.f, kk = 0.f;
      for (int r = lane; r < d; r += 32) {
        const float qv = q_s[tok * dpad + r], kv = k_s[tok * dpad + r];
        qq = fmaf(qv, qv, qq);
        kk = fmaf(kv, kv, kk);
      }
      qq = warp_sum(qq);
      kk = warp_sum(kk);
      if (lane == 0) {
        const float z = beta_pre[(size_t)(t0 + tok) * beta_stride + h];
        t_s[4 * tok] = 1.f / (1.f + expf(-z));
        t_s[4 * tok + 1] = rsqrtf(kk + 1e-6f);
        t_s[4 * tok + 2] = rsqrtf(qq + 1e-6f) * q_scale;
      }
    }
  };

  const int slot = state_slots[b];
  const int col = c0 + lane;
  const bool col_ok = col < dv;
  float* S = state + (size_t)slot * state_stride + (size_t)h * d * dv;
  const int r0 = warp * RPT;
  float s[RPT];
  if (!loader) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) s[i] = (r0 + i < d && col_ok) ? S[(size_t)(r0 + i) * dv + col] : 0.f;
  } else {
    load_chunk(0);
  }
  __syncthreads();
  int par = 0;
  for (int c = 0; c < chunks; ++c) {
    if (loader) {
      if (c + 1 < chunks) load_chunk(c + 1);
    } else {
      const float* q_s = sm + (c & 1) * buf_floats;
      const float* k_s = q_s + CH * dpad;
      const float* g_s = k_s + CH * dpad;
      const float* v_s = g_s + CH * dpad;
      const float* t_s = v_s + CH * 32;
      const int t0 = start + c * CH, nt = min(CH, end - t0);
      for (int tok = 0; tok < nt; ++tok) {
        const float4* q4 = reinterpret_cast<const float4*>(q_s + tok * dpad + r0);
        const float4* k4 = reinterpret_cast<const float4*>(k_s + tok * dpad + r0);
        const float4* g4 = reinterpret_cast<const float4*>(g_s + tok * dpad + r0);
        const float beta = t_s[4 * tok], rk = t_s[4 * tok + 1];
        float p0 = 0.f, p1 = 0.f;
#pragma unroll
        for (int i = 0; i < RPT / 4; ++i) {
          const float4 kk = k4[i], gg = g4[i];
          s[4 * i] *= gg.x;
          s[4 * i + 1] *= gg.y;
          s[4 * i + 2] *= gg.z;
          s[4 * i + 3] *= gg.w;
          p0 = fmaf(s[4 * i], kk.x, p0);
          p1 = fmaf(s[4 * i + 1], kk.y, p1);
          p0 = fmaf(s[4 * i + 2], kk.z, p0);
          p1 = fmaf(s[4 * i + 3], kk.w, p1);
        }
        float pred = p0 + p1;
        if (W > 1) {
          part[(par * W + warp) * 32 + lane] = pred;
          compute_warps_sync(W * 32);
          pred = 0.f;
          for (int w = 0; w < W; ++w) pred += part[(par * W + w) * 32 + lane];
          par ^= 1;
        }
        const float wu = beta * (v_s[tok * 32 + lane] - pred * rk) * rk;
        float o0 = 0.f, o1 = 0.f;
#pragma unroll
        for (int i = 0; i < RPT / 4; ++i) {
          const float4 kk = k4[i], qq = q4[i];
          s[4 * i] = fmaf(kk.x, wu, s[4 * i]);
          s[4 * i + 1] = fmaf(kk.y, wu, s[4 * i + 1]);
          s[4 * i + 2] = fmaf(kk.z, wu, s[4 * i + 2]);
          s[4 * i + 3] = fmaf(kk.w, wu, s[4 * i + 3]);
          o0 = fmaf(s[4 * i], qq.x, o0);
          o1 = fmaf(s[4 * i + 1], qq.y, o1);
          o0 = fmaf(s[4 * i + 2], qq.z, o0);
          o1 = fmaf(s[4 * i + 3], qq.w, o1);
        }
        // the parts of this token's read-out wait in shared memory until the chunk is done
        outp[(tok * W + warp) * 32 + lane] = o0 + o1;
      }
      if (W > 1) compute_warps_sync(W * 32); else __syncwarp();
      for (int tok = warp; tok < nt; tok += W) {
        float o = 0.f;
        for (int w = 0; w < W; ++w) o += outp[(tok * W + w) * 32 + lane];
        if (col_ok) out[((size_t)(t0 + tok) * H + h) * dv + col] = o * t_s[4 * tok + 2];
      }
    }
    __syncthreads();
  }
  if (loader) return;
#pragma unroll
  for (int i = 0; i < RPT; ++i)
    if (r0 + i < d && col_ok) S[(size_t)(r0 + i) * dv + col] = s[i];
}

// ------------------------------------------------- short causal convolution + SiLU
// Input of token tau of request b, channel c: x[tau][c] for tokens of this step, the state's
// row (K - 1) + (tau - start) for the K - 1 tokens before it (zero at a request's start).
template <typename T>
__device__ __forceinline__ float conv_input(const T* x, int x_stride, const float* st, int C, int K, int start,
                                            int tau, int c) {
  return tau >= start ? to_float(x[(size_t)tau * x_stride + c]) : st[(size_t)(K - 1 + tau - start) * C + c];
}

template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ taps,
                                        const float* __restrict__ state, int state_stride,
                                        const int* __restrict__ cu_q, const int* __restrict__ state_slots, int num_seqs,
                                        int num_tokens, int C, int K, float* __restrict__ y) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  // the request of token t: the last b with cu_q[b] <= t
  int lo = 0, hi = num_seqs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_q[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int start = cu_q[lo];
  const float* st = state + (size_t)state_slots[lo] * state_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < K; ++k)
      acc = fmaf(to_float(taps[(size_t)c * K + k]), conv_input(x, x_stride, st, C, K, start, t - (K - 1 - k), c), acc);
    y[(size_t)t * C + c] = acc / (1.f + expf(-acc));
  }
}

template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ state,
                                         int state_stride, const int* __restrict__ cu_q,
                                         const int* __restrict__ state_slots, int C, int K) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x;
  const int start = cu_q[b], end = cu_q[b + 1];
  if (end <= start) return;
  float* st = state + (size_t)state_slots[b] * state_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float keep[SCAN_MAX_TAPS];
    for (int i = 0; i < K - 1; ++i) keep[i] = conv_input(x, x_stride, st, C, K, start, end - (K - 1) + i, c);
    for (int i = 0; i < K - 1; ++i) st[(size_t)i * C + c] = keep[i];
  }
}

}  // namespace ts

using namespace ts;

// Rows of S per thread (32, 64 or 128; a measurement switch, see ts_scan_rows_per_thread), compute
// warps and tokens per staged chunk for a key size.
static int g_scan_rows_per_thread = 0;
extern "C" void ts_scan_rows_per_thread(int rows) { g_scan_rows_per_thread = (rows == 64 || rows == 128) ? rows : 32; }

struct ScanShape { int rpt, warps, chunk; };
static ScanShape scan_shape(int d) {
  ScanShape s;
  s.rpt = g_scan_rows_per_thread > 0 ? g_scan_rows_per_thread : 32;
  s.warps = (d + s.rpt - 1) / s.rpt;
  s.chunk = s.warps * s.rpt <= 128 ? 16 : 8;
  return s;
}

// Shared memory beyond 48 KB has to be allowed per kernel, once: `allowed` remembers the most allowed so far.
template <typename K>
static int allow_smem(K kern, size_t smem, size_t& allowed) {
  if (smem <= 48 * 1024 || smem <= allowed) return 0;
  const int e = (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == 0) allowed = smem;
  return e;
}

template <typename T, int RPT>
static int launch_mlstm(const ScanShape& sh, dim3 grid, cudaStream_t stream, const void* qkv, int stride, int q_off,
                        int k_off, int v_off, const float* gates, const float* gate_bias, float cap, float q_scale,
                        float* state, int state_stride, const int* cu_q, const int* state_slots, int heads, int d, int dv,
                        float* out) {
  const int dpad = sh.warps * RPT;
  const size_t smem = sizeof(float) * (2 * (size_t)sh.chunk * (2 * dpad + 32 + 2) + (size_t)sh.chunk * (sh.warps * 33 + 1));
  auto kern = mlstm_scan_kernel<T, RPT>;
  static size_t allowed = 0;
  if (int e = allow_smem(kern, smem, allowed)) return e;
  return launch(kern, grid, (sh.warps + SCAN_LOADER_WARPS) * 32, smem, stream, (const T*)qkv, stride, q_off, k_off, v_off,
                gates, gate_bias, cap, q_scale, state, state_stride, cu_q, state_slots, heads, d, dv, out, sh.warps, sh.chunk);
}

extern "C" int ts_mlstm_scan(const void* qkv, int stride, int q_off, int k_off, int v_off, const float* gates,
                             const float* gate_bias, float cap, float q_scale, float* state, int state_stride,
                             const int* cu_q, const int* state_slots, int num_seqs, int heads, int d, int dv, float* out,
                             int dtype, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (d <= 0 || dv <= 0 || d > SCAN_MAX_KEY_DIM || !(cap > 0.f)) return TS_ERR_UNSUPPORTED;
  if (dtype != TS_DTYPE_F32 && dtype != TS_DTYPE_BF16) return TS_ERR_BAD_ARGUMENT;
  const ScanShape sh = scan_shape(d);
  dim3 grid(num_seqs, heads, (dv + 31) / 32);
#define TS_MLSTM_CASE(RPT_)                                                                                          \
  return dtype == TS_DTYPE_F32                                                                                       \
             ? launch_mlstm<float, RPT_>(sh, grid, stream, qkv, stride, q_off, k_off, v_off, gates, gate_bias, cap,  \
                                         q_scale, state, state_stride, cu_q, state_slots, heads, d, dv, out)         \
             : launch_mlstm<bf16, RPT_>(sh, grid, stream, qkv, stride, q_off, k_off, v_off, gates, gate_bias, cap,   \
                                        q_scale, state, state_stride, cu_q, state_slots, heads, d, dv, out)
  if (sh.rpt == 32) { TS_MLSTM_CASE(32); }
  if (sh.rpt == 64) { TS_MLSTM_CASE(64); }
  TS_MLSTM_CASE(128);
#undef TS_MLSTM_CASE
}

template <int RPT>
static int launch_delta(const ScanShape& sh, dim3 grid, cudaStream_t stream, const float* qkv, int stride, int q_off,
                        int k_off, int v_off, const float* a, int a_stride, int a_per_head, const float* dt_bias,
                        const float* a_log, const float* beta_pre, int beta_stride, float q_scale, float* state,
                        int state_stride, const int* cu_q,
                        const int* state_slots, int heads, int kv_heads, int d, int dv, float* out) {
  const int dpad = sh.warps * RPT;
  const size_t smem = sizeof(float) * (2 * (size_t)sh.chunk * (3 * dpad + 32 + 4) + (2 + (size_t)sh.chunk) * sh.warps * 32);
  auto kern = delta_scan_kernel<RPT>;
  static size_t allowed = 0;
  if (int e = allow_smem(kern, smem, allowed)) return e;
  return launch(kern, grid, (sh.warps + SCAN_LOADER_WARPS) * 32, smem, stream, qkv, stride, q_off, k_off, v_off, a, a_stride,
                a_per_head, dt_bias, a_log, beta_pre, beta_stride, q_scale, state, state_stride, cu_q, state_slots, heads, kv_heads, d, dv, out, sh.warps,
                sh.chunk);
}

extern "C" int ts_delta_scan(const float* qkv, int stride, int q_off, int k_off, int v_off, const float* a,
                             int a_stride, int a_per_head, const float* dt_bias, const float* a_log,
                             const float* beta_pre, int beta_stride, float q_scale,
                             float* state, int state_stride, const int* cu_q, const int* state_slots, int num_seqs,
                             int heads, int kv_heads, int d, int dv, float* out, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (d <= 0 || dv <= 0 || d > SCAN_MAX_KEY_DIM) return TS_ERR_UNSUPPORTED;
  if (kv_heads <= 0 || heads % kv_heads) return TS_ERR_BAD_ARGUMENT;
  const ScanShape sh = scan_shape(d);
  dim3 grid(num_seqs, heads, (dv + 31) / 32);
#define TS_DELTA_CASE(RPT_)                                                                                        \
  return launch_delta<RPT_>(sh, grid, stream, qkv, stride, q_off, k_off, v_off, a, a_stride, a_per_head, dt_bias, a_log, \
                            beta_pre, beta_stride, q_scale, \
                            state, state_stride, cu_q, state_slots, heads, kv_heads, d, dv, out)
  if (sh.rpt == 32) { TS_DELTA_CASE(32); }
  if (sh.rpt == 64) { TS_DELTA_CASE(64); }
  TS_DELTA_CASE(128);
#undef TS_DELTA_CASE
}

extern "C" int ts_causal_conv_silu(const void* x, int x_stride, const void* taps, float* state, int state_stride, const int* cu_q,
                                   const int* state_slots, int num_seqs, int num_tokens, int channels, int num_taps,
                                   float* y, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0 || num_seqs <= 0) return 0;
  if (num_taps < 1 || num_taps > SCAN_MAX_TAPS) return TS_ERR_UNSUPPORTED;
  const int threads = 128;
  int by = (channels + threads - 1) / threads;
  if (by > 64) by = 64;
  dim3 grid(num_tokens, by), sgrid(num_seqs, by);
  int st;
  if (dtype == TS_DTYPE_F32) {
    st = launch(causal_conv_silu_kernel<float>, grid, threads, 0, stream, (const float*)x, x_stride, (const float*)taps,
                (const float*)state, state_stride, cu_q, state_slots, num_seqs, num_tokens, channels, num_taps, y);
    if (st != 0 || num_taps == 1) return st;
    return launch(conv_state_update_kernel<float>, sgrid, threads, 0, stream, (const float*)x, x_stride, state, state_stride, cu_q,
                  state_slots, channels, num_taps);
  }
  if (dtype == TS_DTYPE_BF16) {
    st = launch(causal_conv_silu_kernel<bf16>, grid, threads, 0, stream, (const bf16*)x, x_stride, (const bf16*)taps,
                (const float*)state, state_stride, cu_q, state_slots, num_seqs, num_tokens, channels, num_taps, y);
    if (st != 0 || num_taps == 1) return st;
    return launch(conv_state_update_kernel<bf16>, sgrid, threads, 0, stream, (const bf16*)x, x_stride, state, state_stride, cu_q,
                  state_slots, channels, num_taps);
  }
  return TS_ERR_BAD_ARGUMENT;
}
