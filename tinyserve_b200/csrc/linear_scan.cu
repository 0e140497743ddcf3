// Linear-attention mixers whose state is a matrix S [d x dv] per (request, head) in a slot of
// 32-bit floats, without a correction term: the state of a token depends on the one before only
// through a decay, so a token's chain is one multiply-add per element.
//
//  * MODE_BONUS (time mixing in the manner of RWKV-6): a decay per key channel and token,
//    w = exp(-exp(w_pre + w_0)); the read-out comes first and sees the current token only through a
//    bonus u per key channel: o = (S + diag(u) k v^T)^T r; then S <- diag(w) S + k v^T.
//  * MODE_DECAY (linear attention with a constant decay per head): q, k, v pass SiLU;
//    S <- decay_h S + k v^T; o = S^T q (the read-out sees the current token's write).
//  * MODE_GATED (gated linear attention): a decay per key channel and token,
//    alpha = sigmoid(z)^(1/tau) = exp(logsigmoid(z) / tau) with z = w_pre + w_0; q is multiplied by a constant;
//    S <- diag(alpha) S + k v^T; o = S^T q (the read-out sees the current token's write).
//
// Work split as in the other recurrent kernels: a CTA owns (request, head, block of 32 value
// columns); compute warp w owns key rows [w * RPT, (w + 1) * RPT) and lane c column c, so a thread
// keeps RPT elements of S in registers. Four loader warps stage the next chunk of tokens in shared
// memory as 32-bit values (activations, decays) while the compute warps walk the current one. The
// parts of a token's read-out (one per compute warp) wait in shared memory until the chunk is done.
// Prompt portions and single decoded tokens are the same kernel; a step in which no request brings more
// than one chunk of tokens (decoding) is launched without loader warps, and the compute warps stage the
// chunk themselves.
//
// A long portion is cut into segments that run side by side (SCAN_LOCAL, SCAN_FINAL): the state after a
// segment is diag(P) S_before + L, where L is what the segment's tokens leave behind from a zero state and
// P the product of its decays (per key channel, exp(-sum_t exp(w_pre_t + w_0)) or exp(sum_t logsigmoid(z_t) / tau), or decay_h^tokens). One
// launch runs every segment but a request's last from zero and stores L; a small kernel walks a request's
// segments in order and leaves each one's starting state in L's place; a last launch runs every segment
// from its starting state, writes the read-outs, and the request's last segment stores the slot. Twice the
// multiply-adds, but the chain is two segments long instead of the whole portion. All of it 32-bit.
//
// Also here: the token shift in front of the time mixing, out_m = h + (h_prev - h) * mu_m for
// several mixes m, where h_prev of a request's first token of the step comes from its state slot
// (zero at the request's start) and the slot then takes the step's last h.
#define TS_PDL_CLASS PDL_OTHER
#include "common.cuh"

namespace ts {

constexpr int LIN_MAX_KEY_DIM = 256;
constexpr int LIN_LOADER_WARPS = 4;
constexpr int LIN_LOADS = 8;
constexpr int LIN_RPT = 16;
constexpr int MODE_BONUS = 0, MODE_DECAY = 1, MODE_GATED = 2;
constexpr int SCAN_WHOLE = 0, SCAN_LOCAL = 1, SCAN_FINAL = 2;

__device__ __forceinline__ float siluf(float z) { return z / (1.f + expf(-z)); }
// log(sigmoid(z)) = min(z, 0) - log(1 + exp(-|z|))
__device__ __forceinline__ float logsigmoidf(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

struct LinScanArgs {
  const void* q; int q_stride;      // [T, H * d] rows q_stride apart (r of the time mixing)
  const void* k; int k_stride;      // [T, H * d]
  const void* v; int v_stride;      // [T, H * dv]
  const float* w_pre; int w_stride; // MODE_BONUS, MODE_GATED: [T, H * d] decay pre-activations
  const float* w_bias;              // MODE_BONUS, MODE_GATED: [H * d]
  float inv_tau, q_scale;           // MODE_GATED: 1 / tau of the decay, and the constant on q
  const float* bonus;               // MODE_BONUS: [H * d]
  const float* decay;               // MODE_DECAY: [H]
  float* state; int state_stride;   // [slots, H * d * dv]
  const int* cu_q; const int* state_slots;
  int H, d, dv;
  float* out;                       // [T, H, dv]
  int W, CH;
  int loader_warps;                 // LIN_LOADER_WARPS, or 0 when every request's tokens fit one chunk
  int seg_len, max_segs;            // segmented: tokens per segment, segments per request in the grid
  float* seg_state;                 // segmented: [num_seqs * max_segs, H * d * dv]
  float* seg_decay;                 // segmented, MODE_BONUS, MODE_GATED: [num_seqs * max_segs, H * d] products of the decays
};

template <typename T, int MODE, int PASS>
__device__ __forceinline__ void linear_scan_body(const LinScanArgs& a) {
  extern __shared__ __align__(16) float sm[];
  constexpr int RPT = LIN_RPT;
  constexpr bool CHANNEL_DECAY = MODE == MODE_BONUS || MODE == MODE_GATED;
  constexpr int NARR = CHANNEL_DECAY ? 3 : 2;
  const int W = a.W, CH = a.CH, d = a.d, dv = a.dv, H = a.H;
  const int dpad = W * RPT;
  const int buf_floats = CH * (NARR * dpad + 32);
  float* part = sm + 2 * buf_floats;            // [CH][W][32]
  const int b = PASS == SCAN_WHOLE ? blockIdx.x : blockIdx.x / a.max_segs;
  const int seg = PASS == SCAN_WHOLE ? 0 : blockIdx.x - b * a.max_segs;
  const int h = blockIdx.y, c0 = blockIdx.z * 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_trigger();
  pdl_wait();
  int start = a.cu_q[b], end = a.cu_q[b + 1];
  if (end <= start) return;
  bool last_seg = true;
  if (PASS != SCAN_WHOLE) {
    const int nsegs = (end - start + a.seg_len - 1) / a.seg_len;
    last_seg = seg == nsegs - 1;
    if (seg >= nsegs || (PASS == SCAN_LOCAL && last_seg)) return;
    start += seg * a.seg_len;
    end = min(end, start + a.seg_len);
  }
  const int chunks = (end - start + CH - 1) / CH;
  const bool loader = warp >= W;
  const bool own_loads = a.loader_warps == 0;    // one chunk a request: the compute warps stage it themselves
  const T* qp = (const T*)a.q;
  const T* kp = (const T*)a.k;
  const T* vp = (const T*)a.v;

  auto load_chunk = [&](int c) {
    float* q_s = sm + (c & 1) * buf_floats;
    float* k_s = q_s + CH * dpad;
    float* w_s = k_s + CH * dpad;                       // a decay per key channel only
    float* v_s = q_s + NARR * CH * dpad;
    const int t0 = start + c * CH, nt = min(CH, end - t0);
    const int lt = own_loads ? tid : tid - W * 32, ln = (own_loads ? W : LIN_LOADER_WARPS) * 32;
    for (int base = lt; base < nt * dpad; base += ln * LIN_LOADS) {
      float qv[LIN_LOADS], kv[LIN_LOADS], wv[LIN_LOADS];
#pragma unroll
      for (int u = 0; u < LIN_LOADS; ++u) {
        const int idx = base + u * ln;
        const int tok = idx / dpad, r = idx - tok * dpad;
        const bool ok = idx < nt * dpad && r < d;
        qv[u] = ok ? to_float(qp[(size_t)(t0 + tok) * a.q_stride + h * d + r]) : 0.f;
        kv[u] = ok ? to_float(kp[(size_t)(t0 + tok) * a.k_stride + h * d + r]) : 0.f;
        if (CHANNEL_DECAY) wv[u] = ok ? a.w_pre[(size_t)(t0 + tok) * a.w_stride + h * d + r] + a.w_bias[h * d + r] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < LIN_LOADS; ++u) {
        const int idx = base + u * ln;
        if (idx < nt * dpad) {
          if (MODE == MODE_DECAY) {
            q_s[idx] = siluf(qv[u]);
            k_s[idx] = siluf(kv[u]);
          } else if (MODE == MODE_GATED) {
            q_s[idx] = qv[u] * a.q_scale;
            k_s[idx] = kv[u];
            w_s[idx] = expf(logsigmoidf(wv[u]) * a.inv_tau);
          } else {
            q_s[idx] = qv[u];
            k_s[idx] = kv[u];
            w_s[idx] = expf(-expf(wv[u]));
          }
        }
      }
    }
    for (int idx = lt; idx < nt * 32; idx += ln) {
      const int tok = idx >> 5, c2 = idx & 31;
      float x = (c0 + c2 < dv) ? to_float(vp[(size_t)(t0 + tok) * a.v_stride + h * dv + c0 + c2]) : 0.f;
      if (MODE == MODE_DECAY) x = siluf(x);
      v_s[idx] = x;
    }
  };

  const int slot = a.state_slots[b];
  const int col = c0 + lane;
  const bool col_ok = col < dv;
  float* S = a.state + (size_t)slot * a.state_stride + (size_t)h * d * dv;
  float* S_seg = PASS == SCAN_WHOLE ? nullptr : a.seg_state + ((size_t)blockIdx.x * H + h) * d * dv;
  const float* S_in = PASS == SCAN_FINAL ? S_seg : S;
  float* S_out = PASS == SCAN_LOCAL ? S_seg : S;
  const int r0 = warp * RPT;
  float s[RPT], u[MODE == MODE_BONUS ? RPT : 1];
  float decay = 1.f;
  if (!loader) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) s[i] = (PASS != SCAN_LOCAL && r0 + i < d && col_ok) ? S_in[(size_t)(r0 + i) * dv + col] : 0.f;
    if (MODE == MODE_BONUS) {
#pragma unroll
      for (int i = 0; i < RPT; ++i) u[i] = (r0 + i < d) ? a.bonus[h * d + r0 + i] : 0.f;
    } else if (MODE == MODE_DECAY) {
      decay = a.decay[h];
    }
  }
  if (loader || own_loads) load_chunk(0);
  __syncthreads();
  for (int c = 0; c < chunks; ++c) {
    if (own_loads && c > 0) {       // not expected (the host saw a shorter step): still every chunk is staged
      load_chunk(c);
      __syncthreads();
    }
    if (loader) {
      if (c + 1 < chunks) load_chunk(c + 1);
    } else {
      const float* q_s = sm + (c & 1) * buf_floats;
      const float* k_s = q_s + CH * dpad;
      const float* w_s = k_s + CH * dpad;
      const float* v_s = q_s + NARR * CH * dpad;
      const int t0 = start + c * CH, nt = min(CH, end - t0);
      for (int tok = 0; tok < nt; ++tok) {
        const float4* q4 = reinterpret_cast<const float4*>(q_s + tok * dpad + r0);
        const float4* k4 = reinterpret_cast<const float4*>(k_s + tok * dpad + r0);
        const float4* w4 = reinterpret_cast<const float4*>(w_s + tok * dpad + r0);
        const float vv = v_s[tok * 32 + lane];
        float o0 = 0.f, o1 = 0.f;
#pragma unroll
        for (int i = 0; i < RPT / 4; ++i) {
          const float4 kk = k4[i], qq = q4[i];
          const float kx[4] = {kk.x, kk.y, kk.z, kk.w}, qx[4] = {qq.x, qq.y, qq.z, qq.w};
          if (MODE == MODE_BONUS) {
            const float4 ww = w4[i];
            const float wx[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float kv = kx[e] * vv;
              if (PASS != SCAN_LOCAL) {
                const float seen = fmaf(u[4 * i + e], kv, s[4 * i + e]);
                if (e & 1) o1 = fmaf(seen, qx[e], o1); else o0 = fmaf(seen, qx[e], o0);
              }
              s[4 * i + e] = fmaf(wx[e], s[4 * i + e], kv);
            }
          } else if (MODE == MODE_GATED) {
            const float4 ww = w4[i];
            const float wx[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              s[4 * i + e] = fmaf(wx[e], s[4 * i + e], kx[e] * vv);
              if (PASS != SCAN_LOCAL) {
                if (e & 1) o1 = fmaf(s[4 * i + e], qx[e], o1); else o0 = fmaf(s[4 * i + e], qx[e], o0);
              }
            }
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              s[4 * i + e] = fmaf(decay, s[4 * i + e], kx[e] * vv);
              if (PASS != SCAN_LOCAL) {
                if (e & 1) o1 = fmaf(s[4 * i + e], qx[e], o1); else o0 = fmaf(s[4 * i + e], qx[e], o0);
              }
            }
          }
        }
        if (PASS != SCAN_LOCAL) part[(tok * W + warp) * 32 + lane] = o0 + o1;
      }
      if (PASS != SCAN_LOCAL) {
        if (W > 1) asm volatile("bar.sync 1, %0;" ::"r"(W * 32) : "memory"); else __syncwarp();
        for (int tok = warp; tok < nt; tok += W) {
          float o = 0.f;
          for (int w = 0; w < W; ++w) o += part[(tok * W + w) * 32 + lane];
          if (col_ok) a.out[((size_t)(t0 + tok) * H + h) * dv + col] = o;
        }
      }
    }
    __syncthreads();
  }
  if (loader || (PASS == SCAN_FINAL && !last_seg)) return;
#pragma unroll
  for (int i = 0; i < RPT; ++i)
    if (r0 + i < d && col_ok) S_out[(size_t)(r0 + i) * dv + col] = s[i];
}

template <typename T, int MODE>
__global__ void linear_scan_kernel(LinScanArgs a) { linear_scan_body<T, MODE, SCAN_WHOLE>(a); }

// The passes over segments: 80 registers a thread (a few spilled words outside the token loop) let three CTAs of
// eight warps share an SM instead of two: 9 to 25 % off a pass at key sizes 64 and 128. The one-launch form, which
// single tokens take, keeps the registers it asks for.
template <typename T, int MODE, int PASS>
__global__ void __maxnreg__(80) linear_scan_segment_kernel(LinScanArgs a) { linear_scan_body<T, MODE, PASS>(a); }

// The product of a segment's decays per key channel, exp(-sum_t exp(w_pre_t + w_0)) (MODE_GATED:
// exp(sum_t logsigmoid(w_pre_t + w_0) / tau)), for every segment but a request's last. A thread per channel; grid
// (request * max_segs + segment, blocks of 128 channels).
template <int MODE>
__global__ void linear_scan_seg_decay_kernel(LinScanArgs a) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x / a.max_segs, seg = blockIdx.x - b * a.max_segs;
  const int ch = blockIdx.y * blockDim.x + threadIdx.x;
  int start = a.cu_q[b];
  const int end = a.cu_q[b + 1];
  const int nsegs = (end - start + a.seg_len - 1) / a.seg_len;
  if (seg >= nsegs - 1 || ch >= a.H * a.d) return;
  start += seg * a.seg_len;
  const float bias = a.w_bias[ch];
  const float* wp = a.w_pre + (size_t)start * a.w_stride + ch;
  float sum = 0.f;
  int t = 0;
  for (; t + 8 <= a.seg_len; t += 8) {           // eight loads in flight
    float x[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = wp[(size_t)(t + j) * a.w_stride];
#pragma unroll
    for (int j = 0; j < 8; ++j) sum += MODE == MODE_GATED ? -logsigmoidf(x[j] + bias) * a.inv_tau : expf(x[j] + bias);
  }
  for (; t < a.seg_len; ++t) {
    const float z = wp[(size_t)t * a.w_stride] + bias;
    sum += MODE == MODE_GATED ? -logsigmoidf(z) * a.inv_tau : expf(z);
  }
  a.seg_decay[(size_t)blockIdx.x * a.H * a.d + ch] = expf(-sum);
}

// A request's segments in order: seg_state[segment] holds what the segment leaves from a zero state and
// receives the state the segment starts from (the slot's for the first). A thread per state element; grid
// (request, head, blocks of 256 elements).
template <int MODE>
__global__ void linear_scan_combine_kernel(LinScanArgs a) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const int idx = blockIdx.z * blockDim.x + threadIdx.x;
  const int start = a.cu_q[b], end = a.cu_q[b + 1];
  const int nsegs = (end - start + a.seg_len - 1) / a.seg_len;
  const int per_head = a.d * a.dv;
  if (nsegs <= 0 || idx >= per_head) return;
  const int r = idx / a.dv;
  float s = a.state[(size_t)a.state_slots[b] * a.state_stride + (size_t)h * per_head + idx];
  float p_const = 1.f;
  if (MODE == MODE_DECAY && nsegs > 1) {
    const float dec = a.decay[h];
    for (int t = 0; t < a.seg_len; ++t) p_const *= dec;
  }
  const size_t seg_stride = (size_t)a.H * per_head;
  float* p0 = a.seg_state + ((size_t)b * a.max_segs * a.H + h) * per_head + idx;
  const float* d0 = a.seg_decay + (size_t)b * a.max_segs * a.H * a.d + h * a.d + r;     // a decay per key channel only
  for (int s0 = 0; s0 < nsegs; s0 += 8) {        // eight segments' loads in flight, then the chain
    float left[8], pp[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool more = s0 + j + 1 < nsegs;
      left[j] = more ? p0[(size_t)(s0 + j) * seg_stride] : 0.f;
      pp[j] = !more ? 0.f : MODE != MODE_DECAY ? d0[(size_t)(s0 + j) * a.H * a.d] : p_const;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (s0 + j < nsegs) {
        p0[(size_t)(s0 + j) * seg_stride] = s;
        if (s0 + j + 1 < nsegs) s = fmaf(pp[j], s, left[j]);
      }
    }
  }
}

// ------------------------------------------------------------------- token shift
// A CTA per token. The CTA of a request's first token of the step is the only one that touches
// the request's state: each of its threads reads its columns of the previous h there and then
// writes the step's last h over them.
template <typename T>
__global__ void token_shift_mix_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ mu, int num_mixes,
                                       float* __restrict__ state, int state_stride, const int* __restrict__ cu_q,
                                       const int* __restrict__ state_slots, int num_seqs, int num_tokens, int C,
                                       T* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int lo = 0, hi = num_seqs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_q[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int start = cu_q[lo], end = cu_q[lo + 1];
  if (t >= end) return;                          // a row that belongs to no request
  float* st = state + (size_t)state_slots[lo] * state_stride;
  const T* cur_row = x + (size_t)t * x_stride;
  const T* last_row = x + (size_t)(end - 1) * x_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    const float cur = to_float(cur_row[c]);
    float prev;
    if (t > start) {
      prev = to_float(x[(size_t)(t - 1) * x_stride + c]);
    } else {
      prev = st[c];
      st[c] = to_float(last_row[c]);
    }
    const float diff = prev - cur;
    for (int m = 0; m < num_mixes; ++m)
      out[((size_t)m * num_tokens + t) * C + c] = from_float<T>(fmaf(diff, to_float(mu[(size_t)m * C + c]), cur));
  }
}

}  // namespace ts

using namespace ts;

template <typename K>
static int lin_allow_smem(K kern, size_t smem, size_t& allowed) {
  if (smem <= 48 * 1024 || smem <= allowed) return 0;
  const int e = (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == 0) allowed = smem;
  return e;
}

template <typename T, int MODE, int PASS>
static int launch_linear_pass(const LinScanArgs& a, dim3 grid, cudaStream_t stream) {
  const int dpad = a.W * LIN_RPT;
  const int narr = MODE == MODE_DECAY ? 2 : 3;
  const size_t smem = sizeof(float) * (2 * (size_t)a.CH * (narr * dpad + 32) + (size_t)a.CH * a.W * 32);
  static size_t allowed = 0;
  if constexpr (PASS == SCAN_WHOLE) {
    auto kern = linear_scan_kernel<T, MODE>;
    if (int e = lin_allow_smem(kern, smem, allowed)) return e;
    return launch(kern, grid, (a.W + a.loader_warps) * 32, smem, stream, a);
  } else {
    auto kern = linear_scan_segment_kernel<T, MODE, PASS>;
    if (int e = lin_allow_smem(kern, smem, allowed)) return e;
    return launch(kern, grid, (a.W + a.loader_warps) * 32, smem, stream, a);
  }
}

template <typename T, int MODE>
static int launch_linear(const LinScanArgs& a, int num_seqs, cudaStream_t stream) {
  const int col_blocks = (a.dv + 31) / 32;
  if (a.max_segs <= 1) return launch_linear_pass<T, MODE, SCAN_WHOLE>(a, dim3(num_seqs, a.H, col_blocks), stream);
  const dim3 grid(num_seqs * a.max_segs, a.H, col_blocks);
  if (MODE != MODE_DECAY)
    if (int e = launch(linear_scan_seg_decay_kernel<MODE>, dim3(num_seqs * a.max_segs, (a.H * a.d + 127) / 128), 128, 0, stream, a)) return e;
  if (int e = launch_linear_pass<T, MODE, SCAN_LOCAL>(a, grid, stream)) return e;
  if (int e = launch(linear_scan_combine_kernel<MODE>, dim3(num_seqs, a.H, (a.d * a.dv + 255) / 256), 256, 0, stream, a)) return e;
  return launch_linear_pass<T, MODE, SCAN_FINAL>(a, grid, stream);
}

// mode 0: bonus read-out with a decay per key channel and token; mode 1: constant decay per head, SiLU on q, k, v;
// mode 2: decay sigmoid(w_pre + w_bias)^(inv_tau) per key channel and token, q times q_scale, read-out after the write.
// max_segs > 1 cuts every request's tokens into segments of seg_len (max_segs * seg_len covers the longest) that
// run side by side (max_query_len = the most tokens any request brings): seg_state [num_seqs * max_segs, heads * d * dv] and, for modes 0 and 2, seg_decay
// [num_seqs * max_segs, heads * d] are scratch.
extern "C" int ts_linear_scan(int mode, const void* q, int q_stride, const void* k, int k_stride, const void* v,
                              int v_stride, const float* w_pre, int w_stride, const float* w_bias, const float* bonus,
                              const float* decay, float* state, int state_stride, const int* cu_q,
                              const int* state_slots, int num_seqs, int heads, int d, int dv, float* out, int dtype,
                              int max_query_len, int seg_len, int max_segs, float* seg_state, float* seg_decay,
                              float inv_tau, float q_scale, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (d <= 0 || dv <= 0 || d > LIN_MAX_KEY_DIM) return TS_ERR_UNSUPPORTED;
  if (mode == MODE_BONUS ? (!w_pre || !w_bias || !bonus) : mode == MODE_GATED ? (!w_pre || !w_bias || !(inv_tau > 0.f))
                                                             : (mode != MODE_DECAY || !decay)) return TS_ERR_BAD_ARGUMENT;
  if (dtype != TS_DTYPE_F32 && dtype != TS_DTYPE_BF16) return TS_ERR_BAD_ARGUMENT;
  if (max_segs > 1 && (seg_len <= 0 || !seg_state || (mode != MODE_DECAY && !seg_decay))) return TS_ERR_BAD_ARGUMENT;
  LinScanArgs a;
  a.q = q; a.q_stride = q_stride; a.k = k; a.k_stride = k_stride; a.v = v; a.v_stride = v_stride;
  a.w_pre = w_pre; a.w_stride = w_stride; a.w_bias = w_bias; a.bonus = bonus; a.decay = decay;
  a.state = state; a.state_stride = state_stride; a.cu_q = cu_q; a.state_slots = state_slots;
  a.H = heads; a.d = d; a.dv = dv; a.out = out; a.inv_tau = inv_tau; a.q_scale = q_scale;
  a.W = (d + LIN_RPT - 1) / LIN_RPT;
  a.CH = a.W * LIN_RPT <= 128 ? 16 : 8;
  a.loader_warps = (max_query_len > 0 && max_query_len <= a.CH) ? 0 : LIN_LOADER_WARPS;
  a.seg_len = seg_len; a.max_segs = max_segs > 1 ? max_segs : 1; a.seg_state = seg_state; a.seg_decay = seg_decay;
  if (mode == MODE_BONUS)
    return dtype == TS_DTYPE_F32 ? launch_linear<float, MODE_BONUS>(a, num_seqs, stream) : launch_linear<bf16, MODE_BONUS>(a, num_seqs, stream);
  if (mode == MODE_GATED)
    return dtype == TS_DTYPE_F32 ? launch_linear<float, MODE_GATED>(a, num_seqs, stream) : launch_linear<bf16, MODE_GATED>(a, num_seqs, stream);
  return dtype == TS_DTYPE_F32 ? launch_linear<float, MODE_DECAY>(a, num_seqs, stream) : launch_linear<bf16, MODE_DECAY>(a, num_seqs, stream);
}

extern "C" int ts_token_shift_mix(const void* x, int x_stride, const void* mu, int num_mixes, float* state,
                                  int state_stride, const int* cu_q, const int* state_slots, int num_seqs,
                                  int num_tokens, int channels, void* out, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0 || num_seqs <= 0) return 0;
  if (num_mixes <= 0 || channels <= 0) return TS_ERR_BAD_ARGUMENT;
  const int threads = 128;
  int by = (channels + threads - 1) / threads;
  if (by > 64) by = 64;
  dim3 grid(num_tokens, by);
  if (dtype == TS_DTYPE_F32)
    return launch(token_shift_mix_kernel<float>, grid, threads, 0, stream, (const float*)x, x_stride, (const float*)mu,
                  num_mixes, state, state_stride, cu_q, state_slots, num_seqs, num_tokens, channels, (float*)out);
  if (dtype == TS_DTYPE_BF16)
    return launch(token_shift_mix_kernel<bf16>, grid, threads, 0, stream, (const bf16*)x, x_stride, (const bf16*)mu,
                  num_mixes, state, state_stride, cu_q, state_slots, num_seqs, num_tokens, channels, (bf16*)out);
  return TS_ERR_BAD_ARGUMENT;
}
