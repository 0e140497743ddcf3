// A routed mixture of gated feed-forward experts, without a trip to the host:
//
//   route    a warp per token picks the `top` largest of its E router logits (32-bit; ties go to
//            the lower index), soft-maxes the picked logits alone, and takes a place in each picked
//            expert's queue (an atomic counter per expert). A second rule (RouteRule::scored) soft-maxes
//            ALL outputs first, picks by score + correction inside the best groups of neighbouring
//            outputs only, and weights the picks by their scores over the picks' sum, times a constant;
//            the last outputs may be identity experts, which have no matrices and no queue: their
//            picks carry the token's own input to the combine step;
//   plan     one thread turns the counters into the experts' row ranges of the sorted order and
//            into a list of row tiles (expert, first row), and clears the counters for the next step;
//   scatter  every (token, pick) learns its row of the sorted order; the row learns its token;
//   products tile by tile over that list: act[row, :] = silu(x[token] Wgate_e^T) * (x[token] Wup_e^T)
//            (the token's row of x is fetched through the list, nothing is copied), then
//            y[row, :] = act[row, :] Wdown_e^T;
//   combine  out[token] = sum_j weight_j y[row_j] (+ the shared expert's output, optionally times the sigmoid
//            of a gate logit per token), 32-bit, rounded once; an identity pick's y is the token's input.
//
// A row's sums run over K in index order whatever its tile holds, so a token's result does not
// depend on which other tokens share the step or on the order in which the queue places were taken.
// Two forms of the products: CUDA cores (float, and bf16 sizes the other form does not take), and
// mma.sync tensor-core tiles for bf16 with cp.async staging.
#define TS_PDL_CLASS PDL_OTHER
#include "common.cuh"

namespace ts {

// ------------------------------------------------------------------------- route
// One token by one warp: picks, weights, and a place in each picked expert's queue (`counts` may be
// in shared memory).
// How a token's picks and weights follow from its router outputs.
struct RouteRule {
  int scored;               // 0: the largest logits, weighted by the softmax over the picks alone
                            // 1: softmax over all outputs; picks by score + correction within the best groups;
                            //    weights = scores of the picks / (their sum + 1e-20) * scale
  int real;                 // outputs that are experts with matrices (the first ones); the rest are identity experts
  int groups, keep;         // scored: equal groups of neighbouring outputs, of which the `keep` best may be picked from
  float scale;              // scored: constant on the weights
  const float* correction;  // scored: [E] added to the scores for the choice only, or null
  int ld;                   // floats between two tokens' rows of router outputs
};

// One token by one warp: picks, weights, and a place in each picked expert's queue (`counts` may be
// in shared memory). A pick of an identity expert (id >= rule.real) takes no place (-1).
__device__ __forceinline__ void route_token(const float* __restrict__ z, int t, int lane, int E, int top, int* __restrict__ ids,
                                            float* __restrict__ weights, int* __restrict__ place, int* counts,
                                            const RouteRule& rule) {
  float zmax = 0.f, inv_sum = 1.f;
  unsigned allowed = 0xffffffffu;          // bit g: group g may be picked from
  int group_size = E;
  if (rule.scored) {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    zmax = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(z[e] - zmax);
    inv_sum = 1.f / warp_sum(sum);
    if (rule.groups > 1) {
      // lane g: the best choice score of group g, then its rank among the groups (value down, index up)
      group_size = E / rule.groups;
      float best = -INFINITY;
      if (lane < rule.groups)
        for (int e = lane * group_size; e < (lane + 1) * group_size; ++e)
          best = fmaxf(best, expf(z[e] - zmax) * inv_sum + (rule.correction ? rule.correction[e] : 0.f));
      int rank = 0;
      for (int g = 0; g < rule.groups; ++g) {
        const float other = __shfl_sync(0xffffffffu, best, g);
        rank += (other > best || (other == best && g < lane)) ? 1 : 0;
      }
      allowed = __ballot_sync(0xffffffffu, lane < rule.groups && rank < rule.keep);
    }
  }
  float prev_v = INFINITY, my_v = -INFINITY;
  int prev_e = -1, my_e = -1;
  for (int j = 0; j < top; ++j) {
    // the largest element that comes after the pick before in the order (value down, index up)
    float bv = -INFINITY;
    int be = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      float v = z[e];
      if (rule.scored) {
        v = expf(v - zmax) * inv_sum + (rule.correction ? rule.correction[e] : 0.f);
        if (!((allowed >> (e / group_size)) & 1u)) continue;
      }
      const bool after = (v < prev_v) || (v == prev_v && e > prev_e);
      if (after && (v > bv || (v == bv && e < be))) { bv = v; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
    }
    if (lane == j) { my_v = bv; my_e = be; }
    prev_v = bv;
    prev_e = be;
  }
  const bool picked = lane < top && my_e >= 0 && my_e < E;   // fewer finite candidates than picks: the pick is dropped
  float p;
  if (rule.scored) {
    p = picked ? expf(z[my_e] - zmax) * inv_sum : 0.f;        // the score itself, without the correction
  } else {
    const float head = __shfl_sync(0xffffffffu, my_v, 0);
    p = lane < top ? expf(my_v - head) : 0.f;
  }
  const float sum = warp_sum(p);
  if (lane < top) {
    const int e = picked ? my_e : 0;
    const float w = rule.scored ? p / (sum + 1e-20f) * rule.scale : p / sum;
    ids[(size_t)t * top + lane] = e;
    weights[(size_t)t * top + lane] = picked ? w : 0.f;
    place[(size_t)t * top + lane] = e < rule.real ? atomicAdd(&counts[e], 1) : -1;
  }
}

__global__ void moe_route_kernel(const float* __restrict__ logits, int num_tokens, int E, int top, int* __restrict__ ids,
                                 float* __restrict__ weights, int* __restrict__ place, int* __restrict__ counts, RouteRule rule) {
  pdl_trigger();
  pdl_wait();
  const int t = (int)(((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (t >= num_tokens) return;
  route_token(logits + (size_t)t * rule.ld, t, lane, E, top, ids, weights, place, counts, rule);
}

// A step of few tokens (decoding): route, plan and scatter by ONE CTA, the queue counters in shared
// memory, so that the three launches become one.
constexpr int ROUTE_SMALL_THREADS = 512, ROUTE_SMALL_MAX_EXPERTS = 1024;
// With `x` (and the router's matrix `w`, both of type T) the CTA first forms the router logits itself,
// logits[t, e] = x[t] . w[e] with 32-bit sums, so that the router's product is no launch of its own either.
template <typename T>
__global__ void __launch_bounds__(ROUTE_SMALL_THREADS) moe_route_small_kernel(
    const T* __restrict__ x, const T* __restrict__ w, int hidden,
    float* logits, int num_tokens, int E, int top, int tile_rows, int* __restrict__ ids,
    float* __restrict__ weights, int* __restrict__ place, int* __restrict__ offsets, int* __restrict__ tile_expert,
    int* __restrict__ tile_row0, int* __restrict__ num_tiles, int max_tiles, int* __restrict__ row_of,
    int* __restrict__ token_of, RouteRule rule) {
  __shared__ int counts[ROUTE_SMALL_MAX_EXPERTS];
  __shared__ int offs[ROUTE_SMALL_MAX_EXPERTS + 1];
  pdl_trigger();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (x != nullptr) {
    constexpr int VEC = Vec<T>::N;
    const bool wide = hidden % VEC == 0 && ((((uintptr_t)x) | ((uintptr_t)w)) & 15) == 0;
    for (int pair = warp; pair < num_tokens * E; pair += warps) {
      const int t = pair / E, e = pair - t * E;
      const T* xr = x + (size_t)t * hidden;
      const T* wr = w + (size_t)e * hidden;
      float sum = 0.f;
      if (wide) {
        for (int i = lane * VEC; i < hidden; i += 32 * VEC) {
          Vec<T> a, b;
          a.load(xr + i);
          b.load(wr + i);
          float fa[VEC], fb[VEC];
          a.unpack(fa);
          b.unpack(fb);
#pragma unroll
          for (int q = 0; q < VEC; ++q) sum = fmaf(fa[q], fb[q], sum);
        }
      } else {
        for (int i = lane; i < hidden; i += 32) sum = fmaf(to_float(xr[i]), to_float(wr[i]), sum);
      }
      sum = warp_sum(sum);
      if (lane == 0) logits[(size_t)t * rule.ld + e] = sum;
    }
  }
  __syncthreads();
  for (int t = warp; t < num_tokens; t += warps)
    route_token(logits + (size_t)t * rule.ld, t, lane, E, top, ids, weights, place, counts, rule);
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, nt = 0;
    for (int e = 0; e < rule.real; ++e) {
      const int c = counts[e];
      offs[e] = off;
      offsets[e] = off;
      for (int r = 0; r < c && nt < max_tiles; r += tile_rows) {
        tile_expert[nt] = e;
        tile_row0[nt] = off + r;
        ++nt;
      }
      off += c;
    }
    offsets[rule.real] = off;
    *num_tiles = nt;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < num_tokens * top; idx += blockDim.x) {
    if (place[idx] < 0) {              // an identity pick: no row of the sorted order
      row_of[idx] = -1;
      continue;
    }
    const int row = offs[ids[idx]] + place[idx];
    row_of[idx] = row;
    token_of[row] = idx / top;
  }
}

// -------------------------------------------------------------------------- plan
__global__ void moe_plan_kernel(int* __restrict__ counts, int E, int tile_rows, int* __restrict__ offsets,
                                int* __restrict__ tile_expert, int* __restrict__ tile_row0, int* __restrict__ num_tiles,
                                int max_tiles) {
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int off = 0, nt = 0;
  for (int e = 0; e < E; ++e) {
    const int c = counts[e];
    offsets[e] = off;
    for (int r = 0; r < c && nt < max_tiles; r += tile_rows) {
      tile_expert[nt] = e;
      tile_row0[nt] = off + r;
      ++nt;
    }
    off += c;
    counts[e] = 0;
  }
  offsets[E] = off;
  *num_tiles = nt;
}

// ----------------------------------------------------------------------- scatter
__global__ void moe_scatter_kernel(const int* __restrict__ ids, const int* __restrict__ place, const int* __restrict__ offsets,
                                   int total, int top, int* __restrict__ row_of, int* __restrict__ token_of) {
  pdl_trigger();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  if (place[idx] < 0) {                // an identity pick: no row of the sorted order
    row_of[idx] = -1;
    return;
  }
  const int row = offsets[ids[idx]] + place[idx];
  row_of[idx] = row;
  token_of[row] = idx / top;
}

// --------------------------------------------------------- products, CUDA cores
constexpr int SG_M = 64, SG_N = 64, SG_K = 16, SG_THREADS = 256;

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

// GATED: w holds, per expert, N gate rows then N up rows; out[row, n] = silu(g) * u.
template <typename T, bool GATED>
__global__ void __launch_bounds__(SG_THREADS) moe_gemm_simt_kernel(
    const T* __restrict__ x, const int* __restrict__ token_of, const T* __restrict__ w, T* __restrict__ out,
    const int* __restrict__ offsets, const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
    const int* __restrict__ num_tiles, int N, int K) {
  __shared__ float As[SG_K][SG_M + 4];
  __shared__ float Bs[GATED ? 2 : 1][SG_K][SG_N + 4];
  pdl_trigger();
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= *(const volatile int*)num_tiles) return;      // volatile: never read in front of the wait
  const int e = tile_expert[tile], r0 = tile_row0[tile], rend = offsets[e + 1];
  const int n0 = blockIdx.x * SG_N;
  const T* we = w + (size_t)e * (GATED ? 2 : 1) * N * K;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  const int am = r0 + lrow;
  const long long arow = am < rend ? (token_of ? token_of[am] : am) : -1;
  float acc[GATED ? 2 : 1][4][4];
#pragma unroll
  for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[g][i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += SG_K) {
    float av[4], bv[GATED ? 2 : 1][4];
    const int bn = n0 + lrow;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int k = k0 + lk + q;
      av[q] = (arow >= 0 && k < K) ? to_float(x[(size_t)arow * K + k]) : 0.f;
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g)
        bv[g][q] = (bn < N && k < K) ? to_float(we[((size_t)g * N + bn) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      As[lk + q][lrow] = av[q];
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g) Bs[g][lk + q][lrow] = bv[g][q];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < SG_K; ++k) {
      float a[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g) {
        float b[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Bs[g][k][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[g][i][j] = fmaf(a[i], b[j], acc[g][i][j]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = r0 + ty * 4 + i;
    if (m >= rend) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[0][i][j];
      if (GATED) v = silu_f(v) * acc[1][i][j];
      out[(size_t)m * N + n] = from_float<T>(v);
    }
  }
}

// ------------------------------------------------------- products, tensor cores
// bf16, K % 64 == 0, N % 8 == 0. A CTA of four warps takes a tile of 64 rows x 64 output columns
// (gated: 64 gate and 64 up columns); a warp 16 rows of it. Operands come through shared memory in
// steps of 64 along K, four steps in flight (cp.async, 16 bytes a request; rows of 144 bytes keep
// the ldmatrix reads free of bank conflicts): two CTAs an SM keep some 150 KB of requests in flight,
// which is what streaming the experts' matrices at the memory's rate takes when a step has few rows.
constexpr int TG_M = 64, TG_N = 64, TG_K = 64, TG_STAGES = 4, TG_THREADS = 128, TG_LD = TG_K + 8;
constexpr int TG_CH = TG_K / 8;      // 16-byte pieces of a row of a stage

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool GATED>
__global__ void __launch_bounds__(TG_THREADS) moe_gemm_mma_kernel(
    const bf16* __restrict__ x, const int* __restrict__ token_of, const bf16* __restrict__ w, bf16* __restrict__ out,
    const int* __restrict__ offsets, const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
    const int* __restrict__ num_tiles, int N, int K) {
  constexpr int NB = GATED ? 2 : 1;
  extern __shared__ __align__(16) unsigned char raw[];
  bf16* As = (bf16*)raw;                                   // [STAGES][TG_M][TG_LD]
  bf16* Bs = As + (size_t)TG_STAGES * TG_M * TG_LD;        // [STAGES][NB][TG_N][TG_LD]
  __shared__ long long a_rows[TG_M];
  pdl_trigger();
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= *(const volatile int*)num_tiles) return;      // volatile: never read in front of the wait
  const int e = tile_expert[tile], r0 = tile_row0[tile], rend = offsets[e + 1];
  const int n0 = blockIdx.x * TG_N;
  const bf16* we = w + (size_t)e * NB * N * K;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < TG_M) {
    const int m = r0 + tid;
    a_rows[tid] = m < rend ? (long long)(token_of ? token_of[m] : m) : -1;
  }
  __syncthreads();

  auto stage_load = [&](int stage, int k0) {
    // A: 64 rows x TG_CH pieces of 8 elements; B: NB x 64 rows x TG_CH pieces
    for (int c = tid; c < TG_M * TG_CH; c += TG_THREADS) {
      const int r = c / TG_CH, ch = c - r * TG_CH;
      const long long ar = a_rows[r];
      const bf16* src = x + (size_t)(ar < 0 ? 0 : ar) * K + k0 + ch * 8;
      cp_async16(As + ((size_t)stage * TG_M + r) * TG_LD + ch * 8, src, ar >= 0);
    }
    for (int c = tid; c < NB * TG_N * TG_CH; c += TG_THREADS) {
      const int g = c / (TG_N * TG_CH), rest = c - g * (TG_N * TG_CH);
      const int r = rest / TG_CH, ch = rest - r * TG_CH;
      const int n = n0 + r;
      const bf16* src = we + ((size_t)g * N + (n < N ? n : 0)) * K + k0 + ch * 8;
      cp_async16(Bs + (((size_t)stage * NB + g) * TG_N + r) * TG_LD + ch * 8, src, n < N);
    }
  };

  float acc[NB][8][4];
#pragma unroll
  for (int g = 0; g < NB; ++g)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[g][j][q] = 0.f;

  const int steps = K / TG_K;
#pragma unroll
  for (int s = 0; s < TG_STAGES - 1; ++s) {
    if (s < steps) stage_load(s, s * TG_K);
    cp_async_commit();
  }
  for (int it = 0; it < steps; ++it) {
    cp_async_wait<TG_STAGES - 2>();
    __syncthreads();
    const int nxt = it + TG_STAGES - 1;
    if (nxt < steps) stage_load(nxt % TG_STAGES, nxt * TG_K);
    cp_async_commit();
    const int stage = it % TG_STAGES;
    const bf16* Asb = As + ((size_t)stage * TG_M + warp * 16) * TG_LD;
#pragma unroll
    for (int kk = 0; kk < TG_K; kk += 16) {
      uint32_t afr[4];
      // rows lane % 16, k half lane / 16
      ldmatrix_x4(afr, Asb + (size_t)(lane & 15) * TG_LD + kk + (lane >> 4) * 8);
#pragma unroll
      for (int g = 0; g < NB; ++g) {
        const bf16* Bsb = Bs + ((size_t)stage * NB + g) * TG_N * TG_LD;
#pragma unroll
        for (int jp = 0; jp < 4; ++jp) {
          // two n-blocks of 8 at once: matrices (n0..7, k lo), (n0..7, k hi), (n8..15, k lo), (n8..15, k hi)
          uint32_t bfr[4];
          const int nrow = jp * 16 + (lane & 7) + ((lane >> 4) << 3);
          const int kcol = kk + ((lane >> 3) & 1) * 8;
          ldmatrix_x4(bfr, Bsb + (size_t)nrow * TG_LD + kcol);
          mma_bf16(acc[g][jp * 2], afr, bfr[0], bfr[1]);
          mma_bf16(acc[g][jp * 2 + 1], afr, bfr[2], bfr[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
  // accumulator layout: rows lane / 4 and + 8, columns (lane % 4) * 2 and + 1 of each 8-wide block
  const int mrow = r0 + warp * 16 + (lane >> 2);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int n = n0 + j * 8 + (lane & 3) * 2;
    if (n >= N) continue;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = mrow + half * 8;
      if (m >= rend) continue;
      float v0 = acc[0][j][half * 2], v1 = acc[0][j][half * 2 + 1];
      if (GATED) { v0 = silu_f(v0) * acc[NB - 1][j][half * 2]; v1 = silu_f(v1) * acc[NB - 1][j][half * 2 + 1]; }
      const __nv_bfloat162 pk = __floats2bfloat162_rn(v0, v1);
      *reinterpret_cast<__nv_bfloat162*>(out + (size_t)m * N + n) = pk;
    }
  }
}

// ------------------------------------------------------------------------ gather
// xs[row, :] = x[token_of[row], :] in pieces of 16 bytes (for the product that takes its rows in the sorted order).
// Only the first *total_rows rows of the sorted order exist (picks of identity experts take none): the rows behind
// them are zero-filled, and token_of is not read there.
// (*total_rows is written two kernels back in the chain. It is read through a volatile pointer: a plain read of a
// const __restrict__ pointer may be moved in front of the wait by the compiler, where a kernel that started early
// sees the value of the step before.)
__global__ void moe_gather_kernel(const uint4* __restrict__ x, const int* __restrict__ token_of, uint4* __restrict__ xs,
                                  int picks, int pieces, const int* total_rows) {
  pdl_trigger();
  pdl_wait();
  const size_t live = (size_t)min(*(const volatile int*)total_rows, picks);
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < (size_t)picks * pieces; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t row = idx / pieces;
    xs[idx] = row < live ? x[(size_t)token_of[row] * pieces + (idx - row * pieces)] : make_uint4(0u, 0u, 0u, 0u);
  }
}

// ----------------------------------------------------------------------- combine
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ row_of, const float* __restrict__ weights,
                                   const T* __restrict__ shared_out, T* __restrict__ out, int top, int hidden,
                                   const T* __restrict__ x, const float* __restrict__ shared_gate, int gate_stride) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  // volatile: this read stands right behind the wait and depends on nothing, so as a plain read it could be moved in front of it
  const float sg = shared_gate ? 1.f / (1.f + expf(-*(const volatile float*)(shared_gate + (size_t)t * gate_stride))) : 1.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = 0.f;
    for (int j = 0; j < top; ++j) {
      const int row = row_of[(size_t)t * top + j];
      v = fmaf(weights[(size_t)t * top + j], to_float(row >= 0 ? y[(size_t)row * hidden + c] : x[(size_t)t * hidden + c]), v);
    }
    if (shared_out) v = fmaf(sg, to_float(shared_out[(size_t)t * hidden + c]), v);
    out[(size_t)t * hidden + c] = from_float<T>(v);
  }
}

// The same with 16-byte accesses (hidden a multiple of the vector length, aligned rows): the picks' rows
// are asked for together, up to eight at a time.
template <typename T>
__global__ void moe_combine_vec_kernel(const T* __restrict__ y, const int* __restrict__ row_of, const float* __restrict__ weights,
                                       const T* __restrict__ shared_out, T* __restrict__ out, int top, int hidden,
                                       const T* __restrict__ x, const float* __restrict__ shared_gate, int gate_stride) {
  constexpr int VEC = Vec<T>::N;
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  // volatile: this read stands right behind the wait and depends on nothing, so as a plain read it could be moved in front of it
  const float sg = shared_gate ? 1.f / (1.f + expf(-*(const volatile float*)(shared_gate + (size_t)t * gate_stride))) : 1.f;
  const int* rows = row_of + (size_t)t * top;
  const float* wt = weights + (size_t)t * top;
  for (int c = threadIdx.x * VEC; c < hidden; c += blockDim.x * VEC) {
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
    for (int j0 = 0; j0 < top; j0 += 8) {
      Vec<T> part[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (j0 + u < top) part[u].load(rows[j0 + u] >= 0 ? y + (size_t)rows[j0 + u] * hidden + c : x + (size_t)t * hidden + c);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (j0 + u < top) {
          float f[VEC];
          part[u].unpack(f);
          const float a = wt[j0 + u];
#pragma unroll
          for (int e = 0; e < VEC; ++e) acc[e] = fmaf(a, f[e], acc[e]);
        }
    }
    if (shared_out) {
      Vec<T> sv;
      sv.load(shared_out + (size_t)t * hidden + c);
      float f[VEC];
      sv.unpack(f);
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = fmaf(sg, f[e], acc[e]);
    }
    Vec<T> ov;
    ov.pack(acc);
    ov.store(out + (size_t)t * hidden + c);
  }
}

}  // namespace ts

using namespace ts;

extern "C" int ts_moe_tile_rows() { return SG_M; }      // both product forms use tiles of 64 rows

// The rule's arguments, checked: E outputs of which the first `real` are experts with matrices.
static int make_rule(RouteRule& r, int E, int real, int top, int scored, int groups, int keep, float scale,
                     const float* correction, int ld) {
  if (E <= 0 || real <= 0 || real > E || top <= 0 || top > 32 || top > E || ld < E) return TS_ERR_BAD_ARGUMENT;
  if (!scored && (real != E || groups > 1 || correction)) return TS_ERR_BAD_ARGUMENT;
  if (groups < 1) groups = 1;
  if (groups > 32 || E % groups || keep < 1 || keep > groups || (E / groups) * keep < top) return TS_ERR_BAD_ARGUMENT;
  r.scored = scored; r.real = real; r.groups = groups; r.keep = keep; r.scale = scale; r.correction = correction; r.ld = ld;
  return 0;
}

// logits [T, ld >= E] float -> ids / weights / place [T, top]; counts [real] (zero on entry, zero again after the plan);
// offsets [real + 1]; tile_expert / tile_row0 [max_tiles]; num_tiles [1]; row_of [T * top]; token_of [T * top].
// tile_rows: rows of a tile of the list (64 for the products of this file, 128 for the tcgen05 product).
// scored / groups / keep / scale / correction / real: see RouteRule (scored 0 wants real = E, groups <= 1).
extern "C" int ts_moe_route(const float* logits, int ld, int num_tokens, int E, int real, int top, int scored, int groups,
                            int keep, float scale, const float* correction, int* ids, float* weights, int* place,
                            int* counts, int* offsets, int* tile_expert, int* tile_row0, int* num_tiles, int max_tiles,
                            int* row_of, int* token_of, int tile_rows, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (tile_rows != 64 && tile_rows != 128) return TS_ERR_BAD_ARGUMENT;
  RouteRule rule;
  if (int e = make_rule(rule, E, real, top, scored, groups, keep, scale, correction, ld)) return e;
  const int picks = num_tokens * top;
  const int most = picks < picks / tile_rows + real ? picks : picks / tile_rows + real;   // every tile has a row; an expert one ragged tile
  if (max_tiles < most) return TS_ERR_BAD_ARGUMENT;
  if (num_tokens <= 64 && E <= ROUTE_SMALL_MAX_EXPERTS)
    return launch(moe_route_small_kernel<float>, 1, ROUTE_SMALL_THREADS, 0, stream, (const float*)nullptr, (const float*)nullptr, 0,
                  const_cast<float*>(logits), num_tokens, E, top, tile_rows, ids, weights, place, offsets, tile_expert, tile_row0,
                  num_tiles, max_tiles, row_of, token_of, rule);
  int st = launch(moe_route_kernel, (num_tokens * 32 + 127) / 128, 128, 0, stream, logits, num_tokens, E, top, ids,
                  weights, place, counts, rule);
  if (st != 0) return st;
  st = launch(moe_plan_kernel, 1, 32, 0, stream, counts, real, tile_rows, offsets, tile_expert, tile_row0, num_tiles, max_tiles);
  if (st != 0) return st;
  const int total = num_tokens * top;
  return launch(moe_scatter_kernel, (total + 255) / 256, 256, 0, stream, (const int*)ids, (const int*)place,
                (const int*)offsets, total, top, row_of, token_of);
}

// The same for a step of up to 64 tokens with the router's product inside: logits (scratch, [T, E] float) are
// formed from x [T, hidden] and w_router [E, hidden] of `dtype` by the one CTA that routes (the plain rule only).
extern "C" int ts_moe_route_fused(const void* x, const void* w_router, int hidden, int dtype, float* logits, int num_tokens,
                                  int E, int top, int* ids, float* weights, int* place, int* offsets, int* tile_expert,
                                  int* tile_row0, int* num_tiles, int max_tiles, int* row_of, int* token_of, int tile_rows,
                                  cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (tile_rows != 64 && tile_rows != 128) return TS_ERR_BAD_ARGUMENT;
  RouteRule rule;
  if (int e = make_rule(rule, E, E, top, 0, 1, 1, 1.f, nullptr, E)) return e;
  const int picks = num_tokens * top;
  const int most = picks < picks / tile_rows + E ? picks : picks / tile_rows + E;
  if (max_tiles < most || hidden <= 0 || !x || !w_router) return TS_ERR_BAD_ARGUMENT;
  if (num_tokens > 64 || E > ROUTE_SMALL_MAX_EXPERTS) return TS_ERR_UNSUPPORTED;
  if (dtype == TS_DTYPE_F32)
    return launch(moe_route_small_kernel<float>, 1, ROUTE_SMALL_THREADS, 0, stream, (const float*)x, (const float*)w_router, hidden,
                  logits, num_tokens, E, top, tile_rows, ids, weights, place, offsets, tile_expert, tile_row0, num_tiles, max_tiles,
                  row_of, token_of, rule);
  if (dtype == TS_DTYPE_BF16)
    return launch(moe_route_small_kernel<bf16>, 1, ROUTE_SMALL_THREADS, 0, stream, (const bf16*)x, (const bf16*)w_router, hidden,
                  logits, num_tokens, E, top, tile_rows, ids, weights, place, offsets, tile_expert, tile_row0, num_tiles, max_tiles,
                  row_of, token_of, rule);
  return TS_ERR_BAD_ARGUMENT;
}

// out[row, :] for every row of the sorted order: x rows are taken through `token_of` when it is
// given (else row by row). w is [E, N (gated: 2 N), K]. `use_mma` 0 forces the CUDA-core form.
extern "C" int ts_moe_gemm(const void* x, const int* token_of, const void* w, void* out, const int* offsets,
                           const int* tile_expert, const int* tile_row0, const int* num_tiles, int max_tiles, int N,
                           int K, int gated, int dtype, int use_mma, cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  if (N <= 0 || K <= 0) return TS_ERR_BAD_ARGUMENT;
  if (dtype == TS_DTYPE_BF16 && use_mma && K % TG_K == 0 && N % 8 == 0 &&
      (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) == 0) {
    const int nb = gated ? 2 : 1;
    const size_t smem = sizeof(bf16) * (size_t)TG_STAGES * (TG_M + nb * TG_N) * TG_LD;
    dim3 grid((N + TG_N - 1) / TG_N, max_tiles);
    if (gated) {
      auto kern = moe_gemm_mma_kernel<true>;
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      return launch(kern, grid, TG_THREADS, smem, stream, (const bf16*)x, token_of, (const bf16*)w, (bf16*)out, offsets,
                    tile_expert, tile_row0, num_tiles, N, K);
    }
    auto kern = moe_gemm_mma_kernel<false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return launch(kern, grid, TG_THREADS, smem, stream, (const bf16*)x, token_of, (const bf16*)w, (bf16*)out, offsets,
                  tile_expert, tile_row0, num_tiles, N, K);
  }
  dim3 grid((N + SG_N - 1) / SG_N, max_tiles);
#define TS_MOE_CASE(T_, G_)                                                                                     \
  return launch(moe_gemm_simt_kernel<T_, G_>, grid, SG_THREADS, 0, stream, (const T_*)x, token_of, (const T_*)w, \
                (T_*)out, offsets, tile_expert, tile_row0, num_tiles, N, K)
  if (dtype == TS_DTYPE_F32) { if (gated) TS_MOE_CASE(float, true); TS_MOE_CASE(float, false); }
  if (dtype == TS_DTYPE_BF16) { if (gated) TS_MOE_CASE(bf16, true); TS_MOE_CASE(bf16, false); }
#undef TS_MOE_CASE
  return TS_ERR_BAD_ARGUMENT;
}

// total_rows: one int on the device, the rows of the sorted order that exist (offsets[experts] of the plan).
extern "C" int ts_moe_gather(const void* x, const int* token_of, void* xs, int picks, int row_bytes, const int* total_rows,
                             cudaStream_t stream) {
  if (picks <= 0) return 0;
  if (!total_rows) return TS_ERR_BAD_ARGUMENT;
  if (row_bytes <= 0 || row_bytes % 16 != 0 || (((uintptr_t)x | (uintptr_t)xs) & 15)) return TS_ERR_UNSUPPORTED;
  const int pieces = row_bytes / 16;
  size_t blocks = ((size_t)picks * pieces + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch(moe_gather_kernel, (int)blocks, 256, 0, stream, (const uint4*)x, token_of, (uint4*)xs, picks, pieces, total_rows);
}

// x [T, hidden] (the tokens' inputs) is read for identity picks (row_of < 0) and may be null when there are none;
// shared_gate (float, one logit per token, gate_stride floats apart) multiplies the shared output by its sigmoid.
extern "C" int ts_moe_combine(const void* y, const int* row_of, const float* weights, const void* shared_out, void* out,
                              int num_tokens, int top, int hidden, const void* x, const float* shared_gate, int gate_stride,
                              int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  const int vec = dtype == TS_DTYPE_F32 ? 4 : 8;
  if (hidden % vec == 0 && (((uintptr_t)y | (uintptr_t)shared_out | (uintptr_t)out | (uintptr_t)x) & 15) == 0) {
    int vthreads = 32;
    while (vthreads < 256 && vthreads * vec < hidden) vthreads <<= 1;
    if (dtype == TS_DTYPE_F32)
      return launch(moe_combine_vec_kernel<float>, num_tokens, vthreads, 0, stream, (const float*)y, row_of, weights,
                    (const float*)shared_out, (float*)out, top, hidden, (const float*)x, shared_gate, gate_stride);
    if (dtype == TS_DTYPE_BF16)
      return launch(moe_combine_vec_kernel<bf16>, num_tokens, vthreads, 0, stream, (const bf16*)y, row_of, weights,
                    (const bf16*)shared_out, (bf16*)out, top, hidden, (const bf16*)x, shared_gate, gate_stride);
    return TS_ERR_BAD_ARGUMENT;
  }
  if (dtype == TS_DTYPE_F32)
    return launch(moe_combine_kernel<float>, num_tokens, threads, 0, stream, (const float*)y, row_of, weights,
                  (const float*)shared_out, (float*)out, top, hidden, (const float*)x, shared_gate, gate_stride);
  if (dtype == TS_DTYPE_BF16)
    return launch(moe_combine_kernel<bf16>, num_tokens, threads, 0, stream, (const bf16*)y, row_of, weights,
                  (const bf16*)shared_out, (bf16*)out, top, hidden, (const bf16*)x, shared_gate, gate_stride);
  return TS_ERR_BAD_ARGUMENT;
}
