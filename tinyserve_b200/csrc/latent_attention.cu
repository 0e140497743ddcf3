// Attention over a cache of latent vectors: every token keeps ONE row of R + P elements, a normed
// latent vector c (R elements) from which all heads' keys and values derive, and a rotated key
// part (P elements) shared by the heads. With the keys' up-projection folded into the queries
// (q'_h = W_uk,h^T q_h) and the values' up-projection applied after the weighted sum, every head
// scores against the same row, score = q'_h . c + q_rot,h . k_rot, and sums the same c: the layer is
// attention with one shared key/value head whose values are the first R elements of its keys.
//
//  * ts_latent_prepare: per token, RMSNorm of the latent part (plain weight), rotation of the shared
//    key part, both written to the cache row of the token's slot; and the full query rows
//    [T, H, R + P] assembled from the folded queries [H, T, R] and the rotated query parts.
//  * ts_latent_attention: causal (optionally windowed) softmax attention of those query rows over
//    the cached rows, on CUDA cores in 32-bit, for float and bf16 storage. A CTA takes a few
//    tokens of one request and a few heads; every key tile it stages is shared by all its rows.
//    A warp owns a row at a time: each lane scores one key of the tile, then each lane owns
//    output columns. Rows of other requests or beyond a request's positions are never loaded.
#define TS_PDL_CLASS PDL_ATTENTION
#include "common.cuh"

namespace ts {

// ------------------------------------------------------------------------ prepare
struct LatentPrepArgs {
  const void* q_in;      // [T, q_stride]: per head `nope` unrotated then P rotated elements
  long long q_stride;
  const void* q_folded;  // [H, T, R]
  const void* ckr;       // [T, ckr_stride]: R latent elements, then P elements of the shared key part
  long long ckr_stride;
  const void* norm_weight;  // [R]
  float eps;
  const float* cos_t;    // [T, rotary_dim / 2]
  const float* sin_t;
  int rotary_dim, interleaved;
  const int* slots;      // [T] cache row of each token (null: nothing is written)
  void* cache;           // [rows, R + P]
  void* q_out;           // [T, H, R + P]
  int num_tokens, heads, nope, rank, rot;
};

// Rotation of element i of a vector of `rot` elements whose first `rotary_dim` turn.
template <typename T>
__device__ __forceinline__ float rotated(const T* v, int i, const float* c, const float* s, int rotary_dim, int interleaved) {
  if (i >= rotary_dim) return to_float(v[i]);
  const int half = rotary_dim >> 1;
  if (interleaved) {
    const int p = i >> 1;
    const float a = to_float(v[2 * p]), b = to_float(v[2 * p + 1]);
    return (i & 1) ? b * c[p] + a * s[p] : a * c[p] - b * s[p];
  }
  if (i < half) return to_float(v[i]) * c[i] - to_float(v[i + half]) * s[i];
  return to_float(v[i]) * c[i - half] + to_float(v[i - half]) * s[i - half];
}

template <typename T>
__global__ void latent_prepare_kernel(LatentPrepArgs a) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int D = a.rank + a.rot;
  const float* c = a.cos_t ? a.cos_t + (size_t)t * (a.rotary_dim >> 1) : nullptr;
  const float* s = a.sin_t ? a.sin_t + (size_t)t * (a.rotary_dim >> 1) : nullptr;
  const int rdim = c ? a.rotary_dim : 0;
  if (a.slots) {
    const T* row = (const T*)a.ckr + (size_t)t * a.ckr_stride;
    T* dst = (T*)a.cache + (size_t)a.slots[t] * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) {
      const float v = to_float(row[i]);
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)a.rank + a.eps);
    const T* w = (const T*)a.norm_weight;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) dst[i] = from_float<T>(to_float(row[i]) * rstd * to_float(w[i]));
    for (int i = threadIdx.x; i < a.rot; i += blockDim.x)
      dst[a.rank + i] = from_float<T>(rotated(row + a.rank, i, c, s, rdim, a.interleaved));
  }
  const T* qf = (const T*)a.q_folded;
  T* qo = (T*)a.q_out + (size_t)t * a.heads * D;
  for (int idx = threadIdx.x; idx < a.heads * a.rank; idx += blockDim.x) {
    const int h = idx / a.rank, i = idx - h * a.rank;
    qo[(size_t)h * D + i] = qf[((size_t)h * a.num_tokens + t) * a.rank + i];
  }
  const T* qi = (const T*)a.q_in + (size_t)t * a.q_stride;
  for (int idx = threadIdx.x; idx < a.heads * a.rot; idx += blockDim.x) {
    const int h = idx / a.rot, i = idx - h * a.rot;
    qo[(size_t)h * D + a.rank + i] =
        from_float<T>(rotated(qi + (size_t)h * (a.nope + a.rot) + a.nope, i, c, s, rdim, a.interleaved));
  }
}

// ---------------------------------------------------------------------- attention
struct LatentAttnArgs {
  const void* q;           // [T, H, D]
  void* out;               // [T, H, R]
  const void* cache;       // [pages * page_size, D]
  const int* block_tables; // [B, table_width]
  const int* cu_q;         // [B + 1]
  const int* ctx_lens;     // [B]
  int table_width, num_seqs, heads, rank, rot, page_size;
  float scale_log2;
  int window;              // 0: every earlier position
  const float* sinks;      // [H] or null: a logit per head (natural base, not scaled) that joins the softmax's
                           // denominator and has no value
  int tokens_per_cta, heads_per_cta;
};

constexpr int LA_WARPS = 8, LA_THREADS = LA_WARPS * 32, LA_TK = 32;
constexpr int LA_RPW = 4;          // rows a warp works on together

// RJ: output columns per lane (rank <= 32 * RJ).
template <typename T, int RJ>
__global__ void __launch_bounds__(LA_THREADS) latent_attention_kernel(LatentAttnArgs a) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int R = a.rank, D = a.rank + a.rot, DS = D + 1;
  const int rows_cta = a.tokens_per_cta * a.heads_per_cta;
  float* Qs = smem;                         // [rows_cta][D]  pre-scaled
  float* Ks = Qs + (size_t)rows_cta * D;    // [LA_TK][DS]
  const int seq = blockIdx.y;
  const int row0 = a.cu_q[seq];
  const int n = a.cu_q[seq + 1] - row0;
  const int t0 = blockIdx.x * a.tokens_per_cta;
  if (t0 >= n) return;
  const int nt = min(a.tokens_per_cta, n - t0);
  const int h0 = blockIdx.z * a.heads_per_cta;
  const int nh = min(a.heads_per_cta, a.heads - h0);
  const int ctx = a.ctx_lens[seq];
  const int first_pos = ctx - n;
  const int* table = a.block_tables + (size_t)seq * a.table_width;
  const T* q = (const T*)a.q;
  const T* cache = (const T*)a.cache;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nrows = nt * nh;                // row r -> token r / nh, head r % nh

  for (int idx = tid; idx < nrows * D; idx += LA_THREADS) {
    const int r = idx / D, d = idx - r * D;
    const int tt = r / nh, hh = r - tt * nh;
    Qs[(size_t)r * D + d] = to_float(q[((size_t)(row0 + t0 + tt) * a.heads + h0 + hh) * D + d]) * a.scale_log2;
  }
  const int qpos_first = first_pos + t0, qpos_last = first_pos + t0 + nt - 1;
  const int k_lo = a.window > 0 ? max(0, qpos_first - a.window + 1) : 0;
  const int k_begin = (k_lo / LA_TK) * LA_TK;

  // a warp's rows: warp, warp + LA_WARPS, ...  (at most LA_RPW of them a pass)
  for (int pass0 = 0; pass0 < nrows; pass0 += LA_WARPS * LA_RPW) {
    float m[LA_RPW], l[LA_RPW], acc[LA_RPW][RJ];
    int qpos[LA_RPW];
    bool live[LA_RPW];
#pragma unroll
    for (int i = 0; i < LA_RPW; ++i) {
      const int r = pass0 + warp + i * LA_WARPS;
      live[i] = r < nrows;
      qpos[i] = live[i] ? first_pos + t0 + r / nh : -1;
      m[i] = -INFINITY;
      l[i] = 0.f;
#pragma unroll
      for (int j = 0; j < RJ; ++j) acc[i][j] = 0.f;
    }
    for (int k0 = k_begin; k0 <= qpos_last; k0 += LA_TK) {
      __syncthreads();       // the tile before is consumed (and Qs is written)
      for (int idx = tid; idx < LA_TK * D; idx += LA_THREADS) {
        const int kk = idx / D, d = idx - kk * D;
        const int kpos = k0 + kk;
        float v = 0.f;
        if (kpos >= k_lo && kpos <= qpos_last) {
          const int pg = kpos / a.page_size;
          const size_t crow = (size_t)table[pg] * a.page_size + (kpos - pg * a.page_size);
          v = to_float(cache[crow * D + d]);
        }
        Ks[kk * DS + d] = v;
      }
      __syncthreads();
      // ---- scores: lane = key of the tile
      float s[LA_RPW];
#pragma unroll
      for (int i = 0; i < LA_RPW; ++i) s[i] = 0.f;
      const float* krow = Ks + lane * DS;
      for (int d = 0; d < D; ++d) {
        const float kv = krow[d];
#pragma unroll
        for (int i = 0; i < LA_RPW; ++i)
          if (live[i]) s[i] = fmaf(Qs[(size_t)(pass0 + warp + i * LA_WARPS) * D + d], kv, s[i]);
      }
      const int kpos = k0 + lane;
#pragma unroll
      for (int i = 0; i < LA_RPW; ++i) {
        if (!live[i]) continue;                       // warp-uniform
        bool ok = kpos <= qpos[i];
        if (a.window > 0) ok = ok && (kpos > qpos[i] - a.window);
        const float sv = ok ? s[i] : -INFINITY;
        const float mx = warp_max(sv);
        if (mx == -INFINITY) continue;                // no key of this tile is visible to the row
        const float m_new = fmaxf(m[i], mx);
        const float corr = exp2f(m[i] - m_new);       // m = -inf gives 0
        const float p = ok ? exp2f(sv - m_new) : 0.f;
        l[i] = l[i] * corr + warp_sum(p);
        m[i] = m_new;
#pragma unroll
        for (int j = 0; j < RJ; ++j) acc[i][j] *= corr;
        // ---- values: lane = output column (+ 32 j); the values are the first R elements of the keys
        for (int kk = 0; kk < LA_TK; ++kk) {
          const float pk = __shfl_sync(0xffffffffu, p, kk);
          if (pk == 0.f) continue;                    // warp-uniform
          const float* vrow = Ks + kk * DS;
#pragma unroll
          for (int j = 0; j < RJ; ++j) {
            const int col = lane + 32 * j;
            if (col < R) acc[i][j] = fmaf(pk, vrow[col], acc[i][j]);
          }
        }
      }
    }
    T* out = (T*)a.out;
#pragma unroll
    for (int i = 0; i < LA_RPW; ++i) {
      if (!live[i]) continue;
      const int r = pass0 + warp + i * LA_WARPS;
      const int tt = r / nh, hh = r - tt * nh;
      float den = l[i], keep = 1.f;
      if (a.sinks) {
        const float sk = a.sinks[h0 + hh] * 1.4426950408889634f;
        const float m_new = fmaxf(m[i], sk);
        keep = exp2f(m[i] - m_new);                   // m = -inf gives 0
        den = den * keep + exp2f(sk - m_new);
      }
      const float inv = den > 0.f ? keep / den : 0.f;
#pragma unroll
      for (int j = 0; j < RJ; ++j) {
        const int col = lane + 32 * j;
        if (col < R) out[((size_t)(row0 + t0 + tt) * a.heads + h0 + hh) * R + col] = from_float<T>(acc[i][j] * inv);
      }
    }
  }
}

template <typename T, int RJ>
static int launch_latent(const LatentAttnArgs& a, int max_query_len, cudaStream_t stream) {
  const int D = a.rank + a.rot;
  const size_t smem = sizeof(float) * ((size_t)a.tokens_per_cta * a.heads_per_cta * D + (size_t)LA_TK * (D + 1));
  auto kern = latent_attention_kernel<T, RJ>;
  if (smem > 200 * 1024) return TS_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((max_query_len + a.tokens_per_cta - 1) / a.tokens_per_cta, a.num_seqs,
            (a.heads + a.heads_per_cta - 1) / a.heads_per_cta);
  return launch(kern, grid, LA_THREADS, smem, stream, a);
}


// ------------------------------------------------------- attention, tensor cores
// bf16, (R + P) % 8 == 0, R % 16 == 0. A CTA of eight warps takes 64 query rows (a few tokens x a few
// heads of one request; all of them score against the same cached rows) and walks over the visible
// keys in tiles of 32, fetched with cp.async two tiles deep. Warp w owns query rows 16 (w % 4) .. + 15
// and half of the output columns (w / 4): it forms S = Q K^T for its rows over all R + P elements
// (mma.sync m16n8k16, operands through ldmatrix), does the online softmax in registers, and adds
// P V to its columns, V being the first R elements of the very same rows in shared memory (read
// transposed by ldmatrix). Both warps of a row group form the same S; that costs a third of the
// multiply-adds again and saves exchanging P through shared memory.
// With `splits` > 1 (steps of single tokens) a CTA takes one range of the keys and leaves an
// unnormalised partial result; latent_merge_kernel adds the ranges up.
constexpr int LM_THREADS = 256, LM_ROWS = 64, LM_TK = 32;

__device__ __forceinline__ void lm_cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void lm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void lm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// `s`: an address in the shared window (32 bits), so that the loops add plain offsets
__device__ __forceinline__ void lm_ldmatrix(uint32_t (&r)[4], uint32_t s) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void lm_ldmatrix_t(uint32_t (&r)[4], uint32_t s) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void lm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lm_pack(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

struct LatentSplit {
  int splits;
  float* part_acc;   // [T, H, splits, R]
  float* part_ml;    // [T, H, splits, 2]
};

// NB: blocks of 8 output columns a warp owns at most (its half of R is 8 NB columns or fewer).
template <int NB>
__global__ void __launch_bounds__(LM_THREADS, 1) latent_attention_mma_kernel(LatentAttnArgs a, LatentSplit sp, int ld) {
  extern __shared__ __align__(16) unsigned char lm_raw[];
  bf16* Qs = (bf16*)lm_raw;                        // [LM_ROWS][ld]
  bf16* Ks = Qs + (size_t)LM_ROWS * ld;            // [2][LM_TK][ld]
  pdl_trigger();
  pdl_wait();
  const int R = a.rank, D = a.rank + a.rot;
  const int seq = blockIdx.y;
  const int row0 = a.cu_q[seq];
  const int n = a.cu_q[seq + 1] - row0;
  const int t0 = blockIdx.x * a.tokens_per_cta;
  if (t0 >= n) return;
  const int nt = min(a.tokens_per_cta, n - t0);
  const int chunk = blockIdx.z / sp.splits, split = blockIdx.z - chunk * sp.splits;
  const int h0 = chunk * a.heads_per_cta;
  const int nh = min(a.heads_per_cta, a.heads - h0);
  const int nrows = nt * nh;
  const int ctx = a.ctx_lens[seq];
  const int first_pos = ctx - n;
  const int* table = a.block_tables + (size_t)seq * a.table_width;
  const bf16* q = (const bf16*)a.q;
  const bf16* cache = (const bf16*)a.cache;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp & 3, ch = warp >> 2;
  const int chunks = D >> 3;                       // 16-byte pieces of a row

  const int qpos_first = first_pos + t0, qpos_last = first_pos + t0 + nt - 1;
  int k_lo = a.window > 0 ? max(0, qpos_first - a.window + 1) : 0;
  int k_hi = qpos_last + 1;
  if (sp.splits > 1) {
    const int per = (((k_hi - k_lo) + sp.splits - 1) / sp.splits + LM_TK - 1) / LM_TK * LM_TK;
    k_lo = k_lo + split * per;
    k_hi = min(k_hi, k_lo + per);
  }
  const int k_begin = (k_lo / LM_TK) * LM_TK;
  const int tiles = k_hi > k_begin ? (k_hi - k_begin + LM_TK - 1) / LM_TK : 0;

  // a warp fetches rows warp, warp + 8, ... of a tile, a lane every 32nd piece of a row: one look-up in the
  // block table per row and no division per piece
  auto load_tile = [&](int buf, int k0) {
    bf16* dst = Ks + (size_t)buf * LM_TK * ld;
#pragma unroll
    for (int kk = warp; kk < LM_TK; kk += LM_THREADS / 32) {
      const int kpos = k0 + kk;
      const bool ok = kpos >= k_lo && kpos < k_hi;
      size_t crow = 0;
      if (ok) {
        const int pg = kpos / a.page_size;
        crow = (size_t)table[pg] * a.page_size + (kpos - pg * a.page_size);
      }
      const bf16* src = cache + crow * D;
      bf16* drow = dst + (size_t)kk * ld;
      for (int piece = lane; piece < chunks; piece += 32) lm_cp_async16(drow + piece * 8, src + piece * 8, ok);
    }
  };
  // the queries (rows beyond the CTA's own are zero) and the first tile
  for (int r = warp; r < LM_ROWS; r += LM_THREADS / 32) {
    const bool ok = r < nrows;
    const int tt = ok ? r / nh : 0, hh = ok ? r - tt * nh : 0;
    const bf16* src = q + ((size_t)(row0 + t0 + tt) * a.heads + h0 + hh) * D;
    for (int piece = lane; piece < chunks; piece += 32) lm_cp_async16(Qs + (size_t)r * ld + piece * 8, src + piece * 8, ok);
  }
  if (tiles > 0) load_tile(0, k_begin);
  lm_commit();

  const uint32_t q_base = (uint32_t)__cvta_generic_to_shared(Qs);
  const int r_lo = rg * 16 + (lane >> 2), r_hi = r_lo + 8;          // this thread's two rows of the CTA
  const int qpos_a = r_lo < nrows ? first_pos + t0 + r_lo / nh : -1;
  const int qpos_b = r_hi < nrows ? first_pos + t0 + r_hi / nh : -1;
  const int col_base = ch * NB * 8;                                  // first output column of this warp
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  float o[NB][4];
#pragma unroll
  for (int j = 0; j < NB; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;

  for (int it = 0; it < tiles; ++it) {
    const int k0 = k_begin + it * LM_TK;
    if (it + 1 < tiles) load_tile((it + 1) & 1, k0 + LM_TK);
    lm_commit();
    lm_wait<1>();
    __syncthreads();
    const uint32_t Kt = (uint32_t)__cvta_generic_to_shared(Ks + (size_t)(it & 1) * LM_TK * ld);   // bytes from here on
    // ---- S = Q K^T for 16 rows x 32 keys
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
    const uint32_t qrow = q_base + 2u * (uint32_t)((rg * 16 + (lane & 15)) * ld + (lane >> 4) * 8);
    const uint32_t krow = Kt + 2u * (uint32_t)(((lane & 7) + ((lane >> 4) << 3)) * ld + ((lane >> 3) & 1) * 8);
    {
      // operands of step kk + 16 are asked for before the products of step kk are issued: with two warps
      // per scheduler nothing else hides the shared-memory latency
      uint32_t fa[3][4], fb[3][4];
      auto fetch = [&](uint32_t (&f)[3][4], int kk) {
        lm_ldmatrix(f[0], qrow + 2u * kk);
        lm_ldmatrix(f[1], krow + 2u * kk);
        lm_ldmatrix(f[2], krow + 2u * (uint32_t)(16 * ld + kk));
      };
      auto multiply = [&](const uint32_t (&f)[3][4]) {
        lm_mma(s[0], f[0], f[1][0], f[1][1]);
        lm_mma(s[1], f[0], f[1][2], f[1][3]);
        lm_mma(s[2], f[0], f[2][0], f[2][1]);
        lm_mma(s[3], f[0], f[2][2], f[2][3]);
      };
      int kk = 0;
      fetch(fa, 0);
      for (; kk + 32 <= D; kk += 32) {
        fetch(fb, kk + 16);
        multiply(fa);
        if (kk + 32 < D) fetch(fa, kk + 32);
        multiply(fb);
      }
      if (kk < D) multiply(fa);
    }
    // ---- mask, online softmax (base 2)
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kpos = k0 + j * 8 + (lane & 3) * 2 + (e & 1);
        const int qp = (e & 2) ? qpos_b : qpos_a;
        bool ok = kpos >= k_lo && kpos < k_hi && kpos <= qp;
        if (a.window > 0) ok = ok && kpos > qp - a.window;
        const float v = ok ? s[j][e] * a.scale_log2 : -INFINITY;
        s[j][e] = v;
        if (e & 2) mx_b = fmaxf(mx_b, v); else mx_a = fmaxf(mx_a, v);
      }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
    const float corr_a = mn_a == -INFINITY ? 1.f : exp2f(m_a - mn_a);   // m = -inf gives 0
    const float corr_b = mn_b == -INFINITY ? 1.f : exp2f(m_b - mn_b);
    float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mn = (e & 2) ? mn_b : mn_a;
        const float p = s[j][e] == -INFINITY ? 0.f : exp2f(s[j][e] - mn);
        s[j][e] = p;
        if (e & 2) sum_b += p; else sum_a += p;
      }
    sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
    sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
    sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
    sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
    l_a = l_a * corr_a + sum_a;
    l_b = l_b * corr_b + sum_b;
    m_a = mn_a;
    m_b = mn_b;
    // ---- O = O corr + P V over this warp's columns
    uint32_t pf[2][4];
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      pf[ks][0] = lm_pack(s[2 * ks][0], s[2 * ks][1]);
      pf[ks][1] = lm_pack(s[2 * ks][2], s[2 * ks][3]);
      pf[ks][2] = lm_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]);
      pf[ks][3] = lm_pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
    }
    const uint32_t vrow = Kt + 2u * (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * ld + (lane >> 4) * 8);
    {
      // step st = 2 jp + ks: 16 keys x 16 columns; the values of step st + 1 are asked for before the
      // products of step st (columns from R on belong to nobody: neither fetched nor multiplied)
      uint32_t vf[2][4];
      if (col_base < R) lm_ldmatrix_t(vf[0], vrow + 2u * col_base);
#pragma unroll
      for (int st = 0; st < NB; ++st) {
        const int jp = st >> 1, ks = st & 1;
        const int col = col_base + jp * 16;
        if (st + 1 < NB) {
          const int ncol = col_base + ((st + 1) >> 1) * 16;
          if (ncol < R) lm_ldmatrix_t(vf[(st + 1) & 1], vrow + 2u * (uint32_t)(((st + 1) & 1) * 16 * ld + ncol));
        }
        if (ks == 0) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            o[2 * jp][e] *= (e & 2) ? corr_b : corr_a;
            o[2 * jp + 1][e] *= (e & 2) ? corr_b : corr_a;
          }
        }
        if (col < R) {                                 // warp-uniform; R % 16 == 0
          lm_mma(o[2 * jp], pf[ks], vf[st & 1][0], vf[st & 1][1]);
          lm_mma(o[2 * jp + 1], pf[ks], vf[st & 1][2], vf[st & 1][3]);
        }
      }
    }
    __syncthreads();       // the tile is consumed before the copy after next overwrites it
  }
  lm_wait<0>();
  // ---- results: rows r_lo (e = 0, 1) and r_hi (e = 2, 3), columns col_base + 8 j + 2 (lane % 4) + (e & 1)
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = half ? r_hi : r_lo;
    if (r >= nrows) continue;
    const int tt = r / nh, hh = r - tt * nh;
    const size_t orow = (size_t)(row0 + t0 + tt) * a.heads + h0 + hh;
    const float l = half ? l_b : l_a, m = half ? m_b : m_a;
    if (sp.splits == 1) {
      float den = l, keep = 1.f;
      if (a.sinks) {
        const float sk = a.sinks[h0 + hh] * 1.4426950408889634f;
        const float m_new = fmaxf(m, sk);
        keep = exp2f(m - m_new);                      // m = -inf gives 0
        den = den * keep + exp2f(sk - m_new);
      }
      const float inv = den > 0.f ? keep / den : 0.f;
      bf16* out = (bf16*)a.out + orow * R;
#pragma unroll
      for (int j = 0; j < NB; ++j) {
        const int col = col_base + j * 8 + (lane & 3) * 2;
        if (col < R) *reinterpret_cast<__nv_bfloat162*>(out + col) = __floats2bfloat162_rn(o[j][half * 2] * inv, o[j][half * 2 + 1] * inv);
      }
    } else {
      float* acc = sp.part_acc + (orow * sp.splits + split) * R;
#pragma unroll
      for (int j = 0; j < NB; ++j) {
        const int col = col_base + j * 8 + (lane & 3) * 2;
        if (col < R) *reinterpret_cast<float2*>(acc + col) = make_float2(o[j][half * 2], o[j][half * 2 + 1]);
      }
      if (ch == 0 && (lane & 3) == 0) {
        sp.part_ml[(orow * sp.splits + split) * 2] = m;
        sp.part_ml[(orow * sp.splits + split) * 2 + 1] = l;
      }
    }
  }
}

// out[row, :] = sum_s 2^(m_s - M) acc_s / sum_s 2^(m_s - M) l_s over the key ranges of a row.
// With sinks, head (row % heads) adds 2^(sink log2(e) - M) to the denominator.
__global__ void latent_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, bf16* __restrict__ out,
                                    int splits, int R, const float* __restrict__ sinks, int heads) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  const float* ml = part_ml + row * splits * 2;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, ml[2 * s]);
  float den = 0.f;
  if (sinks) {
    const float sk = sinks[row % heads] * 1.4426950408889634f;
    mm = fmaxf(mm, sk);
    den = exp2f(sk - mm);
  }
  for (int s = 0; s < splits; ++s) den += ml[2 * s] == -INFINITY ? 0.f : ml[2 * s + 1] * exp2f(ml[2 * s] - mm);
  const float inv = den > 0.f ? 1.f / den : 0.f;
  for (int c = threadIdx.x; c < R; c += blockDim.x) {
    float num = 0.f;
    for (int s = 0; s < splits; ++s)
      if (ml[2 * s] != -INFINITY) num += part_acc[(row * splits + s) * R + c] * exp2f(ml[2 * s] - mm);
    out[row * R + c] = from_float<bf16>(num * inv);
  }
}

template <int NB>
static int launch_latent_mma(const LatentAttnArgs& a, const LatentSplit& sp, int max_query_len, cudaStream_t stream) {
  const int D = a.rank + a.rot;
  int ld = D + 8;
  if (((ld >> 3) & 1) == 0) ld += 8;                 // rows 16 (odd) bytes apart: ldmatrix reads without bank conflicts
  const size_t smem = sizeof(bf16) * (size_t)(LM_ROWS + 2 * LM_TK) * ld;
  if (smem > 220 * 1024) return TS_ERR_UNSUPPORTED;
  auto kern = latent_attention_mma_kernel<NB>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int chunks = (a.heads + a.heads_per_cta - 1) / a.heads_per_cta;
  dim3 grid((max_query_len + a.tokens_per_cta - 1) / a.tokens_per_cta, a.num_seqs, chunks * sp.splits);
  return launch(kern, grid, LM_THREADS, smem, stream, a, sp, ld);
}

}  // namespace ts

using namespace ts;

extern "C" int ts_latent_prepare(const void* q_in, long long q_stride, const void* q_folded, const void* ckr,
                                 long long ckr_stride, const void* norm_weight, float eps, const float* cos_t,
                                 const float* sin_t, int rotary_dim, int interleaved, const int* slots, void* cache,
                                 void* q_out, int num_tokens, int heads, int nope, int rank, int rot, int dtype,
                                 cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (heads <= 0 || nope < 0 || rank <= 0 || rot < 0 || rotary_dim < 0 || rotary_dim > rot || (rotary_dim & 1))
    return TS_ERR_BAD_ARGUMENT;
  if (rotary_dim && (!cos_t || !sin_t)) return TS_ERR_BAD_ARGUMENT;
  if (slots && (!cache || !ckr || !norm_weight)) return TS_ERR_BAD_ARGUMENT;
  LatentPrepArgs a;
  a.q_in = q_in; a.q_stride = q_stride; a.q_folded = q_folded; a.ckr = ckr; a.ckr_stride = ckr_stride;
  a.norm_weight = norm_weight; a.eps = eps; a.cos_t = rotary_dim ? cos_t : nullptr; a.sin_t = rotary_dim ? sin_t : nullptr;
  a.rotary_dim = rotary_dim; a.interleaved = interleaved; a.slots = slots; a.cache = cache; a.q_out = q_out;
  a.num_tokens = num_tokens; a.heads = heads; a.nope = nope; a.rank = rank; a.rot = rot;
  if (dtype == TS_DTYPE_F32) return launch(latent_prepare_kernel<float>, num_tokens, 256, 0, stream, a);
  if (dtype == TS_DTYPE_BF16) return launch(latent_prepare_kernel<bf16>, num_tokens, 256, 0, stream, a);
  return TS_ERR_BAD_ARGUMENT;
}

// Largest latent size the kernel takes (32 output columns per lane and step, 16 steps).
extern "C" int ts_latent_attention_max_rank() { return 512; }

// Whether the tensor-core form takes these sizes (bf16 only).
extern "C" int ts_latent_attention_mma_takes(int rank, int rot) {
  const int D = rank + rot;
  int ld = D + 8;
  if (((ld >> 3) & 1) == 0) ld += 8;
  return rank % 16 == 0 && D % 16 == 0 && rank <= 512 && sizeof(bf16) * (size_t)(LM_ROWS + 2 * LM_TK) * ld <= 220 * 1024;
}

// `splits` > 1 (steps of single tokens, tensor-core form only): key ranges per request, with scratch
// part_acc [T, heads, splits, rank] and part_ml [T, heads, splits, 2] floats.
extern "C" int ts_latent_attention(const void* q, void* out, const void* cache, const int* block_tables, int table_width,
                                   const int* cu_q, const int* ctx_lens, int num_seqs, int max_query_len, int heads,
                                   int rank, int rot, int page_size, float scale, int window, int dtype, int use_mma,
                                   int splits, float* part_acc, float* part_ml, int num_tokens, const float* sinks,
                                   cudaStream_t stream) {
  if (num_seqs <= 0 || max_query_len <= 0) return 0;
  if (heads <= 0 || rank <= 0 || rank > 512 || rot < 0 || page_size <= 0 || window < 0) return TS_ERR_BAD_ARGUMENT;
  LatentAttnArgs a;
  a.q = q; a.out = out; a.cache = cache; a.block_tables = block_tables; a.table_width = table_width;
  a.cu_q = cu_q; a.ctx_lens = ctx_lens; a.num_seqs = num_seqs; a.heads = heads; a.rank = rank; a.rot = rot;
  a.page_size = page_size; a.scale_log2 = scale * 1.4426950408889634f; a.window = window;
  a.sinks = sinks;
  if (dtype == TS_DTYPE_BF16 && use_mma && ts_latent_attention_mma_takes(rank, rot) &&
      (((uintptr_t)q | (uintptr_t)cache | (uintptr_t)out) & 15) == 0) {
    if (splits < 1 || (splits > 1 && (max_query_len != 1 || !part_acc || !part_ml))) return TS_ERR_BAD_ARGUMENT;
    // 64 rows a CTA where the step has them: up to 64 heads of as many tokens as fit
    a.heads_per_cta = heads < LM_ROWS ? heads : LM_ROWS;
    a.tokens_per_cta = max_query_len == 1 ? 1 : (LM_ROWS / a.heads_per_cta);
    LatentSplit sp;
    sp.splits = splits; sp.part_acc = part_acc; sp.part_ml = part_ml;
    const int nb = (rank / 2 + 15) / 16 * 2;        // blocks of 8 columns per half, an even number
    int st;
    if (nb <= 8) st = launch_latent_mma<8>(a, sp, max_query_len, stream);
    else if (nb <= 16) st = launch_latent_mma<16>(a, sp, max_query_len, stream);
    else st = launch_latent_mma<32>(a, sp, max_query_len, stream);
    if (st != 0 || splits == 1) return st;
    return launch(latent_merge_kernel, num_tokens * heads, 128, 0, stream, (const float*)part_acc, (const float*)part_ml,
                  (bf16*)out, splits, rank, sinks, heads);
  }
  // 32 rows a CTA where the step has them: 8 heads of 4 tokens (a single token: 8 heads)
  a.heads_per_cta = heads < 8 ? heads : 8;
  a.tokens_per_cta = max_query_len == 1 ? 1 : (32 / a.heads_per_cta);
  const int rj = (rank + 31) / 32;
#define TS_LA_CASE(T_)                                                        \
  do {                                                                        \
    if (rj <= 4) return launch_latent<T_, 4>(a, max_query_len, stream);       \
    if (rj <= 8) return launch_latent<T_, 8>(a, max_query_len, stream);       \
    return launch_latent<T_, 16>(a, max_query_len, stream);                   \
  } while (0)
  if (dtype == TS_DTYPE_F32) TS_LA_CASE(float);
  if (dtype == TS_DTYPE_BF16) TS_LA_CASE(bf16);
#undef TS_LA_CASE
  return TS_ERR_BAD_ARGUMENT;
}
