// latent_attn.cu — attention over a compressed (latent) KV cache.
//
// A latent-attention layer caches, per token, only a normalised latent vector c (kv_rank values) and ONE rotated key part
// shared by all heads (rot_dim values): cache row = [c | k_rot].  Keys and values of head h are linear maps of c
// (k_h = Uk_h c, v_h = Uv_h c), so with the key map folded into the query the layer is multi-query attention over the
// cache rows themselves:
//     qa_h = Uk_h^T q_h[:dim]                              (nvllm_linear, batched over heads, f32)
//     s_hj = scale * (qa_h . c_j + q_h[dim:] . k_rot_j)     j <= position of the query
//     o_h  = sum_j softmax(s_h)_j c_j                      (this file; kv_rank values per head)
//     out_h = Uv_h o_h                                     (nvllm_linear, batched over heads)
// Entry points: the interleaved-pair rotary table (f64 angles), the per-token preparation (RMS norm of the latent, rotary
// on the shared key part and on the queries' rotated part, store into the paged cache) and the paged attention itself, which
// takes every query token with its own sequence index and position — prompt portions, single decoded tokens and any mix of
// them are one launch.  Softmax, norms and all accumulation are f32; cache and activations are bf16 or f32 (dtype).
// Options of the attention (nvllm_latent_window_attention): a sliding window (position p sees p - window + 1 .. p), a sink
// per head whose exponential joins the softmax denominator, and a gate per head (out *= sigmoid(gate)); the rotated part
// may be absent (rot_dim = 0).
#include "common.cuh"

namespace nvllm {
namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// table[p][i] = (cos, sin)(p * base^(-2i/dims)), i < dims/2, angles in f64
__global__ void rope_table_interleaved_kernel(float2* __restrict__ tab, int max_pos, int half, int dims, double base) {
  const int64_t total = static_cast<int64_t>(max_pos) * half;
  for (int64_t e = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; e < total;
       e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t p = e / half;
    const int i = static_cast<int>(e - p * half);
    const double f = pow(base, -2.0 * i / dims), a = static_cast<double>(p) * f;
    tab[e] = make_float2(static_cast<float>(cos(a)), static_cast<float>(sin(a)));
  }
}

struct PrepArgs {
  void* q; int64_t ldq;
  const void* dkv; int64_t lddkv;
  const float* c_norm_w; float eps;
  const int64_t* positions; const float2* table; int rot_dims, max_pos;
  int n, heads, dim, rot_dim, kv_rank;
  void* cache; int64_t cache_row; const int32_t* slots;
};

// One warp per token: c = rms_norm(dkv[:kv_rank]) * w -> cache row; rotary (pairs (2i, 2i+1), first rot_dims of the
// rotated part) on dkv[kv_rank:] -> cache row, and in place on the rotated part of every query head.
template <typename T>
__global__ void __launch_bounds__(128) latent_prepare_kernel(const PrepArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= a.n) return;
  const T* row = static_cast<const T*>(a.dkv) + static_cast<int64_t>(t) * a.lddkv;
  const int32_t slot = a.slots[t];
  int64_t pos = a.positions[t];
  pos = pos < 0 ? 0 : (pos >= a.max_pos ? a.max_pos - 1 : pos);
  const float2* tab = a.table + pos * (a.rot_dims / 2);
  T* crow = slot >= 0 ? static_cast<T*>(a.cache) + static_cast<int64_t>(slot) * a.cache_row : nullptr;
  float ss = 0.f;
  for (int i = lane; i < a.kv_rank; i += 32) { const float v = ldf(row + i); ss = fmaf(v, v, ss); }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(a.kv_rank) + a.eps);
  if (crow) {
    for (int i = lane; i < a.kv_rank; i += 32) stf(crow + i, ldf(row + i) * inv * a.c_norm_w[i]);
    for (int i = lane; i < a.rot_dim; i += 32) {
      float v = ldf(row + a.kv_rank + i);
      if (i < a.rot_dims) {
        const float2 cs = tab[i >> 1];
        const float o = ldf(row + a.kv_rank + (i ^ 1));
        v = (i & 1) ? fmaf(v, cs.x, o * cs.y) : fmaf(v, cs.x, -o * cs.y);  // (u cos - v sin, v cos + u sin)
      }
      stf(crow + a.kv_rank + i, v);
    }
  }
  T* q = static_cast<T*>(a.q) + static_cast<int64_t>(t) * a.ldq;
  const int half = a.rot_dims / 2;
  for (int e = lane; e < a.heads * half; e += 32) {
    const int h = e / half, i = e - h * half;
    T* p = q + static_cast<int64_t>(h) * (a.dim + a.rot_dim) + a.dim + 2 * i;
    const float u = ldf(p), v = ldf(p + 1);
    const float2 cs = tab[i];
    stf(p, fmaf(u, cs.x, -v * cs.y));
    stf(p + 1, fmaf(v, cs.x, u * cs.y));
  }
}

struct AttnArgs {
  void* out; int64_t ldo;           // [n, heads, kv_rank]
  const float* q_abs; int64_t ldqa;  // [n, heads, kv_rank] f32
  const void* q; int64_t ldq;        // [n, heads, dim + rot_dim]: only the rotated part is read
  const int32_t* tok_seq; const int64_t* positions;
  const int32_t* tables; int table_cap, block_size;
  const void* cache; int64_t cache_row;
  int n, heads, dim, rot_dim, kv_rank;
  float scale;
  int window; const float* sinks; const float* gate; int64_t ldg;   // 0 / null: none
  int splits; float* part;   // splits > 1: CTAs along z share a token's key tiles; partial (acc[kv_rank], m, l) per (token, head, split)
};

constexpr int kKeyTile = 32;

// CTA = one query token x up to 8 heads (one warp per head).  Key tiles of 32 cache rows are staged once in shared memory
// (f32) and shared by the CTA's heads; lane j scores key j, then every lane owns kv_rank/32 output columns.
template <typename T, int RI>
__global__ void __launch_bounds__(256) latent_attn_kernel(const AttnArgs a) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int t = blockIdx.x, h = blockIdx.y * nwarps + warp;
  const bool active = h < a.heads;
  const int D = a.kv_rank + a.rot_dim, stride = D | 1;
  float* qs = smem;                       // [nwarps][D]
  float* ks = smem + nwarps * D;          // [kKeyTile][stride]
  const int seq = a.tok_seq[t];
  const int64_t pos = a.positions[t];
  const int nkeys = static_cast<int>(pos) + 1;
  if (active) {
    const float* qa = a.q_abs + static_cast<int64_t>(t) * a.ldqa + static_cast<int64_t>(h) * a.kv_rank;
    const T* qr = static_cast<const T*>(a.q) + static_cast<int64_t>(t) * a.ldq + static_cast<int64_t>(h) * (a.dim + a.rot_dim) + a.dim;
    for (int d = lane; d < a.kv_rank; d += 32) qs[warp * D + d] = qa[d] * a.scale;
    for (int d = lane; d < a.rot_dim; d += 32) qs[warp * D + a.kv_rank + d] = ldf(qr + d) * a.scale;
  }
  float m = -INFINITY, l = 0.f, acc[RI];
#pragma unroll
  for (int i = 0; i < RI; ++i) acc[i] = 0.f;
  const int32_t* table = a.tables + static_cast<int64_t>(seq) * a.table_cap;
  const int first = a.window > 0 ? max(0, nkeys - a.window) : 0;   // tiles start at multiples of kKeyTile whatever the window
  for (int j0 = first & ~(kKeyTile - 1); j0 < nkeys; j0 += kKeyTile) {
    const int cnt = min(kKeyTile, nkeys - j0);
    __syncthreads();
    for (int e = threadIdx.x; e < cnt * D; e += blockDim.x) {
      const int jj = e / D, d = e - jj * D, j = j0 + jj;
      const int32_t blk = table[j / a.block_size];
      float v = 0.f;
      if (blk >= 0)
        v = ldf(static_cast<const T*>(a.cache) + (static_cast<int64_t>(blk) * a.block_size + j % a.block_size) * a.cache_row + d);
      ks[jj * stride + d] = v;
    }
    __syncthreads();
    if (!active) continue;
    float s = -INFINITY;
    if (lane < cnt && j0 + lane >= first && table[(j0 + lane) / a.block_size] >= 0) {
      s = 0.f;
      const float* k = ks + lane * stride;
      const float* q = qs + warp * D;
      for (int d = 0; d < D; ++d) s = fmaf(q[d], k[d], s);
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;
    const float p = s == -INFINITY ? 0.f : expf(s - m_new);
    const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < RI; ++i) acc[i] *= corr;
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const float* k = ks + jj * stride;
#pragma unroll
      for (int i = 0; i < RI; ++i)
        if (lane + 32 * i < a.kv_rank) acc[i] = fmaf(pj, k[lane + 32 * i], acc[i]);
    }
  }
  if (!active) return;
  T* o = static_cast<T*>(a.out) + static_cast<int64_t>(t) * a.ldo + static_cast<int64_t>(h) * a.kv_rank;
  float oc = 1.0f;
  if (a.sinks) {   // the sink joins the denominator only
    const float sk = a.sinks[h], mn = fmaxf(m, sk);
    oc = expf(m - mn);
    l = l * oc + expf(sk - mn);
  }
  float inv = l > 0.f ? oc / l : 0.f;
  if (a.gate) inv *= 1.0f / (1.0f + expf(-a.gate[static_cast<int64_t>(t) * a.ldg + h]));
#pragma unroll
  for (int i = 0; i < RI; ++i)
    if (lane + 32 * i < a.kv_rank) stf(o + lane + 32 * i, acc[i] * inv);
}

template <typename T, int RI>
int launch_attn(const AttnArgs& a, cudaStream_t st) {
  const int hpb = a.heads < 8 ? a.heads : 8;
  const int D = a.kv_rank + a.rot_dim;
  const size_t smem = (static_cast<size_t>(hpb) * D + static_cast<size_t>(kKeyTile) * (D | 1)) * sizeof(float);
  NVLLM_CHECK_ARG(smem <= 220 * 1024, NVLLM_ERR_ARG, "latent_attention: kv_rank + rot_dim = %d needs %zu bytes of shared memory", D, smem);
  NVLLM_SMEM_ATTR_ONCE((latent_attn_kernel<T, RI>), 220 * 1024);
  dim3 grid(a.n, (a.heads + hpb - 1) / hpb);
  latent_attn_kernel<T, RI><<<grid, 32 * hpb, smem, st>>>(a);
  NVLLM_LAUNCH_CHECK("latent_attn_kernel");
  return 0;
}


// ---- tensor-core variant (bf16 operands) -------------------------------------------------------------------------------
// With the key map folded into the query, all heads of a token score against the SAME cache rows: the heads are the M
// dimension of the matrix products.  CTA = one query token x 16 heads, key tiles of 64 cache rows staged in shared
// memory (bf16, rows padded against bank conflicts, double-buffered with cp.async):
//   S[16 x 64]  = Q[16 x (kv_rank + rot_dim)] . K^T      mma.sync m16n8k16, f32 accumulate
//   online softmax in f32 through shared memory (row max / sum / rescale factor), P rounded to bf16
//   O[16 x kv_rank] += P[16 x 64] . C[64 x kv_rank]      each warp its share of the columns, C read with ldmatrix.trans
// Decoding is bound by reading the cache once per token; prompt portions re-read the tile per token from L2.
constexpr int kMmaKeys = 64, kPsStride = 72, kSsStride = 68, kMmaThreads = 256;

// 8 warps.  Scores: warp w takes 16 keys (w & 3) and one half of the reduction dimension (w >> 2), with two accumulators
// per 8-key block so that the dependent mma chains stay short; the halves meet in shared memory.  Output: every warp owns
// NT2 * 16 of the (padded) kv_rank columns.  TQ = 2 (large batches, i.e. prompt portions): the CTA takes two consecutive
// tokens of the batch; when they belong to the same sequence they share every key tile and every B fragment (the kernel is
// bound by instruction issue and latency, not by the tensor pipe, so the second token is almost free); when they do not,
// the CTA runs them one after the other.
template <int NT2, int TQ>  // kv_rank padded to NT2 * 128
__global__ void __launch_bounds__(kMmaThreads) latent_attn_mma_kernel(const AttnArgs a, int DPS, int DP16) {
  extern __shared__ __align__(16) uint8_t smraw[];
  bf16* Qs = reinterpret_cast<bf16*>(smraw);          // TQ x [16][DPS]
  bf16* Kbuf = Qs + TQ * 16 * DPS;                    // 2 x [64][DPS]: the next tile lands while this one is used
  bf16* Ps = Kbuf + 2 * kMmaKeys * DPS;               // TQ x [16][kPsStride]
  float* Ss = reinterpret_cast<float*>(Ps + TQ * 16 * kPsStride);  // TQ x 2 x [16][kSsStride]: one per half of the reduction
  float* m_s = Ss + TQ * 2 * 16 * kSsStride;          // TQ x 16 each
  float* l_s = m_s + TQ * 16;
  float* c_s = l_s + TQ * 16;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int hbase = blockIdx.y * 16;
  constexpr int RC = NT2 * 16;
  const int vec_per_row = static_cast<int>(a.cache_row / 8);   // cache rows are padded to 8 elements (zeros)
  const int pad0 = vec_per_row * 8, heads_here = a.heads - hbase < 16 ? a.heads - hbase : 16;
  const int nks = DP16 / 16, ks_mid = (nks + 1) / 2;
  const int ks0 = (warp >> 2) ? ks_mid : 0, ks1 = (warp >> 2) ? nks : ks_mid;
  // zero once what no copy ever writes: the columns behind a cache row in every buffer row, and query rows of absent heads
  {
    const int padw = DPS - pad0;   // >= 8
    for (int e = tid; e < (TQ * 16 + 2 * kMmaKeys) * padw; e += kMmaThreads) Qs[(e / padw) * DPS + pad0 + e % padw] = __float2bfloat16_rn(0.f);
    for (int q = 0; q < TQ; ++q)
      for (int e = tid; e < (16 - heads_here) * pad0; e += kMmaThreads)
        Qs[(q * 16 + heads_here + e / pad0) * DPS + e % pad0] = __float2bfloat16_rn(0.f);
  }
  const int tfirst = blockIdx.x * TQ;
  bool together = false;
  if (TQ == 2 && tfirst + 1 < a.n) together = a.tok_seq[tfirst] == a.tok_seq[tfirst + 1];
  const int npass = (TQ == 1 || together || tfirst + 1 >= a.n) ? 1 : 2;
  for (int pass = 0; pass < npass; ++pass) {
    // tokens of this pass: slot q holds token tq[q] (-1: slot unused)
    int tq[TQ], nk[TQ], lo[TQ], nkeys = 0;
    const int t_lead = tfirst + pass;
    const int32_t* table = a.tables + static_cast<int64_t>(a.tok_seq[t_lead]) * a.table_cap;
#pragma unroll
    for (int q = 0; q < TQ; ++q) {
      tq[q] = (q == 0) ? t_lead : (together ? tfirst + 1 : -1);
      nk[q] = tq[q] >= 0 ? static_cast<int>(a.positions[tq[q]]) + 1 : 0;
      nkeys = nk[q] > nkeys ? nk[q] : nkeys;
    }
    for (int b = 0; b * a.block_size < nkeys; ++b)   // a missing block ends the sequence's keys (padding rows of a graph: none)
      if (table[b] < 0) { nkeys = b * a.block_size; break; }
    int jstart = nkeys;
#pragma unroll
    for (int q = 0; q < TQ; ++q) {
      lo[q] = a.window > 0 && nk[q] > a.window ? nk[q] - a.window : 0;   // first key the token sees (from its position alone)
      nk[q] = nk[q] < nkeys ? nk[q] : nkeys;
      if (tq[q] >= 0) jstart = lo[q] < jstart ? lo[q] : jstart;
    }
    jstart &= ~(kMmaKeys - 1);   // key tiles stay anchored at multiples of 64 from the sequence's start
    if (a.splits > 1) {          // this CTA's share of the tiles (single tokens with few CTAs: the keys are split along z)
      const int tiles = (nkeys - jstart + kMmaKeys - 1) / kMmaKeys, per = (tiles + a.splits - 1) / a.splits;
      jstart += static_cast<int>(blockIdx.z) * per * kMmaKeys;
      const int jend = jstart + per * kMmaKeys;
      nkeys = nkeys < jend ? nkeys : jend;
      if (jstart > nkeys) jstart = nkeys;
#pragma unroll
      for (int q = 0; q < TQ; ++q) nk[q] = nk[q] < nkeys ? nk[q] : nkeys;
    }
    __syncthreads();   // previous pass done with every buffer; the zero fill above is ordered before the copies below
    if (tid < TQ * 16) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; c_s[tid] = 1.f; }
    // four threads per cache row: one block-table look-up per thread and tile, 16-byte asynchronous copies (zero fill past
    // the sequence's keys)
    auto prefetch = [&](int j0, bf16* Ks) {
      const int jj = tid >> 2, j = j0 + jj;
      const bf16* src = static_cast<const bf16*>(a.cache);
      int bytes = 0;
      if (j < nkeys) {
        src += (static_cast<int64_t>(table[j / a.block_size]) * a.block_size + j % a.block_size) * a.cache_row;
        bytes = 16;
      }
      const uint32_t dst = smem_u32(Ks + jj * DPS);
      for (int v = tid & 3; v < vec_per_row; v += 4) cp_async_16(dst + v * 16, src + (bytes ? v * 8 : 0), bytes);
      cp_async_commit();
    };
    prefetch(jstart, Kbuf);
    // the queries: [folded q (f32 -> bf16) | rotated part | zeros up to the cache row's width]
#pragma unroll
    for (int q = 0; q < TQ; ++q) {
      bf16* Qq = Qs + q * 16 * DPS;
      if (tq[q] < 0) {
        for (int e = tid; e < heads_here * pad0; e += kMmaThreads) Qq[(e / pad0) * DPS + e % pad0] = __float2bfloat16_rn(0.f);
        continue;
      }
      const float* qa = a.q_abs + static_cast<int64_t>(tq[q]) * a.ldqa + static_cast<int64_t>(hbase) * a.kv_rank;
      const bf16* qr = static_cast<const bf16*>(a.q) + static_cast<int64_t>(tq[q]) * a.ldq + static_cast<int64_t>(hbase) * (a.dim + a.rot_dim) + a.dim;
      if (a.kv_rank % 4 == 0 && (reinterpret_cast<uintptr_t>(qa) & 15u) == 0) {   // rows of one token are contiguous: 16-byte loads
        const int q4 = a.kv_rank / 4;
        for (int e = tid; e < heads_here * q4; e += kMmaThreads) {
          const int r = e / q4, c = (e - r * q4) * 4;
          const float4 v = *reinterpret_cast<const float4*>(qa + static_cast<int64_t>(r) * a.kv_rank + c);
          *reinterpret_cast<uint2*>(Qq + r * DPS + c) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
        }
      } else {
        for (int e = tid; e < heads_here * a.kv_rank; e += kMmaThreads) {
          const int r = e / a.kv_rank, c = e - r * a.kv_rank;
          Qq[r * DPS + c] = __float2bfloat16_rn(qa[static_cast<int64_t>(r) * a.kv_rank + c]);
        }
      }
      const int tail = pad0 - a.kv_rank;   // rotated part, then zeros
      for (int e = tid; e < heads_here * tail; e += kMmaThreads) {
        const int r = e / tail, c = e - r * tail;
        Qq[r * DPS + a.kv_rank + c] = c < a.rot_dim ? qr[static_cast<int64_t>(r) * (a.dim + a.rot_dim) + c] : __float2bfloat16_rn(0.f);
      }
    }
    float acc[TQ][2 * NT2][4];
#pragma unroll
    for (int q = 0; q < TQ; ++q)
#pragma unroll
      for (int i = 0; i < 2 * NT2; ++i) acc[q][i][0] = acc[q][i][1] = acc[q][i][2] = acc[q][i][3] = 0.f;
    int buf = 0;
    for (int j0 = jstart; j0 < nkeys; j0 += kMmaKeys, buf ^= 1) {
      bf16* Ks = Kbuf + buf * kMmaKeys * DPS;
      if (j0 + kMmaKeys < nkeys) {
        prefetch(j0 + kMmaKeys, Kbuf + (buf ^ 1) * kMmaKeys * DPS);   // that buffer's last readers passed the barrier below
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();   // this tile (and, first time round, the queries) visible to all warps
      {  // partial scores: 16 keys x this warp's half of the reduction dimension, for every token of the CTA
        float s[TQ][4][4];
#pragma unroll
        for (int q = 0; q < TQ; ++q)
#pragma unroll
          for (int i = 0; i < 4; ++i) s[q][i][0] = s[q][i][1] = s[q][i][2] = s[q][i][3] = 0.f;
        const int krow = 16 * (warp & 3);
        const uint32_t qa = smem_u32(Qs + (lane & 15) * DPS + (lane >> 4) * 8);
        const uint32_t ka = smem_u32(Ks + (krow + (lane & 7) + 8 * (lane >> 4)) * DPS + 8 * ((lane >> 3) & 1));
        const uint32_t qstep = static_cast<uint32_t>(DPS) * 32;   // 16 query rows in bytes
        int ks = ks0;
        for (; ks + 1 < ks1; ks += 2) {
          uint32_t bq[4], bq2[4];
          ldmatrix_x4(bq, ka + ks * 32);
          ldmatrix_x4(bq2, ka + ks * 32 + 32);
#pragma unroll
          for (int q = 0; q < TQ; ++q) {
            uint32_t af[4], af2[4];
            ldmatrix_x4(af, qa + q * qstep + ks * 32);
            ldmatrix_x4(af2, qa + q * qstep + ks * 32 + 32);
            mma_bf16_16816(s[q][0], af, bq[0], bq[1]);
            mma_bf16_16816(s[q][1], af, bq[2], bq[3]);
            mma_bf16_16816(s[q][2], af2, bq2[0], bq2[1]);
            mma_bf16_16816(s[q][3], af2, bq2[2], bq2[3]);
          }
        }
        if (ks < ks1) {
          uint32_t bq[4];
          ldmatrix_x4(bq, ka + ks * 32);
#pragma unroll
          for (int q = 0; q < TQ; ++q) {
            uint32_t af[4];
            ldmatrix_x4(af, qa + q * qstep + ks * 32);
            mma_bf16_16816(s[q][0], af, bq[0], bq[1]);
            mma_bf16_16816(s[q][1], af, bq[2], bq[3]);
          }
        }
#pragma unroll
        for (int q = 0; q < TQ; ++q) {
          float* So = Ss + (q * 2 + (warp >> 2)) * 16 * kSsStride;
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) {
            const int col = krow + nt * 8 + 2 * t4;
            So[g * kSsStride + col] = s[q][nt][0] + s[q][nt + 2][0];
            So[g * kSsStride + col + 1] = s[q][nt][1] + s[q][nt + 2][1];
            So[(g + 8) * kSsStride + col] = s[q][nt][2] + s[q][nt + 2][2];
            So[(g + 8) * kSsStride + col + 1] = s[q][nt][3] + s[q][nt + 2][3];
          }
        }
      }
      __syncthreads();
      if (warp < 4 * TQ) {  // online softmax: warps 0-3 token 0, warps 4-7 token 1; 4 rows per warp, 8 lanes per row, 8 keys per lane
        const int q = warp >> 2, row = 4 * (warp & 3) + (lane >> 3), sub = lane & 7;
        const float* S0 = Ss + q * 2 * 16 * kSsStride;
        const int nkq = (TQ == 1) ? nk[0] : (q == 0 ? nk[0] : nk[TQ - 1]);
        const int loq = (TQ == 1) ? lo[0] : (q == 0 ? lo[0] : lo[TQ - 1]);
        float sv[8], mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const bool ok = j0 + sub * 8 + i < nkq && j0 + sub * 8 + i >= loq;
          sv[i] = ok ? (S0[row * kSsStride + sub * 8 + i] + S0[(16 + row) * kSsStride + sub * 8 + i]) * a.scale : -INFINITY;
          mx = fmaxf(mx, sv[i]);
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_old = m_s[q * 16 + row], m_new = fmaxf(m_old, mx);
        float sum = 0.f, pv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          pv[i] = (sv[i] == -INFINITY) ? 0.f : expf(sv[i] - m_new);
          sum += pv[i];
        }
        *reinterpret_cast<uint4*>(Ps + (q * 16 + row) * kPsStride + sub * 8) =
            make_uint4(pack_bf16x2(pv[0], pv[1]), pack_bf16x2(pv[2], pv[3]), pack_bf16x2(pv[4], pv[5]), pack_bf16x2(pv[6], pv[7]));
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        __syncwarp();
        if (sub == 0) {
          const float corr = (m_new == -INFINITY || m_old == -INFINITY) ? (m_new == -INFINITY ? 1.f : 0.f) : expf(m_old - m_new);
          c_s[q * 16 + row] = corr;
          l_s[q * 16 + row] = l_s[q * 16 + row] * corr + sum;
          m_s[q * 16 + row] = m_new;
        }
      }
      __syncthreads();
      {  // O += P . C over this warp's RC columns
#pragma unroll
        for (int q = 0; q < TQ; ++q) {
          const float cg = c_s[q * 16 + g], cg8 = c_s[q * 16 + g + 8];
#pragma unroll
          for (int i = 0; i < 2 * NT2; ++i) { acc[q][i][0] *= cg; acc[q][i][1] *= cg; acc[q][i][2] *= cg8; acc[q][i][3] *= cg8; }
        }
        const uint32_t pa = smem_u32(Ps + (lane & 15) * kPsStride + (lane >> 4) * 8);
        const uint32_t va = smem_u32(Ks + ((lane & 7) + 8 * ((lane >> 3) & 1)) * DPS + warp * RC + 8 * (lane >> 4));
        const uint32_t vstep = static_cast<uint32_t>(DPS) * 32;   // 16 cache rows in bytes
#pragma unroll
        for (int kk = 0; kk < kMmaKeys / 16; ++kk) {
          uint32_t pf[TQ][4];
#pragma unroll
          for (int q = 0; q < TQ; ++q) ldmatrix_x4(pf[q], pa + q * (16 * kPsStride * 2) + kk * 32);
#pragma unroll
          for (int p2 = 0; p2 < NT2; ++p2) {
            uint32_t bv[4];
            ldmatrix_x4_trans(bv, va + kk * vstep + p2 * 32);
#pragma unroll
            for (int q = 0; q < TQ; ++q) {
              mma_bf16_16816(acc[q][2 * p2], pf[q], bv[0], bv[1]);
              mma_bf16_16816(acc[q][2 * p2 + 1], pf[q], bv[2], bv[3]);
            }
          }
        }
      }
      __syncthreads();   // tile, P and the row factors are free again
    }
    if (a.splits > 1) {   // unnormalised partial results; latent_attn_merge_kernel finishes the softmax
      cp_async_wait<0>();
      __syncthreads();    // a share without tiles never entered the loop: its row statistics are still the initial ones
#pragma unroll
      for (int q = 0; q < TQ; ++q) {
        if (tq[q] < 0) continue;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = g + 8 * half, h = hbase + r;
          if (h >= a.heads) continue;
          float* pr = a.part + ((static_cast<int64_t>(tq[q]) * a.heads + h) * a.splits + blockIdx.z) * (a.kv_rank + 2);
#pragma unroll
          for (int nt = 0; nt < 2 * NT2; ++nt)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const int col = warp * RC + nt * 8 + 2 * t4 + c;
              if (col < a.kv_rank) pr[col] = acc[q][nt][2 * half + c];
            }
          if (warp == 0 && t4 == 0) { pr[a.kv_rank] = m_s[q * 16 + r]; pr[a.kv_rank + 1] = l_s[q * 16 + r]; }
        }
      }
      continue;
    }
#pragma unroll
    for (int q = 0; q < TQ; ++q) {
      if (tq[q] < 0) continue;
      bf16* out = static_cast<bf16*>(a.out) + static_cast<int64_t>(tq[q]) * a.ldo;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = g + 8 * half, h = hbase + r;
        if (h >= a.heads) continue;
        float l = l_s[q * 16 + r], oc = 1.0f;
        if (a.sinks) {   // the sink joins the denominator only
          const float sk = a.sinks[h], mo = m_s[q * 16 + r], mn = fmaxf(mo, sk);
          oc = expf(mo - mn);
          l = l * oc + expf(sk - mn);
        }
        float inv = l > 0.f ? oc / l : 0.f;
        if (a.gate) inv *= 1.0f / (1.0f + expf(-a.gate[static_cast<int64_t>(tq[q]) * a.ldg + h]));
#pragma unroll
        for (int nt = 0; nt < 2 * NT2; ++nt)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int col = warp * RC + nt * 8 + 2 * t4 + c;
            if (col < a.kv_rank) out[static_cast<int64_t>(h) * a.kv_rank + col] = __float2bfloat16_rn(acc[q][nt][2 * half + c] * inv);
          }
      }
    }
  }
}

// One warp per (token, head): merges the splits' partial softmaxes, adds the sink to the denominator, applies the gate.
__global__ void __launch_bounds__(128) latent_attn_merge_kernel(const AttnArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (item >= static_cast<int64_t>(a.n) * a.heads) return;
  const int64_t t = item / a.heads;
  const int h = static_cast<int>(item - t * a.heads), W = a.kv_rank + 2;
  const float* pr = a.part + item * a.splits * W;
  float mx = a.sinks ? a.sinks[h] : -INFINITY;
  for (int s = 0; s < a.splits; ++s) mx = fmaxf(mx, pr[s * W + a.kv_rank]);
  float den = a.sinks ? expf(a.sinks[h] - mx) : 0.f;
  for (int s = 0; s < a.splits; ++s) {
    const float ms = pr[s * W + a.kv_rank];
    if (ms != -INFINITY) den += expf(ms - mx) * pr[s * W + a.kv_rank + 1];
  }
  float inv = den > 0.f ? 1.0f / den : 0.f;
  if (a.gate) inv *= 1.0f / (1.0f + expf(-a.gate[t * a.ldg + h]));
  bf16* out = static_cast<bf16*>(a.out) + t * a.ldo + static_cast<int64_t>(h) * a.kv_rank;
  for (int c = lane; c < a.kv_rank; c += 32) {
    float v = 0.f;
    for (int s = 0; s < a.splits; ++s) {
      const float ms = pr[s * W + a.kv_rank];
      if (ms != -INFINITY) v = fmaf(expf(ms - mx), pr[s * W + c], v);
    }
    out[c] = __float2bfloat16_rn(v * inv);
  }
}

template <int NT2, int TQ>
int launch_attn_mma_tq(const AttnArgs& a, cudaStream_t st) {
  const int DP16 = (static_cast<int>(a.cache_row) + 15) / 16 * 16, RP = NT2 * 128;
  const int DPS = (DP16 > RP ? DP16 : RP) + 8;
  const size_t smem = static_cast<size_t>(TQ * 16 + 2 * kMmaKeys) * DPS * 2 + TQ * 16 * kPsStride * 2 +
                      (TQ * 2 * 16 * kSsStride + TQ * 48) * 4;
  NVLLM_SMEM_ATTR_ONCE((latent_attn_mma_kernel<NT2, TQ>), 225 * 1024);
  dim3 grid((a.n + TQ - 1) / TQ, (a.heads + 15) / 16, TQ == 1 && a.splits > 1 ? a.splits : 1);
  latent_attn_mma_kernel<NT2, TQ><<<grid, kMmaThreads, smem, st>>>(a, DPS, DP16);
  NVLLM_LAUNCH_CHECK("latent_attn_mma_kernel");
  if (TQ == 1 && a.splits > 1) {
    latent_attn_merge_kernel<<<static_cast<unsigned>((static_cast<int64_t>(a.n) * a.heads + 3) / 4), 128, 0, st>>>(a);
    NVLLM_LAUNCH_CHECK("latent_attn_merge_kernel");
  }
  return 0;
}

// Two tokens per CTA for batches that are mostly prompt portions (more than 256 tokens: a decode batch holds one token per
// sequence, so its neighbours never share keys), when the second token's buffers still fit in shared memory.
template <int NT2>
int launch_attn_mma(const AttnArgs& a, cudaStream_t st) {
  const int DP16 = (static_cast<int>(a.cache_row) + 15) / 16 * 16, RP = NT2 * 128;
  const int DPS = (DP16 > RP ? DP16 : RP) + 8;
  const size_t smem2 = static_cast<size_t>(32 + 2 * kMmaKeys) * DPS * 2 + 32 * kPsStride * 2 + (4 * 16 * kSsStride + 96) * 4;
  if (a.n > 256 && knobs().latent_mma != 2 && smem2 <= 225 * 1024) { AttnArgs b = a; b.splits = 1; return launch_attn_mma_tq<NT2, 2>(b, st); }
  return launch_attn_mma_tq<NT2, 1>(a, st);
}

template <typename T>
int dispatch_attn(const AttnArgs& a, cudaStream_t st) {
  if (a.kv_rank <= 128) return launch_attn<T, 4>(a, st);
  if (a.kv_rank <= 512) return launch_attn<T, 16>(a, st);
  return launch_attn<T, 32>(a, st);
}

}  // namespace
}  // namespace nvllm

using namespace nvllm;

extern "C" int nvllm_rope_table_interleaved(float* cos_sin, int32_t max_pos, int32_t dims, double base, void* stream) {
  NVLLM_CHECK_ARG(cos_sin && max_pos > 0 && dims > 0 && dims % 2 == 0 && base > 0, NVLLM_ERR_ARG,
                  "rope_table_interleaved: max_pos=%d dims=%d (even) base=%g", max_pos, dims, base);
  const int64_t total = static_cast<int64_t>(max_pos) * (dims / 2);
  int64_t blocks = (total + 255) / 256;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  rope_table_interleaved_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<float2*>(cos_sin), max_pos, dims / 2, dims, base);
  NVLLM_LAUNCH_CHECK("rope_table_interleaved_kernel");
  return 0;
}

extern "C" int nvllm_latent_prepare(void* q, int64_t ldq, const void* dkv, int64_t lddkv, const float* c_norm_w, float eps,
                                    const int64_t* positions, const float* rope_table, int32_t rot_dims, int32_t max_pos,
                                    int32_t n, int32_t heads, int32_t dim, int32_t rot_dim, int32_t kv_rank, void* cache,
                                    int64_t cache_row, const int32_t* slots, int32_t dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && heads > 0 && dim >= 0 && rot_dim >= 0 && kv_rank > 0, NVLLM_ERR_ARG, "latent_prepare: sizes");
  NVLLM_CHECK_ARG(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= rot_dim, NVLLM_ERR_ARG,
                  "latent_prepare: rot_dims=%d must be even and at most rot_dim=%d", rot_dims, rot_dim);
  NVLLM_CHECK_ARG(cache_row >= kv_rank + rot_dim && ldq >= static_cast<int64_t>(heads) * (dim + rot_dim) && lddkv >= kv_rank + rot_dim,
                  NVLLM_ERR_ARG, "latent_prepare: strides");
  NVLLM_CHECK_ARG(dtype == NVLLM_BF16 || dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "latent_prepare: dtype %d", dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(q && dkv && c_norm_w && positions && (rope_table || rot_dims == 0) && cache && slots, NVLLM_ERR_ARG, "latent_prepare: NULL");
  const PrepArgs a{q, ldq, dkv, lddkv, c_norm_w, eps, positions, reinterpret_cast<const float2*>(rope_table), rot_dims, max_pos,
                   n, heads, dim, rot_dim, kv_rank, cache, cache_row, slots};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == NVLLM_BF16) latent_prepare_kernel<bf16><<<(n + 3) / 4, 128, 0, st>>>(a);
  else latent_prepare_kernel<float><<<(n + 3) / 4, 128, 0, st>>>(a);
  NVLLM_LAUNCH_CHECK("latent_prepare_kernel");
  return 0;
}

extern "C" int nvllm_latent_attention(void* out, int64_t ldo, const float* q_abs, int64_t ldqa, const void* q, int64_t ldq,
                                      const int32_t* tok_seq, const int64_t* positions, const int32_t* block_tables,
                                      int32_t table_cap, int32_t block_size, const void* cache, int64_t cache_row, int32_t n,
                                      int32_t heads, int32_t dim, int32_t rot_dim, int32_t kv_rank, float scale,
                                      int32_t dtype, void* stream) {
  return nvllm_latent_window_attention(out, ldo, q_abs, ldqa, q, ldq, tok_seq, positions, block_tables, table_cap, block_size, cache,
                                       cache_row, n, heads, dim, rot_dim, kv_rank, scale, 0, nullptr, nullptr, 0, nullptr, 0, dtype, stream);
}

extern "C" int nvllm_latent_window_attention(void* out, int64_t ldo, const float* q_abs, int64_t ldqa, const void* q, int64_t ldq,
                                             const int32_t* tok_seq, const int64_t* positions, const int32_t* block_tables,
                                             int32_t table_cap, int32_t block_size, const void* cache, int64_t cache_row, int32_t n,
                                             int32_t heads, int32_t dim, int32_t rot_dim, int32_t kv_rank, float scale,
                                             int32_t window, const float* sinks, const float* gate, int64_t ldg, void* workspace,
                                             size_t workspace_bytes, int32_t dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && heads > 0 && dim >= 0 && rot_dim >= 0 && kv_rank > 0 && kv_rank <= 1024 && table_cap > 0 && block_size > 0,
                  NVLLM_ERR_ARG, "latent_attention: sizes (kv_rank <= 1024)");
  NVLLM_CHECK_ARG(dtype == NVLLM_BF16 || dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "latent_attention: dtype %d", dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(out && q_abs && (q || rot_dim == 0) && tok_seq && positions && block_tables && cache, NVLLM_ERR_ARG, "latent_attention: NULL");
  const AttnArgs a{out, ldo, q_abs, ldqa, q ? q : q_abs, ldq, tok_seq, positions, block_tables, table_cap, block_size, cache, cache_row,
                   n, heads, dim, rot_dim, kv_rank, scale, window > 0 ? window : 0, sinks, gate, ldg, 1, static_cast<float*>(workspace)};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // bf16 caches with a 16-byte row pitch and kv_rank <= 512 run on the tensor cores (NVLLM_LATENT_MMA=0: the CUDA-core kernel)
  const int dp16 = (static_cast<int>(cache_row) + 15) / 16 * 16;
  if (dtype == NVLLM_BF16 && knobs().latent_mma != 0 && kv_rank <= 512 && cache_row % 8 == 0 && dp16 <= 704 &&
      (reinterpret_cast<uintptr_t>(cache) & 15u) == 0) {
    // Single tokens with a bounded key range (a window) and fewer CTAs than SMs: split every token's key tiles over up to 4
    // CTAs, as many as fill the SMs once and leave each at least eight tiles; the partials meet in latent_attn_merge_kernel.
    // (Measured, 64 tokens x 16 heads, rank 512: a window of 2048 keys 118 -> 79 us; at 512 keys the second launch costs what
    // the shorter loop saves, 39 -> 37 us, so short windows stay on one CTA.)
    AttnArgs b = a;
    if (workspace != nullptr && n <= 256 && window > 0) {
      const int64_t ctas = static_cast<int64_t>(n) * ((heads + 15) / 16);
      int splits = static_cast<int>(sm_count() / (ctas > 0 ? ctas : 1));
      const int tiles = (window + 2 * kMmaKeys - 2) / kMmaKeys;   // tiles a window can touch
      splits = splits > 4 ? 4 : splits;
      splits = splits > tiles / 8 ? tiles / 8 : splits;
      if (splits > 1 && static_cast<size_t>(n) * heads * splits * (kv_rank + 2) * sizeof(float) <= workspace_bytes) b.splits = splits;
    }
    if (kv_rank <= 128) return launch_attn_mma<1>(b, st);
    if (kv_rank <= 256) return launch_attn_mma<2>(b, st);
    if (kv_rank <= 384) return launch_attn_mma<3>(b, st);
    return launch_attn_mma<4>(b, st);
  }
  return dtype == NVLLM_BF16 ? dispatch_attn<bf16>(a, st) : dispatch_attn<float>(a, st);
}
