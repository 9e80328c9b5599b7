// moe.cu — routing side of a mixture-of-experts feed-forward, all on the device with static shapes (legal inside a CUDA
// graph): softmax router with an additive selection bias, top-k choice, weight normalisation, identity experts, the
// counting sort that groups (token, slot) assignments by expert into 32-row tiles (nvllm_linear_grouped) or 128-row tiles
// (nvllm_gemm_bf16_grouped), and the
// weighted combine.  Everything here is f32 arithmetic.
//
//   s = softmax(z) over all router outputs (real experts first, then identity experts)
//   chosen = the `top` largest of s + bias (ties: lowest index);  w_k = s[chosen_k] / (sum_k s[chosen_k] + 1e-20) * scale
//   out[t] = sum_k w_k * (chosen_k < experts ? expert_out[row of (t, k)] : x[t]) + shared[t]
#include "common.cuh"

namespace nvllm {
namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// One warp per token; the warp's scores live in shared memory ([warps][2][e_total]).
__global__ void __launch_bounds__(128) moe_route_kernel(int32_t* __restrict__ idx, float* __restrict__ wts,
                                                        const float* __restrict__ logits, const float* __restrict__ bias,
                                                        int n, int e_total, int top, float scale) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= n) return;
  float* s = sm + static_cast<size_t>(warp) * 2 * e_total;
  float* c = s + e_total;
  const float* z = logits + static_cast<int64_t>(t) * e_total;
  float mx = -INFINITY;
  for (int e = lane; e < e_total; e += 32) mx = fmaxf(mx, z[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < e_total; e += 32) { const float v = expf(z[e] - mx); s[e] = v; sum += v; }
  sum = warp_sum(sum);
  for (int e = lane; e < e_total; e += 32) { const float v = s[e] / sum; s[e] = v; c[e] = v + (bias ? bias[e] : 0.f); }
  __syncwarp();
  float wsum = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < e_total; e += 32) {
      const float v = c[e];
      if (v > best) { best = v; bi = e; }   // ascending e per lane: the first maximum wins
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (bi == 0x7fffffff) bi = 0;  // every score NaN / -inf: degenerate, keep indices valid
    if (lane == 0) {
      idx[static_cast<int64_t>(t) * top + k] = bi;
      wts[static_cast<int64_t>(t) * top + k] = s[bi];
      c[bi] = -INFINITY;
    }
    wsum += s[bi];
    __syncwarp();
  }
  for (int k = lane; k < top; k += 32) {
    const int64_t o = static_cast<int64_t>(t) * top + k;
    wts[o] = wts[o] / (wsum + 1e-20f) * scale;
  }
}

// Routing on the logits themselves: z = logits + bias; the `top` largest z (ties: lowest index); the weights are the softmax
// over the chosen z alone.  One warp per token; z lives in shared memory ([warps][e_total]).
__global__ void __launch_bounds__(128) moe_route_logits_kernel(int32_t* __restrict__ idx, float* __restrict__ wts,
                                                               const float* __restrict__ logits, const float* __restrict__ bias,
                                                               int64_t ld, int n, int e_total, int top) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= n) return;
  float* c = sm + static_cast<size_t>(warp) * e_total;
  const float* z = logits + static_cast<int64_t>(t) * ld;
  for (int e = lane; e < e_total; e += 32) c[e] = z[e] + (bias ? bias[e] : 0.f);
  __syncwarp();
  float first = 0.f, wsum = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < e_total; e += 32) {
      const float v = c[e];
      if (v > best) { best = v; bi = e; }   // ascending e per lane: the first maximum wins
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (bi == 0x7fffffff) { bi = 0; best = first; }  // every score NaN / -inf: degenerate, keep indices valid
    if (k == 0) first = best;                        // the largest of all: the softmax's reference point
    const float w = expf(best - first);
    if (lane == 0) {
      idx[static_cast<int64_t>(t) * top + k] = bi;
      wts[static_cast<int64_t>(t) * top + k] = w;
      c[bi] = -INFINITY;
    }
    wsum += w;
    __syncwarp();
  }
  for (int k = lane; k < top; k += 32) {
    const int64_t o = static_cast<int64_t>(t) * top + k;
    wts[o] = wts[o] / wsum;
  }
}

// Counting sort of the assignments by expert, one CTA.  Output layout: expert e owns rows [off[e], off[e] + cnt[e]) of the
// grouped buffers, off[e] a multiple of the tile height so that no tile spans two experts.
//   row_token[r]  token whose activations row r reads (-1: padding)
//   tile_expert[i] expert of tile i (-1: unused tile)
//   slot_row[t*top + k] row of assignment (t, k), or -1 when it chose an identity expert
__global__ void __launch_bounds__(1024) moe_sort_kernel(int32_t* __restrict__ row_token, int32_t* __restrict__ tile_expert,
                                                        int32_t* __restrict__ slot_row, const int32_t* __restrict__ idx,
                                                        int n_assign, int top, int experts, int max_rows, int tile) {
  extern __shared__ int32_t sh[];
  int32_t* cnt = sh;             // [experts]
  int32_t* off = sh + experts;   // [experts + 1]
  for (int e = threadIdx.x; e < experts; e += blockDim.x) cnt[e] = 0;
  for (int r = threadIdx.x; r < max_rows; r += blockDim.x) row_token[r] = -1;
  for (int i = threadIdx.x; i < max_rows / tile; i += blockDim.x) tile_expert[i] = -1;
  __syncthreads();
  for (int a = threadIdx.x; a < n_assign; a += blockDim.x) {
    const int e = idx[a];
    slot_row[a] = e < experts ? atomicAdd(&cnt[e], 1) : -1;   // rank inside the expert (any order: rows are independent)
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0;
    for (int e = 0; e < experts; ++e) {
      off[e] = o;
      const int tiles = (cnt[e] + tile - 1) / tile;
      for (int i = 0; i < tiles; ++i) tile_expert[o / tile + i] = e;
      o += tiles * tile;
    }
    off[experts] = o;
  }
  __syncthreads();
  for (int a = threadIdx.x; a < n_assign; a += blockDim.x) {
    const int e = idx[a];
    if (e < experts) {
      const int r = off[e] + slot_row[a];
      slot_row[a] = r;
      row_token[r] = a / top;
    }
  }
}

template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, const T* __restrict__ expert_out, const T* __restrict__ x,
                                   const T* __restrict__ shared_out, const int32_t* __restrict__ idx,
                                   const float* __restrict__ wts, const int32_t* __restrict__ slot_row, int n, int hidden,
                                   int top, int experts) {
  const int64_t total = static_cast<int64_t>(n) * hidden;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / hidden;
    const int c = static_cast<int>(i - t * hidden);
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int64_t a = t * top + k;
      const int r = slot_row[a];
      const float v = r >= 0 ? ldf(expert_out + static_cast<int64_t>(r) * hidden + c) : ldf(x + i);
      acc = fmaf(wts[a], v, acc);
    }
    if (shared_out) acc += ldf(shared_out + i);
    stf(out + i, acc);
  }
}


// 8 bf16 values <-> one 16-byte vector
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
  f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

__global__ void moe_combine_vec8_kernel(bf16* __restrict__ out, const bf16* __restrict__ expert_out, const bf16* __restrict__ x,
                                        const bf16* __restrict__ shared_out, const float* __restrict__ wts,
                                        const int32_t* __restrict__ slot_row, int n, int hidden8, int top) {
  const int64_t total = static_cast<int64_t>(n) * hidden8;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / hidden8, c = i - t * hidden8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, v[8];
    for (int k = 0; k < top; ++k) {
      const int64_t a = t * top + k;
      const int r = slot_row[a];
      unpack8(r >= 0 ? reinterpret_cast<const uint4*>(expert_out)[static_cast<int64_t>(r) * hidden8 + c] : reinterpret_cast<const uint4*>(x)[i], v);
      const float w = wts[a];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(w, v[j], acc[j]);
    }
    if (shared_out) {
      unpack8(reinterpret_cast<const uint4*>(shared_out)[i], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
    reinterpret_cast<uint4*>(out)[i] = pack8(acc);
  }
}

// Routing without a router: row ids[t] of a table names the experts of token t, each with the same weight.
__global__ void moe_table_route_kernel(int32_t* __restrict__ topk_idx, float* __restrict__ topk_w, const int32_t* __restrict__ table,
                                       const int64_t* __restrict__ ids, int64_t n, int top, int rows, float weight) {
  const int64_t total = n * top;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / top;
    int64_t id = ids[t];
    id = id < 0 ? 0 : (id >= rows ? rows - 1 : id);
    topk_idx[i] = table[id * top + (i - t * top)];
    topk_w[i] = weight;
  }
}

}  // namespace
}  // namespace nvllm

using namespace nvllm;

extern "C" int nvllm_moe_table_route(int32_t* topk_idx, float* topk_w, const int32_t* table, const int64_t* ids, int32_t n,
                                     int32_t top, int32_t table_rows, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && top > 0 && table_rows > 0, NVLLM_ERR_ARG, "moe_table_route: n=%d top=%d rows=%d", n, top, table_rows);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(topk_idx && topk_w && table && ids, NVLLM_ERR_ARG, "moe_table_route: NULL");
  const int64_t total = static_cast<int64_t>(n) * top;
  moe_table_route_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(topk_idx, topk_w, table, ids, n,
                                                                                                               top, table_rows, 1.0f / top);
  NVLLM_LAUNCH_CHECK("moe_table_route_kernel");
  return 0;
}

extern "C" int nvllm_moe_route(int32_t* topk_idx, float* topk_w, const float* logits, const float* bias, int32_t n,
                               int32_t e_total, int32_t top, float scale, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && e_total > 0 && top > 0 && top <= e_total && e_total <= 1536, NVLLM_ERR_ARG,
                  "moe_route: n=%d outputs=%d top=%d", n, e_total, top);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(topk_idx && topk_w && logits, NVLLM_ERR_ARG, "moe_route: NULL");
  const size_t smem = static_cast<size_t>(4) * 2 * e_total * sizeof(float);
  moe_route_kernel<<<(n + 3) / 4, 128, smem, static_cast<cudaStream_t>(stream)>>>(topk_idx, topk_w, logits, bias, n, e_total, top, scale);
  NVLLM_LAUNCH_CHECK("moe_route_kernel");
  return 0;
}

extern "C" int nvllm_moe_route_logits(int32_t* topk_idx, float* topk_w, const float* logits, int64_t ld, const float* bias, int32_t n,
                                      int32_t experts, int32_t top, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && experts > 0 && top > 0 && top <= experts && experts <= 3072 && ld >= experts, NVLLM_ERR_ARG,
                  "moe_route_logits: n=%d experts=%d top=%d", n, experts, top);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(topk_idx && topk_w && logits, NVLLM_ERR_ARG, "moe_route_logits: NULL");
  const size_t smem = static_cast<size_t>(4) * experts * sizeof(float);
  moe_route_logits_kernel<<<(n + 3) / 4, 128, smem, static_cast<cudaStream_t>(stream)>>>(topk_idx, topk_w, logits, bias, ld, n, experts, top);
  NVLLM_LAUNCH_CHECK("moe_route_logits_kernel");
  return 0;
}

extern "C" int32_t nvllm_moe_max_rows(int32_t n_tokens, int32_t top, int32_t experts, int32_t tile_rows) {
  if (tile_rows <= 0) return 0;
  const int64_t a = static_cast<int64_t>(n_tokens) * top + static_cast<int64_t>(experts) * (tile_rows - 1);
  return static_cast<int32_t>((a + tile_rows - 1) / tile_rows * tile_rows);
}

extern "C" int nvllm_moe_sort(int32_t* row_token, int32_t* tile_expert, int32_t* slot_row, const int32_t* topk_idx,
                              int32_t n, int32_t top, int32_t experts, int32_t max_rows, int32_t tile_rows, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && top > 0 && experts >= 0 && experts <= 8192 && (tile_rows == 32 || tile_rows == 128) &&
                      max_rows % tile_rows == 0 && max_rows >= nvllm_moe_max_rows(n, top, experts, tile_rows), NVLLM_ERR_ARG,
                  "moe_sort: n=%d top=%d experts=%d max_rows=%d tile_rows=%d", n, top, experts, max_rows, tile_rows);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(row_token && tile_expert && slot_row && topk_idx, NVLLM_ERR_ARG, "moe_sort: NULL");
  const size_t smem = (2 * static_cast<size_t>(experts) + 1) * sizeof(int32_t);
  moe_sort_kernel<<<1, 1024, smem, static_cast<cudaStream_t>(stream)>>>(row_token, tile_expert, slot_row, topk_idx, n * top, top,
                                                                      experts, max_rows, tile_rows);
  NVLLM_LAUNCH_CHECK("moe_sort_kernel");
  return 0;
}

extern "C" int nvllm_moe_combine(void* out, const void* expert_out, const void* x, const void* shared_out,
                                 const int32_t* topk_idx, const float* topk_w, const int32_t* slot_row, int32_t n,
                                 int32_t hidden, int32_t top, int32_t experts, int32_t dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && hidden > 0 && top > 0, NVLLM_ERR_ARG, "moe_combine: sizes");
  NVLLM_CHECK_ARG(dtype == NVLLM_BF16 || dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "moe_combine: dtype %d", dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(out && x && topk_idx && topk_w && slot_row && (expert_out || experts == 0), NVLLM_ERR_ARG, "moe_combine: NULL");
  const int64_t total = static_cast<int64_t>(n) * hidden;
  int64_t blocks = (total + 255) / 256;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == NVLLM_BF16 && hidden % 8 == 0 && aligned16(out) && aligned16(expert_out) && aligned16(x) && aligned16(shared_out)) {
    int64_t b8 = (total / 8 + 255) / 256;
    if (b8 > sm_count() * 16) b8 = sm_count() * 16;
    moe_combine_vec8_kernel<<<static_cast<unsigned>(b8), 256, 0, st>>>(static_cast<bf16*>(out), static_cast<const bf16*>(expert_out),
                                                                      static_cast<const bf16*>(x), static_cast<const bf16*>(shared_out),
                                                                      topk_w, slot_row, n, hidden / 8, top);
  } else if (dtype == NVLLM_BF16)
    moe_combine_kernel<bf16><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<bf16*>(out), static_cast<const bf16*>(expert_out), static_cast<const bf16*>(x),
        static_cast<const bf16*>(shared_out), topk_idx, topk_w, slot_row, n, hidden, top, experts);
  else
    moe_combine_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<float*>(out), static_cast<const float*>(expert_out), static_cast<const float*>(x),
        static_cast<const float*>(shared_out), topk_idx, topk_w, slot_row, n, hidden, top, experts);
  NVLLM_LAUNCH_CHECK("moe_combine_kernel");
  return 0;
}
