// rms_norm.cu — RMS norms around an f32 residual stream, and an embedding with a hashed bigram term.
//
//   nvllm_rms_residual_norm   the fused step of a block with a norm before AND after every sublayer:
//                                 h += rms(y) * post_w;   out = rms(h) * pre_w          rms(v) = v / sqrt(mean(v^2) + eps)
//                             (pre_w == NULL: out = h, for blocks whose sublayers read the stream without a norm)
//                             (the sublayer's output norm, the residual add and the next sublayer's input norm in one pass over
//                             the row, as nvllm_dyt_residual_norm does for Dynamic Tanh models)
//   nvllm_rms_norm_rows       rows of an f32 matrix, RMS-normed and weighted, written in the operand type to rows of a
//                             destination chosen by a map (a paged cache's slots) or in place of order
//   nvllm_embedding_stream    h[t] = table[id_t] * scale as f32 and, in the same pass, in the operand type
//   nvllm_embedding_bigram    h[t] = table[id_t] * scale + bigram[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets]; the first
//                             token of a sequence reads the extra row `buckets`.  The token before a portion's first one is
//                             part of the sequence's state (one int32 per state slot).
// Statistics, sums and the stream are f32; y / out / tables are bf16 or f32.
#include "common.cuh"

namespace nvllm {
namespace {

__device__ __forceinline__ float ld_any(const void* p, int dt, int64_t i) {
  return dt == NVLLM_F32 ? static_cast<const float*>(p)[i] : __bfloat162float(static_cast<const bf16*>(p)[i]);
}
template <typename TO>
__device__ __forceinline__ void st_as(TO* p, int64_t i, float v) {
  if (sizeof(TO) == 2) reinterpret_cast<bf16*>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(p)[i] = v;
}

// every thread returns the same sum (fixed order over the warps)
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

// CTA per row; the row lives in shared memory between the passes.
template <typename TO>
__global__ void __launch_bounds__(256) rms_residual_norm_kernel(TO* __restrict__ out, float* __restrict__ h, const void* __restrict__ y, int y_dt,
                                                                const float* __restrict__ post_w, const float* __restrict__ pre_w, int hidden,
                                                                float eps) {
  extern __shared__ float row[];
  __shared__ float red[8];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * hidden;
  float sq = 0.f;
  if (y != nullptr) {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float v = ld_any(y, y_dt, base + c);
      row[c] = v;
      sq = fmaf(v, v, sq);
    }
    const float r = 1.0f / sqrtf(block_sum(sq, red) / hidden + eps);
    sq = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float v = h[base + c] + row[c] * r * post_w[c];
      h[base + c] = v;
      row[c] = v;
      sq = fmaf(v, v, sq);
    }
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float v = h[base + c];
      row[c] = v;
      sq = fmaf(v, v, sq);
    }
  }
  if (out == nullptr) return;
  if (pre_w == nullptr) {   // no norm on the way out: the stream itself in the operand type
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) st_as(out, base + c, row[c]);
    return;
  }
  const float r = 1.0f / sqrtf(block_sum(sq, red) / hidden + eps);
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) st_as(out, base + c, row[c] * r * pre_w[c]);
}

// The same for rows of up to 8192 values in 16-byte vectors: the row stays in registers (one global pass), y and out in f32 or bf16.
template <typename TY, typename TO>
__global__ void __launch_bounds__(256) rms_residual_norm_vec_kernel(TO* __restrict__ out, float* __restrict__ h, const TY* __restrict__ y,
                                                                    const float* __restrict__ post_w, const float* __restrict__ pre_w, int hidden,
                                                                    float eps) {
  __shared__ float red[8];
  const int nv = hidden / 4;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * hidden;
  float4 v[8];
  float sq = 0.f;
  if (y != nullptr) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int c = threadIdx.x + 256 * k;
      if (c < nv) {
        if (sizeof(TY) == 2) {
          const uint2 u = reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(y) + base)[c];
          v[k] = make_float4(bf16_lo(u.x), bf16_hi(u.x), bf16_lo(u.y), bf16_hi(u.y));
        } else {
          v[k] = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(y) + base)[c];
        }
        sq += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
      }
    }
    const float r = 1.0f / sqrtf(block_sum(sq, red) / hidden + eps);
    sq = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int c = threadIdx.x + 256 * k;
      if (c < nv) {
        const float4 hv = reinterpret_cast<const float4*>(h + base)[c], w = reinterpret_cast<const float4*>(post_w)[c];
        v[k] = make_float4(hv.x + v[k].x * r * w.x, hv.y + v[k].y * r * w.y, hv.z + v[k].z * r * w.z, hv.w + v[k].w * r * w.w);
        reinterpret_cast<float4*>(h + base)[c] = v[k];
        sq += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int c = threadIdx.x + 256 * k;
      if (c < nv) {
        v[k] = reinterpret_cast<const float4*>(h + base)[c];
        sq += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
      }
    }
  }
  if (out == nullptr) return;
  const float r = pre_w != nullptr ? 1.0f / sqrtf(block_sum(sq, red) / hidden + eps) : 1.0f;   // pre_w == NULL: the stream itself
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int c = threadIdx.x + 256 * k;
    if (c < nv) {
      const float4 w = pre_w != nullptr ? reinterpret_cast<const float4*>(pre_w)[c] : make_float4(1.f, 1.f, 1.f, 1.f);
      const float4 o = make_float4(v[k].x * r * w.x, v[k].y * r * w.y, v[k].z * r * w.z, v[k].w * r * w.w);
      if (sizeof(TO) == 2) reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(out) + base)[c] = make_uint2(pack_bf16x2(o.x, o.y), pack_bf16x2(o.z, o.w));
      else reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + base)[c] = o;
    }
  }
}

// One warp per row.
template <typename TO>
__global__ void __launch_bounds__(128) rms_norm_rows_kernel(TO* __restrict__ out, int64_t ldo, const float* __restrict__ x, int64_t ldx,
                                                            const float* __restrict__ w, const int32_t* __restrict__ row_map, int n, int cols,
                                                            float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= n) return;
  const int64_t dst = row_map ? row_map[t] : t;
  if (dst < 0) return;
  const float* xr = x + static_cast<int64_t>(t) * ldx;
  float sq = 0.f;
  for (int c = lane; c < cols; c += 32) { const float v = xr[c]; sq = fmaf(v, v, sq); }
  const float r = 1.0f / sqrtf(warp_sum(sq) / cols + eps);
  for (int c = lane; c < cols; c += 32) st_as(out, dst * ldo + c, xr[c] * r * (w ? w[c] : 1.0f));
}

struct BigramArgs {
  float* h;
  const void *table, *bigram;
  const int64_t *ids, *positions;
  const int32_t *tok_seq, *cu_tokens, *seq_slot;
  int32_t* last_token;
  int hidden, vocab, buckets;
  int64_t mul_prev, mul_cur;
  float scale;
};

// CTA per token.  The thread block of a portion's FIRST token is the only one that touches the sequence's state word: it
// reads the token before the portion and then stores the portion's last token.
template <typename T>
__global__ void __launch_bounds__(128) embedding_bigram_kernel(const BigramArgs a) {
  const int t = blockIdx.x;
  const int s = a.tok_seq[t], slot = a.seq_slot[s], c0 = a.cu_tokens[s];
  float* hr = a.h + static_cast<int64_t>(t) * a.hidden;
  if (slot < 0) {  // padding row of a captured batch
    for (int c = threadIdx.x; c < a.hidden; c += blockDim.x) hr[c] = 0.f;
    return;
  }
  int64_t id = a.ids[t];
  id = id < 0 ? 0 : (id >= a.vocab ? a.vocab - 1 : id);
  int64_t row = a.buckets;
  if (a.positions[t] > 0) {
    int64_t prev = t > c0 ? a.ids[t - 1] : a.last_token[slot];
    prev = prev < 0 ? 0 : (prev >= a.vocab ? a.vocab - 1 : prev);
    row = (prev * a.mul_prev + id * a.mul_cur) % a.buckets;
  }
  const T* e = static_cast<const T*>(a.table) + id * a.hidden;
  const T* b = static_cast<const T*>(a.bigram) + row * a.hidden;
  if (sizeof(T) == 2 && a.hidden % 8 == 0 && ((reinterpret_cast<uintptr_t>(a.table) | reinterpret_cast<uintptr_t>(a.bigram) | reinterpret_cast<uintptr_t>(a.h)) & 15u) == 0) {
    for (int c = threadIdx.x; c < a.hidden / 8; c += blockDim.x) {   // 8 bf16 values of each table per step
      const uint4 ev = reinterpret_cast<const uint4*>(e)[c], bv = reinterpret_cast<const uint4*>(b)[c];
      reinterpret_cast<float4*>(hr)[2 * c] = make_float4(fmaf(bf16_lo(ev.x), a.scale, bf16_lo(bv.x)), fmaf(bf16_hi(ev.x), a.scale, bf16_hi(bv.x)),
                                                         fmaf(bf16_lo(ev.y), a.scale, bf16_lo(bv.y)), fmaf(bf16_hi(ev.y), a.scale, bf16_hi(bv.y)));
      reinterpret_cast<float4*>(hr)[2 * c + 1] = make_float4(fmaf(bf16_lo(ev.z), a.scale, bf16_lo(bv.z)), fmaf(bf16_hi(ev.z), a.scale, bf16_hi(bv.z)),
                                                             fmaf(bf16_lo(ev.w), a.scale, bf16_lo(bv.w)), fmaf(bf16_hi(ev.w), a.scale, bf16_hi(bv.w)));
    }
  } else
  for (int c = threadIdx.x; c < a.hidden; c += blockDim.x) hr[c] = fmaf(ld_any(e, sizeof(T) == 2 ? NVLLM_BF16 : NVLLM_F32, c), a.scale,
                                                                        ld_any(b, sizeof(T) == 2 ? NVLLM_BF16 : NVLLM_F32, c));
  if (t == c0) {
    __syncthreads();   // every thread of this block has read last_token[slot]
    if (threadIdx.x == 0) a.last_token[slot] = static_cast<int32_t>(a.ids[a.cu_tokens[s + 1] - 1]);
  }
}


// h[t, :] = table[ids[t], :] * scale as f32, and the same row in the operand type (what the first sublayer of a block without an
// input norm reads).  CTA per token; bf16 tables with rows of 16-byte multiples move 8 values per access.
template <typename TT, typename TO>
__global__ void __launch_bounds__(256) embedding_stream_kernel(float* __restrict__ h, TO* __restrict__ x, const TT* __restrict__ table,
                                                               const int64_t* __restrict__ ids, int hidden, int vocab, float scale, int vec) {
  const int64_t t = blockIdx.x;
  int64_t id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const TT* row = table + id * hidden;
  float* hr = h + t * hidden;
  TO* xr = x + t * hidden;
  if (vec) {   // TT is bf16 here
    for (int c = threadIdx.x; c < hidden / 8; c += 256) {
      const uint4 u = ld_nc_16(reinterpret_cast<const uint4*>(row) + c);
      const float4 a = make_float4(bf16_lo(u.x) * scale, bf16_hi(u.x) * scale, bf16_lo(u.y) * scale, bf16_hi(u.y) * scale);
      const float4 b = make_float4(bf16_lo(u.z) * scale, bf16_hi(u.z) * scale, bf16_lo(u.w) * scale, bf16_hi(u.w) * scale);
      reinterpret_cast<float4*>(hr)[2 * c] = a;
      reinterpret_cast<float4*>(hr)[2 * c + 1] = b;
      if (sizeof(TO) == 2) {
        reinterpret_cast<uint4*>(xr)[c] = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y), pack_bf16x2(b.z, b.w));
      } else {
        reinterpret_cast<float4*>(xr)[2 * c] = a;
        reinterpret_cast<float4*>(xr)[2 * c + 1] = b;
      }
    }
    return;
  }
  for (int c = threadIdx.x; c < hidden; c += 256) {
    const float v = (sizeof(TT) == 2 ? __bfloat162float(reinterpret_cast<const bf16*>(row)[c]) : reinterpret_cast<const float*>(row)[c]) * scale;
    hr[c] = v;
    st_as(xr, c, v);
  }
}

}  // namespace
}  // namespace nvllm

using namespace nvllm;

extern "C" int nvllm_rms_residual_norm(void* out, float* h, const void* y, int32_t y_dtype, const float* post_w, const float* pre_w,
                                       int32_t n, int32_t hidden, float eps, int32_t out_dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && hidden > 0 && hidden <= 48 * 1024, NVLLM_ERR_ARG, "rms_residual_norm: n=%d hidden=%d (<= 49152)", n, hidden);
  NVLLM_CHECK_ARG((out_dtype == NVLLM_BF16 || out_dtype == NVLLM_F32) && (y_dtype == NVLLM_BF16 || y_dtype == NVLLM_F32), NVLLM_ERR_DTYPE,
                  "rms_residual_norm: dtype %d / %d", y_dtype, out_dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(h && (out || y) && (!y || post_w), NVLLM_ERR_ARG, "rms_residual_norm: NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (hidden % 4 == 0 && hidden <= 8192 && aligned16(h) && aligned16(y) && aligned16(out) && aligned16(post_w) && aligned16(pre_w)) {
    const bool yb = y_dtype == NVLLM_BF16, ob = out_dtype == NVLLM_BF16;
    if (yb && ob) rms_residual_norm_vec_kernel<bf16, bf16><<<n, 256, 0, st>>>(static_cast<bf16*>(out), h, static_cast<const bf16*>(y), post_w, pre_w, hidden, eps);
    else if (yb) rms_residual_norm_vec_kernel<bf16, float><<<n, 256, 0, st>>>(static_cast<float*>(out), h, static_cast<const bf16*>(y), post_w, pre_w, hidden, eps);
    else if (ob) rms_residual_norm_vec_kernel<float, bf16><<<n, 256, 0, st>>>(static_cast<bf16*>(out), h, static_cast<const float*>(y), post_w, pre_w, hidden, eps);
    else rms_residual_norm_vec_kernel<float, float><<<n, 256, 0, st>>>(static_cast<float*>(out), h, static_cast<const float*>(y), post_w, pre_w, hidden, eps);
    NVLLM_LAUNCH_CHECK("rms_residual_norm_vec_kernel");
    return 0;
  }
  const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
  if (out_dtype == NVLLM_BF16) {
    NVLLM_SMEM_ATTR_ONCE(rms_residual_norm_kernel<bf16>, 192 * 1024);
    rms_residual_norm_kernel<bf16><<<n, 256, smem, st>>>(static_cast<bf16*>(out), h, y, y_dtype, post_w, pre_w, hidden, eps);
  } else {
    NVLLM_SMEM_ATTR_ONCE(rms_residual_norm_kernel<float>, 192 * 1024);
    rms_residual_norm_kernel<float><<<n, 256, smem, st>>>(static_cast<float*>(out), h, y, y_dtype, post_w, pre_w, hidden, eps);
  }
  NVLLM_LAUNCH_CHECK("rms_residual_norm_kernel");
  return 0;
}

extern "C" int nvllm_rms_norm_rows(void* out, int64_t ldo, const float* x, int64_t ldx, const float* w, const int32_t* row_map, int32_t n,
                                   int32_t cols, float eps, int32_t out_dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && cols > 0 && ldo >= cols && ldx >= cols, NVLLM_ERR_ARG, "rms_norm_rows: n=%d cols=%d", n, cols);
  NVLLM_CHECK_ARG(out_dtype == NVLLM_BF16 || out_dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "rms_norm_rows: dtype %d", out_dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(out && x, NVLLM_ERR_ARG, "rms_norm_rows: NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_dtype == NVLLM_BF16) rms_norm_rows_kernel<bf16><<<(n + 3) / 4, 128, 0, st>>>(static_cast<bf16*>(out), ldo, x, ldx, w, row_map, n, cols, eps);
  else rms_norm_rows_kernel<float><<<(n + 3) / 4, 128, 0, st>>>(static_cast<float*>(out), ldo, x, ldx, w, row_map, n, cols, eps);
  NVLLM_LAUNCH_CHECK("rms_norm_rows_kernel");
  return 0;
}

extern "C" int nvllm_embedding_stream(float* h, void* x, int32_t x_dtype, const void* table, const int64_t* ids, int32_t n, int32_t hidden,
                                      int32_t vocab, float scale, int32_t table_dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && hidden > 0 && vocab > 0, NVLLM_ERR_ARG, "embedding_stream: sizes");
  NVLLM_CHECK_ARG((table_dtype == NVLLM_BF16 || table_dtype == NVLLM_F32) && (x_dtype == NVLLM_BF16 || x_dtype == NVLLM_F32), NVLLM_ERR_DTYPE,
                  "embedding_stream: dtype %d / %d", table_dtype, x_dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(h && x && table && ids, NVLLM_ERR_ARG, "embedding_stream: NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int vec = table_dtype == NVLLM_BF16 && hidden % 8 == 0 && aligned16(h) && aligned16(x) && aligned16(table);
  if (table_dtype == NVLLM_BF16 && x_dtype == NVLLM_BF16)
    embedding_stream_kernel<bf16, bf16><<<n, 256, 0, st>>>(h, static_cast<bf16*>(x), static_cast<const bf16*>(table), ids, hidden, vocab, scale, vec);
  else if (table_dtype == NVLLM_BF16)
    embedding_stream_kernel<bf16, float><<<n, 256, 0, st>>>(h, static_cast<float*>(x), static_cast<const bf16*>(table), ids, hidden, vocab, scale, vec);
  else if (x_dtype == NVLLM_BF16)
    embedding_stream_kernel<float, bf16><<<n, 256, 0, st>>>(h, static_cast<bf16*>(x), static_cast<const float*>(table), ids, hidden, vocab, scale, 0);
  else
    embedding_stream_kernel<float, float><<<n, 256, 0, st>>>(h, static_cast<float*>(x), static_cast<const float*>(table), ids, hidden, vocab, scale, 0);
  NVLLM_LAUNCH_CHECK("embedding_stream_kernel");
  return 0;
}

extern "C" int nvllm_embedding_bigram(float* h, const void* table, const void* bigram, const int64_t* ids, const int64_t* positions,
                                      const int32_t* tok_seq, const int32_t* cu_tokens, const int32_t* seq_slot, int32_t* last_token,
                                      int32_t n, int32_t hidden, int32_t vocab, int32_t buckets, int32_t mul_prev, int32_t mul_cur,
                                      float scale, int32_t table_dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && hidden > 0 && vocab > 0 && buckets > 0, NVLLM_ERR_ARG, "embedding_bigram: n=%d hidden=%d vocab=%d buckets=%d", n,
                  hidden, vocab, buckets);
  NVLLM_CHECK_ARG(table_dtype == NVLLM_BF16 || table_dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "embedding_bigram: dtype %d", table_dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(h && table && bigram && ids && positions && tok_seq && cu_tokens && seq_slot && last_token, NVLLM_ERR_ARG,
                  "embedding_bigram: NULL");
  const BigramArgs a{h, table, bigram, ids, positions, tok_seq, cu_tokens, seq_slot, last_token, hidden, vocab, buckets, mul_prev, mul_cur, scale};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (table_dtype == NVLLM_BF16) embedding_bigram_kernel<bf16><<<n, 128, 0, st>>>(a);
  else embedding_bigram_kernel<float><<<n, 128, 0, st>>>(a);
  NVLLM_LAUNCH_CHECK("embedding_bigram_kernel");
  return 0;
}
