// linear_any.cu — y = x . w^T for ANY sizes, strides, batch counts and for bf16 or f32 operands (nvllm_linear), plus the
// grouped / gathered variants a mixture-of-experts layer needs (nvllm_linear_grouped) and the gated pair with its
// activation in the epilogue (GLU).  Dense bf16 problems whose shapes meet the tensor-core kernel's rules (k % 64, n % 8,
// 16-byte rows) are forwarded to nvllm_gemm_bf16 (tcgen05); everything else — odd sizes, per-head batches, expert groups,
// true 32-bit models — runs on the CUDA-core tile kernel below (bf16 problems with 16-byte rows: on an mma.sync tile kernel): 32 x 64 output tile, 32-wide k steps staged in shared
// memory as f32, f32 accumulation in ascending k order, so a row's result never depends on which other rows are in the
// batch.
#include "common.cuh"

namespace nvllm {
namespace {

struct LinArgs {
  void* y; const void* x; const void* w;
  int M, N, K;
  int64_t ldx, ldw, ldy, bsx, bsw, bsy;
  const int32_t* row_src;     // gathered rows of x (row i of the problem reads x[row_src[i]]; < 0 = zero row, not written)
  const int32_t* tile_group;  // group (expert) of every 32-row tile; < 0 = tile unused.  w += group * bsw
  int64_t up_off;             // GLU: element offset of the `up` rows relative to the `gate` rows inside w
  float limit;                // GLU clamp
  int act;                    // epilogue of the plain product: 0 none, 2 relu(v)^2
};

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int BM = 32, BN = 64, BK = 32;

// GLU epilogue of the gated feed-forward used by the mixture-of-experts layers:
//   g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(1.702 g) * (u + 1)
__device__ __forceinline__ float glu_clamped(float g, float u, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * (1.0f / (1.0f + expf(-1.702f * g))) * (u + 1.0f);
}

template <typename TI, typename TO, bool GLU>
__global__ void __launch_bounds__(256) linear_tile_kernel(const LinArgs a) {
  __shared__ float xs[BM][BK + 1];
  __shared__ float ws[BN][BK + 1];
  __shared__ float us[GLU ? BN : 1][BK + 1];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  int group = 0;
  if (a.tile_group != nullptr) {
    group = a.tile_group[blockIdx.y];
    if (group < 0) return;
  }
  const int b = blockIdx.z;
  const TI* x = static_cast<const TI*>(a.x) + b * a.bsx;
  const TI* w = static_cast<const TI*>(a.w) + (b + group) * a.bsw;
  TO* y = static_cast<TO*>(a.y) + b * a.bsy;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[2][4], acu[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = acu[i][j] = 0.f;
  // each thread stages 4 elements of x and 8 (16 with GLU) of w per k step: row = e / BK, col = e % BK
  for (int k0 = 0; k0 < a.K; k0 += BK) {
#pragma unroll
    for (int e = tid; e < BM * BK; e += 256) {
      const int r = e / BK, c = e % BK, m = m0 + r, k = k0 + c;
      float v = 0.f;
      if (m < a.M && k < a.K) {
        const int64_t src = a.row_src ? a.row_src[m] : m;
        if (src >= 0) v = ldf(x + src * a.ldx + k);
      }
      xs[r][c] = v;
    }
#pragma unroll
    for (int e = tid; e < BN * BK; e += 256) {
      const int r = e / BK, c = e % BK, n = n0 + r, k = k0 + c;
      const bool ok = n < a.N && k < a.K;
      ws[r][c] = ok ? ldf(w + static_cast<int64_t>(n) * a.ldw + k) : 0.f;
      if (GLU) us[r][c] = ok ? ldf(w + a.up_off + static_cast<int64_t>(n) * a.ldw + k) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < BK; ++kk) {
      const float x0 = xs[ty * 2][kk], x1 = xs[ty * 2 + 1][kk];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float wv = ws[tx + 16 * j][kk];
        acc[0][j] = fmaf(x0, wv, acc[0][j]);
        acc[1][j] = fmaf(x1, wv, acc[1][j]);
        if (GLU) {
          const float uv = us[tx + 16 * j][kk];
          acu[0][j] = fmaf(x0, uv, acu[0][j]);
          acu[1][j] = fmaf(x1, uv, acu[1][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = m0 + ty * 2 + i;
    if (m >= a.M || (a.row_src && a.row_src[m] < 0)) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n >= a.N) continue;
      float v = acc[i][j];
      if (GLU) {
        // bf16 models round gate and up to bf16 before the activation, as a separate projection would have
        float g = v, u = acu[i][j];
        if (sizeof(TI) == 2) { g = __bfloat162float(__float2bfloat16_rn(g)); u = __bfloat162float(__float2bfloat16_rn(u)); }
        v = a.act == 3 ? g / (1.0f + expf(-g)) * u : glu_clamped(g, u, a.limit);
      } else if (a.act == 2) {
        if (sizeof(TI) == 2) v = __bfloat162float(__float2bfloat16_rn(v));
        v = fmaxf(v, 0.f);
        v *= v;
      }
      stf(y + static_cast<int64_t>(m) * a.ldy + n, v);
    }
  }
}

template <typename T>
__global__ void glu_clamped_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int64_t n, int ff, float limit) {
  const int64_t total = n * ff;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / ff, c = i - r * ff;
    stf(out + i, glu_clamped(ldf(gate_up + r * 2 * ff + c), ldf(gate_up + r * 2 * ff + ff + c), limit));
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

__global__ void glu_clamped_vec8_kernel(bf16* __restrict__ out, const bf16* __restrict__ gate_up, int64_t n, int ff8, float limit) {
  const int64_t total = n * ff8;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / ff8, c = i - r * ff8;
    float g[8], u[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(gate_up)[r * 2 * ff8 + c], g);
    unpack8(reinterpret_cast<const uint4*>(gate_up)[r * 2 * ff8 + ff8 + c], u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = glu_clamped(g[j], u[j], limit);
    reinterpret_cast<uint4*>(out)[i] = pack8(o);
  }
}

// softplus without overflow: max(x, 0) + log1p(exp(-|x|))
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// kind 0: out[i, c] = silu(in[i, c]) * in[i, ff + c] (in: [n, 2 ff]);  kind 1: out[i, c] = relu(in[i, c])^2 (in: [n, ff]);
// kind 2: out[i, c] = xielu(in[i, c]) with the two learned numbers params[0..1] (in: [n, ff]):
//         z > 0: softplus(p0) z^2 + z / 2;   z <= 0: (1/2 + softplus(p1)) (exp(z) - 1 - z) + z / 2
template <typename T>
__global__ void ff_activation_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t n, int ff, int kind, const float* __restrict__ params) {
  const int64_t total = n * ff;
  const float ap = kind == 2 ? softplus_f(params[0]) : 0.f, an = kind == 2 ? 0.5f + softplus_f(params[1]) : 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / ff, c = i - r * ff;
    float v;
    if (kind == 0) {
      const float g = ldf(in + r * 2 * ff + c);
      v = g / (1.0f + expf(-g)) * ldf(in + r * 2 * ff + ff + c);
    } else if (kind == 2) {
      const float z = ldf(in + i);
      v = z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(an, expm1f(z) - z, 0.5f * z);
    } else {
      v = fmaxf(ldf(in + i), 0.f);
      v *= v;
    }
    stf(out + i, v);
  }
}

// The same for bf16 rows of 16-byte multiples: 8 values per thread and access, no division per element.
__global__ void __launch_bounds__(256) ff_activation_vec8_kernel(bf16* __restrict__ out, const bf16* __restrict__ in, int64_t n, int ff8, int kind,
                                                                 const float* __restrict__ params) {
  const int64_t total = n * ff8;
  const float ap = kind == 2 ? softplus_f(params[0]) : 0.f, an = kind == 2 ? 0.5f + softplus_f(params[1]) : 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float a[8], o[8];
    if (kind == 0) {
      const int64_t r = i / ff8, c = i - r * ff8;
      float u[8];
      unpack8(ld_nc_16(reinterpret_cast<const uint4*>(in) + r * 2 * ff8 + c), a);
      unpack8(ld_nc_16(reinterpret_cast<const uint4*>(in) + r * 2 * ff8 + ff8 + c), u);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = a[j] / (1.0f + expf(-a[j])) * u[j];
    } else {
      unpack8(ld_nc_16(reinterpret_cast<const uint4*>(in) + i), a);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (kind == 2) o[j] = a[j] > 0.f ? fmaf(ap * a[j], a[j], 0.5f * a[j]) : fmaf(an, expm1f(a[j]) - a[j], 0.5f * a[j]);
        else { const float v = fmaxf(a[j], 0.f); o[j] = v * v; }
      }
    }
    reinterpret_cast<uint4*>(out)[i] = pack8(o);
  }
}

// ---- batched products with few rows on tensor cores (bf16) ------------------------------------------------------------
// Per-head projections while decoding (a handful of tokens times `heads` small weight blocks) and products whose reduction
// size the tcgen05 kernel does not take (k % 64 != 0).  CTA = 64 rows x BN columns of ONE batch item, 4 warps of 16 rows;
// 64-wide k steps of x and w staged with cp.async (16-byte chunks, zero fill past k), double-buffered; mma.sync m16n8k16
// with f32 accumulation in ascending k, so a row never depends on which other rows are in the batch.
constexpr int MK = 64, MS = MK + 8;   // k step and the shared-memory row stride (conflict-free ldmatrix)

template <int BNT, typename TO>
__global__ void __launch_bounds__(128) linear_mma_kernel(const LinArgs a) {
  __shared__ __align__(16) bf16 xs[2][64][MS];
  __shared__ __align__(16) bf16 ws[2][BNT][MS];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq4 = lane & 3;
  const int b = blockIdx.z, m0 = blockIdx.y * 64, n0 = blockIdx.x * BNT;
  const bf16* x = static_cast<const bf16*>(a.x) + b * a.bsx;
  const bf16* w = static_cast<const bf16*>(a.w) + b * a.bsw;
  TO* y = static_cast<TO*>(a.y) + b * a.bsy;
  auto load = [&](int k0, int buf) {
    for (int e = tid; e < (64 + BNT) * (MK / 8); e += 128) {
      const int r = e / (MK / 8), c = (e % (MK / 8)) * 8, k = k0 + c;
      const bool is_x = r < 64;
      const int row = is_x ? m0 + r : n0 + r - 64;
      const bool ok = k < a.K && row < (is_x ? a.M : a.N);
      const bf16* src = is_x ? x + static_cast<int64_t>(row) * a.ldx + k : w + static_cast<int64_t>(row) * a.ldw + k;
      cp_async_16(smem_u32(is_x ? &xs[buf][r][c] : &ws[buf][r - 64][c]), ok ? src : static_cast<const bf16*>(a.x), ok ? 16 : 0);
    }
    cp_async_commit();
  };
  float acc[BNT / 8][4];
#pragma unroll
  for (int i = 0; i < BNT / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  const int nk = (a.K + MK - 1) / MK;
  load(0, 0);
  for (int kt = 0; kt < nk; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < nk) { load((kt + 1) * MK, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const uint32_t xa = smem_u32(&xs[buf][warp * 16 + (lane & 15)][(lane >> 4) * 8]);
    const uint32_t wa = smem_u32(&ws[buf][(lane & 7) + (lane >> 4) * 8][((lane >> 3) & 1) * 8]);
#pragma unroll
    for (int kk = 0; kk < MK / 16; ++kk) {
      uint32_t af[4];
      ldmatrix_x4(af, xa + kk * 32);
#pragma unroll
      for (int np = 0; np < BNT / 16; ++np) {
        uint32_t bw[4];
        ldmatrix_x4(bw, wa + np * 16 * MS * 2 + kk * 32);
        mma_bf16_16816(acc[2 * np], af, bw[0], bw[1]);
        mma_bf16_16816(acc[2 * np + 1], af, bw[2], bw[3]);
      }
    }
    __syncthreads();   // the copy issued in the next iteration overwrites this buffer's partner
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = m0 + warp * 16 + gq + 8 * i;
    if (m >= a.M) continue;
#pragma unroll
    for (int nt = 0; nt < BNT / 8; ++nt)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int n = n0 + nt * 8 + 2 * tq4 + c;
        if (n < a.N) stf(y + static_cast<int64_t>(m) * a.ldy + n, acc[nt][2 * i + c]);
      }
  }
}

inline bool mma_applies(const LinArgs& a) {
  return a.K % 8 == 0 && a.ldx % 8 == 0 && a.ldw % 8 == 0 && a.bsx % 8 == 0 && a.bsw % 8 == 0 && aligned16(a.x) && aligned16(a.w);
}

int launch_mma(const LinArgs& a, int batch, int out_dtype, cudaStream_t st) {
  // narrow tiles while the grid would leave most SMs idle
  const int64_t ctas64 = static_cast<int64_t>((a.N + 63) / 64) * ((a.M + 63) / 64) * batch;
  if (ctas64 >= sm_count() || a.N <= 32) {
    dim3 grid((a.N + 63) / 64, (a.M + 63) / 64, batch);
    if (out_dtype == NVLLM_BF16) linear_mma_kernel<64, bf16><<<grid, 128, 0, st>>>(a);
    else linear_mma_kernel<64, float><<<grid, 128, 0, st>>>(a);
  } else {
    dim3 grid((a.N + 31) / 32, (a.M + 63) / 64, batch);
    if (out_dtype == NVLLM_BF16) linear_mma_kernel<32, bf16><<<grid, 128, 0, st>>>(a);
    else linear_mma_kernel<32, float><<<grid, 128, 0, st>>>(a);
  }
  NVLLM_LAUNCH_CHECK("linear_mma_kernel");
  return 0;
}

template <bool GLU>
int launch_tile(const LinArgs& a, int m_tiles, int batch, int dtype, int out_dtype, cudaStream_t st) {
  dim3 grid((a.N + BN - 1) / BN, m_tiles, batch);
  if (dtype == NVLLM_BF16 && out_dtype == NVLLM_BF16) linear_tile_kernel<bf16, bf16, GLU><<<grid, 256, 0, st>>>(a);
  else if (dtype == NVLLM_BF16) linear_tile_kernel<bf16, float, GLU><<<grid, 256, 0, st>>>(a);
  else if (out_dtype == NVLLM_F32) linear_tile_kernel<float, float, GLU><<<grid, 256, 0, st>>>(a);
  else { set_error("linear: f32 operands need an f32 output"); return NVLLM_ERR_DTYPE; }
  NVLLM_LAUNCH_CHECK("linear_tile_kernel");
  return 0;
}

}  // namespace
}  // namespace nvllm

using namespace nvllm;

extern "C" int nvllm_linear(void* y, const void* x, const void* w, int32_t m, int32_t n, int32_t k, int64_t ldx, int64_t ldw,
                            int64_t ldy, int32_t batch, int64_t bsx, int64_t bsw, int64_t bsy, int32_t dtype,
                            int32_t out_dtype, void* stream) {
  NVLLM_CHECK_ARG(m >= 0 && n > 0 && k > 0 && batch > 0, NVLLM_ERR_ARG, "linear: m=%d n=%d k=%d batch=%d", m, n, k, batch);
  NVLLM_CHECK_ARG(ldx >= k && ldw >= k && ldy >= n, NVLLM_ERR_ARG, "linear: leading dimensions");
  NVLLM_CHECK_ARG((dtype == NVLLM_BF16 || dtype == NVLLM_F32) && (out_dtype == NVLLM_BF16 || out_dtype == NVLLM_F32),
                  NVLLM_ERR_DTYPE, "linear: dtype %d / %d", dtype, out_dtype);
  if (m == 0) return 0;
  NVLLM_CHECK_ARG(y && x && w, NVLLM_ERR_ARG, "linear: NULL");
  // dense bf16 problems that fit the tensor-core kernel's rules go there
  if (dtype == NVLLM_BF16 && batch == 1 && k % 64 == 0 && n % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ldy % 8 == 0 &&
      aligned16(y) && aligned16(x) && aligned16(w))
    return nvllm_gemm_bf16(y, x, w, m, n, k, ldx, ldw, ldy, out_dtype, nullptr, 0, stream);
  LinArgs a{y, x, w, m, n, k, ldx, ldw, ldy, bsx, bsw, bsy, nullptr, nullptr, 0, 0.f, 0};
  // other bf16 problems with 16-byte rows (per-head batches, reduction sizes that are not multiples of 64): mma.sync tiles
  if (dtype == NVLLM_BF16 && knobs().linear_mma && mma_applies(a)) return launch_mma(a, batch, out_dtype, static_cast<cudaStream_t>(stream));
  return launch_tile<false>(a, (m + BM - 1) / BM, batch, dtype, out_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int nvllm_linear_grouped(void* y, const void* x, const void* w, int32_t max_rows, int32_t n, int32_t k,
                                    int64_t ldx, int64_t ldw, int64_t ldy, int64_t group_stride_w, const int32_t* row_src,
                                    const int32_t* tile_group, int32_t glu, float limit, int32_t dtype, int32_t out_dtype,
                                    void* stream) {
  NVLLM_CHECK_ARG(max_rows >= 0 && n > 0 && k > 0 && max_rows % BM == 0, NVLLM_ERR_ARG,
                  "linear_grouped: max_rows=%d (multiple of 32) n=%d k=%d", max_rows, n, k);
  NVLLM_CHECK_ARG((dtype == NVLLM_BF16 || dtype == NVLLM_F32) && (out_dtype == NVLLM_BF16 || out_dtype == NVLLM_F32),
                  NVLLM_ERR_DTYPE, "linear_grouped: dtype %d / %d", dtype, out_dtype);
  if (max_rows == 0) return 0;
  NVLLM_CHECK_ARG(y && x && w, NVLLM_ERR_ARG, "linear_grouped: NULL");
  // GLU: every group's weight block is [gate rows (n) | up rows (n)] x k
  LinArgs a{y, x, w, max_rows, n, k, ldx, ldw, ldy, 0, group_stride_w, 0, row_src, tile_group,
            static_cast<int64_t>(n) * ldw, limit, glu == 2 ? 2 : (glu == 3 ? 3 : 0)};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return (glu == 1 || glu == 3) ? launch_tile<true>(a, max_rows / BM, 1, dtype, out_dtype, st)
             : launch_tile<false>(a, max_rows / BM, 1, dtype, out_dtype, st);
}

extern "C" int nvllm_glu_clamped(void* out, const void* gate_up, int32_t n, int32_t ff, float limit, int32_t dtype,
                                 void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && ff > 0, NVLLM_ERR_ARG, "glu_clamped: n=%d ff=%d", n, ff);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(out && gate_up, NVLLM_ERR_ARG, "glu_clamped: NULL");
  const int64_t total = static_cast<int64_t>(n) * ff;
  int64_t blocks = (total + 255) / 256;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == NVLLM_BF16 && ff % 8 == 0 && aligned16(out) && aligned16(gate_up)) {
    int64_t b8 = (total / 8 + 255) / 256;
    if (b8 > sm_count() * 16) b8 = sm_count() * 16;
    glu_clamped_vec8_kernel<<<static_cast<unsigned>(b8), 256, 0, st>>>(static_cast<bf16*>(out), static_cast<const bf16*>(gate_up), n, ff / 8, limit);
  } else if (dtype == NVLLM_BF16)
    glu_clamped_kernel<bf16><<<static_cast<unsigned>(blocks), 256, 0, st>>>(static_cast<bf16*>(out), static_cast<const bf16*>(gate_up), n, ff, limit);
  else if (dtype == NVLLM_F32)
    glu_clamped_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, st>>>(static_cast<float*>(out), static_cast<const float*>(gate_up), n, ff, limit);
  else NVLLM_CHECK_ARG(false, NVLLM_ERR_DTYPE, "glu_clamped: dtype %d", dtype);
  NVLLM_LAUNCH_CHECK("glu_clamped_kernel");
  return 0;
}

extern "C" int nvllm_ff_activation(void* out, const void* in, int32_t n, int32_t ff, int32_t kind, int32_t dtype, void* stream) {
  NVLLM_CHECK_ARG(kind == 0 || kind == 1, NVLLM_ERR_ARG, "ff_activation: kind=%d", kind);
  return nvllm_ff_activation_params(out, in, n, ff, kind, nullptr, dtype, stream);
}

extern "C" int nvllm_ff_activation_params(void* out, const void* in, int32_t n, int32_t ff, int32_t kind, const float* params, int32_t dtype,
                                          void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && ff > 0 && kind >= 0 && kind <= 2 && (kind != 2 || params != nullptr), NVLLM_ERR_ARG,
                  "ff_activation: n=%d ff=%d kind=%d (kind 2 needs its two parameters)", n, ff, kind);
  NVLLM_CHECK_ARG(dtype == NVLLM_BF16 || dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "ff_activation: dtype %d", dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(out && in, NVLLM_ERR_ARG, "ff_activation: NULL");
  const int64_t total = static_cast<int64_t>(n) * ff;
  int64_t blocks = (total + 255) / 256;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == NVLLM_BF16 && ff % 8 == 0 && aligned16(out) && aligned16(in)) {
    int64_t b8 = (total / 8 + 255) / 256;
    if (b8 > sm_count() * 16) b8 = sm_count() * 16;
    ff_activation_vec8_kernel<<<static_cast<unsigned>(b8), 256, 0, st>>>(static_cast<bf16*>(out), static_cast<const bf16*>(in), n, ff / 8, kind, params);
    NVLLM_LAUNCH_CHECK("ff_activation_vec8_kernel");
    return 0;
  }
  if (dtype == NVLLM_BF16) ff_activation_kernel<bf16><<<static_cast<unsigned>(blocks), 256, 0, st>>>(static_cast<bf16*>(out), static_cast<const bf16*>(in), n, ff, kind, params);
  else ff_activation_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, st>>>(static_cast<float*>(out), static_cast<const float*>(in), n, ff, kind, params);
  NVLLM_LAUNCH_CHECK("ff_activation_kernel");
  return 0;
}
