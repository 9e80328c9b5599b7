// capped_attn.cu — grouped-query softmax attention over a paged key / value cache with
//   * no rotary: the only positional signal is a query temperature  1 + coef * ln(floor((p + 1) / every) + 1),
//   * a soft cap on the scores:  s <- cap * tanh(s / cap)   (cap <= 0: none),
//   * an optional output gate:   out *= sigmoid(gate)       (gate: f32 pre-activations, same layout as the output),
//   * key and value sizes that may differ (dim, vdim),
//   * an optional sliding window: position p sees the keys p - window + 1 .. p   (window <= 0: all keys 0 .. p),
//   * optional sinks: a learned number per head whose exponential joins the softmax denominator (no key, no value),
//   * the gate as one number per head instead of one per output value.
// Every query token carries its sequence (a row of the block tables) and its position, so one launch serves whole prompts,
// portions of prompts and single decoded tokens side by side; position p sees the keys 0..p of its sequence.
//
// nvllm_attn_bias_store: the step before it — adds the projection biases, writes the queries in the operand type and the
// keys / values into their cache rows.  nvllm_attn_rope_norm_store: the same step for layers with rotary positions on pairs
// of neighbouring dimensions, a weightless per-head RMS norm after the rotation, and values that are the un-rotated keys.
// Scores, softmax and the accumulation of P.V are f32.
#include "common.cuh"

namespace nvllm {
namespace {

template <typename T> __device__ __forceinline__ float ldv(const T* p);
template <> __device__ __forceinline__ float ldv<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldv<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stv(T* p, float v);
template <> __device__ __forceinline__ void stv<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stv<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// proj row: [q (qn) | k (kn) | v (vn) | ...] f32.  CTA per token.
template <typename T>
__global__ void attn_bias_store_kernel(T* __restrict__ q, int64_t ldq, T* __restrict__ kc, T* __restrict__ vc, int64_t k_row, int64_t v_row,
                                       const float* __restrict__ proj, int64_t ldp, const float* __restrict__ qb,
                                       const float* __restrict__ kb, const float* __restrict__ vb, const int32_t* __restrict__ slots,
                                       int qn, int kn, int vn) {
  const int64_t t = blockIdx.x;
  const float* p = proj + t * ldp;
  for (int c = threadIdx.x; c < qn; c += blockDim.x) stv(q + t * ldq + c, p[c] + (qb ? qb[c] : 0.f));
  const int32_t slot = slots[t];
  if (slot < 0) return;
  for (int c = threadIdx.x; c < kn; c += blockDim.x) stv(kc + slot * k_row + c, p[qn + c] + (kb ? kb[c] : 0.f));
  for (int c = threadIdx.x; c < vn; c += blockDim.x) stv(vc + slot * v_row + c, p[qn + kn + c] + (vb ? vb[c] : 0.f));
}

// The same step for layers whose queries and keys are RMS-normed over the WHOLE projection (all heads of a token at once,
// one weight per column): q = rms(proj_q) * qw in the operand type, k = rms(proj_k) * kw and v into their cache rows.
// kn == 0: the layer has no keys / values of its own (it reads another layer's cache).  CTA per token; statistics f32.
template <typename T>
__global__ void __launch_bounds__(256) attn_wide_norm_store_kernel(T* __restrict__ q, int64_t ldq, T* __restrict__ kc, T* __restrict__ vc,
                                                                   int64_t k_row, int64_t v_row, const float* __restrict__ proj, int64_t ldp,
                                                                   const float* __restrict__ qw, const float* __restrict__ kw,
                                                                   const int32_t* __restrict__ slots, int qn, int kn, int vn, float eps) {
  __shared__ float red[2][8];
  const int64_t t = blockIdx.x;
  const float* p = proj + t * ldp;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  float sq = 0.f, sk = 0.f;
  for (int c = threadIdx.x; c < qn; c += 256) sq = fmaf(p[c], p[c], sq);
  for (int c = threadIdx.x; c < kn; c += 256) sk = fmaf(p[qn + c], p[qn + c], sk);
  sq = warp_sum(sq); sk = warp_sum(sk);
  if (lane == 0) { red[0][wid] = sq; red[1][wid] = sk; }
  __syncthreads();
  sq = sk = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) { sq += red[0][i]; sk += red[1][i]; }   // fixed order: every thread holds the same sums
  const float rq = 1.0f / sqrtf(sq / qn + eps);
  for (int c = threadIdx.x; c < qn; c += 256) stv(q + t * ldq + c, p[c] * rq * (qw ? qw[c] : 1.0f));
  const int32_t slot = slots[t];
  if (slot < 0 || kn == 0) return;
  const float rk = 1.0f / sqrtf(sk / kn + eps);
  for (int c = threadIdx.x; c < kn; c += 256) stv(kc + slot * k_row + c, p[qn + c] * rk * (kw ? kw[c] : 1.0f));
  for (int c = threadIdx.x; c < vn; c += 256) stv(vc + slot * v_row + c, p[qn + kn + c]);
}

struct RopeStoreArgs {
  void* q; int64_t ldq;
  void *kc, *vc; int64_t k_row, v_row;
  const float* proj; int64_t ldp;
  const float *qb, *kb, *vb;
  const int64_t* positions; const float2* table; int rot_dims, max_pos;
  float norm_eps;
  const int32_t* slots;
  int n, heads, kv_heads, dim, vdim, v_from_k;
  int halves;            // pairing of the rotation: 0 = neighbours (2i, 2i + 1); 1 = halves (i, i + rot_dims / 2)
  const float2* vtable;  // non-null: every value head is rotated too, over all of vdim (same pairing), by this table
};

// A warp's head of up to 32 NK values: computed once (value(c)), kept in registers, divided by its root mean square
// (eps > 0) and stored.
template <int NK, typename T, typename F>
__device__ __forceinline__ void head_norm_store(F value, T* dst, int dim, float eps, int lane) {
  float keep[NK], sq = 0.f;
#pragma unroll
  for (int k = 0; k < NK; ++k) {
    const int c = lane + 32 * k;
    keep[k] = c < dim ? value(c) : 0.f;
    sq = fmaf(keep[k], keep[k], sq);
  }
  const float r = eps > 0.f ? 1.0f / sqrtf(warp_sum(sq) / dim + eps) : 1.0f;
#pragma unroll
  for (int k = 0; k < NK; ++k) {
    const int c = lane + 32 * k;
    if (c < dim) stv(dst + c, keep[k] * r);
  }
}

// One warp per (token, head) over the heads [q heads | key heads | value heads].  A query or key head: bias, rotation of the
// pairs (2i, 2i+1) of its first rot_dims values by position * base^(-2i/rot_dims), then (norm_eps > 0) division by the root
// mean square of the whole head; queries go to q, keys to their cache row.  A value head: bias, then its cache row; with
// v_from_k the value head IS the key head as projected (bias added, neither rotated nor normed).
template <typename T>
__global__ void __launch_bounds__(128) attn_rope_norm_store_kernel(const RopeStoreArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = a.heads + a.kv_heads + (a.v_from_k ? 0 : a.kv_heads);
  const int64_t item = static_cast<int64_t>(blockIdx.x) * 4 + warp;
  if (item >= static_cast<int64_t>(a.n) * per) return;
  const int t = static_cast<int>(item / per), hh = static_cast<int>(item % per);
  const float* p = a.proj + static_cast<int64_t>(t) * a.ldp;
  const int32_t slot = a.slots[t];
  const int qn = a.heads * a.dim, kn = a.kv_heads * a.dim;
  if (hh >= a.heads + a.kv_heads) {   // a value head with columns of its own
    if (slot < 0) return;
    const int g = hh - a.heads - a.kv_heads;
    T* dst = static_cast<T*>(a.vc) + static_cast<int64_t>(slot) * a.v_row + static_cast<int64_t>(g) * a.vdim;
    const float* vs = p + qn + kn + g * a.vdim;
    const float* vbias = a.vb ? a.vb + g * a.vdim : nullptr;
    if (a.vtable == nullptr) {
      for (int c = lane; c < a.vdim; c += 32) stv(dst + c, vs[c] + (vbias ? vbias[c] : 0.f));
      return;
    }
    int64_t vp = a.positions[t];
    vp = vp < 0 ? 0 : (vp >= a.max_pos ? a.max_pos - 1 : vp);
    const int hv = a.vdim / 2;
    const float2* vt = a.vtable + vp * hv;
    for (int c = lane; c < a.vdim; c += 32) {
      float v = vs[c] + (vbias ? vbias[c] : 0.f);
      if (c < 2 * hv) {
        const int pc = a.halves ? (c < hv ? c + hv : c - hv) : (c ^ 1);
        const bool second = a.halves ? c >= hv : (c & 1);
        const float o = vs[pc] + (vbias ? vbias[pc] : 0.f);
        const float2 cs = vt[a.halves ? (c < hv ? c : c - hv) : (c >> 1)];
        v = second ? fmaf(v, cs.x, o * cs.y) : fmaf(v, cs.x, -o * cs.y);
      }
      stv(dst + c, v);
    }
    return;
  }
  const bool is_q = hh < a.heads;
  const int h = is_q ? hh : hh - a.heads;
  if (!is_q && slot < 0) return;
  const float* src = p + (is_q ? 0 : qn) + static_cast<int64_t>(h) * a.dim;
  const float* bias = is_q ? a.qb : a.kb;
  if (bias) bias += static_cast<int64_t>(h) * a.dim;
  if (!is_q && a.v_from_k) {
    T* vd = static_cast<T*>(a.vc) + static_cast<int64_t>(slot) * a.v_row + static_cast<int64_t>(h) * a.vdim;
    for (int c = lane; c < a.dim; c += 32) stv(vd + c, src[c] + (bias ? bias[c] : 0.f));
  }
  int64_t pos = a.positions[t];
  pos = pos < 0 ? 0 : (pos >= a.max_pos ? a.max_pos - 1 : pos);
  const float2* tab = a.table + pos * (a.rot_dims / 2);
  T* dst = is_q ? static_cast<T*>(a.q) + static_cast<int64_t>(t) * a.ldq + static_cast<int64_t>(h) * a.dim
                : static_cast<T*>(a.kc) + static_cast<int64_t>(slot) * a.k_row + static_cast<int64_t>(h) * a.dim;
  // two passes over the head (sum of squares, then the store); the rotation is recomputed, nothing is staged
  auto value = [&](int c) {
    float v = src[c] + (bias ? bias[c] : 0.f);
    if (c < a.rot_dims) {
      const int hr = a.rot_dims / 2;
      const int pc = a.halves ? (c < hr ? c + hr : c - hr) : (c ^ 1);
      const bool second = a.halves ? c >= hr : (c & 1);
      const float o = src[pc] + (bias ? bias[pc] : 0.f);
      const float2 cs = tab[a.halves ? (c < hr ? c : c - hr) : (c >> 1)];
      v = second ? fmaf(v, cs.x, o * cs.y) : fmaf(v, cs.x, -o * cs.y);   // (u cos - v sin, v cos + u sin)
    }
    return v;
  };
  float r = 1.0f;
  // heads of up to 512 values stay in registers (one pass over the projection), in the smallest unrolled size that holds them
  if (a.dim <= 64) { head_norm_store<2>(value, dst, a.dim, a.norm_eps, lane); return; }
  if (a.dim <= 128) { head_norm_store<4>(value, dst, a.dim, a.norm_eps, lane); return; }
  if (a.dim <= 256) { head_norm_store<8>(value, dst, a.dim, a.norm_eps, lane); return; }
  if (a.dim <= 512) { head_norm_store<16>(value, dst, a.dim, a.norm_eps, lane); return; }
  if (a.norm_eps > 0.f) {
    float sq = 0.f;
    for (int c = lane; c < a.dim; c += 32) { const float v = value(c); sq = fmaf(v, v, sq); }
    r = 1.0f / sqrtf(warp_sum(sq) / a.dim + a.norm_eps);
  }
  for (int c = lane; c < a.dim; c += 32) stv(dst + c, value(c) * r);
}

// The same with 16-byte accesses (dim a multiple of 4, at most 512; aligned rows): the head stays in registers, one pass.
template <typename T>
__global__ void __launch_bounds__(128) attn_rope_norm_store_vec_kernel(const RopeStoreArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = a.heads + a.kv_heads;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * 4 + warp;
  if (item >= static_cast<int64_t>(a.n) * per) return;
  const int t = static_cast<int>(item / per), hh = static_cast<int>(item % per);
  const int32_t slot = a.slots[t];
  const bool is_q = hh < a.heads;
  const int h = is_q ? hh : hh - a.heads;
  if (!is_q && slot < 0) return;
  const float* src = a.proj + static_cast<int64_t>(t) * a.ldp + (is_q ? 0 : a.heads * a.dim) + static_cast<int64_t>(h) * a.dim;
  const float* bias = is_q ? a.qb : a.kb;
  if (bias) bias += static_cast<int64_t>(h) * a.dim;
  int64_t pos = a.positions[t];
  pos = pos < 0 ? 0 : (pos >= a.max_pos ? a.max_pos - 1 : pos);
  const float2* tab = a.table + pos * (a.rot_dims / 2);
  const int nv = a.dim / 4;
  float4 v[4];
  float sq = 0.f;
  auto store4 = [](T* dst, const float4& o) {
    if (sizeof(T) == 2) *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(o.x, o.y), pack_bf16x2(o.z, o.w));
    else *reinterpret_cast<float4*>(dst) = o;
  };
  T* vd = (!is_q && a.v_from_k) ? static_cast<T*>(a.vc) + static_cast<int64_t>(slot) * a.v_row + static_cast<int64_t>(h) * a.vdim : nullptr;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = lane + 32 * k;
    if (c < nv) {
      float4 x = reinterpret_cast<const float4*>(src)[c];
      if (bias) { const float4 b = reinterpret_cast<const float4*>(bias)[c]; x.x += b.x; x.y += b.y; x.z += b.z; x.w += b.w; }
      if (vd) store4(vd + 4 * c, x);                       // the value is the key as projected
      if (4 * c < a.rot_dims) { const float2 cs = tab[2 * c]; const float u = x.x, w = x.y; x.x = fmaf(u, cs.x, -w * cs.y); x.y = fmaf(w, cs.x, u * cs.y); }
      if (4 * c + 2 < a.rot_dims) { const float2 cs = tab[2 * c + 1]; const float u = x.z, w = x.w; x.z = fmaf(u, cs.x, -w * cs.y); x.w = fmaf(w, cs.x, u * cs.y); }
      v[k] = x;
      sq += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
  }
  const float r = a.norm_eps > 0.f ? 1.0f / sqrtf(warp_sum(sq) / a.dim + a.norm_eps) : 1.0f;
  T* dst = is_q ? static_cast<T*>(a.q) + static_cast<int64_t>(t) * a.ldq + static_cast<int64_t>(h) * a.dim
                : static_cast<T*>(a.kc) + static_cast<int64_t>(slot) * a.k_row + static_cast<int64_t>(h) * a.dim;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = lane + 32 * k;
    if (c < nv) store4(dst + 4 * c, make_float4(v[k].x * r, v[k].y * r, v[k].z * r, v[k].w * r));
  }
}

// The halves pairing with 16-byte accesses: no biases, heads of 4 .. 512 values whose rotated part (and vdim, when the values
// are rotated) is a multiple of 8, aligned rows.  A lane owns chunks of 4 neighbouring values; the partner of a chunk in the
// rotation is the chunk half the rotated part away (read again: it is in L1), so nothing crosses lanes but the norm's sum.
template <typename T>
__global__ void __launch_bounds__(128) attn_rotary_store_halves_vec_kernel(const RopeStoreArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = a.heads + 2 * a.kv_heads;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * 4 + warp;
  if (item >= static_cast<int64_t>(a.n) * per) return;
  const int t = static_cast<int>(item / per), hh = static_cast<int>(item % per);
  const int32_t slot = a.slots[t];
  const bool is_q = hh < a.heads, is_v = hh >= a.heads + a.kv_heads;
  if (!is_q && slot < 0) return;
  const int h = is_q ? hh : (is_v ? hh - a.heads - a.kv_heads : hh - a.heads);
  const int qn = a.heads * a.dim, kn = a.kv_heads * a.dim;
  const int size = is_v ? a.vdim : a.dim, rot = is_v ? (a.vtable ? a.vdim : 0) : a.rot_dims, hr4 = rot / 8;   // chunks in half the rotated part
  const float4* src = reinterpret_cast<const float4*>(a.proj + static_cast<int64_t>(t) * a.ldp + (is_q ? 0 : (is_v ? qn + kn : qn)) +
                                                      static_cast<int64_t>(h) * size);
  int64_t pos = a.positions[t];
  pos = pos < 0 ? 0 : (pos >= a.max_pos ? a.max_pos - 1 : pos);
  const float4* tab = reinterpret_cast<const float4*>((is_v ? a.vtable : a.table) + pos * (rot / 2));   // (cos, sin) of two pairs per float4
  T* dst = is_q ? static_cast<T*>(a.q) + static_cast<int64_t>(t) * a.ldq + static_cast<int64_t>(h) * size
                : (is_v ? static_cast<T*>(a.vc) + static_cast<int64_t>(slot) * a.v_row + static_cast<int64_t>(h) * size
                        : static_cast<T*>(a.kc) + static_cast<int64_t>(slot) * a.k_row + static_cast<int64_t>(h) * size);
  const int nv = size / 4;
  float4 v[4];
  float sq = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = lane + 32 * k;
    if (c < nv) {
      float4 x = src[c];
      if (c < 2 * hr4) {
        const bool second = c >= hr4;
        const float4 o = src[second ? c - hr4 : c + hr4];
        const int m = second ? c - hr4 : c;
        const float4 cs0 = tab[2 * m], cs1 = tab[2 * m + 1];
        const float sg = second ? 1.0f : -1.0f;                 // (u cos - v sin, v cos + u sin)
        x.x = fmaf(x.x, cs0.x, sg * o.x * cs0.y); x.y = fmaf(x.y, cs0.z, sg * o.y * cs0.w);
        x.z = fmaf(x.z, cs1.x, sg * o.z * cs1.y); x.w = fmaf(x.w, cs1.z, sg * o.w * cs1.w);
      }
      v[k] = x;
      sq += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
  }
  const float r = (!is_v && a.norm_eps > 0.f) ? 1.0f / sqrtf(warp_sum(sq) / size + a.norm_eps) : 1.0f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = lane + 32 * k;
    if (c < nv) {
      const float4 o = make_float4(v[k].x * r, v[k].y * r, v[k].z * r, v[k].w * r);
      if (sizeof(T) == 2) *reinterpret_cast<uint2*>(dst + 4 * c) = make_uint2(pack_bf16x2(o.x, o.y), pack_bf16x2(o.z, o.w));
      else *reinterpret_cast<float4*>(dst + 4 * c) = o;
    }
  }
}

struct AttnArgs {
  void* out; int64_t ldo;
  const void* q; int64_t ldq;
  const float* gate; int64_t ldg;
  const void *kc, *vc; int64_t k_row, v_row;
  const int32_t* tok_seq; const int64_t* positions; const int32_t* tables;
  int table_cap, block_size, n, heads, kv_heads, dim, vdim;
  float scale, softcap, temp_coef; int temp_every;
  int window; const float* sinks; int gate_per_head;
  const int32_t* dense_cu;   // non-null (and tables null): keys are not paged, key j of sequence s is row dense_cu[s] + j
  // positional options of nvllm_biased_attention (all off when zero / null)
  int chunk;                 // > 0: position p sees only the keys of its own chunk, floor(p / chunk) * chunk .. p
  const float* head_scale;   // [heads]: a factor per head on the scaled score
  const float* dist_bias;    // [heads, dist_rows]: added to the score of key j: dist_bias[h, min(p - j, dist_rows - 1)]
  int dist_rows;
  const float2* out_rot;     // [max_pos, vdim / 2] (cos, sin): every head's output is turned by -p, value m paired with m + vdim / 2
  int max_pos;
  int bias_staged;           // tensor-core kernel: the CTA copies its heads' rows of dist_bias into shared memory first
};

// shared memory the tensor-core kernel may spend on the distance-bias rows of a CTA's heads (two CTAs per SM still fit)
constexpr int kBiasSmemBytes = 9216;

// first key a row at position p sees
__device__ __forceinline__ int first_key(const AttnArgs& a, int p) {
  int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
  if (a.chunk > 0) lo = max(lo, p / a.chunk * a.chunk);
  return lo;
}

constexpr int kMaxVPerLane = 16;  // vdim <= 512

// One warp per (token, head): 32 keys per pass, lane j scores key j (q broadcast from shared memory), the warp shares
// the online-softmax statistics, then every lane accumulates its output dimensions over the 32 keys.
template <typename T>
__global__ void __launch_bounds__(128) capped_attn_warp_kernel(const AttnArgs a) {
  extern __shared__ float qs[];  // [4 warps][max(dim, vdim)]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * 4 + warp;
  if (item >= static_cast<int64_t>(a.n) * a.heads) return;
  const int t = static_cast<int>(item / a.heads), h = static_cast<int>(item % a.heads);
  const int g = h / (a.heads / a.kv_heads);
  float* qw = qs + warp * max(a.dim, a.vdim);
  const int64_t pos = a.positions[t];
  const float temp = 1.0f + a.temp_coef * logf(floorf(static_cast<float>((pos + 1) / a.temp_every)) + 1.0f);
  const float qscale = a.scale * temp * (a.head_scale ? a.head_scale[h] : 1.0f);
  const T* q = static_cast<const T*>(a.q) + t * a.ldq + static_cast<int64_t>(h) * a.dim;
  for (int c = lane; c < a.dim; c += 32) qw[c] = ldv(q + c) * qscale;
  __syncwarp();
  const int32_t* table = a.tables ? a.tables + static_cast<int64_t>(a.tok_seq[t]) * a.table_cap : nullptr;
  const int64_t dense0 = a.dense_cu ? a.dense_cu[a.tok_seq[t]] : 0;
  const T* kc = static_cast<const T*>(a.kc) + static_cast<int64_t>(g) * a.dim;
  const T* vc = static_cast<const T*>(a.vc) + static_cast<int64_t>(g) * a.vdim;
  float m = -INFINITY, l = 0.f, acc[kMaxVPerLane];
#pragma unroll
  for (int i = 0; i < kMaxVPerLane; ++i) acc[i] = 0.f;
  const int nkeys = static_cast<int>(pos) + 1;
  const int first = first_key(a, static_cast<int>(pos));   // passes start at multiples of 32 whatever the window or chunk
  for (int j0 = first & ~31; j0 < nkeys; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    int64_t slot = -1;
    if (j < nkeys && j >= first) {
      const int32_t blk = table ? table[j / a.block_size] : 0;
      if (blk >= 0) {
        slot = table ? static_cast<int64_t>(blk) * a.block_size + j % a.block_size : dense0 + j;
        const T* kr = kc + slot * a.k_row;
        float d = 0.f;
        for (int c = 0; c < a.dim; ++c) d = fmaf(qw[c], ldv(kr + c), d);
        s = a.softcap > 0.f ? a.softcap * tanhf(d / a.softcap) : d;
        if (a.dist_bias) s += a.dist_bias[static_cast<int64_t>(h) * a.dist_rows + min(nkeys - 1 - j, a.dist_rows - 1)];
      }
    }
    const float mt = warp_max(s);
    const float mn = fmaxf(m, mt);
    if (mn == -INFINITY) continue;
    const float corr = expf(m - mn);   // m = -inf on the first pass: 0
    const float p = s == -INFINITY ? 0.f : expf(s - mn);
    l = l * corr + warp_sum(p);
    m = mn;
#pragma unroll
    for (int i = 0; i < kMaxVPerLane; ++i) acc[i] *= corr;
    const int cnt = min(32, nkeys - j0);
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int64_t sj = __shfl_sync(0xffffffffu, slot, jj);
      if (pj == 0.f || sj < 0) continue;
      const T* vr = vc + sj * a.v_row;
#pragma unroll
      for (int i = 0; i < kMaxVPerLane; ++i) {
        const int c = lane + 32 * i;
        if (c < a.vdim) acc[i] = fmaf(pj, ldv(vr + c), acc[i]);
      }
    }
  }
  if (a.sinks) {   // the sink joins the denominator only
    const float sk = a.sinks[h], mn = fmaxf(m, sk), corr = expf(m - mn);
    l = l * corr + expf(sk - mn);
#pragma unroll
    for (int i = 0; i < kMaxVPerLane; ++i) acc[i] *= corr;
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  T* o = static_cast<T*>(a.out) + t * a.ldo + static_cast<int64_t>(h) * a.vdim;
  const float* gt = a.gate ? a.gate + t * a.ldg + (a.gate_per_head ? h : static_cast<int64_t>(h) * a.vdim) : nullptr;
  if (a.out_rot) {   // the head's output turned by -pos: the pairs span lanes, so the row passes through shared memory
    __syncwarp();
#pragma unroll
    for (int i = 0; i < kMaxVPerLane; ++i) {
      const int c = lane + 32 * i;
      if (c < a.vdim) qw[c] = acc[i] * inv;
    }
    __syncwarp();
    const int hf = a.vdim / 2;
    const float2* tab = a.out_rot + (pos < 0 ? 0 : (pos >= a.max_pos ? a.max_pos - 1 : pos)) * hf;
#pragma unroll
    for (int i = 0; i < kMaxVPerLane; ++i) {
      const int c = lane + 32 * i;
      if (c < 2 * hf) {
        const float2 cs = tab[c < hf ? c : c - hf];
        acc[i] = c < hf ? fmaf(qw[c], cs.x, qw[c + hf] * cs.y) : fmaf(qw[c], cs.x, -qw[c - hf] * cs.y);   // (u cos + v sin, v cos - u sin)
      } else if (c < a.vdim) {
        acc[i] = qw[c];
      }
    }
  }
  const float inv_o = a.out_rot ? 1.0f : inv;
#pragma unroll
  for (int i = 0; i < kMaxVPerLane; ++i) {
    const int c = lane + 32 * i;
    if (c < a.vdim) {
      float v = acc[i] * inv_o;
      if (gt) v *= 1.0f / (1.0f + expf(-gt[a.gate_per_head ? 0 : c]));
      stv(o + c, v);
    }
  }
}


// ---- tensor cores (bf16) ------------------------------------------------------------------------------------------
// CTA = 128 rows x one key/value head; a row is a (token, query head of the group) pair, so the heads that share a key /
// value head and up to 128 / group tokens of ONE sequence read every key tile once: whole prompts fill the M dimension with
// tokens, single decoded tokens with the heads of the group (warps whose 16 rows are all empty only help with the copies).
// 8 warps x 16 rows; key tiles of 64 through the block table,
// double-buffered with cp.async; S = Q.K^T and O += P.V on mma.sync m16n8k16 (P stays in registers); scale, temperature,
// cap, mask and the online softmax in f32.  Key tiles start at multiples of 64 from the sequence's first key whatever the
// portion, so a row's result does not depend on how the prompt was cut.  Head sizes are padded to DMAX / VMAX with zeros in
// shared memory.
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kWarps = 8, kRows = 16 * kWarps, kKeys = 64, kThreads = 32 * kWarps;

// tanh(x) = 1 - 2 / (2^(2 x log2 e) + 1): two MUFU operations (ex2, rcp), absolute error ~1e-6; exact at both saturations
// (2^inf -> 1, 2^-inf -> -1).  The one-instruction tanh.approx is 2^-11 relative: too coarse where two scores near the cap
// compete (cap x 5e-4 apart in the exponent).
__device__ __forceinline__ float fast_tanh(float x) { return 1.0f - __fdividef(2.0f, fast_exp2(x * (2.0f * kLog2e)) + 1.0f); }

// One warp's share of a key tile: 16 rows x (16 NP) keys -> S on tensor cores, cap / mask / online softmax in f32, then
// O[:, 0 .. 16 VP) += P . V.  k_addr / v_addr are the warp's ldmatrix lane addresses of its first key (and first value column).
// bias (EXT): per row, the row of the distance-bias table of the row's head (null: none), one value per distance.
template <int DMAX, int VMAX, int NP, int VP, int QS, int VS, bool EXT>
__device__ __forceinline__ void attn_tile(float (&o)[VMAX / 8][4], float (&m)[2], float (&l)[2], uint32_t q_addr, uint32_t k_addr,
                                          uint32_t v_addr, int key0, const int (&pos)[2], const int (&lo)[2], const float (&qscale)[2],
                                          bool capped, float cap2, bool need_mask, int tq4, const float* const (&bias)[2], int dist_rows) {
  float s[2 * NP][4];
#pragma unroll
  for (int i = 0; i < 2 * NP; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < DMAX / 16; ++kk) {
    uint32_t af[4];
    ldmatrix_x4(af, q_addr + kk * 32);
#pragma unroll
    for (int np = 0; np < NP; ++np) {
      uint32_t bk[4];
      ldmatrix_x4(bk, k_addr + np * 16 * QS * 2 + kk * 32);
      mma_bf16_16816(s[2 * np], af, bk[0], bk[1]);
      mma_bf16_16816(s[2 * np + 1], af, bk[2], bk[3]);
    }
  }
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < 2 * NP; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = e >> 1, j = key0 + nt * 8 + 2 * tq4 + (e & 1);
      float v = s[nt][e] * qscale[i];            // with a cap: the score over the cap; without: the score in log2 units
      if (capped) v = cap2 * fast_tanh(v);
      if (EXT) { if (bias[i] != nullptr && j <= pos[i]) v = fmaf(bias[i][min(pos[i] - j, dist_rows - 1)], kLog2e, v); }
      if (need_mask) v = (j <= pos[i] && j >= lo[i]) ? v : -INFINITY;   // lo: the first key of the row's window or chunk
      s[nt][e] = v;
      mx[i] = fmaxf(mx[i], v);
    }
  float corr[2], mu[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
    const float mn = fmaxf(m[i], mx[i]);
    mu[i] = mn == -INFINITY ? 0.f : mn;
    corr[i] = fast_exp2(m[i] - mu[i]);
    m[i] = mn;
    l[i] *= corr[i];
  }
#pragma unroll
  for (int nt = 0; nt < 2 * NP; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float p = fast_exp2(s[nt][e] - mu[e >> 1]);
      s[nt][e] = p;
      l[e >> 1] += p;
    }
  // once a row's running maximum has settled (soon, with capped scores) the factor is exactly 1: skip the rescaling then
  if (!__all_sync(0xffffffffu, corr[0] == 1.0f && corr[1] == 1.0f)) {
#pragma unroll
    for (int i = 0; i < 2 * VP; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
  }
#pragma unroll
  for (int kc2 = 0; kc2 < NP; ++kc2) {
    uint32_t pf[4];
    pf[0] = pack_bf16x2(s[2 * kc2][0], s[2 * kc2][1]); pf[1] = pack_bf16x2(s[2 * kc2][2], s[2 * kc2][3]);
    pf[2] = pack_bf16x2(s[2 * kc2 + 1][0], s[2 * kc2 + 1][1]); pf[3] = pack_bf16x2(s[2 * kc2 + 1][2], s[2 * kc2 + 1][3]);
#pragma unroll
    for (int vp = 0; vp < VP; ++vp) {
      uint32_t bv[4];
      ldmatrix_x4_trans(bv, v_addr + kc2 * 16 * VS * 2 + vp * 32);
      mma_bf16_16816(o[2 * vp], pf, bv[0], bv[1]);
      mma_bf16_16816(o[2 * vp + 1], pf, bv[2], bv[3]);
    }
  }
}

template <int DMAX, int VMAX, bool EXT>
__global__ void __launch_bounds__(kThreads, 2) capped_attn_mma_kernel(const AttnArgs a, const int32_t* __restrict__ cu_tokens, int n_seqs, int tq,
                                                              int group) {
  constexpr int QS = DMAX + 8, VS = VMAX + 8;       // shared-memory row strides (elements): 16-byte rows, conflict-free ldmatrix
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);     // [64][QS]
  bf16* Ks = Qs + kRows * QS;                        // [2][64][QS]
  bf16* Vs = Ks + 2 * kKeys * QS;                    // [2][64][VS]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq4 = lane & 3;
  const int g = blockIdx.y;
  // which (sequence, token tile) is this CTA's
  // (tiles late in a sequence see the most keys: they are handed out first, so that the last wave is made of short ones)
  int total = 0;
  for (int s = 0; s < n_seqs; ++s) total += (cu_tokens[s + 1] - cu_tokens[s] + tq - 1) / tq;
  int tile = total - 1 - static_cast<int>(blockIdx.x), seq = -1, tok0 = 0, ntok = 0;
  if (tile < 0) return;
  for (int s = 0; s < n_seqs; ++s) {
    const int c0 = cu_tokens[s], len = cu_tokens[s + 1] - c0, nt = (len + tq - 1) / tq;
    if (tile < nt) { seq = s; tok0 = c0 + tile * tq; ntok = min(tq, len - tile * tq); break; }
    tile -= nt;
  }
  if (seq < 0) return;
  const int nkeys = static_cast<int>(a.positions[tok0 + ntok - 1]) + 1;   // tokens of a sequence are in order of position
  const int32_t* table = a.tables ? a.tables + static_cast<int64_t>(seq) * a.table_cap : nullptr;
  const int64_t dense0 = cu_tokens[seq];
  const bf16* qg = static_cast<const bf16*>(a.q);
  const bf16* kc = static_cast<const bf16*>(a.kc) + static_cast<int64_t>(g) * a.dim;
  const bf16* vc = static_cast<const bf16*>(a.vc) + static_cast<int64_t>(g) * a.vdim;
  // zero everything once (padding columns and rows stay zero), then the query rows
  for (int i = tid; i < (kRows * QS + 2 * kKeys * QS + 2 * kKeys * VS) / 8; i += kThreads) reinterpret_cast<uint4*>(smem_raw)[i] = make_uint4(0, 0, 0, 0);
  // the distance-bias rows of this CTA's heads (consecutive rows of the table), behind the tiles: one shared-memory load per
  // score instead of a global one
  float* bias_s = reinterpret_cast<float*>(smem_raw + static_cast<size_t>(kRows * QS + 2 * kKeys * QS + 2 * kKeys * VS) * sizeof(bf16));
  if (EXT && a.bias_staged)
    for (int i = tid; i < group * a.dist_rows; i += kThreads) bias_s[i] = a.dist_bias[static_cast<int64_t>(g) * group * a.dist_rows + i];
  __syncthreads();
  const int dch = a.dim / 8, vch = a.vdim / 8;     // 16-byte chunks per row
  // the query rows travel with the first key tile's copy group (asynchronous: no thread waits for its own row here)
  for (int i = tid; i < kRows * dch; i += kThreads) {
    const int r = i / dch, c = i % dch, t = r / group, hr = r % group;
    if (t < ntok)
      cp_async_16(smem_u32(Qs + r * QS + c * 8),
                  qg + static_cast<int64_t>(tok0 + t) * a.ldq + static_cast<int64_t>(g * group + hr) * a.dim + c * 8, 16);
  }
  // Cache slot of every key of a tile: looked up by 64 threads one tile ahead of the copy that needs it (the table read is a
  // dependent global load; in the copy loop it would serialise), kept in shared memory [2][64].
  __shared__ int64_t slot_s[2][kKeys];
  auto lookup = [&](int kt) -> int64_t {          // threads 0..63: key kt * 64 + tid
    const int j = kt * kKeys + tid;
    if (j >= nkeys) return -1;
    if (table == nullptr) return dense0 + j;
    const int32_t blk = table[j / a.block_size];
    return blk >= 0 ? static_cast<int64_t>(blk) * a.block_size + j % a.block_size : -1;
  };
  // thread -> (key row, every fourth 16-byte chunk of it): no index arithmetic in the copy loop
  const int lr = tid >> 2, lh = tid & 3;
  auto load_tile = [&](int kt, int buf) {
    bf16* kd = Ks + buf * kKeys * QS + lr * QS;
    bf16* vd = Vs + buf * kKeys * VS + lr * VS;
    const int64_t slot = slot_s[kt & 1][lr];
    const bf16* ksrc = slot >= 0 ? kc + slot * a.k_row : kc;
    const bf16* vsrc = slot >= 0 ? vc + slot * a.v_row : vc;
    const int nb = slot >= 0 ? 16 : 0;
    for (int c = lh; c < dch; c += 4) cp_async_16(smem_u32(kd + c * 8), ksrc + (nb ? c * 8 : 0), nb);
    for (int c = lh; c < vch; c += 4) cp_async_16(smem_u32(vd + c * 8), vsrc + (nb ? c * 8 : 0), nb);
    cp_async_commit();
  };
  // Few rows (single tokens: at most 16 (token, head) pairs): all warps work on the SAME 16 rows, warp w on the keys
  // [16 (w & 3), +16) of every tile and half (w >> 2) of the value columns; the four partial softmaxes are merged at the end.
  // Otherwise warp w owns rows [16 w, +16) and walks whole tiles (warps without rows only help with the copies).
  const bool few = ntok * group <= 16;
  const int rbase = few ? 0 : warp * 16, kq = warp & 3, vh = warp >> 2;
  int pos[2], lo[2]; float qscale[2]; bool valid[2];
  const float* bias[2] = {nullptr, nullptr};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = rbase + gq + 8 * i, t = r / group;
    valid[i] = t < ntok && r < tq * group;
    pos[i] = valid[i] ? static_cast<int>(a.positions[tok0 + t]) : -1;
    lo[i] = valid[i] ? first_key(a, pos[i]) : -(1 << 30);   // a row sees the keys lo .. pos
    qscale[i] = a.scale * (1.0f + a.temp_coef * logf(floorf(static_cast<float>((pos[i] + 1) / a.temp_every)) + 1.0f)) *
                (a.softcap > 0.f ? 1.0f / a.softcap : kLog2e);
    if (EXT) {
      const int h = g * group + r % group;
      if (a.head_scale) qscale[i] *= a.head_scale[h];
      if (a.dist_bias) bias[i] = a.bias_staged ? bias_s + (r % group) * a.dist_rows : a.dist_bias + static_cast<int64_t>(h) * a.dist_rows;
    }
  }
  // the smallest position of the warp's rows decides whether a tile needs the causal mask (empty rows count as hidden)
  const bool warp_has_rows = rbase / group < ntok;
  const int min_pos = __reduce_min_sync(0xffffffffu, min(pos[0], pos[1]));
  const int max_lo = __reduce_max_sync(0xffffffffu, max(lo[0], lo[1]));   // a tile that starts before it needs the window's / chunk's mask
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[VMAX / 8][4];
#pragma unroll
  for (int i = 0; i < VMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const bool capped = a.softcap > 0.f;
  const float cap2 = a.softcap * kLog2e;           // scores are kept in log2 units: softmax with exp2
  const int ntiles = (nkeys + kKeys - 1) / kKeys;
  // with a window the first tile is the one that holds the first key the CTA's first token sees (tiles stay anchored at
  // multiples of 64 from the sequence's start)
  const int kt0 = first_key(a, static_cast<int>(a.positions[tok0])) / kKeys;   // (windows and chunks only move forward with the position)
  if (tid < kKeys) { slot_s[kt0 & 1][tid] = lookup(kt0); slot_s[(kt0 + 1) & 1][tid] = lookup(kt0 + 1); }
  __syncthreads();
  load_tile(kt0, kt0 & 1);
  const uint32_t q_addr = smem_u32(Qs + (rbase + (lane & 15)) * QS + (lane >> 4) * 8);
  const int k_lane = ((lane & 7) + (lane >> 4) * 8) * QS + ((lane >> 3) & 1) * 8;
  const int v_lane = ((lane & 7) + ((lane >> 3) & 1) * 8) * VS + (lane >> 4) * 8;
  for (int kt = kt0; kt < ntiles; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < ntiles) { load_tile(kt + 1, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    const int64_t slot_ahead = (tid < kKeys && kt + 2 < ntiles) ? lookup(kt + 2) : -1;   // in flight during this tile's math
    __syncthreads();
    const bf16* kb = Ks + buf * kKeys * QS;
    const bf16* vb = Vs + buf * kKeys * VS;
    if (few) {
      const int key0 = kt * kKeys + kq * 16;
      if (key0 < nkeys)
        attn_tile<DMAX, VMAX, 1, VMAX / 32, QS, VS, EXT>(o, m, l, q_addr, smem_u32(kb + kq * 16 * QS + k_lane),
                                                         smem_u32(vb + kq * 16 * VS + vh * (VMAX / 2) + v_lane), key0, pos, lo, qscale, capped, cap2,
                                                         key0 + 15 > min_pos || key0 < max_lo, tq4, bias, a.dist_rows);
    } else if (warp_has_rows) {
      // two halves of 32 keys: half the score registers of a 64-key pass (no spills under the 128-register cap)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf)
        attn_tile<DMAX, VMAX, 2, VMAX / 16, QS, VS, EXT>(o, m, l, q_addr, smem_u32(kb + hf * 32 * QS + k_lane), smem_u32(vb + hf * 32 * VS + v_lane),
                                                         kt * kKeys + hf * 32, pos, lo, qscale, capped, cap2,
                                                         kt * kKeys + hf * 32 + 31 > min_pos || kt * kKeys + hf * 32 < max_lo, tq4, bias, a.dist_rows);
    }
    if (tid < kKeys) slot_s[kt & 1][tid] = slot_ahead;   // tile kt's slots were consumed by load_tile(kt) an iteration ago
    __syncthreads();   // everyone is done with this buffer before the next load overwrites it
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
  if (few) {
    // merge the four key quarters: (m, l) per quarter and row, O per quarter, row and column, through the (now idle) tile memory
    float* ms = reinterpret_cast<float*>(Ks);          // [4][16]
    float* ls = ms + 64;                               // [4][16]
    float* os = ls + 64;                               // [4][16][VMAX]
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = gq + 8 * i;
      if (vh == 0 && tq4 == 0) { ms[kq * 16 + r] = m[i]; ls[kq * 16 + r] = l[i]; }
#pragma unroll
      for (int vt = 0; vt < VMAX / 16; ++vt) {
        const int c = vh * (VMAX / 2) + vt * 8 + 2 * tq4;
        os[(kq * 16 + r) * VMAX + c] = o[vt][2 * i];
        os[(kq * 16 + r) * VMAX + c + 1] = o[vt][2 * i + 1];
      }
    }
    __syncthreads();
    const int rows = ntok * group;
    // with the output rotation a thread merges both values of a pair (c, c + vdim / 2), turns them and stores them
    const bool rot = a.out_rot != nullptr;
    const int cols = rot ? a.vdim / 2 : a.vdim;
    for (int e = tid; e < rows * cols; e += kThreads) {
      const int r = e / cols, c = e - r * cols, t = r / group, h = g * group + r % group;
      float mm = fmaxf(fmaxf(ms[r], ms[16 + r]), fmaxf(ms[32 + r], ms[48 + r]));
      float num = 0.f, num2 = 0.f, den = 0.f;
      if (a.sinks) {   // the sink joins the denominator only (scores are in log2 units here)
        const float sk = a.sinks[h] * kLog2e;
        mm = fmaxf(mm, sk);
        den = fast_exp2(sk - mm);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float w = fast_exp2(ms[k * 16 + r] - mm);     // a quarter that saw no key: exp2(-inf) = 0
        num = fmaf(w, os[(k * 16 + r) * VMAX + c], num);
        if (rot) num2 = fmaf(w, os[(k * 16 + r) * VMAX + c + cols], num2);
        den = fmaf(w, ls[k * 16 + r], den);
      }
      float v = den > 0.f ? num / den : 0.f;
      bf16* op = static_cast<bf16*>(a.out) + static_cast<int64_t>(tok0 + t) * a.ldo + static_cast<int64_t>(h) * a.vdim;
      const float* gt = a.gate ? a.gate + static_cast<int64_t>(tok0 + t) * a.ldg + (a.gate_per_head ? h : static_cast<int64_t>(h) * a.vdim) : nullptr;
      if (rot) {
        float v2 = den > 0.f ? num2 / den : 0.f;
        const int p = static_cast<int>(a.positions[tok0 + t]);
        const float2 cs = a.out_rot[static_cast<int64_t>(p < 0 ? 0 : (p >= a.max_pos ? a.max_pos - 1 : p)) * cols + c];
        const float u = v;
        v = fmaf(u, cs.x, v2 * cs.y);                      // turned by -position: (u cos + v sin, v cos - u sin)
        v2 = fmaf(v2, cs.x, -u * cs.y);
        if (gt) v2 *= 1.0f / (1.0f + __expf(-gt[a.gate_per_head ? 0 : c + cols]));
        op[c + cols] = __float2bfloat16_rn(v2);
      }
      if (gt) v *= 1.0f / (1.0f + __expf(-gt[a.gate_per_head ? 0 : c]));
      op[c] = __float2bfloat16_rn(v);
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!valid[i]) continue;
    const int r = warp * 16 + gq + 8 * i, t = r / group, h = g * group + r % group;
    float ll = l[i], oc = 1.0f;
    if (a.sinks) {   // the sink joins the denominator only (scores are in log2 units here)
      const float sk = a.sinks[h] * kLog2e, mn = fmaxf(m[i], sk);
      oc = fast_exp2(m[i] - mn);
      ll = ll * oc + fast_exp2(sk - mn);
    }
    const float inv = ll > 0.f ? oc / ll : 0.f;
    bf16* op = static_cast<bf16*>(a.out) + static_cast<int64_t>(tok0 + t) * a.ldo + static_cast<int64_t>(h) * a.vdim;
    const float* gt = a.gate ? a.gate + static_cast<int64_t>(tok0 + t) * a.ldg + (a.gate_per_head ? h : static_cast<int64_t>(h) * a.vdim) : nullptr;
    const float gh = (gt && a.gate_per_head) ? 1.0f / (1.0f + __expf(-gt[0])) : 1.0f;
    if (a.out_rot != nullptr) {   // vdim == VMAX here: a thread's columns c and c + VMAX / 2 are both its own
      const int p = pos[i] >= a.max_pos ? a.max_pos - 1 : pos[i];
      const float4* tab = reinterpret_cast<const float4*>(a.out_rot + static_cast<int64_t>(p) * (VMAX / 2));
#pragma unroll
      for (int vt = 0; vt < VMAX / 16; ++vt) {
        const float4 cs = __ldg(tab + vt * 4 + tq4);     // (cos, sin) of the pairs c and c + 1, c = vt * 8 + 2 tq4
        const float u0 = o[vt][2 * i], w0 = o[vt + VMAX / 16][2 * i], u1 = o[vt][2 * i + 1], w1 = o[vt + VMAX / 16][2 * i + 1];
        o[vt][2 * i] = fmaf(u0, cs.x, w0 * cs.y);            o[vt + VMAX / 16][2 * i] = fmaf(w0, cs.x, -u0 * cs.y);
        o[vt][2 * i + 1] = fmaf(u1, cs.z, w1 * cs.w);        o[vt + VMAX / 16][2 * i + 1] = fmaf(w1, cs.z, -u1 * cs.w);
      }
    }
#pragma unroll
    for (int vt = 0; vt < VMAX / 8; ++vt) {
      const int c = vt * 8 + 2 * tq4;
      if (c >= a.vdim) continue;
      float v0 = o[vt][2 * i] * inv * gh, v1 = o[vt][2 * i + 1] * inv * gh;
      if (gt && !a.gate_per_head) { v0 *= 1.0f / (1.0f + __expf(-gt[c])); v1 *= 1.0f / (1.0f + __expf(-gt[c + 1])); }
      *reinterpret_cast<uint32_t*>(op + c) = pack_bf16x2(v0, v1);
    }
  }
}

template <int DMAX, int VMAX, bool EXT>
int launch_mma(AttnArgs a, const int32_t* cu_tokens, int n_seqs, cudaStream_t st) {
  const int group = a.heads / a.kv_heads, tq = kRows / group;
  const size_t tiles = (static_cast<size_t>(kRows) * (DMAX + 8) + 2 * kKeys * (DMAX + 8) + 2 * kKeys * (VMAX + 8)) * sizeof(bf16);
  const size_t bias_bytes = static_cast<size_t>(group) * a.dist_rows * sizeof(float);
  a.bias_staged = EXT && a.dist_bias != nullptr && bias_bytes <= kBiasSmemBytes;
  const size_t smem = tiles + (a.bias_staged ? bias_bytes : 0);
  NVLLM_SMEM_ATTR_ONCE((capped_attn_mma_kernel<DMAX, VMAX, EXT>), tiles + (EXT ? kBiasSmemBytes : 0));
  dim3 grid((a.n + tq - 1) / tq + n_seqs, a.kv_heads);
  capped_attn_mma_kernel<DMAX, VMAX, EXT><<<grid, kThreads, smem, st>>>(a, cu_tokens, n_seqs, tq, group);
  NVLLM_LAUNCH_CHECK("capped_attn_mma_kernel");
  return 0;
}

}  // namespace
}  // namespace nvllm

using namespace nvllm;

extern "C" int nvllm_attn_bias_store(void* q, int64_t ldq, void* k_cache, void* v_cache, int64_t k_row, int64_t v_row,
                                     const float* proj, int64_t ldp, const float* q_bias, const float* k_bias, const float* v_bias,
                                     const int32_t* slots, int32_t n, int32_t q_cols, int32_t k_cols, int32_t v_cols, int32_t dtype,
                                     void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && q_cols > 0 && k_cols > 0 && v_cols > 0 && ldq >= q_cols && k_row >= k_cols && v_row >= v_cols &&
                      ldp >= q_cols + k_cols + v_cols, NVLLM_ERR_ARG, "attn_bias_store: sizes");
  NVLLM_CHECK_ARG(dtype == NVLLM_BF16 || dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "attn_bias_store: dtype %d", dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(q && k_cache && v_cache && proj && slots, NVLLM_ERR_ARG, "attn_bias_store: NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == NVLLM_BF16)
    attn_bias_store_kernel<bf16><<<n, 256, 0, st>>>(static_cast<bf16*>(q), ldq, static_cast<bf16*>(k_cache), static_cast<bf16*>(v_cache), k_row,
                                                    v_row, proj, ldp, q_bias, k_bias, v_bias, slots, q_cols, k_cols, v_cols);
  else
    attn_bias_store_kernel<float><<<n, 256, 0, st>>>(static_cast<float*>(q), ldq, static_cast<float*>(k_cache), static_cast<float*>(v_cache),
                                                     k_row, v_row, proj, ldp, q_bias, k_bias, v_bias, slots, q_cols, k_cols, v_cols);
  NVLLM_LAUNCH_CHECK("attn_bias_store_kernel");
  return 0;
}

extern "C" int nvllm_attn_wide_norm_store(void* q, int64_t ldq, void* k_cache, void* v_cache, int64_t k_row, int64_t v_row,
                                          const float* proj, int64_t ldp, const float* q_norm_w, const float* k_norm_w, float eps,
                                          const int32_t* slots, int32_t n, int32_t q_cols, int32_t k_cols, int32_t v_cols, int32_t dtype,
                                          void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && q_cols > 0 && k_cols >= 0 && v_cols >= 0 && (k_cols > 0 || v_cols == 0) && ldq >= q_cols && ldp >= q_cols + k_cols + v_cols &&
                      (k_cols == 0 || (k_row >= k_cols && v_row >= v_cols)), NVLLM_ERR_ARG, "attn_wide_norm_store: sizes");
  NVLLM_CHECK_ARG(dtype == NVLLM_BF16 || dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "attn_wide_norm_store: dtype %d", dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(q && proj && slots && (k_cols == 0 || (k_cache && v_cache)), NVLLM_ERR_ARG, "attn_wide_norm_store: NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == NVLLM_BF16)
    attn_wide_norm_store_kernel<bf16><<<n, 256, 0, st>>>(static_cast<bf16*>(q), ldq, static_cast<bf16*>(k_cache), static_cast<bf16*>(v_cache),
                                                         k_row, v_row, proj, ldp, q_norm_w, k_norm_w, slots, q_cols, k_cols, v_cols, eps);
  else
    attn_wide_norm_store_kernel<float><<<n, 256, 0, st>>>(static_cast<float*>(q), ldq, static_cast<float*>(k_cache), static_cast<float*>(v_cache),
                                                          k_row, v_row, proj, ldp, q_norm_w, k_norm_w, slots, q_cols, k_cols, v_cols, eps);
  NVLLM_LAUNCH_CHECK("attn_wide_norm_store_kernel");
  return 0;
}

extern "C" int nvllm_attn_rope_norm_store(void* q, int64_t ldq, void* k_cache, void* v_cache, int64_t k_row, int64_t v_row,
                                          const float* proj, int64_t ldp, const float* q_bias, const float* k_bias,
                                          const float* v_bias, const int64_t* positions, const float* rope_table, int32_t rot_dims,
                                          int32_t max_pos, float norm_eps, const int32_t* slots, int32_t n, int32_t heads,
                                          int32_t kv_heads, int32_t dim, int32_t vdim, int32_t v_from_k, int32_t dtype, void* stream) {
  return nvllm_attn_rotary_store(q, ldq, k_cache, v_cache, k_row, v_row, proj, ldp, q_bias, k_bias, v_bias, positions, rope_table, rot_dims, 0,
                                 nullptr, max_pos, norm_eps, slots, n, heads, kv_heads, dim, vdim, v_from_k, dtype, stream);
}

extern "C" int nvllm_attn_rotary_store(void* q, int64_t ldq, void* k_cache, void* v_cache, int64_t k_row, int64_t v_row,
                                       const float* proj, int64_t ldp, const float* q_bias, const float* k_bias, const float* v_bias,
                                       const int64_t* positions, const float* rope_table, int32_t rot_dims, int32_t halves,
                                       const float* v_rope_table, int32_t max_pos, float norm_eps, const int32_t* slots, int32_t n,
                                       int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t v_from_k, int32_t dtype,
                                       void* stream) {
  NVLLM_CHECK_ARG(v_rope_table == nullptr || !v_from_k, NVLLM_ERR_ARG, "attn_rotary_store: rotated values need a value projection of their own");
  NVLLM_CHECK_ARG(n >= 0 && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dim &&
                      max_pos > 0 && (!v_from_k || vdim == dim), NVLLM_ERR_ARG,
                  "attn_rope_norm_store: heads=%d/%d dim=%d vdim=%d rot_dims=%d (even, <= dim; values from keys need vdim == dim)", heads,
                  kv_heads, dim, vdim, rot_dims);
  NVLLM_CHECK_ARG(ldq >= static_cast<int64_t>(heads) * dim && k_row >= static_cast<int64_t>(kv_heads) * dim &&
                      v_row >= static_cast<int64_t>(kv_heads) * vdim &&
                      ldp >= static_cast<int64_t>(heads + kv_heads) * dim + (v_from_k ? 0 : static_cast<int64_t>(kv_heads) * vdim),
                  NVLLM_ERR_ARG, "attn_rope_norm_store: strides");
  NVLLM_CHECK_ARG(dtype == NVLLM_BF16 || dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "attn_rope_norm_store: dtype %d", dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(q && k_cache && v_cache && proj && positions && slots && (rope_table || rot_dims == 0), NVLLM_ERR_ARG,
                  "attn_rope_norm_store: NULL");
  const RopeStoreArgs a{q, ldq, k_cache, v_cache, k_row, v_row, proj, ldp, q_bias, k_bias, v_bias, positions,
                        reinterpret_cast<const float2*>(rope_table), rot_dims, max_pos, norm_eps, slots, n, heads, kv_heads, dim, vdim, v_from_k,
                        halves != 0, reinterpret_cast<const float2*>(v_rope_table)};
  const int64_t items = static_cast<int64_t>(n) * (heads + kv_heads + (v_from_k ? 0 : kv_heads));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // values from keys, heads of 4..512 values in 16-byte steps, aligned rows: the one-pass kernel
  if (v_from_k && !halves && dim % 4 == 0 && dim <= 512 && ldp % 4 == 0 && ldq % 4 == 0 && k_row % 4 == 0 && v_row % 4 == 0 && aligned16(proj) && aligned16(q) &&
      aligned16(k_cache) && aligned16(v_cache) && aligned16(q_bias) && aligned16(k_bias)) {
    const int64_t vitems = static_cast<int64_t>(n) * (heads + kv_heads);
    if (dtype == NVLLM_BF16) attn_rope_norm_store_vec_kernel<bf16><<<static_cast<unsigned>((vitems + 3) / 4), 128, 0, st>>>(a);
    else attn_rope_norm_store_vec_kernel<float><<<static_cast<unsigned>((vitems + 3) / 4), 128, 0, st>>>(a);
    NVLLM_LAUNCH_CHECK("attn_rope_norm_store_vec_kernel");
    return 0;
  }
  // halves pairing, no biases, values of their own, 16-byte rows and rotated parts that split into chunks of 4: the vector kernel
  if (halves && !v_from_k && !q_bias && !k_bias && !v_bias && dim % 4 == 0 && vdim % 4 == 0 && dim <= 512 && vdim <= 512 && rot_dims % 8 == 0 &&
      (v_rope_table == nullptr || vdim % 8 == 0) && ldp % 4 == 0 && ldq % 4 == 0 && k_row % 4 == 0 && v_row % 4 == 0 && aligned16(proj) && aligned16(q) &&
      aligned16(k_cache) && aligned16(v_cache) && aligned16(rope_table) && aligned16(v_rope_table)) {
    if (dtype == NVLLM_BF16) attn_rotary_store_halves_vec_kernel<bf16><<<static_cast<unsigned>((items + 3) / 4), 128, 0, st>>>(a);
    else attn_rotary_store_halves_vec_kernel<float><<<static_cast<unsigned>((items + 3) / 4), 128, 0, st>>>(a);
    NVLLM_LAUNCH_CHECK("attn_rotary_store_halves_vec_kernel");
    return 0;
  }
  if (dtype == NVLLM_BF16) attn_rope_norm_store_kernel<bf16><<<static_cast<unsigned>((items + 3) / 4), 128, 0, st>>>(a);
  else attn_rope_norm_store_kernel<float><<<static_cast<unsigned>((items + 3) / 4), 128, 0, st>>>(a);
  NVLLM_LAUNCH_CHECK("attn_rope_norm_store_kernel");
  return 0;
}

extern "C" int nvllm_capped_attention(void* out, int64_t ldo, const void* q, int64_t ldq, const float* gate, int64_t ldg,
                                      const void* k_cache, const void* v_cache, int64_t k_row, int64_t v_row,
                                      const int32_t* tok_seq, const int64_t* positions, const int32_t* block_tables,
                                      int32_t table_cap, int32_t block_size, int32_t n, int32_t heads, int32_t kv_heads, int32_t dim,
                                      int32_t vdim, float scale, float softcap, float temp_coef, int32_t temp_every,
                                      const int32_t* cu_tokens, int32_t n_seqs, int32_t dtype, void* stream) {
  return nvllm_window_attention(out, ldo, q, ldq, gate, ldg, 0, k_cache, v_cache, k_row, v_row, tok_seq, positions, block_tables, table_cap,
                                block_size, n, heads, kv_heads, dim, vdim, scale, softcap, temp_coef, temp_every, 0, nullptr, cu_tokens,
                                n_seqs, dtype, stream);
}

extern "C" int nvllm_window_attention(void* out, int64_t ldo, const void* q, int64_t ldq, const float* gate, int64_t ldg,
                                      int32_t gate_per_head, const void* k_cache, const void* v_cache, int64_t k_row, int64_t v_row,
                                      const int32_t* tok_seq, const int64_t* positions, const int32_t* block_tables,
                                      int32_t table_cap, int32_t block_size, int32_t n, int32_t heads, int32_t kv_heads, int32_t dim,
                                      int32_t vdim, float scale, float softcap, float temp_coef, int32_t temp_every, int32_t window,
                                      const float* sinks, const int32_t* cu_tokens, int32_t n_seqs, int32_t dtype, void* stream) {
  return nvllm_biased_attention(out, ldo, q, ldq, gate, ldg, gate_per_head, k_cache, v_cache, k_row, v_row, tok_seq, positions, block_tables,
                                table_cap, block_size, n, heads, kv_heads, dim, vdim, scale, softcap, temp_coef, temp_every, window, sinks, 0,
                                nullptr, nullptr, 0, nullptr, 0, cu_tokens, n_seqs, dtype, stream);
}

extern "C" int nvllm_biased_attention(void* out, int64_t ldo, const void* q, int64_t ldq, const float* gate, int64_t ldg,
                                      int32_t gate_per_head, const void* k_cache, const void* v_cache, int64_t k_row, int64_t v_row,
                                      const int32_t* tok_seq, const int64_t* positions, const int32_t* block_tables,
                                      int32_t table_cap, int32_t block_size, int32_t n, int32_t heads, int32_t kv_heads, int32_t dim,
                                      int32_t vdim, float scale, float softcap, float temp_coef, int32_t temp_every, int32_t window,
                                      const float* sinks, int32_t chunk, const float* head_scale, const float* dist_bias,
                                      int32_t dist_rows, const float* out_rot_table, int32_t max_pos, const int32_t* cu_tokens,
                                      int32_t n_seqs, int32_t dtype, void* stream) {
  NVLLM_CHECK_ARG(chunk >= 0 && (dist_bias == nullptr || dist_rows > 0) && (out_rot_table == nullptr || (max_pos > 0 && vdim % 2 == 0)),
                  NVLLM_ERR_ARG, "attention: chunk=%d dist_rows=%d max_pos=%d vdim=%d (an output rotation pairs the halves of an even vdim)", chunk,
                  dist_rows, max_pos, vdim);
  NVLLM_CHECK_ARG(n >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0 && vdim <= 32 * kMaxVPerLane &&
                      dim <= 2048 && block_size > 0 && table_cap > 0 && temp_every > 0, NVLLM_ERR_ARG,
                  "attention: n=%d heads=%d/%d dim=%d vdim=%d (vdim <= 512)", n, heads, kv_heads, dim, vdim);
  NVLLM_CHECK_ARG(dtype == NVLLM_BF16 || dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "attention: dtype %d", dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(out && q && k_cache && v_cache && tok_seq && positions && (block_tables || cu_tokens), NVLLM_ERR_ARG, "attention: NULL");
  AttnArgs a{out, ldo, q, ldq, gate, ldg, k_cache, v_cache, k_row, v_row, tok_seq, positions, block_tables, table_cap, block_size,
             n, heads, kv_heads, dim, vdim, scale, softcap, temp_coef, temp_every, window > 0 ? window : 0, sinks, gate_per_head, block_tables ? nullptr : cu_tokens,
             chunk, head_scale, dist_bias, dist_rows, reinterpret_cast<const float2*>(out_rot_table), max_pos, 0};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // bf16 with 16-byte rows and a token range per sequence: tensor cores; everything else (f32, odd sizes): one warp per row
  const int group = heads / kv_heads;
  if (dtype == NVLLM_BF16 && cu_tokens != nullptr && n_seqs > 0 && knobs().capped_mma && group <= kRows && dim % 8 == 0 && vdim % 8 == 0 &&
      dim <= 128 && vdim <= 128 && ldq % 8 == 0 && k_row % 8 == 0 && v_row % 8 == 0 && ldo % 2 == 0 && aligned16(q) && aligned16(k_cache) &&
      aligned16(v_cache) && (reinterpret_cast<uintptr_t>(out) & 3u) == 0) {
    // the factor per head and the distance bias live in a second instantiation, so that kernels without them keep their
    // registers (the output rotation only touches the epilogue)
    const bool ext = head_scale != nullptr || dist_bias != nullptr;
    const int vmax = vdim <= 64 ? 64 : 128;
    // the output rotation pairs column c with c + vdim / 2 inside one thread's accumulators: vdim must fill the tile
    if (out_rot_table == nullptr || (vdim == vmax && aligned16(out_rot_table))) {
      if (!ext) {
        if (dim <= 64 && vdim <= 64) return launch_mma<64, 64, false>(a, cu_tokens, n_seqs, st);
        if (vdim <= 64) return launch_mma<128, 64, false>(a, cu_tokens, n_seqs, st);
        return launch_mma<128, 128, false>(a, cu_tokens, n_seqs, st);
      }
      if (dim <= 64 && vdim <= 64) return launch_mma<64, 64, true>(a, cu_tokens, n_seqs, st);
      if (vdim <= 64) return launch_mma<128, 64, true>(a, cu_tokens, n_seqs, st);
      return launch_mma<128, 128, true>(a, cu_tokens, n_seqs, st);
    }
  }
  const unsigned grid = static_cast<unsigned>((static_cast<int64_t>(n) * heads + 3) / 4);
  const size_t smem = static_cast<size_t>(4) * (dim > vdim ? dim : vdim) * sizeof(float);
  if (dtype == NVLLM_BF16) capped_attn_warp_kernel<bf16><<<grid, 128, smem, st>>>(a);
  else capped_attn_warp_kernel<float><<<grid, 128, smem, st>>>(a);
  NVLLM_LAUNCH_CHECK("capped_attn_warp_kernel");
  return 0;
}
