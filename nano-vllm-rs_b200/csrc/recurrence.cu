// recurrence.cu — mixers that carry a fixed-size state from token to token instead of a growing cache.  The state of a
// sequence lives in a SLOT of a state pool (f32) that the scheduler hands out when the sequence is admitted; a step names,
// per sequence, its slot and the range of its tokens in the batch (cu_tokens), so one launch serves whole prompts, portions
// and single decoded tokens.  A portion that begins at position 0 starts from a zero state (a reused slot needs no clearing);
// any other portion continues from what the slot holds.
//
//   nvllm_linear_recurrence   S_t = a_t S_(t-1) + b_t k_t v_t^T,   y_t = S_t^T q_t + d v_t        (S: [dk, dv] per head)
//       covers state-space duality (k = B, q = C, v = x, a = exp(-exp(A_log) dt), b = dt, d = D; B and C shared by the heads
//       of a group) and retention (a = a constant per head, b = 1, d = 0)
//   nvllm_gated_delta_recurrence   the gated delta rule with a decay per key channel:  S <- diag(g_t) S,
//       u = beta_t (v_t - S^T k_t),  S <- S + k_t u^T,  y_t = S^T q_t;  nvllm_delta_prepare makes its inputs (unit-length q and k,
//       beta = sigmoid, g = exp(-exp(A_log) softplus(. + dt_bias)))
//   nvllm_causal_conv         per-channel convolution over the last `taps` tokens (+ bias, SiLU); the slot keeps the window's
//       history, i.e. the raw inputs of the preceding taps - 1 tokens
//   nvllm_ssd_prepare         dt = softplus(raw + bias), a = exp(-exp(A_log) dt)
//   nvllm_rotate_half         rotary positions, dimension i paired with i + dims/2, on the first `dims` values of every head
//   nvllm_gated_group_norm    RMS norm over equal parts of a row with a SiLU (or sigmoid) gate before or after it
// Everything here is f32: inputs, state, arithmetic.  Only nvllm_gated_group_norm writes the operand type (its output
// feeds a projection).
#include <algorithm>

#include "common.cuh"

namespace nvllm {
namespace {

struct RecArgs {
  float* y; int64_t ldy;
  const float *q, *k, *v; int64_t ldq, ldk, ldv;
  int group_div;                 // head h reads q / k of group h / group_div
  const float* decay; int decay_ld;   // [n, heads] (decay_ld = heads) or [heads] (decay_ld = 0)
  const float* step; int step_ld;     // same, or null (1)
  const float* skip;                  // [heads] or null (0)
  float* state;                       // [slots, heads, dk, dv]
  const int32_t *seq_slot, *cu_tokens; const int64_t* positions;
  int heads, dk, dv;
};

constexpr int kRecTile = 16;  // tokens per stage

__device__ __forceinline__ void cp_async_4(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_addr), "l"(gptr) : "memory");
}

// CTA = (head, sequence, slice of dv).  Thread (pc, ns): PP neighbouring columns of the state, rows [ns * NPT, (ns + 1) * NPT) of
// each in registers (every k / q value read from shared memory serves PP columns: the broadcast reads are what binds).
// kRecTile tokens' k, q (rows of dk), v, a, b are staged in shared memory with cp.async, two stages deep: the copies of the
// next stage fly while the current stage's tokens are stepped through, and the steps themselves need no synchronisation.  NSL row
// slices of one column sit in neighbouring lanes and are summed with shuffles.  vec: rows are 16-byte multiples.
template <int NPT, int NSL, int PP>
__global__ void __launch_bounds__(512) linear_recurrence_kernel(const RecArgs a, int pb, int vec) {
  extern __shared__ __align__(16) float sm[];
  // a row of k (or q) in shared memory: NSL slices of NPT values, each followed by 4 floats of padding, so that the NSL
  // 16-byte broadcast reads of one warp instruction (one per slice) fall into different banks
  constexpr int SL = NPT + 4, DKP = SL * NSL;
  const int pbp = (pb + 3) & ~3;
  const int stage = kRecTile * (2 * DKP + pbp + 2);
  const int h = blockIdx.x, s = blockIdx.y, p0 = blockIdx.z * pb;
  // the thread's PP columns lie pb / PP apart, so that neighbouring threads hold neighbouring columns (coalesced state)
  const int tid = threadIdx.x, ns = tid % NSL, pl = tid / NSL, p = p0 + pl, half = (pb + PP - 1) / PP;
  bool live[PP];
#pragma unroll
  for (int j = 0; j < PP; ++j) live[j] = pl < half && pl + j * half < pb && p + j * half < a.dv;
  const int t0 = a.cu_tokens[s], t1 = a.cu_tokens[s + 1];
  const int slot = a.seq_slot[s];
  if (t1 <= t0) return;
  if (slot < 0) {  // padding sequence of a captured batch: defined output, no state
    for (int t = t0; t < t1; ++t)
#pragma unroll
      for (int j = 0; j < PP; ++j)
        if (live[j] && ns == 0) a.y[t * a.ldy + static_cast<int64_t>(h) * a.dv + p + j * half] = 0.f;
    return;
  }
  const int g = h / a.group_div;
  // both stages start as zeros (rows beyond dk and columns beyond dv stay zero) with a step of 1
  for (int e = tid; e < 2 * stage; e += blockDim.x) sm[e] = 0.f;
  __syncthreads();
  if (a.step == nullptr && tid < 2 * kRecTile) sm[(tid / kRecTile) * stage + kRecTile * (2 * DKP + pbp) + kRecTile + tid % kRecTile] = 1.f;
  const int ncol = min(pb, a.dv - p0);
  auto issue = [&](int tb, int buf) {
    float* ks = sm + buf * stage;
    float* qs = ks + kRecTile * DKP;
    float* vs = qs + kRecTile * DKP;
    float* as = vs + kRecTile * pbp;
    float* bs = as + kRecTile;
    const int cnt = min(kRecTile, t1 - tb);
    if (vec) {
      const int kch = a.dk / 4, vch = ncol / 4;
      for (int e = tid; e < cnt * kch; e += blockDim.x) {
        const int tt = e / kch, c = e - tt * kch;
        const int64_t t = tb + tt;
        const int dst = tt * DKP + (c * 4 / NPT) * SL + (c * 4) % NPT;
        cp_async_16(smem_u32(ks + dst), a.k + t * a.ldk + static_cast<int64_t>(g) * a.dk + c * 4, 16);
        cp_async_16(smem_u32(qs + dst), a.q + t * a.ldq + static_cast<int64_t>(g) * a.dk + c * 4, 16);
      }
      for (int e = tid; e < cnt * vch; e += blockDim.x) {
        const int tt = e / vch, c = e - tt * vch;
        cp_async_16(smem_u32(vs + tt * pbp + c * 4), a.v + static_cast<int64_t>(tb + tt) * a.ldv + static_cast<int64_t>(h) * a.dv + p0 + c * 4, 16);
      }
    } else {
      for (int e = tid; e < cnt * a.dk; e += blockDim.x) {
        const int tt = e / a.dk, n = e - tt * a.dk;
        const int64_t t = tb + tt;
        const int dst = tt * DKP + (n / NPT) * SL + n % NPT;
        cp_async_4(smem_u32(ks + dst), a.k + t * a.ldk + static_cast<int64_t>(g) * a.dk + n);
        cp_async_4(smem_u32(qs + dst), a.q + t * a.ldq + static_cast<int64_t>(g) * a.dk + n);
      }
      for (int e = tid; e < cnt * ncol; e += blockDim.x) {
        const int tt = e / ncol, c = e - tt * ncol;
        cp_async_4(smem_u32(vs + tt * pbp + c), a.v + static_cast<int64_t>(tb + tt) * a.ldv + static_cast<int64_t>(h) * a.dv + p0 + c);
      }
    }
    if (tid < cnt) {
      const int64_t t = tb + tid;
      cp_async_4(smem_u32(as + tid), a.decay + (a.decay_ld ? t * a.decay_ld + h : h));
      if (a.step) cp_async_4(smem_u32(bs + tid), a.step + (a.step_ld ? t * a.step_ld + h : h));
    }
    cp_async_commit();
  };
  issue(t0, 0);
  float S[PP][NPT];
  float* sp = a.state + ((static_cast<int64_t>(slot) * a.heads + h) * a.dk) * a.dv;
  const bool fresh = a.positions[t0] == 0;
#pragma unroll
  for (int j = 0; j < PP; ++j)
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = ns * NPT + i;
      S[j][i] = (!fresh && live[j] && n < a.dk) ? sp[static_cast<int64_t>(n) * a.dv + p + j * half] : 0.f;
    }
  const float d = a.skip ? a.skip[h] : 0.f;
  int buf = 0;
  for (int tb = t0; tb < t1; tb += kRecTile, buf ^= 1) {
    const int cnt = min(kRecTile, t1 - tb);
    if (tb + kRecTile < t1) { issue(tb + kRecTile, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const float* ks = sm + buf * stage;
    const float* qs = ks + kRecTile * DKP;
    const float* vs = qs + kRecTile * DKP;
    const float* as = vs + kRecTile * pbp;
    const float* bs = as + kRecTile;
    for (int tt = 0; tt < cnt; ++tt) {
      const float av = as[tt], bt = bs[tt];
      float xv[PP], bv[PP], acc[PP];
#pragma unroll
      for (int j = 0; j < PP; ++j) { xv[j] = vs[tt * pbp + (live[j] ? pl + j * half : 0)]; bv[j] = bt * xv[j]; acc[j] = 0.f; }
      const float4* kr = reinterpret_cast<const float4*>(ks + tt * DKP + ns * SL);   // broadcast reads, 16 bytes each
      const float4* qr = reinterpret_cast<const float4*>(qs + tt * DKP + ns * SL);
#pragma unroll
      for (int i = 0; i < NPT / 4; ++i) {
        const float4 k4 = kr[i], q4 = qr[i];
#pragma unroll
        for (int j = 0; j < PP; ++j) {
          S[j][4 * i] = fmaf(av, S[j][4 * i], bv[j] * k4.x);         acc[j] = fmaf(S[j][4 * i], q4.x, acc[j]);
          S[j][4 * i + 1] = fmaf(av, S[j][4 * i + 1], bv[j] * k4.y); acc[j] = fmaf(S[j][4 * i + 1], q4.y, acc[j]);
          S[j][4 * i + 2] = fmaf(av, S[j][4 * i + 2], bv[j] * k4.z); acc[j] = fmaf(S[j][4 * i + 2], q4.z, acc[j]);
          S[j][4 * i + 3] = fmaf(av, S[j][4 * i + 3], bv[j] * k4.w); acc[j] = fmaf(S[j][4 * i + 3], q4.w, acc[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < PP; ++j) {
#pragma unroll
        for (int o = 1; o < NSL; o <<= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
        if (live[j] && ns == 0) a.y[(tb + tt) * a.ldy + static_cast<int64_t>(h) * a.dv + p + j * half] = fmaf(d, xv[j], acc[j]);
      }
    }
    __syncthreads();   // the copy issued in the next iteration overwrites this stage
  }
#pragma unroll
  for (int j = 0; j < PP; ++j)
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = ns * NPT + i;
      if (live[j] && n < a.dk) sp[static_cast<int64_t>(n) * a.dv + p + j * half] = S[j][i];
    }
}


struct DeltaArgs {
  float* y; int64_t ldy;
  const float *q, *k, *v; int64_t ldq, ldk, ldv;
  int group_div;                       // head h reads q / k of group h / group_div
  const float* decay; int64_t ldd;     // [n, heads * dk]: decay of every key channel
  const float* beta; int64_t ldb;      // [n, heads]
  float* state;                        // [slots, heads, dk, dv]
  const int32_t *seq_slot, *cu_tokens; const int64_t* positions;
  int heads, dk, dv;
};

// The gated delta rule, laid out as linear_recurrence_kernel (CTA = (head, sequence, slice of dv); a thread keeps PP columns x NPT
// rows of S in registers, NSL row slices of a column in neighbouring lanes; kRecTile tokens staged with cp.async two stages
// deep).  Per token one pass over the registers decays S and accumulates both S^T k and S^T q of the DECAYED state; after the
// lanes' partial sums meet (shuffles) u = beta (v - S^T k) is known, a second pass adds k u^T, and the read-out of the updated
// state is  S^T q + u (k . q)  — no third pass.
template <int NPT, int NSL, int PP>
__global__ void __launch_bounds__(512) gated_delta_kernel(const DeltaArgs a, int pb, int vec) {
  extern __shared__ __align__(16) float sm[];
  constexpr int SL = NPT + 4, DKP = SL * NSL;
  const int pbp = (pb + 3) & ~3;
  const int stage = kRecTile * (3 * DKP + pbp + 4);
  const int h = blockIdx.x, s = blockIdx.y, p0 = blockIdx.z * pb;
  const int tid = threadIdx.x, ns = tid % NSL, pl = tid / NSL, p = p0 + pl, half = (pb + PP - 1) / PP;
  bool live[PP];
#pragma unroll
  for (int j = 0; j < PP; ++j) live[j] = pl < half && pl + j * half < pb && p + j * half < a.dv;
  const int t0 = a.cu_tokens[s], t1 = a.cu_tokens[s + 1];
  const int slot = a.seq_slot[s];
  if (t1 <= t0) return;
  if (slot < 0) {  // padding sequence of a captured batch: defined output, no state
    for (int t = t0; t < t1; ++t)
#pragma unroll
      for (int j = 0; j < PP; ++j)
        if (live[j] && ns == 0) a.y[t * a.ldy + static_cast<int64_t>(h) * a.dv + p + j * half] = 0.f;
    return;
  }
  const int g = h / a.group_div;
  for (int e = tid; e < 2 * stage; e += blockDim.x) sm[e] = 0.f;   // rows beyond dk and columns beyond dv stay zero
  __syncthreads();
  const int ncol = min(pb, a.dv - p0);
  auto issue = [&](int tb, int buf) {
    float* ks = sm + buf * stage;
    float* qs = ks + kRecTile * DKP;
    float* gs = qs + kRecTile * DKP;
    float* vs = gs + kRecTile * DKP;
    float* bs = vs + kRecTile * pbp;
    const int cnt = min(kRecTile, t1 - tb);
    if (vec) {
      const int kch = a.dk / 4, vch = ncol / 4;
      for (int e = tid; e < cnt * kch; e += blockDim.x) {
        const int tt = e / kch, c = e - tt * kch;
        const int64_t t = tb + tt;
        const int dst = tt * DKP + (c * 4 / NPT) * SL + (c * 4) % NPT;
        cp_async_16(smem_u32(ks + dst), a.k + t * a.ldk + static_cast<int64_t>(g) * a.dk + c * 4, 16);
        cp_async_16(smem_u32(qs + dst), a.q + t * a.ldq + static_cast<int64_t>(g) * a.dk + c * 4, 16);
        cp_async_16(smem_u32(gs + dst), a.decay + t * a.ldd + static_cast<int64_t>(h) * a.dk + c * 4, 16);
      }
      for (int e = tid; e < cnt * vch; e += blockDim.x) {
        const int tt = e / vch, c = e - tt * vch;
        cp_async_16(smem_u32(vs + tt * pbp + c * 4), a.v + static_cast<int64_t>(tb + tt) * a.ldv + static_cast<int64_t>(h) * a.dv + p0 + c * 4, 16);
      }
    } else {
      for (int e = tid; e < cnt * a.dk; e += blockDim.x) {
        const int tt = e / a.dk, n = e - tt * a.dk;
        const int64_t t = tb + tt;
        const int dst = tt * DKP + (n / NPT) * SL + n % NPT;
        cp_async_4(smem_u32(ks + dst), a.k + t * a.ldk + static_cast<int64_t>(g) * a.dk + n);
        cp_async_4(smem_u32(qs + dst), a.q + t * a.ldq + static_cast<int64_t>(g) * a.dk + n);
        cp_async_4(smem_u32(gs + dst), a.decay + t * a.ldd + static_cast<int64_t>(h) * a.dk + n);
      }
      for (int e = tid; e < cnt * ncol; e += blockDim.x) {
        const int tt = e / ncol, c = e - tt * ncol;
        cp_async_4(smem_u32(vs + tt * pbp + c), a.v + static_cast<int64_t>(tb + tt) * a.ldv + static_cast<int64_t>(h) * a.dv + p0 + c);
      }
    }
    if (tid < cnt) cp_async_4(smem_u32(bs + tid), a.beta + (tb + tid) * a.ldb + h);
    cp_async_commit();
  };
  issue(t0, 0);
  float S[PP][NPT];
  float* sp = a.state + ((static_cast<int64_t>(slot) * a.heads + h) * a.dk) * a.dv;
  const bool fresh = a.positions[t0] == 0;
#pragma unroll
  for (int j = 0; j < PP; ++j)
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = ns * NPT + i;
      S[j][i] = (!fresh && live[j] && n < a.dk) ? sp[static_cast<int64_t>(n) * a.dv + p + j * half] : 0.f;
    }
  int buf = 0;
  for (int tb = t0; tb < t1; tb += kRecTile, buf ^= 1) {
    const int cnt = min(kRecTile, t1 - tb);
    if (tb + kRecTile < t1) { issue(tb + kRecTile, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const float* ks = sm + buf * stage;
    const float* qs = ks + kRecTile * DKP;
    const float* gs = qs + kRecTile * DKP;
    const float* vs = gs + kRecTile * DKP;
    const float* bs = vs + kRecTile * pbp;
    for (int tt = 0; tt < cnt; ++tt) {
      const float bt = bs[tt];
      float xv[PP], rk[PP], rq[PP], kq = 0.f;
#pragma unroll
      for (int j = 0; j < PP; ++j) { xv[j] = vs[tt * pbp + (live[j] ? pl + j * half : 0)]; rk[j] = 0.f; rq[j] = 0.f; }
      const float4* kr = reinterpret_cast<const float4*>(ks + tt * DKP + ns * SL);   // broadcast reads, 16 bytes each
      const float4* qr = reinterpret_cast<const float4*>(qs + tt * DKP + ns * SL);
      const float4* gr = reinterpret_cast<const float4*>(gs + tt * DKP + ns * SL);
#pragma unroll
      for (int i = 0; i < NPT / 4; ++i) {
        const float4 k4 = kr[i], q4 = qr[i], g4 = gr[i];
        kq = fmaf(k4.x, q4.x, fmaf(k4.y, q4.y, fmaf(k4.z, q4.z, fmaf(k4.w, q4.w, kq))));
#pragma unroll
        for (int j = 0; j < PP; ++j) {
          S[j][4 * i] *= g4.x;     rk[j] = fmaf(S[j][4 * i], k4.x, rk[j]);     rq[j] = fmaf(S[j][4 * i], q4.x, rq[j]);
          S[j][4 * i + 1] *= g4.y; rk[j] = fmaf(S[j][4 * i + 1], k4.y, rk[j]); rq[j] = fmaf(S[j][4 * i + 1], q4.y, rq[j]);
          S[j][4 * i + 2] *= g4.z; rk[j] = fmaf(S[j][4 * i + 2], k4.z, rk[j]); rq[j] = fmaf(S[j][4 * i + 2], q4.z, rq[j]);
          S[j][4 * i + 3] *= g4.w; rk[j] = fmaf(S[j][4 * i + 3], k4.w, rk[j]); rq[j] = fmaf(S[j][4 * i + 3], q4.w, rq[j]);
        }
      }
#pragma unroll
      for (int o = 1; o < NSL; o <<= 1) {
        kq += __shfl_xor_sync(0xffffffffu, kq, o);
#pragma unroll
        for (int j = 0; j < PP; ++j) { rk[j] += __shfl_xor_sync(0xffffffffu, rk[j], o); rq[j] += __shfl_xor_sync(0xffffffffu, rq[j], o); }
      }
      float u[PP];
#pragma unroll
      for (int j = 0; j < PP; ++j) {
        u[j] = bt * (xv[j] - rk[j]);
        if (live[j] && ns == 0) a.y[(tb + tt) * a.ldy + static_cast<int64_t>(h) * a.dv + p + j * half] = fmaf(u[j], kq, rq[j]);
      }
#pragma unroll
      for (int i = 0; i < NPT / 4; ++i) {
        const float4 k4 = kr[i];
#pragma unroll
        for (int j = 0; j < PP; ++j) {
          S[j][4 * i] = fmaf(k4.x, u[j], S[j][4 * i]);
          S[j][4 * i + 1] = fmaf(k4.y, u[j], S[j][4 * i + 1]);
          S[j][4 * i + 2] = fmaf(k4.z, u[j], S[j][4 * i + 2]);
          S[j][4 * i + 3] = fmaf(k4.w, u[j], S[j][4 * i + 3]);
        }
      }
    }
    __syncthreads();   // the copy issued in the next iteration overwrites this stage
  }
#pragma unroll
  for (int j = 0; j < PP; ++j)
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = ns * NPT + i;
      if (live[j] && n < a.dk) sp[static_cast<int64_t>(n) * a.dv + p + j * half] = S[j][i];
    }
}

struct DeltaPrepArgs {
  float *q, *k, *beta, *decay; int64_t ldq, ldk, ldb, ldd;
  const float *a_log, *dt_bias;
  int heads, groups, dk; float q_scale, unit_eps;
};

// CTA per token: the warps take the 2 * groups vectors of q and k (unit length; q also scaled), then all threads the
// element-wise parts (beta, decay).
__global__ void __launch_bounds__(128) delta_prepare_kernel(const DeltaPrepArgs a) {
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int u = warp; u < 2 * a.groups; u += 4) {
    const bool is_q = u < a.groups;
    float* x = is_q ? a.q + t * a.ldq + static_cast<int64_t>(u) * a.dk : a.k + t * a.ldk + static_cast<int64_t>(u - a.groups) * a.dk;
    float sq = 0.f;
    for (int c = lane; c < a.dk; c += 32) sq = fmaf(x[c], x[c], sq);
    const float r = (is_q ? a.q_scale : 1.0f) / sqrtf(warp_sum(sq) + a.unit_eps);
    for (int c = lane; c < a.dk; c += 32) x[c] *= r;
  }
  for (int h = threadIdx.x; h < a.heads; h += blockDim.x) {
    float* b = a.beta + t * a.ldb + h;
    *b = 1.0f / (1.0f + expf(-*b));
  }
  const int hd = a.heads * a.dk;
  for (int e = threadIdx.x; e < hd; e += blockDim.x) {
    float* d = a.decay + t * a.ldd + e;
    const float x = *d + a.dt_bias[e];
    const float dt = x > 20.f ? x : log1pf(expf(x));
    *d = expf(-expf(a.a_log[e / a.dk]) * dt);
  }
}

// The same in 16-byte steps (dk a multiple of 4, at most 512; aligned rows): every vector is read once.
__global__ void __launch_bounds__(256) delta_prepare_vec_kernel(const DeltaPrepArgs a) {
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nv = a.dk / 4;
  for (int u = warp; u < 2 * a.groups; u += 8) {
    const bool is_q = u < a.groups;
    float4* x = reinterpret_cast<float4*>(is_q ? a.q + t * a.ldq + static_cast<int64_t>(u) * a.dk : a.k + t * a.ldk + static_cast<int64_t>(u - a.groups) * a.dk);
    float4 v[4];
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = lane + 32 * k;
      if (c < nv) { v[k] = x[c]; sq += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w; }
    }
    const float r = (is_q ? a.q_scale : 1.0f) / sqrtf(warp_sum(sq) + a.unit_eps);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = lane + 32 * k;
      if (c < nv) x[c] = make_float4(v[k].x * r, v[k].y * r, v[k].z * r, v[k].w * r);
    }
  }
  for (int h = threadIdx.x; h < a.heads; h += blockDim.x) {
    float* b = a.beta + t * a.ldb + h;
    *b = 1.0f / (1.0f + expf(-*b));
  }
  auto decay = [](float raw, float bias, float ea) {
    const float x = raw + bias;
    const float dt = x > 20.f ? x : log1pf(expf(x));
    return expf(-ea * dt);
  };
  const int hd4 = a.heads * nv;
  float4* d = reinterpret_cast<float4*>(a.decay + t * a.ldd);
  for (int e = threadIdx.x; e < hd4; e += blockDim.x) {
    const float ea = expf(a.a_log[e / nv]);
    const float4 raw = d[e], b = reinterpret_cast<const float4*>(a.dt_bias)[e];
    d[e] = make_float4(decay(raw.x, b.x, ea), decay(raw.y, b.y, ea), decay(raw.z, b.z, ea), decay(raw.w, b.w, ea));
  }
}

struct ConvArgs {
  float* out; int64_t ldo;
  const float* in; int64_t ldi;
  const float *w, *b;        // [channels, taps], [channels]
  float* state;              // [slots, taps - 1, channels]: raw inputs of the taps - 1 tokens before the next one, oldest first
  const int32_t *tok_seq, *seq_slot, *cu_tokens; const int64_t* positions;
  int n, channels, taps, silu;
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float gate_f(float x, int act) { return act == 0 ? silu_f(x) : 1.0f / (1.0f + expf(-x)); }   // 0: SiLU, 1: sigmoid

// out[t, c] = act(b[c] + sum_j w[c, j] * in(position(t) - (taps - 1 - j), c)); inputs before the portion come from the
// state, inputs before the sequence are zero.  CTA = one token x a run of channels: the token's metadata is read once,
// channels are contiguous across the threads.
__global__ void __launch_bounds__(256) causal_conv_kernel(const ConvArgs a) {
  const int t = blockIdx.x;
  const int s = a.tok_seq[t], slot = a.seq_slot[s];
  const int c0 = a.cu_tokens[s];
  const int64_t p = a.positions[t], pf = a.positions[c0];
  const float* st = slot >= 0 ? a.state + static_cast<int64_t>(slot) * (a.taps - 1) * a.channels : nullptr;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < a.channels; c += gridDim.y * blockDim.x) {
    if (slot < 0) { a.out[t * a.ldo + c] = 0.f; continue; }
    float acc = a.b ? a.b[c] : 0.f;
    for (int j = 0; j < a.taps; ++j) {
      const int back = a.taps - 1 - j;
      const int64_t ps = p - back;
      if (ps < 0) continue;
      float x;
      if (t - back >= c0) x = a.in[static_cast<int64_t>(t - back) * a.ldi + c];
      else x = st[(ps - (pf - (a.taps - 1))) * a.channels + c];
      acc = fmaf(a.w[static_cast<int64_t>(c) * a.taps + j], x, acc);
    }
    a.out[t * a.ldo + c] = a.silu ? silu_f(acc) : acc;
  }
}

// The same for short windows (TAPS <= 4), one thread per channel walking a run of tokens with the window in registers: every
// input is read once.  Where a run enters a new sequence the window is rebuilt from the batch or the sequence's state.
template <int TAPS>
__global__ void __launch_bounds__(256) causal_conv_window_kernel(const ConvArgs a, int run) {
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.channels) return;
  float w[TAPS], win[TAPS > 1 ? TAPS - 1 : 1];
#pragma unroll
  for (int j = 0; j < TAPS; ++j) w[j] = a.w[static_cast<int64_t>(c) * TAPS + j];
  const float bias = a.b ? a.b[c] : 0.f;
  const int t_begin = blockIdx.x * run, t_end = min(a.n, t_begin + run);
  int cur = -1, slot = -1;
  for (int t = t_begin; t < t_end; ++t) {
    const int s = a.tok_seq[t];
    if (s != cur) {
      cur = s;
      slot = a.seq_slot[s];
      const int c0 = a.cu_tokens[s];
      const int64_t p = a.positions[t], pf = a.positions[c0];
#pragma unroll
      for (int k = 0; k < TAPS - 1; ++k) {
        const int back = TAPS - 1 - k;
        const int64_t ps = p - back;
        float x = 0.f;
        if (slot >= 0 && ps >= 0)
          x = t - back >= c0 ? a.in[static_cast<int64_t>(t - back) * a.ldi + c]
                             : a.state[(static_cast<int64_t>(slot) * (TAPS - 1) + (ps - (pf - (TAPS - 1)))) * a.channels + c];
        win[k] = x;
      }
    }
    if (slot < 0) { a.out[t * a.ldo + c] = 0.f; continue; }
    const float x = a.in[static_cast<int64_t>(t) * a.ldi + c];
    float acc = fmaf(w[TAPS - 1], x, bias);
#pragma unroll
    for (int k = 0; k < TAPS - 1; ++k) acc = fmaf(w[k], win[k], acc);
    a.out[t * a.ldo + c] = a.silu ? silu_f(acc) : acc;
#pragma unroll
    for (int k = 0; k + 1 < TAPS - 1; ++k) win[k] = win[k + 1];
    if (TAPS > 1) win[TAPS - 2] = x;
  }
}

constexpr int kMaxTaps = 16;

// After the convolution: the state becomes the raw inputs of the last taps - 1 positions (old state entries shift down when
// the portion is shorter than that).  One thread per (sequence, channel).
__global__ void conv_state_kernel(const ConvArgs a, int n_seqs) {
  const int64_t total = static_cast<int64_t>(n_seqs) * a.channels;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int s = static_cast<int>(i / a.channels), c = static_cast<int>(i % a.channels);
    const int slot = a.seq_slot[s], c0 = a.cu_tokens[s], len = a.cu_tokens[s + 1] - c0;
    if (slot < 0 || len <= 0) continue;
    const int64_t pf = a.positions[c0], pe = pf + len;
    float* st = a.state + static_cast<int64_t>(slot) * (a.taps - 1) * a.channels;
    float nv[kMaxTaps];
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k) {
      if (k >= a.taps - 1) break;
      const int64_t ps = pe - (a.taps - 1) + k;
      float x = 0.f;
      if (ps >= pf) x = a.in[(c0 + (ps - pf)) * a.ldi + c];
      else if (ps >= 0) x = st[(ps - (pf - (a.taps - 1))) * a.channels + c];
      nv[k] = x;
    }
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k) {
      if (k >= a.taps - 1) break;
      st[static_cast<int64_t>(k) * a.channels + c] = nv[k];
    }
  }
}

__global__ void ssd_prepare_kernel(float* __restrict__ step, float* __restrict__ decay, const float* __restrict__ raw, int64_t ldr,
                                   const float* __restrict__ dt_bias, const float* __restrict__ a_log, int64_t n, int heads) {
  const int64_t total = n * heads;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / heads;
    const int h = static_cast<int>(i - t * heads);
    const float x = raw[t * ldr + h] + dt_bias[h];
    const float dt = x > 20.f ? x : log1pf(expf(x));
    step[i] = dt;
    decay[i] = expf(-expf(a_log[h]) * dt);
  }
}

// x[t, h * head_stride + i] for i < dims: (u, v) = (x[i], x[i + dims/2]) -> (u cos - v sin, v cos + u sin), then * scale (all
// `dim` values of the head are scaled).  table: [max_pos, dims/2, 2] (cos, sin) from f64 angles.
__global__ void rotate_half_kernel(float* __restrict__ x, int64_t ldx, const int64_t* __restrict__ positions, const float* __restrict__ table,
                                   int max_pos, int64_t n, int heads, int dim, int dims, float scale) {
  const int half = dims / 2, per = dim - half;  // work items per head: pairs + unrotated tail
  const int64_t total = n * heads * per;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t th = i / per;
    const int e = static_cast<int>(i - th * per);
    const int64_t t = th / heads;
    const int h = static_cast<int>(th - t * heads);
    float* xh = x + t * ldx + static_cast<int64_t>(h) * dim;
    if (e < half) {
      int64_t p = positions[t];
      p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
      const float2 cs = reinterpret_cast<const float2*>(table)[p * half + e];
      const float u = xh[e], v = xh[e + half];
      xh[e] = (u * cs.x - v * cs.y) * scale;
      xh[e + half] = (v * cs.x + u * cs.y) * scale;
    } else if (scale != 1.0f) {
      xh[e + half] *= scale;
    }
  }
}

// One CTA per (token, part): parts of `gs` values.  gate_first: t = y * silu(z), out = rms(t) * w;  else out = rms(y) * silu(z) [* w].
template <typename TO>
__global__ void __launch_bounds__(128) gated_group_norm_kernel(TO* __restrict__ out, int64_t ldo, const float* __restrict__ y, int64_t ldy,
                                                               const float* __restrict__ z, int64_t ldz, const float* __restrict__ w, int gs,
                                                               int parts, float eps, int gate_first, int act, int wst) {
  __shared__ float red[4];
  const int64_t t = blockIdx.x / parts;
  const int g = blockIdx.x % parts;
  const float* yr = y + t * ldy + static_cast<int64_t>(g) * gs;
  const float* zr = z + t * ldz + static_cast<int64_t>(g) * gs;
  float sq = 0.f;
  for (int c = threadIdx.x; c < gs; c += blockDim.x) {
    float v = yr[c];
    if (gate_first) v *= gate_f(zr[c], act);
    sq = fmaf(v, v, sq);
  }
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  const float r = rsqrtf((red[0] + red[1] + red[2] + red[3]) / gs + eps);
  for (int c = threadIdx.x; c < gs; c += blockDim.x) {
    float v = yr[c];
    const float sg = gate_f(zr[c], act);
    v = gate_first ? v * sg * r : v * r * sg;
    if (w) v *= w[static_cast<int64_t>(g) * wst + c];
    if (sizeof(TO) == 2) reinterpret_cast<bf16*>(out)[t * ldo + static_cast<int64_t>(g) * gs + c] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(out)[t * ldo + static_cast<int64_t>(g) * gs + c] = v;
  }
}

// The same with the part's values held in registers (one global pass): parts of up to 2048 values in 16-byte vectors.
template <typename TO>
__global__ void __launch_bounds__(128) gated_group_norm_vec_kernel(TO* __restrict__ out, int64_t ldo, const float* __restrict__ y, int64_t ldy,
                                                                   const float* __restrict__ z, int64_t ldz, const float* __restrict__ w, int gs,
                                                                   int parts, float eps, int gate_first, int act, int wst) {
  __shared__ float red[4];
  const int64_t t = blockIdx.x / parts;
  const int g = blockIdx.x % parts, nv = gs / 4;
  const float4* yr = reinterpret_cast<const float4*>(y + t * ldy + static_cast<int64_t>(g) * gs);
  const float4* zr = reinterpret_cast<const float4*>(z + t * ldz + static_cast<int64_t>(g) * gs);
  float4 v[4], sg[4];
  float sq = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = threadIdx.x + 128 * k;
    if (c < nv) {
      v[k] = yr[c];
      const float4 zz = zr[c];
      sg[k] = make_float4(gate_f(zz.x, act), gate_f(zz.y, act), gate_f(zz.z, act), gate_f(zz.w, act));
      if (gate_first) { v[k].x *= sg[k].x; v[k].y *= sg[k].y; v[k].z *= sg[k].z; v[k].w *= sg[k].w; }
      sq += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
  }
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  const float r = rsqrtf((red[0] + red[1] + red[2] + red[3]) / gs + eps);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = threadIdx.x + 128 * k;
    if (c < nv) {
      float4 o = make_float4(v[k].x * r, v[k].y * r, v[k].z * r, v[k].w * r);
      if (!gate_first) { o.x *= sg[k].x; o.y *= sg[k].y; o.z *= sg[k].z; o.w *= sg[k].w; }
      if (w) {
        const float4 ww = reinterpret_cast<const float4*>(w + static_cast<int64_t>(g) * wst)[c];
        o.x *= ww.x; o.y *= ww.y; o.z *= ww.z; o.w *= ww.w;
      }
      const int64_t at = t * ldo + static_cast<int64_t>(g) * gs + 4 * c;
      if (sizeof(TO) == 2) *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(out) + at) = make_uint2(pack_bf16x2(o.x, o.y), pack_bf16x2(o.z, o.w));
      else *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + at) = o;
    }
  }
}

// Parts of up to 512 values: one WARP per (token, part), four parts per CTA, the part's values in registers.
template <typename TO>
__global__ void __launch_bounds__(128) gated_group_norm_warp_kernel(TO* __restrict__ out, int64_t ldo, const float* __restrict__ y, int64_t ldy,
                                                                    const float* __restrict__ z, int64_t ldz, const float* __restrict__ w, int gs,
                                                                    int parts, int64_t items, float eps, int gate_first, int act, int wst) {
  const int lane = threadIdx.x & 31, nv = gs / 4;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (item >= items) return;
  const int64_t t = item / parts;
  const int g = static_cast<int>(item - t * parts);
  const float4* yr = reinterpret_cast<const float4*>(y + t * ldy + static_cast<int64_t>(g) * gs);
  const float4* zr = reinterpret_cast<const float4*>(z + t * ldz + static_cast<int64_t>(g) * gs);
  float4 v[4], sg[4];
  float sq = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = lane + 32 * k;
    if (c < nv) {
      v[k] = yr[c];
      const float4 zz = zr[c];
      sg[k] = make_float4(gate_f(zz.x, act), gate_f(zz.y, act), gate_f(zz.z, act), gate_f(zz.w, act));
      if (gate_first) { v[k].x *= sg[k].x; v[k].y *= sg[k].y; v[k].z *= sg[k].z; v[k].w *= sg[k].w; }
      sq += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
  }
  const float r = rsqrtf(warp_sum(sq) / gs + eps);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = lane + 32 * k;
    if (c < nv) {
      float4 o = make_float4(v[k].x * r, v[k].y * r, v[k].z * r, v[k].w * r);
      if (!gate_first) { o.x *= sg[k].x; o.y *= sg[k].y; o.z *= sg[k].z; o.w *= sg[k].w; }
      if (w) {
        const float4 ww = reinterpret_cast<const float4*>(w + static_cast<int64_t>(g) * wst)[c];
        o.x *= ww.x; o.y *= ww.y; o.z *= ww.z; o.w *= ww.w;
      }
      const int64_t at = t * ldo + static_cast<int64_t>(g) * gs + 4 * c;
      if (sizeof(TO) == 2) *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(out) + at) = make_uint2(pack_bf16x2(o.x, o.y), pack_bf16x2(o.z, o.w));
      else *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + at) = o;
    }
  }
}

inline unsigned grid_for(int64_t total) {
  int64_t b = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  return static_cast<unsigned>(b > cap ? cap : (b < 1 ? 1 : b));
}

template <int NPT, int NSL, int PP>
int launch_recurrence(const RecArgs& a, int n_seqs, cudaStream_t st) {
  int pb = a.dv;                                  // columns per CTA
  const int max_pb = 512 / NSL * PP;
  if (pb > max_pb) pb = max_pb;
  // more CTAs when few (sequence, head) pairs would leave SMs idle: split the columns (each column is independent)
  while (pb > 32 && static_cast<int64_t>(a.heads) * n_seqs * ((a.dv + pb - 1) / pb) < sm_count() && pb % 2 == 0) pb /= 2;
  const int threads = (((pb + PP - 1) / PP * NSL + 31) / 32) * 32;
  const size_t smem = 2 * static_cast<size_t>(kRecTile) * (2 * (NPT + 4) * NSL + ((pb + 3) & ~3) + 2) * sizeof(float);
  dim3 grid(a.heads, n_seqs, (a.dv + pb - 1) / pb);
  if (smem > 48 * 1024) NVLLM_CUDA(cudaFuncSetAttribute(linear_recurrence_kernel<NPT, NSL, PP>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  // 16-byte copies when every staged row starts and ends on a 16-byte boundary
  const int vec = a.dk % 4 == 0 && a.dv % 4 == 0 && pb % 4 == 0 && a.ldq % 4 == 0 && a.ldk % 4 == 0 && a.ldv % 4 == 0 && aligned16(a.q) &&
                  aligned16(a.k) && aligned16(a.v);
  linear_recurrence_kernel<NPT, NSL, PP><<<grid, threads, smem, st>>>(a, pb, vec);
  NVLLM_LAUNCH_CHECK("linear_recurrence_kernel");
  return 0;
}


template <int NPT, int NSL, int PP>
int launch_delta(const DeltaArgs& a, int n_seqs, cudaStream_t st) {
  int pb = a.dv;                                  // columns per CTA
  const int max_pb = 512 / NSL * PP;
  if (pb > max_pb) pb = max_pb;
  while (pb > 32 && static_cast<int64_t>(a.heads) * n_seqs * ((a.dv + pb - 1) / pb) < sm_count() && pb % 2 == 0) pb /= 2;
  const int threads = (((pb + PP - 1) / PP * NSL + 31) / 32) * 32;
  const size_t smem = 2 * static_cast<size_t>(kRecTile) * (3 * (NPT + 4) * NSL + ((pb + 3) & ~3) + 4) * sizeof(float);
  dim3 grid(a.heads, n_seqs, (a.dv + pb - 1) / pb);
  if (smem > 48 * 1024) NVLLM_CUDA(cudaFuncSetAttribute(gated_delta_kernel<NPT, NSL, PP>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  const int vec = a.dk % 4 == 0 && a.dv % 4 == 0 && pb % 4 == 0 && a.ldq % 4 == 0 && a.ldk % 4 == 0 && a.ldv % 4 == 0 && a.ldd % 4 == 0 &&
                  aligned16(a.q) && aligned16(a.k) && aligned16(a.v) && aligned16(a.decay);
  gated_delta_kernel<NPT, NSL, PP><<<grid, threads, smem, st>>>(a, pb, vec);
  NVLLM_LAUNCH_CHECK("gated_delta_kernel");
  return 0;
}

}  // namespace
}  // namespace nvllm

using namespace nvllm;

extern "C" int nvllm_delta_prepare(float* q, int64_t ldq, float* k, int64_t ldk, float* beta, int64_t ldb, float* decay, int64_t ldd,
                                   const float* a_log, const float* dt_bias, int32_t n, int32_t heads, int32_t groups, int32_t dk,
                                   float q_scale, float unit_eps, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && heads > 0 && groups > 0 && dk > 0 && ldq >= static_cast<int64_t>(groups) * dk && ldk >= static_cast<int64_t>(groups) * dk &&
                      ldb >= heads && ldd >= static_cast<int64_t>(heads) * dk, NVLLM_ERR_ARG, "delta_prepare: sizes");
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(q && k && beta && decay && a_log && dt_bias, NVLLM_ERR_ARG, "delta_prepare: NULL");
  const DeltaPrepArgs a{q, k, beta, decay, ldq, ldk, ldb, ldd, a_log, dt_bias, heads, groups, dk, q_scale, unit_eps};
  if (dk % 4 == 0 && dk <= 512 && ldq % 4 == 0 && ldk % 4 == 0 && ldd % 4 == 0 && aligned16(q) && aligned16(k) && aligned16(decay) && aligned16(dt_bias)) {
    delta_prepare_vec_kernel<<<n, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
    NVLLM_LAUNCH_CHECK("delta_prepare_vec_kernel");
    return 0;
  }
  delta_prepare_kernel<<<n, 128, 0, static_cast<cudaStream_t>(stream)>>>(a);
  NVLLM_LAUNCH_CHECK("delta_prepare_kernel");
  return 0;
}

extern "C" int nvllm_gated_delta_recurrence(float* y, int64_t ldy, const float* q, int64_t ldq, const float* k, int64_t ldk, const float* v,
                                            int64_t ldv, const float* decay, int64_t ldd, const float* beta, int64_t ldb, float* state,
                                            const int32_t* seq_slot, const int32_t* cu_tokens, const int64_t* positions, int32_t n_seqs,
                                            int32_t heads, int32_t groups, int32_t dk, int32_t dv, void* stream) {
  NVLLM_CHECK_ARG(n_seqs >= 0 && heads > 0 && groups > 0 && heads % groups == 0 && dk > 0 && dk <= 512 && dv > 0, NVLLM_ERR_ARG,
                  "gated_delta_recurrence: seqs=%d heads=%d groups=%d dk=%d (<= 512) dv=%d", n_seqs, heads, groups, dk, dv);
  if (n_seqs == 0) return 0;
  NVLLM_CHECK_ARG(y && q && k && v && decay && beta && state && seq_slot && cu_tokens && positions, NVLLM_ERR_ARG, "gated_delta_recurrence: NULL");
  DeltaArgs a{y, ldy, q, k, v, ldq, ldk, ldv, heads / groups, decay, ldd, beta, ldb, state, seq_slot, cu_tokens, positions, heads, dk, dv};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dk <= 16) return launch_delta<16, 1, 2>(a, n_seqs, st);
  if (dk <= 32) return launch_delta<32, 1, 2>(a, n_seqs, st);
  if (dk <= 64) return launch_delta<32, 2, 2>(a, n_seqs, st);
  if (dk <= 128) {
    switch (knobs().delta_cfg) {   // A/B: how a column's rows are split over lanes and how many columns a thread holds
      case 1: return launch_delta<16, 8, 2>(a, n_seqs, st);
      case 2: return launch_delta<32, 4, 1>(a, n_seqs, st);
      case 3: return launch_delta<16, 8, 1>(a, n_seqs, st);
      case 4: return launch_delta<8, 16, 2>(a, n_seqs, st);
      case 5: return launch_delta<16, 8, 4>(a, n_seqs, st);
      default:
        // few (head, sequence) pairs: twice the lanes per column keep more warps in flight (one long prompt: 1.35 vs 2.03 ms
        // for 4096 tokens of 16 heads); otherwise the wider slices win (8 x 1024 tokens: 0.79 vs 0.77 ms, single tokens 41 vs 57 us)
        if (static_cast<int64_t>(heads) * n_seqs * 2 <= sm_count()) return launch_delta<16, 8, 2>(a, n_seqs, st);
        return launch_delta<32, 4, 2>(a, n_seqs, st);
    }
  }
  if (dk <= 256) return launch_delta<32, 8, 2>(a, n_seqs, st);
  return launch_delta<32, 16, 2>(a, n_seqs, st);
}

extern "C" int nvllm_linear_recurrence(float* y, int64_t ldy, const float* q, int64_t ldq, const float* k, int64_t ldk, const float* v,
                                       int64_t ldv, const float* decay, int32_t decay_per_token, const float* step,
                                       int32_t step_per_token, const float* skip, float* state, const int32_t* seq_slot,
                                       const int32_t* cu_tokens, const int64_t* positions, int32_t n_seqs, int32_t heads,
                                       int32_t groups, int32_t dk, int32_t dv, void* stream) {
  NVLLM_CHECK_ARG(n_seqs >= 0 && heads > 0 && groups > 0 && heads % groups == 0 && dk > 0 && dk <= 512 && dv > 0, NVLLM_ERR_ARG,
                  "linear_recurrence: seqs=%d heads=%d groups=%d dk=%d (<= 512) dv=%d", n_seqs, heads, groups, dk, dv);
  if (n_seqs == 0) return 0;
  NVLLM_CHECK_ARG(y && q && k && v && decay && state && seq_slot && cu_tokens && positions, NVLLM_ERR_ARG, "linear_recurrence: NULL");
  RecArgs a{y, ldy, q, k, v, ldq, ldk, ldv, heads / groups, decay, decay_per_token ? heads : 0, step, step_per_token ? heads : 0,
            skip, state, seq_slot, cu_tokens, positions, heads, dk, dv};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dk <= 16) return launch_recurrence<16, 1, 2>(a, n_seqs, st);
  if (dk <= 32) return launch_recurrence<32, 1, 2>(a, n_seqs, st);
  if (dk <= 64) return launch_recurrence<32, 2, 2>(a, n_seqs, st);
  if (dk <= 128) return launch_recurrence<32, 4, 2>(a, n_seqs, st);
  if (dk <= 256) return launch_recurrence<32, 8, 2>(a, n_seqs, st);
  return launch_recurrence<32, 16, 2>(a, n_seqs, st);
}

extern "C" int nvllm_causal_conv(float* out, int64_t ldo, const float* in, int64_t ldi, const float* w, const float* bias, float* state,
                                 const int32_t* tok_seq, const int32_t* seq_slot, const int32_t* cu_tokens, const int64_t* positions,
                                 int32_t n, int32_t n_seqs, int32_t channels, int32_t taps, int32_t silu, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && n_seqs >= 0 && channels > 0 && taps >= 1 && taps <= kMaxTaps, NVLLM_ERR_ARG,
                  "causal_conv: n=%d channels=%d taps=%d (1..16)", n, channels, taps);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(out && in && w && state && tok_seq && seq_slot && cu_tokens && positions && out != in, NVLLM_ERR_ARG, "causal_conv: NULL");
  ConvArgs a{out, ldo, in, ldi, w, bias, state, tok_seq, seq_slot, cu_tokens, positions, n, channels, taps, silu};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (taps >= 2 && taps <= 4 && n >= 8 * n_seqs) {   // runs of a sequence's tokens: worth a register window
    const int run = 32;
    dim3 grid(static_cast<unsigned>((n + run - 1) / run), static_cast<unsigned>((channels + 255) / 256));
    if (taps == 2) causal_conv_window_kernel<2><<<grid, 256, 0, st>>>(a, run);
    else if (taps == 3) causal_conv_window_kernel<3><<<grid, 256, 0, st>>>(a, run);
    else causal_conv_window_kernel<4><<<grid, 256, 0, st>>>(a, run);
  } else {
    dim3 grid(static_cast<unsigned>(n), static_cast<unsigned>(std::min(8, (channels + 255) / 256)));
    causal_conv_kernel<<<grid, 256, 0, st>>>(a);
  }
  NVLLM_LAUNCH_CHECK("causal_conv_kernel");
  if (taps > 1) {
    conv_state_kernel<<<grid_for(static_cast<int64_t>(n_seqs) * channels), 256, 0, st>>>(a, n_seqs);
    NVLLM_LAUNCH_CHECK("conv_state_kernel");
  }
  return 0;
}

extern "C" int nvllm_ssd_prepare(float* step, float* decay, const float* dt_raw, int64_t ld_raw, const float* dt_bias, const float* a_log,
                                 int32_t n, int32_t heads, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && heads > 0 && ld_raw >= heads, NVLLM_ERR_ARG, "ssd_prepare: sizes");
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(step && decay && dt_raw && dt_bias && a_log, NVLLM_ERR_ARG, "ssd_prepare: NULL");
  ssd_prepare_kernel<<<grid_for(static_cast<int64_t>(n) * heads), 256, 0, static_cast<cudaStream_t>(stream)>>>(step, decay, dt_raw, ld_raw, dt_bias,
                                                                                                           a_log, n, heads);
  NVLLM_LAUNCH_CHECK("ssd_prepare_kernel");
  return 0;
}

extern "C" int nvllm_rotate_half(float* x, int64_t ldx, const int64_t* positions, const float* table, int32_t max_pos, int32_t n,
                                 int32_t heads, int32_t dim, int32_t dims, float scale, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && heads > 0 && dim > 0 && dims >= 0 && dims % 2 == 0 && dims <= dim && max_pos > 0, NVLLM_ERR_ARG,
                  "rotate_half: heads=%d dim=%d dims=%d", heads, dim, dims);
  if (n == 0 || (dims == 0 && scale == 1.0f)) return 0;
  NVLLM_CHECK_ARG(x && positions && (table || dims == 0), NVLLM_ERR_ARG, "rotate_half: NULL");
  const int64_t total = static_cast<int64_t>(n) * heads * (dim - dims / 2);
  rotate_half_kernel<<<grid_for(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, ldx, positions, table, max_pos, n, heads, dim, dims, scale);
  NVLLM_LAUNCH_CHECK("rotate_half_kernel");
  return 0;
}

extern "C" int nvllm_gated_group_norm(void* out, int64_t ldo, const float* y, int64_t ldy, const float* gate, int64_t ldg, const float* w,
                                      int32_t n, int32_t cols, int32_t parts, float eps, int32_t gate_first, int32_t out_dtype,
                                      void* stream) {
  return nvllm_gated_group_norm_act(out, ldo, y, ldy, gate, ldg, w, 0, n, cols, parts, eps, gate_first, 0, out_dtype, stream);
}

extern "C" int nvllm_gated_group_norm_act(void* out, int64_t ldo, const float* y, int64_t ldy, const float* gate, int64_t ldg, const float* w,
                                          int32_t w_shared, int32_t n, int32_t cols, int32_t parts, float eps, int32_t gate_first,
                                          int32_t gate_act, int32_t out_dtype, void* stream) {
  NVLLM_CHECK_ARG(n >= 0 && cols > 0 && parts > 0 && cols % parts == 0 && (gate_act == 0 || gate_act == 1), NVLLM_ERR_ARG,
                  "gated_group_norm: cols=%d parts=%d gate_act=%d", cols, parts, gate_act);
  NVLLM_CHECK_ARG(out_dtype == NVLLM_BF16 || out_dtype == NVLLM_F32, NVLLM_ERR_DTYPE, "gated_group_norm: dtype %d", out_dtype);
  if (n == 0) return 0;
  NVLLM_CHECK_ARG(out && y && gate, NVLLM_ERR_ARG, "gated_group_norm: NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(static_cast<int64_t>(n) * parts);
  const int gs = cols / parts, wst = w_shared ? 0 : gs;
  const bool vec_ok = gs % 4 == 0 && ldo % 4 == 0 && ldy % 4 == 0 && ldg % 4 == 0 && aligned16(out) && aligned16(y) && aligned16(gate) && aligned16(w);
  if (vec_ok && gs <= 512) {
    const int64_t items = static_cast<int64_t>(n) * parts;
    const unsigned wgrid = static_cast<unsigned>((items + 3) / 4);
    if (out_dtype == NVLLM_BF16)
      gated_group_norm_warp_kernel<bf16><<<wgrid, 128, 0, st>>>(static_cast<bf16*>(out), ldo, y, ldy, gate, ldg, w, gs, parts, items, eps, gate_first, gate_act, wst);
    else
      gated_group_norm_warp_kernel<float><<<wgrid, 128, 0, st>>>(static_cast<float*>(out), ldo, y, ldy, gate, ldg, w, gs, parts, items, eps, gate_first, gate_act, wst);
    NVLLM_LAUNCH_CHECK("gated_group_norm_warp_kernel");
    return 0;
  }
  if (gs % 4 == 0 && gs <= 2048 && ldo % 4 == 0 && ldy % 4 == 0 && ldg % 4 == 0 && aligned16(out) && aligned16(y) && aligned16(gate) && aligned16(w)) {
    if (out_dtype == NVLLM_BF16)
      gated_group_norm_vec_kernel<bf16><<<grid, 128, 0, st>>>(static_cast<bf16*>(out), ldo, y, ldy, gate, ldg, w, gs, parts, eps, gate_first, gate_act, wst);
    else
      gated_group_norm_vec_kernel<float><<<grid, 128, 0, st>>>(static_cast<float*>(out), ldo, y, ldy, gate, ldg, w, gs, parts, eps, gate_first, gate_act, wst);
    NVLLM_LAUNCH_CHECK("gated_group_norm_vec_kernel");
    return 0;
  }
  if (out_dtype == NVLLM_BF16)
    gated_group_norm_kernel<bf16><<<grid, 128, 0, st>>>(static_cast<bf16*>(out), ldo, y, ldy, gate, ldg, w, gs, parts, eps, gate_first, gate_act, wst);
  else
    gated_group_norm_kernel<float><<<grid, 128, 0, st>>>(static_cast<float*>(out), ldo, y, ldy, gate, ldg, w, gs, parts, eps, gate_first, gate_act, wst);
  NVLLM_LAUNCH_CHECK("gated_group_norm_kernel");
  return 0;
}
