/*
 * nvllm.h — C ABI of the B200-native (sm_100a) paged-attention decode hot path.
 *
 * This is the drop-in boundary for ssvgopal/nano-vllm-rs.  The reference has no FFI of its own
 * (pure Rust on candle); each entry point below replaces one Rust method on the hot path and cites
 * it as  <file>:<lines>  relative to the reference tree.  The Rust-side binding a maintainer
 * would add is shown in INTEGRATION.md and rust/ffi.rs.
 *
 * Conventions (all entry points):
 *   - return 0 on success, <0 for an argument error (shape / alignment / dtype), >0 = cudaError_t;
 *     nvllm_last_error() returns a thread-local message for the last non-zero return.
 *   - the caller owns every buffer (inputs, outputs, KV cache, workspace) and the stream; kernels
 *     never allocate, free or synchronise and keep no global state, so every call is legal inside
 *     CUDA-graph capture.  Pointers are device pointers unless the name starts with `h_`.
 *     (Stated exceptions: nvllm_paged_decode_attention_static owns a per-GPU scratch array and is outside this
 *     paragraph's promises — read its own comment; nvllm_reload_env is not re-entrant; nvllm_comm_* are collectives.)
 *   - activations / weights / KV cache are bf16 (NVLLM_BF16); accumulation is fp32.
 *   - strides are in ELEMENTS.  The innermost (head_dim) dimension is always contiguous and every
 *     row start must be 16-byte aligned.
 *   - `stream` is a cudaStream_t passed as void*.
 */
#ifndef NVLLM_H_
#define NVLLM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NVLLM_VERSION 100 /* 0.1.0 */

enum nvllm_dtype { NVLLM_BF16 = 0, NVLLM_F32 = 1 };

enum nvllm_status {
  NVLLM_OK = 0,
  NVLLM_ERR_ARG = -1,       /* bad shape / null pointer / unsupported size */
  NVLLM_ERR_ALIGN = -2,     /* pointer or stride not 16-byte aligned        */
  NVLLM_ERR_DTYPE = -3,     /* dtype other than the documented one          */
  NVLLM_ERR_WORKSPACE = -4, /* workspace too small                          */
  NVLLM_ERR_STATE = -5,     /* engine-level call in the wrong state         */
  NVLLM_ERR_COMM = -6       /* NCCL / peer-memory failure                   */
};

int nvllm_version(void);
const char* nvllm_last_error(void);
/* 1 when a CUDA device of compute capability 10.x is visible, else 0 (never throws). */
int nvllm_device_ok(void);
/* The NVLLM_* environment knobs (A/B measurement switches) are parsed once per process, never on a
 * dispatch path; benchmark tools that sweep a knob inside one process call this after changing the environment.
 * NOT re-entrant, unlike every other entry point: it rewrites the knob set in place, so call it only while no other thread
 * is inside the library (a dispatch running concurrently could see half of the old set and half of the new). */
int nvllm_reload_env(void);

/* ------------------------------------------------------------------------------------------------
 * KV-cache layout descriptor.  The reference allocates each per-layer cache as
 * [num_blocks, block_size, num_kv_heads, head_dim]  (src/engine/model_runner.rs:379-389); that is
 *   block_stride = block_size*Hkv*D, token_stride = Hkv*D, head_stride = D.
 * The engine in this repo uses the head-major variant [num_blocks, Hkv, block_size, D]
 *   block_stride = Hkv*block_size*D, token_stride = D, head_stride = block_size*D
 * (64 KiB contiguous per (block, head)).  Kernels accept either through these strides.
 * slot s  ->  block s / block_size, offset s % block_size   (slot_mapping semantics of
 * src/layers/attention.rs:150-174 with a flat [num_blocks*block_size, ...] view).
 * ---------------------------------------------------------------------------------------------- */
typedef struct nvllm_kv_layout {
  int32_t block_size;    /* tokens per block (reference: 256, src/config.rs:94)           */
  int32_t num_kv_heads;  /* KV heads held by this rank (Hkv / tp)                           */
  int32_t head_dim;      /* 64 or 128                                                       */
  int32_t reserved;
  int64_t block_stride;  /* elements between consecutive blocks                            */
  int64_t token_stride;  /* elements between consecutive tokens inside a block             */
  int64_t head_stride;   /* elements between consecutive KV heads of one token             */
} nvllm_kv_layout;

/* K1 — replaces Attention::store_kv_cache (src/layers/attention.rs:150-174).
 * cache[slot_mapping[i]] = k[i], v[i] for i in [0, num_tokens); slot < 0 is skipped (padding rows
 * of a captured decode graph).  k, v: [num_tokens, Hkv, D] with `kv_token_stride` elements between
 * tokens (so they may be views into a packed qkv buffer).  Bit-exact copy. */
int nvllm_store_kvcache(const void* k, const void* v, void* k_cache, void* v_cache,
                        const int32_t* slot_mapping, int32_t num_tokens, int64_t kv_token_stride,
                        const nvllm_kv_layout* layout, int32_t dtype, void* stream);

/* K2 — replaces Attention::flash_attention_decode -> compute_attention_with_cache ->
 * gather_cached_kv -> compute_attention (src/layers/attention.rs:225-318,238-261).
 * out[b,h,:] = softmax(scale * q[b,h,:] . K[b,h/g]^T) . V[b,h/g] over the first context_lens[b]
 * slots of the blocks listed in block_tables[b,:] (entries < 0 are skipped, attention.rs:306).
 * q/out: [batch, H, D] with `q_token_stride` / `out_token_stride` elements between sequences.
 * block_tables: i32 [batch, max_blocks_per_seq] padded with -1 (model_runner.rs:280-293);
 * context_lens: i32 [batch] (model_runner.rs:275).  Split-K: `num_splits` >= 1 partitions of the
 * KV length per (sequence, kv head); 0 lets the library choose.  Workspace holds the fp32 partials
 * (only touched when the effective split count is > 1). */
size_t nvllm_paged_decode_workspace_bytes(int32_t batch, int32_t num_heads, int32_t head_dim,
                                          int32_t num_splits);
int nvllm_paged_decode_choose_splits(int32_t batch, int32_t num_heads, int32_t num_kv_heads,
                                     int32_t max_context_len);
int nvllm_paged_decode_attention(void* out, const void* q, const void* k_cache, const void* v_cache,
                                 const int32_t* block_tables, const int32_t* context_lens,
                                 int32_t batch, int32_t num_heads, int32_t max_blocks_per_seq,
                                 int64_t q_token_stride, int64_t out_token_stride,
                                 const nvllm_kv_layout* layout, float scale, void* workspace,
                                 size_t workspace_bytes, int32_t num_splits, int32_t dtype,
                                 void* stream);

/* nvllm_paged_decode_attention for callers that cannot provide a workspace.  NO COUNTERPART IN THE REFERENCE (its
 * decode attention is candle tensor ops that allocate freely); this exists for integrations, not for parity.
 *
 * Who needs it: a caller that sits where device memory cannot be obtained — an operator hook or host callback that is
 * handed only the tensors of one op, an embedder whose memory pool is fixed once serving starts, a C / Rust host with
 * no CUDA allocator of its own.  It still passes q, the caches, the tables and `out`; the f32 split-K partials go to an
 * array built into libnvllm.so's device image.  The call performs no cudaMalloc / cudaFree and calls no allocating
 * library routine.  Same arguments, kernels and results as nvllm_paged_decode_attention (bit for bit at an equal
 * num_splits), minus `workspace` / `workspace_bytes`.
 *
 * Limits and rules:
 *   - the array is nvllm_paged_decode_static_scratch_bytes() = 8 MiB, present on EVERY GPU that loads the library until
 *     the process exits.  A call that needs more — nvllm_paged_decode_workspace_bytes(batch, num_heads, head_dim,
 *     num_splits) > 8 MiB; num_splits = 0 resolves through nvllm_paged_decode_choose_splits first — returns
 *     NVLLM_ERR_WORKSPACE with the sizes in nvllm_last_error() and launches nothing.  One split needs no scratch at all.
 *   - the first call on each device looks up that device's address of the array (cudaGetSymbolAddress, with the calling
 *     thread's current device, which must be the device of `stream` and of every buffer) and remembers it.  Make that
 *     first call during set-up, before any CUDA stream capture begins.
 *   - all calls on a GPU share the one array.  Calls ordered on one stream are safe; calls that can overlap on the GPU
 *     (two streams, or two threads with a stream each) race on the partials and return garbage — serialise them or use
 *     the workspace variant.  The array keeps whatever the last call left; nothing needs clearing, because every
 *     partial a call reads was written by that same call. */
size_t nvllm_paged_decode_static_scratch_bytes(void);
int nvllm_paged_decode_attention_static(void* out, const void* q, const void* k_cache, const void* v_cache,
                                        const int32_t* block_tables, const int32_t* context_lens, int32_t batch,
                                        int32_t num_heads, int32_t max_blocks_per_seq, int64_t q_token_stride,
                                        int64_t out_token_stride, const nvllm_kv_layout* layout, float scale,
                                        int32_t num_splits, int32_t dtype, void* stream);

/* K7 + K1 + K2 in ONE launch for decode steps — replaces, per layer, what Qwen3Attention::forward does between qkv_proj
 * and o_proj (src/models/qwen3.rs:219-233): per-head q/k RMSNorm + RotaryEmbedding::forward
 * (src/layers/rotary_embedding.rs:23-48,145-158), Attention::store_kv_cache (src/layers/attention.rs:150-174) and
 * Attention::flash_attention_decode (:225-318).  qkv: the packed [q | k | v] rows of this step ([batch, (H+2Hkv)*D], read
 * only — nothing is written back into it); the step's K (normed, rotated) and V rows are stored at slot_mapping[b] (< 0:
 * skipped) and attended to from shared memory, so context_lens[b] COUNTS this step's token (context_lens - 1 tokens are
 * read through block_tables).  Same rounding points as nvllm_qknorm_rope_store followed by nvllm_paged_decode_attention
 * (bf16 after the norm, bf16 after the rotation); head_dim 128 only.  q_norm_w / k_norm_w NULL = no qk-norm. */
int nvllm_paged_decode_attention_fused(void* out, const void* qkv, const int64_t* positions, const float* cos_sin,
                                       const void* q_norm_w, const void* k_norm_w, float eps, int32_t max_position,
                                       void* k_cache, void* v_cache, const int32_t* slot_mapping,
                                       const int32_t* block_tables, const int32_t* context_lens, int32_t batch,
                                       int32_t num_heads, int32_t max_blocks_per_seq, int64_t qkv_token_stride,
                                       int64_t out_token_stride, const nvllm_kv_layout* layout, float scale,
                                       void* workspace, size_t workspace_bytes, int32_t num_splits, int32_t dtype,
                                       void* stream);

/* K3 / K4 — replaces Attention::flash_attention_varlen (+ create_causal_mask) and
 * flash_attention_varlen_with_cache (src/layers/attention.rs:177-222,321-339).
 * Causal attention per sequence i over q rows [cu_seqlens_q[i], cu_seqlens_q[i+1]) and keys
 * [cu_seqlens_k[i], cu_seqlens_k[i+1]); the mask is bottom-right aligned (query row j of Lq sees
 * keys 0 .. Lk-Lq+j), which is the plain causal mask when Lq == Lk.
 * If block_tables == NULL keys/values come from the dense k, v: [total_k, Hkv, D];
 * otherwise (prefix-cache prefill) they are read from the paged cache through block_tables[i,:]
 * (the new K/V of this step must already have been stored — note N2 in SURVEY.md §8).
 * total_q / total_k: rows of q / of the dense k, v (bounds of the TMA descriptors; total_k is ignored when paged).
 * Requires Lk >= Lq per sequence and head_dim == 128; runs on tcgen05 tensor cores. */
int nvllm_varlen_prefill_attention(void* out, const void* q, const void* k, const void* v,
                                   const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                   int32_t batch, int32_t total_q, int32_t total_k,
                                   int32_t max_seqlen_q, int32_t max_seqlen_k, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                                   int64_t q_token_stride, int64_t kv_token_stride,
                                   int64_t out_token_stride, const void* k_cache,
                                   const void* v_cache, const int32_t* block_tables,
                                   int32_t max_blocks_per_seq, const nvllm_kv_layout* layout,
                                   float scale, int32_t dtype, void* stream);

/* K5 — replaces LinearBase::forward of ReplicatedLinear / ColumnParallelLinear / RowParallelLinear /
 * QKVParallelLinear / MergedColumnParallelLinear and ParallelLMHead::compute_logits
 * (src/layers/linear.rs:228-239,354-356,437-439; src/layers/embed_head.rs:292-306).
 * y[M,N] = x[M,K] . w[N,K]^T   (x, w bf16 row-major with leading dimensions ldx, ldw; fp32
 * accumulate on tcgen05 tensor cores; y is bf16 or fp32 per `out_dtype`, leading dimension ldy).
 * K % 64 == 0, N % 8 == 0, ldx/ldw % 8 == 0.  workspace: nvllm_gemm_workspace_bytes() bytes
 * (TMA descriptors are passed by value, the workspace is only used for split-K partials; may be
 * NULL when that function returns 0). */
size_t nvllm_gemm_workspace_bytes(int32_t m, int32_t n, int32_t k);
int nvllm_gemm_bf16(void* y, const void* x, const void* w, int32_t m, int32_t n, int32_t k,
                    int64_t ldx, int64_t ldw, int64_t ldy, int32_t out_dtype, void* workspace,
                    size_t workspace_bytes, void* stream);
/* MergedColumnParallelLinear::forward followed by SiluAndMul::forward (linear.rs:437-439, activation.rs:46-63) in one
 * call: out[M, inter] = silu(x . Wgate^T) * (x . Wup^T), w_gate_up = [Wgate | Wup] packed row-wise ([2*inter, K]).
 * When inter %% 128 == 0 the activation runs in the GEMM epilogue (the B tile holds BN/2 gate rows + the matching BN/2
 * up rows; with CTA pairs one CTA stages the gate rows, its peer the up rows) and the [M, 2*inter] intermediate never
 * reaches HBM; other sizes use `workspace` (>= M*2*inter*2 bytes) for it.
 * Same rounding points as nvllm_gemm_bf16 + nvllm_silu_mul (bit-identical results). */
int nvllm_gemm_silu_mul_bf16(void* out, const void* x, const void* w_gate_up, int32_t m, int32_t inter, int32_t k,
                             int64_t ldx, int64_t ldw, int64_t ldout, void* workspace, size_t workspace_bytes,
                             void* stream);
/* QKVParallelLinear::forward (linear.rs:354-356) + the q/k norm, RotaryEmbedding::forward and Attention::store_kv_cache
 * that follow it (qwen3.rs:219-229, attention.rs:150-174) in ONE kernel: qkv[M, (H+2Hkv)*128] = x . Wqkv^T, each 128-wide
 * output tile being one head whose epilogue thread applies the same math (and rounding points) as
 * nvllm_qknorm_rope_store before writing the qkv row and, for k / v heads, the paged cache.  head_dim 128 only.
 * k_cache may be NULL (no store).  Equivalent to nvllm_gemm_bf16 + nvllm_qknorm_rope_store. */
int nvllm_gemm_qkv_rope_store(void* qkv, const void* x, const void* w_qkv, int32_t m, int32_t k, int64_t ldx, int64_t ldw,
                              const int64_t* positions, const float* cos_sin, const void* q_norm_w,
                              const void* k_norm_w, float eps, int32_t num_heads, int32_t num_kv_heads,
                              int32_t head_dim, int32_t max_position, void* k_cache, void* v_cache,
                              const int32_t* slot_mapping, const nvllm_kv_layout* layout, void* stream);
/* Plain CUDA-core version of the same contract; test infrastructure for the kernel above (used to
 * check large shapes on the device where the CPU oracle is too slow).  Never on the product path. */
int nvllm_gemm_bf16_simt(void* y, const void* x, const void* w, int32_t m, int32_t n, int32_t k,
                         int64_t ldx, int64_t ldw, int64_t ldy, int32_t out_dtype, void* stream);

/* K6 — replaces RMSNorm::forward_simple / forward_with_residual (src/layers/layernorm.rs:58-97)
 * and the residual adds of Qwen3Layer::forward (src/models/qwen3.rs:382,389).
 *   residual == NULL : out = rmsnorm(x) * w
 *   residual != NULL : residual <- bf16(residual + x) (in place);  out = rmsnorm(residual) * w
 * f32 math: v * w / sqrt(mean(v^2) + eps).  x/out: [num_tokens, hidden], contiguous rows. */
int nvllm_add_rmsnorm(void* out, const void* x, void* residual, const void* weight,
                      int32_t num_tokens, int32_t hidden, float eps, int32_t dtype, void* stream);

/* K7 (+K1 fused) — replaces RotaryEmbedding::forward / apply_rotary_emb_single
 * (src/layers/rotary_embedding.rs:23-48,136-158), the per-head q_norm/k_norm of the named Qwen3
 * architecture (absent in the reference, SURVEY.md §8 note N1) and, when k_cache != NULL, the
 * store_kv_cache call that follows (attention.rs:78-81).
 * In place on the packed qkv buffer [num_tokens, (H + 2*Hkv) * D] (q | k | v, linear.rs:331-340):
 *   q_h <- rope(rmsnorm_D(q_h) * q_norm_w),  k_h <- rope(rmsnorm_D(k_h) * k_norm_w)
 *   rope: half-split (NeoX) rotation [x1*c - x2*s | x2*c + x1*s], c,s = cos,sin(pos * theta^(-2j/D))
 *   taken from the fp32 table cos_sin: [max_position, D] = (cos[0..D/2) | sin[0..D/2)).
 * q_norm_w / k_norm_w may be NULL (no qk-norm: the reference's behaviour).  positions: i64. */
int nvllm_qknorm_rope_store(void* qkv, const int64_t* positions, const float* cos_sin,
                            const void* q_norm_w, const void* k_norm_w, float eps,
                            int32_t num_tokens, int32_t num_heads, int32_t num_kv_heads,
                            int32_t head_dim, int32_t max_position, void* k_cache, void* v_cache,
                            const int32_t* slot_mapping, const nvllm_kv_layout* layout,
                            int32_t dtype, void* stream);
/* Fills cos_sin [max_position, D] fp32 exactly as the oracle does (f64 inv_freq and angle, rounded
 * to f32) — rotary_embedding.rs:82-110 with the table kept in f32 (note N1). */
int nvllm_rope_table(float* cos_sin, int32_t max_position, int32_t head_dim, double theta,
                     void* stream);

/* K8 — replaces SiluAndMul::forward (src/layers/activation.rs:46-63).
 * out[t, j] = silu(x[t, j]) * x[t, inter + j],  x: [num_tokens, 2*inter], out: [num_tokens, inter]. */
int nvllm_silu_mul(void* out, const void* x, int32_t num_tokens, int32_t inter, int32_t dtype,
                   void* stream);

/* K9 / K10 — replaces VocabParallelEmbedding::forward (src/layers/embed_head.rs:77-97) and
 * ParallelLMHead::extract_last_tokens (embed_head.rs:272-289).
 * gather rows: out[i,:] = table[ids[i],:]  (ids i64).  With `row_index` semantic = last token of each
 * sequence use nvllm_gather_last_tokens: out[i,:] = x[cu_seqlens_q[i+1]-1, :]. */
int nvllm_embedding_gather(void* out, const void* table, const int64_t* ids, int32_t num_tokens,
                           int32_t hidden, int32_t vocab, int32_t dtype, void* stream);
int nvllm_gather_last_tokens(void* out, const void* x, const int32_t* cu_seqlens_q, int32_t batch,
                             int32_t hidden, int32_t dtype, void* stream);

/* K11 — replaces Sampler::greedy_sample (src/layers/sampler.rs:109-112): argmax over the vocab,
 * first maximum wins.  logits: [batch, vocab] (bf16 or f32, leading dimension ld).  Writes the token
 * id (+ vocab_offset, for vocab-sharded heads) to out_ids[b] (i64) and, if out_max != NULL, the
 * maximum as f32 to out_max[b] (used for the cross-rank combine, embed_head.rs:321-336). */
int nvllm_argmax(int64_t* out_ids, float* out_max, const void* logits, int32_t batch, int32_t vocab,
                 int64_t ld, int64_t vocab_offset, int32_t logits_dtype, void* stream);
/* Cross-rank combine of per-shard (max, id) pairs gathered as [tp, batch]: picks the largest max,
 * lowest shard on ties (== first maximum over the concatenated vocab). */
int nvllm_argmax_combine(int64_t* out_ids, const float* all_max, const int64_t* all_ids,
                         int32_t tp, int32_t batch, void* stream);
/* Puts the all-gathered vocab shards of a tensor-parallel LM head back into full rows — the gather the reference leaves as
 * a TODO (src/layers/embed_head.rs:321-336): out[b, r*vshard + j] = gathered[r, b, j] (f32).  With it every rank holds the
 * full [rows, vocab] logits and runs the same deterministic nvllm_sample: temperature / top-k / top-p under TP. */
int nvllm_assemble_vocab_shards(float* out, const float* gathered, int32_t tp, int32_t rows, int32_t vshard,
                                void* stream);

/* K12 — replaces Sampler::forward / batch_sample / sample_single (src/layers/sampler.rs:26-106,221-254) with its
 * helpers apply_top_k (:115-149), apply_top_p (:152-191), multinomial_sample (:194-203) and sample_gumbel (:205-219)
 * for a whole batch in one launch (one CTA per row; selections instead of the reference's two full sorts).
 * logits: f32 [batch, vocab] (leading dimension ld).  Per row b (all arrays are DEVICE pointers):
 *   temperatures[b] == 0  -> greedy argmax, first maximum wins (sampler.rs:79-81)
 *   otherwise s = logits / temperature; top_k[b] in (0, vocab) keeps the first k entries of the stable descending
 *   order (0 or NULL array = None); top_p[b] in (0, 1) keeps the shortest descending prefix whose softmax mass
 *   reaches p (other values or NULL array = None); token = argmax(s + gumbel), gumbel = -log(-log(u)).
 * The reference draws u from an unseeded RNG; here u[j] = ((mix64(row_seeds[b] + (j+1)*0x9E3779B97F4A7C15) >> 41)
 * + 0.5) * 2^-23 with mix64 = the splitmix64 finaliser — the same contract as oracle/layers.py, so a (seed, logits)
 * pair always yields the same token.  kept_count (i32 [batch]) / kept_mask (u8 [batch, vocab]) are optional
 * outputs describing the surviving set (parity tests); pass NULL in production. */
int nvllm_sample(int64_t* out_ids, const float* logits, int32_t batch, int32_t vocab, int64_t ld,
                 const float* temperatures, const int32_t* top_k, const float* top_p, const uint64_t* row_seeds,
                 int32_t* kept_count, uint8_t* kept_mask, void* stream);

/* C1 — the all-reduce the reference leaves as a TODO after o_proj / down_proj
 * (src/layers/linear.rs:236).  One communicator per process (one process per GPU).
 * nvllm_comm_unique_id writes NVLLM_UNIQUE_ID_BYTES bytes on rank 0; the caller broadcasts them
 * (torch.distributed / any transport) and every rank calls nvllm_comm_init. */
#define NVLLM_UNIQUE_ID_BYTES 128
typedef struct nvllm_comm nvllm_comm;
int nvllm_comm_unique_id(void* h_id_out);
int nvllm_comm_init(nvllm_comm** comm, const void* h_id, int32_t rank, int32_t world);
/* Collective tear-down: closes the peer mappings, meets the other ranks once more (an all-reduce of a scratch word, with a
 * host-side deadline of 6 x NVLLM_COMM_TIMEOUT_MS) so nobody frees a region a peer still has mapped, then frees.  When the
 * communicator has already reported NVLLM_ERR_COMM, or the meeting times out, it does NOT wait: the region is leaked, the
 * NCCL communicator aborted, and NVLLM_ERR_COMM returned — a dead peer can never keep this call from returning. */
int nvllm_comm_destroy(nvllm_comm* comm);
/* In-place sum over ranks of buf[count] (bf16 or f32), enqueued on `stream` (graph-capturable). */
int nvllm_allreduce(nvllm_comm* comm, void* buf, size_t count, int32_t dtype, void* stream);
int nvllm_allgather(nvllm_comm* comm, const void* send, void* recv, size_t bytes_per_rank,
                    void* stream);
/* Symmetric (peer-mapped) memory: a collective call — every rank allocates `bytes`, the CUDA IPC handles are exchanged
 * through the communicator and each peer's region is mapped over NVLink.  *local_base = this rank's region. */
int nvllm_comm_symm_alloc(nvllm_comm* comm, size_t bytes, void** local_base);
/* C1 fused with what always follows it (RowParallelLinear all-reduce TODO linear.rs:236 + the residual add and RMSNorm
 * of Qwen3Layer::forward, qwen3.rs:382-385,389): one two-shot kernel over NVLink peer memory —
 *   residual <- bf16(residual + bf16(sum over ranks of x));  out <- rmsnorm(residual) * weight.
 * `out` is complete on EVERY rank afterwards; `residual` is updated only for the rows this rank owns
 * (rows [rank*R, (rank+1)*R), R = ceil(num_tokens / world)) — it is a row-sharded stream whose only readers are
 * subsequent calls of this function with the same num_tokens.
 * out, x, residual: [num_tokens, hidden] bf16 buffers at identical offsets inside every rank's symmetric region
 * (required by the flag protocol; the push protocol only needs 16-byte alignment).
 * Bit-identical results on all ranks (each row is reduced once, by its owner, in fixed rank order). */
int nvllm_allreduce_add_rmsnorm(nvllm_comm* comm, void* out, void* x, void* residual, const void* weight,
                                int32_t num_tokens, int32_t hidden, float eps, int32_t dtype, void* stream);
/* Two protocols sit behind the call above.  Messages up to NVLLM_AR_LL_MAX_BYTES (8 MiB, decode batches) take the
 * low-latency PUSH protocol: no flags, no fences — every 32-bit word of a not-yet-written buffer holds 0x80008000 (two bf16
 * -0.0; senders map that one pattern to +0.0), partial rows are stored straight into the owner's stage buffer, the owner
 * polls the data itself, reduces, and stores the normed rows into every peer's gather buffer, which the peer polls and
 * copies to `out`; three buffer pairs rotate per call (NVLLM_AR_LL=0 disables it).  Larger messages (prefill) take the
 * flag protocol with peer loads.  nvllm_comm_ll_applies: 1 when a [num_tokens, hidden] call takes the push protocol. */
int nvllm_comm_ll_applies(const nvllm_comm* comm, int32_t num_tokens, int32_t hidden);
/* RowParallelLinear::forward (linear.rs:228-239) whose all-reduce is the call below: y = x . w^T (bf16, m <= 512,
 * n == ldy == hidden, nvllm_comm_ll_applies(comm, m, n)); the GEMM's epilogue stores the rows another rank reduces straight
 * into that rank's stage buffer (they never touch y), so the transfer runs tile by tile under the GEMM's tail. */
int nvllm_gemm_bf16_push(nvllm_comm* comm, void* y, const void* x, const void* w, int32_t m, int32_t n, int32_t k,
                         int64_t ldx, int64_t ldw, int64_t ldy, void* stream);
/* nvllm_allreduce_add_rmsnorm for an x produced by nvllm_gemm_bf16_push (same num_tokens / hidden): skips the push. */
int nvllm_allreduce_add_rmsnorm_pushed(nvllm_comm* comm, void* out, void* x, void* residual, const void* weight,
                                       int32_t num_tokens, int32_t hidden, float eps, int32_t dtype, void* stream);

/* 0, or NVLLM_ERR_COMM once a fused kernel of this communicator gave up waiting for a peer (a rank died, or stalled for
 * longer than NVLLM_COMM_TIMEOUT_MS, default 10 min).  The kernel neither hangs nor traps: it raises this host-visible
 * flag, stops waiting in later calls and runs to completion; results from then on are undefined.  Sticky. */
int nvllm_comm_error(const nvllm_comm* comm);

/* Deterministic seeded weight init shared bit-for-bit with the CPU oracle (oracle/weights.py):
 * element i of tensor `tensor_id` = bf16( (sum of the four 16-bit fields of
 * splitmix64(seed ^ tensor_id<<40, i)  - 131070) * std_scale ).  Integer arithmetic + one exact
 * int->f32 multiply, so host and device agree bit-exactly. */
int nvllm_init_weight(void* w, int64_t count, uint64_t seed, uint64_t tensor_id, float std,
                      int32_t dtype, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Mechanisms of architectures beyond the reference's Qwen3 (no counterpart in the reference).  Operands are bf16 or
 * f32 (`dtype`); norm parameters, router tables and the residual stream are f32.  All are legal inside graph capture.
 * ---------------------------------------------------------------------------------------------- */

/* y[b][m, n] = sum_k x[b][m, k] * w[b][n, k] for b < batch, with element strides bsx / bsw / bsy between batch items
 * (per-head projections).  Any sizes and strides; f32 accumulation in ascending k.  Dense bf16 problems that meet the rules
 * of nvllm_gemm_bf16 are forwarded to it (tensor cores); the rest runs on a CUDA-core tile kernel.  f32 operands need an
 * f32 output. */
int nvllm_linear(void* y, const void* x, const void* w, int32_t m, int32_t n, int32_t k, int64_t ldx, int64_t ldw,
                 int64_t ldy, int32_t batch, int64_t bsx, int64_t bsw, int64_t bsy, int32_t dtype, int32_t out_dtype,
                 void* stream);
/* Grouped variant for expert layers.  Rows are cut into 32-row tiles; tile i uses the weights of group tile_group[i]
 * (w + group * group_stride_w; < 0: tile unused).  row_src (nullable): row r reads x[row_src[r]] (< 0: padding row, not
 * written).  glu == 1: every group's weights are [gate rows (n) | up rows (n)] x k and the output is
 * min(g, limit) * sigmoid(1.702 * min(g, limit)) * (clamp(u, -limit, limit) + 1), g and u rounded to the operand type first;
 * glu == 2: the output is relu(v)^2 of the plain product v (rounded to the operand type first);
 * glu == 3: as glu == 1 with the plain gate, silu(g) * u. */
int nvllm_linear_grouped(void* y, const void* x, const void* w, int32_t max_rows, int32_t n, int32_t k, int64_t ldx,
                         int64_t ldw, int64_t ldy, int64_t group_stride_w, const int32_t* row_src,
                         const int32_t* tile_group, int32_t glu, float limit, int32_t dtype, int32_t out_dtype,
                         void* stream);
/* out[i, c] = the same clamped gated activation of gate_up[i, c] and gate_up[i, ff + c]; gate_up is [n, 2 ff]. */
int nvllm_glu_clamped(void* out, const void* gate_up, int32_t n, int32_t ff, float limit, int32_t dtype, void* stream);

/* Dynamic Tanh normalisation, dyt(x) = tanh(alpha x) w + b (no mean, no variance), fused around an f32 residual stream:
 *   y != NULL:   h += dyt_post(y)        out != NULL:   out = dyt_pre(h)      (h: f32 [n, hidden], updated in place) */
int nvllm_dyt_residual_norm(void* out, float* h, const void* y, const float* post_alpha, const float* post_w,
                            const float* post_b, const float* pre_alpha, const float* pre_w, const float* pre_b, int32_t n,
                            int32_t hidden, int32_t dtype, void* stream);
/* h[i, :] = table[ids[i], :] as f32 (ids clamped to the table). */
int nvllm_embedding_gather_f32(float* h, const void* table, const int64_t* ids, int32_t n, int32_t hidden, int32_t vocab,
                               int32_t table_dtype, void* stream);
/* out[i, :] = x[rows[i], :]  (rows clamped to [0, n_src)). */
int nvllm_gather_rows(void* out, const void* x, const int32_t* rows, int32_t n, int32_t hidden, int32_t n_src, int32_t dtype,
                      void* stream);

/* Rotary table for the interleaved pairing (dimension 2i with 2i+1): cos_sin[p][i] = (cos, sin)(p * base^(-2i/dims)),
 * i < dims/2, p < max_pos, angles computed in f64.  f32 [max_pos, dims/2, 2]. */
int nvllm_rope_table_interleaved(float* cos_sin, int32_t max_pos, int32_t dims, double base, void* stream);
/* Latent attention, per-token preparation.  dkv row = [kv_rank latent | rot_dim shared key part]; q row = heads x
 * [dim | rot_dim].  The latent is RMS-normed (x / sqrt(mean(x^2) + eps) * c_norm_w) and the key part rotated (first rot_dims
 * values, interleaved pairs) into cache row slots[i] ([kv_rank | rot_dim], cache_row elements apart; slot < 0: nothing
 * stored); the rotated part of every query head is rotated in place. */
int nvllm_latent_prepare(void* q, int64_t ldq, const void* dkv, int64_t lddkv, const float* c_norm_w, float eps,
                         const int64_t* positions, const float* rope_table, int32_t rot_dims, int32_t max_pos, int32_t n,
                         int32_t heads, int32_t dim, int32_t rot_dim, int32_t kv_rank, void* cache, int64_t cache_row,
                         const int32_t* slots, int32_t dtype, void* stream);
/* Latent attention over the paged cache with the key up-projection folded into the queries:
 *   s[t, h, j] = scale * (q_abs[t, h, :] . c_j + q[t, h, dim:] . k_rot_j),  j <= positions[t] in sequence tok_seq[t]
 *   out[t, h, :] = sum_j softmax_j(s) c_j                                   (kv_rank values per head)
 * q_abs: f32 [n, heads, kv_rank]; block_tables: [sequences, table_cap] (entries < 0 end a sequence's keys). */
int nvllm_latent_attention(void* out, int64_t ldo, const float* q_abs, int64_t ldqa, const void* q, int64_t ldq,
                           const int32_t* tok_seq, const int64_t* positions, const int32_t* block_tables,
                           int32_t table_cap, int32_t block_size, const void* cache, int64_t cache_row, int32_t n,
                           int32_t heads, int32_t dim, int32_t rot_dim, int32_t kv_rank, float scale, int32_t dtype,
                           void* stream);

/* Mixture-of-experts routing.  logits: f32 [n, outputs] (real experts first, identity experts last).
 *   s = softmax(logits); chosen = the `top` largest of s + bias (bias nullable; ties: lowest index);
 *   topk_w[k] = s[chosen_k] / (sum_k s[chosen_k] + 1e-20) * scale.   outputs <= 1536. */
int nvllm_moe_route(int32_t* topk_idx, float* topk_w, const float* logits, const float* bias, int32_t n, int32_t outputs,
                    int32_t top, float scale, void* stream);
/* Rows the grouped buffers need for n tokens when every expert's segment starts on a tile of tile_rows rows. */
int32_t nvllm_moe_max_rows(int32_t n_tokens, int32_t top, int32_t experts, int32_t tile_rows);
/* Counting sort of the (token, slot) assignments by expert for the grouped products (tile_rows 32: nvllm_linear_grouped,
 * 128: nvllm_gemm_bf16_grouped): row_token[max_rows] (token of each row, -1 padding), tile_expert[max_rows / tile_rows]
 * (-1 unused), slot_row[n * top] (row of each assignment; -1 when it chose an identity expert, i.e. an index >= experts). */
int nvllm_moe_sort(int32_t* row_token, int32_t* tile_expert, int32_t* slot_row, const int32_t* topk_idx, int32_t n,
                   int32_t top, int32_t experts, int32_t max_rows, int32_t tile_rows, void* stream);
/* Tensor-core grouped product (bf16): rows in 128-row tiles, tile i times the weight block of group tile_group[i], i.e.
 * rows [group * n, (group + 1) * n) of w ([groups * n, k]); an unused tile (group < 0) is computed against group 0 and its
 * rows mean nothing.  k % 64 == 0, n % 8 == 0, 16-byte aligned rows. */
int nvllm_gemm_bf16_grouped(void* y, const void* x, const void* w, int32_t max_rows, int32_t n, int32_t k, int32_t groups,
                            int64_t ldx, int64_t ldw, int64_t ldy, const int32_t* tile_group, void* stream);
/* out[t] = sum_k topk_w[t, k] * (slot_row[t, k] >= 0 ? expert_out[slot_row[t, k]] : x[t]) + shared_out[t] (nullable). */
int nvllm_moe_combine(void* out, const void* expert_out, const void* x, const void* shared_out, const int32_t* topk_idx,
                      const float* topk_w, const int32_t* slot_row, int32_t n, int32_t hidden, int32_t top, int32_t experts,
                      int32_t dtype, void* stream);

/* ---- Parallel blocks on an f32 residual stream; attention with a score cap; mixers with a recurrent state ---------- */

/* h += s0 a0 + s1 a1 + s2 a2 + bias_scale * bias (each addend [n, hidden], f32 or bf16 per its dt, nullable; bias f32
 * [hidden], nullable), then out = (h - mean) / sqrt(var + eps) * w in out_dtype (out nullable: only the sum).  var is the
 * mean of the squared deviations; all statistics f32. */
int nvllm_residual_layernorm(void* out, float* h, const void* a0, float s0, int32_t dt0, const void* a1, float s1,
                             int32_t dt1, const void* a2, float s2, int32_t dt2, const float* bias, float bias_scale,
                             const float* w, int32_t n, int32_t hidden, float eps, int32_t out_dtype, void* stream);
/* out[i, :] = [a[i, :] | b[i, :]] (f32 inputs) in out_dtype. */
int nvllm_concat_cast(void* out, const float* a, const float* b, int32_t n, int32_t width_a, int32_t width_b,
                      int32_t out_dtype, void* stream);
/* h[i, :] = h_copy[i, :] (nullable) = table[ids[i], :] * scale as f32 (ids clamped to the table). */
int nvllm_embedding_gather_scaled(float* h, float* h_copy, const void* table, const int64_t* ids, int32_t n,
                                  int32_t hidden, int32_t vocab, float scale, int32_t table_dtype, void* stream);
/* out[i, c] = silu(in[i, c]) * in[i, ff + c] (kind 0, in: [n, 2 ff]) or relu(in[i, c])^2 (kind 1, in: [n, ff]). */
int nvllm_ff_activation(void* out, const void* in, int32_t n, int32_t ff, int32_t kind, int32_t dtype, void* stream);
/* Expert choice by table: topk_idx[t, :] = table[ids[t], :] ([table_rows, top] int32), topk_w = 1 / top. */
int nvllm_moe_table_route(int32_t* topk_idx, float* topk_w, const int32_t* table, const int64_t* ids, int32_t n,
                          int32_t top, int32_t table_rows, void* stream);

/* Attention preparation.  proj: f32 [n, >= q_cols + k_cols + v_cols] rows [q | k | v | ...]; adds the biases (nullable),
 * writes q in `dtype` and k / v into cache rows slots[i] (k_row / v_row elements apart; slot < 0: nothing stored). */
int nvllm_attn_bias_store(void* q, int64_t ldq, void* k_cache, void* v_cache, int64_t k_row, int64_t v_row,
                          const float* proj, int64_t ldp, const float* q_bias, const float* k_bias, const float* v_bias,
                          const int32_t* slots, int32_t n, int32_t q_cols, int32_t k_cols, int32_t v_cols, int32_t dtype,
                          void* stream);
/* Grouped-query softmax attention over the paged cache, without rotary:
 *   s[t, h, j] = cap(scale * temp(p_t) * q[t, h] . k[j, h / (heads / kv_heads)]),  j <= p_t = positions[t] in sequence tok_seq[t]
 *   temp(p) = 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1),  cap(s) = softcap * tanh(s / softcap) (softcap <= 0: s)
 *   out[t, h, :] = sum_j softmax_j(s) v[j, ...] * sigmoid(gate[t, h, :])   (gate: f32, nullable)
 * Key size dim, value size vdim (<= 512).  block_tables: [sequences, table_cap].  cu_tokens (nullable): [n_seqs + 1] token
 * range of every sequence in the batch, tokens in order of position; with it, bf16 problems whose rows are 16-byte multiples
 * (dim, vdim <= 128) run on tensor cores, 64 (token, head) rows of one sequence and key / value head per CTA. */
int nvllm_capped_attention(void* out, int64_t ldo, const void* q, int64_t ldq, const float* gate, int64_t ldg,
                           const void* k_cache, const void* v_cache, int64_t k_row, int64_t v_row,
                           const int32_t* tok_seq, const int64_t* positions, const int32_t* block_tables,
                           int32_t table_cap, int32_t block_size, int32_t n, int32_t heads, int32_t kv_heads, int32_t dim,
                           int32_t vdim, float scale, float softcap, float temp_coef, int32_t temp_every,
                           const int32_t* cu_tokens, int32_t n_seqs, int32_t dtype, void* stream);

/* Recurrent mixers.  A step lists its sequences: seq_slot[s] = the state slot of sequence s (< 0: padding, output zero),
 * cu_tokens[s] .. cu_tokens[s + 1] = its tokens in the batch (in order of position), positions[] per token.  A portion
 * whose first position is 0 starts from a zero state, any other from the slot's content; the slot is updated.  All f32.
 *
 * S_t = a_t S_(t-1) + b_t k_t v_t^T,  y_t = S_t^T q_t + skip_h v_t;  S: [dk, dv] per head; state: [slots, heads, dk, dv].
 * q, k: [n, groups * dk] (head h reads group h / (heads / groups)); v, y: [n, heads * dv]; decay / step: [n, heads] when
 * *_per_token, else [heads]; step nullable (1), skip nullable (0).  dk <= 512. */
int nvllm_linear_recurrence(float* y, int64_t ldy, const float* q, int64_t ldq, const float* k, int64_t ldk, const float* v,
                            int64_t ldv, const float* decay, int32_t decay_per_token, const float* step,
                            int32_t step_per_token, const float* skip, float* state, const int32_t* seq_slot,
                            const int32_t* cu_tokens, const int64_t* positions, int32_t n_seqs, int32_t heads,
                            int32_t groups, int32_t dk, int32_t dv, void* stream);
/* out[t, c] = act(bias[c] + sum_j w[c, j] * in[token at position(t) - (taps - 1 - j), c]) (zero before the sequence; act =
 * SiLU when silu != 0); state: [slots, taps - 1, channels] = the raw inputs of the last taps - 1 tokens, read for inputs
 * before the portion and rewritten afterwards.  taps <= 16; out != in. */
int nvllm_causal_conv(float* out, int64_t ldo, const float* in, int64_t ldi, const float* w, const float* bias, float* state,
                      const int32_t* tok_seq, const int32_t* seq_slot, const int32_t* cu_tokens, const int64_t* positions,
                      int32_t n, int32_t n_seqs, int32_t channels, int32_t taps, int32_t silu, void* stream);
/* step[t, h] = softplus(dt_raw[t, h] + dt_bias[h]);  decay[t, h] = exp(-exp(a_log[h]) * step[t, h]). */
int nvllm_ssd_prepare(float* step, float* decay, const float* dt_raw, int64_t ld_raw, const float* dt_bias, const float* a_log,
                      int32_t n, int32_t heads, void* stream);
/* Rotary positions with the half-split pairing, in place on f32 rows [n, heads * dim]: within a head, value i < dims / 2 is
 * paired with i + dims / 2, (u, v) -> (u cos - v sin, v cos + u sin), angle = position * base^(-2i/dims) from `table`
 * ([max_pos, dims/2, 2], as nvllm_rope_table_interleaved builds); values beyond dims pass; the whole head is multiplied by scale. */
int nvllm_rotate_half(float* x, int64_t ldx, const int64_t* positions, const float* table, int32_t max_pos, int32_t n,
                      int32_t heads, int32_t dim, int32_t dims, float scale, void* stream);
/* RMS norm over `parts` equal parts of every row (each by its own root mean square, eps inside the root) with a SiLU gate:
 * gate_first != 0: t = y * silu(gate), out = t / rms(t) * w;   else: out = y / rms(y) * silu(gate) * w.   w nullable (1). */
int nvllm_gated_group_norm(void* out, int64_t ldo, const float* y, int64_t ldy, const float* gate, int64_t ldg, const float* w,
                           int32_t n, int32_t cols, int32_t parts, float eps, int32_t gate_first, int32_t out_dtype,
                           void* stream);

/* ---- Sandwich RMS norms, windowed attention with sinks, latent attention in a window, the gated delta rule --------- */

/* rms(v) = v / sqrt(mean(v^2) + eps).   y != NULL: h += rms(y) * post_w;   out != NULL: out = rms(h) * pre_w.
 * h: f32 [n, hidden], updated in place; y in y_dtype, out in out_dtype; weights f32.  hidden <= 49152. */
int nvllm_rms_residual_norm(void* out, float* h, const void* y, int32_t y_dtype, const float* post_w, const float* pre_w,
                            int32_t n, int32_t hidden, float eps, int32_t out_dtype, void* stream);
/* out[row_map ? row_map[i] : i, :cols] = rms(x[i, :cols]) * w (w nullable: 1); rows whose map entry is < 0 are skipped
 * (the map is a paged cache's slot list, or NULL for row i -> row i).  x f32, out in out_dtype. */
int nvllm_rms_norm_rows(void* out, int64_t ldo, const float* x, int64_t ldx, const float* w, const int32_t* row_map, int32_t n,
                        int32_t cols, float eps, int32_t out_dtype, void* stream);
/* h[t, :] = table[ids[t], :] * scale + bigram[r, :] as f32, r = (ids[t-1] * mul_prev + ids[t] * mul_cur) mod buckets, or
 * r = buckets (the table's last row) where positions[t] == 0.  For the first token of a portion (cu_tokens) ids[t-1] is
 * last_token[seq_slot[sequence]], which is then set to the portion's last token.  Padding sequences (slot < 0): zeros. */
int nvllm_embedding_bigram(float* h, const void* table, const void* bigram, const int64_t* ids, const int64_t* positions,
                           const int32_t* tok_seq, const int32_t* cu_tokens, const int32_t* seq_slot, int32_t* last_token,
                           int32_t n, int32_t hidden, int32_t vocab, int32_t buckets, int32_t mul_prev, int32_t mul_cur, float scale,
                           int32_t table_dtype, void* stream);
/* Attention preparation with rotary positions.  proj: f32 [n, ...] rows [q (heads x dim) | k (kv_heads x dim) | v (kv_heads x
 * vdim, absent with v_from_k) | ...].  Adds the biases (nullable); rotates the pairs (2i, 2i+1) of the first rot_dims values
 * of every query and key head (table as nvllm_rope_table_interleaved builds); norm_eps > 0: divides each rotated head by
 * its root mean square (eps inside the root, no weight); writes q in `dtype` and k / v into cache rows slots[i] (slot < 0:
 * nothing stored).  v_from_k != 0: the values are the keys as projected (bias added, not rotated, not normed); vdim == dim. */
int nvllm_attn_rope_norm_store(void* q, int64_t ldq, void* k_cache, void* v_cache, int64_t k_row, int64_t v_row,
                               const float* proj, int64_t ldp, const float* q_bias, const float* k_bias, const float* v_bias,
                               const int64_t* positions, const float* rope_table, int32_t rot_dims, int32_t max_pos,
                               float norm_eps, const int32_t* slots, int32_t n, int32_t heads, int32_t kv_heads, int32_t dim,
                               int32_t vdim, int32_t v_from_k, int32_t dtype, void* stream);
/* nvllm_capped_attention with three more options: window > 0: position p sees only the keys p - window + 1 .. p;
 * sinks (f32 [heads], nullable): exp(sinks[h]) joins the softmax denominator (unscaled, no value);
 * gate_per_head != 0: gate is [n, heads] (ldg apart) and head h's output is multiplied by sigmoid(gate[t, h]).
 * block_tables == NULL (cu_tokens given): the keys are not paged — every sequence of the step starts at position 0 and key
 * j of sequence s is row cu_tokens[s] + j of k_cache / v_cache (whole prompts whose keys were just computed). */
int nvllm_window_attention(void* out, int64_t ldo, const void* q, int64_t ldq, const float* gate, int64_t ldg,
                           int32_t gate_per_head, const void* k_cache, const void* v_cache, int64_t k_row, int64_t v_row,
                           const int32_t* tok_seq, const int64_t* positions, const int32_t* block_tables, int32_t table_cap,
                           int32_t block_size, int32_t n, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, float scale,
                           float softcap, float temp_coef, int32_t temp_every, int32_t window, const float* sinks,
                           const int32_t* cu_tokens, int32_t n_seqs, int32_t dtype, void* stream);
/* nvllm_latent_attention with a sliding window (window > 0: keys p - window + 1 .. p), sinks (f32 [heads], nullable, as
 * above) and a gate per head (f32 [n, heads], ldg apart, nullable: out[t, h, :] *= sigmoid(gate[t, h])).
 * workspace (nullable, f32): with it, single tokens in a long window (1000 keys and more) whose CTAs would not fill the SMs
 * split their key tiles over up to 4 CTAs; needs n * heads * 4 * (kv_rank + 2) * 4 bytes for n <= 256 (larger batches never split). */
int nvllm_latent_window_attention(void* out, int64_t ldo, const float* q_abs, int64_t ldqa, const void* q, int64_t ldq,
                                  const int32_t* tok_seq, const int64_t* positions, const int32_t* block_tables,
                                  int32_t table_cap, int32_t block_size, const void* cache, int64_t cache_row, int32_t n,
                                  int32_t heads, int32_t dim, int32_t rot_dim, int32_t kv_rank, float scale, int32_t window,
                                  const float* sinks, const float* gate, int64_t ldg, void* workspace, size_t workspace_bytes,
                                  int32_t dtype, void* stream);
/* Per-token preparation of the gated delta rule, in place, all f32:
 *   q, k: [n, groups * dk] -> every head divided by sqrt(sum of squares + unit_eps), q also times q_scale;
 *   beta: [n, heads] -> sigmoid;   decay: [n, heads * dk] -> exp(-exp(a_log[h]) * softplus(decay + dt_bias[h, c])). */
int nvllm_delta_prepare(float* q, int64_t ldq, float* k, int64_t ldk, float* beta, int64_t ldb, float* decay, int64_t ldd,
                        const float* a_log, const float* dt_bias, int32_t n, int32_t heads, int32_t groups, int32_t dk,
                        float q_scale, float unit_eps, void* stream);
/* Gated delta rule with a decay per key channel (sequence / slot conventions of nvllm_linear_recurrence), per head:
 *   S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   y_t = S^T q_t        S: [dk, dv], state [slots, heads, dk, dv]
 * q, k: [n, groups * dk]; v, y: [n, heads * dv]; decay g: [n, heads * dk]; beta: [n, heads].  dk <= 512.  All f32. */
int nvllm_gated_delta_recurrence(float* y, int64_t ldy, const float* q, int64_t ldq, const float* k, int64_t ldk, const float* v,
                                 int64_t ldv, const float* decay, int64_t ldd, const float* beta, int64_t ldb, float* state,
                                 const int32_t* seq_slot, const int32_t* cu_tokens, const int64_t* positions, int32_t n_seqs,
                                 int32_t heads, int32_t groups, int32_t dk, int32_t dv, void* stream);
/* nvllm_gated_group_norm with the gate's activation as a parameter (gate_act 0: SiLU, 1: sigmoid) and, with w_shared != 0, one
 * weight vector of cols / parts values used by every part. */
int nvllm_gated_group_norm_act(void* out, int64_t ldo, const float* y, int64_t ldy, const float* gate, int64_t ldg, const float* w,
                               int32_t w_shared, int32_t n, int32_t cols, int32_t parts, float eps, int32_t gate_first,
                               int32_t gate_act, int32_t out_dtype, void* stream);

/* ---- Post-norm blocks, chunked attention with a distance bias, rotated values, xIELU, routing on logits -------------- */

/* Attention preparation for layers whose queries and keys are RMS-normed over the whole projection (all heads at once).
 * proj: f32 [n, >= q_cols + k_cols + v_cols] rows [q | k | v | ...]; q = rms(q) * q_norm_w in `dtype`; k = rms(k) * k_norm_w and
 * v into cache rows slots[i] (slot < 0: nothing stored).  Weights f32, nullable (1).  k_cols == 0 (then v_cols == 0): the
 * layer reads another layer's keys and values and only its queries are prepared. */
int nvllm_attn_wide_norm_store(void* q, int64_t ldq, void* k_cache, void* v_cache, int64_t k_row, int64_t v_row, const float* proj,
                               int64_t ldp, const float* q_norm_w, const float* k_norm_w, float eps, const int32_t* slots,
                               int32_t n, int32_t q_cols, int32_t k_cols, int32_t v_cols, int32_t dtype, void* stream);
/* nvllm_attn_rope_norm_store with the pairing of the rotation as a parameter (halves == 0: neighbours (2i, 2i+1); != 0: value
 * i with i + rot_dims / 2) and, with v_rope_table (as nvllm_rope_table_interleaved builds for dims = vdim; nullable), the value
 * heads rotated by their position over all of vdim in the same pairing before they are stored. */
int nvllm_attn_rotary_store(void* q, int64_t ldq, void* k_cache, void* v_cache, int64_t k_row, int64_t v_row, const float* proj,
                            int64_t ldp, const float* q_bias, const float* k_bias, const float* v_bias, const int64_t* positions,
                            const float* rope_table, int32_t rot_dims, int32_t halves, const float* v_rope_table, int32_t max_pos,
                            float norm_eps, const int32_t* slots, int32_t n, int32_t heads, int32_t kv_heads, int32_t dim,
                            int32_t vdim, int32_t v_from_k, int32_t dtype, void* stream);
/* nvllm_window_attention with four more options, each off when zero / NULL:
 *   chunk > 0: position p sees only the keys of its own chunk, floor(p / chunk) * chunk .. p (chunks count from position 0);
 *   head_scale (f32 [heads]): the scaled score of head h is multiplied by head_scale[h];
 *   dist_bias (f32 [heads, dist_rows]): dist_bias[h, min(p - j, dist_rows - 1)] is added to the score of key j (after scale,
 *     temperature and cap; the sink gets none);
 *   out_rot_table (f32 [max_pos, vdim / 2, 2] of (cos, sin), as nvllm_rope_table_interleaved builds for dims = vdim): every
 *     head's output is turned by -p, value m paired with m + vdim / 2, before the gate (values that were stored rotated by
 *     their own position thus enter the sum by their distance). */
int nvllm_biased_attention(void* out, int64_t ldo, const void* q, int64_t ldq, const float* gate, int64_t ldg,
                           int32_t gate_per_head, const void* k_cache, const void* v_cache, int64_t k_row, int64_t v_row,
                           const int32_t* tok_seq, const int64_t* positions, const int32_t* block_tables, int32_t table_cap,
                           int32_t block_size, int32_t n, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, float scale,
                           float softcap, float temp_coef, int32_t temp_every, int32_t window, const float* sinks, int32_t chunk,
                           const float* head_scale, const float* dist_bias, int32_t dist_rows, const float* out_rot_table,
                           int32_t max_pos, const int32_t* cu_tokens, int32_t n_seqs, int32_t dtype, void* stream);
/* nvllm_ff_activation with parameters.  kind 2 (in: [n, ff]): xIELU with the two learned numbers params[0..1] (device, f32):
 *   z > 0: softplus(p0) z^2 + z / 2;   z <= 0: (1/2 + softplus(p1)) (exp(z) - 1 - z) + z / 2.   kinds 0 / 1 ignore params. */
int nvllm_ff_activation_params(void* out, const void* in, int32_t n, int32_t ff, int32_t kind, const float* params, int32_t dtype,
                               void* stream);
/* h[i, :] = table[ids[i], :] * scale as f32 and x[i, :] = the same row in x_dtype (ids clamped to the table): the stream and
 * what the first sublayer of a block without an input norm reads, in one pass. */
int nvllm_embedding_stream(float* h, void* x, int32_t x_dtype, const void* table, const int64_t* ids, int32_t n, int32_t hidden,
                           int32_t vocab, float scale, int32_t table_dtype, void* stream);
/* Routing on the logits: z = logits + bias (bias nullable); chosen = the `top` largest z (ties: lowest index);
 * topk_w = softmax over the chosen z alone.  logits: f32 [n, experts] with rows ld apart, experts <= 3072.
 * (nvllm_linear_grouped with glu == 3 is the expert product with the plain gate silu(g) * u.) */
int nvllm_moe_route_logits(int32_t* topk_idx, float* topk_w, const float* logits, int64_t ld, const float* bias, int32_t n,
                           int32_t experts, int32_t top, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Engine-level C ABI: the C++ host runtime that mirrors the reference's Rust types one-to-one
 * (Config, SamplingParams, Sequence, BlockManager, Scheduler, ModelRunner, Qwen3Model, LLMEngine).
 * Declared in nvllm_engine.h; kept separate so a Rust caller that only wants the kernels binds
 * this header alone.
 * ---------------------------------------------------------------------------------------------- */

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* NVLLM_H_ */
