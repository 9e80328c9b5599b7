"""One Python function per kernel entry point of include/nvllm.h.

Arguments are torch CUDA tensors (PyTorch is only the device-memory / stream plumbing); every call is
enqueued on torch's current stream and goes through the C ABI — there is no eager / CPU fallback.
Names mirror the reference layer methods they replace (file:line in include/nvllm.h)."""
import math

import torch

from . import _ffi
from ._ffi import KvLayout, check

BF16, F32 = 0, 1


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


def _need(t, dtype, name):
    if not t.is_cuda:
        raise ValueError(f"{name}: expected a CUDA tensor (no CPU path exists)")
    if t.dtype != dtype:
        raise ValueError(f"{name}: expected {dtype}, got {t.dtype}")


def store_kvcache(k, v, k_cache, v_cache, slot_mapping, layout: KvLayout):
    """Attention::store_kv_cache (attention.rs:150-174). k, v: [N, Hkv, D] (last two dims contiguous)."""
    _need(k, torch.bfloat16, "k"); _need(v, torch.bfloat16, "v"); _need(slot_mapping, torch.int32, "slot_mapping")
    assert k.stride(-1) == 1 and k.stride(1) == k.shape[2] and k.stride() == v.stride()
    check(_ffi.lib().nvllm_store_kvcache(_p(k), _p(v), _p(k_cache), _p(v_cache), _p(slot_mapping), k.shape[0],
                                         k.stride(0), layout, BF16, _stream()))


def paged_decode_workspace_bytes(batch, num_heads, head_dim, num_splits=0):
    return _ffi.lib().nvllm_paged_decode_workspace_bytes(batch, num_heads, head_dim, num_splits)


def paged_decode_attention(q, k_cache, v_cache, block_tables, context_lens, layout: KvLayout, scale=None,
                           num_splits=0, out=None, workspace=None):
    """Attention::flash_attention_decode (attention.rs:225-318). q: [B, H, D] -> out [B, H, D]."""
    _need(q, torch.bfloat16, "q"); _need(block_tables, torch.int32, "block_tables")
    _need(context_lens, torch.int32, "context_lens")
    B, H, D = q.shape
    assert q.stride(2) == 1 and q.stride(1) == D and block_tables.is_contiguous()
    if out is None:
        out = torch.empty((B, H, D), dtype=torch.bfloat16, device=q.device)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if num_splits == 0:
        num_splits = _ffi.lib().nvllm_paged_decode_choose_splits(B, H, layout.num_kv_heads,
                                                                 block_tables.shape[1] * layout.block_size)
    need = paged_decode_workspace_bytes(B, H, D, num_splits)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    check(_ffi.lib().nvllm_paged_decode_attention(
        _p(out), _p(q), _p(k_cache), _p(v_cache), _p(block_tables), _p(context_lens), B, H, block_tables.shape[1],
        q.stride(0), out.stride(0), layout, scale, _p(workspace),
        0 if workspace is None else workspace.numel() * workspace.element_size(), num_splits, BF16, _stream()))
    return out


def paged_decode_attention_fused(qkv, positions, cos_sin, q_norm_w, k_norm_w, eps, k_cache, v_cache, slot_mapping, block_tables,
                                 context_lens, num_heads, layout: KvLayout, scale=None, num_splits=0, out=None, workspace=None):
    """q/k-norm + RoPE + store_kv_cache + flash_attention_decode in one launch (qwen3.rs:219-233).  qkv: [B, (H+2Hkv)*D]
    packed rows of this step (read only); context_lens counts this step's token.  -> out [B, H, D]."""
    _need(qkv, torch.bfloat16, "qkv"); _need(positions, torch.int64, "positions"); _need(cos_sin, torch.float32, "cos_sin")
    _need(block_tables, torch.int32, "block_tables"); _need(context_lens, torch.int32, "context_lens")
    _need(slot_mapping, torch.int32, "slot_mapping")
    B, H, D = qkv.shape[0], num_heads, layout.head_dim
    assert qkv.is_contiguous() and qkv.shape[1] == (H + 2 * layout.num_kv_heads) * D and block_tables.is_contiguous()
    if out is None:
        out = torch.empty((B, H, D), dtype=torch.bfloat16, device=qkv.device)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if num_splits == 0:
        num_splits = _ffi.lib().nvllm_paged_decode_choose_splits(B, H, layout.num_kv_heads,
                                                                 block_tables.shape[1] * layout.block_size)
    need = paged_decode_workspace_bytes(B, H, D, num_splits)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=qkv.device)
    check(_ffi.lib().nvllm_paged_decode_attention_fused(
        _p(out), _p(qkv), _p(positions), _p(cos_sin), _p(q_norm_w), _p(k_norm_w), eps, cos_sin.shape[0], _p(k_cache),
        _p(v_cache), _p(slot_mapping), _p(block_tables), _p(context_lens), B, H, block_tables.shape[1], qkv.stride(0),
        out.stride(0), layout, scale, _p(workspace),
        0 if workspace is None else workspace.numel() * workspace.element_size(), num_splits, BF16, _stream()))
    return out


def varlen_prefill_attention(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, scale=None,
                             k_cache=None, v_cache=None, block_tables=None, layout: KvLayout = None, out=None):
    """Attention::flash_attention_varlen / _with_cache (attention.rs:177-222). q: [N, H, D]; k, v: [Nk, Hkv, D]."""
    _need(q, torch.bfloat16, "q"); _need(cu_seqlens_q, torch.int32, "cu_seqlens_q")
    N, H, D = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty((N, H, D), dtype=torch.bfloat16, device=q.device)
    paged = block_tables is not None
    Hkv = layout.num_kv_heads if paged else k.shape[1]
    check(_ffi.lib().nvllm_varlen_prefill_attention(
        _p(out), _p(q), _p(k), _p(v), _p(cu_seqlens_q), _p(cu_seqlens_k), cu_seqlens_q.numel() - 1,
        N, 0 if k is None else k.shape[0], max_seqlen_q, max_seqlen_k, H, Hkv, D, q.stride(0), 0 if k is None else k.stride(0), out.stride(0),
        _p(k_cache), _p(v_cache), _p(block_tables), block_tables.shape[1] if paged else 0,
        layout if paged else None, scale, BF16, _stream()))
    return out


def gemm_bf16(x, w, out=None, out_dtype=torch.bfloat16, simt=False):
    """LinearBase::forward (linear.rs): y[M,N] = x[M,K] @ w[N,K]^T on tcgen05 (simt=True: test-only CUDA-core path)."""
    _need(x, torch.bfloat16, "x"); _need(w, torch.bfloat16, "w")
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and x.stride(1) == 1 and w.stride(1) == 1
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    od = BF16 if out.dtype == torch.bfloat16 else F32
    L = _ffi.lib()
    if simt:
        check(L.nvllm_gemm_bf16_simt(_p(out), _p(x), _p(w), M, N, K, x.stride(0), w.stride(0), out.stride(0), od, _stream()))
        return out
    need = L.nvllm_gemm_workspace_bytes(M, N, K)
    ws = torch.empty(need, dtype=torch.uint8, device=x.device) if need else None
    check(L.nvllm_gemm_bf16(_p(out), _p(x), _p(w), M, N, K, x.stride(0), w.stride(0), out.stride(0), od, _p(ws), need, _stream()))
    return out


def gemm_silu_mul(x, w_gate_up, out=None):
    """MergedColumnParallelLinear::forward + SiluAndMul::forward fused (linear.rs:437-439, activation.rs:46-63)."""
    _need(x, torch.bfloat16, "x"); _need(w_gate_up, torch.bfloat16, "w_gate_up")
    M, K = x.shape
    inter = w_gate_up.shape[0] // 2
    if out is None:
        out = torch.empty((M, inter), dtype=torch.bfloat16, device=x.device)
    ws = torch.empty((M, 2 * inter), dtype=torch.bfloat16, device=x.device)
    check(_ffi.lib().nvllm_gemm_silu_mul_bf16(_p(out), _p(x), _p(w_gate_up), M, inter, K, x.stride(0), w_gate_up.stride(0),
                                              out.stride(0), _p(ws), ws.numel() * 2, _stream()))
    return out


def gemm_qkv_rope_store(x, w_qkv, positions, cos_sin, q_norm_w, k_norm_w, eps, num_heads, num_kv_heads, head_dim,
                        k_cache=None, v_cache=None, slot_mapping=None, layout: KvLayout = None, out=None):
    """qkv_proj + q/k norm + RoPE + store_kv_cache in one kernel (linear.rs:354-356, qwen3.rs:219-229, attention.rs:150-174)."""
    _need(x, torch.bfloat16, "x"); _need(w_qkv, torch.bfloat16, "w_qkv"); _need(positions, torch.int64, "positions")
    M, K = x.shape
    n = (num_heads + 2 * num_kv_heads) * head_dim
    if out is None:
        out = torch.empty((M, n), dtype=torch.bfloat16, device=x.device)
    check(_ffi.lib().nvllm_gemm_qkv_rope_store(_p(out), _p(x), _p(w_qkv), M, K, x.stride(0), w_qkv.stride(0), _p(positions),
                                               _p(cos_sin), _p(q_norm_w), _p(k_norm_w), eps, num_heads, num_kv_heads, head_dim,
                                               cos_sin.shape[0], _p(k_cache), _p(v_cache), _p(slot_mapping), layout, _stream()))
    return out


def add_rmsnorm(x, weight, eps, residual=None, out=None):
    """RMSNorm::forward (layernorm.rs:50-97). With `residual`, it is updated in place to bf16(residual + x)."""
    _need(x, torch.bfloat16, "x")
    assert x.is_contiguous() and (residual is None or residual.is_contiguous())
    if out is None:
        out = torch.empty_like(x)
    check(_ffi.lib().nvllm_add_rmsnorm(_p(out), _p(x), _p(residual), _p(weight), x.shape[0], x.shape[1], eps, BF16, _stream()))
    return out


def rope_table(max_position, head_dim, theta, device="cuda"):
    t = torch.empty((max_position, head_dim), dtype=torch.float32, device=device)
    check(_ffi.lib().nvllm_rope_table(_p(t), max_position, head_dim, float(theta), _stream()))
    return t


def qknorm_rope_store(qkv, positions, cos_sin, q_norm_w, k_norm_w, eps, num_heads, num_kv_heads, head_dim,
                      k_cache=None, v_cache=None, slot_mapping=None, layout: KvLayout = None):
    """RotaryEmbedding::forward (+ q/k norm, + store_kv_cache), in place on qkv [N, (H+2Hkv)*D]."""
    _need(qkv, torch.bfloat16, "qkv"); _need(positions, torch.int64, "positions"); _need(cos_sin, torch.float32, "cos_sin")
    assert qkv.is_contiguous() and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim
    check(_ffi.lib().nvllm_qknorm_rope_store(_p(qkv), _p(positions), _p(cos_sin), _p(q_norm_w), _p(k_norm_w), eps,
                                             qkv.shape[0], num_heads, num_kv_heads, head_dim, cos_sin.shape[0],
                                             _p(k_cache), _p(v_cache), _p(slot_mapping), layout, BF16, _stream()))
    return qkv


def silu_mul(x, out=None):
    """SiluAndMul::forward (activation.rs:46-63). x: [N, 2I] -> [N, I]."""
    _need(x, torch.bfloat16, "x")
    assert x.is_contiguous()
    inter = x.shape[1] // 2
    if out is None:
        out = torch.empty((x.shape[0], inter), dtype=torch.bfloat16, device=x.device)
    check(_ffi.lib().nvllm_silu_mul(_p(out), _p(x), x.shape[0], inter, BF16, _stream()))
    return out


def embedding_gather(table, ids, out=None):
    """VocabParallelEmbedding::forward (embed_head.rs:77-97)."""
    _need(table, torch.bfloat16, "table"); _need(ids, torch.int64, "ids")
    if out is None:
        out = torch.empty((ids.numel(), table.shape[1]), dtype=torch.bfloat16, device=table.device)
    check(_ffi.lib().nvllm_embedding_gather(_p(out), _p(table), _p(ids), ids.numel(), table.shape[1], table.shape[0], BF16, _stream()))
    return out


def gather_last_tokens(x, cu_seqlens_q, out=None):
    """ParallelLMHead::extract_last_tokens (embed_head.rs:272-289)."""
    _need(x, torch.bfloat16, "x"); _need(cu_seqlens_q, torch.int32, "cu_seqlens_q")
    B = cu_seqlens_q.numel() - 1
    if out is None:
        out = torch.empty((B, x.shape[1]), dtype=torch.bfloat16, device=x.device)
    check(_ffi.lib().nvllm_gather_last_tokens(_p(out), _p(x), _p(cu_seqlens_q), B, x.shape[1], BF16, _stream()))
    return out


def argmax(logits, vocab_offset=0, return_max=False):
    """Sampler::greedy_sample (sampler.rs:109-112)."""
    assert logits.is_cuda and logits.stride(1) == 1
    B, V = logits.shape
    ids = torch.empty(B, dtype=torch.int64, device=logits.device)
    mx = torch.empty(B, dtype=torch.float32, device=logits.device) if return_max else None
    dt = F32 if logits.dtype == torch.float32 else BF16
    check(_ffi.lib().nvllm_argmax(_p(ids), _p(mx), _p(logits), B, V, logits.stride(0), vocab_offset, dt, _stream()))
    return (ids, mx) if return_max else ids


def argmax_combine(all_max, all_ids):
    tp, B = all_max.shape
    out = torch.empty(B, dtype=torch.int64, device=all_max.device)
    check(_ffi.lib().nvllm_argmax_combine(_p(out), _p(all_max), _p(all_ids), tp, B, _stream()))
    return out


def sample(logits, temperatures, row_seeds, top_k=None, top_p=None, debug=False):
    """Sampler::forward (sampler.rs:26-106): temperature / top-k / top-p / Gumbel-max per row, greedy where T == 0.
    logits f32 [B, V]; temperatures f32 [B]; row_seeds: uint64 values (any int64/uint64 tensor of bit patterns) [B];
    top_k i32 [B] / top_p f32 [B] optional.  debug=True also returns (kept_count i32 [B], kept_mask u8 [B, V])."""
    _need(logits, torch.float32, "logits"); _need(temperatures, torch.float32, "temperatures")
    assert logits.stride(1) == 1 and row_seeds.element_size() == 8 and row_seeds.is_cuda
    if top_k is not None:
        _need(top_k, torch.int32, "top_k")
    if top_p is not None:
        _need(top_p, torch.float32, "top_p")
    B, V = logits.shape
    ids = torch.empty(B, dtype=torch.int64, device=logits.device)
    cnt = torch.empty(B, dtype=torch.int32, device=logits.device) if debug else None
    mask = torch.empty((B, V), dtype=torch.uint8, device=logits.device) if debug else None
    check(_ffi.lib().nvllm_sample(_p(ids), _p(logits), B, V, logits.stride(0), _p(temperatures), _p(top_k), _p(top_p),
                                  _p(row_seeds), _p(cnt), _p(mask), _stream()))
    return (ids, cnt, mask) if debug else ids


def init_weight(shape, seed, tensor_id, std, dtype=torch.bfloat16, device="cuda"):
    t = torch.empty(shape, dtype=dtype, device=device)
    check(_ffi.lib().nvllm_init_weight(_p(t), t.numel(), seed, tensor_id, std, BF16 if dtype == torch.bfloat16 else F32, _stream()))
    return t


# ---------------------------------------------------------------------------- mechanisms of registered architectures
# (latent attention, Dynamic Tanh norms, mixture of experts: include/nvllm.h, last section).  Operands are bf16 or f32.


def _dt(t):
    if t.dtype == torch.bfloat16:
        return BF16
    if t.dtype == torch.float32:
        return F32
    raise ValueError(f"expected bfloat16 or float32, got {t.dtype}")


def linear(x, w, out_dtype=None, batch=1, bsx=0, bsw=0, bsy=0, out=None, n=None, k=None):
    """y = x . w^T (nvllm_linear).  x [m, ldx], w [n, ldw] (views with a row stride are fine); batch > 1: element strides."""
    m = x.shape[0]
    n = w.shape[0] if n is None else n
    k = w.shape[1] if k is None else k
    out_dtype = out_dtype or x.dtype
    if out is None:
        out = torch.empty((m, n * batch if bsy == n else n), dtype=out_dtype, device=x.device)
    check(_ffi.lib().nvllm_linear(_p(out), _p(x), _p(w), m, n, k, x.stride(0), w.stride(0), out.stride(0), batch, bsx, bsw, bsy,
                                  _dt(x), _dt(out), _stream()))
    return out


def linear_grouped(x, w, row_src, tile_group, max_rows, n, k, group_stride_w, glu=False, limit=0.0, ldw=None):
    out = torch.zeros((max_rows, n), dtype=x.dtype, device=x.device)
    check(_ffi.lib().nvllm_linear_grouped(_p(out), _p(x), _p(w), max_rows, n, k, x.stride(0), ldw or k, n, group_stride_w,
                                          _p(row_src), _p(tile_group), int(glu), limit, _dt(x), _dt(x), _stream()))
    return out


def glu_clamped(gate_up, limit):
    n, ff2 = gate_up.shape
    out = torch.empty((n, ff2 // 2), dtype=gate_up.dtype, device=gate_up.device)
    check(_ffi.lib().nvllm_glu_clamped(_p(out), _p(gate_up), n, ff2 // 2, limit, _dt(gate_up), _stream()))
    return out


def dyt_residual_norm(h, y=None, post=None, pre=None, dtype=torch.bfloat16):
    """h (f32 [n, hidden], in place) += dyt_post(y); returns dyt_pre(h) (or None).  post / pre: (alpha[1], w, b) f32 tensors."""
    n, hidden = h.shape
    out = torch.empty((n, hidden), dtype=dtype, device=h.device) if pre is not None else None
    pa, pw, pb = post if post is not None else (None, None, None)
    qa, qw, qb = pre if pre is not None else (None, None, None)
    check(_ffi.lib().nvllm_dyt_residual_norm(_p(out), _p(h), _p(y), _p(pa), _p(pw), _p(pb), _p(qa), _p(qw), _p(qb), n, hidden,
                                             _dt(y) if y is not None else _dt(out), _stream()))
    return out


def rope_table_interleaved(max_pos, dims, base, device):
    tab = torch.empty((max_pos, dims // 2, 2), dtype=torch.float32, device=device)
    check(_ffi.lib().nvllm_rope_table_interleaved(_p(tab), max_pos, dims, float(base), _stream()))
    return tab


def latent_prepare(q, dkv, c_norm_w, eps, positions, table, rot_dims, heads, dim, rot_dim, kv_rank, cache, slots):
    """In place on q; writes cache rows (cache: [slots, row] tensor)."""
    check(_ffi.lib().nvllm_latent_prepare(_p(q), q.stride(0), _p(dkv), dkv.stride(0), _p(c_norm_w), eps, _p(positions), _p(table),
                                          rot_dims, table.shape[0] if table is not None else 1, q.shape[0], heads, dim, rot_dim,
                                          kv_rank, _p(cache), cache.stride(0), _p(slots), _dt(q), _stream()))


def latent_attention(q_abs, q, tok_seq, positions, tables, block_size, cache, heads, dim, rot_dim, kv_rank, scale):
    n = q.shape[0]
    out = torch.empty((n, heads * kv_rank), dtype=q.dtype, device=q.device)
    check(_ffi.lib().nvllm_latent_attention(_p(out), out.stride(0), _p(q_abs), q_abs.stride(0), _p(q), q.stride(0), _p(tok_seq),
                                            _p(positions), _p(tables), tables.shape[1], block_size, _p(cache), cache.stride(0), n,
                                            heads, dim, rot_dim, kv_rank, scale, _dt(q), _stream()))
    return out


def moe_route(logits, bias, top, scale):
    n, e = logits.shape
    idx = torch.empty((n, top), dtype=torch.int32, device=logits.device)
    w = torch.empty((n, top), dtype=torch.float32, device=logits.device)
    check(_ffi.lib().nvllm_moe_route(_p(idx), _p(w), _p(logits), _p(bias), n, e, top, scale, _stream()))
    return idx, w


def moe_sort(topk_idx, experts, tile_rows=32):
    n, top = topk_idx.shape
    rows = _ffi.lib().nvllm_moe_max_rows(n, top, experts, tile_rows)
    dev = topk_idx.device
    row_token = torch.empty(rows, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(rows // tile_rows, dtype=torch.int32, device=dev)
    slot_row = torch.empty((n, top), dtype=torch.int32, device=dev)
    check(_ffi.lib().nvllm_moe_sort(_p(row_token), _p(tile_expert), _p(slot_row), _p(topk_idx), n, top, experts, rows, tile_rows,
                                    _stream()))
    return row_token, tile_expert, slot_row


def gemm_bf16_grouped(x, w, tile_group, n, groups):
    """x [max_rows, k] bf16 (rows already grouped in 128-row tiles), w [groups * n, k] -> [max_rows, n]."""
    _need(x, torch.bfloat16, "x"); _need(w, torch.bfloat16, "w"); _need(tile_group, torch.int32, "tile_group")
    out = torch.empty((x.shape[0], n), dtype=torch.bfloat16, device=x.device)
    check(_ffi.lib().nvllm_gemm_bf16_grouped(_p(out), _p(x), _p(w), x.shape[0], n, x.shape[1], groups, x.stride(0), w.stride(0),
                                             n, _p(tile_group), _stream()))
    return out


def moe_combine(expert_out, x, shared_out, topk_idx, topk_w, slot_row, experts):
    n, hidden = x.shape
    out = torch.empty_like(x)
    check(_ffi.lib().nvllm_moe_combine(_p(out), _p(expert_out), _p(x), _p(shared_out), _p(topk_idx), _p(topk_w), _p(slot_row), n,
                                       hidden, topk_idx.shape[1], experts, _dt(x), _stream()))
    return out


# (parallel blocks on an f32 stream, capped attention, recurrent mixers: include/nvllm.h)


def residual_layernorm(h, addends=(), bias=None, bias_scale=1.0, weight=None, eps=1e-5, dtype=torch.bfloat16):
    """h (f32 [n, hidden], in place) += sum of scale * addend (+ bias_scale * bias); returns layer_norm(h) * weight in
    `dtype` (None without a weight).  addends: up to three (tensor, scale), f32 or bf16."""
    n, hidden = h.shape
    out = torch.empty((n, hidden), dtype=dtype, device=h.device) if weight is not None else None
    a = list(addends) + [(None, 0.0)] * (3 - len(addends))
    args = []
    for t, s in a:
        args += [_p(t), float(s), _dt(t) if t is not None else F32]
    check(_ffi.lib().nvllm_residual_layernorm(_p(out), _p(h), *args, _p(bias), float(bias_scale), _p(weight), n, hidden, eps,
                                              BF16 if dtype == torch.bfloat16 else F32, _stream()))
    return out


def concat_cast(a, b, dtype):
    out = torch.empty((a.shape[0], a.shape[1] + b.shape[1]), dtype=dtype, device=a.device)
    check(_ffi.lib().nvllm_concat_cast(_p(out), _p(a), _p(b), a.shape[0], a.shape[1], b.shape[1], _dt(out), _stream()))
    return out


def embedding_gather_scaled(table, ids, scale, copy=False):
    n, hidden = ids.shape[0], table.shape[1]
    h = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    h2 = torch.empty_like(h) if copy else None
    check(_ffi.lib().nvllm_embedding_gather_scaled(_p(h), _p(h2), _p(table), _p(ids), n, hidden, table.shape[0], float(scale),
                                                   _dt(table), _stream()))
    return (h, h2) if copy else h


def ff_activation(x, kind):
    """kind 0: silu(x[:, :ff]) * x[:, ff:];  kind 1: relu(x)^2."""
    n, cols = x.shape
    ff = cols // 2 if kind == 0 else cols
    out = torch.empty((n, ff), dtype=x.dtype, device=x.device)
    check(_ffi.lib().nvllm_ff_activation(_p(out), _p(x), n, ff, kind, _dt(x), _stream()))
    return out


def moe_table_route(table, ids):
    n, top = ids.shape[0], table.shape[1]
    idx = torch.empty((n, top), dtype=torch.int32, device=ids.device)
    w = torch.empty((n, top), dtype=torch.float32, device=ids.device)
    check(_ffi.lib().nvllm_moe_table_route(_p(idx), _p(w), _p(table), _p(ids), n, top, table.shape[0], _stream()))
    return idx, w


def attn_bias_store(proj, q_cols, k_cols, v_cols, q_bias, k_bias, v_bias, k_cache, v_cache, slots, dtype):
    """proj: f32 [n, >= q + k + v columns].  Returns q in `dtype`; k / v (+ biases) go to cache rows `slots`."""
    n = proj.shape[0]
    q = torch.empty((n, q_cols), dtype=dtype, device=proj.device)
    check(_ffi.lib().nvllm_attn_bias_store(_p(q), q.stride(0), _p(k_cache), _p(v_cache), k_cache.stride(0), v_cache.stride(0), _p(proj),
                                           proj.stride(0), _p(q_bias), _p(k_bias), _p(v_bias), _p(slots), n, q_cols, k_cols, v_cols,
                                           _dt(q), _stream()))
    return q


def capped_attention(q, gate, k_cache, v_cache, tok_seq, positions, tables, block_size, heads, kv_heads, dim, vdim, scale,
                     softcap=0.0, temp_coef=0.0, temp_every=1, cu_tokens=None):
    n = q.shape[0]
    out = torch.empty((n, heads * vdim), dtype=q.dtype, device=q.device)
    check(_ffi.lib().nvllm_capped_attention(_p(out), out.stride(0), _p(q), q.stride(0), _p(gate), gate.stride(0) if gate is not None else 0,
                                            _p(k_cache), _p(v_cache), k_cache.stride(0), v_cache.stride(0), _p(tok_seq), _p(positions),
                                            _p(tables), tables.shape[1], block_size, n, heads, kv_heads, dim, vdim, scale, softcap,
                                            temp_coef, temp_every, _p(cu_tokens), cu_tokens.shape[0] - 1 if cu_tokens is not None else 0,
                                            _dt(q), _stream()))
    return out


def linear_recurrence(q, k, v, decay, state, seq_slot, cu_tokens, positions, heads, groups, dk, dv, step=None, skip=None):
    """S <- a S + b k v^T, y = S^T q + skip * v over the sequences of a step; state [slots, heads, dk, dv] f32 is updated.
    decay / step: [n, heads] (per token) or [heads]."""
    n = v.shape[0]
    y = torch.empty((n, heads * dv), dtype=torch.float32, device=v.device)
    check(_ffi.lib().nvllm_linear_recurrence(_p(y), y.stride(0), _p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _p(decay),
                                             int(decay.dim() == 2), _p(step), int(step is not None and step.dim() == 2), _p(skip),
                                             _p(state), _p(seq_slot), _p(cu_tokens), _p(positions), seq_slot.shape[0], heads, groups, dk,
                                             dv, _stream()))
    return y


def causal_conv(x, w, bias, state, tok_seq, seq_slot, cu_tokens, positions, silu=True):
    """x f32 [n, channels] (a view with a row stride is fine), w [channels, taps], state [slots, taps - 1, channels] (updated)."""
    n, ch = x.shape
    out = torch.empty((n, ch), dtype=torch.float32, device=x.device)
    check(_ffi.lib().nvllm_causal_conv(_p(out), out.stride(0), _p(x), x.stride(0), _p(w), _p(bias), _p(state), _p(tok_seq), _p(seq_slot),
                                       _p(cu_tokens), _p(positions), n, seq_slot.shape[0], ch, w.shape[1], int(silu), _stream()))
    return out


def ssd_prepare(dt_raw, dt_bias, a_log):
    n, heads = dt_raw.shape
    step = torch.empty((n, heads), dtype=torch.float32, device=dt_raw.device)
    decay = torch.empty_like(step)
    check(_ffi.lib().nvllm_ssd_prepare(_p(step), _p(decay), _p(dt_raw), dt_raw.stride(0), _p(dt_bias), _p(a_log), n, heads, _stream()))
    return step, decay


def rotate_half(x, positions, table, heads, dim, dims, scale=1.0):
    """In place on f32 x [n, heads * dim] (row stride allowed)."""
    check(_ffi.lib().nvllm_rotate_half(_p(x), x.stride(0), _p(positions), _p(table), table.shape[0] if table is not None else 1,
                                       x.shape[0], heads, dim, dims, float(scale), _stream()))
    return x


def gated_group_norm(y, gate, weight, parts, eps, gate_first, dtype):
    n, cols = y.shape
    out = torch.empty((n, cols), dtype=dtype, device=y.device)
    check(_ffi.lib().nvllm_gated_group_norm(_p(out), out.stride(0), _p(y), y.stride(0), _p(gate), gate.stride(0), _p(weight), n, cols,
                                            parts, eps, int(gate_first), _dt(out), _stream()))
    return out


# (sandwich RMS norms, a hashed bigram embedding, windowed attention with sinks, latent attention in a window, the gated
# delta rule: include/nvllm.h)


def rms_residual_norm(h, y=None, post_w=None, pre_w=None, eps=1e-5, dtype=torch.bfloat16):
    """h (f32 [n, hidden], in place) += rms(y) * post_w; returns rms(h) * pre_w in `dtype` (None without pre_w)."""
    n, hidden = h.shape
    out = torch.empty((n, hidden), dtype=dtype, device=h.device) if pre_w is not None else None
    check(_ffi.lib().nvllm_rms_residual_norm(_p(out), _p(h), _p(y), _dt(y) if y is not None else F32, _p(post_w), _p(pre_w), n, hidden, eps,
                                             BF16 if dtype == torch.bfloat16 else F32, _stream()))
    return out


def rms_norm_rows(x, weight, eps, dtype, out=None, row_map=None):
    """rms(x[i]) * weight into out[row_map[i]] (a cache, rows < 0 skipped) or a new [n, cols] tensor; x f32 (row stride allowed)."""
    n, cols = x.shape
    if out is None:
        out = torch.empty((n, cols), dtype=dtype, device=x.device)
    check(_ffi.lib().nvllm_rms_norm_rows(_p(out), out.stride(0), _p(x), x.stride(0), _p(weight), _p(row_map), n, cols, eps, _dt(out), _stream()))
    return out


def embedding_bigram(table, bigram, ids, positions, tok_seq, cu_tokens, seq_slot, last_token, mul_prev, mul_cur, scale):
    """table[ids] * scale + bigram[hash(previous, current)] as f32; last_token (int32 [slots]) is read and updated."""
    n, hidden = ids.shape[0], table.shape[1]
    h = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    check(_ffi.lib().nvllm_embedding_bigram(_p(h), _p(table), _p(bigram), _p(ids), _p(positions), _p(tok_seq), _p(cu_tokens), _p(seq_slot),
                                            _p(last_token), n, hidden, table.shape[0], bigram.shape[0] - 1, mul_prev, mul_cur, float(scale),
                                            _dt(table), _stream()))
    return h


def attn_rope_norm_store(proj, heads, kv_heads, dim, vdim, q_bias, k_bias, v_bias, positions, table, rot_dims, norm_eps, k_cache, v_cache,
                         slots, dtype, v_from_k=False):
    """proj: f32 [n, >= q + k (+ v) columns].  Returns q in `dtype`; k / v go to cache rows `slots`."""
    n = proj.shape[0]
    q = torch.empty((n, heads * dim), dtype=dtype, device=proj.device)
    check(_ffi.lib().nvllm_attn_rope_norm_store(_p(q), q.stride(0), _p(k_cache), _p(v_cache), k_cache.stride(0), v_cache.stride(0), _p(proj),
                                                proj.stride(0), _p(q_bias), _p(k_bias), _p(v_bias), _p(positions), _p(table), rot_dims,
                                                table.shape[0] if table is not None else 1, float(norm_eps), _p(slots), n, heads, kv_heads,
                                                dim, vdim, int(v_from_k), _dt(q), _stream()))
    return q


def window_attention(q, gate, k_cache, v_cache, tok_seq, positions, tables, block_size, heads, kv_heads, dim, vdim, scale, window=0,
                     sinks=None, gate_per_head=False, softcap=0.0, temp_coef=0.0, temp_every=1, cu_tokens=None):
    """tables None (cu_tokens given): the keys are not paged, key j of sequence s is row cu_tokens[s] + j of k_cache / v_cache."""
    n = q.shape[0]
    out = torch.empty((n, heads * vdim), dtype=q.dtype, device=q.device)
    check(_ffi.lib().nvllm_window_attention(_p(out), out.stride(0), _p(q), q.stride(0), _p(gate), gate.stride(0) if gate is not None else 0,
                                            int(gate_per_head), _p(k_cache), _p(v_cache), k_cache.stride(0), v_cache.stride(0), _p(tok_seq),
                                            _p(positions), _p(tables), tables.shape[1] if tables is not None else 1, block_size, n, heads, kv_heads, dim, vdim, scale,
                                            softcap, temp_coef, temp_every, window, _p(sinks), _p(cu_tokens),
                                            cu_tokens.shape[0] - 1 if cu_tokens is not None else 0, _dt(q), _stream()))
    return out


def latent_window_attention(q_abs, tok_seq, positions, tables, block_size, cache, heads, kv_rank, scale, dtype, window=0, sinks=None,
                            gate=None, workspace=None):
    """q_abs f32 [n, heads * kv_rank] (the key map folded into the query); cache [slots, row >= kv_rank] in `dtype`."""
    n = q_abs.shape[0]
    out = torch.empty((n, heads * kv_rank), dtype=dtype, device=q_abs.device)
    check(_ffi.lib().nvllm_latent_window_attention(_p(out), out.stride(0), _p(q_abs), q_abs.stride(0), None, 0, _p(tok_seq), _p(positions),
                                                   _p(tables), tables.shape[1], block_size, _p(cache), cache.stride(0), n, heads, 0, 0,
                                                   kv_rank, scale, window, _p(sinks), _p(gate), gate.stride(0) if gate is not None else 0,
                                                   _p(workspace), workspace.numel() * 4 if workspace is not None else 0, _dt(out), _stream()))
    return out


def delta_prepare(q, k, beta, decay, a_log, dt_bias, heads, groups, dk, q_scale, unit_eps=1e-6):
    """In place, f32: q / k [n, groups * dk] -> unit vectors (q scaled), beta [n, heads] -> sigmoid, decay [n, heads * dk] ->
    exp(-exp(a_log) softplus(decay + dt_bias))."""
    check(_ffi.lib().nvllm_delta_prepare(_p(q), q.stride(0), _p(k), k.stride(0), _p(beta), beta.stride(0), _p(decay), decay.stride(0), _p(a_log),
                                         _p(dt_bias), q.shape[0], heads, groups, dk, float(q_scale), float(unit_eps), _stream()))


def gated_delta_recurrence(q, k, v, decay, beta, state, seq_slot, cu_tokens, positions, heads, groups, dk, dv):
    """S <- diag(g) S, u = beta (v - S^T k), S <- S + k u^T, y = S^T q over the sequences of a step; state [slots, heads, dk, dv]."""
    n = v.shape[0]
    y = torch.empty((n, heads * dv), dtype=torch.float32, device=v.device)
    check(_ffi.lib().nvllm_gated_delta_recurrence(_p(y), y.stride(0), _p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _p(decay),
                                                  decay.stride(0), _p(beta), beta.stride(0), _p(state), _p(seq_slot), _p(cu_tokens),
                                                  _p(positions), seq_slot.shape[0], heads, groups, dk, dv, _stream()))
    return y


def gated_group_norm_act(y, gate, weight, parts, eps, gate_first, dtype, gate_act=0, w_shared=False):
    """gated_group_norm with the gate's activation (0 SiLU, 1 sigmoid) and optionally one weight vector shared by the parts."""
    n, cols = y.shape
    out = torch.empty((n, cols), dtype=dtype, device=y.device)
    check(_ffi.lib().nvllm_gated_group_norm_act(_p(out), out.stride(0), _p(y), y.stride(0), _p(gate), gate.stride(0), _p(weight), int(w_shared),
                                                n, cols, parts, eps, int(gate_first), gate_act, _dt(out), _stream()))
    return out


# ---- post-norm blocks, chunked attention with a distance bias, rotated values, xIELU, routing on logits (include/nvllm.h)


def residual_cast(h, dtype):
    """The f32 stream in the operand type (nvllm_rms_residual_norm without an incoming sublayer and without a norm)."""
    n, hidden = h.shape
    out = torch.empty((n, hidden), dtype=dtype, device=h.device)
    check(_ffi.lib().nvllm_rms_residual_norm(_p(out), _p(h), None, F32, None, None, n, hidden, 1e-5, BF16 if dtype == torch.bfloat16 else F32,
                                             _stream()))
    return out


def rms_residual_add(h, y, post_w, eps, dtype):
    """h (f32, in place) += rms(y) * post_w; returns h in `dtype`."""
    n, hidden = h.shape
    out = torch.empty((n, hidden), dtype=dtype, device=h.device)
    check(_ffi.lib().nvllm_rms_residual_norm(_p(out), _p(h), _p(y), _dt(y), _p(post_w), None, n, hidden, eps,
                                             BF16 if dtype == torch.bfloat16 else F32, _stream()))
    return out


def attn_wide_norm_store(proj, q_cols, k_cols, v_cols, q_norm_w, k_norm_w, eps, k_cache, v_cache, slots, dtype):
    """proj: f32 [n, >= q + k + v columns].  Returns rms(q) * q_norm_w in `dtype`; rms(k) * k_norm_w and v go to cache rows `slots`."""
    n = proj.shape[0]
    q = torch.empty((n, q_cols), dtype=dtype, device=proj.device)
    check(_ffi.lib().nvllm_attn_wide_norm_store(_p(q), q.stride(0), _p(k_cache), _p(v_cache), k_cache.stride(0) if k_cache is not None else 0,
                                                v_cache.stride(0) if v_cache is not None else 0, _p(proj), proj.stride(0), _p(q_norm_w),
                                                _p(k_norm_w), float(eps), _p(slots), n, q_cols, k_cols, v_cols, _dt(q), _stream()))
    return q


def attn_rotary_store(proj, heads, kv_heads, dim, vdim, positions, table, rot_dims, halves, v_table, norm_eps, k_cache, v_cache, slots, dtype,
                      q_bias=None, k_bias=None, v_bias=None):
    """attn_rope_norm_store with the pairing as a parameter and (v_table) values rotated over all of vdim before the store."""
    n = proj.shape[0]
    q = torch.empty((n, heads * dim), dtype=dtype, device=proj.device)
    max_pos = table.shape[0] if table is not None else (v_table.shape[0] if v_table is not None else 1)
    check(_ffi.lib().nvllm_attn_rotary_store(_p(q), q.stride(0), _p(k_cache), _p(v_cache), k_cache.stride(0), v_cache.stride(0), _p(proj),
                                             proj.stride(0), _p(q_bias), _p(k_bias), _p(v_bias), _p(positions), _p(table), rot_dims, int(halves),
                                             _p(v_table), max_pos, float(norm_eps), _p(slots), n, heads, kv_heads, dim, vdim, 0, _dt(q),
                                             _stream()))
    return q


def biased_attention(q, gate, k_cache, v_cache, tok_seq, positions, tables, block_size, heads, kv_heads, dim, vdim, scale, window=0,
                     sinks=None, gate_per_head=False, chunk=0, head_scale=None, dist_bias=None, out_rot=None, cu_tokens=None):
    """window_attention with a chunk mask, a factor per head, a distance-bias table [heads, rows] and an output rotation table."""
    n = q.shape[0]
    out = torch.empty((n, heads * vdim), dtype=q.dtype, device=q.device)
    check(_ffi.lib().nvllm_biased_attention(_p(out), out.stride(0), _p(q), q.stride(0), _p(gate), gate.stride(0) if gate is not None else 0,
                                            int(gate_per_head), _p(k_cache), _p(v_cache), k_cache.stride(0), v_cache.stride(0), _p(tok_seq),
                                            _p(positions), _p(tables), tables.shape[1] if tables is not None else 1, block_size, n, heads,
                                            kv_heads, dim, vdim, scale, 0.0, 0.0, 1, window, _p(sinks), chunk, _p(head_scale), _p(dist_bias),
                                            dist_bias.shape[1] if dist_bias is not None else 0, _p(out_rot),
                                            out_rot.shape[0] if out_rot is not None else 0, _p(cu_tokens),
                                            cu_tokens.shape[0] - 1 if cu_tokens is not None else 0, _dt(q), _stream()))
    return out


def xielu(x, params):
    """out = softplus(p0) x^2 + x / 2 for x > 0, (1/2 + softplus(p1)) (exp(x) - 1 - x) + x / 2 otherwise; params: f32 [2]."""
    n, ff = x.shape
    out = torch.empty((n, ff), dtype=x.dtype, device=x.device)
    check(_ffi.lib().nvllm_ff_activation_params(_p(out), _p(x), n, ff, 2, _p(params), _dt(x), _stream()))
    return out


def moe_route_logits(logits, bias, top):
    """The `top` largest of logits + bias (ties: lowest index) and the softmax over those alone."""
    n, experts = logits.shape
    idx = torch.empty((n, top), dtype=torch.int32, device=logits.device)
    w = torch.empty((n, top), dtype=torch.float32, device=logits.device)
    check(_ffi.lib().nvllm_moe_route_logits(_p(idx), _p(w), _p(logits), logits.stride(0), _p(bias), n, experts, top, _stream()))
    return idx, w


def embedding_stream(table, ids, scale, dtype):
    """table[ids] * scale as the f32 stream, and the same rows in `dtype`."""
    n, hidden = ids.shape[0], table.shape[1]
    h = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    x = torch.empty((n, hidden), dtype=dtype, device=table.device)
    check(_ffi.lib().nvllm_embedding_stream(_p(h), _p(x), BF16 if dtype == torch.bfloat16 else F32, _p(table), _p(ids), n, hidden, table.shape[0],
                                            float(scale), _dt(table), _stream()))
    return h, x
