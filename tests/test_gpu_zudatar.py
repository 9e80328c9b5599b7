"""GPU tests of the Zudatar architecture: every mechanism's kernel against oracle/zudatar.py (plain numpy, float64), then the
engine — whole prompts, token-by-token decoding, portions down to two tokens, mixed batches with reused pages and state
slots, windows that pass over decoded tokens, greedy generation through LLMEngine.generate and a replay through
bin/trace_run — on small random models.  f32 engines must agree with the oracle to rounding; bf16 engines within the error
of bf16 operands.  Where random weights would hide a fault (one key among hundreds, a window's edge, a sink) the inputs are
made so that one score stands out."""
import json
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import zudatar as Z

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 2e-4, "bfloat16": 6e-2}
F32 = torch.float32


def within(e, dtype):
    """f32: every position to rounding.  bf16: operand rounding through the layers of a narrow model scatters (a few
    positions reach 0.1 of a row's spread, the typical one stays near 0.02); a wrong key, state or page moves rows by O(1)."""
    e = np.asarray(e)
    if not np.isfinite(e).all():
        return False
    return e.max() < TOL[dtype] if dtype == "float32" else (e.max() < 0.2 and e.mean() < 0.05)


def dev_t(a, dev, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev).to(dtype)


def dev_i(a, dev, dtype=torch.int32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev).to(dtype)


def rel_err(got, ref):
    """Per row: rms of the centred difference over the rms of the centred reference."""
    d = np.asarray(got, np.float64) - ref
    d = d - d.mean(-1, keepdims=True)
    r = ref - ref.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt((r ** 2).mean(-1))


f32r = lambda x: np.asarray(x, np.float32).astype(np.float64)


# ------------------------------------------------------------------------------------------------ mechanisms alone


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hid", [50, 256, 1, 3000])
def test_rms_residual_norm(cuda, dtype, hid):
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(hid)
    n, eps = 9, 1e-3
    h, y = rng.standard_normal((n, hid)) * 3 + 0.5, rng.standard_normal((n, hid)) * 2
    post, pre = rng.standard_normal(hid), rng.standard_normal(hid)
    for y_dt in (torch.float32, dtype):
        yy = Z.bf16_round(y) if y_dt == torch.bfloat16 else f32r(y)
        hd = dev_t(h, cuda)
        out = ops.rms_residual_norm(hd, dev_t(yy, cuda, y_dt), dev_t(post, cuda), dev_t(pre, cuda), eps, dtype)
        h_ref = f32r(h) + np.stack([Z.rms(r, eps) for r in yy]) * f32r(post)
        np.testing.assert_allclose(hd.cpu().numpy(), h_ref, rtol=3e-6, atol=3e-6)
        ref = np.stack([Z.rms(r, eps) for r in h_ref]) * f32r(pre)
        tol = 1e-2 if dtype == torch.bfloat16 else 2e-5
        np.testing.assert_allclose(out.float().cpu().numpy(), ref, rtol=tol, atol=tol)
        # the sum alone and the norm alone compose to the same
        h2 = dev_t(h, cuda)
        assert ops.rms_residual_norm(h2, dev_t(yy, cuda, y_dt), dev_t(post, cuda), None, eps, dtype) is None
        assert torch.equal(h2, hd)
        assert torch.equal(ops.rms_residual_norm(h2, None, None, dev_t(pre, cuda), eps, dtype), out) and torch.equal(h2, hd)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rms_norm_rows_into_cache_slots(cuda, dtype):
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(3)
    n, cols, eps = 11, 13, 1e-4
    x, w = rng.standard_normal((n, cols + 5)), rng.standard_normal(cols)
    tol = 1e-2 if dtype == torch.bfloat16 else 2e-5
    ref = np.stack([Z.rms(r, eps) for r in f32r(x)[:, 2:2 + cols]]) * f32r(w)
    got = ops.rms_norm_rows(dev_t(x, cuda)[:, 2:2 + cols], dev_t(w, cuda), eps, dtype)
    np.testing.assert_allclose(got.float().cpu().numpy(), ref, rtol=tol, atol=tol)
    cache = torch.full((40, 16), 7.0, dtype=dtype, device=cuda)       # rows of 16 for 13 values: the padding is not touched
    slots = rng.permutation(40)[:n].astype(np.int32)
    slots[4] = -1
    ops.rms_norm_rows(dev_t(x, cuda)[:, 2:2 + cols], dev_t(w, cuda), eps, dtype, out=cache, row_map=dev_i(slots, cuda))
    c = cache.float().cpu().numpy()
    for i, s in enumerate(slots):
        if s >= 0:
            np.testing.assert_allclose(c[s, :cols], ref[i], rtol=tol, atol=tol)
    untouched = np.ones(40, bool); untouched[slots[slots >= 0]] = False
    assert (c[untouched] == 7.0).all() and (c[:, cols:] == 7.0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hid", [10, 16])
def test_embedding_bigram_across_portions_and_slots(cuda, dtype, hid):
    """Three sequences in portions; the token before a portion comes from the state slot, the first token of a sequence reads
    the extra row although its slot still holds another sequence's last token."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(5)
    vocab, buckets, mp, mc, scale = 29, 17, 13, 5, 2.5
    bg = {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}
    table, bigram = Z.bf16_round(rng.standard_normal((vocab, hid))), Z.bf16_round(rng.standard_normal((buckets + 1, hid)))
    seqs = [rng.integers(0, vocab, n).tolist() for n in (9, 1, 6)]
    last = torch.full((4,), 5, dtype=torch.int32, device=cuda)      # leftovers of earlier users of the slots
    slots = [2, 0, 3]
    steps = [[(0, 0, 4), (1, 0, 1)], [(0, 4, 1), (2, 0, 2)], [(2, 2, 4), (0, 5, 4)]]     # (sequence, first position, count)
    for step in steps:
        ids, pos, tok_seq, cu = [], [], [], [0]
        for k, (s, p0, c) in enumerate(step):
            ids += seqs[s][p0:p0 + c]; pos += list(range(p0, p0 + c)); tok_seq += [k] * c; cu.append(cu[-1] + c)
        h = ops.embedding_bigram(dev_t(table, cuda, dtype), dev_t(bigram, cuda, dtype), dev_i(ids, cuda, torch.int64), dev_i(pos, cuda, torch.int64),
                                 dev_i(tok_seq, cuda), dev_i(cu, cuda), dev_i([slots[s] for s, _, _ in step], cuda), last, mp, mc, scale)
        got, k = h.cpu().numpy(), 0
        for s, p0, c in step:
            for p in range(p0, p0 + c):
                prev = seqs[s][p - 1] if p > 0 else None
                ref = table[seqs[s][p]] * scale + bigram[Z.bigram_row(prev, seqs[s][p], bg)]
                np.testing.assert_allclose(got[k], ref, rtol=1e-6, atol=1e-6); k += 1
    assert last.cpu().tolist() == [seqs[1][-1], 5, seqs[0][-1], seqs[2][-1]]
    # a padding sequence (slot -1) gives zeros and touches nothing
    h = ops.embedding_bigram(dev_t(table, cuda, dtype), dev_t(bigram, cuda, dtype), dev_i([3], cuda, torch.int64), dev_i([0], cuda, torch.int64),
                             dev_i([0], cuda), dev_i([0, 1], cuda), dev_i([-1], cuda), last, mp, mc, scale)
    assert (h == 0).all()


def _paged(rng, ctxs, bs, spare=3):
    """Random page assignment: tables [seqs, cap], and for every (sequence, position) its cache slot."""
    need = [(c + bs - 1) // bs for c in ctxs]
    perm = rng.permutation(sum(need) + spare)
    cap = max(need) + 1
    tables = -np.ones((len(ctxs), cap), np.int32)
    k = 0
    for s, nb in enumerate(need):
        tables[s, :nb] = perm[k:k + nb]; k += nb
    slot = lambda s, p: int(tables[s, p // bs]) * bs + p % bs
    return tables, slot, (sum(need) + spare) * bs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,rot,v_from_k", [(4, 2, 8, 4, True), (3, 3, 10, 10, True), (2, 1, 6, 0, False), (1, 1, 16, 6, False), (5, 5, 12, 6, True),
                                                 (2, 1, 128, 64, True), (3, 1, 132, 132, True), (2, 2, 16, 0, True)])
def test_attn_rope_norm_store(cuda, dtype, H, G, D, rot, v_from_k):
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(H * 100 + D)
    n, eps, base, V = 7, 1e-3, 50.0, (D if v_from_k else 5)
    cols = H * D + G * D + (0 if v_from_k else G * V)
    cols += 4 if cols % 4 == 0 else 3            # rows of 16-byte multiples take the one-pass kernel
    proj = rng.standard_normal((n, cols))
    qb, kb = rng.standard_normal(H * D), rng.standard_normal(G * D)
    vb = None if v_from_k else rng.standard_normal(G * V)
    pos = rng.integers(0, 40, n)
    slots = rng.permutation(20)[:n].astype(np.int32); slots[2] = -1
    kc = torch.zeros((20, G * D), dtype=dtype, device=cuda); vc = torch.zeros((20, G * V), dtype=dtype, device=cuda)
    table = ops.rope_table_interleaved(64, rot, base, cuda) if rot else None
    q = ops.attn_rope_norm_store(dev_t(proj, cuda), H, G, D, V, dev_t(qb, cuda), dev_t(kb, cuda), dev_t(vb, cuda) if vb is not None else None,
                                 dev_i(pos, cuda, torch.int64), table, rot, eps, kc, vc, dev_i(slots, cuda), dtype, v_from_k)
    p = f32r(proj)
    tol = 1.5e-2 if dtype == torch.bfloat16 else 2e-5
    qg, kg, vg = q.float().cpu().numpy(), kc.float().cpu().numpy(), vc.float().cpu().numpy()
    for t in range(n):
        qq = (p[t, :H * D] + f32r(qb)).reshape(H, D)
        kk = (p[t, H * D:H * D + G * D] + f32r(kb)).reshape(G, D)
        ref_q = np.stack([Z.rms(Z.rotate_pairs(x, pos[t], rot, base), eps) for x in qq])
        np.testing.assert_allclose(qg[t].reshape(H, D), ref_q, rtol=tol, atol=tol)
        if slots[t] < 0:
            continue
        ref_k = np.stack([Z.rms(Z.rotate_pairs(x, pos[t], rot, base), eps) for x in kk])
        np.testing.assert_allclose(kg[slots[t]].reshape(G, D), ref_k, rtol=tol, atol=tol)
        ref_v = kk if v_from_k else (p[t, H * D + G * D:H * D + G * D + G * V] + f32r(vb)).reshape(G, V)
        np.testing.assert_allclose(vg[slots[t]].reshape(G, V), ref_v, rtol=tol, atol=tol)
    assert (kg[np.setdiff1d(np.arange(20), slots[slots >= 0])] == 0).all()


def _window_ref(q, keys, vals, H, G, scale, window, pos, sinks=None, gate=None):
    """q [H, D]; keys / vals: arrays [ctx, G, D] / [ctx, G, V] of the whole sequence."""
    lo = max(0, pos - window + 1) if window > 0 else 0
    out = np.zeros((H, vals.shape[-1]))
    for h in range(H):
        g = h // (H // G)
        s = (keys[lo:pos + 1, g] @ q[h]) * scale
        p = Z.window_softmax(s, None if sinks is None else sinks[h])
        out[h] = p @ vals[lo:pos + 1, g]
        if gate is not None:
            out[h] *= Z.sigmoid(gate[h])
    return out


WIN_CASES = [  # heads, kv heads, dim, vdim, window, page, with sinks
    (4, 2, 8, 8, 7, 16, False), (3, 1, 16, 24, 40, 16, True), (2, 2, 64, 64, 64, 32, True), (4, 4, 128, 128, 100, 64, False),
    (1, 1, 5, 3, 3, 4, True), (6, 2, 32, 32, 1, 16, False), (2, 1, 24, 8, 0, 16, True)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", WIN_CASES)
def test_window_attention_prompts_and_single_tokens(cuda, dtype, case):
    """Three sequences in one launch: a whole prompt, a portion that continues a cached prefix, and a single decoded token,
    pages in random order; windows shorter and longer than a page and than the 64-key tiles."""
    from nano_vllm_rs_b200 import ops
    H, G, D, V, window, bs, with_sinks = case
    rng = np.random.default_rng(sum(case))
    ctx = [150, 201, 333]
    first = [0, 150, 332]                        # first position of each sequence's tokens in this step
    tables, slot, nslots = _paged(rng, ctx, bs)
    K = [Z.bf16_round(rng.standard_normal((c, G, D))) for c in ctx]
    Vv = [Z.bf16_round(rng.standard_normal((c, G, V))) for c in ctx]
    kc, vc = np.zeros((nslots, G * D)), np.zeros((nslots, G * V))
    for s, c in enumerate(ctx):
        for p in range(c):
            kc[slot(s, p)], vc[slot(s, p)] = K[s][p].reshape(-1), Vv[s][p].reshape(-1)
    tok_seq = np.concatenate([[s] * (ctx[s] - first[s]) for s in range(3)]).astype(np.int32)
    pos = np.concatenate([np.arange(first[s], ctx[s]) for s in range(3)])
    cu = np.cumsum([0] + [ctx[s] - first[s] for s in range(3)]).astype(np.int32)
    n = len(pos)
    q = Z.bf16_round(rng.standard_normal((n, H, D)))
    gate = rng.standard_normal((n, H + 2))
    sinks = rng.standard_normal(H) + 1.0 if with_sinks else None
    scale = 0.5 / np.sqrt(D)
    ref = np.stack([_window_ref(q[t], K[tok_seq[t]], Vv[tok_seq[t]], H, G, scale, window, pos[t], sinks, f32r(gate)[t, 1:1 + H]) for t in range(n)])
    for use_cu in (True, False):                 # with token ranges: the tensor-core kernel where the sizes allow it
        out = ops.window_attention(dev_t(q.reshape(n, -1), cuda, dtype), dev_t(gate, cuda)[:, 1:1 + H], dev_t(kc, cuda, dtype), dev_t(vc, cuda, dtype),
                                   dev_i(tok_seq, cuda), dev_i(pos, cuda, torch.int64), dev_i(tables, cuda), bs, H, G, D, V, scale, window,
                                   dev_t(sinks, cuda) if with_sinks else None, True, cu_tokens=dev_i(cu, cuda) if use_cu else None)
        tol = 2e-2 if dtype == torch.bfloat16 else 3e-5
        np.testing.assert_allclose(out.float().cpu().numpy().reshape(n, H, V), ref, rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,V,window", [(4, 4, 16, 8, 33), (6, 2, 32, 32, 64), (2, 1, 12, 20, 0), (3, 3, 128, 64, 100)])
def test_window_attention_over_the_steps_own_rows(cuda, dtype, H, G, D, V, window):
    """Whole prompts whose keys and values are not paged: key j of sequence s is row cu_tokens[s] + j of the key / value
    matrices (no block tables), with sinks and head gates; three prompts of unequal length in one launch."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(H * D + window)
    lens = [150, 1, 203]
    cu = np.cumsum([0] + lens).astype(np.int32)
    n = int(cu[-1])
    K, Vv = Z.bf16_round(rng.standard_normal((n, G, D))), Z.bf16_round(rng.standard_normal((n, G, V)))
    q = Z.bf16_round(rng.standard_normal((n, H, D)))
    gate, sinks = rng.standard_normal((n, H)), rng.standard_normal(H)
    tok_seq = np.concatenate([[s] * l for s, l in enumerate(lens)]).astype(np.int32)
    pos = np.concatenate([np.arange(l) for l in lens])
    scale = 0.6 / np.sqrt(D)
    ref = np.stack([_window_ref(q[t], K[cu[tok_seq[t]]:cu[tok_seq[t] + 1]], Vv[cu[tok_seq[t]]:cu[tok_seq[t] + 1]], H, G, scale, window, pos[t],
                                f32r(sinks), f32r(gate)[t]) for t in range(n)])
    kv = dev_t(np.concatenate([K.reshape(n, -1), Vv.reshape(n, -1)], axis=1), cuda, dtype)     # [K | V] side by side, as one projection writes them
    out = ops.window_attention(dev_t(q.reshape(n, -1), cuda, dtype), dev_t(gate, cuda), kv, kv[:, G * D:], dev_i(tok_seq, cuda), dev_i(pos, cuda, torch.int64),
                               None, 16, H, G, D, V, scale, window, dev_t(sinks, cuda), True, cu_tokens=dev_i(cu, cuda))
    tol = 2e-2 if dtype == torch.bfloat16 else 3e-5
    np.testing.assert_allclose(out.float().cpu().numpy().reshape(n, H, V), ref, rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,bs", [(70, 64), (5, 16), (64, 16), (130, 32)])
def test_window_attention_edges_stand_out(cuda, dtype, window, bs):
    """One key is made to dominate: the last one inside the window must carry the output, the first one outside must not
    show; also the query's own key, a key at a page's last and first slot, and with a strong sink nothing dominates.  Both as
    part of a prompt portion and as a single decoded token."""
    from nano_vllm_rs_b200 import ops
    H, G, D, V = 2, 1, 16, 16
    rng = np.random.default_rng(window)
    ctx = 400
    tables, slot, nslots = _paged(rng, [ctx], bs)
    p_q = 389
    edge_in, edge_out = p_q - window + 1, p_q - window
    page_last, page_first = ((p_q - 1) // bs) * bs - 1, ((p_q - 1) // bs) * bs
    for mode in ("prompt", "single"):
        for hot, seen in ((edge_in, True), (edge_out, False), (p_q, True), (page_last, page_last >= edge_in), (page_first, page_first >= edge_in)):
            K = Z.bf16_round(0.1 * rng.standard_normal((ctx, G, D)))
            Vv = Z.bf16_round(rng.standard_normal((ctx, G, V)))
            qv = Z.bf16_round(rng.standard_normal((H, D)))
            K[hot, 0] = Z.bf16_round(8.0 * qv[0] / np.linalg.norm(qv[0]))        # head 0 scores it far above the rest
            kc, vc = np.zeros((nslots, G * D)), np.zeros((nslots, G * V))
            for p in range(ctx):
                kc[slot(0, p)], vc[slot(0, p)] = K[p].reshape(-1), Vv[p].reshape(-1)
            first = p_q - 20 if mode == "prompt" else p_q
            pos = np.arange(first, p_q + 1)
            n = len(pos)
            q = Z.bf16_round(rng.standard_normal((n, H, D)))
            q[-1] = qv
            scale = 1.0
            out = ops.window_attention(dev_t(q.reshape(n, -1), cuda, dtype), None, dev_t(kc, cuda, dtype), dev_t(vc, cuda, dtype),
                                       dev_i(np.zeros(n), cuda), dev_i(pos, cuda, torch.int64), dev_i(tables, cuda), bs, H, G, D, V, scale, window,
                                       None, False, cu_tokens=dev_i([0, n], cuda)).float().cpu().numpy().reshape(n, H, V)
            ref = _window_ref(q[-1], K, Vv, H, G, scale, window, p_q)
            tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
            np.testing.assert_allclose(out[-1], ref, rtol=tol, atol=tol)
            close = np.abs(out[-1, 0] - Vv[hot, 0]).max() < 0.05
            assert close == seen, (mode, hot, seen)
        # a sink far above every score takes the whole mass: the output vanishes; without it the output is of order one
        sinks = np.array([60.0, -60.0])
        out = ops.window_attention(dev_t(q.reshape(n, -1), cuda, dtype), None, dev_t(kc, cuda, dtype), dev_t(vc, cuda, dtype), dev_i(np.zeros(n), cuda),
                                   dev_i(pos, cuda, torch.int64), dev_i(tables, cuda), bs, H, G, D, V, scale, window, dev_t(sinks, cuda), False,
                                   cu_tokens=dev_i([0, n], cuda)).float().cpu().numpy().reshape(n, H, V)
        assert np.abs(out[:, 0]).max() < 1e-6 and np.abs(out[:, 1]).max() > 0.05


LAT_CASES = [  # heads, kv_rank, window, page
    (3, 12, 5, 16), (16, 64, 70, 64), (4, 128, 64, 16), (5, 20, 0, 16), (17, 96, 33, 32), (1, 7, 1, 4)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", LAT_CASES)
def test_latent_window_attention(cuda, dtype, case):
    """Multi-query attention over cached latents (the key map already folded into the query) with a window, sinks and head
    gates: a whole prompt, a portion after a cached prefix and a single token, pages in random order."""
    from nano_vllm_rs_b200 import ops
    H, R, window, bs = case
    rng = np.random.default_rng(sum(case))
    ctx, first = [140, 203, 300], [0, 150, 299]
    tables, slot, nslots = _paged(rng, ctx, bs)
    row = (R + 7) // 8 * 8
    C = [Z.bf16_round(rng.standard_normal((c, R))) for c in ctx]
    cache = np.zeros((nslots, row))
    for s, c in enumerate(ctx):
        for p in range(c):
            cache[slot(s, p), :R] = C[s][p]
    tok_seq = np.concatenate([[s] * (ctx[s] - first[s]) for s in range(3)]).astype(np.int32)
    pos = np.concatenate([np.arange(first[s], ctx[s]) for s in range(3)])
    n = len(pos)
    qa = rng.standard_normal((n, H, R))
    if dtype == torch.bfloat16:
        qa = Z.bf16_round(qa)                   # the tensor-core kernel rounds the folded query to bf16
    gate, sinks = rng.standard_normal((n, H + 1)), rng.standard_normal(H) + 1.0
    scale = 0.7 / np.sqrt(R)
    ref = np.zeros((n, H, R))
    for t in range(n):
        lo = max(0, pos[t] - window + 1) if window > 0 else 0
        Cs = C[tok_seq[t]][lo:pos[t] + 1]
        for h in range(H):
            p = Z.window_softmax((Cs @ f32r(qa)[t, h]) * scale, f32r(sinks)[h])
            ref[t, h] = (p @ Cs) * Z.sigmoid(f32r(gate)[t, h])
    out = ops.latent_window_attention(dev_t(qa.reshape(n, -1), cuda), dev_i(tok_seq, cuda), dev_i(pos, cuda, torch.int64), dev_i(tables, cuda), bs,
                                      dev_t(cache, cuda, dtype), H, R, scale, dtype, window, dev_t(sinks, cuda), dev_t(gate, cuda)[:, :H])
    tol = 2e-2 if dtype == torch.bfloat16 else 3e-5
    np.testing.assert_allclose(out.float().cpu().numpy().reshape(n, H, R), ref, rtol=tol, atol=tol)


@pytest.mark.parametrize("window", [1000, 1100, 64, 5000])
@pytest.mark.parametrize("H,R", [(3, 24), (20, 64)])
def test_latent_window_attention_splits_keys_of_single_tokens(cuda, window, H, R):
    """Few single tokens (bf16): with a workspace every token's key tiles are split over several CTAs and merged; the result is
    the unsplit kernel's to rounding and the oracle's.  Contexts shorter than a tile, at tile borders, and longer than the window."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(window + H)
    ctx, bs = [300, 65, 3, 1100, 64, 1517, 1], 16
    tables, slot, nslots = _paged(rng, ctx, bs)
    C = [Z.bf16_round(rng.standard_normal((c, R))) for c in ctx]
    cache = np.zeros((nslots, R))
    for s, c in enumerate(ctx):
        for p in range(c):
            cache[slot(s, p)] = C[s][p]
    n = len(ctx)
    pos = np.array(ctx) - 1
    qa = Z.bf16_round(rng.standard_normal((n, H, R)))
    gate, sinks = rng.standard_normal((n, H)), rng.standard_normal(H) + 1.0
    scale = 0.7 / np.sqrt(R)
    ref = np.zeros((n, H, R))
    for t in range(n):
        Cs = C[t][max(0, pos[t] - window + 1):pos[t] + 1]
        for h in range(H):
            ref[t, h] = (Z.window_softmax((Cs @ qa[t, h]) * scale, f32r(sinks)[h]) @ Cs) * Z.sigmoid(f32r(gate)[t, h])
    args = (dev_t(qa.reshape(n, -1), cuda), dev_i(np.arange(n), cuda), dev_i(pos, cuda, torch.int64), dev_i(tables, cuda), bs,
            dev_t(cache, cuda, torch.bfloat16), H, R, scale, torch.bfloat16, window, dev_t(sinks, cuda), dev_t(gate, cuda))
    plain = ops.latent_window_attention(*args).float().cpu().numpy().reshape(n, H, R)
    ws = torch.full((n * H * 4 * (R + 2),), float("nan"), device=cuda)
    split = ops.latent_window_attention(*args, workspace=ws).float().cpu().numpy().reshape(n, H, R)
    assert torch.isnan(ws[:n * H * 2 * (R + 2)]).all() == (window < 1000)     # long windows used the workspace
    np.testing.assert_allclose(split, ref, rtol=2e-2, atol=2e-2)
    np.testing.assert_allclose(split, plain, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_tok", [1, 300])
def test_latent_window_edges_stand_out(cuda, dtype, n_tok):
    """A latent just inside the window carries the output, the one just outside does not show (prompt portion of 300 tokens:
    two tokens per CTA on the tensor-core kernel; and a single token)."""
    from nano_vllm_rs_b200 import ops
    H, R, window, bs = 4, 32, 70, 64
    rng = np.random.default_rng(n_tok)
    ctx, p_q = 500, 470
    tables, slot, nslots = _paged(rng, [ctx], bs)
    for hot, seen in ((p_q - window + 1, True), (p_q - window, False), (p_q, True), (p_q + 1, False), (447, True), (448, True)):
        C = Z.bf16_round(0.1 * rng.standard_normal((ctx, R)))
        qv = Z.bf16_round(rng.standard_normal(R))
        C[hot] = Z.bf16_round(9.0 * qv / np.linalg.norm(qv))
        cache = np.zeros((nslots, R))
        for p in range(ctx):
            cache[slot(0, p)] = C[p]
        pos = np.arange(p_q - n_tok + 1, p_q + 1)
        qa = Z.bf16_round(rng.standard_normal((n_tok, H, R)))
        qa[-1, 1] = qv
        out = ops.latent_window_attention(dev_t(qa.reshape(n_tok, -1), cuda), dev_i(np.zeros(n_tok), cuda), dev_i(pos, cuda, torch.int64),
                                          dev_i(tables, cuda), bs, dev_t(cache, cuda, dtype), H, R, 1.0, dtype, window).float().cpu().numpy()
        got = out.reshape(n_tok, H, R)[-1, 1]
        assert (np.abs(got - C[hot]).max() < 0.05) == seen, (hot, seen)


def _delta_inputs(rng, n, H, G, D, V):
    q, k = rng.standard_normal((n, G * D)), rng.standard_normal((n, G * D))
    v = rng.standard_normal((n, H * V))
    beta = rng.standard_normal((n, H))
    raw = rng.standard_normal((n, H * D))
    return q, k, v, beta, raw


@pytest.mark.parametrize("H,G,D,V", [(4, 2, 6, 5), (2, 2, 32, 32), (3, 1, 130, 7), (1, 1, 1, 1), (2, 1, 64, 40), (8, 8, 20, 96)])
def test_gated_delta_rule_in_portions_through_reused_slots(cuda, H, G, D, V):
    """delta_prepare + the recurrence against the oracle's single step, three sequences cut into portions (one token, two,
    many), in slots that hold another sequence's leftovers."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(H * 1000 + D)
    lens, slots = [37, 5, 70], [3, 0, 2]
    a_log, dt_bias = rng.standard_normal(H) - 1.0, rng.standard_normal(H * D)
    data = [_delta_inputs(rng, n, H, G, D, V) for n in lens]
    # the oracle, token by token
    ref = []
    for (q, k, v, beta, raw) in data:
        q, k, v, beta, raw = map(f32r, (q, k, v, beta, raw))
        S, ys = np.zeros((H, D, V)), []
        for t in range(len(q)):
            qq, kk = q[t].reshape(G, D), k[t].reshape(G, D)
            qq = qq / np.sqrt((qq * qq).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
            kk = kk / np.sqrt((kk * kk).sum(-1, keepdims=True) + 1e-6)
            g = np.exp(-np.exp(f32r(a_log))[:, None] * Z.softplus(raw[t] + f32r(dt_bias)).reshape(H, D))
            b = Z.sigmoid(beta[t])
            y = np.zeros((H, V))
            for h in range(H):
                S[h], y[h] = Z.delta_rule_step(S[h], qq[h // (H // G)], kk[h // (H // G)], v[t].reshape(H, V)[h], b[h], g[h])
            ys.append(y.reshape(-1))
        ref.append(np.stack(ys))
    state = dev_t(rng.standard_normal((4, H, D, V)), cuda)          # leftovers everywhere
    at, got = [0, 0, 0], [[], [], []]
    cuts = [[1, 2, 17, 17], [5], [33, 1, 1, 35]]
    for step in range(4):
        part = [(s, cuts[s][step]) for s in range(3) if step < len(cuts[s])]
        sl = [np.s_[at[s]:at[s] + c] for s, c in part]
        cat = lambda j: np.concatenate([data[s][j][x] for (s, _), x in zip(part, sl)])
        q, k, v, beta, raw = (dev_t(cat(j), cuda) for j in range(5))
        pos = np.concatenate([np.arange(at[s], at[s] + c) for s, c in part])
        cu = np.cumsum([0] + [c for _, c in part]).astype(np.int32)
        ops.delta_prepare(q, k, beta, raw, dev_t(a_log, cuda), dev_t(dt_bias, cuda), H, G, D, D ** -0.5)
        y = ops.gated_delta_recurrence(q, k, v, raw, beta, state, dev_i([slots[s] for s, _ in part], cuda), dev_i(cu, cuda),
                                       dev_i(pos, cuda, torch.int64), H, G, D, V).cpu().numpy()
        for i, (s, c) in enumerate(part):
            got[s].append(y[cu[i]:cu[i + 1]]); at[s] += c
    for s in range(3):
        np.testing.assert_allclose(np.concatenate(got[s]), ref[s], rtol=2e-4, atol=2e-5)
    # a padding sequence (slot -1): zeros, no state touched
    before = state.clone()
    q, k, v, beta, raw = (dev_t(x[:1], cuda) for x in data[0])
    y = ops.gated_delta_recurrence(q, k, v, raw, beta, state, dev_i([-1], cuda), dev_i([0, 1], cuda), dev_i([4], cuda, torch.int64), H, G, D, V)
    assert (y == 0).all() and torch.equal(state, before)


def test_gated_delta_rule_keeps_a_far_token(cuda):
    """A value written 400 tokens back under slow decay is still read out by its key; under fast decay it is gone."""
    from nano_vllm_rs_b200 import ops
    H, D, V, n = 2, 16, 8, 401
    rng = np.random.default_rng(9)
    k = 0.01 * rng.standard_normal((n, D)); q = 0.01 * rng.standard_normal((n, D))
    key = np.zeros(D); key[3] = 1.0
    k[0], q[-1] = key, key                         # the preparation makes both unit vectors and scales q by dim^-1/2
    v = np.zeros((n, H * V)); v[0] = np.arange(1, H * V + 1)
    beta = np.full((n, H), -20.0); beta[0] = 20.0  # only the first token writes
    raw = np.zeros((n, H * D))
    a_log = np.array([-9.0, 1.5])                  # head 0 forgets slowly, head 1 fast
    qd, kd, bd, rd = dev_t(q, cuda), dev_t(k, cuda), dev_t(beta, cuda), dev_t(raw, cuda)
    ops.delta_prepare(qd, kd, bd, rd, dev_t(a_log, cuda), dev_t(np.zeros(H * D), cuda), H, 1, D, D ** -0.5)
    state = torch.zeros((1, H, D, V), device=cuda)
    y = ops.gated_delta_recurrence(qd, kd, dev_t(v, cuda), rd, bd, state, dev_i([0], cuda), dev_i([0, n], cuda), dev_i(np.arange(n), cuda, torch.int64),
                                   H, 1, D, V).cpu().numpy()[-1].reshape(H, V)
    keep = np.exp(-np.exp(-9.0) * np.log(2.0)) ** 400
    np.testing.assert_allclose(y[0], np.arange(1, V + 1) * keep * D ** -0.5, rtol=2e-3)
    assert np.abs(y[1]).max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols,parts", [(20, 4), (64, 2), (7, 7), (96, 1)])
def test_gated_group_norm_sigmoid_gate_shared_weight(cuda, dtype, cols, parts):
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(cols)
    n, eps, gs = 5, 1e-3, cols // parts
    y, z, w = rng.standard_normal((n, cols)), rng.standard_normal((n, cols)), rng.standard_normal(gs)
    out = ops.gated_group_norm_act(dev_t(y, cuda), dev_t(z, cuda), dev_t(w, cuda), parts, eps, False, dtype, gate_act=1, w_shared=True)
    ref = np.stack([np.concatenate([Z.rms(p, eps) * f32r(w) for p in np.split(r, parts)]) for r in f32r(y)]) * Z.sigmoid(f32r(z))
    tol = 1e-2 if dtype == torch.bfloat16 else 2e-5
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, rtol=tol, atol=tol)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m,n,k,heads", [(1, 40, 24, 1), (5, 64, 128, 6), (64, 128, 512, 4), (70, 24, 72, 3), (130, 513, 8, 2), (300, 16, 200, 5)])
def test_batched_small_products_on_tensor_cores(cuda, monkeypatch, m, n, k, heads, out_dtype):
    """Per-head products y_h = x_h . w_h^T out of packed activations (few rows, reduction sizes that are not multiples of
    64): the mma.sync tile kernel against float64, and against the CUDA-core tile kernel it stands in for."""
    from nano_vllm_rs_b200 import ops
    rng = np.random.default_rng(m + n + k)
    x = Z.bf16_round(rng.standard_normal((m, heads * k + 8)))
    w = Z.bf16_round(rng.standard_normal((heads * n, k)) / np.sqrt(k))
    xd, wd = dev_t(x, cuda, torch.bfloat16), dev_t(w, cuda, torch.bfloat16)
    run = lambda: ops.linear(xd, wd, out_dtype, batch=heads, bsx=k, bsw=n * k, bsy=n, n=n, k=k,
                             out=torch.zeros((m, heads * n), dtype=out_dtype, device=cuda)).float().cpu().numpy()
    got = run()
    ref = np.concatenate([x[:, h * k:(h + 1) * k] @ w[h * n:(h + 1) * n].T for h in range(heads)], axis=1)
    tol = 1e-2 if out_dtype == torch.bfloat16 else 2e-5
    np.testing.assert_allclose(got, ref, rtol=tol, atol=tol)
    monkeypatch.setenv("NVLLM_LINEAR_MMA", "0")
    np.testing.assert_allclose(run(), got, rtol=tol, atol=tol)
    # a row's result does not depend on the rows beside it
    one = ops.linear(xd[m - 1:], wd, out_dtype, batch=heads, bsx=k, bsw=n * k, bsy=n, n=n, k=k,
                     out=torch.zeros((1, heads * n), dtype=out_dtype, device=cuda)).float().cpu().numpy()
    monkeypatch.delenv("NVLLM_LINEAR_MMA")
    one2 = ops.linear(xd[m - 1:], wd, out_dtype, batch=heads, bsx=k, bsw=n * k, bsy=n, n=n, k=k,
                      out=torch.zeros((1, heads * n), dtype=out_dtype, device=cuda)).float().cpu().numpy()
    assert np.array_equal(one2, got[m - 1:]) and np.allclose(one, got[m - 1:], rtol=tol, atol=tol)


# ------------------------------------------------------------------------------------------------ the engine


def variant(name):
    A, L, D = Z.attention_mixer, Z.latent_mixer, Z.delta_mixer
    if name == "all_kinds":      # every mixer, grouped heads, sizes all different, a layer that reads the latents of layer 1
        return Z.make_config([("channel_delta", D(), None), ("latent_attention", L(), Z.dense_mlp(20)), ("attention", A(), Z.dense_mlp(12)),
                              ("latent_attention", L(heads=2, dim=5, vdim=4, q_rank=7, window=9, kv_from=1), None),
                              ("channel_delta", D(heads=2, kv_heads=1, dim=9, vdim=3, taps=2), Z.dense_mlp(16))])
    if name == "ones":           # sizes that are 1 or equal to one another; one tap; a window of one; no rotation; scales of 1
        return Z.make_config([("attention", A(heads=1, kv_heads=1, dim=6, window=1, rot_dims=0, scale=1.0), None),
                              ("channel_delta", D(heads=1, kv_heads=1, dim=1, vdim=1, taps=1), Z.dense_mlp(8)),
                              ("latent_attention", L(heads=1, dim=1, vdim=1, kv_rank=1, q_rank=1, window=300, scale=1.0), None),
                              ("attention", A(heads=3, kv_heads=3, dim=8, window=300, rot_dims=8, scale=0.3), Z.dense_mlp(8))],
                             width=16, vocab=33, embed_scale=1.0, buckets=1, mul_prev=1, mul_cur=1, logit_scale=1.0)
    if name == "tensor_core":    # sizes the tensor-core kernels accept (bf16): width and inner sizes multiples of 64
        return Z.make_config([("latent_attention", L(heads=2, dim=64, vdim=32, kv_rank=64, q_rank=64, window=40, scale=0.1), Z.dense_mlp(128)),
                              ("channel_delta", dict(D(heads=2, kv_heads=1, dim=32, vdim=32, taps=4), low_rank=64), None),
                              ("attention", A(heads=4, kv_heads=2, dim=32, window=70, rot_dims=16, rot_base=1e4, scale=0.2), Z.dense_mlp(128)),
                              ("latent_attention", L(heads=2, dim=64, vdim=64, kv_rank=64, q_rank=128, window=64, scale=0.1, kv_from=0), None)],
                             width=64, vocab=96, buckets=101)
    raise KeyError(name)


VARIANTS = ["all_kinds", "ones", "tensor_core"]


def weights_for(cfg, rng):
    low = None
    for l in cfg["layers"]:
        if "low_rank" in l["mixer"]:
            low = l["mixer"]["low_rank"]
    return Z.random_weights(cfg, rng, low=low)


def make_engine(tmp_path, cfg, w, dtype, bs=16, blocks=24, max_seqs=4, eager=1):
    from nano_vllm_rs_b200.engine import LLMEngine
    from nano_vllm_rs_b200.loader import write_safetensors
    d = tmp_path / ("m_" + dtype)
    d.mkdir(exist_ok=True)
    (d / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(d / "model.safetensors"), {k: Z.to_bf16_bits(v) for k, v in w.items()})
    return LLMEngine.from_pretrained(str(d), dtype=dtype, kvcache_block_size=bs, num_kvcache_blocks=blocks, max_num_seqs=max_seqs,
                                     max_num_batched_tokens=blocks * bs, max_model_len=blocks * bs, enforce_eager=eager), str(d)


def replay(eng, requests, schedule):
    """schedule: list of steps, each a list of (request index, token count).  Returns every position's logits per request."""
    from nano_vllm_rs_b200.engine import SamplingParams
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    sid, at, out = {}, {}, {i: [] for i in range(len(requests))}
    for step in schedule:
        ids, counts = [], []
        for i, c in step:
            toks = requests[i][at.get(i, 0):at.get(i, 0) + c]
            if i in sid:
                eng.scheduler.extend_sequence(sid[i], toks)
            else:
                sid[i] = eng.scheduler.add_sequence(toks, sp)
            ids.append(sid[i]); counts.append(c)
        lg = eng.step_chunks(ids, counts, list(range(sum(counts))))
        k = 0
        for i, c in step:
            out[i].append(lg[k:k + c]); k += c
            at[i] = at.get(i, 0) + c
            if at[i] == len(requests[i]):
                eng.scheduler.finish_sequence(sid[i]); eng.scheduler.release_sequence(sid[i])
                del sid[i]
    return {i: np.concatenate(v) for i, v in out.items()}


def cut(n, sizes):
    out, k = [], 0
    while n > 0:
        c = min(n, sizes[k % len(sizes)]); out.append(c); n -= c; k += 1
    return out


def greedy(cfg, w, prompt, n_new):
    """The oracle's greedy continuation and the top-1 / top-2 margin of every step (relative to the row's spread)."""
    seq, out, margins, lg = Z.Sequence(cfg), [], [], None
    for t in prompt:
        lg = Z.token_step(cfg, w, seq, int(t))
    for _ in range(n_new):
        o = np.argsort(lg)
        out.append(int(o[-1])); margins.append((lg[o[-1]] - lg[o[-2]]) / lg.std())
        lg = Z.token_step(cfg, w, seq, out[-1])
    return out, margins


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", VARIANTS)
def test_engine_schedules_match_the_oracle(cuda, tmp_path, name, dtype):
    rng = np.random.default_rng(200 + VARIANTS.index(name))
    cfg = variant(name)
    w = weights_for(cfg, rng)
    lens = [1, 2, 37, 90, 33]
    reqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in lens]
    ref = [Z.run_sequence(cfg, w, r) for r in reqs]
    eng, _ = make_engine(tmp_path, cfg, w, dtype, bs=16, blocks=12)    # 192 slots: the requests only fit one after another

    def check(got, what):
        for i, r in enumerate(ref):
            e = rel_err(got[i], r)
            assert within(e, dtype), f"{name} {dtype} {what}: request {i} position {int(e.argmax())} error {e.max():.3g}"

    whole = replay(eng, reqs, [[(i, len(r))] for i, r in enumerate(reqs)])
    check(whole, "whole prompts")
    # most of the prompt at once, the last tokens one by one (the windows pass over decoded tokens and page borders)
    dec = replay(eng, reqs, [s for i, r in enumerate(reqs) for s in ([[(i, max(1, len(r) - 50))]] + [[(i, 1)]] * (len(r) - max(1, len(r) - 50)))])
    check(dec, "prefill + single tokens")
    one = replay(eng, reqs[:3], [[(i, 1)] for i, r in enumerate(reqs[:3]) for _ in r])
    for i in range(3):
        assert within(rel_err(one[i], ref[i]), dtype)
    # portions of changing size down to two tokens (shorter than the convolution's taps, across pages and window edges)
    por = replay(eng, reqs, [[(i, c)] for i, r in enumerate(reqs) for c in cut(len(r), [2, 5, 16, 3, 17, 2, 31])])
    check(por, "portions")
    for i in range(len(reqs)):  # a position must not depend on how the prompt was cut, beyond rounding
        assert rel_err(por[i], whole[i].astype(np.float64)).max() < (1e-4 if dtype == "float32" else 0.2)
        assert rel_err(dec[i], whole[i].astype(np.float64)).max() < (1e-4 if dtype == "float32" else 0.2)


@pytest.mark.parametrize("name", ["tensor_core", "all_kinds"])
def test_whole_prompts_of_latent_layers_unfolded(cuda, tmp_path, monkeypatch, name):
    """Long whole prompts (bf16): a latent-attention layer computes keys and values per head from the step's latents and runs
    as windowed attention over them; the folded form (forced by the switch, and always taken by portions and single tokens)
    gives the same logits to rounding, and both match the oracle.  Two prompts in one step, windows shorter than the prompts."""
    rng = np.random.default_rng(31)
    cfg = variant(name)
    w = weights_for(cfg, rng)
    reqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (300, 270)]
    ref = [Z.run_sequence(cfg, w, r) for r in reqs]
    eng, _ = make_engine(tmp_path, cfg, w, "bfloat16", bs=16, blocks=40)
    both = replay(eng, reqs, [[(0, 300), (1, 270)]])
    monkeypatch.setenv("NVLLM_LATENT_UNFOLD", "0")
    folded = replay(eng, reqs, [[(0, 300), (1, 270)]])
    monkeypatch.delenv("NVLLM_LATENT_UNFOLD")
    cut_up = replay(eng, reqs, [[(0, 150), (1, 270)], [(0, 150)]])       # request 0 continues from its cache: the folded form
    for i in range(2):
        assert within(rel_err(both[i], ref[i]), "bfloat16"), (i, rel_err(both[i], ref[i]).max())
        assert within(rel_err(folded[i], ref[i]), "bfloat16")
        assert rel_err(both[i], folded[i].astype(np.float64)).max() < 0.2 and rel_err(cut_up[i], both[i].astype(np.float64)).max() < 0.2
    if name == "tensor_core":
        assert not np.array_equal(both[0], folded[0])      # the two forms really are different code paths


def test_engine_layer_taps_match_the_oracle(cuda, tmp_path):
    """The residual stream after every layer, for a prompt: each mixer kind is checked where it sits, not only at the logits."""
    rng = np.random.default_rng(21)
    cfg = variant("all_kinds")
    w = weights_for(cfg, rng)
    toks = rng.integers(0, cfg["vocab"], 30).tolist()
    _, taps = Z.run_sequence(cfg, w, toks, layer_taps=True)
    eng, _ = make_engine(tmp_path, cfg, w, "float32")
    from nano_vllm_rs_b200.engine import SamplingParams
    tap = eng.model_runner.layer_tap(len(toks))
    sid = eng.scheduler.add_sequence(toks, SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))
    eng.step_chunks([sid], [len(toks)], [0])
    for i in range(len(cfg["layers"])):
        np.testing.assert_allclose(tap[i], taps[i], rtol=2e-4, atol=2e-4, err_msg="after layer %d" % i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_mixed_batches_reuse_pages_and_state_slots(cuda, tmp_path, dtype):
    """Up to four live requests per step, portions of some beside single tokens of others, in a pool that only holds them
    because finished requests give their pages and state slots back; every request equals its run alone and the oracle."""
    rng = np.random.default_rng(22)
    cfg = variant("all_kinds")
    w = weights_for(cfg, rng)
    lens = [50, 23, 64, 9, 41, 30, 17]
    reqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in lens]
    ref = [Z.run_sequence(cfg, w, r) for r in reqs]
    eng, _ = make_engine(tmp_path, cfg, w, dtype, bs=16, blocks=11, max_seqs=4)   # 176 slots < 234 tokens in total
    need = [(n + 15) // 16 for n in lens]
    at, live, nxt, sched, k = [0] * len(lens), [], 0, [], 0
    while nxt < len(reqs) or live:
        while nxt < len(reqs) and len(live) < 4 and sum(need[i] for i in live) + need[nxt] <= 11:
            live.append(nxt); nxt += 1
        step = []
        for i in live:
            k += 1
            if k % 5 == 0 and len(live) > 1:
                continue                                  # a live request may sit a step out
            c = 1 if (at[i] > lens[i] // 2 or k % 3 == 0) else [2, 7, 16, 5][k % 4]
            c = min(c, lens[i] - at[i])
            step.append((i, c)); at[i] += c
        if step:
            sched.append(step)
        live = [i for i in live if at[i] < lens[i]]
    assert any(len(s) == 4 for s in sched) and any(len({c for _, c in s}) > 1 for s in sched)
    mixed = replay(eng, reqs, sched)
    st = eng.scheduler.get_stats()
    assert st["free_blocks"] == st["total_blocks"] == 11
    alone = replay(eng, reqs, [[(i, len(r))] for i, r in enumerate(reqs)])
    for i, r in enumerate(ref):
        assert within(rel_err(mixed[i], r), dtype), (i, rel_err(mixed[i], r).max())
        assert rel_err(mixed[i], alone[i].astype(np.float64)).max() < (1e-4 if dtype == "float32" else 0.2)


def test_engine_long_decoding_over_many_pages(cuda, tmp_path):
    """300 tokens at once, then 80 one by one over 20+ pages with windows of 70 and 130: each window's far edge moves over
    page borders and over decoded tokens; the delta rule's state carries what the windows no longer see."""
    rng = np.random.default_rng(23)
    cfg = Z.make_config([("latent_attention", Z.latent_mixer(window=70), None), ("channel_delta", Z.delta_mixer(), None),
                         ("attention", Z.attention_mixer(window=130), Z.dense_mlp(16)),
                         ("latent_attention", Z.latent_mixer(heads=2, window=33, kv_from=0), None)])
    w = weights_for(cfg, rng)
    toks = rng.integers(0, cfg["vocab"], 380).tolist()
    ref = Z.run_sequence(cfg, w, toks)
    eng, _ = make_engine(tmp_path, cfg, w, "float32", bs=16, blocks=24, max_seqs=2)
    got = replay(eng, [toks], [[(0, 300)]] + [[(0, 1)]] * 80)
    assert rel_err(got[0], ref).max() < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(cuda, tmp_path, dtype):
    """LLMEngine.generate: the scheduler's own prefill / decode batches, decode steps replayed as CUDA graphs, pages taken
    while decoding, six prompts for four state slots (two wait until a slot is free)."""
    from nano_vllm_rs_b200.engine import SamplingParams
    rng = np.random.default_rng(24)
    cfg = variant("all_kinds")
    w = weights_for(cfg, rng)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (5, 1, 30, 16, 3, 20)]
    n_new = 40
    eng, _ = make_engine(tmp_path, cfg, w, dtype, bs=16, blocks=40, max_seqs=4, eager=0)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    margin_floor = 1e-3 if dtype == "float32" else 0.15
    agreed = 0
    for p, o in zip(prompts, outs):
        assert len(o) == n_new
        ref, margins = greedy(cfg, w, p, n_new)
        for j in range(n_new):
            if o[j] != ref[j]:
                assert margins[j] < margin_floor, (j, margins[j])   # a near-tie may fall either way; later tokens then differ
                break
            agreed += 1
    assert agreed > 0.6 * n_new * len(prompts)
    st = eng.scheduler.get_stats()
    assert st["decode_batches"] >= n_new - 1 and st["free_blocks"] == st["total_blocks"]


def test_generation_survives_preemption(cuda, tmp_path):
    """A cache pool too small for four growing sequences: the scheduler preempts (pages and state slot go back), later
    admits the victim again and recomputes it from position 0 into whatever slot is free; the tokens stay the oracle's."""
    from nano_vllm_rs_b200.engine import SamplingParams
    rng = np.random.default_rng(25)
    cfg = variant("all_kinds")
    w = weights_for(cfg, rng)
    prompts = [rng.integers(0, cfg["vocab"], 16).tolist() for _ in range(4)]
    n_new = 40
    eng, _ = make_engine(tmp_path, cfg, w, "float32", bs=16, blocks=11, max_seqs=4, eager=0)   # 4 x 56 tokens need 16 pages
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    st = eng.scheduler.get_stats()
    assert st["preemptions"] > 0 and st["free_blocks"] == st["total_blocks"]
    for p, o in zip(prompts, outs):
        ref, margins = greedy(cfg, w, p, n_new)
        for j in range(n_new):
            if o[j] != ref[j]:
                assert margins[j] < 1e-3, (j, margins[j])
                break


def test_synthetic_weights_and_command_line(cuda, tmp_path):
    """Seeded synthetic weights (no checkpoint) run a step; `python -m nano_vllm_rs_b200 generate` on a checkpoint gives the
    oracle's greedy tokens and, with a temperature, draws of the device sampler; the registry lists the architecture."""
    import sys
    from nano_vllm_rs_b200.engine import Config, LLMEngine, SamplingParams
    rng = np.random.default_rng(26)
    cfg = variant("tensor_core")
    eng = LLMEngine(Config(model_config=cfg, dtype="bfloat16", kvcache_block_size=16, num_kvcache_blocks=8, max_num_seqs=2,
                                     max_num_batched_tokens=128, max_model_len=128, enforce_eager=1), init_weights=True)
    sid = eng.scheduler.add_sequence(rng.integers(0, cfg["vocab"], 20).tolist(), SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))
    lg = eng.step_chunks([sid], [20], [19])
    assert np.isfinite(lg).all() and lg.std() > 0
    cfg = variant("all_kinds")
    w = weights_for(cfg, rng)
    _, model_dir = make_engine(tmp_path, cfg, w, "float32")
    prompt = rng.integers(0, cfg["vocab"], 9).tolist()
    run = lambda *extra: subprocess.run([sys.executable, "-m", "nano_vllm_rs_b200", "generate", "--model", model_dir, "--dtype", "float32", "--prompt-ids",
                                         ",".join(map(str, prompt)), "--max-tokens", "12", "--block-size", "16", *extra], cwd=ROOT, capture_output=True,
                                        text=True, timeout=600)
    r = run()
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])
    ref, margins = greedy(cfg, w, prompt, 12)
    for j in range(12):
        if out["completion_ids"][j] != ref[j]:
            assert margins[j] < 1e-3
            break
    r = run("--temperature", "1.5", "--top-k", "20")      # the device sampler draws from the same logits
    assert r.returncode == 0, r.stderr[-2000:]
    sampled = json.loads(r.stdout.strip().splitlines()[-1])["completion_ids"]
    assert len(sampled) == 12 and all(0 <= t < cfg["vocab"] for t in sampled) and sampled != ref
    r = subprocess.run([sys.executable, "-m", "nano_vllm_rs_b200", "architectures"], cwd=ROOT, capture_output=True, text=True, timeout=120)
    assert "Zudatar" in r.stdout


def test_trace_run_replays_a_schedule(cuda, tmp_path):
    rng = np.random.default_rng(27)
    cfg = variant("all_kinds")
    w = weights_for(cfg, rng)
    _, model_dir = make_engine(tmp_path, cfg, w, "float32")
    a, b = rng.integers(0, cfg["vocab"], 70).tolist(), rng.integers(0, cfg["vocab"], 9).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": [0, 39]}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[:8], "want": []}, {"id": "a", "tokens": a[40:69], "want": [28]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[69:], "want": [0]}, {"id": "b", "tokens": b[8:], "want": [0]}], "end": ["a", "b"]},
             {"step": 3, "entries": [{"id": "c", "tokens": b, "want": [8]}], "end": ["c"]}]
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "192"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    ra, rb = Z.run_sequence(cfg, w, a), Z.run_sequence(cfg, w, b)
    rd = lambda n: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
    for got, ref in ((rd(0), ra[[0, 39]]), (rd(1), ra[[68]]), (rd(2), np.stack([ra[69], rb[8]])), (rd(3), rb[[8]])):
        assert got.shape == ref.shape and rel_err(got, ref).max() < TOL["float32"]
