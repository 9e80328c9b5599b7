"""CPU tests around the Zasorax integration: properties of the oracle's mechanisms that hold by construction (so that the
yardstick itself is pinned), the model registry's configuration reader, and the scheduler's pages for this design."""
import json
import math

import numpy as np
import pytest

from oracle import zasorax as Z


def small_cfg(**kw):
    return Z.make_config([("attention_2", Z.rotary_mixer(), Z.dense_mlp(10)), ("attention", Z.chunk_mixer(), Z.expert_mlp()),
                          ("attention", Z.chunk_mixer(heads=2, kv_heads=2, kv_from=1), None), ("attention_2", Z.rotary_mixer(heads=2, kv_heads=1), Z.expert_mlp(top=1))],
                         **kw)


# ------------------------------------------------------------------------------------------------ oracle properties


def test_distance_buckets():
    """One row per distance below half the table; above it the rows grow logarithmically and the last one is reached at `far`."""
    rows, far = 16, 200
    b = [Z.distance_bucket(n, rows, far) for n in range(400)]
    assert b[:8] == list(range(8)) and b[8] == 8
    assert all(x <= y for x, y in zip(b, b[1:])) and max(b) == rows - 1
    assert b[far] == rows - 1 and b.index(rows - 1) == math.ceil(8 * (far / 8) ** (7 / 8))   # the last row starts 7/8 of the way (in logs)
    assert b.index(9) == math.ceil(8 * (far / 8) ** (1 / 8))
    # powers of two land exactly on a row's first distance: half = 4, far = 64 -> rows start at 4, 8, 16, 32
    assert [Z.distance_bucket(n, 8, 64) for n in (3, 4, 7, 8, 15, 16, 31, 32, 63, 64, 1000)] == [3, 4, 4, 5, 5, 6, 6, 7, 7, 7, 7]


def test_rotation_pairs_halves_and_depends_on_distance_only():
    rng = np.random.default_rng(1)
    q, k = rng.standard_normal(10), rng.standard_normal(10)
    d = lambda pq, pk: Z.rotate_halves(q, pq, 6, 300.0) @ Z.rotate_halves(k, pk, 6, 300.0)
    assert abs(d(17, 5) - d(112, 100)) < 1e-9 and abs(d(17, 5) - d(17, 6)) > 1e-6
    assert np.allclose(Z.rotate_halves(q, 9, 6, 300.0)[6:], q[6:]) and np.allclose(Z.rotate_halves(q, 0, 6, 300.0), q)
    r = Z.rotate_halves(q, 3, 6, 300.0)                      # value 0 pairs with value 3 and turns by the position itself
    np.testing.assert_allclose([r[0], r[3]], [q[0] * np.cos(3.0) - q[3] * np.sin(3.0), q[3] * np.cos(3.0) + q[0] * np.sin(3.0)])
    a = 3.0 * 300.0 ** (-2.0 / 6)                            # the second pair (1, 4) turns by position * base^(-2/dims)
    np.testing.assert_allclose(r[1], q[1] * np.cos(a) - q[4] * np.sin(a))


def test_rotated_values_enter_by_their_distance():
    """A value stored rotated by j and read through a rotation by -i is the value rotated by j - i."""
    rng = np.random.default_rng(2)
    v = rng.standard_normal(8)
    a = Z.rotate_halves(Z.rotate_halves(v, 41, 8, 50.0), -47, 8, 50.0)
    np.testing.assert_allclose(a, Z.rotate_halves(v, -6, 8, 50.0), atol=1e-12)
    np.testing.assert_allclose(Z.rotate_halves(Z.rotate_halves(v, 9, 8, 50.0), -9, 8, 50.0), v, atol=1e-12)


def test_sink_takes_mass_but_gives_nothing():
    s = np.array([0.3, -1.0, 2.0])
    p = Z.sink_softmax(s, 1.0)
    np.testing.assert_allclose(p.sum(), 1.0 - np.exp(1.0) / (np.exp(s).sum() + np.exp(1.0)))
    np.testing.assert_allclose(Z.sink_softmax(s, 0.0), np.exp(s) / (1.0 + np.exp(s).sum()))     # a sink of score 0: 1 + sum in the denominator
    np.testing.assert_allclose(Z.sink_softmax(s, -1e9).sum(), 1.0)


def test_xielu_branches_meet_and_follow_their_formulas():
    p, q = 0.3, -0.7
    sp = lambda t: math.log1p(math.exp(t))
    np.testing.assert_allclose(Z.xielu(np.array([2.0]), p, q), [sp(p) * 4.0 + 1.0])
    np.testing.assert_allclose(Z.xielu(np.array([-1.5]), p, q), [(0.5 + sp(q)) * (math.exp(-1.5) + 0.5) - 0.75])
    assert abs(Z.xielu(np.array([1e-9]), p, q)[0] - Z.xielu(np.array([-1e-9]), p, q)[0]) < 1e-8 and Z.xielu(np.array([0.0]), p, q)[0] == 0.0


def test_router_picks_the_largest_and_normalises_over_them_alone():
    z = np.array([0.1, 2.0, -1.0, 2.0, 0.5])
    idx, w = Z.route(z, 3)
    assert idx == [1, 3, 4]                                   # ties: the lower index first
    e = np.exp(z[idx])
    np.testing.assert_allclose(w, e / e.sum())
    assert Z.route(z, 1)[1].tolist() == [1.0]


def test_chunks_forget_what_lies_before_them_and_sharing_reads_the_source_layer():
    rng = np.random.default_rng(3)
    cfg = Z.make_config([("attention", Z.chunk_mixer(chunk=5), None), ("attention", Z.chunk_mixer(chunk=3, kv_from=0), Z.dense_mlp(8))])
    w = Z.random_weights(cfg, rng)
    toks = rng.integers(0, cfg["vocab"], 12).tolist()
    base = Z.run_sequence(cfg, w, toks)
    other = list(toks); other[3] = (other[3] + 1) % cfg["vocab"]          # position 3 is in chunk 0 of both layers
    got = Z.run_sequence(cfg, w, other)
    assert np.abs(got[3] - base[3]).max() > 1e-6 and np.abs(got[4] - base[4]).max() > 1e-6
    assert np.abs(got[5] - base[5]).max() > 1e-6                          # layer 1's chunk 3..5 still holds the changed token
    assert np.abs(got[6:] - base[6:]).max() < 1e-12                       # 5 starts a new chunk of layer 0, and 6 one of layer 1
    assert "l1.mix.k" not in w and "l1.mix.v" not in w and "l1.mix.k.norm" not in w and "l1.mix.q.norm" in w
    w2 = dict(w); w2["l0.mix.v"] = w["l0.mix.v"] * 2.0                     # layer 1 reads layer 0's values
    assert np.abs(Z.run_sequence(cfg, w2, toks)[0] - base[0]).max() > 1e-6


# ------------------------------------------------------------------------------------------------ registry, scheduler


def test_model_registry_reads_config_json():
    from nano_vllm_rs_b200.engine import Config, lib
    assert b"Zasorax" in lib().nvllm_registered_architectures()
    c = Config(model_config=json.dumps(small_cfg(vocab=77, width=24)))
    assert (c.arch, c.vocab_size, c.hidden_size, c.num_hidden_layers) == ("Zasorax", 77, 24, 4)
    assert c.recurrent_state == 0                        # attention only: nothing but pages is held per sequence


@pytest.mark.parametrize("breakage,needle", [
    (lambda c: c["layers"][0].update(type="attention_3"), "attention_3"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), "rot dims"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=7), "rotated in pairs"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=0), "layer 0"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "layer 2"),
    (lambda c: c["layers"][2]["mixer"].update(dim=7), "same kv_heads / dim / vdim"),
    (lambda c: c["layers"][1]["mixer"].pop("bias_max"), "bias_max"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "sparse"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
])
def test_bad_model_configs_are_refused_with_a_reason(breakage, needle):
    from nano_vllm_rs_b200 import _ffi
    from nano_vllm_rs_b200.engine import Config
    cfg = small_cfg()
    breakage(cfg)
    with pytest.raises(_ffi.NvllmError) as e:
        Config(model_config=json.dumps(cfg))
    assert needle in str(e.value)


def test_portion_steps_take_pages_as_they_go_and_return_them():
    from nano_vllm_rs_b200.engine import Config, SamplingParams, Scheduler
    cfg = Config(model_config=json.dumps(small_cfg()), kvcache_block_size=16, num_kvcache_blocks=4, max_num_seqs=3,
                 max_num_batched_tokens=64, max_model_len=64)
    s = Scheduler(cfg)
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    a, b = s.add_sequence(list(range(20)), sp), s.add_sequence(list(range(30)), sp)
    s.schedule_chunks([a, b], [17, 2]); s.commit_chunks()           # 2 pages + 1 page
    s.schedule_chunks([a, b], [3, 28]); s.commit_chunks()           # a stays at 2, b grows to 2: the pool is full
    s.finish_sequence(a); s.release_sequence(a)
    c = s.add_sequence(list(range(32)), sp)
    batch = s.schedule_chunks([c], [32])                              # exactly the two pages a gave back
    assert len(set((np.asarray(batch.slot_mapping) // 16).tolist())) == 2
