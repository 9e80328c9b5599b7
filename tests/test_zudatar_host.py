"""CPU tests around the Zudatar integration: properties of the oracle's mechanisms that hold by construction (so that the
yardstick itself is pinned), the model registry's configuration reader, and the scheduler's state slots for this design."""
import json

import numpy as np
import pytest

from oracle import zudatar as Z


def small_cfg(**kw):
    return Z.make_config([("channel_delta", Z.delta_mixer(), None), ("latent_attention", Z.latent_mixer(), Z.dense_mlp(10)),
                          ("attention", Z.attention_mixer(), Z.dense_mlp(12)), ("latent_attention", Z.latent_mixer(heads=2, kv_from=1), None)], **kw)


# ------------------------------------------------------------------------------------------------ oracle properties


def test_delta_rule_equals_its_explicit_form():
    """With beta = 1 and no decay one step stores v under k exactly (S^T k = v afterwards for a unit k); with decay g the
    older content of every key channel shrinks by g before the write; the read-out sees the token's own write."""
    rng = np.random.default_rng(0)
    D, V = 6, 4
    S = rng.standard_normal((D, V))
    k = rng.standard_normal(D); k /= np.linalg.norm(k)
    q, v = rng.standard_normal(D), rng.standard_normal(V)
    S1, o = Z.delta_rule_step(S, q, k, v, 1.0, np.ones(D))
    np.testing.assert_allclose(S1.T @ k, v, atol=1e-12)
    np.testing.assert_allclose(o, S1.T @ q, atol=1e-12)
    g = rng.uniform(0.2, 0.9, D)
    S2, _ = Z.delta_rule_step(S, q, k, v, 0.3, g)
    Sd = g[:, None] * S
    np.testing.assert_allclose(S2, Sd + np.outer(k, 0.3 * (v - Sd.T @ k)), atol=1e-12)
    S3, o3 = Z.delta_rule_step(S, q, k, v, 0.0, g)            # beta = 0: nothing is written, only the decay acts
    np.testing.assert_allclose(S3, Sd, atol=1e-12)


def test_rotation_pairs_neighbours_and_depends_on_distance_only():
    rng = np.random.default_rng(1)
    q, k = rng.standard_normal(10), rng.standard_normal(10)
    d = lambda pq, pk: Z.rotate_pairs(q, pq, 6, 300.0) @ Z.rotate_pairs(k, pk, 6, 300.0)
    assert abs(d(17, 5) - d(112, 100)) < 1e-9 and abs(d(17, 5) - d(17, 6)) > 1e-6
    assert np.allclose(Z.rotate_pairs(q, 9, 6, 300.0)[6:], q[6:]) and np.allclose(Z.rotate_pairs(q, 0, 6, 300.0), q)
    r = Z.rotate_pairs(q, 3, 6, 300.0)                       # dimension 0 pairs with dimension 1
    np.testing.assert_allclose([r[0], r[1]], [q[0] * np.cos(3.0) - q[1] * np.sin(3.0), q[1] * np.cos(3.0) + q[0] * np.sin(3.0)])
    a = 3.0 * 300.0 ** (-2.0 / 6)                            # the second pair turns by position * base^(-2/dims)
    np.testing.assert_allclose(r[2], q[2] * np.cos(a) - q[3] * np.sin(a))


def test_sink_takes_mass_but_gives_nothing():
    s = np.array([0.3, -1.0, 2.0])
    p = Z.window_softmax(s, sink=1.0)
    np.testing.assert_allclose(p.sum(), 1.0 - np.exp(1.0) / (np.exp(s).sum() + np.exp(1.0)))
    np.testing.assert_allclose(Z.window_softmax(s).sum(), 1.0)
    np.testing.assert_allclose(Z.window_softmax(s, sink=-1e9), Z.window_softmax(s))


def test_bigram_rows():
    bg = {"buckets": 17, "mul_prev": 13, "mul_cur": 5}
    assert Z.bigram_row(None, 5, bg) == 17 and Z.bigram_row(0, 0, bg) == 0 and Z.bigram_row(3, 4, bg) == (39 + 20) % 17


def test_windows_forget_and_the_delta_state_remembers():
    """A change of token 0 cannot reach position 30 through attention layers whose windows are shorter — unless a delta
    layer carries it; and the layer that reads another layer's latents sees exactly that layer's window content."""
    rng = np.random.default_rng(2)
    att_only = Z.make_config([("latent_attention", Z.latent_mixer(window=4), None), ("attention", Z.attention_mixer(window=5), Z.dense_mlp(8)),
                              ("latent_attention", Z.latent_mixer(heads=2, window=3, kv_from=0), None)])
    w = Z.random_weights(att_only, rng)
    a = rng.integers(0, 80, 31).tolist()
    b = list(a); b[0] = (a[0] + 1) % 80
    la, lb = Z.run_sequence(att_only, w, a, [5, 30]), Z.run_sequence(att_only, w, b, [5, 30])
    assert np.abs(la[0] - lb[0]).max() > 1e-6          # within reach: 3 layers x windows cover position 5
    assert np.abs(la[1] - lb[1]).max() < 1e-12         # out of reach of (4 - 1) + (5 - 1) + (3 - 1) positions and the bigram's one
    with_delta = Z.make_config([("channel_delta", Z.delta_mixer(), None)] + [(l["type"], l["mixer"], l["mlp"]) for l in att_only["layers"][1:2]])
    w = Z.random_weights(with_delta, rng)
    la, lb = Z.run_sequence(with_delta, w, a, [30]), Z.run_sequence(with_delta, w, b, [30])
    assert np.abs(la - lb).max() > 1e-9


def test_latent_sharing_uses_the_source_layers_latents():
    cfg = small_cfg()
    seq = Z.Sequence(cfg)
    assert seq.layers[3] is seq.layers[1]
    shapes = Z.tensor_shapes(cfg)
    assert "l3.mix.dkv" not in shapes and "l1.mix.dkv" in shapes and shapes["l3.mix.uk"] == (2 * 6, 12)


def test_short_convolution_sees_taps_tokens_and_zeros_before_the_start():
    w = np.array([[1.0, 10.0, 100.0]])
    hist = np.zeros((2, 1))
    ys = []
    for x in (1.0, 2.0, 3.0, 4.0):
        y, hist = Z.short_conv(w, hist, np.array([x]))
        ys.append(y[0])
    assert ys == [100.0, 210.0, 321.0, 432.0]           # the last column is the current token's


# ------------------------------------------------------------------------------------------------ registry / configuration


def test_model_registry_reads_config_json():
    from nano_vllm_rs_b200.engine import Config, lib
    assert b"Zudatar" in lib().nvllm_registered_architectures()
    c = Config(model_config=json.dumps(small_cfg(vocab=77, width=24)))
    assert (c.arch, c.vocab_size, c.hidden_size, c.num_hidden_layers) == ("Zudatar", 77, 24, 4)
    assert c.recurrent_state == 1                        # the token before the next one is per-sequence state in every model


@pytest.mark.parametrize("breakage,needle", [
    (lambda c: c["layers"][0].update(type="windowed"), "windowed"),
    (lambda c: c["layers"][2]["mixer"].update(kv_heads=3), "attention"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=9), "values are the keys"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=3), "attention"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "latents of layer 2"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "latents of layer 3"),
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=5), "same kv_rank"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "delta rule"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "sparse"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "bigram"),
])
def test_bad_model_configs_are_refused_with_a_reason(breakage, needle):
    from nano_vllm_rs_b200 import _ffi
    from nano_vllm_rs_b200.engine import Config
    cfg = small_cfg()
    breakage(cfg)
    with pytest.raises(_ffi.NvllmError) as e:
        Config(model_config=json.dumps(cfg))
    assert needle in str(e.value)


def test_portion_steps_give_each_sequence_a_state_slot():
    from nano_vllm_rs_b200.engine import Config, SamplingParams, Scheduler
    cfg = Config(model_config=json.dumps(small_cfg()), kvcache_block_size=16, num_kvcache_blocks=8, max_num_seqs=3,
                 max_num_batched_tokens=64, max_model_len=128)
    s = Scheduler(cfg)
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    ids = [s.add_sequence(list(range(5)), sp) for _ in range(3)]
    b = s.schedule_chunks(ids, [2, 5, 1])
    assert sorted(b.state_slots.tolist()) == [0, 1, 2]
    s.commit_chunks()
    s.finish_sequence(ids[1]); s.release_sequence(ids[1])
    nid = s.add_sequence(list(range(7)), sp)
    b = s.schedule_chunks([nid], [7])
    assert b.state_slots.tolist() == [1]                  # the freed slot goes to the next sequence
