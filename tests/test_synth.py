"""Seeded synthetic tensors: determinism, distributions and the algorithmic
byte / flop counts the roofline figures are built on."""
import numpy as np

from moonshine_b200 import synth


def test_hash_streams_are_independent_of_length_and_offset():
    key = synth.stream_key(0, synth.TAG_W1P)
    a = synth.bytes_uniform(key, 4096)
    b = synth.bytes_uniform(key, 1024, first=2048)
    assert np.array_equal(a[2048:3072], b)
    assert not np.array_equal(a, synth.bytes_uniform(synth.stream_key(1, synth.TAG_W1P), 4096))


def test_distributions():
    key = synth.stream_key(3, 99)
    s = synth.bytes_uniform(key, 1 << 16, 119, 5)
    assert s.min() == 119 and s.max() == 123
    q = synth.int8_uniform(key, 1 << 16)
    assert q.min() == -127 and q.max() == 127
    u = synth.uniform_f32(key, 1 << 16, 1e-4, 1e-3)
    assert u.min() >= 1e-4 and u.max() < 1e-3 + 1e-9
    n = synth.normal_f32(key, 1 << 18, 0.02)
    assert abs(n.mean()) < 2e-4 and abs(n.std() - 0.02) < 2e-4


def test_baseline_counts():
    cfg = synth.baseline_config()
    # router 12,845,056 + bias 3,584 + x 14,336 + 16 x 23,396,352 + shared 46,792,704 + out 14,336
    assert synth.decode_bytes_per_token(cfg) == 434_011_648
    flops = synth.prefill_flops_per_token(cfg)
    assert flops == {"routed": 1_409_286_144, "shared": 88_080_384, "router": 12_845_056}


def test_layer_shapes_and_ties():
    cfg = synth.tiny_config(duplicate_router_rows=2)
    w = synth.make_layer(cfg, seed=4)
    e, d, i = cfg["experts"], cfg["hidden"], cfg["expert_hidden"]
    assert w["router_weight"].shape == (e, d) and w["w2_packed"].shape == (e, d, i // 2)
    assert w["w1_scales"].shape == (e, i, d // 32) and w["shared_down_s"].dtype == np.float16
    assert np.array_equal(w["router_weight"][0], w["router_weight"][1])
    assert w["router_bias"][2] == w["router_bias"][3]


def test_bias_modes():
    cfg = synth.baseline_config(bias_mode="zipf")
    b = synth.router_bias(cfg, 0)
    assert b.max() == np.float32(0.3 - 0.05) and (b > 0).sum() < 40
    hot = synth.router_bias(synth.baseline_config(bias_mode="hot4"), 0)
    assert (hot == 2.0).sum() == 4
