"""Seeded inputs of the golden cases (shared by the generator and the tests).
Only the *outputs* are stored in the .npz files; inputs are regenerated from
their seeds through moonshine_b200.synth."""
import numpy as np

from moonshine_b200 import synth

MID = dict(hidden=1024, expert_hidden=512, experts=64, top_k=8, shared_hidden=512)
# the reference's real layer shape family: SiTU, Q8-128 with f32 scales, scale 1.0
REF_STYLE = dict(hidden=768, expert_hidden=384, experts=48, top_k=6, shared_hidden=768,
                 q8_block=128, q8_scale_type=synth.Q8_F32, activation=synth.ACT_SITU,
                 route_scale=1.0)

LAYER_CASES = {
    # name: (config overrides on tiny_config/baseline, seed, tokens)
    "tiny_t1": (synth.tiny_config(), 11, 1),
    "tiny_t37": (synth.tiny_config(), 12, 37),
    "tiny_ties_t16": (synth.tiny_config(duplicate_router_rows=4), 13, 16),
    "mid_t64": (synth.baseline_config(**MID), 14, 64),
    "mid_hot4_t128": (synth.baseline_config(**MID, bias_mode="hot4"), 15, 128),
    "mid_extreme_scales_t9": (synth.baseline_config(**MID, scale_low=0, scale_span=128), 16, 9),
    "refstyle_t5": (synth.baseline_config(**REF_STYLE), 17, 5),
}


def layer_inputs(name):
    cfg, seed, tokens = LAYER_CASES[name]
    weights = synth.make_layer(cfg, seed)
    x = synth.activations(seed, tokens, cfg["hidden"])
    return cfg, weights, x


def op_inputs():
    """Inputs of the per-operator golden cases."""
    k = lambda tag: synth.stream_key(77, tag)
    d = {}
    for name, rows, cols, n in (("mx_a", 64, 256, 3), ("mx_b", 40, 3584, 2), ("mx_c", 33, 96, 5)):
        d[name] = dict(rows=rows, cols=cols,
                       packed=synth.bytes_uniform(k(100 + rows), rows * cols // 2),
                       scales=synth.bytes_uniform(k(200 + rows), rows * cols // 32, 119, 9),
                       x=synth.bf16_bits(synth.normal_f32(k(300 + rows), n * cols, 1.0)).reshape(n, cols))
    d["dense"] = dict(rows=48, cols=512,
                      w=synth.bf16_bits(synth.normal_f32(k(401), 48 * 512, 0.05)),
                      x=synth.bf16_bits(synth.normal_f32(k(402), 3 * 512, 1.0)).reshape(3, 512))
    d["dense_odd"] = dict(rows=9, cols=301,
                          w=synth.bf16_bits(synth.normal_f32(k(403), 9 * 301, 0.05)),
                          x=synth.bf16_bits(synth.normal_f32(k(404), 2 * 301, 1.0)).reshape(2, 301))
    d["q8_128"] = dict(rows=24, cols=1024, block=128, st=synth.Q8_F32,
                       q=synth.int8_uniform(k(501), 24 * 1024).reshape(24, 1024),
                       s=synth.uniform_f32(k(502), 24 * 8, 1e-4, 1e-3).reshape(24, 8),
                       x=synth.bf16_bits(synth.normal_f32(k(503), 2 * 1024, 1.0)).reshape(2, 1024))
    d["q8_32"] = dict(rows=20, cols=2304, block=32, st=synth.Q8_F16,
                      q=synth.int8_uniform(k(511), 20 * 2304).reshape(20, 2304),
                      s=synth.uniform_f32(k(512), 20 * 72, 1e-4, 1e-3).astype(np.float16).reshape(20, 72),
                      x=synth.bf16_bits(synth.normal_f32(k(513), 3 * 2304, 1.0)).reshape(3, 2304))
    logits = synth.normal_f32(k(601), 12 * 896, 1.7).reshape(12, 896)
    bias = synth.uniform_f32(k(602), 896, -0.1, 0.1)
    logits[3, 100:140] = logits[3, 100]          # rows with exact score ties
    bias[100:140] = bias[100]
    logits[7, :] = 0.25
    d["router"] = dict(logits=logits, bias=bias, top_k=16, scale=2.5)
    d["router_small"] = dict(logits=synth.normal_f32(k(603), 5 * 40, 2.0).reshape(5, 40),
                             bias=synth.uniform_f32(k(604), 40, -0.2, 0.2), top_k=32, scale=1.0)
    d["wsum"] = dict(tokens=3, count=16, hidden=520,
                     v=synth.bf16_bits(synth.normal_f32(k(701), 3 * 16 * 520, 1.0)),
                     w=synth.uniform_f32(k(702), 48, 0.0, 0.2).reshape(3, 16))
    d["norm"] = dict(hidden=3584, x=synth.bf16_bits(synth.normal_f32(k(801), 2 * 3584, 2.0)).reshape(2, 3584),
                     w=synth.bf16_bits(1.0 + synth.normal_f32(k(802), 3584, 0.1)))
    d["act"] = dict(g=synth.bf16_bits(synth.normal_f32(k(901), 4099, 4.0)),
                    u=synth.bf16_bits(synth.normal_f32(k(902), 4099, 10.0)))
    return d
