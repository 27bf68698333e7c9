"""Seeded synthetic tensors for the routed-MoE layer.

Real Kimi-K3 weights are not available to the tests or the benchmark, so every
tensor is drawn from a counter-based 64-bit hash: element ``i`` of stream
``tag`` under ``seed`` depends on nothing else.  The same integer recipe is
implemented by the ``k3_synth_*`` fill kernels of the native library, so a
tensor generated on the host with numpy and one filled on the device are
bit-identical (checked by the GPU tests).  Floating-point draws (the normal
activations and router weights) are only ever produced here, on the host.

Distributions follow the benchmark description: activations bf16 ~N(0,1);
router weight bf16 ~N(0,0.02); router bias f32 ~U(-0.1,0.1); MXFP4 codes uniform
over the 16 E2M1 values with E8M0 exponent bytes uniform in a range; shared
expert int8 uniform in [-127,127] with per-block scales ~U(1e-4,1e-3).
"""
from __future__ import annotations

import numpy as np

ACT_SITU, ACT_SWIGLU = 0, 1
Q8_F32, Q8_F16 = 0, 1

# stream tags (one per tensor kind)
TAG_X, TAG_ROUTER_W, TAG_ROUTER_B = 1, 2, 3
TAG_W1P, TAG_W1S, TAG_W3P, TAG_W3S, TAG_W2P, TAG_W2S = 10, 11, 12, 13, 14, 15
TAG_SGQ, TAG_SGS, TAG_SUQ, TAG_SUS, TAG_SDQ, TAG_SDS = 20, 21, 22, 23, 24, 25
TAG_PERM = 30

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)
_GOLD = 0x9E3779B97F4A7C15


def stream_key(seed: int, tag: int) -> int:
    """64-bit key of a (seed, tag) stream; passed unchanged to the device fills."""
    return ((int(seed) & 0xFFFFFFFF) << 32 | (int(tag) & 0xFFFFFFFF)) & 0xFFFFFFFFFFFFFFFF


def hash64(key: int, index: np.ndarray) -> np.ndarray:
    """splitmix64 finaliser of (key * golden + index + golden)."""
    with np.errstate(over="ignore"):
        base = np.uint64((int(key) * _GOLD + _GOLD) & 0xFFFFFFFFFFFFFFFF)
        z = index.astype(np.uint64) + base
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return z


def raw_bytes(key: int, count: int, first: int = 0) -> np.ndarray:
    """``count`` hash bytes starting at byte offset ``first`` (multiple of 8):
    byte j of 8-byte chunk c is bits [8j, 8j+8) of hash64(key, c)."""
    assert first % 8 == 0
    chunks = (count + 7) // 8
    z = hash64(key, np.arange(first // 8, first // 8 + chunks, dtype=np.uint64))
    return z.astype("<u8").view(np.uint8)[:count]


def bytes_uniform(key: int, count: int, low: int = 0, span: int = 256, first: int = 0) -> np.ndarray:
    """Bytes in [low, low+span): low + floor(b*span/256)."""
    b = raw_bytes(key, count, first).astype(np.uint32)
    return (low + ((b * span) >> 8)).astype(np.uint8)


def int8_uniform(key: int, count: int, first: int = 0) -> np.ndarray:
    """int8 in [-127,127]."""
    b = raw_bytes(key, count, first).astype(np.int32)
    return (((b * 255) >> 8) - 127).astype(np.int8)


def unit24(key: int, count: int, first: int = 0) -> np.ndarray:
    """float32 in [0,1) with 24 random bits: top 24 bits of hash64(key, i)."""
    z = hash64(key, np.arange(first, first + count, dtype=np.uint64))
    return (z >> np.uint64(40)).astype(np.float32) * np.float32(2.0 ** -24)


def uniform_f32(key: int, count: int, low: float, high: float, first: int = 0) -> np.ndarray:
    """low + u*(high-low), one rounding per operation in float32."""
    u = unit24(key, count, first)
    return (u * np.float32(high - low)).astype(np.float32) + np.float32(low)


def normal_f32(key: int, count: int, sigma: float) -> np.ndarray:
    """Box-Muller on two 24-bit uniforms per pair (host only)."""
    pairs = (count + 1) // 2
    z = hash64(key, np.arange(pairs, dtype=np.uint64))
    u1 = ((z >> np.uint64(40)).astype(np.float64) + 1.0) * 2.0 ** -24      # (0,1]
    u2 = ((z >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.float64) * 2.0 ** -24
    r = np.sqrt(-2.0 * np.log(u1))
    out = np.empty(pairs * 2, np.float64)
    out[0::2] = r * np.cos(2.0 * np.pi * u2)
    out[1::2] = r * np.sin(2.0 * np.pi * u2)
    return (out[:count] * sigma).astype(np.float32)


def bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round-to-nearest-even."""
    bits = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    nan = (bits & 0x7FFFFFFF) > 0x7F800000
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) >> 16
    return np.where(nan, (bits >> 16) | 0x40, rounded).astype(np.uint16)


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(a, np.uint16).astype(np.uint32) << 16).view(np.float32)


def baseline_config(**overrides) -> dict:
    """The benchmark's synthetic layer: d=7168, 896 experts, top-16, I=2048,
    SwiGLU, route scale 2.5, shared expert I=2048 with int8 + fp16 scale per 32."""
    cfg = dict(hidden=7168, expert_hidden=2048, experts=896, top_k=16, shared_hidden=2048,
               q8_block=32, q8_scale_type=Q8_F16, activation=ACT_SWIGLU, beta=4.0,
               linear_beta=25.0, route_scale=2.5, scale_low=119, scale_span=5,
               bias_mode="uniform", duplicate_router_rows=0)
    cfg.update(overrides)
    return cfg


def tiny_config(**overrides) -> dict:
    """A shape small enough for the CPU oracle to finish in milliseconds."""
    cfg = baseline_config(hidden=512, expert_hidden=256, experts=32, top_k=4, shared_hidden=256)
    cfg.update(overrides)
    return cfg


def activations(seed: int, tokens: int, hidden: int) -> np.ndarray:
    return bf16_bits(normal_f32(stream_key(seed, TAG_X), tokens * hidden, 1.0)).reshape(tokens, hidden)


def router_bias(cfg: dict, seed: int) -> np.ndarray:
    e = cfg["experts"]
    key = stream_key(seed, TAG_ROUTER_B)
    mode = cfg.get("bias_mode", "uniform")
    if mode == "uniform":
        bias = uniform_f32(key, e, -0.1, 0.1)
    elif mode == "zipf":
        # popularity rank drawn by sorting hash values; bias = 0.3 * rank^-1.1 - 0.05
        order = np.argsort(hash64(stream_key(seed, TAG_PERM), np.arange(e, dtype=np.uint64)),
                           kind="stable")
        rank = np.empty(e, np.int64)
        rank[order] = np.arange(1, e + 1)
        bias = (0.3 * rank.astype(np.float64) ** -1.1 - 0.05).astype(np.float32)
    elif mode == "hot4":
        # four experts always selected (a token can pick an expert once, so four
        # experts take 4/top_k of all assignments), the rest uniform
        bias = uniform_f32(key, e, -0.1, 0.1)
        order = np.argsort(hash64(stream_key(seed, TAG_PERM), np.arange(e, dtype=np.uint64)),
                           kind="stable")
        bias[order[:4]] = np.float32(2.0)
    else:
        raise ValueError(mode)
    return np.ascontiguousarray(bias, np.float32)


def make_layer(cfg: dict, seed: int = 0, experts: bool = True) -> dict:
    """All tensors of one layer as numpy arrays (host).  With ``experts=False``
    the expert tensors are omitted (they are then filled on the device)."""
    d, i, e, s = cfg["hidden"], cfg["expert_hidden"], cfg["experts"], cfg["shared_hidden"]
    w = {"config": dict(cfg)}
    rw = normal_f32(stream_key(seed, TAG_ROUTER_W), e * d, 0.02).reshape(e, d)
    rb = router_bias(cfg, seed)
    dup = int(cfg.get("duplicate_router_rows", 0))
    for j in range(dup):            # exact score ties: rows 2j and 2j+1 identical
        rw[2 * j + 1] = rw[2 * j]
        rb[2 * j + 1] = rb[2 * j]
    w["router_weight"] = bf16_bits(rw).reshape(e, d)
    w["router_bias"] = rb
    if experts:
        for name, (tp, ts, rows, cols) in expert_tensor_specs(cfg).items():
            w[name + "_packed"] = bytes_uniform(stream_key(seed, tp), e * rows * cols // 2).reshape(e, rows, cols // 2)
            w[name + "_scales"] = bytes_uniform(stream_key(seed, ts), e * rows * cols // 32,
                                                cfg["scale_low"], cfg["scale_span"]).reshape(e, rows, cols // 32)
    if s:
        blk = cfg["q8_block"]
        sdt = np.float16 if cfg["q8_scale_type"] == Q8_F16 else np.float32
        for name, (tq, tsc, rows, cols) in shared_tensor_specs(cfg).items():
            w[name + "_q"] = int8_uniform(stream_key(seed, tq), rows * cols).reshape(rows, cols)
            w[name + "_s"] = uniform_f32(stream_key(seed, tsc), rows * cols // blk, 1e-4, 1e-3
                                         ).astype(sdt).reshape(rows, cols // blk)
    return w


def expert_tensor_specs(cfg: dict) -> dict:
    d, i = cfg["hidden"], cfg["expert_hidden"]
    return {"w1": (TAG_W1P, TAG_W1S, i, d), "w3": (TAG_W3P, TAG_W3S, i, d),
            "w2": (TAG_W2P, TAG_W2S, d, i)}


def shared_tensor_specs(cfg: dict) -> dict:
    d, s = cfg["hidden"], cfg["shared_hidden"]
    return {"shared_gate": (TAG_SGQ, TAG_SGS, s, d), "shared_up": (TAG_SUQ, TAG_SUS, s, d),
            "shared_down": (TAG_SDQ, TAG_SDS, d, s)}


def decode_bytes_per_token(cfg: dict) -> int:
    """Algorithmic HBM bytes of one 1-token layer pass (every weight byte the
    token touches once, plus the vectors in and out)."""
    d, i, e, k, s = cfg["hidden"], cfg["expert_hidden"], cfg["experts"], cfg["top_k"], cfg["shared_hidden"]
    per_expert = 2 * i * (d // 2 + d // 32) + d * (i // 2 + i // 32)
    scale_bytes = 2 if cfg["q8_scale_type"] == Q8_F16 else 4
    shared = 3 * s * d + 3 * s * d // cfg["q8_block"] * scale_bytes if s else 0
    return e * d * 2 + e * 4 + d * 2 + k * per_expert + shared + d * 2


def prefill_flops_per_token(cfg: dict) -> dict:
    d, i, e, k, s = cfg["hidden"], cfg["expert_hidden"], cfg["experts"], cfg["top_k"], cfg["shared_hidden"]
    return {"routed": k * (2 * 2 * i * d + 2 * d * i), "shared": 3 * 2 * s * d, "router": 2 * e * d}
