"""Pins of the CPU oracle against the reference's own model-free tests.

The reference stores no output vectors for the MoE path; its tests pin
tolerances, tie rules and reduction schedules against in-file host loops driven
by xorshift32 streams.  Each test here rebuilds that input recipe (same seed,
same draw order up to the op under test) and applies the reference's bound, and
additionally checks the oracle against an independent numpy restatement.
"""
import numpy as np
import pytest

SEED_COMPONENTS = 0x4B334B33          # tests/test_k3_rocm_components.cu:30


def f32(a):
    return np.asarray(a, np.float32)


def components_stream(oracle):
    """Replays tests/test_k3_rocm_components.cu up to each op, in main()'s order
    (:598-616): SiTU, AttnRes, MXFP4 GEMV, dense/router/reductions."""
    rng = oracle.XorShift(SEED_COMPONENTS)
    out = {}
    # test_situ (:59-62): gate, up interleaved
    gu = rng.unit(2 * 8192)
    sym = lambda u, s: ((u * f32(2.0)) - f32(1.0)) * f32(s)
    out["situ_gate"] = oracle.bf16_from_f32(sym(gu[0::2], 12.0))
    out["situ_up"] = oracle.bf16_from_f32(sym(gu[1::2], 50.0))
    # test_attn_res (:132-142): prefix, blocks, then norm/qk interleaved
    rng.unit(17 * 7168)
    rng.unit(17 * 10 * 7168)
    rng.unit(2 * 7168)
    # test_mxfp4_gemv (:277-286)
    rows, cols = 128, 512
    out["mx_packed"] = (rng.unit(rows * cols // 2) * f32(256.0)).astype(np.uint8)
    out["mx_scales"] = (122 + (rng.unit(rows * cols // 32) * f32(11.0)).astype(np.uint32)).astype(np.uint8)
    out["mx_input"] = oracle.bf16_from_f32(sym(rng.unit(cols), 1.0))
    # test_dense_router_and_reductions (:355-360, 418-421, 494-505)
    out["dense_w"] = oracle.bf16_from_f32(sym(rng.unit(rows * cols), 0.25))
    out["dense_x"] = oracle.bf16_from_f32(sym(rng.unit(cols), 0.5))
    lb = rng.unit(2 * 896)
    out["logits"] = sym(lb[0::2], 4.0)
    out["bias"] = sym(lb[1::2], 0.15)
    out["values"] = oracle.bf16_from_f32(sym(rng.unit(16 * cols), 1.0))
    w = rng.unit(16)
    total = f32(0.0)
    for v in w:
        total = f32(total + v)
    out["vector_weights"] = (w / total).astype(np.float32)
    out["norm_weight"] = oracle.bf16_from_f32(f32(1.0) + sym(rng.unit(cols), 0.1))
    return out


@pytest.fixture(scope="module")
def stream(oracle):
    return components_stream(oracle)


def test_bf16_rounding_matches_scalar(oracle):
    rng = np.random.default_rng(1)
    a = rng.standard_normal(4096).astype(np.float32) * np.float32(3.0)
    a[:4] = [0.0, -0.0, np.inf, 1.00390625]      # tie case rounds to even
    vec = oracle.bf16_from_f32(a)
    lib = oracle.lib()
    for i in range(a.size):
        assert vec[i] == lib.k3o_bf16_from_float(float(a[i]))
    assert np.array_equal(oracle.bf16_to_f32(vec[:2]), [0.0, -0.0])


def test_situ_bound(oracle, stream):
    # tests/test_k3_rocm_components.cu:79-90: <= 0.0625 against the test's formula
    g = oracle.bf16_to_f32(stream["situ_gate"]).astype(np.float64)
    u = oracle.bf16_to_f32(stream["situ_up"]).astype(np.float64)
    want = (4.0 * np.tanh(g / 4.0) / (1.0 + np.exp(-g))) * (25.0 * np.tanh(u / 25.0))
    want = oracle.bf16_to_f32(oracle.bf16_from_f32(want.astype(np.float32)))
    got = oracle.bf16_to_f32(oracle.activation(stream["situ_gate"], stream["situ_up"],
                                               oracle.ACT_SITU, 4.0, 25.0))
    assert np.max(np.abs(got - want)) <= 0.0625


def test_swiglu_is_situ_limit(oracle):
    rng = np.random.default_rng(2)
    g = oracle.bf16_from_f32(rng.standard_normal(2048).astype(np.float32))
    u = oracle.bf16_from_f32(rng.standard_normal(2048).astype(np.float32))
    a = oracle.bf16_to_f32(oracle.activation(g, u, oracle.ACT_SWIGLU))
    b = oracle.bf16_to_f32(oracle.activation(g, u, oracle.ACT_SITU, 1e6, 1e6))
    assert np.max(np.abs(a - b)) <= 2 ** -6


def test_mxfp4_gemv_128x512_bound(oracle, stream):
    # tests/test_k3_rocm_components.cu:306-324: <= 0.015625 vs a sequential fp32 sum
    rows, cols = 128, 512
    p, s, x = stream["mx_packed"], stream["mx_scales"], stream["mx_input"]
    lut = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float32)
    nib = np.empty((rows, cols), np.uint8)
    pr = p.reshape(rows, cols // 2)
    nib[:, 0::2] = pr & 0xF
    nib[:, 1::2] = pr >> 4
    scale = (s.reshape(rows, cols // 32).astype(np.uint32) << 23).view(np.float32)
    w = lut[nib] * np.repeat(scale, 32, axis=1)
    xf = oracle.bf16_to_f32(x)
    expected = np.zeros(rows, np.float32)
    for c in range(cols):
        expected = (expected + w[:, c] * xf[c]).astype(np.float32)
    expected = oracle.bf16_to_f32(oracle.bf16_from_f32(expected))
    for fn in (oracle.mxfp4_gemm, oracle.mxfp4_gemm_kernel_order):
        got = oracle.bf16_to_f32(fn(p, s, x, rows, cols))[0]
        assert np.max(np.abs(got - expected)) <= 0.015625


def test_bf16_gemv_lane_schedule_exact(oracle, stream):
    # tests/test_k3_rocm_components.cu:383-411: exact against the 256-lane emulation
    rows, cols = 128, 512
    w = oracle.bf16_to_f32(stream["dense_w"]).reshape(rows, cols)
    x = oracle.bf16_to_f32(stream["dense_x"])
    partial = np.zeros((rows, 256), np.float32)
    for j in range(cols // 256):
        partial = (partial + w[:, 256 * j:256 * (j + 1)] * x[256 * j:256 * (j + 1)]).astype(np.float32)
    width = 128
    while width:
        partial[:, :width] = partial[:, :width] + partial[:, width:2 * width]
        width //= 2
    f32_out, bf16_out = oracle.bf16_gemm(stream["dense_w"], stream["dense_x"], rows, cols, want_bf16=True)
    assert np.array_equal(f32_out[0], partial[:, 0])
    assert np.array_equal(bf16_out[0], oracle.bf16_from_f32(partial[:, 0]))


def numpy_router(logits, bias, top_k, scale):
    raw = (np.float32(1.0) / (np.float32(1.0) + np.exp(-logits.astype(np.float32)))).astype(np.float32)
    choice = (raw + bias).astype(np.float32)
    order = np.lexsort((np.arange(choice.size), -choice.astype(np.float64)))[:top_k]
    den = np.float32(1e-20)
    for i in order:
        den = np.float32(den + raw[i])
    return order.astype(np.uint32), (raw[order] / den * np.float32(scale)).astype(np.float32)


def test_router_ids_and_weights(oracle, stream):
    # tests/test_k3_rocm_components.cu:443-482: ids exact, weights <= 1e-6
    ids, w = oracle.router_topk(stream["logits"], stream["bias"], 16, 1.0)
    want_ids, want_w = numpy_router(stream["logits"], stream["bias"], 16, 1.0)
    assert np.array_equal(ids[0], want_ids)
    assert np.max(np.abs(w[0] - want_w)) <= 1e-6
    assert abs(float(w[0].sum()) - 1.0) < 1e-5


def test_router_tie_break_lowest_id(oracle):
    logits = np.zeros((1, 64), np.float32)
    bias = np.zeros(64, np.float32)
    logits[0, [40, 7, 23]] = 3.0            # three exact ties at the top
    ids, w = oracle.router_topk(logits, bias, 8, 2.5)
    assert list(ids[0][:3]) == [7, 23, 40]
    assert list(ids[0][3:]) == [0, 1, 2, 3, 4]       # remaining ties: ascending id
    assert abs(float(w[0].sum()) - 2.5) < 1e-5


def test_weighted_sum_norm_add(oracle, stream):
    # tests/test_k3_rocm_components.cu:544-567
    cols = 512
    v = oracle.bf16_to_f32(stream["values"]).reshape(16, cols).astype(np.float64)
    w = stream["vector_weights"].astype(np.float64)
    exact = (w[:, None] * v).sum(0)
    got = oracle.weighted_sum(stream["values"], stream["vector_weights"], 1, 16, cols)
    gotf = oracle.bf16_to_f32(got[0])
    assert np.max(np.abs(gotf - exact)) <= np.max(np.abs(exact)) * 2 ** -8
    norm = oracle.rms_norm(got, stream["norm_weight"], cols, 1e-5)
    x = gotf.astype(np.float64)
    want = x / np.sqrt((x * x).mean() + 1e-5) * oracle.bf16_to_f32(stream["norm_weight"])
    assert np.max(np.abs(oracle.bf16_to_f32(norm[0]) - want)) <= 0.0078125 + 2 ** -7
    added = oracle.add(got, norm)
    want_add = oracle.bf16_from_f32(gotf + oracle.bf16_to_f32(norm[0]))
    assert np.array_equal(added[0], want_add)


def bf16_ulp_distance(a, b):
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, 0x8000 - (x & 0x7FFF), 0x8000 + x)
    return np.abs(key(a) - key(b))


@pytest.mark.parametrize("cols", [3584, 3072])
def test_mxfp4_envelope(oracle, cols):
    # tests/test_k3_mxfp4_envelope.cu:255-343: two schedules within 1 bf16 ULP of each
    # other and within (0.25 abs or 1 % rel) of the fp64 dot product
    rows, vectors = 256, 6
    rng = np.random.default_rng(cols)
    p = rng.integers(0, 256, rows * cols // 2, dtype=np.uint8)
    s = rng.integers(118, 130, rows * cols // 32, dtype=np.uint8)
    x = oracle.bf16_from_f32((rng.standard_normal((vectors, cols)) * 0.5).astype(np.float32))
    a = oracle.mxfp4_gemm(p, s, x, rows, cols)
    b = oracle.mxfp4_gemm_kernel_order(p, s, x, rows, cols)
    ref = oracle.mxfp4_gemm_f64(p, s, x, rows, cols)
    assert bf16_ulp_distance(a, b).max() <= 1
    for got in (a, b):
        g = oracle.bf16_to_f32(got).astype(np.float64)
        err = np.abs(g - ref)
        assert np.all((err <= 0.25) | (err / np.maximum(np.abs(ref), 1e-3) <= 0.01))


def test_e8m0_edge_codes(oracle):
    lib = oracle.lib()
    import ctypes as C
    lib.k3o_e8m0_to_float.restype = C.c_float
    lib.k3o_e8m0_to_float.argtypes = [C.c_uint8]
    assert lib.k3o_e8m0_to_float(127) == 1.0
    assert lib.k3o_e8m0_to_float(0) == 2.0 ** -127
    assert lib.k3o_e8m0_to_float(1) == 2.0 ** -126
    assert lib.k3o_e8m0_to_float(254) == 2.0 ** 127


def test_q8_quantize_and_gemv(oracle):
    # kernel k3_rocm_ops.cu:663-697 and host oracle tests/test_k3_q8_projection.cu:50-76;
    # gates of that test: NRMSE < 0.02, cosine > 0.999 against the BF16 product
    rows, cols = 96, 1024
    rng = np.random.default_rng(5)
    w = oracle.bf16_from_f32((rng.standard_normal((rows, cols)) * 0.02).astype(np.float32))
    w[3, 128:256] = 0                                     # all-zero block -> scale 1.0
    x = oracle.bf16_from_f32(((rng.random(cols) * 2 - 1) * 0.125).astype(np.float32))
    q, s = oracle.q8_quantize(w, rows, cols, 128, oracle.Q8_F32)
    assert s[3, 1] == 1.0 and np.all(q[3, 128:256] == 0)
    wf = oracle.bf16_to_f32(w).reshape(rows, cols)
    blocks = np.abs(wf).reshape(rows, cols // 128, 128).max(-1)
    want_s = np.where(blocks > 0, (blocks / np.float32(127.0)).astype(np.float32), np.float32(1.0))
    assert np.array_equal(s, want_s)
    assert np.abs(q).max() <= 127
    got = oracle.bf16_to_f32(oracle.q8_gemm(q, s, x, rows, cols))[0].astype(np.float64)
    ref = oracle.bf16_gemm(w, x, rows, cols)[0].astype(np.float64)
    deq = (q.astype(np.float64) * np.repeat(s.astype(np.float64), 128, axis=1)) @ oracle.bf16_to_f32(x)
    assert np.max(np.abs(got - deq)) <= 0.0009765625 + np.max(np.abs(deq)) * 2 ** -8
    nrmse = np.sqrt(((got - ref) ** 2).sum() / (ref ** 2).sum())
    cosine = (got * ref).sum() / np.sqrt((got ** 2).sum() * (ref ** 2).sum())
    assert nrmse < 0.02 and cosine > 0.999


def test_q8_block32_f16_scales(oracle):
    rows, cols = 32, 256
    rng = np.random.default_rng(6)
    q = rng.integers(-127, 128, (rows, cols), dtype=np.int8)
    s = (1e-4 + rng.random((rows, cols // 32)) * 9e-4).astype(np.float16)
    x = oracle.bf16_from_f32(rng.standard_normal((3, cols)).astype(np.float32))
    got = oracle.bf16_to_f32(oracle.q8_gemm(q, s, x, rows, cols, 32, oracle.Q8_F16)).astype(np.float64)
    deq = q.astype(np.float64) * np.repeat(s.astype(np.float64), 32, axis=1)
    ref = oracle.bf16_to_f32(x).astype(np.float64) @ deq.T
    assert np.max(np.abs(got - ref)) <= np.max(np.abs(ref)) * 2 ** -7


def test_group_routes_matches_reference_scan(oracle):
    # literal restatement of k3_engine_prefill.inc:1175-1194 (one scan per expert)
    rng = np.random.default_rng(7)
    tokens, top_k, experts = 37, 4, 11
    ids = np.stack([rng.choice(experts, top_k, replace=False) for _ in range(tokens)]).astype(np.uint32)
    offsets, toks, slots = oracle.group_routes(ids, experts)
    want_t, want_s, want_o = [], [], [0]
    for e in range(experts):
        for t in range(tokens):
            for r in range(top_k):
                if ids[t, r] == e:
                    want_t.append(t)
                    want_s.append(t * top_k + r)
        want_o.append(len(want_t))
    assert list(offsets) == want_o and list(toks) == want_t and list(slots) == want_s


def test_group_routes_empty_experts(oracle):
    ids = np.array([[5, 2]], np.uint32)
    offsets, toks, slots = oracle.group_routes(ids, 8)
    assert list(offsets) == [0, 0, 0, 1, 1, 1, 2, 2, 2]
    assert list(slots) == [1, 0]
