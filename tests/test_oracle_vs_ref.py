"""The CPU oracle against the reference's own code, bit for bit.

The reference keeps CPU restatements of its MoE operators inside its test
programs.  ``make -C oracle ref_host REF=<tree>`` cuts them out of the reference
tree and compiles them unchanged (``oracle/ref_host_wrap.cpp``).  Two checks:

* everywhere: the oracle must reproduce the outputs RECORDED from those
  functions (``tests/golden/ref_host.npz``, written by
  ``tests/golden/make_ref_host_golden.py``) on inputs regenerated from their seeds;
* where the compiled functions are present (``oracle/_ref``): the same
  comparison live, on further seeds, plus the recorded file against a fresh run.
"""
import os

import numpy as np
import pytest

from oracle import ref_host
from tests.golden import ref_host_cases as cases

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_host.npz")


@pytest.fixture(scope="module")
def recorded():
    return np.load(GOLDEN)


def same_bits(got, want, what):
    got, want = np.ascontiguousarray(got), np.ascontiguousarray(want)
    assert got.dtype == want.dtype and got.shape == want.shape, (what, got.dtype, want.dtype, got.shape, want.shape)
    differing = int((got.view(np.uint8) != want.view(np.uint8)).sum())
    assert differing == 0, f"{what}: {differing} bytes differ from the reference's host function"


def test_bf16_conversion_and_decode_tables(oracle, recorded):
    values = cases.bf16_values()
    same_bits(oracle.bf16_from_f32(values), recorded["bf16_round"], "float -> bf16")
    scalar = np.array([oracle.lib().k3o_bf16_from_float(float(v)) for v in values[:64]], np.uint16)
    same_bits(scalar, recorded["bf16_round"][:64], "float -> bf16 (scalar entry)")
    lib = oracle.lib()
    import ctypes as C
    lib.k3o_e8m0_to_float.restype = C.c_float
    lib.k3o_e2m1_to_float.restype = C.c_float
    e8 = np.array([lib.k3o_e8m0_to_float(C.c_uint8(b)) for b in range(256)], np.float32)
    e2 = np.array([lib.k3o_e2m1_to_float(C.c_uint8(n)) for n in range(16)], np.float32)
    same_bits(e8, recorded["e8m0"], "E8M0 decode table")
    same_bits(e2, recorded["e2m1"], "E2M1 decode table")


@pytest.mark.parametrize("name,case,rows,columns,sigma", [("router", 1, cases.REF_EXPERTS, 7168, 0.02),
                                                           ("small", 2, 128, 512, 0.25)])
def test_bf16_gemv(oracle, recorded, name, case, rows, columns, sigma):
    w = cases.bf16_matrix(case, rows, columns, sigma)
    x = cases.activations(case, columns)
    f32, b16 = oracle.bf16_gemm(w, x, rows, columns, want_bf16=True)
    same_bits(f32.ravel(), recorded[f"bf16_gemv_{name}_f32"], "BF16 GEMV f32")
    same_bits(b16.ravel(), recorded[f"bf16_gemv_{name}_bf16"], "BF16 GEMV bf16")


MX_CASES = [("gate_real", 3, 512, cases.REF_LATENT, 119, 5), ("down_bench", 4, 512, 2048, 119, 5),
            ("gate_bench_extreme", 5, 256, 7168, 0, 128), ("small", 6, 128, 512, 122, 11)]


@pytest.mark.parametrize("name,case,rows,columns,low,span", MX_CASES)
def test_mxfp4_gemv(oracle, recorded, name, case, rows, columns, low, span):
    p, s = cases.mxfp4_matrix(case, rows, columns, low, span)
    x = cases.activations(case, columns)
    same_bits(oracle.mxfp4_gemm(p, s, x, rows, columns).ravel(), recorded[f"mxfp4_gemv_{name}"], "MXFP4 GEMV")
    if f"mxfp4_f64_{name}" in recorded:
        x4 = cases.activations(case, 4 * columns).reshape(4, columns)
        same_bits(oracle.mxfp4_gemm_f64(p[:64], s[:64], x4, 64, columns), recorded[f"mxfp4_f64_{name}"],
                  "MXFP4 fp64 envelope sum")


def test_situ(oracle, recorded):
    g, u = cases.activations(7, 1 << 16, 4.0), cases.activations(8, 1 << 16, 20.0)
    same_bits(oracle.activation(g, u, oracle.ACT_SITU_HOST), recorded["situ"], "SiTU (host expression)")
    # the kernel's expression (reciprocal then product) may round differently: one ULP, rarely
    kernel_form = oracle.activation(g, u, oracle.ACT_SITU).astype(np.int32)
    distance = np.abs(kernel_form - recorded["situ"].astype(np.int32))
    assert distance.max() <= 1 and (distance != 0).mean() < 1e-4


@pytest.mark.parametrize("name,case,count", [("latent", 9, cases.REF_LATENT), ("hidden", 10, 7168)])
def test_rms_norm(oracle, recorded, name, case, count):
    x = cases.activations(case, count, 2.0)
    w = cases.bf16_matrix(case, 1, count, 0.5).ravel()
    same_bits(oracle.rms_norm(x, w, count, 1e-5).ravel(), recorded[f"rms_norm_{name}"], "RMSNorm")


def test_router(oracle, recorded):
    logits, bias, tied_bias = cases.router_rows(11, 32)
    for parity, b in ((0, bias), (1, tied_bias)):
        ids, weights = oracle.router_topk(logits[parity::2], b, cases.REF_TOP_K, 1.0)
        same_bits(ids, recorded["router_ids"][parity::2], "router ids")
        same_bits(weights, recorded["router_weights"][parity::2], "router weights")
    # the tied rows really hold ties among the selected experts' candidates
    ids = recorded["router_ids"][1::2]
    assert any(np.any((row[:-1] % 2 == 0) & (row[1:] == row[:-1] + 1) & (row[:-1] < 80)) for row in ids)


def test_q8_row(oracle, recorded):
    q, s = cases.q8_rows(12, 64)
    x = cases.activations(12, cases.REF_Q8_COLUMNS)
    got = oracle.q8_gemm(q, s, x, 64, cases.REF_Q8_COLUMNS, 128, oracle.Q8_F32)
    same_bits(got.ravel(), recorded["q8_rows"], "Q8-128 row")


def test_expert_composition_and_weighted_accumulate(oracle, recorded):
    """One token, three experts at the reference's real shape: gate, up, SiTU, down per
    expert (tests/test_k3_moe_smoke.cu:601-609), the weighted accumulation in rank order
    and the final rounding (:610-618)."""
    L, I = cases.REF_LATENT, cases.REF_EXPERT_HIDDEN
    latent = cases.activations(13, L)
    rows = []
    for rank in range(3):
        w1p, w1s, w2p, w2s, w3p, w3s = cases.expert_span(13, rank)
        gate = oracle.mxfp4_gemm(w1p, w1s, latent, I, L)
        up = oracle.mxfp4_gemm(w3p, w3s, latent, I, L)
        act = oracle.activation(gate, up, oracle.ACT_SITU_HOST)
        rows.append(oracle.mxfp4_gemm(w2p, w2s, act, L, I).ravel())
    rows = np.stack(rows)
    same_bits(rows, recorded["expert_rows"], "expert output rows")
    route_weights = np.array([0.41, 0.33, 0.26], np.float32)
    routed = oracle.weighted_sum(rows, route_weights, 1, 3, L)
    same_bits(routed.ravel(), recorded["expert_routed"], "weighted accumulation, rounded")
    # the f32 accumulator depends on multiply-add fusion and the recorded file says so;
    # the oracle follows the fused build, like the reference's own flags
    assert set(recorded["fusion_dependent"].tolist()) <= {"expert_accumulator", "expert_routed"}


@pytest.mark.skipif(not ref_host.available(), reason="reference host functions not compiled on this machine")
def test_recorded_file_matches_a_fresh_run():
    from tests.golden import make_ref_host_golden as gen
    fresh = gen.record(True)
    stored = np.load(GOLDEN)
    for name, value in fresh.items():
        same_bits(stored[name], value, "recorded " + name)


@pytest.mark.skipif(not ref_host.available(), reason="reference host functions not compiled on this machine")
@pytest.mark.parametrize("seed", [101, 102, 103])
def test_live_against_reference_functions(oracle, seed):
    """Further seeds, straight against the compiled reference functions."""
    rows, columns = 96, 1536
    w = cases.bf16_matrix(seed, rows, columns, 0.1)
    x = cases.activations(seed, columns)
    f32, b16 = ref_host.bf16_gemv(w, x, rows, columns)
    o32, o16 = oracle.bf16_gemm(w, x, rows, columns, want_bf16=True)
    same_bits(o32.ravel(), f32, "BF16 GEMV f32")
    same_bits(o16.ravel(), b16, "BF16 GEMV bf16")
    p, s = cases.mxfp4_matrix(seed, rows, columns, 100, 28)
    same_bits(oracle.mxfp4_gemm(p, s, x, rows, columns).ravel(), ref_host.mxfp4_gemv(p, s, x, rows, columns),
              "MXFP4 GEMV")
    same_bits(oracle.mxfp4_gemm_f64(p, s, x, rows, columns), ref_host.mxfp4_f64(p, s, x, rows, columns),
              "MXFP4 fp64")
    g, u = cases.activations(seed + 50, 20000, 6.0), cases.activations(seed + 60, 20000, 30.0)
    same_bits(oracle.activation(g, u, oracle.ACT_SITU_HOST), ref_host.situ(g, u), "SiTU")
    n = cases.activations(seed + 70, columns, 3.0)
    nw = cases.bf16_matrix(seed + 70, 1, columns, 1.0).ravel()
    same_bits(oracle.rms_norm(n, nw, columns, 1e-5).ravel(), ref_host.rms_norm(n, nw, 1e-5), "RMSNorm")
    logits, bias, tied = cases.router_rows(seed, 8)
    for r in range(8):
        b = tied if r % 2 else bias
        ids, weights = ref_host.router(logits[r], b)
        oi, ow = oracle.router_topk(logits[r:r + 1], b, cases.REF_TOP_K, 1.0)
        same_bits(oi.ravel(), ids, "router ids")
        same_bits(ow.ravel(), weights, "router weights")
    q, sc = cases.q8_rows(seed, 8)
    xq = cases.activations(seed, cases.REF_Q8_COLUMNS)
    want = np.array([ref_host.q8_row(q[r], sc[r], xq) for r in range(8)], np.uint16)
    same_bits(oracle.q8_gemm(q, sc, xq, 8, cases.REF_Q8_COLUMNS, 128, oracle.Q8_F32).ravel(), want, "Q8 row")
