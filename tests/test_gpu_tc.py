"""GPU parity of the tensor-core (tcgen05) GEMM paths against the CPU oracle:
dense BF16 router logits, Q8 shared-expert products and the ragged grouped
MXFP4 expert products, including empty, single-row, ragged and multi-tile groups."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
if not torch.cuda.is_available():
    pytest.skip("no CUDA device", allow_module_level=True)

from moonshine_b200 import _native, ops, synth     # noqa: E402
from tests import gpu_util as G                    # noqa: E402


def status_ok():
    torch.cuda.synchronize()
    assert ops.k3_moe_device_status() == 0


@pytest.mark.parametrize("tokens,rows,cols", [(200, 300, 1024), (129, 896, 512), (32, 128, 2048)])
def test_dense_router_logits(oracle, tokens, rows, cols):
    w = synth.bf16_bits(synth.normal_f32(synth.stream_key(1, rows), rows * cols, 0.02))
    x = synth.bf16_bits(synth.normal_f32(synth.stream_key(2, tokens), tokens * cols, 1.0)).reshape(tokens, cols)
    layer = _native.LayerDesc(hidden=cols, expert_hidden=512, expert_count=rows if rows <= 1024 else 1024,
                              top_k=8, route_scale=1.0, local_expert_count=rows,
                              activation=1)
    bias = np.zeros(rows, np.float32)
    wd, bd = G.dev(w), G.dev(bias)
    layer.router_weight, layer.router_bias = wd.data_ptr(), bd.data_ptr()
    ids = G.empty((tokens, 8), np.uint32)
    wts = G.empty((tokens, 8), np.float32)
    logits = G.empty((tokens, rows), np.float32)
    assert ops.k3_moe_route(layer, ids, wts, logits, G.dev(x), tokens)
    status_ok()
    want = oracle.bf16_gemm(w, x, rows, cols)
    got = G.host(logits)
    # same exact products, different fp32 summation order
    assert np.max(np.abs(got - want)) <= 2e-6 * np.sqrt(cols) * np.max(np.abs(want)) + 1e-6


@pytest.mark.parametrize("block,st", [(32, synth.Q8_F16), (128, synth.Q8_F32)])
def test_q8_shared_products(oracle, block, st):
    tokens, d, s = 150, 1024, 512
    cfg = synth.baseline_config(hidden=d, expert_hidden=512, experts=8, top_k=2, shared_hidden=s,
                                q8_block=block, q8_scale_type=st)
    w = synth.make_layer(cfg, seed=9, experts=False)
    x = synth.activations(9, tokens, d)
    desc = _native.LayerDesc(hidden=d, expert_hidden=512, expert_count=8, top_k=2, shared_hidden=s,
                             q8_block=block, q8_scale_type=st, activation=cfg["activation"],
                             route_scale=1.0, local_expert_count=8)
    keep = {k: G.dev(w[k]) for k in w if k.startswith("shared")}
    for k, v in keep.items():
        setattr(desc, k, v.data_ptr())
    out = G.empty((tokens, d), np.uint16)
    g, u, a = (G.empty((tokens, s), np.uint16) for _ in range(3))
    assert ops.k3_moe_shared_expert(desc, out, g, u, a, G.dev(x), tokens)
    status_ok()
    sg = oracle.q8_gemm(w["shared_gate_q"], w["shared_gate_s"], x, s, d, block, st)
    su = oracle.q8_gemm(w["shared_up_q"], w["shared_up_s"], x, s, d, block, st)
    sa = oracle.activation(sg, su, cfg["activation"])
    so = oracle.q8_gemm(w["shared_down_q"], w["shared_down_s"], sa, d, s, block, st)
    # weights are rounded to bf16 before the tensor-core product: ~2^-9 per weight
    assert G.rel_l2(G.host(g, np.uint16), sg) <= 3e-3
    assert G.rel_l2(G.host(out, np.uint16), so) <= 5e-3


@pytest.mark.parametrize("counts", [
    [0, 5, 130, 128, 1, 300, 17, 64],
    [33, 0, 0, 0, 0, 0, 0, 0],
    [16, 16, 16, 16, 16, 16, 16, 16],
    [0, 0, 0, 700, 0, 0, 0, 1],
])
def test_grouped_expert_products(oracle, counts):
    d, i, e = 1024, 512, 8
    cfg = synth.baseline_config(hidden=d, expert_hidden=i, experts=e, top_k=2, shared_hidden=0)
    w = synth.make_layer(cfg, seed=21)
    rows = int(sum(counts))
    x = synth.activations(21, rows, d)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32)
    desc = _native.LayerDesc(hidden=d, expert_hidden=i, expert_count=e, top_k=2, shared_hidden=0,
                             activation=cfg["activation"], route_scale=1.0, local_expert_count=e)
    keep = {k: G.dev(w[k]) for k in w if k.startswith("w")}
    for k, v in keep.items():
        setattr(desc, k, v.data_ptr())
    out = G.empty((rows, d), np.uint16)
    act = G.empty((rows, i), np.uint16)
    assert ops.k3_moe_experts_grouped(desc, out, act, G.dev(x), G.dev(offsets), rows)
    status_ok()
    got_act, got_out = G.host(act, np.uint16), G.host(out, np.uint16)
    for ex in range(e):
        lo, hi = int(offsets[ex]), int(offsets[ex + 1])
        if lo == hi:
            continue
        xe = x[lo:hi]
        gate = oracle.mxfp4_gemm(w["w1_packed"][ex], w["w1_scales"][ex], xe, i, d)
        up = oracle.mxfp4_gemm(w["w3_packed"][ex], w["w3_scales"][ex], xe, i, d)
        a = oracle.activation(gate, up, cfg["activation"])
        assert G.rel_l2(got_act[lo:hi], a) <= 4e-3, ex
        # down product checked on the kernel's own activations: reference envelope
        down = oracle.mxfp4_gemm(w["w2_packed"][ex], w["w2_scales"][ex], got_act[lo:hi], d, i)
        ref = oracle.mxfp4_gemm_f64(w["w2_packed"][ex], w["w2_scales"][ex], got_act[lo:hi], d, i)
        G.check_mxfp4_envelope(got_out[lo:hi], down, ref)


@pytest.mark.parametrize("counts,gathered", [
    ([0, 5, 130, 128, 1, 300, 17, 64], False),
    ([0, 5, 130, 128, 1, 300, 17, 64], True),
    ([33, 0, 0, 0, 0, 0, 0, 0], True),
    ([0, 0, 0, 700, 0, 0, 0, 1], False),
    ([144, 145, 143, 0, 16, 129, 272, 273], False),         # around the 128 + 16 row tile limit
])
def test_grouped_expert_products_block_scaled(oracle, counts, gathered):
    """Block-scaled tensor-core path (packed E2M1 weights and E8M0 scales consumed
    as they are, rows as two E4M3 terms): gate/up/activation and down against the
    oracle, with and without the fused row gather."""
    d, i, e = 1024, 512, 8
    cfg = synth.baseline_config(hidden=d, expert_hidden=i, experts=e, top_k=2, shared_hidden=0)
    w = synth.make_layer(cfg, seed=23)
    rows = int(sum(counts))
    x = synth.activations(23, rows, d)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32)
    desc = _native.LayerDesc(hidden=d, expert_hidden=i, expert_count=e, top_k=2, shared_hidden=0,
                             activation=cfg["activation"], route_scale=1.0, local_expert_count=e)
    keep = {k: G.dev(w[k]) for k in w if k.startswith("w")}
    for k, v in keep.items():
        setattr(desc, k, v.data_ptr())
    out = G.empty((rows, d), np.uint16)
    act = G.empty((rows, i), np.uint16)
    need = ops.k3_moe_experts_workspace_bytes(desc, rows, rows if gathered else 0)
    assert need > 0
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    if gathered:
        perm = np.random.default_rng(5).permutation(rows).astype(np.uint32)
        index = np.argsort(perm).astype(np.uint32)          # x[perm][index] == x
        ok = ops.k3_moe_experts_grouped_ws(desc, out, act, G.dev(np.ascontiguousarray(x[perm])),
                                           G.dev(index), rows, G.dev(offsets), rows, ws, need)
    else:
        ok = ops.k3_moe_experts_grouped_ws(desc, out, act, G.dev(x), None, 0, G.dev(offsets), rows,
                                           ws, need)
    assert ok
    status_ok()
    got_act, got_out = G.host(act, np.uint16), G.host(out, np.uint16)
    for ex in range(e):
        lo, hi = int(offsets[ex]), int(offsets[ex + 1])
        if lo == hi:
            continue
        xe = x[lo:hi]
        gate = oracle.mxfp4_gemm(w["w1_packed"][ex], w["w1_scales"][ex], xe, i, d)
        up = oracle.mxfp4_gemm(w["w3_packed"][ex], w["w3_scales"][ex], xe, i, d)
        a = oracle.activation(gate, up, cfg["activation"])
        # gate and up are rounded to bf16 before the activation on both sides; a last-bit
        # difference there moves the activation by one bf16 step
        assert G.rel_l2(got_act[lo:hi], a) <= 1e-3, ex
        down = oracle.mxfp4_gemm(w["w2_packed"][ex], w["w2_scales"][ex], got_act[lo:hi], d, i)
        ref = oracle.mxfp4_gemm_f64(w["w2_packed"][ex], w["w2_scales"][ex], got_act[lo:hi], d, i)
        G.check_mxfp4_envelope(got_out[lo:hi], down, ref)


def test_block_scaled_workspace_rules():
    """Too-small or missing scratch falls back to the bf16 tensor-core path when that
    is possible (no gather, act given) and fails otherwise."""
    d, i, e = 1024, 512, 4
    cfg = synth.baseline_config(hidden=d, expert_hidden=i, experts=e, top_k=2, shared_hidden=0)
    w = synth.make_layer(cfg, seed=3)
    rows = 64
    x = synth.activations(3, rows, d)
    offsets = np.array([0, 16, 16, 40, 64], np.uint32)
    desc = _native.LayerDesc(hidden=d, expert_hidden=i, expert_count=e, top_k=2, shared_hidden=0,
                             activation=cfg["activation"], route_scale=1.0, local_expert_count=e)
    keep = {k: G.dev(w[k]) for k in w if k.startswith("w")}
    for k, v in keep.items():
        setattr(desc, k, v.data_ptr())
    out, out2 = G.empty((rows, d), np.uint16), G.empty((rows, d), np.uint16)
    act, act2 = G.empty((rows, i), np.uint16), G.empty((rows, i), np.uint16)
    xd, od = G.dev(x), G.dev(offsets)
    index = G.dev(np.arange(rows, dtype=np.uint32))
    assert ops.k3_moe_experts_grouped_ws(desc, out, act, xd, None, 0, od, rows, None, 0)
    assert ops.k3_moe_experts_grouped(desc, out2, act2, xd, od, rows)
    status_ok()
    assert np.array_equal(G.host(out, np.uint16), G.host(out2, np.uint16))
    assert not ops.k3_moe_experts_grouped_ws(desc, out, act, xd, index, rows, od, rows, None, 0)
    assert not ops.k3_moe_experts_grouped_ws(desc, out, None, xd, None, 0, od, rows, None, 0)
    assert ops.k3_moe_experts_workspace_bytes(desc, 8, 0) == 0        # too few rows for the path
