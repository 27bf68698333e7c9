"""Status words, bounded waits, the static-weight wrappers, the phase ledger and
graph replay of the one-token layer, through the C-ABI."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
if not torch.cuda.is_available():
    pytest.skip("no CUDA device", allow_module_level=True)

from moonshine_b200 import _native, ops, synth      # noqa: E402
from moonshine_b200.layer import MoELayer, bf16_tensor_to_bits   # noqa: E402
from tests import gpu_util as G                      # noqa: E402
from tests.golden import cases                       # noqa: E402


def test_dispatch_reports_an_out_of_range_expert_id():
    """An id >= experts is skipped by the placement; the status word says so in both
    dispatch entry points, and clearing it brings the status back to 0."""
    assert ops.k3_moe_device_status_clear()
    tokens, top_k, experts = 64, 4, 32
    ids = synth.hash64(7, np.arange(tokens * top_k, dtype=np.uint64)) % np.uint64(experts)
    ids = ids.astype(np.uint32).reshape(tokens, top_k)
    routes = tokens * top_k
    bufs = [G.empty((experts + 1,), np.uint32)] + [G.empty((routes,), np.uint32) for _ in range(3)]
    ws_bytes = ops.k3_moe_dispatch_workspace_bytes(tokens, top_k, experts)
    ws = G.empty((ws_bytes,), np.uint8)
    assert ops.k3_moe_dispatch_build(*bufs, G.dev(ids), tokens, top_k, experts, ws, ws_bytes)
    assert ops.k3_moe_device_status() == 0
    bad = ids.copy()
    bad[5, 2] = experts                      # one invalid route
    assert ops.k3_moe_dispatch_build(*bufs, G.dev(bad), tokens, top_k, experts, ws, ws_bytes)
    assert ops.k3_moe_device_status() & 2
    assert G.host(bufs[0], np.uint32)[-1] == routes - 1        # the route was counted nowhere
    assert ops.k3_moe_device_status_clear() and ops.k3_moe_device_status() == 0
    err = C.create_string_buffer(128)
    assert ops.k3_moe_dispatch_build_noalloc(*bufs, G.dev(bad), tokens, top_k, experts, err, 128)
    assert ops.k3_moe_device_status() & 2
    assert ops.k3_moe_device_status_clear() and ops.k3_moe_device_status() == 0


def test_bounded_wait_gives_up_and_reports():
    """A wait on a barrier nothing arrives on runs out after its limit (1 ms here),
    the kernel returns, the status word is raised and the context stays usable."""
    assert ops.k3_moe_device_status_clear()
    flag = torch.zeros(1, dtype=torch.int32, device=G.DEV)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    assert ops.k3_moe_selftest_bounded_wait(1000, flag)
    end.record()
    torch.cuda.synchronize()
    assert int(flag.item()) == 1
    assert 0.5 <= begin.elapsed_time(end) <= 100.0
    assert ops.k3_moe_device_status() & 1
    assert ops.k3_moe_device_status_clear() and ops.k3_moe_device_status() == 0
    assert not ops.k3_moe_selftest_bounded_wait(0, flag)
    # the context still runs kernels
    a = torch.ones(1024, device=G.DEV)
    assert float((a + a).sum().item()) == 2048.0


def static_weight(kind, rows, cols, data, scales):
    tensor = _native.StTensor(name=b"w", physical_offset=0, byte_length=rows * cols * 2, shard=0, ndim=2, dtype=1)
    tensor.shape[0], tensor.shape[1] = rows, cols
    w = _native.StaticWeight(tensor=C.pointer(tensor), data=data.data_ptr(),
                             scales=scales.data_ptr() if scales is not None else None,
                             resident_bytes=0, kind=kind)
    return w, tensor


def test_static_weight_wrappers_dispatch_on_the_kind():
    c = cases.op_inputs()
    q = c["q8_128"]
    qd, sd, xd = G.dev(q["q"]), G.dev(q["s"]), G.dev(q["x"])
    n = q["x"].shape[0]
    w, keep = static_weight(2, q["rows"], q["cols"], qd, sd)          # K3_STATIC_WEIGHT_Q8_128
    got, want = G.empty((n, q["rows"]), np.uint16), G.empty((n, q["rows"]), np.uint16)
    assert ops.k3_static_weight_gemm_bf16(w, got, xd, n)
    assert ops.k3_rocm_q8_128_gemm_bf16(want, qd, sd, xd, n, q["rows"], q["cols"])
    assert np.array_equal(G.host(got), G.host(want))
    assert ops.k3_static_weight_gemv_bf16(w, got[0], xd[0])
    assert ops.k3_rocm_q8_128_gemv_bf16(want[0], qd, sd, xd[0], q["rows"], q["cols"])
    assert np.array_equal(G.host(got[0]), G.host(want[0]))
    dn = c["dense"]
    wd, xd = G.dev(dn["w"]), G.dev(dn["x"])
    n = dn["x"].shape[0]
    w, keep = static_weight(1, dn["rows"], dn["cols"], wd, None)       # K3_STATIC_WEIGHT_BF16
    got, want = G.empty((n, dn["rows"]), np.uint16), G.empty((n, dn["rows"]), np.uint16)
    assert ops.k3_static_weight_gemm_bf16(w, got, xd, n)
    assert ops.k3_rocm_bf16_gemm_bf16(want, wd, xd, n, dn["rows"], dn["cols"])
    assert np.array_equal(G.host(got), G.host(want))
    # error behaviour of k3_static_store.cu:315-369: raw kind, wrong rank, no vectors
    w.kind = 0
    assert not ops.k3_static_weight_gemm_bf16(w, got, xd, n)
    w.kind = 1
    keep.ndim = 3
    assert not ops.k3_static_weight_gemv_bf16(w, got, xd)
    keep.ndim = 2
    assert not ops.k3_static_weight_gemm_bf16(w, got, xd, 0)
    assert not ops.k3_static_weight_gemv_bf16(None, got, xd)


def test_phase_ledger_accumulates_under_the_reference_names():
    cfg, weights, x = cases.layer_inputs("mid_t64")
    layer = MoELayer(cfg, weights, seed=14, device=G.DEV, max_tokens=64)
    xd = G.dev(x).view(torch.bfloat16)
    out = torch.empty_like(xd)
    events = [ops.k3_moe_event_create() for _ in range(6)]
    arr = (C.c_void_p * 6)(*events)
    stats = _native.PhaseStats()
    for _ in range(3):
        assert ops.k3_moe_layer_forward_events(layer.desc, out, xd, 64, layer.workspace, layer.workspace.numel(), arr)
        assert ops.k3_moe_phase_stats_add(stats, arr)
    assert stats.layer_passes == 3
    for name in ("router_seconds", "routed_index_seconds", "routed_expert_pipeline_seconds", "moe_tail_seconds"):
        assert 0.0 < getattr(stats, name) < 1.0, name
    assert stats.moe_tail_seconds >= stats.shared_expert_seconds
    missing = (C.c_void_p * 6)(*events[:5], None)
    assert not ops.k3_moe_phase_stats_add(stats, missing)
    for e in events:
        ops.k3_moe_event_destroy(e)


RING_SHAPE = dict(hidden=2048, expert_hidden=1024, experts=32, top_k=8, shared_hidden=1024)


@pytest.mark.parametrize("shape", ["side_stream", "ring"])
def test_one_token_layer_replays_from_a_cuda_graph(shape):
    """One captured one-token call launched again with other tokens gives what eager
    calls give, in both forms of the sequence: row kernels on a side stream with the tail
    inside the kernels (its arrival words count from zero on every replay), and the chain of
    four programmatic launches with the shared expert's ring kernel (its counters and the
    router's done-count are cleared by the kernels themselves)."""
    cfg = synth.baseline_config(**(cases.MID if shape == "side_stream" else RING_SHAPE))
    weights = synth.make_layer(cfg, 21)
    layer = MoELayer(cfg, weights, seed=21, device=G.DEV, max_tokens=1)
    xs = G.dev(synth.activations(22, 3, cfg["hidden"])).view(torch.bfloat16)
    eager = [bf16_tensor_to_bits(layer.forward(xs[i:i + 1])) for i in range(3)]   # first calls outside capture
    torch.cuda.synchronize()
    static_x = xs[0:1].clone()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        layer.forward(static_x)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            static_out = layer.forward(static_x)
    for i in (1, 2, 0, 2):
        static_x.copy_(xs[i:i + 1])
        graph.replay()
        torch.cuda.synchronize()
        assert np.array_equal(bf16_tensor_to_bits(static_out), eager[i]), f"replay with token {i}"
    assert ops.k3_moe_device_status() == 0
