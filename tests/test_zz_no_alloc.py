"""The allocation-free dispatch entry point.

Some callers of the library are not allowed to allocate device memory: an engine
that carves every buffer out of one start-up allocation (as the reference engine
does) and then hands its operators only pointers, or a code path that runs while
allocation is off limits.  k3_moe_dispatch_build_noalloc serves them by keeping
the histogram scratch in a fixed array inside the library.  This test calls it
through the C-ABI twice in a row (the array keeps the previous call's contents,
so the second call proves nothing stale leaks through) and requires exactly the
outputs of k3_moe_dispatch_build, the entry point with a caller workspace.
Collected last so that a failure here cannot hide any other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
if not torch.cuda.is_available():
    pytest.skip("no CUDA device", allow_module_level=True)

from moonshine_b200 import ops, synth      # noqa: E402
from tests import gpu_util as G            # noqa: E402


def route_ids(tokens, top_k, experts, seed):
    h = synth.hash64(synth.stream_key(seed, 5), np.arange(tokens * experts, dtype=np.uint64))
    return np.argsort(h.reshape(tokens, experts), axis=1)[:, :top_k].astype(np.uint32)


def run_both(tokens, top_k, experts, seed):
    ids = G.dev(route_ids(tokens, top_k, experts, seed))
    routes = tokens * top_k
    ref = [G.empty((experts + 1,), np.uint32)] + [G.empty((routes,), np.uint32) for _ in range(3)]
    ws_bytes = ops.k3_moe_dispatch_workspace_bytes(tokens, top_k, experts)
    ws = G.empty((ws_bytes,), np.uint8)
    assert ops.k3_moe_dispatch_build(*ref, ids, tokens, top_k, experts, ws, ws_bytes)
    got = [G.empty((experts + 1,), np.uint32)] + [G.empty((routes,), np.uint32) for _ in range(3)]
    err = C.create_string_buffer(256)
    assert ops.k3_moe_dispatch_build_noalloc(*got, ids, tokens, top_k, experts, err, 256), err.value
    assert err.value == b""
    for a, b in zip(got, ref):
        assert np.array_equal(G.host(a, np.uint32), G.host(b, np.uint32))


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    # a large problem first, then a smaller one with other routing: the second call
    # sees the first call's histograms still sitting in the shared array
    run_both(8192, 16, 896, seed=1)
    run_both(300, 8, 64, seed=2)
    run_both(8192, 16, 896, seed=3)


def test_sizes_beyond_the_built_in_scratch_are_refused():
    assert ops.k3_moe_dispatch_noalloc_max_routes() == 131072
    dummy = G.empty((16,), np.uint32)
    err = C.create_string_buffer(256)
    assert not ops.k3_moe_dispatch_build_noalloc(dummy, dummy, dummy, dummy, dummy, 8193, 16, 896, err, 256)
    assert b"131072" in err.value
    assert not ops.k3_moe_dispatch_build_noalloc(dummy, dummy, dummy, dummy, dummy, 4, 2, 1025, err, 256)
    assert not ops.k3_moe_dispatch_build_noalloc(None, dummy, dummy, dummy, dummy, 4, 2, 8, err, 256)
