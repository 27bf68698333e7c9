"""Partially resident store on the GPU: a token's routed experts served from 24
slots (64 experts in host memory) must equal, bit for bit, the same kernels run
on the fully resident table, for a trace long enough to evict and re-admit; the
hit masks must be the slot policy's."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from moonshine_b200 import _native, ops, replay, synth                     # noqa: E402
from moonshine_b200.layer import MoELayer, bf16_tensor_to_bits             # noqa: E402
from moonshine_b200.store import PartialStore, SlotCache, pack_spans       # noqa: E402


def resident_token(layer: MoELayer, x, ids_dev, weights, grouped=False):
    """The store's kernel sequence on the fully resident table: the one-token expert kernel
    where the shape allows it (as the store does), else (or with ``grouped``) dispatch +
    grouped products + combine."""
    cfg, dev = layer.cfg, layer.device
    k, d, e = cfg["top_k"], cfg["hidden"], cfg["experts"]
    i32 = dict(dtype=torch.int32, device=dev)
    out = torch.empty((1, d), dtype=torch.bfloat16, device=dev)
    token_bytes = ops.k3_moe_experts_token_workspace_bytes(layer.desc)
    if token_bytes and not grouped:
        ws = torch.empty(token_bytes, dtype=torch.uint8, device=dev)
        assert ops.k3_moe_experts_token(layer.desc, out, x, ids_dev, weights, ws, ws.numel())
        return out
    offsets = torch.empty(e + 1, **i32)
    sorted_route, sorted_token, inv_perm = (torch.empty(k, **i32) for _ in range(3))
    ws = torch.empty(max(1, ops.k3_moe_dispatch_workspace_bytes(1, k, e)), dtype=torch.uint8, device=dev)
    rows_in = torch.empty((k, d), dtype=torch.bfloat16, device=dev)
    act = torch.empty((k, cfg["expert_hidden"]), dtype=torch.bfloat16, device=dev)
    rows_out = torch.empty((k, d), dtype=torch.bfloat16, device=dev)
    assert ops.k3_moe_dispatch_build(offsets, sorted_route, sorted_token, inv_perm, ids_dev, 1, k, e, ws, ws.numel())
    assert ops.k3_rocm_gather_rows_bf16(rows_in, x, sorted_token, k, d)
    assert ops.k3_moe_experts_grouped(layer.desc, rows_out, act, rows_in, offsets, k)
    assert ops.k3_moe_combine(out, rows_out, inv_perm, weights, None, 1, k, d)
    return out


def test_store_matches_resident_table_over_a_trace():
    cfg = synth.baseline_config(hidden=1024, expert_hidden=512, experts=64, top_k=16, shared_hidden=0)
    weights = synth.make_layer(cfg, seed=21)
    layer = MoELayer(cfg, weights, seed=21, device="cuda:0", max_tokens=1)
    spans = torch.from_numpy(pack_spans(weights, 64, 1024, 512)).pin_memory()
    store = PartialStore(cfg, spans, slots=24, device="cuda:0")
    routes = replay.synthetic_routes(steps=30, layers=1, experts=64, seed=5, reuse=0.5)
    want_masks = replay.replay_cache(routes, 24)["hit_mask"]
    xs = torch.from_numpy(synth.activations(3, 4, 1024).view(np.int16).copy()).cuda().view(torch.bfloat16)
    w = torch.rand(16, device="cuda") + 0.1
    for i in range(len(routes)):
        x = xs[i % 4:i % 4 + 1]
        got, mask = store.token(x, routes.experts[i], w)
        ids_dev = torch.from_numpy(routes.experts[i].astype(np.int32)).cuda().view(1, 16)
        want = resident_token(layer, x, ids_dev, w)
        torch.cuda.synchronize()
        assert mask == int(want_masks[i]), i
        assert np.array_equal(bf16_tensor_to_bits(got), bf16_tensor_to_bits(want)), i
        if i < 4:
            # the one-token kernel and the grouped kernels are two schedules of the same products
            assert store.token_ws is not None
            slow = resident_token(layer, x, ids_dev, w, grouped=True)
            a = bf16_tensor_to_bits(got).astype(np.uint32) << 16
            b = bf16_tensor_to_bits(slow).astype(np.uint32) << 16
            a, b = a.view(np.float32).astype(np.float64), b.view(np.float32).astype(np.float64)
            assert np.sqrt(((a - b) ** 2).sum() / (b ** 2).sum()) <= 2e-3
    st = store.cache.stats()
    assert st["evictions"] > 0 and st["hits"] > 0
    assert store.bytes_admitted == st["admissions"] * store.span_bytes
    assert _native.lib().k3_moe_device_status() == 0


def test_two_layers_share_one_cache():
    cfg = synth.baseline_config(hidden=1024, expert_hidden=512, experts=64, top_k=16, shared_hidden=0)
    weights = [synth.make_layer(cfg, seed=s) for s in (31, 32)]
    spans = [torch.from_numpy(pack_spans(w, 64, 1024, 512)).pin_memory() for w in weights]
    cache = SlotCache(2, 20)
    stores = {n + 1: PartialStore(cfg, spans[n], slots=20, device="cuda:0", cache=cache, layer=n) for n in range(2)}
    routes = replay.synthetic_routes(steps=10, layers=2, experts=64, seed=8)
    x = torch.from_numpy(synth.activations(4, 1, 1024).view(np.int16).copy()).cuda().view(torch.bfloat16)
    w = torch.full((16,), 0.25, device="cuda")
    res = replay.replay_store(stores, routes, x, w)
    np.testing.assert_array_equal(res["hit_mask"], replay.replay_cache(routes, 20)["hit_mask"])
    assert res["bytes_admitted"] == cache.stats()["admissions"] * stores[1].span_bytes
    # the last line ran on layer 2's weights
    layer2 = MoELayer(cfg, weights[1], seed=32, device="cuda:0", max_tokens=1)
    ids_dev = torch.from_numpy(routes.experts[-1].astype(np.int32)).cuda().view(1, 16)
    want = resident_token(layer2, x, ids_dev, w)
    torch.cuda.synchronize()
    assert np.array_equal(bf16_tensor_to_bits(res["last"]), bf16_tensor_to_bits(want))
