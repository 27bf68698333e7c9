"""GPU checks at the benchmark's hidden sizes (7168 / 2048): long K extents, several
work items per persistent block and wrapped pipeline rings, which the small parity
cases do not reach.  Results must repeat bit for bit from call to call, agree with
the bf16 tensor-core path, and match the oracle on sampled rows."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
if not torch.cuda.is_available():
    pytest.skip("no CUDA device", allow_module_level=True)

from moonshine_b200 import _native, ops, synth     # noqa: E402
from moonshine_b200.layer import MoELayer          # noqa: E402
from tests import gpu_util as G                    # noqa: E402


def test_block_scaled_grouped_repeats_and_matches_at_full_k(oracle):
    d, i, e = 7168, 2048, 8
    counts = [300, 0, 129, 700, 64, 17, 500, 338]           # 20 row tiles x 16 weight tiles > 148 blocks
    cfg = synth.baseline_config(hidden=d, expert_hidden=i, experts=e, top_k=2, shared_hidden=0)
    w = synth.make_layer(cfg, seed=31)
    rows = int(sum(counts))
    x = synth.activations(31, rows, d)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32)
    desc = _native.LayerDesc(hidden=d, expert_hidden=i, expert_count=e, top_k=2, shared_hidden=0,
                             activation=cfg["activation"], route_scale=1.0, local_expert_count=e)
    keep = {k: G.dev(w[k]) for k in w if k.startswith("w")}
    for k, v in keep.items():
        setattr(desc, k, v.data_ptr())
    xd, od = G.dev(x), G.dev(offsets)
    need = ops.k3_moe_experts_workspace_bytes(desc, rows, 0)
    assert need > 0
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    runs = []
    for _ in range(3):
        out = torch.zeros((rows, d), dtype=torch.int16, device="cuda")
        act = torch.zeros((rows, i), dtype=torch.int16, device="cuda")
        assert ops.k3_moe_experts_grouped_ws(desc, out, act, xd, None, 0, od, rows, ws, need)
        torch.cuda.synchronize()
        runs.append((act, out))
    assert ops.k3_moe_device_status() == 0
    for act, out in runs[1:]:
        assert torch.equal(act, runs[0][0]) and torch.equal(out, runs[0][1]), "results differ between calls"
    # against the bf16 tensor-core path (weights rounded to bf16 there: ~4e-3)
    out2 = torch.zeros((rows, d), dtype=torch.int16, device="cuda")
    act2 = torch.zeros((rows, i), dtype=torch.int16, device="cuda")
    assert ops.k3_moe_experts_grouped(desc, out2, act2, xd, od, rows)
    torch.cuda.synchronize()
    got_act, got_out = G.host(runs[0][0], np.uint16), G.host(runs[0][1], np.uint16)
    assert G.rel_l2(got_act, G.host(act2, np.uint16)) <= 6e-3
    assert G.rel_l2(got_out, G.host(out2, np.uint16)) <= 6e-3
    # against the oracle on the first and last rows of two experts (whole K, every weight tile)
    for ex, pick in ((2, [0, 1, 127, 128]), (3, [0, 255, 699])):
        lo = int(offsets[ex])
        r = np.array(pick) + lo
        xe = x[r]
        gate = oracle.mxfp4_gemm(w["w1_packed"][ex], w["w1_scales"][ex], xe, i, d)
        up = oracle.mxfp4_gemm(w["w3_packed"][ex], w["w3_scales"][ex], xe, i, d)
        a = oracle.activation(gate, up, cfg["activation"])
        assert G.rel_l2(got_act[r], a) <= 1e-3, ex
        down = oracle.mxfp4_gemm(w["w2_packed"][ex], w["w2_scales"][ex], got_act[r], d, i)
        assert G.rel_l2(got_out[r], down) <= 1e-3, ex


def test_one_token_layer_repeats_at_full_sizes():
    cfg = synth.baseline_config(experts=32)                  # top-16 of 32, baseline hidden sizes
    layer = MoELayer(cfg, None, seed=5, device=torch.device("cuda"), max_tokens=1)
    xs = torch.from_numpy(synth.activations(5, 4, cfg["hidden"]).view(np.int16).copy()).view(torch.bfloat16).cuda()
    first = [layer.forward(xs[t:t + 1]).clone() for t in range(4)]
    torch.cuda.synchronize()
    outs = [layer.forward(xs[n % 4:n % 4 + 1]) for n in range(200)]
    torch.cuda.synchronize()
    assert ops.k3_moe_device_status() == 0
    assert all(torch.equal(o, first[n % 4]) for n, o in enumerate(outs)), "one-token results differ between calls"


def test_prefill_layer_repeats_at_full_sizes():
    cfg = synth.baseline_config(experts=32, bias_mode="zipf")
    tokens = 1024
    layer = MoELayer(cfg, None, seed=6, device=torch.device("cuda"), max_tokens=tokens)
    x = torch.from_numpy(synth.activations(6, tokens, cfg["hidden"]).view(np.int16).copy()).view(torch.bfloat16).cuda()
    a = layer.forward(x).clone()
    b = layer.forward(x).clone()
    c = layer.forward(x).clone()
    torch.cuda.synchronize()
    assert ops.k3_moe_device_status() == 0
    assert torch.equal(a, b) and torch.equal(a, c), "prefill results differ between calls"
