"""GPU parity of the fused layer (k3_moe_layer_forward through the C-ABI)
against the golden vectors: routing ids and the dispatch permutation bit-exact
except documented near-ties (score gap < 1e-6), layer output within rel-L2
1e-2 (the stated tolerance; in practice ~1e-3), plus size-independent
properties at the full benchmark shape."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
if not torch.cuda.is_available():
    pytest.skip("no CUDA device", allow_module_level=True)

from moonshine_b200 import ops, synth                       # noqa: E402
from moonshine_b200.layer import MoELayer, bf16_tensor_to_bits   # noqa: E402
from tests import gpu_util as G                             # noqa: E402
from tests.golden import cases                              # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = dict(np.load(os.path.join(HERE, "golden", "layers.npz")))
REL_L2_TOLERANCE = 1e-2


def run_layer(name):
    cfg, weights, x = cases.layer_inputs(name)
    layer = MoELayer(cfg, weights, seed=cases.LAYER_CASES[name][1], max_tokens=x.shape[0])
    xd = G.dev(x).view(torch.bfloat16)
    out, ids, w = layer.forward(xd, want_routes=True)
    return cfg, bf16_tensor_to_bits(out), G.host(ids, np.uint32), G.host(w)


@pytest.mark.parametrize("name", list(cases.LAYER_CASES))
def test_layer_matches_golden(name):
    cfg, out, ids, w = run_layer(name)
    want_ids, want_w, gaps = GOLD[name + "_ids"], GOLD[name + "_w"], GOLD[name + "_gap"]
    same = np.all(ids == want_ids, axis=1)
    for t in np.nonzero(~same)[0]:
        assert 0 < gaps[t] < 1e-6, (name, t, gaps[t])       # only documented near-ties
    assert np.max(np.abs(w[same] - want_w[same])) <= 1e-6 * cfg["route_scale"] + 1e-7
    rel = G.rel_l2(out[same], GOLD[name + "_out"][same])
    assert rel <= REL_L2_TOLERANCE, (name, rel)
    assert np.all(np.isfinite(G.bf16_f32(out)))


def test_device_fill_equals_host_weights():
    # a layer whose experts were filled on the device equals one uploaded from numpy
    name = "mid_t64"
    cfg, weights, x = cases.layer_inputs(name)
    seed = cases.LAYER_CASES[name][1]
    a = MoELayer(cfg, weights, seed=seed)
    slim = {k: v for k, v in weights.items() if not k.startswith("w")}
    b = MoELayer(cfg, slim, seed=seed)
    for key in ("w1_packed", "w1_scales", "w3_packed", "w3_scales", "w2_packed", "w2_scales"):
        assert torch.equal(a.t[key].flatten(), b.t[key].flatten()), key


def test_decode_matches_prefill_row():
    # the one-token path (rank order, matrix-vector kernels) and the batched path
    # (dispatch, tensor-core grouped GEMM) are two reduction schedules of the same
    # products: outputs agree to the cross-schedule envelope, routing exactly
    cfg, weights, x = cases.layer_inputs("mid_t64")
    layer = MoELayer(cfg, weights, max_tokens=64)
    xd = G.dev(x).view(torch.bfloat16)
    out, ids, w = layer.forward(xd, want_routes=True)
    batch, ids = bf16_tensor_to_bits(out), G.host(ids, np.uint32)
    gaps = GOLD["mid_t64_gap"]
    for t in (0, 17, 63):
        o1, i1, w1 = layer.forward(xd[t:t + 1].contiguous(), want_routes=True)
        if gaps[t] >= 1e-6:
            assert np.array_equal(G.host(i1, np.uint32)[0], ids[t])
        assert G.rel_l2(bf16_tensor_to_bits(o1)[0], batch[t]) <= 2e-3


def test_store_admit_from_checkpoint_span():
    # six tensors in the checkpoint order w1.p, w1.s, w2.p, w2.s, w3.p, w3.s, span start
    # 8 bytes off a 16-byte boundary (k3_engine.cu:105-114, k3_rocm_ops.cu:212-216)
    cfg, weights, x = cases.layer_inputs("tiny_t37")
    layer = MoELayer(cfg, weights, max_tokens=37)
    ref = bf16_tensor_to_bits(layer.forward(G.dev(x).view(torch.bfloat16)))
    blank = {k: (np.zeros_like(v) if k.startswith("w") else v) for k, v in weights.items()}
    other = MoELayer(cfg, blank, max_tokens=37)
    for e in range(cfg["experts"]):
        parts = [weights[k][e].tobytes() for k in
                 ("w1_packed", "w1_scales", "w2_packed", "w2_scales", "w3_packed", "w3_scales")]
        rel, off = [], 8
        for part in parts:
            rel.append(off)
            off += len(part)
        span = np.frombuffer(b"\0" * 8 + b"".join(parts), np.uint8)
        import ctypes as C
        arr = (C.c_uint64 * 6)(*rel)
        assert ops.k3_moe_store_admit(other.desc, e, G.dev(span), arr)
    got = bf16_tensor_to_bits(other.forward(G.dev(x).view(torch.bfloat16)))
    assert np.array_equal(got, ref)


def test_invalid_layer_arguments():
    cfg, weights, x = cases.layer_inputs("tiny_t1")
    layer = MoELayer(cfg, weights)
    xd = G.dev(x).view(torch.bfloat16)
    out = torch.empty_like(xd)
    assert not ops.k3_moe_layer_forward(layer.desc, out, xd, 1, layer.workspace, 16, None, None)
    assert not ops.k3_moe_layer_forward(layer.desc, None, xd, 1, layer.workspace,
                                        layer.workspace.numel(), None, None)
    assert not ops.k3_moe_layer_forward(layer.desc, out, xd, 0, layer.workspace,
                                        layer.workspace.numel(), None, None)


def test_full_shape_decode_properties(oracle):
    """Benchmark shape (d=7168, I=2048, top-16, MXFP4 experts, Q8 shared) with a
    reduced expert count so the host oracle finishes in seconds; decode T=1 and a
    small prefill are compared with the oracle in full."""
    cfg = synth.baseline_config(experts=64)
    weights = synth.make_layer(cfg, seed=0)
    layer = MoELayer(cfg, weights, seed=0, max_tokens=4)
    for tokens in (1, 4):
        x = synth.activations(100 + tokens, tokens, cfg["hidden"])
        out, ids, w = layer.forward(G.dev(x).view(torch.bfloat16), want_routes=True)
        want_out, want_ids, want_w, logits, _ = oracle.moe_layer(weights, x)
        gaps = oracle.router_min_gap(logits, weights["router_bias"], cfg["top_k"])
        got_ids = G.host(ids, np.uint32)
        same = np.all(got_ids == want_ids, axis=1)
        assert np.all((gaps[~same] > 0) & (gaps[~same] < 1e-6))
        assert G.rel_l2(bf16_tensor_to_bits(out)[same], want_out[same]) <= REL_L2_TOLERANCE


_PATHS_SCRIPT = r"""
import sys
import numpy as np, torch
from moonshine_b200 import synth
from moonshine_b200.layer import MoELayer, bf16_tensor_to_bits
out = []
for block, scale in ((32, synth.Q8_F16), (128, synth.Q8_F32)):
    cfg = synth.baseline_config(experts=32, hidden=2048, expert_hidden=1024, shared_hidden=1024, top_k=8,
                                q8_block=block, q8_scale_type=scale)
    layer = MoELayer(cfg, None, seed=5, device=torch.device("cuda:0"), max_tokens=4)
    x = torch.from_numpy(synth.activations(9, 3, cfg["hidden"]).view(np.int16)).cuda().view(torch.bfloat16)
    for t in range(3):
        out.append(bf16_tensor_to_bits(layer.forward(x[t:t + 1].contiguous())).copy())
np.save(sys.argv[1], np.concatenate(out))
"""


def test_one_token_shared_expert_paths_give_the_same_bits(tmp_path):
    """The shared expert of the one-token layer as the ring kernel (bulk copies into shared
    memory, K3MOE_SHARED_CTAS default) and as the row kernels on a side stream
    (K3MOE_SHARED_CTAS=0) run the same arithmetic: layer outputs equal bit for bit, for f16
    scales per 32 columns and f32 scales per 128."""
    import subprocess
    import sys
    root = os.path.dirname(HERE)
    got = []
    for ctas in ("32", "0"):
        path = str(tmp_path / f"out_{ctas}.npy")
        env = dict(os.environ, K3MOE_SHARED_CTAS=ctas, PYTHONPATH=root)
        subprocess.run([sys.executable, "-c", _PATHS_SCRIPT, path], check=True, env=env, cwd=root, timeout=600)
        got.append(np.load(path))
    assert got[0].shape == got[1].shape and got[0].size == 6 * 2048
    assert np.array_equal(got[0], got[1])


@pytest.mark.parametrize("ties", [False, True])
def test_one_token_routing_prefilter_and_general_method(oracle, ties):
    """The expert kernel routes the token itself: a threshold from a few arg-max rounds per
    warp leaves a few dozen candidates to rank; when more than 256 experts reach the
    threshold (here: every choice value equal, 384 experts) the general method runs.  Both
    must give the oracle's ids (lower id first on ties) and weights."""
    cfg = synth.baseline_config(experts=384, hidden=2048, expert_hidden=1024, shared_hidden=1024, top_k=8)
    weights = synth.make_layer(cfg, seed=11)
    if ties:
        weights["router_weight"][...] = 0          # every logit 0: sigmoid 0.5
        weights["router_bias"][...] = 0.25
    layer = MoELayer(cfg, weights, seed=11, max_tokens=2)
    x = synth.activations(21, 1, cfg["hidden"])
    out, ids, w = layer.forward(G.dev(x).view(torch.bfloat16), want_routes=True)
    want_out, want_ids, want_w, logits, _ = oracle.moe_layer(weights, x)
    got_ids = G.host(ids, np.uint32)
    if ties:
        assert np.array_equal(got_ids[0], np.arange(cfg["top_k"], dtype=np.uint32))
    gaps = oracle.router_min_gap(logits, weights["router_bias"], cfg["top_k"])
    assert np.array_equal(got_ids, want_ids) or (0 < gaps[0] < 1e-6)
    if np.array_equal(got_ids, want_ids):
        assert np.allclose(G.host(w), want_w, rtol=1e-6, atol=0)
        assert G.rel_l2(bf16_tensor_to_bits(out), want_out) <= REL_L2_TOLERANCE
