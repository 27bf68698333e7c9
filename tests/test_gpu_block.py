"""The layer with the step either side of it (k3_moe_block_forward): post-attention
RMSNorm in front, residual add inside the combine kernel, against the oracle's
operators chained in the reference's order (k3_engine.cu:1550-1553, 1889-1897)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
if not torch.cuda.is_available():
    pytest.skip("no CUDA device", allow_module_level=True)

from moonshine_b200 import ops, synth               # noqa: E402
from moonshine_b200.layer import MoELayer           # noqa: E402
from tests import gpu_util as G                     # noqa: E402


@pytest.mark.parametrize("tokens", [1, 48])
@pytest.mark.parametrize("shape", ["tiny", "block_scaled"])
def test_block_forward_matches_oracle(oracle, tokens, shape):
    cfg = synth.tiny_config() if shape == "tiny" else synth.baseline_config(
        hidden=1024, expert_hidden=512, experts=32, top_k=4, shared_hidden=256)
    weights = synth.make_layer(cfg, seed=51)
    d = cfg["hidden"]
    layer = MoELayer(cfg, weights, seed=51, device="cuda:0", max_tokens=tokens)
    hidden_in = synth.activations(51, tokens, d)
    norm_w = synth.bf16_bits(1.0 + synth.normal_f32(synth.stream_key(51, 77), d, 0.1))
    eps = 1e-5
    xn = oracle.rms_norm(hidden_in, norm_w, d, eps)
    moe, want_ids, _, logits, _ = oracle.moe_layer(weights, xn)
    want = oracle.add(hidden_in, moe)

    need = ops.k3_moe_block_workspace_bytes(layer.desc, tokens)
    assert need > ops.k3_moe_layer_workspace_bytes(layer.desc, tokens) > 0
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    out = G.empty((tokens, d), np.uint16)
    assert ops.k3_moe_block_forward(layer.desc, out, G.dev(hidden_in), G.dev(norm_w), eps, tokens, ws, need)
    torch.cuda.synchronize()
    assert ops.k3_moe_device_status() == 0
    # rows whose routing sits on a near-tie may pick another expert (device expf): leave them out
    gaps = oracle.router_min_gap(logits, weights["router_bias"], cfg["top_k"])
    keep = gaps > 1e-6
    assert keep.mean() > 0.9
    assert G.rel_l2(G.host(out, np.uint16)[keep], want[keep]) <= 1e-2
    assert not ops.k3_moe_block_forward(layer.desc, out, G.dev(hidden_in), None, eps, tokens, ws, need)


def test_combine_residual_is_two_rounded_adds(oracle):
    tokens, k, d = 5, 4, 256
    rows = synth.activations(3, tokens * k, d)
    shared = synth.activations(4, tokens, d)
    residual = synth.activations(5, tokens, d)
    w = np.abs(synth.normal_f32(synth.stream_key(6, 1), tokens * k, 0.3)).astype(np.float32).reshape(tokens, k)
    out = G.empty((tokens, d), np.uint16)
    assert ops.k3_moe_combine_residual(out, G.dev(rows), None, G.dev(w), G.dev(shared), G.dev(residual), tokens, k, d)
    routed = oracle.weighted_sum(rows.reshape(tokens, k, d), w, tokens, k, d)
    want = oracle.add(residual, oracle.add(routed, shared))
    assert np.array_equal(G.host(out, np.uint16), want)
