"""The routed layer at the model's real shape (experts on a latent vector): the
fused composition k3_moe_latent_layer_forward against the oracle's operators
chained in the reference's order (k3_engine.cu:1668-1671, 1851-1863, 1889-1893)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
if not torch.cuda.is_available():
    pytest.skip("no CUDA device", allow_module_level=True)

from moonshine_b200 import _native, ops, synth     # noqa: E402
from tests import gpu_util as G                    # noqa: E402

H, L, I, E, K, S = 1024, 512, 512, 16, 4, 256
BLOCK, ST = 128, synth.Q8_F32                        # the reference's static-store format
EPS = 1e-5


def make_weights(seed):
    full = synth.baseline_config(hidden=H, expert_hidden=I, experts=E, top_k=K, shared_hidden=S,
                                 q8_block=BLOCK, q8_scale_type=ST, activation=synth.ACT_SITU,
                                 route_scale=1.0)
    lat = dict(full, hidden=L, shared_hidden=0)
    w = synth.make_layer(full, seed=seed, experts=False)                 # router + shared at width H
    w.update({k: v for k, v in synth.make_layer(lat, seed=seed + 1).items() if k.startswith("w")})
    w["down_w"] = synth.bf16_bits(synth.normal_f32(synth.stream_key(seed, 901), L * H, 0.03)).reshape(L, H)
    w["up_w"] = synth.bf16_bits(synth.normal_f32(synth.stream_key(seed, 902), H * L, 0.03)).reshape(H, L)
    w["norm_w"] = synth.bf16_bits(1.0 + synth.normal_f32(synth.stream_key(seed, 903), L, 0.1))
    return full, w


def oracle_latent_layer(oracle, cfg, w, x):
    t = x.shape[0]
    logits = oracle.bf16_gemm(w["router_weight"], x, E, H)
    ids, wts = oracle.router_topk(logits, w["router_bias"], K, cfg["route_scale"])
    latent = oracle.q8_gemm(w["down_q"], w["down_s"], x, L, H, BLOCK, ST)
    offsets, toks, slots = oracle.group_routes(ids, E)
    outputs = np.zeros((t * K, L), np.uint16)
    for ex in range(E):
        lo, hi = int(offsets[ex]), int(offsets[ex + 1])
        if lo == hi:
            continue
        rows = latent[toks[lo:hi]]
        gate = oracle.mxfp4_gemm(w["w1_packed"][ex], w["w1_scales"][ex], rows, I, L)
        up = oracle.mxfp4_gemm(w["w3_packed"][ex], w["w3_scales"][ex], rows, I, L)
        act = oracle.activation(gate, up, cfg["activation"], cfg["beta"], cfg["linear_beta"])
        outputs[slots[lo:hi]] = oracle.mxfp4_gemm(w["w2_packed"][ex], w["w2_scales"][ex], act, L, I)
    routed = oracle.weighted_sum(outputs, wts, t, K, L)
    normed = oracle.rms_norm(routed, w["norm_w"], L, EPS)
    full = oracle.q8_gemm(w["up_q"], w["up_s"], normed, H, L, BLOCK, ST)
    sg = oracle.q8_gemm(w["shared_gate_q"], w["shared_gate_s"], x, S, H, BLOCK, ST)
    su = oracle.q8_gemm(w["shared_up_q"], w["shared_up_s"], x, S, H, BLOCK, ST)
    sa = oracle.activation(sg, su, cfg["activation"], cfg["beta"], cfg["linear_beta"])
    so = oracle.q8_gemm(w["shared_down_q"], w["shared_down_s"], sa, H, S, BLOCK, ST)
    return oracle.add(full, so), ids, wts, logits


@pytest.mark.parametrize("tokens", [1, 40, 300])
def test_latent_layer_matches_oracle(oracle, tokens):
    cfg, w = make_weights(41)
    w["down_q"], w["down_s"] = oracle.q8_quantize(w["down_w"], L, H, BLOCK, ST)
    w["up_q"], w["up_s"] = oracle.q8_quantize(w["up_w"], H, L, BLOCK, ST)
    x = synth.activations(41, tokens, H)
    want, want_ids, want_w, logits = oracle_latent_layer(oracle, cfg, w, x)

    desc = _native.LatentDesc()
    lay = desc.layer
    lay.hidden, lay.expert_hidden, lay.expert_count, lay.top_k, lay.shared_hidden = H, I, E, K, S
    lay.q8_block, lay.q8_scale_type, lay.activation = BLOCK, ST, cfg["activation"]
    lay.beta, lay.linear_beta, lay.route_scale = cfg["beta"], cfg["linear_beta"], cfg["route_scale"]
    lay.local_expert_first, lay.local_expert_count = 0, E
    names = ["router_weight", "router_bias", "w1_packed", "w1_scales", "w3_packed", "w3_scales", "w2_packed",
             "w2_scales", "shared_gate_q", "shared_gate_s", "shared_up_q", "shared_up_s", "shared_down_q",
             "shared_down_s"]
    keep = {n: G.dev(w[n]) for n in names + ["down_q", "down_s", "up_q", "up_s", "norm_w"]}
    for n in names:
        setattr(lay, n, keep[n].data_ptr())
    desc.latent, desc.norm_epsilon = L, EPS
    desc.down_q, desc.down_s = keep["down_q"].data_ptr(), keep["down_s"].data_ptr()
    desc.up_q, desc.up_s = keep["up_q"].data_ptr(), keep["up_s"].data_ptr()
    desc.norm_weight = keep["norm_w"].data_ptr()

    need = ops.k3_moe_latent_workspace_bytes(desc, tokens)
    assert need > 0
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    out = G.empty((tokens, H), np.uint16)
    ids = G.empty((tokens, K), np.uint32)
    wts = G.empty((tokens, K), np.float32)
    assert ops.k3_moe_latent_layer_forward(desc, out, G.dev(x), tokens, ws, need, ids, wts)
    torch.cuda.synchronize()
    assert ops.k3_moe_device_status() == 0
    got_ids = G.host(ids)
    same = (got_ids == want_ids).all(axis=1)
    # a differing row must be a documented near-tie: score gap below 1e-6 (device expf vs libm)
    gaps = oracle.router_min_gap(logits, w["router_bias"], K)
    assert np.all((gaps[~same] > 0) & (gaps[~same] < 1e-6)), "routing differs beyond near-ties"
    assert np.max(np.abs(G.host(wts)[same] - want_w[same])) <= 1e-6
    assert G.rel_l2(G.host(out, np.uint16)[same], want[same]) <= 1e-2     # the stated layer tolerance
    # a null descriptor field is refused before any launch
    desc.norm_weight = None
    assert not ops.k3_moe_latent_layer_forward(desc, out, G.dev(x), tokens, ws, need, ids, wts)
