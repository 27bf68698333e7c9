"""Parity at the shapes the benchmark runs: 896 experts, hidden 7168, top-16.

The CPU oracle cannot hold 21 GB of expert tables, and does not need to: the
synthetic streams are pure functions of the element index, so for a sample of
tokens the oracle generates just the experts those tokens select
(``oracle.moe_layer_tokens``) and runs the same operators in the same order as
for a whole layer.  Bars: routing ids exact except documented near-ties (score
gap below 1e-6), route weights within 1e-6 x scale, layer output rel-L2 <= 1e-2
(the stated tolerance; the measured figure is printed).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
if not torch.cuda.is_available():
    pytest.skip("no CUDA device", allow_module_level=True)

from moonshine_b200 import ops, synth                             # noqa: E402
from moonshine_b200.layer import MoELayer, bf16_tensor_to_bits    # noqa: E402
from tests import gpu_util as G                                   # noqa: E402

SEED = 0


def has_near_tie(logits, bias, top_k):
    """Per row: is there a POSITIVE gap below 1e-6 between neighbours of the top_k + 1
    largest choices (sigmoid + bias)?  Only such a row may route differently; an exact
    tie (gap 0) never excuses a difference, the lower expert id wins it."""
    choice = (1.0 / (1.0 + np.exp(-logits.astype(np.float64)))).astype(np.float32) + bias[None, :]
    top = -np.sort(-choice, axis=1)[:, :top_k + 1]
    gaps = top[:, :-1] - top[:, 1:]
    return np.any((gaps > 0) & (gaps < 1e-6), axis=1)


def compare(oracle, cfg, weights, x_all, sample, out, ids, wts):
    """Device results of the sampled token rows against the oracle."""
    xs = np.ascontiguousarray(x_all[sample])
    want, want_ids, want_w, logits = oracle.moe_layer_tokens(cfg, SEED, xs, weights)
    got = bf16_tensor_to_bits(out)[sample]
    got_ids = ids.cpu().numpy().view(np.uint32)[sample]
    got_w = wts.cpu().numpy()[sample]
    same = np.all(got_ids == want_ids, axis=1)
    near = has_near_tie(logits, weights["router_bias"], cfg["top_k"])
    assert np.all(same | near), "routing differs on a row without a near-tie (gap in (0, 1e-6))"
    assert same.sum() >= max(1, len(sample) - 2)
    assert np.max(np.abs(got_w[same] - want_w[same])) <= 1e-6 * cfg["route_scale"]
    assert np.all(np.isfinite(G.bf16_f32(got)))
    rel = G.rel_l2(got[same], want[same])
    print(f"tokens={x_all.shape[0]} sample={len(sample)} ids_exact={int(same.sum())} near_ties={int((~same).sum())} "
          f"rel_l2={rel:.2e}")
    assert rel <= 1e-2
    return rel


@pytest.fixture(scope="module")
def bench_layer():
    cfg = synth.baseline_config()
    weights = synth.make_layer(cfg, SEED, experts=False)
    layer = MoELayer(cfg, weights, seed=SEED, device=torch.device("cuda"), max_tokens=8192)
    yield cfg, weights, layer
    del layer
    torch.cuda.empty_cache()


def to_dev(x):
    return torch.from_numpy(x.view(np.int16).copy()).view(torch.bfloat16).cuda()


def test_decode_one_token_896_experts(oracle, bench_layer):
    cfg, weights, layer = bench_layer
    x = synth.activations(7, 3, cfg["hidden"])
    for t in range(3):
        out, ids, wts = layer.forward(to_dev(x[t:t + 1]), want_routes=True)
        torch.cuda.synchronize()
        compare(oracle, cfg, weights, x[t:t + 1], np.array([0]), out, ids, wts)
    assert ops.k3_moe_device_status() == 0


def test_prefill_512_tokens_896_experts(oracle, bench_layer):
    cfg, weights, layer = bench_layer
    x = synth.activations(SEED, 512, cfg["hidden"])
    out, ids, wts = layer.forward(to_dev(x), want_routes=True)
    torch.cuda.synchronize()
    assert ops.k3_moe_device_status() == 0
    compare(oracle, cfg, weights, x, np.arange(5, 512, 34), out, ids, wts)      # 15 tokens


def test_prefill_8192_tokens_zipf_896_experts(oracle, bench_layer):
    """The headline workload: same tensors, Zipf router bias (only the bias differs)."""
    cfg, weights, layer = bench_layer
    zcfg = dict(cfg, bias_mode="zipf")
    zweights = dict(weights, router_bias=synth.router_bias(zcfg, SEED), config=zcfg)
    saved = layer.t["router_bias"].clone()
    try:
        layer.t["router_bias"].copy_(torch.from_numpy(zweights["router_bias"]))
        x = synth.activations(SEED, 8192, cfg["hidden"])
        out, ids, wts = layer.forward(to_dev(x), want_routes=True)
        torch.cuda.synchronize()
        assert ops.k3_moe_device_status() == 0
        counts = np.bincount(ids.cpu().numpy().ravel(), minlength=cfg["experts"])
        assert counts.max() > 4 * counts.mean()                      # the load really is skewed
        compare(oracle, zcfg, zweights, x, np.arange(100, 8192, 520), out, ids, wts)   # 16 tokens
    finally:
        layer.t["router_bias"].copy_(saved)


@pytest.mark.parametrize("tokens", [1, 16, 128, 1024, 4096, 16384])
def test_stress_sweep_hot_experts_ties_extreme_scales(oracle, tokens):
    """The stress configuration at every token count of its sweep: four experts that
    every token selects, 10 % of the router rows duplicated (exact score ties, decided by
    the lower expert id with no near-tie allowance), E8M0 scale bytes over 0..127."""
    cfg = synth.baseline_config(bias_mode="hot4", duplicate_router_rows=45, scale_low=0, scale_span=128)
    weights = synth.make_layer(cfg, SEED, experts=False)
    layer = MoELayer(cfg, weights, seed=SEED, device=torch.device("cuda"), max_tokens=tokens)
    try:
        x = synth.activations(SEED + 1, tokens, cfg["hidden"])
        out, ids, wts = layer.forward(to_dev(x), want_routes=True)
        torch.cuda.synchronize()
        assert ops.k3_moe_device_status() == 0
        host_ids = ids.cpu().numpy()
        counts = np.bincount(host_ids.ravel(), minlength=cfg["experts"])
        assert np.sort(counts)[-4:].min() == tokens                  # the four hot experts take every token
        sample = np.unique(np.linspace(0, tokens - 1, num=min(tokens, 6)).astype(np.int64))
        compare(oracle, cfg, weights, x, sample, out, ids, wts)
    finally:
        del layer
        torch.cuda.empty_cache()
