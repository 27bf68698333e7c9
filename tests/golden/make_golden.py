"""Regenerates the golden output vectors from the CPU oracle:

    python tests/golden/make_golden.py

The reference itself (HIP kernels, 1.6 TB checkpoint) cannot run here, so the
stored vectors are outputs of oracle/k3_oracle.c, which tests/test_oracle_pins.py
pins against the reference's own model-free test recipes.  They freeze the
oracle: any later change of its arithmetic shows up as a golden mismatch.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import k3_oracle as o          # noqa: E402
from tests.golden import cases             # noqa: E402


def ops_golden():
    d = cases.op_inputs()
    g = {}
    for name in ("mx_a", "mx_b", "mx_c"):
        c = d[name]
        g[name] = o.mxfp4_gemm(c["packed"], c["scales"], c["x"], c["rows"], c["cols"])
        g[name + "_f64"] = o.mxfp4_gemm_f64(c["packed"], c["scales"], c["x"], c["rows"], c["cols"])
    for name in ("dense", "dense_odd"):
        c = d[name]
        f, b = o.bf16_gemm(c["w"], c["x"], c["rows"], c["cols"], want_bf16=True)
        g[name + "_f32"], g[name + "_bf16"] = f, b
    for name in ("q8_128", "q8_32"):
        c = d[name]
        g[name] = o.q8_gemm(c["q"], c["s"], c["x"], c["rows"], c["cols"], c["block"], c["st"])
    for name in ("router", "router_small"):
        c = d[name]
        g[name + "_ids"], g[name + "_w"] = o.router_topk(c["logits"], c["bias"], c["top_k"], c["scale"])
    c = d["wsum"]
    g["wsum"] = o.weighted_sum(c["v"], c["w"], c["tokens"], c["count"], c["hidden"])
    c = d["norm"]
    g["norm"] = o.rms_norm(c["x"], c["w"], c["hidden"], 1e-5)
    c = d["act"]
    g["act_situ"] = o.activation(c["g"], c["u"], o.ACT_SITU, 4.0, 25.0)
    g["act_swiglu"] = o.activation(c["g"], c["u"], o.ACT_SWIGLU)
    g["add"] = o.add(c["g"], c["u"])
    qw, qs = o.q8_quantize(d["dense"]["w"], 48, 512, 128, o.Q8_F32)
    g["quant_q"], g["quant_s"] = qw, qs
    return g


def layers_golden():
    g = {}
    for name in cases.LAYER_CASES:
        cfg, weights, x = cases.layer_inputs(name)
        out, ids, w, logits, _ = o.moe_layer(weights, x)
        offsets, toks, slots = o.group_routes(ids, cfg["experts"])
        g[name + "_out"], g[name + "_ids"], g[name + "_w"] = out, ids, w
        g[name + "_offsets"], g[name + "_slots"] = offsets, slots
        g[name + "_gap"] = o.router_min_gap(logits, weights["router_bias"], cfg["top_k"])
    return g


if __name__ == "__main__":
    np.savez_compressed(os.path.join(HERE, "ops.npz"), **ops_golden())
    np.savez_compressed(os.path.join(HERE, "layers.npz"), **layers_golden())
    for f in ("ops.npz", "layers.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")
