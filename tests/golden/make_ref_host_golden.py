"""Records outputs of the reference's own host-side checking functions.

Needs the reference tree: ``python tests/golden/make_ref_host_golden.py <reference tree>``
cuts and compiles those functions (``make -C oracle ref_host``), runs them on the
seeded inputs of ``ref_host_cases.py`` and writes ``tests/golden/ref_host.npz``.
The file holds reference OUTPUTS only (inputs are regenerated from their seeds);
``tests/test_oracle_vs_ref.py`` holds the CPU oracle to them bit for bit on
machines where the reference tree, and so the compiled functions, are absent.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import ref_host as ref                     # noqa: E402
from tests.golden import ref_host_cases as cases       # noqa: E402


def record(fused: bool = True) -> dict:
    out = {}
    out["bf16_round"] = ref.float_to_bf16(cases.bf16_values(), fused)
    out["e8m0"] = ref.e8m0_table(fused)
    out["e2m1"] = ref.e2m1_table(fused)
    # router logits at the router's own shape, and a short ragged-free shape
    for name, case, rows, columns, sigma in (("router", 1, cases.REF_EXPERTS, 7168, 0.02),
                                              ("small", 2, 128, 512, 0.25)):
        w = cases.bf16_matrix(case, rows, columns, sigma)
        x = cases.activations(case, columns)
        out[f"bf16_gemv_{name}_f32"], out[f"bf16_gemv_{name}_bf16"] = ref.bf16_gemv(w, x, rows, columns, fused)
    # MXFP4 GEMV: benchmark scale range, the stress range (bytes 0..127), real and benchmark shapes
    for name, case, rows, columns, low, span in (("gate_real", 3, 512, cases.REF_LATENT, 119, 5),
                                                  ("down_bench", 4, 512, 2048, 119, 5),
                                                  ("gate_bench_extreme", 5, 256, 7168, 0, 128),
                                                  ("small", 6, 128, 512, 122, 11)):
        p, s = cases.mxfp4_matrix(case, rows, columns, low, span)
        x = cases.activations(case, columns)
        out[f"mxfp4_gemv_{name}"] = ref.mxfp4_gemv(p, s, x, rows, columns, fused)
        if name in ("small", "gate_bench_extreme"):
            x4 = cases.activations(case, 4 * columns).reshape(4, columns)
            out[f"mxfp4_f64_{name}"] = ref.mxfp4_f64(p[:64], s[:64], x4, 64, columns, fused)
    g = cases.activations(7, 1 << 16, 4.0)
    u = synth_up = cases.activations(8, 1 << 16, 20.0)
    out["situ"] = ref.situ(g, u, fused)
    for name, case, count in (("latent", 9, cases.REF_LATENT), ("hidden", 10, 7168)):
        x = cases.activations(case, count, 2.0)
        w = cases.bf16_matrix(case, 1, count, 0.5).ravel()
        out[f"rms_norm_{name}"] = ref.rms_norm(x, w, 1e-5, fused)
    logits, bias, tied_bias = cases.router_rows(11, 32)
    ids, weights = [], []
    for r in range(logits.shape[0]):
        i, w = ref.router(logits[r], tied_bias if r % 2 else bias, fused)
        ids.append(i)
        weights.append(w)
    out["router_ids"], out["router_weights"] = np.stack(ids), np.stack(weights)
    q, s = cases.q8_rows(12, 64)
    x = cases.activations(12, cases.REF_Q8_COLUMNS)
    out["q8_rows"] = np.array([ref.q8_row(q[r], s[r], x) for r in range(q.shape[0])], np.uint16)
    # three experts accumulated with route weights, then the final rounding (:616-618)
    latent = cases.activations(13, cases.REF_LATENT)
    acc = np.zeros(cases.REF_LATENT, np.float32)
    route_weights = np.array([0.41, 0.33, 0.26], np.float32)
    rows = []
    for rank in range(3):
        rows.append(ref.expert_accumulate(acc, float(route_weights[rank]), cases.expert_span(13, rank), latent, fused))
    out["expert_rows"] = np.stack(rows)
    out["expert_accumulator"] = acc
    out["expert_routed"] = ref.float_to_bf16(acc, fused)
    return out


if __name__ == "__main__":
    tree = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("K3_REFERENCE_DIR")
    assert tree, "usage: make_ref_host_golden.py <reference tree>"
    ref.build(tree)
    fused = record(True)
    unfused = record(False)
    # which recorded outputs depend on multiply-add fusion (kept in the file so the
    # test can say so): only the Q8 row and the weighted accumulation may
    depends = sorted(k for k in fused if fused[k].tobytes() != unfused[k].tobytes())
    print("outputs that change without fusion:", depends)
    np.savez_compressed(os.path.join(HERE, "ref_host.npz"), fusion_dependent=np.array(depends),
                        **fused, **{"unfused__" + k: unfused[k] for k in depends})
    print("wrote", os.path.join(HERE, "ref_host.npz"), os.path.getsize(os.path.join(HERE, "ref_host.npz")), "bytes")
