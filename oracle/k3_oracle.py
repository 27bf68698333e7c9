"""ctypes/numpy front end of the CPU oracle (``oracle/k3_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
CPU-baseline leg of the benchmark.  The product package never imports it.

bf16 tensors are ``numpy.uint16`` arrays holding the raw bit patterns.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libk3oracle.so")

ACT_SITU, ACT_SWIGLU, ACT_SITU_HOST = 0, 1, 2
Q8_F32, Q8_F16 = 0, 1


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (no-op when the library is up to date)."""
    src = os.path.join(_HERE, "k3_oracle.c")
    hdr = os.path.join(_HERE, "k3_oracle.h")
    stale = (not os.path.exists(_LIB_PATH)
             or os.path.getmtime(_LIB_PATH) < max(os.path.getmtime(src), os.path.getmtime(hdr)))
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.k3o_moe_layer.restype = C.c_uint64
        _lib.k3o_thread_count.restype = C.c_int
        _lib.k3o_bf16_from_float.restype = C.c_uint16
        _lib.k3o_bf16_from_float.argtypes = [C.c_float]
        _lib.k3o_bf16_to_float.restype = C.c_float
        _lib.k3o_bf16_to_float.argtypes = [C.c_uint16]
    return _lib


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(C.c_void_p)


def _u16(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint16, a.dtype
    return a


def set_threads(threads: int) -> None:
    lib().k3o_set_threads(C.c_int(threads))


def thread_count() -> int:
    return int(lib().k3o_thread_count())


# --------------------------------------------------------------------- bf16
def bf16_from_f32(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (vectorised mirror of
    k3o_bf16_from_float; checked against it in the tests)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    nan = (bits & 0x7FFFFFFF) > 0x7F800000
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) >> 16
    out = np.where(nan, (bits >> 16) | 0x40, rounded)
    return out.astype(np.uint16)


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    return (a.astype(np.uint32) << 16).view(np.float32)


# ---------------------------------------------------------------------- ops
def bf16_gemm(weights, x, rows, columns, want_bf16=False):
    x = _u16(x).reshape(-1, columns)
    w = _u16(weights)
    n = x.shape[0]
    out32 = np.empty((n, rows), np.float32)
    out16 = np.empty((n, rows), np.uint16) if want_bf16 else None
    lib().k3o_bf16_gemm(_p(out32), _p(out16), _p(w), _p(x), C.c_uint32(n),
                        C.c_uint32(rows), C.c_uint32(columns))
    return (out32, out16) if want_bf16 else out32


def _mx(fn, dtype, packed, scales, x, rows, columns):
    x = _u16(x).reshape(-1, columns)
    packed = np.ascontiguousarray(packed, np.uint8)
    scales = np.ascontiguousarray(scales, np.uint8)
    assert packed.size == rows * columns // 2 and scales.size == rows * columns // 32
    n = x.shape[0]
    out = np.empty((n, rows), dtype)
    fn(_p(out), _p(packed), _p(scales), _p(x), C.c_uint32(n), C.c_uint32(rows),
       C.c_uint32(columns))
    return out


def mxfp4_gemm(packed, scales, x, rows, columns):
    return _mx(lib().k3o_mxfp4_gemm, np.uint16, packed, scales, x, rows, columns)


def mxfp4_gemm_kernel_order(packed, scales, x, rows, columns):
    return _mx(lib().k3o_mxfp4_gemm_kernel_order, np.uint16, packed, scales, x, rows, columns)


def mxfp4_gemm_f64(packed, scales, x, rows, columns):
    return _mx(lib().k3o_mxfp4_gemm_f64, np.float64, packed, scales, x, rows, columns)


def activation(gate, up, kind=ACT_SITU, beta=4.0, linear_beta=25.0):
    gate, up = _u16(gate), _u16(up)
    out = np.empty_like(gate)
    lib().k3o_activation(_p(out), _p(gate), _p(up), C.c_uint64(gate.size), C.c_int(kind),
                         C.c_float(beta), C.c_float(linear_beta))
    return out


def rms_norm(x, weight, hidden, epsilon=1e-5):
    x = _u16(x).reshape(-1, hidden)
    out = np.empty_like(x)
    lib().k3o_rms_norm(_p(out), _p(x), _p(_u16(weight)), C.c_uint32(x.shape[0]),
                       C.c_uint32(hidden), C.c_float(epsilon))
    return out


def router_topk(logits, bias, top_k, scale=1.0):
    logits = np.ascontiguousarray(logits, np.float32)
    logits = logits.reshape(-1, logits.shape[-1])
    bias = np.ascontiguousarray(bias, np.float32)
    n, e = logits.shape
    ids = np.empty((n, top_k), np.uint32)
    w = np.empty((n, top_k), np.float32)
    lib().k3o_router_topk(_p(ids), _p(w), _p(logits), _p(bias), C.c_uint32(n), C.c_uint32(e),
                          C.c_uint32(top_k), C.c_float(scale))
    return ids, w


def router_min_gap(logits, bias, top_k):
    logits = np.ascontiguousarray(logits, np.float32)
    logits = logits.reshape(-1, logits.shape[-1])
    bias = np.ascontiguousarray(bias, np.float32)
    n, e = logits.shape
    gaps = np.empty(n, np.float32)
    lib().k3o_router_min_gap(_p(gaps), _p(logits), _p(bias), C.c_uint32(n), C.c_uint32(e),
                             C.c_uint32(top_k))
    return gaps


def weighted_sum(vectors, weights, tokens, count, hidden):
    vectors = _u16(vectors)
    weights = np.ascontiguousarray(weights, np.float32)
    out = np.empty((tokens, hidden), np.uint16)
    lib().k3o_weighted_sum(_p(out), _p(vectors), _p(weights), C.c_uint32(tokens),
                           C.c_uint32(count), C.c_uint32(hidden))
    return out


def add(left, right):
    left, right = _u16(left), _u16(right)
    out = np.empty_like(left)
    lib().k3o_add(_p(out), _p(left), _p(right), C.c_uint64(left.size))
    return out


def q8_quantize(weights, rows, columns, block=128, scale_type=Q8_F32):
    weights = _u16(weights)
    q = np.empty((rows, columns), np.int8)
    s = np.empty((rows, columns // block), np.float16 if scale_type == Q8_F16 else np.float32)
    lib().k3o_q8_quantize(_p(q), _p(s), _p(weights), C.c_uint32(rows), C.c_uint32(columns),
                          C.c_uint32(block), C.c_int(scale_type))
    return q, s


def q8_gemm(q, s, x, rows, columns, block=128, scale_type=Q8_F32):
    x = _u16(x).reshape(-1, columns)
    q = np.ascontiguousarray(q, np.int8)
    s = np.ascontiguousarray(s)
    assert s.dtype == (np.float16 if scale_type == Q8_F16 else np.float32)
    out = np.empty((x.shape[0], rows), np.uint16)
    lib().k3o_q8_gemm(_p(out), _p(q), _p(s), _p(x), C.c_uint32(x.shape[0]), C.c_uint32(rows),
                      C.c_uint32(columns), C.c_uint32(block), C.c_int(scale_type))
    return out


def group_routes(ids, experts):
    ids = np.ascontiguousarray(ids, np.uint32)
    tokens, top_k = ids.shape
    offsets = np.empty(experts + 1, np.uint32)
    toks = np.empty(tokens * top_k, np.uint32)
    slots = np.empty(tokens * top_k, np.uint32)
    lib().k3o_group_routes(_p(offsets), _p(toks), _p(slots), _p(ids), C.c_uint32(tokens),
                           C.c_uint32(top_k), C.c_uint32(experts))
    return offsets, toks, slots


class _Layer(C.Structure):
    _fields_ = [
        ("hidden", C.c_uint32), ("expert_hidden", C.c_uint32), ("experts", C.c_uint32),
        ("top_k", C.c_uint32), ("shared_hidden", C.c_uint32), ("q8_block", C.c_uint32),
        ("q8_scale_type", C.c_int), ("activation", C.c_int),
        ("beta", C.c_float), ("linear_beta", C.c_float), ("route_scale", C.c_float),
        ("router_weight", C.c_void_p), ("router_bias", C.c_void_p),
        ("w1_packed", C.c_void_p), ("w1_scales", C.c_void_p),
        ("w3_packed", C.c_void_p), ("w3_scales", C.c_void_p),
        ("w2_packed", C.c_void_p), ("w2_scales", C.c_void_p),
        ("shared_gate_q", C.c_void_p), ("shared_gate_s", C.c_void_p),
        ("shared_up_q", C.c_void_p), ("shared_up_s", C.c_void_p),
        ("shared_down_q", C.c_void_p), ("shared_down_s", C.c_void_p),
    ]


def moe_layer(weights: dict, x: np.ndarray, expert_subset: int = 0):
    """Run one routed-MoE layer.  ``weights`` is the dict produced by
    ``moonshine_b200.synth.make_layer`` (numpy arrays plus scalar config).
    Returns (out bf16 [T,d], ids [T,k], route weights [T,k], logits [T,E], products)."""
    cfg = weights["config"]
    d, e, k = cfg["hidden"], cfg["experts"], cfg["top_k"]
    x = _u16(x).reshape(-1, d)
    t = x.shape[0]
    keep = []

    def ptr(name):
        a = weights.get(name)
        if a is None:
            return None
        a = np.ascontiguousarray(a)
        keep.append(a)
        return a.ctypes.data

    layer = _Layer(
        hidden=d, expert_hidden=cfg["expert_hidden"], experts=e, top_k=k,
        shared_hidden=cfg["shared_hidden"], q8_block=cfg["q8_block"],
        q8_scale_type=cfg["q8_scale_type"], activation=cfg["activation"],
        beta=cfg["beta"], linear_beta=cfg["linear_beta"], route_scale=cfg["route_scale"],
        router_weight=ptr("router_weight"), router_bias=ptr("router_bias"),
        w1_packed=ptr("w1_packed"), w1_scales=ptr("w1_scales"),
        w3_packed=ptr("w3_packed"), w3_scales=ptr("w3_scales"),
        w2_packed=ptr("w2_packed"), w2_scales=ptr("w2_scales"),
        shared_gate_q=ptr("shared_gate_q"), shared_gate_s=ptr("shared_gate_s"),
        shared_up_q=ptr("shared_up_q"), shared_up_s=ptr("shared_up_s"),
        shared_down_q=ptr("shared_down_q"), shared_down_s=ptr("shared_down_s"),
    )
    out = np.empty((t, d), np.uint16)
    ids = np.empty((t, k), np.uint32)
    w = np.empty((t, k), np.float32)
    logits = np.empty((t, e), np.float32)
    products = lib().k3o_moe_layer(_p(out), _p(ids), _p(w), _p(logits), C.byref(layer), _p(x),
                                   C.c_uint32(t), C.c_uint32(expert_subset))
    return out, ids, w, logits, int(products)


def synth_bytes(key: int, count: int, low: int = 0, span: int = 256, first: int = 0) -> np.ndarray:
    """The seeded byte stream ``synth.bytes_uniform(key, count, low, span, first)``,
    generated in C (whole experts of the full-size layers in milliseconds)."""
    assert first % 8 == 0
    out = np.empty(count, np.uint8)
    lib().k3o_synth_bytes(_p(out), C.c_uint64(count), C.c_uint64(key), C.c_uint64(first),
                          C.c_uint32(low), C.c_uint32(span))
    return out


def expert_tensors(cfg: dict, seed: int, expert: int) -> dict:
    """The six tensors of one expert of a synthetic layer, generated on the host from
    the layer's seeded streams (equal to the slices of ``synth.make_layer``)."""
    from moonshine_b200 import synth
    out = {}
    for name, (tp, ts, rows, cols) in synth.expert_tensor_specs(cfg).items():
        per_p, per_s = rows * cols // 2, rows * cols // 32
        out[name + "_packed"] = synth_bytes(synth.stream_key(seed, tp), per_p, first=expert * per_p
                                            ).reshape(rows, cols // 2)
        out[name + "_scales"] = synth_bytes(synth.stream_key(seed, ts), per_s, cfg["scale_low"],
                                            cfg["scale_span"], first=expert * per_s).reshape(rows, cols // 32)
    return out


def moe_layer_tokens(cfg: dict, seed: int, x: np.ndarray, weights: dict | None = None):
    """The layer's answer for a few token rows ``x`` [n, d] of a synthetic layer too large
    to hold on the host: only the experts those tokens select are generated.  Every
    operator is the one ``moe_layer`` uses, in the same order, so the result equals the
    rows ``moe_layer`` would give.  ``weights`` = ``synth.make_layer(cfg, seed, experts=False)``.
    Returns (out bf16 [n, d], ids, route weights, logits)."""
    from moonshine_b200 import synth
    if weights is None:
        weights = synth.make_layer(cfg, seed, experts=False)
    d, i, e, k, s = cfg["hidden"], cfg["expert_hidden"], cfg["experts"], cfg["top_k"], cfg["shared_hidden"]
    x = _u16(x).reshape(-1, d)
    n = x.shape[0]
    logits = bf16_gemm(weights["router_weight"], x, e, d)
    ids, wts = router_topk(logits, weights["router_bias"], k, cfg["route_scale"])
    offsets, toks, slots = group_routes(ids, e)
    outputs = np.zeros((n * k, d), np.uint16)
    for ex in np.unique(ids):
        lo, hi = int(offsets[ex]), int(offsets[ex + 1])
        t = expert_tensors(cfg, seed, int(ex))
        rows = x[toks[lo:hi]]
        gate = mxfp4_gemm(t["w1_packed"], t["w1_scales"], rows, i, d)
        up = mxfp4_gemm(t["w3_packed"], t["w3_scales"], rows, i, d)
        act = activation(gate, up, cfg["activation"], cfg["beta"], cfg["linear_beta"])
        outputs[slots[lo:hi]] = mxfp4_gemm(t["w2_packed"], t["w2_scales"], act, d, i)
    out = weighted_sum(outputs, wts, n, k, d)
    if s:
        q, st = cfg["q8_block"], cfg["q8_scale_type"]
        sg = q8_gemm(weights["shared_gate_q"], weights["shared_gate_s"], x, s, d, q, st)
        su = q8_gemm(weights["shared_up_q"], weights["shared_up_s"], x, s, d, q, st)
        sa = activation(sg, su, cfg["activation"], cfg["beta"], cfg["linear_beta"])
        so = q8_gemm(weights["shared_down_q"], weights["shared_down_s"], sa, d, s, q, st)
        out = add(out, so)
    return out, ids, wts, logits


class XorShift:
    """The reference tests' xorshift32 stream: ``unit(n)`` in [0,1),
    ``symmetric(n, scale)`` = (unit*2-1)*scale, float32 arithmetic as in
    tests/test_k3_rocm_components.cu:32-42."""

    def __init__(self, seed: int):
        self.state = C.c_uint32(seed)

    def unit(self, n: int) -> np.ndarray:
        out = np.empty(n, np.float32)
        lib().k3o_xorshift_unit(C.byref(self.state), _p(out), C.c_uint64(n))
        return out

    def symmetric(self, n: int, scale: float) -> np.ndarray:
        u = self.unit(n)
        return ((u * np.float32(2.0)) - np.float32(1.0)) * np.float32(scale)
