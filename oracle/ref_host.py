"""ctypes front end of the reference's own host-side checking functions.

TEST INFRASTRUCTURE ONLY.  ``oracle/ref_host_wrap.cpp`` compiles the functions
the reference keeps inside its test programs (cut from the reference tree at
build time, never stored here) into ``oracle/_ref/libk3ref_host.so``.  This
module loads that library when it exists; ``available()`` says whether it does.
Machines without the reference tree use the vectors recorded from it under
``tests/golden/ref_host.npz`` instead.

bf16 tensors are ``numpy.uint16`` arrays holding the raw bit patterns.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIBS = {True: os.path.join(_HERE, "_ref", "libk3ref_host.so"),
         False: os.path.join(_HERE, "_ref", "libk3ref_host_unfused.so")}
_loaded = {}


def build(reference_tree: str) -> str:
    """Cut and compile (needs the reference tree); returns the fused library's path."""
    subprocess.run(["make", "-s", "-C", _HERE, "ref_host", "REF=" + reference_tree], check=True,
                   stdout=subprocess.DEVNULL)
    return _LIBS[True]


def available() -> bool:
    return all(os.path.exists(p) for p in _LIBS.values())


def lib(fused: bool = True) -> C.CDLL:
    if fused not in _loaded:
        handle = C.CDLL(_LIBS[fused])
        for name in ("k3ref_latent", "k3ref_expert_hidden", "k3ref_expert_count", "k3ref_top_k",
                     "k3ref_q8_columns"):
            getattr(handle, name).restype = C.c_uint32
        handle.k3ref_q8_row.restype = C.c_uint16
        handle.k3ref_float_to_bf16.restype = C.c_uint16
        handle.k3ref_float_to_bf16.argtypes = [C.c_float]
        handle.k3ref_e8m0_to_float.restype = C.c_float
        handle.k3ref_e8m0_to_float.argtypes = [C.c_uint8]
        handle.k3ref_e2m1_to_float.restype = C.c_float
        handle.k3ref_e2m1_to_float.argtypes = [C.c_uint8]
        _loaded[fused] = handle
    return _loaded[fused]


def _p(a):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    a = np.ascontiguousarray(a)
    assert a.dtype == dtype, (a.dtype, dtype)
    return a


def shape() -> dict:
    h = lib()
    return dict(latent=h.k3ref_latent(), expert_hidden=h.k3ref_expert_hidden(),
                experts=h.k3ref_expert_count(), top_k=h.k3ref_top_k(), q8_columns=h.k3ref_q8_columns())


def float_to_bf16(values, fused=True) -> np.ndarray:
    values = np.ascontiguousarray(values, np.float32).ravel()
    h = lib(fused)
    return np.array([h.k3ref_float_to_bf16(float(v)) for v in values], np.uint16)


def e8m0_table(fused=True) -> np.ndarray:
    h = lib(fused)
    return np.array([h.k3ref_e8m0_to_float(b) for b in range(256)], np.float32)


def e2m1_table(fused=True) -> np.ndarray:
    h = lib(fused)
    return np.array([h.k3ref_e2m1_to_float(n) for n in range(16)], np.float32)


def bf16_gemv(weights, x, rows, columns, fused=True):
    """reference_bf16_gemv: (f32 [rows], bf16 [rows])."""
    w, x = _c(weights, np.uint16), _c(x, np.uint16)
    out32, out16 = np.empty(rows, np.float32), np.empty(rows, np.uint16)
    lib(fused).k3ref_bf16_gemv(_p(out32), _p(out16), _p(w), _p(x), C.c_uint32(rows), C.c_uint32(columns))
    return out32, out16


def mxfp4_gemv(packed, scales, x, rows, columns, fused=True):
    p, s, x = _c(packed, np.uint8), _c(scales, np.uint8), _c(x, np.uint16)
    out = np.empty(rows, np.uint16)
    lib(fused).k3ref_mxfp4_gemv(_p(out), _p(p), _p(s), _p(x), C.c_uint32(rows), C.c_uint32(columns))
    return out


def situ(gate, up, fused=True):
    g, u = _c(gate, np.uint16), _c(up, np.uint16)
    out = np.empty_like(g)
    lib(fused).k3ref_situ(_p(out), _p(g), _p(u), C.c_uint32(g.size))
    return out


def rms_norm(x, weight, epsilon=1e-5, fused=True):
    x, w = _c(x, np.uint16), _c(weight, np.uint16)
    out = np.empty_like(x)
    lib(fused).k3ref_rms_norm(_p(out), _p(x), _p(w), C.c_uint32(x.size), C.c_float(epsilon))
    return out


def router(logits, bias, fused=True):
    """reference_router on one row of 896 logits: (ids [16], weights [16], unscaled)."""
    sh = shape()
    logits, bias = _c(logits, np.float32), _c(bias, np.float32)
    assert logits.size == sh["experts"] and bias.size == sh["experts"]
    ids, w = np.empty(sh["top_k"], np.uint32), np.empty(sh["top_k"], np.float32)
    lib(fused).k3ref_router(_p(ids), _p(w), _p(logits), _p(bias))
    return ids, w


def expert_accumulate(accumulator, weight, tensors, latent, fused=True):
    """accumulator += weight * expert(latent) at the reference's real shape;
    tensors = (w1.packed, w1.scale, w2.packed, w2.scale, w3.packed, w3.scale).
    Returns the expert's bf16 output row; the accumulator is updated in place."""
    sh = shape()
    acc = _c(accumulator, np.float32)
    keep = [_c(t, np.uint8) for t in tensors]
    table = (C.c_void_p * 6)(*[t.ctypes.data for t in keep])
    out = np.empty(sh["latent"], np.uint16)
    lib(fused).k3ref_expert_accumulate(_p(acc), C.c_float(weight), table, _p(_c(latent, np.uint16)), _p(out))
    return out


def q8_row(quantized, scales, x, fused=True) -> int:
    q, s, x = _c(quantized, np.int8), _c(scales, np.float32), _c(x, np.uint16)
    return int(lib(fused).k3ref_q8_row(_p(q), _p(s), _p(x)))


def mxfp4_f64(packed, scales, x, rows, columns, fused=True):
    p, s = _c(packed, np.uint8), _c(scales, np.uint8)
    x = _c(x, np.uint16).reshape(-1, columns)
    out = np.empty((x.shape[0], rows), np.float64)
    lib(fused).k3ref_mxfp4_f64(_p(out), _p(p), _p(s), _p(x), C.c_uint32(x.shape[0]), C.c_uint32(rows),
                               C.c_uint32(columns))
    return out
