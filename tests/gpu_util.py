"""Helpers of the GPU parity tests: numpy <-> device tensors and comparisons."""
import numpy as np
import torch

DEV = "cuda:0"


def dev(a):
    a = np.array(a, copy=True)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(DEV)
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).to(DEV)
    return torch.from_numpy(a).to(DEV)


def empty(shape, dtype):
    t = {np.uint16: torch.int16, np.uint32: torch.int32, np.float32: torch.float32,
         np.int8: torch.int8, np.uint8: torch.uint8, np.float16: torch.float16}[dtype]
    return torch.empty(shape, dtype=t, device=DEV)


def host(t, dtype=None):
    torch.cuda.synchronize()
    a = t.cpu().numpy()
    if dtype is np.uint16:
        return a.view(np.uint16)
    if dtype is np.uint32:
        return a.view(np.uint32)
    return a


def bf16_f32(a):
    return (np.ascontiguousarray(a, np.uint16).astype(np.uint32) << 16).view(np.float32)


def ulp_distance(a, b):
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, 0x8000 - (x & 0x7FFF), 0x8000 + x)
    return np.abs(key(np.asarray(a)) - key(np.asarray(b)))


def rel_l2(got_bits, want_bits):
    g = bf16_f32(got_bits).astype(np.float64)
    w = bf16_f32(want_bits).astype(np.float64)
    return float(np.sqrt(((g - w) ** 2).sum() / max((w ** 2).sum(), 1e-30)))


def check_mxfp4_envelope(got_bits, want_bits, ref_f64):
    """The reference's acceptance rule for a new MXFP4 reduction schedule
    (tests/test_k3_mxfp4_envelope.cu:304-341): at most one bf16 ULP from the
    other schedule, and within 0.25 abs or 1 % rel of the fp64 dot product.
    ULP distance is meaningless where a sum cancels to far below the typical
    magnitude, so there the absolute difference must stay under half a bf16 ULP
    of the root-mean-square output instead."""
    g = bf16_f32(got_bits).astype(np.float64)
    w = bf16_f32(want_bits).astype(np.float64)
    rms = float(np.sqrt((ref_f64 ** 2).mean()))
    close = (ulp_distance(got_bits, want_bits) <= 1) | (np.abs(g - w) <= rms * 2.0 ** -9)
    assert np.all(close)
    err = np.abs(g - ref_f64)
    assert np.all((err <= 0.25) | (err / np.maximum(np.abs(ref_f64), 1e-3) <= 0.01))
    assert np.all(np.isfinite(g))
