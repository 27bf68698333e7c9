"""The reference's C operator interface on torch tensors.

Every function of the native library is exposed under its C name with the same
argument order and the same ``bool`` result (``False`` = invalid argument or
launch error; nothing raises).  Pointer arguments accept a CUDA ``torch.Tensor``
(its ``data_ptr()`` is passed), an integer address, or ``None``.  The trailing
``stream`` argument defaults to the current torch CUDA stream.

Example (compare tests of the reference, tests/test_k3_rocm_components.cu):

    ok = ops.k3_rocm_mxfp4_gemv_bf16(out, packed, scales, x, rows, columns)
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _native


def _ptr(a):
    if a is None:
        return None
    if isinstance(a, C.c_void_p):          # an opaque handle returned through an out parameter
        return a.value
    if isinstance(a, torch.Tensor):
        if not a.is_contiguous():
            raise ValueError("operator arguments must be contiguous")
        return a.data_ptr()
    return int(a)


def current_stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _make(name, restype, argtypes):
    def call(*args, stream=None):
        fn = getattr(_native.lib(), name)
        has_stream = (len(argtypes) > 0 and argtypes[-1] is C.c_void_p
                      and not name.startswith(("k3_moe_event_", "k3_moe_device_status", "k3_moe_ep_destroy",
                                                   "k3_moe_ep_rank", "k3_moe_ep_world", "k3_moe_ep_set_reduced_return")))
        has_stream = has_stream and len(argtypes) > 0
        n_user = len(argtypes) - (1 if has_stream else 0)
        if len(args) == len(argtypes) and has_stream:      # stream passed positionally
            stream, args = args[-1], args[:-1]
        if len(args) != n_user:
            raise TypeError(f"{name} takes {n_user} arguments (+ stream), got {len(args)}")
        conv = []
        for a, t in zip(args, argtypes):
            if t is C.c_void_p:
                conv.append(_ptr(a))
            elif isinstance(t, type) and issubclass(t, C._Pointer) and isinstance(a, C.Structure):
                conv.append(C.byref(a))
            else:
                conv.append(a)
        if has_stream:
            conv.append(current_stream_ptr() if stream is None else _ptr(stream))
        return fn(*conv)

    call.__name__ = name
    call.__doc__ = f"ctypes call of ``{name}`` (see include/*.h for the contract)."
    return call


for _name, (_res, _args) in _native.SIGNATURES.items():
    globals()[_name] = _make(_name, _res, _args)

ACT_SITU, ACT_SWIGLU = 0, 1
Q8_F32, Q8_F16 = 0, 1
