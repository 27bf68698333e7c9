"""ctypes binding of the native library ``libk3moe.so`` (built in-tree by
``moonshine_b200.build``).  There is no fallback: a missing library raises."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libk3moe.so")

u32, u64, f32, i32, vp, sz = C.c_uint32, C.c_uint64, C.c_float, C.c_int, C.c_void_p, C.c_size_t


class LayerDesc(C.Structure):
    """Mirror of ``k3_moe_layer_desc`` (include/k3_moe_layer.h)."""
    _fields_ = [
        ("hidden", u32), ("expert_hidden", u32), ("expert_count", u32), ("top_k", u32),
        ("shared_hidden", u32), ("q8_block", u32), ("q8_scale_type", C.c_int32),
        ("activation", C.c_int32), ("beta", f32), ("linear_beta", f32), ("route_scale", f32),
        ("local_expert_first", u32), ("local_expert_count", u32),
        ("router_weight", vp), ("router_bias", vp),
        ("w1_packed", vp), ("w1_scales", vp), ("w3_packed", vp), ("w3_scales", vp),
        ("w2_packed", vp), ("w2_scales", vp),
        ("shared_gate_q", vp), ("shared_gate_s", vp), ("shared_up_q", vp), ("shared_up_s", vp),
        ("shared_down_q", vp), ("shared_down_s", vp),
    ]


_DP = C.POINTER(LayerDesc)


class LatentDesc(C.Structure):
    """Mirror of ``k3_moe_latent_desc`` (include/k3_moe_layer.h)."""
    _fields_ = [
        ("layer", LayerDesc), ("latent", u32), ("norm_epsilon", f32),
        ("down_q", vp), ("down_s", vp), ("norm_weight", vp), ("up_q", vp), ("up_s", vp),
    ]


_LP = C.POINTER(LatentDesc)


class PhaseStats(C.Structure):
    """Mirror of ``k3_moe_phase_stats`` (include/k3_moe_layer.h)."""
    _fields_ = [("router_seconds", C.c_double), ("routed_index_seconds", C.c_double),
                ("routed_expert_pipeline_seconds", C.c_double), ("moe_tail_seconds", C.c_double),
                ("shared_expert_seconds", C.c_double), ("layer_passes", C.c_uint64)]


class StTensor(C.Structure):
    """Mirror of ``k3_st_tensor`` (include/k3_static_weight.h)."""
    _fields_ = [("name", C.c_char_p), ("physical_offset", C.c_uint64), ("byte_length", C.c_uint64),
                ("shape", C.c_uint64 * 8), ("shard", C.c_uint16), ("ndim", C.c_uint8), ("dtype", C.c_int)]


class StaticWeight(C.Structure):
    """Mirror of ``k3_static_weight`` (include/k3_static_weight.h)."""
    _fields_ = [("tensor", C.POINTER(StTensor)), ("data", C.c_void_p), ("scales", C.c_void_p),
                ("resident_bytes", C.c_uint64), ("kind", C.c_int)]



class SlotAccess(C.Structure):
    """Mirror of ``k3_moe_slot_access`` (include/k3_moe_store.h)."""
    _fields_ = [("hit", C.c_bool), ("admit", C.c_bool), ("source_slot", u32), ("destination_slot", u32)]


class SlotStats(C.Structure):
    """Mirror of ``k3_moe_slot_stats`` (include/k3_moe_store.h)."""
    _fields_ = [("batches", u64), ("accesses", u64), ("hits", u64), ("misses", u64),
                ("admissions", u64), ("evictions", u64)]


u16 = C.c_uint16
_U16P, _U32P = C.POINTER(u16), C.POINTER(u32)

# name -> (restype, argtypes)
SIGNATURES = {
    # slot policy of the partially resident expert store (host code)
    "k3_moe_slot_cache_create": (C.c_bool, [C.POINTER(vp), u16, u16, C.c_char_p, sz]),
    "k3_moe_slot_cache_plan": (C.c_bool, [vp, u16, _U16P, u16, C.POINTER(SlotAccess), C.c_char_p, sz]),
    "k3_moe_slot_cache_commit": (C.c_bool, [vp, u16, C.c_char_p, sz]),
    "k3_moe_slot_cache_abort": (None, [vp, u16]),
    "k3_moe_slot_cache_slot_count": (u32, [vp]),
    "k3_moe_slot_cache_storage_bytes": (u64, [vp, u64]),
    "k3_moe_slot_cache_get_stats": (None, [vp, C.POINTER(SlotStats)]),
    "k3_moe_slot_cache_snapshot_layer": (C.c_bool, [vp, u16, _U16P, u16, _U16P, C.c_char_p, sz]),
    "k3_moe_slot_cache_reset": (C.c_bool, [vp, C.c_char_p, sz]),
    "k3_moe_slot_cache_invalidate_slots": (C.c_bool, [vp, u32, u32, C.c_char_p, sz]),
    "k3_moe_slot_cache_destroy": (None, [vp]),
    "k3_moe_slot_cache_replay_line": (C.c_bool, [vp, u16, _U16P, u16, _U32P, _U32P, C.c_char_p, sz]),
    # legacy operator interface
    "k3_rocm_situ_bf16": (C.c_bool, [vp, vp, vp, u64, f32, f32, vp]),
    "k3_rocm_mxfp4_gemv_bf16": (C.c_bool, [vp, vp, vp, vp, u32, u32, vp]),
    "k3_rocm_mxfp4_gemm_bf16": (C.c_bool, [vp, vp, vp, vp, u32, u32, u32, vp]),
    "k3_rocm_mxfp4_gemm_tiled_bf16": (C.c_bool, [vp, vp, vp, vp, u32, u32, u32, u32, vp]),
    "k3_rocm_bf16_gemv_bf16": (C.c_bool, [vp, vp, vp, u32, u32, vp]),
    "k3_rocm_bf16_gemm_tiled_bf16": (C.c_bool, [vp, vp, vp, u32, u32, u32, u32, vp]),
    "k3_rocm_bf16_gemm_bf16": (C.c_bool, [vp, vp, vp, u32, u32, u32, vp]),
    "k3_rocm_bf16_gemv_f32": (C.c_bool, [vp, vp, vp, u32, u32, vp]),
    "k3_rocm_bf16_gemm_f32": (C.c_bool, [vp, vp, vp, u32, u32, u32, vp]),
    "k3_rocm_bf16_gemm_tiled_f32": (C.c_bool, [vp, vp, vp, u32, u32, u32, u32, vp]),
    "k3_rocm_bf16_quantize_q8_128": (C.c_bool, [vp, vp, vp, u32, u32, vp]),
    "k3_rocm_q8_128_dequantize_bf16": (C.c_bool, [vp, vp, vp, u32, u32, vp]),
    "k3_rocm_q8_128_gemv_bf16": (C.c_bool, [vp, vp, vp, vp, u32, u32, vp]),
    "k3_rocm_q8_128_gemm_bf16": (C.c_bool, [vp, vp, vp, vp, u32, u32, u32, vp]),
    "k3_rocm_q8_128_gemm_tiled_bf16": (C.c_bool, [vp, vp, vp, vp, u32, u32, u32, u32, vp]),
    "k3_rocm_rms_norm_bf16": (C.c_bool, [vp, vp, vp, u32, u32, f32, vp]),
    "k3_rocm_router_topk_f32": (C.c_bool, [vp, vp, vp, vp, u32, u32, f32, vp]),
    "k3_rocm_router_topk_f32_batch": (C.c_bool, [vp, vp, vp, vp, u32, u32, u32, f32, vp]),
    "k3_rocm_weighted_sum_bf16": (C.c_bool, [vp, vp, vp, u32, u32, vp]),
    "k3_rocm_weighted_sum_bf16_batch": (C.c_bool, [vp, vp, vp, u32, u32, u32, vp]),
    "k3_rocm_gather_rows_bf16": (C.c_bool, [vp, vp, vp, u32, u32, vp]),
    "k3_rocm_scatter_rows_bf16": (C.c_bool, [vp, vp, vp, u32, u32, vp]),
    "k3_rocm_add_bf16": (C.c_bool, [vp, vp, vp, u64, vp]),
    # generalised operators
    "k3_moe_activation_bf16": (C.c_bool, [vp, vp, vp, u64, i32, f32, f32, vp]),
    "k3_moe_q8_quantize": (C.c_bool, [vp, vp, vp, u32, u32, u32, i32, vp]),
    "k3_moe_q8_gemm_bf16": (C.c_bool, [vp, vp, vp, vp, u32, u32, u32, u32, i32, vp]),
    # fused layer
    "k3_moe_store_admit": (C.c_bool, [_DP, u32, vp, C.POINTER(u64), vp]),
    "k3_moe_layer_workspace_bytes": (sz, [_DP, u32]),
    "k3_moe_dispatch_workspace_bytes": (sz, [u32, u32, u32]),
    "k3_moe_dispatch_build": (C.c_bool, [vp, vp, vp, vp, vp, u32, u32, u32, vp, sz, vp]),
    "k3_moe_dispatch_noalloc_max_routes": (sz, []),
    "k3_moe_dispatch_build_noalloc": (C.c_bool, [vp, vp, vp, vp, vp, u32, u32, u32, C.c_char_p, sz, vp]),
    "k3_moe_route": (C.c_bool, [_DP, vp, vp, vp, vp, u32, vp]),
    "k3_moe_experts_grouped": (C.c_bool, [_DP, vp, vp, vp, vp, u32, vp]),
    "k3_moe_experts_workspace_bytes": (sz, [_DP, u32, u32]),
    "k3_moe_experts_token_workspace_bytes": (sz, [_DP]),
    "k3_moe_experts_token": (C.c_bool, [_DP, vp, vp, vp, vp, vp, sz, vp]),
    "k3_moe_experts_grouped_ws": (C.c_bool, [_DP, vp, vp, vp, vp, u32, vp, u32, vp, sz, vp]),
    "k3_moe_shared_workspace_bytes": (sz, [_DP, u32]),
    "k3_moe_shared_expert_ws": (C.c_bool, [_DP, vp, vp, vp, u32, vp, sz, vp]),
    "k3_moe_shared_expert": (C.c_bool, [_DP, vp, vp, vp, vp, vp, u32, vp]),
    "k3_moe_combine": (C.c_bool, [vp, vp, vp, vp, vp, u32, u32, u32, vp]),
    "k3_moe_latent_workspace_bytes": (sz, [_LP, u32]),
    "k3_moe_latent_layer_forward": (C.c_bool, [_LP, vp, vp, u32, vp, sz, vp, vp, vp]),
    "k3_moe_combine_residual": (C.c_bool, [vp, vp, vp, vp, vp, vp, u32, u32, u32, vp]),
    "k3_moe_block_workspace_bytes": (sz, [_DP, u32]),
    "k3_moe_block_forward": (C.c_bool, [_DP, vp, vp, vp, f32, u32, vp, sz, vp]),
    "k3_moe_layer_forward": (C.c_bool, [_DP, vp, vp, u32, vp, sz, vp, vp, vp]),
    "k3_moe_layer_forward_events": (C.c_bool, [_DP, vp, vp, u32, vp, sz, C.POINTER(vp), vp]),
    "k3_moe_device_status": (u32, []),
    "k3_moe_peak_launch": (C.c_bool, [i32, u32, C.POINTER(C.c_double), vp]),
    "k3_moe_peak_launch_n": (C.c_bool, [i32, u32, u32, C.POINTER(C.c_double), vp]),
    "k3_moe_device_status_clear": (C.c_bool, []),
    "k3_moe_selftest_bounded_wait": (C.c_bool, [u32, vp, vp]),
    "k3_moe_phase_stats_add": (C.c_bool, [C.POINTER(PhaseStats), C.POINTER(vp)]),
    "k3_static_weight_gemv_bf16": (C.c_bool, [C.POINTER(StaticWeight), vp, vp, vp]),
    "k3_static_weight_gemm_bf16": (C.c_bool, [C.POINTER(StaticWeight), vp, vp, u32, vp]),
    "k3_moe_event_create": (vp, []),
    "k3_moe_event_destroy": (None, [vp]),
    "k3_moe_event_elapsed_ms": (f32, [vp, vp]),
    # expert parallel over NCCL
    "k3_moe_ep_unique_id": (C.c_bool, [vp, C.c_char_p, sz]),
    "k3_moe_ep_create": (C.c_bool, [C.POINTER(vp), vp, C.c_int, C.c_int, C.c_char_p, sz]),
    "k3_moe_ep_destroy": (None, [vp]),
    "k3_moe_ep_set_reduced_return": (C.c_bool, [vp, C.c_bool]),
    "k3_moe_ep_rank": (C.c_int, [vp]),
    "k3_moe_ep_world": (C.c_int, [vp]),
    "k3_moe_ep_plan": (C.c_bool, [_U32P, u32, u32, u32, _U32P, _U32P, _U32P, _U32P, _U32P, _U32P]),
    "k3_moe_ep_workspace_bytes": (sz, [vp, _DP, u32, u32]),
    "k3_moe_ep_layer_forward": (C.c_bool, [vp, _DP, vp, vp, u32, u32, vp, sz, vp, vp, C.c_char_p, sz, vp]),
    "k3_moe_ep_last_pass": (C.c_bool, [vp, C.POINTER(f32), C.POINTER(f32), _U32P]),
    "k3_moe_ep_decode_workspace_bytes": (sz, [vp, _DP]),
    "k3_moe_ep_decode": (C.c_bool, [vp, _DP, vp, vp, vp, vp, sz, vp]),
    "k3_moe_ep_decode_stack": (C.c_bool, [vp, C.POINTER(_DP), u32, vp, vp, vp, f32, vp, sz, vp]),
    "k3_synth_fill_bytes": (C.c_bool, [vp, u64, u64, u64, u32, u32, vp]),
    "k3_synth_fill_int8": (C.c_bool, [vp, u64, u64, u64, vp]),
    "k3_synth_fill_uniform": (C.c_bool, [vp, u64, u64, u64, f32, f32, i32, vp]),
    "k3_moe_version": (C.c_char_p, []),
}

_lib = None


def lib() -> C.CDLL:
    """Load the library and attach signatures.  Raises if it was not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: run `python -m moonshine_b200.build` "
                "(nvcc, sm_100a).  There is no CPU or PyTorch fallback.")
        handle = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)   # AttributeError if a symbol is missing
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib
