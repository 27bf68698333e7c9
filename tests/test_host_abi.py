"""The C-ABI library loads without a GPU and exports every symbol the public
headers declare; argument validation runs on the host before any launch."""
import ctypes as C
import glob
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DECL = re.compile(r"^(?:bool|size_t|float|void|int|uint32_t|uint64_t|void \*|const char \*)\s*(k3_[a-z0-9_]+)\s*\(", re.M)


@pytest.fixture(scope="module")
def native():
    from moonshine_b200 import build, _native
    build.build()
    return _native


def declared_symbols():
    names = []
    for header in sorted(glob.glob(os.path.join(ROOT, "include", "*.h"))):
        names += DECL.findall(open(header).read())
    return names


def test_headers_declare_the_reference_symbols():
    names = set(declared_symbols())
    # the MoE subset of the reference operator interface (k3_rocm_ops.h)
    for required in [
        "k3_rocm_bf16_gemv_f32", "k3_rocm_bf16_gemm_f32", "k3_rocm_bf16_gemm_tiled_f32",
        "k3_rocm_router_topk_f32", "k3_rocm_router_topk_f32_batch", "k3_rocm_mxfp4_gemv_bf16",
        "k3_rocm_mxfp4_gemm_bf16", "k3_rocm_mxfp4_gemm_tiled_bf16", "k3_rocm_situ_bf16",
        "k3_rocm_q8_128_gemv_bf16", "k3_rocm_q8_128_gemm_bf16", "k3_rocm_q8_128_gemm_tiled_bf16",
        "k3_rocm_bf16_quantize_q8_128", "k3_rocm_gather_rows_bf16", "k3_rocm_scatter_rows_bf16",
        "k3_rocm_weighted_sum_bf16", "k3_rocm_weighted_sum_bf16_batch", "k3_rocm_rms_norm_bf16",
        "k3_rocm_add_bf16",
    ]:
        assert required in names, required


def test_library_exports_every_declared_symbol(native):
    handle = C.CDLL(native.LIB_PATH)
    declared = declared_symbols()
    assert len(declared) >= 35
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in include/ but not exported"
    for name in native.SIGNATURES:
        assert name in declared, f"{name} bound in python but not declared in include/"


def test_desc_struct_matches_header(native):
    text = open(os.path.join(ROOT, "include", "k3_moe_layer.h")).read()
    body = text[text.index("typedef struct k3_moe_layer_desc {"):text.index("} k3_moe_layer_desc;")]
    fields = re.findall(r"^\s+(?:const void \*|uint32_t\s+|int32_t\s+|float\s+)(\w+);", body, re.M)
    assert fields == [f[0] for f in native.LayerDesc._fields_]


def test_invalid_arguments_return_false_without_a_device(native):
    # error behaviour of the reference wrappers (k3_rocm_ops.cu:1637-1641, 2555-2560,
    # 2592-2596): null pointers, zero sizes and bad shapes return false before any launch
    lib = native.lib()
    p = 0x1000        # never dereferenced: every call below fails validation first
    assert lib.k3_rocm_mxfp4_gemv_bf16(None, p, p, p, 8, 64, None) is False
    assert lib.k3_rocm_mxfp4_gemv_bf16(p, p, p, p, 8, 48, None) is False          # cols % 32
    assert lib.k3_rocm_mxfp4_gemm_bf16(p, p, p, p, 65536, 8, 64, None) is False   # > 65535 rows
    assert lib.k3_rocm_mxfp4_gemm_tiled_bf16(p, p, p, p, 2, 8, 64, 24, None) is False
    assert lib.k3_rocm_q8_128_gemv_bf16(p, p, p, p, 8, 192, None) is False        # cols % 128
    assert lib.k3_rocm_bf16_gemm_f32(p, p, p, 0, 8, 64, None) is False
    assert lib.k3_rocm_router_topk_f32(p, p, p, p, 1025, 16, 1.0, None) is False
    assert lib.k3_rocm_router_topk_f32(p, p, p, p, 896, 33, 1.0, None) is False
    assert lib.k3_rocm_router_topk_f32(p, p, p, p, 8, 16, 1.0, None) is False     # k > experts
    assert lib.k3_rocm_router_topk_f32(p, p, p, p, 896, 16, 0.0, None) is False
    assert lib.k3_rocm_situ_bf16(p, p, p, 8, 0.0, 25.0, None) is False
    assert lib.k3_rocm_weighted_sum_bf16_batch(p, p, p, 65536, 16, 64, None) is False
    assert lib.k3_rocm_rms_norm_bf16(p, p, p, 1, 64, 0.0, None) is False
    assert lib.k3_rocm_add_bf16(p, p, None, 8, None) is False
    assert lib.k3_rocm_gather_rows_bf16(p, p, p, 0, 64, None) is False
    assert lib.k3_moe_layer_workspace_bytes(None, 4) == 0
    # k3_static_store.cu:315-369: null weight, null tensor, raw kind
    assert lib.k3_static_weight_gemv_bf16(None, p, p, None) is False
    empty = native.StaticWeight()
    assert lib.k3_static_weight_gemm_bf16(empty, p, p, 4, None) is False
    assert lib.k3_moe_selftest_bounded_wait(0, None, None) is False
    assert lib.k3_moe_phase_stats_add(None, None) is False
    assert lib.k3_moe_version().startswith(b"k3moe")
    # one token with host-given routing: null descriptor or pointers
    assert lib.k3_moe_experts_token_workspace_bytes(None) == 0
    assert lib.k3_moe_experts_token(None, p, p, p, p, p, 1 << 20, None) is False
    # tensor-pipe peak loop: N extent out of range, or not a multiple of 16
    assert lib.k3_moe_peak_launch_n(1, 8, 10, None, None) is False
    assert lib.k3_moe_peak_launch_n(1, 272, 10, None, None) is False
    assert lib.k3_moe_peak_launch_n(1, 40, 10, None, None) is False
    assert lib.k3_moe_peak_launch_n(3, 128, 10, None, None) is False
