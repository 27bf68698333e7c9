// Tensor-core GEMM paths (placeholder wiring: exact-order SIMT kernels).
#include "k3_grouped.h"
#include "k3_moe_ops.h"

bool k3_grouped_dense_bf16_f32(void *out, const void *weights, const void *x, uint32_t tokens,
                               uint32_t rows, uint32_t cols, void *stream) {
    return k3_rocm_bf16_gemm_f32(out, weights, x, tokens, rows, cols, stream);
}

bool k3_grouped_q8_bf16(void *out, const void *q, const void *scales, const void *x,
                        uint32_t tokens, uint32_t rows, uint32_t cols, uint32_t block,
                        int scale_type, void *stream) {
    return k3_moe_q8_gemm_bf16(out, q, scales, x, tokens, rows, cols, block, scale_type, stream);
}

bool k3_grouped_tc_supported(const k3_moe_layer_desc *, uint32_t) { return false; }

bool k3_grouped_tc_experts(const k3_moe_layer_desc *, void *, void *, const void *, const void *,
                           uint32_t, void *) {
    return false;
}
