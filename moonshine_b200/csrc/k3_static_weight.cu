// k3_static_weight_gemv_bf16 / k3_static_weight_gemm_bf16: pick the operator the
// weight's kind asks for (k3_static_store.cu:315-369 of the reference).
#include "k3_moe_ops.h"
#include "k3_static_weight.h"

namespace {

bool matrix_shape(const k3_static_weight *weight, uint32_t *rows, uint32_t *columns) {
    if (!weight || !weight->tensor) return false;
    const k3_st_tensor *t = weight->tensor;
    if (t->dtype != K3_ST_DTYPE_BF16 || t->ndim != 2u || t->shape[0] > UINT32_MAX || t->shape[1] > UINT32_MAX)
        return false;
    *rows = (uint32_t)t->shape[0];
    *columns = (uint32_t)t->shape[1];
    return true;
}

}  // namespace

extern "C" bool k3_static_weight_gemv_bf16(const k3_static_weight *weight, void *output, const void *input,
                                           void *stream) {
    uint32_t rows = 0, columns = 0;
    if (!output || !input || !matrix_shape(weight, &rows, &columns)) return false;
    switch (weight->kind) {
    case K3_STATIC_WEIGHT_Q8_128:
        return k3_rocm_q8_128_gemv_bf16(output, weight->data, weight->scales, input, rows, columns, stream);
    case K3_STATIC_WEIGHT_BF16:
        return k3_rocm_bf16_gemv_bf16(output, weight->data, input, rows, columns, stream);
    default:
        return false;
    }
}

extern "C" bool k3_static_weight_gemm_bf16(const k3_static_weight *weight, void *output, const void *input,
                                           uint32_t vector_count, void *stream) {
    uint32_t rows = 0, columns = 0;
    if (!output || !input || vector_count == 0u || !matrix_shape(weight, &rows, &columns)) return false;
    switch (weight->kind) {
    case K3_STATIC_WEIGHT_Q8_128:
        return k3_rocm_q8_128_gemm_bf16(output, weight->data, weight->scales, input, vector_count, rows, columns,
                                        stream);
    case K3_STATIC_WEIGHT_BF16:
        return k3_rocm_bf16_gemm_bf16(output, weight->data, input, vector_count, rows, columns, stream);
    default:
        return false;
    }
}
