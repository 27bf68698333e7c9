/*
 * Dispatch wrappers over a resident static weight: BF16 or Q8-128 projection,
 * one vector or a batch.
 *
 * Replaces k3_static_weight_gemv_bf16 / k3_static_weight_gemm_bf16
 * (k3_static_store.cu:315-369, declared k3_static_store.h:73-82), which the
 * engine calls for routed_expert_down_proj, routed_expert_up_proj and the shared
 * expert's projections (k3_engine.cu:1668-1689, 1860).  Same names, argument
 * meaning and error behaviour: false for a null argument, a tensor that is not
 * a two-dimensional BF16 matrix, a dimension above 2^32-1 or a weight kind other
 * than BF16 / Q8-128; otherwise the result of the operator the kind selects
 * (k3_rocm_q8_128_gemv/gemm_bf16 or k3_rocm_bf16_gemv/gemm_bf16, k3_moe_ops.h).
 *
 * The two structs repeat the reference's layouts field for field
 * (k3_safetensors.h:14-29, k3_static_store.h:14-26), so a weight table built by
 * the reference's loader can be passed unchanged; the loader itself (SafeTensors
 * directory, quantisation at load) is outside this library.
 */
#ifndef K3_STATIC_WEIGHT_H
#define K3_STATIC_WEIGHT_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef K3_ST_MAX_DIMS
#define K3_ST_MAX_DIMS 8

typedef enum {
    K3_ST_DTYPE_UNKNOWN = 0,
    K3_ST_DTYPE_BF16,
    K3_ST_DTYPE_F32,
    K3_ST_DTYPE_U8,
} k3_st_dtype;

typedef struct {
    char        *name;
    uint64_t     physical_offset;
    uint64_t     byte_length;
    uint64_t     shape[K3_ST_MAX_DIMS];
    uint16_t     shard;
    uint8_t      ndim;
    k3_st_dtype  dtype;
} k3_st_tensor;
#endif

typedef enum {
    K3_STATIC_WEIGHT_RAW = 0,
    K3_STATIC_WEIGHT_BF16,
    K3_STATIC_WEIGHT_Q8_128,
} k3_static_weight_kind;

typedef struct {
    const k3_st_tensor    *tensor;          /* shape [rows, columns], dtype BF16 (the source type) */
    void                  *data;            /* device: bf16 [rows, columns] or int8 [rows, columns] */
    void                  *scales;          /* device: f32 [rows, columns/128] for Q8-128, else unused */
    uint64_t               resident_bytes;
    k3_static_weight_kind  kind;
} k3_static_weight;

/* output bf16 [rows] = W * input bf16 [columns] */
bool k3_static_weight_gemv_bf16(const k3_static_weight *weight, void *output,
                                const void *input, void *stream);

/* output bf16 [vector_count, rows] = input bf16 [vector_count, columns] * W^T */
bool k3_static_weight_gemm_bf16(const k3_static_weight *weight, void *output,
                                const void *input, uint32_t vector_count,
                                void *stream);

#ifdef __cplusplus
}
#endif
#endif
