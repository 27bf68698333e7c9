/*
 * C operator interface of the routed-MoE path (CUDA, sm_100a).
 *
 * Part 1 re-exports, with unchanged names, signatures and error behaviour, the
 * operator entry points that the reference engine's MoE section calls
 * (k3_rocm_ops.h of the reference; call sites k3_engine.cu:1032-1066,
 * 1554-1563, 1668-1689, 1851-1897 and k3_engine_prefill.inc:938-997,
 * 1448-1460, 1525-1551, 1575-1609).  A build of that engine for CUDA links
 * against this library instead of its own operator file for these symbols.
 *
 * Conventions (reference k3_rocm_ops.h:14-19): every tensor pointer is a
 * caller-owned device pointer to contiguous storage; BF16 unless stated;
 * `stream` is a cudaStream_t passed as void *, NULL selects the legacy default
 * stream; functions never allocate, free or synchronise; they return false on
 * an invalid argument or a launch error and true otherwise, with execution
 * asynchronous to the host.  The functions keep no state and may be called
 * concurrently on different streams.
 *
 * Part 2 adds generalised forms (activation kind, Q8 block size and scale
 * type) that the benchmark's synthetic layer needs.  They have no counterpart
 * in the reference and follow the same conventions.
 */
#ifndef K3_MOE_OPS_H
#define K3_MOE_OPS_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ Part 1 */

/* SiTU activation beta*tanh(g/beta)*sigmoid(g) * linear_beta*tanh(u/linear_beta).
 * Replaces k3_rocm_ops.h:20-26 (kernel k3_rocm_ops.cu:66-83). */
bool k3_rocm_situ_bf16(void *output, const void *gate, const void *up,
                       uint64_t element_count, float beta, float linear_beta,
                       void *stream);

/* MXFP4 matrix-vector product: packed [rows, columns/2] (even column = low
 * nibble, E2M1), scales [rows, columns/32] (E8M0); packed needs only 8-byte
 * alignment.  Replaces k3_rocm_ops.h:45-51 (kernel k3_rocm_ops.cu:225-273). */
bool k3_rocm_mxfp4_gemv_bf16(void *output, const void *packed,
                             const void *scales, const void *input,
                             uint32_t rows, uint32_t columns, void *stream);

/* Batch form: input [vector_count, columns] -> output [vector_count, rows].
 * Each input row is reduced exactly as by the single-row call.
 * Replaces k3_rocm_ops.h:58-65. */
bool k3_rocm_mxfp4_gemm_bf16(void *output, const void *packed,
                             const void *scales, const void *input,
                             uint32_t vector_count, uint32_t rows,
                             uint32_t columns, void *stream);

/* batch_tile must be 16, 32 or 64; results do not depend on it.
 * Replaces k3_rocm_ops.h:71-80. */
bool k3_rocm_mxfp4_gemm_tiled_bf16(void *output, const void *packed,
                                   const void *scales, const void *input,
                                   uint32_t vector_count, uint32_t rows,
                                   uint32_t columns, uint32_t batch_tile,
                                   void *stream);

/* Dense BF16 products with BF16 output.  Replace k3_rocm_ops.h:82-105. */
bool k3_rocm_bf16_gemv_bf16(void *output, const void *weights,
                            const void *input, uint32_t rows,
                            uint32_t columns, void *stream);
bool k3_rocm_bf16_gemm_tiled_bf16(void *output, const void *weights,
                                  const void *input, uint32_t vector_count,
                                  uint32_t rows, uint32_t columns,
                                  uint32_t batch_tile, void *stream);
bool k3_rocm_bf16_gemm_bf16(void *output, const void *weights,
                            const void *input, uint32_t vector_count,
                            uint32_t rows, uint32_t columns, void *stream);

/* Dense BF16 products with F32 output (router logits).
 * Replace k3_rocm_ops.h:107-130 (kernels k3_rocm_ops.cu:359-425, 512-661). */
bool k3_rocm_bf16_gemv_f32(void *output, const void *weights,
                           const void *input, uint32_t rows, uint32_t columns,
                           void *stream);
bool k3_rocm_bf16_gemm_f32(void *output, const void *weights,
                           const void *input, uint32_t vector_count,
                           uint32_t rows, uint32_t columns, void *stream);
bool k3_rocm_bf16_gemm_tiled_f32(void *output, const void *weights,
                                 const void *input, uint32_t vector_count,
                                 uint32_t rows, uint32_t columns,
                                 uint32_t batch_tile, void *stream);

/* Q8-128: int8 [rows, columns] + F32 scale per 128 columns, symmetric.
 * Replace k3_rocm_ops.h:138-182 (kernels k3_rocm_ops.cu:663-835). */
bool k3_rocm_bf16_quantize_q8_128(void *quantized, void *scales,
                                  const void *weights, uint32_t rows,
                                  uint32_t columns, void *stream);
bool k3_rocm_q8_128_dequantize_bf16(void *weights, const void *quantized,
                                    const void *scales, uint32_t rows,
                                    uint32_t columns, void *stream);
bool k3_rocm_q8_128_gemv_bf16(void *output, const void *quantized,
                              const void *scales, const void *input,
                              uint32_t rows, uint32_t columns, void *stream);
bool k3_rocm_q8_128_gemm_bf16(void *output, const void *quantized,
                              const void *scales, const void *input,
                              uint32_t vector_count, uint32_t rows,
                              uint32_t columns, void *stream);
bool k3_rocm_q8_128_gemm_tiled_bf16(void *output, const void *quantized,
                                    const void *scales, const void *input,
                                    uint32_t vector_count, uint32_t rows,
                                    uint32_t columns, uint32_t batch_tile,
                                    void *stream);

/* RMSNorm with BF16 weight.  Replaces k3_rocm_ops.h:301-307
 * (kernel k3_rocm_ops.cu:837-867). */
bool k3_rocm_rms_norm_bf16(void *output, const void *input, const void *weight,
                           uint32_t vector_count, uint32_t hidden_size,
                           float epsilon, void *stream);

/* Router: sigmoid(logits), top_k by score + bias (descending, lower expert id
 * wins ties), weights = raw score / (1e-20 + sum of selected raw scores) *
 * scaling_factor.  ids are uint32, weights F32; both may alias mapped host
 * memory.  expert_count <= 1024, top_k <= 32.
 * Replace k3_rocm_ops.h:383-401 (kernel k3_rocm_ops.cu:1361-1450). */
bool k3_rocm_router_topk_f32(void *expert_ids, void *expert_weights,
                             const void *logits, const void *correction_bias,
                             uint32_t expert_count, uint32_t top_k,
                             float scaling_factor, void *stream);
bool k3_rocm_router_topk_f32_batch(void *expert_ids, void *expert_weights,
                                   const void *logits,
                                   const void *correction_bias,
                                   uint32_t vector_count, uint32_t expert_count,
                                   uint32_t top_k, float scaling_factor,
                                   void *stream);

/* out[t,:] = bf16(sum_r weights[t,r] * vectors[t,r,:]), r ascending.
 * Replace k3_rocm_ops.h:403-417 (kernel k3_rocm_ops.cu:1452-1474). */
bool k3_rocm_weighted_sum_bf16(void *output, const void *vectors,
                               const void *weights, uint32_t vector_count,
                               uint32_t hidden_size, void *stream);
bool k3_rocm_weighted_sum_bf16_batch(void *output, const void *vectors,
                                     const void *weights, uint32_t token_count,
                                     uint32_t vector_count,
                                     uint32_t hidden_size, void *stream);

/* Row gather out[i,:] = in[row_ids[i],:] and scatter out[row_ids[i],:] =
 * in[i,:]; row_ids are uint32.  Replace k3_rocm_ops.h:419-433
 * (kernel k3_rocm_ops.cu:1476-1497). */
bool k3_rocm_gather_rows_bf16(void *output, const void *input,
                              const void *row_ids, uint32_t row_count,
                              uint32_t row_size, void *stream);
bool k3_rocm_scatter_rows_bf16(void *output, const void *input,
                               const void *row_ids, uint32_t row_count,
                               uint32_t row_size, void *stream);

/* out = bf16(float(left) + float(right)).  Replaces k3_rocm_ops.h:435-439
 * (kernel k3_rocm_ops.cu:1499-1510). */
bool k3_rocm_add_bf16(void *output, const void *left, const void *right,
                      uint64_t element_count, void *stream);

/* ------------------------------------------------------------------ Part 2 */

enum { K3_MOE_ACT_SITU = 0, K3_MOE_ACT_SWIGLU = 1 };
enum { K3_MOE_Q8_SCALE_F32 = 0, K3_MOE_Q8_SCALE_F16 = 1 };

/* Activation with a selectable kind: SiTU as above, or SwiGLU
 * g*sigmoid(g)*u (beta arguments ignored). */
bool k3_moe_activation_bf16(void *output, const void *gate, const void *up,
                            uint64_t element_count, int activation, float beta,
                            float linear_beta, void *stream);

/* Q8 with a selectable block (multiple of 8 dividing columns) and scale type. */
bool k3_moe_q8_quantize(void *quantized, void *scales, const void *weights,
                        uint32_t rows, uint32_t columns, uint32_t block,
                        int scale_type, void *stream);
bool k3_moe_q8_gemm_bf16(void *output, const void *quantized,
                         const void *scales, const void *input,
                         uint32_t vector_count, uint32_t rows, uint32_t columns,
                         uint32_t block, int scale_type, void *stream);

#ifdef __cplusplus
}
#endif
#endif
