// Internal interface between the layer composition and the tensor-core
// (tcgen05) GEMM kernels.  Each function picks the tensor-core kernel when the
// shape, alignment and row count suit it and otherwise runs the exact-order
// SIMT kernel behind the legacy entry points.
#pragma once

#include "k3_moe_layer.h"

#include <cuda_runtime.h>
#include <stdint.h>

// logits f32 [tokens, rows] = x bf16 [tokens, cols] * W bf16 [rows, cols]^T
bool k3_grouped_dense_bf16_f32(void *out, const void *weights, const void *x, uint32_t tokens,
                               uint32_t rows, uint32_t cols, void *stream);

// out bf16 [tokens, rows] = x bf16 [tokens, cols] * dequant(q, scales)^T
bool k3_grouped_q8_bf16(void *out, const void *q, const void *scales, const void *x,
                        uint32_t tokens, uint32_t rows, uint32_t cols, uint32_t block,
                        int scale_type, void *stream);

// One Q8 projection as a plain bf16 tensor-core GEMM: the table is converted to bf16
// once into weight_scratch (rows * cols * 2 bytes).  False when the shape or the
// token count does not suit the path (the caller then uses k3_grouped_q8_bf16).
bool k3_grouped_q8_dense_bf16(void *out, const void *q, const void *scales, const void *x,
                              uint32_t tokens, uint32_t rows, uint32_t cols, uint32_t block,
                              int scale_type, void *weight_scratch, cudaStream_t stream);

// Shared expert with its Q8 tables converted to bf16 once per call in `workspace`
// (k3_grouped_shared_workspace_bytes, 0 when the shape does not suit the path).
// act bf16 [tokens, S] is scratch, out bf16 [tokens, H].
size_t k3_grouped_shared_workspace_bytes(const k3_moe_layer_desc *desc, uint32_t tokens);
bool k3_grouped_shared_expert(const k3_moe_layer_desc *desc, void *out, void *act, const void *x,
                              uint32_t tokens, void *workspace, cudaStream_t stream);

// true when the grouped tensor-core path can run this layer / row count
bool k3_grouped_tc_supported(const k3_moe_layer_desc *desc, uint32_t rows);

// gate/up + activation and down over rows grouped by local expert
bool k3_grouped_tc_experts(const k3_moe_layer_desc *desc, void *rows_out, void *act,
                           const void *rows_in, const void *offsets, uint32_t rows, void *stream);

// One-token layer on persistent matrix-vector kernels (router, routing, expert
// gate/up/down, shared expert and the weighted combine into `out` bf16 [hidden],
// plus `residual` bf16 [hidden] when it is not null).
// All other buffers are caller-owned scratch.
bool k3_decode_supported(const k3_moe_layer_desc *desc);
// With combine == false the call ends after the expert rows (rows_out [top_k, hidden] in
// rank order, rows of experts outside this table untouched), ids, weights and the shared
// expert's output are complete on `stream`; `out` and `residual` are then unused.
bool k3_decode_layer(const k3_moe_layer_desc *desc, const void *x, void *logits, void *ids,
                     void *weights, void *sh_gate, void *sh_up, void *sh_act, void *sh_out,
                     void *act, void *rows_out, void *out, const void *residual, void *scratch,
                     size_t scratch_bytes, void *const *events, cudaStream_t stream,
                     bool combine = true);

// One token's routed experts with the routing given (k3_decode.cu).
bool k3_decode_experts_token(const k3_moe_layer_desc *desc, const void *x, const void *ids, void *act, void *rows_out,
                             void *scratch, size_t scratch_bytes, cudaStream_t stream);
// Block-scaled tensor-core expert products for one token (k3_decode_mx.cu).
bool k3_decode_mx_supported(const k3_moe_layer_desc *desc);
size_t k3_decode_mx_scratch_bytes(const k3_moe_layer_desc *desc);
// where the token's E2M1 terms live inside `scratch`: x_terms [8, hidden / 2] packed
// nibbles (one row per term) and x_sf [8, hidden / 32] block scales
void k3_decode_mx_vector_scratch(const k3_moe_layer_desc *desc, void *scratch, void **x_terms, void **x_sf);
// Expert products of one token from its E2M1 terms already in `scratch`;
// `between` (a CUDA event or null) is recorded after the one expert launch.
// With `tail` the down kernel's epilogue takes part in the layer's tail
// (k3_decode_tail.cuh): it counts an arrival per finished row and 32-column group in
// the words k3_decode_mx_tail_words() returns, and the arrival that completes
// `expected` forms the output columns.  Requires every selected expert in this table.
struct k3_decode_tail {
    void *out;                 // bf16 [hidden]
    const void *weights;       // f32 [top_k] on the device
    const void *shared;        // bf16 [hidden] or null
    const void *residual;      // bf16 [hidden] or null
    uint32_t epoch;            // unique per layer call (24 bits used)
    uint32_t expected;         // arrivals per 32-column group
};
void *k3_decode_mx_tail_words(const k3_moe_layer_desc *desc, void *scratch);
// f32 [2][1024] inside `scratch`: sigmoid scores and score + bias per expert (front kernel)
void *k3_decode_mx_route_words(const k3_moe_layer_desc *desc, void *scratch);
// 64 words inside `scratch` that must be zero when the expert kernel starts (its item
// counter and the per-rank arrival counts); the front kernel clears them
void *k3_decode_mx_control_words(const k3_moe_layer_desc *desc, void *scratch);
void *k3_decode_mx_front_done_word(const k3_moe_layer_desc *desc, void *scratch);
// With route_words (the scores and choices the front kernel's row tasks wrote) the kernel
// routes the token itself in its prologue and writes ids / weights [top_k]; it is then
// launched with programmatic stream serialization behind the front kernel.  With
// route_words null it reads ids (weights untouched).  front_blocks != 0: the front kernel
// counts its finished blocks in word kControlWords of the control words (cleared before it
// started) and the expert kernel waits for that count instead of for the whole chain of
// grids in front of it (k3_decode_mx_front_done_word()).
bool k3_decode_mx_experts(const k3_moe_layer_desc *desc, void *ids, void *weights, const void *route_words,
                          void *act, void *rows_out, void *scratch, void *between, const k3_decode_tail *tail,
                          uint32_t front_blocks,
                          cudaStream_t stream);
// Shared expert of one token as a persistent ring kernel on a few SMs (k3_decode_shared.cu).
bool k3_decode_shared_ring_supported(const k3_moe_layer_desc *desc);
uint32_t k3_decode_shared_ring_ctas();
// zero_word: a word cleared before the kernels queued behind may start (or null).
bool k3_decode_shared_ring(const k3_moe_layer_desc *desc, const void *x, void *sh_gate, void *sh_up, void *sh_out,
                           void *zero_word, cudaStream_t stream);
uint32_t k3_decode_shared_status();
bool k3_decode_shared_status_clear();
uint32_t k3_decode_mx_status();
uint32_t k3_decode_status();
uint32_t k3_dispatch_status();
bool k3_decode_status_clear();
bool k3_decode_mx_status_clear();
bool k3_dispatch_status_clear();
bool k3_grouped_mx_status_clear();
bool k3_status_words_clear();   // all of the above and the dense kernels' word   // 2: a dispatch saw an expert id >= experts

// Block-scaled tensor-core grouped expert products for many rows
// (k3_grouped_mx.cu).  `index` (u32 per row, or null) gathers rows_in, which then
// has source_rows rows; `act` may be null.
bool k3_grouped_mx_supported(const k3_moe_layer_desc *desc, uint32_t rows);
size_t k3_grouped_mx_workspace_bytes(const k3_moe_layer_desc *desc, uint32_t rows,
                                     uint32_t source_rows);
bool k3_grouped_mx_experts(const k3_moe_layer_desc *desc, void *rows_out, void *act,
                           const void *rows_in, const void *index, uint32_t source_rows,
                           const void *offsets, uint32_t rows, void *workspace,
                           cudaStream_t stream);
uint32_t k3_grouped_mx_status();
