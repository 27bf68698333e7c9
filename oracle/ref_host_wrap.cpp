/*
 * C entry points around the reference's own host-side checking functions.
 * TEST INFRASTRUCTURE: a second checker beside k3_oracle.c, never linked into
 * the product library.
 *
 * The reference keeps its CPU restatements of the MoE operators as static
 * functions (and two loop bodies) inside HIP test programs.  Apart from the
 * `hip_bfloat16` type they are plain C.  `make ref_host REF=<reference tree>`
 * cuts these line ranges out of the tree into oracle/_ref/<name>.inc (nothing
 * of the reference is stored in this repository) and compiles this file, which
 * includes them unchanged:
 *
 *   smoke_enum.inc   tests/test_k3_moe_smoke.cu:35-46    shape constants
 *   smoke_host.inc   tests/test_k3_moe_smoke.cu:80-253   bf16 helpers, E8M0 / E2M1 decode,
 *                    reference_bf16_gemv, reference_mxfp4_gemv, reference_situ,
 *                    reference_rms_norm, reference_router
 *   smoke_expert.inc tests/test_k3_moe_smoke.cu:601-613  one expert (gate, up, SiTU, down) and
 *                    its weighted accumulation, a loop body of main()
 *   q8_enum.inc      tests/test_k3_q8_projection.cu:31-38
 *   q8_row.inc       tests/test_k3_q8_projection.cu:50-76   q8_reference_row
 *   env_decode.inc   tests/test_k3_mxfp4_envelope.cu:114-130 host_e8m0/e2m1_to_float
 *   env_f64.inc      tests/test_k3_mxfp4_envelope.cu:265-278 fp64 row sum, a loop body
 *
 * The only piece supplied here is `hip_bfloat16`, whose source is ROCm's and
 * not in the reference tree: a 16-bit storage type, float -> bf16 by
 * round-to-nearest-even with NaN kept quiet, bf16 -> float by a 16-bit shift.
 *
 * Built twice: with -ffp-contract=fast (a multiply feeding an add becomes one
 * fused operation, as the reference's -ffast-math build does on FMA hardware;
 * no other value-changing option is used because none of them is pinned by
 * the reference) and with -ffp-contract=off.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

struct hip_bfloat16 {
    uint16_t data;
    hip_bfloat16() = default;
    explicit hip_bfloat16(float value) {
        uint32_t bits;
        memcpy(&bits, &value, sizeof(bits));
        if ((bits & 0x7fffffffu) > 0x7f800000u) {
            data = (uint16_t)((bits >> 16) | 0x0040u);
        } else {
            bits += 0x7fffu + ((bits >> 16) & 1u);
            data = (uint16_t)(bits >> 16);
        }
    }
    operator float() const {
        uint32_t bits = (uint32_t)data << 16;
        float value;
        memcpy(&value, &bits, sizeof(value));
        return value;
    }
};
static_assert(sizeof(hip_bfloat16) == 2, "bf16 storage");

namespace smoke {
#include "_ref/smoke_enum.inc"
#include "_ref/smoke_host.inc"

/* The loop body at :601-613 names main()'s locals; they are parameters here. */
static void expert_accumulate(float *cpu_accumulator, const float *cpu_weights, uint32_t rank,
                              const uint8_t *const *host, const hip_bfloat16 *cpu_latent,
                              hip_bfloat16 *cpu_expert_gate, hip_bfloat16 *cpu_expert_up,
                              hip_bfloat16 *cpu_expert_activation, hip_bfloat16 *cpu_expert_output) {
#include "_ref/smoke_expert.inc"
}
}  // namespace smoke

namespace q8 {
#include "_ref/q8_enum.inc"
#include "_ref/q8_row.inc"
}  // namespace q8

namespace envelope {
static inline float bf16_to_float(hip_bfloat16 value) { return (float)value; }
#include "_ref/env_decode.inc"
static void f64_rows(double *output, const uint8_t *packed, const uint8_t *scales,
                     const hip_bfloat16 *input, uint32_t vectors, uint32_t rows, uint32_t columns) {
    for (uint32_t vector = 0u; vector < vectors; vector++) {
        for (uint32_t row = 0u; row < rows; row++) {
#include "_ref/env_f64.inc"
            output[(size_t)vector * rows + row] = reference;
        }
    }
}
}  // namespace envelope

extern "C" {

uint32_t k3ref_latent(void) { return smoke::K3_LATENT; }
uint32_t k3ref_expert_hidden(void) { return smoke::K3_EXPERT_HIDDEN; }
uint32_t k3ref_expert_count(void) { return smoke::K3_EXPERT_COUNT; }
uint32_t k3ref_top_k(void) { return smoke::K3_TOP_K; }
uint32_t k3ref_q8_columns(void) { return q8::K3_COLUMNS; }

uint16_t k3ref_float_to_bf16(float value) { return smoke::float_to_bf16(value).data; }
float k3ref_e8m0_to_float(uint8_t exponent) { return smoke::e8m0_to_float(exponent); }
float k3ref_e2m1_to_float(uint8_t nibble) { return smoke::e2m1_to_float(nibble); }

void k3ref_bf16_gemv(float *output_f32, uint16_t *output_bf16, const uint16_t *weights,
                     const uint16_t *input, uint32_t rows, uint32_t columns) {
    smoke::reference_bf16_gemv(output_f32, (hip_bfloat16 *)output_bf16, (const hip_bfloat16 *)weights,
                               (const hip_bfloat16 *)input, rows, columns);
}

void k3ref_mxfp4_gemv(uint16_t *output, const uint8_t *packed, const uint8_t *scales,
                      const uint16_t *input, uint32_t rows, uint32_t columns) {
    smoke::reference_mxfp4_gemv((hip_bfloat16 *)output, packed, scales, (const hip_bfloat16 *)input, rows,
                                columns);
}

void k3ref_situ(uint16_t *output, const uint16_t *gate, const uint16_t *up, uint32_t count) {
    smoke::reference_situ((hip_bfloat16 *)output, (const hip_bfloat16 *)gate, (const hip_bfloat16 *)up,
                          count);
}

void k3ref_rms_norm(uint16_t *output, const uint16_t *input, const uint16_t *weight, uint32_t count,
                    float epsilon) {
    smoke::reference_rms_norm((hip_bfloat16 *)output, (const hip_bfloat16 *)input,
                              (const hip_bfloat16 *)weight, count, epsilon);
}

/* 896 logits, 16 routes: the sizes are compiled into the reference function */
void k3ref_router(uint32_t *ids, float *weights, const float *logits, const float *bias) {
    smoke::reference_router(ids, weights, logits, bias);
}

/* One expert at the reference's real shape (latent 3584, expert hidden 3072):
 * accumulator[d] += weight * down(SiTU(gate(x), up(x)))[d].  tensors[] holds the six
 * tensors of an expert span in checkpoint order: w1.packed, w1.scale, w2.packed,
 * w2.scale, w3.packed, w3.scale.  expert_output receives the bf16 row before weighting. */
void k3ref_expert_accumulate(float *accumulator, float weight, const uint8_t *const *tensors,
                             const uint16_t *latent, uint16_t *expert_output) {
    hip_bfloat16 *gate = (hip_bfloat16 *)malloc(smoke::K3_EXPERT_HIDDEN * 2u);
    hip_bfloat16 *up = (hip_bfloat16 *)malloc(smoke::K3_EXPERT_HIDDEN * 2u);
    hip_bfloat16 *act = (hip_bfloat16 *)malloc(smoke::K3_EXPERT_HIDDEN * 2u);
    smoke::expert_accumulate(accumulator, &weight, 0u, tensors, (const hip_bfloat16 *)latent, gate, up, act,
                             (hip_bfloat16 *)expert_output);
    free(act);
    free(up);
    free(gate);
}

/* one output row of a Q8 projection with 7168 columns and one f32 scale per 128 */
uint16_t k3ref_q8_row(const int8_t *quantized, const float *scales, const uint16_t *input) {
    return q8::q8_reference_row(quantized, scales, (const hip_bfloat16 *)input).data;
}

void k3ref_mxfp4_f64(double *output, const uint8_t *packed, const uint8_t *scales, const uint16_t *input,
                     uint32_t vectors, uint32_t rows, uint32_t columns) {
    envelope::f64_rows(output, packed, scales, (const hip_bfloat16 *)input, vectors, rows, columns);
}

}  /* extern "C" */
