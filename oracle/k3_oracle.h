/*
 * CPU oracle for the routed-MoE path of the Moonshine Kimi-K3 engine.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the reference's
 * own host oracles and kernel arithmetic; it is linked by the tests, by the
 * smoke check and by the CPU-baseline leg of the benchmark, never by the
 * product library.
 *
 * Parity status: pinned to the reference's own code.  The reference's host-side
 * checking functions (plain C inside its test programs) are cut from the
 * reference tree and compiled by `make ref_host` (ref_host_wrap.cpp);
 * tests/test_oracle_vs_ref.py requires every operator here to equal them bit
 * for bit on seeded inputs, live where that library exists and everywhere
 * against the outputs recorded from it in tests/golden/ref_host.npz.  The
 * reference's model-free tests (tolerances, tie rules, reduction schedules,
 * fixed xorshift32 seeds) are replayed by tests/test_oracle_pins.py.  The pins
 * that need the 1.6 TB checkpoint are not reproducible here.
 *
 * Every function cites the reference file:line it follows (paths relative to
 * the reference tree).
 */
#ifndef K3_ORACLE_H
#define K3_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* K3O_ACT_SITU follows the kernel's expression (k3_rocm_ops.cu:66-83: bounded gate x
 * sigmoid x bounded up, the sigmoid formed as a reciprocal); K3O_ACT_SITU_HOST follows the
 * host check's (tests/test_k3_moe_smoke.cu:173-184: bounded gate divided by 1+exp(-g)).
 * The two differ by one bf16 ULP on a few values per million. */
enum { K3O_ACT_SITU = 0, K3O_ACT_SWIGLU = 1, K3O_ACT_SITU_HOST = 2 };
enum { K3O_Q8_SCALE_F32 = 0, K3O_Q8_SCALE_F16 = 1 };

/* bf16 <-> f32, round-to-nearest-even (the behaviour of hip_bfloat16(float)
 * used throughout k3_rocm_ops.cu:32-40). */
uint16_t k3o_bf16_from_float(float value);
float    k3o_bf16_to_float(uint16_t bits);
float    k3o_f16_to_float(uint16_t bits);

/* tests/test_k3_moe_smoke.cu:88-104 (same as k3_rocm_ops.cu:179-191). */
float k3o_e8m0_to_float(uint8_t exponent);
float k3o_e2m1_to_float(uint8_t nibble);

/* tests/test_k3_moe_smoke.cu:106-135: 256 strided lanes + binary tree.
 * output_f32 and/or output_bf16 may be NULL.  input is [vectors, columns],
 * outputs are [vectors, rows]. */
void k3o_bf16_gemm(float *output_f32, uint16_t *output_bf16,
                   const uint16_t *weights, const uint16_t *input,
                   uint32_t vectors, uint32_t rows, uint32_t columns);

/* tests/test_k3_moe_smoke.cu:137-171 (host schedule: one column per lane,
 * 256 lanes, tree). */
void k3o_mxfp4_gemm(uint16_t *output, const uint8_t *packed,
                    const uint8_t *scales, const uint16_t *input,
                    uint32_t vectors, uint32_t rows, uint32_t columns);

/* k3_rocm_ops.cu:193-273: the production kernel's schedule (128 lanes, one
 * 32-column group per lane per step, four 8-term partial sums added
 * together, tree).  Used to measure cross-schedule distance. */
void k3o_mxfp4_gemm_kernel_order(uint16_t *output, const uint8_t *packed,
                                 const uint8_t *scales, const uint16_t *input,
                                 uint32_t vectors, uint32_t rows,
                                 uint32_t columns);

/* tests/test_k3_mxfp4_envelope.cu:263-278: fp64 dot product, no rounding. */
void k3o_mxfp4_gemm_f64(double *output, const uint8_t *packed,
                        const uint8_t *scales, const uint16_t *input,
                        uint32_t vectors, uint32_t rows, uint32_t columns);

/* tests/test_k3_moe_smoke.cu:173-184 / k3_rocm_ops.cu:66-83 (SiTU), and the
 * beta->infinity limit x*sigmoid(x)*u (SwiGLU) the benchmark configs name. */
void k3o_activation(uint16_t *output, const uint16_t *gate,
                    const uint16_t *up, uint64_t count, int activation,
                    float beta, float linear_beta);

/* tests/test_k3_moe_smoke.cu:186-213. */
void k3o_rms_norm(uint16_t *output, const uint16_t *input,
                  const uint16_t *weight, uint32_t vectors, uint32_t hidden,
                  float epsilon);

/* tests/test_k3_moe_smoke.cu:215-253 and k3_rocm_ops.cu:1440-1449 (scale). */
void k3o_router_topk(uint32_t *ids, float *weights, const float *logits,
                     const float *bias, uint32_t vectors, uint32_t experts,
                     uint32_t top_k, float scaling_factor);

/* Smallest gap between consecutive corrected scores around the selection
 * (ranks 0..top_k, i.e. including the first rejected candidate), per vector.
 * Used by parity tests to recognise documented near-ties. */
void k3o_router_min_gap(float *gaps, const float *logits, const float *bias,
                        uint32_t vectors, uint32_t experts, uint32_t top_k);

/* k3_rocm_ops.cu:1452-1474 / tests/test_k3_moe_smoke.cu:610-618. */
void k3o_weighted_sum(uint16_t *output, const uint16_t *vectors,
                      const float *weights, uint32_t tokens,
                      uint32_t vector_count, uint32_t hidden);

/* k3_rocm_ops.cu:1499-1510 / tests/test_k3_moe_smoke.cu:1264-1268. */
void k3o_add(uint16_t *output, const uint16_t *left, const uint16_t *right,
             uint64_t count);

/* k3_rocm_ops.cu:1476-1497. */
void k3o_gather_rows(uint16_t *output, const uint16_t *input,
                     const uint32_t *ids, uint32_t rows, uint32_t row_size);
void k3o_scatter_rows(uint16_t *output, const uint16_t *input,
                      const uint32_t *ids, uint32_t rows, uint32_t row_size);

/* k3_rocm_ops.cu:663-697 generalised to a block size (128 in the reference)
 * and scale type (f32 in the reference). */
void k3o_q8_quantize(int8_t *quantized, void *scales, const uint16_t *weights,
                     uint32_t rows, uint32_t columns, uint32_t block,
                     int scale_type);

/* tests/test_k3_q8_projection.cu:50-76 (256 lanes over 8-wide octets, tree),
 * generalised the same way. */
void k3o_q8_gemm(uint16_t *output, const int8_t *quantized,
                 const void *scales, const uint16_t *input, uint32_t vectors,
                 uint32_t rows, uint32_t columns, uint32_t block,
                 int scale_type);

/* k3_engine_prefill.inc:1175-1194: experts ascending, routes ascending
 * inside an expert.  offsets has experts+1 entries; tokens/routes have
 * tokens*top_k entries. */
void k3o_group_routes(uint32_t *offsets, uint32_t *route_tokens,
                      uint32_t *route_slots, const uint32_t *ids,
                      uint32_t tokens, uint32_t top_k, uint32_t experts);

typedef struct k3o_layer {
    uint32_t hidden;          /* d                                        */
    uint32_t expert_hidden;   /* I                                        */
    uint32_t experts;         /* E                                        */
    uint32_t top_k;
    uint32_t shared_hidden;   /* 0 = no shared expert                     */
    uint32_t q8_block;        /* 32 or 128                                */
    int      q8_scale_type;
    int      activation;
    float    beta, linear_beta;
    float    route_scale;
    const uint16_t *router_weight;   /* bf16 [E, d]                       */
    const float    *router_bias;     /* f32  [E]                          */
    /* per expert, contiguous over experts:                               */
    const uint8_t  *w1_packed;       /* [E, I, d/2]  gate                  */
    const uint8_t  *w1_scales;       /* [E, I, d/32]                       */
    const uint8_t  *w3_packed;       /* [E, I, d/2]  up                    */
    const uint8_t  *w3_scales;
    const uint8_t  *w2_packed;       /* [E, d, I/2]  down                  */
    const uint8_t  *w2_scales;       /* [E, d, I/32]                       */
    const int8_t   *shared_gate_q;   /* [S, d]                             */
    const void     *shared_gate_s;
    const int8_t   *shared_up_q;     /* [S, d]                             */
    const void     *shared_up_s;
    const int8_t   *shared_down_q;   /* [d, S]                             */
    const void     *shared_down_s;
} k3o_layer;

/*
 * One routed-MoE layer over `tokens` rows, following the composition of
 * k3_engine_prefill.inc:1448-1460 (router), :938-997 (per-expert gather,
 * gate, up, activation, down, scatter), :1575-1580 (weighted sum) and
 * :1598-1603 (add of the shared-expert output), with the experts consuming
 * the hidden vector directly (the benchmark's synthetic layer).
 * Outputs: out bf16 [tokens, d]; optional ids u32 / weights f32
 * [tokens, top_k]; optional logits f32 [tokens, E].
 * expert_subset < experts restricts the expert loop to the first
 * `expert_subset` experts that received routes (a bounded sample for
 * timing); pass 0 for all.  Returns the number of (expert,row) products
 * computed.
 */
uint64_t k3o_moe_layer(uint16_t *out, uint32_t *ids, float *weights,
                       float *logits, const k3o_layer *layer,
                       const uint16_t *x, uint32_t tokens,
                       uint32_t expert_subset);

int k3o_thread_count(void);

/* xorshift32 stream of the reference's model-free tests
 * (tests/test_k3_rocm_components.cu:30-42): fills out[i] with
 * (state & 0x00ffffff) / 2^24 after each update; *state carries on. */
void k3o_xorshift_unit(uint32_t *state, float *out, uint64_t count);

/* Seeded byte stream of the synthetic layers (mirror of synth.bytes_uniform);
 * `first` is a multiple of 8. */
void k3o_synth_bytes(uint8_t *out, uint64_t count, uint64_t key,
                     uint64_t first, uint32_t low, uint32_t span);

/* Number of OpenMP threads the parallel loops use from now on (the timed CPU
 * baseline sets it itself instead of inheriting OMP_NUM_THREADS). */
void k3o_set_threads(int threads);

#ifdef __cplusplus
}
#endif
#endif
