/*
 * CPU oracle for the routed-MoE path (see k3_oracle.h).  TEST INFRASTRUCTURE:
 * never linked into the product library.
 *
 * Arithmetic notes.  The reference builds host and device code with
 * -O3 -ffast-math -march=native (Makefile:8-12), so every statement of the
 * form `acc += a * b` is a fused multiply-add there.  This file is compiled
 * with -ffp-contract=off and spells those statements as fmaf() explicitly, so
 * the result does not depend on the compiler.  Where a product is exact in
 * fp32 (bf16 x bf16, e2m1 x e8m0 x bf16) fused and unfused agree bit for bit.
 */
#include "k3_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

enum { K3O_LANES = 256, K3O_MXFP4_KERNEL_LANES = 128 };

void k3o_set_threads(int threads) {
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
}

int k3o_thread_count(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

static inline float bits_to_float(uint32_t bits) {
    float value;
    memcpy(&value, &bits, sizeof(value));
    return value;
}

static inline uint32_t float_to_bits(float value) {
    uint32_t bits;
    memcpy(&bits, &value, sizeof(bits));
    return bits;
}

uint16_t k3o_bf16_from_float(float value) {
    uint32_t bits = float_to_bits(value);
    if ((bits & 0x7fffffffu) > 0x7f800000u) {
        return (uint16_t)((bits >> 16) | 0x0040u); /* quiet NaN */
    }
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}

float k3o_bf16_to_float(uint16_t bits) {
    return bits_to_float((uint32_t)bits << 16);
}

float k3o_f16_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exponent = (h >> 10) & 0x1fu;
    uint32_t mantissa = h & 0x3ffu;
    if (exponent == 0u) {
        if (mantissa == 0u) return bits_to_float(sign);
        float value = (float)mantissa * 5.9604644775390625e-8f; /* 2^-24 */
        return sign ? -value : value;
    }
    if (exponent == 31u) {
        return bits_to_float(sign | 0x7f800000u | (mantissa << 13));
    }
    return bits_to_float(sign | ((exponent + 112u) << 23) | (mantissa << 13));
}

float k3o_e8m0_to_float(uint8_t exponent) {
    return bits_to_float(exponent == 0u ? 0x00400000u
                                        : (uint32_t)exponent << 23);
}

float k3o_e2m1_to_float(uint8_t nibble) {
    static const float magnitude[8] = {
        0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
    };
    float value = magnitude[nibble & 7u];
    return (nibble & 8u) ? -value : value;
}

static inline float tree_reduce(float *partial, uint32_t lanes) {
    for (uint32_t width = lanes / 2u; width > 0u; width /= 2u) {
        for (uint32_t tid = 0; tid < width; tid++) {
            partial[tid] += partial[tid + width];
        }
    }
    return partial[0];
}

void k3o_bf16_gemm(float *output_f32, uint16_t *output_bf16,
                   const uint16_t *weights, const uint16_t *input,
                   uint32_t vectors, uint32_t rows, uint32_t columns) {
    float *x = (float *)malloc((size_t)vectors * columns * sizeof(float));
    for (uint64_t i = 0; i < (uint64_t)vectors * columns; i++) {
        x[i] = k3o_bf16_to_float(input[i]);
    }
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < (int64_t)rows; row++) {
        const uint16_t *w = weights + (uint64_t)row * columns;
        for (uint32_t v = 0; v < vectors; v++) {
            const float *xv = x + (uint64_t)v * columns;
            float partial[K3O_LANES];
            memset(partial, 0, sizeof(partial));
            /* lane t owns columns t, t+256, ... in ascending order (written as
             * blocks of 256 columns so that the compiler can use vector FMAs
             * across lanes; each lane's own order is unchanged) */
            uint32_t column = 0;
            for (; column + K3O_LANES <= columns; column += K3O_LANES) {
                for (uint32_t lane = 0; lane < K3O_LANES; lane++) {
                    partial[lane] =
                        fmaf(k3o_bf16_to_float(w[column + lane]),
                             xv[column + lane], partial[lane]);
                }
            }
            for (uint32_t lane = 0; column < columns; column++, lane++) {
                partial[lane] = fmaf(k3o_bf16_to_float(w[column]), xv[column],
                                     partial[lane]);
            }
            float sum = tree_reduce(partial, K3O_LANES);
            if (output_f32) output_f32[(uint64_t)v * rows + row] = sum;
            if (output_bf16) {
                output_bf16[(uint64_t)v * rows + row] =
                    k3o_bf16_from_float(sum);
            }
        }
    }
    free(x);
}

static void decode_mxfp4_row(float *decoded, const uint8_t *packed,
                             const uint8_t *scales, uint32_t columns) {
    for (uint32_t column = 0; column < columns; column++) {
        uint8_t byte = packed[column / 2u];
        uint8_t nibble = (column & 1u) ? (uint8_t)(byte >> 4u)
                                       : (uint8_t)(byte & 0x0fu);
        decoded[column] = k3o_e2m1_to_float(nibble) *
                          k3o_e8m0_to_float(scales[column / 32u]);
    }
}

void k3o_mxfp4_gemm(uint16_t *output, const uint8_t *packed,
                    const uint8_t *scales, const uint16_t *input,
                    uint32_t vectors, uint32_t rows, uint32_t columns) {
    float *x = (float *)malloc((size_t)vectors * columns * sizeof(float));
    for (uint64_t i = 0; i < (uint64_t)vectors * columns; i++) {
        x[i] = k3o_bf16_to_float(input[i]);
    }
#pragma omp parallel
    {
        float *decoded = (float *)malloc((size_t)columns * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t row = 0; row < (int64_t)rows; row++) {
            decode_mxfp4_row(decoded,
                             packed + (uint64_t)row * (columns / 2u),
                             scales + (uint64_t)row * (columns / 32u),
                             columns);
            for (uint32_t v = 0; v < vectors; v++) {
                const float *xv = x + (uint64_t)v * columns;
                float partial[K3O_LANES];
                memset(partial, 0, sizeof(partial));
                uint32_t column = 0;
                for (; column + K3O_LANES <= columns; column += K3O_LANES) {
                    for (uint32_t lane = 0; lane < K3O_LANES; lane++) {
                        partial[lane] = fmaf(decoded[column + lane],
                                             xv[column + lane], partial[lane]);
                    }
                }
                for (uint32_t lane = 0; column < columns; column++, lane++) {
                    partial[lane] =
                        fmaf(decoded[column], xv[column], partial[lane]);
                }
                output[(uint64_t)v * rows + row] =
                    k3o_bf16_from_float(tree_reduce(partial, K3O_LANES));
            }
        }
        free(decoded);
    }
    free(x);
}

void k3o_mxfp4_gemm_kernel_order(uint16_t *output, const uint8_t *packed,
                                 const uint8_t *scales, const uint16_t *input,
                                 uint32_t vectors, uint32_t rows,
                                 uint32_t columns) {
    const uint32_t groups = columns / 32u;
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < (int64_t)rows; row++) {
        const uint8_t *p = packed + (uint64_t)row * (columns / 2u);
        const uint8_t *s = scales + (uint64_t)row * groups;
        for (uint32_t v = 0; v < vectors; v++) {
            const uint16_t *xv = input + (uint64_t)v * columns;
            float partial[K3O_MXFP4_KERNEL_LANES];
            memset(partial, 0, sizeof(partial));
            for (uint32_t group = 0; group < groups; group++) {
                uint32_t lane = group % K3O_MXFP4_KERNEL_LANES;
                float scale = k3o_e8m0_to_float(s[group]);
                float quarter[4];
                for (uint32_t q = 0; q < 4u; q++) {
                    float dot8 = 0.0f;
                    for (uint32_t i = 0; i < 8u; i++) {
                        uint32_t column = group * 32u + q * 8u + i;
                        uint8_t byte = p[column / 2u];
                        uint8_t nibble = (column & 1u)
                                             ? (uint8_t)(byte >> 4u)
                                             : (uint8_t)(byte & 0x0fu);
                        dot8 = fmaf(k3o_e2m1_to_float(nibble) * scale,
                                    k3o_bf16_to_float(xv[column]), dot8);
                    }
                    quarter[q] = dot8;
                }
                partial[lane] += quarter[0] + quarter[1] + quarter[2] +
                                 quarter[3];
            }
            output[(uint64_t)v * rows + row] = k3o_bf16_from_float(
                tree_reduce(partial, K3O_MXFP4_KERNEL_LANES));
        }
    }
}

void k3o_mxfp4_gemm_f64(double *output, const uint8_t *packed,
                        const uint8_t *scales, const uint16_t *input,
                        uint32_t vectors, uint32_t rows, uint32_t columns) {
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < (int64_t)rows; row++) {
        const uint8_t *p = packed + (uint64_t)row * (columns / 2u);
        const uint8_t *s = scales + (uint64_t)row * (columns / 32u);
        for (uint32_t v = 0; v < vectors; v++) {
            const uint16_t *xv = input + (uint64_t)v * columns;
            double sum = 0.0;
            for (uint32_t column = 0; column < columns; column++) {
                uint8_t byte = p[column / 2u];
                uint8_t nibble = (column & 1u) ? (uint8_t)(byte >> 4u)
                                               : (uint8_t)(byte & 0x0fu);
                double weight = (double)k3o_e2m1_to_float(nibble) *
                                (double)k3o_e8m0_to_float(s[column / 32u]);
                sum += weight * (double)k3o_bf16_to_float(xv[column]);
            }
            output[(uint64_t)v * rows + row] = sum;
        }
    }
}

void k3o_activation(uint16_t *output, const uint16_t *gate,
                    const uint16_t *up, uint64_t count, int activation,
                    float beta, float linear_beta) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)count; i++) {
        float g = k3o_bf16_to_float(gate[i]);
        float u = k3o_bf16_to_float(up[i]);
        float value;
        if (activation == K3O_ACT_SITU) {
            float bounded_gate = beta * tanhf(g / beta);
            float sigmoid_gate = 1.0f / (1.0f + expf(-g));
            float bounded_up = linear_beta * tanhf(u / linear_beta);
            value = bounded_gate * sigmoid_gate * bounded_up;
        } else if (activation == K3O_ACT_SITU_HOST) {
            value = (beta * tanhf(g / beta) / (1.0f + expf(-g))) *
                    (linear_beta * tanhf(u / linear_beta));
        } else {
            float sigmoid_gate = 1.0f / (1.0f + expf(-g));
            value = g * sigmoid_gate * u;
        }
        output[i] = k3o_bf16_from_float(value);
    }
}

void k3o_rms_norm(uint16_t *output, const uint16_t *input,
                  const uint16_t *weight, uint32_t vectors, uint32_t hidden,
                  float epsilon) {
#pragma omp parallel for schedule(static)
    for (int64_t v = 0; v < (int64_t)vectors; v++) {
        const uint16_t *in = input + (uint64_t)v * hidden;
        uint16_t *out = output + (uint64_t)v * hidden;
        float partial[K3O_LANES];
        memset(partial, 0, sizeof(partial));
        for (uint32_t i = 0; i < hidden; i++) {
            float value = k3o_bf16_to_float(in[i]);
            partial[i % K3O_LANES] =
                fmaf(value, value, partial[i % K3O_LANES]);
        }
        float sum = tree_reduce(partial, K3O_LANES);
        float reciprocal_std = 1.0f / sqrtf(sum / (float)hidden + epsilon);
        for (uint32_t i = 0; i < hidden; i++) {
            out[i] = k3o_bf16_from_float(k3o_bf16_to_float(in[i]) *
                                         reciprocal_std *
                                         k3o_bf16_to_float(weight[i]));
        }
    }
}

static void router_one(uint32_t *ids, float *weights, float *choices,
                       const float *logits, const float *bias,
                       uint32_t experts, uint32_t top_k) {
    for (uint32_t rank = 0; rank < top_k; rank++) {
        choices[rank] = -INFINITY;
        weights[rank] = 0.0f;
        ids[rank] = UINT32_MAX;
    }
    for (uint32_t expert = 0; expert < experts; expert++) {
        float raw = 1.0f / (1.0f + expf(-logits[expert]));
        float choice = raw + bias[expert];
        uint32_t position = top_k;
        for (uint32_t rank = 0; rank < top_k; rank++) {
            if (choice > choices[rank] ||
                (choice == choices[rank] && expert < ids[rank])) {
                position = rank;
                break;
            }
        }
        if (position == top_k) continue;
        for (uint32_t rank = top_k - 1u; rank > position; rank--) {
            choices[rank] = choices[rank - 1u];
            weights[rank] = weights[rank - 1u];
            ids[rank] = ids[rank - 1u];
        }
        choices[position] = choice;
        weights[position] = raw;
        ids[position] = expert;
    }
}

void k3o_router_topk(uint32_t *ids, float *weights, const float *logits,
                     const float *bias, uint32_t vectors, uint32_t experts,
                     uint32_t top_k, float scaling_factor) {
#pragma omp parallel for schedule(static)
    for (int64_t v = 0; v < (int64_t)vectors; v++) {
        float choices[64];
        uint32_t *row_ids = ids + (uint64_t)v * top_k;
        float *row_weights = weights + (uint64_t)v * top_k;
        router_one(row_ids, row_weights, choices,
                   logits + (uint64_t)v * experts, bias, experts, top_k);
        float denominator = 1e-20f;
        for (uint32_t rank = 0; rank < top_k; rank++) {
            denominator += row_weights[rank];
        }
        for (uint32_t rank = 0; rank < top_k; rank++) {
            row_weights[rank] =
                row_weights[rank] / denominator * scaling_factor;
        }
    }
}

void k3o_router_min_gap(float *gaps, const float *logits, const float *bias,
                        uint32_t vectors, uint32_t experts, uint32_t top_k) {
    const uint32_t keep = top_k + 1u <= experts ? top_k + 1u : top_k;
#pragma omp parallel for schedule(static)
    for (int64_t v = 0; v < (int64_t)vectors; v++) {
        uint32_t ids[65];
        float weights[65];
        float choices[65];
        router_one(ids, weights, choices, logits + (uint64_t)v * experts,
                   bias, experts, keep);
        float gap = INFINITY;
        for (uint32_t rank = 1; rank < keep; rank++) {
            float d = choices[rank - 1u] - choices[rank];
            if (d < gap) gap = d;
        }
        gaps[v] = gap;
    }
}

void k3o_weighted_sum(uint16_t *output, const uint16_t *vectors,
                      const float *weights, uint32_t tokens,
                      uint32_t vector_count, uint32_t hidden) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < (int64_t)tokens; t++) {
        const uint16_t *v = vectors + (uint64_t)t * vector_count * hidden;
        const float *w = weights + (uint64_t)t * vector_count;
        for (uint32_t d = 0; d < hidden; d++) {
            float sum = 0.0f;
            for (uint32_t r = 0; r < vector_count; r++) {
                sum = fmaf(w[r],
                           k3o_bf16_to_float(v[(uint64_t)r * hidden + d]),
                           sum);
            }
            output[(uint64_t)t * hidden + d] = k3o_bf16_from_float(sum);
        }
    }
}

void k3o_add(uint16_t *output, const uint16_t *left, const uint16_t *right,
             uint64_t count) {
    for (uint64_t i = 0; i < count; i++) {
        output[i] = k3o_bf16_from_float(k3o_bf16_to_float(left[i]) +
                                        k3o_bf16_to_float(right[i]));
    }
}

void k3o_gather_rows(uint16_t *output, const uint16_t *input,
                     const uint32_t *ids, uint32_t rows, uint32_t row_size) {
    for (uint32_t r = 0; r < rows; r++) {
        memcpy(output + (uint64_t)r * row_size,
               input + (uint64_t)ids[r] * row_size,
               (size_t)row_size * sizeof(uint16_t));
    }
}

void k3o_scatter_rows(uint16_t *output, const uint16_t *input,
                      const uint32_t *ids, uint32_t rows, uint32_t row_size) {
    for (uint32_t r = 0; r < rows; r++) {
        memcpy(output + (uint64_t)ids[r] * row_size,
               input + (uint64_t)r * row_size,
               (size_t)row_size * sizeof(uint16_t));
    }
}

static uint16_t f16_from_float(float value) {
    /* round-to-nearest-even f32 -> f16 (scales are small positive normals or
     * subnormals; handles the general case anyway) */
    uint32_t bits = float_to_bits(value);
    uint32_t sign = (bits >> 16) & 0x8000u;
    uint32_t mag = bits & 0x7fffffffu;
    if (mag >= 0x7f800000u) {
        return (uint16_t)(sign | 0x7c00u | (mag > 0x7f800000u ? 0x200u : 0u));
    }
    if (mag >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);
    if (mag < 0x33000001u) return (uint16_t)sign; /* < 2^-25 rounds to 0 */
    int32_t exponent = (int32_t)(mag >> 23) - 127;
    uint32_t mantissa = (mag & 0x7fffffu) | 0x800000u;
    uint32_t shift;
    uint32_t half;
    if (exponent < -14) {
        shift = (uint32_t)(13 + (-14 - exponent));
        uint32_t rounded = mantissa >> shift;
        uint32_t rem = mantissa & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1u);
        if (rem > halfway || (rem == halfway && (rounded & 1u))) rounded++;
        return (uint16_t)(sign | rounded);
    }
    shift = 13u;
    half = ((uint32_t)(exponent + 15) << 10) | ((mantissa >> shift) & 0x3ffu);
    uint32_t rem = mantissa & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;
    return (uint16_t)(sign | half);
}

static inline float q8_scale_at(const void *scales, uint64_t index,
                                int scale_type) {
    return scale_type == K3O_Q8_SCALE_F16
               ? k3o_f16_to_float(((const uint16_t *)scales)[index])
               : ((const float *)scales)[index];
}

void k3o_q8_quantize(int8_t *quantized, void *scales, const uint16_t *weights,
                     uint32_t rows, uint32_t columns, uint32_t block,
                     int scale_type) {
    const uint32_t blocks_per_row = columns / block;
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < (int64_t)rows; row++) {
        for (uint32_t b = 0; b < blocks_per_row; b++) {
            uint64_t block_index = (uint64_t)row * blocks_per_row + b;
            uint64_t base = block_index * block;
            float maximum = 0.0f;
            for (uint32_t i = 0; i < block; i++) {
                maximum = fmaxf(maximum,
                                fabsf(k3o_bf16_to_float(weights[base + i])));
            }
            float scale = maximum > 0.0f ? maximum / 127.0f : 1.0f;
            if (scale_type == K3O_Q8_SCALE_F16) {
                uint16_t h = f16_from_float(scale);
                ((uint16_t *)scales)[block_index] = h;
                scale = k3o_f16_to_float(h);
            } else {
                ((float *)scales)[block_index] = scale;
            }
            for (uint32_t i = 0; i < block; i++) {
                float value = k3o_bf16_to_float(weights[base + i]);
                long q = lrintf(value / scale);
                if (q > 127) q = 127;
                if (q < -127) q = -127;
                quantized[base + i] = (int8_t)q;
            }
        }
    }
}

void k3o_q8_gemm(uint16_t *output, const int8_t *quantized,
                 const void *scales, const uint16_t *input, uint32_t vectors,
                 uint32_t rows, uint32_t columns, uint32_t block,
                 int scale_type) {
    const uint32_t octets = columns / 8u;
    const uint32_t blocks_per_row = columns / block;
    float *x = (float *)malloc((size_t)vectors * columns * sizeof(float));
    for (uint64_t i = 0; i < (uint64_t)vectors * columns; i++) {
        x[i] = k3o_bf16_to_float(input[i]);
    }
#pragma omp parallel
    {
        float *scaled = (float *)malloc((size_t)columns * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t row = 0; row < (int64_t)rows; row++) {
            const int8_t *q = quantized + (uint64_t)row * columns;
            for (uint32_t column = 0; column < columns; column++) {
                scaled[column] =
                    (float)q[column] *
                    q8_scale_at(scales,
                                (uint64_t)row * blocks_per_row +
                                    column / block,
                                scale_type);
            }
            for (uint32_t v = 0; v < vectors; v++) {
                const float *xv = x + (uint64_t)v * columns;
                float partial[K3O_LANES];
                memset(partial, 0, sizeof(partial));
                /* lane t owns octets t, t+256, ...; 8 sequential terms */
                for (uint32_t octet = 0; octet < octets; octet++) {
                    uint32_t lane = octet % K3O_LANES;
                    float acc = partial[lane];
                    for (uint32_t i = 0; i < 8u; i++) {
                        uint32_t column = octet * 8u + i;
                        acc = fmaf(scaled[column], xv[column], acc);
                    }
                    partial[lane] = acc;
                }
                output[(uint64_t)v * rows + row] =
                    k3o_bf16_from_float(tree_reduce(partial, K3O_LANES));
            }
        }
        free(scaled);
    }
    free(x);
}

void k3o_group_routes(uint32_t *offsets, uint32_t *route_tokens,
                      uint32_t *route_slots, const uint32_t *ids,
                      uint32_t tokens, uint32_t top_k, uint32_t experts) {
    const uint64_t routes = (uint64_t)tokens * top_k;
    memset(offsets, 0, (size_t)(experts + 1u) * sizeof(uint32_t));
    for (uint64_t route = 0; route < routes; route++) {
        if (ids[route] < experts) offsets[ids[route] + 1u]++;
    }
    for (uint32_t e = 0; e < experts; e++) offsets[e + 1u] += offsets[e];
    uint32_t *cursor = (uint32_t *)malloc((size_t)experts * sizeof(uint32_t));
    memcpy(cursor, offsets, (size_t)experts * sizeof(uint32_t));
    /* token-major scan keeps routes ascending inside each expert */
    for (uint32_t token = 0; token < tokens; token++) {
        for (uint32_t rank = 0; rank < top_k; rank++) {
            uint32_t route = token * top_k + rank;
            uint32_t expert = ids[route];
            if (expert >= experts) continue;
            uint32_t slot = cursor[expert]++;
            route_tokens[slot] = token;
            route_slots[slot] = route;
        }
    }
    free(cursor);
}

uint64_t k3o_moe_layer(uint16_t *out, uint32_t *ids_out, float *weights_out,
                       float *logits_out, const k3o_layer *layer,
                       const uint16_t *x, uint32_t tokens,
                       uint32_t expert_subset) {
    const uint32_t d = layer->hidden;
    const uint32_t I = layer->expert_hidden;
    const uint32_t E = layer->experts;
    const uint32_t k = layer->top_k;
    const uint64_t routes = (uint64_t)tokens * k;
    float *logits = logits_out
                        ? logits_out
                        : (float *)malloc((size_t)tokens * E * sizeof(float));
    uint32_t *ids =
        ids_out ? ids_out : (uint32_t *)malloc(routes * sizeof(uint32_t));
    float *weights =
        weights_out ? weights_out : (float *)malloc(routes * sizeof(float));
    k3o_bf16_gemm(logits, NULL, layer->router_weight, x, tokens, E, d);
    k3o_router_topk(ids, weights, logits, layer->router_bias, tokens, E, k,
                    layer->route_scale);

    uint32_t *offsets = (uint32_t *)malloc((size_t)(E + 1u) * sizeof(uint32_t));
    uint32_t *route_tokens = (uint32_t *)malloc(routes * sizeof(uint32_t));
    uint32_t *route_slots = (uint32_t *)malloc(routes * sizeof(uint32_t));
    k3o_group_routes(offsets, route_tokens, route_slots, ids, tokens, k, E);

    /* expert_outputs [tokens, k, d], zero-filled first
     * (k3_engine_prefill.inc:1557-1561) */
    uint16_t *expert_outputs =
        (uint16_t *)calloc(routes * d, sizeof(uint16_t));
    uint64_t products = 0;
    uint32_t visited = 0;
    const uint64_t w13_packed = (uint64_t)I * (d / 2u);
    const uint64_t w13_scales = (uint64_t)I * (d / 32u);
    const uint64_t w2_packed = (uint64_t)d * (I / 2u);
    const uint64_t w2_scales = (uint64_t)d * (I / 32u);
    for (uint32_t e = 0; e < E; e++) {
        uint32_t n = offsets[e + 1u] - offsets[e];
        if (n == 0u) continue;
        if (expert_subset != 0u && visited >= expert_subset) break;
        visited++;
        products += n;
        uint16_t *gathered = (uint16_t *)malloc((size_t)n * d * 2u);
        uint16_t *gate = (uint16_t *)malloc((size_t)n * I * 2u);
        uint16_t *up = (uint16_t *)malloc((size_t)n * I * 2u);
        uint16_t *act = (uint16_t *)malloc((size_t)n * I * 2u);
        uint16_t *down = (uint16_t *)malloc((size_t)n * d * 2u);
        k3o_gather_rows(gathered, x, route_tokens + offsets[e], n, d);
        k3o_mxfp4_gemm(gate, layer->w1_packed + e * w13_packed,
                       layer->w1_scales + e * w13_scales, gathered, n, I, d);
        k3o_mxfp4_gemm(up, layer->w3_packed + e * w13_packed,
                       layer->w3_scales + e * w13_scales, gathered, n, I, d);
        k3o_activation(act, gate, up, (uint64_t)n * I, layer->activation,
                       layer->beta, layer->linear_beta);
        k3o_mxfp4_gemm(down, layer->w2_packed + e * w2_packed,
                       layer->w2_scales + e * w2_scales, act, n, d, I);
        k3o_scatter_rows(expert_outputs, down, route_slots + offsets[e], n,
                         d);
        free(down);
        free(act);
        free(up);
        free(gate);
        free(gathered);
    }
    uint16_t *routed = (uint16_t *)malloc((size_t)tokens * d * 2u);
    k3o_weighted_sum(routed, expert_outputs, weights, tokens, k, d);
    if (layer->shared_hidden != 0u) {
        const uint32_t S = layer->shared_hidden;
        uint16_t *sg = (uint16_t *)malloc((size_t)tokens * S * 2u);
        uint16_t *su = (uint16_t *)malloc((size_t)tokens * S * 2u);
        uint16_t *sa = (uint16_t *)malloc((size_t)tokens * S * 2u);
        uint16_t *so = (uint16_t *)malloc((size_t)tokens * d * 2u);
        k3o_q8_gemm(sg, layer->shared_gate_q, layer->shared_gate_s, x, tokens,
                    S, d, layer->q8_block, layer->q8_scale_type);
        k3o_q8_gemm(su, layer->shared_up_q, layer->shared_up_s, x, tokens, S,
                    d, layer->q8_block, layer->q8_scale_type);
        k3o_activation(sa, sg, su, (uint64_t)tokens * S, layer->activation,
                       layer->beta, layer->linear_beta);
        k3o_q8_gemm(so, layer->shared_down_q, layer->shared_down_s, sa,
                    tokens, d, S, layer->q8_block, layer->q8_scale_type);
        k3o_add(out, routed, so, (uint64_t)tokens * d);
        free(so);
        free(sa);
        free(su);
        free(sg);
    } else {
        memcpy(out, routed, (size_t)tokens * d * 2u);
    }
    free(routed);
    free(expert_outputs);
    free(route_slots);
    free(route_tokens);
    free(offsets);
    if (!weights_out) free(weights);
    if (!ids_out) free(ids);
    if (!logits_out) free(logits);
    return products;
}

void k3o_xorshift_unit(uint32_t *state, float *out, uint64_t count) {
    uint32_t s = *state;
    for (uint64_t i = 0; i < count; i++) {
        s ^= s << 13;
        s ^= s >> 17;
        s ^= s << 5;
        out[i] = (float)(s & 0x00ffffffu) / (float)0x01000000u;
    }
    *state = s;
}

/* The seeded byte streams of the synthetic layers (moonshine_b200/synth.py,
 * raw_bytes / bytes_uniform): byte j of 8-byte chunk c is bits [8j, 8j+8) of the
 * splitmix64 finaliser of (key * golden + golden + c); low + floor(b*span/256). */
void k3o_synth_bytes(uint8_t *out, uint64_t count, uint64_t key,
                     uint64_t first, uint32_t low, uint32_t span) {
    const uint64_t golden = 0x9E3779B97F4A7C15ull;
    const uint64_t base = key * golden + golden;
    const uint64_t first_chunk = first / 8u;
    const uint64_t chunks = (count + 7u) / 8u;
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < (int64_t)chunks; c++) {
        uint64_t z = (first_chunk + (uint64_t)c) + base;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z = z ^ (z >> 31);
        for (uint32_t j = 0; j < 8u; j++) {
            const uint64_t i = (uint64_t)c * 8u + j;
            if (i >= count) break;
            const uint32_t b = (uint32_t)((z >> (8u * j)) & 0xffu);
            out[i] = (uint8_t)(low + ((b * span) >> 8));
        }
    }
}
