// Element-wise, row-copy, reduction and router-selection entry points of the
// routed-MoE path.  Signatures, argument checks and return conventions follow
// the reference's C operator interface (k3_rocm_ops.h); the kernels are new.
#include "k3_common.cuh"
#include "k3_moe_ops.h"

#include <math.h>

using namespace k3;

namespace {

constexpr int kThreads = 256;

inline uint32_t grid_for(uint64_t items, uint32_t per_block) {
    uint64_t blocks = (items + per_block - 1) / per_block;
    const uint64_t cap = (uint64_t)sm_count() * 32u;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    return (uint32_t)blocks;
}

// ---------------------------------------------------------------- activation
__global__ void __launch_bounds__(kThreads)
activation_kernel(uint16_t *__restrict__ out, const uint16_t *__restrict__ gate,
                  const uint16_t *__restrict__ up, uint64_t count, int kind, float beta,
                  float linear_beta) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool aligned = ((((uintptr_t)out) | ((uintptr_t)gate) | ((uintptr_t)up)) & 15u) == 0;
    if (aligned) {
        const uint64_t octets = count / 8u;
        for (uint64_t o = i; o < octets; o += stride) {
            const uint4 g = reinterpret_cast<const uint4 *>(gate)[o];
            const uint4 u = reinterpret_cast<const uint4 *>(up)[o];
            const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
            const uint32_t uw[4] = {u.x, u.y, u.z, u.w};
            uint32_t r[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t lo = float_to_bf16_bits(
                    activation(bf16_lo(gw[j]), bf16_lo(uw[j]), kind, beta, linear_beta));
                const uint32_t hi = float_to_bf16_bits(
                    activation(bf16_hi(gw[j]), bf16_hi(uw[j]), kind, beta, linear_beta));
                r[j] = lo | (hi << 16);
            }
            reinterpret_cast<uint4 *>(out)[o] = make_uint4(r[0], r[1], r[2], r[3]);
        }
        i += octets * 8u;  // tail
        for (; i < count; i += stride) {
            out[i] = float_to_bf16_bits(activation(bf16_bits_to_float(gate[i]),
                                                   bf16_bits_to_float(up[i]), kind, beta,
                                                   linear_beta));
        }
        return;
    }
    for (; i < count; i += stride) {
        out[i] = float_to_bf16_bits(activation(bf16_bits_to_float(gate[i]),
                                               bf16_bits_to_float(up[i]), kind, beta,
                                               linear_beta));
    }
}

// ----------------------------------------------------------------------- add
__global__ void __launch_bounds__(kThreads)
add_kernel(uint16_t *__restrict__ out, const uint16_t *__restrict__ a,
           const uint16_t *__restrict__ b, uint64_t count) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool aligned = ((((uintptr_t)out) | ((uintptr_t)a) | ((uintptr_t)b)) & 15u) == 0;
    uint64_t done = 0;
    if (aligned) {
        const uint64_t octets = count / 8u;
        for (uint64_t o = i; o < octets; o += stride) {
            const uint4 x = reinterpret_cast<const uint4 *>(a)[o];
            const uint4 y = reinterpret_cast<const uint4 *>(b)[o];
            const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
            const uint32_t yw[4] = {y.x, y.y, y.z, y.w};
            uint32_t r[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t lo = float_to_bf16_bits(bf16_lo(xw[j]) + bf16_lo(yw[j]));
                const uint32_t hi = float_to_bf16_bits(bf16_hi(xw[j]) + bf16_hi(yw[j]));
                r[j] = lo | (hi << 16);
            }
            reinterpret_cast<uint4 *>(out)[o] = make_uint4(r[0], r[1], r[2], r[3]);
        }
        done = octets * 8u;
    }
    for (uint64_t k = done + i; k < count; k += stride) {
        out[k] = float_to_bf16_bits(bf16_bits_to_float(a[k]) + bf16_bits_to_float(b[k]));
    }
}

// ------------------------------------------------------------ gather/scatter
template <bool Scatter>
__global__ void __launch_bounds__(kThreads)
copy_rows_kernel(uint16_t *__restrict__ out, const uint16_t *__restrict__ in,
                 const uint32_t *__restrict__ ids, uint32_t rows, uint32_t row_size) {
    // one warp per row; 16-byte copies when both sides allow it
    const uint32_t warps_per_block = blockDim.x / kWarp;
    const uint32_t lane = threadIdx.x % kWarp;
    const bool wide = (row_size % 8u == 0) && ((((uintptr_t)out) | ((uintptr_t)in)) & 15u) == 0;
    for (uint32_t r = blockIdx.x * warps_per_block + threadIdx.x / kWarp; r < rows;
         r += gridDim.x * warps_per_block) {
        const uint64_t indexed = (uint64_t)ids[r] * row_size;
        const uint64_t packed = (uint64_t)r * row_size;
        const uint16_t *src = in + (Scatter ? packed : indexed);
        uint16_t *dst = out + (Scatter ? indexed : packed);
        if (wide) {
            const uint32_t n = row_size / 8u;
            for (uint32_t c = lane; c < n; c += kWarp) {
                reinterpret_cast<uint4 *>(dst)[c] = reinterpret_cast<const uint4 *>(src)[c];
            }
        } else {
            for (uint32_t c = lane; c < row_size; c += kWarp) dst[c] = src[c];
        }
    }
}

// -------------------------------------------------------------- weighted sum
// out[t,d] = bf16( sum_r w[t,r] * v[t,r,d] ), r ascending, one fused
// multiply-add per term (k3_rocm_ops.cu:1452-1474 of the reference).
__global__ void __launch_bounds__(kThreads)
weighted_sum_kernel(uint16_t *__restrict__ out, const uint16_t *__restrict__ vectors,
                    const float *__restrict__ weights, uint32_t tokens, uint32_t count,
                    uint32_t hidden) {
    extern __shared__ float w_s[];
    const bool wide = (hidden % 8u == 0) &&
                      ((((uintptr_t)out) | ((uintptr_t)vectors)) & 15u) == 0;
    for (uint32_t token = blockIdx.x; token < tokens; token += gridDim.x) {
        __syncthreads();
        for (uint32_t r = threadIdx.x; r < count; r += blockDim.x) {
            w_s[r] = weights[(uint64_t)token * count + r];
        }
        __syncthreads();
        const uint16_t *v = vectors + (uint64_t)token * count * hidden;
        uint16_t *o = out + (uint64_t)token * hidden;
        if (wide) {
            for (uint32_t c = threadIdx.x; c < hidden / 8u; c += blockDim.x) {
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (uint32_t r = 0; r < count; r++) {
                    const uint4 q =
                        reinterpret_cast<const uint4 *>(v + (uint64_t)r * hidden)[c];
                    const float w = w_s[r];
                    acc[0] = fmaf(w, bf16_lo(q.x), acc[0]);
                    acc[1] = fmaf(w, bf16_hi(q.x), acc[1]);
                    acc[2] = fmaf(w, bf16_lo(q.y), acc[2]);
                    acc[3] = fmaf(w, bf16_hi(q.y), acc[3]);
                    acc[4] = fmaf(w, bf16_lo(q.z), acc[4]);
                    acc[5] = fmaf(w, bf16_hi(q.z), acc[5]);
                    acc[6] = fmaf(w, bf16_lo(q.w), acc[6]);
                    acc[7] = fmaf(w, bf16_hi(q.w), acc[7]);
                }
                uint32_t r4[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    r4[j] = (uint32_t)float_to_bf16_bits(acc[2 * j]) |
                            ((uint32_t)float_to_bf16_bits(acc[2 * j + 1]) << 16);
                }
                reinterpret_cast<uint4 *>(o)[c] = make_uint4(r4[0], r4[1], r4[2], r4[3]);
            }
        } else {
            for (uint32_t d = threadIdx.x; d < hidden; d += blockDim.x) {
                float acc = 0.f;
                for (uint32_t r = 0; r < count; r++) {
                    acc = fmaf(w_s[r], bf16_bits_to_float(v[(uint64_t)r * hidden + d]), acc);
                }
                o[d] = float_to_bf16_bits(acc);
            }
        }
    }
}

// ------------------------------------------------------------------ RMSNorm
// Sum of squares in the reference's order: 256 strided lanes, one fused
// multiply-add per element, binary tree (k3_rocm_ops.cu:837-867).
__global__ void __launch_bounds__(kThreads)
rms_norm_kernel(uint16_t *__restrict__ out, const uint16_t *__restrict__ in,
                const uint16_t *__restrict__ weight, uint32_t vectors, uint32_t hidden,
                float epsilon) {
    __shared__ float red[kThreads];
    for (uint32_t v = blockIdx.x; v < vectors; v += gridDim.x) {
        const uint16_t *x = in + (uint64_t)v * hidden;
        float sum = 0.f;
        for (uint32_t d = threadIdx.x; d < hidden; d += kThreads) {
            const float value = bf16_bits_to_float(x[d]);
            sum = fmaf(value, value, sum);
        }
        red[threadIdx.x] = sum;
        __syncthreads();
        for (uint32_t width = kThreads / 2; width > 0; width >>= 1) {
            if (threadIdx.x < width) red[threadIdx.x] += red[threadIdx.x + width];
            __syncthreads();
        }
        const float reciprocal_std = 1.0f / sqrtf(red[0] / (float)hidden + epsilon);
        __syncthreads();
        for (uint32_t d = threadIdx.x; d < hidden; d += kThreads) {
            const float value = __fmul_rn(__fmul_rn(bf16_bits_to_float(x[d]), reciprocal_std),
                                          bf16_bits_to_float(weight[d]));
            out[(uint64_t)v * hidden + d] = float_to_bf16_bits(value);
        }
    }
}

// ------------------------------------------------------------ router top-k
// One warp per score row.  Lane l owns experts l, l+32, ...; top_k rounds of a
// warp arg-max under the order (score+bias descending, expert id ascending),
// which is the order the reference's insertion oracle and bitonic kernel
// produce (k3_rocm_ops.cu:1398-1449).  Weights: raw score / (1e-20 + sum of the
// selected raw scores in rank order) * scale.
constexpr int kMaxPerLane = 32;  // 1024 experts / 32 lanes

__global__ void __launch_bounds__(128)
router_topk_kernel(uint32_t *__restrict__ ids_out, float *__restrict__ weights_out,
                   const float *__restrict__ logits, const float *__restrict__ bias,
                   uint32_t vectors, uint32_t experts, uint32_t top_k, float scale) {
    const uint32_t lane = threadIdx.x % kWarp;
    const uint32_t warps_per_block = blockDim.x / kWarp;
    const uint32_t per_lane = (experts + kWarp - 1) / kWarp;
    for (uint32_t v = blockIdx.x * warps_per_block + threadIdx.x / kWarp; v < vectors;
         v += gridDim.x * warps_per_block) {
        const float *row = logits + (uint64_t)v * experts;
        float choice[kMaxPerLane];
        float score[kMaxPerLane];
#pragma unroll
        for (int i = 0; i < kMaxPerLane; i++) {
            const uint32_t e = lane + (uint32_t)i * kWarp;
            if ((uint32_t)i < per_lane && e < experts) {
                const float s = sigmoid_exact(row[e]);
                score[i] = s;
                choice[i] = s + bias[e];
            } else {
                score[i] = 0.f;
                choice[i] = -INFINITY;
            }
        }
        uint32_t taken = 0u;  // bit i: local candidate i already selected
        float my_weight = 0.f;
        uint32_t my_id = 0u;
        float denominator = 1e-20f;
        for (uint32_t rank = 0; rank < top_k; rank++) {
            // local best: largest choice, smallest index on ties (ascending scan, strict >)
            float best = -INFINITY;
            int best_i = -1;
#pragma unroll
            for (int i = 0; i < kMaxPerLane; i++) {
                const bool usable = ((taken >> i) & 1u) == 0u && (uint32_t)i < per_lane &&
                                    lane + (uint32_t)i * kWarp < experts;
                if (usable && (best_i < 0 || choice[i] > best)) {
                    best = choice[i];
                    best_i = i;
                }
            }
            uint32_t best_id = best_i < 0 ? 0xffffffffu : lane + (uint32_t)best_i * kWarp;
            float win = best;
            uint32_t win_id = best_id;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float oc = __shfl_xor_sync(0xffffffffu, win, o);
                const uint32_t oid = __shfl_xor_sync(0xffffffffu, win_id, o);
                const bool take = (oid != 0xffffffffu) &&
                                  (win_id == 0xffffffffu || oc > win || (oc == win && oid < win_id));
                if (take) {
                    win = oc;
                    win_id = oid;
                }
            }
            // owner marks the winner and publishes its raw score
            float raw = 0.f;
            if (win_id != 0xffffffffu && (win_id % kWarp) == lane) {
                const int i = (int)(win_id / kWarp);
                taken |= 1u << i;
#pragma unroll
                for (int j = 0; j < kMaxPerLane; j++) {
                    if (j == i) raw = score[j];
                }
            }
            raw = __shfl_sync(0xffffffffu, raw, win_id == 0xffffffffu ? 0 : (int)(win_id % kWarp));
            denominator += raw;
            if (lane == rank) {
                my_weight = raw;
                my_id = win_id;
            }
        }
        if (lane < top_k) {
            ids_out[(uint64_t)v * top_k + lane] = my_id;
            weights_out[(uint64_t)v * top_k + lane] =
                __fmul_rn(__fdiv_rn(my_weight, denominator), scale);
        }
    }
}

// ------------------------------------------------------------ Q8 quantiser
__global__ void q8_quantize_kernel(int8_t *__restrict__ q, void *__restrict__ scales,
                                   const uint16_t *__restrict__ w, uint64_t blocks,
                                   uint32_t block, int scale_f16) {
    // one warp per block of `block` elements
    const uint32_t lane = threadIdx.x % kWarp;
    const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) / kWarp;
    const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) / kWarp;
    for (uint64_t b = warp; b < blocks; b += warps) {
        const uint64_t base = b * block;
        float m = 0.f;
        for (uint32_t i = lane; i < block; i += kWarp) {
            m = fmaxf(m, fabsf(bf16_bits_to_float(w[base + i])));
        }
        m = warp_max(m);
        float scale = m > 0.f ? __fdiv_rn(m, 127.0f) : 1.0f;
        if (scale_f16) {
            const __half h = __float2half_rn(scale);
            if (lane == 0) reinterpret_cast<__half *>(scales)[b] = h;
            scale = __half2float(h);
        } else if (lane == 0) {
            reinterpret_cast<float *>(scales)[b] = scale;
        }
        for (uint32_t i = lane; i < block; i += kWarp) {
            int v = __float2int_rn(__fdiv_rn(bf16_bits_to_float(w[base + i]), scale));
            v = max(-127, min(127, v));
            q[base + i] = (int8_t)v;
        }
    }
}

__global__ void q8_dequantize_kernel(uint16_t *__restrict__ w, const int8_t *__restrict__ q,
                                     const void *__restrict__ scales, uint64_t count,
                                     uint32_t block, int scale_f16) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        const uint64_t b = i / block;
        const float s = scale_f16 ? __half2float(reinterpret_cast<const __half *>(scales)[b])
                                  : reinterpret_cast<const float *>(scales)[b];
        w[i] = float_to_bf16_bits(__fmul_rn((float)q[i], s));
    }
}

}  // namespace

// ======================================================================= C ABI
extern "C" bool k3_moe_activation_bf16(void *output, const void *gate, const void *up,
                                       uint64_t element_count, int activation, float beta,
                                       float linear_beta, void *stream) {
    if (!output || !gate || !up || element_count == 0) return false;
    if (activation != kActSitu && activation != kActSwiglu) return false;
    if (activation == kActSitu && (beta <= 0.0f || linear_beta <= 0.0f)) return false;
    activation_kernel<<<grid_for((element_count + 7) / 8, kThreads), kThreads, 0,
                        (cudaStream_t)stream>>>((uint16_t *)output, (const uint16_t *)gate,
                                                (const uint16_t *)up, element_count, activation,
                                                beta, linear_beta);
    return launch_ok();
}

extern "C" bool k3_rocm_situ_bf16(void *output, const void *gate, const void *up,
                                  uint64_t element_count, float beta, float linear_beta,
                                  void *stream) {
    if (beta <= 0.0f || linear_beta <= 0.0f) return false;
    return k3_moe_activation_bf16(output, gate, up, element_count, kActSitu, beta, linear_beta,
                                  stream);
}

extern "C" bool k3_rocm_add_bf16(void *output, const void *left, const void *right,
                                 uint64_t element_count, void *stream) {
    if (!output || !left || !right || element_count == 0) return false;
    add_kernel<<<grid_for((element_count + 7) / 8, kThreads), kThreads, 0,
                 (cudaStream_t)stream>>>((uint16_t *)output, (const uint16_t *)left,
                                         (const uint16_t *)right, element_count);
    return launch_ok();
}

extern "C" bool k3_rocm_gather_rows_bf16(void *output, const void *input, const void *row_ids,
                                         uint32_t row_count, uint32_t row_size, void *stream) {
    if (!output || !input || !row_ids || row_count == 0u || row_size == 0u) return false;
    copy_rows_kernel<false><<<grid_for(row_count, kThreads / kWarp), kThreads, 0,
                              (cudaStream_t)stream>>>((uint16_t *)output,
                                                      (const uint16_t *)input,
                                                      (const uint32_t *)row_ids, row_count,
                                                      row_size);
    return launch_ok();
}

extern "C" bool k3_rocm_scatter_rows_bf16(void *output, const void *input, const void *row_ids,
                                          uint32_t row_count, uint32_t row_size, void *stream) {
    if (!output || !input || !row_ids || row_count == 0u || row_size == 0u) return false;
    copy_rows_kernel<true><<<grid_for(row_count, kThreads / kWarp), kThreads, 0,
                             (cudaStream_t)stream>>>((uint16_t *)output, (const uint16_t *)input,
                                                     (const uint32_t *)row_ids, row_count,
                                                     row_size);
    return launch_ok();
}

extern "C" bool k3_rocm_weighted_sum_bf16_batch(void *output, const void *vectors,
                                                const void *weights, uint32_t token_count,
                                                uint32_t vector_count, uint32_t hidden_size,
                                                void *stream) {
    if (!output || !vectors || !weights || token_count == 0u || token_count > 65535u ||
        vector_count == 0 || hidden_size == 0) {
        return false;
    }
    const size_t smem = (size_t)vector_count * sizeof(float);
    if (smem > 48 * 1024) return false;
    weighted_sum_kernel<<<grid_for(token_count, 1), kThreads, smem, (cudaStream_t)stream>>>(
        (uint16_t *)output, (const uint16_t *)vectors, (const float *)weights, token_count,
        vector_count, hidden_size);
    return launch_ok();
}

extern "C" bool k3_rocm_weighted_sum_bf16(void *output, const void *vectors, const void *weights,
                                          uint32_t vector_count, uint32_t hidden_size,
                                          void *stream) {
    return k3_rocm_weighted_sum_bf16_batch(output, vectors, weights, 1u, vector_count,
                                           hidden_size, stream);
}

extern "C" bool k3_rocm_rms_norm_bf16(void *output, const void *input, const void *weight,
                                      uint32_t vector_count, uint32_t hidden_size, float epsilon,
                                      void *stream) {
    if (!output || !input || !weight || vector_count == 0 || hidden_size == 0 ||
        epsilon <= 0.0f) {
        return false;
    }
    rms_norm_kernel<<<grid_for(vector_count, 1), kThreads, 0, (cudaStream_t)stream>>>(
        (uint16_t *)output, (const uint16_t *)input, (const uint16_t *)weight, vector_count,
        hidden_size, epsilon);
    return launch_ok();
}

extern "C" bool k3_rocm_router_topk_f32_batch(void *expert_ids, void *expert_weights,
                                              const void *logits, const void *correction_bias,
                                              uint32_t vector_count, uint32_t expert_count,
                                              uint32_t top_k, float scaling_factor,
                                              void *stream) {
    if (!expert_ids || !expert_weights || !logits || !correction_bias || vector_count == 0u ||
        vector_count > 65535u || expert_count == 0 || top_k == 0 || top_k > expert_count ||
        expert_count > 1024u || top_k > 32u || scaling_factor <= 0.0f) {
        return false;
    }
    router_topk_kernel<<<grid_for(vector_count, 4), 128, 0, (cudaStream_t)stream>>>(
        (uint32_t *)expert_ids, (float *)expert_weights, (const float *)logits,
        (const float *)correction_bias, vector_count, expert_count, top_k, scaling_factor);
    return launch_ok();
}

extern "C" bool k3_rocm_router_topk_f32(void *expert_ids, void *expert_weights,
                                        const void *logits, const void *correction_bias,
                                        uint32_t expert_count, uint32_t top_k,
                                        float scaling_factor, void *stream) {
    return k3_rocm_router_topk_f32_batch(expert_ids, expert_weights, logits, correction_bias, 1u,
                                         expert_count, top_k, scaling_factor, stream);
}

extern "C" bool k3_moe_q8_quantize(void *quantized, void *scales, const void *weights,
                                   uint32_t rows, uint32_t columns, uint32_t block,
                                   int scale_type, void *stream) {
    if (!quantized || !scales || !weights || rows == 0 || columns == 0 || block == 0 ||
        block % 8u != 0 || columns % block != 0 || (scale_type != 0 && scale_type != 1)) {
        return false;
    }
    const uint64_t blocks = (uint64_t)rows * (columns / block);
    q8_quantize_kernel<<<grid_for(blocks, kThreads / kWarp), kThreads, 0,
                         (cudaStream_t)stream>>>((int8_t *)quantized, scales,
                                                 (const uint16_t *)weights, blocks, block,
                                                 scale_type);
    return launch_ok();
}

extern "C" bool k3_rocm_bf16_quantize_q8_128(void *quantized, void *scales, const void *weights,
                                             uint32_t rows, uint32_t columns, void *stream) {
    if (columns % 128u != 0) return false;
    return k3_moe_q8_quantize(quantized, scales, weights, rows, columns, 128u, 0, stream);
}

extern "C" bool k3_rocm_q8_128_dequantize_bf16(void *weights, const void *quantized,
                                               const void *scales, uint32_t rows,
                                               uint32_t columns, void *stream) {
    if (!weights || !quantized || !scales || rows == 0u || columns == 0u ||
        columns % 128u != 0u) {
        return false;
    }
    const uint64_t count = (uint64_t)rows * columns;
    q8_dequantize_kernel<<<grid_for(count, kThreads), kThreads, 0, (cudaStream_t)stream>>>(
        (uint16_t *)weights, (const int8_t *)quantized, scales, count, 128u, 0);
    return launch_ok();
}
