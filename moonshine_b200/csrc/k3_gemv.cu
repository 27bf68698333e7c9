// Matrix-vector / small-batch entry points: BF16 (router logits), Q8 block
// quantised (shared expert, static projections) and MXFP4 (routed experts).
// Signatures and argument checks follow the reference operator interface
// (k3_rocm_ops.h:45-182); kernels are new.
//
// Reduction order.  The BF16 and Q8 kernels reproduce the reference's
// 256-lane schedule exactly (lane = column mod 256, or 8-column octet mod 256,
// ascending within a lane, one fused multiply-add per term, then the binary
// tree 128, 64, ... 1), so their results equal the CPU oracle bit for bit.
// Batch entry points run the same code per input row, hence batch == repeated
// single-row calls byte for byte, and the batch_tile argument is validated
// but does not change any result.
#include "k3_gemv.cuh"
#include "k3_moe_ops.h"

#include <algorithm>

using namespace k3;

namespace {

// ------------------------------------------------------------------- BF16
// One warp per weight row.  Thread u keeps the partial sums of virtual lanes
// 8u..8u+7 (columns 256j + 8u + i).
template <typename Out, int VT>
__global__ void __launch_bounds__(256)
bf16_gemm_kernel(Out *__restrict__ out, const uint16_t *__restrict__ w,
                 const uint16_t *__restrict__ x, uint32_t vectors, uint32_t rows,
                 uint32_t columns) {
    const uint32_t lane = threadIdx.x % kWarp;
    const uint32_t warps = (gridDim.x * blockDim.x) / kWarp;
    const bool wide = (columns % 8u == 0) && ((((uintptr_t)w) | ((uintptr_t)x)) & 15u) == 0;
    for (uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) / kWarp; row < rows;
         row += warps) {
        const uint16_t *wr = w + (uint64_t)row * columns;
        for (uint32_t v0 = 0; v0 < vectors; v0 += VT) {
            float acc[VT][8];
#pragma unroll
            for (int v = 0; v < VT; v++)
#pragma unroll
                for (int i = 0; i < 8; i++) acc[v][i] = 0.f;
            for (uint32_t c0 = lane * 8u; c0 < columns; c0 += 256u) {
                float wf[8];
                uint32_t valid = min(8u, columns - c0);
                if (wide) {
                    const uint4 q = *reinterpret_cast<const uint4 *>(wr + c0);
                    wf[0] = bf16_lo(q.x); wf[1] = bf16_hi(q.x); wf[2] = bf16_lo(q.y);
                    wf[3] = bf16_hi(q.y); wf[4] = bf16_lo(q.z); wf[5] = bf16_hi(q.z);
                    wf[6] = bf16_lo(q.w); wf[7] = bf16_hi(q.w);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; i++)
                        wf[i] = (uint32_t)i < valid ? bf16_bits_to_float(wr[c0 + i]) : 0.f;
                }
#pragma unroll
                for (int v = 0; v < VT; v++) {
                    if (v0 + v >= vectors) break;
                    const uint16_t *xr = x + (uint64_t)(v0 + v) * columns + c0;
                    float xf[8];
                    if (wide) {
                        const uint4 q = *reinterpret_cast<const uint4 *>(xr);
                        xf[0] = bf16_lo(q.x); xf[1] = bf16_hi(q.x); xf[2] = bf16_lo(q.y);
                        xf[3] = bf16_hi(q.y); xf[4] = bf16_lo(q.z); xf[5] = bf16_hi(q.z);
                        xf[6] = bf16_lo(q.w); xf[7] = bf16_hi(q.w);
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; i++)
                            xf[i] = (uint32_t)i < valid ? bf16_bits_to_float(xr[i]) : 0.f;
                    }
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        if ((uint32_t)i < valid) acc[v][i] = fmaf(wf[i], xf[i], acc[v][i]);
                    }
                }
            }
#pragma unroll
            for (int v = 0; v < VT; v++) {
                if (v0 + v >= vectors) break;
                // tree over 256 virtual lanes t = 8u + i
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                    for (int i = 0; i < 8; i++)
                        acc[v][i] += __shfl_down_sync(0xffffffffu, acc[v][i], o);
                }
                float r0 = acc[v][0] + acc[v][4], r1 = acc[v][1] + acc[v][5];
                float r2 = acc[v][2] + acc[v][6], r3 = acc[v][3] + acc[v][7];
                r0 += r2; r1 += r3;
                r0 += r1;
                if (lane == 0) {
                    if constexpr (sizeof(Out) == 4) {
                        out[(uint64_t)(v0 + v) * rows + row] = r0;
                    } else {
                        out[(uint64_t)(v0 + v) * rows + row] = float_to_bf16_bits(r0);
                    }
                }
            }
        }
    }
}

// --------------------------------------------------------------------- Q8
// One warp per weight row.  Virtual lane = octet mod 256 = 32*i + u for thread
// u, slot i; 8 sequential fused multiply-adds per octet.
template <int VT>
__global__ void __launch_bounds__(256)
q8_gemm_kernel(uint16_t *__restrict__ out, const int8_t *__restrict__ q,
               const void *__restrict__ scales, const uint16_t *__restrict__ x,
               uint32_t vectors, uint32_t rows, uint32_t columns, uint32_t block,
               int scale_f16) {
    const uint32_t lane = threadIdx.x % kWarp;
    const uint32_t warps = (gridDim.x * blockDim.x) / kWarp;
    const uint32_t octets = columns / 8u;
    const uint32_t blocks_per_row = columns / block;
    for (uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) / kWarp; row < rows;
         row += warps) {
        const int8_t *qr = q + (uint64_t)row * columns;
        const uint64_t sbase = (uint64_t)row * blocks_per_row;
        for (uint32_t v0 = 0; v0 < vectors; v0 += VT) {
            float acc[VT][8];
#pragma unroll
            for (int v = 0; v < VT; v++)
#pragma unroll
                for (int i = 0; i < 8; i++) acc[v][i] = 0.f;
            for (uint32_t o0 = 0; o0 < octets; o0 += 256u) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const uint32_t octet = o0 + 32u * i + lane;
                    if (octet >= octets) continue;
                    const uint2 wq = *reinterpret_cast<const uint2 *>(qr + (uint64_t)octet * 8u);
                    const uint32_t sidx = (octet * 8u) / block;
                    const float s = scale_f16
                                        ? __half2float(reinterpret_cast<const __half *>(scales)[sbase + sidx])
                                        : reinterpret_cast<const float *>(scales)[sbase + sidx];
                    float wf[8];
#pragma unroll
                    for (int b = 0; b < 4; b++) {
                        wf[b] = __fmul_rn((float)(int8_t)(wq.x >> (8 * b)), s);
                        wf[4 + b] = __fmul_rn((float)(int8_t)(wq.y >> (8 * b)), s);
                    }
#pragma unroll
                    for (int v = 0; v < VT; v++) {
                        if (v0 + v >= vectors) break;
                        const uint4 xq = *reinterpret_cast<const uint4 *>(
                            x + (uint64_t)(v0 + v) * columns + (uint64_t)octet * 8u);
                        float a = acc[v][i];
                        a = fmaf(wf[0], bf16_lo(xq.x), a);
                        a = fmaf(wf[1], bf16_hi(xq.x), a);
                        a = fmaf(wf[2], bf16_lo(xq.y), a);
                        a = fmaf(wf[3], bf16_hi(xq.y), a);
                        a = fmaf(wf[4], bf16_lo(xq.z), a);
                        a = fmaf(wf[5], bf16_hi(xq.z), a);
                        a = fmaf(wf[6], bf16_lo(xq.w), a);
                        a = fmaf(wf[7], bf16_hi(xq.w), a);
                        acc[v][i] = a;
                    }
                }
            }
#pragma unroll
            for (int v = 0; v < VT; v++) {
                if (v0 + v >= vectors) break;
                // tree: widths 128, 64, 32 are slot-to-slot, 16..1 lane-to-lane
                float p0 = acc[v][0] + acc[v][4], p1 = acc[v][1] + acc[v][5];
                float p2 = acc[v][2] + acc[v][6], p3 = acc[v][3] + acc[v][7];
                p0 += p2; p1 += p3;
                p0 += p1;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) p0 += __shfl_down_sync(0xffffffffu, p0, o);
                if (lane == 0) out[(uint64_t)(v0 + v) * rows + row] = float_to_bf16_bits(p0);
            }
        }
    }
}

// ------------------------------------------------------------------ MXFP4
// Item = 32 rows.  Two input rows per pass (MMA columns 0-3 and 4-7).
template <bool kAligned16>
__global__ void __launch_bounds__(kGemvThreads)
mxfp4_gemm_kernel(uint16_t *__restrict__ out, const uint8_t *__restrict__ packed,
                  const uint8_t *__restrict__ scales, const uint16_t *__restrict__ x,
                  uint32_t vectors, uint32_t rows, uint32_t k, uint32_t k_pad) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const GemvSmem sm = carve_gemv_smem(smem_raw, k_pad);
    __half *xs = sm.xs;
    float *red = sm.red, *out_s = sm.out_s, *inv_scale = sm.inv_scale, *scratch = sm.scratch;
    const uint32_t items = (rows + kGemvRowsPerItem - 1) / kGemvRowsPerItem;
    for (uint32_t v0 = 0; v0 < vectors; v0 += 2u) {
        const uint32_t nvec = min(2u, vectors - v0);
        __syncthreads();
        stage_vectors_f16(xs, inv_scale, x + (uint64_t)v0 * k,
                          nvec > 1u ? x + (uint64_t)(v0 + 1u) * k : nullptr, k, k_pad, scratch);
        for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
            const uint32_t row0 = item * kGemvRowsPerItem;
            mxfp4_item_32rows<kAligned16>(out_s, red, packed, scales, row0, rows, k, xs, k_pad,
                                          nvec, inv_scale);
            if (threadIdx.x < 64u) {
                const uint32_t vec = threadIdx.x >> 5, r = threadIdx.x & 31u;
                if (vec < nvec && row0 + r < rows) {
                    out[(uint64_t)(v0 + vec) * rows + row0 + r] =
                        float_to_bf16_bits(out_s[vec * 32u + r]);
                }
            }
        }
    }
}

template <typename Out>
bool launch_bf16(void *output, const void *weights, const void *input, uint32_t vectors,
                 uint32_t rows, uint32_t columns, cudaStream_t stream) {
    const uint32_t blocks = (uint32_t)std::min<uint64_t>(((uint64_t)rows + 7) / 8, (uint64_t)sm_count() * 8);
    if (vectors == 1u) {
        bf16_gemm_kernel<Out, 1><<<blocks, 256, 0, stream>>>(
            (Out *)output, (const uint16_t *)weights, (const uint16_t *)input, vectors, rows, columns);
    } else {
        bf16_gemm_kernel<Out, 4><<<blocks, 256, 0, stream>>>(
            (Out *)output, (const uint16_t *)weights, (const uint16_t *)input, vectors, rows, columns);
    }
    return launch_ok();
}

}  // namespace

// ======================================================================= C ABI
extern "C" bool k3_rocm_bf16_gemm_tiled_f32(void *output, const void *weights, const void *input,
                                            uint32_t vector_count, uint32_t rows,
                                            uint32_t columns, uint32_t batch_tile, void *stream) {
    if (!output || !weights || !input || vector_count == 0u || vector_count > 65535u ||
        rows == 0u || columns == 0u) {
        return false;
    }
    if (batch_tile != 16u && batch_tile != 32u && batch_tile != 64u) return false;
    return launch_bf16<float>(output, weights, input, vector_count, rows, columns,
                              (cudaStream_t)stream);
}

extern "C" bool k3_rocm_bf16_gemm_f32(void *output, const void *weights, const void *input,
                                      uint32_t vector_count, uint32_t rows, uint32_t columns,
                                      void *stream) {
    return k3_rocm_bf16_gemm_tiled_f32(output, weights, input, vector_count, rows, columns, 16u,
                                       stream);
}

extern "C" bool k3_rocm_bf16_gemv_f32(void *output, const void *weights, const void *input,
                                      uint32_t rows, uint32_t columns, void *stream) {
    return k3_rocm_bf16_gemm_f32(output, weights, input, 1u, rows, columns, stream);
}

extern "C" bool k3_rocm_bf16_gemm_tiled_bf16(void *output, const void *weights,
                                             const void *input, uint32_t vector_count,
                                             uint32_t rows, uint32_t columns,
                                             uint32_t batch_tile, void *stream) {
    if (!output || !weights || !input || vector_count == 0u || vector_count > 65535u ||
        rows == 0u || columns == 0u) {
        return false;
    }
    if (batch_tile != 16u && batch_tile != 32u && batch_tile != 64u) return false;
    return launch_bf16<uint16_t>(output, weights, input, vector_count, rows, columns,
                                 (cudaStream_t)stream);
}

extern "C" bool k3_rocm_bf16_gemm_bf16(void *output, const void *weights, const void *input,
                                       uint32_t vector_count, uint32_t rows, uint32_t columns,
                                       void *stream) {
    return k3_rocm_bf16_gemm_tiled_bf16(output, weights, input, vector_count, rows, columns, 16u,
                                        stream);
}

extern "C" bool k3_rocm_bf16_gemv_bf16(void *output, const void *weights, const void *input,
                                       uint32_t rows, uint32_t columns, void *stream) {
    return k3_rocm_bf16_gemm_bf16(output, weights, input, 1u, rows, columns, stream);
}

extern "C" bool k3_moe_q8_gemm_bf16(void *output, const void *quantized, const void *scales,
                                    const void *input, uint32_t vector_count, uint32_t rows,
                                    uint32_t columns, uint32_t block, int scale_type,
                                    void *stream) {
    if (!output || !quantized || !scales || !input || vector_count == 0u ||
        vector_count > 65535u || rows == 0u || columns == 0u || block == 0u ||
        block % 8u != 0u || columns % block != 0u || (scale_type != 0 && scale_type != 1)) {
        return false;
    }
    if ((((uintptr_t)quantized) & 7u) != 0 || (((uintptr_t)input) & 15u) != 0) return false;
    const uint32_t blocks = (uint32_t)std::min<uint64_t>(((uint64_t)rows + 7) / 8, (uint64_t)sm_count() * 8);
    if (vector_count == 1u) {
        q8_gemm_kernel<1><<<blocks, 256, 0, (cudaStream_t)stream>>>(
            (uint16_t *)output, (const int8_t *)quantized, scales, (const uint16_t *)input,
            vector_count, rows, columns, block, scale_type);
    } else {
        q8_gemm_kernel<4><<<blocks, 256, 0, (cudaStream_t)stream>>>(
            (uint16_t *)output, (const int8_t *)quantized, scales, (const uint16_t *)input,
            vector_count, rows, columns, block, scale_type);
    }
    return launch_ok();
}

extern "C" bool k3_rocm_q8_128_gemm_tiled_bf16(void *output, const void *quantized,
                                               const void *scales, const void *input,
                                               uint32_t vector_count, uint32_t rows,
                                               uint32_t columns, uint32_t batch_tile,
                                               void *stream) {
    if (columns % 128u != 0u) return false;
    if (batch_tile != 16u && batch_tile != 32u && batch_tile != 64u) return false;
    return k3_moe_q8_gemm_bf16(output, quantized, scales, input, vector_count, rows, columns,
                               128u, 0, stream);
}

extern "C" bool k3_rocm_q8_128_gemm_bf16(void *output, const void *quantized, const void *scales,
                                         const void *input, uint32_t vector_count, uint32_t rows,
                                         uint32_t columns, void *stream) {
    return k3_rocm_q8_128_gemm_tiled_bf16(output, quantized, scales, input, vector_count, rows,
                                          columns, 16u, stream);
}

extern "C" bool k3_rocm_q8_128_gemv_bf16(void *output, const void *quantized, const void *scales,
                                         const void *input, uint32_t rows, uint32_t columns,
                                         void *stream) {
    return k3_rocm_q8_128_gemm_bf16(output, quantized, scales, input, 1u, rows, columns, stream);
}

extern "C" bool k3_rocm_mxfp4_gemm_tiled_bf16(void *output, const void *packed,
                                              const void *scales, const void *input,
                                              uint32_t vector_count, uint32_t rows,
                                              uint32_t columns, uint32_t batch_tile,
                                              void *stream) {
    if (!output || !packed || !scales || !input || vector_count == 0u ||
        vector_count > 65535u || rows == 0u || columns == 0u || columns % 32u != 0u) {
        return false;
    }
    if (batch_tile != 16u && batch_tile != 32u && batch_tile != 64u) return false;
    if ((((uintptr_t)packed) & 7u) != 0) return false;   // the format guarantees 8 bytes
    const uint32_t k_pad = (columns + 127u) / 128u * 128u;
    const size_t smem = gemv_smem_bytes(k_pad);
    const uint32_t items = (rows + kGemvRowsPerItem - 1) / kGemvRowsPerItem;
    const uint32_t blocks = std::min(items, (uint32_t)sm_count() * 2u);
    const bool aligned = (((uintptr_t)packed) & 15u) == 0;
    auto kernel = aligned ? mxfp4_gemm_kernel<true> : mxfp4_gemm_kernel<false>;
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
    }
    kernel<<<blocks, kGemvThreads, smem, (cudaStream_t)stream>>>(
        (uint16_t *)output, (const uint8_t *)packed, (const uint8_t *)scales,
        (const uint16_t *)input, vector_count, rows, columns, k_pad);
    return launch_ok();
}

extern "C" bool k3_rocm_mxfp4_gemm_bf16(void *output, const void *packed, const void *scales,
                                        const void *input, uint32_t vector_count, uint32_t rows,
                                        uint32_t columns, void *stream) {
    return k3_rocm_mxfp4_gemm_tiled_bf16(output, packed, scales, input, vector_count, rows,
                                         columns, 16u, stream);
}

extern "C" bool k3_rocm_mxfp4_gemv_bf16(void *output, const void *packed, const void *scales,
                                        const void *input, uint32_t rows, uint32_t columns,
                                        void *stream) {
    return k3_rocm_mxfp4_gemm_bf16(output, packed, scales, input, 1u, rows, columns, stream);
}
