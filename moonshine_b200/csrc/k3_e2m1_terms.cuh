// A bf16 vector as a sum of E2M1 terms with a block scale per term, the form the
// packed block-scaled MMA (tcgen05.mma kind::mxf4) wants for its second operand:
//
//   x[i] = sum_j 2^(s_j[b] - 127) * t_j[i]      b = i / 32, t_j[i] in {0, +-.5, ..., +-6}
//
// Term j is the residual left by terms 0..j-1, rounded to E2M1 under the block scale
// that puts the residual's largest magnitude in [4, 8).  Every term takes at least
// two bits off the block's largest residual, so kTerms = 8 terms reproduce a block
// of bf16 values (8 significant bits) exactly unless an element lies more than 2^16
// below the block maximum; what is left of such an element is below 2^-16 of the
// block maximum.  The terms are rows of the MMA's N operand (N = 16, rows 8..15
// zero), so they cost no extra weight traffic and no extra instructions; the
// epilogue adds the kTerms accumulator columns.
#pragma once

#include "k3_common.cuh"

#include <cuda_fp4.h>

namespace k3 {

constexpr uint32_t kTerms = 8;

// Whole warp, one element of a 32-element block per lane.  code[j]: this lane's E2M1
// nibble of term j; scale_byte[j]: the block's E8M0 byte of term j (same in every lane).
K3_DEVINL void split_block_e2m1(float value, uint32_t (&code)[kTerms], uint32_t (&scale_byte)[kTerms]) {
    float residual = value;
#pragma unroll
    for (uint32_t j = 0; j < kTerms; j++) {
        // non-negative floats order like their bit patterns
        const uint32_t mx = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(residual)) & 0x7fffffffu);
        const uint32_t be = (mx >> 23) & 0xffu;               // biased exponent of the largest residual
        if (be < 4u || be == 0xffu) {                          // nothing (finite) left in this block
            code[j] = 0u;
            scale_byte[j] = 127u;
            continue;
        }
        const uint32_t sb = be - 2u;                           // largest magnitude / 2^(sb-127) in [4, 8)
        const float scaled = residual * __uint_as_float((254u - sb) << 23);
        const uint32_t c = (uint32_t)__nv_cvt_float_to_fp4(scaled, __NV_E2M1, cudaRoundNearest) & 0xfu;
        const float back = __half2float(__half(__nv_cvt_fp4_to_halfraw((__nv_fp4_storage_t)c, __NV_E2M1)));
        residual -= back * __uint_as_float(sb << 23);
        code[j] = c;
        scale_byte[j] = sb;
    }
}

// Stores one block: terms [kTerms rows][row_bytes] packed nibbles (element 2i in the low
// nibble of byte i), scales [kTerms rows][row_blocks].  `block` = index of the 32-element block.
K3_DEVINL void store_block_e2m1(uint8_t *terms, uint8_t *scales, uint64_t row_bytes, uint64_t row_blocks,
                                uint32_t block, const uint32_t (&code)[kTerms],
                                const uint32_t (&scale_byte)[kTerms], uint32_t lane) {
#pragma unroll
    for (uint32_t j = 0; j < kTerms; j++) {
        const uint32_t upper = __shfl_down_sync(0xffffffffu, code[j], 1);
        if ((lane & 1u) == 0u) terms[j * row_bytes + block * 16u + (lane >> 1)] = (uint8_t)(code[j] | (upper << 4));
        if (lane == 0u) scales[j * row_blocks + block] = (uint8_t)scale_byte[j];
    }
}

}  // namespace k3
