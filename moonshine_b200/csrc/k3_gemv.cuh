// Bandwidth-bound matrix-vector building blocks shared by the legacy entry
// points and the fused decode path.
//
// MXFP4 rows are consumed in their checkpoint-native form: packed [rows, K/2]
// (even column = low nibble) and E8M0 scales [rows, K/32].  A warp owns 16
// rows.  Every lane streams 16-byte nibble chunks (one 32-column scale group)
// of rows g and g+8, converts them in registers to f16 (exact) with byte-permute
// table lookups, and feeds them to mma.sync.m16n8k16 as the A operand.  The B operand is block-diagonal: column n of the MMA carries the
// activation slice of scale group n only, so after 8 MMAs the accumulator
// column n holds the fp32 dot product of exactly one 32-column group.  The
// E8M0 scale (a power of two) is then applied with one fp32 FMA per group into
// a running fp32 sum - the same "dot per group, scale, accumulate" structure
// as the reference kernel (k3_rocm_ops.cu:193-273), with the 32 products of a
// group summed by the tensor core in fp32.
//
// Activations are held in shared memory as f16 after an exact power-of-two
// rescale that maps the vector's largest magnitude into [2^14, 2^15): every
// bf16 value within 2^28 of the maximum converts without rounding, and the
// inverse power of two is applied to the final sum.
#pragma once

#include "k3_common.cuh"

#include <cuda_fp16.h>

namespace k3 {

constexpr int kGemvWarps = 8;               // warps per CTA
constexpr int kGemvThreads = kGemvWarps * kWarp;
constexpr int kGemvKSplit = 4;              // warps sharing one 16-row block along K
constexpr int kGemvRowBlocks = kGemvWarps / kGemvKSplit;  // 16-row blocks per CTA item
constexpr int kGemvRowsPerItem = 16 * kGemvRowBlocks;     // 32

// Eight E2M1 nibbles (one 32-bit word, low nibble first) -> four f16x2
// registers holding elements (0,1), (2,3), (4,5), (6,7).  The f16 encodings of
// the magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 have a zero low byte, so one PRMT
// looks up four high bytes at once; signs are gathered with a second PRMT and
// the bytes are then spread into 16-bit lanes.  Everything runs on the integer
// pipe (the hardware e2m1x2 conversion is issued at a quarter of that rate).
constexpr uint32_t kF16HiLut0 = 0x3E3C3800u, kF16HiLut1 = 0x46444240u;

K3_DEVINL void dequant_word_f16(uint32_t w, uint32_t (&out)[4]) {
    const uint32_t sel = w & 0x77777777u;
    uint32_t m03 = __byte_perm(kF16HiLut0, kF16HiLut1, sel);
    uint32_t m47 = __byte_perm(kF16HiLut0, kF16HiLut1, sel >> 16);
    const uint32_t w4 = w << 4;
    m03 |= __byte_perm(w4, w, 0x5140u) & 0x80808080u;
    m47 |= __byte_perm(w4, w, 0x7362u) & 0x80808080u;
    out[0] = __byte_perm(m03, 0u, 0x1404u);
    out[1] = __byte_perm(m03, 0u, 0x3424u);
    out[2] = __byte_perm(m47, 0u, 0x1404u);
    out[3] = __byte_perm(m47, 0u, 0x3424u);
}

K3_DEVINL void mma_f16_m16n8k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Stage `nvec` (1 or 2) bf16 vectors of K columns into shared memory as f16,
// zero padded to k_pad (multiple of 128).  Returns through inv_scale[v] the
// power of two to multiply final sums with.  All threads of the CTA call it.
template <int kSlots>
K3_DEVINL void stage_vectors_f16_n(__half *xs, float *inv_scale, const uint16_t *x0,
                                   const uint16_t *x1, uint32_t k, uint32_t k_pad,
                                   float *scratch /* >= 2*warps floats */) {
    const uint32_t tid = threadIdx.x;
    const uint32_t nthreads = blockDim.x;
    const uint16_t *src[2] = {x0, x1};
    float mx[2] = {0.f, 0.f};
    // Fast path, same arithmetic: every thread fetches its share with 16-byte loads
    // that are all in flight at once and converts from registers, instead of two
    // passes of 2-byte loads that each wait a memory round trip per few elements.
    const uint32_t chunks = k / 8u;
    if (k == k_pad && k % 8u == 0u && chunks <= 4u * nthreads &&
        ((reinterpret_cast<uintptr_t>(x0) | reinterpret_cast<uintptr_t>(x1)) & 15u) == 0u) {
        uint4 held[2][4];
#pragma unroll
        for (int v = 0; v < kSlots; v++) {
            if (src[v] == nullptr) continue;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t c = tid + (uint32_t)j * nthreads;
                held[v][j] = c < chunks ? reinterpret_cast<const uint4 *>(src[v])[c] : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t w[4] = {held[v][j].x, held[v][j].y, held[v][j].z, held[v][j].w};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    mx[v] = fmaxf(mx[v], fabsf(__uint_as_float(w[q] << 16)));
                    mx[v] = fmaxf(mx[v], fabsf(__uint_as_float(w[q] & 0xffff0000u)));
                }
            }
            mx[v] = warp_max(mx[v]);
            if ((tid % kWarp) == 0) scratch[v * (nthreads / kWarp) + tid / kWarp] = mx[v];
        }
        __syncthreads();
#pragma unroll
        for (int v = 0; v < kSlots; v++) {
            float m = 0.f;
            for (uint32_t w = 0; w < nthreads / kWarp; w++) m = fmaxf(m, scratch[v * (nthreads / kWarp) + w]);
            int e = 0;
            if (m > 0.f && m <= 3.0e38f) {
                e = (int)((__float_as_uint(m) >> 23) & 0xffu) - 127 - 14;
                e = max(-100, min(100, e));
            }
            const float mul = __uint_as_float((uint32_t)(127 - e) << 23);   // 2^-e
            if (tid == 0) inv_scale[v] = __uint_as_float((uint32_t)(127 + e) << 23);  // 2^e
            uint4 *dst = reinterpret_cast<uint4 *>(xs + (size_t)v * k_pad);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t c = tid + (uint32_t)j * nthreads;
                if (c >= chunks) continue;
                uint4 o = make_uint4(0u, 0u, 0u, 0u);
                if (src[v] != nullptr) {
                    const uint32_t w[4] = {held[v][j].x, held[v][j].y, held[v][j].z, held[v][j].w};
                    uint32_t h[4];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const __half2 p = __floats2half2_rn(__uint_as_float(w[q] << 16) * mul,
                                                            __uint_as_float(w[q] & 0xffff0000u) * mul);
                        h[q] = *reinterpret_cast<const uint32_t *>(&p);
                    }
                    o = make_uint4(h[0], h[1], h[2], h[3]);
                }
                dst[c] = o;
            }
        }
        __syncthreads();
        return;
    }
#pragma unroll
    for (int v = 0; v < kSlots; v++) {
        if (src[v] == nullptr) continue;
        for (uint32_t i = tid; i < k; i += nthreads) {
            mx[v] = fmaxf(mx[v], fabsf(bf16_bits_to_float(src[v][i])));
        }
        mx[v] = warp_max(mx[v]);
        if ((tid % kWarp) == 0) scratch[v * (nthreads / kWarp) + tid / kWarp] = mx[v];
    }
    __syncthreads();
    float mul[2];
#pragma unroll
    for (int v = 0; v < kSlots; v++) {
        float m = 0.f;
        for (uint32_t w = 0; w < nthreads / kWarp; w++) m = fmaxf(m, scratch[v * (nthreads / kWarp) + w]);
        int e = 0;
        if (m > 0.f && m <= 3.0e38f) {
            e = (int)((__float_as_uint(m) >> 23) & 0xffu) - 127 - 14;
            e = max(-100, min(100, e));
        }
        mul[v] = __uint_as_float((uint32_t)(127 - e) << 23);   // 2^-e
        if (tid == 0) inv_scale[v] = __uint_as_float((uint32_t)(127 + e) << 23);  // 2^e
    }
#pragma unroll
    for (int v = 0; v < kSlots; v++) {
        __half *dst = xs + (size_t)v * k_pad;
        for (uint32_t i = tid; i < k_pad; i += nthreads) {
            float val = 0.f;
            if (src[v] != nullptr && i < k) val = bf16_bits_to_float(src[v][i]) * mul[v];
            dst[i] = __float2half_rn(val);
        }
    }
    __syncthreads();
}

// two slots (the second zero-filled when x1 is null)
K3_DEVINL void stage_vectors_f16(__half *xs, float *inv_scale, const uint16_t *x0,
                                 const uint16_t *x1, uint32_t k, uint32_t k_pad,
                                 float *scratch /* >= 2*warps floats */) {
    stage_vectors_f16_n<2>(xs, inv_scale, x0, x1, k, k_pad, scratch);
}

// ---------------------------------------------------------------------------
// Q8 rows on the same tensor-core scheme.  A lane streams the 32 int8 of one
// scale-width group (32 columns) of rows g and g+8 per 128-column step, converts
// them to f16 exactly (byte spliced under the mantissa of 1024.0, then 1152.0
// subtracted, two elements per instruction) and feeds mma.sync with the
// block-diagonal B operand, so accumulator column n is the fp32 dot product of
// group n alone; the block scale (fp16 or fp32, block % 32 == 0) is applied with
// one fp32 FMA per group.  Products are exact, sums are fp32; only the order of
// the fp32 additions differs from the reference's Q8 kernel.

// four int8 (one word) -> f16x2 pairs (e0, e1) and (e2, e3)
K3_DEVINL void int8x4_to_f16(uint32_t w, uint32_t &p01, uint32_t &p23) {
    const uint32_t u = w ^ 0x80808080u;
    const uint32_t h01 = __byte_perm(u, 0x64646464u, 0x4140u);
    const uint32_t h23 = __byte_perm(u, 0x64646464u, 0x4342u);
    const __half2 bias = __halves2half2(__ushort_as_half((unsigned short)0x6480u),
                                        __ushort_as_half((unsigned short)0x6480u));
    const __half2 a = __hsub2(*reinterpret_cast<const __half2 *>(&h01), bias);
    const __half2 b = __hsub2(*reinterpret_cast<const __half2 *>(&h23), bias);
    p01 = *reinterpret_cast<const uint32_t *>(&a);
    p23 = *reinterpret_cast<const uint32_t *>(&b);
}

struct Q8Step {
    uint4 a0, a1, b0, b1;      // 32 int8 of row g (a) and row g+8 (b)
    float sa0, sa1, sb0, sb1;  // scales of the two groups this lane accumulates
};

K3_DEVINL float q8_scale_at(const void *scales, uint64_t index, int scale_f16) {
    return scale_f16 ? __half2float(reinterpret_cast<const __half *>(scales)[index])
                     : reinterpret_cast<const float *>(scales)[index];
}

// One 128-column step of 16 Q8 rows on this lane: `cur` holds the lane's 32 int8 of rows g
// and g + 8 and their two group scales, `x_step` points at the lane's 32 f16 of the vector
// for this step (only lanes with b_active carry vector values, the others zeros).
K3_DEVINL void q8_step_apply(float &acc_a, float &acc_b, const Q8Step &cur, const __half *x_step, bool b_active) {
    uint32_t xr[16];
    if (b_active) {
        const uint4 *p = reinterpret_cast<const uint4 *>(x_step);
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const uint4 v = p[w];
            xr[4 * w] = v.x; xr[4 * w + 1] = v.y; xr[4 * w + 2] = v.z; xr[4 * w + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int w = 0; w < 16; w++) xr[w] = 0u;
    }
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t wa[8] = {cur.a0.x, cur.a0.y, cur.a0.z, cur.a0.w, cur.a1.x, cur.a1.y, cur.a1.z, cur.a1.w};
    const uint32_t wb[8] = {cur.b0.x, cur.b0.y, cur.b0.z, cur.b0.w, cur.b1.x, cur.b1.y, cur.b1.z, cur.b1.w};
#pragma unroll
    for (int w = 0; w < 8; w++) {
        uint32_t a01, a23, b01, b23;
        int8x4_to_f16(wa[w], a01, a23);
        int8x4_to_f16(wb[w], b01, b23);
        mma_f16_m16n8k16(c, a01, b01, a23, b23, xr[2 * w], xr[2 * w + 1]);
    }
    acc_a = fmaf(cur.sa0, c[0], acc_a);
    acc_a = fmaf(cur.sa1, c[1], acc_a);
    acc_b = fmaf(cur.sb0, c[2], acc_b);
    acc_b = fmaf(cur.sb1, c[3], acc_b);
}

// One warp: partial dot products of 16 consecutive Q8 rows [row0, row0+16) of a
// [rows, k] matrix (k % 128 == 0, block % 32 == 0) with the f16 vector xs over the
// 128-column steps [step_begin, step_end).  After the call lanes with t == 0 hold
// the partial sums of rows g (r0) and g + 8 (r1), g = lane / 4.
template <int kDepth>
K3_DEVINL void q8_rows16_partial(float &r0, float &r1, const int8_t *q, const void *scales,
                                 int scale_f16, uint32_t block, uint32_t row0, uint32_t k,
                                 uint32_t step_begin, uint32_t step_end, const __half *xs) {
    const uint32_t lane = threadIdx.x % kWarp;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const int8_t *pa = q + (uint64_t)(row0 + g) * k;
    const int8_t *pb = q + (uint64_t)(row0 + g + 8u) * k;
    const uint64_t sa = (uint64_t)(row0 + g) * (k / block), sb = (uint64_t)(row0 + g + 8u) * (k / block);
    const bool b_active = g == t;                 // column g carries group t of the vector
    const __half *xv = xs + 32u * t;
    const uint32_t sgrp = 2u * (t & 1u);
    auto fetch = [&](uint32_t step) {
        Q8Step p;
        const uint32_t col = 128u * step + 32u * t;
        p.a0 = ld_stream_16(pa + col);
        p.a1 = ld_stream_16(pa + col + 16u);
        p.b0 = ld_stream_16(pb + col);
        p.b1 = ld_stream_16(pb + col + 16u);
        const uint32_t c0 = 128u * step + 32u * sgrp;
        p.sa0 = q8_scale_at(scales, sa + c0 / block, scale_f16);
        p.sa1 = q8_scale_at(scales, sa + (c0 + 32u) / block, scale_f16);
        p.sb0 = q8_scale_at(scales, sb + c0 / block, scale_f16);
        p.sb1 = q8_scale_at(scales, sb + (c0 + 32u) / block, scale_f16);
        return p;
    };
    Q8Step pf[kDepth];
#pragma unroll
    for (int i = 0; i < kDepth; i++) {
        if (step_begin + i < step_end) pf[i] = fetch(step_begin + i);
    }
    float acc_a = 0.f, acc_b = 0.f;
    for (uint32_t step0 = step_begin; step0 < step_end; step0 += kDepth) {
#pragma unroll
        for (int i = 0; i < kDepth; i++) {
            const uint32_t step = step0 + i;
            if (step >= step_end) break;
            const Q8Step cur = pf[i];
            if (step + kDepth < step_end) pf[i] = fetch(step + kDepth);
            q8_step_apply(acc_a, acc_b, cur, xv + 128u * step, b_active);
        }
    }
    // lanes t = 0 and 1 hold the two halves (groups 0,1 and 2,3) of every step
    acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 1);
    acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 1);
    r0 = acc_a;
    r1 = acc_b;
}

// Partial sums of one 16-row block over 128-column steps [step_begin, step_end).
// sum[0] / sum[1]: rows g / g+8 for the vector this lane accumulates
// (lanes t=0,1 -> vector 0; t=2,3 -> vector 1), already reduced over the lane
// pair.  Rows >= rows_valid are clamped (their sums are garbage, not stored).
template <bool kAligned16>
K3_DEVINL void mxfp4_rowblock_partial(float (&sum)[2], const uint8_t *packed, const uint8_t *scales,
                                      uint32_t row0, uint32_t rows_valid_end, uint32_t k,
                                      uint32_t step_begin, uint32_t step_end, const __half *xs,
                                      uint32_t k_pad, uint32_t nvec) {
    const uint32_t lane = threadIdx.x % kWarp;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t groups = k / 32u;
    const uint32_t row_a = min(row0 + g, rows_valid_end - 1u);
    const uint32_t row_b = min(row0 + g + 8u, rows_valid_end - 1u);
    const uint8_t *pa = packed + (uint64_t)row_a * (k / 2u);
    const uint8_t *pb = packed + (uint64_t)row_b * (k / 2u);
    const uint8_t *sa = scales + (uint64_t)row_a * groups;
    const uint8_t *sb = scales + (uint64_t)row_b * groups;
    // B operand: lane (g,t) carries data only when (g & 3) == t; vector g >> 2.
    const uint32_t bvec = g >> 2;
    const bool b_active = ((g & 3u) == t) && (bvec < nvec);
    const __half *xv = xs + (size_t)bvec * k_pad + 32u * t;
    // scale groups this lane applies: 4*step + 2*(t&1) + {0,1}
    const uint32_t sgrp = 2u * (t & 1u);
    float acc_a = 0.f, acc_b = 0.f;
#pragma unroll 2
    for (uint32_t step = step_begin; step < step_end; step++) {
        const uint32_t grp = 4u * step + t;       // the group whose nibbles this lane loads
        uint4 wa = make_uint4(0, 0, 0, 0), wb = make_uint4(0, 0, 0, 0);
        if (grp < groups) {
            if (kAligned16) {
                wa = ld_stream_16(pa + (uint64_t)grp * 16u);
                wb = ld_stream_16(pb + (uint64_t)grp * 16u);
            } else {
                const uint2 a0 = ld_stream_8(pa + (uint64_t)grp * 16u);
                const uint2 a1 = ld_stream_8(pa + (uint64_t)grp * 16u + 8u);
                const uint2 b0 = ld_stream_8(pb + (uint64_t)grp * 16u);
                const uint2 b1 = ld_stream_8(pb + (uint64_t)grp * 16u + 8u);
                wa = make_uint4(a0.x, a0.y, a1.x, a1.y);
                wb = make_uint4(b0.x, b0.y, b1.x, b1.y);
            }
        }
        uint32_t xr[16];
        if (b_active) {
            const uint4 *p = reinterpret_cast<const uint4 *>(xv + 128u * step);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const uint4 v = p[q];
                xr[4 * q + 0] = v.x; xr[4 * q + 1] = v.y; xr[4 * q + 2] = v.z; xr[4 * q + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int q = 0; q < 16; q++) xr[q] = 0u;
        }
        // scales of the two groups this lane finishes, rows a and b
        const uint32_t g0 = 4u * step + sgrp;
        float s_a0 = 0.f, s_a1 = 0.f, s_b0 = 0.f, s_b1 = 0.f;
        if (g0 < groups) { s_a0 = e8m0_to_float(sa[g0]); s_b0 = e8m0_to_float(sb[g0]); }
        if (g0 + 1u < groups) { s_a1 = e8m0_to_float(sa[g0 + 1u]); s_b1 = e8m0_to_float(sb[g0 + 1u]); }

        float c[4] = {0.f, 0.f, 0.f, 0.f};
        const uint32_t wa_w[4] = {wa.x, wa.y, wa.z, wa.w};
        const uint32_t wb_w[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t fa[4], fb[4];          // elements 8i .. 8i+7 of rows g and g+8
            dequant_word_f16(wa_w[i], fa);
            dequant_word_f16(wb_w[i], fb);
            mma_f16_m16n8k16(c, fa[0], fb[0], fa[1], fb[1], xr[4 * i], xr[4 * i + 1]);
            mma_f16_m16n8k16(c, fa[2], fb[2], fa[3], fb[3], xr[4 * i + 2], xr[4 * i + 3]);
        }
        acc_a = fmaf(s_a0, c[0], acc_a);
        acc_a = fmaf(s_a1, c[1], acc_a);
        acc_b = fmaf(s_b0, c[2], acc_b);
        acc_b = fmaf(s_b1, c[3], acc_b);
    }
    // lanes t and t^1 hold the two halves of the same vector
    acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 1);
    acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 1);
    sum[0] = acc_a;
    sum[1] = acc_b;
}

// One CTA item: two 16-row blocks, each with its own matrix / first row, K
// split over 4 warps per block.  Results (fp32, already multiplied by
// inv_scale) land in out_s[vec][32] (block 0 -> entries 0..15, block 1 ->
// 16..31) in shared memory; a __syncthreads() separates them from the caller's
// epilogue.  red must hold kGemvWarps*32 floats.
struct RowBlock {
    const uint8_t *packed;
    const uint8_t *scales;
    uint32_t row0;       // first row of the block
    uint32_t rows_end;   // rows in the matrix (block is skipped if row0 >= rows_end)
};

template <bool kAligned16>
K3_DEVINL void mxfp4_item_2x16(float *out_s /* [2][32] */, float *red, const RowBlock &b0,
                               const RowBlock &b1, uint32_t k, const __half *xs, uint32_t k_pad,
                               uint32_t nvec, const float *inv_scale) {
    const uint32_t warp = threadIdx.x / kWarp;
    const uint32_t lane = threadIdx.x % kWarp;
    const uint32_t rb = warp / kGemvKSplit;       // row block inside the item
    const uint32_t ks = warp % kGemvKSplit;       // K split index
    const uint32_t steps = k_pad / 128u;
    const uint32_t per = (steps + kGemvKSplit - 1) / kGemvKSplit;
    const uint32_t sb = min(steps, ks * per), se = min(steps, sb + per);
    const RowBlock &b = rb == 0u ? b0 : b1;
    float sum[2] = {0.f, 0.f};
    if (b.row0 < b.rows_end) {
        mxfp4_rowblock_partial<kAligned16>(sum, b.packed, b.scales, b.row0, b.rows_end, k, sb, se,
                                           xs, k_pad, nvec);
    }
    const uint32_t g = lane >> 2, t = lane & 3u;
    if ((t & 1u) == 0u) {
        const uint32_t vec = t >> 1;
        red[((warp * 2u + vec) * 16u) + g] = sum[0];
        red[((warp * 2u + vec) * 16u) + g + 8u] = sum[1];
    }
    __syncthreads();
    // 64 outputs (2 vectors x 32 rows): sum the K splits in ascending order
    if (threadIdx.x < 64u) {
        const uint32_t vec = threadIdx.x >> 5, r = threadIdx.x & 31u;
        const uint32_t block = r >> 4, rr = r & 15u;
        float total = 0.f;
#pragma unroll
        for (uint32_t s = 0; s < (uint32_t)kGemvKSplit; s++) {
            total += red[(((block * kGemvKSplit + s) * 2u + vec) * 16u) + rr];
        }
        out_s[vec * 32u + r] = total * inv_scale[vec];
    }
    __syncthreads();
}

template <bool kAligned16>
K3_DEVINL void mxfp4_item_32rows(float *out_s, float *red, const uint8_t *packed,
                                 const uint8_t *scales, uint32_t row0, uint32_t rows_end,
                                 uint32_t k, const __half *xs, uint32_t k_pad, uint32_t nvec,
                                 const float *inv_scale) {
    const RowBlock b0{packed, scales, row0, rows_end};
    const RowBlock b1{packed, scales, row0 + 16u, rows_end};
    mxfp4_item_2x16<kAligned16>(out_s, red, b0, b1, k, xs, k_pad, nvec, inv_scale);
}

// Shared-memory layout used by every kernel built on the item routine.
struct GemvSmem {
    __half *xs;        // [2][k_pad]
    float *red;        // [kGemvWarps*32]
    float *out_s;      // [64]
    float *inv_scale;  // [2]
    float *scratch;    // [2*kGemvWarps]
};

K3_DEVINL GemvSmem carve_gemv_smem(unsigned char *raw, uint32_t k_pad) {
    GemvSmem s;
    s.xs = reinterpret_cast<__half *>(raw);
    s.red = reinterpret_cast<float *>(raw + (size_t)2 * k_pad * sizeof(__half));
    s.out_s = s.red + kGemvWarps * 32;
    s.inv_scale = s.out_s + 64;
    s.scratch = s.inv_scale + 2;
    return s;
}

inline size_t gemv_smem_bytes(uint32_t k_pad) {
    return (size_t)2 * k_pad * sizeof(__half) +
           (size_t)(kGemvWarps * 32 + 64 + 2 + 2 * kGemvWarps) * sizeof(float);
}

}  // namespace k3
