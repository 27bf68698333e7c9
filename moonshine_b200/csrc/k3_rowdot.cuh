// Exact-order row dot products shared by the one-token kernels: one warp per
// weight row, the reference's 256-lane schedule (see k3_gemv.cu).
#pragma once

#include "k3_common.cuh"

namespace k3 {

// byte `index` of `word` as a signed 8-bit integer -> float, exactly, without the
// conversion unit: (q + 128) is spliced into the mantissa of 2^23 and the offset
// is subtracted in fp32 (both steps exact).
K3_DEVINL float int8_to_float(uint32_t word, int index) {
    const uint32_t spliced = __byte_perm(word ^ 0x80808080u, 0x4B000000u, 0x7540u | (uint32_t)index);
    return __uint_as_float(spliced) - 8388736.0f;
}

// BF16 row x vector in the reference's order (lane = column mod 256, fused
// multiply-add per term, tree 128..1); one warp, result valid in lane 0.
K3_DEVINL float bf16_row_dot_exact(const uint16_t *__restrict__ wr, const uint16_t *__restrict__ x,
                                   uint32_t columns, uint32_t lane) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (uint32_t c0 = lane * 8u; c0 < columns; c0 += 256u) {
        const uint4 q = *reinterpret_cast<const uint4 *>(wr + c0);
        const uint4 v = *reinterpret_cast<const uint4 *>(x + c0);
        acc[0] = fmaf(bf16_lo(q.x), bf16_lo(v.x), acc[0]);
        acc[1] = fmaf(bf16_hi(q.x), bf16_hi(v.x), acc[1]);
        acc[2] = fmaf(bf16_lo(q.y), bf16_lo(v.y), acc[2]);
        acc[3] = fmaf(bf16_hi(q.y), bf16_hi(v.y), acc[3]);
        acc[4] = fmaf(bf16_lo(q.z), bf16_lo(v.z), acc[4]);
        acc[5] = fmaf(bf16_hi(q.z), bf16_hi(v.z), acc[5]);
        acc[6] = fmaf(bf16_lo(q.w), bf16_lo(v.w), acc[6]);
        acc[7] = fmaf(bf16_hi(q.w), bf16_hi(v.w), acc[7]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int i = 0; i < 8; i++) acc[i] += __shfl_down_sync(0xffffffffu, acc[i], o);
    }
    float r0 = acc[0] + acc[4], r1 = acc[1] + acc[5], r2 = acc[2] + acc[6], r3 = acc[3] + acc[7];
    r0 += r2; r1 += r3;
    return r0 + r1;
}

// Q8 row x vector in the reference's order (lane = octet mod 256, eight fused
// multiply-adds per octet, tree); one warp, result valid in lane 0.
K3_DEVINL float q8_row_dot_exact(const int8_t *__restrict__ qr, const void *__restrict__ scales,
                                 uint64_t scale_base, const uint16_t *__restrict__ x,
                                 uint32_t columns, uint32_t block, int scale_f16, uint32_t lane) {
    const uint32_t octets = columns / 8u;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (uint32_t o0 = 0; o0 < octets; o0 += 256u) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t octet = o0 + 32u * i + lane;
            if (octet >= octets) continue;
            const uint2 wq = *reinterpret_cast<const uint2 *>(qr + (uint64_t)octet * 8u);
            const uint32_t sidx = (octet * 8u) / block;
            const float s = scale_f16
                                ? __half2float(reinterpret_cast<const __half *>(scales)[scale_base + sidx])
                                : reinterpret_cast<const float *>(scales)[scale_base + sidx];
            const uint4 xq = *reinterpret_cast<const uint4 *>(x + (uint64_t)octet * 8u);
            float a = acc[i];
            a = fmaf(__fmul_rn(int8_to_float(wq.x, 0), s), bf16_lo(xq.x), a);
            a = fmaf(__fmul_rn(int8_to_float(wq.x, 1), s), bf16_hi(xq.x), a);
            a = fmaf(__fmul_rn(int8_to_float(wq.x, 2), s), bf16_lo(xq.y), a);
            a = fmaf(__fmul_rn(int8_to_float(wq.x, 3), s), bf16_hi(xq.y), a);
            a = fmaf(__fmul_rn(int8_to_float(wq.y, 0), s), bf16_lo(xq.z), a);
            a = fmaf(__fmul_rn(int8_to_float(wq.y, 1), s), bf16_hi(xq.z), a);
            a = fmaf(__fmul_rn(int8_to_float(wq.y, 2), s), bf16_lo(xq.w), a);
            a = fmaf(__fmul_rn(int8_to_float(wq.y, 3), s), bf16_hi(xq.w), a);
            acc[i] = a;
        }
    }
    float p0 = acc[0] + acc[4], p1 = acc[1] + acc[5], p2 = acc[2] + acc[6], p3 = acc[3] + acc[7];
    p0 += p2; p1 += p3;
    p0 += p1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) p0 += __shfl_down_sync(0xffffffffu, p0, o);
    return p0;
}

}  // namespace k3
