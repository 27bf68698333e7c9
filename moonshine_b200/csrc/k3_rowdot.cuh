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
    // four 256-column passes per trip, all loads issued before the arithmetic
    for (uint32_t c0 = lane * 8u; c0 < columns; c0 += 1024u) {
        uint4 q[4], v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const uint32_t c = c0 + 256u * u;
            const bool in = c < columns;
            q[u] = in ? ld_stream_16(wr + c) : make_uint4(0, 0, 0, 0);
            v[u] = *reinterpret_cast<const uint4 *>(x + (in ? c : 0u));
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            if (c0 + 256u * u >= columns) break;
            acc[0] = fmaf(bf16_lo(q[u].x), bf16_lo(v[u].x), acc[0]);
            acc[1] = fmaf(bf16_hi(q[u].x), bf16_hi(v[u].x), acc[1]);
            acc[2] = fmaf(bf16_lo(q[u].y), bf16_lo(v[u].y), acc[2]);
            acc[3] = fmaf(bf16_hi(q[u].y), bf16_hi(v[u].y), acc[3]);
            acc[4] = fmaf(bf16_lo(q[u].z), bf16_lo(v[u].z), acc[4]);
            acc[5] = fmaf(bf16_hi(q[u].z), bf16_hi(v[u].z), acc[5]);
            acc[6] = fmaf(bf16_lo(q[u].w), bf16_lo(v[u].w), acc[6]);
            acc[7] = fmaf(bf16_hi(q[u].w), bf16_hi(v[u].w), acc[7]);
        }
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
        // all eight weight and scale loads of the pass are issued before the arithmetic
        uint2 wq[8];
        float sc[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t octet = o0 + 32u * i + lane;
            const bool in = octet < octets;
            wq[i] = in ? ld_stream_8(qr + (uint64_t)octet * 8u) : make_uint2(0, 0);
            const uint32_t sidx = in ? (octet * 8u) / block : 0u;
            sc[i] = scale_f16 ? __half2float(reinterpret_cast<const __half *>(scales)[scale_base + sidx])
                              : reinterpret_cast<const float *>(scales)[scale_base + sidx];
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t octet = o0 + 32u * i + lane;
            if (octet >= octets) continue;
            const uint4 xq = *reinterpret_cast<const uint4 *>(x + (uint64_t)octet * 8u);
            const float s = sc[i];
            float a = acc[i];
            a = fmaf(__fmul_rn(int8_to_float(wq[i].x, 0), s), bf16_lo(xq.x), a);
            a = fmaf(__fmul_rn(int8_to_float(wq[i].x, 1), s), bf16_hi(xq.x), a);
            a = fmaf(__fmul_rn(int8_to_float(wq[i].x, 2), s), bf16_lo(xq.y), a);
            a = fmaf(__fmul_rn(int8_to_float(wq[i].x, 3), s), bf16_hi(xq.y), a);
            a = fmaf(__fmul_rn(int8_to_float(wq[i].y, 0), s), bf16_lo(xq.z), a);
            a = fmaf(__fmul_rn(int8_to_float(wq[i].y, 1), s), bf16_hi(xq.z), a);
            a = fmaf(__fmul_rn(int8_to_float(wq[i].y, 2), s), bf16_lo(xq.w), a);
            a = fmaf(__fmul_rn(int8_to_float(wq[i].y, 3), s), bf16_hi(xq.w), a);
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

// ---------------------------------------------------------------------------
// The same two dot products with one 256-thread block per row: thread v is the
// reference's lane v, so a whole row is in flight after one round of loads.
// Results are bit-identical to the warp versions above (same per-lane chains,
// same 128..1 tree).

constexpr uint32_t kRowBlock = 256;

// tree over the 256 lane sums: strides 128, 64, 32 through shared memory, 16..1 by
// shuffles.  `red` holds 256 floats; the caller alternates two buffers between
// consecutive rows so that one __syncthreads per row suffices.  Valid in thread 0.
K3_DEVINL float block_tree_256(float v, float *red) {
    red[threadIdx.x] = v;
    __syncthreads();
    float p0 = 0.f;
    if (threadIdx.x < kWarp) {
        const uint32_t lane = threadIdx.x;
        float a0 = red[lane] + red[lane + 128u], a1 = red[lane + 32u] + red[lane + 160u];
        float a2 = red[lane + 64u] + red[lane + 192u], a3 = red[lane + 96u] + red[lane + 224u];
        a0 += a2; a1 += a3;
        p0 = a0 + a1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) p0 += __shfl_down_sync(0xffffffffu, p0, o);
    }
    return p0;
}

// Q8 row: thread v owns octets v, v + 256, ... (at most 4: columns <= 8192).
// Q8Lane holds what depends only on the thread and the row shape.
struct Q8Lane {
    uint32_t count;        // octets this thread owns
    uint32_t sidx[4];      // scale index of each octet relative to the row's first scale
};

K3_DEVINL Q8Lane q8_lane(uint32_t columns, uint32_t block) {
    Q8Lane l;
    l.count = 0u;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t octet = threadIdx.x + 256u * i;
        l.sidx[i] = 0u;
        if (octet < columns / 8u) {
            l.count = i + 1u;
            l.sidx[i] = (octet * 8u) / block;
        }
    }
    return l;
}

struct Q8RowLoad {
    uint2 w[4];
    float s[4];
};

K3_DEVINL void q8_block_load(Q8RowLoad &p, const Q8Lane &l, const int8_t *__restrict__ qr,
                             const void *__restrict__ scales, uint64_t scale_base, int scale_f16) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        if ((uint32_t)i < l.count) {
            p.w[i] = ld_stream_8(qr + (uint64_t)(threadIdx.x + 256u * i) * 8u);
            p.s[i] = scale_f16 ? __half2float(reinterpret_cast<const __half *>(scales)[scale_base + l.sidx[i]])
                               : reinterpret_cast<const float *>(scales)[scale_base + l.sidx[i]];
        }
    }
}

// this lane's chain; xf is the vector as fp32 (shared memory, 16-byte aligned)
K3_DEVINL float q8_block_lane_sum(const Q8RowLoad &p, const Q8Lane &l, const float *xf) {
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        if ((uint32_t)i >= l.count) break;
        const float4 x0 = reinterpret_cast<const float4 *>(xf)[(threadIdx.x + 256u * i) * 2u];
        const float4 x1 = reinterpret_cast<const float4 *>(xf)[(threadIdx.x + 256u * i) * 2u + 1u];
        const float s = p.s[i];
        const uint32_t w0 = p.w[i].x, w1 = p.w[i].y;
        a = fmaf(__fmul_rn(int8_to_float(w0, 0), s), x0.x, a);
        a = fmaf(__fmul_rn(int8_to_float(w0, 1), s), x0.y, a);
        a = fmaf(__fmul_rn(int8_to_float(w0, 2), s), x0.z, a);
        a = fmaf(__fmul_rn(int8_to_float(w0, 3), s), x0.w, a);
        a = fmaf(__fmul_rn(int8_to_float(w1, 0), s), x1.x, a);
        a = fmaf(__fmul_rn(int8_to_float(w1, 1), s), x1.y, a);
        a = fmaf(__fmul_rn(int8_to_float(w1, 2), s), x1.z, a);
        a = fmaf(__fmul_rn(int8_to_float(w1, 3), s), x1.w, a);
    }
    return a;
}

// R consecutive Q8 rows against one vector, all their loads in flight at once
// (I = octets per thread per row, columns <= 2048 * I).  `red` holds R * 256
// floats.  Warp w returns the dot product of rows row0 + w, row0 + w + 8, ... in
// out[0], out[1], ... (valid in lane 0; R <= 16).  The caller synchronises the
// block before `red` is reused.
template <int R, int I>
K3_DEVINL void q8_block_rows(float (&out)[(R + 7) / 8], const int8_t *__restrict__ q,
                             const void *__restrict__ scales, uint32_t row0, uint32_t columns,
                             uint32_t blocks_per_row, const Q8Lane &l, int scale_f16, const float *xf,
                             float *red) {
    uint2 w[R][I];
    float s[R][I];
#pragma unroll
    for (int i = 0; i < I; i++) {
        if ((uint32_t)i < l.count) {
            const uint32_t octet = threadIdx.x + 256u * i;
#pragma unroll
            for (int r = 0; r < R; r++) {
                const uint64_t row = row0 + r;
                w[r][i] = ld_stream_8(q + row * columns + (uint64_t)octet * 8u);
                const uint64_t si = row * blocks_per_row + l.sidx[i];
                s[r][i] = scale_f16 ? __half2float(reinterpret_cast<const __half *>(scales)[si])
                                    : reinterpret_cast<const float *>(scales)[si];
            }
        }
    }
    float a[R];
#pragma unroll
    for (int r = 0; r < R; r++) a[r] = 0.f;
#pragma unroll
    for (int i = 0; i < I; i++) {
        if ((uint32_t)i >= l.count) break;
        const float4 x0 = reinterpret_cast<const float4 *>(xf)[(threadIdx.x + 256u * i) * 2u];
        const float4 x1 = reinterpret_cast<const float4 *>(xf)[(threadIdx.x + 256u * i) * 2u + 1u];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const float sc = s[r][i];
            const uint32_t w0 = w[r][i].x, w1 = w[r][i].y;
            float acc = a[r];
            acc = fmaf(__fmul_rn(int8_to_float(w0, 0), sc), x0.x, acc);
            acc = fmaf(__fmul_rn(int8_to_float(w0, 1), sc), x0.y, acc);
            acc = fmaf(__fmul_rn(int8_to_float(w0, 2), sc), x0.z, acc);
            acc = fmaf(__fmul_rn(int8_to_float(w0, 3), sc), x0.w, acc);
            acc = fmaf(__fmul_rn(int8_to_float(w1, 0), sc), x1.x, acc);
            acc = fmaf(__fmul_rn(int8_to_float(w1, 1), sc), x1.y, acc);
            acc = fmaf(__fmul_rn(int8_to_float(w1, 2), sc), x1.z, acc);
            acc = fmaf(__fmul_rn(int8_to_float(w1, 3), sc), x1.w, acc);
            a[r] = acc;
        }
    }
#pragma unroll
    for (int r = 0; r < R; r++) red[r * 256 + threadIdx.x] = a[r];
    __syncthreads();
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
#pragma unroll
    for (int j = 0; j < (R + 7) / 8; j++) {
        const uint32_t r = warp + 8u * j;
        float p0 = 0.f;
        if (r < (uint32_t)R) {
            const float *v = red + r * 256u;
            float a0 = v[lane] + v[lane + 128u], a1 = v[lane + 32u] + v[lane + 160u];
            float a2 = v[lane + 64u] + v[lane + 192u], a3 = v[lane + 96u] + v[lane + 224u];
            a0 += a2; a1 += a3;
            p0 = a0 + a1;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) p0 += __shfl_down_sync(0xffffffffu, p0, o);
        }
        out[j] = p0;
    }
}

// BF16 row: thread v owns columns v, v + 256, ... (at most 32: columns <= 8192)
struct Bf16RowLoad {
    uint16_t w[32];
};

K3_DEVINL void bf16_block_load(Bf16RowLoad &p, const uint16_t *__restrict__ wr, uint32_t columns) {
#pragma unroll
    for (int i = 0; i < 32; i++) {
        const uint32_t c = threadIdx.x + 256u * i;
        p.w[i] = c < columns ? __ldg(wr + c) : (uint16_t)0;
    }
}

K3_DEVINL float bf16_block_lane_sum(const Bf16RowLoad &p, const float *xf, uint32_t columns) {
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i++) {
        const uint32_t c = threadIdx.x + 256u * i;
        if (c >= columns) break;
        a = fmaf(bf16_bits_to_float(p.w[i]), xf[c], a);
    }
    return a;
}

}  // namespace k3
