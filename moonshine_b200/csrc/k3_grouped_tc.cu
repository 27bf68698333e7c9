// Ragged grouped GEMM on the 5th-generation tensor cores (tcgen05, sm_100a).
//
//   out[r, m] = sum_k W[g(r)][m, k] * x[r, k]      r: token rows grouped by expert
//
// computed "swapped": the weights are the 128-row M operand (A), the token
// rows are the N operand (B), the fp32 accumulators live in tensor memory.
// One work item = two 128-row weight tiles x up to 128 token rows of one
// group, over the whole K extent:
//   * gate/up mode: tile 0 = gate rows [m0, m0+128) of w1, tile 1 = the same
//     rows of w3; the epilogue rounds both to bf16, applies the activation and
//     writes act[r, m0 + m];
//   * plain mode (down projection, shared expert, router): tiles 0/1 are rows
//     [m0, m0+128) and [m0+128, m0+256) of one matrix.
//
// Warp roles (512 threads, one CTA per SM, persistent over a static item list):
//   warp 0        TMA producer: packed weight tiles + token tile per K step
//   warp 1        MMA issuer (one elected lane), owns the TMEM allocation
//   warps 4-7     epilogue: tcgen05.ld of the accumulators, activation, stores
//   warps 8-15    dequantisers: packed MXFP4 (or int8) in shared memory ->
//                 bf16 in the 128-byte-swizzled K-major layout the MMA reads
// The E2M1 x E8M0 -> bf16 conversion is exact (1 mantissa bit times a power of
// two), so the products equal the reference's; only the fp32 summation order
// differs.  MMA shape M=128, N = rows of the group rounded up to 16, K=16.
//
// Every mbarrier wait is bounded; on give-up the CTA raises a status word,
// drains and frees its tensor memory.
#include "k3_grouped.h"
#include "k3_moe_ops.h"
#include "k3_tc_ptx.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <mutex>

using namespace k3;
using namespace k3::tc;

namespace {

constexpr uint32_t BM = 128, BN = 128, BK = 64;
constexpr uint32_t kThreads = 512;
constexpr uint32_t kDequantWarps = 8;
constexpr uint32_t kAccBufs = 2;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kMaxGroups = 1024;

enum AMode : int { kAMxfp4 = 0, kAQ8 = 1, kABf16 = 2 };
enum EMode : int { kEAct = 0, kEBf16 = 1, kEF32 = 2 };

__device__ uint32_t g_tc_status = 0;   // 0 = ok; 1 = a bounded wait gave up

struct TcArgs {
    const uint8_t *scales0;     // MXFP4: E8M0 [rows_total, K/32]; Q8: scale table
    const uint8_t *scales1;
    const uint32_t *offsets;    // [groups+1] token-row ranges, or nullptr (one group of `rows`)
    void *out;
    uint32_t groups;
    uint32_t rows;              // total token rows
    uint32_t w_rows;            // weight rows per group per matrix
    uint32_t k;
    uint32_t out_width;         // row pitch of `out` in elements
    uint32_t m_items;           // items along the weight-row axis
    uint32_t q8_block;
    int q8_scale_f16;
    int activation;
    float beta, linear_beta;
};

template <int kA>
struct Cfg {
    static constexpr bool kDequant = kA != kABf16;
    static constexpr uint32_t kATile = BM * BK * 2;                        // 16384 (bf16, one K step)
    static constexpr uint32_t kBTile = BN * BK * 2;                        // 16384
    // Packed weights travel in 128-byte rows (the TMA engine spends about the same
    // time on a box row whatever its length), i.e. several K steps per packed stage:
    // 256 columns of MXFP4 or 128 of int8.
    static constexpr uint32_t kPackSteps = kA == kAMxfp4 ? 4 : (kA == kAQ8 ? 2 : 1);
    static constexpr uint32_t kPackedTile = kDequant ? BM * 128u : 0u;     // 16384
    static constexpr uint32_t kPStages = kDequant ? 2 : 0;                 // packed ring: [tile0 | tile1]
    // token ring stage: [B] (dequant) or [A0 | A1 | B] (bf16, everything by TMA)
    static constexpr uint32_t kStageBytes = kDequant ? kBTile : 2 * kATile + kBTile;
    static constexpr uint32_t kStages = 4;
    static constexpr uint32_t kAStages = kDequant ? 2 : 0;                 // dequantised ring: [A0 | A1]
    static constexpr uint32_t kRingBytes =
        kStages * kStageBytes + kPStages * 2 * kPackedTile + kAStages * 2 * kATile;
    static constexpr uint32_t kSmemBytes = kRingBytes + 1024 /*align*/ + 512 /*barriers*/ +
                                           (kMaxGroups + 1) * 4;
};

struct Item {
    uint32_t group, row_start, rows_valid, m_item;
};

// n-tile prefix in shared memory -> (group, first row, valid rows, m item)
K3_DEVINL Item decode_item(uint32_t w, const uint32_t *prefix, const TcArgs &a) {
    Item it;
    const uint32_t nt = w / a.m_items;
    it.m_item = w % a.m_items;
    if (a.offsets == nullptr) {
        it.group = 0;
        it.row_start = nt * BN;
        it.rows_valid = min(BN, a.rows - it.row_start);
        return it;
    }
    uint32_t lo = 0, hi = a.groups;          // largest g with prefix[g] <= nt
    while (hi - lo > 1u) {
        const uint32_t mid = (lo + hi) >> 1;
        if (prefix[mid] <= nt) lo = mid; else hi = mid;
    }
    it.group = lo;
    const uint32_t begin = a.offsets[lo], end = a.offsets[lo + 1u];
    it.row_start = begin + (nt - prefix[lo]) * BN;
    it.rows_valid = min(BN, end - it.row_start);
    return it;
}

// ---- dequantisers: 32 consecutive K elements of one weight row -> 4 x 16 bytes of bf16
// E2M1 magnitudes as bf16: 0, .5, 1, 1.5, 2, 3, 4, 6 -> byte-planar lookup tables for PRMT
constexpr uint32_t kLutLo0 = 0xC0800000u, kLutLo1 = 0xC0804000u;   // low bytes
constexpr uint32_t kLutHi0 = 0x3F3F3F00u, kLutHi1 = 0x40404040u;   // high bytes

K3_DEVINL void dequant_word_mxfp4(uint32_t w, uint32_t scale2, uint32_t (&out)[4]) {
    const uint32_t sel = w & 0x77777777u;
    const uint32_t lo03 = __byte_perm(kLutLo0, kLutLo1, sel);
    uint32_t hi03 = __byte_perm(kLutHi0, kLutHi1, sel);
    const uint32_t lo47 = __byte_perm(kLutLo0, kLutLo1, sel >> 16);
    uint32_t hi47 = __byte_perm(kLutHi0, kLutHi1, sel >> 16);
    const uint32_t u = w & 0x88888888u;
    const uint32_t u4 = u << 4;
    hi03 |= __byte_perm(u4, u, 0x5140u) & 0x80808080u;
    hi47 |= __byte_perm(u4, u, 0x7362u) & 0x80808080u;
    const uint32_t p[4] = {__byte_perm(lo03, hi03, 0x5140u), __byte_perm(lo03, hi03, 0x7362u),
                           __byte_perm(lo47, hi47, 0x5140u), __byte_perm(lo47, hi47, 0x7362u)};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(out[i]) : "r"(p[i]), "r"(scale2));
    }
}

// E8M0 byte -> bf16x2 of 2^(b-127); b == 0 -> 2^-127 (bf16 subnormal 0x0040)
K3_DEVINL uint32_t e8m0_to_bf16x2(uint32_t b) {
    const uint32_t h = b == 0u ? 0x0040u : (b << 7);
    return h | (h << 16);
}

K3_DEVINL uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

template <int kA, int kE>
__global__ void __launch_bounds__(kThreads, 1)
grouped_tc_kernel(const __grid_constant__ CUtensorMap map_a0,
                  const __grid_constant__ CUtensorMap map_a1,
                  const __grid_constant__ CUtensorMap map_b, TcArgs a) {
    using C = Cfg<kA>;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    unsigned char *base = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    unsigned char *ring = base;                                     // token (or all-TMA) ring
    unsigned char *pring = base + C::kStages * C::kStageBytes;      // packed weight ring
    unsigned char *aring = pring + C::kPStages * 2u * C::kPackedTile;   // dequantised A ring
    uint64_t *bars = reinterpret_cast<uint64_t *>(base + C::kRingBytes);
    uint64_t *full = bars;                         // [kStages]
    uint64_t *empty = full + C::kStages;           // [kStages]
    uint64_t *a_full = empty + C::kStages;         // [kAStages]
    uint64_t *a_empty = a_full + 4;                // [kAStages]
    uint64_t *p_full = a_empty + 4;                // [kPStages]
    uint64_t *p_empty = p_full + 2;                // [kPStages]
    uint64_t *acc_full = p_empty + 2;              // [2]
    uint64_t *acc_empty = acc_full + 2;            // [2]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    uint32_t *total_items_s = tmem_slot + 2;
    uint32_t *prefix = reinterpret_cast<uint32_t *>(base + C::kRingBytes + 512);

    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t ksteps = a.k / BK;

    // ---- prologue: n-tile prefix of the groups, barriers, tensor memory
    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (uint32_t s = 0; s < C::kStages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (uint32_t s = 0; s < C::kPStages; s++) {
            mbar_init(&p_full[s], 1);
            mbar_init(&p_empty[s], kDequantWarps);
        }
        for (uint32_t s = 0; s < C::kAStages; s++) {
            mbar_init(&a_full[s], kDequantWarps);
            mbar_init(&a_empty[s], 1);
        }
        for (uint32_t b = 0; b < kAccBufs; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
        }
        fence_barrier_init();
    }
    if (a.offsets != nullptr) {
        // exclusive prefix of ceil(rows_g / BN); groups <= 1024, two elements per thread
        __shared__ uint32_t warp_tot[kThreads / kWarp];
        uint32_t v[2], incl[2];
        uint32_t run = 0;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const uint32_t g = threadIdx.x * 2u + j;
            v[j] = g < a.groups ? (a.offsets[g + 1u] - a.offsets[g] + BN - 1u) / BN : 0u;
            run += v[j];
            incl[j] = run;
        }
        uint32_t scan = run;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t n = __shfl_up_sync(0xffffffffu, scan, o);
            if (lane >= (uint32_t)o) scan += n;
        }
        if (lane == 31) warp_tot[warp] = scan;
        __syncthreads();
        uint32_t warp_base = 0;
        for (uint32_t wv = 0; wv < warp; wv++) warp_base += warp_tot[wv];
        const uint32_t excl_thread = warp_base + scan - run;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const uint32_t g = threadIdx.x * 2u + j;
            if (g < a.groups) prefix[g] = excl_thread + incl[j] - v[j];
            if (g + 1u == a.groups) {
                prefix[a.groups] = excl_thread + incl[j];
                *total_items_s = (excl_thread + incl[j]) * a.m_items;
            }
        }
    } else if (threadIdx.x == 0) {
        *total_items_s = ((a.rows + BN - 1u) / BN) * a.m_items;
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t total_items = *total_items_s;

    if (warp == 0) {
        // ===================================================== TMA producer
        if (lane == 0) {
            prefetch_tensormap(&map_a0);
            prefetch_tensormap(&map_a1);
            prefetch_tensormap(&map_b);
            uint32_t s = 0, ph = 0, ps = 0, pph = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; ok && w < total_items; w += gridDim.x) {
                const Item it = decode_item(w, prefix, a);
                const int32_t y0 = (int32_t)(it.group * a.w_rows + it.m_item * (kE == kEAct ? BM : 2u * BM));
                const int32_t y1 = kE == kEAct ? y0 : y0 + (int32_t)BM;
                for (uint32_t ks = 0; ks < ksteps; ks++) {
                    if (C::kDequant && (ks % C::kPackSteps) == 0u) {
                        if (!mbar_wait(&p_empty[ps], pph ^ 1u, abort_flag)) { ok = false; break; }
                        unsigned char *pt = pring + ps * 2u * C::kPackedTile;
                        mbar_arrive_expect_tx(&p_full[ps], 2u * C::kPackedTile);
                        const int32_t xb = (int32_t)((ks / C::kPackSteps) * 128u);      // bytes
                        tma_load_2d(pt, &map_a0, &p_full[ps], xb, y0);
                        tma_load_2d(pt + C::kPackedTile, &map_a1, &p_full[ps], xb, y1);
                        if (++ps == C::kPStages) { ps = 0; pph ^= 1u; }
                    }
                    if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                    unsigned char *st = ring + s * C::kStageBytes;
                    mbar_arrive_expect_tx(&full[s], C::kStageBytes);
                    if (C::kDequant) {
                        tma_load_2d(st, &map_b, &full[s], (int32_t)(ks * BK), (int32_t)it.row_start);
                    } else {
                        tma_load_2d(st, &map_a0, &full[s], (int32_t)(ks * BK), y0);
                        tma_load_2d(st + C::kATile, &map_a1, &full[s], (int32_t)(ks * BK), y1);
                        tma_load_2d(st + 2 * C::kATile, &map_b, &full[s], (int32_t)(ks * BK),
                                    (int32_t)it.row_start);
                    }
                    if (++s == C::kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ======================================================= MMA issuer
        if (lane == 0) {
            uint32_t s = 0, ph = 0, sa = 0, pha = 0, buf = 0, pacc = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; ok && w < total_items; w += gridDim.x) {
                const Item it = decode_item(w, prefix, a);
                const uint32_t n_eff = max(16u, (it.rows_valid + 15u) & ~15u);
                const uint32_t idesc = make_idesc_bf16(BM, n_eff);
                if (!mbar_wait(&acc_empty[buf], pacc ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d0 = tmem_base + buf * (2u * BN);
                const uint32_t d1 = d0 + BN;
                for (uint32_t ks = 0; ks < ksteps; ks++) {
                    if (!mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
                    unsigned char *st = ring + s * C::kStageBytes;
                    uint32_t a0_addr, a1_addr, b_addr;
                    if (C::kDequant) {
                        if (!mbar_wait(&a_full[sa], pha, abort_flag)) { ok = false; break; }
                        a0_addr = smem_u32(aring + sa * 2u * C::kATile);
                        a1_addr = a0_addr + C::kATile;
                        b_addr = smem_u32(st);
                    } else {
                        a0_addr = smem_u32(st);
                        a1_addr = a0_addr + C::kATile;
                        b_addr = smem_u32(st + 2 * C::kATile);
                    }
                    tc_fence_after();
                    const uint64_t da0 = make_desc_sw128(a0_addr), da1 = make_desc_sw128(a1_addr);
                    const uint64_t db = make_desc_sw128(b_addr);
#pragma unroll
                    for (uint32_t j = 0; j < BK / 16u; j++) {
                        const uint32_t acc = (ks | j) != 0u ? 1u : 0u;
                        // advance 16 K elements = 32 bytes inside the swizzle atom
                        mma_f16_ss(d0, da0 + 2u * j, db + 2u * j, idesc, acc);
                        mma_f16_ss(d1, da1 + 2u * j, db + 2u * j, idesc, acc);
                    }
                    if (C::kDequant) {
                        mma_commit(&a_empty[sa]);
                        if (++sa == C::kAStages) { sa = 0; pha ^= 1u; }
                    }
                    mma_commit(&empty[s]);
                    if (++s == C::kStages) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                mma_commit(&acc_full[buf]);
                if (++buf == kAccBufs) { buf = 0; pacc ^= 1u; }
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ========================================================= epilogue
        const uint32_t q = warp - 4u;                 // TMEM lane quarter
        const uint32_t m = 32u * q + lane;            // weight row inside the tile
        uint32_t buf = 0, pacc = 0;
        bool ok = true;
        for (uint32_t w = blockIdx.x; ok && w < total_items; w += gridDim.x) {
            const Item it = decode_item(w, prefix, a);
            const uint32_t n_eff = max(16u, (it.rows_valid + 15u) & ~15u);
            if (!mbar_wait(&acc_full[buf], pacc, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t t0 = tmem_base + ((32u * q) << 16) + buf * (2u * BN);
            const uint32_t col0 = it.m_item * (kE == kEAct ? BM : 2u * BM) + m;   // column of tile 0
            const uint32_t col1 = kE == kEAct ? col0 : col0 + BM;
            for (uint32_t c = 0; c < n_eff; c += 32u) {
                uint32_t r0[32], r1[32];
                tmem_ld_32x32(t0 + c, r0);
                tmem_ld_32x32(t0 + BN + c, r1);
                tmem_ld_wait();
#pragma unroll
                for (uint32_t j = 0; j < 32u; j++) {
                    const uint32_t n = c + j;
                    if (n >= it.rows_valid) continue;
                    const uint64_t row = (uint64_t)(it.row_start + n) * a.out_width;
                    const float v0 = __uint_as_float(r0[j]), v1 = __uint_as_float(r1[j]);
                    if (kE == kEAct) {
                        if (col0 < a.w_rows) {
                            const float g = bf16_bits_to_float(float_to_bf16_bits(v0));
                            const float u = bf16_bits_to_float(float_to_bf16_bits(v1));
                            reinterpret_cast<uint16_t *>(a.out)[row + col0] = float_to_bf16_bits(
                                activation(g, u, a.activation, a.beta, a.linear_beta));
                        }
                    } else if (kE == kEBf16) {
                        if (col0 < a.w_rows) reinterpret_cast<uint16_t *>(a.out)[row + col0] = float_to_bf16_bits(v0);
                        if (col1 < a.w_rows) reinterpret_cast<uint16_t *>(a.out)[row + col1] = float_to_bf16_bits(v1);
                    } else {
                        if (col0 < a.w_rows) reinterpret_cast<float *>(a.out)[row + col0] = v0;
                        if (col1 < a.w_rows) reinterpret_cast<float *>(a.out)[row + col1] = v1;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            if (++buf == kAccBufs) { buf = 0; pacc ^= 1u; }
        }
    } else if (C::kDequant && warp >= 8) {
        // ====================================================== dequantisers
        const uint32_t t = threadIdx.x - 8u * kWarp;     // 0..255
        const uint32_t row = t & 127u, half = t >> 7;    // weight row in tile, 32-column half
        uint32_t ps = 0, pph = 0, sa = 0, pha = 0;
        bool ok = true;
        const uint64_t total_w_rows = (uint64_t)a.groups * a.w_rows;
        for (uint32_t w = blockIdx.x; ok && w < total_items; w += gridDim.x) {
            const Item it = decode_item(w, prefix, a);
            const uint64_t y0 = (uint64_t)it.group * a.w_rows + it.m_item * (kE == kEAct ? BM : 2u * BM) + row;
            const uint64_t y1 = kE == kEAct ? y0 : y0 + BM;
            const uint64_t yc0 = min(y0, total_w_rows - 1u), yc1 = min(y1, total_w_rows - 1u);
            uint4 sc0 = make_uint4(0, 0, 0, 0), sc1 = make_uint4(0, 0, 0, 0);
            const uint8_t *srow0 = nullptr, *srow1 = nullptr;
            if (kA == kAMxfp4) {
                srow0 = a.scales0 + yc0 * (a.k / 32u);
                srow1 = a.scales1 + yc1 * (a.k / 32u);
            }
            for (uint32_t ks = 0; ks < ksteps; ks++) {
                if (kA == kAMxfp4 && (ks & 7u) == 0u) {
                    sc0 = *reinterpret_cast<const uint4 *>(srow0 + (ks >> 3) * 16u);
                    sc1 = *reinterpret_cast<const uint4 *>(srow1 + (ks >> 3) * 16u);
                }
                const uint32_t sub = ks % C::kPackSteps;
                if (sub == 0u && !mbar_wait(&p_full[ps], pph, abort_flag)) { ok = false; break; }
                // packed tiles are 128-byte rows written with the 128-byte swizzle: 16-byte
                // chunk c of row r sits at chunk position c ^ (r % 8)
                const unsigned char *pt0 = pring + ps * 2u * C::kPackedTile + row * 128u;
                const unsigned char *pt1 = pt0 + C::kPackedTile;
                uint32_t o0[16], o1[16];          // 32 bf16 per tile
                if (kA == kAMxfp4) {
                    const uint32_t chunk = ((sub * 2u + half) ^ (row & 7u)) * 16u;
                    const uint4 p0 = *reinterpret_cast<const uint4 *>(pt0 + chunk);
                    const uint4 p1 = *reinterpret_cast<const uint4 *>(pt1 + chunk);
                    const uint32_t bi = (ks & 7u) * 2u + half;        // byte inside the 16-byte scale chunk
                    const uint32_t wi = bi >> 2;
                    const uint32_t ws0 = wi == 0u ? sc0.x : (wi == 1u ? sc0.y : (wi == 2u ? sc0.z : sc0.w));
                    const uint32_t ws1 = wi == 0u ? sc1.x : (wi == 1u ? sc1.y : (wi == 2u ? sc1.z : sc1.w));
                    const uint32_t s0 = e8m0_to_bf16x2((ws0 >> ((bi & 3u) * 8u)) & 0xffu);
                    const uint32_t s1 = e8m0_to_bf16x2((ws1 >> ((bi & 3u) * 8u)) & 0xffu);
                    const uint32_t pw0[4] = {p0.x, p0.y, p0.z, p0.w};
                    const uint32_t pw1[4] = {p1.x, p1.y, p1.z, p1.w};
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        uint32_t t4[4];
                        dequant_word_mxfp4(pw0[i], s0, t4);
                        o0[4 * i] = t4[0]; o0[4 * i + 1] = t4[1]; o0[4 * i + 2] = t4[2]; o0[4 * i + 3] = t4[3];
                        dequant_word_mxfp4(pw1[i], s1, t4);
                        o1[4 * i] = t4[0]; o1[4 * i + 1] = t4[1]; o1[4 * i + 2] = t4[2]; o1[4 * i + 3] = t4[3];
                    }
                } else {
                    const uint32_t col = ks * BK + half * 32u;
                    const uint32_t sidx = col / a.q8_block;
                    const uint64_t pitch = a.k / a.q8_block;
                    float f0, f1;
                    if (a.q8_scale_f16) {
                        f0 = __half2float(reinterpret_cast<const __half *>(a.scales0)[yc0 * pitch + sidx]);
                        f1 = __half2float(reinterpret_cast<const __half *>(a.scales1)[yc1 * pitch + sidx]);
                    } else {
                        f0 = reinterpret_cast<const float *>(a.scales0)[yc0 * pitch + sidx];
                        f1 = reinterpret_cast<const float *>(a.scales1)[yc1 * pitch + sidx];
                    }
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const uint32_t chunk = ((sub * 4u + half * 2u + (uint32_t)h) ^ (row & 7u)) * 16u;
                        const uint4 a4 = *reinterpret_cast<const uint4 *>(pt0 + chunk);
                        const uint4 b4 = *reinterpret_cast<const uint4 *>(pt1 + chunk);
                        const uint32_t aw[4] = {a4.x, a4.y, a4.z, a4.w};
                        const uint32_t bw[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
                        for (int i = 0; i < 4; i++) {
#pragma unroll
                            for (int p = 0; p < 2; p++) {
                                const float al = __fmul_rn((float)(int8_t)(aw[i] >> (16 * p)), f0);
                                const float ah = __fmul_rn((float)(int8_t)(aw[i] >> (16 * p + 8)), f0);
                                const float bl = __fmul_rn((float)(int8_t)(bw[i] >> (16 * p)), f1);
                                const float bh = __fmul_rn((float)(int8_t)(bw[i] >> (16 * p + 8)), f1);
                                o0[h * 8 + i * 2 + p] = pack_bf16x2(al, ah);
                                o1[h * 8 + i * 2 + p] = pack_bf16x2(bl, bh);
                            }
                        }
                    }
                }
                if (!mbar_wait(&a_empty[sa], pha ^ 1u, abort_flag)) { ok = false; break; }
                // row `row` of the tile: 128 bytes at atom (row/8), line (row%8); 16-byte
                // chunk c is stored at chunk position c ^ (row % 8)
                unsigned char *dst0 = aring + sa * 2u * C::kATile + (row >> 3) * 1024u + (row & 7u) * 128u;
                unsigned char *dst1 = dst0 + C::kATile;
#pragma unroll
                for (uint32_t c4 = 0; c4 < 4u; c4++) {
                    const uint32_t chunk = (half * 4u + c4) ^ (row & 7u);
                    *reinterpret_cast<uint4 *>(dst0 + chunk * 16u) =
                        make_uint4(o0[4 * c4], o0[4 * c4 + 1], o0[4 * c4 + 2], o0[4 * c4 + 3]);
                    *reinterpret_cast<uint4 *>(dst1 + chunk * 16u) =
                        make_uint4(o1[4 * c4], o1[4 * c4 + 1], o1[4 * c4 + 2], o1[4 * c4 + 3]);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[sa]);
                if (++sa == C::kAStages) { sa = 0; pha ^= 1u; }
                if (sub == C::kPackSteps - 1u) {
                    // The packed stage goes back to the TMA producer only here: the stores
                    // above consumed every value loaded from it, so those loads have
                    // completed (an arrive right after issuing them would not wait).
                    if (lane == 0) mbar_arrive(&p_empty[ps]);
                    if (++ps == C::kPStages) { ps = 0; pph ^= 1u; }
                }
            }
        }
    }

    // ---- teardown
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0u) atomicExch(&g_tc_status, 1u);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------ host side
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
        } else {
            (void)cudaGetLastError();
        }
    });
    return fn;
}

// 2-D row-major tensor [rows, cols] of `elem` bytes; box {box_cols, box_rows}
bool make_map(CUtensorMap *map, const void *ptr, CUtensorMapDataType type, uint32_t elem,
              uint64_t rows, uint64_t cols, uint32_t box_cols, uint32_t box_rows,
              CUtensorMapSwizzle swizzle) {
    auto fn = encode_fn();
    if (!fn || (((uintptr_t)ptr) & 15u) != 0 || (cols * elem) % 16u != 0) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * elem};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, type, 2, const_cast<void *>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int kA, int kE>
bool launch_tc(const void *a0, const void *a1, const TcArgs &args, const void *b_rows,
               cudaStream_t stream) {
    using C = Cfg<kA>;
    CUtensorMap ma0, ma1, mb;
    const uint64_t w_total = (uint64_t)args.groups * args.w_rows;
    bool ok;
    if (kA == kAMxfp4) {
        ok = make_map(&ma0, a0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_total, args.k / 2u, 128u, BM,
                      CU_TENSOR_MAP_SWIZZLE_128B) &&
             make_map(&ma1, a1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_total, args.k / 2u, 128u, BM,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    } else if (kA == kAQ8) {
        ok = make_map(&ma0, a0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_total, args.k, 128u, BM,
                      CU_TENSOR_MAP_SWIZZLE_128B) &&
             make_map(&ma1, a1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_total, args.k, 128u, BM,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    } else {
        ok = make_map(&ma0, a0, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_total, args.k, BK, BM,
                      CU_TENSOR_MAP_SWIZZLE_128B) &&
             make_map(&ma1, a1, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_total, args.k, BK, BM,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    }
    ok = ok && make_map(&mb, b_rows, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, args.rows, args.k, BK, BN,
                        CU_TENSOR_MAP_SWIZZLE_128B);
    if (!ok) return false;
    auto kernel = grouped_tc_kernel<kA, kE>;
    if (!set_max_dynamic_smem((const void *)kernel, C::kSmemBytes)) return false;
    kernel<<<sm_count(), kThreads, C::kSmemBytes, stream>>>(ma0, ma1, mb, args);
    return launch_ok();
}

// Q8 weights -> bf16 (each product q * scale rounded once, as the in-kernel
// conversion of the Q8 mode does); 16 elements per thread, block % 16 == 0.
__global__ void __launch_bounds__(256)
q8_to_bf16_kernel(uint4 *__restrict__ w, const uint4 *__restrict__ q, const void *__restrict__ scales,
                  uint64_t units, uint32_t block, int scale_f16) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < units; i += stride) {
        const uint64_t b = i * 16u / block;
        const float s = scale_f16 ? __half2float(reinterpret_cast<const __half *>(scales)[b])
                                  : reinterpret_cast<const float *>(scales)[b];
        const uint4 v = q[i];
        const uint32_t in[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 4; j++) {
#pragma unroll
            for (int p = 0; p < 2; p++) {
                const float lo = __fmul_rn((float)(int8_t)(in[j] >> (16 * p)), s);
                const float hi = __fmul_rn((float)(int8_t)(in[j] >> (16 * p + 8)), s);
                o[2 * j + p] = pack_bf16x2(lo, hi);
            }
        }
        w[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
        w[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

bool tc_shape_ok(uint32_t k, uint32_t rows) {
    return k % 512u == 0 && k >= 512u && rows >= 1u;
}

}  // namespace

extern "C" uint32_t k3_moe_device_status(void) {
    uint32_t v = 0xffffffffu;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(v)) != cudaSuccess) (void)cudaGetLastError();
    return v | k3_decode_mx_status() | k3_decode_status() | k3_decode_shared_status() | k3_grouped_mx_status() |
           k3_dispatch_status();
}

bool k3_status_words_clear() {
    const uint32_t zero = 0u;
    bool ok = cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(zero)) == cudaSuccess;
    if (!ok) (void)cudaGetLastError();
    ok = k3_decode_status_clear() && ok;
    ok = k3_decode_mx_status_clear() && ok;
    ok = k3_decode_shared_status_clear() && ok;
    ok = k3_dispatch_status_clear() && ok;
    ok = k3_grouped_mx_status_clear() && ok;
    return ok;
}

extern "C" bool k3_moe_device_status_clear(void) {
    return k3_status_words_clear();
}

namespace {

// One warp waits on an mbarrier that nobody arrives on, with a limit given by the
// caller; when the wait gives up it takes the same way out as the product kernels
// (abort flag in shared memory -> status word), touches no tensor memory and returns.
__global__ void bounded_wait_selftest_kernel(unsigned long long limit_ns, uint32_t *gave_up) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_word;
    volatile uint32_t *abort_flag = &abort_word;
    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        mbar_init(&bar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool ok = mbar_wait(&bar, 0u, abort_flag, limit_ns);
        if (gave_up) *gave_up = ok ? 0u : 1u;
    }
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0u) atomicExch(&g_tc_status, 1u);
}

}  // namespace

extern "C" bool k3_moe_selftest_bounded_wait(uint32_t limit_us, void *gave_up, void *stream) {
    if (limit_us == 0u || limit_us > 1000000u) return false;          // at most one second
    bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((unsigned long long)limit_us * 1000ull,
                                                                     (uint32_t *)gave_up);
    return launch_ok();
}

bool k3_grouped_dense_bf16_f32(void *out, const void *weights, const void *x, uint32_t tokens,
                               uint32_t rows, uint32_t cols, void *stream) {
    const bool aligned = ((((uintptr_t)weights) | ((uintptr_t)x)) & 15u) == 0;
    if (tokens >= 32u && tc_shape_ok(cols, tokens) && aligned && encode_fn()) {
        TcArgs a{};
        a.out = out;
        a.groups = 1;
        a.rows = tokens;
        a.w_rows = rows;
        a.k = cols;
        a.out_width = rows;
        a.m_items = (rows + 2u * BM - 1u) / (2u * BM);
        return launch_tc<kABf16, kEF32>(weights, weights, a, x, (cudaStream_t)stream);
    }
    return k3_rocm_bf16_gemm_f32(out, weights, x, tokens, rows, cols, stream);
}

bool k3_grouped_q8_bf16(void *out, const void *q, const void *scales, const void *x,
                        uint32_t tokens, uint32_t rows, uint32_t cols, uint32_t block,
                        int scale_type, void *stream) {
    const bool aligned = ((((uintptr_t)q) | ((uintptr_t)x)) & 15u) == 0;
    if (tokens >= 32u && tc_shape_ok(cols, tokens) && aligned && encode_fn() && block % 32u == 0) {
        TcArgs a{};
        a.scales0 = a.scales1 = (const uint8_t *)scales;
        a.out = out;
        a.groups = 1;
        a.rows = tokens;
        a.w_rows = rows;
        a.k = cols;
        a.out_width = rows;
        a.m_items = (rows + 2u * BM - 1u) / (2u * BM);
        a.q8_block = block;
        a.q8_scale_f16 = scale_type;
        return launch_tc<kAQ8, kEBf16>(q, q, a, x, (cudaStream_t)stream);
    }
    return k3_moe_q8_gemm_bf16(out, q, scales, x, tokens, rows, cols, block, scale_type, stream);
}

// out bf16 [tokens, rows] = x [tokens, cols] * dequant(q, scales)^T with the table
// converted to bf16 once into weight_scratch (rows * cols * 2 bytes), then a plain
// bf16 tensor-core GEMM.  False when the shape does not suit the path.
bool k3_grouped_q8_dense_bf16(void *out, const void *q, const void *scales, const void *x, uint32_t tokens,
                              uint32_t rows, uint32_t cols, uint32_t block, int scale_type,
                              void *weight_scratch, cudaStream_t stream) {
    if (tokens < 32u || !tc_shape_ok(cols, tokens) || block % 16u != 0 || !encode_fn() || !weight_scratch ||
        ((((uintptr_t)q) | ((uintptr_t)x) | ((uintptr_t)weight_scratch)) & 15u) != 0) {
        return false;
    }
    const uint64_t units = (uint64_t)rows * cols / 16u;
    const uint32_t blocks = (uint32_t)std::min<uint64_t>((units + 255u) / 256u, (uint64_t)sm_count() * 16u);
    q8_to_bf16_kernel<<<blocks, 256, 0, stream>>>((uint4 *)weight_scratch, (const uint4 *)q, scales, units, block,
                                                  scale_type);
    if (!launch_ok()) return false;
    TcArgs a{};
    a.out = out;
    a.groups = 1;
    a.rows = tokens;
    a.w_rows = rows;
    a.k = cols;
    a.out_width = rows;
    a.m_items = (rows + 2u * BM - 1u) / (2u * BM);
    return launch_tc<kABf16, kEBf16>(weight_scratch, weight_scratch, a, x, stream);
}

size_t k3_grouped_shared_workspace_bytes(const k3_moe_layer_desc *d, uint32_t tokens) {
    if (d->shared_hidden == 0 || tokens < 32u || !tc_shape_ok(d->hidden, tokens) ||
        !tc_shape_ok(d->shared_hidden, tokens) || d->q8_block % 16u != 0 || !encode_fn()) {
        return 0;
    }
    return (size_t)3u * d->shared_hidden * d->hidden * 2u + 256u;
}

// Shared expert for many tokens: the three Q8 tables are converted to bf16 once
// per call (tens of microseconds at memory speed) and the products run as plain
// bf16 tensor-core GEMMs with the activation fused into the gate/up epilogue.
bool k3_grouped_shared_expert(const k3_moe_layer_desc *d, void *out, void *act, const void *x,
                              uint32_t tokens, void *workspace, cudaStream_t stream) {
    const uint32_t S = d->shared_hidden, H = d->hidden;
    const uint64_t units = (uint64_t)S * H / 16u;
    uint16_t *wg = (uint16_t *)(((uintptr_t)workspace + 255u) & ~(uintptr_t)255u);
    uint16_t *wu = wg + (size_t)S * H, *wd = wu + (size_t)S * H;
    const void *q[3] = {d->shared_gate_q, d->shared_up_q, d->shared_down_q};
    const void *sc[3] = {d->shared_gate_s, d->shared_up_s, d->shared_down_s};
    uint16_t *dst[3] = {wg, wu, wd};
    const uint32_t blocks = (uint32_t)std::min<uint64_t>((units + 255u) / 256u, (uint64_t)sm_count() * 16u);
    for (int t = 0; t < 3; t++) {
        if ((((uintptr_t)q[t]) & 15u) != 0) return false;
        q8_to_bf16_kernel<<<blocks, 256, 0, stream>>>((uint4 *)dst[t], (const uint4 *)q[t], sc[t], units,
                                                      d->q8_block, d->q8_scale_type);
    }
    if (!launch_ok()) return false;
    TcArgs a{};
    a.groups = 1;
    a.rows = tokens;
    a.activation = d->activation;
    a.beta = d->beta;
    a.linear_beta = d->linear_beta;
    a.out = act;
    a.w_rows = S;
    a.k = H;
    a.out_width = S;
    a.m_items = (S + BM - 1u) / BM;
    if (!launch_tc<kABf16, kEAct>(wg, wu, a, x, stream)) return false;
    a.out = out;
    a.w_rows = H;
    a.k = S;
    a.out_width = H;
    a.m_items = (H + 2u * BM - 1u) / (2u * BM);
    return launch_tc<kABf16, kEBf16>(wd, wd, a, act, stream);
}

bool k3_grouped_tc_supported(const k3_moe_layer_desc *d, uint32_t rows) {
    return rows >= 32u && tc_shape_ok(d->hidden, rows) && tc_shape_ok(d->expert_hidden, rows) &&
           encode_fn() != nullptr;
}

bool k3_grouped_tc_experts(const k3_moe_layer_desc *d, void *rows_out, void *act,
                           const void *rows_in, const void *offsets, uint32_t rows,
                           void *stream_pointer) {
    cudaStream_t stream = (cudaStream_t)stream_pointer;
    TcArgs a{};
    a.offsets = (const uint32_t *)offsets;
    a.groups = d->local_expert_count;
    a.rows = rows;
    a.activation = d->activation;
    a.beta = d->beta;
    a.linear_beta = d->linear_beta;
    // gate/up + activation: act[r, :] bf16 [rows, I]
    a.scales0 = (const uint8_t *)d->w1_scales;
    a.scales1 = (const uint8_t *)d->w3_scales;
    a.out = act;
    a.w_rows = d->expert_hidden;
    a.k = d->hidden;
    a.out_width = d->expert_hidden;
    a.m_items = (d->expert_hidden + BM - 1u) / BM;
    if (!launch_tc<kAMxfp4, kEAct>(d->w1_packed, d->w3_packed, a, rows_in, stream)) return false;
    // down: rows_out[r, :] bf16 [rows, d]
    a.scales0 = a.scales1 = (const uint8_t *)d->w2_scales;
    a.out = rows_out;
    a.w_rows = d->hidden;
    a.k = d->expert_hidden;
    a.out_width = d->hidden;
    a.m_items = (d->hidden + 2u * BM - 1u) / (2u * BM);
    return launch_tc<kAMxfp4, kEBf16>(d->w2_packed, d->w2_packed, a, act, stream);
}
