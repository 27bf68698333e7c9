// One-token expert products on the packed block-scaled tensor-core path
// (tcgen05.mma kind::mxf4, 32-element blocks with E8M0 scales).
//
// The MXFP4 weights are consumed as they are stored: packed E2M1 nibbles arrive by
// TMA as plain bytes (128 rows x 128 bytes = 256 K elements per box, the layout the
// MMA reads) and the E8M0 scales are written into tensor memory with tcgen05.st, so
// no thread touches a weight and shared memory holds exactly the bytes HBM delivered.
// The activation vector is split once into kTerms E2M1 terms with a block scale per
// term (k3_e2m1_terms.cuh), exact for bf16 inputs; the terms are rows 0..7 of the
// N = 16 operand, so accumulator columns 0..7 hold the partial dot products and
// their sum is the result.
//
// One CTA per SM, persistent over (expert rank, 128-row tile) items:
//   warp 0      TMA producer (A: 128 rows x 256 K, B: 8 term rows x 256 K per stage)
//   warp 1      MMA issuer: 4 MMAs of K=64 per stage, even stages
//   warps 2-5   scale writers: per batch the tile's 128x16 E8M0 bytes (512 K, two
//               stages) -> 16 TMEM columns (lane = row % 32, column = row / 32,
//               copied into every lane quadrant) plus the terms' block scales
//   warps 6-9   epilogue: tcgen05.ld of the term columns, sum, bf16, activation;
//               the gate/up epilogue also splits the activation it produces into
//               the E2M1 terms the down projection reads
//   warp 10     scale producer: block scales of two stages into a shared-memory ring
//   warp 11     second MMA issuer (odd stages, its own accumulator columns)
// Every barrier wait is bounded (see k3_tc_ptx.cuh).
#include "k3_decode_tail.cuh"
#include "k3_e2m1_terms.cuh"
#include "k3_grouped.h"
#include "k3_rowdot.cuh"
#include "k3_tc_ptx.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <atomic>
#include <cstring>
#include <map>
#include <mutex>

using namespace k3;
using namespace k3::tc;

namespace {

constexpr uint32_t kStages = 12;            // TMA ring of weight / term tiles
constexpr uint32_t kKStage = 256;           // K elements per stage (128 packed bytes per row)
constexpr uint32_t kSfBatches = 6;          // scale ring in tensor memory: batches of 2 stages (512 K)
constexpr uint32_t kSfSlots = 4;            // scale ring in shared memory (one batch per slot)
constexpr uint32_t kSfaBytes = 128 * 16;    // 128 rows x 16 scale bytes (512 K)
constexpr uint32_t kSfSlotBytes = kSfaBytes + 128;   // + the 8 term rows' 16 scale bytes each
constexpr uint32_t kATile = 128 * 128;     // bytes in shared memory = bytes the TMA brings
constexpr uint32_t kBTile = 16 * 128;      // N = 16 rows; the TMA fills rows 0..7, rows 8..15 stay zero
constexpr uint32_t kBTx = kTerms * 128;
constexpr uint32_t kStageBytes = kATile + kBTile;
constexpr uint32_t kThreads = 384;          // 12 warps, see the role list above
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccCol = 0;            // 2 buffers x 2 issuers x 2 phases x 16 columns
constexpr uint32_t kSfaCol = 128;          // kSfBatches x 16 columns
constexpr uint32_t kSfbCol = 128 + 16 * kSfBatches;  // kSfBatches x 16 columns
constexpr uint32_t kBarrierBytes = 512;
constexpr uint32_t kSmemBytes =
    kStages * kStageBytes + kSfSlots * kSfSlotBytes + 1024 + kBarrierBytes;   // 1024: alignment slack
static_assert(kTerms == 8, "one swizzle atom of term rows per stage");

__device__ uint32_t g_mx_status = 0;

K3_DEVINL void tmem_st_32x1(uint32_t taddr, uint32_t v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(v) : "memory");
}
// 16 consecutive 32-bit columns of this warp's lane quadrant in one instruction
K3_DEVINL void tmem_st_32x16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
K3_DEVINL void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// eight consecutive 32-bit columns of this warp's lane quadrant
K3_DEVINL void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

K3_DEVINL float sum_terms(const uint32_t (&r)[8]) {
    return ((__uint_as_float(r[0]) + __uint_as_float(r[1])) + (__uint_as_float(r[2]) + __uint_as_float(r[3]))) +
           ((__uint_as_float(r[4]) + __uint_as_float(r[5])) + (__uint_as_float(r[6]) + __uint_as_float(r[7])));
}

K3_DEVINL void mma_mx4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                       uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::
            "r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc)
        : "memory");
}

// Block-scaled instruction descriptor: A = B = E2M1 (1), UE8M0 scales, M = 128, N = 16,
// K = 64, K-major operands; sf = first of the two scale bytes (0 or 2) of the 32-bit
// scale column that this MMA's two 32-element blocks use.
K3_DEVINL uint32_t make_idesc_mx4(uint32_t sf) {
    return (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24) | (sf << 29) |
           (sf << 4);
}

struct MxArgs {
    const uint32_t *ids;        // expert id per rank
    uint16_t *out;              // [ranks, out_width] bf16
    uint32_t ranks, first_local, local_count;
    uint32_t w_rows;            // rows per expert per matrix
    uint32_t k;
    uint32_t shared_vector;     // 1: every rank uses activation vector 0 (gate/up)
    int activation;
    float beta, linear_beta;
    uint8_t *act_terms;         // gate/up: E2M1 terms of the produced activation [ranks * kTerms, w_rows / 2]
    uint8_t *act_sf;            //          and their block scales [ranks * kTerms, w_rows / 32]
    DecodeTail tail;            // down: the layer's tail (tail.out null: none)
};

struct MxMaps {
    CUtensorMap a0, a1;        // packed E2M1 weights of phase 0 / phase 1, as bytes [rows, K/2]
    CUtensorMap b;             // vector terms, packed E2M1: rows kTerms*v .. kTerms*v + 7 of [vectors*kTerms, K/2]
    CUtensorMap sfa0, sfa1;    // weight block scales [rows, K/32]
    CUtensorMap sfb;           // term block scales [vectors*kTerms, K/32]
};

// kGateUp: two phases (w1 then w3) into accumulator columns [0,16) and [16,32) per issuer,
// fused activation.  Otherwise one phase, plain bf16 output.
template <bool kGateUp>
__global__ void __launch_bounds__(kThreads, 1)
decode_mx_kernel(const __grid_constant__ MxMaps maps, MxArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char *sf_smem = base + kStages * kStageBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sf_smem + kSfSlots * kSfSlotBytes);
    uint64_t *full = bars, *empty = bars + kStages;
    uint64_t *sf_full = bars + 2 * kStages;            // [kSfBatches]
    uint64_t *sf_empty = sf_full + kSfBatches;         // [kSfBatches]
    uint64_t *sfs_full = sf_empty + kSfBatches;        // [kSfSlots]
    uint64_t *sfs_empty = sfs_full + kSfSlots;         // [kSfSlots]
    uint64_t *acc_full = sfs_empty + kSfSlots, *acc_empty = acc_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t steps = a.k / kKStage;
    const uint32_t phases = kGateUp ? 2u : 1u;
    const uint32_t tiles = a.w_rows / 128u;
    const uint32_t items = a.ranks * tiles;

    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (uint32_t s = 0; s < kStages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (uint32_t b = 0; b < kSfBatches; b++) {
            mbar_init(&sf_full[b], 4);
            mbar_init(&sf_empty[b], 2);
        }
        for (uint32_t b = 0; b < kSfSlots; b++) {
            mbar_init(&sfs_full[b], 1);
            mbar_init(&sfs_empty[b], 4);
        }
        for (uint32_t b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 2);
            mbar_init(&acc_empty[b], 4);
        }
        fence_barrier_init();
    }
    // rows 8..15 of every stage's N = 16 operand (its second swizzle atom) are never
    // written by the TMA: zero them once
    for (uint32_t i = threadIdx.x; i < kStages * (kBTile - kBTx) / 16u; i += blockDim.x) {
        const uint32_t stage = i / ((kBTile - kBTx) / 16u), unit = i % ((kBTile - kBTx) / 16u);
        reinterpret_cast<uint4 *>(base + stage * kStageBytes + kATile + kBTx)[unit] = make_uint4(0u, 0u, 0u, 0u);
    }
    fence_proxy_async();
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // weight tile + term tile of every stage
        if (lane == 0) {
            prefetch_tensormap(&maps.a0);
            prefetch_tensormap(&maps.a1);
            prefetch_tensormap(&maps.b);
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (uint32_t it = blockIdx.x; ok && it < items; it += gridDim.x) {
                const uint32_t rank = it / tiles, tile = it % tiles;
                const uint32_t id = a.ids[rank];
                if (id < a.first_local || id >= a.first_local + a.local_count) continue;
                const int32_t y = (int32_t)((id - a.first_local) * a.w_rows + tile * 128u);
                const int32_t yb = a.shared_vector ? 0 : (int32_t)(kTerms * rank);
                for (uint32_t p = 0; ok && p < phases; p++) {
                    const void *map_a = p == 0 ? (const void *)&maps.a0 : (const void *)&maps.a1;
                    for (uint32_t st = 0; st < steps; st++) {
                        if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                        unsigned char *dst = base + s * kStageBytes;
                        mbar_arrive_expect_tx(&full[s], kATile + kBTx);
                        tma_load_2d(dst, map_a, &full[s], (int32_t)(st * 128u), y);            // x in bytes
                        tma_load_2d(dst + kATile, &maps.b, &full[s], (int32_t)(st * 128u), yb);
                        if (++s == kStages) { s = 0; ph ^= 1u; }
                    }
                }
            }
        }
    } else if (warp == 10) {
        // block scales of two stages (512 K) at a time: 128 weight rows x 16 bytes and the
        // 8 term rows x 16 bytes, into the shared-memory scale ring
        if (lane == 0) {
            prefetch_tensormap(&maps.sfa0);
            prefetch_tensormap(&maps.sfa1);
            prefetch_tensormap(&maps.sfb);
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (uint32_t it = blockIdx.x; ok && it < items; it += gridDim.x) {
                const uint32_t rank = it / tiles, tile = it % tiles;
                const uint32_t id = a.ids[rank];
                if (id < a.first_local || id >= a.first_local + a.local_count) continue;
                const int32_t y = (int32_t)((id - a.first_local) * a.w_rows + tile * 128u);
                const int32_t yb = a.shared_vector ? 0 : (int32_t)(kTerms * rank);
                for (uint32_t p = 0; ok && p < phases; p++) {
                    const void *map_s = p == 0 ? (const void *)&maps.sfa0 : (const void *)&maps.sfa1;
                    for (uint32_t st = 0; st < steps; st += 2u) {
                        if (!mbar_wait(&sfs_empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                        unsigned char *dst = sf_smem + s * kSfSlotBytes;
                        mbar_arrive_expect_tx(&sfs_full[s], kSfaBytes + kTerms * 16u);
                        tma_load_2d(dst, map_s, &sfs_full[s], (int32_t)(st * 8u), y);
                        tma_load_2d(dst + kSfaBytes, &maps.sfb, &sfs_full[s], (int32_t)(st * 8u), yb);
                        if (++s == kSfSlots) { s = 0; ph ^= 1u; }
                    }
                }
            }
        }
    } else if (warp == 1 || warp == 11) {
        // Two MMA issuers: the issue loop of one thread, not the tensor pipe, bounds
        // the rate of these small MMAs, so warp 1 takes the even stages and warp 11
        // the odd ones, each into its own accumulator columns (summed in the epilogue).
        // A scale batch covers two stages, one per issuer.
        if (lane == 0) {
            const uint32_t q = warp == 1 ? 0u : 1u;
            uint32_t s = q, ph = 0, buf = 0, pacc = 0, sb = 0, sph = 0;
            bool ok = true;
            for (uint32_t it = blockIdx.x; ok && it < items; it += gridDim.x) {
                const uint32_t rank = it / tiles;
                const uint32_t id = a.ids[rank];
                if (id < a.first_local || id >= a.first_local + a.local_count) continue;
                if (!mbar_wait(&acc_empty[buf], pacc ^ 1u, abort_flag)) break;
                tc_fence_after();
                for (uint32_t p = 0; ok && p < phases; p++) {
                    const uint32_t d = tmem + kAccCol + buf * 64u + q * 32u + p * 16u;
                    for (uint32_t st = q; st < steps; st += 2u) {
                        if (!mbar_wait(&full[s], ph, abort_flag) || !mbar_wait(&sf_full[sb], sph, abort_flag)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        unsigned char *src = base + s * kStageBytes;
                        const uint64_t da = make_desc_sw128(smem_u32(src));
                        const uint64_t db = make_desc_sw128(smem_u32(src + kATile));
#pragma unroll
                        for (uint32_t j = 0; j < 4u; j++) {
                            // stage q of the batch holds the 128-K chunks 2q and 2q + 1 (4 columns
                            // each); MMA j takes scale bytes 2 (j & 1), 2 (j & 1) + 1 of chunk 2q + j / 2
                            const uint32_t sfs = sb * 16u + (2u * q + (j >> 1)) * 4u;
                            mma_mx4(d, da + 2u * j, db + 2u * j, make_idesc_mx4(2u * (j & 1u)), tmem + kSfaCol + sfs,
                                    tmem + kSfbCol + sfs, (st != q || j != 0u) ? 1u : 0u);
                        }
                        mma_commit(&empty[s]);
                        s += 2u;
                        if (s >= kStages) { s -= kStages; ph ^= 1u; }
                        mma_commit(&sf_empty[sb]);
                        if (++sb == kSfBatches) { sb = 0; sph ^= 1u; }
                    }
                }
                if (!ok) break;
                mma_commit(&acc_full[buf]);
                if (++buf == 2u) { buf = 0; pacc ^= 1u; }
            }
        }
    } else if (warp < 6) {
        // scale writers: shared memory -> tensor memory, warp w fills lane quadrant w % 4
        const uint32_t quad = warp & 3u;
        const uint32_t lane_base = (32u * quad) << 16;
        uint32_t sb = 0, sph = 0, ss = 0, ssph = 0;
        bool ok = true;
        for (uint32_t it = blockIdx.x; ok && it < items; it += gridDim.x) {
            const uint32_t id = a.ids[it / tiles];
            if (id < a.first_local || id >= a.first_local + a.local_count) continue;
            for (uint32_t st = 0; st < phases * steps; st += 2u) {
                if (!mbar_wait(&sfs_full[ss], ssph, abort_flag)) { ok = false; break; }
                const unsigned char *src = sf_smem + ss * kSfSlotBytes;
                uint4 cur[4];
#pragma unroll
                for (uint32_t c = 0; c < 4u; c++)
                    cur[c] = *reinterpret_cast<const uint4 *>(src + (32u * c + lane) * 16u);
                // scale rows of the N operand sit in lanes 0..15 of the first column of a group:
                // term rows 0..7 (lanes 8.. repeat them: those operand rows are zero)
                const uint4 curb = *reinterpret_cast<const uint4 *>(src + kSfaBytes + (lane & (kTerms - 1u)) * 16u);
                if (!mbar_wait(&sf_empty[sb], sph ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                // column (128-K chunk q, row group c) = q * 4 + c of the batch's 16 columns
                const uint32_t va[16] = {cur[0].x, cur[1].x, cur[2].x, cur[3].x, cur[0].y, cur[1].y,
                                         cur[2].y, cur[3].y, cur[0].z, cur[1].z, cur[2].z, cur[3].z,
                                         cur[0].w, cur[1].w, cur[2].w, cur[3].w};
                const uint32_t vbb[16] = {curb.x, curb.x, curb.x, curb.x, curb.y, curb.y, curb.y, curb.y,
                                          curb.z, curb.z, curb.z, curb.z, curb.w, curb.w, curb.w, curb.w};
                tmem_st_32x16(tmem + lane_base + kSfaCol + sb * 16u, va);
                tmem_st_32x16(tmem + lane_base + kSfbCol + sb * 16u, vbb);
                // The shared-memory slot goes back to the TMA producer only now: the
                // stores above consumed every loaded register, so the loads have
                // completed (an arrive right after issuing them would not wait for that).
                __syncwarp();
                if (lane == 0) mbar_arrive(&sfs_empty[ss]);
                if (++ss == kSfSlots) { ss = 0; ssph ^= 1u; }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sf_full[sb]);
                if (++sb == kSfBatches) { sb = 0; sph ^= 1u; }
            }
        }
    } else if (warp < 10) {
        // epilogue: warp w reads lane quadrant w % 4
        const uint32_t quad = warp & 3u;
        const uint32_t m = 32u * quad + lane;
        uint32_t buf = 0, pacc = 0;
        for (uint32_t it = blockIdx.x; it < items; it += gridDim.x) {
            const uint32_t rank = it / tiles, tile = it % tiles;
            const uint32_t id = a.ids[rank];
            if (id < a.first_local || id >= a.first_local + a.local_count) continue;
            if (!mbar_wait(&acc_full[buf], pacc, abort_flag)) break;
            tc_fence_after();
            const uint32_t t0 = tmem + ((32u * quad) << 16) + kAccCol + buf * 64u;
            uint32_t e0[8], o0[8], e1[8], o1[8];
            tmem_ld_32x8(t0, e0);                           // even stages
            tmem_ld_32x8(t0 + 32u, o0);                     // odd stages
            if (kGateUp) {
                tmem_ld_32x8(t0 + 16u, e1);
                tmem_ld_32x8(t0 + 48u, o1);
            }
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            if (++buf == 2u) { buf = 0; pacc ^= 1u; }
            const float v0 = sum_terms(e0) + sum_terms(o0);
            uint16_t *dst = a.out + (uint64_t)rank * a.w_rows + tile * 128u + m;
            if (kGateUp) {
                const float v1 = sum_terms(e1) + sum_terms(o1);
                const float g = bf16_bits_to_float(float_to_bf16_bits(v0));
                const float u = bf16_bits_to_float(float_to_bf16_bits(v1));
                const uint16_t act_bits = float_to_bf16_bits(activation(g, u, a.activation, a.beta, a.linear_beta));
                *dst = act_bits;
                if (a.act_terms != nullptr) {
                    uint32_t code[kTerms], sbyte[kTerms];
                    split_block_e2m1(bf16_bits_to_float(act_bits), code, sbyte);
                    store_block_e2m1(a.act_terms + (uint64_t)rank * kTerms * (a.w_rows / 2u),
                                     a.act_sf + (uint64_t)rank * kTerms * (a.w_rows / 32u), a.w_rows / 2u,
                                     a.w_rows / 32u, tile * 4u + quad, code, sbyte, lane);
                }
            } else {
                *dst = float_to_bf16_bits(v0);
                if (a.tail.out != nullptr && !tail_arrive(a.tail, tile * 4u + quad, lane)) *abort_flag = 1u;
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0u) atomicExch(&g_mx_status, 1u);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

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

// bytes [rows, row_bytes], box = 128 bytes x box_rows rows, 128-byte swizzle
bool map_bytes(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
    auto fn = encode_fn();
    if (!fn || (((uintptr_t)ptr) & 15u) != 0 || row_bytes % 16u != 0) return false;
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {128, box_rows};
    const cuuint32_t es[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, es,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// block scales [rows, K/32] bytes, box = 16 bytes (512 K) x box_rows rows
bool map_sf(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t k, uint32_t box_rows) {
    auto fn = encode_fn();
    if (!fn || (((uintptr_t)ptr) & 15u) != 0) return false;
    const cuuint64_t dims[2] = {k / 32u, rows};
    const cuuint64_t strides[1] = {k / 32u};
    const cuuint32_t box[2] = {16, box_rows};
    const cuuint32_t es[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, es,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

uint32_t k3_decode_mx_status() {
    uint32_t v = 0xffffffffu;
    if (cudaMemcpyFromSymbol(&v, g_mx_status, sizeof(v)) != cudaSuccess) (void)cudaGetLastError();
    return v;
}

bool k3_decode_mx_status_clear() {
    const uint32_t zero = 0u;
    if (cudaMemcpyToSymbol(g_mx_status, &zero, sizeof(zero)) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return true;
}

size_t k3_decode_mx_scratch_bytes(const k3_moe_layer_desc *d) {
    // token terms and scales, activation terms and scales, arrival words of the tail,
    // scores and choices of the routing step
    return (size_t)kTerms * d->hidden / 2u + (size_t)kTerms * d->hidden / 32u +
           (size_t)kTerms * d->top_k * d->expert_hidden / 2u + (size_t)kTerms * d->top_k * d->expert_hidden / 32u +
           (size_t)d->hidden / 32u * 4u + 2u * 1024u * 4u + 6u * 256u;
}

bool k3_decode_mx_supported(const k3_moe_layer_desc *d) {
    return d->hidden % 512u == 0 && d->expert_hidden % 512u == 0 && d->top_k <= 32u && encode_fn() != nullptr &&
           d->shared_hidden <= 8192u &&
           ((((uintptr_t)d->w1_packed) | ((uintptr_t)d->w3_packed) | ((uintptr_t)d->w2_packed)) & 15u) == 0 &&
           ((((uintptr_t)d->w1_scales) | ((uintptr_t)d->w3_scales) | ((uintptr_t)d->w2_scales)) & 15u) == 0;
}

void k3_decode_mx_vector_scratch(const k3_moe_layer_desc *d, void *scratch, void **x_terms, void **x_sf) {
    auto align = [](uint8_t *p) { return (uint8_t *)(((uintptr_t)p + 255u) & ~(uintptr_t)255u); };
    uint8_t *terms = align((uint8_t *)scratch);
    *x_terms = terms;
    *x_sf = align(terms + (size_t)kTerms * d->hidden / 2u);
}

void *k3_decode_mx_tail_words(const k3_moe_layer_desc *d, void *scratch) {
    auto align = [](uint8_t *p) { return (uint8_t *)(((uintptr_t)p + 255u) & ~(uintptr_t)255u); };
    uint8_t *x_terms = nullptr, *x_sf = nullptr;
    k3_decode_mx_vector_scratch(d, scratch, (void **)&x_terms, (void **)&x_sf);
    uint8_t *a_terms = align(x_sf + (size_t)kTerms * d->hidden / 32u);
    uint8_t *a_sf = align(a_terms + (size_t)kTerms * d->top_k * d->expert_hidden / 2u);
    return align(a_sf + (size_t)kTerms * d->top_k * d->expert_hidden / 32u);
}

void *k3_decode_mx_route_words(const k3_moe_layer_desc *d, void *scratch) {
    uint8_t *tail = (uint8_t *)k3_decode_mx_tail_words(d, scratch);
    return (void *)(((uintptr_t)(tail + (size_t)d->hidden / 32u * 4u) + 255u) & ~(uintptr_t)255u);
}

// Routed experts of one token: act [top_k, I] and rows_out [top_k, hidden] in rank
// order (ids on the device) from the token's E2M1 terms in `scratch`.
bool k3_decode_mx_experts(const k3_moe_layer_desc *d, const void *ids, void *act, void *rows_out,
                          void *scratch, void *between, const k3_decode_tail *tail, cudaStream_t stream) {
    const uint32_t H = d->hidden, I = d->expert_hidden, k = d->top_k;
    auto align = [](uint8_t *p) { return (uint8_t *)(((uintptr_t)p + 255u) & ~(uintptr_t)255u); };
    uint8_t *x_terms = nullptr, *x_sf = nullptr;
    k3_decode_mx_vector_scratch(d, scratch, (void **)&x_terms, (void **)&x_sf);
    uint8_t *a_terms = align(x_sf + (size_t)kTerms * H / 32u);
    uint8_t *a_sf = align(a_terms + (size_t)kTerms * k * I / 2u);
    const size_t smem = kSmemBytes;
    if (!set_max_dynamic_smem((const void *)decode_mx_kernel<true>, smem) ||
        !set_max_dynamic_smem((const void *)decode_mx_kernel<false>, smem)) {
        return false;
    }
    // Tensor maps depend only on the tables, the scratch block and the shape.  Encoding
    // ten maps costs more host time than the launches, so the sets of the most recent
    // layers are kept (a model alternates between its layers' descriptors token by
    // token); when the table is full it starts over.
    struct MapKey {
        int device;
        const void *p[7];
        uint32_t dims[4];
        bool operator<(const MapKey &o) const {
            if (device != o.device) return device < o.device;
            const int c = memcmp(p, o.p, sizeof(p));
            return c != 0 ? c < 0 : memcmp(dims, o.dims, sizeof(dims)) < 0;
        }
    };
    struct MapSet {
        MxMaps gu, dn;
    };
    constexpr size_t kCachedLayers = 256;
    static std::mutex map_lock;
    static std::map<MapKey, MapSet> cached;
    MapKey key{};
    key.device = current_device();
    const void *ptrs[7] = {d->w1_packed, d->w3_packed, d->w2_packed, d->w1_scales, d->w3_scales, d->w2_scales, scratch};
    memcpy(key.p, ptrs, sizeof(ptrs));
    key.dims[0] = H; key.dims[1] = I; key.dims[2] = k; key.dims[3] = d->local_expert_count;
    MxMaps gu, dn;
    {
        std::lock_guard<std::mutex> guard(map_lock);
        auto it = cached.find(key);
        if (it == cached.end()) {
            const uint64_t total = (uint64_t)d->local_expert_count;
            if (!map_bytes(&gu.a0, d->w1_packed, total * I, H / 2u, 128) ||
                !map_bytes(&gu.a1, d->w3_packed, total * I, H / 2u, 128) ||
                !map_bytes(&gu.b, x_terms, kTerms, H / 2u, kTerms) || !map_sf(&gu.sfa0, d->w1_scales, total * I, H, 128) ||
                !map_sf(&gu.sfa1, d->w3_scales, total * I, H, 128) || !map_sf(&gu.sfb, x_sf, kTerms, H, kTerms) ||
                !map_bytes(&dn.a0, d->w2_packed, total * H, I / 2u, 128) ||
                !map_bytes(&dn.b, a_terms, (uint64_t)kTerms * k, I / 2u, kTerms) ||
                !map_sf(&dn.sfa0, d->w2_scales, total * H, I, 128) ||
                !map_sf(&dn.sfb, a_sf, (uint64_t)kTerms * k, I, kTerms)) {
                return false;
            }
            dn.a1 = dn.a0;
            dn.sfa1 = dn.sfa0;
            if (cached.size() >= kCachedLayers) cached.clear();
            cached.emplace(key, MapSet{gu, dn});
        } else {
            gu = it->second.gu;
            dn = it->second.dn;
        }
    }
    MxArgs a{};
    a.ids = (const uint32_t *)ids;
    a.ranks = k;
    a.first_local = d->local_expert_first;
    a.local_count = d->local_expert_count;
    a.activation = d->activation;
    a.beta = d->beta;
    a.linear_beta = d->linear_beta;
    const int sms = sm_count();
    // gate/up + activation
    a.out = (uint16_t *)act;
    a.act_terms = a_terms;
    a.act_sf = a_sf;
    a.w_rows = I;
    a.k = H;
    a.shared_vector = 1u;
    decode_mx_kernel<true><<<sms, kThreads, smem, stream>>>(gu, a);
    if (!launch_ok()) return false;
    if (between && cudaEventRecord((cudaEvent_t)between, stream) != cudaSuccess) return false;
    // down (+ its share of the layer's tail)
    if (tail != nullptr) {
        if (d->local_expert_first != 0u || d->local_expert_count != d->expert_count) return false;
        a.tail.out = (uint16_t *)tail->out;
        a.tail.rows = (const uint16_t *)rows_out;
        a.tail.weights = (const float *)tail->weights;
        a.tail.shared = (const uint16_t *)tail->shared;
        a.tail.residual = (const uint16_t *)tail->residual;
        a.tail.count = (uint32_t *)k3_decode_mx_tail_words(d, scratch);
        a.tail.epoch = tail->epoch & 0xffffffu;
        a.tail.expected = tail->expected;
        a.tail.ranks = k;
        a.tail.hidden = H;
    }
    a.out = (uint16_t *)rows_out;
    a.act_terms = nullptr;
    a.act_sf = nullptr;
    a.w_rows = H;
    a.k = I;
    a.shared_vector = 0u;
    decode_mx_kernel<false><<<sms, kThreads, smem, stream>>>(dn, a);
    return launch_ok();
}
