// Ragged grouped GEMM on the block-scaled tensor-core path
// (tcgen05.mma kind::mxf8f6f4, scale_vec::1X) for layer-major prefill.
//
//   out[r, m] = sum_k W[g(r)][m, k] * x[r, k]      r: token rows grouped by expert
//
// Weights stay in their checkpoint form: packed E2M1 nibbles are expanded into
// the MMA's 8-bit containers by the TMA unit (tensor-map type 16U4_ALIGN16B) and
// the E8M0 scales go to tensor memory with tcgen05.st - no thread converts a
// weight.  Token rows are split once into two E4M3 terms with a shared E8M0
// scale per 32 columns, x = 2^s (hi + lo); bf16 carries 8 significant bits and
// each term 4, so every element within 2^10 of its block maximum is exact and
// the rest is held to 2^-17 of the block maximum.  Each K block of 32 issues two
// MMAs per weight tile (hi and lo against the same weight tile and scales).
//
// Work item = two 128-row weight tiles x up to 128 token rows of one group over
// the whole K extent (gate+up with fused activation, or 256 rows of the down
// projection).  One CTA per SM, persistent; the item list is derived in-kernel from the
// group offsets and handed out by a global counter: the weight producer takes the next
// item with one atomicAdd and publishes it to the other roles through a mailbox in
// shared memory, so a CTA that drew short row tiles simply takes more of them.  Items
// are numbered with the row tiles of one (expert, weight tile) adjacent: CTAs that take
// neighbouring items stream the same weights at the same time and the second reader
// finds them in L2.  Warps: 0 TMA producer (weights), 2 TMA producer (token terms),
// 3 TMA producer (block scales), 1 and 16 MMA issuers (one per weight tile), 4-7
// scale writers (shared memory -> tensor memory, one lane quadrant each), 8-15
// epilogue.  All barrier waits are bounded.
#include "k3_grouped.h"
#include "k3_moe_ops.h"
#include "k3_tc_ptx.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

using namespace k3;
using namespace k3::tc;

namespace {

constexpr uint32_t BM = 128, BN = 128, KS = 128;          // K per pipeline stage
constexpr uint32_t kStages = 3;
constexpr uint32_t kATile = BM * 128u;                    // bytes in shared memory (8-bit containers)
constexpr uint32_t kATx = BM * 64u;                       // bytes the TMA transaction counts (packed)
constexpr uint32_t kBTile = BN * 128u;
constexpr uint32_t kBBox = 32u;                           // token rows per TMA box
constexpr uint32_t kStageBytes = 2u * kATile + 2u * kBTile;        // A0 | A1 | Bhi | Blo
constexpr uint32_t kThreads = 544;                        // 17 warps
constexpr uint32_t kSfBatches = 3;                        // scale ring in tensor memory: batches of 4 stages
constexpr uint32_t kSfSlots = 4;                          // scale ring in shared memory
constexpr uint32_t kSfKind = BM * 16u;                    // one table's 128 rows x 16 scale bytes
constexpr uint32_t kSfSlotBytes = 3u * kSfKind;           // SFA0 | SFA1 | SFB
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccCol = 0;                           // tile 0: [0,128), tile 1: [128,256)
constexpr uint32_t kSfa0Col = 256;                        // kSfBatches x 16 columns each
constexpr uint32_t kSfa1Col = kSfa0Col + 16u * kSfBatches;
constexpr uint32_t kSfbCol = kSfa1Col + 16u * kSfBatches;
constexpr uint32_t kMaxGroups = 1024;
constexpr uint32_t kItemSlots = 4;                        // mailbox of item numbers, producer -> other roles
constexpr uint32_t kItemReaders = 16;                     // term + scale producers, 2 issuers, 4 writers, 8 epilogue warps
constexpr uint32_t kNoItem = 0xffffffffu;
constexpr uint32_t kBarBytes = 512;
constexpr uint32_t kSmemBytes =
    kStages * kStageBytes + kSfSlots * kSfSlotBytes + 1024u + kBarBytes + (kMaxGroups + 1u) * 4u;

enum EMode : int { kEAct = 0, kEBf16 = 1 };

__device__ uint32_t g_gmx_status = 0;

K3_DEVINL void tmem_st_32x16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
K3_DEVINL void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

K3_DEVINL void mma_mx(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                      uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::
            "r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc)
        : "memory");
}

// A = E2M1 (5), B = E4M3 (0), UE8M0 scales, M = 128, K-major; sf = byte of the scale column
K3_DEVINL uint32_t make_idesc_mx(uint32_t n, uint32_t sf) {
    return (5u << 7) | (0u << 10) | ((n >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24) | (sf << 29) | (sf << 4);
}

// Two-term E4M3 form of a block of 32 values held one per lane:
// v = 2^(scale_byte - 127) * (hi + lo).  The block exponent puts the largest
// magnitude in [128, 256), inside E4M3's finite range (448).
struct SplitScale {
    float mult;             // 2^-(block exponent)
    uint32_t scale_byte;    // E8M0
};
K3_DEVINL SplitScale block_scale(float v) {
    const uint32_t mx = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(v)));
    uint32_t be = (mx >> 23) & 0xffu;                 // biased exponent of the block maximum
    be = min(max(be, 8u), 254u);
    SplitScale s;
    s.mult = __uint_as_float((261u - be) << 23);      // 2^(7 - (be - 127))
    s.scale_byte = be - 7u;
    return s;
}
// (hi0, hi1) in the low 16 bits, (lo0, lo1) in the high 16 bits
K3_DEVINL uint32_t split_pair(float a, float b) {
    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(hi, __NV_E4M3);
    const float2 hf = __half22float2(__half2(hr));
    const __nv_fp8x2_storage_t lo =
        __nv_cvt_float2_to_fp8x2(make_float2(a - hf.x, b - hf.y), __NV_SATFINITE, __NV_E4M3);
    return (uint32_t)hi | ((uint32_t)lo << 16);
}

struct GmxArgs {
    const uint32_t *offsets;             // [groups+1]
    uint16_t *out;                       // bf16 [rows, out_width] (may be null in gate/up mode)
    uint8_t *act_hi, *act_lo, *act_sf;   // gate/up mode: E4M3 terms and block scales of the activation
    uint32_t groups, rows, w_rows, k, out_width, m_items;
    uint32_t *item_counter;              // zero before the launch; items are drawn from it
    int activation;
    float beta, linear_beta;
};

struct Item {
    uint32_t group, row_start, rows_valid, m_item;
};

// Item w -> (group, weight tile, row tile).  prefix[g] = row tiles of the groups before
// g; group g owns items [prefix[g] * m_items, prefix[g + 1] * m_items), numbered with
// the row tile fastest.
K3_DEVINL Item decode_item(uint32_t w, const uint32_t *prefix, const GmxArgs &a) {
    Item it;
    const uint32_t nt = w / a.m_items;             // prefix[group] <= nt < prefix[group + 1]
    uint32_t lo = 0, hi = a.groups;
    while (hi - lo > 1u) {
        const uint32_t mid = (lo + hi) >> 1;
        if (prefix[mid] <= nt) lo = mid; else hi = mid;
    }
    it.group = lo;
    const uint32_t tiles = prefix[lo + 1u] - prefix[lo];
    const uint32_t j = w - prefix[lo] * a.m_items;
    it.m_item = j / tiles;
    const uint32_t begin = a.offsets[lo], end = a.offsets[lo + 1u];
    it.row_start = begin + (j % tiles) * BN;
    it.rows_valid = min(BN, end - it.row_start);
    return it;
}

// Accumulator columns [0, 256) as two buffers of 128: a row tile of at most 64 rows takes
// one buffer (tile 0 in its first 64 columns, tile 1 in the other 64), so that its MMAs run
// while the epilogue still reads the item before; a larger tile takes both (tile 0 in
// [0, 128), tile 1 in [128, 256)).  Issuers and epilogue warps walk the items in the same
// order and keep the same books: uses per buffer (the barriers' phase) and whose turn it is.
struct AccBuffers {
    uint32_t use0 = 0u, use1 = 0u;
    uint32_t turn = 0u;
    __device__ uint32_t uses(uint32_t b) const { return b == 0u ? use0 : use1; }
    __device__ bool small(uint32_t rows_valid) const { return rows_valid <= 64u; }
    __device__ uint32_t first(bool is_small) const { return is_small ? turn : 0u; }
    __device__ uint32_t column(bool is_small, uint32_t b0, uint32_t tile) const {
        return is_small ? b0 * 128u + tile * 64u : tile * BN;
    }
    __device__ void advance(bool is_small, uint32_t b0) {
        if (is_small) {
            if (b0 == 0u) use0++; else use1++;
            turn ^= 1u;
        } else {
            use0++;
            use1++;
            turn = 0u;
        }
    }
};

struct GmxMaps {
    CUtensorMap a0, a1;        // packed E2M1 weights (4-bit elements, expanded by the copy)
    CUtensorMap bhi, blo;      // token terms, E4M3 bytes
    CUtensorMap sfa0, sfa1;    // weight block scales [rows, K/32]
    CUtensorMap sfb;           // token block scales  [rows, K/32]
};

template <int kE>
__global__ void __launch_bounds__(kThreads, 1)
grouped_mx_kernel(const __grid_constant__ GmxMaps maps, GmxArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char *sf_smem = base + kStages * kStageBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sf_smem + kSfSlots * kSfSlotBytes);
    uint64_t *full = bars, *empty = full + kStages;
    uint64_t *sf_full = empty + kStages, *sf_empty = sf_full + kSfBatches;
    uint64_t *sfs_full = sf_empty + kSfBatches, *sfs_empty = sfs_full + kSfSlots;
    uint64_t *acc_full = sfs_empty + kSfSlots, *acc_empty = acc_full + 2;      // two accumulator buffers
    uint64_t *item_full = acc_empty + 2, *item_empty = item_full + kItemSlots;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(item_empty + kItemSlots);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    uint32_t *total_items_s = tmem_slot + 2;
    volatile uint32_t *item_box = tmem_slot + 3;          // [kItemSlots]
    uint32_t *prefix = reinterpret_cast<uint32_t *>(reinterpret_cast<unsigned char *>(bars) + kBarBytes);
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t steps = a.k / KS;
    const uint32_t tile_rows = kE == kEAct ? BM : 2u * BM;     // weight rows one item advances

    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (uint32_t s = 0; s < kStages; s++) {
            mbar_init(&full[s], 2);          // two producers arrive (weights, token terms)
            mbar_init(&empty[s], 2);         // both MMA issuers release a stage
        }
        for (uint32_t b = 0; b < kSfBatches; b++) {
            mbar_init(&sf_full[b], 4);
            mbar_init(&sf_empty[b], 2);
        }
        for (uint32_t b = 0; b < kSfSlots; b++) {
            mbar_init(&sfs_full[b], 1);
            mbar_init(&sfs_empty[b], 4);
        }
        for (uint32_t b = 0; b < 2u; b++) {
            mbar_init(&acc_full[b], 2);
            mbar_init(&acc_empty[b], 8);
        }
        for (uint32_t b = 0; b < kItemSlots; b++) {
            mbar_init(&item_full[b], 1);
            mbar_init(&item_empty[b], kItemReaders);
        }
        fence_barrier_init();
    }
    {   // exclusive prefix of ceil(rows_g / BN) over the groups (<= 1024)
        __shared__ uint32_t warp_tot[kThreads / kWarp];
        uint32_t v[2], incl[2], run = 0;
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
        const uint32_t excl = warp_base + scan - run;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const uint32_t g = threadIdx.x * 2u + j;
            if (g < a.groups) prefix[g] = excl + incl[j] - v[j];
            if (g + 1u == a.groups) {
                prefix[a.groups] = excl + incl[j];
                *total_items_s = (excl + incl[j]) * a.m_items;
            }
        }
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t total_items = *total_items_s;

    // Reader side of the item mailbox (whole warp, or one thread with lane_count 1):
    // the n-th call returns the n-th item this CTA drew, kNoItem when there are no more.
    uint32_t item_seq = 0;
    auto next_item = [&]() -> uint32_t {
        const uint32_t slot = item_seq % kItemSlots, parity = (item_seq / kItemSlots) & 1u;
        item_seq++;
        uint32_t w = kNoItem;
        if (lane == 0) {
            if (mbar_wait(&item_full[slot], parity, abort_flag)) {
                w = item_box[slot];
                mbar_arrive(&item_empty[slot]);
            }
        }
        return w;
    };

    if (warp == 0) {
        // ================================ TMA producer: weights; draws the items
        if (lane == 0) {
            prefetch_tensormap(&maps.a0);
            prefetch_tensormap(&maps.a1);
            uint32_t s = 0, ph = 0, seq = 0;
            bool ok = true;
            uint32_t w = atomicAdd(a.item_counter, 1u);
            while (ok) {
                const uint32_t slot = seq % kItemSlots, parity = (seq / kItemSlots) & 1u;
                seq++;
                if (!mbar_wait(&item_empty[slot], parity ^ 1u, abort_flag)) break;
                const bool valid = w < total_items;
                item_box[slot] = valid ? w : kNoItem;
                mbar_arrive(&item_full[slot]);
                if (!valid) break;
                const Item it = decode_item(w, prefix, a);
                w = atomicAdd(a.item_counter, 1u);                 // the next draw travels while this item streams
                const int32_t y0 = (int32_t)(it.group * a.w_rows + it.m_item * tile_rows);
                const int32_t y1 = kE == kEAct ? y0 : y0 + (int32_t)BM;
                for (uint32_t st = 0; st < steps; st++) {
                    if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                    unsigned char *dst = base + s * kStageBytes;
                    const int32_t x = (int32_t)(st * KS);
                    mbar_arrive_expect_tx(&full[s], 2u * kATx);
                    tma_load_2d(dst, &maps.a0, &full[s], x, y0);
                    tma_load_2d(dst + kATile, &maps.a1, &full[s], x, y1);
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 2) {
        // ================================ TMA producer: token terms
        if (lane == 0) {
            prefetch_tensormap(&maps.bhi);
            prefetch_tensormap(&maps.blo);
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (uint32_t w = next_item(); ok && w != kNoItem; w = next_item()) {
                const Item it = decode_item(w, prefix, a);
                const uint32_t boxes = (it.rows_valid + kBBox - 1u) / kBBox;
                for (uint32_t st = 0; st < steps; st++) {
                    if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                    unsigned char *dst = base + s * kStageBytes;
                    const int32_t x = (int32_t)(st * KS);
                    // only as many 32-row boxes as the tile has rows
                    mbar_arrive_expect_tx(&full[s], 2u * boxes * kBBox * 128u);
                    unsigned char *bh = dst + 2u * kATile, *bl = bh + kBTile;
                    for (uint32_t b = 0; b < boxes; b++) {
                        const int32_t y = (int32_t)(it.row_start + b * kBBox);
                        tma_load_2d(bh + b * kBBox * 128u, &maps.bhi, &full[s], x, y);
                        tma_load_2d(bl + b * kBBox * 128u, &maps.blo, &full[s], x, y);
                    }
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 3) {
        // ====================== TMA producer: block scales, 4 stages at a time
        if (lane == 0) {
            prefetch_tensormap(&maps.sfa0);
            prefetch_tensormap(&maps.sfa1);
            prefetch_tensormap(&maps.sfb);
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (uint32_t w = next_item(); ok && w != kNoItem; w = next_item()) {
                const Item it = decode_item(w, prefix, a);
                const int32_t y0 = (int32_t)(it.group * a.w_rows + it.m_item * tile_rows);
                const int32_t y1 = kE == kEAct ? y0 : y0 + (int32_t)BM;
                for (uint32_t st = 0; st < steps; st += 4u) {
                    if (!mbar_wait(&sfs_empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                    unsigned char *dst = sf_smem + s * kSfSlotBytes;
                    mbar_arrive_expect_tx(&sfs_full[s], kSfSlotBytes);
                    tma_load_2d(dst, &maps.sfa0, &sfs_full[s], (int32_t)(st * 4u), y0);
                    tma_load_2d(dst + kSfKind, &maps.sfa1, &sfs_full[s], (int32_t)(st * 4u), y1);
                    tma_load_2d(dst + 2u * kSfKind, &maps.sfb, &sfs_full[s], (int32_t)(st * 4u),
                                (int32_t)it.row_start);
                    if (++s == kSfSlots) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1 || warp == 16) {
        // ==================================================== MMA issuers
        // One thread's issue loop cannot keep the tensor pipe fed with K = 32 MMAs, so
        // warp 1 issues the MMAs of weight tile 0 and warp 16 those of tile 1.  Both
        // commit to the same stage / scale / accumulator barriers (count 2).
        if (lane == 0) {
            const uint32_t q = warp == 1 ? 0u : 1u;
            uint32_t s = 0, ph = 0, sb = 0, sph = 0;
            AccBuffers acc;
            bool ok = true;
            for (uint32_t w = next_item(); ok && w != kNoItem; w = next_item()) {
                const Item it = decode_item(w, prefix, a);
                const uint32_t n_eff = max(16u, (it.rows_valid + 15u) & ~15u);
                uint32_t idesc[4];
#pragma unroll
                for (uint32_t j = 0; j < 4u; j++) idesc[j] = make_idesc_mx(n_eff, j);
                const bool small = acc.small(it.rows_valid);
                const uint32_t b0 = acc.first(small);
                if (!mbar_wait(&acc_empty[b0], (acc.uses(b0) & 1u) ^ 1u, abort_flag) ||
                    (!small && !mbar_wait(&acc_empty[1], (acc.use1 & 1u) ^ 1u, abort_flag))) {
                    break;
                }
                tc_fence_after();
                const uint32_t d = tmem + kAccCol + acc.column(small, b0, q);
                const uint32_t sfa_col = tmem + (q == 0u ? kSfa0Col : kSfa1Col);
                for (uint32_t st = 0; st < steps; st++) {
                    if (!mbar_wait(&full[s], ph, abort_flag) ||
                        ((st & 3u) == 0u && !mbar_wait(&sf_full[sb], sph, abort_flag))) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    unsigned char *src = base + s * kStageBytes;
                    const uint64_t da = make_desc_sw128(smem_u32(src + q * kATile));
                    const uint64_t dbh = make_desc_sw128(smem_u32(src + 2u * kATile));
                    const uint64_t dbl = make_desc_sw128(smem_u32(src + 2u * kATile + kBTile));
                    const uint32_t sfs = sb * 16u + (st & 3u) * 4u;
#pragma unroll
                    for (uint32_t j = 0; j < 4u; j++) {          // K blocks of 32 inside the stage
                        mma_mx(d, da + 2u * j, dbh + 2u * j, idesc[j], sfa_col + sfs, tmem + kSfbCol + sfs,
                               (st | j) != 0u ? 1u : 0u);
                        mma_mx(d, da + 2u * j, dbl + 2u * j, idesc[j], sfa_col + sfs, tmem + kSfbCol + sfs, 1u);
                    }
                    mma_commit(&empty[s]);
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                    if ((st & 3u) == 3u) {
                        mma_commit(&sf_empty[sb]);
                        if (++sb == kSfBatches) { sb = 0; sph ^= 1u; }
                    }
                }
                if (!ok) break;
                mma_commit(&acc_full[b0]);
                if (!small) mma_commit(&acc_full[1]);
                acc.advance(small, b0);
            }
        }
    } else if (warp < 8) {
        // ================== scale writers: shared memory -> tensor memory
        // A scale column holds rows 32c .. 32c+31 (lane = row % 32), the same in every
        // lane quadrant; each warp fills its own quadrant.  One batch = 4 stages =
        // 16 columns per table.
        const uint32_t quad = warp & 3u;
        const uint32_t lane_base = (32u * quad) << 16;
        uint32_t sb = 0, sph = 0, ss = 0, ssph = 0;
        bool ok = true;
        for (uint32_t w = __shfl_sync(0xffffffffu, next_item(), 0); ok && w != kNoItem;
             w = __shfl_sync(0xffffffffu, next_item(), 0)) {
            for (uint32_t st = 0; st < steps; st += 4u) {
                if (!mbar_wait(&sfs_full[ss], ssph, abort_flag)) { ok = false; break; }
                const unsigned char *src = sf_smem + ss * kSfSlotBytes;
                uint4 v[3][4];
#pragma unroll
                for (uint32_t t = 0; t < 3u; t++)
#pragma unroll
                    for (uint32_t c = 0; c < 4u; c++)
                        v[t][c] = *reinterpret_cast<const uint4 *>(src + t * kSfKind + (32u * c + lane) * 16u);
                if (!mbar_wait(&sf_empty[sb], sph ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (uint32_t t = 0; t < 3u; t++) {
                    const uint32_t cols[16] = {v[t][0].x, v[t][1].x, v[t][2].x, v[t][3].x,
                                               v[t][0].y, v[t][1].y, v[t][2].y, v[t][3].y,
                                               v[t][0].z, v[t][1].z, v[t][2].z, v[t][3].z,
                                               v[t][0].w, v[t][1].w, v[t][2].w, v[t][3].w};
                    const uint32_t col = (t == 0 ? kSfa0Col : t == 1 ? kSfa1Col : kSfbCol) + sb * 16u;
                    tmem_st_32x16(tmem + lane_base + col, cols);
                }
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
    } else {
        // ======================================================== epilogue
        // Eight warps: quadrant = warp % 4 (tensor-memory lanes), column chunks of 32
        // token rows alternate between the two warps of a quadrant.  A warp signals
        // the accumulators free right after its last tensor-memory load.
        const uint32_t quad = warp & 3u;
        const uint32_t half = (warp - 8u) >> 2;
        const uint32_t m = 32u * quad + lane;            // weight row inside the tile
        AccBuffers acc;
        for (uint32_t w = __shfl_sync(0xffffffffu, next_item(), 0); w != kNoItem;
             w = __shfl_sync(0xffffffffu, next_item(), 0)) {
            const Item it = decode_item(w, prefix, a);
            const bool small = acc.small(it.rows_valid);
            const uint32_t b0 = acc.first(small);
            if (!mbar_wait(&acc_full[b0], acc.uses(b0) & 1u, abort_flag) ||
                (!small && !mbar_wait(&acc_full[1], acc.use1 & 1u, abort_flag))) {
                break;
            }
            acc.advance(small, b0);
            tc_fence_after();
            const uint32_t t0 = tmem + ((32u * quad) << 16) + kAccCol + acc.column(small, b0, 0u);
            const uint32_t tile1 = acc.column(small, b0, 1u) - acc.column(small, b0, 0u);
            const uint32_t col0 = it.m_item * tile_rows + m;
            const uint32_t col1 = kE == kEAct ? col0 : col0 + BM;
            const bool in0 = col0 < a.w_rows, in1 = col1 < a.w_rows;
            bool released = false;
#pragma unroll 1
            for (uint32_t c = 32u * half; c < BN; c += 64u) {
                const bool mine = c < it.rows_valid;
                uint32_t r0[32], r1[32];
                if (mine) {
                    tmem_ld_32x32(t0 + c, r0);
                    tmem_ld_32x32(t0 + tile1 + c, r1);
                    tmem_ld_wait();
                }
                if (!released && (!mine || c + 64u >= it.rows_valid)) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&acc_empty[b0]);
                        if (!small) mbar_arrive(&acc_empty[1]);
                    }
                    released = true;
                }
                if (!mine) break;
                const uint32_t n_here = min(32u, it.rows_valid - c);
                if (kE == kEAct) {
#pragma unroll
                    for (uint32_t j = 0; j < 32u; j += 2u) {
                        if (j >= n_here) break;                          // uniform across the warp
                        const uint64_t row = (uint64_t)(it.row_start + c + j);
                        float av[2];
#pragma unroll
                        for (uint32_t q = 0; q < 2u; q++) {
                            const float g = bf16_bits_to_float(float_to_bf16_bits(__uint_as_float(r0[j + q])));
                            const float u = bf16_bits_to_float(float_to_bf16_bits(__uint_as_float(r1[j + q])));
                            const uint16_t bits =
                                float_to_bf16_bits(activation(g, u, a.activation, a.beta, a.linear_beta));
                            av[q] = in0 ? bf16_bits_to_float(bits) : 0.f;
                            if (a.out != nullptr && in0 && j + q < n_here)
                                a.out[(row + q) * a.out_width + col0] = bits;
                        }
                        const SplitScale s0 = block_scale(av[0]), s1 = block_scale(av[1]);
                        const uint32_t packed = split_pair(av[0] * s0.mult, av[1] * s1.mult);
                        if (in0) {
                            a.act_hi[row * a.w_rows + col0] = (uint8_t)packed;
                            a.act_lo[row * a.w_rows + col0] = (uint8_t)(packed >> 16);
                            if (lane == 0) a.act_sf[row * (a.w_rows / 32u) + col0 / 32u] = (uint8_t)s0.scale_byte;
                            if (j + 1u < n_here) {
                                a.act_hi[(row + 1u) * a.w_rows + col0] = (uint8_t)(packed >> 8);
                                a.act_lo[(row + 1u) * a.w_rows + col0] = (uint8_t)(packed >> 24);
                                if (lane == 0)
                                    a.act_sf[(row + 1u) * (a.w_rows / 32u) + col0 / 32u] = (uint8_t)s1.scale_byte;
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (uint32_t j = 0; j < 32u; j++) {
                        if (j >= n_here) break;
                        const uint64_t row = (uint64_t)(it.row_start + c + j);
                        if (in0) a.out[row * a.out_width + col0] = float_to_bf16_bits(__uint_as_float(r0[j]));
                        if (in1) a.out[row * a.out_width + col1] = float_to_bf16_bits(__uint_as_float(r1[j]));
                    }
                }
            }
            if (!released) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&acc_empty[b0]);
                    if (!small) mbar_arrive(&acc_empty[1]);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0u) atomicExch(&g_gmx_status, 1u);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// bf16 rows -> E4M3 terms + block scales.  Four lanes share a block of 32
// columns (8 each); a warp converts 256 columns per pass.
__global__ void __launch_bounds__(256)
split_rows_kernel(uint8_t *__restrict__ hi, uint8_t *__restrict__ lo, uint8_t *__restrict__ sf,
                  const uint16_t *__restrict__ x, uint32_t rows, uint32_t k) {
    const uint32_t lane = threadIdx.x % kWarp;
    const uint32_t warps = (gridDim.x * blockDim.x) / kWarp;
    const uint32_t blocks = k / 32u;
    for (uint32_t r = (blockIdx.x * blockDim.x + threadIdx.x) / kWarp; r < rows; r += warps) {
        const uint16_t *src = x + (uint64_t)r * k;
        for (uint32_t c = lane * 8u; c < k; c += 256u) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(src + c);
            const uint32_t wv[4] = {raw.x, raw.y, raw.z, raw.w};
            float v[8];
            uint32_t mx = 0;
#pragma unroll
            for (int q = 0; q < 4; q++) {
                v[2 * q] = bf16_lo(wv[q]);
                v[2 * q + 1] = bf16_hi(wv[q]);
                mx = max(mx, max(__float_as_uint(fabsf(v[2 * q])), __float_as_uint(fabsf(v[2 * q + 1]))));
            }
            mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            uint32_t be = min(max((mx >> 23) & 0xffu, 8u), 254u);
            const float mult = __uint_as_float((261u - be) << 23);
            uint32_t h[2], l[2];
#pragma unroll
            for (int q = 0; q < 2; q++) {
                const uint32_t p0 = split_pair(v[4 * q] * mult, v[4 * q + 1] * mult);
                const uint32_t p1 = split_pair(v[4 * q + 2] * mult, v[4 * q + 3] * mult);
                h[q] = (p0 & 0xffffu) | (p1 << 16);
                l[q] = (p0 >> 16) | (p1 & 0xffff0000u);
            }
            *reinterpret_cast<uint2 *>(hi + (uint64_t)r * k + c) = make_uint2(h[0], h[1]);
            *reinterpret_cast<uint2 *>(lo + (uint64_t)r * k + c) = make_uint2(l[0], l[1]);
            if ((lane & 3u) == 0u) sf[(uint64_t)r * blocks + c / 32u] = (uint8_t)(be - 7u);
        }
    }
}

// rows of 16-byte units gathered through an index: dst[r] = src[index[r]]
__global__ void __launch_bounds__(256)
gather_units_kernel(uint4 *__restrict__ dst, const uint4 *__restrict__ src, const uint32_t *__restrict__ index,
                    uint32_t rows, uint32_t units) {
    const uint32_t lane = threadIdx.x % kWarp;
    const uint32_t warps = (gridDim.x * blockDim.x) / kWarp;
    for (uint32_t r = (blockIdx.x * blockDim.x + threadIdx.x) / kWarp; r < rows; r += warps) {
        const uint4 *s = src + (uint64_t)index[r] * units;
        uint4 *d = dst + (uint64_t)r * units;
        for (uint32_t u = lane; u < units; u += kWarp) d[u] = s[u];
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

bool map_2d(CUtensorMap *map, const void *ptr, CUtensorMapDataType type, uint64_t rows, uint64_t inner,
            uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swizzle,
            uint32_t align) {
    auto fn = encode_fn();
    if (!fn || (((uintptr_t)ptr) & (align - 1u)) != 0) return false;
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t es[2] = {1, 1};
    return fn(map, type, 2, const_cast<void *>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Operands {
    const void *a0, *a1;               // packed weights of tile 0 / tile 1
    const void *sfa0, *sfa1;           // their scale tables
    const uint8_t *bhi, *blo, *sfb;    // token terms and scales
};

// Tensor maps depend only on the tables, the term buffers and the shape: the sets of the most
// recent calls are kept (a model alternates between its layers' tables and a few row counts),
// so a steady-state pass encodes nothing; when the table is full it starts over.
struct MapKey {
    int device, mode;
    const void *p[7];
    uint32_t dims[4];
    bool operator<(const MapKey &o) const {
        if (device != o.device) return device < o.device;
        if (mode != o.mode) return mode < o.mode;
        const int c = memcmp(p, o.p, sizeof(p));
        return c != 0 ? c < 0 : memcmp(dims, o.dims, sizeof(dims)) < 0;
    }
};

template <int kE>
bool launch(const Operands &op, const GmxArgs &args, cudaStream_t stream) {
    constexpr size_t kCachedSets = 256;
    static std::mutex map_lock;
    static std::map<MapKey, GmxMaps> cached;
    MapKey key{};
    key.device = current_device();
    key.mode = kE;
    const void *ptrs[7] = {op.a0, op.a1, op.sfa0, op.sfa1, op.bhi, op.blo, op.sfb};
    memcpy(key.p, ptrs, sizeof(ptrs));
    key.dims[0] = args.groups; key.dims[1] = args.w_rows; key.dims[2] = args.k; key.dims[3] = args.rows;
    GmxMaps maps;
    {
        std::lock_guard<std::mutex> guard(map_lock);
        auto it = cached.find(key);
        if (it == cached.end()) {
            const uint64_t w_total = (uint64_t)args.groups * args.w_rows;
            const uint64_t kb = args.k / 32u;
            const auto u4 = CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B;
            const auto u8 = CU_TENSOR_MAP_DATA_TYPE_UINT8;
            const auto sw = CU_TENSOR_MAP_SWIZZLE_128B, none = CU_TENSOR_MAP_SWIZZLE_NONE;
            if (!map_2d(&maps.a0, op.a0, u4, w_total, args.k, args.k / 2u, 128, BM, sw, 32u) ||
                !map_2d(&maps.a1, op.a1, u4, w_total, args.k, args.k / 2u, 128, BM, sw, 32u) ||
                !map_2d(&maps.bhi, op.bhi, u8, args.rows, args.k, args.k, 128, kBBox, sw, 16u) ||
                !map_2d(&maps.blo, op.blo, u8, args.rows, args.k, args.k, 128, kBBox, sw, 16u) ||
                !map_2d(&maps.sfa0, op.sfa0, u8, w_total, kb, kb, 16, BM, none, 16u) ||
                !map_2d(&maps.sfa1, op.sfa1, u8, w_total, kb, kb, 16, BM, none, 16u) ||
                !map_2d(&maps.sfb, op.sfb, u8, args.rows, kb, kb, 16, BN, none, 16u)) {
                return false;
            }
            if (cached.size() >= kCachedSets) cached.clear();
            cached.emplace(key, maps);
        } else {
            maps = it->second;
        }
    }
    if (!set_max_dynamic_smem((const void *)grouped_mx_kernel<kE>, kSmemBytes)) return false;
    grouped_mx_kernel<kE><<<sm_count(), kThreads, kSmemBytes, stream>>>(maps, args);
    return launch_ok();
}

inline size_t up256(size_t v) { return (v + 255u) & ~(size_t)255u; }

struct Scratch {
    uint8_t *t_hi, *t_lo, *t_sf;       // per source row (only with an index)
    uint8_t *x_hi, *x_lo, *x_sf;       // per product row
    uint8_t *a_hi, *a_lo, *a_sf;       // activation, per product row
    uint32_t *counters;                // item counters of the two launches (zeroed per call)
    size_t total;
};

Scratch carve_scratch(const k3_moe_layer_desc *d, uint32_t rows, uint32_t source_rows, void *workspace) {
    const size_t H = d->hidden, I = d->expert_hidden, R = rows, S = source_rows;
    uint8_t *p = (uint8_t *)(((uintptr_t)workspace + 255u) & ~(uintptr_t)255u);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        uint8_t *q = p + off;
        off += up256(bytes);
        return q;
    };
    Scratch s{};
    s.t_hi = take(S * H);
    s.t_lo = take(S * H);
    s.t_sf = take(S * (H / 32u));
    s.x_hi = take(R * H);
    s.x_lo = take(R * H);
    s.x_sf = take(R * (H / 32u));
    s.a_hi = take(R * I);
    s.a_lo = take(R * I);
    s.a_sf = take(R * (I / 32u));
    s.counters = (uint32_t *)take(256);
    s.total = off + 256u;
    return s;
}

}  // namespace

uint32_t k3_grouped_mx_status() {
    uint32_t v = 0xffffffffu;
    if (cudaMemcpyFromSymbol(&v, g_gmx_status, sizeof(v)) != cudaSuccess) (void)cudaGetLastError();
    return v;
}

bool k3_grouped_mx_status_clear() {
    const uint32_t zero = 0u;
    if (cudaMemcpyToSymbol(g_gmx_status, &zero, sizeof(zero)) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return true;
}

size_t k3_grouped_mx_workspace_bytes(const k3_moe_layer_desc *d, uint32_t rows, uint32_t source_rows) {
    return carve_scratch(d, rows, source_rows, nullptr).total;
}

bool k3_grouped_mx_supported(const k3_moe_layer_desc *d, uint32_t rows) {
    return rows >= 32u && d->hidden % 512u == 0 && d->expert_hidden % 512u == 0 &&
           d->local_expert_count >= 1u && d->local_expert_count <= kMaxGroups && encode_fn() != nullptr &&
           ((((uintptr_t)d->w1_packed) | ((uintptr_t)d->w3_packed) | ((uintptr_t)d->w2_packed)) & 31u) == 0 &&
           ((((uintptr_t)d->w1_scales) | ((uintptr_t)d->w3_scales) | ((uintptr_t)d->w2_scales)) & 15u) == 0;
}

// rows_in bf16 [source_rows, H]; product row r reads rows_in[index[r]] (or row r
// when index == nullptr, source_rows == 0).  `act` bf16 [rows, I] is written when
// not null; rows_out bf16 [rows, H].
bool k3_grouped_mx_experts(const k3_moe_layer_desc *d, void *rows_out, void *act, const void *rows_in,
                           const void *index, uint32_t source_rows, const void *offsets, uint32_t rows,
                           void *workspace, cudaStream_t stream) {
    const uint32_t H = d->hidden, I = d->expert_hidden;
    const Scratch s = carve_scratch(d, rows, index ? source_rows : 0u, workspace);
    const uint32_t conv_rows = index ? source_rows : rows;
    const uint32_t cap = (uint32_t)sm_count() * 16u;
    split_rows_kernel<<<std::min<uint32_t>((conv_rows + 7u) / 8u, cap), 256, 0, stream>>>(
        index ? s.t_hi : s.x_hi, index ? s.t_lo : s.x_lo, index ? s.t_sf : s.x_sf, (const uint16_t *)rows_in,
        conv_rows, H);
    if (!launch_ok()) return false;
    if (index) {
        const uint32_t blocks = std::min<uint32_t>((rows + 7u) / 8u, cap);
        gather_units_kernel<<<blocks, 256, 0, stream>>>((uint4 *)s.x_hi, (const uint4 *)s.t_hi,
                                                       (const uint32_t *)index, rows, H / 16u);
        gather_units_kernel<<<blocks, 256, 0, stream>>>((uint4 *)s.x_lo, (const uint4 *)s.t_lo,
                                                       (const uint32_t *)index, rows, H / 16u);
        gather_units_kernel<<<blocks, 256, 0, stream>>>((uint4 *)s.x_sf, (const uint4 *)s.t_sf,
                                                       (const uint32_t *)index, rows, H / 512u);
        if (!launch_ok()) return false;
    }
    if (cudaMemsetAsync(s.counters, 0, 256, stream) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    GmxArgs a{};
    a.offsets = (const uint32_t *)offsets;
    a.item_counter = s.counters;
    a.groups = d->local_expert_count;
    a.rows = rows;
    a.activation = d->activation;
    a.beta = d->beta;
    a.linear_beta = d->linear_beta;
    // gate/up + activation
    a.out = (uint16_t *)act;
    a.act_hi = s.a_hi;
    a.act_lo = s.a_lo;
    a.act_sf = s.a_sf;
    a.w_rows = I;
    a.k = H;
    a.out_width = I;
    a.m_items = (I + BM - 1u) / BM;
    const Operands gu{d->w1_packed, d->w3_packed, d->w1_scales, d->w3_scales, s.x_hi, s.x_lo, s.x_sf};
    if (!launch<kEAct>(gu, a, stream)) return false;
    // down
    a.item_counter = s.counters + 32;
    a.out = (uint16_t *)rows_out;
    a.act_hi = a.act_lo = a.act_sf = nullptr;
    a.w_rows = H;
    a.k = I;
    a.out_width = H;
    a.m_items = (H + 2u * BM - 1u) / (2u * BM);
    const Operands dn{d->w2_packed, d->w2_packed, d->w2_scales, d->w2_scales, s.a_hi, s.a_lo, s.a_sf};
    return launch<kEBf16>(dn, a, stream);
}
