// One-token expert products on the packed block-scaled tensor-core path
// (tcgen05.mma kind::mxf4, 32-element blocks with E8M0 scales), gate/up and down in
// ONE persistent launch.
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
// Work items: G = (rank, 128-row tile) of gate and up over the hidden width, with the
// activation fused; D = (rank, 128-row tile) of down over the expert width.  All G
// items come first in the numbering, then the D items rank by rank.  One CTA per SM
// draws items from a global counter, so the byte load evens out whatever the item mix;
// a D item needs its rank's activation, which the G items' epilogues publish through a
// per-rank arrival counter - only the (small) term loads of a D item wait for it, the
// weight stream never does.  Warps:
//   0       weight producer: draws items, streams 16 KB weight tiles through a TMA ring
//   1, 11   MMA issuers: 4 MMAs of K=64 per stage, even / odd stages, own accumulators
//   2-5     scale writers: weight scales shared memory -> tensor memory, term scales too
//   6-9     epilogue: tcgen05.ld of the term columns, sum, bf16; G: activation, its
//           E2M1 terms, arrival; D: output row (and, where the layer's tail has no
//           kernel of its own, its arrival for the tail)
//   10      weight-scale producer (TMA, 512 K per box)
//   12      term producer: the token's terms once (they serve every G item), then per D
//           item the rank's activation terms and scales, after its arrival count is full
// The kernel is launched behind the router rows' kernel with programmatic serialization.
// In its prologue every CTA waits for that kernel (for its count of finished blocks when a
// longer-running grid sits in front of it), routes the token itself (k3_route_block.cuh)
// and draws its first item under the routing.  Weight and scale loads carry the
// evict-first L2 policy.  Every wait is bounded (see k3_tc_ptx.cuh).
#include "k3_decode_tail.cuh"
#include "k3_e2m1_terms.cuh"
#include "k3_grouped.h"
#include "k3_route_block.cuh"
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

constexpr uint32_t kStages = 8;             // TMA ring of weight tiles
constexpr uint32_t kKStage = 256;           // K elements per stage (128 packed bytes per row)
constexpr uint32_t kSfBatches = 6;          // scale ring in tensor memory: batches of 2 stages (512 K)
constexpr uint32_t kSfSlots = 4;            // weight-scale ring in shared memory (one batch per slot)
constexpr uint32_t kSfaBytes = 128 * 16;    // 128 rows x 16 scale bytes (512 K)
constexpr uint32_t kATile = 128 * 128;     // bytes in shared memory = bytes the TMA brings
constexpr uint32_t kBAtom = kTerms * 128;   // one stage of term rows: one 8-row swizzle atom
constexpr uint32_t kSfbBatch = kTerms * 16; // term scales of one batch: 8 rows x 16 bytes
constexpr uint32_t kThreads = 416;          // 13 warps, see the role list above
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccCol = 0;            // 2 buffers x 2 issuers x 2 phases x 16 columns
constexpr uint32_t kSfaCol = 128;          // kSfBatches x 16 columns
constexpr uint32_t kSfbCol = 128 + 16 * kSfBatches;  // kSfBatches x 16 columns
constexpr uint32_t kBarrierBytes = 1024;     // barriers, mailbox, the token's ids and weights
constexpr uint32_t kItemSlots = 4;          // mailbox of drawn items, weight producer -> other roles
constexpr uint32_t kItemReaders = 12;       // 2 issuers, 4 writers, 4 epilogue warps, scale and term producers
constexpr uint32_t kNoItem = 0xffffffffu;
constexpr uint32_t kControlWords = 64;      // [0] item counter, [16 + rank] arrivals of the rank's G epilogues
static_assert(kTerms == 8, "one swizzle atom of term rows per stage");

__device__ uint32_t g_mx_status = 0;

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
    uint32_t *ids;              // expert id per rank: read, or written when the kernel routes
    float *weights;             // route weights, written when the kernel routes
    const float *route_words;   // scores [1024] and choices [1024] of the router rows, or null
    uint32_t experts;
    float route_scale;
    uint16_t *act;              // [ranks, I] bf16 activation (also kept as bf16 for callers)
    uint16_t *rows_out;         // [ranks, H] bf16 expert rows
    uint32_t ranks, first_local, local_count;
    uint32_t hidden, expert_hidden;
    int activation;
    float beta, linear_beta;
    uint8_t *act_terms;         // E2M1 terms of the activation [ranks * kTerms, I / 2]
    uint8_t *act_sf;            // and their block scales [ranks * kTerms, I / 32]
    uint32_t *control;          // kControlWords words, zero at launch
    const uint32_t *front_done; // blocks of the front kernel that have finished, or null
    uint32_t front_blocks;      // its grid size
    DecodeTail tail;            // the layer's tail, run by the D epilogues (tail.out null: none)
};

struct MxMaps {
    CUtensorMap w1, w3, w2;            // packed E2M1 weights as bytes [rows, K/2]
    CUtensorMap s1, s3, s2;            // weight block scales [rows, K/32]
    CUtensorMap x_terms, x_sf;         // the token: [kTerms, H/2], [kTerms, H/32]
    CUtensorMap a_terms, a_sf;         // the activations: [ranks*kTerms, I/2], [ranks*kTerms, I/32]
};

// Shared-memory layout, derived the same way on the host (bytes) and in the kernel.
struct MxSmem {
    uint32_t ring, bg, bd, zero, sfb_g, sfb_d, sfa, bars, total;
};
__host__ __device__ inline MxSmem mx_smem_layout(uint32_t steps_g, uint32_t steps_d) {
    MxSmem m;
    uint32_t off = 0;
    m.ring = off;  off += kStages * kATile;
    m.bg = off;    off += steps_g * kBAtom;                 // the token's terms, every stage resident
    m.bd = off;    off += 2u * steps_d * kBAtom;            // two D items' activation terms
    m.zero = off;  off += kBAtom;                           // rows 8..15 of every N = 16 operand
    m.sfb_g = off; off += (steps_g / 2u) * kSfbBatch;
    m.sfb_d = off; off += 2u * (steps_d / 2u) * kSfbBatch;
    m.sfa = off;   off += kSfSlots * kSfaBytes;
    m.bars = off;  off += kBarrierBytes;
    m.total = off + 1024u;                                  // alignment slack
    return m;
}

// K-major 128-byte-swizzled operand of N = 16 rows whose second 8-row atom lives at
// `second` (any 1024-byte aligned address above `first`): the stride between the atoms
// is a field of the descriptor.
K3_DEVINL uint64_t make_desc_sw128_split(uint32_t first, uint32_t second) {
    uint64_t d = 0;
    d |= (uint64_t)((first & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(((second - first) & 0x3FFFFu) >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}


K3_DEVINL void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

K3_DEVINL uint32_t ld_acquire(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// (72 registers: a 256-thread block of the shared expert's kernels, which run beside this
// one on another stream, still fits in the register file of the SM)
__global__ void __maxnreg__(64)
decode_experts_kernel(const __grid_constant__ MxMaps maps, MxArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t steps_g = a.hidden / kKStage, steps_d = a.expert_hidden / kKStage;
    const MxSmem lay = mx_smem_layout(steps_g, steps_d);
    uint64_t *bars = reinterpret_cast<uint64_t *>(base + lay.bars);
    uint64_t *full = bars, *empty = bars + kStages;
    uint64_t *sf_full = empty + kStages;               // [kSfBatches] scales in tensor memory
    uint64_t *sf_empty = sf_full + kSfBatches;
    uint64_t *sfs_full = sf_empty + kSfBatches;        // [kSfSlots] weight scales in shared memory
    uint64_t *sfs_empty = sfs_full + kSfSlots;
    uint64_t *acc_full = sfs_empty + kSfSlots, *acc_empty = acc_full + 2;
    uint64_t *item_full = acc_empty + 2, *item_empty = item_full + kItemSlots;
    uint64_t *bg_full = item_empty + kItemSlots;       // the token's terms and scales have landed
    uint64_t *bd_full = bg_full + 1, *bd_empty = bd_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bd_empty + 2);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    volatile uint32_t *item_box = tmem_slot + 2;       // [kItemSlots]
    uint32_t *ids_s = tmem_slot + 8;                   // [32]
    float *weights_s = reinterpret_cast<float *>(tmem_slot + 40);   // [32]
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t tiles_g = a.expert_hidden / 128u, tiles_d = a.hidden / 128u;
    const uint32_t items_g = a.ranks * tiles_g, items = items_g + a.ranks * tiles_d;

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
            mbar_init(&bd_full[b], 1);
            mbar_init(&bd_empty[b], 6);               // two issuers, four scale writers
        }
        for (uint32_t b = 0; b < kItemSlots; b++) {
            mbar_init(&item_full[b], 1);
            mbar_init(&item_empty[b], kItemReaders);
        }
        mbar_init(bg_full, 1);
        fence_barrier_init();
    }
    // the atom of zeros that stands for rows 8..15 of every N = 16 operand
    for (uint32_t i = threadIdx.x; i < kBAtom / 16u; i += blockDim.x)
        reinterpret_cast<uint4 *>(base + lay.zero)[i] = make_uint4(0u, 0u, 0u, 0u);
    fence_proxy_async();
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (threadIdx.x == 0) {
        prefetch_tensormap(&maps.w1);
        prefetch_tensormap(&maps.w3);
        prefetch_tensormap(&maps.w2);
    }
    // a kernel queued behind this one with programmatic serialization (the layer's tail) may
    // take its places now; it waits for this grid to finish before it reads anything
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Everything above needed nothing from the front kernel; what follows does (scores,
    // token terms, cleared control words).
    if (a.front_done == nullptr) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
    } else {
        // Waiting for the grid in front would also wait for the grid in front of that one
        // (the shared expert's, which runs until the layer's end).  The front kernel's blocks
        // are all resident by the time this grid was allowed to start, so their count of
        // finished blocks is waited for instead.
        if (threadIdx.x == 0) {
            const unsigned long long t0 = global_timer_ns();
            uint32_t spins = 0;
            while (ld_acquire(a.front_done) < a.front_blocks) {
                if ((++spins & 63u) == 0u && global_timer_ns() - t0 > kWaitLimitNs) {
                    *abort_flag = 1u;
                    break;
                }
            }
            fence_proxy_async_global();          // the token's terms are read by bulk copies
        }
        __syncthreads();
    }
    // the first work item is drawn now, so that the counter's round trip runs under the routing
    uint32_t first_item = 0u;
    if (threadIdx.x == 0) first_item = atomicAdd(a.control, 1u);
    if (a.route_words != nullptr) {
        // every CTA routes the token itself (the ring is still free: it serves as scratch)
        RouteScratch &rs = *reinterpret_cast<RouteScratch *>(base + lay.ring);
        route_topk_block(rs, ids_s, weights_s, a.route_words, a.experts, a.ranks, a.route_scale);
        // the same values from every CTA; whoever reads them later is ordered behind at least
        // one of these stores (the kernel's end, or the fence in front of a tail arrival of
        // the CTA whose epilogue completes the count)
        if (threadIdx.x < a.ranks) {
            a.ids[threadIdx.x] = ids_s[threadIdx.x];
            a.weights[threadIdx.x] = weights_s[threadIdx.x];
        }
    } else if (threadIdx.x < a.ranks) {
        ids_s[threadIdx.x] = a.ids[threadIdx.x];
    }
    __syncthreads();

    struct Item {
        bool valid, down, local;
        uint32_t rank, tile, expert;
    };
    auto decode = [&](uint32_t w) {
        Item it;
        it.valid = w != kNoItem;
        it.down = it.valid && w >= items_g;
        const uint32_t j = it.down ? w - items_g : w;
        const uint32_t tiles = it.down ? tiles_d : tiles_g;
        it.rank = it.valid ? j / tiles : 0u;
        it.tile = it.valid ? j % tiles : 0u;
        const uint32_t id = it.valid ? ids_s[it.rank] : 0u;
        it.local = it.valid && id >= a.first_local && id < a.first_local + a.local_count;
        it.expert = id - a.first_local;
        return it;
    };
    // Reader side of the item mailbox: the n-th call returns the n-th item this CTA drew.
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
        return __shfl_sync(0xffffffffu, w, 0);
    };

    if (warp == 0) {
        // ===================================== weight producer; draws the items
        uint32_t s = 0, ph = 0, seq = 0;
        bool ok = true;
        uint32_t w = 0;
        const uint64_t stream_once = l2_policy_evict_first();      // every weight byte is read once
        if (lane == 0) w = first_item;
        while (ok) {
            const uint32_t slot = seq % kItemSlots, parity = (seq / kItemSlots) & 1u;
            seq++;
            uint32_t cur = kNoItem;
            if (lane == 0) {
                if (mbar_wait(&item_empty[slot], parity ^ 1u, abort_flag)) {
                    cur = w < items ? w : kNoItem;
                    item_box[slot] = cur;
                    mbar_arrive(&item_full[slot]);
                    if (cur != kNoItem) w = atomicAdd(a.control, 1u);   // travels while this item streams
                }
            }
            cur = __shfl_sync(0xffffffffu, cur, 0);
            if (cur == kNoItem) break;
            const Item it = decode(cur);
            if (!it.local) continue;
            if (lane == 0) {
                const uint32_t w_rows = it.down ? a.hidden : a.expert_hidden;
                const int32_t y = (int32_t)(it.expert * w_rows + it.tile * 128u);
                const uint32_t phases = it.down ? 1u : 2u, steps = it.down ? steps_d : steps_g;
                for (uint32_t p = 0; ok && p < phases; p++) {
                    const void *map = it.down ? (const void *)&maps.w2
                                              : (p == 0 ? (const void *)&maps.w1 : (const void *)&maps.w3);
                    for (uint32_t st = 0; st < steps; st++) {
                        if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                        mbar_arrive_expect_tx(&full[s], kATile);
                        tma_load_2d_hint(base + lay.ring + s * kATile, map, &full[s], (int32_t)(st * 128u), y, stream_once);
                        if (++s == kStages) { s = 0; ph ^= 1u; }
                    }
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1u : 0u, 0) != 0u;
        }
    } else if (warp == 12) {
        // ===================================== term producer
        bool ok = true;
        if (lane == 0) {
            prefetch_tensormap(&maps.x_terms);
            prefetch_tensormap(&maps.x_sf);
            prefetch_tensormap(&maps.a_terms);
            prefetch_tensormap(&maps.a_sf);
            // the token's terms serve every G item: all stages resident
            mbar_arrive_expect_tx(bg_full, steps_g * kBAtom + (steps_g / 2u) * kSfbBatch);
            for (uint32_t st = 0; st < steps_g; st++)
                tma_load_2d(base + lay.bg + st * kBAtom, &maps.x_terms, bg_full, (int32_t)(st * 128u), 0);
            for (uint32_t bt = 0; bt < steps_g / 2u; bt++)
                tma_load_2d(base + lay.sfb_g + bt * kSfbBatch, &maps.x_sf, bg_full, (int32_t)(bt * 16u), 0);
        }
        uint32_t dcount = 0;
        for (uint32_t w = next_item(); ok && w != kNoItem; w = next_item()) {
            const Item it = decode(w);
            if (!it.local || !it.down) continue;
            const uint32_t buf = dcount & 1u, par = (dcount >> 1) & 1u;
            dcount++;
            if (lane == 0) {
                // the rank's activation is complete when all its G epilogue warps have arrived
                const uint32_t need = 4u * tiles_g;
                const uint32_t *word = a.control + 16u + it.rank;
                const unsigned long long t0 = global_timer_ns();
                uint32_t spins = 0;
                while (ld_acquire(word) < need) {
                    if ((++spins & 63u) == 0u && (*abort_flag != 0u || global_timer_ns() - t0 > kWaitLimitNs)) {
                        *abort_flag = 1u;
                        ok = false;
                        break;
                    }
                }
                fence_proxy_async_global();      // what other SMs stored is now ordered before this TMA read
                if (ok && !mbar_wait(&bd_empty[buf], par ^ 1u, abort_flag)) ok = false;
                if (ok) {
                    mbar_arrive_expect_tx(&bd_full[buf], steps_d * kBAtom + (steps_d / 2u) * kSfbBatch);
                    const int32_t y = (int32_t)(kTerms * it.rank);
                    for (uint32_t st = 0; st < steps_d; st++)
                        tma_load_2d(base + lay.bd + (buf * steps_d + st) * kBAtom, &maps.a_terms, &bd_full[buf],
                                    (int32_t)(st * 128u), y);
                    for (uint32_t bt = 0; bt < steps_d / 2u; bt++)
                        tma_load_2d(base + lay.sfb_d + (buf * (steps_d / 2u) + bt) * kSfbBatch, &maps.a_sf,
                                    &bd_full[buf], (int32_t)(bt * 16u), y);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1u : 0u, 0) != 0u;
        }
    } else if (warp == 10) {
        // ===================================== weight-scale producer: 512 K per box
        uint32_t s = 0, ph = 0;
        bool ok = true;
        const uint64_t stream_once = l2_policy_evict_first();
        if (lane == 0) {
            prefetch_tensormap(&maps.s1);
            prefetch_tensormap(&maps.s3);
            prefetch_tensormap(&maps.s2);
        }
        for (uint32_t w = next_item(); ok && w != kNoItem; w = next_item()) {
            const Item it = decode(w);
            if (!it.local) continue;
            if (lane == 0) {
                const uint32_t w_rows = it.down ? a.hidden : a.expert_hidden;
                const int32_t y = (int32_t)(it.expert * w_rows + it.tile * 128u);
                const uint32_t phases = it.down ? 1u : 2u, steps = it.down ? steps_d : steps_g;
                for (uint32_t p = 0; ok && p < phases; p++) {
                    const void *map = it.down ? (const void *)&maps.s2
                                              : (p == 0 ? (const void *)&maps.s1 : (const void *)&maps.s3);
                    for (uint32_t bt = 0; bt < steps / 2u; bt++) {
                        if (!mbar_wait(&sfs_empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                        mbar_arrive_expect_tx(&sfs_full[s], kSfaBytes);
                        tma_load_2d_hint(base + lay.sfa + s * kSfaBytes, map, &sfs_full[s], (int32_t)(bt * 16u), y,
                                         stream_once);
                        if (++s == kSfSlots) { s = 0; ph ^= 1u; }
                    }
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1u : 0u, 0) != 0u;
        }
    } else if (warp == 1 || warp == 11) {
        // ===================================== MMA issuers
        // The issue loop of one thread, not the tensor pipe, bounds the rate of these small
        // MMAs, so warp 1 takes the even stages and warp 11 the odd ones, each into its own
        // accumulator columns (summed in the epilogue).  A scale batch covers two stages,
        // one per issuer.
        const uint32_t q = warp == 1 ? 0u : 1u;
        uint32_t s = q, ph = 0, buf = 0, pacc = 0, sb = 0, sph = 0, dcount = 0;
        bool ok = true;
        for (uint32_t w = next_item(); ok && w != kNoItem; w = next_item()) {
            const Item it = decode(w);
            if (!it.local) continue;
            uint32_t dbuf = 0;
            if (it.down) {
                dbuf = dcount & 1u;
                dcount++;
            }
            if (lane == 0) {
                const uint32_t dpar = ((dcount - 1u) >> 1) & 1u;
                const uint32_t phases = it.down ? 1u : 2u, steps = it.down ? steps_d : steps_g;
                const uint32_t b_base = smem_u32(base + (it.down ? lay.bd + dbuf * steps_d * kBAtom : lay.bg));
                const uint32_t zero_atom = smem_u32(base + lay.zero);
                if (!mbar_wait(&acc_empty[buf], pacc ^ 1u, abort_flag) ||
                    !(it.down ? mbar_wait(&bd_full[dbuf], dpar, abort_flag) : mbar_wait(bg_full, 0u, abort_flag))) {
                    ok = false;
                }
                tc_fence_after();
                for (uint32_t p = 0; ok && p < phases; p++) {
                    const uint32_t d = tmem + kAccCol + buf * 64u + q * 32u + p * 16u;
                    for (uint32_t st = q; st < steps; st += 2u) {
                        if (!mbar_wait(&full[s], ph, abort_flag) || !mbar_wait(&sf_full[sb], sph, abort_flag)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint64_t da = make_desc_sw128(smem_u32(base + lay.ring + s * kATile));
                        const uint64_t db = make_desc_sw128_split(b_base + st * kBAtom, zero_atom);
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
                if (ok) {
                    mma_commit(&acc_full[buf]);
                    if (it.down) mma_commit(&bd_empty[dbuf]);      // the MMAs have read the activation terms
                }
            }
            if (++buf == 2u) { buf = 0; pacc ^= 1u; }
            ok = __shfl_sync(0xffffffffu, ok ? 1u : 0u, 0) != 0u;
        }
    } else if (warp < 6) {
        // ===================================== scale writers: shared memory -> tensor memory,
        // warp w fills lane quadrant w % 4
        const uint32_t quad = warp & 3u;
        const uint32_t lane_base = (32u * quad) << 16;
        uint32_t sb = 0, sph = 0, ss = 0, ssph = 0, dcount = 0;
        bool ok = true;
        for (uint32_t w = next_item(); ok && w != kNoItem; w = next_item()) {
            const Item it = decode(w);
            if (!it.local) continue;
            uint32_t dbuf = 0, dpar = 0;
            if (it.down) {
                dbuf = dcount & 1u;
                dpar = (dcount >> 1) & 1u;
                dcount++;
            }
            if (!(it.down ? mbar_wait(&bd_full[dbuf], dpar, abort_flag) : mbar_wait(bg_full, 0u, abort_flag))) break;
            const uint32_t phases = it.down ? 1u : 2u, steps = it.down ? steps_d : steps_g;
            const unsigned char *sfb =
                base + (it.down ? lay.sfb_d + dbuf * (steps_d / 2u) * kSfbBatch : lay.sfb_g);
            for (uint32_t p = 0; ok && p < phases; p++) {
                for (uint32_t bt = 0; bt < steps / 2u; bt++) {
                    if (!mbar_wait(&sfs_full[ss], ssph, abort_flag)) { ok = false; break; }
                    const unsigned char *src = base + lay.sfa + ss * kSfaBytes;
                    uint4 cur[4];
#pragma unroll
                    for (uint32_t c = 0; c < 4u; c++)
                        cur[c] = *reinterpret_cast<const uint4 *>(src + (32u * c + lane) * 16u);
                    // scale rows of the N operand sit in lanes 0..15 of the first column of a group:
                    // term rows 0..7 (lanes 8.. repeat them: those operand rows are zero)
                    const uint4 curb =
                        *reinterpret_cast<const uint4 *>(sfb + bt * kSfbBatch + (lane & (kTerms - 1u)) * 16u);
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
            if (ok && it.down) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&bd_empty[dbuf]);       // this warp has read the item's term scales
            }
        }
    } else if (warp < 10) {
        // ===================================== epilogue: warp w reads lane quadrant w % 4
        const uint32_t quad = warp & 3u;
        const uint32_t m = 32u * quad + lane;
        uint32_t buf = 0, pacc = 0;
        for (uint32_t w = next_item(); w != kNoItem; w = next_item()) {
            const Item it = decode(w);
            if (!it.local) continue;
            if (!mbar_wait(&acc_full[buf], pacc, abort_flag)) break;
            tc_fence_after();
            const uint32_t t0 = tmem + ((32u * quad) << 16) + kAccCol + buf * 64u;
            uint32_t e0[8], o0[8], e1[8], o1[8];
            tmem_ld_32x8(t0, e0);                           // even stages
            tmem_ld_32x8(t0 + 32u, o0);                     // odd stages
            if (!it.down) {
                tmem_ld_32x8(t0 + 16u, e1);
                tmem_ld_32x8(t0 + 48u, o1);
            }
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            if (++buf == 2u) { buf = 0; pacc ^= 1u; }
            const float v0 = sum_terms(e0) + sum_terms(o0);
            if (!it.down) {
                const float v1 = sum_terms(e1) + sum_terms(o1);
                const float g = bf16_bits_to_float(float_to_bf16_bits(v0));
                const float u = bf16_bits_to_float(float_to_bf16_bits(v1));
                const uint16_t act_bits = float_to_bf16_bits(activation(g, u, a.activation, a.beta, a.linear_beta));
                const uint32_t I = a.expert_hidden;
                a.act[(uint64_t)it.rank * I + it.tile * 128u + m] = act_bits;
                uint32_t code[kTerms], sbyte[kTerms];
                split_block_e2m1(bf16_bits_to_float(act_bits), code, sbyte);
                store_block_e2m1(a.act_terms + (uint64_t)it.rank * kTerms * (I / 2u),
                                 a.act_sf + (uint64_t)it.rank * kTerms * (I / 32u), I / 2u, I / 32u,
                                 it.tile * 4u + quad, code, sbyte, lane);
                // publish: these 32 activation elements are in memory for every SM's TMA reads
                fence_proxy_async_global();
                __threadfence();
                __syncwarp();
                if (lane == 0) atomicAdd(a.control + 16u + it.rank, 1u);
            } else {
                a.rows_out[(uint64_t)it.rank * a.hidden + it.tile * 128u + m] = float_to_bf16_bits(v0);
                if (a.tail.out != nullptr && !tail_arrive(a.tail, it.tile * 4u + quad, lane)) *abort_flag = 1u;
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
           (size_t)d->hidden / 32u * 4u + 2u * 1024u * 4u + 2u * kControlWords * 4u + 7u * 256u;
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

void *k3_decode_mx_control_words(const k3_moe_layer_desc *d, void *scratch) {
    uint8_t *route = (uint8_t *)k3_decode_mx_route_words(d, scratch);
    return (void *)(((uintptr_t)(route + 2u * 1024u * 4u) + 255u) & ~(uintptr_t)255u);
}

void *k3_decode_mx_front_done_word(const k3_moe_layer_desc *d, void *scratch) {
    return (uint32_t *)k3_decode_mx_control_words(d, scratch) + kControlWords;
}

// Routed experts of one token: act [top_k, I] and rows_out [top_k, hidden] in rank
// order (ids on the device) from the token's E2M1 terms in `scratch`.
bool k3_decode_mx_experts(const k3_moe_layer_desc *d, void *ids, void *weights, const void *route_words,
                          void *act, void *rows_out, void *scratch, void *between, const k3_decode_tail *tail,
                          uint32_t front_blocks, cudaStream_t stream) {
    if (route_words != nullptr && (d->expert_count > 1024u || !weights)) return false;
    const uint32_t H = d->hidden, I = d->expert_hidden, k = d->top_k;
    auto align = [](uint8_t *p) { return (uint8_t *)(((uintptr_t)p + 255u) & ~(uintptr_t)255u); };
    uint8_t *x_terms = nullptr, *x_sf = nullptr;
    k3_decode_mx_vector_scratch(d, scratch, (void **)&x_terms, (void **)&x_sf);
    uint8_t *a_terms = align(x_sf + (size_t)kTerms * H / 32u);
    uint8_t *a_sf = align(a_terms + (size_t)kTerms * k * I / 2u);
    const MxSmem lay = mx_smem_layout(H / kKStage, I / kKStage);
    if (lay.total > 227u * 1024u) return false;
    if (!set_max_dynamic_smem((const void *)decode_experts_kernel, lay.total)) return false;
    // Tensor maps depend only on the tables, the scratch block and the shape.  Encoding
    // ten maps costs more host time than the launch, so the sets of the most recent
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
    constexpr size_t kCachedLayers = 256;
    static std::mutex map_lock;
    static std::map<MapKey, MxMaps> cached;
    MapKey key{};
    key.device = current_device();
    const void *ptrs[7] = {d->w1_packed, d->w3_packed, d->w2_packed, d->w1_scales, d->w3_scales, d->w2_scales, scratch};
    memcpy(key.p, ptrs, sizeof(ptrs));
    key.dims[0] = H; key.dims[1] = I; key.dims[2] = k; key.dims[3] = d->local_expert_count;
    MxMaps maps;
    {
        std::lock_guard<std::mutex> guard(map_lock);
        auto it = cached.find(key);
        if (it == cached.end()) {
            const uint64_t total = (uint64_t)d->local_expert_count;
            if (!map_bytes(&maps.w1, d->w1_packed, total * I, H / 2u, 128) ||
                !map_bytes(&maps.w3, d->w3_packed, total * I, H / 2u, 128) ||
                !map_bytes(&maps.w2, d->w2_packed, total * H, I / 2u, 128) ||
                !map_sf(&maps.s1, d->w1_scales, total * I, H, 128) || !map_sf(&maps.s3, d->w3_scales, total * I, H, 128) ||
                !map_sf(&maps.s2, d->w2_scales, total * H, I, 128) ||
                !map_bytes(&maps.x_terms, x_terms, kTerms, H / 2u, kTerms) || !map_sf(&maps.x_sf, x_sf, kTerms, H, kTerms) ||
                !map_bytes(&maps.a_terms, a_terms, (uint64_t)kTerms * k, I / 2u, kTerms) ||
                !map_sf(&maps.a_sf, a_sf, (uint64_t)kTerms * k, I, kTerms)) {
                return false;
            }
            if (cached.size() >= kCachedLayers) cached.clear();
            cached.emplace(key, maps);
        } else {
            maps = it->second;
        }
    }
    MxArgs a{};
    a.ids = (uint32_t *)ids;
    a.weights = (float *)weights;
    a.route_words = (const float *)route_words;
    a.experts = d->expert_count;
    a.route_scale = d->route_scale;
    a.act = (uint16_t *)act;
    a.rows_out = (uint16_t *)rows_out;
    a.ranks = k;
    a.first_local = d->local_expert_first;
    a.local_count = d->local_expert_count;
    a.hidden = H;
    a.expert_hidden = I;
    a.activation = d->activation;
    a.beta = d->beta;
    a.linear_beta = d->linear_beta;
    a.act_terms = a_terms;
    a.act_sf = a_sf;
    a.control = (uint32_t *)k3_decode_mx_control_words(d, scratch);
    a.front_done = front_blocks != 0u ? (const uint32_t *)k3_decode_mx_front_done_word(d, scratch) : nullptr;
    a.front_blocks = front_blocks;
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
    cudaLaunchConfig_t config{};
    config.gridDim = dim3((unsigned)sm_count());
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = lay.total;
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    // behind the front kernel: blocks may take their places (and set up barriers and tensor
    // memory) while the front grid drains; they wait for it before they read its results
    config.numAttrs = route_words != nullptr ? 1u : 0u;
    if (cudaLaunchKernelEx(&config, decode_experts_kernel, maps, a) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return !between || cudaEventRecord((cudaEvent_t)between, stream) == cudaSuccess;
}
