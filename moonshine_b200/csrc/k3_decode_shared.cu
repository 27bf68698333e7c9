// Shared expert of the one-token layer as one persistent kernel on a few SMs.
//
// The shared expert (Q8 gate / up / down tables, reference: the static projections of
// decode_routed_layer, k3_engine.cu:1668-1689) depends only on the token, so it can run
// beside everything that depends on the routing.  Next to the routed experts' TMA stream
// a kernel that fetches its weights with ordinary loads is starved by the memory system
// (it has a tenth of the bytes in flight), so this one streams too: a producer thread
// brings 16 KB stages into a shared-memory ring with tiled bulk copies, two groups of eight
// consumer warps take the int8 values from shared memory and run the same tensor-core Q8
// arithmetic as the row kernels (k3_gemv.cuh: int8 -> f16 exactly, block-diagonal vector
// operand, one fp32 FMA per scale group).  A few CTAs, one per SM, hold their SMs from
// the start of the layer until the shared expert is done; the expert kernel's CTAs for
// those SMs start late and draw what is left of the item list.
//
// Work split: a task is 16 rows over the whole K extent; CTA c takes tasks c, c + n, ...
// of the gate / up phase, then (after every CTA's gate / up rows are in memory, counted in
// a word of the library) of the down phase.  Inside a task warp w owns the 128-column
// steps [w * per, (w + 1) * per), per = K / 1024, summed in order; the eight partial sums
// are added in warp order - the arithmetic of decode_shared_gateup_kernel /
// decode_shared_down_kernel, so either path gives the same bits.  Stage j of a task holds
// step j of every warp: one 4-D box {128 bytes, 16 rows, 1 step, 8 warps}, 128-byte
// swizzle, which puts each warp's 16 x 128 tile in 2 KB of its own.
#include "k3_gemv.cuh"
#include "k3_grouped.h"
#include "k3_moe_ops.h"
#include "k3_tc_ptx.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

using namespace k3;
using namespace k3::tc;

namespace {

constexpr uint32_t kStages = 8;
constexpr uint32_t kStageBytes = 16u * 1024u;
constexpr uint32_t kWarps = 8;                       // consumer warps of a group (the K split of a task)
constexpr uint32_t kGroups = 2;                      // groups work on different tasks at the same time
constexpr uint32_t kConsumers = kGroups * kWarps * kWarp;
constexpr uint32_t kProducerWarp = kGroups * kWarps;
constexpr uint32_t kThreads = kConsumers + kWarp + kGroups * kWarp;    // + producer + one finisher per group
constexpr uint32_t kScaleSlots = 2;                  // per group
constexpr uint32_t kScaleSlotBytes = 16u * 1024u;    // 16 rows x at most 1024 bytes of scales
constexpr uint32_t kSyncSlots = 64;

// [slot][0] gate / up tasks in memory, [slot][1] CTAs that have left; zero between calls
__device__ uint32_t g_shared_sync[kSyncSlots][2];
__device__ uint32_t g_shared_status = 0;

struct RingArgs {
    const uint16_t *x;                  // [H] bf16
    uint16_t *sh_gate, *sh_up, *sh_out; // [S], [S], [H] bf16
    uint32_t H, S;
    uint32_t scale_bytes;               // 2 (f16) or 4 (f32)
    uint32_t block_shift;               // log2 of the columns per scale
    int activation;
    float beta, linear_beta;
    uint32_t *sync;                     // two words of g_shared_sync
    uint32_t *zero_word;                // word this kernel clears before its dependents may start, or null
};

struct RingMaps {
    CUtensorMap gate, up, down;         // int8 [rows, K] as {128, rows, K / 1024, 8}
    CUtensorMap gate_s, up_s, down_s;   // scales [rows, K / block] as 32-bit words
};

K3_DEVINL void tma_load_4d(void *dst, const void *map, uint64_t *bar, int32_t c0, int32_t c1, int32_t c2,
                           int32_t c3, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%3, %4, %5, %6}], [%2], %7;" ::"r"(smem_u32(dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
        : "memory");
}

K3_DEVINL void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }

// Roles: warps 0-7 and 8-15 are two consumer groups, warp 16 (one lane) the producer,
// warps 17 and 18 the groups' finishers.  The CTA's tasks of a phase are c, c + n, ...;
// group q takes every second one starting with the q-th, and the producer interleaves the
// stages of the two tasks of a pair, so both groups always have stages in the ring.  A
// finisher adds the eight partial sums of a finished task and stores the 16 results, off
// the consumers' path.  The layer's tail reads sh_out after this grid has finished (it is
// a kernel of its own that waits for every grid in front of it).
__global__ void __launch_bounds__(kThreads, 1)
decode_shared_ring_kernel(const __grid_constant__ RingMaps maps, RingArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char *ring = base;                                        // kStages x 16 KB
    unsigned char *scale_slot = ring + kStages * kStageBytes;          // kGroups x kScaleSlots x 16 KB
    __half *vec = reinterpret_cast<__half *>(scale_slot + kGroups * kScaleSlots * kScaleSlotBytes);   // [max(H, S)] f16
    __shared__ uint64_t full[kStages], empty[kStages];
    __shared__ uint64_t sc_full[kGroups][kScaleSlots], sc_empty[kGroups][kScaleSlots];
    __shared__ uint64_t fin_full[kGroups][2], fin_empty[kGroups][2];
    __shared__ float part[kGroups][2][kWarps][16];
    __shared__ float inv_scale_s[2], warp_max_s[kGroups * kWarps];
    __shared__ uint32_t abort_word;
    volatile uint32_t *abort_flag = &abort_word;
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t H = a.H, S = a.S, n = gridDim.x;
    const uint32_t tasks_gu = 2u * S / 16u, tasks_dn = H / 16u;
    const uint32_t per_gu = H / 1024u, per_dn = S / 1024u;

    if (threadIdx.x == 0) {
        abort_word = 0u;
        for (uint32_t s = 0; s < kStages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kWarps);
        }
        for (uint32_t q = 0; q < kGroups; q++) {
            for (uint32_t s = 0; s < kScaleSlots; s++) {
                mbar_init(&sc_full[q][s], 1);
                mbar_init(&sc_empty[q][s], kWarps);
            }
            for (uint32_t b = 0; b < 2u; b++) {
                mbar_init(&fin_full[q][b], kWarps);
                mbar_init(&fin_empty[q][b], 1);
            }
        }
        fence_barrier_init();
        if (blockIdx.x == 0 && a.zero_word != nullptr) {
            *a.zero_word = 0u;
            __threadfence();
        }
    }
    __syncthreads();
    // The kernels queued behind this one with programmatic serialization read none of its
    // results before the layer's end (they never wait for this grid): they may start now.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // number of this CTA's tasks in a phase
    auto my_tasks = [&](uint32_t tasks) { return blockIdx.x < tasks ? (tasks - 1u - blockIdx.x) / n + 1u : 0u; };

    if (warp == kProducerWarp) {
        // ===================================================== producer
        if (lane == 0) {
            prefetch_tensormap(&maps.gate);
            prefetch_tensormap(&maps.up);
            prefetch_tensormap(&maps.down);
            prefetch_tensormap(&maps.gate_s);
            prefetch_tensormap(&maps.up_s);
            prefetch_tensormap(&maps.down_s);
            uint32_t s = 0, ph = 0, sc[kGroups] = {0u, 0u}, sc_ph[kGroups] = {0u, 0u};
            bool ok = true;
            const uint64_t stream_once = l2_policy_evict_first();  // every weight byte is read once
            for (uint32_t phase = 0; ok && phase < 2u; phase++) {
                const uint32_t tasks = phase == 0 ? tasks_gu : tasks_dn;
                const uint32_t per = phase == 0 ? per_gu : per_dn;
                const uint32_t k = phase == 0 ? H : S;
                const uint32_t scale_row_bytes = (k >> a.block_shift) * a.scale_bytes;
                const uint32_t mine = my_tasks(tasks);
                for (uint32_t i0 = 0; ok && i0 < mine; i0 += kGroups) {
                    const void *wmap[kGroups];
                    int32_t row0[kGroups];
                    for (uint32_t q = 0; ok && q < kGroups && i0 + q < mine; q++) {
                        const uint32_t task = blockIdx.x + (i0 + q) * n;
                        const bool up = phase == 0 && task * 16u >= S;
                        row0[q] = (int32_t)(up ? task * 16u - S : task * 16u);
                        wmap[q] = phase == 1 ? (const void *)&maps.down
                                             : (up ? (const void *)&maps.up : (const void *)&maps.gate);
                        const void *smap = phase == 1 ? (const void *)&maps.down_s
                                                      : (up ? (const void *)&maps.up_s : (const void *)&maps.gate_s);
                        if (!mbar_wait(&sc_empty[q][sc[q]], sc_ph[q] ^ 1u, abort_flag)) { ok = false; break; }
                        mbar_arrive_expect_tx(&sc_full[q][sc[q]], 16u * scale_row_bytes);
                        tma_load_2d_hint(scale_slot + (q * kScaleSlots + sc[q]) * kScaleSlotBytes, smap,
                                         &sc_full[q][sc[q]], 0, row0[q], stream_once);
                        if (++sc[q] == kScaleSlots) { sc[q] = 0; sc_ph[q] ^= 1u; }
                    }
                    for (uint32_t j = 0; ok && j < per; j++) {
                        for (uint32_t q = 0; q < kGroups && i0 + q < mine; q++) {
                            if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                            mbar_arrive_expect_tx(&full[s], kStageBytes);
                            tma_load_4d(ring + s * kStageBytes, wmap[q], &full[s], 0, row0[q], (int32_t)j, 0, stream_once);
                            if (++s == kStages) { s = 0; ph ^= 1u; }
                        }
                    }
                }
            }
        }
    } else if (warp > kProducerWarp) {
        // ===================================================== finishers
        const uint32_t q = warp - kProducerWarp - 1u;
        uint32_t count = 0;
        bool ok = true;
        for (uint32_t phase = 0; ok && phase < 2u; phase++) {
            const uint32_t tasks = phase == 0 ? tasks_gu : tasks_dn;
            const uint32_t mine = my_tasks(tasks);
            uint32_t done = 0;
            for (uint32_t i = q; ok && i < mine; i += kGroups) {
                const uint32_t task = blockIdx.x + i * n;
                const bool up = phase == 0 && task * 16u >= S;
                const uint32_t row0 = up ? task * 16u - S : task * 16u;
                const uint32_t buf = count & 1u, par = (count >> 1) & 1u;
                count++;
                if (!mbar_wait(&fin_full[q][buf], par, abort_flag)) { ok = false; break; }
                if (lane < 16u) {
                    float v = 0.f;
#pragma unroll
                    for (uint32_t w = 0; w < kWarps; w++) v += part[q][buf][w][lane];
                    uint16_t *dst = phase == 1 ? a.sh_out : (up ? a.sh_up : a.sh_gate);
                    dst[row0 + lane] = float_to_bf16_bits(v * inv_scale_s[phase]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&fin_empty[q][buf]);
                done++;
            }
            // this group's rows are in memory (phase 0: counted for the other CTAs' down phase;
            // phase 1: before this CTA counts itself out below)
            __threadfence();
            __syncwarp();
            if (phase == 0 && lane == 0) atomicAdd(a.sync, done);
        }
    } else {
        // ===================================================== consumers
        const uint32_t tid = threadIdx.x;                  // 0 .. 511
        const uint32_t q = warp / kWarps, w8 = warp % kWarps;
        const uint32_t g = lane >> 2, t = lane & 3u;
        const bool b_active = g == t;
        const uint32_t sgrp = 2u * (t & 1u);
        uint32_t s = 0, ph = 0, sc = 0, sc_ph = 0, count = 0;
        bool ok = true;
        // Stages a bf16 vector of `elements` (elements / 8 <= 4 * 512) as f16 after the exact
        // power-of-two rescale of stage_vectors_f16_n; `fetch(chunk)` returns eight bf16 values.
        auto stage_vector = [&](uint32_t elements, uint32_t slot, auto fetch) {
            uint4 held[4];
            float mx = 0.f;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t c = tid + (uint32_t)j * kConsumers;
                held[j] = c < elements / 8u ? fetch(c) : make_uint4(0u, 0u, 0u, 0u);
                const uint32_t w[4] = {held[j].x, held[j].y, held[j].z, held[j].w};
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    mx = fmaxf(mx, fabsf(__uint_as_float(w[r] << 16)));
                    mx = fmaxf(mx, fabsf(__uint_as_float(w[r] & 0xffff0000u)));
                }
            }
            mx = warp_max(mx);
            if (lane == 0) warp_max_s[warp] = mx;
            consumer_sync();
            float m = 0.f;
            for (uint32_t w = 0; w < kGroups * kWarps; w++) m = fmaxf(m, warp_max_s[w]);
            int e = 0;
            if (m > 0.f && m <= 3.0e38f) {
                e = (int)((__float_as_uint(m) >> 23) & 0xffu) - 127 - 14;
                e = max(-100, min(100, e));
            }
            const float mul = __uint_as_float((uint32_t)(127 - e) << 23);        // 2^-e
            if (tid == 0) inv_scale_s[slot] = __uint_as_float((uint32_t)(127 + e) << 23);   // 2^e
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t c = tid + (uint32_t)j * kConsumers;
                if (c >= elements / 8u) continue;
                const uint32_t w[4] = {held[j].x, held[j].y, held[j].z, held[j].w};
                uint32_t h[4];
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    const __half2 p = __floats2half2_rn(__uint_as_float(w[r] << 16) * mul,
                                                        __uint_as_float(w[r] & 0xffff0000u) * mul);
                    h[r] = *reinterpret_cast<const uint32_t *>(&p);
                }
                reinterpret_cast<uint4 *>(vec)[c] = make_uint4(h[0], h[1], h[2], h[3]);
            }
            consumer_sync();
        };
        stage_vector(H, 0u, [&](uint32_t c) { return __ldg(reinterpret_cast<const uint4 *>(a.x) + c); });

        // After a wait gave up (`ok` false) a warp keeps walking the same sequence of named
        // barriers without waiting or computing, so that no other warp is left alone at one.
        for (uint32_t phase = 0; phase < 2u; phase++) {
            const uint32_t tasks = phase == 0 ? tasks_gu : tasks_dn;
            const uint32_t per = phase == 0 ? per_gu : per_dn;
            const uint32_t k = phase == 0 ? H : S;
            const uint32_t scale_row_bytes = (k >> a.block_shift) * a.scale_bytes;
            const uint32_t mine = my_tasks(tasks);
            if (phase == 1) {
                // every CTA's gate and up rows must be in memory (the finishers count them)
                consumer_sync();                         // nobody reads the token in `vec` any more
                if (tid == 0) {
                    const unsigned long long t0 = global_timer_ns();
                    uint32_t spins = 0;
                    while (*reinterpret_cast<volatile uint32_t *>(a.sync) < tasks_gu) {
                        if ((++spins & 63u) == 0u && (*abort_flag != 0u || global_timer_ns() - t0 > kWaitLimitNs)) {
                            *abort_flag = 1u;
                            break;
                        }
                    }
                    __threadfence();
                }
                consumer_sync();
                if (*abort_flag != 0u) ok = false;
                // activation of (gate, up) as bf16, then staged like the token
                stage_vector(S, 1u, [&](uint32_t c) {
                    const uint4 gv = __ldcg(reinterpret_cast<const uint4 *>(a.sh_gate) + c);
                    const uint4 uv = __ldcg(reinterpret_cast<const uint4 *>(a.sh_up) + c);
                    const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
                    uint32_t o[4];
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        const uint32_t lo = float_to_bf16_bits(activation(__uint_as_float(gw[r] << 16),
                                                                          __uint_as_float(uw[r] << 16), a.activation,
                                                                          a.beta, a.linear_beta));
                        const uint32_t hi = float_to_bf16_bits(activation(__uint_as_float(gw[r] & 0xffff0000u),
                                                                          __uint_as_float(uw[r] & 0xffff0000u),
                                                                          a.activation, a.beta, a.linear_beta));
                        o[r] = lo | (hi << 16);
                    }
                    return make_uint4(o[0], o[1], o[2], o[3]);
                });
            }
            for (uint32_t i0 = 0; i0 < mine; i0 += kGroups) {
                const bool have = i0 + q < mine;                    // this group has a task in the pair
                const uint32_t pair = min(kGroups, mine - i0);      // tasks in the pair
                const unsigned char *scales = scale_slot + (q * kScaleSlots + sc) * kScaleSlotBytes;
                if (have && ok && !mbar_wait(&sc_full[q][sc], sc_ph, abort_flag)) ok = false;
                float acc_a = 0.f, acc_b = 0.f;
                for (uint32_t j = 0; j < per; j++) {
                    // the pair's stages of step j sit in ring order: group 0's, then group 1's
                    const uint32_t mine_s = (s + q) % kStages, mine_ph = ph ^ ((s + q) >= kStages ? 1u : 0u);
                    s += pair;
                    if (s >= kStages) { s -= kStages; ph ^= 1u; }
                    if (!have || !ok) continue;
                    if (!mbar_wait(&full[mine_s], mine_ph, abort_flag)) { ok = false; continue; }
                    const uint32_t step = w8 * per + j;
                    // this warp's 16 x 128 tile; 16-byte chunk c of row r sits at chunk c ^ (r & 7)
                    const unsigned char *tile = ring + mine_s * kStageBytes + w8 * 2048u;
                    Q8Step cur;
                    cur.a0 = *reinterpret_cast<const uint4 *>(tile + g * 128u + (((2u * t) ^ g) << 4));
                    cur.a1 = *reinterpret_cast<const uint4 *>(tile + g * 128u + (((2u * t + 1u) ^ g) << 4));
                    cur.b0 = *reinterpret_cast<const uint4 *>(tile + (g + 8u) * 128u + (((2u * t) ^ g) << 4));
                    cur.b1 = *reinterpret_cast<const uint4 *>(tile + (g + 8u) * 128u + (((2u * t + 1u) ^ g) << 4));
                    const uint32_t c0 = 128u * step + 32u * sgrp;
                    const unsigned char *ra = scales + g * scale_row_bytes, *rb = scales + (g + 8u) * scale_row_bytes;
                    const uint32_t i0 = c0 >> a.block_shift, i1 = (c0 + 32u) >> a.block_shift;
                    if (a.scale_bytes == 2u) {
                        cur.sa0 = __half2float(reinterpret_cast<const __half *>(ra)[i0]);
                        cur.sa1 = __half2float(reinterpret_cast<const __half *>(ra)[i1]);
                        cur.sb0 = __half2float(reinterpret_cast<const __half *>(rb)[i0]);
                        cur.sb1 = __half2float(reinterpret_cast<const __half *>(rb)[i1]);
                    } else {
                        cur.sa0 = reinterpret_cast<const float *>(ra)[i0];
                        cur.sa1 = reinterpret_cast<const float *>(ra)[i1];
                        cur.sb0 = reinterpret_cast<const float *>(rb)[i0];
                        cur.sb1 = reinterpret_cast<const float *>(rb)[i1];
                    }
                    q8_step_apply(acc_a, acc_b, cur, vec + 32u * t + 128u * step, b_active);
                    // the stage goes back to the producer after an instruction that consumed
                    // every loaded register (the arithmetic above), not right after the loads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[mine_s]);
                }
                if (!have) continue;
                __syncwarp();
                if (lane == 0) mbar_arrive(&sc_empty[q][sc]);
                if (++sc == kScaleSlots) { sc = 0; sc_ph ^= 1u; }
                acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 1);
                acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 1);
                const uint32_t buf = count & 1u, par = (count >> 1) & 1u;
                count++;
                if (ok && !mbar_wait(&fin_empty[q][buf], par ^ 1u, abort_flag)) ok = false;
                if (t == 0) {
                    part[q][buf][w8][g] = acc_a;
                    part[q][buf][w8][g + 8u] = acc_b;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&fin_full[q][buf]);
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (*abort_flag != 0u) atomicExch(&g_shared_status, 1u);
        // the last CTA to leave puts the words back to zero for the next call
        __threadfence();
        if (atomicAdd(a.sync + 1, 1u) == n - 1u) {
            atomicExch(a.sync, 0u);
            atomicExch(a.sync + 1, 0u);
        }
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

// int8 [rows, k] seen as {128 bytes, rows, k / 1024 steps of a warp's slice, 8 warps}
bool map_weights(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t k) {
    auto fn = encode_fn();
    if (!fn) return false;
    const uint64_t per = k / 1024u;
    const cuuint64_t dims[4] = {128, rows, per, 8};
    const cuuint64_t strides[3] = {k, 128, 128 * per};
    const cuuint32_t box[4] = {128, 16, 1, 8};
    const cuuint32_t es[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(ptr), dims, strides, box, es,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// scales [rows, row_bytes] as 32-bit words, box = 16 whole rows
bool map_scales(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t row_bytes) {
    auto fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {row_bytes / 4u, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)(row_bytes / 4u), 16};
    const cuuint32_t es[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(ptr), dims, strides, box, es,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

size_t ring_smem_bytes(const k3_moe_layer_desc *d) {
    return (size_t)kStages * kStageBytes + (size_t)kGroups * kScaleSlots * kScaleSlotBytes +
           (size_t)std::max(d->hidden, d->shared_hidden) * 2u + 1024u;
}

}  // namespace

uint32_t k3_decode_shared_status() {
    uint32_t v = 0xffffffffu;
    if (cudaMemcpyFromSymbol(&v, g_shared_status, sizeof(v)) != cudaSuccess) (void)cudaGetLastError();
    return v;
}

bool k3_decode_shared_status_clear() {
    const uint32_t zero = 0u;
    if (cudaMemcpyToSymbol(g_shared_status, &zero, sizeof(zero)) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return true;
}

bool k3_decode_shared_ring_supported(const k3_moe_layer_desc *d) {
    const uint32_t H = d->hidden, S = d->shared_hidden;
    if (S == 0u || H % 1024u != 0u || S % 1024u != 0u || H > 8192u || S > 8192u) return false;
    if (d->q8_block < 32u || (d->q8_block & (d->q8_block - 1u)) != 0u || H % d->q8_block != 0u ||
        S % d->q8_block != 0u) {
        return false;                                            // a power of two: scale index by shift
    }
    const uint32_t sb = d->q8_scale_type == K3_MOE_Q8_SCALE_F16 ? 2u : 4u;
    const uint32_t row_gu = H / d->q8_block * sb, row_dn = S / d->q8_block * sb;
    if (row_gu % 16u != 0u || row_dn % 16u != 0u || row_gu > 1024u || row_dn > 1024u) return false;
    const uintptr_t all = (uintptr_t)d->shared_gate_q | (uintptr_t)d->shared_up_q | (uintptr_t)d->shared_down_q |
                          (uintptr_t)d->shared_gate_s | (uintptr_t)d->shared_up_s | (uintptr_t)d->shared_down_s;
    return (all & 15u) == 0u && encode_fn() != nullptr;
}

// CTAs (= SMs) the shared expert's kernel holds: 32 by default (8 gate / up tasks and 14 down
// tasks each at the benchmark shape).  The environment variable K3MOE_SHARED_CTAS, read once,
// overrides it (1..64); 0 turns the ring kernel off (the row kernels on a side stream run).
uint32_t k3_decode_shared_ring_ctas() {
    static const uint32_t value = [] {
        const char *env = std::getenv("K3MOE_SHARED_CTAS");
        if (env == nullptr || *env == '\0') return 32u;
        const long v = std::strtol(env, nullptr, 10);
        return (uint32_t)(v >= 0 && v <= 64 ? v : 32);
    }();
    return std::min<uint32_t>(value, (uint32_t)sm_count() / 2u);
}

// Launches the shared expert of one token on `stream`: sh_gate / sh_up [S] and sh_out [H]
// (bf16) from x [H].  The kernel lets programmatically serialized successors start at once.
bool k3_decode_shared_ring(const k3_moe_layer_desc *d, const void *x, void *sh_gate, void *sh_up, void *sh_out,
                           void *zero_word, cudaStream_t stream) {
    if ((((uintptr_t)x | (uintptr_t)sh_gate | (uintptr_t)sh_up) & 15u) != 0u) return false;
    const uint32_t H = d->hidden, S = d->shared_hidden;
    const uint32_t sb = d->q8_scale_type == K3_MOE_Q8_SCALE_F16 ? 2u : 4u;
    struct MapKey {
        int device;
        const void *p[6];
        uint32_t dims[4];
        bool operator<(const MapKey &o) const {
            if (device != o.device) return device < o.device;
            const int c = memcmp(p, o.p, sizeof(p));
            return c != 0 ? c < 0 : memcmp(dims, o.dims, sizeof(dims)) < 0;
        }
    };
    constexpr size_t kCachedLayers = 256;
    static std::mutex map_lock;
    static std::map<MapKey, RingMaps> cached;
    MapKey key{};
    key.device = current_device();
    const void *ptrs[6] = {d->shared_gate_q, d->shared_up_q, d->shared_down_q,
                           d->shared_gate_s, d->shared_up_s, d->shared_down_s};
    memcpy(key.p, ptrs, sizeof(ptrs));
    key.dims[0] = H; key.dims[1] = S; key.dims[2] = d->q8_block; key.dims[3] = sb;
    RingMaps maps;
    {
        std::lock_guard<std::mutex> guard(map_lock);
        auto it = cached.find(key);
        if (it == cached.end()) {
            if (!map_weights(&maps.gate, d->shared_gate_q, S, H) || !map_weights(&maps.up, d->shared_up_q, S, H) ||
                !map_weights(&maps.down, d->shared_down_q, H, S) ||
                !map_scales(&maps.gate_s, d->shared_gate_s, S, (uint64_t)H / d->q8_block * sb) ||
                !map_scales(&maps.up_s, d->shared_up_s, S, (uint64_t)H / d->q8_block * sb) ||
                !map_scales(&maps.down_s, d->shared_down_s, H, (uint64_t)S / d->q8_block * sb)) {
                return false;
            }
            if (cached.size() >= kCachedLayers) cached.clear();
            cached.emplace(key, maps);
        } else {
            maps = it->second;
        }
    }
    // the words of the next slot on this device (calls in flight at once on different
    // streams use different slots unless more than kSyncSlots of them overlap)
    static std::mutex sync_lock;
    static std::map<int, uint32_t *> sync_base;
    static std::atomic<uint32_t> next_slot{0};
    uint32_t *words = nullptr;
    {
        std::lock_guard<std::mutex> guard(sync_lock);
        auto it = sync_base.find(key.device);
        if (it == sync_base.end()) {
            if (cudaGetSymbolAddress((void **)&words, g_shared_sync) != cudaSuccess) {
                (void)cudaGetLastError();
                return false;
            }
            sync_base[key.device] = words;
        } else {
            words = it->second;
        }
    }
    RingArgs a{};
    a.x = (const uint16_t *)x;
    a.sh_gate = (uint16_t *)sh_gate;
    a.sh_up = (uint16_t *)sh_up;
    a.sh_out = (uint16_t *)sh_out;
    a.H = H;
    a.S = S;
    a.scale_bytes = sb;
    a.block_shift = 0u;
    while ((1u << a.block_shift) < d->q8_block) a.block_shift++;
    a.activation = d->activation;
    a.beta = d->beta;
    a.linear_beta = d->linear_beta;
    a.sync = words + 2u * (next_slot.fetch_add(1u) % kSyncSlots);
    a.zero_word = (uint32_t *)zero_word;
    const size_t smem = ring_smem_bytes(d);
    if (!set_max_dynamic_smem((const void *)decode_shared_ring_kernel, smem)) return false;
    decode_shared_ring_kernel<<<k3_decode_shared_ring_ctas(), kThreads, smem, stream>>>(maps, a);
    return launch_ok();
}
