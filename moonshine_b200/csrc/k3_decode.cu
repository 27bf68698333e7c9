// One-token (decode) routed-MoE layer: four launches on the caller's stream, one chain of
// programmatic launches, no host round trip.
//
//   shared   the shared expert (Q8 rows on mma.sync) as a ring kernel on a few SMs
//            (k3_decode_shared.cu); it depends only on the token, starts first and lets
//            the kernels behind it start at once
//   router   router logits (the reference's reduction order, all rows of a block in
//            flight at once), scores, and the token's E2M1 terms
//   experts  every CTA routes the token (sigmoid + bias top-k), then the selected
//            experts' gate/up + activation and down products (k3_decode_mx.cu)
//   tail     weighted sum in rank order + shared output + residual (k3_decode_tail.cuh)
// Shapes the ring kernel does not take run the shared expert as two row kernels on a
// low-priority side stream, and the tail then has no launch of its own: the producers of
// its inputs (down epilogue warps, shared-down blocks) count arrivals per 32 output
// columns and the last one forms them.  With an expert-parallel shard (not every expert
// local) a combine launch follows instead of the tail.
//
// It replaces the per-token sequence of the reference's decode_routed_layer
// (k3_engine.cu:1554-1563 router, :1668-1689 static projections, :1032-1066
// launch_expert x 16, :1851-1897 tail), which needs three host synchronisations
// and ~70 launches per layer.
//
// The expert kernel of the main path is the block-scaled tensor-core kernel of
// k3_decode_mx.cu.  The ones in this file serve the remaining shapes: persistent,
// a CTA stages the activation vector(s) in shared memory once (as f16 after an
// exact power-of-two rescale), then each warp streams whole 16-row blocks of
// MXFP4 weights over the full K extent with a three-deep register prefetch,
// converts nibbles to f16 with byte-permute lookups and accumulates per 32-column
// scale group on mma.sync (see k3_gemv.cuh for the fragment layout).
#include "k3_decode_tail.cuh"
#include "k3_e2m1_terms.cuh"
#include "k3_gemv.cuh"
#include "k3_grouped.h"
#include "k3_rowdot.cuh"
#include "k3_moe_layer.h"
#include "k3_moe_ops.h"

#include <algorithm>
#include <atomic>
#include <map>
#include <mutex>


using namespace k3;

namespace {

constexpr int kDecodeWarps = 16;
constexpr int kDecodeThreads = kDecodeWarps * kWarp;
constexpr int kPrefetch = 3;

struct DecodeArgs {
    k3_moe_layer_desc d;
    const uint16_t *x;        // [hidden]
    float *logits;            // [E]
    uint32_t *ids;            // [top_k]
    float *weights;           // [top_k]
    uint16_t *sh_gate, *sh_up, *sh_act, *sh_out;   // shared expert buffers
    uint16_t *act;            // [top_k, I]
    uint16_t *rows_out;       // [top_k, hidden]
    uint32_t skip_shared;     // down kernel: the shared expert's rows are computed elsewhere
    uint8_t *x_terms, *x_sf;  // front: E2M1 terms of x ([kTerms, hidden/2] packed, [kTerms, hidden/32]) or null
    float *route_words;       // front: [2][1024] scores and choices written by the row tasks, or null
    unsigned int *ticket;     // front: completion counter of this call
    uint32_t *control;        // front: words the expert kernel needs zeroed (64), or null
    uint32_t *front_done;     // router kernel: count of finished blocks for the expert kernel, or null
    uint32_t rows_in_flight;  // router kernel: rows a block fetches at once (<= kRouterRowsInFlight)
    uint32_t route_elsewhere; // front: only the row tasks; the expert kernel routes from the scores
    uint32_t shared_elsewhere;  // front: the shared expert runs in its own kernels (side stream)
    DecodeTail tail;            // shared down: its share of the layer's tail (tail.out null: none)
};


// ------------------------------------------------------------------- front
// Tickets of the "last block finishes the job" step of the front kernel.  A call
// takes the next slot round-robin, the last block of the grid resets it, so calls
// running at once on different streams do not share a counter unless more than
// kTicketSlots of them are in flight.
constexpr uint32_t kTicketSlots = 64;
__device__ unsigned int g_front_tickets[kTicketSlots];
__device__ uint32_t g_decode_status = 0;     // set when an arrival count of the tail did not go through

// float -> unsigned key with the same order (-0 is folded into +0 first)
K3_DEVINL uint32_t order_key(float f) {
    const uint32_t b = __float_as_uint(f + 0.0f);
    return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
}

// One 256-thread block per row task: router rows and the shared expert's gate
// and up rows (reference reduction order, thread v = the reference's lane v, the
// whole row in flight at once), plus the 32-column blocks of the token's E2M1
// terms.  The last block to finish then routes the token (sigmoid + bias
// top-k in the reference's order: larger choice first, lower expert id on ties)
// and applies the shared expert's activation.
template <bool kWithShared>
__global__ void __launch_bounds__(256, kWithShared ? 2 : 4)
decode_front_kernel(DecodeArgs a) {
    extern __shared__ __align__(16) unsigned char front_smem[];
    float *xf = reinterpret_cast<float *>(front_smem);                       // [hidden] as fp32
    __half *xh = reinterpret_cast<__half *>(front_smem + (size_t)a.d.hidden * 4u);   // [2][hidden] f16, rescaled
    __shared__ float inv_scale[2], stage_scratch[2 * 8], part[8][16];
    __shared__ float choice_s[1024], score_s[1024];
    __shared__ float red[kRowBlock];
    __shared__ float top_score[32];
    __shared__ uint32_t top_id[32], list_key[8 * 32], list_id[8 * 32];
    __shared__ uint32_t is_last;
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t E = a.d.expert_count, S = a.d.shared_hidden, H = a.d.hidden, k = a.d.top_k;
    const uint32_t split_tasks = a.x_terms ? (H / 32u + 7u) / 8u : 0u;        // 8 blocks (one per warp) each
    if (blockIdx.x == 0 && a.control != nullptr && threadIdx.x < 64u) a.control[threadIdx.x] = 0u;
    if ((reinterpret_cast<uintptr_t>(a.x) & 15u) == 0u && H % 8u == 0u) {
        // 16 bytes per load: the whole token is in flight after at most four loads per thread
        for (uint32_t i = threadIdx.x; i < H / 8u; i += blockDim.x) {
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(a.x) + i);
            float4 *dst = reinterpret_cast<float4 *>(xf + 8u * i);
            dst[0] = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u),
                                 __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u));
            dst[1] = make_float4(__uint_as_float(v.z << 16), __uint_as_float(v.z & 0xffff0000u),
                                 __uint_as_float(v.w << 16), __uint_as_float(v.w & 0xffff0000u));
        }
    } else {
        for (uint32_t i = threadIdx.x; i < H; i += blockDim.x) xf[i] = bf16_bits_to_float(a.x[i]);
    }
    if (kWithShared) {
        stage_vectors_f16(xh, inv_scale, a.x, nullptr, H, H, stage_scratch);     // ends with a block barrier
    } else {
        __syncthreads();
    }
    // tasks: router rows one at a time, then blocks of 16 gate / up rows
    const uint32_t groups = kWithShared ? 2u * S / 16u : 0u;
    const uint32_t tasks_total = E + groups + split_tasks;
    // The extra last block of the grid takes no tasks: it runs the routing code once
    // on stale data without storing anything, so that those instructions are already
    // cached when the last worker block needs them - on its own they cost a chain of
    // instruction fetches from memory several times longer than the arithmetic.
    // (when the routing is done by the expert kernel there is no such block and no last-block step)
    const bool warmer = a.route_elsewhere == 0u && blockIdx.x == gridDim.x - 1u;
    const uint32_t workers = a.route_elsewhere != 0u ? gridDim.x : gridDim.x - 1u;
    // the kernel queued behind this one with programmatic serialization may be placed as
    // soon as every block of this grid has started
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    for (uint32_t task = blockIdx.x; !warmer && task < tasks_total; task += workers) {
        if (task < E) {
            // the row's bias is fetched with the row, so the routing step finds score and
            // choice ready instead of starting from the logits
            float bias = 0.f;
            if (threadIdx.x == 0 && a.route_words != nullptr) bias = __ldg((const float *)a.d.router_bias + task);
            Bf16RowLoad p;
            bf16_block_load(p, (const uint16_t *)a.d.router_weight + (uint64_t)task * H, H);
            const float v = block_tree_256(bf16_block_lane_sum(p, xf, H), red);
            if (threadIdx.x == 0) {
                a.logits[task] = v;
                if (a.route_words != nullptr) {
                    const float sc = sigmoid_exact(v);
                    a.route_words[task] = sc;
                    a.route_words[1024u + task] = sc + bias;
                }
            }
        } else if (kWithShared && task < E + groups) {
            // 16 gate or up rows on the tensor-core Q8 scheme, the K extent split over the 8 warps
            const uint32_t r0 = (task - E) * 16u;                     // S % 16 == 0
            const bool up = r0 >= S;
            const uint32_t row0 = up ? r0 - S : r0;
            const uint32_t steps = H / 128u, per = (steps + 7u) / 8u;
            float p0, p1;
            q8_rows16_partial<3>(p0, p1, (const int8_t *)(up ? a.d.shared_up_q : a.d.shared_gate_q),
                                 up ? a.d.shared_up_s : a.d.shared_gate_s, a.d.q8_scale_type, a.d.q8_block,
                                 row0, H, min(steps, warp * per), min(steps, (warp + 1u) * per), xh);
            if ((lane & 3u) == 0u) {
                part[warp][lane >> 2] = p0;
                part[warp][(lane >> 2) + 8u] = p1;
            }
            __syncthreads();
            if (threadIdx.x < 16u) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < 8; w++) v += part[w][threadIdx.x];
                (up ? a.sh_up : a.sh_gate)[row0 + threadIdx.x] = float_to_bf16_bits(v * inv_scale[0]);
            }
        } else {
            const uint32_t blk = (task - E - groups) * 8u + warp;
            if (blk < H / 32u) {
                uint32_t code[kTerms], sbyte[kTerms];
                split_block_e2m1(xf[blk * 32u + lane], code, sbyte);
                store_block_e2m1(a.x_terms, a.x_sf, H / 2u, H / 32u, blk, code, sbyte, lane);
            }
        }
        __syncthreads();            // `red` is reused by the next task
    }
    if (a.route_elsewhere != 0u) return;
    if (!warmer) {
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned int ticket = atomicAdd(a.ticket, 1u);
            is_last = ticket == workers - 1u ? 1u : 0u;
        }
        __syncthreads();
        if (is_last == 0u) return;
        __threadfence();
        if (threadIdx.x == 0) *a.ticket = 0u;
    }
    const bool commit = !warmer;
    // ---- routing and shared activation: results of the other blocks come from L2
    if (a.route_words != nullptr) {
        float sc[4], ch[4];
#pragma unroll
        for (uint32_t j = 0; j < 4u; j++) {                 // all eight loads in flight
            const uint32_t e = threadIdx.x + j * 256u;
            sc[j] = e < E ? __ldcg(a.route_words + e) : 0.f;
            ch[j] = e < E ? __ldcg(a.route_words + 1024u + e) : 0.f;
        }
#pragma unroll
        for (uint32_t j = 0; j < 4u; j++) {
            score_s[threadIdx.x + j * 256u] = sc[j];
            choice_s[threadIdx.x + j * 256u] = ch[j];
        }
    } else {
        for (uint32_t e = threadIdx.x; e < 1024u; e += blockDim.x) {
            float sc = 0.f, ch = 0.f;
            if (e < E) {
                sc = sigmoid_exact(__ldcg(a.logits + e));
                ch = sc + ((const float *)a.d.router_bias)[e];
            }
            score_s[e] = sc;
            choice_s[e] = ch;
        }
    }
    __syncthreads();
    // Two levels of arg-max rounds on order keys (0 = none).  Level 1: warp w owns
    // experts [128 w, 128 w + 128), four per lane, and lists its top_k best.  Level 2:
    // warp 0 merges the eight lists.  Ties go to the lower expert id at both levels.
    {
        uint32_t key[4];
#pragma unroll
        for (uint32_t j = 0; j < 4u; j++) {
            const uint32_t e = warp * 128u + j * 32u + lane;
            key[j] = e < E ? order_key(choice_s[e]) : 0u;
        }
        for (uint32_t rank = 0; rank < k; rank++) {
            uint32_t best_key = key[0], best_slot = 0u;
#pragma unroll
            for (uint32_t j = 1; j < 4u; j++) {
                if (key[j] > best_key) { best_key = key[j]; best_slot = j; }
            }
            const uint32_t top = __reduce_max_sync(0xffffffffu, best_key);
            const uint32_t id = warp * 128u + best_slot * 32u + lane;
            const uint32_t win = __reduce_min_sync(0xffffffffu, (top != 0u && best_key == top) ? id : 0xffffffffu);
            if (lane == 0) {
                list_key[warp * 32u + rank] = top;
                list_id[warp * 32u + rank] = win;
            }
            if (win == id) {
#pragma unroll
                for (uint32_t j = 0; j < 4u; j++) {
                    if (j == best_slot) key[j] = 0u;
                }
            }
        }
    }
    __syncthreads();
    // Level 2 by rank counting: candidate t of the 8 * top_k listed ones counts the
    // candidates that beat it; ranks are unique because ids are.
    if (threadIdx.x < 32u) { top_id[threadIdx.x] = 0xffffffffu; top_score[threadIdx.x] = 0.f; }
    __syncthreads();
    {
        const uint32_t n = 8u * k;                                  // <= 256 = blockDim.x
        // compact the eight lists (stride 32) into choice_s / red, which are free now
        uint32_t *ckey = reinterpret_cast<uint32_t *>(choice_s), *cid = reinterpret_cast<uint32_t *>(red);
        uint32_t my_key = 0u, my_id = 0xffffffffu;
        if (threadIdx.x < n) {
            const uint32_t src = (threadIdx.x / k) * 32u + threadIdx.x % k;
            my_key = list_key[src];
            my_id = list_id[src];
        }
        __syncthreads();                                            // choice_s was read by level 1
        ckey[threadIdx.x] = my_key;
        cid[threadIdx.x] = my_id;
        __syncthreads();
        uint32_t rank = 0u;
#pragma unroll 8
        for (uint32_t u = 0; u < n; u++) {
            const uint32_t ok = ckey[u], oi = cid[u];
            rank += (ok > my_key || (ok == my_key && oi < my_id)) ? 1u : 0u;
        }
        if (my_key != 0u && rank < k) {
            top_id[rank] = my_id;
            top_score[rank] = score_s[my_id];
        }
    }
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        float denominator = 1e-20f;
        for (uint32_t r = 0; r < k; r++) denominator += top_score[r];
        if (lane < k && commit) {
            a.ids[lane] = top_id[lane];
            a.weights[lane] = __fmul_rn(__fdiv_rn(top_score[lane], denominator), a.d.route_scale);
        }
    } else if (kWithShared) {
        for (uint32_t i = threadIdx.x - kWarp; i < S; i += blockDim.x - kWarp) {
            const uint16_t bits =
                float_to_bf16_bits(activation(bf16_bits_to_float(__ldcg(a.sh_gate + i)),
                                              bf16_bits_to_float(__ldcg(a.sh_up + i)), a.d.activation,
                                              a.d.beta, a.d.linear_beta));
            if (commit) a.sh_act[i] = bits;
        }
    }
}

// ------------------------------------------------------------ router rows
// Front kernel of the block-scaled path: router rows and the token's E2M1 terms, nothing
// else (the expert kernel routes, the shared expert has its own kernels).  A block owns
// rows b, b + G, b + 2G, b + 3G of a grid of G blocks and has all of them in flight at
// once (16-byte asynchronous copies into shared memory, no registers held), so the whole
// router table is requested in the kernel's first microsecond.  The arithmetic is the
// reference's: thread v sums columns v, v + 256, ... in order, then the 256-lane tree.
constexpr uint32_t kRouterRowsInFlight = 6;      // at most; a launch asks for what its grid needs

// (evict-first in L2: the router table is read once per token)
K3_DEVINL void cp_async_16(void *dst_shared, const void *src_global, uint64_t policy) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"(
                     (uint32_t)__cvta_generic_to_shared(dst_shared)),
                 "l"(src_global), "l"(policy)
                 : "memory");
}

__global__ void __launch_bounds__(256, 2)
decode_router_kernel(DecodeArgs a) {
    extern __shared__ __align__(16) unsigned char router_smem[];
    const uint32_t E = a.d.expert_count, H = a.d.hidden, G = gridDim.x;
    float *xf = reinterpret_cast<float *>(router_smem);                                    // [H] fp32
    uint16_t *rows = reinterpret_cast<uint16_t *>(router_smem + (size_t)H * 4u);          // [4][H] bf16
    __shared__ float red[kRouterRowsInFlight][kRowBlock];
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    if (blockIdx.x == 0 && a.control != nullptr && threadIdx.x < 64u) a.control[threadIdx.x] = 0u;
    // the expert kernel, queued behind this one with programmatic serialization, may take
    // its places as soon as every block of this grid has started
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint16_t *table = (const uint16_t *)a.d.router_weight;
    uint64_t stream_once;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(stream_once));
    bool staged = false;
    const uint32_t batch = a.rows_in_flight;
    for (uint32_t first = blockIdx.x; first < E; first += batch * G) {
#pragma unroll
        for (uint32_t j = 0; j < kRouterRowsInFlight; j++) {
            const uint32_t row = first + j * G;
            if (j < batch && row < E) {
                for (uint32_t c = threadIdx.x; c < H / 8u; c += blockDim.x)
                    cp_async_16(rows + (size_t)j * H + 8u * c, table + (uint64_t)row * H + 8u * c, stream_once);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (!staged) {
            // the token as fp32, loaded while the rows travel
            for (uint32_t i = threadIdx.x; i < H / 8u; i += blockDim.x) {
                const uint4 v = __ldg(reinterpret_cast<const uint4 *>(a.x) + i);
                float4 *dst = reinterpret_cast<float4 *>(xf + 8u * i);
                dst[0] = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u),
                                     __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u));
                dst[1] = make_float4(__uint_as_float(v.z << 16), __uint_as_float(v.z & 0xffff0000u),
                                     __uint_as_float(v.w << 16), __uint_as_float(v.w & 0xffff0000u));
            }
            staged = true;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
#pragma unroll
        for (uint32_t j = 0; j < kRouterRowsInFlight; j++) {
            if (j < batch && first + j * G < E) {
                const uint16_t *wr = rows + (size_t)j * H;
                float sum = 0.f;
                for (uint32_t c = threadIdx.x; c < H; c += 256u) sum = fmaf(bf16_bits_to_float(wr[c]), xf[c], sum);
                red[j][threadIdx.x] = sum;
            }
        }
        __syncthreads();
        if (warp < batch && first + warp * G < E) {
            // the tree of block_tree_256, one warp per row
            const uint32_t row = first + warp * G;
            const float *r = red[warp];
            float a0 = r[lane] + r[lane + 128u], a1 = r[lane + 32u] + r[lane + 160u];
            float a2 = r[lane + 64u] + r[lane + 192u], a3 = r[lane + 96u] + r[lane + 224u];
            a0 += a2; a1 += a3;
            float v = a0 + a1;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
            if (lane == 0) {
                a.logits[row] = v;
                const float sc = sigmoid_exact(v);
                a.route_words[row] = sc;
                a.route_words[1024u + row] = sc + __ldg((const float *)a.d.router_bias + row);
            }
        }
        __syncthreads();            // `rows` and `red` are reused by the next batch
    }
    if (!staged) {
        for (uint32_t i = threadIdx.x; i < H; i += blockDim.x) xf[i] = bf16_bits_to_float(a.x[i]);
        __syncthreads();
    }
    // the token's E2M1 terms: 32-column blocks, one per warp, taken from the far end of the
    // grid (the blocks there own one row fewer)
    const uint32_t split_tasks = (H / 32u + 7u) / 8u;
    for (uint32_t task = G - 1u - blockIdx.x; task < split_tasks; task += G) {
        const uint32_t blk = task * 8u + warp;
        if (blk < H / 32u) {
            uint32_t code[kTerms], sbyte[kTerms];
            split_block_e2m1(xf[blk * 32u + lane], code, sbyte);
            store_block_e2m1(a.x_terms, a.x_sf, H / 2u, H / 32u, blk, code, sbyte, lane);
        }
    }
    if (a.front_done != nullptr) {
        // everything this block wrote is in memory before its count
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) atomicAdd(a.front_done, 1u);
    }
}

// ----------------------------------------------------------------- terms
// The token's E2M1 terms alone (and the expert kernel's control words cleared), for a
// caller that brings its own routing: 32-column blocks, one per warp.
__global__ void __launch_bounds__(256)
decode_terms_kernel(const uint16_t *__restrict__ x, uint8_t *x_terms, uint8_t *x_sf, uint32_t *control,
                    uint32_t hidden) {
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    if (blockIdx.x == 0 && threadIdx.x < 64u) control[threadIdx.x] = 0u;
    const uint32_t blk = blockIdx.x * 8u + warp;
    if (blk < hidden / 32u) {
        uint32_t code[kTerms], sbyte[kTerms];
        split_block_e2m1(bf16_bits_to_float(x[blk * 32u + lane]), code, sbyte);
        store_block_e2m1(x_terms, x_sf, hidden / 2u, hidden / 32u, blk, code, sbyte, lane);
    }
}

// ------------------------------------------------------------------ tail
// The layer's tail as a kernel of its own, queued behind the expert kernel with programmatic
// serialization: its blocks take their places while the experts stream and wait for the
// grids in front (the expert kernel, and through it the shared expert's) to finish.
__global__ void __launch_bounds__(128)
decode_tail_kernel(DecodeTail t) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t group = blockIdx.x * 4u + threadIdx.x / kWarp;
    if (group * 32u < t.hidden) tail_columns(t, group, threadIdx.x % kWarp);
}

// ------------------------------------------------------- persistent experts
struct Prefetched {
    uint4 wa, wb;
    uint32_t sa, sb;      // two scale bytes each (groups g0, g0+1) in the low 16 bits
};

K3_DEVINL Prefetched fetch_step(const uint8_t *pa, const uint8_t *pb, const uint8_t *sa,
                                const uint8_t *sb, uint32_t step, uint32_t t, uint32_t sgrp) {
    Prefetched p;
    const uint32_t grp = 4u * step + t;
    p.wa = ld_stream_16(pa + (uint64_t)grp * 16u);
    p.wb = ld_stream_16(pb + (uint64_t)grp * 16u);
    const uint32_t g0 = 4u * step + sgrp;
    p.sa = *reinterpret_cast<const uint16_t *>(sa + g0);
    p.sb = *reinterpret_cast<const uint16_t *>(sb + g0);
    return p;
}

// One warp: dot products of 16 consecutive rows (row0..row0+15) of an MXFP4
// matrix [rows, k] with one f16 vector in shared memory; k % 128 == 0.
// Result: lanes with t == 0 hold rows g (r0) and g+8 (r1), g = lane / 4.
K3_DEVINL void warp_rows16(float &r0, float &r1, const uint8_t *packed, const uint8_t *scales,
                           uint32_t row0, uint32_t k, const __half *xs) {
    const uint32_t lane = threadIdx.x % kWarp;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t groups = k / 32u, steps = k / 128u;
    const uint8_t *pa = packed + (uint64_t)(row0 + g) * (k / 2u);
    const uint8_t *pb = packed + (uint64_t)(row0 + g + 8u) * (k / 2u);
    const uint8_t *sa = scales + (uint64_t)(row0 + g) * groups;
    const uint8_t *sb = scales + (uint64_t)(row0 + g + 8u) * groups;
    const bool b_active = g == t;                 // column g carries group t of the vector
    const __half *xv = xs + 32u * t;
    const uint32_t sgrp = 2u * (t & 1u);
    Prefetched pf[kPrefetch];
#pragma unroll
    for (int i = 0; i < kPrefetch; i++) {
        if ((uint32_t)i < steps) pf[i] = fetch_step(pa, pb, sa, sb, i, t, sgrp);
    }
    float acc_a = 0.f, acc_b = 0.f;
    for (uint32_t step0 = 0; step0 < steps; step0 += kPrefetch) {
#pragma unroll
        for (int i = 0; i < kPrefetch; i++) {
            const uint32_t step = step0 + i;
            if (step >= steps) break;
            const Prefetched cur = pf[i];
            if (step + kPrefetch < steps) pf[i] = fetch_step(pa, pb, sa, sb, step + kPrefetch, t, sgrp);
            uint32_t xr[16];
            if (b_active) {
                const uint4 *p = reinterpret_cast<const uint4 *>(xv + 128u * step);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint4 v = p[q];
                    xr[4 * q] = v.x; xr[4 * q + 1] = v.y; xr[4 * q + 2] = v.z; xr[4 * q + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int q = 0; q < 16; q++) xr[q] = 0u;
            }
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t wa_w[4] = {cur.wa.x, cur.wa.y, cur.wa.z, cur.wa.w};
            const uint32_t wb_w[4] = {cur.wb.x, cur.wb.y, cur.wb.z, cur.wb.w};
#pragma unroll
            for (int w = 0; w < 4; w++) {
                uint32_t fa[4], fb[4];
                dequant_word_f16(wa_w[w], fa);
                dequant_word_f16(wb_w[w], fb);
                mma_f16_m16n8k16(c, fa[0], fb[0], fa[1], fb[1], xr[4 * w], xr[4 * w + 1]);
                mma_f16_m16n8k16(c, fa[2], fb[2], fa[3], fb[3], xr[4 * w + 2], xr[4 * w + 3]);
            }
            acc_a = fmaf(e8m0_to_float(cur.sa & 0xffu), c[0], acc_a);
            acc_a = fmaf(e8m0_to_float((cur.sa >> 8) & 0xffu), c[1], acc_a);
            acc_b = fmaf(e8m0_to_float(cur.sb & 0xffu), c[2], acc_b);
            acc_b = fmaf(e8m0_to_float((cur.sb >> 8) & 0xffu), c[3], acc_b);
        }
    }
    // lanes t = 0 and 1 hold the two halves (groups 0,1 and 2,3) of the vector
    acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 1);
    acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 1);
    r0 = acc_a;
    r1 = acc_b;
}

// gate/up + activation for the selected experts; x shared by all of them
__global__ void __launch_bounds__(kDecodeThreads, 1)
decode_gateup_kernel(DecodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half *xs = reinterpret_cast<__half *>(smem_raw);
    float *inv_scale = reinterpret_cast<float *>(smem_raw + (size_t)2 * a.d.hidden * sizeof(__half));
    float *scratch = inv_scale + 2;
    const uint32_t H = a.d.hidden, I = a.d.expert_hidden, k = a.d.top_k;
    stage_vectors_f16(xs, inv_scale, a.x, nullptr, H, H, scratch);
    const float inv = inv_scale[0];
    const uint32_t warp_global = blockIdx.x * kDecodeWarps + threadIdx.x / kWarp;
    const uint32_t warps = gridDim.x * kDecodeWarps;
    const uint32_t lane = threadIdx.x % kWarp;
    const uint32_t blocks = I / 16u;
    const uint64_t pstride = (uint64_t)I * (H / 2u), sstride = (uint64_t)I * (H / 32u);
    for (uint32_t task = warp_global; task < k * blocks; task += warps) {
        const uint32_t rank = task / blocks, rb = task % blocks;
        const uint32_t id = a.ids[rank];
        if (id < a.d.local_expert_first || id >= a.d.local_expert_first + a.d.local_expert_count) continue;
        const uint32_t e = id - a.d.local_expert_first;
        float g0, g1, u0, u1;
        warp_rows16(g0, g1, (const uint8_t *)a.d.w1_packed + e * pstride,
                    (const uint8_t *)a.d.w1_scales + e * sstride, rb * 16u, H, xs);
        warp_rows16(u0, u1, (const uint8_t *)a.d.w3_packed + e * pstride,
                    (const uint8_t *)a.d.w3_scales + e * sstride, rb * 16u, H, xs);
        if ((lane & 3u) == 0u) {
            const uint32_t g = lane >> 2;
            uint16_t *out = a.act + (uint64_t)rank * I + rb * 16u;
            const float ga = bf16_bits_to_float(float_to_bf16_bits(g0 * inv));
            const float gb = bf16_bits_to_float(float_to_bf16_bits(g1 * inv));
            const float ua = bf16_bits_to_float(float_to_bf16_bits(u0 * inv));
            const float ub = bf16_bits_to_float(float_to_bf16_bits(u1 * inv));
            out[g] = float_to_bf16_bits(activation(ga, ua, a.d.activation, a.d.beta, a.d.linear_beta));
            out[g + 8u] = float_to_bf16_bits(activation(gb, ub, a.d.activation, a.d.beta, a.d.linear_beta));
        }
    }
}

// down rows of the selected experts (+ the shared expert's down rows)
__global__ void __launch_bounds__(kDecodeThreads, 1)
decode_down_kernel(DecodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const uint32_t H = a.d.hidden, I = a.d.expert_hidden, k = a.d.top_k, S = a.d.shared_hidden;
    __half *xs = reinterpret_cast<__half *>(smem_raw);                       // [k][I]
    float *inv_scale = reinterpret_cast<float *>(smem_raw + (size_t)(k + 1u) * I * sizeof(__half));  // [k+1]
    float *scratch = inv_scale + 34;
    for (uint32_t r = 0; r < k; r += 2u) {
        __syncthreads();
        stage_vectors_f16(xs + (size_t)r * I, inv_scale + r, a.act + (uint64_t)r * I,
                          r + 1u < k ? a.act + (uint64_t)(r + 1u) * I : nullptr, I, I, scratch);
    }
    const uint32_t warp_global = blockIdx.x * kDecodeWarps + threadIdx.x / kWarp;
    const uint32_t warps = gridDim.x * kDecodeWarps;
    const uint32_t lane = threadIdx.x % kWarp;
    const uint32_t blocks = H / 16u;
    const uint64_t pstride = (uint64_t)H * (I / 2u), sstride = (uint64_t)H * (I / 32u);
    const uint32_t expert_tasks = k * blocks;
    const uint32_t shared_tasks = (S && !a.skip_shared) ? H : 0u;            // one warp per shared down row
    for (uint32_t task = warp_global; task < expert_tasks + shared_tasks; task += warps) {
        if (task < expert_tasks) {
            const uint32_t rank = task % k, rb = task / k;
            const uint32_t id = a.ids[rank];
            if (id < a.d.local_expert_first || id >= a.d.local_expert_first + a.d.local_expert_count) continue;
            const uint32_t e = id - a.d.local_expert_first;
            float y0, y1;
            warp_rows16(y0, y1, (const uint8_t *)a.d.w2_packed + e * pstride,
                        (const uint8_t *)a.d.w2_scales + e * sstride, rb * 16u, I,
                        xs + (size_t)rank * I);
            if ((lane & 3u) == 0u) {
                const uint32_t g = lane >> 2;
                const float inv = inv_scale[rank];
                uint16_t *out = a.rows_out + (uint64_t)rank * H + rb * 16u;
                out[g] = float_to_bf16_bits(y0 * inv);
                out[g + 8u] = float_to_bf16_bits(y1 * inv);
            }
        } else {
            const uint32_t row = task - expert_tasks;
            const float v = q8_row_dot_exact((const int8_t *)a.d.shared_down_q + (uint64_t)row * S,
                                             a.d.shared_down_s, (uint64_t)row * (S / a.d.q8_block),
                                             a.sh_act, S, a.d.q8_block, a.d.q8_scale_type, lane);
            if (lane == 0) a.sh_out[row] = float_to_bf16_bits(v);
        }
    }
}

// ---------------------------------------------------- shared expert, on its own
// The shared expert depends only on the token, not on the routing: these two
// kernels run on a side stream next to the front and expert kernels.

// gate and up rows: one 256-thread block per 16 rows, K split over the 8 warps
__global__ void __maxnreg__(120)
decode_shared_gateup_kernel(DecodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half *xh = reinterpret_cast<__half *>(smem_raw);                       // [hidden] f16, rescaled
    __shared__ float inv_scale[2], stage_scratch[2 * 8], part[8][16];
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t S = a.d.shared_hidden, H = a.d.hidden;
    stage_vectors_f16_n<1>(xh, inv_scale, a.x, nullptr, H, H, stage_scratch);
    const uint32_t steps = H / 128u, per = (steps + 7u) / 8u;
    for (uint32_t task = blockIdx.x; task < 2u * S / 16u; task += gridDim.x) {
        const uint32_t r0 = task * 16u;
        const bool up = r0 >= S;
        const uint32_t row0 = up ? r0 - S : r0;
        float p0, p1;
        q8_rows16_partial<3>(p0, p1, (const int8_t *)(up ? a.d.shared_up_q : a.d.shared_gate_q),
                             up ? a.d.shared_up_s : a.d.shared_gate_s, a.d.q8_scale_type, a.d.q8_block, row0, H,
                             min(steps, warp * per), min(steps, (warp + 1u) * per), xh);
        if ((lane & 3u) == 0u) {
            part[warp][lane >> 2] = p0;
            part[warp][(lane >> 2) + 8u] = p1;
        }
        __syncthreads();
        if (threadIdx.x < 16u) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) v += part[w][threadIdx.x];
            (up ? a.sh_up : a.sh_gate)[row0 + threadIdx.x] = float_to_bf16_bits(v * inv_scale[0]);
        }
        __syncthreads();
    }
}

// activation of (gate, up) and the down rows: one 128-thread block per 16 rows
__global__ void __launch_bounds__(128, 4)
decode_shared_down_kernel(DecodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half *act_h = reinterpret_cast<__half *>(smem_raw);                   // [2][S] f16, rescaled
    uint16_t *act_b = reinterpret_cast<uint16_t *>(smem_raw + (size_t)a.d.shared_hidden * 4u);   // [S] bf16
    __shared__ float part[4][16];
    __shared__ float inv_scale[2], stage_scratch[2 * 4];
    const uint32_t H = a.d.hidden, S = a.d.shared_hidden;
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    // eight elements per 16-byte load (S % 128 == 0), all loads of a thread in flight together
    for (uint32_t c = threadIdx.x; c < S / 8u; c += blockDim.x) {
        const uint4 g = reinterpret_cast<const uint4 *>(a.sh_gate)[c], u = reinterpret_cast<const uint4 *>(a.sh_up)[c];
        const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const uint32_t lo = float_to_bf16_bits(activation(__uint_as_float(gw[q] << 16), __uint_as_float(uw[q] << 16),
                                                              a.d.activation, a.d.beta, a.d.linear_beta));
            const uint32_t hi = float_to_bf16_bits(activation(__uint_as_float(gw[q] & 0xffff0000u),
                                                              __uint_as_float(uw[q] & 0xffff0000u), a.d.activation,
                                                              a.d.beta, a.d.linear_beta));
            o[q] = lo | (hi << 16);
        }
        reinterpret_cast<uint4 *>(act_b)[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    __syncthreads();
    stage_vectors_f16(act_h, inv_scale, act_b, nullptr, S, S, stage_scratch);
    const uint32_t steps = S / 128u, per = (steps + 3u) / 4u;
    for (uint32_t c0 = blockIdx.x * 16u; c0 < H; c0 += gridDim.x * 16u) {           // H % 16 == 0
        float p0, p1;
        q8_rows16_partial<2>(p0, p1, (const int8_t *)a.d.shared_down_q, a.d.shared_down_s, a.d.q8_scale_type,
                             a.d.q8_block, c0, S, min(steps, warp * per), min(steps, (warp + 1u) * per), act_h);
        if ((lane & 3u) == 0u) {
            part[warp][lane >> 2] = p0;
            part[warp][(lane >> 2) + 8u] = p1;
        }
        __syncthreads();
        if (threadIdx.x < 16u) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < 4; w++) v += part[w][threadIdx.x];
            a.sh_out[c0 + threadIdx.x] = float_to_bf16_bits(v * inv_scale[0]);
        }
        // these 16 columns are one of the inputs of their 32-column group of the layer output
        if (warp == 0 && a.tail.out != nullptr && !tail_arrive(a.tail, c0 / 32u, lane)) g_decode_status = 1u;
        __syncthreads();
    }
}


}  // namespace

uint32_t k3_decode_status() {
    uint32_t v = 0xffffffffu;
    if (cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(v)) != cudaSuccess) (void)cudaGetLastError();
    return v;
}

bool k3_decode_status_clear() {
    const uint32_t zero = 0u;
    if (cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(zero)) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return true;
}

namespace {

// One side stream and a fork / join event pair per device, created on first use
// (the one allocation-like step of the one-token path; never destroyed).
struct SideStream {
    cudaStream_t stream;
    cudaEvent_t fork, join;
};

SideStream *side_stream() {
    static std::mutex lock;
    static std::map<int, SideStream> made;
    int device = 0;
    (void)cudaGetDevice(&device);
    std::lock_guard<std::mutex> guard(lock);
    auto it = made.find(device);
    if (it != made.end()) return &it->second;
    SideStream s{};
    int least = 0, greatest = 0;
    if (cudaDeviceGetStreamPriorityRange(&least, &greatest) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    if (cudaStreamCreateWithPriority(&s.stream, cudaStreamNonBlocking, least) != cudaSuccess ||
        cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return &made.emplace(device, s).first->second;
}

}  // namespace

// Shapes the persistent one-token kernels handle; anything else takes the generic path.
bool k3_decode_supported(const k3_moe_layer_desc *d) {
    return d->hidden % 256u == 0 && d->expert_hidden % 128u == 0 && d->hidden % 128u == 0 &&
           d->expert_count <= 1024u && d->top_k <= 32u && d->hidden <= 8192u && d->shared_hidden <= 8192u &&
           (d->shared_hidden == 0 || (d->shared_hidden % 128u == 0 && d->q8_block % 32u == 0)) &&
           (size_t)(d->top_k + 1u) * d->expert_hidden * 2u + 512u <= 200u * 1024u &&
           ((d->hidden / 32u) % 2u == 0) && ((d->expert_hidden / 32u) % 2u == 0);
}

// One token's routed experts with the routing given (ids on the device, rank order): act
// [top_k, I] and rows_out [top_k, hidden] through the block-scaled expert kernel.  False for
// shapes it does not take (the caller runs the grouped kernels instead).
bool k3_decode_experts_token(const k3_moe_layer_desc *d, const void *x, const void *ids, void *act, void *rows_out,
                             void *scratch, size_t scratch_bytes, cudaStream_t stream) {
    if (scratch == nullptr || !k3_decode_mx_supported(d) || d->top_k >= 32u || d->hidden % 32u != 0u ||
        scratch_bytes < k3_decode_mx_scratch_bytes(d)) {
        return false;
    }
    uint8_t *x_terms = nullptr, *x_sf = nullptr;
    k3_decode_mx_vector_scratch(d, scratch, (void **)&x_terms, (void **)&x_sf);
    decode_terms_kernel<<<(d->hidden / 32u + 7u) / 8u, 256, 0, stream>>>(
        (const uint16_t *)x, x_terms, x_sf, (uint32_t *)k3_decode_mx_control_words(d, scratch), d->hidden);
    if (!launch_ok()) return false;
    return k3_decode_mx_experts(d, const_cast<void *>(ids), nullptr, nullptr, act, rows_out, scratch, nullptr, nullptr,
                                0u, stream);
}

// buffers: see DecodeArgs; all caller-owned scratch carved from the layer workspace
bool k3_decode_layer(const k3_moe_layer_desc *d, const void *x, void *logits, void *ids,
                     void *weights, void *sh_gate, void *sh_up, void *sh_act, void *sh_out,
                     void *act, void *rows_out, void *out, const void *residual, void *scratch,
                     size_t scratch_bytes, void *const *events, cudaStream_t stream, bool combine) {
    // optional phase events: [1], [2] after the front kernel, [3] after gate/up,
    // [4] after down (the caller records [0] before and [5] after the call)
    auto mark = [&](int index) {
        return !events || !events[index] ||
               cudaEventRecord((cudaEvent_t)events[index], stream) == cudaSuccess;
    };
    DecodeArgs a{};
    a.d = *d;
    a.x = (const uint16_t *)x;
    a.logits = (float *)logits;
    a.ids = (uint32_t *)ids;
    a.weights = (float *)weights;
    a.sh_gate = (uint16_t *)sh_gate;
    a.sh_up = (uint16_t *)sh_up;
    a.sh_act = (uint16_t *)sh_act;
    a.sh_out = (uint16_t *)sh_out;
    a.act = (uint16_t *)act;
    a.rows_out = (uint16_t *)rows_out;
    const int sms = sm_count();
    const bool mx = scratch != nullptr && k3_decode_mx_supported(d) && d->top_k < 32u &&
                    scratch_bytes >= k3_decode_mx_scratch_bytes(d);
    if (mx) {
        k3_decode_mx_vector_scratch(d, scratch, (void **)&a.x_terms, (void **)&a.x_sf);
        a.route_words = (float *)k3_decode_mx_route_words(d, scratch);
        a.control = (uint32_t *)k3_decode_mx_control_words(d, scratch);
        a.route_elsewhere = 1u;
    }
    static std::atomic<uint32_t> next_ticket{0};
    // address of the ticket array on the current device (looked up once per device)
    static std::mutex ticket_lock;
    static std::map<int, unsigned int *> ticket_base;
    unsigned int *tickets = nullptr;
    {
        int device = 0;
        (void)cudaGetDevice(&device);
        std::lock_guard<std::mutex> guard(ticket_lock);
        auto it = ticket_base.find(device);
        if (it == ticket_base.end()) {
            if (cudaGetSymbolAddress((void **)&tickets, g_front_tickets) != cudaSuccess) {
                (void)cudaGetLastError();
                return false;
            }
            ticket_base[device] = tickets;
        } else {
            tickets = it->second;
        }
    }
    a.ticket = tickets + next_ticket.fetch_add(1u) % kTicketSlots;
    // rows by 16-byte copies: the table and the token 16-byte aligned, whole 16-byte chunks per row
    const bool router_kernel = mx && d->shared_hidden != 0 && d->hidden % 8u == 0 &&
                               ((((uintptr_t)d->router_weight) | ((uintptr_t)x)) & 15u) == 0;
    // The shared expert depends only on the token.  Main form (ring path): a ring kernel on a
    // few SMs (k3_decode_shared.cu), all on the caller's stream: ring kernel (lets its
    // successors start at once) -> router kernel (programmatic launch, never waits for the ring
    // kernel, counts its finished blocks) -> expert kernel (programmatic launch, waits for that
    // count) -> tail kernel (programmatic launch, waits for everything in front).  Other
    // shapes: two row kernels on a low-priority side stream, and with every expert in this
    // table no tail launch - the down epilogue warps and the shared-down blocks count arrivals
    // per 32 output columns and the last one adds them up.
    const bool ring = router_kernel && k3_decode_shared_ring_supported(d) && k3_decode_shared_ring_ctas() != 0u &&
                      ((((uintptr_t)sh_gate) | ((uintptr_t)sh_up)) & 15u) == 0;
    const bool whole_tail = combine && mx && d->local_expert_first == 0u &&
                            d->local_expert_count == d->expert_count && d->hidden % 32u == 0u;
    const bool tail_kernel = ring && whole_tail;
    const bool fused_tail = whole_tail && !ring;
    static std::atomic<uint32_t> tail_epoch{1};
    if (fused_tail) {
        a.tail.out = (uint16_t *)out;
        a.tail.rows = (const uint16_t *)rows_out;
        a.tail.weights = (const float *)weights;
        a.tail.shared = d->shared_hidden ? (const uint16_t *)sh_out : nullptr;
        a.tail.residual = (const uint16_t *)residual;
        a.tail.count = (uint32_t *)k3_decode_mx_tail_words(d, scratch);
        a.tail.epoch = tail_epoch.fetch_add(1u) & 0xffffffu;
        a.tail.expected = d->top_k + (d->shared_hidden ? 2u : 0u);     // + two 16-column shared blocks
        a.tail.ranks = d->top_k;
        a.tail.hidden = d->hidden;
    }
    uint32_t ring_ctas = 0;
    if (ring) {
        a.front_done = (uint32_t *)k3_decode_mx_front_done_word(d, scratch);
        if (!k3_decode_shared_ring(d, x, sh_gate, sh_up, sh_out, a.front_done, stream)) {
            return false;
        }
        ring_ctas = k3_decode_shared_ring_ctas();
    }
    SideStream *side = nullptr;
    if (mx && d->shared_hidden != 0 && !ring) {
        side = side_stream();
        if (!side) return false;
        a.shared_elsewhere = 1u;
        // the side stream may start once everything queued before this call is done
        if (cudaEventRecord(side->fork, stream) != cudaSuccess ||
            cudaStreamWaitEvent(side->stream, side->fork, 0) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
    }
    const uint32_t front_tasks = d->expert_count + (side ? 0u : 2u * d->shared_hidden / 16u) +
                                 (mx ? (d->hidden / 32u + 7u) / 8u : 0u);
    // fp32 copy of the token; with the shared rows in the kernel also two f16 slots (the
    // second stays zero).  Without them four blocks fit on an SM and the grid is one wave.
    const size_t front_smem = (size_t)d->hidden * (side ? 4u : 8u);
    auto launch_side = [&]() -> bool {
        const size_t gu_smem = (size_t)d->hidden * 2u;
        const size_t dn_smem = (size_t)d->shared_hidden * 6u;
        if (!set_max_dynamic_smem((const void *)decode_shared_gateup_kernel, gu_smem) ||
            !set_max_dynamic_smem((const void *)decode_shared_down_kernel, dn_smem) ||
            !prefer_max_shared_carveout((const void *)decode_shared_gateup_kernel) ||
            !prefer_max_shared_carveout((const void *)decode_shared_down_kernel)) {
            return false;
        }
        decode_shared_gateup_kernel<<<std::min<uint32_t>(2u * d->shared_hidden / 16u, (uint32_t)sms), 256, gu_smem,
                                      side->stream>>>(a);
        decode_shared_down_kernel<<<d->hidden / 16u, 128, dn_smem, side->stream>>>(a);
        if (!launch_ok() || cudaEventRecord(side->join, side->stream) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
        return true;
    };
    uint32_t router_blocks = 0;
    if (router_kernel) {
        // two blocks on every SM the ring kernel leaves free, each with as many rows in flight
        // as one pass over the table needs (fewer, and more passes, if shared memory says so)
        const uint32_t grid = std::min<uint32_t>(d->expert_count, ((uint32_t)sms - ring_ctas) * 2u);
        uint32_t batch = std::min<uint32_t>((d->expert_count + grid - 1u) / grid, kRouterRowsInFlight);
        while (batch > 1u && (size_t)d->hidden * (4u + 2u * batch) + 8u * 1024u > 113u * 1024u) batch--;
        a.rows_in_flight = batch;
        const size_t smem = (size_t)d->hidden * (4u + 2u * batch);
        if (!set_max_dynamic_smem((const void *)decode_router_kernel, smem) ||
            !prefer_max_shared_carveout((const void *)decode_router_kernel)) {
            return false;
        }
        // behind the ring kernel with programmatic serialization and without waiting for it
        // (nothing here reads its results)
        cudaLaunchConfig_t config{};
        config.gridDim = dim3(grid);
        config.blockDim = dim3(256);
        config.dynamicSmemBytes = smem;
        config.stream = stream;
        cudaLaunchAttribute attribute{};
        attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute.val.programmaticStreamSerializationAllowed = 1;
        config.attrs = &attribute;
        config.numAttrs = ring ? 1u : 0u;
        router_blocks = config.gridDim.x;
        if (cudaLaunchKernelEx(&config, decode_router_kernel, a) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
    } else if (side) {
        if (!set_max_dynamic_smem((const void *)decode_front_kernel<false>, front_smem) ||
            !prefer_max_shared_carveout((const void *)decode_front_kernel<false>)) {
            return false;
        }
        decode_front_kernel<false><<<std::min<uint32_t>(front_tasks, (uint32_t)sms * 4u - 1u) + (mx ? 0u : 1u), 256,
                                     front_smem, stream>>>(a);
    } else {
        if (!set_max_dynamic_smem((const void *)decode_front_kernel<true>, front_smem)) return false;
        decode_front_kernel<true><<<std::min<uint32_t>(front_tasks, (uint32_t)sms * 2u - 1u) + 1u, 256, front_smem,
                                    stream>>>(a);
    }
    if (!launch_ok()) return false;
    // after the front kernel in launch order (measured: the order makes no difference);
    // the side stream has the lowest priority and fills what the critical path leaves free
    if (side && !launch_side()) return false;
    if (!mark(1) || !mark(2)) return false;
    if (mx) {
        k3_decode_tail tail{out, weights, a.tail.shared, residual, a.tail.epoch, a.tail.expected};
        if (!k3_decode_mx_experts(d, ids, weights, a.route_words, act, rows_out, scratch, events ? events[3] : nullptr,
                                  fused_tail ? &tail : nullptr, ring ? router_blocks : 0u, stream) ||
            !mark(4)) {
            return false;
        }
        // what follows on the caller's stream also follows the shared expert
        if (side && cudaStreamWaitEvent(stream, side->join, 0) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
        if (fused_tail || !combine) return true;
        if (tail_kernel) {
            DecodeTail t{};
            t.out = (uint16_t *)out;
            t.rows = (const uint16_t *)rows_out;
            t.weights = (const float *)weights;
            t.shared = (const uint16_t *)sh_out;
            t.residual = (const uint16_t *)residual;
            t.ranks = d->top_k;
            t.hidden = d->hidden;
            cudaLaunchConfig_t config{};
            config.gridDim = dim3((d->hidden / 32u + 3u) / 4u);
            config.blockDim = dim3(128);
            config.stream = stream;
            cudaLaunchAttribute attribute{};
            attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attribute.val.programmaticStreamSerializationAllowed = 1;
            config.attrs = &attribute;
            config.numAttrs = 1u;
            if (cudaLaunchKernelEx(&config, decode_tail_kernel, t) != cudaSuccess) {
                (void)cudaGetLastError();
                return false;
            }
            return true;
        }
        return k3_moe_combine_residual(out, rows_out, nullptr, weights, d->shared_hidden ? sh_out : nullptr,
                                       residual, 1u, d->top_k, d->hidden, stream);
    }
    size_t smem = (size_t)2 * d->hidden * sizeof(__half) + (2 + 2 * kDecodeWarps) * sizeof(float);
    if (!set_max_dynamic_smem((const void *)decode_gateup_kernel, smem)) return false;
    decode_gateup_kernel<<<sms, kDecodeThreads, smem, stream>>>(a);
    if (!launch_ok() || !mark(3)) return false;
    smem = (size_t)(d->top_k + 1u) * d->expert_hidden * sizeof(__half) + (34 + 2 * kDecodeWarps) * sizeof(float);
    if (!set_max_dynamic_smem((const void *)decode_down_kernel, smem)) return false;
    decode_down_kernel<<<sms, kDecodeThreads, smem, stream>>>(a);
    if (!launch_ok() || !mark(4)) return false;
    if (!combine) return true;
    return k3_moe_combine_residual(out, rows_out, nullptr, weights, d->shared_hidden ? sh_out : nullptr,
                                   residual, 1u, d->top_k, d->hidden, stream);
}
