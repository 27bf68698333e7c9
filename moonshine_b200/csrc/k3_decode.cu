// One-token (decode) routed-MoE layer: four launches, no host round trip.
//
//   front    router logits (896 BF16 rows), shared-expert gate/up rows (Q8), one
//            warp per weight row in the reference reduction order, and the
//            token's two-term E4M3 form; the last block to finish routes the
//            token (sigmoid + bias top-k) and applies the shared activation
//   gate/up  the top_k selected experts' gate and up rows + activation
//            (+ the shared expert's down rows on spare warps)
//   down     the selected experts' down rows
//   combine  weighted sum in rank order + shared output
//
// It replaces the per-token sequence of the reference's decode_routed_layer
// (k3_engine.cu:1554-1563 router, :1668-1689 static projections, :1032-1066
// launch_expert x 16, :1851-1897 tail), which needs three host synchronisations
// and ~70 launches per layer.
//
// The expert kernels are persistent: a CTA stages the activation vector(s) in
// shared memory once (as f16 after an exact power-of-two rescale), then each
// warp streams whole 16-row blocks of MXFP4 weights over the full K extent with
// a three-deep register prefetch, converts nibbles to f16 with byte-permute
// lookups and accumulates per 32-column scale group on mma.sync (see
// k3_gemv.cuh for the fragment layout).  No cross-warp reduction is needed.
#include "k3_gemv.cuh"
#include "k3_grouped.h"
#include "k3_rowdot.cuh"
#include "k3_moe_layer.h"
#include "k3_moe_ops.h"

#include <algorithm>
#include <atomic>

#include <cuda_fp8.h>

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
    uint8_t *x_hl, *x_sf;     // front: two-term E4M3 form of x ([2, hidden], [hidden/32]) or null
    unsigned int *ticket;     // front: completion counter of this call
};

// ------------------------------------------------------------------- front
// Tickets of the "last block finishes the job" step of the front kernel.  A call
// takes the next slot round-robin, the last block of the grid resets it, so calls
// running at once on different streams do not share a counter unless more than
// kTicketSlots of them are in flight.
constexpr uint32_t kTicketSlots = 64;
__device__ unsigned int g_front_tickets[kTicketSlots];

// float -> unsigned key with the same order (-0 is folded into +0 first)
K3_DEVINL uint32_t order_key(float f) {
    const uint32_t b = __float_as_uint(f + 0.0f);
    return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
}

// Block of 32 values (one per lane) -> two E4M3 terms and the E8M0 block scale:
// value = 2^(scale - 127) * (hi + lo).
K3_DEVINL void split_block(float val, uint8_t &hi, uint8_t &lo, uint8_t &scale_byte) {
    const float mx = warp_max(fabsf(val));
    int e = 0;
    if (mx > 0.f && mx < 3.0e38f) e = (int)((__float_as_uint(mx) >> 23) & 0xffu) - 127 - 7;
    e = max(-127, min(127, e));
    const float scaled = val * __uint_as_float((uint32_t)(127 - e) << 23);      // |scaled| < 256
    hi = __nv_cvt_float_to_fp8(scaled, __NV_SATFINITE, __NV_E4M3);
    const float hi_f = __half2float(__half(__nv_cvt_fp8_to_halfraw(hi, __NV_E4M3)));
    lo = __nv_cvt_float_to_fp8(scaled - hi_f, __NV_SATFINITE, __NV_E4M3);
    scale_byte = (uint8_t)(e + 127);
}

// One warp per task: router rows, shared-expert gate and up rows (reference
// reduction order), and the 32-column blocks of the token's two-term E4M3 form.
// The last block to finish then routes the token (sigmoid + bias top-k in the
// reference's order: larger choice first, lower expert id on ties) and applies the
// shared expert's activation.
__global__ void __launch_bounds__(256)
decode_front_kernel(DecodeArgs a) {
    __shared__ float choice_s[1024], score_s[1024];
    __shared__ float top_score[32];
    __shared__ uint32_t top_id[32];
    __shared__ uint32_t is_last;
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t warps = (gridDim.x * blockDim.x) / kWarp;
    const uint32_t E = a.d.expert_count, S = a.d.shared_hidden, H = a.d.hidden, k = a.d.top_k;
    const uint32_t split_tasks = a.x_hl ? H / 32u : 0u;
    const uint32_t tasks = E + 2u * S + split_tasks;
    const uint32_t blocks_per_row = S ? H / a.d.q8_block : 0u;
    for (uint32_t task = (blockIdx.x * blockDim.x + threadIdx.x) / kWarp; task < tasks; task += warps) {
        if (task < E) {
            const float v = bf16_row_dot_exact((const uint16_t *)a.d.router_weight + (uint64_t)task * H,
                                               a.x, H, lane);
            if (lane == 0) a.logits[task] = v;
        } else if (task < E + 2u * S) {
            const uint32_t r = task - E;
            const bool up = r >= S;
            const uint32_t row = up ? r - S : r;
            const int8_t *q = (const int8_t *)(up ? a.d.shared_up_q : a.d.shared_gate_q);
            const void *sc = up ? a.d.shared_up_s : a.d.shared_gate_s;
            const float v = q8_row_dot_exact(q + (uint64_t)row * H, sc, (uint64_t)row * blocks_per_row,
                                             a.x, H, a.d.q8_block, a.d.q8_scale_type, lane);
            if (lane == 0) (up ? a.sh_up : a.sh_gate)[row] = float_to_bf16_bits(v);
        } else {
            const uint32_t blk = task - E - 2u * S;
            uint8_t hi, lo, sb;
            split_block(bf16_bits_to_float(a.x[blk * 32u + lane]), hi, lo, sb);
            a.x_hl[blk * 32u + lane] = hi;
            a.x_hl[H + blk * 32u + lane] = lo;
            if (lane == 0) a.x_sf[blk] = sb;
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int ticket = atomicAdd(a.ticket, 1u);
        is_last = ticket == gridDim.x - 1u ? 1u : 0u;
    }
    __syncthreads();
    if (is_last == 0u) return;
    __threadfence();
    if (threadIdx.x == 0) *a.ticket = 0u;
    // ---- routing and shared activation: results of the other blocks come from L2
    for (uint32_t e = threadIdx.x; e < 1024u; e += blockDim.x) {
        float sc = 0.f, ch = 0.f;
        if (e < E) {
            sc = sigmoid_exact(__ldcg(a.logits + e));
            ch = sc + ((const float *)a.d.router_bias)[e];
        }
        score_s[e] = sc;
        choice_s[e] = ch;
    }
    __syncthreads();
    if (warp == 0) {
        // lane owns experts lane, lane + 32, ...; its best candidate is cached
        const uint32_t slots = (E + 31u) / 32u;
        uint32_t best_key = 0u, best_id = 0xffffffffu;
        for (uint32_t i = 0; i < slots; i++) {
            const uint32_t e = i * 32u + lane;
            if (e < E) {
                const uint32_t key = order_key(choice_s[e]);
                if (best_id == 0xffffffffu || key > best_key) { best_key = key; best_id = e; }
            }
        }
        for (uint32_t rank = 0; rank < k; rank++) {
            const uint32_t has = best_id != 0xffffffffu ? 1u : 0u;
            const uint32_t top = __reduce_max_sync(0xffffffffu, has ? best_key : 0u);
            const uint32_t any = __reduce_max_sync(0xffffffffu, has);
            const uint32_t cand = (has && best_key == top) ? best_id : 0xffffffffu;
            const uint32_t win = any ? __reduce_min_sync(0xffffffffu, cand) : 0xffffffffu;
            if (lane == 0) {
                top_id[rank] = win;
                top_score[rank] = win != 0xffffffffu ? score_s[win] : 0.f;
            }
            if (win != 0xffffffffu && (win & 31u) == lane) {
                // winner leaves the pool; rescan this lane's candidates
                choice_s[win] = __uint_as_float(0x7fc00000u);       // marks "taken"
                best_key = 0u;
                best_id = 0xffffffffu;
                for (uint32_t i = 0; i < slots; i++) {
                    const uint32_t e = i * 32u + lane;
                    if (e >= E) continue;
                    const float c = choice_s[e];
                    if (__float_as_uint(c) == 0x7fc00000u) continue;
                    const uint32_t key = order_key(c);
                    if (best_id == 0xffffffffu || key > best_key) { best_key = key; best_id = e; }
                }
            }
        }
        __syncwarp();
        float denominator = 1e-20f;
        for (uint32_t r = 0; r < k; r++) denominator += top_score[r];
        if (lane < k) {
            a.ids[lane] = top_id[lane];
            a.weights[lane] = __fmul_rn(__fdiv_rn(top_score[lane], denominator), a.d.route_scale);
        }
    } else {
        for (uint32_t i = threadIdx.x - kWarp; i < S; i += blockDim.x - kWarp) {
            a.sh_act[i] = float_to_bf16_bits(activation(bf16_bits_to_float(__ldcg(a.sh_gate + i)),
                                                        bf16_bits_to_float(__ldcg(a.sh_up + i)),
                                                        a.d.activation, a.d.beta, a.d.linear_beta));
        }
    }
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

bool set_smem(const void *kernel, size_t smem) {
    if (smem <= 48 * 1024) return true;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return true;
}

}  // namespace

// Shapes the persistent one-token kernels handle; anything else takes the generic path.
bool k3_decode_supported(const k3_moe_layer_desc *d) {
    return d->hidden % 256u == 0 && d->expert_hidden % 128u == 0 && d->hidden % 128u == 0 &&
           d->expert_count <= 1024u && d->top_k <= 32u &&
           (d->shared_hidden == 0 || (d->shared_hidden % 8u == 0 && d->q8_block % 8u == 0)) &&
           (size_t)(d->top_k + 1u) * d->expert_hidden * 2u + 512u <= 200u * 1024u &&
           ((d->hidden / 32u) % 2u == 0) && ((d->expert_hidden / 32u) % 2u == 0);
}

// buffers: see DecodeArgs; all caller-owned scratch carved from the layer workspace
bool k3_decode_layer(const k3_moe_layer_desc *d, const void *x, void *logits, void *ids,
                     void *weights, void *sh_gate, void *sh_up, void *sh_act, void *sh_out,
                     void *act, void *rows_out, void *scratch, size_t scratch_bytes,
                     cudaStream_t stream) {
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
    const bool mx = scratch != nullptr && k3_decode_mx_supported(d) &&
                    scratch_bytes >= k3_decode_mx_scratch_bytes(d);
    if (mx) k3_decode_mx_vector_scratch(d, scratch, (void **)&a.x_hl, (void **)&a.x_sf);
    static std::atomic<uint32_t> next_ticket{0};
    unsigned int *tickets = nullptr;
    if (cudaGetSymbolAddress((void **)&tickets, g_front_tickets) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    a.ticket = tickets + next_ticket.fetch_add(1u) % kTicketSlots;
    const uint32_t front_tasks = d->expert_count + 2u * d->shared_hidden + (mx ? d->hidden / 32u : 0u);
    decode_front_kernel<<<std::min<uint32_t>((front_tasks + 7u) / 8u, (uint32_t)sms * 8u), 256, 0, stream>>>(a);
    if (!launch_ok()) return false;
    if (mx) {
        return k3_decode_mx_experts(d, ids, act, rows_out, sh_act, sh_out, scratch, stream);
    }
    size_t smem = (size_t)2 * d->hidden * sizeof(__half) + (2 + 2 * kDecodeWarps) * sizeof(float);
    if (!set_smem((const void *)decode_gateup_kernel, smem)) return false;
    decode_gateup_kernel<<<sms, kDecodeThreads, smem, stream>>>(a);
    if (!launch_ok()) return false;
    smem = (size_t)(d->top_k + 1u) * d->expert_hidden * sizeof(__half) + (34 + 2 * kDecodeWarps) * sizeof(float);
    if (!set_smem((const void *)decode_down_kernel, smem)) return false;
    decode_down_kernel<<<sms, kDecodeThreads, smem, stream>>>(a);
    return launch_ok();
}
