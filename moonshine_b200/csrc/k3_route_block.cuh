// Top-k routing of one token by a whole thread block from the per-expert scores the
// router rows left in memory: choice = sigmoid(logit) + bias decides (larger first,
// lower expert id on ties, k3_rocm_ops.cu:1385-1450 / tests/test_k3_moe_smoke.cu:215-253),
// weight = score / (1e-20 + sum of the selected scores in rank order) * scale.
//
// Warps 0..7 each own 128 experts, four per lane, as order keys (0 = none).  A few arg-max
// rounds per warp give a threshold: with W fully populated warps and r = ceil(top_k / W), the
// r-th best key of every such warp is reached by at least top_k experts, so the smallest of
// them bounds the top_k-th best overall.  The experts at or above it (a few dozen of 896 for
// continuous scores) are compacted and rank themselves by counting who beats them.  If more
// than 256 pass (ties on a grand scale), the general method runs instead: every warp lists its
// top_k best in top_k rounds and the 8 * top_k listed candidates rank themselves.
#pragma once

#include "k3_common.cuh"

namespace k3 {

// float -> unsigned key with the same order (-0 is folded into +0 first)
K3_DEVINL uint32_t route_order_key(float f) {
    const uint32_t b = __float_as_uint(f + 0.0f);
    return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
}

struct RouteScratch {          // shared memory, 10.6 KB
    float score[1024], choice[1024];
    uint32_t list_key[8 * 32], list_id[8 * 32];
    uint32_t cand_key[256], cand_id[256];
    uint32_t warp_bound[8], passed;
};

// One arg-max round of a warp over its lanes' keys: the best key and, among the lanes that
// hold it, the lowest expert id.  The winning lane zeroes its key.
K3_DEVINL void route_round(uint32_t (&key)[4], uint32_t warp, uint32_t lane, uint32_t &top, uint32_t &win) {
    uint32_t best_key = key[0], best_slot = 0u;
#pragma unroll
    for (uint32_t j = 1; j < 4u; j++) {
        if (key[j] > best_key) { best_key = key[j]; best_slot = j; }
    }
    top = __reduce_max_sync(0xffffffffu, best_key);
    const uint32_t id = warp * 128u + best_slot * 32u + lane;
    win = __reduce_min_sync(0xffffffffu, (top != 0u && best_key == top) ? id : 0xffffffffu);
    if (win == id) {
#pragma unroll
        for (uint32_t j = 0; j < 4u; j++) {
            if (j == best_slot) key[j] = 0u;
        }
    }
}

// All threads of a block of at least 256 threads call this (it contains block barriers).
// route_words: f32 [2][1024] = scores, choices.  Results: ids_s / weights_s [top_k] in
// shared memory, valid after the call for every thread.
K3_DEVINL void route_topk_block(RouteScratch &rs, uint32_t *ids_s, float *weights_s, const float *route_words,
                                uint32_t experts, uint32_t top_k, float route_scale) {
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    {
        // all of a thread's loads in flight at once (blockDim >= 256: at most four experts each)
        float sc[4], ch[4];
#pragma unroll
        for (uint32_t j = 0; j < 4u; j++) {
            const uint32_t e = threadIdx.x + j * blockDim.x;
            sc[j] = e < experts ? __ldcg(route_words + e) : 0.f;
            ch[j] = e < experts ? __ldcg(route_words + 1024u + e) : 0.f;
        }
#pragma unroll
        for (uint32_t j = 0; j < 4u; j++) {
            const uint32_t e = threadIdx.x + j * blockDim.x;
            if (e < 1024u) {
                rs.score[e] = sc[j];
                rs.choice[e] = ch[j];
            }
        }
    }
    if (threadIdx.x == 0) rs.passed = 0u;
    if (threadIdx.x < 32u) {
        ids_s[threadIdx.x] = 0xffffffffu;
        weights_s[threadIdx.x] = 0.f;
    }
    __syncthreads();
    uint32_t key[4] = {0u, 0u, 0u, 0u};
    const uint32_t full_warps = max(experts / 128u, 1u);            // warps whose 128 experts all exist
    const uint32_t rounds = (top_k + full_warps - 1u) / full_warps;
    if (warp < 8u) {
#pragma unroll
        for (uint32_t j = 0; j < 4u; j++) {
            const uint32_t e = warp * 128u + j * 32u + lane;
            key[j] = e < experts ? route_order_key(rs.choice[e]) : 0u;
        }
        if (warp < full_warps) {
            uint32_t probe[4] = {key[0], key[1], key[2], key[3]}, top = 0u, win = 0u;
            for (uint32_t r = 0; r < rounds; r++) route_round(probe, warp, lane, top, win);
            if (lane == 0) rs.warp_bound[warp] = top;              // the warp's rounds-th best key (0: fewer exist)
        }
    }
    __syncthreads();
    if (warp < 8u) {
        uint32_t bound = 0xffffffffu;
        for (uint32_t w = 0; w < full_warps; w++) bound = min(bound, rs.warp_bound[w]);
#pragma unroll
        for (uint32_t j = 0; j < 4u; j++) {
            const bool pass = key[j] != 0u && key[j] >= bound;
            const uint32_t mask = __ballot_sync(0xffffffffu, pass);
            uint32_t base = 0u;
            if (lane == 0 && mask != 0u) base = atomicAdd(&rs.passed, (uint32_t)__popc(mask));
            base = __shfl_sync(0xffffffffu, base, 0);
            const uint32_t pos = base + (uint32_t)__popc(mask & ((1u << lane) - 1u));
            if (pass && pos < 256u) {
                rs.cand_key[pos] = key[j];
                rs.cand_id[pos] = warp * 128u + j * 32u + lane;
            }
        }
    }
    __syncthreads();
    uint32_t n = rs.passed;
    if (n > 256u) {
        // general method: top_k rounds per warp, then the listed candidates
        __syncthreads();                                            // everyone has read `passed` and the candidates
        if (warp < 8u) {
            for (uint32_t rank = 0; rank < top_k; rank++) {
                uint32_t top, win;
                route_round(key, warp, lane, top, win);
                if (lane == 0) {
                    rs.list_key[warp * 32u + rank] = top;
                    rs.list_id[warp * 32u + rank] = win;
                }
            }
        }
        __syncthreads();
        n = 8u * top_k;                                             // <= 256
        if (threadIdx.x < 256u) {
            const uint32_t src = (threadIdx.x / top_k) * 32u + threadIdx.x % top_k;
            rs.cand_key[threadIdx.x] = threadIdx.x < n ? rs.list_key[src] : 0u;
            rs.cand_id[threadIdx.x] = threadIdx.x < n ? rs.list_id[src] : 0xffffffffu;
        }
        __syncthreads();
    }
    if (threadIdx.x < n) {
        const uint32_t my_key = rs.cand_key[threadIdx.x], my_id = rs.cand_id[threadIdx.x];
        if (my_key != 0u) {
            uint32_t rank = 0u;
#pragma unroll 4
            for (uint32_t u = 0; u < n; u++) {
                const uint32_t ok = rs.cand_key[u], oi = rs.cand_id[u];
                rank += (ok > my_key || (ok == my_key && oi < my_id)) ? 1u : 0u;
            }
            if (rank < top_k) {
                ids_s[rank] = my_id;
                weights_s[rank] = rs.score[my_id];                  // the raw score for now
            }
        }
    }
    __syncthreads();
    if (warp == 0) {
        float denominator = 1e-20f;
        for (uint32_t r = 0; r < top_k; r++) denominator += weights_s[r];
        const float w = lane < top_k ? __fmul_rn(__fdiv_rn(weights_s[lane], denominator), route_scale) : 0.f;
        __syncwarp();
        if (lane < top_k) weights_s[lane] = w;
    }
    __syncthreads();
}

}  // namespace k3
