// Top-k routing of one token by a whole thread block from the per-expert scores the
// router rows left in memory: choice = sigmoid(logit) + bias decides (larger first,
// lower expert id on ties, k3_rocm_ops.cu:1385-1450 / tests/test_k3_moe_smoke.cu:215-253),
// weight = score / (1e-20 + sum of the selected scores in rank order) * scale.
// Two levels of arg-max rounds on order keys (0 = none): warps 0..7 each own 128
// experts, four per lane, and list their top_k best; then the 8 * top_k listed
// candidates rank themselves by counting who beats them.
#pragma once

#include "k3_common.cuh"

namespace k3 {

// float -> unsigned key with the same order (-0 is folded into +0 first)
K3_DEVINL uint32_t route_order_key(float f) {
    const uint32_t b = __float_as_uint(f + 0.0f);
    return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
}

struct RouteScratch {          // shared memory, 10.5 KB
    float score[1024], choice[1024];
    uint32_t list_key[8 * 32], list_id[8 * 32];
    uint32_t cand_key[256], cand_id[256];
};

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
    __syncthreads();
    if (warp < 8u) {
        uint32_t key[4];
#pragma unroll
        for (uint32_t j = 0; j < 4u; j++) {
            const uint32_t e = warp * 128u + j * 32u + lane;
            key[j] = e < experts ? route_order_key(rs.choice[e]) : 0u;
        }
        for (uint32_t rank = 0; rank < top_k; rank++) {
            uint32_t best_key = key[0], best_slot = 0u;
#pragma unroll
            for (uint32_t j = 1; j < 4u; j++) {
                if (key[j] > best_key) { best_key = key[j]; best_slot = j; }
            }
            const uint32_t top = __reduce_max_sync(0xffffffffu, best_key);
            const uint32_t id = warp * 128u + best_slot * 32u + lane;
            const uint32_t win = __reduce_min_sync(0xffffffffu, (top != 0u && best_key == top) ? id : 0xffffffffu);
            if (lane == 0) {
                rs.list_key[warp * 32u + rank] = top;
                rs.list_id[warp * 32u + rank] = win;
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
    const uint32_t n = 8u * top_k;                                  // <= 256
    uint32_t my_key = 0u, my_id = 0xffffffffu;
    if (threadIdx.x < n) {
        const uint32_t src = (threadIdx.x / top_k) * 32u + threadIdx.x % top_k;
        my_key = rs.list_key[src];
        my_id = rs.list_id[src];
    }
    if (threadIdx.x < 256u) {
        rs.cand_key[threadIdx.x] = my_key;
        rs.cand_id[threadIdx.x] = my_id;
    }
    if (threadIdx.x < 32u) {
        ids_s[threadIdx.x] = 0xffffffffu;
        weights_s[threadIdx.x] = 0.f;
    }
    __syncthreads();
    if (threadIdx.x < n && my_key != 0u) {
        uint32_t rank = 0u;
#pragma unroll 8
        for (uint32_t u = 0; u < n; u++) {
            const uint32_t ok = rs.cand_key[u], oi = rs.cand_id[u];
            rank += (ok > my_key || (ok == my_key && oi < my_id)) ? 1u : 0u;
        }
        if (rank < top_k) {
            ids_s[rank] = my_id;
            weights_s[rank] = rs.score[my_id];                      // the raw score for now
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
