// Tail of the one-token layer without a kernel of its own:
//   out = bf16( bf16( bf16(sum_r w_r * row_r) + shared ) + residual )
// per 32-column group, formed by whichever warp delivers the group's last input -
// the top_k expert rows come from the down kernel's epilogue warps, the shared
// expert's columns from the shared-down kernel on another stream.  Nobody waits:
// a producer stores its part, fences, counts its arrival, and the one that sees
// the full count reads all parts (from L2) and writes the columns.  The sum runs
// in rank order, so the result does not depend on who is last.
#pragma once

#include "k3_common.cuh"

namespace k3 {

struct DecodeTail {
    uint16_t *out;              // bf16 [hidden]; null: no tail
    const uint16_t *rows;       // bf16 [ranks, hidden] expert rows in rank order
    const float *weights;       // f32 [ranks]
    const uint16_t *shared;     // bf16 [hidden] or null
    const uint16_t *residual;   // bf16 [hidden] or null
    uint32_t *count;            // [hidden / 32] arrival words
    uint32_t epoch;             // 24 bits, unique per layer call
    uint32_t expected;          // arrivals per group: ranks (+ shared blocks per group)
    uint32_t ranks, hidden;
};

// Counts an arrival in a word that carries the call's epoch in its upper 24 bits:
// a word left by an earlier call (or by whatever used the memory before) reads as
// zero arrivals, so the words need no clearing before first use (the arrival that
// completes a group clears the word again).  Returns the arrivals including this
// one, or 0 if the update did not go through in 1024 attempts (a few dozen warps
// at most contend for a word).
K3_DEVINL uint32_t count_arrival(uint32_t *word, uint32_t epoch24) {
    uint32_t seen = *reinterpret_cast<volatile uint32_t *>(word);
    for (uint32_t attempt = 0; attempt < 1024u; attempt++) {
        const uint32_t next = (seen >> 8) == epoch24 ? seen + 1u : ((epoch24 << 8) | 1u);
        const uint32_t prev = atomicCAS(word, seen, next);
        if (prev == seen) return next & 0xffu;
        seen = prev;
    }
    return 0u;
}

// The 32 output columns of `group` from parts that are complete in memory (whole warp).
K3_DEVINL void tail_columns(const DecodeTail &t, uint32_t group, uint32_t lane) {
    const uint32_t col = group * 32u + lane;
    // eight rows in flight at a time, summed in rank order
    float acc = 0.f;
    for (uint32_t r0 = 0; r0 < t.ranks; r0 += 8u) {
        uint16_t v[8];
        float w[8];
#pragma unroll
        for (uint32_t j = 0; j < 8u; j++) {
            const uint32_t r = min(r0 + j, t.ranks - 1u);
            v[j] = __ldcg(t.rows + (uint64_t)r * t.hidden + col);
            w[j] = __ldcg(t.weights + r);
        }
#pragma unroll
        for (uint32_t j = 0; j < 8u; j++) {
            if (r0 + j < t.ranks) acc = fmaf(w[j], bf16_bits_to_float(v[j]), acc);
        }
    }
    uint16_t bits = float_to_bf16_bits(acc);
    if (t.shared != nullptr)
        bits = float_to_bf16_bits(bf16_bits_to_float(bits) + bf16_bits_to_float(__ldcg(t.shared + col)));
    if (t.residual != nullptr)
        bits = float_to_bf16_bits(bf16_bits_to_float(__ldcg(t.residual + col)) + bf16_bits_to_float(bits));
    t.out[col] = bits;
}

// Whole warp, after its stores to the group's inputs.  False if the count failed.
K3_DEVINL bool tail_arrive(const DecodeTail &t, uint32_t group, uint32_t lane) {
    __threadfence();
    __syncwarp();
    uint32_t arrivals = 0u;
    if (lane == 0) arrivals = count_arrival(t.count + group, t.epoch);
    arrivals = __shfl_sync(0xffffffffu, arrivals, 0);
    if (arrivals == 0u) return false;
    if (arrivals != t.expected) return true;
    __threadfence();
    tail_columns(t, group, lane);
    // Last toucher of the group's word: leave it at zero, so that the same call
    // replayed with the same epoch (a captured graph launched again) counts from
    // zero like a fresh one instead of finding the full count of its last run.
    __syncwarp();
    if (lane == 0) atomicExch(t.count + group, 0u);
    return true;
}

}  // namespace k3
