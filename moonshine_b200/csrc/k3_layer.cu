// Fused routed-MoE layer: slot table admission, routing, grouped expert
// products, shared expert, combine, and the single-GPU composition.
//
// Composition follows the reference engine's MoE section (decode:
// k3_engine.cu:1553-1909; layer-major prefill: k3_engine_prefill.inc:1448-1609
// and :938-997), with the experts consuming the hidden vector directly.  The
// host scans, D2H copies and per-expert stream synchronisations of the
// reference are replaced by device-side dispatch and one grouped launch per
// projection.
#include "k3_gemv.cuh"
#include "k3_grouped.h"
#include "k3_moe_layer.h"
#include "k3_moe_ops.h"

#include <algorithm>

using namespace k3;

namespace {

struct GroupedArgs {
    const uint8_t *w_a_packed;   // block 0 matrix slot table (gate / down)
    const uint8_t *w_a_scales;
    const uint8_t *w_b_packed;   // block 1 matrix slot table (up / down)
    const uint8_t *w_b_scales;
    const uint32_t *offsets;     // [local+1] row ranges, or nullptr in rank mode
    const uint32_t *rank_ids;    // rank mode: expert id per rank (row = rank)
    uint32_t first_local, local_count;
    uint32_t out_rows;           // rows of the weight matrix (I or d)
    uint32_t k, k_pad;
    uint32_t in_shared_row;      // 1: every row reads input row 0 (one-token decode)
    int activation;
    float beta, linear_beta;
};

// gate/up + activation: item = 16 gate rows (block 0) + the same 16 up rows
// (block 1) of one expert; loops over the expert's input rows two at a time.
template <bool kFuseAct>
__global__ void __launch_bounds__(kGemvThreads)
grouped_rows_kernel(uint16_t *__restrict__ out, const uint16_t *__restrict__ in, GroupedArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const GemvSmem sm = carve_gemv_smem(smem_raw, a.k_pad);
    uint32_t expert, row_begin, n;
    if (a.rank_ids != nullptr) {
        const uint32_t id = a.rank_ids[blockIdx.y];
        if (id < a.first_local || id >= a.first_local + a.local_count) return;
        expert = id - a.first_local;
        row_begin = blockIdx.y;
        n = 1u;
    } else {
        expert = blockIdx.y;
        row_begin = a.offsets[expert];
        n = a.offsets[expert + 1u] - row_begin;
        if (n == 0u) return;
    }
    const uint64_t packed_stride = (uint64_t)a.out_rows * (a.k / 2u);
    const uint64_t scale_stride = (uint64_t)a.out_rows * (a.k / 32u);
    const uint32_t rows_per_item = kFuseAct ? 16u : 32u;
    const uint32_t r0 = blockIdx.x * rows_per_item;
    RowBlock b0{a.w_a_packed + expert * packed_stride, a.w_a_scales + expert * scale_stride, r0,
                a.out_rows};
    RowBlock b1{a.w_b_packed + expert * packed_stride, a.w_b_scales + expert * scale_stride,
                kFuseAct ? r0 : r0 + 16u, a.out_rows};
    const uint32_t out_width = a.out_rows;
    for (uint32_t v0 = 0; v0 < n; v0 += 2u) {
        const uint32_t nvec = min(2u, n - v0);
        const uint64_t in0 = a.in_shared_row ? 0u : (uint64_t)(row_begin + v0);
        __syncthreads();
        stage_vectors_f16(sm.xs, sm.inv_scale, in + in0 * a.k,
                          nvec > 1u ? in + (in0 + 1u) * a.k : nullptr, a.k, a.k_pad, sm.scratch);
        mxfp4_item_2x16<true>(sm.out_s, sm.red, b0, b1, a.k, sm.xs, a.k_pad, nvec, sm.inv_scale);
        if (kFuseAct) {
            if (threadIdx.x < 32u) {
                const uint32_t vec = threadIdx.x >> 4, i = threadIdx.x & 15u;
                if (vec < nvec && r0 + i < a.out_rows) {
                    // gate and up are rounded to bf16 before the activation, as the
                    // reference stores them in bf16 buffers between the launches
                    const float g = bf16_bits_to_float(float_to_bf16_bits(sm.out_s[vec * 32u + i]));
                    const float u =
                        bf16_bits_to_float(float_to_bf16_bits(sm.out_s[vec * 32u + 16u + i]));
                    out[(uint64_t)(row_begin + v0 + vec) * out_width + r0 + i] =
                        float_to_bf16_bits(activation(g, u, a.activation, a.beta, a.linear_beta));
                }
            }
        } else {
            if (threadIdx.x < 64u) {
                const uint32_t vec = threadIdx.x >> 5, r = threadIdx.x & 31u;
                if (vec < nvec && r0 + r < a.out_rows) {
                    out[(uint64_t)(row_begin + v0 + vec) * out_width + r0 + r] =
                        float_to_bf16_bits(sm.out_s[vec * 32u + r]);
                }
            }
        }
    }
}

// out[t] = bf16( bf16( bf16(sum_r w[t,r] * rows[idx[t,r]]) + shared[t] ) + residual[t] )
// (shared and residual optional)
__global__ void __launch_bounds__(256)
combine_kernel(uint16_t *__restrict__ out, const uint16_t *__restrict__ rows,
               const uint32_t *__restrict__ index, const float *__restrict__ weights,
               const uint16_t *__restrict__ shared, const uint16_t *__restrict__ residual,
               uint32_t tokens, uint32_t top_k, uint32_t hidden) {
    __shared__ float w_s[32];
    __shared__ uint32_t idx_s[32];
    for (uint32_t token = blockIdx.x; token < tokens; token += gridDim.x) {
        __syncthreads();
        if (threadIdx.x < top_k) {
            const uint32_t route = token * top_k + threadIdx.x;
            w_s[threadIdx.x] = weights[route];
            idx_s[threadIdx.x] = index ? index[route] : route;
        }
        __syncthreads();
        for (uint32_t c = blockIdx.y * blockDim.x + threadIdx.x; c < hidden / 8u;
             c += gridDim.y * blockDim.x) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
            for (uint32_t r = 0; r < top_k; r++) {
                const uint4 q = reinterpret_cast<const uint4 *>(rows + (uint64_t)idx_s[r] * hidden)[c];
                const float w = w_s[r];
                acc[0] = fmaf(w, bf16_lo(q.x), acc[0]);
                acc[1] = fmaf(w, bf16_hi(q.x), acc[1]);
                acc[2] = fmaf(w, bf16_lo(q.y), acc[2]);
                acc[3] = fmaf(w, bf16_hi(q.y), acc[3]);
                acc[4] = fmaf(w, bf16_lo(q.z), acc[4]);
                acc[5] = fmaf(w, bf16_hi(q.z), acc[5]);
                acc[6] = fmaf(w, bf16_lo(q.w), acc[6]);
                acc[7] = fmaf(w, bf16_hi(q.w), acc[7]);
            }
            float sh[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (shared) {
                const uint4 q = reinterpret_cast<const uint4 *>(shared + (uint64_t)token * hidden)[c];
                sh[0] = bf16_lo(q.x); sh[1] = bf16_hi(q.x); sh[2] = bf16_lo(q.y); sh[3] = bf16_hi(q.y);
                sh[4] = bf16_lo(q.z); sh[5] = bf16_hi(q.z); sh[6] = bf16_lo(q.w); sh[7] = bf16_hi(q.w);
            }
            uint32_t res[4] = {0u, 0u, 0u, 0u};
            if (residual) {
                const uint4 q = reinterpret_cast<const uint4 *>(residual + (uint64_t)token * hidden)[c];
                res[0] = q.x; res[1] = q.y; res[2] = q.z; res[3] = q.w;
            }
            uint32_t r4[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint32_t lo = float_to_bf16_bits(acc[2 * j]);
                uint32_t hi = float_to_bf16_bits(acc[2 * j + 1]);
                if (shared) {
                    lo = float_to_bf16_bits(bf16_bits_to_float(lo) + sh[2 * j]);
                    hi = float_to_bf16_bits(bf16_bits_to_float(hi) + sh[2 * j + 1]);
                }
                if (residual) {
                    lo = float_to_bf16_bits(bf16_lo(res[j]) + bf16_bits_to_float(lo));
                    hi = float_to_bf16_bits(bf16_hi(res[j]) + bf16_bits_to_float(hi));
                }
                r4[j] = lo | (hi << 16);
            }
            reinterpret_cast<uint4 *>(out + (uint64_t)token * hidden)[c] =
                make_uint4(r4[0], r4[1], r4[2], r4[3]);
        }
    }
}

bool desc_ok(const k3_moe_layer_desc *d) {
    return d && d->hidden != 0 && d->hidden % 32u == 0 && d->expert_hidden != 0 &&
           d->expert_hidden % 32u == 0 && d->expert_count != 0 && d->expert_count <= 1024u &&
           d->top_k != 0 && d->top_k <= 32u && d->top_k <= d->expert_count &&
           d->route_scale > 0.0f && d->local_expert_count != 0 &&
           d->local_expert_first + d->local_expert_count <= d->expert_count &&
           (d->activation == K3_MOE_ACT_SITU || d->activation == K3_MOE_ACT_SWIGLU) &&
           (d->activation != K3_MOE_ACT_SITU || (d->beta > 0.0f && d->linear_beta > 0.0f));
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Workspace {
    float *logits;
    uint32_t *ids;
    float *weights;
    uint32_t *offsets, *sorted_route, *sorted_token, *inv_perm;
    void *dispatch_ws;
    size_t dispatch_bytes;
    void *mx_ws, *sh_ws, *decode_ws;
    size_t mx_bytes, sh_bytes, decode_bytes;
    uint16_t *rows_in, *act, *rows_out, *sh_gate, *sh_up, *sh_act, *sh_out;
    size_t total;
};

Workspace carve(const k3_moe_layer_desc *d, uint32_t tokens, void *base) {
    Workspace w{};
    char *p = (char *)base;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        char *q = base ? p + off : nullptr;
        off += align_up(bytes, 256);
        return (void *)q;
    };
    const uint64_t routes = (uint64_t)tokens * d->top_k;
    w.logits = (float *)take((size_t)tokens * d->expert_count * sizeof(float));
    w.ids = (uint32_t *)take(routes * sizeof(uint32_t));
    w.weights = (float *)take(routes * sizeof(float));
    w.offsets = (uint32_t *)take((size_t)(d->expert_count + 1) * sizeof(uint32_t));
    w.sorted_route = (uint32_t *)take(routes * sizeof(uint32_t));
    w.sorted_token = (uint32_t *)take(routes * sizeof(uint32_t));
    w.inv_perm = (uint32_t *)take(routes * sizeof(uint32_t));
    w.dispatch_bytes = k3_moe_dispatch_workspace_bytes(tokens, d->top_k, d->expert_count);
    w.dispatch_ws = take(w.dispatch_bytes);
    w.rows_in = (uint16_t *)take(routes * d->hidden * 2u);
    w.act = (uint16_t *)take(routes * d->expert_hidden * 2u);
    w.rows_out = (uint16_t *)take(routes * d->hidden * 2u);
    w.mx_bytes = k3_grouped_mx_supported(d, (uint32_t)routes)
                     ? k3_grouped_mx_workspace_bytes(d, (uint32_t)routes, tokens) : 0;
    w.mx_ws = take(w.mx_bytes);
    w.sh_bytes = k3_grouped_shared_workspace_bytes(d, tokens);
    w.sh_ws = take(w.sh_bytes);
    w.decode_bytes = tokens == 1u ? k3_decode_mx_scratch_bytes(d) : 0;
    w.decode_ws = take(w.decode_bytes);
    if (d->shared_hidden) {
        w.sh_gate = (uint16_t *)take((size_t)tokens * d->shared_hidden * 2u);
        w.sh_up = (uint16_t *)take((size_t)tokens * d->shared_hidden * 2u);
        w.sh_act = (uint16_t *)take((size_t)tokens * d->shared_hidden * 2u);
        w.sh_out = (uint16_t *)take((size_t)tokens * d->hidden * 2u);
    }
    w.total = off;
    return w;
}

// SIMT/mma.sync grouped path: any row count, weights re-streamed per row pair.
bool launch_grouped_rows(const k3_moe_layer_desc *d, void *rows_out, void *act,
                         const void *rows_in, const uint32_t *offsets, const uint32_t *rank_ids,
                         uint32_t groups_y, bool shared_row, cudaStream_t stream) {
    GroupedArgs a{};
    a.offsets = offsets;
    a.rank_ids = rank_ids;
    a.first_local = d->local_expert_first;
    a.local_count = d->local_expert_count;
    a.activation = d->activation;
    a.beta = d->beta;
    a.linear_beta = d->linear_beta;
    // gate/up + activation
    a.w_a_packed = (const uint8_t *)d->w1_packed;
    a.w_a_scales = (const uint8_t *)d->w1_scales;
    a.w_b_packed = (const uint8_t *)d->w3_packed;
    a.w_b_scales = (const uint8_t *)d->w3_scales;
    a.out_rows = d->expert_hidden;
    a.k = d->hidden;
    a.k_pad = (a.k + 127u) / 128u * 128u;
    a.in_shared_row = shared_row ? 1u : 0u;
    size_t smem = gemv_smem_bytes(a.k_pad);
    if (!set_max_dynamic_smem((const void *)grouped_rows_kernel<true>, smem)) return false;
    dim3 grid((d->expert_hidden + 15u) / 16u, groups_y);
    grouped_rows_kernel<true><<<grid, kGemvThreads, smem, stream>>>(
        (uint16_t *)act, (const uint16_t *)rows_in, a);
    if (!launch_ok()) return false;
    // down
    a.w_a_packed = a.w_b_packed = (const uint8_t *)d->w2_packed;
    a.w_a_scales = a.w_b_scales = (const uint8_t *)d->w2_scales;
    a.out_rows = d->hidden;
    a.k = d->expert_hidden;
    a.k_pad = (a.k + 127u) / 128u * 128u;
    a.in_shared_row = 0u;
    smem = gemv_smem_bytes(a.k_pad);
    if (!set_max_dynamic_smem((const void *)grouped_rows_kernel<false>, smem)) return false;
    grid = dim3((d->hidden + 31u) / 32u, groups_y);
    grouped_rows_kernel<false><<<grid, kGemvThreads, smem, stream>>>(
        (uint16_t *)rows_out, (const uint16_t *)act, a);
    return launch_ok();
}

bool slot_pointers_aligned(const k3_moe_layer_desc *d) {
    const uintptr_t all = (uintptr_t)d->w1_packed | (uintptr_t)d->w3_packed |
                          (uintptr_t)d->w2_packed;
    return (all & 15u) == 0 && d->w1_packed && d->w1_scales && d->w3_packed && d->w3_scales &&
           d->w2_packed && d->w2_scales;
}

}  // namespace

extern "C" const char *k3_moe_version(void) { return "k3moe-b200 0.1.0"; }

extern "C" bool k3_moe_store_admit(const k3_moe_layer_desc *d, uint32_t slot, const void *span,
                                   const uint64_t relative[6], void *stream_pointer) {
    if (!desc_ok(d) || !span || !relative || slot >= d->local_expert_count ||
        !slot_pointers_aligned(d)) {
        return false;
    }
    cudaStream_t stream = (cudaStream_t)stream_pointer;
    const size_t p13 = (size_t)d->expert_hidden * (d->hidden / 2u);
    const size_t s13 = (size_t)d->expert_hidden * (d->hidden / 32u);
    const size_t p2 = (size_t)d->hidden * (d->expert_hidden / 2u);
    const size_t s2 = (size_t)d->hidden * (d->expert_hidden / 32u);
    struct Copy { const void *table; size_t bytes; int rel; };
    const Copy copies[6] = {
        {d->w1_packed, p13, 0}, {d->w1_scales, s13, 1}, {d->w2_packed, p2, 2},
        {d->w2_scales, s2, 3},  {d->w3_packed, p13, 4}, {d->w3_scales, s13, 5},
    };
    for (const Copy &c : copies) {
        char *dst = (char *)c.table + (size_t)slot * c.bytes;
        if (cudaMemcpyAsync(dst, (const char *)span + relative[c.rel], c.bytes, cudaMemcpyDefault,
                            stream) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
    }
    return true;
}

extern "C" size_t k3_moe_layer_workspace_bytes(const k3_moe_layer_desc *d, uint32_t tokens) {
    if (!desc_ok(d) || tokens == 0) return 0;
    // a workspace sized for `tokens` also serves any smaller call, the one-token
    // sequence (which has scratch of its own) included
    return std::max(carve(d, tokens, nullptr).total, carve(d, 1u, nullptr).total);
}

extern "C" bool k3_moe_route(const k3_moe_layer_desc *d, void *expert_ids, void *expert_weights,
                             void *logits, const void *x, uint32_t tokens, void *stream) {
    if (!desc_ok(d) || !expert_ids || !expert_weights || !logits || !x || tokens == 0 ||
        !d->router_weight || !d->router_bias) {
        return false;
    }
    return k3_grouped_dense_bf16_f32(logits, d->router_weight, x, tokens, d->expert_count,
                                     d->hidden, stream) &&
           k3_rocm_router_topk_f32_batch(expert_ids, expert_weights, logits, d->router_bias,
                                         tokens, d->expert_count, d->top_k, d->route_scale,
                                         stream);
}

extern "C" bool k3_moe_experts_grouped(const k3_moe_layer_desc *d, void *rows_out, void *act,
                                       const void *rows_in, const void *offsets, uint32_t rows,
                                       void *stream) {
    if (!desc_ok(d) || !rows_out || !act || !rows_in || !offsets || rows == 0 ||
        !slot_pointers_aligned(d)) {
        return false;
    }
    if (k3_grouped_tc_supported(d, rows)) {
        return k3_grouped_tc_experts(d, rows_out, act, rows_in, offsets, rows, stream);
    }
    return launch_grouped_rows(d, rows_out, act, rows_in, (const uint32_t *)offsets, nullptr,
                               d->local_expert_count, false, (cudaStream_t)stream);
}

// One token with the routing given: the block-scaled one-token expert kernel, then the
// weighted sum in rank order.  Workspace: act | rows_out | the kernel's scratch.
extern "C" size_t k3_moe_experts_token_workspace_bytes(const k3_moe_layer_desc *d) {
    if (!desc_ok(d) || !slot_pointers_aligned(d) || !k3_decode_mx_supported(d) || d->top_k >= 32u) return 0;
    const size_t act = ((size_t)d->top_k * d->expert_hidden * 2u + 255u) & ~(size_t)255u;
    const size_t rows = ((size_t)d->top_k * d->hidden * 2u + 255u) & ~(size_t)255u;
    return act + rows + k3_decode_mx_scratch_bytes(d) + 512u;
}

extern "C" bool k3_moe_experts_token(const k3_moe_layer_desc *d, void *out, const void *x, const void *ids,
                                     const void *weights, void *workspace, size_t workspace_bytes, void *stream) {
    const size_t need = k3_moe_experts_token_workspace_bytes(d);
    if (need == 0 || !out || !x || !ids || !weights || !workspace || workspace_bytes < need) return false;
    uint8_t *p = (uint8_t *)(((uintptr_t)workspace + 255u) & ~(uintptr_t)255u);
    const size_t act_bytes = ((size_t)d->top_k * d->expert_hidden * 2u + 255u) & ~(size_t)255u;
    const size_t rows_bytes = ((size_t)d->top_k * d->hidden * 2u + 255u) & ~(size_t)255u;
    void *act = p, *rows_out = p + act_bytes, *scratch = p + act_bytes + rows_bytes;
    const size_t scratch_bytes = workspace_bytes - (size_t)((uint8_t *)scratch - (uint8_t *)workspace);
    if (!k3_decode_experts_token(d, x, ids, act, rows_out, scratch, scratch_bytes, (cudaStream_t)stream)) return false;
    return k3_moe_combine(out, rows_out, nullptr, weights, nullptr, 1u, d->top_k, d->hidden, stream);
}

extern "C" size_t k3_moe_experts_workspace_bytes(const k3_moe_layer_desc *d, uint32_t rows,
                                                 uint32_t source_rows) {
    if (!desc_ok(d) || rows == 0 || !slot_pointers_aligned(d) || !k3_grouped_mx_supported(d, rows)) return 0;
    return k3_grouped_mx_workspace_bytes(d, rows, source_rows);
}

extern "C" bool k3_moe_experts_grouped_ws(const k3_moe_layer_desc *d, void *rows_out, void *act,
                                          const void *rows_in, const void *index,
                                          uint32_t source_rows, const void *offsets,
                                          uint32_t rows, void *workspace, size_t workspace_bytes,
                                          void *stream) {
    if (!desc_ok(d) || !rows_out || !rows_in || !offsets || rows == 0 || !slot_pointers_aligned(d) ||
        (index != nullptr && source_rows == 0)) {
        return false;
    }
    const size_t need = k3_moe_experts_workspace_bytes(d, rows, index ? source_rows : 0u);
    if (need != 0 && workspace && workspace_bytes >= need) {
        return k3_grouped_mx_experts(d, rows_out, act, rows_in, index, source_rows, offsets, rows,
                                     workspace, (cudaStream_t)stream);
    }
    if (index || !act) return false;
    return k3_moe_experts_grouped(d, rows_out, act, rows_in, offsets, rows, stream);
}

extern "C" bool k3_moe_shared_expert(const k3_moe_layer_desc *d, void *out, void *gate, void *up,
                                     void *act, const void *x, uint32_t tokens, void *stream) {
    if (!desc_ok(d) || d->shared_hidden == 0 || !out || !gate || !up || !act || !x ||
        tokens == 0) {
        return false;
    }
    const uint32_t S = d->shared_hidden;
    return k3_grouped_q8_bf16(gate, d->shared_gate_q, d->shared_gate_s, x, tokens, S, d->hidden,
                              d->q8_block, d->q8_scale_type, stream) &&
           k3_grouped_q8_bf16(up, d->shared_up_q, d->shared_up_s, x, tokens, S, d->hidden,
                              d->q8_block, d->q8_scale_type, stream) &&
           k3_moe_activation_bf16(act, gate, up, (uint64_t)tokens * S, d->activation, d->beta,
                                  d->linear_beta, stream) &&
           k3_grouped_q8_bf16(out, d->shared_down_q, d->shared_down_s, act, tokens, d->hidden, S,
                              d->q8_block, d->q8_scale_type, stream);
}

extern "C" size_t k3_moe_shared_workspace_bytes(const k3_moe_layer_desc *d, uint32_t tokens) {
    if (!desc_ok(d) || tokens == 0) return 0;
    return k3_grouped_shared_workspace_bytes(d, tokens);
}

extern "C" bool k3_moe_shared_expert_ws(const k3_moe_layer_desc *d, void *out, void *act, const void *x,
                                        uint32_t tokens, void *workspace, size_t workspace_bytes,
                                        void *stream) {
    if (!desc_ok(d) || d->shared_hidden == 0 || !out || !act || !x || tokens == 0 || !workspace) return false;
    const size_t need = k3_grouped_shared_workspace_bytes(d, tokens);
    if (need == 0 || workspace_bytes < need) return false;
    return k3_grouped_shared_expert(d, out, act, x, tokens, workspace, (cudaStream_t)stream);
}

extern "C" bool k3_moe_combine_residual(void *out, const void *rows, const void *index,
                                        const void *weights, const void *shared, const void *residual,
                                        uint32_t tokens, uint32_t top_k, uint32_t hidden, void *stream) {
    if (!out || !rows || !weights || tokens == 0 || top_k == 0 || top_k > 32u || hidden == 0 ||
        hidden % 8u != 0) {
        return false;
    }
    if ((((uintptr_t)out | (uintptr_t)rows | (uintptr_t)shared | (uintptr_t)residual) & 15u) != 0) return false;
    // few tokens: spread the columns of a token over several small CTAs
    const bool few = tokens < 128u;
    const uint32_t threads = few ? 64u : 256u;
    const dim3 grid(std::min<uint32_t>(tokens, (uint32_t)sm_count() * 8u),
                    few ? (hidden / 8u + threads - 1u) / threads : 1u);
    combine_kernel<<<grid, threads, 0, (cudaStream_t)stream>>>(
        (uint16_t *)out, (const uint16_t *)rows, (const uint32_t *)index, (const float *)weights,
        (const uint16_t *)shared, (const uint16_t *)residual, tokens, top_k, hidden);
    return launch_ok();
}

extern "C" bool k3_moe_combine(void *out, const void *rows, const void *index, const void *weights,
                               const void *shared, uint32_t tokens, uint32_t top_k, uint32_t hidden,
                               void *stream) {
    return k3_moe_combine_residual(out, rows, index, weights, shared, nullptr, tokens, top_k, hidden, stream);
}

namespace {

bool mark(void *const *events, int index, cudaStream_t stream) {
    if (!events || !events[index]) return true;
    return cudaEventRecord((cudaEvent_t)events[index], stream) == cudaSuccess;
}

bool layer_forward_impl(const k3_moe_layer_desc *d, void *out, const void *x, uint32_t tokens,
                        void *workspace, size_t workspace_bytes, void *ids_out,
                        void *weights_out, void *const *events, const void *residual,
                        void *stream_pointer) {
    if (!desc_ok(d) || !out || !x || tokens == 0 || tokens > 65535u || !workspace ||
        d->local_expert_first != 0 || d->local_expert_count != d->expert_count ||
        !slot_pointers_aligned(d)) {
        return false;
    }
    const Workspace w = carve(d, tokens, workspace);
    if (workspace_bytes < w.total) return false;
    cudaStream_t stream = (cudaStream_t)stream_pointer;
    const uint32_t routes = tokens * d->top_k;

    if (!mark(events, 0, stream)) return false;
    const uint32_t *index = nullptr;
    const bool one_token = tokens == 1u && k3_decode_supported(d);
    if (one_token) {
        // one token: persistent matrix-vector kernels, rows stay in rank order, the
        // combine is part of the sequence
        // (phase events there: front | gate/up | down | tail)
        if (!k3_decode_layer(d, x, w.logits, w.ids, w.weights, w.sh_gate, w.sh_up, w.sh_act,
                             w.sh_out, w.act, w.rows_out, out, residual, w.decode_ws, w.decode_bytes,
                             events, stream)) {
            return false;
        }
    } else {
        if (!k3_moe_route(d, w.ids, w.weights, w.logits, x, tokens, stream)) return false;
        if (!mark(events, 1, stream)) return false;
        if (d->shared_hidden &&
            !(w.sh_bytes != 0
                  ? k3_grouped_shared_expert(d, w.sh_out, w.sh_act, x, tokens, w.sh_ws, stream)
                  : k3_moe_shared_expert(d, w.sh_out, w.sh_gate, w.sh_up, w.sh_act, x, tokens, stream))) {
            return false;
        }
        if (!mark(events, 2, stream)) return false;
        if (tokens == 1u) {
            if (!mark(events, 3, stream)) return false;
            if (!launch_grouped_rows(d, w.rows_out, w.act, x, nullptr, w.ids, d->top_k, true, stream)) {
                return false;
            }
        } else {
            if (!k3_moe_dispatch_build(w.offsets, w.sorted_route, w.sorted_token, w.inv_perm, w.ids,
                                       tokens, d->top_k, d->expert_count, w.dispatch_ws,
                                       w.dispatch_bytes, stream)) {
                return false;
            }
            if (w.mx_bytes != 0) {
                // block-scaled path: tokens are converted once, then gathered as bytes
                if (!mark(events, 3, stream)) return false;
                if (!k3_grouped_mx_experts(d, w.rows_out, nullptr, x, w.sorted_token, tokens, w.offsets,
                                           routes, w.mx_ws, stream)) {
                    return false;
                }
            } else {
                if (!k3_rocm_gather_rows_bf16(w.rows_in, x, w.sorted_token, routes, d->hidden, stream)) {
                    return false;
                }
                if (!mark(events, 3, stream)) return false;
                if (!k3_moe_experts_grouped(d, w.rows_out, w.act, w.rows_in, w.offsets, routes, stream)) {
                    return false;
                }
            }
            index = w.inv_perm;
        }
    }
    if (!one_token && !mark(events, 4, stream)) return false;
    if (!one_token &&
        !k3_moe_combine_residual(out, w.rows_out, index, w.weights, d->shared_hidden ? w.sh_out : nullptr,
                                 residual, tokens, d->top_k, d->hidden, stream)) {
        return false;
    }
    if (!mark(events, 5, stream)) return false;
    if (ids_out && cudaMemcpyAsync(ids_out, w.ids, (size_t)routes * 4u, cudaMemcpyDefault,
                                   stream) != cudaSuccess) {
        return false;
    }
    if (weights_out && cudaMemcpyAsync(weights_out, w.weights, (size_t)routes * 4u,
                                       cudaMemcpyDefault, stream) != cudaSuccess) {
        return false;
    }
    return true;
}

}  // namespace

extern "C" bool k3_moe_layer_forward(const k3_moe_layer_desc *d, void *out, const void *x,
                                     uint32_t tokens, void *workspace, size_t workspace_bytes,
                                     void *ids_out, void *weights_out, void *stream) {
    return layer_forward_impl(d, out, x, tokens, workspace, workspace_bytes, ids_out, weights_out,
                              nullptr, nullptr, stream);
}

extern "C" bool k3_moe_layer_forward_events(const k3_moe_layer_desc *d, void *out, const void *x,
                                            uint32_t tokens, void *workspace,
                                            size_t workspace_bytes, void *const *events,
                                            void *stream) {
    return layer_forward_impl(d, out, x, tokens, workspace, workspace_bytes, nullptr, nullptr,
                              events, nullptr, stream);
}

// The layer with the step either side of it: post-attention RMSNorm in front (its
// output feeds router, shared expert and experts) and the residual add behind, the
// latter inside the combine kernel.  (k3_engine.cu:1550-1553 norm, :1889-1897 adds.)
extern "C" size_t k3_moe_block_workspace_bytes(const k3_moe_layer_desc *d, uint32_t tokens) {
    const size_t inner = k3_moe_layer_workspace_bytes(d, tokens);
    return inner ? inner + align_up((size_t)tokens * d->hidden * 2u, 256) + 256u : 0;
}

extern "C" bool k3_moe_block_forward(const k3_moe_layer_desc *d, void *out, const void *hidden_in,
                                     const void *norm_weight, float epsilon, uint32_t tokens,
                                     void *workspace, size_t workspace_bytes, void *stream) {
    if (!desc_ok(d) || !out || !hidden_in || !norm_weight || !workspace || tokens == 0 || !(epsilon > 0.0f)) {
        return false;
    }
    const size_t need = k3_moe_block_workspace_bytes(d, tokens);
    if (need == 0 || workspace_bytes < need) return false;
    char *base = (char *)(((uintptr_t)workspace + 255u) & ~(uintptr_t)255u);
    void *normed = base;
    char *inner = base + align_up((size_t)tokens * d->hidden * 2u, 256);
    const size_t inner_bytes = workspace_bytes - (size_t)(inner - (char *)workspace);
    return k3_rocm_rms_norm_bf16(normed, hidden_in, norm_weight, tokens, d->hidden, epsilon, stream) &&
           layer_forward_impl(d, out, normed, tokens, inner, inner_bytes, nullptr, nullptr, nullptr, hidden_in,
                              stream);
}

// Device-timed phase ledger under the reference's field names.
extern "C" bool k3_moe_phase_stats_add(k3_moe_phase_stats *stats, void *const *events) {
    if (!stats || !events) return false;
    for (int i = 0; i < 6; i++) {
        if (!events[i]) return false;
    }
    if (cudaEventSynchronize((cudaEvent_t)events[5]) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    float ms[5];
    for (int i = 0; i < 5; i++) {
        if (cudaEventElapsedTime(&ms[i], (cudaEvent_t)events[i], (cudaEvent_t)events[i + 1]) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
    }
    stats->router_seconds += 1e-3 * ms[0];
    stats->shared_expert_seconds += 1e-3 * ms[1];
    stats->routed_index_seconds += 1e-3 * ms[2];
    stats->routed_expert_pipeline_seconds += 1e-3 * ms[3];
    stats->moe_tail_seconds += 1e-3 * (ms[1] + ms[4]);
    stats->layer_passes += 1u;
    return true;
}

// Thin wrappers so a host language without CUDA runtime bindings can own the
// events it hands to k3_moe_layer_forward_events.
extern "C" void *k3_moe_event_create(void) {
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return (void *)e;
}

extern "C" void k3_moe_event_destroy(void *event) {
    if (event) (void)cudaEventDestroy((cudaEvent_t)event);
}

extern "C" float k3_moe_event_elapsed_ms(void *begin, void *end) {
    float ms = -1.0f;
    if (!begin || !end || cudaEventSynchronize((cudaEvent_t)end) != cudaSuccess ||
        cudaEventElapsedTime(&ms, (cudaEvent_t)begin, (cudaEvent_t)end) != cudaSuccess) {
        (void)cudaGetLastError();
        return -1.0f;
    }
    return ms;
}
