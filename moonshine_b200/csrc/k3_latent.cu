// The routed layer at the model's real shape: the experts work on a latent
// vector narrower than the model width.
//
//   ids, w      = router(x)                                     x: [T, hidden]
//   latent      = routed_expert_down_proj(x)                    Q8 [latent, hidden]
//   rows        = experts(latent rows grouped by expert)        MXFP4, width latent
//   routed      = sum_r w[r] * rows[r]                          [T, latent]
//   routed_full = routed_expert_up_proj(rms_norm(routed))       Q8 [hidden, latent]
//   out         = routed_full + shared_expert(x)
//
// This is the sequence of the reference's decode_routed_layer
// (k3_engine.cu:1668-1671 latent projection, :1851-1863 weighted sum / norm /
// routed up, :1889-1893 add of the shared output) and of prefill_routed_layer
// (k3_engine_prefill.inc:1525-1590), composed from the same kernels as
// k3_moe_layer_forward: no host round trip, device dispatch, grouped expert GEMMs.
#include "k3_common.cuh"
#include "k3_grouped.h"
#include "k3_moe_layer.h"
#include "k3_moe_ops.h"

#include <cstring>

using namespace k3;

namespace {

struct LatentWorkspace {
    float *logits;
    uint32_t *ids, *offsets, *sorted_route, *sorted_token, *inv_perm;
    float *weights;
    void *dispatch_ws;
    size_t dispatch_bytes;
    uint16_t *latent, *rows_in, *act, *rows_out, *routed, *routed_norm, *routed_full;
    uint16_t *sh_gate, *sh_up, *sh_act, *sh_out;
    void *mx_ws, *sh_ws, *proj_w;
    uint16_t *token_act;           // one token through the one-token expert kernel: activation rows
    void *token_scratch;           //   and the kernel's scratch (null: that kernel does not take the shape)
    size_t token_scratch_bytes;
    size_t mx_bytes, sh_bytes, total;
};

k3_moe_layer_desc expert_view(const k3_moe_latent_desc *d) {
    k3_moe_layer_desc e = d->layer;
    e.hidden = d->latent;           // expert tables are [local, I, latent/2] and [local, latent, I/2]
    e.shared_hidden = 0;
    return e;
}

bool latent_ok(const k3_moe_latent_desc *d) {
    return d && d->latent != 0 && d->latent % 32u == 0 && d->layer.hidden % 32u == 0 && d->down_q && d->down_s &&
           d->norm_weight && d->up_q && d->up_s && d->norm_epsilon > 0.0f && d->layer.q8_block != 0 &&
           d->layer.hidden % d->layer.q8_block == 0 && d->latent % d->layer.q8_block == 0;
}

LatentWorkspace carve(const k3_moe_latent_desc *d, uint32_t tokens, void *base) {
    LatentWorkspace w{};
    char *p = (char *)base;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        char *q = base ? p + off : nullptr;
        off += (bytes + 255u) & ~(size_t)255u;
        return (void *)q;
    };
    const k3_moe_layer_desc &l = d->layer;
    const k3_moe_layer_desc e = expert_view(d);
    const uint64_t routes = (uint64_t)tokens * l.top_k;
    const size_t H = l.hidden, L = d->latent, I = l.expert_hidden, S = l.shared_hidden;
    w.logits = (float *)take((size_t)tokens * l.expert_count * sizeof(float));
    w.ids = (uint32_t *)take(routes * 4u);
    w.weights = (float *)take(routes * 4u);
    w.offsets = (uint32_t *)take((size_t)(l.expert_count + 1u) * 4u);
    w.sorted_route = (uint32_t *)take(routes * 4u);
    w.sorted_token = (uint32_t *)take(routes * 4u);
    w.inv_perm = (uint32_t *)take(routes * 4u);
    w.dispatch_bytes = k3_moe_dispatch_workspace_bytes(tokens, l.top_k, l.expert_count);
    w.dispatch_ws = take(w.dispatch_bytes);
    w.latent = (uint16_t *)take((size_t)tokens * L * 2u);
    w.rows_out = (uint16_t *)take(routes * L * 2u);
    w.routed = (uint16_t *)take((size_t)tokens * L * 2u);
    w.routed_norm = (uint16_t *)take((size_t)tokens * L * 2u);
    w.routed_full = (uint16_t *)take((size_t)tokens * H * 2u);
    w.proj_w = tokens >= 32u ? take(H * L * 2u) : nullptr;      // bf16 copy of one projection table
    w.mx_bytes = k3_grouped_mx_supported(&e, (uint32_t)routes)
                     ? k3_grouped_mx_workspace_bytes(&e, (uint32_t)routes, tokens) : 0;
    w.mx_ws = take(w.mx_bytes);
    if (tokens == 1u && k3_decode_mx_supported(&e) && e.top_k < 32u) {
        w.token_act = (uint16_t *)take(routes * I * 2u);
        w.token_scratch_bytes = k3_decode_mx_scratch_bytes(&e) + 256u;
        w.token_scratch = take(w.token_scratch_bytes);
    }
    if (w.mx_bytes == 0) {              // fallback path gathers bf16 rows and keeps the activation
        w.rows_in = (uint16_t *)take(routes * L * 2u);
        w.act = (uint16_t *)take(routes * I * 2u);
    }
    if (S) {
        w.sh_gate = (uint16_t *)take((size_t)tokens * S * 2u);
        w.sh_up = (uint16_t *)take((size_t)tokens * S * 2u);
        w.sh_act = (uint16_t *)take((size_t)tokens * S * 2u);
        w.sh_out = (uint16_t *)take((size_t)tokens * H * 2u);
        w.sh_bytes = k3_grouped_shared_workspace_bytes(&l, tokens);
        w.sh_ws = take(w.sh_bytes);
    }
    w.total = off;
    return w;
}

}  // namespace

extern "C" size_t k3_moe_latent_workspace_bytes(const k3_moe_latent_desc *d, uint32_t tokens) {
    if (!latent_ok(d) || tokens == 0) return 0;
    return carve(d, tokens, nullptr).total;
}

extern "C" bool k3_moe_latent_layer_forward(const k3_moe_latent_desc *d, void *out, const void *x,
                                            uint32_t tokens, void *workspace, size_t workspace_bytes,
                                            void *ids_out, void *weights_out, void *stream_pointer) {
    if (!latent_ok(d) || !out || !x || !workspace || tokens == 0 || tokens > 65535u ||
        d->layer.local_expert_first != 0 || d->layer.local_expert_count != d->layer.expert_count) {
        return false;
    }
    const k3_moe_layer_desc &l = d->layer;
    const k3_moe_layer_desc e = expert_view(d);
    const LatentWorkspace w = carve(d, tokens, workspace);
    if (workspace_bytes < w.total) return false;
    cudaStream_t stream = (cudaStream_t)stream_pointer;
    const uint32_t routes = tokens * l.top_k;
    const uint32_t H = l.hidden, L = d->latent;

    // router on the full-width token, experts on the latent projection
    if (!k3_moe_route(&l, w.ids, w.weights, w.logits, x, tokens, stream)) return false;
    if (!(w.proj_w && k3_grouped_q8_dense_bf16(w.latent, d->down_q, d->down_s, x, tokens, L, H, l.q8_block,
                                               l.q8_scale_type, w.proj_w, stream)) &&
        !k3_grouped_q8_bf16(w.latent, d->down_q, d->down_s, x, tokens, L, H, l.q8_block, l.q8_scale_type,
                            stream)) {
        return false;
    }
    if (l.shared_hidden) {
        const bool ok = w.sh_bytes != 0
                            ? k3_grouped_shared_expert(&l, w.sh_out, w.sh_act, x, tokens, w.sh_ws, stream)
                            : k3_moe_shared_expert(&l, w.sh_out, w.sh_gate, w.sh_up, w.sh_act, x, tokens, stream);
        if (!ok) return false;
    }
    // one token: its 16 experts through the block-scaled one-token expert kernel on the latent
    // vector, rows in rank order (no dispatch); shapes that kernel refuses fall through
    const bool token_path = tokens == 1u && w.token_scratch != nullptr && workspace != nullptr &&
                            k3_decode_experts_token(&e, w.latent, w.ids, w.token_act, w.rows_out, w.token_scratch,
                                                    w.token_scratch_bytes, stream);
    if (token_path) {
        // nothing to group
    } else if (!k3_moe_dispatch_build(w.offsets, w.sorted_route, w.sorted_token, w.inv_perm, w.ids, tokens, l.top_k,
                                      l.expert_count, w.dispatch_ws, w.dispatch_bytes, stream)) {
        return false;
    }
    if (token_path) {
        // rows_out already holds the expert rows
    } else if (w.mx_bytes != 0) {
        if (!k3_grouped_mx_experts(&e, w.rows_out, nullptr, w.latent, w.sorted_token, tokens, w.offsets, routes,
                                   w.mx_ws, stream)) {
            return false;
        }
    } else {
        if (!k3_rocm_gather_rows_bf16(w.rows_in, w.latent, w.sorted_token, routes, L, stream) ||
            !k3_moe_experts_grouped(&e, w.rows_out, w.act, w.rows_in, w.offsets, routes, stream)) {
            return false;
        }
    }
    // weighted sum in rank order, norm, projection back to the model width, shared output
    if (!k3_moe_combine(w.routed, w.rows_out, token_path ? nullptr : w.inv_perm, w.weights, nullptr, tokens, l.top_k, L,
                        stream) ||
        !k3_rocm_rms_norm_bf16(w.routed_norm, w.routed, d->norm_weight, tokens, L, d->norm_epsilon, stream)) {
        return false;
    }
    void *full = l.shared_hidden ? (void *)w.routed_full : out;
    if (!(w.proj_w && k3_grouped_q8_dense_bf16(full, d->up_q, d->up_s, w.routed_norm, tokens, H, L, l.q8_block,
                                               l.q8_scale_type, w.proj_w, stream)) &&
        !k3_grouped_q8_bf16(full, d->up_q, d->up_s, w.routed_norm, tokens, H, L, l.q8_block, l.q8_scale_type,
                            stream)) {
        return false;
    }
    if (l.shared_hidden && !k3_rocm_add_bf16(out, w.routed_full, w.sh_out, (uint64_t)tokens * H, stream)) {
        return false;
    }
    if (ids_out && cudaMemcpyAsync(ids_out, w.ids, (size_t)routes * 4u, cudaMemcpyDefault, stream) != cudaSuccess) {
        return false;
    }
    if (weights_out &&
        cudaMemcpyAsync(weights_out, w.weights, (size_t)routes * 4u, cudaMemcpyDefault, stream) != cudaSuccess) {
        return false;
    }
    return true;
}
