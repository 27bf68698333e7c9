/*
 * Fused routed-MoE layer entry points (CUDA, sm_100a).
 *
 * These have no one-to-one counterpart in the reference: they replace the
 * *sequences* of operator calls, host scans, copies and stream
 * synchronisations that the reference engine issues per layer -
 * decode_routed_layer (k3_engine.cu:1553-1909) and prefill_routed_layer /
 * prefill_stream_routed_layer / launch_prefill_expert
 * (k3_engine_prefill.inc:938-997, 1137-1243, 1448-1609) - with device-resident
 * routing, dispatch and grouped expert products.  Conventions are those of
 * k3_moe_ops.h: caller-owned device pointers, a cudaStream_t as void *,
 * bool return, no allocation, no synchronisation.
 *
 * The routed experts live in a caller-allocated slot table: six contiguous
 * arrays holding `local_expert_count` experts, the expert-parallel shard
 * [local_expert_first, local_expert_first + local_expert_count) of the
 * layer's `expert_count` experts.  It takes the place of the reference's
 * per-layer LRU cache slots fed from NVMe (k3_expert_cache.h:43-58,
 * k3_engine.cu:1696-1822): every expert of the shard is resident.
 */
#ifndef K3_MOE_LAYER_H
#define K3_MOE_LAYER_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct k3_moe_layer_desc {
    uint32_t hidden;               /* d: router / expert input and output width   */
    uint32_t expert_hidden;        /* I: routed expert intermediate width          */
    uint32_t expert_count;         /* E: experts of the layer (<= 1024)            */
    uint32_t top_k;                /* <= 32                                        */
    uint32_t shared_hidden;        /* shared expert intermediate width, 0 = none   */
    uint32_t q8_block;             /* shared expert quantisation block (32, 128)   */
    int32_t  q8_scale_type;        /* K3_MOE_Q8_SCALE_F32 / _F16                   */
    int32_t  activation;           /* K3_MOE_ACT_SITU / _SWIGLU                    */
    float    beta;                 /* SiTU only                                    */
    float    linear_beta;          /* SiTU only                                    */
    float    route_scale;          /* router weight scaling factor (> 0)           */
    uint32_t local_expert_first;   /* first expert held in the slot table          */
    uint32_t local_expert_count;   /* experts held in the slot table               */
    const void *router_weight;     /* bf16 [E, d]                                  */
    const void *router_bias;       /* f32  [E]                                     */
    const void *w1_packed;         /* u8 [local, I, d/2]   gate                    */
    const void *w1_scales;         /* u8 [local, I, d/32]                          */
    const void *w3_packed;         /* u8 [local, I, d/2]   up                      */
    const void *w3_scales;         /* u8 [local, I, d/32]                          */
    const void *w2_packed;         /* u8 [local, d, I/2]   down                    */
    const void *w2_scales;         /* u8 [local, d, I/32]                          */
    const void *shared_gate_q;     /* i8 [S, d]                                    */
    const void *shared_gate_s;     /* scale [S, d/q8_block]                        */
    const void *shared_up_q;
    const void *shared_up_s;
    const void *shared_down_q;     /* i8 [d, S]                                    */
    const void *shared_down_s;     /* scale [d, S/q8_block]                        */
} k3_moe_layer_desc;

/* Copy one expert's six tensors into slot `slot` of the table described by
 * `desc`.  `span` points at the expert's contiguous checkpoint span (host or
 * device memory) and relative[i] are the byte offsets of w1.packed, w1.scale,
 * w2.packed, w2.scale, w3.packed, w3.scale inside it - the order and meaning
 * of k3_engine_expert_layout.relative (k3_engine.cu:105-114, 1038-1065).
 * Source offsets need no alignment. */
bool k3_moe_store_admit(const k3_moe_layer_desc *desc, uint32_t slot,
                        const void *span, const uint64_t relative[6],
                        void *stream);

/* Bytes of device workspace the layer entry points need for `tokens` rows. */
size_t k3_moe_layer_workspace_bytes(const k3_moe_layer_desc *desc,
                                    uint32_t tokens);

/* Token-to-expert dispatch (replaces the host scan of
 * k3_engine_prefill.inc:1175-1194): from expert_ids u32 [tokens, top_k] build
 * offsets u32 [experts+1], and for every sorted position p: sorted_route[p] =
 * token*top_k+rank, sorted_token[p] = token; inv_perm[route] = p.  Order:
 * expert ascending, route ascending inside an expert.  Every id must be
 * < experts; an id that is not raises bit 1 of k3_moe_device_status(). */
size_t k3_moe_dispatch_workspace_bytes(uint32_t tokens, uint32_t top_k,
                                       uint32_t experts);
bool k3_moe_dispatch_build(void *offsets, void *sorted_route,
                           void *sorted_token, void *inv_perm,
                           const void *expert_ids, uint32_t tokens,
                           uint32_t top_k, uint32_t experts, void *workspace,
                           size_t workspace_bytes, void *stream);

/* Dispatch without a caller workspace.  No counterpart in the reference.
 * For hosts that may not allocate device memory (a plugin inside an engine
 * that carved all of its memory at start-up, or a call made while allocation
 * is off limits): the per-chunk histograms live in a fixed array of about
 * 1 MiB inside the library's device image, present once on every GPU that
 * loads the library until the process exits.  Same outputs as
 * k3_moe_dispatch_build.  Limits: tokens*top_k <= 131072 (also returned by
 * k3_moe_dispatch_noalloc_max_routes) and experts <= 1024; anything larger
 * returns false with a message in `error` (optional, NUL-terminated) and
 * launches nothing.  All calls on a GPU share the array: calls whose kernels
 * may overlap on the GPU race and must be serialised by the caller.  The
 * first call on each GPU resolves the array's device address and should be
 * made outside stream capture.  Never calls cudaMalloc or cudaFree. */
size_t k3_moe_dispatch_noalloc_max_routes(void);
bool k3_moe_dispatch_build_noalloc(void *offsets, void *sorted_route,
                                   void *sorted_token, void *inv_perm,
                                   const void *expert_ids, uint32_t tokens,
                                   uint32_t top_k, uint32_t experts,
                                   char *error, size_t error_size,
                                   void *stream);

/* Router for `tokens` rows: logits f32 [tokens, E] (scratch, caller-owned),
 * ids u32 / weights f32 [tokens, top_k].  Replaces the pair
 * k3_rocm_bf16_gemm_f32 + k3_rocm_router_topk_f32_batch
 * (k3_engine_prefill.inc:1448-1460). */
bool k3_moe_route(const k3_moe_layer_desc *desc, void *expert_ids,
                  void *expert_weights, void *logits, const void *x,
                  uint32_t tokens, void *stream);

/* Grouped expert products over rows already grouped by expert: rows_in bf16
 * [rows, d] where rows [offsets[e], offsets[e+1]) belong to local expert e
 * (offsets has local_expert_count+1 u32 entries on the device).  Computes
 * gate, up, activation and down for every row (replaces the per-expert
 * sequence of launch_prefill_expert, k3_engine_prefill.inc:956-990) and
 * writes rows_out bf16 [rows, d] in the same order.  `act` is scratch bf16
 * [rows, I]. */
bool k3_moe_experts_grouped(const k3_moe_layer_desc *desc, void *rows_out,
                            void *act, const void *rows_in,
                            const void *offsets, uint32_t rows, void *stream);

/* The same products on the block-scaled tensor-core path, which needs device
 * scratch for the two-term E4M3 form of the rows and of the activation:
 * k3_moe_experts_workspace_bytes(desc, rows, source_rows) bytes (0 when the
 * layer shape or row count does not suit the path).  `index` (u32 per row on
 * the device, or NULL) gathers rows_in: product row r reads rows_in[index[r]]
 * and rows_in has source_rows rows, which folds gather_rows_bf16
 * (k3_engine_prefill.inc:1203) into the conversion; with index NULL pass
 * source_rows 0.  `act` may be NULL on this path.  Falls back to
 * k3_moe_experts_grouped when workspace is NULL or too small, index is NULL
 * and act is given; fails otherwise. */
size_t k3_moe_experts_workspace_bytes(const k3_moe_layer_desc *desc, uint32_t rows,
                                      uint32_t source_rows);
bool k3_moe_experts_grouped_ws(const k3_moe_layer_desc *desc, void *rows_out,
                               void *act, const void *rows_in, const void *index,
                               uint32_t source_rows, const void *offsets,
                               uint32_t rows, void *workspace,
                               size_t workspace_bytes, void *stream);

/* One token whose routing the host brings (the partially resident store plans
 * on the host, k3_engine.cu:1580-1590): ids u32 [top_k] on the device index the
 * descriptor's expert tables (slot numbers for a slot table), weights f32
 * [top_k] on the device -> out bf16 [hidden] = the weighted sum of the expert
 * rows in rank order.  Runs the block-scaled one-token expert kernel (three
 * launches).  k3_moe_experts_token_workspace_bytes returns 0 for shapes that
 * kernel does not take; the caller then uses dispatch + k3_moe_experts_grouped
 * + k3_moe_combine. */
size_t k3_moe_experts_token_workspace_bytes(const k3_moe_layer_desc *desc);
bool k3_moe_experts_token(const k3_moe_layer_desc *desc, void *out, const void *x, const void *ids,
                          const void *weights, void *workspace, size_t workspace_bytes, void *stream);

/* Shared expert for `tokens` rows: out bf16 [tokens, d]; gate/up/act are
 * scratch bf16 [tokens, S] (k3_engine_prefill.inc:1530-1551). */
bool k3_moe_shared_expert(const k3_moe_layer_desc *desc, void *out, void *gate,
                          void *up, void *act, const void *x, uint32_t tokens,
                          void *stream);

/* The same with the three Q8 tables converted to bf16 once per call into device
 * scratch (k3_moe_shared_workspace_bytes(desc, tokens) bytes, 0 when the shape
 * or token count does not suit the path), so that the products run as plain bf16
 * tensor-core GEMMs with the activation fused into the gate/up epilogue; `act`
 * is scratch bf16 [tokens, S].  Fails when the workspace is missing or too
 * small (k3_moe_shared_expert needs none). */
size_t k3_moe_shared_workspace_bytes(const k3_moe_layer_desc *desc, uint32_t tokens);
bool k3_moe_shared_expert_ws(const k3_moe_layer_desc *desc, void *out, void *act,
                             const void *x, uint32_t tokens, void *workspace,
                             size_t workspace_bytes, void *stream);

/* Combine: out[t] = bf16( bf16(sum_r weights[t,r] * rows[index[t*top_k+r]])
 * + shared[t] ), r ascending; index == NULL means the identity; shared ==
 * NULL skips the add (k3_engine_prefill.inc:1575-1580, 1598-1603). */
bool k3_moe_combine(void *out, const void *rows, const void *index,
                    const void *weights, const void *shared, uint32_t tokens,
                    uint32_t top_k, uint32_t hidden, void *stream);

/* The same with a residual row added last: out = bf16(residual + bf16(routed +
 * shared)), the two adds of k3_engine.cu:1889-1897 inside the combine kernel.
 * `residual` bf16 [tokens, d] may be NULL. */
bool k3_moe_combine_residual(void *out, const void *rows, const void *index,
                             const void *weights, const void *shared,
                             const void *residual, uint32_t tokens,
                             uint32_t top_k, uint32_t hidden, void *stream);

/* Whole layer on one GPU holding every expert (local range == all experts):
 * x bf16 [tokens, d] -> out bf16 [tokens, d].  `workspace` must hold
 * k3_moe_layer_workspace_bytes(desc, tokens).  When ids_out / weights_out are
 * non-NULL the routing decision is copied there (u32 / f32 [tokens, top_k]). */
bool k3_moe_layer_forward(const k3_moe_layer_desc *desc, void *out,
                          const void *x, uint32_t tokens, void *workspace,
                          size_t workspace_bytes, void *ids_out,
                          void *weights_out, void *stream);

/* Same as k3_moe_layer_forward, recording caller-created cudaEvent_t handles
 * (as void *, NULL entries skipped) on `stream` at the phase boundaries:
 * events[0] start, [1] router done, [2] shared expert done, [3] dispatch and
 * row gather done, [4] grouped expert products done, [5] combine done.  This is
 * the device-timed form of the reference's host phase ledger
 * (router_seconds, routed_expert_pipeline_seconds, moe_tail_seconds of
 * k3_engine_prefill_stats, k3_engine.h:69-99). */
bool k3_moe_layer_forward_events(const k3_moe_layer_desc *desc, void *out,
                                 const void *x, uint32_t tokens,
                                 void *workspace, size_t workspace_bytes,
                                 void *const *events, void *stream);

/* Phase ledger under the reference's field names (k3_engine_prefill_stats,
 * k3_engine.h:90-96), filled from the six events of one
 * k3_moe_layer_forward_events call; every call ADDS to the fields, as the
 * reference's host ledger does per layer (k3_engine_prefill.inc:1521, 1196,
 * 1224, 1624), so an engine can copy the sums into its own statistics.
 * Mapping: router_seconds = events 0->1; routed_index_seconds = 2->3 (dispatch
 * and row gather); routed_expert_pipeline_seconds = 3->4 (grouped expert
 * products); moe_tail_seconds = 1->2 + 4->5 (shared expert and combine, the
 * work the reference's tail interval spans); shared_expert_seconds = 1->2 on
 * its own.  Waits for events[5]; false if an event is missing or unrecorded. */
typedef struct k3_moe_phase_stats {
    double   router_seconds;
    double   routed_index_seconds;
    double   routed_expert_pipeline_seconds;
    double   moe_tail_seconds;
    double   shared_expert_seconds;
    uint64_t layer_passes;
} k3_moe_phase_stats;

bool k3_moe_phase_stats_add(k3_moe_phase_stats *stats, void *const *events);

/* The layer with the step either side of it: out = hidden_in + moe(rms_norm(hidden_in)).
 * The post-attention RMSNorm (k3_engine.cu:1550-1553) runs first and feeds router,
 * shared expert and experts; the residual add (k3_engine.cu:1889-1897) happens in
 * the combine kernel.  hidden_in bf16 [tokens, d], norm_weight bf16 [d]. */
size_t k3_moe_block_workspace_bytes(const k3_moe_layer_desc *desc, uint32_t tokens);
bool k3_moe_block_forward(const k3_moe_layer_desc *desc, void *out,
                          const void *hidden_in, const void *norm_weight,
                          float epsilon, uint32_t tokens, void *workspace,
                          size_t workspace_bytes, void *stream);

/* The routed layer at the model's real shape, where the experts work on a
 * latent vector narrower than the model width (k3: hidden 7168, latent 3584):
 *
 *   ids, w      = router(x)                                   x: [T, hidden]
 *   latent      = routed_expert_down_proj(x)                  Q8 [latent, hidden]
 *   rows        = experts(latent rows grouped by expert)      MXFP4 tables of width latent
 *   routed      = sum_r w[r] * rows[r]                        [T, latent]
 *   routed_full = routed_expert_up_proj(rms_norm(routed))     Q8 [hidden, latent]
 *   out         = routed_full + shared_expert(x)
 *
 * i.e. k3_engine.cu:1668-1671 (latent projection), :1851-1863 (weighted sum,
 * routed_expert_norm, routed_expert_up_proj), :1889-1893 (add of the shared
 * output) and k3_engine_prefill.inc:1525-1590, without the host round trips.
 * `layer.hidden` is the model width (router weight [E, hidden], shared expert
 * [S, hidden]); the six expert tables of `layer` are shaped with `latent` in
 * place of hidden.  The two projections use layer.q8_block / q8_scale_type.
 * No reference operator is replaced one to one: it is the composition. */
typedef struct k3_moe_latent_desc {
    k3_moe_layer_desc layer;
    uint32_t latent;               /* width the experts work at                   */
    float norm_epsilon;            /* routed_expert_norm epsilon (1e-5)           */
    const void *down_q;            /* i8 [latent, hidden]                         */
    const void *down_s;            /* scale [latent, hidden / q8_block]           */
    const void *norm_weight;       /* bf16 [latent]                               */
    const void *up_q;              /* i8 [hidden, latent]                         */
    const void *up_s;              /* scale [hidden, latent / q8_block]           */
} k3_moe_latent_desc;

size_t k3_moe_latent_workspace_bytes(const k3_moe_latent_desc *desc, uint32_t tokens);
bool k3_moe_latent_layer_forward(const k3_moe_latent_desc *desc, void *out,
                                 const void *x, uint32_t tokens, void *workspace,
                                 size_t workspace_bytes, void *ids_out,
                                 void *weights_out, void *stream);

/* Device-side status since the library was loaded, a bit mask: 0 = ok;
 * bit 0 (1) = a bounded barrier wait of a tensor-core kernel gave up (that
 * launch's output is undefined); bit 1 (2) = a dispatch (either entry point)
 * met an expert id >= experts: such routes are skipped, so the offsets
 * undercount and the sorted arrays keep stale entries for them.
 * Synchronises with the device. */
uint32_t k3_moe_device_status(void);

/* Reset the status to 0 (after the host has dealt with what it reported). */
bool k3_moe_device_status_clear(void);

/* Self test of the bounded waits: one warp waits on a barrier that nothing
 * arrives on, gives up after `limit_us` microseconds (1 .. 1000000), and leaves
 * by the same path as the product kernels: bit 0 of k3_moe_device_status() is
 * raised and, if `gave_up` (a device u32) is given, 1 is stored there.  The
 * kernel touches no tensor memory and the context stays usable.  No
 * counterpart in the reference. */
bool k3_moe_selftest_bounded_wait(uint32_t limit_us, void *gave_up, void *stream);

/* Tensor-pipe peak of an MMA kind, for roofline denominators measured on the
 * GPU at hand: one CTA per SM issues 4 * iterations tcgen05.mma instructions of
 * M = 128, N = 256 on operand tiles that stay in shared memory.  kind: 0 = bf16
 * (kind::f16), 1 = block-scaled E2M1 x E4M3 (kind::mxf8f6f4, what the expert
 * kernels issue), 2 = block-scaled E2M1 x E2M1 (kind::mxf4, the MXFP4 peak).
 * *flop_per_launch (optional) receives the operations of the launch; time the
 * launch with events.  No counterpart in the reference. */
bool k3_moe_peak_launch(int kind, uint32_t iterations, double *flop_per_launch, void *stream);
/* The same with N = n (16 .. 256, a multiple of 16): the rate of the MMA shape a
 * kernel actually issues (the prefill expert kernel: N = rows of the tile, at
 * most 128; half the operations per operand byte of N = 256). */
bool k3_moe_peak_launch_n(int kind, uint32_t n, uint32_t iterations, double *flop_per_launch, void *stream);

/* Event helpers for hosts without CUDA runtime bindings: create / destroy a
 * timing event and read the milliseconds between two recorded events (waits
 * for `end`; negative on error). */
void *k3_moe_event_create(void);
void k3_moe_event_destroy(void *event);
float k3_moe_event_elapsed_ms(void *begin, void *end);

/* Seeded synthetic tensor fills used by the tests and the benchmark.  Element
 * first+i of stream `key` is a pure function of (key, first+i), so a shard of a
 * tensor can be filled on its own; the numpy mirror lives in
 * moonshine_b200/synth.py.  `first` must be a multiple of 8 for the byte fills.
 * bytes: low + floor(b*span/256); int8: uniform in [-127,127];
 * uniform: low + u*width, u in [0,1) with 24 bits, one rounding per operation,
 * stored as f32 or (as_f16) f16. */
bool k3_synth_fill_bytes(void *out, uint64_t count, uint64_t key, uint64_t first,
                         uint32_t low, uint32_t span, void *stream);
bool k3_synth_fill_int8(void *out, uint64_t count, uint64_t key, uint64_t first,
                        void *stream);
bool k3_synth_fill_uniform(void *out, uint64_t count, uint64_t key,
                           uint64_t first, float low, float width, int as_f16,
                           void *stream);

/* Version string of the library. */
const char *k3_moe_version(void);

#ifdef __cplusplus
}
#endif
#endif
