/*
 * Expert-parallel routed-MoE layer over NCCL, one process (rank) per GPU.
 *
 * No counterpart in the reference, which runs on one GPU and feeds experts
 * from NVMe (k3_engine.cu:1696-1822).  Here the layer's experts are sharded
 * contiguously over the ranks and stay resident in each GPU's slot table
 * (rank g holds experts [g*E/G, (g+1)*E/G), described by the
 * local_expert_first / local_expert_count fields of k3_moe_layer_desc), and
 * tokens are data-parallel: rank r owns a contiguous block of the batch's rows.
 * Router, top-k and the shared expert run where the token lives.  One exchange
 * each way per layer pass:
 *
 *   counts   one all-gather of every rank's expert offsets (the only host read)
 *   dispatch grouped ncclSend/ncclRecv of bf16 rows, one row per route, sorted
 *            (expert asc, route asc) on the source
 *   regroup  received rows (source asc, expert asc, route asc) are read in the
 *            order (expert asc, source asc, route asc) - with contiguous token
 *            blocks that is the single-GPU grouping order
 *            (k3_engine_prefill.inc:1175-1194), so results equal the one-GPU
 *            layer bit for bit
 *   dispatch sends each token row once per destination rank (however many of its
 *            routes go there) plus a 4-byte slot per route
 *   return   the reverse grouped send/recv, then the weighted combine in rank
 *            order on the source (or partial sums per rank, k3_moe_ep_set_reduced_return)
 *
 * One token (decode): x is replicated, every rank routes it identically, runs
 * the selected experts it holds, and one all-reduce merges the rows (integer
 * sum of the bf16 bit patterns: every row is produced by exactly one rank, all
 * others contribute zero bits, so the merge is exact).
 *
 * Conventions are those of k3_moe_layer.h: caller-owned device pointers, the
 * stream as void *, bool results, messages through `error`.  NCCL is loaded
 * with dlopen("libnccl.so.2") when the first handle is created (or from the
 * path in K3_NCCL_LIBRARY); a process that never creates a handle needs no NCCL.
 * All ranks must make the same calls in the same order.
 */
#ifndef K3_MOE_EP_H
#define K3_MOE_EP_H

#include "k3_moe_layer.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct k3_moe_ep k3_moe_ep;

#define K3_MOE_EP_ID_BYTES 128

/* Rank 0 makes the identifier (ncclGetUniqueId) and gives its 128 bytes to the
 * other ranks by whatever channel the host has; every rank then creates its
 * handle with the device that will run its kernels current. */
bool k3_moe_ep_unique_id(void *id_bytes, char *error, size_t error_size);
bool k3_moe_ep_create(k3_moe_ep **out, const void *id_bytes, int rank, int world,
                      char *error, size_t error_size);
void k3_moe_ep_destroy(k3_moe_ep *ep);
/* Return direction of k3_moe_ep_layer_forward.  Default (false): every expert row comes
 * back and the token's own rank sums the top_k rows in rank order - results equal the
 * one-GPU layer bit for bit.  Reduced (true): the expert rank forms, per token it
 * served, the weighted sum of that token's rows in rank order (fp32, rounded to bf16
 * once) and returns ONE row per (token, rank); the token's rank adds the partial sums
 * in rank-of-GPU order.  top_k / (distinct ranks per token) times fewer bytes come back
 * (8x at 2 ranks, 2.3x at 8 for top-16); the result differs from the exact mode by
 * the extra roundings (rel-L2 about 1e-3, inside the layer tolerance of 1e-2).  All
 * ranks must use the same setting. */
bool k3_moe_ep_set_reduced_return(k3_moe_ep *ep, bool reduced);
int k3_moe_ep_rank(const k3_moe_ep *ep);
int k3_moe_ep_world(const k3_moe_ep *ep);

/* Host-side plan of one exchange, exported for tests and for hosts that issue
 * their own transfers.  offsets_all u32 [world][experts + 1] are the ranks'
 * dispatch offsets.  Outputs (row units): send_rows[g] / recv_rows[s] of this
 * rank, and for each (local expert e, source s) block, in (e, s) order:
 * block_recv_start (first row among the received rows), block_dest_start
 * (first row in grouped order), block_rows; offsets_local u32 [per + 1].
 * Arrays hold world, world, per*world, per*world, per*world, per+1 entries. */
bool k3_moe_ep_plan(const uint32_t *offsets_all, uint32_t world, uint32_t rank,
                    uint32_t experts, uint32_t *send_rows, uint32_t *recv_rows,
                    uint32_t *block_recv_start, uint32_t *block_dest_start,
                    uint32_t *block_rows, uint32_t *offsets_local);

/* Device workspace for passes of up to `local_tokens` rows on this rank when at
 * most `max_recv_rows` routed rows arrive here (the sure bound is
 * world * local_tokens * top_k).  0 if the description is not usable. */
size_t k3_moe_ep_workspace_bytes(const k3_moe_ep *ep, const k3_moe_layer_desc *desc,
                                 uint32_t local_tokens, uint32_t max_recv_rows);

/* One layer pass: x bf16 [local_tokens, d] -> out bf16 [local_tokens, d].
 * desc describes this rank's shard.  local_tokens may be 0 on a rank (it still
 * serves its experts).  Waits on the host once, for the count exchange.  Fails
 * with a message if more than max_recv_rows rows arrive.  ids_out / weights_out
 * (optional) receive the routing of the local tokens. */
bool k3_moe_ep_layer_forward(k3_moe_ep *ep, const k3_moe_layer_desc *desc, void *out,
                             const void *x, uint32_t local_tokens, uint32_t max_recv_rows,
                             void *workspace, size_t workspace_bytes, void *ids_out,
                             void *weights_out, char *error, size_t error_size,
                             void *stream);

/* Timing of the last k3_moe_ep_layer_forward call on this handle, from CUDA
 * events on the call's stream (waits for the call to finish): milliseconds of the
 * grouped expert products and of the whole pass, and the rows received. */
bool k3_moe_ep_last_pass(k3_moe_ep *ep, float *experts_ms, float *pass_ms, uint32_t *recv_rows);

/* One token on every rank (x bf16 [d], the same on all ranks) -> out bf16 [d],
 * the same on all ranks.  residual (optional, bf16 [d]) is added last.  No host
 * wait.  Workspace: k3_moe_ep_decode_workspace_bytes. */
size_t k3_moe_ep_decode_workspace_bytes(const k3_moe_ep *ep, const k3_moe_layer_desc *desc);
bool k3_moe_ep_decode(k3_moe_ep *ep, const k3_moe_layer_desc *desc, void *out, const void *x,
                      const void *residual, void *workspace, size_t workspace_bytes, void *stream);

/* A stack of layers for one token: h = x; for each layer l:
 * h = h + moe_l(rms_norm(h) * norm_weight) - the MoE section of the engine's layer
 * loop (k3_engine.cu:2453-2498 with :1550-1553 and :1889-1897 per layer) without
 * the attention half.  descs is an array of `layers` pointers (a layer may appear
 * several times); norm_weight bf16 [d]; x and out bf16 [d] (may alias).  Works with
 * world == 1 too, and then needs no NCCL.  Workspace:
 * k3_moe_ep_decode_workspace_bytes of the largest layer + 3 * d * 2 + 768 bytes. */
bool k3_moe_ep_decode_stack(k3_moe_ep *ep, const k3_moe_layer_desc *const *descs, uint32_t layers,
                            void *out, const void *x, const void *norm_weight, float epsilon,
                            void *workspace, size_t workspace_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif
