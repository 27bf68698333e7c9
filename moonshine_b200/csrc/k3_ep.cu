// Expert-parallel layer over NCCL (see k3_moe_ep.h): the count exchange, the two
// grouped send/recv steps and this library's kernels issued from one C++ call on the
// caller's stream.  NCCL is bound at run time with dlopen, so the library loads (and
// every single-GPU entry point works) on machines without it.
#include "k3_grouped.h"
#include "k3_common.cuh"
#include "k3_moe_ep.h"
#include "k3_moe_ops.h"

#include <dlfcn.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#if __has_include(<nccl.h>)
#include <nccl.h>
#else
// the few declarations used, as NCCL 2.x publishes them
extern "C" {
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef enum { ncclSuccess = 0 } ncclResult_t;
typedef enum { ncclInt8 = 0, ncclUint8 = 1, ncclInt32 = 2, ncclUint32 = 3, ncclBfloat16 = 9 } ncclDataType_t;
typedef enum { ncclSum = 0 } ncclRedOp_t;
}
#endif

using namespace k3;

namespace {

struct NcclApi {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                              cudaStream_t) = nullptr;
    ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

void set_error(char *error, size_t error_size, const char *message) {
    if (!error || error_size == 0) return;
    snprintf(error, error_size, "%s", message);
}

// Loaded once per process.  Returns nullptr (with a message) when NCCL is absent.
const NcclApi *nccl_api(char *error, size_t error_size) {
    static std::mutex lock;
    static NcclApi api;
    static bool tried = false, ok = false;
    std::lock_guard<std::mutex> guard(lock);
    if (!tried) {
        tried = true;
        const char *path = getenv("K3_NCCL_LIBRARY");
        api.lib = dlopen(path && *path ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (api.lib) {
            auto sym = [&](const char *name) { return dlsym(api.lib, name); };
            api.GetUniqueId = (decltype(api.GetUniqueId))sym("ncclGetUniqueId");
            api.CommInitRank = (decltype(api.CommInitRank))sym("ncclCommInitRank");
            api.CommDestroy = (decltype(api.CommDestroy))sym("ncclCommDestroy");
            api.AllGather = (decltype(api.AllGather))sym("ncclAllGather");
            api.AllReduce = (decltype(api.AllReduce))sym("ncclAllReduce");
            api.Send = (decltype(api.Send))sym("ncclSend");
            api.Recv = (decltype(api.Recv))sym("ncclRecv");
            api.GroupStart = (decltype(api.GroupStart))sym("ncclGroupStart");
            api.GroupEnd = (decltype(api.GroupEnd))sym("ncclGroupEnd");
            api.GetErrorString = (decltype(api.GetErrorString))sym("ncclGetErrorString");
            ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.AllReduce &&
                 api.Send && api.Recv && api.GroupStart && api.GroupEnd;
        }
    }
    if (!ok) {
        set_error(error, error_size, "NCCL is not available (dlopen of libnccl.so.2 failed; set K3_NCCL_LIBRARY)");
        return nullptr;
    }
    return &api;
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// --- each token row crosses to a destination once, however many of its routes go there
// mask[t] = set of destination ranks of token t's routes
__global__ void __launch_bounds__(256)
ep_mask_kernel(unsigned long long *__restrict__ mask, const uint32_t *__restrict__ ids, uint32_t tokens,
               uint32_t top_k, uint32_t per) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= tokens) return;
    unsigned long long m = 0ull;
    for (uint32_t r = 0; r < top_k; r++) m |= 1ull << (ids[(uint64_t)t * top_k + r] / per);
    mask[t] = m;
}

// One block per destination g: the tokens that have a route to g, in token order -
// token_list[g * tokens + slot] = t, slot[t * world + g] = slot, unique[g] = how many.
__global__ void __launch_bounds__(1024)
ep_unique_kernel(uint32_t *__restrict__ slot, uint32_t *__restrict__ token_list, uint32_t *__restrict__ unique,
                 const unsigned long long *__restrict__ mask, uint32_t tokens, uint32_t world) {
    __shared__ uint32_t warp_total[32];
    __shared__ uint32_t running_s;
    const uint32_t g = blockIdx.x, lane = threadIdx.x % kWarp, warp = threadIdx.x / kWarp;
    if (threadIdx.x == 0) running_s = 0u;
    __syncthreads();
    for (uint32_t base = 0; base < tokens; base += blockDim.x) {
        const uint32_t t = base + threadIdx.x;
        const bool flag = t < tokens && ((mask[t] >> g) & 1ull) != 0ull;
        const uint32_t ballot = __ballot_sync(0xffffffffu, flag);
        if (lane == 0) warp_total[warp] = __popc(ballot);
        __syncthreads();
        uint32_t before = running_s;
        for (uint32_t w = 0; w < warp; w++) before += warp_total[w];
        if (flag) {
            const uint32_t pos = before + __popc(ballot & ((1u << lane) - 1u));
            slot[(uint64_t)t * world + g] = pos;
            token_list[(uint64_t)g * tokens + pos] = t;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t total = 0;
            for (uint32_t w = 0; w < blockDim.x / kWarp; w++) total += warp_total[w];
            running_s += total;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) unique[g] = running_s;
}

// route_slot[p] = slot of the route's token among the rows sent to the route's destination
__global__ void __launch_bounds__(256)
ep_route_slot_kernel(uint32_t *__restrict__ route_slot, const uint32_t *__restrict__ slot,
                     const uint32_t *__restrict__ sorted_route, const uint32_t *__restrict__ sorted_token,
                     const uint32_t *__restrict__ ids, uint32_t routes, uint32_t per, uint32_t world) {
    const uint32_t p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= routes) return;
    const uint32_t g = ids[sorted_route[p]] / per;
    route_slot[p] = slot[(uint64_t)sorted_token[p] * world + g];
}

// rows_send[g * tokens + i] = x[token_list[g * tokens + i]] for i < unique[g]; one warp per row
__global__ void __launch_bounds__(256)
ep_gather_unique_kernel(uint4 *__restrict__ rows_send, const uint4 *__restrict__ x,
                        const uint32_t *__restrict__ token_list, const uint32_t *__restrict__ unique,
                        uint32_t tokens, uint32_t world, uint32_t units) {
    const uint32_t lane = threadIdx.x % kWarp;
    const uint32_t warps = gridDim.x * blockDim.x / kWarp;
    for (uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) / kWarp; row < world * tokens; row += warps) {
        const uint32_t g = row / tokens, i = row % tokens;
        if (i >= unique[g]) continue;
        const uint4 *src = x + (uint64_t)token_list[row] * units;
        uint4 *dst = rows_send + (uint64_t)row * units;
        for (uint32_t u = lane; u < units; u += kWarp) dst[u] = src[u];
    }
}

// like ep_order_kernel, for rows sent once per destination: the product row at a grouped
// position reads the received row (first row of the block's source + the route's slot)
__global__ void __launch_bounds__(256)
ep_order_slots_kernel(uint32_t *__restrict__ row_index, uint32_t *__restrict__ inverse,
                      const uint32_t *__restrict__ slots_recv, const uint32_t *__restrict__ block_recv_start,
                      const uint32_t *__restrict__ block_dest_start, const uint32_t *__restrict__ block_rows,
                      const uint32_t *__restrict__ source_first_row, uint32_t blocks, uint32_t world) {
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t warps = gridDim.x * blockDim.x / kWarp;
    for (uint32_t b = warp; b < blocks; b += warps) {
        const uint32_t from = block_recv_start[b], to = block_dest_start[b], n = block_rows[b];
        const uint32_t first = source_first_row[b % world];
        for (uint32_t i = lane; i < n; i += kWarp) {
            row_index[to + i] = first + slots_recv[from + i];
            inverse[from + i] = to + i;
        }
    }
}

// --- reduced return: the expert rank forms sum_r w_r * row_r over the routes of one token
// that it served (in rank order) and sends ONE row per (token, destination) back.
// On the source: for every (destination g, unique row i) the positions of the token's
// routes among the routes sent to g (rank order, 0xffffffff = none) and their weights.
__global__ void __launch_bounds__(256)
ep_unique_routes_kernel(uint32_t *__restrict__ unique_routes, float *__restrict__ unique_weights,
                        const uint32_t *__restrict__ ids, const float *__restrict__ weights,
                        const uint32_t *__restrict__ inv_perm, const uint32_t *__restrict__ offsets,
                        const uint32_t *__restrict__ slot, uint32_t tokens, uint32_t top_k, uint32_t per,
                        uint32_t world) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= tokens) return;
    uint8_t count[64];                           // routes of this token per destination so far
    for (uint32_t g = 0; g < world; g++) count[g] = 0;
    for (uint32_t r = 0; r < top_k; r++) {
        const uint32_t route = t * top_k + r;
        const uint32_t g = ids[route] / per;
        const uint32_t j = count[g]++;
        const uint64_t at = ((uint64_t)g * tokens + slot[(uint64_t)t * world + g]) * top_k + j;
        unique_routes[at] = inv_perm[route] - offsets[g * per];
        unique_weights[at] = weights[route];
    }
    for (uint32_t g = 0; g < world; g++) {
        if (count[g] == 0) continue;
        const uint64_t at = ((uint64_t)g * tokens + slot[(uint64_t)t * world + g]) * top_k;
        for (uint32_t j = count[g]; j < top_k; j++) unique_routes[at + j] = 0xffffffffu;
    }
}

// On the expert rank: partial[u] = bf16(sum_j w_j * rows_out[inverse[route_base(u) + pos_j]]), one
// 64-thread group per unique row, 8 columns per thread and pass.
__global__ void __launch_bounds__(256)
ep_reduce_kernel(uint16_t *__restrict__ partial, const uint16_t *__restrict__ rows_out,
                 const uint32_t *__restrict__ inverse, const uint32_t *__restrict__ routes_recv,
                 const float *__restrict__ weights_recv, const uint32_t *__restrict__ source_first_row,
                 const uint32_t *__restrict__ source_route_base, uint32_t world, uint32_t n_unique, uint32_t top_k,
                 uint32_t hidden) {
    const uint32_t groups = gridDim.x * (blockDim.x / 64u);
    const uint32_t lane64 = threadIdx.x % 64u;
    for (uint32_t u = blockIdx.x * (blockDim.x / 64u) + threadIdx.x / 64u; u < n_unique; u += groups) {
        uint32_t src = 0;                                  // the source whose rows contain unique row u
        while (src + 1u < world && source_first_row[src + 1u] <= u) src++;
        const uint32_t base = source_route_base[src];
        for (uint32_t c = lane64; c < hidden / 8u; c += 64u) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (uint32_t j = 0; j < top_k; j++) {
                const uint32_t pos = routes_recv[(uint64_t)u * top_k + j];
                if (pos == 0xffffffffu) break;
                const float w = weights_recv[(uint64_t)u * top_k + j];
                const uint4 q = reinterpret_cast<const uint4 *>(rows_out + (uint64_t)inverse[base + pos] * hidden)[c];
                acc[0] = fmaf(w, bf16_lo(q.x), acc[0]); acc[1] = fmaf(w, bf16_hi(q.x), acc[1]);
                acc[2] = fmaf(w, bf16_lo(q.y), acc[2]); acc[3] = fmaf(w, bf16_hi(q.y), acc[3]);
                acc[4] = fmaf(w, bf16_lo(q.z), acc[4]); acc[5] = fmaf(w, bf16_hi(q.z), acc[5]);
                acc[6] = fmaf(w, bf16_lo(q.w), acc[6]); acc[7] = fmaf(w, bf16_hi(q.w), acc[7]);
            }
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; i++)
                o[i] = (uint32_t)float_to_bf16_bits(acc[2 * i]) | ((uint32_t)float_to_bf16_bits(acc[2 * i + 1]) << 16);
            reinterpret_cast<uint4 *>(partial + (uint64_t)u * hidden)[c] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

// On the source: out[t] = bf16( bf16(sum over the token's destinations g, ascending, of
// partial_home[g * tokens + slot[t, g]]) + shared[t] )
__global__ void __launch_bounds__(256)
ep_combine_partials_kernel(uint16_t *__restrict__ out, const uint16_t *__restrict__ partial_home,
                           const unsigned long long *__restrict__ mask, const uint32_t *__restrict__ slot,
                           const uint16_t *__restrict__ shared, uint32_t tokens, uint32_t world, uint32_t hidden) {
    for (uint32_t t = blockIdx.x; t < tokens; t += gridDim.x) {
        const unsigned long long m = mask[t];
        for (uint32_t c = threadIdx.x; c < hidden / 8u; c += blockDim.x) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (uint32_t g = 0; g < world; g++) {
                if (((m >> g) & 1ull) == 0ull) continue;
                const uint64_t row = (uint64_t)g * tokens + slot[(uint64_t)t * world + g];
                const uint4 q = reinterpret_cast<const uint4 *>(partial_home + row * hidden)[c];
                acc[0] += bf16_lo(q.x); acc[1] += bf16_hi(q.x); acc[2] += bf16_lo(q.y); acc[3] += bf16_hi(q.y);
                acc[4] += bf16_lo(q.z); acc[5] += bf16_hi(q.z); acc[6] += bf16_lo(q.w); acc[7] += bf16_hi(q.w);
            }
            float sh[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (shared) {
                const uint4 q = reinterpret_cast<const uint4 *>(shared + (uint64_t)t * hidden)[c];
                sh[0] = bf16_lo(q.x); sh[1] = bf16_hi(q.x); sh[2] = bf16_lo(q.y); sh[3] = bf16_hi(q.y);
                sh[4] = bf16_lo(q.z); sh[5] = bf16_hi(q.z); sh[6] = bf16_lo(q.w); sh[7] = bf16_hi(q.w);
            }
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t lo = float_to_bf16_bits(acc[2 * i]), hi = float_to_bf16_bits(acc[2 * i + 1]);
                if (shared) {
                    lo = float_to_bf16_bits(bf16_bits_to_float(lo) + sh[2 * i]);
                    hi = float_to_bf16_bits(bf16_bits_to_float(hi) + sh[2 * i + 1]);
                }
                o[i] = lo | (hi << 16);
            }
            reinterpret_cast<uint4 *>(out + (uint64_t)t * hidden)[c] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

}  // namespace

struct k3_moe_ep {
    int rank = 0, world = 1, device = 0;
    const NcclApi *api = nullptr;
    ncclComm_t comm = nullptr;
    uint32_t *pinned = nullptr;          // [world][kPinnedRow] offsets of every rank, then the plan tables
    size_t pinned_words = 0;
    cudaStream_t side = nullptr;         // the shared expert runs here, beside the exchange
    cudaEvent_t fork = nullptr, join = nullptr;
    cudaEvent_t counts_ready = nullptr, t_begin = nullptr, t_experts0 = nullptr, t_experts1 = nullptr,
                t_end = nullptr;
    uint32_t last_recv_rows = 0;
    bool timed = false;
    bool reduced_return = false;
    std::vector<uint32_t> send_rows, recv_rows, send_unique, recv_unique;
};

namespace {

constexpr uint32_t kMaxExpertsEp = 1024;
constexpr uint32_t kMaxWorld = 64;

bool nccl_ok(const k3_moe_ep *ep, ncclResult_t r, char *error, size_t error_size, const char *what) {
    if (r == ncclSuccess) return true;
    char text[256];
    snprintf(text, sizeof(text), "%s failed: %s", what,
             ep->api && ep->api->GetErrorString ? ep->api->GetErrorString(r) : "NCCL error");
    set_error(error, error_size, text);
    return false;
}

struct EpWorkspace {
    float *logits;
    uint32_t *ids;
    float *weights;
    uint32_t *offsets, *sorted_route, *sorted_token, *inv_perm;
    void *dispatch_ws;
    size_t dispatch_bytes;
    uint32_t *offsets_all;                 // [world][E + 1 + world]: every rank's offsets and unique-row counts
    uint32_t *tables;                      // block_recv_start | block_dest_start | block_rows | offsets_local | source_first_row
    unsigned long long *dest_mask;         // [tokens]
    uint32_t *slot, *token_list;           // [tokens, world], [world, tokens]
    uint32_t *route_slot, *slots_recv;     // [routes], [max_recv]
    uint32_t *unique_routes, *routes_recv; // reduced return: [world * tokens, top_k] sent, [max_recv rows of top_k] received
    float *unique_weights, *weights_recv;
    uint32_t *order, *inverse;             // [max_recv]
    uint16_t *rows_send, *rows_home;       // [routes, d]
    uint16_t *rows_recv, *rows_out, *rows_back;   // [max_recv, d]
    uint16_t *act;                         // [max_recv, I] (only without the block-scaled path)
    uint16_t *rows_in;                     // [max_recv, d] (only without the block-scaled path)
    void *mx_ws;
    size_t mx_bytes;
    void *sh_ws;
    size_t sh_bytes;
    uint16_t *sh_gate, *sh_up, *sh_act, *sh_out;
    size_t total;
};

EpWorkspace carve_ep(const k3_moe_layer_desc *d, uint32_t world, uint32_t tokens, uint32_t max_recv, void *base) {
    EpWorkspace w{};
    char *p = (char *)base;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        char *q = base ? p + off : nullptr;
        off += align_up(std::max<size_t>(bytes, 16), 256);
        return (void *)q;
    };
    const uint32_t t1 = std::max(tokens, 1u);
    const uint64_t routes = (uint64_t)t1 * d->top_k;
    const uint32_t per = d->local_expert_count;
    const uint32_t cap = std::max(max_recv, 1u);
    w.logits = (float *)take((size_t)t1 * d->expert_count * 4u);
    w.ids = (uint32_t *)take(routes * 4u);
    w.weights = (float *)take(routes * 4u);
    w.offsets = (uint32_t *)take((size_t)(d->expert_count + 1u + world) * 4u);   // + this rank's unique-row counts
    w.sorted_route = (uint32_t *)take(routes * 4u);
    w.sorted_token = (uint32_t *)take(routes * 4u);
    w.inv_perm = (uint32_t *)take(routes * 4u);
    w.dispatch_bytes = k3_moe_dispatch_workspace_bytes(t1, d->top_k, d->expert_count);
    w.dispatch_ws = take(w.dispatch_bytes);
    w.offsets_all = (uint32_t *)take((size_t)world * (d->expert_count + 1u + world) * 4u);
    w.tables = (uint32_t *)take(((size_t)3u * per * world + per + 1u + 2u * world) * 4u);
    w.dest_mask = (unsigned long long *)take((size_t)t1 * 8u);
    w.slot = (uint32_t *)take((size_t)t1 * world * 4u);
    w.token_list = (uint32_t *)take((size_t)t1 * world * 4u);
    w.route_slot = (uint32_t *)take(routes * 4u);
    w.slots_recv = (uint32_t *)take((size_t)cap * 4u);
    w.unique_routes = (uint32_t *)take((size_t)t1 * world * d->top_k * 4u);
    w.unique_weights = (float *)take((size_t)t1 * world * d->top_k * 4u);
    w.routes_recv = (uint32_t *)take((size_t)cap * 4u);          // at most max_recv / 1 unique rows x top_k ... see below
    w.weights_recv = (float *)take((size_t)cap * 4u);
    w.order = (uint32_t *)take((size_t)cap * 4u);
    w.inverse = (uint32_t *)take((size_t)cap * 4u);
    w.rows_send = (uint16_t *)take((size_t)t1 * world * d->hidden * 2u);       // one region of t1 rows per destination
    w.rows_home = (uint16_t *)take(routes * d->hidden * 2u);
    w.rows_recv = (uint16_t *)take((size_t)cap * d->hidden * 2u);
    w.rows_out = (uint16_t *)take((size_t)cap * d->hidden * 2u);
    w.rows_back = (uint16_t *)take((size_t)cap * d->hidden * 2u);
    w.mx_bytes = k3_grouped_mx_supported(d, std::max(cap, 32u)) ? k3_grouped_mx_workspace_bytes(d, cap, cap) : 0;
    w.mx_ws = take(w.mx_bytes);
    // rows too few for the block-scaled path, or a shape it does not take: bf16 path scratch
    w.act = (uint16_t *)take((size_t)cap * d->expert_hidden * 2u);
    w.rows_in = (uint16_t *)take((size_t)(w.mx_bytes ? 32u : cap) * d->hidden * 2u);
    w.sh_bytes = d->shared_hidden ? k3_grouped_shared_workspace_bytes(d, t1) : 0;
    w.sh_ws = take(w.sh_bytes);
    if (d->shared_hidden) {
        w.sh_gate = (uint16_t *)take((size_t)t1 * d->shared_hidden * 2u);
        w.sh_up = (uint16_t *)take((size_t)t1 * d->shared_hidden * 2u);
        w.sh_act = (uint16_t *)take((size_t)t1 * d->shared_hidden * 2u);
        w.sh_out = (uint16_t *)take((size_t)t1 * d->hidden * 2u);
    }
    w.total = off;
    return w;
}

bool shard_ok(const k3_moe_ep *ep, const k3_moe_layer_desc *d) {
    return ep && d && d->expert_count != 0 && d->expert_count <= kMaxExpertsEp &&
           d->expert_count % (uint32_t)ep->world == 0 &&
           d->local_expert_count == d->expert_count / (uint32_t)ep->world &&
           d->local_expert_first == (uint32_t)ep->rank * d->local_expert_count && d->hidden % 32u == 0 &&
           d->top_k != 0 && d->top_k <= 32u;
}

struct DecodeWorkspace {
    float *logits;
    uint32_t *ids;
    float *weights;
    uint16_t *sh_gate, *sh_up, *sh_act, *sh_out, *act, *rows_out;
    void *scratch;
    size_t scratch_bytes, total;
};

DecodeWorkspace carve_decode(const k3_moe_layer_desc *d, void *base) {
    DecodeWorkspace w{};
    char *p = (char *)base;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        char *q = base ? p + off : nullptr;
        off += align_up(std::max<size_t>(bytes, 16), 256);
        return (void *)q;
    };
    w.logits = (float *)take((size_t)d->expert_count * 4u);
    w.ids = (uint32_t *)take((size_t)d->top_k * 4u);
    w.weights = (float *)take((size_t)d->top_k * 4u);
    w.sh_gate = (uint16_t *)take((size_t)d->shared_hidden * 2u);
    w.sh_up = (uint16_t *)take((size_t)d->shared_hidden * 2u);
    w.sh_act = (uint16_t *)take((size_t)d->shared_hidden * 2u);
    w.sh_out = (uint16_t *)take((size_t)d->hidden * 2u);
    w.act = (uint16_t *)take((size_t)d->top_k * d->expert_hidden * 2u);
    w.rows_out = (uint16_t *)take((size_t)d->top_k * d->hidden * 2u);
    w.scratch_bytes = k3_decode_mx_scratch_bytes(d);
    w.scratch = take(w.scratch_bytes);
    w.total = off;
    return w;
}

}  // namespace

extern "C" bool k3_moe_ep_unique_id(void *id_bytes, char *error, size_t error_size) {
    set_error(error, error_size, "");
    if (!id_bytes) {
        set_error(error, error_size, "null identifier buffer");
        return false;
    }
    const NcclApi *api = nccl_api(error, error_size);
    if (!api) return false;
    static_assert(sizeof(ncclUniqueId) == K3_MOE_EP_ID_BYTES, "identifier size");
    ncclUniqueId id;
    const ncclResult_t r = api->GetUniqueId(&id);
    if (r != ncclSuccess) {
        set_error(error, error_size, "ncclGetUniqueId failed");
        return false;
    }
    memcpy(id_bytes, &id, sizeof(id));
    return true;
}

extern "C" bool k3_moe_ep_create(k3_moe_ep **out, const void *id_bytes, int rank, int world, char *error,
                                 size_t error_size) {
    set_error(error, error_size, "");
    if (!out || world < 1 || world > (int)kMaxWorld || rank < 0 || rank >= world || (world > 1 && !id_bytes)) {
        set_error(error, error_size, "invalid rank, world size or identifier");
        return false;
    }
    k3_moe_ep *ep = new k3_moe_ep();
    ep->rank = rank;
    ep->world = world;
    ep->device = current_device();
    ep->send_rows.resize(world);
    ep->recv_rows.resize(world);
    ep->send_unique.resize(world);
    ep->recv_unique.resize(world);
    // every rank's offsets, then the plan tables of the largest shard
    ep->pinned_words = (size_t)world * (kMaxExpertsEp + 1u + kMaxWorld) + (size_t)3u * kMaxExpertsEp + kMaxExpertsEp + 1u + 2u * kMaxWorld;
    bool ok = cudaHostAlloc((void **)&ep->pinned, ep->pinned_words * 4u, cudaHostAllocDefault) == cudaSuccess;
    for (cudaEvent_t *e : {&ep->t_begin, &ep->t_experts0, &ep->t_experts1, &ep->t_end}) {
        ok = ok && cudaEventCreate(e) == cudaSuccess;
    }
    ok = ok && cudaEventCreateWithFlags(&ep->counts_ready, cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&ep->fork, cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&ep->join, cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&ep->side, cudaStreamNonBlocking) == cudaSuccess;
    if (!ok) {
        (void)cudaGetLastError();
        set_error(error, error_size, "host buffer or event creation failed");
        k3_moe_ep_destroy(ep);
        return false;
    }
    if (world > 1) {
        ep->api = nccl_api(error, error_size);
        if (!ep->api) {
            k3_moe_ep_destroy(ep);
            return false;
        }
        ncclUniqueId id;
        memcpy(&id, id_bytes, sizeof(id));
        if (!nccl_ok(ep, ep->api->CommInitRank(&ep->comm, world, id, rank), error, error_size, "ncclCommInitRank")) {
            ep->comm = nullptr;
            k3_moe_ep_destroy(ep);
            return false;
        }
    }
    *out = ep;
    return true;
}

extern "C" void k3_moe_ep_destroy(k3_moe_ep *ep) {
    if (!ep) return;
    if (ep->comm && ep->api) (void)ep->api->CommDestroy(ep->comm);
    if (ep->pinned) (void)cudaFreeHost(ep->pinned);
    for (cudaEvent_t e : {ep->counts_ready, ep->t_begin, ep->t_experts0, ep->t_experts1, ep->t_end, ep->fork, ep->join}) {
        if (e) (void)cudaEventDestroy(e);
    }
    if (ep->side) (void)cudaStreamDestroy(ep->side);
    delete ep;
}

extern "C" bool k3_moe_ep_set_reduced_return(k3_moe_ep *ep, bool reduced) {
    if (!ep) return false;
    ep->reduced_return = reduced;
    return true;
}

extern "C" int k3_moe_ep_rank(const k3_moe_ep *ep) { return ep ? ep->rank : -1; }
extern "C" int k3_moe_ep_world(const k3_moe_ep *ep) { return ep ? ep->world : 0; }

namespace {
bool plan_impl(const uint32_t *offsets_all, uint32_t stride, uint32_t world, uint32_t rank, uint32_t experts,
               uint32_t *send_rows, uint32_t *recv_rows, uint32_t *block_recv_start, uint32_t *block_dest_start,
               uint32_t *block_rows, uint32_t *offsets_local);
}

extern "C" bool k3_moe_ep_plan(const uint32_t *offsets_all, uint32_t world, uint32_t rank, uint32_t experts,
                               uint32_t *send_rows, uint32_t *recv_rows, uint32_t *block_recv_start,
                               uint32_t *block_dest_start, uint32_t *block_rows, uint32_t *offsets_local) {
    return plan_impl(offsets_all, experts + 1u, world, rank, experts, send_rows, recv_rows, block_recv_start,
                     block_dest_start, block_rows, offsets_local);
}

namespace {
bool plan_impl(const uint32_t *offsets_all, uint32_t stride, uint32_t world, uint32_t rank, uint32_t experts,
               uint32_t *send_rows, uint32_t *recv_rows, uint32_t *block_recv_start, uint32_t *block_dest_start,
               uint32_t *block_rows, uint32_t *offsets_local) {
    if (!offsets_all || !send_rows || !recv_rows || !block_recv_start || !block_dest_start || !block_rows ||
        !offsets_local || world == 0 || rank >= world || experts == 0 || experts % world != 0) {
        return false;
    }
    const uint32_t per = experts / world, first = rank * per;
    const uint32_t *own = offsets_all + (size_t)rank * stride;
    for (uint32_t g = 0; g < world; g++) send_rows[g] = own[(g + 1u) * per] - own[g * per];
    // rows arrive source by source; inside a source (expert asc, route asc)
    uint32_t recv_base = 0;
    std::vector<uint32_t> source_base(world);
    for (uint32_t s = 0; s < world; s++) {
        const uint32_t *o = offsets_all + (size_t)s * stride;
        source_base[s] = recv_base;
        recv_rows[s] = o[first + per] - o[first];
        recv_base += recv_rows[s];
    }
    uint32_t dest = 0;
    for (uint32_t e = 0; e < per; e++) {
        offsets_local[e] = dest;
        for (uint32_t s = 0; s < world; s++) {
            const uint32_t *o = offsets_all + (size_t)s * stride;
            const uint32_t n = o[first + e + 1u] - o[first + e];
            const uint32_t b = e * world + s;
            block_recv_start[b] = source_base[s] + (o[first + e] - o[first]);
            block_dest_start[b] = dest;
            block_rows[b] = n;
            dest += n;
        }
    }
    offsets_local[per] = dest;
    return true;
}
}  // namespace

extern "C" size_t k3_moe_ep_workspace_bytes(const k3_moe_ep *ep, const k3_moe_layer_desc *d,
                                            uint32_t local_tokens, uint32_t max_recv_rows) {
    if (!shard_ok(ep, d) || local_tokens > 65535u) return 0;
    return carve_ep(d, (uint32_t)ep->world, local_tokens, max_recv_rows, nullptr).total + 256u;
}

extern "C" bool k3_moe_ep_layer_forward(k3_moe_ep *ep, const k3_moe_layer_desc *d, void *out, const void *x,
                                        uint32_t tokens, uint32_t max_recv, void *workspace,
                                        size_t workspace_bytes, void *ids_out, void *weights_out, char *error,
                                        size_t error_size, void *stream_pointer) {
    set_error(error, error_size, "");
    if (!shard_ok(ep, d) || !workspace || tokens > 65535u || (tokens != 0 && (!out || !x))) {
        set_error(error, error_size, "invalid handle, description or buffers (the description must be this rank's shard)");
        return false;
    }
    char *base = (char *)(((uintptr_t)workspace + 255u) & ~(uintptr_t)255u);
    const EpWorkspace w = carve_ep(d, (uint32_t)ep->world, tokens, max_recv, base);
    if (workspace_bytes < w.total + (size_t)(base - (char *)workspace)) {
        set_error(error, error_size, "workspace too small (k3_moe_ep_workspace_bytes)");
        return false;
    }
    cudaStream_t stream = (cudaStream_t)stream_pointer;
    const uint32_t world = (uint32_t)ep->world, rank = (uint32_t)ep->rank;
    const uint32_t E = d->expert_count, per = d->local_expert_count, k = d->top_k, H = d->hidden;
    const uint32_t routes = tokens * k;
    auto fail = [&](const char *message) {
        (void)cudaGetLastError();
        set_error(error, error_size, message);
        return false;
    };
    if (cudaEventRecord(ep->t_begin, stream) != cudaSuccess) return fail("event record failed");
    ep->timed = false;

    // 1. routing and dispatch of the local tokens; which destinations each token goes to
    const uint32_t stride = E + 1u + world;                 // offsets, then unique-row counts per destination
    uint32_t *unique_dev = w.offsets + E + 1u;
    if (tokens != 0) {
        if (!k3_moe_route(d, w.ids, w.weights, w.logits, x, tokens, stream)) return fail("k3_moe_route failed");
        if (!k3_moe_dispatch_build(w.offsets, w.sorted_route, w.sorted_token, w.inv_perm, w.ids, tokens, k, E,
                                   w.dispatch_ws, w.dispatch_bytes, stream)) {
            return fail("k3_moe_dispatch_build failed");
        }
        ep_mask_kernel<<<(tokens + 255u) / 256u, 256, 0, stream>>>(w.dest_mask, w.ids, tokens, k, per);
        ep_unique_kernel<<<world, 1024, 0, stream>>>(w.slot, w.token_list, unique_dev, w.dest_mask, tokens, world);
        if (!launch_ok()) return fail("destination kernels failed");
    } else if (cudaMemsetAsync(w.offsets, 0, (size_t)stride * 4u, stream) != cudaSuccess) {
        return fail("memset failed");
    }

    // 2. every rank's offsets and unique-row counts to every rank, and on to the host
    uint32_t *host_offsets = ep->pinned;
    if (world > 1) {
        if (!nccl_ok(ep, ep->api->AllGather(w.offsets, w.offsets_all, stride, ncclUint32, ep->comm, stream), error,
                     error_size, "ncclAllGather of the expert offsets")) {
            return false;
        }
    } else if (cudaMemcpyAsync(w.offsets_all, w.offsets, (size_t)stride * 4u, cudaMemcpyDeviceToDevice, stream) !=
               cudaSuccess) {
        return fail("offset copy failed");
    }
    if (cudaMemcpyAsync(host_offsets, w.offsets_all, (size_t)world * stride * 4u, cudaMemcpyDeviceToHost, stream) !=
            cudaSuccess ||
        cudaEventRecord(ep->counts_ready, stream) != cudaSuccess) {
        return fail("copy of the offsets to the host failed");
    }

    // 3. while they travel: the rows to send (each token once per destination it has a route
    // to, in token order, destination g's rows in region g), the slot of every route among
    // them, and the shared expert
    if (tokens != 0) {
        ep_gather_unique_kernel<<<std::min<uint32_t>((world * tokens + 7u) / 8u, (uint32_t)sm_count() * 16u), 256, 0,
                                  stream>>>((uint4 *)w.rows_send, (const uint4 *)x, w.token_list, unique_dev, tokens,
                                            world, H / 8u);
        ep_route_slot_kernel<<<(routes + 255u) / 256u, 256, 0, stream>>>(w.route_slot, w.slot, w.sorted_route,
                                                                         w.sorted_token, w.ids, routes, per, world);
        if (ep->reduced_return) {
            ep_unique_routes_kernel<<<(tokens + 255u) / 256u, 256, 0, stream>>>(
                w.unique_routes, w.unique_weights, w.ids, w.weights, w.inv_perm, w.offsets, w.slot, tokens, k, per, world);
        }
        if (!launch_ok()) return fail("row gather failed");
        // the shared expert depends only on the local tokens: on the handle's second stream it
        // runs beside the exchange (whose kernels take a few SMs) and is joined before the combine
        if (d->shared_hidden) {
            if (cudaEventRecord(ep->fork, stream) != cudaSuccess || cudaStreamWaitEvent(ep->side, ep->fork, 0) != cudaSuccess)
                return fail("stream fork failed");
            if (!(w.sh_bytes != 0 ? k3_grouped_shared_expert(d, w.sh_out, w.sh_act, x, tokens, w.sh_ws, ep->side)
                                  : k3_moe_shared_expert(d, w.sh_out, w.sh_gate, w.sh_up, w.sh_act, x, tokens, ep->side))) {
                return fail("shared expert failed");
            }
            if (cudaEventRecord(ep->join, ep->side) != cudaSuccess) return fail("stream join failed");
        }
    }

    // 4. the one host wait of the pass, then the plan
    if (cudaEventSynchronize(ep->counts_ready) != cudaSuccess) return fail("waiting for the offsets failed");
    uint32_t *plan = ep->pinned + (size_t)world * (kMaxExpertsEp + 1u + kMaxWorld);
    uint32_t *block_recv_start = plan, *block_dest_start = plan + (size_t)per * world,
             *block_rows = plan + (size_t)2u * per * world, *offsets_local = plan + (size_t)3u * per * world,
             *source_first_row = offsets_local + per + 1u, *source_route_base = source_first_row + world;
    if (!plan_impl(host_offsets, stride, world, rank, E, ep->send_rows.data(), ep->recv_rows.data(), block_recv_start,
                   block_dest_start, block_rows, offsets_local)) {
        return fail("exchange plan failed");
    }
    uint32_t n_unique = 0, n_routes_before = 0;
    for (uint32_t g = 0; g < world; g++) {
        ep->send_unique[g] = host_offsets[(size_t)rank * stride + E + 1u + g];
        ep->recv_unique[g] = host_offsets[(size_t)g * stride + E + 1u + rank];
        source_first_row[g] = n_unique;
        source_route_base[g] = n_routes_before;
        n_unique += ep->recv_unique[g];
        n_routes_before += ep->recv_rows[g];
    }
    const bool reduced = ep->reduced_return;
    if (reduced && (size_t)n_unique * k > (size_t)max_recv) return fail("workspace too small for the reduced return");
    const uint32_t n_recv = offsets_local[per];
    ep->last_recv_rows = n_recv;
    if (n_recv > max_recv) {
        char text[160];
        snprintf(text, sizeof(text), "%u rows arrive on rank %u but the workspace was sized for %u", n_recv, rank,
                 max_recv);
        return fail(text);
    }
    const size_t table_words = (size_t)3u * per * world + per + 1u + 2u * world;
    if (cudaMemcpyAsync(w.tables, plan, table_words * 4u, cudaMemcpyHostToDevice, stream) != cudaSuccess) {
        return fail("plan upload failed");
    }

    // 5. dispatch: one grouped send/recv (token rows once per destination + a slot per route),
    // the own rank's share by device copies
    {
        size_t roff_rows = 0, roff_routes = 0, soff_routes = 0, self_rows = 0, self_routes_s = 0, self_routes_r = 0;
        if (world > 1 && !nccl_ok(ep, ep->api->GroupStart(), error, error_size, "ncclGroupStart")) return false;
        for (uint32_t g = 0; g < world; g++) {
            const uint16_t *region = w.rows_send + (size_t)g * std::max(tokens, 1u) * H;
            if (g == rank) {
                self_rows = roff_rows;
                self_routes_s = soff_routes;
                self_routes_r = roff_routes;
            } else {
                if (ep->send_unique[g] != 0 &&
                    (!nccl_ok(ep, ep->api->Send(region, (size_t)ep->send_unique[g] * H, ncclBfloat16, (int)g, ep->comm, stream),
                              error, error_size, "dispatch send") ||
                     !nccl_ok(ep, ep->api->Send(w.route_slot + soff_routes, ep->send_rows[g], ncclUint32, (int)g, ep->comm,
                                                stream), error, error_size, "dispatch send of the slots"))) {
                    return false;
                }
                if (reduced && ep->send_unique[g] != 0 &&
                    (!nccl_ok(ep, ep->api->Send(w.unique_routes + (size_t)g * std::max(tokens, 1u) * k,
                                                (size_t)ep->send_unique[g] * k, ncclUint32, (int)g, ep->comm, stream), error,
                              error_size, "dispatch send of the route lists") ||
                     !nccl_ok(ep, ep->api->Send(w.unique_weights + (size_t)g * std::max(tokens, 1u) * k,
                                                (size_t)ep->send_unique[g] * k, ncclUint32, (int)g, ep->comm, stream), error,
                              error_size, "dispatch send of the route weights"))) {
                    return false;
                }
                if (ep->recv_unique[g] != 0 &&
                    (!nccl_ok(ep, ep->api->Recv(w.rows_recv + roff_rows * H, (size_t)ep->recv_unique[g] * H, ncclBfloat16,
                                                (int)g, ep->comm, stream), error, error_size, "dispatch recv") ||
                     !nccl_ok(ep, ep->api->Recv(w.slots_recv + roff_routes, ep->recv_rows[g], ncclUint32, (int)g, ep->comm,
                                                stream), error, error_size, "dispatch recv of the slots"))) {
                    return false;
                }
                if (reduced && ep->recv_unique[g] != 0 &&
                    (!nccl_ok(ep, ep->api->Recv(w.routes_recv + roff_rows * k, (size_t)ep->recv_unique[g] * k, ncclUint32,
                                                (int)g, ep->comm, stream), error, error_size, "dispatch recv of the route lists") ||
                     !nccl_ok(ep, ep->api->Recv(w.weights_recv + roff_rows * k, (size_t)ep->recv_unique[g] * k, ncclUint32,
                                                (int)g, ep->comm, stream), error, error_size, "dispatch recv of the route weights"))) {
                    return false;
                }
            }
            soff_routes += ep->send_rows[g];
            roff_rows += ep->recv_unique[g];
            roff_routes += ep->recv_rows[g];
        }
        if (world > 1 && !nccl_ok(ep, ep->api->GroupEnd(), error, error_size, "ncclGroupEnd")) return false;
        if (ep->send_unique[rank] != 0 &&
            (cudaMemcpyAsync(w.rows_recv + self_rows * H, w.rows_send + (size_t)rank * std::max(tokens, 1u) * H,
                             (size_t)ep->send_unique[rank] * H * 2u, cudaMemcpyDeviceToDevice, stream) != cudaSuccess ||
             cudaMemcpyAsync(w.slots_recv + self_routes_r, w.route_slot + self_routes_s, (size_t)ep->send_rows[rank] * 4u,
                             cudaMemcpyDeviceToDevice, stream) != cudaSuccess)) {
            return fail("copy of the rank's own rows failed");
        }
        if (reduced && ep->send_unique[rank] != 0 &&
            (cudaMemcpyAsync(w.routes_recv + self_rows * k, w.unique_routes + (size_t)rank * std::max(tokens, 1u) * k,
                             (size_t)ep->send_unique[rank] * k * 4u, cudaMemcpyDeviceToDevice, stream) != cudaSuccess ||
             cudaMemcpyAsync(w.weights_recv + self_rows * k, w.unique_weights + (size_t)rank * std::max(tokens, 1u) * k,
                             (size_t)ep->send_unique[rank] * k * 4u, cudaMemcpyDeviceToDevice, stream) != cudaSuccess)) {
            return fail("copy of the rank's own route lists failed");
        }
    }

    // 6. grouped order of the received routes, expert products on the local shard
    if (n_recv != 0) {
        const uint32_t blocks = per * world;
        const uint32_t *offsets_local_dev = w.tables + 3u * blocks;
        ep_order_slots_kernel<<<std::min<uint32_t>((blocks + 7u) / 8u, (uint32_t)sm_count() * 4u), 256, 0, stream>>>(
            w.order, w.inverse, w.slots_recv, w.tables, w.tables + blocks, w.tables + 2u * blocks,
            offsets_local_dev + per + 1u, blocks, world);
        if (!launch_ok()) return fail("order kernel launch failed");
        if (cudaEventRecord(ep->t_experts0, stream) != cudaSuccess) return fail("event record failed");
        if (w.mx_bytes != 0 && k3_grouped_mx_supported(d, n_recv)) {
            // product row p reads received row order[p]; the received rows are converted once each
            if (!k3_grouped_mx_experts(d, w.rows_out, nullptr, w.rows_recv, w.order, n_unique, offsets_local_dev, n_recv,
                                       w.mx_ws, stream)) {
                return fail("grouped expert products failed");
            }
        } else {
            uint16_t *rows_in = w.mx_bytes ? w.rows_back : w.rows_in;      // rows_back is free until step 7
            if (!k3_rocm_gather_rows_bf16(rows_in, w.rows_recv, w.order, n_recv, H, stream) ||
                !k3_moe_experts_grouped(d, w.rows_out, w.act, rows_in, offsets_local_dev, n_recv, stream)) {
                return fail("grouped expert products failed");
            }
        }
        if (cudaEventRecord(ep->t_experts1, stream) != cudaSuccess) return fail("event record failed");
        ep->timed = true;
        // 7. back into received order, and home (one row per route: the combine stays exact) -
        // or, in the reduced mode, one weighted partial sum per (token, this rank)
        if (reduced) {
            ep_reduce_kernel<<<std::min<uint32_t>((n_unique + 3u) / 4u, (uint32_t)sm_count() * 8u), 256, 0, stream>>>(
                w.rows_back, w.rows_out, w.inverse, w.routes_recv, w.weights_recv, offsets_local_dev + per + 1u,
                offsets_local_dev + per + 1u + world, world, n_unique, k, H);
            if (!launch_ok()) return fail("partial sum kernel failed");
        } else if (!k3_rocm_gather_rows_bf16(w.rows_back, w.rows_out, w.inverse, n_recv, H, stream)) {
            return fail("return gather failed");
        }
    }
    if (reduced) {
        // partial rows go home into the regions the token rows were sent from (same slots)
        size_t soff = 0;
        if (world > 1 && !nccl_ok(ep, ep->api->GroupStart(), error, error_size, "ncclGroupStart")) return false;
        for (uint32_t g = 0; g < world; g++) {
            uint16_t *region = w.rows_send + (size_t)g * std::max(tokens, 1u) * H;
            if (g != rank) {
                if (ep->recv_unique[g] != 0 &&
                    !nccl_ok(ep, ep->api->Send(w.rows_back + soff * H, (size_t)ep->recv_unique[g] * H, ncclBfloat16, (int)g,
                                               ep->comm, stream), error, error_size, "return send")) {
                    return false;
                }
                if (ep->send_unique[g] != 0 &&
                    !nccl_ok(ep, ep->api->Recv(region, (size_t)ep->send_unique[g] * H, ncclBfloat16, (int)g, ep->comm, stream),
                             error, error_size, "return recv")) {
                    return false;
                }
            }
            soff += ep->recv_unique[g];
        }
        if (world > 1 && !nccl_ok(ep, ep->api->GroupEnd(), error, error_size, "ncclGroupEnd")) return false;
        if (ep->send_unique[rank] != 0 &&
            cudaMemcpyAsync(w.rows_send + (size_t)rank * std::max(tokens, 1u) * H, w.rows_back + (size_t)source_first_row[rank] * H,
                            (size_t)ep->send_unique[rank] * H * 2u, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) {
            return fail("copy of the rank's own rows failed");
        }
    } else {
        size_t soff = 0, roff = 0, self_soff = 0, self_roff = 0;
        if (world > 1 && !nccl_ok(ep, ep->api->GroupStart(), error, error_size, "ncclGroupStart")) return false;
        for (uint32_t g = 0; g < world; g++) {
            if (g == rank) {
                self_soff = soff;
                self_roff = roff;
            } else {
                if (ep->recv_rows[g] != 0 &&
                    !nccl_ok(ep, ep->api->Send(w.rows_back + soff * H, (size_t)ep->recv_rows[g] * H, ncclBfloat16, (int)g,
                                               ep->comm, stream), error, error_size, "return send")) {
                    return false;
                }
                if (ep->send_rows[g] != 0 &&
                    !nccl_ok(ep, ep->api->Recv(w.rows_home + roff * H, (size_t)ep->send_rows[g] * H, ncclBfloat16, (int)g,
                                               ep->comm, stream), error, error_size, "return recv")) {
                    return false;
                }
            }
            soff += ep->recv_rows[g];
            roff += ep->send_rows[g];
        }
        if (world > 1 && !nccl_ok(ep, ep->api->GroupEnd(), error, error_size, "ncclGroupEnd")) return false;
        if (ep->send_rows[rank] != 0 &&
            cudaMemcpyAsync(w.rows_home + self_roff * H, w.rows_back + self_soff * H, (size_t)ep->send_rows[rank] * H * 2u,
                            cudaMemcpyDeviceToDevice, stream) != cudaSuccess) {
            return fail("copy of the rank's own rows failed");
        }
    }

    // 8. combine in rank order on the token's own rank
    if (tokens != 0) {
        if (d->shared_hidden && cudaStreamWaitEvent(stream, ep->join, 0) != cudaSuccess) return fail("stream join failed");
        if (reduced) {
            ep_combine_partials_kernel<<<std::min<uint32_t>(tokens, (uint32_t)sm_count() * 8u), 256, 0, stream>>>(
                (uint16_t *)out, w.rows_send, w.dest_mask, w.slot, d->shared_hidden ? w.sh_out : nullptr, tokens, world, H);
            if (!launch_ok()) return fail("combine failed");
        } else if (!k3_moe_combine(out, w.rows_home, w.inv_perm, w.weights, d->shared_hidden ? w.sh_out : nullptr,
                                   tokens, k, H, stream)) {
            return fail("combine failed");
        }
        if (ids_out && cudaMemcpyAsync(ids_out, w.ids, (size_t)routes * 4u, cudaMemcpyDefault, stream) != cudaSuccess)
            return fail("copy of the ids failed");
        if (weights_out &&
            cudaMemcpyAsync(weights_out, w.weights, (size_t)routes * 4u, cudaMemcpyDefault, stream) != cudaSuccess)
            return fail("copy of the weights failed");
    }
    if (cudaEventRecord(ep->t_end, stream) != cudaSuccess) return fail("event record failed");
    return true;
}

extern "C" bool k3_moe_ep_last_pass(k3_moe_ep *ep, float *experts_ms, float *pass_ms, uint32_t *recv_rows) {
    if (!ep) return false;
    if (cudaEventSynchronize(ep->t_end) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    float e = 0.f, p = 0.f;
    if ((ep->timed && cudaEventElapsedTime(&e, ep->t_experts0, ep->t_experts1) != cudaSuccess) ||
        cudaEventElapsedTime(&p, ep->t_begin, ep->t_end) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    if (experts_ms) *experts_ms = e;
    if (pass_ms) *pass_ms = p;
    if (recv_rows) *recv_rows = ep->last_recv_rows;
    return true;
}

extern "C" size_t k3_moe_ep_decode_workspace_bytes(const k3_moe_ep *ep, const k3_moe_layer_desc *d) {
    if (!shard_ok(ep, d) || !k3_decode_supported(d)) return 0;
    return carve_decode(d, nullptr).total + 256u;
}

extern "C" bool k3_moe_ep_decode(k3_moe_ep *ep, const k3_moe_layer_desc *d, void *out, const void *x,
                                 const void *residual, void *workspace, size_t workspace_bytes,
                                 void *stream_pointer) {
    if (!shard_ok(ep, d) || !k3_decode_supported(d) || !out || !x || !workspace) return false;
    char *base = (char *)(((uintptr_t)workspace + 255u) & ~(uintptr_t)255u);
    const DecodeWorkspace w = carve_decode(d, base);
    if (workspace_bytes < w.total + (size_t)(base - (char *)workspace)) return false;
    cudaStream_t stream = (cudaStream_t)stream_pointer;
    if (ep->world == 1) {
        return k3_decode_layer(d, x, w.logits, w.ids, w.weights, w.sh_gate, w.sh_up, w.sh_act, w.sh_out, w.act,
                               w.rows_out, out, residual, w.scratch, w.scratch_bytes, nullptr, stream, true);
    }
    // rows of experts held elsewhere stay zero bits, so that the integer sum over the
    // ranks below is a copy of the one rank's row
    const size_t row_bytes = (size_t)d->top_k * d->hidden * 2u;
    if (cudaMemsetAsync(w.rows_out, 0, row_bytes, stream) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    if (!k3_decode_layer(d, x, w.logits, w.ids, w.weights, w.sh_gate, w.sh_up, w.sh_act, w.sh_out, w.act, w.rows_out,
                         nullptr, nullptr, w.scratch, w.scratch_bytes, nullptr, stream, false)) {
        return false;
    }
    if (ep->api->AllReduce(w.rows_out, w.rows_out, row_bytes / 4u, ncclUint32, ncclSum, ep->comm, stream) !=
        ncclSuccess) {
        return false;
    }
    return k3_moe_combine_residual(out, w.rows_out, nullptr, w.weights, d->shared_hidden ? w.sh_out : nullptr,
                                   residual, 1u, d->top_k, d->hidden, stream);
}

extern "C" bool k3_moe_ep_decode_stack(k3_moe_ep *ep, const k3_moe_layer_desc *const *descs, uint32_t layers,
                                       void *out, const void *x, const void *norm_weight, float epsilon,
                                       void *workspace, size_t workspace_bytes, void *stream_pointer) {
    if (!ep || !descs || layers == 0 || !out || !x || !norm_weight || !workspace || !(epsilon > 0.0f)) return false;
    const uint32_t H = descs[0]->hidden;
    size_t inner = 0;
    for (uint32_t l = 0; l < layers; l++) {
        if (!descs[l] || descs[l]->hidden != H) return false;
        const size_t need = k3_moe_ep_decode_workspace_bytes(ep, descs[l]);
        if (need == 0) return false;
        inner = std::max(inner, need);
    }
    char *base = (char *)(((uintptr_t)workspace + 255u) & ~(uintptr_t)255u);
    const size_t vec = align_up((size_t)H * 2u, 256);
    if (workspace_bytes < (size_t)(base - (char *)workspace) + 3u * vec + inner) return false;
    uint16_t *h[2] = {(uint16_t *)base, (uint16_t *)(base + vec)};
    uint16_t *normed = (uint16_t *)(base + 2u * vec);
    char *layer_ws = base + 3u * vec;
    cudaStream_t stream = (cudaStream_t)stream_pointer;
    const void *cur = x;
    for (uint32_t l = 0; l < layers; l++) {
        void *next = l + 1u == layers ? out : (void *)h[l & 1u];
        if (!k3_rocm_rms_norm_bf16(normed, cur, norm_weight, 1u, H, epsilon, stream) ||
            !k3_moe_ep_decode(ep, descs[l], next, normed, cur, layer_ws, inner, stream)) {
            return false;
        }
        cur = next;
    }
    return true;
}
