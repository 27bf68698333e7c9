// Token-to-expert dispatch on the device: histogram, prefix scan and a stable
// permutation that reproduces the reference's grouping order - experts
// ascending, and inside one expert routes (token*top_k + rank) ascending -
// which the reference builds on the host by scanning all routes once per
// expert (k3_engine_prefill.inc:1175-1194).
//
// Routes are cut into chunks of kChunk consecutive routes, one warp per chunk.
//   pass 1: per-chunk histogram                      -> hist[chunk][expert]
//   pass 2: per expert, exclusive scan over chunks and over experts
//   pass 3: each warp walks its chunk in order; lanes holding the same expert
//           rank themselves with __match_any_sync, so the placement is stable.
#include "k3_common.cuh"
#include "k3_moe_layer.h"

using namespace k3;

namespace {

constexpr uint32_t kChunk = 512;        // routes per warp
constexpr uint32_t kWarpsPerBlock = 4;
constexpr uint32_t kMaxExperts = 1024;

// Set (to 2) when a dispatch saw an expert id >= experts; read by k3_moe_device_status().
// Such routes are counted nowhere and placed nowhere, so the outputs of that call
// are incomplete.  Shared by both dispatch entry points.
__device__ uint32_t g_dispatch_status = 0;

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
route_hist_kernel(uint32_t *__restrict__ hist, const uint32_t *__restrict__ ids,
                  uint32_t routes, uint32_t experts, uint32_t chunks,
                  uint32_t *__restrict__ error_flag) {
    extern __shared__ uint32_t smem_hist[];   // [kWarpsPerBlock][experts]
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t chunk = blockIdx.x * kWarpsPerBlock + warp;
    uint32_t *h = smem_hist + warp * experts;
    for (uint32_t e = lane; e < experts; e += kWarp) h[e] = 0u;
    __syncwarp();
    if (chunk < chunks) {
        const uint32_t begin = chunk * kChunk;
        const uint32_t end = min(routes, begin + kChunk);
        for (uint32_t r = begin + lane; r < end; r += kWarp) {
            const uint32_t e = ids[r];
            if (e < experts) atomicAdd(&h[e], 1u);
            else {                                     // invalid route id
                atomicExch(error_flag, 1u);
                g_dispatch_status = 2u;
            }
        }
        __syncwarp();
        for (uint32_t e = lane; e < experts; e += kWarp) {
            hist[(uint64_t)chunk * experts + e] = h[e];
        }
    }
}

// One block, one thread per expert.
__global__ void __launch_bounds__(kMaxExperts)
route_scan_kernel(uint32_t *__restrict__ hist, uint32_t *__restrict__ offsets,
                  uint32_t experts, uint32_t chunks) {
    __shared__ uint32_t warp_sums[kMaxExperts / 32];
    const uint32_t e = threadIdx.x;
    uint32_t running = 0u;
    if (e < experts) {
        for (uint32_t c = 0; c < chunks; c++) {
            const uint64_t i = (uint64_t)c * experts + e;
            const uint32_t v = hist[i];
            hist[i] = running;
            running += v;
        }
    }
    // exclusive scan over experts
    const uint32_t lane = e % kWarp, warp = e / kWarp;
    uint32_t incl = running;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= (uint32_t)o) incl += n;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = lane < kMaxExperts / 32 ? warp_sums[lane] : 0u;
        uint32_t wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t n = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= (uint32_t)o) wi += n;
        }
        warp_sums[lane] = wi - w;   // exclusive
    }
    __syncthreads();
    const uint32_t excl = warp_sums[warp] + incl - running;
    if (e < experts) offsets[e] = excl;
    if (e == experts - 1u) offsets[experts] = excl + running;
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
route_place_kernel(uint32_t *__restrict__ sorted_route, uint32_t *__restrict__ sorted_token,
                   uint32_t *__restrict__ inv_perm, const uint32_t *__restrict__ hist,
                   const uint32_t *__restrict__ offsets, const uint32_t *__restrict__ ids,
                   uint32_t routes, uint32_t experts, uint32_t chunks, uint32_t top_k) {
    extern __shared__ uint32_t smem_cursor[];   // [kWarpsPerBlock][experts]
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const uint32_t chunk = blockIdx.x * kWarpsPerBlock + warp;
    if (chunk >= chunks) return;
    uint32_t *cursor = smem_cursor + warp * experts;
    for (uint32_t e = lane; e < experts; e += kWarp) {
        cursor[e] = offsets[e] + hist[(uint64_t)chunk * experts + e];
    }
    __syncwarp();
    const uint32_t begin = chunk * kChunk;
    const uint32_t end = min(routes, begin + kChunk);
    for (uint32_t r0 = begin; r0 < end; r0 += kWarp) {
        const uint32_t r = r0 + lane;
        const bool valid = r < end;
        const uint32_t e = valid ? ids[r] : 0xffffffffu;
        const bool usable = valid && e < experts;
        const uint32_t active = __ballot_sync(0xffffffffu, usable);
        if (usable) {
            const uint32_t peers = __match_any_sync(active, e);
            const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
            const uint32_t base = cursor[e];
            __syncwarp(active);
            if (rank == 0u) cursor[e] = base + __popc(peers);
            const uint32_t pos = base + rank;
            sorted_route[pos] = r;
            sorted_token[pos] = r / top_k;
            inv_perm[r] = pos;
        }
        __syncwarp();
    }
}

}  // namespace

uint32_t k3_dispatch_status() {
    uint32_t v = 0xffffffffu;
    if (cudaMemcpyFromSymbol(&v, g_dispatch_status, sizeof(v)) != cudaSuccess) (void)cudaGetLastError();
    return v;
}

bool k3_dispatch_status_clear() {
    const uint32_t zero = 0u;
    if (cudaMemcpyToSymbol(g_dispatch_status, &zero, sizeof(zero)) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return true;
}

extern "C" size_t k3_moe_dispatch_workspace_bytes(uint32_t tokens, uint32_t top_k,
                                                  uint32_t experts) {
    const uint64_t routes = (uint64_t)tokens * top_k;
    const uint64_t chunks = (routes + kChunk - 1) / kChunk;
    return (size_t)(chunks * experts * sizeof(uint32_t) + 256);
}

extern "C" bool k3_moe_dispatch_build(void *offsets, void *sorted_route, void *sorted_token,
                                      void *inv_perm, const void *expert_ids, uint32_t tokens,
                                      uint32_t top_k, uint32_t experts, void *workspace,
                                      size_t workspace_bytes, void *stream_pointer) {
    if (!offsets || !sorted_route || !sorted_token || !inv_perm || !expert_ids || !workspace ||
        tokens == 0u || top_k == 0u || experts == 0u || experts > kMaxExperts) {
        return false;
    }
    const uint64_t routes64 = (uint64_t)tokens * top_k;
    if (routes64 > 0x7fffffffull) return false;
    if (workspace_bytes < k3_moe_dispatch_workspace_bytes(tokens, top_k, experts)) return false;
    const uint32_t routes = (uint32_t)routes64;
    const uint32_t chunks = (routes + kChunk - 1) / kChunk;
    cudaStream_t stream = (cudaStream_t)stream_pointer;
    uint32_t *error_flag = (uint32_t *)workspace;          // first 256 bytes: status words
    uint32_t *hist = (uint32_t *)((char *)workspace + 256);
    if (cudaMemsetAsync(error_flag, 0, 256, stream) != cudaSuccess) return false;
    const uint32_t blocks = (chunks + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const size_t smem = (size_t)kWarpsPerBlock * experts * sizeof(uint32_t);
    route_hist_kernel<<<blocks, kWarpsPerBlock * 32, smem, stream>>>(
        hist, (const uint32_t *)expert_ids, routes, experts, chunks, error_flag);
    if (!launch_ok()) return false;
    route_scan_kernel<<<1, kMaxExperts, 0, stream>>>(hist, (uint32_t *)offsets, experts, chunks);
    if (!launch_ok()) return false;
    route_place_kernel<<<blocks, kWarpsPerBlock * 32, smem, stream>>>(
        (uint32_t *)sorted_route, (uint32_t *)sorted_token, (uint32_t *)inv_perm, hist,
        (const uint32_t *)offsets, (const uint32_t *)expert_ids, routes, experts, chunks, top_k);
    return launch_ok();
}

// ---------------------------------------------------------------------------
// Dispatch for callers that cannot allocate device memory.
//
// Some hosts of this library never get to call cudaMalloc themselves: a plugin
// loaded into an engine whose memory pool was sized and handed out at start-up
// (the reference engine does exactly that: every buffer is carved from one
// preflighted allocation and the operators "never allocate"), or a call site
// that runs while allocation is forbidden.  k3_moe_dispatch_build needs a
// caller-supplied workspace for its per-chunk histograms; this variant keeps
// that workspace in a fixed array inside the library's device image instead.
// The array exists once per GPU that loads the library, for the life of the
// process, and costs kNoAllocScratchBytes (about 1 MiB) of device memory there.
//
// Limits and rules:
//   * tokens * top_k <= kNoAllocMaxRoutes (131072) and experts <= 1024; larger
//     problems are refused with a message, nothing is launched.
//   * All calls on one GPU share the array.  Two calls whose kernels overlap in
//     time (different streams, or different host threads) corrupt each other's
//     histograms: serialise them on one stream.  The array keeps the previous
//     call's contents; the status words are cleared and every histogram entry
//     a call reads is rewritten by that call first.
//   * The first call on each GPU looks up the array's device address
//     (cudaGetSymbolAddress, with that GPU current).  Make that first call
//     outside any stream capture.
// No cudaMalloc, cudaFree or other allocating routine is called.
constexpr uint32_t kNoAllocMaxRoutes = 131072;
constexpr uint32_t kNoAllocMaxChunks = kNoAllocMaxRoutes / kChunk;
constexpr size_t kNoAllocScratchBytes = 256 + (size_t)kNoAllocMaxChunks * kMaxExperts * sizeof(uint32_t);

static __device__ __align__(256) unsigned char g_dispatch_scratch[kNoAllocScratchBytes];

namespace {

// device address of g_dispatch_scratch per GPU; several host threads may make the first call
std::atomic<void *> g_scratch_address[kMaxDevices];

void set_error(char *error, size_t error_size, const char *message) {
    if (!error || error_size == 0) return;
    size_t i = 0;
    for (; message[i] != '\0' && i + 1 < error_size; i++) error[i] = message[i];
    error[i] = '\0';
}

// The array's name is only a host-side handle: kernels must be given the address
// cudaGetSymbolAddress reports for the current device.
void *scratch_for_current_device(char *error, size_t error_size) {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        (void)cudaGetLastError();
        set_error(error, error_size, "no current CUDA device (or ordinal >= 64)");
        return nullptr;
    }
    void *address = g_scratch_address[device].load(std::memory_order_acquire);
    if (address == nullptr) {
        if (cudaGetSymbolAddress(&address, g_dispatch_scratch) != cudaSuccess || !address) {
            (void)cudaGetLastError();
            set_error(error, error_size, "cudaGetSymbolAddress failed for the dispatch scratch");
            return nullptr;
        }
        g_scratch_address[device].store(address, std::memory_order_release);   // same value from every thread
    }
    return address;
}

}  // namespace

extern "C" size_t k3_moe_dispatch_noalloc_max_routes(void) { return kNoAllocMaxRoutes; }

extern "C" bool k3_moe_dispatch_build_noalloc(void *offsets, void *sorted_route,
                                              void *sorted_token, void *inv_perm,
                                              const void *expert_ids, uint32_t tokens,
                                              uint32_t top_k, uint32_t experts, char *error,
                                              size_t error_size, void *stream_pointer) {
    set_error(error, error_size, "");
    if (!offsets || !sorted_route || !sorted_token || !inv_perm || !expert_ids || tokens == 0u ||
        top_k == 0u || experts == 0u) {
        set_error(error, error_size, "null pointer or zero size");
        return false;
    }
    const uint64_t routes64 = (uint64_t)tokens * top_k;
    if (routes64 > kNoAllocMaxRoutes || experts > kMaxExperts) {
        set_error(error, error_size,
                  "problem exceeds the built-in scratch: tokens*top_k must be <= 131072 and "
                  "experts <= 1024; use k3_moe_dispatch_build with a caller workspace");
        return false;
    }
    unsigned char *scratch = (unsigned char *)scratch_for_current_device(error, error_size);
    if (!scratch) return false;
    const uint32_t routes = (uint32_t)routes64;
    const uint32_t chunks = (routes + kChunk - 1) / kChunk;
    cudaStream_t stream = (cudaStream_t)stream_pointer;
    uint32_t *error_flag = (uint32_t *)scratch;                 // status words, must start at zero
    uint32_t *hist = (uint32_t *)(scratch + 256);               // rewritten below before it is read
    if (cudaMemsetAsync(error_flag, 0, 256, stream) != cudaSuccess) {
        (void)cudaGetLastError();
        set_error(error, error_size, "cudaMemsetAsync of the status words failed");
        return false;
    }
    const uint32_t blocks = (chunks + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const size_t smem = (size_t)kWarpsPerBlock * experts * sizeof(uint32_t);
    route_hist_kernel<<<blocks, kWarpsPerBlock * 32, smem, stream>>>(
        hist, (const uint32_t *)expert_ids, routes, experts, chunks, error_flag);
    if (!launch_ok()) {
        set_error(error, error_size, "histogram kernel launch failed");
        return false;
    }
    route_scan_kernel<<<1, kMaxExperts, 0, stream>>>(hist, (uint32_t *)offsets, experts, chunks);
    if (!launch_ok()) {
        set_error(error, error_size, "scan kernel launch failed");
        return false;
    }
    route_place_kernel<<<blocks, kWarpsPerBlock * 32, smem, stream>>>(
        (uint32_t *)sorted_route, (uint32_t *)sorted_token, (uint32_t *)inv_perm, hist,
        (const uint32_t *)offsets, (const uint32_t *)expert_ids, routes, experts, chunks, top_k);
    if (!launch_ok()) {
        set_error(error, error_size, "placement kernel launch failed");
        return false;
    }
    return true;
}
