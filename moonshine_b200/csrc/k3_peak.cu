// Tensor-pipe peak of one SM group of MMA kinds, measured: one CTA per SM issues
// tcgen05.mma back to back on operand tiles that stay in shared memory (no loads
// inside the loop), so the figure is the ceiling of the instruction kind itself.
// Kinds: bf16 (kind::f16), block-scaled E2M1 x E4M3 (kind::mxf8f6f4, the kind the
// expert kernels use) and block-scaled E2M1 x E2M1 (kind::mxf4, the MXFP4 peak).
// M = 128, N = 256 per instruction: the shape with the least shared-memory traffic
// per FLOP.  The accumulated values are never read: only the rate matters.
#include "k3_moe_layer.h"
#include "k3_tc_ptx.cuh"

using namespace k3;
using namespace k3::tc;

namespace {

constexpr uint32_t kPeakThreads = 128;
constexpr uint32_t kATile = 128 * 128;        // 128 rows x one 128-byte swizzle row
constexpr uint32_t kBTile = 256 * 128;
constexpr uint32_t kSmem = kATile + kBTile + 1024 + 64;
constexpr uint32_t kScaleCol = 256;           // scale columns behind the 256 accumulator columns

enum PeakKind : int { kPeakBf16 = 0, kPeakMxf8f6f4 = 1, kPeakMxf4 = 2 };

__device__ uint32_t g_peak_status = 0;

K3_DEVINL void mma_block_scaled(bool mxf4, uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa,
                                uint32_t sfb, uint32_t acc) {
    if (mxf4) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::
                "r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::
                "r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc)
            : "memory");
    }
}

K3_DEVINL void tmem_st_32x4(uint32_t taddr, uint32_t v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %1, %1, %1};" ::"r"(taddr), "r"(v) : "memory");
}

__global__ void __launch_bounds__(kPeakThreads, 1) peak_kernel(int kind, uint32_t n, uint32_t iterations) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t *done = reinterpret_cast<uint64_t *>(base + kATile + kBTile);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(done + 1);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const uint32_t warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    // operand bytes: small finite values in every format used (E4M3 / E2M1 pairs / bf16 halves)
    for (uint32_t i = threadIdx.x; i < (kATile + kBTile) / 4u; i += blockDim.x) {
        const uint32_t h = (i * 2654435761u) ^ (blockIdx.x * 40503u);
        reinterpret_cast<uint32_t *>(base)[i] = 0x30303030u | (h & 0x07070707u);
    }
    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        mbar_init(done, 1);
        fence_barrier_init();
    }
    fence_proxy_async();
    if (warp == 0) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // block scales of 1.0 (E8M0 byte 127) in eight columns of every lane
    tmem_st_32x4(tmem + ((32u * warp) << 16) + kScaleCol, 0x7f7f7f7fu);
    tmem_st_32x4(tmem + ((32u * warp) << 16) + kScaleCol + 4u, 0x7f7f7f7fu);
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) {
        tc_fence_after();
        const uint64_t da = make_desc_sw128(smem_u32(base));
        const uint64_t db = make_desc_sw128(smem_u32(base + kATile));
        if (kind == kPeakBf16) {
            const uint32_t idesc = make_idesc_bf16(128, n);
            for (uint32_t it = 0; it < iterations; it++) {
#pragma unroll
                for (uint32_t j = 0; j < 4u; j++) mma_f16_ss(tmem, da + 2u * j, db + 2u * j, idesc, (it | j) != 0u);
            }
        } else {
            const bool mxf4 = kind == kPeakMxf4;
            // A E2M1, B E4M3 (mxf8f6f4) or E2M1 (mxf4), UE8M0 scales, M = 128, N = 256
            const uint32_t formats = mxf4 ? ((1u << 7) | (1u << 10)) : ((5u << 7) | (0u << 10));
            const uint32_t common = formats | ((n >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);
            for (uint32_t it = 0; it < iterations; it++) {
#pragma unroll
                for (uint32_t j = 0; j < 4u; j++) {
                    // scale id: byte j of the column (1X), or byte pair 0 / 2 (2X)
                    const uint32_t sf = mxf4 ? 2u * (j & 1u) : j;
                    mma_block_scaled(mxf4, tmem, da + 2u * j, db + 2u * j, common | (sf << 29) | (sf << 4),
                                     tmem + kScaleCol, tmem + kScaleCol + 4u, (it | j) != 0u);
                }
            }
        }
        mma_commit(done);
        if (!mbar_wait(done, 0u, abort_flag)) atomicExch(&g_peak_status, 1u);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace

// kind: 0 bf16, 1 mxf8f6f4 block-scaled (E2M1 x E4M3), 2 mxf4 block-scaled.  Launches one
// CTA per SM, each issuing 4 * iterations MMAs of M = 128 and N = n (16 .. 256, a multiple of
// 16) on operands that stay in shared memory; *flop_per_launch (optional) receives the
// floating-point operations of the whole launch.  Time it with events.
extern "C" bool k3_moe_peak_launch_n(int kind, uint32_t n, uint32_t iterations, double *flop_per_launch,
                                     void *stream) {
    if (kind < 0 || kind > 2 || iterations == 0u || iterations > 4000000u || n < 16u || n > 256u || n % 16u != 0u)
        return false;
    if (!set_max_dynamic_smem((const void *)peak_kernel, kSmem)) return false;
    const int sms = sm_count();
    const uint32_t k_per_mma = kind == kPeakBf16 ? 16u : kind == kPeakMxf8f6f4 ? 32u : 64u;
    if (flop_per_launch) *flop_per_launch = 2.0 * 128.0 * (double)n * k_per_mma * 4.0 * iterations * sms;
    peak_kernel<<<sms, kPeakThreads, kSmem, (cudaStream_t)stream>>>(kind, n, iterations);
    return launch_ok();
}

// N = 256: the shape with the least operand traffic per operation.
extern "C" bool k3_moe_peak_launch(int kind, uint32_t iterations, double *flop_per_launch, void *stream) {
    return k3_moe_peak_launch_n(kind, 256u, iterations, flop_per_launch, stream);
}
