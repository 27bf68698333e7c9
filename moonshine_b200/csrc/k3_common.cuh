// Shared device helpers for the routed-MoE kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <map>
#include <mutex>
#include <utility>

#define K3_DEVINL __device__ __forceinline__

namespace k3 {

constexpr int kWarp = 32;

K3_DEVINL float bf16_bits_to_float(uint32_t bits16) {
    return __uint_as_float(bits16 << 16);
}

// float -> bf16 bit pattern, round-to-nearest-even (hip_bfloat16(float) semantics).
K3_DEVINL uint16_t float_to_bf16_bits(float value) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(value));
}

K3_DEVINL float bf16_lo(uint32_t pair) { return __uint_as_float(pair << 16); }
K3_DEVINL float bf16_hi(uint32_t pair) { return __uint_as_float(pair & 0xffff0000u); }

// E8M0 scale byte -> float: 2^(b-127); b == 0 decodes to 2^-127 (a subnormal),
// as k3_rocm_ops.cu:179-183 of the reference does.
K3_DEVINL float e8m0_to_float(uint32_t exponent) {
    return __uint_as_float(exponent == 0u ? 0x00400000u : exponent << 23);
}

K3_DEVINL float e2m1_to_float(uint32_t nibble) {
    // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 : exponent/mantissa bits of the code
    // placed into an fp32 pattern and rescaled (exact).
    const uint32_t mag = nibble & 7u;
    const float value = __uint_as_float(mag << 22) * 0x1p126f;
    return (nibble & 8u) ? -value : value;
}

K3_DEVINL float sigmoid_exact(float x) { return 1.0f / (1.0f + expf(-x)); }

enum Activation : int { kActSitu = 0, kActSwiglu = 1 };

K3_DEVINL float activation(float g, float u, int kind, float beta, float linear_beta) {
    const float sig = 1.0f / (1.0f + expf(-g));
    if (kind == kActSitu) {
        const float bounded_gate = __fmul_rn(beta, tanhf(g / beta));
        const float bounded_up = __fmul_rn(linear_beta, tanhf(u / linear_beta));
        return __fmul_rn(__fmul_rn(bounded_gate, sig), bounded_up);
    }
    return __fmul_rn(__fmul_rn(g, sig), u);
}

K3_DEVINL float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

K3_DEVINL float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// 16-byte global load that does not allocate in L1 (weights are streamed once).
K3_DEVINL uint4 ld_stream_16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

K3_DEVINL uint2 ld_stream_8(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
                 : "=r"(v.x), "=r"(v.y)
                 : "l"(p));
    return v;
}

inline bool launch_ok() { return cudaGetLastError() == cudaSuccess; }

// Host-side per-device state.  One process may drive several GPUs, and both the SM
// count and a kernel's dynamic shared-memory limit belong to the device that is
// current when the call is made.
constexpr int kMaxDevices = 64;

inline int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return dev;
}

inline int sm_count() {
    static std::atomic<int> cached[kMaxDevices];
    const int dev = current_device();
    if (dev < 0 || dev >= kMaxDevices) return 148;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            return 148;
        }
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize for `kernel` on the current device,
// remembered per (device, kernel) so that the call is made once each (it costs
// microseconds of host time).  Requests of 48 KB or less need no attribute.
inline bool set_max_dynamic_smem(const void *kernel, size_t bytes) {
    if (bytes <= 48u * 1024u) return true;
    static std::mutex lock;
    static std::map<std::pair<int, const void *>, size_t> done;
    const int dev = current_device();
    std::lock_guard<std::mutex> guard(lock);
    const auto key = std::make_pair(dev, kernel);
    auto it = done.find(key);
    if (it != done.end() && it->second >= bytes) return true;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    done[key] = bytes;
    return true;
}

// Kernels meant to share an SM with a kernel that needs most of its shared memory must
// ask for the same split between L1 and shared memory: an SM changes the split only when
// it is empty, so a block with a smaller preference waits for the large kernel to leave
// (and the other way round).  Sets the preference to the maximum once per (device, kernel).
inline bool prefer_max_shared_carveout(const void *kernel) {
    static std::mutex lock;
    static std::map<std::pair<int, const void *>, bool> done;
    const int dev = current_device();
    std::lock_guard<std::mutex> guard(lock);
    const auto key = std::make_pair(dev, kernel);
    if (done.count(key)) return true;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                             (int)cudaSharedmemCarveoutMaxShared) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    done[key] = true;
    return true;
}

}  // namespace k3
