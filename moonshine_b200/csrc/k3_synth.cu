// Seeded synthetic tensor fills (test and benchmark inputs).  Integer recipe
// shared with moonshine_b200/synth.py: chunk c of 8 bytes is the little-endian
// image of splitmix64-finalise(key * golden + golden + c).
#include "k3_common.cuh"
#include "k3_moe_layer.h"

namespace {

__host__ __device__ inline uint64_t hash64(uint64_t base, uint64_t index) {
    uint64_t z = index + base;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

inline uint64_t key_base(uint64_t key) { return key * 0x9E3779B97F4A7C15ull + 0x9E3779B97F4A7C15ull; }

// mode 0: low + floor(b*span/256) ; mode 1: int8 in [-127,127]
__global__ void fill_bytes_kernel(uint8_t *out, uint64_t count, uint64_t base, uint64_t first_chunk,
                                  uint32_t low, uint32_t span, int mode) {
    const uint64_t chunks = (count + 7) / 8;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += stride) {
        const uint64_t z = hash64(base, first_chunk + c);
        uint64_t packed = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t b = (uint32_t)(z >> (8 * j)) & 0xffu;
            const uint32_t v = mode == 0 ? low + ((b * span) >> 8)
                                         : (uint32_t)(int32_t)(((b * 255u) >> 8) - 127) & 0xffu;
            packed |= (uint64_t)(v & 0xffu) << (8 * j);
        }
        if (c * 8 + 8 <= count && (((uintptr_t)out) & 7u) == 0) {
            reinterpret_cast<uint64_t *>(out)[c] = packed;
        } else {
            for (int j = 0; j < 8 && c * 8 + j < count; j++) out[c * 8 + j] = (uint8_t)(packed >> (8 * j));
        }
    }
}

__global__ void fill_uniform_kernel(void *out, uint64_t count, uint64_t base, uint64_t first,
                                    float low, float width, int as_f16) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        const float u = (float)(uint32_t)(hash64(base, first + i) >> 40) * 5.9604644775390625e-8f;
        const float v = __fadd_rn(__fmul_rn(u, width), low);
        if (as_f16) reinterpret_cast<__half *>(out)[i] = __float2half_rn(v);
        else reinterpret_cast<float *>(out)[i] = v;
    }
}

inline uint32_t blocks_for(uint64_t items) {
    uint64_t b = (items + 255) / 256;
    const uint64_t cap = (uint64_t)k3::sm_count() * 16;
    return (uint32_t)(b > cap ? cap : (b == 0 ? 1 : b));
}

}  // namespace

extern "C" bool k3_synth_fill_bytes(void *out, uint64_t count, uint64_t key, uint64_t first,
                                    uint32_t low, uint32_t span, void *stream) {
    if (!out || count == 0 || span == 0 || low + span > 256u || first % 8u != 0) return false;
    fill_bytes_kernel<<<blocks_for((count + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
        (uint8_t *)out, count, key_base(key), first / 8u, low, span, 0);
    return k3::launch_ok();
}

extern "C" bool k3_synth_fill_int8(void *out, uint64_t count, uint64_t key, uint64_t first,
                                   void *stream) {
    if (!out || count == 0 || first % 8u != 0) return false;
    fill_bytes_kernel<<<blocks_for((count + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
        (uint8_t *)out, count, key_base(key), first / 8u, 0, 0, 1);
    return k3::launch_ok();
}

extern "C" bool k3_synth_fill_uniform(void *out, uint64_t count, uint64_t key, uint64_t first,
                                      float low, float width, int as_f16, void *stream) {
    if (!out || count == 0) return false;
    fill_uniform_kernel<<<blocks_for(count), 256, 0, (cudaStream_t)stream>>>(
        out, count, key_base(key), first, low, width, as_f16);
    return k3::launch_ok();
}
