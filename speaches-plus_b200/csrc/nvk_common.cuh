// Shared device/host helpers for the NVFP4 linear path (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <mutex>

#include "nvk_launch.cuh"

// Return codes follow the reference launchers: 0 = enqueued, -1 = shape/route refused
// without launching, -2 = bad argument/alignment, -3 = resource limit, -9 = grid axis too
// large; a positive value is a cudaError_t.
#define NVK_OK 0
#define NVK_ERR_SHAPE (-1)
#define NVK_ERR_ARG (-2)
#define NVK_ERR_RESOURCE (-3)
#define NVK_ERR_GRID_AXIS (-9)

namespace nvk {

// True if any of the pointers is null.  Launchers refuse null operands (NVK_ERR_ARG) after their
// shape checks instead of handing them to a kernel.
template <typename... P>
inline bool any_null(P... ptrs) {
    const void* v[] = {static_cast<const void*>(ptrs)...};
    for (const void* q : v)
        if (q == nullptr) return true;
    return false;
}


__host__ __device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Byte offset of the ue4m3 scale of (row m, 16-block kb) in the 128x4 swizzled layout
// (the tcgen05 block-scale atom): 512-byte tiles of 128 rows x 4 blocks, tile-major by
// (row tile, k tile); inside a tile byte = (m%32)*16 + ((m/32)%4)*4 + kb%4.
__host__ __device__ __forceinline__ size_t swz_offset(int m, int kb, int k_blocks) {
    size_t k_tiles = (size_t)((k_blocks + 3) >> 2);
    return (((size_t)(m >> 7) * k_tiles + (size_t)(kb >> 2)) * 32 + (size_t)(m & 31)) * 16 +
           (size_t)((m >> 5) & 3) * 4 + (size_t)(kb & 3);
}

// ue4m3 byte -> f32.  Bits 6..3 exponent (bias 7), 2..0 mantissa, exponent 0 = m * 2^-9.
// Placing the 7 payload bits at f32 bits 26..20 yields value * 2^-120 with f32 subnormals
// covering the exponent-0 case, so one multiply by 2^120 decodes every byte exactly
// (bit 7 is ignored, 0x7F decodes to 480 like the formula does).
__device__ __forceinline__ float ue4m3_to_f32(uint32_t b) {
    return __uint_as_float((b & 0x7Fu) << 20) * 1.329227995784916e36f;  // 2^120
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b16) { return __uint_as_float(b16 << 16); }

__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}

// Four packed e2m1 bytes (8 values, even element in the low nibble) -> four f16x2.
__device__ __forceinline__ void e2m1x8_to_f16x2x4(uint32_t w, uint32_t& h0, uint32_t& h1, uint32_t& h2,
                                                  uint32_t& h3) {
    ptx::e2m1x8_to_f16x2x4(w, h0, h1, h2, h3);
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) { return ptx::hmul2(a, b); }
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) { return ptx::hfma2(a, b, c); }

// e2m1 nearest-code search, first minimum wins (ties go to the lower code).
__device__ __forceinline__ uint32_t encode_e2m1(float x) {
    const float a = fabsf(x);
    // Midpoints of the codebook {0,.5,1,1.5,2,3,4,6}; "greater than" keeps ties low.
    uint32_t c = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
    return c | (signbit(x) ? 8u : 0u);
}

// ue4m3 encoder: clamp to 448, subnormal grid below 2^-6, round-half-away mantissa with
// carry, never emits 0x7F.  Exponent from the f32 bit field (exact floor(log2)).
__device__ __forceinline__ uint32_t encode_ue4m3(float s) {
    if (!(s > 0.f) || !isfinite(s)) return 0u;
    const float c = fminf(s, 448.f);
    if (c < 0.015625f) {
        int m = (int)roundf(c / 0.001953125f);
        return m <= 0 ? 0u : (m <= 7 ? (uint32_t)m : 8u);
    }
    int e2;
    (void)frexpf(c, &e2);
    int ex = e2 - 1;
    float mf = ldexpf(c, -ex) - 1.f;
    int mant = (int)roundf(mf * 8.f);
    if (mant < 0) mant = 0;
    if (mant > 7) {
        mant = 0;
        ex += 1;
    }
    int biased = ex + 7;
    biased = biased < 1 ? 1 : (biased > 15 ? 15 : biased);
    uint32_t byte = ((uint32_t)biased << 3) | (uint32_t)mant;
    return byte == 0x7Fu ? 0x7Eu : byte;
}

// Polls *p (acquire, system scope) until it is >= target or `limit` polls have passed; false = gave up.
// Every wait on another CTA or GPU in this library goes through here: none of them is unbounded.
__device__ __forceinline__ bool bounded_wait_ge(const uint32_t* p, uint32_t target, uint32_t limit) {
    for (uint32_t polls = 0; ptx::ld_acquire_sys(p) < target;)
        if (++polls > limit) return false;
    return true;
}

// Polls per wait before a kernel gives up (about a second on the device); nvk_b200_set_wait_limit
// changes it for later calls of the calling thread.
constexpr uint32_t kDefaultWaitLimit = 2000000u;
inline uint32_t& wait_limit_setting() {
    static thread_local uint32_t polls = kDefaultWaitLimit;
    return polls;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Raise the dynamic shared memory limit of a kernel, never lower it.  The attribute belongs to the
// current device's context, so the raised size is remembered per device; callable from any thread.
struct SmemOptin {
    static constexpr int kMaxDevices = 64;
    size_t raised[kMaxDevices] = {};
    std::mutex mu;
    int ensure(const void* func, size_t bytes) {
        if (bytes <= 48 * 1024) return 0;
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return (int)e;
        if (dev < 0 || dev >= kMaxDevices) return NVK_ERR_ARG;
        std::lock_guard<std::mutex> lock(mu);
        if (bytes <= raised[dev]) return 0;
        e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return (int)e;
        raised[dev] = bytes;
        return 0;
    }
};

}  // namespace nvk
