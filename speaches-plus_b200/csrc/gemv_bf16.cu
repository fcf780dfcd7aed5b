// bf16 weight GEMV at M=1 (the lm_head of a decode step): y[n] = bf16( sum_k W[n,k] * x[k] ),
// fp32 accumulate.  One warp per output row, 128-bit coalesced weight loads with four in flight
// per lane; x (a few KB) is re-read through L1.
#include "nvk_common.cuh"

namespace {

using nvk::ptx::ldg_stream_v4;

__device__ __forceinline__ float dot8(const uint4& w, const uint4& x, float acc) {
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w}, xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        acc = fmaf(__uint_as_float(ws[i] << 16), __uint_as_float(xs[i] << 16), acc);
        acc = fmaf(__uint_as_float(ws[i] & 0xFFFF0000u), __uint_as_float(xs[i] & 0xFFFF0000u), acc);
    }
    return acc;
}

template <bool VEC>
__global__ void __launch_bounds__(256) gemv_bf16_kernel(const uint16_t* __restrict__ W, const uint16_t* __restrict__ x,
                                                        uint16_t* __restrict__ y, int N, int K) {
    // stream order through programmatic dependent launch: nothing of the predecessor's is read before this
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (n >= N) return;
    const uint16_t* wr = W + (size_t)n * K;
    float acc = 0.f;
    if (VEC) {
        const int nv = K >> 3;  // 16-byte pieces per row
        const uint4* w4 = reinterpret_cast<const uint4*>(wr);
        const uint4* x4 = reinterpret_cast<const uint4*>(x);
        int i = lane;
        for (; i + 96 < nv; i += 128) {
            const uint4 a = ldg_stream_v4(w4 + i), b = ldg_stream_v4(w4 + i + 32), c = ldg_stream_v4(w4 + i + 64),
                        d = ldg_stream_v4(w4 + i + 96);
            acc = dot8(a, __ldg(x4 + i), acc);
            acc = dot8(b, __ldg(x4 + i + 32), acc);
            acc = dot8(c, __ldg(x4 + i + 64), acc);
            acc = dot8(d, __ldg(x4 + i + 96), acc);
        }
        for (; i < nv; i += 32) acc = dot8(ldg_stream_v4(w4 + i), __ldg(x4 + i), acc);
    } else {
        for (int k = lane; k < K; k += 32)
            acc = fmaf(nvk::bf16_bits_to_f32(wr[k]), nvk::bf16_bits_to_f32(x[k]), acc);
    }
    acc = nvk::warp_sum(acc);
    if (lane == 0) y[n] = nvk::f32_to_bf16_bits(acc);
}

}  // namespace

extern "C" int nv_kernels_gemv_bf16(void* stream, const uint16_t* W, const uint16_t* x, uint16_t* y, int N, int K) {
    if (N <= 0 || K <= 0) return 0;
    if (nvk::any_null(W, x, y)) return NVK_ERR_ARG;
    const unsigned grid = (unsigned)((N + 7) / 8);
    const bool vec = (K & 7) == 0 && ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(x)) & 15u) == 0;
    const nvk::Launch l = nvk::launch_1d((cudaStream_t)stream, grid, 256, 0, true);
    return vec ? nvk::launch(l, gemv_bf16_kernel<true>, W, x, y, N, K) : nvk::launch(l, gemv_bf16_kernel<false>, W, x, y, N, K);
}

extern "C" int nv_kernels_capability(int* sm_major, int* sm_minor) {
    int dev = 0, major = 0, minor = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (e != cudaSuccess) return (int)e;
    if (sm_major) *sm_major = major;
    if (sm_minor) *sm_minor = minor;
    return 0;
}
