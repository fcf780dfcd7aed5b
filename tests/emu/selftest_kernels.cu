// Kernels that exist only to check the emulation's race checker: one rotates a shared-memory array with
// the barrier between write and read in place, one without it.  Compiled into the ThreadSanitizer build
// of the emulated library alone; never built by nvcc and never launched on a GPU.
#include "nvk_common.cuh"

namespace {

template <bool SYNCED>
__global__ void rotate_kernel(const int* in, int* out) {
    __shared__ int s[64];
    s[threadIdx.x] = in[threadIdx.x];
    if (SYNCED) __syncthreads();
    out[threadIdx.x] = s[(threadIdx.x + 33) & 63];   // another warp's element
}

}  // namespace

extern "C" int emu_selftest_rotate(const int* in, int* out, int synced) {
    const nvk::Launch l = nvk::launch_1d(nullptr, 1, 64);
    return synced ? nvk::launch(l, rotate_kernel<true>, in, out) : nvk::launch(l, rotate_kernel<false>, in, out);
}
