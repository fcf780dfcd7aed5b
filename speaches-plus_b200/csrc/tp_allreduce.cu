// One-shot all-reduce of a small bf16 vector across the GPUs of one node, over peer memory.
//
// The row-parallel linears of a tensor-parallel decode step end in a sum of a few KB per rank; a
// library collective costs ~10 us there, more than the GEMV it follows.  Here every rank pushes its
// partial vector straight into an inbox on every peer (plain 16-byte stores over NVLink, no
// multicast, no TMA), raises a flag on each peer, waits for the flags of all peers and sums the
// inbox slots in rank order in fp32 -- the same order on every rank, so all ranks get the same bits.
//
// Memory (one buffer per rank, same layout everywhere, shared with CUDA IPC; peers' base pointers
// are passed in):
//   [0, 4096)            flags: uint32 flags[kMaxCtas][kMaxRanks], written by peers
//   [4096, ...)          inbox: 2 parities x world x max_elems bf16
// The call number ("epoch") lives in device memory and is advanced by the kernel itself, so a
// captured CUDA graph replays correctly.  Flags carry the epoch and are never reset; the inbox
// alternates between two halves, which is enough because a rank can only be one call ahead of any
// peer (it needs that peer's flag to finish a call).
//
// Every wait is bounded: after the wait limit (nvk_b200_set_wait_limit; about a second by default) the
// kernel records an error and returns, leaving the context usable.  The caller must run the same sequence of calls on every rank.
#include <string.h>

#include "nvk_common.cuh"

namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxCtas = 32;
constexpr int kFlagBytes = 4096;           // kMaxCtas * kMaxRanks * 4 = 1024 used
constexpr int kElemsPerCta = 8192;          // 16 KB of bf16 per CTA

struct ArParams {
    uint8_t* peer[kMaxRanks];   // base of every rank's symmetric buffer (peer[rank] is our own)
    const uint16_t* x;          // this rank's partial vector
    uint16_t* y;                // reduced result (may alias x)
    uint32_t* epoch;            // [kMaxCtas] call counters in local memory
    int* err;                   // set to 1 + peer index on a wait that gave up
    int rank, world, n, max_elems;
    uint32_t wait_limit;        // polls per peer before the wait gives up
};

using nvk::ptx::st_release_sys;

__global__ void __launch_bounds__(512) tp_allreduce_kernel(const ArParams p) {
    __shared__ int s_ok;
    // Programmatic dependent launch: x is the output of the kernel before this one; the kernel after
    // this one may start prefetching its weights now and waits for our completion before it reads y.
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const int cta = blockIdx.x;
    const int e0 = cta * kElemsPerCta;
    const int cnt = min(kElemsPerCta, p.n - e0);           // elements of this CTA (multiple of 8)
    const uint32_t epoch = p.epoch[cta] + 1u;
    const size_t half = (size_t)p.world * p.max_elems;      // elements per parity
    const size_t slot0 = (size_t)(epoch & 1u) * half;
    if (threadIdx.x == 0) s_ok = 1;

    // push this rank's chunk into slot [rank] of every peer's inbox (16-byte stores)
    const uint4* src = reinterpret_cast<const uint4*>(p.x + e0);
    for (int r = 0; r < p.world; ++r) {
        uint16_t* inbox = reinterpret_cast<uint16_t*>(p.peer[r] + kFlagBytes);
        uint4* dst = reinterpret_cast<uint4*>(inbox + slot0 + (size_t)p.rank * p.max_elems + e0);
        for (int i = threadIdx.x; i < cnt / 8; i += blockDim.x) dst[i] = src[i];
    }
    __threadfence_system();
    __syncthreads();
    // raise our flag on every peer, then wait for every peer's flag here
    if (threadIdx.x < p.world) {
        const int r = threadIdx.x;
        st_release_sys(reinterpret_cast<uint32_t*>(p.peer[r]) + cta * kMaxRanks + p.rank, epoch);
        const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.peer[p.rank]) + cta * kMaxRanks + r;
        if (!nvk::bounded_wait_ge(mine, epoch, p.wait_limit)) {
            atomicExch(p.err, 1 + r);
            s_ok = 0;
        }
    }
    __syncthreads();
    if (s_ok) {
        const uint16_t* inbox = reinterpret_cast<const uint16_t*>(p.peer[p.rank] + kFlagBytes) + slot0 + e0;
        for (int i = threadIdx.x; i < cnt / 8; i += blockDim.x) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < p.world; ++r) {
                const uint4 v = reinterpret_cast<const uint4*>(inbox + (size_t)r * p.max_elems)[i];
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[2 * j] += nvk::bf16_bits_to_f32(w[j] & 0xFFFFu);
                    acc[2 * j + 1] += nvk::bf16_bits_to_f32(w[j] >> 16);
                }
            }
            uint4 o;
            o.x = nvk::f32_to_bf16_bits(acc[0]) | ((uint32_t)nvk::f32_to_bf16_bits(acc[1]) << 16);
            o.y = nvk::f32_to_bf16_bits(acc[2]) | ((uint32_t)nvk::f32_to_bf16_bits(acc[3]) << 16);
            o.z = nvk::f32_to_bf16_bits(acc[4]) | ((uint32_t)nvk::f32_to_bf16_bits(acc[5]) << 16);
            o.w = nvk::f32_to_bf16_bits(acc[6]) | ((uint32_t)nvk::f32_to_bf16_bits(acc[7]) << 16);
            reinterpret_cast<uint4*>(p.y + e0)[i] = o;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) p.epoch[cta] = epoch;  // advance even after a failed wait: ranks stay in step
}

}  // namespace

extern "C" {

// Polls a kernel of this library spends in one wait on another CTA or GPU before it gives up and
// reports through its error word; 0 restores the default (about a second).  Applies to later calls
// made by the calling thread.
int nvk_b200_set_wait_limit(unsigned polls) {
    nvk::wait_limit_setting() = polls ? polls : nvk::kDefaultWaitLimit;
    return 0;
}

// ---- set-up helpers (host side, not on the launch path) ------------------------------------------
// The exchange buffer is plain device memory shared between the ranks of one node with CUDA IPC
// handles: each rank allocates its buffer, exports a 64-byte handle, the handles travel over the
// host-side process group, and every rank opens its peers' handles.  Nothing here binds memory to a
// multicast object, so a rank that exits leaves its peers' GPUs alone.
int nvk_b200_tp_buffer_alloc(size_t bytes, void** dev_ptr) {
    if (!dev_ptr || bytes == 0) return NVK_ERR_ARG;
    cudaError_t e = cudaMalloc(dev_ptr, bytes);
    if (e != cudaSuccess) return (int)e;
    e = cudaMemset(*dev_ptr, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    return (int)e;
}

int nvk_b200_tp_buffer_free(void* dev_ptr) { return dev_ptr ? (int)cudaFree(dev_ptr) : 0; }

// handle_out: 64 bytes (sizeof(cudaIpcMemHandle_t)).
int nvk_b200_tp_ipc_export(void* dev_ptr, void* handle_out) {
    if (!dev_ptr || !handle_out) return NVK_ERR_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    return (int)cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle_out), dev_ptr);
}

int nvk_b200_tp_ipc_open(const void* handle, void** dev_ptr) {
    if (!handle || !dev_ptr) return NVK_ERR_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    return (int)cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess);
}

int nvk_b200_tp_ipc_close(void* dev_ptr) { return dev_ptr ? (int)cudaIpcCloseMemHandle(dev_ptr) : 0; }

// Bytes of the symmetric buffer every rank must provide for vectors of up to max_elems bf16 values.
size_t nvk_b200_tp_allreduce_buffer_bytes(int world, int max_elems) {
    if (world <= 0 || world > kMaxRanks || max_elems <= 0) return 0;
    return (size_t)kFlagBytes + (size_t)2 * world * max_elems * sizeof(uint16_t);
}

// y = sum over ranks of x (bf16 in, fp32 sum in rank order, bf16 out), n % 8 == 0, n <= max_elems.
// peer_bufs: `world` device pointers, the symmetric buffers of ranks 0..world-1 as mapped in this
// process (zero-filled before the first call); epoch: 32 uint32 of local device memory, zero-filled
// before the first call and otherwise private to this function; err: one int of local device memory
// that becomes non-zero (1 + the peer that never arrived) if a wait gave up.
// Returns -2 on bad arguments, -3 when n needs more than 32 CTAs (n > 262144).
int nvk_b200_tp_allreduce_bf16(void* stream, const void* const* peer_bufs, int rank, int world, const uint16_t* x,
                               uint16_t* y, int n, int max_elems, uint32_t* epoch, int* err) {
    if (n <= 0) return 0;
    if (world <= 0 || world > kMaxRanks || rank < 0 || rank >= world || !peer_bufs || !x || !y || !epoch || !err)
        return NVK_ERR_ARG;
    if ((n & 7) != 0 || n > max_elems || (max_elems & 7) != 0) return NVK_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) return NVK_ERR_ARG;
    const int ctas = (n + kElemsPerCta - 1) / kElemsPerCta;
    if (ctas > kMaxCtas) return NVK_ERR_RESOURCE;
    ArParams p = {};
    for (int r = 0; r < world; ++r) {
        if (!peer_bufs[r]) return NVK_ERR_ARG;
        p.peer[r] = static_cast<uint8_t*>(const_cast<void*>(peer_bufs[r]));
    }
    p.x = x; p.y = y; p.epoch = epoch; p.err = err;
    p.rank = rank; p.world = world; p.n = n; p.max_elems = max_elems;
    p.wait_limit = nvk::wait_limit_setting();
    return nvk::launch(nvk::launch_1d((cudaStream_t)stream, (unsigned)ctas, 512, 0, true), tp_allreduce_kernel, p);
}

}  // extern "C"
