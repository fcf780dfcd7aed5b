// Host-side SIMT emulation of the CUDA constructs the kernels under speaches-plus_b200/csrc use.
//
// TEST INFRASTRUCTURE ONLY.  With -DNVK_EMU the .cu sources of the product library compile as plain
// C++ against this header (through the stub headers in shim/), and every kernel launch runs on the
// host: one fiber per CUDA thread, one OS thread per concurrently running block, warp collectives
// and barriers with their CUDA meaning, mma.sync with the fragment layouts of the PTX ISA, cp.async
// completed as LATE as the ISA allows (at the matching wait_group), shared and global buffers fenced
// by guard pages.  The tests use it to execute the kernels' real index arithmetic against the CPU
// oracle where no GPU is present, and as a bounds checker.  The product package never loads the
// emulated library and has no CPU path: nothing under speaches-plus_b200/ refers to this directory.
#pragma once
#ifndef NVK_EMU
#error "cuda_emu.h is only for -DNVK_EMU builds of the test emulation library"
#endif

#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <cmath>
#include <functional>
#include <type_traits>
#include <vector>

// ---- qualifiers ------------------------------------------------------------------------------
#define __global__
#define __device__
#define __host__
#define __forceinline__ inline __attribute__((always_inline))
#define __noinline__ __attribute__((noinline))
#define __restrict__ __restrict
#define __launch_bounds__(...)
#define __grid_constant__
#define __align__(n) __attribute__((aligned(n)))
#define __shared__ static thread_local   // one OS thread runs one block at a time
#define __constant__ static

// ---- vector types ----------------------------------------------------------------------------
struct uint2 { uint32_t x, y; };
struct __attribute__((aligned(16))) uint4 { uint32_t x, y, z, w; };
struct int2 { int x, y; };
struct __attribute__((aligned(16))) int4 { int x, y, z, w; };
struct float2 { float x, y; };
struct __attribute__((aligned(16))) float4 { float x, y, z, w; };
struct uint3 { unsigned x, y, z; };
struct dim3 {
    unsigned x, y, z;
    constexpr dim3(unsigned x_ = 1, unsigned y_ = 1, unsigned z_ = 1) : x(x_), y(y_), z(z_) {}
};
static inline uint2 make_uint2(uint32_t x, uint32_t y) { return uint2{x, y}; }
static inline uint4 make_uint4(uint32_t x, uint32_t y, uint32_t z, uint32_t w) { return uint4{x, y, z, w}; }
static inline int4 make_int4(int x, int y, int z, int w) { return int4{x, y, z, w}; }
static inline float2 make_float2(float x, float y) { return float2{x, y}; }
static inline float4 make_float4(float x, float y, float z, float w) { return float4{x, y, z, w}; }

// ---- runtime types ---------------------------------------------------------------------------
typedef void* cudaStream_t;
enum cudaError_t : int {
    cudaSuccess = 0,
    cudaErrorInvalidValue = 1,
    cudaErrorMemoryAllocation = 2,
    cudaErrorInvalidConfiguration = 9,
    cudaErrorInvalidDevice = 101,
    cudaErrorNotSupported = 801,
};
enum cudaFuncAttribute { cudaFuncAttributeMaxDynamicSharedMemorySize = 8 };
enum cudaDeviceAttr {
    cudaDevAttrMultiProcessorCount = 16,
    cudaDevAttrComputeCapabilityMajor = 75,
    cudaDevAttrComputeCapabilityMinor = 76,
};
enum cudaMemcpyKind { cudaMemcpyHostToDevice = 1, cudaMemcpyDeviceToHost = 2, cudaMemcpyDeviceToDevice = 3 };
struct cudaIpcMemHandle_t { char reserved[64]; };
enum { cudaIpcMemLazyEnablePeerAccess = 1 };

namespace emu {

// ---- execution state -------------------------------------------------------------------------
struct Block;
struct Fiber;
extern thread_local Block* g_block;
extern thread_local Fiber* g_fiber;

struct FiberPublic {   // the part of a fiber that inline code reads
    uint3 tidx;
    int lane, warp;
};
struct BlockPublic {
    uint3 bidx;
    dim3 bdim, gdim;
    uint8_t* dyn_smem;
    size_t dyn_bytes;
    unsigned cluster_rank, cluster_size;
};
FiberPublic& fiber();
BlockPublic& block();

void syncthreads();
void syncwarp();
void cluster_sync();
void* cluster_map(void* p, unsigned rank);
void spin_yield();   // inside a wait loop on memory another block or rank writes
// Warp exchange: every live lane of the warp publishes `n_words` 32-bit words and receives a
// pointer to the whole warp's table [32][8] (valid until the lane's next warp collective).
const uint32_t (*warp_publish(const uint32_t* words, int n_words))[8];

// cp.async, completed at the matching wait_group (or at once when option cp_async_early is set)
void cp_async(uint32_t dst_shared, const void* src, int bytes, int src_bytes);
void note_fetch(const void* src, int bytes);   // weight-stream accounting, see emu_rt.cpp
void cp_async_commit();
void cp_async_wait(int allowed_pending);
uint32_t shared_addr(const void* p);        // generic -> shared window address
void* shared_ptr(uint32_t a, size_t bytes);  // and back, bounds-checked

struct LaunchCfg {
    dim3 grid, block;
    size_t smem = 0;
    unsigned cluster_x = 1;
    bool cooperative = false;
};
int run_grid(const LaunchCfg& cfg, const void* func, const std::function<void()>& body);
int func_set_max_dyn_smem(const void* func, int bytes);
int sm_count();

}  // namespace emu

#define threadIdx (::emu::fiber().tidx)
#define blockIdx (::emu::block().bidx)
#define blockDim (::emu::block().bdim)
#define gridDim (::emu::block().gdim)
static inline void __syncthreads() { emu::syncthreads(); }
static inline void __syncwarp(unsigned = 0xffffffffu) { emu::syncwarp(); }
static inline void __threadfence() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
static inline void __threadfence_system() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
static inline void __threadfence_block() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }

// ---- warp collectives ------------------------------------------------------------------------
namespace emu {
template <class T>
inline T shfl_from(const T& v, int src_lane) {
    static_assert(sizeof(T) <= 32 && std::is_trivially_copyable<T>::value, "shuffle payload");
    uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    memcpy(w, &v, sizeof(T));
    const uint32_t(*tab)[8] = warp_publish(w, (int)((sizeof(T) + 3) / 4));
    T r;
    memcpy(&r, tab[src_lane & 31], sizeof(T));
    return r;
}
}  // namespace emu
template <class T> static inline T __shfl_sync(unsigned, T v, int src, int = 32) { return emu::shfl_from(v, src); }
template <class T> static inline T __shfl_xor_sync(unsigned, T v, int m, int = 32) {
    return emu::shfl_from(v, emu::fiber().lane ^ m);
}
template <class T> static inline T __shfl_down_sync(unsigned, T v, unsigned d, int = 32) {
    const int s = emu::fiber().lane + (int)d;
    return emu::shfl_from(v, s < 32 ? s : emu::fiber().lane);
}
template <class T> static inline T __shfl_up_sync(unsigned, T v, unsigned d, int = 32) {
    const int s = emu::fiber().lane - (int)d;
    return emu::shfl_from(v, s >= 0 ? s : emu::fiber().lane);
}
static inline unsigned __ballot_sync(unsigned, int pred) {
    uint32_t w[1] = {pred ? 1u : 0u};
    // lanes that already left the kernel keep a zero in the table
    const uint32_t(*tab)[8] = emu::warp_publish(w, 1);
    unsigned m = 0;
    for (int l = 0; l < 32; ++l) m |= (tab[l][0] & 1u) << l;
    return m;
}
static inline int __any_sync(unsigned m, int pred) { return __ballot_sync(m, pred) != 0; }
// redux.sync / match.sync over the lanes named by `mask` (every live lane calls them)
static inline unsigned __reduce_max_sync(unsigned mask, unsigned v) {
    uint32_t w[1] = {v};
    const uint32_t(*tab)[8] = emu::warp_publish(w, 1);
    unsigned m = 0;
    for (int l = 0; l < 32; ++l) if (mask & (1u << l)) m = tab[l][0] > m ? tab[l][0] : m;
    return m;
}
static inline unsigned __reduce_min_sync(unsigned mask, unsigned v) {
    uint32_t w[1] = {v};
    const uint32_t(*tab)[8] = emu::warp_publish(w, 1);
    unsigned m = 0xFFFFFFFFu;
    for (int l = 0; l < 32; ++l) if (mask & (1u << l)) m = tab[l][0] < m ? tab[l][0] : m;
    return m;
}
static inline unsigned __reduce_add_sync(unsigned mask, unsigned v) {
    uint32_t w[1] = {v};
    const uint32_t(*tab)[8] = emu::warp_publish(w, 1);
    unsigned m = 0;
    for (int l = 0; l < 32; ++l) if (mask & (1u << l)) m += tab[l][0];
    return m;
}
static inline unsigned __match_any_sync(unsigned mask, int v) {
    uint32_t w[1] = {(uint32_t)v};
    const uint32_t(*tab)[8] = emu::warp_publish(w, 1);
    unsigned m = 0;
    for (int l = 0; l < 32; ++l) if ((mask & (1u << l)) && tab[l][0] == (uint32_t)v) m |= 1u << l;
    return m;
}

// ---- bit casts, math ---------------------------------------------------------------------------
static inline float __uint_as_float(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t __float_as_uint(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline int __float_as_int(float f) { int u; memcpy(&u, &f, 4); return u; }
static inline float __int_as_float(int u) { float f; memcpy(&f, &u, 4); return f; }
static inline float rsqrtf(float x) { return 1.0f / sqrtf(x); }
static inline int __float2int_rn(float x) { return (int)nearbyintf(x); }   // round to nearest even (default mode)
static inline int __popc(unsigned v) { return __builtin_popcount(v); }
static inline int __ffs(int v) { return __builtin_ffs(v); }
static inline int __clz(int v) { return v == 0 ? 32 : __builtin_clz((unsigned)v); }
static inline uint32_t __byte_perm(uint32_t a, uint32_t b, uint32_t s) {
    const uint64_t t = ((uint64_t)b << 32) | a;
    uint32_t r = 0;
    for (int i = 0; i < 4; ++i) {
        const uint32_t sel = (s >> (4 * i)) & 0xF;
        uint32_t byte = (uint32_t)((t >> (8 * (sel & 7))) & 0xFF);
        if (sel & 8) byte = (byte & 0x80) ? 0xFF : 0x00;
        r |= byte << (8 * i);
    }
    return r;
}
using std::isfinite;
using std::signbit;
static inline int min(int a, int b) { return a < b ? a : b; }
static inline int max(int a, int b) { return a > b ? a : b; }
static inline unsigned min(unsigned a, unsigned b) { return a < b ? a : b; }
static inline unsigned max(unsigned a, unsigned b) { return a > b ? a : b; }
static inline long long min(long long a, long long b) { return a < b ? a : b; }
static inline long long max(long long a, long long b) { return a > b ? a : b; }
static inline unsigned long min(unsigned long a, unsigned long b) { return a < b ? a : b; }
static inline unsigned long max(unsigned long a, unsigned long b) { return a > b ? a : b; }
static inline float min(float a, float b) { return fminf(a, b); }
static inline float max(float a, float b) { return fmaxf(a, b); }

template <class T> static inline T __ldg(const T* p) { return *p; }
template <class T> static inline T __ldcg(const T* p) { return *p; }
template <class T> static inline T __ldcs(const T* p) { return *p; }
template <class T> static inline void __stcg(T* p, T v) { *p = v; }

// ---- atomics -----------------------------------------------------------------------------------
static inline int atomicAdd(int* p, int v) { return __atomic_fetch_add(p, v, __ATOMIC_SEQ_CST); }
static inline unsigned atomicAdd(unsigned* p, unsigned v) { return __atomic_fetch_add(p, v, __ATOMIC_SEQ_CST); }
static inline unsigned long long atomicAdd(unsigned long long* p, unsigned long long v) {
    return __atomic_fetch_add(p, v, __ATOMIC_SEQ_CST);
}
static inline float atomicAdd(float* p, float v) {
    uint32_t* q = reinterpret_cast<uint32_t*>(p);
    uint32_t old = __atomic_load_n(q, __ATOMIC_SEQ_CST);
    for (;;) {
        const uint32_t want = __float_as_uint(__uint_as_float(old) + v);
        if (__atomic_compare_exchange_n(q, &old, want, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST))
            return __uint_as_float(old);
    }
}
static inline unsigned atomicMax(unsigned* p, unsigned v) {
    unsigned old = __atomic_load_n(p, __ATOMIC_SEQ_CST);
    while (old < v && !__atomic_compare_exchange_n(p, &old, v, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST)) {}
    return old;
}
static inline int atomicMax(int* p, int v) {
    int old = __atomic_load_n(p, __ATOMIC_SEQ_CST);
    while (old < v && !__atomic_compare_exchange_n(p, &old, v, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST)) {}
    return old;
}
static inline unsigned atomicInc(unsigned* p, unsigned limit) {   // old >= limit ? 0 : old + 1
    unsigned old = __atomic_load_n(p, __ATOMIC_SEQ_CST);
    while (!__atomic_compare_exchange_n(p, &old, old >= limit ? 0u : old + 1u, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST)) {}
    return old;
}
static inline int atomicExch(int* p, int v) { return __atomic_exchange_n(p, v, __ATOMIC_SEQ_CST); }
static inline unsigned atomicExch(unsigned* p, unsigned v) { return __atomic_exchange_n(p, v, __ATOMIC_SEQ_CST); }
static inline unsigned atomicOr(unsigned* p, unsigned v) { return __atomic_fetch_or(p, v, __ATOMIC_SEQ_CST); }
static inline int atomicOr(int* p, int v) { return __atomic_fetch_or(p, v, __ATOMIC_SEQ_CST); }
static inline int atomicCAS(int* p, int cmp, int v) {
    __atomic_compare_exchange_n(p, &cmp, v, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST);
    return cmp;
}

// ---- bf16 / f16 --------------------------------------------------------------------------------
struct __nv_bfloat16 { uint16_t bits; };
static inline __nv_bfloat16 __float2bfloat16_rn(float f) {
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return __nv_bfloat16{0x7FFF};
    u += 0x7FFFu + ((u >> 16) & 1u);
    return __nv_bfloat16{(uint16_t)(u >> 16)};
}
static inline uint16_t __bfloat16_as_ushort(__nv_bfloat16 b) { return b.bits; }
static inline float __bfloat162float(__nv_bfloat16 b) { return __uint_as_float((uint32_t)b.bits << 16); }

struct __half { uint16_t bits; };
struct __half2 { __half x, y; };
static inline float __half2float(__half h) { _Float16 v; memcpy(&v, &h.bits, 2); return (float)v; }
static inline __half __float2half_rn(float f) { _Float16 v = (_Float16)f; __half h; memcpy(&h.bits, &v, 2); return h; }
static inline __half __double2half_rn_emu(double f) { _Float16 v = (_Float16)f; __half h; memcpy(&h.bits, &v, 2); return h; }
static inline __half2 __floats2half2_rn(float a, float b) { return __half2{__float2half_rn(a), __float2half_rn(b)}; }
static inline float2 __half22float2(__half2 h) { return float2{__half2float(h.x), __half2float(h.y)}; }
static inline __half2 __hisnan2(__half2 h) {
    const float a = __half2float(h.x), b = __half2float(h.y);
    return __half2{__float2half_rn(a != a ? 1.f : 0.f), __float2half_rn(b != b ? 1.f : 0.f)};
}
static inline __half2 __high2half2(__half2 h) { return __half2{h.y, h.y}; }
static inline __half2 __low2half2(__half2 h) { return __half2{h.x, h.x}; }
// f16 x f16 is exact in f32 (11 + 11 significand bits), so one rounding to f16 is the IEEE result
static inline __half2 __hmul2(__half2 a, __half2 b) {
    return __half2{__float2half_rn(__half2float(a.x) * __half2float(b.x)),
                   __float2half_rn(__half2float(a.y) * __half2float(b.y))};
}
// a*b exact in double, + c exact or rounded once far below f16 precision, then one rounding to f16
static inline __half2 __hfma2(__half2 a, __half2 b, __half2 c) {
    return __half2{__double2half_rn_emu((double)__half2float(a.x) * (double)__half2float(b.x) + (double)__half2float(c.x)),
                   __double2half_rn_emu((double)__half2float(a.y) * (double)__half2float(b.y) + (double)__half2float(c.y))};
}

// ---- host runtime calls (synchronous here) -------------------------------------------------------
static inline cudaError_t cudaGetLastError() { return cudaSuccess; }
static inline cudaError_t cudaPeekAtLastError() { return cudaSuccess; }
static inline cudaError_t cudaMemsetAsync(void* p, int v, size_t n, cudaStream_t) { memset(p, v, n); return cudaSuccess; }
static inline cudaError_t cudaMemset(void* p, int v, size_t n) { memset(p, v, n); return cudaSuccess; }
static inline cudaError_t cudaMemcpy(void* d, const void* s, size_t n, cudaMemcpyKind) { memcpy(d, s, n); return cudaSuccess; }
static inline cudaError_t cudaMemcpyAsync(void* d, const void* s, size_t n, cudaMemcpyKind, cudaStream_t) {
    memcpy(d, s, n);
    return cudaSuccess;
}
static inline cudaError_t cudaDeviceSynchronize() { return cudaSuccess; }
static inline cudaError_t cudaGetDevice(int* d) { *d = 0; return cudaSuccess; }
static inline cudaError_t cudaDeviceGetAttribute(int* v, cudaDeviceAttr a, int) {
    *v = a == cudaDevAttrMultiProcessorCount ? emu::sm_count() : a == cudaDevAttrComputeCapabilityMajor ? 10 : 0;
    return cudaSuccess;
}
cudaError_t cudaMalloc(void** p, size_t n);   // guard-paged
cudaError_t cudaFree(void* p);
static inline cudaError_t cudaFuncSetAttribute(const void* f, cudaFuncAttribute, int bytes) {
    return (cudaError_t)emu::func_set_max_dyn_smem(f, bytes);
}
template <class F>
static inline cudaError_t cudaOccupancyMaxActiveBlocksPerMultiprocessor(int* n, F, int, size_t smem) {
    *n = smem > 113 * 1024 ? 1 : 2;
    return cudaSuccess;
}
template <class T> static inline cudaError_t cudaGetSymbolAddress(void** p, T& sym) { *p = (void*)&sym; return cudaSuccess; }
static inline cudaError_t cudaIpcGetMemHandle(cudaIpcMemHandle_t*, void*) { return cudaErrorNotSupported; }
static inline cudaError_t cudaIpcOpenMemHandle(void**, cudaIpcMemHandle_t, unsigned) { return cudaErrorNotSupported; }
static inline cudaError_t cudaIpcCloseMemHandle(void*) { return cudaErrorNotSupported; }

// ---- cooperative groups: the cluster part --------------------------------------------------------
namespace cooperative_groups {
struct cluster_group {
    void sync() const { emu::cluster_sync(); }
    unsigned block_rank() const { return emu::block().cluster_rank; }
    unsigned num_blocks() const { return emu::block().cluster_size; }
    template <class T> T* map_shared_rank(T* p, unsigned rank) const {
        return static_cast<T*>(emu::cluster_map(const_cast<void*>(static_cast<const void*>(p)), rank));
    }
};
inline cluster_group this_cluster() { return cluster_group{}; }
}  // namespace cooperative_groups
