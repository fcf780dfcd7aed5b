// Host implementations of the wrappers in csrc/nvk_ptx.cuh for the SIMT emulation (tests only).
// Fragment layouts follow the PTX ISA's tables for mma.sync m16n8k16 (.f16/.bf16) and m16n8k32 (.s8).
#pragma once
#include "cuda_emu.h"

namespace nvk {
namespace ptx {

inline void pdl_wait() {}
inline void pdl_launch_dependents() {}

namespace detail {
inline float f16_bits_to_f32(uint32_t b) { __half h; h.bits = (uint16_t)b; return __half2float(h); }
inline float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }

// D = A(16x16) * B(16x8) + C for 16-bit inputs; lane = 4*gid + tg.
//   a0: row gid,   k = 2tg + {0,1}      a1: row gid+8, same k      a2/a3: the same rows, k + 8
//   b0: k = 2tg + {0,1}, col gid        b1: k + 8
//   c0/c1: row gid, cols 2tg, 2tg+1     c2/c3: row gid+8
template <float (*CVT)(uint32_t)>
inline void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    const uint32_t mine[6] = {a0, a1, a2, a3, b0, b1};
    const uint32_t(*tab)[8] = emu::warp_publish(mine, 6);
    const int lane = emu::fiber().lane, gid = lane >> 2, tg = lane & 3;
    for (int j = 0; j < 4; ++j) {
        const int row = gid + 8 * (j >> 1), col = 2 * tg + (j & 1);
        float acc = d[j];
        for (int k = 0; k < 16; ++k) {
            const int la = (row & 7) * 4 + ((k & 7) >> 1);
            const uint32_t ar = tab[la][(row >> 3) + 2 * (k >> 3)];
            const int lb = col * 4 + ((k & 7) >> 1);
            const uint32_t br = tab[lb][4 + (k >> 3)];
            const float av = CVT((ar >> (16 * (k & 1))) & 0xFFFFu), bv = CVT((br >> (16 * (k & 1))) & 0xFFFFu);
            acc = fmaf(av, bv, acc);
        }
        d[j] = acc;
    }
}
}  // namespace detail

inline void mma_m16n8k16_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                             uint32_t b1) {
    detail::mma16816<detail::f16_bits_to_f32>(d, a0, a1, a2, a3, b0, b1);
}
inline void mma_m16n8k16_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                              uint32_t b1) {
    detail::mma16816<detail::bf16_bits_to_f32>(d, a0, a1, a2, a3, b0, b1);
}
//   a0: row gid, k = 4tg + 0..3   a1: row gid+8   a2/a3: k + 16     b0: k = 4tg + 0..3, col gid   b1: k + 16
inline void mma_m16n8k32_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    const uint32_t mine[6] = {a0, a1, a2, a3, b0, b1};
    const uint32_t(*tab)[8] = emu::warp_publish(mine, 6);
    const int lane = emu::fiber().lane, gid = lane >> 2, tg = lane & 3;
    for (int j = 0; j < 4; ++j) {
        const int row = gid + 8 * (j >> 1), col = 2 * tg + (j & 1);
        int acc = d[j];
        for (int k = 0; k < 32; ++k) {
            const int la = (row & 7) * 4 + ((k & 15) >> 2);
            const uint32_t ar = tab[la][(row >> 3) + 2 * (k >> 4)];
            const int lb = col * 4 + ((k & 15) >> 2);
            const uint32_t br = tab[lb][4 + (k >> 4)];
            acc += (int)(int8_t)((ar >> (8 * (k & 3))) & 0xFF) * (int)(int8_t)((br >> (8 * (k & 3))) & 0xFF);
        }
        d[j] = acc;
    }
}

inline uint32_t smem_addr(const void* p) { return emu::shared_addr(p); }
inline void cp_async16(uint32_t dst, const void* src, int src_bytes) { emu::cp_async(dst, src, 16, src_bytes); }
inline void cp_async8(uint32_t dst, const void* src, int src_bytes) { emu::cp_async(dst, src, 8, src_bytes); }
inline void cp_async_commit() { emu::cp_async_commit(); }
template <int N>
inline void cp_async_wait() { emu::cp_async_wait(N); }

namespace detail {
inline uint32_t f32_to_f16_bits(float f) { return __float2half_rn(f).bits; }
inline float e2m1_value(uint32_t nib) {
    static const float tab[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    const float v = tab[nib & 7];
    return (nib & 8) ? -v : v;
}
inline float e4m3_value(uint32_t b) {
    const uint32_t e = (b >> 3) & 0xF, m = b & 7;
    float v;
    if ((b & 0x7F) == 0x7F) v = NAN;
    else if (e == 0) v = ldexpf((float)m, -9);
    else v = ldexpf(1.f + (float)m / 8.f, (int)e - 7);
    return (b & 0x80) ? -v : v;
}
}  // namespace detail

inline uint32_t e2m1x2_to_f16x2(uint32_t byte) {
    return detail::f32_to_f16_bits(detail::e2m1_value(byte & 0xF)) |
           (detail::f32_to_f16_bits(detail::e2m1_value((byte >> 4) & 0xF)) << 16);
}
inline void e2m1x8_to_f16x2x4(uint32_t w, uint32_t& h0, uint32_t& h1, uint32_t& h2, uint32_t& h3) {
    h0 = e2m1x2_to_f16x2(w & 0xFF);
    h1 = e2m1x2_to_f16x2((w >> 8) & 0xFF);
    h2 = e2m1x2_to_f16x2((w >> 16) & 0xFF);
    h3 = e2m1x2_to_f16x2((w >> 24) & 0xFF);
}
inline uint32_t e4m3x2_to_f16x2(uint32_t w) {
    return detail::f32_to_f16_bits(detail::e4m3_value(w & 0xFF)) |
           (detail::f32_to_f16_bits(detail::e4m3_value((w >> 8) & 0xFF)) << 16);
}
inline uint32_t hmul2(uint32_t a, uint32_t b) {
    __half2 x, y;
    memcpy(&x, &a, 4);
    memcpy(&y, &b, 4);
    const __half2 r = __hmul2(x, y);
    uint32_t o;
    memcpy(&o, &r, 4);
    return o;
}
inline uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
    __half2 x, y, z;
    memcpy(&x, &a, 4);
    memcpy(&y, &b, 4);
    memcpy(&z, &c, 4);
    const __half2 r = __hfma2(x, y, z);
    uint32_t o;
    memcpy(&o, &r, 4);
    return o;
}
inline int dp4a_s8(uint32_t a, uint32_t b, int c) {
    for (int i = 0; i < 4; ++i) c += (int)(int8_t)((a >> (8 * i)) & 0xFF) * (int)(int8_t)((b >> (8 * i)) & 0xFF);
    return c;
}

inline uint4 ldg_stream_v4(const void* p) {
    emu::note_fetch(p, 16);
    return *static_cast<const uint4*>(p);
}
inline void st_release_sys(uint32_t* p, uint32_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
inline uint32_t ld_acquire_sys(const uint32_t* p) {
    const uint32_t v = __atomic_load_n(p, __ATOMIC_ACQUIRE);
    emu::spin_yield();   // polling loads sit in wait loops: let the other fibers and blocks run
    return v;
}
inline uint32_t ld_acquire_gpu(const uint32_t* p) { return ld_acquire_sys(p); }
inline unsigned long long globaltimer_ns() {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (unsigned long long)ts.tv_sec * 1000000000ull + (unsigned long long)ts.tv_nsec;
}

}  // namespace ptx
}  // namespace nvk
