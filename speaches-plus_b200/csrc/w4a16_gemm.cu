// NVFP4 weight-only (W4A16) linear for decode-sized M on sm_100a.
//
//   y[m, n] = bf16( alpha * sum_k e2m1(W[n,k]) * ue4m3(S[n, k/16]) * x[m, k] ),  fp32 accumulate
//
// Weights are streamed once from HBM with 128-bit loads straight into registers, unpacked with
// the native e2m1x2 -> f16x2 convert, multiplied by their block scale in f16 (exact: a 2-bit by
// 4-bit significand product) and contracted against the activations on the tensor cores with
// fp32 accumulation (m16n8k16).  One CTA owns one 128-row tile of the swizzled scale layout, so
// every 512-byte scale tile is read as whole 16-byte lines; K is split across the CTAs of a
// thread-block cluster and the partial tiles are summed through distributed shared memory in a
// fixed order (deterministic, no global scratch).
//
// Activations are bf16.  They are staged per CTA into shared memory as f16 after an exact
// power-of-two pre-scale chosen from the slice's own maximum (bf16 has 8 significand bits, f16
// has 11, so every value within 2^31 of the slice maximum converts exactly); the power of two is
// undone in fp32 before alpha is applied.
#include <cooperative_groups.h>

#include "nvk_common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int kRowsPerCta = 128;
constexpr int kSuper = 256;  // K elements one warp consumes per iteration (4 scale k-tiles)

struct GemmParams {
    const uint8_t* wq[2];
    const uint8_t* sc[2];
    const uint16_t* x;    // [M, K] bf16, or gate when PRO == 1
    const uint16_t* x2;   // up when PRO == 1
    uint16_t* y[2];       // [M, N] bf16 per arm
    float alpha[2];
    int M, N, K;
    int tiles_per_arm;  // ceil(N / 128)
    int k_tiles;        // ceil(K / 64): scale tiles along K
    int nsc;            // ceil(K / 256)
    int spc;            // super-chunks per CTA (the CTA's K slice)
    int ph;             // super-chunks staged per phase
    int x_stride;       // bytes between token rows of the staged activations
};

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Two ue4m3 scale bytes (the low or high half of `w`, bit 7 of each byte already cleared) -> f16x2.
// ue4m3 is the non-negative half of e4m3, so the hardware e4m3 convert is exact for 0x00..0x7E;
// 0x7F (never produced by an NVFP4 encoder, NaN in e4m3) converts to NaN.
__device__ __forceinline__ __half2 scales2_f16(uint32_t w, int half) {
    uint32_t d;
    asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.rn.f16x2.e4m3x2 %0, lo;}" : "=r"(d) : "r"(half ? (w >> 16) : w));
    return *reinterpret_cast<__half2*>(&d);
}

struct WFrag {
    uint32_t w[4][8];  // the thread's 32-byte run of one k-tile (64 values), rows d2 = 0..3
    uint4 sc;          // word d2 = the 4 block scales of row d2 in this k-tile
};

// One 256-bit load: a whole 32-byte sector per thread (address must be 32-byte aligned).
__device__ __forceinline__ void ldg_nc_v8(uint32_t (&d)[8], const void* p) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7])
                 : "l"(p));
}

// NT: 8-token column tiles; HG: 32-row groups per CTA (rows per CTA = 32*HG); KW: warps along K.
template <int NT, bool DUAL, int PRO, int HG, int KW, bool V8>
__global__ void __launch_bounds__(32 * HG * KW, NT <= 2 ? 2 : 1) w4a16_mma_kernel(const GemmParams p) {
    constexpr int THREADS = 32 * HG * KW;
    constexpr int MT = 8 * NT;       // token columns
    constexpr int ROWS = 32 * HG;    // weight rows per CTA
    constexpr int SUB = 4 / HG;      // CTAs per 128-row scale tile
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ uint32_t s_amax[MT];   // slice maximum (bf16 magnitude bits), then f32 bits of 2^-pw
    __shared__ int s_pw[MT];          // power of two currently folded into the accumulators
    __shared__ float s_rescale[MT];   // 2^(pw_old - pw_new) at a phase boundary

    cg::cluster_group cluster = cg::this_cluster();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hl = warp % HG, kw = warp / HG;  // local row group, K-warp
    const int gid = lane >> 2, tg = lane & 3;
    const int tile = blockIdx.y;
    const int arm = DUAL ? (tile >= p.tiles_per_arm ? 1 : 0) : 0;
    const int sub = tile - arm * p.tiles_per_arm;
    const int mt = sub / SUB;                 // 128-row scale tile
    const int h = (sub % SUB) * HG + hl;      // 32-row group inside it: rows 8h+gid + 32*d2
    const int crank = blockIdx.x;
    const int nranks = gridDim.x;
    const int M = p.M, N = p.N, K = p.K;

    const uint8_t* __restrict__ wq = p.wq[arm];
    const uint8_t* __restrict__ sc = p.sc[arm];
    const int row0 = mt * kRowsPerCta + 8 * h + gid;  // + 32 * d2
    const size_t half_k = (size_t)(K >> 1);
    const uint8_t* sc_thread = sc + (size_t)mt * p.k_tiles * 512 + (size_t)(8 * h + gid) * 16;

    const int sc_begin = crank * p.spc;
    const int sc_end = min(p.nsc, sc_begin + p.spc);

    float acc[2][NT][4];
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[t][n][i] = 0.f;

    auto load_frag = [&](WFrag& f, int s) {
        const int kt = 4 * s + tg;
        const int k0 = kt * 64;
        const bool v0 = k0 < K, v1 = (k0 + 32) < K;
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int d2 = 0; d2 < 4; ++d2) {
            const int r = row0 + 32 * d2;
            const uint8_t* src = wq + (size_t)r * half_k + (size_t)(k0 >> 1);
            const bool rv = r < N;
            if (V8) {
                if (rv && v0) {
                    ldg_nc_v8(f.w[d2], src);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) f.w[d2][i] = 0u;
                }
            } else {
                const uint4 lo = (rv && v0) ? ldg_nc_v4(src) : z;
                const uint4 hi = (rv && v1) ? ldg_nc_v4(src + 16) : z;
                f.w[d2][0] = lo.x; f.w[d2][1] = lo.y; f.w[d2][2] = lo.z; f.w[d2][3] = lo.w;
                f.w[d2][4] = hi.x; f.w[d2][5] = hi.y; f.w[d2][6] = hi.z; f.w[d2][7] = hi.w;
            }
        }
        f.sc = v0 ? ldg_nc_v4(sc_thread + (size_t)kt * 512) : z;
    };

    // B-fragment source rows: token 8n+gid, clamped to the last real token so that no load needs a
    // predicate (columns past M compute a duplicate that is never written out).
    const uint8_t* xs_tok[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) xs_tok[n] = smem + (size_t)min(8 * n + gid, M - 1) * p.x_stride + tg * 16;

    auto compute = [&](const WFrag& f, int s_local) {
        const int xoff = s_local * 512;
        const uint32_t scw[4] = {f.sc.x & 0x7F7F7F7Fu, f.sc.y & 0x7F7F7F7Fu, f.sc.z & 0x7F7F7F7Fu,
                                 f.sc.w & 0x7F7F7F7Fu};
        __half2 sp[4][2];  // row d2: {s0,s1}, {s2,s3}
#pragma unroll
        for (int d2 = 0; d2 < 4; ++d2) {
            sp[d2][0] = scales2_f16(scw[d2], 0);
            sp[d2][1] = scales2_f16(scw[d2], 1);
        }
#pragma unroll
        for (int wi = 0; wi < 8; ++wi) {
            uint32_t a[4][4];
#pragma unroll
            for (int d2 = 0; d2 < 4; ++d2) {
                nvk::e2m1x8_to_f16x2x4(f.w[d2][wi], a[d2][0], a[d2][1], a[d2][2], a[d2][3]);
                const __half2 pr = sp[d2][wi >> 2];
                const __half2 s = ((wi >> 1) & 1) ? __high2half2(pr) : __low2half2(pr);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const __half2 v = __hmul2(*reinterpret_cast<__half2*>(&a[d2][i]), s);
                    a[d2][i] = *reinterpret_cast<const uint32_t*>(&v);
                }
            }
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const uint4 xv = *reinterpret_cast<const uint4*>(xs_tok[n] + xoff + wi * 64);
                mma_f16(acc[0][n], a[0][0], a[1][0], a[0][1], a[1][1], xv.x, xv.y);
                mma_f16(acc[1][n], a[2][0], a[3][0], a[2][1], a[3][1], xv.x, xv.y);
                mma_f16(acc[0][n], a[0][2], a[1][2], a[0][3], a[1][3], xv.z, xv.w);
                mma_f16(acc[1][n], a[2][2], a[3][2], a[2][3], a[3][3], xv.z, xv.w);
            }
        }
    };

    for (int p0 = sc_begin; p0 < sc_end; p0 += p.ph) {
        const int pend = min(sc_end, p0 + p.ph);
        const int nsp = pend - p0;
        // Weight loads do not depend on the activations: put the first ones in flight now.
        WFrag f0, f1;
        int s = p0 + kw;
        if (s < pend) load_frag(f0, s);

        // ---- stage activations for super-chunks [p0, pend) ----
        if (threadIdx.x < MT) s_amax[threadIdx.x] = 0u;
        __syncthreads();  // also orders the previous phase's reads before this phase's writes
        const int pieces_per_tok = nsp * 32;
        const int total_pieces = M * pieces_per_tok;
        for (int idx = threadIdx.x; idx < total_pieces; idx += THREADS) {
            const int m = idx / pieces_per_tok;
            const int rem = idx - m * pieces_per_tok;
            const int k = (p0 + (rem >> 5)) * kSuper + (rem & 31) * 8;
            uint32_t mx = 0u;
            if (k < K) {
                uint4 v = *reinterpret_cast<const uint4*>(p.x + (size_t)m * K + k);
                uint32_t ws[4] = {v.x, v.y, v.z, v.w};
                if (PRO == 1) {
                    uint4 u = *reinterpret_cast<const uint4*>(p.x2 + (size_t)m * K + k);
                    uint32_t us[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float g0 = nvk::bf16_bits_to_f32(ws[i] & 0xFFFFu), g1 = nvk::bf16_bits_to_f32(ws[i] >> 16);
                        float u0 = nvk::bf16_bits_to_f32(us[i] & 0xFFFFu), u1 = nvk::bf16_bits_to_f32(us[i] >> 16);
                        uint32_t a0 = nvk::f32_to_bf16_bits((g0 / (1.0f + expf(-g0))) * u0);
                        uint32_t a1 = nvk::f32_to_bf16_bits((g1 / (1.0f + expf(-g1))) * u1);
                        ws[i] = a0 | (a1 << 16);
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) mx = max(mx, max(ws[i] & 0x7FFFu, (ws[i] >> 16) & 0x7FFFu));
            }
            if (mx) atomicMax(&s_amax[m], mx);
        }
        __syncthreads();
        if (threadIdx.x < MT) {
            // bf16 magnitude bits -> biased exponent; map the slice maximum into [2^14, 2^15).
            const int e8 = (int)(s_amax[threadIdx.x] >> 7);
            const int pw = max(e8 - 141, -100);  // x' = x * 2^-pw
            const int diff = p0 > sc_begin ? min(max(s_pw[threadIdx.x] - pw, -126), 126) : 0;
            s_rescale[threadIdx.x] = __uint_as_float((uint32_t)(127 + diff) << 23);
            s_pw[threadIdx.x] = pw;
            s_amax[threadIdx.x] = (uint32_t)(127 - pw) << 23;  // f32 bits of 2^-pw
        }
        __syncthreads();
        if (p0 > sc_begin) {
            // accumulators carry 2^-pw_old; move them to this phase's power of two (exact)
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const float r0 = s_rescale[8 * n + 2 * tg], r1 = s_rescale[8 * n + 2 * tg + 1];
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    acc[t][n][0] *= r0; acc[t][n][1] *= r1; acc[t][n][2] *= r0; acc[t][n][3] *= r1;
                }
            }
        }
        for (int idx = threadIdx.x; idx < total_pieces; idx += THREADS) {
            const int m = idx / pieces_per_tok;
            const int rem = idx - m * pieces_per_tok;
            const int scl = rem >> 5, q = rem & 31;
            const int k = (p0 + scl) * kSuper + q * 8;
            uint4 o = make_uint4(0u, 0u, 0u, 0u);
            if (k < K) {
                uint4 v = *reinterpret_cast<const uint4*>(p.x + (size_t)m * K + k);
                uint32_t ws[4] = {v.x, v.y, v.z, v.w};
                if (PRO == 1) {
                    uint4 u = *reinterpret_cast<const uint4*>(p.x2 + (size_t)m * K + k);
                    uint32_t us[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float g0 = nvk::bf16_bits_to_f32(ws[i] & 0xFFFFu), g1 = nvk::bf16_bits_to_f32(ws[i] >> 16);
                        float u0 = nvk::bf16_bits_to_f32(us[i] & 0xFFFFu), u1 = nvk::bf16_bits_to_f32(us[i] >> 16);
                        uint32_t a0 = nvk::f32_to_bf16_bits((g0 / (1.0f + expf(-g0))) * u0);
                        uint32_t a1 = nvk::f32_to_bf16_bits((g1 / (1.0f + expf(-g1))) * u1);
                        ws[i] = a0 | (a1 << 16);
                    }
                }
                const float sc2 = __uint_as_float(s_amax[m]);
                uint32_t os[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float lo = nvk::bf16_bits_to_f32(ws[i] & 0xFFFFu) * sc2;
                    float hi = nvk::bf16_bits_to_f32(ws[i] >> 16) * sc2;
                    __half2 h2 = __floats2half2_rn(lo, hi);
                    os[i] = *reinterpret_cast<uint32_t*>(&h2);
                }
                o = make_uint4(os[0], os[1], os[2], os[3]);
            }
            // piece q of a super-chunk: k-tile tg' = q / 8, 16-byte piece j2 = q % 8; stored so that
            // the four k-tiles' pieces with equal j2 are adjacent (conflict-free fragment reads).
            const int off = m * p.x_stride + scl * 512 + ((q & 7) * 4 + (q >> 3)) * 16;
            *reinterpret_cast<uint4*>(smem + off) = o;
        }
        __syncthreads();

        // ---- stream this phase's weights ----
        for (; s < pend; s += 2 * KW) {
            const int s1 = s + KW;
            if (s1 < pend) load_frag(f1, s1);
            compute(f0, s - p0);
            if (s1 < pend) {
                if (s1 + KW < pend) load_frag(f0, s1 + KW);
                compute(f1, s1 - p0);
            }
        }
    }
    if (sc_begin >= sc_end && threadIdx.x < MT) s_pw[threadIdx.x] = 0;  // empty slice: acc is zero

    // ---- sum the K-warps of this CTA: red[kw][token][row] ----
    __syncthreads();
    float* red = reinterpret_cast<float*>(smem);
    constexpr int RS = ROWS + 4;  // padded row count per token column
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            // local row index = hl*32 + d2*8 + gid with d2 = 2t (c0/c1) and 2t+1 (c2/c3)
            const int rl = hl * 32 + 16 * t + gid;
            const int c = 8 * n + 2 * tg;
            float* base = red + (size_t)kw * MT * RS;
            // undo the activation power of two
            const float d0 = __uint_as_float((uint32_t)(127 + s_pw[c]) << 23);
            const float d1 = __uint_as_float((uint32_t)(127 + s_pw[c + 1]) << 23);
            base[(c)*RS + rl] = acc[t][n][0] * d0;
            base[(c + 1) * RS + rl] = acc[t][n][1] * d1;
            base[(c)*RS + rl + 8] = acc[t][n][2] * d0;
            base[(c + 1) * RS + rl + 8] = acc[t][n][3] * d1;
        }
    __syncthreads();
    float* part = red + (size_t)KW * MT * RS;  // [token][row] partial of this CTA
    for (int i = threadIdx.x; i < M * ROWS; i += THREADS) {
        const int m = i / ROWS, rl = i % ROWS;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < KW; ++w) v += red[((size_t)w * MT + m) * RS + rl];
        part[m * RS + rl] = v;
    }

    // ---- sum the CTAs of the cluster through distributed shared memory, fixed order ----
    if (nranks > 1) cluster.sync(); else __syncthreads();
    const float alpha = p.alpha[arm];
    uint16_t* __restrict__ y = p.y[arm];
    const int rows_per_rank = ROWS / nranks;  // nranks in {1,2,4,8}
    for (int i = threadIdx.x; i < M * rows_per_rank; i += THREADS) {
        const int m = i / rows_per_rank;
        const int rl = crank * rows_per_rank + (i - m * rows_per_rank);
        float v = 0.f;
        if (nranks > 1) {
            for (int r = 0; r < nranks; ++r) {
                const float* rp = cluster.map_shared_rank(part, r);
                v += rp[m * RS + rl];
            }
        } else {
            v = part[m * RS + rl];
        }
        // undo the local row numbering: rl = hl*32 + d2*8 + g
        const int n_out = mt * kRowsPerCta + 32 * ((rl >> 3) & 3) + 8 * ((sub % SUB) * HG + (rl >> 5)) + (rl & 7);
        if (n_out < N) y[(size_t)m * N + n_out] = nvk::f32_to_bf16_bits(v * alpha);
    }
    if (nranks > 1) cluster.sync();  // peers may still be reading this CTA's partial
}

// ------------------------------------------------------------------------------------------
// Generic route: one warp per output row, fp32 FMAs.  Takes every shape the reference
// launchers take (K % 16 == 0, any N, any alignment the reference requires) and is used when
// the tensor-core route's layout conditions do not hold.
template <int PRO>
__global__ void __launch_bounds__(256) w4a16_rowwarp_kernel(const GemmParams p) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int total = p.wq[1] ? 2 * p.N : p.N;
    if (row >= total) return;
    const int arm = row >= p.N ? 1 : 0;
    const int r = row - arm * p.N;
    const int kb_total = p.K >> 4;
    const uint8_t* wrow = p.wq[arm] + (size_t)r * (p.K >> 1);
    const uint8_t* sc = p.sc[arm];
    for (int m = 0; m < p.M; ++m) {
        const uint16_t* xr = p.x + (size_t)m * p.K;
        const uint16_t* ur = PRO == 1 ? p.x2 + (size_t)m * p.K : nullptr;
        float acc = 0.f;
        for (int kb = lane; kb < kb_total; kb += 32) {
            const float s = nvk::ue4m3_to_f32(sc[nvk::swz_offset(r, kb, kb_total)]);
            float bd = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t byte = wrow[kb * 8 + i];
                uint32_t h2;
                asm("{ .reg .b8 t, z; .reg .b16 w; cvt.u16.u32 w, %1; mov.b16 {t, z}, w; cvt.rn.f16x2.e2m1x2 %0, t; }\n"
                    : "=r"(h2)
                    : "r"(byte));
                float2 wf = __half22float2(*reinterpret_cast<__half2*>(&h2));
                float x0 = nvk::bf16_bits_to_f32(xr[kb * 16 + 2 * i]);
                float x1 = nvk::bf16_bits_to_f32(xr[kb * 16 + 2 * i + 1]);
                if (PRO == 1) {
                    float u0 = nvk::bf16_bits_to_f32(ur[kb * 16 + 2 * i]);
                    float u1 = nvk::bf16_bits_to_f32(ur[kb * 16 + 2 * i + 1]);
                    x0 = nvk::bf16_bits_to_f32(nvk::f32_to_bf16_bits((x0 / (1.0f + expf(-x0))) * u0));
                    x1 = nvk::bf16_bits_to_f32(nvk::f32_to_bf16_bits((x1 / (1.0f + expf(-x1))) * u1));
                }
                bd = fmaf(wf.x, x0, bd);
                bd = fmaf(wf.y, x1, bd);
            }
            acc = fmaf(s, bd, acc);
        }
        acc = nvk::warp_sum(acc);
        if (lane == 0) p.y[arm][(size_t)m * p.N + r] = nvk::f32_to_bf16_bits(acc * p.alpha[arm]);
    }
}

// ------------------------------------------------------------------------------------------
// test/tuning hooks, set through nvk_b200_set_tuning (0 = automatic)
int g_force_ksplit = 0, g_force_hg = 0;

template <int NT, bool DUAL, int PRO, int HG, int KW, bool V8>
int launch_mma_v(cudaStream_t stream, GemmParams& p, int ksplit) {
    constexpr int MT = 8 * NT;
    constexpr int RS = 32 * HG + 4;
    constexpr int SUB = 4 / HG;
    p.tiles_per_arm = nvk::ceil_div(p.N, kRowsPerCta) * SUB;
    // phase length: keep the staged activations near 64 KiB
    int ph_cap = (64 * 1024) / (max(p.M, 1) * 512);
    ph_cap = max(KW, (ph_cap / KW) * KW);
    p.spc = nvk::ceil_div(p.nsc, ksplit);
    p.ph = min(ph_cap, nvk::ceil_div(p.spc, KW) * KW);
    p.x_stride = p.ph * 512 + 64;
    const size_t smem_x = (size_t)p.M * p.x_stride;
    const size_t smem_red = (size_t)(KW + 1) * MT * RS * sizeof(float);
    const size_t smem = max(smem_x, smem_red);
    static nvk::SmemOptin optin;
    auto* kern = w4a16_mma_kernel<NT, DUAL, PRO, HG, KW, V8>;
    if (int rc = optin.ensure((const void*)kern, smem)) return rc;
    const size_t ctas = (size_t)(DUAL ? 2 : 1) * p.tiles_per_arm;
    if (ctas > 65535) return NVK_ERR_GRID_AXIS;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ksplit, (unsigned)ctas, 1);
    cfg.blockDim = dim3(32 * HG * KW, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)ksplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ksplit > 1 ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kern, p);
}

template <int NT, bool DUAL, int PRO, int HG, int KW>
int launch_mma(cudaStream_t stream, GemmParams& p) {
    // 256-bit weight loads need K % 64 == 0 and 32-byte aligned matrices.
    const bool v8 = (p.K & 63) == 0 && (reinterpret_cast<uintptr_t>(p.wq[0]) & 31u) == 0 &&
                    (!DUAL || (reinterpret_cast<uintptr_t>(p.wq[1]) & 31u) == 0);
    // Split K across a cluster only when the row tiles alone leave most SMs idle and every
    // K-warp still keeps at least two super-chunks.
    int ksplit = 1;
    if (g_force_ksplit > 0) {
        ksplit = g_force_ksplit;
    } else {
        const int ctas = (DUAL ? 2 : 1) * nvk::ceil_div(p.N, kRowsPerCta) * (4 / HG);
        while (ksplit < 8 && ctas * ksplit < 148 && nvk::ceil_div(p.nsc, ksplit * 2) >= 2 * KW) ksplit *= 2;
    }
    return v8 ? launch_mma_v<NT, DUAL, PRO, HG, KW, true>(stream, p, ksplit)
              : launch_mma_v<NT, DUAL, PRO, HG, KW, false>(stream, p, ksplit);
}

template <int NT, bool DUAL, int PRO>
int launch_small_nt(cudaStream_t stream, GemmParams& p, int hg) {
    if (hg == 1) return launch_mma<NT, DUAL, PRO, 1, 8>(stream, p);
    if (hg == 2) return launch_mma<NT, DUAL, PRO, 2, 4>(stream, p);
    return launch_mma<NT, DUAL, PRO, 4, 2>(stream, p);
}

template <bool DUAL, int PRO>
int dispatch_mma(cudaStream_t stream, GemmParams& p) {
    // Rows per CTA grow with M: a CTA re-stages the activations of its whole K range, so more
    // tokens want more weight rows per staged activation byte.
    int hg = p.M <= 2 ? 1 : (p.M <= 4 ? 2 : 4);
    if (g_force_hg == 1 || g_force_hg == 2 || g_force_hg == 4) hg = g_force_hg;
    if (p.M <= 8) return launch_small_nt<1, DUAL, PRO>(stream, p, hg);
    if (p.M <= 16) return launch_small_nt<2, DUAL, PRO>(stream, p, hg);
    if (p.M <= 32) return launch_mma<4, DUAL, PRO, 4, 2>(stream, p);
    return launch_mma<8, DUAL, PRO, 4, 2>(stream, p);
}

bool aligned16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; }

// Common entry: validates, then picks the tensor-core route or the generic one.
int w4a16_linear(cudaStream_t stream, const uint8_t* wq_a, const uint8_t* sc_a, const uint8_t* wq_b,
                 const uint8_t* sc_b, const uint16_t* x, const uint16_t* x2, uint16_t* y_a, uint16_t* y_b,
                 float alpha_a, float alpha_b, int M, int N, int K, int pro, int max_m) {
    if (M <= 0 || M > max_m) return NVK_ERR_SHAPE;
    if ((K & 15) != 0) return NVK_ERR_SHAPE;
    GemmParams p = {};
    p.wq[0] = wq_a; p.wq[1] = wq_b;
    p.sc[0] = sc_a; p.sc[1] = sc_b;
    p.x = x; p.x2 = x2;
    p.y[0] = y_a; p.y[1] = y_b;
    p.alpha[0] = alpha_a; p.alpha[1] = alpha_b;
    p.M = M; p.N = N; p.K = K;
    p.tiles_per_arm = nvk::ceil_div(N, kRowsPerCta);
    p.k_tiles = nvk::ceil_div(K, 64);
    p.nsc = nvk::ceil_div(K, kSuper);
    const bool dual = wq_b != nullptr;
    const bool fast = (K & 31) == 0 && M <= 64 && aligned16(wq_a) && aligned16(sc_a) && aligned16(x) &&
                      (!dual || (aligned16(wq_b) && aligned16(sc_b))) && (pro == 0 || aligned16(x2)) &&
                      (size_t)(dual ? 2 : 1) * p.tiles_per_arm * 4 <= 65535;
    if (fast) {
        if (dual) return pro ? dispatch_mma<true, 1>(stream, p) : dispatch_mma<true, 0>(stream, p);
        return pro ? dispatch_mma<false, 1>(stream, p) : dispatch_mma<false, 0>(stream, p);
    }
    const int total = dual ? 2 * N : N;
    dim3 grid((unsigned)nvk::ceil_div(total, 8));
    if (pro)
        w4a16_rowwarp_kernel<1><<<grid, 256, 0, stream>>>(p);
    else
        w4a16_rowwarp_kernel<0><<<grid, 256, 0, stream>>>(p);
    return (int)cudaGetLastError();
}

}  // namespace

// ------------------------------------------------------------------------------------------
// C ABI.  Reference-named symbols keep the reference's argument order and refusals.
extern "C" {

int nvk_b200_set_tuning(int force_ksplit, int force_rows_per_cta) {
    if (force_ksplit != 0 && force_ksplit != 1 && force_ksplit != 2 && force_ksplit != 4 && force_ksplit != 8)
        return NVK_ERR_ARG;
    if (force_rows_per_cta != 0 && force_rows_per_cta != 32 && force_rows_per_cta != 64 && force_rows_per_cta != 128)
        return NVK_ERR_ARG;
    g_force_ksplit = force_ksplit;
    g_force_hg = force_rows_per_cta / 32;
    return 0;
}

int nv_kernels_nvfp4_gemv_bf16act(void* stream, const uint8_t* W_packed, const uint8_t* W_scales,
                                  const uint16_t* x_bf16, uint16_t* y, float alpha, int N, int K) {
    if (N <= 0 || K <= 0) return 0;
    if ((K & 15) != 0) return NVK_ERR_SHAPE;
    return w4a16_linear((cudaStream_t)stream, W_packed, W_scales, nullptr, nullptr, x_bf16, nullptr, y, nullptr,
                        alpha, 0.f, 1, N, K, 0, 1);
}

int nv_kernels_gemv_nvfp4_w4a16_dual_m1(void* stream, const uint8_t* wq_a, const uint8_t* sc_a,
                                        const uint8_t* wq_b, const uint8_t* sc_b, const uint16_t* x,
                                        uint16_t* y_a, uint16_t* y_b, float alpha_a, float alpha_b, int N,
                                        int K) {
    if (N <= 0 || K <= 0 || (K & 31) != 0) return NVK_ERR_SHAPE;
    if ((wq_b == nullptr) != (y_b == nullptr)) return NVK_ERR_SHAPE;
    if ((wq_b == nullptr) != (sc_b == nullptr)) return NVK_ERR_SHAPE;
    return w4a16_linear((cudaStream_t)stream, wq_a, sc_a, wq_b, sc_b, x, nullptr, y_a, y_b, alpha_a, alpha_b, 1,
                        N, K, 0, 1);
}

int nv_kernels_gemv_nvfp4_w4a16_silu_gate_up_in_m1(void* stream, const uint8_t* wq, const uint8_t* sc,
                                                   const uint16_t* gate, const uint16_t* up, uint16_t* y,
                                                   float alpha, int N, int K) {
    if (N <= 0 || K <= 0 || (K & 31) != 0) return NVK_ERR_SHAPE;
    return w4a16_linear((cudaStream_t)stream, wq, sc, nullptr, nullptr, gate, up, y, nullptr, alpha, 0.f, 1, N, K,
                        1, 1);
}

int nv_kernels_gemm_nvfp4_w4a16_mk_dual(void* stream, const uint8_t* wq_a, const uint8_t* sc_a,
                                        const uint8_t* wq_b, const uint8_t* sc_b, const uint16_t* x,
                                        uint16_t* y_a, uint16_t* y_b, float alpha_a, float alpha_b, int M, int N,
                                        int K) {
    if (M <= 0 || M > 16) return NVK_ERR_SHAPE;
    if (N <= 0 || K <= 0 || (K & 31) != 0) return NVK_ERR_SHAPE;
    if ((wq_b == nullptr) != (y_b == nullptr)) return NVK_ERR_SHAPE;
    if ((wq_b == nullptr) != (sc_b == nullptr)) return NVK_ERR_SHAPE;
    if (N % 32 != 0) return NVK_ERR_SHAPE;
    return w4a16_linear((cudaStream_t)stream, wq_a, sc_a, wq_b, sc_b, x, nullptr, y_a, y_b, alpha_a, alpha_b, M,
                        N, K, 0, 16);
}

// Additive entry: the same contraction for 1 <= M <= 64 tokens, optional second arm, optional
// SiLU(gate)*up prologue (x = gate, x2 = up; pass x2 = NULL for a plain activation).
int nvk_b200_linear_nvfp4_w4a16(void* stream, const uint8_t* wq_a, const uint8_t* sc_a, const uint8_t* wq_b,
                                const uint8_t* sc_b, const uint16_t* x, const uint16_t* x2, uint16_t* y_a,
                                uint16_t* y_b, float alpha_a, float alpha_b, int M, int N, int K) {
    if (N <= 0 || K <= 0) return 0;
    if ((wq_b == nullptr) != (y_b == nullptr)) return NVK_ERR_SHAPE;
    if ((wq_b == nullptr) != (sc_b == nullptr)) return NVK_ERR_SHAPE;
    return w4a16_linear((cudaStream_t)stream, wq_a, sc_a, wq_b, sc_b, x, x2, y_a, y_b, alpha_a, alpha_b, M, N, K,
                        x2 ? 1 : 0, 64);
}

}  // extern "C"
