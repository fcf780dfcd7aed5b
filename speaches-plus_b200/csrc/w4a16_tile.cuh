// Per-CTA tile of the NVFP4 W4A16 linear: parameter blocks, the cp.async weight ring, fragment
// dequantization and the m16n8k16 contraction.  Included by the translation units that wrap it in
// kernels; everything is in an unnamed namespace, so each of them gets its own copy.
#pragma once
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
    int bal_ctas;       // > 0: 16-row units are dealt round-robin over this many CTAs (see TileView::unit_p1)
    int spc;            // super-chunks per CTA (the CTA's K slice)
    int ph;             // super-chunks staged per phase
    int x_stride;       // bytes between token rows of the staged activations
    int ring_off;       // byte offset of the weight ring in dynamic shared memory
};

// One of a pair of per-arm parameters.  A select, not an indexed load: indexing a kernel parameter array
// with a run-time value makes the compiler copy the parameter block to local memory.
template <class T>
__device__ __forceinline__ T arm_pick(const T (&pair)[2], int arm) {
    return arm ? pair[1] : pair[0];
}

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    nvk::ptx::mma_m16n8k16_f16(d, a0, a1, a2, a3, b0, b1);
}

// CTAs per SM the tile kernels are compiled for (the register cap of __launch_bounds__).  The weight ring
// alone is 80 KB per CTA, so shared memory never admits a third CTA.  Up to 8 token columns: three, the
// setting the measured M = 1 kernel was built with (80 registers, no spills).  16 and 32 columns: two.
// 64: the staged activations and the ring together exceed half an SM's shared memory for all but the
// shortest K, so one CTA per SM runs whatever the registers, and none are given up for a second.
template <int NT>
constexpr int kTileCtasPerSm = NT >= 8 ? 1 : NT >= 2 ? 2 : 3;

constexpr int kDepth = 4;           // cp.async groups in flight per thread
constexpr int kSlotBytes = 2560;    // one warp, one iteration: 4 x 512 B of weights + 2 x 256 B of scales

// 16-byte (weights) and 8-byte (scales) asynchronous global -> shared copies; src_bytes == 0 writes
// zeros without touching global memory.
using nvk::ptx::cp_async16;
using nvk::ptx::cp_async8;
using nvk::ptx::cp_async_commit;
using nvk::ptx::cp_async_wait;

// Two ue4m3 scale bytes (the low half of `w`, bit 7 of each byte already cleared) -> f16x2.
// ue4m3 is the non-negative half of e4m3, so the hardware e4m3 convert is exact for 0x00..0x7E;
// 0x7F (never produced by an NVFP4 encoder, NaN in e4m3) converts to NaN and is repaired by
// fix_scale_7f below: the decode rule gives (1 + 7/8) * 2^8 = 480 for that byte.
__device__ __forceinline__ __half2 scales2_f16(uint32_t w) {
    uint32_t d = nvk::ptx::e4m3x2_to_f16x2(w);
    return *reinterpret_cast<__half2*>(&d);
}

// Non-zero if either half is NaN (only a 0x7F scale byte can make one).
__device__ __forceinline__ uint32_t scale_nan_bits(__half2 s) {
    const __half2 f = __hisnan2(s);   // 1.0 where NaN, else 0.0
    return *reinterpret_cast<const uint32_t*>(&f);
}
// Each NaN half becomes 480.0 (0x5F80); the other half is kept.  Off the hot path.
__device__ __noinline__ uint32_t fix_scale_7f(uint32_t bits) {
    if ((bits & 0x7FFFu) > 0x7C00u) bits = (bits & 0xFFFF0000u) | 0x5F80u;
    if ((bits & 0x7FFF0000u) > 0x7C000000u) bits = (bits & 0x0000FFFFu) | 0x5F800000u;
    return bits;
}

// In place: eight bf16 gate values (as 4 words) -> bf16(SiLU(gate) * up), fp32 math, one rounding.
__device__ __forceinline__ void silu_mul_bf16x8(uint32_t (&ws)[4], const uint4 u) {
    const uint32_t us[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float g0 = nvk::bf16_bits_to_f32(ws[i] & 0xFFFFu), g1 = nvk::bf16_bits_to_f32(ws[i] >> 16);
        const float u0 = nvk::bf16_bits_to_f32(us[i] & 0xFFFFu), u1 = nvk::bf16_bits_to_f32(us[i] >> 16);
        const uint32_t a0 = nvk::f32_to_bf16_bits((g0 / (1.0f + expf(-g0))) * u0);
        const uint32_t a1 = nvk::f32_to_bf16_bits((g1 / (1.0f + expf(-g1))) * u1);
        ws[i] = a0 | (a1 << 16);
    }
}

// A 128-row scale tile holds eight 16-row units u = 2*h + pair: rows 8h + g + 32*(2*pair + i),
// g = 0..7, i = 0..1 -- the 16 rows of one m16n8k16 A tile whose scales are 8 contiguous bytes per
// (g, k-tile).  One warp owns one unit; a CTA owns UG consecutive units and KW warps along K.
// A warp iteration covers 256 K values ("super-chunk"): lane (g, tg) takes, for each of its two
// rows, the two 16-byte pieces at K offsets 32*tg and 128 + 32*tg, so that one cp.async instruction
// moves whole 64-byte runs per row.  NT: number of 8-token column tiles.
// EPI == 2: how the GPUs of a K-sharded linear reach each other (see exchange_* below).
struct ExchangeArgs {
    uint8_t* peer[8];      // every rank's exchange buffer as mapped here; peer[rank] is our own
    uint32_t* epoch;       // [max_ctas] call counters of this rank, local memory
    int* err;              // becomes 1 + the rank that never arrived if a wait gives up
    const uint16_t* residual;
    int rank, world, max_ctas;
    int cta_elems;         // bf16 values of one CTA's inbox region: 128 rows x the row capacity of the buffers
    unsigned wait_limit;
};

// What one CTA works on: one arm's matrix, a set of token rows and where their outputs go.
struct TileView {
    const uint8_t* wq;
    const uint8_t* sc;
    const uint16_t* x;       // activation rows (gate when PRO == 1; packed e2m1 rows when PRO is 2 or 3)
    const uint16_t* x2;      // up rows when PRO == 1; the activation's ue4m3 scales when PRO is 2 or 3
    const int32_t* xrows;    // optional gather: token m reads row xrows[xrow0 + m]; else row xrow0 + m
    int x_rows;              // rows of x a gathered index may name (others read as zeros and are reported)
    int* status;             // optional word, bit 1 set when a gathered row index was out of range
    uint16_t* y;             // output row of token m is y + m * N
    float alpha;
    int xrow0;
    int M;                   // tokens (<= 8 * NT)
    int sub;                 // CTA index within the arm
    int unit_p1;             // 0: this warp's 16-row unit follows from `sub`; else 1 + its unit index within the
                             // arm, chosen by the caller (only where a warp sums all of K itself: KW == 1, no cluster)
    bool pdl;                // signal/await the neighbouring kernels of the stream here
    const uint8_t* ws;       // prepared activations (XWS only): 256-byte header of int pw[], then f16 stages
    // Used only by hooks that wait inside the kernel for an earlier operation of the same launch:
    const unsigned* gate;    // arrival counter of the operation that produces x (null: nothing to wait for)
    unsigned gate_target;    // arrivals that mean "complete"
    int* gate_err;           // set to 1 when the wait gives up
    unsigned gate_limit;     // polls before it does
    // Used only when EPI == 1 (the output is a residual update and/or carries a per-token multiplier):
    const uint16_t* residual;   // [M, N] bf16 added to the product before the single rounding, or null
    const float* row_scale;     // [M] per-token multiplier (an int8 row's dequant scale), or null
    float* rstd_pack;           // {rstd, sum of squares, arrival count}: see emit_rstd; or null
    float rstd_eps;
    unsigned rstd_blocks;       // CTAs of the launch (each arrives once)
    // Used only when PRO == 5 (the int8 scale is derived here from partial maxima):
    const float* absmax_partials;
    int n_partials;
    // Used only when EPI == 2 (the outputs are partial sums of a K-sharded linear that meet the other GPUs'
    // partials inside this launch; see exchange_* below):
    const ExchangeArgs* xch;    // the launch's exchange description (a __grid_constant__ kernel parameter)
    int xch_cta;                // this CTA's index in the launch (cluster ranks included)
    // Used only when PRO == 6 (an RMSNorm is applied while the activations are staged):
    const uint16_t* norm_w;     // [K] bf16
    const float* rstd_in;       // [rows] 1/rms per activation row, or null: computed here from the row
    float norm_eps;
};

// Exchange buffer of the fused linear + all-reduce (one per rank, the same layout everywhere):
//   [0, max_ctas * 32)   flags: uint32 flag[cta][8 ranks], written by the peers, carry the call number
//   then                  inbox: 2 parities x world x max_ctas x (128 * max_rows) bf16
// A CTA owns the same region of every inbox in every call (regions of different CTAs never overlap,
// whatever the matrix), so the two parities suffice: a rank can be at most one call ahead of a peer.
__host__ __device__ inline size_t exchange_flag_bytes(int max_ctas) { return (size_t)max_ctas * 8 * sizeof(uint32_t); }
__host__ __device__ inline size_t exchange_buffer_bytes(int world, int max_ctas, int max_rows) {
    return exchange_flag_bytes(max_ctas) + (size_t)2 * world * max_ctas * (128 * max_rows) * sizeof(uint16_t);
}
// element offset of (parity, source rank, cta) in an inbox
__device__ __forceinline__ size_t exchange_slot(const ExchangeArgs& xa, uint32_t parity, int src_rank, int cta) {
    return (((size_t)parity * xa.world + src_rank) * xa.max_ctas + cta) * (size_t)xa.cta_elems;
}

// The last CTA of a launch to arrive turns the launch's sum of squared outputs into the next
// RMSNorm's 1/rms: pack[0] = rsqrt(pack[1] / n + eps), then pack[1] and the arrival count return to
// zero for the next launch.  The float additions of the CTAs' partial sums arrive in no fixed order.
__device__ __forceinline__ void emit_rstd(float* pack, float block_ssq, unsigned blocks, int n, float eps) {
    atomicAdd(&pack[1], block_ssq);
    __threadfence();
    unsigned* count = reinterpret_cast<unsigned*>(pack) + 2;
    const unsigned prev = atomicInc(count, blocks - 1u);
    if (prev == blocks - 1u) {
        __threadfence();
        const float ssq = *reinterpret_cast<volatile float*>(&pack[1]);
        pack[0] = rsqrtf(ssq / (float)n + eps);
        pack[1] = 0.f;
    }
}

// How a tile sits in its launch.  LaunchHooks: one tile per CTA, K split over the CTAs along
// gridDim.x (a cluster when there is more than one), activations written by an earlier kernel.
struct LaunchHooks {
    __device__ static __forceinline__ int crank() { return (int)blockIdx.x; }
    __device__ static __forceinline__ int nranks() { return (int)gridDim.x; }
    __device__ static __forceinline__ void before_activations(const TileView&) {}
    __device__ static __forceinline__ uint4 load_x(const uint16_t* q) { return *reinterpret_cast<const uint4*>(q); }
};

// PRO: 0 = bf16 activations; 1 = bf16(SiLU(x) * x2); 2 = an NVFP4 activation row whose scales are row 0
// of a 128x4 swizzled tile; 3 = an NVFP4 activation row with a flat [K/16] scale array; 4 = int8
// activation rows (their dequant scales are applied in the epilogue through row_scale); 5 = one bf16
// activation row quantized to int8 here, scale = max(absmax_partials) / 127; 6 = bf16 rows through an
// RMSNorm, a = bf16(x * rstd * norm_w) with rstd = rsqrt(mean(x^2) + eps) summed in the order of the
// stand-alone norm kernel (256 threads striding the row, lanes, then warps) or taken from rstd_in.
// EPI: 0 = y = bf16(alpha * sum); 1 = y = bf16(fma(sum, alpha * row_scale, residual)), optionally
// followed by emit_rstd over the launch's outputs; 2 = the launch is one GPU's share of a K-sharded
// linear: bf16(alpha * sum) is a partial that is stored into every GPU's inbox (peer stores), the
// CTA raises its flag on every GPU, waits (bounded) for the same CTA of every other GPU and writes
// y = bf16(sum of the partials in rank order (+ residual)) -- the all-reduce happens tile by tile
// inside the linear's own launch.
// XWS: the activations were converted beforehand (x_prepare_kernel) into per-super-chunk f16 stages
// in a caller-supplied workspace; the CTA streams them through a shared ring next to the weights
// instead of converting its whole K range itself.  Needs KW == 1 (all warps walk K together).
template <int NT, int PRO, int UG, int KW, bool XWS = false, class HK = LaunchHooks, int EPI = 0>
__device__ __forceinline__ void w4a16_tile(const GemmParams& p, const TileView& t) {
    static_assert(!XWS || KW == 1, "the shared activation ring needs every warp on the same K step");
    constexpr int THREADS = 32 * UG * KW;
    constexpr int MT = 8 * NT;      // token columns
    constexpr int ROWS = 16 * UG;   // weight rows per CTA
    constexpr int SUB = 8 / UG;     // CTAs per 128-row scale tile
    NVK_DYN_SMEM_AS(uint8_t, smem);
    __shared__ uint32_t s_amax[MT];   // slice maximum (bf16 magnitude bits), then f32 bits of 2^-pw
    __shared__ int s_pw[MT];          // power of two currently folded into the accumulators
    __shared__ float s_rescale[MT];   // 2^(pw_old - pw_new) at a phase boundary
    __shared__ float s_q8[2];         // PRO == 5: the int8 row's dequant scale and its reciprocal
    __shared__ float s_ssq[32];       // EPI == 1: per-warp sums of squared outputs
    __shared__ int s_xch_ok;          // EPI == 2: every peer's partial arrived
    __shared__ float s_rstd[MT];      // PRO == 6: 1/rms of each activation row
    __shared__ float s_red8[8];       // PRO == 6: per-warp sums of squares

    cg::cluster_group cluster = cg::this_cluster();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ul = warp % UG, kw = warp / UG;  // local unit, K-warp
    const int gid = lane >> 2, tg = lane & 3;
    const int sub = t.sub;
    const int gu = t.unit_p1 > 0 ? t.unit_p1 - 1 : sub * UG + ul;   // 16-row unit within the arm
    const int mt = gu >> 3;                 // 128-row scale tile (== sub / SUB when derived from sub)
    const int u = gu & 7;                   // unit inside it
    const int h = u >> 1, pair = u & 1;
    const int crank = HK::crank();
    const int nranks = HK::nranks();
    const int M = t.M, N = p.N, K = p.K;

    const uint8_t* __restrict__ wq = t.wq;
    const uint8_t* __restrict__ sc = t.sc;
    const int row0 = mt * kRowsPerCta + 64 * pair + 8 * h + gid;  // second row is 32 further
    const size_t half_k = (size_t)(K >> 1);
    const bool rv0 = row0 < N, rv1 = row0 + 32 < N;
    // every row of the unit lies past N: the warp copies and multiplies nothing, it only keeps the barriers
    const bool idle = mt * kRowsPerCta + 64 * pair + 8 * h >= N;
    const uint8_t* w_row0 = rv0 ? wq + (size_t)row0 * half_k + tg * 16 : wq;
    const uint8_t* w_row1 = rv1 ? wq + (size_t)(row0 + 32) * half_k + tg * 16 : wq;
    const uint8_t* sc_thread =
        sc + (size_t)mt * p.k_tiles * 512 + (size_t)(8 * h + gid) * 16 + pair * 8 + (size_t)(tg >> 1) * 512;

    // shared memory: [activations / reduction scratch | weight ring]
    const uint32_t ring = nvk::ptx::smem_addr(smem) + (uint32_t)p.ring_off +
                          (uint32_t)(warp * kDepth * kSlotBytes) + (uint32_t)lane * 16;
    const uint8_t* ring_g = smem + p.ring_off + warp * kDepth * kSlotBytes + lane * 16;

    const int sc_begin = crank * p.spc;
    const int sc_end = min(p.nsc, sc_begin + p.spc);

    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;

    // Enqueue the copies of super-chunk s into ring slot `slot` (a no-op past the end of the slice).
    auto issue = [&](int s, int slot) {
        if (s < sc_end) {
            const uint32_t dst = ring + (uint32_t)(slot * kSlotBytes);
            if (XWS) {
                // this stage's activations: M rows of 512 bytes, row stride 576 in shared memory
                const uint8_t* xsrc = t.ws + 256 + (size_t)s * M * 512;
                const uint32_t xdst = nvk::ptx::smem_addr(smem) + (uint32_t)(slot * M * 576);
                for (int idx = threadIdx.x; idx < M * 32; idx += THREADS)
                    cp_async16(xdst + (idx >> 5) * 576 + (idx & 31) * 16, xsrc + (size_t)idx * 16, 16);
            }
            if (!idle) {
#pragma unroll
            for (int pc = 0; pc < 2; ++pc) {
                const int kk = s * kSuper + 128 * pc + 32 * tg;   // first K value of this piece
                const int okk = kk < K ? 16 : 0;
                const size_t off = (size_t)s * 128 + pc * 64;
                cp_async16(dst + (0 * 2 + pc) * 512, w_row0 + off, rv0 ? okk : 0);
                cp_async16(dst + (1 * 2 + pc) * 512, w_row1 + off, rv1 ? okk : 0);
                cp_async8(dst - (uint32_t)lane * 8 + 2048 + pc * 256, sc_thread + (size_t)(4 * s + 2 * pc) * 512,
                          okk ? 8 : 0);
            }
            }
        }
        cp_async_commit();
    };

    // B-fragment source rows: token 8n+gid, clamped to the last real token so that no load needs a
    // predicate (columns past M compute a duplicate that is never written out).
    uint32_t xs_tok[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n)
        xs_tok[n] = (uint32_t)(min(8 * n + gid, M - 1) * (XWS ? 576 : p.x_stride) + tg * 16);

    auto compute = [&](int slot, int xbase) {
        const uint8_t* src = ring_g + slot * kSlotBytes;
        const uint8_t* xs = smem + xbase;
        uint4 w[2][2];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int pc = 0; pc < 2; ++pc) w[i][pc] = *reinterpret_cast<const uint4*>(src + (i * 2 + pc) * 512);
        __half2 sp[2][2];  // [row i][piece]: the two block scales this lane's 32 values use
#pragma unroll
        for (int pc = 0; pc < 2; ++pc) {
            const uint2 sw = *reinterpret_cast<const uint2*>(src - lane * 8 + 2048 + pc * 256);
            sp[0][pc] = scales2_f16((sw.x & 0x7F7F7F7Fu) >> (16 * (tg & 1)));
            sp[1][pc] = scales2_f16((sw.y & 0x7F7F7F7Fu) >> (16 * (tg & 1)));
        }
        // a 0x7F scale byte (NaN after the hardware convert) decodes to 480 like every other route
        if (scale_nan_bits(sp[0][0]) | scale_nan_bits(sp[0][1]) | scale_nan_bits(sp[1][0]) | scale_nan_bits(sp[1][1])) {
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int pc = 0; pc < 2; ++pc) {
                    const uint32_t b = fix_scale_7f(*reinterpret_cast<const uint32_t*>(&sp[i][pc]));
                    sp[i][pc] = *reinterpret_cast<const __half2*>(&b);
                }
        }
#pragma unroll
        for (int wi = 0; wi < 8; ++wi) {
            uint32_t a[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint4& q = w[i][wi >> 2];
                const uint32_t word = (wi & 3) == 0 ? q.x : (wi & 3) == 1 ? q.y : (wi & 3) == 2 ? q.z : q.w;
                nvk::e2m1x8_to_f16x2x4(word, a[i][0], a[i][1], a[i][2], a[i][3]);
                const __half2 pr = sp[i][wi >> 2];
                const __half2 sc2 = (wi & 2) ? __high2half2(pr) : __low2half2(pr);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __half2 v = __hmul2(*reinterpret_cast<__half2*>(&a[i][j]), sc2);
                    a[i][j] = *reinterpret_cast<const uint32_t*>(&v);
                }
            }
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const uint4 xv = *reinterpret_cast<const uint4*>(xs + xs_tok[n] + wi * 64);
                mma_f16(acc[n], a[0][0], a[1][0], a[0][1], a[1][1], xv.x, xv.y);
                mma_f16(acc[n], a[0][2], a[1][2], a[0][3], a[1][3], xv.z, xv.w);
            }
        }
    };

    // Programmatic dependent launch: let the next kernel in the stream start its own weight
    // prefetch while this one runs, and prefetch our weights (which no earlier kernel writes) before
    // waiting for the previous kernel, whose output may be our activations.
    if (t.pdl) nvk::ptx::pdl_launch_dependents();
    int s_issue = sc_begin + kw, n_issued = 0, n_done = 0;
    if (XWS) {
        // The prepared activations come from the kernel just before this one.
        if (t.pdl) nvk::ptx::pdl_wait();
        if (threadIdx.x < MT) s_pw[threadIdx.x] = reinterpret_cast<const int*>(t.ws)[min((int)threadIdx.x, M - 1)];
#pragma unroll
        for (int d = 0; d < kDepth - 1; ++d) {
            issue(s_issue, n_issued % kDepth);
            s_issue += KW;
            ++n_issued;
        }
        for (int s = sc_begin; s < sc_end; ++s) {
            cp_async_wait<kDepth - 2>();  // this thread's copies for super-chunk s have landed
            __syncthreads();              // ... and everyone's; all warps are done with step s - 1
            issue(s_issue, n_issued % kDepth);  // refills the slot of step s - 1
            s_issue += KW;
            ++n_issued;
            if (!idle) compute(n_done % kDepth, (n_done % kDepth) * M * 576);
            ++n_done;
        }
        cp_async_wait<0>();
    } else {
#pragma unroll
    for (int d = 0; d < kDepth - 1; ++d) {
        issue(s_issue, n_issued % kDepth);
        s_issue += KW;
        ++n_issued;
    }
    if (t.pdl) nvk::ptx::pdl_wait();
    HK::before_activations(t);
    if (PRO == 5) {
        // row maximum = the largest partial maximum (first warp), then scale = max / 127
        if (warp == 0) {
            float a = 0.f;
            for (int i = lane; i < t.n_partials; i += 32) a = fmaxf(a, t.absmax_partials[i]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
            if (lane == 0) {
                const float scale = a / 127.0f;
                s_q8[0] = scale;
                s_q8[1] = scale > 0.f ? 1.0f / scale : 0.f;
            }
        }
        __syncthreads();
    }

    if (PRO == 6) {
        static_assert(PRO != 6 || THREADS == 256, "the row sum follows the 256-thread norm kernel");
        for (int m = 0; m < M; ++m) {
            float rs;
            if (t.rstd_in != nullptr) {
                rs = t.rstd_in[t.xrow0 + m];
            } else {
                const uint16_t* xr = t.x + (size_t)(t.xrow0 + m) * K;
                float ss = 0.f;
                for (int i = threadIdx.x; i < K; i += THREADS) {
                    const float f = nvk::bf16_bits_to_f32(xr[i]);
                    ss = fmaf(f, f, ss);   // an explicit fma: every copy of this sum rounds alike
                }
                ss = nvk::warp_sum(ss);
                if (lane == 0) s_red8[warp] = ss;
                __syncthreads();
                float tot = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) tot += s_red8[i];
                rs = rsqrtf(tot / (float)K + t.norm_eps);
                __syncthreads();   // s_red8 is rewritten for the next row
            }
            if (threadIdx.x == 0) s_rstd[m] = rs;
        }
        __syncthreads();
    }

    for (int p0 = sc_begin; p0 < sc_end; p0 += p.ph) {
        const int pend = min(sc_end, p0 + p.ph);
        const int nsp = pend - p0;

        // ---- stage activations for super-chunks [p0, pend) ----
        if (threadIdx.x < MT) s_amax[threadIdx.x] = 0u;
        __syncthreads();  // also orders the previous phase's reads before this phase's writes
        const int pieces_per_tok = nsp * 32;
        const int total_pieces = M * pieces_per_tok;
        // Each 16-byte piece (8 activations) is loaded once and kept in registers across the
        // block-wide maximum when the phase is small enough (kXRegs pieces per thread); larger
        // phases re-read the piece (an L1/L2 hit) for the conversion pass.
        constexpr int kXRegs = 4;
        const bool keep = total_pieces <= kXRegs * THREADS;
        uint4 xr[kXRegs];
        auto load_piece = [&](int idx, uint32_t (&ws)[4]) -> bool {
            const int m = idx / pieces_per_tok;
            const int rem = idx - m * pieces_per_tok;
            const int k = (p0 + (rem >> 5)) * kSuper + (rem & 31) * 8;
            if (k >= K) return false;
            int xrow = t.xrow0 + m;
            if (t.xrows != nullptr) {
                xrow = t.xrows[t.xrow0 + m];
                if ((unsigned)xrow >= (unsigned)t.x_rows) {   // a routing table must not steer a load
                    if (t.status != nullptr) atomicOr(t.status, 2);
                    return false;
                }
            }
            if (PRO == 4) {
                // int8 row: the integers (at most 7 bits) are exact as bf16
                const uint2 q8 = *reinterpret_cast<const uint2*>(reinterpret_cast<const int8_t*>(t.x) + (size_t)xrow * K + k);
                const uint32_t qs[2] = {q8.x, q8.y};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float lo = (float)(int)(int8_t)((qs[i >> 1] >> (16 * (i & 1))) & 0xFFu);
                    const float hi = (float)(int)(int8_t)((qs[i >> 1] >> (16 * (i & 1) + 8)) & 0xFFu);
                    ws[i] = (uint32_t)nvk::f32_to_bf16_bits(lo) | ((uint32_t)nvk::f32_to_bf16_bits(hi) << 16);
                }
                return true;
            }
            if (PRO == 5) {
                // bf16 row -> int8 with the row scale derived above: q = clamp(rn(v / scale), +-127)
                const uint4 v = HK::load_x(t.x + (size_t)xrow * K + k);
                const uint32_t vs[4] = {v.x, v.y, v.z, v.w};
                const float inv = s_q8[1];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int q0 = max(-127, min(127, __float2int_rn(nvk::bf16_bits_to_f32(vs[i] & 0xFFFFu) * inv)));
                    const int q1 = max(-127, min(127, __float2int_rn(nvk::bf16_bits_to_f32(vs[i] >> 16) * inv)));
                    ws[i] = (uint32_t)nvk::f32_to_bf16_bits((float)q0) | ((uint32_t)nvk::f32_to_bf16_bits((float)q1) << 16);
                }
                return true;
            }
            if (PRO == 2 || PRO == 3) {
                // NVFP4 activation row: eight e2m1 values times their block's ue4m3 scale.  The product
                // has at most six significand bits, so it is exact as bf16 and the W4A4 contraction
                // sum (w*ws)*(a*as) is this tile's ordinary W4A16 sum over an exactly dequantized row.
                const uint8_t* xa = reinterpret_cast<const uint8_t*>(t.x) + (size_t)xrow * (size_t)(K >> 1);
                const uint8_t* xs = reinterpret_cast<const uint8_t*>(t.x2);
                const int kb = k >> 4;
                const uint32_t sb = PRO == 2 ? xs[(size_t)(kb >> 2) * 512 + (kb & 3)]   // row 0 of a swizzled tile
                                             : xs[kb];                                  // flat [K/16]
                const float sf = nvk::ue4m3_to_f32(sb);
                uint32_t h[4];
                nvk::e2m1x8_to_f16x2x4(*reinterpret_cast<const uint32_t*>(xa + (k >> 1)), h[0], h[1], h[2], h[3]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[i]));
                    ws[i] = (uint32_t)nvk::f32_to_bf16_bits(f.x * sf) | ((uint32_t)nvk::f32_to_bf16_bits(f.y * sf) << 16);
                }
                return true;
            }
            const size_t xr0 = (size_t)xrow * K + k;
            const uint4 v = HK::load_x(t.x + xr0);
            ws[0] = v.x; ws[1] = v.y; ws[2] = v.z; ws[3] = v.w;
            if (PRO == 6) {
                const uint4 nw = *reinterpret_cast<const uint4*>(t.norm_w + k);
                const uint32_t nws[4] = {nw.x, nw.y, nw.z, nw.w};
                const float rs = s_rstd[m];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float lo = nvk::bf16_bits_to_f32(ws[i] & 0xFFFFu) * rs * nvk::bf16_bits_to_f32(nws[i] & 0xFFFFu);
                    const float hi = nvk::bf16_bits_to_f32(ws[i] >> 16) * rs * nvk::bf16_bits_to_f32(nws[i] >> 16);
                    ws[i] = (uint32_t)nvk::f32_to_bf16_bits(lo) | ((uint32_t)nvk::f32_to_bf16_bits(hi) << 16);
                }
            }
            if (PRO == 1) silu_mul_bf16x8(ws, HK::load_x(t.x2 + xr0));
            return true;
        };
        auto store_piece = [&](int idx, const uint32_t (&ws)[4], bool valid) {
            const int m = idx / pieces_per_tok;
            const int rem = idx - m * pieces_per_tok;
            const int scl = rem >> 5, q = rem & 31;
            uint4 o = make_uint4(0u, 0u, 0u, 0u);
            if (valid) {
                const float sc2 = __uint_as_float(s_amax[m]);
                uint32_t os[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float lo = nvk::bf16_bits_to_f32(ws[i] & 0xFFFFu) * sc2;
                    const float hi = nvk::bf16_bits_to_f32(ws[i] >> 16) * sc2;
                    const __half2 h2 = __floats2half2_rn(lo, hi);
                    os[i] = *reinterpret_cast<const uint32_t*>(&h2);
                }
                o = make_uint4(os[0], os[1], os[2], os[3]);
            }
            // 8-value piece q of a super-chunk belongs to lane column tg' = (q % 16) / 4 and is that
            // lane's fragment word wi = 4*(q / 16) + q % 4; pieces with equal wi are stored adjacently
            // (conflict-free 128-bit fragment reads).
            const int off = m * p.x_stride + scl * 512 + ((4 * (q >> 4) + (q & 3)) * 4 + ((q & 15) >> 2)) * 16;
            *reinterpret_cast<uint4*>(smem + off) = o;
        };
#pragma unroll
        for (int j = 0; j < kXRegs; ++j) xr[j] = make_uint4(0u, 0u, 0u, 0u);
        {
            int j = 0;
            for (int idx = threadIdx.x; idx < total_pieces; idx += THREADS, ++j) {
                uint32_t ws[4] = {0u, 0u, 0u, 0u};
                const bool valid = load_piece(idx, ws);
                uint32_t mx = 0u;
#pragma unroll
                for (int i = 0; i < 4; ++i) mx = max(mx, max(ws[i] & 0x7FFFu, (ws[i] >> 16) & 0x7FFFu));
                if (valid && mx) atomicMax(&s_amax[idx / pieces_per_tok], mx);
                if (keep) {
#pragma unroll
                    for (int r = 0; r < kXRegs; ++r)
                        if (r == j) xr[r] = make_uint4(ws[0], ws[1], ws[2], ws[3]);
                }
            }
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
                acc[n][0] *= r0; acc[n][1] *= r1; acc[n][2] *= r0; acc[n][3] *= r1;
            }
        }
        {
            int j = 0;
            for (int idx = threadIdx.x; idx < total_pieces; idx += THREADS, ++j) {
                uint32_t ws[4] = {0u, 0u, 0u, 0u};
                bool valid;
                if (keep) {
                    uint4 v = xr[0];
#pragma unroll
                    for (int r = 1; r < kXRegs; ++r)
                        if (r == j) v = xr[r];
                    ws[0] = v.x; ws[1] = v.y; ws[2] = v.z; ws[3] = v.w;
                    const int rem = idx % pieces_per_tok;
                    valid = (p0 + (rem >> 5)) * kSuper + (rem & 31) * 8 < K;
                } else {
                    valid = load_piece(idx, ws);
                }
                store_piece(idx, ws, valid);
            }
        }
        __syncthreads();
        // ---- stream this phase's weights through the ring ----
        if (!idle)
        for (int s = p0 + kw; s < pend; s += KW) {
            issue(s_issue, n_issued % kDepth);
            s_issue += KW;
            ++n_issued;
            cp_async_wait<kDepth - 1>();  // this thread's copies for super-chunk s have landed
            compute(n_done % kDepth, (s - p0) * 512);
            ++n_done;
        }
    }
    cp_async_wait<0>();
    if (sc_begin >= sc_end && threadIdx.x < MT) s_pw[threadIdx.x] = 0;  // empty slice: acc is zero
    }  // !XWS

    // y for (token m, row r) from the finished sum v (the activation power of two already undone)
    float ssq = 0.f;   // EPI == 1 with rstd_pack: this thread's sum of squared (rounded) outputs
    uint32_t xch_call = 0u;   // EPI == 2: this call's number for this CTA
    if (EPI == 2) xch_call = t.xch->epoch[t.xch_cta] + 1u;
    auto finish = [&](float v, int m, int r, uint16_t* __restrict__ y, float alpha) {
        uint16_t out;
        if (EPI == 2) {
            // the partial goes to slot [our rank] of this CTA's region in every GPU's inbox, ours included
            out = nvk::f32_to_bf16_bits(v * alpha);
            const ExchangeArgs& xa = *t.xch;
            const size_t at = exchange_slot(xa, xch_call & 1u, xa.rank, t.xch_cta) +
                              (size_t)(m * kRowsPerCta + (r - mt * kRowsPerCta));
            for (int g = 0; g < xa.world; ++g)
                reinterpret_cast<uint16_t*>(xa.peer[g] + exchange_flag_bytes(xa.max_ctas))[at] = out;
            return;
        }
        if (EPI == 0) {
            out = nvk::f32_to_bf16_bits(v * alpha);
        } else {
            float mult = alpha;
            if (PRO == 5) mult *= s_q8[0];
            if (t.row_scale != nullptr) mult *= t.row_scale[m];
            const float base = t.residual != nullptr ? nvk::bf16_bits_to_f32(t.residual[(size_t)m * N + r]) : 0.f;
            out = nvk::f32_to_bf16_bits(fmaf(v, mult, base));
            const float o = nvk::bf16_bits_to_f32(out);
            ssq = fmaf(o, o, ssq);
        }
        y[(size_t)m * N + r] = out;
    };

    if (KW == 1 && nranks == 1) {
        // One warp saw the whole of K for its rows: the accumulator fragment is the result.
        const float alpha1 = t.alpha;
        uint16_t* __restrict__ y1 = t.y;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int m = 8 * n + 2 * tg + (j & 1);
                const int r = row0 + 32 * (j >> 1);
                if (m < M && r < N) {
                    const float d = __uint_as_float((uint32_t)(127 + s_pw[m]) << 23);
                    finish(acc[n][j] * d, m, r, y1, alpha1);
                }
            }
        }
    } else {
    // ---- sum the K-warps of this CTA: red[kw][token][row] ----
    __syncthreads();
    float* red = reinterpret_cast<float*>(smem);
    constexpr int RS = ROWS + 4;  // padded row count per token column
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        // local row index = ul*16 + i*8 + gid with i = 0 (c0/c1) and 1 (c2/c3)
        const int rl = ul * 16 + gid;
        const int c = 8 * n + 2 * tg;
        float* base = red + (size_t)kw * MT * RS;
        // undo the activation power of two
        const float d0 = __uint_as_float((uint32_t)(127 + s_pw[c]) << 23);
        const float d1 = __uint_as_float((uint32_t)(127 + s_pw[c + 1]) << 23);
        base[(c)*RS + rl] = acc[n][0] * d0;
        base[(c + 1) * RS + rl] = acc[n][1] * d1;
        base[(c)*RS + rl + 8] = acc[n][2] * d0;
        base[(c + 1) * RS + rl + 8] = acc[n][3] * d1;
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
    const float alpha = t.alpha;
    uint16_t* __restrict__ y = t.y;
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
        // undo the local row numbering: rl = ul*16 + i*8 + g, unit = (sub % SUB)*UG + ul
        const int uu = (sub % SUB) * UG + (rl >> 4);
        const int n_out = mt * kRowsPerCta + 32 * (2 * (uu & 1) + ((rl >> 3) & 1)) + 8 * (uu >> 1) + (rl & 7);
        if (n_out < N) finish(v, m, n_out, y, alpha);
    }
    if (nranks > 1) cluster.sync();  // peers may still be reading this CTA's partial
    }

    if (EPI == 2) {
        const ExchangeArgs& xa = *t.xch;
        // every partial of this CTA is on its way: make them visible system-wide, then one flag per GPU
        if (threadIdx.x == 0) s_xch_ok = 1;
        __threadfence_system();
        __syncthreads();
        uint8_t* own = xa.peer[xa.rank];
        if ((int)threadIdx.x < xa.world) {
            const int g = (int)threadIdx.x;
            nvk::ptx::st_release_sys(reinterpret_cast<uint32_t*>(xa.peer[g]) + t.xch_cta * 8 + xa.rank, xch_call);
            const uint32_t* mine = reinterpret_cast<const uint32_t*>(own) + t.xch_cta * 8 + g;
            if (!nvk::bounded_wait_ge(mine, xch_call, xa.wait_limit)) {
                atomicExch(xa.err, 1 + g);
                s_xch_ok = 0;
            }
        }
        __syncthreads();
        if (s_xch_ok) {
            const uint16_t* inbox = reinterpret_cast<const uint16_t*>(own + exchange_flag_bytes(xa.max_ctas));
            auto collect = [&](int m, int r) {
                const size_t local = (size_t)(m * kRowsPerCta + (r - mt * kRowsPerCta));
                float acc = 0.f;
                for (int g = 0; g < xa.world; ++g)
                    acc += nvk::bf16_bits_to_f32(inbox[exchange_slot(xa, xch_call & 1u, g, t.xch_cta) + local]);
                if (xa.residual != nullptr) acc += nvk::bf16_bits_to_f32(xa.residual[(size_t)m * N + r]);
                t.y[(size_t)m * N + r] = nvk::f32_to_bf16_bits(acc);
            };
            // the elements this thread pushed, in the same enumeration as above
            if (KW == 1 && nranks == 1) {
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int m = 8 * n + 2 * tg + (j & 1);
                        const int r = row0 + 32 * (j >> 1);
                        if (m < M && r < N) collect(m, r);
                    }
            } else {
                const int rows_per_rank = ROWS / nranks;
                for (int i = threadIdx.x; i < M * rows_per_rank; i += THREADS) {
                    const int m = i / rows_per_rank;
                    const int rl = crank * rows_per_rank + (i - m * rows_per_rank);
                    const int uu = (sub % SUB) * UG + (rl >> 4);
                    const int n_out = mt * kRowsPerCta + 32 * (2 * (uu & 1) + ((rl >> 3) & 1)) + 8 * (uu >> 1) + (rl & 7);
                    if (n_out < N) collect(m, n_out);
                }
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) xa.epoch[t.xch_cta] = xch_call;   // also after a failed wait: the ranks stay in step
    }

    if (EPI == 1 && t.rstd_pack != nullptr) {
        // CTA's sum of squares: lanes, then warps in order, then one arrival for the whole CTA
        ssq = nvk::warp_sum(ssq);
        if (lane == 0) s_ssq[warp] = ssq;
        __syncthreads();
        if (threadIdx.x == 0) {
            float blk = 0.f;
            for (int w = 0; w < THREADS / 32; ++w) blk += s_ssq[w];
            emit_rstd(t.rstd_pack, blk, t.rstd_blocks, N, t.rstd_eps);
        }
    }
}

// Host side: lays out one launch's dynamic shared memory ([staged activations or reduction scratch |
// weight ring]) for a CTA of 8 warps owning one 128-row scale tile (UG = 8, KW = 1) with K split over
// `ksplit` CTAs, and returns its size.  M tokens, MT = 8 * NT token columns.
inline size_t tile_layout_rows128(GemmParams& p, int M, int MT, int ksplit) {
    constexpr int RS = 128 + 4;
    int ph_cap = (48 * 1024) / ((M > 1 ? M : 1) * 512);
    if (ph_cap < 1) ph_cap = 1;
    p.spc = nvk::ceil_div(p.nsc, ksplit);
    p.ph = ph_cap < p.spc ? ph_cap : p.spc;
    if (p.ph < 1) p.ph = 1;
    p.x_stride = p.ph * 512 + 64;
    const size_t smem_x = (size_t)M * p.x_stride;
    const size_t smem_red = (size_t)2 * MT * RS * sizeof(float);
    p.ring_off = (int)(((smem_x > smem_red ? smem_x : smem_red) + 127) / 128 * 128);
    return (size_t)p.ring_off + (size_t)8 * kDepth * kSlotBytes;
}

// K split for a launch of `ctas` row-tile CTAs: over a cluster, only while the row tiles alone leave
// SMs idle and every CTA keeps at least two super-chunks.
inline int tile_ksplit(int ctas, int nsc) {
    int ksplit = 1;
    while (ksplit < 8 && ctas * ksplit < 148 && nvk::ceil_div(nsc, ksplit * 2) >= 2) ksplit *= 2;
    return ksplit;
}

}  // namespace
