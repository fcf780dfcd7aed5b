// NVFP4 weight-only (W4A16) linear for decode-sized M on sm_100a.
//
//   y[m, n] = bf16( alpha * sum_k e2m1(W[n,k]) * ue4m3(S[n, k/16]) * x[m, k] ),  fp32 accumulate
//
// Weights are streamed once from HBM.  Every thread copies its own fragment bytes with 16-byte
// cp.async (L1 bypass) into a thread-private slot of a shared-memory ring kDepth iterations ahead
// of use, so the bytes in flight per SM do not depend on registers or on how many warps share the
// issue slots.  Fragments are unpacked with the native e2m1x2 -> f16x2 convert, multiplied by their
// block scale in f16 (exact: a 2-bit by 4-bit significand product; scales come from the native
// e4m3x2 -> f16x2 convert) and contracted against the activations on the tensor cores with fp32
// accumulation (m16n8k16).  A warp owns a 16-row unit of the 128x4 swizzled scale layout whose
// scales are 8 contiguous bytes per (row pair, k-tile); K is split over the warps of a CTA and, for
// small N, over the CTAs of a thread-block cluster whose partial tiles are summed through
// distributed shared memory in a fixed order (deterministic, no global scratch).
//
// Activations are bf16.  They are staged per CTA into shared memory as f16 after an exact
// power-of-two pre-scale chosen from the slice's own maximum (bf16 has 8 significand bits, f16
// has 11, so every value within 2^31 of the slice maximum converts exactly); the power of two is
// undone in fp32 before alpha is applied.
#include "w4a16_tile.cuh"

namespace {

template <int NT, bool DUAL, int PRO, int UG, int KW>
__global__ void __launch_bounds__(32 * UG * KW, kTileCtasPerSm<NT>) w4a16_mma_kernel(const GemmParams p) {
    const int tile = blockIdx.y;
    int arm = DUAL ? (tile >= p.tiles_per_arm ? 1 : 0) : 0;
    int unit_p1 = 0;
    if (UG == 8 && KW == 1 && p.bal_ctas > 0) {
        // Units dealt round-robin: warp w of CTA c takes unit w * bal_ctas + c of the launch (both arms
        // counted through), so that the CTAs -- all resident at once -- carry equal numbers of busy warps.
        // Units past the end name rows >= N and idle.
        const int units_per_arm = p.tiles_per_arm * 8;
        int gu = (int)(threadIdx.x >> 5) * p.bal_ctas + tile;
        arm = DUAL && gu >= units_per_arm ? 1 : 0;
        gu -= arm * units_per_arm;
        unit_p1 = gu + 1;
    }
    TileView t = {};
    t.unit_p1 = unit_p1;
    t.wq = arm_pick(p.wq, arm);
    t.sc = arm_pick(p.sc, arm);
    t.x = p.x;
    t.x2 = p.x2;
    t.xrows = nullptr;
    t.x_rows = 0;
    t.status = nullptr;
    t.y = arm_pick(p.y, arm);
    t.alpha = arm_pick(p.alpha, arm);
    t.xrow0 = 0;
    t.M = p.M;
    t.sub = tile - arm * p.tiles_per_arm;
    t.pdl = true;
    t.ws = nullptr;
    w4a16_tile<NT, PRO, UG, KW>(p, t);
}

template <int NT, bool DUAL>
__global__ void __launch_bounds__(256, NT >= 4 ? 1 : 2) w4a16_mma_ws_kernel(const GemmParams p, const uint8_t* ws) {
    const int tile = blockIdx.y;
    const int arm = DUAL ? (tile >= p.tiles_per_arm ? 1 : 0) : 0;
    TileView t = {};
    t.wq = arm_pick(p.wq, arm);
    t.sc = arm_pick(p.sc, arm);
    t.x = nullptr;
    t.x2 = nullptr;
    t.xrows = nullptr;
    t.x_rows = 0;
    t.status = nullptr;
    t.y = arm_pick(p.y, arm);
    t.alpha = arm_pick(p.alpha, arm);
    t.xrow0 = 0;
    t.M = p.M;
    t.sub = tile - arm * p.tiles_per_arm;
    t.pdl = true;
    t.ws = ws;
    w4a16_tile<NT, 0, 8, 1, true>(p, t);
}

// Converts the activations of one token (one CTA per token) to f16 once for all CTAs of the GEMM:
// exact power-of-two pre-scale from the token's maximum, written as ceil(K/256) stages of 512 bytes
// in the fragment order the GEMM reads, zero-padded past K.  Header word m = the token's power of two.
template <int PRO>
__global__ void __launch_bounds__(256) x_prepare_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ x2,
                                                         uint8_t* __restrict__ ws, int M, int K, int nsc) {
    __shared__ uint32_t s_max;
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const int m = blockIdx.x;
    if (threadIdx.x == 0) s_max = 0u;
    __syncthreads();
    const int pieces = nsc * 32;
    auto load = [&](int idx, uint32_t (&ws4)[4]) -> bool {
        const int k = idx * 8;
        if (k >= K) return false;
        const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)m * K + k);
        ws4[0] = v.x; ws4[1] = v.y; ws4[2] = v.z; ws4[3] = v.w;
        if (PRO == 1) silu_mul_bf16x8(ws4, *reinterpret_cast<const uint4*>(x2 + (size_t)m * K + k));
        return true;
    };
    uint32_t mx = 0u;
    for (int idx = threadIdx.x; idx < pieces; idx += 256) {
        uint32_t w4[4];
        if (load(idx, w4)) {
#pragma unroll
            for (int i = 0; i < 4; ++i) mx = max(mx, max(w4[i] & 0x7FFFu, (w4[i] >> 16) & 0x7FFFu));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0 && mx) atomicMax(&s_max, mx);
    __syncthreads();
    const int pw = max((int)(s_max >> 7) - 141, -100);
    if (threadIdx.x == 0) reinterpret_cast<int*>(ws)[m] = pw;
    const float sc2 = __uint_as_float((uint32_t)(127 - pw) << 23);
    for (int idx = threadIdx.x; idx < pieces; idx += 256) {
        uint32_t w4[4];
        uint4 o = make_uint4(0u, 0u, 0u, 0u);
        if (load(idx, w4)) {
            uint32_t os[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __half2 h2 = __floats2half2_rn(nvk::bf16_bits_to_f32(w4[i] & 0xFFFFu) * sc2,
                                                     nvk::bf16_bits_to_f32(w4[i] >> 16) * sc2);
                os[i] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            o = make_uint4(os[0], os[1], os[2], os[3]);
        }
        const int sidx = idx >> 5, q = idx & 31;
        const int perm = (4 * (q >> 4) + (q & 3)) * 4 + ((q & 15) >> 2);
        *reinterpret_cast<uint4*>(ws + 256 + ((size_t)sidx * M + m) * 512 + perm * 16) = o;
    }
}

// Grouped experts: blockIdx.z is an expert whose matrices sit at a fixed stride in a bank, whose
// tokens are the sorted slots [offsets[e], offsets[e+1]) and whose alpha is alphas[e].  A CTA of an
// expert without tokens exits at once; an expert with more than 8 tokens is walked in chunks of 8
// (its weights then come from L2).  Outputs are written in sorted-slot order.
struct GroupedParams {
    const float* alphas[2];
    const int32_t* offsets;    // [E + 1]
    const int32_t* xrows;      // [slots] gather index into x rows, or null (row = slot)
    size_t w_stride;           // bytes between experts in the packed-weight banks
    size_t sc_stride;          // bytes between experts in the scale banks
    const int32_t* active;     // optional: the experts that have slots; blockIdx.z indexes this list
    const int32_t* n_active;   // its length (device)
    int n_experts;
    int n_slots;               // rows of the output buffers (and entries of xrows)
    int x_rows;                // rows of x
    int* status;               // optional: bit 0 set when an offset, bit 1 when a row index was out of range
};

template <bool DUAL, int PRO>
__global__ void __launch_bounds__(256, 3) w4a16_grouped_kernel(const GemmParams p, const GroupedParams g) {
    // The routing tables are written by the kernels just before this one in the stream.
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    int e = blockIdx.z;
    if (g.active != nullptr) {
        // grid z covers the most experts that can be active; entries past the list's end have no work
        if ((int)blockIdx.z >= min(*g.n_active, g.n_experts)) return;
        e = g.active[blockIdx.z];
        if (e < 0 || e >= g.n_experts) {
            if (g.status != nullptr && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(g.status, 1);
            return;
        }
    }
    // Offsets are data, not trusted: a slot range is cut to the buffers' rows, and a range that had
    // to be cut is reported instead of followed.
    const int raw_begin = g.offsets[e], raw_end = g.offsets[e + 1];
    const int begin = min(max(raw_begin, 0), g.n_slots);
    const int end = min(max(raw_end, begin), g.n_slots);
    if ((begin != raw_begin || end != raw_end) && g.status != nullptr && threadIdx.x == 0 && blockIdx.y == 0)
        atomicOr(g.status, 1);
    if (end <= begin) return;
    const int tile = blockIdx.y;
    const int arm = DUAL ? (tile >= p.tiles_per_arm ? 1 : 0) : 0;
    TileView t = {};
    t.wq = arm_pick(p.wq, arm) + (size_t)e * g.w_stride;
    t.sc = arm_pick(p.sc, arm) + (size_t)e * g.sc_stride;
    t.x = p.x;
    t.x2 = p.x2;
    t.xrows = g.xrows;
    t.x_rows = g.x_rows;
    t.status = g.status;
    t.alpha = arm_pick(g.alphas, arm)[e];
    t.sub = tile - arm * p.tiles_per_arm;
    t.pdl = false;
    t.ws = nullptr;
    for (int c0 = begin; c0 < end; c0 += 8) {
        t.xrow0 = c0;
        t.M = min(8, end - c0);
        t.y = arm_pick(p.y, arm) + (size_t)c0 * p.N;
        if (c0 > begin) __syncthreads();  // the previous chunk's shared-memory reads are done
        w4a16_tile<1, PRO, 8, 1>(p, t);
    }
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
    const uint8_t* wrow = arm_pick(p.wq, arm) + (size_t)r * (p.K >> 1);
    const uint8_t* sc = arm_pick(p.sc, arm);
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
                uint32_t h2 = nvk::ptx::e2m1x2_to_f16x2(byte);
                float2 wf = __half22float2(*reinterpret_cast<__half2*>(&h2));
                float x0, x1;
                if (PRO >= 2) {
                    const uint8_t* xa = reinterpret_cast<const uint8_t*>(p.x) + (size_t)m * (p.K >> 1);
                    const uint8_t* xs = reinterpret_cast<const uint8_t*>(p.x2);
                    const float sf = nvk::ue4m3_to_f32(PRO == 2 ? xs[(size_t)(kb >> 2) * 512 + (kb & 3)] : xs[kb]);
                    uint32_t a2 = nvk::ptx::e2m1x2_to_f16x2(xa[kb * 8 + i]);
                    const float2 af = __half22float2(*reinterpret_cast<__half2*>(&a2));
                    x0 = af.x * sf;
                    x1 = af.y * sf;
                } else {
                    x0 = nvk::bf16_bits_to_f32(xr[kb * 16 + 2 * i]);
                    x1 = nvk::bf16_bits_to_f32(xr[kb * 16 + 2 * i + 1]);
                }
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
        if (lane == 0) arm_pick(p.y, arm)[(size_t)m * p.N + r] = nvk::f32_to_bf16_bits(acc * arm_pick(p.alpha, arm));
    }
}

// ------------------------------------------------------------------------------------------
// Test/tuning hooks (0 = automatic), set through nvk_b200_set_tuning / nvk_b200_set_pdl.  They are
// per calling thread: the entry points may be called from any thread, and one thread's experiment
// must not change another thread's launches.
thread_local int g_force_ksplit = 0, g_force_ug = 0;
thread_local int g_balance = 0;  // unit dealing over a full-GPU grid: 0 = where it evens the SMs' load, 1 = wherever possible, 2 = never

constexpr int kSmCount = 148;                 // B200
constexpr size_t kSmemPerSm = 227 * 1024;     // usable by CTAs; each CTA also reserves 1 KiB

// Grid size (CTAs) for dealing `units` 16-row units round-robin, or 0 to keep one 128-row tile per CTA.
// `ctas` tile CTAs of `smem` bytes, at most `max_per_sm` of them resident per SM by registers.
// Dealing pays when the tile CTAs fit the GPU at once but not evenly: some SMs would hold one CTA more
// than others and the launch lasts as long as those.  With r CTAs on every SM and the units dealt over
// all of them, an SM carries about units / 148 busy warps instead of 8 * ceil(ctas / 148).
inline int balanced_grid(long ctas, size_t smem, int max_per_sm, int mode) {
    if (mode == 2 || ctas <= 0) return 0;
    const int r = (int)((ctas + kSmCount - 1) / kSmCount);
    const long grid = (long)r * kSmCount;
    if (grid > 65535) return 0;
    if (mode == 1) return (int)grid;
    const int per_sm = (int)std::min<size_t>((size_t)max_per_sm, kSmemPerSm / (smem + 1024));
    if (ctas <= kSmCount || r > per_sm) return 0;   // fewer tiles than SMs, or more than one wave
    const long units = ctas * 8;
    const long dealt_max = (long)r * ((units + grid - 1) / grid);
    return dealt_max < 8L * r ? (int)grid : 0;
}

template <int NT, bool DUAL, int PRO, int UG, int KW>
int launch_mma(cudaStream_t stream, GemmParams& p) {
    constexpr int MT = 8 * NT;
    constexpr int RS = 16 * UG + 4;
    constexpr int SUB = 8 / UG;
    // Split K across a cluster only when the row tiles alone leave most SMs idle and every
    // K-warp still keeps at least two super-chunks.
    int ksplit = 1;
    if (g_force_ksplit > 0) {
        ksplit = g_force_ksplit;
    } else {
        const int ctas = (DUAL ? 2 : 1) * nvk::ceil_div(p.N, kRowsPerCta) * SUB;
        while (ksplit < 8 && ctas * ksplit < 148 && nvk::ceil_div(p.nsc, ksplit * 2) >= 2 * KW) ksplit *= 2;
    }
    p.tiles_per_arm = nvk::ceil_div(p.N, kRowsPerCta) * SUB;
    // phase length: keep the staged activations near 48 KiB
    int ph_cap = (48 * 1024) / (max(p.M, 1) * 512);
    ph_cap = max(KW, (ph_cap / KW) * KW);
    p.spc = nvk::ceil_div(p.nsc, ksplit);
    p.ph = min(ph_cap, nvk::ceil_div(p.spc, KW) * KW);
    p.x_stride = p.ph * 512 + 64;
    const size_t smem_x = (size_t)p.M * p.x_stride;
    const size_t smem_red = (size_t)(KW + 1) * MT * RS * sizeof(float);
    p.ring_off = (int)((max(smem_x, smem_red) + 127) / 128 * 128);
    const size_t smem = (size_t)p.ring_off + (size_t)UG * KW * kDepth * kSlotBytes;
    static nvk::SmemOptin optin;
    auto* kern = w4a16_mma_kernel<NT, DUAL, PRO, UG, KW>;
    if (int rc = optin.ensure((const void*)kern, smem)) return rc;
    size_t ctas = (size_t)(DUAL ? 2 : 1) * p.tiles_per_arm;
    if (ctas > 65535) return NVK_ERR_GRID_AXIS;
    p.bal_ctas = 0;
    if (UG == 8 && KW == 1 && ksplit == 1) {
        p.bal_ctas = balanced_grid((long)ctas, smem, kTileCtasPerSm<NT>, g_balance);
        if (p.bal_ctas > 0) ctas = (size_t)p.bal_ctas;
    }

    nvk::Launch l;
    l.grid = dim3((unsigned)ksplit, (unsigned)ctas, 1);
    l.block = dim3(32 * UG * KW, 1, 1);
    l.smem = smem;
    l.stream = stream;
    l.cluster_x = (unsigned)ksplit;
    l.pdl = true;
    return nvk::launch(l, kern, p);
}

template <int NT, bool DUAL, int PRO>
int launch_by_rows(cudaStream_t stream, GemmParams& p, int ug) {
    if (ug == 1) return launch_mma<NT, DUAL, PRO, 1, 8>(stream, p);
    if (ug == 2) return launch_mma<NT, DUAL, PRO, 2, 4>(stream, p);
    if (ug == 4) return launch_mma<NT, DUAL, PRO, 4, 2>(stream, p);
    return launch_mma<NT, DUAL, PRO, 8, 1>(stream, p);
}

template <bool DUAL, int PRO>
int dispatch_mma(cudaStream_t stream, GemmParams& p) {
    // One CTA owns a whole 128-row scale tile and each warp sums all of its K slice in order, for
    // every M: the order in which K is summed depends on (N, K) only, so a row gives the same bits
    // whatever the batch size.  Smaller CTAs (more K-warps) exist for tuning and are tested.
    int ug = 8;
    if (g_force_ug == 1 || g_force_ug == 2 || g_force_ug == 4 || g_force_ug == 8) ug = g_force_ug;
    if (p.M <= 8) return launch_by_rows<1, DUAL, PRO>(stream, p, ug);
    if (p.M <= 16) return launch_by_rows<2, DUAL, PRO>(stream, p, ug < 2 ? 2 : ug);
    if (p.M <= 32) return launch_mma<4, DUAL, PRO, 8, 1>(stream, p);
    return launch_mma<8, DUAL, PRO, 8, 1>(stream, p);
}

bool aligned16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; }

size_t linear_ws_bytes(int M, int K) { return 256 + (size_t)nvk::ceil_div(K, kSuper) * (size_t)M * 512; }

template <int NT, bool DUAL>
int launch_mma_ws(cudaStream_t stream, GemmParams& p, const uint8_t* ws) {
    constexpr int MT = 8 * NT, RS = 128 + 4;
    int ksplit = 1;
    if (g_force_ksplit > 0) {
        ksplit = g_force_ksplit;
    } else {
        const int ctas = (DUAL ? 2 : 1) * nvk::ceil_div(p.N, kRowsPerCta);
        while (ksplit < 8 && ctas * ksplit < 148 && nvk::ceil_div(p.nsc, ksplit * 2) >= 2) ksplit *= 2;
    }
    p.tiles_per_arm = nvk::ceil_div(p.N, kRowsPerCta);
    p.spc = nvk::ceil_div(p.nsc, ksplit);
    p.ph = p.spc;
    p.x_stride = 576;
    const size_t smem_x = (size_t)kDepth * p.M * 576;
    const size_t smem_red = (size_t)2 * MT * RS * sizeof(float);
    p.ring_off = (int)((max(smem_x, smem_red) + 127) / 128 * 128);
    const size_t smem = (size_t)p.ring_off + (size_t)8 * kDepth * kSlotBytes;
    static nvk::SmemOptin optin;
    auto* kern = w4a16_mma_ws_kernel<NT, DUAL>;
    if (int rc = optin.ensure((const void*)kern, smem)) return rc;
    const size_t ctas = (size_t)(DUAL ? 2 : 1) * p.tiles_per_arm;
    if (ctas > 65535) return NVK_ERR_GRID_AXIS;
    nvk::Launch l;
    l.grid = dim3((unsigned)ksplit, (unsigned)ctas, 1);
    l.block = dim3(256, 1, 1);
    l.smem = smem;
    l.stream = stream;
    l.cluster_x = (unsigned)ksplit;
    l.pdl = true;
    return nvk::launch(l, kern, p, ws);
}

int launch_prepare(cudaStream_t stream, const uint16_t* x, const uint16_t* x2, uint8_t* ws, int M, int K, int nsc) {
    const nvk::Launch l = nvk::launch_1d(stream, (unsigned)M, 256, 0, true);
    if (x2) return nvk::launch(l, x_prepare_kernel<1>, x, x2, ws, M, K, nsc);
    return nvk::launch(l, x_prepare_kernel<0>, x, x2, ws, M, K, nsc);
}

template <bool DUAL, int PRO>
int launch_grouped(cudaStream_t stream, GemmParams& p, const GroupedParams& g, int E) {
    p.M = 8;
    p.tiles_per_arm = nvk::ceil_div(p.N, kRowsPerCta);
    const size_t ctas = (size_t)(DUAL ? 2 : 1) * p.tiles_per_arm;
    if (ctas > 65535 || E > 65535) return NVK_ERR_GRID_AXIS;
    // K split over a cluster by the rule of the dense launches, applied to ONE expert's row tiles: a
    // decode step may route to a single expert, and a rule that looked at the number of routed experts
    // or tokens would make a slot's bits depend on the rest of the batch.
    int ksplit = g_force_ksplit > 0 ? g_force_ksplit : tile_ksplit((int)ctas, p.nsc);
    const size_t smem = tile_layout_rows128(p, 8, 8, ksplit);
    static nvk::SmemOptin optin;
    auto* kern = w4a16_grouped_kernel<DUAL, PRO>;
    if (int rc = optin.ensure((const void*)kern, smem)) return rc;
    nvk::Launch l;
    // with a list of active experts the grid covers only as many experts as there are slots
    const int grid_z = g.active != nullptr ? max(1, min(E, g.n_slots)) : E;
    l.grid = dim3((unsigned)ksplit, (unsigned)ctas, (unsigned)grid_z);
    l.block = dim3(256, 1, 1);
    l.smem = smem;
    l.stream = stream;
    l.cluster_x = (unsigned)ksplit;
    l.pdl = true;
    return nvk::launch(l, kern, p, g);
}

// Common entry: validates, then picks the tensor-core route or the generic one.
int w4a16_linear(cudaStream_t stream, const uint8_t* wq_a, const uint8_t* sc_a, const uint8_t* wq_b,
                 const uint8_t* sc_b, const uint16_t* x, const uint16_t* x2, uint16_t* y_a, uint16_t* y_b,
                 float alpha_a, float alpha_b, int M, int N, int K, int pro, int max_m) {
    if (M <= 0 || M > max_m) return NVK_ERR_SHAPE;
    if ((K & 15) != 0) return NVK_ERR_SHAPE;
    if (nvk::any_null(wq_a, sc_a, x, y_a) || (pro && x2 == nullptr)) return NVK_ERR_ARG;
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
    const nvk::Launch l = nvk::launch_1d(stream, (unsigned)nvk::ceil_div(total, 8), 256);
    return pro ? nvk::launch(l, w4a16_rowwarp_kernel<1>, p) : nvk::launch(l, w4a16_rowwarp_kernel<0>, p);
}

// ------------------------------------------------------------------------------------------
// W4A4 at M = 1: an NVFP4 activation row against NVFP4 weights.  The activation is dequantized
// exactly while it is staged (tile prologues 2 and 3), so this is the W4A16 tile with another
// prologue: weights stream once with 16-byte copies, a 128-row x k-tile scale tile is read as
// contiguous bytes, and the sum over K is taken in the tile's fixed order (bit-stable run to run).
int w4a4_gemv(cudaStream_t stream, const uint8_t* W_packed, const uint8_t* W_scales, const uint8_t* x_packed,
              const uint8_t* x_scales, uint16_t* y, float alpha, int N, int K) {
    GemmParams p = {};
    p.wq[0] = W_packed;
    p.sc[0] = W_scales;
    p.x = reinterpret_cast<const uint16_t*>(x_packed);
    p.x2 = reinterpret_cast<const uint16_t*>(x_scales);
    p.y[0] = y;
    p.alpha[0] = alpha;
    p.M = 1; p.N = N; p.K = K;
    p.tiles_per_arm = nvk::ceil_div(N, kRowsPerCta);
    p.k_tiles = nvk::ceil_div(K, 64);
    p.nsc = nvk::ceil_div(K, kSuper);
    const bool fast = (K & 31) == 0 && aligned16(W_packed) && aligned16(W_scales) &&
                      (reinterpret_cast<uintptr_t>(x_packed) & 3u) == 0 && p.tiles_per_arm <= 65535;
    if (fast) return launch_mma<1, false, 3, 8, 1>(stream, p);
    return nvk::launch(nvk::launch_1d(stream, (unsigned)nvk::ceil_div(N, 8), 256), w4a16_rowwarp_kernel<3>, p);
}

// Grouped form: group g is one (token, expert) pair -- expert ids[g], activation = row 0 of the
// g-th activation tile, output row g.  A group whose id is outside [0, num_experts) gets a zero row.
struct W4a4GroupArgs {
    const uint8_t* a_packed;
    const uint8_t* a_scales;
    const float* alphas;
    const int32_t* ids;
    int num_experts;
    size_t a_group_bytes;      // packed bytes between the activation tiles of consecutive groups
    size_t a_sf_group_bytes;   // scale bytes between them
    size_t w_stride, sc_stride;
    long long d_group_stride;  // output elements between groups
};

__global__ void __launch_bounds__(256, 3) w4a4_m1_grouped_kernel(const GemmParams p, const W4a4GroupArgs g) {
    // ids and activations come from the kernels just before this one.
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const int grp = blockIdx.z, tile = blockIdx.y;
    const int e = g.ids[grp];
    uint16_t* y = p.y[0] + (size_t)grp * (size_t)g.d_group_stride;
    if (e < 0 || e >= g.num_experts) {   // the same for every CTA of a K-split cluster
        if (blockIdx.x == 0)
            for (int r = threadIdx.x; r < kRowsPerCta; r += 256)
                if (tile * kRowsPerCta + r < p.N) y[tile * kRowsPerCta + r] = 0;
        return;
    }
    TileView t = {};
    t.wq = p.wq[0] + (size_t)e * g.w_stride;
    t.sc = p.sc[0] + (size_t)e * g.sc_stride;
    t.x = reinterpret_cast<const uint16_t*>(g.a_packed + (size_t)grp * g.a_group_bytes);
    t.x2 = reinterpret_cast<const uint16_t*>(g.a_scales + (size_t)grp * g.a_sf_group_bytes);
    t.xrows = nullptr;
    t.x_rows = 0;
    t.status = nullptr;
    t.y = y;
    t.alpha = g.alphas[e];
    t.xrow0 = 0;
    t.M = 1;
    t.sub = tile;
    t.pdl = false;
    t.ws = nullptr;
    w4a16_tile<1, 2, 8, 1>(p, t);
}

// Shapes the tile does not take (K % 32 != 0, unaligned banks): one warp per (row, group), fp32 FMAs.
__global__ void __launch_bounds__(256) w4a4_m1_grouped_rowwarp_kernel(const GemmParams p, const W4a4GroupArgs g) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int grp = blockIdx.y;
    if (n >= p.N) return;
    uint16_t* y = p.y[0] + (size_t)grp * (size_t)g.d_group_stride;
    const int e = g.ids[grp];
    if (e < 0 || e >= g.num_experts) {
        if (lane == 0) y[n] = 0;
        return;
    }
    const int kb_total = p.K >> 4;
    const uint8_t* wrow = p.wq[0] + (size_t)e * g.w_stride + (size_t)n * (p.K >> 1);
    const uint8_t* wsc = p.sc[0] + (size_t)e * g.sc_stride;
    const uint8_t* xa = g.a_packed + (size_t)grp * g.a_group_bytes;
    const uint8_t* xs = g.a_scales + (size_t)grp * g.a_sf_group_bytes;
    float acc = 0.f;
    for (int kb = lane; kb < kb_total; kb += 32) {
        const float ws = nvk::ue4m3_to_f32(wsc[nvk::swz_offset(n, kb, kb_total)]);
        const float as = nvk::ue4m3_to_f32(xs[(size_t)(kb >> 2) * 512 + (kb & 3)]);
        float bd = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint32_t w2 = nvk::ptx::e2m1x2_to_f16x2(wrow[kb * 8 + i]), a2 = nvk::ptx::e2m1x2_to_f16x2(xa[kb * 8 + i]);
            const float2 wf = __half22float2(*reinterpret_cast<__half2*>(&w2));
            const float2 af = __half22float2(*reinterpret_cast<__half2*>(&a2));
            bd = fmaf(wf.x, af.x, bd);   // exact: multiples of 1/4, at most 16 * 36
            bd = fmaf(wf.y, af.y, bd);
        }
        acc = fmaf(ws * as, bd, acc);
    }
    acc = nvk::warp_sum(acc);
    if (lane == 0) y[n] = nvk::f32_to_bf16_bits(acc * g.alphas[e]);
}

int w4a4_grouped(cudaStream_t stream, GemmParams& p, const W4a4GroupArgs& g, int num_groups, bool fast) {
    if (!fast) {
        nvk::Launch l;
        l.grid = dim3((unsigned)nvk::ceil_div(p.N, 8), (unsigned)num_groups, 1);
        l.block = dim3(256, 1, 1);
        l.stream = stream;
        return nvk::launch(l, w4a4_m1_grouped_rowwarp_kernel, p, g);
    }
    constexpr int MT = 8, RS = 128 + 4, KW = 1;
    p.M = 1;
    p.tiles_per_arm = nvk::ceil_div(p.N, kRowsPerCta);
    int ksplit = 1;
    if (g_force_ksplit > 0) {
        ksplit = g_force_ksplit;
    } else {
        const long long ctas = (long long)p.tiles_per_arm * num_groups;
        while (ksplit < 8 && ctas * ksplit < 148 && nvk::ceil_div(p.nsc, ksplit * 2) >= 2) ksplit *= 2;
    }
    p.spc = nvk::ceil_div(p.nsc, ksplit);
    p.ph = min(96, p.spc);
    p.x_stride = p.ph * 512 + 64;
    const size_t smem_x = (size_t)p.x_stride;
    const size_t smem_red = (size_t)(KW + 1) * MT * RS * sizeof(float);
    p.ring_off = (int)((max(smem_x, smem_red) + 127) / 128 * 128);
    const size_t smem = (size_t)p.ring_off + (size_t)8 * kDepth * kSlotBytes;
    static nvk::SmemOptin optin;
    if (int rc = optin.ensure((const void*)w4a4_m1_grouped_kernel, smem)) return rc;
    if (p.tiles_per_arm > 65535 || num_groups > 65535) return NVK_ERR_GRID_AXIS;
    nvk::Launch l;
    l.grid = dim3((unsigned)ksplit, (unsigned)p.tiles_per_arm, (unsigned)num_groups);
    l.block = dim3(256, 1, 1);
    l.smem = smem;
    l.stream = stream;
    l.cluster_x = (unsigned)ksplit;
    l.pdl = true;
    return nvk::launch(l, w4a4_m1_grouped_kernel, p, g);
}

}  // namespace

// ------------------------------------------------------------------------------------------
// C ABI.  Reference-named symbols keep the reference's argument order and refusals.
extern "C" {

int nvk_b200_set_pdl(int enabled) {
    nvk::g_pdl_enabled = enabled ? 1 : 0;
    return 0;
}

int nvk_b200_set_row_balance(int mode) {
    if (mode < 0 || mode > 2) return NVK_ERR_ARG;
    g_balance = mode;
    return 0;
}

int nvk_b200_row_balance_grid(int tile_ctas, size_t smem_bytes, int max_ctas_per_sm) {
    return balanced_grid((long)tile_ctas, smem_bytes, max_ctas_per_sm, 0);
}

int nvk_b200_set_tuning(int force_ksplit, int force_rows_per_cta) {
    if (force_ksplit != 0 && force_ksplit != 1 && force_ksplit != 2 && force_ksplit != 4 && force_ksplit != 8)
        return NVK_ERR_ARG;
    if (force_rows_per_cta != 0 && force_rows_per_cta != 16 && force_rows_per_cta != 32 && force_rows_per_cta != 64 &&
        force_rows_per_cta != 128)
        return NVK_ERR_ARG;
    g_force_ksplit = force_ksplit;
    g_force_ug = force_rows_per_cta / 16;
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

// Grouped-expert W4A16 linear for routed MoE tokens (no counterpart in the reference, whose grouped
// decode path quantizes activations to NVFP4 and gives every (token, expert) pair its own tile).
// Expert e works on the sorted slots [expert_offsets[e], expert_offsets[e + 1]); slot s reads row
// row_index[s] of x (row s when row_index is NULL) and writes row s of the outputs.  With
// `active_experts` / `n_active` (device; as nvk_b200_moe_route_permute writes them) the launch covers
// min(num_experts, num_slots) experts instead of all of them -- at batch 1 with top-8 routing that is 8
// CTAs per row tile instead of 128.  `num_slots` is
// the number of rows the outputs (and row_index) hold, `x_rows` the number of rows of x: offsets and
// row indices outside them are never followed -- the slots are skipped or read as zeros and, when
// `status` (one device int, zeroed by the caller) is given, bit 0 (offset) or bit 1 (row) is set in it.
int nvk_b200_moe_grouped_w4a16(void* stream, const uint8_t* wq_bank_a, const uint8_t* sc_bank_a,
                               const uint8_t* wq_bank_b, const uint8_t* sc_bank_b, const float* alphas_a,
                               const float* alphas_b, const uint16_t* x, const uint16_t* x2,
                               const int32_t* row_index, const int32_t* expert_offsets,
                               const int32_t* active_experts, const int32_t* n_active, uint16_t* y_a,
                               uint16_t* y_b, int num_experts, int N, int K, int num_slots, int x_rows,
                               int* status) {
    if (num_experts <= 0 || N <= 0 || K <= 0) return 0;
    if (num_slots < 0 || x_rows < 0) return NVK_ERR_ARG;
    if ((active_experts == nullptr) != (n_active == nullptr)) return NVK_ERR_ARG;
    if ((K & 31) != 0) return NVK_ERR_SHAPE;
    if ((wq_bank_b == nullptr) != (y_b == nullptr) || (wq_bank_b == nullptr) != (sc_bank_b == nullptr) ||
        (wq_bank_b == nullptr) != (alphas_b == nullptr))
        return NVK_ERR_SHAPE;
    const size_t w_stride = (size_t)N * (K >> 1);
    const size_t sc_stride = (size_t)nvk::ceil_div(N, 128) * 128 * (size_t)nvk::ceil_div(K, 64) * 4;
    if ((w_stride & 15) != 0 || !aligned16(wq_bank_a) || !aligned16(sc_bank_a) || !aligned16(x) ||
        (wq_bank_b && (!aligned16(wq_bank_b) || !aligned16(sc_bank_b))) || (x2 && !aligned16(x2)))
        return NVK_ERR_ARG;
    if (nvk::any_null(wq_bank_a, sc_bank_a, alphas_a, x, expert_offsets, y_a)) return NVK_ERR_ARG;
    GemmParams p = {};
    p.wq[0] = wq_bank_a; p.wq[1] = wq_bank_b;
    p.sc[0] = sc_bank_a; p.sc[1] = sc_bank_b;
    p.x = x; p.x2 = x2;
    p.y[0] = y_a; p.y[1] = y_b;
    p.N = N; p.K = K;
    p.k_tiles = nvk::ceil_div(K, 64);
    p.nsc = nvk::ceil_div(K, kSuper);
    GroupedParams g = {};
    g.alphas[0] = alphas_a; g.alphas[1] = alphas_b;
    g.offsets = expert_offsets;
    g.xrows = row_index;
    g.w_stride = w_stride;
    g.sc_stride = sc_stride;
    g.active = active_experts;
    g.n_active = n_active;
    g.n_experts = num_experts;
    g.n_slots = num_slots;
    g.x_rows = row_index ? x_rows : num_slots;
    g.status = status;
    cudaStream_t s = (cudaStream_t)stream;
    const bool dual = wq_bank_b != nullptr;
    if (dual) return x2 ? launch_grouped<true, 1>(s, p, g, num_experts) : launch_grouped<true, 0>(s, p, g, num_experts);
    return x2 ? launch_grouped<false, 1>(s, p, g, num_experts) : launch_grouped<false, 0>(s, p, g, num_experts);
}

// Workspace the caller provides to nvk_b200_linear_nvfp4_w4a16_ws for M tokens of K values.
size_t nvk_b200_linear_workspace_bytes(int M, int K) {
    if (M <= 0 || K <= 0) return 0;
    return linear_ws_bytes(M, K);
}

// The W4A16 linear with a caller-supplied workspace (device memory, 16-byte aligned, at least
// nvk_b200_linear_workspace_bytes(M, K) bytes, private to this call until it completes).  For M >= 3
// the activations are converted once into the workspace by a small kernel and every CTA of the GEMM
// streams them from there; without a workspace (NULL) or for M <= 2 this is
// nvk_b200_linear_nvfp4_w4a16.  Results are bit-identical either way.
int nvk_b200_linear_nvfp4_w4a16_ws(void* stream, const uint8_t* wq_a, const uint8_t* sc_a, const uint8_t* wq_b,
                                   const uint8_t* sc_b, const uint16_t* x, const uint16_t* x2, uint16_t* y_a,
                                   uint16_t* y_b, float alpha_a, float alpha_b, int M, int N, int K,
                                   void* workspace, size_t workspace_bytes) {
    if (N <= 0 || K <= 0) return 0;
    if ((wq_b == nullptr) != (y_b == nullptr)) return NVK_ERR_SHAPE;
    if ((wq_b == nullptr) != (sc_b == nullptr)) return NVK_ERR_SHAPE;
    if (M <= 0 || M > 64 || (K & 15) != 0) return NVK_ERR_SHAPE;
    const bool dual = wq_b != nullptr;
    const bool fast = (K & 31) == 0 && aligned16(wq_a) && aligned16(sc_a) && aligned16(x) &&
                      (!dual || (aligned16(wq_b) && aligned16(sc_b))) && (!x2 || aligned16(x2));
    // The extra launch pays off once the per-CTA conversion it replaces is large: many tokens, or a
    // few tokens against a big matrix.  Both routes give the same bits, so the switch is invisible.
    if (workspace != nullptr && (!aligned16(workspace) || workspace_bytes < linear_ws_bytes(M, K))) return NVK_ERR_ARG;
    const double elems = (double)N * (double)K * (dual ? 2.0 : 1.0);
    const bool worth = (M >= 9 && elems >= 32e6) || (M >= 3 && elems >= 100e6);
    if (workspace == nullptr || !worth || !fast)
        return w4a16_linear((cudaStream_t)stream, wq_a, sc_a, wq_b, sc_b, x, x2, y_a, y_b, alpha_a, alpha_b, M, N, K,
                            x2 ? 1 : 0, 64);
    if (nvk::any_null(wq_a, sc_a, x, y_a)) return NVK_ERR_ARG;
    GemmParams p = {};
    p.wq[0] = wq_a; p.wq[1] = wq_b;
    p.sc[0] = sc_a; p.sc[1] = sc_b;
    p.y[0] = y_a; p.y[1] = y_b;
    p.alpha[0] = alpha_a; p.alpha[1] = alpha_b;
    p.M = M; p.N = N; p.K = K;
    p.k_tiles = nvk::ceil_div(K, 64);
    p.nsc = nvk::ceil_div(K, kSuper);
    cudaStream_t s = (cudaStream_t)stream;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    if (int rc = launch_prepare(s, x, x2, ws, M, K, p.nsc)) return rc;
    if (dual) {
        if (M <= 8) return launch_mma_ws<1, true>(s, p, ws);
        if (M <= 16) return launch_mma_ws<2, true>(s, p, ws);
        if (M <= 32) return launch_mma_ws<4, true>(s, p, ws);
        return launch_mma_ws<8, true>(s, p, ws);
    }
    if (M <= 8) return launch_mma_ws<1, false>(s, p, ws);
    if (M <= 16) return launch_mma_ws<2, false>(s, p, ws);
    if (M <= 32) return launch_mma_ws<4, false>(s, p, ws);
    return launch_mma_ws<8, false>(s, p, ws);
}

// W4A4 at M = 1 (the reference's test/shader-mirror pair with the flat row quantizer): packed e2m1
// activation row with a flat [K/16] ue4m3 scale array against swizzled NVFP4 weights.
int nv_kernels_nvfp4_gemv_bf16(void* stream, const uint8_t* W_packed, const uint8_t* W_scales, const uint8_t* x_packed,
                               const uint8_t* x_scales, uint16_t* y, float alpha, int N, int K) {
    if (N <= 0 || K <= 0) return 0;
    if ((K & 15) != 0) return NVK_ERR_SHAPE;
    if (nvk::any_null(W_packed, W_scales, x_packed, x_scales, y)) return NVK_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(W_packed) & 7) != 0 || (reinterpret_cast<uintptr_t>(x_packed) & 7) != 0)
        return NVK_ERR_ARG;
    return w4a4_gemv((cudaStream_t)stream, W_packed, W_scales, x_packed, x_scales, y, alpha, N, K);
}

// Grouped M = 1 expert GEMV with NVFP4 activations: d[g, :] = bf16(alphas[e] * W_e a_g), e = ids[g],
// a_g = row 0 of the g-th activation tile (tiles are a_tile_stride_rows rows apart).
int nv_kernels_moe_grouped_fp4_gemv_m1_bf16(void* stream, const uint8_t* a_packed, const uint8_t* a_scales,
                                            const uint8_t* b_packed, const uint8_t* b_scales, const float* alphas,
                                            uint16_t* d_bf16, const int32_t* group_expert_ids, int num_groups,
                                            int num_experts_total, int n, int k, int a_tile_stride_rows,
                                            long long d_group_stride_elems) {
    if (num_groups <= 0 || num_experts_total <= 0 || n <= 0 || k <= 0) return NVK_ERR_SHAPE;
    if ((k & 15) != 0) return NVK_ERR_SHAPE;
    if (a_tile_stride_rows <= 0 || (a_tile_stride_rows & 127) != 0) return NVK_ERR_SHAPE;
    if (d_group_stride_elems < (long long)n) return NVK_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(a_packed) & 7) != 0 || (reinterpret_cast<uintptr_t>(b_packed) & 7) != 0)
        return NVK_ERR_ARG;
    if (num_groups > 65535) return NVK_ERR_GRID_AXIS;
    if (nvk::any_null(a_packed, a_scales, b_packed, b_scales, alphas, d_bf16, group_expert_ids)) return NVK_ERR_ARG;
    GemmParams p = {};
    p.wq[0] = b_packed;
    p.sc[0] = b_scales;
    p.y[0] = d_bf16;
    p.N = n; p.K = k;
    p.k_tiles = nvk::ceil_div(k, 64);
    p.nsc = nvk::ceil_div(k, kSuper);
    W4a4GroupArgs g = {};
    g.a_packed = a_packed; g.a_scales = a_scales; g.alphas = alphas; g.ids = group_expert_ids;
    g.num_experts = num_experts_total;
    g.a_group_bytes = (size_t)a_tile_stride_rows * (size_t)(k >> 1);
    g.a_sf_group_bytes = (size_t)(a_tile_stride_rows / 128) * (size_t)p.k_tiles * 512;
    g.w_stride = (size_t)n * (size_t)(k >> 1);
    g.sc_stride = (size_t)nvk::ceil_div(n, 128) * 128 * (size_t)p.k_tiles * 4;
    g.d_group_stride = d_group_stride_elems;
    const bool fast = (k & 31) == 0 && aligned16(b_packed) && aligned16(b_scales) && (g.w_stride & 15) == 0;
    return w4a4_grouped((cudaStream_t)stream, p, g, num_groups, fast);
}

}  // extern "C"
