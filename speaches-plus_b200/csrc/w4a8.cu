// W4A8 decode MLP family: NVFP4 weights against int8 activation rows (one dequant scale per row), and
// the small kernels that produce those rows.
//
//   y[m, n] = bf16( fma( sum_k e2m1(W[n,k]) * ue4m3(S[n,k/16]) * q[m,k],  alpha * scale[m],  residual[m,n] ) )
//
// The GEMVs are the W4A16 tile with two more prologues: the int8 row is staged as exact small
// integers (tile prologue 4), or a bf16 row is quantized to int8 while it is staged, its scale taken
// from partial maxima a previous kernel left (prologue 5).  Weights stream once with 16-byte copies,
// scale tiles are read as contiguous bytes, the contraction runs on the tensor cores with fp32
// accumulation, and the row scale, alpha and the residual meet in one fused multiply-add before the
// single rounding to bf16.  The "rstd emit" form also leaves 1/rms of the new residual row for the
// next RMSNorm (see emit_rstd in w4a16_tile.cuh).
#include "w4a16_tile.cuh"

namespace {

struct EpiArgs {
    const uint16_t* residual;
    const float* row_scale;
    float* rstd_pack;
    float rstd_eps;
    unsigned rstd_blocks;
    const float* absmax_partials;
    int n_partials;
};

template <int NT, bool DUAL, int PRO>
__global__ void __launch_bounds__(256, kTileCtasPerSm<NT>) w4a8_kernel(const GemmParams p, const EpiArgs e) {
    const int tile = blockIdx.y;
    const int arm = DUAL ? (tile >= p.tiles_per_arm ? 1 : 0) : 0;
    TileView t = {};
    t.wq = arm_pick(p.wq, arm);
    t.sc = arm_pick(p.sc, arm);
    t.x = p.x;
    t.y = arm_pick(p.y, arm);
    t.alpha = arm_pick(p.alpha, arm);
    t.M = p.M;
    t.sub = tile - arm * p.tiles_per_arm;
    t.pdl = true;
    t.residual = e.residual;
    t.row_scale = e.row_scale;
    t.rstd_pack = e.rstd_pack;
    t.rstd_eps = e.rstd_eps;
    t.rstd_blocks = e.rstd_blocks;
    t.absmax_partials = e.absmax_partials;
    t.n_partials = e.n_partials;
    w4a16_tile<NT, PRO, 8, 1, false, LaunchHooks, 1>(p, t);
}

bool aligned16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; }

template <int NT, bool DUAL, int PRO>
int launch_w4a8(cudaStream_t stream, GemmParams& p, EpiArgs& e) {
    p.tiles_per_arm = nvk::ceil_div(p.N, kRowsPerCta);
    const int ctas = (DUAL ? 2 : 1) * p.tiles_per_arm;
    if (ctas > 65535) return NVK_ERR_GRID_AXIS;
    const int ksplit = tile_ksplit(ctas, p.nsc);
    const size_t smem = tile_layout_rows128(p, p.M, 8 * NT, ksplit);
    static nvk::SmemOptin optin;
    auto* kern = w4a8_kernel<NT, DUAL, PRO>;
    if (int rc = optin.ensure((const void*)kern, smem)) return rc;
    e.rstd_blocks = (unsigned)(ctas * ksplit);
    nvk::Launch l;
    l.grid = dim3((unsigned)ksplit, (unsigned)ctas, 1);
    l.block = dim3(256, 1, 1);
    l.smem = smem;
    l.stream = stream;
    l.cluster_x = (unsigned)ksplit;
    l.pdl = true;
    return nvk::launch(l, kern, p, e);
}

template <bool DUAL, int PRO>
int dispatch_w4a8(cudaStream_t stream, GemmParams& p, EpiArgs& e) {
    if (p.M <= 8) return launch_w4a8<1, DUAL, PRO>(stream, p, e);
    if (p.M <= 16) return launch_w4a8<2, DUAL, PRO>(stream, p, e);
    if (p.M <= 32) return launch_w4a8<4, DUAL, PRO>(stream, p, e);
    return launch_w4a8<8, DUAL, PRO>(stream, p, e);
}

// Rows of int8 activations against one or two matrices, in chunks of up to 64 rows.
int w4a8_linear(cudaStream_t stream, const uint8_t* wq_a, const uint8_t* sc_a, const uint8_t* wq_b, const uint8_t* sc_b,
                const int8_t* x_q8, const float* x_scales, const uint16_t* residual, uint16_t* y_a, uint16_t* y_b,
                float alpha_a, float alpha_b, int M, int N, int K, float* rstd_pack, float rstd_eps) {
    if (M <= 0 || N <= 0 || K <= 0 || (K & 31) != 0) return NVK_ERR_SHAPE;
    const bool dual = wq_b != nullptr;
    if (nvk::any_null(wq_a, sc_a, x_q8, x_scales, y_a) || (dual && nvk::any_null(sc_b, y_b))) return NVK_ERR_ARG;
    if (!aligned16(wq_a) || !aligned16(sc_a) || (reinterpret_cast<uintptr_t>(x_q8) & 7u) != 0 ||
        (dual && (!aligned16(wq_b) || !aligned16(sc_b))))
        return NVK_ERR_ARG;
    for (int m0 = 0; m0 < M; m0 += 64) {
        GemmParams p = {};
        p.wq[0] = wq_a; p.wq[1] = wq_b;
        p.sc[0] = sc_a; p.sc[1] = sc_b;
        p.x = reinterpret_cast<const uint16_t*>(x_q8 + (size_t)m0 * K);
        p.y[0] = y_a + (size_t)m0 * N;
        p.y[1] = y_b ? y_b + (size_t)m0 * N : nullptr;
        p.alpha[0] = alpha_a; p.alpha[1] = alpha_b;
        p.M = M - m0 < 64 ? M - m0 : 64;
        p.N = N; p.K = K;
        p.k_tiles = nvk::ceil_div(K, 64);
        p.nsc = nvk::ceil_div(K, kSuper);
        EpiArgs e = {};
        e.residual = residual ? residual + (size_t)m0 * N : nullptr;
        e.row_scale = x_scales + m0;
        e.rstd_pack = rstd_pack;
        e.rstd_eps = rstd_eps;
        const int rc = dual ? dispatch_w4a8<true, 4>(stream, p, e) : dispatch_w4a8<false, 4>(stream, p, e);
        if (rc != 0) return rc;
    }
    return 0;
}

// ---- activation producers ----------------------------------------------------------------------------
constexpr int kSplitThreads = 256;
constexpr int kSplitMaxBlocks = 128;   // partial maxima per row, at most

__host__ __device__ inline int split_blocks(int K) {
    const int b = (K + kSplitThreads - 1) / kSplitThreads;
    return b < kSplitMaxBlocks ? b : kSplitMaxBlocks;
}

__device__ __forceinline__ float silu_mul_bf16(uint16_t g_bits, uint16_t u_bits, uint16_t& out_bits) {
    const float g = nvk::bf16_bits_to_f32(g_bits), u = nvk::bf16_bits_to_f32(u_bits);
    out_bits = nvk::f32_to_bf16_bits((g / (1.0f + expf(-g))) * u);
    return fabsf(nvk::bf16_bits_to_f32(out_bits));
}

__device__ __forceinline__ int8_t quant_i8(uint16_t v_bits, float inv) {
    return (int8_t)max(-127, min(127, __float2int_rn(nvk::bf16_bits_to_f32(v_bits) * inv)));
}

// Block-wide maximum of non-negative values (bit patterns order like the values).  All threads call.
__device__ __forceinline__ float block_max_nonneg(float v, uint32_t* s_slot) {
    if (threadIdx.x == 0) *s_slot = 0u;
    __syncthreads();
    const uint32_t m = __reduce_max_sync(0xffffffffu, __float_as_uint(v));
    if ((threadIdx.x & 31) == 0 && m) atomicMax(s_slot, m);
    __syncthreads();
    return __uint_as_float(*s_slot);
}

// Pass 1 (grid: blocks x rows): act = bf16(SiLU(gate) * up) staged in global memory, one partial
// maximum per block.
__global__ void __launch_bounds__(kSplitThreads) silu_stage_absmax_kernel(const uint16_t* __restrict__ gate,
                                                                          const uint16_t* __restrict__ up,
                                                                          uint16_t* __restrict__ staged,
                                                                          float* __restrict__ partial_absmax, int K) {
    __shared__ uint32_t s_max;
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const size_t row = blockIdx.y;
    float amax = 0.f;
    for (int i = blockIdx.x * kSplitThreads + threadIdx.x; i < K; i += gridDim.x * kSplitThreads) {
        uint16_t a;
        amax = fmaxf(amax, silu_mul_bf16(gate[row * K + i], up[row * K + i], a));
        staged[row * K + i] = a;
    }
    const float bmax = block_max_nonneg(amax, &s_max);
    if (threadIdx.x == 0) partial_absmax[row * gridDim.x + blockIdx.x] = bmax;
}

// Pass 2 (same grid): scale = max(partials) / 127; q = clamp(rn(act / scale), +-127).
__global__ void __launch_bounds__(kSplitThreads) rowquant_from_staged_kernel(const uint16_t* __restrict__ staged,
                                                                             const float* __restrict__ partial_absmax,
                                                                             int num_partials, int8_t* __restrict__ q8,
                                                                             float* __restrict__ scales, int K) {
    __shared__ uint32_t s_max;
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const size_t row = blockIdx.y;
    float a = 0.f;
    for (int i = threadIdx.x; i < num_partials; i += kSplitThreads) a = fmaxf(a, partial_absmax[row * num_partials + i]);
    const float scale = block_max_nonneg(a, &s_max) / 127.0f;
    const float inv = scale > 0.f ? 1.0f / scale : 0.f;
    if (blockIdx.x == 0 && threadIdx.x == 0) scales[row] = scale;
    for (int i = blockIdx.x * kSplitThreads + threadIdx.x; i < K; i += gridDim.x * kSplitThreads)
        q8[row * K + i] = quant_i8(staged[row * K + i], inv);
}

// One row, one CTA: act staged in shared memory between the two passes.
__global__ void __launch_bounds__(1024) silu_rowquant_m1_kernel(const uint16_t* __restrict__ gate,
                                                                const uint16_t* __restrict__ up, int8_t* __restrict__ q8,
                                                                float* __restrict__ scale_out, int K) {
    NVK_DYN_SMEM_AS(uint16_t, s_act);
    __shared__ uint32_t s_max;
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    float amax = 0.f;
    for (int i = threadIdx.x; i < K; i += blockDim.x) {
        uint16_t a;
        amax = fmaxf(amax, silu_mul_bf16(gate[i], up[i], a));
        s_act[i] = a;
    }
    const float scale = block_max_nonneg(amax, &s_max) / 127.0f;
    const float inv = scale > 0.f ? 1.0f / scale : 0.f;
    if (threadIdx.x == 0) scale_out[0] = scale;
    for (int i = threadIdx.x; i < K; i += blockDim.x) q8[i] = quant_i8(s_act[i], inv);
}

// Sum of a float over the CTA in a fixed order (lanes by shuffle, warps in order).  All threads call.
__device__ __forceinline__ float block_sum(float v, float* s_warp /*[32]*/) {
    v = nvk::warp_sum(v);
    if ((threadIdx.x & 31) == 0) s_warp[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_warp[w];
    __syncthreads();
    return tot;
}

// s = x + res_in (stored as bf16 to res_out, squared unrounded); v = bf16(bf16(s) * rstd * w).
// Q8: v is quantized to an int8 row (one row, staged in shared memory); else v is written as bf16.
template <bool Q8>
__global__ void __launch_bounds__(1024) rmsnorm_residual_kernel(const uint16_t* __restrict__ x,
                                                                const uint16_t* __restrict__ res_in,
                                                                const uint16_t* __restrict__ weight,
                                                                uint16_t* __restrict__ res_out, uint16_t* __restrict__ out,
                                                                int8_t* __restrict__ out_q8, float* __restrict__ out_scale,
                                                                size_t hidden, float eps) {
    NVK_DYN_SMEM_AS(uint16_t, s_v);   // Q8 only: the normalised row
    __shared__ float s_warp[32];
    __shared__ uint32_t s_max;
    nvk::ptx::pdl_wait();
    nvk::ptx::pdl_launch_dependents();
    const size_t row = blockIdx.x;
    x += row * hidden; res_in += row * hidden; res_out += row * hidden;
    float ss = 0.f;
    for (size_t i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float s = nvk::bf16_bits_to_f32(x[i]) + nvk::bf16_bits_to_f32(res_in[i]);
        res_out[i] = nvk::f32_to_bf16_bits(s);
        ss = fmaf(s, s, ss);
    }
    const float rstd = rsqrtf(block_sum(ss, s_warp) / (float)hidden + eps);
    float amax = 0.f;
    for (size_t i = threadIdx.x; i < hidden; i += blockDim.x) {   // each thread re-reads what it wrote
        const uint16_t vb = nvk::f32_to_bf16_bits(nvk::bf16_bits_to_f32(res_out[i]) * rstd * nvk::bf16_bits_to_f32(weight[i]));
        if (Q8) {
            s_v[i] = vb;
            amax = fmaxf(amax, fabsf(nvk::bf16_bits_to_f32(vb)));
        } else {
            out[row * hidden + i] = vb;
        }
    }
    if (Q8) {
        const float scale = block_max_nonneg(amax, &s_max) / 127.0f;
        const float inv = scale > 0.f ? 1.0f / scale : 0.f;
        if (threadIdx.x == 0) out_scale[0] = scale;
        for (size_t i = threadIdx.x; i < hidden; i += blockDim.x) out_q8[i] = quant_i8(s_v[i], inv);
    }
}

}  // namespace

extern "C" {

int nv_kernels_gemv_nvfp4_w4a8_dual_m1(void* stream, const uint8_t* wq_a, const uint8_t* sc_a, const uint8_t* wq_b,
                                       const uint8_t* sc_b, const int8_t* x_q8, const float* x_dequant_scale,
                                       uint16_t* y_a, uint16_t* y_b, float alpha_a, float alpha_b, int N, int K) {
    if (N <= 0 || K <= 0 || (K & 31) != 0) return NVK_ERR_SHAPE;
    if (nvk::any_null(wq_b, sc_b, y_b)) return NVK_ERR_ARG;
    return w4a8_linear((cudaStream_t)stream, wq_a, sc_a, wq_b, sc_b, x_q8, x_dequant_scale, nullptr, y_a, y_b, alpha_a,
                       alpha_b, 1, N, K, nullptr, 0.f);
}

int nv_kernels_gemv_nvfp4_w4a8_dual_mk(void* stream, const uint8_t* wq_a, const uint8_t* sc_a, const uint8_t* wq_b,
                                       const uint8_t* sc_b, const int8_t* x_q8, const float* x_dequant_scales,
                                       uint16_t* y_a, uint16_t* y_b, float alpha_a, float alpha_b, int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0 || (K & 31) != 0) return NVK_ERR_SHAPE;
    if (nvk::any_null(wq_b, sc_b, y_b)) return NVK_ERR_ARG;
    return w4a8_linear((cudaStream_t)stream, wq_a, sc_a, wq_b, sc_b, x_q8, x_dequant_scales, nullptr, y_a, y_b, alpha_a,
                       alpha_b, M, N, K, nullptr, 0.f);
}

int nv_kernels_gemv_nvfp4_w4a8_down_residual_m1(void* stream, const uint8_t* wq, const uint8_t* sc, const int8_t* x_q8,
                                                const float* x_dequant_scale, const uint16_t* residual, uint16_t* y,
                                                float alpha, int N, int K) {
    if (N <= 0 || K <= 0 || (K & 31) != 0) return NVK_ERR_SHAPE;
    return w4a8_linear((cudaStream_t)stream, wq, sc, nullptr, nullptr, x_q8, x_dequant_scale, residual, y, nullptr, alpha,
                       0.f, 1, N, K, nullptr, 0.f);
}

int nv_kernels_gemv_nvfp4_w4a8_down_residual_m1_rstd_emit(void* stream, const uint8_t* wq, const uint8_t* sc,
                                                          const int8_t* x_q8, const float* x_dequant_scale,
                                                          const uint16_t* residual, uint16_t* y, float alpha,
                                                          float* rstd_ssq_count_pack, float rstd_eps, int N, int K) {
    if (N <= 0 || K <= 0 || (K & 31) != 0) return NVK_ERR_SHAPE;
    if (rstd_ssq_count_pack == nullptr) return NVK_ERR_ARG;
    return w4a8_linear((cudaStream_t)stream, wq, sc, nullptr, nullptr, x_q8, x_dequant_scale, residual, y, nullptr, alpha,
                       0.f, 1, N, K, rstd_ssq_count_pack, rstd_eps);
}

int nv_kernels_gemv_nvfp4_w4a8_down_residual_mk(void* stream, const uint8_t* wq, const uint8_t* sc, const int8_t* x_q8,
                                                const float* x_dequant_scales, const uint16_t* residual, uint16_t* y,
                                                float alpha, int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0 || (K & 31) != 0) return NVK_ERR_SHAPE;
    return w4a8_linear((cudaStream_t)stream, wq, sc, nullptr, nullptr, x_q8, x_dequant_scales, residual, y, nullptr, alpha,
                       0.f, M, N, K, nullptr, 0.f);
}

int nv_kernels_gemv_nvfp4_w4a8_down_residual_quant_prologue_m1(void* stream, const uint8_t* wq, const uint8_t* sc,
                                                               const uint16_t* act_staged_bf16,
                                                               const float* partial_absmax, int num_partials,
                                                               const uint16_t* residual, uint16_t* y, float alpha, int N,
                                                               int K) {
    if (N <= 0 || K <= 0 || (K & 31) != 0 || num_partials <= 0) return NVK_ERR_SHAPE;
    if (nvk::any_null(wq, sc, act_staged_bf16, partial_absmax, y)) return NVK_ERR_ARG;
    if (!aligned16(wq) || !aligned16(sc) || !aligned16(act_staged_bf16)) return NVK_ERR_ARG;
    GemmParams p = {};
    p.wq[0] = wq; p.sc[0] = sc;
    p.x = act_staged_bf16;
    p.y[0] = y;
    p.alpha[0] = alpha;
    p.M = 1; p.N = N; p.K = K;
    p.k_tiles = nvk::ceil_div(K, 64);
    p.nsc = nvk::ceil_div(K, kSuper);
    EpiArgs e = {};
    e.residual = residual;
    e.absmax_partials = partial_absmax;
    e.n_partials = num_partials;
    return launch_w4a8<1, false, 5>((cudaStream_t)stream, p, e);
}

int nv_kernels_silu_mul_rowquant_i8_m1(void* stream, const uint16_t* gate, const uint16_t* up, int8_t* act_q8,
                                       float* act_dequant_scale, int K) {
    if (K <= 0 || (K & 3) != 0) return NVK_ERR_SHAPE;
    const size_t smem = (size_t)K * sizeof(uint16_t);
    if (smem > 96 * 1024) return NVK_ERR_SHAPE;
    if (nvk::any_null(gate, up, act_q8, act_dequant_scale)) return NVK_ERR_ARG;
    static nvk::SmemOptin optin;
    if (int rc = optin.ensure((const void*)silu_rowquant_m1_kernel, smem)) return rc;
    return nvk::launch(nvk::launch_1d((cudaStream_t)stream, 1, 1024, smem, true), silu_rowquant_m1_kernel, gate, up, act_q8,
                       act_dequant_scale, K);
}

int nv_kernels_silu_mul_rowquant_i8_mk_partials_len(int M, int K) {
    if (M <= 0 || K <= 0) return NVK_ERR_SHAPE;
    return M * split_blocks(K);
}

int nv_kernels_silu_mul_rowquant_i8_mk(void* stream, const uint16_t* gate, const uint16_t* up, uint16_t* act_staged_bf16,
                                       float* partial_absmax, int8_t* act_q8, float* act_dequant_scales, int M, int K) {
    if (M <= 0 || K <= 0 || (K & 15) != 0) return NVK_ERR_SHAPE;
    if (nvk::any_null(gate, up, act_staged_bf16, partial_absmax, act_q8, act_dequant_scales)) return NVK_ERR_ARG;
    if (M > 65535) return NVK_ERR_GRID_AXIS;
    const int bx = split_blocks(K);
    nvk::Launch l;
    l.grid = dim3((unsigned)bx, (unsigned)M, 1);
    l.block = dim3(kSplitThreads, 1, 1);
    l.stream = (cudaStream_t)stream;
    l.pdl = true;
    if (int rc = nvk::launch(l, silu_stage_absmax_kernel, gate, up, act_staged_bf16, partial_absmax, K)) return rc;
    return nvk::launch(l, rowquant_from_staged_kernel, (const uint16_t*)act_staged_bf16, (const float*)partial_absmax, bx,
                       act_q8, act_dequant_scales, K);
}

int nv_kernels_silu_mul_stage_partial_absmax_m1(void* stream, const uint16_t* gate, const uint16_t* up,
                                                uint16_t* act_staged_bf16, float* partial_absmax, int K) {
    if (K <= 0 || (K & 15) != 0) return NVK_ERR_SHAPE;
    if (nvk::any_null(gate, up, act_staged_bf16, partial_absmax)) return NVK_ERR_ARG;
    nvk::Launch l;
    l.grid = dim3((unsigned)split_blocks(K), 1, 1);
    l.block = dim3(kSplitThreads, 1, 1);
    l.stream = (cudaStream_t)stream;
    l.pdl = true;
    return nvk::launch(l, silu_stage_absmax_kernel, gate, up, act_staged_bf16, partial_absmax, K);
}

int nv_kernels_rmsnorm_residual_writeout_rowquant_i8_m1(void* stream, const uint16_t* x, const uint16_t* res_in,
                                                        const uint16_t* weight, uint16_t* res_out, int8_t* out_q8,
                                                        float* out_dequant_scale, int hidden, float eps) {
    if (hidden <= 0 || hidden > 24576) return NVK_ERR_SHAPE;
    if (nvk::any_null(x, res_in, weight, res_out, out_q8, out_dequant_scale)) return NVK_ERR_ARG;
    const size_t smem = (size_t)hidden * sizeof(uint16_t);
    static nvk::SmemOptin optin;
    if (int rc = optin.ensure((const void*)rmsnorm_residual_kernel<true>, smem)) return rc;
    return nvk::launch(nvk::launch_1d((cudaStream_t)stream, 1, 1024, smem, true), rmsnorm_residual_kernel<true>, x, res_in,
                       weight, res_out, (uint16_t*)nullptr, out_q8, out_dequant_scale, (size_t)hidden, eps);
}

int nv_kernels_rmsnorm_residual_writeout_bf16(void* stream, const uint16_t* x, const uint16_t* res_in,
                                              const uint16_t* weight, uint16_t* res_out, uint16_t* out, size_t batch,
                                              size_t hidden, float eps) {
    if (batch == 0 || hidden == 0) return 0;
    if (nvk::any_null(x, res_in, weight, res_out, out)) return NVK_ERR_ARG;
    if (batch > 0x7FFFFFFFull) return NVK_ERR_GRID_AXIS;
    const unsigned threads = hidden >= 4096 ? 1024 : 256;
    return nvk::launch(nvk::launch_1d((cudaStream_t)stream, (unsigned)batch, threads, 0, true), rmsnorm_residual_kernel<false>,
                       x, res_in, weight, res_out, out, (int8_t*)nullptr, (float*)nullptr, hidden, eps);
}

}  // extern "C"
