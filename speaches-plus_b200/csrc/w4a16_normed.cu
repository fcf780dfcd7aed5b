// W4A16 linear with an RMSNorm in front, in one launch:
//
//   y[m, n] = bf16( alpha * sum_k W[n, k] * a[m, k] ),   a[m, k] = bf16( x[m, k] * rstd[m] * norm_w[k] ),
//   rstd[m] = rsqrt( mean_k x[m, k]^2 + eps )
//
// for one or two weight matrices sharing x (a decoder layer's QKV projection, or gate and up).  The
// norm is applied while the tile stages its activations (tile prologue 6): a is rounded to bf16
// exactly as the stand-alone norm kernel rounds it and rstd is summed in that kernel's order, so the
// result equals nv_kernels_rmsnorm_bf16 followed by the plain linear, bit for bit, with one launch
// and one pass over x less.  rstd may also be handed in (one f32 per row), e.g. the value a previous
// residual-update launch left behind (nvk_b200_linear_nvfp4_w4a16_residual_rstd_emit).
#include "w4a16_tile.cuh"

namespace {

struct NormArgs {
    const uint16_t* norm_w;
    const float* rstd;
    float eps;
};

template <int NT, bool DUAL>
__global__ void __launch_bounds__(256, kTileCtasPerSm<NT>) w4a16_normed_kernel(const GemmParams p, const NormArgs a) {
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
    t.norm_w = a.norm_w;
    t.rstd_in = a.rstd;
    t.norm_eps = a.eps;
    w4a16_tile<NT, 6, 8, 1>(p, t);
}

template <int NT, bool DUAL>
int launch_normed(cudaStream_t stream, GemmParams& p, const NormArgs& a) {
    p.tiles_per_arm = nvk::ceil_div(p.N, kRowsPerCta);
    const int ctas = (DUAL ? 2 : 1) * p.tiles_per_arm;
    if (ctas > 65535) return NVK_ERR_GRID_AXIS;
    const int ksplit = tile_ksplit(ctas, p.nsc);
    const size_t smem = tile_layout_rows128(p, p.M, 8 * NT, ksplit);
    static nvk::SmemOptin optin;
    auto* kern = w4a16_normed_kernel<NT, DUAL>;
    if (int rc = optin.ensure((const void*)kern, smem)) return rc;
    nvk::Launch l;
    l.grid = dim3((unsigned)ksplit, (unsigned)ctas, 1);
    l.block = dim3(256, 1, 1);
    l.smem = smem;
    l.stream = stream;
    l.cluster_x = (unsigned)ksplit;
    l.pdl = true;
    return nvk::launch(l, kern, p, a);
}

template <bool DUAL>
int dispatch_normed(cudaStream_t stream, GemmParams& p, const NormArgs& a) {
    if (p.M <= 8) return launch_normed<1, DUAL>(stream, p, a);
    if (p.M <= 16) return launch_normed<2, DUAL>(stream, p, a);
    if (p.M <= 32) return launch_normed<4, DUAL>(stream, p, a);
    return launch_normed<8, DUAL>(stream, p, a);
}

bool aligned16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; }

}  // namespace

extern "C" {

// No counterpart in the reference with this signature (its fused norms feed the quantizing routes).
// wq_b / sc_b / y_b all null: one matrix.  rstd null: every CTA sums its rows' squares itself, which is
// meant for a few rows -- M <= 8; with rstd given, M <= 64.  0 for an empty problem; -1 for M outside
// that range, K % 32 != 0 or a half-given second matrix; -2 for a null or not 16-byte aligned operand.
int nvk_b200_linear_nvfp4_w4a16_normed(void* stream, const uint8_t* wq_a, const uint8_t* sc_a, const uint8_t* wq_b,
                                       const uint8_t* sc_b, const uint16_t* x, const uint16_t* norm_weight,
                                       const float* rstd, float eps, uint16_t* y_a, uint16_t* y_b, float alpha_a,
                                       float alpha_b, int M, int N, int K) {
    if (N <= 0 || K <= 0) return 0;
    if (M <= 0 || M > (rstd != nullptr ? 64 : 8) || (K & 31) != 0) return NVK_ERR_SHAPE;
    const bool dual = wq_b != nullptr;
    if (dual != (sc_b != nullptr) || dual != (y_b != nullptr)) return NVK_ERR_SHAPE;
    if (nvk::any_null(wq_a, sc_a, x, norm_weight, y_a)) return NVK_ERR_ARG;
    if (!aligned16(wq_a) || !aligned16(sc_a) || !aligned16(x) || !aligned16(norm_weight) ||
        (dual && (!aligned16(wq_b) || !aligned16(sc_b))))
        return NVK_ERR_ARG;
    GemmParams p = {};
    p.wq[0] = wq_a; p.wq[1] = wq_b;
    p.sc[0] = sc_a; p.sc[1] = sc_b;
    p.x = x;
    p.y[0] = y_a; p.y[1] = y_b;
    p.alpha[0] = alpha_a; p.alpha[1] = alpha_b;
    p.M = M; p.N = N; p.K = K;
    p.k_tiles = nvk::ceil_div(K, 64);
    p.nsc = nvk::ceil_div(K, kSuper);
    NormArgs a;
    a.norm_w = norm_weight;
    a.rstd = rstd;
    a.eps = eps;
    return dual ? dispatch_normed<true>((cudaStream_t)stream, p, a) : dispatch_normed<false>((cudaStream_t)stream, p, a);
}

}  // extern "C"
