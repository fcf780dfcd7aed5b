// W4A16 linear whose output is a residual update:
//
//   y[m, n] = bf16( fma( sum_k e2m1(W[n,k]) * ue4m3(S[n,k/16]) * a[m,k],  alpha,  residual[m,n] ) )
//
// with a = x, or a = bf16(SiLU(x) * x2) formed while the activations are staged -- the tail of a decoder
// MLP (gate/up outputs in, new hidden state out) or an attention output projection, in one launch and
// with one rounding.  The W4A16 tile with its residual epilogue; nothing else is new here.
#include "w4a16_tile.cuh"

namespace {

struct ResidualArgs {
    const uint16_t* residual;
    float* rstd_pack;      // optional {rstd, sum of squares, arrivals}: see emit_rstd in w4a16_tile.cuh
    float rstd_eps;
    unsigned rstd_blocks;
};

template <int NT, int PRO>
__global__ void __launch_bounds__(256, kTileCtasPerSm<NT>) w4a16_residual_kernel(const GemmParams p, const ResidualArgs r) {
    TileView t = {};
    t.wq = p.wq[0];
    t.sc = p.sc[0];
    t.x = p.x;
    t.x2 = p.x2;
    t.y = p.y[0];
    t.alpha = p.alpha[0];
    t.M = p.M;
    t.sub = blockIdx.y;
    t.pdl = true;
    t.residual = r.residual;
    t.rstd_pack = r.rstd_pack;
    t.rstd_eps = r.rstd_eps;
    t.rstd_blocks = r.rstd_blocks;
    w4a16_tile<NT, PRO, 8, 1, false, LaunchHooks, 1>(p, t);
}

template <int NT, int PRO>
int launch_residual(cudaStream_t stream, GemmParams& p, ResidualArgs r) {
    p.tiles_per_arm = nvk::ceil_div(p.N, kRowsPerCta);
    if (p.tiles_per_arm > 65535) return NVK_ERR_GRID_AXIS;
    const int ksplit = tile_ksplit(p.tiles_per_arm, p.nsc);
    const size_t smem = tile_layout_rows128(p, p.M, 8 * NT, ksplit);
    static nvk::SmemOptin optin;
    auto* kern = w4a16_residual_kernel<NT, PRO>;
    if (int rc = optin.ensure((const void*)kern, smem)) return rc;
    r.rstd_blocks = (unsigned)(p.tiles_per_arm * ksplit);
    nvk::Launch l;
    l.grid = dim3((unsigned)ksplit, (unsigned)p.tiles_per_arm, 1);
    l.block = dim3(256, 1, 1);
    l.smem = smem;
    l.stream = stream;
    l.cluster_x = (unsigned)ksplit;
    l.pdl = true;
    return nvk::launch(l, kern, p, r);
}

template <int PRO>
int dispatch_residual(cudaStream_t stream, GemmParams& p, const ResidualArgs& r) {
    if (p.M <= 8) return launch_residual<1, PRO>(stream, p, r);
    if (p.M <= 16) return launch_residual<2, PRO>(stream, p, r);
    if (p.M <= 32) return launch_residual<4, PRO>(stream, p, r);
    return launch_residual<8, PRO>(stream, p, r);
}

bool aligned16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; }

int residual_linear(cudaStream_t stream, const uint8_t* wq, const uint8_t* sc, const uint16_t* x, const uint16_t* x2,
                    const uint16_t* residual, uint16_t* y, float alpha, int M, int N, int K, float* rstd_pack,
                    float eps) {
    if (N <= 0 || K <= 0) return 0;
    if (M <= 0 || M > 64 || (K & 31) != 0) return NVK_ERR_SHAPE;
    if (nvk::any_null(wq, sc, x, residual, y)) return NVK_ERR_ARG;
    if (!aligned16(wq) || !aligned16(sc) || !aligned16(x) || (x2 != nullptr && !aligned16(x2))) return NVK_ERR_ARG;
    GemmParams p = {};
    p.wq[0] = wq;
    p.sc[0] = sc;
    p.x = x;
    p.x2 = x2;
    p.y[0] = y;
    p.alpha[0] = alpha;
    p.M = M; p.N = N; p.K = K;
    p.k_tiles = nvk::ceil_div(K, 64);
    p.nsc = nvk::ceil_div(K, kSuper);
    ResidualArgs r = {};
    r.residual = residual;
    r.rstd_pack = rstd_pack;
    r.rstd_eps = eps;
    return x2 != nullptr ? dispatch_residual<1>(stream, p, r) : dispatch_residual<0>(stream, p, r);
}

}  // namespace

extern "C" {

// No counterpart in the reference (its residual epilogues exist for int8 activations only).  x [M, K]
// bf16; x2 null, or [M, K] bf16 for the SiLU(x) * x2 prologue; residual [M, N] bf16, which y may alias
// (every element is read before it is written, by the same thread); 1 <= M <= 64.  0 for an empty
// problem, -1 for M outside [1, 64] or K % 32 != 0, -2 for null or not 16-byte aligned operands.
int nvk_b200_linear_nvfp4_w4a16_residual(void* stream, const uint8_t* wq, const uint8_t* sc, const uint16_t* x,
                                         const uint16_t* x2, const uint16_t* residual, uint16_t* y, float alpha, int M,
                                         int N, int K) {
    return residual_linear((cudaStream_t)stream, wq, sc, x, x2, residual, y, alpha, M, N, K, nullptr, 0.f);
}

// One row (M = 1), and the launch also leaves 1/rms of the new row for the RMSNorm that follows:
// rstd_pack[0] = rsqrt(mean(y^2) + eps) over the N rounded outputs.  rstd_pack is three floats in device
// memory, {rstd, running sum of squares, arrival count}; the last two must be zero before the first
// launch and are returned to zero by every launch.  The CTAs' partial sums are added with float
// atomics in arrival order, so the last bits of rstd may differ from run to run (as in the reference's
// int8 form, rust/crates/nv-kernels/include/nv_kernels.h:652-678).  -2 for a null rstd_pack.
int nvk_b200_linear_nvfp4_w4a16_residual_rstd_emit(void* stream, const uint8_t* wq, const uint8_t* sc,
                                                   const uint16_t* x, const uint16_t* x2, const uint16_t* residual,
                                                   uint16_t* y, float alpha, float* rstd_pack, float eps, int N, int K) {
    if (N <= 0 || K <= 0) return 0;
    if (rstd_pack == nullptr) return NVK_ERR_ARG;
    return residual_linear((cudaStream_t)stream, wq, sc, x, x2, residual, y, alpha, 1, N, K, rstd_pack, eps);
}

}  // extern "C"
