// Row-parallel (K-sharded) W4A16 linear and its all-reduce in ONE launch per GPU.
//
// Every GPU of a tensor-parallel group holds a K slice of the weight and of the activations; the
// outputs are partial sums that have to be added across the GPUs.  Run as two kernels (the linear,
// then an all-reduce) the step pays a second launch and a flag round trip that cannot start before the
// whole linear is done.  Here the tile's epilogue does the exchange itself: each CTA stores its
// bf16 partials straight into its own region of every GPU's inbox (plain peer stores over NVLink),
// raises one flag per GPU, waits -- bounded -- for the same CTA of every other GPU, and writes the sum of
// the partials in rank order (plus an optional residual).  A CTA only ever waits for the CTA with its
// own index on the other GPUs, all GPUs run the same grid in the same order, and tiles that finish
// early exchange while later tiles still stream weights.  No multicast, no TMA, no library kernel is
// handed peer memory.
//
// Results equal the two-kernel form bit for bit (bf16 partials, fp32 sum in rank order, one rounding).
// Up to 64 rows (the buffers are sized for a row capacity); the exchange buffers
// (nvk_b200_tp_fused_buffer_bytes) are plain device memory shared with CUDA IPC like the all-reduce's.
// The ranks must make the same sequence of calls.
#include "w4a16_tile.cuh"

namespace {

constexpr int kMaxRanks = 8;

template <int NT, int PRO>
__global__ void __launch_bounds__(256, kTileCtasPerSm<NT>)
    tp_linear_kernel(const GemmParams p, const __grid_constant__ ExchangeArgs a) {
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
    t.xch = &a;   // a grid-constant parameter: its address is usable as it stands, nothing is copied
    t.xch_cta = (int)(blockIdx.y * gridDim.x + blockIdx.x);
    w4a16_tile<NT, PRO, 8, 1, false, LaunchHooks, 2>(p, t);
}

template <int NT, int PRO>
int launch_tp_linear(cudaStream_t stream, GemmParams& p, const ExchangeArgs& a) {
    p.tiles_per_arm = nvk::ceil_div(p.N, kRowsPerCta);
    const int ksplit = tile_ksplit(p.tiles_per_arm, p.nsc);
    if ((long)p.tiles_per_arm * ksplit > a.max_ctas) return NVK_ERR_RESOURCE;
    const size_t smem = tile_layout_rows128(p, p.M, 8 * NT, ksplit);
    static nvk::SmemOptin optin;
    auto* kern = tp_linear_kernel<NT, PRO>;
    if (int rc = optin.ensure((const void*)kern, smem)) return rc;
    nvk::Launch l;
    l.grid = dim3((unsigned)ksplit, (unsigned)p.tiles_per_arm, 1);
    l.block = dim3(256, 1, 1);
    l.smem = smem;
    l.stream = stream;
    l.cluster_x = (unsigned)ksplit;
    l.pdl = true;
    return nvk::launch(l, kern, p, a);
}

template <int PRO>
int dispatch_tp_linear(cudaStream_t stream, GemmParams& p, const ExchangeArgs& a) {
    if (p.M <= 8) return launch_tp_linear<1, PRO>(stream, p, a);
    if (p.M <= 16) return launch_tp_linear<2, PRO>(stream, p, a);
    if (p.M <= 32) return launch_tp_linear<4, PRO>(stream, p, a);
    return launch_tp_linear<8, PRO>(stream, p, a);
}

bool aligned16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; }

}  // namespace

extern "C" {

// Bytes of the exchange buffer every rank provides (zero-filled before the first call) for launches of
// up to max_ctas CTAs and up to max_rows activation rows; 0 for arguments out of range.
size_t nvk_b200_tp_fused_buffer_bytes(int world, int max_ctas, int max_rows) {
    if (world <= 0 || world > kMaxRanks || max_ctas <= 0 || max_ctas > 4096 || max_rows <= 0 || max_rows > 64) return 0;
    return exchange_buffer_bytes(world, max_ctas, max_rows);
}

// y [M, N] = bf16( sum over ranks of bf16(alpha * x_r W_r^T)  (+ residual) ), the same bits on every rank.
// wq / sc: this rank's K slice of the weight ([N, K/2] packed, its own swizzled scales); x (and x2 for
// the SiLU(x) * x2 prologue): this rank's [M, K] slice of the activations; K is the slice's length.
// peer_bufs: `world` device pointers, the exchange buffers of ranks 0..world-1 as mapped in this
// process, sized for (max_ctas, max_rows); epoch: max_ctas uint32 of local device memory, zero before the
// first call; err: one int that becomes 1 + r if rank r never arrived within the wait limit (the call
// then leaves y unwritten for the affected tiles and returns normally: the context stays usable).
// 1 <= M <= max_rows <= 64.  0 for an empty problem; -1 for M outside that range or K % 32 != 0; -2 for
// null or misaligned operands or a rank outside the world; -3 when the launch needs more CTAs than max_ctas.
int nvk_b200_tp_linear_nvfp4_w4a16_allreduce(void* stream, const void* const* peer_bufs, int rank, int world,
                                             const uint8_t* wq, const uint8_t* sc, const uint16_t* x, const uint16_t* x2,
                                             const uint16_t* residual, uint16_t* y, float alpha, int M, int N, int K,
                                             int max_ctas, int max_rows, uint32_t* epoch, int* err) {
    if (N <= 0 || K <= 0) return 0;
    if (max_rows <= 0 || max_rows > 64) return NVK_ERR_ARG;
    if (M <= 0 || M > max_rows || (K & 31) != 0) return NVK_ERR_SHAPE;
    if (world <= 0 || world > kMaxRanks || rank < 0 || rank >= world || max_ctas <= 0 || max_ctas > 4096)
        return NVK_ERR_ARG;
    if (!peer_bufs || nvk::any_null(wq, sc, x, y, epoch, err)) return NVK_ERR_ARG;
    if (!aligned16(wq) || !aligned16(sc) || !aligned16(x) || (x2 != nullptr && !aligned16(x2))) return NVK_ERR_ARG;
    ExchangeArgs a = {};
    for (int r = 0; r < world; ++r) {
        if (!peer_bufs[r]) return NVK_ERR_ARG;
        a.peer[r] = static_cast<uint8_t*>(const_cast<void*>(peer_bufs[r]));
    }
    a.epoch = epoch;
    a.err = err;
    a.residual = residual;
    a.rank = rank;
    a.world = world;
    a.max_ctas = max_ctas;
    a.cta_elems = 128 * max_rows;
    a.wait_limit = nvk::wait_limit_setting();
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
    return x2 != nullptr ? dispatch_tp_linear<1>((cudaStream_t)stream, p, a) : dispatch_tp_linear<0>((cudaStream_t)stream, p, a);
}

}  // extern "C"
