// Prefill-sized block-scaled NVFP4 GEMM on the 5th-generation tensor cores:
//
//   D[m, n] = bf16( alpha * sum_k A[m, k] * B[n, k] ),  A and B packed e2m1 with one ue4m3 scale per 16
//   values along K (128x4 swizzled scale layout), alpha an fp32 scalar in device memory.
//
// The contraction is the CUTLASS sm100 block-scaled collective (tcgen05.mma kind::mxf4nvf4 with the
// scale factors in tensor memory, TMA operand loads, accumulators in TMEM), instantiated here for a
// 1-SM 128x128x256 tile (no cluster; the default) and a 2-SM 256x128x256 tile (cluster 2x1x1).  The
// 2-SM collective loads its operands with TMA cluster multicast, and its tensor maps are built over
// the pointers the caller passes: they must be this GPU's own memory.  The library is therefore for
// single-GPU processes only -- the host binding refuses to load or call it from one rank of a
// multi-GPU job, where rows beyond 64 run in chunks on the decode-sized kernels instead.  This file
// is the whole integration: problem setup, workspace protocol and the reference's entry points for
// this route.
//
// Built only when CUTLASS headers are found (NVK_HAVE_CUTLASS); otherwise the entry points refuse
// with -1 ("route unavailable"), as the reference's GPU-less stubs do.
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <type_traits>

#include "../csrc/nvk_common.cuh"

#ifdef NVK_HAVE_CUTLASS
#include "cutlass/cutlass.h"
#include "cute/tensor.hpp"
#include "cutlass/detail/sm100_blockscaled_layout.hpp"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/epilogue/thread/linear_combination.h"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/dispatch_policy.hpp"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/util/packed_stride.hpp"

namespace {

using namespace cute;

using ElementAB = cutlass::nv_float4_t<cutlass::float_e2m1_t>;
using ElementD = cutlass::bfloat16_t;
using ElementAcc = float;
using LayoutA = cutlass::layout::RowMajor;      // activations [m, k], K contiguous
using LayoutB = cutlass::layout::ColumnMajor;   // weights [n, k] seen as a K x N column-major operand
using LayoutD = cutlass::layout::RowMajor;
constexpr int kAlignAB = 32;                    // elements: 16 bytes of packed e2m1
constexpr int kAlignD = 128 / cutlass::sizeof_bits<ElementD>::value;

template <class TileShape, class ClusterShape, class Scheduler = void>
struct GemmConfig {
    using Epilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassBlockScaledTensorOp, TileShape, ClusterShape,
        cutlass::epilogue::collective::EpilogueTileAuto, ElementAcc, ElementAcc, void, LayoutD, kAlignD, ElementD,
        LayoutD, kAlignD, cutlass::epilogue::collective::EpilogueScheduleAuto>::CollectiveOp;
    using Mainloop = typename cutlass::gemm::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassBlockScaledTensorOp, ElementAB, LayoutA, kAlignAB, ElementAB,
        LayoutB, kAlignAB, ElementAcc, TileShape, ClusterShape,
        cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epilogue::SharedStorage))>,
        cutlass::gemm::collective::KernelScheduleAuto>::CollectiveOp;
    using GemmKernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, Mainloop, Epilogue, Scheduler>;
    using Gemm = cutlass::gemm::device::GemmUniversalAdapter<GemmKernel>;
    using SfConfig = typename GemmKernel::CollectiveMainloop::Sm1xxBlkScaledConfig;
};

// 1-SM tile, no cluster, no multicast: the default.
using Cfg1 = GemmConfig<Shape<_128, _128, _256>, Shape<_1, _1, _1>>;
// 2-SM tile (cta_group::2 pair sharing one 256x128 accumulator tile), cluster 2x1x1, operands loaded
// with cluster multicast: opt-in through nvk_b200_set_prefill_config(2), single-GPU processes only,
// every operand this GPU's own memory.
using Cfg2 = GemmConfig<Shape<_256, _128, _256>, Shape<_2, _1, _1>>;

// The 1-SM tile under the stream-K scheduler: output tiles that do not fill the last wave are split
// along K over the idle SMs and reduced through the workspace (K = 25600 with 320 output tiles on 148
// SMs is the case it exists for).
using Cfg1SK = GemmConfig<Shape<_128, _128, _256>, Shape<_1, _1, _1>, cutlass::gemm::StreamKScheduler>;

// The tile choice is per calling thread (the entry points may be called from any thread).
thread_local int g_prefill_cfg = 1;

template <class Cfg>
typename Cfg::Gemm::Arguments make_args(const void* a, const void* a_sf, const void* b, const void* b_sf,
                                   const float* alpha_dev, void* d, int m, int n, int k, int splits = 0) {
    using Gemm = typename Cfg::Gemm;
    using GemmKernel = typename Cfg::GemmKernel;
    using SfConfig = typename Cfg::SfConfig;
    using StrideA = typename Gemm::GemmKernel::StrideA;
    using StrideB = typename Gemm::GemmKernel::StrideB;
    using StrideD = typename Gemm::GemmKernel::StrideD;
    using ElemA = typename Gemm::ElementA;
    using ElemB = typename Gemm::ElementB;
    using ElemSF = typename GemmKernel::CollectiveMainloop::ElementSF;
    typename Gemm::Arguments args{};
    args.mode = cutlass::gemm::GemmUniversalMode::kGemm;
    args.problem_shape = {m, n, k, 1};
    args.mainloop.ptr_A = static_cast<const ElemA*>(a);
    args.mainloop.dA = cutlass::make_cute_packed_stride(StrideA{}, {m, k, 1});
    args.mainloop.ptr_B = static_cast<const ElemB*>(b);
    args.mainloop.dB = cutlass::make_cute_packed_stride(StrideB{}, {n, k, 1});
    args.mainloop.ptr_SFA = static_cast<const ElemSF*>(a_sf);
    args.mainloop.layout_SFA = SfConfig::tile_atom_to_shape_SFA(cute::make_shape(m, n, k, 1));
    args.mainloop.ptr_SFB = static_cast<const ElemSF*>(b_sf);
    args.mainloop.layout_SFB = SfConfig::tile_atom_to_shape_SFB(cute::make_shape(m, n, k, 1));
    args.epilogue.thread.alpha = 1.0f;
    args.epilogue.thread.beta = 0.0f;
    args.epilogue.thread.alpha_ptr = alpha_dev;
    args.epilogue.ptr_C = nullptr;
    args.epilogue.dC = cutlass::make_cute_packed_stride(StrideD{}, {m, n, 1});
    args.epilogue.ptr_D = static_cast<ElementD*>(d);
    args.epilogue.dD = cutlass::make_cute_packed_stride(StrideD{}, {m, n, 1});
    if constexpr (std::is_same_v<Cfg, Cfg1SK>) {
        if (splits >= 2) args.scheduler.splits = splits;   // forced split of every tile; else the heuristic
    }
    return args;
}

template <class Cfg>
int run_gemm_cfg(cudaStream_t stream, const void* a, const void* a_sf, const void* b, const void* b_sf,
                 const float* alpha_dev, void* d, int m, int n, int k, void* workspace, size_t workspace_bytes,
                 size_t* required_workspace, int splits = 0) {
    using Gemm = typename Cfg::Gemm;
    if (m <= 0 || n <= 0 || k <= 0) return NVK_ERR_SHAPE;
    if ((k % 32) != 0 || (n % 8) != 0) return NVK_ERR_SHAPE;  // 16-byte rows of packed operands and of D
    try {
        auto args = make_args<Cfg>(a, a_sf, b, b_sf, alpha_dev, d, m, n, k, splits);
        const size_t need = Gemm::get_workspace_size(args);
        if (required_workspace) *required_workspace = need;
        // all data pointers null: a pure workspace query, nothing is launched
        if (!a && !a_sf && !b && !b_sf && !d) return 0;
        if (!a || !a_sf || !b || !b_sf || !d || !alpha_dev) return NVK_ERR_ARG;
        if (need > workspace_bytes || (need > 0 && !workspace)) return -10;
        Gemm gemm;
        if (gemm.can_implement(args) != cutlass::Status::kSuccess) return -11;
        if (gemm.initialize(args, workspace, stream) != cutlass::Status::kSuccess) return -12;
        if (gemm.run(stream) != cutlass::Status::kSuccess) return -13;
        return 0;
    } catch (...) {
        return NVK_ERR_SHAPE;
    }
}

int run_gemm(cudaStream_t stream, const void* a, const void* a_sf, const void* b, const void* b_sf,
             const float* alpha_dev, void* d, int m, int n, int k, void* workspace, size_t workspace_bytes,
             size_t* required_workspace) {
    if (g_prefill_cfg == 2)
        return run_gemm_cfg<Cfg2>(stream, a, a_sf, b, b_sf, alpha_dev, d, m, n, k, workspace, workspace_bytes,
                                  required_workspace);
    return run_gemm_cfg<Cfg1>(stream, a, a_sf, b, b_sf, alpha_dev, d, m, n, k, workspace, workspace_bytes,
                              required_workspace);
}

int run_gemm_streamk(cudaStream_t stream, const void* a, const void* a_sf, const void* b, const void* b_sf,
                     const float* alpha_dev, void* d, int m, int n, int k, void* workspace, size_t workspace_bytes,
                     size_t* required_workspace, int splits) {
    return run_gemm_cfg<Cfg1SK>(stream, a, a_sf, b, b_sf, alpha_dev, d, m, n, k, workspace, workspace_bytes,
                                required_workspace, splits);
}

}  // namespace
#else   // !NVK_HAVE_CUTLASS
namespace { thread_local int g_prefill_cfg = 1; }
namespace {
int run_gemm(cudaStream_t, const void*, const void*, const void*, const void*, const float*, void*, int, int, int,
             void*, size_t, size_t* required_workspace) {
    if (required_workspace) *required_workspace = 0;
    return NVK_ERR_SHAPE;
}
int run_gemm_streamk(cudaStream_t, const void*, const void*, const void*, const void*, const float*, void*, int, int, int,
                     void*, size_t, size_t* required_workspace, int) {
    if (required_workspace) *required_workspace = 0;
    return NVK_ERR_SHAPE;
}
}  // namespace
#endif

extern "C" {

// Tuning hook (no counterpart in the reference): 1 = 1-SM 128x128x256 tile (default), 2 = 2-SM
// 256x128x256 tile with cluster-multicast operand loads (single-GPU processes, local operands only).
// Applies to later calls made by the calling thread.
int nvk_b200_set_prefill_config(int cfg) {
    if (cfg != 1 && cfg != 2) return NVK_ERR_ARG;
    g_prefill_cfg = cfg;
    return 0;
}

// The reference names these after the architecture of its own tensor-core kernels; the symbols are
// kept so that its call sites bind unchanged.
//   ..._bf16          the data-parallel kernel with the tile nvk_b200_set_prefill_config selected;
//   ..._bf16_streamk  the 1-SM tile under the stream-K scheduler (its own, larger workspace: query it
//                     through this symbol);
//   ..._bf16_tiled    `tile` 0..2 names one of the reference's sm_120 tile shapes -- all three map to
//                     the one 1-SM 128x128x256 tile here, any other value is -3 as in the reference --
//                     and `stream_k` keeps its meaning: 0 data-parallel, 1 stream-K, >= 2 that many
//                     forced splits of every output tile along K.
int nv_kernels_cutlass_fp4_gemm_sm120_bf16(void* stream, const void* a_fp4, const void* a_sf, const void* b_fp4,
                                           const void* b_sf, const float* global_sf, void* d_bf16, int m, int n, int k,
                                           void* workspace, size_t workspace_bytes, size_t* required_workspace) {
    return run_gemm((cudaStream_t)stream, a_fp4, a_sf, b_fp4, b_sf, global_sf, d_bf16, m, n, k, workspace,
                    workspace_bytes, required_workspace);
}

int nv_kernels_cutlass_fp4_gemm_sm120_bf16_streamk(void* stream, const void* a_fp4, const void* a_sf,
                                                   const void* b_fp4, const void* b_sf, const float* global_sf,
                                                   void* d_bf16, int m, int n, int k, void* workspace,
                                                   size_t workspace_bytes, size_t* required_workspace) {
    return run_gemm_streamk((cudaStream_t)stream, a_fp4, a_sf, b_fp4, b_sf, global_sf, d_bf16, m, n, k, workspace,
                            workspace_bytes, required_workspace, 0);
}

int nv_kernels_cutlass_fp4_gemm_sm120_bf16_tiled(void* stream, const void* a_fp4, const void* a_sf, const void* b_fp4,
                                                 const void* b_sf, const float* global_sf, void* d_bf16, int m, int n,
                                                 int k, int tile, int stream_k, void* workspace,
                                                 size_t workspace_bytes, size_t* required_workspace) {
    if (tile < 0 || tile > 2 || stream_k < 0) return NVK_ERR_RESOURCE;
    if (stream_k >= 1)
        return run_gemm_streamk((cudaStream_t)stream, a_fp4, a_sf, b_fp4, b_sf, global_sf, d_bf16, m, n, k, workspace,
                                workspace_bytes, required_workspace, stream_k >= 2 ? stream_k : 0);
#ifdef NVK_HAVE_CUTLASS
    return run_gemm_cfg<Cfg1>((cudaStream_t)stream, a_fp4, a_sf, b_fp4, b_sf, global_sf, d_bf16, m, n, k, workspace,
                              workspace_bytes, required_workspace);
#else
    return run_gemm((cudaStream_t)stream, a_fp4, a_sf, b_fp4, b_sf, global_sf, d_bf16, m, n, k, workspace,
                    workspace_bytes, required_workspace);
#endif
}

}  // extern "C"
