// Grouped block-scaled NVFP4 GEMM for prefill-sized MoE steps on the 5th-generation tensor cores:
// one launch runs, for every active expert group g,
//
//   D_g[m_g, n] = bf16( alpha[e_g] * A_g[m_g, k] * B[e_g][n, k]^T )
//
// with A (activations, quantized online) and B (expert weights) packed e2m1 plus one ue4m3 scale per
// 16 values along K in the 128x4 swizzled layout, and the problem sizes, row offsets and expert ids
// in DEVICE memory, so that a routed step never round-trips to the host.
//
// Addressing (the reference's convention, rust/crates/nv-layers/src/moe_grouped.rs:352-573):
//   group g holds rows [expert_offsets[g], expert_offsets[g] + m_g) of the stacked activations and
//   writes the same rows of D; its activation scales start at sf_offsets[g] rows (a multiple of 128)
//   of the stacked, 128-row-padded scale buffer; its weights are expert
//   e_g = active_expert_indices ? active_expert_indices[g] : g of the bank ([N, K/2] bytes and
//   ceil(N/128)*128 x ceil(K/64)*4 scale bytes per expert); (m_g, n_g, k_g) = problem_sizes[3g..3g+2].
//
// The contraction is the CUTLASS sm100 pointer-array block-scaled collective (tcgen05.mma
// kind::mxf4nvf4, scale factors in tensor memory, TMA operand loads with per-group descriptors,
// accumulators in TMEM) with a 1-SM 128x128x256 tile and no cluster: library templates instantiated
// here, not a hand-written kernel.  What this file adds is the planning step in front of it: one
// kernel turns the routing tables into the per-group argument arrays the collective reads (their
// structure-of-arrays form is the collective's interface) AND checks them -- the tables are data
// written by earlier kernels, so a group whose sizes disagree with the launch's (N, K), whose row
// count or offsets are negative, or whose expert id is negative is given zero rows in a private copy
// of the problem sizes instead of being followed.
//
// Built only when CUTLASS headers are found (NVK_HAVE_CUTLASS); otherwise the entry points refuse.
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../csrc/nvk_common.cuh"

#ifdef NVK_HAVE_CUTLASS
#include "cutlass/cutlass.h"
#include "cute/tensor.hpp"
#include "cutlass/detail/sm100_blockscaled_layout.hpp"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/dispatch_policy.hpp"
#include "cutlass/gemm/group_array_problem_shape.hpp"
#include "cutlass/gemm/kernel/gemm_universal.hpp"

// A named namespace: CuTe has an unnamed one of its own, and a kernel in ours would be ambiguous
// next to `using namespace cute`.
namespace nvk_moe_grouped {

using namespace cute;

using GroupShape = cutlass::gemm::GroupProblemShape<Shape<int32_t, int32_t, int32_t>>;
using ElementAB = cutlass::nv_float4_t<cutlass::float_e2m1_t>;
using ElementD = cutlass::bfloat16_t;
using ElementAcc = float;
using LayoutA = cutlass::layout::RowMajor;      // activations [m, k], K contiguous
using LayoutB = cutlass::layout::ColumnMajor;   // weights [n, k] seen as a K x N column-major operand
using LayoutD = cutlass::layout::RowMajor;
constexpr int kAlignAB = 32;                    // elements: 16 bytes of packed e2m1
constexpr int kAlignD = 128 / cutlass::sizeof_bits<ElementD>::value;

using TileShape = Shape<_128, _128, _256>;
using ClusterShape = Shape<_1, _1, _1>;

// alpha comes from an array of per-group pointers; no C operand (beta = 0)
using Fusion = cutlass::epilogue::fusion::LinearCombination<ElementD, ElementAcc, ElementD, ElementAcc>;

using Epilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassBlockScaledTensorOp, TileShape, ClusterShape,
    cutlass::epilogue::collective::EpilogueTileAuto, ElementAcc, ElementAcc, ElementD, LayoutD*, kAlignD, ElementD,
    LayoutD*, kAlignD, cutlass::epilogue::PtrArrayTmaWarpSpecialized1Sm, Fusion>::CollectiveOp;
using Mainloop = typename cutlass::gemm::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassBlockScaledTensorOp, ElementAB, LayoutA*, kAlignAB, ElementAB,
    LayoutB*, kAlignAB, ElementAcc, TileShape, ClusterShape,
    cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epilogue::SharedStorage))>,
    cutlass::gemm::KernelPtrArrayTmaWarpSpecialized1SmNvf4Sm100>::CollectiveOp;
using GemmKernel = cutlass::gemm::kernel::GemmUniversal<GroupShape, Mainloop, Epilogue>;
using Gemm = cutlass::gemm::device::GemmUniversalAdapter<GemmKernel>;

using StrideA = typename GemmKernel::InternalStrideA;
using StrideB = typename GemmKernel::InternalStrideB;
using StrideD = typename GemmKernel::InternalStrideD;
using LayoutSFA = typename GemmKernel::CollectiveMainloop::InternalLayoutSFA;
using LayoutSFB = typename GemmKernel::CollectiveMainloop::InternalLayoutSFB;
using SfConfig = typename GemmKernel::CollectiveMainloop::Sm1xxBlkScaledConfig;
using ElemA = typename Gemm::ElementA;   // the packed e2m1 data type
using ElemB = typename Gemm::ElementB;
using ElemSF = typename GemmKernel::CollectiveMainloop::ElementSF;

// The per-group argument arrays, carved out of the caller's scratch buffer.
struct GroupArrays {
    const ElemA** a;
    const ElemB** b;
    ElementD** d;
    const ElemSF** sfa;
    const ElemSF** sfb;
    const float** alpha;
    StrideA* da;
    StrideB* db;
    StrideD* dd;
    LayoutSFA* lsfa;
    LayoutSFB* lsfb;
    int32_t* sizes;   // checked copy of the caller's (m, n, k) triples: what the GEMM actually reads
};

struct Carver {
    uint8_t* base;
    size_t off;
    template <typename T>
    T* take(int count) {
        off = (off + 127) & ~size_t{127};
        T* p = reinterpret_cast<T*>(base + off);
        off += sizeof(T) * (size_t)count;
        return p;
    }
};

GroupArrays carve(uint8_t* scratch, int groups, size_t* bytes) {
    Carver c{scratch, 0};
    GroupArrays g;
    g.a = c.take<const ElemA*>(groups);
    g.b = c.take<const ElemB*>(groups);
    g.d = c.take<ElementD*>(groups);
    g.sfa = c.take<const ElemSF*>(groups);
    g.sfb = c.take<const ElemSF*>(groups);
    g.alpha = c.take<const float*>(groups);
    g.da = c.take<StrideA>(groups);
    g.db = c.take<StrideB>(groups);
    g.dd = c.take<StrideD>(groups);
    g.lsfa = c.take<LayoutSFA>(groups);
    g.lsfb = c.take<LayoutSFB>(groups);
    g.sizes = c.take<int32_t>(3 * groups);
    *bytes = c.off;
    return g;
}

// One thread per group: routing tables -> checked problem size, pointers, strides and scale layouts.
__global__ void plan_groups_kernel(GroupArrays g, const uint8_t* a_packed, const uint8_t* a_scales,
                                   const uint8_t* b_packed, const uint8_t* b_scales, const float* alphas,
                                   uint16_t* d_bf16, const int32_t* expert_offsets, const int32_t* sf_offsets,
                                   const int32_t* problem_sizes, const int32_t* active_expert_indices, int groups,
                                   int launch_n, int launch_k, int64_t a_row_stride, int64_t b_row_stride,
                                   int64_t d_row_stride) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= groups) return;
    int m = problem_sizes[3 * i];
    const int n = launch_n, k = launch_k;
    int64_t row0 = expert_offsets[i];
    int64_t sf_row0 = sf_offsets[i];
    int64_t e = active_expert_indices ? active_expert_indices[i] : i;
    const bool sane = m >= 0 && problem_sizes[3 * i + 1] == n && problem_sizes[3 * i + 2] == k && row0 >= 0 &&
                      sf_row0 >= 0 && (sf_row0 & 127) == 0 && e >= 0;
    if (!sane) {   // an empty group at the start of the buffers: nothing is read or written for it
        m = 0;
        row0 = sf_row0 = e = 0;
    }
    g.sizes[3 * i] = m;
    g.sizes[3 * i + 1] = n;
    g.sizes[3 * i + 2] = k;
    const int64_t k_bytes = k / 2;                                   // packed bytes per row
    const int64_t sf_cols = (int64_t)((k / 16 + 3) / 4) * 4;          // scale bytes per row, padded to k-tiles
    const int64_t n_pad = (int64_t)((n + 127) / 128) * 128;
    g.a[i] = reinterpret_cast<const ElemA*>(a_packed + row0 * k_bytes);
    g.b[i] = reinterpret_cast<const ElemB*>(b_packed + e * n * k_bytes);
    g.d[i] = reinterpret_cast<ElementD*>(d_bf16 + row0 * n);
    g.sfa[i] = reinterpret_cast<const ElemSF*>(a_scales + sf_row0 * sf_cols);
    g.sfb[i] = reinterpret_cast<const ElemSF*>(b_scales + e * n_pad * sf_cols);
    g.alpha[i] = alphas + e;
    g.da[i] = cute::make_stride(a_row_stride, cute::_1{}, cute::_0{});
    g.db[i] = cute::make_stride(b_row_stride, cute::_1{}, cute::_0{});
    g.dd[i] = cute::make_stride(d_row_stride, cute::_1{}, cute::_0{});
    g.lsfa[i] = SfConfig::tile_atom_to_shape_SFA(cute::make_shape(m, n, k, 1));
    g.lsfb[i] = SfConfig::tile_atom_to_shape_SFB(cute::make_shape(m, n, k, 1));
}

int sm_count_of_current_device() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (cached[dev] == 0) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
    return cached[dev];
}

int run_grouped(void* stream, const void* a_packed, const void* a_scales, const void* b_packed, const void* b_scales,
                const float* alphas, void* d_bf16, const int32_t* expert_offsets, const int32_t* sf_offsets,
                const int32_t* problem_sizes, const int32_t* active_expert_indices, int N, int K, int num_groups,
                int64_t a_row_stride_elems, int64_t b_row_stride_elems, int64_t c_row_stride_elems, void* meta_scratch,
                size_t meta_scratch_bytes, void* gemm_workspace, size_t gemm_workspace_bytes,
                size_t* required_workspace) {
    if (num_groups <= 0 || N <= 0 || K <= 0) return NVK_ERR_SHAPE;
    if ((K % 32) != 0 || (N % 8) != 0) return NVK_ERR_SHAPE;   // 16-byte rows of packed operands and of D
    if (num_groups > 1024) return NVK_ERR_RESOURCE;
    try {
        size_t meta_need = 0;
        GroupArrays g = carve(static_cast<uint8_t*>(meta_scratch), num_groups, &meta_need);

        typename Gemm::Arguments args{};
        args.mode = cutlass::gemm::GemmUniversalMode::kGrouped;
        // the GEMM reads the checked copy of the sizes that plan_groups_kernel writes, not the caller's
        args.problem_shape = {num_groups, reinterpret_cast<typename GroupShape::UnderlyingProblemShape*>(g.sizes),
                              nullptr};
        args.mainloop.ptr_A = g.a;
        args.mainloop.dA = g.da;
        args.mainloop.ptr_B = g.b;
        args.mainloop.dB = g.db;
        args.mainloop.ptr_SFA = g.sfa;
        args.mainloop.layout_SFA = g.lsfa;
        args.mainloop.ptr_SFB = g.sfb;
        args.mainloop.layout_SFB = g.lsfb;
        args.epilogue.thread.alpha = 1.0f;
        args.epilogue.thread.beta = 0.0f;
        args.epilogue.thread.alpha_ptr_array = g.alpha;
        args.epilogue.thread.dAlpha = {cute::_0{}, cute::_0{}, 1};   // one alpha per group
        args.epilogue.ptr_C = nullptr;
        args.epilogue.dC = g.dd;
        args.epilogue.ptr_D = g.d;
        args.epilogue.dD = g.dd;
        args.hw_info.device_id = 0;
        cudaGetDevice(&args.hw_info.device_id);
        args.hw_info.sm_count = sm_count_of_current_device();

        const size_t need = Gemm::get_workspace_size(args);
        if (required_workspace) *required_workspace = need;
        // all data pointers null: a pure workspace query, nothing is launched
        if (!a_packed && !b_packed && !d_bf16) return 0;
        if (nvk::any_null(a_packed, a_scales, b_packed, b_scales, alphas, d_bf16, expert_offsets, sf_offsets,
                          problem_sizes))
            return NVK_ERR_ARG;
        if (!meta_scratch || meta_scratch_bytes < 64 * 1024) return -10;   // the reference's minimum
        if (meta_scratch_bytes < meta_need) return -11;
        if (need > gemm_workspace_bytes || (need > 0 && !gemm_workspace)) return -12;

        cudaStream_t s = (cudaStream_t)stream;
        if (int rc = nvk::launch(nvk::launch_1d(s, (unsigned)((num_groups + 127) / 128), 128), plan_groups_kernel, g,
                                 static_cast<const uint8_t*>(a_packed), static_cast<const uint8_t*>(a_scales),
                                 static_cast<const uint8_t*>(b_packed), static_cast<const uint8_t*>(b_scales), alphas,
                                 static_cast<uint16_t*>(d_bf16), expert_offsets, sf_offsets, problem_sizes,
                                 active_expert_indices, num_groups, N, K, a_row_stride_elems, b_row_stride_elems,
                                 c_row_stride_elems))
            return rc;

        Gemm gemm;
        if (gemm.can_implement(args) != cutlass::Status::kSuccess) return -13;
        if (gemm.initialize(args, gemm_workspace, s) != cutlass::Status::kSuccess) return -14;
        if (gemm.run(s) != cutlass::Status::kSuccess) return -15;
        return 0;
    } catch (...) {
        return NVK_ERR_SHAPE;
    }
}

}  // namespace nvk_moe_grouped
#else   // !NVK_HAVE_CUTLASS
namespace nvk_moe_grouped {
int run_grouped(void*, const void*, const void*, const void*, const void*, const float*, void*, const int32_t*,
                const int32_t*, const int32_t*, const int32_t*, int, int, int, int64_t, int64_t, int64_t, void*, size_t,
                void*, size_t, size_t* required_workspace) {
    if (required_workspace) *required_workspace = 0;
    return NVK_ERR_SHAPE;
}
}  // namespace nvk_moe_grouped
#endif

using nvk_moe_grouped::run_grouped;

extern "C" {

// The reference names these after the architecture of its own kernels and builds two tile shapes (a
// prefill one and a narrower decode one); both symbols are kept so that its call sites bind
// unchanged, and both run the same sm_100a kernel, whose 128-row MMA is the smallest the hardware
// offers for this operand type.
int nv_kernels_cutlass_moe_grouped_fp4_gemm_sm120_bf16(
    void* stream, const void* a_packed, const void* a_scales, const void* b_packed, const void* b_scales,
    const float* alphas, void* d_bf16, const int32_t* expert_offsets, const int32_t* sf_offsets,
    const int32_t* problem_sizes, const int32_t* active_expert_indices, int N, int K, int num_experts,
    int64_t a_row_stride_elems, int64_t b_row_stride_elems, int64_t c_row_stride_elems, void* meta_scratch,
    size_t meta_scratch_bytes, void* gemm_workspace, size_t gemm_workspace_bytes, size_t* required_workspace) {
    return run_grouped(stream, a_packed, a_scales, b_packed, b_scales, alphas, d_bf16, expert_offsets, sf_offsets,
                       problem_sizes, active_expert_indices, N, K, num_experts, a_row_stride_elems,
                       b_row_stride_elems, c_row_stride_elems, meta_scratch, meta_scratch_bytes, gemm_workspace,
                       gemm_workspace_bytes, required_workspace);
}

int nv_kernels_cutlass_moe_grouped_fp4_gemm_sm120_bf16_decode(
    void* stream, const void* a_packed, const void* a_scales, const void* b_packed, const void* b_scales,
    const float* alphas, void* d_bf16, const int32_t* expert_offsets, const int32_t* sf_offsets,
    const int32_t* problem_sizes, const int32_t* active_expert_indices, int N, int K, int num_experts,
    int64_t a_row_stride_elems, int64_t b_row_stride_elems, int64_t c_row_stride_elems, void* meta_scratch,
    size_t meta_scratch_bytes, void* gemm_workspace, size_t gemm_workspace_bytes, size_t* required_workspace) {
    return run_grouped(stream, a_packed, a_scales, b_packed, b_scales, alphas, d_bf16, expert_offsets, sf_offsets,
                       problem_sizes, active_expert_indices, N, K, num_experts, a_row_stride_elems,
                       b_row_stride_elems, c_row_stride_elems, meta_scratch, meta_scratch_bytes, gemm_workspace,
                       gemm_workspace_bytes, required_workspace);
}

}  // extern "C"
