// The library route of the prefill-sized NVFP4 GEMM: the same contraction as prefill_fp4_gemm.cu,
//
//   D[m, n] = bf16( alpha * sum_k A[m, k] * B[n, k] ),  packed e2m1 operands, one ue4m3 scale per 16
//   values along K in the 128x4 swizzled layout,
//
// handed to cuBLASLt as a CUDA_R_4F_E2M1 x CUDA_R_4F_E2M1 matmul with VEC16_UE4M3 block scaling -- what
// the reference's runner does when its backend is "cublaslt" (rust/crates/nv-quant/src/nvfp4.rs:866-1067:
// TN operands, weights as the library's A, a 64 MiB workspace, one descriptor per shape, the scale
// pointers set on every call).  Nothing here is a kernel of this library; the file is the binding.
//
// cuBLASLt is opened at run time (dlopen of libcublasLt.so.12, which a process that already uses
// cuBLAS has mapped); without it every call returns NVK_ERR_RESOURCE.  Operands must be this GPU's own
// memory and the process single-GPU, like the rest of this library.
#include <cublasLt.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stddef.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <tuple>

#include "../csrc/nvk_common.cuh"

namespace {

// cuBLASLt's status, folded into this library's negative codes: -100 - status.
inline int lt_error(cublasStatus_t st) { return -100 - (int)st; }

struct LtApi {
    void* so = nullptr;
    decltype(&cublasLtCreate) create = nullptr;
    decltype(&cublasLtMatmulDescCreate) desc_create = nullptr;
    decltype(&cublasLtMatmulDescDestroy) desc_destroy = nullptr;
    decltype(&cublasLtMatmulDescSetAttribute) desc_set = nullptr;
    decltype(&cublasLtMatrixLayoutCreate) layout_create = nullptr;
    decltype(&cublasLtMatrixLayoutDestroy) layout_destroy = nullptr;
    decltype(&cublasLtMatmulPreferenceCreate) pref_create = nullptr;
    decltype(&cublasLtMatmulPreferenceDestroy) pref_destroy = nullptr;
    decltype(&cublasLtMatmulPreferenceSetAttribute) pref_set = nullptr;
    decltype(&cublasLtMatmulAlgoGetHeuristic) heuristic = nullptr;
    decltype(&cublasLtMatmul) matmul = nullptr;
    bool ok = false;
};

template <class F>
bool bind(void* so, const char* name, F& fn) {
    fn = reinterpret_cast<F>(dlsym(so, name));
    return fn != nullptr;
}

const LtApi& lt_api() {
    static LtApi api = [] {
        LtApi a;
        for (const char* name : {"libcublasLt.so.12", "libcublasLt.so"}) {
            a.so = dlopen(name, RTLD_NOW | RTLD_LOCAL);
            if (a.so != nullptr) break;
        }
        if (a.so == nullptr) return a;
        a.ok = bind(a.so, "cublasLtCreate", a.create) && bind(a.so, "cublasLtMatmulDescCreate", a.desc_create) &&
               bind(a.so, "cublasLtMatmulDescDestroy", a.desc_destroy) &&
               bind(a.so, "cublasLtMatmulDescSetAttribute", a.desc_set) &&
               bind(a.so, "cublasLtMatrixLayoutCreate", a.layout_create) &&
               bind(a.so, "cublasLtMatrixLayoutDestroy", a.layout_destroy) &&
               bind(a.so, "cublasLtMatmulPreferenceCreate", a.pref_create) &&
               bind(a.so, "cublasLtMatmulPreferenceDestroy", a.pref_destroy) &&
               bind(a.so, "cublasLtMatmulPreferenceSetAttribute", a.pref_set) &&
               bind(a.so, "cublasLtMatmulAlgoGetHeuristic", a.heuristic) && bind(a.so, "cublasLtMatmul", a.matmul);
        return a;
    }();
    return api;
}

// One plan per (device, m, n, k, workspace size): descriptor, layouts and the heuristic's first algorithm.
struct Plan {
    cublasLtMatmulDesc_t desc = nullptr;
    cublasLtMatrixLayout_t weights = nullptr, acts = nullptr, out = nullptr;
    cublasLtMatmulAlgo_t algo;
};

constexpr int kMaxDevices = 64;

struct LtState {
    std::mutex mu;
    cublasLtHandle_t handle[kMaxDevices] = {};
    std::map<std::tuple<int, int, int, int, size_t>, Plan> plans;
};
LtState& lt_state() {
    static LtState s;
    return s;
}

template <class T>
cublasStatus_t set_desc(const LtApi& lt, cublasLtMatmulDesc_t d, cublasLtMatmulDescAttributes_t attr, const T& v) {
    return lt.desc_set(d, attr, &v, sizeof(T));
}

void drop(const LtApi& lt, Plan& p) {
    if (p.weights) lt.layout_destroy(p.weights);
    if (p.acts) lt.layout_destroy(p.acts);
    if (p.out) lt.layout_destroy(p.out);
    if (p.desc) lt.desc_destroy(p.desc);
    p = Plan();
}

int make_plan(const LtApi& lt, cublasLtHandle_t handle, int m, int n, int k, size_t ws_bytes, Plan& p) {
    cublasStatus_t st;
#define LT_TRY(expr)                                                                                          \
    if ((st = (expr)) != CUBLAS_STATUS_SUCCESS) {                                                             \
        drop(lt, p);                                                                                          \
        return lt_error(st);                                                                                  \
    }
    // Column-major view: D^T [n, m] = W [n, k] * X^T [k, m].  W (row-major [n, k]) is a k x n matrix
    // with leading dimension k, transposed; X (row-major [m, k]) a k x m matrix, not transposed.
    LT_TRY(lt.desc_create(&p.desc, CUBLAS_COMPUTE_32F, CUDA_R_32F));
    LT_TRY(set_desc(lt, p.desc, CUBLASLT_MATMUL_DESC_TRANSA, CUBLAS_OP_T));
    LT_TRY(set_desc(lt, p.desc, CUBLASLT_MATMUL_DESC_TRANSB, CUBLAS_OP_N));
    LT_TRY(set_desc(lt, p.desc, CUBLASLT_MATMUL_DESC_A_SCALE_MODE, CUBLASLT_MATMUL_MATRIX_SCALE_VEC16_UE4M3));
    LT_TRY(set_desc(lt, p.desc, CUBLASLT_MATMUL_DESC_B_SCALE_MODE, CUBLASLT_MATMUL_MATRIX_SCALE_VEC16_UE4M3));
    LT_TRY(lt.layout_create(&p.weights, CUDA_R_4F_E2M1, (uint64_t)k, (uint64_t)n, (int64_t)k));
    LT_TRY(lt.layout_create(&p.acts, CUDA_R_4F_E2M1, (uint64_t)k, (uint64_t)m, (int64_t)k));
    LT_TRY(lt.layout_create(&p.out, CUDA_R_16BF, (uint64_t)n, (uint64_t)m, (int64_t)n));

    cublasLtMatmulPreference_t pref = nullptr;
    LT_TRY(lt.pref_create(&pref));
    st = lt.pref_set(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ws_bytes, sizeof(ws_bytes));
    cublasLtMatmulHeuristicResult_t heur;
    int returned = 0;
    if (st == CUBLAS_STATUS_SUCCESS)
        st = lt.heuristic(handle, p.desc, p.weights, p.acts, p.out, p.out, pref, 1, &heur, &returned);
    lt.pref_destroy(pref);
    if (st == CUBLAS_STATUS_SUCCESS && (returned < 1 || heur.state != CUBLAS_STATUS_SUCCESS))
        st = CUBLAS_STATUS_NOT_SUPPORTED;
    LT_TRY(st);
#undef LT_TRY
    p.algo = heur.algo;
    return 0;
}

}  // namespace

extern "C" {

// Workspace the library route is given by the reference's runner (nvfp4.rs:377): 64 MiB per stream.
size_t nvk_b200_cublaslt_fp4_workspace_bytes(void) { return (size_t)64 << 20; }

// d [m, n] bf16 = alpha * a [m, k] * b [n, k]^T through cuBLASLt.  a/b packed e2m1 (k/2 bytes per row),
// a_scales/b_scales their 128x4-swizzled ue4m3 block scales, alpha a host value (the reference passes
// its host copy on this route).  Refusals follow the reference's (nvfp4.rs:564-590): k % 16, and m, n, k
// at least 128 for the library route; -2 for null or misaligned operands; -3 when cuBLASLt cannot be
// opened or no handle can be made; -100 - status for a cuBLASLt status (no algorithm for the shape is
// -115).  Safe to call from several threads; capturable once the shape's plan exists (first call).
int nvk_b200_cublaslt_fp4_gemm_bf16(void* stream, const uint8_t* a_packed, const uint8_t* a_scales,
                                    const uint8_t* b_packed, const uint8_t* b_scales, uint16_t* d, int m, int n,
                                    int k, float alpha, void* workspace, size_t workspace_bytes) {
    if (m == 0 || n == 0) return 0;
    if (m < 0 || n < 0 || k <= 0 || (k & 15) != 0) return NVK_ERR_SHAPE;
    if (m < 128 || n < 128 || k < 128) return NVK_ERR_SHAPE;
    if (nvk::any_null(a_packed, a_scales, b_packed, b_scales, d)) return NVK_ERR_ARG;
    if (workspace == nullptr && workspace_bytes != 0) return NVK_ERR_ARG;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(a_packed) | reinterpret_cast<uintptr_t>(b_packed) |
                           reinterpret_cast<uintptr_t>(a_scales) | reinterpret_cast<uintptr_t>(b_scales) |
                           reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(workspace);
    if ((bits & 15u) != 0) return NVK_ERR_ARG;

    const LtApi& lt = lt_api();
    if (!lt.ok) return NVK_ERR_RESOURCE;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return NVK_ERR_RESOURCE;

    LtState& s = lt_state();
    Plan plan;
    cublasLtHandle_t handle;
    {
        std::lock_guard<std::mutex> lock(s.mu);
        if (s.handle[dev] == nullptr && lt.create(&s.handle[dev]) != CUBLAS_STATUS_SUCCESS) {
            s.handle[dev] = nullptr;
            return NVK_ERR_RESOURCE;
        }
        handle = s.handle[dev];
        const auto key = std::make_tuple(dev, m, n, k, workspace_bytes);
        auto it = s.plans.find(key);
        if (it == s.plans.end()) {
            Plan fresh;
            if (int rc = make_plan(lt, handle, m, n, k, workspace_bytes, fresh)) return rc;
            it = s.plans.emplace(key, fresh).first;
        }
        // The scale pointers live in the descriptor: set them and launch under the lock, so that two
        // threads sharing a shape cannot swap each other's pointers between the two steps.
        plan = it->second;
        const void* w_sf = b_scales;
        const void* x_sf = a_scales;
        cublasStatus_t st = set_desc(lt, plan.desc, CUBLASLT_MATMUL_DESC_A_SCALE_POINTER, w_sf);
        if (st == CUBLAS_STATUS_SUCCESS) st = set_desc(lt, plan.desc, CUBLASLT_MATMUL_DESC_B_SCALE_POINTER, x_sf);
        const float beta = 0.f;
        if (st == CUBLAS_STATUS_SUCCESS)
            st = lt.matmul(handle, plan.desc, &alpha, b_packed, plan.weights, a_packed, plan.acts, &beta, d, plan.out,
                           d, plan.out, &plan.algo, workspace, workspace_bytes, (cudaStream_t)stream);
        if (st != CUBLAS_STATUS_SUCCESS) return lt_error(st);
    }
    return 0;
}

}  // extern "C"
