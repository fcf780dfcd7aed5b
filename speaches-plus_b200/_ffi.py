"""ctypes binding of libnvk_b200.so: one Python function per C symbol of include/nvk_b200.h.

Pointers are passed as integers (`tensor.data_ptr()`), the stream as the integer value of a
cudaStream_t.  Nothing here computes: a missing library or symbol raises at import/first use.
"""
from __future__ import annotations

import ctypes as C
import pathlib

_HERE = pathlib.Path(__file__).resolve().parent
LIB_PATH = _HERE / "libnvk_b200.so"
PREFILL_LIB_PATH = _HERE / "libnvk_b200_prefill.so"  # the prefill GEMM lives in a library of its own

_vp, _i, _f, _ll = C.c_void_p, C.c_int, C.c_float, C.c_longlong

# name -> argument types (every function returns int)
SIGNATURES = {
    "nv_kernels_capability": [_vp, _vp],
    "nv_kernels_nvfp4_gemv_bf16act": [_vp, _vp, _vp, _vp, _vp, _f, _i, _i],
    "nv_kernels_nvfp4_gemv_bf16": [_vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i],
    "nv_kernels_gemv_nvfp4_w4a16_dual_m1": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _f, _i, _i],
    "nv_kernels_gemv_nvfp4_w4a16_silu_gate_up_in_m1": [_vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i],
    "nv_kernels_gemm_nvfp4_w4a16_mk_dual": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _f, _i, _i, _i],
    "nvk_b200_linear_nvfp4_w4a16": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _f, _i, _i, _i],
    "nvk_b200_linear_nvfp4_w4a16_ws": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _f, _i, _i, _i, _vp, C.c_size_t],
    "nvk_b200_linear_workspace_bytes": [_i, _i],
    "nvk_b200_stack_plan_bytes": [_i],
    "nvk_b200_stack_build": [_vp, _i, _i, _vp, C.c_size_t, _vp],
    "nvk_b200_stack_run": [_vp, _vp, _i, _i, _i, _i, _vp],
    "nvk_b200_linear_nvfp4_w4a16_residual": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i, _i],
    "nvk_b200_linear_nvfp4_w4a16_residual_rstd_emit": [_vp] * 7 + [_f, _vp, _f, _i, _i],
    "nvk_b200_linear_nvfp4_w4a16_normed": [_vp] * 8 + [_f, _vp, _vp, _f, _f, _i, _i, _i],
    "nvk_b200_tp_linear_nvfp4_w4a16_allreduce": [_vp, _vp, _i, _i] + [_vp] * 6 + [_f, _i, _i, _i, _i, _i, _vp, _vp],
    "nvk_b200_tp_fused_buffer_bytes": [_i, _i, _i],
    "nvk_b200_moe_combine_allreduce": [_vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _i, _vp, _vp],
    "nvk_b200_moe_combine_buffer_bytes": [_i, _i],
    "nvk_b200_set_tuning": [_i, _i],
    "nvk_b200_set_row_balance": [_i],
    "nvk_b200_row_balance_grid": [_i, C.c_size_t, _i],
    "nvk_b200_set_pdl": [_i],
    "nvk_b200_set_wait_limit": [C.c_uint],
    "nv_kernels_gemv_bf16": [_vp, _vp, _vp, _vp, _i, _i],
    "nvk_b200_linear_bf16": [_vp, _vp, _vp, _vp, _i, _i, _i],
    "nv_kernels_quantize_nvfp4_bf16": [_vp, _vp, _vp, _vp, _f, _i, _i, _i],
    "nv_kernels_quantize_nvfp4_bf16_rows": [_vp, _vp, _vp, _vp, _f, _i, _i],
    "nv_kernels_nvfp4_quantize_row_bf16": [_vp, _vp, _vp, _vp, _f, _i],
    "nv_kernels_quantize_nvfp4_bf16_per_expert": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i],
    "nv_kernels_quantize_nvfp4_bf16_per_expert_strided": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i],
    "nv_kernels_silu_mul_quantize_nvfp4_bf16_per_expert": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i],
    "nv_kernels_silu_mul_quantize_nvfp4_bf16_per_expert_strided": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i],
    "nv_kernels_rmsnorm_bf16": [_vp, _vp, _vp, _vp, C.c_size_t, C.c_size_t, _f],
    "nv_kernels_rmsnorm_quantize_nvfp4_bf16": [_vp, _vp, _vp, _vp, _vp, _f, _f, _i, _i, _i],
    "nv_kernels_moe_route_topk": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _f],
    "nv_kernels_moe_route_topk_shared_tail": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _f, _i],
    "nv_kernels_gather_rows_bf16": [_vp, _vp, _vp, _vp, _i, _i, _i],
    "nv_kernels_gather_rows_bf16_strided": [_vp, _vp, _vp, _vp, _i, _i, _i, _i],
    "nv_kernels_gather_f32_by_ids": [_vp, _vp, _vp, _vp, _i],
    "nv_kernels_moe_unpermute_scatter": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i],
    "nv_kernels_moe_unpermute_scatter_tail": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i],
    "nv_kernels_mul_sigmoid_rowgate_f32": [_vp, _vp, _vp, _vp, _i, _i],
    "nv_kernels_moe_permute": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i],
    "nvk_b200_moe_grouped_w4a16": [_vp] * 15 + [_i, _i, _i, _i, _i, _vp],
    "nvk_b200_tp_allreduce_buffer_bytes": [_i, _i],
    "nvk_b200_tp_buffer_alloc": [C.c_size_t, _vp],
    "nvk_b200_tp_buffer_free": [_vp],
    "nvk_b200_tp_ipc_export": [_vp, _vp],
    "nvk_b200_tp_ipc_open": [_vp, _vp],
    "nvk_b200_tp_ipc_close": [_vp],
    "nvk_b200_tp_allreduce_bf16": [_vp, _vp, _i, _i, _vp, _vp, _i, _i, _vp, _vp],
    "nvk_b200_moe_route_permute": [_vp] * 10 + [_i, _i, _i, _i, _f, _i, _f],
    "nvk_b200_moe_combine": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "nv_kernels_moe_route_gather_quant_m1": [_vp] * 12 + [_i, _i, _i, _f, _i, _f, _i, _i, _i],
    "nv_kernels_prof_timestamp": [_vp, _vp],
    "nv_kernels_gemv_nvfp4_w4a8_dual_m1": [_vp] * 9 + [_f, _f, _i, _i],
    "nv_kernels_gemv_nvfp4_w4a8_dual_mk": [_vp] * 9 + [_f, _f, _i, _i, _i],
    "nv_kernels_gemv_nvfp4_w4a8_down_residual_m1": [_vp] * 7 + [_f, _i, _i],
    "nv_kernels_gemv_nvfp4_w4a8_down_residual_m1_rstd_emit": [_vp] * 7 + [_f, _vp, _f, _i, _i],
    "nv_kernels_gemv_nvfp4_w4a8_down_residual_mk": [_vp] * 7 + [_f, _i, _i, _i],
    "nv_kernels_gemv_nvfp4_w4a8_down_residual_quant_prologue_m1": [_vp] * 5 + [_i, _vp, _vp, _f, _i, _i],
    "nv_kernels_silu_mul_rowquant_i8_m1": [_vp] * 5 + [_i],
    "nv_kernels_silu_mul_rowquant_i8_mk_partials_len": [_i, _i],
    "nv_kernels_silu_mul_rowquant_i8_mk": [_vp] * 7 + [_i, _i],
    "nv_kernels_silu_mul_stage_partial_absmax_m1": [_vp] * 5 + [_i],
    "nv_kernels_rmsnorm_residual_writeout_rowquant_i8_m1": [_vp] * 7 + [_i, _f],
    "nv_kernels_rmsnorm_residual_writeout_bf16": [_vp] * 6 + [C.c_size_t, C.c_size_t, _f],
    "nvk_b200_moe_permute_static": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i],
    "nv_kernels_moe_grouped_fp4_gemv_m1_bf16": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _ll],
}

# symbols exported by the prefill library
PREFILL_SIGNATURES = {
    "nvk_b200_set_prefill_config": [_i],
    "nvk_b200_cublaslt_fp4_gemm_bf16": [_vp] * 6 + [_i, _i, _i, _f, _vp, C.c_size_t],
    "nvk_b200_cublaslt_fp4_workspace_bytes": [],
    "nv_kernels_cutlass_fp4_gemm_sm120_bf16": [_vp] * 7 + [_i, _i, _i, _vp, C.c_size_t, _vp],
    "nv_kernels_cutlass_fp4_gemm_sm120_bf16_streamk": [_vp] * 7 + [_i, _i, _i, _vp, C.c_size_t, _vp],
    "nv_kernels_cutlass_fp4_gemm_sm120_bf16_tiled": [_vp] * 7 + [_i, _i, _i, _i, _i, _vp, C.c_size_t, _vp],
    "nv_kernels_cutlass_moe_grouped_fp4_gemm_sm120_bf16":
        [_vp] * 11 + [_i, _i, _i, _ll, _ll, _ll, _vp, C.c_size_t, _vp, C.c_size_t, _vp],
    "nv_kernels_cutlass_moe_grouped_fp4_gemm_sm120_bf16_decode":
        [_vp] * 11 + [_i, _i, _i, _ll, _ll, _ll, _vp, C.c_size_t, _vp, C.c_size_t, _vp],
}



class NvkStackOp(C.Structure):
    """One linear of a persistent decode step (include/nvk_b200.h: NvkStackOp)."""
    _fields_ = [("wq_a", _vp), ("sc_a", _vp), ("wq_b", _vp), ("sc_b", _vp), ("x", _vp), ("x2", _vp), ("y_a", _vp),
                ("y_b", _vp), ("alpha_a", _f), ("alpha_b", _f), ("N", _i), ("K", _i), ("dep", _i),
                ("rows_per_item", _i)]


_lib = None
EMULATED = False   # set by the test harness when it points this binding at the host emulation
_prefill_lib = None


class NvkError(RuntimeError):
    """A launcher returned a non-zero status."""

    def __init__(self, name: str, rc: int):
        self.name, self.rc = name, rc
        kind = {-1: "shape/route refused", -2: "bad argument or alignment", -3: "resource limit",
                -9: "grid axis too large"}.get(rc, "cudaError_t" if rc > 0 else "error")
        super().__init__(f"{name} returned {rc} ({kind})")


def lib() -> C.CDLL:
    """Load the CUDA library.  There is no fallback: a missing build is an error."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python speaches-plus_b200/build.py` "
                "(this package has no CPU or PyTorch fallback)")
        L = C.CDLL(str(LIB_PATH))
        for name, args in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if a declared symbol is not exported
            fn.argtypes = args
            fn.restype = C.c_size_t if name.endswith("_bytes") else C.c_int
        _lib = L
    return _lib


class MultiGpuRefused(RuntimeError):
    """The prefill library was asked for in a process that is one rank of several."""


def distributed_world() -> int:
    """Ranks this process is one of: the size of torch.distributed's default group once it exists,
    else what the launcher's WORLD_SIZE says, else 1."""
    import os
    import sys
    td = sys.modules.get("torch.distributed")
    if td is not None and td.is_available() and td.is_initialized():
        return int(td.get_world_size())
    try:
        return max(1, int(os.environ.get("WORLD_SIZE", "1")))
    except ValueError:
        return 1


def _refuse_prefill_on_several_gpus(what: str) -> None:
    """libnvk_b200_prefill.so holds a 2-SM tile whose TMA operand loads use cluster multicast.  Its
    tensor maps are built over this GPU's own memory only, and it stays that way because no process
    that is one rank of a multi-GPU job may load or call the library at all: tensor- and
    expert-parallel code keeps M > 64 on the decode-sized kernels of libnvk_b200.so."""
    world = distributed_world()
    if world > 1:
        raise MultiGpuRefused(
            f"{what}: libnvk_b200_prefill.so is for single-GPU processes only (this process is one of "
            f"{world} ranks); multi-GPU code runs rows in chunks of 64 on libnvk_b200.so instead")


def prefill_available() -> bool:
    return PREFILL_LIB_PATH.exists() and distributed_world() == 1


def prefill_lib() -> C.CDLL:
    """Load the prefill-GEMM library.  A missing build is an error, not a fallback; so is asking for
    it from one rank of a multi-GPU job."""
    global _prefill_lib
    _refuse_prefill_on_several_gpus("prefill_lib()")
    if _prefill_lib is None:
        if not PREFILL_LIB_PATH.exists():
            raise RuntimeError(
                f"{PREFILL_LIB_PATH} is missing: the prefill (M > 64) route needs it; build it with "
                "`python speaches-plus_b200/build.py` (needs CUTLASS headers; there is no fallback)")
        L = C.CDLL(str(PREFILL_LIB_PATH))
        for name, args in PREFILL_SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = C.c_size_t if name.endswith("_bytes") else C.c_int
        _prefill_lib = L
    return _prefill_lib


def call(name: str, *args) -> int:
    """Call a launcher and return its raw status."""
    if name in PREFILL_SIGNATURES:
        _refuse_prefill_on_several_gpus(name)
        return int(getattr(prefill_lib(), name)(*args))
    return int(getattr(lib(), name)(*args))


def check(name: str, *args) -> None:
    """Call a launcher; raise NvkError on a non-zero status."""
    rc = call(name, *args)
    if rc != 0:
        raise NvkError(name, rc)


def capability() -> tuple[int, int]:
    a, b = C.c_int(0), C.c_int(0)
    rc = int(lib().nv_kernels_capability(C.addressof(a), C.addressof(b)))
    if rc != 0:
        raise NvkError("nv_kernels_capability", rc)
    return a.value, b.value
