"""The reference's backend registry (rust/crates/nv-layers/src/backend.rs:14-233), as far as this
library takes part in it: one backend -- `BackendKind.CUDA` -- and the kernel ids of the NVFP4 linear
path it implements.  `BackendSel` parses the reference's NV_KERNELS_BACKEND values; selecting wgpu or
cpu is an error here (there is no second backend and no fallback), `auto` means cuda."""
from __future__ import annotations

import enum
import os

BACKEND_ENV = "NV_KERNELS_BACKEND"


class BackendError(RuntimeError):
    pass


class BackendKind(enum.Enum):
    CUDA = "cuda"
    WGPU = "wgpu"
    CPU = "cpu"

    def __str__(self) -> str:
        return self.value


class BackendSel(enum.Enum):
    AUTO = "auto"
    CUDA = "cuda"
    WGPU = "wgpu"
    CPU = "cpu"

    @classmethod
    def parse(cls, s: str):
        v = s.strip().lower()
        if v == "":
            return cls.AUTO
        try:
            return cls(v)
        except ValueError:
            return None

    @classmethod
    def from_env(cls, env=None) -> "BackendSel":
        env = os.environ if env is None else env
        if BACKEND_ENV not in env:
            return cls.AUTO
        sel = cls.parse(env[BACKEND_ENV])
        if sel is None:
            raise BackendError(f"{BACKEND_ENV}={env[BACKEND_ENV]!r} is not one of auto|cuda|wgpu|cpu")
        return sel


class KernelId(enum.Enum):
    """The reference's ids for the kernels of this path (backend.rs:72-105, names as in :160-200)."""
    GATHER_ROWS_BF16 = "gather_rows_bf16"
    RMSNORM = "rmsnorm"
    RMSNORM_RESIDUAL = "rmsnorm_residual"
    GEMV_BF16 = "gemv_bf16"
    GEMV_W4A16 = "gemv_w4a16"
    GEMV_NVFP4 = "gemv_nvfp4"
    GEMM_NVFP4 = "gemm_nvfp4"
    QUANTIZE_NVFP4_BF16 = "quantize_nvfp4_bf16"
    MOE_PERMUTE = "moe_permute"
    MOE_UNPERMUTE_SCATTER = "moe_unpermute_scatter"
    MOE_GROUPED_GEMM_NVFP4 = "moe_grouped_fp4_gemm"


# which library serves an id
_PREFILL_IDS = {KernelId.GEMM_NVFP4, KernelId.MOE_GROUPED_GEMM_NVFP4}


def kind_supports(kind: BackendKind, kernel: KernelId) -> bool:
    """Cuda serves every id of the path; this library has no wgpu or cpu backend."""
    return kind is BackendKind.CUDA and isinstance(kernel, KernelId)


def missing_on(kind: BackendKind, needed) -> list:
    return [k for k in needed if not kind_supports(kind, k)]


def supporting_backends(kernel: KernelId) -> list:
    return [b for b in BackendKind if kind_supports(b, kernel)]


def resolve(sel: BackendSel | None = None) -> BackendKind:
    """The backend a selection means here: auto and cuda are cuda; anything else is refused."""
    sel = BackendSel.from_env() if sel is None else sel
    if sel in (BackendSel.AUTO, BackendSel.CUDA):
        return BackendKind.CUDA
    raise BackendError(f"backend {sel.value!r} is not part of this library: the NVFP4 linear path runs on "
                       "BackendKind::Cuda only (no CPU or wgpu fallback)")


def library_for(kernel: KernelId) -> str:
    """The shared object that exports the entry points behind an id."""
    return "libnvk_b200_prefill.so" if kernel in _PREFILL_IDS else "libnvk_b200.so"
