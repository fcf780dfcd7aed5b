"""Host-side mirror of the reference's `Nvfp4GemmRunner` (rust/crates/nv-quant/src/nvfp4.rs:359-1084) for
the prefill-sized FP4 x FP4 GEMM: which scheduler a shape gets, the per-stream workspace created ahead of
graph capture, and the environment knobs, over this library's three GEMM entry points.

Two backends, as in the reference: this library's block-scaled tensor-core GEMM (`cutlass`, and what
`auto` picks for every shape) and cuBLASLt's FP4 matmul (`cublaslt`, only when asked for: the reference's
automatic reroute of skinny shapes to it is answered by the stream-K scheduler here).  Single-GPU
processes only (the prefill library refuses to load in a rank of several).
"""
from __future__ import annotations

import ctypes as C
import enum
import os
import threading

import torch

from . import _ffi

WORKSPACE_BYTES = 64 * 1024 * 1024      # per stream (nvfp4.rs:377)
TILE_M = TILE_N = 128                   # the tile the scheduler rule counts in (nvfp4.rs:365-367)
MIN_TILE = 128                          # smallest n, k of any route and smallest m of the library route
SM_COUNT = 148                          # B200


# ---- environment knobs: the reference's parsers, name for name (nvfp4.rs:213-229, 424-463) ------------
def skinny_lt_from(raw):
    return raw != "0"


def k256_from(raw):
    return raw != "0"


def streamk_k256_from(raw):
    return raw is not None and raw != "" and raw != "0"


def streamk_down_splits_from(raw) -> int:
    try:
        s = int(raw.strip()) if raw is not None else 0
    except ValueError:
        return 0
    return s if s >= 2 else 0


class StreamkMode(enum.Enum):
    NEVER = 0
    ALWAYS = 1
    AUTO = 2


def streamk_mode_from(raw) -> StreamkMode:
    return {"0": StreamkMode.NEVER, "1": StreamkMode.ALWAYS}.get(raw, StreamkMode.AUTO)


class Nvfp4Backend(enum.Enum):
    CUBLASLT = "cublaslt"
    CUTLASS = "cutlass"
    AUTO = "auto"

    @classmethod
    def from_env(cls, raw=None) -> "Nvfp4Backend":
        raw = os.environ.get("SPEACHES_NVFP4_BACKEND") if raw is None else raw
        v = (raw or "auto").strip().lower()
        if v in ("cublaslt", "cublas"):
            return cls.CUBLASLT
        if v == "cutlass":
            return cls.CUTLASS
        return cls.AUTO      # unrecognised values fall back to auto, as the reference does


# ---- scheduler rule ---------------------------------------------------------------------------------------
def skinny_tiles(m: int, n: int) -> bool:
    """The reference's rule (nvfp4.rs:667-671): few enough output tiles that a data-parallel launch
    leaves SMs idle."""
    return -(-m // TILE_M) * -(-n // TILE_N) <= 192


def ragged_last_wave(m: int, n: int, sms: int = SM_COUNT) -> bool:
    """This library's addition for a 148-SM part: at most eight waves of output tiles of which the last
    is at most half full (M = 2048, N = 5120: 640 tiles = 4 waves + 48 tiles)."""
    tiles = -(-m // TILE_M) * -(-n // TILE_N)
    full, rest = divmod(tiles, sms)
    return 0 < rest <= sms // 2 and full < 8


# ---- per-stream workspaces ----------------------------------------------------------------------------------
_WORKSPACES: dict = {}


def _stream_key() -> tuple:
    return (torch.cuda.current_device(), torch.cuda.current_stream().cuda_stream)


def ensure_workspace_for_stream() -> torch.Tensor:
    """The current stream's 64 MiB workspace, created on first use -- which must not be inside a graph
    capture (nvfp4.rs:391-409): call this on the capture stream before capturing."""
    key = _stream_key()
    ws = _WORKSPACES.get(key)
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(f"nvfp4 workspace for stream {key[1]:#x} must be created before graph capture "
                               "(call ensure_workspace_for_stream on the capture stream first)")
        ws = torch.zeros(WORKSPACE_BYTES, dtype=torch.uint8, device=f"cuda:{key[0]}")
        _WORKSPACES[key] = ws
    return ws


def release_stream_workspace(device_index: int, cu_stream: int) -> None:
    _WORKSPACES.pop((device_index, cu_stream), None)


# ---- stream epochs and per-stream activation staging (rust/crates/nv-quant/src/lib.rs:9-51,
# rust/crates/nv-layers/src/linear.rs:317-323,1620-1660) -------------------------------------------------
# Buffers cached per stream must not outlive the stream: whoever retires a stream bumps its epoch, and
# every cache entry remembers the epoch it was made under and is dropped when the two differ.
_STREAM_EPOCHS: dict = {}
_EPOCH_LOCK = threading.Lock()


def stream_epoch(stream_key: int) -> int:
    with _EPOCH_LOCK:
        return _STREAM_EPOCHS.get(stream_key, 0)


def bump_stream_epoch(stream_key: int) -> None:
    with _EPOCH_LOCK:
        _STREAM_EPOCHS[stream_key] = _STREAM_EPOCHS.get(stream_key, 0) + 1


def stream_cache_key() -> int:
    """The current stream as a cache key (rust/crates/nv-quant/src/lib.rs:16-30): its handle, except that
    the per-thread default stream (handle 2) is a different stream in every thread and gets the thread's
    identity folded in."""
    raw = int(torch.cuda.current_stream().cuda_stream) if torch.cuda.is_available() else 0
    if raw != 0x2:
        return raw
    return 0x2 | (threading.get_ident() << 8)


def release_stream_resources(stream_key: int) -> None:
    """A stream is going away: drop its GEMM workspaces (on every device) and invalidate what linears
    staged for it."""
    for key in [k for k in _WORKSPACES if k[1] == stream_key]:
        _WORKSPACES.pop(key, None)
    bump_stream_epoch(stream_key)


class StagedActivations:
    """One (stream, padded row count) staging entry of a quantized linear: packed activations and their
    swizzled scales, zero beyond the rows last written."""
    __slots__ = ("epoch", "hwm_rows", "packed", "scales", "extra")

    def __init__(self, epoch: int, packed, scales):
        self.epoch, self.hwm_rows, self.packed, self.scales, self.extra = epoch, 0, packed, scales, {}


class StagingCache:
    """The reference's `a_staging` map.  Entries are created with zeroed buffers, outside graph capture
    only; rows-only quantizers then write the live rows and rely on the rest being zero, so a call with
    fewer rows than the one before first zeroes the buffers (`hwm_rows` is that high-water mark).  During
    a capture that finds no entry the caller must use buffers of its own and a quantizer that writes the
    pad rows too: `acquire` returns None."""

    def __init__(self):
        self._map: dict = {}
        self._lock = threading.Lock()

    def acquire(self, stream_key: int, m_padded: int, m_logical: int, capturing: bool, alloc_zeros, zero):
        """alloc_zeros() -> (packed, scales) zero-filled; zero(buffer) clears one in stream order."""
        key = (stream_key, m_padded)
        with self._lock:
            if not capturing:
                for k in [k for k, v in self._map.items() if v.epoch != stream_epoch(k[0])]:
                    del self._map[k]
                if key not in self._map:
                    packed, scales = alloc_zeros()
                    self._map[key] = StagedActivations(stream_epoch(stream_key), packed, scales)
            entry = self._map.get(key)
            if entry is None:
                return None
            if m_logical < entry.hwm_rows:
                zero(entry.packed)
                zero(entry.scales)
            entry.hwm_rows = m_logical
            return entry

    def diag(self, stream_key: int, m_padded: int):
        """(epoch, high-water mark) of an entry, or None (linear.rs:1802-1808)."""
        with self._lock:
            e = self._map.get((stream_key, m_padded))
            return None if e is None else (e.epoch, e.hwm_rows)

    def __len__(self):
        return len(self._map)


# ---- the runner -------------------------------------------------------------------------------------------
class Nvfp4GemmRunner:
    """d [m, n] bf16 = alpha * A [m, k] * B [n, k]^T for NVFP4 operands with swizzled block scales."""

    def __init__(self, backend: Nvfp4Backend | None = None, env=None):
        env = os.environ if env is None else env
        self.backend = Nvfp4Backend.from_env(env.get("SPEACHES_NVFP4_BACKEND")) if backend is None else backend
        self.streamk_mode = streamk_mode_from(env.get("NV_NVFP4_STREAMK"))
        self.k256 = k256_from(env.get("NV_NVFP4_K256"))
        self.streamk_k256 = streamk_k256_from(env.get("NV_NVFP4_STREAMK_K256"))
        self.streamk_down_splits = streamk_down_splits_from(env.get("NV_NVFP4_STREAMK_DOWN_SPLITS"))
        self.streamk_failed = False     # a stream-K launch that fails switches it off for good (nvfp4.rs:719-727)

    def streamk_wanted(self, m: int, n: int) -> bool:
        if self.streamk_failed or self.streamk_mode is StreamkMode.NEVER:
            return False
        if self.streamk_mode is StreamkMode.ALWAYS:
            return True
        return skinny_tiles(m, n) or ragged_last_wave(m, n)

    def plan(self, m: int, n: int, k: int, stream_k: bool):
        """(entry point, extra integer arguments) for one launch -- the reference's choice tree
        (nvfp4.rs:767-854) over this library's symbols."""
        tiled = "nv_kernels_cutlass_fp4_gemm_sm120_bf16_tiled"
        if stream_k and self.streamk_down_splits >= 2:
            return tiled, (0, self.streamk_down_splits)
        if stream_k:
            if k % 256 == 0 and self.streamk_k256:
                return tiled, (1, 1)
            return "nv_kernels_cutlass_fp4_gemm_sm120_bf16_streamk", ()
        if k % 256 == 0 and self.k256:
            return tiled, (1, 0)
        return "nv_kernels_cutlass_fp4_gemm_sm120_bf16", ()

    def _launch(self, entry, extra, a_packed, a_scales, b_packed, b_scales, alpha_dev, d, m, n, k, ws) -> int:
        need = C.c_size_t(0)
        return _ffi.call(entry, torch.cuda.current_stream().cuda_stream, a_packed.data_ptr(), a_scales.data_ptr(),
                         b_packed.data_ptr(), b_scales.data_ptr(), alpha_dev.data_ptr(), d.data_ptr(), m, n, k, *extra,
                         ws.data_ptr(), ws.numel(), C.addressof(need))

    def matmul_cublaslt(self, a_packed, a_scales, b_packed, b_scales, alpha_host: float, d, m, n, k, ws) -> None:
        """The library route (nvfp4.rs:866-1067): needs m >= 128 -- pad the activation -- and a host alpha."""
        if m < MIN_TILE:
            raise ValueError(f"NVFP4 cuBLASLt path requires m >= {MIN_TILE} (got m={m}); pad the activation "
                             "or use the cutlass backend")
        entry = "nvk_b200_cublaslt_fp4_gemm_bf16"
        rc = _ffi.call(entry, torch.cuda.current_stream().cuda_stream, a_packed.data_ptr(), a_scales.data_ptr(),
                       b_packed.data_ptr(), b_scales.data_ptr(), d.data_ptr(), m, n, k, float(alpha_host),
                       ws.data_ptr(), ws.numel())
        if rc != 0:
            raise _ffi.NvkError(entry, rc)

    def matmul(self, a_packed, a_scales, b_packed, b_scales, alpha_dev, d, m: int, n: int, k: int,
               alpha_host: float | None = None) -> None:
        """`alpha_host` is the host copy of `alpha_dev` the reference's callers keep beside it
        (nvfp4.rs:556-563); only the cuBLASLt backend reads it, and reads nothing else."""
        if k % 16 != 0:
            raise ValueError(f"k={k} must be a multiple of 16")
        if m == 0 or n < MIN_TILE or k < MIN_TILE:
            raise ValueError(f"NVFP4 GEMM requires m >= 1 and n,k >= {MIN_TILE}; got m={m} n={n} k={k}")
        ws = ensure_workspace_for_stream()
        if self.backend is Nvfp4Backend.CUBLASLT:
            if alpha_host is None:
                raise ValueError("the cublaslt backend takes alpha from the host: pass alpha_host")
            return self.matmul_cublaslt(a_packed, a_scales, b_packed, b_scales, alpha_host, d, m, n, k, ws)
        if self.streamk_wanted(m, n):
            entry, extra = self.plan(m, n, k, True)
            rc = self._launch(entry, extra, a_packed, a_scales, b_packed, b_scales, alpha_dev, d, m, n, k, ws)
            if rc == 0:
                return
            self.streamk_failed = True   # fall back to the data-parallel scheduler, permanently
        entry, extra = self.plan(m, n, k, False)
        rc = self._launch(entry, extra, a_packed, a_scales, b_packed, b_scales, alpha_dev, d, m, n, k, ws)
        if rc != 0:
            raise _ffi.NvkError(entry, rc)
