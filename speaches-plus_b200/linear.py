"""Host-side mirror of the reference's NVFP4 `Linear` (rust/crates/nv-layers/src/linear.rs) and of
its dense W4A16 MLP pair (rust/crates/nv-models/src/qwen3_5_moe.rs:661-792), over libnvk_b200.

torch is used for device memory and streams only; every operator is one or more launches of the
CUDA library on the current stream.  There is one route per M class and no fallback.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _ffi

BLOCK_SIZE = 16   # rust/crates/nv-quant/src/nvfp4.rs:1
MIN_TILE = 128    # rust/crates/nv-quant/src/nvfp4.rs:2 ; linear.rs:1565-1579 refuses smaller dims
MAX_DECODE_M = 64  # rows one launch of the decode-sized route takes


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_WORKSPACES: dict = {}


def linear_workspace(device, m: int, k: int) -> torch.Tensor:
    """Activation workspace for nvk_b200_linear_nvfp4_w4a16_ws, one per (device, stream), grown on
    demand.  Launches on one stream are ordered, so consecutive linears may share it."""
    need = int(_ffi.lib().nvk_b200_linear_workspace_bytes(m, k))
    key = (torch.device(device).index, torch.cuda.current_stream().cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


def linear_w4a16(lin_a, lin_b, x, x2, y_a, y_b, m: int) -> None:
    """One launch of the decode-sized W4A16 linear (optionally two arms / SiLU prologue) for m <= 64."""
    n, k = lin_a.out_features, lin_a.in_features
    ws = linear_workspace(x.device, m, k) if m >= 3 else None
    _ffi.check("nvk_b200_linear_nvfp4_w4a16_ws", _stream(), lin_a.weight_u8.data_ptr(), lin_a.weight_scales.data_ptr(),
               lin_b.weight_u8.data_ptr() if lin_b is not None else None,
               lin_b.weight_scales.data_ptr() if lin_b is not None else None, x.data_ptr(),
               x2.data_ptr() if x2 is not None else None, y_a.data_ptr(), y_b.data_ptr() if y_b is not None else None,
               lin_a.alpha_w4a16, lin_b.alpha_w4a16 if lin_b is not None else 0.0, m, n, k,
               ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0)


def swizzled_scale_bytes(rows: int, cols: int) -> int:
    """Size of the swizzled block-scale buffer (rust/crates/nv-layers/src/linear.rs:2178-2180)."""
    return -(-rows // 128) * 128 * -(-(cols // 16) // 4) * 4


def stored_global_from_amax(amax: float) -> float:
    """448*6/amax in f32 (rust/crates/nv-layers/src/linear.rs:2161-2175); 1.0 for an all-zero tensor."""
    a = np.float32(amax)
    if a == 0 or not np.isfinite(a):
        return 1.0
    return float(np.float32(np.float32(448.0) * np.float32(6.0)) / a)


def quantize_nvfp4_bf16(x: torch.Tensor, stored_global: float, m_padded: int | None = None):
    """bf16 [m, K] -> (packed [m_padded, K/2] u8, swizzled scales u8) via nv_kernels_quantize_nvfp4_bf16."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
    m, k = x.shape
    mp = m if m_padded is None else m_padded
    packed = torch.empty((mp, k // 2), dtype=torch.uint8, device=x.device)
    scales = torch.zeros(swizzled_scale_bytes(mp, k), dtype=torch.uint8, device=x.device)
    _ffi.check("nv_kernels_quantize_nvfp4_bf16", _stream(), x.data_ptr(), packed.data_ptr(), scales.data_ptr(),
               float(stored_global), mp, m, k)
    return packed, scales


def quantize_weight_nvfp4(w: torch.Tensor):
    """bf16 weight [N, K] on the GPU -> (packed, scales_swizzled, weight_alpha, stored_global).

    Follows Linear::from_bf16_quantized_nvfp4_dev (rust/crates/nv-layers/src/linear.rs:2124-2226):
    stored_global = 448*6/max|W|, weight_alpha = 1/stored_global, activation global 1.0."""
    assert w.dim() == 2
    w = w.contiguous()
    amax = float(w.abs().max().float().item())
    g = stored_global_from_amax(amax)
    packed, scales = quantize_nvfp4_bf16(w, g)
    return packed, scales, float(np.float32(1.0) / np.float32(g)), g


class Nvfp4Linear:
    """NVFP4 weight-only linear: y = x W^T (+ bias), bf16 in/out, fp32 accumulate.

    Storage mirrors `Nvfp4Storage` (rust/crates/nv-layers/src/linear.rs:308-318): packed weights
    [out, in/2], swizzled block scales, `weight_alpha` = 1/stored weight global (times the
    reciprocal of a stored input global when a checkpoint carries one)."""

    def __init__(self, weight_u8: torch.Tensor, weight_scales: torch.Tensor, weight_alpha: float,
                 in_features: int, out_features: int, bias: torch.Tensor | None = None,
                 input_stored_global: float = 1.0):
        if in_features % BLOCK_SIZE != 0:
            raise ValueError(f"nvfp4 linear: in_features {in_features} is not a multiple of {BLOCK_SIZE}")
        if in_features < MIN_TILE or out_features < MIN_TILE:
            raise ValueError(f"nvfp4 linear: dims ({out_features},{in_features}) below MIN_TILE={MIN_TILE}")
        if weight_u8.numel() != out_features * in_features // 2:
            raise ValueError("nvfp4 linear: packed weight has the wrong number of bytes")
        if weight_scales.numel() < swizzled_scale_bytes(out_features, in_features):
            raise ValueError("nvfp4 linear: swizzled scale buffer too small")
        self.weight_u8 = weight_u8.contiguous()
        self.weight_scales = weight_scales.contiguous()
        self.weight_alpha = float(weight_alpha)
        self.input_stored_global = float(input_stored_global)
        self.in_features, self.out_features = in_features, out_features
        self.bias = bias
        self._lora = None   # adapter hook, see set_lora_hook

    # -- constructors (names follow the reference) --
    @classmethod
    def new_nvfp4(cls, weight_u8, weight_scales_swizzled, weight_alpha, in_features, out_features, bias=None):
        return cls(weight_u8, weight_scales_swizzled, weight_alpha, in_features, out_features, bias)

    @classmethod
    def new_nvfp4_scaled(cls, weight_u8, weight_scales_swizzled, in_features, out_features, bias, weight_alpha,
                         input_stored_global):
        """A checkpoint's linear: `weight_alpha` = 1/(weight global) x 1/(input global), and the stored input
        global the activations are quantized with on the FP4 x FP4 route (linear.rs:2080-2115)."""
        return cls(weight_u8, weight_scales_swizzled, weight_alpha, in_features, out_features, bias,
                   input_stored_global)

    @classmethod
    def from_bf16_quantized_nvfp4_dev(cls, weight: torch.Tensor, bias: torch.Tensor | None = None):
        n, k = weight.shape
        packed, scales, alpha, _ = quantize_weight_nvfp4(weight)
        return cls(packed, scales, alpha, k, n, bias)

    @classmethod
    def from_bf16_quantized_nvfp4(cls, weight: torch.Tensor, bias: torch.Tensor | None = None):
        """The reference's host-quantized constructor (linear.rs:2228-2275): blocks quantized with a
        global of 1.0 (no per-tensor rescale) and alpha 1.0.  The bytes are produced by the device
        quantizer, which is byte-exact against the host rule."""
        if weight.dim() != 2:
            raise ValueError(f"Linear weight must be 2-D, got rank {weight.dim()}")
        n, k = weight.shape
        packed, scales = quantize_nvfp4_bf16(weight.to(torch.bfloat16).contiguous(), 1.0)
        return cls(packed, scales, 1.0, k, n, bias)

    def nvfp4_parts(self):
        """(packed weights, swizzled scales, weight_alpha) -- linear.rs:411-451."""
        return self.weight_u8, self.weight_scales, self.weight_alpha

    def nvfp4_parts_full(self):
        """The same plus the stored input global (linear.rs:411-427)."""
        return self.weight_u8, self.weight_scales, self.weight_alpha, self.input_stored_global

    def dequant_weight(self) -> torch.Tensor:
        """The bf16 weight this linear stands for, [out, in] on the linear's device.  Load-time /
        diagnostic helper done on the host, as in the reference (linear.rs:508-539): download the packed
        bytes and scales, value = e2m1 * (ue4m3 * weight_alpha) in f32, round to bf16, upload."""
        from . import weights as W
        kb = self.in_features // BLOCK_SIZE
        packed = self.weight_u8.cpu().numpy()
        lin = W.unswizzle_scales(self.weight_scales.cpu().numpy(), self.out_features, kb)
        bits = W.dequantize_packed_to_bf16_bits(packed, lin, self.out_features, self.in_features, self.weight_alpha)
        return torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).to(self.weight_u8.device)

    @property
    def alpha_w4a16(self) -> float:
        """Output multiplier when the activations stay bf16: the reciprocal of the weight global alone.
        `weight_alpha` also carries the reciprocal of the input global, which only the route that
        quantizes activations needs, so it is multiplied back out here, as the reference's W4A16 call
        sites do (rust/crates/nv-models/src/qwen3_5_moe.rs:718-727)."""
        return float(np.float32(self.weight_alpha) * np.float32(self.input_stored_global))

    # -- adapter hook (rust/crates/nv-layers/src/linear.rs:591-606) --
    def set_lora_hook(self, hook) -> None:
        """`hook(x2, y2, window)` runs after the base matmul on the flattened [rows, in] input and
        [rows, out] output (window is None for a whole linear) and returns a replacement for y2, or None
        to keep it -- the adapter's low-rank delta is its business.  None removes the hook."""
        self._lora = hook

    def has_lora(self) -> bool:
        return self._lora is not None

    # -- forward --
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.in_features:
            raise ValueError(f"nvfp4 linear: input last dim {x.shape[-1]} != {self.in_features}")
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        y = torch.empty((x2.shape[0], self.out_features), dtype=torch.bfloat16, device=x.device)
        self.forward_into(x2, y)
        if self._lora is not None:
            replaced = self._lora(x2, y, None)
            if replaced is not None:
                y = replaced
        if self.bias is not None:
            y += self.bias
        return y.reshape(*lead, self.out_features)

    __call__ = forward

    def forward_into(self, x2: torch.Tensor, y: torch.Tensor, allow_prefill: bool = True) -> None:
        """x2 [M, in] bf16 contiguous -> y [M, out].  M <= 64 is one launch of the W4A16 kernel.  Larger
        M takes the FP4 x FP4 tensor-core GEMM of the prefill library -- in a single-GPU process only:
        with `allow_prefill=False`, or when this process is one rank of several, the rows run as chunks
        of 64 on the W4A16 kernel instead (rows are independent there, so the result does not depend on
        the chunking), and the prefill library is never touched."""
        assert x2.is_cuda and x2.dtype == torch.bfloat16 and x2.is_contiguous() and y.is_contiguous()
        m = x2.shape[0]
        s = _stream()
        route = self.route_for(m, allow_prefill)
        if route == "gemv":
            _ffi.check("nv_kernels_nvfp4_gemv_bf16act", s, self.weight_u8.data_ptr(), self.weight_scales.data_ptr(),
                       x2.data_ptr(), y.data_ptr(), self.alpha_w4a16, self.out_features, self.in_features)
            return
        if route == "prefill":
            self.forward_prefill_into(x2, y)
            return
        for r0 in range(0, m, MAX_DECODE_M):
            mm = min(MAX_DECODE_M, m - r0)
            linear_w4a16(self, None, x2[r0:], None, y[r0:], None, mm)

    def forward_residual_into(self, x2: torch.Tensor, residual: torch.Tensor, y: torch.Tensor,
                              up: torch.Tensor | None = None) -> None:
        """y [M, out] = bf16(residual + (a W^T) * alpha) with one rounding, a = x2 or -- when `up` is given --
        bf16(SiLU(x2) * up); rows in chunks of up to 64.  `y` may be `residual` itself (an in-place update
        of the hidden state).  The decode-sized W4A16 route only."""
        assert x2.is_cuda and x2.dtype == torch.bfloat16 and x2.is_contiguous()
        assert residual.dtype == torch.bfloat16 and residual.is_contiguous() and y.is_contiguous()
        assert residual.shape == (x2.shape[0], self.out_features) and y.shape == residual.shape
        assert up is None or (up.shape == x2.shape and up.is_contiguous() and up.dtype == torch.bfloat16)
        s = _stream()
        for r0 in range(0, x2.shape[0], MAX_DECODE_M):
            mm = min(MAX_DECODE_M, x2.shape[0] - r0)
            _ffi.check("nvk_b200_linear_nvfp4_w4a16_residual", s, self.weight_u8.data_ptr(),
                       self.weight_scales.data_ptr(), x2[r0:].data_ptr(), up[r0:].data_ptr() if up is not None else None,
                       residual[r0:].data_ptr(), y[r0:].data_ptr(), self.alpha_w4a16, mm, self.out_features,
                       self.in_features)

    def forward_nvfp4_gemv_m1(self, x: torch.Tensor) -> torch.Tensor:
        """One row through the M = 1 GEMV whatever else is configured (no bias, no adapter): what a
        draft-only lm_head asks for (linear.rs:1420-1442)."""
        lead = 1
        for d in x.shape[:-1]:
            lead *= d
        if lead != 1:
            raise ValueError(f"forward_nvfp4_gemv_m1: draft lm_head serves one row per step, got leading {lead}")
        if x.shape[-1] != self.in_features:
            raise ValueError(f"forward_nvfp4_gemv_m1: input last dim {x.shape[-1]} != in_features {self.in_features}")
        x2 = x.reshape(1, self.in_features).contiguous()
        y = torch.empty((1, self.out_features), dtype=torch.bfloat16, device=x.device)
        _ffi.check("nv_kernels_nvfp4_gemv_bf16act", _stream(), self.weight_u8.data_ptr(), self.weight_scales.data_ptr(),
                   x2.data_ptr(), y.data_ptr(), self.alpha_w4a16, self.out_features, self.in_features)
        return y.reshape(*x.shape[:-1], self.out_features)

    def route_for(self, m: int, allow_prefill: bool = True) -> str:
        """Which kernels M rows take: "gemv" (M = 1), "decode" (row chunks of up to 64 on the W4A16
        kernel) or "prefill" (the FP4 x FP4 GEMM of the prefill library).  The last is chosen only in
        a single-GPU process: the prefill library holds a tile that loads with TMA cluster multicast
        and is never used from one rank of several."""
        if m == 1:
            return "gemv"
        if (m > MAX_DECODE_M and allow_prefill and _ffi.distributed_world() == 1
                and self.out_features % 8 == 0 and self.in_features % 32 == 0):
            return "prefill"
        return "decode"

    def prenorm_nvfp4_eligible(self) -> bool:
        """linear.rs:648-651: an NVFP4 projection without bias and without an adapter."""
        return self.bias is None and not self.has_lora()

    def forward_prenorm_nvfp4(self, x_pre: torch.Tensor, norm_weight: torch.Tensor, eps: float) -> torch.Tensor:
        """RMSNorm fused into the activation quantizer, then the FP4 x FP4 GEMM (linear.rs:653-689 with
        `FusedPreNorm`): y = (rmsnorm(x_pre) * norm_weight) W^T, the normalised row rounded to bf16 once
        before it is quantized.  One row of K bf16 values must fit the quantizer's 48 KiB of shared
        memory (K <= 24576)."""
        if not self.prenorm_nvfp4_eligible():
            raise ValueError("forward_prenorm_nvfp4: linear is not an eligible NVFP4 projection")
        if x_pre.shape[-1] != self.in_features:
            raise ValueError(f"forward_prenorm_nvfp4: input last dim {x_pre.shape[-1]} != in_features "
                             f"{self.in_features}")
        lead = x_pre.shape[:-1]
        x2 = x_pre.reshape(-1, self.in_features).contiguous()
        assert x2.is_cuda and x2.dtype == torch.bfloat16 and norm_weight.dtype == torch.bfloat16
        m, k = x2.shape
        m_pad = -(-m // 128) * 128
        entry = self._acquire_staging(m, x2.device)
        if entry is not None:
            # live rows only: the rest of the staging entry is zero (linear.rs:1713)
            a_packed, a_scales, rows = entry.packed, entry.scales, m
        else:
            a_packed = torch.empty((m_pad, k // 2), dtype=torch.uint8, device=x2.device)
            a_scales = torch.zeros(swizzled_scale_bytes(m_pad, k), dtype=torch.uint8, device=x2.device)
            rows = m_pad
        _ffi.check("nv_kernels_rmsnorm_quantize_nvfp4_bf16", _stream(), x2.data_ptr(), norm_weight.data_ptr(),
                   a_packed.data_ptr(), a_scales.data_ptr(), float(self.input_stored_global), float(eps), rows, m, k)
        y = torch.empty((m, self.out_features), dtype=torch.bfloat16, device=x2.device)
        self._fp4_gemm(a_packed, a_scales, y, m, entry)
        return y.reshape(*lead, self.out_features)

    def forward_prenorm_decode(self, x_pre: torch.Tensor, norm_weight: torch.Tensor, eps: float) -> torch.Tensor:
        """Decode-sized rows with an RMSNorm in front, on the route that keeps activations in bf16
        (linear.rs:1444-1542 with a pre-norm): one RMSNorm launch into a bf16 buffer, then the W4A16
        linear.  x_pre [..., in] bf16 with at most 64 rows."""
        if x_pre.shape[-1] != self.in_features:
            raise ValueError(f"forward_prenorm_decode: input last dim {x_pre.shape[-1]} != in_features "
                             f"{self.in_features}")
        lead = x_pre.shape[:-1]
        x2 = x_pre.reshape(-1, self.in_features).contiguous()
        if x2.shape[0] > MAX_DECODE_M:
            raise ValueError(f"forward_prenorm_decode: {x2.shape[0]} rows; the decode route takes up to {MAX_DECODE_M}")
        assert x2.is_cuda and x2.dtype == torch.bfloat16 and norm_weight.dtype == torch.bfloat16
        y = torch.empty((x2.shape[0], self.out_features), dtype=torch.bfloat16, device=x2.device)
        if x2.shape[0] <= 8 and self.in_features % 32 == 0:
            # a few rows: the norm is applied while the linear stages its activations (same bits, one launch)
            _ffi.check("nvk_b200_linear_nvfp4_w4a16_normed", _stream(), self.weight_u8.data_ptr(),
                       self.weight_scales.data_ptr(), None, None, x2.data_ptr(), norm_weight.data_ptr(), None,
                       float(eps), y.data_ptr(), None, self.alpha_w4a16, 0.0, x2.shape[0], self.out_features,
                       self.in_features)
        else:
            xn = torch.empty_like(x2)
            _ffi.check("nv_kernels_rmsnorm_bf16", _stream(), x2.data_ptr(), norm_weight.data_ptr(), xn.data_ptr(),
                       x2.shape[0], self.in_features, float(eps))
            self.forward_into(xn, y)
        if self.bias is not None:
            y += self.bias
        return y.reshape(*lead, self.out_features)

    # -- prefill-sized rows: activation staging per (stream, padded rows), as the reference keeps it --
    def _staging_cache(self):
        from .runner import StagingCache
        c = getattr(self, "_staging", None)
        if c is None:
            c = self._staging = StagingCache()
        return c

    def _alpha_on(self, device) -> torch.Tensor:
        """weight_alpha as one f32 in device memory (`weight_alpha_dev`, linear.rs:314).  Made on first use,
        which must not be inside a graph capture: `prepare_prefill` makes it ahead of time."""
        cache = self.__dict__.setdefault("_alpha_dev", {})
        t = cache.get(device)
        if t is None:
            if device.type == "cuda" and torch.cuda.is_current_stream_capturing():
                raise RuntimeError("nvfp4 linear: the device copy of alpha must exist before graph capture "
                                   "(call prepare_prefill first)")
            t = cache[device] = torch.tensor([self.weight_alpha], dtype=torch.float32, device=device)
        return t

    def _workspace_for(self, m_pad: int, device, entry) -> torch.Tensor:
        """The data-parallel GEMM's workspace for `m_pad` rows: kept with the staging entry, or made for
        this call when there is none."""
        if entry is not None and "ws" in entry.extra:
            return entry.extra["ws"]
        need = C.c_size_t(0)
        _ffi.check("nv_kernels_cutlass_fp4_gemm_sm120_bf16", _stream(), None, None, None, None, None, None, m_pad,
                   self.out_features, self.in_features, None, 0, C.addressof(need))
        ws = torch.empty(max(int(need.value), 16), dtype=torch.uint8, device=device)
        if entry is not None:
            entry.extra["ws"] = ws
        return ws

    def _acquire_staging(self, m: int, device):
        """The current stream's staging entry for ceil(m / 128) * 128 rows (made on first use outside a
        capture, evicted when the stream's epoch has moved, zeroed when fewer rows arrive than last time:
        linear.rs:1620-1660), or None inside a capture that finds none."""
        from .runner import stream_cache_key
        k = self.in_features
        m_pad = -(-m // 128) * 128
        capturing = device.type == "cuda" and torch.cuda.is_current_stream_capturing()

        def alloc_zeros():
            return (torch.zeros((m_pad, k // 2), dtype=torch.uint8, device=device),
                    torch.zeros(swizzled_scale_bytes(m_pad, k), dtype=torch.uint8, device=device))

        return self._staging_cache().acquire(stream_cache_key(), m_pad, m, capturing, alloc_zeros,
                                             lambda buf: buf.zero_())

    def prepare_prefill(self, max_m: int, device=None) -> None:
        """Create, on the current stream, everything a later call with ceil(max_m / 128) * 128 padded rows
        needs -- the staging entry, the GEMM workspace and the device copy of alpha -- so that such a call
        allocates nothing and can be captured (the reference creates its runner's workspace ahead of
        time for the same reason, rust/crates/nv-quant/src/nvfp4.rs:391-409).  Other row counts get their
        entry on first use."""
        dev = self.weight_u8.device if device is None else torch.device(device)
        self._alpha_on(dev)
        entry = self._acquire_staging(max_m, dev)
        entry.hwm_rows = 0   # nothing has been written yet
        self._workspace_for(-(-max_m // 128) * 128, dev, entry)

    def nvfp4_staging_diag(self, stream_key: int, m_padded: int):
        """(epoch, high-water mark) of a staging entry, or None (linear.rs:1802-1808)."""
        return self._staging_cache().diag(stream_key, m_padded)

    def forward_prefill_into(self, x2: torch.Tensor, y: torch.Tensor) -> None:
        """Prefill-sized M: the reference's default route (rust/crates/nv-layers/src/linear.rs:1590-1795) --
        quantize the activations to NVFP4 (global 1.0, rows padded to a multiple of 128 with zeros), then one
        block-scaled FP4 x FP4 tensor-core GEMM with alpha = weight_alpha in device memory.  With a
        staging entry the quantizer writes the live rows only (the rest of the entry is zero); without
        one -- a capture that was not prepared for this row count -- buffers of this call and the
        quantizer that writes the pad rows too."""
        m, k = x2.shape
        m_pad = -(-m // 128) * 128
        entry = self._acquire_staging(m, x2.device)
        if entry is not None:
            a_packed, a_scales = entry.packed, entry.scales
            _ffi.check("nv_kernels_quantize_nvfp4_bf16_rows", _stream(), x2.data_ptr(), a_packed.data_ptr(),
                       a_scales.data_ptr(), float(self.input_stored_global), m, k)
        else:
            a_packed = torch.empty((m_pad, k // 2), dtype=torch.uint8, device=x2.device)
            a_scales = torch.empty(swizzled_scale_bytes(m_pad, k), dtype=torch.uint8, device=x2.device)
            _ffi.check("nv_kernels_quantize_nvfp4_bf16", _stream(), x2.data_ptr(), a_packed.data_ptr(),
                       a_scales.data_ptr(), float(self.input_stored_global), m_pad, m, k)
        self._fp4_gemm(a_packed, a_scales, y, m, entry)

    def _fp4_gemm(self, a_packed: torch.Tensor, a_scales: torch.Tensor, y: torch.Tensor, m: int, entry=None) -> None:
        """y [m, out] = alpha * A W^T for activations already quantized (rows padded to 128)."""
        k, n = self.in_features, self.out_features
        dev = a_packed.device
        m_pad = a_packed.shape[0]
        alpha = self._alpha_on(dev)
        runner = getattr(self, "runner", None)
        if runner is not None:
            # an Nvfp4GemmRunner (runner.py) picks the scheduler for the shape and owns the workspace
            if runner.backend.value == "cublaslt":
                # the library route computes every padded row: into a padded buffer, then trimmed
                # (pad -> quantize -> GEMM -> trim, rust/crates/nv-layers/src/linear.rs:1590-1795)
                yp = entry.extra.get("y_pad") if entry is not None else None
                if yp is None:
                    yp = torch.empty((m_pad, n), dtype=torch.bfloat16, device=dev)
                    if entry is not None:
                        entry.extra["y_pad"] = yp
                runner.matmul(a_packed, a_scales, self.weight_u8, self.weight_scales, alpha, yp, m_pad, n, k,
                              alpha_host=self.weight_alpha)
                y.copy_(yp[:m])
                return
            runner.matmul(a_packed, a_scales, self.weight_u8, self.weight_scales, alpha, y, m, n, k)
            return
        ws = self._workspace_for(m_pad, dev, entry)
        need = C.c_size_t(0)
        _ffi.check("nv_kernels_cutlass_fp4_gemm_sm120_bf16", _stream(), a_packed.data_ptr(), a_scales.data_ptr(),
                   self.weight_u8.data_ptr(), self.weight_scales.data_ptr(), alpha.data_ptr(), y.data_ptr(),
                   m, n, k, ws.data_ptr(), ws.numel(), C.addressof(need))


class Bf16Linear:
    """bf16 linear (lm_head, router gate): nv_kernels_gemv_bf16 at M = 1, nvk_b200_linear_bf16 -- one pass
    over the weight for all rows -- for up to 64 rows, row chunks of 64 beyond that."""

    def __init__(self, weight: torch.Tensor):
        assert weight.dtype == torch.bfloat16 and weight.dim() == 2
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape

    def nvfp4_draft_twin_rows(self, row0: int, rows: int) -> "Nvfp4Linear":
        """An NVFP4 copy of rows [row0, row0 + rows) of this weight, quantized on the device with the
        global of those rows; this linear stays as it is (linear.rs:2277-2296)."""
        if rows < 1 or row0 < 0 or row0 + rows > self.out_features:
            raise ValueError(f"nvfp4 draft twin: rows [{row0}, {row0}+{rows}) out of range for out_features "
                             f"{self.out_features}")
        return Nvfp4Linear.from_bf16_quantized_nvfp4_dev(self.weight[row0:row0 + rows].contiguous())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2 = x.reshape(-1, self.in_features).contiguous()
        y = torch.empty((x2.shape[0], self.out_features), dtype=torch.bfloat16, device=x.device)
        self.forward_into(x2, y)
        return y.reshape(*x.shape[:-1], self.out_features)

    def forward_into(self, x2: torch.Tensor, y: torch.Tensor, row_off: int = 0, rows: int | None = None) -> None:
        """x2 [M, in] bf16 contiguous -> y [M, rows] (contiguous), allocating nothing; `rows` weight rows
        from `row_off` (default: all of them)."""
        s = _stream()
        m = x2.shape[0]
        rows = self.out_features if rows is None else rows
        w = self.weight.data_ptr() + 2 * row_off * self.in_features
        if m == 1:
            _ffi.check("nv_kernels_gemv_bf16", s, w, x2.data_ptr(), y.data_ptr(), rows, self.in_features)
            return
        for r0 in range(0, m, MAX_DECODE_M):
            mm = min(MAX_DECODE_M, m - r0)
            _ffi.check("nvk_b200_linear_bf16", s, w, x2[r0:].data_ptr(), y[r0:].data_ptr(), mm, rows, self.in_features)

    def forward_rows(self, x: torch.Tensor, row_off: int, rows: int) -> torch.Tensor:
        """The product with weight rows [row_off, row_off + rows) only -- a slice of a vocabulary, say
        (rust/crates/nv-layers/src/linear.rs:883-913)."""
        if row_off < 0 or rows < 0 or row_off + rows > self.out_features:
            raise ValueError(f"forward_rows: rows {row_off}..{row_off + rows} out of range (out_features "
                             f"{self.out_features})")
        if x.shape[-1] != self.in_features:
            raise ValueError(f"forward_rows: input last dim {x.shape[-1]} != in_features {self.in_features}")
        x2 = x.reshape(-1, self.in_features).contiguous()
        y = torch.empty((x2.shape[0], rows), dtype=torch.bfloat16, device=x.device)
        if rows:
            self.forward_into(x2, y, row_off, rows)
        return y.reshape(*x.shape[:-1], rows)

    __call__ = forward


class Nvfp4Mlp:
    """SwiGLU MLP on the W4A16 route: one dual launch for gate+up sharing x, one launch for down
    with SiLU(gate)*up fused as its prologue (the activation is rounded to bf16 first, as the
    reference's decode kernel does; rust/crates/nv-kernels/cuda/gemv_nvfp4_w4a16_decode.cu:165-170)."""

    def __init__(self, gate: Nvfp4Linear, up: Nvfp4Linear, down: Nvfp4Linear):
        assert gate.in_features == up.in_features and gate.out_features == up.out_features
        assert down.in_features == gate.out_features
        self.gate, self.up, self.down = gate, up, down
        self._gu = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2 = x.reshape(-1, self.gate.in_features).contiguous()
        m = x2.shape[0]
        inter, hidden = self.gate.out_features, self.down.out_features
        if self._gu is None or self._gu.shape[1] != m or self._gu.device != x.device:
            self._gu = torch.empty((2, m, inter), dtype=torch.bfloat16, device=x.device)
        g, u = self._gu[0], self._gu[1]
        y = torch.empty((m, hidden), dtype=torch.bfloat16, device=x.device)
        s = _stream()
        for r0 in range(0, m, MAX_DECODE_M):
            mm = min(MAX_DECODE_M, m - r0)
            linear_w4a16(self.gate, self.up, x2[r0:], None, g[r0:], u[r0:], mm)
            linear_w4a16(self.down, None, g[r0:], u[r0:], y[r0:], None, mm)
        return y.reshape(*x.shape[:-1], hidden)

    def forward_residual(self, x: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        """residual + MLP(x), the sum rounded once: gate/up as in `forward`, then the down projection with
        the SiLU prologue and the residual epilogue in one launch.  Returns a new tensor."""
        x2 = x.reshape(-1, self.gate.in_features).contiguous()
        m = x2.shape[0]
        inter, hidden = self.gate.out_features, self.down.out_features
        r2 = residual.reshape(m, hidden).contiguous()
        if self._gu is None or self._gu.shape[1] != m or self._gu.device != x.device:
            self._gu = torch.empty((2, m, inter), dtype=torch.bfloat16, device=x.device)
        g, u = self._gu[0], self._gu[1]
        y = torch.empty((m, hidden), dtype=torch.bfloat16, device=x.device)
        for r0 in range(0, m, MAX_DECODE_M):
            mm = min(MAX_DECODE_M, m - r0)
            linear_w4a16(self.gate, self.up, x2[r0:], None, g[r0:], u[r0:], mm)
        self.down.forward_residual_into(g, r2, y, up=u)
        return y.reshape(*x.shape[:-1], hidden)

    def forward_block(self, h: torch.Tensor, norm_weight: torch.Tensor, eps: float) -> torch.Tensor:
        """A decoder layer's MLP block, h + MLP(RMSNorm(h)): for up to 8 rows two launches -- gate and up with
        the norm in their prologue, then down with the SiLU prologue and the residual epilogue; more rows
        run the norm kernel first.  Returns a new tensor."""
        hidden, inter = self.gate.in_features, self.gate.out_features
        h2 = h.reshape(-1, hidden).contiguous()
        m = h2.shape[0]
        if m > 8 or hidden % 32 != 0:
            xn = torch.empty_like(h2)
            _ffi.check("nv_kernels_rmsnorm_bf16", _stream(), h2.data_ptr(), norm_weight.data_ptr(), xn.data_ptr(), m,
                       hidden, float(eps))
            return self.forward_residual(xn, h2).reshape(h.shape)
        if self._gu is None or self._gu.shape[1] != m or self._gu.device != h.device:
            self._gu = torch.empty((2, m, inter), dtype=torch.bfloat16, device=h.device)
        g, u = self._gu[0], self._gu[1]
        _ffi.check("nvk_b200_linear_nvfp4_w4a16_normed", _stream(), self.gate.weight_u8.data_ptr(),
                   self.gate.weight_scales.data_ptr(), self.up.weight_u8.data_ptr(), self.up.weight_scales.data_ptr(),
                   h2.data_ptr(), norm_weight.data_ptr(), None, float(eps), g.data_ptr(), u.data_ptr(),
                   self.gate.alpha_w4a16, self.up.alpha_w4a16, m, inter, hidden)
        y = torch.empty_like(h2)
        self.down.forward_residual_into(g, h2, y, up=u)
        return y.reshape(h.shape)

    __call__ = forward
