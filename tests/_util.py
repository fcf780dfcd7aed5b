"""Helpers shared by the GPU parity tests: seeded inputs, device buffers, C-ABI calls."""
from __future__ import annotations

import numpy as np
import torch

import speaches_plus_b200 as sp
from oracle import ref

ffi = sp.ffi


def require_gpu():
    # GPU tests fail (not skip) without a device: a green run must have executed the kernels.
    assert torch.cuda.is_available(), "GPU test selected but no CUDA device is visible"
    return torch.device("cuda:0")


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def dev(a: np.ndarray) -> torch.Tensor:
    """numpy (u8/u16/i32/f32) -> device tensor with the same bytes (u16 travels as int16)."""
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).cuda()
    return torch.from_numpy(a).cuda()


def host_u16(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        t = t.view(torch.int16)
    return t.cpu().numpy().view(np.uint16)


def gauss_bf16(rng, shape, std=1.0) -> np.ndarray:
    return ref.f32_to_bf16((rng.standard_normal(shape) * std).astype(np.float32))


def make_weight(rng, n, k, std=0.02):
    """Seeded N(0, std) bf16 weight quantized by the ORACLE (so the GEMV tests do not depend on the
    GPU quantizer): returns packed [n,k/2], swizzled scales, alpha, and the bf16 bits."""
    w = gauss_bf16(rng, (n, k), std)
    packed, sw, alpha = ref.quantize_weight_bf16(w)
    return packed, sw, alpha, w


def rel_err_floor(got_f32, want, floor=1e-3):
    """The reference's GEMV tolerance form (rust/crates/nv-quant/tests/nvfp4_m1_gemv_ab.rs:103-118):
    |got-want| / max(|want|, rms(want), floor), worst element."""
    want = np.asarray(want, np.float64)
    rms = float(np.sqrt(np.mean(want ** 2)))
    den = np.maximum(np.abs(want), max(rms, floor))
    return float(np.max(np.abs(np.asarray(got_f32, np.float64) - want) / den))


def bf16_ulp_diff(a_bits, b_bits):
    """Distance in bf16 ulps between two bf16 bit arrays (monotone integer mapping)."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(np.asarray(a_bits)) - key(np.asarray(b_bits)))
