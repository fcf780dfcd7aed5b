"""numpy front-end to the C oracle (oracle/nvfp4_oracle.c).

TEST INFRASTRUCTURE: imported only by tests/, the smoke check and the benchmark's
CPU-baseline leg.  The shipped package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import pathlib

import numpy as np

from . import build as _build

_HERE = pathlib.Path(__file__).resolve().parent
_lib = None

u8p = C.POINTER(C.c_uint8)
u16p = C.POINTER(C.c_uint16)
f32p = C.POINTER(C.c_float)
f64p = C.POINTER(C.c_double)
i32p = C.POINTER(C.c_int32)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = _build.build()
        L = C.CDLL(str(path))
        L.nvo_bf16_to_f32.restype = C.c_float
        L.nvo_bf16_to_f32.argtypes = [C.c_uint16]
        L.nvo_f32_to_bf16.restype = C.c_uint16
        L.nvo_f32_to_bf16.argtypes = [C.c_float]
        L.nvo_encode_e2m1.restype = C.c_uint8
        L.nvo_encode_e2m1.argtypes = [C.c_float]
        L.nvo_decode_e2m1.restype = C.c_float
        L.nvo_decode_e2m1.argtypes = [C.c_uint8]
        L.nvo_encode_ue4m3.restype = C.c_uint8
        L.nvo_encode_ue4m3.argtypes = [C.c_float]
        L.nvo_decode_ue4m3.restype = C.c_float
        L.nvo_decode_ue4m3.argtypes = [C.c_uint8]
        L.nvo_quantize_block.restype = None
        L.nvo_quantize_block.argtypes = [f32p, C.c_float, u8p, u8p]
        L.nvo_dequantize_block.restype = None
        L.nvo_dequantize_block.argtypes = [u8p, C.c_uint8, f32p]
        L.nvo_quantize_rows.restype = C.c_int
        L.nvo_quantize_rows.argtypes = [f32p, C.c_int, C.c_int, C.c_float, u8p, u8p]
        L.nvo_quantize_rows_bf16.restype = C.c_int
        L.nvo_quantize_rows_bf16.argtypes = [u16p, C.c_int, C.c_int, C.c_int, C.c_float, u8p, u8p]
        L.nvo_swizzled_len.restype = C.c_size_t
        L.nvo_swizzled_len.argtypes = [C.c_int, C.c_int]
        L.nvo_swizzle_scales.restype = None
        L.nvo_swizzle_scales.argtypes = [u8p, C.c_int, C.c_int, u8p]
        L.nvo_unswizzle_scales.restype = None
        L.nvo_unswizzle_scales.argtypes = [u8p, C.c_int, C.c_int, u8p]
        for name in ("nvo_dequantize_packed_linear", "nvo_dequantize_packed_swizzled"):
            f = getattr(L, name)
            f.restype = C.c_int
            f.argtypes = [u8p, u8p, C.c_int, C.c_int, C.c_float, f32p]
        L.nvo_dequantize_to_bf16.restype = C.c_int
        L.nvo_dequantize_to_bf16.argtypes = [u8p, u8p, C.c_int, C.c_int, C.c_float, u16p]
        L.nvo_linear_cpu_backend.restype = C.c_int
        L.nvo_linear_cpu_backend.argtypes = [u16p, u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_int]
        L.nvo_linear_cpu_backend_lanes16.restype = C.c_int
        L.nvo_linear_cpu_backend_lanes16.argtypes = [u16p, u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_int]
        L.nvo_linear_w4a16_f64.restype = C.c_int
        L.nvo_linear_w4a16_f64.argtypes = [u8p, u8p, u16p, C.c_float, C.c_int, C.c_int, C.c_int, f64p]
        L.nvo_matmul_w4a4.restype = C.c_int
        L.nvo_matmul_w4a4.argtypes = [u8p, u8p, u8p, u8p, C.c_float, C.c_int, C.c_int, C.c_int, u16p]
        L.nvo_silu_mul.restype = None
        L.nvo_silu_mul.argtypes = [u16p, u16p, C.c_size_t, C.c_int, f32p]
        L.nvo_moe_route_topk.restype = C.c_int
        L.nvo_moe_route_topk.argtypes = [f32p, f32p, i32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int,
                                         C.c_float, C.c_int, C.c_float]
        L.nvo_moe_unpermute_scatter.restype = None
        L.nvo_moe_unpermute_scatter.argtypes = [u16p, f32p, i32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int]
        L.nvo_num_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def _c(a, dt) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dt)


# ---- scalar codecs -------------------------------------------------------------------------
def encode_e2m1(x: float) -> int:
    return int(lib().nvo_encode_e2m1(float(np.float32(x))))


def decode_e2m1(code: int) -> float:
    return float(lib().nvo_decode_e2m1(code & 0xFF))


def encode_ue4m3(x: float) -> int:
    return int(lib().nvo_encode_ue4m3(float(np.float32(x))))


def decode_ue4m3(b: int) -> float:
    return float(lib().nvo_decode_ue4m3(b & 0xFF))


# ---- bf16 helpers (vectorised, numpy only) ---------------------------------------------------
def f32_to_bf16(x) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bits (uint16)."""
    u = _c(x, np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u.astype(np.uint64) + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def bf16_to_f32(b) -> np.ndarray:
    return (_c(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---- quantizer -------------------------------------------------------------------------------
def quantize_block(v16, stored_global: float = 1.0):
    v = _c(v16, np.float32)
    assert v.size == 16
    packed = np.zeros(8, np.uint8)
    sb = np.zeros(1, np.uint8)
    lib().nvo_quantize_block(_p(v, f32p), np.float32(stored_global), _p(packed, u8p), _p(sb, u8p))
    return packed, int(sb[0])


def dequantize_block(packed8, scale_byte: int) -> np.ndarray:
    p = _c(packed8, np.uint8)
    out = np.zeros(16, np.float32)
    lib().nvo_dequantize_block(_p(p, u8p), scale_byte, _p(out, f32p))
    return out


def quantize_rows(x, stored_global: float = 1.0):
    """f32 [rows, cols] -> (packed [rows, cols/2] u8, scales_linear [rows, cols/16] u8)."""
    x = _c(x, np.float32)
    rows, cols = x.shape
    packed = np.zeros((rows, cols // 2), np.uint8)
    scales = np.zeros((rows, cols // 16), np.uint8)
    rc = lib().nvo_quantize_rows(_p(x, f32p), rows, cols, np.float32(stored_global), _p(packed, u8p),
                                 _p(scales, u8p))
    assert rc == 0
    return packed, scales


def quantize_rows_bf16(x_bits, stored_global: float = 1.0, m_padded: int | None = None):
    """bf16 bits [m_logical, cols] -> packed/scales for m_padded rows (pad rows quantize zeros)."""
    x = _c(x_bits, np.uint16)
    m_logical, cols = x.shape
    mp = m_logical if m_padded is None else m_padded
    packed = np.zeros((mp, cols // 2), np.uint8)
    scales = np.zeros((mp, cols // 16), np.uint8)
    rc = lib().nvo_quantize_rows_bf16(_p(x, u16p), mp, m_logical, cols, np.float32(stored_global),
                                      _p(packed, u8p), _p(scales, u8p))
    assert rc == 0
    return packed, scales


def swizzled_len(rows: int, k_blocks: int) -> int:
    return int(lib().nvo_swizzled_len(rows, k_blocks))


def swizzle_scales(linear, rows: int | None = None, k_blocks: int | None = None) -> np.ndarray:
    lin = _c(linear, np.uint8)
    if rows is None:
        rows, k_blocks = lin.shape
    out = np.zeros(swizzled_len(rows, k_blocks), np.uint8)
    lib().nvo_swizzle_scales(_p(lin, u8p), rows, k_blocks, _p(out, u8p))
    return out


def unswizzle_scales(sw, rows: int, k_blocks: int) -> np.ndarray:
    s = _c(sw, np.uint8)
    out = np.zeros((rows, k_blocks), np.uint8)
    lib().nvo_unswizzle_scales(_p(s, u8p), rows, k_blocks, _p(out, u8p))
    return out


def dequantize_packed_linear(packed, scales_linear, rows, cols, mult=1.0) -> np.ndarray:
    p, s = _c(packed, np.uint8), _c(scales_linear, np.uint8)
    out = np.zeros((rows, cols), np.float32)
    assert lib().nvo_dequantize_packed_linear(_p(p, u8p), _p(s, u8p), rows, cols, np.float32(mult),
                                              _p(out, f32p)) == 0
    return out


def dequantize_packed_swizzled(packed, scales_sw, rows, cols, mult=1.0) -> np.ndarray:
    p, s = _c(packed, np.uint8), _c(scales_sw, np.uint8)
    out = np.zeros((rows, cols), np.float32)
    assert lib().nvo_dequantize_packed_swizzled(_p(p, u8p), _p(s, u8p), rows, cols, np.float32(mult),
                                                _p(out, f32p)) == 0
    return out


def dequantize_to_bf16(packed, scales_sw, rows, cols, mult=1.0) -> np.ndarray:
    p, s = _c(packed, np.uint8), _c(scales_sw, np.uint8)
    out = np.zeros((rows, cols), np.uint16)
    assert lib().nvo_dequantize_to_bf16(_p(p, u8p), _p(s, u8p), rows, cols, np.float32(mult),
                                        _p(out, u16p)) == 0
    return out


def weight_global(w_f32) -> float:
    """stored_global = 448*6/amax, as rust/crates/nv-layers/src/linear.rs:2161-2175 (f32 arithmetic)."""
    amax = np.float32(np.max(np.abs(_c(w_f32, np.float32))))
    if amax == 0:
        return 1.0
    return float(np.float32(np.float32(448.0) * np.float32(6.0)) / amax)


def quantize_weight_bf16(w_bits):
    """bf16 weight bits [N,K] -> (packed, scales_swizzled, alpha) per the reference's
    from_bf16_quantized_nvfp4_dev rule: global = 448*6/amax, alpha = 1/global."""
    w_bits = _c(w_bits, np.uint16)
    n, k = w_bits.shape
    g = np.float32(weight_global(bf16_to_f32(w_bits)))
    packed, lin = quantize_rows_bf16(w_bits, float(g))
    return packed, swizzle_scales(lin), float(np.float32(1.0) / g)


# ---- linears ---------------------------------------------------------------------------------
def linear_cpu_backend(w_bf16_bits, x_bits, threads: int = 0) -> np.ndarray:
    w, x = _c(w_bf16_bits, np.uint16), _c(x_bits, np.uint16)
    n, k = w.shape
    m = x.shape[0]
    y = np.zeros((m, n), np.uint16)
    assert lib().nvo_linear_cpu_backend(_p(w, u16p), _p(x, u16p), _p(y, u16p), m, n, k, threads) == 0
    return y


def linear_cpu_backend_lanes16(w_bf16_bits, x_bits, threads: int = 0) -> np.ndarray:
    """The Cpu-backend linear with 16 partial sums per output (the order a SIMD matmul adds in)."""
    w, x = _c(w_bf16_bits, np.uint16), _c(x_bits, np.uint16)
    n, k = w.shape
    m = x.shape[0]
    y = np.zeros((m, n), np.uint16)
    assert lib().nvo_linear_cpu_backend_lanes16(_p(w, u16p), _p(x, u16p), _p(y, u16p), m, n, k, threads) == 0
    return y


def linear_w4a16_f64(packed, scales_sw, x_bits, alpha: float, n: int, k: int) -> np.ndarray:
    p, s, x = _c(packed, np.uint8), _c(scales_sw, np.uint8), _c(x_bits, np.uint16)
    x = x.reshape(-1, k)
    m = x.shape[0]
    y = np.zeros((m, n), np.float64)
    assert lib().nvo_linear_w4a16_f64(_p(p, u8p), _p(s, u8p), _p(x, u16p), np.float32(alpha), m, n, k,
                                      _p(y, f64p)) == 0
    return y


def matmul_w4a4(a_packed, a_scales_lin, b_packed, b_scales_lin, m, n, k, alpha: float = 1.0) -> np.ndarray:
    ap, asl = _c(a_packed, np.uint8), _c(a_scales_lin, np.uint8)
    bp, bsl = _c(b_packed, np.uint8), _c(b_scales_lin, np.uint8)
    d = np.zeros((m, n), np.uint16)
    assert lib().nvo_matmul_w4a4(_p(ap, u8p), _p(asl, u8p), _p(bp, u8p), _p(bsl, u8p), np.float32(alpha),
                                 m, n, k, _p(d, u16p)) == 0
    return d


def silu_mul(gate_bits, up_bits, round_bf16: bool) -> np.ndarray:
    g, u = _c(gate_bits, np.uint16), _c(up_bits, np.uint16)
    out = np.zeros(g.shape, np.float32)
    lib().nvo_silu_mul(_p(g, u16p), _p(u, u16p), g.size, int(round_bf16), _p(out, f32p))
    return out


def moe_route_topk(logits, k: int, bias=None, mode: int = 0, softcap: float = 0.0, norm_topk: bool = True,
                   routed_scaling: float = 1.0):
    lg = _c(logits, np.float32)
    n, e = lg.shape
    ids = np.zeros((n, k), np.int32)
    w = np.zeros((n, k), np.float32)
    b = None if bias is None else _c(bias, np.float32)
    rc = lib().nvo_moe_route_topk(_p(lg, f32p), None if b is None else _p(b, f32p), _p(ids, i32p), _p(w, f32p),
                                  n, e, k, mode, np.float32(softcap), int(norm_topk), np.float32(routed_scaling))
    assert rc == 0
    return ids, w


def moe_unpermute_scatter(y_sorted_bits, weights, inv_perm, hidden: int, row_stride: int) -> np.ndarray:
    y, w, ip = _c(y_sorted_bits, np.uint16), _c(weights, np.float32), _c(inv_perm, np.int32)
    n, k = w.shape
    out = np.zeros((n, hidden), np.float32)
    lib().nvo_moe_unpermute_scatter(_p(y, u16p), _p(w, f32p), _p(ip, i32p), _p(out, f32p), n, k, hidden, row_stride)
    return out


def rowquant_i8(x_f32):
    """Per-row int8 quantizer of the W4A8 route: scale = max|x| / 127 (f32), q = clamp(rn(x * (1 / scale)), +-127),
    ties to even -- the host statement in rust/crates/nv-kernels/tests/gemv_nvfp4_w4a8_decode_parity.rs:19-29
    (and cuda/gemv_nvfp4_w4a8_decode.cu:146-183).  x [rows, K] f32 -> (q int8 [rows, K], scales f32 [rows])."""
    x = np.atleast_2d(_c(x_f32, np.float32))
    amax = np.max(np.abs(x), axis=1).astype(np.float32)
    scale = (amax / np.float32(127.0)).astype(np.float32)
    inv = np.where(scale > 0, np.float32(1.0) / np.where(scale > 0, scale, np.float32(1.0)), np.float32(0.0)).astype(np.float32)
    q = np.clip(np.rint((x * inv[:, None]).astype(np.float32)), -127, 127).astype(np.int8)   # rint: ties to even
    return q, scale


def linear_w4a8_f64(packed, scales_sw, q_i8, x_scales, alpha: float, n: int, k: int, residual_bits=None) -> np.ndarray:
    """y = residual + alpha * scale[m] * sum_k W[n,k] q[m,k] in f64 (integer-exact block dots): the
    "int8 mechanics oracle" of gemv_nvfp4_w4a8_decode_parity.rs:130-190."""
    w = dequantize_packed_swizzled(packed, scales_sw, n, k, 1.0).astype(np.float64).reshape(n, k)
    q = np.atleast_2d(np.asarray(q_i8)).astype(np.float64)
    y = (q @ w.T) * (np.float64(np.float32(alpha)) * np.asarray(x_scales, np.float32).astype(np.float64))[:, None]
    if residual_bits is not None:
        y = y + bf16_to_f32(residual_bits).astype(np.float64).reshape(y.shape)
    return y


def rmsnorm_residual(x_bits, res_bits, w_bits, eps: float):
    """s = x + res (f32), res_out = bf16(s), rstd = 1 / sqrt(mean(s^2) + eps) with s unrounded, v =
    bf16(res_out * rstd * w): rust/crates/nv-kernels/cuda/rmsnorm_residual_writeout.cu:6-52.  Returns
    (res_out bits, v bits), the mean taken in f64 (the device sums in f32 in its own order)."""
    s = bf16_to_f32(x_bits) + bf16_to_f32(res_bits)
    res_out = f32_to_bf16(s)
    rstd = np.float32(1.0 / np.sqrt(np.mean(s.astype(np.float64) ** 2, axis=-1, keepdims=True) + np.float64(np.float32(eps))))
    v = f32_to_bf16((bf16_to_f32(res_out) * rstd).astype(np.float32) * bf16_to_f32(w_bits))
    return res_out, v


def num_threads() -> int:
    return int(lib().nvo_num_threads())
