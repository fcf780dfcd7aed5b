"""GPU parity of the prefill-sized block-scaled FP4 x FP4 GEMM (tcgen05 kind::mxf4nvf4) against the
reference's W4A4 host oracle (rust/crates/nv-quant/src/nvfp4.rs:1086-1106: dequantize both operands,
sequential f32 dot, bf16 out).

Tolerance: the tensor core sums the same exact products in a different order, so results agree to
fp32 accumulation noise before the bf16 rounding: at most 2 bf16 ulp (or 1e-3 absolute near zero) per
element, and < 1e-2 in the floored relative form used for the linear path."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import ref
from tests import _util as U

pytestmark = pytest.mark.gpu


def run_gemm(ap, asw, bp, bsw, alpha, m, n, k, entry="nv_kernels_cutlass_fp4_gemm_sm120_bf16"):
    d = [U.dev(a) for a in (ap, asw, bp, bsw)]
    al = torch.tensor([alpha], dtype=torch.float32, device="cuda")
    out = torch.full((m * n + 64,), 0x7FC0, dtype=torch.int16, device="cuda")
    need = ctypes.c_size_t(0)
    extra = [0, 0] if entry.endswith("_tiled") else []
    assert U.ffi.call(entry, U.stream(), None, None, None, None, None, None, m, n, k, *extra, None, 0,
                      ctypes.addressof(need)) == 0  # size query
    ws = torch.zeros(max(need.value, 16), dtype=torch.uint8, device="cuda")
    rc = U.ffi.call(entry, U.stream(), d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(),
                    al.data_ptr(), out.data_ptr(), m, n, k, *extra, ws.data_ptr(), ws.numel(), ctypes.addressof(need))
    assert rc == 0
    torch.cuda.synchronize()
    o = U.host_u16(out)
    assert np.all(o[m * n:] == 0x7FC0)
    return o[:m * n].reshape(m, n)


def quantized_operand(rng, rows, k, std, global_=None):
    x = U.gauss_bf16(rng, (rows, k), std)
    g = ref.weight_global(ref.bf16_to_f32(x)) if global_ is None else global_
    packed, lin = ref.quantize_rows_bf16(x, g)
    return packed, lin, ref.swizzle_scales(lin), g


@pytest.fixture(params=[2, 1], ids=["2sm", "1sm"])
def tile_config(request):
    assert U.ffi.call("nvk_b200_set_prefill_config", request.param) == 0
    yield request.param
    U.ffi.call("nvk_b200_set_prefill_config", 2)


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 384, 512), (130, 264, 1056), (2048, 512, 768)])
def test_block_scaled_gemm_matches_w4a4_oracle(m, n, k, tile_config):
    U.require_gpu()
    rng = np.random.default_rng(m + n + k)
    ap, alin, asw, _ = quantized_operand(rng, m, k, 1.0, 1.0)
    bp, blin, bsw, gb = quantized_operand(rng, n, k, 0.02)
    alpha = float(np.float32(1.0) / np.float32(gb))
    # the scale buffer of A is padded to whole 128-row tiles
    got = run_gemm(ap, asw, bp, bsw, alpha, m, n, k)
    want = ref.matmul_w4a4(ap, alin, bp, blin, m, n, k, alpha)
    ulp = U.bf16_ulp_diff(got, want)
    absd = np.abs(ref.bf16_to_f32(got) - ref.bf16_to_f32(want))
    assert np.all((ulp <= 2) | (absd <= 1e-3)), f"max ulp {ulp.max()}"
    assert U.rel_err_floor(ref.bf16_to_f32(got), ref.bf16_to_f32(want).astype(np.float64)) < 1e-2
    if (m, n, k) == (256, 384, 512):
        for entry in ("nv_kernels_cutlass_fp4_gemm_sm120_bf16_streamk", "nv_kernels_cutlass_fp4_gemm_sm120_bf16_tiled"):
            assert np.array_equal(run_gemm(ap, asw, bp, bsw, alpha, m, n, k, entry), got)


def test_linear_prefill_route_and_chunk_invariance(tile_config):
    """Nvfp4Linear with M > 64 takes the W4A4 route: equals the oracle on the same quantized bytes, and
    (rust/crates/nv-layers/tests/nvfp4_chunk_invariance.rs) is bit-identical under row chunking."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(9)
    m, n, k = 512, 1024, 1024
    w = U.gauss_bf16(rng, (n, k), 0.02)
    packed, sw, alpha = ref.quantize_weight_bf16(w)
    lin = sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(sw), alpha, k, n)
    x = U.gauss_bf16(rng, (m, k))
    xt = U.dev(x).view(torch.bfloat16)
    y = lin(xt)
    torch.cuda.synchronize()
    got = U.host_u16(y)
    ap, alin = ref.quantize_rows_bf16(x, 1.0)
    want = ref.matmul_w4a4(ap, alin, packed, ref.unswizzle_scales(sw, n, k // 16), m, n, k, alpha)
    ulp = U.bf16_ulp_diff(got, want)
    absd = np.abs(ref.bf16_to_f32(got) - ref.bf16_to_f32(want))
    assert np.all((ulp <= 2) | (absd <= 1e-3))
    for chunk in (256, 128):
        parts = [U.host_u16(lin(xt[r:r + chunk].contiguous())) for r in range(0, m, chunk)]
        torch.cuda.synchronize()
        assert np.array_equal(np.concatenate(parts, 0), got), f"chunk {chunk}"


def test_refusals_and_workspace_protocol():
    U.require_gpu()
    need = ctypes.c_size_t(123)
    f = U.ffi.call
    e = "nv_kernels_cutlass_fp4_gemm_sm120_bf16"
    assert f(e, U.stream(), None, None, None, None, None, None, 128, 128, 100, None, 0, ctypes.addressof(need)) == -1
    assert f(e, U.stream(), None, None, None, None, None, None, 128, 100, 128, None, 0, ctypes.addressof(need)) == -1
    assert f(e, U.stream(), None, None, None, None, None, None, 0, 128, 128, None, 0, ctypes.addressof(need)) == -1
    assert f(e, U.stream(), None, None, None, None, None, None, 256, 256, 256, None, 0, ctypes.addressof(need)) == 0
    t = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    # data pointers but no alpha -> argument error
    assert f(e, U.stream(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None, t.data_ptr(), 128, 128, 128,
             None, 0, ctypes.addressof(need)) == -2
    torch.cuda.synchronize()
