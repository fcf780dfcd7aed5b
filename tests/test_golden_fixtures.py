"""The committed golden fixture (tests/golden/nvfp4_small.npz, written by tests/golden/make_golden.py):
the oracle must still reproduce every array in it exactly, and the CUDA path must agree with it --
bytes, indices and bf16 bits exactly, the contraction within the stated tolerance."""
import pathlib

import numpy as np
import pytest
import torch

from oracle import ref

GOLDEN = pathlib.Path(__file__).parent / "golden" / "nvfp4_small.npz"
TOL = 1e-4 + 1e-2   # the reference's GEMV bound, rust/crates/nv-quant/tests/nvfp4_m1_gemv_ab.rs:103-118


@pytest.fixture(scope="module")
def g():
    return dict(np.load(GOLDEN))


def test_generator_reproduces_the_committed_file(g):
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", GOLDEN.with_name("make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    fresh = mod.build()
    assert sorted(fresh) == sorted(g)
    for name, want in g.items():
        assert fresh[name].dtype == want.dtype and np.array_equal(fresh[name], want), name


def test_fixture_is_self_consistent(g):
    n, k = g["w_packed"].shape[0], g["w_packed"].shape[1] * 2
    assert np.array_equal(ref.unswizzle_scales(g["w_scales_swizzled"], n, k // 16), g["w_scales_linear"])
    # quantization error of a 4-bit block format: every weight within half a code step of its block scale
    deq = ref.dequantize_packed_linear(g["w_packed"], g["w_scales_linear"], n, k, float(g["alpha"][0]))
    w = ref.bf16_to_f32(g["w_bf16"])
    blk_max = np.abs(w).reshape(n, k // 16, 16).max(-1, keepdims=True)
    assert np.all(np.abs(deq - w).reshape(n, k // 16, 16) <= blk_max / 6 * 1.07 + 1e-7)
    # the tie at the top of the last router row goes to the lower index
    assert g["router_ids"][5, 0] == 10 and g["router_ids"][5, 1] == 70
    assert np.allclose(g["router_weights"].sum(-1), 1.0, atol=1e-6)


# ---- the CUDA path against the fixture -------------------------------------------------------
@pytest.mark.gpu
def test_cuda_path_matches_the_fixture(g):
    from tests import _util as U
    U.require_gpu()
    import speaches_plus_b200 as sp
    n, k = g["w_packed"].shape[0], g["w_packed"].shape[1] * 2
    # weight quantizer: bytes, scales and global
    w_dev = U.dev(g["w_bf16"]).view(torch.bfloat16)
    packed, scales, alpha, stored = sp.quantize_weight_nvfp4(w_dev)
    torch.cuda.synchronize()
    assert np.float32(stored) == g["w_global"][0] and np.float32(alpha) == g["alpha"][0]
    assert np.array_equal(packed.cpu().numpy().reshape(n, k // 2), g["w_packed"])
    assert np.array_equal(scales.cpu().numpy()[: g["w_scales_swizzled"].size], g["w_scales_swizzled"])
    # W4A16 linear, M = 1 and M = 5
    lin = sp.Nvfp4Linear.new_nvfp4(U.dev(g["w_packed"]), U.dev(g["w_scales_swizzled"]), float(g["alpha"][0]), k, n)
    x = U.dev(g["x_bf16"]).view(torch.bfloat16)
    y5, y1 = lin.forward(x), lin.forward(x[:1].contiguous())
    torch.cuda.synchronize()
    assert U.rel_err_floor(y5.float().cpu().numpy(), g["y_f64"]) < TOL
    assert torch.equal(y5[:1].contiguous().view(torch.int16), y1.view(torch.int16))   # the same bits at any M
    assert U.rel_err_floor(y5.float().cpu().numpy(), ref.bf16_to_f32(g["y_cpu_backend_bf16"])) < 1.5e-2
    # activation quantizer, padded to 128 rows
    from speaches_plus_b200.linear import quantize_nvfp4_bf16
    a_packed, a_scales = quantize_nvfp4_bf16(x, 1.0, m_padded=128)
    torch.cuda.synchronize()
    assert np.array_equal(a_packed.cpu().numpy().reshape(128, k // 2), g["a_packed"])
    assert np.array_equal(a_scales.cpu().numpy()[: g["a_scales_swizzled"].size], g["a_scales_swizzled"])
    # router
    E, top_k = g["router_logits"].shape[1], g["router_ids"].shape[1]
    ids = torch.zeros((6, top_k), dtype=torch.int32, device="cuda")
    wts = torch.zeros((6, top_k), dtype=torch.float32, device="cuda")
    lg = U.dev(g["router_logits"])
    rc = U.ffi.call("nv_kernels_moe_route_topk", U.stream(), lg.data_ptr(), None, ids.data_ptr(), wts.data_ptr(),
                    6, E, top_k, 0, 0.0, 1, 1.0)
    assert rc == 0
    torch.cuda.synchronize()
    assert np.array_equal(ids.cpu().numpy(), g["router_ids"])
    assert np.allclose(wts.cpu().numpy(), g["router_weights"], rtol=2e-6, atol=1e-7)


@pytest.mark.gpu
def test_cuda_path_matches_the_fixture_routers_sort_w4a8_and_norm(g):
    """The second half of the fixture: the sigmoid router, the stable slot sort, the W4A8 product on the
    fixture's int8 rows (with and without a residual), and the residual RMSNorm."""
    from tests import _util as U
    from tests.test_gpu_w4a8 import TOL as W4A8_TOL, rel_quarter, w4a8
    U.require_gpu()
    n, k = g["w_packed"].shape[0], g["w_packed"].shape[1] * 2
    # sigmoid router with bias and routed scaling
    lg, bias = U.dev(g["router1_logits"]), U.dev(g["router1_bias"])
    rows, E = g["router1_logits"].shape
    top_k = g["router1_ids"].shape[1]
    ids = torch.zeros((rows, top_k), dtype=torch.int32, device="cuda")
    wts = torch.zeros((rows, top_k), dtype=torch.float32, device="cuda")
    assert U.ffi.call("nv_kernels_moe_route_topk", U.stream(), lg.data_ptr(), bias.data_ptr(), ids.data_ptr(),
                      wts.data_ptr(), rows, E, top_k, 1, 0.0, 1, 2.5) == 0
    torch.cuda.synchronize()
    assert np.array_equal(ids.cpu().numpy(), g["router1_ids"])
    assert np.allclose(wts.cpu().numpy(), g["router1_weights"], rtol=2e-6, atol=1e-7)
    # stable slot sort of the first router's ids
    r_ids = U.dev(g["router_ids"])
    n_tok, kk = g["router_ids"].shape
    perm = torch.zeros(n_tok * kk, dtype=torch.int32, device="cuda")
    offs = torch.zeros(129, dtype=torch.int32, device="cuda")
    inv = torch.zeros(n_tok * kk, dtype=torch.int32, device="cuda")
    scr = torch.zeros(128, dtype=torch.int32, device="cuda")
    assert U.ffi.call("nv_kernels_moe_permute", U.stream(), r_ids.data_ptr(), perm.data_ptr(), offs.data_ptr(),
                      inv.data_ptr(), scr.data_ptr(), n_tok, kk, 128) == 0
    torch.cuda.synchronize()
    assert np.array_equal(offs.cpu().numpy(), g["sort_offsets"])
    assert np.array_equal(perm.cpu().numpy(), g["sort_perm_token"])
    assert np.array_equal(inv.cpu().numpy(), g["sort_inv_perm"])
    # W4A8: the oracle's row quantizer reproduces the stored integers; the product on them
    q, sc = ref.rowquant_i8(g["x8_f32"])
    assert np.array_equal(q, g["x8_q"]) and np.array_equal(sc, g["x8_scales"])
    wts_ = (g["w_packed"], g["w_scales_swizzled"], float(g["alpha"][0]))
    y = w4a8("nv_kernels_gemv_nvfp4_w4a8_down_residual_mk", wts_, g["x8_q"], g["x8_scales"], 3, n, k)
    assert rel_quarter(y, g["y_w4a8_f64"]) < W4A8_TOL
    yr = w4a8("nv_kernels_gemv_nvfp4_w4a8_down_residual_mk", wts_, g["x8_q"], g["x8_scales"], 3, n, k,
              residual=g["w4a8_residual_bf16"])
    assert rel_quarter(yr, g["y_w4a8_residual_f64"]) < W4A8_TOL
    # residual RMSNorm: the new residual is exact, the normed row within a bf16 step of the oracle's
    hx, hres, hw = U.dev(g["norm_x_bf16"]), U.dev(g["norm_res_bf16"]), U.dev(g["norm_w_bf16"])
    b, hidden = g["norm_x_bf16"].shape
    res_out = torch.zeros((b, hidden), dtype=torch.int16, device="cuda")
    v = torch.zeros((b, hidden), dtype=torch.int16, device="cuda")
    assert U.ffi.call("nv_kernels_rmsnorm_residual_writeout_bf16", U.stream(), hx.data_ptr(), hres.data_ptr(),
                      hw.data_ptr(), res_out.data_ptr(), v.data_ptr(), b, hidden, 1e-6) == 0
    torch.cuda.synchronize()
    assert np.array_equal(U.host_u16(res_out), g["norm_res_out_bf16"])
    assert np.max(U.bf16_ulp_diff(U.host_u16(v), g["norm_out_bf16"])) <= 1
