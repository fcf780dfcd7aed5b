"""GPU parity of the W4A16 NVFP4 linear against the CPU oracle, through the C ABI.

Tolerances (written here, as the contract asks):
  * vs the f64 statement of the contraction: |got-want| / max(|want|, rms, 1e-3) < 1e-4 + 1e-2 -- the
    reference's own GEMV bound (rust/crates/nv-quant/tests/nvfp4_m1_gemv_ab.rs:103-118), i.e.
    fp32-accumulate noise plus bf16 output rounding; in practice the worst case is ~2^-9.
  * vs the reference's Cpu-backend linear (weights dequantized to bf16, f32 matmul, bf16 out):
    max relative error < 1e-2 with the same floored denominator for K >= 1024 (every benchmark
    shape).  That path rounds every weight to bf16 (2^-9 relative each) and both sides round the
    output to bf16, so for short rows the two roundings plus the weight noise can by themselves
    reach 1e-2; below K = 1024 the bound used is 1.5e-2 (the f64 bound above still applies).
"""
import numpy as np
import pytest
import torch

from oracle import ref
from tests import _util as U

pytestmark = pytest.mark.gpu

TOL_F64 = 1e-4 + 1e-2
TOL_CPU_BACKEND = 1e-2


def run_gemv(packed, sw, x_bits, alpha, n, k, entry="nv_kernels_nvfp4_gemv_bf16act"):
    d_w, d_s, d_x = U.dev(packed), U.dev(sw), U.dev(x_bits)
    y = torch.full((n + 64,), 0x7FC0, dtype=torch.int16, device="cuda")  # canary tail
    rc = U.ffi.call(entry, U.stream(), d_w.data_ptr(), d_s.data_ptr(), d_x.data_ptr(), y.data_ptr(), float(alpha),
                    n, k)
    assert rc == 0
    torch.cuda.synchronize()
    out = U.host_u16(y)
    assert np.all(out[n:] == 0x7FC0), "wrote past the end of y"
    return out[:n]


def run_linear(packed, sw, x_bits, alpha, m, n, k, packed_b=None, sw_b=None, alpha_b=0.0, up_bits=None):
    d = [U.dev(packed), U.dev(sw), U.dev(x_bits)]
    db = [U.dev(packed_b), U.dev(sw_b)] if packed_b is not None else None
    du = U.dev(up_bits) if up_bits is not None else None
    y = torch.full((m * n + 64,), 0x7FC0, dtype=torch.int16, device="cuda")
    yb = torch.full((m * n + 64,), 0x7FC0, dtype=torch.int16, device="cuda") if db else None
    rc = U.ffi.call("nvk_b200_linear_nvfp4_w4a16", U.stream(), d[0].data_ptr(), d[1].data_ptr(),
                    db[0].data_ptr() if db else None, db[1].data_ptr() if db else None, d[2].data_ptr(),
                    du.data_ptr() if du is not None else None, y.data_ptr(), yb.data_ptr() if db else None,
                    float(alpha), float(alpha_b), m, n, k)
    assert rc == 0
    torch.cuda.synchronize()
    out = U.host_u16(y)
    assert np.all(out[m * n:] == 0x7FC0)
    if db:
        outb = U.host_u16(yb)
        assert np.all(outb[m * n:] == 0x7FC0)
        return out[:m * n].reshape(m, n), outb[:m * n].reshape(m, n)
    return out[:m * n].reshape(m, n)


def check_against_oracle(got_bits, packed, sw, x_bits, alpha, n, k, cpu_backend=True):
    got = ref.bf16_to_f32(got_bits).reshape(-1, n)
    want = ref.linear_w4a16_f64(packed, sw, x_bits, alpha, n, k)
    e = U.rel_err_floor(got, want)
    assert e < TOL_F64, f"vs f64 oracle: {e}"
    if cpu_backend:
        w_bf16 = ref.dequantize_to_bf16(packed, sw, n, k, alpha)
        want2 = ref.bf16_to_f32(ref.linear_cpu_backend(w_bf16, np.asarray(x_bits).reshape(-1, k)))
        e2 = U.rel_err_floor(got, want2)
        assert e2 < (TOL_CPU_BACKEND if k >= 1024 else 1.5e-2), f"vs Cpu-backend linear: {e2}"
    return e


def test_capability_is_sm100():
    U.require_gpu()
    assert U.ffi.capability() == (10, 0)


def test_config0_single_linear_seed0():
    """The single-linear case the reference's Cpu backend can run: x [1,4096] ~ N(0,1), W [4096,4096] ~ N(0,0.02), seed 0."""
    U.require_gpu()
    rng = np.random.default_rng(0)
    x = U.gauss_bf16(rng, (1, 4096))
    packed, sw, alpha, _ = U.make_weight(rng, 4096, 4096)
    got = run_gemv(packed, sw, x, alpha, 4096, 4096)
    e = check_against_oracle(got, packed, sw, x, alpha, 4096, 4096)
    assert e < 6e-3  # bf16 output rounding (2^-9 ~ 2e-3 of |want|, relative to the floored denominator)


def sin_bf16(n, seed, scale):
    j = np.arange(n, dtype=np.float32)
    return ref.f32_to_bf16(np.sin(j * np.float32(seed)).astype(np.float32) * np.float32(scale))


@pytest.mark.parametrize("n,k,alpha", [(64, 256, 1.0), (129, 1024, 1.0), (640, 5376, 0.5), (5376, 5376, 1.0)])
def test_m1_gemv_reference_shapes(n, k, alpha):
    """Shapes, generators and bound of rust/crates/nv-quant/tests/nvfp4_m1_gemv_ab.rs:61-120
    (sin-wave weights quantized with global 1.0, sin-wave x times 2)."""
    U.require_gpu()
    w = sin_bf16(n * k, 0.00071, 1.0).reshape(n, k)
    packed, lin = ref.quantize_rows_bf16(w, 1.0)
    sw = ref.swizzle_scales(lin)
    x = sin_bf16(k, 0.00131, 2.0).reshape(1, k)
    got = run_gemv(packed, sw, x, alpha, n, k)
    check_against_oracle(got, packed, sw, x, alpha, n, k, cpu_backend=False)


@pytest.mark.parametrize("n", [1, 7, 8, 9, 31, 33, 127, 128, 129, 255, 257])
@pytest.mark.parametrize("k", [16, 32, 48, 64, 128, 144, 256, 272, 1040])
def test_m1_ragged_shapes(n, k):
    """Every residue class the launch geometry cares about: N around the 8/32/128 row groupings,
    K around the 16/32/64/256 groupings (K % 32 != 0 takes the generic route)."""
    U.require_gpu()
    rng = np.random.default_rng(1000 * n + k)
    packed, sw, alpha, _ = U.make_weight(rng, n, k, std=0.5)
    x = U.gauss_bf16(rng, (1, k))
    got = run_gemv(packed, sw, x, alpha, n, k)
    check_against_oracle(got, packed, sw, x, alpha, n, k, cpu_backend=False)


@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 9, 11, 16, 17, 31, 32, 33, 63, 64])
@pytest.mark.parametrize("n,k", [(256, 512), (96, 320), (384, 4096)])
def test_skinny_m_sweep(m, n, k):
    U.require_gpu()
    rng = np.random.default_rng(7 * m + n + k)
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    x = U.gauss_bf16(rng, (m, k))
    got = run_linear(packed, sw, x, alpha, m, n, k)
    check_against_oracle(got, packed, sw, x, alpha, n, k)


@pytest.mark.parametrize("ks", [1, 2, 4, 8])
def test_cluster_split_k_is_consistent(ks):
    """Every cluster size gives the oracle's answer (the partial tiles are summed through
    distributed shared memory in a fixed order), and each is bit-stable run to run."""
    U.require_gpu()
    rng = np.random.default_rng(42)
    n, k, m = 384, 2048 + 256, 4
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    x = U.gauss_bf16(rng, (m, k))
    assert U.ffi.call("nvk_b200_set_tuning", ks, 0) == 0
    try:
        a = run_linear(packed, sw, x, alpha, m, n, k)
        b = run_linear(packed, sw, x, alpha, m, n, k)
    finally:
        U.ffi.call("nvk_b200_set_tuning", 0, 0)
    assert np.array_equal(a, b)
    check_against_oracle(a, packed, sw, x, alpha, n, k)


@pytest.mark.parametrize("rows", [16, 32, 64, 128])
@pytest.mark.parametrize("m", [1, 7, 16])
def test_rows_per_cta_variants_agree(rows, m):
    """Each CTA shape (16/32/64/128 weight rows per CTA) gives the oracle's answer."""
    U.require_gpu()
    rng = np.random.default_rng(rows + m)
    n, k = 640 + 40, 1536
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    x = U.gauss_bf16(rng, (m, k))
    assert U.ffi.call("nvk_b200_set_tuning", 0, rows) == 0
    try:
        got = run_linear(packed, sw, x, alpha, m, n, k)
    finally:
        U.ffi.call("nvk_b200_set_tuning", 0, 0)
    check_against_oracle(got, packed, sw, x, alpha, n, k)


@pytest.mark.parametrize("m", [1, 5, 16])
@pytest.mark.parametrize("dual", [False, True])
def test_units_dealt_over_a_full_grid_give_the_same_bits(m, dual):
    """The launch that deals 16-row units round-robin over 148 * r CTAs (forced here on a small matrix
    whose last 128-row tile is ragged, so most warps idle) gives bit for bit what one CTA per 128-row
    tile gives, for one and for two arms, and both give the oracle's answer."""
    U.require_gpu()
    rng = np.random.default_rng(90 + m)
    n, k = 3 * 128 + 40, 768
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    packed_b, sw_b, alpha_b, _ = U.make_weight(rng, n, k) if dual else (None, None, 0.0, None)
    x = U.gauss_bf16(rng, (m, k))
    outs = []
    for mode in (2, 1):
        assert U.ffi.call("nvk_b200_set_row_balance", mode) == 0
        try:
            outs.append(run_linear(packed, sw, x, alpha, m, n, k, packed_b, sw_b, alpha_b))
        finally:
            U.ffi.call("nvk_b200_set_row_balance", 0)
    if dual:
        assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
        check_against_oracle(outs[1][0], packed, sw, x, alpha, n, k)
        check_against_oracle(outs[1][1], packed_b, sw_b, x, alpha_b, n, k)
    else:
        assert np.array_equal(outs[0], outs[1])
        check_against_oracle(outs[1], packed, sw, x, alpha, n, k)


def test_row_balance_is_chosen_for_a_one_and_a_half_wave_launch():
    """150 row tiles on 148 SMs: the automatic choice deals the 1200 units over 296 CTAs (five warps busy in
    most of them); the result equals the per-tile launch bit for bit."""
    U.require_gpu()
    rng = np.random.default_rng(17)
    n, k, m = 150 * 128, 256, 2
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    x = U.gauss_bf16(rng, (m, k))
    auto = run_linear(packed, sw, x, alpha, m, n, k)
    assert U.ffi.call("nvk_b200_set_row_balance", 2) == 0
    try:
        per_tile = run_linear(packed, sw, x, alpha, m, n, k)
    finally:
        U.ffi.call("nvk_b200_set_row_balance", 0)
    assert np.array_equal(auto, per_tile)
    check_against_oracle(auto, packed, sw, x, alpha, n, k, cpu_backend=False)


def run_residual(packed, sw, x_bits, resid_bits, alpha, m, n, k, up_bits=None, in_place=False):
    d = [U.dev(packed), U.dev(sw), U.dev(x_bits)]
    du = U.dev(up_bits) if up_bits is not None else None
    y = torch.full((m * n + 64,), 0x7FC0, dtype=torch.int16, device="cuda")
    if in_place:
        y[:m * n] = U.dev(resid_bits).view(torch.int16).reshape(-1)
        r_ptr = y.data_ptr()
    else:
        dr = U.dev(resid_bits)
        r_ptr = dr.data_ptr()
    rc = U.ffi.call("nvk_b200_linear_nvfp4_w4a16_residual", U.stream(), d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(),
                    du.data_ptr() if du is not None else None, r_ptr, y.data_ptr(), float(alpha), m, n, k)
    assert rc == 0
    torch.cuda.synchronize()
    out = U.host_u16(y)
    assert np.all(out[m * n:] == 0x7FC0)
    return out[:m * n].reshape(m, n)


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 33, 64])
@pytest.mark.parametrize("n,k", [(384, 768), (200, 2304), (2048, 256)])
def test_residual_epilogue_matches_the_oracle(m, n, k):
    """y = bf16(residual + alpha * x W^T), one rounding: against the f64 statement of the product plus
    the residual, with the linear's bound (the floor of the denominator is the rms of the expected
    output); updating the residual in place gives the same bits as writing elsewhere."""
    U.require_gpu()
    rng = np.random.default_rng(m + n + k)
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    x = U.gauss_bf16(rng, (m, k))
    resid = U.gauss_bf16(rng, (m, n), 2.0)
    got = run_residual(packed, sw, x, resid, alpha, m, n, k)
    want = ref.linear_w4a16_f64(packed, sw, x, alpha, n, k) + ref.bf16_to_f32(resid).astype(np.float64)
    assert U.rel_err_floor(ref.bf16_to_f32(got), want) < TOL_F64
    assert np.array_equal(run_residual(packed, sw, x, resid, alpha, m, n, k, in_place=True), got)
    # a zero residual leaves the plain linear, bit for bit (fma(v, alpha, 0) == v * alpha)
    zero = np.zeros((m, n), np.uint16)
    assert np.array_equal(run_residual(packed, sw, x, zero, alpha, m, n, k), run_linear(packed, sw, x, alpha, m, n, k))


@pytest.mark.parametrize("m", [1, 5, 20])
def test_mlp_tail_in_one_launch(m):
    """SiLU(gate) * up prologue + down projection + residual: equals the prologue linear followed by an
    addition in f64 within the bound, and Nvfp4Mlp.forward_residual uses it."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(40 + m)
    hidden, inter = 256, 640
    wts = [U.make_weight(rng, n, k)[:3] for (n, k) in ((inter, hidden), (inter, hidden), (hidden, inter))]
    lins = [sp.Nvfp4Linear.new_nvfp4(U.dev(p), U.dev(s_), a, k, n)
            for (p, s_, a), (n, k) in zip(wts, ((inter, hidden), (inter, hidden), (hidden, inter)))]
    mlp = sp.Nvfp4Mlp(*lins)
    x = U.gauss_bf16(rng, (m, hidden))
    resid = U.gauss_bf16(rng, (m, hidden), 1.5)
    xt, rt = U.dev(x).view(torch.bfloat16), U.dev(resid).view(torch.bfloat16)
    y_plain = U.host_u16(mlp(xt))
    y_res = U.host_u16(mlp.forward_residual(xt, rt))
    want = ref.bf16_to_f32(y_plain).astype(np.float64) + ref.bf16_to_f32(resid).astype(np.float64)
    # y_plain is itself rounded to bf16: allow that rounding on top of the fused result's own
    assert U.rel_err_floor(ref.bf16_to_f32(y_res), want) < 1.2e-2
    gate, up = U.gauss_bf16(rng, (m, inter)), U.gauss_bf16(rng, (m, inter))
    got = run_residual(wts[2][0], wts[2][1], gate, resid, wts[2][2], m, hidden, inter, up_bits=up)
    act = ref.f32_to_bf16(ref.silu_mul(gate, up, round_bf16=True))
    want2 = ref.linear_w4a16_f64(wts[2][0], wts[2][1], act, wts[2][2], hidden, inter) + ref.bf16_to_f32(resid).astype(np.float64)
    assert U.rel_err_floor(ref.bf16_to_f32(got), want2) < 2e-2


def run_normed(wa, x_bits, norm_bits, eps, m, n, k, wb=None, rstd=None):
    d = [U.dev(wa[0]), U.dev(wa[1]), U.dev(x_bits), U.dev(norm_bits)]
    db = [U.dev(wb[0]), U.dev(wb[1])] if wb is not None else None
    dr = U.dev(np.asarray(rstd, np.float32)) if rstd is not None else None
    y = torch.full((m * n + 64,), 0x7FC0, dtype=torch.int16, device="cuda")
    yb = torch.full((m * n + 64,), 0x7FC0, dtype=torch.int16, device="cuda") if db else None
    rc = U.ffi.call("nvk_b200_linear_nvfp4_w4a16_normed", U.stream(), d[0].data_ptr(), d[1].data_ptr(),
                    db[0].data_ptr() if db else None, db[1].data_ptr() if db else None, d[2].data_ptr(), d[3].data_ptr(),
                    dr.data_ptr() if dr is not None else None, float(eps), y.data_ptr(), yb.data_ptr() if db else None,
                    float(wa[2]), float(wb[2]) if wb is not None else 0.0, m, n, k)
    assert rc == 0
    torch.cuda.synchronize()
    out = U.host_u16(y)
    assert np.all(out[m * n:] == 0x7FC0)
    if db:
        outb = U.host_u16(yb)
        assert np.all(outb[m * n:] == 0x7FC0)
        return out[:m * n].reshape(m, n), outb[:m * n].reshape(m, n)
    return out[:m * n].reshape(m, n)


def device_rmsnorm(x_bits, norm_bits, eps):
    m, k = x_bits.shape
    dx, dw = U.dev(x_bits), U.dev(norm_bits)
    out = torch.zeros((m, k), dtype=torch.int16, device="cuda")
    assert U.ffi.call("nv_kernels_rmsnorm_bf16", U.stream(), dx.data_ptr(), dw.data_ptr(), out.data_ptr(), m, k,
                      float(eps)) == 0
    torch.cuda.synchronize()
    return U.host_u16(out)


@pytest.mark.parametrize("m", [1, 3, 8])
@pytest.mark.parametrize("n,k,dual", [(384, 1024, False), (256, 2560, True), (130, 4352, False)])
def test_norm_in_the_prologue_equals_norm_then_linear_bitwise(m, n, k, dual):
    """RMSNorm applied while the activations are staged == nv_kernels_rmsnorm_bf16 followed by the plain
    linear, bit for bit (one and two matrices, K split over a cluster at the small N), and both give the
    oracle's answer for the normed rows."""
    U.require_gpu()
    rng = np.random.default_rng(m + n + k)
    wa = U.make_weight(rng, n, k)[:3]
    wb = U.make_weight(rng, n, k)[:3] if dual else None
    x = U.gauss_bf16(rng, (m, k), 3.0)
    nw = U.gauss_bf16(rng, (k,), 1.0)
    eps = 1e-6
    normed = device_rmsnorm(x, nw, eps)
    if dual:
        fa, fb = run_normed(wa, x, nw, eps, m, n, k, wb)
        pa, pb = run_linear(wa[0], wa[1], normed, wa[2], m, n, k, wb[0], wb[1], wb[2])
        assert np.array_equal(fa, pa) and np.array_equal(fb, pb)
    else:
        fa = run_normed(wa, x, nw, eps, m, n, k)
        assert np.array_equal(fa, run_linear(wa[0], wa[1], normed, wa[2], m, n, k))
    xf = ref.bf16_to_f32(x)
    rstd = (1.0 / np.sqrt((xf.astype(np.float64) ** 2).mean(1) + eps)).astype(np.float32)
    want_rows = ref.f32_to_bf16((xf * rstd[:, None]) * ref.bf16_to_f32(nw)[None, :])
    want = ref.linear_w4a16_f64(wa[0], wa[1], want_rows, wa[2], n, k)
    assert U.rel_err_floor(ref.bf16_to_f32(fa), want) < 2e-2     # a normed value may round to a neighbouring bf16


def test_norm_with_rstd_handed_in_and_the_emit_consume_chain():
    """(i) rstd given per row, 20 rows: the oracle's answer.  (ii) One row through a layer boundary: the
    residual-update launch leaves rstd of the new hidden row, the normed linear of the next layer takes
    it; the result equals norm + linear on that row up to the last bits of rstd."""
    U.require_gpu()
    rng = np.random.default_rng(91)
    n, k, eps = 256, 768, 1e-5
    wa = U.make_weight(rng, n, k)[:3]
    nw = U.gauss_bf16(rng, (k,), 1.0)
    x = U.gauss_bf16(rng, (20, k), 2.0)
    xf = ref.bf16_to_f32(x)
    rstd = (1.0 / np.sqrt((xf.astype(np.float64) ** 2).mean(1) + eps)).astype(np.float32)
    got = run_normed(wa, x, nw, eps, 20, n, k, rstd=rstd)
    rows = ref.f32_to_bf16((xf * rstd[:, None]) * ref.bf16_to_f32(nw)[None, :])
    assert U.rel_err_floor(ref.bf16_to_f32(got), ref.linear_w4a16_f64(wa[0], wa[1], rows, wa[2], n, k)) < 2e-2

    # (ii) hidden = k: down projection [k, inter] with residual + rstd emit, then the normed linear [n, k]
    inter = 512
    wd = U.make_weight(rng, k, inter)[:3]
    act = U.gauss_bf16(rng, (1, inter))
    resid = U.gauss_bf16(rng, (1, k), 1.5)
    d = [U.dev(wd[0]), U.dev(wd[1]), U.dev(act), U.dev(resid)]
    h = torch.full((k + 64,), 0x7FC0, dtype=torch.int16, device="cuda")
    pack = torch.zeros(3, dtype=torch.float32, device="cuda")
    for _ in range(2):   # the second launch finds the pack's sum and count back at zero
        assert U.ffi.call("nvk_b200_linear_nvfp4_w4a16_residual_rstd_emit", U.stream(), d[0].data_ptr(), d[1].data_ptr(),
                          d[2].data_ptr(), None, d[3].data_ptr(), h.data_ptr(), float(wd[2]), pack.data_ptr(), eps,
                          k, inter) == 0
    torch.cuda.synchronize()
    hb = U.host_u16(h)
    assert np.all(hb[k:] == 0x7FC0)
    hidden = hb[:k].reshape(1, k)
    pk = pack.cpu().numpy()
    hf = ref.bf16_to_f32(hidden).astype(np.float64)
    assert abs(float(pk[0]) - 1.0 / np.sqrt((hf ** 2).mean() + eps)) < 1e-5 * float(pk[0])
    assert pk[1] == 0.0 and pack.view(torch.int32).cpu().numpy()[2] == 0
    dn = [U.dev(wa[0]), U.dev(wa[1]), U.dev(hidden), U.dev(nw)]
    y = torch.zeros(n, dtype=torch.int16, device="cuda")
    assert U.ffi.call("nvk_b200_linear_nvfp4_w4a16_normed", U.stream(), dn[0].data_ptr(), dn[1].data_ptr(), None, None,
                      dn[2].data_ptr(), dn[3].data_ptr(), pack.data_ptr(), eps, y.data_ptr(), None, float(wa[2]), 0.0,
                      1, n, k) == 0
    torch.cuda.synchronize()
    two_step = run_linear(wa[0], wa[1], device_rmsnorm(hidden, nw, eps), wa[2], 1, n, k)
    assert U.rel_err_floor(ref.bf16_to_f32(U.host_u16(y)).reshape(1, n), ref.bf16_to_f32(two_step).astype(np.float64)) < 1e-2


@pytest.mark.parametrize("m", [1, 5])
def test_bf16_forward_rows_and_the_unconditional_m1_gemv(m):
    """rust/crates/nv-layers/src/linear.rs:883-913,1420-1442: a slice of the weight's rows gives exactly the
    corresponding columns of the full product; the M = 1 NVFP4 entry refuses more than one row."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(60 + m)
    n, k = 1000, 512
    w = U.gauss_bf16(rng, (n, k), 0.05)
    lin = sp.Bf16Linear(U.dev(w).view(torch.bfloat16))
    xt = U.dev(U.gauss_bf16(rng, (m, k))).view(torch.bfloat16)
    full = U.host_u16(lin(xt))
    part = U.host_u16(lin.forward_rows(xt, 128, 300))
    assert part.shape == (m, 300) and np.array_equal(part, full[:, 128:428])
    assert lin.forward_rows(xt, 990, 0).shape == (m, 0)
    with pytest.raises(ValueError, match="out of range"):
        lin.forward_rows(xt, 900, 101)
    packed, sw, alpha, _ = U.make_weight(rng, 256, k)
    q = sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(sw), alpha, k, 256)
    if m == 1:
        assert np.array_equal(U.host_u16(q.forward_nvfp4_gemv_m1(xt)), U.host_u16(q(xt)))
    else:
        with pytest.raises(ValueError, match="one row per step"):
            q.forward_nvfp4_gemv_m1(xt)


@pytest.mark.parametrize("m", [1, 4, 12])
def test_mlp_block_with_norm_and_residual(m):
    """Nvfp4Mlp.forward_block: h + MLP(RMSNorm(h)) in two launches for a few rows; the same bits as the norm
    kernel followed by forward_residual, and the many-row route agrees with the few-row one row by row."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(70 + m)
    hidden, inter, eps = 256, 384, 1e-6
    shapes = ((inter, hidden), (inter, hidden), (hidden, inter))
    lins = []
    for (n, k) in shapes:
        p_, s_, a_, _ = U.make_weight(rng, n, k)
        lins.append(sp.Nvfp4Linear.new_nvfp4(U.dev(p_), U.dev(s_), a_, k, n))
    mlp = sp.Nvfp4Mlp(*lins)
    h = U.gauss_bf16(rng, (m, hidden), 2.0)
    nw = U.gauss_bf16(rng, (hidden,), 1.0)
    ht, nwt = U.dev(h).view(torch.bfloat16), U.dev(nw).view(torch.bfloat16)
    got = U.host_u16(mlp.forward_block(ht, nwt, eps))
    normed = U.dev(device_rmsnorm(h, nw, eps)).view(torch.bfloat16)
    want = U.host_u16(mlp.forward_residual(normed, ht))
    assert np.array_equal(got, want)
    one = U.host_u16(mlp.forward_block(ht[:1].contiguous(), nwt, eps))
    assert np.array_equal(one[0], got[0])


def test_multi_phase_activation_staging():
    """K large enough at M=64 that the activations are staged in several phases, with magnitudes
    that change by 2^40 along K so the per-phase power-of-two rescale is exercised."""
    U.require_gpu()
    rng = np.random.default_rng(5)
    n, k, m = 128, 4096, 64
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    xf = rng.standard_normal((m, k)).astype(np.float32)
    xf[:, 1024:2048] *= np.float32(2.0 ** 20)
    xf[:, 3072:] *= np.float32(2.0 ** -20)
    x = ref.f32_to_bf16(xf)
    U.ffi.call("nvk_b200_set_tuning", 1, 0)
    try:
        got = run_linear(packed, sw, x, alpha, m, n, k)
    finally:
        U.ffi.call("nvk_b200_set_tuning", 0, 0)
    check_against_oracle(got, packed, sw, x, alpha, n, k, cpu_backend=False)


def test_wide_dynamic_range_and_special_values():
    U.require_gpu()
    rng = np.random.default_rng(9)
    n, k = 256, 1024
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    xf = rng.standard_normal((1, k)).astype(np.float32) * np.exp2(rng.integers(-30, 10, size=(1, k))).astype(np.float32)
    x = ref.f32_to_bf16(xf)
    got = run_gemv(packed, sw, x, alpha, n, k)
    check_against_oracle(got, packed, sw, x, alpha, n, k, cpu_backend=False)
    # all-zero activation -> exact zeros
    z = np.zeros((1, k), np.uint16)
    assert np.all(ref.bf16_to_f32(run_gemv(packed, sw, z, alpha, n, k)) == 0)
    # tiny activations (below f16 range before the power-of-two pre-scale)
    tiny = ref.f32_to_bf16((rng.standard_normal((1, k)) * 1e-30).astype(np.float32))
    got = ref.bf16_to_f32(run_gemv(packed, sw, tiny, alpha, n, k))
    want = ref.linear_w4a16_f64(packed, sw, tiny, alpha, n, k)
    assert np.max(np.abs(got - want)) <= 1e-2 * np.sqrt(np.mean(want ** 2)) + 1e-38


def test_every_scale_byte_and_code_decodes_like_the_oracle():
    """Random nibbles and random scale bytes over the whole 0..0x7F range, plus bytes with bit 7 set
    (the reference's decode formula ignores that bit).  0x7F -- which no NVFP4 encoder emits and which is
    NaN to the hardware's e4m3 convert -- decodes to 480 as the formula says (rust/crates/nv-quant/src/nvfp4.rs:76-85),
    on the tensor-core route and on the generic one."""
    U.require_gpu()
    rng = np.random.default_rng(11)
    n, k = 128, 512
    packed = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    lin = rng.integers(0, 0x80, size=(n, k // 16), dtype=np.uint8)
    lin[0, :10] = [0x80, 0xFE, 0x81, 0x00, 0x01, 0x07, 0x08, 0x7E, 0x7F, 0xFF]
    lin[5:9, :] = 0x7F
    assert (lin == 0x7F).sum() > 100
    sw = ref.swizzle_scales(lin)
    x = U.gauss_bf16(rng, (1, k))
    got = run_gemv(packed, sw, x, 2.0 ** -12, n, k)
    assert not np.any(np.isnan(ref.bf16_to_f32(got)))
    check_against_oracle(got, packed, sw, x, 2.0 ** -12, n, k, cpu_backend=False)
    # the generic route (K % 32 != 0) and several tokens decode the same way
    k2 = 48
    lin2 = np.full((n, k2 // 16), 0x7F, np.uint8)
    packed2 = rng.integers(0, 256, size=(n, k2 // 2), dtype=np.uint8)
    x2 = U.gauss_bf16(rng, (1, k2))
    got2 = run_gemv(packed2, ref.swizzle_scales(lin2), x2, 2.0 ** -12, n, k2)
    check_against_oracle(got2, packed2, ref.swizzle_scales(lin2), x2, 2.0 ** -12, n, k2, cpu_backend=False)
    x5 = U.gauss_bf16(rng, (5, k))
    got5 = run_linear(packed, sw, x5, 2.0 ** -12, 5, n, k)
    check_against_oracle(got5, packed, sw, x5, 2.0 ** -12, n, k, cpu_backend=False)


def test_dual_and_silu_prologue_m1():
    """gate+up in one launch, then the down projection with SiLU(gate)*up as its prologue; shapes of
    rust/crates/nv-kernels/tests/gemv_nvfp4_w4a16_decode_parity.rs (N=256, K=512) and a wider one."""
    U.require_gpu()
    for (inter, hidden) in [(256, 512), (1536, 1024)]:
        rng = np.random.default_rng(inter)
        pg, sg, ag, _ = U.make_weight(rng, inter, hidden)
        pu, su, au, _ = U.make_weight(rng, inter, hidden)
        pd, sd, ad, _ = U.make_weight(rng, hidden, inter)
        x = U.gauss_bf16(rng, (1, hidden), 4.0)
        d = [U.dev(a) for a in (pg, sg, pu, su, x)]
        yg = torch.zeros(inter, dtype=torch.int16, device="cuda")
        yu = torch.zeros(inter, dtype=torch.int16, device="cuda")
        assert U.ffi.call("nv_kernels_gemv_nvfp4_w4a16_dual_m1", U.stream(), d[0].data_ptr(), d[1].data_ptr(),
                          d[2].data_ptr(), d[3].data_ptr(), d[4].data_ptr(), yg.data_ptr(), yu.data_ptr(), ag, au,
                          inter, hidden) == 0
        torch.cuda.synchronize()
        g_bits, u_bits = U.host_u16(yg), U.host_u16(yu)
        check_against_oracle(g_bits, pg, sg, x, ag, inter, hidden)
        check_against_oracle(u_bits, pu, su, x, au, inter, hidden)
        dd = [U.dev(a) for a in (pd, sd)]
        yd = torch.zeros(hidden, dtype=torch.int16, device="cuda")
        assert U.ffi.call("nv_kernels_gemv_nvfp4_w4a16_silu_gate_up_in_m1", U.stream(), dd[0].data_ptr(),
                          dd[1].data_ptr(), yg.data_ptr(), yu.data_ptr(), yd.data_ptr(), ad, hidden, inter) == 0
        torch.cuda.synchronize()
        act = ref.f32_to_bf16(ref.silu_mul(g_bits, u_bits, round_bf16=True)).reshape(1, inter)
        want = ref.linear_w4a16_f64(pd, sd, act, ad, hidden, inter)
        e = U.rel_err_floor(ref.bf16_to_f32(U.host_u16(yd)).reshape(1, hidden), want)
        assert e < 2e-2  # reference bound for this pair (gemv_nvfp4_w4a16_decode_parity.rs: 2e-2)


@pytest.mark.parametrize("m", [2, 6, 16])
def test_mk_dual_reference_symbol(m):
    U.require_gpu()
    rng = np.random.default_rng(m)
    n, k = 512, 640
    pa, sa, aa, _ = U.make_weight(rng, n, k)
    pb, sb, ab, _ = U.make_weight(rng, n, k)
    x = U.gauss_bf16(rng, (m, k))
    d = [U.dev(a) for a in (pa, sa, pb, sb, x)]
    ya = torch.zeros(m * n, dtype=torch.int16, device="cuda")
    yb = torch.zeros(m * n, dtype=torch.int16, device="cuda")
    assert U.ffi.call("nv_kernels_gemm_nvfp4_w4a16_mk_dual", U.stream(), *[t.data_ptr() for t in d], ya.data_ptr(),
                      yb.data_ptr(), aa, ab, m, n, k) == 0
    torch.cuda.synchronize()
    check_against_oracle(U.host_u16(ya), pa, sa, x, aa, n, k)
    check_against_oracle(U.host_u16(yb), pb, sb, x, ab, n, k)
    # single arm through the same symbol
    yc = torch.zeros(m * n, dtype=torch.int16, device="cuda")
    assert U.ffi.call("nv_kernels_gemm_nvfp4_w4a16_mk_dual", U.stream(), d[0].data_ptr(), d[1].data_ptr(), None, None,
                      d[4].data_ptr(), yc.data_ptr(), None, aa, 0.0, m, n, k) == 0
    torch.cuda.synchronize()
    assert np.array_equal(U.host_u16(yc), U.host_u16(ya))


@pytest.mark.big
@pytest.mark.parametrize("m", [3, 8, 9, 16, 24, 33, 64])
@pytest.mark.parametrize("n,k", [(8192, 4096), (6200, 5408), (20480, 5120)])
def test_workspace_path_is_bit_identical(m, n, k):
    """With a caller workspace the activations are converted once by a separate kernel; the result
    must equal the in-kernel conversion bit for bit (same products, same order), for one and two arms
    and with the SiLU prologue."""
    U.require_gpu()
    rng = np.random.default_rng(m * 1000 + n + k)
    pa, sa, aa, _ = U.make_weight(rng, n, k)
    pb, sb, ab, _ = U.make_weight(rng, n, k)
    x = U.gauss_bf16(rng, (m, k))
    up = U.gauss_bf16(rng, (m, k))
    nbytes = U.ffi.lib().nvk_b200_linear_workspace_bytes(m, k)
    ws = torch.zeros(nbytes + 64, dtype=torch.uint8, device="cuda")
    ws[nbytes:] = 0xEE
    d = [U.dev(a) for a in (pa, sa, pb, sb, x, up)]
    for dual, silu in [(False, False), (True, False), (False, True)]:
        outs = []
        for use_ws in (False, True):
            ya = torch.zeros(m * n, dtype=torch.int16, device="cuda")
            yb = torch.zeros(m * n, dtype=torch.int16, device="cuda")
            rc = U.ffi.call("nvk_b200_linear_nvfp4_w4a16_ws", U.stream(), d[0].data_ptr(), d[1].data_ptr(),
                            d[2].data_ptr() if dual else None, d[3].data_ptr() if dual else None, d[4].data_ptr(),
                            d[5].data_ptr() if silu else None, ya.data_ptr(), yb.data_ptr() if dual else None, aa, ab,
                            m, n, k, ws.data_ptr() if use_ws else None, nbytes if use_ws else 0)
            assert rc == 0
            torch.cuda.synchronize()
            outs.append((U.host_u16(ya).copy(), U.host_u16(yb).copy()))
        assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
        assert np.all(ws[nbytes:].cpu().numpy() == 0xEE), "wrote past the workspace"
        if not silu and not dual and n <= 8192 and m in (3, 16):
            check_against_oracle(outs[1][0], pa, sa, x, aa, n, k, cpu_backend=False)
    assert U.ffi.call("nvk_b200_linear_nvfp4_w4a16_ws", U.stream(), d[0].data_ptr(), d[1].data_ptr(), None, None,
                      d[4].data_ptr(), None, ws.data_ptr(), None, aa, 0.0, m, n, k, ws.data_ptr(), 16) == -2


def test_refusals_match_the_reference():
    U.require_gpu()
    t = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p, s = t.data_ptr(), U.stream()
    f = U.ffi.call
    assert f("nv_kernels_nvfp4_gemv_bf16act", s, p, p, p, p, 1.0, 0, 256) == 0       # empty: no-op
    assert f("nv_kernels_nvfp4_gemv_bf16act", s, p, p, p, p, 1.0, 64, 250) == -1     # K % 16
    assert f("nv_kernels_gemv_nvfp4_w4a16_dual_m1", s, p, p, None, None, p, p, None, 1.0, 1.0, 64, 48) == -1  # K % 32
    assert f("nv_kernels_gemv_nvfp4_w4a16_dual_m1", s, p, p, p, None, p, p, None, 1.0, 1.0, 64, 64) == -1  # half-null arm
    assert f("nv_kernels_gemv_nvfp4_w4a16_silu_gate_up_in_m1", s, p, p, p, p, p, 1.0, 0, 64) == -1
    assert f("nv_kernels_gemm_nvfp4_w4a16_mk_dual", s, p, p, None, None, p, p, None, 1.0, 1.0, 17, 64, 64) == -1
    assert f("nv_kernels_gemm_nvfp4_w4a16_mk_dual", s, p, p, None, None, p, p, None, 1.0, 1.0, 0, 64, 64) == -1
    assert f("nvk_b200_linear_nvfp4_w4a16", s, p, p, None, None, p, None, p, None, 1.0, 0.0, 65, 128, 128) == -1
    torch.cuda.synchronize()


def test_row_chunk_invariance_is_bitwise():
    """rust/crates/nv-layers/tests/nvfp4_chunk_invariance.rs: a projection is bit-identical under
    row chunking, and does change when an input changes.  Rows are independent and the order in
    which K is summed depends on (N, K) only, so a row gives the same bits whatever else is in its
    batch, whatever the batch size (1..64), and wherever it sits."""
    U.require_gpu()
    rng = np.random.default_rng(77)
    n, k, m = (384, 1536, 64) if getattr(U.ffi, "EMULATED", False) else (1024, 5376, 64)   # the host emulation is given less to do
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    x = U.gauss_bf16(rng, (m, k))
    full = run_linear(packed, sw, x, alpha, m, n, k)
    for chunk in (1, 3, 8, 16, 24, 40):
        parts = [run_linear(packed, sw, x[r:r + chunk], alpha, min(chunk, m - r), n, k) for r in range(0, m, chunk)]
        assert np.array_equal(np.concatenate(parts, 0), full), f"chunk {chunk}"
    # the M=1 reference symbol is the same computation
    assert np.array_equal(run_gemv(packed, sw, x[5:6], alpha, n, k), full[5])
    x2 = x.copy()
    x2[5, 100] ^= 0x0100
    changed = run_linear(packed, sw, x2, alpha, m, n, k)
    assert not np.array_equal(changed[5], full[5])
    assert np.array_equal(np.delete(changed, 5, 0), np.delete(full, 5, 0))  # other rows untouched


def test_bf16_lm_head_gemv():
    U.require_gpu()
    rng = np.random.default_rng(3)
    for n, k in [(1000, 5120), (37, 200), (4096, 4104)]:
        w = U.gauss_bf16(rng, (n, k), 0.02)
        x = U.gauss_bf16(rng, (1, k))
        dw, dx = U.dev(w), U.dev(x)
        y = torch.zeros(n, dtype=torch.int16, device="cuda")
        assert U.ffi.call("nv_kernels_gemv_bf16", U.stream(), dw.data_ptr(), dx.data_ptr(), y.data_ptr(), n, k) == 0
        torch.cuda.synchronize()
        want = ref.bf16_to_f32(x).astype(np.float64) @ ref.bf16_to_f32(w).astype(np.float64).T
        assert U.rel_err_floor(ref.bf16_to_f32(U.host_u16(y)).reshape(1, n), want) < 1e-2
        cpu = ref.linear_cpu_backend(w, x)
        assert U.bf16_ulp_diff(U.host_u16(y), cpu[0]).max() <= 2


@pytest.mark.parametrize("m", [2, 3, 8, 9, 16, 17, 33, 64])
@pytest.mark.parametrize("n,k", [(1000, 1024), (37, 200), (20000, 264), (128, 2048), (19008, 512)])
def test_bf16_linear_for_a_few_rows(m, n, k):
    """nvk_b200_linear_bf16: one pass over W for all rows of x.  Oracle: the reference's Cpu-backend
    linear (bf16 -> f32 both sides, f32 matmul, bf16 out; rust/crates/nv-layers/src/linear.rs:1148-1161)
    with its test's bound (linear.rs:2612-2660: relative error below 1e-2), here in the floored form, and
    an f64 dot.  N = 20000 and 19008 take the warp-per-16-rows kernel, the others split K over a CTA."""
    U.require_gpu()
    rng = np.random.default_rng(m * 1000 + n + k)
    w = U.gauss_bf16(rng, (n, k), 0.02)
    x = U.gauss_bf16(rng, (m, k))
    dw, dx = U.dev(w), U.dev(x)
    y = torch.full((m * n + 64,), 0x7FC0, dtype=torch.int16, device="cuda")
    assert U.ffi.call("nvk_b200_linear_bf16", U.stream(), dw.data_ptr(), dx.data_ptr(), y.data_ptr(), m, n, k) == 0
    torch.cuda.synchronize()
    out = U.host_u16(y)
    assert np.all(out[m * n:] == 0x7FC0)
    got = ref.bf16_to_f32(out[:m * n]).reshape(m, n)
    want = ref.bf16_to_f32(x).astype(np.float64) @ ref.bf16_to_f32(w).astype(np.float64).T
    assert U.rel_err_floor(got, want) < 1e-2
    cpu = ref.linear_cpu_backend(w, x)
    assert U.rel_err_floor(got, ref.bf16_to_f32(cpu)) < 1e-2
    # element by element: within 2 bf16 ulp of the sequential f32 dot, or (near a cancellation) within
    # the f32 summation-order noise of a sum of this size
    ulp = U.bf16_ulp_diff(out[:m * n].reshape(m, n), cpu)
    absd = np.abs(got - ref.bf16_to_f32(cpu))
    rms = float(np.sqrt(np.mean(want ** 2)))
    assert np.all((ulp <= 2) | (absd <= 2e-3 * rms))
    assert U.ffi.call("nvk_b200_linear_bf16", U.stream(), dw.data_ptr(), dx.data_ptr(), y.data_ptr(), 65, n, k) == -1
    assert U.ffi.call("nvk_b200_linear_bf16", U.stream(), dw.data_ptr(), dx.data_ptr(), y.data_ptr(), 0, n, k) == -1


def test_bf16_linear_odd_shapes_take_the_row_loop():
    U.require_gpu()
    rng = np.random.default_rng(77)
    m, n, k = 3, 50, 100   # K % 8 != 0
    w, x = U.gauss_bf16(rng, (n, k), 0.02), U.gauss_bf16(rng, (m, k))
    y = torch.zeros(m * n, dtype=torch.int16, device="cuda")
    assert U.ffi.call("nvk_b200_linear_bf16", U.stream(), U.dev(w).data_ptr(), U.dev(x).data_ptr(), y.data_ptr(), m, n, k) == 0
    torch.cuda.synchronize()
    assert U.bf16_ulp_diff(U.host_u16(y).reshape(m, n), ref.linear_cpu_backend(w, x)).max() <= 2


@pytest.mark.big
@pytest.mark.parametrize("k,n", [(4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096)])
@pytest.mark.parametrize("m", [1, 4, 16, 64])
def test_configs1_full_size_sweep(k, n, m):
    """The decode GEMV shape sweep at full size: every (K, N) x M against the f64 oracle on a seeded subset of
    rows (all tokens; 512 output rows spread over the matrix, so every launch path is exercised while
    the CPU side stays at seconds), plus a size-independent property on the whole output: with the
    split of K pinned (it is otherwise chosen from the number of row tiles), rows computed as part of
    the full matrix equal rows computed from a 128-row-aligned slice of it, bit for bit."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    torch.manual_seed(k + n)
    w = (torch.randn((n, k), device="cuda") * 0.02).to(torch.bfloat16)
    lin = sp.Nvfp4Linear.from_bf16_quantized_nvfp4_dev(w)
    x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    y = lin(x)
    torch.cuda.synchronize()
    packed = lin.weight_u8.cpu().numpy().reshape(n, k // 2)
    sw = lin.weight_scales.cpu().numpy()
    xb = U.host_u16(x).reshape(m, k)
    got = U.host_u16(y).reshape(m, n)
    rng = np.random.default_rng(n)
    tiles = rng.choice(n // 128, size=4, replace=False)
    lin_scales = ref.unswizzle_scales(sw, n, k // 16)
    subs = []
    for t in tiles:
        r0 = int(t) * 128
        sub_p, sub_s = packed[r0:r0 + 128], ref.swizzle_scales(lin_scales[r0:r0 + 128])
        want = ref.linear_w4a16_f64(sub_p, sub_s, xb, lin.weight_alpha, 128, k)
        e = U.rel_err_floor(ref.bf16_to_f32(got[:, r0:r0 + 128]), want)
        assert e < TOL_F64, f"tile {t}: {e}"
        subs.append((r0, sp.Nvfp4Linear.new_nvfp4(U.dev(sub_p), U.dev(sub_s), lin.weight_alpha, k, 128)))
    assert U.ffi.call("nvk_b200_set_tuning", 1, 0) == 0   # every warp sums all of K for its rows, in order
    try:
        pinned = U.host_u16(lin(x)).reshape(m, n)
        for r0, small in subs:
            assert np.array_equal(U.host_u16(small(x)).reshape(m, 128), pinned[:, r0:r0 + 128]), f"rows {r0}.."
    finally:
        U.ffi.call("nvk_b200_set_tuning", 0, 0)
    # the default split changes only the order of the fp32 additions
    assert U.rel_err_floor(ref.bf16_to_f32(pinned), ref.bf16_to_f32(got).astype(np.float64)) < 1e-2


@pytest.mark.parametrize("m", [1, 4, 8])
@pytest.mark.parametrize("rows", [0, 16, 128])
def test_persistent_step_equals_the_standalone_launches(m, rows):
    """Two SwiGLU MLP layers (gate+up sharing x -> down with the SiLU(gate)*up prologue) as ONE persistent
    launch: every output equals, bit for bit, the chain of stand-alone launches with the same rows per
    CTA and no split of K; the wait flag stays clear; a second run and a replay from a CUDA graph give
    the same bits."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    from speaches_plus_b200 import linear as L
    rng = np.random.default_rng(900 + m)
    hidden, inter = 512, 1536

    def make(n, k):
        packed, sw, alpha, _ = U.make_weight(rng, n, k, 0.05)
        return sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(sw), alpha, k, n)

    layers = [(make(inter, hidden), make(inter, hidden), make(hidden, inter)) for _ in range(2)]
    x0 = U.dev(U.gauss_bf16(rng, (m, hidden))).view(torch.bfloat16)
    bf = dict(dtype=torch.bfloat16, device="cuda")

    def buffers():
        return [(torch.zeros((m, inter), **bf), torch.zeros((m, inter), **bf), torch.zeros((m, hidden), **bf))
                for _ in layers]

    # stand-alone launches; the persistent step picks 16-row items for these shapes unless told otherwise
    tune_rows = 16 if rows == 0 else rows
    want = buffers()
    assert U.ffi.call("nvk_b200_set_tuning", 1, tune_rows) == 0
    try:
        x = x0
        for (g, u, d), (yg, yu, yd) in zip(layers, want):
            L.linear_w4a16(g, u, x, None, yg, yu, m)
            L.linear_w4a16(d, None, yg, yu, yd, None, m)
            x = yd
        torch.cuda.synchronize()
    finally:
        U.ffi.call("nvk_b200_set_tuning", 0, 0)

    got = buffers()
    step = sp.DecodeStep(m, "cuda")
    x, dep = x0, -1
    for (g, u, d), (yg, yu, yd) in zip(layers, got):
        gu = step.add(g, x, yg, lin_b=u, y_b=yu, dep=dep, rows_per_item=rows)
        dep = step.add(d, yg, yd, x2=yu, dep=gu, rows_per_item=rows)
        x = yd
    step.build()

    def same():
        return all(torch.equal(a.view(torch.int16), b.view(torch.int16)) for w, g_ in zip(want, got) for a, b in zip(w, g_))

    for _ in range(2):
        for t in got:
            for b in t:
                b.zero_()
        step.run()
        torch.cuda.synchronize()
        step.check()
        assert same()
    # the run call checks its arguments against what the plan was built for
    n_ops, (grid, smem) = len(step._ops), step._launch
    bad = [(n_ops + 1, m, grid, smem), (n_ops, m + 1 if m < 8 else m - 1, grid, smem), (n_ops, m, grid + 1, smem),
           (n_ops, m, grid, smem + 16)]
    for a_ops, a_m, a_grid, a_smem in bad:
        assert U.ffi.call("nvk_b200_stack_run", U.stream(), step._plan.data_ptr(), a_ops, a_m, a_grid, a_smem,
                          step.err.data_ptr()) == -2
    if getattr(U.ffi, "EMULATED", False):
        return   # graph capture needs the real CUDA runtime
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        step.run()
        s.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            step.run()
        for t in got:
            for b in t:
                b.zero_()
        graph.replay()
        s.synchronize()
    step.check()
    assert same()
    del graph


def test_a_wait_on_a_peer_that_never_arrives_runs_out_and_reports():
    """The peer all-reduce's wait is bounded: with a peer whose flag nobody raises the kernel gives up
    after the configured number of polls, sets err = 1 + that peer, leaves y alone and returns; the
    context stays usable and the next call works.  One GPU, both "ranks'" buffers local; nothing
    faults, traps or hangs."""
    U.require_gpu()
    import ctypes as C
    n, max_elems, world = 256, 256, 2
    nbytes = U.ffi.lib().nvk_b200_tp_allreduce_buffer_bytes(world, max_elems)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    ptrs = (C.c_void_p * world)(*[b.data_ptr() for b in bufs])
    rng = np.random.default_rng(4)
    x = U.dev(U.gauss_bf16(rng, (n,)))
    y = torch.full((n,), 0x7FC0, dtype=torch.int16, device="cuda")
    epoch = torch.zeros(32, dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert U.ffi.call("nvk_b200_set_wait_limit", 1000) == 0
    try:
        assert U.ffi.call("nvk_b200_tp_allreduce_bf16", U.stream(), C.addressof(ptrs), 0, world, x.data_ptr(), y.data_ptr(), n,
                          max_elems, epoch.data_ptr(), err.data_ptr()) == 0
        torch.cuda.synchronize()                       # returns: the wait ran out
        assert int(err.cpu().numpy()[0]) == 2          # 1 + the peer that never arrived
        assert np.all(U.host_u16(y) == 0x7FC0)         # no sum was written
        assert int(epoch.cpu().numpy()[0]) == 1        # the call still counted: ranks stay in step
    finally:
        assert U.ffi.call("nvk_b200_set_wait_limit", 0) == 0
    # the next call (a world of one) works
    err.zero_()
    one = (C.c_void_p * 1)(bufs[0].data_ptr())
    assert U.ffi.call("nvk_b200_tp_allreduce_bf16", U.stream(), C.addressof(one), 0, 1, x.data_ptr(), y.data_ptr(), n, max_elems,
                      epoch.data_ptr(), err.data_ptr()) == 0
    torch.cuda.synchronize()
    assert int(err.cpu().numpy()[0]) == 0 and np.array_equal(U.host_u16(y), U.host_u16(x))


def test_fused_linear_allreduce_on_one_device():
    """nvk_b200_tp_linear_nvfp4_w4a16_allreduce on one GPU: (i) a world of one gives the plain linear's bits
    (with a residual: the residual-update form's semantics on bf16 partials); (ii) with a second rank that
    never arrives the bounded wait runs out, err names it, y stays untouched, the call returns, and the
    next call works.  Nothing faults, traps or hangs."""
    U.require_gpu()
    import ctypes as C
    rng = np.random.default_rng(88)
    m, n, k, max_ctas = 3, 384, 512, 64
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    x = U.gauss_bf16(rng, (m, k))
    d = [U.dev(packed), U.dev(sw), U.dev(x)]
    nbytes = U.ffi.lib().nvk_b200_tp_fused_buffer_bytes(2, max_ctas, 8)
    assert nbytes > 0 and U.ffi.lib().nvk_b200_tp_fused_buffer_bytes(9, max_ctas, 8) == 0
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    epoch = torch.zeros(max_ctas, dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = torch.full((m * n,), 0x7FC0, dtype=torch.int16, device="cuda")

    def call(world, ptrs, residual=None):
        return U.ffi.call("nvk_b200_tp_linear_nvfp4_w4a16_allreduce", U.stream(), C.addressof(ptrs), 0, world,
                          d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), None,
                          residual.data_ptr() if residual is not None else None, y.data_ptr(), float(alpha), m, n, k,
                          max_ctas, 8, epoch.data_ptr(), err.data_ptr())

    one = (C.c_void_p * 1)(bufs[0].data_ptr())
    assert call(1, one) == 0
    torch.cuda.synchronize()
    plain = run_linear(packed, sw, x, alpha, m, n, k)
    assert int(err.cpu().numpy()[0]) == 0 and np.array_equal(U.host_u16(y).reshape(m, n), plain)
    resid = U.gauss_bf16(rng, (m, n), 2.0)
    assert call(1, one, U.dev(resid)) == 0
    torch.cuda.synchronize()
    want = ref.f32_to_bf16(ref.bf16_to_f32(plain) + ref.bf16_to_f32(resid))
    assert np.array_equal(U.host_u16(y).reshape(m, n), want)
    # a peer that never arrives
    y.fill_(0x7FC0)
    two = (C.c_void_p * 2)(bufs[0].data_ptr(), bufs[1].data_ptr())
    assert U.ffi.call("nvk_b200_set_wait_limit", 1000) == 0
    try:
        assert call(2, two) == 0
        torch.cuda.synchronize()
        assert int(err.cpu().numpy()[0]) == 2 and np.all(U.host_u16(y) == 0x7FC0)
    finally:
        assert U.ffi.call("nvk_b200_set_wait_limit", 0) == 0
    err.zero_()
    assert call(1, one) == 0
    torch.cuda.synchronize()
    assert int(err.cpu().numpy()[0]) == 0 and np.array_equal(U.host_u16(y).reshape(m, n), plain)
    assert call(1, one) == 0 and U.ffi.call("nvk_b200_tp_linear_nvfp4_w4a16_allreduce", U.stream(), C.addressof(one), 0, 1,
                                            d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), None, None, y.data_ptr(),
                                            float(alpha), 9, n, k, max_ctas, 8, epoch.data_ptr(), err.data_ptr()) == -1
    torch.cuda.synchronize()


def test_two_ranks_of_the_peer_all_reduce_on_one_device_buffer_pair():
    """Both ranks' kernels of one exchange, run one after the other on ONE GPU with a short wait limit,
    is NOT how the kernel is meant to run (ranks are processes on different GPUs and wait for each other);
    what can be checked on one device is the data path: rank 1 first (its wait for rank 0 runs out, its
    push has landed), then rank 0 finds rank 1's slot and flag and produces the sum in rank order."""
    U.require_gpu()
    import ctypes as C
    n, max_elems, world = 512, 512, 2
    nbytes = U.ffi.lib().nvk_b200_tp_allreduce_buffer_bytes(world, max_elems)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    ptrs = (C.c_void_p * world)(*[b.data_ptr() for b in bufs])
    rng = np.random.default_rng(8)
    xs = [U.gauss_bf16(rng, (n,)) for _ in range(world)]
    dx = [U.dev(v) for v in xs]
    ys = [torch.zeros(n, dtype=torch.int16, device="cuda") for _ in range(world)]
    epochs = [torch.zeros(32, dtype=torch.int32, device="cuda") for _ in range(world)]
    errs = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(world)]
    assert U.ffi.call("nvk_b200_set_wait_limit", 1000) == 0
    try:
        for r in (1, 0):
            assert U.ffi.call("nvk_b200_tp_allreduce_bf16", U.stream(), C.addressof(ptrs), r, world, dx[r].data_ptr(),
                              ys[r].data_ptr(), n, max_elems, epochs[r].data_ptr(), errs[r].data_ptr()) == 0
            torch.cuda.synchronize()
    finally:
        U.ffi.call("nvk_b200_set_wait_limit", 0)
    assert int(errs[1].cpu().numpy()[0]) == 1 and int(errs[0].cpu().numpy()[0]) == 0
    want = ref.f32_to_bf16(ref.bf16_to_f32(xs[0]) + ref.bf16_to_f32(xs[1]))   # fp32 sum in rank order, one rounding
    assert np.array_equal(U.host_u16(ys[0]), want)


def test_lora_hook_runs_after_the_base_matmul_and_before_the_bias():
    """rust/crates/nv-layers/src/linear.rs:624-645: matmul, adapter hook (may replace the output), bias."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(2)
    n, k, m, r = 256, 512, 3, 8
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    bias = U.dev(U.gauss_bf16(rng, (n,))).view(torch.bfloat16)
    lin = sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(sw), alpha, k, n, bias)
    x = U.dev(U.gauss_bf16(rng, (m, k))).view(torch.bfloat16)
    base = lin(x).float().cpu()
    a = sp.Bf16Linear(U.dev(U.gauss_bf16(rng, (r, k), 0.05)).view(torch.bfloat16))     # down-projection [r, k]
    b = sp.Bf16Linear(U.dev(U.gauss_bf16(rng, (n, r), 0.05)).view(torch.bfloat16))     # up-projection [n, r]
    seen = []

    def hook(x2, y2, window):
        seen.append((tuple(x2.shape), tuple(y2.shape), window))
        return y2 + 2.0 * b(a(x2))

    assert lin.prenorm_nvfp4_eligible() is False            # it has a bias
    lin.set_lora_hook(hook)
    assert lin.has_lora()
    got = lin(x).float().cpu()
    torch.cuda.synchronize()
    assert seen == [((m, k), (m, n), None)]
    delta = (2.0 * b(a(x))).float().cpu()
    want = ((base - bias.float().cpu()).to(torch.bfloat16).float() + delta).to(torch.bfloat16).float() + bias.float().cpu()
    assert torch.allclose(got, want.to(torch.bfloat16).float(), atol=0.05, rtol=0.02)
    lin.set_lora_hook(lambda x2, y2, w: None)                # a hook may decline
    assert torch.equal(lin(x).float().cpu(), base)
    lin.set_lora_hook(None)
    assert not lin.has_lora()
    nb = sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(sw), alpha, k, n)
    assert nb.prenorm_nvfp4_eligible()
    nb.set_lora_hook(hook)
    assert not nb.prenorm_nvfp4_eligible()
