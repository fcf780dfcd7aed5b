"""The W4A8 decode MLP family (NVFP4 weights x int8 activation rows) against the CPU oracle, through
the C ABI.  Bounds and properties are the reference's own
(rust/crates/nv-kernels/tests/gemv_nvfp4_w4a8_decode_parity.rs):
  * |got - want| / max(|want|, 0.25) < 8e-3 against integer-exact dots in f64 ("two bf16 output ulps");
  * the quantizers are exact (integers and their scale);
  * M rows at once == one row at a time, bit for bit; the quantizing down projection == quantizer
    followed by the plain down projection, bit for bit.
"""
import numpy as np
import pytest
import torch

from oracle import ref
from tests import _util as U

pytestmark = pytest.mark.gpu
TOL = 8e-3


def rel_quarter(got_bits, want):
    got = ref.bf16_to_f32(got_bits).astype(np.float64).reshape(np.shape(want))
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), 0.25)))


def i8dev(q):
    return torch.from_numpy(np.ascontiguousarray(q)).cuda()


def w4a8(entry, wts, q, scales, m, n, k, residual=None, second=None, pack=None, eps=0.0):
    (packed, sw, alpha) = wts
    d = [U.dev(packed), U.dev(sw), i8dev(q), U.dev(np.asarray(scales, np.float32))]
    y = torch.full((m * n + 64,), 0x7FC0, dtype=torch.int16, device="cuda")
    args = [U.stream(), d[0].data_ptr(), d[1].data_ptr()]
    yb = db = None
    if second is not None:
        db = [U.dev(second[0]), U.dev(second[1])]
        yb = torch.full((m * n + 64,), 0x7FC0, dtype=torch.int16, device="cuda")
        args += [db[0].data_ptr(), db[1].data_ptr()]
    args += [d[2].data_ptr(), d[3].data_ptr()]
    dr = U.dev(residual) if residual is not None else None
    if second is not None:
        args += [y.data_ptr(), yb.data_ptr(), float(alpha), float(second[2])]
    else:
        args += [dr.data_ptr() if dr is not None else None, y.data_ptr(), float(alpha)]
    if pack is not None:
        args += [pack.data_ptr(), float(eps)]
    if entry.endswith("_mk"):
        args.append(m)
    args += [n, k]
    assert U.ffi.call(entry, *args) == 0
    torch.cuda.synchronize()
    out = U.host_u16(y)
    assert np.all(out[m * n:] == 0x7FC0)
    if yb is not None:
        outb = U.host_u16(yb)
        assert np.all(outb[m * n:] == 0x7FC0)
        return out[:m * n].reshape(m, n), outb[:m * n].reshape(m, n)
    return out[:m * n].reshape(m, n)


@pytest.mark.parametrize("n,k", [(256, 512), (384, 2304), (130, 1056)])
def test_dual_m1_and_down_residual_m1_match_the_int8_mechanics_oracle(n, k):
    U.require_gpu()
    rng = np.random.default_rng(n + k)
    wa, wb = U.make_weight(rng, n, k)[:3], U.make_weight(rng, n, k)[:3]
    x = (rng.standard_normal((1, k)) * 1.5).astype(np.float32)
    q, sc = ref.rowquant_i8(x)
    ya, yb = w4a8("nv_kernels_gemv_nvfp4_w4a8_dual_m1", wa, q, sc, 1, n, k, second=wb)
    assert rel_quarter(ya, ref.linear_w4a8_f64(wa[0], wa[1], q, sc, wa[2], n, k)) < TOL
    assert rel_quarter(yb, ref.linear_w4a8_f64(wb[0], wb[1], q, sc, wb[2], n, k)) < TOL
    resid = U.gauss_bf16(rng, (1, n))
    yd = w4a8("nv_kernels_gemv_nvfp4_w4a8_down_residual_m1", wa, q, sc, 1, n, k, residual=resid)
    assert rel_quarter(yd, ref.linear_w4a8_f64(wa[0], wa[1], q, sc, wa[2], n, k, resid)) < TOL
    y0 = w4a8("nv_kernels_gemv_nvfp4_w4a8_down_residual_m1", wa, q, sc, 1, n, k)   # residual may be NULL
    assert np.array_equal(y0, ya)


@pytest.mark.parametrize("m", [2, 7, 8, 9, 20, 64, 70])
def test_mk_equals_per_row_m1_calls_bitwise(m):
    U.require_gpu()
    rng = np.random.default_rng(m)
    n, k = 256, 768
    wa, wb = U.make_weight(rng, n, k)[:3], U.make_weight(rng, n, k)[:3]
    x = (rng.standard_normal((m, k)) * np.linspace(0.2, 3.0, m)[:, None]).astype(np.float32)
    q, sc = ref.rowquant_i8(x)
    ya, yb = w4a8("nv_kernels_gemv_nvfp4_w4a8_dual_mk", wa, q, sc, m, n, k, second=wb)
    resid = U.gauss_bf16(rng, (m, n))
    yd = w4a8("nv_kernels_gemv_nvfp4_w4a8_down_residual_mk", wa, q, sc, m, n, k, residual=resid)
    assert rel_quarter(yd, ref.linear_w4a8_f64(wa[0], wa[1], q, sc, wa[2], n, k, resid)) < TOL
    for r in sorted({0, m // 2, m - 1}):
        a1, b1 = w4a8("nv_kernels_gemv_nvfp4_w4a8_dual_m1", wa, q[r:r + 1], sc[r:r + 1], 1, n, k, second=wb)
        assert np.array_equal(a1[0], ya[r]) and np.array_equal(b1[0], yb[r])
        d1 = w4a8("nv_kernels_gemv_nvfp4_w4a8_down_residual_m1", wa, q[r:r + 1], sc[r:r + 1], 1, n, k,
                  residual=resid[r:r + 1])
        assert np.array_equal(d1[0], yd[r])


def silu_act(gate, up):
    return ref.bf16_to_f32(ref.f32_to_bf16(ref.silu_mul(gate, up, round_bf16=True)))


@pytest.mark.parametrize("k", [256, 3072, 25600])
def test_silu_rowquant_m1_mk_and_the_quantizing_down_projection(k):
    U.require_gpu()
    rng = np.random.default_rng(k)
    m, n = 3, 256
    gate, up = U.gauss_bf16(rng, (m, k), 2.0), U.gauss_bf16(rng, (m, k))
    act = silu_act(gate, up)
    q_want, s_want = ref.rowquant_i8(act)
    dg, du = U.dev(gate), U.dev(up)
    # one row, one CTA
    q1 = torch.zeros(k, dtype=torch.int8, device="cuda")
    s1 = torch.zeros(1, dtype=torch.float32, device="cuda")
    assert U.ffi.call("nv_kernels_silu_mul_rowquant_i8_m1", U.stream(), dg.data_ptr(), du.data_ptr(), q1.data_ptr(),
                      s1.data_ptr(), k) == 0
    # M rows, two passes
    plen = U.ffi.call("nv_kernels_silu_mul_rowquant_i8_mk_partials_len", m, k)
    assert plen == m * min(-(-k // 256), 128)
    staged = torch.zeros((m, k), dtype=torch.int16, device="cuda")
    part = torch.full((plen + 8,), -1.0, dtype=torch.float32, device="cuda")
    qm = torch.zeros((m, k), dtype=torch.int8, device="cuda")
    sm = torch.zeros(m, dtype=torch.float32, device="cuda")
    assert U.ffi.call("nv_kernels_silu_mul_rowquant_i8_mk", U.stream(), dg.data_ptr(), du.data_ptr(), staged.data_ptr(),
                      part.data_ptr(), qm.data_ptr(), sm.data_ptr(), m, k) == 0
    torch.cuda.synchronize()
    assert np.all(part.cpu().numpy()[plen:] == -1.0)
    # device expf may differ from the host's by an ulp: the staged activation may differ in rare last bits
    agree = (U.host_u16(staged) == ref.f32_to_bf16(act)).mean()
    assert agree > 0.999
    act_dev = ref.bf16_to_f32(U.host_u16(staged))
    q_dev, s_dev = ref.rowquant_i8(act_dev)          # the quantizer itself is exact on what was staged
    assert np.array_equal(qm.cpu().numpy(), q_dev) and np.array_equal(sm.cpu().numpy(), s_dev)
    assert np.array_equal(q1.cpu().numpy(), q_dev[0]) and s1.cpu().numpy()[0] == s_dev[0]
    if agree == 1.0:
        assert np.array_equal(q_dev, q_want) and np.array_equal(s_dev, s_want)
    # down projection that quantizes while it stages == quantizer, then plain down projection (bitwise)
    wd = U.make_weight(rng, n, k)[:3]
    resid = U.gauss_bf16(rng, (1, n))
    want = w4a8("nv_kernels_gemv_nvfp4_w4a8_down_residual_m1", wd, q_dev[0:1], s_dev[0:1], 1, n, k, residual=resid)
    st1 = torch.zeros(k, dtype=torch.int16, device="cuda")
    p1n = min(-(-k // 256), 128)
    p1 = torch.zeros(p1n, dtype=torch.float32, device="cuda")
    assert U.ffi.call("nv_kernels_silu_mul_stage_partial_absmax_m1", U.stream(), dg.data_ptr(), du.data_ptr(), st1.data_ptr(),
                      p1.data_ptr(), k) == 0
    y = torch.full((n + 64,), 0x7FC0, dtype=torch.int16, device="cuda")
    dw, ds, dr = U.dev(wd[0]), U.dev(wd[1]), U.dev(resid)
    assert U.ffi.call("nv_kernels_gemv_nvfp4_w4a8_down_residual_quant_prologue_m1", U.stream(), dw.data_ptr(), ds.data_ptr(),
                      st1.data_ptr(), p1.data_ptr(), p1n, dr.data_ptr(), y.data_ptr(), float(wd[2]), n, k) == 0
    torch.cuda.synchronize()
    out = U.host_u16(y)
    assert np.all(out[n:] == 0x7FC0) and np.array_equal(out[:n], want[0])


def test_down_residual_rstd_emit():
    U.require_gpu()
    rng = np.random.default_rng(9)
    n, k, eps = 640, 1024, 1e-6
    wd = U.make_weight(rng, n, k)[:3]
    q, sc = ref.rowquant_i8((rng.standard_normal((1, k)) * 2).astype(np.float32))
    resid = U.gauss_bf16(rng, (1, n))
    plain = w4a8("nv_kernels_gemv_nvfp4_w4a8_down_residual_m1", wd, q, sc, 1, n, k, residual=resid)
    pack = torch.zeros(3, dtype=torch.float32, device="cuda")
    for _ in range(2):   # the pack resets itself: a second launch gives the same answer
        got = w4a8("nv_kernels_gemv_nvfp4_w4a8_down_residual_m1_rstd_emit", wd, q, sc, 1, n, k, residual=resid,
                   pack=pack, eps=eps)
        assert np.array_equal(got, plain)
        pk = pack.cpu().numpy()
        y = ref.bf16_to_f32(got[0]).astype(np.float64)
        want = 1.0 / np.sqrt(np.mean(y ** 2) + eps)
        assert abs(pk[0] - want) / want < 1e-5
        assert pk[1] == 0.0 and pk.view(np.uint32)[2] == 0


@pytest.mark.parametrize("hidden", [256, 5120, 24576])
def test_rmsnorm_residual_writeout(hidden):
    U.require_gpu()
    rng = np.random.default_rng(hidden)
    batch, eps = 3, 1e-6
    x, res, w = U.gauss_bf16(rng, (batch, hidden)), U.gauss_bf16(rng, (batch, hidden)), U.gauss_bf16(rng, (hidden,), 0.5)
    want_res, want_v = ref.rmsnorm_residual(x, res, w, eps)
    dx, dr, dw = U.dev(x), U.dev(res), U.dev(w)
    ro = torch.zeros((batch, hidden), dtype=torch.int16, device="cuda")
    out = torch.zeros((batch, hidden), dtype=torch.int16, device="cuda")
    assert U.ffi.call("nv_kernels_rmsnorm_residual_writeout_bf16", U.stream(), dx.data_ptr(), dr.data_ptr(), dw.data_ptr(),
                      ro.data_ptr(), out.data_ptr(), batch, hidden, eps) == 0
    torch.cuda.synchronize()
    assert np.array_equal(U.host_u16(ro), want_res)
    assert U.bf16_ulp_diff(U.host_u16(out), want_v).max() <= 1    # rsqrt and the sum's order: one ulp
    # the int8 form (one row): the same v, then the exact quantizer
    ro1 = torch.zeros(hidden, dtype=torch.int16, device="cuda")
    q = torch.zeros(hidden, dtype=torch.int8, device="cuda")
    s = torch.zeros(1, dtype=torch.float32, device="cuda")
    assert U.ffi.call("nv_kernels_rmsnorm_residual_writeout_rowquant_i8_m1", U.stream(), dx.data_ptr(), dr.data_ptr(),
                      dw.data_ptr(), ro1.data_ptr(), q.data_ptr(), s.data_ptr(), hidden, eps) == 0
    torch.cuda.synchronize()
    assert np.array_equal(U.host_u16(ro1), want_res[0])
    q_want, s_want = ref.rowquant_i8(ref.bf16_to_f32(U.host_u16(out)[0:1]))   # two-kernel chain == fused kernel
    assert np.array_equal(q.cpu().numpy(), q_want[0]) and s.cpu().numpy()[0] == s_want[0]
    assert U.ffi.call("nv_kernels_rmsnorm_residual_writeout_rowquant_i8_m1", U.stream(), dx.data_ptr(), dr.data_ptr(),
                      dw.data_ptr(), ro1.data_ptr(), q.data_ptr(), s.data_ptr(), 24577, eps) == -1


def test_w4a8_refusals():
    """Ragged K, missing operands and misalignment are refused without a launch
    (gemv_nvfp4_w4a8_decode_parity.rs:951-1000)."""
    U.require_gpu()
    t = torch.zeros(4096, dtype=torch.int16, device="cuda")
    p, s = t.data_ptr(), U.stream()
    f = U.ffi.call
    assert f("nv_kernels_gemv_nvfp4_w4a8_dual_m1", s, p, p, p, p, p, p, p, p, 1.0, 1.0, 128, 48) == -1
    assert f("nv_kernels_gemv_nvfp4_w4a8_dual_m1", s, p, p, p, p, p, p, p, p, 1.0, 1.0, 0, 64) == -1
    assert f("nv_kernels_gemv_nvfp4_w4a8_dual_m1", s, p, p, None, p, p, p, p, p, 1.0, 1.0, 128, 64) == -2
    assert f("nv_kernels_gemv_nvfp4_w4a8_down_residual_m1", s, p + 4, p, p, p, None, p, 1.0, 128, 64) == -2
    assert f("nv_kernels_gemv_nvfp4_w4a8_down_residual_mk", s, p, p, p, p, None, p, 1.0, 0, 128, 64) == -1
    assert f("nv_kernels_gemv_nvfp4_w4a8_down_residual_quant_prologue_m1", s, p, p, p, p, 0, None, p, 1.0, 128, 64) == -1
    assert f("nv_kernels_silu_mul_rowquant_i8_m1", s, p, p, p, p, 6) == -1
    assert f("nv_kernels_silu_mul_rowquant_i8_m1", s, p, p, p, p, 49156) == -1    # > 96 KiB of staging
    assert f("nv_kernels_silu_mul_rowquant_i8_mk", s, p, p, p, p, p, p, 2, 24) == -1
    assert f("nv_kernels_silu_mul_rowquant_i8_mk_partials_len", 0, 64) == -1
