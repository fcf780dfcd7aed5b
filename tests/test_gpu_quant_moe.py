"""GPU parity of the quantizers (byte-exact) and the MoE decode plumbing against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import ref
from tests import _util as U

pytestmark = pytest.mark.gpu


def gpu_quantize(x_bits, g, m_padded=None):
    m, k = x_bits.shape
    mp = m if m_padded is None else m_padded
    dx = U.dev(x_bits)
    packed = torch.full((mp * k // 2 + 32,), 0xAB, dtype=torch.uint8, device="cuda")
    nsw = ref.swizzled_len(mp, k // 16)
    scales = torch.zeros(nsw + 32, dtype=torch.uint8, device="cuda")
    scales[nsw:] = 0xCD
    rc = U.ffi.call("nv_kernels_quantize_nvfp4_bf16", U.stream(), dx.data_ptr(), packed.data_ptr(),
                    scales.data_ptr(), float(g), mp, m, k)
    assert rc == 0
    torch.cuda.synchronize()
    p, s = packed.cpu().numpy(), scales.cpu().numpy()
    assert np.all(p[mp * k // 2:] == 0xAB) and np.all(s[nsw:] == 0xCD)
    return p[:mp * k // 2].reshape(mp, k // 2), s[:nsw]


@pytest.mark.parametrize("m,k,g", [(128, 128, 1.0), (130, 272, 1.0), (7, 48, 3.5), (256, 1024, 0.0073),
                                   (64, 4096, 448.0), (33, 64, 0.0), (512, 5376, 134.4)])
def test_quantizer_is_byte_exact(m, k, g):
    """rust/crates/nv-kernels/tests/quantize_nvfp4_bf16.rs: device bytes == host quantizer + swizzle
    (sin-wave inputs times 2.5), extended with gaussian magnitudes from 1e-4 to 500."""
    U.require_gpu()
    j = np.arange(m * k, dtype=np.float32)
    x1 = ref.f32_to_bf16(np.sin(j * np.float32(0.37)).astype(np.float32) * np.float32(2.5)).reshape(m, k)
    rng = np.random.default_rng(m * k)
    mags = np.exp(rng.uniform(np.log(1e-4), np.log(500.0), size=(m, 1))).astype(np.float32)
    x2 = ref.f32_to_bf16((rng.standard_normal((m, k)).astype(np.float32) * mags))
    x2[0, :16] = 0  # an all-zero block
    for x in (x1, x2):
        p, s = gpu_quantize(x, g)
        pw, lw = ref.quantize_rows_bf16(x, g)
        assert np.array_equal(p, pw)
        assert np.array_equal(s, ref.swizzle_scales(lw))


def test_quantizer_ties_and_pad_rows():
    U.require_gpu()
    k = 64
    x = np.zeros((3, k), np.float32)
    x[0, :8] = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0]
    x[1, :8] = [-0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0]
    x[2, 16:24] = [6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
    xb = ref.f32_to_bf16(x)
    p, s = gpu_quantize(xb, 1.0, m_padded=128)
    pw, lw = ref.quantize_rows_bf16(xb, 1.0, m_padded=128)
    assert np.array_equal(p, pw) and np.array_equal(s, ref.swizzle_scales(lw))
    assert np.all(p[3:] == 0)  # pad rows quantize zeros
    assert U.ffi.call("nv_kernels_quantize_nvfp4_bf16", U.stream(), 0, 0, 0, 1.0, 4, 5, 64) == -2
    assert U.ffi.call("nv_kernels_quantize_nvfp4_bf16", U.stream(), 0, 0, 0, 1.0, 4, 4, 40) == -1
    assert U.ffi.call("nv_kernels_quantize_nvfp4_bf16", U.stream(), 0, 0, 0, 1.0, 0, 0, 64) == 0


def test_device_scale_byte_at_power_of_two_neighbours():
    """rust/crates/nv-kernels/tests/ue4m3_log2f_boundary.rs: a block whose maximum is 6 makes the block
    scale equal the global, so the device encoder can be probed with chosen scales -- every power of two
    from 2^-9 to 2^8 and its f32 neighbours, where an encoder that takes log2 in floating point picks the
    wrong exponent.  The byte must equal the host encoder's (itself pinned to the exact-floor form)."""
    U.require_gpu()
    f32 = np.float32
    x = np.zeros((1, 16), np.uint16)
    x[0, 0] = ref.f32_to_bf16(np.array([6.0], f32))[0]
    probes = []
    for e in range(-9, 9):
        p = f32(2.0) ** f32(e)
        probes += [np.nextafter(p, f32(0)), p, np.nextafter(p, f32(1e9))]
    probes += [f32(448.0), np.nextafter(f32(448.0), f32(0)), f32(1e9), f32(447.9), f32(1.0 / 1024.0)]
    for stored in probes:
        _, s = gpu_quantize(x, float(stored))
        want = int(ref.encode_ue4m3(float(stored)))
        assert int(s[0]) == want, f"scale {float(stored)!r}: device {int(s[0]):#x}, host {want:#x}"
        assert int(s[0]) != 0x7F


def test_weight_quantizer_matches_oracle_and_feeds_the_gemv():
    """Linear::from_bf16_quantized_nvfp4_dev rule end to end on the GPU: global 448*6/amax,
    alpha = 1/global; bytes equal the oracle's, so the GEMV sees identical operands."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(0)
    w = U.gauss_bf16(rng, (384, 1024), 0.02)
    wt = U.dev(w).view(torch.bfloat16)
    lin = sp.Nvfp4Linear.from_bf16_quantized_nvfp4_dev(wt)
    packed, sw, alpha = ref.quantize_weight_bf16(w)
    assert np.array_equal(lin.weight_u8.cpu().numpy(), packed)
    assert np.array_equal(lin.weight_scales.cpu().numpy(), sw)
    assert lin.weight_alpha == alpha
    x = U.gauss_bf16(rng, (5, 1024))
    y = lin(U.dev(x).view(torch.bfloat16))
    want = ref.linear_w4a16_f64(packed, sw, x, alpha, 384, 1024)
    assert U.rel_err_floor(y.float().cpu().numpy(), want) < 1e-2


def test_row_quantizer_linear_scales():
    U.require_gpu()
    rng = np.random.default_rng(4)
    k = 1024
    x = U.gauss_bf16(rng, (1, k), 3.0)
    dx = U.dev(x)
    packed = torch.zeros(k // 2, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(k // 16, dtype=torch.uint8, device="cuda")
    assert U.ffi.call("nv_kernels_nvfp4_quantize_row_bf16", U.stream(), dx.data_ptr(), packed.data_ptr(),
                      scales.data_ptr(), 2.0, k) == 0
    torch.cuda.synchronize()
    pw, lw = ref.quantize_rows_bf16(x, 2.0)
    assert np.array_equal(packed.cpu().numpy(), pw[0]) and np.array_equal(scales.cpu().numpy(), lw[0])


@pytest.mark.parametrize("strided", [False, True])
def test_per_expert_quantizers(strided):
    U.require_gpu()
    rng = np.random.default_rng(8)
    mpe, tiles, k = 128, 5, 768
    m = mpe * tiles
    x = U.gauss_bf16(rng, (m, k), 2.0)
    up = U.gauss_bf16(rng, (m, k), 1.0)
    globals_ = np.array([1.0, 0.5, 37.0, 0.0, 448.0], np.float32)
    name = "nv_kernels_quantize_nvfp4_bf16_per_expert" + ("_strided" if strided else "")
    dx, du, dg = U.dev(x), U.dev(up), U.dev(globals_)
    nsw = ref.swizzled_len(m, k // 16)
    packed = torch.zeros((m, k // 2), dtype=torch.uint8, device="cuda")
    scales = torch.zeros(nsw, dtype=torch.uint8, device="cuda")
    assert U.ffi.call(name, U.stream(), dx.data_ptr(), packed.data_ptr(), scales.data_ptr(), dg.data_ptr(), mpe, m,
                      k) == 0
    torch.cuda.synchronize()
    p, s = packed.cpu().numpy(), ref.unswizzle_scales(scales.cpu().numpy(), m, k // 16)
    rows = range(0, m, mpe) if strided else range(m)
    for r in rows:
        pw, lw = ref.quantize_rows_bf16(x[r:r + 1], float(globals_[r // mpe]))
        assert np.array_equal(p[r], pw[0]) and np.array_equal(s[r], lw[0]), r
    if strided:
        assert np.all(p[1:mpe] == 0)  # untouched rows
        assert U.ffi.call(name, U.stream(), dx.data_ptr(), packed.data_ptr(), scales.data_ptr(), dg.data_ptr(), mpe,
                          m - 1, k) == -3

    # fused SiLU(gate)*up -> quantize: device expf may differ from libm by an ulp, so allow a
    # handful of off-by-one codes and no larger difference (the reference's own test allows 2%).
    name2 = "nv_kernels_silu_mul_quantize_nvfp4_bf16_per_expert" + ("_strided" if strided else "")
    packed.zero_(); scales.zero_()
    assert U.ffi.call(name2, U.stream(), dx.data_ptr(), du.data_ptr(), packed.data_ptr(), scales.data_ptr(),
                      dg.data_ptr(), mpe, m, k) == 0
    torch.cuda.synchronize()
    p, s = packed.cpu().numpy(), ref.unswizzle_scales(scales.cpu().numpy(), m, k // 16)
    act = ref.silu_mul(x, up, round_bf16=False)
    off_by_one = worse = total = 0
    for r in rows:
        g = float(globals_[r // mpe])
        pw, lw = ref.quantize_rows(act[r:r + 1], g)
        same_scale = s[r] == lw[0]
        assert same_scale.mean() > 0.995
        for shift in (0, 4):
            a = ((p[r] >> shift) & 0xF).astype(np.int32).reshape(-1, 8)[same_scale].ravel()
            b = ((pw[0] >> shift) & 0xF).astype(np.int32).reshape(-1, 8)[same_scale].ravel()
            d = np.abs((a & 7) - (b & 7))
            sign_ok = ((a >> 3) == (b >> 3)) | (((a & 7) == 0) & ((b & 7) == 0))
            off_by_one += int(np.sum((d == 1) & sign_ok))
            worse += int(np.sum((d > 1) | ~sign_ok))
            total += a.size
    assert worse == 0 and off_by_one <= total // 1000


def test_rmsnorm_quantize():
    U.require_gpu()
    rng = np.random.default_rng(12)
    m, k, eps, g = 5, 2048, 1e-6, 3.0
    x = U.gauss_bf16(rng, (m, k), 1.5)
    w = U.gauss_bf16(rng, (k,), 1.0)
    dx, dw = U.dev(x), U.dev(w)
    mp = 128
    nsw = ref.swizzled_len(mp, k // 16)
    packed = torch.zeros((mp, k // 2), dtype=torch.uint8, device="cuda")
    scales = torch.zeros(nsw, dtype=torch.uint8, device="cuda")
    assert U.ffi.call("nv_kernels_rmsnorm_quantize_nvfp4_bf16", U.stream(), dx.data_ptr(), dw.data_ptr(),
                      packed.data_ptr(), scales.data_ptr(), g, eps, mp, m, k) == 0
    torch.cuda.synchronize()
    xf, wf = ref.bf16_to_f32(x), ref.bf16_to_f32(w)
    rstd = (1.0 / np.sqrt((xf.astype(np.float64) ** 2).mean(1) + eps)).astype(np.float32)
    normed = ref.f32_to_bf16((xf * rstd[:, None]) * wf[None, :])
    pw, lw = ref.quantize_rows_bf16(normed, g, m_padded=mp)
    p, s = packed.cpu().numpy(), ref.unswizzle_scales(scales.cpu().numpy(), mp, k // 16)
    # rsqrtf and the sum order differ from numpy by an ulp: require near-total byte agreement
    assert (p == pw).mean() > 0.999 and (s == lw).mean() > 0.999
    assert np.all(p[m:] == 0)
    assert U.ffi.call("nv_kernels_rmsnorm_quantize_nvfp4_bf16", U.stream(), dx.data_ptr(), dw.data_ptr(),
                      packed.data_ptr(), scales.data_ptr(), g, eps, 1, 1, 32768) == -3


@pytest.mark.parametrize("E,K,mode", [(128, 8, 0), (256, 8, 0), (16, 4, 0), (512, 6, 0), (128, 8, 1)])
def test_router(E, K, mode):
    U.require_gpu()
    rng = np.random.default_rng(E + K)
    n = 33
    lg = rng.standard_normal((n, E)).astype(np.float32)
    lg[0, 5] = lg[0, 77 % E] = 9.0  # a tie at the top
    bias = (rng.standard_normal(E) * 0.1).astype(np.float32) if mode == 1 else None
    dl = U.dev(lg)
    db = U.dev(bias) if bias is not None else None
    ids = torch.zeros((n, K), dtype=torch.int32, device="cuda")
    w = torch.zeros((n, K), dtype=torch.float32, device="cuda")
    assert U.ffi.call("nv_kernels_moe_route_topk", U.stream(), dl.data_ptr(), db.data_ptr() if db is not None else None,
                      ids.data_ptr(), w.data_ptr(), n, E, K, mode, 0.0, 1, 2.5 if mode == 1 else 1.0) == 0
    torch.cuda.synchronize()
    wi, ww = ref.moe_route_topk(lg, K, bias=bias, mode=mode, norm_topk=True, routed_scaling=2.5 if mode == 1 else 1.0)
    assert np.array_equal(ids.cpu().numpy(), wi)
    np.testing.assert_allclose(w.cpu().numpy(), ww, rtol=2e-6, atol=1e-7)
    if mode == 0:
        np.testing.assert_allclose(w.cpu().numpy().sum(1), 1.0, rtol=1e-5)
    assert U.ffi.call("nv_kernels_moe_route_topk", U.stream(), 0, 0, 0, 0, 1, 8, 9, 0, 0.0, 1, 1.0) == -2


def test_router_shared_tail():
    U.require_gpu()
    rng = np.random.default_rng(2)
    n, E, K = 4, 64, 4
    lg = rng.standard_normal((n, E)).astype(np.float32)
    dl = U.dev(lg)
    ids = torch.zeros((n, K + 1), dtype=torch.int32, device="cuda")
    w = torch.zeros((n, K + 1), dtype=torch.float32, device="cuda")
    assert U.ffi.call("nv_kernels_moe_route_topk_shared_tail", U.stream(), dl.data_ptr(), None, ids.data_ptr(),
                      w.data_ptr(), n, E, K, 0, 0.0, 1, 1.0, E) == 0
    torch.cuda.synchronize()
    wi, ww = ref.moe_route_topk(lg, K)
    assert np.array_equal(ids.cpu().numpy()[:, :K], wi) and np.all(ids.cpu().numpy()[:, K] == E)
    assert np.all(w.cpu().numpy()[:, K] == 1.0)


def test_gather_unpermute_permute():
    U.require_gpu()
    rng = np.random.default_rng(6)
    n_tok, H, k, E = 6, 200, 3, 10
    x = U.gauss_bf16(rng, (n_tok, H))
    src = np.array([2, -1, 5, 0, 9, 3, 3], np.int32)  # -1 and 9 are out of range -> zero rows
    dx, ds = U.dev(x), U.dev(src)
    out = torch.full((len(src), H), 0x1111, dtype=torch.int16, device="cuda")
    assert U.ffi.call("nv_kernels_gather_rows_bf16", U.stream(), dx.data_ptr(), ds.data_ptr(), out.data_ptr(),
                      len(src), H, n_tok) == 0
    torch.cuda.synchronize()
    o = U.host_u16(out)
    for r, s_ in enumerate(src):
        assert np.array_equal(o[r], x[s_] if 0 <= s_ < n_tok else np.zeros(H, np.uint16))
    # strided: only rows 0, 3, 6 are written
    out.fill_(0x1111)
    src9 = np.array([1, 0, 0, 4, 0, 0, -1, 0, 0], np.int32)
    ds9 = U.dev(src9)
    out9 = torch.full((9, H), 0x1111, dtype=torch.int16, device="cuda")
    assert U.ffi.call("nv_kernels_gather_rows_bf16_strided", U.stream(), dx.data_ptr(), ds9.data_ptr(),
                      out9.data_ptr(), 9, H, n_tok, 3) == 0
    torch.cuda.synchronize()
    o9 = U.host_u16(out9)
    assert np.array_equal(o9[0], x[1]) and np.array_equal(o9[3], x[4]) and np.all(o9[6] == 0)
    assert np.all(o9[1] == 0x1111)
    assert U.ffi.call("nv_kernels_gather_rows_bf16_strided", U.stream(), dx.data_ptr(), ds9.data_ptr(),
                      out9.data_ptr(), 9, H, n_tok, 4) == -3

    # gather_f32_by_ids
    srcf = rng.standard_normal(E).astype(np.float32)
    idsf = np.array([3, -1, 9, 0], np.int32)
    dsf, dif = U.dev(srcf), U.dev(idsf)
    dst = torch.zeros(4, dtype=torch.float32, device="cuda")
    assert U.ffi.call("nv_kernels_gather_f32_by_ids", U.stream(), dsf.data_ptr(), dif.data_ptr(), dst.data_ptr(), 4) == 0
    torch.cuda.synchronize()
    assert np.array_equal(dst.cpu().numpy(), np.array([srcf[3], 0, srcf[9], srcf[0]], np.float32))

    # permute + unpermute
    topk = np.stack([rng.permutation(E)[:k] for _ in range(n_tok)]).astype(np.int32)
    dt = U.dev(topk)
    perm = torch.zeros(n_tok * k, dtype=torch.int32, device="cuda")
    offs = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    inv = torch.zeros(n_tok * k, dtype=torch.int32, device="cuda")
    scr = torch.zeros(E, dtype=torch.int32, device="cuda")
    assert U.ffi.call("nv_kernels_moe_permute", U.stream(), dt.data_ptr(), perm.data_ptr(), offs.data_ptr(),
                      inv.data_ptr(), scr.data_ptr(), n_tok, k, E) == 0
    torch.cuda.synchronize()
    perm_h, offs_h, inv_h = perm.cpu().numpy(), offs.cpu().numpy(), inv.cpu().numpy()
    counts = np.bincount(topk.ravel(), minlength=E)
    assert np.array_equal(offs_h, np.concatenate([[0], np.cumsum(counts)]))
    assert sorted(inv_h) == list(range(n_tok * k))
    for t in range(n_tok * k):
        e = topk.ravel()[t]
        assert offs_h[e] <= inv_h[t] < offs_h[e + 1] and perm_h[inv_h[t]] == t // k

    stride = H + 8
    ys = U.gauss_bf16(rng, (n_tok * k, stride))
    wts = rng.random((n_tok, k)).astype(np.float32)
    dy, dw = U.dev(ys), U.dev(wts)
    acc = torch.zeros((n_tok, H), dtype=torch.float32, device="cuda")
    assert U.ffi.call("nv_kernels_moe_unpermute_scatter", U.stream(), dy.data_ptr(), dw.data_ptr(), inv.data_ptr(),
                      acc.data_ptr(), n_tok, k, H, stride) == 0
    torch.cuda.synchronize()
    want = ref.moe_unpermute_scatter(ys, wts, inv_h.reshape(n_tok, k), H, stride)
    np.testing.assert_allclose(acc.cpu().numpy(), want, rtol=1e-6, atol=1e-7)

    shared = rng.standard_normal((n_tok, H)).astype(np.float32)
    resid = U.gauss_bf16(rng, (n_tok, H))
    dsh, dr = U.dev(shared), U.dev(resid)
    outb = torch.zeros((n_tok, H), dtype=torch.int16, device="cuda")
    assert U.ffi.call("nv_kernels_moe_unpermute_scatter_tail", U.stream(), dy.data_ptr(), dw.data_ptr(),
                      inv.data_ptr(), dsh.data_ptr(), dr.data_ptr(), outb.data_ptr(), n_tok, k, H, stride) == 0
    torch.cuda.synchronize()
    fb = ref.bf16_to_f32(ref.f32_to_bf16(acc.cpu().numpy() + shared))
    want_tail = ref.f32_to_bf16(ref.bf16_to_f32(resid) + fb)
    assert U.bf16_ulp_diff(U.host_u16(outb), want_tail).max() <= 1


@pytest.mark.parametrize("n,k", [(512, 2048), (2048, 512), (768, 2048), (200, 272)])
def test_grouped_w4a4_expert_gemv(n, k):
    """rust/crates/nv-kernels/tests/moe_grouped_fp4_gemv_parity.rs shapes: grouped == per-expert
    oracle within 2 bf16 ulp or 1e-3 abs, out-of-range ids write zeros, bit-stable run to run."""
    U.require_gpu()
    rng = np.random.default_rng(n + k)
    E, groups, tile = 6, 9, 128
    ids = np.array([0, 5, 2, 2, -1, 3, 6, 1, 4], np.int32)  # -1 and 6 are out of range
    wf = (rng.standard_normal((E, n, k)) * 0.05).astype(np.float32)
    bp = np.zeros((E, n, k // 2), np.uint8)
    n_pad, kb_pad = -(-n // 128) * 128, -(-(k // 16) // 4) * 4
    bs = np.zeros((E, n_pad * kb_pad), np.uint8)
    b_lin = []
    alphas = np.zeros(E, np.float32)
    for e in range(E):
        g = ref.weight_global(wf[e])
        p, lin = ref.quantize_rows(wf[e], g)
        bp[e], bs[e] = p, ref.swizzle_scales(lin)
        b_lin.append(lin)
        alphas[e] = np.float32(1.0) / np.float32(g)
    xa = (rng.standard_normal((groups, k)) * 2.0).astype(np.float32)
    ap = np.zeros((groups * tile, k // 2), np.uint8)
    a_sw = np.zeros((groups, tile * kb_pad), np.uint8)
    a_lin = []
    for g_ in range(groups):
        p, lin = ref.quantize_rows(xa[g_:g_ + 1], 1.0)
        ap[g_ * tile] = p[0]
        full = np.zeros((tile, k // 16), np.uint8)
        full[0] = lin[0]
        a_sw[g_] = ref.swizzle_scales(full)
        a_lin.append(lin)
    d_stride = n + 16
    dev = [U.dev(a) for a in (ap, a_sw, bp, bs, alphas, ids)]
    d = torch.full((groups, d_stride), 0x7FC0, dtype=torch.int16, device="cuda")

    def run():
        rc = U.ffi.call("nv_kernels_moe_grouped_fp4_gemv_m1_bf16", U.stream(), dev[0].data_ptr(), dev[1].data_ptr(),
                        dev[2].data_ptr(), dev[3].data_ptr(), dev[4].data_ptr(), d.data_ptr(), dev[5].data_ptr(),
                        groups, E, n, k, tile, d_stride)
        assert rc == 0
        torch.cuda.synchronize()
        return U.host_u16(d).copy()

    out = run()
    assert np.array_equal(out, run())  # bit-stable
    assert np.all(out[:, n:] == 0x7FC0)
    for g_ in range(groups):
        e = ids[g_]
        if e < 0 or e >= E:
            assert np.all(out[g_, :n] == 0)
            continue
        want = ref.matmul_w4a4(ap[g_ * tile:g_ * tile + 1], a_lin[g_], bp[e], b_lin[e], 1, n, k, float(alphas[e]))
        ulp = U.bf16_ulp_diff(out[g_, :n], want[0])
        absd = np.abs(ref.bf16_to_f32(out[g_, :n]) - ref.bf16_to_f32(want[0]))
        assert np.all((ulp <= 2) | (absd <= 1e-3))
    s = U.stream()
    assert U.ffi.call("nv_kernels_moe_grouped_fp4_gemv_m1_bf16", s, 0, 0, 0, 0, 0, 0, 0, 70000, E, n, k, 128, n) == -9
    assert U.ffi.call("nv_kernels_moe_grouped_fp4_gemv_m1_bf16", s, 0, 0, 0, 0, 0, 0, 0, 4, E, n, k, 100, n) == -1
    assert U.ffi.call("nv_kernels_moe_grouped_fp4_gemv_m1_bf16", s, 4, 0, 0, 0, 0, 0, 0, 4, E, n, k, 128, n) == -2


@pytest.mark.parametrize("n_tok", [1, 5, 16, 64])
def test_grouped_w4a16_moe_decode_matches_the_per_pair_oracle(n_tok):
    """Tokens grouped per expert must equal the per-(token, expert) computation: route, expert MLP
    (gate/up W4A16 -> bf16, SiLU(gate)*up rounded to bf16, down W4A16 -> bf16), f32 weighted combine.
    Router ids and the permutation are exact; outputs are within bf16 rounding of the f64 oracle."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(100 + n_tok)
    E, top_k, hidden, inter = 16, 4, 256, 384
    experts, host = [], []
    for e in range(E):
        trip, htrip = [], []
        for (n, k) in ((inter, hidden), (inter, hidden), (hidden, inter)):
            w = U.gauss_bf16(rng, (n, k), 0.05)
            packed, sw, alpha = ref.quantize_weight_bf16(w)
            trip.append(sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(sw), alpha, k, n))
            htrip.append((packed, sw, alpha))
        experts.append(tuple(trip))
        host.append(htrip)
    w = sp.MoeGroupedWeights.build_from_experts(experts)
    ctx = sp.GroupedDecodeContext(w, 64, top_k, "cuda")
    x = U.gauss_bf16(rng, (n_tok, hidden))
    logits = rng.standard_normal((n_tok, E)).astype(np.float32)
    if n_tok >= 16:
        logits[:, 3] += 4.0  # one hot expert: more than 8 tokens on it (walks the chunk loop)
    xt = U.dev(x).view(torch.bfloat16)
    y = sp.forward_grouped_decode(w, ctx, xt, U.dev(logits))
    torch.cuda.synchronize()
    ctx.check_status()   # no kernel met a routing table it had to refuse
    got = y.cpu().numpy()
    # the fused router's list of active experts: ascending, exactly the experts that won a slot
    n_act = int(ctx.n_active.cpu().numpy()[0])
    assert np.array_equal(ctx.active.cpu().numpy()[:n_act], np.unique(ctx.topk_ids[:n_tok].cpu().numpy()))
    ids, wts = ref.moe_route_topk(logits, top_k)
    assert np.array_equal(ctx.topk_ids[:n_tok].cpu().numpy(), ids)
    want = np.zeros((n_tok, hidden), np.float64)
    for t in range(n_tok):
        for j in range(top_k):
            e = ids[t, j]
            (pg, sg, ag), (pu, su, au), (pd, sd, ad) = host[e]
            gate = ref.f32_to_bf16(ref.linear_w4a16_f64(pg, sg, x[t:t + 1], ag, inter, hidden).astype(np.float32))
            up = ref.f32_to_bf16(ref.linear_w4a16_f64(pu, su, x[t:t + 1], au, inter, hidden).astype(np.float32))
            act = ref.f32_to_bf16(ref.silu_mul(gate, up, round_bf16=True))
            down = ref.f32_to_bf16(ref.linear_w4a16_f64(pd, sd, act, ad, hidden, inter).astype(np.float32))
            want[t] += np.float64(wts[t, j]) * ref.bf16_to_f32(down)[0].astype(np.float64)
    assert U.rel_err_floor(got, want) < 1e-2
    # grouped == per-pair: the same tokens sent one at a time give the same bits
    if n_tok == 5:
        for t in range(n_tok):
            y1 = sp.forward_grouped_decode(w, ctx, xt[t:t + 1].contiguous(), U.dev(logits[t:t + 1])).cpu().numpy().copy()
            assert np.array_equal(y1[0], got[t])


@pytest.mark.parametrize("E,K,mode,n", [(128, 8, 0, 1), (128, 8, 0, 64), (256, 8, 0, 33), (16, 4, 0, 7), (128, 8, 1, 16),
                                        (200, 6, 0, 5)])
def test_fused_route_permute_equals_the_two_kernels(E, K, mode, n):
    """nvk_b200_moe_route_permute writes exactly what nv_kernels_moe_route_topk + nv_kernels_moe_permute
    write (ids, offsets, permutation: equal; weights: bit-equal)."""
    U.require_gpu()
    rng = np.random.default_rng(E * 100 + n)
    lg = rng.standard_normal((n, E)).astype(np.float32)
    lg[0, 1] = lg[0, E - 1] = 8.0
    bias = (rng.standard_normal(E) * 0.1).astype(np.float32) if mode == 1 else None
    dl = U.dev(lg)
    db = U.dev(bias) if bias is not None else None
    scaling = 2.5 if mode == 1 else 1.0

    def bufs():
        i32 = dict(dtype=torch.int32, device="cuda")
        return (torch.full((n, K), -5, **i32), torch.zeros((n, K), dtype=torch.float32, device="cuda"),
                torch.full((n * K,), -5, **i32), torch.full((E + 1,), -5, **i32), torch.full((n * K,), -5, **i32))

    a = bufs()
    scr = torch.zeros(E, dtype=torch.int32, device="cuda")
    assert U.ffi.call("nv_kernels_moe_route_topk", U.stream(), dl.data_ptr(), db.data_ptr() if db is not None else None,
                      a[0].data_ptr(), a[1].data_ptr(), n, E, K, mode, 0.0, 1, scaling) == 0
    assert U.ffi.call("nv_kernels_moe_permute", U.stream(), a[0].data_ptr(), a[2].data_ptr(), a[3].data_ptr(),
                      a[4].data_ptr(), scr.data_ptr(), n, K, E) == 0
    b = bufs()
    assert U.ffi.call("nvk_b200_moe_route_permute", U.stream(), dl.data_ptr(), db.data_ptr() if db is not None else None,
                      b[0].data_ptr(), b[1].data_ptr(), b[2].data_ptr(), b[3].data_ptr(), b[4].data_ptr(), None, None, n, E,
                      K, mode, 0.0, 1, scaling) == 0
    torch.cuda.synchronize()
    for x, y in zip(a, b):
        assert np.array_equal(x.cpu().numpy().view(np.int32), y.cpu().numpy().view(np.int32))
    # with the list of active experts: same outputs, plus the experts that received slots, ascending
    c = bufs()
    act = torch.full((min(E, n * K),), -5, dtype=torch.int32, device="cuda")
    n_act = torch.full((1,), -5, dtype=torch.int32, device="cuda")
    assert U.ffi.call("nvk_b200_moe_route_permute", U.stream(), dl.data_ptr(), db.data_ptr() if db is not None else None,
                      c[0].data_ptr(), c[1].data_ptr(), c[2].data_ptr(), c[3].data_ptr(), c[4].data_ptr(),
                      act.data_ptr(), n_act.data_ptr(), n, E, K, mode, 0.0, 1, scaling) == 0
    torch.cuda.synchronize()
    for x, y in zip(a, c):
        assert np.array_equal(x.cpu().numpy().view(np.int32), y.cpu().numpy().view(np.int32))
    want_active = np.unique(a[0].cpu().numpy())
    assert int(n_act.cpu().numpy()[0]) == want_active.size
    assert np.array_equal(act.cpu().numpy()[:want_active.size], want_active)
    # the permutation is the stable sort of the slots by expert
    flat = a[0].cpu().numpy().ravel()
    order = np.argsort(flat, kind="stable")
    assert np.array_equal(a[2].cpu().numpy(), (order // K).astype(np.int32))
    assert np.array_equal(a[4].cpu().numpy()[order], np.arange(n * K, dtype=np.int32))
    assert U.ffi.call("nvk_b200_moe_route_permute", U.stream(), 0, 0, 0, 0, 0, 0, 0, 0, 0, 4, 257, 4, 0, 0.0, 1, 1.0) == -3
    assert U.ffi.call("nvk_b200_moe_route_permute", U.stream(), 0, 0, 0, 0, 0, 0, 0, 0, 0, 4, 8, 9, 0, 0.0, 1, 1.0) == -2


@pytest.mark.parametrize("n_tok", [3, pytest.param(200, marks=pytest.mark.needs_cuda_runtime)])
def test_moe_block_matches_the_mixture_formula(n_tok):
    """MoeBlock.forward == sum_j softmax(top-k logits)_j * expert_j(x) + sigmoid(x . w_g) * shared(x)
    (rust/crates/nv-layers/src/moe.rs:1035-1133 checks the same closed form on the Cpu backend).
    3 tokens take the decode path (W4A16 experts), 200 the prefill route (FP4 x FP4 experts); the oracle
    follows each route's own numerics."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(500 + n_tok)
    E, top_k, hidden, inter, sh_inter = 8, 2, 256, 384, 512

    def make(n, k, std=0.05):
        w = U.gauss_bf16(rng, (n, k), std)
        packed, sw, alpha = ref.quantize_weight_bf16(w)
        return sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(sw), alpha, k, n), (packed, sw, alpha)

    experts, host = [], []
    for e in range(E):
        trip = [make(inter, hidden), make(inter, hidden), make(hidden, inter)]
        experts.append(tuple(t[0] for t in trip))
        host.append([t[1] for t in trip])
    shared = [make(sh_inter, hidden), make(sh_inter, hidden), make(hidden, sh_inter)]
    w_router = U.gauss_bf16(rng, (E, hidden), 0.5)
    w_sgate = U.gauss_bf16(rng, (1, hidden), 0.1)
    cfg = sp.MoeConfig(hidden, E, top_k, inter, sh_inter)
    blk = sp.MoeBlock(cfg, sp.Bf16Linear(U.dev(w_router).view(torch.bfloat16)),
                      sp.MoeGroupedWeights.build_from_experts(experts),
                      sp.Nvfp4Mlp(*[s[0] for s in shared]), sp.Bf16Linear(U.dev(w_sgate).view(torch.bfloat16)))
    x = U.gauss_bf16(rng, (n_tok, hidden))
    y = blk.forward(U.dev(x).view(torch.bfloat16))
    torch.cuda.synchronize()
    assert y.dtype == torch.bfloat16 and tuple(y.shape) == (n_tok, hidden)
    got = y.float().cpu().numpy()

    # router: bf16 GEMV output widened to f32, top-k, softmax over the winners.  The routing decision
    # is taken from the device's own logits (the GEMV has its parity test; a logit one bf16 ulp away
    # from the host's could otherwise swap two near-equal experts), after checking them against the host.
    logits = blk.gate.forward(U.dev(x).view(torch.bfloat16)).float().cpu().numpy()
    host_logits = ref.bf16_to_f32(ref.linear_cpu_backend(w_router, x))
    assert U.rel_err_floor(logits, host_logits.astype(np.float64)) < 1e-2
    ids, wts = ref.moe_route_topk(logits, top_k)

    def mlp_w4a16(h, xrow, n_int):
        (pg, sg, ag), (pu, su, au), (pd, sd, ad) = h
        gate = ref.f32_to_bf16(ref.linear_w4a16_f64(pg, sg, xrow, ag, n_int, hidden).astype(np.float32))
        up = ref.f32_to_bf16(ref.linear_w4a16_f64(pu, su, xrow, au, n_int, hidden).astype(np.float32))
        act = ref.f32_to_bf16(ref.silu_mul(gate, up, round_bf16=True))
        return ref.bf16_to_f32(ref.f32_to_bf16(ref.linear_w4a16_f64(pd, sd, act, ad, hidden, n_int).astype(np.float32)))[0]

    def mlp_w4a4(h, xrow):
        (pg, sg, ag), (pu, su, au), (pd, sd, ad) = h
        lg, lu, ld = (ref.unswizzle_scales(s, n, k // 16) for s, n, k in ((sg, inter, hidden), (su, inter, hidden),
                                                                          (sd, hidden, inter)))
        xp, xl = ref.quantize_rows_bf16(xrow, 1.0)
        gate = ref.matmul_w4a4(xp, xl, pg, lg, 1, inter, hidden, ag)
        up = ref.matmul_w4a4(xp, xl, pu, lu, 1, inter, hidden, au)
        ap, al = ref.quantize_rows(ref.silu_mul(gate, up, round_bf16=False).reshape(1, inter), 1.0)
        return ref.bf16_to_f32(ref.matmul_w4a4(ap, al, pd, ld, 1, hidden, inter, ad))[0]

    sg_logit = ref.bf16_to_f32(ref.linear_cpu_backend(w_sgate, x))[:, 0]
    want = np.zeros((n_tok, hidden), np.float64)
    for t in range(n_tok):
        for j in range(top_k):
            h = host[ids[t, j]]
            out = mlp_w4a16(h, x[t:t + 1], inter) if n_tok <= 64 else mlp_w4a4(h, x[t:t + 1])
            want[t] += np.float64(wts[t, j]) * out.astype(np.float64)
        sh = mlp_w4a16([s[1] for s in shared], x[t:t + 1], sh_inter)
        want[t] += (1.0 / (1.0 + np.exp(-np.float64(sg_logit[t])))) * sh.astype(np.float64)
    assert U.rel_err_floor(got, want) < 2e-2


def test_host_rule_constructor_and_draft_twin():
    """from_bf16_quantized_nvfp4: global 1.0, alpha 1.0, bytes of the host quantizer
    (rust/crates/nv-layers/src/linear.rs:2228-2275); a bf16 linear's draft twin is the device-quantized
    NVFP4 copy of a row range, with that range's own global (linear.rs:2277-2296)."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(77)
    n, k = 256, 512
    w = U.gauss_bf16(rng, (n, k), 0.5)
    wt = U.dev(w).view(torch.bfloat16)
    lin = sp.Nvfp4Linear.from_bf16_quantized_nvfp4(wt)
    packed, lw = ref.quantize_rows_bf16(w, 1.0)
    assert lin.weight_alpha == 1.0
    assert np.array_equal(lin.weight_u8.cpu().numpy(), packed)
    assert np.array_equal(lin.weight_scales.cpu().numpy(), ref.swizzle_scales(lw))
    twin = sp.Bf16Linear(wt).nvfp4_draft_twin_rows(128, 128)
    p2, s2, a2 = ref.quantize_weight_bf16(w[128:256])
    assert np.array_equal(twin.weight_u8.cpu().numpy(), p2) and np.array_equal(twin.weight_scales.cpu().numpy(), s2)
    assert twin.weight_alpha == a2 and (twin.out_features, twin.in_features) == (128, k)
    with pytest.raises(ValueError, match="out of range"):
        sp.Bf16Linear(wt).nvfp4_draft_twin_rows(200, 128)


@pytest.mark.parametrize("n,k", [(64, 256), (129, 1024), (512, 2048), (7, 48)])
def test_w4a4_single_gemv_matches_the_oracle(n, k):
    """nv_kernels_nvfp4_gemv_bf16 with an activation row quantized by nv_kernels_nvfp4_quantize_row_bf16
    (flat scales): equals the W4A4 host oracle (rust/crates/nv-quant/src/nvfp4.rs:1086-1106) within 2 bf16
    ulp -- the block dots are exact, only the order of the f32 block sum differs."""
    U.require_gpu()
    rng = np.random.default_rng(n * 7 + k)
    w = U.gauss_bf16(rng, (n, k), 0.02)
    packed, sw, alpha = ref.quantize_weight_bf16(w)
    x = U.gauss_bf16(rng, (1, k))
    dx = U.dev(x)
    xp = torch.zeros(k // 2, dtype=torch.uint8, device="cuda")
    xs = torch.zeros(k // 16, dtype=torch.uint8, device="cuda")
    assert U.ffi.call("nv_kernels_nvfp4_quantize_row_bf16", U.stream(), dx.data_ptr(), xp.data_ptr(), xs.data_ptr(),
                      1.0, k) == 0
    y = torch.full((n + 64,), 0x7FC0, dtype=torch.int16, device="cuda")
    dw, ds = U.dev(packed), U.dev(sw)
    assert U.ffi.call("nv_kernels_nvfp4_gemv_bf16", U.stream(), dw.data_ptr(), ds.data_ptr(), xp.data_ptr(),
                      xs.data_ptr(), y.data_ptr(), alpha, n, k) == 0
    torch.cuda.synchronize()
    out = U.host_u16(y)
    assert np.all(out[n:] == 0x7FC0)
    ap, alin = ref.quantize_rows_bf16(x, 1.0)
    assert np.array_equal(xp.cpu().numpy(), ap[0]) and np.array_equal(xs.cpu().numpy(), alin[0])
    want = ref.matmul_w4a4(ap, alin, packed, ref.unswizzle_scales(sw, n, k // 16), 1, n, k, alpha)[0]
    ulp = U.bf16_ulp_diff(out[:n], want)
    absd = np.abs(ref.bf16_to_f32(out[:n]) - ref.bf16_to_f32(want))
    assert np.all((ulp <= 2) | (absd <= 1e-3))
    assert U.ffi.call("nv_kernels_nvfp4_gemv_bf16", U.stream(), dw.data_ptr(), ds.data_ptr(), xp.data_ptr(),
                      xs.data_ptr(), y.data_ptr(), alpha, n, 40) == -1


def test_sigmoid_rowgate():
    U.require_gpu()
    rng = np.random.default_rng(8)
    rows, hidden = 5, 300
    x = rng.standard_normal((rows, hidden)).astype(np.float32)
    g = (rng.standard_normal(rows) * 3).astype(np.float32)
    dx, dg = U.dev(x), U.dev(g)
    y = torch.zeros((rows, hidden), dtype=torch.float32, device="cuda")
    assert U.ffi.call("nv_kernels_mul_sigmoid_rowgate_f32", U.stream(), dx.data_ptr(), dg.data_ptr(), y.data_ptr(),
                      rows, hidden) == 0
    torch.cuda.synchronize()
    want = x * (1.0 / (1.0 + np.exp(-g.astype(np.float64))))[:, None]
    np.testing.assert_allclose(y.cpu().numpy(), want, rtol=2e-6, atol=1e-7)
    # in place
    assert U.ffi.call("nv_kernels_mul_sigmoid_rowgate_f32", U.stream(), dx.data_ptr(), dg.data_ptr(), dx.data_ptr(),
                      rows, hidden) == 0
    torch.cuda.synchronize()
    assert torch.equal(dx, y)


def test_rmsnorm_bf16_and_the_prenorm_decode_route():
    """nv_kernels_rmsnorm_bf16 == bf16((x * rstd) * w) up to the device's rsqrt / sum order (at most one
    bf16 ulp on a few elements); Nvfp4Linear.forward_prenorm_decode == the linear applied to that."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(61)
    m, k, n, eps = 3, 1024, 256, 1e-6
    x = U.gauss_bf16(rng, (m, k), 1.5)
    nw = U.gauss_bf16(rng, (k,), 1.0)
    dx, dw = U.dev(x), U.dev(nw)
    y = torch.zeros((m, k), dtype=torch.int16, device="cuda")
    assert U.ffi.call("nv_kernels_rmsnorm_bf16", U.stream(), dx.data_ptr(), dw.data_ptr(), y.data_ptr(), m, k, eps) == 0
    torch.cuda.synchronize()
    xf, wf = ref.bf16_to_f32(x), ref.bf16_to_f32(nw)
    rstd = (1.0 / np.sqrt((xf.astype(np.float64) ** 2).mean(1) + eps)).astype(np.float32)
    normed = ref.f32_to_bf16((xf * rstd[:, None]) * wf[None, :])
    got = U.host_u16(y)
    assert U.bf16_ulp_diff(got, normed).max() <= 1 and (got == normed).mean() > 0.99
    w = U.gauss_bf16(rng, (n, k), 0.02)
    packed, sw, alpha = ref.quantize_weight_bf16(w)
    lin = sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(sw), alpha, k, n)
    out = lin.forward_prenorm_decode(dx.view(torch.bfloat16), dw.view(torch.bfloat16), eps)
    direct = lin.forward(y.view(torch.bfloat16))
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), direct.view(torch.int16))
    want = ref.linear_w4a16_f64(packed, sw, got, alpha, n, k)
    assert U.rel_err_floor(out.float().cpu().numpy(), want) < 1e-4 + 1e-2


# ---- routing tables are data, not trusted: nothing may index with an id, offset or row that is out of range ----

def test_router_rows_with_too_few_usable_scores():
    """NaN never wins, an expert wins at most once, missing winners are id -1 / weight 0 and still take
    part in the softmax like a padded loop over K entries would."""
    U.require_gpu()
    E, K = 16, 4
    lg = np.zeros((5, E), np.float32)
    lg[0] = np.nan                                    # nothing usable
    lg[1] = np.nan; lg[1, [3, 9]] = [1.0, 2.0]        # two usable
    lg[2] = -np.inf; lg[2, 7] = 0.5                   # -inf is an ordinary (lowest) score: lowest ids first
    lg[3] = np.arange(E, dtype=np.float32); lg[3, 5] = np.nan
    lg[4] = 1.0                                       # all tied: lowest ids
    ids = torch.full((5, K), -9, dtype=torch.int32, device="cuda")
    w = torch.full((5, K), -9.0, dtype=torch.float32, device="cuda")
    assert U.ffi.call("nv_kernels_moe_route_topk", U.stream(), U.dev(lg).data_ptr(), None, ids.data_ptr(), w.data_ptr(),
                      5, E, K, 0, 0.0, 1, 1.0) == 0
    torch.cuda.synchronize()
    got, gw = ids.cpu().numpy(), w.cpu().numpy()
    assert got[0].tolist() == [-1, -1, -1, -1]
    assert got[1].tolist() == [9, 3, -1, -1]
    assert got[2].tolist() == [7, 0, 1, 2]
    assert got[3].tolist() == [15, 14, 13, 12]
    assert got[4].tolist() == [0, 1, 2, 3]
    # row 1: softmax over (2, 1, 0, 0), the two padded entries with raw score 0
    e = np.exp(np.array([2, 1, 0, 0], np.float32) - np.float32(2))
    np.testing.assert_allclose(gw[1], e / e.sum(), rtol=1e-6)
    np.testing.assert_allclose(gw[4], 0.25, rtol=1e-6)
    # rows without degenerate scores equal the oracle exactly
    wi, ww = ref.moe_route_topk(lg[3:5].copy(), K)
    assert np.array_equal(got[4], wi[1])


def test_slot_sort_and_combine_skip_ids_outside_the_expert_range():
    U.require_gpu()
    rng = np.random.default_rng(11)
    n_tok, k, E, H = 7, 4, 6, 64
    topk = rng.integers(0, E, (n_tok, k)).astype(np.int32)
    topk[0, 1] = -1
    topk[3, 0] = E          # one past the last expert
    topk[5, 3] = 1 << 20
    flat = topk.ravel()
    valid = (flat >= 0) & (flat < E)
    for entry, with_scratch in (("nv_kernels_moe_permute", True), ("nvk_b200_moe_permute_static", False)):
        dt = U.dev(topk)
        perm = torch.full((n_tok * k + 8,), -7, dtype=torch.int32, device="cuda")
        offs = torch.full((E + 1 + 8,), -7, dtype=torch.int32, device="cuda")
        inv = torch.full((n_tok * k + 8,), -7, dtype=torch.int32, device="cuda")
        args = [U.stream(), dt.data_ptr(), perm.data_ptr(), offs.data_ptr(), inv.data_ptr()]
        scr = None
        if with_scratch:
            scr = torch.full((E + 8,), 12345, dtype=torch.int32, device="cuda")   # stale contents, canary tail
            args.append(scr.data_ptr())
        assert U.ffi.call(entry, *args, n_tok, k, E) == 0
        torch.cuda.synchronize()
        perm_h, offs_h, inv_h = perm.cpu().numpy(), offs.cpu().numpy(), inv.cpu().numpy()
        assert np.all(perm_h[n_tok * k:] == -7) and np.all(offs_h[E + 1:] == -7) and np.all(inv_h[n_tok * k:] == -7)
        if scr is not None:
            assert np.all(scr.cpu().numpy()[E:] == 12345)   # nothing written in front of or behind the counters
        counts = np.bincount(flat[valid], minlength=E)
        assert np.array_equal(offs_h[:E + 1], np.concatenate([[0], np.cumsum(counts)]))
        order = np.argsort(np.where(valid, flat, E), kind="stable")[:valid.sum()]   # stable sort of the valid slots
        assert np.array_equal(perm_h[:valid.sum()], (order // k).astype(np.int32))
        assert np.array_equal(inv_h[:n_tok * k][order], np.arange(valid.sum(), dtype=np.int32))
        assert np.all(inv_h[:n_tok * k][~valid] == -1)
    # combine: slots with inv_perm -1 add nothing; a row past the sorted buffer is skipped and reported
    ys = U.gauss_bf16(rng, (n_tok * k, H))
    wts = rng.random((n_tok, k)).astype(np.float32)
    inv_c = inv_h[:n_tok * k].copy()
    want = ref.moe_unpermute_scatter(ys, wts, inv_c.reshape(n_tok, k), H, H)
    dy, dw, di = U.dev(ys), U.dev(wts), U.dev(inv_c)
    acc = torch.zeros((n_tok, H), dtype=torch.float32, device="cuda")
    assert U.ffi.call("nv_kernels_moe_unpermute_scatter", U.stream(), dy.data_ptr(), dw.data_ptr(), di.data_ptr(),
                      acc.data_ptr(), n_tok, k, H, H) == 0
    torch.cuda.synchronize()
    np.testing.assert_allclose(acc.cpu().numpy(), want, rtol=1e-6, atol=1e-7)
    inv_bad = inv_c.copy()
    bad_slot = int(np.flatnonzero(valid)[2])
    inv_bad[bad_slot] = n_tok * k + 1000
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert U.ffi.call("nvk_b200_moe_combine", U.stream(), dy.data_ptr(), dw.data_ptr(), U.dev(inv_bad).data_ptr(),
                      acc.data_ptr(), n_tok, k, H, H, n_tok * k, status.data_ptr()) == 0
    torch.cuda.synchronize()
    assert int(status.cpu().numpy()[0]) == 4
    inv_skip = inv_c.copy()
    inv_skip[bad_slot] = -1
    want2 = ref.moe_unpermute_scatter(ys, wts, inv_skip.reshape(n_tok, k), H, H)
    np.testing.assert_allclose(acc.cpu().numpy(), want2, rtol=1e-6, atol=1e-7)


def test_combine_allreduce_on_one_device():
    """nvk_b200_moe_combine_allreduce on one GPU: a world of one equals nvk_b200_moe_combine bit for bit; with
    a second rank that never arrives the bounded wait runs out, err names it, y_acc stays untouched and the
    next call works."""
    U.require_gpu()
    import ctypes as C
    rng = np.random.default_rng(31)
    n_tok, k, hidden, max_ctas = 3, 4, 1032, 64
    slots = n_tok * k
    rows = U.dev(U.gauss_bf16(rng, (slots, hidden)))
    wts = U.dev(rng.random(slots).astype(np.float32))
    inv = U.dev(rng.permutation(slots).astype(np.int32))
    want = torch.zeros((n_tok, hidden), dtype=torch.float32, device="cuda")
    assert U.ffi.call("nvk_b200_moe_combine", U.stream(), rows.data_ptr(), wts.data_ptr(), inv.data_ptr(), want.data_ptr(),
                      n_tok, k, hidden, hidden, slots, None) == 0
    nbytes = U.ffi.lib().nvk_b200_moe_combine_buffer_bytes(2, max_ctas)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    epoch = torch.zeros(max_ctas, dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = torch.full((n_tok, hidden), -7.0, dtype=torch.float32, device="cuda")

    def call(world, ptrs):
        return U.ffi.call("nvk_b200_moe_combine_allreduce", U.stream(), C.addressof(ptrs), 0, world, rows.data_ptr(),
                          wts.data_ptr(), inv.data_ptr(), y.data_ptr(), n_tok, k, hidden, hidden, slots, None, max_ctas,
                          epoch.data_ptr(), err.data_ptr())

    one = (C.c_void_p * 1)(bufs[0].data_ptr())
    assert call(1, one) == 0
    torch.cuda.synchronize()
    assert int(err.cpu().numpy()[0]) == 0 and torch.equal(y, want)
    y.fill_(-7.0)
    two = (C.c_void_p * 2)(bufs[0].data_ptr(), bufs[1].data_ptr())
    assert U.ffi.call("nvk_b200_set_wait_limit", 1000) == 0
    try:
        assert call(2, two) == 0
        torch.cuda.synchronize()
        assert int(err.cpu().numpy()[0]) == 2 and bool((y == -7.0).all())
    finally:
        assert U.ffi.call("nvk_b200_set_wait_limit", 0) == 0
    err.zero_()
    assert call(1, one) == 0
    torch.cuda.synchronize()
    assert int(err.cpu().numpy()[0]) == 0 and torch.equal(y, want)


def test_grouped_linear_does_not_follow_offsets_or_rows_outside_its_buffers():
    U.require_gpu()
    rng = np.random.default_rng(12)
    E, n, k, slots, x_rows = 3, 128, 64, 6, 4
    packed = np.zeros((E, n, k // 2), np.uint8)
    scales = np.zeros((E, ref.swizzled_len(n, k // 16)), np.uint8)
    alphas = np.zeros(E, np.float32)
    host = []
    for e in range(E):
        p_, s_, a_, _ = U.make_weight(rng, n, k, 0.05)
        packed[e], scales[e], alphas[e] = p_, s_, a_
        host.append((p_, s_, a_))
    x = U.gauss_bf16(rng, (x_rows, k))
    offsets = np.array([0, 2, 9, 2000], np.int32)            # expert 1 and 2 run past the 6 slots
    rows = np.array([1, 3, 0, -4, 7, 2], np.int32)            # slots 3 and 4 name rows that do not exist
    y = torch.full((slots + 4, n), 0x7FC0, dtype=torch.int16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    dev = [U.dev(a) for a in (packed, scales, alphas, x, rows, offsets)]
    assert U.ffi.call("nvk_b200_moe_grouped_w4a16", U.stream(), dev[0].data_ptr(), dev[1].data_ptr(), None, None,
                      dev[2].data_ptr(), None, dev[3].data_ptr(), None, dev[4].data_ptr(), dev[5].data_ptr(), None,
                      None, y.data_ptr(), None, E, n, k, slots, x_rows, status.data_ptr()) == 0
    torch.cuda.synchronize()
    out = U.host_u16(y)
    assert np.all(out[slots:] == 0x7FC0)                      # nothing past the last slot
    assert int(status.cpu().numpy()[0]) == 3                  # both kinds of violation reported
    for slot, e in ((0, 0), (1, 0), (2, 1), (5, 1)):
        want = ref.linear_w4a16_f64(host[e][0], host[e][1], x[rows[slot]:rows[slot] + 1], host[e][2], n, k)
        assert U.rel_err_floor(ref.bf16_to_f32(out[slot]), want[0]) < 1e-2
    assert np.all(out[3] == 0) and np.all(out[4] == 0)        # rows that do not exist read as zeros


@pytest.mark.parametrize("n_tok,folded", [(1, False), (1, True), (3, False), (2, True)])
def test_tiled_w4a4_decode_step_matches_the_per_pair_oracle(n_tok, folded):
    """forward_grouped_decode_into: every (token, winner) pair a 128-row tile with row 0 live, activations
    quantized to NVFP4 with the winner's stored global, FP4 x FP4 expert GEMVs.  One token routes, gathers
    and quantizes in one launch (nv_kernels_moe_route_gather_quant_m1); several tokens take the separate
    kernels.  Oracle: the W4A4 statement per pair (rust/crates/nv-quant/src/nvfp4.rs:1086-1106)."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(500 + 10 * n_tok + folded)
    E, top_k, hidden, inter = 12, 3, 256, 128
    n_bank = E + (1 if folded else 0)
    experts, host = [], []
    for e in range(n_bank):
        trip, htrip = [], []
        for (n, k) in ((inter, hidden), (inter, hidden), (hidden, inter)):
            wf = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
            g = ref.weight_global(wf)
            packed, lin = ref.quantize_rows(wf, g)
            alpha = float(np.float32(1.0) / np.float32(g))
            trip.append(sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(ref.swizzle_scales(lin)), alpha, k, n))
            htrip.append((packed, lin, alpha))
        experts.append(tuple(trip))
        host.append(htrip)
    w = sp.MoeGroupedWeights.build_from_experts(experts[:E], shared=experts[E] if folded else None)
    gu = (0.5 + rng.random(n_bank)).astype(np.float32)
    dn = (0.5 + rng.random(n_bank)).astype(np.float32)
    w.input_globals_gate_up, w.input_globals_down = U.dev(gu), U.dev(dn)
    ctx = sp.TiledDecodeContext(w, n_tok, top_k, "cuda", folded_shared=folded)
    x = U.gauss_bf16(rng, (n_tok, hidden))
    logits = rng.standard_normal((n_tok, E)).astype(np.float32)
    ctx.x_in.copy_(U.dev(x).view(torch.bfloat16))
    ctx.logits_f32.copy_(U.dev(logits))
    stamps = torch.zeros(5, dtype=torch.int64, device="cuda")
    sp.forward_grouped_decode_into(w, ctx, prof_base=stamps.data_ptr())
    torch.cuda.synchronize()
    got = ctx.y_acc.cpu().numpy()
    ids, wts = ref.moe_route_topk(logits, top_k)
    tpt = top_k + (1 if folded else 0)
    got_ids = ctx.topk_ids.cpu().numpy().reshape(n_tok, tpt)
    assert np.array_equal(got_ids[:, :top_k], ids)
    if folded:
        assert np.all(got_ids[:, top_k] == E) and np.all(ctx.topk_weights.cpu().numpy().reshape(n_tok, tpt)[:, top_k] == 1.0)
    st = stamps.cpu().numpy()
    assert np.all(st > 0) and np.all(np.diff(st) >= 0)   # timestamps were written, in stream order
    want = np.zeros((n_tok, hidden), np.float64)
    for t in range(n_tok):
        pairs = [(int(ids[t, j]), float(wts[t, j])) for j in range(top_k)] + ([(E, 1.0)] if folded else [])
        for e, wt in pairs:
            (pg, lg_, ag), (pu, lu, au), (pd, ld, ad) = host[e]
            xq, xlin = ref.quantize_rows_bf16(x[t:t + 1], float(gu[e]))
            a_gu = float(np.float32(ag) / gu[e])
            gate = ref.matmul_w4a4(xq, xlin, pg, lg_, 1, inter, hidden, a_gu)
            up = ref.matmul_w4a4(xq, xlin, pu, lu, 1, inter, hidden, float(np.float32(au) / gu[e]))
            act = ref.silu_mul(gate, up, round_bf16=False)                 # f32, not rounded before the quantizer
            aq, alin = ref.quantize_rows(act, float(dn[e]))
            down = ref.matmul_w4a4(aq, alin, pd, ld, 1, hidden, inter, float(np.float32(ad) / dn[e]))
            want[t] += np.float64(np.float32(wt)) * ref.bf16_to_f32(down)[0].astype(np.float64)
    assert U.rel_err_floor(got, want) < 1e-2
