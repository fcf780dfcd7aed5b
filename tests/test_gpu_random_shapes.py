"""Seeded random shapes through the C ABI: sizes nobody picked by hand (ragged last tiles, K that is a
multiple of 16 but not of 32 or 256, token counts between the template steps, expert counts around the
router's warp/CTA switch), each checked against the oracle with the bound of the hand-picked tests.
Every output buffer has a canary tail; on the host emulation every buffer also ends at a guard page, so
an index that leaves its buffer on any of these shapes ends the run."""
import numpy as np
import pytest
import torch

from oracle import ref
from tests import _util as U
from tests.test_gpu_linear import check_against_oracle, run_linear
from tests.test_gpu_quant_moe import gpu_quantize

pytestmark = pytest.mark.gpu


def _linear_cases(seed, count):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(count):
        m = int(rng.choice([1, 1, 2, 3, 5, 8, 9, 15, 16, 17, 31, 33, 48, 64]))
        n = int(rng.integers(1, 700))
        k = 16 * int(rng.integers(1, 90))
        if i % 3 == 0:
            k = (k + 31) // 32 * 32          # the tensor-core route's K rule
        form = int(rng.integers(0, 3))       # 0 plain, 1 two arms, 2 SiLU(x) * x2 prologue
        out.append((m, n, k, form, seed * 1000 + i))
    return out


@pytest.mark.parametrize("m,n,k,form,seed", _linear_cases(11, 36))
def test_random_linear_shapes(m, n, k, form, seed):
    U.require_gpu()
    rng = np.random.default_rng(seed)
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    x = U.gauss_bf16(rng, (m, k))
    if form == 1:
        packed_b, sw_b, alpha_b, _ = U.make_weight(rng, n, k)
        ya, yb = run_linear(packed, sw, x, alpha, m, n, k, packed_b, sw_b, alpha_b)
        check_against_oracle(ya, packed, sw, x, alpha, n, k, cpu_backend=False)
        check_against_oracle(yb, packed_b, sw_b, x, alpha_b, n, k, cpu_backend=False)
    elif form == 2:
        up = U.gauss_bf16(rng, (m, k))
        got = run_linear(packed, sw, x, alpha, m, n, k, up_bits=up)
        g, u = ref.bf16_to_f32(x), ref.bf16_to_f32(up)
        act = ref.f32_to_bf16((g / (np.float32(1.0) + np.exp(-g))).astype(np.float32) * u)
        want = ref.linear_w4a16_f64(packed, sw, act, alpha, n, k)
        # expf on the device and numpy's exp may round an activation to neighbouring bf16 values
        assert U.rel_err_floor(ref.bf16_to_f32(got).reshape(-1, n), want) < 2e-2
    else:
        got = run_linear(packed, sw, x, alpha, m, n, k)
        check_against_oracle(got, packed, sw, x, alpha, n, k, cpu_backend=False)


def _quant_cases(seed, count):
    rng = np.random.default_rng(seed)
    return [(int(rng.integers(1, 300)), 16 * int(rng.integers(1, 70)), float(rng.choice([1.0, 0.37, 96.0, 2688.0])),
             int(rng.integers(0, 2)), seed * 1000 + i) for i in range(count)]


@pytest.mark.parametrize("m,k,g,pad,seed", _quant_cases(12, 16))
def test_random_quantizer_shapes_are_byte_exact(m, k, g, pad, seed):
    U.require_gpu()
    rng = np.random.default_rng(seed)
    mags = np.exp(rng.uniform(np.log(1e-3), np.log(300.0), size=(m, 1))).astype(np.float32)
    x = ref.f32_to_bf16(rng.standard_normal((m, k)).astype(np.float32) * mags)
    m_pad = -(-m // 128) * 128 if pad else None
    p, s = gpu_quantize(x, g, m_pad)
    pw, lw = ref.quantize_rows_bf16(x, g, m_padded=m_pad) if pad else ref.quantize_rows_bf16(x, g)
    assert np.array_equal(p, pw)
    assert np.array_equal(s, ref.swizzle_scales(lw))


def _router_cases(seed, count):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(count):
        E = int(rng.choice([2, 7, 31, 32, 33, 64, 100, 128, 255, 256, 257, 384, 600]))
        K = int(rng.integers(1, min(E, 16) + 1))
        out.append((int(rng.integers(1, 70)), E, K, int(rng.integers(0, 2)), seed * 1000 + i))
    return out


@pytest.mark.parametrize("n,E,K,mode,seed", _router_cases(13, 16))
def test_random_router_shapes(n, E, K, mode, seed):
    """Ids bit-exact, weights to the last float operation's rounding, for every (tokens, experts, winners)
    drawn; then the slot sort of those ids against numpy's stable sort."""
    U.require_gpu()
    rng = np.random.default_rng(seed)
    lg = rng.standard_normal((n, E)).astype(np.float32)
    bias = (rng.standard_normal(E) * 0.1).astype(np.float32) if mode == 1 else None
    dl = U.dev(lg)
    db = U.dev(bias) if bias is not None else None
    ids = torch.full((n * K + 16,), -7, dtype=torch.int32, device="cuda")
    w = torch.full((n * K + 16,), -7.0, dtype=torch.float32, device="cuda")
    scaling = 2.5 if mode == 1 else 1.0
    assert U.ffi.call("nv_kernels_moe_route_topk", U.stream(), dl.data_ptr(), db.data_ptr() if db is not None else None,
                      ids.data_ptr(), w.data_ptr(), n, E, K, mode, 0.0, 1, scaling) == 0
    torch.cuda.synchronize()
    wi, ww = ref.moe_route_topk(lg, K, bias=bias, mode=mode, norm_topk=True, routed_scaling=scaling)
    got_ids, got_w = ids.cpu().numpy(), w.cpu().numpy()
    assert np.all(got_ids[n * K:] == -7) and np.all(got_w[n * K:] == -7.0)
    assert np.array_equal(got_ids[:n * K].reshape(n, K), wi)
    np.testing.assert_allclose(got_w[:n * K].reshape(n, K), ww, rtol=2e-6, atol=1e-7)

    total = n * K
    perm = torch.full((total + 8,), -7, dtype=torch.int32, device="cuda")
    offs = torch.full((E + 1 + 8,), -7, dtype=torch.int32, device="cuda")
    inv = torch.full((total + 8,), -7, dtype=torch.int32, device="cuda")
    scr = torch.zeros(E, dtype=torch.int32, device="cuda")
    assert U.ffi.call("nv_kernels_moe_permute", U.stream(), ids.data_ptr(), perm.data_ptr(), offs.data_ptr(),
                      inv.data_ptr(), scr.data_ptr(), n, K, E) == 0
    torch.cuda.synchronize()
    flat = wi.reshape(-1)
    order = np.argsort(flat, kind="stable")
    p, o, iv = perm.cpu().numpy(), offs.cpu().numpy(), inv.cpu().numpy()
    assert np.all(p[total:] == -7) and np.all(o[E + 1:] == -7) and np.all(iv[total:] == -7)
    assert np.array_equal(o[:E + 1], np.concatenate([[0], np.cumsum(np.bincount(flat, minlength=E))]))
    assert np.array_equal(p[:total], (order // K).astype(np.int32))     # sorted slot -> its token
    want_inv = np.empty(total, np.int32)
    want_inv[order] = np.arange(total, dtype=np.int32)
    assert np.array_equal(iv[:total], want_inv)


def _bf16_cases(seed, count):
    rng = np.random.default_rng(seed)
    return [(int(rng.integers(1, 65)), int(rng.integers(1, 900)), 8 * int(rng.integers(1, 120)), seed * 1000 + i)
            for i in range(count)]


@pytest.mark.parametrize("m,n,k,seed", _bf16_cases(14, 12))
def test_random_bf16_linear_shapes(m, n, k, seed):
    U.require_gpu()
    rng = np.random.default_rng(seed)
    w = U.gauss_bf16(rng, (n, k), 0.05)
    x = U.gauss_bf16(rng, (m, k))
    dw, dx = U.dev(w), U.dev(x)
    y = torch.full((m * n + 64,), 0x7FC0, dtype=torch.int16, device="cuda")
    assert U.ffi.call("nvk_b200_linear_bf16", U.stream(), dw.data_ptr(), dx.data_ptr(), y.data_ptr(), m, n, k) == 0
    torch.cuda.synchronize()
    out = U.host_u16(y)
    assert np.all(out[m * n:] == 0x7FC0)
    want = ref.bf16_to_f32(w).astype(np.float64) @ ref.bf16_to_f32(x).astype(np.float64).T   # [n, m]
    got = ref.bf16_to_f32(out[:m * n].reshape(m, n))
    assert U.rel_err_floor(got, want.T) < 1e-2


def _moe_cases(seed, count):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(count):
        E = int(rng.choice([2, 5, 8, 24, 40]))
        out.append((int(rng.choice([1, 2, 7, 9, 20, 33])), E, int(rng.integers(1, min(E, 6) + 1)),
                    32 * int(rng.integers(4, 14)), 32 * int(rng.integers(4, 14)), seed * 1000 + i))   # >= 128, the host rule
    return out


# the last two: K long enough that an expert's row tiles split K over a cluster (gate/up, and down too)
@pytest.mark.parametrize("n_tok,E,top_k,hidden,inter,seed", _moe_cases(15, 8) + [(3, 4, 2, 1024, 512, 15100),
                                                                                  (11, 6, 3, 1536, 1280, 15101)])
def test_random_moe_decode_shapes(n_tok, E, top_k, hidden, inter, seed):
    """The grouped decode step (router + slot sort + active list, gate/up, SiLU prologue + down, f32
    combine) on drawn (tokens, experts, winners, hidden, expert width), against the per-(token, expert)
    oracle; status word clean."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(seed)
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
    ctx = sp.GroupedDecodeContext(w, max(n_tok, 4), top_k, "cuda")
    x = U.gauss_bf16(rng, (n_tok, hidden))
    logits = rng.standard_normal((n_tok, E)).astype(np.float32)
    y = sp.forward_grouped_decode(w, ctx, U.dev(x).view(torch.bfloat16), U.dev(logits))
    torch.cuda.synchronize()
    ctx.check_status()
    got = y.cpu().numpy()
    ids, wts = ref.moe_route_topk(logits, top_k)
    assert np.array_equal(ctx.topk_ids[:n_tok].cpu().numpy(), ids)
    want = np.zeros((n_tok, hidden), np.float64)
    for t in range(n_tok):
        for j in range(top_k):
            (pg, sg, ag), (pu, su, au), (pd, sd, ad) = host[ids[t, j]]
            gate = ref.f32_to_bf16(ref.linear_w4a16_f64(pg, sg, x[t:t + 1], ag, inter, hidden).astype(np.float32))
            up = ref.f32_to_bf16(ref.linear_w4a16_f64(pu, su, x[t:t + 1], au, inter, hidden).astype(np.float32))
            act = ref.f32_to_bf16(ref.silu_mul(gate, up, round_bf16=True))
            down = ref.f32_to_bf16(ref.linear_w4a16_f64(pd, sd, act, ad, hidden, inter).astype(np.float32))
            want[t] += np.float64(wts[t, j]) * ref.bf16_to_f32(down)[0].astype(np.float64)
    assert U.rel_err_floor(got, want) < 1e-2
    if seed == 15100:
        # a token's bits do not depend on what else is in the batch, split K or not
        got = got.copy()
        xt = U.dev(x).view(torch.bfloat16)
        for t in range(n_tok):
            y1 = sp.forward_grouped_decode(w, ctx, xt[t:t + 1].contiguous(), U.dev(logits[t:t + 1])).cpu().numpy()
            assert np.array_equal(y1[0], got[t])


def _w4a8_cases(seed, count):
    rng = np.random.default_rng(seed)
    return [(int(rng.integers(1, 80)), int(rng.integers(1, 500)), 32 * int(rng.integers(1, 60)), seed * 1000 + i)
            for i in range(count)]


@pytest.mark.parametrize("m,n,k,seed", _w4a8_cases(16, 12))
def test_random_w4a8_shapes(m, n, k, seed):
    """int8 rows x NVFP4 weights, two arms and the residual form, M rows per call (chunks of 64 beyond):
    the W4A8 parity bound against integer-exact f64 dots."""
    U.require_gpu()
    from tests.test_gpu_w4a8 import TOL, rel_quarter, w4a8
    rng = np.random.default_rng(seed)
    wa, wb = U.make_weight(rng, n, k)[:3], U.make_weight(rng, n, k)[:3]
    x = (rng.standard_normal((m, k)) * np.linspace(0.2, 3.0, m)[:, None]).astype(np.float32)
    q, sc = ref.rowquant_i8(x)
    ya, yb = w4a8("nv_kernels_gemv_nvfp4_w4a8_dual_mk", wa, q, sc, m, n, k, second=wb)
    assert rel_quarter(ya, ref.linear_w4a8_f64(wa[0], wa[1], q, sc, wa[2], n, k)) < TOL
    assert rel_quarter(yb, ref.linear_w4a8_f64(wb[0], wb[1], q, sc, wb[2], n, k)) < TOL
    resid = U.gauss_bf16(rng, (m, n))
    yd = w4a8("nv_kernels_gemv_nvfp4_w4a8_down_residual_mk", wa, q, sc, m, n, k, residual=resid)
    assert rel_quarter(yd, ref.linear_w4a8_f64(wa[0], wa[1], q, sc, wa[2], n, k, resid)) < TOL


def _w4a4_cases(seed, count):
    rng = np.random.default_rng(seed)
    return [(int(rng.integers(1, 600)), 16 * int(rng.integers(1, 150)), seed * 1000 + i) for i in range(count)]


@pytest.mark.parametrize("n,k,seed", _w4a4_cases(17, 12))
def test_random_w4a4_gemv_shapes(n, k, seed):
    """Row quantizer (flat scales) + the M = 1 FP4 x FP4 GEMV on drawn (N, K): quantizer bytes exact, the
    product within 2 bf16 ulp of the W4A4 host oracle."""
    U.require_gpu()
    rng = np.random.default_rng(seed)
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


def _fused_cases(seed, count):
    rng = np.random.default_rng(seed)
    return [(int(rng.choice([1, 2, 5, 8, 13, 40, 64])), int(rng.integers(1, 600)), 32 * int(rng.integers(1, 70)),
             int(rng.integers(0, 2)), seed * 1000 + i) for i in range(count)]


@pytest.mark.parametrize("m,n,k,silu,seed", _fused_cases(18, 14))
def test_random_residual_and_normed_shapes(m, n, k, silu, seed):
    """The residual-update linear (with and without the SiLU prologue) on drawn shapes against the f64
    oracle, and -- for up to 8 rows -- the norm-in-prologue linear against norm kernel + plain linear,
    bit for bit."""
    U.require_gpu()
    from tests.test_gpu_linear import TOL_F64, device_rmsnorm, run_normed, run_residual
    rng = np.random.default_rng(seed)
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    x = U.gauss_bf16(rng, (m, k))
    resid = U.gauss_bf16(rng, (m, n), 2.0)
    if silu:
        up = U.gauss_bf16(rng, (m, k))
        got = run_residual(packed, sw, x, resid, alpha, m, n, k, up_bits=up)
        act = ref.f32_to_bf16(ref.silu_mul(x, up, round_bf16=True))
        want = ref.linear_w4a16_f64(packed, sw, act, alpha, n, k) + ref.bf16_to_f32(resid).astype(np.float64)
        assert U.rel_err_floor(ref.bf16_to_f32(got), want) < 2e-2
    else:
        got = run_residual(packed, sw, x, resid, alpha, m, n, k)
        want = ref.linear_w4a16_f64(packed, sw, x, alpha, n, k) + ref.bf16_to_f32(resid).astype(np.float64)
        assert U.rel_err_floor(ref.bf16_to_f32(got), want) < TOL_F64
    if m <= 8:
        nw = U.gauss_bf16(rng, (k,), 1.0)
        fused = run_normed((packed, sw, alpha), x, nw, 1e-6, m, n, k)
        assert np.array_equal(fused, run_linear(packed, sw, device_rmsnorm(x, nw, 1e-6), alpha, m, n, k))
