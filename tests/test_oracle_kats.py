"""Pins the CPU oracle to the reference's own known-answer tests.

Each test restates a check from rust/crates/nv-quant/src/nvfp4.rs:1180-1563
(modules `ue4m3_tests` and `paper_validation`) or from
rust/crates/nv-quant/tests/{nvfp4_oracle_fuzz,ue4m3_fuzz}.rs.  The reference has no
golden-vector files for this path; these known answers are its pins.
"""
import numpy as np
import pytest

from oracle import ref

STEP = 2.0 ** -9
f32 = np.float32


def hw_decode(b):
    e, m = (b >> 3) & 0xF, b & 7
    return (m / 8.0) * 2.0 ** -6 if e == 0 else (1 + m / 8.0) * 2.0 ** (e - 7)


def test_ue4m3_decode_every_byte_matches_hardware_formula():
    for b in range(0x7F):
        assert ref.decode_ue4m3(b) == hw_decode(b)


def test_ue4m3_subnormal_grid_round_trips():
    for m in range(8):
        v = m * STEP
        if m:
            assert ref.encode_ue4m3(v) == m
        assert ref.decode_ue4m3(m) == v
    assert ref.encode_ue4m3(8 * STEP) == 0x08
    assert ref.decode_ue4m3(0x08) == 2.0 ** -6


def test_ue4m3_subnormal_boundaries_round_to_nearest():
    for m in range(7):
        assert ref.encode_ue4m3(float(f32(m + 0.49) * f32(STEP))) == m
        assert ref.encode_ue4m3(float(f32(m + 0.51) * f32(STEP))) == m + 1
    assert ref.encode_ue4m3(7.6 * STEP) == 0x08
    assert ref.encode_ue4m3(0.49 * STEP) == 0
    assert ref.encode_ue4m3(0.51 * STEP) == 1


def test_ue4m3_small_values_known_bytes():
    cases = [2.0 ** -7, 1.5 * 2.0 ** -7, 2.5 * 2.0 ** -9, 2.0 ** -8, 2.0 ** -9, 2.0 ** -20]
    want = [4, 6, 3, 2, 1, 0]
    for v, w in zip(cases, want):
        b = ref.encode_ue4m3(v)
        assert b == w
        assert abs(hw_decode(b) - v) <= 0.5 * STEP + np.finfo(np.float32).eps


def test_ue4m3_normal_range():
    assert ref.encode_ue4m3(1.0) == 0x38 and ref.decode_ue4m3(0x38) == 1.0
    assert ref.encode_ue4m3(448.0) == 0x7E
    assert ref.encode_ue4m3(1e9) == 0x7E
    assert ref.encode_ue4m3(2.0 ** -6) == 0x08
    for b in range(0x08, 0x7F):
        assert ref.encode_ue4m3(hw_decode(b)) == b
    assert ref.encode_ue4m3(447.9999) != 0x7F
    assert ref.decode_ue4m3(ref.encode_ue4m3(1.0e6)) == 448.0
    for bad in (0.0, -1.0, float("nan"), float("inf"), float("-inf")):
        assert ref.encode_ue4m3(bad) == 0


def test_ue4m3_sweep_nearest_monotone_never_7f():
    # rust/crates/nv-quant/tests/ue4m3_fuzz.rs: nearest representable over a dense sweep,
    # monotone non-decreasing, 0x7F never emitted.
    grid = np.array(sorted({hw_decode(b) for b in range(0x7F)}), dtype=np.float64)
    xs = np.exp(np.linspace(np.log(2.0 ** -11), np.log(600.0), 20000)).astype(np.float32)
    prev = -1.0
    for x in xs:
        b = ref.encode_ue4m3(float(x))
        assert b != 0x7F
        d = ref.decode_ue4m3(b)
        best = np.min(np.abs(grid - min(float(x), 448.0)))
        assert abs(abs(d - min(float(x), 448.0)) - best) <= 1e-7 * max(1.0, float(x))
        assert d >= prev
        prev = d


def test_ue4m3_power_of_two_neighbours():
    # rust/crates/nv-kernels/tests/ue4m3_log2f_boundary.rs: exact floor(log2) at the f32
    # neighbours of powers of two.
    for e in range(-6, 9):
        p = f32(2.0) ** f32(e)
        below = np.nextafter(p, f32(0))
        above = np.nextafter(p, f32(1e9))
        for v in (below, p, above):
            v = min(float(v), 448.0)
            b = ref.encode_ue4m3(v)
            cands = [hw_decode(c) for c in range(0x7F)]
            best = min(abs(c - v) for c in cands)
            assert abs(hw_decode(b) - v) == pytest.approx(best, abs=1e-12)


def test_e2m1_codebook_and_roundtrip():
    expect = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for i, v in enumerate(expect):
        assert ref.decode_e2m1(i) == v
        assert ref.encode_e2m1(v) & 7 == i
        assert ref.decode_e2m1(i | 8) == -v
    for code in range(16):
        v = ref.decode_e2m1(code)
        assert ref.decode_e2m1(ref.encode_e2m1(v)) == v


def test_e2m1_nearest_and_ties_to_lower_code():
    book = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    x = -8.0
    while x < 8.0:
        d = ref.decode_e2m1(ref.encode_e2m1(x))
        best = np.min(np.abs(abs(np.float32(x)) - book))
        assert abs(abs(abs(np.float32(x)) - abs(d)) - best) < 1e-6
        x += 0.111
    for v, code in [(0.75, 1), (1.75, 3), (3.5, 5), (0.25, 0), (2.5, 4), (5.0, 6), (1.25, 2)]:
        assert ref.encode_e2m1(v) & 7 == code
        assert ref.encode_e2m1(-v) == (code | 8)
    assert ref.encode_e2m1(-0.0) == 8


def test_pack_order_even_k_in_low_nibble():
    v = np.zeros(16, np.float32)
    v[0], v[1], v[15] = 1.0, -2.0, 6.0
    packed, sb = ref.quantize_block(v)
    assert sb == 0x38  # amax 6 -> local scale 1.0
    assert packed[0] == ((ref.encode_e2m1(-2.0) << 4) | ref.encode_e2m1(1.0))
    assert packed[7] == (ref.encode_e2m1(6.0) << 4)


def _lcg_unit(seed):
    s = seed

    def nxt():
        nonlocal s
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        return np.float32(np.float64(s >> 33) / np.float64(1 << 31)) - np.float32(0.5)

    return nxt


def test_block_roundtrip_error_bound_and_zero_block():
    nxt = _lcg_unit(0x12345678)
    for amp in (0.05, 1.0, 37.0, 400.0):
        for _ in range(50):
            vals = np.array([nxt() * np.float32(2.0) * np.float32(amp) for _ in range(16)], np.float32)
            packed, sb = ref.quantize_block(vals)
            deq = ref.dequantize_block(packed, sb)
            assert np.all(np.abs(vals - deq) <= ref.decode_ue4m3(sb) + 1e-6)
    packed, sb = ref.quantize_block(np.zeros(16, np.float32))
    assert np.all(ref.dequantize_block(packed, sb) == 0)


def ref_slot(m, kb, k_blocks):
    k_tiles = -(-k_blocks // 4)
    tile = (m // 128) * k_tiles + kb // 4
    return tile * 512 + (m % 32) * 16 + ((m // 32) % 4) * 4 + kb % 4


@pytest.mark.parametrize("rows,kb", [(1, 1), (7, 3), (128, 4), (130, 9), (256, 8)])
def test_swizzle_matches_sm1xx_slot_formula_injective_and_invertible(rows, kb):
    lin = ((np.arange(rows * kb) % 251) + 1).astype(np.uint8).reshape(rows, kb)
    sw = ref.swizzle_scales(lin)
    assert sw.size == -(-rows // 128) * 128 * -(-kb // 4) * 4
    seen = np.zeros(sw.size, bool)
    for m in range(rows):
        for b in range(kb):
            d = ref_slot(m, b, kb)
            assert sw[d] == lin[m, b]
            assert not seen[d]
            seen[d] = True
    assert np.all(sw[~seen] == 0)
    assert np.array_equal(ref.unswizzle_scales(sw, rows, kb), lin)


def det_weight(out_f, in_f, seed):
    s = seed
    out = np.empty(out_f * in_f, np.float32)
    for i in range(out.size):
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        u = np.float32(np.float32((s >> 40) & 0xFFFFFFFF) / np.float32(1 << 24))
        out[i] = (u * np.float32(2.0) - np.float32(1.0)) * np.float32(0.35)
    return out.reshape(out_f, in_f)


def test_linear_swizzled_and_block_dequant_agree_bit_for_bit():
    w = det_weight(5, 32, 0xA11CE)
    g = ref.weight_global(w)
    mult = float(np.float32(1.0) / np.float32(g))
    packed, lin = ref.quantize_rows(w, g)
    a = ref.dequantize_packed_linear(packed, lin, 5, 32, mult)
    b = ref.dequantize_packed_swizzled(packed, ref.swizzle_scales(lin), 5, 32, mult)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    # tensor route: per-block dequant, then multiply by mult (Nvfp4Tensor::dequantize_scaled)
    # differs from the packed route only in where mult is applied; check values, not bits.
    c = np.stack([np.concatenate([ref.dequantize_block(packed[r, 8 * j:8 * j + 8], int(lin[r, j]))
                                  for j in range(2)]) for r in range(5)])
    np.testing.assert_allclose(c * np.float32(mult), a, rtol=2e-7)


def test_packed_dequant_roundtrip_relrms_in_nvfp4_band():
    w = det_weight(128, 256, 0xDECAF)
    g = ref.weight_global(w)
    packed, lin = ref.quantize_rows(w, g)
    deq = ref.dequantize_packed_linear(packed, lin, 128, 256, float(np.float32(1.0) / np.float32(g)))
    rr = np.sqrt(np.sum((deq.astype(np.float64) - w) ** 2) / np.sum(w.astype(np.float64) ** 2))
    assert 0.005 < rr < 0.15


def test_tensor_dequant_within_block_bound():
    rows = np.array([[((r * 37 + c * 13) % 11) - 5.0 for c in range(32)] for r in range(4)], np.float32)
    packed, lin = ref.quantize_rows(rows)
    deq = ref.dequantize_packed_linear(packed, lin, 4, 32)
    for r in range(4):
        for b in range(2):
            s = ref.decode_ue4m3(int(lin[r, b]))
            assert np.all(np.abs(rows[r, 16 * b:16 * b + 16] - deq[r, 16 * b:16 * b + 16]) <= s + 1e-6)


# ---- independent second route (bit fields instead of frexp / nearest search) ---------------
E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)


def enc_e2m1_midpoints(x, tie_up=False):
    x = np.float32(x)
    sign = 8 if np.signbit(x) else 0
    a = abs(x)
    idx = 0
    for i in range(7):
        mid = (E2M1[i] + E2M1[i + 1]) * np.float32(0.5)
        if (a >= mid) if tie_up else (a > mid):
            idx = i + 1
    return sign | idx


def enc_ue4m3_bits(scale, truncate=False):
    scale = np.float32(scale)
    if not np.isfinite(scale) or scale <= 0:
        return 0
    c = min(scale, np.float32(448.0))
    if c < np.float32(0.015625):
        q = np.float32(c / np.float32(0.001953125))
        m = int(np.floor(q + np.float32(0.5)))  # round half away from zero, positive input
        return 0 if m <= 0 else (m if m <= 7 else 8)
    bits = int(np.float32(c).view(np.uint32))
    e = ((bits >> 23) & 0xFF) - 127
    m23 = bits & 0x7FFFFF
    if truncate:
        m3 = m23 >> 20
    else:
        m3 = (m23 + (1 << 19)) >> 20
        if m3 >= 8:
            m3, e = 0, e + 1
    m3 = max(0, min(7, m3))
    be = max(1, min(15, e + 7))
    if be == 15 and m3 == 7:
        return 0x7E
    return (be << 3) | m3


def quantize_block_independent(v, g, bug=None):
    v = np.asarray(v, np.float32)
    amax = np.float32(np.max(np.abs(v)))
    stored = np.float32(1.0) if (g == 0 or not np.isfinite(g)) else np.float32(g)
    local = np.float32(1.0) if amax == 0 else np.float32(amax / np.float32(6.0))
    sb = enc_ue4m3_bits(np.float32(stored * local), truncate=(bug == "trunc"))
    dec = np.float32(ref.decode_ue4m3(sb))
    if bug == "inv":
        inv = np.float32(1.0) if stored * local == 0 else np.float32(stored / np.float32(stored * local))
    else:
        inv = np.float32(1.0) if dec == 0 else np.float32(stored / dec)
    out = []
    for i in range(8):
        lo = enc_e2m1_midpoints(np.clip(np.float32(v[2 * i] * inv), -6, 6), tie_up=(bug == "tie"))
        hi = enc_e2m1_midpoints(np.clip(np.float32(v[2 * i + 1] * inv), -6, 6), tie_up=(bug == "tie"))
        out.append(((lo << 4) | hi) if bug == "swap" else ((hi << 4) | lo))
    return np.array(out, np.uint8), sb


def fuzz_blocks(seed):
    state = seed | 1

    def nf():
        nonlocal state
        state = (state * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        return np.float32(np.float32(np.float64(state >> 32) / np.float64(0xFFFFFFFF)) * np.float32(2.0)
                          - np.float32(1.0))

    cases = []
    for mag in (1e-4, 3e-3, 0.02, 1.0, 37.0, 500.0):
        for _ in range(24):
            cases.append((np.array([nf() * np.float32(mag) for _ in range(16)], np.float32), 1.0))
    for g in (0.0, 0.0073, 1.0, 3.5, 448.0):
        for _ in range(12):
            cases.append((np.array([nf() for _ in range(16)], np.float32), g))
    cases.append((np.zeros(16, np.float32), 1.0))
    cases.append((np.full(16, -0.0, np.float32), 1.0))
    spikes = np.zeros(16, np.float32)
    spikes[7], spikes[8] = 6.0, -6.0
    cases.append((spikes, 1.0))
    for tie in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0):
        b = np.zeros(16, np.float32)
        b[0], b[1], b[15] = tie, -tie, 6.0
        cases.append((b, 1.0))
    return cases


def test_independent_bit_route_matches_oracle_byte_for_byte():
    checked = 0
    for seed in (1, 0x9E3779B9, 0xFEEDFACE):
        for block, g in fuzz_blocks(seed):
            pa, sa = ref.quantize_block(block, g)
            pb, sb = quantize_block_independent(block, g)
            assert sa == sb and np.array_equal(pa, pb), (block, g)
            checked += 1
    assert checked >= 450


@pytest.mark.parametrize("bug", ["trunc", "inv", "tie", "swap"])
def test_planted_bugs_are_caught(bug):
    caught = False
    for block, g in fuzz_blocks(0xABCDEF):
        good = quantize_block_independent(block, g)
        bad = quantize_block_independent(block, g, bug)
        if good[1] != bad[1] or not np.array_equal(good[0], bad[0]):
            caught = True
            break
    assert caught


def test_bf16_round_to_nearest_even():
    xs = np.array([1.0, 1.00390625, 1.0078125, 1.01171875, -3.1415927, 0.0, 65504.0, 1e-40], np.float32)
    got = ref.f32_to_bf16(xs)
    for x, g in zip(xs, got):
        assert int(g) == ref.lib().nvo_f32_to_bf16(float(x))
    assert ref.f32_to_bf16(np.array([1.00390625], np.float32))[0] == 0x3F80  # tie -> even
    assert ref.f32_to_bf16(np.array([1.01171875], np.float32))[0] == 0x3F82  # tie -> even (up)
    rng = np.random.default_rng(0)
    r = rng.standard_normal(4096).astype(np.float32)
    assert np.array_equal(ref.f32_to_bf16(r),
                          np.array([ref.lib().nvo_f32_to_bf16(float(v)) for v in r], np.uint16))


def test_cpu_backend_linear_matches_hand_dot_and_f64():
    # rust/crates/nv-layers/src/linear.rs:2612-2660: CPU bf16 linear vs hand f32 dot, rel < 1e-2
    rng = np.random.default_rng(3)
    n, k, m = 96, 256, 3
    w = ref.f32_to_bf16(rng.standard_normal((n, k)).astype(np.float32) * 0.02)
    x = ref.f32_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    y = ref.bf16_to_f32(ref.linear_cpu_backend(w, x))
    want = ref.bf16_to_f32(x).astype(np.float64) @ ref.bf16_to_f32(w).astype(np.float64).T
    rel = np.abs(y - want) / np.maximum(np.abs(want), 1e-3)
    assert rel.max() < 1e-2
    y1 = ref.linear_cpu_backend(w, x, threads=1)
    assert np.array_equal(y1, ref.linear_cpu_backend(w, x, threads=0))  # thread count does not change bits


def test_router_matches_closed_form_and_tie_breaks_low():
    rng = np.random.default_rng(1)
    lg = rng.standard_normal((5, 16)).astype(np.float32)
    lg[0, 3] = lg[0, 9] = 7.0  # tie at the top
    ids, w = ref.moe_route_topk(lg, 4)
    assert ids[0, 0] == 3 and ids[0, 1] == 9
    for t in range(5):
        order = np.argsort(-lg[t], kind="stable")[:4]
        assert list(ids[t]) == list(order)
        e = np.exp(lg[t, order] - lg[t, order].max())
        np.testing.assert_allclose(w[t], e / e.sum(), rtol=1e-5)
        assert abs(w[t].sum() - 1) < 1e-5


def test_cpu_linear_with_simd_summation_order():
    """The timed CPU baseline keeps 16 partial sums per output.  Its order is fixed (lane j takes
    k = j, j+16, ...; lanes added 8+8, 4+4, 2+2, 1+1; separate multiply and add), so it can be
    restated in numpy exactly, and it stays within bf16 rounding of the sequential statement."""
    rng = np.random.default_rng(12)
    n, k = 64, 4096 + 16 + 5   # a ragged tail after the last full group of 16
    w = ref.f32_to_bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    x = ref.f32_to_bf16(rng.standard_normal((2, k)).astype(np.float32))
    got = ref.linear_cpu_backend_lanes16(w, x)
    wf, xf = ref.bf16_to_f32(w), ref.bf16_to_f32(x)
    k16 = k // 16 * 16
    for m in range(2):
        for r in range(0, n, 7):
            acc = np.zeros(16, np.float32)
            for kk in range(0, k16, 16):
                acc += (wf[r, kk:kk + 16] * xf[m, kk:kk + 16]).astype(np.float32)
            for kk in range(k16, k):
                acc[kk & 15] += f32(wf[r, kk] * xf[m, kk])
            s = 8
            while s >= 1:
                acc[:s] += acc[s:2 * s]
                s //= 2
            assert ref.f32_to_bf16(acc[:1])[0] == got[m, r]
    seq = ref.bf16_to_f32(ref.linear_cpu_backend(w, x))
    lanes = ref.bf16_to_f32(got)
    rms = float(np.sqrt(np.mean(seq ** 2)))
    assert np.max(np.abs(seq - lanes) / np.maximum(np.abs(seq), max(rms, 1e-3))) < 1e-2
    assert np.array_equal(ref.linear_cpu_backend_lanes16(w, x, threads=1), got)   # thread count does not matter
