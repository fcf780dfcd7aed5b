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

pytestmark = [pytest.mark.gpu, pytest.mark.needs_cuda_runtime]   # the CUTLASS library runs on a GPU only


def run_gemm(ap, asw, bp, bsw, alpha, m, n, k, entry="nv_kernels_cutlass_fp4_gemm_sm120_bf16", tile=0, stream_k=0):
    d = [U.dev(a) for a in (ap, asw, bp, bsw)]
    al = torch.tensor([alpha], dtype=torch.float32, device="cuda")
    out = torch.full((m * n + 64,), 0x7FC0, dtype=torch.int16, device="cuda")
    need = ctypes.c_size_t(0)
    extra = [tile, stream_k] if entry.endswith("_tiled") else []
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
    U.ffi.call("nvk_b200_set_prefill_config", 1)


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
    if (m, n, k) == (256, 384, 512) and tile_config == 1:
        # the data-parallel form of the tiled symbol is the same kernel: same bits, whatever tile id
        for tile in (0, 1, 2):
            assert np.array_equal(run_gemm(ap, asw, bp, bsw, alpha, m, n, k,
                                           "nv_kernels_cutlass_fp4_gemm_sm120_bf16_tiled", tile, 0), got)


@pytest.mark.parametrize("m,n,k,stream_k", [(256, 384, 512, 1), (256, 256, 4096, 1), (256, 256, 4096, 4), (130, 264, 1056, 2),
                                            (2048, 640, 3200, 1)])
def test_stream_k_forms_match_the_oracle(m, n, k, stream_k):
    """Stream-K splits output tiles along K and reduces the parts through the workspace, so the
    summation order differs from the data-parallel kernel: same bound against the W4A4 oracle
    (2 bf16 ulp or 1e-3 absolute), bit-stable run to run."""
    U.require_gpu()
    rng = np.random.default_rng(m + n + k + stream_k)
    ap, alin, asw, _ = quantized_operand(rng, m, k, 1.0, 1.0)
    bp, blin, bsw, gb = quantized_operand(rng, n, k, 0.02)
    alpha = float(np.float32(1.0) / np.float32(gb))
    want = ref.matmul_w4a4(ap, alin, bp, blin, m, n, k, alpha)
    runs = [run_gemm(ap, asw, bp, bsw, alpha, m, n, k, "nv_kernels_cutlass_fp4_gemm_sm120_bf16_tiled", 1, stream_k)
            for _ in range(2)]
    if stream_k == 1:
        runs.append(run_gemm(ap, asw, bp, bsw, alpha, m, n, k, "nv_kernels_cutlass_fp4_gemm_sm120_bf16_streamk"))
    for got in runs:
        ulp = U.bf16_ulp_diff(got, want)
        absd = np.abs(ref.bf16_to_f32(got) - ref.bf16_to_f32(want))
        assert np.all((ulp <= 2) | (absd <= 1e-3)), f"max ulp {ulp.max()}"
    assert np.array_equal(runs[0], runs[1])
    need = ctypes.c_size_t(0)
    assert U.ffi.call("nv_kernels_cutlass_fp4_gemm_sm120_bf16_tiled", U.stream(), None, None, None, None, None, None, m, n, k,
                      3, 0, None, 0, ctypes.addressof(need)) == -3     # no such tile


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 384, 512), (384, 640, 1056)])
def test_library_route_matches_the_oracle_and_the_tensor_core_route(m, n, k):
    """The cuBLASLt route (the reference's `cublaslt` backend, nvfp4.rs:866-1067) against the W4A4 oracle
    with the bound of the other routes, and against this library's own GEMM within the 4 bf16 ulp the
    reference allows between its two backends (nv-quant/tests/nvfp4_default_routing_split.rs)."""
    U.require_gpu()
    rng = np.random.default_rng(3 * m + n + k)
    ap, alin, asw, _ = quantized_operand(rng, m, k, 1.0, 1.0)
    bp, blin, bsw, gb = quantized_operand(rng, n, k, 0.02)
    alpha = float(np.float32(1.0) / np.float32(gb))
    d = [U.dev(a) for a in (ap, asw, bp, bsw)]
    out = torch.full((m * n + 64,), 0x7FC0, dtype=torch.int16, device="cuda")
    ws = torch.zeros(U.ffi.prefill_lib().nvk_b200_cublaslt_fp4_workspace_bytes(), dtype=torch.uint8, device="cuda")
    for _ in range(2):   # the second call reuses the shape's plan
        rc = U.ffi.call("nvk_b200_cublaslt_fp4_gemm_bf16", U.stream(), d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(),
                        d[3].data_ptr(), out.data_ptr(), m, n, k, alpha, ws.data_ptr(), ws.numel())
        assert rc == 0, rc
    torch.cuda.synchronize()
    o = U.host_u16(out)
    assert np.all(o[m * n:] == 0x7FC0)
    got = o[:m * n].reshape(m, n)
    want = ref.matmul_w4a4(ap, alin, bp, blin, m, n, k, alpha)
    ulp = U.bf16_ulp_diff(got, want)
    absd = np.abs(ref.bf16_to_f32(got) - ref.bf16_to_f32(want))
    assert np.all((ulp <= 2) | (absd <= 1e-3)), f"max ulp {ulp.max()}"
    ours = run_gemm(ap, asw, bp, bsw, alpha, m, n, k)
    ulp2 = U.bf16_ulp_diff(got, ours)
    absd2 = np.abs(ref.bf16_to_f32(got) - ref.bf16_to_f32(ours))
    assert np.all((ulp2 <= 4) | (absd2 <= 1e-3)), f"max ulp between the routes {ulp2.max()}"


def test_runner_with_the_library_backend_pads_and_trims():
    """Nvfp4Linear with an Nvfp4GemmRunner whose backend is cublaslt: 200 rows are padded to 256, computed by
    the library route and trimmed; same bound against the linear's oracle as the default route."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    from speaches_plus_b200 import runner as R
    rng = np.random.default_rng(77)
    n, k, m = 256, 512, 200
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    x = U.gauss_bf16(rng, (m, k))
    lin = sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(sw), alpha, k, n)
    xt = U.dev(x).view(torch.bfloat16)
    base = lin(xt)
    lin.runner = R.Nvfp4GemmRunner(env={"SPEACHES_NVFP4_BACKEND": "cublaslt"})
    got = lin(xt)
    torch.cuda.synchronize()
    a = ref.bf16_to_f32(U.host_u16(got).reshape(m, n))
    b = ref.bf16_to_f32(U.host_u16(base).reshape(m, n))
    assert U.rel_err_floor(a, b.astype(np.float64)) < 1e-2


def test_staging_lifecycle_on_the_device():
    """rust/crates/nv-layers/tests/nvfp4_staging_lifecycle.rs: the linear's staging entry for the current
    stream tracks the live rows, a shrinking call resets the mark, releasing the stream's resources rebuilds
    the entry under a new epoch, and none of it changes the values."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    from speaches_plus_b200 import runner as R
    rng = np.random.default_rng(9)
    n, k = 128, 256
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    lin = sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(sw), alpha, k, n)
    key = R.stream_cache_key()
    y = torch.empty((200, n), dtype=torch.bfloat16, device="cuda")
    x200 = U.dev(U.gauss_bf16(rng, (200, k))).view(torch.bfloat16)
    x70 = x200[:70].contiguous()
    lin.forward_prefill_into(x200, y)
    assert lin.nvfp4_staging_diag(key, 256) == (R.stream_epoch(key), 200)
    lin.forward_prefill_into(x200[:130].contiguous(), y[:130])
    assert lin.nvfp4_staging_diag(key, 256)[1] == 130           # the shrink path ran and reset the mark
    lin.forward_prefill_into(x70, y[:70])
    a = U.host_u16(y[:70]).copy()
    assert lin.nvfp4_staging_diag(key, 128)[1] == 70
    epoch_before = lin.nvfp4_staging_diag(key, 128)[0]
    R.release_stream_resources(key)
    lin.forward_prefill_into(x70, y[:70])
    torch.cuda.synchronize()
    assert lin.nvfp4_staging_diag(key, 128)[0] > epoch_before   # rebuilt under the new epoch
    assert lin.nvfp4_staging_diag(key, 256) is None             # ... and the stale entry is gone
    assert np.array_equal(U.host_u16(y[:70]), a)                # eviction is value-preserving
    # rows left over from the 200-row call must not leak into a 130-row call's pad rows: same bits as fresh
    fresh = sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(sw), alpha, k, n)
    y2 = torch.empty((130, n), dtype=torch.bfloat16, device="cuda")
    lin.forward_prefill_into(x200, y)
    lin.forward_prefill_into(x200[:130].contiguous(), y[:130])
    fresh.forward_prefill_into(x200[:130].contiguous(), y2)
    torch.cuda.synchronize()
    assert np.array_equal(U.host_u16(y[:130]), U.host_u16(y2))


def test_true_m_equals_padded_m_bitwise():
    """rust/crates/nv-quant/tests/nvfp4_true_m.rs: a GEMM told the true row count gives the same bits
    for those rows as one told the 128-padded count (pad rows are zeros and are not part of the result)."""
    U.require_gpu()
    rng = np.random.default_rng(31)
    n, k = 384, 1024
    bp, blin, bsw, gb = quantized_operand(rng, n, k, 0.02)
    alpha = float(np.float32(1.0) / np.float32(gb))
    for m in (1, 64, 130, 200):
        m_pad = -(-m // 128) * 128
        x = U.gauss_bf16(rng, (m, k))
        ap, alin = ref.quantize_rows_bf16(x, 1.0, m_padded=m_pad)      # pad rows quantize to zeros
        asw = ref.swizzle_scales(alin)
        true_m = run_gemm(ap, asw, bp, bsw, alpha, m, n, k)
        padded = run_gemm(ap, asw, bp, bsw, alpha, m_pad, n, k)
        assert np.array_equal(true_m, padded[:m])
        assert np.all(padded[m:] == 0)


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


def _ulp_close(got, want):
    ulp = U.bf16_ulp_diff(got, want)
    absd = np.abs(ref.bf16_to_f32(got) - ref.bf16_to_f32(want))
    return bool(np.all((ulp <= 2) | (absd <= 1e-3)))


@pytest.mark.parametrize("entry", ["nv_kernels_cutlass_moe_grouped_fp4_gemm_sm120_bf16",
                                   "nv_kernels_cutlass_moe_grouped_fp4_gemm_sm120_bf16_decode"])
def test_grouped_block_scaled_gemm_matches_w4a4_oracle(entry):
    """Three groups with different row counts against a bank of five experts, picked through
    active_expert_indices: every group equals the single-problem W4A4 oracle on its own rows; rows of D
    outside the groups are left alone."""
    U.require_gpu()
    rng = np.random.default_rng(31)
    E, n, k = 5, 256, 512
    bank = [quantized_operand(rng, n, k, 0.02) for _ in range(E)]
    b_packed = np.stack([b[0] for b in bank])
    b_sw = np.stack([b[2] for b in bank])
    alphas = np.array([np.float32(1.0) / np.float32(b[3]) for b in bank], np.float32)
    active = np.array([3, 0, 4], np.int32)
    m_real = [128, 40, 97]                       # rows of each group; every group owns a 128-row slot
    slots = len(active)
    a_packed = np.zeros((slots * 128, k // 2), np.uint8)
    a_lin = np.zeros((slots * 128, k // 16), np.uint8)
    for g in range(slots):
        ap, alin, _, _ = quantized_operand(rng, 128, k, 1.0, 1.0)
        a_packed[g * 128:(g + 1) * 128], a_lin[g * 128:(g + 1) * 128] = ap, alin
    a_sw = ref.swizzle_scales(a_lin)             # 128-row tiles, one after the other
    offs = (np.arange(slots) * 128).astype(np.int32)
    sizes = np.array([[m, n, k] for m in m_real], np.int32).reshape(-1)
    d = [U.dev(t) for t in (a_packed, a_sw, b_packed, b_sw, alphas, offs, sizes, active)]
    out = torch.full((slots * 128 * n + 64,), 0x7FC0, dtype=torch.int16, device="cuda")
    meta = torch.zeros(128 * 1024, dtype=torch.uint8, device="cuda")
    need = ctypes.c_size_t(0)
    f = U.ffi.call
    assert f(entry, U.stream(), None, None, None, None, None, None, None, None, d[6].data_ptr(), None, n, k, slots,
             k, k, n, None, 0, None, 0, ctypes.addressof(need)) == 0       # workspace query
    ws = torch.zeros(max(need.value, 16), dtype=torch.uint8, device="cuda")
    rc = f(entry, U.stream(), d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(), d[4].data_ptr(),
           out.data_ptr(), d[5].data_ptr(), d[5].data_ptr(), d[6].data_ptr(), d[7].data_ptr(), n, k, slots, k, k, n,
           meta.data_ptr(), meta.numel(), ws.data_ptr(), ws.numel(), ctypes.addressof(need))
    assert rc == 0
    torch.cuda.synchronize()
    o = U.host_u16(out)
    assert np.all(o[slots * 128 * n:] == 0x7FC0)
    got = o[:slots * 128 * n].reshape(slots * 128, n)
    for g in range(slots):
        e, m = int(active[g]), m_real[g]
        r0 = g * 128
        want = ref.matmul_w4a4(a_packed[r0:r0 + m], a_lin[r0:r0 + m], bank[e][0], bank[e][1], m, n, k, float(alphas[e]))
        assert _ulp_close(got[r0:r0 + m], want), f"group {g}"
        assert np.all(got[r0 + m:r0 + 128] == 0x7FC0), f"group {g} wrote past its {m} rows"
    # refusals: meta scratch below the minimum, workspace too small, ragged K
    args = [d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(), d[4].data_ptr(), out.data_ptr(),
            d[5].data_ptr(), d[5].data_ptr(), d[6].data_ptr(), d[7].data_ptr()]
    assert f(entry, U.stream(), *args, n, k, slots, k, k, n, meta.data_ptr(), 1024, ws.data_ptr(), ws.numel(),
             ctypes.addressof(need)) == -10
    if need.value > 0:
        assert f(entry, U.stream(), *args, n, k, slots, k, k, n, meta.data_ptr(), meta.numel(), ws.data_ptr(), 0,
                 ctypes.addressof(need)) == -12
    assert f(entry, U.stream(), *args, n, 500, slots, k, k, n, meta.data_ptr(), meta.numel(), ws.data_ptr(), ws.numel(),
             ctypes.addressof(need)) == -1


def test_forward_grouped_matches_the_per_pair_w4a4_oracle():
    """The prefill-shaped MoE step (gather -> quantize -> grouped gate/up -> SiLU*up quantize -> grouped
    down -> combine) against the same chain restated with the oracle per (token, expert) pair."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(32)
    E, top_k, hidden, inter, n_tok = 8, 2, 256, 384, 24
    experts, host = [], []
    for e in range(E):
        trip, htrip = [], []
        for (n, k) in ((inter, hidden), (inter, hidden), (hidden, inter)):
            w = U.gauss_bf16(rng, (n, k), 0.05)
            packed, sw, alpha = ref.quantize_weight_bf16(w)
            trip.append(sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(sw), alpha, k, n))
            htrip.append((packed, ref.unswizzle_scales(sw, n, k // 16), alpha))
        experts.append(tuple(trip))
        host.append(htrip)
    w = sp.MoeGroupedWeights.build_from_experts(experts)
    x = U.gauss_bf16(rng, (n_tok, hidden))
    logits = rng.standard_normal((n_tok, E)).astype(np.float32)
    ids, wts = ref.moe_route_topk(logits, top_k)
    y = sp.forward_grouped(w, U.dev(x).view(torch.bfloat16), ids, U.dev(wts))
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    want = np.zeros((n_tok, hidden), np.float64)
    for t in range(n_tok):
        xp, xl = ref.quantize_rows_bf16(x[t:t + 1], 1.0)
        for j in range(top_k):
            (pg, lg, ag), (pu, lu, au), (pd, ld, ad) = host[ids[t, j]]
            gate = ref.matmul_w4a4(xp, xl, pg, lg, 1, inter, hidden, ag)
            up = ref.matmul_w4a4(xp, xl, pu, lu, 1, inter, hidden, au)
            act = ref.silu_mul(gate, up, round_bf16=False)             # f32, quantized without a bf16 rounding
            ap, al = ref.quantize_rows(act.reshape(1, inter), 1.0)
            down = ref.matmul_w4a4(ap, al, pd, ld, 1, hidden, inter, ad)
            want[t] += np.float64(wts[t, j]) * ref.bf16_to_f32(down)[0].astype(np.float64)
    # a gate/up value that lands one bf16 ulp away can move an activation code: the bound is the
    # linear path's, not bit equality
    assert U.rel_err_floor(got, want) < 2e-2


def test_forward_prenorm_nvfp4():
    """RMSNorm fused into the activation quantizer, then the FP4 x FP4 GEMM
    (rust/crates/nv-layers/src/linear.rs:653-689): equals norm -> bf16 -> quantize -> W4A4 oracle.  The
    device's rsqrt and sum order differ from the host's by an ulp, which can move a few 4-bit codes, so
    the bound is the linear path's relative one, not 2 ulp."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(41)
    m, n, k, eps = 70, 512, 1024, 1e-6
    w = U.gauss_bf16(rng, (n, k), 0.02)
    packed, sw, alpha = ref.quantize_weight_bf16(w)
    lin = sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(sw), alpha, k, n)
    x = U.gauss_bf16(rng, (m, k), 1.5)
    nw = U.gauss_bf16(rng, (k,), 1.0)
    y = lin.forward_prenorm_nvfp4(U.dev(x).view(torch.bfloat16), U.dev(nw).view(torch.bfloat16), eps)
    torch.cuda.synchronize()
    assert tuple(y.shape) == (m, n)
    xf, wf = ref.bf16_to_f32(x), ref.bf16_to_f32(nw)
    rstd = (1.0 / np.sqrt((xf.astype(np.float64) ** 2).mean(1) + eps)).astype(np.float32)
    normed = ref.f32_to_bf16((xf * rstd[:, None]) * wf[None, :])
    ap, alin = ref.quantize_rows_bf16(normed, 1.0)
    want = ref.matmul_w4a4(ap, alin, packed, ref.unswizzle_scales(sw, n, k // 16), m, n, k, alpha)
    assert U.rel_err_floor(y.float().cpu().numpy(), ref.bf16_to_f32(want).astype(np.float64)) < 2e-2
    # the same rows through the unfused pair (norm on the host, then the linear's own prefill route)
    y2 = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    lin.forward_prefill_into(U.dev(normed).view(torch.bfloat16), y2)
    torch.cuda.synchronize()
    assert U.rel_err_floor(y.float().cpu().numpy(), y2.float().cpu().numpy().astype(np.float64)) < 2e-2
    biased = sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(sw), alpha, k, n, bias=torch.zeros(n, device="cuda"))
    with pytest.raises(ValueError, match="not an eligible"):
        biased.forward_prenorm_nvfp4(U.dev(x).view(torch.bfloat16), U.dev(nw).view(torch.bfloat16), eps)
