"""Weight-stream traffic of the launches, counted on the host emulation: every global range a block fetches
with cp.async or a streaming load is recorded as 32-byte sectors once per block, and the sum over the
blocks of a launch must equal the algorithmic bytes -- packed weights + block scales (or the bf16 matrix)
crossing to the SMs exactly once, whatever the launch geometry (cluster split of K, dealt units, two arms,
grouped experts with the active list, the fused collective's epilogue).  Activations are not part of
the count.  On a GPU the same statement is the profiler's dram__bytes figure; these tests exist where
no profiler does and are skipped on a real device."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import ref
from tests import _util as U
from tests.test_gpu_linear import run_linear, run_normed, run_residual

pytestmark = pytest.mark.gpu


def _counting():
    if not getattr(U.ffi, "EMULATED", False):
        pytest.skip("byte accounting exists on the host emulation only (on a GPU: the profiler's DRAM counters)")
    L = U.ffi.lib()
    L.emu_fetched_bytes.restype = C.c_ulonglong
    L.emu_fetch_accounting.argtypes = [C.c_int]
    L.emu_fetch_accounting.restype = None
    return L


class counted:
    def __enter__(self):
        self.L = _counting()
        self.L.emu_fetch_accounting(1)
        return self

    def __exit__(self, *a):
        self.bytes = int(self.L.emu_fetched_bytes())
        self.L.emu_fetch_accounting(0)


def nvfp4_bytes(n, k):
    return n * k // 2 + n * k // 16        # N % 128 == 0 and K % 64 == 0 in every case below


@pytest.mark.parametrize("m,n,k,what", [(1, 1024, 1024, "cluster split of K"), (1, 640, 512, "dealt units"),
                                        (5, 256, 2048, "several rows"), (1, 2304, 256, "one tile per CTA"),
                                        (2, 512, 768, "two arms")])
def test_dense_launches_fetch_every_weight_byte_once(m, n, k, what):
    U.require_gpu()
    rng = np.random.default_rng(n + k)
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    x = U.gauss_bf16(rng, (m, k))
    if what == "two arms":
        pb, sb, ab, _ = U.make_weight(rng, n, k)
        with counted() as c:
            run_linear(packed, sw, x, alpha, m, n, k, pb, sb, ab)
        assert c.bytes == 2 * nvfp4_bytes(n, k)
        return
    if what == "dealt units":
        assert U.ffi.call("nvk_b200_set_row_balance", 1) == 0
    try:
        with counted() as c:
            run_linear(packed, sw, x, alpha, m, n, k)
    finally:
        U.ffi.call("nvk_b200_set_row_balance", 0)
    if what == "dealt units":
        # the two units that share a scale tile's 32-byte sectors (rows g and g + 64) now sit in different
        # CTAs: every scale sector is asked for by two blocks (L2 traffic; DRAM still sees it once),
        # every weight byte by one
        assert c.bytes == nvfp4_bytes(n, k) + n * k // 16, what
    else:
        assert c.bytes == nvfp4_bytes(n, k), what
    resid = U.gauss_bf16(rng, (m, n))
    with counted() as c:
        run_residual(packed, sw, x, resid, alpha, m, n, k)
    assert c.bytes == nvfp4_bytes(n, k)
    nw = U.gauss_bf16(rng, (k,), 1.0)
    with counted() as c:
        run_normed((packed, sw, alpha), x, nw, 1e-6, m, n, k)
    assert c.bytes == nvfp4_bytes(n, k)


def test_bf16_linear_streams_the_matrix_once_for_all_rows():
    U.require_gpu()
    rng = np.random.default_rng(3)
    n, k = 19008, 256
    w, = [U.gauss_bf16(rng, (n, k), 0.05)]
    dw = U.dev(w)
    for m in (1, 16, 64):
        x = U.dev(U.gauss_bf16(rng, (m, k)))
        y = torch.zeros(m * n, dtype=torch.int16, device="cuda")
        entry = "nv_kernels_gemv_bf16" if m == 1 else "nvk_b200_linear_bf16"
        with counted() as c:
            if m == 1:
                assert U.ffi.call(entry, U.stream(), dw.data_ptr(), x.data_ptr(), y.data_ptr(), n, k) == 0
            else:
                assert U.ffi.call(entry, U.stream(), dw.data_ptr(), x.data_ptr(), y.data_ptr(), m, n, k) == 0
            torch.cuda.synchronize()
        assert c.bytes == 2 * n * k, m


def test_grouped_decode_step_fetches_each_routed_expert_once():
    """One MoE decode step, 3 tokens x top-2 of 8 experts: gate, up and down of every expert that received
    a slot cross exactly once (experts without tokens cost nothing), K split over a cluster included."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(12)
    E, top_k, hidden, inter, n_tok = 8, 2, 1024, 512, 3
    experts = []
    for e in range(E):
        trip = []
        for (n, k) in ((inter, hidden), (inter, hidden), (hidden, inter)):
            p_, s_, a_, _ = U.make_weight(rng, n, k, 0.05)
            trip.append(sp.Nvfp4Linear.new_nvfp4(U.dev(p_), U.dev(s_), a_, k, n))
        experts.append(tuple(trip))
    w = sp.MoeGroupedWeights.build_from_experts(experts)
    ctx = sp.GroupedDecodeContext(w, 4, top_k, "cuda")
    x = U.dev(U.gauss_bf16(rng, (n_tok, hidden))).view(torch.bfloat16)
    logits = rng.standard_normal((n_tok, E)).astype(np.float32)
    with counted() as c:
        sp.forward_grouped_decode(w, ctx, x, U.dev(logits))
        torch.cuda.synchronize()
    ctx.check_status()
    ids, _ = ref.moe_route_topk(logits, top_k)
    distinct = len(np.unique(ids))
    assert c.bytes == distinct * (2 * nvfp4_bytes(inter, hidden) + nvfp4_bytes(hidden, inter))


def test_fused_collective_epilogue_adds_no_weight_traffic():
    U.require_gpu()
    rng = np.random.default_rng(21)
    m, n, k, max_ctas = 2, 512, 1024, 64
    packed, sw, alpha, _ = U.make_weight(rng, n, k)
    d = [U.dev(packed), U.dev(sw), U.dev(U.gauss_bf16(rng, (m, k)))]
    nbytes = U.ffi.lib().nvk_b200_tp_fused_buffer_bytes(1, max_ctas, 8)
    buf = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    one = (C.c_void_p * 1)(buf.data_ptr())
    epoch = torch.zeros(max_ctas, dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = torch.zeros(m * n, dtype=torch.int16, device="cuda")
    with counted() as c:
        assert U.ffi.call("nvk_b200_tp_linear_nvfp4_w4a16_allreduce", U.stream(), C.addressof(one), 0, 1, d[0].data_ptr(),
                          d[1].data_ptr(), d[2].data_ptr(), None, None, y.data_ptr(), float(alpha), m, n, k, max_ctas, 8,
                          epoch.data_ptr(), err.data_ptr()) == 0
        torch.cuda.synchronize()
    assert c.bytes == nvfp4_bytes(n, k) and int(err.cpu().numpy()[0]) == 0


def test_w4a8_and_fp4_gemv_fetch_every_weight_byte_once():
    U.require_gpu()
    from tests.test_gpu_w4a8 import w4a8
    rng = np.random.default_rng(8)
    n, k, m = 384, 1024, 6
    wa, wb = U.make_weight(rng, n, k)[:3], U.make_weight(rng, n, k)[:3]
    q, sc = ref.rowquant_i8((rng.standard_normal((m, k)) * 1.5).astype(np.float32))
    with counted() as c:
        w4a8("nv_kernels_gemv_nvfp4_w4a8_dual_mk", wa, q, sc, m, n, k, second=wb)
    assert c.bytes == 2 * nvfp4_bytes(n, k)
    with counted() as c:
        w4a8("nv_kernels_gemv_nvfp4_w4a8_down_residual_mk", wa, q, sc, m, n, k, residual=U.gauss_bf16(rng, (m, n)))
    assert c.bytes == nvfp4_bytes(n, k)
    # the M = 1 FP4 x FP4 GEMV: weights once; the activation row's 4-bit codes are not part of this count
    x = U.dev(U.gauss_bf16(rng, (1, k)))
    xp = torch.zeros(k // 2, dtype=torch.uint8, device="cuda")
    xs = torch.zeros(k // 16, dtype=torch.uint8, device="cuda")
    assert U.ffi.call("nv_kernels_nvfp4_quantize_row_bf16", U.stream(), x.data_ptr(), xp.data_ptr(), xs.data_ptr(), 1.0, k) == 0
    y = torch.zeros(n, dtype=torch.int16, device="cuda")
    dw, ds = U.dev(wa[0]), U.dev(wa[1])
    with counted() as c:
        assert U.ffi.call("nv_kernels_nvfp4_gemv_bf16", U.stream(), dw.data_ptr(), ds.data_ptr(), xp.data_ptr(), xs.data_ptr(),
                          y.data_ptr(), float(wa[2]), n, k) == 0
        torch.cuda.synchronize()
    assert c.bytes == nvfp4_bytes(n, k)


@pytest.mark.parametrize("rows", [16, 128])
def test_persistent_step_fetches_every_weight_byte_once(rows):
    """A two-layer SwiGLU step as ONE persistent launch: the work items (128-row or 16-row slabs drawn from
    per-operation counters) partition every matrix, so each weight byte still crosses once; with 16-row
    items the two units of a scale-sector pair can sit in different CTAs, which asks for scale sectors up
    to twice (an upper bound here: items are drawn dynamically)."""
    U.require_gpu()
    import speaches_plus_b200 as sp
    rng = np.random.default_rng(33)
    m, hidden, inter = 2, 512, 1024

    def make(n, k):
        packed, sw, alpha, _ = U.make_weight(rng, n, k, 0.05)
        return sp.Nvfp4Linear.new_nvfp4(U.dev(packed), U.dev(sw), alpha, k, n)

    layers = [(make(inter, hidden), make(inter, hidden), make(hidden, inter)) for _ in range(2)]
    bf = dict(dtype=torch.bfloat16, device="cuda")
    x = U.dev(U.gauss_bf16(rng, (m, hidden))).view(torch.bfloat16)
    step = sp.DecodeStep(m, "cuda")
    dep = -1
    for (g, u, d) in layers:
        yg, yu, yd = torch.zeros((m, inter), **bf), torch.zeros((m, inter), **bf), torch.zeros((m, hidden), **bf)
        gu = step.add(g, x, yg, lin_b=u, y_b=yu, dep=dep, rows_per_item=rows)
        dep = step.add(d, yg, yd, x2=yu, dep=gu, rows_per_item=rows)
        x = yd
    step.build()
    with counted() as c:
        step.run()
        torch.cuda.synchronize()
    step.check()
    weights = 2 * (2 * inter * hidden // 2 + hidden * inter // 2)
    scales = 2 * (2 * inter * hidden // 16 + hidden * inter // 16)
    if rows == 128:
        assert c.bytes == weights + scales
    else:
        assert weights + scales <= c.bytes <= weights + 2 * scales
