"""The fused row-parallel linear + all-reduce (nvk_b200_tp_linear_nvfp4_w4a16_allreduce) with every rank
running AT THE SAME TIME on the host emulation (each rank's launch is a group of host threads; on GPUs the
ranks are processes on different devices).  Every rank must end with the same bits, equal to its own
plain linear's bf16 partials summed in rank order in fp32 and rounded once -- the two-kernel form -- and
within the linear's bound of the f64 oracle of the whole (unsharded) product."""
import ctypes as C
import threading

import numpy as np
import pytest

from oracle import ref
from tests import _util as U
from tests.emu import harness as H

MAX_CTAS = 512
MAX_ROWS = 24


def _run_ranks(fn, world):
    # every host thread that runs blocks keeps a set of guard-paged fiber stacks (hundreds of mappings):
    # with several ranks at once, a few block-running threads per launch keep the process's map count low
    H.set_option("threads", max(1, 8 // world))
    out = [None] * world

    def go(r):
        out[r] = fn(r)

    th = [threading.Thread(target=go, args=(r,)) for r in range(world)]
    try:
        for t in th:
            t.start()
        for t in th:
            t.join(timeout=600)
            assert not t.is_alive()
    finally:
        H.set_option("threads", 0)
    return out


@pytest.mark.parametrize("world,m,n,k_rank,silu,resid", [(2, 1, 384, 512, False, False), (4, 3, 200, 1024, True, True),
                                                         (8, 8, 640, 256, False, True), (2, 5, 19200, 256, False, False),
                                                         (2, 13, 256, 512, False, True), (4, 24, 384, 256, True, False)])
def test_fused_linear_allreduce_equals_the_two_kernel_form(world, m, n, k_rank, silu, resid):
    rng = np.random.default_rng(world * 100 + m + n)
    nbytes = H.lib().nvk_b200_tp_fused_buffer_bytes(world, MAX_CTAS, MAX_ROWS)
    bufs = [H.Buf(np.zeros(nbytes, np.uint8)) for _ in range(world)]
    ptrs = (C.c_void_p * world)(*[b.ptr for b in bufs])
    epochs = [H.Buf(np.zeros(MAX_CTAS, np.uint32)) for _ in range(world)]
    errs = [H.Buf(np.zeros(1, np.int32)) for _ in range(world)]
    residual = U.gauss_bf16(rng, (m, n), 2.0) if resid else None
    for call in range(3):   # both inbox parities, flags never reset
        shards = [U.make_weight(rng, n, k_rank)[:3] for _ in range(world)]
        xs = [U.gauss_bf16(rng, (m, k_rank)) for _ in range(world)]
        ups = [U.gauss_bf16(rng, (m, k_rank)) for _ in range(world)] if silu else [None] * world
        dw = [(H.Buf(p), H.Buf(s)) for (p, s, _) in shards]
        dx = [H.Buf(x) for x in xs]
        du = [H.Buf(u) if u is not None else None for u in ups]
        dr = [H.Buf(residual) if resid else None for _ in range(world)]
        ys = [H.Buf(np.full((m, n), 0x7FC0, np.uint16)) for _ in range(world)]

        def fused(r):
            return H.call("nvk_b200_tp_linear_nvfp4_w4a16_allreduce", None, C.addressof(ptrs), r, world, dw[r][0], dw[r][1],
                          dx[r], du[r], dr[r], ys[r], float(shards[r][2]), m, n, k_rank, MAX_CTAS, MAX_ROWS, epochs[r], errs[r])

        assert _run_ranks(fused, world) == [0] * world
        # the two-kernel form: every rank's plain linear, then the fp32 sum in rank order, one rounding
        acc = np.zeros((m, n), np.float32)
        want64 = np.zeros((m, n), np.float64)
        for r in range(world):
            part = H.Buf(np.zeros((m, n), np.uint16))
            assert H.call("nvk_b200_linear_nvfp4_w4a16", None, dw[r][0], dw[r][1], None, None, dx[r], du[r], part, None,
                          float(shards[r][2]), 0.0, m, n, k_rank) == 0
            acc = acc + ref.bf16_to_f32(part.read())
            a = ref.f32_to_bf16(ref.silu_mul(xs[r], ups[r], round_bf16=True)) if silu else xs[r]
            want64 += ref.linear_w4a16_f64(shards[r][0], shards[r][1], a, shards[r][2], n, k_rank)
        if resid:
            acc = acc + ref.bf16_to_f32(residual)
            want64 += ref.bf16_to_f32(residual).astype(np.float64)
        want = ref.f32_to_bf16(acc)
        for r in range(world):
            assert int(errs[r].read()[0]) == 0
            assert np.array_equal(ys[r].read(), want), (call, r)
        assert U.rel_err_floor(ref.bf16_to_f32(want), want64) < 2e-2


def test_a_rank_that_never_arrives_is_reported_and_the_next_call_works():
    """One rank of two runs alone with a short wait limit: its wait on the absent peer runs out, the error
    word names the peer, the call returns normally; then both ranks run and agree."""
    world, m, n, k = 2, 2, 256, 256
    rng = np.random.default_rng(5)
    nbytes = H.lib().nvk_b200_tp_fused_buffer_bytes(world, MAX_CTAS, MAX_ROWS)
    bufs = [H.Buf(np.zeros(nbytes, np.uint8)) for _ in range(world)]
    ptrs = (C.c_void_p * world)(*[b.ptr for b in bufs])
    epochs = [H.Buf(np.zeros(MAX_CTAS, np.uint32)) for _ in range(world)]
    errs = [H.Buf(np.zeros(1, np.int32)) for _ in range(world)]
    shards = [U.make_weight(rng, n, k)[:3] for _ in range(world)]
    dw = [(H.Buf(p), H.Buf(s)) for (p, s, _) in shards]
    dx = [H.Buf(U.gauss_bf16(rng, (m, k))) for _ in range(world)]
    ys = [H.Buf(np.zeros((m, n), np.uint16)) for _ in range(world)]

    def fused(r):
        return H.call("nvk_b200_tp_linear_nvfp4_w4a16_allreduce", None, C.addressof(ptrs), r, world, dw[r][0], dw[r][1],
                      dx[r], None, None, ys[r], float(shards[r][2]), m, n, k, MAX_CTAS, MAX_ROWS, epochs[r], errs[r])

    assert H.call("nvk_b200_set_wait_limit", 2000) == 0
    try:
        assert fused(0) == 0                      # rank 1 is absent
    finally:
        H.call("nvk_b200_set_wait_limit", 0)
    assert int(errs[0].read()[0]) == 2            # 1 + the rank that never arrived
    errs[0].write(np.zeros(1, np.int32))
    # rank 1 now makes the call it missed (rank 0's partial and flag for it are already there) ...
    assert fused(1) == 0 and int(errs[1].read()[0]) == 0
    # ... and the next call, made by both, is complete on both
    assert _run_ranks(fused, world) == [0, 0]
    assert int(errs[0].read()[0]) == 0 and int(errs[1].read()[0]) == 0
    assert np.array_equal(ys[0].read(), ys[1].read())


@pytest.mark.parametrize("world,n_tok,top_k,hidden", [(2, 1, 4, 256), (4, 5, 2, 2048), (8, 3, 8, 1032)])
def test_expert_parallel_combine_sums_over_ranks_in_one_launch(world, n_tok, top_k, hidden):
    """nvk_b200_moe_combine_allreduce with all ranks at once: each rank holds the rows of the slots routed to
    its own experts (the other slots have inv_perm = -1 there); every rank ends with the same bits, equal to
    the ranks' own combines (nvk_b200_moe_combine) added in rank order in fp32."""
    rng = np.random.default_rng(world * 7 + n_tok)
    slots = n_tok * top_k
    nbytes = H.lib().nvk_b200_moe_combine_buffer_bytes(world, MAX_CTAS)
    bufs = [H.Buf(np.zeros(nbytes, np.uint8)) for _ in range(world)]
    ptrs = (C.c_void_p * world)(*[b.ptr for b in bufs])
    epochs = [H.Buf(np.zeros(MAX_CTAS, np.uint32)) for _ in range(world)]
    errs = [H.Buf(np.zeros(1, np.int32)) for _ in range(world)]
    for call in range(3):
        owner = rng.integers(0, world, size=slots)              # which rank's expert each slot went to
        weights = rng.random(slots).astype(np.float32)
        rows = U.gauss_bf16(rng, (slots, hidden))
        perm = rng.permutation(slots).astype(np.int32)          # slot -> row of the sorted buffer
        dw = H.Buf(weights)
        per_rank = []
        for r in range(world):
            inv = np.where(owner == r, perm, -1).astype(np.int32)
            sorted_rows = np.zeros((slots, hidden), np.uint16)
            sorted_rows[perm[owner == r]] = rows[owner == r]
            per_rank.append((H.Buf(sorted_rows), H.Buf(inv)))
        ys = [H.Buf(np.full((n_tok, hidden), np.nan, np.float32)) for _ in range(world)]
        status = [H.Buf(np.zeros(1, np.int32)) for _ in range(world)]

        def fused(r):
            return H.call("nvk_b200_moe_combine_allreduce", None, C.addressof(ptrs), r, world, per_rank[r][0], dw,
                          per_rank[r][1], ys[r], n_tok, top_k, hidden, hidden, slots, status[r], MAX_CTAS, epochs[r], errs[r])

        assert _run_ranks(fused, world) == [0] * world
        acc = np.zeros((n_tok, hidden), np.float32)
        for r in range(world):
            own = H.Buf(np.zeros((n_tok, hidden), np.float32))
            assert H.call("nvk_b200_moe_combine", None, per_rank[r][0], dw, per_rank[r][1], own, n_tok, top_k, hidden, hidden,
                          slots, None) == 0
            acc = acc + own.read()
        for r in range(world):
            assert int(errs[r].read()[0]) == 0 and int(status[r].read()[0]) == 0
            assert np.array_equal(ys[r].read(), acc), (call, r)
        # and it is the mixture: sum_s w_s * row_s per token
        want = (weights[:, None].astype(np.float64) * ref.bf16_to_f32(rows).astype(np.float64)).reshape(n_tok, top_k, hidden).sum(1)
        assert np.allclose(acc, want, rtol=1e-5, atol=1e-5)
