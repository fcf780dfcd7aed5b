"""Tensor-parallel host logic on CPU: two gloo ranks shard an NVFP4 linear column- and row-parallel,
run the local shards through the CPU oracle, complete them with the package's own collectives and
must reproduce the unsharded oracle (column: bit-exact; row: within the bf16 partial-sum rounding)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ref


class OracleLocal:
    """Stands in for the CUDA shard: same attributes, the contraction done by the CPU oracle."""

    def __init__(self, packed, scales, alpha, k, n):
        self.p, self.s, self.alpha = packed.numpy(), scales.numpy(), alpha
        self.in_features, self.out_features = k, n

    def forward_into(self, x, y, allow_prefill=True):
        assert not allow_prefill or dist.get_world_size() == 1   # sharded linears never ask for the prefill library
        xb = x.contiguous().view(torch.int16).numpy().view(np.uint16)
        out = ref.linear_w4a16_f64(self.p, self.s, xb, self.alpha, self.out_features, self.in_features)
        y.copy_(torch.from_numpy(ref.f32_to_bf16(out.astype(np.float32)).view(np.int16)).view(torch.bfloat16))


def _worker(rank, world, port, n, k, m, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import speaches_plus_b200 as sp
        from speaches_plus_b200 import tp
        rng = np.random.default_rng(0)
        w = ref.f32_to_bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        packed, sw, alpha = ref.quantize_weight_bf16(w)
        x = ref.f32_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
        xt = torch.from_numpy(x.view(np.int16)).view(torch.bfloat16)
        want = ref.linear_w4a16_f64(packed, sw, x, alpha, n, k)
        res = {}
        for mode in ("column", "row"):
            p, s, nl, kl, off = tp.shard_nvfp4(torch.from_numpy(packed), torch.from_numpy(sw), n, k, mode, rank, world)
            # the shard must be exactly the oracle's slice
            if mode == "column":
                lin = ref.unswizzle_scales(sw, n, k // 16)
                assert np.array_equal(p.numpy(), packed[off:off + nl])
                assert np.array_equal(ref.unswizzle_scales(s.numpy(), nl, k // 16), lin[off:off + nl])
            else:
                lin = ref.unswizzle_scales(sw, n, k // 16)
                assert np.array_equal(p.numpy(), packed[:, off // 2:(off + kl) // 2])
                assert np.array_equal(ref.unswizzle_scales(s.numpy(), n, kl // 16), lin[:, off // 16:(off + kl) // 16])
            t = tp.TpNvfp4Linear(OracleLocal(p, s, alpha, kl, nl), mode, rank, world, n, k, off)
            y = t.forward(xt).float().numpy()
            res[mode] = y
        if rank == 0:
            q.put((res, want))
    finally:
        assert tp.shutdown_process_group(join_s=60.0)   # the package's own orderly teardown


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("m", [1, 3])
def test_two_rank_column_and_row_parallel(m):
    n, k, world = 512, 1024, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, k, m, q)) for r in range(world)]
    for p in procs:
        p.start()
    res, want = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    col = res["column"]
    assert np.array_equal(ref.f32_to_bf16(col), ref.f32_to_bf16(want.astype(np.float32)))
    rms = float(np.sqrt(np.mean(want ** 2)))
    err = np.max(np.abs(res["row"] - want) / np.maximum(np.abs(want), max(rms, 1e-3)))
    assert err < 1e-2  # two bf16 partials + bf16 sum: well inside the 1e-2 bound


def test_shard_ranges_cover_everything():
    from speaches_plus_b200 import tp
    for n, world in [(10240, 8), (51200, 8), (4096, 4), (6144, 2), (28672, 8), (151936, 8), (384, 2)]:
        edges = [tp.column_shard_rows(n, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == n
        for a, b in zip(edges, edges[1:]):
            assert a[1] == b[0] and a[0] % 128 == 0
    for k, world in [(8192, 8), (25600, 8), (14336, 8), (14336, 4), (4096, 2)]:
        edges = [tp.row_shard_cols(k, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == k
        for a, b in zip(edges, edges[1:]):
            assert a[1] == b[0] and a[0] % 64 == 0


def test_fused_column_shard_keeps_pairs_together():
    """[gate; up] sharded per part: rank r holds gate rows [r0, r1) and the same up rows, and its
    scale tiles are those rows' tiles."""
    import numpy as np
    import torch

    from oracle import ref
    from speaches_plus_b200 import tp
    rng = np.random.default_rng(3)
    n_each, k, world = 512, 256, 4
    packed = rng.integers(0, 256, (2 * n_each, k // 2), dtype=np.uint8)
    lin = rng.integers(0, 0x7F, (2 * n_each, k // 16), dtype=np.uint8)
    sw = ref.swizzle_scales(lin)
    for rank in range(world):
        p, s, nl, r0 = tp.shard_nvfp4_fused(torch.from_numpy(packed), torch.from_numpy(sw), 2, n_each, k, rank, world)
        assert (nl, r0) == (128, 128 * rank)
        rows = np.r_[r0:r0 + nl, n_each + r0:n_each + r0 + nl]
        assert np.array_equal(p.numpy(), packed[rows])
        assert np.array_equal(s.numpy(), ref.swizzle_scales(lin[rows]))
    import pytest
    with pytest.raises(ValueError, match="multiple of 128"):
        tp.shard_nvfp4_fused(torch.from_numpy(packed), torch.from_numpy(sw), 2, 192, k, 0, 2)


def test_shard_from_disk_equals_shard_of_the_whole(tmp_path):
    """A rank's shard cut on the host from a checkpoint is the slice `shard_nvfp4` cuts from the whole
    matrix (checked on the host: the constructor itself needs a CUDA device only to run)."""
    import numpy as np
    import torch

    from oracle import ref
    from speaches_plus_b200 import tp, weights as W
    from tests.test_weights_ingest import ct_tensors, make_module, write_safetensors
    rng = np.random.default_rng(4)
    n, k = 512, 512
    packed, lin, g = make_module(rng, n, k)
    wl = W.WeightLoader.open_file(write_safetensors(tmp_path / "m.safetensors", ct_tensors("a", packed, lin, g, 2.0)))
    for mode in ("column", "row"):
        for rank in range(2):
            t = tp.TpNvfp4Linear.from_disk(wl, "a", n, k, mode, rank, 2, device=None)
            p, s, nl, kl, off = tp.shard_nvfp4(torch.from_numpy(packed), torch.from_numpy(ref.swizzle_scales(lin)), n, k,
                                               mode, rank, 2)
            assert torch.equal(t.local.weight_u8, p) and torch.equal(t.local.weight_scales, s)
            assert (t.local.out_features, t.local.in_features, t.offset) == (nl, kl, off)
            assert t.local.input_stored_global == 2.0
            assert abs(t.local.alpha_w4a16 * float(g) - 1) < 3e-7


def test_expert_shard_ranges():
    from speaches_plus_b200.moe import expert_shard_range
    assert [expert_shard_range(128, r, 8) for r in range(8)] == [(16 * r, 16 * r + 16) for r in range(8)]
    for E, world in [(128, 8), (60, 8), (7, 2), (3, 4)]:
        edges = [expert_shard_range(E, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == E
        assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
        sizes = [b - a for a, b in edges]
        assert max(sizes) - min(sizes) <= 1


def _ep_worker(rank, world, port, q):
    """Expert parallelism on the host: every rank routes all tokens, computes the slots of ITS experts
    (here through the oracle), leaves zeros elsewhere, combines, and the partial outputs are summed."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from speaches_plus_b200.moe import expert_shard_range
        rng = np.random.default_rng(11)
        E, top_k, hidden, inter, n_tok = 8, 2, 128, 256, 5
        host = []
        for e in range(E):
            trip = []
            for (n, k) in ((inter, hidden), (inter, hidden), (hidden, inter)):
                w = ref.f32_to_bf16((rng.standard_normal((n, k)) * 0.05).astype(np.float32))
                trip.append(ref.quantize_weight_bf16(w))
            host.append(trip)
        x = ref.f32_to_bf16(rng.standard_normal((n_tok, hidden)).astype(np.float32))
        logits = rng.standard_normal((n_tok, E)).astype(np.float32)
        ids, wts = ref.moe_route_topk(logits, top_k)
        e0, e1 = expert_shard_range(E, rank, world)

        def expert_out(e, t):
            (pg, sg, ag), (pu, su, au), (pd, sd, ad) = host[e]
            gate = ref.f32_to_bf16(ref.linear_w4a16_f64(pg, sg, x[t:t + 1], ag, inter, hidden).astype(np.float32))
            up = ref.f32_to_bf16(ref.linear_w4a16_f64(pu, su, x[t:t + 1], au, inter, hidden).astype(np.float32))
            act = ref.f32_to_bf16(ref.silu_mul(gate, up, round_bf16=True))
            return ref.f32_to_bf16(ref.linear_w4a16_f64(pd, sd, act, ad, hidden, inter).astype(np.float32))[0]

        # sorted-slot layout, as the permutation produces it; rows of other ranks' experts stay zero
        order = np.argsort(ids.reshape(-1), kind="stable")
        inv = np.empty_like(order)
        inv[order] = np.arange(order.size)
        down = np.zeros((n_tok * top_k, hidden), np.uint16)
        for slot in range(n_tok * top_k):
            e = int(ids.reshape(-1)[slot])
            if e0 <= e < e1:
                down[inv[slot]] = expert_out(e, slot // top_k)
        part = ref.moe_unpermute_scatter(down, wts, inv.reshape(n_tok, top_k).astype(np.int32), hidden, hidden)
        y = torch.from_numpy(part.copy())
        dist.all_reduce(y)
        if rank == 0:
            full = np.zeros_like(down)
            for slot in range(n_tok * top_k):
                full[inv[slot]] = expert_out(int(ids.reshape(-1)[slot]), slot // top_k)
            want = ref.moe_unpermute_scatter(full, wts, inv.reshape(n_tok, top_k).astype(np.int32), hidden, hidden)
            q.put((y.numpy(), want))
    finally:
        dist.destroy_process_group()


def test_two_rank_expert_parallel_sum_equals_the_whole():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got, want = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # each token's k products are the same numbers; only the order of the f32 additions differs
    assert np.allclose(got, want, rtol=1e-6, atol=1e-6 * float(np.abs(want).max()))


def test_prefill_routing_plan_equals_the_bucket_walk():
    """plan_routing against a direct restatement of the reference's plan
    (rust/crates/nv-layers/src/moe_grouped.rs:310-350): buckets filled in (token, slot) order, one
    128-row tile per expert that received tokens, overflow past 128 rows."""
    import numpy as np

    from speaches_plus_b200.moe import plan_routing
    rng = np.random.default_rng(0)
    for n, k, E in [(5, 2, 8), (64, 4, 16), (300, 2, 4), (1, 1, 3)]:
        ids = np.stack([rng.choice(E, k, replace=False) for _ in range(n)])
        p = plan_routing(ids, E)
        buckets = [[] for _ in range(E)]
        for t in range(n):
            for j in range(k):
                buckets[ids[t, j]].append((t, j))
        active = [e for e in range(E) if buckets[e]]
        src = np.full(len(active) * 128, -1, np.int32)
        inv = np.full(n * k, -1, np.int32)
        overflow = False
        for i, e in enumerate(active):
            for j, (t, slot) in enumerate(buckets[e]):
                if j >= 128:
                    overflow = True
                    break
                src[i * 128 + j] = t
                inv[t * k + slot] = i * 128 + j
        assert list(p["active_experts"]) == active and p["m_total_padded"] == 128 * len(active)
        assert list(p["real_m_per_active"]) == [len(buckets[e]) for e in active]
        assert np.array_equal(p["src_idx"], src) and np.array_equal(p["inv_perm"].reshape(-1), inv)
        assert p["overflow"] == overflow
    assert plan_routing(np.zeros((300, 1), np.int64), 2)["overflow"]


def _leaver_worker(rank, world, port, q):
    """Failure made on the host: rank 1 completes one step and leaves between steps; rank 0's next
    collective must end with an error within the process group's timeout, not hang."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from speaches_plus_b200 import tp
    n, k = 256, 512
    rng = np.random.default_rng(5)
    w = ref.f32_to_bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    packed, sw, alpha = ref.quantize_weight_bf16(w)
    x = torch.from_numpy(ref.f32_to_bf16(rng.standard_normal((1, k)).astype(np.float32)).view(np.int16)).view(torch.bfloat16)
    p, s, nl, kl, off = tp.shard_nvfp4(torch.from_numpy(packed), torch.from_numpy(sw), n, k, "row", rank, world)
    t = tp.TpNvfp4Linear(OracleLocal(p, s, alpha, kl, nl), "row", rank, world, n, k, off)
    t.forward(x)                      # step 1: both ranks take part
    if rank == 1:
        os._exit(0)                   # leaves between steps, nothing of its own in flight
    time.sleep(1.0)
    t0 = time.time()
    try:
        t.forward(x)                  # step 2: the peer is gone
        q.put(("no error", time.time() - t0))
    except Exception as e:           # noqa: BLE001 - any collective error is the expected outcome
        q.put((type(e).__name__, time.time() - t0))
    q.close()
    q.join_thread()                   # the result must reach the parent before this process goes away
    os._exit(0)                       # the group cannot be torn down in order: its peer is gone


def test_a_rank_that_leaves_between_steps_surfaces_as_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_leaver_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    kind, seconds = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
    assert kind != "no error", "the collective completed although the peer had left"
    assert seconds < 30, f"took {seconds:.1f} s to notice"


def _prefill_refusal_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import speaches_plus_b200 as sp
        from speaches_plus_b200 import tp
        ffi = sp.ffi
        seen = {"world": ffi.distributed_world(), "available": ffi.prefill_available()}
        for what, fn in (("load", ffi.prefill_lib),
                         ("config2", lambda: ffi.call("nvk_b200_set_prefill_config", 2)),
                         ("gemm", lambda: ffi.call("nv_kernels_cutlass_fp4_gemm_sm120_bf16", *([None] * 13)))):
            try:
                fn()
                seen[what] = "ran"
            except ffi.MultiGpuRefused:
                seen[what] = "refused"
        # a linear whose shapes would qualify for the tensor-core GEMM: 65 rows still stay on the decode kernels
        n, k = 256, 256
        lin = sp.Nvfp4Linear(torch.zeros(n * k // 2, dtype=torch.uint8), torch.zeros(n * k // 16, dtype=torch.uint8),
                             1.0, k, n)
        seen["route65"] = lin.route_for(65)
        seen["route2048"] = lin.route_for(2048)

        calls = []

        class Recorder(OracleLocal):
            def forward_into(self, x, y, allow_prefill=True):
                calls.append(allow_prefill)
                y.zero_()

        z = torch.zeros
        for mode in ("column", "row"):
            nl, kl = (n // world, k) if mode == "column" else (n, k // world)
            t = tp.TpNvfp4Linear(Recorder(z(1, dtype=torch.uint8), z(1, dtype=torch.uint8), 1.0, kl, nl), mode, rank,
                                 world, n, k, 0)
            t.forward(torch.zeros((65, k), dtype=torch.bfloat16))
        seen["tp_allow_prefill"] = calls
        if rank == 0:
            q.put(seen)
    finally:
        assert tp.shutdown_process_group(join_s=60.0)


def test_prefill_library_is_unreachable_from_a_rank_of_several():
    """The prefill library's 2-SM tile loads with TMA cluster multicast; no multi-GPU process may load
    it, select that tile, call its GEMM, or be routed to it by a linear, whatever M is."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_prefill_refusal_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    seen = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert seen == {"world": 2, "available": False, "load": "refused", "config2": "refused", "gemm": "refused",
                    "route65": "decode", "route2048": "decode", "tp_allow_prefill": [False, False]}


def test_single_process_still_routes_large_m_to_the_prefill_gemm():
    import speaches_plus_b200 as sp
    n, k = 256, 256
    lin = sp.Nvfp4Linear(torch.zeros(n * k // 2, dtype=torch.uint8), torch.zeros(n * k // 16, dtype=torch.uint8), 1.0,
                         k, n)
    assert sp.ffi.distributed_world() == 1
    assert [lin.route_for(m) for m in (1, 2, 64, 65)] == ["gemv", "decode", "decode", "prefill"]
    assert lin.route_for(65, allow_prefill=False) == "decode"


@pytest.mark.parametrize("world", [2, 4, 8])
def test_random_shards_reconstruct_the_whole_product(world):
    """shard_nvfp4 on random shapes, no process group needed: the column shards' oracle products are the
    column blocks of the whole product bit for bit (same rows, same K order), and the row shards'
    products -- each over its own K slice, scales re-laid for the slice -- add up to the whole in f64."""
    import numpy as np
    import torch
    from oracle import ref
    from speaches_plus_b200 import tp
    rng = np.random.default_rng(world)
    for _ in range(3):
        n = 128 * world * int(rng.integers(1, 4))
        k = 64 * world * int(rng.integers(1, 5))
        w = ref.f32_to_bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        packed, sw, alpha = ref.quantize_weight_bf16(w)
        x = ref.f32_to_bf16(rng.standard_normal((3, k)).astype(np.float32))
        whole = ref.linear_w4a16_f64(packed, sw, x, alpha, n, k)
        tp_, ts_ = torch.from_numpy(packed), torch.from_numpy(sw)
        cols, acc = [], np.zeros_like(whole)
        for r in range(world):
            p_c, s_c, n_l, k_l, _ = tp.shard_nvfp4(tp_, ts_, n, k, "column", r, world)
            assert (n_l, k_l) == (n // world, k)
            cols.append(ref.linear_w4a16_f64(p_c.numpy(), s_c.numpy(), x, alpha, n_l, k))
            p_r, s_r, n_l, k_l, off = tp.shard_nvfp4(tp_, ts_, n, k, "row", r, world)
            assert (n_l, k_l) == (n, k // world) and off == r * (k // world)
            acc += ref.linear_w4a16_f64(p_r.numpy(), s_r.numpy(), np.ascontiguousarray(x[:, off:off + k_l]), alpha, n, k_l)
        assert np.array_equal(np.concatenate(cols, axis=1), whole)
        assert np.allclose(acc, whole, rtol=1e-12, atol=1e-12)
