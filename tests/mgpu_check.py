"""Multi-GPU checks, run as `torchrun --nproc-per-node N tests/mgpu_check.py` (one rank per GPU):
the peer-memory all-reduce equals the fp32 rank-order sum bit for bit (eagerly and replayed from a
CUDA graph); tensor-parallel NVFP4 linears (column and row, the row form also with its all-reduce
fused into the linear's launch) and the expert-parallel MoE step (also with the fused combine) are
checked against the CPU oracle (f64 statement of the contraction, the tolerance form of the GEMV
tests), not against the unsharded GPU result."""
import os
import pathlib
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(pathlib.Path(__file__).resolve().parents[1]))
import speaches_plus_b200 as sp  # noqa: E402
from oracle import ref  # noqa: E402
from speaches_plus_b200 import tp  # noqa: E402


def rel_err_floor(got, want, floor=1e-3):
    want = np.asarray(want, np.float64)
    rms = float(np.sqrt(np.mean(want ** 2)))
    return float(np.max(np.abs(np.asarray(got, np.float64) - want) / np.maximum(np.abs(want), max(rms, floor))))


def bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    tp.init_process_group_for_node(dev, timeout_s=60)
    ar = tp.PeerAllReduce(None, 64 * 5120, dev)

    def expected(parts):
        acc = torch.zeros_like(parts[0], dtype=torch.float32)
        for p in parts:
            acc += p.float()
        return acc.to(torch.bfloat16)

    for n in (8, 5120, 8192 + 64, 16 * 5120):
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        x = torch.randn(n, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        want = expected(parts)
        for rep in range(3):
            y = x.clone()
            ar.all_reduce_(y)
            torch.cuda.synchronize()
            assert torch.equal(y.view(torch.int16), want.view(torch.int16)), f"rank {rank} n={n} rep={rep}"
        # replayed from a graph: the call counter lives in device memory
        y = x.clone()
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            ar.all_reduce_(y)
            s.synchronize()
            y.copy_(x)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=s):
                ar.all_reduce_(y)
            for _ in range(3):
                y.copy_(x)
                graph.replay()
                s.synchronize()
                assert torch.equal(y.view(torch.int16), want.view(torch.int16)), f"graph rank {rank} n={n}"
        del graph
    ar.check()

    # tensor-parallel linears against the CPU oracle: weights quantized by the oracle on the host (the
    # same bytes on every rank), sharded, run on the GPUs, completed by the collectives
    rng = np.random.default_rng(7)
    for (n, k, mode) in ((1024, 2048, "column"), (512, 4096, "row")):
        w = ref.f32_to_bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        packed, sw, alpha = ref.quantize_weight_bf16(w)
        shard = tp.TpNvfp4Linear.from_parts(torch.from_numpy(packed), torch.from_numpy(sw), alpha, n, k, mode, rank, world,
                                            device=dev)
        shard.peer_ar = ar
        for m in (1, 5):
            x = ref.f32_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
            xt = torch.from_numpy(x.view(np.int16)).to(dev).view(torch.bfloat16)
            got = ref.bf16_to_f32(bits(shard.forward(xt))).reshape(m, n)
            torch.cuda.synchronize()
            want = ref.linear_w4a16_f64(packed, sw, x, alpha, n, k)
            err = rel_err_floor(got, want)
            # column: each output is one rank's full-K sum (fp32 accumulate + bf16 rounding);
            # row: bf16 partials summed in fp32 and rounded once more
            assert err < 1e-4 + 1e-2, f"{mode}-parallel vs the f64 oracle: {err} (rank {rank}, m={m})"
    ar.check()

    # the same row-parallel linear with the exchange inside its own launch: bit-equal to linear + all-reduce
    fused = tp.PeerFusedLinear(None, dev)
    n, k = 512, 4096
    w = ref.f32_to_bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    packed, sw, alpha = ref.quantize_weight_bf16(w)
    shard = tp.TpNvfp4Linear.from_parts(torch.from_numpy(packed), torch.from_numpy(sw), alpha, n, k, "row", rank, world,
                                        device=dev)
    shard.peer_ar = ar
    for m in (1, 5):
        x = ref.f32_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
        xt = torch.from_numpy(x.view(np.int16)).to(dev).view(torch.bfloat16)
        two_kernels = bits(shard.forward(xt)).copy()
        shard.peer_fused = fused
        one_kernel = bits(shard.forward(xt)).copy()
        shard.peer_fused = None
        torch.cuda.synchronize()
        assert np.array_equal(one_kernel, two_kernels), f"fused row-parallel linear differs (rank {rank}, m={m})"
        err = rel_err_floor(ref.bf16_to_f32(one_kernel).reshape(m, n), ref.linear_w4a16_f64(packed, sw, x, alpha, n, k))
        assert err < 1e-4 + 1e-2, f"fused row-parallel linear vs the f64 oracle: {err}"
    fused.check()
    fused.close()

    # expert parallelism against the per-(token, expert) oracle
    E, top_k, hidden, inter, n_tok = 16, 4, 256, 384, 7
    experts, host = [], []
    for e in range(E):
        trip, htrip = [], []
        for (n, k) in ((inter, hidden), (inter, hidden), (hidden, inter)):
            w = ref.f32_to_bf16((rng.standard_normal((n, k)) * 0.05).astype(np.float32))
            packed, sw, alpha = ref.quantize_weight_bf16(w)
            trip.append(sp.Nvfp4Linear.new_nvfp4(torch.from_numpy(packed).to(dev), torch.from_numpy(sw).to(dev), alpha, k, n))
            htrip.append((packed, sw, alpha))
        experts.append(tuple(trip))
        host.append(htrip)
    whole = sp.MoeGroupedWeights.build_from_experts(experts)
    mine = whole.shard_experts(rank, world)
    ctx = sp.GroupedDecodeContext(whole, 8, top_k, dev)
    x = ref.f32_to_bf16(rng.standard_normal((n_tok, hidden)).astype(np.float32))
    logits = rng.standard_normal((n_tok, E)).astype(np.float32)
    xt = torch.from_numpy(x.view(np.int16)).to(dev).view(torch.bfloat16)
    got = sp.forward_grouped_decode(mine, ctx, xt, torch.from_numpy(logits).to(dev)).cpu().numpy()
    torch.cuda.synchronize()
    ctx.check_status()
    ids, wts = ref.moe_route_topk(logits, top_k)
    want = np.zeros((n_tok, hidden), np.float64)
    for t in range(n_tok):
        for j in range(top_k):
            (pg, sg, ag), (pu, su, au), (pd, sd, ad) = host[ids[t, j]]
            gate = ref.f32_to_bf16(ref.linear_w4a16_f64(pg, sg, x[t:t + 1], ag, inter, hidden).astype(np.float32))
            up = ref.f32_to_bf16(ref.linear_w4a16_f64(pu, su, x[t:t + 1], au, inter, hidden).astype(np.float32))
            act = ref.f32_to_bf16(ref.silu_mul(gate, up, round_bf16=True))
            down = ref.f32_to_bf16(ref.linear_w4a16_f64(pd, sd, act, ad, hidden, inter).astype(np.float32))
            want[t] += np.float64(wts[t, j]) * ref.bf16_to_f32(down)[0].astype(np.float64)
    err = rel_err_floor(got, want)
    assert err < 1e-2, f"expert-parallel MoE step vs the per-pair oracle: {err} (rank {rank})"
    # ... and with the sum over the ranks inside the combine's own launch
    pc = tp.PeerMoeCombine(None, dev)
    got2 = sp.forward_grouped_decode(mine, ctx, xt, torch.from_numpy(logits).to(dev), peer_combine=pc).cpu().numpy()
    torch.cuda.synchronize()
    ctx.check_status()
    pc.check()
    assert rel_err_floor(got2, want) < 1e-2, f"fused expert-parallel combine vs the per-pair oracle (rank {rank})"
    pc.close()

    if rank == 0:
        print("mgpu_check ok", flush=True)
    ar.close()
    clean = tp.shutdown_process_group()
    sys.stdout.flush()
    if not clean:
        os._exit(0)


if __name__ == "__main__":
    main()
