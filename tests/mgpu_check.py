"""Multi-GPU checks, run as `torchrun --nproc-per-node N tests/mgpu_check.py` (one rank per GPU):
the peer-memory all-reduce equals the fp32 rank-order sum bit for bit (eagerly and replayed from a
CUDA graph), and tensor-parallel NVFP4 linears (column and row) equal the unsharded linear."""
import os
import pathlib
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(pathlib.Path(__file__).resolve().parents[1]))
import speaches_plus_b200 as sp  # noqa: E402
from speaches_plus_b200 import tp  # noqa: E402


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

    # tensor-parallel linears against the unsharded one
    gen = torch.Generator(device=dev).manual_seed(7)
    for (n, k, mode) in ((1024, 2048, "column"), (512, 4096, "row")):
        w = (torch.randn((n, k), generator=gen, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        full = sp.Nvfp4Linear.from_bf16_quantized_nvfp4_dev(w)
        shard = tp.TpNvfp4Linear.from_bf16(w, mode, rank, world)
        shard.peer_ar = ar
        for m in (1, 5):
            x = torch.randn((m, k), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
            want = full(x).float()
            got = shard.forward(x).float()
            torch.cuda.synchronize()
            if mode == "column":
                assert torch.equal(got, want), f"column-parallel differs (rank {rank}, m={m})"
            else:
                rms = want.pow(2).mean().sqrt().item()
                err = ((got - want).abs() / torch.clamp(want.abs(), min=max(rms, 1e-3))).max().item()
                assert err < 1e-2, f"row-parallel error {err}"
    ar.check()

    # expert parallelism: the ranks' partial MoE outputs sum to the single-GPU result
    import numpy as np
    E, top_k, hidden, inter, n_tok = 16, 4, 256, 384, 7
    gen = torch.Generator(device=dev).manual_seed(9)
    experts = []
    for e in range(E):
        trip = []
        for (n, k) in ((inter, hidden), (inter, hidden), (hidden, inter)):
            w = (torch.randn((n, k), generator=gen, device=dev, dtype=torch.float32) * 0.05).to(torch.bfloat16)
            trip.append(sp.Nvfp4Linear.from_bf16_quantized_nvfp4_dev(w))
        experts.append(tuple(trip))
    whole = sp.MoeGroupedWeights.build_from_experts(experts)
    mine = whole.shard_experts(rank, world)
    ctx = sp.GroupedDecodeContext(whole, 8, top_k, dev)
    x = torch.randn((n_tok, hidden), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    logits = torch.randn((n_tok, E), generator=gen, device=dev, dtype=torch.float32)
    want = sp.forward_grouped_decode(whole, ctx, x, logits).clone()
    got = sp.forward_grouped_decode(mine, ctx, x, logits).clone()
    torch.cuda.synchronize()
    scale = float(want.abs().max().item())
    assert float((got - want).abs().max().item()) <= 1e-5 * scale, f"expert-parallel sum differs (rank {rank})"

    if rank == 0:
        print("mgpu_check ok", flush=True)
    ar.close()
    clean = tp.shutdown_process_group()
    sys.stdout.flush()
    if not clean:
        os._exit(0)


if __name__ == "__main__":
    main()
