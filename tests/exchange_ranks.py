"""Run under torchrun with one rank per GPU (see test_exchange_gpu.py), any world size up to 8:
every rank computes its rows of a few projections; the outputs assembled by the NVLink exchange
(inside a CUDA graph replayed many times) and by the NCCL all-gather of the C ABI must be, bit for
bit, what each rank's shard gives when it is recomputed locally, and identical on all ranks."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from ishizuki_b200 import synth  # noqa: E402
from ishizuki_b200.interface import FusedLinear, GGMLType, GGUFBlocks, PackedLinear  # noqa: E402
from ishizuki_b200.sharding import NcclGroup, OutputExchange, row_range, shard_ggml  # noqa: E402

REPLAYS = int(os.environ.get("ISHI_EXCHANGE_REPLAYS", "200"))


def shard(blocks, n, k, q, world):
    lo, hi = row_range(n, q, world)
    return GGUFBlocks(torch.from_numpy(shard_ggml(blocks, 12, n, k, q, world)).cuda(), GGMLType.q4K, (hi - lo, k))


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")  # the host side only passes handles around
    rng = np.random.default_rng(11)  # the same weights on every rank
    # (rows of every matrix of the launch, k); rows divide by 8 ranks
    # a third entry marks gate / up as a gated pair: silu(gate) * up, sharded along its own rows
    launches = [((2048,), 1024), ((1024, 512, 512), 2048), ((4096, 4096), 1024), ((640,), 4352), ((1024, 1024), 2048, "gated")]
    ex = OutputExchange(4 << 20)
    cases = []
    for sizes, k, *kind in launches:
        mats = [synth.q4k_blocks(rng, n, k) for n in sizes]

        def build(q):
            parts = [shard(b, n, k, q, world) for b, n in zip(mats, sizes)]
            if kind:
                return FusedLinear(parts, gated=True)
            return FusedLinear(parts) if len(parts) > 1 else PackedLinear(ggml=parts[0])

        local = build(rank)
        x = torch.from_numpy(synth.activations(rng, 8, k)).cuda()
        n_local = local.outputDim
        off, view = ex.reserve(n_local * world)
        # what every rank's shard gives, computed here under the launch plan its owner measured
        # (the plan fixes the order of the partial sums, hence the bits)
        plans = [None] * world
        dist.all_gather_object(plans, local.plan)
        pieces = []
        for q in range(world):
            ref = build(q)
            ref.set_plan(plans[q])
            pieces.append(ref(x, transposed=True))
        want = torch.cat(pieces)
        cases.append((local, x, off, view, n_local, want))
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for local, x, off, _, n_local, _ in cases:
            ex.apply(local, x, off, rank * n_local)
        ex.wait()
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for local, x, off, _, n_local, _ in cases:
                ex.apply(local, x, off, rank * n_local)
            ex.wait()
        for it in range(REPLAYS):
            graph.replay()
            if it % 50 == 49 or it == REPLAYS - 1:
                torch.cuda.synchronize()
                for _, _, _, view, _, want in cases:
                    assert torch.equal(view, want), "rank %d: exchanged output differs at replay %d" % (rank, it)
    cases[0][0].ctx.poll()
    sums = torch.tensor([int(v.contiguous().view(torch.int16).to(torch.int64).sum().item()) for _, _, _, v, _, _ in cases])
    everyone = [torch.empty_like(sums) for _ in range(world)]
    dist.all_gather(everyone, sums)
    assert all(torch.equal(e, sums) for e in everyone), "the ranks hold different outputs"
    print("exchange ok (%d ranks, %d graph replays, bitwise)" % (world, REPLAYS), flush=True)

    group = NcclGroup()
    for local, x, _, _, n_local, want in cases:
        for rows in (8, 13):
            xr = x if rows == 8 else torch.cat([x, x[:5]])
            y_all = torch.zeros((n_local * world, rows), dtype=torch.float16, device="cuda")
            group.apply(local, xr, y_all)
            torch.cuda.synchronize()
            assert torch.equal(y_all[:, :8], want), "rank %d: all-gathered output differs" % rank
            if rows == 13:
                assert torch.equal(y_all[:, 8:], want[:, :5])
    dist.barrier()
    print("all-gather ok", flush=True)
    group.close()
    ex.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
