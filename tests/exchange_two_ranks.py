"""Run under torchrun with one rank per GPU (see test_exchange_gpu.py): every rank computes its rows
of two projections and must end up with all rows of both, identical to the unsharded product."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from ishizuki_b200 import synth  # noqa: E402
from ishizuki_b200.interface import GGMLType, GGUFBlocks, PackedLinear  # noqa: E402
from ishizuki_b200.sharding import OutputExchange, row_range, shard_ggml  # noqa: E402


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")  # the host side only passes handles around
    rng = np.random.default_rng(11)  # the same weights on every rank
    shapes = [(2000, 1024), (1024, 2048)]
    ex = OutputExchange(1 << 20)
    cases = []
    for n, k in shapes:
        blocks = synth.q4k_blocks(rng, n, k)
        lo, hi = row_range(n, rank, world)
        local = PackedLinear(ggml=GGUFBlocks(torch.from_numpy(shard_ggml(blocks, 12, n, k, rank, world)).cuda(), GGMLType.q4K,
                                            (hi - lo, k)))
        whole = PackedLinear(ggml=GGUFBlocks(torch.from_numpy(blocks).cuda(), GGMLType.q4K, (n, k)))
        x = torch.from_numpy(synth.activations(rng, 8, k)).cuda()
        off, view = ex.reserve(n)
        cases.append((local, whole, x, off, view, lo))
    for _ in range(5):
        for local, _, x, off, _, lo in cases:
            ex.apply(local, x, off, lo)
    ex.wait()
    torch.cuda.synchronize()
    cases[0][0].ctx.poll()
    for _, whole, x, _, view, _ in cases:
        # the shard's launch plan may add the partial sums in another order than the whole's
        want = whole(x, transposed=True).float()
        err = float((view.float() - want).abs().max() / want.abs().max())
        assert err < 1e-3, "rank %d: exchanged output differs by %g" % (rank, err)
    dist.barrier()
    print("exchange ok", flush=True)
    ex.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
