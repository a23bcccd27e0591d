"""N-sharding and the output all-gather, as two gloo ranks on CPU.

Each rank takes its row range of a seeded weight, computes its slab of y^T with the CPU oracle
(standing in for the GPU kernel, which this test is not about), gathers, and compares with the
unsharded oracle product.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ishizuki_b200 import sharding, synth
from oracle import oracle


def test_row_ranges_cover_and_balance():
    for n in (17, 128, 1024, 5120, 17408):
        for world in (1, 2, 3, 4, 8):
            ranges = [sharding.row_range(n, r, world) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [hi - lo for lo, hi in ranges]
            assert max(sizes) - min(sizes) <= 1


def test_ggml_shards_are_the_rows_bytes():
    rng = np.random.default_rng(0)
    n, k = 40, 512
    for type_id in (12, 14, 17):
        blocks = synth.ggml_blocks(rng, type_id, n, k)
        whole = oracle.dequantize(type_id, blocks).reshape(n, k)
        for world in (2, 3):
            for rank in range(world):
                lo, hi = sharding.row_range(n, rank, world)
                part = sharding.shard_ggml(blocks, type_id, n, k, rank, world)
                assert np.array_equal(oracle.dequantize(type_id, part).reshape(hi - lo, k), whole[lo:hi])


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, n: int, k: int, m: int, type_id: int, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)  # every rank draws the same full weight
        blocks = synth.ggml_blocks(rng, type_id, n, k)
        x = synth.activations(rng, m, k)
        lo, hi = sharding.row_range(n, rank, world)
        part = sharding.shard_ggml(blocks, type_id, n, k, rank, world)
        _, y_local = oracle.ggml_matmul(type_id, part, x, hi - lo)  # [m, n_local] fp16
        y_t = sharding.gather_rows(torch.from_numpy(np.ascontiguousarray(y_local.T)), n)
        _, want = oracle.ggml_matmul(type_id, blocks, x, n)
        ok = np.array_equal(y_t.numpy().T.view(np.uint16), want.view(np.uint16))
        with open(os.path.join(out_dir, f"rank{rank}"), "w") as f:
            f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n", [256, 131])  # even slabs, and uneven ones
def test_two_ranks_gather_the_whole_projection(tmp_path, n):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, n, 512, 5, 12, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}").read_text() == "ok"
