"""The multi-GPU path on CPU: two gloo ranks shard a batch, run the (oracle) operators on
their images, gather the output rows, and every rank ends with the unsharded result."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_bounds_cover_the_batch_once():
    from mace_b200.sharding import shard_bounds, shard_sizes
    for batch in (0, 1, 7, 64, 65):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(batch, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = shard_sizes(batch, world)
            assert sum(sizes) == batch and max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def _worker(rank, world, port, batch, out_path):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    from oracle import pyoracle as orc
    from mace_b200.sharding import shard_bounds, gather_rows
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.Generator(np.random.PCG64(5))  # every rank draws the same full batch
        x = rng.integers(0, 256, size=(batch, 6, 6, 8), dtype=np.uint8)
        f = rng.integers(1, 256, size=(12, 1, 1, 8), dtype=np.uint8)
        bias = np.rint(rng.normal(0, 300, size=12)).astype(np.int32)
        mult, shift = orc.output_multiplier_and_shift(np.float32(0.02), np.float32(0.01), np.float32(0.9))
        lo, hi = shard_bounds(batch, world, rank)
        mine = orc.conv2d_u8(x[lo:hi], f, bias, (1, 1), (0, 0), (6, 6), 128, 120, mult, shift, 100)
        full = gather_rows(dist, mine, batch)
        ref = orc.conv2d_u8(x, f, bias, (1, 1), (0, 0), (6, 6), 128, 120, mult, shift, 100)
        ok = full.shape == ref.shape and np.array_equal(full, ref)
        with open("%s.%d" % (out_path, rank), "w") as fh:
            fh.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("batch", [8, 5])  # even and ragged shards
def test_two_ranks_shard_and_gather(tmp_path, batch):
    import torch.multiprocessing as mp
    world = 2
    port = 29500 + (os.getpid() % 2000) + batch
    out = str(tmp_path / "result")
    mp.spawn(_worker, args=(world, port, batch, out), nprocs=world, join=True)
    for r in range(world):
        with open("%s.%d" % (out, r)) as fh:
            assert fh.read() == "ok"
