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


def _lossy_worker(rank, world, port, mode, out_path):
    """Rank 1 takes part in the first gather and then drops out before the second one: it exits
    (mode "exit") or simply never calls the collective (mode "stall").  Rank 0 must come back
    from its second gather with PeerLost -- by the closed connection or by the process group's
    short timeout -- instead of waiting forever, and still hold its own rows."""
    sys.path.insert(0, ROOT)
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch
    import torch.distributed as dist
    from mace_b200.sharding import PeerLost, RowGather
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    g = RowGather(dist, 6, (5,), torch.uint8)
    mine = torch.full((3, 5), rank + 1, dtype=torch.uint8)
    g.gather(mine)
    first_ok = g.assemble()[:, 0].tolist() == [1, 1, 1, 2, 2, 2]
    if rank == 1:
        if mode == "stall":
            time.sleep(8)
        os._exit(0)
    t0 = time.time()
    verdict = "no error"
    try:
        g.gather(mine)
    except PeerLost as e:
        verdict = "peer lost" if "rank 0" in str(e) else "wrong message"
    waited = time.time() - t0
    own_rows_intact = bool((g.send[:3] == 1).all())
    with open(out_path, "w") as fh:
        fh.write("%s %s %s %.1f" % (first_ok, verdict, own_rows_intact, waited))
    os._exit(0)


@pytest.mark.parametrize("mode", ["exit", "stall"])
def test_a_rank_that_leaves_before_the_gather_is_noticed(tmp_path, mode):
    import torch.multiprocessing as mp
    port = 31500 + (os.getpid() % 2000) + (7 if mode == "stall" else 0)
    out = str(tmp_path / "verdict")
    mp.spawn(_lossy_worker, args=(2, port, mode, out), nprocs=2, join=True)
    first_ok, verdict, verdict2, own, waited = open(out).read().split()
    assert first_ok == "True"
    assert (verdict, verdict2) == ("peer", "lost")
    assert own == "True"
    assert float(waited) < 30.0
