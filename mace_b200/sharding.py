"""Data-parallel sharding of an inference batch over the GPUs of one box, one process per GPU.

Every operator on the path is independent across the batch dimension (Conv2D / depthwise /
pooling per image, FullyConnected per row, batched MatMul per batch entry), so the batch is
split into contiguous runs of images, one per rank, the weights are replicated, and the only
exchange is the final gather of the output rows.  `dist` is ``torch.distributed`` with the NCCL
backend on GPUs (gloo in the CPU tests).  Inside one process the C++ MultiGpuRunner
(mace_b200/host/multi_gpu.h) does the same with one host thread per GPU and no collective.

The reference has no counterpart: it runs one net on one device
(mace/core/net/serial_net.cc:103-124).
"""
import numpy as np


class PeerLost(RuntimeError):
    """A rank did not take part in the gather (it left, or the process group's timeout ran
    out).  The caller still holds its own rows; nothing of the collective's result is valid."""


def shard_bounds(batch, world, rank):
    """[begin, end) of the images rank `rank` of `world` processes: contiguous runs whose
    sizes differ by at most one (the first ``batch % world`` ranks get the extra image)."""
    if world < 1 or not (0 <= rank < world) or batch < 0:
        raise ValueError("bad shard request: batch=%d world=%d rank=%d" % (batch, world, rank))
    base, extra = divmod(batch, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_sizes(batch, world):
    return [shard_bounds(batch, world, r)[1] - shard_bounds(batch, world, r)[0] for r in range(world)]


class RowGather:
    """The final gather with everything allocated once: a send buffer of the largest shard's
    rows and a receive buffer of ``world`` such blocks, on `device`; every call is ONE
    ``all_gather_into_tensor``.  On a GPU nothing in `gather` waits for the host: the collective
    is ordered behind the work already enqueued on the current torch stream, and the caller
    copies the result out (or not) when it wants to."""

    def __init__(self, dist, batch, row_shape, dtype, device=None):
        import torch
        self.dist = dist
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.batch = batch
        self.sizes = shard_sizes(batch, self.world)
        self.width = max(self.sizes) if self.sizes else 0
        shape = (self.width,) + tuple(row_shape)
        self.send = torch.zeros(shape, dtype=dtype, device=device)
        self.recv = torch.zeros((self.world,) + shape, dtype=dtype, device=device)

    def gather(self, local_rows=None):
        """local_rows: this rank's [sizes[rank], ...] tensor, or None when the caller has already
        written its rows into ``self.send[:sizes[rank]]``.  Returns the [world, width, ...]
        receive buffer (rows past a shard's size are padding)."""
        n = self.sizes[self.rank]
        if local_rows is not None:
            if local_rows.shape[0] != n:
                raise ValueError("rank %d holds %d rows, its shard has %d" % (self.rank, local_rows.shape[0], n))
            self.send[:n].copy_(local_rows, non_blocking=True)
        try:
            self.dist.all_gather_into_tensor(self.recv.view((-1,) + tuple(self.send.shape[1:])), self.send)
        except RuntimeError as e:  # a peer closed its connection, or the group's timeout ran out
            raise PeerLost("gather of the output rows failed on rank %d: %s" % (self.rank, str(e)[:200])) from e
        return self.recv

    def assemble(self, recv=None):
        """The [batch, ...] result in image order from a receive buffer (a host-side helper)."""
        recv = self.recv if recv is None else recv
        parts = [recv[r, :n] for r, n in enumerate(self.sizes)]
        import torch
        return torch.cat(parts, dim=0)


def gather_rows(dist, local_rows, batch, device=None):
    """All ranks receive the [batch, ...] output assembled from every rank's rows (rank order =
    image order); shards may be ragged.  `local_rows` is a numpy array; returns numpy.  A
    convenience for tests and one-off calls: it allocates and waits; a serving loop keeps one
    RowGather."""
    import torch
    g = RowGather(dist, batch, local_rows.shape[1:], torch.from_numpy(local_rows[:0]).dtype, device)
    mine = torch.from_numpy(np.ascontiguousarray(local_rows))
    if device is not None:
        mine = mine.to(device)
    g.gather(mine)
    return g.assemble().cpu().numpy()


class _DeviceView:
    """A device allocation owned by someone else, presented through the CUDA array interface."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 2}


def torch_view(ptr, shape, typestr="|u1"):
    """A torch tensor over `ptr` (no copy, no ownership): typestr as in numpy ('|u1', '<f4')."""
    import torch
    return torch.as_tensor(_DeviceView(ptr, shape, typestr), device="cuda")


class AsyncRowGather:
    """The final gather of a serving loop on GPUs, kept off the critical path.  Per step the
    engine's stream only copies this rank's output rows (kilobytes) into a send buffer; the
    collective, and on rank 0 the copy of the gathered rows to pinned host memory, run on a side
    stream, so the next step's kernels do not wait for them.  Two buffer sets alternate; a set is
    reused only after the side stream has finished with it (an event wait on the device, no host
    wait anywhere).

    engine_stream: the cudaStream_t (integer) the network runs on; rows: a torch view of the
    engine's output tensor, [rows of this rank, ...]."""

    def __init__(self, dist, batch, rows, engine_stream, to_host_on_rank0=True):
        import torch
        self.torch = torch
        self.rows = rows
        self.stream = torch.cuda.ExternalStream(int(engine_stream))
        self.side = torch.cuda.Stream()
        self.sets = [RowGather(dist, batch, rows.shape[1:], rows.dtype, rows.device) for _ in range(2)]
        self.ready = [torch.cuda.Event() for _ in range(2)]   # send buffer filled (engine stream)
        self.done = [torch.cuda.Event() for _ in range(2)]    # collective (+ host copy) finished (side stream)
        self.used = [False, False]
        self.step = 0
        self.host = None
        if to_host_on_rank0 and dist.get_rank() == 0:
            self.host = [torch.empty(tuple(g.recv.shape), dtype=rows.dtype).pin_memory() for g in self.sets]

    def enqueue(self):
        """Call right after the step's kernels have been enqueued on the engine's stream."""
        k = self.step & 1
        g = self.sets[k]
        n = g.sizes[g.rank]
        with self.torch.cuda.stream(self.stream):
            if self.used[k]:
                self.stream.wait_event(self.done[k])
            g.send[:n].copy_(self.rows[:n], non_blocking=True)
            self.ready[k].record(self.stream)
        with self.torch.cuda.stream(self.side):
            self.side.wait_event(self.ready[k])
            g.gather()
            if self.host is not None:
                self.host[k].copy_(g.recv, non_blocking=True)
            self.done[k].record(self.side)
        self.used[k] = True
        self.step += 1
        return k

    def wait(self):
        """Host wait for everything enqueued so far; returns rank 0's last gathered rows in image
        order (None on the other ranks)."""
        self.side.synchronize()
        if self.host is None or self.step == 0:
            return None
        k = (self.step - 1) & 1
        return self.sets[k].assemble(self.host[k])
