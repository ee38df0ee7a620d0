"""Data-parallel plumbing around the library: how a mini-batch is split over ranks and how the weight
and bias gradients of all layers live in one contiguous arena that is all-reduced once per step.

The reference is single-GPU (cuda/cuda.cu:81 fixes device 0); what exists there is the reduction of
per-sample gradients over W (AddSumW, netlayer/cnetlayerconvolution.cu.h:507-508) and the batch_scale
argument of TrainingUpdateWeight (netlayer/inetlayer.cu.h:87).  Here every rank reduces its own shard
inside the weight-gradient kernel and the shards are summed with one all-reduce.
"""
import ctypes as C

import torch
import torch.distributed as dist

from .lib import load


def shard_bounds(batch, rank, world):
    """[begin, end) of the samples rank owns; shards differ by at most one sample."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad rank/world")
    base, rem = divmod(batch, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def slice_bounds(n, rank, world):
    """[begin, end) in floats of the part of an n-float arena that `rank` reduces and updates in the library's fused
    exchange (b200_comm_slice: 16-byte groups dealt out in equal runs, the last ranks may get less or nothing)."""
    b, e = C.c_size_t(0), C.c_size_t(0)
    r = load().b200_comm_slice(n, rank, world, C.byref(b), C.byref(e))
    if r:
        raise ValueError(load().b200_last_error().decode())
    return b.value, e.value


def arena_layout(shapes):
    """name -> (offset, count, shape) with every tensor starting on a 16-byte boundary, and the total float count."""
    offsets, total = {}, 0
    for name, shape in shapes.items():
        n = 1
        for d in shape:
            n *= d
        offsets[name] = (total, n, tuple(shape))
        total += (n + 3) // 4 * 4
    return offsets, total


class _DeviceSpan:
    """Lets torch view device memory that the library allocated (CUDA array interface, version 2)."""

    def __init__(self, ptr, floats):
        self.__cuda_array_interface__ = dict(shape=(floats,), typestr="<f4", data=(ptr, False), version=2)


class PeerBuffer:
    """A communicator of the library (b200_comm_*): device memory that every rank of the process group maps, so that the
    library's exchange kernels can read and write the peers' arenas over NVLink.  The handles travel through
    torch.distributed (all_gather of a byte tensor); torch does nothing else here."""

    def __init__(self, floats, strict=True):
        """Collective over the process group.  strict=False: a rank that cannot create or map the memory (no peer access
        between two devices, say) does not raise; every rank then ends with `failed` set to the reason and no buffer, so
        that the caller can fall back to NCCL on all ranks together."""
        lib = load()
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.floats = (floats + 63) // 64 * 64
        self.comm = C.c_void_p()
        self.failed = None
        self.buffer = None
        self.taken = 0
        from .ops import _check
        handle = (C.c_ubyte * 128)()
        error = None
        try:
            _check(lib.b200_comm_create(C.byref(self.comm), self.rank, self.world, self.floats * 4))
            _check(lib.b200_comm_handle(self.comm, handle))
        except Exception as e:      # every rank still takes part in the collectives below
            error = e
        mine = torch.tensor(list(handle), dtype=torch.uint8, device="cuda")
        everyone = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(everyone, mine)
        bad = torch.tensor([1 if error else 0], device="cuda")
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if not int(bad.item()):
            try:
                blob = bytes(torch.stack(everyone).cpu().numpy().tobytes())
                _check(lib.b200_comm_connect(self.comm, blob))
            except Exception as e:
                error = e
            bad = torch.tensor([1 if error else 0], device="cuda")
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()):
            self.failed = str(error) if error else "another rank could not create or map the peer memory"
            if self.comm:
                lib.b200_comm_destroy(self.comm)
                self.comm = C.c_void_p()
            if strict:
                raise RuntimeError("peer buffer: " + self.failed)
            return
        self._span = _DeviceSpan(lib.b200_comm_buffer(self.comm), self.floats)
        self.buffer = torch.as_tensor(self._span, device="cuda")
        dist.barrier()

    def self_test(self, floats=1 << 16):
        """Collective: sums small integers (exact in fp32 in any order) over the ranks with the library's exchange kernel and
        checks the result on every rank.  Returns None, or the reason it failed (the same verdict on every rank)."""
        lib = load()
        from .ops import _check, _stream, stream_status
        n = min(self.floats, floats) // 4 * 4
        error = None
        try:
            base = torch.arange(n, device="cuda", dtype=torch.float32) % 251
            self.buffer[:n] = base + self.rank
            dist.barrier()
            _check(lib.b200_allreduce(self.comm, 0, n, 0, _stream()))
            torch.cuda.synchronize()
            stream_status()
            want = base * self.world + self.world * (self.world - 1) // 2
            if not torch.equal(self.buffer[:n], want):
                error = "the sum over the ranks is wrong"
        except Exception as e:
            error = str(e)
        bad = torch.tensor([1 if error else 0], device="cuda")
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()):
            return error or "the self-test failed on another rank"
        return None

    def take(self, floats):
        """The next `floats` floats of the buffer (a multiple of 4, so every span starts on a 16-byte boundary) as
        (offset, tensor): several networks place their arenas in one buffer and share one exchange launch."""
        floats = (floats + 3) // 4 * 4
        if self.taken + floats > self.floats:
            raise ValueError("peer buffer exhausted: %d + %d > %d floats" % (self.taken, floats, self.floats))
        offset, self.taken = self.taken, self.taken + floats
        return offset, self.buffer[offset:offset + floats]

    def close(self):
        if self.comm:
            torch.cuda.synchronize()
            dist.barrier()
            self.buffer = None
            load().b200_comm_destroy(self.comm)
            self.comm = C.c_void_p()


class GradArena:
    """One contiguous fp32 buffer holding every layer's dW and dB; `views[name]` are the tensors the
    weight-gradient kernels write into directly (no staging copy before the collective).  `storage`: a float tensor of the
    arena's size to build the views on (a span of a PeerBuffer) instead of a fresh allocation."""

    def __init__(self, shapes, device, storage=None):
        self.offsets, total = arena_layout(shapes)
        if storage is None:
            self.buffer = torch.zeros(total, dtype=torch.float32, device=device)
        else:
            assert storage.numel() == total and storage.dtype == torch.float32
            self.buffer = storage
            self.buffer.zero_()
        self.views = {k: self.buffer[o:o + n].view(shape) for k, (o, n, shape) in self.offsets.items()}

    def all_reduce(self):
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(self.buffer, op=dist.ReduceOp.SUM)
        return self.buffer
