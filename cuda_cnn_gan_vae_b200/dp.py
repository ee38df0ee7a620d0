"""Data-parallel plumbing around the library: how a mini-batch is split over ranks and how the weight
and bias gradients of all layers live in one contiguous arena that is all-reduced once per step.

The reference is single-GPU (cuda/cuda.cu:81 fixes device 0); what exists there is the reduction of
per-sample gradients over W (AddSumW, netlayer/cnetlayerconvolution.cu.h:507-508) and the batch_scale
argument of TrainingUpdateWeight (netlayer/inetlayer.cu.h:87).  Here every rank reduces its own shard
inside the weight-gradient kernel and the shards are summed with one all-reduce.
"""
import torch
import torch.distributed as dist


def shard_bounds(batch, rank, world):
    """[begin, end) of the samples rank owns; shards differ by at most one sample."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad rank/world")
    base, rem = divmod(batch, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


class GradArena:
    """One contiguous fp32 buffer holding every layer's dW and dB; `views[name]` are the tensors the
    weight-gradient kernels write into directly (no staging copy before the collective)."""

    def __init__(self, shapes, device):
        self.offsets, total = {}, 0
        for name, shape in shapes.items():
            n = 1
            for d in shape:
                n *= d
            self.offsets[name] = (total, n, tuple(shape))
            total += (n + 3) // 4 * 4            # keep every view 16-byte aligned
        self.buffer = torch.zeros(total, dtype=torch.float32, device=device)
        self.views = {k: self.buffer[o:o + n].view(shape) for k, (o, n, shape) in self.offsets.items()}

    def all_reduce(self):
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(self.buffer, op=dist.ReduceOp.SUM)
        return self.buffer
