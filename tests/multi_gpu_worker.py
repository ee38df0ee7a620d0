"""Worker of tests/test_gpu_multi.py: one rank of a torch.distributed (NCCL) job on its own GPU.  Checks the library's peer-
memory exchange kernels (b200_allreduce, b200_allreduce_adam) against sums formed from an NCCL all-gather in the same rank
order and against the single-rank Adam entry point, over several consecutive exchanges and two channels."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from cuda_cnn_gan_vae_b200 import ops
    from cuda_cnn_gan_vae_b200.dp import PeerBuffer, slice_bounds
    from cuda_cnn_gan_vae_b200.lib import load
    lib = load()
    sizes = [4, 64, 1000, 4096 * 3 + 8, 1 << 20, 3_600_000]
    total = sum(sizes) * 3 + 64
    peer = PeerBuffer(total)
    assert peer.failed is None
    why = peer.self_test()
    assert why is None, why
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)

    def gathered_sum(t):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        s = parts[0].clone()
        for q in parts[1:]:
            s += q                      # rank order, one rounding per addition: the kernel's order
        return s

    # ---- plain all-reduce, several rounds per size, alternating channels ------------------------------------------
    offset = 0
    for n in sizes:
        view = peer.buffer[offset:offset + n]
        for rounds in range(3):
            view.copy_(torch.randn(n, device="cuda", generator=gen))
            want = gathered_sum(view)
            ops._check(lib.b200_allreduce(peer.comm, offset, n, rounds % 2, ops._stream()))
            ops.stream_status()
            assert torch.equal(view, want), ("allreduce", n, rounds, (view - want).abs().max().item())
        offset += n
    # ---- reduce-scatter + Adam + all-gather --------------------------------------------------------------------------
    for n in sizes:
        g_off, w_off = offset, offset + n
        offset += 2 * n
        grads, weights = peer.buffer[g_off:g_off + n], peer.buffer[w_off:w_off + n]
        w0 = torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7))      # identical on every rank
        weights.copy_(w0)
        m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        rw, rm, rv = w0.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        for it in (1, 2, 3):
            grads.copy_(torch.randn(n, device="cuda", generator=gen))
            mine = grads.clone()
            total_g = gathered_sum(grads)
            ops._check(lib.b200_allreduce_adam(peer.comm, g_off, w_off, ops._ptr(m), ops._ptr(v), n, 16 * world, 1e-3, 0.9, 0.999, 1e-8,
                                               float(it), None, 1, ops._stream()))
            ops.stream_status()
            ops._check(lib.b200_adam(ops._ptr(rw), ops._ptr(total_g), ops._ptr(rm), ops._ptr(rv), n, 16 * world, 1e-3, 0.9, 0.999, 1e-8, float(it),
                                     ops._stream()))
            ops.stream_status()
            assert torch.equal(weights, rw), ("fused adam weights", n, it, (weights - rw).abs().max().item())
            b, e = slice_bounds(n, rank, world)
            assert torch.equal(m[b:e], rm[b:e]) and torch.equal(v[b:e], rv[b:e]), ("moments of the own slice", n, it)
            assert torch.equal(grads, mine), "the gradient arena keeps this rank's contents"
    # ---- two arenas in one launch (b200_allreduce_adam_multi) against two single launches ------------------------------
    from cuda_cnn_gan_vae_b200.lib import ExchangeSegment
    na, nb = sizes[2], sizes[3]
    offs = [0, na, 2 * na, 2 * na + nb]                 # gradients a, weights a, gradients b, weights b (reusing the front of the buffer)
    init = torch.randn(2 * na + 2 * nb, device="cuda", generator=torch.Generator(device="cuda").manual_seed(11))
    init[0:na] = torch.randn(na, device="cuda", generator=gen)
    init[2 * na:2 * na + nb] = torch.randn(nb, device="cuda", generator=gen)
    results = []
    for together in (False, True):
        peer.buffer[:init.numel()].copy_(init)
        ma, va, mb, vb = (torch.zeros(k, device="cuda") for k in (na, na, nb, nb))
        dist.barrier()
        if together:
            segs = (ExchangeSegment * 2)()
            segs[0].grad_offset, segs[0].weight_offset, segs[0].n, segs[0].m, segs[0].v = offs[0], offs[1], na, ma.data_ptr(), va.data_ptr()
            segs[1].grad_offset, segs[1].weight_offset, segs[1].n, segs[1].m, segs[1].v = offs[2], offs[3], nb, mb.data_ptr(), vb.data_ptr()
            ops._check(lib.b200_allreduce_adam_multi(peer.comm, 2, segs, 16 * world, 1e-3, 0.9, 0.999, 1e-8, 1.0, None, 2, ops._stream()))
        else:
            ops._check(lib.b200_allreduce_adam(peer.comm, offs[0], offs[1], ops._ptr(ma), ops._ptr(va), na, 16 * world, 1e-3, 0.9, 0.999, 1e-8, 1.0,
                                               None, 2, ops._stream()))
            ops._check(lib.b200_allreduce_adam(peer.comm, offs[2], offs[3], ops._ptr(mb), ops._ptr(vb), nb, 16 * world, 1e-3, 0.9, 0.999, 1e-8, 1.0,
                                               None, 2, ops._stream()))
        ops.stream_status()
        dist.barrier()
        results.append((peer.buffer[:init.numel()].clone(), ma, va, mb, vb))
    for a_t, b_t in zip(*results):
        assert torch.equal(a_t, b_t), "one launch for two arenas differs from two launches"
    # ---- device time of the two exchanges at the sizes of the benchmark (reported, not asserted) ----------------------
    n = sizes[-1]
    g_off, w_off = offset - 2 * n, offset - n
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    for name, fn in (("allreduce_adam of %d floats" % n, lambda: lib.b200_allreduce_adam(peer.comm, g_off, w_off, ops._ptr(m), ops._ptr(v), n, 64 * world, 1e-3,
                                                                                          0.9, 0.999, 1e-8, 2.0, None, 1, ops._stream())),
                     ("allreduce of %d floats" % n, lambda: lib.b200_allreduce(peer.comm, g_off, n, 0, ops._stream())),
                     ("allreduce of 590080 floats", lambda: lib.b200_allreduce(peer.comm, 0, 590080, 0, ops._stream())),
                     ("NCCL all_reduce of %d floats (for comparison)" % n, lambda: dist.all_reduce(peer.buffer[g_off:g_off + n])),
                     ("NCCL all_reduce of 590080 floats (for comparison)", lambda: dist.all_reduce(peer.buffer[:590080]))):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ops.stream_status()
        if rank == 0:
            print("device time per call, %d ranks: %s: %.1f us" % (world, name, e0.elapsed_time(e1) / 20 * 1e3))
    dist.barrier()
    peer.close()
    if rank == 0:
        print("MULTI_GPU_WORKER_OK")
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()
