"""The data-parallel path on two CPU ranks (gloo): shard the batch, take each shard's batch-summed
weight gradient (here with the CPU oracle standing in for the per-rank kernel), all-reduce the gradient
arena, and compare with the full-batch oracle result."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402


def test_shard_bounds_cover_the_batch():
    from cuda_cnn_gan_vae_b200.dp import shard_bounds
    for batch in (1, 7, 64, 1024):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(batch, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from cuda_cnn_gan_vae_b200.dp import GradArena, shard_bounds
    from oracle import Oracle
    from tests.util import conv_inputs
    orc = Oracle("port")
    B, C, H, W, K, k, s, p = 6, 4, 8, 8, 5, 3, 1, 1
    x, wt, b, d = conv_inputs(21, B, C, H, W, K, k, s, p)          # same seed on every rank: the global batch
    lo, hi = shard_bounds(B, rank, world)
    arena = GradArena({"conv.dW": (1, 1, K, C * k * k), "conv.dB": (1, K, 1, 1)}, "cpu")
    n = hi - lo
    dk, db = orc.conv_wgrad(np.zeros((n, K, C * k * k), np.float32), np.zeros((n, K), np.float32), x[lo:hi], d[lo:hi], k, k, s, s, p, p)
    arena.views["conv.dW"].copy_(torch.from_numpy(dk.sum(0)).view(1, 1, K, -1))
    arena.views["conv.dB"].copy_(torch.from_numpy(db.sum(0)).view(1, K, 1, 1))
    arena.all_reduce()
    if rank == 0:
        np.save(os.path.join(out_dir, "dW.npy"), arena.views["conv.dW"].numpy())
        np.save(os.path.join(out_dir, "dB.npy"), arena.views["conv.dB"].numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gradient_arena_matches_full_batch(tmp_path, port):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    from tests.util import conv_inputs
    B, C, H, W, K, k, s, p = 6, 4, 8, 8, 5, 3, 1, 1
    x, wt, b, d = conv_inputs(21, B, C, H, W, K, k, s, p)
    dk, db = port.conv_wgrad(np.zeros((B, K, C * k * k), np.float32), np.zeros((B, K), np.float32), x, d, k, k, s, s, p, p)
    got_w = np.load(tmp_path / "dW.npy").reshape(K, -1)
    got_b = np.load(tmp_path / "dB.npy").reshape(K)
    assert np.allclose(got_w, dk.astype(np.float64).sum(0), rtol=1e-5, atol=1e-5)
    assert np.allclose(got_b, db.astype(np.float64).sum(0), rtol=1e-5, atol=1e-5)


def test_slice_arithmetic_of_the_fused_exchange():
    """b200_comm_slice (host arithmetic of the library): the slices of all ranks tile the arena in 16-byte groups, in rank
    order, for every world size; misuse is rejected."""
    from cuda_cnn_gan_vae_b200.dp import slice_bounds
    for n in (0, 4, 8, 1000, 4096 * 3 + 8, 3_600_000):
        for world in (1, 2, 3, 4, 8, 16):
            cursor = 0
            for rank in range(world):
                b, e = slice_bounds(n, rank, world)
                assert b == cursor and e >= b and b % 4 == 0 and e % 4 == 0
                cursor = e
            assert cursor == n
    import pytest
    with pytest.raises(ValueError):
        slice_bounds(10, 0, 2)          # not a multiple of 4 floats
    with pytest.raises(ValueError):
        slice_bounds(8, 2, 2)
