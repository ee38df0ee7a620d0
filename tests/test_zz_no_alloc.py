"""The allocation-free weight-gradient entry point against the regular one, through the C-ABI.

Some callers of the library may not allocate device memory at the moment they call it (their memory
comes from a pool filled at start-up, or they run where cudaMalloc's device-wide stall or a runtime
restriction rules allocation out).  b200_conv_wgrad_batch_static serves them from a fixed array inside
the library; it must give what b200_conv_wgrad_batch gives, call after call (the array keeps the
previous call's contents, so the second call checks that stale scratch is cleared), and must refuse
work that does not fit the array.  Collected last so that a failure here cannot hide another test."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tests.util import TOL_X3, conv_inputs, dot_rel_err  # noqa: E402


def _call(fn, g, dk, db, accumulate, x, d, batch):
    return fn(C.byref(g), C.c_void_p(dk.data_ptr()), C.c_void_p(db.data_ptr()), accumulate, C.c_void_p(x.data_ptr()),
              C.c_void_p(d.data_ptr()), batch, C.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_weight_gradient_matches_regular_entry_point(port):
    from cuda_cnn_gan_vae_b200 import ops
    from cuda_cnn_gan_vae_b200.lib import load
    lib = load()
    assert lib.b200_static_scratch_bytes() == 16 << 20
    cases = [(16, 3, 64, 64, 32, 3, 1, 1), (6, 8, 9, 7, 5, 4, 2, 1)]   # first: the CPU-runnable headline layer
    for call_no, (B, Cc, H, W, K, k, s, p) in enumerate(cases * 2):    # every case twice, interleaved: stale scratch must not leak
        x, wt, b, d = conv_inputs(40 + call_no, B, Cc, H, W, K, k, s, p)
        X, D = torch.from_numpy(x).cuda(), torch.from_numpy(d).cuda()
        g = ops.geom(Cc, H, W, K, k, k, s, s, p, p)
        base_k = torch.randn(1, 1, K, Cc * k * k, device="cuda")
        base_b = torch.randn(1, K, 1, 1, device="cuda")
        for accumulate in (0, 1):
            dk_s, db_s = base_k.clone(), base_b.clone()
            torch.cuda.synchronize()
            # what the driver reports as free device memory sees every cudaMalloc of the process, the library's included
            before = torch.cuda.mem_get_info()[0], lib.b200_scratch_bytes()
            assert _call(lib.b200_conv_wgrad_batch_static, g, dk_s, db_s, accumulate, X, D, B) == 0, lib.b200_last_error()
            torch.cuda.synchronize()
            assert lib.b200_scratch_bytes() == before[1]               # the growing arena was not touched
            if call_no > 0:                                            # the first call on the device may load the kernels' module
                assert torch.cuda.mem_get_info()[0] >= before[0], "the allocation-free entry point took device memory"
            # regular entry point, same fp32 CUDA-core arithmetic: identical bits
            ops.set_precision(ops.FP32)
            dk_r, db_r = base_k.clone(), base_b.clone()
            assert _call(lib.b200_conv_wgrad_batch, g, dk_r, db_r, accumulate, X, D, B) == 0, lib.b200_last_error()
            ops.stream_status()
            assert dk_s.cpu().numpy().tobytes() == dk_r.cpu().numpy().tobytes()
            assert db_s.cpu().numpy().tobytes() == db_r.cpu().numpy().tobytes()
            # regular entry point on the tensor cores (default mode): within the 3xTF32 tolerance
            ops.set_precision(ops.TF32X3)
            dk_t, db_t = base_k.clone(), base_b.clone()
            assert _call(lib.b200_conv_wgrad_batch, g, dk_t, db_t, accumulate, X, D, B) == 0, lib.b200_last_error()
            ops.stream_status()
            mag, _ = port.conv_wgrad(np.zeros((B, K, Cc * k * k), np.float32), np.zeros((B, K), np.float32), np.abs(x), np.abs(d),
                                     k, k, s, s, p, p)
            den = mag.astype(np.float64).sum(0).reshape(1, 1, K, -1) + accumulate * np.abs(base_k.cpu().numpy())
            assert dot_rel_err(dk_s.cpu().numpy(), dk_t.cpu().numpy(), den) <= TOL_X3
            bias_den = D.abs().sum((0, 2, 3)).cpu().numpy().reshape(1, K, 1, 1) + accumulate * np.abs(base_b.cpu().numpy())
            assert dot_rel_err(db_s.cpu().numpy(), db_t.cpu().numpy(), bias_den) <= 1e-5
    # the oracle agrees too (last case, accumulate = 0)
    dko, dbo = port.conv_wgrad(np.zeros((B, K, Cc * k * k), np.float32), np.zeros((B, K), np.float32), x, d, k, k, s, s, p, p)
    dk_s, db_s = base_k.clone(), base_b.clone()
    assert _call(lib.b200_conv_wgrad_batch_static, g, dk_s, db_s, 0, X, D, B) == 0
    ops.stream_status()
    assert np.allclose(dk_s.cpu().numpy().reshape(K, -1), dko.astype(np.float64).sum(0), rtol=1e-5, atol=1e-4)


def test_static_scratch_rejects_oversized_work():
    from cuda_cnn_gan_vae_b200 import ops
    from cuda_cnn_gan_vae_b200.lib import load
    lib = load()
    B, Cc, K, k = 64, 256, 256, 3                      # 64 * 256*256*9 floats = 151 MiB of per-sample gradients
    g = ops.geom(Cc, 8, 8, K, k, k, 1, 1, 1, 1)
    X = torch.zeros(B, Cc, 8, 8, device="cuda")
    D = torch.zeros(B, K, 8, 8, device="cuda")
    dk = torch.full((1, 1, K, Cc * k * k), 7.0, device="cuda")
    db = torch.full((1, K, 1, 1), 7.0, device="cuda")
    assert _call(lib.b200_conv_wgrad_batch_static, g, dk, db, 0, X, D, B) == 5          # B200_E_NOMEM
    assert b"fixed scratch" in lib.b200_last_error()
    torch.cuda.synchronize()
    assert (dk == 7.0).all() and (db == 7.0).all()      # a rejected call does nothing
