"""Caller-owned tensors that start at an odd float offset (a slice of a larger buffer: 4-byte aligned only) must take
the scalar code paths, not the 8- and 16-byte vector ones; results stay equal to the CPU oracle's."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tests.util import TOL_X3, conv_inputs, dot_rel_err  # noqa: E402


@pytest.fixture(scope="module")
def ops():
    from cuda_cnn_gan_vae_b200 import ops as o
    yield o
    o.set_precision(o.TF32X3)


def odd_view(a):
    """A contiguous CUDA copy of `a` that starts one float past a 256-byte boundary."""
    buf = torch.empty(a.size + 1, device="cuda")
    view = buf[1:].view(a.shape)
    view.copy_(torch.from_numpy(np.ascontiguousarray(a)))
    assert view.data_ptr() % 8 == 4
    return view


def test_maxpool_on_a_4_byte_aligned_view(ops, port):
    r = np.random.default_rng(31)
    x = r.integers(-3, 4, (3, 4, 8, 12)).astype(np.float32)
    o, p = port.maxpool(x, 2, 2)
    out = torch.empty(o.shape, device="cuda")
    pos = torch.empty(p.shape, dtype=torch.int32, device="cuda")
    ops.CTensorMath.MaxPooling(out, pos, odd_view(x), 2, 2)
    ops.stream_status()
    assert out.cpu().numpy().tobytes() == o.tobytes() and pos.cpu().numpy().tobytes() == p.tobytes()
    d = r.normal(0, 1, o.shape).astype(np.float32)
    back = odd_view(np.zeros(x.shape, np.float32))
    ops.CTensorMath.MaxPoolingBackward(back, pos, odd_view(d), 2, 2)
    ops.stream_status()
    assert back.cpu().numpy().tobytes() == port.maxpool_backward(d, p, 2, 2).tobytes()


def test_position_tensor_must_be_8_byte_aligned(ops):
    from cuda_cnn_gan_vae_b200.lib import load
    x = torch.zeros(1, 1, 4, 4, device="cuda")
    out = torch.empty(1, 1, 2, 2, device="cuda")
    raw = torch.empty(9, dtype=torch.int32, device="cuda")
    r = load().b200_maxpool(out.data_ptr(), raw.data_ptr() + 4, x.data_ptr(), 1, 1, 4, 4, 2, 2, None)
    assert r == 2 and b"8-byte" in load().b200_last_error()          # B200_E_ARG, nothing launched
    torch.cuda.synchronize()


@pytest.mark.parametrize("case", [(8, 256, 8, 8, 512, 4, 2, 1), (5, 512, 4, 4, 100, 3, 1, 1)])
def test_split_contraction_into_a_4_byte_aligned_output(ops, port, case):
    """Layers with few output pixels split the contraction and sum the partial outputs with 16-byte stores; an output
    that is not 16-byte aligned must not take that route."""
    B, C, H, W, K, k, s, p = case
    ops.set_precision(ops.TF32X3)
    x, wt, b, d = conv_inputs(sum(case) + 9, B, C, H, W, K, k, s, p)
    layer = ops.ConvLayer(C, H, W, K, k, k, s, s, p, p, B)
    X, WT, BI, D = (torch.from_numpy(a).cuda() for a in (x, wt, b, d))
    y = odd_view(np.zeros(d.shape, np.float32))
    layer.forward(y, X, WT, BI)
    dx = odd_view(np.zeros(x.shape, np.float32))
    layer.backward(dx, None, None, D, X, WT)
    ops.stream_status()
    assert ops.last_path() == ops.PATH_TCGEN05
    zb = np.zeros((1, K), np.float32)
    assert dot_rel_err(y.cpu().numpy(), port.conv_forward(x, wt[0], b.reshape(1, K), k, k, s, s, p, p),
                       port.conv_forward(np.abs(x), np.abs(wt[0]), np.abs(b).reshape(1, K), k, k, s, s, p, p)) <= TOL_X3
    assert dot_rel_err(dx.cpu().numpy(), port.conv_backward(d, wt[0], zb, (C, H, W), k, k, s, s, p, p),
                       port.conv_backward(np.abs(d), np.abs(wt[0]), zb, (C, H, W), k, k, s, s, p, p)) <= TOL_X3
    layer.close()
