"""GPU parity of the convolution trio, called through the C-ABI (ctypes) and compared with the CPU
oracle on the same seeded inputs.  Tolerances: bit-exact for the CUDA-core fp32 path, 1e-4 (3xTF32)
and 2e-3 (plain TF32) for the tcgen05 path, on tests.util.max_rel_err."""
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tests.util import TOL_TF32, TOL_X3, conv_inputs, dot_rel_err, max_rel_err  # noqa: E402

G = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def ops():
    from cuda_cnn_gan_vae_b200 import ops as o
    assert torch.cuda.is_available()
    yield o
    o.set_precision(o.TF32X3)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_trio(ops, x, wt, b, d, k, s, p):
    """forward, backward-data, batch-summed wgrad through the library; returns numpy results + paths."""
    B, C, H, W = x.shape
    K = wt.shape[2]
    X, WT, BI, D = dev(x), dev(wt), dev(b), dev(d)
    y = torch.full(d.shape, float("nan"), device="cuda")
    ops.CTensorConv.ForwardConvolution(y, X, WT, k, k, C, K, BI, s, s, p, p)
    p_f = ops.last_path()
    dx = torch.full(x.shape, float("nan"), device="cuda")
    ops.CTensorConv.BackwardConvolution(dx, D, WT, k, k, C, K, None, s, s, p, p)
    p_b = ops.last_path()
    dk = torch.full((1, 1, K, C * k * k), float("nan"), device="cuda")
    db = torch.full((1, K, 1, 1), float("nan"), device="cuda")
    ops.CTensorConv.CreateDeltaWeightAndBiasBatch(dk, k, k, C, K, db, X, D, s, s, p, p, accumulate=False)
    p_w = ops.last_path()
    ops.stream_status()
    return (y.cpu().numpy(), dx.cpu().numpy(), dk.cpu().numpy().reshape(K, -1), db.cpu().numpy().reshape(K)), (p_f, p_b, p_w)


def oracle_trio(port, x, wt, b, d, k, s, p):
    B, C, H, W = x.shape
    K = wt.shape[2]
    y = port.conv_forward(x, wt[0], b.reshape(1, K), k, k, s, s, p, p)
    dx = port.conv_backward(d, wt[0], np.zeros((1, K), np.float32), (C, H, W), k, k, s, s, p, p)
    dk, db = port.conv_wgrad(np.zeros((B, K, C * k * k), np.float32), np.zeros((B, K), np.float32), x, d, k, k, s, s, p, p)
    # the layer's reduction over the batch (AddSumW), in float64 so that the oracle adds no order noise
    return y, dx, dk.astype(np.float64).sum(0), db.astype(np.float64).sum(0)


# B, C, H, W, K, k, s, p -- the layer shapes of the headline configurations at reduced batch, plus ragged ones
TC_CASES = [
    (2, 3, 64, 64, 32, 3, 1, 1),      # config 1 layer
    (2, 256, 32, 32, 256, 3, 1, 1),   # data-parallel sweep layer
    (4, 3, 64, 64, 64, 4, 2, 1),      # DCGAN discriminator layers
    (4, 64, 32, 32, 128, 4, 2, 1),
    (4, 256, 8, 8, 512, 4, 2, 1),
    (4, 64, 32, 32, 3, 4, 2, 1),      # as transposed conv: generator's last layer (3 output channels)
    (2, 32, 128, 128, 64, 3, 1, 1),   # VAE encoder layer
    (3, 40, 12, 12, 24, 3, 1, 1),     # ragged: nothing is a multiple of the tile
    (2, 16, 9, 7, 8, 5, 2, 2),
    (5, 7, 5, 6, 3, 1, 1, 0),
    (2, 8, 6, 10, 4, 3, 3, 1),        # stride 3
]


@pytest.mark.parametrize("case", TC_CASES)
@pytest.mark.parametrize("mode", ["x3", "tf32"])
def test_tensor_core_trio_matches_oracle(ops, port, case, mode):
    B, C, H, W, K, k, s, p = case
    ops.set_precision(ops.TF32X3 if mode == "x3" else ops.TF32)
    tol = TOL_X3 if mode == "x3" else TOL_TF32
    x, wt, b, d = conv_inputs(sum(case), B, C, H, W, K, k, s, p)
    got, paths = run_trio(ops, x, wt, b, d, k, s, p)
    want = oracle_trio(port, x, wt, b, d, k, s, p)
    mag = oracle_trio(port, np.abs(x), np.abs(wt), np.abs(b), np.abs(d), k, s, p)   # the contractions on |operands|
    assert paths == (ops.PATH_TCGEN05,) * 3, paths
    for name, g, w, m in zip(("forward", "backward", "dkernel", "dbias"), got, want, mag):
        assert not np.isnan(g).any(), name
        err = dot_rel_err(g, w, m)
        assert err <= (tol if name != "dbias" else 1e-5), (name, err)
        if mode == "x3":          # the stricter RMS-floored element-wise metric also holds in 3xTF32 mode
            assert max_rel_err(g, w) <= tol, (name, max_rel_err(g, w))


@pytest.mark.parametrize("case", [(3, 3, 9, 8, 4, 3, 1, 1), (2, 5, 11, 7, 3, 5, 2, 2), (4, 2, 8, 8, 6, 4, 2, 1)])
def test_cuda_core_path_is_bit_exact(ops, port, case):
    B, C, H, W, K, k, s, p = case
    ops.set_precision(ops.FP32)
    x, wt, b, d = conv_inputs(3, B, C, H, W, K, k, s, p)
    X, WT, BI, D = dev(x), dev(wt), dev(b), dev(d)
    y = torch.empty_like(D)
    ops.CTensorConv.ForwardConvolution(y, X, WT, k, k, C, K, BI, s, s, p, p)
    assert ops.last_path() == ops.PATH_SIMT
    assert y.cpu().numpy().tobytes() == port.conv_forward(x, wt[0], b.reshape(1, K), k, k, s, s, p, p).tobytes()
    dx = torch.empty_like(X)
    ops.CTensorConv.BackwardConvolution(dx, D, WT, k, k, C, K, None, s, s, p, p)
    zb = np.zeros((1, K), np.float32)
    assert dx.cpu().numpy().tobytes() == port.conv_backward(d, wt[0], zb, (C, H, W), k, k, s, s, p, p).tobytes()
    # a non-zero bias in the backward pass follows the CPU backend's rule (added once per tap and filter)
    ops.CTensorConv.BackwardConvolution(dx, D, WT, k, k, C, K, BI, s, s, p, p)
    assert dx.cpu().numpy().tobytes() == port.conv_backward(d, wt[0], b.reshape(1, K), (C, H, W), k, k, s, s, p, p).tobytes()
    # per-sample weight gradients, accumulating into non-zero tensors
    r = np.random.default_rng(1)
    dk0 = r.normal(0, 1, (B, 1, K, C * k * k)).astype(np.float32)
    db0 = r.normal(0, 1, (B, K, 1, 1)).astype(np.float32)
    DK, DB = dev(dk0), dev(db0)
    ops.CTensorConv.CreateDeltaWeightAndBias(DK, k, k, C, K, DB, X, D, s, s, p, p)
    dko, dbo = port.conv_wgrad(dk0[:, 0], db0.reshape(B, K), x, d, k, k, s, s, p, p)
    assert DK.cpu().numpy().tobytes() == dko.tobytes() and DB.cpu().numpy().tobytes() == dbo.tobytes()
    ops.stream_status()


def test_per_sample_kernels_and_broadcast(ops, port):
    """W-broadcast rule: one image against per-sample kernels (the reference's own test uses W = batch kernels)."""
    ops.set_precision(ops.TF32X3)
    r = np.random.default_rng(7)
    x = r.normal(0, 1, (1, 2, 6, 6)).astype(np.float32)
    wt = r.normal(0, 1, (4, 1, 3, 18)).astype(np.float32)
    b = r.normal(0, 1, (4, 3, 1, 1)).astype(np.float32)
    y = torch.empty(4, 3, 6, 6, device="cuda")
    ops.CTensorConv.ForwardConvolution(y, dev(x), dev(wt), 3, 3, 2, 3, dev(b), 1, 1, 1, 1)
    assert ops.last_path() == ops.PATH_SIMT
    assert y.cpu().numpy().tobytes() == port.conv_forward(x, wt[:, 0], b.reshape(4, 3), 3, 3, 1, 1, 1, 1).tobytes()


def test_reference_known_answer_vectors(ops):
    """The reference's in-binary known-answer tests (cuda/ctensortest.cu.h), through the C-ABI, in every
    precision mode: all values are small integers, so every path must reproduce them exactly."""
    kat = np.load(os.path.join(G, "reference_kat.npz"))
    B = 10
    for mode in (ops.TF32X3, ops.TF32, ops.FP32):
        ops.set_precision(mode)
        y = torch.empty(B, 2, 2, 2, device="cuda")
        ops.CTensorConv.ForwardConvolution(y, dev(kat["fwd_image"]), dev(kat["fwd_kernel"].reshape(1, 1, 2, 12)), 2, 2, 3, 2,
                                           torch.zeros(1, 2, 1, 1, device="cuda"), 1, 1, 0, 0)
        assert np.array_equal(y.cpu().numpy(), kat["fwd_expected"])
        y = torch.empty(B, 2, 3, 3, device="cuda")
        ops.CTensorConv.ForwardConvolution(y, dev(kat["fwd_s2_image"]), dev(kat["fwd_s2_kernel"].reshape(1, 1, 2, 27)), 3, 3, 3, 2,
                                           torch.zeros(1, 2, 1, 1, device="cuda"), 2, 2, 1, 1)
        assert np.array_equal(y.cpu().numpy(), kat["fwd_s2_expected"])
        dk = torch.zeros(B, 1, 1, 25, device="cuda")
        db = torch.zeros(B, 1, 1, 1, device="cuda")
        ops.CTensorConv.CreateDeltaWeightAndBias(dk, 5, 5, 1, 1, db, dev(kat["wgrad_s2_image"]), dev(kat["wgrad_s2_delta"]), 2, 2, 2, 2)
        assert np.array_equal(dk.cpu().numpy().reshape(B, 1, 25), kat["wgrad_s2_expected"])
        assert np.array_equal(db.cpu().numpy().reshape(B, 1), kat["wgrad_s2_dbias"])
        dk = torch.zeros(B, 1, 1, 9, device="cuda")
        db = torch.zeros(B, 1, 1, 1, device="cuda")
        ops.CTensorConv.CreateDeltaWeightAndBias(dk, 3, 3, 1, 1, db, dev(kat["wgrad_s1_image"]), dev(kat["wgrad_s1_delta"]), 1, 1, 0, 0)
        assert np.array_equal(dk.cpu().numpy().reshape(B, 1, 9), kat["wgrad_s1_expected"])
        # the batch-summed entry point on the same data: ten identical samples
        dks = torch.zeros(1, 1, 1, 9, device="cuda")
        ops.CTensorConv.CreateDeltaWeightAndBiasBatch(dks, 3, 3, 1, 1, None, dev(kat["wgrad_s1_image"]), dev(kat["wgrad_s1_delta"]),
                                                      1, 1, 0, 0, accumulate=False)
        assert np.array_equal(dks.cpu().numpy().reshape(9), kat["wgrad_s1_expected"][0, 0] * B)
        dx = torch.empty(B, 1, 7, 7, device="cuda")
        ops.CTensorConv.BackwardConvolution(dx, dev(kat["bwd_delta"]), dev(kat["bwd_kernel"].reshape(1, 1, 1, 25)), 5, 5, 1, 1, None, 2, 2, 2, 2)
        assert np.array_equal(dx.cpu().numpy(), kat["bwd_expected"])
        ops.stream_status()


def test_transposed_conv_layer_weight_gradient(ops, port):
    """CreateBackDeltaWeightAndBias: image and delta exchanged, bias gradient forced to zero."""
    ops.set_precision(ops.TF32X3)
    r = np.random.default_rng(5)
    B, K, C, k, s, p = 3, 4, 2, 4, 2, 1
    small = r.normal(0, 1, (B, K, 4, 4)).astype(np.float32)
    big = r.normal(0, 1, (B, C, 8, 8)).astype(np.float32)
    dk = torch.zeros(B, 1, K, C * k * k, device="cuda")
    db = torch.ones(B, K, 1, 1, device="cuda")
    ops.CTensorConv.CreateBackDeltaWeightAndBias(dk, k, k, C, K, db, dev(small), dev(big), s, s, p, p)
    dko, dbo = port.conv_wgrad(np.zeros((B, K, C * k * k), np.float32), np.ones((B, K), np.float32), small, big, k, k, s, s, p, p,
                               back_variant=True)
    assert dk.cpu().numpy().reshape(dko.shape).tobytes() == dko.tobytes()
    assert not db.cpu().numpy().any()


def test_wgrad_batch_accumulates(ops, port):
    ops.set_precision(ops.TF32X3)
    B, C, H, W, K, k, s, p = 4, 32, 16, 16, 32, 3, 1, 1
    x, wt, b, d = conv_inputs(11, B, C, H, W, K, k, s, p)
    base = np.random.default_rng(2).normal(0, 5, (1, 1, K, C * k * k)).astype(np.float32)
    dk = dev(base)
    db = torch.full((1, K, 1, 1), 2.0, device="cuda")
    ops.CTensorConv.CreateDeltaWeightAndBiasBatch(dk, k, k, C, K, db, dev(x), dev(d), s, s, p, p, accumulate=True)
    assert ops.last_path() == ops.PATH_TCGEN05
    dko, dbo = port.conv_wgrad(np.zeros((B, K, C * k * k), np.float32), np.zeros((B, K), np.float32), x, d, k, k, s, s, p, p)
    want = base.reshape(K, -1) + dko.astype(np.float64).sum(0)
    assert max_rel_err(dk.cpu().numpy().reshape(K, -1), want) <= TOL_X3
    assert max_rel_err(db.cpu().numpy().reshape(K), 2.0 + dbo.astype(np.float64).sum(0)) <= 1e-5
    ops.stream_status()


def test_linearity_and_adjointness_at_scale(ops):
    """Size-independent properties at a size the CPU oracle cannot finish quickly:
    <conv(x), d> == <x, conv_backward(d)> == <W, wgrad(x, d)> (the three kernels are adjoints of one
    bilinear map), checked in float64 on the results of the three tensor-core kernels."""
    ops.set_precision(ops.TF32X3)
    B, C, H, W, K, k, s, p = 32, 256, 32, 32, 256, 3, 1, 1
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(B, C, H, W, device="cuda", generator=g)
    wt = torch.randn(1, 1, K, C * k * k, device="cuda", generator=g) * (2.0 / (C * k * k)) ** 0.5
    d = torch.randn(B, K, H, W, device="cuda", generator=g)
    zero_b = torch.zeros(1, K, 1, 1, device="cuda")
    y = torch.empty_like(d)
    ops.CTensorConv.ForwardConvolution(y, x, wt, k, k, C, K, zero_b, s, s, p, p)
    dx = torch.empty_like(x)
    ops.CTensorConv.BackwardConvolution(dx, d, wt, k, k, C, K, None, s, s, p, p)
    dk = torch.empty_like(wt)
    ops.CTensorConv.CreateDeltaWeightAndBiasBatch(dk, k, k, C, K, None, x, d, s, s, p, p, accumulate=False)
    ops.stream_status()
    a = (y.double() * d.double()).sum().item()
    b_ = (x.double() * dx.double()).sum().item()
    c = (wt.double() * dk.double()).sum().item()
    scale = (y.double().norm() * d.double().norm()).item()
    assert abs(a - b_) <= 1e-6 * scale and abs(a - c) <= 1e-6 * scale, (a, b_, c, scale)


# degenerate and tile-boundary geometries: a single pixel, a kernel larger than the image, stride equal to the kernel,
# channel / filter counts one past a tile boundary (32 channels per K block, 128 filter rows, 256 columns), one image
EDGE_CASES = [
    (1, 1, 1, 1, 1, 1, 1, 0),
    (1, 1, 3, 3, 1, 3, 1, 1),
    (1, 2, 2, 2, 3, 5, 1, 2),          # 5x5 kernel over a 2x2 image
    (2, 5, 8, 8, 7, 4, 4, 0),          # stride == kernel size: disjoint windows
    (1, 33, 5, 5, 257, 3, 1, 1),       # one past 32 channels and 256 filters
    (3, 129, 6, 6, 129, 3, 1, 1),      # one past 128
    (130, 4, 4, 4, 4, 3, 1, 1),        # batch one past the 128-row tile
    (2, 6, 17, 5, 5, 3, 2, 0),         # no padding, stride 2, odd sizes
]


@pytest.mark.parametrize("case", EDGE_CASES)
@pytest.mark.parametrize("mode", ["x3", "fp32"])
def test_edge_geometries(ops, port, case, mode):
    B, C, H, W, K, k, s, p = case
    ops.set_precision(ops.TF32X3 if mode == "x3" else ops.FP32)
    x, wt, b, d = conv_inputs(sum(case) + 11, B, C, H, W, K, k, s, p)
    got, _ = run_trio(ops, x, wt, b, d, k, s, p)
    want = oracle_trio(port, x, wt, b, d, k, s, p)
    mag = oracle_trio(port, np.abs(x), np.abs(wt), np.abs(b), np.abs(d), k, s, p)
    for name, g, w, m in zip(("forward", "backward", "dkernel", "dbias"), got, want, mag):
        assert not np.isnan(g).any(), name
        assert g.shape == w.shape
        assert dot_rel_err(g, w, m) <= (TOL_X3 if mode == "x3" else 1e-5), (name, dot_rel_err(g, w, m))


@pytest.mark.parametrize("case", [(4, 3, 16, 16, 32, 3, 1, 1), (4, 3, 32, 32, 64, 4, 2, 1), (3, 1, 12, 10, 20, 5, 1, 2), (2, 8, 9, 9, 16, 3, 2, 1)])
@pytest.mark.parametrize("transposed", [False, True])
def test_few_channel_layers(ops, port, case, transposed):
    """Layers with <= 8 channels on one side run with the taps folded into the channel dimension: same results as the
    oracle's convolution trio, for the convolution layer and for the transposed-convolution layer."""
    B, C, H, W, K, k, s, p = case
    ops.set_precision(ops.TF32X3)
    big, wt, b, small = conv_inputs(sum(case) + 5, B, C, H, W, K, k, s, p)      # big: C channels H x W; small: K channels oy x ox
    layer = ops.ConvLayer(C, H, W, K, k, k, s, s, p, p, B, transposed=transposed)
    zb = np.zeros((1, K), np.float32)
    zk = np.zeros((B, K, C * k * k), np.float32)
    if not transposed:
        out = torch.full(small.shape, float("nan"), device="cuda")
        layer.forward(out, dev(big), dev(wt), dev(b))
        assert ops.last_path() == ops.PATH_TCGEN05
        d_in, dk, db = torch.full(big.shape, float("nan"), device="cuda"), torch.empty(1, 1, K, C * k * k, device="cuda"), torch.empty(1, K, 1, 1, device="cuda")
        layer.backward(d_in, dk, db, dev(small), dev(big), dev(wt), accumulate=False)
        want = (port.conv_forward(big, wt[0], b.reshape(1, K), k, k, s, s, p, p),
                port.conv_backward(small, wt[0], zb, (C, H, W), k, k, s, s, p, p))
        mag = (port.conv_forward(np.abs(big), np.abs(wt[0]), np.abs(b).reshape(1, K), k, k, s, s, p, p),
               port.conv_backward(np.abs(small), np.abs(wt[0]), zb, (C, H, W), k, k, s, s, p, p))
        dko, dbo = port.conv_wgrad(zk, np.zeros((B, K), np.float32), big, small, k, k, s, s, p, p)
        mk, mb = port.conv_wgrad(zk, np.zeros((B, K), np.float32), np.abs(big), np.abs(small), k, k, s, s, p, p)
        assert dot_rel_err(db.cpu().numpy().reshape(K), dbo.astype(np.float64).sum(0), mb.astype(np.float64).sum(0)) <= 1e-5
    else:
        out = torch.full(big.shape, float("nan"), device="cuda")
        layer.forward(out, dev(small), dev(wt))
        assert ops.last_path() == ops.PATH_TCGEN05
        d_in, dk, db = torch.full(small.shape, float("nan"), device="cuda"), torch.empty(1, 1, K, C * k * k, device="cuda"), torch.full((1, K, 1, 1), 3.0, device="cuda")
        layer.backward(d_in, dk, db, dev(big), dev(small), dev(wt), accumulate=False)
        want = (port.conv_backward(small, wt[0], zb, (C, H, W), k, k, s, s, p, p), port.conv_forward(big, wt[0], zb, k, k, s, s, p, p))
        mag = (port.conv_backward(np.abs(small), np.abs(wt[0]), zb, (C, H, W), k, k, s, s, p, p),
               port.conv_forward(np.abs(big), np.abs(wt[0]), zb, k, k, s, s, p, p))
        dko, _ = port.conv_wgrad(zk, np.ones((B, K), np.float32), small, big, k, k, s, s, p, p, back_variant=True)
        mk, _ = port.conv_wgrad(zk, np.ones((B, K), np.float32), np.abs(small), np.abs(big), k, k, s, s, p, p, back_variant=True)
        assert not db.cpu().numpy().any()
    ops.stream_status()
    assert dot_rel_err(out.cpu().numpy(), want[0], mag[0]) <= TOL_X3
    assert dot_rel_err(d_in.cpu().numpy(), want[1], mag[1]) <= TOL_X3
    assert dot_rel_err(dk.cpu().numpy().reshape(K, -1), dko.astype(np.float64).sum(0), mk.astype(np.float64).sum(0)) <= TOL_X3
    layer.close()


@pytest.mark.parametrize("mode", ["x3", "tf32"])
def test_single_layer_configuration_at_full_size(ops, port, mode):
    """The CPU-runnable configuration at its stated size: batch 16 of 3x64x64 uniform[-1,1], 32 filters 3x3 stride 1 pad 1,
    He-normal weights, zero bias, upstream delta N(0,1), seed 1 -- through the tensor-math calls and through the layer calls
    (the few-channel path), forward + backward-data + batch-summed weight and bias gradients."""
    B, C, H, W, K, k, s, p = 16, 3, 64, 64, 32, 3, 1, 1
    ops.set_precision(ops.TF32X3 if mode == "x3" else ops.TF32)
    tol = TOL_X3 if mode == "x3" else TOL_TF32
    rng = np.random.default_rng(1)
    x = rng.uniform(-1, 1, (B, C, H, W)).astype(np.float32)
    wt = (rng.standard_normal((1, 1, K, C * k * k)) * np.sqrt(2.0 / (C * k * k))).astype(np.float32)
    b = np.zeros((1, K, 1, 1), np.float32)
    d = rng.standard_normal((B, K, H, W)).astype(np.float32)
    want = oracle_trio(port, x, wt, b, d, k, s, p)
    mag = oracle_trio(port, np.abs(x), np.abs(wt), np.abs(b), np.abs(d), k, s, p)
    got, _ = run_trio(ops, x, wt, b, d, k, s, p)
    layer = ops.ConvLayer(C, H, W, K, k, k, s, s, p, p, B)
    y, dx = torch.empty(B, K, H, W, device="cuda"), torch.empty(B, C, H, W, device="cuda")
    dk, db = torch.empty(1, 1, K, C * k * k, device="cuda"), torch.empty(1, K, 1, 1, device="cuda")
    layer.forward(y, dev(x), dev(wt), dev(b))
    layer.backward(dx, dk, db, dev(d), dev(x), dev(wt), accumulate=False)
    ops.stream_status()
    via_layer = (y.cpu().numpy(), dx.cpu().numpy(), dk.cpu().numpy().reshape(K, -1), db.cpu().numpy().reshape(K))
    for which, result in (("tensor-math calls", got), ("layer calls", via_layer)):
        for name, g, w, m in zip(("forward", "backward", "dkernel", "dbias"), result, want, mag):
            err = dot_rel_err(g, w, m)
            assert err <= (tol if name != "dbias" else 1e-5), (which, name, err)
    layer.close()
