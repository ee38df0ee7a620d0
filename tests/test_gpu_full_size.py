"""Parity at the sizes of the benchmark configurations, in both tensor-core modes (plain TF32: 2e-3, 3xTF32: 1e-4).

  * the data-parallel convolution sweep at its full batch (1024 images of 256x32x32, 256 filters 3x3) through the layer
    calls the benchmark times: sampled images of the forward and backward-data results and a weight gradient whose output
    error is non-zero on sampled images only against the reference CPU backend, the dense full-batch results through the
    adjoint identity in float64;
  * the DCGAN generator and discriminator at full widths and batch 64, the VAE encoder and decoder at 3x128x128 with
    widths 32..256 (batch 32: the CPU twin of batch 128 would take minutes per mode), layer by layer against the CPU twin.

Every comparison is gated on dot_rel_err (|error| / sum |a||b|) and also records survey_rel_err (|error| / max(|want|,
1e-3 max |want|)); the latter is bounded by what was measured (PARITY_BOUNDS)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import tests.test_gpu_nets as nets_tests  # noqa: E402
from tests.util import TOL_TF32, TOL_X3, record_parity  # noqa: E402

MODES = [("tf32x3", TOL_X3), ("tf32", TOL_TF32)]
# survey_rel_err judges an output element that cancels to nearly zero against a thousandth of the tensor's largest element,
# not against what was summed to get it.  Measured on the convolution sweep (2304-term sums, |output| up to ~7.5, floor
# 7.5e-3): 0.22-0.24 in plain TF32 (absolute errors of ~1.7e-3, operand rounding 2^-11) and 5e-3..7e-3 in 3xTF32 (absolute
# errors of ~5e-5: the tensor core's fp32 accumulator does not round to nearest).  The bounds below are those figures with
# a factor of two of head-room; the 2e-3 / 1e-4 tolerances are met on dot_rel_err.
PARITY_BOUNDS = {"tf32": 0.5, "tf32x3": 2e-2}


@pytest.fixture(scope="module")
def ops():
    from cuda_cnn_gan_vae_b200 import ops as o
    yield o
    o.set_precision(o.TF32X3)
    nets_tests.REPORT_PREFIX = ""


def _mode(ops, name):
    ops.set_precision(ops.TF32X3 if name == "tf32x3" else ops.TF32)


@pytest.mark.parametrize("mode,tol", MODES)
def test_conv_sweep_layer_at_batch_1024(ops, port_mt, mode, tol):
    _mode(ops, mode)
    B, C, H, W, K, k = 1024, 256, 32, 32, 256, 3
    gen = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(B, C, H, W, device="cuda", generator=gen)
    d = torch.randn(B, K, H, W, device="cuda", generator=gen)
    wt = torch.randn(1, 1, K, C * k * k, device="cuda", generator=gen) * (2.0 / (C * k * k)) ** 0.5
    bias = torch.randn(1, K, 1, 1, device="cuda", generator=gen) * 0.1
    y, dx = torch.empty_like(d), torch.empty_like(x)
    dk, db = torch.empty_like(wt), torch.empty_like(bias)
    layer = ops.ConvLayer(C, H, W, K, k, k, 1, 1, 1, 1, B)
    layer.forward(y, x, wt, bias)
    assert ops.last_path() == ops.PATH_TCGEN05
    layer.backward(dx, dk, db, d, x, wt, accumulate=False)
    ops.stream_status()
    # sampled images against the reference CPU backend
    idx = [0, 333, 512, 1023]
    xs, ds = x[idx].cpu().numpy(), d[idx].cpu().numpy()
    w_h, b_h = wt.cpu().numpy()[0], bias.cpu().numpy().reshape(1, K)
    zb = np.zeros((1, K), np.float32)
    want_y = port_mt.conv_forward(xs, w_h, b_h, k, k, 1, 1, 1, 1)
    mag_y = port_mt.conv_forward(np.abs(xs), np.abs(w_h), np.abs(b_h), k, k, 1, 1, 1, 1)
    e, sv = record_parity(f"conv_sweep B=1024 {mode}: forward, 4 sampled images", y[idx].cpu().numpy(), want_y, mag_y)
    assert e <= tol and sv <= PARITY_BOUNDS[mode], (e, sv)
    want_dx = port_mt.conv_backward(ds, w_h, zb, (C, H, W), k, k, 1, 1, 1, 1)
    mag_dx = port_mt.conv_backward(np.abs(ds), np.abs(w_h), zb, (C, H, W), k, k, 1, 1, 1, 1)
    e, sv = record_parity(f"conv_sweep B=1024 {mode}: backward-data, 4 sampled images", dx[idx].cpu().numpy(), want_dx, mag_dx)
    assert e <= tol and sv <= PARITY_BOUNDS[mode], (e, sv)
    # the dense full-batch results: <conv(x) - bias, d> = <x, conv_backward(d)> = <W, wgrad(x, d)> and dB = sum d, in float64
    dd = d.double()
    lhs = ((y.double() - bias.double()) * dd).sum().item()
    mid = (x.double() * dx.double()).sum().item()
    rhs = (wt.double() * dk.double()).sum().item()
    scale = (y.double().abs() * dd.abs()).sum().item()
    rel = tol * 1e-2                                   # the identity sums 2.7e8 products: rounding errors average out
    assert abs(lhs - mid) <= rel * scale and abs(lhs - rhs) <= rel * scale, (lhs, mid, rhs, scale)
    assert torch.allclose(db.double().view(K), dd.sum((0, 2, 3)), rtol=1e-5, atol=1e-2)
    # the weight gradient of the full-batch launch (same tiles, same split of the 1024 x 32 x 32 pixels) with an output
    # error that is non-zero on 8 scattered images only: equals the CPU sum over those images
    idx8 = [0, 1, 255, 256, 511, 640, 1022, 1023]
    d8 = torch.zeros_like(d)
    d8[idx8] = d[idx8]
    layer.backward(None, dk, db, d8, x, wt, accumulate=False)
    ops.stream_status()
    xs8, ds8 = x[idx8].cpu().numpy(), d[idx8].cpu().numpy()
    z = np.zeros((8, K, C * k * k), np.float32)
    dko, dbo = port_mt.conv_wgrad(z, np.zeros((8, K), np.float32), xs8, ds8, k, k, 1, 1, 1, 1)
    mko, _ = port_mt.conv_wgrad(z, np.zeros((8, K), np.float32), np.abs(xs8), np.abs(ds8), k, k, 1, 1, 1, 1)
    e, sv = record_parity(f"conv_sweep B=1024 {mode}: weight gradient, error on 8 scattered images",
                         dk.cpu().numpy().reshape(K, -1), dko.astype(np.float64).sum(0), mko.astype(np.float64).sum(0))
    assert e <= tol and sv <= PARITY_BOUNDS[mode], (e, sv)
    assert np.allclose(db.cpu().numpy().reshape(K), dbo.astype(np.float64).sum(0), rtol=1e-5, atol=1e-3)
    layer.close()


@pytest.mark.parametrize("mode,tol", MODES)
def test_dcgan_generator_full_size(ops, port_mt, mode, tol):
    """Linear 100 -> 512x4x4, transposed convolutions 256, 128, 64, 3 to 3x64x64, batch 64."""
    from cuda_cnn_gan_vae_b200.nets import dcgan_generator
    _mode(ops, mode)
    nets_tests.REPORT_PREFIX = f"dcgan generator B=64 {mode}: "
    B = 64
    net = dcgan_generator(B)
    assert net.out_shape == (3, 64, 64)
    rng = np.random.default_rng(2)
    z = rng.standard_normal((B, 1, 100, 1)).astype(np.float32)
    error = rng.standard_normal((B, 3, 64, 64)).astype(np.float32)
    nets_tests.run_and_compare(ops, port_mt, net, z, error, tol, True)


@pytest.mark.parametrize("mode,tol", MODES)
def test_dcgan_discriminator_full_size(ops, port_mt, mode, tol):
    """Convolutions 64, 128, 256, 512 on 3x64x64 images, Linear to one logit, batch 64, error = sigmoid(out) - label."""
    from cuda_cnn_gan_vae_b200.nets import dcgan_discriminator
    _mode(ops, mode)
    nets_tests.REPORT_PREFIX = f"dcgan discriminator B=64 {mode}: "
    B = 64
    net = dcgan_discriminator(B)
    rng = np.random.default_rng(3)
    x = rng.uniform(-1, 1, (B, 3, 64, 64)).astype(np.float32)
    labels = rng.integers(0, 2, (B, 1, 1, 1)).astype(np.float32)
    out = net.Forward(torch.from_numpy(x).cuda()).cpu().numpy()
    nets_tests.run_and_compare(ops, port_mt, net, x, (out - labels).astype(np.float32), tol, True, need_input_error=True)


@pytest.mark.parametrize("mode,tol", MODES)
def test_vae_chains_full_size(ops, port_mt, mode, tol):
    """Encoder and decoder of the VAE configuration at 3x128x128 with widths 32, 64, 128, 256 (batch 32)."""
    from cuda_cnn_gan_vae_b200.nets import vae_decoder, vae_encoder
    _mode(ops, mode)
    B = 32
    rng = np.random.default_rng(4)
    nets_tests.REPORT_PREFIX = f"vae encoder B=32 {mode}: "
    enc = vae_encoder(B)
    assert enc.out_shape == (256, 8, 8)
    x = rng.uniform(0, 1, (B, 3, 128, 128)).astype(np.float32)
    nets_tests.run_and_compare(ops, port_mt, enc, x, rng.standard_normal((B, 256, 8, 8)).astype(np.float32), tol, True, need_input_error=True)
    nets_tests.REPORT_PREFIX = f"vae decoder B=32 {mode}: "
    dec = vae_decoder(B)
    assert dec.out_shape == (3, 128, 128)
    z = rng.standard_normal((B, 1, 256, 1)).astype(np.float32)
    nets_tests.run_and_compare(ops, port_mt, dec, z, rng.standard_normal((B, 3, 128, 128)).astype(np.float32), tol, True, need_input_error=True)
