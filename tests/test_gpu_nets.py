"""The layer chains of the DCGAN configurations (generator: Linear + transposed convolutions, discriminator:
convolutions + Linear, both with batch normalisation and activations) on the GPU against the CPU twin built from the
oracle's tensor routines (oracle/net_twin.py), layer by layer: outputs, errors handed down, weight gradients, and the
Adam update of the whole parameter arena."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle.net_twin import OracleNet  # noqa: E402
from tests.util import TOL_X3, record_parity  # noqa: E402


@pytest.fixture(scope="module")
def ops():
    from cuda_cnn_gan_vae_b200 import ops as o
    assert torch.cuda.is_available()
    yield o
    o.set_precision(o.TF32X3)


REPORT_PREFIX = ""       # set by the full-size tests: comparisons are then also recorded for the parity report


def check(name, got, want, tol, strict, mag=None):
    """mag: the same sum over absolute values, the scale of the error when the sum itself cancels.  strict: every
    element within tol of the RMS-scaled expectation.  Otherwise (batch normalisation over a handful of samples can
    turn a 1e-6 difference into a large one at isolated elements of small variance): RMS error within tol and at most
    0.01 % of elements beyond 10 tol."""
    got, want = np.asarray(got, np.float64).ravel(), np.asarray(want, np.float64).ravel()
    assert got.shape == want.shape, name
    assert np.isfinite(got).all(), name
    if REPORT_PREFIX:
        record_parity(REPORT_PREFIX + name, got, want, None if mag is None else np.maximum(np.asarray(mag, np.float64).ravel(), 1e-30))
    scale = np.sqrt(np.mean(want ** 2)) + 1e-30
    if mag is not None:
        scale = max(scale, np.sqrt(np.mean(np.asarray(mag, np.float64) ** 2)))
    err = np.abs(got - want) / scale
    if strict:
        assert err.max() <= tol, (name, err.max())
    else:
        assert np.sqrt(np.mean(err ** 2)) <= tol, (name, np.sqrt(np.mean(err ** 2)))
        assert np.mean(err > 10 * tol) <= 1e-4, (name, np.mean(err > 10 * tol), err.max())


def run_and_compare(ops, port, net, x, error, tol, strict, need_input_error=False):
    """Every layer of the chain is compared on the operands the GPU chain actually fed it (its input on the way up, the
    error from above on the way down), so each comparison is one layer operation against the oracle's, and a LeakyReLU
    input that rounding puts on the other side of zero cannot carry a step of the derivative into the layers below.
    The free-running twin is compared at the net's output (the forward pass is continuous)."""
    twin = OracleNet(port, net)
    B = x.shape[0]
    net.TrainingResetDeltaWeight()
    cur = torch.from_numpy(x).cuda()
    for layer in net.layers:
        cur = layer.Forward(cur.view((B,) + layer.in_shape))
    out = cur.cpu().numpy()
    # the input of layer i is the output tensor of layer i-1 (a function layer folded into the convolution layer behind it
    # passes its own input on and lets that layer write its output tensor)
    inputs = [x] + [layer.H.cpu().numpy().reshape((B,) + nxt.in_shape) for layer, nxt in zip(net.layers[:-1], net.layers[1:])]
    errors_in, errors_out, cur = [None] * len(net.layers), [None] * len(net.layers), torch.from_numpy(error).cuda()
    for i in range(len(net.layers) - 1, -1, -1):
        layer = net.layers[i]
        cur = cur.view((B,) + layer.out_shape)
        errors_in[i] = cur.cpu().numpy()
        cur = layer.TrainingBackward(cur, True, need_prev=(i > 0 or need_input_error))
        errors_out[i] = cur.cpu().numpy() if cur is not None else None
    ops.stream_status()
    check("net output, free-running twin", out, twin.forward(x), 10 * tol, False)
    # the same contractions on absolute values: sum |a||b|, the scale the rounding error of a dot product is bounded by
    # (the tensor core's fp32 accumulator adds an error that grows with the length of the contraction)
    mags = OracleNet(port, net, absolute=True)
    contraction = lambda layer: type(layer).__name__ in ("NetLayerConvolution", "NetLayerBackConvolution", "NetLayerLinear")
    for i, layer in enumerate(net.layers):
        name = "layer %d %s" % (i, type(layer).__name__)
        want = twin.forward_layer(i, inputs[i])
        mag = mags.forward_layer(i, np.abs(inputs[i])) if contraction(layer) else None
        check("output of " + name, layer.H.cpu().numpy(), want, tol, strict, mag)
    for i in range(len(net.layers) - 1, -1, -1):
        layer = net.layers[i]
        name = "layer %d %s" % (i, type(layer).__name__)
        need = i > 0 or need_input_error
        want = twin.backward_layer(i, errors_in[i], need)
        mag = mags.backward_layer(i, np.abs(errors_in[i]), need) if contraction(layer) else None
        if need:
            check("error below " + name, errors_out[i], want, tol, strict, mag)
        for pname in layer.param_shapes():
            want = twin.grads[i][pname]
            if not want.any():
                assert not layer.g[pname].cpu().numpy().any(), (name, pname)
                continue
            mag = mags.grads[i][pname] if contraction(layer) else twin.grad_mag[i].get(pname)
            check("gradient %s of %s" % (pname, name), layer.g[pname].cpu().numpy(), want, tol, strict, mag)
    return twin


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("mode", ["fp32", "x3"])
def test_dcgan_discriminator_chain(ops, port, mode, fused):
    from cuda_cnn_gan_vae_b200.nets import dcgan_discriminator
    ops.set_precision(ops.FP32 if mode == "fp32" else ops.TF32X3)
    B = 8
    net = dcgan_discriminator(B, image=(3, 32, 32), widths=(16, 32, 64), leaky_slope=0.1 if mode == "fp32" else 0.2, fused=fused)
    rng = np.random.default_rng(3)
    x = rng.uniform(-1, 1, (B, 3, 32, 32)).astype(np.float32)
    labels = rng.integers(0, 2, (B, 1, 1, 1)).astype(np.float32)
    out = net.Forward(torch.from_numpy(x).cuda()).cpu().numpy()
    error = (out - labels).astype(np.float32)
    run_and_compare(ops, port, net, x, error, 2e-5 if mode == "fp32" else TOL_X3, True, need_input_error=True)


@pytest.mark.parametrize("mode", ["fp32", "x3"])
def test_dcgan_generator_chain(ops, port, mode):
    from cuda_cnn_gan_vae_b200.nets import dcgan_generator
    ops.set_precision(ops.FP32 if mode == "fp32" else ops.TF32X3)
    B = 8
    net = dcgan_generator(B, noise=20, base=64, widths=(32, 16, 3), leaky_slope=0.1 if mode == "fp32" else 0.2)
    assert net.out_shape == (3, 32, 32)
    rng = np.random.default_rng(2)
    z = rng.standard_normal((B, 1, 20, 1)).astype(np.float32)
    error = rng.standard_normal((B, 3, 32, 32)).astype(np.float32)
    run_and_compare(ops, port, net, z, error, 2e-5 if mode == "fp32" else TOL_X3, True)


def test_adam_over_the_parameter_arena(ops, port):
    from cuda_cnn_gan_vae_b200.nets import dcgan_generator
    ops.set_precision(ops.TF32X3)
    B = 4
    net = dcgan_generator(B, noise=20, base=64, widths=(32, 16, 3))
    rng = np.random.default_rng(5)
    net.TrainingResetDeltaWeight()
    net.Forward(torch.from_numpy(rng.standard_normal((B, 1, 20, 1)).astype(np.float32)).cuda())
    net.TrainingBackward(torch.from_numpy(rng.standard_normal((B, 3, 32, 32)).astype(np.float32)).cuda(), True)
    w0, g = net.weights.buffer.cpu().numpy().copy(), net.grads.buffer.cpu().numpy().copy()
    zeros = np.zeros_like(w0)
    net.TrainingUpdateWeight(2e-4, 1, batch_scale=2)
    ops.stream_status()
    want_w, want_m, want_v = port.adam(w0, g, zeros, zeros, B * 2, 2e-4, 0.9, 0.999, 1e-8, 1)
    assert np.allclose(net.weights.buffer.cpu().numpy(), want_w, rtol=0, atol=1e-7)
    assert np.allclose(net.m.buffer.cpu().numpy(), want_m, rtol=1e-6, atol=1e-12)
    assert np.allclose(net.v.buffer.cpu().numpy(), want_v, rtol=1e-6, atol=1e-20)
    assert np.abs(net.weights.buffer.cpu().numpy() - w0).max() > 1e-5


def test_moving_average_of_the_weights(ops, port):
    """EnableEMA / SetUseEMA of the layers (netlayer/cnetlayerconvolution.cu.h:547-551, 622-634; inetlayer.cu.h:97-101): the
    averaged weights follow every update and Forward can be switched over to them."""
    from cuda_cnn_gan_vae_b200.nets import dcgan_generator
    ops.set_precision(ops.FP32)
    B = 4
    net = dcgan_generator(B, noise=20, base=64, widths=(32, 16, 3))
    net.EnableEMA(True, 0.9)
    rng = np.random.default_rng(6)
    z = torch.from_numpy(rng.standard_normal((B, 1, 20, 1)).astype(np.float32)).cuda()
    err = torch.from_numpy(rng.standard_normal((B, 3, 32, 32)).astype(np.float32)).cuda()
    ema = net.weights.buffer.cpu().numpy().copy()
    for it in (1, 2):
        net.TrainingResetDeltaWeight()
        net.Forward(z)
        net.TrainingBackward(err, True)
        net.TrainingUpdateWeight(1e-2, it)
        w = net.weights.buffer.cpu().numpy()
        ema = port.binary("add", ema.reshape(1, 1, 1, -1), w.reshape(1, 1, 1, -1), 0.9, 1.0 - 0.9).ravel()
        assert net.ema.buffer.cpu().numpy().tobytes() == ema.tobytes()
    out_w = net.Forward(z).clone()
    net.SetUseEMA(True)
    out_e = net.Forward(z).clone()
    net.SetUseEMA(False)
    assert torch.equal(net.Forward(z), out_w) and not torch.equal(out_e, out_w)
    # the same forward pass with the averaged weights copied into the weight arena
    net.weights.buffer.copy_(net.ema.buffer)
    assert torch.equal(net.Forward(z), out_e)
    net.EnableEMA(False)
    assert net.ema is None
    ops.stream_status()


@pytest.mark.parametrize("mode", ["fp32", "x3", "tf32"])
def test_folded_function_layers_change_nothing(ops, mode):
    """Nets with their function layers folded into the neighbouring convolution layers (default), folded without writing the
    function layers' own outputs, and not folded at all give bit-identical outputs, input errors and gradients."""
    from cuda_cnn_gan_vae_b200.nets import dcgan_discriminator, dcgan_generator, vae_encoder
    ops.set_precision({"fp32": ops.FP32, "x3": ops.TF32X3, "tf32": ops.TF32}[mode])
    B = 8
    rng = np.random.default_rng(12)
    from cuda_cnn_gan_vae_b200.layers import Net, NetLayerConvolution, NetLayerFunction, NetLayerMaxPooling
    # the last: a contraction long enough (128 channels x 3 x 3 taps) for the function layer behind it to go into the epilogue
    long_conv = [(NetLayerConvolution, dict(kernel_amount=16, kernel_size=3, stride=1, padding=1)), (NetLayerFunction, dict(func="leaky_relu", leaky_slope=0.2)),
                 (NetLayerMaxPooling, dict(pooling=2)), (NetLayerConvolution, dict(kernel_amount=24, kernel_size=3, stride=1, padding=1)),
                 (NetLayerFunction, dict(func="tanh"))]
    builders = [(lambda: dcgan_discriminator(B, image=(3, 32, 32), widths=(16, 32, 64)), (B, 3, 32, 32), True),
                (lambda: dcgan_generator(B, noise=20, base=64, widths=(32, 16, 3)), (B, 1, 20, 1), True),
                (lambda: vae_encoder(B, image=(3, 32, 32), widths=(8, 16, 32)), (B, 3, 32, 32), False),       # short contractions: nothing to fold
                (lambda: Net((128, 8, 8), B, long_conv, seed=9), (B, 128, 8, 8), True)]
    for build, in_shape, expect_folds in builders:
        x = torch.from_numpy(rng.uniform(-1, 1, in_shape).astype(np.float32)).cuda()
        results = []
        for variant in ("folded", "lean", "separate"):
            net = build()
            net.fold_functions(variant != "separate", materialise=(variant != "lean"))
            folded = sum(1 for l in net.layers if getattr(l, "folded", None))
            assert (folded > 0) == (variant != "separate" and expect_folds)
            err = torch.from_numpy(np.random.default_rng(13).standard_normal((B,) + net.out_shape).astype(np.float32)).cuda()
            net.TrainingResetDeltaWeight()
            out = net.Forward(x).clone()
            d_in = net.TrainingBackward(err, True, need_input_error=True).clone()
            ops.stream_status()
            results.append((out, d_in, net.grads.buffer.clone()))
        for other in results[1:]:
            for a, b in zip(results[0], other):
                assert torch.equal(a, b)


def test_dcgan_step_graph_replay_matches_eager(ops):
    """The combined step replayed from its CUDA graph gives the same weights and outputs as the eager launches."""
    from cuda_cnn_gan_vae_b200.nets import DCGANStep
    ops.set_precision(ops.TF32X3)
    B = 8
    kw = dict(widths_g=(32, 16, 3), widths_d=(16, 32, 64), base=64, noise=20)
    rng = np.random.default_rng(9)
    z = torch.from_numpy(rng.standard_normal((B, 1, 20, 1)).astype(np.float32)).cuda()
    labels = torch.from_numpy(rng.integers(0, 2, (B, 1, 1, 1)).astype(np.float32)).cuda()
    results = []
    for use_graph in (False, True):
        step = DCGANStep(B, use_graph=use_graph, **kw)
        assert step.G.out_shape == (3, 32, 32)
        outs = [step(z, labels).cpu().numpy().copy() for _ in range(6)]
        ops.stream_status()
        assert (step.graph is not None) == use_graph
        results.append((outs, step.G.weights.buffer.cpu().numpy(), step.D.weights.buffer.cpu().numpy()))
    (eo, eg, ed), (go, gg, gd) = results
    assert not np.array_equal(eo[0], eo[5])                    # the weights do move
    for a, b in zip(eo, go):
        assert np.array_equal(a, b)
    assert np.array_equal(eg, gg) and np.array_equal(ed, gd)


@pytest.mark.parametrize("mode", ["fp32", "x3"])
def test_vae_encoder_and_decoder_chains(ops, port, mode):
    """Convolution + LeakyReLU + max-pooling (argmax routed back) and Linear + upsampling + convolution chains."""
    from cuda_cnn_gan_vae_b200.nets import vae_decoder, vae_encoder
    ops.set_precision(ops.FP32 if mode == "fp32" else ops.TF32X3)
    tol, B = (2e-5 if mode == "fp32" else TOL_X3), 4
    rng = np.random.default_rng(4)
    enc = vae_encoder(B, image=(3, 32, 32), widths=(8, 16, 32))
    assert enc.out_shape == (32, 4, 4)
    x = rng.uniform(0, 1, (B, 3, 32, 32)).astype(np.float32)
    run_and_compare(ops, port, enc, x, rng.standard_normal((B, 32, 4, 4)).astype(np.float32), tol, True, need_input_error=True)
    dec = vae_decoder(B, latent=24, start=(32, 4, 4), widths=(16, 8, 3))
    assert dec.out_shape == (3, 32, 32)
    z = rng.standard_normal((B, 1, 24, 1)).astype(np.float32)
    run_and_compare(ops, port, dec, z, rng.standard_normal((B, 3, 32, 32)).astype(np.float32), tol, True, need_input_error=True)


def test_vae_step_matches_twin(ops, port):
    """The whole VAE step (two heads on one feature tensor, reparameterisation with supplied noise, reconstruction and
    Kullback-Leibler errors) against the same composition of oracle routines, free-running, in FP32 mode."""
    from cuda_cnn_gan_vae_b200.nets import VAEStep
    ops.set_precision(ops.FP32)
    B, image = 4, (3, 16, 16)
    step = VAEStep(B, image=image, widths=(8, 16), latent=12, kl_speed=0.5)
    twins = [OracleNet(port, net) for net in step.nets]
    rng = np.random.default_rng(8)
    x = rng.uniform(0, 1, (B,) + image).astype(np.float32)
    eps = rng.standard_normal((B, 1, 12, 1)).astype(np.float32)
    w0 = [net.weights.buffer.cpu().numpy().copy() for net in step.nets]
    x_hat = step(torch.from_numpy(x).cuda(), torch.from_numpy(eps).cuda(), want_kl=True)
    ops.stream_status()
    enc, mu_t, lv_t, dec = twins
    feat = enc.forward(x)
    mu, lv = mu_t.forward(feat), lv_t.forward(feat)
    z, kl = port.vae_forward(mu.reshape(B, -1), lv.reshape(B, -1), eps.reshape(B, -1))
    want_hat = dec.forward(z.reshape(B, 1, 12, 1))
    check("reconstruction", x_hat.cpu().numpy(), want_hat, 2e-5, True)
    assert abs(step.kl - kl) <= 1e-4 * max(1.0, abs(kl))
    n = float(np.prod(image))
    err = port.binary("sub", want_hat, x, 2.0 / n, 2.0 / n)
    d_z = dec.backward(err, need_input_error=True)
    d_mu, d_lv = port.vae_backward(d_z.reshape(B, -1), mu.reshape(B, -1), lv.reshape(B, -1), eps.reshape(B, -1), 0.5)
    e = port.binary("add", mu_t.backward(d_mu.reshape(B, 1, 12, 1), need_input_error=True),
                    lv_t.backward(d_lv.reshape(B, 1, 12, 1), need_input_error=True))
    enc.backward(e)
    check("error at the encoder output", step.feat_error.cpu().numpy(), e, 5e-5, True)
    for net, twin, before in zip(step.nets, twins, w0):
        for i, layer in enumerate(net.layers):
            for name in layer.param_shapes():
                check("gradient %d.%s" % (i, name), layer.g[name].cpu().numpy(), twin.grads[i][name], 1e-4, False, twin.grad_mag[i].get(name))
        assert np.abs(net.weights.buffer.cpu().numpy() - before).max() > 0      # Adam moved the weights


@pytest.mark.parametrize("w_n", [(16, (16, 32, 64)), (5, (8, 12, 20))])     # staged kernels (batch >= 8) and the general ones
def test_fused_normalisation_and_function_layers_are_bit_identical(ops, w_n):
    """The fused batch-normalisation + function layer gives bit for bit what the two layers give in sequence."""
    from cuda_cnn_gan_vae_b200.nets import dcgan_discriminator
    ops.set_precision(ops.FP32)
    B, widths = w_n
    rng = np.random.default_rng(21)
    x = torch.from_numpy(rng.uniform(-1, 1, (B, 3, 32, 32)).astype(np.float32)).cuda()
    err = torch.from_numpy(rng.standard_normal((B, 1, 1, 1)).astype(np.float32)).cuda()
    results = []
    for fused in (False, True):
        net = dcgan_discriminator(B, image=(3, 32, 32), widths=widths, leaky_slope=0.2, fused=fused)
        assert (len(net.layers) == 3 * len(widths) + 2) == (not fused)
        net.TrainingResetDeltaWeight()
        out = net.Forward(x).clone()
        d_in = net.TrainingBackward(err, True, need_input_error=True).clone()
        ops.stream_status()
        results.append((out, d_in, net.weights.buffer.clone(), net.grads.buffer.clone()))
    for a, b in zip(*results):
        assert torch.equal(a, b)


def test_separable_gan_iteration_matches_twin(ops, port):
    """One iteration of the reference's separable GAN training (discriminator on fakes, discriminator on real images,
    generator through the discriminator; hinge errors, three Adam updates) against the same sequence on the oracle twin."""
    from cuda_cnn_gan_vae_b200.nets import GANSeparableTrainer, dcgan_discriminator, dcgan_generator
    ops.set_precision(ops.FP32)
    B = 6
    G = dcgan_generator(B, noise=12, base=16, widths=(8, 3), leaky_slope=0.1)
    assert G.out_shape == (3, 16, 16)
    D = dcgan_discriminator(B, image=(3, 16, 16), widths=(8, 16), leaky_slope=0.1)
    D.layers.pop()                                            # the reference's hinge rules act on the Linear output, no sigmoid
    D.out_shape = D.layers[-1].out_shape
    tg, td = OracleNet(port, G), OracleNet(port, D)
    trainer = GANSeparableTrainer(G, D)
    rng = np.random.default_rng(31)
    z1, z2 = (rng.uniform(-1, 1, (B, 1, 12, 1)).astype(np.float32) for _ in range(2))
    real = rng.uniform(-1, 1, (B, 3, 16, 16)).astype(np.float32)
    answers = trainer.TrainingSeparable(torch.from_numpy(z1).cuda(), torch.from_numpy(real).cuda(), torch.from_numpy(z2).cuda(), 1e-3, 2e-3, 1)
    ops.stream_status()
    # the twin
    out = td.forward(tg.forward(z1)).reshape(B, 1, 1, 1)
    td.backward(np.where(out > -1, 1.0, 0.0).astype(np.float32))
    td.update(1e-3, 1, B)
    td.reset_gradients()
    out = td.forward(real).reshape(B, 1, 1, 1)
    td.backward(np.where(out < 1, -1.0, 0.0).astype(np.float32))
    td.update(1e-3, 1, B)
    want_answers = td.forward(tg.forward(z2))
    keep = {i: {k: v.copy() for k, v in g.items()} for i, g in enumerate(td.grads)}
    d_image = td.backward(np.full((B, 1, 1, 1), -1.0, np.float32), need_input_error=True)
    tg.backward(d_image)
    tg.update(2e-3, 1, B)
    check("discriminator answers in the generator pass", answers.cpu().numpy(), want_answers, 1e-4, True)
    for net, twin, speed in ((D, td, 1e-3), (G, tg, 2e-3)):
        for i, layer in enumerate(net.layers):
            for name in layer.param_shapes():
                got, want = layer.w[name].cpu().numpy(), twin.params[i][name]
                # Adam's first step moves a weight by speed * g / (|g| + epsilon): about the learning rate whatever the size of
                # the gradient.  A bias in front of a batch normalisation has a gradient that cancels to rounding noise (the
                # error below the normalisation sums to zero over the batch), so its step is noise of up to the learning rate
                # on both sides; every other weight must agree to a hundredth of a step.
                noise_gradient = name in ("bias", "b") and i + 1 < len(net.layers) and type(layer).__name__ != "NetLayerBackConvolution"
                tol = 2.1 * speed * 2 if noise_gradient else 0.01 * speed
                assert np.max(np.abs(got - want)) <= tol, (type(layer).__name__, name, np.max(np.abs(got - want)))
    assert keep is not None
