"""The plain-C oracle must reproduce the reference CPU backend bit for bit (same loop order, same
fp32 arithmetic) on seeded random inputs, including W-broadcast, stride, padding and ragged sizes."""
import numpy as np
import pytest

CONV_CASES = [
    # B, C, H, W, K, kx, ky, sx, sy, px, py
    (3, 3, 9, 8, 4, 3, 3, 1, 1, 1, 1),
    (2, 5, 11, 7, 3, 5, 5, 2, 2, 2, 2),
    (4, 2, 8, 8, 6, 4, 4, 2, 2, 1, 1),
    (2, 1, 6, 10, 2, 2, 3, 1, 2, 0, 1),
    (1, 4, 5, 5, 5, 1, 1, 1, 1, 0, 0),
]


def _rng(seed):
    return np.random.default_rng(seed)


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_trio_bit_exact(port, reference, case):
    B, Cc, H, W, K, kx, ky, sx, sy, px, py = case
    r = _rng(hash(case) % 1000)
    x = r.uniform(-1, 1, (B, Cc, H, W)).astype(np.float32)
    wt = r.normal(0, 0.3, (1, K, Cc * kx * ky)).astype(np.float32)
    b = r.normal(0, 1, (1, K)).astype(np.float32)
    y_p = port.conv_forward(x, wt, b, kx, ky, sx, sy, px, py)
    y_r = reference.conv_forward(x, wt, b, kx, ky, sx, sy, px, py)
    assert y_p.tobytes() == y_r.tobytes()
    d = r.normal(0, 1, y_p.shape).astype(np.float32)
    zb = np.zeros((1, K), np.float32)
    dx_p = port.conv_backward(d, wt, zb, (Cc, H, W), kx, ky, sx, sy, px, py)
    dx_r = reference.conv_backward(d, wt, zb, (Cc, H, W), kx, ky, sx, sy, px, py)
    assert dx_p.tobytes() == dx_r.tobytes()
    # non-zero bias is added once per tap and filter by the reference: keep the quirk identical
    dxb_p = port.conv_backward(d, wt, b, (Cc, H, W), kx, ky, sx, sy, px, py)
    dxb_r = reference.conv_backward(d, wt, b, (Cc, H, W), kx, ky, sx, sy, px, py)
    assert dxb_p.tobytes() == dxb_r.tobytes()
    dk0 = r.normal(0, 1, (B, K, Cc * kx * ky)).astype(np.float32)
    db0 = r.normal(0, 1, (B, K)).astype(np.float32)
    for dk, db in ((dk0, db0), (dk0[:1], db0[:1])):
        a = port.conv_wgrad(dk, db, x, d, kx, ky, sx, sy, px, py)
        c = reference.conv_wgrad(dk, db, x, d, kx, ky, sx, sy, px, py)
        assert a[0].tobytes() == c[0].tobytes() and a[1].tobytes() == c[1].tobytes()


def test_back_wgrad_bit_exact(port, reference):
    # transposed-conv layer: "image" is the layer input (K channels, small), "delta" the layer output error
    r = _rng(5)
    B, K, Cc, kx, s, p = 3, 4, 2, 4, 2, 1
    small = r.normal(0, 1, (B, K, 4, 4)).astype(np.float32)
    big = r.normal(0, 1, (B, Cc, 8, 8)).astype(np.float32)
    dk = np.zeros((B, K, Cc * kx * kx), np.float32)
    db = np.ones((B, K), np.float32)
    # CreateBackDeltaWeightAndBias(dKernel, ..., image = layer input, delta = output error) swaps the two roles internally
    a = port.conv_wgrad(dk, db, small, big, kx, kx, s, s, p, p, back_variant=True)
    c = reference.conv_wgrad(dk, db, small, big, kx, kx, s, s, p, p, back_variant=True)
    assert a[0].tobytes() == c[0].tobytes() and a[1].tobytes() == c[1].tobytes()
    assert not a[1].any()


def test_per_sample_kernels_broadcast(port, reference):
    r = _rng(7)
    x = r.normal(0, 1, (1, 2, 6, 6)).astype(np.float32)          # one image, broadcast
    wt = r.normal(0, 1, (4, 3, 2 * 9)).astype(np.float32)        # per-sample kernels
    b = r.normal(0, 1, (4, 3)).astype(np.float32)
    assert port.conv_forward(x, wt, b, 3, 3, 1, 1, 1, 1).tobytes() == \
        reference.conv_forward(x, wt, b, 3, 3, 1, 1, 1, 1).tobytes()


@pytest.mark.parametrize("shape", [(3, 2, 5, 7, 4), (1, 1, 40, 33, 70), (4, 1, 64, 1, 1), (2, 1, 1, 50, 3)])
def test_mul_tmul_bit_exact(port, reference, shape):
    W, Z, LY, LX, RX = shape
    r = _rng(sum(shape))
    a = r.normal(0, 1, (W, Z, LY, LX)).astype(np.float32)
    b = r.normal(0, 1, (W, Z, LX, RX)).astype(np.float32)
    assert port.mul(a, b).tobytes() == reference.mul(a, b).tobytes()
    assert port.mul(a[:1], b).tobytes() == reference.mul(a[:1], b).tobytes()
    assert port.mul(a, b[:1]).tobytes() == reference.mul(a, b[:1]).tobytes()
    c = r.normal(0, 1, (W, Z, LY, RX)).astype(np.float32)
    assert port.tmul(a, c).tobytes() == reference.tmul(a, c).tobytes()
    assert port.tmul(a[:1], c).tobytes() == reference.tmul(a[:1], c).tobytes()


def test_elementwise_and_reductions_bit_exact(port, reference):
    r = _rng(11)
    a = r.normal(0, 1, (5, 3, 4, 6)).astype(np.float32)
    b = r.normal(0, 1, (5, 3, 4, 6)).astype(np.float32)
    for op in ("add", "sub", "add_sum_w", "item_product"):
        for l, rr in ((a, b), (a[:1], b), (a, b[:1])):
            assert port.binary(op, l, rr, 0.5, -1.5).tobytes() == reference.binary(op, l, rr, 0.5, -1.5).tobytes(), op
    pos = np.abs(a) + 0.1
    for op, x, p, q in (("pow2", a, 0.7, 0), ("sqrt", pos, 1.3, 1e-6), ("inv", pos, 0, 0), ("scale", a, -2.5, 0)):
        assert port.unary(op, x, p, q).tobytes() == reference.unary(op, x, p, q).tobytes(), op
        assert port.unary(op, x[:1], p, q, out_w=4).tobytes() == reference.unary(op, x[:1], p, q, out_w=4).tobytes()
    bias = r.normal(0, 1, (1, 3)).astype(np.float32)
    assert port.add_bias(a, bias).tobytes() == reference.add_bias(a, bias).tobytes()
    assert port.summ_xy(a).tobytes() == reference.summ_xy(a).tobytes()


def test_pool_and_resample_bit_exact(port, reference):
    r = _rng(13)
    x = r.integers(-3, 4, (3, 4, 8, 12)).astype(np.float32)   # many ties: argmax must pick the first
    for px, py in ((2, 2), (3, 2), (4, 4)):
        o_p, p_p = port.maxpool(x, px, py)
        o_r, p_r = reference.maxpool(x, px, py)
        assert o_p.tobytes() == o_r.tobytes() and p_p.tobytes() == p_r.tobytes()
        d = r.normal(0, 1, o_p.shape).astype(np.float32)
        ys, xs = o_p.shape[2] * py, o_p.shape[3] * px
        assert port.maxpool_backward(d, p_p, px, py).tobytes() == reference.maxpool_backward(d, p_r, px, py).tobytes()
    xf = r.normal(0, 1, (2, 3, 5, 6)).astype(np.float32)
    assert port.upsample(xf, 2, 3).tobytes() == reference.upsample(xf, 2, 3).tobytes()
    big = r.normal(0, 1, (2, 3, 6, 8)).astype(np.float32)
    assert port.downsample(big, 2, 3).tobytes() == reference.downsample(big, 2, 3).tobytes()


@pytest.mark.parametrize("func", ["sigmoid", "relu", "leaky_relu", "linear", "tanh", "gelu"])
def test_activations_bit_exact(port, reference, func):
    x = np.concatenate([np.linspace(-40, 40, 2001), [0.0, -0.0, 30.0, -30.0, 30.5, -31]]).astype(np.float32)
    x = x.reshape(1, 1, 1, -1)
    for d in (False, True):
        a, b = port.activation(x, func, d), reference.activation(x, func, d)
        assert a.tobytes() == b.tobytes(), (func, d, np.abs(a - b).max())


def test_adam_bit_exact(port, reference):
    r = _rng(17)
    w, dw = r.normal(0, 1, 300).astype(np.float32), r.normal(0, 1, 300).astype(np.float32)
    m, v = r.normal(0, .1, 300).astype(np.float32), np.abs(r.normal(0, .1, 300)).astype(np.float32)
    a = port.adam(w, dw, m, v, 16, 2e-4, 0.5, 0.999, 1e-8, 3)
    b = reference.adam(w, dw, m, v, 16, 2e-4, 0.5, 0.999, 1e-8, 3)
    for p, q in zip(a, b):
        assert p.tobytes() == q.tobytes()


@pytest.mark.parametrize("shape", [(16, 3, 4, 5), (64, 2, 3, 7), (5, 1, 1, 9)])
def test_batch_normalisation_sequence_bit_exact(port, reference, shape):
    """The batch-normalisation layer's forward and backward passes: the restatement against the reference's own tensor
    routines driven in the layer's order (netlayer/cnetlayerbatchnormalization.cu.h:301-379, 578-604)."""
    r = _rng(sum(shape))
    x = r.normal(1.5, 2.0, shape).astype(np.float32)
    gamma = r.normal(1, 0.2, shape[1:]).astype(np.float32)
    beta = r.normal(0, 0.3, shape[1:]).astype(np.float32)
    nm = r.normal(0, 1, shape[1:]).astype(np.float32)
    nv = np.abs(r.normal(1, 0.2, shape[1:])).astype(np.float32)
    a = port.bn_forward(x, gamma, beta, 0.9, 1e-6, nm, nv)
    b = reference.bn_forward(x, gamma, beta, 0.9, 1e-6, nm, nv)
    for key in ("y", "xhat", "ivar", "mean", "var", "new_mean", "new_var"):
        assert a[key].tobytes() == b[key].tobytes(), key
    dy = r.normal(0, 1, shape).astype(np.float32)
    dg0 = r.normal(0, 1, shape[1:]).astype(np.float32)
    db0 = r.normal(0, 1, shape[1:]).astype(np.float32)
    pa = port.bn_backward(dy, a["xhat"], a["ivar"], gamma, dg0, db0)
    pb = reference.bn_backward(dy, a["xhat"], a["ivar"], gamma, dg0, db0)
    for p, q, key in zip(pa, pb, ("dx", "dgamma", "dbeta")):
        assert p.tobytes() == q.tobytes(), key


@pytest.mark.parametrize("kl_speed", [0.0, 0.25, 1.0])
def test_vae_output_layer_bit_exact(port, reference, kl_speed):
    """The reference's own CNetLayerVAECoderOutput<float> object (netlayer/cnetlayervaecoderoutput.cu.h:244-287, 424-460) runs
    Forward and SetOutputError; the restatement, given the noise that object drew, must reproduce its output and the two
    errors bit for bit, including log-variances beyond the clamp at +-10."""
    r = _rng(23)
    mu = r.normal(0, 1, (6, 1, 40, 1)).astype(np.float32)
    lv = r.normal(0, 4, (6, 1, 40, 1)).astype(np.float32)
    lv[0, 0, :4, 0] = [11, -11, 10, -10]
    delta = r.normal(0, 1, mu.shape).astype(np.float32)
    z, eps, dmu, dlv = reference.vae_layer(mu, lv, delta, kl_speed)
    assert np.isfinite(eps).all() and eps.std() > 0.5
    zp, _ = port.vae_forward(mu, lv, eps)
    assert zp.tobytes() == z.tobytes()
    pmu, plv = port.vae_backward(delta, mu, lv, eps, kl_speed)
    assert pmu.tobytes() == dmu.tobytes() and plv.tobytes() == dlv.tobytes()
