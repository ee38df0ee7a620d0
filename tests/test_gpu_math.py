"""GPU parity of the dense products and of the memory-bound kernels (through the C-ABI) with the CPU oracle."""
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tests.util import TOL_TF32, TOL_X3, dot_rel_err, max_rel_err  # noqa: E402

G = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def ops():
    from cuda_cnn_gan_vae_b200 import ops as o
    yield o
    o.set_precision(o.TF32X3)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_kat_batched_mul_with_broadcast(ops):
    kat = np.load(os.path.join(G, "reference_kat.npz"))
    a = kat["mul_a"]
    for l, r in ((a, a), (a[:1], a), (a, a[:1])):
        out = torch.empty(10, 1, 2, 2, device="cuda")
        ops.CTensorMath.Mul(out, dev(l), dev(r))
        assert np.array_equal(out.cpu().numpy(), kat["mul_expected"])


def test_kat_summ_xy_all_ones(ops):
    for s in range(1, 512, 32):   # cuda/ctensortest.cu.h:904-926
        out = torch.empty(8, 16, 1, 1, device="cuda")
        ops.CTensorMath.SummXY(out, torch.ones(8, 16, s, s, device="cuda"))
        assert np.array_equal(out.cpu().numpy().ravel(), np.full(128, s * s, np.float32))


# Linear-layer products of the headline configurations (batch reduced): forward W*x, backward W^T*delta
# the last two: the VAE heads and the decoder input at the batch of the configuration (one output tile, 512 K steps: split-K)
LINEAR = [(64, 8192, 100), (16, 1, 8192), (32, 256, 16384), (32, 16384, 256), (128, 256, 16384), (128, 16384, 256)]


@pytest.mark.parametrize("shape", LINEAR)
@pytest.mark.parametrize("mode", ["x3", "tf32"])
def test_linear_layer_products(ops, port, shape, mode):
    B, out_f, in_f = shape
    ops.set_precision(ops.TF32X3 if mode == "x3" else ops.TF32)
    tol = TOL_X3 if mode == "x3" else TOL_TF32
    r = np.random.default_rng(out_f)
    Wm = r.normal(0, np.sqrt(2.0 / in_f), (1, 1, out_f, in_f)).astype(np.float32)
    x = r.normal(0, 1, (B, 1, in_f, 1)).astype(np.float32)
    d = r.normal(0, 1, (B, 1, out_f, 1)).astype(np.float32)
    h = torch.full((B, 1, out_f, 1), float("nan"), device="cuda")
    ops.CTensorMath.Mul(h, dev(Wm), dev(x))                       # cnetlayerlinear.cu.h:273
    path_f = ops.last_path()
    assert dot_rel_err(h.cpu().numpy(), port.mul(Wm, x), port.mul(np.abs(Wm), np.abs(x))) <= tol
    dx = torch.full((B, 1, in_f, 1), float("nan"), device="cuda")
    ops.CTensorMath.TransponseMul(dx, dev(Wm), dev(d))            # cnetlayerlinear.cu.h:426
    assert dot_rel_err(dx.cpu().numpy(), port.tmul(Wm, d), port.tmul(np.abs(Wm), np.abs(d))) <= tol
    if out_f * B >= 4096:
        assert path_f == ops.PATH_TCGEN05
    ops.stream_status()


@pytest.mark.parametrize("mnk", [(128, 64, 32), (384, 96, 200), (1000, 520, 100), (5, 7, 3)])
def test_plain_products(ops, port, mnk):
    m, n, k = mnk
    ops.set_precision(ops.TF32X3)
    r = np.random.default_rng(m)
    a = r.normal(0, 1, (1, 1, m, k)).astype(np.float32)
    b = r.normal(0, 1, (1, 1, k, n)).astype(np.float32)
    c = r.normal(0, 1, (1, 1, m, n)).astype(np.float32)
    out = torch.full((1, 1, m, n), float("nan"), device="cuda")
    ops.CTensorMath.Mul(out, dev(a), dev(b))
    assert dot_rel_err(out.cpu().numpy(), port.mul(a, b), port.mul(np.abs(a), np.abs(b))) <= TOL_X3
    assert max_rel_err(out.cpu().numpy(), port.mul(a, b)) <= TOL_X3
    out = torch.full((1, 1, k, n), float("nan"), device="cuda")
    ops.CTensorMath.TransponseMul(out, dev(a), dev(c))
    assert dot_rel_err(out.cpu().numpy(), port.tmul(a, c), port.tmul(np.abs(a), np.abs(c))) <= TOL_X3
    ops.stream_status()


def test_batched_products_general_path_bit_exact(ops, port):
    r = np.random.default_rng(9)
    a = r.normal(0, 1, (3, 2, 5, 7)).astype(np.float32)
    b = r.normal(0, 1, (3, 2, 7, 4)).astype(np.float32)
    out = torch.empty(3, 2, 5, 4, device="cuda")
    ops.CTensorMath.Mul(out, dev(a), dev(b))
    assert ops.last_path() == ops.PATH_SIMT
    assert out.cpu().numpy().tobytes() == port.mul(a, b).tobytes()
    ops.CTensorMath.Mul(out, dev(a[:1]), dev(b))
    assert out.cpu().numpy().tobytes() == port.mul(a[:1], b).tobytes()
    c = r.normal(0, 1, (3, 2, 5, 6)).astype(np.float32)
    out = torch.empty(3, 2, 7, 6, device="cuda")
    ops.CTensorMath.TransponseMul(out, dev(a), dev(c))
    assert out.cpu().numpy().tobytes() == port.tmul(a, c).tobytes()


def test_elementwise_bit_exact(ops, port):
    r = np.random.default_rng(11)
    for shape in ((5, 3, 4, 6), (4, 2, 3, 5)):    # vectorised and scalar tails
        a = r.normal(0, 1, shape).astype(np.float32)
        b = r.normal(0, 1, shape).astype(np.float32)
        for l, rr in ((a, b), (a[:1], b), (a, b[:1])):
            ow = max(l.shape[0], rr.shape[0])
            out = torch.empty((ow,) + shape[1:], device="cuda")
            ops.CTensorMath.Add(out, dev(l), dev(rr), 0.5, -1.5)
            assert out.cpu().numpy().tobytes() == port.binary("add", l, rr, 0.5, -1.5).tobytes()
            ops.CTensorMath.Sub(out, dev(l), dev(rr), 0.5, -1.5)
            assert out.cpu().numpy().tobytes() == port.binary("sub", l, rr, 0.5, -1.5).tobytes()
            ops.CTensorMath.TensorItemProduction(out, dev(l), dev(rr))
            assert out.cpu().numpy().tobytes() == port.binary("item_product", l, rr).tobytes()
            ops.CTensorMath.AddSumW(out, dev(l), dev(rr), 0.5, -1.5)
            assert out.cpu().numpy().tobytes() == port.binary("add_sum_w", l, rr, 0.5, -1.5).tobytes()
        pos = np.abs(a) + 0.1
        out = torch.empty(shape, device="cuda")
        ops.CTensorMath.Pow2(out, dev(a), 0.7)
        assert out.cpu().numpy().tobytes() == port.unary("pow2", a, 0.7).tobytes()
        ops.CTensorMath.SQRT(out, dev(pos), 1.3, 1e-6)
        assert out.cpu().numpy().tobytes() == port.unary("sqrt", pos, 1.3, 1e-6).tobytes()
        ops.CTensorMath.Inv(out, dev(pos))
        assert out.cpu().numpy().tobytes() == port.unary("inv", pos).tobytes()
        ops.CTensorMath.MulValue(out, dev(a), -2.5)
        assert out.cpu().numpy().tobytes() == port.unary("scale", a, -2.5).tobytes()
        bias = r.normal(0, 1, (1, shape[1], 1, 1)).astype(np.float32)
        t = dev(a)
        ops.CTensorMath.AddBias(t, dev(bias))
        assert t.cpu().numpy().tobytes() == port.add_bias(a, bias).tobytes()
        ops.CTensorMath.Fill(t, 3.25)
        assert (t.cpu().numpy() == 3.25).all()
        out = torch.empty(shape[0], shape[1], 1, 1, device="cuda")
        ops.CTensorMath.SummXY(out, dev(a))
        assert np.allclose(out.cpu().numpy(), port.summ_xy(a), rtol=1e-5, atol=1e-5)
    # AddSumW in place (the layer calls AddSumW(dK, dK, per_sample)) and an empty-ish edge: W = 1
    per = r.normal(0, 1, (6, 1, 4, 9)).astype(np.float32)
    acc = r.normal(0, 1, (1, 1, 4, 9)).astype(np.float32)
    t = dev(acc)
    ops.CTensorMath.AddSumW(t, t, dev(per))
    assert t.cpu().numpy().tobytes() == port.binary("add_sum_w", acc, per, out_w=1).tobytes()


@pytest.mark.parametrize("func", ["sigmoid", "relu", "leaky_relu", "linear", "tanh", "gelu"])
def test_activations(ops, port, func):
    x = np.concatenate([np.linspace(-40, 40, 4001), [0.0, -0.0, 30.0, -30.0, 30.5, -31]]).astype(np.float32).reshape(1, 1, 1, -1)
    X = dev(x)
    out = torch.empty_like(X)
    ops.CTensorApplyFunc.Apply(out, X, func)
    assert np.allclose(out.cpu().numpy(), port.activation(x, func), rtol=2e-6, atol=1e-6)
    ops.CTensorApplyFunc.ApplyDifferential(out, X, func)
    assert np.allclose(out.cpu().numpy(), port.activation(x, func, True), rtol=5e-6, atol=2e-6)
    err = np.random.default_rng(1).normal(0, 1, x.shape).astype(np.float32)
    ops.CTensorApplyFunc.Backward(out, X, dev(err), func)      # cnetlayerfunction.cu.h:347-358
    assert np.allclose(out.cpu().numpy(), port.activation(x, func, True) * err, rtol=5e-6, atol=2e-6)
    if func in ("relu", "leaky_relu", "linear"):                # exact where no transcendental is involved
        ops.CTensorApplyFunc.Apply(out, X, func)
        assert out.cpu().numpy().tobytes() == port.activation(x, func).tobytes()
    # the slope is a parameter of this library (the reference constant is 0.1)
    ops.CTensorApplyFunc.Apply(out, X, "leaky_relu", 0.2)
    assert np.array_equal(out.cpu().numpy(), np.where(x > 0, x, (0.2 * x.astype(np.float64)).astype(np.float32)))


def test_bias_activation_fused(ops, port):
    r = np.random.default_rng(2)
    a = r.normal(0, 1, (4, 6, 8, 8)).astype(np.float32)
    bias = r.normal(0, 1, (1, 6, 1, 1)).astype(np.float32)
    t, pre = dev(a), torch.empty(4, 6, 8, 8, device="cuda")
    ops.CTensorApplyFunc.BiasActivation(t, dev(bias), "leaky_relu", 0.1, pre)
    z = port.add_bias(a, bias)
    assert pre.cpu().numpy().tobytes() == z.tobytes()
    assert t.cpu().numpy().tobytes() == port.activation(z, "leaky_relu").tobytes()


def test_pooling_and_resampling_bit_exact(ops, port):
    r = np.random.default_rng(13)
    x = r.integers(-3, 4, (3, 4, 8, 12)).astype(np.float32)      # many ties
    for px, py in ((2, 2), (3, 2), (4, 4)):
        o, p = port.maxpool(x, px, py)
        out = torch.empty(o.shape, device="cuda")
        pos = torch.empty(p.shape, dtype=torch.int32, device="cuda")
        ops.CTensorMath.MaxPooling(out, pos, dev(x), px, py)
        assert out.cpu().numpy().tobytes() == o.tobytes()
        assert pos.cpu().numpy().tobytes() == p.tobytes()          # argmax indices bit-exact
        d = r.normal(0, 1, o.shape).astype(np.float32)
        back = torch.empty(3, 4, o.shape[2] * py, o.shape[3] * px, device="cuda")
        ops.CTensorMath.MaxPoolingBackward(back, pos, dev(d), px, py)
        assert back.cpu().numpy().tobytes() == port.maxpool_backward(d, p, px, py).tobytes()
    big = r.normal(0, 1, (8, 32, 64, 64)).astype(np.float32)       # VAE-shaped 2x2 pooling
    o, p = port.maxpool(big, 2, 2)
    out = torch.empty(o.shape, device="cuda")
    pos = torch.empty(p.shape, dtype=torch.int32, device="cuda")
    ops.CTensorMath.MaxPooling(out, pos, dev(big), 2, 2)
    assert out.cpu().numpy().tobytes() == o.tobytes() and pos.cpu().numpy().tobytes() == p.tobytes()
    xf = r.normal(0, 1, (2, 3, 5, 6)).astype(np.float32)
    up = torch.empty(2, 3, 15, 12, device="cuda")
    ops.CTensorMath.UpSampling(up, dev(xf), 2, 3)
    assert up.cpu().numpy().tobytes() == port.upsample(xf, 2, 3).tobytes()
    bigx = r.normal(0, 1, (2, 3, 6, 8)).astype(np.float32)
    down = torch.empty(2, 3, 2, 4, device="cuda")
    ops.CTensorMath.DownSampling(down, dev(bigx), 2, 3)
    assert down.cpu().numpy().tobytes() == port.downsample(bigx, 2, 3).tobytes()
    # factor 2 x 2 (the decoder's case: 8-byte vector kernels), even and odd sizes
    for shape in ((3, 5, 8, 16), (2, 3, 7, 9), (1, 2, 6, 10)):
        xs = r.normal(0, 1, shape).astype(np.float32)
        up = torch.empty(shape[0], shape[1], shape[2] * 2, shape[3] * 2, device="cuda")
        ops.CTensorMath.UpSampling(up, dev(xs), 2, 2)
        assert up.cpu().numpy().tobytes() == port.upsample(xs, 2, 2).tobytes()
        down = torch.empty(shape[0], shape[1], shape[2] // 2, shape[3] // 2, device="cuda")
        ops.CTensorMath.DownSampling(down, dev(xs), 2, 2)
        assert down.cpu().numpy().tobytes() == port.downsample(xs, 2, 2).tobytes()


@pytest.mark.parametrize("zyx", [(16, 8, 8), (5, 9, 11), (3, 7, 5)])    # rows 16-byte aligned (staged through shared memory) or not, ragged last block
@pytest.mark.parametrize("batch", [5, 24, 64, 100, 130, 330])            # every register-resident variant and the general kernel
def test_batchnorm_fused_bit_exact(ops, port, batch, zyx):
    r = np.random.default_rng(3)
    x = r.normal(1.5, 2.0, (batch,) + zyx).astype(np.float32)
    gamma = r.normal(1, 0.1, (1,) + zyx).astype(np.float32)
    beta = r.normal(0, 0.1, (1,) + zyx).astype(np.float32)
    nm = r.normal(0, 1, gamma.shape).astype(np.float32)
    nv = np.abs(r.normal(1, 0.1, gamma.shape)).astype(np.float32)
    want = port.bn_forward(x, gamma[0], beta[0], 0.9, 1e-6, nm[0], nv[0])
    NM, NV = dev(nm), dev(nv)
    got = ops.bn_forward(dev(x), dev(gamma), dev(beta), 0.9, 1e-6, NM, NV)
    for key in ("y", "xhat"):
        assert got[key].cpu().numpy().tobytes() == want[key].tobytes(), key
    for key in ("ivar", "mean", "var"):
        assert got[key].cpu().numpy().reshape(want[key].shape).tobytes() == want[key].tobytes(), key
    assert NM.cpu().numpy().reshape(want["new_mean"].shape).tobytes() == want["new_mean"].tobytes()
    assert NV.cpu().numpy().reshape(want["new_var"].shape).tobytes() == want["new_var"].tobytes()
    dy = r.normal(0, 1, x.shape).astype(np.float32)
    dg0 = r.normal(0, 1, gamma.shape).astype(np.float32)
    db0 = r.normal(0, 1, gamma.shape).astype(np.float32)
    dxo, dgo, dbo = port.bn_backward(dy, want["xhat"], want["ivar"], gamma[0], dg0[0], db0[0])
    DG, DB = dev(dg0), dev(db0)
    dx = ops.bn_backward(dev(dy), got["xhat"], got["ivar"], dev(gamma), DG, DB)
    assert dx.cpu().numpy().tobytes() == dxo.tobytes()
    assert DG.cpu().numpy().reshape(dgo.shape).tobytes() == dgo.tobytes()
    assert DB.cpu().numpy().reshape(dbo.shape).tobytes() == dbo.tobytes()


def test_vae_output_layer(ops, port):
    r = np.random.default_rng(4)
    mu = r.normal(0, 1, (128, 1, 1, 256)).astype(np.float32)
    lv = r.normal(0, 4, mu.shape).astype(np.float32)
    lv[0, 0, 0, :4] = [11, -11, 10, -10]
    eps = r.normal(0, 1, mu.shape).astype(np.float32)
    z, kl = ops.vae_forward(dev(mu), dev(lv), dev(eps))
    zo, klo = port.vae_forward(mu, lv, eps)
    assert np.allclose(z.cpu().numpy(), zo, rtol=2e-6, atol=1e-6)
    assert abs(kl - klo) <= 2e-5 * abs(klo)
    delta = r.normal(0, 1, mu.shape).astype(np.float32)
    dmu, dlv = ops.vae_backward(dev(delta), dev(mu), dev(lv), dev(eps), 0.25)
    dmo, dlo = port.vae_backward(delta, mu, lv, eps, 0.25)
    assert np.allclose(dmu.cpu().numpy(), dmo, rtol=1e-6, atol=1e-6)
    assert np.allclose(dlv.cpu().numpy(), dlo, rtol=5e-6, atol=1e-5)


@pytest.mark.parametrize("batch", [16, 48])          # reciprocal of the batch exact or not
@pytest.mark.parametrize("n", [32 * 27, 10007])       # 16-byte path with and without a scalar tail
def test_adam(ops, port, batch, n):
    """Moments bit-identical to the CPU backend; the weight, whose step is evaluated in fp32 instead of double, within one
    unit in the last place and bit-identical for nearly every element."""
    r = np.random.default_rng(17)
    shape = (1, 1, 1, n)
    w, dw = r.normal(0, 1, shape).astype(np.float32), r.normal(0, 1, shape).astype(np.float32)
    m, v = r.normal(0, .1, shape).astype(np.float32), np.abs(r.normal(0, .1, shape)).astype(np.float32)
    wo, mo, vo = port.adam(w, dw, m, v, batch, 2e-4, 0.5, 0.999, 1e-8, 3)
    W, M, V = dev(w), dev(m), dev(v)
    ops.CTensorMath.Adam(W, dev(dw), M, V, batch, 2e-4, 0.5, 0.999, 1e-8, 3)
    assert M.cpu().numpy().tobytes() == mo.reshape(shape).tobytes() and V.cpu().numpy().tobytes() == vo.reshape(shape).tobytes()
    got, want = W.cpu().numpy().ravel(), wo.ravel()
    assert np.all(np.abs(got - want) <= np.spacing(np.abs(want)))
    assert np.mean(got == want) > 0.99


def test_adam_with_moving_average(ops, port):
    """b200_adam_ema: the update followed by ema = k * ema + (1 - k) * weight (the reference's Add with scales), one launch."""
    from cuda_cnn_gan_vae_b200.lib import load
    r = np.random.default_rng(23)
    n, k = 5003, 0.999
    w, dw, e = (r.normal(0, 1, n).astype(np.float32) for _ in range(3))
    m, v = r.normal(0, .1, n).astype(np.float32), np.abs(r.normal(0, .1, n)).astype(np.float32)
    W, DW, M, V, E = dev(w), dev(dw), dev(m), dev(v), dev(e)
    ops._check(load().b200_adam_ema(ops._ptr(W), ops._ptr(DW), ops._ptr(M), ops._ptr(V), ops._ptr(E), n, 64, 1e-3, 0.9, 0.999, 1e-8, 2.0, None, k,
                                    ops._stream()))
    ops.stream_status()
    got_w = W.cpu().numpy()
    want_e = port.binary("add", e.reshape(1, 1, 1, n), got_w.reshape(1, 1, 1, n), k, 1.0 - k)
    assert E.cpu().numpy().tobytes() == want_e.ravel().tobytes()
    wo, _, _ = port.adam(w, dw, m, v, 64, 1e-3, 0.9, 0.999, 1e-8, 2.0)
    assert np.all(np.abs(got_w - wo.ravel()) <= np.spacing(np.abs(wo.ravel())))


def test_set_clip_signum_div_transpose_bit_exact(ops):
    """Element-wise operations without an oracle entry: single IEEE operations, so numpy float32 is the expectation."""
    rng = np.random.default_rng(11)
    a = rng.standard_normal((3, 2, 37, 45)).astype(np.float32)
    b = (rng.standard_normal((1, 2, 37, 45)).astype(np.float32) + np.float32(3.0))
    A, B = dev(a), dev(b)
    out = torch.empty_like(A)
    ops.CTensorMath.Set(out, A, 1.5, -0.25)
    assert np.array_equal(out.cpu().numpy(), a * np.float32(1.5) + np.float32(-0.25))
    ops.CTensorMath.Div(out, A, B, 2.0, 0.5)
    assert np.array_equal(out.cpu().numpy(), (a * np.float32(2.0)) / (b * np.float32(0.5)))
    c = A.clone()
    ops.CTensorMath.Clip(c, -0.5, 0.75)
    assert np.array_equal(c.cpu().numpy(), np.clip(a, np.float32(-0.5), np.float32(0.75)))
    c = A.clone()
    c[0, 0, 0, 0] = 0.0
    ops.CTensorMath.Signum(c)
    want = np.sign(a)
    want[0, 0, 0, 0] = 0.0
    assert np.array_equal(c.cpu().numpy(), want)
    t = torch.empty(3, 2, 45, 37, device="cuda")
    ops.CTensorMath.Transponse(t, A)
    assert np.array_equal(t.cpu().numpy(), a.transpose(0, 1, 3, 2))
    ops.stream_status()


def test_concatenation_and_split_along_z(ops):
    rng = np.random.default_rng(12)
    a = rng.standard_normal((3, 2, 5, 7)).astype(np.float32)
    b = rng.standard_normal((1, 4, 5, 7)).astype(np.float32)          # broadcast over W
    out = torch.empty(3, 6, 5, 7, device="cuda")
    ops.CTensorMath.ConcatecationZ(out, dev(a), dev(b))
    want = np.concatenate([a, np.broadcast_to(b, (3, 4, 5, 7))], axis=1)
    assert np.array_equal(out.cpu().numpy(), want)
    pa, pb = torch.empty(3, 2, 5, 7, device="cuda"), torch.empty(3, 4, 5, 7, device="cuda")
    ops.CTensorMath.SplitZ(pa, pb, out)
    assert np.array_equal(pa.cpu().numpy(), want[:, :2]) and np.array_equal(pb.cpu().numpy(), want[:, 2:])
    with pytest.raises(ops.B200Error):
        ops.CTensorMath.ConcatecationZ(out, dev(a), dev(a))
    ops.stream_status()


def test_shape_errors_raise(ops):
    a = torch.zeros(2, 3, 4, 4, device="cuda")
    with pytest.raises(ops.B200Error):
        ops.CTensorMath.Add(a, a, torch.zeros(2, 3, 4, 5, device="cuda"))
    with pytest.raises(ops.B200Error):
        ops.CTensorConv.ForwardConvolution(torch.zeros(2, 4, 3, 3, device="cuda"), a, torch.zeros(1, 1, 4, 27, device="cuda"),
                                           3, 3, 3, 4, torch.zeros(1, 4, 1, 1, device="cuda"), 1, 1, 1, 1)   # wrong output size


def test_adam_with_device_resident_corrections(ops):
    """b200_adam_prepared (bias corrections read from device memory) gives bit for bit what b200_adam gives."""
    from cuda_cnn_gan_vae_b200.layers import AdamCorrections
    from cuda_cnn_gan_vae_b200.lib import load
    r = np.random.default_rng(19)
    n = 10007
    w, dw = r.normal(0, 1, n).astype(np.float32), r.normal(0, 1, n).astype(np.float32)
    m, v = r.normal(0, .1, n).astype(np.float32), np.abs(r.normal(0, .1, n)).astype(np.float32)
    W1, M1, V1 = dev(w).view(1, 1, 1, -1), dev(m).view(1, 1, 1, -1), dev(v).view(1, 1, 1, -1)
    ops.CTensorMath.Adam(W1, dev(dw).view(1, 1, 1, -1), M1, V1, 16, 2e-4, 0.9, 0.999, 1e-8, 7)
    W2, M2, V2, DW = dev(w), dev(m), dev(v), dev(dw)
    corr = AdamCorrections()
    c = corr.set(7)
    ops._check(load().b200_adam_prepared(ops._ptr(W2), ops._ptr(DW), ops._ptr(M2), ops._ptr(V2), n, 16, 2e-4, 0.9, 0.999, 1e-8, ops._ptr(c), ops._stream()))
    ops.stream_status()
    assert torch.equal(W1.view(-1), W2) and torch.equal(M1.view(-1), M2) and torch.equal(V1.view(-1), V2)


def test_timeout_status_is_reported_and_cleared(ops):
    """The status word a device-side wait that gave up would write is set from the host (no kernel is made to wait):
    b200_stream_status reports B200_E_TIMEOUT once, with the recorded code in the error text, and is clean again afterwards."""
    from cuda_cnn_gan_vae_b200.lib import load
    lib = load()
    ops.stream_status()
    x = torch.zeros(4, device="cuda")
    ops.CTensorMath.Fill(x.view(1, 1, 1, 4), 1.0)               # any call: the status word exists once the library ran on the device
    ops.set_precision(ops.TF32X3)
    a = torch.randn(1, 1, 64, 64, device="cuda")
    out = torch.empty(1, 1, 64, 64, device="cuda")
    ops.CTensorMath.Mul(out, a, a)                              # a tensor-core launch creates the word
    ops.stream_status()
    assert lib.b200_debug_set_status(0x304) == 0                # issuer wait, B200_E_TIMEOUT
    assert lib.b200_stream_status(None) == 4
    assert b"0x304" in lib.b200_last_error()
    assert lib.b200_stream_status(None) == 0
    ops.CTensorMath.Mul(out, a, a)                              # the context is still usable
    ops.stream_status()
