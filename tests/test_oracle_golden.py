"""Pins the plain-C oracle to the committed golden vectors: the reference's own known-answer tests
(cuda/ctensortest.cu.h) and seeded cases computed by the reference CPU backend.  Needs neither the
reference tree nor a GPU."""
import os

import numpy as np
import pytest

G = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def kat():
    return np.load(os.path.join(G, "reference_kat.npz"))


@pytest.fixture(scope="module")
def seeded():
    return np.load(os.path.join(G, "seeded_cases.npz"))


def test_kat_forward(port, kat):
    z = np.zeros((1, 2), np.float32)
    assert np.array_equal(port.conv_forward(kat["fwd_image"], kat["fwd_kernel"], z, 2, 2, 1, 1, 0, 0), kat["fwd_expected"])
    assert np.array_equal(port.conv_forward(kat["fwd_s2_image"], kat["fwd_s2_kernel"], z, 3, 3, 2, 2, 1, 1),
                          kat["fwd_s2_expected"])


def test_kat_wgrad(port, kat):
    B = 10
    dk, db = port.conv_wgrad(np.zeros((B, 1, 25), np.float32), np.zeros((B, 1), np.float32),
                             kat["wgrad_s2_image"], kat["wgrad_s2_delta"], 5, 5, 2, 2, 2, 2)
    assert np.array_equal(dk, kat["wgrad_s2_expected"]) and np.array_equal(db, kat["wgrad_s2_dbias"])
    dk, db = port.conv_wgrad(np.zeros((B, 1, 9), np.float32), np.zeros((B, 1), np.float32),
                             kat["wgrad_s1_image"], kat["wgrad_s1_delta"], 3, 3, 1, 1, 0, 0)
    assert np.array_equal(dk, kat["wgrad_s1_expected"]) and np.array_equal(db, kat["wgrad_s1_dbias"])


def test_kat_backward(port, kat):
    got = port.conv_backward(kat["bwd_delta"], kat["bwd_kernel"], np.zeros((1, 1), np.float32), (1, 7, 7), 5, 5, 2, 2, 2, 2)
    assert np.array_equal(got, kat["bwd_expected"])


def test_kat_mul_broadcast(port, kat):
    a = kat["mul_a"]
    for l, r in ((a, a), (a[:1], a), (a, a[:1])):
        assert np.array_equal(port.mul(l, r), kat["mul_expected"])


def test_kat_summ_xy(port):
    # ctensortest.cu.h:904-926: all-ones [8,16,s,s] sums to s*s for s = 1, 33, ... 481
    for s in range(1, 512, 32):
        out = port.summ_xy(np.ones((8, 16, s, s), np.float32))
        assert np.array_equal(out.ravel(), np.full(8 * 16, s * s, np.float32))


@pytest.mark.parametrize("name", ["c3x3", "c4x4s2", "c5x5s2", "c1x1"])
def test_seeded_conv(port, seeded, name):
    B, Cc, H, W, K, k, s, p = (int(v) for v in seeded[f"{name}_cfg"])
    x, wt, b, d = (seeded[f"{name}_{t}"] for t in "xwbd")
    assert port.conv_forward(x, wt, b, k, k, s, s, p, p).tobytes() == seeded[f"{name}_y"].tobytes()
    zb = np.zeros((1, K), np.float32)
    assert port.conv_backward(d, wt, zb, (Cc, H, W), k, k, s, s, p, p).tobytes() == seeded[f"{name}_dx"].tobytes()
    dk, db = port.conv_wgrad(np.zeros((B, K, Cc * k * k), np.float32), np.zeros((B, K), np.float32), x, d, k, k, s, s, p, p)
    assert dk.tobytes() == seeded[f"{name}_dk"].tobytes() and db.tobytes() == seeded[f"{name}_db"].tobytes()


def test_seeded_memory_bound(port, seeded):
    o, p = port.maxpool(seeded["pool_x"], 2, 2)
    assert o.tobytes() == seeded["pool_out"].tobytes() and p.tobytes() == seeded["pool_pos"].tobytes()
    assert port.maxpool_backward(seeded["pool_delta"], p, 2, 2).tobytes() == seeded["pool_back"].tobytes()
    up = port.upsample(seeded["up_x"], 2, 2)
    assert up.tobytes() == seeded["up_out"].tobytes()
    assert port.downsample(up, 2, 2).tobytes() == seeded["down_out"].tobytes()
    assert port.mul(seeded["gemm_a"], seeded["gemm_b"]).tobytes() == seeded["gemm_mul"].tobytes()
    assert port.tmul(seeded["gemm_a"], seeded["gemm_c"]).tobytes() == seeded["gemm_tmul"].tobytes()
    from oracle import Oracle
    for f in Oracle.FUNCS:
        assert port.activation(seeded["act_x"], f).tobytes() == seeded[f"act_{f}"].tobytes()
        assert port.activation(seeded["act_x"], f, True).tobytes() == seeded[f"dact_{f}"].tobytes()


def test_seeded_batchnorm_and_vae(port, seeded):
    """Fixtures generated from the reference run in the build container (tests/golden/make_golden.py): the reference's
    tensor routines in the batch-normalisation layer's order, and its VAE output layer object with the noise it drew."""
    f = port.bn_forward(seeded["bn_x"], seeded["bn_gamma"], seeded["bn_beta"], 0.9, 1e-6, np.zeros((3, 4, 5), np.float32),
                        np.ones((3, 4, 5), np.float32))
    for key in ("y", "xhat", "ivar", "mean", "var", "new_mean", "new_var"):
        assert f[key].tobytes() == seeded["bn_" + key].tobytes(), key
    dx, dg, db = port.bn_backward(seeded["bn_dy"], f["xhat"], f["ivar"], seeded["bn_gamma"])
    assert dx.tobytes() == seeded["bn_dx"].tobytes() and dg.tobytes() == seeded["bn_dgamma"].tobytes() and db.tobytes() == seeded["bn_dbeta"].tobytes()
    z, _ = port.vae_forward(seeded["vae_mu"], seeded["vae_logvar"], seeded["vae_eps"])
    assert z.tobytes() == seeded["vae_z"].tobytes()
    dmu, dlv = port.vae_backward(seeded["vae_delta"], seeded["vae_mu"], seeded["vae_logvar"], seeded["vae_eps"], float(seeded["vae_kl_speed"]))
    assert dmu.tobytes() == seeded["vae_dmu"].tobytes() and dlv.tobytes() == seeded["vae_dlogvar"].tobytes()


def test_batchnorm_restatement_properties(port):
    # closed forms in float64, next to the bit-exact comparison with the reference (test_oracle_vs_reference.py)
    r = np.random.default_rng(3)
    x = r.normal(1.5, 2.0, (16, 3, 4, 5)).astype(np.float32)
    gamma = r.normal(1, 0.1, (3, 4, 5)).astype(np.float32)
    beta = r.normal(0, 0.1, (3, 4, 5)).astype(np.float32)
    f = port.bn_forward(x, gamma, beta)
    x64 = x.astype(np.float64)
    mean, var = x64.mean(0), x64.var(0)
    xhat = (x64 - mean) / np.sqrt(var + 1e-6)
    assert np.allclose(f["xhat"], xhat, atol=2e-5)
    assert np.allclose(f["y"], gamma * xhat + beta, atol=2e-5)
    dy = r.normal(0, 1, x.shape).astype(np.float32)
    dx, dg, db = port.bn_backward(dy, f["xhat"], f["ivar"], gamma)
    dxhat = dy.astype(np.float64) * gamma
    N = x.shape[0]
    ref_dx = (1.0 / N) / np.sqrt(var + 1e-6) * (N * dxhat - dxhat.sum(0) - xhat * (dxhat * xhat).sum(0))
    assert np.allclose(dx, ref_dx, atol=5e-5)
    assert np.allclose(dg, (dy * xhat).sum(0), atol=5e-5) and np.allclose(db, dy.sum(0), atol=5e-5)


def test_vae_restatement_properties(port):
    r = np.random.default_rng(4)
    mu = r.normal(0, 1, (8, 32)).astype(np.float32)
    lv = r.normal(0, 4, (8, 32)).astype(np.float32)
    lv[0, :4] = [11, -11, 10, -10]
    eps = r.normal(0, 1, (8, 32)).astype(np.float32)
    z, kl = port.vae_forward(mu, lv, eps)
    lvc = np.clip(lv.astype(np.float64), -10, 10)
    assert np.allclose(z, mu + np.exp(lvc / 2) * eps, rtol=1e-5, atol=1e-5)
    assert np.isclose(kl, -0.5 / 8 * np.sum(1 + lvc - mu.astype(np.float64) ** 2 - np.exp(lvc)), rtol=1e-4)
    delta = r.normal(0, 1, mu.shape).astype(np.float32)
    dmu, dlv = port.vae_backward(delta, mu, lv, eps, 0.25)
    assert np.allclose(dmu, delta + mu * 0.25, atol=1e-6)
    lv64 = lv.astype(np.float64)
    assert np.allclose(dlv, delta * 0.5 * eps * np.exp(lv64 / 2) - 0.5 * (1 - np.exp(lv64)) * 0.25, rtol=2e-5, atol=1e-5)
