"""The diffusion model's tensor helpers and the two layers built on them (time embedding, concatenator), through the
C-ABI.  The reference has SetTimeStep / GetNoiseImageAndNoise / SetNormalNoise / CreateDropOutMatrix on its CUDA backend
only, so the expectation is the checker's restatement of those kernels (not pinned to a reference run); the random
streams are checked against an independent numpy statement of Philox4x32-10, itself checked against the generator's
published known-answer vectors."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from cuda_cnn_gan_vae_b200 import ops as o
    return o


def philox4x32_10(counter, key):
    """counter: uint32 array [n, 4], key: (k0, k1).  Salmon et al. 2011; ten rounds."""
    c = counter.astype(np.uint64)
    k0, k1 = np.uint64(key[0]), np.uint64(key[1])
    m0, m1, mask = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57), np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0, p1 = m0 * c[:, 0], m1 * c[:, 2]
        c = np.stack([(p1 >> np.uint64(32)) ^ c[:, 1] ^ k0, p1 & mask, (p0 >> np.uint64(32)) ^ c[:, 3] ^ k1, p0 & mask], 1)
        k0, k1 = (k0 + np.uint64(0x9E3779B9)) & mask, (k1 + np.uint64(0xBB67AE85)) & mask
    return c.astype(np.uint32)


def test_philox_statement_known_answers():
    z = philox4x32_10(np.zeros((1, 4), np.uint32), (0, 0))[0]
    assert [hex(int(v)) for v in z] == ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]
    f = philox4x32_10(np.full((1, 4), 0xFFFFFFFF, np.uint32), (0xFFFFFFFF, 0xFFFFFFFF))[0]
    assert [hex(int(v)) for v in f] == ["0x408f276d", "0x41c83b0e", "0xa20bc7c6", "0x6d5451fd"]


def _uniform(bits):
    return ((bits >> 8).astype(np.float32) + np.float32(1)) * np.float32(1.0 / 16777216.0)


def _normals(n, seed):
    groups = (n + 3) // 4
    ctr = np.zeros((groups, 4), np.uint32)
    ctr[:, 0] = np.arange(groups) & 0xFFFFFFFF
    r = philox4x32_10(ctr, (seed & 0xFFFFFFFF, seed >> 32))
    u = _uniform(r).astype(np.float64)
    out = np.empty((groups, 4))
    for j in range(2):
        radius = np.sqrt(-2.0 * np.log(u[:, 2 * j]))
        out[:, 2 * j] = radius * np.cos(2 * np.pi * u[:, 2 * j + 1])
        out[:, 2 * j + 1] = radius * np.sin(2 * np.pi * u[:, 2 * j + 1])
    return out.ravel()[:n], u.ravel()[:n]


def test_normal_noise_stream(ops):
    n, seed = 100003, 0x1234ABCD5678
    a = torch.empty(1, 1, 1, n, device="cuda")
    ops.CTensorMath.SetNormalNoise(a, seed)
    want, _ = _normals(n, seed)
    got = a.cpu().numpy().ravel()
    assert np.max(np.abs(got - want)) <= 2e-5            # device logf / sincospif against float64
    assert abs(got.mean()) < 0.02 and abs(got.std() - 1) < 0.02
    b = torch.empty_like(a)
    ops.CTensorMath.SetNormalNoise(b, seed)
    assert torch.equal(a, b)
    ops.CTensorMath.SetNormalNoise(b, seed + 1)
    assert not torch.equal(a, b)


def test_dropout_mask(ops):
    n, seed, p = 40001, 77, 0.3
    m = torch.empty(1, 1, 1, n, device="cuda")
    ops.CTensorMath.CreateDropOutMatrix(m, p, seed)
    groups = (n + 3) // 4
    ctr = np.zeros((groups, 4), np.uint32)
    ctr[:, 0] = np.arange(groups)
    u = _uniform(philox4x32_10(ctr, (seed, 0))).ravel()[:n]
    want = np.where(u > np.float32(p), np.float32(1.0 / (1.0 - p)), np.float32(0))
    assert np.array_equal(m.cpu().numpy().ravel(), want)
    assert abs((want == 0).mean() - p) < 0.02


def test_set_time_step_and_time_embedding_layer(ops, port):
    from cuda_cnn_gan_vae_b200.layers import NetLayerTimeEmbedding
    r = np.random.default_rng(5)
    B, shape = 6, (3, 8, 10)
    x = r.normal(0, 1, (B,) + shape).astype(np.float32)
    steps = np.array([0, 1, 17, 250, 999, 4], np.uint32)
    layer = NetLayerTimeEmbedding(shape, B)
    for i, t in enumerate(steps):
        layer.SetTimeStep(i, t)
    out = layer.Forward(torch.from_numpy(x).cuda())
    want = port.set_time_step(x, steps)
    # the device's powf is accurate to a few units in the last place of the ANGLE, so the sine / cosine of a sample with
    # time step t may be off by ~1e-6 * t: the bound scales with the time step
    bound = (4e-6 * (1.0 + steps.astype(np.float64))).reshape(B, 1, 1, 1)
    assert np.all(np.abs(out.cpu().numpy().astype(np.float64) - want) <= bound)
    err = torch.from_numpy(r.normal(0, 1, (B,) + shape).astype(np.float32)).cuda()
    assert layer.TrainingBackward(err) is err
    with pytest.raises(ops.B200Error):
        ops.CTensorMath.SetTimeStep(out, torch.zeros(B, 3, 8, 9, device="cuda"), layer.time_line)


def test_noisy_image(ops, port):
    r = np.random.default_rng(6)
    B, shape = 5, (3, 16, 12)
    image = r.uniform(-1, 1, (B,) + shape).astype(np.float32)
    noise = r.normal(0, 1, (B,) + shape).astype(np.float32)
    sa = r.uniform(0.1, 1, (B, 1, 1, 1)).astype(np.float32)
    so = np.sqrt(1 - sa * sa).astype(np.float32)
    I, N, SA, SO = (torch.from_numpy(a).cuda() for a in (image, noise, sa, so))
    noisy = torch.empty_like(I)
    ops.CTensorMath.GetNoiseImageAndNoise(noisy, N, I, SA, SO)
    assert noisy.cpu().numpy().tobytes() == port.noisy_image(image, noise, sa, so).tobytes()
    # noise drawn inside the call: the same stream as SetNormalNoise, and the image built from it
    drawn, ref = torch.empty_like(I), torch.empty_like(I)
    ops.CTensorMath.GetNoiseImageAndNoise(noisy, drawn, I, SA, SO, seed=99)
    ops.CTensorMath.SetNormalNoise(ref, 99)
    assert torch.equal(drawn, ref)
    assert noisy.cpu().numpy().tobytes() == port.noisy_image(image, drawn.cpu().numpy(), sa, so).tobytes()


def test_concatenator_layer(ops):
    from cuda_cnn_gan_vae_b200.layers import NetLayerConcatenator
    B = 4
    a = torch.randn(B, 3, 5, 7, device="cuda")
    b = torch.randn(B, 6, 5, 7, device="cuda")
    layer = NetLayerConcatenator((3, 5, 7), (6, 5, 7), B)
    out = layer.Forward(a, b)
    assert torch.equal(out, torch.cat([a, b], 1))
    ea, eb = layer.TrainingBackward(out)
    assert torch.equal(ea, a) and torch.equal(eb, b)
    with pytest.raises(ops.B200Error):
        NetLayerConcatenator((3, 5, 7), (6, 5, 8), B)
