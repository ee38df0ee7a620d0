"""The C++ drop-in on the GPU: the reference's own programs compiled against this package's headers.

oracle/_ref/dropin/ holds (built by cuda_cnn_gan_vae_b200/host/build_dropin.py where the reference tree exists)
  dropin_kat         the reference's known-answer suite cuda/ctensortest.cu.h, unmodified, over host/cuda/*.cu.h
  dropin_layers      the reference's unmodified layer classes (convolution input, convolution, function, linear)
                     running forward / backward / Adam / forward through libb200conv.so
  dump_cpu.txt       the same program built with -DUSE_CPU against the reference's CPU backend (the expectation)
"""
import os
import subprocess

import numpy as np
import pytest

from util import TOL_X3, TOL_TF32

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DROPIN = os.path.join(ROOT, "oracle", "_ref", "dropin")

pytestmark = pytest.mark.gpu


def _need(name):
    path = os.path.join(DROPIN, name)
    if not os.path.exists(path):
        pytest.skip("drop-in artefact not built: " + name)
    return path


def _read_dump(path):
    tensors = {}
    with open(path) as f:
        lines = f.read().split("\n")
    i = 0
    while i < len(lines):
        if lines[i].startswith("tensor "):
            _, name, count = lines[i].split()
            count = int(count)
            tensors[name] = np.array([float(v) for v in lines[i + 1:i + 1 + count]], dtype=np.float64)
            i += 1 + count
        else:
            i += 1
    return tensors


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_reference_known_answer_suite_over_the_c_abi(mode):
    """cuda/ctensortest.cu.h:CTensorTest<float>::Test() passes in every precision mode (its inputs are small integers)."""
    exe = _need("dropin_kat")
    r = subprocess.run([exe, str(mode)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "PASS" in r.stdout


@pytest.mark.parametrize("mode,tol", [(0, TOL_X3), (1, TOL_TF32), (2, 1e-5)])
def test_reference_layers_match_the_cpu_backend(tmp_path, mode, tol):
    """Forward, backward, Adam step and second forward of the reference's own layer classes agree with its CPU backend."""
    exe = _need("dropin_layers")
    want = _read_dump(_need("dump_cpu.txt"))
    out = str(tmp_path / "dump_gpu.txt")
    r = subprocess.run([exe, "run", _need("w0.net"), out, str(mode)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    got = _read_dump(out)
    assert set(got) == set(want) and len(want) == 13
    # deltas that have passed the derivative of LeakyReLU (a step from 0.1 to 1 at zero): where the convolution output lies
    # within the rounding error of zero, either side of the step is right.  The delta right below the step is compared
    # away from those elements; deltas further down receive such an element through a convolution's backward pass, so for
    # them a small fraction of elements may deviate (none do in FP32 mode).
    at_step = {"conv1_delta": "conv1_output", "up_conv_delta": "up_conv_output"}
    below_step = ("up_upsampling_delta", "up_input_delta")
    for name in want:
        assert got[name].shape == want[name].shape, name
        scale = np.sqrt(np.mean(want[name] ** 2)) + 1e-30
        diff = np.abs(got[name] - want[name]) / scale
        if name in at_step:
            out_ref = want[at_step[name]]
            keep = np.abs(out_ref) > 16 * tol * np.sqrt(np.mean(out_ref ** 2))
            assert keep.mean() > 0.9
            diff = diff[keep]
        if name in below_step and mode != 2:
            assert np.mean(diff > 4 * tol) <= (0.15 if mode == 1 else 0.01), (name, np.mean(diff > 4 * tol))
            assert np.median(diff) <= 4 * tol, (name, np.median(diff))
            continue
        assert np.max(diff) <= 4 * tol, (name, np.max(diff))


@pytest.mark.parametrize("mode,tol", [(2, 2e-5), (0, TOL_X3), (1, TOL_TF32)])
def test_own_layer_classes_match_the_cpu_twin(tmp_path, port, mode, tol):
    """host/netlayer/: this package's CNetLayerLinear, CNetLayerBackConvolution, CNetLayerBatchNormalization and
    CNetLayerConvolution (fast path: layer contexts, batch-summed gradients) chained with the reference's unmodified input and
    function layers.  The C++ program dumps its weights and every tensor of one training step; the same chain is rebuilt on
    the CPU checker from the dumped weights (the reference's transposed-convolution and batch-normalisation layer classes do
    not work at its head revision, so the expectation is the checker's sequence of the reference's tensor routines).  The
    program itself asserts that both convolution layers' backward passes ran on the tensor cores and that a checkpoint in
    the reference's format reloads into an identical network."""
    import torch
    from cuda_cnn_gan_vae_b200 import ops
    from cuda_cnn_gan_vae_b200.layers import (Net, NetLayerBackConvolution, NetLayerBatchNormalization, NetLayerConvolution, NetLayerFunction,
                                              NetLayerLinear)
    from oracle.net_twin import OracleNet
    from tests.test_gpu_nets import check as check_strict

    def check(name, got_t, want_t, tol_t, exact_t, mag=None):
        """Bit-exact mode: every element.  Tensor-core modes: the root-mean-square error only -- a rounding difference that puts
        one LeakyReLU input on the other side of zero changes isolated elements below it by O(1) in a free-running chain."""
        if exact_t:
            return check_strict(name, got_t, want_t, tol_t, True, mag)
        g, w = np.asarray(got_t, np.float64).ravel(), np.asarray(want_t, np.float64).ravel()
        scale = np.sqrt(np.mean(w ** 2)) + 1e-30
        if mag is not None:
            scale = max(scale, np.sqrt(np.mean(np.asarray(mag, np.float64) ** 2)))
        assert np.isfinite(g).all() and np.sqrt(np.mean((g - w) ** 2)) / scale <= tol_t, (name, np.sqrt(np.mean((g - w) ** 2)) / scale)

    exe = _need("dropin_fastlayers")
    dump = str(tmp_path / "dump_fast.txt")
    r = subprocess.run([exe, dump, str(tmp_path / "net.bin"), str(mode)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout[-3000:] + r.stderr[-2000:]
    got = _read_dump(dump)
    B = 16
    ops.set_precision(ops.FP32)
    net = Net((1, 20, 1), B, [(NetLayerLinear, dict(neurons=512)), ("reshape", (32, 4, 4)),
                              (NetLayerBackConvolution, dict(kernel_amount=16, kernel_size=4, stride=2, padding=1)),
                              (NetLayerBatchNormalization, dict(momentum=0.9)), (NetLayerFunction, dict(func="leaky_relu", leaky_slope=0.1)),
                              (NetLayerConvolution, dict(kernel_amount=24, kernel_size=4, stride=2, padding=1)), (NetLayerFunction, dict(func="tanh"))])
    names = {0: ("linear", ("w", "b")), 1: ("backconv", ("kernel", "bias")), 2: ("bn", ("gamma", "beta")), 4: ("conv", ("kernel", "bias"))}
    for i, (prefix, params) in names.items():
        for j, p in enumerate(params):
            view = net.layers[i].w[p]
            view.copy_(torch.from_numpy(got["%s_param%d" % (prefix, j)].astype(np.float32)).view(view.shape))
    twin = OracleNet(port, net)
    x = got["input"].astype(np.float32).reshape(B, 1, 20, 1)
    error = got["error"].astype(np.float32).reshape(B, 24, 4, 4)
    twin.forward(x)
    exact = mode == 2
    for n in range(1, 7):
        check("output of layer %d" % n, got["output_%d" % n], twin.outputs[n - 1], tol if exact else 4 * tol, exact)
    twin.backward(error)
    # Free-running comparison.  In plain TF32 the forward outputs agree to ~7e-4 (RMS), which puts a few of the 16384 inputs of
    # LeakyReLU on the other side of zero; each of them changes the derivative from 0.1 to 1, and those elements pass down
    # through the batch normalisation's backward pass (16 samples) and the transposed convolution.  Over twelve weight seeds
    # of this program the RMS error of the tensors below the step lay between 1.4e-3 and 5.4e-2 in plain TF32 (2.5e-6 at most in
    # 3xTF32, where no input changes side); the program draws its weights with a fixed seed, and the bound for plain TF32 is
    # set above that range.  The layer-by-layer comparisons on identical operands, with the tight bounds, are in
    # tests/test_gpu_nets.py and tests/test_gpu_full_size.py.
    down = 4 * tol if exact else (0.1 if mode == 1 else 16 * tol)
    for n in (1, 2, 3, 5):          # own layers: the error that arrived at their output
        check("delta at layer %d" % n, got["delta_%d" % n], twin.deltas[n], down, exact)
    for n in (4, 6):                # the reference's function layers: f'(input) * error
        check("delta of function layer %d" % n, got["delta_%d" % n], twin.deltas[n - 1], down, exact)
    for i, (prefix, params) in names.items():
        for j, p in enumerate(params):
            want = twin.grads[i][p]
            g = got["%s_gradient%d" % (prefix, j)]
            if not want.any():
                assert not g.any(), (prefix, p)
                continue
            check("gradient %s.%s" % (prefix, p), g, want, down, exact, twin.grad_mag[i].get(p))
    # Adam with iteration + 1 = 1 (the reference CUDA backend's rule): every weight moves by about the learning rate
    twin.update(0.01, 1, B)
    for i, (prefix, params) in names.items():
        for j, p in enumerate(params):
            before, after, want = got["%s_param%d" % (prefix, j)], got["updated_%s_param%d" % (prefix, j)], twin.params[i][p].ravel()
            if exact and not (prefix in ("linear", "backconv") and p in ("b", "bias")):      # biases before a normalisation: noise gradients
                assert np.max(np.abs(after - want)) <= 1e-4 * 0.01 + 1e-6, (prefix, p, np.max(np.abs(after - want)))
            assert np.max(np.abs(after - before)) <= 0.0101
    assert np.isfinite(got["output_after_update"]).all()
