"""The layer-level calls (Forward / TrainingBackward of the convolution and transposed-convolution layers)
against the CPU oracle's sequence of tensor routines, through the C-ABI."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tests.util import TOL_TF32, TOL_X3, conv_inputs, dot_rel_err  # noqa: E402


@pytest.fixture(scope="module")
def ops():
    from cuda_cnn_gan_vae_b200 import ops as o
    yield o
    o.set_precision(o.TF32X3)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


# the last two: few output pixels and a long contraction (the 8x8 / 4x4 layers of the DCGAN nets), where the library
# splits the contraction of a tile over several work items and sums the partial outputs in a second kernel
# the last three: few filters (an RGB output layer), whose input error and weight gradient run on the mirrored problem
CASES = [(4, 64, 16, 16, 96, 3, 1, 1), (4, 3, 64, 64, 64, 4, 2, 1), (3, 40, 12, 12, 24, 3, 1, 1), (6, 128, 8, 8, 256, 4, 2, 1),
         (8, 256, 8, 8, 512, 4, 2, 1), (5, 512, 4, 4, 100, 3, 1, 1),
         (4, 32, 24, 20, 3, 3, 1, 1), (3, 16, 12, 12, 5, 4, 1, 2), (2, 24, 10, 14, 8, 3, 1, 0)]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("mode", ["x3", "tf32", "fp32"])
def test_convolution_layer(ops, port, case, mode):
    """cnetlayerconvolution.cu.h: Forward = ForwardConvolution; TrainingBackward = BackwardConvolution with a zero
    bias + per-sample CreateDeltaWeightAndBias + AddSumW into dKernel/dBias (accumulating)."""
    B, C, H, W, K, k, s, p = case
    ops.set_precision({"x3": ops.TF32X3, "tf32": ops.TF32, "fp32": ops.FP32}[mode])
    tol = {"x3": TOL_X3, "tf32": TOL_TF32, "fp32": 1e-5}[mode]
    x, wt, b, d = conv_inputs(sum(case) + 1, B, C, H, W, K, k, s, p)
    layer = ops.ConvLayer(C, H, W, K, k, k, s, s, p, p, B)
    X, WT, BI, D = dev(x), dev(wt), dev(b), dev(d)
    base_k = np.random.default_rng(1).normal(0, 1, (1, 1, K, C * k * k)).astype(np.float32)
    base_b = np.random.default_rng(2).normal(0, 1, (1, K, 1, 1)).astype(np.float32)
    zb = np.zeros((1, K), np.float32)
    ax, aw, ab, ad = np.abs(x), np.abs(wt), np.abs(b), np.abs(d)
    for rep in range(2):                       # twice: the context is reused step after step
        y = torch.full(d.shape, float("nan"), device="cuda")
        layer.forward(y, X, WT, BI)
        if mode != "fp32":
            assert ops.last_path() == ops.PATH_TCGEN05
        dx = torch.full(x.shape, float("nan"), device="cuda")
        dk, db = dev(base_k), dev(base_b)
        layer.backward(dx, dk, db, D, X, WT, accumulate=True)
        ops.stream_status()
        assert dot_rel_err(y.cpu().numpy(), port.conv_forward(x, wt[0], b.reshape(1, K), k, k, s, s, p, p),
                           port.conv_forward(ax, aw[0], ab.reshape(1, K), k, k, s, s, p, p)) <= tol
        assert dot_rel_err(dx.cpu().numpy(), port.conv_backward(d, wt[0], zb, (C, H, W), k, k, s, s, p, p),
                           port.conv_backward(ad, aw[0], zb, (C, H, W), k, k, s, s, p, p)) <= tol
        z = np.zeros((B, K, C * k * k), np.float32)
        dko, dbo = port.conv_wgrad(z, np.zeros((B, K), np.float32), x, d, k, k, s, s, p, p)
        mk, mb = port.conv_wgrad(z, np.zeros((B, K), np.float32), ax, ad, k, k, s, s, p, p)
        assert dot_rel_err(dk.cpu().numpy().reshape(K, -1), base_k.reshape(K, -1) + dko.astype(np.float64).sum(0),
                           np.abs(base_k.reshape(K, -1)) + mk.astype(np.float64).sum(0)) <= tol
        assert dot_rel_err(db.cpu().numpy().reshape(K), base_b.reshape(K) + dbo.astype(np.float64).sum(0),
                           np.abs(base_b.reshape(K)) + mb.astype(np.float64).sum(0)) <= 1e-5
    # a backward call without a preceding forward in this mode packs the input itself
    layer2 = ops.ConvLayer(C, H, W, K, k, k, s, s, p, p, B)
    dk2 = torch.zeros(1, 1, K, C * k * k, device="cuda")
    layer2.backward(None, dk2, None, D, X, WT, accumulate=False)
    ops.stream_status()
    assert dot_rel_err(dk2.cpu().numpy().reshape(K, -1), dko.astype(np.float64).sum(0), mk.astype(np.float64).sum(0)) <= tol
    layer.close()
    layer2.close()


@pytest.mark.parametrize("case", [(4, 64, 16, 16, 128, 4, 2, 1), (4, 3, 64, 64, 64, 4, 2, 1), (3, 24, 12, 12, 40, 3, 1, 1),
                                  (8, 256, 8, 8, 512, 4, 2, 1)])
@pytest.mark.parametrize("mode", ["x3", "fp32"])
def test_transposed_convolution_layer(ops, port, case, mode):
    """cnetlayerbackconvolution.cu.h: Forward = BackwardConvolution of the layer input; TrainingBackward =
    ForwardConvolution of the output error (zero bias) + CreateBackDeltaWeightAndBias (bias gradient cleared).
    case = geometry of the underlying convolution: the layer maps K x oy x ox -> C x H x W."""
    B, C, H, W, K, k, s, p = case
    ops.set_precision(ops.TF32X3 if mode == "x3" else ops.FP32)
    tol = TOL_X3 if mode == "x3" else 1e-5
    big, wt, b, small = conv_inputs(sum(case) + 2, B, C, H, W, K, k, s, p)     # small: layer input, big: layer output error
    layer = ops.ConvLayer(C, H, W, K, k, k, s, s, p, p, B, transposed=True)
    S, WT, G = dev(small), dev(wt), dev(big)
    zb = np.zeros((1, K), np.float32)
    out = torch.full(big.shape, float("nan"), device="cuda")
    layer.forward(out, S, WT)
    d_in = torch.full(small.shape, float("nan"), device="cuda")
    dk = torch.full((1, 1, K, C * k * k), float("nan"), device="cuda")
    db = torch.full((1, K, 1, 1), 3.0, device="cuda")
    layer.backward(d_in, dk, db, G, S, WT, accumulate=False)
    ops.stream_status()
    a_s, a_w, a_g = np.abs(small), np.abs(wt), np.abs(big)
    assert dot_rel_err(out.cpu().numpy(), port.conv_backward(small, wt[0], zb, (C, H, W), k, k, s, s, p, p),
                       port.conv_backward(a_s, a_w[0], zb, (C, H, W), k, k, s, s, p, p)) <= tol
    assert dot_rel_err(d_in.cpu().numpy(), port.conv_forward(big, wt[0], zb, k, k, s, s, p, p),
                       port.conv_forward(a_g, a_w[0], zb, k, k, s, s, p, p)) <= tol
    z = np.zeros((B, K, C * k * k), np.float32)
    dko, dbo = port.conv_wgrad(z, np.ones((B, K), np.float32), small, big, k, k, s, s, p, p, back_variant=True)
    mk, _ = port.conv_wgrad(z, np.ones((B, K), np.float32), a_s, a_g, k, k, s, s, p, p, back_variant=True)
    assert dot_rel_err(dk.cpu().numpy().reshape(K, -1), dko.astype(np.float64).sum(0), mk.astype(np.float64).sum(0)) <= tol
    assert not db.cpu().numpy().any() and not dbo.any()
    layer.close()


def test_split_backward_call_reuses_the_packed_error(ops):
    """Gradients-only then input-error-only calls on the same output error give what the single call gives."""
    ops.set_precision(ops.TF32X3)
    B, C, H, W, K, k, s, p = 4, 64, 16, 16, 96, 3, 1, 1
    x, wt, b, d = conv_inputs(77, B, C, H, W, K, k, s, p)
    X, WT, BI, D = dev(x), dev(wt), dev(b), dev(d)
    layer = ops.ConvLayer(C, H, W, K, k, k, s, s, p, p, B)
    y = torch.empty_like(D)
    layer.forward(y, X, WT, BI)
    dx1, dk1, db1 = torch.empty_like(X), torch.empty(1, 1, K, C * k * k, device="cuda"), torch.empty(1, K, 1, 1, device="cuda")
    layer.backward(dx1, dk1, db1, D, X, WT, accumulate=False)
    dx2, dk2, db2 = torch.full_like(X, float("nan")), torch.empty_like(dk1), torch.empty_like(db1)
    layer.forward(y, X, WT, BI)
    layer.backward(None, dk2, db2, D, X, WT, accumulate=False)
    layer.backward(dx2, None, None, D, X, WT)
    ops.stream_status()
    assert torch.equal(dx1, dx2) and torch.equal(dk1, dk2) and torch.equal(db1, db2)
    # a changed pointer is packed afresh
    D2 = D.clone() * 2
    layer.backward(None, dk2, db2, D, X, WT, accumulate=False)
    layer.backward(dx2, None, None, D2, X, WT)
    ops.stream_status()
    assert torch.allclose(dx2, 2 * dx1, rtol=1e-4, atol=1e-5)
    layer.close()


def test_few_filter_layer_in_either_call_order(ops, port):
    """A layer with few filters: the weights-only call followed by the input-only call (the order that lets the gradient
    exchange start early) gives what the combined call gives, step after step with a changing output error."""
    B, C, H, W, K, k, s, p = 4, 32, 24, 20, 3, 3, 1, 1
    ops.set_precision(ops.TF32X3)
    x, wt, b, d = conv_inputs(77, B, C, H, W, K, k, s, p)
    X, WT, BI = dev(x), dev(wt), dev(b)
    layer = ops.ConvLayer(C, H, W, K, k, k, s, s, p, p, B)
    y = torch.empty(d.shape, device="cuda")
    for rep in range(3):
        D = dev(d * (rep + 1) + rep)
        layer.forward(y, X, WT, BI)
        dx_a, dk_a, db_a = torch.empty_like(X), torch.empty_like(WT), torch.empty_like(BI)
        layer.backward(dx_a, dk_a, db_a, D, X, WT, accumulate=False)
        dx_b, dk_b, db_b = torch.full_like(X, float("nan")), torch.full_like(WT, float("nan")), torch.full_like(BI, float("nan"))
        layer.backward(None, dk_b, db_b, D, X, WT, accumulate=False)
        layer.backward(dx_b, None, None, D, X, WT)
        ops.stream_status()
        assert ops.last_path() == ops.PATH_TCGEN05
        assert torch.equal(dx_a, dx_b) and torch.equal(dk_a, dk_b) and torch.equal(db_a, db_b)
        dn = D.cpu().numpy()
        zb = np.zeros((1, K), np.float32)
        assert dot_rel_err(dx_a.cpu().numpy(), port.conv_backward(dn, wt[0], zb, (C, H, W), k, k, s, s, p, p),
                           port.conv_backward(np.abs(dn), np.abs(wt)[0], zb, (C, H, W), k, k, s, s, p, p)) <= TOL_X3
    layer.close()


@pytest.mark.parametrize("case", [(4, 64, 16, 16, 96, 3, 1, 1, False), (4, 64, 16, 16, 128, 4, 2, 1, True), (4, 3, 64, 64, 64, 4, 2, 1, False),
                                  (4, 32, 16, 16, 3, 3, 1, 1, False)])
@pytest.mark.parametrize("mode", ["x3", "tf32", "fp32"])
def test_prepacked_weights_change_nothing(ops, case, mode):
    """b200_conv_layers_prepack (the weight packs of several layers in one launch) before a forward call gives bit for bit
    what the layer's own packing gives, forward and backward; the mark is good for one forward call only, so a forward call
    after the weights have changed, without a fresh prepack, sees the new weights."""
    B, C, H, W, K, k, s, p, transposed = case
    ops.set_precision({"x3": ops.TF32X3, "tf32": ops.TF32, "fp32": ops.FP32}[mode])
    x, wt, b, d = conv_inputs(sum(case[:8]) + 9, B, C, H, W, K, k, s, p)
    if transposed:
        x, d = d, x
    X, WT, BI, D = dev(x), dev(wt), dev(b), dev(d)
    bias = None if transposed else BI
    plain = ops.ConvLayer(C, H, W, K, k, k, s, s, p, p, B, transposed=transposed)
    packed = ops.ConvLayer(C, H, W, K, k, k, s, s, p, p, B, transposed=transposed)
    other = ops.ConvLayer(C, H, W, K, k, k, s, s, p, p, B, transposed=transposed)       # a second layer in the same launch
    WT2 = WT * 0.5

    def run(layer, kernel):
        y, dx, dk = torch.full_like(D, float("nan")), torch.full_like(X, float("nan")), torch.zeros_like(WT)
        layer.forward(y, X, kernel, bias)
        layer.backward(dx, dk, None, D, X, kernel, accumulate=False)
        return y, dx, dk

    for rep in range(2):
        want = run(plain, WT)
        ops.prepack_conv_layers([packed, other], [WT, WT2])
        got = run(packed, WT)
        got_other = run(other, WT2)
        want_other = run(plain, WT2)
        assert all(torch.equal(a, b) for a, b in zip(got, want))
        assert all(torch.equal(a, b) for a, b in zip(got_other, want_other))
        # the weights change in place; no prepack: the layer must pack the new values itself
        WT.mul_(1.25)
        assert all(torch.equal(a, b) for a, b in zip(run(packed, WT), run(plain, WT)))
    ops.stream_status()
    for layer in (plain, packed, other):
        layer.close()


FUSED_CASES = [(4, 64, 16, 16, 96, 3, 1, 1, False), (6, 128, 8, 8, 256, 4, 2, 1, False), (5, 512, 4, 4, 100, 3, 1, 1, False),      # plain, strided, split-K
               (4, 3, 64, 64, 64, 4, 2, 1, False), (3, 40, 12, 12, 24, 3, 1, 1, False),                                           # few-channel input, ragged
               (4, 64, 16, 16, 128, 4, 2, 1, True), (4, 3, 64, 64, 64, 4, 2, 1, True),                                            # transposed layers
               (4, 32, 16, 16, 3, 3, 1, 1, False)]                                                                                # few filters


@pytest.mark.parametrize("case", FUSED_CASES)
@pytest.mark.parametrize("mode", ["x3", "tf32", "fp32"])
def test_fused_forward_equals_separate_calls(ops, case, mode):
    """b200_conv_layer_forward_fused (function layer in front applied while packing, function layer behind applied in the
    epilogue) gives bit for bit what activation -> forward -> activation give, on every path; the backward call that follows
    gives the same gradients although the activated input was never handed to it as a tensor."""
    B, C, H, W, K, k, s, p, transposed = case
    ops.set_precision({"x3": ops.TF32X3, "tf32": ops.TF32, "fp32": ops.FP32}[mode])
    x, wt, b, d = conv_inputs(sum(case[:8]) + 5, B, C, H, W, K, k, s, p)
    if transposed:
        x, d = d, x                                     # layer input: K channels (small), output error: C channels (large)
    X, WT, BI, D = dev(x), dev(wt), dev(b), dev(d)
    bias = None if transposed else BI
    # separate launches
    ref = ops.ConvLayer(C, H, W, K, k, k, s, s, p, p, B, transposed=transposed)
    fx = torch.empty_like(X)
    ops.CTensorApplyFunc.Apply(fx, X, "leaky_relu", 0.2)
    pre_ref = torch.empty_like(D)
    ref.forward(pre_ref, fx, WT, bias)
    out_ref = torch.empty_like(D)
    ops.CTensorApplyFunc.Apply(out_ref, pre_ref, "tanh")
    dk_ref, dx_ref = torch.zeros_like(WT), torch.empty_like(X)
    ref.backward(dx_ref, dk_ref, None, D, fx, WT, accumulate=False)
    # fused
    lay = ops.ConvLayer(C, H, W, K, k, k, s, s, p, p, B, transposed=transposed)
    for act_out in (torch.full_like(X, float("nan")), None):
        pre, out = torch.full_like(D, float("nan")), torch.full_like(D, float("nan"))
        lay.forward_fused(out, X, WT, bias, input_func="leaky_relu", input_slope=0.2, input_act_out=act_out, output_func="tanh", output_pre=pre)
        assert torch.equal(out, out_ref) and torch.equal(pre, pre_ref)
        if act_out is not None:
            assert torch.equal(act_out, fx)
        dk, dx = torch.zeros_like(WT), torch.empty_like(X)
        lay.backward(dx, dk, None, D, act_out if act_out is not None else X, WT, accumulate=False)     # X: NOT the layer input; must not be read
        assert torch.equal(dk, dk_ref) and torch.equal(dx, dx_ref)
    # one side only
    out = torch.full_like(D, float("nan"))
    lay.forward_fused(out, fx, WT, bias, output_func="tanh")
    assert torch.equal(out, out_ref)
    lay.forward_fused(out, X, WT, bias, input_func="leaky_relu", input_slope=0.2)
    assert torch.equal(out, pre_ref)
    ops.stream_status()
    ref.close()
    lay.close()
