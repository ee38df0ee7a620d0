"""Host-side mirrors of the reference's layer classes on torch CUDA tensors, each a thin sequence of calls into
libb200conv.so.  A layer keeps the reference's tensors (output H, delta, weights, weight gradients) and its
three training entry points:

    Forward()                          netlayer/*.cu.h  Forward
    TrainingBackward(create_dw)        netlayer/*.cu.h  SetOutputError + TrainingBackward
    TrainingResetDeltaWeight / TrainingUpdateWeight are done for the whole net at once on the arenas (Net).

Tensors are [W=batch, Z, Y, X] fp32 like CTensor.  Weights, gradients and the two Adam moments of all layers of a
net live in four contiguous arenas (weights / gradients / m / v) with identical offsets: the gradient arena is what
a data-parallel step all-reduces, and one b200_adam call updates every parameter of the net.
"""
import ctypes as C
import os

import numpy as np
import torch

from . import ops
from .dp import GradArena, PeerBuffer, arena_layout
from .lib import load
from .ops import ACT, _check, _ptr, _stream


class _Layer:
    """Common part: shapes, parameter declaration, binding of arena views."""
    params = ()                     # names of this layer's parameter tensors

    def param_shapes(self):
        return {}

    def bind(self, weights, grads):
        self.w, self.g = weights, grads

    def init(self, rng):
        pass

    def host_params(self):
        return {k: v.detach().cpu().numpy() for k, v in self.w.items()}


class NetLayerConvolution(_Layer):
    """netlayer/cnetlayerconvolution.cu.h: Forward :310 (ForwardConvolution with bias), TrainingBackward :484
    (BackwardConvolution with a zero bias, per-sample CreateDeltaWeightAndBias reduced over W into dKernel/dBias)."""
    transposed = False

    def __init__(self, in_shape, batch, kernel_amount, kernel_size, stride, padding):
        z, y, x = in_shape
        self.in_shape, self.batch = tuple(in_shape), batch
        self.K, self.k, self.s, self.p = kernel_amount, kernel_size, stride, padding
        if self.transposed:
            oy, ox = (y - 1) * stride - 2 * padding + kernel_size, (x - 1) * stride - 2 * padding + kernel_size
            # the layer's kernel tensor is that of the convolution it transposes: [in_z filters][out_z*k*k]
            self.ctx = ops.ConvLayer(kernel_amount, oy, ox, z, kernel_size, kernel_size, stride, stride, padding, padding, batch,
                                     transposed=True)
            self.kernel_shape, self.bias_shape = (1, 1, z, kernel_amount * kernel_size * kernel_size), (1, z, 1, 1)
        else:
            oy, ox = (y - kernel_size + 2 * padding) // stride + 1, (x - kernel_size + 2 * padding) // stride + 1
            self.ctx = ops.ConvLayer(z, y, x, kernel_amount, kernel_size, kernel_size, stride, stride, padding, padding, batch)
            self.kernel_shape, self.bias_shape = (1, 1, kernel_amount, z * kernel_size * kernel_size), (1, kernel_amount, 1, 1)
        self.out_shape = (kernel_amount, oy, ox)
        self.H = torch.empty((batch,) + self.out_shape, device="cuda")
        self.prev_error = torch.empty((batch,) + self.in_shape, device="cuda")

    def param_shapes(self):
        return {"kernel": self.kernel_shape, "bias": self.bias_shape}

    def init(self, rng):
        # He-normal on the fan-in of one output element, zero bias
        fan_in = self.kernel_shape[3] if not self.transposed else self.in_shape[0] * self.k * self.k
        self.w["kernel"].copy_(torch.from_numpy((rng.standard_normal(self.kernel_shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)))
        self.w["bias"].zero_()

    # Function layers folded into this layer's Forward (set by Net when it finds the pairs; netlayer/cnetlayerfunction.cu.h:202):
    # `before` is the function layer in front (its function is applied while this layer packs its input), `after` the one
    # behind (applied in the epilogue of the convolution kernel; this layer's H still receives the value before the function).
    before = after = None

    def Forward(self, x):
        """x: the layer input, or the INPUT of the function layer in front when that layer is folded in."""
        bias = None if self.transposed else self.w["bias"]
        if self.before is None and self.after is None:
            self.x = x
            self.ctx.forward(self.H, x, self.w["kernel"], bias)
            return self.H
        b, a = self.before, self.after
        # what TrainingBackward hands to the library as the layer input: f(x) where it exists as a tensor
        self.x = (b.H if b.materialise else x) if b is not None else x
        self.ctx.forward_fused(a.H if a is not None else self.H, x, self.w["kernel"], bias,
                               input_func=b.func if b is not None else None, input_slope=b.slope if b is not None else 0.1,
                               input_act_out=b.H if (b is not None and b.materialise) else None,
                               output_func=a.func if a is not None else None, output_slope=a.slope if a is not None else 0.1,
                               output_pre=self.H if a is not None else None)
        if a is not None:
            a.x = self.H                    # the function layer's input, for its derivative on the way back
        return self.H                       # the function layer behind, if folded, hands its H on from its own Forward

    def TrainingBackward(self, delta, create_delta_weight=True, need_prev=True):
        self.ctx.backward(self.prev_error if need_prev else None,
                          self.g["kernel"] if create_delta_weight else None,
                          self.g["bias"] if create_delta_weight else None,
                          delta, self.x, self.w["kernel"], accumulate=True)
        return self.prev_error if need_prev else None


class NetLayerBackConvolution(NetLayerConvolution):
    """netlayer/cnetlayerbackconvolution.cu.h: Forward :303 is BackwardConvolution of the layer input, TrainingBackward
    :475 is ForwardConvolution of the delta plus CreateBackDeltaWeightAndBias (which clears the bias gradient)."""
    transposed = True


class NetLayerLinear(_Layer):
    """netlayer/cnetlayerlinear.cu.h: Forward :262 (H = W*x + B per sample), TrainingBackward :415 (prev error =
    W^T*delta; dW += sum over samples of delta*x^T; dB += sum of delta).  The three products are one GEMM each over the
    whole batch; the reference's [batch, out, in] scratch of per-sample outer products is not materialised."""

    def __init__(self, in_shape, batch, neurons):
        self.in_shape, self.batch, self.neurons = tuple(in_shape), batch, neurons
        self.n_in = int(np.prod(in_shape))
        self.out_shape = (1, neurons, 1)
        self.H = torch.empty((batch, 1, neurons, 1), device="cuda")
        self.prev_error = torch.empty((batch,) + self.in_shape, device="cuda")
        self.tmp_dw = torch.empty((1, 1, neurons, self.n_in), device="cuda")

    def param_shapes(self):
        return {"w": (1, 1, self.neurons, self.n_in), "b": (1, 1, self.neurons, 1)}

    def init(self, rng):
        self.w["w"].copy_(torch.from_numpy((rng.standard_normal((1, 1, self.neurons, self.n_in)) * np.sqrt(2.0 / self.n_in)).astype(np.float32)))
        self.w["b"].zero_()

    def Forward(self, x):
        self.x = x
        ops.CTensorMath.Mul(self.H, self.w["w"], x.view(self.batch, 1, self.n_in, 1))
        ops.CTensorMath.Add(self.H, self.H, self.w["b"])
        return self.H

    def TrainingBackward(self, delta, create_delta_weight=True, need_prev=True):
        delta = delta.view(self.batch, 1, self.neurons, 1)
        if need_prev:
            ops.CTensorMath.TransponseMul(self.prev_error.view(self.batch, 1, self.n_in, 1), self.w["w"], delta)
        if create_delta_weight:
            # sum_b delta_b * x_b^T = D^T * X with D = [batch, out] and X = [batch, in] as stored
            ops.CTensorMath.TransponseMul(self.tmp_dw, delta.view(1, 1, self.batch, self.neurons), self.x.view(1, 1, self.batch, self.n_in))
            ops.CTensorMath.Add(self.g["w"], self.g["w"], self.tmp_dw)
            ops.CTensorMath.AddSumW(self.g["b"], self.g["b"], delta)
        return self.prev_error if need_prev else None


class NetLayerFunction(_Layer):
    """netlayer/cnetlayerfunction.cu.h: Forward applies the neuron function; SetOutputError :347-358 forms
    delta = f'(layer input) * error, which TrainingBackward hands to the previous layer."""

    # folded = "into_next": the convolution layer behind applies the function while it packs its input (Forward here only
    # remembers its input; H is written by that layer when `materialise` is set); folded = "into_prev": the convolution layer
    # in front applies it in its epilogue and writes H.  Net sets these; a stand-alone layer has neither.
    folded = None
    materialise = True

    def __init__(self, in_shape, batch, func, leaky_slope=0.1):
        self.in_shape = self.out_shape = tuple(in_shape)
        self.batch, self.func, self.slope = batch, func, leaky_slope
        self.H = torch.empty((batch,) + self.in_shape, device="cuda")
        self.delta = torch.empty((batch,) + self.in_shape, device="cuda")

    def Forward(self, x):
        if self.folded == "into_prev":
            return self.H                   # written by the convolution layer in front; self.x was set by Net
        self.x = x
        if self.folded == "into_next":
            return x                        # the convolution layer behind applies the function to x
        ops.CTensorApplyFunc.Apply(self.H, x, self.func, self.slope)
        return self.H

    def TrainingBackward(self, error, create_delta_weight=True, need_prev=True):
        ops.CTensorApplyFunc.Backward(self.delta, self.x, error, self.func, self.slope)
        return self.delta


class NetLayerBatchNormalization(_Layer):
    """netlayer/cnetlayerbatchnormalization.cu.h: Forward (training) :301-379 and TrainingBackward :578-604, statistics per
    (z,y,x) element over the batch; one fused kernel each instead of about a dozen element-wise launches."""

    def __init__(self, in_shape, batch, momentum=0.9, eps=1e-6):
        self.in_shape = self.out_shape = tuple(in_shape)
        self.batch, self.momentum, self.eps = batch, momentum, eps
        self.n = int(np.prod(in_shape))
        full, stat = (batch,) + self.in_shape, (1,) + self.in_shape
        self.H, self.xhat, self.prev_error = (torch.empty(full, device="cuda") for _ in range(3))
        self.ivar, self.mean, self.var = (torch.empty(stat, device="cuda") for _ in range(3))
        self.new_mean, self.new_var = torch.zeros(stat, device="cuda"), torch.ones(stat, device="cuda")

    def param_shapes(self):
        return {"gamma": (1,) + self.in_shape, "beta": (1,) + self.in_shape}

    def init(self, rng):
        self.w["gamma"].fill_(1.0)
        self.w["beta"].zero_()

    def Forward(self, x):
        _check(load().b200_bn_forward(_ptr(self.H), _ptr(self.xhat), _ptr(self.ivar), _ptr(self.mean), _ptr(self.var),
                                      _ptr(self.new_mean), _ptr(self.new_var), _ptr(x), _ptr(self.w["gamma"]), _ptr(self.w["beta"]),
                                      self.batch, self.n, self.momentum, self.eps, _stream()))
        return self.H

    def TrainingBackward(self, delta, create_delta_weight=True, need_prev=True):
        _check(load().b200_bn_backward(_ptr(self.prev_error), _ptr(self.g["gamma"]), _ptr(self.g["beta"]), _ptr(delta), _ptr(self.xhat),
                                       _ptr(self.ivar), _ptr(self.w["gamma"]), self.batch, self.n, int(create_delta_weight), _stream()))
        return self.prev_error


class NetLayerBatchNormalizationFunction(NetLayerBatchNormalization):
    """A batch-normalisation layer and the function layer that follows it as one layer (same arithmetic as the two in
    sequence, netlayer/cnetlayerbatchnormalization.cu.h:301-379,578-604 + netlayer/cnetlayerfunction.cu.h:347-358): the
    activation is applied when the normalised values are written, and on the way back the function layer's delta is formed
    from the recomputed output while the error column is staged, so neither the pre-activation tensor nor the delta is ever
    stored."""

    def __init__(self, in_shape, batch, func, leaky_slope=0.1, momentum=0.9, eps=1e-6):
        super().__init__(in_shape, batch, momentum, eps)
        self.func, self.slope = func, leaky_slope

    def Forward(self, x):
        _check(load().b200_bn_act_forward(_ptr(self.H), _ptr(self.xhat), _ptr(self.ivar), _ptr(self.mean), _ptr(self.var),
                                          _ptr(self.new_mean), _ptr(self.new_var), _ptr(x), _ptr(self.w["gamma"]), _ptr(self.w["beta"]),
                                          self.batch, self.n, self.momentum, self.eps, ACT[self.func], self.slope, _stream()))
        return self.H

    def TrainingBackward(self, error, create_delta_weight=True, need_prev=True):
        _check(load().b200_bn_act_backward(_ptr(self.prev_error), _ptr(self.g["gamma"]), _ptr(self.g["beta"]), _ptr(error), _ptr(self.xhat),
                                           _ptr(self.ivar), _ptr(self.w["gamma"]), _ptr(self.w["beta"]), self.batch, self.n,
                                           int(create_delta_weight), ACT[self.func], self.slope, _stream()))
        return self.prev_error


class NetLayerMaxPooling(_Layer):
    """netlayer/cnetlayermaxpooling.cu.h: Forward :246 (window maximum and its absolute position), TrainingBackward :367."""

    def __init__(self, in_shape, batch, pooling):
        z, y, x = in_shape
        self.in_shape, self.out_shape, self.batch, self.pool = tuple(in_shape), (z, y // pooling, x // pooling), batch, pooling
        self.H = torch.empty((batch,) + self.out_shape, device="cuda")
        self.P = torch.empty((batch,) + self.out_shape + (2,), dtype=torch.int32, device="cuda")     # SPos {X, Y}
        self.prev_error = torch.empty((batch,) + self.in_shape, device="cuda")

    def Forward(self, x):
        ops.CTensorMath.MaxPooling(self.H, self.P, x, self.pool, self.pool)
        return self.H

    def TrainingBackward(self, delta, create_delta_weight=True, need_prev=True):
        ops.CTensorMath.MaxPoolingBackward(self.prev_error, self.P, delta, self.pool, self.pool)
        return self.prev_error


class NetLayerUpSampling(_Layer):
    """netlayer/cnetlayerupsampling.cu.h: Forward :249 (nearest-neighbour replication), TrainingBackward :366 (DownSampling)."""

    def __init__(self, in_shape, batch, factor):
        z, y, x = in_shape
        self.in_shape, self.out_shape, self.batch, self.f = tuple(in_shape), (z, y * factor, x * factor), batch, factor
        self.H = torch.empty((batch,) + self.out_shape, device="cuda")
        self.prev_error = torch.empty((batch,) + self.in_shape, device="cuda")

    def Forward(self, x):
        ops.CTensorMath.UpSampling(self.H, x, self.f, self.f)
        return self.H

    def TrainingBackward(self, delta, create_delta_weight=True, need_prev=True):
        ops.CTensorMath.DownSampling(self.prev_error, delta, self.f, self.f)
        return self.prev_error


class NetLayerTimeEmbedding(_Layer):
    """netlayer/cnetlayertimeembedding.cu.h: Forward :224 adds the sinusoidal code of each sample's time step (SetTimeStep);
    the error passes through unchanged (:318-322)."""

    def __init__(self, in_shape, batch):
        self.in_shape = self.out_shape = tuple(in_shape)
        self.batch = batch
        self.H = torch.empty((batch,) + self.in_shape, device="cuda")
        self.time_line = torch.zeros((batch, 1, 1, 1), dtype=torch.int32, device="cuda")

    def SetTimeStep(self, index, time_step):
        self.time_line[index] = int(time_step)

    def Forward(self, x):
        ops.CTensorMath.SetTimeStep(self.H, x, self.time_line)
        return self.H

    def TrainingBackward(self, delta, create_delta_weight=True, need_prev=True):
        return delta


class NetLayerConcatenator(_Layer):
    """netlayer/cnetlayerconcatenator.cu.h: Forward :235 joins the outputs of two layers along Z (ConcatecationZ);
    SetOutputError :372 splits the error back (SplitZ).  Two inputs, so it sits outside Net's single chain."""

    def __init__(self, in_shape_a, in_shape_b, batch):
        if tuple(in_shape_a[1:]) != tuple(in_shape_b[1:]):
            raise ops.B200Error(1, "concatenated layers must have the same Y and X size")
        self.in_shape_a, self.in_shape_b, self.batch = tuple(in_shape_a), tuple(in_shape_b), batch
        self.out_shape = (in_shape_a[0] + in_shape_b[0],) + tuple(in_shape_a[1:])
        self.H = torch.empty((batch,) + self.out_shape, device="cuda")
        self.prev_error_a = torch.empty((batch,) + self.in_shape_a, device="cuda")
        self.prev_error_b = torch.empty((batch,) + self.in_shape_b, device="cuda")

    def Forward(self, a, b):
        ops.CTensorMath.ConcatecationZ(self.H, a, b)
        return self.H

    def TrainingBackward(self, delta, create_delta_weight=True, need_prev=True):
        ops.CTensorMath.SplitZ(self.prev_error_a, self.prev_error_b, delta)
        return self.prev_error_a, self.prev_error_b


class AdamCorrections:
    """The two bias corrections of Adam for the current step in device memory, refreshed from the host before a step by a
    16-byte stream-ordered copy.  The copy reads pinned host memory when it executes, and the host may run many steps ahead
    of the device, so every step has its own slot in a ring of pinned pairs (far longer than a stream's queue of pending
    work)."""
    SLOTS = 4096

    def __init__(self, beta1=0.9, beta2=0.999):
        self.beta1, self.beta2 = beta1, beta2
        self.host = torch.zeros(self.SLOTS, 2, dtype=torch.float64).pin_memory()
        self.device = torch.zeros(2, dtype=torch.float64, device="cuda")
        self.calls = 0

    def set(self, iteration):
        slot = self.host[self.calls % self.SLOTS]
        self.calls += 1
        slot[0] = 1.0 - self.beta1 ** iteration
        slot[1] = 1.0 - self.beta2 ** iteration
        self.device.copy_(slot, non_blocking=True)
        return self.device


class Net:
    """A chain of layers with the reference's training protocol (cuda/netmodel/cmodelmain.cu.h drives every net the same way:
    TrainingResetDeltaWeight, Forward of all layers, SetOutputError on the last, TrainingBackward in reverse order,
    TrainingUpdateWeight) on four arenas: weights, gradients, Adam m and v."""

    def __init__(self, in_shape, batch, spec, seed=0, peer=False, channel=0, fold=True):
        """spec: list of (class, kwargs).  The input of layer i is the output of layer i-1.
        peer: True, or a PeerBuffer shared with other nets.  With several ranks, the weight and gradient arenas are placed in
        the PeerBuffer (memory every rank maps), and
        TrainingUpdateWeight(fused=True) runs the library's reduce-scatter + Adam + all-gather kernel on `channel`.
        fold: function layers next to a convolution layer are folded into that layer's Forward (see fold_functions)."""
        self.batch, self.in_shape = batch, tuple(in_shape)
        self.layers, shape = [], tuple(in_shape)
        for cls, kw in spec:
            if cls == "reshape":             # ReinterpretSize of the previous output (cuda/ctensor.cu.h): no data moves
                shape = tuple(kw)
                continue
            layer = cls(shape, batch, **kw)
            self.layers.append(layer)
            shape = layer.out_shape
        self.out_shape = shape
        self.fold_functions(fold)
        shapes = {}
        for i, layer in enumerate(self.layers):
            for name, s in layer.param_shapes().items():
                shapes["%d.%s" % (i, name)] = s
        self.peer, self.channel = None, channel
        import torch.distributed as dist
        if peer and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            _, total = arena_layout(shapes)
            self.peer = peer if isinstance(peer, PeerBuffer) else PeerBuffer(2 * total)
            self.weight_offset, w_span = self.peer.take(total)
            self.grad_offset, g_span = self.peer.take(total)
            self.weights = GradArena(shapes, "cuda", w_span[:total])
            self.grads = GradArena(shapes, "cuda", g_span[:total])
            self.m, self.v = (GradArena(shapes, "cuda") for _ in range(2))
        else:
            self.weights, self.grads, self.m, self.v = (GradArena(shapes, "cuda") for _ in range(4))
        rng = np.random.default_rng(seed)
        for i, layer in enumerate(self.layers):
            names = list(layer.param_shapes())
            layer.bind({n: self.weights.views["%d.%s" % (i, n)] for n in names}, {n: self.grads.views["%d.%s" % (i, n)] for n in names})
            layer.init(rng)

        self.ema, self.ema_k, self.use_ema = None, 0.999, False

    def fold_functions(self, enable=True, materialise=True):
        """Folds every function layer that directly follows a convolution layer into that layer's epilogue, and every other
        function layer that directly precedes one into that layer's input pack (b200_conv_layer_forward_fused): same values, one
        launch and one pass over the tensor less per pair (in B200_FP32 mode the library runs the same sequence as separate
        launches).  materialise=False: a function layer folded into the layer BEHIND it no
        longer writes its own output tensor (nothing else reads it in a chain)."""
        conv = (NetLayerConvolution, NetLayerBackConvolution)
        for layer in self.layers:
            if isinstance(layer, conv):
                layer.before = layer.after = None
            if isinstance(layer, NetLayerFunction):
                layer.folded, layer.materialise = None, True
        if not enable or os.environ.get("B200CONV_FOLD") == "0":          # tuning aid: B200CONV_FOLD=0 keeps every layer separate
            return
        for i, layer in enumerate(self.layers):
            if not isinstance(layer, NetLayerFunction):
                continue
            prev_l = self.layers[i - 1] if i > 0 else None
            next_l = self.layers[i + 1] if i + 1 < len(self.layers) else None
            # into the epilogue only where the contraction is long enough to hide the second output stream behind the tensor-core
            # work of the next tile (measured on the VAE encoder: with 27..576-term sums the kernel is bound by its epilogue's
            # stores and the folded layer was slower than the two launches)
            if isinstance(prev_l, conv) and prev_l.out_shape == layer.in_shape and prev_l.kernel_shape[3] >= 1024:
                layer.folded, prev_l.after = "into_prev", layer
            elif isinstance(next_l, conv) and next_l.in_shape == layer.out_shape:
                layer.folded, layer.materialise, next_l.before = "into_next", materialise, layer

    @property
    def parameter_count(self):
        return self.weights.buffer.numel()

    def EnableEMA(self, state, ema_k=0.999):
        """INetLayer::EnableEMA for every layer of the net (netlayer/cnetlayerconvolution.cu.h:622-634): the averaged weights
        start as a copy of the weights; TrainingUpdateWeight then keeps ema = ema_k * ema + (1 - ema_k) * weight in the same
        launch as Adam.  Disabling drops them."""
        if state:
            self.ema = GradArena({k: v[2] for k, v in self.weights.offsets.items()}, "cuda")
            self.ema.buffer.copy_(self.weights.buffer)
            self.ema_k = ema_k
        else:
            self.SetUseEMA(False)
            self.ema = None

    def SetUseEMA(self, state):
        """INetLayer::SetUseEMA (netlayer/inetlayer.cu.h:97-101): Forward uses the averaged weights instead of the trained ones."""
        if state and self.ema is None:
            raise ops.B200Error(2, "SetUseEMA: the averaged weights were not enabled")
        source = self.ema if state else self.weights
        for i, layer in enumerate(self.layers):
            names = list(layer.param_shapes())
            layer.bind({n: source.views["%d.%s" % (i, n)] for n in names}, layer.g if names else {})
        self.use_ema = bool(state)

    def TrainingResetDeltaWeight(self):
        ops.CTensorMath.Fill(self.grads.buffer.view(1, 1, 1, -1), 0.0)

    def Forward(self, x):
        for layer in self.layers:
            x = layer.Forward(x.view((self.batch,) + layer.in_shape))
        return x

    def TrainingBackward(self, error, create_delta_weight=True, need_input_error=False):
        for i in range(len(self.layers) - 1, -1, -1):
            layer = self.layers[i]
            error = layer.TrainingBackward(error.view((self.batch,) + layer.out_shape), create_delta_weight, need_prev=(i > 0 or need_input_error))
        return error

    @staticmethod
    def PrepackWeights(nets):
        """The tensor-core packs of the convolution kernels of all layers of `nets` in one launch (b200_conv_layers_prepack),
        for the forward passes that follow: call at the start of a training step, after the weights were last changed.  Each
        layer's next Forward then skips its own weight-pack launch; nothing else changes."""
        layers = [layer for net in nets for layer in net.layers if isinstance(layer, NetLayerConvolution)]
        ops.prepack_conv_layers([layer.ctx for layer in layers], [layer.w["kernel"] for layer in layers])

    def TrainingUpdateWeightFused(self, speed, iteration, batch_scale=1, beta1=0.9, beta2=0.999, epsilon=1e-8, corrections=None):
        """The data-parallel update in one kernel (b200_allreduce_adam): every rank sums its slice of the gradient arenas of
        all ranks over NVLink, applies Adam to that slice and writes the new weights to all ranks.  Replaces grads.all_reduce()
        followed by TrainingUpdateWeight; the moving average of the weights is not kept on this path."""
        if self.peer is None:
            self.grads.all_reduce()
            return self.TrainingUpdateWeight(speed, iteration, batch_scale, beta1, beta2, epsilon, corrections)
        if self.ema is not None:
            raise ops.B200Error(2, "the fused update does not keep the moving average of the weights")
        n = self.weights.buffer.numel()
        _check(load().b200_allreduce_adam(self.peer.comm, self.grad_offset, self.weight_offset, _ptr(self.m.buffer), _ptr(self.v.buffer), n,
                                          int(self.batch * batch_scale), speed, beta1, beta2, epsilon, 0.0 if iteration is None else iteration,
                                          _ptr(corrections), self.channel, _stream()))

    @staticmethod
    def TrainingUpdateWeightFusedTogether(nets, speed, iteration, batch_scale=1, beta1=0.9, beta2=0.999, epsilon=1e-8, corrections=None):
        """The fused data-parallel update of several nets that share one PeerBuffer in ONE launch (b200_allreduce_adam_multi):
        one pair of device-side barriers for all of them."""
        from .lib import ExchangeSegment
        peer = nets[0].peer
        if peer is None or any(net.peer is not peer for net in nets) or len({net.batch for net in nets}) != 1:
            for net in nets:
                net.TrainingUpdateWeightFused(speed, iteration, batch_scale, beta1, beta2, epsilon, corrections)
            return
        segs = (ExchangeSegment * len(nets))()
        for seg, net in zip(segs, nets):
            seg.grad_offset, seg.weight_offset, seg.n = net.grad_offset, net.weight_offset, net.weights.buffer.numel()
            seg.m, seg.v = net.m.buffer.data_ptr(), net.v.buffer.data_ptr()
        _check(load().b200_allreduce_adam_multi(peer.comm, len(nets), segs, int(nets[0].batch * batch_scale), speed, beta1, beta2, epsilon,
                                                0.0 if iteration is None else iteration, _ptr(corrections), nets[0].channel, _stream()))

    def peer_all_reduce(self):
        """Sum of the gradient arenas over the ranks by the library's own exchange kernel (b200_allreduce), in place."""
        if self.peer is None:
            return self.grads.all_reduce()
        _check(load().b200_allreduce(self.peer.comm, self.grad_offset, self.grads.buffer.numel(), self.channel, _stream()))
        return self.grads.buffer

    def TrainingUpdateWeight(self, speed, iteration, batch_scale=1, beta1=0.9, beta2=0.999, epsilon=1e-8, corrections=None):
        """CTensorMath::Adam over every parameter of the net in one launch; batch_size = batch*batch_scale divides the
        summed gradient (netlayer/cnetlayerconvolution.cu.h:533-552).  corrections: a float64 CUDA tensor holding
        {1 - beta1^iteration, 1 - beta2^iteration} (see adam_corrections); the launch then has fixed arguments and can be
        part of a CUDA graph."""
        w, g, m, v = (a.buffer for a in (self.weights, self.grads, self.m, self.v))
        ema = self.ema.buffer if self.ema is not None else None
        _check(load().b200_adam_ema(_ptr(w), _ptr(g), _ptr(m), _ptr(v), _ptr(ema), w.numel(), int(self.batch * batch_scale), speed, beta1,
                                    beta2, epsilon, 0.0 if iteration is None else iteration, _ptr(corrections), self.ema_k, _stream()))

    def broadcast_weights(self):
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.broadcast(self.weights.buffer, src=0)
