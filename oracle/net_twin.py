"""Test infrastructure, not product code.  CPU twin of a layers.Net for the parity tests and the CPU baseline of the
benchmark: the same chain of layers evaluated with the oracle's tensor routines
in the order the reference's layer classes call them (netlayer/cnetlayerconvolution.cu.h:310,484;
cnetlayerbackconvolution.cu.h:303,475; cnetlayerlinear.cu.h:262,415; cnetlayerfunction.cu.h:347-358;
cnetlayerbatchnormalization.cu.h:301-379,578-604; cnetlayermaxpooling.cu.h:246,367; cnetlayerupsampling.cu.h:249,366).
Per-sample weight gradients are summed over the batch in float64 so that the twin adds no ordering noise."""
import numpy as np


class OracleNet:
    def __init__(self, port, net, absolute=False):
        """absolute: the parameters are replaced by their absolute values (with absolute inputs a contraction layer then
        yields sum |a||b|, the scale of its rounding error)."""
        self.port, self.net = port, net
        self.params = [layer.host_params() if layer.param_shapes() else {} for layer in net.layers]
        if absolute:
            self.params = [{k: np.abs(v) for k, v in p.items()} for p in self.params]
        self.grads = [{k: np.zeros(v.shape, np.float64) for k, v in p.items()} for p in self.params]
        # bias gradients summed over |delta|: the scale of a bias gradient that cancels to rounding noise (any bias in
        # front of a batch normalisation: the error below it sums to zero over the batch)
        self.grad_mag = [{} for _ in self.params]
        self.cache = [None] * len(net.layers)
        self.outputs = [None] * len(net.layers)
        self.deltas = [None] * len(net.layers)      # error handed to the layer below (index = layer that produced it)

    # ---- optimiser -----------------------------------------------------------------------------
    def reset_gradients(self):
        for g in self.grads:
            for k in g:
                g[k][...] = 0

    def update(self, speed, iteration, batch_size, beta1=0.9, beta2=0.999, epsilon=1e-8):
        """CTensorMath::Adam on every parameter tensor (cpu/ctensormath.h:1119-1165), moments kept per tensor."""
        if not hasattr(self, "moments"):
            self.moments = [{k: (np.zeros(v.shape, np.float32), np.zeros(v.shape, np.float32)) for k, v in p.items()} for p in self.params]
        for i, p in enumerate(self.params):
            for k in p:
                m, v = self.moments[i][k]
                w, m, v = self.port.adam(p[k], self.grads[i][k].astype(np.float32), m, v, batch_size, speed, beta1, beta2, epsilon, iteration)
                p[k] = w.reshape(p[k].shape)
                self.moments[i][k] = (m.reshape(p[k].shape), v.reshape(p[k].shape))

    # ---- forward -------------------------------------------------------------------------------
    def forward(self, x):
        B = x.shape[0]
        for i, layer in enumerate(self.net.layers):
            x = np.ascontiguousarray(x, np.float32).reshape((B,) + layer.in_shape)
            x = getattr(self, "_f_" + type(layer).__name__)(i, layer, x)
            self.outputs[i] = x
        return x

    def forward_layer(self, i, x):
        """Layer i alone on the given input (its cache is what backward_layer then uses)."""
        layer = self.net.layers[i]
        x = np.ascontiguousarray(x, np.float32).reshape((x.shape[0],) + layer.in_shape)
        return getattr(self, "_f_" + type(layer).__name__)(i, layer, x)

    def backward_layer(self, i, error, need_prev=True):
        layer = self.net.layers[i]
        error = np.ascontiguousarray(error, np.float32).reshape((error.shape[0],) + layer.out_shape)
        return getattr(self, "_b_" + type(layer).__name__)(i, layer, error, need_prev)

    def backward(self, error, need_input_error=False):
        B = error.shape[0]
        for i in range(len(self.net.layers) - 1, -1, -1):
            layer = self.net.layers[i]
            error = np.ascontiguousarray(error, np.float32).reshape((B,) + layer.out_shape)
            error = getattr(self, "_b_" + type(layer).__name__)(i, layer, error, i > 0 or need_input_error)
            self.deltas[i] = error
        return error

    # ---- convolution ---------------------------------------------------------------------------
    def _f_NetLayerConvolution(self, i, L, x):
        self.cache[i] = x
        w = self.params[i]
        return self.port.conv_forward(x, w["kernel"].reshape(1, L.K, -1), w["bias"].reshape(1, L.K), L.k, L.k, L.s, L.s, L.p, L.p)

    def _b_NetLayerConvolution(self, i, L, d, need_prev):
        x, w, B = self.cache[i], self.params[i], d.shape[0]
        kern = w["kernel"].reshape(1, L.K, -1)
        dk, db = self.port.conv_wgrad(np.zeros((B,) + kern.shape[1:], np.float32), np.zeros((B, L.K), np.float32), x, d, L.k, L.k, L.s, L.s, L.p, L.p)
        self.grads[i]["kernel"] += dk.astype(np.float64).sum(0).reshape(w["kernel"].shape)
        self.grads[i]["bias"] += db.astype(np.float64).sum(0).reshape(w["bias"].shape)
        self.grad_mag[i]["bias"] = np.abs(d).astype(np.float64).sum((0, 2, 3)).reshape(w["bias"].shape)
        if not need_prev:
            return np.zeros((B,) + L.in_shape, np.float32)
        return self.port.conv_backward(d, kern, np.zeros((1, L.K), np.float32), L.in_shape, L.k, L.k, L.s, L.s, L.p, L.p)

    def _f_NetLayerBackConvolution(self, i, L, x):
        self.cache[i] = x
        kern = self.params[i]["kernel"].reshape(1, L.in_shape[0], -1)
        return self.port.conv_backward(x, kern, np.zeros((1, L.in_shape[0]), np.float32), L.out_shape, L.k, L.k, L.s, L.s, L.p, L.p)

    def _b_NetLayerBackConvolution(self, i, L, d, need_prev):
        x, w, B, Kf = self.cache[i], self.params[i], d.shape[0], L.in_shape[0]
        kern = w["kernel"].reshape(1, Kf, -1)
        dk, _ = self.port.conv_wgrad(np.zeros((B,) + kern.shape[1:], np.float32), np.zeros((B, Kf), np.float32), x, d, L.k, L.k, L.s, L.s, L.p, L.p,
                                     back_variant=True)
        self.grads[i]["kernel"] += dk.astype(np.float64).sum(0).reshape(w["kernel"].shape)
        if not need_prev:
            return np.zeros((B,) + L.in_shape, np.float32)
        return self.port.conv_forward(d, kern, np.zeros((1, Kf), np.float32), L.k, L.k, L.s, L.s, L.p, L.p)

    # ---- linear --------------------------------------------------------------------------------
    def _f_NetLayerLinear(self, i, L, x):
        B = x.shape[0]
        self.cache[i] = x
        w = self.params[i]
        h = self.port.mul(w["w"], x.reshape(B, 1, L.n_in, 1))
        return self.port.binary("add", h, w["b"])

    def _b_NetLayerLinear(self, i, L, d, need_prev):
        B, x, w = d.shape[0], self.cache[i], self.params[i]
        d = d.reshape(B, 1, L.neurons, 1)
        tmp = self.port.mul(d, x.reshape(B, 1, 1, L.n_in))                   # per-sample outer products
        self.grads[i]["w"] += tmp.astype(np.float64).sum(0, keepdims=True)
        self.grads[i]["b"] += d.astype(np.float64).sum(0, keepdims=True)
        self.grad_mag[i]["b"] = np.abs(d).astype(np.float64).sum(0, keepdims=True)
        return self.port.tmul(w["w"], d).reshape((B,) + L.in_shape)

    # ---- function ------------------------------------------------------------------------------
    def _f_NetLayerFunction(self, i, L, x):
        self.cache[i] = x
        if L.func == "leaky_relu" and L.slope != 0.1:      # the oracle's LeakyReLU has the reference's fixed slope
            return np.where(x > 0, x, (L.slope * x.astype(np.float64)).astype(np.float32))
        return self.port.activation(x, L.func)

    def _b_NetLayerFunction(self, i, L, e, need_prev):
        x = self.cache[i]
        if L.func == "leaky_relu" and L.slope != 0.1:
            diff = np.where(x >= 0, np.float32(1), np.float32(L.slope))       # derivative 1 at zero, as cpu/ctensorapplyfunc.h:236
        else:
            diff = self.port.activation(x, L.func, derivative=True)
        return self.port.binary("item_product", e, diff)

    # ---- batch normalisation -------------------------------------------------------------------
    def _f_NetLayerBatchNormalization(self, i, L, x):
        w = self.params[i]
        r = self.port.bn_forward(x, w["gamma"][0], w["beta"][0], L.momentum, L.eps)
        self.cache[i] = r
        return r["y"]

    def _b_NetLayerBatchNormalization(self, i, L, d, need_prev):
        r, w = self.cache[i], self.params[i]
        dx, dg, db = self.port.bn_backward(d, r["xhat"], r["ivar"], w["gamma"][0])
        self.grads[i]["gamma"] += dg.reshape(w["gamma"].shape)
        self.grads[i]["beta"] += db.reshape(w["beta"].shape)
        return dx

    # ---- batch normalisation + function as one layer: the two layers in sequence ------------------
    def _f_NetLayerBatchNormalizationFunction(self, i, L, x):
        y = self._f_NetLayerBatchNormalization(i, L, x)
        self.cache[i] = (self.cache[i], y)
        if L.func == "leaky_relu" and L.slope != 0.1:
            return np.where(y > 0, y, (L.slope * y.astype(np.float64)).astype(np.float32))
        return self.port.activation(y, L.func)

    def _b_NetLayerBatchNormalizationFunction(self, i, L, e, need_prev):
        r, y = self.cache[i]
        if L.func == "leaky_relu" and L.slope != 0.1:
            diff = np.where(y >= 0, np.float32(1), np.float32(L.slope))
        else:
            diff = self.port.activation(y, L.func, derivative=True)
        d = self.port.binary("item_product", e, diff)
        self.cache[i] = r
        out = self._b_NetLayerBatchNormalization(i, L, d, need_prev)
        self.cache[i] = (r, y)
        return out

    # ---- pooling / resampling ------------------------------------------------------------------
    def _f_NetLayerMaxPooling(self, i, L, x):
        out, pos = self.port.maxpool(x, L.pool, L.pool)
        self.cache[i] = pos
        return out

    def _b_NetLayerMaxPooling(self, i, L, d, need_prev):
        return self.port.maxpool_backward(d, self.cache[i], L.pool, L.pool)

    def _f_NetLayerUpSampling(self, i, L, x):
        return self.port.upsample(x, L.f, L.f)

    def _b_NetLayerUpSampling(self, i, L, d, need_prev):
        return self.port.downsample(d, L.f, L.f)
