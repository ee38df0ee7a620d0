"""numpy front-end of the CPU oracle.  TEST INFRASTRUCTURE ONLY (see oracle/oracle.c).

`Oracle("port")` binds oracle/liboracle.so (the plain-C restatement); `Oracle("reference")`
binds oracle/_ref/libref.so (the reference's own CPU backend behind a C-ABI shim).  Both expose
the same methods, so the restatement can be checked against the reference call by call.
Arrays are fp32 in W,Z,Y,X order; weights are (Wk, K, C*ky*kx) with the reference's
c*ky*kx + i*kx + j ordering of a filter row.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

_f = C.POINTER(C.c_float)
_u = C.POINTER(C.c_uint32)


def _p(a):
    return a.ctypes.data_as(_f)


def _c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Oracle:
    def __init__(self, kind="port", threads=1):
        """threads > 1: the batched routines (convolution trio, products) split their W range over that many host threads --
        every W index is computed by the same single-threaded routine as before (the loops are independent per w,
        cpu/ctensorconv.h:111), the threads only shorten the wait of a test on a full-size configuration."""
        self.kind = kind
        self.threads = max(1, int(threads))
        if kind == "port":
            path = _build.build_oracle()
            self.pfx = "orc_"
        elif kind == "reference":
            path = _build.build_ref()
            if path is None or not os.path.exists(path):
                raise FileNotFoundError("oracle/_ref/libref.so is not built and the reference tree is absent")
            self.pfx = "ref_"
        else:
            raise ValueError(kind)
        self.lib = C.CDLL(path)
        if kind == "port":
            self.lib.orc_vae_forward.restype = C.c_float

    def _fn(self, name):
        return getattr(self.lib, self.pfx + name)

    def _over_w(self, W, fn):
        """fn(begin, end) -> array or tuple of arrays for the W range [begin, end); results are concatenated along W."""
        n = min(self.threads, W)
        if n <= 1:
            return fn(0, W)
        from concurrent.futures import ThreadPoolExecutor
        bounds = [(W * i // n, W * (i + 1) // n) for i in range(n)]
        with ThreadPoolExecutor(n) as pool:
            parts = list(pool.map(lambda b: fn(*b), bounds))
        if isinstance(parts[0], tuple):
            return tuple(np.concatenate([p[j] for p in parts], 0) for j in range(len(parts[0])))
        return np.concatenate(parts, 0)

    def _single(self):
        one = Oracle.__new__(Oracle)
        one.__dict__.update(self.__dict__)
        one.threads = 1
        return one

    # ---- convolution trio -------------------------------------------------------------------
    def conv_forward(self, image, kernel, bias, kx, ky, sx, sy, px, py, out_w=None):
        image, kernel, bias = _c(image), _c(kernel), _c(bias)
        if self.threads > 1 and out_w is None and kernel.shape[0] == 1 and bias.size == kernel.shape[1] and image.shape[0] > 1:
            one = self._single()
            return self._over_w(image.shape[0], lambda b, e: one.conv_forward(image[b:e], kernel, bias, kx, ky, sx, sy, px, py))
        iw, cz, iy, ix = image.shape
        kw, K, klen = kernel.shape
        assert klen == cz * kx * ky
        bias = bias.reshape(-1, K)
        oy = (iy - ky + 2 * py) // sy + 1
        ox = (ix - kx + 2 * px) // sx + 1
        ow = out_w or max(iw, kw)
        out = np.empty((ow, K, oy, ox), np.float32)
        r = self._fn("conv_forward")(_p(out), ow, oy, ox, _p(image), iw, cz, iy, ix, _p(kernel), kw, kx, ky, K,
                                     _p(bias), bias.shape[0], sx, sy, px, py)
        assert r == 0, r
        return out

    def conv_backward(self, delta, kernel, bias, out_zyx, kx, ky, sx, sy, px, py, out_w=None):
        delta, kernel, bias = _c(delta), _c(kernel), _c(bias)
        if self.threads > 1 and out_w is None and kernel.shape[0] == 1 and bias.size == kernel.shape[1] and delta.shape[0] > 1:
            one = self._single()
            return self._over_w(delta.shape[0], lambda b, e: one.conv_backward(delta[b:e], kernel, bias, out_zyx, kx, ky, sx, sy, px, py))
        dw, K, dy, dx = delta.shape
        kw = kernel.shape[0]
        oz, oy, ox = out_zyx
        assert kernel.shape[1] == K and kernel.shape[2] == oz * kx * ky
        bias = bias.reshape(-1, K)
        ow = out_w or max(dw, kw)
        out = np.empty((ow, oz, oy, ox), np.float32)
        r = self._fn("conv_backward")(_p(out), ow, oz, oy, ox, _p(delta), dw, dy, dx, _p(kernel), kw, kx, ky, K,
                                      _p(bias), bias.shape[0], sx, sy, px, py)
        assert r == 0, r
        return out

    def conv_wgrad(self, dkernel, dbias, image, delta, kx, ky, sx, sy, px, py, back_variant=False):
        """Accumulates into copies of dkernel (Wd,K,C*ky*kx) / dbias (Wb,K) and returns them."""
        dkernel, dbias, image, delta = _c(dkernel).copy(), _c(dbias).copy(), _c(image), _c(delta)
        if self.threads > 1 and dkernel.shape[0] > 1 and dkernel.shape[0] == image.shape[0] == delta.shape[0] and \
                dbias.size == dkernel.shape[0] * dkernel.shape[1]:
            one = self._single()
            db2 = dbias.reshape(dkernel.shape[0], dkernel.shape[1])
            return self._over_w(dkernel.shape[0], lambda b, e: one.conv_wgrad(dkernel[b:e], db2[b:e], image[b:e], delta[b:e], kx, ky, sx, sy,
                                                                             px, py, back_variant))
        wd, K, klen = dkernel.shape
        kz = klen // (kx * ky)
        dbias = dbias.reshape(-1, K)
        # the back variant swaps the roles inside: its image argument is the transposed layer's input (K channels)
        assert (image.shape[1], delta.shape[1]) == ((K, kz) if back_variant else (kz, K)), "operand channels do not match the kernel tensor"
        if self.kind == "port":
            fn = self.lib.orc_conv_back_wgrad if back_variant else self.lib.orc_conv_wgrad
            r = fn(_p(dkernel), wd, kx, ky, kz, K, _p(dbias), dbias.shape[0],
                   _p(image), image.shape[0], image.shape[2], image.shape[3],
                   _p(delta), delta.shape[0], delta.shape[2], delta.shape[3], sx, sy, px, py)
        else:
            r = self.lib.ref_conv_wgrad(_p(dkernel), wd, kx, ky, kz, K, _p(dbias), dbias.shape[0],
                                        _p(image), image.shape[0], image.shape[2], image.shape[3],
                                        _p(delta), delta.shape[0], delta.shape[2], delta.shape[3],
                                        sx, sy, px, py, int(back_variant))
        assert r == 0, r
        return dkernel, dbias

    # ---- dense products ---------------------------------------------------------------------
    def mul(self, left, right, out_w=None):
        left, right = _c(left), _c(right)
        if self.threads > 1 and out_w is None and max(left.shape[0], right.shape[0]) > 1 and min(left.shape[0], right.shape[0]) in (1, max(left.shape[0], right.shape[0])):
            one, W = self._single(), max(left.shape[0], right.shape[0])
            return self._over_w(W, lambda b, e: one.mul(left if left.shape[0] == 1 else left[b:e], right if right.shape[0] == 1 else right[b:e]))
        lw, Z, LY, LX = left.shape
        rw, _, _, RX = right.shape
        ow = out_w or max(lw, rw)
        out = np.empty((ow, Z, LY, RX), np.float32)
        if self.kind == "port":
            self.lib.orc_mul(_p(out), ow, _p(left), lw, _p(right), rw, Z, LY, LX, RX)
        else:
            assert self.lib.ref_mul(_p(out), ow, _p(left), lw, _p(right), rw, Z, LY, LX, RX, 0) == 0
        return out

    def tmul(self, left, right, out_w=None):
        left, right = _c(left), _c(right)
        if self.threads > 1 and out_w is None and max(left.shape[0], right.shape[0]) > 1 and min(left.shape[0], right.shape[0]) in (1, max(left.shape[0], right.shape[0])):
            one, W = self._single(), max(left.shape[0], right.shape[0])
            return self._over_w(W, lambda b, e: one.tmul(left if left.shape[0] == 1 else left[b:e], right if right.shape[0] == 1 else right[b:e]))
        lw, Z, KD, LX = left.shape
        rw, _, _, RX = right.shape
        ow = out_w or max(lw, rw)
        out = np.empty((ow, Z, LX, RX), np.float32)
        if self.kind == "port":
            self.lib.orc_tmul(_p(out), ow, _p(left), lw, _p(right), rw, Z, KD, LX, RX)
        else:
            assert self.lib.ref_mul(_p(out), ow, _p(left), lw, _p(right), rw, Z, KD, LX, RX, 1) == 0
        return out

    # ---- element-wise / reductions ----------------------------------------------------------
    def binary(self, op, left, right, ls=1.0, rs=1.0, out_w=None):
        """op: 'add' | 'sub' | 'add_sum_w' | 'item_product'."""
        left, right = _c(left), _c(right)
        lw, rw = left.shape[0], right.shape[0]
        zyx = left.shape[1:]
        n = int(np.prod(zyx))
        ow = out_w or max(lw, rw)
        out = np.zeros((ow,) + zyx, np.float32)
        if self.kind == "reference":
            code = {"add": 0, "sub": 1, "add_sum_w": 2, "item_product": 3}[op]
            assert self.lib.ref_binary(_p(out), ow, _p(left), lw, _p(right), rw, zyx[0], zyx[1], zyx[2],
                                       C.c_float(ls), C.c_float(rs), code) == 0
        elif op in ("add", "sub"):
            self.lib.orc_add(_p(out), ow, _p(left), lw, _p(right), rw, C.c_size_t(n), C.c_float(ls), C.c_float(rs),
                             int(op == "sub"))
        elif op == "add_sum_w":
            self.lib.orc_add_sum_w(_p(out), ow, _p(left), lw, _p(right), rw, C.c_size_t(n), C.c_float(ls), C.c_float(rs))
        else:
            self.lib.orc_item_product(_p(out), ow, _p(left), lw, _p(right), rw, C.c_size_t(n))
        return out

    def unary(self, op, x, a=1.0, b=0.0, out_w=None):
        """op: 'pow2' | 'sqrt' | 'inv' | 'scale'."""
        x = _c(x)
        code = {"pow2": 0, "sqrt": 1, "inv": 2, "scale": 3}[op]
        ow = out_w or x.shape[0]
        out = np.empty((ow,) + x.shape[1:], np.float32)
        if self.kind == "port":
            self.lib.orc_unary(_p(out), ow, _p(x), x.shape[0], C.c_size_t(int(np.prod(x.shape[1:]))), code,
                               C.c_float(a), C.c_float(b))
        else:
            assert self.lib.ref_unary(_p(out), ow, _p(x), x.shape[0], x.shape[1], x.shape[2], x.shape[3], code,
                                      C.c_float(a), C.c_float(b)) == 0
        return out

    def add_bias(self, t, bias):
        t, bias = _c(t).copy(), _c(bias)
        W, Z, Y, X = t.shape
        bias = bias.reshape(-1, Z)
        if self.kind == "port":
            self.lib.orc_add_bias(_p(t), W, Z, C.c_size_t(Y * X), _p(bias), bias.shape[0])
        else:
            assert self.lib.ref_add_bias(_p(t), W, Z, Y, X, _p(bias), bias.shape[0]) == 0
        return t

    def summ_xy(self, x, out_w=None):
        x = _c(x)
        W, Z, Y, X = x.shape
        ow = out_w or W
        out = np.empty((ow, Z, 1, 1), np.float32)
        if self.kind == "port":
            self.lib.orc_summ_xy(_p(out), ow, _p(x), W, Z, C.c_size_t(Y * X))
        else:
            assert self.lib.ref_summ_xy(_p(out), ow, _p(x), W, Z, Y, X) == 0
        return out

    # ---- pooling / resampling ---------------------------------------------------------------
    def maxpool(self, x, pool_x, pool_y):
        x = _c(x)
        W, Z, Y, X = x.shape
        out = np.empty((W, Z, Y // pool_y, X // pool_x), np.float32)
        pos = np.empty(out.shape + (2,), np.uint32)
        r = self._fn("maxpool")(_p(out), pos.ctypes.data_as(_u), _p(x), W, Z, Y, X, pool_x, pool_y)
        assert self.kind == "port" or r == 0
        return out, pos

    def maxpool_backward(self, delta, pos, pool_x, pool_y):
        delta = _c(delta)
        pos = np.ascontiguousarray(pos, dtype=np.uint32)
        W, Z, dy, dx = delta.shape
        out = np.empty((W, Z, dy * pool_y, dx * pool_x), np.float32)
        r = self._fn("maxpool_backward")(_p(out), pos.ctypes.data_as(_u), _p(delta), W, Z, dy * pool_y, dx * pool_x,
                                         pool_x, pool_y)
        assert self.kind == "port" or r == 0
        return out

    def upsample(self, x, ux, uy):
        x = _c(x)
        W, Z, Y, X = x.shape
        out = np.empty((W, Z, Y * uy, X * ux), np.float32)
        if self.kind == "port":
            self.lib.orc_upsample(_p(out), _p(x), W, Z, Y, X, Y * uy, X * ux, ux, uy)
        else:
            assert self.lib.ref_resample(_p(out), _p(x), W, Z, Y, X, Y * uy, X * ux, ux, uy, 0) == 0
        return out

    def downsample(self, x, dx, dy):
        x = _c(x)
        W, Z, Y, X = x.shape
        out = np.empty((W, Z, Y // dy, X // dx), np.float32)
        if self.kind == "port":
            self.lib.orc_downsample(_p(out), _p(x), W, Z, Y, X, Y // dy, X // dx, dx, dy)
        else:
            assert self.lib.ref_resample(_p(out), _p(x), W, Z, Y, X, Y // dy, X // dx, dx, dy, 1) == 0
        return out

    # ---- activations ------------------------------------------------------------------------
    FUNCS = {"sigmoid": 0, "relu": 1, "leaky_relu": 2, "linear": 3, "tanh": 4, "gelu": 5}

    def activation(self, x, func, derivative=False):
        x = _c(x)
        x4 = x.reshape((-1, 1, 1, x.shape[-1])) if x.ndim != 4 else x
        out = np.empty_like(x4)
        if self.kind == "port":
            self.lib.orc_activation(_p(out), _p(x4), C.c_size_t(x4.size), self.FUNCS[func], int(derivative))
        else:
            assert self.lib.ref_activation(_p(out), _p(x4), x4.shape[0], x4.shape[1], x4.shape[2], x4.shape[3],
                                           self.FUNCS[func], int(derivative)) == 0
        return out.reshape(x.shape)

    # ---- layer-level sequences ---------------------------------------------------------------------
    # port: the plain-C restatement.  reference: the reference's own CTensorMath<float> routines called in
    # the batch-normalisation layer's order (its class does not compile at the reference's head revision),
    # and the reference's own CNetLayerVAECoderOutput<float> object.
    def bn_forward(self, x, gamma, beta, momentum=0.9, eps=1e-6, new_mean=None, new_var=None):
        x, gamma, beta = _c(x), _c(gamma), _c(beta)
        W = x.shape[0]
        n = x[0].size
        y, xhat = np.empty_like(x), np.empty_like(x)
        ivar, mean, var = (np.empty(x.shape[1:], np.float32) for _ in range(3))
        nm = _c(new_mean).copy() if new_mean is not None else None
        nv = _c(new_var).copy() if new_var is not None else None
        if self.kind == "port":
            self.lib.orc_bn_forward(_p(y), _p(xhat), _p(ivar), _p(mean), _p(var),
                                    _p(nm) if nm is not None else None, _p(nv) if nv is not None else None,
                                    _p(x), _p(gamma), _p(beta), W, C.c_size_t(n), C.c_float(momentum), C.c_float(eps))
        else:
            zyx = (tuple(x.shape[1:]) + (1, 1, 1))[:3] if x.ndim < 4 else x.shape[1:]
            assert self.lib.ref_bn_forward(_p(y), _p(xhat), _p(ivar), _p(mean), _p(var),
                                           _p(nm) if nm is not None else None, _p(nv) if nv is not None else None,
                                           _p(x), _p(gamma), _p(beta), W, zyx[0], zyx[1], zyx[2], C.c_float(momentum),
                                           C.c_double(eps)) == 0
        return dict(y=y, xhat=xhat, ivar=ivar, mean=mean, var=var, new_mean=nm, new_var=nv)

    def bn_backward(self, dy, xhat, ivar, gamma, dgamma=None, dbeta=None):
        dy, xhat, ivar, gamma = _c(dy), _c(xhat), _c(ivar), _c(gamma)
        W = dy.shape[0]
        n = dy[0].size
        dx = np.empty_like(dy)
        dg = _c(dgamma).copy() if dgamma is not None else np.zeros(dy.shape[1:], np.float32)
        db = _c(dbeta).copy() if dbeta is not None else np.zeros(dy.shape[1:], np.float32)
        if self.kind == "port":
            self.lib.orc_bn_backward(_p(dx), _p(dg), _p(db), _p(dy), _p(xhat), _p(ivar), _p(gamma), W, C.c_size_t(n), 1)
        else:
            zyx = (tuple(dy.shape[1:]) + (1, 1, 1))[:3] if dy.ndim < 4 else dy.shape[1:]
            assert self.lib.ref_bn_backward(_p(dx), _p(dg), _p(db), _p(dy), _p(xhat), _p(ivar), _p(gamma), W, zyx[0], zyx[1],
                                            zyx[2], 1) == 0
        return dx, dg, db

    def vae_forward(self, mu, logvar, eps):
        assert self.kind == "port"
        mu, logvar, eps = _c(mu), _c(logvar), _c(eps)
        z = np.empty_like(mu)
        kl = self.lib.orc_vae_forward(_p(z), _p(mu), _p(logvar), _p(eps), mu.shape[0], C.c_size_t(mu[0].size))
        return z, float(kl)

    def vae_backward(self, delta, mu, logvar, eps, k):
        assert self.kind == "port"
        delta, mu, logvar, eps = _c(delta), _c(mu), _c(logvar), _c(eps)
        dmu, dlv = np.empty_like(mu), np.empty_like(mu)
        self.lib.orc_vae_backward(_p(dmu), _p(dlv), _p(delta), _p(mu), _p(logvar), _p(eps), C.c_size_t(mu.size),
                                  C.c_float(k))
        return dmu, dlv

    def vae_layer(self, mu, logvar, delta, k):
        """reference only: one Forward + SetOutputError of the reference's own VAE output layer object.  The layer draws
        its noise from an unseedable generator, so the noise it used is returned with its results:
        (z, eps, d_mu, d_logvar); feed eps to vae_forward / vae_backward of the port to compare."""
        assert self.kind == "reference"
        mu, logvar, delta = _c(mu), _c(logvar), _c(delta)
        shape4 = (mu.shape + (1, 1, 1))[:4]
        z, eps, dmu, dlv = (np.empty_like(mu) for _ in range(4))
        devnull = os.open(os.devnull, os.O_WRONLY)       # the layer prints its KL loss to the console
        keep = os.dup(1)
        os.dup2(devnull, 1)
        try:
            r = self.lib.ref_vae_layer(_p(z), _p(eps), _p(dmu), _p(dlv), _p(mu), _p(logvar), _p(delta), shape4[0], shape4[1],
                                       shape4[2], shape4[3], C.c_float(k))
        finally:
            os.dup2(keep, 1)
            os.close(keep)
            os.close(devnull)
        assert r == 0, r
        return z, eps, dmu, dlv

    def set_time_step(self, x, time_step):
        """port only (the reference has SetTimeStep on its CUDA backend alone)."""
        assert self.kind == "port"
        x = _c(x)
        t = np.ascontiguousarray(time_step, dtype=np.uint32).ravel()
        out = np.empty_like(x)
        self.lib.orc_set_time_step(_p(out), _p(x), t.ctypes.data_as(_u), x.shape[0], C.c_size_t(x[0].size))
        return out

    def noisy_image(self, image, noise, sa, so):
        assert self.kind == "port"
        image, noise, sa, so = _c(image), _c(noise), _c(sa).ravel(), _c(so).ravel()
        out = np.empty_like(image)
        self.lib.orc_noisy_image(_p(out), _p(image), _p(noise), _p(sa), _p(so), image.shape[0], C.c_size_t(image[0].size))
        return out

    def adam(self, weight, dweight, m, v, batch_size, speed, beta1, beta2, epsilon, iteration):
        weight, dweight, m, v = _c(weight).copy(), _c(dweight), _c(m).copy(), _c(v).copy()
        n = weight.size
        args = (_p(weight), _p(dweight), _p(m), _p(v))
        tail = (C.c_uint32(batch_size), C.c_double(speed), C.c_double(beta1), C.c_double(beta2),
                C.c_double(epsilon), C.c_double(iteration))
        if self.kind == "port":
            self.lib.orc_adam(*args, C.c_size_t(n), *tail)
        else:
            assert self.lib.ref_adam(*args, n, *tail) == 0
        return weight, m, v
