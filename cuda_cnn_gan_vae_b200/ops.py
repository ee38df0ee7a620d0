"""Host-side mirror of the reference tensor-math interface on torch CUDA tensors.

Names, argument order and error behaviour follow the reference's static classes
(cuda/ctensorconv.cu.h:63-66, cuda/ctensormath.cu.h:92-135, cuda/ctensorapplyfunc.cu.h:78-90):
the output tensor comes first and is pre-sized by the caller, tensors are 4-D (W,Z,Y,X) fp32,
operands broadcast over W by modulo, and a shape error raises B200Error carrying the library's
message (the reference throws a C string).  All work happens in libb200conv.so on the current
torch CUDA stream; nothing here computes.
"""
import ctypes as C

import torch

from .lib import ConvGeom, load

TF32X3, TF32, FP32 = 0, 1, 2
PATH_SIMT, PATH_TCGEN05 = 1, 2
ACT = {"sigmoid": 0, "relu": 1, "leaky_relu": 2, "linear": 3, "tanh": 4, "gelu": 5}


class B200Error(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"b200conv error {code}: {text}")
        self.code = code


def _check(code):
    if code != 0:
        raise B200Error(code, load().b200_last_error().decode(errors="replace"))


def _t(x, name="tensor"):
    if not (isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()):
        raise B200Error(2, f"{name} must be a contiguous fp32 CUDA tensor")
    return x


def _ptr(x):
    return C.c_void_p(x.data_ptr()) if x is not None else None


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def set_precision(mode):
    _check(load().b200_set_precision(mode))


def get_precision():
    return load().b200_get_precision()


def last_path():
    return load().b200_last_path()


def stream_status():
    """Synchronises the current stream and raises if a kernel recorded a failure."""
    _check(load().b200_stream_status(_stream()))


def geom(in_z, in_y, in_x, kernel_amount, kernel_x, kernel_y, stride_x, stride_y, padding_x, padding_y, out_y=None, out_x=None):
    if out_y is None:
        out_y = (in_y - kernel_y + 2 * padding_y) // stride_y + 1
    if out_x is None:
        out_x = (in_x - kernel_x + 2 * padding_x) // stride_x + 1
    return ConvGeom(in_z, in_y, in_x, kernel_amount, kernel_y, kernel_x, stride_y, stride_x, padding_y, padding_x, out_y, out_x)


class CTensorConv:
    """cuda/ctensorconv.cu.h:63-66."""

    @staticmethod
    def ForwardConvolution(output, image, kernel, kernel_x, kernel_y, kernel_z, kernel_amount, bias,
                           stride_x, stride_y, padding_x, padding_y):
        _t(output), _t(image), _t(kernel), _t(bias)
        if bias.shape[1] != kernel_amount:
            raise B200Error(1, "the number of kernels and biases must match")
        if image.shape[1] != kernel_z:
            raise B200Error(1, "filter depth and image depth must match")
        if kernel.shape[2] != kernel_amount or kernel.shape[3] != kernel_x * kernel_y * kernel_z:
            raise B200Error(1, "kernel tensor must be [Wk,1,K,C*ky*kx]")
        if output.shape[1] != kernel_amount:
            raise B200Error(1, "wrong output depth for convolution")
        g = geom(kernel_z, image.shape[2], image.shape[3], kernel_amount, kernel_x, kernel_y, stride_x, stride_y,
                 padding_x, padding_y, output.shape[2], output.shape[3])
        _check(load().b200_conv_forward(C.byref(g), _ptr(output), output.shape[0], _ptr(image), image.shape[0],
                                        _ptr(kernel), kernel.shape[0], _ptr(bias), bias.shape[0], _stream()))

    @staticmethod
    def BackwardConvolution(output_delta, delta, kernel, kernel_x, kernel_y, kernel_z, kernel_amount, bias,
                            stride_x, stride_y, padding_x, padding_y):
        """bias=None stands for the all-zero bias every reference caller passes."""
        _t(output_delta), _t(delta), _t(kernel)
        if delta.shape[1] != kernel_amount:
            raise B200Error(1, "the number of filters and the delta depth must match")
        if output_delta.shape[1] != kernel_z:
            raise B200Error(1, "wrong output depth for backward convolution")
        g = geom(kernel_z, output_delta.shape[2], output_delta.shape[3], kernel_amount, kernel_x, kernel_y, stride_x,
                 stride_y, padding_x, padding_y, delta.shape[2], delta.shape[3])
        _check(load().b200_conv_backward(C.byref(g), _ptr(output_delta), output_delta.shape[0], _ptr(delta), delta.shape[0],
                                         _ptr(kernel), kernel.shape[0], _ptr(bias) if bias is not None else None,
                                         bias.shape[0] if bias is not None else 0, _stream()))

    @staticmethod
    def _wgrad(fn, dkernel, kx, ky, kz, amount, dbias, image, delta, sx, sy, px, py, in_yx, out_yx):
        _t(dkernel), _t(dbias), _t(image), _t(delta)
        if dbias.shape[1] != amount:
            raise B200Error(1, "the number of kernel and bias corrections must match")
        g = geom(kz, in_yx[0], in_yx[1], amount, kx, ky, sx, sy, px, py, out_yx[0], out_yx[1])
        _check(fn(C.byref(g), _ptr(dkernel), dkernel.shape[0], _ptr(dbias), dbias.shape[0], _ptr(image), image.shape[0],
                  _ptr(delta), delta.shape[0], _stream()))

    @staticmethod
    def CreateDeltaWeightAndBias(dkernel, dkernel_x, dkernel_y, dkernel_z, dkernel_amount, dbias, image, delta,
                                 stride_x, stride_y, padding_x, padding_y):
        if image.shape[1] != dkernel_z or delta.shape[1] != dkernel_amount:
            raise B200Error(1, "image / delta depth does not match the kernel corrections")
        CTensorConv._wgrad(load().b200_conv_wgrad, dkernel, dkernel_x, dkernel_y, dkernel_z, dkernel_amount, dbias, image,
                           delta, stride_x, stride_y, padding_x, padding_y, image.shape[2:], delta.shape[2:])

    @staticmethod
    def CreateBackDeltaWeightAndBias(dkernel, dkernel_x, dkernel_y, dkernel_z, dkernel_amount, dbias, image, delta,
                                     stride_x, stride_y, padding_x, padding_y):
        if image.shape[1] != dkernel_amount or delta.shape[1] != dkernel_z:
            raise B200Error(1, "image / delta depth does not match the kernel corrections")
        CTensorConv._wgrad(load().b200_conv_back_wgrad, dkernel, dkernel_x, dkernel_y, dkernel_z, dkernel_amount, dbias,
                           image, delta, stride_x, stride_y, padding_x, padding_y, delta.shape[2:], image.shape[2:])

    @staticmethod
    def CreateDeltaWeightAndBiasBatch(dkernel, dkernel_x, dkernel_y, dkernel_z, dkernel_amount, dbias, image, delta,
                                      stride_x, stride_y, padding_x, padding_y, accumulate=True):
        """Batch-summed form used by the layers: dkernel [1,1,K,C*ky*kx] (+)= sum over the batch."""
        _t(dkernel), _t(image), _t(delta)
        g = geom(dkernel_z, image.shape[2], image.shape[3], dkernel_amount, dkernel_x, dkernel_y, stride_x, stride_y,
                 padding_x, padding_y, delta.shape[2], delta.shape[3])
        if image.shape[0] != delta.shape[0]:
            raise B200Error(1, "image and delta batch sizes differ")
        _check(load().b200_conv_wgrad_batch(C.byref(g), _ptr(dkernel), _ptr(dbias) if dbias is not None else None,
                                            int(accumulate), _ptr(image), _ptr(delta), image.shape[0], _stream()))


def _n(x):
    return x.shape[1] * x.shape[2] * x.shape[3]


def _same_zyx(*ts):
    s = ts[0].shape[1:]
    if any(t.shape[1:] != s for t in ts):
        raise B200Error(1, "tensor sizes do not match")


class CTensorMath:
    """cuda/ctensormath.cu.h:92-135."""

    @staticmethod
    def Mul(output, left, right, tensor_core=False):
        _t(output), _t(left), _t(right)
        if left.shape[3] != right.shape[2] or left.shape[1] != right.shape[1] or output.shape[2] != left.shape[2] or \
                output.shape[3] != right.shape[3] or output.shape[1] != right.shape[1]:
            raise B200Error(1, "CTensor::Mul: tensor sizes do not match")
        _check(load().b200_mul(_ptr(output), output.shape[0], _ptr(left), left.shape[0], _ptr(right), right.shape[0],
                               left.shape[1], left.shape[2], left.shape[3], right.shape[3], 0, _stream()))

    @staticmethod
    def TransponseMul(output, left, right, tensor_core=False):
        _t(output), _t(left), _t(right)
        if left.shape[2] != right.shape[2] or left.shape[1] != right.shape[1] or output.shape[2] != left.shape[3] or \
                output.shape[3] != right.shape[3] or output.shape[1] != right.shape[1]:
            raise B200Error(1, "CTensor::TransponseMul: tensor sizes do not match")
        _check(load().b200_mul(_ptr(output), output.shape[0], _ptr(left), left.shape[0], _ptr(right), right.shape[0],
                               left.shape[1], left.shape[2], left.shape[3], right.shape[3], 1, _stream()))

    @staticmethod
    def MulValue(output, inp, value):
        _t(output), _t(inp)
        _same_zyx(output, inp)
        _check(load().b200_unary(_ptr(output), output.shape[0], _ptr(inp), inp.shape[0], _n(output), 3, value, 0.0, _stream()))

    @staticmethod
    def Add(output, left, right, left_scale=1.0, right_scale=1.0):
        _t(output), _t(left), _t(right)
        _same_zyx(output, left, right)
        _check(load().b200_add(_ptr(output), output.shape[0], _ptr(left), left.shape[0], _ptr(right), right.shape[0],
                               _n(output), left_scale, right_scale, 0, _stream()))

    @staticmethod
    def Sub(output, left, right, left_scale=1.0, right_scale=1.0):
        _t(output), _t(left), _t(right)
        _same_zyx(output, left, right)
        _check(load().b200_add(_ptr(output), output.shape[0], _ptr(left), left.shape[0], _ptr(right), right.shape[0],
                               _n(output), left_scale, right_scale, 1, _stream()))

    @staticmethod
    def AddSumW(output, left, right, left_scale=1.0, right_scale=1.0):
        _t(output), _t(left), _t(right)
        _same_zyx(output, left, right)
        _check(load().b200_add_sum_w(_ptr(output), output.shape[0], _ptr(left), left.shape[0], _ptr(right), right.shape[0],
                                     _n(output), left_scale, right_scale, _stream()))

    @staticmethod
    def AddBias(working, bias):
        _t(working), _t(bias)
        if working.shape[1] != bias.shape[1]:
            raise B200Error(1, "CTensor::AddBias: tensor sizes do not match")
        _check(load().b200_add_bias(_ptr(working), working.shape[0], working.shape[1], working.shape[2] * working.shape[3],
                                    _ptr(bias), bias.shape[0], _stream()))

    @staticmethod
    def SummXY(output, inp):
        _t(output), _t(inp)
        if output.shape[1] != inp.shape[1]:
            raise B200Error(1, "CTensor::SummXY: tensor sizes do not match")
        _check(load().b200_summ_xy(_ptr(output), output.shape[0], _ptr(inp), inp.shape[0], inp.shape[1],
                                   inp.shape[2] * inp.shape[3], _stream()))

    @staticmethod
    def _unary(op, output, inp, a, b):
        _t(output), _t(inp)
        _same_zyx(output, inp)
        _check(load().b200_unary(_ptr(output), output.shape[0], _ptr(inp), inp.shape[0], _n(output), op, a, b, _stream()))

    @staticmethod
    def Pow2(output, inp, scale=1.0):
        CTensorMath._unary(0, output, inp, scale, 0.0)

    @staticmethod
    def SQRT(output, inp, scale, add_sqrt_value):
        CTensorMath._unary(1, output, inp, scale, add_sqrt_value)

    @staticmethod
    def Inv(output, inp):
        CTensorMath._unary(2, output, inp, 0.0, 0.0)

    @staticmethod
    def Set(output, inp, scale=1.0, add_value=0.0):
        """output = input*scale + add_value (cuda/ctensormath.cu.h: Set, AddValue, SubValue)."""
        CTensorMath._unary(4, output, inp, scale, add_value)

    @staticmethod
    def Clip(tensor, min_value, max_value):
        CTensorMath._unary(5, tensor, tensor, min_value, max_value)

    @staticmethod
    def Signum(tensor):
        CTensorMath._unary(6, tensor, tensor, 0.0, 0.0)

    @staticmethod
    def Div(output, left, right, left_scale=1.0, right_scale=1.0):
        """output = (left*left_scale) / (right*right_scale), W broadcast per operand."""
        _t(output), _t(left), _t(right)
        _same_zyx(output, left, right)
        _check(load().b200_div(_ptr(output), output.shape[0], _ptr(left), left.shape[0], _ptr(right), right.shape[0],
                               _n(output), left_scale, right_scale, _stream()))

    @staticmethod
    def Transponse(output, inp):
        """Every (w,z) plane transposed: output is [W,Z,X,Y] for an input [W,Z,Y,X]."""
        _t(output), _t(inp)
        if output.shape[0] != inp.shape[0] or output.shape[1] != inp.shape[1] or output.shape[2] != inp.shape[3] or output.shape[3] != inp.shape[2]:
            raise B200Error("CTensorMath::Transponse: tensor sizes do not match!")
        _check(load().b200_transpose(_ptr(output), _ptr(inp), inp.shape[0] * inp.shape[1], inp.shape[2], inp.shape[3], _stream()))

    @staticmethod
    def ConcatecationZ(output, input_a, input_b):
        _t(output), _t(input_a), _t(input_b)
        if output.shape[2:] != input_a.shape[2:] or output.shape[2:] != input_b.shape[2:] or \
                output.shape[1] != input_a.shape[1] + input_b.shape[1]:
            raise B200Error(1, "CTensor::ConcatecationZ: tensor sizes do not match")
        _check(load().b200_concat_z(_ptr(output), output.shape[0], _ptr(input_a), input_a.shape[0], input_a.shape[1], _ptr(input_b),
                                    input_b.shape[0], input_b.shape[1], output.shape[2] * output.shape[3], _stream()))

    @staticmethod
    def SplitZ(output_a, output_b, inp):
        _t(output_a), _t(output_b), _t(inp)
        if inp.shape[2:] != output_a.shape[2:] or inp.shape[2:] != output_b.shape[2:] or inp.shape[0] != output_a.shape[0] or \
                inp.shape[0] != output_b.shape[0] or inp.shape[1] != output_a.shape[1] + output_b.shape[1]:
            raise B200Error(1, "CTensor::SplitZ: tensor sizes do not match")
        _check(load().b200_split_z(_ptr(output_a), output_a.shape[1], _ptr(output_b), output_b.shape[1], _ptr(inp), inp.shape[0],
                                   inp.shape[2] * inp.shape[3], _stream()))

    @staticmethod
    def SetTimeStep(output, inp, time_step):
        """time_step: uint32 (torch.int32 storage) tensor [W,1,1,1] (cuda/ctensormath.cu.h:3061)."""
        _t(output), _t(inp)
        if output.shape != inp.shape or time_step.numel() != inp.shape[0] or time_step.dtype != torch.int32:
            raise B200Error(1, "CTensor::SetTimeStep: tensor sizes do not match")
        _check(load().b200_set_time_step(_ptr(output), _ptr(inp), _ptr(time_step), inp.shape[0], _n(inp), _stream()))

    @staticmethod
    def SetNormalNoise(output, seed):
        _t(output)
        _check(load().b200_normal_noise(_ptr(output), output.numel(), seed, _stream()))

    @staticmethod
    def CreateDropOutMatrix(output, drop_out, seed):
        _t(output)
        _check(load().b200_dropout_mask(_ptr(output), output.numel(), drop_out, seed, _stream()))

    @staticmethod
    def GetNoiseImageAndNoise(noisy_image, noise, image, sqrt_alpha_bar, sqrt_one_minus_alpha_bar, seed=None):
        """seed given: the noise is drawn and written to `noise` (the reference's behaviour, cuda/ctensormath.cu.h:3250);
        seed None: `noise` is an input supplied by the caller."""
        _t(noisy_image), _t(noise), _t(image), _t(sqrt_alpha_bar), _t(sqrt_one_minus_alpha_bar)
        if noisy_image.shape != noise.shape or noisy_image.shape != image.shape:
            raise B200Error(1, "CTensor::GetNoiseImageAndNoise: the sizes of NoisyImage, Noise and Image do not match")
        if sqrt_alpha_bar.numel() != image.shape[0] or sqrt_one_minus_alpha_bar.numel() != image.shape[0]:
            raise B200Error(1, "CTensor::GetNoiseImageAndNoise: the sizes of SqrtAlphaBar/SqrtOneMinusAlphaBar and Image do not match")
        _check(load().b200_noisy_image(_ptr(noisy_image), _ptr(noise), _ptr(image), _ptr(sqrt_alpha_bar), _ptr(sqrt_one_minus_alpha_bar),
                                       image.shape[0], _n(image), int(seed is not None), seed or 0, _stream()))

    @staticmethod
    def TensorItemProduction(output, left, right):
        _t(output), _t(left), _t(right)
        _same_zyx(output, left, right)
        _check(load().b200_item_product(_ptr(output), output.shape[0], _ptr(left), left.shape[0], _ptr(right),
                                        right.shape[0], _n(output), _stream()))

    @staticmethod
    def Fill(output, value=0.0):
        _t(output)
        _check(load().b200_fill(_ptr(output), output.numel(), value, _stream()))

    @staticmethod
    def MaxPooling(output, position, inp, pooling_x, pooling_y):
        _t(output), _t(inp)
        if inp.shape[3] // pooling_x != output.shape[3] or inp.shape[2] // pooling_y != output.shape[2] or \
                inp.shape[:2] != output.shape[:2]:
            raise B200Error(1, "CTensor::MaxPooling: tensor sizes do not match")
        _check(load().b200_maxpool(_ptr(output), _ptr(position), _ptr(inp), inp.shape[0], inp.shape[1], inp.shape[2],
                                   inp.shape[3], pooling_x, pooling_y, _stream()))

    @staticmethod
    def MaxPoolingBackward(output, position, inp, pooling_x, pooling_y):
        _t(output), _t(inp)
        if inp.shape[3] != output.shape[3] // pooling_x or inp.shape[2] != output.shape[2] // pooling_y or \
                inp.shape[:2] != output.shape[:2]:
            raise B200Error(1, "CTensor::MaxPooling: tensor sizes do not match")
        _check(load().b200_maxpool_backward(_ptr(output), _ptr(position), _ptr(inp), output.shape[0], output.shape[1],
                                            output.shape[2], output.shape[3], pooling_x, pooling_y, _stream()))

    @staticmethod
    def UpSampling(output, inp, upsampling_x, upsampling_y):
        _t(output), _t(inp)
        if inp.shape[3] != output.shape[3] // upsampling_x or inp.shape[2] != output.shape[2] // upsampling_y or \
                inp.shape[1] != output.shape[1]:
            raise B200Error(1, "CTensor::UpSampling: tensor sizes do not match")
        _check(load().b200_upsample(_ptr(output), _ptr(inp), inp.shape[0], inp.shape[1], inp.shape[2], inp.shape[3],
                                    upsampling_x, upsampling_y, _stream()))

    @staticmethod
    def DownSampling(output, inp, downsampling_x, downsampling_y):
        _t(output), _t(inp)
        if inp.shape[3] // downsampling_x != output.shape[3] or inp.shape[2] // downsampling_y != output.shape[2] or \
                inp.shape[:2] != output.shape[:2]:
            raise B200Error(1, "CTensor::DownSampling: tensor sizes do not match")
        _check(load().b200_downsample(_ptr(output), _ptr(inp), inp.shape[0], inp.shape[1], inp.shape[2], inp.shape[3],
                                      downsampling_x, downsampling_y, _stream()))

    @staticmethod
    def Adam(weight, dweight, m, v, batch_size, speed, beta1, beta2, epsilon, iteration):
        _t(weight), _t(dweight), _t(m), _t(v)
        if not (weight.shape == dweight.shape == m.shape == v.shape):
            raise B200Error(1, "CTensor::Adam: tensor sizes do not match")
        _check(load().b200_adam(_ptr(weight), _ptr(dweight), _ptr(m), _ptr(v), weight.numel(), batch_size, speed, beta1,
                                beta2, epsilon, iteration, _stream()))


class CTensorApplyFunc:
    """cuda/ctensorapplyfunc.cu.h:78-90; `func` is one of ACT."""

    @staticmethod
    def Apply(output, inp, func, leaky_slope=0.1):
        _t(output), _t(inp)
        _check(load().b200_activation(_ptr(output), _ptr(inp), inp.numel(), ACT[func], 0, leaky_slope, _stream()))

    @staticmethod
    def ApplyDifferential(output, inp, func, leaky_slope=0.1):
        _t(output), _t(inp)
        _check(load().b200_activation(_ptr(output), _ptr(inp), inp.numel(), ACT[func], 1, leaky_slope, _stream()))

    @staticmethod
    def Backward(output, z, error, func, leaky_slope=0.1):
        _t(output), _t(z), _t(error)
        _check(load().b200_activation_backward(_ptr(output), _ptr(z), _ptr(error), z.numel(), ACT[func], leaky_slope, _stream()))

    @staticmethod
    def BiasActivation(working, bias, func, leaky_slope=0.1, pre=None):
        _t(working), _t(bias)
        _check(load().b200_bias_activation(_ptr(working), _ptr(pre) if pre is not None else None, working.shape[0],
                                           working.shape[1], working.shape[2] * working.shape[3], _ptr(bias), ACT[func],
                                           leaky_slope, _stream()))


def bn_forward(x, gamma, beta, momentum=0.9, eps=1e-6, new_mean=None, new_var=None):
    """CNetLayerBatchNormalization::Forward (training).  Returns dict(y, xhat, ivar, mean, var)."""
    _t(x), _t(gamma), _t(beta)
    y, xhat = torch.empty_like(x), torch.empty_like(x)
    ivar, mean, var = (torch.empty_like(gamma) for _ in range(3))
    _check(load().b200_bn_forward(_ptr(y), _ptr(xhat), _ptr(ivar), _ptr(mean), _ptr(var),
                                  _ptr(new_mean) if new_mean is not None else None,
                                  _ptr(new_var) if new_var is not None else None, _ptr(x), _ptr(gamma), _ptr(beta),
                                  x.shape[0], x[0].numel(), momentum, eps, _stream()))
    return dict(y=y, xhat=xhat, ivar=ivar, mean=mean, var=var)


def bn_backward(dy, xhat, ivar, gamma, dgamma, dbeta, create_delta_weight=True):
    _t(dy), _t(xhat), _t(ivar), _t(gamma)
    dx = torch.empty_like(dy)
    _check(load().b200_bn_backward(_ptr(dx), _ptr(dgamma), _ptr(dbeta), _ptr(dy), _ptr(xhat), _ptr(ivar), _ptr(gamma),
                                   dy.shape[0], dy[0].numel(), int(create_delta_weight), _stream()))
    return dx


def vae_forward(mu, logvar, eps, want_kl=True):
    _t(mu), _t(logvar), _t(eps)
    z = torch.empty_like(mu)
    kl = C.c_float(0.0)
    _check(load().b200_vae_forward(_ptr(z), _ptr(mu), _ptr(logvar), _ptr(eps), mu.shape[0], mu[0].numel(),
                                   C.byref(kl) if want_kl else None, _stream()))
    return z, kl.value


def vae_backward(delta, mu, logvar, eps, kl_speed):
    _t(delta), _t(mu), _t(logvar), _t(eps)
    dmu, dlv = torch.empty_like(mu), torch.empty_like(mu)
    _check(load().b200_vae_backward(_ptr(dmu), _ptr(dlv), _ptr(delta), _ptr(mu), _ptr(logvar), _ptr(eps), mu.numel(),
                                    kl_speed, _stream()))
    return dmu, dlv


def prepack_conv_layers(layers, kernels):
    """b200_conv_layers_prepack: the tensor-core weight packs of several ConvLayer objects in one launch, each good for the
    layer's next forward call with that kernel tensor."""
    if not layers:
        return
    handles = (C.c_void_p * len(layers))(*[layer._h for layer in layers])
    pointers = (C.c_void_p * len(layers))(*[_t(k).data_ptr() for k in kernels])
    _check(load().b200_conv_layers_prepack(handles, pointers, len(layers), _stream()))


class ConvLayer:
    """Forward / TrainingBackward of the reference's convolution layer (netlayer/cnetlayerconvolution.cu.h:310,484)
    or, with transposed=True, of its transposed-convolution layer (netlayer/cnetlayerbackconvolution.cu.h:303,475).
    The library context keeps the packed layer input between the two calls."""

    def __init__(self, in_z, in_y, in_x, kernel_amount, kernel_x, kernel_y, stride_x, stride_y, padding_x, padding_y, batch,
                 transposed=False):
        self.g = geom(in_z, in_y, in_x, kernel_amount, kernel_x, kernel_y, stride_x, stride_y, padding_x, padding_y)
        self.batch, self.transposed = batch, transposed
        self._h = C.c_void_p()
        _check(load().b200_conv_layer_create(C.byref(self._h), C.byref(self.g), batch, int(transposed)))

    def forward(self, output, inp, kernel, bias=None):
        _t(output), _t(inp), _t(kernel)
        _check(load().b200_conv_layer_forward(self._h, _ptr(output), _ptr(inp), _ptr(kernel),
                                              _ptr(bias) if bias is not None else None, _stream()))

    def forward_fused(self, output, inp, kernel, bias=None, input_func=None, input_slope=0.1, input_act_out=None, output_func=None,
                      output_slope=0.1, output_pre=None):
        """b200_conv_layer_forward_fused: input_func is the function layer in front of this layer (applied while the input is
        packed; input_act_out optionally receives f(inp)), output_func the one behind it (applied in the epilogue; output_pre
        optionally receives the value before the function)."""
        from .lib import ConvFusion
        _t(output), _t(inp), _t(kernel)
        f = ConvFusion(ACT[input_func] if input_func else -1, input_slope, input_act_out.data_ptr() if input_act_out is not None else None,
                       ACT[output_func] if output_func else -1, output_slope, output_pre.data_ptr() if output_pre is not None else None)
        _check(load().b200_conv_layer_forward_fused(self._h, _ptr(output), _ptr(inp), _ptr(kernel), _ptr(bias) if bias is not None else None,
                                                    C.byref(f), _stream()))

    def backward(self, input_delta, dkernel, dbias, output_delta, inp, kernel, accumulate=True):
        _t(output_delta), _t(inp), _t(kernel)
        _check(load().b200_conv_layer_backward(self._h, _ptr(input_delta) if input_delta is not None else None,
                                               _ptr(dkernel) if dkernel is not None else None,
                                               _ptr(dbias) if dbias is not None else None, int(accumulate),
                                               _ptr(output_delta), _ptr(inp), _ptr(kernel), _stream()))

    def close(self):
        if self._h:
            load().b200_conv_layer_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
