"""ctypes binding of libb200conv.so: one Python callable per symbol of include/b200conv.h."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200conv.so")


class ConvGeom(C.Structure):
    """struct b200_conv_geom."""
    _fields_ = [(n, C.c_int) for n in ("in_z", "in_y", "in_x", "kernel_amount", "kernel_y", "kernel_x", "stride_y",
                                       "stride_x", "padding_y", "padding_x", "out_y", "out_x")]


_fp, _vp, _i, _sz, _f, _d = C.c_void_p, C.c_void_p, C.c_int, C.c_size_t, C.c_float, C.c_double


class ExchangeSegment(C.Structure):
    """struct b200_exchange_segment."""
    _fields_ = [("grad_offset", C.c_size_t), ("weight_offset", C.c_size_t), ("n", C.c_size_t), ("m", C.c_void_p), ("v", C.c_void_p)]


class ConvFusion(C.Structure):
    """struct b200_conv_fusion."""
    _fields_ = [("input_func", C.c_int), ("input_slope", C.c_double), ("input_act_out", C.c_void_p), ("output_func", C.c_int),
                ("output_slope", C.c_double), ("output_pre", C.c_void_p)]
_G = C.POINTER(ConvGeom)

# name -> (restype, argtypes); must list every function declared in include/b200conv.h
SIGNATURES = {
    "b200_last_error": (C.c_char_p, []),
    "b200_last_path": (_i, []),
    "b200_set_precision": (_i, [_i]),
    "b200_get_precision": (_i, []),
    "b200_shutdown": (_i, []),
    "b200_scratch_bytes": (_sz, []),
    "b200_stream_status": (_i, [_vp]),
    "b200_debug_set_status": (_i, [C.c_uint]),
    "b200_launch_count": (C.c_ulonglong, []),
    "b200_profile_tensor_core": (_i, [_i]),
    "b200_profile_read": (_i, [C.POINTER(C.c_double), C.POINTER(C.c_int)]),
    "b200_conv_forward": (_i, [_G, _fp, _i, _fp, _i, _fp, _i, _fp, _i, _vp]),
    "b200_conv_backward": (_i, [_G, _fp, _i, _fp, _i, _fp, _i, _fp, _i, _vp]),
    "b200_conv_wgrad": (_i, [_G, _fp, _i, _fp, _i, _fp, _i, _fp, _i, _vp]),
    "b200_conv_back_wgrad": (_i, [_G, _fp, _i, _fp, _i, _fp, _i, _fp, _i, _vp]),
    "b200_conv_wgrad_batch": (_i, [_G, _fp, _fp, _i, _fp, _fp, _i, _vp]),
    "b200_conv_layer_create": (_i, [C.POINTER(C.c_void_p), _G, _i, _i]),
    "b200_conv_layer_destroy": (_i, [_vp]),
    "b200_conv_layer_forward": (_i, [_vp, _fp, _fp, _fp, _fp, _vp]),
    "b200_conv_layer_forward_fused": (_i, [_vp, _fp, _fp, _fp, _fp, _vp, _vp]),
    "b200_conv_layers_prepack": (_i, [_vp, _vp, _i, _vp]),
    "b200_conv_layer_backward": (_i, [_vp, _fp, _fp, _fp, _i, _fp, _fp, _fp, _vp]),
    "b200_conv_wgrad_batch_static": (_i, [_G, _fp, _fp, _i, _fp, _fp, _i, _vp]),
    "b200_static_scratch_bytes": (_sz, []),
    "b200_mul": (_i, [_fp, _i, _fp, _i, _fp, _i, _i, _i, _i, _i, _i, _vp]),
    "b200_add": (_i, [_fp, _i, _fp, _i, _fp, _i, _sz, _f, _f, _i, _vp]),
    "b200_add_sum_w": (_i, [_fp, _i, _fp, _i, _fp, _i, _sz, _f, _f, _vp]),
    "b200_add_bias": (_i, [_fp, _i, _i, _sz, _fp, _i, _vp]),
    "b200_summ_xy": (_i, [_fp, _i, _fp, _i, _i, _sz, _vp]),
    "b200_unary": (_i, [_fp, _i, _fp, _i, _sz, _i, _f, _f, _vp]),
    "b200_div": (_i, [_fp, _i, _fp, _i, _fp, _i, _sz, _f, _f, _vp]),
    "b200_transpose": (_i, [_fp, _fp, _i, _i, _i, _vp]),
    "b200_item_product": (_i, [_fp, _i, _fp, _i, _fp, _i, _sz, _vp]),
    "b200_fill": (_i, [_fp, _sz, _f, _vp]),
    "b200_activation": (_i, [_fp, _fp, _sz, _i, _i, _d, _vp]),
    "b200_activation_backward": (_i, [_fp, _fp, _fp, _sz, _i, _d, _vp]),
    "b200_bias_activation": (_i, [_fp, _fp, _i, _i, _sz, _fp, _i, _d, _vp]),
    "b200_maxpool": (_i, [_fp, _fp, _fp, _i, _i, _i, _i, _i, _i, _vp]),
    "b200_maxpool_backward": (_i, [_fp, _fp, _fp, _i, _i, _i, _i, _i, _i, _vp]),
    "b200_upsample": (_i, [_fp, _fp, _i, _i, _i, _i, _i, _i, _vp]),
    "b200_downsample": (_i, [_fp, _fp, _i, _i, _i, _i, _i, _i, _vp]),
    "b200_concat_z": (_i, [_fp, _i, _fp, _i, _i, _fp, _i, _i, _sz, _vp]),
    "b200_split_z": (_i, [_fp, _i, _fp, _i, _fp, _i, _sz, _vp]),
    "b200_bn_forward": (_i, [_fp] * 10 + [_i, _sz, _f, _f, _vp]),
    "b200_bn_backward": (_i, [_fp] * 7 + [_i, _sz, _i, _vp]),
    "b200_bn_act_forward": (_i, [_fp] * 10 + [_i, _sz, _f, _f, _i, _d, _vp]),
    "b200_bn_act_backward": (_i, [_fp] * 8 + [_i, _sz, _i, _i, _d, _vp]),
    "b200_vae_forward": (_i, [_fp, _fp, _fp, _fp, _i, _sz, C.POINTER(C.c_float), _vp]),
    "b200_vae_backward": (_i, [_fp] * 6 + [_sz, _f, _vp]),
    "b200_adam": (_i, [_fp, _fp, _fp, _fp, _sz, C.c_uint32, _d, _d, _d, _d, _d, _vp]),
    "b200_adam_prepared": (_i, [_fp, _fp, _fp, _fp, _sz, C.c_uint32, _d, _d, _d, _d, _vp, _vp]),
    "b200_set_time_step": (_i, [_fp, _fp, _vp, _i, _sz, _vp]),
    "b200_normal_noise": (_i, [_fp, _sz, C.c_ulonglong, _vp]),
    "b200_dropout_mask": (_i, [_fp, _sz, _f, C.c_ulonglong, _vp]),
    "b200_noisy_image": (_i, [_fp, _fp, _fp, _fp, _fp, _i, _sz, _i, C.c_ulonglong, _vp]),
    "b200_adam_ema": (_i, [_fp, _fp, _fp, _fp, _fp, _sz, C.c_uint32, _d, _d, _d, _d, _d, _vp, _d, _vp]),
    "b200_comm_create": (_i, [C.POINTER(C.c_void_p), _i, _i, _sz]),
    "b200_comm_handle": (_i, [_vp, _vp]),
    "b200_comm_connect": (_i, [_vp, _vp]),
    "b200_comm_buffer": (C.c_void_p, [_vp]),
    "b200_comm_buffer_bytes": (_sz, [_vp]),
    "b200_comm_destroy": (_i, [_vp]),
    "b200_comm_slice": (_i, [_sz, _i, _i, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "b200_allreduce": (_i, [_vp, _sz, _sz, _i, _vp]),
    "b200_allreduce_adam": (_i, [_vp, _sz, _sz, _fp, _fp, _sz, C.c_uint32, _d, _d, _d, _d, _d, _vp, _i, _vp]),
    "b200_allreduce_adam_multi": (_i, [_vp, _i, _vp, C.c_uint32, _d, _d, _d, _d, _d, _vp, _i, _vp]),
}

_lib = None


def load():
    """Loads the C-ABI library.  Raises if it has not been built: there is no fallback path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python -m cuda_cnn_gan_vae_b200.build` (nvcc, sm_100a)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
