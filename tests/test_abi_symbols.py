"""CPU-side checks of the C-ABI library: it loads without a GPU, exports every symbol that
include/b200conv.h declares, and rejects bad arguments with the documented codes before touching CUDA."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from cuda_cnn_gan_vae_b200 import build, lib as L
    build.build()
    return L.load()


def test_every_declared_symbol_is_exported(lib):
    from cuda_cnn_gan_vae_b200 import lib as L
    header = open(os.path.join(ROOT, "include", "b200conv.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(b200_\w+)\s*\(", header))
    assert len(declared) >= 30
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/b200conv.h but not exported"
    assert declared == set(L.SIGNATURES), "ctypes signature table out of sync with the header"


def test_precision_control(lib):
    assert lib.b200_get_precision() == 0
    assert lib.b200_set_precision(1) == 0 and lib.b200_get_precision() == 1
    assert lib.b200_set_precision(0) == 0
    assert lib.b200_set_precision(99) == 2            # B200_E_ARG
    assert b"precision" in lib.b200_last_error()


def test_argument_validation_needs_no_gpu(lib):
    from cuda_cnn_gan_vae_b200.lib import ConvGeom
    g = ConvGeom(3, 8, 8, 4, 3, 3, 1, 1, 1, 1, 8, 8)
    assert lib.b200_conv_forward(None, None, 1, None, 1, None, 1, None, 1, None) == 2
    assert lib.b200_conv_forward(C.byref(g), None, 1, None, 1, None, 1, None, 1, None) == 2      # null tensors
    bad = ConvGeom(3, 8, 8, 0, 3, 3, 1, 1, 1, 1, 8, 8)
    assert lib.b200_conv_forward(C.byref(bad), None, 1, None, 1, None, 1, None, 1, None) == 1    # no kernels
    assert b"at least one kernel" in lib.b200_last_error()
    wrong = ConvGeom(3, 8, 8, 4, 3, 3, 1, 1, 1, 1, 7, 8)
    assert lib.b200_conv_forward(C.byref(wrong), None, 1, None, 1, None, 1, None, 1, None) == 1  # wrong output size
    assert lib.b200_mul(None, 1, None, 1, None, 1, 1, 2, 2, 2, 0, None) == 2
    assert lib.b200_add(None, 1, None, 1, None, 1, 4, 1.0, 1.0, 0, None) == 2
    assert lib.b200_maxpool(None, None, None, 1, 1, 4, 4, 2, 2, None) == 2


def test_python_mirror_raises_reference_style_errors():
    torch = pytest.importorskip("torch")
    from cuda_cnn_gan_vae_b200 import ops
    with pytest.raises(ops.B200Error):
        ops.CTensorMath.Mul(torch.zeros(1, 1, 2, 2), torch.zeros(1, 1, 2, 2), torch.zeros(1, 1, 2, 2))  # CPU tensors


def test_wgrad_batch_rejects_an_inconsistent_output_size(lib):
    from cuda_cnn_gan_vae_b200.lib import ConvGeom
    wrong = ConvGeom(3, 8, 8, 4, 3, 3, 1, 1, 1, 1, 9, 8)
    assert lib.b200_conv_wgrad_batch(C.byref(wrong), None, None, 0, None, None, 2, None) == 1          # B200_E_SHAPE before anything else
    assert lib.b200_conv_wgrad_batch_static(C.byref(wrong), C.c_void_p(8), None, 0, C.c_void_p(8), C.c_void_p(8), 2, None) == 1
    assert b"output size" in lib.b200_last_error()
