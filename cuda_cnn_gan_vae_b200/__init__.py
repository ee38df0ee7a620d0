"""B200-native convolution hot path behind the tensor-math interface of da-nie/CUDA-CNN-GAN-VAE.

The product is the C-ABI library libb200conv.so (sources in csrc/, declarations in
include/b200conv.h).  This package loads it and mirrors the reference's static tensor-math classes
(CTensorConv, CTensorMath, CTensorApplyFunc) on torch CUDA tensors; torch only provides device
memory and streams.  There is no CPU fallback: importing `ops` without the built library raises.
"""
from . import build as _build  # noqa: F401

__all__ = ["lib", "ops"]
