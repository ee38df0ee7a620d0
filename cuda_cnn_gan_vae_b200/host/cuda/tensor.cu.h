#ifndef B200_TENSOR_CU_H
#define B200_TENSOR_CU_H

// Tensors and the operations on them: stands in for cuda/tensor.cu.h of da-nie/CUDA-CNN-GAN-VAE.

#include "ctensor.cu.h"
#include "ctensormath.cu.h"
#include "ctensorconv.cu.h"
#include "ctensorapplyfunc.cu.h"

#endif
