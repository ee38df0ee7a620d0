#ifndef C_NET_LAYER_CONVOLUTION_H
#define C_NET_LAYER_CONVOLUTION_H

// CNetLayerConvolution of da-nie/CUDA-CNN-GAN-VAE (netlayer/cnetlayerconvolution.cu.h: interface :73-133, Forward :310,
// TrainingBackward :484, checkpoint :351-413) on the layer-level entry points of libb200conv.so.  Same constructor, same
// INetLayer interface, same checkpoint bytes; what differs is inside: the reference's TrainingBackward makes a zeroed copy of
// the bias, fills a [batch, kernels, depth*ky*kx] tensor, runs one weight-gradient product per sample and reduces it with two
// AddSumW passes -- here it is one call that reuses the packed layer input of Forward and forms the batch-summed gradient on
// the tensor cores.

#include "b200convlayer.cu.h"

template<class type_t>
class CNetLayerConvolution:public CB200ConvLayerCore<type_t>
{
  typedef CB200ConvLayerCore<type_t> Core;
 public:
  CNetLayerConvolution(uint32_t kernel_amount,uint32_t kernel_size,int32_t stride_x,int32_t stride_y,int32_t padding_x,int32_t padding_y,INetLayer<type_t> *prev_layer_ptr=NULL,uint32_t batch_size=1):Core("Convolution",false)
  {
   Create(kernel_amount,kernel_size,stride_x,stride_y,padding_x,padding_y,prev_layer_ptr,batch_size);
  }
  void Create(uint32_t kernel_amount,uint32_t kernel_size,int32_t stride_x,int32_t stride_y,int32_t padding_x,int32_t padding_y,INetLayer<type_t> *prev_layer_ptr=NULL,uint32_t batch_size=1)
  {
   Core::Attach(prev_layer_ptr,batch_size,false,"a convolution layer cannot be the input layer: put a CNetLayerConvolutionInput in front of it");
   Core::Configure(kernel_amount,prev_layer_ptr->GetOutputTensor().GetSizeZ(),kernel_size,stride_x,stride_y,padding_x,padding_y);
  }
  /// uniform weights in +-sqrt(6/fan_in), biases 0.1 (the reference's initialisation, :232-265)
  void Reset(void)
  {
   CTensor<type_t> &kernel=Core::Slot[Core::KERNEL].Weight;
   const uint32_t fan_in=Core::Kernel_X*Core::Kernel_Y*Core::Kernel_Z;
   const type_t limit=static_cast<type_t>(sqrt(6.0/static_cast<double>(fan_in)));
   for(uint32_t k=0;k<Core::Kernel_Amount;k++)
    for(uint32_t m=0;m<fan_in;m++) kernel.SetElement(0,0,k,m,static_cast<type_t>(CRandom<type_t>::GetRandValue(2.0)-1.0)*limit);
   for(uint32_t k=0;k<Core::Kernel_Amount;k++) Core::Slot[Core::BIAS].Weight.SetElement(0,k,0,0,static_cast<type_t>(0.1));
  }
};

#endif
