#ifndef C_NET_LAYER_BACK_CONVOLUTION_H
#define C_NET_LAYER_BACK_CONVOLUTION_H

// CNetLayerBackConvolution of da-nie/CUDA-CNN-GAN-VAE (netlayer/cnetlayerbackconvolution.cu.h: interface :73-133, Forward
// :303, TrainingBackward :475): the transposed-convolution layer.  Its kernel tensor is that of the convolution it
// transposes, [1,1,input depth,kernel_depth*ky*kx]; Forward is that convolution's backward-data pass, the error of the
// previous layer its forward pass, the weight gradient the convolution's with image and error exchanged, the bias gradient
// stays zero.  The reference's class does not work at its head revision (it creates the kernel tensor with three sizes and
// its per-sample gradient tensors never exist); this one keeps the constructor, the interface and the checkpoint layout.

#include "b200convlayer.cu.h"

template<class type_t>
class CNetLayerBackConvolution:public CB200ConvLayerCore<type_t>
{
  typedef CB200ConvLayerCore<type_t> Core;
 public:
  CNetLayerBackConvolution(uint32_t kernel_size,uint32_t kernel_depth,int32_t stride_x,int32_t stride_y,int32_t padding_x,int32_t padding_y,INetLayer<type_t> *prev_layer_ptr=NULL,uint32_t batch_size=1):Core("BackConvolution",true)
  {
   Create(kernel_size,kernel_depth,stride_x,stride_y,padding_x,padding_y,prev_layer_ptr,batch_size);
  }
  void Create(uint32_t kernel_size,uint32_t kernel_depth,int32_t stride_x,int32_t stride_y,int32_t padding_x,int32_t padding_y,INetLayer<type_t> *prev_layer_ptr=NULL,uint32_t batch_size=1)
  {
   Core::Attach(prev_layer_ptr,batch_size,false,"a transposed convolution layer cannot be the input layer: put a CNetLayerConvolutionInput in front of it");
   Core::Configure(prev_layer_ptr->GetOutputTensor().GetSizeZ(),kernel_depth,kernel_size,stride_x,stride_y,padding_x,padding_y);
  }
  /// normal weights scaled by sqrt(2/(depth*ky*kx)), zero biases (the reference's initialisation, :232-262)
  void Reset(void)
  {
   CTensor<type_t> &kernel=Core::Slot[Core::KERNEL].Weight;
   const uint32_t size=Core::Kernel_X*Core::Kernel_Y*Core::Kernel_Z;
   const double limit=sqrt(2.0/static_cast<double>(size));
   CTensor<type_t> row(1,1,1,size);
   for(uint32_t k=0;k<Core::Kernel_Amount;k++)
   {
    CRandom<type_t>::SetRandomNormal(row,-limit,limit);
    for(uint32_t m=0;m<size;m++) kernel.SetElement(0,0,k,m,row.GetElement(0,0,0,m));
   }
   CTensorMath<type_t>::Fill(Core::Slot[Core::BIAS].Weight,0);
  }
};

#endif
