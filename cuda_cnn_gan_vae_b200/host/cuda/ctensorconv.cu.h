#ifndef B200_C_TENSOR_CONV_CU_H
#define B200_C_TENSOR_CONV_CU_H

// CTensorConv<T>: the convolution class of da-nie/CUDA-CNN-GAN-VAE (cuda/ctensorconv.cu.h:63-66)
// over the C ABI of libb200conv.so: same four static methods, same argument order, the reference's
// own shape checks (cuda/ctensorconv.cu.h:281-295, 689-707, 1173-1185), errors thrown as C strings.

#include "ctensor.cu.h"
#include "ctensormath.cu.h"

template<class type_t>
class CTensorConv
{
 public:
  static void ForwardConvolution(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Image,const CTensor<type_t> &cTensor_Kernel,int32_t kernel_x,int32_t kernel_y,int32_t kernel_z,uint32_t kernel_amount,const CTensor<type_t> &cTensor_Bias,int32_t stride_x,int32_t stride_y,int32_t padding_x,int32_t padding_y);
  static void BackwardConvolution(CTensor<type_t> &cTensor_OutputDelta,const CTensor<type_t> &cTensor_Delta,const CTensor<type_t> &cTensor_Kernel,int32_t kernel_x,int32_t kernel_y,int32_t kernel_z,uint32_t kernel_amount,const CTensor<type_t> &cTensor_Bias,int32_t stride_x,int32_t stride_y,int32_t padding_x,int32_t padding_y);
  static void CreateDeltaWeightAndBias(CTensor<type_t> &cTensor_dKernel,int32_t dkernel_x,int32_t dkernel_y,int32_t dkernel_z,uint32_t dkernel_amount,CTensor<type_t> &cTensor_dBias,const CTensor<type_t> &cTensor_Image,CTensor<type_t> &cTensor_Delta,int32_t stride_x,int32_t stride_y,int32_t padding_x,int32_t padding_y);
  static void CreateBackDeltaWeightAndBias(CTensor<type_t> &cTensor_dKernel,int32_t dkernel_x,int32_t dkernel_y,int32_t dkernel_z,uint32_t dkernel_amount,CTensor<type_t> &cTensor_dBias,CTensor<type_t> &cTensor_Image,const CTensor<type_t> &cTensor_Delta,int32_t stride_x,int32_t stride_y,int32_t padding_x,int32_t padding_y);
 private:
  static void* Stream(void) {return(static_cast<void*>(B200TensorStream()));}
  static b200_conv_geom Geometry(int32_t in_z,uint32_t in_y,uint32_t in_x,uint32_t amount,int32_t kernel_x,int32_t kernel_y,int32_t stride_x,int32_t stride_y,int32_t padding_x,int32_t padding_y,uint32_t out_y,uint32_t out_x)
  {
   b200_conv_geom g;
   g.in_z=in_z;g.in_y=static_cast<int>(in_y);g.in_x=static_cast<int>(in_x);
   g.kernel_amount=static_cast<int>(amount);g.kernel_y=kernel_y;g.kernel_x=kernel_x;
   g.stride_y=stride_y;g.stride_x=stride_x;g.padding_y=padding_y;g.padding_x=padding_x;
   g.out_y=static_cast<int>(out_y);g.out_x=static_cast<int>(out_x);
   return(g);
  }
};

template<class type_t>
void CTensorConv<type_t>::ForwardConvolution(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Image,const CTensor<type_t> &cTensor_Kernel,int32_t kernel_x,int32_t kernel_y,int32_t kernel_z,uint32_t kernel_amount,const CTensor<type_t> &cTensor_Bias,int32_t stride_x,int32_t stride_y,int32_t padding_x,int32_t padding_y)
{
 if (kernel_amount==0) throw("ForwardConvolution needs at least one kernel");
 if (kernel_amount!=cTensor_Bias.GetSizeZ()) throw("ForwardConvolution: the number of kernels and of biases must match");
 int32_t output_x=(static_cast<int32_t>(cTensor_Image.Size_X)-kernel_x+2*padding_x)/stride_x+1;
 int32_t output_y=(static_cast<int32_t>(cTensor_Image.Size_Y)-kernel_y+2*padding_y)/stride_y+1;
 if (static_cast<int32_t>(cTensor_Output.Size_X)!=output_x || static_cast<int32_t>(cTensor_Output.Size_Y)!=output_y || cTensor_Output.Size_Z!=kernel_amount) throw("ForwardConvolution: wrong size of the output tensor");
 if (static_cast<int32_t>(cTensor_Image.Size_Z)!=kernel_z) throw("ForwardConvolution: the depth of the filters and of the image must match");
 if (cTensor_Kernel.Size_Y!=kernel_amount || static_cast<int32_t>(cTensor_Kernel.Size_X)!=kernel_x*kernel_y*kernel_z) throw("ForwardConvolution: wrong size of the kernel tensor");
 b200_conv_geom g=Geometry(kernel_z,cTensor_Image.Size_Y,cTensor_Image.Size_X,kernel_amount,kernel_x,kernel_y,stride_x,stride_y,padding_x,padding_y,cTensor_Output.Size_Y,cTensor_Output.Size_X);
 const float *image=B200FloatPtr(cTensor_Image.DeviceRead());
 const float *kernel=B200FloatPtr(cTensor_Kernel.DeviceRead());
 const float *bias=B200FloatPtr(cTensor_Bias.DeviceRead());
 B200Check(b200_conv_forward(&g,B200FloatPtr(cTensor_Output.DeviceWrite()),cTensor_Output.Size_W,image,cTensor_Image.Size_W,kernel,cTensor_Kernel.Size_W,bias,cTensor_Bias.Size_W,Stream()));
 cTensor_Output.SetDeviceOnChange();
}

// The bias argument is ignored, as in the reference's CUDA backend (cuda/ctensorconv.cu.h:683-725);
// every caller passes zeros.
template<class type_t>
void CTensorConv<type_t>::BackwardConvolution(CTensor<type_t> &cTensor_OutputDelta,const CTensor<type_t> &cTensor_Delta,const CTensor<type_t> &cTensor_Kernel,int32_t kernel_x,int32_t kernel_y,int32_t kernel_z,uint32_t kernel_amount,const CTensor<type_t> &cTensor_Bias,int32_t stride_x,int32_t stride_y,int32_t padding_x,int32_t padding_y)
{
 if (kernel_amount==0) throw("BackwardConvolution needs at least one kernel");
 if (kernel_amount!=cTensor_Bias.GetSizeZ()) throw("BackwardConvolution: the number of kernels and of biases must match");
 if (static_cast<int32_t>(cTensor_OutputDelta.Size_Z)!=kernel_z) throw("BackwardConvolution: wrong size of the output tensor");
 if (cTensor_Delta.Size_Z!=kernel_amount) throw("BackwardConvolution: the number of filters and the depth of the delta tensor must match");
 if (cTensor_Kernel.Size_Y!=kernel_amount || static_cast<int32_t>(cTensor_Kernel.Size_X)!=kernel_x*kernel_y*kernel_z) throw("BackwardConvolution: wrong size of the kernel tensor");
 b200_conv_geom g=Geometry(kernel_z,cTensor_OutputDelta.Size_Y,cTensor_OutputDelta.Size_X,kernel_amount,kernel_x,kernel_y,stride_x,stride_y,padding_x,padding_y,cTensor_Delta.Size_Y,cTensor_Delta.Size_X);
 const float *delta=B200FloatPtr(cTensor_Delta.DeviceRead());
 const float *kernel=B200FloatPtr(cTensor_Kernel.DeviceRead());
 B200Check(b200_conv_backward(&g,B200FloatPtr(cTensor_OutputDelta.DeviceWrite()),cTensor_OutputDelta.Size_W,delta,cTensor_Delta.Size_W,kernel,cTensor_Kernel.Size_W,NULL,0,Stream()));
 cTensor_OutputDelta.SetDeviceOnChange();
}

template<class type_t>
void CTensorConv<type_t>::CreateDeltaWeightAndBias(CTensor<type_t> &cTensor_dKernel,int32_t dkernel_x,int32_t dkernel_y,int32_t dkernel_z,uint32_t dkernel_amount,CTensor<type_t> &cTensor_dBias,const CTensor<type_t> &cTensor_Image,CTensor<type_t> &cTensor_Delta,int32_t stride_x,int32_t stride_y,int32_t padding_x,int32_t padding_y)
{
 if (dkernel_amount==0) throw("CreateDeltaWeightAndBias needs a non-empty kernel correction tensor");
 if (cTensor_dBias.GetSizeZ()!=dkernel_amount) throw("CreateDeltaWeightAndBias: the number of kernel and of bias corrections must match");
 if (dkernel_z!=static_cast<int32_t>(cTensor_Image.Size_Z)) throw("CreateDeltaWeightAndBias: wrong depth of the kernel correction tensor");
 if (cTensor_Delta.Size_Z!=dkernel_amount) throw("CreateDeltaWeightAndBias: the depth of the delta tensor must match the number of kernels");
 if (cTensor_dKernel.Size_Y!=dkernel_amount || static_cast<int32_t>(cTensor_dKernel.Size_X)!=dkernel_x*dkernel_y*dkernel_z) throw("CreateDeltaWeightAndBias: wrong size of the kernel correction tensor");
 b200_conv_geom g=Geometry(dkernel_z,cTensor_Image.Size_Y,cTensor_Image.Size_X,dkernel_amount,dkernel_x,dkernel_y,stride_x,stride_y,padding_x,padding_y,cTensor_Delta.Size_Y,cTensor_Delta.Size_X);
 const float *image=B200FloatPtr(cTensor_Image.DeviceRead());
 const float *delta=B200FloatPtr(cTensor_Delta.DeviceRead());
 float *dkernel=B200FloatPtr(cTensor_dKernel.DeviceRead());     // accumulated into: the current contents count
 float *dbias=B200FloatPtr(cTensor_dBias.DeviceRead());
 B200Check(b200_conv_wgrad(&g,dkernel,cTensor_dKernel.Size_W,dbias,cTensor_dBias.Size_W,image,cTensor_Image.Size_W,delta,cTensor_Delta.Size_W,Stream()));
 cTensor_dKernel.SetDeviceOnChange();
 cTensor_dBias.SetDeviceOnChange();
}

template<class type_t>
void CTensorConv<type_t>::CreateBackDeltaWeightAndBias(CTensor<type_t> &cTensor_dKernel,int32_t dkernel_x,int32_t dkernel_y,int32_t dkernel_z,uint32_t dkernel_amount,CTensor<type_t> &cTensor_dBias,CTensor<type_t> &cTensor_Image,const CTensor<type_t> &cTensor_Delta,int32_t stride_x,int32_t stride_y,int32_t padding_x,int32_t padding_y)
{
 // the same gradient with image and delta exchanged, then the bias gradient is cleared (cuda/ctensorconv.cu.h:1218-1222)
 CTensor<type_t> &cTensor_DeltaAsImage=const_cast<CTensor<type_t>&>(cTensor_Delta);
 CTensorConv<type_t>::CreateDeltaWeightAndBias(cTensor_dKernel,dkernel_x,dkernel_y,dkernel_z,dkernel_amount,cTensor_dBias,cTensor_DeltaAsImage,cTensor_Image,stride_x,stride_y,padding_x,padding_y);
 CTensorMath<type_t>::Fill(cTensor_dBias,0);
}

#endif
