#ifndef B200_CONV_LAYER_CORE_CU_H
#define B200_CONV_LAYER_CORE_CU_H

// Shared body of CNetLayerConvolution and CNetLayerBackConvolution: the geometry of the underlying convolution, the layer
// context of libb200conv.so (b200_conv_layer_*: packed operands kept between Forward and TrainingBackward, batch-summed
// weight gradient on the tensor cores) and the reference's checkpoint layout of the two layers, which is the same
// (netlayer/cnetlayerconvolution.cu.h:351-413, netlayer/cnetlayerbackconvolution.cu.h:344-392): eight int32 geometry words,
// then the kernel tensor [1,1,amount,depth*ky*kx] and the bias tensor [1,amount,1,1].

#include "b200netlayer.cu.h"

template<class type_t>
class CB200ConvLayerCore:public CB200NetLayer<type_t>
{
 protected:
  typedef CB200NetLayer<type_t> Base;
  typedef CB200LayerPort<type_t> Port;
  using Base::Slot;
  using Base::PrevLayerPtr;
  using Base::BatchSize;
  using Base::cTensor_H;
  using Base::cTensor_Delta;
  using Base::cTensor_PrevLayerError;
  enum {KERNEL=0,BIAS=1};
  bool Transposed;///<the layer applies the transposed convolution (its forward pass is the convolution's backward-data pass)
  uint32_t Kernel_X,Kernel_Y,Kernel_Z,Kernel_Amount;
  uint32_t Padding_X,Padding_Y,Stride_X,Stride_Y;
  uint32_t InputSize_X,InputSize_Y,InputSize_Z;
  b200_conv_geom Geometry;
  b200_conv_layer *Context;
 protected:
  CB200ConvLayerCore(const char *name,bool transposed):Base(name),Transposed(transposed),Context(NULL) {}
  ~CB200ConvLayerCore() {Release();}
  void Release(void)
  {
   if (Context!=NULL) b200_conv_layer_destroy(Context);
   Context=NULL;
  }
  /// geometry of the underlying convolution from the layer's input size; (re)creates the context and the tensors
  void Configure(uint32_t amount,uint32_t depth,uint32_t kernel_size,int32_t stride_x,int32_t stride_y,int32_t padding_x,int32_t padding_y)
  {
   CTensor<type_t> &input=PrevLayerPtr->GetOutputTensor();
   InputSize_X=input.GetSizeX();
   InputSize_Y=input.GetSizeY();
   InputSize_Z=input.GetSizeZ();
   Kernel_X=kernel_size;Kernel_Y=kernel_size;Kernel_Z=depth;Kernel_Amount=amount;
   Stride_X=stride_x;Stride_Y=stride_y;Padding_X=padding_x;Padding_Y=padding_y;
   if (Kernel_Amount==0) throw("a convolution layer needs at least one kernel");
   if (Stride_X==0 || Stride_Y==0) throw("a convolution layer needs a positive stride");
   int32_t output_x,output_y,output_z;
   if (Transposed==false)
   {
    output_x=(static_cast<int32_t>(InputSize_X)-static_cast<int32_t>(Kernel_X)+2*static_cast<int32_t>(Padding_X))/static_cast<int32_t>(Stride_X)+1;
    output_y=(static_cast<int32_t>(InputSize_Y)-static_cast<int32_t>(Kernel_Y)+2*static_cast<int32_t>(Padding_Y))/static_cast<int32_t>(Stride_Y)+1;
    output_z=Kernel_Amount;
   }
   else
   {
    output_x=Stride_X*(InputSize_X-1)+Kernel_X-2*Padding_X;
    output_y=Stride_Y*(InputSize_Y-1)+Kernel_Y-2*Padding_Y;
    output_z=Kernel_Z;
   }
   if (output_x<=0 || output_y<=0) throw("the convolution layer's output would be empty");
   // the convolution whose forward pass maps the large tensor to the small one: image = layer input (convolution layer) or
   // layer output (transposed layer)
   Geometry.in_z=Kernel_Z;
   Geometry.in_y=Transposed?output_y:InputSize_Y;
   Geometry.in_x=Transposed?output_x:InputSize_X;
   Geometry.kernel_amount=Kernel_Amount;
   Geometry.kernel_y=Kernel_Y;Geometry.kernel_x=Kernel_X;
   Geometry.stride_y=Stride_Y;Geometry.stride_x=Stride_X;
   Geometry.padding_y=Padding_Y;Geometry.padding_x=Padding_X;
   Geometry.out_y=Transposed?InputSize_Y:output_y;
   Geometry.out_x=Transposed?InputSize_X:output_x;
   Slot.resize(2);
   Slot[KERNEL].Weight=CTensor<type_t>(1,1,Kernel_Amount,Kernel_Z*Kernel_X*Kernel_Y);
   Slot[BIAS].Weight=CTensor<type_t>(1,Kernel_Amount,1,1);
   cTensor_H=CTensor<type_t>(BatchSize,output_z,output_y,output_x);
   Release();
   B200Check(b200_conv_layer_create(&Context,&Geometry,BatchSize,Transposed?1:0));
   PrevLayerPtr->SetNextLayerPtr(this);
  }
  void CheckInput(void)
  {
   if (Base::InputCount()!=static_cast<size_t>(InputSize_X)*InputSize_Y*InputSize_Z) throw("the previous layer's output no longer has the size the convolution layer was created for");
  }
 public:
  void Forward(void)
  {
   CheckInput();
   const float *input=Port::Read(PrevLayerPtr->GetOutputTensor());
   const float *kernel=Port::Read(Base::Active(KERNEL));
   const float *bias=Port::Read(Base::Active(BIAS));
   B200Check(b200_conv_layer_forward(Context,Port::Write(cTensor_H),input,kernel,bias,Port::Stream()));
  }
  /// error of the previous layer; with create_delta_weight the kernel and bias gradients are added to (one batch-summed
  /// product, no per-sample tensor).  The bias gradient of the transposed layer stays zero, as in the reference
  /// (cuda/ctensorconv.cu.h:1221).
  void TrainingBackward(bool create_delta_weight=true)
  {
   CheckInput();
   const float *delta=Port::Read(cTensor_Delta);
   const float *input=Port::Read(PrevLayerPtr->GetOutputTensor());
   const float *kernel=Port::Read(Slot[KERNEL].Weight);
   float *dkernel=create_delta_weight?Port::Update(Slot[KERNEL].Gradient):NULL;
   float *dbias=(create_delta_weight && Transposed==false)?Port::Update(Slot[BIAS].Gradient):NULL;
   B200Check(b200_conv_layer_backward(Context,Port::Write(cTensor_PrevLayerError),dkernel,dbias,1,delta,input,kernel,Port::Stream()));
   PrevLayerPtr->SetOutputError(cTensor_PrevLayerError);
  }
  bool Save(IDataStream *iDataStream_Ptr)
  {
   const uint32_t word[8]={Kernel_Amount,Kernel_X,Kernel_Y,Kernel_Z,Stride_X,Stride_Y,Padding_X,Padding_Y};
   for(size_t n=0;n<8;n++) iDataStream_Ptr->SaveInt32(word[n]);
   Slot[KERNEL].Weight.Save(iDataStream_Ptr);
   Slot[BIAS].Weight.Save(iDataStream_Ptr);
   return(true);
  }
  bool Load(IDataStream *iDataStream_Ptr,bool check_size=false)
  {
   uint32_t word[8];
   word[0]=iDataStream_Ptr->LoadUInt32();
   for(size_t n=1;n<8;n++) word[n]=static_cast<uint32_t>(iDataStream_Ptr->LoadInt32());
   const uint32_t have[8]={Kernel_Amount,Kernel_X,Kernel_Y,Kernel_Z,Stride_X,Stride_Y,Padding_X,Padding_Y};
   bool same=true;
   for(size_t n=0;n<8;n++) if (word[n]!=have[n]) same=false;
   if (check_size==true && same==false) throw("loading a convolution layer: the stored geometry differs from the layer's");
   if (same==false)
   {
    if (Transposed==false && word[3]!=InputSize_Z) throw("loading a convolution layer: the stored kernel depth does not fit the layer input");
    if (Transposed==true && word[0]!=InputSize_Z) throw("loading a transposed convolution layer: the stored number of kernels does not fit the layer input");
    Configure(word[0],word[3],word[1],word[4],word[5],word[6],word[7]);
   }
   Slot[KERNEL].Weight.Load(iDataStream_Ptr,check_size);
   Slot[BIAS].Weight.Load(iDataStream_Ptr,check_size);
   return(true);
  }
};

#endif
