#ifndef B200_C_TENSOR_APPLY_FUNC_CU_H
#define B200_C_TENSOR_APPLY_FUNC_CU_H

// CTensorApplyFunc<T>: activation functions and their derivatives (cuda/ctensorapplyfunc.cu.h:78-90)
// over the C ABI of libb200conv.so.  LeakyReLU uses the reference's slope 0.1.  SoftMax is outside the
// convolution hot path and is not provided.

#include "ctensor.cu.h"
#include "ctensormath.cu.h"

template<class type_t>
class CTensorApplyFunc
{
 public:
  static void ApplySigmoid(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input) {Apply(cTensor_Output,cTensor_Input,B200_ACT_SIGMOID,0);}
  static void ApplyReLU(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input) {Apply(cTensor_Output,cTensor_Input,B200_ACT_RELU,0);}
  static void ApplyGeLU(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input) {Apply(cTensor_Output,cTensor_Input,B200_ACT_GELU,0);}
  static void ApplyLeakyReLU(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input) {Apply(cTensor_Output,cTensor_Input,B200_ACT_LEAKY_RELU,0);}
  static void ApplyLinear(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input) {Apply(cTensor_Output,cTensor_Input,B200_ACT_LINEAR,0);}
  static void ApplyTangence(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input) {Apply(cTensor_Output,cTensor_Input,B200_ACT_TANH,0);}
  static void ApplySoftMax(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input) {(void)cTensor_Output;(void)cTensor_Input;throw("ApplySoftMax is not part of this library");}

  static void ApplyDifferentialSigmoid(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input) {Apply(cTensor_Output,cTensor_Input,B200_ACT_SIGMOID,1);}
  static void ApplyDifferentialReLU(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input) {Apply(cTensor_Output,cTensor_Input,B200_ACT_RELU,1);}
  static void ApplyDifferentialGeLU(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input) {Apply(cTensor_Output,cTensor_Input,B200_ACT_GELU,1);}
  static void ApplyDifferentialLeakyReLU(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input) {Apply(cTensor_Output,cTensor_Input,B200_ACT_LEAKY_RELU,1);}
  static void ApplyDifferentialLinear(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input) {Apply(cTensor_Output,cTensor_Input,B200_ACT_LINEAR,1);}
  static void ApplyDifferentialTangence(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input) {Apply(cTensor_Output,cTensor_Input,B200_ACT_TANH,1);}
  static void ApplyDifferentialSoftMax(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input) {(void)cTensor_Output;(void)cTensor_Input;throw("ApplyDifferentialSoftMax is not part of this library");}
 private:
  static void Apply(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,int func,int derivative)
  {
   if (cTensor_Input.Size_X!=cTensor_Output.Size_X || cTensor_Input.Size_Y!=cTensor_Output.Size_Y || cTensor_Input.Size_Z!=cTensor_Output.Size_Z || cTensor_Input.Size_W!=cTensor_Output.Size_W)
   {
    throw "CTensorApplyFunc: tensor sizes do not match!";
   }
   const float *in=B200FloatPtr(cTensor_Input.DeviceRead());
   B200Check(b200_activation(B200FloatPtr(cTensor_Output.DeviceWrite()),in,cTensor_Output.Count(),func,derivative,0.1,static_cast<void*>(B200TensorStream())));
   cTensor_Output.SetDeviceOnChange();
  }
};

#endif
