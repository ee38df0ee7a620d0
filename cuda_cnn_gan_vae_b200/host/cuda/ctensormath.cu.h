#ifndef B200_C_TENSOR_MATH_CU_H
#define B200_C_TENSOR_MATH_CU_H

// CTensorMath<T>: the static tensor-math class of da-nie/CUDA-CNN-GAN-VAE
// (cuda/ctensormath.cu.h:92-135) over the C ABI of libb200conv.so.  Each method keeps the reference's
// name, signature and shape checks (a mismatch throws a C string), makes its operands
// device-resident, calls one ABI entry point on B200TensorStream() and marks the output as changed on
// the device.  Compute entry points exist for float; other element types are storage only.
// Not provided (outside the convolution hot path): SetTimeStep, CreateDropOutMatrix, SetNormalNoise,
// GetNoiseImageAndNoise.

#include "ctensor.cu.h"

template<class type_t>
class CTensorMath
{
 public:
  struct SPos
  {
   uint32_t X;
   uint32_t Y;
  };
 public:
  static void Fill(CTensor<type_t> &cTensor_Output,type_t value=0);
  static void Inv(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input);
  static void Div(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right,type_t left_scale=1,type_t right_scale=1);
  static void Add(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right,type_t left_scale=1,type_t right_scale=1);
  static void AddSumW(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right,type_t left_scale=1,type_t right_scale=1);
  static void AddValue(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,type_t tensor_scale,type_t value);
  static void Sub(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right,type_t left_scale=1,type_t right_scale=1);
  static void SubValue(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,type_t tensor_scale,type_t value);
  static void Set(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,type_t scale=1,type_t add_value=0);
  static void Pow2(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,type_t scale=1);
  static void SQRT(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,type_t scale,type_t add_sqrt_value);
  static void AddBias(CTensor<type_t> &cTensor_Working,const CTensor<type_t> &cTensor_Bias);
  static void SummXY(CTensor<type_t> &cTensor_Output,CTensor<type_t> &cTensor_Input);
  static void Mul(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right,bool tensor_core=false);
  static void TransponseMul(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right,bool tensor_core=false);
  static void Mul(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const type_t &value_right);
  static void Mul(CTensor<type_t> &cTensor_Output,const type_t &value_left,const CTensor<type_t> &cTensor_Right);
  static void Transponse(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input);
  static void ConcatecationZ(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_InputA,const CTensor<type_t> &cTensor_InputB);
  static void SplitZ(CTensor<type_t> &cTensor_OutputA,CTensor<type_t> &cTensor_OutputB,const CTensor<type_t> &cTensor_Input);
  static void TensorItemProduction(CTensor<type_t> &cTensor_Output,CTensor<type_t> &cTensor_Left,CTensor<type_t> &cTensor_Right);
  static CTensor<type_t> Transpose(const CTensor<type_t> &cTensor_Input);
  static void UpSampling(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,uint32_t upsampling_x,uint32_t upsampling_y);
  static void DownSampling(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,uint32_t downsampling_x,uint32_t downsampling_y);
  static void MaxPooling(CTensor<type_t> &cTensor_Output,const CTensor<typename CTensorMath<type_t>::SPos> &cTensor_Position,const CTensor<type_t> &cTensor_Input,uint32_t pooling_x,uint32_t pooling_y);
  static void MaxPoolingBackward(CTensor<type_t> &cTensor_Output,const CTensor<typename CTensorMath<type_t>::SPos> &cTensor_Position,const CTensor<type_t> &cTensor_Input,uint32_t pooling_x,uint32_t pooling_y);
  static void Clip(CTensor<type_t> &cTensor,type_t min_value,type_t max_value);
  static void Signum(CTensor<type_t> &cTensor);
  static void Adam(CTensor<type_t> &cTensor_Weight,CTensor<type_t> &cTensor_dWeight,CTensor<type_t> &cTensor_M,CTensor<type_t> &cTensor_V,uint32_t batch_size,double speed,double beta1,double beta2,double epsilon,double iteration);
  static void SetTimeStep(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,const CTensor<uint32_t> &cTensor_TimeStep);
  static void CreateDropOutMatrix(CTensor<type_t> &cTensor_Output,type_t drop_out);
  static void SetNormalNoise(CTensor<type_t> &cTensor_Output);
  static void GetNoiseImageAndNoise(CTensor<type_t> &cTensor_NoisyImage,CTensor<type_t> &cTensor_Noise,const CTensor<type_t> &cTensor_Image,const CTensor<type_t> &cTensor_SqrtAlphaBar,const CTensor<type_t> &cTensor_SqrtOneMinusAlphaBar);
 private:
  // seed of the next random tensor: rand() as in the reference (cuda/ctensormath.cu.h:3205), widened by a call counter
  static unsigned long long NextSeed(void) {static unsigned long long counter=0;counter++;return((static_cast<unsigned long long>(rand())<<32)^counter);}
  static bool SameZYX(const CTensor<type_t> &a,const CTensor<type_t> &b) {return(a.Size_X==b.Size_X && a.Size_Y==b.Size_Y && a.Size_Z==b.Size_Z);}
  static size_t PlaneCount(const CTensor<type_t> &a) {return(static_cast<size_t>(a.Size_X)*a.Size_Y*a.Size_Z);}
  static void* Stream(void) {return(static_cast<void*>(B200TensorStream()));}
  static void Unary(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,int op,type_t a,type_t b,const char *error);
  static void Binary(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right,int op,type_t left_scale,type_t right_scale,const char *error);
};

// device pointer helpers: the compute entry points take float; any other instantiation is refused
template<class type_t> inline float* B200FloatPtr(type_t *ptr) {(void)ptr;throw("CTensorMath: compute entry points exist for float tensors only.");return(NULL);}
template<> inline float* B200FloatPtr<float>(float *ptr) {return(ptr);}

//----------------------------------------------------------------------------------------------------
// element-wise helpers
//----------------------------------------------------------------------------------------------------
template<class type_t>
void CTensorMath<type_t>::Unary(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,int op,type_t a,type_t b,const char *error)
{
 if (SameZYX(cTensor_Output,cTensor_Input)==false) throw error;
 const float *in=B200FloatPtr(cTensor_Input.DeviceRead());
 B200Check(b200_unary(B200FloatPtr(cTensor_Output.DeviceWrite()),cTensor_Output.Size_W,in,cTensor_Input.Size_W,PlaneCount(cTensor_Output),op,static_cast<float>(a),static_cast<float>(b),Stream()));
 cTensor_Output.SetDeviceOnChange();
}

// op: 0 add, 1 subtract, 2 item product, 3 divide, 4 sum over W
template<class type_t>
void CTensorMath<type_t>::Binary(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right,int op,type_t left_scale,type_t right_scale,const char *error)
{
 if (SameZYX(cTensor_Left,cTensor_Right)==false || SameZYX(cTensor_Output,cTensor_Right)==false) throw error;
 const float *l=B200FloatPtr(cTensor_Left.DeviceRead());
 const float *r=B200FloatPtr(cTensor_Right.DeviceRead());
 float *o=B200FloatPtr(cTensor_Output.DeviceWrite());
 const size_t n=PlaneCount(cTensor_Output);
 const float ls=static_cast<float>(left_scale),rs=static_cast<float>(right_scale);
 int status;
 if (op==0 || op==1) status=b200_add(o,cTensor_Output.Size_W,l,cTensor_Left.Size_W,r,cTensor_Right.Size_W,n,ls,rs,op,Stream());
 else if (op==2) status=b200_item_product(o,cTensor_Output.Size_W,l,cTensor_Left.Size_W,r,cTensor_Right.Size_W,n,Stream());
 else if (op==3) status=b200_div(o,cTensor_Output.Size_W,l,cTensor_Left.Size_W,r,cTensor_Right.Size_W,n,ls,rs,Stream());
 else status=b200_add_sum_w(o,cTensor_Output.Size_W,l,cTensor_Left.Size_W,r,cTensor_Right.Size_W,n,ls,rs,Stream());
 B200Check(status);
 cTensor_Output.SetDeviceOnChange();
}

template<class type_t>
void CTensorMath<type_t>::Fill(CTensor<type_t> &cTensor_Output,type_t value)
{
 B200Check(b200_fill(B200FloatPtr(cTensor_Output.DeviceWrite()),cTensor_Output.Count(),static_cast<float>(value),Stream()));
 cTensor_Output.SetDeviceOnChange();
}

template<class type_t>
void CTensorMath<type_t>::Inv(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input)
{
 Unary(cTensor_Output,cTensor_Input,2,0,0,"CTensor::Inv: tensor sizes do not match!");
}
template<class type_t>
void CTensorMath<type_t>::Pow2(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,type_t scale)
{
 Unary(cTensor_Output,cTensor_Input,0,scale,0,"CTensor::Pow2: tensor sizes do not match!");
}
template<class type_t>
void CTensorMath<type_t>::SQRT(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,type_t scale,type_t add_sqrt_value)
{
 Unary(cTensor_Output,cTensor_Input,1,scale,add_sqrt_value,"CTensor::SQRT: tensor sizes do not match!");
}
template<class type_t>
void CTensorMath<type_t>::AddValue(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,type_t tensor_scale,type_t value)
{
 Unary(cTensor_Output,cTensor_Input,4,tensor_scale,value,"CTensor::AddValue: tensor sizes do not match!");
}
template<class type_t>
void CTensorMath<type_t>::SubValue(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,type_t tensor_scale,type_t value)
{
 Unary(cTensor_Output,cTensor_Input,4,tensor_scale,-value,"CTensor::SubValue: tensor sizes do not match!");
}
template<class type_t>
void CTensorMath<type_t>::Set(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,type_t scale,type_t add_value)
{
 Unary(cTensor_Output,cTensor_Input,4,scale,add_value,"CTensor::Set: tensor sizes do not match!");
}
template<class type_t>
void CTensorMath<type_t>::Mul(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const type_t &value_right)
{
 Unary(cTensor_Output,cTensor_Left,3,value_right,0,"CTensor::Mul: tensor sizes do not match!");
}
template<class type_t>
void CTensorMath<type_t>::Mul(CTensor<type_t> &cTensor_Output,const type_t &value_left,const CTensor<type_t> &cTensor_Right)
{
 Unary(cTensor_Output,cTensor_Right,3,value_left,0,"CTensor::Mul: tensor sizes do not match!");
}
template<class type_t>
void CTensorMath<type_t>::Clip(CTensor<type_t> &cTensor,type_t min_value,type_t max_value)
{
 Unary(cTensor,cTensor,5,min_value,max_value,"CTensor::Clip");
}
template<class type_t>
void CTensorMath<type_t>::Signum(CTensor<type_t> &cTensor)
{
 Unary(cTensor,cTensor,6,0,0,"CTensor::Signum");
}

template<class type_t>
void CTensorMath<type_t>::Add(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right,type_t left_scale,type_t right_scale)
{
 Binary(cTensor_Output,cTensor_Left,cTensor_Right,0,left_scale,right_scale,"CTensor::Add: tensor sizes do not match!");
}
template<class type_t>
void CTensorMath<type_t>::Sub(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right,type_t left_scale,type_t right_scale)
{
 Binary(cTensor_Output,cTensor_Left,cTensor_Right,1,left_scale,right_scale,"CTensor::Sub: tensor sizes do not match!");
}
template<class type_t>
void CTensorMath<type_t>::Div(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right,type_t left_scale,type_t right_scale)
{
 Binary(cTensor_Output,cTensor_Left,cTensor_Right,3,left_scale,right_scale,"CTensor::Div: tensor sizes do not match!");
}
template<class type_t>
void CTensorMath<type_t>::AddSumW(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right,type_t left_scale,type_t right_scale)
{
 Binary(cTensor_Output,cTensor_Left,cTensor_Right,4,left_scale,right_scale,"CTensor::AddSumW: tensor sizes do not match!");
}
template<class type_t>
void CTensorMath<type_t>::TensorItemProduction(CTensor<type_t> &cTensor_Output,CTensor<type_t> &cTensor_Left,CTensor<type_t> &cTensor_Right)
{
 Binary(cTensor_Output,cTensor_Left,cTensor_Right,2,1,1,"CTensor::TensorItemProduction: tensor sizes do not match!");
}

template<class type_t>
void CTensorMath<type_t>::AddBias(CTensor<type_t> &cTensor_Working,const CTensor<type_t> &cTensor_Bias)
{
 if (cTensor_Working.Size_Z!=cTensor_Bias.Size_Z) throw "CTensor::AddBias: tensor sizes do not match!";
 const float *bias=B200FloatPtr(cTensor_Bias.DeviceRead());
 B200Check(b200_add_bias(B200FloatPtr(cTensor_Working.DeviceRead()),cTensor_Working.Size_W,cTensor_Working.Size_Z,static_cast<size_t>(cTensor_Working.Size_Y)*cTensor_Working.Size_X,bias,cTensor_Bias.Size_W,Stream()));
 cTensor_Working.SetDeviceOnChange();
}

template<class type_t>
void CTensorMath<type_t>::SummXY(CTensor<type_t> &cTensor_Output,CTensor<type_t> &cTensor_Input)
{
 if (cTensor_Input.Size_Z!=cTensor_Output.Size_Z) throw "CTensor::SummXY: tensor sizes do not match!";
 const float *in=B200FloatPtr(cTensor_Input.DeviceRead());
 B200Check(b200_summ_xy(B200FloatPtr(cTensor_Output.DeviceWrite()),cTensor_Output.Size_W,in,cTensor_Input.Size_W,cTensor_Input.Size_Z,static_cast<size_t>(cTensor_Input.Size_Y)*cTensor_Input.Size_X,Stream()));
 cTensor_Output.SetDeviceOnChange();
}

//----------------------------------------------------------------------------------------------------
// matrix products (cuda/ctensormath.cu.h:2237-2255): per (w,z) plane, operands broadcast over W by modulo.
// tensor_core is accepted for source compatibility; the library picks its own kernel.
//----------------------------------------------------------------------------------------------------
template<class type_t>
void CTensorMath<type_t>::Mul(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right,bool tensor_core)
{
 (void)tensor_core;
 if (cTensor_Left.Size_X!=cTensor_Right.Size_Y || cTensor_Left.Size_Z!=cTensor_Right.Size_Z ||
     cTensor_Output.Size_Y!=cTensor_Left.Size_Y || cTensor_Output.Size_X!=cTensor_Right.Size_X || cTensor_Output.Size_Z!=cTensor_Right.Size_Z)
 {
  throw "CTensor::Mul: tensor sizes do not match!";
 }
 const float *l=B200FloatPtr(cTensor_Left.DeviceRead());
 const float *r=B200FloatPtr(cTensor_Right.DeviceRead());
 B200Check(b200_mul(B200FloatPtr(cTensor_Output.DeviceWrite()),cTensor_Output.Size_W,l,cTensor_Left.Size_W,r,cTensor_Right.Size_W,
                    cTensor_Left.Size_Z,cTensor_Left.Size_Y,cTensor_Left.Size_X,cTensor_Right.Size_X,0,Stream()));
 cTensor_Output.SetDeviceOnChange();
}

template<class type_t>
void CTensorMath<type_t>::TransponseMul(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right,bool tensor_core)
{
 (void)tensor_core;
 if (cTensor_Left.Size_Y!=cTensor_Right.Size_Y || cTensor_Left.Size_Z!=cTensor_Right.Size_Z ||
     cTensor_Output.Size_Y!=cTensor_Left.Size_X || cTensor_Output.Size_X!=cTensor_Right.Size_X || cTensor_Output.Size_Z!=cTensor_Right.Size_Z)
 {
  throw "CTensor::TransponseMul: tensor sizes do not match!";
 }
 const float *l=B200FloatPtr(cTensor_Left.DeviceRead());
 const float *r=B200FloatPtr(cTensor_Right.DeviceRead());
 B200Check(b200_mul(B200FloatPtr(cTensor_Output.DeviceWrite()),cTensor_Output.Size_W,l,cTensor_Left.Size_W,r,cTensor_Right.Size_W,
                    cTensor_Left.Size_Z,cTensor_Left.Size_Y,cTensor_Left.Size_X,cTensor_Right.Size_X,1,Stream()));
 cTensor_Output.SetDeviceOnChange();
}

// cuda/ctensormath.cu.h:502
template<class type_t>
void CTensorMath<type_t>::ConcatecationZ(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_InputA,const CTensor<type_t> &cTensor_InputB)
{
 if (cTensor_Output.Size_X!=cTensor_InputA.Size_X || cTensor_Output.Size_X!=cTensor_InputB.Size_X ||
     cTensor_Output.Size_Y!=cTensor_InputA.Size_Y || cTensor_Output.Size_Y!=cTensor_InputB.Size_Y ||
     cTensor_Output.Size_Z!=(cTensor_InputA.Size_Z+cTensor_InputB.Size_Z))
 {
  throw "CTensor::ConcatecationZ: tensor sizes do not match!";
 }
 const float *a=B200FloatPtr(cTensor_InputA.DeviceRead());
 const float *b=B200FloatPtr(cTensor_InputB.DeviceRead());
 B200Check(b200_concat_z(B200FloatPtr(cTensor_Output.DeviceWrite()),cTensor_Output.Size_W,a,cTensor_InputA.Size_W,cTensor_InputA.Size_Z,
                         b,cTensor_InputB.Size_W,cTensor_InputB.Size_Z,static_cast<size_t>(cTensor_Output.Size_X)*cTensor_Output.Size_Y,Stream()));
 cTensor_Output.SetDeviceOnChange();
}

// cuda/ctensormath.cu.h:569
template<class type_t>
void CTensorMath<type_t>::SplitZ(CTensor<type_t> &cTensor_OutputA,CTensor<type_t> &cTensor_OutputB,const CTensor<type_t> &cTensor_Input)
{
 if (cTensor_Input.Size_X!=cTensor_OutputA.Size_X || cTensor_Input.Size_X!=cTensor_OutputB.Size_X ||
     cTensor_Input.Size_Y!=cTensor_OutputA.Size_Y || cTensor_Input.Size_Y!=cTensor_OutputB.Size_Y ||
     cTensor_Input.Size_Z!=(cTensor_OutputA.Size_Z+cTensor_OutputB.Size_Z) ||
     cTensor_Input.Size_W!=cTensor_OutputA.Size_W || cTensor_Input.Size_W!=cTensor_OutputB.Size_W)
 {
  throw "CTensor::SplitZ: tensor sizes do not match!";
 }
 const float *in=B200FloatPtr(cTensor_Input.DeviceRead());
 B200Check(b200_split_z(B200FloatPtr(cTensor_OutputA.DeviceWrite()),cTensor_OutputA.Size_Z,B200FloatPtr(cTensor_OutputB.DeviceWrite()),cTensor_OutputB.Size_Z,
                        in,cTensor_Input.Size_W,static_cast<size_t>(cTensor_Input.Size_X)*cTensor_Input.Size_Y,Stream()));
 cTensor_OutputA.SetDeviceOnChange();
 cTensor_OutputB.SetDeviceOnChange();
}

// cuda/ctensormath.cu.h:3061
template<class type_t>
void CTensorMath<type_t>::SetTimeStep(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,const CTensor<uint32_t> &cTensor_TimeStep)
{
 if (!SameZYX(cTensor_Input,cTensor_Output) || cTensor_Input.Size_W!=cTensor_Output.Size_W || cTensor_TimeStep.Size_W!=cTensor_Input.Size_W ||
     cTensor_TimeStep.Size_X!=1 || cTensor_TimeStep.Size_Y!=1 || cTensor_TimeStep.Size_Z!=1)
 {
  throw "CTensor::SetTimeStep: tensor sizes do not match!";
 }
 const float *in=B200FloatPtr(cTensor_Input.DeviceRead());
 const uint32_t *time_step=cTensor_TimeStep.DeviceRead();
 B200Check(b200_set_time_step(B200FloatPtr(cTensor_Output.DeviceWrite()),in,time_step,cTensor_Input.Size_W,PlaneCount(cTensor_Input),Stream()));
 cTensor_Output.SetDeviceOnChange();
}

// cuda/ctensormath.cu.h:3131
template<class type_t>
void CTensorMath<type_t>::CreateDropOutMatrix(CTensor<type_t> &cTensor_Output,type_t drop_out)
{
 B200Check(b200_dropout_mask(B200FloatPtr(cTensor_Output.DeviceWrite()),PlaneCount(cTensor_Output)*cTensor_Output.Size_W,static_cast<float>(drop_out),NextSeed(),Stream()));
 cTensor_Output.SetDeviceOnChange();
}

// cuda/ctensormath.cu.h:3187
template<class type_t>
void CTensorMath<type_t>::SetNormalNoise(CTensor<type_t> &cTensor_Output)
{
 B200Check(b200_normal_noise(B200FloatPtr(cTensor_Output.DeviceWrite()),PlaneCount(cTensor_Output)*cTensor_Output.Size_W,NextSeed(),Stream()));
 cTensor_Output.SetDeviceOnChange();
}

// cuda/ctensormath.cu.h:3250
template<class type_t>
void CTensorMath<type_t>::GetNoiseImageAndNoise(CTensor<type_t> &cTensor_NoisyImage,CTensor<type_t> &cTensor_Noise,const CTensor<type_t> &cTensor_Image,const CTensor<type_t> &cTensor_SqrtAlphaBar,const CTensor<type_t> &cTensor_SqrtOneMinusAlphaBar)
{
 if (!SameZYX(cTensor_NoisyImage,cTensor_Noise) || cTensor_NoisyImage.Size_W!=cTensor_Noise.Size_W)
 {
  throw "CTensor::GetNoiseImageAndNoise: the sizes of NoisyImage and Noise do not match!";
 }
 if (!SameZYX(cTensor_NoisyImage,cTensor_Image) || cTensor_NoisyImage.Size_W!=cTensor_Image.Size_W)
 {
  throw "CTensor::GetNoiseImageAndNoise: the sizes of NoisyImage and Image do not match!";
 }
 if (cTensor_SqrtAlphaBar.Size_W!=cTensor_Image.Size_W || cTensor_SqrtOneMinusAlphaBar.Size_W!=cTensor_Image.Size_W)
 {
  throw "CTensor::GetNoiseImageAndNoise: the sizes of SqrtAlphaBar/SqrtOneMinusAlphaBar and Image do not match!";
 }
 const float *image=B200FloatPtr(cTensor_Image.DeviceRead());
 const float *sa=B200FloatPtr(cTensor_SqrtAlphaBar.DeviceRead());
 const float *so=B200FloatPtr(cTensor_SqrtOneMinusAlphaBar.DeviceRead());
 B200Check(b200_noisy_image(B200FloatPtr(cTensor_NoisyImage.DeviceWrite()),B200FloatPtr(cTensor_Noise.DeviceWrite()),image,sa,so,cTensor_Image.Size_W,
                            PlaneCount(cTensor_Image),1,NextSeed(),Stream()));
 cTensor_Noise.SetDeviceOnChange();
 cTensor_NoisyImage.SetDeviceOnChange();
}

template<class type_t>
void CTensorMath<type_t>::Transponse(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input)
{
 if (cTensor_Output.Size_Y!=cTensor_Input.Size_X || cTensor_Output.Size_X!=cTensor_Input.Size_Y || cTensor_Output.Size_Z!=cTensor_Input.Size_Z || cTensor_Output.Size_W!=cTensor_Input.Size_W)
 {
  throw "CTensor::Transponse: tensor sizes do not match!";
 }
 const float *in=B200FloatPtr(cTensor_Input.DeviceRead());
 B200Check(b200_transpose(B200FloatPtr(cTensor_Output.DeviceWrite()),in,cTensor_Input.Size_W*cTensor_Input.Size_Z,cTensor_Input.Size_Y,cTensor_Input.Size_X,Stream()));
 cTensor_Output.SetDeviceOnChange();
}

template<class type_t>
CTensor<type_t> CTensorMath<type_t>::Transpose(const CTensor<type_t> &cTensor_Input)
{
 CTensor<type_t> cTensor(cTensor_Input.Size_W,cTensor_Input.Size_Z,cTensor_Input.Size_X,cTensor_Input.Size_Y);
 Transponse(cTensor,cTensor_Input);
 return(cTensor);
}

//----------------------------------------------------------------------------------------------------
// resampling and pooling
//----------------------------------------------------------------------------------------------------
template<class type_t>
void CTensorMath<type_t>::UpSampling(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,uint32_t upsampling_x,uint32_t upsampling_y)
{
 if (cTensor_Input.Size_X!=cTensor_Output.Size_X/upsampling_x || cTensor_Input.Size_Y!=cTensor_Output.Size_Y/upsampling_y || cTensor_Input.Size_Z!=cTensor_Output.Size_Z ||
     cTensor_Input.Size_W!=cTensor_Output.Size_W || cTensor_Output.Size_X!=cTensor_Input.Size_X*upsampling_x || cTensor_Output.Size_Y!=cTensor_Input.Size_Y*upsampling_y)
 {
  throw "CTensor::UpSampling: tensor sizes do not match!";
 }
 const float *in=B200FloatPtr(cTensor_Input.DeviceRead());
 B200Check(b200_upsample(B200FloatPtr(cTensor_Output.DeviceWrite()),in,cTensor_Input.Size_W,cTensor_Input.Size_Z,cTensor_Input.Size_Y,cTensor_Input.Size_X,upsampling_x,upsampling_y,Stream()));
 cTensor_Output.SetDeviceOnChange();
}

template<class type_t>
void CTensorMath<type_t>::DownSampling(CTensor<type_t> &cTensor_Output,const CTensor<type_t> &cTensor_Input,uint32_t downsampling_x,uint32_t downsampling_y)
{
 if (cTensor_Input.Size_X/downsampling_x!=cTensor_Output.Size_X || cTensor_Input.Size_Y/downsampling_y!=cTensor_Output.Size_Y || cTensor_Input.Size_Z!=cTensor_Output.Size_Z || cTensor_Input.Size_W!=cTensor_Output.Size_W)
 {
  throw "CTensor::DownSampling: tensor sizes do not match!";
 }
 const float *in=B200FloatPtr(cTensor_Input.DeviceRead());
 B200Check(b200_downsample(B200FloatPtr(cTensor_Output.DeviceWrite()),in,cTensor_Input.Size_W,cTensor_Input.Size_Z,cTensor_Input.Size_Y,cTensor_Input.Size_X,downsampling_x,downsampling_y,Stream()));
 cTensor_Output.SetDeviceOnChange();
}

// The position tensor is written although it is passed by const reference: the reference's signature
// (cuda/ctensormath.cu.h:127), which relies on the members being mutable.
template<class type_t>
void CTensorMath<type_t>::MaxPooling(CTensor<type_t> &cTensor_Output,const CTensor<typename CTensorMath<type_t>::SPos> &cTensor_Position,const CTensor<type_t> &cTensor_Input,uint32_t pooling_x,uint32_t pooling_y)
{
 if ((cTensor_Input.GetSizeX()/pooling_x)!=cTensor_Output.Size_X || (cTensor_Input.GetSizeY()/pooling_y)!=cTensor_Output.Size_Y || cTensor_Input.Size_Z!=cTensor_Output.Size_Z || cTensor_Input.Size_W!=cTensor_Output.Size_W ||
     cTensor_Position.GetSizeX()!=cTensor_Output.Size_X || cTensor_Position.GetSizeY()!=cTensor_Output.Size_Y || cTensor_Position.GetSizeZ()!=cTensor_Output.Size_Z || cTensor_Position.GetSizeW()!=cTensor_Output.Size_W)
 {
  throw "CTensor::MaxPooling: tensor sizes do not match!";
 }
 const float *in=B200FloatPtr(cTensor_Input.DeviceRead());
 uint32_t *pos=reinterpret_cast<uint32_t*>(cTensor_Position.GetDeviceVector().get());
 B200Check(b200_maxpool(B200FloatPtr(cTensor_Output.DeviceWrite()),pos,in,cTensor_Input.Size_W,cTensor_Input.Size_Z,cTensor_Input.Size_Y,cTensor_Input.Size_X,pooling_x,pooling_y,Stream()));
 cTensor_Output.SetDeviceOnChange();
 cTensor_Position.SetDeviceOnChange();
}

template<class type_t>
void CTensorMath<type_t>::MaxPoolingBackward(CTensor<type_t> &cTensor_Output,const CTensor<typename CTensorMath<type_t>::SPos> &cTensor_Position,const CTensor<type_t> &cTensor_Input,uint32_t pooling_x,uint32_t pooling_y)
{
 if (cTensor_Input.Size_X!=(cTensor_Output.Size_X/pooling_x) || cTensor_Input.Size_Y!=(cTensor_Output.Size_Y/pooling_y) || cTensor_Input.Size_Z!=cTensor_Output.Size_Z || cTensor_Input.Size_W!=cTensor_Output.Size_W)
 {
  throw "CTensor::MaxPoolingBackward: tensor sizes do not match!";
 }
 const float *in=B200FloatPtr(cTensor_Input.DeviceRead());
 cTensor_Position.CopyToDevice();
 const uint32_t *pos=reinterpret_cast<const uint32_t*>(cTensor_Position.GetDeviceVector().get());
 B200Check(b200_maxpool_backward(B200FloatPtr(cTensor_Output.DeviceWrite()),pos,in,cTensor_Output.Size_W,cTensor_Output.Size_Z,cTensor_Output.Size_Y,cTensor_Output.Size_X,pooling_x,pooling_y,Stream()));
 cTensor_Output.SetDeviceOnChange();
}

template<class type_t>
void CTensorMath<type_t>::Adam(CTensor<type_t> &cTensor_Weight,CTensor<type_t> &cTensor_dWeight,CTensor<type_t> &cTensor_M,CTensor<type_t> &cTensor_V,uint32_t batch_size,double speed,double beta1,double beta2,double epsilon,double iteration)
{
 if (cTensor_Weight.Count()!=cTensor_dWeight.Count() || cTensor_Weight.Count()!=cTensor_M.Count() || cTensor_Weight.Count()!=cTensor_V.Count() ||
     SameZYX(cTensor_Weight,cTensor_dWeight)==false || SameZYX(cTensor_Weight,cTensor_M)==false || SameZYX(cTensor_Weight,cTensor_V)==false)
 {
  throw "CTensor::Adam: tensor sizes do not match!";
 }
 const float *dw=B200FloatPtr(cTensor_dWeight.DeviceRead());
 float *m=B200FloatPtr(cTensor_M.DeviceRead());
 float *v=B200FloatPtr(cTensor_V.DeviceRead());
 // the reference's CUDA kernel corrects the moments with iteration+1 (cuda/ctensormath.cu.h:3011)
 B200Check(b200_adam(B200FloatPtr(cTensor_Weight.DeviceRead()),dw,m,v,cTensor_Weight.Count(),batch_size,speed,beta1,beta2,epsilon,iteration+1,Stream()));
 cTensor_Weight.SetDeviceOnChange();
 cTensor_M.SetDeviceOnChange();
 cTensor_V.SetDeviceOnChange();
}

#endif
