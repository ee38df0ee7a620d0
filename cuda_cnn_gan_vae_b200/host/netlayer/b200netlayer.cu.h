#ifndef B200_NET_LAYER_CU_H
#define B200_NET_LAYER_CU_H

// Common part of this package's own layer classes (cnetlayerconvolution.cu.h, cnetlayerbackconvolution.cu.h,
// cnetlayerlinear.cu.h, cnetlayerbatchnormalization.cu.h in this directory).  They carry the reference's class names and the
// whole INetLayer interface (netlayer/inetlayer.cu.h:73-96 of da-nie/CUDA-CNN-GAN-VAE) so that a network assembled from the
// reference's layer classes can take them in place of the reference's headers of the same names, but their bodies go to the
// layer-level entry points of libb200conv.so: one batch-summed weight gradient on the tensor cores instead of a per-sample
// gradient tensor reduced with AddSumW, whole-batch products in the Linear layer, one kernel per batch-normalisation pass.
//
// Own design, not the reference's: every trainable tensor of a layer is a "slot" (weight, gradient, the two Adam moments,
// the moving average); reset, update, clipping, the training-state and moving-average files run over the slots in checkpoint
// order, so a layer class only states its geometry, its Forward and its TrainingBackward.

#include <stdio.h>
#include <stdint.h>
#include <math.h>
#include <string>
#include <vector>

#include "../common/idatastream.h"
#include "../common/crandom.h"
#include "inetlayer.cu.h"
#include "../cuda/tensor.cu.h"

// Device-side access to a CTensor for the layer classes (CTensor keeps its device pointer private).
template<class type_t>
class CB200LayerPort
{
 public:
  static const float* Read(const CTensor<type_t> &t) {return(reinterpret_cast<const float*>(t.DeviceRead()));}
  static float* Update(CTensor<type_t> &t) {float *p=reinterpret_cast<float*>(t.DeviceRead());t.SetDeviceOnChange();return(p);}
  static float* Write(CTensor<type_t> &t) {float *p=reinterpret_cast<float*>(t.DeviceWrite());t.SetDeviceOnChange();return(p);}
  static size_t Count(const CTensor<type_t> &t) {return(t.Count());}
  static void* Stream(void) {return(static_cast<void*>(B200TensorStream()));}
};

template<class type_t>
class CB200NetLayer:public INetLayer<type_t>
{
 protected:
  struct SSlot
  {
   CTensor<type_t> Weight;
   CTensor<type_t> Gradient;
   CTensor<type_t> M;
   CTensor<type_t> V;
   CTensor<type_t> Average;
  };
  typedef CB200LayerPort<type_t> Port;
  std::vector<SSlot> Slot;///<trainable tensors in checkpoint order
  INetLayer<type_t> *PrevLayerPtr;
  INetLayer<type_t> *NextLayerPtr;
  uint32_t BatchSize;
  CTensor<type_t> cTensor_H;///<layer output
  CTensor<type_t> cTensor_Delta;///<error at the layer output
  CTensor<type_t> cTensor_PrevLayerError;///<error handed to the previous layer
  const char *Name;
  using INetLayer<type_t>::Beta1;
  using INetLayer<type_t>::Beta2;
  using INetLayer<type_t>::Epsilon;
  using INetLayer<type_t>::EMAEnabled;
  using INetLayer<type_t>::UseEMA;
  using INetLayer<type_t>::EMA_K;
 protected:
  CB200NetLayer(const char *name):PrevLayerPtr(NULL),NextLayerPtr(NULL),BatchSize(1),cTensor_H(1,1,1,1),cTensor_Delta(1,1,1,1),cTensor_PrevLayerError(1,1,1,1),Name(name) {}
  /// the weights Forward uses: the trained ones or their moving average
  CTensor<type_t>& Active(size_t slot) {return(UseEMA==true?Slot[slot].Average:Slot[slot].Weight);}
  void Attach(INetLayer<type_t> *prev_layer_ptr,uint32_t batch_size,bool may_be_input,const char *input_error)
  {
   PrevLayerPtr=prev_layer_ptr;
   NextLayerPtr=NULL;
   BatchSize=batch_size;
   if (prev_layer_ptr==NULL && may_be_input==false) throw(input_error);
  }
  /// elements of one sample of the previous layer's output, whatever its current interpretation
  size_t InputCount(void) {return(Port::Count(PrevLayerPtr->GetOutputTensor())/BatchSize);}
 public:
  virtual ~CB200NetLayer() {}
  /// additions to the reference interface: the trainable tensors and their gradients in checkpoint order
  size_t GetParamCount(void) const {return(Slot.size());}
  CTensor<type_t>& GetParamTensor(size_t index) {return(Slot[index].Weight);}
  CTensor<type_t>& GetParamGradientTensor(size_t index) {return(Slot[index].Gradient);}

  void SetOutput(CTensor<type_t> &output) {cTensor_H.CopyItem(output);}
  void GetOutput(CTensor<type_t> &output)
  {
   if (output.GetSizeX()!=cTensor_H.GetSizeX() || output.GetSizeY()!=cTensor_H.GetSizeY() || output.GetSizeZ()!=cTensor_H.GetSizeZ() || output.GetSizeW()!=cTensor_H.GetSizeW()) throw("GetOutput: the size of the output tensor does not match the layer");
   output=cTensor_H;
  }
  CTensor<type_t>& GetOutputTensor(void) {return(cTensor_H);}
  void SetNextLayerPtr(INetLayer<type_t> *next_layer_ptr) {NextLayerPtr=next_layer_ptr;}
  CTensor<type_t>& GetDeltaTensor(void) {return(cTensor_Delta);}
  void SetOutputError(CTensor<type_t>& error) {cTensor_Delta=error;}
  void SetTimeStep(uint32_t index,uint32_t time_step) {}
  void PrintInputTensorSize(const std::string &name) {if (PrevLayerPtr!=NULL) PrevLayerPtr->GetOutputTensor().Print(name+" "+Name+": input",false);}
  void PrintOutputTensorSize(const std::string &name) {GetOutputTensor().Print(name+" "+Name+": output",false);}

  bool SaveTrainingParam(IDataStream *iDataStream_Ptr)
  {
   for(size_t n=0;n<Slot.size();n++)
   {
    Slot[n].M.Save(iDataStream_Ptr);
    Slot[n].V.Save(iDataStream_Ptr);
   }
   return(true);
  }
  bool LoadTrainingParam(IDataStream *iDataStream_Ptr)
  {
   for(size_t n=0;n<Slot.size();n++)
   {
    Slot[n].M.Load(iDataStream_Ptr);
    Slot[n].V.Load(iDataStream_Ptr);
   }
   return(true);
  }
  void TrainingStart(void)
  {
   cTensor_Delta=cTensor_H;
   if (PrevLayerPtr!=NULL) cTensor_PrevLayerError=PrevLayerPtr->GetOutputTensor();
   for(size_t n=0;n<Slot.size();n++)
   {
    Slot[n].Gradient=Slot[n].Weight;
    Slot[n].M=Slot[n].Weight;
    Slot[n].V=Slot[n].Weight;
    CTensorMath<type_t>::Fill(Slot[n].Gradient,0);
    CTensorMath<type_t>::Fill(Slot[n].M,0);
    CTensorMath<type_t>::Fill(Slot[n].V,0);
   }
   OnTrainingStart();
  }
  void TrainingStop(void)
  {
   cTensor_Delta=CTensor<type_t>(1,1,1,1);
   cTensor_PrevLayerError=CTensor<type_t>(1,1,1,1);
   for(size_t n=0;n<Slot.size();n++)
   {
    Slot[n].Gradient=CTensor<type_t>(1,1,1,1);
    Slot[n].M=CTensor<type_t>(1,1,1,1);
    Slot[n].V=CTensor<type_t>(1,1,1,1);
   }
   OnTrainingStop();
  }
  void TrainingResetDeltaWeight(void)
  {
   for(size_t n=0;n<Slot.size();n++) CTensorMath<type_t>::Fill(Slot[n].Gradient,0);
   OnResetDeltaWeight();
  }
  /// Adam (with the moving average of the weights in the same launch when it is enabled) or plain gradient descent over every
  /// slot; batch_scale multiplies the divisor of the summed gradient (data-parallel steps pass the number of devices).
  /// Adam's bias correction uses iteration+1, the rule of the reference's CUDA backend (cuda/ctensormath.cu.h:3011).
  void TrainingUpdateWeight(double speed,double iteration,double batch_scale=1)
  {
   for(size_t n=0;n<Slot.size();n++)
   {
    SSlot &s=Slot[n];
    if (INetLayer<type_t>::GetTrainingMode()==INetLayer<type_t>::TRAINING_MODE_ADAM)
    {
     float *average=(EMAEnabled==true)?Port::Update(s.Average):NULL;
     const float *gradient=Port::Read(s.Gradient);
     B200Check(b200_adam_ema(Port::Update(s.Weight),gradient,Port::Update(s.M),Port::Update(s.V),average,Port::Count(s.Weight),
                             static_cast<uint32_t>(BatchSize*batch_scale),speed,Beta1,Beta2,Epsilon,iteration+1,NULL,EMA_K,Port::Stream()));
    }
    else
    {
     CTensorMath<type_t>::Sub(s.Weight,s.Weight,s.Gradient,1,static_cast<type_t>(speed/static_cast<double>(BatchSize)/batch_scale));
     if (EMAEnabled==true) CTensorMath<type_t>::Add(s.Average,s.Average,s.Weight,static_cast<type_t>(EMA_K),static_cast<type_t>(1.0-EMA_K));
    }
   }
   OnUpdateWeight();
  }
  void ClipWeight(type_t min,type_t max)
  {
   for(size_t n=0;n<Slot.size();n++) CTensorMath<type_t>::Clip(Slot[n].Weight,min,max);
  }
  void EnableEMA(bool state)
  {
   EMAEnabled=state;
   for(size_t n=0;n<Slot.size();n++)
   {
    if (state==true) Slot[n].Average=Slot[n].Weight;
                else Slot[n].Average=CTensor<type_t>(1,1,1,1);
   }
   OnEnableEMA(state);
  }
  bool LoadEMAWeight(IDataStream *iDataStream_Ptr,bool check_size=false)
  {
   for(size_t n=0;n<Slot.size();n++) Slot[n].Average.Load(iDataStream_Ptr,check_size);
   return(true);
  }
  bool SaveEMAWeight(IDataStream *iDataStream_Ptr)
  {
   for(size_t n=0;n<Slot.size();n++) Slot[n].Average.Save(iDataStream_Ptr);
   return(true);
  }
 protected:
  virtual void OnTrainingStart(void) {}
  virtual void OnTrainingStop(void) {}
  virtual void OnResetDeltaWeight(void) {}
  virtual void OnUpdateWeight(void) {}
  virtual void OnEnableEMA(bool state) {}
 private:
  CB200NetLayer(const CB200NetLayer<type_t>&);
  CB200NetLayer<type_t>& operator=(const CB200NetLayer<type_t>&);
};

#endif
