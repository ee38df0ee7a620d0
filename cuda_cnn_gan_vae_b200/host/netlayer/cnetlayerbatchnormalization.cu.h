#ifndef C_NET_LAYER_BATCH_NORMALIZATION_H
#define C_NET_LAYER_BATCH_NORMALIZATION_H

// CNetLayerBatchNormalization of da-nie/CUDA-CNN-GAN-VAE (netlayer/cnetlayerbatchnormalization.cu.h: interface :96-134,
// Forward :301-379, TrainingBackward :578-604, checkpoint :411-433): statistics per (z,y,x) element over the batch, eps 1e-6,
// running mean / variance blended with `momentum` during training and used when training is off.  The reference runs about a
// dozen element-wise launches per pass (and does not compile at its head revision); here the training passes are one kernel
// each (b200_bn_forward / b200_bn_backward, same order of floating-point operations), the inference pass a short chain of the
// tensor routines.  Checkpoint order: beta, gamma, mean, variance, momentum (double); training state: the Adam moments of
// gamma, then of beta.

#include "b200netlayer.cu.h"

template<class type_t>
class CNetLayerBatchNormalization:public CB200NetLayer<type_t>
{
  typedef CB200NetLayer<type_t> Base;
  typedef CB200LayerPort<type_t> Port;
  using Base::Slot;
  using Base::PrevLayerPtr;
  using Base::BatchSize;
  using Base::cTensor_H;
  using Base::cTensor_Delta;
  using Base::cTensor_PrevLayerError;
  using Base::EMAEnabled;
  using Base::UseEMA;
  using Base::EMA_K;
  enum {GAMMA=0,BETA=1};
  static constexpr double EPSILON_VARIANCE=1E-6;
  type_t Momentum;
  bool TrainingEnabled;
  CTensor<type_t> cTensor_XHAT;
  CTensor<type_t> cTensor_IVAR;
  CTensor<type_t> cTensor_BatchMean;
  CTensor<type_t> cTensor_BatchVariable;
  CTensor<type_t> cTensor_Mean;///<running statistics
  CTensor<type_t> cTensor_Variable;
  CTensor<type_t> cTensor_NewMean;///<running statistics of the step in progress (taken over by TrainingUpdateWeight)
  CTensor<type_t> cTensor_NewVariable;
  CTensor<type_t> cTensor_Mean_EMA;
  CTensor<type_t> cTensor_Variable_EMA;
  size_t ElementCount(void) const {return(static_cast<size_t>(cTensor_H.GetSizeX())*cTensor_H.GetSizeY()*cTensor_H.GetSizeZ());}
 public:
  CNetLayerBatchNormalization(type_t momentum,INetLayer<type_t> *prev_layer_ptr=NULL,uint32_t batch_size=1):Base("BatchNormalization"),
   cTensor_XHAT(1,1,1,1),cTensor_IVAR(1,1,1,1),cTensor_BatchMean(1,1,1,1),cTensor_BatchVariable(1,1,1,1),cTensor_Mean(1,1,1,1),cTensor_Variable(1,1,1,1),
   cTensor_NewMean(1,1,1,1),cTensor_NewVariable(1,1,1,1),cTensor_Mean_EMA(1,1,1,1),cTensor_Variable_EMA(1,1,1,1)
  {
   Create(momentum,prev_layer_ptr,batch_size);
  }
  void Create(type_t momentum,INetLayer<type_t> *prev_layer_ptr=NULL,uint32_t batch_size=1)
  {
   Base::Attach(prev_layer_ptr,batch_size,false,"a batch-normalisation layer cannot be the input layer");
   Momentum=momentum;
   TrainingEnabled=false;
   CTensor<type_t> &input=PrevLayerPtr->GetOutputTensor();
   const uint32_t z=input.GetSizeZ(),y=input.GetSizeY(),x=input.GetSizeX();
   cTensor_H=CTensor<type_t>(BatchSize,z,y,x);
   cTensor_XHAT=CTensor<type_t>(BatchSize,z,y,x);
   CTensor<type_t> statistic(1,z,y,x);
   cTensor_IVAR=statistic;cTensor_BatchMean=statistic;cTensor_BatchVariable=statistic;
   cTensor_Mean=statistic;cTensor_Variable=statistic;cTensor_NewMean=statistic;cTensor_NewVariable=statistic;
   Slot.resize(2);
   Slot[GAMMA].Weight=statistic;
   Slot[BETA].Weight=statistic;
   PrevLayerPtr->SetNextLayerPtr(this);
  }
  void Reset(void)
  {
   CTensorMath<type_t>::Fill(Slot[GAMMA].Weight,1);
   CTensorMath<type_t>::Fill(Slot[BETA].Weight,0);
   CTensorMath<type_t>::Fill(cTensor_Mean,0);
   CTensorMath<type_t>::Fill(cTensor_Variable,1);
  }
  void Forward(void)
  {
   if (Base::InputCount()!=ElementCount()) throw("the previous layer's output no longer has the size the batch-normalisation layer was created for");
   CTensor<type_t> &input=PrevLayerPtr->GetOutputTensor();
   if (TrainingEnabled==true)
   {
    const float *x=Port::Read(input);
    const float *gamma=Port::Read(Base::Active(GAMMA));
    const float *beta=Port::Read(Base::Active(BETA));
    B200Check(b200_bn_forward(Port::Write(cTensor_H),Port::Write(cTensor_XHAT),Port::Write(cTensor_IVAR),Port::Write(cTensor_BatchMean),Port::Write(cTensor_BatchVariable),
                              Port::Update(cTensor_NewMean),Port::Update(cTensor_NewVariable),x,gamma,beta,BatchSize,ElementCount(),
                              static_cast<float>(Momentum),static_cast<float>(EPSILON_VARIANCE),Port::Stream()));
    return;
   }
   // inference: the running statistics (or their moving average) instead of the batch's
   CTensor<type_t> &mean=(UseEMA==true)?cTensor_Mean_EMA:cTensor_Mean;
   CTensor<type_t> &variable=(UseEMA==true)?cTensor_Variable_EMA:cTensor_Variable;
   const uint32_t w=input.GetSizeW(),z=input.GetSizeZ(),y=input.GetSizeY(),x=input.GetSizeX();
   input.ReinterpretSize(BatchSize,cTensor_H.GetSizeZ(),cTensor_H.GetSizeY(),cTensor_H.GetSizeX());
   CTensorMath<type_t>::Sub(cTensor_XHAT,input,mean,1.0,1.0);
   input.ReinterpretSize(w,z,y,x);
   CTensorMath<type_t>::SQRT(cTensor_IVAR,variable,1,static_cast<type_t>(EPSILON_VARIANCE));
   CTensorMath<type_t>::Inv(cTensor_IVAR,cTensor_IVAR);
   CTensorMath<type_t>::TensorItemProduction(cTensor_XHAT,cTensor_XHAT,cTensor_IVAR);
   CTensorMath<type_t>::TensorItemProduction(cTensor_H,Base::Active(GAMMA),cTensor_XHAT);
   CTensorMath<type_t>::Add(cTensor_H,cTensor_H,Base::Active(BETA));
  }
  void TrainingBackward(bool create_delta_weight=true)
  {
   const float *delta=Port::Read(cTensor_Delta);
   const float *xhat=Port::Read(cTensor_XHAT);
   const float *ivar=Port::Read(cTensor_IVAR);
   const float *gamma=Port::Read(Slot[GAMMA].Weight);
   B200Check(b200_bn_backward(Port::Write(cTensor_PrevLayerError),Port::Update(Slot[GAMMA].Gradient),Port::Update(Slot[BETA].Gradient),delta,xhat,ivar,gamma,
                              BatchSize,ElementCount(),create_delta_weight?1:0,Port::Stream()));
   PrevLayerPtr->SetOutputError(cTensor_PrevLayerError);
  }
  bool Save(IDataStream *iDataStream_Ptr)
  {
   Slot[BETA].Weight.Save(iDataStream_Ptr);
   Slot[GAMMA].Weight.Save(iDataStream_Ptr);
   cTensor_Mean.Save(iDataStream_Ptr);
   cTensor_Variable.Save(iDataStream_Ptr);
   iDataStream_Ptr->SaveDouble(Momentum);
   return(true);
  }
  bool Load(IDataStream *iDataStream_Ptr,bool check_size=false)
  {
   Slot[BETA].Weight.Load(iDataStream_Ptr,check_size);
   Slot[GAMMA].Weight.Load(iDataStream_Ptr,check_size);
   cTensor_Mean.Load(iDataStream_Ptr,check_size);
   cTensor_Variable.Load(iDataStream_Ptr,check_size);
   Momentum=static_cast<type_t>(iDataStream_Ptr->LoadDouble());
   return(true);
  }
  bool LoadEMAWeight(IDataStream *iDataStream_Ptr,bool check_size=false)
  {
   Base::LoadEMAWeight(iDataStream_Ptr,check_size);
   cTensor_Mean_EMA.Load(iDataStream_Ptr,check_size);
   cTensor_Variable_EMA.Load(iDataStream_Ptr,check_size);
   return(true);
  }
  bool SaveEMAWeight(IDataStream *iDataStream_Ptr)
  {
   Base::SaveEMAWeight(iDataStream_Ptr);
   cTensor_Mean_EMA.Save(iDataStream_Ptr);
   cTensor_Variable_EMA.Save(iDataStream_Ptr);
   return(true);
  }
 protected:
  void OnTrainingStart(void) {TrainingEnabled=true;}
  void OnTrainingStop(void) {TrainingEnabled=false;}
  /// every step starts from the accepted running statistics (the reference's TrainingResetDeltaWeight, :611-618)
  void OnResetDeltaWeight(void)
  {
   cTensor_NewMean=cTensor_Mean;
   cTensor_NewVariable=cTensor_Variable;
  }
  /// the step's running statistics are accepted with the weights (:650-660)
  void OnUpdateWeight(void)
  {
   cTensor_Mean=cTensor_NewMean;
   cTensor_Variable=cTensor_NewVariable;
   if (EMAEnabled==false) return;
   CTensorMath<type_t>::Add(cTensor_Mean_EMA,cTensor_Mean_EMA,cTensor_Mean,static_cast<type_t>(EMA_K),static_cast<type_t>(1.0-EMA_K));
   CTensorMath<type_t>::Add(cTensor_Variable_EMA,cTensor_Variable_EMA,cTensor_Variable,static_cast<type_t>(EMA_K),static_cast<type_t>(1.0-EMA_K));
  }
  void OnEnableEMA(bool state)
  {
   if (state==true)
   {
    cTensor_Mean_EMA=cTensor_Mean;
    cTensor_Variable_EMA=cTensor_Variable;
   }
   else
   {
    cTensor_Mean_EMA=CTensor<type_t>(1,1,1,1);
    cTensor_Variable_EMA=CTensor<type_t>(1,1,1,1);
   }
  }
};

#endif
