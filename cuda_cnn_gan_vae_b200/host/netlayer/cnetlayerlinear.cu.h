#ifndef C_NET_LAYER_LINEAR_H
#define C_NET_LAYER_LINEAR_H

// CNetLayerLinear of da-nie/CUDA-CNN-GAN-VAE (netlayer/cnetlayerlinear.cu.h: interface :73-131, Forward :262,
// TrainingBackward :415, checkpoint :309-327) on libb200conv.so.  The reference multiplies the weight matrix with one column
// vector per sample, and for the weight gradient fills a [batch, neurons, inputs] tensor with per-sample outer products that
// AddSumW then reduces; here each of the three products is ONE matrix product over the whole batch (out[B x n] = X * W^T,
// prev[B x in] = D * W, dW[n x in] = D^T * X) that b200_mul runs on the tensor cores, and nothing of size batch x weights exists.

#include "b200netlayer.cu.h"

template<class type_t>
class CNetLayerLinear:public CB200NetLayer<type_t>
{
  typedef CB200NetLayer<type_t> Base;
  typedef CB200LayerPort<type_t> Port;
  using Base::Slot;
  using Base::PrevLayerPtr;
  using Base::BatchSize;
  using Base::cTensor_H;
  using Base::cTensor_Delta;
  using Base::cTensor_PrevLayerError;
  enum {WEIGHT=0,SHIFT=1};
  uint32_t Neurons;
  uint32_t Inputs;
  CTensor<type_t> cTensor_BatchGradient;///<dW of the current batch, [1,1,neurons,inputs]
 public:
  CNetLayerLinear(uint32_t neurons,INetLayer<type_t> *prev_layer_ptr=NULL,uint32_t batch_size=1):Base("Linear"),cTensor_BatchGradient(1,1,1,1)
  {
   Create(neurons,prev_layer_ptr,batch_size);
  }
  void Create(uint32_t neurons,INetLayer<type_t> *prev_layer_ptr=NULL,uint32_t batch_size=1)
  {
   Base::Attach(prev_layer_ptr,batch_size,true,"");
   Neurons=neurons;
   cTensor_H=CTensor<type_t>(BatchSize,1,Neurons,1);
   Slot.resize(2);
   if (PrevLayerPtr==NULL)        // an input layer only holds its output
   {
    Inputs=1;
    Slot[WEIGHT].Weight=CTensor<type_t>(1,1,1,1);
    Slot[SHIFT].Weight=CTensor<type_t>(1,1,1,1);
    return;
   }
   CTensor<type_t> &input=PrevLayerPtr->GetOutputTensor();
   Inputs=input.GetSizeX()*input.GetSizeY()*input.GetSizeZ();
   Slot[WEIGHT].Weight=CTensor<type_t>(1,1,Neurons,Inputs);
   Slot[SHIFT].Weight=CTensor<type_t>(1,1,Neurons,1);
   PrevLayerPtr->SetNextLayerPtr(this);
  }
  /// uniform weights in +-sqrt(6/inputs), shifts 0.1 (the reference's initialisation, :196-227)
  void Reset(void)
  {
   if (PrevLayerPtr==NULL) return;
   const type_t limit=static_cast<type_t>(sqrt(6.0/static_cast<double>(Inputs)));
   for(uint32_t y=0;y<Neurons;y++)
    for(uint32_t x=0;x<Inputs;x++) Slot[WEIGHT].Weight.SetElement(0,0,y,x,static_cast<type_t>(CRandom<type_t>::GetRandValue(2.0)-1.0)*limit);
   for(uint32_t y=0;y<Neurons;y++) Slot[SHIFT].Weight.SetElement(0,0,y,0,static_cast<type_t>(0.1));
  }
  void Forward(void)
  {
   if (PrevLayerPtr==NULL) return;
   if (Base::InputCount()!=Inputs) throw("the previous layer's output no longer has the size the Linear layer was created for");
   const float *input=Port::Read(PrevLayerPtr->GetOutputTensor());
   const float *weight=Port::Read(Base::Active(WEIGHT));
   const float *shift=Port::Read(Base::Active(SHIFT));
   float *output=Port::Write(cTensor_H);
   B200Check(b200_mul(output,BatchSize,weight,1,input,BatchSize,1,Neurons,Inputs,1,0,Port::Stream()));
   B200Check(b200_add(output,BatchSize,output,BatchSize,shift,1,Neurons,1.0f,1.0f,0,Port::Stream()));
  }
  void TrainingBackward(bool create_delta_weight=true)
  {
   if (PrevLayerPtr==NULL) return;
   const float *delta=Port::Read(cTensor_Delta);
   const float *weight=Port::Read(Slot[WEIGHT].Weight);
   // error of the previous layer: W^T * delta for every sample
   B200Check(b200_mul(Port::Write(cTensor_PrevLayerError),BatchSize,weight,1,delta,BatchSize,1,Neurons,Inputs,1,1,Port::Stream()));
   PrevLayerPtr->SetOutputError(cTensor_PrevLayerError);
   if (create_delta_weight==false) return;
   // sum over the samples of delta * input^T = D^T * X with D = [batch x neurons] and X = [batch x inputs] as stored
   const float *input=Port::Read(PrevLayerPtr->GetOutputTensor());
   float *batch_gradient=Port::Write(cTensor_BatchGradient);
   B200Check(b200_mul(batch_gradient,1,delta,1,input,1,1,BatchSize,Neurons,Inputs,1,Port::Stream()));
   float *dweight=Port::Update(Slot[WEIGHT].Gradient);
   B200Check(b200_add(dweight,1,dweight,1,batch_gradient,1,static_cast<size_t>(Neurons)*Inputs,1.0f,1.0f,0,Port::Stream()));
   float *dshift=Port::Update(Slot[SHIFT].Gradient);
   B200Check(b200_add_sum_w(dshift,1,dshift,1,delta,BatchSize,Neurons,1.0f,1.0f,Port::Stream()));
  }
  bool Save(IDataStream *iDataStream_Ptr)
  {
   Slot[WEIGHT].Weight.Save(iDataStream_Ptr);
   Slot[SHIFT].Weight.Save(iDataStream_Ptr);
   return(true);
  }
  bool Load(IDataStream *iDataStream_Ptr,bool check_size=false)
  {
   Slot[WEIGHT].Weight.Load(iDataStream_Ptr,check_size);
   Slot[SHIFT].Weight.Load(iDataStream_Ptr,check_size);
   return(true);
  }
 protected:
  void OnTrainingStart(void) {cTensor_BatchGradient=CTensor<type_t>(1,1,Neurons,Inputs);}
  void OnTrainingStop(void) {cTensor_BatchGradient=CTensor<type_t>(1,1,1,1);}
};

#endif
