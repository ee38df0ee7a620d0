// Drop-in check at layer level: a small network built from the reference's UNMODIFIED layer classes
// (netlayer/cnetlayerconvolutioninput, cnetlayerconvolution, cnetlayerfunction, cnetlayerlinear of
// da-nie/CUDA-CNN-GAN-VAE) runs one training step.  The same source is compiled twice by
// host/build_dropin.py: against the reference's CPU backend (-DUSE_CPU) and against this package's
// tensor headers + libb200conv.so.  Both load the same weight file (the reference's own checkpoint
// format), and dump outputs and deltas as text; tests/test_gpu_dropin.py compares the two dumps.
//   dropin_layers gen  <weights>            initialise the weights (reference initialiser) and save them
//   dropin_layers run  <weights> <dump> [precision mode]   load, forward, backward, Adam update, forward again, dump
#include <cstring>
#include <cstdlib>
#include <string>
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cmath>
#include <memory>
#include <vector>

#include "netlayer/cnetlayerconvolutioninput.cu.h"
#include "netlayer/cnetlayerconvolution.cu.h"
#include "netlayer/cnetlayerfunction.cu.h"
#include "netlayer/cnetlayerlinear.cu.h"
#include "netlayer/cnetlayerupsampling.cu.h"

typedef float type_t;
static const uint32_t BATCH=6;

static void Dump(FILE *file,const char *name,CTensor<type_t> &t)
{
 size_t count=static_cast<size_t>(t.GetSizeW())*t.GetSizeZ()*t.GetSizeY()*t.GetSizeX();
 fprintf(file,"tensor %s %lu\n",name,static_cast<unsigned long>(count));
 for(uint32_t w=0;w<t.GetSizeW();w++)
  for(uint32_t z=0;z<t.GetSizeZ();z++)
   for(uint32_t y=0;y<t.GetSizeY();y++)
    for(uint32_t x=0;x<t.GetSizeX();x++) fprintf(file,"%.9g\n",static_cast<double>(t.GetElement(w,z,y,x)));
}

int main(int argc,char **argv)
{
 if (argc<3) return(3);
 try
 {
#ifndef USE_CPU
  if (argc>4) B200Check(b200_set_precision(atoi(argv[4])));
#endif
  std::vector<std::shared_ptr<INetLayer<type_t> > > net;
  net.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerConvolutionInput<type_t>(3,16,16,BATCH)));
  net.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerConvolution<type_t>(32,3,1,1,1,1,net.back().get(),BATCH)));
  net.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerFunction<type_t>(NNeuron::NEURON_FUNCTION_LEAKY_RELU,net.back().get(),BATCH)));
  net.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerConvolution<type_t>(48,4,2,2,1,1,net.back().get(),BATCH)));
  net.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerFunction<type_t>(NNeuron::NEURON_FUNCTION_TANGENCE,net.back().get(),BATCH)));
  net.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerLinear<type_t>(10,net.back().get(),BATCH)));
  net.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerFunction<type_t>(NNeuron::NEURON_FUNCTION_SIGMOID,net.back().get(),BATCH)));

  // a second chain through the upsampling layer (UpSampling forward, DownSampling backward)
  std::vector<std::shared_ptr<INetLayer<type_t> > > up;
  up.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerConvolutionInput<type_t>(3,8,8,BATCH)));
  up.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerUpSampling<type_t>(2,2,up.back().get(),BATCH)));
  up.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerConvolution<type_t>(16,3,1,1,1,1,up.back().get(),BATCH)));
  up.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerFunction<type_t>(NNeuron::NEURON_FUNCTION_LEAKY_RELU,up.back().get(),BATCH)));
  up.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerLinear<type_t>(5,up.back().get(),BATCH)));
  up.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerFunction<type_t>(NNeuron::NEURON_FUNCTION_SIGMOID,up.back().get(),BATCH)));

  if (strcmp(argv[1],"gen")==0)
  {
   for(size_t n=0;n<net.size();n++) net[n]->Reset();
   for(size_t n=0;n<up.size();n++) up[n]->Reset();
   std::unique_ptr<IDataStream> stream(IDataStream::CreateNewDataStreamFile(argv[2],true));
   for(size_t n=0;n<net.size();n++) net[n]->Save(stream.get());
   for(size_t n=0;n<up.size();n++) up[n]->Save(stream.get());
   return(0);
  }
  if (argc<4) return(3);
  {
   std::unique_ptr<IDataStream> stream(IDataStream::CreateNewDataStreamFile(argv[2],false));
   if (stream->IsFail()==true) throw("cannot open the weight file");
   for(size_t n=0;n<net.size();n++) net[n]->Load(stream.get(),true);
   for(size_t n=0;n<up.size();n++) up[n]->Load(stream.get(),true);
  }
  for(size_t n=0;n<net.size();n++) net[n]->TrainingStart();
  for(size_t n=0;n<up.size();n++) up[n]->TrainingStart();

  CTensor<type_t> input(BATCH,3,16,16);
  for(uint32_t w=0;w<BATCH;w++)
   for(uint32_t z=0;z<3;z++)
    for(uint32_t y=0;y<16;y++)
     for(uint32_t x=0;x<16;x++) input.SetElement(w,z,y,x,static_cast<type_t>(sin(0.37*x+0.91*y+1.7*z+2.3*w)));
  CTensor<type_t> error(BATCH,1,10,1);
  for(uint32_t w=0;w<BATCH;w++)
   for(uint32_t y=0;y<10;y++) error.SetElement(w,0,y,0,static_cast<type_t>(cos(0.53*y+1.1*w)));

  FILE *file=fopen(argv[3],"wb");
  if (file==NULL) throw("cannot open the dump file");
  net[0]->SetOutput(input);
  for(size_t n=0;n<net.size();n++) net[n]->Forward();
  Dump(file,"output_1",net.back()->GetOutputTensor());
  Dump(file,"conv1_output",net[1]->GetOutputTensor());
  Dump(file,"conv2_output",net[3]->GetOutputTensor());

  for(size_t n=0;n<net.size();n++) net[n]->TrainingResetDeltaWeight();
  net.back()->SetOutputError(error);
  for(size_t m=0,n=net.size()-1;m<net.size();m++,n--) net[n]->TrainingBackward();
  Dump(file,"linear_delta",net[5]->GetDeltaTensor());
  Dump(file,"conv2_delta",net[3]->GetDeltaTensor());
  Dump(file,"conv1_delta",net[1]->GetDeltaTensor());

  // The reference's two backends disagree on the Adam bias correction (the CUDA backend uses iteration+1,
  // cuda/ctensormath.cu.h:3011; the CPU backend the value given, cpu/ctensormath.h:1151): ask for the same step.
#ifdef USE_CPU
  const double iteration=2;
#else
  const double iteration=1;
#endif
  for(size_t n=0;n<net.size();n++) net[n]->TrainingUpdateWeight(0.01,iteration);
  for(size_t n=0;n<net.size();n++) net[n]->Forward();
  Dump(file,"output_2",net.back()->GetOutputTensor());

  // the upsampling chain: forward, backward
  CTensor<type_t> small(BATCH,3,8,8);
  for(uint32_t w=0;w<BATCH;w++)
   for(uint32_t z=0;z<3;z++)
    for(uint32_t y=0;y<8;y++)
     for(uint32_t x=0;x<8;x++) small.SetElement(w,z,y,x,static_cast<type_t>(cos(0.71*x+0.43*y+1.3*z+0.9*w)));
  CTensor<type_t> error_up(BATCH,1,5,1);
  for(uint32_t w=0;w<BATCH;w++)
   for(uint32_t y=0;y<5;y++) error_up.SetElement(w,0,y,0,static_cast<type_t>(sin(0.77*y+0.6*w)));
  up[0]->SetOutput(small);
  for(size_t n=0;n<up.size();n++) up[n]->Forward();
  Dump(file,"up_upsampled",up[1]->GetOutputTensor());
  Dump(file,"up_conv_output",up[2]->GetOutputTensor());
  Dump(file,"up_output",up.back()->GetOutputTensor());
  for(size_t n=0;n<up.size();n++) up[n]->TrainingResetDeltaWeight();
  up.back()->SetOutputError(error_up);
  for(size_t m=0,n=up.size()-1;m<up.size();m++,n--) up[n]->TrainingBackward();
  Dump(file,"up_conv_delta",up[2]->GetDeltaTensor());
  Dump(file,"up_upsampling_delta",up[1]->GetDeltaTensor());
  Dump(file,"up_input_delta",up[0]->GetDeltaTensor());
  fclose(file);
  for(size_t n=0;n<net.size();n++) net[n]->TrainingStop();
  for(size_t n=0;n<up.size();n++) up[n]->TrainingStop();
  return(0);
 }
 catch(const char *text)
 {
  printf("thrown: %s\n",text);
  return(2);
 }
}
