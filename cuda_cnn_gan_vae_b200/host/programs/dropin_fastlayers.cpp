// This package's own layer classes (host/netlayer/: CNetLayerLinear, CNetLayerBackConvolution,
// CNetLayerBatchNormalization, CNetLayerConvolution) in one network with the reference's unmodified
// CNetLayerConvolutionInput and CNetLayerFunction classes, driven through the INetLayer interface the way the
// reference's models drive their layers: Reset, TrainingStart, Forward, SetOutputError, TrainingBackward,
// TrainingUpdateWeight, Forward.  Every tensor of the step is dumped as text; tests/test_gpu_dropin.py rebuilds the
// same chain on the CPU checker from the dumped weights and compares.  The program also saves the network to the
// reference's checkpoint format, loads it into a second network and checks that the second network reproduces the
// first one's output, and asserts that the weight gradient of the convolution layers ran on the tensor cores.
//   dropin_fastlayers <dump> <checkpoint> [precision mode]
#include <cstring>
#include <cstdlib>
#include <string>
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cmath>
#include <memory>
#include <vector>
#include <random>

#include "netlayer/cnetlayerconvolutioninput.cu.h"
#include "netlayer/cnetlayerlinear.cu.h"
#include "netlayer/cnetlayerbackconvolution.cu.h"
#include "netlayer/cnetlayerbatchnormalization.cu.h"
#include "netlayer/cnetlayerfunction.cu.h"
#include "netlayer/cnetlayerconvolution.cu.h"

typedef float type_t;
typedef std::vector<std::shared_ptr<INetLayer<type_t> > > net_t;
static const uint32_t BATCH=16;

static void Dump(FILE *file,const std::string &name,CTensor<type_t> &t)
{
 size_t count=static_cast<size_t>(t.GetSizeW())*t.GetSizeZ()*t.GetSizeY()*t.GetSizeX();
 fprintf(file,"tensor %s %lu\n",name.c_str(),static_cast<unsigned long>(count));
 for(uint32_t w=0;w<t.GetSizeW();w++)
  for(uint32_t z=0;z<t.GetSizeZ();z++)
   for(uint32_t y=0;y<t.GetSizeY();y++)
    for(uint32_t x=0;x<t.GetSizeX();x++) fprintf(file,"%.9g\n",static_cast<double>(t.GetElement(w,z,y,x)));
}

// noise[20] -> Linear 32x4x4 -> transposed convolution 4x4 s2 p1 to 16x8x8 -> batch normalisation -> LeakyReLU
//           -> convolution 4x4 s2 p1 with 24 kernels to 24x4x4 -> tanh
static void Build(net_t &net)
{
 net.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerConvolutionInput<type_t>(1,20,1,BATCH)));
 net.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerLinear<type_t>(32*4*4,net.back().get(),BATCH)));
 net.back()->GetOutputTensor().ReinterpretSize(BATCH,32,4,4);        // the reference's models view the Linear output as a volume (cmodel_gan.cu.h:150)
 net.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerBackConvolution<type_t>(4,16,2,2,1,1,net.back().get(),BATCH)));
 net.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerBatchNormalization<type_t>(0.9,net.back().get(),BATCH)));
 net.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerFunction<type_t>(NNeuron::NEURON_FUNCTION_LEAKY_RELU,net.back().get(),BATCH)));
 net.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerConvolution<type_t>(24,4,2,2,1,1,net.back().get(),BATCH)));
 net.push_back(std::shared_ptr<INetLayer<type_t> >(new CNetLayerFunction<type_t>(NNeuron::NEURON_FUNCTION_TANGENCE,net.back().get(),BATCH)));
}

template<class layer_t>
static void DumpParams(FILE *file,const char *prefix,INetLayer<type_t> *layer,bool gradients)
{
 layer_t *own=dynamic_cast<layer_t*>(layer);
 if (own==NULL) throw("unexpected layer class");
 for(size_t n=0;n<own->GetParamCount();n++)
 {
  char name[64];
  snprintf(name,sizeof(name),"%s_%s%u",prefix,gradients?"gradient":"param",static_cast<unsigned>(n));
  Dump(file,name,gradients?own->GetParamGradientTensor(n):own->GetParamTensor(n));
 }
}

static void DumpAllParams(FILE *file,net_t &net,const char *tag,bool gradients)
{
 std::string t(tag);
 DumpParams<CNetLayerLinear<type_t> >(file,(t+"linear").c_str(),net[1].get(),gradients);
 DumpParams<CNetLayerBackConvolution<type_t> >(file,(t+"backconv").c_str(),net[2].get(),gradients);
 DumpParams<CNetLayerBatchNormalization<type_t> >(file,(t+"bn").c_str(),net[3].get(),gradients);
 DumpParams<CNetLayerConvolution<type_t> >(file,(t+"conv").c_str(),net[5].get(),gradients);
}

// Reset() of the Linear and of the convolution layer draws its weights from std::random_device (common/crandom.h:94): another
// network on every run.  The comparison wants ONE network, so the weights are drawn again over the same range from a
// generator with a fixed seed.
template<class layer_t>
static void RedrawWeights(INetLayer<type_t> *layer,uint32_t seed)
{
 layer_t *own=dynamic_cast<layer_t*>(layer);
 if (own==NULL) throw("unexpected layer class");
 CTensor<type_t> &weight=own->GetParamTensor(0);
 type_t limit=0;
 for(uint32_t w=0;w<weight.GetSizeW();w++)
  for(uint32_t z=0;z<weight.GetSizeZ();z++)
   for(uint32_t y=0;y<weight.GetSizeY();y++)
    for(uint32_t x=0;x<weight.GetSizeX();x++) limit=std::max(limit,static_cast<type_t>(fabs(weight.GetElement(w,z,y,x))));
 std::mt19937 generator(seed);
 std::uniform_real_distribution<type_t> distribution(-limit,limit);
 for(uint32_t w=0;w<weight.GetSizeW();w++)
  for(uint32_t z=0;z<weight.GetSizeZ();z++)
   for(uint32_t y=0;y<weight.GetSizeY();y++)
    for(uint32_t x=0;x<weight.GetSizeX();x++) weight.SetElement(w,z,y,x,distribution(generator));
}

int main(int argc,char **argv)
{
 if (argc<3) return(3);
 try
 {
  const int mode=(argc>3)?atoi(argv[3]):B200_TF32X3;
  B200Check(b200_set_precision(mode));
  srand(12345);
  net_t net;
  Build(net);
  for(size_t n=0;n<net.size();n++) net[n]->Reset();
  const uint32_t seed=(argc>4)?static_cast<uint32_t>(atoi(argv[4])):777u;
  RedrawWeights<CNetLayerLinear<type_t> >(net[1].get(),seed);
  RedrawWeights<CNetLayerBackConvolution<type_t> >(net[2].get(),seed+1);
  RedrawWeights<CNetLayerConvolution<type_t> >(net[5].get(),seed+2);
  for(size_t n=0;n<net.size();n++) net[n]->TrainingModeAdam();
  for(size_t n=0;n<net.size();n++) net[n]->TrainingStart();

  CTensor<type_t> input(BATCH,1,20,1);
  for(uint32_t w=0;w<BATCH;w++)
   for(uint32_t y=0;y<20;y++) input.SetElement(w,0,y,0,static_cast<type_t>(sin(0.37*y+2.3*w)+0.3*cos(1.9*y*w)));
  CTensor<type_t> error(BATCH,24,4,4);
  for(uint32_t w=0;w<BATCH;w++)
   for(uint32_t z=0;z<24;z++)
    for(uint32_t y=0;y<4;y++)
     for(uint32_t x=0;x<4;x++) error.SetElement(w,z,y,x,static_cast<type_t>(cos(0.53*x+0.71*y+1.3*z+1.1*w)));

  FILE *file=fopen(argv[1],"wb");
  if (file==NULL) throw("cannot open the dump file");
  Dump(file,"input",input);
  Dump(file,"error",error);
  DumpAllParams(file,net,"",false);

  net[0]->SetOutput(input);
  for(size_t n=0;n<net.size();n++) net[n]->TrainingResetDeltaWeight();
  for(size_t n=0;n<net.size();n++) net[n]->Forward();
  for(size_t n=1;n<net.size();n++) Dump(file,"output_"+std::to_string(n),net[n]->GetOutputTensor());

  net.back()->SetOutputError(error);
  for(size_t m=0,n=net.size()-1;m<net.size();m++,n--)
  {
   net[n]->TrainingBackward();
   // both convolution layers must have formed their weight gradient on the tensor cores (not in the bit-exact fp32 mode)
   if ((n==5 || n==2) && mode!=B200_FP32 && b200_last_path()!=B200_PATH_TCGEN05) throw("the convolution layer's backward pass did not run on the tensor cores");
  }
  for(size_t n=1;n<net.size();n++) Dump(file,"delta_"+std::to_string(n),net[n]->GetDeltaTensor());
  DumpAllParams(file,net,"",true);

  for(size_t n=0;n<net.size();n++) net[n]->TrainingUpdateWeight(0.01,0);      // iteration 0: the update uses iteration+1
  DumpAllParams(file,net,"updated_",false);
  for(size_t n=0;n<net.size();n++) net[n]->Forward();
  Dump(file,"output_after_update",net.back()->GetOutputTensor());
  fclose(file);

  // checkpoint round trip in the reference's format: a second network loads what the first saved
  {
   std::unique_ptr<IDataStream> stream(IDataStream::CreateNewDataStreamFile(argv[2],true));
   for(size_t n=0;n<net.size();n++) net[n]->Save(stream.get());
  }
  net_t twin;
  Build(twin);
  {
   std::unique_ptr<IDataStream> stream(IDataStream::CreateNewDataStreamFile(argv[2],false));
   if (stream->IsFail()==true) throw("cannot reopen the checkpoint");
   for(size_t n=0;n<twin.size();n++) twin[n]->Load(stream.get(),true);
  }
  for(size_t n=0;n<twin.size();n++) twin[n]->TrainingStart();      // batch statistics, as in the first network
  twin[0]->SetOutput(input);
  for(size_t n=0;n<twin.size();n++) twin[n]->Forward();
  if (twin.back()->GetOutputTensor().Compare(net.back()->GetOutputTensor(),"",false)==false) throw("the reloaded network gives another output");
  for(size_t n=0;n<net.size();n++) net[n]->TrainingStop();
  for(size_t n=0;n<twin.size();n++) twin[n]->TrainingStop();
  printf("PASS\n");
  return(0);
 }
 catch(const char *text)
 {
  printf("thrown: %s\n",text);
  return(2);
 }
}
