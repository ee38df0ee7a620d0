// Drop-in check: the reference's own known-answer suite, CTensorTest<float>::Test()
// (cuda/ctensortest.cu.h of da-nie/CUDA-CNN-GAN-VAE), compiled UNMODIFIED against this package's
// tensor headers (host/cuda/*.cu.h standing in for the reference's cuda/*.cu.h) and run on the GPU
// through libb200conv.so.  Built by host/build_dropin.py; exit code 0 = every check passed.
#include <cstring>
#include <string>
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cmath>

#include "cuda/ctensortest.cu.h"

int main(int argc,char **argv)
{
 int mode=B200_TF32X3;
 if (argc>1) mode=atoi(argv[1]);
 try
 {
  B200Check(b200_set_precision(mode));
  bool ok=CTensorTest<float>::Test();
  B200Check(b200_stream_status(B200TensorStream()));
  printf("\nreference CTensorTest<float>::Test() on libb200conv.so (precision mode %i): %s\n",mode,ok?"PASS":"FAIL");
  return(ok?0:1);
 }
 catch(const char *text)
 {
  printf("thrown: %s\n",text);
  return(2);
 }
}
