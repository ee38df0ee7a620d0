"""The C++ mirror of the reference's tensor layer (cuda_cnn_gan_vae_b200/host/cuda/*.cu.h) compiles on its own and links
against the C-ABI library; no GPU is touched (nothing is executed beyond shape checks that throw before any launch)."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "cuda_cnn_gan_vae_b200", "host")
LIBDIR = os.path.join(ROOT, "cuda_cnn_gan_vae_b200")

PROGRAM = r"""
#include <cstdio>
#include <cstring>
#include "cuda/tensor.cu.h"
template class CTensor<float>;
template class CTensorMath<float>;
template class CTensorConv<float>;
template class CTensorApplyFunc<float>;
int main(void)
{
 // every public name the reference's layers use resolves; nothing is run on a device
 void (*forward)(CTensor<float>&,const CTensor<float>&,const CTensor<float>&,int32_t,int32_t,int32_t,uint32_t,const CTensor<float>&,int32_t,int32_t,int32_t,int32_t)=&CTensorConv<float>::ForwardConvolution;
 void (*mul)(CTensor<float>&,const CTensor<float>&,const CTensor<float>&,bool)=&CTensorMath<float>::Mul;
 printf("%i\n",(forward!=NULL && mul!=NULL)?1:0);
 return(0);
}
"""


def test_host_headers_compile_and_link(tmp_path):
    src = tmp_path / "host_check.cpp"
    src.write_text(PROGRAM)
    exe = tmp_path / "host_check"
    cmd = ["g++", "-std=c++14", "-w", "-I" + HOST, "-I" + os.path.join(ROOT, "include"), "-I/usr/local/cuda/include",
           "-o", str(exe), str(src), "-L" + LIBDIR, "-lb200conv", "-L/usr/local/cuda/lib64", "-lcudart",
           "-Wl,-rpath," + LIBDIR, "-Wl,-rpath,/usr/local/cuda/lib64"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.strip() == "1", r.stdout + r.stderr
