#ifndef B200_C_TENSOR_CU_H
#define B200_C_TENSOR_CU_H

// CTensor<T>: the 4-D tensor (W = batch, Z = channel, Y, X; dense, row-major) of
// da-nie/CUDA-CNN-GAN-VAE, re-implemented over libb200conv.so and the CUDA runtime API.  Same class
// name, same public members and the same friend-visible private members as the reference
// (cuda/ctensor.cu.h:68-168), so that the reference's layer headers (netlayer/*.cu.h), its
// known-answer suite (cuda/ctensortest.cu.h) and main.cpp compile against this file unchanged when
// it stands in for cuda/ctensor.cu.h.  Plain C++ (no device code): a host vector, a device buffer
// and the reference's lazy coherence protocol (HostOnChange / DeviceOnChange, cuda/ctensor.cu.h:664-704).
// Errors follow the reference: logic errors throw a C string, CUDA failures throw too (the
// reference prints and calls exit(), cuda/handle_error.cu.h:7-18).

#include <stdint.h>
#include <stdio.h>
#include <math.h>
#include <string.h>
#include <string>
#include <vector>
#include <algorithm>

#include <cuda_runtime_api.h>
#include "b200conv.h"

#if defined(__has_include)
#if __has_include("../common/idatastream.h")
#include "../common/idatastream.h"
#define B200_HAVE_IDATASTREAM 1
#endif
#if __has_include("../system/system.h")
#include "../system/system.h"
#define B200_HAVE_SYSTEM 1
#endif
#endif
#ifndef B200_HAVE_IDATASTREAM
class IDataStream;
#endif

// Stream every tensor operation of this header set runs on (the reference uses the default stream).
inline cudaStream_t &B200TensorStream(void)
{
 static cudaStream_t stream=0;
 return(stream);
}

inline void B200CheckCuda(cudaError_t error,const char *what)
{
 if (error==cudaSuccess) return;
 static char text[256];
 snprintf(text,sizeof(text),"CUDA error in %s: %s",what,cudaGetErrorString(error));
 throw (const char*)text;
}

// Turns a status of the C ABI into the reference's error convention (throw "text").
inline void B200Check(int status)
{
 if (status!=B200_OK) throw b200_last_error();
}

template<class type_t> class CTensor;
template<class type_t> class CTensorMath;
template<class type_t> class CTensorConv;
template<class type_t> class CTensorApplyFunc;
template<class type_t> class CTensorTest;
template<class type_t> struct STensorKernel;
template<class type_t> class CB200LayerPort;

template<class type_t> CTensor<type_t> operator+(const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right);
template<class type_t> CTensor<type_t> operator-(const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right);
template<class type_t> CTensor<type_t> operator*(const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right);
template<class type_t> CTensor<type_t> operator*(const CTensor<type_t> &cTensor_Left,const type_t &value_right);
template<class type_t> CTensor<type_t> operator*(const type_t &value_left,const CTensor<type_t> &cTensor_Right);

// Device buffer of a tensor (counterpart of CCUDADeviceVector, cuda/ccudadevicevector.cu.h:40-72):
// RAII cudaMalloc/cudaFree, deep copy on copy.
template<class type_t>
class CCUDADeviceVector
{
 private:
  type_t *Ptr;
  size_t Size;
 public:
  CCUDADeviceVector(size_t size=0):Ptr(NULL),Size(0) {resize(size);}
  CCUDADeviceVector(const CCUDADeviceVector<type_t> &v):Ptr(NULL),Size(0) {*this=v;}
  ~CCUDADeviceVector() {release();}
  CCUDADeviceVector<type_t>& operator=(const CCUDADeviceVector<type_t> &v)
  {
   if (this==&v) return(*this);
   resize(v.Size);
   if (Size>0) B200CheckCuda(cudaMemcpyAsync(Ptr,v.Ptr,Size*sizeof(type_t),cudaMemcpyDeviceToDevice,B200TensorStream()),"device copy");
   return(*this);
  }
  void release(void)
  {
   if (Ptr!=NULL) cudaFree(Ptr);
   Ptr=NULL;
   Size=0;
  }
  void resize(size_t size)
  {
   if (size==Size) return;
   release();
   if (size==0) return;
   void *ptr=NULL;
   B200CheckCuda(cudaMalloc(&ptr,size*sizeof(type_t)),"cudaMalloc");
   Ptr=static_cast<type_t*>(ptr);
   Size=size;
  }
  void swap(CCUDADeviceVector<type_t> &v) {std::swap(Ptr,v.Ptr);std::swap(Size,v.Size);}
  type_t* get(void) const {return(Ptr);}
  size_t size(void) const {return(Size);}
};

template<class type_t>
class CTensor
{
 template<class new_type_t> friend struct STensorKernel;
 template<class new_type_t> friend class CTensorMath;
 template<class new_type_t> friend class CTensorConv;
 template<class new_type_t> friend class CTensorApplyFunc;
 template<class new_type_t> friend class CTensorTest;
 template<class new_type_t> friend class CB200LayerPort;
 private:
  mutable uint32_t Size_X;
  mutable uint32_t Size_Y;
  mutable uint32_t Size_Z;
  mutable uint32_t Size_W;
  mutable uint32_t BasedSize_X;
  mutable uint32_t BasedSize_Y;
  mutable uint32_t BasedSize_Z;
  mutable uint32_t BasedSize_W;
  mutable std::vector<type_t> Item;                 // host copy
  mutable CCUDADeviceVector<type_t> DeviceItem;     // device copy
  mutable bool HostOnChange;                        // the host copy is newer
  mutable bool DeviceOnChange;                      // the device copy is newer
 public:
  CTensor(uint32_t size_w=1,uint32_t size_z=1,uint32_t size_y=1,uint32_t size_x=1);
  CTensor(const CTensor<type_t> &cTensor);
  ~CTensor() {}
 public:
  uint32_t GetSizeX(void) const {return(Size_X);}
  uint32_t GetSizeY(void) const {return(Size_Y);}
  uint32_t GetSizeZ(void) const {return(Size_Z);}
  uint32_t GetSizeW(void) const {return(Size_W);}
  type_t GetElement(uint32_t w,uint32_t z,uint32_t y,uint32_t x) const;
  void SetElement(uint32_t w,uint32_t z,uint32_t y,uint32_t x,type_t value);
  type_t* GetColumnPtr(uint32_t w,uint32_t z,uint32_t y);
  const type_t* GetColumnPtr(uint32_t w,uint32_t z,uint32_t y) const;
  CCUDADeviceVector<type_t>& GetDeviceVector(void) const {return(DeviceItem);}
  void Unitary(void);
  void Zero(void);
  void Fill(type_t value);
  void Move(CTensor<type_t> &cTensor);
  void CopyItem(CTensor<type_t> &cTensor);
  void CopyItemToHost(type_t *item_array,uint32_t size);
  void CopyItemToDevice(type_t *item_array,uint32_t size);
  void CopyItemLayerWToHost(uint32_t w,type_t *item_array,uint32_t size);
  void CopyItemLayerWToDevice(uint32_t w,type_t *item_array,uint32_t size);
  CTensor<type_t>& operator=(const CTensor<type_t> &cTensor);

  friend CTensor<type_t> operator+<type_t>(const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right);
  friend CTensor<type_t> operator-<type_t>(const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right);
  friend CTensor<type_t> operator*<type_t>(const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right);
  friend CTensor<type_t> operator*<type_t>(const CTensor<type_t> &cTensor_Left,const type_t &value_right);
  friend CTensor<type_t> operator*<type_t>(const type_t &value_left,const CTensor<type_t> &cTensor_Right);

  bool Save(IDataStream *iDataStream_Ptr);
  bool Load(IDataStream *iDataStream_Ptr,bool check_size=false);

  void ExchangeSizeXY(void) const {std::swap(Size_X,Size_Y);}
  void ReinterpretSize(uint32_t size_w,uint32_t size_z,uint32_t size_y,uint32_t size_x) const;
  void RestoreSize(void) const;

  void Normalize(void);
  type_t GetNorma(uint32_t w,uint32_t z) const;

  void CopyToDevice(bool force=false) const;
  void CopyFromDevice(bool force=false) const;
  void SetDeviceOnChange(void) const {DeviceOnChange=true;HostOnChange=false;}
  void SetHostOnChange(void) const {HostOnChange=true;DeviceOnChange=false;}

  void Print(const std::string &name,bool print_value=true) const;
  void PrintToFile(const std::string &file_name,const std::string &name,bool print_value=true) const;
  bool Compare(const CTensor<type_t> &cTensor_Control,const std::string &name="",bool print_value=true) const;
 private:
  size_t Count(void) const {return(static_cast<size_t>(Size_X)*Size_Y*Size_Z*Size_W);}
  size_t Offset(uint32_t w,uint32_t z,uint32_t y,uint32_t x) const {return(((static_cast<size_t>(w)*Size_Z+z)*Size_Y+y)*Size_X+x);}
  // device pointer with the device copy made current (what the tensor-math classes hand to the C ABI)
  type_t* DeviceRead(void) const {CopyToDevice();return(DeviceItem.get());}
  type_t* DeviceWrite(void) const {return(DeviceItem.get());}
  void PrintLine(FILE *file,const char *text) const;
};

//----------------------------------------------------------------------------------------------------
// construction, copies
//----------------------------------------------------------------------------------------------------
template<class type_t>
CTensor<type_t>::CTensor(uint32_t size_w,uint32_t size_z,uint32_t size_y,uint32_t size_x)
{
 Size_X=BasedSize_X=size_x;
 Size_Y=BasedSize_Y=size_y;
 Size_Z=BasedSize_Z=size_z;
 Size_W=BasedSize_W=size_w;
 Item.resize(Count());
 DeviceItem.resize(Count());
 HostOnChange=true;
 DeviceOnChange=false;
}

template<class type_t>
CTensor<type_t>::CTensor(const CTensor<type_t> &cTensor)
{
 HostOnChange=true;
 DeviceOnChange=false;
 *this=cTensor;
}

// Deep copy (host vector and, when it holds the newer data, the device buffer: a device-to-device copy
// as in cuda/ccudadevicevector.cu.h:92-100); the interpretation of the size is copied as well.
template<class type_t>
CTensor<type_t>& CTensor<type_t>::operator=(const CTensor<type_t> &cTensor)
{
 if (this==&cTensor) return(*this);
 Size_X=cTensor.Size_X;Size_Y=cTensor.Size_Y;Size_Z=cTensor.Size_Z;Size_W=cTensor.Size_W;
 BasedSize_X=cTensor.BasedSize_X;BasedSize_Y=cTensor.BasedSize_Y;BasedSize_Z=cTensor.BasedSize_Z;BasedSize_W=cTensor.BasedSize_W;
 if (cTensor.DeviceOnChange==true)
 {
  Item.resize(cTensor.Item.size());
  DeviceItem=cTensor.DeviceItem;
  SetDeviceOnChange();
 }
 else
 {
  Item=cTensor.Item;
  DeviceItem.resize(Item.size());
  SetHostOnChange();
 }
 return(*this);
}

template<class type_t>
void CTensor<type_t>::Move(CTensor<type_t> &cTensor)
{
 if (this==&cTensor) return;
 std::swap(Size_X,cTensor.Size_X);std::swap(Size_Y,cTensor.Size_Y);std::swap(Size_Z,cTensor.Size_Z);std::swap(Size_W,cTensor.Size_W);
 std::swap(BasedSize_X,cTensor.BasedSize_X);std::swap(BasedSize_Y,cTensor.BasedSize_Y);
 std::swap(BasedSize_Z,cTensor.BasedSize_Z);std::swap(BasedSize_W,cTensor.BasedSize_W);
 std::swap(Item,cTensor.Item);
 DeviceItem.swap(cTensor.DeviceItem);
 std::swap(HostOnChange,cTensor.HostOnChange);
 std::swap(DeviceOnChange,cTensor.DeviceOnChange);
}

//----------------------------------------------------------------------------------------------------
// coherence between the host vector and the device buffer
//----------------------------------------------------------------------------------------------------
template<class type_t>
void CTensor<type_t>::CopyToDevice(bool force) const
{
 if (HostOnChange==false && force==false) return;
 if (DeviceItem.size()!=Item.size()) DeviceItem.resize(Item.size());
 if (Item.size()>0) B200CheckCuda(cudaMemcpyAsync(DeviceItem.get(),&Item[0],Item.size()*sizeof(type_t),cudaMemcpyHostToDevice,B200TensorStream()),"copy to device");
 // the host vector is pageable: the copy has been staged when the call returns, later host writes are safe
 HostOnChange=false;
 DeviceOnChange=false;
}

template<class type_t>
void CTensor<type_t>::CopyFromDevice(bool force) const
{
 if (DeviceOnChange==false && force==false) return;
 if (Item.size()!=DeviceItem.size()) Item.resize(DeviceItem.size());
 if (Item.size()>0)
 {
  B200CheckCuda(cudaMemcpyAsync(&Item[0],DeviceItem.get(),Item.size()*sizeof(type_t),cudaMemcpyDeviceToHost,B200TensorStream()),"copy from device");
  // a host read is the point where the reference synchronises and checks for errors; so does this
  B200Check(b200_stream_status(B200TensorStream()));
 }
 HostOnChange=false;
 DeviceOnChange=false;
}

//----------------------------------------------------------------------------------------------------
// element access
//----------------------------------------------------------------------------------------------------
template<class type_t>
type_t CTensor<type_t>::GetElement(uint32_t w,uint32_t z,uint32_t y,uint32_t x) const
{
 if (x>=Size_X || y>=Size_Y || z>=Size_Z || w>=Size_W) throw("CTensor::GetElement: index out of range.");
 CopyFromDevice();
 return(Item[Offset(w,z,y,x)]);
}

template<class type_t>
void CTensor<type_t>::SetElement(uint32_t w,uint32_t z,uint32_t y,uint32_t x,type_t value)
{
 if (x>=Size_X || y>=Size_Y || z>=Size_Z || w>=Size_W) throw("CTensor::SetElement: index out of range.");
 CopyFromDevice();
 Item[Offset(w,z,y,x)]=value;
 SetHostOnChange();
}

template<class type_t>
type_t* CTensor<type_t>::GetColumnPtr(uint32_t w,uint32_t z,uint32_t y)
{
 if (y>=Size_Y || z>=Size_Z || w>=Size_W) throw("CTensor::GetColumnPtr: index out of range.");
 CopyFromDevice();
 SetHostOnChange();
 return(&Item[Offset(w,z,y,0)]);
}

template<class type_t>
const type_t* CTensor<type_t>::GetColumnPtr(uint32_t w,uint32_t z,uint32_t y) const
{
 if (y>=Size_Y || z>=Size_Z || w>=Size_W) throw("CTensor::GetColumnPtr: index out of range.");
 CopyFromDevice();
 return(&Item[Offset(w,z,y,0)]);
}

template<class type_t>
void CTensor<type_t>::Unitary(void)
{
 for(uint32_t w=0;w<Size_W;w++)
  for(uint32_t z=0;z<Size_Z;z++)
   for(uint32_t y=0;y<Size_Y;y++)
    for(uint32_t x=0;x<Size_X;x++) Item[Offset(w,z,y,x)]=(x==y)?static_cast<type_t>(1):static_cast<type_t>(0);
 SetHostOnChange();
}

template<class type_t>
void CTensor<type_t>::Zero(void)
{
 std::fill(Item.begin(),Item.end(),type_t());
 SetHostOnChange();
}

template<class type_t>
void CTensor<type_t>::Fill(type_t value)
{
 std::fill(Item.begin(),Item.end(),value);
 SetHostOnChange();
}

template<class type_t>
void CTensor<type_t>::CopyItem(CTensor<type_t> &cTensor)
{
 if (Count()!=cTensor.Count()) throw("CTensor::CopyItem: the element counts differ.");
 if (cTensor.DeviceOnChange==true)
 {
  if (Count()>0) B200CheckCuda(cudaMemcpyAsync(DeviceItem.get(),cTensor.DeviceItem.get(),Count()*sizeof(type_t),cudaMemcpyDeviceToDevice,B200TensorStream()),"device copy");
  SetDeviceOnChange();
  return;
 }
 Item=cTensor.Item;
 SetHostOnChange();
}

template<class type_t>
void CTensor<type_t>::CopyItemToHost(type_t *item_array,uint32_t size)
{
 if (Item.size()<size) throw("CTensor::CopyItemToHost: the array is larger than the tensor.");
 CopyFromDevice();
 memcpy(&Item[0],item_array,size*sizeof(type_t));
 SetHostOnChange();
}

template<class type_t>
void CTensor<type_t>::CopyItemToDevice(type_t *item_array,uint32_t size)
{
 CopyItemLayerWToDevice(0,item_array,size);
}

template<class type_t>
void CTensor<type_t>::CopyItemLayerWToHost(uint32_t w,type_t *item_array,uint32_t size)
{
 const size_t offset=static_cast<size_t>(w)*Size_X*Size_Y*Size_Z;
 if (Item.size()<size+offset) throw("CTensor::CopyItemLayerWToHost: the array is larger than the tensor.");
 CopyFromDevice();
 memcpy(&Item[offset],item_array,size*sizeof(type_t));
 SetHostOnChange();
}

template<class type_t>
void CTensor<type_t>::CopyItemLayerWToDevice(uint32_t w,type_t *item_array,uint32_t size)
{
 const size_t offset=static_cast<size_t>(w)*Size_X*Size_Y*Size_Z;
 if (Item.size()<size+offset) throw("CTensor::CopyItemLayerWToDevice: the array is larger than the tensor.");
 CopyToDevice();
 B200CheckCuda(cudaMemcpyAsync(DeviceItem.get()+offset,item_array,size*sizeof(type_t),cudaMemcpyHostToDevice,B200TensorStream()),"copy to device");
 SetDeviceOnChange();
}

template<class type_t>
void CTensor<type_t>::ReinterpretSize(uint32_t size_w,uint32_t size_z,uint32_t size_y,uint32_t size_x) const
{
 if (Count()!=static_cast<size_t>(size_x)*size_y*size_z*size_w) throw("CTensor::ReinterpretSize: the element counts differ.");
 Size_X=size_x;Size_Y=size_y;Size_Z=size_z;Size_W=size_w;
}

template<class type_t>
void CTensor<type_t>::RestoreSize(void) const
{
 Size_X=BasedSize_X;Size_Y=BasedSize_Y;Size_Z=BasedSize_Z;Size_W=BasedSize_W;
}

template<class type_t>
type_t CTensor<type_t>::GetNorma(uint32_t w,uint32_t z) const
{
 CopyFromDevice();
 type_t norma=0;
 for(uint32_t y=0;y<Size_Y;y++)
  for(uint32_t x=0;x<Size_X;x++) {type_t v=Item[Offset(w,z,y,x)];norma+=v*v;}
 return(static_cast<type_t>(sqrt(norma)));
}

template<class type_t>
void CTensor<type_t>::Normalize(void)
{
 CopyFromDevice();
 for(uint32_t w=0;w<Size_W;w++)
  for(uint32_t z=0;z<Size_Z;z++)
  {
   type_t norma=GetNorma(w,z);
   if (norma<static_cast<type_t>(1e-5)) continue;
   for(uint32_t y=0;y<Size_Y;y++)
    for(uint32_t x=0;x<Size_X;x++) Item[Offset(w,z,y,x)]/=norma;
  }
 SetHostOnChange();
}

//----------------------------------------------------------------------------------------------------
// file format (cuda/ctensor.cu.h:525-571): four uint32 sizes W,Z,Y,X, then every element as a double
//----------------------------------------------------------------------------------------------------
#ifdef B200_HAVE_IDATASTREAM
template<class type_t>
bool CTensor<type_t>::Save(IDataStream *iDataStream_Ptr)
{
 CopyFromDevice();
 iDataStream_Ptr->SaveUInt32(Size_W);
 iDataStream_Ptr->SaveUInt32(Size_Z);
 iDataStream_Ptr->SaveUInt32(Size_Y);
 iDataStream_Ptr->SaveUInt32(Size_X);
 for(size_t n=0;n<Count();n++) iDataStream_Ptr->SaveDouble(static_cast<double>(Item[n]));
 return(true);
}

template<class type_t>
bool CTensor<type_t>::Load(IDataStream *iDataStream_Ptr,bool check_size)
{
 uint32_t w=iDataStream_Ptr->LoadUInt32();
 uint32_t z=iDataStream_Ptr->LoadUInt32();
 uint32_t y=iDataStream_Ptr->LoadUInt32();
 uint32_t x=iDataStream_Ptr->LoadUInt32();
 if (check_size==true && (w!=Size_W || z!=Size_Z || y!=Size_Y || x!=Size_X)) throw("CTensor::Load: the stored tensor has a different size.");
 Size_W=w;Size_Z=z;Size_Y=y;Size_X=x;
 Item.assign(Count(),type_t());
 DeviceItem.resize(Item.size());
 for(size_t n=0;n<Count();n++) Item[n]=static_cast<type_t>(iDataStream_Ptr->LoadDouble());
 SetHostOnChange();
 return(true);
}
#endif

//----------------------------------------------------------------------------------------------------
// printing and comparison
//----------------------------------------------------------------------------------------------------
template<class type_t>
void CTensor<type_t>::PrintLine(FILE *file,const char *text) const
{
#ifdef B200_HAVE_SYSTEM
 if (file==NULL) {SYSTEM::PutMessageToConsole(text);return;}
#endif
 fprintf(file==NULL?stdout:file,"%s\n",text);
}

template<class type_t>
void CTensor<type_t>::Print(const std::string &name,bool print_value) const
{
 PrintToFile("",name,print_value);
}

template<class type_t>
void CTensor<type_t>::PrintToFile(const std::string &file_name,const std::string &name,bool print_value) const
{
 FILE *file=NULL;
 if (file_name.length()>0) file=fopen(file_name.c_str(),"ab");
 CopyFromDevice();
 char str[256];
 PrintLine(file,name.c_str());
 snprintf(str,sizeof(str),"W:%u Z:%u Y:%u X:%u",Size_W,Size_Z,Size_Y,Size_X);
 PrintLine(file,str);
 if (print_value==true)
 {
  for(uint32_t w=0;w<Size_W;w++)
   for(uint32_t z=0;z<Size_Z;z++)
   {
    snprintf(str,sizeof(str),"-----(W:%u Z:%u)-----",w,z);
    PrintLine(file,str);
    for(uint32_t y=0;y<Size_Y;y++)
    {
     std::string line;
     for(uint32_t x=0;x<Size_X;x++)
     {
      snprintf(str,sizeof(str),"%g\t",static_cast<double>(Item[Offset(w,z,y,x)]));
      line+=str;
     }
     PrintLine(file,line.c_str());
    }
   }
 }
 if (file!=NULL) fclose(file);
}

// equal within an absolute 1e-5, the reference's CTENSOR_EPS (cuda/ctensor.cu.h:787,812)
template<class type_t>
bool CTensor<type_t>::Compare(const CTensor<type_t> &cTensor_Control,const std::string &name,bool print_value) const
{
 if (Size_X!=cTensor_Control.Size_X || Size_Y!=cTensor_Control.Size_Y || Size_Z!=cTensor_Control.Size_Z || Size_W!=cTensor_Control.Size_W) return(false);
 CopyFromDevice();
 cTensor_Control.CopyFromDevice();
 bool ret=true;
 char str[256];
 for(size_t n=0;n<Count();n++)
 {
  double a=static_cast<double>(Item[n]);
  double b=static_cast<double>(cTensor_Control.Item[n]);
  if (fabs(a-b)>1e-5)
  {
   ret=false;
   if (print_value==true)
   {
    snprintf(str,sizeof(str),"%s element %lu: %g != %g",name.c_str(),static_cast<unsigned long>(n),a,b);
    PrintLine(NULL,str);
   }
  }
 }
 return(ret);
}

//----------------------------------------------------------------------------------------------------
// operators (cuda/ctensormath.cu.h:417-462): the result takes its W from the right operand; computed by CTensorMath
//----------------------------------------------------------------------------------------------------
template<class type_t>
CTensor<type_t> operator+(const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right)
{
 CTensor<type_t> cTensor(cTensor_Right.Size_W,cTensor_Left.Size_Z,cTensor_Left.Size_Y,cTensor_Left.Size_X);
 CTensorMath<type_t>::Add(cTensor,cTensor_Left,cTensor_Right);
 return(cTensor);
}

template<class type_t>
CTensor<type_t> operator-(const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right)
{
 CTensor<type_t> cTensor(cTensor_Right.Size_W,cTensor_Left.Size_Z,cTensor_Left.Size_Y,cTensor_Left.Size_X);
 CTensorMath<type_t>::Sub(cTensor,cTensor_Left,cTensor_Right);
 return(cTensor);
}

template<class type_t>
CTensor<type_t> operator*(const CTensor<type_t> &cTensor_Left,const CTensor<type_t> &cTensor_Right)
{
 CTensor<type_t> cTensor(cTensor_Right.Size_W,cTensor_Left.Size_Z,cTensor_Left.Size_Y,cTensor_Right.Size_X);
 CTensorMath<type_t>::Mul(cTensor,cTensor_Left,cTensor_Right);
 return(cTensor);
}

template<class type_t>
CTensor<type_t> operator*(const CTensor<type_t> &cTensor_Left,const type_t &value_right)
{
 CTensor<type_t> cTensor(cTensor_Left.Size_W,cTensor_Left.Size_Z,cTensor_Left.Size_Y,cTensor_Left.Size_X);
 CTensorMath<type_t>::Mul(cTensor,cTensor_Left,value_right);
 return(cTensor);
}

template<class type_t>
CTensor<type_t> operator*(const type_t &value_left,const CTensor<type_t> &cTensor_Right)
{
 CTensor<type_t> cTensor(cTensor_Right.Size_W,cTensor_Right.Size_Z,cTensor_Right.Size_Y,cTensor_Right.Size_X);
 CTensorMath<type_t>::Mul(cTensor,value_left,cTensor_Right);
 return(cTensor);
}

#endif
