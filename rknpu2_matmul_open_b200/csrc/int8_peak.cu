// int8_peak.cu -- measures the dense int8 tensor peak of the GPU it runs on: every SM issues
// back-to-back tcgen05.mma kind::i8 (128 x N x 32) on operands that stay resident in shared /
// tensor memory, so nothing but the tensor pipe is exercised.  The figure is the denominator
// of the tensor-bound roofline fractions (the pool's measured-peaks file has no int8 entry).
// Usage: int8_peak [iterations]   (prints one line per operand mode and N; last line is JSON)
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include <cstdlib>
__device__ __forceinline__ uint32_t smem_u32(const void* p){return (uint32_t)__cvta_generic_to_shared(p);}
__device__ __forceinline__ uint64_t desc(uint32_t a,uint32_t lbo,uint32_t sbo){uint32_t lo=((a&0x3FFFF)>>4)|((lbo>>4)<<16);uint32_t hi=(sbo>>4)|(1u<<14);return ((uint64_t)hi<<32)|lo;}
template<int MODE> // 0: A from TMEM (TS), 1: A from smem (SS)
__global__ void __launch_bounds__(128,1) peak(int iters,int N,unsigned long long* out){
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bar; __shared__ uint32_t tm;
  int tid=threadIdx.x, warp=tid>>5;
  for(int i=tid;i<(64*1024)/4;i+=128) ((uint32_t*)smem)[i]=0x01010101u*(i&3);
  if(tid==0){asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;"::"r"(smem_u32(&bar)));asm volatile("fence.mbarrier_init.release.cluster;");}
  if(warp==0){asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;"::"r"(smem_u32(&tm)));asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");}
  asm volatile("fence.proxy.async.shared::cta;");
  asm volatile("tcgen05.fence::before_thread_sync;"); __syncthreads(); asm volatile("tcgen05.fence::after_thread_sync;");
  uint32_t base=tm;
  unsigned long long t0=0,t1=0;
  if(tid==0){
    uint32_t idesc=(2u<<4)|(1u<<7)|(1u<<10)|((uint32_t)(N>>3)<<17)|(8u<<24);
    uint64_t bd=desc(smem_u32(smem), (uint32_t)N*16, 128);
    uint64_t ad=desc(smem_u32(smem+32768), 128*16, 128);
    asm volatile("mov.u64 %0, %globaltimer;":"=l"(t0));
    for(int i=0;i<iters;++i){
      uint32_t acc=i>0;
      if(MODE==0) asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p,%4,0;\ntcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, {%5,%5,%5,%5}, p;\n}"::"r"(base),"r"(base+256+(i&3)*8),"l"(bd),"r"(idesc),"r"(acc),"r"(0u):"memory");
      else asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p,%4,0;\ntcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5,%5,%5,%5}, p;\n}"::"r"(base),"l"(ad),"l"(bd),"r"(idesc),"r"(acc),"r"(0u):"memory");
    }
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"::"r"(smem_u32(&bar)):"memory");
    uint32_t ok=0; long spins=0;
    while(!ok && spins<400000000L){asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p,[%1],0;\nselp.u32 %0,1,0,p;\n}":"=r"(ok):"r"(smem_u32(&bar)):"memory");++spins;}
    asm volatile("mov.u64 %0, %globaltimer;":"=l"(t1));
    out[blockIdx.x]=t1-t0;
  }
  asm volatile("tcgen05.fence::before_thread_sync;"); __syncthreads();
  if(warp==0){asm volatile("tcgen05.fence::after_thread_sync;");asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;"::"r"(base));}
}
int main(int argc,char**argv){
  int iters=argc>1?atoi(argv[1]):20000; int sms=148;
  unsigned long long* d; cudaMalloc(&d,sms*8); unsigned long long h[148];
  cudaFuncSetAttribute(peak<0>,cudaFuncAttributeMaxDynamicSharedMemorySize,65536);
  cudaFuncSetAttribute(peak<1>,cudaFuncAttributeMaxDynamicSharedMemorySize,65536);
  for(int mode=0;mode<2;++mode) for(int N:{256,128,64,32,16}) for(int rep=0;rep<2;++rep){
    cudaEvent_t e0,e1; cudaEventCreate(&e0);cudaEventCreate(&e1);
    cudaEventRecord(e0);
    if(mode==0) peak<0><<<sms,128,65536>>>(iters,N,d); else peak<1><<<sms,128,65536>>>(iters,N,d);
    cudaEventRecord(e1); cudaError_t e=cudaDeviceSynchronize();
    float ms; cudaEventElapsedTime(&ms,e0,e1); cudaMemcpy(h,d,sms*8,cudaMemcpyDeviceToHost);
    double ops=2.0*128*N*32*(double)iters*sms;
    unsigned long long mx=0; for(int i=0;i<sms;++i) if(h[i]>mx) mx=h[i];
    printf("mode=%s N=%d iters=%d: kernel %.3f ms -> %.1f TOPS (event), slowest CTA %.3f ms -> %.1f TOPS, err=%s\n",mode?"SS":"TS",N,iters,ms,ops/(ms*1e-3)/1e12,mx*1e-6,ops/(mx*1e-9)/1e12,cudaGetErrorString(e));
  }
  return 0;
}
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o int8_peak int8_peak.cu
