// bulk_copy_bw.cu -- how fast can cp.async.bulk stream DRAM into shared memory?  One thread per CTA
// keeps a ring of stages in flight over its own contiguous slice of a 4 GB buffer (nothing reads the
// data).  The table it prints (CTAs per SM, stage size, stages, requests per stage) is the ceiling any
// weight-streaming kernel built on bulk copies can reach, and shows the request rate one thread sustains.
// Usage: bulk_copy_bw        (about 4 GB of device memory, a few milliseconds of kernels)
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include <cstdlib>
__device__ __forceinline__ uint32_t s32(const void* p){return (uint32_t)__cvta_generic_to_shared(p);}
__global__ void __launch_bounds__(128) stream(const uint8_t* src, size_t bytes_per_cta, int stage_bytes, int nstages, int pieces, unsigned long long* sink){
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bar = (uint64_t*)(smem + (size_t)nstages*stage_bytes);
  if(threadIdx.x==0){
    for(int s=0;s<nstages;++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;"::"r"(s32(&bar[s])));
    asm volatile("fence.mbarrier_init.release.cluster;");
    const uint8_t* base = src + (size_t)blockIdx.x*bytes_per_cta;
    long n = bytes_per_cta/stage_bytes; int piece=stage_bytes/pieces;
    auto issue=[&](long i,int s){
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"::"r"(s32(&bar[s])),"r"(stage_bytes):"memory");
      for(int q=0;q<pieces;++q)
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"::"r"(s32(smem+(size_t)s*stage_bytes+q*piece)),"l"(base+(size_t)i*stage_bytes+q*piece),"r"(piece),"r"(s32(&bar[s])):"memory");
    };
    long issued=0; for(;issued<nstages&&issued<n;++issued) issue(issued,(int)issued);
    for(long i=0;i<n;++i){
      int s=(int)(i%nstages); uint32_t par=(uint32_t)((i/nstages)&1); uint32_t ok=0; long spins=0;
      while(!ok && spins<100000000L){asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p,[%1],%2,%3;\nselp.u32 %0,1,0,p;\n}":"=r"(ok):"r"(s32(&bar[s])),"r"(par),"r"(1000u):"memory");++spins;}
      if(issued<n){issue(issued,s);++issued;}
    }
    sink[blockIdx.x]=smem[0];
  }
}
int main(){
  size_t total=(size_t)4<<30; uint8_t* d; cudaMalloc(&d,total); cudaMemset(d,1,total); unsigned long long* sink; cudaMalloc(&sink,8*2048);
  cudaFuncSetAttribute(stream,cudaFuncAttributeMaxDynamicSharedMemorySize,220*1024);
  int cfgs[][4]={{1,16384,12,1},{1,16384,12,4},{1,32768,6,1},{1,8192,24,1},{1,4096,48,1},{2,16384,6,1},{4,16384,3,1},{2,8192,12,1},{4,8192,6,1},{1,16384,4,1},{1,16384,8,1},{1,65536,3,1}};
  for(auto& c:cfgs){
    int per_sm=c[0],sb=c[1],ns=c[2],pieces=c[3]; int ctas=148*per_sm; size_t per=(total/ctas)/sb*sb; size_t smem=(size_t)sb*ns+ns*8+64;
    for(int rep=0;rep<2;++rep){
      cudaEvent_t e0,e1; cudaEventCreate(&e0);cudaEventCreate(&e1); cudaEventRecord(e0);
      stream<<<ctas,128,smem>>>(d,per,sb,ns,pieces,sink);
      cudaEventRecord(e1); cudaError_t e=cudaDeviceSynchronize(); float ms; cudaEventElapsedTime(&ms,e0,e1);
      if(rep) printf("ctas/SM=%d stage=%d B stages=%d pieces=%d in-flight/SM=%d KB: %.3f ms -> %.0f GB/s (%s)\n",per_sm,sb,ns,pieces,per_sm*sb*ns/1024,ms,(double)per*ctas/ms/1e6,cudaGetErrorString(e));
    }
  }
  return 0;
}
