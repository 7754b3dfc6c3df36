// NVLink microbenchmark (2 GPUs, one process): what a kernel can pull from / push to a peer,
// for several load and store flavours, unrolls and grids, next to cudaMemcpyPeer. It gives the
// link-rate denominator for the allreduce kernels' roofline.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o p2p_microbench bench/p2p_microbench.cu
//   ./p2p_microbench
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <vector>
#define CK(x) do{cudaError_t e=(x); if(e!=cudaSuccess){printf("ERR %s line %d: %s\n",#x,__LINE__,cudaGetErrorString(e)); exit(1);} }while(0)

__device__ __forceinline__ uint4 ld_weak(const void* p){ return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint4 ld_relaxed_sys(const void* p){ uint4 v; asm volatile("ld.relaxed.sys.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];":"=r"(v.x),"=r"(v.y),"=r"(v.z),"=r"(v.w):"l"(p):"memory"); return v; }
__device__ __forceinline__ uint4 ld_nc(const void* p){ uint4 v; asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];":"=r"(v.x),"=r"(v.y),"=r"(v.z),"=r"(v.w):"l"(p)); return v; }
__device__ __forceinline__ uint4 ld_volatile(const void* p){ uint4 v; asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];":"=r"(v.x),"=r"(v.y),"=r"(v.z),"=r"(v.w):"l"(p):"memory"); return v; }
__device__ __forceinline__ void st_weak(void* p, uint4 v){ *reinterpret_cast<uint4*>(p)=v; }
__device__ __forceinline__ void st_relaxed_sys(void* p, uint4 v){ asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};"::"l"(p),"r"(v.x),"r"(v.y),"r"(v.z),"r"(v.w):"memory"); }

template<int LD, int U>
__global__ void __launch_bounds__(512) k_read(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n){
  size_t stride=(size_t)gridDim.x*blockDim.x; size_t i0=(size_t)blockIdx.x*blockDim.x+threadIdx.x;
  for(size_t i=i0;i<n;i+=stride*U){ uint4 v[U];
#pragma unroll
    for(int u=0;u<U;u++){ size_t j=i+u*stride; if(j<n){ if(LD==0) v[u]=ld_weak(src+j); else if(LD==1) v[u]=ld_relaxed_sys(src+j); else if(LD==2) v[u]=ld_nc(src+j); else v[u]=ld_volatile(src+j);} }
#pragma unroll
    for(int u=0;u<U;u++){ size_t j=i+u*stride; if(j<n) st_weak(dst+j, v[u]); }
  }
}
template<int ST, int U>
__global__ void __launch_bounds__(512) k_write(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n){
  size_t stride=(size_t)gridDim.x*blockDim.x; size_t i0=(size_t)blockIdx.x*blockDim.x+threadIdx.x;
  for(size_t i=i0;i<n;i+=stride*U){ uint4 v[U];
#pragma unroll
    for(int u=0;u<U;u++){ size_t j=i+u*stride; if(j<n) v[u]=ld_weak(src+j); }
#pragma unroll
    for(int u=0;u<U;u++){ size_t j=i+u*stride; if(j<n){ if(ST==0) st_weak(dst+j,v[u]); else st_relaxed_sys(dst+j,v[u]); } }
  }
}
// both: read remote src_r + local src_l, add, write to local dst_l and remote dst_r (like 2-rank two-shot)
template<int LD, int ST, int U>
__global__ void __launch_bounds__(512) k_both(const uint4* src_l, const uint4* src_r, uint4* dst_l, uint4* dst_r, size_t n){
  size_t stride=(size_t)gridDim.x*blockDim.x; size_t i0=(size_t)blockIdx.x*blockDim.x+threadIdx.x;
  for(size_t i=i0;i<n;i+=stride*U){ uint4 a[U], b[U];
#pragma unroll
    for(int u=0;u<U;u++){ size_t j=i+u*stride; if(j<n){ if(LD==0){a[u]=ld_weak(src_l+j); b[u]=ld_weak(src_r+j);} else {a[u]=ld_relaxed_sys(src_l+j); b[u]=ld_relaxed_sys(src_r+j);} } }
#pragma unroll
    for(int u=0;u<U;u++){ size_t j=i+u*stride; if(j<n){ uint4 r; r.x=a[u].x+b[u].x; r.y=a[u].y+b[u].y; r.z=a[u].z+b[u].z; r.w=a[u].w+b[u].w;
      if(ST==0){ st_weak(dst_l+j,r); st_weak(dst_r+j,r);} else { st_relaxed_sys(dst_l+j,r); st_relaxed_sys(dst_r+j,r);} } }
  }
}

template<typename F> float timeit(F f, cudaStream_t s0, cudaStream_t s1, int iters){
  cudaEvent_t a,b; CK(cudaSetDevice(0)); CK(cudaEventCreate(&a)); CK(cudaEventCreate(&b));
  for(int i=0;i<2;i++) f();
  CK(cudaSetDevice(0)); CK(cudaStreamSynchronize(s0)); if(s1){CK(cudaSetDevice(1)); CK(cudaStreamSynchronize(s1));}
  CK(cudaSetDevice(0)); CK(cudaEventRecord(a,s0));
  for(int i=0;i<iters;i++) f();
  CK(cudaSetDevice(0)); CK(cudaEventRecord(b,s0)); CK(cudaEventSynchronize(b));
  if(s1){CK(cudaSetDevice(1)); CK(cudaStreamSynchronize(s1));}
  float ms; CK(cudaEventElapsedTime(&ms,a,b)); return ms/iters;
}

int main(int argc,char**argv){
  size_t bytes=(size_t)256<<20; size_t n=bytes/16;
  int nd; CK(cudaGetDeviceCount(&nd)); if(nd<2){printf("need 2 gpus\n"); return 0;}
  uint4 *a0,*b0,*a1,*b1;
  CK(cudaSetDevice(0)); CK(cudaDeviceEnablePeerAccess(1,0)); CK(cudaMalloc(&a0,bytes)); CK(cudaMalloc(&b0,bytes)); CK(cudaMemset(a0,1,bytes)); CK(cudaMemset(b0,0,bytes));
  CK(cudaSetDevice(1)); CK(cudaDeviceEnablePeerAccess(0,0)); CK(cudaMalloc(&a1,bytes)); CK(cudaMalloc(&b1,bytes)); CK(cudaMemset(a1,2,bytes)); CK(cudaMemset(b1,0,bytes));
  cudaStream_t s0,s1; CK(cudaSetDevice(0)); CK(cudaStreamCreate(&s0)); CK(cudaSetDevice(1)); CK(cudaStreamCreate(&s1));
  CK(cudaSetDevice(0));
  float ms=timeit([&]{ CK(cudaMemcpyPeerAsync(b1,1,a0,0,bytes,s0)); }, s0,nullptr,10);
  printf("memcpyPeer 0->1           : %.1f GB/s\n", bytes/ms/1e6);
  ms=timeit([&]{ CK(cudaSetDevice(0)); CK(cudaMemcpyPeerAsync(b1,1,a0,0,bytes,s0)); CK(cudaSetDevice(1)); CK(cudaMemcpyPeerAsync(b0,0,a1,1,bytes,s1)); }, s0,s1,10);
  printf("memcpyPeer bidirectional  : %.1f GB/s per direction\n", bytes/ms/1e6);
  int blocks_list[]={32,64,128,148,296};
  for(int blocks: blocks_list){
#define RD(LD,U,name) ms=timeit([&]{ k_read<LD,U><<<blocks,512,0,s0>>>(a1,b0,n); }, s0,nullptr,10); printf("read  %-14s U=%d blocks=%3d : %.1f GB/s\n",name,U,blocks,bytes/ms/1e6);
    RD(0,4,"weak") RD(0,8,"weak") RD(1,4,"relaxed.sys") RD(1,8,"relaxed.sys") RD(2,8,"nc") RD(3,8,"volatile")
#define WR(ST,U,name) ms=timeit([&]{ k_write<ST,U><<<blocks,512,0,s0>>>(a0,b1,n); }, s0,nullptr,10); printf("write %-14s U=%d blocks=%3d : %.1f GB/s\n",name,U,blocks,bytes/ms/1e6);
    WR(0,4,"weak") WR(1,4,"relaxed.sys") WR(0,8,"weak")
    // both directions by both GPUs at once (each GPU: half the data like two-shot)
#define BOTH(LD,ST,U,name) ms=timeit([&]{ CK(cudaSetDevice(0)); k_both<LD,ST,U><<<blocks,512,0,s0>>>(a0,a1,b0,b1,n/2); CK(cudaSetDevice(1)); k_both<LD,ST,U><<<blocks,512,0,s1>>>(a1+n/2,a0+n/2,b1+n/2,b0+n/2,n/2); }, s0,s1,10); printf("two-shot-like %-20s U=%d blocks=%3d : %.3f ms  busbw(=N/t) %.1f GB/s\n",name,U,blocks,ms,bytes/ms/1e6);
    BOTH(0,0,4,"weak/weak") BOTH(1,1,4,"relaxed.sys/relaxed.sys") BOTH(0,0,8,"weak/weak") BOTH(1,0,4,"relaxed.sys/weak")
  }
  // read-only from both sides simultaneously and write-only from both sides
  for(int blocks: {64,148}){
    ms=timeit([&]{ CK(cudaSetDevice(0)); k_read<0,8><<<blocks,512,0,s0>>>(a1,b0,n); CK(cudaSetDevice(1)); k_read<0,8><<<blocks,512,0,s1>>>(a0,b1,n); }, s0,s1,10);
    printf("read both sides weak U=8 blocks=%d: %.1f GB/s per direction\n",blocks,bytes/ms/1e6);
    ms=timeit([&]{ CK(cudaSetDevice(0)); k_write<0,8><<<blocks,512,0,s0>>>(a0,b1,n); CK(cudaSetDevice(1)); k_write<0,8><<<blocks,512,0,s1>>>(a1,b0,n); }, s0,s1,10);
    printf("write both sides weak U=8 blocks=%d: %.1f GB/s per direction\n",blocks,bytes/ms/1e6);
  }
  return 0;
}
