// FP32 FMA issue-rate probe for the operand patterns of the tiled kernels.
//
// Build and run (one B200, a few seconds):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o ffma_operands ffma_operands.cu && ./ffma_operands
//
// The library's roofline peak (ca_probe_ffma) is measured with packed FMAs whose
// multiplicands stay the same from one instruction to the next.  The attention
// kernels cannot do that: a score is a dot product (few accumulators, fresh
// multiplicands every instruction) and the weighted sum is an outer product
// over 4 pixels x 16 channels.  This probe times exactly those two register
// patterns, packed (fma.rn.f32x2) and scalar (fma.rn.f32), with one and two
// warps per scheduler and no memory traffic, so the measured kernels can be
// read against what the register file can actually feed.
#include <cstdio>
#include <cuda_runtime.h>
typedef unsigned long long u64;
__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c){u64 d; asm("fma.rn.f32x2 %0,%1,%2,%3;":"=l"(d):"l"(a),"l"(b),"l"(c)); return d;}
// MODE 0: S-phase only (4 chains x 8, r outer); 1: S-phase i outer; 2: PV only (32 independent); 3: S + PV like the kernel
template<int MODE> __global__ void __launch_bounds__(256) packed_kernel(int iters, float* out, long long* cyc){
  u64 q[4][8], acc[4][8], k2[8];
  for(int r=0;r<4;r++) for(int i=0;i<8;i++){ q[r][i]=0x3a8000003a800000ull+(threadIdx.x+r*8+i); acc[r][i]=0; }
  for(int i=0;i<8;i++) k2[i]=0x3f8000003f800000ull+i+threadIdx.x;
  u64 sa[4]={1,2,3,4};
  long long t0=clock64();
  #pragma unroll 1
  for(int it=0;it<iters;it++){
    #pragma unroll
    for(int i=0;i<8;i++) k2[i]+= 0x0000000100000001ull;   // new "key" each iteration (8 IADD.64 = 16 ALU)
    if(MODE==0||MODE==3){
      #pragma unroll
      for(int r=0;r<4;r++){ sa[r]=(u64)it;
        #pragma unroll
        for(int i=0;i<8;i++) sa[r]=fma2(q[r][i],k2[i],sa[r]); }
    }
    if(MODE==1){
      #pragma unroll
      for(int r=0;r<4;r++) sa[r]=(u64)it;
      #pragma unroll
      for(int i=0;i<8;i++){
        #pragma unroll
        for(int r=0;r<4;r++) sa[r]=fma2(q[r][i],k2[i],sa[r]); }
    }
    if(MODE==2||MODE==3){
      #pragma unroll
      for(int r=0;r<4;r++){
        #pragma unroll
        for(int i=0;i<8;i++) acc[r][i]=fma2(sa[r],k2[i],acc[r][i]); }
    }
    if(MODE<2){ acc[0][0]^=sa[0]^sa[1]^sa[2]^sa[3]; }
  }
  long long t1=clock64();
  float s=0; for(int r=0;r<4;r++) for(int i=0;i<8;i++) s+=(float)(acc[r][i]&0xffff);
  out[blockIdx.x*blockDim.x+threadIdx.x]=s; if(threadIdx.x==0&&blockIdx.x==0) *cyc=t1-t0;
}
template<int MODE> void run_packed(int threads, int nf){
  float* out; long long* cyc; cudaMalloc(&out,1<<20); cudaMalloc(&cyc,8); int iters=4000; long long h;
  packed_kernel<MODE><<<1,threads>>>(iters,out,cyc); cudaMemcpy(&h,cyc,8,cudaMemcpyDeviceToHost);
  printf("packed mode=%d threads=%d: %.1f cycles/iter for %d FFMA2 per warp (%d warps/sched) -> %.2f cycles per FFMA2 per scheduler\n",MODE,threads,(double)h/iters,nf,threads/128,(double)h/iters/nf/(threads/128));
  cudaFree(out); cudaFree(cyc);
}

// scalar FFMA versions of the S and PV phases: 4 queries x 16 channels
template<int MODE> __global__ void __launch_bounds__(256) scalar_kernel(int iters, float* out, long long* cyc){
  float q[4][16], acc[4][16], k2[16];
  for(int r=0;r<4;r++) for(int i=0;i<16;i++){ q[r][i]=1e-3f*(threadIdx.x+r*16+i); acc[r][i]=0; }
  for(int i=0;i<16;i++) k2[i]=1.f+i+threadIdx.x;
  float sa[4]={1,2,3,4};
  long long t0=clock64();
  #pragma unroll 1
  for(int it=0;it<iters;it++){
    #pragma unroll
    for(int i=0;i<16;i++) k2[i]=__int_as_float(__float_as_int(k2[i])+1);   // 16 ALU
    if(MODE==0||MODE==3){
      #pragma unroll
      for(int r=0;r<4;r++){ sa[r]=(float)it;
        #pragma unroll
        for(int i=0;i<16;i++) sa[r]=fmaf(q[r][i],k2[i],sa[r]); }
    }
    if(MODE==1){
      #pragma unroll
      for(int r=0;r<4;r++) sa[r]=(float)it;
      #pragma unroll
      for(int i=0;i<16;i++){
        #pragma unroll
        for(int r=0;r<4;r++) sa[r]=fmaf(q[r][i],k2[i],sa[r]); }
    }
    if(MODE==2||MODE==3){
      #pragma unroll
      for(int r=0;r<4;r++){
        #pragma unroll
        for(int i=0;i<16;i++) acc[r][i]=fmaf(sa[r],k2[i],acc[r][i]); }
    }
    if(MODE<2){ acc[0][0]+=sa[0]+sa[1]+sa[2]+sa[3]; }
  }
  long long t1=clock64();
  float s=0; for(int r=0;r<4;r++) for(int i=0;i<16;i++) s+=acc[r][i];
  out[blockIdx.x*blockDim.x+threadIdx.x]=s; if(threadIdx.x==0&&blockIdx.x==0) *cyc=t1-t0;
}
template<int MODE> void run_scalar(int threads, int nf){
  float* out; long long* cyc; cudaMalloc(&out,1<<20); cudaMalloc(&cyc,8); int iters=4000; long long h;
  scalar_kernel<MODE><<<1,threads>>>(iters,out,cyc); cudaMemcpy(&h,cyc,8,cudaMemcpyDeviceToHost);
  printf("scalar mode=%d threads=%d: %.1f cycles/iter for %d FFMA per warp (%d warps/sched) -> %.2f cycles per FFMA per scheduler\n",MODE,threads,(double)h/iters,nf,threads/128,(double)h/iters/nf/(threads/128));
  cudaFree(out); cudaFree(cyc);
}

// modes: 0 = score phase (4 chains of 8/16), 1 = same with the chains interleaved in the source,
//        2 = weighted-sum phase (32/64 independent FMAs), 3 = both, as in the forward kernel
int main() {
    for (int th : {128, 256}) {
        run_packed<0>(th, 32); run_packed<1>(th, 32); run_packed<2>(th, 32); run_packed<3>(th, 64);
        run_scalar<0>(th, 64); run_scalar<1>(th, 64); run_scalar<2>(th, 64); run_scalar<3>(th, 128);
    }
    return 0;
}
