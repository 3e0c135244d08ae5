// Microbenchmark: back-to-back tcgen05.mma (M=128, K=16, bf16) issue and completion rate per operand mode.
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o umma_rate umma_rate.cu ; run: ./umma_rate
#include <cstdio>
#include <cuda_runtime.h>
#include "../csrc/ptx_sm100.cuh"
using namespace wb200;
__device__ __forceinline__ void umma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred P;\n\tsetp.ne.b32 P, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, P;\n\t}" ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
// mode 0: SS A K-major, B K-major (S = Q K^T); 1: TS, B MN-major (PV); 2: SS A K-major, B MN-major; 3: TS, B K-major
__global__ void __launch_bounds__(128, 1) bench(int mode, int n, int iters, long long *out) {
  extern __shared__ uint8_t raw[];
  uint8_t *smem = raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u);
  const uint32_t base = smem_u32(smem);
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  __shared__ int abortw;
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); abortw = 0; fence_mbar_init(); }
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&slot), 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tm = slot;
  if (threadIdx.x == 0) {
    const bool b_mn = (mode == 1 || mode == 2);
    const uint32_t idesc = umma_idesc_f16(128, n, true, false, b_mn);
    const uint64_t a_desc = umma_desc_kmajor(base);
    const uint64_t b_desc = b_mn ? umma_desc_mnmajor(base + 32768, 16384) : umma_desc_kmajor(base + 32768);
    long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t aoff = ((ks >> 2) * 16384 + (ks & 3) * 32) >> 4;
        const uint64_t boff = b_mn ? (ks * 2048) >> 4 : aoff;
        if (mode == 1 || mode == 3) umma_ts(tm + 256, tm + ks * 8, b_desc + boff, idesc, 1);
        else umma_f16_ss(tm + 256, a_desc + aoff, b_desc + boff, idesc, 1);
      }
    }
    long long t1 = clock64();
    umma_commit(smem_u32(&bar));
    mbar_wait(smem_u32(&bar), 0, &abortw);
    long long t2 = clock64();
    if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
  }
  tc_fence_before(); __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tm, 512); }
}
int main() {
  long long *d; cudaMalloc(&d, 16);
  cudaFuncSetAttribute(bench, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  const char *names[] = {"SS  A:K  B:K ", "TS  A:tm B:MN", "SS  A:K  B:MN", "TS  A:tm B:K "};
  for (int grid : {1, 148}) for (int n : {128, 256}) for (int mode = 0; mode < 4; ++mode) {
    if (n == 256 && (mode == 1 || mode == 2)) {}  // B MN-major with N=256 needs 4 blocks: descriptor still valid for timing
    const int iters = 200;
    bench<<<grid, 128, 100 * 1024>>>(mode, n, iters, d);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[2]; cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
    printf("grid %3d N=%3d %s: issue %.1f clk/MMA, complete %.1f clk/MMA (%s)\n", grid, n, names[mode], h[0] / (iters * 8.0), h[1] / (iters * 8.0), cudaGetErrorString(e));
  }
  return 0;
}
