// Microbenchmark: softmax inner loop of the prefill kernel in isolation: per warp, per 128x128 tile: TMEM load of 128 scores per row, row max,
// exp2, bf16 pack, TMEM store of P. One or two warps per SM sub-partition.
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o softmax_rate softmax_rate.cu ; run: ./softmax_rate
#include <cstdio>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "../csrc/ptx_sm100.cuh"
using namespace wb200;
__device__ __forceinline__ float fmax3(float a, float b, float c) { float d; asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }
__device__ __forceinline__ float ex2_approx(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) { unsigned long long r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void unpack2(unsigned long long v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) { unsigned long long d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) { unsigned long long d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
// 2^x on the FMA pipe (x <= 0 here): Cody-Waite split x = n + f, degree-3 polynomial for 2^f on [-0.5, 0.5], exponent add.
__device__ __forceinline__ float ex2_poly3(float x) {
  x = fmaxf(x, -126.0f);
  const float shifted = x + 12582912.0f;
  const float f = x - (shifted - 12582912.0f);
  float p = fmaf(0.05550357f, f, 0.24022652f);
  p = fmaf(p, f, 0.69314718f);
  p = fmaf(p, f, 1.0f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(shifted) << 23));
}
// phases: bit0 ld, bit1 max, bit2 exp+pack, bit3 st
template <int kVariant>
__global__ void __launch_bounds__(256, 1) softmax_bench(int iters, int phases, float scale, long long *out, float *sink) {
  __shared__ uint32_t slot;
  __shared__ uint64_t bar;
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&slot), 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tm = slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = warp >> 2, quarter = warp & 3;
  const uint32_t s_addr = tm + (static_cast<uint32_t>(quarter * 32) << 16) + t * 256;
  // fill S with something score-like
  {
    uint32_t r[32];
    for (int c = 0; c < 4; ++c) {
      for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(0.01f * ((lane * 131 + c * 32 + i * 7) % 97) - 0.5f);
      tmem_st_32x32(s_addr + c * 32, r);
    }
    tmem_wait_st();
  }
  __syncthreads();
  float m_ref = 0.5f, l_run = 0.f;
  long long t0 = clock64();
  for (int it = 0; it < iters; ++it) {
    uint32_t r[128];
    if (phases & 1) {
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32 * c]));
      tmem_wait_ld();
    } else {
#pragma unroll
      for (int i = 0; i < 128; ++i) r[i] = __float_as_uint(0.01f * i + l_run * 1e-30f);
    }
    float raw_max = 0.4f;
    if (phases & 2) {
      float mx[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) mx[a] = fmax3(__uint_as_float(r[32 * a]), __uint_as_float(r[32 * a + 1]), __uint_as_float(r[32 * a + 2]));
#pragma unroll
      for (int i = 3; i + 1 < 32; i += 2) {
#pragma unroll
        for (int a = 0; a < 4; ++a) mx[a] = fmax3(mx[a], __uint_as_float(r[32 * a + i]), __uint_as_float(r[32 * a + i + 1]));
      }
#pragma unroll
      for (int a = 0; a < 4; ++a) mx[a] = fmaxf(mx[a], __uint_as_float(r[32 * a + 31]));
      raw_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
    }
    m_ref = fmaxf(m_ref, raw_max * scale);
    const float m_exp = m_ref;
    if (phases & 4) {
      if constexpr (kVariant == 0) {
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float x0 = fmaf(__uint_as_float(r[32 * c + i]), scale, -m_exp);
            const float x1 = fmaf(__uint_as_float(r[32 * c + i + 1]), scale, -m_exp);
            const float e0 = ex2_approx(x0), e1 = ex2_approx(x1);
            sum[(i >> 1) & 3] += e0 + e1;
            __nv_bfloat162 v = __floats2bfloat162_rn(e0, e1);
            packed[i >> 1] = *reinterpret_cast<uint32_t *>(&v);
          }
          if (phases & 8) {
            tmem_st_32x16(s_addr + c * 16, packed);
            if (c & 1) { tmem_wait_st(); tc_fence_before(); }
          } else {
            uint32_t x = 0;
#pragma unroll
            for (int i = 0; i < 16; ++i) x ^= packed[i];
            l_run += __uint_as_float(x & 0x3f800000u);
          }
        }
        l_run += (sum[0] + sum[1]) + (sum[2] + sum[3]);
      } else {
        // packed f32x2 arithmetic for the scaling and the sums; kVariant 2, 3: every 4th / every 2nd pair on the FMA pipe
        const unsigned long long scale2 = pack2(scale, scale), neg_m2 = pack2(-m_exp, -m_exp);
        unsigned long long sum2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const unsigned long long x2 = fma2(pack2(__uint_as_float(r[32 * c + i]), __uint_as_float(r[32 * c + i + 1])), scale2, neg_m2);
            float x0, x1;
            unpack2(x2, x0, x1);
            const bool poly = (kVariant == 2 && ((i >> 1) & 3) == 3) || (kVariant == 3 && ((i >> 1) & 1) == 1) || (kVariant == 4 && ((i >> 1) & 3) != 0);
            const float e0 = poly ? ex2_poly3(x0) : ex2_approx(x0);
            const float e1 = poly ? ex2_poly3(x1) : ex2_approx(x1);
            sum2[(i >> 1) & 3] = add2(sum2[(i >> 1) & 3], pack2(e0, e1));
            __nv_bfloat162 v = __floats2bfloat162_rn(e0, e1);
            packed[i >> 1] = *reinterpret_cast<uint32_t *>(&v);
          }
          if (phases & 8) {
            tmem_st_32x16(s_addr + c * 16, packed);
            if (c & 1) { tmem_wait_st(); tc_fence_before(); }
          } else {
            uint32_t x = 0;
#pragma unroll
            for (int i = 0; i < 16; ++i) x ^= packed[i];
            l_run += __uint_as_float(x & 0x3f800000u);
          }
        }
        float a0, a1, b0, b1, c0, c1, d0, d1;
        unpack2(sum2[0], a0, a1); unpack2(sum2[1], b0, b1); unpack2(sum2[2], c0, c1); unpack2(sum2[3], d0, d1);
        l_run += ((a0 + a1) + (b0 + b1)) + ((c0 + c1) + (d0 + d1));
      }
    } else {
      float x = 0.f;
#pragma unroll
      for (int i = 0; i < 128; ++i) x += __uint_as_float(r[i]);
      l_run += x;
    }
  }
  long long t1 = clock64();
  if (blockIdx.x == 0 && lane == 0) out[warp] = t1 - t0;
  sink[blockIdx.x * blockDim.x + threadIdx.x] = l_run + m_ref;
  tc_fence_before(); __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tm, 512); }
}
template <int kVariant>
void run(long long *d, float *sink) {
  const int iters = 200;
  for (int threads : {128, 256})
    for (int phases : {15, 1, 3, 4, 12, 7}) {
      cudaMemset(d, 0, 64);
      softmax_bench<kVariant><<<148, threads>>>(iters, phases, 0.1275f, d, sink);
      cudaError_t e = cudaDeviceSynchronize();
      long long h[8]; cudaMemcpy(h, d, 64, cudaMemcpyDeviceToHost);
      printf("variant %d warps/SMSP %d phases %2d (ld%d max%d exp%d st%d): %.0f clk/tile (warp0) %.0f (warp%d) (%s)\n", kVariant, threads / 128, phases, phases & 1, (phases >> 1) & 1, (phases >> 2) & 1, (phases >> 3) & 1,
             h[0] / double(iters), h[threads / 32 - 1] / double(iters), threads / 32 - 1, cudaGetErrorString(e));
    }
}
int main() {
  long long *d; cudaMalloc(&d, 64);
  float *sink; cudaMalloc(&sink, 148 * 256 * 4);
  run<0>(d, sink); run<1>(d, sink); run<2>(d, sink); run<3>(d, sink); run<4>(d, sink);
  return 0;
}
