// Microbenchmark: back-to-back tcgen05.mma (K = 16, bf16) issue and completion rate per operand mode,
// for single-CTA instructions (cta_group::1, M = 128) and for CTA pairs (cta_group::2, M = 256: each CTA of
// a two-CTA cluster holds 128 rows of A and half of the N rows of B).
// Three issue-loop forms are timed: runtime operand mode (a branch per instruction, `bench`), two issuing warps
// (`bench_dual`), and compile-time shapes with the loop walked by one lane or by the whole warp (`issue`).
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o umma_rate umma_rate.cu ; run: ./umma_rate
#include <cstdio>
#include <cuda_runtime.h>
#include "../csrc/ptx_sm100.cuh"
using namespace wb200;

template <int kGroup>
__device__ __forceinline__ void mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  if constexpr (kGroup == 1)
    asm volatile("{\n\t.reg .pred P;\n\tsetp.ne.b32 P, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, P;\n\t}" ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
  else
    asm volatile("{\n\t.reg .pred P;\n\tsetp.ne.b32 P, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, P;\n\t}" ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
template <int kGroup>
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  if constexpr (kGroup == 1)
    asm volatile("{\n\t.reg .pred P;\n\tsetp.ne.b32 P, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, P;\n\t}" ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
  else
    asm volatile("{\n\t.reg .pred P;\n\tsetp.ne.b32 P, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, P;\n\t}" ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
// mode 0: SS A K-major, B K-major (S = Q K^T); 1: TS, B MN-major (PV); 2: SS A K-major, B MN-major; 3: TS, B K-major.
// accumulators: 1 = every instruction adds into one TMEM tile; 2 = alternate between two tiles every 8 instructions.
template <int kGroup>
__global__ void __launch_bounds__(128, 1) bench(int mode, int n, int iters, int accumulators, long long *out) {
  extern __shared__ uint8_t raw[];
  uint8_t *smem = raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u);
  const uint32_t base = smem_u32(smem);
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  __shared__ int abortw;
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); abortw = 0; fence_mbar_init(); }
  if (threadIdx.x < 32) {
    if constexpr (kGroup == 1) {
      tmem_alloc(smem_u32(&slot), 512);
      tmem_relinquish();
    } else {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&slot)), "r"(512) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
  }
  fence_proxy_async_smem();
  tc_fence_before();
  if constexpr (kGroup == 2) cluster_sync_all(); else __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  const bool leader = kGroup == 1 || (cluster_cta_rank() == 0);
  if (threadIdx.x == 0 && leader) {
    const bool b_mn = (mode == 1 || mode == 2);
    const uint32_t idesc = umma_idesc_f16(128 * kGroup, n, true, false, b_mn);
    const uint64_t a_desc = umma_desc_kmajor(base);
    const uint64_t b_desc = b_mn ? umma_desc_mnmajor(base + 32768, 16384) : umma_desc_kmajor(base + 32768);
    // Two accumulators only when they fit beside the 64 columns the TMEM A operand occupies.
    const uint32_t d0 = tm + 128, d1 = (accumulators == 2 && n <= 128) ? tm + 256 : tm + 128;
    long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
      const uint32_t d = (it & 1) ? d1 : d0;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t aoff = ((ks >> 2) * 16384 + (ks & 3) * 32) >> 4;
        const uint64_t boff = b_mn ? (ks * 2048) >> 4 : aoff;
        if (mode == 1 || mode == 3) mma_ts<kGroup>(d, tm + ks * 8, b_desc + boff, idesc, 1);
        else mma_ss<kGroup>(d, a_desc + aoff, b_desc + boff, idesc, 1);
      }
    }
    long long t1 = clock64();
    if constexpr (kGroup == 1)
      umma_commit(smem_u32(&bar));
    else
      asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
    mbar_wait(smem_u32(&bar), 0, &abortw);
    long long t2 = clock64();
    if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; out[2] = abortw; }
  }
  tc_fence_before();
  if constexpr (kGroup == 2) cluster_sync_all(); else __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    if constexpr (kGroup == 1) tmem_dealloc(tm, 512);
    else asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tm), "r"(512) : "memory");
  }
}


// Two issuing threads (lane 0 of warps 0 and 1), each with its own accumulator and barrier: tells an issue limit of
// one thread apart from a limit of the tensor pipe. collector: 0 = plain; 1 = consecutive instruction pairs share the
// A operand, the first with .collector::a::fill, the second with .collector::a::lastuse (SS only).
__global__ void __launch_bounds__(128, 1) bench_dual(int ts, int n, int iters, int issuers, int collector, long long *out) {
  extern __shared__ uint8_t raw[];
  uint8_t *smem = raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u);
  const uint32_t base = smem_u32(smem);
  __shared__ uint64_t bar[2];
  __shared__ uint32_t slot;
  __shared__ int abortw;
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { mbar_init(smem_u32(&bar[0]), 1); mbar_init(smem_u32(&bar[1]), 1); abortw = 0; fence_mbar_init(); }
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&slot), 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  const int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0 && warp < issuers) {
    const uint32_t idesc = umma_idesc_f16(128, n, true, false, false);
    const uint64_t a_desc = umma_desc_kmajor(base + warp * 49152);
    const uint64_t b_desc = umma_desc_kmajor(base + warp * 49152 + 16384);
    const uint32_t d = tm + 128 + warp * 128;       // n <= 128 here
    const uint32_t a_tm = tm + warp * 64;
    long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t off = ((ks & 3) * 32) >> 4;
        if (ts) {
          mma_ts<1>(d, a_tm + ks * 8, b_desc + off, idesc, 1);
        } else if (!collector) {
          mma_ss<1>(d, a_desc + off, b_desc + off, idesc, 1);
        } else if ((ks & 1) == 0) {
          asm volatile("{\n\t.reg .pred P;\n\tsetp.ne.b32 P, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16.collector::a::fill [%0], %1, %2, %3, P;\n\t}" ::"r"(d), "l"(a_desc + off), "l"(b_desc + off), "r"(idesc), "r"(1) : "memory");
        } else {
          const uint64_t prev = (((ks - 1) & 3) * 32) >> 4;
          asm volatile("{\n\t.reg .pred P;\n\tsetp.ne.b32 P, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16.collector::a::lastuse [%0], %1, %2, %3, P;\n\t}" ::"r"(d), "l"(a_desc + prev), "l"(b_desc + off), "r"(idesc), "r"(1) : "memory");
        }
      }
    }
    long long t1 = clock64();
    umma_commit(smem_u32(&bar[warp]));
    mbar_wait(smem_u32(&bar[warp]), 0, &abortw);
    long long t2 = clock64();
    if (blockIdx.x == 0) { out[2 * warp] = t1 - t0; out[2 * warp + 1] = t2 - t0; }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tm, 512); }
}

static void run_dual(int grid, int n, int ts, int issuers, int collector, long long *d) {
  const int iters = 200;
  cudaFuncSetAttribute(bench_dual, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  cudaMemset(d, 0, 32);
  bench_dual<<<grid, 128, 100 * 1024>>>(ts, n, iters, issuers, collector, d);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[4];
  cudaMemcpy(h, d, 32, cudaMemcpyDeviceToHost);
  printf("dual: %s N=%3d grid %3d issuers %d collector %d: thread0 complete %.1f clk/MMA, thread1 complete %.1f clk/MMA (%s)\n", ts ? "TS" : "SS", n, grid,
         issuers, collector, h[1] / (iters * 8.0), h[3] / (iters * 8.0), cudaGetErrorString(e));
}


// ---- How the shape of the issuing code affects the rate: compile-time instruction shape, and who walks the loop.
// kShape 0: if (threadIdx.x == 0) { loop }   1: warp-wide loop, elect_one_sync() around each MMA   2: warp-wide loop, lane == 0 around each MMA
// 3: warp-wide loop, one elect_one_sync() per group of 8 MMAs
template <int kShape, int kTs, int kN>
__global__ void __launch_bounds__(128, 1) issue(int iters, int issuers, long long *out) {
  extern __shared__ uint8_t raw[];
  uint8_t *smem = raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u);
  const uint32_t base = smem_u32(smem);
  __shared__ uint64_t bar[4];
  __shared__ uint32_t slot;
  __shared__ int abortw;
  for (int i = threadIdx.x; i < 200 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&bar[i]), 1); abortw = 0; fence_mbar_init(); }
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&slot), 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tm = slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < issuers) {
    const uint32_t idesc = umma_idesc_f16(128, kN, true, false, false);
    const uint64_t a_desc = umma_desc_kmajor(base + warp * 98304);
    const uint64_t b_desc = umma_desc_kmajor(base + warp * 98304 + 32768);
    const uint32_t d = tm + 128 + warp * 128;
    const uint32_t a_tm = tm + warp * 64;
    long long t0 = 0, t2 = 0;
    if (kShape == 0) {
      if (lane == 0) {
        t0 = clock64();
        for (int it = 0; it < iters; ++it) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t off = ((ks >> 2) * 16384 + (ks & 3) * 32) >> 4;
            if (kTs) mma_ts<1>(d, a_tm + ks * 8, b_desc + off, idesc, 1);
            else mma_ss<1>(d, a_desc + off, b_desc + off, idesc, 1);
          }
        }
        umma_commit(smem_u32(&bar[warp]));
        mbar_wait(smem_u32(&bar[warp]), 0, &abortw);
        t2 = clock64();
      }
    } else {
      t0 = clock64();
      for (int it = 0; it < iters; ++it) {
        if (kShape == 3) {
          if (elect_one_sync()) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint64_t off = ((ks >> 2) * 16384 + (ks & 3) * 32) >> 4;
              if (kTs) mma_ts<1>(d, a_tm + ks * 8, b_desc + off, idesc, 1);
              else mma_ss<1>(d, a_desc + off, b_desc + off, idesc, 1);
            }
          }
          __syncwarp();
        } else {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t off = ((ks >> 2) * 16384 + (ks & 3) * 32) >> 4;
            const bool mine = kShape == 1 ? elect_one_sync() : (lane == 0);
            if (mine) {
              if (kTs) mma_ts<1>(d, a_tm + ks * 8, b_desc + off, idesc, 1);
              else mma_ss<1>(d, a_desc + off, b_desc + off, idesc, 1);
            }
          }
        }
      }
      if (elect_one_sync()) umma_commit(smem_u32(&bar[warp]));
      __syncwarp();
      mbar_wait(smem_u32(&bar[warp]), 0, &abortw);
      t2 = clock64();
    }
    if (blockIdx.x == 0 && lane == 0) { out[warp] = t2 - t0; }
  }
  tc_fence_before(); __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tm, 512); }
}
template <int kShape, int kTs, int kN>
void run_issue(long long *d) {
  const int iters = 200;
  cudaFuncSetAttribute(issue<kShape, kTs, kN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 204 * 1024);
  for (int issuers = 1; issuers <= 2; ++issuers) {
    cudaMemset(d, 0, 32);
    issue<kShape, kTs, kN><<<148, 128, 204 * 1024>>>(iters, issuers, d);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[2]; cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
    printf("shape %d %s N=%3d issuers %d: warp0 %.1f clk/MMA  warp1 %.1f clk/MMA (%s)\n", kShape, kTs ? "TS" : "SS", kN, issuers, h[0] / (iters * 8.0), h[1] / (iters * 8.0), cudaGetErrorString(e));
  }
}
template <int kShape>
void run_shape(long long *d) {
  run_issue<kShape, 0, 64>(d); run_issue<kShape, 0, 128>(d);
  run_issue<kShape, 1, 64>(d); run_issue<kShape, 1, 128>(d);
}

template <int kGroup>
static void run(int grid, int n, int mode, int accumulators, long long *d) {
  const char *names[] = {"SS  A:K  B:K ", "TS  A:tm B:MN", "SS  A:K  B:MN", "TS  A:tm B:K "};
  const int iters = 200;
  cudaFuncSetAttribute(bench<kGroup>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(128);
  config.dynamicSmemBytes = 100 * 1024;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = kGroup;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  cudaMemset(d, 0, 32);
  cudaError_t launch = cudaLaunchKernelEx(&config, bench<kGroup>, mode, n, iters, accumulators, d);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[3];
  cudaMemcpy(h, d, 24, cudaMemcpyDeviceToHost);
  printf("cta_group::%d M=%3d N=%3d grid %3d acc %d %s: issue %.1f clk/MMA, complete %.1f clk/MMA, %.0f flop/clk/SM (%s, %s, abort %lld)\n", kGroup,
         128 * kGroup, n, grid, accumulators, names[mode], h[0] / (iters * 8.0), h[1] / (iters * 8.0),
         2.0 * 128 * n * 16 / (h[1] / (iters * 8.0)), cudaGetErrorString(launch), cudaGetErrorString(e), h[2]);
}

int main(int argc, char **argv) {
  long long *d;
  cudaMalloc(&d, 32);
  for (int n : {32, 64, 128})
    for (int ts = 0; ts < 2; ++ts)
      for (int issuers = 1; issuers <= 2; ++issuers) run_dual(148, n, ts, issuers, 0, d);
  for (int n : {64, 128}) run_dual(148, n, 0, 1, 1, d);
  run_shape<0>(d); run_shape<1>(d); run_shape<2>(d); run_shape<3>(d);
  run_issue<1, 0, 256>(d); run_issue<1, 1, 256>(d); run_issue<0, 0, 256>(d); run_issue<0, 1, 256>(d);
  if (argc > 1) return 0;   // any argument: skip the table of runtime-mode issue loops below
  for (int grid : {2, 148})
    for (int n : {32, 64, 128, 256})
      for (int mode = 0; mode < 4; ++mode) {
        if (grid == 2 && (mode >= 2 || n < 128)) continue;
        run<1>(grid, n, mode, 1, d);
        if (n <= 128) run<1>(grid, n, mode, 2, d);
      }
  for (int grid : {2, 148})
    for (int n : {64, 128, 256})
      for (int mode = 0; mode < 4; ++mode) {
        if (grid == 2 && (mode >= 2 || n < 128)) continue;
        run<2>(grid, n, mode, 1, d);
        if (n <= 128) run<2>(grid, n, mode, 2, d);
      }
  return 0;
}
