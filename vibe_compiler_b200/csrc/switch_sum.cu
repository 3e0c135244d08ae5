// Sum over the shards of a tensor-parallel region (the two sums of the decoder layer) as ONE kernel per GPU that uses
// the NVSwitch for the arithmetic: every rank's buffer lies at the same offset of a symmetric allocation that is also
// bound to an NVLink multicast object. Rank r owns the r-th slice of the buffer: it reads the slice through the multicast
// address with multimem.ld_reduce (the switch fetches the slice from every GPU, adds the values with an f32 accumulator
// and returns one sum), and writes the sum back through the multicast address with multimem.st (the switch stores it
// into every GPU's buffer). Each GPU therefore sends and receives the buffer about once, at the link's full rate, where
// a ring passes it 2 (G - 1) / G times with G - 1 latency steps; and every rank ends with bit-identical sums, because
// each element is added once, by its owner's request.
//
// The reference realises such a sum as a Tile collective (lib/Wafer/Transforms/Tile/DistributedCollectiveMovement.cpp:
// 675-735: reduce-scatter followed by all-gather over the participating dies); this is the same decomposition with the
// switch doing both halves.
//
// Protocol. Signals are 32-bit words in peer-mapped memory: every rank has [2][world] of them (enter / exit, by source
// rank), zero-initialised. A device-side epoch advances by one per launch, the same on every rank; its successor is
// the tag written to the signals, so no word ever needs resetting. Enter: block 0 publishes "my partial sums are
// complete" to every rank (system-scope fence, then the tag), every block waits until all ranks' enter words in its own
// memory carry the tag. Exit: every thread fences its multimem stores, the last block to finish publishes the exit tag
// to every rank, waits for all ranks' exit words, and advances the epoch: when the kernel ends on a GPU, every slice of
// its buffer has landed. All waits are bounded (about a second); a wait that runs out sets the backend's status word
// and the kernel carries on to its end, so a missing peer costs a second and an error, never a hung GPU.
// One sequence of launches per signal area: sums that may run concurrently need areas of their own.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "backend.h"
#include "kernels.h"

namespace wb200 {
namespace {

constexpr int kSwitchThreads = 512;
constexpr int kSwitchUnroll = 8;            // 16-byte requests in flight per thread
constexpr long long kSwitchWaitCycles = 2000000000LL;
// The kernel is launched as pairs of blocks (clusters of two) that each ask for more than half of an SM's shared memory:
// a pair then takes both SMs of a TPC and nothing else shares them. Beside persistent compute kernels that are launched
// as CTA pairs themselves and leave whole TPCs free, the sum neither waits for an SM nor breaks up a TPC that a compute
// pair needs (a pair that finds no whole TPC waits for the end of the kernel's first wave).
constexpr int kSwitchSmemBytes = 120 * 1024;

struct SwitchSumParams {
  uint8_t *multicast;                        // multicast address of the buffer
  uint8_t *multicast_out;                    // multicast address the sums are stored to (the buffer itself: in place)
  const uint8_t *residual;                   // optional: this rank's copy of a tensor added to the sums before the store
  uint64_t chunks;                           // 16-byte chunks in the buffer
  int format;
  int rank, world;
  unsigned int *signals[kMaxSwitchRanks];    // every rank's signal words, [rank] = this rank's own
  unsigned int *epoch;                       // this rank's {epoch, finished blocks}
  int *status;
};

__device__ __forceinline__ void signal_store(unsigned int *address, unsigned int value) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(address), "r"(value) : "memory");
}
__device__ __forceinline__ unsigned int signal_load(const unsigned int *address) {
  unsigned int value;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
  return value;
}
// Bounded wait until `*word == tag`; false when it ran out.
__device__ __forceinline__ bool signal_wait(const unsigned int *word, unsigned int tag) {
  const long long start = clock64();
  unsigned int polls = 0;
  while (signal_load(word) != tag) {
    if ((++polls & 63u) == 0u && clock64() - start > kSwitchWaitCycles) return false;
  }
  return true;
}

template <int kFormat>
__device__ __forceinline__ uint4 switch_load_sum(const uint8_t *address) {
  uint4 v;
  if constexpr (kFormat == WB200_BF16)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(address) : "memory");
  else if constexpr (kFormat == WB200_F16)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(address) : "memory");
  else
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(address) : "memory");
  return v;
}
// sums + residual, element by element: widened to f32, added, rounded once to the storage format (the arithmetic of the
// layer's residual add kernel, so fusing the add into the sum changes no bit).
template <int kFormat>
__device__ __forceinline__ uint4 add_residual(const uint4 &sums, const uint4 &residual) {
  const uint32_t a[4] = {sums.x, sums.y, sums.z, sums.w}, b[4] = {residual.x, residual.y, residual.z, residual.w};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (kFormat == WB200_F32) {
      o[i] = __float_as_uint(__uint_as_float(a[i]) + __uint_as_float(b[i]));
    } else if constexpr (kFormat == WB200_BF16) {
      const float lo = __uint_as_float(a[i] << 16) + __uint_as_float(b[i] << 16);
      const float hi = __uint_as_float(a[i] & 0xffff0000u) + __uint_as_float(b[i] & 0xffff0000u);
      const __nv_bfloat162 packed = __floats2bfloat162_rn(lo, hi);
      o[i] = *reinterpret_cast<const uint32_t *>(&packed);
    } else {
      const float2 fa = __half22float2(*reinterpret_cast<const __half2 *>(&a[i])), fb = __half22float2(*reinterpret_cast<const __half2 *>(&b[i]));
      const __half2 packed = __floats2half2_rn(fa.x + fb.x, fa.y + fb.y);
      o[i] = *reinterpret_cast<const uint32_t *>(&packed);
    }
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}
__device__ __forceinline__ void switch_store(uint8_t *address, const uint4 &v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(address), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w) : "memory");
}

template <int kFormat>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kSwitchThreads) switch_sum_kernel(const SwitchSumParams p) {
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int *>(p.epoch);
  const unsigned int tag = epoch + 1u;
  unsigned int *own = p.signals[p.rank];
  // ---- enter: this rank's partial sums (written by earlier kernels of the stream) are published to every rank
  if (blockIdx.x == 0 && threadIdx.x < p.world) {
    __threadfence_system();
    signal_store(p.signals[threadIdx.x] + p.rank, tag);
  }
  if (threadIdx.x < p.world && !signal_wait(own + threadIdx.x, tag)) atomicExch(p.status, 3);
  __syncthreads();

  // ---- this rank's slice: switch-side sum, then switch-side broadcast
  const uint64_t per_rank = (p.chunks + p.world - 1) / p.world;
  const uint64_t begin = per_rank * p.rank;
  const uint64_t end = begin + per_rank < p.chunks ? begin + per_rank : p.chunks;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kSwitchThreads;
  for (uint64_t base = begin + static_cast<uint64_t>(blockIdx.x) * kSwitchThreads + threadIdx.x; base < end; base += stride * kSwitchUnroll) {
    uint4 sums[kSwitchUnroll], rest[kSwitchUnroll];
#pragma unroll
    for (int u = 0; u < kSwitchUnroll; ++u) {   // all requests of the round are in flight together, the residual's too
      const uint64_t chunk = base + u * stride;
      if (chunk < end) {
        sums[u] = switch_load_sum<kFormat>(p.multicast + chunk * 16);
        if (p.residual) rest[u] = __ldcs(reinterpret_cast<const uint4 *>(p.residual + chunk * 16));
      }
    }
#pragma unroll
    for (int u = 0; u < kSwitchUnroll; ++u) {
      const uint64_t chunk = base + u * stride;
      if (chunk < end) {
        if (p.residual) sums[u] = add_residual<kFormat>(sums[u], rest[u]);
        switch_store(p.multicast_out + chunk * 16, sums[u]);
      }
    }
  }

  // ---- exit: the last block of this rank tells every rank that its slice has been stored, and waits for theirs
  __threadfence_system();
  __syncthreads();
  __shared__ bool last_block;
  if (threadIdx.x == 0) last_block = atomicAdd(p.epoch + 1, 1u) == gridDim.x - 1u;
  __syncthreads();
  if (!last_block) return;
  if (threadIdx.x < p.world) {
    __threadfence_system();
    signal_store(p.signals[threadIdx.x] + p.world + p.rank, tag);
    if (!signal_wait(own + p.world + threadIdx.x, tag)) atomicExch(p.status, 3);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    p.epoch[1] = 0u;
    __threadfence();
    *reinterpret_cast<volatile unsigned int *>(p.epoch) = tag;
  }
}

}  // namespace

wb200_status launch_switch_sum(void *multicast, uint64_t elements, int format, int rank, int world, void *const *signals,
                               unsigned int *epoch, int blocks, int *device_status, cudaStream_t stream, void *multicast_out,
                               const void *residual) {
  if (world < 2 || world > kMaxSwitchRanks || rank < 0 || rank >= world)
    return fail(WB200_ERR_INVALID_ARGUMENT, "the switch sum takes 2 to 16 ranks and a rank inside the world");
  const uint64_t bytes = elements * (format == WB200_F32 ? 4u : 2u);
  if (format != WB200_BF16 && format != WB200_F16 && format != WB200_F32)
    return fail(WB200_ERR_UNSUPPORTED, "the switch sum takes bf16, f16 or f32 values");
  if ((reinterpret_cast<uintptr_t>(multicast) & 15u) || (bytes & 15u) || bytes == 0)
    return fail(WB200_ERR_INVALID_ARGUMENT, "the switch sum takes a 16-byte aligned buffer whose size is a positive multiple of 16 bytes");
  SwitchSumParams p;
  if ((reinterpret_cast<uintptr_t>(multicast_out) & 15u) || (reinterpret_cast<uintptr_t>(residual) & 15u))
    return fail(WB200_ERR_INVALID_ARGUMENT, "the switch sum's output and residual must be 16-byte aligned");
  p.multicast = static_cast<uint8_t *>(multicast);
  p.multicast_out = multicast_out ? static_cast<uint8_t *>(multicast_out) : p.multicast;
  p.residual = static_cast<const uint8_t *>(residual);
  p.chunks = bytes / 16;
  p.format = format;
  p.rank = rank; p.world = world;
  for (int r = 0; r < kMaxSwitchRanks; ++r) p.signals[r] = r < world ? static_cast<unsigned int *>(signals[r]) : nullptr;
  p.epoch = epoch;
  p.status = device_status;
  // No more blocks than the slice has rounds of work for.
  const uint64_t per_rank = (p.chunks + world - 1) / world;
  const uint64_t useful = (per_rank + kSwitchThreads * kSwitchUnroll - 1) / (kSwitchThreads * kSwitchUnroll);
  if (static_cast<uint64_t>(blocks) > useful) blocks = static_cast<int>(useful);
  blocks = blocks < 2 ? 2 : blocks - blocks % 2;      // whole pairs
  static PerDeviceOnce attributes;
  const wb200_status attribute_status = attributes.run([]() -> wb200_status {
    WB200_CUDA_CHECK(cudaFuncSetAttribute(switch_sum_kernel<WB200_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSwitchSmemBytes));
    WB200_CUDA_CHECK(cudaFuncSetAttribute(switch_sum_kernel<WB200_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSwitchSmemBytes));
    WB200_CUDA_CHECK(cudaFuncSetAttribute(switch_sum_kernel<WB200_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSwitchSmemBytes));
    return WB200_OK;
  });
  if (attribute_status != WB200_OK) return attribute_status;
  if (format == WB200_BF16) switch_sum_kernel<WB200_BF16><<<blocks, kSwitchThreads, kSwitchSmemBytes, stream>>>(p);
  else if (format == WB200_F16) switch_sum_kernel<WB200_F16><<<blocks, kSwitchThreads, kSwitchSmemBytes, stream>>>(p);
  else switch_sum_kernel<WB200_F32><<<blocks, kSwitchThreads, kSwitchSmemBytes, stream>>>(p);
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

}  // namespace wb200

extern "C" uint64_t wb200_switch_sum_signal_bytes(uint32_t world) { return static_cast<uint64_t>(2) * world * sizeof(uint32_t); }

extern "C" wb200_status wb200_switch_sum(wb200_backend *backend, const wb200_switch_sum_params *x) {
  using namespace wb200;
  if (!backend || !x || !x->multicast || !x->epoch) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  if (x->world < 2 || x->world > WB200_MAX_EXCHANGE_RANKS || x->rank >= x->world)
    return fail(WB200_ERR_INVALID_ARGUMENT, "the switch sum takes 2 to 16 ranks and a rank inside the world");
  for (uint32_t r = 0; r < x->world; ++r)
    if (!x->signals[r] || (reinterpret_cast<uintptr_t>(x->signals[r]) & 3u))
      return fail(WB200_ERR_INVALID_ARGUMENT, "every rank's signal words must be given");
  DeviceGuard guard(backend->device);
  const int blocks = x->blocks ? static_cast<int>(x->blocks) : 32;
  wb200_status st = launch_switch_sum(x->multicast, x->elements, static_cast<int>(x->format), static_cast<int>(x->rank),
                                      static_cast<int>(x->world), x->signals, x->epoch, blocks, backend->d_status,
                                      static_cast<cudaStream_t>(x->stream), x->multicast_out, x->residual);
  if (st == WB200_OK) backend->launches += 1;
  return st;
}
