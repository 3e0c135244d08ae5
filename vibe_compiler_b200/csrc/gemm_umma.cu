// Persistent tcgen05 GEMM for sm_100a: out = epilogue(A x B) with fp32 accumulation in TMEM and a
// single round-to-nearest-even narrowing, the accumulation contract of the reference's NE GEMM
// command (lib/Wafer/Transforms/Linalg/ContractionAccumulation.cpp:147-218; finalize
// lib/Wafer/Simulator/Reference/Formal/FormalNumericGemm.cpp:115-157).
//
// Tile 128 x 256 x 64, 4-stage TMA ring, two 256-column TMEM accumulators so the epilogue of tile i
// overlaps the main loop of tile i+1. Warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner,
// warps 2-5 = epilogue (one TMEM lane quarter each). Roofline: tensor pipe; algorithmic work is
// 2*M*N*K flop per launch.
#include "kernels.h"
#include "ptx_sm100.cuh"

namespace wb200 {
namespace {

constexpr int kBM = 128, kBN = 256, kBK = 64, kStages = 4;
constexpr int kABytes = kBM * kBK * 2;        // 16 KiB
constexpr int kBBytes = kBN * kBK * 2;        // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 512;
constexpr int kThreads = 192;
constexpr int kGroupM = 8;
constexpr size_t kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct GemmUmmaParams {
  int m, n, k;
  int out_format;
  int a_mn_major, b_mn_major;
  int epilogue;
  int bf16;
  const float *bias;
  void *out;
  int *status;
  int num_m_tiles, num_n_tiles;
  int group_m;   // tile rows walked together (see tile_coords)
};

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int group_m, int &m_blk, int &n_blk) {
  const int per_group = group_m * num_n;
  const int group = tile / per_group;
  const int first_m = group * group_m;
  const int group_size = min(num_m - first_m, group_m);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % group_size;
  n_blk = in_group / group_size;
}

__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
}

// Epilogue of 32 accumulator columns [col0, col0 + 32) of output row `row`: bias / GELU / SwiGLU in f32, one
// round-to-nearest-even narrowing, 16-byte stores.
__device__ __forceinline__ void epilogue_chunk(const GemmUmmaParams &p, uint32_t (&r)[32], int row, int col0) {
  if (p.epilogue == WB200_EPI_SWIGLU) {
    // Columns (2j, 2j+1) hold (gate_j, up_j): out[row, j] = silu(gate) * up, 16 outputs per 32 columns.
    if (row < p.m && col0 + 32 <= p.n) {
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float o[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float gate = __uint_as_float(r[4 * j + 2 * h]), up = __uint_as_float(r[4 * j + 2 * h + 1]);
          o[h] = __fdividef(gate, 1.0f + __expf(-gate)) * up;
        }
        w[j] = narrow_bits(o[0], p.out_format) | (narrow_bits(o[1], p.out_format) << 16);
      }
      uint16_t *dst = reinterpret_cast<uint16_t *>(p.out) + static_cast<size_t>(row) * (p.n / 2) + col0 / 2;
      *reinterpret_cast<uint4 *>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
      *reinterpret_cast<uint4 *>(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
    }
    return;
  }
  if (p.epilogue != WB200_EPI_NONE) {
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (col0 + i + 4 <= p.n) b = __ldg(reinterpret_cast<const float4 *>(p.bias + col0 + i));
      float v0 = __uint_as_float(r[i]) + b.x, v1 = __uint_as_float(r[i + 1]) + b.y;
      float v2 = __uint_as_float(r[i + 2]) + b.z, v3 = __uint_as_float(r[i + 3]) + b.w;
      if (p.epilogue == WB200_EPI_BIAS_GELU) {
        v0 = gelu_erf(v0); v1 = gelu_erf(v1); v2 = gelu_erf(v2); v3 = gelu_erf(v3);
      }
      r[i] = __float_as_uint(v0); r[i + 1] = __float_as_uint(v1);
      r[i + 2] = __float_as_uint(v2); r[i + 3] = __float_as_uint(v3);
    }
  }
  if (row < p.m) {
    if (p.out_format == WB200_F32) {
      float *dst = reinterpret_cast<float *>(p.out) + static_cast<size_t>(row) * p.n + col0;
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        if (col0 + i + 4 <= p.n)
          *reinterpret_cast<uint4 *>(dst + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
    } else {
      uint16_t *dst = reinterpret_cast<uint16_t *>(p.out) + static_cast<size_t>(row) * p.n + col0;
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        if (col0 + i + 8 <= p.n) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t lo = narrow_bits(__uint_as_float(r[i + 2 * j]), p.out_format);
            const uint32_t hi = narrow_bits(__uint_as_float(r[i + 2 * j + 1]), p.out_format);
            w[j] = lo | (hi << 16);
          }
          *reinterpret_cast<uint4 *>(dst + i) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  }
}

template <bool kAMn, bool kBMn, bool kBf16>
__global__ void __launch_bounds__(kThreads, 1)
gemm_umma_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmUmmaParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t *smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t smem_base = smem_u32(smem);

  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kStages * kStageBytes);
  const uint32_t bar_base = smem_base + kStages * kStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bars + 2 * kStages + 4);
  volatile int *abort_word = reinterpret_cast<volatile int *>(bars + 2 * kStages + 5);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 128);
    }
    *abort_word = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  const int k_blocks = (p.k + kBK - 1) / kBK;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(tile, p.num_m_tiles, p.num_n_tiles, p.group_m, m_blk, n_blk);
        const int m0 = m_blk * kBM, n0 = n_blk * kBN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_word)) { ok = false; break; }
          mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          const uint32_t b_dst = a_dst + kABytes;
          const int k0 = kb * kBK;
          if constexpr (!kAMn) {
            tma_load_2d(a_dst, &tmap_a, full_bar(stage), k0, m0);            // box {64 k, 128 m}
          } else {
            tma_load_2d(a_dst, &tmap_a, full_bar(stage), m0, k0);            // box {64 m, 64 k}
            tma_load_2d(a_dst + 8192, &tmap_a, full_bar(stage), m0 + 64, k0);
          }
          if constexpr (kBMn) {
#pragma unroll
            for (int i = 0; i < 4; ++i)                                       // box {64 n, 64 k}
              tma_load_2d(b_dst + i * 8192, &tmap_b, full_bar(stage), n0 + 64 * i, k0);
          } else {
            tma_load_2d(b_dst, &tmap_b, full_bar(stage), k0, n0);            // box {64 k, 256 n}
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // The whole warp walks the loop (waits included) and one elected lane issues: with warp-uniform control flow the
    // descriptor arithmetic stays on the uniform datapath, which keeps the issue cost per instruction well below the
    // 128 clocks a 128 x 256 x 16 product occupies the tensor pipe (a loop run by a single diverged lane measured
    // 171 clocks per instruction, the converged form 128).
    constexpr uint32_t idesc = umma_idesc_f16(kBM, kBN, kBf16, kAMn, kBMn);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, abort_word)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * kBN;
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait(full_bar(stage), phase, abort_word)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_src = smem_base + stage * kStageBytes;
        const uint32_t b_src = a_src + kABytes;
        const uint64_t adesc = kAMn ? umma_desc_mnmajor(a_src, 8192) : umma_desc_kmajor(a_src);
        const uint64_t bdesc = kBMn ? umma_desc_mnmajor(b_src, 8192) : umma_desc_kmajor(b_src);
        if (elect_one_sync()) {
#pragma unroll
          for (int ks = 0; ks < kBK / 16; ++ks) {
            // a k-step of 16 advances the start address by 32 B in a K-major tile and by 2 KiB in an MN-major one
            constexpr uint64_t a_step = (kAMn ? 2048 : 32) >> 4, b_step = (kBMn ? 2048 : 32) >> 4;
            umma_f16_ss(d_tmem, adesc + ks * a_step, bdesc + ks * b_step, idesc, (kb | ks) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      if (elect_one_sync()) umma_commit(tmem_full_bar(acc));
      __syncwarp();
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  } else {
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      int m_blk, n_blk;
      tile_coords(tile, p.num_m_tiles, p.num_n_tiles, p.group_m, m_blk, n_blk);
      const int row = m_blk * kBM + quarter * 32 + lane;
      const int n0 = n_blk * kBN;
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, abort_word)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kBN;
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_wait_ld();
        epilogue_chunk(p, r, row, n0 + c * 32);
      }
      tc_fence_before();
      mbar_arrive(tmem_empty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  __syncthreads();
  if (*abort_word != 0) {
    // Give copies still in flight time to land before the shared memory is released.
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
    if (threadIdx.x == 0) atomicExch(p.status, *abort_word);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}


// ---------------------------------------------------------------- CTA-pair kernel: 256 x 256 x 64 tiles
// Two CTAs of a cluster share one output tile: CTA r of the pair owns rows [128 r, 128 r + 128) of it (A rows,
// accumulator lanes, epilogue) and loads half of the tile's B columns; the even CTA issues cta_group::2 instructions of
// M = 256, N = 256 that read both halves. Against the single-CTA tile that halves the B bytes each SM pulls from L2 and
// shared memory per flop, and the 32 KiB stage leaves room for six stages instead of four. Loads carry no multicast
// qualifier: every CTA fetches its own bytes.
constexpr int kPairStages = 6;
constexpr int kPairBHalf = (kBN / 2) * kBK * 2;            // 16 KiB: this CTA's 128 B columns of a k-block
constexpr int kPairStageBytes = kABytes + kPairBHalf;      // 32 KiB
constexpr size_t kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + 256;

template <bool kAMn, bool kBMn, bool kBf16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_umma_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const GemmUmmaParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t *smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t smem_base = smem_u32(smem);

  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kPairStages * kPairStageBytes);
  const uint32_t bar_base = smem_base + kPairStages * kPairStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };                              // used in the issuing CTA only
  auto empty_bar = [&](int s) { return bar_base + 8u * (kPairStages + s); };             // one per CTA
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kPairStages + a); };     // one per CTA
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kPairStages + 2 + a); };// issuing CTA: 256 arrivals
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bars + 2 * kPairStages + 4);
  volatile int *abort_word = reinterpret_cast<volatile int *>(bars + 2 * kPairStages + 5);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_cta_rank();
  const bool issuer = cta_rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 256);
    }
    *abort_word = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();     // both CTAs' barriers exist before either touches the partner's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_pair_m = (p.m + 2 * kBM - 1) / (2 * kBM);
  const int num_tiles = num_pair_m * p.num_n_tiles;
  const int k_blocks = (p.k + kBK - 1) / kBK;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters) {
        int m_blk, n_blk;
        tile_coords(tile, num_pair_m, p.num_n_tiles, p.group_m, m_blk, n_blk);
        const int m0 = m_blk * 2 * kBM + static_cast<int>(cta_rank) * kBM;         // this CTA's 128 rows
        const int n0 = n_blk * kBN + static_cast<int>(cta_rank) * (kBN / 2);       // this CTA's 128 B columns
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_word)) { ok = false; break; }
          // Both CTAs' bytes are counted on the issuing CTA's barrier, which expects the two stages together.
          const uint32_t full = cluster_map_shared(full_bar(stage), 0);
          if (issuer) mbar_arrive_expect_tx(full_bar(stage), 2 * kPairStageBytes);
          const uint32_t a_dst = smem_base + stage * kPairStageBytes;
          const uint32_t b_dst = a_dst + kABytes;
          const int k0 = kb * kBK;
          if constexpr (!kAMn) {
            tma_load_2d_pair(a_dst, &tmap_a, full, k0, m0);                   // box {64 k, 128 m}
          } else {
            tma_load_2d_pair(a_dst, &tmap_a, full, m0, k0);                   // box {64 m, 64 k}
            tma_load_2d_pair(a_dst + 8192, &tmap_a, full, m0 + 64, k0);
          }
          if constexpr (kBMn) {
            tma_load_2d_pair(b_dst, &tmap_b, full, n0, k0);                   // box {64 n, 64 k}
            tma_load_2d_pair(b_dst + 8192, &tmap_b, full, n0 + 64, k0);
          } else {
            tma_load_2d_pair(b_dst, &tmap_b, full, k0, n0);                   // box {64 k, 128 n}
          }
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (issuer) {
      // The whole warp walks the loop and one elected lane issues (warp-uniform control flow keeps the descriptor
      // arithmetic on the uniform datapath).
      constexpr uint32_t idesc = umma_idesc_f16(2 * kBM, kBN, kBf16, kAMn, kBMn);
      const uint32_t peer_bar_base = cluster_map_shared(bar_base, 1);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters) {
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, abort_word)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_word)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_src = smem_base + stage * kPairStageBytes;
          const uint32_t b_src = a_src + kABytes;
          const uint64_t adesc = kAMn ? umma_desc_mnmajor(a_src, 8192) : umma_desc_kmajor(a_src);
          const uint64_t bdesc = kBMn ? umma_desc_mnmajor(b_src, 8192) : umma_desc_kmajor(b_src);
          if (elect_one_sync()) {
#pragma unroll
            for (int ks = 0; ks < kBK / 16; ++ks) {
              constexpr uint64_t a_step = (kAMn ? 2048 : 32) >> 4, b_step = (kBMn ? 2048 : 32) >> 4;
              umma_f16_ss_pair(d_tmem, adesc + ks * a_step, bdesc + ks * b_step, idesc, (kb | ks) != 0 ? 1u : 0u);
            }
            // the stage is free in both CTAs once these instructions have read it
            umma_commit_pair(empty_bar(stage));
            umma_commit_pair(peer_bar_base + 8u * (kPairStages + stage));
          }
          __syncwarp();
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (elect_one_sync()) {
          umma_commit_pair(tmem_full_bar(acc));
          umma_commit_pair(peer_bar_base + 8u * (2 * kPairStages + acc));
        }
        __syncwarp();
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const uint32_t issuer_bar_base = cluster_map_shared(bar_base, 0);
    for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters) {
      int m_blk, n_blk;
      tile_coords(tile, num_pair_m, p.num_n_tiles, p.group_m, m_blk, n_blk);
      const int row = m_blk * 2 * kBM + static_cast<int>(cta_rank) * kBM + quarter * 32 + lane;
      const int n0 = n_blk * kBN;
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, abort_word)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kBN;
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_wait_ld();
        epilogue_chunk(p, r, row, n0 + c * 32);
      }
      tc_fence_before();
      mbar_arrive_cluster(issuer_bar_base + 8u * (2 * kPairStages + 2 + acc));   // both CTAs' epilogues free the accumulator
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
    if (threadIdx.x == 0) atomicExch(p.status, *abort_word);
  }
  cluster_sync_all();     // neither CTA leaves while the partner may still read its shared memory or signal its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace

bool gemm_umma_supports(const GemmUmmaArgs &a) {
  if (a.in_format != WB200_BF16 && a.in_format != WB200_F16) return false;
  if (a.out_format != WB200_BF16 && a.out_format != WB200_F16 && a.out_format != WB200_F32) return false;
  if (a.m <= 0 || a.n <= 0 || a.k <= 0) return false;
  // TMA needs 16-byte row pitches; the epilogue stores 16-byte vectors.
  if (a.k % 8 != 0 || a.n % 8 != 0 || a.m % 8 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(a.a) | reinterpret_cast<uintptr_t>(a.b) |
       reinterpret_cast<uintptr_t>(a.out)) & 15u)
    return false;
  if ((a.epilogue == WB200_EPI_BIAS || a.epilogue == WB200_EPI_BIAS_GELU) &&
      (a.bias == nullptr || (reinterpret_cast<uintptr_t>(a.bias) & 15u)))
    return false;
  if (a.epilogue == WB200_EPI_SWIGLU && (a.n % 32 != 0 || a.out_format == WB200_F32)) return false;
  return true;
}

namespace {
using GemmKernel = void (*)(const CUtensorMap, const CUtensorMap, const GemmUmmaParams);
const GemmKernel kernels[8] = {
    gemm_umma_kernel<false, false, false>, gemm_umma_kernel<false, false, true>, gemm_umma_kernel<false, true, false>,
    gemm_umma_kernel<false, true, true>,   gemm_umma_kernel<true, false, false>, gemm_umma_kernel<true, false, true>,
    gemm_umma_kernel<true, true, false>,   gemm_umma_kernel<true, true, true>};
const GemmKernel pair_kernels[8] = {
    gemm_umma_pair_kernel<false, false, false>, gemm_umma_pair_kernel<false, false, true>, gemm_umma_pair_kernel<false, true, false>,
    gemm_umma_pair_kernel<false, true, true>,   gemm_umma_pair_kernel<true, false, false>, gemm_umma_pair_kernel<true, false, true>,
    gemm_umma_pair_kernel<true, true, false>,   gemm_umma_pair_kernel<true, true, true>};
}  // namespace

wb200_status gemm_umma_prepare() {
  static PerDeviceOnce attributes;
  return attributes.run([]() -> wb200_status {
    for (GemmKernel kernel : kernels)
      WB200_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes)));
    for (GemmKernel kernel : pair_kernels)
      WB200_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kPairSmemBytes)));
    return WB200_OK;
  });
}

wb200_status launch_gemm_umma(const GemmUmmaArgs &a, int sm_count, int *device_status,
                              cudaStream_t stream) {
  if (!gemm_umma_supports(a)) return fail(WB200_ERR_UNSUPPORTED, "GEMM outside the tcgen05 kernel's domain");
  // CTA pairs when the problem has at least one full 256 x 256 tile per pair of SMs to amortise the pairing; the
  // single-CTA kernel otherwise (small or narrow problems, WB200_GEMM_PAIR=0).
  static const bool pair_enabled = []() { const char *env = getenv("WB200_GEMM_PAIR"); return !(env && env[0] == '0'); }();
  const int pair_tiles = ((a.m + 2 * kBM - 1) / (2 * kBM)) * ((a.n + kBN - 1) / kBN);
  const bool use_pairs = pair_enabled && a.m >= 2 * kBM && a.n >= kBN && pair_tiles * 4 >= sm_count;
  CUtensorMap tmap_a, tmap_b;
  wb200_status st;
  if (!a.lhs_transposed)  // A[m,k], k contiguous: K-major
    st = encode_tmap_2d(&tmap_a, a.a, a.in_format, a.k, a.m, static_cast<uint64_t>(a.k) * 2, 64, kBM);
  else                    // A[k,m], m contiguous: MN-major
    st = encode_tmap_2d(&tmap_a, a.a, a.in_format, a.m, a.k, static_cast<uint64_t>(a.m) * 2, 64, 64);
  if (st != WB200_OK) return st;
  if (!a.rhs_transposed)  // B[k,n], n contiguous: MN-major
    st = encode_tmap_2d(&tmap_b, a.b, a.in_format, a.n, a.k, static_cast<uint64_t>(a.n) * 2, 64, 64);
  else                    // B[n,k], k contiguous: K-major
    st = encode_tmap_2d(&tmap_b, a.b, a.in_format, a.k, a.n, static_cast<uint64_t>(a.k) * 2, 64, use_pairs ? kBN / 2 : kBN);
  if (st != WB200_OK) return st;

  GemmUmmaParams p;
  p.m = a.m; p.n = a.n; p.k = a.k;
  p.out_format = a.out_format;
  p.a_mn_major = a.lhs_transposed ? 1 : 0;
  p.b_mn_major = a.rhs_transposed ? 0 : 1;
  p.epilogue = a.epilogue;
  p.bf16 = a.in_format == WB200_BF16;
  p.bias = a.bias;
  p.out = a.out;
  p.status = device_status;
  p.num_m_tiles = (a.m + kBM - 1) / kBM;
  p.num_n_tiles = (a.n + kBN - 1) / kBN;
  static const int group_override = []() { const char *env = getenv("WB200_GEMM_GROUP_M"); return env ? atoi(env) : 0; }();
  p.group_m = group_override > 0 ? group_override : kGroupM;

  wb200_status st_attributes = gemm_umma_prepare();
  if (st_attributes != WB200_OK) return st_attributes;
  const int variant = (p.a_mn_major ? 4 : 0) | (p.b_mn_major ? 2 : 0) | (p.bf16 ? 1 : 0);
  if (use_pairs) {
    int clusters = sm_count / 2;
    if (pair_tiles < clusters) clusters = pair_tiles;
    pair_kernels[variant]<<<2 * clusters, kThreads, kPairSmemBytes, stream>>>(tmap_a, tmap_b, p);
    WB200_CUDA_CHECK(cudaGetLastError());
    return WB200_OK;
  }
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  const int grid = tiles < sm_count ? tiles : sm_count;
  kernels[variant]<<<grid, kThreads, kSmemBytes, stream>>>(tmap_a, tmap_b, p);
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

}  // namespace wb200
