// Flash-decoding (split-KV attention for query length 1, grouped queries) for sm_100a.
//
// Arithmetic follows the reference's online-attention materialisation:
//   per KV tile   lib/Wafer/Transforms/Linalg/OnlineAttentionDecomposition.cpp:568-594
//   state merge   lib/Wafer/Transforms/Linalg/OnlineAttentionMaterialization.cpp:264-373
//   finalize      lib/Wafer/Transforms/Linalg/OnlineAttentionMaterialization.cpp:196-262
//   fold order    lib/Wafer/Transforms/Linalg/SpatialRegionMaterialization.cpp:2420-2433 (ascending)
// exp is the target's ExpLp, exp2(x * log2e) in f32
// (lib/Wafer/Simulator/Reference/ManagedReferenceTargetModel.cpp:265-270).
//
// Stage 1 (fd_partial_kernel): one CTA per (split, kv head, batch). Each of the 4 warps streams its
// own contiguous quarter of the CTA's KV interval through a private 3-deep cp.async ring of 16-row
// tiles (128-bit coalesced copies, XOR-swizzled rows), computes S = Q K^T and acc += P V with
// mma.sync m16n8k16 on the group's query heads (rows padded to 16) and carries (m, l, acc) in
// registers. Warps then left-fold their states in ascending KV order through shared memory and the
// CTA writes one (acc[D], m, l) record. Stage 2 (fd_combine_kernel) left-folds the records of all
// splits in ascending order and finalizes. The kernel is HBM-bound: algorithmic bytes per launch
// are the K and V bytes of the visible keys, read exactly once.
#include "kernels.h"

namespace wb200 {
namespace {

constexpr int kD = 128;            // head dimension
constexpr int kTileRows = 16;      // KV rows per warp tile
constexpr int kWarps = 4;
constexpr int kStagesFd = 3;
constexpr int kTileBytes = kTileRows * kD * 2;  // 4 KiB for K, same for V
constexpr int kRecord = kD + 2;    // acc[D], m, l
constexpr int kQBytes = 16 * kD * 2;
constexpr int kFdSmemBytes = kWarps * kStagesFd * 2 * kTileBytes + kQBytes;

__device__ __forceinline__ float exp_lp(float x) { return exp2f(x * 0x1.715476p+0f); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
template <bool kBf16>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (kBf16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
        "{%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
        "{%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}
template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kBf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
  }
}

struct FdParams {
  int batch, q_heads, kv_heads, group;
  int kv_len;         // rows physically present per (batch, kv head)
  int kv_visible;     // keys [0, kv_visible) are visible
  int splits, rows_per_split, rows_per_warp;
  float scale;
  const uint16_t *q, *k, *v;
  float *partials;    // [batch, q_heads, splits, kRecord]
};

// Tail of the sequence-sharded decode step, run by the last CTA of a (batch, kv head) to finish stage 1 (see
// fd_exchange_rows): the exchange buffers of all ranks and this rank's epoch words.
constexpr int kMaxExchangeRanks = 16;
struct FdTailParams {
  int rank, world;
  float *peer[kMaxExchangeRanks];    // exchange buffers of all ranks, [rank] = this rank's own
  unsigned int *epoch;               // this rank's {epoch, finished rows}, zero-initialised
  unsigned int *arrivals;            // [batch * kv_heads] finished stage-1 CTAs, zero-initialised, reset by the last one
  int out_format, zero_fully_masked;
  void *out;
  float *lse, *row_max, *row_sum;
  int *status;
};
template <int kRowsAtOnce>
__device__ void fd_exchange_rows(const FdTailParams &x, const float *records, int splits, int first_row, int row_count, int rows_total);

// Swizzled byte offset of 16-byte chunk `c` of row `r` inside a 16 x 256-byte tile.
__device__ __forceinline__ uint32_t tile_offset(int r, int c) {
  return static_cast<uint32_t>(r * 256 + ((c ^ (r & 7)) << 4));
}

template <bool kBf16, bool kTail>
__global__ void __launch_bounds__(kWarps * 32, 2) fd_partial_kernel(const FdParams p, const FdTailParams tail) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  uint8_t *q_smem = smem + kWarps * kStagesFd * 2 * kTileBytes;
  // Stage the group's query rows, zero-padded to 16 rows.
  {
    const uint16_t *q_src = p.q + (static_cast<size_t>(b) * p.q_heads + static_cast<size_t>(hk) * p.group) * kD;
    for (int i = threadIdx.x; i < 16 * kD / 8; i += blockDim.x) {
      const int row = i / (kD / 8), chunk = i % (kD / 8);
      uint4 value = make_uint4(0, 0, 0, 0);
      if (row < p.group) value = *reinterpret_cast<const uint4 *>(q_src + row * kD + chunk * 8);
      *reinterpret_cast<uint4 *>(q_smem + row * (kD * 2) + chunk * 16) = value;
    }
  }
  __syncthreads();
  uint32_t q_frag[kD / 16][4];
#pragma unroll
  for (int ks = 0; ks < kD / 16; ++ks) {
    const uint32_t *row_lo = reinterpret_cast<const uint32_t *>(q_smem + g * (kD * 2));
    const uint32_t *row_hi = reinterpret_cast<const uint32_t *>(q_smem + (g + 8) * (kD * 2));
    q_frag[ks][0] = row_lo[ks * 8 + t];
    q_frag[ks][1] = row_hi[ks * 8 + t];
    q_frag[ks][2] = row_lo[ks * 8 + 4 + t];
    q_frag[ks][3] = row_hi[ks * 8 + 4 + t];
  }

  // This warp's KV interval.
  const int split_begin = split * p.rows_per_split;
  const int warp_begin = split_begin + warp * p.rows_per_warp;
  int warp_end = warp_begin + p.rows_per_warp;
  if (warp_end > p.kv_visible) warp_end = p.kv_visible;
  const int tiles = warp_end > warp_begin ? (warp_end - warp_begin + kTileRows - 1) / kTileRows : 0;

  const size_t head_offset = (static_cast<size_t>(b) * p.kv_heads + hk) * static_cast<size_t>(p.kv_len) * kD;
  const uint16_t *k_base = p.k + head_offset;
  const uint16_t *v_base = p.v + head_offset;
  uint8_t *ring = smem + warp * (kStagesFd * 2 * kTileBytes);
  const uint32_t ring_addr = static_cast<uint32_t>(__cvta_generic_to_shared(ring));

  auto issue_tile = [&](int tile, int slot) {
    if (tile < tiles) {
      const int row0 = warp_begin + tile * kTileRows;
      const uint32_t k_dst = ring_addr + slot * (2 * kTileBytes);
      const uint32_t v_dst = k_dst + kTileBytes;
#pragma unroll
      for (int i = 0; i < (kTileRows * 16) / 32; ++i) {
        const int idx = i * 32 + lane;
        const int r = idx >> 4, c = idx & 15;
        const int row = row0 + r;
        const bool in_range = row < p.kv_len;
        const size_t src = static_cast<size_t>(in_range ? row : 0) * kD + c * 8;
        cp_async16(k_dst + tile_offset(r, c), k_base + src, in_range ? 16u : 0u);
        cp_async16(v_dst + tile_offset(r, c), v_base + src, in_range ? 16u : 0u);
      }
    }
    cp_async_commit();
  };

  float m_run[2] = {-INFINITY, -INFINITY};  // rows g and g + 8
  float l_run[2] = {0.f, 0.f};              // this lane's share of the row sum
  float acc[kD / 8][4];
#pragma unroll
  for (int j = 0; j < kD / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

#pragma unroll
  for (int s = 0; s < kStagesFd - 1; ++s) issue_tile(s, s);

  for (int tile = 0; tile < tiles; ++tile) {
    cp_async_wait<kStagesFd - 2>();
    __syncwarp();
    issue_tile(tile + kStagesFd - 1, (tile + kStagesFd - 1) % kStagesFd);

    const uint32_t k_src = ring_addr + (tile % kStagesFd) * (2 * kTileBytes);
    const uint32_t v_src = k_src + kTileBytes;
    const int row0 = warp_begin + tile * kTileRows;

    // S = Q K^T for 16 keys: two n-tiles of 8 keys.
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < kD / 16; ++ks) {
      const int mi = lane >> 3;
      const int r = (mi >> 1) * 8 + (lane & 7);
      const int c = 2 * ks + (mi & 1);
      uint32_t bfrag[4];
      ldmatrix_x4(k_src + tile_offset(r, c), bfrag);
      mma_16816<kBf16>(s0, q_frag[ks], bfrag[0], bfrag[1]);
      mma_16816<kBf16>(s1, q_frag[ks], bfrag[2], bfrag[3]);
    }
    // score region: scale, then mask keys outside the visible interval.
    const int key0 = row0 + 2 * t;
    float sc[2][4];  // [row half][key 2t, 2t+1, 8+2t, 8+2t+1]
    sc[0][0] = s0[0] * p.scale; sc[0][1] = s0[1] * p.scale; sc[0][2] = s1[0] * p.scale; sc[0][3] = s1[1] * p.scale;
    sc[1][0] = s0[2] * p.scale; sc[1][1] = s0[3] * p.scale; sc[1][2] = s1[2] * p.scale; sc[1][3] = s1[3] * p.scale;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (key0 >= warp_end) sc[h][0] = -INFINITY;
      if (key0 + 1 >= warp_end) sc[h][1] = -INFINITY;
      if (key0 + 8 >= warp_end) sc[h][2] = -INFINITY;
      if (key0 + 9 >= warp_end) sc[h][3] = -INFINITY;
    }
    uint32_t p_frag[4];
    float alpha[2];
    float pr[2][4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float tile_max = fmaxf(fmaxf(sc[h][0], sc[h][1]), fmaxf(sc[h][2], sc[h][3]));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
      const float m_new = fmaxf(tile_max, m_run[h]);
      const float m_exp = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[h] = exp_lp(m_run[h] - m_exp);
      float row_sum = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        pr[h][i] = exp_lp(sc[h][i] - m_exp);
        row_sum += pr[h][i];
      }
      l_run[h] = l_run[h] * alpha[h] + row_sum;
      m_run[h] = m_new;
    }
    // Probabilities are rounded to the storage type of V at the PV input.
    p_frag[0] = pack2<kBf16>(pr[0][0], pr[0][1]);
    p_frag[1] = pack2<kBf16>(pr[1][0], pr[1][1]);
    p_frag[2] = pack2<kBf16>(pr[0][2], pr[0][3]);
    p_frag[3] = pack2<kBf16>(pr[1][2], pr[1][3]);
#pragma unroll
    for (int j = 0; j < kD / 8; ++j) {
      acc[j][0] *= alpha[0]; acc[j][1] *= alpha[0];
      acc[j][2] *= alpha[1]; acc[j][3] *= alpha[1];
    }
#pragma unroll
    for (int j = 0; j < kD / 8; j += 2) {
      const int mi = lane >> 3;
      const int r = (mi & 1) * 8 + (lane & 7);
      const int c = j + (mi >> 1);
      uint32_t vfrag[4];
      ldmatrix_x4_trans(v_src + tile_offset(r, c), vfrag);
      mma_16816<kBf16>(acc[j], p_frag, vfrag[0], vfrag[1]);
      mma_16816<kBf16>(acc[j + 1], p_frag, vfrag[2], vfrag[3]);
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  __syncthreads();  // every warp is done with its ring; reuse it for the merge records

  float *records = reinterpret_cast<float *>(smem);  // [warp][16][kRecord]
  {
    float *mine = records + static_cast<size_t>(warp) * 16 * kRecord;
#pragma unroll
    for (int j = 0; j < kD / 8; ++j) {
      mine[g * kRecord + j * 8 + 2 * t] = acc[j][0];
      mine[g * kRecord + j * 8 + 2 * t + 1] = acc[j][1];
      mine[(g + 8) * kRecord + j * 8 + 2 * t] = acc[j][2];
      mine[(g + 8) * kRecord + j * 8 + 2 * t + 1] = acc[j][3];
    }
    if (t == 0) {
      mine[g * kRecord + kD] = m_run[0];
      mine[g * kRecord + kD + 1] = l_run[0];
      mine[(g + 8) * kRecord + kD] = m_run[1];
      mine[(g + 8) * kRecord + kD + 1] = l_run[1];
    }
  }
  __syncthreads();
  // Left fold over the warps (ascending KV order), one thread per (head, d).
  for (int idx = threadIdx.x; idx < p.group * kD; idx += blockDim.x) {
    const int head = idx / kD, d = idx % kD;
    const float *rec = records + head * kRecord;
    float m = rec[kD], l = rec[kD + 1], a = rec[d];
    for (int w = 1; w < kWarps; ++w) {
      const float *right = records + static_cast<size_t>(w) * 16 * kRecord + head * kRecord;
      const float m_right = right[kD], l_right = right[kD + 1], a_right = right[d];
      const float m_new = fmaxf(m, m_right);
      const float m_exp = (m_new == -INFINITY) ? 0.f : m_new;
      const float scale_left = exp_lp(m - m_exp), scale_right = exp_lp(m_right - m_exp);
      l = l * scale_left + l_right * scale_right;
      a = a * scale_left + a_right * scale_right;
      m = m_new;
    }
    float *out = p.partials +
                 ((static_cast<size_t>(b) * p.q_heads + hk * p.group + head) * p.splits + split) * kRecord;
    out[d] = a;
    if (d == 0) {
      out[kD] = m;
      out[kD + 1] = l;
    }
  }
  if constexpr (kTail) {
    // The CTA that finishes last among the splits of this (batch, kv head) folds the splits of the group's query heads,
    // exchanges the states with the other ranks and writes the outputs: the decode step is this one launch.
    __shared__ bool last_of_head;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned int *arrivals = tail.arrivals + b * p.kv_heads + hk;
      last_of_head = atomicAdd(arrivals, 1u) == static_cast<unsigned int>(p.splits) - 1u;
      if (last_of_head) *arrivals = 0u;     // ready for the next launch
    }
    __syncthreads();
    if (last_of_head) {
      __threadfence();
      const int first_row = b * p.q_heads + hk * p.group;
      fd_exchange_rows<kD / 32>(tail, p.partials, p.splits, first_row, p.group, p.batch * p.q_heads);
    }
  }
}

struct FdCombineParams {
  int rows;            // batch * q_heads
  int records;         // number of records folded per row
  size_t row_stride;   // floats between consecutive rows of one record index
  size_t record_stride;// floats between consecutive records of one row
  const float *records_ptr;
  int out_format;
  int zero_fully_masked;
  int finalize;
  void *out;
  float *lse, *row_max, *row_sum, *state_out;
};

__global__ void __launch_bounds__(kD) fd_combine_kernel(const FdCombineParams p) {
  const int row = blockIdx.x, d = threadIdx.x;
  const float *rec = p.records_ptr + row * p.row_stride;
  float m = rec[kD], l = rec[kD + 1], a = rec[d];
  for (int i = 1; i < p.records; ++i) {
    const float *right = rec + i * p.record_stride;
    const float m_right = right[kD], l_right = right[kD + 1], a_right = right[d];
    const float m_new = fmaxf(m, m_right);
    const float m_exp = (m_new == -INFINITY) ? 0.f : m_new;
    const float scale_left = exp_lp(m - m_exp), scale_right = exp_lp(m_right - m_exp);
    l = l * scale_left + l_right * scale_right;
    a = a * scale_left + a_right * scale_right;
    m = m_new;
  }
  if (!p.finalize) {
    float *state = p.state_out + static_cast<size_t>(row) * kRecord;
    state[d] = a;
    if (d == 0) {
      state[kD] = m;
      state[kD + 1] = l;
    }
    return;
  }
  float coefficient = 1.0f / l;
  if (p.zero_fully_masked && l == 0.f) coefficient = 0.f;
  const float value = a * coefficient;
  if (p.out_format == WB200_F32)
    reinterpret_cast<float *>(p.out)[static_cast<size_t>(row) * kD + d] = value;
  else
    reinterpret_cast<uint16_t *>(p.out)[static_cast<size_t>(row) * kD + d] =
        static_cast<uint16_t>(narrow_bits(value, p.out_format));
  if (d == 0) {
    if (p.lse) p.lse[row] = (l == 0.f) ? -INFINITY : m + logf(l);
    if (p.row_max) p.row_max[row] = m;
    if (p.row_sum) p.row_sum[row] = l;
  }
}

// Sequence-sharded decode, one shard per GPU: the fold over this GPU's splits, the exchange of the per-head states
// between the GPUs and the final merge in one kernel (one CTA per (batch, query head) row, thread = head dimension).
// Every rank owns an exchange buffer that all ranks can address (peer-mapped memory):
//   states [2][world][rows][kRecord] floats, then flags [2][world][rows] words, both indexed by the parity of an epoch
// that advances by one per call on every rank. A CTA writes its row's state into slot [parity][rank][row] of every
// rank's buffer with plain stores over NVLink, publishes it with a release store of the epoch tag to the matching
// flag, waits (bounded) until the flags of all ranks for its row carry the tag in its own buffer, and folds the world's
// states in ascending rank order - the shard order of the reference's spatial flash-decoding fold
// (lib/Wafer/Transforms/Linalg/SpatialRegionMaterialization.cpp:2420-2433). A rank can run at most one epoch ahead of
// another (its next exchange cannot complete before the other has entered it), so two parities suffice.
__device__ __forceinline__ void st_relaxed_sys(unsigned int *address, unsigned int value) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(address), "r"(value) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int *address) {
  unsigned int value;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
  return value;
}

// Rows [first_row, first_row + row_count) of the (batch, query head) rows, by one CTA of kD threads = four warps: a warp
// takes a row, a lane four consecutive head dimensions. Per batch of four rows: fold of the rows' split records in
// ascending order, stores of the states into every rank's buffer, flags, bounded wait for the world's flags, merge in
// ascending rank order, outputs. The rows of a batch travel together, so the NVLink round trip is paid once per batch.
__device__ __forceinline__ void fd_merge_right(float &m, float &l, float4 &a, float m_right, float l_right, const float4 &a_right) {
  const float m_new = fmaxf(m, m_right);
  const float m_exp = (m_new == -INFINITY) ? 0.f : m_new;
  const float scale_left = exp_lp(m - m_exp), scale_right = exp_lp(m_right - m_exp);
  l = l * scale_left + l_right * scale_right;
  a.x = a.x * scale_left + a_right.x * scale_right;
  a.y = a.y * scale_left + a_right.y * scale_right;
  a.z = a.z * scale_left + a_right.z * scale_right;
  a.w = a.w * scale_left + a_right.w * scale_right;
  m = m_new;
}
// Four consecutive floats of a record (records are 130 floats long: 8-byte, not 16-byte, aligned), read past L1.
__device__ __forceinline__ float4 ldcg_quad(const float *address) {
  const float2 lo = __ldcg(reinterpret_cast<const float2 *>(address)), hi = __ldcg(reinterpret_cast<const float2 *>(address + 2));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
template <int kRowsAtOnce>
__device__ void fd_exchange_rows(const FdTailParams &x, const float *records, int splits, int first_row, int row_count, int rows_total) {
  static_assert(kRowsAtOnce == kD / 32, "one warp per row");
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int *>(x.epoch);
  const unsigned int parity = epoch & 1u, tag = epoch + 1u;
  const size_t state_floats = static_cast<size_t>(2) * x.world * rows_total * kRecord;
  float *own = x.peer[x.rank];
  for (int base = 0; base < row_count; base += kRowsAtOnce) {
    const int count = row_count - base < kRowsAtOnce ? row_count - base : kRowsAtOnce;
    const int row = first_row + base + warp;
    const bool active = warp < count;
    if (active) {
      // fold this rank's splits (records of other CTAs: read past L1), twelve records in flight: the fold is a chain
      // of L2 round trips otherwise (a single resident wave of a long sequence has 37 splits per head)
      const float *rec = records + static_cast<size_t>(row) * splits * kRecord;
      float m = __ldcg(rec + kD), l = __ldcg(rec + kD + 1);
      float4 a = ldcg_quad(rec + 4 * lane);
      int s = 1;
      constexpr int kBatch = 12;
      for (; s + kBatch <= splits; s += kBatch) {
        float mr[kBatch], lr[kBatch];
        float4 ar[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const float *right = rec + static_cast<size_t>(s + u) * kRecord;
          const float2 ml = __ldcg(reinterpret_cast<const float2 *>(right + kD));
          mr[u] = ml.x; lr[u] = ml.y;
          ar[u] = ldcg_quad(right + 4 * lane);
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) fd_merge_right(m, l, a, mr[u], lr[u], ar[u]);
      }
      for (; s + 4 <= splits; s += 4) {
        float mr[4], lr[4];
        float4 ar[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float *right = rec + static_cast<size_t>(s + u) * kRecord;
          mr[u] = __ldcg(right + kD); lr[u] = __ldcg(right + kD + 1);
          ar[u] = ldcg_quad(right + 4 * lane);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) fd_merge_right(m, l, a, mr[u], lr[u], ar[u]);
      }
      for (; s < splits; ++s) {
        const float *right = rec + static_cast<size_t>(s) * kRecord;
        const float4 ar = ldcg_quad(right + 4 * lane);
        fd_merge_right(m, l, a, __ldcg(right + kD), __ldcg(right + kD + 1), ar);
      }
      // the state into slot [parity][rank][row] of every rank's buffer (records are 130 floats: 8-byte aligned rows)
      const size_t my_slot = (static_cast<size_t>(parity) * x.world + x.rank) * rows_total + row;
      for (int r = 0; r < x.world; ++r) {
        float *dst = x.peer[r] + my_slot * kRecord;
        *reinterpret_cast<float2 *>(dst + 4 * lane) = make_float2(a.x, a.y);
        *reinterpret_cast<float2 *>(dst + 4 * lane + 2) = make_float2(a.z, a.w);
        if (lane == 0) *reinterpret_cast<float2 *>(dst + kD) = make_float2(m, l);
      }
    }
    __syncthreads();   // the rows are written before they are published
    // One thread per (row, peer): a system-scope fence (cumulative over the rows' stores, which the barrier ordered
    // before it) and then the flag; the fences of the peers run side by side. Then the bounded wait for every rank's
    // flag of every row, again one thread per (row, rank).
    for (int j = tid; j < count * x.world; j += kD) {
      const int flag_row = first_row + base + j / x.world, peer = j % x.world;
      const size_t my_slot = (static_cast<size_t>(parity) * x.world + x.rank) * rows_total + flag_row;
      __threadfence_system();
      st_relaxed_sys(reinterpret_cast<unsigned int *>(x.peer[peer] + state_floats) + my_slot, tag);
    }
    for (int j = tid; j < count * x.world; j += kD) {
      const int flag_row = first_row + base + j / x.world, source = j % x.world;
      const unsigned int *flag = reinterpret_cast<const unsigned int *>(own + state_floats) + (static_cast<size_t>(parity) * x.world + source) * rows_total + flag_row;
      const long long start = clock64();
      unsigned int polls = 0;
      while (ld_acquire_sys(flag) != tag) {
        if ((++polls & 63u) == 0u && clock64() - start > 2000000000LL) {   // about a second: give up, report, carry on
          atomicExch(x.status, 2);
          break;
        }
      }
    }
    __syncthreads();
    if (active) {
      // merge the world's states in ascending shard order (L1 is bypassed: peers wrote these lines)
      auto load_state = [&](int r, float &m, float &l, float4 &a) {
        const float *state = own + ((static_cast<size_t>(parity) * x.world + r) * rows_total + row) * kRecord;
        const float2 ml = __ldcg(reinterpret_cast<const float2 *>(state + kD));
        a = ldcg_quad(state + 4 * lane);
        m = ml.x; l = ml.y;
      };
      float m, l;
      float4 a;
      load_state(0, m, l, a);
      int r = 1;
      for (; r + 7 <= x.world; r += 7) {   // the states of seven more ranks in flight together (eight GPUs: one batch)
        float mr[7], lr[7];
        float4 ar[7];
#pragma unroll
        for (int u = 0; u < 7; ++u) load_state(r + u, mr[u], lr[u], ar[u]);
#pragma unroll
        for (int u = 0; u < 7; ++u) fd_merge_right(m, l, a, mr[u], lr[u], ar[u]);
      }
      for (; r < x.world; ++r) {
        float m_right, l_right;
        float4 a_right;
        load_state(r, m_right, l_right, a_right);
        fd_merge_right(m, l, a, m_right, l_right, a_right);
      }
      float coefficient = 1.0f / l;
      if (x.zero_fully_masked && l == 0.f) coefficient = 0.f;
      const float value[4] = {a.x * coefficient, a.y * coefficient, a.z * coefficient, a.w * coefficient};
      if (x.out_format == WB200_F32) {
        *(reinterpret_cast<float4 *>(x.out) + static_cast<size_t>(row) * (kD / 4) + lane) = make_float4(value[0], value[1], value[2], value[3]);
      } else {
        const uint32_t lo = narrow_bits(value[0], x.out_format) | (static_cast<uint32_t>(narrow_bits(value[1], x.out_format)) << 16);
        const uint32_t hi = narrow_bits(value[2], x.out_format) | (static_cast<uint32_t>(narrow_bits(value[3], x.out_format)) << 16);
        *(reinterpret_cast<uint2 *>(x.out) + static_cast<size_t>(row) * (kD / 4) + lane) = make_uint2(lo, hi);
      }
      if (lane == 0) {
        if (x.lse) x.lse[row] = (l == 0.f) ? -INFINITY : m + logf(l);
        if (x.row_max) x.row_max[row] = m;
        if (x.row_sum) x.row_sum[row] = l;
      }
    }
  }
  // the CTA that completes the last rows of the launch advances the epoch for the next call
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(x.epoch + 1, static_cast<unsigned int>(row_count)) + row_count == static_cast<unsigned int>(rows_total)) {
      x.epoch[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned int *>(x.epoch) = epoch + 1u;
    }
  }
}

// The same tail as a launch of its own (four rows per CTA), behind a stage 1 without it.
__global__ void __launch_bounds__(kD) fd_exchange_kernel(const FdTailParams x, const float *records, int splits, int rows_total) {
  const int first_row = blockIdx.x * (kD / 32);
  const int row_count = rows_total - first_row < kD / 32 ? rows_total - first_row : kD / 32;
  fd_exchange_rows<kD / 32>(x, records, splits, first_row, row_count, rows_total);
}

int visible_keys(const AttentionArgs &a) {
  int64_t visible = a.kv_valid < a.kv_len ? a.kv_valid : a.kv_len;
  if (a.causal && a.causal_offset + 1 < visible) visible = a.causal_offset + 1;
  return visible < 0 ? 0 : static_cast<int>(visible);
}

}  // namespace

bool attention_fd_supports(const AttentionArgs &a) {
  if (a.q_len != 1 || a.head_dim != kD) return false;
  if (a.format != WB200_BF16 && a.format != WB200_F16) return false;
  if (a.kv_heads <= 0 || a.q_heads % a.kv_heads != 0 || a.q_heads / a.kv_heads > 16) return false;
  if ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v)) & 15u)
    return false;
  return a.kv_len > 0 && a.batch > 0;
}

uint32_t fd_choose_splits(const AttentionArgs &a, int sm_count) {
  const int64_t visible = visible_keys(a);
  const int64_t units = static_cast<int64_t>(a.batch) * a.kv_heads;
  const int64_t slots = 2LL * sm_count;                 // two CTAs are resident per SM
  const int64_t base = (visible + 2047) / 2048;         // 2048-key splits
  // More (batch, kv head) units than resident slots: 2048-key splits give many short CTAs, which the hardware deals out
  // as slots free up (the tail is one short CTA), and the fold over a unit's few splits is short.
  if (units >= slots) return static_cast<uint32_t>(base < 2 ? 2 : (base > 4096 ? 4096 : base));
  // Otherwise pick the split count with the least estimated time, in units of one key streamed by one CTA:
  // waves x (keys per split + the CTA's fixed cost) + the serial fold over the splits (one record costs about as much
  // as six keys). A long sequence with few (batch, kv head) units ends up with exactly one resident wave.
  int64_t limit = visible / 256;                        // at least 256 keys per split
  if (limit > 4096) limit = 4096;
  int64_t best_splits = 2, best_cost = -1;
  for (int64_t splits = 2; splits <= (limit < 2 ? 2 : limit); ++splits) {
    const int64_t rows = ((visible + splits - 1) / splits + 63) / 64 * 64;
    const int64_t waves = (units * splits + slots - 1) / slots;
    const int64_t cost = waves * (rows + 130) + 6 * splits;
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_splits = splits; }
  }
  return static_cast<uint32_t>(best_splits);            // flash-decoding splits K2 into at least two intervals
}

size_t fd_partial_floats(const AttentionArgs &a, uint32_t splits) {
  return static_cast<size_t>(a.batch) * a.q_heads * splits * kRecord;
}

namespace {
wb200_status launch_fd_stage1(const AttentionArgs &a, uint32_t splits, float *partials, cudaStream_t stream,
                              const FdTailParams *tail = nullptr);
}

size_t fd_exchange_floats(int rows, int world) {
  // states [2][world][rows][kRecord] floats followed by flags [2][world][rows] words
  return static_cast<size_t>(2) * world * rows * (kRecord + 1);
}

wb200_status launch_attention_fd_exchange(const AttentionArgs &a, uint32_t splits, float *partials, int rank, int world,
                                          void *const *peer_buffers, unsigned int *epoch, unsigned int *arrivals,
                                          int *device_status, cudaStream_t stream) {
  if (world < 1 || world > kMaxExchangeRanks || rank < 0 || rank >= world)
    return fail(WB200_ERR_INVALID_ARGUMENT, "exchange takes 1 to 16 ranks and a rank inside the world");
  FdTailParams x;
  x.rank = rank; x.world = world;
  for (int r = 0; r < kMaxExchangeRanks; ++r) x.peer[r] = r < world ? static_cast<float *>(peer_buffers[r]) : nullptr;
  x.epoch = epoch;
  x.arrivals = arrivals;
  x.out_format = a.format;
  x.zero_fully_masked = a.zero_fully_masked;
  x.out = a.out; x.lse = a.lse; x.row_max = a.row_max; x.row_sum = a.row_sum;
  x.status = device_status;
  // With arrival counters the tail runs inside stage 1 (its last CTA per (batch, kv head)): one launch per step.
  // Without them it is a launch of its own behind stage 1.
  wb200_status st = launch_fd_stage1(a, splits, partials, stream, arrivals ? &x : nullptr);
  if (st != WB200_OK) return st;
  if (!arrivals) {
    const int rows = a.batch * a.q_heads;
    fd_exchange_kernel<<<(rows + kD / 32 - 1) / (kD / 32), kD, 0, stream>>>(x, partials, static_cast<int>(splits), rows);
    WB200_CUDA_CHECK(cudaGetLastError());
  }
  return WB200_OK;
}

wb200_status launch_attention_fd(const AttentionArgs &a, uint32_t splits, float *partials, int finalize,
                                 float *state_out, cudaStream_t stream) {
  wb200_status st = launch_fd_stage1(a, splits, partials, stream);
  if (st != WB200_OK) return st;
  FdCombineParams c;
  c.rows = a.batch * a.q_heads;
  c.records = static_cast<int>(splits);
  c.row_stride = static_cast<size_t>(splits) * kRecord;
  c.record_stride = kRecord;
  c.records_ptr = partials;
  c.out_format = a.format;
  c.zero_fully_masked = a.zero_fully_masked;
  c.finalize = finalize;
  c.out = a.out; c.lse = a.lse; c.row_max = a.row_max; c.row_sum = a.row_sum; c.state_out = state_out;
  fd_combine_kernel<<<c.rows, kD, 0, stream>>>(c);
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

namespace {
wb200_status launch_fd_stage1(const AttentionArgs &a, uint32_t splits, float *partials, cudaStream_t stream, const FdTailParams *tail) {
  if (!attention_fd_supports(a)) return fail(WB200_ERR_UNSUPPORTED, "flash-decoding request outside the kernel's domain");
  if (splits < 1) return fail(WB200_ERR_INVALID_ARGUMENT, "kv_splits must be positive");
  FdParams p;
  p.batch = a.batch; p.q_heads = a.q_heads; p.kv_heads = a.kv_heads; p.group = a.q_heads / a.kv_heads;
  p.kv_len = a.kv_len;
  p.kv_visible = visible_keys(a);
  p.splits = static_cast<int>(splits);
  const int64_t per_split = (static_cast<int64_t>(p.kv_visible) + splits - 1) / splits;
  const int64_t granule = kWarps * kTileRows;
  p.rows_per_split = static_cast<int>(((per_split + granule - 1) / granule) * granule);
  if (p.rows_per_split == 0) p.rows_per_split = static_cast<int>(granule);
  p.rows_per_warp = p.rows_per_split / kWarps;
  p.scale = a.scale;
  p.q = static_cast<const uint16_t *>(a.q);
  p.k = static_cast<const uint16_t *>(a.k);
  p.v = static_cast<const uint16_t *>(a.v);
  p.partials = partials;

  static PerDeviceOnce attributes;
  const wb200_status attribute_status = attributes.run([]() -> wb200_status {
    WB200_CUDA_CHECK(cudaFuncSetAttribute(fd_partial_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFdSmemBytes));
    WB200_CUDA_CHECK(cudaFuncSetAttribute(fd_partial_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFdSmemBytes));
    WB200_CUDA_CHECK(cudaFuncSetAttribute(fd_partial_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFdSmemBytes));
    WB200_CUDA_CHECK(cudaFuncSetAttribute(fd_partial_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFdSmemBytes));
    return WB200_OK;
  });
  if (attribute_status != WB200_OK) return attribute_status;
  dim3 grid(splits, a.kv_heads, a.batch);
  static_assert(kWarps * 32 == kD, "the tail of the sharded decode runs with one thread per head dimension");
  const FdTailParams none{};
  if (tail) {
    if (a.format == WB200_BF16) fd_partial_kernel<true, true><<<grid, kWarps * 32, kFdSmemBytes, stream>>>(p, *tail);
    else fd_partial_kernel<false, true><<<grid, kWarps * 32, kFdSmemBytes, stream>>>(p, *tail);
  } else {
    if (a.format == WB200_BF16) fd_partial_kernel<true, false><<<grid, kWarps * 32, kFdSmemBytes, stream>>>(p, none);
    else fd_partial_kernel<false, false><<<grid, kWarps * 32, kFdSmemBytes, stream>>>(p, none);
  }
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}
}  // namespace

wb200_status launch_attention_fd_merge(const AttentionArgs &a, const float *states, uint32_t shard_count,
                                       cudaStream_t stream) {
  if (a.head_dim != kD) return fail(WB200_ERR_UNSUPPORTED, "merge supports head_dim 128");
  if (shard_count < 1) return fail(WB200_ERR_INVALID_ARGUMENT, "shard_count must be positive");
  FdCombineParams c;
  c.rows = a.batch * a.q_heads;
  c.records = static_cast<int>(shard_count);
  c.row_stride = kRecord;
  c.record_stride = static_cast<size_t>(c.rows) * kRecord;
  c.records_ptr = states;
  c.out_format = a.format;
  c.zero_fully_masked = a.zero_fully_masked;
  c.finalize = 1;
  c.out = a.out; c.lse = a.lse; c.row_max = a.row_max; c.row_sum = a.row_sum; c.state_out = nullptr;
  fd_combine_kernel<<<c.rows, kD, 0, stream>>>(c);
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

}  // namespace wb200

// ------------------------------------------------------------------ allocation-free entry point
// Some callers may not allocate device memory when they reach this library: a latency-critical
// serving loop whose memory was carved up at start-up and where a cudaMalloc (an implicit device
// synchronisation) is not acceptable, a host that shares the GPU under a fixed memory budget, or code
// that runs at a point where the CUDA runtime refuses allocation calls. For them the split-KV partial records live in
// a fixed array inside the library image instead of in a buffer the backend allocates on demand.
#include <mutex>

#include "backend.h"

namespace wb200 {
namespace {

constexpr size_t kStaticScratchFloats = size_t(4) << 20;   // 16 MiB, held by every GPU that loads the library
static __device__ __align__(256) float g_fd_static_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
float *g_fd_static_scratch_address[kMaxDevices] = {nullptr};
std::mutex g_fd_static_scratch_mutex;

// In host code `g_fd_static_scratch` names a host-side handle, not device memory; the address a kernel
// can use has to be asked for, once per device, with that device current.
wb200_status static_scratch_for_device(int device, float **out) {
  if (device < 0 || device >= kMaxDevices) return fail(WB200_ERR_LIMIT, "device index beyond the static scratch table");
  std::lock_guard<std::mutex> lock(g_fd_static_scratch_mutex);
  if (!g_fd_static_scratch_address[device]) {
    void *address = nullptr;
    WB200_CUDA_CHECK(cudaGetSymbolAddress(&address, g_fd_static_scratch));
    g_fd_static_scratch_address[device] = static_cast<float *>(address);
  }
  *out = g_fd_static_scratch_address[device];
  return WB200_OK;
}

}  // namespace
}  // namespace wb200

extern "C" wb200_status wb200_attention_fd_static(wb200_backend *backend, const wb200_attention_params *p,
                                                  uint32_t kv_splits) {
  using namespace wb200;
  if (!backend || !p) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  if (p->memory != WB200_MEM_DEVICE)
    return fail(WB200_ERR_UNSUPPORTED, "the allocation-free decode takes device buffers only (staging host buffers would allocate)");
  if (!p->q || !p->k || !p->v || !p->out) return fail(WB200_ERR_INVALID_ARGUMENT, "q, k, v and out must not be null");
  if (p->q_len != 1) return fail(WB200_ERR_INVALID_ARGUMENT, "flash-decoding takes query length 1");
  if (p->batch == 0 || p->q_heads == 0 || p->kv_heads == 0 || p->kv_len == 0 || p->q_heads % p->kv_heads != 0 ||
      p->kv_len > 0x7fffffffu)
    return fail(WB200_ERR_INVALID_ARGUMENT, "invalid attention extents");
  AttentionArgs a{};
  a.batch = p->batch; a.q_heads = p->q_heads; a.kv_heads = p->kv_heads;
  a.q_len = 1; a.kv_len = p->kv_len; a.head_dim = p->head_dim;
  a.format = p->format;
  a.causal = p->causal ? 1 : 0;
  a.zero_fully_masked = p->zero_fully_masked ? 1 : 0;
  a.scale = p->scale;
  a.causal_offset = p->query_start - p->key_start;
  a.kv_valid = p->key_end > 0 ? p->key_end - p->key_start : static_cast<int64_t>(p->kv_len);
  a.q = p->q; a.k = p->k; a.v = p->v; a.out = p->out;
  a.lse = p->lse; a.row_max = p->row_max; a.row_sum = p->row_sum;
  if (!attention_fd_supports(a))
    return fail(WB200_ERR_UNSUPPORTED, "flash-decoding kernel takes f16/bf16 storage, head_dim 128, group size <= 16");
  DeviceGuard guard(backend->device);
  uint32_t splits = kv_splits;
  if (splits == 0) {
    splits = fd_choose_splits(a, backend->sm_count);
    while (splits > 2 && fd_partial_floats(a, splits) > kStaticScratchFloats) splits = (splits + 1) / 2;
  }
  const size_t needed = fd_partial_floats(a, splits);
  if (needed > kStaticScratchFloats)
    return fail(WB200_ERR_LIMIT, "allocation-free decode: batch * q_heads * kv_splits * (head_dim + 2) = " + std::to_string(needed) +
                                     " floats exceeds the fixed scratch of " + std::to_string(kStaticScratchFloats) + " floats (16 MiB)");
  float *scratch = nullptr;
  wb200_status st = static_scratch_for_device(backend->device, &scratch);
  if (st != WB200_OK) return st;
  // Stage 1 writes every record stage 2 reads, so nothing left by an earlier call needs clearing.
  st = launch_attention_fd(a, splits, scratch, 1, nullptr, static_cast<cudaStream_t>(p->stream));
  if (st == WB200_OK) backend->launches += 2;
  return st;
}
