// Flash-attention prefill for sm_100a on tcgen05 tensor cores (bf16 / f16 storage, head_dim 128).
//
// Arithmetic is the reference's online-attention update per KV tile
// (lib/Wafer/Transforms/Linalg/OnlineAttentionDecomposition.cpp:568-594):
//   S = Q K^T (f32), s = S*scale (+mask), m' = max(m, rowmax s), m_e = (m' == -inf ? 0 : m'),
//   alpha = exp(m - m_e), l' = l*alpha + sum exp(s - m_e), acc' = acc*alpha + round(P) V,
// with P rounded to the storage type at the PV input, and finalize out = acc * (1/l)
// (lib/Wafer/Transforms/Linalg/OnlineAttentionMaterialization.cpp:196-262). The KV axis is never
// split across workers. Scores are kept in the log2 domain (scale*log2e folded into one f32
// constant) so exp is one ex2 per element.
//
// One work item is 256 query rows of one (batch, head): two 128-row Q tiles, each with its own S and O
// accumulators in TMEM (S0 S1 O0 O1 = 4 x 128 columns) and its own softmax warpgroup, so the tensor
// pipe works on one tile while the other tile's softmax runs. A persistent grid of one CTA per SM walks
// a host-made plan of items, so the loads and first scores of an item overlap the softmax tail and
// write-out of the previous one and every CTA ends at nearly the same time. Warp 0 = TMA producer (per
// item: Q, then K0 V0 K1 V1 ... through a ring of five 32 KiB slots that runs on across items), warp 1 =
// MMA issuer and TMEM owner (the whole warp walks the loop, one elected lane issues), warps 4-7 / 8-11 =
// softmax + rescale + epilogue for Q tile 0 / 1 (thread = query row, so row max and row sum need no
// shuffles; setmaxnreg moves registers from warpgroup 0 to the softmax warpgroups). All mbarriers are
// reused across items with running completion counts as parities. The rounded P lives in TMEM over the
// first 64 columns of its scores and is the A operand of the PV product: with P in shared memory instead
// every product would read both operands from shared memory, whose bandwidth (128 B per clock) a
// 128 x 128 x 16 product with two shared-memory operands already uses in full.
// Roofline: tensor pipe; algorithmic work is 4 * head_dim flop per visible (query, key) pair.
#include <algorithm>
#include <map>
#include <mutex>
#include <queue>
#include <tuple>
#include <type_traits>
#include <vector>

#include "kernels.h"
#include "ptx_sm100.cuh"

namespace wb200 {
namespace {

constexpr int kHd = 128;          // head dimension
constexpr int kTileM = 128;       // query rows per Q tile (TMEM lanes)
constexpr int kTileN = 128;       // keys per KV tile
constexpr int kTileBytesFa = kTileN * kHd * 2;  // 32 KiB: two 64-element column blocks of 128 rows
constexpr int kBlockBytes = 128 * 128;          // one [128 rows][128 B] swizzled block
constexpr int kFaThreads = 384;          // warpgroup 0: TMA + MMA warps; warpgroups 1, 2: softmax of Q tile 0, 1
constexpr int kPParts = 2;               // P of a tile is published in two halves so PV starts on the first
constexpr int kChunksPerPart = 2;        // 32-key chunks per half
constexpr uint32_t kColS0 = 0, kColO0 = 256;    // S_t at t*128, O_t at 256 + t*128

struct FaSmem {
  static constexpr int kSlots = 5;         // K / V ring
  static constexpr int kQOff = 0;
  static constexpr int kRingOff = 2 * kTileBytesFa;
  static constexpr int kBarOff = kRingOff + kSlots * kTileBytesFa;
  static constexpr size_t kBytes = kBarOff + 256 + 1024;
};

struct FaParams {
  int batch, q_heads, kv_heads, group;
  int q_len, kv_len;
  int kv_visible;          // keys >= kv_visible are masked
  int causal;
  long long causal_offset; // key j visible to query row q iff j <= causal_offset + q
  int zero_fully_masked;
  int out_format;
  int bf16;
  int num_pairs;           // ceil(q_len / 256)
  int out_token_major;     // out is [batch, q_len, q_heads, head_dim] instead of [batch, q_heads, q_len, head_dim]
  const int *plan;         // [grid][plan_stride] item ids of each CTA in execution order, -1 terminated; null: CTA b runs item b
  int plan_stride;
  float scale_log2;        // scale * log2(e)
  void *out;
  float *lse, *row_max, *row_sum;
  int *status;
};

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}
// 2^x on the FMA pipe for x <= 0: x = n + f with n = round(x), f in [-0.5, 0.5]; 2^f by a degree-3 polynomial (maximum
// relative error 7.5e-5, far below the rounding of P to 16 bits), 2^n by adding n to the exponent field. x is clamped at
// -126, so the result is never exactly zero: tiles that hold masked (-inf) scores use the hardware ex2 throughout.
#ifndef WB200_FA_POLY_PERIOD
#define WB200_FA_POLY_PERIOD 4
#endif
constexpr int kPolyPeriod = WB200_FA_POLY_PERIOD;   // one pair of exponentials in kPolyPeriod runs on the FMA pipe
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -126.0f);
  const float shifted = x + 12582912.0f;                 // 1.5 * 2^23: the low mantissa bits now hold n
  const float f = x - (shifted - 12582912.0f);
  float p = fmaf(0.0551716685295105f, f, 0.2426111251115799f);
  p = fmaf(p, f, 0.6932609677314758f);
  p = fmaf(p, f, 0.9999280571937561f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(shifted) << 23));
}
// Packed pairs of f32 (sm_100 has two-wide f32 fma / add): halves the issue slots of the scaling and of the row sums.
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_f32x2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long add_f32x2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "setp.ne.b32 P, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, P;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// Number of KV tiles a Q tile starting at query row `row0` has to visit.
__device__ __forceinline__ int kv_tiles_for(const FaParams &p, int row0) {
  long long last = static_cast<long long>(p.kv_visible) - 1;
  if (p.causal) {
    const long long causal_last = p.causal_offset + row0 + (kTileM - 1);
    if (causal_last < last) last = causal_last;
  }
  if (row0 >= p.q_len || last < 0) return 0;
  return static_cast<int>(last / kTileN) + 1;
}

// One work item = 256 query rows (two Q tiles) of one (batch, head); item g covers pair num_pairs-1 - g / (batch*heads)
// of (batch, head) g % (batch*heads), so low ids are the heaviest under a causal mask. The launcher deals the items to
// the CTAs of a persistent grid with a longest-processing-time plan (each CTA: its items, heaviest first), so every
// CTA ends at nearly the same time; the kernel only walks its row of the plan.
struct FaItem {
  int valid;
  int bh, bh_kv, b, h;
  int row_base;
  int n0, n1;       // KV tiles Q tile 0 / 1 visits (scalars: a runtime-indexed array would live in local memory)
  int n_max;
  __device__ __forceinline__ int tiles(int t) const { return t ? n1 : n0; }
};
__device__ __forceinline__ FaItem fa_item(const FaParams &p, int k) {
  FaItem item;
  // 32-bit arithmetic only: a 64-bit division is an out-of-line call, and a call inside the MMA warp's code costs
  // about 8 % per KV step of its issue loop.
  int id;
  if (p.plan) id = p.plan[static_cast<size_t>(blockIdx.x) * p.plan_stride + k];
  else id = k == 0 ? static_cast<int>(blockIdx.x) : -1;   // no plan: CTA b runs item b only
  const unsigned g = static_cast<unsigned>(id);
  const unsigned bh_count = static_cast<unsigned>(p.batch * p.q_heads);
  item.valid = id >= 0;
  item.bh = item.bh_kv = item.b = item.h = item.row_base = item.n0 = item.n1 = item.n_max = 0;
  if (!item.valid) return item;
  const unsigned pair_rank = g / bh_count;
  const int pair = p.num_pairs - 1 - static_cast<int>(pair_rank);   // heaviest pairs first
  item.bh = static_cast<int>(g - pair_rank * bh_count);
  item.b = item.bh / p.q_heads;
  item.h = item.bh % p.q_heads;
  item.bh_kv = item.b * p.kv_heads + item.h / p.group;
  item.row_base = pair * 2 * kTileM;
  item.n0 = kv_tiles_for(p, item.row_base);
  item.n1 = kv_tiles_for(p, item.row_base + kTileM);
  item.n_max = item.n0 > item.n1 ? item.n0 : item.n1;
  return item;
}
// First item at or after position k that has KV tiles to visit (items without any are handled by the softmax
// warps alone); advances k past it.
__device__ __forceinline__ FaItem fa_next_working_item(const FaParams &p, int &k) {
  while (true) {
    const FaItem item = fa_item(p, k++);
    if (!item.valid || item.n_max > 0) return item;
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(kFaThreads, 1)
fa_umma_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  using L = FaSmem;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t *smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t smem_base = smem_u32(smem);

  const uint32_t bar_base = smem_base + L::kBarOff;
  auto kv_full = [&](int s) { return bar_base + 8u * s; };
  auto kv_empty = [&](int s) { return bar_base + 8u * (L::kSlots + s); };
  const uint32_t q_full = bar_base + 8u * (2 * L::kSlots);
  auto s_full = [&](int t) { return bar_base + 8u * (2 * L::kSlots + 1 + t); };
  // P of one tile is published in two halves (keys 0-63, 64-127) so PV can start on the first half.
  auto p_part = [&](int t, int part) { return bar_base + 8u * (2 * L::kSlots + 3 + kPParts * t + part); };
  auto o_done = [&](int t) { return bar_base + 8u * (2 * L::kSlots + 3 + 2 * kPParts + t); };
  const uint32_t q_empty = bar_base + 8u * (2 * L::kSlots + 5 + 2 * kPParts);   // every S product of an item has finished
  uint8_t *bar_ptr = smem + L::kBarOff;
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bar_ptr + 8 * (2 * L::kSlots + 6 + 2 * kPParts));
  volatile int *abort_word = reinterpret_cast<volatile int *>(bar_ptr + 8 * (2 * L::kSlots + 7 + 2 * kPParts));
  // All barriers are reused across work items; every role keeps running completion counts for the parities.

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::kSlots; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full(t), 1);
      for (int part = 0; part < kPParts; ++part) mbar_init(p_part(t, part), kTileM);
      mbar_init(o_done(t), 1);
    }
    *abort_word = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // setmaxnreg.inc blocks until the CTA's own register pool can supply the request, so the totals after
  // reallocation (128 * 104 + 256 * 200) must not exceed what the CTA was launched with (384 * 168).
  static_assert(128 * 104 + 256 * 200 <= kFaThreads * 168, "setmaxnreg totals exceed the launch allocation");
  if (warp < 4) {
  setmaxnreg_dec<104>();
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int slot = 0;
      uint32_t phase = 0, q_loads = 0;
      bool ok = true;
      int k = 0;
      while (ok) {
        const FaItem item = fa_next_working_item(p, k);
        if (!item.valid) break;
        // The Q buffer is free once every S product of the previous item has finished.
        if (q_loads > 0 && !mbar_wait(q_empty, (q_loads - 1) & 1u, abort_word, 101)) break;
        ++q_loads;
        mbar_arrive_expect_tx(q_full, 2 * kTileBytesFa);
        for (int t = 0; t < 2; ++t)
          for (int c = 0; c < 2; ++c)
            tma_load_3d(smem_base + L::kQOff + t * kTileBytesFa + c * kBlockBytes, &tmap_q, q_full, c * 64,
                        item.row_base + t * kTileM, item.bh);
        for (int i = 0; i < 2 * item.n_max; ++i) {  // ring position 2j = K_j, 2j+1 = V_j
          if (!mbar_wait(kv_empty(slot), phase ^ 1u, abort_word, 102)) { ok = false; break; }
          mbar_arrive_expect_tx(kv_full(slot), kTileBytesFa);
          const CUtensorMap *map = (i & 1) ? &tmap_v : &tmap_k;
          const uint32_t dst = smem_base + L::kRingOff + slot * kTileBytesFa;
          tma_load_3d(dst, map, kv_full(slot), 0, (i >> 1) * kTileN, item.bh_kv);
          tma_load_3d(dst + kBlockBytes, map, kv_full(slot), 64, (i >> 1) * kTileN, item.bh_kv);
          if (++slot == L::kSlots) { slot = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp walks this code (waits included) and one elected lane issues: with warp-uniform control flow
    // the descriptor arithmetic stays on the uniform datapath, so an instruction costs far fewer issue slots than in
    // a loop run by a single diverged lane (which measured 80-100 clocks per 128 x 128 x 16 product here, against the
    // 64 clocks the product occupies the tensor pipe).
    {
      constexpr uint32_t idesc_s = umma_idesc_f16(kTileM, kTileN, kBf16, false, false);
      constexpr uint32_t idesc_o = umma_idesc_f16(kTileM, kHd, kBf16, false, true);
      int slot = 0;
      uint32_t phase = 0;
      bool ok = true;
      auto advance = [&]() { if (++slot == L::kSlots) { slot = 0; phase ^= 1u; } };
      // Descriptors differ only in the 14-bit start-address field: one descriptor per buffer, and every ring slot or
      // k-step adds a constant to it.
      const uint64_t q_desc0 = umma_desc_kmajor(smem_base + L::kQOff);
      const uint64_t q_desc1 = umma_desc_kmajor(smem_base + L::kQOff + kTileBytesFa);
      const uint64_t ring_k_desc = umma_desc_kmajor(smem_base + L::kRingOff);
      const uint64_t ring_v_desc = umma_desc_mnmajor(smem_base + L::kRingOff, kBlockBytes);
      constexpr uint32_t kSlotStep = kTileBytesFa >> 4;
      auto issue_s = [&](auto tile_tag, int k_slot) {
        constexpr int t = decltype(tile_tag)::value;
        const uint64_t k_desc = ring_k_desc + static_cast<uint32_t>(k_slot) * kSlotStep;
        const uint64_t q_desc = t ? q_desc1 : q_desc0;
        const uint32_t d_tmem = tmem_base + kColS0 + t * 128;
        if (elect_one_sync()) {
#pragma unroll
          for (int ks = 0; ks < kHd / 16; ++ks) {
            constexpr uint32_t kBlockStep = kBlockBytes >> 4;
            const uint32_t off = (ks >> 2) * kBlockStep + (ks & 3) * 2;
            umma_f16_ss(d_tmem, q_desc + off, k_desc + off, idesc_s, ks != 0 ? 1u : 0u);
          }
          umma_commit(s_full(t));
        }
        __syncwarp();
      };
      // PV over the keys of one published part of P.
      auto issue_pv_part = [&](auto tile_tag, auto part_tag, int v_slot, bool accumulate) {
        constexpr int t = decltype(tile_tag)::value;
        constexpr int part = decltype(part_tag)::value;
        const uint64_t v_desc = ring_v_desc + static_cast<uint32_t>(v_slot) * kSlotStep;
        const uint32_t d_tmem = tmem_base + kColO0 + t * 128;
        if (elect_one_sync()) {
#pragma unroll
          for (int ks = (8 / kPParts) * part; ks < (8 / kPParts) * (part + 1); ++ks) {
            const uint64_t bdesc = v_desc + static_cast<uint32_t>((ks * 2048) >> 4);
            const uint32_t acc = (accumulate || ks != 0) ? 1u : 0u;
            umma_f16_ts(d_tmem, tmem_base + kColS0 + t * 128 + ks * 8, bdesc, idesc_o, acc);
          }
          if (part == kPParts - 1) umma_commit(o_done(t));
        }
        __syncwarp();
      };
      auto commit = [&](uint32_t bar) {
        if (elect_one_sync()) umma_commit(bar);
        __syncwarp();
      };

      // Work items follow one another on the same barriers; base[t] counts the tiles Q-tile slot t has consumed in
      // earlier items, q_count the Q loads, so every parity is a running count.
      uint32_t base0 = 0, base1 = 0;
      uint32_t q_count = 0;
      int item_cursor = 0;
      FaItem item = fa_next_working_item(p, item_cursor);
      while (ok && item.valid) {
        const int n0 = item.n0, n1 = item.n1;
        const int n_max = item.n_max;
        ok = mbar_wait(q_full, q_count & 1u, abort_word);
        ++q_count;
        // K_0: first scores of both tiles.
        if (ok) ok = mbar_wait(kv_full(slot), phase, abort_word);
        if (ok) {
          tc_fence_after();
          if (n0 > 0) issue_s(std::integral_constant<int, 0>{}, slot);
          if (n1 > 0) issue_s(std::integral_constant<int, 1>{}, slot);
          commit(kv_empty(slot));
          if (n_max == 1) commit(q_empty);   // the only S products of the item are in flight
          advance();
        }
        for (int j = 0; ok && j < n_max; ++j) {
          // ring now points at V_j; K_{j+1} follows it.
          const int v_slot = slot;
          const uint32_t v_phase = phase;
          advance();
          const int k_slot = slot;
          const uint32_t k_phase = phase;
          const bool has_next = j + 1 < n_max;
          if (has_next) advance();
          if (!mbar_wait(kv_full(v_slot), v_phase, abort_word)) { ok = false; break; }
          bool k_ready = false;
          auto tile_step = [&](auto tile_tag, int n_tiles, uint32_t tile_base) {
            constexpr int t = decltype(tile_tag)::value;
            if (j < n_tiles) {
              if (!mbar_wait_spin(p_part(t, 0), (tile_base + j) & 1u, abort_word)) { ok = false; return; }
              tc_fence_after();
              issue_pv_part(tile_tag, std::integral_constant<int, 0>{}, v_slot, j > 0);
              if constexpr (kPParts > 1) {
                if (!mbar_wait_spin(p_part(t, kPParts - 1), (tile_base + j) & 1u, abort_word)) { ok = false; return; }
                tc_fence_after();
                issue_pv_part(tile_tag, std::integral_constant<int, kPParts - 1>{}, v_slot, j > 0);
              }
            }
            if (j + 1 < n_tiles) {
              if (!k_ready) {
                if (!mbar_wait(kv_full(k_slot), k_phase, abort_word)) { ok = false; return; }
                tc_fence_after();
                k_ready = true;
              }
              issue_s(tile_tag, k_slot);
            }
          };
          tile_step(std::integral_constant<int, 0>{}, n0, base0);
          if (ok) tile_step(std::integral_constant<int, 1>{}, n1, base1);
          if (!ok) break;
          commit(kv_empty(v_slot));
          if (has_next) commit(kv_empty(k_slot));
          if (j + 2 == n_max) commit(q_empty);   // the last S products of the item are in flight: Q may be replaced
        }
        base0 += n0;
        base1 += n1;
        item = fa_next_working_item(p, item_cursor);
      }   // items
    }
  }
  } else {
    setmaxnreg_inc<200>();
    // ------------------------------------------------------------ softmax / rescale / epilogue
    const int t = (warp - 4) >> 2;          // Q tile of this warpgroup
    const int quarter = warp & 3;           // TMEM lane quarter this warp may access
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_sel + kColS0 + t * 128;
    const uint32_t o_addr = tmem_base + lane_sel + kColO0 + t * 128;
    uint32_t tiles_done = 0;   // S tiles of this Q-tile slot consumed so far, over all items (barrier parities)
    bool ok = true;
    for (int item_index = 0; ok; ++item_index) {
    // Only the row, the tile count and the mask limit stay live through the tile loop; the output coordinates are
    // recomputed after it (the softmax threads need every register for the 128 scores they hold).
    int row_base, my_tiles;
    {
      const FaItem item = fa_item(p, item_index);
      if (!item.valid) break;
      row_base = item.row_base;
      my_tiles = item.tiles(t);
    }
    const int row = row_base + t * kTileM + row_in_tile;   // query row inside the head
    // m_ref is the exponent reference the stored P, l and acc are scaled by; m_true is the running row
    // maximum. The reference moves to the new maximum only when the maximum has grown by more than
    // kRescaleThreshold (log2 units), so P stays below 2^8 and the rescale of acc is rare. acc / l and
    // m_ref + log2(l) do not depend on the reference chosen, and every rounding keeps its relative error.
    constexpr float kRescaleThreshold = 8.0f;
    float m_ref = -INFINITY, m_true = -INFINITY, l_run = 0.f;
    // Last visible key of this row, relative to key 0, clamped to 32 bits (rows see keys <= limit).
    long long limit64 = static_cast<long long>(p.kv_visible) - 1;
    if (p.causal && p.causal_offset + row < limit64) limit64 = p.causal_offset + row;
    const int row_limit = limit64 < -1 ? -1 : static_cast<int>(limit64);

    for (int j = 0; ok && j < my_tiles; ++j, ++tiles_done) {
      if (!mbar_wait(s_full(t), tiles_done & 1u, abort_word, 110 + t)) { ok = false; break; }
      tc_fence_after();
      const int key0 = j * kTileN;
      uint32_t r[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32 * c]));
      tmem_wait_ld();
      // Masking is needed only when the tile sticks out of the visible region of some row of the tile.
      const bool need_mask = (key0 + kTileN > p.kv_visible) ||
                             (p.causal && key0 + kTileN - 1 > p.causal_offset + row_base + t * kTileM);
      if (need_mask) {
        const int visible_in_tile = row_limit - key0;   // keys i <= visible_in_tile of this tile are visible
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i > visible_in_tile) r[i] = 0xff800000u;   // -inf
      }
      // Row maximum: four independent chains of 3-input max.
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
      const float raw_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      m_true = fmaxf(m_true, raw_max * p.scale_log2);     // scale > 0, so max commutes with the scaling
      float alpha = 1.0f;
      if (m_true - m_ref > kRescaleThreshold) {           // also taken when m_ref is still -inf
        alpha = exp2f(m_ref - m_true);
        m_ref = m_true;
      }
      const float m_exp = (m_ref == -INFINITY) ? 0.f : m_ref;
      // acc' = acc * alpha (rare) needs the PV product of the previous tile in TMEM and has to land before any PV of
      // this tile is issued, i.e. before the first half of P is published; the wait for that product sits there, behind
      // the first 64 exponentials, where it costs nothing.
      const unsigned long long scale2 = pack_f32x2(p.scale_log2, p.scale_log2), neg_m2 = pack_f32x2(-m_exp, -m_exp);
      unsigned long long sum2[4] = {0ull, 0ull, 0ull, 0ull};
      auto exp_phase = [&](auto masked_tag) {
      constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const unsigned long long x2 = fma_f32x2(pack_f32x2(__uint_as_float(r[32 * c + i]), __uint_as_float(r[32 * c + i + 1])), scale2, neg_m2);
          float x0, x1;
          unpack_f32x2(x2, x0, x1);
          // Every fourth pair of exponentials runs on the FMA pipe: the special-function pipe (ex2 and the 16-bit
          // conversions) is the busiest unit of the softmax warps.
          const bool poly = !kMasked && ((i >> 1) % kPolyPeriod) == kPolyPeriod - 1;
          const float e0 = poly ? ex2_poly(x0) : ex2_approx(x0);
          const float e1 = poly ? ex2_poly(x1) : ex2_approx(x1);
          sum2[(i >> 1) & 3] = add_f32x2(sum2[(i >> 1) & 3], pack_f32x2(e0, e1));
          if constexpr (kBf16) {
            __nv_bfloat162 v = __floats2bfloat162_rn(e0, e1);
            packed[i >> 1] = *reinterpret_cast<uint32_t *>(&v);
          } else {
            __half2 v = __floats2half2_rn(e0, e1);
            packed[i >> 1] = *reinterpret_cast<uint32_t *>(&v);
          }
        }
        tmem_st_32x16(s_addr + c * 16, packed);   // P aliases the first 64 columns of S
        if (c == kChunksPerPart - 1 && j > 0) {
          if (!mbar_wait(o_done(t), (tiles_done - 1) & 1u, abort_word, 112 + t)) { ok = false; return; }
          if (__any_sync(0xffffffffu, alpha != 1.0f)) {
            tc_fence_after();
#pragma unroll 1
            for (int oc = 0; oc < 4; ++oc) {
              uint32_t o[32];
              tmem_ld_32x32(o_addr + oc * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st_32x32(o_addr + oc * 32, o);
            }
          }
        }
        if ((c + 1) % kChunksPerPart == 0) {   // a half of P is complete: publish it
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(p_part(t, c / kChunksPerPart));
        }
      }
      };
      if (need_mask) exp_phase(std::true_type{});
      else exp_phase(std::false_type{});
      if (!ok) break;
      float s0, s1, s2, s3, s4, s5, s6, s7;
      unpack_f32x2(sum2[0], s0, s1); unpack_f32x2(sum2[1], s2, s3); unpack_f32x2(sum2[2], s4, s5); unpack_f32x2(sum2[3], s6, s7);
      l_run = l_run * alpha + (((s0 + s1) + (s2 + s3)) + ((s4 + s5) + (s6 + s7)));
    }

    // Finalize: out = acc * (1 / l), rounded once to the storage type.
    if (ok && my_tiles > 0) ok = mbar_wait(o_done(t), (tiles_done - 1) & 1u, abort_word, 114 + t);
    if (ok && row_base + t * kTileM < p.q_len) {
      tc_fence_after();
      float coefficient = 1.0f / l_run;
      if (p.zero_fully_masked && l_run == 0.f) coefficient = 0.f;
      const FaItem where = fa_item(p, item_index);
      const int bh = where.bh, b = where.b, h = where.h;
      const size_t out_row = p.out_token_major
                                 ? ((static_cast<size_t>(b) * p.q_len + row) * p.q_heads + h) * kHd
                                 : (static_cast<size_t>(bh) * p.q_len + row) * kHd;
      uint32_t r[128];
      if (my_tiles > 0) {
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_32x32(o_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32 * c]));
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 128; ++i) r[i] = 0u;
      }
      if (row < p.q_len) {
        uint16_t *dst = reinterpret_cast<uint16_t *>(p.out) + out_row;
        // 0 * (1/0): a row that saw no key and is not zero-filled is the canonical quiet NaN of the format.
        const bool nan_row = !(coefficient == coefficient) || (l_run == 0.f && !p.zero_fully_masked);
        const uint32_t nan_pair = kBf16 ? 0x7fc07fc0u : 0x7e007e00u;
#pragma unroll
        for (int i = 0; i < 128; i += 8) {
          uint32_t w[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float lo = __uint_as_float(r[i + 2 * k]) * coefficient, hi = __uint_as_float(r[i + 2 * k + 1]) * coefficient;
            if constexpr (kBf16) {
              __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
              w[k] = *reinterpret_cast<uint32_t *>(&v);
            } else {
              __half2 v = __floats2half2_rn(lo, hi);
              w[k] = *reinterpret_cast<uint32_t *>(&v);
            }
            if (nan_row) w[k] = nan_pair;
          }
          *reinterpret_cast<uint4 *>(dst + i) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      if (row < p.q_len) {
        const size_t stat = static_cast<size_t>(bh) * p.q_len + row;
        const float ln2 = 0.69314718055994530942f;  // back from the log2 domain
        if (p.lse) p.lse[stat] = (l_run == 0.f) ? -INFINITY : m_ref * ln2 + logf(l_run);
        if (p.row_max) p.row_max[stat] = m_true * ln2;
        // the carried sum is reported relative to the true maximum, as the reference carries it
        if (p.row_sum) p.row_sum[stat] = (l_run == 0.f) ? 0.f : l_run * exp2f(m_ref - m_true);
      }
    }
    }   // items
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
    if (threadIdx.x == 0) atomicExch(p.status, *abort_word);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Host mirror of kv_tiles_for.
int host_kv_tiles(const FaParams &p, long long row0) {
  long long last = static_cast<long long>(p.kv_visible) - 1;
  if (p.causal) last = std::min(last, p.causal_offset + row0 + (kTileM - 1));
  if (row0 >= p.q_len || last < 0) return 0;
  return static_cast<int>(last / kTileN) + 1;
}

// The plan of a launch shape: which items each of the `grid` CTAs runs, in order. Items are dealt head by head
// (all 256-row items of one (batch, head), heaviest first, each to the CTA with the least work so far), so the CTAs
// that share a head's K and V run at about the same time and find them in L2; the last heads' items are dealt in one
// pool by descending weight (longest-processing-time order), which evens out the finish times. The weight of an item
// is the KV steps of its longer Q tile plus a constant for the hand-over.
std::vector<std::vector<int>> build_plan_rows(const FaParams &p, int grid) {
  const int bh_count = p.batch * p.q_heads;
  std::vector<int> weight(p.num_pairs);
  for (int pair = 0; pair < p.num_pairs; ++pair) {
    const long long row0 = static_cast<long long>(pair) * 2 * kTileM;
    weight[pair] = std::max(host_kv_tiles(p, row0), host_kv_tiles(p, row0 + kTileM)) * 4 + 2;   // quarter steps; hand-over = half a step
  }
  auto weight_of = [&](int g) { return weight[p.num_pairs - 1 - g / bh_count]; };   // item g = pair rank * bh_count + bh
  std::vector<std::vector<int>> rows(grid);
  using Load = std::pair<long long, int>;   // (load, CTA): the least loaded CTA takes the next item
  std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
  for (int c = 0; c < grid; ++c) heap.push({0, c});
  auto deal = [&](int g) {
    Load least = heap.top();
    heap.pop();
    rows[least.second].push_back(g);
    heap.push({least.first + weight_of(g), least.second});
  };
  // The pooled tail holds about three items per CTA.
  const int tail_heads = std::min(bh_count, (3 * grid + p.num_pairs - 1) / p.num_pairs);
  const int head_major = bh_count - tail_heads;
  for (int bh = 0; bh < head_major; ++bh)
    for (int rank = 0; rank < p.num_pairs; ++rank) deal(rank * bh_count + bh);
  for (int rank = 0; rank < p.num_pairs; ++rank)
    for (int bh = head_major; bh < bh_count; ++bh) deal(rank * bh_count + bh);
  return rows;
}

// Plans live in device memory for the lifetime of the library (a few KiB each, at most kMaxPlansPerDevice per
// device; nothing is ever freed, so neither a launch in flight nor a captured graph can hold a stale pointer).
// Building one allocates and copies, so a shape's first launch should come outside stream capture; when that is not
// possible (a capture is in progress, or the device's cap is reached) the launch gets no plan and runs one CTA per item.
struct PlanKey {
  int device, num_pairs, bh_count, q_len, kv_visible, causal, grid;
  long long causal_offset;
  bool operator<(const PlanKey &o) const {
    return std::tie(device, num_pairs, bh_count, q_len, kv_visible, causal, grid, causal_offset) <
           std::tie(o.device, o.num_pairs, o.bh_count, o.q_len, o.kv_visible, o.causal, o.grid, o.causal_offset);
  }
};
struct PlanEntry { int *device_plan; int stride; };
constexpr int kMaxPlansPerDevice = 1024;

wb200_status get_plan(const FaParams &p, int grid, cudaStream_t stream, const int **plan, int *stride) {
  static std::mutex mutex;
  static std::map<PlanKey, PlanEntry> cache;
  static int plans_on_device[PerDeviceOnce::kMaxDevices] = {};
  PlanKey key{0, p.num_pairs, p.batch * p.q_heads, p.q_len, p.kv_visible, p.causal, grid, p.causal_offset};
  WB200_CUDA_CHECK(cudaGetDevice(&key.device));
  std::lock_guard<std::mutex> lock(mutex);
  auto found = cache.find(key);
  if (found != cache.end()) { *plan = found->second.device_plan; *stride = found->second.stride; return WB200_OK; }
  *plan = nullptr;
  *stride = 0;
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  WB200_CUDA_CHECK(cudaStreamIsCapturing(stream, &capture));
  const int slot = PerDeviceOnce::slot_of(key.device);
  if (capture != cudaStreamCaptureStatusNone || slot < 0 || plans_on_device[slot] >= kMaxPlansPerDevice) return WB200_OK;
  const std::vector<std::vector<int>> rows = build_plan_rows(p, grid);
  size_t longest = 0;
  for (const auto &row : rows) longest = std::max(longest, row.size());
  const int row_stride = static_cast<int>(longest) + 1;
  std::vector<int> flat(static_cast<size_t>(grid) * row_stride, -1);
  for (int c = 0; c < grid; ++c) std::copy(rows[c].begin(), rows[c].end(), flat.begin() + static_cast<size_t>(c) * row_stride);
  PlanEntry entry{nullptr, row_stride};
  WB200_CUDA_CHECK(cudaMalloc(&entry.device_plan, flat.size() * sizeof(int)));
  // Pageable source: the copy is staged before the call returns, and it is ordered before the launch on `stream`.
  WB200_CUDA_CHECK(cudaMemcpyAsync(entry.device_plan, flat.data(), flat.size() * sizeof(int), cudaMemcpyHostToDevice, stream));
  cache[key] = entry;
  plans_on_device[slot] += 1;
  *plan = entry.device_plan;
  *stride = row_stride;
  return WB200_OK;
}

}  // namespace

bool attention_fa_umma_supports(const AttentionArgs &a) {
  if (a.format != WB200_BF16 && a.format != WB200_F16) return false;
  if (a.head_dim != kHd || a.q_len <= 0 || a.kv_len <= 0 || a.batch <= 0) return false;
  if (a.kv_heads <= 0 || a.q_heads % a.kv_heads != 0) return false;
  if ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v) |
       reinterpret_cast<uintptr_t>(a.out)) & 15u)
    return false;
  return true;
}

wb200_status launch_attention_fa_umma(const AttentionArgs &a, int sm_count, int *device_status,
                                      cudaStream_t stream) {
  if (sm_count <= 0) sm_count = 148;
  if (!attention_fa_umma_supports(a))
    return fail(WB200_ERR_UNSUPPORTED, "attention request outside the tcgen05 prefill kernel's domain");
  CUtensorMap tq, tk, tv;
  const uint64_t row_pitch = kHd * 2;
  wb200_status st = encode_tmap_3d(&tq, a.q, a.format, kHd, a.q_len, static_cast<uint64_t>(a.batch) * a.q_heads,
                                   row_pitch, row_pitch * a.q_len, 64, kTileM);
  if (st != WB200_OK) return st;
  st = encode_tmap_3d(&tk, a.k, a.format, kHd, a.kv_len, static_cast<uint64_t>(a.batch) * a.kv_heads, row_pitch,
                      row_pitch * a.kv_len, 64, kTileN);
  if (st != WB200_OK) return st;
  st = encode_tmap_3d(&tv, a.v, a.format, kHd, a.kv_len, static_cast<uint64_t>(a.batch) * a.kv_heads, row_pitch,
                      row_pitch * a.kv_len, 64, kTileN);
  if (st != WB200_OK) return st;

  FaParams p;
  p.batch = a.batch; p.q_heads = a.q_heads; p.kv_heads = a.kv_heads; p.group = a.q_heads / a.kv_heads;
  p.q_len = a.q_len; p.kv_len = a.kv_len;
  int64_t visible = a.kv_valid < a.kv_len ? a.kv_valid : a.kv_len;
  if (visible < 0) visible = 0;
  p.kv_visible = static_cast<int>(visible);
  p.causal = a.causal;
  p.causal_offset = a.causal_offset;
  p.zero_fully_masked = a.zero_fully_masked;
  p.out_format = a.format;
  p.bf16 = a.format == WB200_BF16;
  p.num_pairs = (a.q_len + 2 * kTileM - 1) / (2 * kTileM);
  if (static_cast<long long>(p.num_pairs) * a.batch * a.q_heads > (1LL << 24))
    return fail(WB200_ERR_UNSUPPORTED, "more than 2^24 (batch, head, 256-row) items in one attention launch");
  p.out_token_major = a.out_token_major;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.out = a.out; p.lse = a.lse; p.row_max = a.row_max; p.row_sum = a.row_sum;
  p.status = device_status;
  p.plan = nullptr;
  p.plan_stride = 0;

  static PerDeviceOnce attributes;
  st = attributes.run([]() -> wb200_status {
    WB200_CUDA_CHECK(cudaFuncSetAttribute(fa_umma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(FaSmem::kBytes)));
    WB200_CUDA_CHECK(cudaFuncSetAttribute(fa_umma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(FaSmem::kBytes)));
    return WB200_OK;
  });
  if (st != WB200_OK) return st;
  // Persistent grid: one CTA per SM walks its share of the items, so the first loads and scores of an item overlap the
  // softmax tail and write-out of the previous one. With no more items than SMs, or when no plan can be had (see
  // get_plan), one CTA per item.
  const int items = p.num_pairs * a.batch * a.q_heads;
  int grid = items;
  if (items > sm_count) {
    st = get_plan(p, sm_count, stream, &p.plan, &p.plan_stride);
    if (st != WB200_OK) return st;
    if (p.plan) grid = sm_count;
  }
  // The persistent grid is launched as clusters of two CTAs. The kernel makes no use of the cluster; the point is the
  // placement: a pair takes both SMs of a TPC, so the SMs a persistent grid leaves free are whole TPCs, where the CTA
  // pairs of a kernel that runs beside it (the sum over shards of a decoder layer, whose neighbours are CTA-pair GEMMs)
  // still fit. With single CTAs the free SMs are scattered and such pairs wait for the whole grid to end.
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(kFaThreads);
  config.dynamicSmemBytes = FaSmem::kBytes;
  config.stream = stream;
  cudaLaunchAttribute cluster;
  cluster.id = cudaLaunchAttributeClusterDimension;
  cluster.val.clusterDim.x = 2; cluster.val.clusterDim.y = 1; cluster.val.clusterDim.z = 1;
  if (p.plan && grid % 2 == 0) {
    config.attrs = &cluster;
    config.numAttrs = 1;
  }
  if (a.format == WB200_BF16)
    WB200_CUDA_CHECK(cudaLaunchKernelEx(&config, fa_umma_kernel<true>, tq, tk, tv, p));
  else
    WB200_CUDA_CHECK(cudaLaunchKernelEx(&config, fa_umma_kernel<false>, tq, tk, tv, p));
  return WB200_OK;
}

}  // namespace wb200
