// Flash-attention prefill on CUDA cores, f32 arithmetic throughout: the path for f32 storage (where
// the 1e-5 parity bound rules out tensor-core inputs narrower than f32) and for shapes the tcgen05
// kernel does not take. One warp owns one query row and walks the keys in tiles of 32 that the block's sixteen
// rows share through shared memory, applying the reference's online update literally
// (lib/Wafer/Transforms/Linalg/OnlineAttentionDecomposition.cpp:568-594):
//   s = (q.k)*scale (+mask); m' = max(m, max s); m_e = (m' == -inf ? 0 : m'); alpha = ExpLp(m - m_e);
//   l = l*alpha + sum ExpLp(s - m_e); acc = acc*alpha + round_to_storage(P) V
// and the finalize acc * (1/l) of OnlineAttentionMaterialization.cpp:196-262. ExpLp is
// exp2(x * log2e) in f32 (lib/Wafer/Simulator/Reference/ManagedReferenceTargetModel.cpp:265-270).
#include "kernels.h"

namespace wb200 {
namespace {

constexpr int kWarpsPerBlock = 16;   // query rows of one head per block; they share every staged K / V tile
constexpr int kMaxDPerLane = 8;      // head_dim <= 256
constexpr int kTileKeys = 32;

struct SimtParams {
  AttentionArgs a;
  int group;
  int kv_visible;
  int vector;   // K and V are 16-byte aligned: the staging loop may use wide loads
};

__device__ __forceinline__ float exp_lp(float x) { return exp2f(__fmul_rn(x, 0x1.715476p+0f)); }

// Shared memory: q rows [kWarpsPerBlock][D], the K tile [32][D + 1] (the pad keeps the per-lane row reads of the score
// loop on distinct banks) and the V tile [32][D], all widened to f32 once per block instead of once per query row.
// kD fixes head_dim at compile time (0: runtime) so the score and PV loops unroll and their shared-memory reads pipeline.
template <int kD>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) fa_simt_kernel(const SimtParams p) {
  const AttentionArgs &a = p.a;
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerBlock + warp;
  const int bh = blockIdx.y;
  const int b = bh / a.q_heads, h = bh % a.q_heads;
  const int D = kD ? kD : a.head_dim;
  const int per_lane = D / 32;
  const bool active = row < a.q_len;
  float *q_smem = smem, *k_tile = smem + kWarpsPerBlock * D, *v_tile = k_tile + kTileKeys * (D + 1);

  const size_t q_off = (static_cast<size_t>(bh) * a.q_len + (active ? row : 0)) * D;
  const size_t kv_off = (static_cast<size_t>(b) * a.kv_heads + h / p.group) * static_cast<size_t>(a.kv_len) * D;
  const uint8_t *q = static_cast<const uint8_t *>(a.q);
  const uint8_t *k = static_cast<const uint8_t *>(a.k);
  const uint8_t *v = static_cast<const uint8_t *>(a.v);
  float *my_q = q_smem + warp * D;
  if (active)
    for (int d = lane; d < D; d += 32) my_q[d] = widen_bits(load_element_bits(q, q_off + d, a.format), a.format);

  auto visible_of = [&](int r) {
    long long last = static_cast<long long>(p.kv_visible) - 1;
    if (a.causal && a.causal_offset + r < last) last = a.causal_offset + r;
    return last < 0 ? 0 : static_cast<int>(last + 1);
  };
  const int visible = active ? visible_of(row) : 0;
  // the last row of the block sees the most keys
  const int last_row = min(static_cast<int>(blockIdx.x) * kWarpsPerBlock + kWarpsPerBlock - 1, a.q_len - 1);
  const int block_visible = visible_of(last_row);

  float m_run = -INFINITY, l_run = 0.0f;
  float acc[kMaxDPerLane];
#pragma unroll
  for (int i = 0; i < kMaxDPerLane; ++i) acc[i] = 0.0f;

  for (int key0 = 0; key0 < block_visible; key0 += kTileKeys) {
    __syncthreads();   // the previous tile has been consumed (and, first time round, the q rows are written)
    const int tile_keys = min(kTileKeys, block_visible - key0);
    // four consecutive elements per thread and step (head_dim is a multiple of 32): the loads of a step are issued
    // together, 128 bits wide for f32 storage and 64 bits wide for the 16-bit formats
    const int quads = p.vector ? tile_keys * D / 4 : 0;
    for (int e = threadIdx.x; e < quads; e += kWarpsPerBlock * 32) {
      const int j = (e * 4) / D, d = e * 4 - j * D;
      const size_t at = kv_off + static_cast<size_t>(key0 + j) * D + d;
      float kf[4], vf[4];
      if (a.format == WB200_F32) {
        const float4 kq = *reinterpret_cast<const float4 *>(k + at * 4), vq = *reinterpret_cast<const float4 *>(v + at * 4);
        kf[0] = kq.x; kf[1] = kq.y; kf[2] = kq.z; kf[3] = kq.w;
        vf[0] = vq.x; vf[1] = vq.y; vf[2] = vq.z; vf[3] = vq.w;
      } else {
        const uint2 kq = *reinterpret_cast<const uint2 *>(k + at * 2), vq = *reinterpret_cast<const uint2 *>(v + at * 2);
        kf[0] = widen_bits(kq.x & 0xffffu, a.format); kf[1] = widen_bits(kq.x >> 16, a.format);
        kf[2] = widen_bits(kq.y & 0xffffu, a.format); kf[3] = widen_bits(kq.y >> 16, a.format);
        vf[0] = widen_bits(vq.x & 0xffffu, a.format); vf[1] = widen_bits(vq.x >> 16, a.format);
        vf[2] = widen_bits(vq.y & 0xffffu, a.format); vf[3] = widen_bits(vq.y >> 16, a.format);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        k_tile[j * (D + 1) + d + i] = kf[i];
        v_tile[j * D + d + i] = vf[i];
      }
    }
    if (!p.vector)
      for (int e = threadIdx.x; e < tile_keys * D; e += kWarpsPerBlock * 32) {
        const int j = e / D, d = e - j * D;
        const size_t at = kv_off + static_cast<size_t>(key0 + j) * D + d;
        k_tile[j * (D + 1) + d] = widen_bits(load_element_bits(k, at, a.format), a.format);
        v_tile[j * D + d] = widen_bits(load_element_bits(v, at, a.format), a.format);
      }
    __syncthreads();
    if (key0 >= visible) continue;   // this row's keys ended in an earlier tile (causal rows above the block's last)
    const int key = key0 + lane;
    float s = -INFINITY;
    if (key < visible) {
      float dot = 0.0f;
      const float *k_row = k_tile + lane * (D + 1);
#pragma unroll 16
      for (int d = 0; d < D; ++d) dot = __fmaf_rn(my_q[d], k_row[d], dot);
      s = __fmul_rn(dot, a.scale);
    }
    float tile_max = s;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, off));
    const float m_new = fmaxf(tile_max, m_run);
    const float m_exp = (m_new == -INFINITY) ? 0.0f : m_new;
    const float alpha = exp_lp(__fsub_rn(m_run, m_exp));
    const float prob = exp_lp(__fsub_rn(s, m_exp));
    float tile_sum = prob;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) tile_sum += __shfl_xor_sync(0xffffffffu, tile_sum, off);
    l_run = __fadd_rn(__fmul_rn(l_run, alpha), tile_sum);
    m_run = m_new;
    // P is rounded to the storage type of V before the PV contraction.
    const float prob_rounded = widen_bits(narrow_bits(prob, a.format), a.format);
#pragma unroll
    for (int i = 0; i < kMaxDPerLane; ++i) acc[i] = __fmul_rn(acc[i], alpha);
    const int count = min(kTileKeys, visible - key0);
#pragma unroll 8
    for (int j = 0; j < count; ++j) {
      const float pj = __shfl_sync(0xffffffffu, prob_rounded, j);
      const float *v_row = v_tile + j * D;
#pragma unroll
      for (int i = 0; i < kMaxDPerLane; ++i)
        if (i < per_lane) acc[i] = __fmaf_rn(pj, v_row[i * 32 + lane], acc[i]);
    }
  }
  if (!active) return;

  float coefficient = __fdiv_rn(1.0f, l_run);
  if (a.zero_fully_masked && l_run == 0.0f) coefficient = 0.0f;
  uint8_t *out = static_cast<uint8_t *>(a.out);
  const size_t out_off = a.out_token_major ? ((static_cast<size_t>(b) * a.q_len + row) * a.q_heads + h) * D : q_off;
#pragma unroll
  for (int i = 0; i < kMaxDPerLane; ++i)
    if (i < per_lane)
      store_element_bits(out, out_off + i * 32 + lane, a.format, narrow_bits(__fmul_rn(acc[i], coefficient), a.format));
  if (lane == 0) {
    const size_t stat = static_cast<size_t>(bh) * a.q_len + row;
    if (a.lse) a.lse[stat] = (l_run == 0.0f) ? -INFINITY : m_run + logf(l_run);
    if (a.row_max) a.row_max[stat] = m_run;
    if (a.row_sum) a.row_sum[stat] = l_run;
  }
}

}  // namespace

wb200_status launch_attention_fa_simt(const AttentionArgs &a, cudaStream_t stream) {
  if (!is_float_format(a.format)) return fail(WB200_ERR_UNSUPPORTED, "attention admits f16, bf16 and f32 storage");
  if (a.head_dim <= 0 || a.head_dim % 32 != 0 || a.head_dim > 32 * kMaxDPerLane)
    return fail(WB200_ERR_UNSUPPORTED, "head_dim must be a multiple of 32 up to 256");
  if (a.kv_heads <= 0 || a.q_heads % a.kv_heads != 0 || a.q_len <= 0 || a.kv_len <= 0 || a.batch <= 0)
    return fail(WB200_ERR_INVALID_ARGUMENT, "invalid attention extents");
  SimtParams p;
  p.a = a;
  p.group = a.q_heads / a.kv_heads;
  int64_t visible = a.kv_valid < a.kv_len ? a.kv_valid : a.kv_len;
  p.kv_visible = visible < 0 ? 0 : static_cast<int>(visible);
  dim3 grid((a.q_len + kWarpsPerBlock - 1) / kWarpsPerBlock, a.batch * a.q_heads);
  const size_t smem_bytes = (static_cast<size_t>(kWarpsPerBlock) * a.head_dim + kTileKeys * (a.head_dim + 1) + kTileKeys * a.head_dim) * sizeof(float);
  // wide staging loads need 16-byte aligned K / V bases; head_dim % 32 == 0 keeps every row aligned
  p.vector = ((reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v)) & 15) == 0;
#define WB200_SIMT_LAUNCH(KD)                                                                                                  \
  do {                                                                                                                         \
    if (smem_bytes > 48 * 1024)                                                                                                \
      WB200_CUDA_CHECK(cudaFuncSetAttribute(fa_simt_kernel<KD>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_bytes))); \
    fa_simt_kernel<KD><<<grid, kWarpsPerBlock * 32, smem_bytes, stream>>>(p);                                                  \
  } while (0)
  if (a.head_dim == 64) WB200_SIMT_LAUNCH(64);
  else if (a.head_dim == 128) WB200_SIMT_LAUNCH(128);
  else WB200_SIMT_LAUNCH(0);
#undef WB200_SIMT_LAUNCH
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

}  // namespace wb200
