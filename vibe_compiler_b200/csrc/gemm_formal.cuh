// The formal GEMM's 64 x 64 tile as a device function, shared by the command's own kernel (gemm_formal.cu) and by the
// command-run kernel (tensor_ops.cu), plus the address helpers and the host-side choice of the variant.
#pragma once
#include "kernels.h"

namespace wb200 {
namespace {

// Physical element index of element (batch, row, col) of a logical [batch, rows, cols] GEMM operand without the
// divisions of the general row-major-to-physical map (64-bit divisions dominated the kernels' time): the operand's
// coordinates are already known. Cx of rank 2 / 3 and NCx of rank 3 are resolved here, anything else falls back.
// kResolved: the host has checked that every operand is in one of the resolved forms, so the general map (and its
// divisions, which otherwise bloat the unrolled loops past the instruction cache) is not even compiled in.
template <bool kResolved = false>
__device__ __forceinline__ int64_t operand_index(const LayoutMap &map, int64_t batch, int64_t rows, int64_t row, int64_t cols, int64_t col) {
  const int64_t outer_all = batch * rows + row;
  if (map.layout == WB200_LAYOUT_TENSOR || map.layout == WB200_LAYOUT_NTENSOR) return outer_all * cols + col;
  const bool ncx3 = map.layout == WB200_LAYOUT_NCX && map.rank == 3;
  const bool cx = map.layout == WB200_LAYOUT_CX && (map.rank == 2 || map.rank == 3);
  if (!kResolved && (!(ncx3 || cx) || (map.c_block & (map.c_block - 1)) != 0)) return physical_index(map, outer_all * cols + col);
  const int64_t base = ncx3 ? batch * map.outer_slice_stride : 0;
  const int64_t outer = ncx3 ? row : outer_all;
  const int64_t full_c = map.cx_blocks * map.c_block;
  if (col < full_c) {
    const int shift = __ffsll(map.c_block) - 1;
    return base + (col >> shift) * (map.block_outer_elements * map.c_block) + outer * map.c_block + (col & (map.c_block - 1));
  }
  return base + map.cx_blocks * map.block_outer_elements * map.c_block + outer * map.c0 + (col - full_c);
}

// For Tensor layouts and for Cx / NCx operands without a channel tail the physical index separates into a part that
// depends on the row only and a part that depends on the column only: index = row_part + col_part. The tiled kernel uses
// this to keep the per-element address arithmetic out of its k loop.
__host__ __device__ inline bool separable_layout(const LayoutMap &m) {
  if (m.layout == WB200_LAYOUT_TENSOR || m.layout == WB200_LAYOUT_NTENSOR) return true;
  const bool ncx3 = m.layout == WB200_LAYOUT_NCX && m.rank == 3, cx = m.layout == WB200_LAYOUT_CX && (m.rank == 2 || m.rank == 3);
  return (ncx3 || cx) && (m.c_block & (m.c_block - 1)) == 0 && m.c0 == 0;
}
__device__ __forceinline__ int64_t row_part(const LayoutMap &map, int64_t batch, int64_t rows, int64_t row, int64_t cols) {
  if (map.layout == WB200_LAYOUT_TENSOR || map.layout == WB200_LAYOUT_NTENSOR) return (batch * rows + row) * cols;
  if (map.layout == WB200_LAYOUT_NCX) return batch * map.outer_slice_stride + row * map.c_block;
  return (batch * rows + row) * map.c_block;
}
__device__ __forceinline__ int64_t col_part(const LayoutMap &map, int64_t col) {
  if (map.layout == WB200_LAYOUT_TENSOR || map.layout == WB200_LAYOUT_NTENSOR) return col;
  const int shift = __ffsll(map.c_block) - 1;
  return (col >> shift) * (map.block_outer_elements * map.c_block) + (col & (map.c_block - 1));
}

// Register-tiled variant for commands with at least 32 x 32 outputs: a 64 x 64 output tile per 256-thread block,
// 4 x 4 outputs per thread, 16-wide k panels staged through shared memory in k-major order. Each output still sees
// exactly the chain acc = fma(lhs[k], rhs[k], acc) for k = 0, 1, ... (the k tail is not padded: fma(0, 0, -0) would
// turn a negative zero into +0), so the bits equal the one-output-per-thread kernel's. CUDA-core bound:
// m * n * k FMAs per command, 0.5 shared-memory loads per FMA.
constexpr int kBlockM = 64, kBlockN = 64, kPanelK = 16;

// kWide (implies kSeparable; 16-bit operands, both untransposed, 16-byte aligned bases, k and n multiples of 8): a thread
// stages eight consecutive elements with one 128-bit load - threads 0..127 a run of lhs along k, threads 128..255 a run of
// rhs along n - instead of eight 2-byte loads with eight addresses.
// One 64 x 64 output tile by 256 threads (`tid` 0 .. 255) through the caller's two shared-memory panels. Every thread of
// the block must make the call (it contains block barriers); threads with `active` false only take part in the barriers,
// which lets a larger block work on several tiles side by side, each 256-thread group with panels of its own.
template <bool kResolved, bool kSeparable, bool kWide>
__device__ __forceinline__ void gemm_formal_tile(const GemmFormalArgs &a, int batch, int row0, int col0, int tid, bool active,
                                                 float (*lhs_panel)[kBlockM + 4], float (*rhs_panel)[kBlockN + 4]) {
  const int tx = tid & 15, ty = tid >> 4;
  const int m_extent = active ? a.m : 0, n_extent = active ? a.n : 0;   // an inactive thread finds every element out of range
  float acc[4][4];   // outputs (row0 + ty * 4 + i, col0 + tx * 4 + j)
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  // Staging: 64 x 16 lhs and 16 x 64 rhs elements per panel, 4 + 4 per thread; consecutive threads take consecutive
  // elements of the operand's fastest logical dimension. Element e of a thread: flat index tid + 256 e.
  int l_r[4], l_kk[4], r_c[4], r_kk[4];
  int64_t l_fixed[4], r_fixed[4];   // kSeparable: the part of the address that does not move with the panel
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int index = tid + e * 256;
    if (a.lhs_transposed) { l_r[e] = index & 63; l_kk[e] = index >> 6; } else { l_kk[e] = index & 15; l_r[e] = index >> 4; }
    if (a.rhs_transposed) { r_kk[e] = index & 15; r_c[e] = index >> 4; } else { r_c[e] = index & 63; r_kk[e] = index >> 6; }
    if (kSeparable) {
      // lhs element (m index row0 + r, k index k0 + kk); rhs element (k index k0 + kk, n index col0 + c)
      l_fixed[e] = a.lhs_transposed ? col_part(a.lhs_map, row0 + l_r[e]) : row_part(a.lhs_map, batch, a.m, row0 + l_r[e], a.k);
      r_fixed[e] = a.rhs_transposed ? row_part(a.rhs_map, batch, a.n, col0 + r_c[e], a.k) : col_part(a.rhs_map, col0 + r_c[e]);
    }
  }
  // kWide staging roles: lhs run = row (tid >> 1) of the tile, k offset (tid & 1) * 8; rhs run = k row ((tid - 128) >> 3),
  // columns ((tid - 128) & 7) * 8 .. + 7.
  const bool wide_lhs = tid < 128;
  const int wide_row = wide_lhs ? (tid >> 1) : ((tid - 128) >> 3);
  const int wide_off = wide_lhs ? (tid & 1) * 8 : ((tid - 128) & 7) * 8;
  int64_t wide_fixed = 0;
  if (kWide) wide_fixed = wide_lhs ? row_part(a.lhs_map, batch, a.m, row0 + wide_row, a.k) : col_part(a.rhs_map, col0 + wide_off);
  for (int k0 = 0; k0 < a.k; k0 += kPanelK) {
    if (kWide) {
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (wide_lhs) {
        const int k = k0 + wide_off;
        if (row0 + wide_row < m_extent && k < a.k)
          raw = *reinterpret_cast<const uint4 *>(a.lhs + (wide_fixed + col_part(a.lhs_map, k)) * 2);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          lhs_panel[wide_off + 2 * i][wide_row] = widen_bits(w[i] & 0xffffu, a.in_format);
          lhs_panel[wide_off + 2 * i + 1][wide_row] = widen_bits(w[i] >> 16, a.in_format);
        }
      } else {
        const int k = k0 + wide_row;
        if (col0 + wide_off < n_extent && k < a.k)
          raw = *reinterpret_cast<const uint4 *>(a.rhs + (wide_fixed + row_part(a.rhs_map, batch, a.k, k, a.n)) * 2);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        float4 lo, hi;
        lo.x = widen_bits(w[0] & 0xffffu, a.in_format); lo.y = widen_bits(w[0] >> 16, a.in_format);
        lo.z = widen_bits(w[1] & 0xffffu, a.in_format); lo.w = widen_bits(w[1] >> 16, a.in_format);
        hi.x = widen_bits(w[2] & 0xffffu, a.in_format); hi.y = widen_bits(w[2] >> 16, a.in_format);
        hi.z = widen_bits(w[3] & 0xffffu, a.in_format); hi.w = widen_bits(w[3] >> 16, a.in_format);
        *reinterpret_cast<float4 *>(&rhs_panel[wide_row][wide_off]) = lo;
        *reinterpret_cast<float4 *>(&rhs_panel[wide_row][wide_off + 4]) = hi;
      }
    } else {
  #pragma unroll
      for (int e = 0; e < 4; ++e) {
        float value = 0.0f;
        const int k = k0 + l_kk[e];
        if (row0 + l_r[e] < m_extent && k < a.k) {
          int64_t at;
          if (kSeparable) at = l_fixed[e] + (a.lhs_transposed ? row_part(a.lhs_map, batch, a.k, k, a.m) : col_part(a.lhs_map, k));
          else at = a.lhs_transposed ? operand_index<kResolved>(a.lhs_map, batch, a.k, k, a.m, row0 + l_r[e])
                                     : operand_index<kResolved>(a.lhs_map, batch, a.m, row0 + l_r[e], a.k, k);
          value = widen_bits(load_element_bits(a.lhs, at, a.in_format), a.in_format);
        }
        lhs_panel[l_kk[e]][l_r[e]] = value;
      }
  #pragma unroll
      for (int e = 0; e < 4; ++e) {
        float value = 0.0f;
        const int k = k0 + r_kk[e];
        if (col0 + r_c[e] < n_extent && k < a.k) {
          int64_t at;
          if (kSeparable) at = r_fixed[e] + (a.rhs_transposed ? col_part(a.rhs_map, k) : row_part(a.rhs_map, batch, a.k, k, a.n));
          else at = a.rhs_transposed ? operand_index<kResolved>(a.rhs_map, batch, a.n, col0 + r_c[e], a.k, k)
                                     : operand_index<kResolved>(a.rhs_map, batch, a.k, k, a.n, col0 + r_c[e]);
          value = widen_bits(load_element_bits(a.rhs, at, a.in_format), a.in_format);
        }
        rhs_panel[r_kk[e]][r_c[e]] = value;
      }
    }
    __syncthreads();
    const int k_count = min(kPanelK, a.k - k0);
    for (int kk = 0; kk < k_count; ++kk) {
      const float4 lv = *reinterpret_cast<const float4 *>(&lhs_panel[kk][ty * 4]);
      const float4 rv = *reinterpret_cast<const float4 *>(&rhs_panel[kk][tx * 4]);
      const float l[4] = {lv.x, lv.y, lv.z, lv.w}, r[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(l[i], r[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int row = row0 + ty * 4 + i, col = col0 + tx * 4 + j;
      if (row < m_extent && col < n_extent) {
        float value = acc[i][j];
        if (a.has_psum) value = __fadd_rn(value, __uint_as_float(load_element_bits(a.psum, operand_index<kResolved>(a.psum_map, batch, a.m, row, a.n, col), WB200_F32)));
        store_element_bits(a.dst, operand_index<kResolved>(a.dst_map, batch, a.m, row, a.n, col), a.out_format, narrow_bits(value, a.out_format));
      }
    }
}


// Which instantiation a command takes: 3 wide staging, 2 separable addresses, 1 resolved layouts, 0 the general map.
inline int gemm_formal_variant(const GemmFormalArgs &args) {
  auto resolved = [](const LayoutMap &m) {
    if (m.layout == WB200_LAYOUT_TENSOR || m.layout == WB200_LAYOUT_NTENSOR) return true;
    const bool ncx3 = m.layout == WB200_LAYOUT_NCX && m.rank == 3, cx = m.layout == WB200_LAYOUT_CX && (m.rank == 2 || m.rank == 3);
    return (ncx3 || cx) && (m.c_block & (m.c_block - 1)) == 0;
  };
  const bool all_resolved = resolved(args.lhs_map) && resolved(args.rhs_map) && resolved(args.dst_map) && (!args.has_psum || resolved(args.psum_map));
  const bool separable = all_resolved && separable_layout(args.lhs_map) && separable_layout(args.rhs_map);
  const bool wide = separable && args.in_format != WB200_F32 && !args.lhs_transposed && !args.rhs_transposed && args.k % 8 == 0 &&
                    args.n % 8 == 0 && ((reinterpret_cast<uintptr_t>(args.lhs) | reinterpret_cast<uintptr_t>(args.rhs)) & 15) == 0;
  return wide ? 3 : separable ? 2 : all_resolved ? 1 : 0;
}

}  // namespace
}  // namespace wb200
