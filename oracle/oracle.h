/* oracle.h - CPU restatement of the reference's numeric path. TEST INFRASTRUCTURE ONLY.
 *
 * Nothing in the product (vibe_compiler_b200/, libwb200.so) may include, link or call this. It is
 * used by tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline legs as the checker and
 * as the timed CPU baseline.
 *
 * Parity status: the scalar formats, the physical layout, the formal GEMM, and the managed
 * convert / elementwise / reduce commands are pinned against the known-answer vectors of the
 * reference's own unit tests (tests/golden/reference_kats.json lists each vector with the reference
 * test file and line it was read from). The attention functions have no bit-level vector in the
 * reference ("tolerance-pinned"): they restate the published update order and are checked against
 * PyTorch scaled-dot-product attention the way the reference's integration tests do.
 * Transcendental elementwise operations use the host libm, as the reference does: parity unpinned
 * at bit level for those.
 */
#ifndef WB200_ORACLE_H
#define WB200_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* formats / layouts use the ordinals of include/wb200.h (which are the reference's). */

typedef struct oracle_geometry {
  int64_t element_bytes, compact_bytes, physical_elements, physical_bytes;
  int64_t c_block, cx_blocks, c0, aligned_c, outer_elements, block_outer_elements;
  int64_t outer_slice_stride_elements, bank_align_elements;
} oracle_geometry;

int oracle_physical_geometry(int format, int layout, int rank, const uint64_t *shape, oracle_geometry *out);
/* bit offset of a logical coordinate (StaticPhysicalTensorOffsetCalculator::getBitOffset) */
int64_t oracle_physical_bit_offset(int format, int layout, int rank, const uint64_t *shape, const int64_t *index);
int oracle_pack(int format, int layout, int rank, const uint64_t *shape, const uint8_t *compact,
                const uint8_t *storage_template, uint8_t *storage_out);
int oracle_unpack(int format, int layout, int rank, const uint64_t *shape, const uint8_t *storage, uint8_t *compact_out);

/* scalar conversions on raw bits */
uint32_t oracle_widen_to_f32_bits(int format, uint32_t bits);
/* RNE narrowing of an f32 value; NaN -> canonical quiet NaN of the destination */
uint32_t oracle_narrow_from_f32_bits(int format, uint32_t f32_bits);

/* Formal GEMM on compact logical arrays (element = 2 or 4 bytes little endian). psum may be NULL. */
int oracle_formal_gemm(int in_format, int out_format, int batch, int m, int k, int n, int lhs_transposed,
                       int rhs_transposed, const void *lhs, const void *rhs, const float *psum, void *out, int threads);

/* Managed-reference commands on compact arrays. Return 0 ok, 3 NaN domain, 2 unsupported. */
int oracle_elementwise(int op, int format, int64_t count, const void *in0, const void *in1, void *out);
int oracle_convert(int src_format, int dst_format, int64_t count, const void *src, void *dst);
int oracle_reduce(int op, int format, int rank, const uint64_t *shape, uint32_t reduced_mask, const void *src, void *dst);

/* Attention on compact [batch, heads, len, dim] arrays. tile_n = keys per online-update step. */
typedef struct oracle_attention {
  int batch, q_heads, kv_heads, q_len, kv_len, head_dim;
  int format, causal, zero_fully_masked;
  float scale;
  int64_t query_start, key_start, key_end; /* key_end <= 0: key_start + kv_len */
  const void *q, *k, *v;
  void *out;
  float *lse, *row_max, *row_sum; /* optional */
  int tile_n;
  int threads;
} oracle_attention;
int oracle_attention_fa(const oracle_attention *p);
/* splits >= 1 contiguous KV intervals, each an independent online pass, left-folded in order. */
int oracle_attention_fd(const oracle_attention *p, int splits);
/* Un-finalized state of the whole visible range: state[(b*Hq+h)*(D+2)] = acc[D], m, l */
int oracle_attention_fd_state(const oracle_attention *p, int splits, float *state);
int oracle_attention_fd_merge(int rows, int head_dim, int format, int zero_fully_masked, int shards,
                              const float *states, void *out, float *lse);

/* GEMM region with epilogue: out = narrow(epi(widen(A) x widen(B))) with k-ascending f32 FMA chains.
 * epilogue 0 none, 1 +bias, 2 gelu_erf(+bias). */
int oracle_gemm_epilogue(int in_format, int out_format, int m, int n, int k, int lhs_transposed, int rhs_transposed,
                         int epilogue, const void *a, const void *b, const float *bias, void *out, int threads);

/* Comparator statistics (ProgramTensorComparison.cpp:20-52): */
typedef struct oracle_comparison {
  uint64_t element_count, exact_count, mismatch_count;
  double mean_abs, p99_abs, p999_abs, max_abs, cosine, relative_l2, mean_ulp;
  uint64_t p99_ulp, p999_ulp, max_ulp;
  int finite; /* 0 when a non-finite value was met (the reference rejects those) */
} oracle_comparison;
int oracle_compare(int format, int64_t count, const void *actual, const void *expected, double atol, double rtol,
                   oracle_comparison *out);

#ifdef __cplusplus
}
#endif
#endif
