// Internal launcher interface between the C-ABI layer (api.cu) and the kernel translation units.
// All pointers are device pointers. Launchers enqueue on `stream` and never synchronise.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "common.cuh"

namespace wb200 {

// Function attributes (the opt-in to more than 48 KiB of dynamic shared memory) belong to a device, not to the
// process: a launcher keeps one of these per kernel family and runs its set-up the first time each device is used.
class PerDeviceOnce {
 public:
  static constexpr int kMaxDevices = 64;
  // Returns the table slot of `device`, or -1 when the index lies outside the table (the set-up then runs on every call).
  static int slot_of(int device) { return (device >= 0 && device < kMaxDevices) ? device : -1; }
  template <typename Setup>
  wb200_status run(Setup &&setup) {
    int device = -1;
    WB200_CUDA_CHECK(cudaGetDevice(&device));
    const int slot = slot_of(device);
    std::lock_guard<std::mutex> lock(mutex_);
    if (slot >= 0 && done_[slot]) return WB200_OK;
    const wb200_status st = setup();
    if (st == WB200_OK && slot >= 0) done_[slot] = true;
    return st;
  }
  bool done_for(int device) {
    std::lock_guard<std::mutex> lock(mutex_);
    const int slot = slot_of(device);
    return slot >= 0 && done_[slot];
  }

 private:
  std::mutex mutex_;
  bool done_[kMaxDevices] = {};
};

// ---- TMA descriptor encoding (driver entry point fetched at run time; libcuda is not linked)
// `inner`/`outer`(/`batch`) are extents in elements, innermost first; the box is {box_inner,
// box_outer(,1)} with 128-byte swizzle; 16-bit elements only.
wb200_status encode_tmap_2d(CUtensorMap *map, const void *base, int format, uint64_t inner,
                            uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner,
                            uint32_t box_outer);
wb200_status encode_tmap_3d(CUtensorMap *map, const void *base, int format, uint64_t inner,
                            uint64_t outer, uint64_t batch, uint64_t row_pitch_bytes,
                            uint64_t batch_pitch_bytes, uint32_t box_inner, uint32_t box_outer);

// ---- tcgen05 GEMM with fused epilogue (gemm_umma.cu)
struct GemmUmmaArgs {
  int m, n, k;
  int in_format, out_format;   // wb200_format
  int lhs_transposed;          // 0: A[m,k] row-major, 1: A[k,m] row-major
  int rhs_transposed;          // 0: B[k,n] row-major, 1: B[n,k] row-major
  int epilogue;                // wb200_epilogue
  const void *a, *b;
  const float *bias;
  void *out;
};
bool gemm_umma_supports(const GemmUmmaArgs &args);
// Sets the kernels' per-device launch attributes (also done lazily by the first launch): call before a stream capture that
// will contain tensor-core GEMM launches.
wb200_status gemm_umma_prepare();
wb200_status launch_gemm_umma(const GemmUmmaArgs &args, int sm_count, int *device_status,
                              cudaStream_t stream);

// ---- bit-exact sequential-k GEMM on physical or compact storage (gemm_formal.cu)
struct GemmFormalArgs {
  int m, k, n, batch;
  int in_format, out_format;
  int lhs_transposed, rhs_transposed;
  int has_psum;
  const uint8_t *lhs, *rhs, *psum;
  uint8_t *dst;
  LayoutMap lhs_map, rhs_map, psum_map, dst_map;  // physical placement of every operand
};
wb200_status launch_gemm_formal(const GemmFormalArgs &args, cudaStream_t stream);

// ---- managed-reference tensor commands (tensor_ops.cu)
// `nan_flag` is set to 1 by the kernel if any input or result is NaN (the contract rejects those).
wb200_status launch_elementwise(int op, int format, int input_count, const uint8_t *in0,
                                const uint8_t *in1, uint8_t *dst, const LayoutMap &map, int *nan_flag,
                                cudaStream_t stream);
// Formal (bit-exact, NaN-canonicalising, flag-raising) elementwise family; `flags_word` collects the OR of the
// per-element IEEE flags (bit0 invalid, bit1 divByZero, bit2 overflow, bit3 underflow, bit4 inexact).
// How the second operand of a binary formal elementwise command is addressed: the same index as the first, a unit of
// `parameter` elements repeated, one 64-element row per group of `parameter` elements, or the immediate bits `parameter`.
enum { WB200_RHS_SAME = 0, WB200_RHS_UNIT = 1, WB200_RHS_GROUP = 2, WB200_RHS_SCALAR = 3 };
struct RhsBroadcast {
  uint32_t mode = WB200_RHS_SAME, parameter = 0;
};
struct PoolWindow {
  uint32_t kernel_w, kernel_h, stride_w, stride_h;
};
wb200_status launch_elementwise_formal(int op, int in_format, int out_format, int input_count, const uint8_t *in0, const uint8_t *in1,
                                       uint8_t *dst, const LayoutMap &in_map, const LayoutMap &out_map, uint32_t *flags_word,
                                       cudaStream_t stream, RhsBroadcast rhs = RhsBroadcast());
// A run of formal elementwise commands over 1-D Tensor vectors of one format and element count in which every command's
// first operand is the previous command's destination: one launch carries the value in registers from step to step and
// still writes every step's destination. Second operands are a full vector (WB200_RHS_SAME), immediate bits
// (WB200_RHS_SCALAR) or absent (unary; scalar = 0).
constexpr int kMaxChainSteps = 8;
struct ChainStep {
  int32_t op;
  uint32_t rhs_mode, scalar, reserved;
  const uint8_t *rhs;
  uint8_t *dst;
};
struct ElementwiseChain {
  int32_t steps, format;
  int64_t count;
  const uint8_t *lhs;
  ChainStep step[kMaxChainSteps];
};
wb200_status launch_elementwise_chain(const ElementwiseChain &chain, uint32_t *flags_word, cudaStream_t stream);
// A run of formal commands of one Tile - GEMMs (one matrix, formal policy), elementwise commands over 1-D vectors and
// NCx [n, h, w, c] reductions in any order, e.g. the scores, running maximum, probabilities, running sum and PV product
// of an online-attention step - executed by ONE launch: a single thread block walks the commands in issue order with a
// block barrier between them, so a command sees what the commands before it wrote, every destination the commands
// name is written, and every element goes through the same arithmetic as in the command's own kernel (bit-identical).
// Only small commands qualify (formal_run_admits): one block is a fraction of the machine.
constexpr int kMaxRunCommands = 16;
enum { WB200_RUN_ELEMENTWISE = 0, WB200_RUN_REDUCE = 1, WB200_RUN_GEMM = 2 };
struct RunElementwise {
  int32_t op, in_format, out_format, input_count;
  const uint8_t *in0, *in1;
  uint8_t *dst;
  LayoutMap in_map, out_map;
  RhsBroadcast rhs;
};
struct RunReduce {
  int32_t op, format;
  const uint8_t *src;
  uint8_t *dst;
  LayoutMap src_map, dst_map;
  uint32_t reduced_mask;
};
struct RunCommand {
  int32_t kind;
  int32_t variant = 0;   // GEMM: which instantiation of the tile function (gemm_formal_variant)
  union Payload {
    RunElementwise elementwise;
    RunReduce reduce;
    GemmFormalArgs gemm;
    __host__ __device__ Payload() {}
  } u;
  __host__ __device__ RunCommand() : kind(0), variant(0) {}
};
struct FormalRun {
  int32_t count = 0;
  RunCommand command[kMaxRunCommands];
};
bool formal_run_admits(const RunCommand &command);
int formal_gemm_variant(const GemmFormalArgs &args);   // gemm_formal.cu
wb200_status launch_formal_run(const FormalRun &run, uint32_t *flags_word, cudaStream_t stream);
// Formal reduction: NaN-canonicalising, flag-raising fold in row-major input order (bit d of `reduced_mask` = dimension d reduced).
wb200_status launch_reduce_formal(int op, int format, const uint8_t *src, uint8_t *dst, const LayoutMap &src_map, const LayoutMap &dst_map,
                                  uint32_t reduced_mask, uint32_t *flags_word, cudaStream_t stream);
// Plain pooling over NCx [n, h, w, c] tensors: `combine` is WB200_EW_MAX, WB200_EW_MIN or WB200_EW_ADD.
wb200_status launch_pool_formal(int combine, int format, const uint8_t *src, uint8_t *dst, const LayoutMap &src_map,
                                const LayoutMap &dst_map, PoolWindow window, uint32_t *flags_word, cudaStream_t stream);
wb200_status launch_convert(int src_format, int dst_format, const uint8_t *src, uint8_t *dst,
                            const LayoutMap &src_map, const LayoutMap &dst_map, int *nan_flag,
                            cudaStream_t stream);
wb200_status launch_reduce(int op, int format, const uint8_t *src, uint8_t *dst,
                           const LayoutMap &src_map, const LayoutMap &dst_map, uint32_t reduced_mask,
                           int *nan_flag, cudaStream_t stream);
// Device codec: compact <-> physical.
wb200_status launch_unpack(const uint8_t *storage, uint8_t *compact, const LayoutMap &map,
                           int element_bytes, cudaStream_t stream);
wb200_status launch_pack(const uint8_t *compact, uint8_t *storage, const LayoutMap &map,
                         int element_bytes, cudaStream_t stream);

// ---- attention (attention_fa.cu, attention_fa_f32.cu, attention_fd.cu)
struct AttentionArgs {
  int batch, q_heads, kv_heads, q_len, kv_len, head_dim;
  int format;
  int causal, zero_fully_masked;
  float scale;
  int64_t causal_offset;  // query_start - key_start
  int64_t kv_valid;       // keys with index >= kv_valid are masked (key_end - key_start)
  const void *q, *k, *v;
  void *out;
  float *lse, *row_max, *row_sum;
  int out_token_major;    // 1: out is [batch, q_len, q_heads, head_dim] (rows of a following projection GEMM)
};
bool attention_fa_umma_supports(const AttentionArgs &args);
wb200_status launch_attention_fa_umma(const AttentionArgs &args, int sm_count, int *device_status,
                                      cudaStream_t stream);
wb200_status launch_attention_fa_simt(const AttentionArgs &args, cudaStream_t stream);

// Flash-decoding. `partials` is scratch of fd_partial_floats(args, splits) floats.
// Stage 1 writes one (acc[D], m, l) record per (batch, q_head, split); stage 2 left-folds records in
// ascending split order. With `finalize` == 0 stage 2 writes the merged state to `state_out`
// instead of out / lse.
bool attention_fd_supports(const AttentionArgs &args);
uint32_t fd_choose_splits(const AttentionArgs &args, int sm_count);
size_t fd_partial_floats(const AttentionArgs &args, uint32_t splits);
wb200_status launch_attention_fd(const AttentionArgs &args, uint32_t splits, float *partials,
                                 int finalize, float *state_out, cudaStream_t stream);
wb200_status launch_attention_fd_merge(const AttentionArgs &args, const float *states,
                                       uint32_t shard_count, cudaStream_t stream);
// Sequence-sharded decode with the exchange inside the kernel: stage 1, then one kernel that folds this rank's splits,
// writes the state into every rank's exchange buffer (peer-mapped memory), waits for the world's states and merges
// them in ascending rank order. `peer_buffers` holds `world` buffers of fd_exchange_floats() floats, zero-initialised;
// `epoch` is this rank's pair of zero-initialised words. With `arrivals` (batch * kv_heads zero-initialised words that the
// kernel leaves zeroed) the fold, exchange and merge run in the last stage-1 CTA of every (batch, kv head): one launch.
size_t fd_exchange_floats(int rows, int world);
wb200_status launch_attention_fd_exchange(const AttentionArgs &args, uint32_t splits, float *partials, int rank, int world,
                                          void *const *peer_buffers, unsigned int *epoch, unsigned int *arrivals,
                                          int *device_status, cudaStream_t stream);

// Sum over the ranks of a buffer that lies at `multicast` in an NVLink multicast mapping of a symmetric allocation
// (switch_sum.cu): in place, every rank ends with the same sums. `signals` holds every rank's 2 * world zero-initialised
// signal words (peer-mapped), `epoch` this rank's pair of zero-initialised words.
constexpr int kMaxSwitchRanks = 16;
// `multicast_out` (null: in place) is the multicast address the sums are stored to; `residual` (null: none) is this rank's
// copy of a tensor of the same extent that is added to the sums before the store (round(sum + residual), one rounding).
wb200_status launch_switch_sum(void *multicast, uint64_t elements, int format, int rank, int world, void *const *signals,
                               unsigned int *epoch, int blocks, int *device_status, cudaStream_t stream, void *multicast_out = nullptr,
                               const void *residual = nullptr);


// ---- decoder-layer pieces (layer_ops.cu); device pointers, bf16 / f16 storage
wb200_status launch_rmsnorm(int format, const void *x, const void *gamma, void *y, int rows, int dim, float eps,
                            cudaStream_t stream);
wb200_status launch_rope_split(int format, const void *qkv, void *q, void *k, void *v, int batch, int seq, int q_heads,
                               int kv_heads, int head_dim, float theta, int position_offset, cudaStream_t stream);
wb200_status launch_residual_add(int format, const void *a, const void *b, void *out, size_t elements, cudaStream_t stream);

// ---- movement commands on device-resident memory images (tile_movement.cu)
struct StridedLayout {
  uint32_t inner_bytes;
  uint32_t strides[3];
  uint32_t iterations[3];
};
uint64_t strided_segments(const StridedLayout &layout);
uint64_t strided_span(const StridedLayout &layout);   // bytes from the first to one past the last byte touched
wb200_status launch_strided_copy(const uint8_t *src, const StridedLayout &from, uint8_t *dst, const StridedLayout &to,
                                 cudaStream_t stream);
wb200_status launch_fill(uint8_t *dst, uint32_t value_bits, uint64_t count, int element_bytes, cudaStream_t stream);
// Packed Bool -> 1.0 / 0 of `format`; masked element move (store = 0: validate only; *first_refused = smallest element << 8 | 4
// whose mask is neither 0 nor 1.0).
wb200_status launch_bit2fp(const uint8_t *src, uint8_t *dst, uint32_t count, int format, cudaStream_t stream);
wb200_status launch_mask_move(const uint8_t *src, const uint8_t *mask, uint8_t *dst, uint32_t count, int format, int store,
                              unsigned long long *first_refused, cudaStream_t stream);

}  // namespace wb200
