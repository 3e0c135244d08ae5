/* wb200.h - C ABI of the B200 numeric backend for the Wafer functional model's numeric path.
 *
 * The library executes, on one B200 (sm_100a), the tensor commands the reference's functional model
 * hands to its numeric backends (GEMM / elementwise / convert / reduce) and the attention regions
 * (flash-attention prefill, flash-decoding) those commands implement after lowering.
 *
 * Everything here is plain C: pointers, sizes and POD structs. No C++ or torch types cross the
 * boundary. All entry points return a wb200_status; wb200_last_error() returns the message of the
 * last failure on the calling thread. No entry point falls back to the CPU: without a usable device
 * wb200_backend_create() fails with WB200_ERR_NO_DEVICE.
 *
 * Reference interfaces replaced (paths inside the reference project):
 *   include/Wafer/Simulator/Kernel/TargetModelKernel.h:164-170   TargetModelOneDNNBackend::tryExecute
 *   include/Wafer/Simulator/Kernel/TargetModelKernel.h:187-200   TargetModelManagedReferenceBackend::execute x3
 *   include/Wafer/Simulator/Reference/FormalOperations.h:21-113  Formal{Convert,Elementwise,Gemm,Reduce}Operation
 *   include/Wafer/Target/PhysicalTensor/PhysicalTensorDescriptor.h:20-53
 *   lib/Wafer/Target/TargetCall.cpp:86-147 (wafer_tx81_* argument order, see wb200_target_call_*)
 */
#ifndef WB200_H
#define WB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WB200_ABI_VERSION 4
#define WB200_MAX_RANK 8

typedef struct wb200_backend wb200_backend;

typedef enum wb200_status {
  WB200_OK = 0,
  WB200_ERR_INVALID_ARGUMENT = 1, /* malformed descriptor, size mismatch, null pointer            */
  WB200_ERR_UNSUPPORTED = 2,      /* valid request outside the domain this backend executes        */
  WB200_ERR_NAN_DOMAIN = 3,       /* managed-reference contract: NaN input or NaN result rejected  */
  WB200_ERR_BUDGET = 4,           /* scalar-evaluation / byte budget exceeded before any work      */
  WB200_ERR_CUDA = 5,             /* a CUDA runtime call failed; message carries the CUDA error    */
  WB200_ERR_DEVICE_TIMEOUT = 6,   /* a bounded device-side wait gave up; context remains usable    */
  WB200_ERR_NO_DEVICE = 7,        /* no sm_100 device / extension cannot run                       */
  WB200_ERR_LIMIT = 8,            /* a fixed capacity of an entry point was exceeded               */
  WB200_ERR_CALLBACK = 9          /* a caller-supplied callback reported a failure                 */
} wb200_status;

/* Logical formats. Ordinals equal the reference's LogicalFormat enum and its Data_Format codes
 * (include/Wafer/Target/TargetFormat.h:17-31, lib/Wafer/Target/TargetFormat.cpp:61-66). */
typedef enum wb200_format {
  WB200_I8 = 0, WB200_I16 = 1, WB200_F16 = 2, WB200_BF16 = 3, WB200_I32 = 4, WB200_F32 = 5,
  WB200_TF32 = 6, WB200_BOOL = 7, WB200_U8 = 8, WB200_U16 = 9, WB200_U32 = 10, WB200_I64 = 11,
  WB200_U64 = 12, WB200_FORMAT_NONE = 13
} wb200_format;

/* Physical layouts (include/Wafer/Target/PhysicalTensor/PhysicalLayout.h:18). */
typedef enum wb200_layout {
  WB200_LAYOUT_TENSOR = 0, WB200_LAYOUT_NTENSOR = 1, WB200_LAYOUT_CX = 2, WB200_LAYOUT_NCX = 3
} wb200_layout;

/* Mirror of PhysicalTensorDescriptor {format, layout, shape}. */
typedef struct wb200_tensor_desc {
  uint8_t format; /* wb200_format */
  uint8_t layout; /* wb200_layout */
  uint8_t rank;   /* 1..WB200_MAX_RANK */
  uint8_t reserved[5];
  uint64_t shape[WB200_MAX_RANK];
} wb200_tensor_desc;

/* Geometry of a physical tensor (computePhysicalTensorGeometry,
 * lib/Wafer/Target/PhysicalTensor/PhysicalLayout.cpp:111-200). */
typedef struct wb200_geometry {
  int64_t element_bytes, compact_bytes, physical_elements, physical_bytes;
  int64_t c_block, cx_blocks, c0, aligned_c, outer_elements, block_outer_elements;
  int64_t outer_slice_stride_elements, bank_align_elements;
} wb200_geometry;

/* TargetElementwiseOperation ordinals (include/Wafer/Target/TargetOperation.h:58-93). */
typedef enum wb200_elementwise_op {
  WB200_EW_ABS = 0, WB200_EW_RECIP = 1, WB200_EW_SQUARE = 2, WB200_EW_SQRT = 3, WB200_EW_RSQRT = 4,
  WB200_EW_NEG = 5, WB200_EW_MAX = 6, WB200_EW_MIN = 7, WB200_EW_ADD = 8, WB200_EW_SUB = 9,
  WB200_EW_MUL = 10, WB200_EW_EQ = 12, WB200_EW_NE = 13, WB200_EW_GE = 14, WB200_EW_GT = 15,
  WB200_EW_LE = 16, WB200_EW_LT = 17, WB200_EW_LOGIC_NOT = 18, WB200_EW_LOGIC_AND = 19,
  WB200_EW_LOGIC_OR = 20, WB200_EW_LOGIC_XOR = 21, WB200_EW_LOG2 = 22, WB200_EW_LN = 23,
  WB200_EW_POW2 = 24, WB200_EW_EXP = 25, WB200_EW_EXPLP = 26, WB200_EW_SIN = 27, WB200_EW_COS = 28,
  WB200_EW_TANH = 29, WB200_EW_SIGMOID = 30, WB200_EW_RELU = 31, WB200_EW_SATRELU = 32,
  WB200_EW_LEAKYRELU = 33, WB200_EW_SOFTPLUS = 34
} wb200_elementwise_op;

/* TargetReduceOperation / TargetReduceDimension (TargetOperation.h:102-113). */
typedef enum wb200_reduce_op { WB200_RED_SUM = 0, WB200_RED_MAX = 1, WB200_RED_MIN = 2, WB200_RED_AVG = 3 } wb200_reduce_op;
typedef enum wb200_reduce_dim {
  WB200_RED_TRAILING0 = 0, WB200_RED_TRAILING1 = 1, WB200_RED_TRAILING2 = 2, WB200_RED_TRAILING3 = 3,
  WB200_RED_TRAILING2AND1 = 4, WB200_RED_TRAILING2AND1AND0 = 5
} wb200_reduce_dim;

typedef enum wb200_orientation { WB200_NORMAL = 0, WB200_TRANSPOSE = 1 } wb200_orientation;

/* How a GEMM command is evaluated.
 *   FORMAL: every output is the k-ascending chain acc = fma_f32(widen(a), widen(b), acc) from +0,
 *           then the optional f32 psum add, then one RNE rounding to the destination format
 *           (lib/Wafer/Simulator/Reference/Numeric/FormalTensorNumeric.cpp:271-361). Bit-exact.
 *   TENSOR: tcgen05 UMMA with fp32 TMEM accumulation and the same single final rounding; the
 *           summation order is the tensor core's, as the oneDNN path's is oneDNN's
 *           (lib/Wafer/Simulator/OneDNN/OneDNNGemmAdapter.cpp:351-357,419-429). Tolerance-level. */
typedef enum wb200_gemm_policy { WB200_GEMM_FORMAL = 0, WB200_GEMM_TENSOR = 1 } wb200_gemm_policy;

/* Evidence returned with every command-level result; mirrors TargetModelOneDNNDispatchEvidence and
 * TargetModelManagedReferenceEvidence (TargetModelKernel.h:143-150, 172-176) plus the
 * FormalNumericExceptionFlags bit set (bit0 invalid, bit1 divByZero, bit2 overflow, bit3 underflow,
 * bit4 inexact). The managed-reference contract returns flags == 0. */
typedef struct wb200_evidence {
  uint64_t matmul_invocations;
  uint64_t reorder_invocations;
  uint64_t formal_fused_multiply_adds;
  uint64_t scalar_evaluations;
  uint32_t evidence_kind; /* 0 none, 2 managed-reference environment */
  uint32_t flags;
  uint32_t gpu_launches;  /* kernels this call launched */
  uint32_t device_us;     /* device time of those kernels in microseconds (CUDA events; tensor commands only, else 0) */
  char digest[96];         /* "b200:<device name>:sm_<cc>:abi<version>" */
  char implementation[64]; /* kernel family that produced the result */
} wb200_evidence;

/* ------------------------------------------------------------------ lifecycle */

/* Creates a backend bound to CUDA device `device`. Fails with WB200_ERR_NO_DEVICE when the device
 * is absent or is not compute capability 10.x. */
wb200_status wb200_backend_create(int device, wb200_backend **out);
void wb200_backend_destroy(wb200_backend *backend);
/* Message of the most recent failure on the calling thread (empty string if none). */
const char *wb200_last_error(void);
int wb200_abi_version(void);
/* Budgets of the managed-reference contract (ManagedReferenceTargetModel.cpp:470-490):
 * maximum total physical bytes and maximum logical scratch bytes per request. 0 = unlimited. */
wb200_status wb200_backend_set_budget(wb200_backend *backend, uint64_t max_total_bytes,
                                      uint64_t max_scratch_bytes);

/* ------------------------------------------------------------------ physical layout (host math) */

/* replaces computePhysicalTensorGeometry (PhysicalLayout.cpp:111-200) */
wb200_status wb200_physical_geometry(const wb200_tensor_desc *desc, wb200_geometry *out);
/* replaces getPhysicalTensorStorageBytes (PhysicalTensorCodec.h) */
wb200_status wb200_physical_bytes(const wb200_tensor_desc *desc, uint64_t *out_bytes);

/* Device codec. replaces pack/unpackPhysicalTensorLogicalValues (PhysicalTensorCodec.h:57-73).
 * unpack: physical storage -> compact row-major little-endian elements.
 * pack:   compact elements written into a copy of `storage_template`; non-logical bytes keep the
 *         template's values. All pointers are HOST pointers; the codec itself runs on the device. */
wb200_status wb200_unpack(wb200_backend *backend, const wb200_tensor_desc *desc,
                          const uint8_t *storage, uint64_t storage_bytes, uint8_t *compact_out,
                          uint64_t compact_bytes);
wb200_status wb200_pack(wb200_backend *backend, const wb200_tensor_desc *desc,
                        const uint8_t *compact, uint64_t compact_bytes,
                        const uint8_t *storage_template, uint8_t *storage_out,
                        uint64_t storage_bytes);

/* ------------------------------------------------------------------ command level (Seam 1) */
/* All storage pointers are HOST pointers to full physical storage, as the reference's
 * TargetModelNumericTensor::storage vectors are. `destination_out` receives the full physical
 * storage of the result, padding bytes copied from `destination_template`. */

typedef struct wb200_gemm_request { /* FormalGemmOperation + TargetModelNumericOperands */
  wb200_tensor_desc lhs, rhs, destination, psum;
  uint32_t m, k, n, batch_count;
  uint8_t lhs_orientation, rhs_orientation; /* wb200_orientation */
  uint8_t has_psum;
  uint8_t policy; /* wb200_gemm_policy */
  uint32_t reserved;
  const uint8_t *lhs_storage;  uint64_t lhs_bytes;
  const uint8_t *rhs_storage;  uint64_t rhs_bytes;
  const uint8_t *psum_storage; uint64_t psum_bytes;
  const uint8_t *destination_template;
  uint8_t *destination_out;
  uint64_t destination_bytes;
} wb200_gemm_request;

/* replaces TargetModelOneDNNBackend::tryExecute (TargetModelKernel.h:164-170) and the formal GEMM
 * (FormalTensorNumeric.cpp:271-361). `*handled` = 0 with WB200_OK means "declined, use the formal
 * path" exactly like the reference's successful null optional (TENSOR policy only). */
wb200_status wb200_gemm(wb200_backend *backend, const wb200_gemm_request *request, int *handled,
                        wb200_evidence *evidence);

typedef struct wb200_elementwise_request { /* FormalElementwiseOperation + operands */
  uint32_t operation; /* wb200_elementwise_op */
  uint32_t input_count;
  wb200_tensor_desc inputs[2];
  wb200_tensor_desc destination;
  const uint8_t *input_storage[2];
  uint64_t input_bytes[2];
  const uint8_t *destination_template;
  uint8_t *destination_out;
  uint64_t destination_bytes;
  uint64_t max_scalar_evaluations; /* FormalNumericWorkBudget */
} wb200_elementwise_request;
/* replaces TargetModelManagedReferenceBackend::execute(TargetModelElementwiseRequest)
 * (ManagedReferenceTargetModel.cpp:230-342, 561-566) */
wb200_status wb200_elementwise(wb200_backend *backend, const wb200_elementwise_request *request,
                               wb200_evidence *evidence);

/* The formal (bit-exact) elementwise family of lib/Wafer/Simulator/Reference/Formal/FormalNumericElementwise.cpp:23-248,
 * which the reference runs when the managed backend declines: abs, neg, recip, square, max, min, add, sub, mul, relu in the
 * operand format with one RNE rounding; eq / ne / ge / gt / le / lt to Bool or to 1.0 / 0.0 of a float format (with a NaN
 * operand only `ne` holds); logic not / and / or / xor on "bits != 0" to Bool; and, for F16 / BF16 operands, the
 * correctly rounded functions of lib/Wafer/Simulator/Reference/Numeric/MPFRNumeric.cpp:372-470, 560-682 (sqrt, rsqrt,
 * log2, ln, pow2, exp, sin, cos, tanh, sigmoid, softplus: the exact function rounded once to nearest-even with
 * gradual underflow; F32 operands are declined). NaN results are the canonical quiet NaN
 * (nothing is rejected); `evidence->flags` is the OR of the IEEE flags over all elements. Bool tensors are bit-packed,
 * least significant bit first, and are taken in Tensor / NTensor layout. */
wb200_status wb200_elementwise_formal(wb200_backend *backend, const wb200_elementwise_request *request,
                                      wb200_evidence *evidence);

typedef struct wb200_convert_request { /* FormalConvertOperation + operands */
  uint32_t opcode;        /* target convert route 139..174 */
  uint32_t rounding_mode; /* 0 nearest-even (the only mode of the managed contract) */
  wb200_tensor_desc source, destination;
  const uint8_t *source_storage;
  uint64_t source_bytes;
  const uint8_t *destination_template;
  uint8_t *destination_out;
  uint64_t destination_bytes;
  uint64_t max_scalar_evaluations;
} wb200_convert_request;
/* replaces TargetModelManagedReferenceBackend::execute(TargetModelConvertRequest)
 * (ManagedReferenceTargetModel.cpp:344-379, 554-559) */
wb200_status wb200_convert(wb200_backend *backend, const wb200_convert_request *request,
                           wb200_evidence *evidence);

/* The formal scalar conversion routes (lib/Wafer/Target/PhysicalTensor/TargetScalarConversion.cpp:166-361), which the
 * reference runs when the managed backend declines: opcodes 143..174 between I16 / I32 and F16 / BF16 / F32 / TF32 and
 * between those floating formats, `rounding_mode` 0 nearest-even, 1 toward zero, 2 toward +inf, 3 toward -inf on the routes
 * that carry one (4, stochastic, and the zero-point routes 139..142 are WB200_ERR_UNSUPPORTED like in the reference).
 * TF32 keeps its 19 semantic bits in storage [31:13]; other low bits set is an invalid source encoding. NaN becomes the
 * canonical quiet NaN (invalid for a signalling one); floating -> integer refuses NaN, infinity and values outside the
 * destination range after rounding (WB200_ERR_NAN_DOMAIN, nothing written). evidence->flags: the OR of the IEEE flags
 * (inexact; overflow also when a directed mode returns the largest finite value; underflow by tininess after rounding). */
wb200_status wb200_convert_formal(wb200_backend *backend, const wb200_convert_request *request, wb200_evidence *evidence);

typedef struct wb200_reduce_request { /* FormalReduceOperation + operands */
  uint32_t operation; /* wb200_reduce_op */
  uint32_t dimension; /* wb200_reduce_dim */
  wb200_tensor_desc input, destination;
  const uint8_t *input_storage;
  uint64_t input_bytes;
  const uint8_t *destination_template;
  uint8_t *destination_out;
  uint64_t destination_bytes;
  uint64_t max_scalar_evaluations;
} wb200_reduce_request;
/* replaces TargetModelManagedReferenceBackend::execute(TargetModelReduceRequest)
 * (ManagedReferenceTargetModel.cpp:381-458, 568-573) */
wb200_status wb200_reduce(wb200_backend *backend, const wb200_reduce_request *request,
                          wb200_evidence *evidence);

/* The formal reduction (lib/Wafer/Simulator/Reference/Numeric/FormalTensorNumeric.cpp:363-425, step
 * Reference/Formal/FormalNumericReduce.cpp:12-67), which the reference runs when the managed backend declines: the same domain
 * as wb200_reduce, but every output folds its inputs in row-major order from +0 (sum) or -inf / +inf (max / min) with the formal
 * add / maximum / minimum, so a NaN input gives the canonical quiet NaN (invalid for a signalling one) instead of a refusal,
 * max / min order -0 below +0, and evidence->flags carries the OR of the IEEE flags of all steps. */
wb200_status wb200_reduce_formal(wb200_backend *backend, const wb200_reduce_request *request, wb200_evidence *evidence);

/* ------------------------------------------------------------------ region level */
/* Regions are what a run of lowered commands computes as a whole. Buffers are compact row-major.
 * `memory` selects where ALL data pointers of the call live. With WB200_MEM_HOST the call stages
 * inputs to the device, runs, copies results back and synchronises before returning. With
 * WB200_MEM_DEVICE the kernels are enqueued on `stream` (a cudaStream_t, may be NULL) and the call
 * returns without synchronising; device status is then read by wb200_backend_poll(). */
typedef enum wb200_memory { WB200_MEM_HOST = 0, WB200_MEM_DEVICE = 1 } wb200_memory;

/* Where wb200_attention_fa writes `out`: head-major like q, or token-major [batch, q_len, q_heads, head_dim]
 * (the row layout a following output-projection GEMM reads). */
typedef enum wb200_out_layout { WB200_OUT_HEAD_MAJOR = 0, WB200_OUT_TOKEN_MAJOR = 1 } wb200_out_layout;

typedef struct wb200_attention_params {
  uint32_t batch, q_heads, kv_heads; /* q_heads % kv_heads == 0 (grouped queries) */
  uint32_t q_len, kv_len, head_dim;
  uint8_t format;            /* WB200_BF16, WB200_F16 or WB200_F32: Q, K, V and out share it
                                (lib/Wafer/IR/LinalgExt/AttentionOps.cpp:405-419) */
  uint8_t causal;            /* key j visible to query q iff j <= (query_start - key_start) + q */
  uint8_t zero_fully_masked; /* finalize coefficient 0 instead of 1/0 when l == 0 */
  uint8_t memory;            /* wb200_memory */
  float scale;               /* score = (Q.K) * scale */
  int64_t query_start, key_start, key_end; /* position operands; key_end <= 0 means key_start+kv_len
                                (lib/Wafer/IR/LinalgExt/AttentionOps.cpp:31-60) */
  const void *q;   /* [batch, q_heads, q_len, head_dim]  */
  const void *k;   /* [batch, kv_heads, kv_len, head_dim] */
  const void *v;   /* [batch, kv_heads, kv_len, head_dim] */
  void *out;       /* [batch, q_heads, q_len, head_dim], same format as q */
  float *lse;      /* optional [batch, q_heads, q_len]: m + ln(l), -inf when l == 0 */
  float *row_max;  /* optional: carried state m */
  float *row_sum;  /* optional: carried state l */
  void *stream;
  uint32_t out_layout; /* wb200_out_layout; flash-attention prefill only */
  uint32_t reserved;
} wb200_attention_params;

/* Flash-attention prefill: online (m, l, acc) update over KV tiles, K2 never split across workers.
 * replaces the command run materialised from
 * lib/Wafer/Transforms/Linalg/OnlineAttentionDecomposition.cpp:568-594 and finalize
 * lib/Wafer/Transforms/Linalg/OnlineAttentionMaterialization.cpp:196-262. */
/* Notes on wb200_attention_fa: with WB200_MEM_HOST and at least two (batch, kv-head) units the call pipelines copy-in,
 * kernels and copy-out over chunks on three streams (use pinned host memory for the overlap). The tcgen05 kernel runs a
 * persistent grid over a work plan that is built on the first call of each distinct shape (a few KiB of device memory,
 * one allocation and one copy, cached per device): make that first call outside any stream capture. */
wb200_status wb200_attention_fa(wb200_backend *backend, const wb200_attention_params *params);

/* Flash-decoding: KV axis split into `kv_splits` >= 2 contiguous intervals (0 = choose), each
 * producing a partial (m, l, acc); partials are left-folded in ascending interval order and then
 * finalized. replaces OnlineAttentionMaterialization.cpp:264-373 and the fold order of
 * lib/Wafer/Transforms/Linalg/SpatialRegionMaterialization.cpp:2420-2433. q_len must be 1.
 * The split-KV partial records of this entry and of wb200_attention_fd_partial / _exchange live in a grow-only scratch
 * buffer of the backend: a call that needs more than every call before it frees and reallocates that buffer (cudaFree
 * waits for the device's outstanding work first), so a CUDA graph that captured an earlier decode call would replay
 * with a dangling address. Run the largest shape once before capturing. */
wb200_status wb200_attention_fd(wb200_backend *backend, const wb200_attention_params *params,
                                uint32_t kv_splits);

/* Flash-decoding for callers that must not allocate device memory at call time: a serving loop whose
 * memory was divided up at start-up and that cannot afford the implicit synchronisation of an allocation,
 * a process held to a fixed memory budget, or code that runs at a point where the CUDA runtime refuses
 * allocation calls.
 * It has no counterpart in the reference. Same arithmetic and results as wb200_attention_fd; the split-KV
 * partial records go to a fixed 16 MiB array inside the library image (every GPU that loads the library
 * holds it until exit) instead of a buffer allocated on demand, and the call itself performs no
 * allocation. Limits: device buffers only (memory == WB200_MEM_DEVICE);
 * batch * q_heads * kv_splits * (head_dim + 2) <= 4 194 304 floats, otherwise WB200_ERR_LIMIT
 * (kv_splits == 0 takes the split count wb200_attention_fd would choose and halves it until it fits). The first call on a device looks up the
 * array's device address; make that call before any stream capture begins. All calls share the one
 * array: two calls whose kernels overlap on the GPU (different streams) race on it, so serialise them.
 * Nothing in the array has to be cleared between calls (every record read is written first). */
wb200_status wb200_attention_fd_static(wb200_backend *backend, const wb200_attention_params *params,
                                       uint32_t kv_splits);

/* Sequence-sharded flash-decoding, one shard per GPU: computes this shard's un-finalized state.
 * `state_out` is [batch, q_heads, head_dim + 2] fp32: acc[0..D), then m, then l. `out`, `lse` are
 * ignored. */
wb200_status wb200_attention_fd_partial(wb200_backend *backend, const wb200_attention_params *params,
                                        uint32_t kv_splits, float *state_out);
/* Left-folds `shard_count` states (ascending shard order, layout [shard, batch*q_heads, D+2]) and
 * finalizes into out / lse. */
wb200_status wb200_attention_fd_merge(wb200_backend *backend, const wb200_attention_params *params,
                                      const float *states, uint32_t shard_count);

/* Sequence-sharded flash-decoding with the exchange inside the kernel (one shard of the KV sequence per GPU, one
 * process per GPU). Stage 1 as in wb200_attention_fd_partial; then one kernel folds this rank's splits, stores the
 * per-head state (head_dim + 2 floats) into every rank's exchange buffer with plain peer stores over NVLink, waits
 * (bounded: WB200_ERR_DEVICE_TIMEOUT at the next wb200_backend_poll) for the states of all ranks and merges them in
 * ascending rank order, the fold order of lib/Wafer/Transforms/Linalg/SpatialRegionMaterialization.cpp:2420-2433.
 * No collective library call is involved, so the step can be captured into a CUDA graph.
 *   peer_buffers[r]  rank r's exchange buffer as addressable from this GPU (peer-mapped / symmetric memory; entry
 *                    [rank] is this rank's own), wb200_fd_exchange_bytes() bytes each, zero-filled before first use
 *   epoch            two zero-filled 32-bit words in this rank's memory; the kernel keeps the call count there
 * Every rank must make the same sequence of calls with the same batch and q_heads. Device buffers only. */
#define WB200_MAX_EXCHANGE_RANKS 16
typedef struct wb200_fd_exchange {
  uint32_t rank, world;
  void *peer_buffers[WB200_MAX_EXCHANGE_RANKS];
  uint32_t *epoch;
} wb200_fd_exchange;
uint64_t wb200_fd_exchange_bytes(uint32_t batch, uint32_t q_heads, uint32_t world);
wb200_status wb200_attention_fd_exchange(wb200_backend *backend, const wb200_attention_params *params, uint32_t kv_splits,
                                         const wb200_fd_exchange *exchange);

typedef enum wb200_epilogue {
  WB200_EPI_NONE = 0,      /* out = round(acc)                                   */
  WB200_EPI_BIAS = 1,      /* out = round(acc + bias[n])                         */
  WB200_EPI_BIAS_GELU = 2, /* out = round(gelu_erf(acc + bias[n])), f32 math     */
  WB200_EPI_SWIGLU = 3     /* out[m, j] = round(silu(acc[m, 2j]) * acc[m, 2j+1]): gate and up columns
                              interleaved in B; out is [m, n / 2]                 */
} wb200_epilogue;

typedef struct wb200_gemm_epilogue_params {
  uint32_t m, n, k;
  uint8_t in_format;  /* WB200_BF16 or WB200_F16 (A and B) */
  uint8_t out_format; /* WB200_BF16, WB200_F16 or WB200_F32 */
  uint8_t lhs_orientation, rhs_orientation; /* NORMAL: A[m,k], B[k,n]; TRANSPOSE: A[k,m], B[n,k] */
  uint8_t epilogue;   /* wb200_epilogue */
  uint8_t memory;     /* wb200_memory */
  uint8_t reserved[2];
  const void *a, *b;
  const float *bias;  /* [n] fp32, required unless epilogue == NONE */
  void *out;          /* [m, n] */
  void *stream;
} wb200_gemm_epilogue_params;

/* Tiled GEMM region with fused producer/epilogue chain (dot_general -> +bias -> GELU -> narrow):
 * fp32 accumulation and a single final rounding (ContractionAccumulation.cpp:147-218). */
wb200_status wb200_gemm_epilogue(wb200_backend *backend, const wb200_gemm_epilogue_params *params);

/* Pieces of a Llama-style decoder layer between the GEMM and attention regions (device buffers, bf16 / f16,
 * enqueued on `stream`). They are the fused producer / epilogue chains of config "decoder layer": the reference
 * lowers them to elementwise / reduce command runs (lib/Wafer/Simulator/Reference/ManagedReferenceTargetModel.cpp:
 * 230-458); here each chain is one kernel with f32 arithmetic and one rounding per produced element.
 *   rmsnorm:      y = round(round(x * rsqrt(mean(x^2) + eps)) * gamma), rows x dim
 *   rope_split:   token-major qkv rows [q heads | k heads | v heads] -> head-major Q, K (rotary, pairs (i, i + D/2),
 *                 angle = (position_offset + s) * theta^(-2i/D)) and V
 *   residual_add: out = round(a + b) */
wb200_status wb200_rmsnorm(wb200_backend *backend, uint32_t format, const void *x, const void *gamma, void *y,
                           uint32_t rows, uint32_t dim, float eps, void *stream);
wb200_status wb200_rope_split(wb200_backend *backend, uint32_t format, const void *qkv, void *q, void *k, void *v,
                              uint32_t batch, uint32_t seq, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                              float theta, uint32_t position_offset, void *stream);
wb200_status wb200_residual_add(wb200_backend *backend, uint32_t format, const void *a, const void *b, void *out,
                                uint64_t elements, void *stream);

/* One rank's shard of a Llama-style decoder layer forward as ONE call: RMSNorm -> fused QKV projection ->
 * rotary + head-major split -> causal grouped-query flash attention -> output projection -> [sum over shards]
 * -> residual -> RMSNorm -> gate/up projection with SwiGLU epilogue -> down projection -> [sum over shards]
 * -> residual. The reference lowers such a block to GEMM / attention / elementwise command regions and realises
 * the two sums with Tile collectives (lib/Wafer/Transforms/Tile/DistributedCollectiveMovement.cpp:675-735); the
 * block its own tests run is test/Board/PyTorch/wafer_pytorch_board_cases.py:817-867. Ten kernels are enqueued
 * on `stream`; nothing is allocated: the caller passes `workspace` of at least
 * wb200_decoder_layer_workspace_bytes() bytes (256-byte aligned). All pointers are device pointers.
 *   q_heads, kv_heads, ffn   this shard's query heads, KV heads and FFN columns
 *   wqkv  [d_model, (q_heads + 2 kv_heads) head_dim]   columns [q heads | k heads | v heads]
 *   wo    [q_heads head_dim, d_model]
 *   wgu   [d_model, 2 ffn]   gate and up columns interleaved: (gate_0, up_0, gate_1, up_1, ...)
 *   wdown [ffn, d_model]
 * `allreduce` (may be null for a single shard) is called twice per part, after the kernels producing the partial sum
 * have been enqueued, with a buffer inside `workspace` holding `elements` values of `format` and a stream that is
 * already ordered after those kernels; it must enqueue an in-place sum over the shards ordered after the work already
 * on that stream and before work enqueued on it later (an NCCL all-reduce on that stream, or on another stream with
 * event edges), and return 0. */
typedef int32_t (*wb200_allreduce_fn)(void *user, void *device_buffer, uint64_t elements, uint32_t format, void *stream);
typedef struct wb200_decoder_layer_params {
  uint32_t batch, seq, d_model, head_dim;
  uint32_t q_heads, kv_heads, ffn;
  uint32_t format;             /* WB200_BF16 or WB200_F16 */
  float eps, rope_theta;
  uint32_t position_offset;
  uint32_t micro_batches;      /* > 1 with an allreduce callback: the batch flows through the layer as that many equal
                                  parts (whole sequences) on `stream`, and the sum of each part is enqueued on a second,
                                  internal stream (which the callback then receives), so that it travels while the
                                  following parts compute. 0 / 1: one pass, sums on `stream` */
  uint32_t reserved_sms;       /* with micro_batches > 1: SMs the persistent compute kernels leave free for the
                                  collective's kernels (0: none) */
  const void *x;               /* [batch * seq, d_model] */
  void *out;                   /* [batch * seq, d_model] */
  const void *norm1, *wqkv, *wo, *norm2, *wgu, *wdown;
  void *workspace;
  uint64_t workspace_bytes;
  wb200_allreduce_fn allreduce;
  void *allreduce_user;
  void *stream;
  const struct wb200_switch_sum_params *switch_sum; /* optional, instead of `allreduce`: the sums are done by the library's
                                  NVSwitch kernel (wb200_switch_sum, below) without leaving the call. `multicast` is the
                                  multicast address of `workspace`, which must then be a symmetric allocation bound to a
                                  multicast object; rank, world, signals and epoch as for wb200_switch_sum; blocks 0 means
                                  reserved_sms; elements, format, stream, multicast_out and residual are ignored (the layer
                                  sets them: its two residual adds are done by the sums, bit-identically) */
} wb200_decoder_layer_params;
uint64_t wb200_decoder_layer_workspace_bytes(const wb200_decoder_layer_params *params);
wb200_status wb200_decoder_layer(wb200_backend *backend, const wb200_decoder_layer_params *params);
/* Device timeline of the last wb200_decoder_layer call that ran with micro_batches > 1 (waits for that call to finish):
 * milliseconds from the call's first kernel to, for part i and phase f (0 attention, 1 FFN), ms[4 i + 2 f] = the part's
 * partial sum is ready (its kernels are done) and ms[4 i + 2 f + 1] = the sum over shards is done; ms[4 parts] = the
 * layer's last kernel is done. *count = 4 parts + 1 (0 if there was no such call); ms may be null to ask for the count. */
wb200_status wb200_decoder_layer_timeline(wb200_backend *backend, float *ms, uint32_t capacity, uint32_t *count);

/* Sum over the shards of a tensor-parallel region (the `allreduce` of wb200_decoder_layer, or any buffer) as one kernel
 * per GPU that lets the NVSwitch add and broadcast: the reference's Tile collectives realise such a sum as reduce-scatter
 * followed by all-gather over the dies (lib/Wafer/Transforms/Tile/DistributedCollectiveMovement.cpp:675-735); here rank
 * r reads the r-th slice of the buffer through an NVLink multicast address with multimem.ld_reduce (one sum of all
 * ranks' values comes back, accumulated in f32) and stores it through the same address with multimem.st (it lands in
 * every rank's buffer). In place; all ranks end with bit-identical values.
 *   multicast   the multicast address of this call's buffer: the buffer must lie at the same offset of a symmetric
 *               allocation on every rank, and that allocation must be bound to a multicast object (torch symmetric
 *               memory: handle.multicast_ptr + offset). 16-byte aligned, elements * size a multiple of 16 bytes.
 *   signals     every rank's signal words (peer-mapped device memory, wb200_switch_sum_signal_bytes(world) bytes each,
 *               zero-initialised), [rank] this rank's own
 *   epoch       two zero-initialised 32-bit words in this rank's device memory; the kernel advances them
 *   blocks      thread blocks of the kernel (0: 32). Beside persistent compute kernels, give it the SMs they leave free.
 * Every rank must make the same sequence of calls per signal area; calls that may overlap in time need areas of their
 * own. The waits on the other ranks are bounded (about a second): a rank that never arrives leaves
 * WB200_ERR_DEVICE_TIMEOUT for the next wb200_backend_poll, not a hung GPU. */
typedef struct wb200_switch_sum_params {
  uint32_t rank, world;
  void *multicast;
  uint64_t elements;
  uint32_t format;             /* WB200_BF16, WB200_F16 or WB200_F32 */
  uint32_t blocks;
  void *signals[WB200_MAX_EXCHANGE_RANKS];
  uint32_t *epoch;
  void *stream;
  void *multicast_out;         /* optional: multicast address (same allocation rules) the sums are stored to instead of the
                                  buffer itself */
  const void *residual;        /* optional: this rank's device copy of a tensor of the same extent and format, identical on
                                  every rank, added to the sums before the store: out = round(sum + residual). The decoder
                                  layer's residual adds ride in the sum this way */
} wb200_switch_sum_params;
uint64_t wb200_switch_sum_signal_bytes(uint32_t world);
wb200_status wb200_switch_sum(wb200_backend *backend, const wb200_switch_sum_params *params);

/* Reads and clears the device status word of asynchronous (WB200_MEM_DEVICE) calls after
 * synchronising `stream`. Returns WB200_ERR_DEVICE_TIMEOUT if a kernel gave up a bounded wait. */
wb200_status wb200_backend_poll(wb200_backend *backend, void *stream);

/* Self-test of the bounded device-side waits: launches a kernel that waits, for at most `cycle_limit` SM clocks, on a
 * barrier nothing arrives on. The kernel gives up, records the timeout and returns; the call reports the cycles it
 * waited, and the next wb200_backend_poll(backend, NULL) returns WB200_ERR_DEVICE_TIMEOUT (and clears it). Replaces
 * nothing in the reference: its commands run synchronously on the host and cannot time out. */
wb200_status wb200_selftest_bounded_wait(wb200_backend *backend, uint64_t cycle_limit, uint64_t *waited_cycles);

/* Number of kernels this backend has launched since creation (for bench accounting). */
uint64_t wb200_backend_launch_count(const wb200_backend *backend);

/* ------------------------------------------------------------------ TargetCall ABI (Seam 2) */
/* Decoded argument vectors of the wafer_tx81_* calls, same field order as the reference decoder
 * (lib/Wafer/Target/TargetCallDecoder.cpp:99-134, 231-308). Addresses are byte offsets into one
 * flat device-resident image of a Tile's scratch-pad memory owned by the backend. */
typedef struct wb200_spm_image wb200_spm_image;
wb200_status wb200_spm_create(wb200_backend *backend, uint64_t base_address, uint64_t bytes,
                              wb200_spm_image **out);
void wb200_spm_destroy(wb200_spm_image *image);
wb200_status wb200_spm_write(wb200_spm_image *image, uint64_t address, const uint8_t *src, uint64_t bytes);
wb200_status wb200_spm_read(wb200_spm_image *image, uint64_t address, uint8_t *dst, uint64_t bytes);
/* wafer_tx81_gemm(lhs, rhs, dst, psum : i64; m, k, n, batch, inFmt, outFmt, psumFmt, lhsOri, rhsOri)
 * psumFmt == WB200_FORMAT_NONE means no partial sum (include/Wafer/Target/TargetCall.h:72). */
wb200_status wb200_target_call_gemm(wb200_spm_image *image, uint64_t lhs, uint64_t rhs, uint64_t dst,
                                    uint64_t psum, uint32_t m, uint32_t k, uint32_t n, uint32_t batch,
                                    uint32_t in_format, uint32_t out_format, uint32_t psum_format,
                                    uint32_t lhs_orientation, uint32_t rhs_orientation,
                                    uint32_t policy);

/* Movement commands of the TargetCall ABI on device-resident memory images, same argument order as the reference
 * decoder (lib/Wafer/Target/TargetCallDecoder.cpp:52-81); executors replaced:
 * lib/Wafer/Simulator/Kernel/TargetModelMovement.cpp:52-146 (strided DMA, gather / scatter) and
 * lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:874-899 (memset). A strided byte layout is
 * {inner_bytes, strides[3], iterations[3]}, dimension 0 fastest; byte_count must equal inner_bytes * segments.
 *   rdma:  DDR image, strided  -> scratch-pad image, contiguous
 *   wdma:  scratch-pad image, contiguous -> DDR image, strided
 *   gather_scatter: scratch-pad strided -> same scratch-pad strided, with snapshot semantics (the whole source is
 *                   read before anything is written; overlapping ranges go through a staging buffer)
 *   memset: element_count elements of `format` set to the low bits of `value_bits`
 * Synchronous: each call returns after its kernels have completed. */
wb200_status wb200_target_call_rdma(wb200_spm_image *ddr, wb200_spm_image *spm, uint64_t source, uint64_t destination,
                                    uint32_t byte_count, uint32_t inner_bytes, const uint32_t strides[3],
                                    const uint32_t iterations[3]);
wb200_status wb200_target_call_wdma(wb200_spm_image *spm, wb200_spm_image *ddr, uint64_t source, uint64_t destination,
                                    uint32_t byte_count, uint32_t inner_bytes, const uint32_t strides[3],
                                    const uint32_t iterations[3]);
wb200_status wb200_target_call_gather_scatter(wb200_spm_image *spm, uint64_t source, uint64_t destination,
                                              uint32_t byte_count, uint32_t inner_bytes,
                                              const uint32_t source_strides[3], const uint32_t source_iterations[3],
                                              const uint32_t destination_strides[3],
                                              const uint32_t destination_iterations[3]);
wb200_status wb200_target_call_memset(wb200_spm_image *spm, uint64_t destination, uint32_t value_bits,
                                      uint32_t element_count, uint32_t format);

/* wafer_tx81_bit2fp (lib/Wafer/Target/TargetCall.cpp:142, lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:198-236): bit i of
 * the packed Bool vector at `source` (least significant bit first) becomes 1.0 or +0 of `format` (F16 / BF16 / F32). */
wb200_status wb200_target_call_bit2fp(wb200_spm_image *spm, uint64_t source, uint64_t destination, uint32_t element_count, uint32_t format);
/* wafer_tx81_mask_move (TargetCall.cpp:143-145, TargetModelTensorNumeric.cpp:238-286): destination elements whose mask element is
 * exactly 1.0 take the source element, a zero mask keeps them; any other mask value (-0 included) refuses the command with
 * WB200_ERR_UNSUPPORTED before anything is written. */
wb200_status wb200_target_call_mask_move(wb200_spm_image *spm, uint64_t source, uint64_t mask, uint64_t destination, uint32_t element_count,
                                         uint32_t format);
/* wafer_tx81_elementwise_<op> on a scratch-pad image (lib/Wafer/Target/TargetCall.cpp:86-95, decode
 * lib/Wafer/Target/TargetCallDecoder.cpp:231-268): operands are 1-D Tensor vectors of `count` elements of `format`;
 * relations write bit-packed Bool, or 1.0 / 0.0 of `format` when `relation_numeric_or_rhs_group` is 1; logic calls write
 * Bool. Arithmetic and relation calls take the second operand in one of four forms
 * (lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:296-372): a full vector; a unit of `rhs_unit_elements`
 * elements repeated (index % unit); for arithmetic calls one 64-element row per group of `relation_numeric_or_rhs_group`
 * elements (index / group * 64 + index % 64); or, with `scalar_flag` = 1, the immediate bits in `rhs_or_scalar_bits`.
 * Unary and logic calls ignore the three extra fields. Every form runs the formal family of wb200_elementwise_formal;
 * `flags` (may be null) receives the OR of the IEEE flags. */
wb200_status wb200_target_call_elementwise(wb200_spm_image *image, uint32_t operation, uint64_t lhs, uint64_t rhs_or_scalar_bits,
                                           uint64_t dst, uint32_t count, uint32_t format, uint32_t rhs_unit_elements,
                                           uint32_t scalar_flag, uint32_t relation_numeric_or_rhs_group, uint32_t *flags);
/* wafer_tx81_convert_<route> on a scratch-pad image (lib/Wafer/Target/TargetCall.cpp:101-106, decode
 * lib/Wafer/Target/TargetCallDecoder.cpp:283-308): 1-D Tensor vectors of `count` elements in the route's formats, executed
 * by the formal conversion of wb200_convert_formal. A refused element fails the call before anything is written. */
wb200_status wb200_target_call_convert(wb200_spm_image *image, uint32_t opcode, uint64_t source, uint64_t destination, uint32_t count,
                                       uint32_t zero_point, uint32_t rounding_mode, uint32_t *flags);
/* wafer_tx81_reduce_{sum,max,min} (operation 0 / 1 / 2) on a scratch-pad image (lib/Wafer/Target/TargetCall.cpp:97-99, decode
 * lib/Wafer/Target/TargetCallDecoder.cpp:270-281): NCx [n, h, w, c] input, NCx destination with the reduced dimensions set to 1,
 * `dimension` a wb200_reduce_dimension; executed by the formal fold of wb200_reduce_formal. */
wb200_status wb200_target_call_reduce(wb200_spm_image *image, uint32_t operation, uint64_t source, uint64_t destination, uint32_t dimension,
                                      const uint32_t nhwc[4], uint32_t format, uint32_t *flags);
/* wafer_tx81_pool_{sum,max,min} (kind 116 / 117 / 119; lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:466-583):
 * NCx [n, h, w, c] input and output, `kernel_strides` = {kernel w, kernel h, stride w, stride h}, all `pads` zero; each
 * output folds its window in (kh, kw) order with the formal max / min, or for sum (F32 only) adds every tap to +0.
 * Average and the indexed kinds are declined like in the reference. */
wb200_status wb200_target_call_pool(wb200_spm_image *image, uint32_t kind, uint64_t input, uint64_t dst, const uint32_t source_shape[4],
                                    const uint32_t destination_shape[4], const uint32_t pads[4], const uint32_t kernel_strides[4],
                                    uint32_t format, uint32_t *flags);

/* ------------------------------------------------------------------ Tile program replay (Seam 2, whole invocation) */
/* Executes the per-Tile target LLVM modules the reference compiler emits (text form, one module per Tile) the way the
 * reference's host execution does: it admits the closed integer subset of LLVM IR of
 * lib/Wafer/Simulator/Invocation/TargetCallExecution.cpp:188-294 (integer binary ops, icmp, phi, select, casts, freeze,
 * br / switch, smin / smax / umin / umax, calls to wafer_tx81_* descriptors) and routes every wafer_tx81_* call to
 * the device executors above in place of waferTargetCallDispatch (TargetCallExecution.cpp:116-119). Tiles run as
 * cooperatively scheduled interpreters on the calling thread, like the reference's SC_THREAD coroutines; Direct-DTE
 * sends and receives are matched by (sender Tile, receiver Tile, receiver FSM) and a send issue blocks until its
 * receiver is prepared (lib/Wafer/Simulator/SystemC/SystemCTargetModel.cpp:1110-1200). Entry arguments are planned
 * from the !wafer.target.entry_arguments metadata (lib/Wafer/CodeGen/LLVM/TargetLLVMTranslation.cpp:119-140) into one
 * DDR arena. Calls outside {ncc_join, direct_dte_{begin,begin_after_prepare,send_prepare,send_issue,recv_prepare,wait,
 * finish}, rdma, wdma, gather_scatter, memset, gemm, gemm_oriented, elementwise_<op>, convert_<route>, reduce_<op>, pool_<sum|max|min>, bit2fp, mask_move} are rejected with
 * WB200_ERR_UNSUPPORTED at load. Elementwise, convert and reduce calls run the formal families of wb200_target_call_elementwise /
 * wb200_target_call_convert / wb200_target_call_reduce; a convert element the reference refuses fails the run after the command stream has drained.
 * A run of arithmetic / function elementwise commands of one Tile, same format and element count, each taking the previous
 * command's destination as its first operand (second operand: a same-index vector or an immediate), is issued as one
 * kernel launch that still writes every command's destination; the scratch-pad ends bit-identical to the
 * command-by-command replay and gpu_launches counts the fused launch once. WB200_REPLAY_FUSE=0 in the environment at load
 * time issues every command on its own; WB200_REPLAY_GRAPH=0 at run time replays without the captured CUDA graph. */
typedef struct wb200_tile_program wb200_tile_program;
typedef struct wb200_program_stats {
  uint64_t instructions;              /* IR instructions interpreted */
  uint64_t commands;                  /* wafer_tx81_* calls issued */
  uint64_t gemm_commands, movement_commands, fill_commands, transfer_commands, sync_commands;
  uint64_t gemm_fused_multiply_adds;  /* sum of m * k * n * batch */
  uint64_t bytes_moved;               /* payload bytes of DMA, gather / scatter, fill and Direct-DTE transfers */
  uint64_t gpu_launches;
  float device_ms;                    /* command stream only (CUDA events); excludes host <-> device tensor copies */
  uint32_t numeric_flags;             /* OR of the IEEE flags of all elementwise / convert / reduce / pool commands (bit 0 invalid .. bit 4 inexact) */
} wb200_program_stats;
/* One issued command in a trace: `kind` indexes wb200_program_command_name(); args in ABI order without the worker.
 * The trace also holds one "direct_dte_transfer" record (sender Tile, receiver Tile, source, destination, bytes) at
 * the point of the command order where a matched Direct-DTE payload moves. */
typedef struct wb200_program_command {
  uint32_t tile, kind, argc;
  uint32_t operation; /* elementwise operation (wb200_elementwise_op) or convert opcode of the symbol-selected families, else 0 */
  uint64_t args[20];
} wb200_program_command;

/* `backend` may be null: the program can then be inspected and traced but not run. `spm_bytes` is the scratch-pad
 * capacity per Tile (0: 3 MiB). */
wb200_status wb200_tile_program_load(wb200_backend *backend, const char *const *module_texts, uint32_t tile_count,
                                     uint64_t spm_bytes, wb200_tile_program **out);
void wb200_tile_program_destroy(wb200_tile_program *program);
/* External tensors in resource-index order. `compact_bytes` is the row-major size run() exchanges. */
wb200_status wb200_tile_program_tensor_count(const wb200_tile_program *program, uint32_t *inputs, uint32_t *outputs);
wb200_status wb200_tile_program_tensor_info(const wb200_tile_program *program, uint32_t is_output, uint32_t index,
                                            wb200_tensor_desc *desc, uint64_t *compact_bytes);
/* Where the address plan put an external tensor: its DDR address and physical size, and the arena's extent. */
wb200_status wb200_tile_program_placement(const wb200_tile_program *program, uint32_t is_output, uint32_t index,
                                          uint64_t *address, uint64_t *physical_bytes, uint64_t *ddr_base,
                                          uint64_t *ddr_bytes);
/* Interprets all Tiles without touching a device and records the issued commands in scheduling order.
 * `records` may be null to query `count`. */
wb200_status wb200_tile_program_trace(wb200_tile_program *program, wb200_program_command *records, uint64_t capacity,
                                      uint64_t *count, wb200_program_stats *stats);
const char *wb200_program_command_name(uint32_t kind);
/* Runs the invocation: host compact row-major inputs are packed into their physical DDR layout, all Tiles execute,
 * outputs are unpacked to `outputs`. `gemm_policy`: wb200_gemm_policy for psum-free, untransposed GEMM commands
 * (commands with a partial sum always take the bit-exact sequential-k path). */
wb200_status wb200_tile_program_run(wb200_tile_program *program, const void *const *inputs, void *const *outputs,
                                    uint32_t gemm_policy, wb200_program_stats *stats);

/* ------------------------------------------------------------------ Expected-output comparison (acceptance gate) */
/* Device evaluation of the reference's output gate: compareProgramTensorExpectedOutput and
 * computeProgramTensorComparisonStatistics (lib/Wafer/Simulator/Invocation/ProgramTensorComparison.cpp:276-403,
 * :405-503) on two compact little-endian tensors of one floating format. Values are decoded exactly to f64; the
 * absolute error, the tolerance atol + rtol * |expected| (two separate roundings, no contraction), the ULP distance on
 * the sign-magnitude order key and every count are the reference's own f64 / integer results. Quantiles are the
 * nearest-rank order statistics (rank = ceil(q * n), clamped to [1, n]) found by an exact radix select. The four
 * similarity sums and the two means, which the reference accumulates sequentially in x87 extended precision, are
 * accumulated in double-double (about 106 bits) and rounded once, so cosine, relative_l2, mean_abs and mean_ulp agree
 * with the reference to within a few units of 1e-16 relative rather than bit for bit. */
typedef enum wb200_comparison_outcome {
  WB200_CMP_MATCH = 0,
  WB200_CMP_INVALID_TOLERANCE = 1,  /* negative / non-finite tolerance, or atol + rtol * |expected| overflowed */
  WB200_CMP_ACTUAL_NONFINITE = 2,
  WB200_CMP_EXPECTED_NONFINITE = 3,
  WB200_CMP_NUMERIC_MISMATCH = 4,
  WB200_CMP_EMPTY = 5,              /* similarity was requested on an empty tensor */
  WB200_CMP_RAW_MISMATCH = 6        /* wb200_compare_raw only */
} wb200_comparison_outcome;
typedef struct wb200_comparison {
  uint32_t outcome;  /* wb200_comparison_outcome */
  uint32_t reserved;
  uint64_t element;  /* the element (or byte) the outcome names: first non-finite / overflowing / differing one */
  uint64_t element_count, exact_count, mismatch_count;
  double exact_fraction, mean_abs, p99_abs, p999_abs, max_abs;
  double cosine, relative_l2, mean_ulp;
  uint64_t p99_ulp, p999_ulp, max_ulp;
  /* Elementwise mismatches (|actual - expected| > tolerance), in the reference's tie rules: the first in index order,
   * the first one attaining the largest absolute error, the first one attaining the largest error / tolerance. */
  uint64_t first_mismatch, max_abs_mismatch, max_ratio_mismatch;
  char detail[512];  /* the reference's detail text for a failing outcome (its "%e" number format); empty on a match */
} wb200_comparison;
/* `format`: WB200_F16, WB200_BF16 or WB200_F32; `memory`: where `actual` and `expected` live (wb200_memory).
 * `use_similarity` != 0 selects the cosine / relative-L2 gate (minimum_cosine in [0, 1], maximum_relative_l2 >= 0);
 * otherwise every element must be within tolerance. Statistics are filled whenever the tensors are non-empty and
 * finite. The status is WB200_OK for every outcome; it reports only malformed calls and CUDA failures. */
wb200_status wb200_compare(wb200_backend *backend, uint32_t format, uint64_t count, const void *actual,
                           const void *expected, uint32_t memory, double atol, double rtol, uint32_t use_similarity,
                           double minimum_cosine, double maximum_relative_l2, wb200_comparison *out);
/* Exact comparison for every non-floating element type (ProgramTensorComparison.cpp:306-323): outcome MATCH or
 * RAW_MISMATCH with `element` = the first differing byte. */
wb200_status wb200_compare_raw(wb200_backend *backend, uint64_t bytes, const void *actual, const void *expected,
                               uint32_t memory, wb200_comparison *out);

#ifdef __cplusplus
}
#endif
#endif /* WB200_H */
