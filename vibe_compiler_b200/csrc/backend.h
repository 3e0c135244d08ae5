// Internal definition of the backend object and request-validation helpers shared by the C-ABI
// translation units.
#pragma once

#include <string.h>

#include <string>
#include <vector>

#include "kernels.h"

namespace wb200 {
const char *last_error_cstr();
}

struct wb200_backend {
  int device = 0;
  int sm_count = 0;
  cudaStream_t stream = nullptr;  // used by WB200_MEM_HOST calls
  int *d_status = nullptr;        // [0] bounded-wait status, [1] NaN flag
  uint64_t launches = 0;
  uint64_t max_total_bytes = 0, max_scratch_bytes = 0;
  char digest[96] = {0};
  struct Slot { void *ptr = nullptr; size_t bytes = 0; };
  std::vector<Slot> slots;
  // Two auxiliary streams and three events for calls that overlap independent parts of their work (created on first use).
  cudaStream_t aux_stream[2] = {nullptr, nullptr};
  cudaEvent_t aux_event[3] = {nullptr, nullptr, nullptr};
  cudaEvent_t timing_event[2] = {nullptr, nullptr};   // brackets the kernels of one command call (created on first use)
  wb200_status timing_begin(cudaStream_t s) {
    if (!timing_event[0])
      for (int i = 0; i < 2; ++i) WB200_CUDA_CHECK(cudaEventCreate(&timing_event[i]));
    WB200_CUDA_CHECK(cudaEventRecord(timing_event[0], s));
    return WB200_OK;
  }
  // Call after the stream has been synchronised past timing_end()'s record.
  wb200_status timing_end(cudaStream_t s) {
    WB200_CUDA_CHECK(cudaEventRecord(timing_event[1], s));
    return WB200_OK;
  }
  uint32_t timing_microseconds() const {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, timing_event[0], timing_event[1]) != cudaSuccess) return 0;
    return static_cast<uint32_t>(ms * 1000.f + 0.5f);
  }
  std::vector<cudaEvent_t> pipeline_event;   // edges of host-buffer pipelines, grown on demand
  uint32_t layer_timeline_parts = 0;         // parts of the last micro-batched decoder layer call (its events are still there)
  wb200_status pipeline_events(size_t count) {
    while (pipeline_event.size() < count) {
      cudaEvent_t event;
      WB200_CUDA_CHECK(cudaEventCreate(&event));   // with timing: wb200_decoder_layer_timeline reads them
      pipeline_event.push_back(event);
    }
    return WB200_OK;
  }
  wb200_status auxiliary_streams() {
    if (aux_stream[0]) return WB200_OK;
    // highest priority: the blocks of a sum or a copy enqueued here are placed before the queued blocks of the compute
    // kernels they run beside
    int least = 0, greatest = 0;
    WB200_CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&least, &greatest));
    for (int i = 0; i < 2; ++i) WB200_CUDA_CHECK(cudaStreamCreateWithPriority(&aux_stream[i], cudaStreamNonBlocking, greatest));
    for (int i = 0; i < 3; ++i) WB200_CUDA_CHECK(cudaEventCreateWithFlags(&aux_event[i], cudaEventDisableTiming));
    return WB200_OK;
  }

  // Grow-only staging buffer number `index`.
  wb200_status buffer(size_t index, size_t bytes, void **out) {
    if (slots.size() <= index) slots.resize(index + 1);
    Slot &slot = slots[index];
    if (slot.bytes < bytes) {
      if (slot.ptr) cudaFree(slot.ptr);
      slot.ptr = nullptr;
      slot.bytes = 0;
      const size_t rounded = ((bytes + 255) / 256) * 256;
      WB200_CUDA_CHECK(cudaMalloc(&slot.ptr, rounded));
      slot.bytes = rounded;
    }
    *out = slot.ptr;
    return WB200_OK;
  }
  // The same, zero-filled whenever it is (re)allocated: for counters that the kernels using them leave at zero.
  wb200_status zeroed_buffer(size_t index, size_t bytes, void **out) {
    const size_t before = slots.size() > index ? slots[index].bytes : 0;
    wb200_status st = buffer(index, bytes, out);
    if (st != WB200_OK) return st;
    if (slots[index].bytes != before) WB200_CUDA_CHECK(cudaMemset(*out, 0, slots[index].bytes));
    return WB200_OK;
  }
};

// One flat device-resident memory image (a Tile's scratch-pad, or a DDR arena) addressed by the byte
// addresses the TargetCall ABI carries.
struct wb200_spm_image {
  wb200_backend *backend;
  uint64_t base, bytes;
  uint8_t *device;
  cudaStream_t stream = nullptr;     // null: the backend stream
  uint8_t *staging = nullptr;        // private scratch of `bytes` bytes for in-place gather / scatter (null: a backend slot)
  uint8_t *gemm_staging = nullptr;   // private scratch of 3 * `bytes` bytes for the tensor-core GEMM's compact operands (null: backend slots)
  cudaStream_t work_stream() const { return stream ? stream : backend->stream; }
};

namespace wb200 {

wb200_status image_range(const wb200_spm_image *image, uint64_t address, uint64_t bytes, const char *what);
// wafer_tx81_gemm on a scratch-pad image, enqueued on the backend stream without synchronising.
// `defer` (here and in the elementwise and reduce forms): when given, nothing is launched: the validated command is
// described there and *deferred says whether it fits a command run (formal_run_admits); the caller launches the run, or,
// when the command does not fit, calls again without `defer`.
wb200_status enqueue_image_gemm(wb200_spm_image *image, uint64_t lhs, uint64_t rhs, uint64_t dst, uint64_t psum,
                                uint32_t m, uint32_t k, uint32_t n, uint32_t batch, uint32_t in_format,
                                uint32_t out_format, uint32_t psum_format, uint32_t lhs_orientation,
                                uint32_t rhs_orientation, uint32_t policy, RunCommand *defer = nullptr, bool *deferred = nullptr);

wb200_status enqueue_image_elementwise(wb200_spm_image *image, uint32_t operation, uint64_t lhs, uint64_t rhs_or_scalar_bits,
                                       uint64_t dst, uint32_t count, uint32_t format, uint32_t rhs_unit_elements,
                                       uint32_t scalar_flag, uint32_t relation_numeric_or_rhs_group, uint32_t *d_flags, bool execute,
                                       RunCommand *defer = nullptr, bool *deferred = nullptr);
wb200_status enqueue_image_reduce(wb200_spm_image *image, uint32_t operation, uint64_t source, uint64_t destination, uint32_t dimension,
                                  const uint32_t nhwc[4], uint32_t format, uint32_t *d_flags, bool execute, RunCommand *defer = nullptr,
                                  bool *deferred = nullptr);
wb200_status enqueue_image_pool(wb200_spm_image *image, uint32_t kind, uint64_t input, uint64_t dst, const uint32_t source_shape[4],
                                const uint32_t destination_shape[4], const uint32_t pads[4], const uint32_t kernel_strides[4],
                                uint32_t format, uint32_t *d_flags, bool execute);

wb200_status enqueue_image_convert(wb200_spm_image *image, uint32_t opcode, uint64_t source, uint64_t destination, uint32_t count,
                                   uint32_t rounding_mode, bool execute, uint32_t *d_flags, unsigned long long *d_error);
wb200_status convert_refusal(unsigned long long key);   // the error of a refused element key (element << 8 | code)

struct DeviceGuard {
  int previous = -1;
  explicit DeviceGuard(int device) {
    cudaGetDevice(&previous);
    if (previous != device) cudaSetDevice(device);
    else previous = -1;
  }
  ~DeviceGuard() { if (previous >= 0) cudaSetDevice(previous); }
};

inline void fill_evidence(const wb200_backend *backend, wb200_evidence *evidence, const char *implementation) {
  if (!evidence) return;
  memset(evidence, 0, sizeof(*evidence));
  evidence->evidence_kind = 2;
  strncpy(evidence->digest, backend->digest, sizeof(evidence->digest) - 1);
  strncpy(evidence->implementation, implementation, sizeof(evidence->implementation) - 1);
}

// Reads and clears the device status words. status[0] != 0 -> a bounded wait gave up.
inline wb200_status read_device_status(wb200_backend *backend, cudaStream_t stream, int *nan_flag) {
  int host[2] = {0, 0};
  WB200_CUDA_CHECK(cudaMemcpyAsync(host, backend->d_status, sizeof(host), cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  if (host[0] != 0 || host[1] != 0) {
    WB200_CUDA_CHECK(cudaMemsetAsync(backend->d_status, 0, sizeof(host), stream));
    WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  }
  if (nan_flag) *nan_flag = host[1];
  if (host[0] != 0) return fail(WB200_ERR_DEVICE_TIMEOUT, "a device-side bounded wait gave up (status " + std::to_string(host[0]) + ")");
  return WB200_OK;
}

inline wb200_status check_storage(const wb200_tensor_desc &desc, uint64_t bytes, const void *ptr, const char *what,
                           LayoutMap *map, wb200_geometry *geometry) {
  wb200_status st = make_layout_map(desc, map, geometry);
  if (st != WB200_OK) return st;
  if (!ptr) return fail(WB200_ERR_INVALID_ARGUMENT, std::string(what) + " storage pointer is null");
  if (bytes != static_cast<uint64_t>(geometry->physical_bytes))
    return fail(WB200_ERR_INVALID_ARGUMENT, std::string(what) + " storage size does not match its physical geometry");
  return WB200_OK;
}

inline bool same_shape(const wb200_tensor_desc &a, const wb200_tensor_desc &b) {
  if (a.rank != b.rank) return false;
  for (int d = 0; d < a.rank; ++d)
    if (a.shape[d] != b.shape[d]) return false;
  return true;
}

inline wb200_status check_budget(const wb200_backend *backend, uint64_t scalar_evaluations, uint64_t max_scalar,
                          uint64_t total_bytes, uint64_t logical_values) {
  if (scalar_evaluations > max_scalar) return fail(WB200_ERR_BUDGET, "scalar evaluation budget exceeded");
  if (backend->max_total_bytes && total_bytes > backend->max_total_bytes)
    return fail(WB200_ERR_BUDGET, "physical byte budget exceeded");
  // The reference accounts 16 bytes of scratch per logical value (sizeof(RawLogicalValue)).
  if (backend->max_scratch_bytes && logical_values * 16 > backend->max_scratch_bytes)
    return fail(WB200_ERR_BUDGET, "logical scratch budget exceeded");
  return WB200_OK;
}

}  // namespace wb200

