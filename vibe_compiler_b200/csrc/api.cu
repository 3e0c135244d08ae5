// C-ABI entry points of libwb200.so (declared in include/wb200.h). This layer validates requests the
// way the reference's command executors do (lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp,
// lib/Wafer/Simulator/Reference/ManagedReferenceTargetModel.cpp), owns device staging memory and
// dispatches to the kernels. It never computes results on the host.
#include "backend.h"

using namespace wb200;

extern "C" {

int wb200_abi_version(void) { return WB200_ABI_VERSION; }
const char *wb200_last_error(void) { return last_error_cstr(); }

wb200_status wb200_backend_create(int device, wb200_backend **out) {
  if (!out) return fail(WB200_ERR_INVALID_ARGUMENT, "out pointer is null");
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
    cudaGetLastError();
    return fail(WB200_ERR_NO_DEVICE, "no CUDA device is visible; this backend has no CPU path");
  }
  if (device < 0 || device >= count) return fail(WB200_ERR_NO_DEVICE, "CUDA device index out of range");
  cudaDeviceProp prop;
  WB200_CUDA_CHECK(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(WB200_ERR_NO_DEVICE, std::string("device '") + prop.name + "' is not compute capability 10.x (sm_100a kernels only)");
  DeviceGuard guard(device);
  wb200_backend *backend = new wb200_backend();
  backend->device = device;
  backend->sm_count = prop.multiProcessorCount;
  snprintf(backend->digest, sizeof(backend->digest), "b200:%s:sm_%d%d:abi%d", prop.name, prop.major, prop.minor, WB200_ABI_VERSION);
  cudaError_t err = cudaStreamCreateWithFlags(&backend->stream, cudaStreamNonBlocking);
  if (err == cudaSuccess) err = cudaMalloc(&backend->d_status, 2 * sizeof(int));
  if (err == cudaSuccess) err = cudaMemset(backend->d_status, 0, 2 * sizeof(int));
  if (err != cudaSuccess) {
    delete backend;
    return fail(WB200_ERR_CUDA, std::string("backend setup: ") + cudaGetErrorString(err));
  }
  *out = backend;
  return WB200_OK;
}

void wb200_backend_destroy(wb200_backend *backend) {
  if (!backend) return;
  DeviceGuard guard(backend->device);
  cudaStreamSynchronize(backend->stream);
  for (auto &slot : backend->slots)
    if (slot.ptr) cudaFree(slot.ptr);
  if (backend->d_status) cudaFree(backend->d_status);
  for (cudaStream_t aux : backend->aux_stream)
    if (aux) { cudaStreamSynchronize(aux); cudaStreamDestroy(aux); }
  for (cudaEvent_t event : backend->aux_event)
    if (event) cudaEventDestroy(event);
  for (cudaEvent_t event : backend->pipeline_event) cudaEventDestroy(event);
  for (cudaEvent_t event : backend->timing_event)
    if (event) cudaEventDestroy(event);
  if (backend->stream) cudaStreamDestroy(backend->stream);
  delete backend;
}

wb200_status wb200_backend_set_budget(wb200_backend *backend, uint64_t max_total_bytes, uint64_t max_scratch_bytes) {
  if (!backend) return fail(WB200_ERR_INVALID_ARGUMENT, "backend is null");
  backend->max_total_bytes = max_total_bytes;
  backend->max_scratch_bytes = max_scratch_bytes;
  return WB200_OK;
}

uint64_t wb200_backend_launch_count(const wb200_backend *backend) { return backend ? backend->launches : 0; }

wb200_status wb200_backend_poll(wb200_backend *backend, void *stream) {
  if (!backend) return fail(WB200_ERR_INVALID_ARGUMENT, "backend is null");
  DeviceGuard guard(backend->device);
  return read_device_status(backend, static_cast<cudaStream_t>(stream), nullptr);
}

wb200_status wb200_physical_geometry(const wb200_tensor_desc *desc, wb200_geometry *out) {
  if (!desc || !out) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  return make_layout_map(*desc, nullptr, out);
}

wb200_status wb200_physical_bytes(const wb200_tensor_desc *desc, uint64_t *out_bytes) {
  if (!desc || !out_bytes) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  wb200_geometry g;
  wb200_status st = make_layout_map(*desc, nullptr, &g);
  if (st == WB200_OK) *out_bytes = static_cast<uint64_t>(g.physical_bytes);
  return st;
}

wb200_status wb200_unpack(wb200_backend *backend, const wb200_tensor_desc *desc, const uint8_t *storage,
                          uint64_t storage_bytes, uint8_t *compact_out, uint64_t compact_bytes) {
  if (!backend || !desc || !compact_out) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  LayoutMap map; wb200_geometry g;
  wb200_status st = check_storage(*desc, storage_bytes, storage, "unpack source", &map, &g);
  if (st != WB200_OK) return st;
  if (format_bits(desc->format) < 8) return fail(WB200_ERR_UNSUPPORTED, "bit-packed formats are not handled by the device codec");
  if (compact_bytes != static_cast<uint64_t>(g.compact_bytes)) return fail(WB200_ERR_INVALID_ARGUMENT, "compact size mismatch");
  DeviceGuard guard(backend->device);
  void *d_storage, *d_compact;
  if ((st = backend->buffer(0, storage_bytes, &d_storage)) != WB200_OK) return st;
  if ((st = backend->buffer(1, compact_bytes, &d_compact)) != WB200_OK) return st;
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_storage, storage, storage_bytes, cudaMemcpyHostToDevice, backend->stream));
  st = launch_unpack(static_cast<const uint8_t *>(d_storage), static_cast<uint8_t *>(d_compact), map, static_cast<int>(g.element_bytes), backend->stream);
  if (st != WB200_OK) return st;
  backend->launches += 1;
  WB200_CUDA_CHECK(cudaMemcpyAsync(compact_out, d_compact, compact_bytes, cudaMemcpyDeviceToHost, backend->stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(backend->stream));
  return WB200_OK;
}

wb200_status wb200_pack(wb200_backend *backend, const wb200_tensor_desc *desc, const uint8_t *compact,
                        uint64_t compact_bytes, const uint8_t *storage_template, uint8_t *storage_out,
                        uint64_t storage_bytes) {
  if (!backend || !desc || !compact || !storage_out) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  LayoutMap map; wb200_geometry g;
  wb200_status st = check_storage(*desc, storage_bytes, storage_template, "pack template", &map, &g);
  if (st != WB200_OK) return st;
  if (format_bits(desc->format) < 8) return fail(WB200_ERR_UNSUPPORTED, "bit-packed formats are not handled by the device codec");
  if (compact_bytes != static_cast<uint64_t>(g.compact_bytes)) return fail(WB200_ERR_INVALID_ARGUMENT, "compact size mismatch");
  DeviceGuard guard(backend->device);
  void *d_storage, *d_compact;
  if ((st = backend->buffer(0, storage_bytes, &d_storage)) != WB200_OK) return st;
  if ((st = backend->buffer(1, compact_bytes, &d_compact)) != WB200_OK) return st;
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_storage, storage_template, storage_bytes, cudaMemcpyHostToDevice, backend->stream));
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_compact, compact, compact_bytes, cudaMemcpyHostToDevice, backend->stream));
  st = launch_pack(static_cast<const uint8_t *>(d_compact), static_cast<uint8_t *>(d_storage), map, static_cast<int>(g.element_bytes), backend->stream);
  if (st != WB200_OK) return st;
  backend->launches += 1;
  WB200_CUDA_CHECK(cudaMemcpyAsync(storage_out, d_storage, storage_bytes, cudaMemcpyDeviceToHost, backend->stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(backend->stream));
  return WB200_OK;
}

}  // extern "C"
