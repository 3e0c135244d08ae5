// Command-level entry points: the four tensor commands the reference's functional model offers to
// its numeric backends, executed on physical storage bytes. Validation mirrors
// lib/Wafer/Simulator/Reference/ManagedReferenceTargetModel.cpp:301-319, 344-364, 381-400 and
// lib/Wafer/Simulator/OneDNN/OneDNNGemmAdapter.cpp:176-210.
#include "backend.h"

using namespace wb200;

namespace {

struct DeviceGemm {
  uint32_t m, k, n, batch;
  int in_format, out_format;
  int lhs_transposed, rhs_transposed, has_psum;
  LayoutMap lhs_map, rhs_map, psum_map, dst_map;
  const uint8_t *lhs, *rhs, *psum;  // device, physical storage
  uint8_t *dst;                     // device, physical storage (pre-filled with the template)
};

// Runs one GEMM command whose operands already sit on the device. `scratch_slot` is the first of
// three backend staging slots the tensor path may use for compact operands.
// `private_staging` (three areas of `private_each` bytes) replaces the backend slots when given: commands of different
// Tiles that run side by side on streams of their own must not share the compact operands.
wb200_status run_device_gemm(wb200_backend *backend, const DeviceGemm &g, int policy, size_t scratch_slot,
                             cudaStream_t stream, const char **implementation, uint8_t *private_staging = nullptr,
                             size_t private_each = 0) {
  const bool tensor_domain = policy == WB200_GEMM_TENSOR && !g.has_psum &&
                             (g.in_format == WB200_BF16 || g.in_format == WB200_F16);
  if (tensor_domain) {
    const size_t in_bytes = 2;
    const size_t out_bytes = g.out_format == WB200_F32 ? 4 : 2;
    const size_t lhs_count = static_cast<size_t>(g.batch) * g.m * g.k, rhs_count = static_cast<size_t>(g.batch) * g.k * g.n;
    const size_t dst_count = static_cast<size_t>(g.batch) * g.m * g.n;
    GemmUmmaArgs probe{};
    probe.m = g.m; probe.n = g.n; probe.k = g.k;
    probe.in_format = g.in_format; probe.out_format = g.out_format;
    probe.lhs_transposed = g.lhs_transposed; probe.rhs_transposed = g.rhs_transposed;
    probe.epilogue = WB200_EPI_NONE;
    // Per-batch operand offsets must keep 16-byte alignment for TMA.
    const bool batch_aligned = g.batch == 1 || ((static_cast<size_t>(g.m) * g.k * in_bytes) % 16 == 0 &&
                                                (static_cast<size_t>(g.k) * g.n * in_bytes) % 16 == 0 &&
                                                (static_cast<size_t>(g.m) * g.n * out_bytes) % 16 == 0);
    void *c_lhs, *c_rhs, *c_dst;
    wb200_status st;
    if (private_staging) {
      if (lhs_count * in_bytes > private_each || rhs_count * in_bytes > private_each || dst_count * out_bytes > private_each)
        return fail(WB200_ERR_LIMIT, "GEMM operand larger than the image's private staging area");
      c_lhs = private_staging; c_rhs = private_staging + private_each; c_dst = private_staging + 2 * private_each;
    } else {
      if ((st = backend->buffer(scratch_slot, lhs_count * in_bytes, &c_lhs)) != WB200_OK) return st;
      if ((st = backend->buffer(scratch_slot + 1, rhs_count * in_bytes, &c_rhs)) != WB200_OK) return st;
      if ((st = backend->buffer(scratch_slot + 2, dst_count * out_bytes, &c_dst)) != WB200_OK) return st;
    }
    probe.a = c_lhs; probe.b = c_rhs; probe.out = c_dst;
    if (batch_aligned && gemm_umma_supports(probe)) {
      if ((st = launch_unpack(g.lhs, static_cast<uint8_t *>(c_lhs), g.lhs_map, 2, stream)) != WB200_OK) return st;
      if ((st = launch_unpack(g.rhs, static_cast<uint8_t *>(c_rhs), g.rhs_map, 2, stream)) != WB200_OK) return st;
      backend->launches += 2;
      for (uint32_t b = 0; b < g.batch; ++b) {
        GemmUmmaArgs args = probe;
        args.a = static_cast<uint8_t *>(c_lhs) + static_cast<size_t>(b) * g.m * g.k * in_bytes;
        args.b = static_cast<uint8_t *>(c_rhs) + static_cast<size_t>(b) * g.k * g.n * in_bytes;
        args.out = static_cast<uint8_t *>(c_dst) + static_cast<size_t>(b) * g.m * g.n * out_bytes;
        if ((st = launch_gemm_umma(args, backend->sm_count, backend->d_status, stream)) != WB200_OK) return st;
        backend->launches += 1;
      }
      if ((st = launch_pack(static_cast<const uint8_t *>(c_dst), g.dst, g.dst_map, static_cast<int>(out_bytes), stream)) != WB200_OK) return st;
      backend->launches += 1;
      *implementation = "sm100a-tcgen05-umma-f32acc";
      return WB200_OK;
    }
  }
  GemmFormalArgs f{};
  f.m = g.m; f.k = g.k; f.n = g.n; f.batch = g.batch;
  f.in_format = g.in_format; f.out_format = g.out_format;
  f.lhs_transposed = g.lhs_transposed; f.rhs_transposed = g.rhs_transposed;
  f.has_psum = g.has_psum;
  f.lhs = g.lhs; f.rhs = g.rhs; f.psum = g.psum; f.dst = g.dst;
  f.lhs_map = g.lhs_map; f.rhs_map = g.rhs_map; f.psum_map = g.psum_map; f.dst_map = g.dst_map;
  wb200_status st = launch_gemm_formal(f, stream);
  if (st != WB200_OK) return st;
  backend->launches += 1;
  *implementation = "sm100a-simt-sequential-k-fma";
  return WB200_OK;
}

wb200_status expect_matrix(const wb200_tensor_desc &desc, uint32_t batch, uint64_t rows, uint64_t cols, const char *what) {
  // Rank 2 for unbatched Cx operands, rank 3 [batch, rows, cols] otherwise.
  if (desc.rank == 2 && batch == 1 && desc.shape[0] == rows && desc.shape[1] == cols) return WB200_OK;
  if (desc.rank == 3 && desc.shape[0] == batch && desc.shape[1] == rows && desc.shape[2] == cols) return WB200_OK;
  return fail(WB200_ERR_INVALID_ARGUMENT, std::string(what) + " descriptor shape does not match m/k/n/batch and orientation");
}

}  // namespace

extern "C" {

wb200_status wb200_gemm(wb200_backend *backend, const wb200_gemm_request *r, int *handled, wb200_evidence *evidence) {
  if (!backend || !r || !handled) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  *handled = 0;
  if (r->m == 0 || r->k == 0 || r->n == 0 || r->batch_count == 0 || r->m > 65535 || r->n > 65535 || r->k > 16384 || r->batch_count > 4096)
    return fail(WB200_ERR_INVALID_ARGUMENT, "GEMM extents outside the command domain (m,n<=65535, k<=16384, batch<=4096)");
  if (!is_float_format(r->lhs.format) || r->lhs.format != r->rhs.format || !is_float_format(r->destination.format))
    return fail(WB200_ERR_UNSUPPORTED, "GEMM admits f16, bf16 and f32 operands of one common input format");
  if (r->destination.format != r->lhs.format && r->destination.format != WB200_F32)
    return fail(WB200_ERR_UNSUPPORTED, "GEMM destination must be the input format or f32");
  const bool lt = r->lhs_orientation == WB200_TRANSPOSE, rt = r->rhs_orientation == WB200_TRANSPOSE;
  wb200_status st;
  if ((st = expect_matrix(r->lhs, r->batch_count, lt ? r->k : r->m, lt ? r->m : r->k, "lhs")) != WB200_OK) return st;
  if ((st = expect_matrix(r->rhs, r->batch_count, rt ? r->n : r->k, rt ? r->k : r->n, "rhs")) != WB200_OK) return st;
  if ((st = expect_matrix(r->destination, r->batch_count, r->m, r->n, "destination")) != WB200_OK) return st;
  DeviceGemm g{};
  wb200_geometry lhs_geo, rhs_geo, dst_geo, psum_geo{};
  if ((st = check_storage(r->lhs, r->lhs_bytes, r->lhs_storage, "lhs", &g.lhs_map, &lhs_geo)) != WB200_OK) return st;
  if ((st = check_storage(r->rhs, r->rhs_bytes, r->rhs_storage, "rhs", &g.rhs_map, &rhs_geo)) != WB200_OK) return st;
  if ((st = check_storage(r->destination, r->destination_bytes, r->destination_template, "destination template", &g.dst_map, &dst_geo)) != WB200_OK) return st;
  if (!r->destination_out) return fail(WB200_ERR_INVALID_ARGUMENT, "destination_out is null");
  if (r->has_psum) {
    if (r->psum.format != WB200_F32) return fail(WB200_ERR_UNSUPPORTED, "psum must be f32");
    if ((st = expect_matrix(r->psum, r->batch_count, r->m, r->n, "psum")) != WB200_OK) return st;
    if ((st = check_storage(r->psum, r->psum_bytes, r->psum_storage, "psum", &g.psum_map, &psum_geo)) != WB200_OK) return st;
  }
  // The reference offers a GEMM to the tensor backend only without psum, with both operands in
  // Normal orientation and with one common format (TargetModelTensorNumeric.cpp:750-753,
  // OneDNNGemmAdapter.cpp:192-196); anything else is the formal path's.
  if (r->policy == WB200_GEMM_TENSOR && (r->has_psum || lt || rt || r->destination.format != r->lhs.format)) {
    *handled = 0;
    return WB200_OK;
  }
  DeviceGuard guard(backend->device);
  cudaStream_t stream = backend->stream;
  void *d_lhs, *d_rhs, *d_dst, *d_psum = nullptr;
  if ((st = backend->buffer(0, r->lhs_bytes, &d_lhs)) != WB200_OK) return st;
  if ((st = backend->buffer(1, r->rhs_bytes, &d_rhs)) != WB200_OK) return st;
  if ((st = backend->buffer(2, r->destination_bytes, &d_dst)) != WB200_OK) return st;
  if (r->has_psum && (st = backend->buffer(3, r->psum_bytes, &d_psum)) != WB200_OK) return st;
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_lhs, r->lhs_storage, r->lhs_bytes, cudaMemcpyHostToDevice, stream));
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_rhs, r->rhs_storage, r->rhs_bytes, cudaMemcpyHostToDevice, stream));
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_dst, r->destination_template, r->destination_bytes, cudaMemcpyHostToDevice, stream));
  if (r->has_psum) WB200_CUDA_CHECK(cudaMemcpyAsync(d_psum, r->psum_storage, r->psum_bytes, cudaMemcpyHostToDevice, stream));
  g.m = r->m; g.k = r->k; g.n = r->n; g.batch = r->batch_count;
  g.in_format = r->lhs.format; g.out_format = r->destination.format;
  g.lhs_transposed = lt; g.rhs_transposed = rt; g.has_psum = r->has_psum ? 1 : 0;
  g.lhs = static_cast<const uint8_t *>(d_lhs); g.rhs = static_cast<const uint8_t *>(d_rhs);
  g.psum = static_cast<const uint8_t *>(d_psum); g.dst = static_cast<uint8_t *>(d_dst);
  const uint64_t launches_before = backend->launches;
  const char *implementation = "";
  if ((st = run_device_gemm(backend, g, r->policy, 4, stream, &implementation)) != WB200_OK) return st;
  WB200_CUDA_CHECK(cudaMemcpyAsync(r->destination_out, d_dst, r->destination_bytes, cudaMemcpyDeviceToHost, stream));
  if ((st = read_device_status(backend, stream, nullptr)) != WB200_OK) return st;
  *handled = 1;
  fill_evidence(backend, evidence, implementation);
  if (evidence) {
    const uint64_t fmas = static_cast<uint64_t>(r->batch_count) * r->m * r->n * r->k;
    if (r->policy == WB200_GEMM_TENSOR) { evidence->matmul_invocations = 1; evidence->reorder_invocations = 0; evidence->formal_fused_multiply_adds = 0; }
    else { evidence->formal_fused_multiply_adds = fmas; }
    evidence->gpu_launches = static_cast<uint32_t>(backend->launches - launches_before);
  }
  return WB200_OK;
}

wb200_status wb200_elementwise(wb200_backend *backend, const wb200_elementwise_request *r, wb200_evidence *evidence) {
  if (!backend || !r) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  int arity;
  switch (r->operation) {
    case WB200_EW_MAX: case WB200_EW_MIN: case WB200_EW_ADD: case WB200_EW_SUB: case WB200_EW_MUL: arity = 2; break;
    case WB200_EW_ABS: case WB200_EW_RECIP: case WB200_EW_SQUARE: case WB200_EW_SQRT: case WB200_EW_RSQRT: case WB200_EW_NEG:
    case WB200_EW_LOG2: case WB200_EW_LN: case WB200_EW_POW2: case WB200_EW_EXP: case WB200_EW_EXPLP: case WB200_EW_SIN:
    case WB200_EW_COS: case WB200_EW_TANH: case WB200_EW_SIGMOID: case WB200_EW_RELU: case WB200_EW_SOFTPLUS: arity = 1; break;
    default: return fail(WB200_ERR_UNSUPPORTED, "elementwise operation is not in the managed domain");
  }
  if (static_cast<int>(r->input_count) != arity) return fail(WB200_ERR_INVALID_ARGUMENT, "elementwise input arity does not match semantics");
  const wb200_tensor_desc &dst = r->destination;
  if (!is_float_format(dst.format)) return fail(WB200_ERR_UNSUPPORTED, "elementwise result is not F16, BF16 or F32");
  LayoutMap map; wb200_geometry geo;
  wb200_status st = check_storage(dst, r->destination_bytes, r->destination_template, "destination template", &map, &geo);
  if (st != WB200_OK) return st;
  if (!r->destination_out) return fail(WB200_ERR_INVALID_ARGUMENT, "destination_out is null");
  uint64_t total_bytes = r->destination_bytes, logical = map.element_count;
  for (int i = 0; i < arity; ++i) {
    const wb200_tensor_desc &in = r->inputs[i];
    if (in.format != dst.format || in.layout != dst.layout || !same_shape(in, dst))
      return fail(WB200_ERR_INVALID_ARGUMENT, "elementwise tensors do not have one same-shape F16/BF16/F32 domain");
    if (!r->input_storage[i] || r->input_bytes[i] != r->destination_bytes)
      return fail(WB200_ERR_INVALID_ARGUMENT, "elementwise input storage size does not match its physical geometry");
    total_bytes += r->input_bytes[i];
    logical += map.element_count;
  }
  if ((st = check_budget(backend, map.element_count, r->max_scalar_evaluations, total_bytes, logical)) != WB200_OK) return st;
  DeviceGuard guard(backend->device);
  cudaStream_t stream = backend->stream;
  void *d_in[2] = {nullptr, nullptr}, *d_dst;
  for (int i = 0; i < arity; ++i) {
    if ((st = backend->buffer(i, r->input_bytes[i], &d_in[i])) != WB200_OK) return st;
    WB200_CUDA_CHECK(cudaMemcpyAsync(d_in[i], r->input_storage[i], r->input_bytes[i], cudaMemcpyHostToDevice, stream));
  }
  if ((st = backend->buffer(2, r->destination_bytes, &d_dst)) != WB200_OK) return st;
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_dst, r->destination_template, r->destination_bytes, cudaMemcpyHostToDevice, stream));
  if ((st = backend->timing_begin(stream)) != WB200_OK) return st;
  st = launch_elementwise(r->operation, dst.format, arity, static_cast<const uint8_t *>(d_in[0]), static_cast<const uint8_t *>(d_in[1]),
                          static_cast<uint8_t *>(d_dst), map, backend->d_status + 1, stream);
  if (st != WB200_OK) return st;
  backend->launches += 1;
  if ((st = backend->timing_end(stream)) != WB200_OK) return st;
  int nan_flag = 0;
  if ((st = read_device_status(backend, stream, &nan_flag)) != WB200_OK) return st;
  if (nan_flag) return fail(WB200_ERR_NAN_DOMAIN, "managed-reference tensor: value is outside the non-NaN domain");
  WB200_CUDA_CHECK(cudaMemcpyAsync(r->destination_out, d_dst, r->destination_bytes, cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  fill_evidence(backend, evidence, "sm100a-non-nan-f16-bf16-f32-tensor");
  if (evidence) evidence->device_us = backend->timing_microseconds();
  if (evidence) { evidence->scalar_evaluations = map.element_count; evidence->gpu_launches = 1; }
  return WB200_OK;
}

wb200_status wb200_elementwise_formal(wb200_backend *backend, const wb200_elementwise_request *r, wb200_evidence *evidence) {
  if (!backend || !r) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  int arity;
  bool relation = false, logic = false, function_family = false;
  switch (r->operation) {
    case WB200_EW_MAX: case WB200_EW_MIN: case WB200_EW_ADD: case WB200_EW_SUB: case WB200_EW_MUL: arity = 2; break;
    case WB200_EW_EQ: case WB200_EW_NE: case WB200_EW_GE: case WB200_EW_GT: case WB200_EW_LE: case WB200_EW_LT: arity = 2; relation = true; break;
    case WB200_EW_LOGIC_AND: case WB200_EW_LOGIC_OR: case WB200_EW_LOGIC_XOR: arity = 2; logic = true; break;
    case WB200_EW_LOGIC_NOT: arity = 1; logic = true; break;
    case WB200_EW_ABS: case WB200_EW_RECIP: case WB200_EW_SQUARE: case WB200_EW_NEG: case WB200_EW_RELU: arity = 1; break;
    case WB200_EW_SQRT: case WB200_EW_RSQRT: case WB200_EW_LOG2: case WB200_EW_LN: case WB200_EW_POW2: case WB200_EW_EXP:
    case WB200_EW_SIN: case WB200_EW_COS: case WB200_EW_TANH: case WB200_EW_SIGMOID: case WB200_EW_SOFTPLUS:
      arity = 1;
      function_family = true;
      break;
    default: return fail(WB200_ERR_UNSUPPORTED, "elementwise operation is outside the formal arithmetic, relation, logic and function families");
  }
  if (static_cast<int>(r->input_count) != arity) return fail(WB200_ERR_INVALID_ARGUMENT, "elementwise input arity does not match semantics");
  const wb200_tensor_desc &dst = r->destination, &first = r->inputs[0];
  const bool bool_out = dst.format == WB200_BOOL, bool_in = first.format == WB200_BOOL;
  // TF32 (19 significant bits in storage bits 31..13) is an operand format of the correctly rounded function family only.
  const bool tf32_function = function_family && first.format == WB200_TF32;
  if (logic ? !(bool_out && (bool_in || is_float_format(first.format))) : !(is_float_format(first.format) || tf32_function))
    return fail(WB200_ERR_UNSUPPORTED, "formal elementwise operands must be F16, BF16 or F32 (Bool for logic, TF32 for the function family)");
  if (!logic && !(relation ? (bool_out || is_float_format(dst.format)) : dst.format == first.format))
    return fail(WB200_ERR_UNSUPPORTED, "formal elementwise result format does not fit the operation");
  auto packed_ok = [](const wb200_tensor_desc &d) { return d.format != WB200_BOOL || d.layout == WB200_LAYOUT_TENSOR || d.layout == WB200_LAYOUT_NTENSOR; };
  if (!packed_ok(dst) || !packed_ok(first)) return fail(WB200_ERR_UNSUPPORTED, "bit-packed Bool tensors are taken in Tensor / NTensor layout only");
  LayoutMap out_map, in_map; wb200_geometry out_geo, in_geo;
  wb200_status st = check_storage(dst, r->destination_bytes, r->destination_template, "destination template", &out_map, &out_geo);
  if (st != WB200_OK) return st;
  if (!r->destination_out) return fail(WB200_ERR_INVALID_ARGUMENT, "destination_out is null");
  uint64_t total_bytes = r->destination_bytes, logical = out_map.element_count;
  for (int i = 0; i < arity; ++i) {
    const wb200_tensor_desc &in = r->inputs[i];
    if (in.format != first.format || in.layout != first.layout || !same_shape(in, dst))
      return fail(WB200_ERR_INVALID_ARGUMENT, "elementwise tensors do not have one same-shape domain");
    if ((st = check_storage(in, r->input_bytes[i], r->input_storage[i], "input", &in_map, &in_geo)) != WB200_OK) return st;
    total_bytes += r->input_bytes[i];
    logical += in_map.element_count;
  }
  if ((st = check_budget(backend, out_map.element_count, r->max_scalar_evaluations, total_bytes, logical)) != WB200_OK) return st;
  DeviceGuard guard(backend->device);
  cudaStream_t stream = backend->stream;
  void *d_in[2] = {nullptr, nullptr}, *d_dst, *d_flags;
  for (int i = 0; i < arity; ++i) {
    if ((st = backend->buffer(i, r->input_bytes[i], &d_in[i])) != WB200_OK) return st;
    WB200_CUDA_CHECK(cudaMemcpyAsync(d_in[i], r->input_storage[i], r->input_bytes[i], cudaMemcpyHostToDevice, stream));
  }
  if ((st = backend->buffer(2, r->destination_bytes, &d_dst)) != WB200_OK) return st;
  if ((st = backend->buffer(3, sizeof(uint32_t), &d_flags)) != WB200_OK) return st;
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_dst, r->destination_template, r->destination_bytes, cudaMemcpyHostToDevice, stream));
  WB200_CUDA_CHECK(cudaMemsetAsync(d_flags, 0, sizeof(uint32_t), stream));
  if ((st = backend->timing_begin(stream)) != WB200_OK) return st;
  st = launch_elementwise_formal(r->operation, first.format, dst.format, arity, static_cast<const uint8_t *>(d_in[0]),
                                 static_cast<const uint8_t *>(d_in[1]), static_cast<uint8_t *>(d_dst), in_map, out_map,
                                 static_cast<uint32_t *>(d_flags), stream);
  if (st != WB200_OK) return st;
  backend->launches += 1;
  if ((st = backend->timing_end(stream)) != WB200_OK) return st;
  uint32_t flags = 0;
  WB200_CUDA_CHECK(cudaMemcpyAsync(&flags, d_flags, sizeof(flags), cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaMemcpyAsync(r->destination_out, d_dst, r->destination_bytes, cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  fill_evidence(backend, evidence, "sm100a-formal-elementwise");
  if (evidence) evidence->device_us = backend->timing_microseconds();
  if (evidence) { evidence->scalar_evaluations = out_map.element_count; evidence->gpu_launches = 1; evidence->flags = flags; }
  return WB200_OK;
}

wb200_status wb200_convert(wb200_backend *backend, const wb200_convert_request *r, wb200_evidence *evidence) {
  if (!backend || !r) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  if (r->opcode < 139 || r->opcode > 174) return fail(WB200_ERR_INVALID_ARGUMENT, "convert opcode is not a target route");
  if (r->rounding_mode != 0) return fail(WB200_ERR_UNSUPPORTED, "convert is not nearest-even");
  const wb200_tensor_desc &src = r->source, &dst = r->destination;
  if (!is_float_format(src.format) || !is_float_format(dst.format) || src.layout != dst.layout || !same_shape(src, dst))
    return fail(WB200_ERR_UNSUPPORTED, "convert is outside the F16/BF16/F32 same-shape domain");
  // Route table rows for float <-> float (lib/Wafer/Target/TargetFormat.cpp:163-200).
  static const struct { uint32_t opcode; int from, to; } kRoutes[] = {
      {154, WB200_BF16, WB200_F16}, {155, WB200_BF16, WB200_F32}, {160, WB200_F16, WB200_BF16},
      {161, WB200_F16, WB200_F32},  {166, WB200_F32, WB200_F16},  {167, WB200_F32, WB200_BF16}};
  bool route_ok = false;
  for (const auto &route : kRoutes) route_ok |= route.opcode == r->opcode && route.from == src.format && route.to == dst.format;
  if (!route_ok) return fail(WB200_ERR_INVALID_ARGUMENT, "convert opcode does not match the tensor formats");
  LayoutMap src_map, dst_map; wb200_geometry src_geo, dst_geo;
  wb200_status st;
  if ((st = check_storage(src, r->source_bytes, r->source_storage, "source", &src_map, &src_geo)) != WB200_OK) return st;
  if ((st = check_storage(dst, r->destination_bytes, r->destination_template, "destination template", &dst_map, &dst_geo)) != WB200_OK) return st;
  if (!r->destination_out) return fail(WB200_ERR_INVALID_ARGUMENT, "destination_out is null");
  if ((st = check_budget(backend, dst_map.element_count, r->max_scalar_evaluations, r->source_bytes + r->destination_bytes,
                         2 * static_cast<uint64_t>(dst_map.element_count))) != WB200_OK) return st;
  DeviceGuard guard(backend->device);
  cudaStream_t stream = backend->stream;
  void *d_src, *d_dst;
  if ((st = backend->buffer(0, r->source_bytes, &d_src)) != WB200_OK) return st;
  if ((st = backend->buffer(2, r->destination_bytes, &d_dst)) != WB200_OK) return st;
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_src, r->source_storage, r->source_bytes, cudaMemcpyHostToDevice, stream));
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_dst, r->destination_template, r->destination_bytes, cudaMemcpyHostToDevice, stream));
  if ((st = backend->timing_begin(stream)) != WB200_OK) return st;
  st = launch_convert(src.format, dst.format, static_cast<const uint8_t *>(d_src), static_cast<uint8_t *>(d_dst), src_map, dst_map,
                      backend->d_status + 1, stream);
  if (st != WB200_OK) return st;
  backend->launches += 1;
  if ((st = backend->timing_end(stream)) != WB200_OK) return st;
  int nan_flag = 0;
  if ((st = read_device_status(backend, stream, &nan_flag)) != WB200_OK) return st;
  if (nan_flag) return fail(WB200_ERR_NAN_DOMAIN, "managed-reference tensor: input value is outside the non-NaN domain");
  WB200_CUDA_CHECK(cudaMemcpyAsync(r->destination_out, d_dst, r->destination_bytes, cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  fill_evidence(backend, evidence, "sm100a-non-nan-f16-bf16-f32-tensor");
  if (evidence) evidence->device_us = backend->timing_microseconds();
  if (evidence) { evidence->scalar_evaluations = dst_map.element_count; evidence->gpu_launches = 1; }
  return WB200_OK;
}

// Domain, reduced dimensions (getTargetReduceLogicalDimensions, lib/Wafer/Target/TargetOperation.cpp:93-139) and the
// destination shape of a reduce command. Bit d of *mask = logical dimension d is reduced.
static wb200_status plan_reduce(const wb200_tensor_desc &in, const wb200_tensor_desc &dst, uint32_t operation, uint32_t dimension, uint32_t *mask_out) {
  if ((operation != WB200_RED_SUM && operation != WB200_RED_MAX && operation != WB200_RED_MIN) ||
      !is_float_format(in.format) || dst.format != in.format || (operation == WB200_RED_SUM && in.format != WB200_F32))
    return fail(WB200_ERR_UNSUPPORTED, "reduce requires F32 sum or F16/BF16/F32 max/min");
  const int rank = in.rank;
  uint32_t mask = 0;
  auto trailing = [&](int index) { if (index < rank) mask |= 1u << (rank - 1 - index); return index < rank; };
  bool ok = true;
  switch (dimension) {
    case WB200_RED_TRAILING0: ok = trailing(0); break;
    case WB200_RED_TRAILING1: ok = trailing(1); break;
    case WB200_RED_TRAILING2: ok = trailing(2); break;
    case WB200_RED_TRAILING3: ok = trailing(3); break;
    case WB200_RED_TRAILING2AND1: ok = rank > 2; if (ok) { trailing(2); trailing(1); } break;
    case WB200_RED_TRAILING2AND1AND0: ok = rank > 2; if (ok) { trailing(2); trailing(1); trailing(0); } break;
    default: return fail(WB200_ERR_INVALID_ARGUMENT, "unknown reduce dimension");
  }
  if (!ok || mask == 0) return fail(WB200_ERR_INVALID_ARGUMENT, "reduce has no logical dimensions");
  if (dst.rank != in.rank) return fail(WB200_ERR_INVALID_ARGUMENT, "reduce destination rank differs from the input rank");
  for (int d = 0; d < rank; ++d) {
    const uint64_t expected = (mask & (1u << d)) ? 1 : in.shape[d];
    if (dst.shape[d] != expected) return fail(WB200_ERR_INVALID_ARGUMENT, "reduce destination shape does not match the reduced input shape");
  }
  *mask_out = mask;
  return WB200_OK;
}

wb200_status wb200_reduce(wb200_backend *backend, const wb200_reduce_request *r, wb200_evidence *evidence) {
  if (!backend || !r) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  const wb200_tensor_desc &in = r->input, &dst = r->destination;
  uint32_t mask = 0;
  wb200_status st = plan_reduce(in, dst, r->operation, r->dimension, &mask);
  if (st != WB200_OK) return st;
  LayoutMap in_map, dst_map; wb200_geometry in_geo, dst_geo;
  if ((st = check_storage(in, r->input_bytes, r->input_storage, "input", &in_map, &in_geo)) != WB200_OK) return st;
  if ((st = check_storage(dst, r->destination_bytes, r->destination_template, "destination template", &dst_map, &dst_geo)) != WB200_OK) return st;
  if (!r->destination_out) return fail(WB200_ERR_INVALID_ARGUMENT, "destination_out is null");
  if ((st = check_budget(backend, in_map.element_count, r->max_scalar_evaluations, r->input_bytes + r->destination_bytes,
                         static_cast<uint64_t>(in_map.element_count) + dst_map.element_count)) != WB200_OK) return st;
  DeviceGuard guard(backend->device);
  cudaStream_t stream = backend->stream;
  void *d_src, *d_dst;
  if ((st = backend->buffer(0, r->input_bytes, &d_src)) != WB200_OK) return st;
  if ((st = backend->buffer(2, r->destination_bytes, &d_dst)) != WB200_OK) return st;
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_src, r->input_storage, r->input_bytes, cudaMemcpyHostToDevice, stream));
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_dst, r->destination_template, r->destination_bytes, cudaMemcpyHostToDevice, stream));
  if ((st = backend->timing_begin(stream)) != WB200_OK) return st;
  st = launch_reduce(r->operation, in.format, static_cast<const uint8_t *>(d_src), static_cast<uint8_t *>(d_dst), in_map, dst_map, mask,
                     backend->d_status + 1, stream);
  if (st != WB200_OK) return st;
  backend->launches += 1;
  if ((st = backend->timing_end(stream)) != WB200_OK) return st;
  int nan_flag = 0;
  if ((st = read_device_status(backend, stream, &nan_flag)) != WB200_OK) return st;
  if (nan_flag) return fail(WB200_ERR_NAN_DOMAIN, "managed-reference tensor: reduce left the non-NaN domain");
  WB200_CUDA_CHECK(cudaMemcpyAsync(r->destination_out, d_dst, r->destination_bytes, cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  fill_evidence(backend, evidence, "sm100a-non-nan-f16-bf16-f32-tensor");
  if (evidence) evidence->device_us = backend->timing_microseconds();
  if (evidence) { evidence->scalar_evaluations = in_map.element_count; evidence->gpu_launches = 1; }
  return WB200_OK;
}

wb200_status wb200_reduce_formal(wb200_backend *backend, const wb200_reduce_request *r, wb200_evidence *evidence) {
  if (!backend || !r) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  const wb200_tensor_desc &in = r->input, &dst = r->destination;
  uint32_t mask = 0;
  wb200_status st = plan_reduce(in, dst, r->operation, r->dimension, &mask);
  if (st != WB200_OK) return st;
  LayoutMap in_map, dst_map; wb200_geometry in_geo, dst_geo;
  if ((st = check_storage(in, r->input_bytes, r->input_storage, "input", &in_map, &in_geo)) != WB200_OK) return st;
  if ((st = check_storage(dst, r->destination_bytes, r->destination_template, "destination template", &dst_map, &dst_geo)) != WB200_OK) return st;
  if (!r->destination_out) return fail(WB200_ERR_INVALID_ARGUMENT, "destination_out is null");
  if ((st = check_budget(backend, in_map.element_count, r->max_scalar_evaluations, r->input_bytes + r->destination_bytes,
                         static_cast<uint64_t>(in_map.element_count) + dst_map.element_count)) != WB200_OK) return st;
  DeviceGuard guard(backend->device);
  cudaStream_t stream = backend->stream;
  void *d_src, *d_dst, *d_flags;
  if ((st = backend->buffer(0, r->input_bytes, &d_src)) != WB200_OK) return st;
  if ((st = backend->buffer(2, r->destination_bytes, &d_dst)) != WB200_OK) return st;
  if ((st = backend->buffer(3, sizeof(uint32_t), &d_flags)) != WB200_OK) return st;
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_src, r->input_storage, r->input_bytes, cudaMemcpyHostToDevice, stream));
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_dst, r->destination_template, r->destination_bytes, cudaMemcpyHostToDevice, stream));
  WB200_CUDA_CHECK(cudaMemsetAsync(d_flags, 0, sizeof(uint32_t), stream));
  if ((st = backend->timing_begin(stream)) != WB200_OK) return st;
  if ((st = launch_reduce_formal(r->operation, in.format, static_cast<const uint8_t *>(d_src), static_cast<uint8_t *>(d_dst), in_map, dst_map, mask,
                                 static_cast<uint32_t *>(d_flags), stream)) != WB200_OK) return st;
  backend->launches += 1;
  if ((st = backend->timing_end(stream)) != WB200_OK) return st;
  uint32_t flags = 0;
  WB200_CUDA_CHECK(cudaMemcpyAsync(&flags, d_flags, sizeof(flags), cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaMemcpyAsync(r->destination_out, d_dst, r->destination_bytes, cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  fill_evidence(backend, evidence, "sm100a-formal-reduce");
  if (evidence) evidence->device_us = backend->timing_microseconds();
  if (evidence) { evidence->scalar_evaluations = in_map.element_count; evidence->gpu_launches = 1; evidence->flags = flags; }
  return WB200_OK;
}

}  // extern "C"

// ------------------------------------------------------------------ TargetCall ABI (Seam 2)
extern "C" {

wb200_status wb200_spm_create(wb200_backend *backend, uint64_t base_address, uint64_t bytes, wb200_spm_image **out) {
  if (!backend || !out || bytes == 0) return fail(WB200_ERR_INVALID_ARGUMENT, "invalid scratch-pad image request");
  DeviceGuard guard(backend->device);
  wb200_spm_image *image = new wb200_spm_image{backend, base_address, bytes, nullptr};
  cudaError_t err = cudaMalloc(&image->device, bytes);
  if (err == cudaSuccess) err = cudaMemset(image->device, 0, bytes);
  if (err != cudaSuccess) { delete image; return fail(WB200_ERR_CUDA, std::string("scratch-pad image: ") + cudaGetErrorString(err)); }
  *out = image;
  return WB200_OK;
}

void wb200_spm_destroy(wb200_spm_image *image) {
  if (!image) return;
  DeviceGuard guard(image->backend->device);
  cudaStreamSynchronize(image->backend->stream);
  cudaFree(image->device);
  delete image;
}

static wb200_status spm_range(const wb200_spm_image *image, uint64_t address, uint64_t bytes, const char *what) {
  return wb200::image_range(image, address, bytes, what);
}

wb200_status wb200_spm_write(wb200_spm_image *image, uint64_t address, const uint8_t *src, uint64_t bytes) {
  if (!image || !src) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  wb200_status st = spm_range(image, address, bytes, "write");
  if (st != WB200_OK) return st;
  DeviceGuard guard(image->backend->device);
  WB200_CUDA_CHECK(cudaMemcpyAsync(image->device + (address - image->base), src, bytes, cudaMemcpyHostToDevice, image->backend->stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(image->backend->stream));
  return WB200_OK;
}

wb200_status wb200_spm_read(wb200_spm_image *image, uint64_t address, uint8_t *dst, uint64_t bytes) {
  if (!image || !dst) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  wb200_status st = spm_range(image, address, bytes, "read");
  if (st != WB200_OK) return st;
  DeviceGuard guard(image->backend->device);
  WB200_CUDA_CHECK(cudaMemcpyAsync(dst, image->device + (address - image->base), bytes, cudaMemcpyDeviceToHost, image->backend->stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(image->backend->stream));
  return WB200_OK;
}

}  // extern "C"

namespace wb200 {

wb200_status image_range(const wb200_spm_image *image, uint64_t address, uint64_t bytes, const char *what) {
  if (address < image->base || bytes > image->bytes || address - image->base > image->bytes - bytes)
    return fail(WB200_ERR_INVALID_ARGUMENT, std::string(what) + " lies outside the memory image");
  return WB200_OK;
}

wb200_status enqueue_image_gemm(wb200_spm_image *image, uint64_t lhs, uint64_t rhs, uint64_t dst, uint64_t psum,
                                uint32_t m, uint32_t k, uint32_t n, uint32_t batch, uint32_t in_format,
                                uint32_t out_format, uint32_t psum_format, uint32_t lhs_orientation,
                                uint32_t rhs_orientation, uint32_t policy, RunCommand *defer, bool *deferred) {
  if (deferred) *deferred = false;
  if (!image) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  if (m == 0 || k == 0 || n == 0 || batch == 0 || m > 65535 || n > 65535 || k > 16384 || batch > 4096)
    return fail(WB200_ERR_INVALID_ARGUMENT, "GEMM extents outside the command domain");
  if (!is_float_format(in_format) || (out_format != in_format && out_format != WB200_F32))
    return fail(WB200_ERR_UNSUPPORTED, "GEMM formats outside the NE engine's f16/bf16/f32 domain");
  const bool has_psum = psum_format != WB200_FORMAT_NONE;
  if (has_psum && psum_format != WB200_F32) return fail(WB200_ERR_UNSUPPORTED, "psum must be f32");
  const bool lt = lhs_orientation == WB200_TRANSPOSE, rt = rhs_orientation == WB200_TRANSPOSE;
  // Implicit storage contract of the command: Cx for one matrix, NCx for a batch
  // (lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:667-699).
  auto describe = [&](uint32_t format, uint64_t rows, uint64_t cols) {
    wb200_tensor_desc d{};
    d.format = static_cast<uint8_t>(format);
    if (batch == 1) { d.layout = WB200_LAYOUT_CX; d.rank = 2; d.shape[0] = rows; d.shape[1] = cols; }
    else { d.layout = WB200_LAYOUT_NCX; d.rank = 3; d.shape[0] = batch; d.shape[1] = rows; d.shape[2] = cols; }
    return d;
  };
  const wb200_tensor_desc lhs_desc = describe(in_format, lt ? k : m, lt ? m : k);
  const wb200_tensor_desc rhs_desc = describe(in_format, rt ? n : k, rt ? k : n);
  const wb200_tensor_desc dst_desc = describe(out_format, m, n);
  const wb200_tensor_desc psum_desc = describe(WB200_F32, m, n);
  DeviceGemm g{};
  wb200_geometry lhs_geo, rhs_geo, dst_geo, psum_geo{};
  wb200_status st;
  if ((st = make_layout_map(lhs_desc, &g.lhs_map, &lhs_geo)) != WB200_OK) return st;
  if ((st = make_layout_map(rhs_desc, &g.rhs_map, &rhs_geo)) != WB200_OK) return st;
  if ((st = make_layout_map(dst_desc, &g.dst_map, &dst_geo)) != WB200_OK) return st;
  if ((st = spm_range(image, lhs, lhs_geo.physical_bytes, "lhs")) != WB200_OK) return st;
  if ((st = spm_range(image, rhs, rhs_geo.physical_bytes, "rhs")) != WB200_OK) return st;
  if ((st = spm_range(image, dst, dst_geo.physical_bytes, "destination")) != WB200_OK) return st;
  if (has_psum) {
    if ((st = make_layout_map(psum_desc, &g.psum_map, &psum_geo)) != WB200_OK) return st;
    if ((st = spm_range(image, psum, psum_geo.physical_bytes, "psum")) != WB200_OK) return st;
    const uint64_t dst_end = dst + dst_geo.physical_bytes, psum_end = psum + psum_geo.physical_bytes;
    if (dst < psum_end && psum < dst_end)
      return fail(WB200_ERR_INVALID_ARGUMENT, "psum and destination must occupy disjoint physical storage");
  }
  wb200_backend *backend = image->backend;
  DeviceGuard guard(backend->device);
  g.m = m; g.k = k; g.n = n; g.batch = batch;
  g.in_format = in_format; g.out_format = out_format;
  g.lhs_transposed = lt; g.rhs_transposed = rt; g.has_psum = has_psum;
  g.lhs = image->device + (lhs - image->base);
  g.rhs = image->device + (rhs - image->base);
  g.psum = has_psum ? image->device + (psum - image->base) : nullptr;
  g.dst = image->device + (dst - image->base);
  const char *implementation = "";
  const int effective_policy = (policy == WB200_GEMM_TENSOR && !has_psum && !lt && !rt) ? WB200_GEMM_TENSOR : WB200_GEMM_FORMAL;
  if (defer && deferred && effective_policy == WB200_GEMM_FORMAL) {
    RunCommand command;
    command.kind = WB200_RUN_GEMM;
    GemmFormalArgs &f = command.u.gemm;
    f = GemmFormalArgs{};
    f.m = g.m; f.k = g.k; f.n = g.n; f.batch = g.batch;
    f.in_format = g.in_format; f.out_format = g.out_format;
    f.lhs_transposed = g.lhs_transposed; f.rhs_transposed = g.rhs_transposed;
    f.has_psum = g.has_psum;
    f.lhs = g.lhs; f.rhs = g.rhs; f.psum = g.psum; f.dst = g.dst;
    f.lhs_map = g.lhs_map; f.rhs_map = g.rhs_map; f.psum_map = g.psum_map; f.dst_map = g.dst_map;
    command.variant = formal_gemm_variant(f);
    *defer = command;
    *deferred = formal_run_admits(command);
    return WB200_OK;
  }
  if (defer && deferred) return WB200_OK;   // tensor-core policy: not part of a run, *deferred stays false
  return run_device_gemm(backend, g, effective_policy, 4, image->work_stream(), &implementation, image->gemm_staging,
                         static_cast<size_t>(image->bytes));
}


// wafer_tx81_elementwise_<op> on a scratch-pad image: 1-D Tensor operands of `count` elements, the result format
// chosen by the operation class, the second operand in one of its four forms
// (lib/Wafer/Target/TargetCallDecoder.cpp:231-268, lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:288-400).
wb200_status enqueue_image_elementwise(wb200_spm_image *image, uint32_t operation, uint64_t lhs, uint64_t rhs_or_scalar_bits,
                                       uint64_t dst, uint32_t count, uint32_t format, uint32_t rhs_unit_elements,
                                       uint32_t scalar_flag, uint32_t relation_numeric_or_rhs_group, uint32_t *d_flags, bool execute,
                                       RunCommand *defer, bool *deferred) {
  if (deferred) *deferred = false;
  if (!image) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  int arity;
  bool relation = false, logic = false, function_family = false;
  switch (operation) {
    case WB200_EW_MAX: case WB200_EW_MIN: case WB200_EW_ADD: case WB200_EW_SUB: case WB200_EW_MUL: arity = 2; break;
    case WB200_EW_EQ: case WB200_EW_NE: case WB200_EW_GE: case WB200_EW_GT: case WB200_EW_LE: case WB200_EW_LT: arity = 2; relation = true; break;
    case WB200_EW_LOGIC_AND: case WB200_EW_LOGIC_OR: case WB200_EW_LOGIC_XOR: arity = 2; logic = true; break;
    case WB200_EW_LOGIC_NOT: arity = 1; logic = true; break;
    case WB200_EW_ABS: case WB200_EW_RECIP: case WB200_EW_SQUARE: case WB200_EW_NEG: case WB200_EW_RELU: arity = 1; break;
    case WB200_EW_SQRT: case WB200_EW_RSQRT: case WB200_EW_LOG2: case WB200_EW_LN: case WB200_EW_POW2: case WB200_EW_EXP:
    case WB200_EW_SIN: case WB200_EW_COS: case WB200_EW_TANH: case WB200_EW_SIGMOID: case WB200_EW_SOFTPLUS:
      arity = 1;
      function_family = true;
      break;
    default: return fail(WB200_ERR_UNSUPPORTED, "elementwise operation has no formal evaluation");
  }
  if (count == 0) return fail(WB200_ERR_INVALID_ARGUMENT, "elementwise element count must be positive");
  if (logic ? !(format == WB200_BOOL || is_float_format(format)) : !(is_float_format(format) || (function_family && format == WB200_TF32)))
    return fail(WB200_ERR_UNSUPPORTED, "elementwise operand format must be F16, BF16 or F32 (Bool for logic, TF32 for the function family)");
  const bool extras = arity == 2 && !logic;   // only arithmetic and relation calls carry the three extra fields
  if (!extras) rhs_unit_elements = scalar_flag = relation_numeric_or_rhs_group = 0;
  if (scalar_flag > 1) return fail(WB200_ERR_INVALID_ARGUMENT, "elementwise scalar flag must be 0 or 1");
  if (scalar_flag && rhs_or_scalar_bits > 0xffffffffull) return fail(WB200_ERR_INVALID_ARGUMENT, "elementwise scalar bits must fit uint32");
  if (relation && relation_numeric_or_rhs_group > 1) return fail(WB200_ERR_INVALID_ARGUMENT, "relation numeric_result must be 0 or 1");
  const uint32_t rhs_group = relation ? 0u : relation_numeric_or_rhs_group;
  const int out_format = logic ? WB200_BOOL : relation ? (relation_numeric_or_rhs_group ? static_cast<int>(format) : WB200_BOOL) : static_cast<int>(format);
  RhsBroadcast rhs;
  uint64_t rhs_elements = count;
  if (scalar_flag) {
    rhs.mode = WB200_RHS_SCALAR;
    rhs.parameter = static_cast<uint32_t>(rhs_or_scalar_bits);
    rhs_elements = 0;
  } else if (rhs_group) {
    if (rhs_group < 64 || rhs_group % 64 != 0 || count % rhs_group != 0)
      return fail(WB200_ERR_INVALID_ARGUMENT, "grouped second operand needs whole groups that are multiples of 64 elements");
    rhs.mode = WB200_RHS_GROUP;
    rhs.parameter = rhs_group;
  } else if (rhs_unit_elements) {
    rhs.mode = WB200_RHS_UNIT;
    rhs.parameter = rhs_unit_elements;
    rhs_elements = rhs_unit_elements;
  }
  auto vector = [](uint32_t fmt, uint64_t elements) {
    wb200_tensor_desc d{};
    d.format = static_cast<uint8_t>(fmt);
    d.layout = WB200_LAYOUT_TENSOR;
    d.rank = 1;
    d.shape[0] = elements;
    return d;
  };
  LayoutMap in_map, out_map, rhs_map;
  wb200_geometry in_geo, out_geo, rhs_geo{};
  wb200_status st;
  if ((st = make_layout_map(vector(format, count), &in_map, &in_geo)) != WB200_OK) return st;
  if ((st = make_layout_map(vector(out_format, count), &out_map, &out_geo)) != WB200_OK) return st;
  if ((st = spm_range(image, lhs, in_geo.physical_bytes, "lhs")) != WB200_OK) return st;
  if ((st = spm_range(image, dst, out_geo.physical_bytes, "destination")) != WB200_OK) return st;
  if (arity == 2 && rhs_elements) {
    if ((st = make_layout_map(vector(format, rhs_elements), &rhs_map, &rhs_geo)) != WB200_OK) return st;
    if ((st = spm_range(image, rhs_or_scalar_bits, rhs_geo.physical_bytes, "rhs")) != WB200_OK) return st;
  }
  if (!execute) return WB200_OK;   // validation only (device-free trace)
  wb200_backend *backend = image->backend;
  DeviceGuard guard(backend->device);
  const uint8_t *d_lhs = image->device + (lhs - image->base);
  const uint8_t *d_rhs = (arity == 2 && rhs_elements) ? image->device + (rhs_or_scalar_bits - image->base) : nullptr;
  if (defer && deferred) {
    RunCommand command;
    command.kind = WB200_RUN_ELEMENTWISE;
    RunElementwise &e = command.u.elementwise;
    e.op = static_cast<int32_t>(operation); e.in_format = static_cast<int32_t>(format); e.out_format = out_format; e.input_count = arity;
    e.in0 = d_lhs; e.in1 = d_rhs; e.dst = image->device + (dst - image->base);
    e.in_map = in_map; e.out_map = out_map; e.rhs = rhs;
    *defer = command;
    *deferred = formal_run_admits(command);
    return WB200_OK;
  }
  st = launch_elementwise_formal(operation, format, out_format, arity, d_lhs, d_rhs, image->device + (dst - image->base), in_map,
                                 out_map, d_flags, image->work_stream(), rhs);
  if (st == WB200_OK) backend->launches += 1;
  return st;
}

// wafer_tx81_reduce_{sum,max,min} on a scratch-pad image: NCx [n, h, w, c] input, NCx destination with the reduced
// dimensions set to 1 (lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:586-660), executed by the formal fold.
wb200_status enqueue_image_reduce(wb200_spm_image *image, uint32_t operation, uint64_t source, uint64_t destination, uint32_t dimension,
                                  const uint32_t nhwc[4], uint32_t format, uint32_t *d_flags, bool execute, RunCommand *defer, bool *deferred) {
  if (deferred) *deferred = false;
  if (!image || !nhwc) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  wb200_tensor_desc in{}, dst{};
  in.format = dst.format = static_cast<uint8_t>(format);
  in.layout = dst.layout = WB200_LAYOUT_NCX;
  in.rank = dst.rank = 4;
  for (int i = 0; i < 4; ++i) in.shape[i] = dst.shape[i] = nhwc[i];
  // the destination keeps every dimension the command does not reduce
  uint32_t mask = 0;
  {
    const int trailing[6][3] = {{0, -1, -1}, {1, -1, -1}, {2, -1, -1}, {3, -1, -1}, {2, 1, -1}, {2, 1, 0}};
    if (dimension > 5) return fail(WB200_ERR_INVALID_ARGUMENT, "reduce dimension is invalid for the fixed ABI shape");
    for (int i = 0; i < 3; ++i)
      if (trailing[dimension][i] >= 0) dst.shape[3 - trailing[dimension][i]] = 1;
  }
  wb200_status st = plan_reduce(in, dst, operation, dimension, &mask);
  if (st != WB200_OK) return st;
  LayoutMap in_map, dst_map;
  wb200_geometry in_geo, dst_geo;
  if ((st = make_layout_map(in, &in_map, &in_geo)) != WB200_OK) return st;
  if ((st = make_layout_map(dst, &dst_map, &dst_geo)) != WB200_OK) return st;
  if ((st = spm_range(image, source, in_geo.physical_bytes, "reduce source")) != WB200_OK) return st;
  if ((st = spm_range(image, destination, dst_geo.physical_bytes, "reduce destination")) != WB200_OK) return st;
  if (!execute) return WB200_OK;
  if (defer && deferred) {
    RunCommand command;
    command.kind = WB200_RUN_REDUCE;
    RunReduce &r = command.u.reduce;
    r.op = static_cast<int32_t>(operation); r.format = static_cast<int32_t>(format);
    r.src = image->device + (source - image->base); r.dst = image->device + (destination - image->base);
    r.src_map = in_map; r.dst_map = dst_map; r.reduced_mask = mask;
    *defer = command;
    *deferred = formal_run_admits(command);
    return WB200_OK;
  }
  DeviceGuard guard(image->backend->device);
  st = launch_reduce_formal(operation, format, image->device + (source - image->base), image->device + (destination - image->base), in_map,
                            dst_map, mask, d_flags, image->work_stream());
  if (st == WB200_OK) image->backend->launches += 1;
  return st;
}

// wafer_tx81_pool_{max,min,sum} on a scratch-pad image (NCx [n, h, w, c] in and out, no padding, no index output).
wb200_status enqueue_image_pool(wb200_spm_image *image, uint32_t kind, uint64_t input, uint64_t dst, const uint32_t source_shape[4],
                                const uint32_t destination_shape[4], const uint32_t pads[4], const uint32_t kernel_strides[4],
                                uint32_t format, uint32_t *d_flags, bool execute) {
  if (!image || !source_shape || !destination_shape || !pads || !kernel_strides) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  int combine;
  switch (kind) {
    case 117: combine = WB200_EW_MAX; break;
    case 119: combine = WB200_EW_MIN; break;
    case 116:
      if (format != WB200_F32) return fail(WB200_ERR_UNSUPPORTED, "plain sum pooling currently qualifies F32 accumulation only");
      combine = WB200_EW_ADD;
      break;
    default: return fail(WB200_ERR_UNSUPPORTED, "pooling kind has no qualified plain numeric implementation");
  }
  if (!is_float_format(format)) return fail(WB200_ERR_UNSUPPORTED, "pooling operands must be F16, BF16 or F32");
  for (int i = 0; i < 4; ++i)
    if (pads[i] != 0) return fail(WB200_ERR_UNSUPPORTED, "plain pooling requires explicit input padding and no index output");
  if (source_shape[0] != destination_shape[0] || source_shape[3] != destination_shape[3])
    return fail(WB200_ERR_INVALID_ARGUMENT, "pooling must preserve batch and channel extents");
  for (int axis = 0; axis < 2; ++axis) {
    const uint64_t source = source_shape[axis + 1], kernel = kernel_strides[1 - axis], stride = kernel_strides[3 - axis];
    if (kernel == 0 || stride == 0 || source < kernel || (source - kernel) / stride + 1 != destination_shape[axis + 1])
      return fail(WB200_ERR_INVALID_ARGUMENT, "pooling result disagrees with its window geometry");
  }
  auto describe = [&](const uint32_t shape[4]) {
    wb200_tensor_desc d{};
    d.format = static_cast<uint8_t>(format);
    d.layout = WB200_LAYOUT_NCX;
    d.rank = 4;
    for (int i = 0; i < 4; ++i) d.shape[i] = shape[i];
    return d;
  };
  LayoutMap src_map, dst_map;
  wb200_geometry src_geo, dst_geo;
  wb200_status st;
  if ((st = make_layout_map(describe(source_shape), &src_map, &src_geo)) != WB200_OK) return st;
  if ((st = make_layout_map(describe(destination_shape), &dst_map, &dst_geo)) != WB200_OK) return st;
  if ((st = spm_range(image, input, src_geo.physical_bytes, "pooling input")) != WB200_OK) return st;
  if ((st = spm_range(image, dst, dst_geo.physical_bytes, "pooling destination")) != WB200_OK) return st;
  if (!execute) return WB200_OK;   // validation only (device-free trace)
  wb200_backend *backend = image->backend;
  DeviceGuard guard(backend->device);
  const PoolWindow window{kernel_strides[0], kernel_strides[1], kernel_strides[2], kernel_strides[3]};
  st = launch_pool_formal(combine, format, image->device + (input - image->base), image->device + (dst - image->base), src_map,
                          dst_map, window, d_flags, image->work_stream());
  if (st == WB200_OK) backend->launches += 1;
  return st;
}

}  // namespace wb200

namespace {
// Runs `enqueue(d_flags)` with a zeroed device flag word and reads the OR of the IEEE flags back.
template <typename Enqueue>
wb200_status with_flag_word(wb200_spm_image *image, uint32_t *flags, Enqueue enqueue) {
  if (!image) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  wb200_backend *backend = image->backend;
  DeviceGuard guard(backend->device);
  void *word;
  wb200_status st = backend->buffer(3, sizeof(uint32_t), &word);
  if (st != WB200_OK) return st;
  cudaStream_t stream = image->work_stream();
  WB200_CUDA_CHECK(cudaMemsetAsync(word, 0, sizeof(uint32_t), stream));
  if ((st = enqueue(static_cast<uint32_t *>(word))) != WB200_OK) return st;
  uint32_t host = 0;
  WB200_CUDA_CHECK(cudaMemcpyAsync(&host, word, sizeof(host), cudaMemcpyDeviceToHost, stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(stream));
  if (flags) *flags = host;
  return WB200_OK;
}
}  // namespace

extern "C" {

wb200_status wb200_target_call_gemm(wb200_spm_image *image, uint64_t lhs, uint64_t rhs, uint64_t dst, uint64_t psum,
                                    uint32_t m, uint32_t k, uint32_t n, uint32_t batch, uint32_t in_format,
                                    uint32_t out_format, uint32_t psum_format, uint32_t lhs_orientation,
                                    uint32_t rhs_orientation, uint32_t policy) {
  wb200_status st = enqueue_image_gemm(image, lhs, rhs, dst, psum, m, k, n, batch, in_format, out_format, psum_format,
                                       lhs_orientation, rhs_orientation, policy);
  if (st != WB200_OK) return st;
  return read_device_status(image->backend, image->backend->stream, nullptr);
}

wb200_status wb200_target_call_elementwise(wb200_spm_image *image, uint32_t operation, uint64_t lhs, uint64_t rhs_or_scalar_bits,
                                           uint64_t dst, uint32_t count, uint32_t format, uint32_t rhs_unit_elements,
                                           uint32_t scalar_flag, uint32_t relation_numeric_or_rhs_group, uint32_t *flags) {
  return with_flag_word(image, flags, [&](uint32_t *word) {
    return enqueue_image_elementwise(image, operation, lhs, rhs_or_scalar_bits, dst, count, format, rhs_unit_elements, scalar_flag,
                                     relation_numeric_or_rhs_group, word, true);
  });
}

wb200_status wb200_target_call_reduce(wb200_spm_image *image, uint32_t operation, uint64_t source, uint64_t destination, uint32_t dimension,
                                      const uint32_t nhwc[4], uint32_t format, uint32_t *flags) {
  return with_flag_word(image, flags, [&](uint32_t *word) {
    return enqueue_image_reduce(image, operation, source, destination, dimension, nhwc, format, word, true);
  });
}

wb200_status wb200_target_call_pool(wb200_spm_image *image, uint32_t kind, uint64_t input, uint64_t dst, const uint32_t source_shape[4],
                                    const uint32_t destination_shape[4], const uint32_t pads[4], const uint32_t kernel_strides[4],
                                    uint32_t format, uint32_t *flags) {
  return with_flag_word(image, flags, [&](uint32_t *word) {
    return enqueue_image_pool(image, kind, input, dst, source_shape, destination_shape, pads, kernel_strides, format, word, true);
  });
}

}  // extern "C"
