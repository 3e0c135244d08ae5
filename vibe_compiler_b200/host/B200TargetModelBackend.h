// C++ host-side mirror of the reference's numeric-backend seam over the libwb200 C ABI.
//
// The reference selects its tensor backends through two abstract classes
// (include/Wafer/Simulator/Kernel/TargetModelKernel.h:164-170 TargetModelOneDNNBackend::tryExecute and
// :187-200 TargetModelManagedReferenceBackend::execute x3) whose requests carry a PhysicalTensorDescriptor
// plus the full physical storage bytes of every operand. This header offers the same four calls with the same
// names, argument meaning and error behaviour, with std:: types in place of LLVM's (llvm::Expected<T> becomes
// wafer_b200::Expected<T>, llvm::ArrayRef becomes std::vector), so that a reference-side adapter is a field-by-field
// copy. Header only; link with -lwb200.
#pragma once

#include <cstdint>
#include <optional>
#include <string>
#include <utility>
#include <vector>

#include "../../include/wb200.h"

namespace wafer_b200 {

// Minimal stand-in for llvm::Expected<T>: either a value or an error message with the wb200 status.
template <typename T>
class Expected {
public:
  Expected(T value) : value_(std::move(value)) {}
  static Expected failure(wb200_status status, std::string message) {
    Expected e;
    e.status_ = status;
    e.message_ = std::move(message);
    return e;
  }
  explicit operator bool() const { return value_.has_value(); }
  T &operator*() { return *value_; }
  const T &operator*() const { return *value_; }
  T *operator->() { return &*value_; }
  wb200_status status() const { return status_; }
  const std::string &message() const { return message_; }

private:
  Expected() = default;
  std::optional<T> value_;
  wb200_status status_ = WB200_OK;
  std::string message_;
};

// Mirrors wafer::PhysicalTensorDescriptor {format, layout, shape}.
struct PhysicalTensorDescriptor {
  wb200_format format;
  wb200_layout layout;
  std::vector<uint64_t> shape;

  wb200_tensor_desc c() const {
    wb200_tensor_desc d{};
    d.format = static_cast<uint8_t>(format);
    d.layout = static_cast<uint8_t>(layout);
    d.rank = static_cast<uint8_t>(shape.size());
    for (size_t i = 0; i < shape.size() && i < WB200_MAX_RANK; ++i) d.shape[i] = shape[i];
    return d;
  }
};

// Mirrors TargetModelNumericTensor / TargetModelNumericOperands (TargetModelKernel.h:108-116).
struct TargetModelNumericTensor {
  PhysicalTensorDescriptor key;
  std::vector<uint8_t> storage;
};
struct TargetModelNumericOperands {
  std::vector<TargetModelNumericTensor> inputs;
  TargetModelNumericTensor destinationTemplate;
};

// Mirrors FormalGemmOperation / FormalElementwiseOperation / FormalConvertOperation / FormalReduceOperation
// (include/Wafer/Simulator/Reference/FormalOperations.h:21-113).
struct FormalGemmOperation {
  PhysicalTensorDescriptor lhs, rhs, destination;
  uint32_t m, k, n, batchCount;
  wb200_orientation lhsOrientation = WB200_NORMAL, rhsOrientation = WB200_NORMAL;
  std::optional<PhysicalTensorDescriptor> psum;
};
struct FormalElementwiseOperation {
  wb200_elementwise_op operation;
  std::vector<PhysicalTensorDescriptor> inputs;
  PhysicalTensorDescriptor destination;
};
struct FormalConvertOperation {
  uint16_t opcode;
  PhysicalTensorDescriptor source, destination;
  uint32_t roundingMode = 0;  // TargetRoundingMode::NearestEven
};
struct FormalReduceOperation {
  wb200_reduce_op operation;
  PhysicalTensorDescriptor input, destination;
  wb200_reduce_dim dimension;
};
struct TargetModelGemmRequest { FormalGemmOperation operation; TargetModelNumericOperands tensors; };
struct TargetModelElementwiseRequest { FormalElementwiseOperation operation; TargetModelNumericOperands tensors; };
struct TargetModelConvertRequest { FormalConvertOperation operation; TargetModelNumericOperands tensors; };
struct TargetModelReduceRequest { FormalReduceOperation operation; TargetModelNumericOperands tensors; };

// Mirrors TargetModelOneDNNDispatchEvidence + TargetModelManagedReferenceEvidence (:143-150, :172-176).
struct TargetModelB200Result {
  TargetModelNumericTensor destination;
  wb200_evidence evidence;
};

// Mirrors FormalNumericWorkBudget (only the scalar-evaluation limit matters to the managed contract).
struct FormalNumericWorkBudget { uint64_t maximumScalarEvaluations = ~0ull; };

class TargetModelB200Backend {
public:
  static Expected<TargetModelB200Backend> create(int device = 0, uint64_t maximumTotalBytes = 0,
                                                 uint64_t maximumScratchpadBytes = 0) {
    wb200_backend *handle = nullptr;
    wb200_status st = wb200_backend_create(device, &handle);
    if (st != WB200_OK) return Expected<TargetModelB200Backend>::failure(st, wb200_last_error());
    wb200_backend_set_budget(handle, maximumTotalBytes, maximumScratchpadBytes);
    return Expected<TargetModelB200Backend>(TargetModelB200Backend(handle));
  }
  TargetModelB200Backend(TargetModelB200Backend &&other) noexcept : handle_(other.handle_) { other.handle_ = nullptr; }
  TargetModelB200Backend &operator=(TargetModelB200Backend &&other) noexcept {
    std::swap(handle_, other.handle_);
    return *this;
  }
  TargetModelB200Backend(const TargetModelB200Backend &) = delete;
  ~TargetModelB200Backend() { if (handle_) wb200_backend_destroy(handle_); }

  // TargetModelOneDNNBackend::tryExecute: a successful null optional means "outside this backend's domain,
  // use the formal path" (psum, transposed operands, mixed formats), exactly as the reference declines.
  Expected<std::optional<TargetModelB200Result>> tryExecute(const TargetModelGemmRequest &request,
                                                            wb200_gemm_policy policy = WB200_GEMM_TENSOR) const {
    using Out = Expected<std::optional<TargetModelB200Result>>;
    const FormalGemmOperation &op = request.operation;
    if (request.tensors.inputs.size() != (op.psum ? 3u : 2u))
      return Out::failure(WB200_ERR_INVALID_ARGUMENT, "NE GEMM execution requires two inputs (three with psum)");
    wb200_gemm_request r{};
    r.lhs = op.lhs.c(); r.rhs = op.rhs.c(); r.destination = op.destination.c();
    r.m = op.m; r.k = op.k; r.n = op.n; r.batch_count = op.batchCount;
    r.lhs_orientation = static_cast<uint8_t>(op.lhsOrientation);
    r.rhs_orientation = static_cast<uint8_t>(op.rhsOrientation);
    r.policy = static_cast<uint8_t>(policy);
    const auto &in = request.tensors.inputs;
    r.lhs_storage = in[0].storage.data(); r.lhs_bytes = in[0].storage.size();
    r.rhs_storage = in[1].storage.data(); r.rhs_bytes = in[1].storage.size();
    if (op.psum) {
      r.has_psum = 1;
      r.psum = op.psum->c();
      r.psum_storage = in[2].storage.data(); r.psum_bytes = in[2].storage.size();
    }
    TargetModelB200Result result{{op.destination, request.tensors.destinationTemplate.storage}, {}};
    r.destination_template = request.tensors.destinationTemplate.storage.data();
    r.destination_out = result.destination.storage.data();
    r.destination_bytes = result.destination.storage.size();
    int handled = 0;
    wb200_status st = wb200_gemm(handle_, &r, &handled, &result.evidence);
    if (st != WB200_OK) return Out::failure(st, wb200_last_error());
    if (!handled) return Out(std::optional<TargetModelB200Result>());
    return Out(std::optional<TargetModelB200Result>(std::move(result)));
  }

  // `formal` selects the bit-exact family the reference falls back to when its managed backend declines a request
  // (NaN operands, relations, logic, IEEE flags in evidence.flags): wb200_elementwise_formal / wb200_convert_formal /
  // wb200_reduce_formal in place of the managed entries.
  Expected<TargetModelB200Result> execute(const TargetModelElementwiseRequest &request,
                                          FormalNumericWorkBudget scalarBudget, bool formal = false) const {
    using Out = Expected<TargetModelB200Result>;
    const auto &op = request.operation;
    if (request.tensors.inputs.size() != op.inputs.size() || op.inputs.size() > 2)
      return Out::failure(WB200_ERR_INVALID_ARGUMENT, "elementwise input arity does not match semantics");
    wb200_elementwise_request r{};
    r.operation = op.operation;
    r.input_count = static_cast<uint32_t>(op.inputs.size());
    for (size_t i = 0; i < op.inputs.size(); ++i) {
      r.inputs[i] = op.inputs[i].c();
      r.input_storage[i] = request.tensors.inputs[i].storage.data();
      r.input_bytes[i] = request.tensors.inputs[i].storage.size();
    }
    r.destination = op.destination.c();
    TargetModelB200Result result{{op.destination, request.tensors.destinationTemplate.storage}, {}};
    r.destination_template = request.tensors.destinationTemplate.storage.data();
    r.destination_out = result.destination.storage.data();
    r.destination_bytes = result.destination.storage.size();
    r.max_scalar_evaluations = scalarBudget.maximumScalarEvaluations;
    wb200_status st = formal ? wb200_elementwise_formal(handle_, &r, &result.evidence) : wb200_elementwise(handle_, &r, &result.evidence);
    if (st != WB200_OK) return Out::failure(st, wb200_last_error());
    return Out(std::move(result));
  }

  Expected<TargetModelB200Result> execute(const TargetModelConvertRequest &request,
                                          FormalNumericWorkBudget scalarBudget, bool formal = false) const {
    using Out = Expected<TargetModelB200Result>;
    if (request.tensors.inputs.size() != 1) return Out::failure(WB200_ERR_INVALID_ARGUMENT, "convert takes one input");
    const auto &op = request.operation;
    wb200_convert_request r{};
    r.opcode = op.opcode;
    r.rounding_mode = op.roundingMode;
    r.source = op.source.c(); r.destination = op.destination.c();
    r.source_storage = request.tensors.inputs[0].storage.data();
    r.source_bytes = request.tensors.inputs[0].storage.size();
    TargetModelB200Result result{{op.destination, request.tensors.destinationTemplate.storage}, {}};
    r.destination_template = request.tensors.destinationTemplate.storage.data();
    r.destination_out = result.destination.storage.data();
    r.destination_bytes = result.destination.storage.size();
    r.max_scalar_evaluations = scalarBudget.maximumScalarEvaluations;
    wb200_status st = formal ? wb200_convert_formal(handle_, &r, &result.evidence) : wb200_convert(handle_, &r, &result.evidence);
    if (st != WB200_OK) return Out::failure(st, wb200_last_error());
    return Out(std::move(result));
  }

  Expected<TargetModelB200Result> execute(const TargetModelReduceRequest &request,
                                          FormalNumericWorkBudget scalarBudget, bool formal = false) const {
    using Out = Expected<TargetModelB200Result>;
    if (request.tensors.inputs.size() != 1) return Out::failure(WB200_ERR_INVALID_ARGUMENT, "reduce takes one input");
    const auto &op = request.operation;
    wb200_reduce_request r{};
    r.operation = op.operation;
    r.dimension = op.dimension;
    r.input = op.input.c(); r.destination = op.destination.c();
    r.input_storage = request.tensors.inputs[0].storage.data();
    r.input_bytes = request.tensors.inputs[0].storage.size();
    TargetModelB200Result result{{op.destination, request.tensors.destinationTemplate.storage}, {}};
    r.destination_template = request.tensors.destinationTemplate.storage.data();
    r.destination_out = result.destination.storage.data();
    r.destination_bytes = result.destination.storage.size();
    r.max_scalar_evaluations = scalarBudget.maximumScalarEvaluations;
    wb200_status st = formal ? wb200_reduce_formal(handle_, &r, &result.evidence) : wb200_reduce(handle_, &r, &result.evidence);
    if (st != WB200_OK) return Out::failure(st, wb200_last_error());
    return Out(std::move(result));
  }

  wb200_backend *handle() const { return handle_; }

private:
  explicit TargetModelB200Backend(wb200_backend *handle) : handle_(handle) {}
  wb200_backend *handle_ = nullptr;
};

}  // namespace wafer_b200
