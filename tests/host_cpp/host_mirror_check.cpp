// Drives the C++ mirror of the reference's backend interface (TargetModelOneDNNBackend::tryExecute,
// TargetModelManagedReferenceBackend::execute) the way a reference-side adapter would: physical storage in, physical
// storage out, evidence checked like lib/Wafer/Simulator/Kernel/TargetModelTensorNumeric.cpp:787-795 and :101-109.
// Exit codes: 0 pass, 3 no device, anything else a failed check.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include "../../vibe_compiler_b200/host/B200TargetModelBackend.h"

using namespace wafer_b200;

static std::vector<uint8_t> pack_f32(wb200_backend *raw, const PhysicalTensorDescriptor &key, const std::vector<float> &values) {
  wb200_tensor_desc desc = key.c();
  uint64_t bytes = 0;
  if (wb200_physical_bytes(&desc, &bytes) != WB200_OK) return {};
  std::vector<uint8_t> blank(bytes, 0xAB), out(bytes);   // padding bytes must survive: use a recognisable template
  if (wb200_pack(raw, &desc, reinterpret_cast<const uint8_t *>(values.data()), values.size() * 4, blank.data(), out.data(), bytes) != WB200_OK) return {};
  return out;
}
static std::vector<float> unpack_f32(wb200_backend *raw, const PhysicalTensorDescriptor &key, const std::vector<uint8_t> &storage, size_t count) {
  wb200_tensor_desc desc = key.c();
  std::vector<float> out(count);
  if (wb200_unpack(raw, &desc, storage.data(), storage.size(), reinterpret_cast<uint8_t *>(out.data()), count * 4) != WB200_OK) out.clear();
  return out;
}

int main() {
  auto backend = TargetModelB200Backend::create(0);
  if (!backend) {
    std::printf("create failed: %s\n", backend.message().c_str());
    return backend.status() == WB200_ERR_NO_DEVICE ? 3 : 4;
  }
  wb200_backend *raw = nullptr;   // a second handle for the codec helpers
  if (wb200_backend_create(0, &raw) != WB200_OK) return 5;

  // GEMM 2x3 . 3x4 in f32 on Cx storage, small integers: every partial sum is exact.
  const std::vector<float> a = {1, 2, 3, 4, 5, 6}, b = {1, 0, 2, 1, 0, 1, 1, 2, 1, 1, 0, 3};
  PhysicalTensorDescriptor lhs{WB200_F32, WB200_LAYOUT_CX, {2, 3}}, rhs{WB200_F32, WB200_LAYOUT_CX, {3, 4}}, dst{WB200_F32, WB200_LAYOUT_CX, {2, 4}};
  TargetModelGemmRequest gemm;
  gemm.operation = FormalGemmOperation{lhs, rhs, dst, 2, 3, 4, 1};
  gemm.tensors.inputs = {{lhs, pack_f32(raw, lhs, a)}, {rhs, pack_f32(raw, rhs, b)}};
  gemm.tensors.destinationTemplate = {dst, pack_f32(raw, dst, std::vector<float>(8, 0.f))};
  if (gemm.tensors.inputs[0].storage.empty() || gemm.tensors.destinationTemplate.storage.empty()) return 6;
  for (wb200_gemm_policy policy : {WB200_GEMM_FORMAL, WB200_GEMM_TENSOR}) {
    auto result = backend->tryExecute(gemm, policy);
    if (!result) { std::printf("tryExecute failed: %s\n", result.message().c_str()); return 7; }
    if (!result->has_value()) {
      // A successful null optional means "outside this backend's domain, use the formal path": the tensor-core policy
      // takes f16 / bf16 operands only, so it may decline this f32 request; the formal policy may not.
      if (policy == WB200_GEMM_TENSOR) continue;
      std::printf("tryExecute declined a plain GEMM\n");
      return 8;
    }
    const TargetModelB200Result &r = **result;
    const std::vector<float> got = unpack_f32(raw, dst, r.destination.storage, 8);
    for (int i = 0; i < 2; ++i)
      for (int j = 0; j < 4; ++j) {
        float want = 0;
        for (int k = 0; k < 3; ++k) want += a[i * 3 + k] * b[k * 4 + j];
        if (got.size() != 8 || got[i * 4 + j] != want) { std::printf("GEMM mismatch at %d,%d\n", i, j); return 9; }
      }
    if (r.destination.storage.size() != gemm.tensors.destinationTemplate.storage.size()) return 10;
    // The tensor policy reports one matmul invocation and no formal FMAs (the oneDNN seam's rule); the formal policy
    // reports its m * k * n fused multiply-adds instead.
    const bool counted = policy == WB200_GEMM_TENSOR ? (r.evidence.matmul_invocations == 1 && r.evidence.formal_fused_multiply_adds == 0)
                                                     : (r.evidence.formal_fused_multiply_adds == 2 * 3 * 4);
    if (!counted || r.evidence.reorder_invocations > 1 || r.evidence.evidence_kind == 0 || r.evidence.digest[0] == 0 ||
        r.evidence.implementation[0] == 0) { std::printf("GEMM evidence incomplete\n"); return 11; }
  }

  // Elementwise add on a 1-D Tensor, then the NaN rejection of the managed contract.
  PhysicalTensorDescriptor vec{WB200_F32, WB200_LAYOUT_TENSOR, {8}};
  std::vector<float> x = {1, 2, 3, 4, 5, 6, 7, 8}, y = {0.5f, -2, 10, 0, 1, 1, 1, -8};
  TargetModelElementwiseRequest add;
  add.operation = FormalElementwiseOperation{WB200_EW_ADD, {vec, vec}, vec};
  add.tensors.inputs = {{vec, pack_f32(raw, vec, x)}, {vec, pack_f32(raw, vec, y)}};
  add.tensors.destinationTemplate = {vec, pack_f32(raw, vec, std::vector<float>(8, 0.f))};
  auto sum = backend->execute(add, FormalNumericWorkBudget{});
  if (!sum) { std::printf("execute(add) failed: %s\n", sum.message().c_str()); return 12; }
  const std::vector<float> got = unpack_f32(raw, vec, sum->destination.storage, 8);
  for (int i = 0; i < 8; ++i)
    if (got.size() != 8 || got[i] != x[i] + y[i]) return 13;
  if (sum->evidence.scalar_evaluations != 8) return 14;
  auto starved = backend->execute(add, FormalNumericWorkBudget{4});
  if (starved || starved.status() != WB200_ERR_BUDGET) { std::printf("budget was not enforced\n"); return 15; }
  x[3] = std::nanf("");
  add.tensors.inputs[0].storage = pack_f32(raw, vec, x);
  auto rejected = backend->execute(add, FormalNumericWorkBudget{});
  if (rejected || rejected.status() != WB200_ERR_NAN_DOMAIN) { std::printf("NaN input was not rejected\n"); return 16; }

  // The formal family takes the same request: the NaN element becomes the canonical quiet NaN instead of a refusal, the
  // other elements are the same sums, and 1 + 0.5 ... are exact so only no flag or the inexact flag may be raised.
  auto formal = backend->execute(add, FormalNumericWorkBudget{}, /*formal=*/true);
  if (!formal) { std::printf("formal execute(add) failed: %s\n", formal.message().c_str()); return 17; }
  const std::vector<float> formal_got = unpack_f32(raw, vec, formal->destination.storage, 8);
  for (int i = 0; i < 8; ++i) {
    if (i == 3) {
      uint32_t bits;
      std::memcpy(&bits, &formal_got[i], sizeof(bits));
      if (bits != 0x7fc00000u) { std::printf("formal NaN is not canonical\n"); return 18; }
    } else if (formal_got[i] != got[i]) {
      return 19;
    }
  }
  if (formal->evidence.flags & ~16u) { std::printf("unexpected formal flags %u\n", formal->evidence.flags); return 20; }

  wb200_backend_destroy(raw);
  std::printf("PASS\n");
  return 0;
}
