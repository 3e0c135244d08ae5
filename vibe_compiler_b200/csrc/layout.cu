// Host-side physical tensor geometry: the arithmetic of the reference's
// computePhysicalTensorGeometry (lib/Wafer/Target/PhysicalTensor/PhysicalLayout.cpp:111-200) and
// computeCxC0 / alignCxTail (:51-85), restated on plain integers.
#include <mutex>

#include "common.cuh"

namespace wb200 {

namespace {
thread_local std::string g_last_error;
}

void set_last_error(const std::string &message) { g_last_error = message; }
wb200_status fail(wb200_status status, const std::string &message) {
  g_last_error = message;
  return status;
}
const char *last_error_cstr() { return g_last_error.c_str(); }

static int64_t align_cx_tail(int64_t tail) {
  if (tail <= 4) return 4;
  if (tail <= 8) return 8;
  if (tail <= 16) return 16;
  if (tail <= 32) return 32;
  return 64;
}

wb200_status make_layout_map(const wb200_tensor_desc &desc, LayoutMap *map, wb200_geometry *geometry) {
  const int bits = format_bits(desc.format);
  if (bits == 0) return fail(WB200_ERR_INVALID_ARGUMENT, "unknown logical format");
  if (desc.rank < 1 || desc.rank > WB200_MAX_RANK) return fail(WB200_ERR_INVALID_ARGUMENT, "tensor rank must be 1..8");
  if (desc.layout > WB200_LAYOUT_NCX) return fail(WB200_ERR_INVALID_ARGUMENT, "unknown physical layout");
  LayoutMap m{};
  wb200_geometry g{};
  m.layout = desc.layout;
  m.rank = desc.rank;
  int64_t count = 1;
  for (int d = 0; d < desc.rank; ++d) {
    if (desc.shape[d] > (1ull << 40)) return fail(WB200_ERR_INVALID_ARGUMENT, "tensor dimension too large");
    m.shape[d] = static_cast<int64_t>(desc.shape[d]);
    count *= m.shape[d];
    if (count > (1ll << 46)) return fail(WB200_ERR_INVALID_ARGUMENT, "tensor element count too large");
  }
  m.element_count = count;
  g.element_bytes = (bits + 7) / 8;
  g.compact_bytes = (count * bits + 7) / 8;
  if (desc.layout == WB200_LAYOUT_TENSOR || desc.layout == WB200_LAYOUT_NTENSOR) {
    m.physical_elements = count;
    g.physical_elements = count;
    g.physical_bytes = (count * bits + 7) / 8;
  } else {
    const bool int8_block = desc.format == WB200_I8 || desc.format == WB200_U8;
    const int64_t block = int8_block ? 128 : 64;
    const int64_t retain = int8_block ? 64 : 32;
    const int64_t channels = m.shape[desc.rank - 1];
    const int64_t quotient = channels / block, remainder = channels % block;
    int64_t blocks, tail, aligned;
    if (remainder == 0) { blocks = quotient; tail = 0; aligned = quotient * block; }
    else if (remainder <= retain) { blocks = quotient; tail = align_cx_tail(remainder); aligned = quotient * block + tail; }
    else { blocks = quotient + 1; tail = 0; aligned = blocks * block; }
    constexpr int64_t kBankLineBits = 256 * 8;
    if (kBankLineBits % bits != 0) return fail(WB200_ERR_INVALID_ARGUMENT, "element width does not divide the bank line");
    const int64_t bank_align = kBankLineBits / bits;
    int64_t outer_slices = 1, block_outer = 1;
    if (desc.layout == WB200_LAYOUT_NCX) {
      outer_slices = desc.rank > 1 ? m.shape[0] : 1;
      for (int d = 1; d + 1 < desc.rank; ++d) block_outer *= m.shape[d];
    } else {
      for (int d = 0; d + 1 < desc.rank; ++d) block_outer *= m.shape[d];
    }
    const int64_t unpadded = block_outer * aligned;
    const int64_t slice_stride = ((unpadded + bank_align - 1) / bank_align) * bank_align;
    m.c_block = block; m.cx_blocks = blocks; m.c0 = tail;
    m.block_outer_elements = block_outer;
    m.outer_slice_stride = slice_stride;
    m.physical_elements = outer_slices * slice_stride;
    g.c_block = block; g.cx_blocks = blocks; g.c0 = tail; g.aligned_c = aligned;
    g.outer_elements = outer_slices * block_outer;
    g.block_outer_elements = block_outer;
    g.outer_slice_stride_elements = slice_stride;
    g.bank_align_elements = bank_align;
    g.physical_elements = m.physical_elements;
    g.physical_bytes = (m.physical_elements * bits + 7) / 8;
  }
  if (map) *map = m;
  if (geometry) *geometry = g;
  return WB200_OK;
}

}  // namespace wb200
