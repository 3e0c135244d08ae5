// Memory-bound producer / epilogue pieces of a Llama-style decoder layer that sit between the GEMM and
// attention regions: RMSNorm, rotary embedding fused with the head-major relayout of the QKV projection,
// and the residual add. Arithmetic is f32 with one rounding to the storage type per produced element,
// the accumulation contract of the reference's elementwise chains
// (lib/Wafer/Simulator/Reference/ManagedReferenceTargetModel.cpp:230-342: decode to f32, operate, RNE encode).
// All three are HBM-bound: algorithmic bytes = bytes read + bytes written once.
#include "kernels.h"

namespace wb200 {
namespace {

constexpr int kNormThreads = 256;

template <bool kBf16>
__device__ __forceinline__ float2 unpack2(uint32_t bits) {
  if constexpr (kBf16) return make_float2(__uint_as_float(bits << 16), __uint_as_float(bits & 0xffff0000u));
  else return __half22float2(*reinterpret_cast<const __half2 *>(&bits));
}
template <bool kBf16>
__device__ __forceinline__ uint32_t pack2f(float lo, float hi) {
  if constexpr (kBf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
  }
}

// y[row] = round(round(x * rsqrt(mean(x^2) + eps)) * gamma): the normalised value is rounded to the storage
// type before the weight is applied, as the eager module the reference's block test runs does.
template <bool kBf16>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(const uint16_t *x, const uint16_t *gamma, uint16_t *y,
                                                                int rows, int dim, float eps) {
  const int row = blockIdx.x;
  const uint4 *src = reinterpret_cast<const uint4 *>(x + static_cast<size_t>(row) * dim);
  const int chunks = dim / 8;
  float partial = 0.f;
  for (int c = threadIdx.x; c < chunks; c += kNormThreads) {
    const uint4 v = src[c];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = unpack2<kBf16>(w[i]);
      partial = fmaf(f.x, f.x, partial);
      partial = fmaf(f.y, f.y, partial);
    }
  }
  __shared__ float warp_sums[kNormThreads / 32];
  __shared__ float inv_rms;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, off);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = partial;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int w = 0; w < kNormThreads / 32; ++w) total += warp_sums[w];
    inv_rms = rsqrtf(total / static_cast<float>(dim) + eps);
  }
  __syncthreads();
  const float inv = inv_rms;
  const uint4 *g = reinterpret_cast<const uint4 *>(gamma);
  uint4 *dst = reinterpret_cast<uint4 *>(y + static_cast<size_t>(row) * dim);
  for (int c = threadIdx.x; c < chunks; c += kNormThreads) {
    const uint4 v = src[c], gv = g[c];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = unpack2<kBf16>(w[i]);
      const float2 normalised = unpack2<kBf16>(pack2f<kBf16>(f.x * inv, f.y * inv));
      const float2 gf = unpack2<kBf16>(gw[i]);
      o[i] = pack2f<kBf16>(normalised.x * gf.x, normalised.y * gf.y);
    }
    dst[c] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// qkv is the projection output, token-major: row (b * seq + s) holds [q heads | k heads | v heads] x head_dim.
// Writes head-major Q [B, Hq, S, D], K [B, Hkv, S, D], V [B, Hkv, S, D]; Q and K get the rotary embedding
// (pairs (i, i + D/2), angle = (position_offset + s) * theta^(-2i/D), f32 math, one rounding).
template <bool kBf16>
__global__ void __launch_bounds__(256) rope_split_kernel(const uint16_t *qkv, uint16_t *q, uint16_t *k, uint16_t *v,
                                                          int batch, int seq, int q_heads, int kv_heads, int head_dim,
                                                          float log2_theta, int position_offset) {
  const int token = blockIdx.x;
  const int b = token / seq, s = token % seq;
  const int heads = q_heads + 2 * kv_heads;
  const int half = head_dim / 2;
  const uint16_t *row = qkv + static_cast<size_t>(token) * heads * head_dim;
  const int pairs_per_head = half / 2;   // each thread handles two adjacent rotation pairs (4 elements)
  for (int idx = threadIdx.x; idx < heads * pairs_per_head; idx += blockDim.x) {
    const int head = idx / pairs_per_head, i = (idx % pairs_per_head) * 2;
    const uint16_t *src = row + static_cast<size_t>(head) * head_dim;
    const float2 lo = unpack2<kBf16>(*reinterpret_cast<const uint32_t *>(src + i));
    const float2 hi = unpack2<kBf16>(*reinterpret_cast<const uint32_t *>(src + i + half));
    uint16_t *dst;
    bool rotate = true;
    if (head < q_heads) dst = q + ((static_cast<size_t>(b) * q_heads + head) * seq + s) * head_dim;
    else if (head < q_heads + kv_heads) dst = k + ((static_cast<size_t>(b) * kv_heads + (head - q_heads)) * seq + s) * head_dim;
    else { dst = v + ((static_cast<size_t>(b) * kv_heads + (head - q_heads - kv_heads)) * seq + s) * head_dim; rotate = false; }
    float2 out_lo = lo, out_hi = hi;
    if (rotate) {
      const float position = static_cast<float>(position_offset + s);
      float s0, c0, s1, c1;
      sincosf(position * exp2f(-2.0f * static_cast<float>(i) / static_cast<float>(head_dim) * log2_theta), &s0, &c0);
      sincosf(position * exp2f(-2.0f * static_cast<float>(i + 1) / static_cast<float>(head_dim) * log2_theta), &s1, &c1);
      out_lo = make_float2(lo.x * c0 - hi.x * s0, lo.y * c1 - hi.y * s1);
      out_hi = make_float2(hi.x * c0 + lo.x * s0, hi.y * c1 + lo.y * s1);
    }
    *reinterpret_cast<uint32_t *>(dst + i) = pack2f<kBf16>(out_lo.x, out_lo.y);
    *reinterpret_cast<uint32_t *>(dst + i + half) = pack2f<kBf16>(out_hi.x, out_hi.y);
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(256) residual_add_kernel(const uint4 *a, const uint4 *b, uint4 *out, size_t chunks) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t c = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < chunks; c += stride) {
    const uint4 x = a[c], y = b[c];
    const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, yw[4] = {y.x, y.y, y.z, y.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 fx = unpack2<kBf16>(xw[i]), fy = unpack2<kBf16>(yw[i]);
      o[i] = pack2f<kBf16>(fx.x + fy.x, fx.y + fy.y);
    }
    out[c] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

wb200_status launch_rmsnorm(int format, const void *x, const void *gamma, void *y, int rows, int dim, float eps,
                            cudaStream_t stream) {
  if (format != WB200_BF16 && format != WB200_F16) return fail(WB200_ERR_UNSUPPORTED, "rmsnorm takes bf16 or f16 storage");
  if (rows <= 0 || dim <= 0 || dim % 8 != 0 || !aligned16(x) || !aligned16(gamma) || !aligned16(y))
    return fail(WB200_ERR_INVALID_ARGUMENT, "rmsnorm needs dim % 8 == 0 and 16-byte aligned buffers");
  if (format == WB200_BF16)
    rmsnorm_kernel<true><<<rows, kNormThreads, 0, stream>>>(static_cast<const uint16_t *>(x), static_cast<const uint16_t *>(gamma), static_cast<uint16_t *>(y), rows, dim, eps);
  else
    rmsnorm_kernel<false><<<rows, kNormThreads, 0, stream>>>(static_cast<const uint16_t *>(x), static_cast<const uint16_t *>(gamma), static_cast<uint16_t *>(y), rows, dim, eps);
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

wb200_status launch_rope_split(int format, const void *qkv, void *q, void *k, void *v, int batch, int seq, int q_heads,
                               int kv_heads, int head_dim, float theta, int position_offset, cudaStream_t stream) {
  if (format != WB200_BF16 && format != WB200_F16) return fail(WB200_ERR_UNSUPPORTED, "rope takes bf16 or f16 storage");
  if (batch <= 0 || seq <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || head_dim % 4 != 0 || !(theta > 0.f))
    return fail(WB200_ERR_INVALID_ARGUMENT, "invalid rope extents (head_dim % 4 == 0, theta > 0)");
  const int tokens = batch * seq;
  const float log2_theta = log2f(theta);
  if (format == WB200_BF16)
    rope_split_kernel<true><<<tokens, 256, 0, stream>>>(static_cast<const uint16_t *>(qkv), static_cast<uint16_t *>(q), static_cast<uint16_t *>(k),
                                                         static_cast<uint16_t *>(v), batch, seq, q_heads, kv_heads, head_dim, log2_theta, position_offset);
  else
    rope_split_kernel<false><<<tokens, 256, 0, stream>>>(static_cast<const uint16_t *>(qkv), static_cast<uint16_t *>(q), static_cast<uint16_t *>(k),
                                                          static_cast<uint16_t *>(v), batch, seq, q_heads, kv_heads, head_dim, log2_theta, position_offset);
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

wb200_status launch_residual_add(int format, const void *a, const void *b, void *out, size_t elements, cudaStream_t stream) {
  if (format != WB200_BF16 && format != WB200_F16) return fail(WB200_ERR_UNSUPPORTED, "residual add takes bf16 or f16 storage");
  if (elements == 0 || elements % 8 != 0 || !aligned16(a) || !aligned16(b) || !aligned16(out))
    return fail(WB200_ERR_INVALID_ARGUMENT, "residual add needs a multiple of 8 elements and 16-byte aligned buffers");
  const size_t chunks = elements / 8;
  size_t blocks = (chunks + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (format == WB200_BF16)
    residual_add_kernel<true><<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<const uint4 *>(a), static_cast<const uint4 *>(b), static_cast<uint4 *>(out), chunks);
  else
    residual_add_kernel<false><<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<const uint4 *>(a), static_cast<const uint4 *>(b), static_cast<uint4 *>(out), chunks);
  WB200_CUDA_CHECK(cudaGetLastError());
  return WB200_OK;
}

}  // namespace wb200
