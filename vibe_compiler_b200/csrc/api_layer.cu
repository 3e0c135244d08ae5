// wb200_decoder_layer: one rank's shard of a Llama-style decoder layer forward as a single C-ABI call.
// The ten kernels are the library's own regions (RMSNorm, tcgen05 GEMM with NONE / SwiGLU epilogues, rotary +
// head-major split, tcgen05 flash attention, residual add); the two sums over shards are delegated to the caller's
// all-reduce callback, which stands where the reference places its Tile collectives
// (lib/Wafer/Transforms/Tile/DistributedCollectiveMovement.cpp:675-735).
#include "backend.h"

namespace wb200 {
namespace {

constexpr size_t kAlign = 256;
size_t round_up(size_t bytes) { return (bytes + kAlign - 1) / kAlign * kAlign; }

struct LayerPlan {
  size_t tokens, qkv_cols, attn_cols;
  size_t off_h, off_qkv, off_q, off_k, off_v, off_attn, off_partial, off_x1, off_act, total;
};

wb200_status plan_layer(const wb200_decoder_layer_params *p, LayerPlan *plan) {
  if (p->format != WB200_BF16 && p->format != WB200_F16) return fail(WB200_ERR_UNSUPPORTED, "decoder layer takes bf16 or f16 storage");
  if (!p->batch || !p->seq || !p->d_model || !p->head_dim || !p->q_heads || !p->kv_heads || !p->ffn)
    return fail(WB200_ERR_INVALID_ARGUMENT, "decoder layer extents must be positive");
  if (p->q_heads % p->kv_heads != 0) return fail(WB200_ERR_INVALID_ARGUMENT, "q_heads must be a multiple of kv_heads");
  if (p->d_model % 8 != 0 || p->head_dim % 8 != 0 || p->ffn % 16 != 0 || (static_cast<uint64_t>(p->batch) * p->seq) % 8 != 0)
    return fail(WB200_ERR_UNSUPPORTED, "decoder layer needs d_model % 8 == 0, head_dim % 8 == 0, ffn % 16 == 0 and tokens % 8 == 0");
  const size_t e = 2;
  plan->tokens = static_cast<size_t>(p->batch) * p->seq;
  plan->qkv_cols = static_cast<size_t>(p->q_heads + 2 * p->kv_heads) * p->head_dim;
  plan->attn_cols = static_cast<size_t>(p->q_heads) * p->head_dim;
  size_t at = 0;
  auto take = [&](size_t elements) { const size_t here = at; at += round_up(elements * e); return here; };
  plan->off_h = take(plan->tokens * p->d_model);          // normalised activations (both norms)
  plan->off_qkv = take(plan->tokens * plan->qkv_cols);
  plan->off_q = take(plan->tokens * plan->attn_cols);
  plan->off_k = take(plan->tokens * p->kv_heads * p->head_dim);
  plan->off_v = take(plan->tokens * p->kv_heads * p->head_dim);
  plan->off_attn = take(plan->tokens * plan->attn_cols);
  plan->off_partial = take(plan->tokens * p->d_model);    // both partial sums
  plan->off_x1 = take(plan->tokens * p->d_model);
  plan->off_act = take(plan->tokens * p->ffn);
  plan->total = at;
  return WB200_OK;
}

}  // namespace
}  // namespace wb200

using namespace wb200;

extern "C" {

uint64_t wb200_decoder_layer_workspace_bytes(const wb200_decoder_layer_params *p) {
  LayerPlan plan;
  if (!p || plan_layer(p, &plan) != WB200_OK) return 0;
  return plan.total;
}

wb200_status wb200_decoder_layer(wb200_backend *backend, const wb200_decoder_layer_params *p) {
  if (!backend || !p) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  if (!p->x || !p->out || !p->norm1 || !p->wqkv || !p->wo || !p->norm2 || !p->wgu || !p->wdown || !p->workspace)
    return fail(WB200_ERR_INVALID_ARGUMENT, "decoder layer pointers must not be null");
  LayerPlan plan;
  wb200_status st = plan_layer(p, &plan);
  if (st != WB200_OK) return st;
  if (p->workspace_bytes < plan.total) return fail(WB200_ERR_LIMIT, "workspace smaller than wb200_decoder_layer_workspace_bytes()");
  if (reinterpret_cast<uintptr_t>(p->workspace) % kAlign) return fail(WB200_ERR_INVALID_ARGUMENT, "workspace must be 256-byte aligned");
  DeviceGuard guard(backend->device);
  cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  uint8_t *ws = static_cast<uint8_t *>(p->workspace);
  void *h = ws + plan.off_h, *qkv = ws + plan.off_qkv, *q = ws + plan.off_q, *k = ws + plan.off_k, *v = ws + plan.off_v;
  void *attn = ws + plan.off_attn, *partial = ws + plan.off_partial, *x1 = ws + plan.off_x1, *act = ws + plan.off_act;
  const int tokens = static_cast<int>(plan.tokens), d = p->d_model, fmt = p->format;

  auto gemm = [&](const void *a, const void *b, void *out, int m, int n, int kk, int epilogue) -> wb200_status {
    GemmUmmaArgs g{};
    g.m = m; g.n = n; g.k = kk;
    g.in_format = fmt; g.out_format = fmt;
    g.epilogue = epilogue;
    g.a = a; g.b = b; g.out = out;
    wb200_status s = launch_gemm_umma(g, backend->sm_count, backend->d_status, stream);
    if (s == WB200_OK) backend->launches += 1;
    return s;
  };
  auto reduce = [&](void *buffer) -> wb200_status {
    if (!p->allreduce) return WB200_OK;
    if (p->allreduce(p->allreduce_user, buffer, static_cast<uint64_t>(tokens) * d, p->format, p->stream) != 0)
      return fail(WB200_ERR_CALLBACK, "the all-reduce callback reported a failure");
    return WB200_OK;
  };

  if ((st = launch_rmsnorm(fmt, p->x, p->norm1, h, tokens, d, p->eps, stream)) != WB200_OK) return st;
  backend->launches += 1;
  if ((st = gemm(h, p->wqkv, qkv, tokens, static_cast<int>(plan.qkv_cols), d, WB200_EPI_NONE)) != WB200_OK) return st;
  if ((st = launch_rope_split(fmt, qkv, q, k, v, p->batch, p->seq, p->q_heads, p->kv_heads, p->head_dim, p->rope_theta,
                              static_cast<int>(p->position_offset), stream)) != WB200_OK) return st;
  backend->launches += 1;
  AttentionArgs a{};
  a.batch = p->batch; a.q_heads = p->q_heads; a.kv_heads = p->kv_heads; a.q_len = p->seq; a.kv_len = p->seq; a.head_dim = p->head_dim;
  a.format = fmt; a.causal = 1; a.zero_fully_masked = 0;
  a.scale = 1.0f / sqrtf(static_cast<float>(p->head_dim));
  a.causal_offset = 0; a.kv_valid = p->seq;
  a.q = q; a.k = k; a.v = v; a.out = attn;
  a.out_token_major = 1;
  st = attention_fa_umma_supports(a) ? launch_attention_fa_umma(a, backend->sm_count, backend->d_status, stream)
                                     : launch_attention_fa_simt(a, stream);
  if (st != WB200_OK) return st;
  backend->launches += 1;
  if ((st = gemm(attn, p->wo, partial, tokens, d, static_cast<int>(plan.attn_cols), WB200_EPI_NONE)) != WB200_OK) return st;
  if ((st = reduce(partial)) != WB200_OK) return st;
  if ((st = launch_residual_add(fmt, p->x, partial, x1, plan.tokens * d, stream)) != WB200_OK) return st;
  backend->launches += 1;
  if ((st = launch_rmsnorm(fmt, x1, p->norm2, h, tokens, d, p->eps, stream)) != WB200_OK) return st;
  backend->launches += 1;
  if ((st = gemm(h, p->wgu, act, tokens, 2 * static_cast<int>(p->ffn), d, WB200_EPI_SWIGLU)) != WB200_OK) return st;
  if ((st = gemm(act, p->wdown, partial, tokens, d, static_cast<int>(p->ffn), WB200_EPI_NONE)) != WB200_OK) return st;
  if ((st = reduce(partial)) != WB200_OK) return st;
  if ((st = launch_residual_add(fmt, x1, partial, p->out, plan.tokens * d, stream)) != WB200_OK) return st;
  backend->launches += 1;
  return WB200_OK;
}

}  // extern "C"
