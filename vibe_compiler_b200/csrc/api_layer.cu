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
  // Micro-batches: the batch is cut into `micro_batches` equal parts (whole sequences) that flow through the layer one
  // after the other on the caller's stream, while the all-reduce of each part runs on a second stream: the sum of part i
  // travels over NVLink while the kernels of parts i + 1 ... compute. The compute kernels are persistent (one CTA per
  // SM); `reserved_sms` of the SMs are left to the collective's kernels, which could otherwise not start before a
  // compute kernel ends, or would hold back that kernel's CTAs.
  const wb200_switch_sum_params *switch_sum = p->switch_sum;
  if (switch_sum) {
    if (!switch_sum->multicast || !switch_sum->epoch || switch_sum->world < 2 || switch_sum->world > WB200_MAX_EXCHANGE_RANKS ||
        switch_sum->rank >= switch_sum->world)
      return fail(WB200_ERR_INVALID_ARGUMENT, "switch_sum needs the workspace's multicast address, epoch words and 2 to 16 ranks");
    for (uint32_t r = 0; r < switch_sum->world; ++r)
      if (!switch_sum->signals[r]) return fail(WB200_ERR_INVALID_ARGUMENT, "switch_sum needs every rank's signal words");
  }
  const bool has_sum = p->allreduce || switch_sum;
  // WB200_LAYER_FUSED_RESIDUAL=0 in the environment keeps the residual adds as kernels of their own beside the library's sum.
  static const bool fuse_residual_enabled = []() { const char *env = getenv("WB200_LAYER_FUSED_RESIDUAL"); return !(env && env[0] == '0'); }();
  const bool fused_residual = switch_sum && fuse_residual_enabled;
  const uint32_t parts = (p->micro_batches > 1 && has_sum) ? p->micro_batches : 1;
  if (parts > 1 && (p->batch % parts != 0 || ((static_cast<uint64_t>(p->batch / parts) * p->seq) % 8) != 0))
    return fail(WB200_ERR_INVALID_ARGUMENT, "micro_batches must divide the batch into parts of a multiple of 8 tokens");
  if (parts > 64) return fail(WB200_ERR_INVALID_ARGUMENT, "at most 64 micro-batches");
  DeviceGuard guard(backend->device);
  cudaStream_t user_stream = static_cast<cudaStream_t>(p->stream);
  if (parts > 1 && (st = backend->auxiliary_streams()) != WB200_OK) return st;
  if (parts > 1 && (st = backend->pipeline_events(4 * parts + 2)) != WB200_OK) return st;
  backend->layer_timeline_parts = 0;
  if (parts > 1) WB200_CUDA_CHECK(cudaEventRecord(backend->pipeline_event[4 * parts], user_stream));   // timeline origin
  cudaStream_t comm_stream = parts > 1 ? backend->aux_stream[0] : user_stream;
  int compute_sms = backend->sm_count;
  if (parts > 1 && p->reserved_sms > 0 && static_cast<int>(p->reserved_sms) < backend->sm_count / 2)
    compute_sms = backend->sm_count - static_cast<int>(p->reserved_sms);
  const int fmt = p->format, d = p->d_model;
  const size_t part_tokens = plan.tokens / parts;
  const size_t e = 2;

  struct Part {
    uint32_t index;
    cudaStream_t stream;
    const uint8_t *x;
    uint8_t *out, *h, *qkv, *q, *k, *v, *attn, *partial, *x1, *act;
  };
  auto part_of = [&](uint32_t index) {
    // every buffer of the whole-batch plan is cut at token granularity; the head-major Q / K / V buffers are cut at
    // batch granularity, which is the same thing because a part is a whole number of sequences
    uint8_t *ws = static_cast<uint8_t *>(p->workspace);
    const size_t t0 = index * part_tokens;
    Part part;
    part.index = index;
    part.stream = user_stream;
    part.x = static_cast<const uint8_t *>(p->x) + t0 * d * e;
    part.out = static_cast<uint8_t *>(p->out) + t0 * d * e;
    part.h = ws + plan.off_h + t0 * d * e;
    part.qkv = ws + plan.off_qkv + t0 * plan.qkv_cols * e;
    part.q = ws + plan.off_q + t0 * plan.attn_cols * e;
    part.k = ws + plan.off_k + t0 * p->kv_heads * p->head_dim * e;
    part.v = ws + plan.off_v + t0 * p->kv_heads * p->head_dim * e;
    part.attn = ws + plan.off_attn + t0 * plan.attn_cols * e;
    part.partial = ws + plan.off_partial + t0 * d * e;
    part.x1 = ws + plan.off_x1 + t0 * d * e;
    part.act = ws + plan.off_act + t0 * p->ffn * e;
    return part;
  };
  const int tokens = static_cast<int>(part_tokens);
  const int part_batch = static_cast<int>(p->batch / parts);

  auto gemm = [&](cudaStream_t stream, const void *a, const void *b, void *out, int m, int n, int kk, int epilogue) -> wb200_status {
    GemmUmmaArgs g{};
    g.m = m; g.n = n; g.k = kk;
    g.in_format = fmt; g.out_format = fmt;
    g.epilogue = epilogue;
    g.a = a; g.b = b; g.out = out;
    wb200_status s = launch_gemm_umma(g, compute_sms, backend->d_status, stream);
    if (s == WB200_OK) backend->launches += 1;
    return s;
  };
  // The sum over shards of a part's partial output: ordered after the part's kernels by an event, enqueued on the
  // communication stream; `done` is recorded behind it for the kernels that consume the sum.
  // With the library's own sum the residual add rides in the sum kernel: the owner of a slice adds its copy of the
  // residual to the switch's sum and stores round(residual + sum) - phase 0: x1 = x + attention, into the x1 buffer;
  // phase 1: x1 + FFN, in place - so the layer's residual add kernels (three passes over [tokens, d_model] each) are
  // not launched. The arithmetic is that of the add kernel, bit for bit.
  auto reduce = [&](const Part &part, int phase) -> wb200_status {
    if (!has_sum) return WB200_OK;
    if (parts > 1) {
      cudaEvent_t ready = backend->pipeline_event[4 * part.index + 2 * phase];
      WB200_CUDA_CHECK(cudaEventRecord(ready, part.stream));
      WB200_CUDA_CHECK(cudaStreamWaitEvent(comm_stream, ready, 0));
    }
    if (switch_sum) {
      // the library's own sum: the switch adds and broadcasts the part's region of the (symmetric) workspace
      uint8_t *multicast = static_cast<uint8_t *>(switch_sum->multicast) + (part.partial - static_cast<uint8_t *>(p->workspace));
      uint8_t *multicast_out = multicast;
      const void *residual = nullptr;
      if (fused_residual) {
        if (phase == 0) multicast_out = static_cast<uint8_t *>(switch_sum->multicast) + (part.x1 - static_cast<uint8_t *>(p->workspace));
        residual = phase == 0 ? static_cast<const void *>(part.x) : static_cast<const void *>(part.x1);
      }
      const int blocks = switch_sum->blocks ? static_cast<int>(switch_sum->blocks) : (p->reserved_sms ? static_cast<int>(p->reserved_sms) : 32);
      wb200_status s = launch_switch_sum(multicast, static_cast<uint64_t>(tokens) * d, p->format, static_cast<int>(switch_sum->rank),
                                         static_cast<int>(switch_sum->world), switch_sum->signals, switch_sum->epoch, blocks,
                                         backend->d_status, comm_stream, multicast_out, residual);
      if (s != WB200_OK) return s;
      backend->launches += 1;
    } else if (p->allreduce(p->allreduce_user, part.partial, static_cast<uint64_t>(tokens) * d, p->format, comm_stream) != 0) {
      return fail(WB200_ERR_CALLBACK, "the all-reduce callback reported a failure");
    }
    if (parts > 1) WB200_CUDA_CHECK(cudaEventRecord(backend->pipeline_event[4 * part.index + 2 * phase + 1], comm_stream));
    return WB200_OK;
  };
  auto await_sum = [&](const Part &part, int phase) -> wb200_status {
    if (parts > 1 && has_sum)
      WB200_CUDA_CHECK(cudaStreamWaitEvent(part.stream, backend->pipeline_event[4 * part.index + 2 * phase + 1], 0));
    return WB200_OK;
  };
  // RMSNorm -> QKV -> rotary split -> attention -> output projection -> [sum over shards]
  auto attention_phase = [&](const Part &part) -> wb200_status {
    wb200_status s;
    if ((s = launch_rmsnorm(fmt, part.x, p->norm1, part.h, tokens, d, p->eps, part.stream)) != WB200_OK) return s;
    backend->launches += 1;
    if ((s = gemm(part.stream, part.h, p->wqkv, part.qkv, tokens, static_cast<int>(plan.qkv_cols), d, WB200_EPI_NONE)) != WB200_OK) return s;
    if ((s = launch_rope_split(fmt, part.qkv, part.q, part.k, part.v, part_batch, p->seq, p->q_heads, p->kv_heads, p->head_dim, p->rope_theta,
                               static_cast<int>(p->position_offset), part.stream)) != WB200_OK) return s;
    backend->launches += 1;
    AttentionArgs a{};
    a.batch = part_batch; a.q_heads = p->q_heads; a.kv_heads = p->kv_heads; a.q_len = p->seq; a.kv_len = p->seq; a.head_dim = p->head_dim;
    a.format = fmt; a.causal = 1; a.zero_fully_masked = 0;
    a.scale = 1.0f / sqrtf(static_cast<float>(p->head_dim));
    a.causal_offset = 0; a.kv_valid = p->seq;
    a.q = part.q; a.k = part.k; a.v = part.v; a.out = part.attn;
    a.out_token_major = 1;
    s = attention_fa_umma_supports(a) ? launch_attention_fa_umma(a, compute_sms, backend->d_status, part.stream)
                                      : launch_attention_fa_simt(a, part.stream);
    if (s != WB200_OK) return s;
    backend->launches += 1;
    if ((s = gemm(part.stream, part.attn, p->wo, part.partial, tokens, d, static_cast<int>(plan.attn_cols), WB200_EPI_NONE)) != WB200_OK) return s;
    return reduce(part, 0);
  };
  // residual -> RMSNorm -> gate/up with SwiGLU epilogue -> down projection -> [sum over shards] -> residual
  auto ffn_phase = [&](const Part &part) -> wb200_status {
    wb200_status s;
    if ((s = await_sum(part, 0)) != WB200_OK) return s;
    if (!fused_residual) {
      if ((s = launch_residual_add(fmt, part.x, part.partial, part.x1, static_cast<size_t>(tokens) * d, part.stream)) != WB200_OK) return s;
      backend->launches += 1;
    }
    if ((s = launch_rmsnorm(fmt, part.x1, p->norm2, part.h, tokens, d, p->eps, part.stream)) != WB200_OK) return s;
    backend->launches += 1;
    if ((s = gemm(part.stream, part.h, p->wgu, part.act, tokens, 2 * static_cast<int>(p->ffn), d, WB200_EPI_SWIGLU)) != WB200_OK) return s;
    if ((s = gemm(part.stream, part.act, p->wdown, part.partial, tokens, d, static_cast<int>(p->ffn), WB200_EPI_NONE)) != WB200_OK) return s;
    return reduce(part, 1);
  };
  auto final_residual = [&](const Part &part) -> wb200_status {
    wb200_status s;
    if ((s = await_sum(part, 1)) != WB200_OK) return s;
    if (fused_residual) {   // the sum kernel left x1 + FFN in the partial buffer
      WB200_CUDA_CHECK(cudaMemcpyAsync(part.out, part.partial, static_cast<size_t>(tokens) * d * e, cudaMemcpyDeviceToDevice, part.stream));
      return WB200_OK;
    }
    if ((s = launch_residual_add(fmt, part.x1, part.partial, part.out, static_cast<size_t>(tokens) * d, part.stream)) != WB200_OK) return s;
    backend->launches += 1;
    return WB200_OK;
  };

  // Phase by phase over the parts, so that the all-reduces are issued in the order their inputs become ready. Every
  // kernel is on the caller's stream and every sum's `done` event is waited for there, so the call leaves no work
  // behind that the caller's stream is not ordered after; on a failure the enqueued part is simply left to finish.
  for (uint32_t i = 0; i < parts; ++i)
    if ((st = attention_phase(part_of(i))) != WB200_OK) break;
  for (uint32_t i = 0; st == WB200_OK && i < parts; ++i) st = ffn_phase(part_of(i));
  for (uint32_t i = 0; st == WB200_OK && i < parts; ++i) st = final_residual(part_of(i));
  if (st == WB200_OK && parts > 1) {
    cudaEventRecord(backend->pipeline_event[4 * parts + 1], user_stream);   // timeline end
    backend->layer_timeline_parts = parts;
  }
  if (st != WB200_OK && parts > 1) {
    // join: later work on the caller's stream must not overtake a collective that is still running on the other stream
    cudaEventRecord(backend->aux_event[0], comm_stream);
    cudaStreamWaitEvent(user_stream, backend->aux_event[0], 0);
  }
  return st;
}

wb200_status wb200_decoder_layer_timeline(wb200_backend *backend, float *ms, uint32_t capacity, uint32_t *count) {
  if (!backend || !count) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  const uint32_t parts = backend->layer_timeline_parts;
  *count = parts ? 4 * parts + 1 : 0;
  if (parts == 0 || !ms) return WB200_OK;
  if (capacity < *count) return fail(WB200_ERR_LIMIT, "timeline buffer too small");
  DeviceGuard guard(backend->device);
  cudaEvent_t origin = backend->pipeline_event[4 * parts];
  WB200_CUDA_CHECK(cudaEventSynchronize(backend->pipeline_event[4 * parts + 1]));
  for (uint32_t i = 0; i < 4 * parts; ++i) WB200_CUDA_CHECK(cudaEventElapsedTime(&ms[i], origin, backend->pipeline_event[i]));
  WB200_CUDA_CHECK(cudaEventElapsedTime(&ms[4 * parts], origin, backend->pipeline_event[4 * parts + 1]));
  return WB200_OK;
}

}  // extern "C"
