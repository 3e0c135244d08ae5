// Region-level entry points: attention (flash-attention prefill, flash-decoding) and the GEMM with a
// fused epilogue chain. With WB200_MEM_HOST the call stages through the backend's device buffers and
// synchronises; with WB200_MEM_DEVICE it only enqueues kernels on the caller's stream.
#include "backend.h"

using namespace wb200;

namespace {

size_t element_bytes_of(int format) { return format == WB200_F32 ? 4 : 2; }

wb200_status make_attention_args(const wb200_attention_params *p, AttentionArgs *a) {
  if (!is_float_format(p->format)) return fail(WB200_ERR_UNSUPPORTED, "attention storage must be f16, bf16 or f32");
  if (p->batch == 0 || p->q_heads == 0 || p->kv_heads == 0 || p->q_len == 0 || p->kv_len == 0 || p->head_dim == 0)
    return fail(WB200_ERR_INVALID_ARGUMENT, "attention extents must be positive");
  if (p->q_heads % p->kv_heads != 0) return fail(WB200_ERR_INVALID_ARGUMENT, "q_heads must be a multiple of kv_heads");
  if (p->kv_len > 0x7fffffffu || p->q_len > 0x7fffffffu) return fail(WB200_ERR_INVALID_ARGUMENT, "sequence length too large");
  if (!p->q || !p->k || !p->v) return fail(WB200_ERR_INVALID_ARGUMENT, "q, k and v must not be null");
  a->batch = p->batch; a->q_heads = p->q_heads; a->kv_heads = p->kv_heads;
  a->q_len = p->q_len; a->kv_len = p->kv_len; a->head_dim = p->head_dim;
  a->format = p->format;
  a->causal = p->causal ? 1 : 0;
  a->zero_fully_masked = p->zero_fully_masked ? 1 : 0;
  a->scale = p->scale;
  a->causal_offset = p->query_start - p->key_start;
  a->kv_valid = p->key_end > 0 ? p->key_end - p->key_start : static_cast<int64_t>(p->kv_len);
  a->q = p->q; a->k = p->k; a->v = p->v; a->out = p->out;
  a->lse = p->lse; a->row_max = p->row_max; a->row_sum = p->row_sum;
  a->out_token_major = p->out_layout == WB200_OUT_TOKEN_MAJOR ? 1 : 0;
  if (p->out_layout > WB200_OUT_TOKEN_MAJOR) return fail(WB200_ERR_INVALID_ARGUMENT, "unknown attention output layout");
  return WB200_OK;
}

struct StagedAttention {
  AttentionArgs args;
  size_t q_bytes, kv_bytes, out_bytes, stat_bytes;
  float *d_lse = nullptr, *d_max = nullptr, *d_sum = nullptr;
};

// Copies q, k, v to device staging buffers (slots 0-2), allocates out (slot 3) and statistics
// (slots 4-6). On return `staged.args` points at device memory.
wb200_status stage_attention_inputs(wb200_backend *backend, const wb200_attention_params *p, StagedAttention *s, bool need_out) {
  const size_t eb = element_bytes_of(p->format);
  s->q_bytes = static_cast<size_t>(p->batch) * p->q_heads * p->q_len * p->head_dim * eb;
  s->kv_bytes = static_cast<size_t>(p->batch) * p->kv_heads * p->kv_len * p->head_dim * eb;
  s->out_bytes = s->q_bytes;
  s->stat_bytes = static_cast<size_t>(p->batch) * p->q_heads * p->q_len * sizeof(float);
  void *dq, *dk, *dv, *dout = nullptr;
  wb200_status st;
  if ((st = backend->buffer(0, s->q_bytes, &dq)) != WB200_OK) return st;
  if ((st = backend->buffer(1, s->kv_bytes, &dk)) != WB200_OK) return st;
  if ((st = backend->buffer(2, s->kv_bytes, &dv)) != WB200_OK) return st;
  if (need_out && (st = backend->buffer(3, s->out_bytes, &dout)) != WB200_OK) return st;
  cudaStream_t stream = backend->stream;
  WB200_CUDA_CHECK(cudaMemcpyAsync(dq, p->q, s->q_bytes, cudaMemcpyHostToDevice, stream));
  WB200_CUDA_CHECK(cudaMemcpyAsync(dk, p->k, s->kv_bytes, cudaMemcpyHostToDevice, stream));
  WB200_CUDA_CHECK(cudaMemcpyAsync(dv, p->v, s->kv_bytes, cudaMemcpyHostToDevice, stream));
  s->args.q = dq; s->args.k = dk; s->args.v = dv; s->args.out = dout;
  void *tmp;
  if (p->lse) { if ((st = backend->buffer(4, s->stat_bytes, &tmp)) != WB200_OK) return st; s->d_lse = static_cast<float *>(tmp); }
  if (p->row_max) { if ((st = backend->buffer(5, s->stat_bytes, &tmp)) != WB200_OK) return st; s->d_max = static_cast<float *>(tmp); }
  if (p->row_sum) { if ((st = backend->buffer(6, s->stat_bytes, &tmp)) != WB200_OK) return st; s->d_sum = static_cast<float *>(tmp); }
  s->args.lse = s->d_lse; s->args.row_max = s->d_max; s->args.row_sum = s->d_sum;
  return WB200_OK;
}

wb200_status return_attention_outputs(wb200_backend *backend, const wb200_attention_params *p, const StagedAttention &s) {
  cudaStream_t stream = backend->stream;
  WB200_CUDA_CHECK(cudaMemcpyAsync(p->out, s.args.out, s.out_bytes, cudaMemcpyDeviceToHost, stream));
  if (p->lse) WB200_CUDA_CHECK(cudaMemcpyAsync(p->lse, s.d_lse, s.stat_bytes, cudaMemcpyDeviceToHost, stream));
  if (p->row_max) WB200_CUDA_CHECK(cudaMemcpyAsync(p->row_max, s.d_max, s.stat_bytes, cudaMemcpyDeviceToHost, stream));
  if (p->row_sum) WB200_CUDA_CHECK(cudaMemcpyAsync(p->row_sum, s.d_sum, s.stat_bytes, cudaMemcpyDeviceToHost, stream));
  return read_device_status(backend, stream, nullptr);
}

wb200_status run_fa(wb200_backend *backend, const AttentionArgs &a, cudaStream_t stream) {
  wb200_status st;
  if (attention_fa_umma_supports(a)) {
    st = launch_attention_fa_umma(a, backend->sm_count, backend->d_status, stream);
  } else {
    st = launch_attention_fa_simt(a, stream);
  }
  if (st == WB200_OK) backend->launches += 1;
  return st;
}

// Host-buffer prefill as a three-stage pipeline over chunks of (batch, kv-head) units: chunk c is copied in on one
// auxiliary stream, computed on the backend stream and copied out on the other auxiliary stream, so the copy-out of a
// chunk overlaps the copy-in of the next ones (PCIe is full duplex) and the kernels hide behind both. A unit is one
// KV head with its group of query heads; consecutive units are contiguous in Q, K, V, out and the statistics, so a
// chunk of n units is the attention problem {batch = n, q_heads = group, kv_heads = 1}.
wb200_status run_fa_host_pipelined(wb200_backend *backend, const wb200_attention_params *p, const AttentionArgs &whole) {
  const size_t eb = element_bytes_of(p->format);
  const uint32_t group = p->q_heads / p->kv_heads;
  const uint32_t units = p->batch * p->kv_heads;
  const uint32_t chunks = units < 8 ? units : 8;
  const size_t q_unit = static_cast<size_t>(group) * p->q_len * p->head_dim * eb;       // also the out bytes of a unit
  const size_t kv_unit = static_cast<size_t>(p->kv_len) * p->head_dim * eb;
  const size_t stat_unit = static_cast<size_t>(group) * p->q_len * sizeof(float);
  wb200_status st;
  void *dq, *dk, *dv, *dout, *dl = nullptr, *dm = nullptr, *ds = nullptr;
  if ((st = backend->buffer(0, q_unit * units, &dq)) != WB200_OK) return st;
  if ((st = backend->buffer(1, kv_unit * units, &dk)) != WB200_OK) return st;
  if ((st = backend->buffer(2, kv_unit * units, &dv)) != WB200_OK) return st;
  if ((st = backend->buffer(3, q_unit * units, &dout)) != WB200_OK) return st;
  if (p->lse && (st = backend->buffer(4, stat_unit * units, &dl)) != WB200_OK) return st;
  if (p->row_max && (st = backend->buffer(5, stat_unit * units, &dm)) != WB200_OK) return st;
  if (p->row_sum && (st = backend->buffer(6, stat_unit * units, &ds)) != WB200_OK) return st;
  if ((st = backend->auxiliary_streams()) != WB200_OK) return st;
  if ((st = backend->pipeline_events(2 * chunks)) != WB200_OK) return st;
  cudaStream_t copy_in = backend->aux_stream[0], compute = backend->stream, copy_out = backend->aux_stream[1];
  // the auxiliary streams start after whatever the backend stream still has in flight (it owns the staging buffers)
  WB200_CUDA_CHECK(cudaEventRecord(backend->aux_event[0], compute));
  WB200_CUDA_CHECK(cudaStreamWaitEvent(copy_in, backend->aux_event[0], 0));
  WB200_CUDA_CHECK(cudaStreamWaitEvent(copy_out, backend->aux_event[0], 0));
  auto at = [](const void *base, size_t offset) { return static_cast<const uint8_t *>(base) + offset; };
  auto at_mut = [](void *base, size_t offset) { return static_cast<uint8_t *>(base) + offset; };
  // The pipeline proper; any failure inside leaves copies in flight that write the caller's buffers, so whatever it
  // returns, the three streams are drained before this call does.
  auto enqueue = [&]() -> wb200_status {
  uint32_t first = 0;
  for (uint32_t c = 0; c < chunks; ++c) {
    const uint32_t count = units / chunks + (c < units % chunks ? 1 : 0);
    const size_t q_at = first * q_unit, kv_at = first * kv_unit, stat_at = first * stat_unit;
    WB200_CUDA_CHECK(cudaMemcpyAsync(at_mut(dq, q_at), at(p->q, q_at), count * q_unit, cudaMemcpyHostToDevice, copy_in));
    WB200_CUDA_CHECK(cudaMemcpyAsync(at_mut(dk, kv_at), at(p->k, kv_at), count * kv_unit, cudaMemcpyHostToDevice, copy_in));
    WB200_CUDA_CHECK(cudaMemcpyAsync(at_mut(dv, kv_at), at(p->v, kv_at), count * kv_unit, cudaMemcpyHostToDevice, copy_in));
    WB200_CUDA_CHECK(cudaEventRecord(backend->pipeline_event[2 * c], copy_in));
    WB200_CUDA_CHECK(cudaStreamWaitEvent(compute, backend->pipeline_event[2 * c], 0));
    AttentionArgs a = whole;
    a.batch = static_cast<int>(count); a.q_heads = static_cast<int>(group); a.kv_heads = 1;
    a.q = at_mut(dq, q_at); a.k = at_mut(dk, kv_at); a.v = at_mut(dv, kv_at); a.out = at_mut(dout, q_at);
    a.lse = dl ? reinterpret_cast<float *>(at_mut(dl, stat_at)) : nullptr;
    a.row_max = dm ? reinterpret_cast<float *>(at_mut(dm, stat_at)) : nullptr;
    a.row_sum = ds ? reinterpret_cast<float *>(at_mut(ds, stat_at)) : nullptr;
    if ((st = run_fa(backend, a, compute)) != WB200_OK) return st;
    WB200_CUDA_CHECK(cudaEventRecord(backend->pipeline_event[2 * c + 1], compute));
    WB200_CUDA_CHECK(cudaStreamWaitEvent(copy_out, backend->pipeline_event[2 * c + 1], 0));
    WB200_CUDA_CHECK(cudaMemcpyAsync(at_mut(p->out, q_at), at(dout, q_at), count * q_unit, cudaMemcpyDeviceToHost, copy_out));
    if (p->lse) WB200_CUDA_CHECK(cudaMemcpyAsync(at_mut(p->lse, stat_at), at(dl, stat_at), count * stat_unit, cudaMemcpyDeviceToHost, copy_out));
    if (p->row_max) WB200_CUDA_CHECK(cudaMemcpyAsync(at_mut(p->row_max, stat_at), at(dm, stat_at), count * stat_unit, cudaMemcpyDeviceToHost, copy_out));
    if (p->row_sum) WB200_CUDA_CHECK(cudaMemcpyAsync(at_mut(p->row_sum, stat_at), at(ds, stat_at), count * stat_unit, cudaMemcpyDeviceToHost, copy_out));
    first += count;
  }
  return WB200_OK;
  };
  st = enqueue();
  const cudaError_t drained_in = cudaStreamSynchronize(copy_in), drained_out = cudaStreamSynchronize(copy_out);
  const cudaError_t drained_compute = st != WB200_OK ? cudaStreamSynchronize(compute) : cudaSuccess;
  if (st != WB200_OK) return st;
  WB200_CUDA_CHECK(drained_in);
  WB200_CUDA_CHECK(drained_out);
  WB200_CUDA_CHECK(drained_compute);
  return read_device_status(backend, compute, nullptr);
}

}  // namespace

extern "C" {

wb200_status wb200_attention_fa(wb200_backend *backend, const wb200_attention_params *p) {
  if (!backend || !p) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  if (!p->out) return fail(WB200_ERR_INVALID_ARGUMENT, "out must not be null");
  AttentionArgs a;
  wb200_status st = make_attention_args(p, &a);
  if (st != WB200_OK) return st;
  DeviceGuard guard(backend->device);
  if (p->memory == WB200_MEM_DEVICE) return run_fa(backend, a, static_cast<cudaStream_t>(p->stream));
  if (p->batch * p->kv_heads >= 2 && !a.out_token_major) return run_fa_host_pipelined(backend, p, a);
  StagedAttention s;
  s.args = a;
  if ((st = stage_attention_inputs(backend, p, &s, true)) != WB200_OK) return st;
  if ((st = run_fa(backend, s.args, backend->stream)) != WB200_OK) return st;
  return return_attention_outputs(backend, p, s);
}

wb200_status wb200_attention_fd(wb200_backend *backend, const wb200_attention_params *p, uint32_t kv_splits) {
  if (!backend || !p) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  if (!p->out) return fail(WB200_ERR_INVALID_ARGUMENT, "out must not be null");
  if (p->q_len != 1) return fail(WB200_ERR_INVALID_ARGUMENT, "flash-decoding takes query length 1");
  AttentionArgs a;
  wb200_status st = make_attention_args(p, &a);
  if (st != WB200_OK) return st;
  if (!attention_fd_supports(a) && p->memory == WB200_MEM_DEVICE)
    return fail(WB200_ERR_UNSUPPORTED, "flash-decoding kernel takes f16/bf16 storage, head_dim 128, group size <= 16");
  DeviceGuard guard(backend->device);
  const uint32_t splits = kv_splits ? kv_splits : fd_choose_splits(a, backend->sm_count);
  void *partials;
  if ((st = backend->buffer(7, fd_partial_floats(a, splits) * sizeof(float), &partials)) != WB200_OK) return st;
  if (p->memory == WB200_MEM_DEVICE) {
    st = launch_attention_fd(a, splits, static_cast<float *>(partials), 1, nullptr, static_cast<cudaStream_t>(p->stream));
    if (st == WB200_OK) backend->launches += 2;
    return st;
  }
  StagedAttention s;
  s.args = a;
  if ((st = stage_attention_inputs(backend, p, &s, true)) != WB200_OK) return st;
  if (!attention_fd_supports(s.args))
    return fail(WB200_ERR_UNSUPPORTED, "flash-decoding kernel takes f16/bf16 storage, head_dim 128, group size <= 16");
  if ((st = launch_attention_fd(s.args, splits, static_cast<float *>(partials), 1, nullptr, backend->stream)) != WB200_OK) return st;
  backend->launches += 2;
  return return_attention_outputs(backend, p, s);
}

wb200_status wb200_attention_fd_partial(wb200_backend *backend, const wb200_attention_params *p, uint32_t kv_splits, float *state_out) {
  if (!backend || !p || !state_out) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  if (p->q_len != 1) return fail(WB200_ERR_INVALID_ARGUMENT, "flash-decoding takes query length 1");
  AttentionArgs a;
  wb200_status st = make_attention_args(p, &a);
  if (st != WB200_OK) return st;
  DeviceGuard guard(backend->device);
  const uint32_t splits = kv_splits ? kv_splits : fd_choose_splits(a, backend->sm_count);
  void *partials;
  if ((st = backend->buffer(7, fd_partial_floats(a, splits) * sizeof(float), &partials)) != WB200_OK) return st;
  const size_t state_bytes = static_cast<size_t>(p->batch) * p->q_heads * (p->head_dim + 2) * sizeof(float);
  if (p->memory == WB200_MEM_DEVICE) {
    st = launch_attention_fd(a, splits, static_cast<float *>(partials), 0, state_out, static_cast<cudaStream_t>(p->stream));
    if (st == WB200_OK) backend->launches += 2;
    return st;
  }
  StagedAttention s;
  s.args = a;
  wb200_attention_params inputs_only = *p;
  inputs_only.lse = inputs_only.row_max = inputs_only.row_sum = nullptr;
  if ((st = stage_attention_inputs(backend, &inputs_only, &s, false)) != WB200_OK) return st;
  void *d_state;
  if ((st = backend->buffer(8, state_bytes, &d_state)) != WB200_OK) return st;
  if ((st = launch_attention_fd(s.args, splits, static_cast<float *>(partials), 0, static_cast<float *>(d_state), backend->stream)) != WB200_OK) return st;
  backend->launches += 2;
  WB200_CUDA_CHECK(cudaMemcpyAsync(state_out, d_state, state_bytes, cudaMemcpyDeviceToHost, backend->stream));
  return read_device_status(backend, backend->stream, nullptr);
}

uint64_t wb200_fd_exchange_bytes(uint32_t batch, uint32_t q_heads, uint32_t world) {
  return fd_exchange_floats(static_cast<int>(batch * q_heads), static_cast<int>(world)) * sizeof(float);
}

wb200_status wb200_attention_fd_exchange(wb200_backend *backend, const wb200_attention_params *p, uint32_t kv_splits,
                                         const wb200_fd_exchange *x) {
  if (!backend || !p || !x || !p->out || !x->epoch) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  if (p->q_len != 1) return fail(WB200_ERR_INVALID_ARGUMENT, "flash-decoding takes query length 1");
  if (p->memory != WB200_MEM_DEVICE) return fail(WB200_ERR_UNSUPPORTED, "the in-kernel exchange takes device buffers only");
  if (x->world < 1 || x->world > WB200_MAX_EXCHANGE_RANKS || x->rank >= x->world)
    return fail(WB200_ERR_INVALID_ARGUMENT, "exchange takes 1 to 16 ranks and a rank inside the world");
  for (uint32_t r = 0; r < x->world; ++r)
    if (!x->peer_buffers[r] || (reinterpret_cast<uintptr_t>(x->peer_buffers[r]) & 15u))
      return fail(WB200_ERR_INVALID_ARGUMENT, "every rank's exchange buffer must be given, 16-byte aligned");
  AttentionArgs a;
  wb200_status st = make_attention_args(p, &a);
  if (st != WB200_OK) return st;
  DeviceGuard guard(backend->device);
  const uint32_t splits = kv_splits ? kv_splits : fd_choose_splits(a, backend->sm_count);
  void *partials;
  if ((st = backend->buffer(7, fd_partial_floats(a, splits) * sizeof(float), &partials)) != WB200_OK) return st;
  // One launch: the last stage-1 CTA of every (batch, kv head) folds, exchanges and merges. WB200_FD_EXCHANGE_FUSED=0 in
  // the environment keeps the tail as a second launch.
  static const bool fused = []() { const char *env = getenv("WB200_FD_EXCHANGE_FUSED"); return !(env && env[0] == '0'); }();
  void *arrivals = nullptr;
  if (fused && (st = backend->zeroed_buffer(11, static_cast<size_t>(a.batch) * a.kv_heads * sizeof(unsigned int), &arrivals)) != WB200_OK) return st;
  st = launch_attention_fd_exchange(a, splits, static_cast<float *>(partials), static_cast<int>(x->rank), static_cast<int>(x->world),
                                    x->peer_buffers, x->epoch, static_cast<unsigned int *>(arrivals), backend->d_status,
                                    static_cast<cudaStream_t>(p->stream));
  if (st == WB200_OK) backend->launches += fused ? 1 : 2;
  return st;
}

wb200_status wb200_attention_fd_merge(wb200_backend *backend, const wb200_attention_params *p, const float *states, uint32_t shard_count) {
  if (!backend || !p || !states || !p->out) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  if (p->q_len != 1) return fail(WB200_ERR_INVALID_ARGUMENT, "flash-decoding takes query length 1");
  if (!is_float_format(p->format)) return fail(WB200_ERR_UNSUPPORTED, "attention storage must be f16, bf16 or f32");
  AttentionArgs a{};
  a.batch = p->batch; a.q_heads = p->q_heads; a.kv_heads = p->kv_heads; a.q_len = 1; a.kv_len = p->kv_len; a.head_dim = p->head_dim;
  a.format = p->format; a.zero_fully_masked = p->zero_fully_masked ? 1 : 0;
  a.out = p->out; a.lse = p->lse; a.row_max = p->row_max; a.row_sum = p->row_sum;
  DeviceGuard guard(backend->device);
  if (p->memory == WB200_MEM_DEVICE) {
    wb200_status st = launch_attention_fd_merge(a, states, shard_count, static_cast<cudaStream_t>(p->stream));
    if (st == WB200_OK) backend->launches += 1;
    return st;
  }
  const size_t rows = static_cast<size_t>(p->batch) * p->q_heads;
  const size_t state_bytes = rows * (p->head_dim + 2) * sizeof(float) * shard_count;
  const size_t out_bytes = rows * p->head_dim * element_bytes_of(p->format);
  const size_t stat_bytes = rows * sizeof(float);
  void *d_states, *d_out, *tmp;
  wb200_status st;
  if ((st = backend->buffer(8, state_bytes, &d_states)) != WB200_OK) return st;
  if ((st = backend->buffer(3, out_bytes, &d_out)) != WB200_OK) return st;
  StagedAttention s;
  s.out_bytes = out_bytes; s.stat_bytes = stat_bytes;
  if (p->lse) { if ((st = backend->buffer(4, stat_bytes, &tmp)) != WB200_OK) return st; s.d_lse = static_cast<float *>(tmp); }
  if (p->row_max) { if ((st = backend->buffer(5, stat_bytes, &tmp)) != WB200_OK) return st; s.d_max = static_cast<float *>(tmp); }
  if (p->row_sum) { if ((st = backend->buffer(6, stat_bytes, &tmp)) != WB200_OK) return st; s.d_sum = static_cast<float *>(tmp); }
  a.out = d_out; a.lse = s.d_lse; a.row_max = s.d_max; a.row_sum = s.d_sum;
  s.args = a;
  WB200_CUDA_CHECK(cudaMemcpyAsync(d_states, states, state_bytes, cudaMemcpyHostToDevice, backend->stream));
  if ((st = launch_attention_fd_merge(a, static_cast<const float *>(d_states), shard_count, backend->stream)) != WB200_OK) return st;
  backend->launches += 1;
  return return_attention_outputs(backend, p, s);
}

wb200_status wb200_gemm_epilogue(wb200_backend *backend, const wb200_gemm_epilogue_params *p) {
  if (!backend || !p) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  if (!p->a || !p->b || !p->out) return fail(WB200_ERR_INVALID_ARGUMENT, "a, b and out must not be null");
  if (p->epilogue > WB200_EPI_SWIGLU) return fail(WB200_ERR_INVALID_ARGUMENT, "unknown epilogue");
  if ((p->epilogue == WB200_EPI_BIAS || p->epilogue == WB200_EPI_BIAS_GELU) && !p->bias) return fail(WB200_ERR_INVALID_ARGUMENT, "bias must not be null for this epilogue");
  GemmUmmaArgs g{};
  g.m = p->m; g.n = p->n; g.k = p->k;
  g.in_format = p->in_format; g.out_format = p->out_format;
  g.lhs_transposed = p->lhs_orientation == WB200_TRANSPOSE; g.rhs_transposed = p->rhs_orientation == WB200_TRANSPOSE;
  g.epilogue = p->epilogue;
  g.a = p->a; g.b = p->b; g.bias = p->bias; g.out = p->out;
  DeviceGuard guard(backend->device);
  wb200_status st;
  if (p->memory == WB200_MEM_DEVICE) {
    st = launch_gemm_umma(g, backend->sm_count, backend->d_status, static_cast<cudaStream_t>(p->stream));
    if (st == WB200_OK) backend->launches += 1;
    return st;
  }
  const size_t a_bytes = static_cast<size_t>(p->m) * p->k * 2, b_bytes = static_cast<size_t>(p->k) * p->n * 2;
  const size_t out_cols = p->epilogue == WB200_EPI_SWIGLU ? p->n / 2 : p->n;
  const size_t out_bytes = static_cast<size_t>(p->m) * out_cols * element_bytes_of(p->out_format);
  void *da, *db, *dout, *dbias = nullptr;
  if ((st = backend->buffer(0, a_bytes, &da)) != WB200_OK) return st;
  if ((st = backend->buffer(1, b_bytes, &db)) != WB200_OK) return st;
  if ((st = backend->buffer(2, out_bytes, &dout)) != WB200_OK) return st;
  cudaStream_t stream = backend->stream;
  WB200_CUDA_CHECK(cudaMemcpyAsync(da, p->a, a_bytes, cudaMemcpyHostToDevice, stream));
  WB200_CUDA_CHECK(cudaMemcpyAsync(db, p->b, b_bytes, cudaMemcpyHostToDevice, stream));
  if (p->bias) {
    if ((st = backend->buffer(3, static_cast<size_t>(p->n) * sizeof(float), &dbias)) != WB200_OK) return st;
    WB200_CUDA_CHECK(cudaMemcpyAsync(dbias, p->bias, static_cast<size_t>(p->n) * sizeof(float), cudaMemcpyHostToDevice, stream));
  }
  g.a = da; g.b = db; g.out = dout; g.bias = static_cast<const float *>(dbias);
  if ((st = launch_gemm_umma(g, backend->sm_count, backend->d_status, stream)) != WB200_OK) return st;
  backend->launches += 1;
  WB200_CUDA_CHECK(cudaMemcpyAsync(p->out, dout, out_bytes, cudaMemcpyDeviceToHost, stream));
  return read_device_status(backend, stream, nullptr);
}

}  // extern "C"

// ------------------------------------------------------------------ decoder-layer pieces (device buffers)
extern "C" {

wb200_status wb200_rmsnorm(wb200_backend *backend, uint32_t format, const void *x, const void *gamma, void *y,
                           uint32_t rows, uint32_t dim, float eps, void *stream) {
  if (!backend || !x || !gamma || !y) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard guard(backend->device);
  wb200_status st = launch_rmsnorm(format, x, gamma, y, rows, dim, eps, static_cast<cudaStream_t>(stream));
  if (st == WB200_OK) backend->launches += 1;
  return st;
}

wb200_status wb200_rope_split(wb200_backend *backend, uint32_t format, const void *qkv, void *q, void *k, void *v,
                              uint32_t batch, uint32_t seq, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                              float theta, uint32_t position_offset, void *stream) {
  if (!backend || !qkv || !q || !k || !v) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard guard(backend->device);
  wb200_status st = launch_rope_split(format, qkv, q, k, v, batch, seq, q_heads, kv_heads, head_dim, theta,
                                      position_offset, static_cast<cudaStream_t>(stream));
  if (st == WB200_OK) backend->launches += 1;
  return st;
}

wb200_status wb200_residual_add(wb200_backend *backend, uint32_t format, const void *a, const void *b, void *out,
                                uint64_t elements, void *stream) {
  if (!backend || !a || !b || !out) return fail(WB200_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard guard(backend->device);
  wb200_status st = launch_residual_add(format, a, b, out, elements, static_cast<cudaStream_t>(stream));
  if (st == WB200_OK) backend->launches += 1;
  return st;
}

}  // extern "C"
