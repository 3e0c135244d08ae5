"""Llama-style decoder layer: a plain f32 restatement is checked against the committed Hugging Face output
(CPU), and the B200 layer - single shard and a two-way head / FFN sharding whose partial sums are added by the
test - against both (GPU). Bound: bf16 storage, max |a - e| / max |e| <= 1e-2 and the reference's similarity gate."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import helpers
from vibe_compiler_b200.decoder_layer import LayerConfig, random_weights

ROOT = Path(__file__).resolve().parent.parent
_spec = importlib.util.spec_from_file_location("make_llama_layer_fixture", ROOT / "tests" / "golden" / "make_llama_layer_fixture.py")
fixture = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(fixture)


def reference_layer(cfg: LayerConfig, w, x):
    """f32 restatement: RMSNorm, QKV, rotary (pairs (i, i + D/2)), causal GQA softmax attention, output projection,
    residual, RMSNorm, SwiGLU FFN, residual."""
    b, s, d = x.shape
    hd = cfg.head_dim

    def rms(t, g):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + cfg.eps) * g.float()
    x = x.float()
    h = rms(x, w.norm1)
    q = (h @ w.wq.float()).view(b, s, cfg.q_heads, hd).transpose(1, 2)
    k = (h @ w.wk.float()).view(b, s, cfg.kv_heads, hd).transpose(1, 2)
    v = (h @ w.wv.float()).view(b, s, cfg.kv_heads, hd).transpose(1, 2)
    inv_freq = cfg.rope_theta ** (-torch.arange(0, hd, 2).float() / hd)
    angle = torch.arange(s).float()[:, None] * inv_freq[None, :]
    cos, sin = torch.cat([angle.cos(), angle.cos()], -1), torch.cat([angle.sin(), angle.sin()], -1)

    def rope(t):
        rotated = torch.cat([-t[..., hd // 2:], t[..., :hd // 2]], -1)
        return t * cos + rotated * sin
    q, k = rope(q), rope(k)
    g = cfg.q_heads // cfg.kv_heads
    scores = q @ k.repeat_interleave(g, 1).transpose(-1, -2) * hd ** -0.5
    scores = scores.masked_fill(torch.ones(s, s, dtype=torch.bool).triu(1), float("-inf"))
    attn = (torch.softmax(scores, -1) @ v.repeat_interleave(g, 1)).transpose(1, 2).reshape(b, s, cfg.q_heads * hd)
    x1 = x + attn @ w.wo.float()
    h2 = rms(x1, w.norm2)
    act = torch.nn.functional.silu(h2 @ w.wgate.float()) * (h2 @ w.wup.float())
    return x1 + act @ w.wdown.float()


def test_f32_restatement_matches_hugging_face_layer():
    cfg = fixture.CFG
    expected = np.load(ROOT / "tests" / "golden" / "llama_layer_expected.npz")["expected"]
    got = reference_layer(cfg, random_weights(cfg), fixture.layer_input()).numpy()
    assert helpers.max_rel_err(got.astype(np.float64), expected.astype(np.float64)) <= 1e-5


def test_sampled_row_recomputation_matches_the_f32_restatement():
    # The float64 sampled-row checker used on full-size outputs, against the whole-layer restatement above.
    from vibe_compiler_b200 import selfcheck
    cfg = fixture.CFG
    w, x = random_weights(cfg), fixture.layer_input()
    want = reference_layer(cfg, w, x)
    rows = [0, 1, 77, x.shape[1] - 1]
    got = selfcheck.layer_rows_f64(cfg, w, x, 1, rows, torch.device("cpu"))
    assert selfcheck.max_rel_err(got, want[1, rows]) <= 1e-5


def _gate(oracle, got: torch.Tensor, expected: np.ndarray):
    want_bits = helpers.bits(torch.from_numpy(expected).bfloat16())
    err = helpers.max_rel_err(got.double().cpu().numpy(), expected.astype(np.float64))
    assert err <= 1e-2, err
    helpers.reference_gate(oracle, "bf16", helpers.bits(got), want_bits)


@pytest.mark.gpu
def test_layer_single_shard_matches_hugging_face(backend, oracle):
    from vibe_compiler_b200.decoder_layer import ShardedDecoderLayer
    cfg = fixture.CFG
    layer = ShardedDecoderLayer(backend, cfg, random_weights(cfg))
    out = layer.forward(fixture.layer_input().cuda())
    torch.cuda.synchronize()
    backend.poll()
    _gate(oracle, out, np.load(ROOT / "tests" / "golden" / "llama_layer_expected.npz")["expected"])


@pytest.mark.gpu
def test_layer_two_way_sharding_sums_to_the_same_output(backend, oracle):
    # Both shards run on this GPU one after the other; the test adds their partial outputs where the all-reduce
    # would (the NCCL path itself is exercised by `bench.py --workload layer` on two or more GPUs).
    from vibe_compiler_b200.decoder_layer import ShardedDecoderLayer
    cfg = fixture.CFG
    weights = random_weights(cfg)
    shards = [ShardedDecoderLayer(backend, cfg, weights, rank=r, world_size=2) for r in range(2)]
    x = fixture.layer_input().cuda()
    b, s, d = x.shape
    tokens = x.reshape(b * s, d)
    partial = sum(shard.attention_partial(tokens, b, s).float() for shard in shards).bfloat16()
    x1 = backend.residual_add(tokens, partial)
    partial2 = sum(shard.ffn_partial(x1).float() for shard in shards).bfloat16()
    out = backend.residual_add(x1, partial2).reshape(b, s, d)
    torch.cuda.synchronize()
    backend.poll()
    _gate(oracle, out, np.load(ROOT / "tests" / "golden" / "llama_layer_expected.npz")["expected"])


@pytest.mark.gpu
def test_layer_pieces_against_f32(backend):
    g = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn(300, 1024, generator=g).bfloat16()
    gamma = (1 + 0.1 * torch.randn(1024, generator=g)).bfloat16()
    y = backend.rmsnorm(x.cuda(), gamma.cuda(), 1e-5).cpu()
    xf = x.float()
    want = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).bfloat16().float() * gamma.float()
    assert torch.equal(y, want.bfloat16())          # same two roundings: bit-exact unless rsqrt differs in the last ulp
    a, b2 = torch.randn(4096, generator=g).bfloat16(), torch.randn(4096, generator=g).bfloat16()
    assert torch.equal(backend.residual_add(a.cuda(), b2.cuda()).cpu(), (a.float() + b2.float()).bfloat16())
    # rotary + relayout
    batch, seq, hq, hkv, hd = 2, 37, 4, 2, 128
    qkv = torch.randn(batch * seq, (hq + 2 * hkv) * hd, generator=g).bfloat16()
    q, k, v = (t.cpu() for t in backend.rope_split(qkv.cuda(), batch, seq, hq, hkv, hd, 10000.0))
    rows = qkv.float().view(batch, seq, hq + 2 * hkv, hd).transpose(1, 2)
    inv_freq = 10000.0 ** (-torch.arange(0, hd, 2).float() / hd)
    angle = torch.arange(seq).float()[:, None] * inv_freq[None, :]
    cos, sin = torch.cat([angle.cos(), angle.cos()], -1), torch.cat([angle.sin(), angle.sin()], -1)
    rotated = rows * cos + torch.cat([-rows[..., hd // 2:], rows[..., :hd // 2]], -1) * sin
    assert (q.float() - rotated[:, :hq]).abs().max() <= 2 ** -6 and (k.float() - rotated[:, hq:hq + hkv]).abs().max() <= 2 ** -6
    assert torch.equal(v, rows[:, hq + hkv:].bfloat16())
    # SwiGLU epilogue
    from vibe_compiler_b200 import _abi as abi
    a2 = (torch.rand(256, 192, generator=g) * 2 - 1).bfloat16()
    w = (torch.rand(192, 128, generator=g) * 2 - 1).bfloat16()
    act = backend.gemm_epilogue(a2.cuda(), w.cuda(), epilogue=abi.EPI_SWIGLU).cpu()
    prod = a2.double() @ w.double()
    want_act = torch.nn.functional.silu(prod[:, 0::2]) * prod[:, 1::2]
    assert ((act.double() - want_act).abs().max() / want_act.abs().max()).item() <= 1e-2


@pytest.mark.gpu
def test_single_call_layer_equals_the_composed_calls(backend):
    from vibe_compiler_b200.decoder_layer import ShardedDecoderLayer
    cfg = fixture.CFG
    weights = random_weights(cfg)
    x = fixture.layer_input().cuda()
    layer = ShardedDecoderLayer(backend, cfg, weights)
    assert torch.equal(layer.forward_fused(x), layer.forward(x))
    assert torch.equal(layer.forward_fused(x), layer.forward(x))      # workspace reuse

    # two shards: the callback of shard 0 adds what shard 1 computed with the composed calls
    shards = [ShardedDecoderLayer(backend, cfg, weights, rank=r, world_size=2) for r in range(2)]
    b, s, d = x.shape
    tokens = x.reshape(b * s, d)
    partials = [shard.attention_partial(tokens, b, s) for shard in shards]
    x1 = backend.residual_add(tokens, (partials[0].float() + partials[1].float()).bfloat16())
    ffn = [shard.ffn_partial(x1) for shard in shards]
    want = backend.residual_add(x1, (ffn[0].float() + ffn[1].float()).bfloat16()).reshape(b, s, d)
    others = iter([partials[1], ffn[1]])
    calls = []

    def fake_all_reduce(t):
        calls.append(t.numel())
        other = next(others)
        t.copy_((t.view_as(other).float() + other.float()).bfloat16().view_as(t))
    s0 = shards[0]
    got, _ = backend.decoder_layer(x, norm1=s0.norm1, wqkv=s0.wqkv, wo=s0.wo, norm2=s0.norm2, wgu=s0.wgu, wdown=s0.wdown, q_heads=s0.hq,
                                   kv_heads=s0.hkv, head_dim=cfg.head_dim, eps=cfg.eps, rope_theta=cfg.rope_theta, allreduce=fake_all_reduce)
    torch.cuda.synchronize()
    backend.poll()
    assert calls == [b * s * d, b * s * d]
    assert torch.equal(got, want)


@pytest.mark.gpu
def test_single_call_layer_reports_callback_failure_and_small_workspace(backend):
    from vibe_compiler_b200.backend import WB200Error
    from vibe_compiler_b200.decoder_layer import ShardedDecoderLayer
    cfg = fixture.CFG
    layer = ShardedDecoderLayer(backend, cfg, random_weights(cfg))
    x = fixture.layer_input().cuda()
    kwargs = dict(norm1=layer.norm1, wqkv=layer.wqkv, wo=layer.wo, norm2=layer.norm2, wgu=layer.wgu, wdown=layer.wdown, q_heads=layer.hq,
                  kv_heads=layer.hkv, head_dim=cfg.head_dim, eps=cfg.eps, rope_theta=cfg.rope_theta)

    def broken(_tensor):
        raise RuntimeError("link down")
    with pytest.raises(RuntimeError, match="link down"):
        backend.decoder_layer(x, allreduce=broken, **kwargs)
    torch.cuda.synchronize()
    backend.poll()
    with pytest.raises(WB200Error):
        backend.decoder_layer(x[:, :3], **kwargs)          # 6 tokens: not a multiple of 8
    out, _ = backend.decoder_layer(x, **kwargs)              # the backend is still usable
    assert torch.isfinite(out.float()).all()


@pytest.mark.gpu
def test_micro_batched_layer_equals_one_pass(backend):
    # With micro_batches = 2 the two sequences flow through the layer one after the other and their sums are enqueued on
    # the backend's communication stream (the callback is entered with it current); with SMs reserved for the collective
    # the persistent kernels run on fewer CTAs. The arithmetic per token is unchanged, so the bits must be.
    from vibe_compiler_b200.decoder_layer import ShardedDecoderLayer
    cfg = fixture.CFG
    layer = ShardedDecoderLayer(backend, cfg, random_weights(cfg))
    x = fixture.layer_input().cuda()
    kwargs = dict(norm1=layer.norm1, wqkv=layer.wqkv, wo=layer.wo, norm2=layer.norm2, wgu=layer.wgu, wdown=layer.wdown, q_heads=layer.hq,
                  kv_heads=layer.hkv, head_dim=cfg.head_dim, eps=cfg.eps, rope_theta=cfg.rope_theta)
    seen = []

    def identity(tensor):
        seen.append((torch.cuda.current_stream().cuda_stream, tensor.numel()))
    one, _ = backend.decoder_layer(x, allreduce=identity, micro_batches=1, **kwargs)
    two, _ = backend.decoder_layer(x, allreduce=identity, micro_batches=2, **kwargs)
    reserved, _ = backend.decoder_layer(x, allreduce=identity, micro_batches=2, reserved_sms=16, **kwargs)
    torch.cuda.synchronize()
    backend.poll()
    assert torch.equal(one, two) and torch.equal(one, reserved)
    tokens = x.shape[0] * x.shape[1] * x.shape[2]
    assert [n for _, n in seen] == [tokens, tokens] + [tokens // 2] * 8
    main = seen[0][0]
    assert seen[1][0] == main                            # one pass: sums on the caller's stream
    part_streams = [s for s, _ in seen[2:]]
    assert all(s != main for s in part_streams) and len(set(part_streams)) == 1   # one communication stream


@pytest.mark.gpu
def test_full_size_layer_properties(backend):
    """The benchmark's shape (d_model 4096, 32 / 8 heads, FFN 14336, batch 8 x seq 2048) on one GPU: sampled token rows
    against a float64 recomputation from the same bf16 weights and inputs, bound 1e-2 (16-bit storage path)."""
    from vibe_compiler_b200 import selfcheck
    from vibe_compiler_b200.decoder_layer import ShardedDecoderLayer
    cfg = LayerConfig()
    weights = random_weights(cfg)
    g = torch.Generator(device="cpu").manual_seed(20260808)
    x = torch.randn(8, 2048, cfg.d_model, generator=g).bfloat16()
    layer = ShardedDecoderLayer(backend, cfg, weights)
    out = layer.forward_fused(x.cuda())
    torch.cuda.synchronize()
    backend.poll()
    assert torch.isfinite(out.float()).all()
    device = torch.device("cuda", backend.device)
    for batch_index, rows in ((0, [0, 1, 127, 128, 1000, 2047]), (5, [255, 256, 1531, 2046])):
        want = selfcheck.layer_rows_f64(cfg, weights, x, batch_index, rows, device)
        err = selfcheck.max_rel_err(out[batch_index, rows], want)
        assert err <= 1e-2, (batch_index, err)
