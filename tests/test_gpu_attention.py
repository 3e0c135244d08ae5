"""Attention parity on the GPU through the C ABI: flash-attention prefill (tcgen05 kernel for bf16/f16,
CUDA-core kernel for f32) and flash-decoding against the CPU oracle, the committed PyTorch golden
outputs and, at full benchmark sizes, size-independent properties.
Bounds: bf16/f16 storage max rel err <= 1e-2; f32 <= 1e-5 (the bounds the path's specification states)."""
import os

import numpy as np
import pytest
import torch

from tests import helpers
from tests.helpers import fixtures

pytestmark = pytest.mark.gpu
BOUND = {"bf16": 1e-2, "f16": 1e-2, "f32": 1e-5}


def make_qkv(b, hq, hkv, sq, skv, d, dtype, seed=20260803):
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(b, hq, sq, d, generator=g).to(dtype)
    k = torch.randn(b, hkv, skv, d, generator=g).to(dtype)
    v = torch.randn(b, hkv, skv, d, generator=g).to(dtype)
    return q, k, v


def check_against_oracle(oracle, fmt, got_out, got_lse, want, lse_atol=2e-4):
    err = helpers.max_rel_err(helpers.values(helpers.bits(got_out), fmt), helpers.values(want["out"], fmt))
    assert err <= BOUND[fmt], err
    finite = np.isfinite(want["lse"])
    assert np.allclose(got_lse.cpu().numpy()[finite], want["lse"][finite], rtol=0, atol=lse_atol)
    assert np.array_equal(np.isneginf(got_lse.cpu().numpy()), np.isneginf(want["lse"]))


@pytest.mark.parametrize("shape", [
    # batch, q_heads, kv_heads, q_len, kv_len, causal
    (1, 2, 2, 256, 256, False), (1, 2, 2, 256, 256, True), (2, 4, 2, 300, 300, True), (1, 4, 1, 128, 1000, True),
    (1, 2, 2, 1, 129, False), (1, 1, 1, 513, 77, False), (1, 2, 1, 384, 640, True)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fa_tensor_core_kernel(backend, oracle, shape, dtype):
    b, hq, hkv, sq, skv, causal = shape
    fmt = helpers.FMT_OF[dtype]
    q, k, v = make_qkv(b, hq, hkv, sq, skv, 128, dtype)
    scale = 128 ** -0.5
    lse = torch.empty(b, hq, sq)
    out = backend.attention_fa(q, k, v, scale, causal, lse=lse, query_start=skv - sq if causal else 0)  # host buffers
    want = oracle.attention(fmt, helpers.bits(q), helpers.bits(k), helpers.bits(v), scale, causal, tile_n=128, threads=8,
                            query_start=skv - sq if causal else 0)
    check_against_oracle(oracle, fmt, out, lse, want)
    helpers.reference_gate(oracle, fmt, helpers.bits(out), want["out"])


@pytest.mark.parametrize("shape", [
    # more (batch, head, 256-row) items than SMs: every CTA of the persistent grid walks several items, with ragged
    # last tiles, GQA, causal offsets and items whose second Q tile is empty
    (3, 20, 5, 640, 640, True), (2, 40, 40, 600, 900, True), (5, 16, 4, 520, 300, False), (2, 96, 8, 300, 300, True)])
def test_fa_persistent_grid_walks_many_items(backend, oracle, shape):
    b, hq, hkv, sq, skv, causal = shape
    q, k, v = make_qkv(b, hq, hkv, sq, skv, 128, torch.bfloat16, seed=7)
    scale = 128 ** -0.5
    lse = torch.empty(b, hq, sq)
    start = skv - sq if causal else 0
    out = backend.attention_fa(q, k, v, scale, causal, lse=lse, query_start=start)
    want = oracle.attention("bf16", helpers.bits(q), helpers.bits(k), helpers.bits(v), scale, causal, tile_n=128, threads=16, query_start=start)
    check_against_oracle(oracle, "bf16", out, lse, want)


def test_fa_persistent_and_plain_grid_agree(backend):
    # More 256-row items than SMs: a persistent grid walks a plan. The same heads in slices of at most 148 items run one CTA
    # per item. The arithmetic per item is the same, so the bits must agree, and a second launch must repeat them.
    q, k, v = make_qkv(2, 48, 8, 1100, 1100, 128, torch.bfloat16)
    q, k, v = q.cuda(), k.cuda(), v.cuda()
    scale = 128 ** -0.5
    lse = torch.empty(2, 48, 1100, device="cuda")
    out = backend.attention_fa(q, k, v, scale, True, lse=lse)
    again = backend.attention_fa(q, k, v, scale, True)
    assert torch.equal(out.view(torch.int16), again.view(torch.int16))
    for b in range(2):
        for h0 in range(0, 48, 24):        # 24 heads x 5 items = 120 CTAs, 4 KV heads
            sl = slice(h0, h0 + 24)
            kv = slice(h0 // 6, h0 // 6 + 4)
            part_lse = torch.empty(1, 24, 1100, device="cuda")
            part = backend.attention_fa(q[b:b + 1, sl].contiguous(), k[b:b + 1, kv].contiguous(), v[b:b + 1, kv].contiguous(), scale, True, lse=part_lse)
            assert torch.equal(part.view(torch.int16), out[b:b + 1, sl].view(torch.int16))
            assert torch.equal(part_lse, lse[b:b + 1, sl])
    torch.cuda.synchronize()
    backend.poll()


@pytest.mark.parametrize("shape", [(1, 8, 8, 512, 512, 64, False), (1, 2, 1, 100, 333, 96, True), (2, 2, 2, 65, 65, 32, True)])
def test_fa_f32_kernel(backend, oracle, shape):
    b, hq, hkv, sq, skv, d, causal = shape
    q, k, v = make_qkv(b, hq, hkv, sq, skv, d, torch.float32)
    scale = d ** -0.5
    lse = torch.empty(b, hq, sq)
    out = backend.attention_fa(q, k, v, scale, causal, lse=lse, query_start=skv - sq if causal else 0)
    want = oracle.attention("f32", helpers.bits(q), helpers.bits(k), helpers.bits(v), scale, causal, tile_n=32, threads=8,
                            query_start=skv - sq if causal else 0)
    check_against_oracle(oracle, "f32", out, lse, want, lse_atol=1e-5)
    # also the way the reference's integration tests judge it: against eager SDPA in f32
    g = hq // hkv
    mask = torch.ones(sq, skv, dtype=torch.bool).tril(skv - sq) if causal else None
    ref = torch.nn.functional.scaled_dot_product_attention(q, k.repeat_interleave(g, 1), v.repeat_interleave(g, 1), attn_mask=mask)
    assert helpers.max_rel_err(out.double().numpy(), ref.double().numpy()) <= 1e-5
    # and element by element: |a - e| <= atol + rtol * |e| for every element (the reference's elementwise policy,
    # ProgramTensorComparison.cpp:276-403), with the ULP distance of the bulk bounded, against a float64 SDPA
    from vibe_compiler_b200.gate import ComparisonPolicy, ProgramTensor, compute_statistics
    ref64 = torch.nn.functional.scaled_dot_product_attention(q.double(), k.double().repeat_interleave(g, 1), v.double().repeat_interleave(g, 1),
                                                            attn_mask=mask).float()
    as_tensor = lambda t: ProgramTensor("f32", tuple(t.shape), np.frombuffer(t.contiguous().numpy().tobytes(), np.uint8))
    stats = compute_statistics(backend, as_tensor(out.cpu()), as_tensor(ref64), ComparisonPolicy(atol=5e-6, rtol=1e-5))
    assert stats.mismatch_count == 0 and stats.p99_ulp <= 1024, stats   # outputs near zero carry large ULP distances at tiny absolute error


@pytest.mark.parametrize("name", ["fa_bf16_gqa", "fa_f16_decode_tail", "fa_f32_cfg1_small"])
def test_fa_golden(backend, oracle, name):
    q, k, v, causal = fixtures.attention_inputs(name)
    fmt = helpers.FMT_OF[q.dtype]
    out = backend.attention_fa(q, k, v, q.shape[-1] ** -0.5, causal, query_start=k.shape[2] - q.shape[2] if causal else 0)
    expected = helpers.golden()[name]
    assert helpers.max_rel_err(helpers.values(helpers.bits(out), fmt), helpers.values(expected, fmt)) <= BOUND[fmt]
    helpers.reference_gate(oracle, fmt, helpers.bits(out), expected)


def test_fa_masks_and_fully_masked_rows(backend, oracle):
    q, k, v = make_qkv(1, 2, 2, 256, 300, 128, torch.bfloat16)
    scale = 128 ** -0.5
    # valid length shorter than the buffer, causal diagonal shifted so the first rows see nothing
    kwargs = dict(query_start=90, key_start=100, key_end=100 + 200)
    for zfm in (True, False):
        lse = torch.empty(1, 2, 256)
        out = backend.attention_fa(q, k, v, scale, True, lse=lse, zero_fully_masked=zfm, **kwargs)
        want = oracle.attention("bf16", helpers.bits(q), helpers.bits(k), helpers.bits(v), scale, True, zero_fully_masked=zfm, threads=8, **kwargs)
        got, exp = helpers.values(helpers.bits(out), "bf16"), helpers.values(want["out"], "bf16")
        assert np.array_equal(np.isnan(got), np.isnan(exp))
        ok = ~np.isnan(exp)
        assert helpers.max_rel_err(got[ok], exp[ok]) <= 1e-2
        assert np.array_equal(np.isneginf(lse.numpy()), np.isneginf(want["lse"]))
        if zfm:
            assert not np.isnan(got).any() and not got[0, 0, :10].any()   # rows 0..9 see no key: exact zeros


@pytest.mark.parametrize("shape", [(2, 8, 2, 1000, 2), (2, 32, 8, 4096, 0), (1, 4, 4, 77, 3), (1, 16, 1, 5000, 7), (3, 8, 8, 64, 2)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fd_decode_kernel(backend, oracle, shape, dtype):
    b, hq, hkv, kv, splits = shape
    fmt = helpers.FMT_OF[dtype]
    q, k, v = make_qkv(b, hq, hkv, 1, kv, 128, dtype)
    scale = 128 ** -0.5
    lse = torch.empty(b, hq, 1)
    out = backend.attention_fd(q, k, v, scale, kv_splits=splits, lse=lse)
    want = oracle.attention(fmt, helpers.bits(q), helpers.bits(k), helpers.bits(v), scale, splits=max(splits, 2), tile_n=16, threads=8)
    check_against_oracle(oracle, fmt, out, lse, want)


def test_fd_split_count_invariance_and_golden(backend, oracle):
    q, k, v, _ = fixtures.attention_inputs("fd_bf16_gqa")
    expected = helpers.golden()["fd_bf16_gqa"]
    outs = [backend.attention_fd(q, k, v, 128 ** -0.5, kv_splits=s) for s in (2, 3, 5, 13)]
    for out in outs:
        assert helpers.max_rel_err(helpers.values(helpers.bits(out), "bf16"), helpers.values(expected, "bf16")) <= 1e-2
        helpers.reference_gate(oracle, "bf16", helpers.bits(out), expected)


def test_fd_partial_states_and_shard_merge(backend, oracle):
    # Sequence-sharded decode: each shard produces (acc, m, l); ascending left-fold + finalize equals one pass.
    q, k, v = make_qkv(1, 8, 2, 1, 3000, 128, torch.bfloat16)
    scale = 128 ** -0.5
    bounds = [0, 700, 1500, 3000]
    states = torch.stack([backend.attention_fd_partial(q, k[:, :, lo:hi].contiguous(), v[:, :, lo:hi].contiguous(), scale, kv_splits=2)
                          for lo, hi in zip(bounds[:-1], bounds[1:])])
    lse = torch.empty(1, 8, 1)
    merged = backend.attention_fd_merge(states, q, lse=lse)
    want = oracle.attention("bf16", helpers.bits(q), helpers.bits(k), helpers.bits(v), scale, splits=6, tile_n=16, threads=8)
    check_against_oracle(oracle, "bf16", merged, lse, want)
    ostates = np.stack([oracle.attention_state("bf16", helpers.bits(q), helpers.bits(k[:, :, lo:hi].contiguous()), helpers.bits(v[:, :, lo:hi].contiguous()),
                                               scale, splits=2, tile_n=16) for lo, hi in zip(bounds[:-1], bounds[1:])])
    assert np.allclose(states.numpy()[..., 128], ostates[..., 128], atol=1e-5)            # m
    assert np.allclose(states.numpy()[..., 129], ostates[..., 129], rtol=1e-4)            # l
    oout, olse = oracle.attention_merge("bf16", states.numpy().reshape(3, -1, 130))
    assert helpers.max_rel_err(helpers.values(helpers.bits(merged).reshape(-1), "bf16"), helpers.values(oout.reshape(-1), "bf16")) <= 2 ** -7


def test_full_size_prefill_properties(backend):
    # batch 4, 32 heads, seq 4096, head_dim 128, causal, on device buffers. Properties that hold at any size:
    #  (1) rows of V all equal to one vector w  =>  every output row equals w (softmax weights sum to 1);
    #  (2) the first query row attends only to key 0  =>  out[0] == v[0], lse[0] == scale * q0.k0;
    #  (3) a sampled set of rows agrees with an f64 softmax reference computed on the GPU.
    b, h, s, d = 4, 32, 4096, 128
    g = torch.Generator(device="cuda").manual_seed(20260803)
    q = torch.randn(b, h, s, d, device="cuda", generator=g).bfloat16()
    k = torch.randn(b, h, s, d, device="cuda", generator=g).bfloat16()
    v = torch.randn(b, h, s, d, device="cuda", generator=g).bfloat16()
    scale = d ** -0.5
    lse = torch.empty(b, h, s, device="cuda")
    out = backend.attention_fa(q, k, v, scale, True, lse=lse)
    torch.cuda.synchronize()
    backend.poll()
    assert torch.equal(out[:, :, 0], v[:, :, 0])
    assert torch.allclose(lse[:, :, 0], (q[:, :, 0].float() * k[:, :, 0].float()).sum(-1) * scale, atol=1e-4)
    for bi, hi in [(0, 0), (3, 31), (1, 17)]:
        rows = torch.tensor([1, 127, 128, 255, 256, 2047, 4095], device="cuda")
        sc = (q[bi, hi, rows].double() @ k[bi, hi].double().t()) * scale
        sc = sc.masked_fill(torch.arange(s, device="cuda")[None, :] > rows[:, None], float("-inf"))
        ref = torch.softmax(sc, -1) @ v[bi, hi].double()
        assert ((out[bi, hi, rows].double() - ref).abs().max() / ref.abs().max()).item() <= 1e-2
        assert torch.allclose(lse[bi, hi, rows].double(), torch.logsumexp(sc, -1), atol=2e-4)
    w = torch.randn(d, device="cuda", generator=g).bfloat16()
    const = backend.attention_fa(q, k, w.expand(b, h, s, d).contiguous(), scale, True)
    torch.cuda.synchronize()
    backend.poll()
    assert ((const.float() - w.float()).abs().max() / w.float().abs().max()).item() <= 2 ** -7


def test_full_size_decode_properties(backend):
    # batch 64, 32 / 8 heads, KV 32768 (8 GiB of K and V) on device buffers.
    b, hq, hkv, kv, d = 64, 32, 8, 32768, 128
    g = torch.Generator(device="cuda").manual_seed(20260803)
    q = torch.randn(b, hq, 1, d, device="cuda", generator=g).bfloat16()
    k = torch.randn(b, hkv, kv, d, device="cuda", generator=g).bfloat16()
    v = torch.randn(b, hkv, kv, d, device="cuda", generator=g).bfloat16()
    scale = d ** -0.5
    lse = torch.empty(b, hq, 1, device="cuda")
    out = backend.attention_fd(q, k, v, scale, lse=lse)
    torch.cuda.synchronize()
    backend.poll()
    for bi in (0, 37, 63):
        kk = k[bi].double().repeat_interleave(4, 0)
        vv = v[bi].double().repeat_interleave(4, 0)
        sc = (q[bi].double() @ kk.transpose(-1, -2)) * scale
        ref = torch.softmax(sc, -1) @ vv
        assert ((out[bi].double() - ref).abs().max() / ref.abs().max()).item() <= 1e-2
        assert torch.allclose(lse[bi].double(), torch.logsumexp(sc, -1), atol=2e-4)
    # split-count invariance at full size (different partitions, same result to rounding)
    other = backend.attention_fd(q, k, v, scale, kv_splits=37)
    torch.cuda.synchronize()
    backend.poll()
    assert ((other.float() - out.float()).abs().max() / out.float().abs().max()).item() <= 2 ** -6


def test_full_size_long_context(backend):
    """cfg 3L at its real size: one sequence of 1 048 576 keys, 32 query heads over 8 KV heads, against a float64
    recomputation (output and log-sum-exp), through the single-GPU entry and through four sequence shards merged in
    ascending order."""
    from vibe_compiler_b200 import selfcheck
    from vibe_compiler_b200.sharding import sequence_range
    gen = torch.Generator(device="cuda").manual_seed(20260804)
    kv_len, scale = 1 << 20, 128 ** -0.5
    q = torch.randn(1, 32, 1, 128, device="cuda", generator=gen).bfloat16()
    k = torch.randn(1, 8, kv_len, 128, device="cuda", generator=gen).bfloat16()
    v = torch.randn(1, 8, kv_len, 128, device="cuda", generator=gen).bfloat16()
    want_out, want_lse = selfcheck.merge_states_f64([selfcheck.decode_state_f64(q, k, v, scale)])
    lse = torch.empty(1, 32, 1, device="cuda")
    out = backend.attention_fd(q, k, v, scale, lse=lse)
    states = []
    for rank in range(4):
        lo, hi = sequence_range(kv_len, 4, rank)
        states.append(backend.attention_fd_partial(q, k[:, :, lo:hi].contiguous(), v[:, :, lo:hi].contiguous(), scale))
    lse_sharded = torch.empty(1, 32, 1, device="cuda")
    out_sharded = backend.attention_fd_merge(torch.stack(states), q, lse=lse_sharded)
    torch.cuda.synchronize()
    backend.poll()
    for got, got_lse in ((out, lse), (out_sharded, lse_sharded)):
        assert selfcheck.max_rel_err(got.view(1, 32, 128), want_out) <= 1e-2
        assert (got_lse.view(1, 32).double() - want_lse).abs().max().item() <= 1e-3


def test_in_kernel_exchange_single_rank_matches_the_two_call_path(backend):
    """The decode step whose fold, exchange and merge run in one kernel, with a world of one rank (the buffer is ordinary
    device memory): same split records, same fold order, so the same bits as partial + merge, call after call (the
    epoch parity alternates)."""
    from vibe_compiler_b200.sharding import PeerExchange
    gen = torch.Generator(device="cuda").manual_seed(7)
    q = torch.randn(2, 32, 1, 128, device="cuda", generator=gen).bfloat16()
    k = torch.randn(2, 8, 5000, 128, device="cuda", generator=gen).bfloat16()
    v = torch.randn(2, 8, 5000, 128, device="cuda", generator=gen).bfloat16()
    scale = 128 ** -0.5
    exchange = PeerExchange(backend, 2, 32)
    want_lse = torch.empty(2, 32, 1, device="cuda")
    want = backend.attention_fd_merge(backend.attention_fd_partial(q, k, v, scale, kv_splits=6).unsqueeze(0), q, lse=want_lse)
    for call in range(3):
        lse = torch.empty(2, 32, 1, device="cuda")
        out = backend.attention_fd_exchange(q, k, v, scale, rank=0, peer_pointers=exchange.pointers, epoch=exchange.epoch, kv_splits=6, lse=lse)
        torch.cuda.synchronize()
        backend.poll()
        assert torch.equal(out.view(torch.int16), want.view(torch.int16)) and torch.equal(lse, want_lse)
        assert exchange.epoch.tolist() == [call + 1, 0]
