"""The allocation-free decode entry point (wb200_attention_fd_static) against the regular one.

Callers that cannot allocate at call time (a fixed memory plan, a latency-critical loop, a
process under a memory cap) use this entry; it must give the same result as wb200_attention_fd, call after
call, although every call reuses the one scratch array inside the library. Collected last on purpose."""
import numpy as np
import pytest
import torch

from tests import helpers
from vibe_compiler_b200 import _abi as abi
from vibe_compiler_b200.backend import WB200Error

pytestmark = pytest.mark.gpu


def make(b, hq, hkv, kv, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(b, hq, 1, 128, generator=g).bfloat16().cuda()
    k = torch.randn(b, hkv, kv, 128, generator=g).bfloat16().cuda()
    v = torch.randn(b, hkv, kv, 128, generator=g).bfloat16().cuda()
    return q, k, v


def test_static_scratch_decode_matches_regular_entry_twice(backend, oracle):
    scale = 128 ** -0.5
    # two calls in a row with different shapes and split counts: the second must not see the first's records
    for call, (shape, splits) in enumerate([((2, 32, 8, 5000), 7), ((3, 8, 2, 1234), 3)]):
        q, k, v = make(*shape, seed=100 + call)
        lse_static = torch.empty(shape[0], shape[1], 1, device="cuda")
        lse_regular = torch.empty_like(lse_static)
        out_static = torch.empty_like(q)
        backend.attention_fd_static(q, k, v, scale, kv_splits=splits, out=out_static, lse=lse_static)
        out_regular = backend.attention_fd(q, k, v, scale, kv_splits=splits, lse=lse_regular)
        torch.cuda.synchronize()
        backend.poll()
        # same kernels, same partition: identical bits; the suite's bf16 bound (1e-2) is the stated tolerance
        err = helpers.max_rel_err(out_static.double().cpu().numpy(), out_regular.double().cpu().numpy())
        assert err <= 1e-2
        assert torch.equal(out_static.view(torch.int16), out_regular.view(torch.int16))
        assert torch.equal(lse_static, lse_regular)
        want = oracle.attention("bf16", helpers.bits(q), helpers.bits(k), helpers.bits(v), scale, splits=splits, tile_n=16, threads=8)
        assert helpers.max_rel_err(helpers.values(helpers.bits(out_static), "bf16"), helpers.values(want["out"], "bf16")) <= 1e-2


def test_static_scratch_decode_limits(backend):
    q, k, v = make(1, 8, 2, 256, seed=3)
    with pytest.raises(WB200Error) as err:   # 64 * 32 * 64 * 130 floats > 4 Mi
        big_q = torch.zeros(64, 32, 1, 128, dtype=torch.bfloat16, device="cuda")
        big_k = torch.zeros(64, 8, 128, 128, dtype=torch.bfloat16, device="cuda")
        backend.attention_fd_static(big_q, big_k, big_k, 1.0, kv_splits=64)
    assert err.value.status == abi.ERR_LIMIT and "16 MiB" in err.value.message
    with pytest.raises(ValueError):
        backend.attention_fd_static(q.cpu(), k.cpu(), v.cpu(), 1.0)
    # kv_splits == 0 picks a split count that fits
    big_q = torch.randn(64, 32, 1, 128, device="cuda").bfloat16()
    big_k = torch.randn(64, 8, 4096, 128, device="cuda").bfloat16()
    out = backend.attention_fd_static(big_q, big_k, big_k, 128 ** -0.5)
    ref = backend.attention_fd(big_q, big_k, big_k, 128 ** -0.5)
    torch.cuda.synchronize()
    backend.poll()
    assert ((out.float() - ref.float()).abs().max() / ref.float().abs().max()).item() <= 1e-2
