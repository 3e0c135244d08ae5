"""Oracle against outputs of the reference's Python expected-output generator (PyTorch eager on CPU),
committed as tests/golden/torch_expected.npz. CPU only."""
import numpy as np
import pytest

from tests import helpers
from tests.helpers import fixtures


@pytest.mark.parametrize("name", list(fixtures.ATTENTION_CASES))
def test_attention_oracle_meets_reference_gate(oracle, name):
    q, k, v, causal = fixtures.attention_inputs(name)
    fmt = helpers.FMT_OF[q.dtype]
    expected = helpers.golden()[name]
    d = q.shape[-1]
    is_decode = q.shape[2] == 1
    got = oracle.attention(fmt, helpers.bits(q), helpers.bits(k), helpers.bits(v), d ** -0.5, causal,
                           splits=3 if is_decode else 1, tile_n=64,
                           query_start=k.shape[2] - q.shape[2] if causal else 0)
    helpers.reference_gate(oracle, fmt, got["out"], expected)
    bound = 1e-5 if fmt == "f32" else 1e-2
    assert helpers.max_rel_err(helpers.values(got["out"], fmt), helpers.values(expected, fmt)) <= bound


def test_attention_oracle_tile_and_split_invariance(oracle):
    # The online update and the state merge are exact rewrites of softmax(QK^T)V: results for any tile
    # size or split count agree to rounding (f32: 1e-5).
    q, k, v, _ = fixtures.attention_inputs("fa_f32_cfg1_small")
    base = oracle.attention("f32", helpers.bits(q), helpers.bits(k), helpers.bits(v), 0.125, tile_n=64)
    for tile, splits in [(7, 1), (16, 1), (64, 1)]:
        other = oracle.attention("f32", helpers.bits(q), helpers.bits(k), helpers.bits(v), 0.125, tile_n=tile, splits=splits)
        assert helpers.max_rel_err(helpers.values(other["out"], "f32"), helpers.values(base["out"], "f32")) <= 1e-5
        assert np.allclose(other["lse"], base["lse"], rtol=0, atol=1e-5)


def test_fd_state_merge_equals_direct(oracle):
    q, k, v, _ = fixtures.attention_inputs("fd_bf16_gqa")
    qb, kb, vb = helpers.bits(q), helpers.bits(k), helpers.bits(v)
    direct = oracle.attention("bf16", qb, kb, vb, 128 ** -0.5, splits=4, tile_n=16)
    half = k.shape[2] // 2
    states = np.stack([
        oracle.attention_state("bf16", qb, kb, vb, 128 ** -0.5, splits=2, tile_n=16, key_start=0, key_end=half),
        # second shard: keys [half, end) of the same tensors
        oracle.attention_state("bf16", qb, np.ascontiguousarray(kb[:, :, half:]), np.ascontiguousarray(vb[:, :, half:]),
                               128 ** -0.5, splits=2, tile_n=16),
    ]).reshape(2, -1, 130)
    out, lse = oracle.attention_merge("bf16", states)
    assert helpers.max_rel_err(helpers.values(out.reshape(-1), "bf16"), helpers.values(direct["out"].reshape(-1), "bf16")) <= 1e-2
    assert np.allclose(lse, direct["lse"].reshape(-1), atol=1e-4)


def test_fully_masked_rows(oracle):
    q, k, v, _ = fixtures.attention_inputs("fa_f32_cfg1_small")
    # causal with query_start far before key_start: no key is visible to any row.
    got = oracle.attention("f32", helpers.bits(q), helpers.bits(k), helpers.bits(v), 0.125, True, query_start=-1000,
                           zero_fully_masked=True)
    assert not got["out"].any() and np.all(np.isneginf(got["lse"])) and not got["l"].any()
    got = oracle.attention("f32", helpers.bits(q), helpers.bits(k), helpers.bits(v), 0.125, True, query_start=-1000)
    assert np.all(np.isnan(helpers.values(got["out"], "f32")))  # 0 * (1/0), as eager softmax gives


@pytest.mark.parametrize("name", list(fixtures.GEMM_CASES))
def test_gemm_oracle_against_torch_matmul(oracle, name):
    a, b = fixtures.gemm_inputs(name)
    fmt = helpers.FMT_OF[a.dtype]
    m, k = a.shape
    n = b.shape[1]
    expected = helpers.golden()[name]
    got = oracle.formal_gemm(fmt, fmt, 1, m, k, n, helpers.bits(a).reshape(-1), helpers.bits(b).reshape(-1)).reshape(m, n)
    if fixtures.GEMM_CASES[name][4]:
        assert np.array_equal(got, expected)  # exact-input long-K variant: EXACT policy in the reference
    else:
        bound = 1e-5 if fmt == "f32" else 1e-2
        assert helpers.max_rel_err(helpers.values(got, fmt), helpers.values(expected, fmt)) <= bound
    same = oracle.gemm_epilogue(fmt, fmt, m, n, k, helpers.bits(a), helpers.bits(b))
    assert np.array_equal(same, got)


def test_comparator_statistics(oracle):
    expected = np.array([1.0, -2.0, 0.0, 4.0], dtype=np.float32)
    actual = np.array([1.0, -2.0, -0.0, 4.0 + 2 ** -21], dtype=np.float32)
    stats = oracle.compare("f32", actual.view(np.uint32), expected.view(np.uint32), atol=0.0, rtol=0.0)
    assert stats["element_count"] == 4 and stats["mismatch_count"] == 1
    # signed zeros differ in bits but count as exact (ProgramTensorComparisonTest.cpp:360-367)
    assert stats["max_ulp"] == 1 and stats["exact_count"] == 3
    assert stats["cosine"] > 0.999999 and stats["relative_l2"] < 1e-6
    zero = np.zeros(4, dtype=np.uint32)
    assert oracle.compare("f32", zero, zero)["cosine"] == 1.0
    assert oracle.compare("f32", actual.view(np.uint32), zero)["relative_l2"] == float("inf")
    bad = np.array([0x7f800000], dtype=np.uint32)
    assert oracle.compare("f32", bad, bad)["finite"] == 0
