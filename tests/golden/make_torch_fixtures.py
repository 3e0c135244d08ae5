"""Generates tests/golden/torch_expected.npz: expected outputs computed the way the reference's own
integration tests compute them - PyTorch eager on the CPU, attention on f32-promoted copies of the
already-quantised inputs and cast back (the recipe of the reference's test/Board/PyTorch cases:
Q, K ~ N(0,1) * 0.125, V ~ N(0,1), seed 20260803; GEMM by torch.matmul in the storage dtype; the
exact-input GEMM variant uses signed sixteenths so every f32 product and sum is exact).

Run from the repository root:  python tests/golden/make_torch_fixtures.py
Only inputs' seeds and shapes are stored besides the expected outputs; tests regenerate the inputs.
"""
from pathlib import Path

import numpy as np
import torch

SEED = 20260803
OUT = Path(__file__).resolve().parent / "torch_expected.npz"

ATTENTION_CASES = {
    # name: (dtype, batch, q_heads, kv_heads, q_len, kv_len, head_dim, causal)
    "fa_bf16_gqa": (torch.bfloat16, 1, 4, 2, 160, 160, 128, True),
    "fa_f16_decode_tail": (torch.float16, 1, 2, 2, 96, 333, 128, True),
    "fa_f32_cfg1_small": (torch.float32, 1, 2, 2, 64, 64, 64, False),
    "fd_bf16_gqa": (torch.bfloat16, 2, 8, 2, 1, 777, 128, False),
}
GEMM_CASES = {
    # name: (dtype, m, k, n, exact_inputs)
    "gemm_bf16": (torch.bfloat16, 136, 264, 200, False),
    "gemm_f16_exact_long_k": (torch.float16, 64, 2048, 72, True),
    "gemm_f32": (torch.float32, 33, 65, 17, False),
}


def attention_inputs(name):
    dtype, b, hq, hkv, sq, skv, d, causal = ATTENTION_CASES[name]
    g = torch.Generator(device="cpu").manual_seed(SEED + sum(map(ord, name)))
    q = (torch.randn(b, hq, sq, d, generator=g) * 0.125).to(dtype)
    k = (torch.randn(b, hkv, skv, d, generator=g) * 0.125).to(dtype)
    v = torch.randn(b, hkv, skv, d, generator=g).to(dtype)
    return q, k, v, causal


def attention_expected(name):
    q, k, v, causal = attention_inputs(name)
    group = q.shape[1] // k.shape[1]
    kf, vf = k.float().repeat_interleave(group, 1), v.float().repeat_interleave(group, 1)
    mask = None
    if causal:
        sq, skv = q.shape[2], k.shape[2]
        mask = torch.ones(sq, skv, dtype=torch.bool).tril(skv - sq)
    out = torch.nn.functional.scaled_dot_product_attention(q.float(), kf, vf, attn_mask=mask)
    return out.to(q.dtype)


def gemm_inputs(name):
    dtype, m, k, n, exact = GEMM_CASES[name]
    g = torch.Generator(device="cpu").manual_seed(SEED + sum(map(ord, name)))
    if exact:
        def values(shape):
            integers = torch.randint(-8, 9, shape, generator=g)
            integers[integers == 0] = 1
            return integers.to(dtype) / 16
        return values((m, k)), values((k, n))
    return torch.randn(m, k, generator=g).to(dtype), torch.randn(k, n, generator=g).to(dtype)


def gemm_expected(name):
    a, b = gemm_inputs(name)
    return torch.matmul(a, b)


def bits(t):
    t = t.contiguous()
    return t.view(torch.int32).numpy().view(np.uint32) if t.dtype == torch.float32 else t.view(torch.int16).numpy().view(np.uint16)


if __name__ == "__main__":
    torch.set_num_threads(1)
    arrays = {name: bits(attention_expected(name)) for name in ATTENTION_CASES}
    arrays.update({name: bits(gemm_expected(name)) for name in GEMM_CASES})
    np.savez_compressed(OUT, **arrays)
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes)")
