"""Generates tests/golden/llama_layer_expected.npz: the output of Hugging Face's eager LlamaDecoderLayer in f32 on
the CPU for a small grouped-query configuration - the module family the reference's own decoder-block test runs
(its case uses the Llama-2-7B block at sequence length 16). Weights and input come from
vibe_compiler_b200.decoder_layer.random_weights / a seeded generator, quantised to bf16 once and widened to f32
for the expected output, the reference's rule for expected values.

Run from the repository root:  python tests/golden/make_llama_layer_fixture.py
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from vibe_compiler_b200.decoder_layer import LayerConfig, random_weights  # noqa: E402

OUT = Path(__file__).resolve().parent / "llama_layer_expected.npz"
CFG = LayerConfig(d_model=512, q_heads=4, kv_heads=2, head_dim=128, ffn=768, eps=1e-5, rope_theta=10000.0)
BATCH, SEQ, SEED = 2, 160, 20260803


def layer_input():
    g = torch.Generator(device="cpu").manual_seed(SEED + 7)
    return torch.randn(BATCH, SEQ, CFG.d_model, generator=g).bfloat16()


def hf_expected():
    from transformers.models.llama.configuration_llama import LlamaConfig
    from transformers.models.llama.modeling_llama import LlamaDecoderLayer, LlamaRotaryEmbedding
    config = LlamaConfig(hidden_size=CFG.d_model, intermediate_size=CFG.ffn, num_attention_heads=CFG.q_heads,
                         num_key_value_heads=CFG.kv_heads, head_dim=CFG.head_dim, rms_norm_eps=CFG.eps,
                         rope_theta=CFG.rope_theta, max_position_embeddings=4096, attention_bias=False, mlp_bias=False,
                         num_hidden_layers=1, vocab_size=32)
    config._attn_implementation = "eager"
    weights = random_weights(CFG)
    layer = LlamaDecoderLayer(config, layer_idx=0).float().eval()
    with torch.no_grad():
        layer.input_layernorm.weight.copy_(weights.norm1.float())
        layer.post_attention_layernorm.weight.copy_(weights.norm2.float())
        layer.self_attn.q_proj.weight.copy_(weights.wq.float().t())
        layer.self_attn.k_proj.weight.copy_(weights.wk.float().t())
        layer.self_attn.v_proj.weight.copy_(weights.wv.float().t())
        layer.self_attn.o_proj.weight.copy_(weights.wo.float().t())
        layer.mlp.gate_proj.weight.copy_(weights.wgate.float().t())
        layer.mlp.up_proj.weight.copy_(weights.wup.float().t())
        layer.mlp.down_proj.weight.copy_(weights.wdown.float().t())
        x = layer_input().float()
        positions = torch.arange(SEQ)[None, :].expand(BATCH, SEQ)
        cos_sin = LlamaRotaryEmbedding(config)(x, positions)
        mask = torch.full((SEQ, SEQ), float("-inf")).triu(1)[None, None]
        out = layer(x, attention_mask=mask, position_ids=positions, position_embeddings=cos_sin)
        out = out[0] if isinstance(out, tuple) else out
    return out


if __name__ == "__main__":
    torch.set_num_threads(4)
    expected = hf_expected()
    np.savez_compressed(OUT, expected=expected.numpy().astype(np.float32))
    print(f"wrote {OUT}: shape {tuple(expected.shape)}, |max| {expected.abs().max():.3f}")
