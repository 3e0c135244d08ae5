"""Independent float64 recomputations of the two multi-GPU regions, used to check full-size outputs.

The reference judges a whole transformer block against eager PyTorch
(test/Board/PyTorch/wafer_pytorch_board_cases.py:817-867, expected output :1019-1028). At the benchmark's
sizes a full eager recomputation is too large to run beside the kernels, so these helpers recompute
*sampled* token rows of the decoder layer (every row of the sequence is needed for K and V, only the sampled
rows for everything else) and the complete decode output, in float64 with plain torch operators on the
same device. Nothing here calls the library's kernels: it is the checker, not the path.
"""
from __future__ import annotations

from typing import Sequence, Tuple

import torch

from .decoder_layer import LayerConfig, LayerWeights


def layer_rows_f64(cfg: LayerConfig, w: LayerWeights, x: torch.Tensor, batch_index: int, rows: Sequence[int],
                   device: torch.device) -> torch.Tensor:
    """Rows `rows` of sequence `batch_index` of the decoder layer's output, in float64.

    x: [batch, seq, d_model] (any device); w: the full, unsharded weights. Position ids start at 0."""
    f64 = torch.float64
    hd, hq, hkv = cfg.head_dim, cfg.q_heads, cfg.kv_heads
    seq = x.shape[1]
    xs = x[batch_index].to(device=device, dtype=f64)                      # [seq, d]
    idx = torch.as_tensor(list(rows), device=device)

    def rms(t, g):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + cfg.eps) * g.to(device=device, dtype=f64)

    def on(t):
        return t.to(device=device, dtype=f64)
    h = rms(xs, w.norm1)
    inv_freq = cfg.rope_theta ** (-torch.arange(0, hd, 2, device=device, dtype=f64) / hd)

    def rope(t, positions):                                               # t: [n, heads, hd]
        angle = positions.to(f64)[:, None] * inv_freq[None, :]
        cos = torch.cat([angle.cos(), angle.cos()], -1)[:, None, :]
        sin = torch.cat([angle.sin(), angle.sin()], -1)[:, None, :]
        rotated = torch.cat([-t[..., hd // 2:], t[..., :hd // 2]], -1)
        return t * cos + rotated * sin
    all_pos = torch.arange(seq, device=device)
    k = rope((h @ on(w.wk)).view(seq, hkv, hd), all_pos)                   # [seq, hkv, hd]
    v = (h @ on(w.wv)).view(seq, hkv, hd)
    q = rope((h[idx] @ on(w.wq)).view(len(idx), hq, hd), idx)              # [n, hq, hd]
    group = hq // hkv
    k_rep, v_rep = k.repeat_interleave(group, 1), v.repeat_interleave(group, 1)   # [seq, hq, hd]
    scores = torch.einsum("nhd,shd->nhs", q, k_rep) * hd ** -0.5
    visible = all_pos[None, :] <= idx[:, None]                             # causal
    scores = scores.masked_fill(~visible[:, None, :], float("-inf"))
    attn = torch.einsum("nhs,shd->nhd", torch.softmax(scores, -1), v_rep).reshape(len(idx), hq * hd)
    x1 = xs[idx] + attn @ on(w.wo)
    h2 = rms(x1, w.norm2)
    act = torch.nn.functional.silu(h2 @ on(w.wgate)) * (h2 @ on(w.wup))
    return x1 + act @ on(w.wdown)


def decode_state_f64(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Un-normalised attention state of one KV shard in float64: (m [B, Hq], l [B, Hq], acc [B, Hq, D]).

    q: [B, Hq, 1, D]; k, v: [B, Hkv, S, D]. Keys are processed per KV head in chunks to bound memory."""
    f64 = torch.float64
    b, hq, _, d = q.shape
    hkv, s = k.shape[1], k.shape[2]
    group = hq // hkv
    qg = q.to(f64).view(b, hkv, group, d)
    m = torch.full((b, hkv, group), float("-inf"), dtype=f64, device=q.device)
    l = torch.zeros((b, hkv, group), dtype=f64, device=q.device)
    acc = torch.zeros((b, hkv, group, d), dtype=f64, device=q.device)
    chunk = 1 << 17
    for begin in range(0, s, chunk):
        kc = k[:, :, begin:begin + chunk].to(f64)
        vc = v[:, :, begin:begin + chunk].to(f64)
        scores = torch.einsum("bhgd,bhsd->bhgs", qg, kc) * scale
        m_new = torch.maximum(m, scores.amax(-1))
        alpha = torch.exp(m - m_new)
        p = torch.exp(scores - m_new[..., None])
        l = l * alpha + p.sum(-1)
        acc = acc * alpha[..., None] + torch.einsum("bhgs,bhsd->bhgd", p, vc)
        m = m_new
    return m.view(b, hq), l.view(b, hq), acc.view(b, hq, d)


def merge_states_f64(states: Sequence[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Combines shard states (ascending shard order) into (out [B, Hq, D], lse [B, Hq]) in float64."""
    m = torch.stack([s[0] for s in states]).amax(0)
    l = sum(s[1] * torch.exp(s[0] - m) for s in states)
    acc = sum(s[2] * torch.exp(s[0] - m)[..., None] for s in states)
    return acc / l[..., None], m + torch.log(l)


def max_rel_err(actual: torch.Tensor, expected: torch.Tensor) -> float:
    """max |a - e| / max |e| in float64: the bound stated for 16-bit storage paths (1e-2)."""
    a, e = actual.double(), expected.double()
    return float((a - e).abs().max() / e.abs().max().clamp_min(1e-30))
