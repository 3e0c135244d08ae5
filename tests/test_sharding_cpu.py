"""Host logic of the multi-GPU paths on CPU: partitioning, and the sequence-sharded decode exchange on a
world-size-2 gloo group with the CPU oracle standing in for the device kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests import helpers
from vibe_compiler_b200 import sharding


def test_unit_range_covers_everything_once():
    for units in (0, 1, 7, 128, 513):
        for world in (1, 2, 3, 8):
            spans = [sharding.unit_range(units, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == units
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.unit_range(4, 2, 2)


def test_sequence_range_is_tile_aligned_and_contiguous():
    for kv in (1, 63, 64, 1000, 1048576, 12345):
        for world in (1, 2, 4, 8):
            spans = [sharding.sequence_range(kv, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == kv
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(b % 64 == 0 or b == kv for b, _ in spans)


def _worker(rank, world, port, q, k, v, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import binding as oracle
    scale = q.shape[-1] ** -0.5
    qb = helpers.bits(q)

    def state_fn(begin, end):
        kb, vb = helpers.bits(k[:, :, begin:end].contiguous()), helpers.bits(v[:, :, begin:end].contiguous())
        if end == begin:   # an empty shard contributes the neutral state (m = -inf, l = 0, acc = 0)
            state = np.zeros((q.shape[0], q.shape[1], q.shape[3] + 2), np.float32)
            state[..., -2] = -np.inf
            return torch.from_numpy(state)
        return torch.from_numpy(oracle.attention_state("bf16", qb, kb, vb, scale, splits=2, tile_n=16))

    def merge_fn(states):
        out, _ = oracle.attention_merge("bf16", states.numpy().reshape(states.shape[0], -1, states.shape[-1]))
        return oracle.from_bits(out, "bf16").reshape(q.shape)

    out = sharding.sharded_decode(state_fn, merge_fn, k.shape[2])
    if rank == 0:
        torch.save(out, out_path)
    dist.barrier()
    dist.destroy_process_group()


def test_sequence_sharded_decode_world2(tmp_path, oracle):
    g = torch.Generator().manual_seed(20260803)
    q = torch.randn(1, 8, 1, 128, generator=g).bfloat16()
    k = torch.randn(1, 2, 1500, 128, generator=g).bfloat16()
    v = torch.randn(1, 2, 1500, 128, generator=g).bfloat16()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out_path = str(tmp_path / "out.pt")
    mp.spawn(_worker, args=(2, port, q, k, v, out_path), nprocs=2, join=True)
    sharded = torch.load(out_path)
    direct = oracle.attention("bf16", helpers.bits(q), helpers.bits(k), helpers.bits(v), 128 ** -0.5, splits=4, tile_n=16)
    err = helpers.max_rel_err(helpers.values(helpers.bits(sharded), "bf16"), helpers.values(direct["out"], "bf16"))
    assert err <= 1e-2
