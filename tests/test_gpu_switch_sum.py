"""The NVSwitch sum (wb200_switch_sum) on two or more GPUs: one process per GPU, values checked against a float64 sum
of every rank's (seeded) input, bit-identical results on all ranks, and the decoder layer through it against the same
layer with torch.distributed's all-reduce. Skipped on a machine with fewer than two GPUs."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_values(rank, elements, dtype, device):
    gen = torch.Generator(device=device).manual_seed(4242 + rank)
    return (torch.rand(elements, device=device, generator=gen) * 2 - 1).to(dtype)


def _worker(rank, world, port, results):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    from vibe_compiler_b200.backend import B200TargetModelBackend
    from vibe_compiler_b200.sharding import SwitchSum
    from vibe_compiler_b200.decoder_layer import LayerConfig, ShardedDecoderLayer, random_weights
    backend = B200TargetModelBackend(rank)
    report = {}
    sums = SwitchSum(backend, None, device)
    report["available"] = bool(sums.available)
    if sums.available:
        # ragged sizes: fewer chunks than ranks, a slice boundary inside a block, and a few MiB; three formats
        buffer = sums.allocate(48 << 20)
        worst = 0.0
        identical = True
        for dtype in (torch.bfloat16, torch.float16, torch.float32):
            for elements in (8, 8 * 3, 8 * 1027, (8 << 20) + 64):
                region = buffer[4096:4096 + elements * dtype.itemsize].view(dtype)
                for _ in range(3):          # the same signal words serve call after call
                    region.copy_(_rank_values(rank, elements, dtype, device))
                    torch.cuda.synchronize()
                    dist.barrier()
                    sums(region)
                    torch.cuda.synchronize()
                    backend.poll()
                    dist.barrier()
                want = sum(_rank_values(r, elements, dtype, device).double() for r in range(world))
                worst = max(worst, float((region.double() - want).abs().max() / want.abs().max()))
                gathered = [torch.empty_like(region) for _ in range(world)]
                dist.all_gather(gathered, region.clone())
                identical = identical and all(torch.equal(gathered[0], g) for g in gathered)
        # sum + residual stored to another region: the residual is the same tensor on every rank
        elements = 8 * 4099
        region = buffer[4096:4096 + elements * 2].view(torch.bfloat16)
        target = buffer[(24 << 20):(24 << 20) + elements * 2].view(torch.bfloat16)
        region.copy_(_rank_values(rank, elements, torch.bfloat16, device))
        residual = _rank_values(1000, elements, torch.bfloat16, device)
        torch.cuda.synchronize()
        dist.barrier()
        sums(region, residual=residual, out=target)
        torch.cuda.synchronize()
        backend.poll()
        dist.barrier()
        total = sum(_rank_values(r, elements, torch.bfloat16, device).double() for r in range(world))
        want = (total.to(torch.bfloat16).float() + residual.float()).to(torch.bfloat16)       # the sum is rounded, then the add
        close = (target.double() - want.double()).abs().max() / want.double().abs().max()
        report["residual_rel_err"] = float(close)
        report["partials_kept"] = bool(torch.equal(region, _rank_values(rank, elements, torch.bfloat16, device)))
        report["max_rel_err"], report["identical"] = worst, identical
        # the decoder layer with the switch doing its sums against the same layer with the library all-reduce
        cfg = LayerConfig(d_model=1024, q_heads=8, kv_heads=4, head_dim=128, ffn=2048)
        weights = random_weights(cfg, seed=7)
        layer = ShardedDecoderLayer(backend, cfg, weights, rank=rank, world_size=world, device=device)
        gen = torch.Generator(device=device).manual_seed(99)
        x = torch.randn(4, 256, cfg.d_model, device=device, generator=gen).bfloat16()
        got = layer.forward_fused(x, micro_batches=2).clone()
        report["layer_used_switch"] = layer.switch_sums() is not None
        os.environ["WB200_LAYER_SUM"] = "nccl"
        plain = ShardedDecoderLayer(backend, cfg, weights, rank=rank, world_size=world, device=device)
        want = plain.forward_fused(x, micro_batches=2)
        torch.cuda.synchronize()
        backend.poll()
        report["layer_rel_err"] = float((got.double() - want.double()).abs().max() / want.double().abs().max())
        torch.cuda.synchronize()
        dist.barrier()
    if rank == 0:
        results.update(report)
    dist.barrier()
    dist.destroy_process_group()


def test_switch_sum_matches_a_float64_sum_on_every_rank():
    world = 4 if torch.cuda.device_count() >= 4 else 2
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    results = dict(results)
    if not results["available"]:
        pytest.skip("these GPUs offer no NVLink multicast")
    assert results["identical"]
    assert results["max_rel_err"] <= 2.0 ** -7        # one rounding to 16 bits of an f32 sum
    assert results["residual_rel_err"] <= 2.0 ** -6 and results["partials_kept"]
    assert results["layer_used_switch"]
    assert results["layer_rel_err"] <= 1e-2
