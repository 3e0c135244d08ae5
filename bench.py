#!/usr/bin/env python
"""Benchmark of the hot path: flash-attention prefill (tensor-pipe bound) as the headline line, with
flash-decoding (HBM bound) and the GEMM + bias + GELU region reported beside it in the same JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: FA prefill bf16, batch 4, 32 heads, seq 4096, head_dim 128, causal, synthetic N(0,1) inputs
from a seed. One step = one pass of the kernel over that batch. At N > 1 the 128 independent
(batch, head) units of that fixed problem are dealt out in contiguous blocks, 128 / N per rank, with no
data-path collective (strong scaling: value = the whole problem's flop / the slowest rank's time).
`value` is device-timed with inputs resident in HBM; `e2e` goes through the public host-buffer call
(pinned host memory, copies inside the timed region). `--impl reference` times the CPU restatement
of the reference's numeric path (the reference itself needs LLVM/MLIR/SystemC and cannot be built
here) on all host threads on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FA = dict(batch=4, heads=32, kv_heads=32, seq=4096, head_dim=128)
FD = dict(batch=64, q_heads=32, kv_heads=8, kv_len=32768, head_dim=128)
GEMM = dict(m=8192, n=8192, k=8192)
FD_LONG = dict(q_heads=32, kv_heads=8, kv_len=1048576, head_dim=128)
LAYER = dict(batch=8, seq=2048)   # Llama-style decoder layer: d_model 4096, 32/8 heads, head_dim 128, FFN 14336
SEED = 20260803
# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures summarised under profiles/,
# taken on reduced cases (bench.py --profile-case) and scaled to a full launch by the units processed.
TRAFFIC = {
    "fa": 2 * (214.2e6 + 46.1e6),      # profiles/fa_umma_kernel_cfg2.md: batch 2 of 4 captured
    "fd": 8 * (1.073832e9 + 6.2e6),    # profiles/fd_partial_kernel_cfg3.md: batch 8 of 64 captured
    "layer": 8.259e9 + 1.472e9,        # profiles/decoder_layer_tp1_dram.md: the ten kernels of one full-size forward on one GPU
    "gemm": 1.118e9 + 0.124e9,         # profiles/gemm_umma_pair_kernel_cfg4.md: the full 8192^3 launch, one-pass capture
}


def fa_flops(batch, heads, seq, d):
    """Visible (query, key) pairs only: 4 * B * H * D * S (S + 1) / 2."""
    return 4 * batch * heads * d * seq * (seq + 1) // 2


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": data["hbm_gbs"], "bf16_tflops": data["bf16_tflops"],
                "bf16_tflops_sustained": data.get("bf16_tflops_sustained", data["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: an NVML polling thread (a reading every
    millisecond or so, since the timed region lasts only milliseconds), or nvidia-smi when NVML cannot be loaded."""
    QUERY = ("index,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.thread = None
        self.samples, self.reason_bits, self.max_clock = [], 0, None

    def _poll(self, nvml, handle):
        while not self.stop.is_set():
            try:
                self.samples.append(float(nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM)))
                self.reason_bits |= int(nvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle))
            except Exception:
                break
            time.sleep(0.0005)

    def __enter__(self):
        try:
            import pynvml as nvml
            import threading
            nvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            index = int(visible.split(",")[self.device_index]) if visible and visible.split(",")[self.device_index].isdigit() else self.device_index
            handle = nvml.nvmlDeviceGetHandleByIndex(index)
            self.max_clock = float(nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM))
            self.stop = threading.Event()
            self.thread = threading.Thread(target=self._poll, args=(nvml, handle), daemon=True)
            self.thread.start()
            return self
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.thread:
            self.stop.set()
            self.thread.join(timeout=2)
            if self.samples:
                reasons = sorted(name for bit, name in self.REASON_BITS.items() if self.reason_bits & bit)
                self.result = {"sm_mhz": statistics.median(self.samples), "sm_min_mhz": min(self.samples), "sm_max_mhz": self.max_clock,
                               "reasons": reasons, "samples": len(self.samples), "source": "nvml"}
            return
        if not self.proc:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, reasons, max_clock = [], set(), None
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[1]))
                max_clock = float(parts[2])
            except ValueError:
                continue
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        if clocks:
            self.result = {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max_clock, "reasons": sorted(reasons), "samples": len(clocks),
                           "source": "nvidia-smi"}


def timed_steps(fn, steps, warmup, torch, dist=None, check=None, flush=None):
    """Warm-up, then `steps` launches bracketed by barrier + synchronize; per-launch CUDA events on the
    launching stream. Returns (total ms over the bracket, mean per-launch ms). `check` runs after the
    first warm-up launch and raises if the device reported a failure, before any time is spent.
    `flush`: a buffer larger than the L2, rewritten before every timed launch (for inputs that would fit the
    L2); the flush writes are then taken out of the total, which becomes the sum of the per-launch times."""
    for i in range(warmup):
        fn()
        if i == 0 and check is not None:
            torch.cuda.synchronize()
            check()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for index, (begin, end) in enumerate(events):
        if flush is not None:
            flush.fill_(index & 0xff)
        begin.record()
        fn()
        end.record()
    stop.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    per_launch = sum(b.elapsed_time(e) for b, e in events) / steps
    total = start.elapsed_time(stop) if flush is None else per_launch * steps
    return total, per_launch


CPU_SAMPLE_UNITS = 4


def cpu_sample(threads: int, units: int = CPU_SAMPLE_UNITS):
    """`units` (batch, head) units of the FA workload through the CPU oracle. Returns (seconds, flops, description)."""
    import numpy as np
    from oracle import binding
    binding.build()
    rng = np.random.default_rng(SEED)
    s, d = FA["seq"], FA["head_dim"]

    def bf16(shape):
        x = rng.standard_normal(shape, dtype=np.float32)
        return binding.convert("f32", "bf16", x.view(np.uint32).reshape(-1))[1].reshape(shape)
    q, k, v = bf16((1, units, s, d)), bf16((1, units, s, d)), bf16((1, units, s, d))
    t0 = time.perf_counter()
    binding.attention("bf16", q, k, v, d ** -0.5, True, tile_n=128, threads=threads)
    seconds = time.perf_counter() - t0
    return seconds, fa_flops(1, units, s, d), (f"{units} of {FA['batch'] * FA['heads']} (batch, head) units: seq {s}, head_dim {d}, causal, "
                                               f"{threads} threads")


def cpu_baselines(threads: int):
    """CPU numbers beside the other configurations, each on a stated fraction of the workload (rank 0, N = 1 only).
    Decode: the oracle (the reference's online update restated, `kind: port`) on 2 of the 64 sequences, all threads.
    GEMM: the reference's oneDNN profile (OneDNNGemmAdapter.cpp:94-126, 351-357): operands widened to f32 once, a
    sequential f32 matmul on ONE thread (torch's bundled oneDNN stands in for the pinned build), 512 of the 8192 rows.
    Decoder layer: eager f32 torch on all threads, one sequence of 256 tokens, scaled by flop."""
    import numpy as np
    import torch
    from oracle import binding
    binding.build()
    rng = np.random.default_rng(SEED)

    def bf16(shape):
        x = rng.standard_normal(shape, dtype=np.float32)
        return binding.convert("f32", "bf16", x.view(np.uint32).reshape(-1))[1].reshape(shape)
    out = {}
    sequences = 2
    q = bf16((sequences, FD["q_heads"], 1, FD["head_dim"]))
    k = bf16((sequences, FD["kv_heads"], FD["kv_len"], FD["head_dim"]))
    v = bf16((sequences, FD["kv_heads"], FD["kv_len"], FD["head_dim"]))
    t0 = time.perf_counter()
    binding.attention("bf16", q, k, v, FD["head_dim"] ** -0.5, splits=16, tile_n=16, threads=threads)
    seconds = time.perf_counter() - t0
    out["fd_decode"] = {"value": 2 * k.size * 2 / seconds / 1e9, "unit": "GB/s", "cores": threads, "kind": "port", "seconds": seconds,
                        "sample": f"{sequences} of {FD['batch']} sequences (KV {FD['kv_len']}, 32 / 8 heads), {threads} threads"}
    previous = torch.get_num_threads()
    torch.set_num_threads(1)
    rows = 512
    a = (torch.rand(rows, GEMM["k"]) * 2 - 1).bfloat16().float()      # widened once, as the adapter does
    b = (torch.rand(GEMM["k"], GEMM["n"]) * 2 - 1).bfloat16().float()
    bias = torch.randn(GEMM["n"]) * 0.02
    t0 = time.perf_counter()
    torch.nn.functional.gelu(a @ b + bias).bfloat16()
    seconds = time.perf_counter() - t0
    out["gemm_bias_gelu"] = {"value": 2 * rows * GEMM["n"] * GEMM["k"] / seconds / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": "port", "seconds": seconds,
                             "sample": f"{rows} of {GEMM['m']} rows, operands widened to f32, sequential f32 matmul on one thread (the reference's oneDNN profile)"}
    torch.set_num_threads(previous)
    from vibe_compiler_b200.decoder_layer import LayerConfig, layer_flops
    cfg = LayerConfig()
    tokens = 256
    g = torch.Generator().manual_seed(SEED)
    w = lambda *shape: torch.randn(*shape, generator=g) * 0.02   # noqa: E731
    wq, wk, wv, wo = w(cfg.d_model, cfg.q_heads * cfg.head_dim), w(cfg.d_model, cfg.kv_heads * cfg.head_dim), w(cfg.d_model, cfg.kv_heads * cfg.head_dim), w(cfg.q_heads * cfg.head_dim, cfg.d_model)
    wg, wu, wd = w(cfg.d_model, cfg.ffn), w(cfg.d_model, cfg.ffn), w(cfg.ffn, cfg.d_model)
    x = torch.randn(tokens, cfg.d_model, generator=g)
    t0 = time.perf_counter()
    rms = lambda t: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + cfg.eps)   # noqa: E731
    h = rms(x)
    qh = (h @ wq).view(tokens, cfg.q_heads, cfg.head_dim).transpose(0, 1)
    kh = (h @ wk).view(tokens, cfg.kv_heads, cfg.head_dim).transpose(0, 1).repeat_interleave(cfg.q_heads // cfg.kv_heads, 0)
    vh = (h @ wv).view(tokens, cfg.kv_heads, cfg.head_dim).transpose(0, 1).repeat_interleave(cfg.q_heads // cfg.kv_heads, 0)
    attn = torch.nn.functional.scaled_dot_product_attention(qh[None], kh[None], vh[None], is_causal=True)[0].transpose(0, 1).reshape(tokens, -1)
    x1 = x + attn @ wo
    h2 = rms(x1)
    (x1 + (torch.nn.functional.silu(h2 @ wg) * (h2 @ wu)) @ wd).sum().item()
    seconds = time.perf_counter() - t0
    out["decoder_layer"] = {"value": layer_flops(cfg, 1, tokens) / seconds / 1e12, "unit": "TFLOP/s", "cores": previous, "kind": "port", "seconds": seconds,
                            "sample": f"one sequence of {tokens} tokens of the 8 x 2048 (rotary omitted), eager f32 torch on {previous} threads"}
    return out


def layer_extra(backend, args, torch, dist, rank, world, device, peak, failures):
    """Llama-style decoder layer forward (batch 8 x seq 2048), tensor-parallel over the ranks: heads and FFN columns are
    sharded, the two partial sums are done by the NVSwitch through the library's multimem kernel (torch.distributed's
    all-reduce where the GPUs have no NVLink multicast). Strong scaling: total work is fixed as the world grows."""
    from vibe_compiler_b200.decoder_layer import LayerConfig, ShardedDecoderLayer, layer_flops, random_weights
    cfg = LayerConfig()
    weights = random_weights(cfg, seed=SEED)
    layer = ShardedDecoderLayer(backend, cfg, weights, rank=rank, world_size=world, device=device)
    gen = torch.Generator(device="cpu").manual_seed(SEED + 5)
    x = torch.randn(LAYER["batch"], LAYER["seq"], cfg.d_model, generator=gen).bfloat16().to(device)
    parts = int(os.environ.get("WB200_LAYER_MICRO_BATCHES", "0")) or None   # default: 4 when tensor parallel
    reserved = int(os.environ.get("WB200_LAYER_RESERVED_SMS", str(layer.default_reserved_sms())))   # SMs left to NCCL
    total_ms, _ = timed_steps(lambda: layer.forward_fused(x, micro_batches=parts, reserved_sms=reserved), args.steps, args.warmup, torch, dist=dist, check=backend.poll)
    backend.poll()
    elapsed = torch.tensor([total_ms], device=device)
    if dist is not None:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms = elapsed.item() / args.steps
    flops = layer_flops(cfg, LAYER["batch"], LAYER["seq"])
    tflops = flops / (ms * 1e-3) / 1e12
    # Check what was timed (the tensor-parallel output, all-reduces included): sampled token rows of rank 0's copy against
    # a float64 recomputation from the full weights, as the reference judges its transformer block against eager PyTorch.
    from vibe_compiler_b200 import selfcheck
    out = layer.forward_fused(x, micro_batches=parts, reserved_sms=reserved)
    torch.cuda.synchronize()
    backend.poll()
    layer_err = 0.0
    if rank == 0:
        for batch_index, rows in ((0, [0, 1, 127, 1000, 2047]), (LAYER["batch"] - 1, [255, 256, 1531])):
            want = selfcheck.layer_rows_f64(cfg, weights, x, batch_index, rows, device)
            layer_err = max(layer_err, selfcheck.max_rel_err(out[batch_index, rows], want))
        if not layer_err <= 1e-2:
            failures.append(f"decoder_layer TP{world}: max rel err {layer_err:.3e} on sampled rows")
    del weights
    breakdown = None
    if world > 1:
        # Where the step's time goes: the same layer with the sums left out (compute only; its output is meaningless), and
        # one all-reduce of a whole [tokens, d_model] partial sum on its own.
        layer._all_reduce_enabled = False
        compute_ms, _ = timed_steps(lambda: layer.forward_fused(x, micro_batches=parts, reserved_sms=reserved), max(3, args.steps // 2), 2, torch, dist=dist)
        layer._all_reduce_enabled = True
        message = torch.empty(LAYER["batch"] * LAYER["seq"], cfg.d_model, dtype=torch.bfloat16, device=device)
        steps_half = max(3, args.steps // 2)
        reduce_ms, _ = timed_steps(lambda: dist.all_reduce(message), steps_half, 2, torch, dist=dist)
        switch_ms = float("nan")
        sums = layer.switch_sums(blocks=reserved)
        if sums is not None:      # the same whole-partial-sum message through the switch kernel, inside the layer's workspace
            region = layer._workspace[:message.numel() * 2].view(torch.bfloat16)
            switch_ms, _ = timed_steps(lambda: sums(region), steps_half, 2, torch, dist=dist, check=backend.poll)
        both = torch.tensor([compute_ms / steps_half, reduce_ms / steps_half, switch_ms / steps_half], device=device)
        dist.all_reduce(both, op=dist.ReduceOp.MAX)
        breakdown = {"compute_only_ms": both[0].item(), "nccl_allreduce_128MiB_ms": both[1].item(),
                     "switch_sum_128MiB_ms": both[2].item() if sums is not None else None, "sums_per_step": 2,
                     "exposed_ms": ms - both[0].item(),
                     "note": "compute_only_ms runs the layer with its sums left out and so with the two residual add kernels, which the timed step folds into its sums", "micro_batches": parts or layer.default_micro_batches(LAYER["batch"]), "reserved_sms": reserved}
        del message
    sum_kind = "one shard" if world == 1 else ("NVSwitch multimem kernel of the library" if layer.switch_sums(blocks=reserved) is not None else "NCCL all-reduce")
    return {"workload": f"decoder layer forward bf16 d4096 32/8 heads hd128 FFN14336, batch 8 x seq 2048, TP{world} (sum over shards after o-proj and down-proj: {sum_kind})",
            "sum_over_shards": sum_kind,
            "value": tflops, "unit": "TFLOP/s", "ms_per_step": ms, "scaling": "strong", "tokens_per_s": LAYER["batch"] * LAYER["seq"] / (ms * 1e-3),
            "kernels_per_step": 10, "collectives_per_step": 0 if world == 1 else 2,
            "breakdown": breakdown,
            "verified": bool(layer_err <= 1e-2), "max_rel_err": layer_err,
            "verified_against": "float64 torch recomputation of 8 sampled token rows from the full weights",
            "roofline": {"bound": "tensor", "achieved": tflops / world, "peak": peak["bf16_tflops_sustained"], "unit": "TFLOP/s per GPU",
                         "frac": tflops / world / peak["bf16_tflops_sustained"], "traffic": TRAFFIC["layer"] if world == 1 else None,
                         "peak_source": peak["source"] + " (sustained)"}}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = os.cpu_count() or 1
    for _ in range(min(args.warmup, 1)):
        cpu_sample(threads)
    seconds, flops, sample = 0.0, 0, ""
    t_all = []
    for _ in range(args.steps):
        sec, fl, sample = cpu_sample(threads)
        t_all.append(sec)
        flops = fl
    seconds = sum(t_all) / len(t_all)
    value = flops / seconds / 1e12
    line = {"impl": "reference", "metric": "fa_prefill_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "FA prefill bf16 B4 H32 S4096 D128 causal", "sample": sample},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "CPU restatement of the reference's numeric path (reference sources need LLVM/MLIR/SystemC: not buildable here)"}
    emit(line)
    return 0


def run_profile_case(name: str):
    """Three launches of one kernel on a case a few hundred MB large (above the 126 MB L2, far below a full-size
    workload) so that a multi-pass ncu capture ends within a minute or two. Prints nothing to parse."""
    import torch
    from vibe_compiler_b200 import _abi as abi
    from vibe_compiler_b200.backend import B200TargetModelBackend
    backend = B200TargetModelBackend(0)
    device = torch.device("cuda", 0)
    gen = torch.Generator(device=device).manual_seed(SEED)
    if name == "fa":       # batch 2 of the benchmark's 4: Q + K + V = 201 MB
        shape = (2, FA["heads"], FA["seq"], FA["head_dim"])
        q, k, v = (torch.randn(shape, device=device, generator=gen).bfloat16() for _ in range(3))
        fn = lambda: backend.attention_fa(q, k, v, FA["head_dim"] ** -0.5, True)
    elif name == "fd":     # batch 8 of the benchmark's 64: K + V = 1.07 GB
        q = torch.randn(8, FD["q_heads"], 1, FD["head_dim"], device=device, generator=gen).bfloat16()
        k = torch.randn(8, FD["kv_heads"], FD["kv_len"], FD["head_dim"], device=device, generator=gen).bfloat16()
        v = torch.randn(8, FD["kv_heads"], FD["kv_len"], FD["head_dim"], device=device, generator=gen).bfloat16()
        fn = lambda: backend.attention_fd(q, k, v, FD["head_dim"] ** -0.5)
    elif name == "layer":  # the decoder layer at the benchmark's shape, for single-pass captures (DRAM bytes) only
        from vibe_compiler_b200.decoder_layer import LayerConfig, ShardedDecoderLayer, random_weights
        cfg = LayerConfig()
        layer = ShardedDecoderLayer(backend, cfg, random_weights(cfg, seed=SEED), device=device)
        x = torch.randn(LAYER["batch"], LAYER["seq"], cfg.d_model, device=device, generator=gen).bfloat16()
        fn = lambda: layer.forward_fused(x)
    else:                  # 4096^3 of the benchmark's 8192^3: A + B + out = 100 MB; "gemm_full": 8192^3, single-pass captures only
        size = GEMM["m"] if name == "gemm_full" else 4096
        a = (torch.rand(size, size, device=device, generator=gen) * 2 - 1).bfloat16()
        b = (torch.rand(size, size, device=device, generator=gen) * 2 - 1).bfloat16()
        bias = torch.randn(size, device=device, generator=gen) * 0.02
        fn = lambda: backend.gemm_epilogue(a, b, bias, epilogue=abi.EPI_BIAS_GELU)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    backend.poll()
    print(f"profile case {name}: 3 launches done")
    return 0


def emit(line: dict):
    """The JSON line goes to the process's original stdout; everything else written to file descriptor 1 meanwhile
    (NCCL's version banner comes from C code) has been pointed at stderr by main()."""
    os.write(RESULT_FD, (json.dumps(line) + "\n").encode())


RESULT_FD = 1


def main():
    global RESULT_FD
    sys.stdout.flush()
    RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--skip-extras", action="store_true", help="only the headline FA workload")
    parser.add_argument("--profile-case", choices=["fa", "fd", "gemm", "gemm_full", "layer"],
                        help="run three launches of a reduced-size case of one kernel and exit (for ncu captures)")
    args = parser.parse_args()
    if args.profile_case:
        return run_profile_case(args.profile_case)
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(args.warmup, 3)

    import torch
    from vibe_compiler_b200 import _abi as abi
    from vibe_compiler_b200.backend import B200TargetModelBackend

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # Where the decoder layer falls back to NCCL for its sums, NCCL has to fit in the SMs the persistent kernels leave free.
        os.environ.setdefault("NCCL_MAX_CTAS", "16")
        torch.cuda.set_device(local_rank)
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    backend = B200TargetModelBackend(local_rank)
    peak = peaks()
    failures = []      # outputs that disagree with their recomputation: reported in the line, and the exit code is 1

    # ---------------------------------------------------------------- FA prefill (headline)
    # The fixed problem is 128 independent (batch, head) units; this rank owns a contiguous block of them, laid out as
    # the heads of one batch entry (each unit has its own K and V).
    from vibe_compiler_b200.sharding import unit_range
    gen = torch.Generator(device=device).manual_seed(SEED + rank)
    unit_begin, unit_end = unit_range(FA["batch"] * FA["heads"], world, rank)
    units = unit_end - unit_begin
    shape = (1, units, FA["seq"], FA["head_dim"]) if world > 1 else (FA["batch"], FA["heads"], FA["seq"], FA["head_dim"])
    q = torch.randn(shape, device=device, generator=gen).bfloat16()
    k = torch.randn(shape, device=device, generator=gen).bfloat16()
    v = torch.randn(shape, device=device, generator=gen).bfloat16()
    out = torch.empty_like(q)
    lse = torch.empty(shape[:3], device=device)
    scale = FA["head_dim"] ** -0.5
    flops = fa_flops(FA["batch"], FA["heads"], FA["seq"], FA["head_dim"])      # the whole problem
    rank_flops = fa_flops(1, units, FA["seq"], FA["head_dim"])                  # this rank's units

    q_bytes = q.numel() * 2
    # At 8 ranks a rank's Q + K + V (50 MB) fit the L2: write a buffer larger than the L2 between timed launches there.
    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=device) if 3 * q_bytes <= 126e6 else None

    def fa_step():
        backend.attention_fa(q, k, v, scale, True, out=out, lse=lse)

    launches_before = backend.launch_count
    with ClockSampler(local_rank) as sampler:
        total_ms, launch_ms = timed_steps(fa_step, args.steps, args.warmup, torch, dist, check=backend.poll, flush=flush)
    backend.poll()
    launches = backend.launch_count - launches_before - args.warmup
    times = torch.tensor([total_ms, launch_ms], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, launch_ms = times.tolist()
    ms_per_step = total_ms / args.steps
    value = flops / (ms_per_step * 1e-3) / 1e12
    achieved = rank_flops / (launch_ms * 1e-3) / 1e12    # per GPU (ranks own equal shares)

    # ---------------------------------------------------------------- e2e through host buffers
    e2e_steps = max(1, min(args.steps, 5))
    hq, hk, hv = (torch.empty(shape, dtype=torch.bfloat16).pin_memory() for _ in range(3))
    hq.copy_(q); hk.copy_(k); hv.copy_(v)
    hout = torch.empty(shape, dtype=torch.bfloat16).pin_memory()
    hlse = torch.empty(shape[:3], dtype=torch.float32).pin_memory()
    backend.attention_fa(hq, hk, hv, scale, True, out=hout, lse=hlse)   # warm-up (allocates staging)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        backend.attention_fa(hq, hk, hv, scale, True, out=hout, lse=hlse)   # synchronous: returns after D2H
    e2e_seconds = torch.tensor([(time.perf_counter() - t0) / e2e_steps], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(e2e_seconds, op=dist.ReduceOp.MAX)
    e2e_value = flops / e2e_seconds.item() / 1e12
    h2d = world * 3 * q.numel() * 2
    d2h = world * (out.numel() * 2 + lse.numel() * 4)
    assert torch.equal(hout.view(torch.int16), out.cpu().view(torch.int16)), "host-buffer path disagrees with device path"
    del hq, hk, hv, hout, hlse, flush

    extras = {}
    if not args.skip_extras:
        q = k = v = out = None
        torch.cuda.empty_cache()
    if not args.skip_extras:
        # ------------------------------------------------------------ FD decode (HBM bound): the fixed batch of 64 sequences is
        # dealt out in contiguous blocks (64 / N sequences = 512 / N (batch, kv-head) units per rank), no collective
        seq_begin, seq_end = unit_range(FD["batch"], world, rank)
        fd_batch = seq_end - seq_begin
        fq = torch.randn(fd_batch, FD["q_heads"], 1, FD["head_dim"], device=device, generator=gen).bfloat16()
        fk = torch.randn(fd_batch, FD["kv_heads"], FD["kv_len"], FD["head_dim"], device=device, generator=gen).bfloat16()
        fv = torch.randn(fd_batch, FD["kv_heads"], FD["kv_len"], FD["head_dim"], device=device, generator=gen).bfloat16()
        fout = torch.empty_like(fq)
        flse = torch.empty(fd_batch, FD["q_heads"], 1, device=device)
        fd_bytes = 2 * fk.numel() * 2                 # this rank's K + V
        fd_total, fd_launch = timed_steps(lambda: backend.attention_fd(fq, fk, fv, scale, out=fout, lse=flse), args.steps, args.warmup, torch, dist, check=backend.poll)
        backend.poll()
        fd_times = torch.tensor([fd_total, fd_launch], device=device, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(fd_times, op=dist.ReduceOp.MAX)
        fd_ms, fd_launch_ms = fd_times[0].item() / args.steps, fd_times[1].item()
        fd_gbs = fd_bytes / (fd_launch_ms * 1e-3) / 1e9
        extras["fd_decode"] = {"workload": f"FD decode bf16 B64 Hq32 Hkv8 KV32768 D128, 64 sequences dealt over {world} rank(s); per-rank K + V ({fd_bytes / 1e9:.1f} GB) larger than L2",
                               "value": world * fd_bytes / (fd_ms * 1e-3) / 1e9,
                               "unit": "GB/s", "ms_per_step": fd_ms, "scaling": "strong", "n_gpus": world,
                               "roofline": {"bound": "hbm", "achieved": fd_gbs, "peak": peak["hbm_gbs"], "unit": "GB/s per GPU",
                                            "frac": fd_gbs / peak["hbm_gbs"], "traffic": TRAFFIC["fd"] * fd_batch / FD["batch"], "peak_source": peak["source"], "launch_ms": fd_launch_ms}}
        del fq, fk, fv
        torch.cuda.empty_cache()
        # ------------------------------------------------------------ long-context decode: the KV sequence is sharded over the ranks
        from vibe_compiler_b200.sharding import sequence_range
        lo, hi = sequence_range(FD_LONG["kv_len"], world, rank)
        shared_gen = torch.Generator(device=device).manual_seed(SEED + 77)   # the query is the same on every rank
        lq = torch.randn(1, FD_LONG["q_heads"], 1, FD_LONG["head_dim"], device=device, generator=shared_gen).bfloat16()
        lk = torch.randn(1, FD_LONG["kv_heads"], hi - lo, FD_LONG["head_dim"], device=device, generator=gen).bfloat16()
        lv = torch.randn(1, FD_LONG["kv_heads"], hi - lo, FD_LONG["head_dim"], device=device, generator=gen).bfloat16()
        lout = torch.empty_like(lq)
        group = None
        # One step = stage 1 over this rank's KV shard + one kernel that folds the splits, exchanges the per-head states
        # with plain peer stores over NVLink and merges them in ascending shard order. No collective library call, so
        # the two launches replay as one CUDA graph at every world size.
        from vibe_compiler_b200.sharding import PeerExchange
        exchange = PeerExchange(backend, 1, FD_LONG["q_heads"], group, device)
        long_lse = torch.empty(1, FD_LONG["q_heads"], 1, device=device)

        def long_step():
            backend.attention_fd_exchange(lq, lk, lv, scale, rank=exchange.rank, peer_pointers=exchange.pointers, epoch=exchange.epoch,
                                          out=lout, lse=long_lse)
        for _ in range(2):      # sizes the library's scratch before the capture
            long_step()
        torch.cuda.synchronize()
        backend.poll()
        eager_out = lout.clone()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                long_step()
        torch.cuda.current_stream().wait_stream(side)
        if dist is not None:
            dist.barrier()          # every rank has captured before anyone replays (a replay waits for the peers' kernels)
        graph.replay()
        torch.cuda.synchronize()
        backend.poll()
        assert torch.equal(eager_out, lout), "graph replay of the decode step disagrees with the eager step"
        step = graph.replay
        long_total, _ = timed_steps(step, args.steps, args.warmup, torch, dist, check=backend.poll)
        backend.poll()
        long_t = torch.tensor([long_total], device=device, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(long_t, op=dist.ReduceOp.MAX)
        long_ms = long_t.item() / args.steps
        long_bytes = 2 * FD_LONG["kv_heads"] * FD_LONG["kv_len"] * FD_LONG["head_dim"] * 2
        long_gbs = long_bytes / (long_ms * 1e-3) / 1e9
        # Check what was timed: every rank recomputes the state of its own KV shard in float64 with torch operators, the
        # states are gathered and merged in float64, and the library's output (this rank's copy) is compared with that.
        from vibe_compiler_b200 import selfcheck
        graph.replay()
        torch.cuda.synchronize()
        backend.poll()
        m64, l64, acc64 = selfcheck.decode_state_f64(lq, lk, lv, scale)
        packed = torch.cat([m64[..., None], l64[..., None], acc64], -1).contiguous()          # [1, Hq, D + 2] float64
        all_packed = [torch.empty_like(packed) for _ in range(world)]
        if dist is not None:
            dist.all_gather(all_packed, packed)
        else:
            all_packed = [packed]
        want_out, want_lse = selfcheck.merge_states_f64([(t[..., 0], t[..., 1], t[..., 2:]) for t in all_packed])
        long_err = selfcheck.max_rel_err(lout.view(1, FD_LONG["q_heads"], FD_LONG["head_dim"]), want_out)
        long_lse_err = float((long_lse.view(1, -1).double() - want_lse).abs().max())
        long_ok = long_err <= 1e-2 and long_lse_err <= 1e-3
        if not long_ok:
            failures.append(f"fd_long_context: max rel err {long_err:.3e}, lse abs err {long_lse_err:.3e} on rank {rank}")
        extras["fd_long_context"] = {"workload": f"FD decode bf16 B1 Hq32 Hkv8 KV1048576 D128, KV sequence sharded over {world} rank(s); exchange of (acc, m, l) states by peer stores inside the merge kernel; the step replays as one CUDA graph",
                                     "value": long_gbs, "unit": "GB/s", "ms_per_step": long_ms, "scaling": "strong", "n_gpus": world,
                                     "exchange_bytes_per_rank": FD_LONG["q_heads"] * (FD_LONG["head_dim"] + 2) * 4,
                                     "verified": long_ok, "max_rel_err": long_err, "lse_abs_err": long_lse_err,
                                     "verified_against": "float64 torch recomputation of every rank's shard, merged in float64",
                                     "roofline": {"bound": "hbm", "achieved": long_gbs / world, "peak": peak["hbm_gbs"], "unit": "GB/s per GPU",
                                                  "frac": long_gbs / world / peak["hbm_gbs"],
                                                  "traffic": long_bytes / world * TRAFFIC["fd"] / (FD["batch"] * 2 * FD["kv_heads"] * FD["kv_len"] * FD["head_dim"] * 2),
                                                  "traffic_note": "the same stage-1 kernel as the decode configuration: its captured DRAM bytes per algorithmic byte, times this rank's K and V bytes",
                                                  "peak_source": peak["source"]}}
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()          # no rank releases its exchange buffer while a peer may still write to it
        del lk, lv, graph, step, exchange
        torch.cuda.empty_cache()
    if not args.skip_extras and world == 1:
        # ------------------------------------------------------------ GEMM + bias + GELU (tensor bound)
        ga = (torch.rand(GEMM["m"], GEMM["k"], device=device, generator=gen) * 2 - 1).bfloat16()
        gb = (torch.rand(GEMM["k"], GEMM["n"], device=device, generator=gen) * 2 - 1).bfloat16()
        gbias = torch.randn(GEMM["n"], device=device, generator=gen) * 0.02
        gout = torch.empty(GEMM["m"], GEMM["n"], device=device, dtype=torch.bfloat16)
        _, g_ms = timed_steps(lambda: backend.gemm_epilogue(ga, gb, gbias, epilogue=abi.EPI_BIAS_GELU, out=gout), args.steps, args.warmup, torch, check=backend.poll)
        backend.poll()
        g_tflops = 2 * GEMM["m"] * GEMM["n"] * GEMM["k"] / (g_ms * 1e-3) / 1e12
        extras["gemm_bias_gelu"] = {"workload": "GEMM 8192^3 bf16 + f32 bias + GELU(erf) -> bf16", "value": g_tflops, "unit": "TFLOP/s",
                                    "ms_per_step": g_ms,
                                    "roofline": {"bound": "tensor", "achieved": g_tflops, "peak": peak["bf16_tflops"], "unit": "TFLOP/s",
                                                 "frac": g_tflops / peak["bf16_tflops"], "traffic": TRAFFIC["gemm"], "peak_source": peak["source"]}}

    if not args.skip_extras and world == 1:
        # ------------------------------------------------------------ cfg 1: the reference's own CPU-runnable attention case
        # (f32, batch 1, 8 heads, seq 512, head_dim 64, non-causal): latency bound, half a GFLOP; reported with its parity error.
        c1 = torch.Generator(device=device).manual_seed(SEED + 1)
        q1, k1, v1 = (torch.randn(1, 8, 512, 64, device=device, generator=c1) for _ in range(3))
        o1 = torch.empty_like(q1)
        flush1 = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=device)
        _, c1_ms = timed_steps(lambda: backend.attention_fa(q1, k1, v1, 0.125, False, out=o1), args.steps, args.warmup, torch, check=backend.poll, flush=flush1)
        backend.poll()
        ref1 = torch.nn.functional.scaled_dot_product_attention(q1.double(), k1.double(), v1.double())
        c1_flops = 4 * 8 * 512 * 512 * 64
        extras["fa_f32_cfg1"] = {"workload": "attention f32 B1 H8 S512 D64 non-causal (the reference's CPU-runnable case); L2 flushed between launches",
                                 "value": c1_flops / (c1_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": c1_ms,
                                 "max_rel_err_vs_f64": float((o1.double() - ref1).abs().max() / ref1.abs().max()),
                                 "roofline": {"bound": "latency", "achieved": c1_flops / (c1_ms * 1e-3) / 1e12, "peak": None, "unit": "TFLOP/s", "frac": None,
                                              "traffic": None, "note": "0.5 GFLOP on 1024 warps: launch and dependency latency, not a pipe, bound it"}}
        del flush1
    if not args.skip_extras:
        ga = gb = gout = fk = fv = None
        torch.cuda.empty_cache()
        extras["decoder_layer"] = layer_extra(backend, args, torch, dist, rank, world, device, peak, failures)

    if rank == 0:
        cpu_threads = os.cpu_count() or 1
        cpu_seconds, cpu_flops, cpu_desc = cpu_sample(cpu_threads) if world == 1 else (None, None, None)
        # the reference runs its numeric path on one OS thread (sequential oneDNN, SystemC coroutines): one unit, one thread
        one_seconds, one_flops, one_desc = cpu_sample(1, units=1) if world == 1 else (None, None, None)
        line = {
            "metric": "fa_prefill_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "FA prefill bf16 B4 H32 S4096 D128 causal (+f32 LSE)", "batch": FA["batch"], "heads": FA["heads"],
                       "seq_len": FA["seq"], "head_dim": FA["head_dim"], "causal": True,
                       "flops_per_step": flops, "units_per_rank": units, "flops_counting": "visible (query,key) pairs only",
                       "l2": f"per-rank inputs (Q+K+V {3 * q_bytes / 1e6:.0f} MB)" + (" larger than the 126 MB L2" if 3 * q_bytes > 126e6 else
                                                                                     " fit the 126 MB L2: a buffer larger than L2 is written between timed launches"),
                       "parallelism": f"the 128 independent (batch, head) units dealt over {world} rank(s), no collective"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak["bf16_tflops"], "unit": "TFLOP/s per GPU",
                         "frac": achieved / peak["bf16_tflops"], "traffic": TRAFFIC["fa"] * units / (FA["batch"] * FA["heads"]), "peak_source": peak["source"],
                         "frac_of_sustained": achieved / peak["bf16_tflops_sustained"], "launch_ms": launch_ms},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps},
            "gpu_launches": launches,
            "clocks": sampler.result,
        }
        if cpu_seconds is not None:
            line["cpu_baseline"] = {"value": cpu_flops / cpu_seconds / 1e12, "unit": "TFLOP/s", "cores": cpu_threads, "kind": "port",
                                    "sample": cpu_desc, "seconds": cpu_seconds,
                                    "single_thread": {"value": one_flops / one_seconds / 1e12, "unit": "TFLOP/s", "cores": 1, "sample": one_desc,
                                                      "seconds": one_seconds}}
        if cpu_seconds is not None and not args.skip_extras:
            for name, baseline in cpu_baselines(cpu_threads).items():
                if name in extras:
                    extras[name]["cpu_baseline"] = baseline
        line.update(extras)
        if failures:
            line["failures"] = failures
        emit(line)
    bad = torch.tensor([1 if failures else 0], device=device)
    if dist is not None:
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        dist.barrier()
        dist.destroy_process_group()
    if failures:
        print("\n".join(failures), file=sys.stderr)
    return 1 if bad.item() else 0


if __name__ == "__main__":
    sys.exit(main())
