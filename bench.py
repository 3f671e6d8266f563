#!/usr/bin/env python
"""Benchmark of the headline hot path: bf16 batched GEMM [64,2048,4096] x [4096,4096] with fp32
accumulation and bf16 output (the second configuration of BASELINE.json), through the C ABI.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one pass of the GEMM over one batch of 64 matrices. With N > 1 (launched by
torch.distributed.run, one rank per GPU) every rank multiplies its own 64-matrix shard of a
64*N batch: batch items are independent, there is no collective on the data path, and the value
is the whole job's TFLOP/s (weak scaling). Prints ONE JSON line on rank 0.

`--impl reference` times the reference's own CPU implementation (oracle/_ref when it is built,
else the plain-C oracle port) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

BATCH, M, K, N = 64, 2048, 4096, 4096
FLOPS_PER_STEP = 2.0 * BATCH * M * K * N          # 4 398 046 511 104
# dram__bytes_read.sum + dram__bytes_write.sum per launch, from the ncu capture summarised under profiles/
TRAFFIC_BYTES_PER_LAUNCH = 2.048e9
WORKLOAD = "configs[1]: bf16 batched GEMM A[64,2048,4096] . B[4096,4096], fp32 accumulate, bf16 out"


def make_config(world: int) -> dict:
    return {"workload": WORKLOAD, "global_batch": BATCH * world, "m": M, "k": K, "n": N,
            "parallelism": f"batch-sharded x{world}, no collective",
            "l2": "inputs larger than L2 (A is 1.07 GB per step), no flush needed"}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "hbm_gbs": d["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, interval_ms: int = 100):
        self.idx = gpu_index
        self.interval_ms = interval_ms
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", str(self.interval_ms),
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------------------- reference arm
def reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from oracle import oracle as O

    kind = "reference" if O.ref_available() else "port"
    cores = os.cpu_count() or 1
    if kind == "reference":
        os.environ.setdefault("OMP_NUM_THREADS", str(cores))
        os.environ.setdefault("OMP_PROC_BIND", "close")
        be = O.ref(threads=cores)
        cores = be.threads()
    else:
        be = O.port()
    rng = np.random.default_rng(1)
    items = 1  # batch items per step: a bounded sample of the 64-item workload
    a = be.f32_to_bf16(rng.standard_normal((items, M, K)).astype(np.float32))
    b = be.f32_to_bf16((rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32))
    for _ in range(min(args.warmup, 1)):
        be.matmul_16(a, b, 1)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        be.matmul_16(a, b, 1)
    dt = (time.perf_counter() - t0) / args.steps
    tfl = 2.0 * items * M * K * N / dt / 1e12
    sample = (f"{items} of {BATCH} batch items per step (widen bf16->f32, YTensor<float>::matmul AVX2, narrow with "
              f"yt::bfloat16), {args.steps} steps, scaled by FLOPs")
    print(json.dumps({
        "impl": "reference", "metric": "bf16_gemm_tflops", "value": tfl, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3 * (BATCH / items),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 compute on bf16 storage",
        "data": "synthetic", "config": make_config(args.gpus),
        "cpu_baseline": {"value": tfl, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": tfl, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def cpu_baseline(budget_s: float = 12.0) -> dict:
    """Times the reference CPU path on a bounded sample (rank 0, N = 1 only)."""
    import numpy as np
    from oracle import oracle as O

    kind = "reference" if O.ref_available() else "port"
    cores = os.cpu_count() or 1
    be = O.ref(threads=cores) if kind == "reference" else O.port()
    if kind == "reference":
        cores = be.threads()
    rng = np.random.default_rng(1)
    a = be.f32_to_bf16(rng.standard_normal((1, M, K)).astype(np.float32))
    b = be.f32_to_bf16((rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32))
    be.matmul_16(a[:, :256], b, 1)  # warm the thread pool
    t0 = time.perf_counter()
    be.matmul_16(a, b, 1)
    one = time.perf_counter() - t0
    reps = max(1, min(8, int(budget_s / max(one, 1e-3)) - 1))
    t0 = time.perf_counter()
    for _ in range(reps):
        be.matmul_16(a, b, 1)
    dt = (time.perf_counter() - t0) / reps
    return {"value": 2.0 * M * K * N / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": kind,
            "sample": f"1 of {BATCH} batch items (2048x4096x4096), best-effort mean of {reps} runs, scaled by FLOPs"}


# --------------------------------------------------------------------------------------- device arm
def end_to_end(args, L, a, b, c, world, dev, barrier):
    """Host buffers through ytcuda_gemm_host: H2D of A and B and D2H of C inside every timed step."""
    import torch
    import torch.distributed as dist

    from ytensor_b200 import _lib

    e2e_steps = max(2, min(args.steps, 5))
    ha = torch.empty(BATCH, M, K, dtype=torch.bfloat16, pin_memory=True)
    hb = torch.empty(K, N, dtype=torch.bfloat16, pin_memory=True)
    hc = torch.empty(BATCH, M, N, dtype=torch.bfloat16, pin_memory=True)
    ha.copy_(a)
    hb.copy_(b)

    def host_step():
        _lib.check(L.ytcuda_gemm_host(_lib.BF16, _lib.BF16, ha.data_ptr(), hb.data_ptr(), hc.data_ptr(), M, N, K, 1.0,
                                      0.0, K, 1, N, 1, N, 1, BATCH, M * K, 0, M * N))

    host_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        host_step()
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t.item())
    same = bool(torch.equal(hc[BATCH - 1], c[BATCH - 1].cpu()))
    e2e = {"value": FLOPS_PER_STEP * world / e2e_s / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": (ha.numel() + hb.numel()) * 2, "d2h_bytes_per_step": hc.numel() * 2,
           "ms_per_step": e2e_s * 1e3, "steps": e2e_steps, "matches_device_result": same,
           "api": "ytcuda_gemm_host (pinned host buffers)"}
    return e2e


def device_arm(args) -> None:
    import torch
    import torch.distributed as dist

    from ytensor_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the device backend has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    L = _lib.lib()
    dev = torch.device("cuda", local)
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    # plumbing only: torch provides device memory and the synthetic draw; the GEMM is ytcuda_gemm
    a = torch.randn(BATCH, M, K, device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    b = (torch.randn(K, N, device=dev, generator=g, dtype=torch.float32) / K ** 0.5).to(torch.bfloat16)
    c = torch.empty(BATCH, M, N, device=dev, dtype=torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream

    def step():
        _lib.check(L.ytcuda_gemm(_lib.BF16, _lib.BF16, a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, 1.0, 0.0,
                                 K, 1, N, 1, N, 1, BATCH, M * K, 0, M * N, stream))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = L.ytcuda_launch_count()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    evs[0].record()
    for i in range(args.steps):
        step()
        evs[i + 1].record()
    barrier()
    total_ms = evs[0].elapsed_time(evs[-1])
    per_launch_ms = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
    launches = L.ytcuda_launch_count() - launches0
    _lib.check(L.ytcuda_device_status(None))
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = FLOPS_PER_STEP * world / (ms_per_step * 1e-3) / 1e12

    e2e = None
    if not args.no_e2e:
        e2e = end_to_end(args, L, a, b, c, world, dev, barrier)

    if rank == 0:
        peaks = measured_peaks()
        avg_launch_ms = statistics.mean(per_launch_ms)
        achieved = FLOPS_PER_STEP / (avg_launch_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["bf16_tflops"], "traffic": TRAFFIC_BYTES_PER_LAUNCH if BATCH == 64 else None,
                    "traffic_note": "ncu dram read+write of a batch-8 capture scaled to batch 64 (A and C x8, B once); "
                                    "see profiles/gemm_tc_kernel_bf16_config2.md",
                    "kernel": "gemm_tc2_kernel (cta_group::2, 256x256 tile per CTA pair)", "peak_source": f"{peaks['source']} (burst cuBLAS bf16)",
                    "frac_of_sustained_peak": (achieved / peaks["bf16_tflops_sustained"]
                                               if peaks.get("bf16_tflops_sustained") else None),
                    "algorithmic_flops_per_launch": FLOPS_PER_STEP}
        out = {
            "metric": "bf16_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": make_config(world),
            "roofline": roofline, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline()
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------- other configs
def _time_steps(torch, fn, steps, warmup):
    for _ in range(max(warmup, 3)):
        fn()
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    evs[0].record()
    for i in range(steps):
        fn()
        evs[i + 1].record()
    torch.cuda.synchronize()
    return [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]


def attention_arm(args) -> None:
    """BASELINE configs[2]: causal flash attention bf16, batch 16, 32 q / 8 kv heads, head_dim 128, seq 4096.
    `--batch` shrinks the batch for profiling captures. Single GPU; prints one JSON line."""
    import torch

    from ytensor_b200 import _lib, api

    torch.cuda.set_device(0)
    L = _lib.lib()
    B = 16 if args.batch == 64 else args.batch
    H, KVH, S, D = 32, 8, 4096, 128
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(B, H, S, D, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(B, KVH, S, D, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(B, KVH, S, D, device="cuda", generator=g).to(torch.bfloat16)
    flops = 4.0 * B * H * S * S * D / 2  # causal convention: half of the square
    sampler = ClockSampler(0)
    sampler.start()
    n0 = L.ytcuda_launch_count()
    ts = _time_steps(torch, lambda: api.scaledDotProductAttention(q, k, v, causal=True), args.steps, args.warmup)
    launches = L.ytcuda_launch_count() - n0 - max(args.warmup, 3)
    clocks = sampler.stop()
    _lib.check(L.ytcuda_device_status(None))
    peaks = measured_peaks()
    ms = statistics.mean(ts)
    val = flops / (ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": "flash_attn_causal_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"configs[2]: causal flash attention bf16, batch {B}, 32 q / 8 kv heads, head_dim 128, "
                               f"seq 4096" + ("" if B == 16 else " (PROFILING CASE: reduced batch)"),
                   "l2": "inputs larger than L2 (Q alone is 33.5 MB per batch item)"},
        "roofline": {"bound": "tensor", "achieved": val, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": val / peaks["bf16_tflops"], "traffic": None, "kernel": "flash_tc_kernel<128>",
                     "peak_source": f"{peaks['source']} (burst cuBLAS bf16)",
                     "algorithmic_flops_per_launch": flops, "non_causal_equivalent_tflops": 2 * val},
        "gpu_launches": int(launches), "clocks": clocks}))


def gemm32_arm(args) -> None:
    """BASELINE configs[0]: fp32 GEMM 1024 x 1024 x 1024 (the reference's own CPU-runnable case). The device forms
    the product on the tensor cores from three bf16 planes per operand (six partial products side by side along k, one
    GEMM launch); the L2 is flushed
    between steps because the 12.6 MB of operands would otherwise stay cached. Single GPU; one JSON line."""
    import torch

    from ytensor_b200 import _lib, api

    torch.cuda.set_device(0)
    L = _lib.lib()
    n = 1024
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn(n, n, device="cuda", generator=g)
    b = torch.randn(n, n, device="cuda", generator=g)
    c = torch.empty(n, n, device="cuda")
    flush = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")  # larger than the 126 MB L2
    flops = 2.0 * n * n * n
    res = {}
    for name, mode in (("tensor cores (3 x bf16 planes, 6 products)", 0), ("FFMA kernel", 1)):
        L.ytcuda_gemm_set_f32_mode(mode)
        for _ in range(max(args.warmup, 3)):
            api.matmul(a, b, c)
        ts = []
        n0 = L.ytcuda_launch_count()
        for _ in range(args.steps):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            api.matmul(a, b, c)
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        res[name] = (statistics.median(ts), (L.ytcuda_launch_count() - n0) // args.steps)
    L.ytcuda_gemm_set_f32_mode(0)
    _lib.check(L.ytcuda_device_status(None))
    peaks = measured_peaks()
    ms, launches = res["tensor cores (3 x bf16 planes, 6 products)"]
    val = flops / (ms * 1e-3) / 1e12
    peak = peaks["bf16_tflops"] / 6.0
    print(json.dumps({
        "metric": "fp32_gemm_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 (three bf16 planes per operand, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": "configs[0]: fp32 GEMM 1024 x 1024 x 1024", "l2": "flushed between steps (192 MB write)"},
        "roofline": {"bound": "tensor", "achieved": val, "peak": peak, "unit": "TFLOP/s", "frac": val / peak,
                     "traffic": None, "kernel": "gemm_tc_kernel over k' = 6 k + gemm_split3_kernel (two launches)",
                     "peak_source": f"{peaks['source']} (burst cuBLAS bf16 / 6 partial products)",
                     "algorithmic_flops_per_launch": flops},
        "ffma_kernel": {"ms_per_step": res["FFMA kernel"][0], "tflops": flops / (res["FFMA kernel"][0] * 1e-3) / 1e12},
        "gpu_launches": int(launches * args.steps), "clocks": None}))


def chain_arm(args) -> None:
    """BASELINE configs[3]: y = bf16(softmax(rmsNorm(x, w, -1, 1e-6) + r, -1)) on x [32,4096,4096] fp32 with the
    residual [1,4096,4096] shared by the batch. `--batch` shrinks the batch for profiling captures."""
    import torch

    from ytensor_b200 import _lib, api

    torch.cuda.set_device(0)
    L = _lib.lib()
    B = 32 if args.batch == 64 else args.batch
    R, H = 4096, 4096
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(B, R, H, device="cuda", generator=g)
    w = torch.rand(H, device="cuda", generator=g) * 0.2 + 0.9
    r = torch.randn(1, R, H, device="cuda", generator=g)
    algo_bytes = x.numel() * 4 + r.numel() * 4 + H * 4 + x.numel() * 2
    sampler = ClockSampler(0)
    sampler.start()
    n0 = L.ytcuda_launch_count()
    ts = _time_steps(torch, lambda: api.rmsnorm_add_softmax_cast(x, w, r), args.steps, args.warmup)
    launches = L.ytcuda_launch_count() - n0 - max(args.warmup, 3)
    clocks = sampler.stop()
    peaks = measured_peaks()
    ms = statistics.mean(ts)
    val = algo_bytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "memory_chain_gbs", "value": val, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 in, bf16 out", "data": "synthetic",
        "config": {"workload": f"configs[3]: RMSNorm + broadcast residual + row softmax + cast on [{B},4096,4096]"
                               + ("" if B == 32 else " (PROFILING CASE: reduced batch)"),
                   "l2": "inputs larger than L2 (x is 2.1 GB)"},
        "roofline": {"bound": "hbm", "achieved": val, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": val / peaks["hbm_gbs"], "traffic": None, "kernel": "chain_fast_kernel<4>",
                     "peak_source": f"{peaks['source']} (copy bandwidth)", "algorithmic_bytes_per_launch": algo_bytes},
        "gpu_launches": int(launches), "clocks": clocks}))


def decode_arm(args) -> None:
    """BASELINE configs[4]: random-init decoder of the Qwen3-0.6B shape, 512-token prompt, greedy decode of 256
    tokens. `--batch` = sequences (1 or 32; the default 64 of the GEMM workload means 1 here). Under
    torch.distributed.run the ranks form one tensor-parallel group (total work fixed: strong scaling).
    value = decoded tokens per second over all sequences; the prompt pass is reported next to it."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from ytensor_b200 import _lib
    from ytensor_b200 import qwen3 as Q

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    L = _lib.lib()
    B = 1 if args.batch == 64 else args.batch
    prompt_len, new_tokens = 512, (256 if args.steps == 100 else args.steps)
    cfg = Q.Qwen3Config(max_position_embeddings=prompt_len + new_tokens)
    m = Q.Qwen3ForCausalLM(cfg, batch=B, tp_rank=rank, tp_world=world)
    m.load_weights(Q.random_weights(cfg, seed=4))
    prompt_host = torch.from_numpy(np.random.default_rng(4).integers(0, cfg.vocab_size, (B, prompt_len))
                                   .astype(np.int32)).pin_memory()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run():
        m.reset_kv_cache()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev[0].record()
        ids = prompt_host.cuda(non_blocking=True)           # H2D of the step's input
        logits = m.forward(ids)
        tok, _ = m.argmax(logits)
        ev[1].record()
        out = [tok]
        for _ in range(new_tokens - 1):
            logits = m.forward(tok.reshape(B, 1).contiguous())
            tok, _ = m.argmax(logits)
            out.append(tok)
        ev[2].record()
        toks = torch.stack(out, 1).cpu()                     # D2H of the result
        torch.cuda.synchronize()
        return ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2]), toks

    run()  # warm-up: allocations, first-use attributes
    barrier()
    # a slow sampling period: every nvidia-smi query briefly holds the driver and delays kernel launches,
    # which a launch-bound decode loop feels
    sampler = ClockSampler(local, interval_ms=1000 if not args.no_clock_sampling else 10 ** 6)
    if rank == 0 and not args.no_clock_sampling:
        sampler.start()
    n0 = L.ytcuda_launch_count()
    t0 = time.perf_counter()
    prefill_ms, decode_ms, toks = run()
    barrier()
    wall = time.perf_counter() - t0
    launches = L.ytcuda_launch_count() - n0
    clocks = sampler.stop() if (rank == 0 and not args.no_clock_sampling) else None
    t = torch.tensor([prefill_ms, decode_ms, wall], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    prefill_ms, decode_ms, wall = (float(v) for v in t)
    if rank == 0:
        peaks = measured_peaks()
        steps = new_tokens - 1
        tok_s = B * steps / (decode_ms * 1e-3)
        params = 28 * 15728640 + 151936 * 1024
        bytes_per_step = params * 2 / world
        achieved = bytes_per_step / (decode_ms * 1e-3 / steps) / 1e9
        print(json.dumps({
            "metric": "decode_tokens_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": new_tokens,
            "warmup": 1, "ms_per_step": decode_ms / steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16 weights, f32 activations", "data": "synthetic",
            "config": {"workload": "configs[4]: Qwen3-0.6B-shape decoder, random bf16 weights, prompt 512, greedy decode",
                       "batch": B, "new_tokens": new_tokens, "parallelism": f"tp{world}",
                       "l2": "weights (1.19 GB) larger than L2"},
            "prefill_tokens_per_s": B * prompt_len / (prefill_ms * 1e-3), "prefill_ms": prefill_ms,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                         "kernel": ("decode_step_kernel (FFMA linear phases)" if B <= 4 else
                                    "decode_step_kernel (mma.sync linear phases)" if B <= (6 if world == 1 else 8) else
                                    "gemm_tc_kernel (hi + lo planes, split-k pieces) + fused glue kernels"),
                         "peak_source": f"{peaks['source']} (copy bandwidth)",
                         "algorithmic_bytes_per_launch": bytes_per_step,
                         "note": "bytes of this rank's bf16 weights streamed once per decode step / step time"},
            "e2e": {"value": B * new_tokens / wall, "unit": "tok/s", "h2d_bytes_per_step": int(prompt_host.numel() * 4),
                    "d2h_bytes_per_step": int(toks.numel() * 4),
                    "note": "prompt H2D + prefill + decode + tokens D2H, wall clock, generated tokens / s"},
            "gpu_launches": int(launches), "clocks": clocks, "first_tokens": toks[0, :8].tolist()}))
    m.close()
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    global BATCH, FLOPS_PER_STEP, WORKLOAD
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemm", choices=["gemm", "gemm32", "attn", "chain", "decode"],
                    help="gemm (default) is the headline bench line; gemm32, attn, chain and decode measure "
                         "configs[0], [2], [3] and [4]")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-clock-sampling", action="store_true", help="decode workload: do not run nvidia-smi beside it")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling captures only)")
    ap.add_argument("--batch", type=int, default=BATCH,
                    help="batch items per step; anything but 64 is a profiling case, not a bench line")
    args = ap.parse_args()
    if args.workload == "gemm32":
        return gemm32_arm(args)
    if args.workload == "attn":
        return attention_arm(args)
    if args.workload == "chain":
        return chain_arm(args)
    if args.workload == "decode":
        return decode_arm(args)
    if args.batch != BATCH:
        BATCH = args.batch
        FLOPS_PER_STEP = 2.0 * BATCH * M * K * N
        WORKLOAD = f"PROFILING CASE (batch {BATCH}, not configs[1]): bf16 GEMM A[{BATCH},2048,4096] . B[4096,4096]"
    if args.impl == "reference":
        reference_arm(args)
    else:
        device_arm(args)


if __name__ == "__main__":
    main()
