#!/usr/bin/env python
"""Benchmark of the dense hot path through the C ABI of libytensor_cuda.so.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME] [--no-secondary]

The headline line is the bf16 batched GEMM [64,2048,4096] x [4096,4096] with fp32 accumulation and bf16 output.
One "step" is one pass of that GEMM over the 64 matrices. With N > 1 (launched by torch.distributed.run, one rank
per GPU) the 64 matrices are SPLIT over the ranks (64 / N each): batch items are independent, there is no collective
on the data path, and the value is the whole job's TFLOP/s (strong scaling).

The same JSON line carries a "secondary" array with the other workloads the metric names, each with its own
roofline, end-to-end (host buffers) and CPU-baseline legs:
  attn      causal flash attention bf16, batch 16, 32 q / 8 kv heads, head_dim 128, seq 4096
            (N > 1: the 128 batch x kv-head units are split over the ranks, no collective)
  decode    Qwen3-0.6B-shape decoder, prompt 512, greedy decode of 256 tokens, batch 1 and batch 32
            (N > 1: the ranks form ONE tensor-parallel group of size N)
  chain     rmsNorm + broadcast residual + row softmax + bf16 cast on [32,4096,4096] fp32   (N = 1 only)
  gemm32    fp32 GEMM 1024^3                                                                (N = 1 only)
  gemm_weak the headline GEMM with 64 matrices PER RANK                                     (N > 1 only)
Every secondary workload runs in a child process of its own (same rank environment, its own rendezvous port), so a
failure there is recorded in its entry and cannot take the headline with it.

`--impl reference` times the reference's own CPU implementation (the unmodified reference compiled into
oracle/_ref when that is built, else the plain-C oracle port) on bounded samples of the same workloads.
Prints ONE JSON line on rank 0.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one launch over 64 matrices (ncu capture of 8 matrices: A and C
# scale with the batch, B is read once)
GEMM_TRAFFIC_64 = 2.048e9
GEMM_WORKLOAD = "configs[1]: bf16 batched GEMM A[64,2048,4096] . B[4096,4096], fp32 accumulate, bf16 out"


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


class Dist:
    """Rank plumbing: one process per GPU under torch.distributed.run, or a single process."""

    def __init__(self):
        import torch
        self.torch = torch
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the device backend has no CPU fallback")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.dist = None
        if self.world > 1:
            import datetime

            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev, timeout=datetime.timedelta(seconds=120))
            self.dist = dist

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.dist:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, *vals):
        t = self.torch.tensor(list(vals), device=self.dev, dtype=self.torch.float64)
        if self.dist:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def gather(self, val: float) -> list[float]:
        t = self.torch.tensor([val], device=self.dev, dtype=self.torch.float64)
        if not self.dist:
            return [float(val)]
        out = [self.torch.empty_like(t) for _ in range(self.world)]
        self.dist.all_gather(out, t)
        return [float(o.item()) for o in out]

    def close(self):
        if self.dist:
            self.dist.destroy_process_group()


def _time_steps(torch, fn, steps, warmup):
    """CUDA events on the launching stream around each of `steps` calls, after max(warmup, 3) untimed ones."""
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


def pcie_rates(D: Dist, mib: int = 256) -> dict:
    """Plain pinned-memory copy rates of every rank, all ranks copying at the same time: shows whether PCIe, the host
    memory controllers or the copy engines cap the end-to-end numbers."""
    torch = D.torch
    from ytensor_b200 import host
    h, numa = host.pinned_near(D.local, (mib << 20,), torch.uint8)
    d = torch.empty(mib << 20, dtype=torch.uint8, device=D.dev)
    out = {}
    for name, (dst, src) in (("h2d", (d, h)), ("d2h", (h, d))):
        dst.copy_(src, non_blocking=True)
        D.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(4):
            dst.copy_(src, non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        out[name + "_gbs_per_rank"] = [round(v, 1) for v in D.gather(4 * (mib << 20) / (e0.elapsed_time(e1) * 1e-3) / 1e9)]
    out["numa_node"] = numa["node"]
    return out


# ======================================================================================= CPU baselines
def _cpu_backend():
    from oracle import oracle as O
    kind = "reference" if O.ref_available() else "port"
    cores = os.cpu_count() or 1
    if kind == "reference":
        os.environ.setdefault("OMP_NUM_THREADS", str(cores))
        os.environ.setdefault("OMP_PROC_BIND", "close")
        be = O.ref(threads=cores)
        cores = be.threads()
    else:
        be, cores = O.port(), 1
    return be, kind, cores


def cpu_gemm(budget_s: float = 12.0, items: int = 4) -> dict:
    """The reference's recipe for 16-bit storage (widen, YTensor<float>::matmul, narrow) on `items` of the 64 matrices."""
    import numpy as np
    be, kind, cores = _cpu_backend()
    rng = np.random.default_rng(1)
    a = be.f32_to_bf16(rng.standard_normal((items, M, K)).astype(np.float32))
    b = be.f32_to_bf16((rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32))
    be.matmul_16(a[:1, :256], b, 1)  # warm the thread pool
    t0 = time.perf_counter()
    be.matmul_16(a, b, 1)
    one = time.perf_counter() - t0
    reps = max(0, min(4, int(budget_s / max(one, 1e-3)) - 1))
    ts = [one]
    for _ in range(reps):
        t0 = time.perf_counter()
        be.matmul_16(a, b, 1)
        ts.append(time.perf_counter() - t0)
    dt = min(ts)
    return {"value": 2.0 * items * M * K * N / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": kind,
            "seconds": dt,
            "sample": f"{items} of {BATCH} batch items ({items}x2048x4096x4096; widen bf16->f32, "
                      f"YTensor<float>::matmul AVX2, narrow with yt::bfloat16), best of {len(ts)} runs, scaled by FLOPs"}


def cpu_gemm32() -> dict:
    import numpy as np
    be, kind, cores = _cpu_backend()
    rng = np.random.default_rng(0)
    a = rng.standard_normal((1024, 1024)).astype(np.float32)
    b = rng.standard_normal((1024, 1024)).astype(np.float32)
    be.matmul(a, b)
    ts = []
    for _ in range(10):
        t0 = time.perf_counter()
        be.matmul(a, b)
        ts.append(time.perf_counter() - t0)
    dt = min(ts)
    return {"value": 2.0 * 1024 ** 3 / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": kind, "seconds": dt,
            "sample": "the whole 1024^3 product (YTensor<float>::matmul), best of 10"}


def cpu_attn() -> dict:
    """scaledDotProductAttention(FLASH_AVX2) with the causal predicate on one of the 16 batch items, all 32 heads."""
    import numpy as np
    be, kind, cores = _cpu_backend()
    rng = np.random.default_rng(2)
    S, D = 4096, 128
    kvh = 8 if kind == "reference" else 1
    q = rng.standard_normal((1, kvh, 4, S, D)).astype(np.float32)
    k = rng.standard_normal((1, kvh, S, D)).astype(np.float32)
    v = rng.standard_normal((1, kvh, S, D)).astype(np.float32)
    ts = []
    for _ in range(2):
        t0 = time.perf_counter()
        be.sdpa(q, k, v, causal=True)
        ts.append(time.perf_counter() - t0)
    dt = min(ts)
    flops = 4.0 * kvh * 4 * S * S * D / 2
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": kind, "seconds": dt,
            "sample": f"1 of 16 batch items, {kvh * 4} of 32 query heads (fp32, FLASH_AVX2 path, causal predicate), "
                      f"best of 2, scaled by FLOPs (causal convention)"}


def cpu_chain() -> dict:
    import numpy as np
    be, kind, cores = _cpu_backend()
    rng = np.random.default_rng(3)
    b = 2 if kind == "reference" else 1
    rows = 4096 if kind == "reference" else 256
    x = rng.standard_normal((b, rows, 4096)).astype(np.float32)
    w = (rng.random(4096) * 0.2 + 0.9).astype(np.float32)
    r = rng.standard_normal((1, rows, 4096)).astype(np.float32)
    ts = []
    for _ in range(2):
        t0 = time.perf_counter()
        be.chain(x, w, r)
        ts.append(time.perf_counter() - t0)
    dt = min(ts)
    nbytes = x.size * 4 + r.size * 4 + 4096 * 4 + x.size * 2
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": kind, "seconds": dt,
            "sample": f"[{b},{rows},4096] of [32,4096,4096] (rmsNorm, +=, softmax_, copy_ to bfloat16 in sequence), "
                      f"best of 2, algorithmic bytes of the fused form / time"}


def cpu_decode(batches=(1, 32)) -> list[dict]:
    """qwen3::Qwen3ForCausalLM on the CPU with the same random weights widened to fp32: a short prompt and a few
    greedy decode steps per batch size."""
    import numpy as np

    from ytensor_b200 import qwen3 as Q
    be, kind, cores = _cpu_backend()
    cfg = Q.Qwen3Config(max_position_embeddings=64)
    if kind != "reference":
        cfg.num_hidden_layers = 2
    weights = Q.random_weights(cfg, seed=4)
    res = []
    for B in batches:
        prompt_len, steps = (16, 16) if B == 1 else (2, 2)
        h = be.qwen3(cfg.oracle_dict(), batch=B)
        for key, arr in weights.items():
            name, layer = (key, 0) if isinstance(key, str) else key
            h.set_weight(name, layer, Q.bf16_bits_to_f32(arr) if arr.dtype == np.uint16 else arr)
        ids = np.random.default_rng(4).integers(0, cfg.vocab_size, (B, prompt_len)).astype(np.int32)
        t0 = time.perf_counter()
        logits = h.forward(ids)
        t1 = time.perf_counter()
        for _ in range(steps):
            tok = logits.argmax(axis=1).astype(np.int32).reshape(B, 1)
            logits = h.forward(tok)
        t2 = time.perf_counter()
        h.close()
        res.append({"value": B * steps / (t2 - t1), "unit": "tok/s", "cores": cores, "kind": kind,
                    "seconds": t2 - t0, "prefill_tokens_per_s": B * prompt_len / (t1 - t0),
                    "sample": f"batch {B}: prompt of {prompt_len} tokens, then {steps} greedy decode steps "
                              f"({cfg.num_hidden_layers} layers, fp32 Qwen3ForCausalLM::forward + host argmax); "
                              f"decode steps only in the value"})
    return res


# ======================================================================================= reference arm
def reference_arm(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    items = 4
    runs = []
    for _ in range(max(1, min(args.steps, 3))):
        runs.append(cpu_gemm(budget_s=0.0, items=items))
    best = max(runs, key=lambda r: r["value"])
    tfl = best["value"]
    best["sample"] = (f"{items} of {BATCH} batch items per step (widen bf16->f32, YTensor<float>::matmul AVX2, narrow "
                      f"with yt::bfloat16), best of {len(runs)} steps, scaled by FLOPs")
    out = {
        "impl": "reference", "metric": "bf16_gemm_tflops", "value": tfl, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": len(runs), "warmup": 1, "ms_per_step": best["seconds"] * 1e3,
        "ms_per_full_workload_extrapolated": best["seconds"] * 1e3 * BATCH / items,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32 compute on bf16 storage",
        "data": "synthetic", "config": gemm_config(world, BATCH),
        "cpu_baseline": best,
        "e2e": {"value": tfl, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if not args.no_secondary:
        sec = []
        for name, fn in (("flash_attn_causal_tflops", cpu_attn), ("decode_tokens_per_s", cpu_decode),
                         ("memory_chain_gbs", cpu_chain), ("fp32_gemm_tflops", cpu_gemm32)):
            try:
                r = fn()
                for e in (r if isinstance(r, list) else [r]):
                    sec.append({"metric": name, "value": e["value"], "unit": e["unit"], "cpu_baseline": e})
            except Exception as ex:  # noqa: BLE001 - a failed leg is recorded, the headline stands
                sec.append({"metric": name, "error": repr(ex)[:300]})
        out["secondary"] = sec
    print(json.dumps(out))


# ======================================================================================= GEMM (headline)
def gemm_config(world: int, batch_per_rank: int) -> dict:
    return {"workload": GEMM_WORKLOAD, "global_batch": batch_per_rank * world, "batch_per_rank": batch_per_rank,
            "m": M, "k": K, "n": N, "parallelism": f"batch-sharded x{world}, no collective",
            "l2": "L2 flushed between steps when a rank's operands are smaller than 4x the L2, else inputs larger "
                  "than L2 (A is 1.07 GB per 64 matrices)"}


def gemm_arm(args, weak: bool = False) -> dict | None:
    """configs[1]. Strong scaling by default: the 64 matrices are split over the ranks. weak=True gives every rank 64."""
    D = Dist()
    torch = D.torch
    from ytensor_b200 import _lib, host
    L = _lib.lib()
    batch = args.batch if args.batch else (BATCH if weak else max(1, BATCH // D.world))
    profiling_case = bool(args.batch)
    flops_rank = 2.0 * batch * M * K * N
    g = torch.Generator(device=D.dev).manual_seed(1 + D.rank)
    # plumbing only: torch provides device memory and the synthetic draw; the GEMM is ytcuda_gemm
    a = torch.randn(batch, M, K, device=D.dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    b = (torch.randn(K, N, device=D.dev, generator=g, dtype=torch.float32) / K ** 0.5).to(torch.bfloat16)
    c = torch.empty(batch, M, N, device=D.dev, dtype=torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    rank_bytes = (a.numel() + b.numel() + c.numel()) * 2
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=D.dev) if rank_bytes < (512 << 20) else None

    def step():
        _lib.check(L.ytcuda_gemm(_lib.BF16, _lib.BF16, a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, 1.0, 0.0,
                                 K, 1, N, 1, N, 1, batch, M * K, 0, M * N, stream))

    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    D.barrier()
    sampler = ClockSampler(D.local)
    if D.rank == 0:
        sampler.start()
    launches0 = L.ytcuda_launch_count()
    ev0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ev1 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    D.barrier()
    for i in range(args.steps):
        if flush is not None:
            flush.zero_()
        ev0[i].record()
        step()
        ev1[i].record()
    D.barrier()
    per_launch_ms = [ev0[i].elapsed_time(ev1[i]) for i in range(args.steps)]
    launches = L.ytcuda_launch_count() - launches0
    _lib.check(L.ytcuda_device_status(None))
    clocks = sampler.stop() if D.rank == 0 else None
    # device time of the step = the GEMM launches themselves (the L2 flush between them is not part of a step)
    (total_ms,) = D.max_over_ranks(sum(per_launch_ms))
    ms_per_step = total_ms / args.steps
    value = flops_rank * D.world / (ms_per_step * 1e-3) / 1e12

    e2e = None
    if not args.no_e2e:
        e2e_steps = max(2, min(args.steps, 5))
        (ha, numa), (hb, _), (hc, _) = (host.pinned_near(D.local, t.shape, t.dtype) for t in (a, b, c))
        ha.copy_(a)
        hb.copy_(b)

        def host_step():
            _lib.check(L.ytcuda_gemm_host(_lib.BF16, _lib.BF16, ha.data_ptr(), hb.data_ptr(), hc.data_ptr(), M, N, K,
                                          1.0, 0.0, K, 1, N, 1, N, 1, batch, M * K, 0, M * N))

        host_step()
        D.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            host_step()
        D.barrier()
        (e2e_s,) = D.max_over_ranks((time.perf_counter() - t0) / e2e_steps)
        same = bool(torch.equal(hc[batch - 1], c[batch - 1].cpu()))
        e2e = {"value": flops_rank * D.world / e2e_s / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": (ha.numel() + hb.numel()) * 2, "d2h_bytes_per_step": hc.numel() * 2,
               "bytes_are": "per rank", "ms_per_step": e2e_s * 1e3, "steps": e2e_steps, "matches_device_result": same,
               "api": "ytcuda_gemm_host (pinned host buffers placed on the GPU's NUMA node)",
               "pinned_numa_node": numa["node"], "pcie": pcie_rates(D)}

    out = None
    if D.rank == 0:
        peaks = measured_peaks()
        avg_launch_ms = statistics.mean(per_launch_ms)
        achieved = flops_rank / (avg_launch_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["bf16_tflops"], "traffic": GEMM_TRAFFIC_64 * batch / 64.0,
                    "traffic_note": "ncu dram read+write of a capture of 8 matrices scaled to this launch "
                                    "(A and C per matrix, B once)",
                    "kernel": "gemm_tc2_kernel (cta_group::2, 256x256 tile per CTA pair)",
                    "peak_source": f"{peaks['source']} (burst cuBLAS bf16)",
                    "frac_of_sustained_peak": (achieved / peaks["bf16_tflops_sustained"]
                                               if peaks.get("bf16_tflops_sustained") else None),
                    "algorithmic_flops_per_launch": flops_rank}
        cfg = gemm_config(D.world, batch)
        if profiling_case:
            cfg["workload"] = f"PROFILING CASE ({batch} matrices, not configs[1]): " + GEMM_WORKLOAD
        out = {
            "metric": "bf16_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": D.world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak" if weak else "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": cfg, "roofline": roofline, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        }
    del a, b, c
    D.close()
    return out


# ======================================================================================= attention
def attention_arm(args) -> dict | None:
    """configs[2]: causal flash attention bf16, batch 16, 32 q / 8 kv heads, head_dim 128, seq 4096. With N ranks the
    16 x 8 = 128 (batch, kv head) units are split evenly (whole batch items first, then kv heads of one item); every
    unit is independent, no collective. `--batch` shrinks the batch for profiling captures."""
    D = Dist()
    torch = D.torch
    from ytensor_b200 import _lib, api, host
    L = _lib.lib()
    B_all = args.batch if args.batch else 16
    H, KVH, S, Dh = 32, 8, 4096, 128
    units = B_all * KVH
    if units % D.world:
        raise SystemExit(f"{units} attention units do not split over {D.world} ranks")
    per = units // D.world
    if per >= KVH:
        B, kvh = per // KVH, KVH
    else:
        B, kvh = 1, per
    heads = kvh * (H // KVH)
    g = torch.Generator(device=D.dev).manual_seed(2 + D.rank)
    q = torch.randn(B, heads, S, Dh, device=D.dev, generator=g).to(torch.bfloat16)
    k = torch.randn(B, kvh, S, Dh, device=D.dev, generator=g).to(torch.bfloat16)
    v = torch.randn(B, kvh, S, Dh, device=D.dev, generator=g).to(torch.bfloat16)
    flops_rank = 4.0 * B * heads * S * S * Dh / 2  # causal convention: half of the square
    rank_bytes = (2 * q.numel() + 2 * k.numel()) * 2
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=D.dev) if rank_bytes < (512 << 20) else None
    out_holder = [None]

    def step():
        out_holder[0] = api.scaledDotProductAttention(q, k, v, causal=True)

    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    D.barrier()
    sampler = ClockSampler(D.local)
    if D.rank == 0:
        sampler.start()
    n0 = L.ytcuda_launch_count()
    ev0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ev1 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    D.barrier()
    for i in range(args.steps):
        if flush is not None:
            flush.zero_()
        ev0[i].record()
        step()
        ev1[i].record()
    D.barrier()
    ts = [ev0[i].elapsed_time(ev1[i]) for i in range(args.steps)]
    launches = L.ytcuda_launch_count() - n0
    clocks = sampler.stop() if D.rank == 0 else None
    _lib.check(L.ytcuda_device_status(None))
    (total_ms,) = D.max_over_ranks(sum(ts))
    ms = total_ms / args.steps
    val = flops_rank * D.world / (ms * 1e-3) / 1e12

    e2e = None
    if not args.no_e2e:
        (hq, numa), (hk, _), (hv, _), (ho, _) = (host.pinned_near(D.local, t.shape, t.dtype) for t in (q, k, v, q))
        hq.copy_(q)
        hk.copy_(k)
        hv.copy_(v)
        chunk = 2 if B >= 4 else 1
        host.scaledDotProductAttention_host(hq, hk, hv, ho, causal=True, chunk=chunk)
        D.barrier()
        reps = 3
        t0 = time.perf_counter()
        for _ in range(reps):
            host.scaledDotProductAttention_host(hq, hk, hv, ho, causal=True, chunk=chunk)
        D.barrier()
        (e2e_s,) = D.max_over_ranks((time.perf_counter() - t0) / reps)
        same = bool(torch.equal(ho[B - 1], out_holder[0][B - 1].cpu()))
        e2e = {"value": flops_rank * D.world / e2e_s / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": (hq.numel() + hk.numel() + hv.numel()) * 2, "d2h_bytes_per_step": ho.numel() * 2,
               "bytes_are": "per rank", "ms_per_step": e2e_s * 1e3, "steps": reps, "matches_device_result": same,
               "api": "ytensor_b200.host.scaledDotProductAttention_host (pinned host tensors, batch chunks pipelined "
                      "over three streams)", "pinned_numa_node": numa["node"]}
    out = None
    if D.rank == 0:
        peaks = measured_peaks()
        achieved = flops_rank / (statistics.mean(ts) * 1e-3) / 1e12
        out = {
            "metric": "flash_attn_causal_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": D.world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"configs[2]: causal flash attention bf16, batch {B_all}, 32 q / 8 kv heads, "
                                   f"head_dim 128, seq 4096" + ("" if B_all == 16 else " (PROFILING CASE: reduced batch)"),
                       "parallelism": f"{units} (batch, kv head) units split x{D.world}: {B} batch items x {kvh} kv "
                                      f"heads per rank, no collective",
                       "l2": "flushed between steps when a rank's tensors are under 512 MB, else larger than L2"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16_tflops"], "traffic": None, "kernel": "flash_tc_kernel<128>",
                         "peak_source": f"{peaks['source']} (burst cuBLAS bf16)",
                         "frac_of_sustained_peak": (achieved / peaks["bf16_tflops_sustained"]
                                                    if peaks.get("bf16_tflops_sustained") else None),
                         "algorithmic_flops_per_launch": flops_rank, "non_causal_equivalent_tflops": 2 * achieved},
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks}
        if D.world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_attn()
    D.close()
    return out


# ======================================================================================= fp32 GEMM
def gemm32_arm(args) -> dict | None:
    """configs[0]: fp32 GEMM 1024 x 1024 x 1024 (the reference's own CPU-runnable case). The device forms the product
    on the tensor cores from three bf16 planes per operand (six partial products side by side along k, one GEMM
    launch). The L2 is flushed between steps because the 12.6 MB of operands would otherwise stay cached."""
    D = Dist()
    torch = D.torch
    from ytensor_b200 import _lib, api
    L = _lib.lib()
    n = 1024
    g = torch.Generator(device=D.dev).manual_seed(0)
    a = torch.randn(n, n, device=D.dev, generator=g)
    b = torch.randn(n, n, device=D.dev, generator=g)
    c = torch.empty(n, n, device=D.dev)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=D.dev)  # larger than the 126 MB L2
    flops = 2.0 * n * n * n
    res = {}
    for name, mode in (("tc", 0), ("ffma", 1)):
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
    api.matmul(a, b, c)  # leave the tensor-core result in c: the host-buffer call below is compared with it
    _lib.check(L.ytcuda_device_status(None))
    ha, hb, hc = a.cpu().pin_memory(), b.cpu().pin_memory(), torch.empty(n, n).pin_memory()

    def host_step():
        _lib.check(L.ytcuda_gemm_host(_lib.F32, _lib.F32, ha.data_ptr(), hb.data_ptr(), hc.data_ptr(), n, n, n, 1.0,
                                      0.0, n, 1, n, 1, n, 1, 1, 0, 0, 0))

    host_step()
    reps = 10
    t0 = time.perf_counter()
    for _ in range(reps):
        host_step()
    e2e_s = (time.perf_counter() - t0) / reps
    peaks = measured_peaks()
    ms, launches = res["tc"]
    val = flops / (ms * 1e-3) / 1e12
    peak = peaks["bf16_tflops"] / 6.0
    out = {
        "metric": "fp32_gemm_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "replicas only",
        "vs_baseline": None, "dtype": "f32 (three bf16 planes per operand, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": "configs[0]: fp32 GEMM 1024 x 1024 x 1024", "l2": "flushed between steps (192 MB write)"},
        "roofline": {"bound": "tensor", "achieved": val, "peak": peak, "unit": "TFLOP/s", "frac": val / peak,
                     "traffic": None, "kernel": "gemm_split3_kernel (one launch for both operands) + gemm_tc kernel over k' = 6 k, queued as dependent launches",
                     "peak_source": f"{peaks['source']} (burst cuBLAS bf16 / 6 partial products)",
                     "algorithmic_flops_per_launch": flops},
        "ffma_kernel": {"ms_per_step": res["ffma"][0], "tflops": flops / (res["ffma"][0] * 1e-3) / 1e12},
        "e2e": {"value": flops / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": 2 * n * n * 4,
                "d2h_bytes_per_step": n * n * 4, "ms_per_step": e2e_s * 1e3, "steps": reps,
                "matches_device_result": bool(torch.equal(hc, c.cpu())),
                "api": "ytcuda_gemm_host (pinned host buffers)"},
        "gpu_launches": int(launches * args.steps), "clocks": None}
    if not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_gemm32()
    D.close()
    return out if D.rank == 0 else None


# ======================================================================================= memory chain
def chain_arm(args) -> dict | None:
    """configs[3]: y = bf16(softmax(rmsNorm(x, w, -1, 1e-6) + r, -1)) on x [32,4096,4096] fp32 with the residual
    [1,4096,4096] shared by the batch. `--batch` shrinks the batch for profiling captures. Single GPU."""
    D = Dist()
    torch = D.torch
    from ytensor_b200 import _lib, api, host
    L = _lib.lib()
    B = args.batch if args.batch else 32
    R, H = 4096, 4096
    g = torch.Generator(device=D.dev).manual_seed(3)
    x = torch.randn(B, R, H, device=D.dev, generator=g)
    w = torch.rand(H, device=D.dev, generator=g) * 0.2 + 0.9
    r = torch.randn(1, R, H, device=D.dev, generator=g)
    algo_bytes = x.numel() * 4 + r.numel() * 4 + H * 4 + x.numel() * 2
    sampler = ClockSampler(D.local)
    sampler.start()
    n0 = L.ytcuda_launch_count()
    ts = _time_steps(torch, lambda: api.rmsnorm_add_softmax_cast(x, w, r), args.steps, args.warmup)
    launches = L.ytcuda_launch_count() - n0 - max(args.warmup, 3)
    clocks = sampler.stop()
    ms = statistics.mean(ts)
    val = algo_bytes / (ms * 1e-3) / 1e9
    e2e = None
    if not args.no_e2e:
        want = api.rmsnorm_add_softmax_cast(x[B - 1:], w, r).cpu()
        (hx, numa), (ho, _) = host.pinned_near(D.local, x.shape, x.dtype), host.pinned_near(D.local, x.shape, torch.bfloat16)
        hr, hw = r.cpu().pin_memory(), w.cpu().pin_memory()
        hx.copy_(x)
        del x
        torch.cuda.empty_cache()
        host.rmsnorm_add_softmax_cast_host(hx, hw, hr, ho, chunk=2)
        reps = 2
        t0 = time.perf_counter()
        for _ in range(reps):
            host.rmsnorm_add_softmax_cast_host(hx, hw, hr, ho, chunk=2)
        e2e_s = (time.perf_counter() - t0) / reps
        e2e = {"value": algo_bytes / e2e_s / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": hx.numel() * 4 + hr.numel() * 4 + H * 4, "d2h_bytes_per_step": ho.numel() * 2,
               "ms_per_step": e2e_s * 1e3, "steps": reps, "matches_device_result": bool(torch.equal(ho[B - 1:], want)),
               "api": "ytensor_b200.host.rmsnorm_add_softmax_cast_host (pinned host tensors, batch chunks pipelined "
                      "over three streams)", "pinned_numa_node": numa["node"]}
    peaks = measured_peaks()
    out = {
        "metric": "memory_chain_gbs", "value": val, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "single GPU",
        "vs_baseline": None, "dtype": "f32 in, bf16 out", "data": "synthetic",
        "config": {"workload": f"configs[3]: RMSNorm + broadcast residual + row softmax + cast on [{B},4096,4096]"
                               + ("" if B == 32 else " (PROFILING CASE: reduced batch)"),
                   "l2": "inputs larger than L2 (x is 2.1 GB)"},
        "roofline": {"bound": "hbm", "achieved": val, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": val / peaks["hbm_gbs"], "traffic": None, "kernel": "chain_fast_kernel<4>",
                     "peak_source": f"{peaks['source']} (copy bandwidth)", "algorithmic_bytes_per_launch": algo_bytes},
        "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks}
    if not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_chain()
    D.close()
    return out if D.rank == 0 else None


# ======================================================================================= decoder
def decode_arm(args) -> list | None:
    """configs[4]: random-init decoder of the Qwen3-0.6B shape, 512-token prompt, greedy decode of 256 tokens, for
    1 and for 32 sequences (`--batch` picks one). Under torch.distributed.run the ranks form one tensor-parallel
    group (total work fixed: strong scaling). value = decoded tokens per second over all sequences; the prompt pass
    is reported next to it."""
    import numpy as np
    D = Dist()
    torch = D.torch
    from ytensor_b200 import _lib
    from ytensor_b200 import qwen3 as Q
    L = _lib.lib()
    prompt_len, new_tokens = 512, args.new_tokens
    cfg = Q.Qwen3Config(max_position_embeddings=prompt_len + new_tokens)
    weights = Q.random_weights(cfg, seed=4)
    results = []
    for B in ([args.batch] if args.batch else [1, 32]):
        m = Q.Qwen3ForCausalLM(cfg, batch=B, tp_rank=D.rank, tp_world=D.world)
        m.load_weights(weights)
        prompt_host = torch.from_numpy(np.random.default_rng(4).integers(0, cfg.vocab_size, (B, prompt_len))
                                       .astype(np.int32)).pin_memory()

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
        D.barrier()
        # a slow sampling period: every nvidia-smi query briefly holds the driver and delays kernel launches,
        # which a launch-bound decode loop feels
        sampler = ClockSampler(D.local, interval_ms=1000)
        if D.rank == 0 and not args.no_clock_sampling:
            sampler.start()
        n0 = L.ytcuda_launch_count()
        t0 = time.perf_counter()
        prefill_ms, decode_ms, toks = run()
        D.barrier()
        wall = time.perf_counter() - t0
        launches = L.ytcuda_launch_count() - n0
        status = L.ytcuda_device_status(None)
        clocks = sampler.stop() if (D.rank == 0 and not args.no_clock_sampling) else None
        prefill_ms, decode_ms, wall = D.max_over_ranks(prefill_ms, decode_ms, wall)
        if D.rank == 0:
            peaks = measured_peaks()
            steps = new_tokens - 1
            tok_s = B * steps / (decode_ms * 1e-3)
            params = cfg.num_hidden_layers * 15728640 + cfg.vocab_size * cfg.hidden_size
            weight_bytes = params * 2 / D.world
            mean_keys = prompt_len + (new_tokens + 1) / 2.0
            kv_bytes = (cfg.num_hidden_layers * 2 * cfg.num_key_value_heads * cfg.head_dim * 4 * mean_keys * B) / D.world
            bytes_per_step = weight_bytes + kv_bytes
            achieved = bytes_per_step / (decode_ms * 1e-3 / steps) / 1e9
            entry = {
                "metric": "decode_tokens_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": D.world,
                "steps": new_tokens, "warmup": 1, "ms_per_step": decode_ms / steps, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "bf16 weights, f32 activations and KV cache",
                "data": "synthetic",
                "config": {"workload": f"configs[4]: Qwen3-0.6B-shape decoder, random bf16 weights, prompt 512, greedy "
                                       f"decode of {new_tokens} tokens, batch {B}", "batch": B,
                           "new_tokens": new_tokens, "parallelism": f"tp{D.world}",
                           "l2": "weights (1.19 GB) larger than L2"},
                "prefill_tokens_per_s": B * prompt_len / (prefill_ms * 1e-3), "prefill_ms": prefill_ms,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                             "kernel": m.decode_kernel_name(),
                             "peak_source": f"{peaks['source']} (copy bandwidth)",
                             "algorithmic_bytes_per_launch": bytes_per_step,
                             "note": "this rank's bf16 weights streamed once per decode step + its share of the fp32 "
                                     "K/V rows read (mean context over the run) / step time"},
                "e2e": {"value": B * new_tokens / wall, "unit": "tok/s",
                        "h2d_bytes_per_step": int(prompt_host.numel() * 4), "d2h_bytes_per_step": int(toks.numel() * 4),
                        "ms_per_step": wall * 1e3,
                        "api": "ytensor_b200.qwen3.Qwen3ForCausalLM.forward + argmax (prompt H2D from pinned memory, "
                               "prefill, decode, tokens D2H; wall clock, generated tokens / s)"},
                "gpu_launches": int(launches), "device_status": int(status), "clocks": clocks,
                "first_tokens": toks[0, :8].tolist()}
            results.append(entry)
        m.close()
        del m
        torch.cuda.empty_cache()
    if D.rank == 0 and D.world == 1 and not args.no_cpu_baseline:
        try:
            cpu = cpu_decode([e["config"]["batch"] for e in results])
            for e, c in zip(results, cpu):
                e["cpu_baseline"] = c
        except Exception as ex:  # noqa: BLE001
            for e in results:
                e["cpu_baseline"] = {"error": repr(ex)[:300]}
    D.close()
    return results if D.rank == 0 else None


# ======================================================================================= driver of the children
ARMS = {"attn": attention_arm, "decode": decode_arm, "chain": chain_arm, "gemm32": gemm32_arm,
        "gemm_weak": lambda a: gemm_arm(a, weak=True)}


def run_secondary(args, names, budget_s: float) -> list:
    """Runs each named workload as a child process of this rank (children of the ranks rendezvous among themselves on
    a port of their own). Returns the entries rank 0's children printed; failures become entries too."""
    rank = int(os.environ.get("RANK", "0"))
    base_port = int(os.environ.get("MASTER_PORT", "29500"))
    t_start = time.perf_counter()
    entries = []
    for i, name in enumerate(names):
        left = budget_s - (time.perf_counter() - t_start)
        if left < 20:
            entries.append({"workload": name, "skipped": "time budget of the secondary workloads used up"})
            continue
        env = dict(os.environ)
        env["MASTER_PORT"] = str(base_port + 17 + i)
        # under torch.distributed.run the ranks are clients of the launcher's own store on MASTER_PORT; the children
        # rendezvous on another port, where the child of rank 0 has to host the store itself
        env["TORCHELASTIC_USE_AGENT_STORE"] = "False"
        cmd = [sys.executable, str(Path(__file__).resolve()), "--child", name, "--gpus", str(args.gpus),
               "--steps", str(max(3, min(args.steps, 10))), "--warmup", str(args.warmup)]
        if args.no_cpu_baseline:
            cmd.append("--no-cpu-baseline")
        try:
            r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=min(left, 420))
            line = next((ln for ln in reversed(r.stdout.splitlines()) if ln.startswith("{\"child\"")), None)
            if rank != 0:
                continue
            if line is None:
                entries.append({"workload": name, "error": f"exit {r.returncode}: " + (r.stderr or r.stdout)[-400:]})
            else:
                got = json.loads(line)["entries"]
                entries.extend(got)
        except subprocess.TimeoutExpired:
            if rank == 0:
                entries.append({"workload": name, "error": "timed out"})
    return entries


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="all", choices=["all", "gemm", "gemm_weak", "gemm32", "attn", "chain", "decode"],
                    help="all (default): the headline GEMM line with the other workloads in its `secondary` array; a "
                         "name: that workload alone, printed as its own line")
    ap.add_argument("--child", default=None, help=argparse.SUPPRESS)
    ap.add_argument("--no-secondary", action="store_true")
    ap.add_argument("--secondary-budget", type=float, default=420.0, help="seconds for all secondary workloads")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-clock-sampling", action="store_true", help="decode workload: do not run nvidia-smi beside it")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling captures only)")
    ap.add_argument("--new-tokens", type=int, default=256, help="decode workload: tokens generated per sequence")
    ap.add_argument("--batch", type=int, default=0,
                    help="batch items per rank and step; anything but the default is a profiling case, not a bench line")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        return reference_arm(args)
    if args.child:
        out = ARMS[args.child](args)
        if rank == 0:
            entries = out if isinstance(out, list) else [out]
            print(json.dumps({"child": args.child, "entries": entries}))
        return
    if args.workload not in ("all", "gemm"):
        out = ARMS[args.workload](args)
        if rank == 0:
            for e in (out if isinstance(out, list) else [out]):
                print(json.dumps(e))
        return
    out = gemm_arm(args)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_gemm()
    if args.workload == "all" and not args.no_secondary:
        names = ["attn", "decode", "chain", "gemm32"] if world == 1 else ["attn", "decode", "gemm_weak"]
        sec = run_secondary(args, names, args.secondary_budget)
        if rank == 0:
            out["secondary"] = sec
    if rank == 0:
        print(json.dumps(out))


if __name__ == "__main__":
    main()
