"""Host-buffer forms of the attention and memory-chain operators, and NUMA placement of pinned buffers.

The reference's tensors always live in host memory (include/ytensor_base.hpp:388-393), so the call a YTensor user
makes hands HOST buffers to the backend. ytcuda_gemm_host does that for GEMM inside the C library; the two functions
here do it for scaledDotProductAttention (src/function/ops.inl:368-425) and for the rmsNorm -> += -> softmax_ -> copy_
chain: batch items are cut into chunks, and three streams overlap the upload of chunk i + 1, the kernels of chunk i and
the download of chunk i - 1 through two sets of device buffers. torch provides streams, events and device memory only.
"""
from __future__ import annotations

import contextlib
import os
from pathlib import Path

import torch

from . import api


# ------------------------------------------------------------------ NUMA placement
def device_numa_node(index: int) -> int | None:
    """NUMA node the GPU's PCIe slot hangs off (sysfs), or None when the platform does not say (-1, VM, no sysfs)."""
    try:
        p = torch.cuda.get_device_properties(index)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        node = int(Path(f"/sys/bus/pci/devices/{bdf}/numa_node").read_text().strip())
        return node if node >= 0 else None
    except (OSError, ValueError, AttributeError):
        return None


def _parse_cpulist(text: str) -> set[int]:
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def node_cpus(node: int) -> set[int]:
    try:
        return _parse_cpulist(Path(f"/sys/devices/system/node/node{node}/cpulist").read_text())
    except OSError:
        return set()


@contextlib.contextmanager
def near_device(index: int):
    """Runs the body with the calling thread bound to the CPUs of the GPU's NUMA node, so that pinned buffers
    allocated (and first touched) inside land in the memory next to the GPU's PCIe root. Yields a small record
    {"node", "cpus"}; a platform without the information yields {"node": None} and binds nothing."""
    info = {"node": None, "cpus": 0}
    old = None
    node = device_numa_node(index)
    if node is not None and hasattr(os, "sched_setaffinity"):
        try:
            old = os.sched_getaffinity(0)
            cpus = node_cpus(node) & old
            if cpus:
                os.sched_setaffinity(0, cpus)
                info = {"node": node, "cpus": len(cpus)}
            else:
                old = None
        except OSError:
            old = None
    try:
        yield info
    finally:
        if old is not None:
            os.sched_setaffinity(0, old)


def pinned_near(index: int, shape, dtype) -> tuple[torch.Tensor, dict]:
    """A pinned host tensor placed next to GPU `index` (first touched while bound to its NUMA node)."""
    with near_device(index) as info:
        t = torch.empty(shape, dtype=dtype, pin_memory=True)
        t.view(torch.uint8).reshape(-1)[:: 4096].zero_()  # touch every page while bound
    return t, info


# ------------------------------------------------------------------ pipelined host-buffer operators
class _Pipe:
    """Three streams and two buffer sets: upload / run / download of consecutive chunks overlap."""

    def __init__(self):
        self.s_in, self.s_run, self.s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        self.in_done = [torch.cuda.Event() for _ in range(2)]
        self.run_done = [torch.cuda.Event() for _ in range(2)]
        self.out_done = [torch.cuda.Event() for _ in range(2)]
        self.bufs: dict = {}

    def buffers(self, key, make):
        if key not in self.bufs:
            self.bufs.clear()  # one workload shape at a time: do not keep old device buffers alive
            self.bufs[key] = make()
        return self.bufs[key]


_pipes: dict[int, _Pipe] = {}


def _pipe() -> _Pipe:
    dev = torch.cuda.current_device()
    if dev not in _pipes:
        _pipes[dev] = _Pipe()
    return _pipes[dev]


def _run_chunks(pipe: _Pipe, n_chunks: int, upload, run, download) -> None:
    cur = torch.cuda.current_stream()
    for s in (pipe.s_in, pipe.s_run, pipe.s_out):
        s.wait_stream(cur)
    for i in range(n_chunks):
        j = i & 1
        with torch.cuda.stream(pipe.s_in):
            if i >= 2:
                pipe.s_in.wait_event(pipe.run_done[j])  # the kernels that read buffer set j have finished
            upload(i, j)
            pipe.in_done[j].record()
        with torch.cuda.stream(pipe.s_run):
            pipe.s_run.wait_event(pipe.in_done[j])
            if i >= 2:
                pipe.s_run.wait_event(pipe.out_done[j])  # the result buffer j has left the device
            run(i, j)
            pipe.run_done[j].record()
        with torch.cuda.stream(pipe.s_out):
            pipe.s_out.wait_event(pipe.run_done[j])
            download(i, j)
            pipe.out_done[j].record()
    pipe.s_out.synchronize()
    pipe.s_run.synchronize()
    pipe.s_in.synchronize()


def scaledDotProductAttention_host(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, out: torch.Tensor,
                                   scale: float = 0.0, *, causal: bool = False, chunk: int = 2) -> torch.Tensor:
    """scaledDotProductAttention on HOST tensors (pinned for full speed): query [b, heads, q_len, d], key / value
    [b, kv_heads, kv_len, d], `out` like query. Returns when `out` is complete. Batch items travel in chunks of
    `chunk` so that copies overlap the kernels."""
    assert not query.is_cuda and query.dim() == 4 and out.shape == query.shape[:-1] + value.shape[-1:]
    b = query.shape[0]
    chunk = max(1, min(chunk, b))
    pipe = _pipe()
    dev = torch.device("cuda", torch.cuda.current_device())
    key_ = ("sdpa", tuple(query.shape[1:]), tuple(key.shape[1:]), tuple(value.shape[1:]), query.dtype, chunk)

    def make():
        mk = lambda t: [torch.empty((chunk, *t.shape[1:]), dtype=t.dtype, device=dev) for _ in range(2)]  # noqa: E731
        return mk(query), mk(key), mk(value), [None, None]

    dq, dk, dv, do = pipe.buffers(key_, make)
    n_chunks = (b + chunk - 1) // chunk

    def upload(i, j):
        b0, c = i * chunk, min(chunk, b - i * chunk)
        dq[j][:c].copy_(query[b0:b0 + c], non_blocking=True)
        dk[j][:c].copy_(key[b0:b0 + c], non_blocking=True)
        dv[j][:c].copy_(value[b0:b0 + c], non_blocking=True)

    def run(i, j):
        c = min(chunk, b - i * chunk)
        do[j] = api.scaledDotProductAttention(dq[j][:c], dk[j][:c], dv[j][:c], scale, causal=causal)

    def download(i, j):
        b0, c = i * chunk, min(chunk, b - i * chunk)
        out[b0:b0 + c].copy_(do[j], non_blocking=True)
        do[j].record_stream(pipe.s_out)

    _run_chunks(pipe, n_chunks, upload, run, download)
    return out


def rmsnorm_add_softmax_cast_host(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, out: torch.Tensor,
                                  eps: float = 1e-6, *, chunk: int = 2) -> torch.Tensor:
    """out = bf16(softmax(rmsNorm(x, weight, -1, eps) + residual, -1)) on HOST tensors: x [b, rows, hidden] fp32,
    residual [1, rows, hidden] shared by the batch (uploaded once) or [b, rows, hidden], out like x in bf16 / fp16 /
    fp32. Returns when `out` is complete."""
    assert not x.is_cuda and x.dim() == 3 and out.shape == x.shape
    b = x.shape[0]
    chunk = max(1, min(chunk, b))
    shared = residual.shape[0] == 1
    pipe = _pipe()
    dev = torch.device("cuda", torch.cuda.current_device())
    key_ = ("chain", tuple(x.shape[1:]), x.dtype, out.dtype, chunk, shared)

    def make():
        dx = [torch.empty((chunk, *x.shape[1:]), dtype=x.dtype, device=dev) for _ in range(2)]
        dr = ([torch.empty((1, *x.shape[1:]), dtype=torch.float32, device=dev)] if shared else
              [torch.empty((chunk, *x.shape[1:]), dtype=torch.float32, device=dev) for _ in range(2)])
        return dx, dr, [None, None]

    dx, dr, do = pipe.buffers(key_, make)
    dw = weight.to(dev, non_blocking=True)
    n_chunks = (b + chunk - 1) // chunk

    def upload(i, j):
        b0, c = i * chunk, min(chunk, b - i * chunk)
        if shared:
            if i == 0:
                dr[0].copy_(residual, non_blocking=True)
        else:
            dr[j][:c].copy_(residual[b0:b0 + c], non_blocking=True)
        dx[j][:c].copy_(x[b0:b0 + c], non_blocking=True)

    def run(i, j):
        c = min(chunk, b - i * chunk)
        do[j] = api.rmsnorm_add_softmax_cast(dx[j][:c], dw, dr[0] if shared else dr[j][:c], eps=eps,
                                             out_dtype=out.dtype)

    def download(i, j):
        b0, c = i * chunk, min(chunk, b - i * chunk)
        out[b0:b0 + c].copy_(do[j], non_blocking=True)
        do[j].record_stream(pipe.s_out)

    _run_chunks(pipe, n_chunks, upload, run, download)
    return out
