"""Host-side mirror of the reference's operator interface for the dense hot path.

Function names and argument meaning follow yt::YTensor / yt::function in the reference
(matmul, linear, scaledDotProductAttention, softmax, rmsNorm, layerNorm, sum/mean/max, cast);
tensors are torch tensors that only serve as device memory with a shape and strides. Every
function calls the C ABI of libytensor_cuda.so; nothing here computes with torch.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import BF16, F16, F32, check, lib

_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise _lib.YtCudaInvalidArgument(_lib.UNSUPPORTED, f"unsupported dtype {t.dtype}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "device backend: tensor is not on a CUDA device")


def _batch_view(t: torch.Tensor):
    """Splits a [..., r, c] view into (batch_count, batch_stride) if the leading dims collapse
    into one stride; returns None otherwise."""
    lead_shape, lead_stride = t.shape[:-2], t.stride()[:-2]
    dims = [(n, s) for n, s in zip(lead_shape, lead_stride) if n != 1]
    if not dims:
        return 1, 0
    count, stride = dims[-1]
    for n, s in reversed(dims[:-1]):
        if s != stride * count and not (s == 0 and stride == 0):
            return None
        count *= n
    return count, stride


def matmul(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, *, alpha: float = 1.0,
           beta: float = 0.0, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """C[..., m, n] = A[..., m, k] . B[..., k, n] with broadcast batch dims.

    Mirrors YTensor<T,dim>::matmul (reference src/ytensor_math.inl:284-316): the last dim of
    `a` must equal the second-to-last of `b` or std::invalid_argument (here ValueError) is raised.
    One batched launch replaces the reference's per-matrix loop (:1035-1049).
    """
    _require_cuda(a, b, out)
    if a.dim() < 1 or b.dim() < 1:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "matmul: operands must have at least 1 dim")
    a2 = a if a.dim() >= 2 else a.unsqueeze(0)
    b2 = b if b.dim() >= 2 else b.unsqueeze(-1)
    if a2.shape[-1] != b2.shape[-2]:
        raise _lib.YtCudaInvalidArgument(
            _lib.INVALID_ARG, f"matmul: inner dims differ ({a2.shape[-1]} vs {b2.shape[-2]})")
    if a2.dtype != b2.dtype:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "matmul: operand dtypes differ")
    m, k = a2.shape[-2:]
    n = b2.shape[-1]
    bshape = torch.broadcast_shapes(a2.shape[:-2], b2.shape[:-2])
    ae = a2.expand(*bshape, m, k)
    be = b2.expand(*bshape, k, n)
    odt = out_dtype or a2.dtype
    if out is None:
        out = torch.empty(*bshape, m, n, dtype=odt, device=a.device)
    elif tuple(out.shape) != (*bshape, m, n):
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "matmul: out has the wrong shape")
    av, bv, ov = _batch_view(ae), _batch_view(be), _batch_view(out)
    L = lib()
    if av is not None and bv is not None and ov is not None:
        batch = max(av[0], bv[0], ov[0])
        check(L.ytcuda_gemm(_dt(ae), _dt(out), ae.data_ptr(), be.data_ptr(), out.data_ptr(), m, n, k, alpha, beta,
                            ae.stride(-2), ae.stride(-1), be.stride(-2), be.stride(-1), out.stride(-2),
                            out.stride(-1), batch, av[1], bv[1], ov[1], _stream()))
    else:
        # Leading dims that do not collapse into one stride: one call per outermost slice.
        for idx in range(bshape[0]):
            matmul(ae[idx], be[idx], out[idx], alpha=alpha, beta=beta)
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """x . weight^T (+ bias), weight [out_features, in_features] (reference src/function/ops.inl:84-105)."""
    y = matmul(x, weight.transpose(-1, -2))
    if bias is not None:
        from .api import add_  # noqa: F401  (defined with the elementwise ops)
        add_(y, bias)
    return y
