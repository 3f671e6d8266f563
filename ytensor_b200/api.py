"""Host-side mirror of the reference's operator interface for the dense hot path.

Function names and argument meaning follow yt::YTensor / yt::function in the reference
(matmul, linear, scaledDotProductAttention, softmax, rmsNorm, layerNorm, sum/mean/max, cast);
tensors are torch tensors that only serve as device memory with a shape and strides. Every
function calls the C ABI of libytensor_cuda.so; nothing here computes with torch.
"""
from __future__ import annotations

import builtins
import ctypes as C

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
        batch = builtins.max(av[0], bv[0], ov[0])
        check(L.ytcuda_gemm(_dt(ae), _dt(out), ae.data_ptr(), be.data_ptr(), out.data_ptr(), m, n, k, alpha, beta,
                            ae.stride(-2), ae.stride(-1), be.stride(-2), be.stride(-1), out.stride(-2),
                            out.stride(-1), batch, av[1], bv[1], ov[1], _stream()))
    else:
        # Leading dims that do not collapse into one stride: one call per outermost slice.
        for idx in range(bshape[0]):
            matmul(ae[idx], be[idx], out[idx], alpha=alpha, beta=beta)
    return out


class Causal:
    """The predicate j <= i + offset, for the predicate forms of masked_matmul and scaledDotProductAttention
    (reference src/ytensor_math.inl:368-412, src/function/ops.inl:427-503): evaluated on the device, no mask tensor."""

    def __init__(self, offset: int = 0):
        self.offset = int(offset)

    def __call__(self, i: int, j: int) -> bool:
        return j <= i + self.offset


def masked_matmul(a: torch.Tensor, b: torch.Tensor, mask, masked_value: float = 0.0, *,
                  out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """C[..., i, j] = (A . B)[..., i, j] where mask[i, j], masked_value elsewhere; mask is bool [m, n], a `Causal`
    predicate (evaluated on the device), or any callable (i, j) -> bool (materialised once into a bool mask).

    Mirrors YTensor<T,dim>::masked_matmul with a bool mask or a predicate (reference src/ytensor_math.inl:318-412): a
    mask of another shape is refused as the reference refuses it (std::invalid_argument, here ValueError). Output
    tiles in which the mask holds nowhere are not computed.
    """
    causal = mask if isinstance(mask, Causal) else None
    if causal is None and callable(mask) and not isinstance(mask, torch.Tensor):
        mm, nn = a.shape[-2], b.shape[-1]
        mask = torch.tensor([[bool(mask(i, j)) for j in range(nn)] for i in range(mm)], dtype=torch.bool,
                            device=a.device)
    _require_cuda(a, b, None if causal else mask)
    if a.dim() < 2 or b.dim() < 2:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "masked_matmul: operands must have at least 2 dims")
    if a.shape[-1] != b.shape[-2]:
        raise _lib.YtCudaInvalidArgument(
            _lib.INVALID_ARG, f"masked_matmul: inner dims differ ({a.shape[-1]} vs {b.shape[-2]})")
    m, k = a.shape[-2:]
    n = b.shape[-1]
    if causal is None:
        if mask.dtype != torch.bool or tuple(mask.shape) != (m, n):
            raise _lib.YtCudaInvalidArgument(
                _lib.INVALID_ARG, f"masked_matmul: mask must be bool [{m}, {n}], got {mask.dtype} {tuple(mask.shape)}")
        if mask.stride(1) != 1:
            mask = mask.contiguous()
    bshape = torch.broadcast_shapes(a.shape[:-2], b.shape[:-2])
    ae, be = a.expand(*bshape, m, k), b.expand(*bshape, k, n)
    out = torch.empty(*bshape, m, n, dtype=out_dtype or a.dtype, device=a.device)
    av, bv, ov = _batch_view(ae), _batch_view(be), _batch_view(out)
    if av is None or bv is None or ov is None:
        for idx in range(bshape[0]):
            out[idx] = masked_matmul(ae[idx], be[idx], mask, masked_value, out_dtype=out_dtype)
        return out
    batch = builtins.max(av[0], bv[0], ov[0])
    if causal is not None:
        check(lib().ytcuda_gemm_masked_causal(_dt(ae), _dt(out), ae.data_ptr(), be.data_ptr(), out.data_ptr(), m, n, k,
                                              ae.stride(-2), ae.stride(-1), be.stride(-2), be.stride(-1),
                                              out.stride(-2), out.stride(-1), batch, av[1], bv[1], ov[1],
                                              causal.offset, float(masked_value), _stream()))
        return out
    check(lib().ytcuda_gemm_masked(_dt(ae), _dt(out), ae.data_ptr(), be.data_ptr(), out.data_ptr(), m, n, k,
                                   ae.stride(-2), ae.stride(-1), be.stride(-2), be.stride(-1), out.stride(-2),
                                   out.stride(-1), batch, av[1], bv[1], ov[1], mask.data_ptr(), mask.stride(0),
                                   float(masked_value), _stream()))
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """x . weight^T (+ bias), weight [out_features, in_features] (reference src/function/ops.inl:84-105)."""
    y = matmul(x, weight.transpose(-1, -2))
    if bias is not None:
        add_(y, bias)
    return y


# ------------------------------------------------------------------ N-d helpers
def _i64(vals):
    return (C.c_int64 * len(vals))(*[int(v) for v in vals])


def _i32(vals):
    return (C.c_int * len(vals))(*[int(v) for v in vals])


def _axes(axes) -> list[int]:
    return [int(axes)] if isinstance(axes, int) else [int(a) for a in axes]


def _nd(t: torch.Tensor):
    if t.dim() == 0:
        t = t.reshape(1)
    return t, _i64(t.shape), _i64(t.stride())


# ------------------------------------------------------------------ softmax / norms
def softmax(x: torch.Tensor, axes=-1, out: torch.Tensor | None = None) -> torch.Tensor:
    """Softmax jointly over `axes` (reference yt::function::softmax, src/function/activation.inl:336-375)."""
    _require_cuda(x, out)
    y = torch.empty_like(x, memory_format=torch.contiguous_format) if out is None else out
    ax = _axes(axes)
    xx, shape, xs = _nd(x)
    check(lib().ytcuda_softmax(_dt(x), _dt(y), x.data_ptr(), y.data_ptr(), shape, xs, _i64(y.stride() or (1,)),
                               xx.dim(), _i32(ax), len(ax), _stream()))
    return y


def softmax_(x: torch.Tensor, axes=-1) -> torch.Tensor:
    """In-place form (reference yt::function::softmax_, src/function/activation.inl:376-409)."""
    return softmax(x, axes, out=x)


def rmsNorm(x: torch.Tensor, weight: torch.Tensor | None, axes=-1, eps: float = 1e-5,
            out: torch.Tensor | None = None) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight (reference yt::function::rmsNorm, src/function/normalization.inl:234-277).
    `weight` has one dim per axis; a shape mismatch raises like the reference's _makeAffineView."""
    _require_cuda(x, weight, out)
    ax = _axes(axes)
    if weight is not None:
        want = [x.shape[a] for a in ax]
        if list(weight.shape) != want:
            raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "rmsNorm: weight shape must match affine axes")
        weight = weight.contiguous()
    y = torch.empty_like(x, memory_format=torch.contiguous_format) if out is None else out
    xx, shape, xs = _nd(x)
    check(lib().ytcuda_rmsnorm(_dt(x), _dt(y), _dt(weight) if weight is not None else F32, x.data_ptr(),
                               weight.data_ptr() if weight is not None else None, y.data_ptr(), shape, xs,
                               _i64(y.stride() or (1,)), xx.dim(), _i32(ax), len(ax), eps, _stream()))
    return y


def rmsNorm_(x, weight, axes=-1, eps: float = 1e-5):
    return rmsNorm(x, weight, axes, eps, out=x)


def layerNorm(x: torch.Tensor, gamma: torch.Tensor | None = None, bias: torch.Tensor | None = None, axes=-1,
              eps: float = 1e-5, out: torch.Tensor | None = None) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) [* gamma + bias] (reference yt::function::layerNorm,
    src/function/normalization.inl:159-230)."""
    _require_cuda(x, gamma, bias, out)
    ax = _axes(axes)
    if (gamma is None) != (bias is None):
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "layerNorm: gamma and bias come together")
    if gamma is not None:
        want = [x.shape[a] for a in ax]
        if list(gamma.shape) != want or list(bias.shape) != want:
            raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "layerNorm: gamma/bias shape must match affine axes")
        gamma, bias = gamma.contiguous(), bias.contiguous().to(gamma.dtype)
    y = torch.empty_like(x, memory_format=torch.contiguous_format) if out is None else out
    xx, shape, xs = _nd(x)
    check(lib().ytcuda_layernorm(_dt(x), _dt(y), _dt(gamma) if gamma is not None else F32, x.data_ptr(),
                                 gamma.data_ptr() if gamma is not None else None,
                                 bias.data_ptr() if bias is not None else None, y.data_ptr(), shape, xs,
                                 _i64(y.stride() or (1,)), xx.dim(), _i32(ax), len(ax), eps, _stream()))
    return y


def layerNorm_(x, gamma=None, bias=None, axes=-1, eps: float = 1e-5):
    return layerNorm(x, gamma, bias, axes, eps, out=x)


def _affine_(y: torch.Tensor, gamma, bias, axes) -> torch.Tensor:
    """y *= gamma; y += bias with gamma / bias holding one dim per axis (the reference's _applyScale_ / _applyBias_,
    src/function/normalization.inl:88-116, through _makeAffineView)."""
    if gamma is None and bias is None:
        return y
    if gamma is None or bias is None:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "gamma and bias come together")
    ax = [a % y.dim() for a in axes]
    want = [y.shape[a] for a in ax]
    if list(gamma.shape) != want or list(bias.shape) != want:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "gamma/bias shape must match affine axes")
    # the reference views the affine tensor's MEMORY with the axis sizes in ascending axis order, whatever order the
    # axes were listed in (src/ytensor_function.inl:137-158): a plain reshape of the contiguous tensor does the same
    view = [1] * y.dim()
    for a in ax:
        view[a] = y.shape[a]
    g = gamma.contiguous().reshape(view)
    b = bias.contiguous().reshape(view)
    _binary("mul", y, g.to(y.dtype), y)
    _binary("add", y, b.to(y.dtype), y)
    return y


def normalize(x: torch.Tensor, axes=-1, p: float = 2.0, eps: float = 1e-12, gamma=None, bias=None,
              out: torch.Tensor | None = None) -> torch.Tensor:
    """x / (sum_axes |x|^p + eps)^(1/p) [* gamma + bias] (reference yt::function::normalize,
    src/function/normalization.inl:56-85, 278-372)."""
    _require_cuda(x, gamma, bias, out)
    if p <= 0:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "yt::function::normalize: p must be positive")
    ax = _axes(axes)
    y = torch.empty_like(x, memory_format=torch.contiguous_format) if out is None else out
    xx, shape, xs = _nd(x)
    check(lib().ytcuda_normalize(_dt(x), _dt(y), x.data_ptr(), y.data_ptr(), shape, xs, _i64(y.stride() or (1,)),
                                 xx.dim(), _i32(ax), len(ax), float(p), float(eps), _stream()))
    return _affine_(y, gamma, bias, ax)


def normalize_(x, axes=-1, p: float = 2.0, eps: float = 1e-12, gamma=None, bias=None):
    return normalize(x, axes, p, eps, gamma, bias, out=x)


def _channel_axis(x: torch.Tensor, channelAxis: int, who: str) -> int:
    c = channelAxis % x.dim()
    if x.dim() < 2:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, f"{who} requires dim >= 2")
    if c == 0:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, f"{who}: channelAxis must not be batch axis 0")
    return c


def instanceNorm(x: torch.Tensor, gamma=None, bias=None, channelAxis: int = 1, eps: float = 1e-5,
                 out: torch.Tensor | None = None) -> torch.Tensor:
    """Standardises every (sample, channel) over the remaining axes (reference yt::function::instanceNorm,
    src/function/normalization.inl:378-433); gamma / bias are per channel."""
    c = _channel_axis(x, channelAxis, "yt::function::instanceNorm_")
    axes = [a for a in range(x.dim()) if a not in (0, c)]
    if not axes:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "yt::function::instanceNorm: requires at least one spatial axis")
    y = layerNorm(x, None, None, axes, eps, out=out)
    return _affine_(y, gamma, bias, [c])


def instanceNorm_(x, gamma=None, bias=None, channelAxis: int = 1, eps: float = 1e-5):
    return instanceNorm(x, gamma, bias, channelAxis, eps, out=x)


def batchNorm(x: torch.Tensor, gamma=None, bias=None, channelAxis: int = 1, eps: float = 1e-5,
              out: torch.Tensor | None = None) -> torch.Tensor:
    """Standardises every channel over all other axes, batch included (reference yt::function::batchNorm,
    src/function/normalization.inl:435-489: statistics of the tensor itself, no running averages)."""
    c = _channel_axis(x, channelAxis, "yt::function::batchNorm_")
    axes = [a for a in range(x.dim()) if a != c]
    y = layerNorm(x, None, None, axes, eps, out=out)
    return _affine_(y, gamma, bias, [c])


def batchNorm_(x, gamma=None, bias=None, channelAxis: int = 1, eps: float = 1e-5):
    return batchNorm(x, gamma, bias, channelAxis, eps, out=x)


def groupNorm(x: torch.Tensor, groups: int, gamma=None, bias=None, channelAxis: int = 1, eps: float = 1e-5,
              out: torch.Tensor | None = None) -> torch.Tensor:
    """Standardises every (sample, group of channels) over the group's channels and the remaining axes (reference
    yt::function::groupNorm, src/function/normalization.inl:491-577). The reference permutes the channel axis to the
    front and copies; here the grouped tensor is a strided VIEW [n, groups, channels / groups, ...] of x and of the
    output, handed to the generic-axes kernel as it is."""
    c = _channel_axis(x, channelAxis, "yt::function::groupNorm_")
    if groups <= 0:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "yt::function::groupNorm: groups must be positive")
    ch = x.shape[c]
    if ch % groups:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG,
                                         "yt::function::groupNorm: channel count must be divisible by groups")
    if x.dim() + 1 > 8:
        raise _lib.YtCudaInvalidArgument(_lib.UNSUPPORTED, "groupNorm: at most 7 dims")
    y = torch.empty_like(x, memory_format=torch.contiguous_format) if out is None else out
    xg = x.movedim(c, 1).unflatten(1, (groups, ch // groups))
    yg = y.movedim(c, 1).unflatten(1, (groups, ch // groups))
    layerNorm(xg, None, None, list(range(2, xg.dim())), eps, out=yg)
    return _affine_(y, gamma, bias, [c])


def groupNorm_(x, groups: int, gamma=None, bias=None, channelAxis: int = 1, eps: float = 1e-5):
    return groupNorm(x, groups, gamma, bias, channelAxis, eps, out=x)


def rmsnorm_add_softmax_cast(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor,
                             out_dtype: torch.dtype = torch.bfloat16, eps: float = 1e-6) -> torch.Tensor:
    """cast(softmax(rmsNorm(x, w, -1, eps) + residual, -1)) in one pass. x [B, L, H] fp32 contiguous,
    residual [B, L, H] or [1, L, H]."""
    _require_cuda(x, weight, residual)
    if x.dim() != 3 or x.dtype != torch.float32 or not x.is_contiguous():
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "chain: x must be a contiguous fp32 [B, L, H] tensor")
    B, Lr, H = x.shape
    if tuple(residual.shape) not in ((B, Lr, H), (1, Lr, H)) or tuple(weight.shape) != (H,):
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "chain: residual / weight shape mismatch")
    residual, weight = residual.contiguous().float(), weight.contiguous().float()
    out = torch.empty(B, Lr, H, dtype=out_dtype, device=x.device)
    check(lib().ytcuda_rmsnorm_add_softmax_cast(_DT[out_dtype], x.data_ptr(), weight.data_ptr(), residual.data_ptr(),
                                                out.data_ptr(), B, Lr, H, int(residual.shape[0] == B), eps, _stream()))
    return out


# ------------------------------------------------------------------ reductions
def _reduce(op: int, x: torch.Tensor, axes, want_index: bool):
    _require_cuda(x)
    ax = _axes(axes)
    xx, shape, xs = _nd(x)
    ks = list(xx.shape)
    for a in ax:
        ks[a % xx.dim()] = 1
    y = torch.empty(ks, dtype=x.dtype, device=x.device)
    idx = torch.empty(ks, dtype=torch.int32, device=x.device) if want_index else None
    check(lib().ytcuda_reduce(op, _dt(x), _dt(y), x.data_ptr(), y.data_ptr(), idx.data_ptr() if want_index else None,
                              shape, xs, xx.dim(), _i32(ax), len(ax), _stream()))
    return (y, idx) if want_index else y


def sum(x: torch.Tensor, axes) -> torch.Tensor:  # noqa: A001 - mirrors YTensor::sum
    """Keep-dim sum over an axis or axes (reference YTensor::sum, src/ytensor_math.inl:414-509)."""
    return _reduce(0, x, axes, False)


def mean(x: torch.Tensor, axes) -> torch.Tensor:
    """Keep-dim mean (reference YTensor::mean, src/ytensor_math.inl:531-574)."""
    return _reduce(1, x, axes, False)


def max(x: torch.Tensor, axes):  # noqa: A001 - mirrors YTensor::max
    """Keep-dim maximum and the int index of its first occurrence (reference YTensor::max,
    src/ytensor_math.inl:591-692)."""
    return _reduce(2, x, axes, True)


# ------------------------------------------------------------------ elementwise
_BIN = {"add": 0, "sub": 1, "mul": 2, "div": 3}


def _binary(op: str, a: torch.Tensor, b, out: torch.Tensor | None) -> torch.Tensor:
    if not isinstance(b, torch.Tensor):
        return _unary({"add": 3, "sub": 3, "mul": 2, "div": 2}[op], a, out,
                      {"add": float(b), "sub": -float(b), "mul": float(b), "div": 1.0 / float(b)}[op])
    _require_cuda(a, b, out)
    try:
        shape = torch.broadcast_shapes(a.shape, b.shape)
    except RuntimeError as e:  # std::runtime_error in the reference (src/kernel/broadcast.inl:133)
        raise _lib.YtCudaError(_lib.INVALID_ARG, f"broadcast mismatch: {e}")
    if out is None:
        out = torch.empty(shape, dtype=a.dtype, device=a.device)
    elif tuple(out.shape) != tuple(shape):
        raise _lib.YtCudaError(_lib.INVALID_ARG, "in-place operand cannot be broadcast to the result shape")
    ae, be = a.expand(shape), b.expand(shape)
    if len(shape) == 0:
        ae, be, o = ae.reshape(1), be.reshape(1), out.reshape(1)
    else:
        o = out
    check(lib().ytcuda_binary(_BIN[op], _dt(a), _dt(b), _dt(out), ae.data_ptr(), be.data_ptr(), o.data_ptr(), o.dim(),
                              _i64(o.shape), _i64(ae.stride()), _i64(be.stride()), _i64(o.stride()), _stream()))
    return out


def add(a, b): return _binary("add", a, b, None)
def sub(a, b): return _binary("sub", a, b, None)
def mul(a, b): return _binary("mul", a, b, None)
def div(a, b): return _binary("div", a, b, None)
def add_(a, b): return _binary("add", a, b, a)
def sub_(a, b): return _binary("sub", a, b, a)
def mul_(a, b): return _binary("mul", a, b, a)
def div_(a, b): return _binary("div", a, b, a)


def _unary(op: int, x: torch.Tensor, out: torch.Tensor | None, param: float = 0.0,
           out_dtype: torch.dtype | None = None) -> torch.Tensor:
    _require_cuda(x, out)
    if out is None:
        out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    elif tuple(out.shape) != tuple(x.shape):
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "unary: shape mismatch")
    xx, oo = (x.reshape(1), out.reshape(1)) if x.dim() == 0 else (x, out)
    check(lib().ytcuda_unary(op, _dt(x), _dt(out), xx.data_ptr(), oo.data_ptr(), xx.dim(), _i64(xx.shape),
                             _i64(xx.stride()), _i64(oo.stride()), param, _stream()))
    return out


def swish(x, order=0): return _unary(_act_op("swish", 1, order), x, None)


def swish_(x, order=0):
    """x * sigmoid(x) in place (reference yt::function::swish_, src/function/activation.inl:631-647); order 1: its
    first derivative."""
    return _unary(_act_op("swish", 1, order), x, x)

# The other activations of yt::function (reference src/function/activation.inl); `name_` works in place.
_ACTIVATIONS = {"relu": 4, "exp": 5, "sigmoid": 6, "leakyRelu": 7, "elu": 8, "selu": 9, "gelu": 10, "tanh": 11,
                "softplus": 12, "mish": 13, "hardSigmoid": 14, "hardSwish": 15}
_ACT_DEFAULT_PARAM = {"leakyRelu": 0.01, "elu": 1.0}


def _act_op(name: str, op: int, order: int) -> int:
    if order == 0:
        return op
    if order == 1:
        return 32 + op
    raise _lib.YtCudaInvalidArgument(_lib.UNSUPPORTED, f"{name}: order {order} is not on the device (0 and 1 are)")


def _make_activation(name: str, op: int):
    default = _ACT_DEFAULT_PARAM.get(name)
    if default is None:
        def f(x, order=0):
            return _unary(_act_op(name, op, order), x, None, 0.0)

        def f_(x, order=0):
            return _unary(_act_op(name, op, order), x, x, 0.0)
    else:
        def f(x, alpha=default, order=0):
            return _unary(_act_op(name, op, order), x, None, float(alpha))

        def f_(x, alpha=default, order=0):
            return _unary(_act_op(name, op, order), x, x, float(alpha))

    f.__name__, f_.__name__ = name, name + "_"
    f.__doc__ = f_.__doc__ = (f"yt::function::{name} (reference src/function/activation.inl): order 0 the function, "
                              "order 1 its first derivative.")
    return f, f_


for _n, _op in _ACTIVATIONS.items():
    globals()[_n], globals()[_n + "_"] = _make_activation(_n, _op)


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """dtype conversion with the reference's rounding (YTensorBase::cast, include/ytensor_base.hpp:399-404)."""
    _require_cuda(x)
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    return copy_(out, x)


FP8_KINDS = {"float8_e5m2": _lib.F8_E5M2, "float8_e4m3": _lib.F8_E4M3, "float8_e8m0": _lib.F8_E8M0}


def cast_to_fp8(x: torch.Tensor, kind: str) -> torch.Tensor:
    """float / bfloat16 / float16 -> the reference's 8-bit storage types (yt::float8_e5m2, float8_e4m3, float8_e8m0,
    include/types/float_spec.hpp:534-536) as uint8 bit patterns, with FloatSpec::fromFloat32's rounding (:435-491).
    These are the reference's own formats (the largest exponent is infinity / NaN), not the OCP fn variants, so the
    result is a uint8 tensor rather than a torch float8 dtype."""
    _require_cuda(x)
    out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    s_, d = (x.reshape(1), out.reshape(1)) if x.dim() == 0 else (x, out)
    check(lib().ytcuda_cast(_dt(x), FP8_KINDS[kind], s_.data_ptr(), d.data_ptr(), d.dim(), _i64(d.shape),
                            _i64(s_.stride()), _i64(d.stride()), _stream()))
    return out


def cast_from_fp8(bits: torch.Tensor, kind: str, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """uint8 bit patterns of one of the reference's 8-bit types -> float / bfloat16 / float16 (FloatSpec::toFloat32,
    include/types/float_spec.hpp:299-371, then the target type's own constructor)."""
    _require_cuda(bits)
    if bits.dtype != torch.uint8:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "cast_from_fp8: uint8 bit patterns expected")
    out = torch.empty(bits.shape, dtype=dtype, device=bits.device)
    s_, d = (bits.reshape(1), out.reshape(1)) if bits.dim() == 0 else (bits, out)
    check(lib().ytcuda_cast(FP8_KINDS[kind], _dt(out), s_.data_ptr(), d.data_ptr(), d.dim(), _i64(d.shape),
                            _i64(s_.stride()), _i64(d.stride()), _stream()))
    return out


def copy_(dst: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """Strided copy with conversion (YTensorBase::copy_, src/ytensor_base.inl:257-430)."""
    _require_cuda(dst, src)
    if tuple(dst.shape) != tuple(src.shape):
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "copy_: shape mismatch")
    d, s_ = (dst.reshape(1), src.reshape(1)) if dst.dim() == 0 else (dst, src)
    check(lib().ytcuda_cast(_dt(src), _dt(dst), s_.data_ptr(), d.data_ptr(), d.dim(), _i64(d.shape), _i64(s_.stride()),
                            _i64(d.stride()), _stream()))
    return dst


def topk_sample(logits: torch.Tensor, k: int = 20, uniform: torch.Tensor | None = None):
    """Top-k sampling as qwen3::Qwen3ForCausalLM::generate does it (example/qwen3/src/qwen3.cpp:465-486).

    logits fp32 [rows, vocab]. Returns (top_probs [rows, k], top_idx [rows, k] int32, sampled [rows] int32 or None):
    the k most probable tokens of softmax(logits) in descending order and, when `uniform` (fp32 [rows], numbers in
    [0, 1]) is given, the token whose running sum first reaches uniform * sum(top_probs)."""
    _require_cuda(logits, uniform)
    if logits.dim() != 2 or logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "topk_sample: logits must be fp32 [rows, vocab], unit stride")
    rows, vocab = logits.shape
    probs = torch.empty(rows, k, dtype=torch.float32, device=logits.device)
    idx = torch.empty(rows, k, dtype=torch.int32, device=logits.device)
    sampled = None
    if uniform is not None:
        if uniform.dtype != torch.float32 or uniform.numel() != rows or not uniform.is_contiguous():
            raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "topk_sample: uniform must be fp32 [rows]")
        sampled = torch.empty(rows, dtype=torch.int32, device=logits.device)
    check(lib().ytcuda_topk_sample(logits.data_ptr(), logits.stride(0), rows, vocab, k,
                                   uniform.data_ptr() if uniform is not None else None, probs.data_ptr(),
                                   idx.data_ptr(), sampled.data_ptr() if sampled is not None else None, _stream()))
    return probs, idx, sampled


def swiglu(gate_up: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """swish(gate) * up for a fused [..., 2*I] projection (example/qwen3/src/qwen3.cpp:193-200)."""
    _require_cuda(gate_up)
    if gate_up.stride(-1) != 1 or gate_up.shape[-1] % 2:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "swiglu: last dim must be contiguous and even")
    inter = gate_up.shape[-1] // 2
    g2 = gate_up.reshape(-1, 2 * inter)
    out = torch.empty(*gate_up.shape[:-1], inter, dtype=out_dtype or gate_up.dtype, device=gate_up.device)
    check(lib().ytcuda_swiglu(_dt(g2), _dt(out), g2.data_ptr(), out.data_ptr(), g2.shape[0], inter, g2.stride(0), inter,
                              _stream()))
    return out


# ------------------------------------------------------------------ attention
def _heads_view(t: torch.Tensor, what: str):
    """[batch..., heads..., len, dim] -> (tensor, batch, heads, strides {batch, head, row}); the leading dims must
    collapse into one batch stride and one head stride, and the last dim must have unit stride."""
    if t.stride(-1) != 1 and t.shape[-1] != 1:
        t = copy_(torch.empty(t.shape, dtype=t.dtype, device=t.device), t)
    return t


def scaledDotProductAttention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, scale: float = 0.0,
                              mask: torch.Tensor | None = None, bias: torch.Tensor | None = None, *,
                              causal: bool = False, causal_offset: int | None = None) -> torch.Tensor:
    """softmax(scale * Q K^T + bias, masked) V (reference yt::function::scaledDotProductAttention,
    src/function/ops.inl:368-425).

    Shapes as the reference's callers use them: query [b, kv_heads, groups, q_len, d] with key / value either the
    zero-stride repeat [b, kv_heads, groups, kv_len, d] or plain [b, kv_heads, kv_len, d]; 4-D query
    [b, heads, q_len, d] with [b, kv_heads, kv_len, d] keys (heads a multiple of kv_heads); 3-D and 2-D forms have no
    batch / head dims. `mask` is a bool [q_len, kv_len] tensor; `causal=True` is the predicate form c <= r + offset
    with offset = kv_len - q_len unless given. Mismatched shapes raise ValueError like std::invalid_argument."""
    _require_cuda(query, key, value, mask, bias)
    if query.shape[-1] != key.shape[-1]:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "Query and key head dim must match.")
    if key.shape[-2] != value.shape[-2]:
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "Key/value sequence length must match.")
    if not (query.dtype == key.dtype == value.dtype):
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "scaledDotProductAttention: dtypes differ")
    lq, d = query.shape[-2:]
    lk, dv = value.shape[-2:]
    out_shape = (*query.shape[:-1], dv)
    q, k, v = query, key, value
    if q.dim() == 5:
        b, kvh, g = q.shape[:3]
        if k.dim() == 5:
            k, v = k[:, :, 0], v[:, :, 0]
        q = q.reshape(b, kvh * g, lq, d)
    elif q.dim() == 4:
        b, h = q.shape[:2]
        kvh = k.shape[1]
        if h % kvh:
            raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "query heads must be a multiple of key/value heads")
        g = h // kvh
    else:
        lead = q.shape[:-2]
        n = 1
        for x in lead:
            n *= x
        q, k, v = q.reshape(1, n, lq, d), k.reshape(1, n, lk, d), v.reshape(1, n, lk, dv)
        b, kvh, g = 1, n, 1
    if tuple(k.shape) != (b, kvh, lk, d) or tuple(v.shape) != (b, kvh, lk, dv):
        raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, "key/value batch or head dims do not match the query")
    q, k, v = _heads_view(q, "query"), _heads_view(k, "key"), _heads_view(v, "value")
    mask_kind, mptr, mrs, off = 0, None, 0, 0
    if mask is not None:
        if tuple(mask.shape) != (lq, lk):
            raise _lib.YtCudaInvalidArgument(
                _lib.INVALID_ARG, "Mask shape must match the last two dimensions of the score tensor.")
        m8 = mask.to(torch.uint8) if mask.dtype != torch.uint8 else mask
        m8 = m8.contiguous()
        mask_kind, mptr, mrs = 2, m8.data_ptr(), m8.stride(0)
    elif causal:
        mask_kind, off = 1, (lk - lq) if causal_offset is None else int(causal_offset)
    bptr, brs, bcs = None, 0, 0
    if bias is not None:
        if tuple(bias.shape) != (lq, lk):
            raise _lib.YtCudaInvalidArgument(
                _lib.INVALID_ARG, "Bias shape must match the last two dimensions of the score tensor.")
        bias = bias.float()
        bptr, brs, bcs = bias.data_ptr(), bias.stride(0), bias.stride(1)
    out = torch.empty(b, kvh * g, lq, dv, dtype=query.dtype, device=query.device)
    check(lib().ytcuda_flash_attn_fwd(_dt(q), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), b, kvh, g, lq,
                                      lk, d, dv, float(scale), _i64(q.stride()[:3]), _i64(k.stride()[:3]),
                                      _i64(v.stride()[:3]), _i64(out.stride()[:3]), mask_kind, off, mptr, mrs, bptr,
                                      brs, bcs, _stream()))
    return out.reshape(out_shape)
