"""TEST INFRASTRUCTURE: numpy front-end of the CPU oracle.

Two back-ends with the same call surface:
  * `port`  - oracle/libyt_oracle.so, the plain-C restatement in yt_oracle.c (always available
              after `make -C oracle liboracle`);
  * `ref`   - oracle/_ref/libyt_ref.so, the unmodified reference compiled behind ref_shim.cpp
              (available where it was built from the reference sources).
Only tests, the smoke check and the benchmark's CPU-baseline legs may import this module.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
PORT_LIB = HERE / "libyt_oracle.so"
REF_LIB = HERE / "_ref" / "libyt_ref.so"

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")


def build_port() -> Path:
    subprocess.run(["make", "-s", "-C", str(HERE), "liboracle"], check=True)
    return PORT_LIB


def build_ref() -> Path | None:
    subprocess.run(["make", "-s", "-C", str(HERE), "ref"], check=True)
    return REF_LIB if REF_LIB.exists() else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ints(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _opt(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class _Backend:
    prefix = ""

    def __init__(self, path: Path):
        self.lib = C.CDLL(str(path))

    def _fn(self, name):
        return getattr(self.lib, self.prefix + name)

    # ---- casts -------------------------------------------------------------------------
    def f32_to_bf16(self, x):
        x = _f32(x)
        y = np.empty(x.shape, np.uint16)
        self._fn("f32_to_bf16")(_opt(x), _opt(y), C.c_int64(x.size))
        return y

    def bf16_to_f32(self, x):
        x = np.ascontiguousarray(x, np.uint16)
        y = np.empty(x.shape, np.float32)
        self._fn("bf16_to_f32")(_opt(x), _opt(y), C.c_int64(x.size))
        return y

    def f32_to_f16(self, x):
        x = _f32(x)
        y = np.empty(x.shape, np.uint16)
        self._fn("f32_to_f16")(_opt(x), _opt(y), C.c_int64(x.size))
        return y

    def f16_to_f32(self, x):
        x = np.ascontiguousarray(x, np.uint16)
        y = np.empty(x.shape, np.float32)
        self._fn("f16_to_f32")(_opt(x), _opt(y), C.c_int64(x.size))
        return y

    # ---- N-d ops -----------------------------------------------------------------------
    def softmax(self, x, axes):
        x = _f32(x)
        y = np.empty_like(x)
        axes = _ints(np.atleast_1d(axes))
        rc = self._fn("softmax_f32")(_opt(x), _opt(y), _opt(_ints(x.shape)), x.ndim, _opt(axes), axes.size)
        assert rc == 0, rc
        return y

    def topk_sample(self, logits, k=20, uniform=None):
        """sample_token of Qwen3ForCausalLM::generate (reference example/qwen3/src/qwen3.cpp:465-486): softmax over
        the row, the k largest probabilities in descending order (stable: the lower index first on ties), and the
        token whose running sum first reaches uniform * sum(kept), the first kept token otherwise."""
        probs = self.softmax(_f32(logits), [-1])
        order = np.argsort(-probs, axis=1, kind="stable")[:, :k]
        top = np.take_along_axis(probs, order, axis=1)
        sampled = None
        if uniform is not None:
            sampled = np.empty(probs.shape[0], np.int32)
            for r in range(probs.shape[0]):
                kept = np.float32(0)
                for j in range(k):
                    kept = np.float32(kept + top[r, j])
                target, cum, pick = np.float32(uniform[r]) * kept, np.float32(0), order[r, 0]
                for j in range(k):
                    cum = np.float32(cum + top[r, j])
                    if target <= cum:
                        pick = order[r, j]
                        break
                sampled[r] = pick
        return top, order.astype(np.int32), sampled

    def rmsnorm(self, x, w, axes, eps):
        x, w = _f32(x), _f32(w)
        y = np.empty_like(x)
        axes = _ints(np.atleast_1d(axes))
        rc = self._fn("rmsnorm_f32")(_opt(x), _opt(w), _opt(y), _opt(_ints(x.shape)), x.ndim, _opt(axes), axes.size,
                                     C.c_float(eps))
        assert rc == 0, rc
        return y

    def layernorm(self, x, gamma, beta, axes, eps):
        x = _f32(x)
        g = None if gamma is None else _f32(gamma)
        b = None if beta is None else _f32(beta)
        y = np.empty_like(x)
        axes = _ints(np.atleast_1d(axes))
        rc = self._fn("layernorm_f32")(_opt(x), _opt(g), _opt(b), _opt(y), _opt(_ints(x.shape)), x.ndim, _opt(axes),
                                       axes.size, C.c_float(eps))
        assert rc == 0, rc
        return y

    def norm(self, kind, x, axes, gamma=None, bias=None, groups=1, p=2.0, eps=1e-5):
        """kind: 'normalize' (Lp over axes) | 'instanceNorm' | 'batchNorm' | 'groupNorm' (axes = [channel axis])
        (reference yt::function::normalize / instanceNorm / batchNorm / groupNorm, src/function/normalization.inl:
        278-577). Reference back-end only."""
        x = _f32(x)
        y = np.empty_like(x)
        axes = _ints(np.atleast_1d(axes))
        g = None if gamma is None else _f32(gamma)
        b = None if bias is None else _f32(bias)
        k = {"normalize": 0, "instanceNorm": 1, "batchNorm": 2, "groupNorm": 3}[kind]
        rc = self._fn("norm_f32")(k, _opt(x), _opt(g), _opt(b), _opt(y), _opt(_ints(x.shape)), x.ndim, _opt(axes),
                                  axes.size, int(groups), C.c_float(p), C.c_float(eps))
        assert rc == 0, rc
        return y

    def fp8(self, kind, x):
        """float32 -> bits of yt::float8_e5m2 / float8_e4m3 / float8_e8m0 (kind 'float8_e5m2' ...). Reference only."""
        x = _f32(x)
        out = np.empty(x.shape, np.uint8)
        k = {"float8_e5m2": 3, "float8_e4m3": 4, "float8_e8m0": 5}[kind]
        rc = self._fn("f32_to_fp8")(k, _opt(x), _opt(out), C.c_int64(x.size))
        assert rc == 0, rc
        return out

    def fp8_to_f32(self, kind, bits):
        bits = np.ascontiguousarray(bits, np.uint8)
        out = np.empty(bits.shape, np.float32)
        k = {"float8_e5m2": 3, "float8_e4m3": 4, "float8_e8m0": 5}[kind]
        rc = self._fn("fp8_to_f32")(k, _opt(bits), _opt(out), C.c_int64(bits.size))
        assert rc == 0, rc
        return out

    def reduce(self, x, axes, op):
        """op: 'sum' | 'mean' | 'max'. Returns keep-dim result (and int32 indices for max)."""
        x = _f32(x)
        axes = _ints(np.atleast_1d(axes))
        ks = list(x.shape)
        for a in axes:
            ks[int(a) % x.ndim] = 1
        y = np.empty(ks, np.float32)
        idx = np.zeros(ks, np.int32)
        code = {"sum": 0, "mean": 1, "max": 2}[op]
        rc = self._fn("reduce_f32")(_opt(x), _opt(y), _opt(idx), _opt(_ints(x.shape)), x.ndim, _opt(axes), axes.size,
                                    code)
        assert rc == 0, rc
        return (y, idx) if op == "max" else y

    def binary(self, a, b, op):
        a, b = _f32(a), _f32(b)
        nd = max(a.ndim, b.ndim)
        a = a.reshape((1,) * (nd - a.ndim) + a.shape)
        b = b.reshape((1,) * (nd - b.ndim) + b.shape)
        out = np.empty(np.broadcast_shapes(a.shape, b.shape), np.float32)
        code = {"add": 0, "sub": 1, "mul": 2, "div": 3}[op]
        rc = self._fn("binary_f32")(_opt(a), _opt(_ints(a.shape)), _opt(b), _opt(_ints(b.shape)), nd, _opt(out), code)
        assert rc == 0, rc
        return out

    def qwen3(self, cfg: dict, batch: int = 1) -> "_Qwen3Handle":
        return _Qwen3Handle(self, cfg, batch)

    def swish(self, x):
        x = _f32(x)
        y = np.empty_like(x)
        self._fn("swish_f32")(_opt(x), _opt(y), C.c_int64(x.size))
        return y

    ACTIVATIONS = {"swish": 1, "relu": 4, "exp": 5, "sigmoid": 6, "leakyRelu": 7, "elu": 8, "selu": 9, "gelu": 10,
                   "tanh": 11, "softplus": 12, "mish": 13, "hardSigmoid": 14, "hardSwish": 15}

    def activation(self, name, x, alpha=None, order=0):
        """yt::function::<name> (reference include/function/activation.hpp:9-109): order 0 the function, order 1 its
        first derivative."""
        x = _f32(x)
        y = np.empty_like(x)
        if alpha is None:
            alpha = {"leakyRelu": 0.01, "elu": 1.0}.get(name, 0.0)
        if order == 0:
            rc = self._fn("activation_f32")(self.ACTIVATIONS[name], _opt(x), _opt(y), C.c_int64(x.size),
                                            C.c_float(alpha))
        else:
            rc = self._fn("activation_order_f32")(self.ACTIVATIONS[name], int(order), _opt(x), _opt(y),
                                                  C.c_int64(x.size), C.c_float(alpha))
        assert rc == 0, rc
        return y

    def chain(self, x, w, r, eps=1e-6):
        x, w, r = _f32(x), _f32(w), _f32(r)
        B, L, H = x.shape
        out = np.empty(x.shape, np.uint16)
        rc = self._fn("chain_f32")(_opt(x), _opt(w), _opt(r), _opt(out), B, L, H, int(r.shape[0] == B),
                                   C.c_float(eps))
        assert rc == 0, rc
        return out

    def sdpa(self, q, k, v, scale=0.0, mask=None, causal=False, bias=None, **kw):
        """q [b,kvh,g,ql,d], k [b,kvh,kl,d], v [b,kvh,kl,dv] -> [b,kvh,g,ql,dv]."""
        q, k, v = _f32(q), _f32(k), _f32(v)
        b, kvh, g, ql, d = q.shape
        kl, dv = k.shape[2], v.shape[3]
        out = np.empty((b, kvh, g, ql, dv), np.float32)
        kind, m = 0, None
        if mask is not None:
            kind, m = 1, np.ascontiguousarray(mask, np.uint8)
        elif causal:
            kind = 2
        bs = None if bias is None else _f32(bias)
        rc = self._sdpa(q, k, v, out, b, kvh, g, ql, kl, d, dv, scale, kind, m, bs, **kw)
        assert rc == 0, rc
        return out


class _Qwen3Handle:
    """The reference's Qwen3ForCausalLM (ref back-end) or its restatement (port back-end) on the CPU."""

    def __init__(self, backend: "_Backend", cfg: dict, batch: int):
        self.be, self.cfg, self.batch = backend, cfg, batch
        create = backend._fn("qwen3_create")
        create.restype = C.c_void_p
        self.h = C.c_void_p(create(cfg["hidden"], cfg["layers"], cfg["vocab"], cfg["inter"], cfg["heads"],
                                   cfg["kv_heads"], cfg["head_dim"], C.c_float(cfg["eps"]), C.c_float(cfg["theta"]),
                                   cfg["max_pos"], batch))
        assert self.h.value, "qwen3_create failed"

    def set_weight(self, name: str, layer: int, data_f32: np.ndarray):
        a = _f32(data_f32)
        rows, cols = (a.shape[0], a.shape[1]) if a.ndim == 2 else (a.shape[0], 1)
        rc = self.be._fn("qwen3_set_weight")(self.h, name.encode(), layer, _opt(a), rows, cols)
        assert rc == 0, (name, rc)

    def reset(self):
        self.be._fn("qwen3_reset")(self.h)

    def forward(self, ids: np.ndarray) -> np.ndarray:
        ids = np.ascontiguousarray(ids, np.int32)
        assert ids.shape[0] == self.batch
        logits = np.empty((self.batch, self.cfg["vocab"]), np.float32)
        rc = self.be._fn("qwen3_forward")(self.h, _opt(ids), ids.shape[1], _opt(logits))
        assert rc == 0, rc
        return logits

    def close(self):
        if self.h:
            fn = self.be._fn("qwen3_destroy")
            fn.restype = None
            fn(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class PortOracle(_Backend):
    prefix = "yto_"

    def norm(self, kind, x, axes, gamma=None, bias=None, groups=1, p=2.0, eps=1e-5):
        """Restatement of yt::function::normalize / instanceNorm / batchNorm / groupNorm
        (src/function/normalization.inl:56-116, 278-577) on top of the port's standardisation (layernorm without
        affine) and broadcast operators: the channel norms standardise over the axes the reference's _instanceAxes /
        _batchAxes name; groupNorm does it on the [n, groups, channels / groups, ...] view of the channel-first
        tensor; gamma and bias are applied afterwards along the channel axis (or the single normalised axis)."""
        x = _f32(x)
        nd = x.ndim
        axes = [int(a) % nd for a in np.atleast_1d(axes)]

        def affine(y, ax):
            if gamma is None:
                return y
            view = [1] * nd
            view[ax] = x.shape[ax]
            g, b = _f32(gamma).reshape(view), _f32(bias).reshape(view)
            return self.binary(self.binary(y, np.broadcast_to(g, [1 if i != ax else x.shape[ax] for i in range(nd)]),
                                           "mul"), b, "add")

        if kind == "normalize":
            ap = np.abs(x).astype(np.float32) ** np.float32(p)
            s = self.reduce(ap.astype(np.float32), axes, "sum")
            y = (x / (s + np.float32(eps)) ** np.float32(1.0 / p)).astype(np.float32)
            return affine(y, axes[0]) if gamma is not None else y
        c = axes[0]
        if kind == "instanceNorm":
            y = self.layernorm(x, None, None, [a for a in range(nd) if a not in (0, c)], eps)
        elif kind == "batchNorm":
            y = self.layernorm(x, None, None, [a for a in range(nd) if a != c], eps)
        else:
            xc = np.ascontiguousarray(np.moveaxis(x, c, 1))
            grouped = xc.reshape((xc.shape[0], groups, xc.shape[1] // groups) + xc.shape[2:])
            yg = self.layernorm(grouped, None, None, list(range(2, grouped.ndim)), eps)
            y = np.ascontiguousarray(np.moveaxis(yg.reshape(xc.shape), 1, c))
        return affine(y, c)

    def fp8(self, kind, x):
        x = _f32(x)
        out = np.empty(x.shape, np.uint8)
        rc = self.lib.yto_f32_to_fp8({"float8_e5m2": 3, "float8_e4m3": 4, "float8_e8m0": 5}[kind], _opt(x), _opt(out),
                                     C.c_int64(x.size))
        assert rc == 0, rc
        return out

    def fp8_to_f32(self, kind, bits):
        bits = np.ascontiguousarray(bits, np.uint8)
        out = np.empty(bits.shape, np.float32)
        rc = self.lib.yto_fp8_to_f32({"float8_e5m2": 3, "float8_e4m3": 4, "float8_e8m0": 5}[kind], _opt(bits),
                                     _opt(out), C.c_int64(bits.size))
        assert rc == 0, rc
        return out

    def masked_matmul_causal(self, a, b, offset, masked_value=0.0):
        m, n = np.asarray(a).shape[-2], np.asarray(b).shape[-1]
        mask = np.arange(n)[None, :] <= np.arange(m)[:, None] + int(offset)
        return self.masked_matmul(a, b, mask, masked_value)

    def __init__(self):
        if not PORT_LIB.exists():
            build_port()
        super().__init__(PORT_LIB)

    def matmul(self, a, b):
        """a [batch,m,k] (or [m,k]) . b [k,n] or [batch,k,n], fp32."""
        a, b = _f32(a), _f32(b)
        a3 = a.reshape((-1,) + a.shape[-2:])
        batch, m, k = a3.shape
        n = b.shape[-1]
        bb = int(b.ndim == 3)
        c = np.empty((batch, m, n), np.float32)
        self.lib.yto_matmul_f32(_opt(a3), _opt(b), _opt(c), batch, m, n, k, bb)
        return c.reshape(a.shape[:-1] + (n,))

    def masked_matmul(self, a, b, mask, masked_value=0.0):
        """a [batch,m,k] . b [k,n] or [batch,k,n] where mask [m,n] (bool), masked_value elsewhere; fp32."""
        a, b = _f32(a), _f32(b)
        a3 = a.reshape((-1,) + a.shape[-2:])
        batch, m, k = a3.shape
        n = b.shape[-1]
        mk = np.ascontiguousarray(mask, np.uint8)
        c = np.empty((batch, m, n), np.float32)
        self.lib.yto_masked_matmul_f32(_opt(a3), _opt(b), _opt(mk), C.c_float(masked_value), _opt(c), batch, m, n, k,
                                       int(b.ndim == 3))
        return c.reshape(a.shape[:-1] + (n,))

    def matmul_16(self, a_bits, b_bits, dtype):
        """bf16 (dtype=1) / fp16 (dtype=2) storage, fp32 compute; uint16 bit patterns in and out."""
        a = np.ascontiguousarray(a_bits, np.uint16)
        b = np.ascontiguousarray(b_bits, np.uint16)
        a3 = a.reshape((-1,) + a.shape[-2:])
        batch, m, k = a3.shape
        n = b.shape[-1]
        c = np.empty((batch, m, n), np.uint16)
        self.lib.yto_matmul_16(_opt(a3), _opt(b), _opt(c), batch, m, n, k, int(b.ndim == 3), dtype)
        return c.reshape(a.shape[:-1] + (n,))

    def sgemm(self, A, B, Cin, alpha, beta):
        """Strided form on numpy views: returns alpha*A@B + beta*Cin (fp32)."""
        A, B = np.asarray(A, np.float32), np.asarray(B, np.float32)
        out = np.array(Cin, np.float32, copy=True, order="C")
        m, k = A.shape
        n = B.shape[1]
        es = 4
        self.lib.yto_sgemm(C.c_void_p(A.ctypes.data), C.c_void_p(B.ctypes.data), _opt(out), m, n, k, C.c_float(alpha),
                           C.c_float(beta), C.c_int64(A.strides[0] // es), C.c_int64(A.strides[1] // es),
                           C.c_int64(B.strides[0] // es), C.c_int64(B.strides[1] // es), C.c_int64(n), C.c_int64(1))
        return out

    def _sdpa(self, q, k, v, out, b, kvh, g, ql, kl, d, dv, scale, kind, m, bs):
        return self.lib.yto_sdpa_f32(_opt(q), _opt(k), _opt(v), _opt(out), b, kvh, g, ql, kl, d, dv, C.c_float(scale),
                                     kind, _opt(m), _opt(bs))


class RefOracle(_Backend):
    prefix = "ytref_"

    def __init__(self, threads: int = 0):
        if not REF_LIB.exists():
            raise FileNotFoundError(f"{REF_LIB} is not built (needs the reference sources)")
        super().__init__(REF_LIB)
        self.lib.ytref_set_threads(threads)
        self.lib.ytref_qwen3_create.restype = C.c_void_p

    def threads(self) -> int:
        return self.lib.ytref_get_threads()

    def matmul(self, a, b, backend=2):
        a, b = _f32(a), _f32(b)
        a3 = a.reshape((-1,) + a.shape[-2:])
        batch, m, k = a3.shape
        n = b.shape[-1]
        c = np.empty((batch, m, n), np.float32)
        rc = self.lib.ytref_matmul_f32(_opt(a3), _opt(b), _opt(c), batch, m, n, k, int(b.ndim == 3), backend)
        assert rc == 0, rc
        return c.reshape(a.shape[:-1] + (n,))

    def masked_matmul(self, a, b, mask, masked_value=0.0, backend=2):
        a, b = _f32(a), _f32(b)
        a3 = a.reshape((-1,) + a.shape[-2:])
        batch, m, k = a3.shape
        n = b.shape[-1]
        mk = np.ascontiguousarray(mask, np.uint8)
        c = np.empty((batch, m, n), np.float32)
        rc = self.lib.ytref_masked_matmul_f32(_opt(a3), _opt(b), _opt(mk), C.c_float(masked_value), _opt(c), batch, m,
                                              n, k, int(b.ndim == 3), backend)
        assert rc == 0, rc
        return c.reshape(a.shape[:-1] + (n,))

    def masked_matmul_causal(self, a, b, offset, masked_value=0.0):
        a, b = _f32(a), _f32(b)
        a3 = a.reshape((-1,) + a.shape[-2:])
        batch, m, k = a3.shape
        n = b.shape[-1]
        c = np.empty((batch, m, n), np.float32)
        rc = self.lib.ytref_masked_matmul_causal_f32(_opt(a3), _opt(b), int(offset), C.c_float(masked_value), _opt(c),
                                                     batch, m, n, k)
        assert rc == 0, rc
        return c.reshape(a.shape[:-1] + (n,))

    def matmul_16(self, a_bits, b_bits, dtype):
        """The recipe for 16-bit storage: widen, YTensor<float>::matmul, narrow with the type's constructor."""
        widen = self.bf16_to_f32 if dtype == 1 else self.f16_to_f32
        narrow = self.f32_to_bf16 if dtype == 1 else self.f32_to_f16
        return narrow(self.matmul(widen(a_bits), widen(b_bits)))

    def linear(self, x, w, bias=None):
        x, w = _f32(x), _f32(w)
        rows, k = x.shape
        n = w.shape[0]
        y = np.empty((rows, n), np.float32)
        bs = None if bias is None else _f32(bias)
        rc = self.lib.ytref_linear_f32(_opt(x), _opt(w), _opt(bs), _opt(y), rows, n, k)
        assert rc == 0, rc
        return y

    def sgemm(self, A, B, Cin, alpha, beta):
        A, B = np.asarray(A, np.float32), np.asarray(B, np.float32)
        out = np.array(Cin, np.float32, copy=True, order="C")
        m, k = A.shape
        n = B.shape[1]
        es = 4
        self.lib.ytref_sgemm_strided(C.c_void_p(A.ctypes.data), C.c_void_p(B.ctypes.data), _opt(out), m, n, k,
                                     C.c_float(alpha), C.c_float(beta), C.c_int64(A.strides[0] // es),
                                     C.c_int64(A.strides[1] // es), C.c_int64(B.strides[0] // es),
                                     C.c_int64(B.strides[1] // es), C.c_int64(n), C.c_int64(1))
        return out

    def _sdpa(self, q, k, v, out, b, kvh, g, ql, kl, d, dv, scale, kind, m, bs, backend=1):
        return self.lib.ytref_sdpa_f32(_opt(q), _opt(k), _opt(v), _opt(out), b, kvh, g, ql, kl, d, dv, C.c_float(scale),
                                       kind, _opt(m), _opt(bs), backend)


_port = None
_ref = None


def port() -> PortOracle:
    global _port
    if _port is None:
        _port = PortOracle()
    return _port


def ref_available() -> bool:
    return REF_LIB.exists()


def ref(threads: int = 0) -> RefOracle:
    global _ref
    if _ref is None:
        _ref = RefOracle(threads)
    return _ref
