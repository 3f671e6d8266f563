"""GPU test of ytcuda_reduce_noalloc, the entry point for callers that may not allocate device memory while they
run (real-time loops, processes with a fixed device-memory budget): its results must equal those of ytcuda_reduce, call after call,
although every call reuses the same fixed scratch array inside the library.

The file name keeps this test last in collection order, so that a run stopping at the first failure has already
executed every other test."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _reduce(L, fn_name, op, x, axes):
    """Calls ytcuda_reduce or ytcuda_reduce_noalloc through the C ABI; returns (values, indices)."""
    from ytensor_b200 import _lib
    nd = x.dim()
    ks = list(x.shape)
    for a in axes:
        ks[a % nd] = 1
    y = torch.empty(ks, dtype=torch.float32, device="cuda")
    idx = torch.full(ks, -1, dtype=torch.int32, device="cuda")
    shape = (C.c_int64 * nd)(*x.shape)
    strides = (C.c_int64 * nd)(*x.stride())
    ax = (C.c_int * len(axes))(*axes)
    _lib.check(getattr(L, fn_name)(op, _lib.F32, _lib.F32, x.data_ptr(), y.data_ptr(), idx.data_ptr(), shape, strides,
                                   nd, ax, len(axes), None))
    torch.cuda.synchronize()
    return y.cpu().numpy(), idx.cpu().numpy()


def _call(L, fn_name, op, x, axes, y, idx):
    """One call through the C ABI into outputs the caller has allocated beforehand."""
    from ytensor_b200 import _lib
    nd = x.dim()
    shape = (C.c_int64 * nd)(*x.shape)
    strides = (C.c_int64 * nd)(*x.stride())
    ax = (C.c_int * len(axes))(*axes)
    return getattr(L, fn_name)(op, _lib.F32, _lib.F32, x.data_ptr(), y.data_ptr(), idx.data_ptr(), shape, strides,
                               nd, ax, len(axes), None)


def test_noalloc_reduce_matches_allocating_entry_point_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from ytensor_b200 import _lib
    L = _lib.lib()
    g = torch.Generator(device="cuda").manual_seed(11)
    # shapes that take the long-reduction (scratch) path: few outputs, many elements each; the second call uses
    # different data and a different shape, so leftovers of the first call in the shared array would show
    cases = [(torch.randn(1000, 1000, device="cuda", generator=g), [0, 1]),
             (torch.randn(3, 400000, device="cuda", generator=g), [1]),
             (torch.randn(48, 5000, 7, device="cuda", generator=g), [1, 0])]
    # the entry point under test runs FIRST, before any allocating reduction of this process has grown the library's
    # workspace, into outputs allocated up front; after its first call (which looks up the array's address and may
    # load the module) the free device memory must not move
    outs = []
    for x, axes in cases:
        ks = list(x.shape)
        for a in axes:
            ks[a % x.dim()] = 1
        outs.append((torch.empty(ks, dtype=torch.float32, device="cuda"),
                     torch.full(ks, -1, dtype=torch.int32, device="cuda")))
    got = {}
    _lib.check(_call(L, "ytcuda_reduce_noalloc", 0, cases[0][0], cases[0][1], *outs[0]))
    torch.cuda.synchronize()
    for round_ in range(2):
        for ci, (x, axes) in enumerate(cases):
            xin = x if round_ == 0 else x * -0.5 + 1.0
            free_mid = torch.cuda.mem_get_info()[0] if round_ == 0 else None
            for op in (0, 1, 2):
                y, idx = outs[ci]
                _lib.check(_call(L, "ytcuda_reduce_noalloc", op, xin, axes, y, idx))
                torch.cuda.synchronize()
                got[(round_, ci, op)] = (y.cpu().numpy().copy(), idx.cpu().numpy().copy())
            if round_ == 0:
                assert torch.cuda.mem_get_info()[0] == free_mid, "ytcuda_reduce_noalloc changed the free device memory"
    for round_ in range(2):
        for ci, (x, axes) in enumerate(cases):
            xin = x if round_ == 0 else x * -0.5 + 1.0
            for op in (0, 1, 2):
                want_v, want_i = _reduce(L, "ytcuda_reduce", op, xin, axes)
                got_v, got_i = got[(round_, ci, op)]
                # same kernels, same chunking, same order of additions: the two entry points agree to the bit
                assert np.array_equal(got_v, want_v), (round_, tuple(x.shape), op)
                if op == 2:
                    assert np.array_equal(got_i, want_i)
    # a short reduction (no scratch involved) goes through the same entry point
    x = torch.randn(64, 512, device="cuda", generator=g)
    want_v, _ = _reduce(L, "ytcuda_reduce", 0, x, [1])
    got_v, _ = _reduce(L, "ytcuda_reduce_noalloc", 0, x, [1])
    assert np.array_equal(got_v, want_v)


def test_noalloc_reduce_refuses_what_does_not_fit():
    """With the library's own chunking a request never exceeds the 64 KiB array, so the refusal is reached by lowering
    the usable part of the array: the call must fail with a message naming both sizes, launch nothing, and work again
    once the limit is back."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from ytensor_b200 import _lib
    L = _lib.lib()
    x = torch.randn(1000, 1000, device="cuda")
    y = torch.full((1, 1), 7.0, device="cuda")
    idx = torch.full((1, 1), -1, dtype=torch.int32, device="cuda")
    assert L.ytcuda_reduce_noalloc_set_limit(1 << 20) == _lib.INVALID_ARG  # more than the array holds
    _lib.check(L.ytcuda_reduce_noalloc_set_limit(1024))
    try:
        n0 = L.ytcuda_launch_count()
        assert _call(L, "ytcuda_reduce_noalloc", 0, x, [0, 1], y, idx) == _lib.INVALID_ARG
        msg = _lib.last_error()
        assert "1024" in msg and "needs" in msg, msg
        assert L.ytcuda_launch_count() == n0
        torch.cuda.synchronize()
        assert float(y.item()) == 7.0
    finally:
        _lib.check(L.ytcuda_reduce_noalloc_set_limit(0))
    _lib.check(_call(L, "ytcuda_reduce_noalloc", 0, x, [0, 1], y, idx))
    want, _ = _reduce(L, "ytcuda_reduce", 0, x, [0, 1])
    assert np.array_equal(y.cpu().numpy(), want)


def test_noalloc_reduce_validates_arguments_like_the_allocating_one():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from ytensor_b200 import _lib
    L = _lib.lib()
    x = torch.zeros(4, 4, device="cuda")
    shape = (C.c_int64 * 2)(4, 4)
    strides = (C.c_int64 * 2)(4, 1)
    ax = (C.c_int * 1)(1)
    assert L.ytcuda_reduce_noalloc(7, 0, 0, x.data_ptr(), x.data_ptr(), None, shape, strides, 2, ax, 1, None) == _lib.INVALID_ARG
    assert L.ytcuda_reduce_noalloc(0, 0, 0, x.data_ptr(), x.data_ptr(), None, shape, strides, 0, ax, 1, None) == _lib.INVALID_ARG
