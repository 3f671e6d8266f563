"""GPU tests of the library's behaviour around its kernels: a bounded device-side wait that runs out, scratch memory
under two streams, and the shared-memory attribute on every device of a process. No test here faults or hangs a GPU:
the wait that runs out is a wait with a short cycle budget on a barrier nothing arrives on, after which the kernel
returns by itself."""
import numpy as np
import pytest

from _util import normwise

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from ytensor_b200 import _lib
    return _lib.lib()


def test_bounded_wait_runs_out_and_the_device_stays_usable(L, port):
    from ytensor_b200 import _lib, api
    old = L.ytcuda_get_wait_limit()
    assert old > 0
    assert L.ytcuda_set_wait_limit(0) == _lib.INVALID_ARG
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    _lib.check(L.ytcuda_device_status(None))             # clean before the probe
    _lib.check(L.ytcuda_set_wait_limit(2_000_000))       # about a millisecond
    try:
        _lib.check(L.ytcuda_wait_probe(waited.data_ptr(), None))
        assert L.ytcuda_device_status(None) == _lib.TIMEOUT
        assert "wait" in _lib.last_error()
        assert 2_000_000 <= int(waited.item()) < 200_000_000  # it gave up at the budget, not much later
        assert L.ytcuda_device_status(None) == _lib.OK    # reading the status clears it
    finally:
        _lib.check(L.ytcuda_set_wait_limit(old))
    # the next call on the same context works
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((64, 48)).astype(np.float32), rng.standard_normal((48, 32)).astype(np.float32)
    got = api.matmul(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()).cpu().numpy()
    assert normwise(got, port.matmul(a, b)) < 1e-5
    _lib.check(L.ytcuda_device_status(None))


def test_scratch_is_per_stream(L):
    """Two calls that need scratch memory (the fp32 product on the tensor cores; attention over a long cache, split
    over keys) run at the same time on two streams and must give what they give one after the other."""
    from ytensor_b200 import api
    g = torch.Generator(device="cuda").manual_seed(5)
    n = 1024
    a1, b1 = torch.randn(n, n, device="cuda", generator=g), torch.randn(n, n, device="cuda", generator=g)
    a2, b2 = torch.randn(n, n, device="cuda", generator=g), torch.randn(n, n, device="cuda", generator=g)
    q = torch.randn(2, 8, 1, 128, device="cuda", generator=g)
    k = torch.randn(2, 4, 8192, 128, device="cuda", generator=g)
    v = torch.randn(2, 4, 8192, 128, device="cuda", generator=g)
    q2 = torch.randn(2, 8, 1, 128, device="cuda", generator=g)
    want = (api.matmul(a1, b1), api.matmul(a2, b2), api.scaledDotProductAttention(q, k, v),
            api.scaledDotProductAttention(q2, k, v))
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    for _ in range(4):
        with torch.cuda.stream(s1):
            g1 = api.matmul(a1, b1)
            g3 = api.scaledDotProductAttention(q, k, v)
        with torch.cuda.stream(s2):
            g2 = api.matmul(a2, b2)
            g4 = api.scaledDotProductAttention(q2, k, v)
        torch.cuda.synchronize()
        for got, w in zip((g1, g2, g3, g4), want):
            assert torch.equal(got, w)


def test_every_device_of_a_process_gets_its_shared_memory_limit(L):
    """The tcgen05 GEMM needs more dynamic shared memory than the default limit; a process that uses two GPUs must be
    able to launch it on both."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs in one process")
    from ytensor_b200 import api
    outs = []
    for d in range(2):
        with torch.cuda.device(d):
            g = torch.Generator(device=f"cuda:{d}").manual_seed(3)
            a = torch.randn(512, 512, device=f"cuda:{d}", generator=g).to(torch.bfloat16)
            b = torch.randn(512, 512, device=f"cuda:{d}", generator=g).to(torch.bfloat16)
            outs.append(api.matmul(a, b).float().cpu())
            q = torch.randn(1, 4, 256, 128, device=f"cuda:{d}", generator=g).to(torch.bfloat16)
            outs.append(api.scaledDotProductAttention(q, q, q, causal=True).float().cpu())
    assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[3])
