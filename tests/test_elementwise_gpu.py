"""GPU parity tests: broadcast binary operators, swish, SwiGLU and dtype casts (bit-exact) against the oracle."""
import hashlib

import numpy as np
import pytest

from _util import normwise, torch_to_bits

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from ytensor_b200 import api
    return api


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_binary_golden_exact(api, golden):
    x, y = dev(golden["nd_x"]), dev(golden["bin_y"])
    for op in ("add", "sub", "mul", "div"):
        got = getattr(api, op)(x, y).cpu().numpy()
        assert np.array_equal(got, golden[f"bin_{op}"])  # one IEEE operation per element: exact


def test_binary_broadcast_forms(api, port):
    rng = np.random.default_rng(1)
    a = rng.standard_normal((4, 6, 256)).astype(np.float32)
    for bshape in [(4, 6, 256), (1, 6, 256), (256,), (6, 1), (4, 1, 1), (1,)]:
        b = rng.standard_normal(bshape).astype(np.float32)
        assert np.array_equal(api.add(dev(a), dev(b)).cpu().numpy(), a + b)
        d = dev(a)
        api.mul_(d, dev(b))
        assert np.array_equal(d.cpu().numpy(), a * b)
    # in-place on a non-contiguous slice, as the decoder's gate *= up on halves of one tensor
    h = dev(rng.standard_normal((5, 512)).astype(np.float32))
    ref = h.cpu().numpy().copy()
    api.mul_(h[:, :256], h[:, 256:])
    ref[:, :256] *= ref[:, 256:]
    assert np.array_equal(h.cpu().numpy(), ref)
    with pytest.raises(RuntimeError):  # std::runtime_error on a broadcast mismatch (src/kernel/broadcast.inl:133)
        api.add(dev(a), dev(np.zeros((5, 256), np.float32)))


def test_swish_and_swiglu(api, port, golden):
    got = api.swish(dev(golden["swish_x"])).cpu().numpy()
    assert normwise(got, golden["swish_y"]) < 1e-6
    rng = np.random.default_rng(2)
    gu = (rng.standard_normal((7, 2 * 3072)) * 3).astype(np.float32)
    want = port.swish(gu[:, :3072]) * gu[:, 3072:]
    assert normwise(api.swiglu(dev(gu)).cpu().numpy(), want) < 1e-6


def test_casts_bit_exact(api, port, golden):
    x = golden["cast_x"]
    assert np.array_equal(torch_to_bits(api.cast(dev(x), torch.bfloat16)), golden["cast_bf16"])
    assert np.array_equal(torch_to_bits(api.cast(dev(x), torch.float16)), golden["cast_f16"])
    allbits = np.arange(65536, dtype=np.uint16)
    for dt, key in ((torch.float16, "cast_f16_to_f32_all_sha256"), (torch.bfloat16, "cast_bf16_to_f32_all_sha256")):
        t = torch.from_numpy(allbits.view(np.int16)).cuda().view(dt)
        f = api.cast(t, torch.float32).cpu().numpy().view(np.uint32)
        assert hashlib.sha256(f.tobytes()).hexdigest() == str(golden[key])
    # a strided source: transpose while converting
    rng = np.random.default_rng(4)
    y = rng.standard_normal((33, 70)).astype(np.float32)
    got = torch_to_bits(api.cast(dev(y).t(), torch.bfloat16))
    assert np.array_equal(got, port.f32_to_bf16(np.ascontiguousarray(y.T)))


def test_cast_round_rule_known_answers(api):
    x = torch.tensor([1.0 + 3.0 / 512, 1.0 + 1.0 / 128 + 1.0 / 256], device="cuda")
    out = api.cast(x, torch.bfloat16).float().cpu().tolist()
    assert out == [1.0, 1.015625]  # the reference's rule, not IEEE round-to-nearest-even (which gives 1.0078125)
