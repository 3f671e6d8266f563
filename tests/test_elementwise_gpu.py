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


@pytest.mark.parametrize("name,alpha,key", [
    ("relu", None, "act_relu"), ("exp", None, "act_exp"), ("sigmoid", None, "act_sigmoid"),
    ("leakyRelu", None, "act_leakyRelu"), ("leakyRelu", 0.2, "act_leakyRelu_0p2"), ("elu", None, "act_elu"),
    ("elu", 0.5, "act_elu_0p5"), ("selu", None, "act_selu"), ("gelu", None, "act_gelu"), ("tanh", None, "act_tanh"),
    ("softplus", None, "act_softplus"), ("mish", None, "act_mish"), ("hardSigmoid", None, "act_hardSigmoid"),
    ("hardSwish", None, "act_hardSwish")])
def test_activations_match_reference(api, golden, name, alpha, key):
    x, want = golden["act_x"], golden[key]
    args = () if alpha is None else (alpha,)
    got = getattr(api, name)(dev(x), *args).cpu().numpy()
    if name in ("relu", "leakyRelu", "hardSwish", "hardSigmoid"):
        assert np.array_equal(got, want)  # comparisons and one or two IEEE operations: exact
    else:
        # device exp / erf / tanh / log1p differ from the host libm by a few ulp: 1e-5 relative per element, with an
        # absolute floor for results that cancel towards zero (elu and selu near 0, gelu in its negative tail)
        assert np.all(np.abs(got.astype(np.float64) - want) <= 1e-5 * np.abs(want) + 2e-7)
    d = dev(x)
    r = getattr(api, name + "_")(d, *args)
    assert r.data_ptr() == d.data_ptr() and np.array_equal(d.cpu().numpy(), got)  # the in-place form


@pytest.mark.parametrize("name,alpha", [
    ("swish", None), ("relu", None), ("exp", None), ("sigmoid", None), ("leakyRelu", None), ("leakyRelu", 0.2),
    ("elu", None), ("elu", 0.5), ("selu", None), ("gelu", None), ("tanh", None), ("softplus", None), ("mish", None),
    ("hardSigmoid", None), ("hardSwish", None)])
def test_activation_first_derivatives_match_reference(api, golden, name, alpha):
    key = f"actd_{name}" + ("" if alpha is None else "_0p2" if name == "leakyRelu" else "_0p5")
    x, want = golden["act_x"], golden[key]
    kw = {} if alpha is None else {"alpha": alpha}
    got = getattr(api, name)(dev(x), order=1, **kw).cpu().numpy()
    if name in ("relu", "leakyRelu", "hardSigmoid", "hardSwish"):
        assert np.array_equal(got, want)
    else:
        assert np.all(np.abs(got.astype(np.float64) - want) <= 1e-5 * np.abs(want) + 2e-7)
    d = dev(x)
    getattr(api, name + "_")(d, order=1, **kw)
    assert np.array_equal(d.cpu().numpy(), got)
    with pytest.raises(ValueError):  # the reference's other orders (integrals, higher derivatives) stay on the host
        getattr(api, name)(dev(x), order=2, **kw)


def test_activation_dtypes_and_bad_op(api, port):
    from ytensor_b200 import _lib
    x = (np.random.default_rng(5).standard_normal(3000) * 2).astype(np.float32)
    xb = dev(x).to(torch.bfloat16)
    got = api.gelu(xb)
    assert got.dtype == torch.bfloat16
    want = port.activation("gelu", xb.float().cpu().numpy())
    assert normwise(got.float().cpu().numpy(), want) < 2e-2
    assert api.relu(dev(np.zeros((0, 4), np.float32))).shape == (0, 4)
    t = dev(x)
    with pytest.raises(RuntimeError):
        api._unary(16, t, None, 0.0)
    with pytest.raises(RuntimeError):
        api._unary(34, t, None, 0.0)  # 32 + scale: not an activation
    with pytest.raises(RuntimeError):
        api._unary(-1, t, None, 0.0)


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
