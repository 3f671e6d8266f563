"""GPU parity tests: softmax, RMSNorm, LayerNorm, reductions and the fused chain against the CPU oracle
and the golden vectors. fp32 tolerance 1e-5 (normwise), bf16 output 2e-2; argmax indices must be equal."""
import numpy as np
import pytest

from _util import normwise, torch_to_bits

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TOL = 1e-5
AXES_TAGS = ("m1", "a1", "a0", "a23", "a13", "a31")


@pytest.fixture(scope="module")
def api():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from ytensor_b200 import api
    return api


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("tag", AXES_TAGS)
def test_golden_nd(api, golden, tag):
    x, axes = dev(golden["nd_x"]), [int(a) for a in golden[f"nd_{tag}_axes"]]
    w, b = dev(golden[f"nd_{tag}_w"]), dev(golden[f"nd_{tag}_b"])
    assert normwise(api.softmax(x, axes).cpu().numpy(), golden[f"nd_{tag}_softmax"]) < TOL
    assert normwise(api.rmsNorm(x, w, axes, 1e-6).cpu().numpy(), golden[f"nd_{tag}_rmsnorm"]) < TOL
    assert normwise(api.layerNorm(x, w, b, axes, 1e-5).cpu().numpy(), golden[f"nd_{tag}_layernorm"]) < TOL
    assert normwise(api.layerNorm(x, None, None, axes, 1e-5).cpu().numpy(), golden[f"nd_{tag}_layernorm_plain"]) < TOL
    assert normwise(api.sum(x, axes).cpu().numpy(), golden[f"nd_{tag}_sum"]) < TOL
    # a mean of N(0,1) draws is small against its terms: bound the error by the data's scale
    assert np.abs(api.mean(x, axes).cpu().numpy() - golden[f"nd_{tag}_mean"]).max() < TOL * np.abs(golden["nd_x"]).max()
    mv, mi = api.max(x, axes)
    assert np.array_equal(mv.cpu().numpy(), golden[f"nd_{tag}_max"])
    assert np.array_equal(mi.cpu().numpy(), golden[f"nd_{tag}_argmax"])


@pytest.mark.parametrize("shape", [(3, 128), (5, 7, 4096), (2, 4100), (9, 1000), (4, 16384), (2, 20000), (6, 37),
                                   (1, 1), (33, 8)])
def test_trailing_axis_vs_oracle(api, port, shape):
    rng = np.random.default_rng(sum(shape))
    x = (rng.standard_normal(shape) * 3).astype(np.float32)
    w = rng.uniform(0.9, 1.1, shape[-1]).astype(np.float32)
    b = rng.standard_normal(shape[-1]).astype(np.float32)
    dx = dev(x)
    # the reference adds a row up sequentially in fp32: its own rounding error grows like sqrt(row length) * 6e-8
    # and passes 1e-5 beyond about 8k elements, so longer rows get the bound scaled by sqrt(L / 4096)
    tol = TOL * max(1.0, (shape[-1] / 4096) ** 0.5)
    assert normwise(api.softmax(dx, -1).cpu().numpy(), port.softmax(x, [-1])) < tol
    assert normwise(api.rmsNorm(dx, dev(w), -1, 1e-6).cpu().numpy(), port.rmsnorm(x, w, [-1], 1e-6)) < tol
    assert normwise(api.layerNorm(dx, dev(w), dev(b), -1, 1e-5).cpu().numpy(), port.layernorm(x, w, b, [-1], 1e-5)) < 3e-5
    assert normwise(api.sum(dx, -1).cpu().numpy(), port.reduce(x, [-1], "sum")) < 1e-4  # cancellation in the sum itself
    mv, mi = api.max(dx, -1)
    wv, wi = port.reduce(x, [-1], "max")
    assert np.array_equal(mv.cpu().numpy(), wv) and np.array_equal(mi.cpu().numpy(), wi)


def test_inplace_and_views(api, port):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((4, 6, 64)).astype(np.float32)
    w = rng.uniform(0.9, 1.1, 64).astype(np.float32)
    d = dev(x)
    api.rmsNorm_(d, dev(w), -1, 1e-6)
    assert normwise(d.cpu().numpy(), port.rmsnorm(x, w, [-1], 1e-6)) < TOL
    d = dev(x)
    api.softmax_(d, -1)
    assert normwise(d.cpu().numpy(), port.softmax(x, [-1])) < TOL
    # a permuted (non-contiguous) view: per-head norm of [b, l, h, d] seen as [b, h, l, d]
    xv = dev(x.reshape(4, 6, 4, 16)).permute(0, 2, 1, 3)
    want = port.rmsnorm(np.ascontiguousarray(x.reshape(4, 6, 4, 16).transpose(0, 2, 1, 3)), w[:16], [-1], 1e-6)
    assert normwise(api.rmsNorm(xv, dev(w[:16].copy()), -1, 1e-6).cpu().numpy(), want) < TOL
    # softmax down the columns of a wide matrix (one thread per line on the device)
    y = rng.standard_normal((50, 6000)).astype(np.float32)
    assert normwise(api.softmax(dev(y), 0).cpu().numpy(), port.softmax(y, [0])) < TOL
    mv, mi = api.max(dev(y), 0)
    wv, wi = port.reduce(y, [0], "max")
    assert np.array_equal(mv.cpu().numpy(), wv) and np.array_equal(mi.cpu().numpy(), wi)


@pytest.mark.parametrize("shape,axes", [((1000, 1000), [0, 1]), ((3, 500000), [1]), ((40, 5000, 9), [0, 1]),
                                        ((2, 300, 300), [2, 1])])
def test_long_reductions_split_over_ctas(api, port, shape, axes):
    """Few outputs, very long reductions: the device splits each line over many CTAs through a scratch buffer."""
    rng = np.random.default_rng(len(shape) + shape[0])
    x = rng.standard_normal(shape).astype(np.float32)
    x.flat[123457 % x.size] = 9.0
    x.flat[(123457 % x.size) + 1000] = 9.0  # a tie: the first one in the walk must win
    d = dev(x)
    # the reference's sequential fp32 sum drifts from the exact sum more than the device's tree sum does:
    # the device must be at least as close to the exact value as the oracle is (plus round-off of the result)
    exact = x.astype(np.float64).sum(axis=tuple(axes), keepdims=True)
    oracle_err = np.abs(port.reduce(x, axes, "sum") - exact).max()
    assert np.abs(api.sum(d, axes).cpu().numpy() - exact).max() <= oracle_err + 1e-3
    n = int(np.prod([shape[a] for a in axes]))
    assert np.abs(api.mean(d, axes).cpu().numpy() - exact / n).max() < 1e-5
    mv, mi = api.max(d, axes)
    wv, wi = port.reduce(x, axes, "max")
    assert np.array_equal(mv.cpu().numpy(), wv) and np.array_equal(mi.cpu().numpy(), wi)


def test_first_maximum_wins(api):
    x = torch.zeros(3, 700, device="cuda")
    x[0, 5] = x[0, 300] = 2.0
    x[2, 699] = 1.0
    mv, mi = api.max(x, -1)
    assert mi.flatten().tolist() == [5, 0, 699]


def test_16bit_io(api, port):
    rng = np.random.default_rng(8)
    x = port.f32_to_bf16(rng.standard_normal((7, 1024)).astype(np.float32))
    want = port.softmax(port.bf16_to_f32(x), [-1])
    tx = torch.from_numpy(x.view(np.int16)).cuda().view(torch.bfloat16)
    got = port.bf16_to_f32(torch_to_bits(api.softmax(tx, -1)))
    assert normwise(got, want) < 2e-2


def test_invalid_arguments(api):
    x = torch.zeros(2, 3, 4, device="cuda")
    with pytest.raises(ValueError):  # weight shape must match the affine axes (std::invalid_argument)
        api.rmsNorm(x, torch.ones(3, device="cuda"), -1)
    with pytest.raises(ValueError):
        api.softmax(x, [1, 1])
    assert api.softmax(torch.zeros(0, 4, device="cuda"), -1).shape == (0, 4)


def test_chain_golden_and_oracle(api, port, golden):
    for r in ("r1", "r2"):
        out = api.rmsnorm_add_softmax_cast(dev(golden["chain_x"]), dev(golden["chain_w"]), dev(golden[f"chain_{r}"]))
        got = port.bf16_to_f32(torch_to_bits(out))
        assert normwise(got, port.bf16_to_f32(golden[f"chain_out_{r}"])) < 2e-2
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 17, 4096)).astype(np.float32)
    w = rng.uniform(0.9, 1.1, 4096).astype(np.float32)
    r = rng.standard_normal((1, 17, 4096)).astype(np.float32)
    out = api.rmsnorm_add_softmax_cast(dev(x), dev(w), dev(r))
    want_bits = port.chain(x, w, r)
    got_bits = torch_to_bits(out)
    assert normwise(port.bf16_to_f32(got_bits), port.bf16_to_f32(want_bits)) < 2e-2
    assert (got_bits == want_bits).mean() > 0.98  # same rounding rule: only last-bit ties of the fp32 value differ
    # unfused sequence through the single ops gives the same result as the fused kernel
    y = api.rmsNorm(dev(x), dev(w), -1, 1e-6)
    api.add_(y, dev(r))
    api.softmax_(y, -1)
    seq = api.cast(y, torch.bfloat16)
    assert normwise(port.bf16_to_f32(torch_to_bits(seq)), port.bf16_to_f32(want_bits)) < 2e-2


def test_chain_full_size_properties(api):
    """benchmark configuration 4 shape [32,4096,4096]: rows of a softmax sum to one and are non-negative; the residual
    is shared by the batch, so equal x rows in different batch items give equal outputs."""
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(32, 4096, 4096, device="cuda", generator=g)
    x[31] = x[0]
    w = torch.rand(4096, device="cuda", generator=g) * 0.2 + 0.9
    r = torch.randn(1, 4096, 4096, device="cuda", generator=g)
    out = api.rmsnorm_add_softmax_cast(x, w, r)
    assert torch.equal(out[0], out[31])
    s = out[::7, ::113].float().sum(-1)
    assert torch.all((s - 1).abs() < 2e-2) and torch.all(out[::7, ::113] >= 0)
