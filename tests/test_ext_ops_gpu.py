"""GPU parity tests of the operators added after the first golden file: the Lp / instance / batch / group norms,
the reference's 8-bit float types, and masked products that skip dead tiles (bool mask and the causal predicate
evaluated on the device). References: tests/golden/golden_ext.npz (written by the unmodified reference) and, at
sizes where the tensor-core kernels run, the CPU oracle. fp32 1e-5 normwise, casts bit-exact, bf16 2e-2."""
from pathlib import Path

import numpy as np
import pytest

from _util import bits_to_torch, normwise, torch_to_bits

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def g():
    return np.load(Path(__file__).resolve().parent / "golden" / "golden_ext.npz")


@pytest.fixture(scope="module")
def api():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from ytensor_b200 import api
    return api


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_norm_family_matches_reference(api, g):
    X = dev(g["norm_x"])
    g6, b6, g5, b5 = dev(g["norm_gamma6"]), dev(g["norm_bias6"]), dev(g["norm_gamma5"]), dev(g["norm_bias5"])
    cases = [
        (api.normalize(X, -1, 2.0, 1e-12), "norm_l2_m1"),
        (api.normalize(X, [1, 3], 1.5, 1e-6), "norm_l15_a13"),
        (api.normalize(X, [1], 2.0, 1e-12, g6, b6), "norm_l2_a1_affine"),
        (api.instanceNorm(X, channelAxis=1), "norm_inst_c1"),
        (api.instanceNorm(X, g6, b6, 1), "norm_inst_c1_affine"),
        (api.instanceNorm(X, g5, b5, 2), "norm_inst_c2_affine"),
        (api.batchNorm(X, channelAxis=1), "norm_batch_c1"),
        (api.batchNorm(X, g6, b6, 1), "norm_batch_c1_affine"),
        (api.batchNorm(X, channelAxis=-1), "norm_batch_cm1"),
        (api.groupNorm(X, 2, channelAxis=1), "norm_group2_c1"),
        (api.groupNorm(X, 3, g6, b6, 1), "norm_group3_c1_affine"),
        (api.groupNorm(dev(g["norm_xg"]), 2, dev(g["norm_gamma4"]), dev(g["norm_bias4"]), 2), "norm_group2_c2_affine"),
    ]
    for got, name in cases:
        assert normwise(got.cpu().numpy(), g[name]) < 1e-5, name
    # in-place forms, and a strided input (every other row of a taller tensor)
    Y = X.clone()
    api.groupNorm_(Y, 2, channelAxis=1)
    assert normwise(Y.cpu().numpy(), g["norm_group2_c1"]) < 1e-5
    tall = torch.zeros(3, 6, 10, 8, device="cuda")
    tall[:, :, ::2] = X
    assert normwise(api.instanceNorm(tall[:, :, ::2], channelAxis=1).cpu().numpy(), g["norm_inst_c1"]) < 1e-5
    # the reference's argument checks
    from ytensor_b200 import _lib
    for bad in (lambda: api.groupNorm(X, 4, channelAxis=1), lambda: api.groupNorm(X, 0), lambda: api.batchNorm(X, channelAxis=0),
                lambda: api.normalize(X, -1, 0.0), lambda: api.instanceNorm(X[:, :, 0, 0])):
        with pytest.raises(_lib.YtCudaInvalidArgument):
            bad()


@pytest.mark.parametrize("kind", ["float8_e5m2", "float8_e4m3", "float8_e8m0"])
def test_fp8_casts_are_bit_exact(api, g, kind):
    x = dev(g["fp8_in"])
    assert np.array_equal(api.cast_to_fp8(x, kind).cpu().numpy(), g[f"fp8_{kind}_bits"])
    table = api.cast_from_fp8(torch.arange(256, dtype=torch.uint8, device="cuda"), kind).cpu().numpy()
    assert np.array_equal(table.view(np.uint32), g[f"fp8_{kind}_table"].view(np.uint32))
    # strided input and output (the generic-index kernel), and a 16-bit source type
    x2 = x[: 4096].reshape(64, 64)
    got = torch.zeros(64, 128, dtype=torch.uint8, device="cuda")
    from ytensor_b200 import _lib
    import ctypes as C
    _lib.check(_lib.lib().ytcuda_cast(_lib.F32, api.FP8_KINDS[kind], x2.t().data_ptr(), got[:, ::2].data_ptr(), 2,
                                      (C.c_int64 * 2)(64, 64), (C.c_int64 * 2)(1, 64), (C.c_int64 * 2)(128, 2), None))
    assert np.array_equal(got[:, ::2].cpu().numpy(), g[f"fp8_{kind}_bits"][:4096].reshape(64, 64).T)
    xb = x[:4096].to(torch.bfloat16)
    want = api.cast_to_fp8(xb.float(), kind)
    assert torch.equal(api.cast_to_fp8(xb, kind), want)


def test_causal_masked_matmul_matches_reference(api, g):
    a, b = dev(g["mmc_a"]), dev(g["mmc_b"])
    assert normwise(api.masked_matmul(a, b, api.Causal(0), -1e9).cpu().numpy(), g["mmc_off0"]) < 1e-5
    assert normwise(api.masked_matmul(a, b, api.Causal(20), 0.5).cpu().numpy(), g["mmc_off20"]) < 1e-5
    # any other predicate is materialised into a bool mask
    got = api.masked_matmul(a, b, lambda i, j: j <= i + 20, 0.5).cpu().numpy()
    assert normwise(got, g["mmc_off20"]) < 1e-5


def test_masked_products_skip_dead_tiles_on_every_kernel(api, port):
    """Sizes at which the tcgen05 kernel (bf16) and the fp32-on-tensor-cores form run: the causal predicate leaves
    whole 128 x 128 / 128 x 256 tiles empty, a bool mask leaves a block of them empty; results equal the oracle's and
    the dead region holds the fill value exactly."""
    from ytensor_b200 import _lib
    L = _lib.lib()
    rng = np.random.default_rng(5)
    m, n, k = 640, 768, 256
    a32 = rng.standard_normal((2, m, k)).astype(np.float32)
    b32 = (rng.standard_normal((k, n)) / 16).astype(np.float32)
    mask = rng.random((m, n)) < 0.7
    mask[:256, 256:] = False          # two rows of dead tiles
    mask[300, :] = False
    want_c = port.masked_matmul_causal(a32, b32, 0, -7.0)
    want_m = port.masked_matmul(a32, b32, mask, 3.0)
    # fp32 operands: the three-plane tensor-core form (m, n, k >= 256)
    got = api.masked_matmul(dev(a32), dev(b32), api.Causal(0), -7.0).cpu().numpy()
    assert normwise(got, want_c) < 1e-5
    assert np.all(got[:, np.triu_indices(m, 1, n)[0], np.triu_indices(m, 1, n)[1]] == -7.0)
    got = api.masked_matmul(dev(a32), dev(b32), dev(mask), 3.0).cpu().numpy()
    assert normwise(got, want_m) < 1e-5
    assert np.all(got[:, ~mask] == 3.0)
    # bf16 operands on tcgen05
    ab, bb = port.f32_to_bf16(a32), port.f32_to_bf16(b32)
    af, bf = port.bf16_to_f32(ab), port.bf16_to_f32(bb)
    L.ytcuda_gemm_set_path(2)
    try:
        n0 = L.ytcuda_launch_count()
        got = api.masked_matmul(bits_to_torch(ab, torch.bfloat16), bits_to_torch(bb, torch.bfloat16), api.Causal(0),
                                -7.0).float().cpu().numpy()
        assert L.ytcuda_launch_count() - n0 == 3          # tile liveness, product, fill
        assert normwise(got, port.masked_matmul_causal(af, bf, 0, -7.0)) < 2e-2
        got = api.masked_matmul(bits_to_torch(ab, torch.bfloat16), bits_to_torch(bb, torch.bfloat16), dev(mask),
                                3.0).float().cpu().numpy()
        assert normwise(got, port.masked_matmul(af, bf, mask, 3.0)) < 2e-2
        assert np.all(got[:, ~mask] == 3.0)
    finally:
        L.ytcuda_gemm_set_path(0)
    _lib.check(L.ytcuda_device_status(None))
