"""GPU parity tests of ytcuda_gemm / ytcuda_gemm_host against the CPU oracle and the golden vectors.

Tolerances (normwise, max|d| / max|ref|): 1e-5 for fp32, 2e-2 for bf16 / fp16 storage with fp32
accumulation. The bf16 comparison is never bitwise: device and oracle add in different orders and a
one-ulp difference before rounding moves the rounded value."""
import ctypes

import numpy as np
import pytest

from _util import bits_to_torch, normwise, torch_to_bits

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

F32_TOL, H_TOL = 1e-5, 2e-2


@pytest.fixture(scope="module")
def L():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from ytensor_b200 import _lib
    lib = _lib.lib()
    yield lib
    lib.ytcuda_gemm_set_path(0)


@pytest.fixture(scope="module")
def api(L):
    from ytensor_b200 import api
    return api


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def status_ok(L):
    assert L.ytcuda_device_status(None) == 0


# ------------------------------------------------------------------ fp32 (FFMA path)
def test_doc_example_exact(L, api, golden):
    c = api.matmul(dev(golden["doc_matmul_a"]), dev(golden["doc_matmul_b"])).cpu().numpy()
    assert np.array_equal(c, golden["doc_matmul_c"])


def test_fp32_golden(L, api, golden):
    a = dev(golden["mm_a"])
    assert normwise(api.matmul(a, dev(golden["mm_b2"])).cpu().numpy(), golden["mm_c_shared"]) < F32_TOL
    assert normwise(api.matmul(a, dev(golden["mm_b3"])).cpu().numpy(), golden["mm_c_batched"]) < F32_TOL
    got = api.matmul(dev(golden["mm_big_a"]), dev(golden["mm_big_b"])).cpu().numpy()
    assert normwise(got, golden["mm_big_c"]) < F32_TOL
    y = api.linear(dev(golden["lin_x"]), dev(golden["lin_w"])).cpu().numpy()
    assert normwise(y, golden["lin_y"]) < F32_TOL


def test_fp32_strided_alpha_beta_golden(L, api, golden):
    a, bt, c0 = dev(golden["sgemm_a"]), dev(golden["sgemm_bt"]), dev(golden["sgemm_c0"])
    out = c0.clone()
    api.matmul(a, bt.t(), out, alpha=0.5, beta=2.0)
    assert normwise(out.cpu().numpy(), golden["sgemm_out"]) < F32_TOL
    out = c0.clone()
    api.matmul(dev(golden["sgemm_at"]).t(), bt.t(), out)
    assert normwise(out.cpu().numpy(), golden["sgemm_out_at"]) < F32_TOL


EDGE = [1, 5, 6, 7, 16, 17, 127, 128, 129]


@pytest.mark.parametrize("m,n,k", [(m, n, k) for m in (1, 6, 129) for n in (1, 17, 128) for k in (1, 7, 127)]
                         + [(1024, 1024, 1024)])
def test_fp32_vs_oracle_shapes(L, api, port, m, n, k):
    rng = np.random.default_rng(m * 10007 + n * 101 + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    want = port.matmul(a, b)
    assert normwise(api.matmul(dev(a), dev(b)).cpu().numpy(), want) < F32_TOL
    # the same product through transposed views of transposed storage
    got = api.matmul(dev(a.T.copy()).t(), dev(b.T.copy()).t()).cpu().numpy()
    assert normwise(got, want) < F32_TOL


def test_fp32_config1_seed0(L, api, port):
    """benchmark configuration 1: C[1024,1024] = A.B, A, B ~ N(0,1) from seed 0, rel err 1e-5 vs the CPU result."""
    rng = np.random.default_rng(0)
    a = rng.standard_normal((1024, 1024)).astype(np.float32)
    b = rng.standard_normal((1024, 1024)).astype(np.float32)
    assert normwise(api.matmul(dev(a), dev(b)).cpu().numpy(), port.matmul(a, b)) < F32_TOL


# ------------------------------------------------------------------ 16-bit storage (tcgen05 path)
@pytest.mark.parametrize("name,dt,tdt", [("bf16", 1, torch.bfloat16), ("f16", 2, torch.float16)])
def test_16bit_golden(L, api, port, golden, name, dt, tdt):
    a, b = golden[f"mm16_{name}_a"], golden[f"mm16_{name}_b"]
    widen = port.bf16_to_f32 if dt == 1 else port.f16_to_f32
    want = widen(golden[f"mm16_{name}_c"])
    for path in (2, 1):  # tcgen05, then FFMA: same contract
        L.ytcuda_gemm_set_path(path)
        got_bits = torch_to_bits(api.matmul(bits_to_torch(a, tdt), bits_to_torch(b, tdt)))
        L.ytcuda_gemm_set_path(0)
        assert normwise(widen(got_bits), want) < H_TOL
        status_ok(L)
        # most outputs are bit-identical; the rest differ by one rounding step
        assert (got_bits == golden[f"mm16_{name}_c"]).mean() > 0.9


LAYOUTS = ["kn", "kk", "mn", "mk"]  # A unit stride along k or m; B unit stride along n or k


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (8, 8, 8), (136, 264, 72), (1000, 776, 200), (256, 128, 4096),
                                   (128, 512, 1088)])
def test_bf16_tcgen05_vs_oracle(L, api, port, layout, m, n, k):
    rng = np.random.default_rng(m + 3 * n + 7 * k)
    a = port.f32_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    b = port.f32_to_bf16((rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32))
    want = port.bf16_to_f32(port.matmul_16(a, b, 1))
    ta = bits_to_torch(a, torch.bfloat16) if layout[0] == "k" else bits_to_torch(a.T.copy(), torch.bfloat16).t()
    tb = bits_to_torch(b, torch.bfloat16) if layout[1] == "n" else bits_to_torch(b.T.copy(), torch.bfloat16).t()
    L.ytcuda_gemm_set_path(2)
    try:
        got = port.bf16_to_f32(torch_to_bits(api.matmul(ta, tb)))
    finally:
        L.ytcuda_gemm_set_path(0)
    status_ok(L)
    assert normwise(got, want) < H_TOL


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (1000, 776, 200), (512, 512, 1088), (264, 520, 72)])
def test_bf16_cta_pair_kernel_vs_oracle(L, api, port, layout, m, n, k):
    """The 2-CTA form (cta_group::2, 256 x 256 tile per CTA pair) forced on, against the oracle."""
    rng = np.random.default_rng(m + 5 * n + 11 * k)
    a = port.f32_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    b = port.f32_to_bf16((rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32))
    want = port.bf16_to_f32(port.matmul_16(a, b, 1))
    ta = bits_to_torch(a, torch.bfloat16) if layout[0] == "k" else bits_to_torch(a.T.copy(), torch.bfloat16).t()
    tb = bits_to_torch(b, torch.bfloat16) if layout[1] == "n" else bits_to_torch(b.T.copy(), torch.bfloat16).t()
    L.ytcuda_gemm_set_path(2)
    L.ytcuda_gemm_set_pair_mode(1)
    try:
        got_pair = torch_to_bits(api.matmul(ta, tb))
        L.ytcuda_gemm_set_pair_mode(2)
        got_single = torch_to_bits(api.matmul(ta, tb))
    finally:
        L.ytcuda_gemm_set_path(0)
        L.ytcuda_gemm_set_pair_mode(0)
    status_ok(L)
    assert normwise(port.bf16_to_f32(got_pair), want) < H_TOL
    assert np.array_equal(got_pair, got_single)  # same products, same order of accumulation along k


def test_bf16_fp32_output_is_tight(L, api, port):
    """With fp32 output the tensor-core result matches the fp32 oracle far inside the 16-bit tolerance."""
    rng = np.random.default_rng(5)
    a = port.f32_to_bf16(rng.standard_normal((256, 384)).astype(np.float32))
    b = port.f32_to_bf16(rng.standard_normal((384, 512)).astype(np.float32))
    want = port.matmul(port.bf16_to_f32(a), port.bf16_to_f32(b))
    L.ytcuda_gemm_set_path(2)
    try:
        got = api.matmul(bits_to_torch(a, torch.bfloat16), bits_to_torch(b, torch.bfloat16),
                         out_dtype=torch.float32).cpu().numpy()
    finally:
        L.ytcuda_gemm_set_path(0)
    assert normwise(got, want) < 1e-5


def test_unqualified_layout_uses_ffma_and_matches(L, api, port):
    """Rows that are not 16-byte aligned cannot be fetched by TMA: the FFMA kernel takes over on the device."""
    rng = np.random.default_rng(9)
    a = port.f32_to_bf16(rng.standard_normal((37, 45)).astype(np.float32))
    b = port.f32_to_bf16(rng.standard_normal((45, 29)).astype(np.float32))
    want = port.bf16_to_f32(port.matmul_16(a, b, 1))
    ta, tb = bits_to_torch(a, torch.bfloat16), bits_to_torch(b, torch.bfloat16)
    assert normwise(port.bf16_to_f32(torch_to_bits(api.matmul(ta, tb))), want) < H_TOL
    from ytensor_b200 import _lib
    L.ytcuda_gemm_set_path(2)
    try:
        with pytest.raises(_lib.YtCudaInvalidArgument):
            api.matmul(ta, tb)
    finally:
        L.ytcuda_gemm_set_path(0)


def test_batched_broadcast_and_views(L, api, port):
    rng = np.random.default_rng(11)
    a = port.f32_to_bf16(rng.standard_normal((2, 3, 72, 136)).astype(np.float32))
    b = port.f32_to_bf16((rng.standard_normal((3, 136, 64)) / 12).astype(np.float32))
    fa, fb = port.bf16_to_f32(a), port.bf16_to_f32(b)
    want = np.stack([np.stack([port.matmul(fa[i, j], fb[j]) for j in range(3)]) for i in range(2)])
    got = api.matmul(bits_to_torch(a, torch.bfloat16), bits_to_torch(b, torch.bfloat16), out_dtype=torch.float32)
    assert normwise(got.cpu().numpy(), want) < 1e-5
    # zero-stride (repeated) left operand, as the attention caller repeats K/V over query groups
    a1 = bits_to_torch(a[0, :1], torch.bfloat16).expand(3, 72, 136)
    got = api.matmul(a1, bits_to_torch(b, torch.bfloat16), out_dtype=torch.float32).cpu().numpy()
    want = np.stack([port.matmul(fa[0, 0], fb[j]) for j in range(3)])
    assert normwise(got, want) < 1e-5


def test_alpha_beta_bf16(L, api, port):
    rng = np.random.default_rng(13)
    a = port.f32_to_bf16(rng.standard_normal((128, 64)).astype(np.float32))
    b = port.f32_to_bf16(rng.standard_normal((64, 256)).astype(np.float32))
    c0 = rng.standard_normal((128, 256)).astype(np.float32)
    want = port.sgemm(port.bf16_to_f32(a), port.bf16_to_f32(b), c0, 0.25, -1.5)
    out = dev(c0)
    api.matmul(bits_to_torch(a, torch.bfloat16), bits_to_torch(b, torch.bfloat16), out, alpha=0.25, beta=-1.5)
    assert normwise(out.cpu().numpy(), want) < 1e-5


@pytest.mark.parametrize("m,n,k,batch", [(1024, 1024, 1024, 1), (300, 264, 520, 3), (129, 8, 8, 1), (512, 768, 2048, 2)])
def test_fp32_on_tensor_cores_vs_oracle(L, api, port, m, n, k, batch):
    """fp32 operands split into three bf16 planes, six tcgen05 products accumulated in fp32: the result keeps fp32
    accuracy (same 1e-5 bound as the FFMA kernel), with alpha / beta and a shared or batched right operand."""
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((batch, m, k)).astype(np.float32)
    b = rng.standard_normal((k, n) if batch != 3 else (batch, k, n)).astype(np.float32)
    want = port.matmul(a, b)
    L.ytcuda_gemm_set_f32_mode(2)
    try:
        n0 = L.ytcuda_launch_count()
        got = api.matmul(dev(a), dev(b))
        launches = L.ytcuda_launch_count() - n0
        assert normwise(got.cpu().numpy(), want) < F32_TOL
        # one launch splits both operands (a right operand shared by several batch items is split on its own first),
        # one product over k' = 6 k
        assert launches == (3 if (batch > 1 and batch != 3) else 2)
        c0 = rng.standard_normal((batch, m, n)).astype(np.float32)
        out = dev(c0)
        api.matmul(dev(a), dev(b), out, alpha=0.5, beta=-2.0)
        assert normwise(out.cpu().numpy(), 0.5 * want - 2.0 * c0) < F32_TOL
        # a transposed view of the left operand goes through the same path (the split reads any strides)
        at = dev(np.ascontiguousarray(a.transpose(0, 2, 1)))
        assert normwise(api.matmul(at.transpose(1, 2), dev(b)).cpu().numpy(), want) < F32_TOL
    finally:
        L.ytcuda_gemm_set_f32_mode(0)
    # the FFMA kernel on the same inputs, for the record of both paths
    L.ytcuda_gemm_set_f32_mode(1)
    try:
        assert normwise(api.matmul(dev(a), dev(b)).cpu().numpy(), want) < F32_TOL
    finally:
        L.ytcuda_gemm_set_f32_mode(0)
    status_ok(L)


@pytest.mark.gpu
def test_fp32_on_tensor_cores_extreme_values(L, api):
    """Values next to the largest float go through the three-plane split exactly (rounding the top plane would
    overflow: it is truncated instead). An infinite operand is the one documented deviation: the tensor-core form
    answers NaN in the outputs it reaches, the FFMA kernel answers the infinity as the reference's sgemm does."""
    rng = np.random.default_rng(5)
    m = n = k = 256
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = np.zeros((k, n), dtype=np.float32)
    b[np.arange(k), np.arange(n)] = 0.5  # C = 0.5 * A: no sums, so huge values stay finite
    big = np.float32(3.4e38)             # above the largest bfloat16 after rounding (3.39e38)
    a[3, 7] = big
    a[200, 100] = -np.float32(np.finfo(np.float32).max)
    L.ytcuda_gemm_set_f32_mode(2)
    try:
        got = api.matmul(dev(a), dev(b)).cpu().numpy()
        assert np.isfinite(got).all()
        assert got[3, 7] == np.float32(0.5) * big and got[200, 100] == -np.float32(np.finfo(np.float32).max) * np.float32(0.5)
        assert normwise(got, 0.5 * a) < F32_TOL
        a[5, 9] = np.inf
        got = api.matmul(dev(a), dev(b)).cpu().numpy()
        assert np.isnan(got[5]).any() and np.isfinite(np.delete(got, 5, axis=0)).all()  # the deviation, row 5 only
    finally:
        L.ytcuda_gemm_set_f32_mode(0)
    L.ytcuda_gemm_set_f32_mode(1)
    try:
        got = api.matmul(dev(a), dev(b)).cpu().numpy()
        assert got[5, 9] == np.inf  # as sgemm: inf * 0.5
    finally:
        L.ytcuda_gemm_set_f32_mode(0)
    status_ok(L)


def test_fp32_split_keeps_extreme_values(L, api):
    """Values far apart in magnitude and 24-bit integers: the three-plane split must not lose them. (Non-finite
    inputs are outside the contract of this path: an infinity times the zero low planes of the other operand gives
    NaN where fp32 arithmetic gives infinity; what is checked is that the result is still not finite.)"""
    L.ytcuda_gemm_set_f32_mode(2)
    try:
        a = np.zeros((256, 256), np.float32)
        b = np.eye(256, dtype=np.float32)
        a[0, :4] = [1.0, 2.0 ** -20, 16777215.0, 3.0e38]
        a[1, 0] = np.inf
        a[2, :3] = [1.0 + 2.0 ** -23, -(1.0 + 2.0 ** -23), 1e-30]
        got = api.matmul(dev(a), dev(b)).cpu().numpy()
        assert np.array_equal(got[0, :4], a[0, :4]) and not np.isfinite(got[1, 0]) and np.array_equal(got[2, :3], a[2, :3])
        assert np.all(got[3:] == 0)
    finally:
        L.ytcuda_gemm_set_f32_mode(0)


def test_masked_matmul_golden_and_16bit(L, api, port, golden):
    """YTensor::masked_matmul: products where the mask holds, the fill value elsewhere (mask shared by the batch)."""
    a, mk = golden["mmask_a"], golden["mmask_mask"]
    tm = dev(mk)
    got = api.masked_matmul(dev(a), dev(golden["mmask_b2"]), tm, -1.5).cpu().numpy()
    assert normwise(got, golden["mmask_c_shared"]) < F32_TOL and np.all(got[:, ~mk] == -1.5)
    got = api.masked_matmul(dev(a), dev(golden["mmask_b3"]), tm, 0.0).cpu().numpy()
    assert normwise(got, golden["mmask_c_batched"]) < F32_TOL and np.all(got[:, ~mk] == 0.0)
    # bf16 on the tensor-core path, a strided mask view, fill value rounded as the reference rounds
    rng = np.random.default_rng(5)
    m, n, k = 256, 264, 128
    A = torch.from_numpy(rng.standard_normal((3, m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    B = torch.from_numpy(rng.standard_normal((k, n)).astype(np.float32)).cuda().to(torch.bfloat16)
    wide = torch.from_numpy(rng.random((m, 2 * n)) < 0.5).cuda()
    mask = wide[:, :n]
    out = api.masked_matmul(A, B, mask, 0.3).float().cpu().numpy()
    want = port.masked_matmul(A.float().cpu().numpy(), B.float().cpu().numpy(), mask.cpu().numpy(), 0.3)
    keep = mask.cpu().numpy()
    assert normwise(out[:, keep], want[:, keep]) < H_TOL
    fill = port.bf16_to_f32(port.f32_to_bf16(np.array([0.3], np.float32)))[0]
    assert np.all(out[:, ~keep] == fill)
    with pytest.raises(ValueError):
        api.masked_matmul(A, B, mask[:, :-1], 0.0)
    status_ok(L)


def test_empty_and_invalid(L, api):
    from ytensor_b200 import _lib
    n0 = L.ytcuda_launch_count()
    out = api.matmul(torch.empty(0, 8, device="cuda"), torch.empty(8, 4, device="cuda"))
    assert out.shape == (0, 4) and L.ytcuda_launch_count() == n0  # empty dims: success, no launch
    z = api.matmul(torch.empty(3, 0, device="cuda"), torch.empty(0, 4, device="cuda"))
    assert torch.equal(z, torch.zeros(3, 4, device="cuda"))  # k == 0: C = beta*C = 0
    with pytest.raises(ValueError):  # std::invalid_argument in the reference (src/ytensor_math.inl:290-292)
        api.matmul(torch.empty(3, 5, device="cuda"), torch.empty(4, 2, device="cuda"))
    with pytest.raises(_lib.YtCudaInvalidArgument):
        api.matmul(torch.empty(3, 5), torch.empty(5, 2))  # host tensors: no CPU fallback


# ------------------------------------------------------------------ full size (benchmark configuration 2)
def test_config2_full_size_properties(L, api, port):
    """[64,2048,4096] x [4096,4096] bf16. The oracle needs about a minute per batch item, so the full size is
    checked through properties: (1) B = a permutation matrix moves columns exactly (bit-exact);
    (2) sampled rows against the oracle."""
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(64, 2048, 4096, device="cuda", generator=g).to(torch.bfloat16)
    perm = torch.randperm(4096, device="cuda", generator=g)
    p = torch.zeros(4096, 4096, device="cuda", dtype=torch.bfloat16)
    p[perm, torch.arange(4096, device="cuda")] = 1  # column j of A.P is column perm[j] of A
    c = api.matmul(a, p)
    status_ok(L)
    assert torch.equal(c, a[:, :, perm])
    b = (torch.randn(4096, 4096, device="cuda", generator=g) / 64).to(torch.bfloat16)
    c = api.matmul(a, b)
    status_ok(L)
    rows = [(0, 0), (21, 777), (42, 1024), (63, 2047)]
    a_rows = np.stack([torch_to_bits(a[i, r]) for i, r in rows])
    want = port.bf16_to_f32(port.matmul_16(a_rows[None], torch_to_bits(b), 1))[0]
    got = np.stack([port.bf16_to_f32(torch_to_bits(c[i, r])) for i, r in rows])
    assert normwise(got, want) < H_TOL


def test_host_buffer_variant_matches_device(L, api):
    from ytensor_b200 import _lib
    g = torch.Generator().manual_seed(3)
    a = torch.randn(6, 512, 1024, generator=g).to(torch.bfloat16).pin_memory()
    b = (torch.randn(1024, 768, generator=g) / 32).to(torch.bfloat16).pin_memory()
    c = torch.empty(6, 512, 768, dtype=torch.bfloat16).pin_memory()
    _lib.check(L.ytcuda_gemm_host(_lib.BF16, _lib.BF16, a.data_ptr(), b.data_ptr(), c.data_ptr(), 512, 768, 1024, 1.0,
                                  0.0, 1024, 1, 768, 1, 768, 1, 6, 512 * 1024, 0, 512 * 768))
    want = api.matmul(a.cuda(), b.cuda()).cpu()
    assert torch.equal(c, want)
    # pageable memory and a C view with a row pitch
    a2, b2 = a.clone(), b.clone()
    cbig = torch.full((6, 512, 800), 7.0, dtype=torch.bfloat16)
    cv = cbig[:, :, :768]
    _lib.check(L.ytcuda_gemm_host(_lib.BF16, _lib.BF16, a2.data_ptr(), b2.data_ptr(), cv.data_ptr(), 512, 768, 1024,
                                  1.0, 0.0, 1024, 1, 768, 1, 800, 1, 6, 512 * 1024, 0, 512 * 800))
    assert torch.equal(cv, want)
    assert torch.all(cbig[:, :, 768:] == 7.0)  # the gap between rows is left alone
