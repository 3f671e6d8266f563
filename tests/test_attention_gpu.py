"""GPU parity tests of ytcuda_flash_attn_fwd against the CPU oracle and the golden vectors.
fp32 (one-warp-per-row kernel): 1e-5 normwise. bf16 / fp16 (tcgen05 kernel, fp32 accumulation, P rounded to
16 bits before P.V): 2e-2 normwise against the fp32 oracle run on the same 16-bit inputs."""
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
    lib.ytcuda_attn_set_path(0)


@pytest.fixture(scope="module")
def api(L):
    from ytensor_b200 import api
    return api


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


# ------------------------------------------------------------------ fp32, golden vectors
def test_doc_example(api, golden):
    q, k, v = dev(golden["doc_sdpa_q"]), dev(golden["doc_sdpa_k"]), dev(golden["doc_sdpa_v"])
    m = dev(golden["doc_sdpa_mask"]).bool()
    got = api.scaledDotProductAttention(q, k, v, 0.0, m).cpu().numpy()
    assert normwise(got, golden["doc_sdpa_out_flash_mask"]) < F32_TOL
    assert normwise(got, golden["doc_sdpa_out_math_mask"]) < F32_TOL
    # the documentation's predicate j <= i is the causal form with offset 0
    got = api.scaledDotProductAttention(q, k, v, 0.0, causal=True, causal_offset=0).cpu().numpy()
    assert normwise(got, golden["doc_sdpa_out_flash_pred"]) < F32_TOL


def test_fp32_golden(api, golden):
    q, k, v = dev(golden["att_q"]), dev(golden["att_k"]), dev(golden["att_v"])
    A = api.scaledDotProductAttention
    assert normwise(A(q, k, v, causal=True).cpu().numpy(), golden["att_causal"]) < F32_TOL
    assert normwise(A(q, k, v).cpu().numpy(), golden["att_full"]) < F32_TOL
    got = A(q, k, v, 0.0, dev(golden["att_mask"]).bool()).cpu().numpy()
    assert normwise(got, golden["att_masked"]) < F32_TOL
    assert np.all(got[:, :, :, 4, :] == 0.0)  # a row that sees no key is zero
    got = A(q, k, v, 0.2, None, dev(golden["att_bias"]), causal=True).cpu().numpy()
    assert normwise(got, golden["att_bias_causal"]) < F32_TOL
    assert normwise(A(dev(golden["att_q_short"]), k, v, causal=True).cpu().numpy(), golden["att_short_causal"]) < F32_TOL
    assert normwise(A(dev(golden["att_q_one"]), k, v, causal=True).cpu().numpy(), golden["att_decode"]) < F32_TOL
    # the zero-stride repeat form of the keys, as the decoder passes them
    k5 = k.unsqueeze(2).expand(-1, -1, 2, -1, -1)
    v5 = v.unsqueeze(2).expand(-1, -1, 2, -1, -1)
    assert normwise(A(q, k5, v5, causal=True).cpu().numpy(), golden["att_causal"]) < F32_TOL


def test_shape_errors(api):
    q = torch.zeros(1, 2, 2, 4, 8, device="cuda")
    with pytest.raises(ValueError):
        api.scaledDotProductAttention(q, torch.zeros(1, 2, 5, 16, device="cuda"), torch.zeros(1, 2, 5, 8, device="cuda"))
    with pytest.raises(ValueError):
        api.scaledDotProductAttention(q, torch.zeros(1, 2, 5, 8, device="cuda"), torch.zeros(1, 2, 6, 8, device="cuda"))
    with pytest.raises(ValueError):
        api.scaledDotProductAttention(q, torch.zeros(1, 2, 5, 8, device="cuda"), torch.zeros(1, 2, 5, 8, device="cuda"),
                                      0.0, torch.ones(3, 5, device="cuda").bool())


# ------------------------------------------------------------------ 16-bit, tensor-core kernel
def run_tc(L, api, port, q, k, v, dt=1, **kw):
    """q, k, v fp32 numpy; rounds to the 16-bit type, runs the device kernel (tcgen05 forced) and the oracle."""
    f2b, b2f = (port.f32_to_bf16, port.bf16_to_f32) if dt == 1 else (port.f32_to_f16, port.f16_to_f32)
    tdt = torch.bfloat16 if dt == 1 else torch.float16
    qb, kb, vb = f2b(q), f2b(k), f2b(v)
    okw = {}
    dkw = {}
    if kw.get("mask") is not None:
        okw["mask"] = kw["mask"]
        dkw["mask"] = dev(kw["mask"]).bool()
    if kw.get("causal"):
        okw["causal"] = True
        dkw["causal"] = True
    if kw.get("bias") is not None:
        okw["bias"] = kw["bias"]
        dkw["bias"] = dev(kw["bias"])
    want = port.sdpa(b2f(qb), b2f(kb), b2f(vb), scale=kw.get("scale", 0.0), **okw)
    L.ytcuda_attn_set_path(2)
    try:
        out = api.scaledDotProductAttention(bits_to_torch(qb, tdt), bits_to_torch(kb, tdt), bits_to_torch(vb, tdt),
                                            kw.get("scale", 0.0), dkw.get("mask"), dkw.get("bias"),
                                            causal=dkw.get("causal", False))
    finally:
        L.ytcuda_attn_set_path(0)
    assert L.ytcuda_device_status(None) == 0
    return b2f(torch_to_bits(out)), want


@pytest.mark.parametrize("b,kvh,g,lq,lk,d,causal", [
    (1, 1, 2, 128, 128, 128, False),
    (1, 1, 2, 128, 128, 128, True),
    (2, 2, 2, 256, 256, 128, True),
    (1, 1, 4, 384, 384, 128, True),
    (1, 2, 1, 512, 512, 128, True),     # no head pairs: two neighbouring row blocks share the K/V stream
    (1, 1, 1, 300, 300, 128, True),
    (1, 1, 2, 200, 333, 128, True),     # ragged lengths, causal window anchored at the end of the keys
    (1, 1, 2, 77, 500, 128, False),
    (1, 1, 3, 130, 130, 128, True),     # odd group count
    (1, 2, 2, 256, 256, 64, True),
    (1, 1, 2, 100, 640, 64, False),
    (1, 1, 2, 1, 300, 128, True),       # a decode step through the same kernel
])
def test_bf16_vs_oracle(L, api, port, b, kvh, g, lq, lk, d, causal):
    rng = np.random.default_rng(b + kvh * 3 + g * 5 + lq + lk * 7 + d)
    q = rng.standard_normal((b, kvh, g, lq, d)).astype(np.float32)
    k = rng.standard_normal((b, kvh, lk, d)).astype(np.float32)
    v = rng.standard_normal((b, kvh, lk, d)).astype(np.float32)
    got, want = run_tc(L, api, port, q, k, v, causal=causal)
    assert normwise(got, want) < H_TOL


def test_fp16_mask_bias_and_empty_rows(L, api, port):
    rng = np.random.default_rng(21)
    q = rng.standard_normal((1, 2, 2, 150, 128)).astype(np.float32)
    k = rng.standard_normal((1, 2, 260, 128)).astype(np.float32)
    v = rng.standard_normal((1, 2, 260, 128)).astype(np.float32)
    m = (rng.random((150, 260)) < 0.5).astype(np.uint8)
    m[7] = 0
    m[140] = 0
    bias = rng.standard_normal((150, 260)).astype(np.float32)
    got, want = run_tc(L, api, port, q, k, v, dt=2, mask=m)
    assert normwise(got, want) < H_TOL
    assert np.all(got[:, :, :, 7, :] == 0) and np.all(got[:, :, :, 140, :] == 0)
    got, want = run_tc(L, api, port, q, k, v, dt=2, causal=True, bias=bias, scale=0.05)
    assert normwise(got, want) < H_TOL


def test_large_logits_rescale_path(L, api, port):
    """Scores that grow along the keys force the running maximum to move by more than 2^8 many times."""
    rng = np.random.default_rng(5)
    lk = 640
    q = np.ones((1, 1, 2, 128, 128), np.float32)
    k = (np.linspace(0.0, 1.5, lk)[:, None] * np.ones((1, 128))).astype(np.float32)[None, None]
    k = k + 0.05 * rng.standard_normal(k.shape).astype(np.float32)
    v = rng.standard_normal((1, 1, lk, 128)).astype(np.float32)
    got, want = run_tc(L, api, port, q, k, v, scale=1.0)
    assert normwise(got, want) < H_TOL


def test_strided_views_of_fused_qkv(L, api, port):
    """q, k, v as slices of one fused projection output [b, l, (h + 2 kvh) * d], permuted to [b, h, l, d]."""
    rng = np.random.default_rng(9)
    b, l, h, kvh, d = 2, 256, 4, 2, 128
    qkv = rng.standard_normal((b, l, (h + 2 * kvh) * d)).astype(np.float32)
    bits = port.f32_to_bf16(qkv)
    t = bits_to_torch(bits, torch.bfloat16)
    q = t[..., : h * d].view(b, l, h, d).permute(0, 2, 1, 3)
    k = t[..., h * d: (h + kvh) * d].view(b, l, kvh, d).permute(0, 2, 1, 3)
    v = t[..., (h + kvh) * d:].view(b, l, kvh, d).permute(0, 2, 1, 3)
    f = port.bf16_to_f32(bits)
    qf = f[..., : h * d].reshape(b, l, h, d).transpose(0, 2, 1, 3).reshape(b, kvh, h // kvh, l, d)
    kf = f[..., h * d: (h + kvh) * d].reshape(b, l, kvh, d).transpose(0, 2, 1, 3)
    vf = f[..., (h + kvh) * d:].reshape(b, l, kvh, d).transpose(0, 2, 1, 3)
    want = port.sdpa(qf, kf, vf, causal=True).reshape(b, h, l, d)
    L.ytcuda_attn_set_path(2)
    try:
        out = api.scaledDotProductAttention(q, k, v, causal=True)
    finally:
        L.ytcuda_attn_set_path(0)
    assert normwise(port.bf16_to_f32(torch_to_bits(out)), want) < H_TOL


def test_config3_full_size_properties(L, api, port):
    """benchmark configuration 3: batch 16, 32 query / 8 kv heads, head_dim 128, seq 4096, causal, bf16.
    Full size through properties: (1) two batch items with the same inputs give the same bits, (2) the first
    256 and the last 128 query rows of one kv head against the oracle, (3) row 0 equals V[0]."""
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(16, 32, 4096, 128, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(16, 8, 4096, 128, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(16, 8, 4096, 128, device="cuda", generator=g).to(torch.bfloat16)
    q[15], k[15], v[15] = q[3], k[3], v[3]
    L.ytcuda_attn_set_path(2)
    try:
        out = api.scaledDotProductAttention(q, k, v, causal=True)
    finally:
        L.ytcuda_attn_set_path(0)
    assert L.ytcuda_device_status(None) == 0
    assert torch.equal(out[15], out[3])
    # row 0 sees one key: its softmax weight is 1 up to fp32 round-off, so the output is V[0] within one bf16 step
    v0 = v[:, :, 0, :].repeat_interleave(4, dim=1).float()
    assert torch.all((out[:, :, 0, :].float() - v0).abs() <= v0.abs() * 2.0 ** -7 + 1e-30)
    b2f = port.bf16_to_f32
    qf = b2f(torch_to_bits(q[5, 8:12])).reshape(1, 1, 4, 4096, 128)
    kf = b2f(torch_to_bits(k[5, 2])).reshape(1, 1, 4096, 128)
    vf = b2f(torch_to_bits(v[5, 2])).reshape(1, 1, 4096, 128)
    got = b2f(torch_to_bits(out[5, 8:12])).reshape(1, 1, 4, 4096, 128)
    want_head = port.sdpa(qf[:, :, :, :256], kf[:, :, :256], vf[:, :, :256], causal=True)
    assert normwise(got[:, :, :, :256], want_head) < H_TOL
    want_tail = port.sdpa(qf[:, :, :, -128:], kf, vf, causal=True)  # offset kv_len - q_len: the last 128 rows
    assert normwise(got[:, :, :, -128:], want_tail) < H_TOL
