"""CPU: pins the plain-C oracle (oracle/yt_oracle.c) against the golden vectors that the unmodified
reference produced (tests/golden/make_golden.py), and against the reference live where it is built."""
import hashlib

import numpy as np
import pytest

AXES_TAGS = ("m1", "a1", "a0", "a23", "a13", "a31")


def normwise(a, b):
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / max(np.abs(b).max(), 1e-30))


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_casts_bit_exact(golden, port):
    x = golden["cast_x"]
    assert np.array_equal(port.f32_to_bf16(x), golden["cast_bf16"])
    assert np.array_equal(port.f32_to_f16(x), golden["cast_f16"])
    allbits = np.arange(65536, dtype=np.uint16)
    assert sha(port.f16_to_f32(allbits).view(np.uint32)) == str(golden["cast_f16_to_f32_all_sha256"])
    assert sha(port.bf16_to_f32(allbits).view(np.uint32)) == str(golden["cast_bf16_to_f32_all_sha256"])


def test_bf16_round_rule_known_answers(port):
    # yt::bfloat16 adds half an ulp only when the kept LSB is 1 (include/types/bfloat16.hpp:78-80):
    # 1 + 3/512 truncates to 1.0 although true round-to-nearest-even gives 1.0078125.
    out = port.bf16_to_f32(port.f32_to_bf16(np.array([1.0 + 3.0 / 512, 1.0 + 1.0 / 128 + 1.0 / 256], np.float32)))
    assert out[0] == 1.0
    assert out[1] == 1.015625


def test_doc_matmul_known_answer(golden, port):
    want = np.array([[4, 5, 2, 1], [10, 11, 5, 4]], np.float32)
    assert np.array_equal(golden["doc_matmul_c"], want)
    assert np.array_equal(port.matmul(golden["doc_matmul_a"], golden["doc_matmul_b"]), want)


def test_masked_matmul(golden, port):
    a, mk = golden["mmask_a"], golden["mmask_mask"]
    assert np.array_equal(port.masked_matmul(a, golden["mmask_b2"], mk, -1.5), golden["mmask_c_shared"])
    assert np.array_equal(port.masked_matmul(a, golden["mmask_b3"], mk, 0.0), golden["mmask_c_batched"])
    # masked-out entries hold the fill value, masked-in ones the plain product; the two backends agree to round-off
    c = golden["mmask_c_shared"]
    assert np.all(c[:, ~mk] == -1.5) and np.all(np.delete(c[:, 5, :], 7, axis=1) == -1.5)
    assert np.array_equal(c[:, mk], port.matmul(a, golden["mmask_b2"])[:, mk])
    assert normwise(golden["mmask_c_shared_naive"], c) < 1e-6


def test_topk_sampling(golden, port):
    tp, ti, ts = port.topk_sample(golden["topk_logits"], 20, golden["topk_uniform"])
    assert np.array_equal(ti, golden["topk_idx"]) and np.array_equal(tp, golden["topk_probs"])
    assert np.array_equal(ts, golden["topk_sampled"])
    assert np.all(np.diff(golden["topk_probs"], axis=1) <= 0)


def test_matmul(golden, port):
    a = golden["mm_a"]
    assert np.array_equal(port.matmul(a, golden["mm_b2"]), golden["mm_c_shared"])
    assert np.array_equal(port.matmul(a, golden["mm_b3"]), golden["mm_c_batched"])
    # the reference's own two backends agree to fp32 round-off
    assert normwise(golden["mm_c_shared_naive"], golden["mm_c_shared"]) < 1e-6
    assert normwise(port.matmul(golden["mm_big_a"], golden["mm_big_b"]), golden["mm_big_c"]) < 1e-5
    w = golden["lin_w"]
    assert normwise(port.matmul(golden["lin_x"], w.T.copy()), golden["lin_y"]) < 1e-6
    assert normwise(port.matmul(golden["lin_x"], w.T.copy()) + golden["lin_bias"], golden["lin_y_bias"]) < 1e-6


def test_sgemm_strided_alpha_beta(golden, port):
    out = port.sgemm(golden["sgemm_a"], golden["sgemm_bt"].T, golden["sgemm_c0"], 0.5, 2.0)
    assert np.array_equal(out, golden["sgemm_out"])
    out = port.sgemm(golden["sgemm_at"].T, golden["sgemm_bt"].T, golden["sgemm_c0"], 1.0, 0.0)
    assert np.array_equal(out, golden["sgemm_out_at"])


@pytest.mark.parametrize("name,dt", [("bf16", 1), ("f16", 2)])
def test_matmul_16bit_recipe(golden, port, name, dt):
    got = port.matmul_16(golden[f"mm16_{name}_a"], golden[f"mm16_{name}_b"], dt)
    assert np.array_equal(got, golden[f"mm16_{name}_c"])


@pytest.mark.parametrize("tag", AXES_TAGS)
def test_nd_ops(golden, port, tag):
    x, axes = golden["nd_x"], golden[f"nd_{tag}_axes"]
    w, b = golden[f"nd_{tag}_w"], golden[f"nd_{tag}_b"]
    assert np.array_equal(port.softmax(x, axes), golden[f"nd_{tag}_softmax"])
    assert np.array_equal(port.rmsnorm(x, w, axes, 1e-6), golden[f"nd_{tag}_rmsnorm"])
    assert np.array_equal(port.layernorm(x, w, b, axes, 1e-5), golden[f"nd_{tag}_layernorm"])
    assert np.array_equal(port.layernorm(x, None, None, axes, 1e-5), golden[f"nd_{tag}_layernorm_plain"])
    assert np.array_equal(port.reduce(x, axes, "sum"), golden[f"nd_{tag}_sum"])
    assert np.array_equal(port.reduce(x, axes, "mean"), golden[f"nd_{tag}_mean"])
    mv, mi = port.reduce(x, axes, "max")
    assert np.array_equal(mv, golden[f"nd_{tag}_max"])
    assert np.array_equal(mi, golden[f"nd_{tag}_argmax"])


def test_elementwise(golden, port):
    for op in ("add", "sub", "mul", "div"):
        assert np.array_equal(port.binary(golden["nd_x"], golden["bin_y"], op), golden[f"bin_{op}"])
    assert np.array_equal(port.swish(golden["swish_x"]), golden["swish_y"])


ACT_CASES = [("relu", None, "act_relu"), ("exp", None, "act_exp"), ("sigmoid", None, "act_sigmoid"),
             ("leakyRelu", None, "act_leakyRelu"), ("leakyRelu", 0.2, "act_leakyRelu_0p2"), ("elu", None, "act_elu"),
             ("elu", 0.5, "act_elu_0p5"), ("selu", None, "act_selu"), ("gelu", None, "act_gelu"),
             ("tanh", None, "act_tanh"), ("softplus", None, "act_softplus"), ("mish", None, "act_mish"),
             ("hardSigmoid", None, "act_hardSigmoid"), ("hardSwish", None, "act_hardSwish")]


@pytest.mark.parametrize("name,alpha,key", ACT_CASES)
def test_activations(golden, port, name, alpha, key):
    # the same libm calls in the same order as the reference: bit-exact on this host
    assert np.array_equal(port.activation(name, golden["act_x"], alpha), golden[key], equal_nan=True)


DERIV_CASES = [(n, None, f"actd_{n}") for n in ("swish", "relu", "exp", "sigmoid", "leakyRelu", "elu", "selu", "gelu",
                                                 "tanh", "softplus", "mish", "hardSigmoid", "hardSwish")]
DERIV_CASES += [("leakyRelu", 0.2, "actd_leakyRelu_0p2"), ("elu", 0.5, "actd_elu_0p5")]


@pytest.mark.parametrize("name,alpha,key", DERIV_CASES)
def test_activation_derivatives(golden, port, name, alpha, key):
    got, want = port.activation(name, golden["act_x"], alpha, order=1), golden[key]
    if name in ("swish", "tanh", "mish"):
        # the reference was compiled with FMA contraction (1 - t * t as one fused operation), the port without
        assert np.all(np.abs(got.astype(np.float64) - want) <= 2.5e-7 * np.abs(want) + 1.5e-7)  # (one ulp at 1)
    else:
        assert np.array_equal(got, want, equal_nan=True)


def test_chain(golden, port):
    for r in ("r1", "r2"):
        got = port.chain(golden["chain_x"], golden["chain_w"], golden[f"chain_{r}"])
        assert np.array_equal(got, golden[f"chain_out_{r}"])


def test_attention(golden, port):
    q, k, v = golden["doc_sdpa_q"], golden["doc_sdpa_k"], golden["doc_sdpa_v"]
    m = golden["doc_sdpa_mask"]
    assert np.array_equal(port.sdpa(q, k, v, mask=m), golden["doc_sdpa_out_flash_mask"])
    assert normwise(port.sdpa(q, k, v, mask=m), golden["doc_sdpa_out_math_mask"]) < 1e-6
    tri = np.tril(np.ones((2, 3), np.uint8))
    assert np.array_equal(port.sdpa(q, k, v, mask=tri), golden["doc_sdpa_out_flash_pred"])
    # first query row may only see key 0 under j <= i: its output is value row 0
    assert np.allclose(golden["doc_sdpa_out_flash_pred"][0, 0, 0, 0], v[0, 0, 0])

    q, k, v = golden["att_q"], golden["att_k"], golden["att_v"]
    assert np.array_equal(port.sdpa(q, k, v, causal=True), golden["att_causal"])
    assert normwise(golden["att_causal_math"], golden["att_causal"]) < 1e-6
    assert np.array_equal(port.sdpa(q, k, v), golden["att_full"])
    got = port.sdpa(q, k, v, mask=golden["att_mask"])
    assert np.array_equal(got, golden["att_masked"])
    assert np.all(got[:, :, :, 4, :] == 0.0)  # fully masked row -> zeros
    got = port.sdpa(q, k, v, causal=True, bias=golden["att_bias"], scale=0.2)
    assert np.array_equal(got, golden["att_bias_causal"])
    assert np.array_equal(port.sdpa(golden["att_q_short"], k, v, causal=True), golden["att_short_causal"])
    assert normwise(port.sdpa(golden["att_q_one"], k, v, causal=True), golden["att_decode"]) < 1e-6


def test_port_matches_reference_live(port, ref):
    """Where the reference is built, compare the restatement with it on fresh random inputs."""
    rng = np.random.default_rng(7)
    x = rng.standard_normal((3, 4, 6, 40)).astype(np.float32)
    for axes in ([-1], [0, 2], [3, 1]):
        w = rng.uniform(0.9, 1.1, [x.shape[a] for a in axes]).astype(np.float32)
        assert np.array_equal(port.rmsnorm(x, w, axes, 1e-6), ref.rmsnorm(x, w, axes, 1e-6))
        assert np.array_equal(port.softmax(x, axes), ref.softmax(x, axes))
        assert np.array_equal(port.reduce(x, axes, "max")[1], ref.reduce(x, axes, "max")[1])
    a = rng.standard_normal((2, 50, 96)).astype(np.float32)
    b = rng.standard_normal((96, 33)).astype(np.float32)
    assert normwise(port.matmul(a, b), ref.matmul(a, b)) < 1e-6
    q = rng.standard_normal((1, 2, 4, 70, 64)).astype(np.float32)
    k = rng.standard_normal((1, 2, 70, 64)).astype(np.float32)
    v = rng.standard_normal((1, 2, 70, 64)).astype(np.float32)
    assert normwise(port.sdpa(q, k, v, causal=True), ref.sdpa(q, k, v, causal=True)) < 1e-6
    assert normwise(port.sdpa(q, k, v, causal=True), ref.sdpa(q, k, v, causal=True, backend=0)) < 1e-5


# ------------------------------------------------------------------ later operators (golden_ext.npz)
@pytest.fixture(scope="module")
def golden_ext():
    from pathlib import Path
    return np.load(Path(__file__).resolve().parent / "golden" / "golden_ext.npz")


@pytest.mark.parametrize("kind", ["float8_e5m2", "float8_e4m3", "float8_e8m0"])
def test_port_fp8_conversions_are_the_references(port, golden_ext, kind):
    assert np.array_equal(port.fp8(kind, golden_ext["fp8_in"]), golden_ext[f"fp8_{kind}_bits"])
    table = port.fp8_to_f32(kind, np.arange(256, dtype=np.uint8))
    assert np.array_equal(table.view(np.uint32), golden_ext[f"fp8_{kind}_table"].view(np.uint32))


def test_port_norm_family_matches_reference(port, golden_ext):
    g = golden_ext
    X = g["norm_x"]
    exact = [
        (port.norm("normalize", X, [-1], p=2.0, eps=1e-12), "norm_l2_m1"),
        (port.norm("normalize", X, [1], g["norm_gamma6"], g["norm_bias6"], p=2.0, eps=1e-12), "norm_l2_a1_affine"),
        (port.norm("instanceNorm", X, [1]), "norm_inst_c1"),
        (port.norm("instanceNorm", X, [1], g["norm_gamma6"], g["norm_bias6"]), "norm_inst_c1_affine"),
        (port.norm("instanceNorm", X, [2], g["norm_gamma5"], g["norm_bias5"]), "norm_inst_c2_affine"),
        (port.norm("batchNorm", X, [1]), "norm_batch_c1"),
        (port.norm("batchNorm", X, [1], g["norm_gamma6"], g["norm_bias6"]), "norm_batch_c1_affine"),
        (port.norm("batchNorm", X, [-1]), "norm_batch_cm1"),
        (port.norm("groupNorm", X, [1], groups=2), "norm_group2_c1"),
        (port.norm("groupNorm", X, [1], g["norm_gamma6"], g["norm_bias6"], groups=3), "norm_group3_c1_affine"),
        (port.norm("groupNorm", g["norm_xg"], [2], g["norm_gamma4"], g["norm_bias4"], groups=2), "norm_group2_c2_affine"),
    ]
    for got, name in exact:
        assert np.array_equal(got, g[name]), name
    # p = 1.5 goes through pow(): one ulp of libm against numpy
    got = port.norm("normalize", X, [1, 3], p=1.5, eps=1e-6)
    assert np.abs(got - g["norm_l15_a13"]).max() / np.abs(g["norm_l15_a13"]).max() < 1e-6


def test_port_causal_masked_matmul_matches_reference(port, golden_ext):
    g = golden_ext
    assert np.array_equal(port.masked_matmul_causal(g["mmc_a"], g["mmc_b"], 0, -1e9), g["mmc_off0"])
    assert np.array_equal(port.masked_matmul_causal(g["mmc_a"], g["mmc_b"], 20, 0.5), g["mmc_off20"])
