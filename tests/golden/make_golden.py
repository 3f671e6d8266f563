"""Generates tests/golden/golden_ops.npz by running the UNMODIFIED reference (compiled behind
oracle/ref_shim.cpp into oracle/_ref/libyt_ref.so) on small seeded inputs.

Run from the repository root, where the reference sources are available:
    make -C oracle ref REF=<YTensor source tree> && python tests/golden/make_golden.py
Inputs are stored next to outputs, so the fixtures do not depend on a random generator staying
stable. Cases named doc_* use the literal inputs of the reference's documentation examples
(doc/en/api/function/fused.mdx:69-73 matmul, :190-201 scaledDotProductAttention).
"""
from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle as O  # noqa: E402

OUT = Path(__file__).resolve().parent / "golden_ops.npz"


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main() -> None:
    R = O.ref(threads=1)
    rng = np.random.default_rng(20240607)
    g: dict[str, np.ndarray] = {}

    def N(*shape, scale=1.0):
        return (rng.standard_normal(shape) * scale).astype(np.float32)

    # ---- casts ---------------------------------------------------------------------------
    x = (rng.standard_normal(4096) * np.exp(rng.uniform(-24, 14, 4096))).astype(np.float32)
    x[:16] = [0.0, -0.0, np.inf, -np.inf, np.nan, 1e-8, 65504.0, 65520.0, 6.0e-5, 6.1035e-5, 6.104e-5, 1.0 + 3.0 / 512,
              1.0 + 1.0 / 256, 3.3895e38, -1.0, 2.0 ** -14 * (1 - 2.0 ** -12)]
    g["cast_x"] = x
    g["cast_bf16"] = R.f32_to_bf16(x)
    g["cast_f16"] = R.f32_to_f16(x)
    allbits = np.arange(65536, dtype=np.uint16)
    g["cast_f16_to_f32_all_sha256"] = np.array(sha(R.f16_to_f32(allbits).view(np.uint32)))
    g["cast_bf16_to_f32_all_sha256"] = np.array(sha(R.bf16_to_f32(allbits).view(np.uint32)))

    # ---- matmul --------------------------------------------------------------------------
    a = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    b = np.array([[1, 0, 0, 1], [0, 1, 1, 0], [1, 1, 0, 0]], np.float32)
    g["doc_matmul_a"], g["doc_matmul_b"], g["doc_matmul_c"] = a, b, R.matmul(a[None], b)[0]
    a, b2, b3 = N(3, 33, 29), N(29, 17), N(3, 29, 17)
    g["mm_a"], g["mm_b2"], g["mm_b3"] = a, b2, b3
    g["mm_c_shared"], g["mm_c_batched"] = R.matmul(a, b2), R.matmul(a, b3)
    g["mm_c_shared_naive"] = R.matmul(a, b2, backend=0)
    a, b = N(1, 140, 610), N(610, 75)  # k above the reference's KC = 500 block
    g["mm_big_a"], g["mm_big_b"], g["mm_big_c"] = a, b, R.matmul(a, b)
    x, w, bias = N(7, 40), N(24, 40), N(24)
    g["lin_x"], g["lin_w"], g["lin_bias"] = x, w, bias
    g["lin_y"], g["lin_y_bias"] = R.linear(x, w), R.linear(x, w, bias)
    A, B, C0 = N(40, 30), N(20, 30), N(40, 20)
    g["sgemm_a"], g["sgemm_bt"], g["sgemm_c0"] = A, B, C0
    g["sgemm_out"] = R.sgemm(A, B.T, C0, 0.5, 2.0)
    At = N(30, 40)
    g["sgemm_at"] = At
    g["sgemm_out_at"] = R.sgemm(At.T, B.T, C0, 1.0, 0.0)
    # 16-bit storage recipe: widen -> fp32 matmul -> narrow with the type's own constructor
    for name, dt, f2b in (("bf16", 1, R.f32_to_bf16), ("f16", 2, R.f32_to_f16)):
        a_bits, b_bits = f2b(N(2, 48, 64, scale=1.0)), f2b(N(64, 40, scale=0.125))
        g[f"mm16_{name}_a"], g[f"mm16_{name}_b"] = a_bits, b_bits
        g[f"mm16_{name}_c"] = R.matmul_16(a_bits, b_bits, dt)

    # ---- N-d ops -------------------------------------------------------------------------
    X = N(2, 3, 5, 16)
    g["nd_x"] = X
    for tag, axes in (("m1", [-1]), ("a1", [1]), ("a0", [0]), ("a23", [2, 3]), ("a13", [1, 3]), ("a31", [3, 1])):
        ax_shape = [X.shape[a] for a in axes]
        w = rng.uniform(0.9, 1.1, ax_shape).astype(np.float32)
        bb = N(*ax_shape)
        g[f"nd_{tag}_axes"] = np.array(axes, np.int32)
        g[f"nd_{tag}_w"], g[f"nd_{tag}_b"] = w, bb
        g[f"nd_{tag}_softmax"] = R.softmax(X, axes)
        g[f"nd_{tag}_rmsnorm"] = R.rmsnorm(X, w, axes, 1e-6)
        g[f"nd_{tag}_layernorm"] = R.layernorm(X, w, bb, axes, 1e-5)
        g[f"nd_{tag}_layernorm_plain"] = R.layernorm(X, None, None, axes, 1e-5)
        g[f"nd_{tag}_sum"] = R.reduce(X, axes, "sum")
        g[f"nd_{tag}_mean"] = R.reduce(X, axes, "mean")
        mv, mi = R.reduce(X, axes, "max")
        g[f"nd_{tag}_max"], g[f"nd_{tag}_argmax"] = mv, mi
    Y = X[:1, :, :1, :] + 3.0
    g["bin_y"] = np.ascontiguousarray(Y)
    for op in ("add", "sub", "mul", "div"):
        g[f"bin_{op}"] = R.binary(X, Y, op)
    sx = N(513, scale=6.0)
    g["swish_x"], g["swish_y"] = sx, R.swish(sx)

    # ---- the memory-bound chain ----------------------------------------------------------
    x, w = N(2, 5, 128), rng.uniform(0.9, 1.1, 128).astype(np.float32)
    r1, r2 = N(1, 5, 128), N(2, 5, 128)
    g["chain_x"], g["chain_w"], g["chain_r1"], g["chain_r2"] = x, w, r1, r2
    g["chain_out_r1"], g["chain_out_r2"] = R.chain(x, w, r1), R.chain(x, w, r2)

    # ---- attention -----------------------------------------------------------------------
    q = np.array([[0.1, 0.0, 0.2, 0.3], [0.0, 0.4, 0.2, 0.1]], np.float32).reshape(1, 1, 1, 2, 4)
    k = np.array([[0.2, 0.1, 0.0, 0.3], [0.0, 0.2, 0.4, 0.1], [0.3, 0.0, 0.1, 0.2]], np.float32).reshape(1, 1, 3, 4)
    v = np.eye(3, 5, dtype=np.float32).reshape(1, 1, 3, 5)
    m = np.array([[1, 1, 0], [1, 1, 1]], np.uint8)
    g["doc_sdpa_q"], g["doc_sdpa_k"], g["doc_sdpa_v"], g["doc_sdpa_mask"] = q, k, v, m
    g["doc_sdpa_out_math_mask"] = R.sdpa(q, k, v, mask=m, backend=0)
    g["doc_sdpa_out_flash_mask"] = R.sdpa(q, k, v, mask=m, backend=1)
    # the documentation's predicate is j <= i, i.e. causal with offset 0: a bool mask states it exactly
    tri = np.tril(np.ones((2, 3), np.uint8))
    g["doc_sdpa_out_flash_pred"] = R.sdpa(q, k, v, mask=tri, backend=1)

    q, k, v = N(1, 2, 2, 19, 32), N(1, 2, 19, 32), N(1, 2, 19, 32)
    g["att_q"], g["att_k"], g["att_v"] = q, k, v
    g["att_causal"] = R.sdpa(q, k, v, causal=True)
    g["att_causal_math"] = R.sdpa(q, k, v, mask=np.tril(np.ones((19, 19), np.uint8)), backend=0)
    g["att_full"] = R.sdpa(q, k, v)
    m = (rng.random((19, 19)) < 0.5).astype(np.uint8)
    m[4] = 0  # a query row that sees no key: output row must be zero
    g["att_mask"] = m
    g["att_masked"] = R.sdpa(q, k, v, mask=m)
    bias = N(19, 19)
    g["att_bias"] = bias
    g["att_bias_causal"] = R.sdpa(q, k, v, causal=True, bias=bias, scale=0.2)
    q2 = N(1, 2, 2, 7, 32)  # q_len != kv_len: causal window anchored at the end of the keys
    g["att_q_short"] = q2
    g["att_short_causal"] = R.sdpa(q2, k, v, causal=True)
    q1 = N(1, 2, 2, 1, 32)  # decode step
    g["att_q_one"] = q1
    g["att_decode"] = R.sdpa(q1, k, v, causal=True)

    # ---- masked matmul (appended last so that the draws above stay what they were) -------------
    a, b2, b3 = N(2, 37, 45), N(45, 26), N(2, 45, 26)
    mk = np.random.default_rng(77).random((37, 26)) < 0.6
    mk[5, :] = False   # a row with nothing kept
    mk[:, 7] = True    # a column kept everywhere
    g["mmask_a"], g["mmask_b2"], g["mmask_b3"], g["mmask_mask"] = a, b2, b3, mk
    g["mmask_c_shared"] = R.masked_matmul(a, b2, mk, -1.5)
    g["mmask_c_batched"] = R.masked_matmul(a, b3, mk, 0.0)
    g["mmask_c_shared_naive"] = R.masked_matmul(a, b2, mk, -1.5, backend=0)

    # ---- top-k sampling: probabilities from the reference's softmax, k = 20 as in its generate loop -----------
    lg = (N(3, 5000) * 3.0).astype(np.float32)
    un = np.array([0.0, 0.37, 0.999], np.float32)
    tp, ti, ts = R.topk_sample(lg, 20, un)
    g["topk_logits"], g["topk_uniform"], g["topk_probs"], g["topk_idx"], g["topk_sampled"] = lg, un, tp, ti, ts

    # ---- the other activations, forward form; values around the branch points and in both tails -------------
    ax = np.concatenate([N(4000) * 3.0, np.array([0.0, -0.0, 3.0, -3.0, 2.9999998, -2.9999998, 20.0, -20.0, 88.0,
                                                  -88.0, -104.0, 1e-8, -1e-8], np.float32)]).astype(np.float32)
    g["act_x"] = ax
    for name in ("relu", "exp", "sigmoid", "leakyRelu", "elu", "selu", "gelu", "tanh", "softplus", "mish",
                 "hardSigmoid", "hardSwish"):
        g[f"act_{name}"] = R.activation(name, ax)
    g["act_leakyRelu_0p2"] = R.activation("leakyRelu", ax, 0.2)
    g["act_elu_0p5"] = R.activation("elu", ax, 0.5)

    # ---- first derivatives (order = 1) of the activations on the same inputs -------------
    for name in ("swish", "relu", "exp", "sigmoid", "leakyRelu", "elu", "selu", "gelu", "tanh", "softplus", "mish",
                 "hardSigmoid", "hardSwish"):
        g[f"actd_{name}"] = R.activation(name, ax, order=1)
    g["actd_leakyRelu_0p2"] = R.activation("leakyRelu", ax, 0.2, order=1)
    g["actd_elu_0p5"] = R.activation("elu", ax, 0.5, order=1)

    np.savez_compressed(OUT, **g)
    print(f"wrote {OUT} ({OUT.stat().st_size / 1024:.0f} KiB, {len(g)} arrays)")


if __name__ == "__main__":
    main()
