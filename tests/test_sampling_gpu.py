"""GPU parity of ytcuda_topk_sample with the sample_token step of the reference's generate loop (softmax, the 20 most
probable tokens, a uniform draw over their sum): golden vectors from the reference's softmax, and the oracle on a
vocabulary of the Qwen3 size. Probabilities within 1e-5 (relative to the largest), indices and sampled tokens equal."""
import numpy as np
import pytest

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


def test_golden(api, golden):
    p, i, s = api.topk_sample(dev(golden["topk_logits"]), 20, dev(golden["topk_uniform"]))
    assert np.array_equal(i.cpu().numpy(), golden["topk_idx"])
    assert np.abs(p.cpu().numpy() - golden["topk_probs"]).max() < 1e-5 * golden["topk_probs"].max()
    assert np.array_equal(s.cpu().numpy(), golden["topk_sampled"])


@pytest.mark.parametrize("rows,vocab,k", [(1, 151936, 20), (4, 151936, 20), (2, 33, 33), (3, 1000, 1), (2, 5000, 64)])
def test_against_oracle(api, port, rows, vocab, k):
    rng = np.random.default_rng(rows * 7 + k)
    logits = (rng.standard_normal((rows, vocab)) * 4).astype(np.float32)
    uniform = rng.random(rows).astype(np.float32)
    uniform[0] = 1.0  # the far end of the interval picks the last kept token at most
    wp, wi, ws = port.topk_sample(logits, k, uniform)
    wide = dev(np.concatenate([logits, np.zeros((rows, 5), np.float32)], axis=1))[:, :vocab]  # a strided row view
    p, i, s = api.topk_sample(wide, k, dev(uniform))
    got_p = p.cpu().numpy()
    assert np.array_equal(i.cpu().numpy(), wi)
    # the reference's softmax adds the exponentials of a row one after the other in fp32, which drifts on a row of
    # 150 k entries: the bound is 1e-5 against exact (float64) probabilities, or the oracle's own distance from them
    z = logits.astype(np.float64) - logits.max(1, keepdims=True)
    exact = np.take_along_axis(np.exp(z) / np.exp(z).sum(1, keepdims=True), wi.astype(np.int64), axis=1)
    bound = np.maximum(1e-5 * exact.max(), np.abs(wp - exact).max())
    assert np.abs(got_p - exact).max() <= bound
    # the selection rule of the reference applied to the probabilities the device kept
    for r in range(rows):
        kept = np.float32(0)
        for j in range(k):
            kept = np.float32(kept + got_p[r, j])
        cum, want = np.float32(0), wi[r, 0]
        for j in range(k):
            cum = np.float32(cum + got_p[r, j])
            if np.float32(uniform[r]) * kept <= cum:
                want = wi[r, j]
                break
        assert int(s[r]) == int(want)
    if vocab <= 5000:
        assert np.array_equal(s.cpu().numpy(), ws) and np.abs(got_p - wp).max() < 1e-5 * wp.max()
    # without a uniform draw nothing is sampled; probabilities descend
    p2, i2, s2 = api.topk_sample(dev(logits), k)
    assert s2 is None and torch.equal(i2, i) and bool((p2[:, :-1] >= p2[:, 1:]).all())


def test_ties_take_the_lower_index_and_bad_k_is_refused(api):
    x = torch.zeros(1, 100, device="cuda")
    x[0, [7, 3, 50]] = 2.0
    p, i, _ = api.topk_sample(x, 4)
    assert i[0, :3].tolist() == [3, 7, 50] and i[0, 3].item() == 0
    with pytest.raises(ValueError):
        api.topk_sample(x, 65)
    with pytest.raises(ValueError):
        api.topk_sample(x, 0)


def test_sampled_generation_stays_inside_the_top_k(api):
    from ytensor_b200 import qwen3 as Q
    cfg = Q.Qwen3Config(hidden_size=64, num_hidden_layers=2, vocab_size=512, intermediate_size=96, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=128, max_position_embeddings=64)
    m = Q.Qwen3ForCausalLM(cfg, batch=2)
    m.load_weights(Q.random_weights(cfg, seed=4, std=0.05))
    ids = dev(np.random.default_rng(0).integers(0, 512, (2, 7)).astype(np.int32))
    a = m.generate_topk(ids, 12, k=5, seed=1).cpu().numpy()
    m.reset_kv_cache()
    b = m.generate_topk(ids, 12, k=5, seed=1).cpu().numpy()
    assert np.array_equal(a, b)                      # the same seed gives the same tokens
    m.reset_kv_cache()
    g = m.generate_topk(ids, 12, k=1).cpu().numpy()  # k = 1 is greedy decoding
    m.reset_kv_cache()
    assert np.array_equal(g, m.generate_greedy(ids, 12).cpu().numpy())
    m.close()
