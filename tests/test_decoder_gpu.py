"""GPU parity tests of the decoder (ytcuda_qwen3_*) against the reference example model.

Contract: fp32 logits within 1e-4 of the reference's (normwise; fp32 sums in another order over 28 layers), and
argmax-identical greedy tokens for the first 32 decode steps on the Qwen3-0.6B shape with random bf16 weights."""
import hashlib

import numpy as np
import pytest

from _util import normwise

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

SMALL = dict(hidden_size=64, num_hidden_layers=2, vocab_size=512, intermediate_size=96, num_attention_heads=4,
             num_key_value_heads=2, head_dim=128, max_position_embeddings=64)


@pytest.fixture(scope="module")
def qwen3_golden():
    from pathlib import Path
    return np.load(Path(__file__).resolve().parent / "golden" / "golden_qwen3.npz")


@pytest.fixture(scope="module")
def Q():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from ytensor_b200 import qwen3
    return qwen3


def dev_ids(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.int32)).cuda()


@pytest.mark.parametrize("B", [1, 2])
def test_small_model_logits_match_reference(Q, qwen3_golden, B):
    cfg = Q.Qwen3Config(**SMALL)
    w = Q.random_weights(cfg, seed=4, std=0.05)
    assert hashlib.sha256(w["embed"].tobytes()).hexdigest() == str(qwen3_golden["small_embed_sha256"])
    m = Q.Qwen3ForCausalLM(cfg, batch=B)
    m.load_weights(w)
    want = qwen3_golden[f"small_logits_b{B}"]
    logits = m.forward(dev_ids(qwen3_golden[f"small_ids_b{B}"]))
    for step in range(6):
        got = logits.cpu().numpy()
        assert normwise(got, want[step]) < 1e-4
        assert np.array_equal(got.argmax(1), want[step].argmax(1))
        if step < 5:
            logits = m.forward(dev_ids(want[step].argmax(1).reshape(B, 1)))
    assert m.get_kv_cache_len() == 9 + 5
    m.reset_kv_cache()
    assert m.get_kv_cache_len() == 0
    m.close()


@pytest.mark.parametrize("B", [1, 2, 3, 4, 5, 8, 13, 16, 32])
def test_single_kernel_decode_step_matches_operator_path(Q, B):
    """The persistent step kernel (path 2: up to four sequences without grid barriers, activations exchanged as
    tagged pairs, weights streamed through a shared-memory ring, linear phases on mma.sync from bf16 planes of the
    activations; from five sequences on the kernel with grid barriers and tensor-core linear phases;
    path 3: FFMA linear phases where the kernel with grid barriers runs; path 4: the form without the weight ring;
    path 5: the ring with grid barriers)
    and the one-launch-per-operator forward compute the same logits and leave the same KV cache behind: 70 steps
    after a 40-token prompt (the attention of the step kernel goes from 2 to 4 key chunks), every model fed the
    tokens of the operator path."""
    # (the FFN width is larger than what the step kernel stages at once: the down projection then takes its input in
    # pieces, the last one shorter)
    cfg = Q.Qwen3Config(hidden_size=256, num_hidden_layers=3, vocab_size=1000, intermediate_size=2816,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=128)
    w = Q.random_weights(cfg, seed=11, std=0.05)
    ids = dev_ids(np.random.default_rng(B).integers(0, cfg.vocab_size, (B, 40)))
    ms = []
    for path in (1, 2, 3, 4, 5):
        m = Q.Qwen3ForCausalLM(cfg, batch=B)
        m.load_weights(w)
        m.set_decode_path(path)
        ms.append(m)
    # a single token into an empty cache (no prefill before it), then start over with the prompt
    first = ids[:, :1].contiguous()
    fa = ms[0].forward(first).cpu().numpy()
    for m in ms[1:]:
        assert normwise(m.forward(first).cpu().numpy(), fa) < 2e-5
    for m in ms:
        m.reset_kv_cache()
    la = ms[0].forward(ids)  # prefill: the same kernels in all three
    for m in ms[1:]:
        assert torch.equal(la, m.forward(ids))
    count = Q._lib.lib().ytcuda_launch_count
    for step in range(70):
        tok, _ = ms[0].argmax(la)
        tok = tok.reshape(B, 1).contiguous()
        n0 = count()
        la = ms[0].forward(tok)
        assert count() - n0 > 20
        a = la.cpu().numpy()
        for m in ms[1:]:
            n0 = count()
            lb = m.forward(tok)
            assert count() - n0 == 1
            assert normwise(lb.cpu().numpy(), a) < 2e-5, f"step {step}"
    assert all(m.get_kv_cache_len() == 110 for m in ms)
    assert Q._lib.lib().ytcuda_device_status(None) == 0
    for m in ms:
        m.close()
    if B == 32:  # more sequences than the step kernel holds: forcing it is refused, not silently rerouted
        m = Q.Qwen3ForCausalLM(cfg, batch=33)
        m.load_weights(w)
        m.set_decode_path(2)
        m.forward(dev_ids(np.zeros((33, 4))))
        with pytest.raises(Exception):
            m.forward(dev_ids(np.zeros((33, 1))))
        m.close()


def test_long_prefill_uses_tensor_cores_and_matches_oracle(Q, port):
    """More than 32 rows: activations are split into two bf16 planes and multiplied on tcgen05."""
    cfg = Q.Qwen3Config(**SMALL)
    w = Q.random_weights(cfg, seed=5, std=0.05)
    ids = np.random.default_rng(1).integers(0, cfg.vocab_size, (2, 40)).astype(np.int32)
    om = port.qwen3(cfg.oracle_dict(), 2)
    for key, arr in w.items():
        name, layer = (key, 0) if isinstance(key, str) else key
        om.set_weight(name, layer, Q.bf16_bits_to_f32(arr) if arr.dtype == np.uint16 else arr)
    want = om.forward(ids)
    m = Q.Qwen3ForCausalLM(cfg, batch=2)
    m.load_weights(w)
    got = m.forward(dev_ids(ids)).cpu().numpy()
    assert normwise(got, want) < 1e-4
    nxt = want.argmax(1).astype(np.int32).reshape(2, 1)
    assert normwise(m.forward(dev_ids(nxt)).cpu().numpy(), om.forward(nxt)) < 1e-4
    m.close()
    om.close()


@pytest.mark.parametrize("path", [1, 2])
def test_ring_buffer_cache_past_its_end_matches_reference(Q, path):
    """The reference's KV cache is a ring buffer: past its end a token overwrites the oldest slot, sees every slot and
    takes rotary position 0. Golden logits: 9-token prompt + 19 steps with max_position_embeddings = 16."""
    from pathlib import Path
    from ytensor_b200 import _lib
    g = np.load(Path(__file__).resolve().parent / "golden" / "golden_qwen3_wrap.npz")
    cfg = Q.Qwen3Config(**{**SMALL, "max_position_embeddings": 16})
    m = Q.Qwen3ForCausalLM(cfg, batch=1)
    m.load_weights(Q.random_weights(cfg, seed=4, std=0.05))
    m.set_decode_path(path)
    want = g["wrap_logits"]
    logits = m.forward(dev_ids(g["wrap_ids"]))
    for step in range(20):
        got = logits.cpu().numpy()
        assert normwise(got, want[step]) < 1e-4, step
        assert np.array_equal(got.argmax(1), want[step].argmax(1))
        assert m.get_kv_cache_len() == min(9 + step, 16)
        if step < 19:
            logits = m.forward(dev_ids(want[step].argmax(1).reshape(1, 1)))
    with pytest.raises(_lib.YtCudaInvalidArgument):  # more tokens at once than the ring has slots: refused
        m.forward(dev_ids(np.zeros((1, 17), np.int32)))
    m.close()


def test_several_tokens_per_call_across_the_end_of_the_ring(Q):
    """A forward of several tokens that runs over the end of the cache: every token is appended (the later ones
    overwrite the oldest slots), each query sees the slots that are not younger than itself, and the rotary positions
    restart as in Qwen3Model::forward (reference qwen3.cpp:70-126, 365-375). Golden logits: calls of 9, 5, 6, 3, 1 and
    10 tokens into a ring of 16 slots, two sequences."""
    from pathlib import Path
    g = np.load(Path(__file__).resolve().parent / "golden" / "golden_qwen3_wrap.npz")
    cfg = Q.Qwen3Config(**{**SMALL, "max_position_embeddings": 16})
    m = Q.Qwen3ForCausalLM(cfg, batch=2)
    m.load_weights(Q.random_weights(cfg, seed=4, std=0.05))
    want = g["multi_logits"]
    for i in range(want.shape[0]):
        got = m.forward(dev_ids(g[f"multi_ids_{i}"])).cpu().numpy()
        assert normwise(got, want[i]) < 1e-4, i
        assert np.array_equal(got.argmax(1), want[i].argmax(1)), i
    assert m.get_kv_cache_len() == 16
    m.close()


def test_cache_overflow_is_reported(Q):
    from ytensor_b200 import _lib
    cfg = Q.Qwen3Config(**SMALL)
    m = Q.Qwen3ForCausalLM(cfg, batch=1)
    m.load_weights(Q.random_weights(cfg, seed=4, std=0.05))
    m.forward(dev_ids(np.zeros((1, 60), np.int32)))
    m.forward(dev_ids(np.zeros((1, 5), np.int32)))  # runs over the end of the 64-slot ring: allowed
    assert m.get_kv_cache_len() == 64
    with pytest.raises(_lib.YtCudaInvalidArgument):  # more tokens than the ring has slots
        m.forward(dev_ids(np.zeros((1, 65), np.int32)))
    m.close()


def test_linear_w16_kernels(Q, port):
    from ytensor_b200 import _lib
    L = _lib.lib()
    rng = np.random.default_rng(2)
    for M, N, K in [(1, 1000, 1024), (3, 200, 768), (5, 77, 512), (32, 300, 3072), (100, 256, 1024), (9, 8, 8)]:
        x = rng.standard_normal((M, K)).astype(np.float32)
        wb = Q.f32_to_bf16_bits((rng.standard_normal((N, K)) * 0.05).astype(np.float32))
        want = port.matmul(x, np.ascontiguousarray(Q.bf16_bits_to_f32(wb).T))
        tx = torch.from_numpy(x).cuda()
        tw = torch.from_numpy(wb.view(np.int16)).cuda()
        y = torch.empty(M, N, device="cuda")
        scratch = torch.empty(4 * M * K, dtype=torch.uint8, device="cuda")
        _lib.check(L.ytcuda_linear_w16(tx.data_ptr(), K, tw.data_ptr(), y.data_ptr(), N, M, N, K, 0,
                                       scratch.data_ptr(), None))
        assert normwise(y.cpu().numpy(), want) < 2e-5
        _lib.check(L.ytcuda_linear_w16(tx.data_ptr(), K, tw.data_ptr(), y.data_ptr(), N, M, N, K, 1,
                                       scratch.data_ptr(), None))
        assert normwise(y.cpu().numpy(), 2 * want) < 2e-5


def test_full_model_greedy_tokens_match_reference(Q, qwen3_golden):
    """benchmark configuration 5, batch 1: 512-token prompt, 32 greedy steps, tokens identical to the reference's."""
    cfg = Q.Qwen3Config(max_position_embeddings=768)
    w = Q.random_weights(cfg, seed=4)
    assert hashlib.sha256(w["embed"].tobytes()).hexdigest() == str(qwen3_golden["full_embed_sha256"])
    m = Q.Qwen3ForCausalLM(cfg, batch=1)
    m.load_weights(w)
    logits = m.forward(dev_ids(qwen3_golden["full_prompt"]))
    want_tok, top_i, top_v = qwen3_golden["full_tokens"], qwen3_golden["full_top8_indices"], qwen3_golden["full_top8_values"]
    for s in range(32):
        tok, _ = m.argmax(logits)
        got = logits[0].cpu().numpy()
        assert int(tok[0]) == int(want_tok[s]), f"step {s}: margin in the reference was {qwen3_golden['full_margins'][s]}"
        assert np.abs(got[top_i[s]] - top_v[s]).max() < 1e-3
        if s < 31:
            logits = m.forward(tok.reshape(1, 1).contiguous())
    # batch 2 with the same prompt twice gives the same tokens in both rows
    m.close()
    m2 = Q.Qwen3ForCausalLM(cfg, batch=2)
    m2.load_weights(w)
    p2 = np.repeat(qwen3_golden["full_prompt"], 2, axis=0)
    toks = m2.generate_greedy(dev_ids(p2), 8).cpu().numpy()
    assert np.array_equal(toks[0], want_tok[:8]) and np.array_equal(toks[1], want_tok[:8])
    m2.close()


def test_full_model_32_sequences_match_reference(Q):
    """benchmark configuration 5 at batch 32: the operator path that 32 sequences take (tcgen05 linears on hi + lo bf16 planes
    with split-k pieces, attn_decode_fast_kernel, fused glue) against the reference run with 32 distinct prompts.
    The reference's prompt is 16 tokens per sequence (its prefill of 32 x 512 tokens would take most of an hour on the
    CPU); the 32 greedy decode steps are the full count. Tokens must be identical wherever the reference's own margin
    between its two best logits is above the fp32 noise of the comparison, and the logits of the reference's four
    best tokens must agree to 1e-3 at every step; the device is fed the reference's tokens, so that one near-tie
    cannot hide the steps after it."""
    from pathlib import Path
    g = np.load(Path(__file__).resolve().parent / "golden" / "golden_qwen3_b32.npz")
    cfg = Q.Qwen3Config(max_position_embeddings=64)
    w = Q.random_weights(cfg, seed=4)
    assert hashlib.sha256(w["embed"].tobytes()).hexdigest() == str(g["embed_sha256"])
    m = Q.Qwen3ForCausalLM(cfg, batch=32)
    m.load_weights(w)
    want_tok, margins, top_i, top_v = g["tokens"], g["margins"], g["top4_indices"], g["top4_values"]
    logits = m.forward(dev_ids(g["prompt"]))
    free_running_equal = True
    fed = None
    for s in range(32):
        tok, _ = m.argmax(logits)
        got_tok = tok.cpu().numpy()
        got = logits.cpu().numpy()
        picked = np.take_along_axis(got, top_i[:, s, :].astype(np.int64), axis=1)
        assert np.abs(picked - top_v[:, s, :]).max() < 1e-3, s
        clear = margins[:, s] > 2e-3
        assert np.array_equal(got_tok[clear], want_tok[clear, s]), (s, got_tok, want_tok[:, s])
        free_running_equal &= bool(np.array_equal(got_tok, want_tok[:, s]))
        if s < 31:
            fed = dev_ids(want_tok[:, s].reshape(32, 1))
            logits = m.forward(fed)
    assert (margins > 2e-3).mean() > 0.97  # the check above covered nearly every token
    assert free_running_equal or (margins <= 2e-3).any()
    m.close()
