"""CPU (gloo, world_size 2): the host-side tensor-parallel logic of the decoder. Each rank slices the weights with
shard_weight, computes its partial projections with numpy, and an all-reduce over gloo must reproduce the unsharded
result; the vocabulary split must tile the vocabulary; the (value, index) exchange must find the first global
maximum. No GPU and no device library involved."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

SMALL = dict(hidden_size=64, num_hidden_layers=1, vocab_size=515, intermediate_size=96, num_attention_heads=4,
             num_key_value_heads=2, head_dim=128, max_position_embeddings=16)


def _worker(rank: int, world: int, port: int, ret):
    import torch
    import torch.distributed as dist
    from ytensor_b200.qwen3 import Qwen3Config, bf16_bits_to_f32, random_weights, shard_weight, vocab_rows

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = Qwen3Config(**SMALL)
        w = random_weights(cfg, seed=3, std=0.05)
        f = lambda name: bf16_bits_to_f32(w[(name, 0)])  # noqa: E731
        H, KV, D, I = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size
        rng = np.random.default_rng(0)
        x = rng.standard_normal((5, cfg.hidden_size)).astype(np.float32)

        # attention block: local heads -> partial o_proj output -> all-reduce == full
        qkv_full = x @ f("qkv").T
        qkv_loc = x @ bf16_bits_to_f32(shard_weight(cfg, "qkv", w[("qkv", 0)], rank, world)).T
        hq, hk = H // world, KV // world
        assert np.array_equal(qkv_loc[:, : hq * D], qkv_full[:, rank * hq * D: (rank + 1) * hq * D])
        assert np.array_equal(qkv_loc[:, hq * D: (hq + hk) * D],
                              qkv_full[:, (H + rank * hk) * D: (H + (rank + 1) * hk) * D])
        assert np.array_equal(qkv_loc[:, (hq + hk) * D:],
                              qkv_full[:, (H + KV + rank * hk) * D: (H + KV + (rank + 1) * hk) * D])
        attn_full = rng.standard_normal((5, H * D)).astype(np.float32)  # stands for the attention output
        attn_loc = attn_full[:, rank * hq * D: (rank + 1) * hq * D]
        part = torch.from_numpy(attn_loc @ bf16_bits_to_f32(shard_weight(cfg, "o", w[("o", 0)], rank, world)).T)
        dist.all_reduce(part)
        assert np.allclose(part.numpy(), attn_full @ f("o").T, rtol=1e-5, atol=1e-5)

        # MLP: local gate/up columns -> swiglu -> partial down -> all-reduce == full
        gu_loc = x @ bf16_bits_to_f32(shard_weight(cfg, "gate_up", w[("gate_up", 0)], rank, world)).T
        il = I // world
        sw = lambda g: g / (1.0 + np.exp(-g))  # noqa: E731
        act_loc = sw(gu_loc[:, :il]) * gu_loc[:, il:]
        part = torch.from_numpy((act_loc @ bf16_bits_to_f32(shard_weight(cfg, "down", w[("down", 0)], rank, world)).T)
                                .astype(np.float32))
        dist.all_reduce(part)
        gu = x @ f("gate_up").T
        full = (sw(gu[:, :I]) * gu[:, I:]) @ f("down").T
        assert np.allclose(part.numpy(), full, rtol=1e-4, atol=1e-5)

        # vocabulary split and the greedy-token exchange
        b, e = vocab_rows(cfg, rank, world)
        spans = [None] * world
        dist.all_gather_object(spans, (b, e))
        assert spans[0][0] == 0 and spans[-1][1] == cfg.vocab_size
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        emb = bf16_bits_to_f32(w["embed"])
        logits = x @ emb.T
        logits[0, 7] = logits[0, 400] = logits[0].max() + 1.0  # a tie across the two ranks: the first index wins
        loc = logits[:, b:e]
        val = torch.from_numpy(loc.max(1).astype(np.float32))
        idx = torch.from_numpy((loc.argmax(1) + b).astype(np.int64))
        vals = [torch.empty_like(val) for _ in range(world)]
        idxs = [torch.empty_like(idx) for _ in range(world)]
        dist.all_gather(vals, val)
        dist.all_gather(idxs, idx)
        v = torch.stack(vals, 1).numpy()
        which = v.argmax(1)  # numpy argmax returns the first maximum, ranks are in ascending vocabulary order
        tok = torch.stack(idxs, 1).numpy()[np.arange(5), which]
        assert np.array_equal(tok, logits.argmax(1))
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_sharding_with_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = 29500 + (os.getpid() % 2000)
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
        for p in procs:
            if p.is_alive():
                p.kill()
                pytest.fail("a gloo rank did not finish")
        assert dict(ret) == {0: "ok", 1: "ok"}, f"ranks failed: {dict(ret)}, exit codes {[p.exitcode for p in procs]}"


def test_shard_weight_is_identity_for_one_rank():
    from ytensor_b200.qwen3 import Qwen3Config, random_weights, shard_weight
    cfg = Qwen3Config(**SMALL)
    w = random_weights(cfg, seed=3)
    for key, arr in w.items():
        name = key if isinstance(key, str) else key[0]
        assert shard_weight(cfg, name, arr, 0, 1) is arr
