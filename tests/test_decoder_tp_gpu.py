"""GPU (2, 4 or 8 devices): the tensor-parallel decoder gives the reference's logits and greedy tokens.
One child process per GPU; the partial sums after the attention output and down projections are reduced by NCCL
(prefill, and decode with one launch per operator) or inside the persistent decode-step kernel over peer memory.
A second test lets one rank skip a decode step: the other rank's step kernel waits for it with a short cycle budget,
gives up, reports YTC_TIMEOUT, and the group recovers. Each case is skipped when too few devices are visible."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]

SMALL = dict(hidden_size=64, num_hidden_layers=2, vocab_size=512, intermediate_size=96, num_attention_heads=4,
             num_key_value_heads=2, head_dim=128, max_position_embeddings=64)


def _worker(rank, world, port, ret):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    from ytensor_b200 import qwen3 as Q
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        g = np.load(ROOT / "tests" / "golden" / "golden_qwen3.npz")
        # small model: full logits against the reference, every rank holding its vocabulary rows; first with the
        # decode steps as one kernel per rank (all-reduce inside it, through the peers' exchange buffers), then with
        # one launch per operator and the NCCL all-reduce callback
        cfg = Q.Qwen3Config(**SMALL)
        want = g["small_logits_b2"]
        ids = torch.from_numpy(g["small_ids_b2"]).cuda()
        for path in ((2, 1) if world == 2 else ()):  # (the small reference model has two kv heads)
            m = Q.Qwen3ForCausalLM(cfg, batch=2, tp_rank=rank, tp_world=world)
            m.load_weights(Q.random_weights(cfg, seed=4, std=0.05))
            m.set_decode_path(path)
            logits = m.forward(ids)
            for step in range(6):
                got = logits.cpu().numpy()
                ref = want[step][:, m.v0:m.v1]
                err = np.abs(got - ref).max() / np.abs(want[step]).max()
                assert err < 1e-4, (path, step, err)
                tok, _ = m.argmax(logits)
                assert np.array_equal(tok.cpu().numpy(), want[step].argmax(1))
                if step < 5:
                    n0 = Q._lib.lib().ytcuda_launch_count()
                    logits = m.forward(tok.reshape(2, 1).contiguous())
                    launched = Q._lib.lib().ytcuda_launch_count() - n0
                    assert (launched == 1) if path == 2 else (launched > 10), (path, launched)
            assert Q._lib.lib().ytcuda_device_status(None) == 0
            m.close()
        # six sequences: the step kernel's linear phases run on the tensor cores (mma.sync form), the sums over ranks
        # still inside the kernel; against the operator path with the NCCL callback, both fed the same tokens
        cfg = Q.Qwen3Config(hidden_size=256, num_hidden_layers=3, vocab_size=1000, intermediate_size=2816,
                            num_attention_heads=4 if world == 2 else 16, num_key_value_heads=2 if world == 2 else 8,
                            head_dim=128, max_position_embeddings=128)
        w = Q.random_weights(cfg, seed=11, std=0.05)
        # path 6: one launch per operator, sums over ranks by the NCCL callback; path 1: the same launches with the
        # ranks' shares pushed to the peers inside the kernels that add a projection to the residual stream;
        # path 2: the step kernel. All fed the tokens of path 6.
        for nseq in (6, 16):
            ids = torch.from_numpy(np.random.default_rng(nseq).integers(0, cfg.vocab_size, (nseq, 20)).astype(np.int32)).cuda()
            ms = []
            for path in (6, 1, 2):
                m = Q.Qwen3ForCausalLM(cfg, batch=nseq, tp_rank=rank, tp_world=world)
                m.load_weights(w)
                m.set_decode_path(path)
                ms.append(m)
            la = ms[0].forward(ids)
            for m in ms[1:]:
                b, a = m.forward(ids).cpu().numpy(), la.cpu().numpy()
                assert np.linalg.norm(b - a) / np.linalg.norm(a) < 2e-5, (nseq, "prefill")
            for step in range(12):
                tok, _ = ms[0].argmax(la)
                tok = tok.reshape(nseq, 1).contiguous()
                la = ms[0].forward(tok)
                a = la.cpu().numpy()
                for m, launches in ((ms[1], None), (ms[2], 1)):
                    n0 = Q._lib.lib().ytcuda_launch_count()
                    b = m.forward(tok).cpu().numpy()
                    if launches:
                        assert Q._lib.lib().ytcuda_launch_count() - n0 == launches
                    assert np.linalg.norm(b - a) / np.linalg.norm(a) < 2e-5, (nseq, step, np.linalg.norm(b - a) / np.linalg.norm(a))
            assert Q._lib.lib().ytcuda_device_status(None) == 0
            for m in ms:
                m.close()
        # Qwen3-0.6B shape: the first 16 greedy tokens of the reference
        cfg = Q.Qwen3Config(max_position_embeddings=768)
        m = Q.Qwen3ForCausalLM(cfg, batch=1, tp_rank=rank, tp_world=world)
        m.load_weights(Q.random_weights(cfg, seed=4))
        toks = m.generate_greedy(torch.from_numpy(g["full_prompt"]).cuda(), 16).cpu().numpy()[0]
        assert np.array_equal(toks, g["full_tokens"][:16]), (toks, g["full_tokens"][:16])
        m.close()
        ret[rank] = "ok"
    except Exception as e:  # noqa: BLE001 - reported to the parent
        ret[rank] = f"{type(e).__name__}: {e}"
    finally:
        dist.destroy_process_group()


def _run_ranks(target, world):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = 29600 + (os.getpid() % 2000) + world
        procs = [ctx.Process(target=target, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(900)
        for p in procs:
            if p.is_alive():
                p.kill()
                pytest.fail("a rank did not finish")
        assert dict(ret) == {r: "ok" for r in range(world)}, dict(ret)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_matches_reference(world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} CUDA devices")
    _run_ranks(_worker, world)


def _timeout_worker(rank, world, port, ret):
    """Rank 1 leaves out one decode step (between steps, nothing of its own in flight); rank 0's step kernel waits for
    rank 1's arrival word with a 20 ms budget, gives up and returns; the status word says so; the group recovers and
    reproduces the reference's logits."""
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    from ytensor_b200 import _lib
    from ytensor_b200 import qwen3 as Q
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    L = _lib.lib()
    try:
        g = np.load(ROOT / "tests" / "golden" / "golden_qwen3.npz")
        cfg = Q.Qwen3Config(**SMALL)
        want = g["small_logits_b2"]
        ids = torch.from_numpy(g["small_ids_b2"]).cuda()
        m = Q.Qwen3ForCausalLM(cfg, batch=2, tp_rank=rank, tp_world=world)
        m.load_weights(Q.random_weights(cfg, seed=4, std=0.05))
        m.set_decode_path(2)
        logits = m.forward(ids)
        tok, _ = m.argmax(logits)
        tok = tok.reshape(2, 1).contiguous()
        logits = m.forward(tok)       # one good step on both ranks
        m.check_status()
        dist.barrier()
        old = L.ytcuda_get_wait_limit()
        _lib.check(L.ytcuda_set_wait_limit(40_000_000))   # about 20 ms
        if rank == 0:
            t0 = __import__("time").perf_counter()
            m.forward(tok)            # rank 1 never launches this step
            try:
                m.check_status()
                raise AssertionError("the step kernel should have given up on its peer")
            except _lib.YtCudaError as e:
                assert e.status == _lib.TIMEOUT, e
            assert __import__("time").perf_counter() - t0 < 5.0
        _lib.check(L.ytcuda_set_wait_limit(old))
        m.recover()                   # every rank: barrier, counters and arrival words to zero, barrier
        logits = m.forward(ids)
        for step in range(4):
            got = logits.cpu().numpy()
            err = np.abs(got - want[step][:, m.v0:m.v1]).max() / np.abs(want[step]).max()
            assert err < 1e-4, (step, err)
            tok, _ = m.argmax(logits)
            logits = m.forward(tok.reshape(2, 1).contiguous())
        m.check_status()
        m.close()
        ret[rank] = "ok"
    except Exception as e:  # noqa: BLE001 - reported to the parent
        ret[rank] = f"{type(e).__name__}: {e}"
    finally:
        dist.destroy_process_group()


def test_step_kernel_gives_up_on_a_missing_peer_and_the_group_recovers():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    _run_ranks(_timeout_worker, 2)
