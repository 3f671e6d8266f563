"""Host side of the decoder workload: configuration, seeded random weights, tensor-parallel slicing and a thin
wrapper over the model handle of the C ABI (ytcuda_qwen3_*).

Mirrors qwen3::Qwen3Config / Qwen3ForCausalLM of the reference's example (example/qwen3/include/qwen3.hpp:46-168):
same defaults, same fused weight layout (qkv_proj = [q; k; v] rows, gate_up = [gate; up] rows, weights stored
[out_features, in_features]). torch is used for device memory and for the NCCL all-reduce only.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import asdict, dataclass

import numpy as np

from . import _lib
from ._lib import check, lib


@dataclass
class Qwen3Config:
    hidden_size: int = 1024
    num_hidden_layers: int = 28
    vocab_size: int = 151936
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    intermediate_size: int = 3072
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    max_position_embeddings: int = 4096

    def oracle_dict(self) -> dict:
        return {"hidden": self.hidden_size, "layers": self.num_hidden_layers, "vocab": self.vocab_size,
                "inter": self.intermediate_size, "heads": self.num_attention_heads,
                "kv_heads": self.num_key_value_heads, "head_dim": self.head_dim, "eps": self.rms_norm_eps,
                "theta": self.rope_theta, "max_pos": self.max_position_embeddings}


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """yt::bfloat16(float) on the host (reference include/types/bfloat16.hpp:78-80), vectorised."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + ((u & np.uint32(0x10000)) >> np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def random_weights(cfg: Qwen3Config, seed: int = 4, std: float = 0.02) -> dict:
    """bf16 weights ~ N(0, std) (uint16 bit patterns), norm weights = 1 (fp32), tied vocabulary matrix.
    Key: name or (name, layer). One generator, fixed order: embed, then per layer qkv, o, gate_up, down."""
    rng = np.random.Generator(np.random.PCG64(seed))
    H, D = cfg.hidden_size, cfg.head_dim
    qkv_rows = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * D

    def mat(rows, cols):
        return f32_to_bf16_bits(rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(std))

    w: dict = {"embed": mat(cfg.vocab_size, H), "norm": np.ones(H, np.float32)}
    for l in range(cfg.num_hidden_layers):
        w[("qkv", l)] = mat(qkv_rows, H)
        w[("o", l)] = mat(H, cfg.num_attention_heads * D)
        w[("gate_up", l)] = mat(2 * cfg.intermediate_size, H)
        w[("down", l)] = mat(H, cfg.intermediate_size)
        w[("q_norm", l)] = np.ones(D, np.float32)
        w[("k_norm", l)] = np.ones(D, np.float32)
        w[("norm1", l)] = np.ones(H, np.float32)
        w[("norm2", l)] = np.ones(H, np.float32)
    return w


def vocab_rows(cfg: Qwen3Config, rank: int, world: int) -> tuple[int, int]:
    """[begin, end) of the vocabulary rows whose logits rank `rank` computes."""
    per = (cfg.vocab_size + world - 1) // world
    return rank * per, min(cfg.vocab_size, (rank + 1) * per)


def shard_weight(cfg: Qwen3Config, name: str, w: np.ndarray, rank: int, world: int) -> np.ndarray:
    """The slice of one weight that tensor-parallel rank `rank` of `world` holds.
    Heads (with their K/V heads) and FFN columns are split; the rows of the fused matrices are re-packed so that a
    rank's qkv is [its q heads; its k heads; its v heads] and its gate_up is [its gate rows; its up rows]."""
    if world == 1:
        return w
    D, H, KV, I = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
    hq, hk, il = H // world, KV // world, I // world
    if name == "qkv":
        q, k, v = w[: H * D], w[H * D: (H + KV) * D], w[(H + KV) * D:]
        return np.concatenate([q[rank * hq * D: (rank + 1) * hq * D], k[rank * hk * D: (rank + 1) * hk * D],
                               v[rank * hk * D: (rank + 1) * hk * D]], axis=0)
    if name == "o":      # [hidden, heads * D]: input columns follow the heads
        return np.ascontiguousarray(w[:, rank * hq * D: (rank + 1) * hq * D])
    if name == "gate_up":
        g, u = w[:I], w[I:]
        return np.concatenate([g[rank * il: (rank + 1) * il], u[rank * il: (rank + 1) * il]], axis=0)
    if name == "down":   # [hidden, inter]
        return np.ascontiguousarray(w[:, rank * il: (rank + 1) * il])
    if name == "lm_head":
        b, e = vocab_rows(cfg, rank, world)
        return w[b:e]
    return w             # embed and the norm weights are replicated


_ALLREDUCE_T = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int64, C.c_void_p)


class Qwen3ForCausalLM:
    """Device model for `batch` sequences; rank `tp_rank` of `tp_world` tensor-parallel ranks."""

    def __init__(self, cfg: Qwen3Config, batch: int = 1, tp_rank: int = 0, tp_world: int = 1, group=None,
                 connect_peers: bool = True):
        import torch
        self.torch = torch
        self.cfg, self.batch, self.tp_rank, self.tp_world, self.group = cfg, batch, tp_rank, tp_world, group
        self.L = lib()
        h = self.L.ytcuda_qwen3_create(cfg.hidden_size, cfg.num_hidden_layers, cfg.vocab_size, cfg.intermediate_size,
                                       cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                                       cfg.rms_norm_eps, cfg.rope_theta, cfg.max_position_embeddings, batch, tp_rank,
                                       tp_world)
        if not h:
            raise _lib.YtCudaInvalidArgument(_lib.INVALID_ARG, _lib.last_error())
        self.h = C.c_void_p(h)
        self._keep = []          # device tensors the handle borrows
        self.v0, self.v1 = vocab_rows(cfg, tp_rank, tp_world)
        self._cb = None
        if tp_world > 1:
            import torch.distributed as dist
            self._comm = {}

            def allreduce(buf, count, _user):
                try:
                    t = self._comm.get(buf)
                    if t is None or t.numel() < count:
                        t = self._wrap(buf, count)
                        self._comm[buf] = t
                    dist.all_reduce(t[:count], group=self.group)
                    return 0
                except Exception:  # reported to the C side as a failed collective
                    return 1

            self._cb = _ALLREDUCE_T(allreduce)
            check(self.L.ytcuda_qwen3_set_allreduce(self.h, C.cast(self._cb, C.c_void_p), None))
            if batch <= 32 and connect_peers:
                self._connect_peers()

    def _connect_peers(self) -> None:
        """Exchange the CUDA IPC handles of the ranks' exchange buffers (one all-gather) so that decode steps can run
        as one kernel per rank with the all-reduces inside it (ytcuda_qwen3_tp_export / _import)."""
        import torch.distributed as dist
        mine = (C.c_char * 64)()
        check(self.L.ytcuda_qwen3_tp_export(self.h, C.cast(mine, C.c_void_p)))
        handles = [None] * self.tp_world
        dist.all_gather_object(handles, bytes(mine.raw), group=self.group)
        for r, hb in enumerate(handles):
            buf = (C.c_char * 64).from_buffer_copy(hb)
            check(self.L.ytcuda_qwen3_tp_import(self.h, r, C.cast(buf, C.c_void_p)))
        dist.barrier(group=self.group)

    def _wrap(self, ptr: int, count: int):
        """A torch view of `count` floats of device memory owned by the model handle (for NCCL)."""
        torch = self.torch

        class _Arr:
            __cuda_array_interface__ = {"shape": (int(count),), "typestr": "<f4", "data": (int(ptr), False),
                                        "version": 2}
        return torch.as_tensor(_Arr(), device=torch.device("cuda", torch.cuda.current_device()))

    def load_weights(self, weights: dict) -> None:
        """weights: name or (name, layer) -> host array (uint16 bf16 bits for matrices, fp32 for norms), FULL size;
        sliced here for this rank and uploaded."""
        torch = self.torch
        dev = torch.device("cuda", torch.cuda.current_device())
        tied = "lm_head" not in weights
        for key, arr in weights.items():
            name, layer = (key, 0) if isinstance(key, str) else key
            part = np.ascontiguousarray(shard_weight(self.cfg, name, arr, self.tp_rank, self.tp_world))
            if part.dtype == np.uint16:
                t = torch.from_numpy(part.view(np.int16)).to(dev)
            else:
                t = torch.from_numpy(part.astype(np.float32)).to(dev)
            self._keep.append(t)
            check(self.L.ytcuda_qwen3_set_weight(self.h, name.encode(), layer, t.data_ptr()))
            if name == "embed" and tied:  # tied vocabulary matrix: this rank's rows of the embedding
                if self.tp_world == 1:
                    check(self.L.ytcuda_qwen3_set_weight(self.h, b"lm_head", 0, t.data_ptr()))
                else:
                    lt = t[self.v0:self.v1].contiguous()
                    self._keep.append(lt)
                    check(self.L.ytcuda_qwen3_set_weight(self.h, b"lm_head", 0, lt.data_ptr()))

    def reset_kv_cache(self) -> None:
        check(self.L.ytcuda_qwen3_reset(self.h))

    def set_decode_path(self, path: int) -> None:
        """0: automatic, 1: one launch per operator, 2: the single persistent kernel per decode step (or an error),
        3: as 2 with FFMA linear phases at every batch size, 4: as 3 without the shared-memory weight ring, 5: the
        ring with grid barriers (2 on one GPU with up to four sequences has neither barriers nor a cold ring), 6: as 1
        with every tensor-parallel sum through the all-reduce callback (1 exchanges the ranks' shares of inputs of
        5 to 128 rows inside its own kernels)."""
        check(self.L.ytcuda_qwen3_set_decode_path(self.h, int(path)))

    def get_kv_cache_len(self) -> int:
        return self.L.ytcuda_qwen3_cache_len(self.h)

    def decode_kernel_name(self) -> str:
        """Name of the kernel(s) an automatic-path decode step (one new token per sequence) of this model runs:
        the persistent step kernel up to 6 sequences (8 under tensor parallelism), its FFMA form below 5 sequences,
        the operator path with tcgen05 linears beyond."""
        limit = 6 if self.tp_world == 1 else 8
        if self.batch <= limit:
            if self.batch < 5:
                return ("decode_ll_kernel (no grid barriers: tagged-pair activations, weights through a shared-memory "
                        "ring, mma.sync linear phases" +
                        (")" if self.tp_world == 1 else "; partial sums pushed to the peers as pairs over NVLink)"))
            return "decode_step_kernel (mma.sync linear phases)"
        return "gemm_tc_kernel (hi + lo planes, split-k pieces) + attn_decode_fast_kernel + fused glue kernels"

    def forward(self, ids):
        """ids int32 [batch, len] on the device -> fp32 logits [batch, this rank's vocab rows] of the last position."""
        torch = self.torch
        assert ids.is_cuda and ids.dtype == torch.int32 and ids.shape[0] == self.batch and ids.is_contiguous()
        logits = torch.empty(self.batch, self.v1 - self.v0, dtype=torch.float32, device=ids.device)
        check(self.L.ytcuda_qwen3_forward(self.h, ids.data_ptr(), ids.shape[1], logits.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream))
        return logits

    def argmax(self, logits):
        """Greedy token per sequence (global over the tensor-parallel group): value / index pairs of the local
        maxima are all-gathered and the first global maximum wins, as a host argmax over the full row would."""
        from . import api
        torch = self.torch
        val, idx = api.max(logits, -1)
        idx = idx.reshape(-1) + self.v0
        if self.tp_world == 1:
            return idx.to(torch.int32), val.reshape(-1)
        import torch.distributed as dist
        vals = [torch.empty_like(val.reshape(-1)) for _ in range(self.tp_world)]
        idxs = [torch.empty_like(idx) for _ in range(self.tp_world)]
        dist.all_gather(vals, val.reshape(-1).contiguous(), group=self.group)
        dist.all_gather(idxs, idx.contiguous(), group=self.group)
        v = torch.stack(vals, 1).contiguous()          # [batch, world]; ranks hold ascending vocabulary ranges
        best, which = api.max(v, -1)
        tok = torch.stack(idxs, 1).gather(1, which.reshape(-1, 1).long()).reshape(-1)
        return tok.to(torch.int32), best.reshape(-1)

    def check_status(self) -> None:
        """Reads the device status word (synchronises the stream). A bounded wait that ran out - under tensor
        parallelism: a peer that never arrived at an exchange - raises; the KV caches are then half written and the
        group has to call recover() before the next forward."""
        st = self.L.ytcuda_device_status(self.torch.cuda.current_stream().cuda_stream)
        if st != _lib.OK:
            raise _lib.YtCudaError(st, _lib.last_error() or "a bounded device-side wait ran out")

    def recover(self) -> None:
        """After check_status raised on some rank: EVERY rank of the group calls this. Kernels are waited for,
        exchange counters and arrival words are zeroed between two barriers, the KV caches are reset."""
        self.torch.cuda.synchronize()
        if self.tp_world > 1:
            import torch.distributed as dist
            dist.barrier(group=self.group)
            check(self.L.ytcuda_qwen3_tp_resync(self.h))
            dist.barrier(group=self.group)
        else:
            self.reset_kv_cache()

    def generate_greedy(self, prompt_ids, steps: int):
        """prompt_ids int32 [batch, len] (device). Returns int32 [batch, steps] greedy tokens. The device status is
        checked once at the end, so that a step kernel that gave up on a peer raises instead of yielding tokens."""
        torch = self.torch
        out = torch.empty(self.batch, steps, dtype=torch.int32, device=prompt_ids.device)
        logits = self.forward(prompt_ids)
        for s in range(steps):
            tok, _ = self.argmax(logits)
            out[:, s] = tok
            if s + 1 < steps:
                logits = self.forward(tok.reshape(self.batch, 1).contiguous())
        self.check_status()
        return out

    def generate_topk(self, prompt_ids, steps: int, k: int = 20, seed: int = 42):
        """Sampled generation as Qwen3ForCausalLM::generate does it (reference qwen3.cpp:459-516): after every
        forward the next token is drawn among the k most probable ones. The uniform numbers come from a host
        generator (numpy's MT19937 seeded with `seed`; the reference's std::uniform_real_distribution consumes its
        std::mt19937 differently, so the streams are not the same). Single GPU. Returns int32 [batch, steps]."""
        from . import api
        torch = self.torch
        assert self.tp_world == 1, "sampling needs the whole vocabulary on one GPU"
        rng = np.random.Generator(np.random.MT19937(seed))
        out = torch.empty(self.batch, steps, dtype=torch.int32, device=prompt_ids.device)
        logits = self.forward(prompt_ids)
        for s in range(steps):
            u = torch.from_numpy(rng.random(self.batch, dtype=np.float32)).to(prompt_ids.device)
            _, _, tok = api.topk_sample(logits, k, u)
            out[:, s] = tok
            if s + 1 < steps:
                logits = self.forward(tok.reshape(self.batch, 1).contiguous())
        return out

    def close(self):
        """Destroys the model. Under tensor parallelism every rank must call it (it runs a barrier over the group
        between closing the peers' exchange buffers and freeing its own, as CUDA IPC requires)."""
        if self.h:
            if self.tp_world > 1:
                self.L.ytcuda_qwen3_tp_disconnect(self.h)
                try:
                    import torch.distributed as dist
                    if dist.is_initialized():
                        dist.barrier(group=self.group)
                except Exception:  # the group is already gone (interpreter exit): nothing left to wait for
                    pass
            self.L.ytcuda_qwen3_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
