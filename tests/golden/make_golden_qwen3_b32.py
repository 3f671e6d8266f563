"""Generates tests/golden/golden_qwen3_b32.npz: the UNMODIFIED reference example model (example/qwen3, compiled behind
oracle/ref_shim.cpp) at the Qwen3-0.6B shape with 32 sequences at once.

    make -C oracle ref REF=<YTensor source tree> && python tests/golden/make_golden_qwen3_b32.py      (about five minutes on 8 cores)

32 distinct prompts of 16 token ids (uniform in [0, vocab), seed 32), 32 greedy steps; per step and sequence the token,
the margin between the best and second-best logit, and the 4 largest logits with their indices. The prompt is short
because the reference's prefill of 32 x 512 tokens would take most of an hour on the CPU; the decode steps, which are
what the 32-sequence device path differs in, are the full 32. The KV caches are re-initialised for 32 sequences as the
shim does (the example hard-codes one sequence, example/qwen3/src/qwen3.cpp:415-423)."""
from __future__ import annotations

import hashlib
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle as O  # noqa: E402
from ytensor_b200.qwen3 import Qwen3Config, bf16_bits_to_f32, random_weights  # noqa: E402

OUT = Path(__file__).resolve().parent / "golden_qwen3_b32.npz"
B, PROMPT, STEPS = 32, 16, 32


def main():
    R = O.ref(threads=0)
    cfg = Qwen3Config(max_position_embeddings=64)
    w = random_weights(cfg, seed=4)
    g = {"embed_sha256": np.array(hashlib.sha256(w["embed"].tobytes()).hexdigest())}
    m = R.qwen3(cfg.oracle_dict(), B)
    for key, arr in w.items():
        name, layer = (key, 0) if isinstance(key, str) else key
        m.set_weight(name, layer, bf16_bits_to_f32(arr) if arr.dtype == np.uint16 else arr)
    prompt = np.random.default_rng(32).integers(0, cfg.vocab_size, (B, PROMPT)).astype(np.int32)
    t0 = time.time()
    logits = m.forward(prompt)
    print(f"prefill in {time.time() - t0:.1f}s", flush=True)
    toks, margins, top_v, top_i = [], [], [], []
    t0 = time.time()
    for s in range(STEPS):
        order = np.argsort(-logits, axis=1, kind="stable")[:, :4]
        vals = np.take_along_axis(logits, order, axis=1)
        toks.append(order[:, 0].copy())
        margins.append(vals[:, 0] - vals[:, 1])
        top_v.append(vals)
        top_i.append(order)
        if s + 1 < STEPS:
            logits = m.forward(order[:, :1].astype(np.int32))
    print(f"{STEPS} decode steps in {time.time() - t0:.1f}s; min margin {np.min(margins):.3e}", flush=True)
    g["prompt"] = prompt
    g["tokens"] = np.stack(toks, 1).astype(np.int32)            # [B, STEPS]
    g["margins"] = np.stack(margins, 1).astype(np.float32)      # [B, STEPS]
    g["top4_values"] = np.stack(top_v, 1).astype(np.float32)    # [B, STEPS, 4]
    g["top4_indices"] = np.stack(top_i, 1).astype(np.int32)
    np.savez_compressed(OUT, **g)
    print(f"wrote {OUT} ({OUT.stat().st_size / 1024:.0f} KiB)")


if __name__ == "__main__":
    main()
