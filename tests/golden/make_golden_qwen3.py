"""Generates tests/golden/golden_qwen3.npz by running the UNMODIFIED reference example model
(example/qwen3, compiled behind oracle/ref_shim.cpp) on seeded random weights.

    make -C oracle ref REF=<YTensor source tree> && python tests/golden/make_golden_qwen3.py

Two cases:
  small_* : a 2-layer toy configuration; full logits of the prefill and of 5 greedy steps, batch 1 and 2.
  full_*  : the Qwen3-0.6B shape of benchmark configuration 5 (28 layers, hidden 1024, 16 q / 8 kv heads, head_dim 128,
            FFN 3072, vocab 151936, bf16 weights ~ N(0, 0.02) from seed 4, norm weights 1, tied vocabulary matrix),
            prompt = 512 token ids uniform in [0, vocab) from seed 4, 32 greedy steps: the tokens, the margin
            between the best and second-best logit at every step, and the 8 largest logits with their indices.
Weights are re-created from the seed by ytensor_b200.qwen3.random_weights; a checksum of the embedding guards
against a generator that changed.
"""
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

OUT = Path(__file__).resolve().parent / "golden_qwen3.npz"
SMALL = dict(hidden_size=64, num_hidden_layers=2, vocab_size=512, intermediate_size=96, num_attention_heads=4,
             num_key_value_heads=2, head_dim=128, max_position_embeddings=64)


def load(model, weights):
    for key, arr in weights.items():
        name, layer = (key, 0) if isinstance(key, str) else key
        model.set_weight(name, layer, bf16_bits_to_f32(arr) if arr.dtype == np.uint16 else arr)


def main():
    R = O.ref(threads=0)
    g = {}
    cfg = Qwen3Config(**SMALL)
    w = random_weights(cfg, seed=4, std=0.05)
    g["small_embed_sha256"] = np.array(hashlib.sha256(w["embed"].tobytes()).hexdigest())
    for B in (1, 2):
        m = R.qwen3(cfg.oracle_dict(), B)
        load(m, w)
        ids = np.random.default_rng(10 + B).integers(0, cfg.vocab_size, (B, 9)).astype(np.int32)
        logits = [m.forward(ids)]
        for _ in range(5):
            logits.append(m.forward(logits[-1].argmax(1).astype(np.int32).reshape(B, 1)))
        g[f"small_ids_b{B}"] = ids
        g[f"small_logits_b{B}"] = np.stack(logits)  # [6, B, vocab]
        m.close()

    cfg = Qwen3Config(max_position_embeddings=768)
    t0 = time.time()
    w = random_weights(cfg, seed=4)
    print(f"weights in {time.time() - t0:.1f}s")
    g["full_embed_sha256"] = np.array(hashlib.sha256(w["embed"].tobytes()).hexdigest())
    m = R.qwen3(cfg.oracle_dict(), 1)
    load(m, w)
    prompt = np.random.default_rng(4).integers(0, cfg.vocab_size, (1, 512)).astype(np.int32)
    t0 = time.time()
    logits = m.forward(prompt)
    print(f"prefill in {time.time() - t0:.1f}s")
    toks, margins, top_v, top_i = [], [], [], []
    t0 = time.time()
    for s in range(32):
        order = np.argsort(-logits[0])[:8]
        toks.append(order[0])
        margins.append(logits[0, order[0]] - logits[0, order[1]])
        top_v.append(logits[0, order])
        top_i.append(order)
        if s < 31:
            logits = m.forward(np.array([[order[0]]], np.int32))
    print(f"32 decode steps in {time.time() - t0:.1f}s; min margin {min(margins):.3e}")
    g["full_prompt"] = prompt
    g["full_tokens"] = np.array(toks, np.int32)
    g["full_margins"] = np.array(margins, np.float32)
    g["full_top8_values"] = np.array(top_v, np.float32)
    g["full_top8_indices"] = np.array(top_i, np.int32)
    np.savez_compressed(OUT, **g)
    print(f"wrote {OUT} ({OUT.stat().st_size / 1024:.0f} KiB)")


if __name__ == "__main__":
    main()
