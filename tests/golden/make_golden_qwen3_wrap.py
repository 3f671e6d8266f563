"""Generates tests/golden/golden_qwen3_wrap.npz: the reference decoder (unmodified, behind oracle/ref_shim.cpp) run
past the end of its KV cache, which is a ring buffer (example/qwen3/src/qwen3.cpp:70-126): a 9-token prompt and 19
single-token steps with max_position_embeddings = 16, so the cache fills at step 7 and the later steps overwrite the
oldest slots; and a second run that feeds SEVERAL tokens per call across the end of the ring (two sequences).
Run from the repository root: make -C oracle ref REF=<YTensor source tree> && python tests/golden/make_golden_qwen3_wrap.py
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))
from make_golden_qwen3 import SMALL, load  # noqa: E402
from oracle import oracle as O  # noqa: E402
from ytensor_b200.qwen3 import Qwen3Config, random_weights  # noqa: E402

OUT = Path(__file__).resolve().parent / "golden_qwen3_wrap.npz"


def main():
    R = O.ref(threads=0)
    cfg = Qwen3Config(**{**SMALL, "max_position_embeddings": 16})
    w = random_weights(cfg, seed=4, std=0.05)
    m = R.qwen3(cfg.oracle_dict(), 1)
    load(m, w)
    ids = np.random.default_rng(21).integers(0, cfg.vocab_size, (1, 9)).astype(np.int32)
    logits = [m.forward(ids)]
    for _ in range(19):
        logits.append(m.forward(logits[-1].argmax(1).astype(np.int32).reshape(1, 1)))
    m.close()
    # several tokens per call across the end of the ring: 9 + 5 (fits), + 6 (runs over the end), + 3 (already full),
    # + 1, + 10 (more than half the ring), for two sequences
    m = R.qwen3(cfg.oracle_dict(), 2)
    load(m, w)
    rng = np.random.default_rng(22)
    chunks = [rng.integers(0, cfg.vocab_size, (2, n)).astype(np.int32) for n in (9, 5, 6, 3, 1, 10)]
    multi = [m.forward(c) for c in chunks]
    m.close()
    extra = {f"multi_ids_{i}": c for i, c in enumerate(chunks)}
    np.savez_compressed(OUT, wrap_ids=ids, wrap_logits=np.stack(logits), multi_logits=np.stack(multi), **extra)
    print(f"wrote {OUT} ({OUT.stat().st_size / 1024:.0f} KiB)")


if __name__ == "__main__":
    main()
