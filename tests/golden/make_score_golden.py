"""Generates tests/golden/score_golden.npz: teacher-forced scoring (`grad eval`'s mean loss)
computed by the reference itself (oracle/_ref: its full-sequence forward, log_softmax and
cross_entropy operators, batched as src/training/trainer.cpp:319-340 does).

Run from the repository root where the reference sources are available:

    make -C oracle ref && python tests/golden/make_score_golden.py

Models are the seeded checkpoints of make_golden.py; windows are cut from one seeded id stream
with stride = window length, target = input shifted by one (src/data/token_file.cpp:153-176).
"""
from __future__ import annotations

import sys
import zlib
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent))
from make_golden import MODEL_CASES, ROOT, Ref, ck  # noqa: E402

OUT = Path(__file__).resolve().parent

# name -> (windows, window length, windows per batch); 5 windows in batches of 2 leave a ragged last batch
SCORE_CASES = {
    "tiny_gpt2": (5, 12, 2),
    "tiny_modern": (5, 16, 2),
    "hs64_gpt2": (6, 40, 8),
    "hs64_modern": (5, 33, 2),
    "odd_modern": (3, 24, 1),
}


def windows(seed: int, vocab: int, n: int, S: int):
    stream = np.random.default_rng(seed).integers(0, vocab, n * S + 1).astype(np.int32)
    inp = np.stack([stream[i * S:i * S + S] for i in range(n)])
    tgt = np.stack([stream[i * S + 1:i * S + S + 1] for i in range(n)])
    return inp, tgt


def main() -> None:
    R = Ref()
    store = {}
    for name, (n, S, bw) in SCORE_CASES.items():
        dm, seed, std, perturb = MODEL_CASES[name]
        path = f"/tmp/gradb_golden_{name}.bin"
        ck.write_synthetic(path, dm, seed, std, perturb)
        m = R.load(path)
        inp, tgt = windows(seed + 2000, dm.vocab, n, S)
        if name == "tiny_modern":
            tgt[1, 3] = dm.vocab  # an id outside the vocabulary contributes nothing (variable.cpp:547-552)
            tgt[4, 0] = -1
        mean, batch, logp = R.mean_loss(m, inp, tgt, bw)
        store[f"{name}/inputs"] = inp
        store[f"{name}/targets"] = tgt
        store[f"{name}/batch_windows"] = np.array([bw], np.int32)
        store[f"{name}/mean"] = np.array([mean], np.float64)
        store[f"{name}/batch_loss"] = batch
        store[f"{name}/row_logp"] = logp
        store[f"{name}/file_crc"] = np.array([zlib.crc32(open(path, "rb").read())], np.uint32)
        print(name, mean, batch)
        R.free(m)
    np.savez_compressed(OUT / "score_golden.npz", **store)
    print("wrote", OUT / "score_golden.npz")


if __name__ == "__main__":
    main()
