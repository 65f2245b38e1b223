"""Generates tests/golden/*.npz and tests/golden/ref_tiny_*.bin from the
reference itself (oracle/_ref, the unmodified grad.cpp decode path).

Run from the repository root where the reference sources are available:

    make -C oracle ref && python tests/golden/make_golden.py

The fixtures pin the CPU restatement (oracle/decode_oracle.c) and, through it,
the CUDA path. Inputs are regenerated from seeds by the tests; each fixture
stores a CRC of those inputs so a drift in the generator is caught rather than
silently compared against.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import zlib
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
os.environ["GRADREF_SEED"] = "20250101"

from oracle.oracle import Ref  # noqa: E402

spec = importlib.util.spec_from_file_location("gradb_checkpoint", ROOT / "grad.cpp_b200" / "checkpoint.py")
ck = importlib.util.module_from_spec(spec)
sys.modules["gradb_checkpoint"] = ck
spec.loader.exec_module(ck)

OUT = Path(__file__).resolve().parent

# name -> (dims, weight seed, std, perturb biases/gains)
MODEL_CASES = {
    "tiny_gpt2": (ck.ModelDims(23, 32, 2, 4, 16, ck.GPT2), 101, 0.3, True),
    "tiny_modern": (ck.ModelDims(23, 32, 2, 4, 16, ck.MODERN), 102, 0.3, True),
    "hs64_gpt2": (ck.ModelDims(301, 128, 2, 2, 40, ck.GPT2), 103, 0.08, True),
    "hs64_modern": (ck.ModelDims(301, 128, 3, 2, 40, ck.MODERN), 104, 0.08, True),
    # d_model 192 = 3 heads of 64; vocab not a multiple of any tile size.
    "odd_modern": (ck.ModelDims(1003, 192, 2, 3, 24, ck.MODERN), 105, 0.05, False),
}


def crc(a: np.ndarray) -> int:
    return zlib.crc32(np.ascontiguousarray(a).tobytes())


def sampler_logits(seed: int, vocab: int, scale: float, quantum: float) -> np.ndarray:
    """Seeded logits; quantum > 0 snaps them to a grid so that exact ties occur."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(vocab, dtype=np.float32) * np.float32(scale)
    if quantum > 0:
        x = (np.round(x / np.float32(quantum)) * np.float32(quantum)).astype(np.float32)
    return x


# (seed, vocab, scale, quantum, temperature, top_k, top_p)
SAMPLER_CASES = [
    (1, 16000, 0.55, 0.0, 0.8, 40, 0.9),
    (2, 16000, 0.55, 0.0, 0.8, 0, 0.9),
    (3, 16000, 0.55, 0.0, 1.0, 0, 1.0),
    (4, 16000, 0.55, 0.0, 0.8, 40, 1.0),
    (5, 16000, 2.5, 0.0, 0.5, 0, 0.5),
    (6, 16000, 0.55, 0.25, 0.8, 40, 0.9),      # ties at the top-k and top-p thresholds
    (7, 16000, 0.55, 0.0, 0.8, 1, 1.0),        # --greedy in chat = top-k 1 through the sampler
    (8, 16000, 0.55, 0.0, 0.8, 16000, 0.9),    # top_k == vocab disables the filter
    (9, 16000, 0.55, 0.0, 1.0, 0, 0.99999994), # a threshold the running sum may never reach
    (10, 16000, 0.55, 0.0, 1.3, 0, 0.0),       # p = 0 keeps the maximum only
    (11, 5000, 0.7, 0.0, 0.8, 0, 1.0),
    (12, 5000, 0.7, 0.5, 0.9, 7, 0.8),
    (13, 23, 1.5, 0.0, 0.8, 5, 0.9),
    (14, 23, 1.5, 1.0, 1.0, 3, 0.7),
    (15, 1003, 30.0, 0.0, 0.8, 0, 0.9),        # very peaked: -1e10 sentinel and exp underflow
    (16, 16000, 0.55, 0.0, 0.8, 40, 0.9),
    (17, 16000, 0.55, 0.0, 0.8, 0, 0.9),
    (18, 16000, 0.55, 0.0, 0.8, 0, 0.9),
]


def main() -> None:
    R = Ref()
    store: dict[str, np.ndarray] = {}

    for name, (dm, seed, std, perturb) in MODEL_CASES.items():
        path = f"/tmp/gradb_golden_{name}.bin"
        ck.write_synthetic(path, dm, seed, std, perturb)
        store[f"{name}/file_crc"] = np.array([zlib.crc32(open(path, "rb").read())], np.uint32)
        m = R.load(path)
        rng = np.random.default_rng(seed + 1000)
        toks = rng.integers(0, dm.vocab, dm.max_len).astype(np.int32)
        store[f"{name}/tokens"] = toks
        store[f"{name}/logits"] = R.logits_for(m, toks)
        prompt = toks[: max(2, dm.max_len // 4)]
        n_new = dm.max_len  # more than fits: exercises the stop at capacity
        store[f"{name}/prompt"] = prompt
        store[f"{name}/greedy_p1.0"] = R.generate_greedy(m, prompt, n_new, 1.0)
        store[f"{name}/greedy_p1.2"] = R.generate_greedy(m, prompt, n_new, 1.2)
        store[f"{name}/greedy_short"] = R.generate_greedy(m, prompt, 3, 1.2)
        for tag, (t, pen, k, p) in {"a": (0.8, 1.1, 40, 0.9), "b": (1.0, 1.2, 0, 1.0),
                                    "c": (0.7, 1.0, 5, 0.6)}.items():
            ids, draws = R.generate_sample(m, prompt, t, n_new, pen, k, p)
            store[f"{name}/sample_{tag}_ids"] = ids
            store[f"{name}/sample_{tag}_draws"] = draws
            store[f"{name}/sample_{tag}_params"] = np.array([t, pen, k, p], np.float64)
        ids, draws = R.generate_sample(m, prompt, 0.9, 6, 1.2, 0, 0.95, stream=True)
        store[f"{name}/stream_ids"] = ids
        store[f"{name}/stream_draws"] = draws
        # error behaviour: token out of range -> 2 (std::out_of_range), context full -> 1.
        s = R.session(m)
        rc_bad = R.step(s, dm.vocab, dm.vocab, want=False)[0]
        rc_neg = R.step(s, -1, dm.vocab, want=False)[0]
        for t in toks:
            assert R.step(s, int(t), dm.vocab, want=False)[0] == 0
        rc_full = R.step(s, 0, dm.vocab, want=False)[0]
        R.session_free(s)
        store[f"{name}/error_codes"] = np.array([rc_bad, rc_neg, rc_full], np.int32)
        R.free(m)

    any_model = R.new(23, 32, 1, 4, 16, 0)
    rows = []
    for case in SAMPLER_CASES:
        seed, vocab, scale, quantum, t, k, p = case
        lg = sampler_logits(seed, vocab, scale, quantum)
        # Several draws per case pin the filtered distribution's CDF at several points.
        for _ in range(24):
            tok, u = R.sample_from_logits(any_model, lg, t, k, p)
            rows.append([seed, vocab, scale, quantum, t, k, p, u, tok, crc(lg)])
    store["sampler/cases"] = np.array(rows, np.float64)

    # Checkpoints written by the reference's own save(): byte-for-byte fixtures
    # for the reader/writer. Tiny shapes keep them to a few KB.
    for arch, label in ((0, "gpt2"), (1, "modern")):
        m = R.new(11, 8, 1, 2, 4, arch)
        assert R.save(m, OUT / f"ref_tiny_{label}.bin") == 0
        assert R.save(m, OUT / f"ref_tiny_{label}_fp.bin", fingerprint=(2, 0x1122334455667788)) == 0
        R.free(m)

    np.savez_compressed(OUT / "decode_golden.npz", **store)
    print("wrote", OUT / "decode_golden.npz", os.path.getsize(OUT / "decode_golden.npz"), "bytes")


if __name__ == "__main__":
    main()
