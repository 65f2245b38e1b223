"""Generates tests/golden/ref_tokens.bin (a token file written by the reference's own
tokenfile::write) and tests/golden/tokenfile_golden.npz (what the reference's MappedTokenDataset
and DataLoader make of it, and the messages it raises on damaged copies).

    make -C oracle ref && python tests/golden/make_tokenfile_golden.py
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent))
from make_golden import MODEL_CASES, Ref, ck  # noqa: E402

OUT = Path(__file__).resolve().parent
VOCAB = 23          # the tiny golden models' vocabulary
N_IDS = 203
EVAL_SEED = 20260921  # src/cli/eval.cpp:86


def main() -> None:
    R = Ref()
    ids = np.random.default_rng(4242).integers(0, VOCAB, N_IDS).astype(np.int32)
    path = OUT / "ref_tokens.bin"
    R.tokenfile_write(path, ids, VOCAB)
    store = {"ids": ids}
    for seq, stride in ((5, 5), (12, 12), (7, 1), (16, 16)):
        store[f"open_{seq}_{stride}"] = np.array(R.dataset_open(path, seq, stride), np.int64)
    # `grad eval`: sequential when everything is scored, random windows when capped (eval.cpp:87-92)
    for tag, (seq, batch, shuffle, seed, cap) in {
        "seq": (5, 3, False, EVAL_SEED, 0),
        "capped": (5, 3, True, EVAL_SEED, 2),
        "train": (12, 8, True, EVAL_SEED + 1, 2),
        "ragged": (12, 8, False, EVAL_SEED, 0),
    }.items():
        inp, tgt = R.loader_windows(path, seq, seq, batch, shuffle, seed, cap)
        store[f"{tag}/inputs"], store[f"{tag}/targets"] = inp, tgt
        store[f"{tag}/params"] = np.array([seq, batch, int(shuffle), seed, cap], np.int64)
    # the loss `grad eval` would print for the tiny golden models over those loaders
    for name in ("tiny_gpt2", "tiny_modern"):
        dm, seed, std, perturb = MODEL_CASES[name]
        mpath = f"/tmp/gradb_golden_{name}.bin"
        ck.write_synthetic(mpath, dm, seed, std, perturb)
        m = R.load(mpath)
        for tag in ("seq", "capped", "train", "ragged"):
            batch = int(store[f"{tag}/params"][1])
            mean, _, _ = R.mean_loss(m, store[f"{tag}/inputs"], store[f"{tag}/targets"], batch)
            store[f"{name}/{tag}/mean"] = np.array([mean], np.float64)
        R.free(m)
    # damaged copies -> the reference's messages (the path is replaced by {path})
    raw = path.read_bytes()
    cases = {
        "missing": None,
        "short_header": raw[:10],
        "bad_magic": b"TOK2" + raw[4:],
        "zero_vocab": raw[:4] + (0).to_bytes(4, "little") + raw[8:],
        "big_vocab": raw[:4] + (65537).to_bytes(4, "little") + raw[8:],
        "count_lies": raw[:8] + (N_IDS + 1).to_bytes(8, "little") + raw[16:],
        "too_few": raw[:8] + (4).to_bytes(8, "little") + raw[16:],
    }
    msgs = []
    for tag, blob in cases.items():
        p = Path("/tmp/gradb_tok_case.bin")
        if p.exists():
            p.unlink()
        if blob is not None:
            p.write_bytes(blob)
        try:
            R.dataset_open(p, 5, 5)
            msgs.append(f"{tag}\tOK")
        except RuntimeError as e:
            msgs.append(f"{tag}\t" + str(e).replace(str(p), "{path}"))
    store["messages"] = np.array(msgs)
    # an id beyond the header's vocabulary is reported when its window is read (token_file.cpp:163-170)
    blob = bytearray(raw[:4] + (20).to_bytes(4, "little") + raw[8:])
    p = Path("/tmp/gradb_tok_case.bin")
    p.write_bytes(bytes(blob))
    try:
        R.loader_windows(p, 5, 5, 3, False, 1, 0)
        store["id_message"] = np.array(["OK"])
    except RuntimeError as e:
        store["id_message"] = np.array([str(e)])
    p.unlink()
    np.savez_compressed(OUT / "tokenfile_golden.npz", **store)
    for k in ("messages", "id_message"):
        print(store[k])
    print({k: v for k, v in store.items() if k.endswith("/mean") or k.startswith("open_")})


if __name__ == "__main__":
    main()
