"""Test support (not part of the product; a grad.cpp build reads token files with its own classes).
Pre-tokenized corpus files, the input of `grad eval`: "TOK1", uint32 vocab size, uint64 id count,
then the ids as uint16 (reference: src/data/token_file.cpp:14-16 header, :33-70 writer, :83-176
reader and windows). Error messages are the reference's."""
from __future__ import annotations

import struct
from pathlib import Path

import numpy as np

MAGIC = b"TOK1"
HEADER_BYTES = 16


def write(path, ids, vocab_size: int) -> None:
    if vocab_size <= 0 or vocab_size > 65536:
        raise ValueError("token file requires 0 < vocab_size <= 65536 (uint16 storage)")
    a = np.ascontiguousarray(ids, np.int64)
    if a.size and (a.min() < 0 or a.max() >= vocab_size):
        raise RuntimeError(f"token id out of range for vocab while writing {path}")
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<IQ", vocab_size, a.size))
        f.write(a.astype("<u2").tobytes())


class MappedTokenDataset:
    """Windows of seq_length ids every `stride` ids; the target is the input shifted by one.
    `grad eval` uses stride = seq_length (src/cli/eval.cpp:78-79)."""

    def __init__(self, path, seq_length: int, stride: int = 1):
        if stride < 1:
            raise ValueError("stride must be >= 1")
        if seq_length < 1:
            raise ValueError("seq_length must be >= 1")
        path = str(path)
        if not Path(path).is_file():
            raise RuntimeError(f"Cannot open token file: {path}")
        raw = np.memmap(path, dtype=np.uint8, mode="r") if Path(path).stat().st_size else np.zeros(0, np.uint8)
        if raw.size < HEADER_BYTES:
            raise RuntimeError(f"Token file truncated or unreadable: {path}")
        if bytes(raw[:4]) != MAGIC:
            raise RuntimeError(f"Not a token file (bad magic): {path}")
        vocab, count = struct.unpack("<IQ", bytes(raw[4:16]))
        if vocab == 0 or vocab > 65536:
            raise RuntimeError(f"Token file vocab {vocab} outside (0, 65536]: {path}")
        if count > (raw.size - HEADER_BYTES) // 2:
            raise RuntimeError(f"Token file shorter than its header claims: {path}")
        if count < seq_length + 1:
            raise RuntimeError(f"Not enough tokens for even one sequence: {path}")
        self.vocab_size, self.token_count = int(vocab), int(count)
        self.seq_length, self.stride = seq_length, stride
        self.tokens = np.frombuffer(raw, dtype="<u2", count=self.token_count, offset=HEADER_BYTES)

    def __len__(self) -> int:
        return (self.token_count - self.seq_length - 1) // self.stride + 1

    def get_item(self, index: int):
        if index < 0 or index >= len(self):
            raise IndexError("MappedTokenDataset index out of range")
        start = index * self.stride
        w = self.tokens[start:start + self.seq_length + 1].astype(np.int32)
        bad = np.nonzero(w >= self.vocab_size)[0]
        if bad.size:
            i = int(bad[0])
            raise RuntimeError(f"token id {int(w[i])} at offset {start + i} is outside the file's vocab of "
                               f"{self.vocab_size}")
        return w[:-1], w[1:]

    def windows(self, first: int = 0, count: int | None = None):
        """(inputs, targets) of `count` consecutive windows, in file order."""
        n = len(self) - first if count is None else min(count, len(self) - first)
        items = [self.get_item(first + i) for i in range(max(n, 0))]
        if not items:
            z = np.zeros((0, self.seq_length), np.int32)
            return z, z.copy()
        return np.stack([a for a, _ in items]), np.stack([b for _, b in items])
