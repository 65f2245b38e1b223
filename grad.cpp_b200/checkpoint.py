"""Host-side tools for the ``GPTM`` checkpoint file that grad.cpp models live in.

The product reads and writes this format in C++ (csrc/checkpoint.cpp); this
module is the numpy counterpart used to MAKE synthetic checkpoints for tests
and benchmarks, since no trained weights are available offline.

Format (reference: src/transformer/gpt_model.cpp:292-381 for the writer,
:383-525 for the reader): u32 magic 0x4750544D, u32 version (1 or 2), u32 arch
(version 2 only; 0 GPT-2, 1 Modern), i32 vocab, d_model, layers, heads,
max_len, f32 dropout, then tensors as (i32 rows, i32 cols, rows*cols f32
row-major) in a fixed order, then optional trailer sections
(tag[4], u32 length, payload).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np

MAGIC = 0x4750544D
GPT2, MODERN = 0, 1


@dataclass(frozen=True)
class ModelDims:
    vocab: int
    d_model: int
    layers: int
    heads: int
    max_len: int
    arch: int  # 0 GPT-2, 1 Modern

    @property
    def d_ff(self) -> int:
        # include/grad/transformer/feedforward.h:24-28
        if self.arch == MODERN:
            return ((8 * self.d_model // 3) + 63) // 64 * 64
        return 4 * self.d_model

    @property
    def head_dim(self) -> int:
        return self.d_model // self.heads


# The configurations the benchmark and parity tests use.
PRESETS = {
    "small": ModelDims(5000, 512, 6, 8, 1024, GPT2),
    "modern": ModelDims(16000, 768, 8, 12, 256, MODERN),
    "modern2k": ModelDims(16000, 768, 8, 12, 2048, MODERN),
    "medium": ModelDims(16000, 768, 8, 12, 1024, GPT2),
}


def tensor_shapes(dm: ModelDims):
    """(name, rows, cols) for every tensor in file order."""
    d, f = dm.d_model, dm.d_ff
    out = [("token_embedding", dm.vocab, d)]
    if dm.arch == GPT2:
        out.append(("position_embedding", dm.max_len, d))
    for l in range(dm.layers):
        p = f"layer{l}."
        out += [(p + "W_q", d, d), (p + "W_k", d, d), (p + "W_v", d, d), (p + "W_o", d, d),
                (p + "b_q", 1, d), (p + "b_k", 1, d), (p + "b_v", 1, d), (p + "b_o", 1, d)]
        if dm.arch == MODERN:
            out += [(p + "ffn_gate", d, f), (p + "ffn_up", d, f), (p + "ffn_down", f, d)]
        else:
            out += [(p + "ffn_W1", d, f), (p + "ffn_b1", 1, f), (p + "ffn_W2", f, d), (p + "ffn_b2", 1, d)]
        out += [(p + "norm1_gamma", 1, d), (p + "norm1_beta", 1, d),
                (p + "norm2_gamma", 1, d), (p + "norm2_beta", 1, d)]
    out += [("final_norm_gamma", 1, d), ("final_norm_beta", 1, d)]
    return out


def synthetic_tensors(dm: ModelDims, seed: int, std: float = 0.02, perturb_vectors: bool = False):
    """Random-init weights: N(0, std) for every matrix, zero biases/betas, unit gains.

    ``perturb_vectors`` instead draws biases and betas from N(0, std) and gains
    from 1 + N(0, std), so that parity tests exercise those terms too."""
    rng = np.random.default_rng(seed)
    tensors = []
    for name, r, c in tensor_shapes(dm):
        if r > 1:
            t = rng.standard_normal((r, c), dtype=np.float32) * np.float32(std)
        elif name.endswith("gamma"):
            t = np.ones((r, c), np.float32)
            if perturb_vectors:
                t += rng.standard_normal((r, c), dtype=np.float32) * np.float32(std)
        else:
            t = np.zeros((r, c), np.float32)
            if perturb_vectors:
                t += rng.standard_normal((r, c), dtype=np.float32) * np.float32(std)
        tensors.append(t)
    return tensors


def write_checkpoint(path, dm: ModelDims, tensors, dropout: float = 0.0, version: int = 2,
                     fingerprint=None, extra_trailers=()):
    shapes = tensor_shapes(dm)
    assert len(tensors) == len(shapes)
    with open(path, "wb") as f:
        f.write(struct.pack("<II", MAGIC, version))
        if version == 2:
            f.write(struct.pack("<I", dm.arch))
        else:
            assert dm.arch == GPT2, "version 1 files are GPT-2 only"
        f.write(struct.pack("<iiiiif", dm.vocab, dm.d_model, dm.layers, dm.heads, dm.max_len, dropout))
        for (name, r, c), t in zip(shapes, tensors):
            t = np.ascontiguousarray(t, dtype="<f4")
            assert t.shape == (r, c), (name, t.shape, (r, c))
            f.write(struct.pack("<ii", r, c))
            f.write(t.tobytes())
        for tag, payload in extra_trailers:
            f.write(tag + struct.pack("<I", len(payload)) + payload)
        if fingerprint is not None:
            kind, h = fingerprint
            f.write(b"TKFP" + struct.pack("<IIQ", 12, kind, h))


def write_synthetic(path, dm: ModelDims, seed: int, std: float = 0.02, perturb_vectors: bool = False):
    write_checkpoint(path, dm, synthetic_tensors(dm, seed, std, perturb_vectors))
    return path


def read_checkpoint(path):
    """Returns (ModelDims, [tensors], fingerprint-or-None). Minimal checks; the
    checked reader is the C++ one."""
    with open(path, "rb") as f:
        buf = f.read()
    magic, version = struct.unpack_from("<II", buf, 0)
    assert magic == MAGIC
    off = 8
    arch = GPT2
    if version == 2:
        (arch,) = struct.unpack_from("<I", buf, off)
        off += 4
    vocab, d, layers, heads, max_len, _ = struct.unpack_from("<iiiiif", buf, off)
    off += 24
    dm = ModelDims(vocab, d, layers, heads, max_len, arch)
    tensors = []
    for _, r, c in tensor_shapes(dm):
        fr, fc = struct.unpack_from("<ii", buf, off)
        assert (fr, fc) == (r, c)
        off += 8
        tensors.append(np.frombuffer(buf, "<f4", r * c, off).reshape(r, c).copy())
        off += 4 * r * c
    fp = None
    while off < len(buf):
        tag = buf[off:off + 4]
        (ln,) = struct.unpack_from("<I", buf, off + 4)
        off += 8
        if tag == b"TKFP":
            fp = struct.unpack_from("<IQ", buf, off)
        off += ln
    return dm, tensors, fp
