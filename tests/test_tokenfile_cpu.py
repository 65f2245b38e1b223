"""Token files, windows and batch order (the data path of `grad eval`) against fixtures produced by
the reference's own tokenfile::write, MappedTokenDataset and DataLoader
(tests/golden/ref_tokens.bin, tests/golden/tokenfile_golden.npz). No GPU."""
import subprocess

import numpy as np
import pytest

from conftest import ROOT

GOLD = ROOT / "tests" / "golden"


@pytest.fixture(scope="module")
def tg():
    return np.load(GOLD / "tokenfile_golden.npz")


@pytest.fixture(scope="module")
def tokenfile(pkg):
    from support import tokenfile as tf
    return tf


def damaged_copies(tmp_path):
    raw = (GOLD / "ref_tokens.bin").read_bytes()
    n = int.from_bytes(raw[8:16], "little")
    blobs = {
        "missing": None,
        "short_header": raw[:10],
        "bad_magic": b"TOK2" + raw[4:],
        "zero_vocab": raw[:4] + (0).to_bytes(4, "little") + raw[8:],
        "big_vocab": raw[:4] + (65537).to_bytes(4, "little") + raw[8:],
        "count_lies": raw[:8] + (n + 1).to_bytes(8, "little") + raw[16:],
        "too_few": raw[:8] + (4).to_bytes(8, "little") + raw[16:],
    }
    out = {}
    for tag, blob in blobs.items():
        p = tmp_path / f"{tag}.bin"
        if blob is not None:
            p.write_bytes(blob)
        out[tag] = p
    return out


def test_python_writer_is_byte_identical_and_reader_matches(tokenfile, tg, tmp_path):
    p = tmp_path / "mine.bin"
    tokenfile.write(p, tg["ids"], 23)
    assert p.read_bytes() == (GOLD / "ref_tokens.bin").read_bytes()
    for key in ("open_5_5", "open_12_12", "open_7_1", "open_16_16"):
        _, seq, stride = key.split("_")
        ds = tokenfile.MappedTokenDataset(GOLD / "ref_tokens.bin", int(seq), int(stride))
        assert [len(ds), ds.vocab_size, ds.token_count] == list(tg[key])
    for tag in ("seq", "ragged"):
        seq = int(tg[f"{tag}/params"][0])
        ds = tokenfile.MappedTokenDataset(GOLD / "ref_tokens.bin", seq, seq)
        inp, tgt = ds.windows()
        assert np.array_equal(inp, tg[f"{tag}/inputs"]) and np.array_equal(tgt, tg[f"{tag}/targets"])


def test_python_reader_raises_the_reference_messages(tokenfile, tg, tmp_path):
    want = dict(line.split("\t", 1) for line in tg["messages"])
    for tag, p in damaged_copies(tmp_path).items():
        with pytest.raises(RuntimeError) as e:
            tokenfile.MappedTokenDataset(p, 5, 5)
        assert str(e.value) == want[tag].replace("{path}", str(p))
    raw = (GOLD / "ref_tokens.bin").read_bytes()
    p = tmp_path / "small_vocab.bin"
    p.write_bytes(raw[:4] + (20).to_bytes(4, "little") + raw[8:])
    with pytest.raises(RuntimeError) as e:
        tokenfile.MappedTokenDataset(p, 5, 5).windows()
    assert str(e.value) == str(tg["id_message"][0])
    with pytest.raises(ValueError, match="0 < vocab_size <= 65536"):
        tokenfile.write(tmp_path / "x.bin", [1], 70000)
    with pytest.raises(RuntimeError, match="token id out of range for vocab while writing"):
        tokenfile.write(tmp_path / "x.bin", [1, 9], 9)


def test_cpp_data_classes_match_reference(tg, tmp_path):
    """Compiled against libstdc++ like the reference, so the shuffled loaders draw the same windows."""
    exe = tmp_path / "tokenfile_shim_check"
    libdir = ROOT / "grad.cpp_b200"
    subprocess.run(["g++", "-std=c++20", "-O1", str(ROOT / "tests" / "tokenfile_shim_check.cpp"), "-o", str(exe),
                    f"-L{libdir}", "-lgradb", f"-Wl,-rpath,{libdir}"], check=True)
    dmg = damaged_copies(tmp_path)
    order = list(dmg)
    scratch = tmp_path / "copy.bin"
    out = subprocess.run([str(exe), str(GOLD / "ref_tokens.bin"), str(scratch)] + [str(dmg[t]) for t in order],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    lines = out.stdout.splitlines()
    for key in ("open_5_5", "open_12_12", "open_7_1", "open_16_16"):
        got = [ln for ln in lines if ln.startswith(key + " ")][0].split()[1:]
        assert [int(x) for x in got] == list(tg[key])
    assert "batches 14" in lines
    for tag in ("seq", "capped", "train", "ragged"):
        rows = [ln[len(tag) + 1:] for ln in lines if ln.startswith(tag + " ")]
        inp = np.array([[int(x) for x in r.split(" | ")[0].split()] for r in rows], np.int32)
        tgt = np.array([[int(x) for x in r.split(" | ")[1].split()] for r in rows], np.int32)
        assert np.array_equal(inp, tg[f"{tag}/inputs"]), tag
        assert np.array_equal(tgt, tg[f"{tag}/targets"]), tag
    assert scratch.read_bytes() == (GOLD / "ref_tokens.bin").read_bytes()
    assert "exists 1 0" in lines
    assert "stride\tstride must be >= 1" in lines
    assert "batch\tbatch_size must be >= 1" in lines
    assert "vocab\ttoken file requires 0 < vocab_size <= 65536 (uint16 storage)" in lines
    assert any(ln.startswith("range\ttoken id out of range for vocab while writing") for ln in lines)
    want = dict(line.split("\t", 1) for line in tg["messages"])
    for i, tag in enumerate(order):
        got = [ln for ln in lines if ln.startswith(f"damaged{i}\t")][0].split("\t", 1)[1]
        assert got == want[tag].replace("{path}", str(dmg[tag])), tag
