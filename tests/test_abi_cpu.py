"""CPU: the C-ABI library loads, exports every declared symbol, and its host-only
entry points (checkpoint reader/writer) behave like the reference's.

Checkpoint cases mirror tests/unit/test_core_regressions.cpp:426-541 of the
reference: bitwise round trip, byte offsets, truncation and bad-field messages,
the 20-byte tokenizer trailer, unknown trailer tags.
"""
import ctypes as C
import re
import struct
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
GOLD = ROOT / "tests" / "golden"


@pytest.fixture(scope="module")
def B(pkg):
    from grad_cpp_b200 import binding
    binding.lib()
    return binding


def test_library_exports_every_declared_symbol(B):
    header = (ROOT / "include" / "gradb.h").read_text()
    declared = set(re.findall(r"\b(gradb_[a-z_0-9]+)\s*\(", header))
    assert declared == set(B.SIGNATURES), declared ^ set(B.SIGNATURES)
    L = B.lib()
    for name in declared:
        assert hasattr(L, name), name


def test_no_device_is_an_error_not_a_fallback(B, tmp_path, ck):
    n = C.c_int(-1)
    rc = B.lib().gradb_device_count(C.byref(n))
    if n.value > 0:
        pytest.skip("a GPU is present")
    assert rc == B.ERR_NO_DEVICE
    dm = ck.ModelDims(23, 32, 1, 4, 8, 1)
    p = ck.write_synthetic(tmp_path / "m.bin", dm, 1)
    with pytest.raises(B.GradbError) as e:
        B.GPTModel.load(p)
    assert e.value.status == B.ERR_NO_DEVICE and "no CPU path" in str(e.value)


@pytest.mark.parametrize("name", ["ref_tiny_gpt2", "ref_tiny_modern", "ref_tiny_gpt2_fp", "ref_tiny_modern_fp"])
def test_reads_files_written_by_the_reference_and_rewrites_them_bit_for_bit(B, ck, name, tmp_path):
    src = GOLD / f"{name}.bin"
    d = B.inspect_checkpoint(src)
    assert (d.vocab_size, d.d_model, d.num_layers, d.num_heads, d.max_len) == (11, 8, 1, 2, 4)
    assert d.arch == (1 if "modern" in name else 0)
    assert d.d_ff == (64 if "modern" in name else 32)
    assert d.has_fingerprint == (1 if name.endswith("_fp") else 0)
    if d.has_fingerprint:
        assert (d.fingerprint_kind, d.fingerprint_hash) == (2, 0x1122334455667788)
    dm, tensors, fp = ck.read_checkpoint(src)
    out = tmp_path / "rewritten.bin"
    B.write_checkpoint(out, d, tensors)
    assert out.read_bytes() == src.read_bytes()
    # the tokenizer trailer is exactly 20 bytes (test_core_regressions.cpp:502)
    if name.endswith("_fp"):
        assert src.stat().st_size - (GOLD / f"{name[:-3]}.bin").stat().st_size == 20


def test_header_byte_offsets(B):
    raw = (GOLD / "ref_tiny_gpt2.bin").read_bytes()
    assert raw[:4] == bytes([0x4D, 0x54, 0x50, 0x47])
    assert struct.unpack_from("<I", raw, 4)[0] == 2
    # fields at 8 (arch), 12.. hyperparameters, first tensor dims at 36 (test_core_regressions.cpp:455-457)
    assert struct.unpack_from("<iiiiii", raw, 8) == (0, 11, 8, 1, 2, 4)
    assert struct.unpack_from("<ii", raw, 36) == (11, 8)


def _expect_fail(B, path, needle):
    with pytest.raises(B.GradbError) as e:
        B.inspect_checkpoint(path)
    assert e.value.status == B.ERR_CHECKPOINT
    msg = str(e.value)
    assert msg.startswith(f"Failed to load model from {path}: "), msg
    assert needle in msg, msg


def test_corrupt_files_fail_with_the_reference_messages(B, tmp_path):
    raw = bytearray((GOLD / "ref_tiny_gpt2.bin").read_bytes())
    p = tmp_path / "c.bin"

    p.write_bytes(raw[:20])
    _expect_fail(B, p, "file ends while reading")
    p.write_bytes(raw[:100])
    _expect_fail(B, p, "file ends inside token embedding")
    p.write_bytes(raw[:-7])
    _expect_fail(B, p, "file ends inside final norm beta")

    bad = bytearray(raw); bad[0] ^= 0xFF
    p.write_bytes(bad)
    _expect_fail(B, p, "not a grad.cpp checkpoint (wrong magic number)")
    bad = bytearray(raw); struct.pack_into("<I", bad, 4, 3)
    p.write_bytes(bad)
    _expect_fail(B, p, "unsupported format version 3")
    bad = bytearray(raw); struct.pack_into("<I", bad, 8, 7)
    p.write_bytes(bad)
    _expect_fail(B, p, "unknown architecture tag 7")
    bad = bytearray(raw); struct.pack_into("<i", bad, 12, 0)
    p.write_bytes(bad)
    _expect_fail(B, p, "header field vocab_size = 0 is outside [1, 16777216]")
    bad = bytearray(raw); struct.pack_into("<i", bad, 24, 3)
    p.write_bytes(bad)
    _expect_fail(B, p, "d_model 8 is not divisible by num_heads 3")
    bad = bytearray(raw); struct.pack_into("<f", bad, 32, 1.5)
    p.write_bytes(bad)
    _expect_fail(B, p, "dropout_rate 1.500000 is outside [0, 1)")
    bad = bytearray(raw); struct.pack_into("<ii", bad, 36, 8, 11)
    p.write_bytes(bad)
    _expect_fail(B, p, "token embedding is 8x11, model expects 11x8")

    with pytest.raises(B.GradbError) as e:
        B.inspect_checkpoint(tmp_path / "missing.bin")
    assert str(e.value) == f"Could not open checkpoint for reading: {tmp_path / 'missing.bin'}"


def test_trailer_sections(B, tmp_path):
    raw = (GOLD / "ref_tiny_gpt2.bin").read_bytes()
    p = tmp_path / "t.bin"
    # unknown tags are skipped, the tokenizer section still read after them
    p.write_bytes(raw + b"XTRA" + struct.pack("<I", 5) + b"hello" + b"TKFP" + struct.pack("<IIQ", 12, 1, 0xABCDEF))
    d = B.inspect_checkpoint(p)
    assert (d.has_fingerprint, d.fingerprint_kind, d.fingerprint_hash) == (1, 1, 0xABCDEF)
    p.write_bytes(raw + b"TKFP" + struct.pack("<I", 8) + b"12345678")
    _expect_fail(B, p, "tokenizer trailer has length 8, expected 12")
    p.write_bytes(raw + b"TKFP" + struct.pack("<IIQ", 12, 9, 1))
    _expect_fail(B, p, "unknown tokenizer kind 9")
    p.write_bytes(raw + b"XTRA" + struct.pack("<I", (1 << 20) + 1))
    _expect_fail(B, p, "implausible length")
    p.write_bytes(raw + b"XTRA" + struct.pack("<I", 50) + b"short")
    _expect_fail(B, p, "file ends inside trailer section")
    p.write_bytes(raw + b"XT")
    _expect_fail(B, p, "file ends while reading trailer section header")


def test_version_1_files_load_as_gpt2(B, ck, tmp_path):
    dm = ck.ModelDims(11, 8, 1, 2, 4, 0)
    p = tmp_path / "v1.bin"
    ck.write_checkpoint(p, dm, ck.synthetic_tensors(dm, 3), version=1)
    d = B.inspect_checkpoint(p)
    assert (d.format_version, d.arch, d.d_ff) == (1, 0, 32)


def test_tensor_shapes_match_the_python_writer(B, ck):
    for arch in (0, 1):
        dm = ck.ModelDims(50, 24, 3, 4, 9, arch)
        d = B.ModelDesc(dm.vocab, dm.d_model, dm.layers, dm.heads, dm.max_len, dm.arch)
        n = C.c_int()
        assert B.lib().gradb_tensor_count(C.byref(d), C.byref(n)) == 0
        shapes = ck.tensor_shapes(dm)
        assert n.value == len(shapes)
        for i, (_, r, c) in enumerate(shapes):
            rr, cc = C.c_int(), C.c_int()
            assert B.lib().gradb_tensor_shape(C.byref(d), i, C.byref(rr), C.byref(cc)) == 0
            assert (rr.value, cc.value) == (r, c)


def test_oracle_reader_agrees_on_reference_files(port):
    m = port.load(GOLD / "ref_tiny_modern_fp.bin")
    d = port.dims(m)
    assert (d["vocab"], d["d_model"], d["arch"], d["d_ff"], d["has_fp"], d["fp_kind"]) == (11, 8, 1, 64, 1, 2)
    assert d["fp_hash"] == 0x1122334455667788
    port.free(m)


def test_exact_sum_arithmetic_matches_sequential_fp32(tmp_path):
    """The selection kernel's parallel-scan arithmetic, run on the host against plain loops."""
    import subprocess
    exe = tmp_path / "exact_sum_check"
    subprocess.run(["g++", "-std=c++17", "-O1", "-ffp-contract=off", str(ROOT / "tests" / "exact_sum_check.cpp"),
                    "-o", str(exe)], check=True)
    out = subprocess.run([str(exe), "400", "7"], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr


def test_host_code_is_clean_under_address_and_undefined_behaviour_sanitizers(tmp_path):
    """The checkpoint reader/writer over good and damaged files, and the exact-sum arithmetic shared with the
    selection kernel, built with -fsanitize=address,undefined; any report aborts the run."""
    import subprocess
    san = ["-fsanitize=address,undefined", "-fno-sanitize-recover=all", "-fno-omit-frame-pointer", "-g", "-O1"]
    exe = tmp_path / "checkpoint_sanitize_check"
    subprocess.run(["g++", "-std=c++17", *san, str(ROOT / "tests" / "checkpoint_sanitize_check.cpp"),
                    str(ROOT / "grad.cpp_b200" / "csrc" / "checkpoint.cpp"), "-o", str(exe)], check=True)
    files = [str(GOLD / f"ref_{n}.bin") for n in ("tiny_gpt2", "tiny_modern", "tiny_gpt2_fp", "tiny_modern_fp")]
    out = subprocess.run([str(exe), str(tmp_path / "scratch.bin"), *files], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = re.search(r"parsed (\d+) rejected (\d+)", out.stdout)
    assert int(m.group(1)) >= 4 and int(m.group(2)) > 100, out.stdout
    exe2 = tmp_path / "exact_sum_check_san"
    subprocess.run(["g++", "-std=c++17", *san, "-ffp-contract=off", str(ROOT / "tests" / "exact_sum_check.cpp"),
                    "-o", str(exe2)], check=True)
    out = subprocess.run([str(exe2), "60", "7"], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
