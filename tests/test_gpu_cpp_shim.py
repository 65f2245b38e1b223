"""GPU: the C++20 drop-in classes (include/gradb/engine.hpp) compiled against the library,
driven like the reference's own decode parity test, and compared with the CPU oracle."""
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def test_cpp_classes_match_oracle(golden_ckpt, port, tmp_path):
    dm, path = golden_ckpt("tiny_modern")
    exe = tmp_path / "engine_shim_check"
    libdir = ROOT / "grad.cpp_b200"
    subprocess.run(["g++", "-std=c++20", "-O1", str(ROOT / "tests" / "engine_shim_check.cpp"), "-o", str(exe),
                    f"-L{libdir}", "-lgradb", f"-Wl,-rpath,{libdir}"], check=True)
    tokens = tmp_path / "tokens.bin"
    tokens.write_bytes((ROOT / "tests" / "golden" / "ref_tokens.bin").read_bytes())
    out = subprocess.run([str(exe), path, str(tokens)], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    text = out.stdout
    assert f"missing: Could not open checkpoint for reading: {path}.missing" in text
    assert f"dims {dm.vocab} {dm.d_model} {dm.layers} {dm.heads} {dm.max_len} {dm.arch}" in text
    assert "bad id: InferenceSession: token id out of vocab range" in text
    assert f"full at {dm.max_len} of {dm.max_len}: InferenceSession: context exceeds max_len" in text
    om = port.load(path)
    want = port.logits_for(om, [3, 11, 7, 0, 19, 5])
    rows = re.findall(r"logits (\d+) (\S+) (\S+) (\S+)", text)
    assert len(rows) == 6
    for i, (pos, a, b, c) in enumerate(rows):
        assert int(pos) == i + 1
        got = np.array([float(a), float(b), float(c)])
        ref = np.array([want[i, 0], want[i, 1], want[i, -1]])
        assert np.abs(got - ref).max() < 1e-4 * np.abs(want).max()
    greedy = [int(x) for x in re.search(r"greedy((?: \d+)+)", text).group(1).split()]
    assert greedy == list(port.generate(om, [3, 11, 7, 0], 8, greedy=True, penalty=1.2))
    sample = [int(x) for x in re.search(r"sample((?: \d+)+)", text).group(1).split()]
    assert len(sample) == 12 and sample[:4] == [3, 11, 7, 0]
    assert "stream 5 5" in text
    assert "stream stopped after 3: enough" in text
    assert "draws aligned" in text
    assert "empty ''" in text
    # `grad eval` through the C++ classes: token file -> loaders -> training::mean_loss, against the loss the
    # reference computes over the same loaders (tests/golden/tokenfile_golden.npz)
    tg = np.load(ROOT / "tests" / "golden" / "tokenfile_golden.npz")
    assert "dataset 40 23 203" in text and "batches 14" in text
    got_all = float(re.search(r"mean_loss_all (\S+)", text).group(1))
    got_capped = float(re.search(r"mean_loss_capped (\S+)", text).group(1))
    assert abs(got_all - float(tg["tiny_modern/seq/mean"][0])) < 2e-5 * got_all
    assert abs(got_capped - float(tg["tiny_modern/capped/mean"][0])) < 2e-5 * got_capped
    shuffled = [int(x) for x in re.search(r"shuffled((?: \d+)+)", text).group(1).split()]
    assert shuffled == list(tg["capped/inputs"][:3].reshape(-1))
    assert (tmp_path / "tokens.bin.copy").read_bytes()[:16] == (ROOT / "tests/golden/ref_tokens.bin").read_bytes()[:8] \
        + (200).to_bytes(8, "little")
    assert f"bad magic: Not a token file (bad magic): {path}" in text
    assert "too short: Not enough tokens for even one sequence: " in text
    port.free(om)
