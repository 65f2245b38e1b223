"""GPU: grad.cpp's own command line driving the engine. `grad-b200` is built from integration/ plus the reference's
unmodified CLI, tokenizer, data and model sources (make -C integration REF=<grad.cpp tree>, done by the build step
where that tree exists; the binary travels with the working tree). One binary holds both engines, so every command
is run twice on the same files - `--device cpu` (the reference's classes) and `--device b200` - and compared."""
import json
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
EXE = ROOT / "oracle" / "_ref" / "grad-b200"


def run(args, cwd, stdin=None, ok=True):
    out = subprocess.run([str(EXE), *args], cwd=cwd, input=stdin, capture_output=True, text=True, encoding="latin-1", timeout=600)
    if ok:
        assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    return out


@pytest.fixture(scope="module")
def workdir(ck, tmp_path_factory):
    if not EXE.exists():
        pytest.skip("grad-b200 has not been built (needs the grad.cpp tree at build time)")
    d = tmp_path_factory.mktemp("cli")
    rng = np.random.default_rng(7)
    syll = ["ka", "lo", "mi", "ren", "tu", "sa", "vor", "el", "ni", "dra", "po", "qui", "zen", "ba", "ith", "ou", "ar", "em"]
    words = ["".join(rng.choice(syll, rng.integers(1, 4))) for _ in range(120)]
    lines = [" ".join(rng.choice(words, rng.integers(4, 11))).capitalize() + str(rng.choice([".", "!", "?", ","]))
             for _ in range(400)]
    (d / "corpus.txt").write_text("\n".join(lines) + "\n")
    out = run(["prepare", "corpus.txt", "300", "--tokenizer", "v2"], d)   # the reference's own prepare
    vocab = int(re.search(r"Vocab size: (\d+)", out.stdout).group(1))
    ck.write_synthetic(d / "model.bin", ck.ModelDims(vocab, 128, 2, 2, 64, 1), 501, 0.08, True)
    return d


def greedy_block(text):
    m = re.search(r"--- Greedy Decoding ---\n\nPrompt: \"(.*?)\"\n(.*?)(?:\n\n--- Sampling|\Z)", text, re.S)
    return m.group(1), m.group(2).rstrip("\n")


def test_generate_greedy_text_is_the_reference_clis(workdir):
    base = ["generate", "--ckpt", "model.bin", "--corpus", "corpus.txt", "--max-tokens", "40", "--tokenizer", "v2"]
    for prompt in ("Kalo miren", ""):   # "" picks a held-out prompt from the val token file
        cpu = run(base + ["--prompt", prompt, "--device", "cpu"], workdir)
        gpu = run(base + ["--prompt", prompt, "--device", "b200"], workdir)
        assert "Device: b200:0 (fp32)" in gpu.stdout
        assert greedy_block(cpu.stdout) == greedy_block(gpu.stdout)
        assert "--- Sampling (temp=0.8) ---" in gpu.stdout
    only = run(base + ["--prompt", "Kalo", "--greedy", "--device", "b200"], workdir)
    assert "--- Sampling" not in only.stdout
    bf16 = run(base + ["--prompt", "Kalo miren", "--greedy", "--device", "b200-bf16"], workdir)
    assert "bf16 weights" in bf16.stdout and greedy_block(bf16.stdout)[1].startswith("Kalo miren")


def test_chat_streams_the_same_pieces(workdir):
    args = ["chat", "--ckpt", "model.bin", "--corpus", "corpus.txt", "--max-tokens", "20", "--tokenizer", "v2", "--greedy"]
    lines = "Kalo miren\nVor el ni\n\n"
    cpu = run(args + ["--device", "cpu"], workdir, stdin=lines)
    gpu = run(args + ["--device", "b200"], workdir, stdin=lines)
    tail = lambda s: s[s.index("Empty line or 'exit' quits."):]
    assert tail(cpu.stdout) == tail(gpu.stdout) and tail(gpu.stdout).count("\n> ") >= 3


def test_eval_reports_the_same_losses(workdir):
    args = ["eval", "model.bin", "corpus.txt", "--seq", "16", "--batches", "3", "--tokenizer", "v2"]
    losses = {}
    for dev in ("cpu", "b200"):
        out = run(args + ["--device", dev], workdir).stdout
        losses[dev] = [float(x) for x in re.findall(r"^(?:val|train)\s+loss (\S+)", out, re.M)]
        assert len(losses[dev]) == 2
    assert np.allclose(losses["cpu"], losses["b200"], atol=2e-4), losses
    whole = [run(["eval", "model.bin", "corpus.txt", "--seq", "16", "--tokenizer", "v2", "--device", d], workdir).stdout
             for d in ("cpu", "b200")]
    vals = [float(re.search(r"^val\s+loss (\S+)", w, re.M).group(1)) for w in whole]
    assert abs(vals[0] - vals[1]) < 2e-4, vals


def test_bench_generation_section_and_json(workdir):
    out = run(["bench", "--device", "b200", "--trials", "3", "--corpus", "corpus.txt", "--json", "bench.json"], workdir)
    assert out.stdout.count("  trial ") == 3 and "median:" in out.stdout
    rec = json.loads((workdir / "bench.json").read_text())
    assert rec["schema_version"] == 1 and rec["device"] == "b200" and rec["config"]["d_model"] == 512
    assert len(rec["generation_tokens_per_second"]) == 3
    assert rec["median_generation_tokens_per_second"] > 1000   # the reference's laptops: ~850 tok/s
    print(f"grad bench --device b200: {rec['median_generation_tokens_per_second']:.0f} tok/s (22M small, 64 sampled ids, "
          "call incl. weight-independent session set-up)")


def test_usage_errors_keep_the_reference_exit_codes(workdir):
    assert run(["generate", "--device", "b200:x"], workdir, ok=False).returncode == 2
    assert run(["generate", "--ckpt", "nope.bin", "--device", "b200"], workdir, ok=False).returncode == 1
    assert run(["nonsense"], workdir, ok=False).returncode == 2
    assert run(["generate", "--device", "b200:7"], workdir, ok=False).returncode in (0, 1)  # 1 unless 8 GPUs are here
