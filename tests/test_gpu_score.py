"""GPU: teacher-forced scoring (the device half of `grad eval`) through the C ABI, against values
the reference itself produced (tests/golden/score_golden.npz) and against the CPU restatement.

fp32 mode bars: every target log-probability within 2e-4 absolute, batch losses and the mean
within 2e-5 relative (the same bars the restatement meets against the reference). bf16 mode is
not a bit-exact mode; its error is bounded against the fp32 restatement."""
import numpy as np
import pytest

from conftest import GOLDEN_MODELS, ROOT

pytestmark = pytest.mark.gpu
ROW_TOL = 2e-4
LOSS_TOL = 2e-5


@pytest.fixture(scope="module")
def G(pkg):
    import grad_cpp_b200 as g
    g.lib()
    return g


@pytest.fixture(scope="module")
def score_golden():
    return np.load(ROOT / "tests" / "golden" / "score_golden.npz")


# max_batch 1 scores through the single-sequence persistent kernel, 2 and 64 through the batched
# streaming kernels; 2 also makes the windows span several resident groups.
@pytest.mark.parametrize("max_batch", [1, 2, 64])
@pytest.mark.parametrize("name", list(GOLDEN_MODELS))
def test_fp32_scores_match_reference_fixture(name, max_batch, G, golden_ckpt, score_golden):
    dm, path = golden_ckpt(name)
    g = score_golden
    inp, tgt = g[f"{name}/inputs"], g[f"{name}/targets"]
    bw = int(g[f"{name}/batch_windows"][0])
    m = G.GPTModel.load(path, 0, G.FP32)
    s = G.BatchSession(m, max_batch)
    logp = s.score(inp, tgt)
    np.testing.assert_allclose(logp, g[f"{name}/row_logp"], rtol=0, atol=ROW_TOL)
    mean, batch = s.mean_loss(inp, tgt, bw)
    np.testing.assert_allclose(batch, g[f"{name}/batch_loss"], rtol=LOSS_TOL)
    assert abs(mean - float(g[f"{name}/mean"][0])) <= LOSS_TOL * abs(mean)
    # the session is left holding the last group, positioned after its window
    assert s.position(0) == inp.shape[1]
    s.close()
    m.close()


def test_scoring_errors_and_empty_input(G, golden_ckpt):
    dm, path = golden_ckpt("tiny_gpt2")
    m = G.GPTModel.load(path, 0, G.FP32)
    s = G.BatchSession(m, 4)
    ok = np.zeros((2, dm.max_len), np.int32)
    s.score(ok, ok)
    with pytest.raises(RuntimeError, match="InferenceSession: context exceeds max_len"):
        s.score(np.zeros((2, dm.max_len + 1), np.int32), np.zeros((2, dm.max_len + 1), np.int32))
    bad = ok.copy()
    bad[1, 2] = dm.vocab
    with pytest.raises(IndexError, match="InferenceSession: token id out of vocab range"):
        s.score(bad, ok)
    mean, batch = s.mean_loss(np.zeros((0, 4), np.int32), np.zeros((0, 4), np.int32), 8)
    assert mean == -1.0 and len(batch) == 0   # no batches: trainer.cpp:339
    s.close()
    m.close()


@pytest.mark.parametrize("name,n_windows", [("hs64_modern", 20), ("hs64_gpt2", 40), ("odd_modern", 17)])
def test_bf16_batched_scoring_tracks_fp32_oracle(name, n_windows, G, golden_ckpt, port, monkeypatch):
    """>= 16 windows in bf16 mode: all windows' positions go through the tensor-core GEMMs at once
    and every row's logits are formed by one GEMM over the tied embedding."""
    dm, path = golden_ckpt(name)
    S = dm.max_len - 3
    stream = np.random.default_rng(31).integers(0, dm.vocab, n_windows * S + 1).astype(np.int32)
    inp = np.stack([stream[i * S:i * S + S] for i in range(n_windows)])
    tgt = np.stack([stream[i * S + 1:i * S + S + 1] for i in range(n_windows)])
    tgt[2, 1] = -1
    m16 = G.GPTModel.load(path, 0, G.BF16)
    s = G.BatchSession(m16, n_windows)
    got = s.score(inp, tgt)
    assert got[2, 1] == 0.0
    om = port.load(path)
    _, _, want = port.mean_loss(om, inp[:6], tgt[:6], 8)
    port.free(om)
    err = float(np.abs(got[:6] - want).max())
    assert err < 6e-2, err
    # the same windows position by position through the bf16 step kernels
    monkeypatch.setenv("GRADB_NO_BATCHED_FEED", "1")
    s2 = G.BatchSession(m16, n_windows)
    stepwise = s2.score(inp, tgt)
    assert float(np.abs(got - stepwise).max()) < 6e-2
    mean_a, _ = s.mean_loss(inp, tgt, 8)
    mean_b, _ = s2.mean_loss(inp, tgt, 8)
    assert abs(mean_a - mean_b) < 2e-3 * mean_b
    s.close(); s2.close(); m16.close()


def test_eval_shape_windows_of_256_on_the_69m_model(G, ck, port, tmp_path, monkeypatch):
    """`grad eval`'s shape: windows of 256 ids in batches of 8 (src/cli/eval.cpp:77,142) on the 69.0M
    modern block. The oracle scores the start of one window; the rest is checked through properties:
    with N(0, 0.02) tied embeddings over unit-RMS hidden rows the logits are near N(0, d * 0.02^2) and
    independent of the target, so every batch loss sits near ln(vocab) + d * 0.02^2 / 2; and the bf16
    and fp32 modes agree."""
    dm = ck.PRESETS["modern"]
    path = str(ck.write_synthetic(tmp_path / "modern.bin", dm, 1004))
    n, S = 40, 256
    stream = np.random.default_rng(2011).integers(0, dm.vocab, n * S + 1).astype(np.int32)
    inp = np.stack([stream[i * S:i * S + S] for i in range(n)])
    tgt = np.stack([stream[i * S + 1:i * S + S + 1] for i in range(n)])
    m16 = G.GPTModel.load(path, 0, G.BF16)
    s16 = G.BatchSession(m16, 32, 256)
    lp16 = s16.score(inp, tgt)
    ms = s16.last_score_ms
    mean16, batch16 = s16.mean_loss(inp, tgt, 8)
    # K and V rows of the last resident group (windows 32..39 sit in slots 0..7), first and last layer
    probes = [(w, layer, which, pos) for w in (0, 7) for layer in (0, dm.layers - 1) for which in (0, 1)
              for pos in (0, 100, 255)]
    wide_rows = [s16.cache_row(w, layer, which, pos) for (w, layer, which, pos) in probes]
    s16.close(); m16.close()
    assert len(batch16) == 5
    assert np.all(np.abs(batch16 - (np.log(dm.vocab) + dm.d_model * 0.02 ** 2 / 2)) < 0.03)
    m32 = G.GPTModel.load(path, 0, G.FP32)
    s32 = G.BatchSession(m32, 8, 256)
    lp32 = s32.score(inp[:8], tgt[:8])
    s32.close(); m32.close()
    # bf16 weights and activations against fp32: rms near 5e-3 over the 2048 positions, the largest near 2e-2
    assert float(np.sqrt(np.mean((lp16[:8] - lp32) ** 2))) < 7e-3 and float(np.abs(lp16[:8] - lp32).max()) < 3e-2
    om = port.load(path)
    _, _, want = port.mean_loss(om, inp[:1, :12], tgt[:1, :12], 8)
    port.free(om)
    np.testing.assert_allclose(lp32[0, :12], want[0], rtol=0, atol=ROW_TOL)
    # the persistent many-tile GEMM kernel against the one-tile-per-CTA kernel on the same rows
    monkeypatch.setenv("GRADB_NO_WIDE_GEMM", "1")
    m16 = G.GPTModel.load(path, 0, G.BF16)
    s16 = G.BatchSession(m16, 32, 256)
    lp16_narrow = s16.score(inp, tgt)
    narrow_rows = [s16.cache_row(w, layer, which, pos) for (w, layer, which, pos) in probes]
    s16.close(); m16.close()
    # same arithmetic up to the rounding of one fused multiply-add in RoPE, which bf16 activations downstream amplify
    assert float(np.abs(lp16 - lp16_narrow).max()) < 2e-2
    for a, b in zip(wide_rows, narrow_rows):
        assert np.abs(a - b).max() < 1e-2 * max(np.abs(b).max(), 1e-6)
    print(f"scored {n * S} ids in {ms:.2f} ms ({n * S / ms * 1e3:.0f} ids/s), mean loss {mean16:.4f}")


@pytest.mark.parametrize("name", ["tiny_gpt2", "tiny_modern"])
def test_eval_over_a_token_file_matches_reference(name, G, golden_ckpt):
    """`grad eval` end to end: the reference's token file -> windows -> device scoring -> the loss the
    reference reports for the same loader (sequential, ragged last batch, and its shuffled picks)."""
    from support import tokenfile
    tg = np.load(ROOT / "tests" / "golden" / "tokenfile_golden.npz")
    dm, path = golden_ckpt(name)
    m = G.GPTModel.load(path, 0, G.FP32)
    s = G.BatchSession(m, 16)
    for tag in ("seq", "ragged"):
        seq, batch = int(tg[f"{tag}/params"][0]), int(tg[f"{tag}/params"][1])
        ds = tokenfile.MappedTokenDataset(ROOT / "tests" / "golden" / "ref_tokens.bin", seq, seq)
        inp, tgt = ds.windows()
        mean, _ = s.mean_loss(inp, tgt, batch)
        want = float(tg[f"{name}/{tag}/mean"][0])
        assert abs(mean - want) <= LOSS_TOL * want, (tag, mean, want)
    for tag in ("capped", "train"):
        batch = int(tg[f"{tag}/params"][1])
        mean, _ = s.mean_loss(tg[f"{tag}/inputs"], tg[f"{tag}/targets"], batch)
        want = float(tg[f"{name}/{tag}/mean"][0])
        assert abs(mean - want) <= LOSS_TOL * want, (tag, mean, want)
    s.close()
    m.close()


PAIRS_SCRIPT = """
import sys
import numpy as np
sys.path.insert(0, sys.argv[1] + "/tests"); sys.path.insert(0, sys.argv[1])
from conftest import load_package
g = load_package()
from grad_cpp_b200 import checkpoint as ck
g.lib()
dm = ck.PRESETS[sys.argv[4]]
n, S = 128, 256
stream = np.random.default_rng(2012).integers(0, dm.vocab, n * S + 1).astype(np.int32)
inp = np.stack([stream[i * S:i * S + S] for i in range(n)])
tgt = np.stack([stream[i * S + 1:i * S + S + 1] for i in range(n)])
m = g.GPTModel.load(sys.argv[2], 0, g.BF16)
s = g.BatchSession(m, 128, 256)
np.save(sys.argv[3], s.score(inp, tgt))
"""


@pytest.mark.parametrize("preset", ["modern", "medium"])
def test_cta_pair_gemm_equals_the_single_cta_gemm(preset, G, ck, tmp_path):
    """32768 rows in one pass: every single-weight-tile projection (Q|K|V, the two residual projections, the
    log-sum-exp logits, whose 125 feature tiles leave the last pair's odd CTA without a tile) runs on clusters of
    two CTAs with cta_group::2 MMAs. The same arithmetic in the same order as the one-CTA kernel with 256-token
    tiles (GRADB_WIDE_PAIRS=0, read once per process, hence the child processes): equal log-probabilities. `medium`
    is the GPT-2 block: biases, LayerNorm and the GELU epilogue (24 feature tiles) on pairs as well. The first
    windows are also scored by an fp32 session."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    dm = ck.PRESETS[preset]
    path = str(ck.write_synthetic(tmp_path / "model.bin", dm, 1004))
    outs = []
    for name, extra in (("pairs", {}), ("single", {"GRADB_WIDE_PAIRS": "0"})):
        out = tmp_path / f"lp_{name}.npy"
        r = subprocess.run([sys.executable, "-c", PAIRS_SCRIPT, str(root), path, str(out), preset],
                           env=dict(os.environ, **extra), capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-3000:]
        outs.append(np.load(out))
    assert np.isfinite(outs[0]).all()
    assert abs(float(-outs[0].mean()) - (np.log(dm.vocab) + dm.d_model * 0.02 ** 2 / 2)) < 0.03
    assert np.abs(outs[0] - outs[1]).max() < 1e-6
    n, S = 4, 256
    stream = np.random.default_rng(2012).integers(0, dm.vocab, 128 * S + 1).astype(np.int32)
    inp = np.stack([stream[i * S:i * S + S] for i in range(n)])
    tgt = np.stack([stream[i * S + 1:i * S + S + 1] for i in range(n)])
    m32 = G.GPTModel.load(path, 0, G.FP32)
    s32 = G.BatchSession(m32, 4, 256)
    lp32 = s32.score(inp, tgt)
    s32.close(); m32.close()
    assert float(np.sqrt(np.mean((outs[0][:n] - lp32) ** 2))) < 7e-3 and float(np.abs(outs[0][:n] - lp32).max()) < 3e-2
