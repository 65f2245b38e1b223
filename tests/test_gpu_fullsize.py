"""GPU: the benchmark's own model shapes. The oracle needs seconds per rollout
here, so the teacher-forced comparisons use a short context and the long
rollouts are compared id by id."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


@pytest.fixture(scope="module")
def G(pkg):
    import grad_cpp_b200 as g
    g.lib()
    return g


@pytest.fixture(scope="module")
def ckpts(ck, tmp_path_factory):
    base = tmp_path_factory.mktemp("full")
    made = {}

    def get(preset, seed):
        if preset not in made:
            made[preset] = (ck.PRESETS[preset], str(ck.write_synthetic(base / f"{preset}.bin", ck.PRESETS[preset], seed)))
        return made[preset]

    return get


def test_small_gpt2_config_greedy_rollout_and_logits(G, ckpts, port):
    """d512 L6 H8 vocab 5000, 16-id prompt, greedy to context 96."""
    dm, path = ckpts("small", 1001)
    rng = np.random.default_rng(2001)
    prompt = rng.integers(0, dm.vocab, 16).astype(np.int32)
    m = G.GPTModel.load(path)
    om = port.load(path)
    for pen in (1.0, 1.2):
        got = G.TextGen(m).generate_greedy(prompt, 80, pen)
        want = port.generate(om, prompt, 80, greedy=True, penalty=pen)
        assert len(got) == 96 and np.array_equal(got, want), pen
    s = G.InferenceSession(m)
    lg = np.stack([s.step(int(t)) for t in want[:40]])
    ref = port.logits_for(om, want[:40])
    assert rel_err(lg, ref) < 1e-4, rel_err(lg, ref)
    port.free(om)
    m.close()


def test_modern_config_greedy_and_sampled_rollouts_to_context_256(G, ckpts, port):
    """d768 L8 H12 vocab 16000 (69.0M parameters), 32-id prompt, decode to context 256."""
    dm, path = ckpts("modern", 1002)
    rng = np.random.default_rng(2002)
    prompt = rng.integers(0, dm.vocab, 32).astype(np.int32)
    m = G.GPTModel.load(path)
    om = port.load(path)
    got = G.TextGen(m).generate_greedy(prompt, 224, 1.0)
    want = port.generate(om, prompt, 224, greedy=True, penalty=1.0)
    assert len(got) == 256
    first_diff = next((i for i in range(len(want)) if got[i] != want[i]), None)
    assert first_diff is None, f"greedy rollout diverges at id {first_diff}"
    draws = rng.random(224, dtype=np.float32)
    got = G.TextGen(m).generate_sample(prompt, 0.8, 224, 1.1, 40, 0.9, draws=draws)
    want = port.generate(om, prompt, 224, greedy=False, temperature=0.8, penalty=1.1, top_k=40, top_p=0.9, draws=draws)
    assert np.array_equal(got, want)
    # teacher-forced logits over the first 48 positions
    s = G.InferenceSession(m)
    lg = np.stack([s.step(int(t)) for t in want[:48]])
    ref = port.logits_for(om, want[:48])
    assert rel_err(lg, ref) < 1e-4, rel_err(lg, ref)
    port.free(om)
    m.close()


def test_medium_config_batch_of_ragged_prompts(G, ckpts, port):
    """d768 L8 H12 GELU 3072, 64 sequences with prompt lengths in [8, 64]; a few
    sequences are checked against independent oracle sessions."""
    dm, path = ckpts("medium", 1003)
    rng = np.random.default_rng(2003)
    lens = rng.integers(8, 65, 64)
    prompts = [rng.integers(0, dm.vocab, int(n)).astype(np.int32) for n in lens]
    m = G.GPTModel.load(path)
    s = G.BatchSession(m, 64, 256)
    outs = s.generate(prompts, G.Sampling(1, 1.0, 1.0, 0, 1.0), 24)
    om = port.load(path)
    for i in (0, 17, 63):
        want = port.generate(om, prompts[i], 24, greedy=True, penalty=1.0)
        assert np.array_equal(outs[i], want), i
    # the same model, one sequence: the persistent single-sequence kernel with 32 hidden units per CTA
    # (d_ff 3072 over 148 SMs), i.e. two ring slots of FFN-down rows per CTA
    s1 = G.BatchSession(m, 1, 256)
    out1 = s1.generate([prompts[17]], G.Sampling(1, 1.0, 1.0, 0, 1.0), 24)[0]
    assert np.array_equal(out1, port.generate(om, prompts[17], 24, greedy=True, penalty=1.0))
    s1.close()
    port.free(om)
    s.close()
    m.close()


def test_long_context_split_attention_matches_oracle(G, ck, port, tmp_path):
    """Context 2048 exercises the split-context attention path: a 2-layer model of
    the modern shape keeps the oracle's cost to seconds."""
    dm = ck.ModelDims(16000, 768, 2, 12, 2048, 1)
    path = str(ck.write_synthetic(tmp_path / "long.bin", dm, 1005))
    rng = np.random.default_rng(2005)
    toks = rng.integers(0, dm.vocab, 1100).astype(np.int32)
    m = G.GPTModel.load(path)
    s = G.BatchSession(m, 2)
    got = s.prefill([toks, toks[:700]])
    om = port.load(path)
    want = port.logits_for(om, toks)
    assert rel_err(got[0], want[-1]) < 1e-4
    assert rel_err(got[1], want[699]) < 1e-4
    port.free(om)
    s.close()
    m.close()
