"""GPU: the CUDA path, called through the C ABI, against the CPU oracle and the
fixtures recorded from the reference.

fp32 mode bars: logits within 1e-4 relative (max-abs over max-abs), identical
greedy and sampled id sequences, selection stage bit for bit on identical logits.
"""
import zlib

import numpy as np
import pytest

from conftest import GOLDEN_MODELS, sampler_logits

pytestmark = pytest.mark.gpu
MODELS = list(GOLDEN_MODELS)
TOL = 1e-4


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


@pytest.fixture(scope="module")
def G(pkg):
    import grad_cpp_b200 as g
    g.lib()
    return g


@pytest.fixture(scope="module")
def models(G, golden_ckpt):
    cache = {}

    def get(name, precision=0):
        key = (name, precision)
        if key not in cache:
            dm, path = golden_ckpt(name)
            cache[key] = (dm, path, G.GPTModel.load(path, 0, precision))
        return cache[key]

    yield get
    for _, _, m in cache.values():
        m.close()


@pytest.mark.parametrize("name", MODELS)
def test_step_logits_match_reference_fixture(name, G, models, golden):
    dm, path, m = models(name)
    s = G.InferenceSession(m)
    want = golden[f"{name}/logits"]
    got = np.stack([s.step(int(t)) for t in golden[f"{name}/tokens"]])
    assert s.position() == dm.max_len == s.capacity()
    assert rel_err(got, want) < TOL, rel_err(got, want)


@pytest.mark.parametrize("name", MODELS)
def test_kv_cache_rows_match_oracle(name, G, models, golden, port):
    dm, path, m = models(name)
    toks = golden[f"{name}/tokens"][:7]
    s = G.BatchSession(m, 1)
    om = port.load(path)
    osess = port.session(om)
    for t in toks:
        s.step([int(t)], want_logits=False)
        port.step(osess, int(t), dm.vocab)
    for layer in range(dm.layers):
        for which in (0, 1):
            for pos in (0, 3, 6):
                got = s.cache_row(0, layer, which, pos)
                want = port.cache_row(osess, layer, which, pos, dm.d_model)
                assert np.abs(got - want).max() <= TOL * max(np.abs(want).max(), 1e-6), (layer, which, pos)
    port.session_free(osess)
    port.free(om)
    s.close()


@pytest.mark.parametrize("name", MODELS)
def test_errors_match_reference(name, G, models, golden):
    dm, path, m = models(name)
    s = G.InferenceSession(m)
    with pytest.raises(IndexError, match="InferenceSession: token id out of vocab range"):
        s.step(dm.vocab)
    with pytest.raises(IndexError):
        s._s.step([dm.vocab + 5])
    assert s.position() == 0  # a rejected id leaves the context untouched
    for t in golden[f"{name}/tokens"]:
        s.step(int(t))
    with pytest.raises(RuntimeError, match="InferenceSession: context exceeds max_len"):
        s.step(0)
    assert s.position() == dm.max_len


@pytest.mark.parametrize("name", MODELS)
def test_greedy_rollouts_match_reference_fixture(name, G, models, golden):
    dm, path, m = models(name)
    gen = G.TextGen(m)
    prompt = golden[f"{name}/prompt"]
    for pen, key in ((1.0, "greedy_p1.0"), (1.2, "greedy_p1.2")):
        got = gen.generate_greedy(prompt, dm.max_len, pen)
        assert np.array_equal(got, golden[f"{name}/{key}"]), (pen, got, golden[f"{name}/{key}"])
    assert np.array_equal(gen.generate_greedy(prompt, 3, 1.2), golden[f"{name}/greedy_short"])
    assert len(gen.generate_greedy([], 5)) == 0


@pytest.mark.parametrize("name", MODELS)
def test_sampled_rollouts_match_reference_fixture(name, G, models, golden):
    dm, path, m = models(name)
    gen = G.TextGen(m)
    prompt = golden[f"{name}/prompt"]
    for tag in "abc":
        t, pen, k, p = golden[f"{name}/sample_{tag}_params"]
        want = golden[f"{name}/sample_{tag}_ids"]
        got = gen.generate_sample(prompt, float(t), dm.max_len, float(pen), int(k), float(p),
                                  draws=golden[f"{name}/sample_{tag}_draws"])
        assert np.array_equal(got, want), (tag, got, want)
    seen = []
    n = gen.generate_stream(prompt, seen.append, 0.9, 6, 1.2, 0, 0.95, draws=golden[f"{name}/stream_draws"])
    assert n == 6 and np.array_equal(seen, golden[f"{name}/stream_ids"])


def test_selection_stage_is_bit_exact_on_reference_cases(G, models, golden, port):
    """Same logits, same draw -> same id as the reference sampler, and the same
    filtered distribution bit for bit as the restatement."""
    cases = golden["sampler/cases"]
    sessions = {}
    checked_probs = set()
    for seed, vocab, scale, quantum, t, k, p, u, tok, crc in cases:
        vocab = int(vocab)
        if vocab not in sessions:
            name = {16000: None, 5000: None, 23: "tiny_gpt2", 1003: "odd_modern"}[vocab]
            sessions[vocab] = name
        lg = sampler_logits(seed, vocab, np.float32(scale), np.float32(quantum))
        assert zlib.crc32(lg.tobytes()) == int(crc)
        s = _session_for_vocab(G, models, vocab)
        sp = G.Sampling(0, np.float32(t), 1.0, int(k), np.float32(p))
        got, probs = s.select(sp, uniforms=[np.float32(u)], logits=lg[None, :], want_probs=True)
        assert int(got[0]) == int(tok), (seed, t, k, p, u, int(got[0]), int(tok))
        if int(seed) not in checked_probs:
            checked_probs.add(int(seed))
            _, want_probs = port.sample(lg, np.float32(t), int(k), np.float32(p), np.float32(u), want_probs=True)
            assert np.array_equal(probs[0].view(np.uint32), want_probs.view(np.uint32)), seed


_VOCAB_SESSIONS = {}


def _session_for_vocab(G, models, vocab):
    """A session whose vocabulary has the wanted size (the selection stage only
    depends on the vocabulary, so any model of that width will do)."""
    if vocab not in _VOCAB_SESSIONS:
        from grad_cpp_b200 import checkpoint as ck
        import tempfile, os
        dm = ck.ModelDims(vocab, 8, 1, 2, 256, 1)
        path = os.path.join(tempfile.mkdtemp(), f"v{vocab}.bin")
        ck.write_synthetic(path, dm, 9)
        m = G.GPTModel.load(path)
        _VOCAB_SESSIONS[vocab] = (m, G.BatchSession(m, 4))
    return _VOCAB_SESSIONS[vocab][1]


def test_selection_stage_random_sweep_against_oracle(G, models, port):
    """Many random (logits, T, k, p, u) at the benchmark's vocabulary, ids and
    distributions compared bit for bit with the restatement."""
    rng = np.random.default_rng(77)
    s = _session_for_vocab(G, models, 16000)
    for i in range(60):
        scale = [0.55, 0.55, 2.0, 8.0][i % 4]
        lg = rng.standard_normal(16000, dtype=np.float32) * np.float32(scale)
        if i % 5 == 0:
            lg = np.round(lg * 4) / 4  # ties
        t = np.float32([0.8, 1.0, 0.5, 1.7][i % 4])
        k = [0, 40, 1, 500, 15999, 16000][i % 6]
        p = np.float32([0.9, 1.0, 0.5, 0.99, 0.1][i % 5])
        u = np.float32(rng.random())
        sp = G.Sampling(0, t, 1.0, k, p)
        got, probs = s.select(sp, uniforms=[u], logits=lg[None, :], want_probs=True)
        want, want_probs = port.sample(lg, t, k, p, u, want_probs=True)
        assert int(got[0]) == want, (i, t, k, p, u)
        assert np.array_equal(probs[0].view(np.uint32), want_probs.view(np.uint32)), i
    # small k around the sizes where the k-th value is read off a short list of values above a threshold (k up to
    # 256, one to sixteen maxima per warp), with and without equal values at the k-th place
    for i, k in enumerate([2, 16, 17, 100, 256, 257, 40, 40, 3, 255]):
        lg = rng.standard_normal(16000, dtype=np.float32) * np.float32([2.0, 0.55, 8.0][i % 3])
        if i % 2 == 1:
            lg = np.round(lg * 64) / 64
        t = np.float32([0.8, 1.3][i % 2])
        p = np.float32([0.9, 1.0, 0.3][i % 3])
        u = np.float32(rng.random())
        got, probs = s.select(G.Sampling(0, t, 1.0, k, p), uniforms=[u], logits=lg[None, :], want_probs=True)
        want, want_probs = port.sample(lg, t, k, p, u, want_probs=True)
        assert int(got[0]) == want, (i, k, t, p, u)
        assert np.array_equal(probs[0].view(np.uint32), want_probs.view(np.uint32)), (i, k)
    # tight clusters far apart: the probabilities crowd into a few of the sort's buckets, whatever their layout, and
    # the stage has to fall back on its slow sort; a single cluster of nearly equal values; one dominant id
    for i in range(4):
        jitter = rng.standard_normal(16000, dtype=np.float32) * np.float32(1e-4)
        if i < 2:
            lg = np.where(rng.random(16000) < 0.5, np.float32(-4.0), np.float32(3.0)).astype(np.float32) + jitter
        elif i == 2:
            lg = np.float32(1.5) + jitter
        else:
            lg = jitter.copy()
            lg[123] = np.float32(30.0)
        p = np.float32([0.9, 0.5, 0.9, 0.9][i])
        u = np.float32(rng.random())
        got, probs = s.select(G.Sampling(0, np.float32(1.0), 1.0, 0, p), uniforms=[u], logits=lg[None, :], want_probs=True)
        want, want_probs = port.sample(lg, np.float32(1.0), 0, p, u, want_probs=True)
        assert int(got[0]) == want, (i, p, u)
        assert np.array_equal(probs[0].view(np.uint32), want_probs.view(np.uint32)), i
    # every logit below the top-k sentinel (-1e10): the filtered entries end up ABOVE the survivors, as in the reference
    lg = (np.float32(-2e10) - np.abs(rng.standard_normal(16000, dtype=np.float32)) * np.float32(1e9)).astype(np.float32)
    for k in (300, 40):
        u = np.float32(rng.random())
        got, probs = s.select(G.Sampling(0, np.float32(1.0), 1.0, k, np.float32(0.9)), uniforms=[u], logits=lg[None, :],
                              want_probs=True)
        want, want_probs = port.sample(lg, np.float32(1.0), k, np.float32(0.9), u, want_probs=True)
        assert int(got[0]) == want, (k, u, int(got[0]), want)
        assert np.array_equal(probs[0].view(np.uint32), want_probs.view(np.uint32)), k
    # the ends of the draw: u = 0 is satisfied at index 0 whatever its probability, a draw beyond the total mass
    # falls through to the last id -- with few candidates after top-k (their own code path) and with all of them
    lg = rng.standard_normal(16000, dtype=np.float32) * np.float32(2.0)
    for k in (40, 0):
        for u in (np.float32(0.0), np.float32(1.0), np.float32(1e-30)):
            sp = G.Sampling(0, np.float32(0.8), 1.0, k, np.float32(0.9))
            got, _ = s.select(sp, uniforms=[u], logits=lg[None, :], want_probs=True)
            want, _ = port.sample(lg, np.float32(0.8), k, np.float32(0.9), u, want_probs=True)
            assert int(got[0]) == want, (k, u, int(got[0]), want)


def test_penalty_and_argmax_match_oracle(G, models, port):
    rng = np.random.default_rng(5)
    s = _session_for_vocab(G, models, 5000)
    for i in range(12):
        lg = rng.standard_normal(5000, dtype=np.float32)
        hist = rng.integers(0, 5000, [6, 50, 80, 120][i % 4]).astype(np.int32)
        hist[-5:] = hist[-6]  # repeats inside the window are penalised once per occurrence
        pen = np.float32([1.2, 1.1, 1.0, 2.0][i % 4])
        s.set_history(0, hist)
        got = s.select(G.Sampling(1, 1.0, pen, 0, 1.0), logits=lg[None, :])
        want = port.argmax(port.apply_penalty(lg, hist, pen))
        assert int(got[0]) == want
    # ties: first maximum wins
    lg = np.zeros(5000, np.float32); lg[[17, 400, 4999]] = 3.0
    s.set_history(0, [])
    assert int(s.select(G.Sampling(1, 1.0, 1.0, 0, 1.0), logits=lg[None, :])[0]) == 17


@pytest.mark.parametrize("name", ["hs64_gpt2", "hs64_modern", "tiny_modern"])
def test_batched_sequences_equal_independent_sessions(name, G, models, golden, port):
    """The reference decodes one sequence per session; a batch here must equal
    that many independent reference sessions, ragged lengths included."""
    dm, path, m = models(name)
    rng = np.random.default_rng(11)
    n_seq = 5
    lens = [3, dm.max_len // 2, 1, 7, dm.max_len // 3]
    prompts = [rng.integers(0, dm.vocab, n).astype(np.int32) for n in lens]
    om = port.load(path)
    s = G.BatchSession(m, n_seq)
    got = s.prefill(prompts)
    for i, p in enumerate(prompts):
        want = port.logits_for(om, p)[-1]
        assert rel_err(got[i], want) < TOL, (i, rel_err(got[i], want))
        assert s.position(i) == len(p)
    # a step that skips some sequences leaves them untouched
    nxt = np.array([1, -1, 2, -1, 3], np.int32)
    lg = s.step(nxt)
    for i in (0, 2, 4):
        want = port.logits_for(om, list(prompts[i]) + [int(nxt[i])])[-1]
        assert rel_err(lg[i], want) < TOL
    assert [s.position(i) for i in range(n_seq)] == [4, lens[1], 2, 7, lens[4] + 1]
    # batched generate equals per-sequence oracle rollouts (greedy and sampled)
    max_new = 9
    sp = G.Sampling(1, 1.0, 1.2, 0, 1.0)
    outs = s.generate(prompts, sp, max_new)
    for i, p in enumerate(prompts):
        want = port.generate(om, p, max_new, greedy=True, penalty=1.2)
        assert np.array_equal(outs[i], want), (i, outs[i], want)
    draws = rng.random((n_seq, max_new), dtype=np.float32)
    sp = G.Sampling(0, 0.8, 1.1, 40, 0.9)
    outs = s.generate(prompts, sp, max_new, uniforms=draws)
    for i, p in enumerate(prompts):
        want = port.generate(om, p, max_new, greedy=False, temperature=0.8, penalty=1.1, top_k=40, top_p=0.9,
                             draws=draws[i])
        assert np.array_equal(outs[i], want), (i, outs[i], want)
    port.free(om)
    s.close()


def test_graph_and_eager_loops_agree(G, models, golden, monkeypatch):
    dm, path, m = models("hs64_modern")
    prompt = golden["hs64_modern/prompt"]
    a = G.TextGen(m).generate_greedy(prompt, 20, 1.2)
    monkeypatch.setenv("GRADB_NO_GRAPH", "1")
    b = G.TextGen(m).generate_greedy(prompt, 20, 1.2)
    assert np.array_equal(a, b)


def test_model_save_round_trips_bitwise(G, models, tmp_path):
    dm, path, m = models("tiny_modern")
    out = tmp_path / "saved.bin"
    assert m.save(out)
    assert out.read_bytes() == open(path, "rb").read()


@pytest.mark.parametrize("name", ["hs64_modern", "hs64_gpt2"])
def test_bf16_weight_mode_stays_close(name, G, models, golden):
    """bf16 weights (fp32 accumulate): error is reported, bounded loosely."""
    dm, path, m16 = models(name, 1)
    s = G.InferenceSession(m16)
    want = golden[f"{name}/logits"]
    got = np.stack([s.step(int(t)) for t in golden[f"{name}/tokens"]])
    err = rel_err(got, want)
    assert err < 3e-2, err


@pytest.mark.parametrize("vocab,arch", [(20011, 1), (50257, 0)])
def test_greedy_has_no_vocabulary_limit(vocab, arch, G, ck, port, tmp_path):
    """Greedy selection reads the logits from global memory and keeps only the penalty window's entries on chip,
    so vocabularies beyond one CTA's shared memory work (the reference's argmax is a plain loop,
    text_gen.cpp:52-60; its checkpoints allow 2^24 ids). The sampled stage works up to about 47000 ids (its exact
    scans run in windows) and beyond that refuses before anything is fed."""
    dm = ck.ModelDims(vocab, 128, 2, 2, 48, arch)
    path = str(ck.write_synthetic(tmp_path / "bigvocab.bin", dm, 131, 0.08, True))
    rng = np.random.default_rng(132)
    prompts = [rng.integers(0, vocab, n).astype(np.int32) for n in (5, 1, 17)]
    m = G.GPTModel.load(path)
    om = port.load(path)
    for pen in (1.0, 1.3):
        got = G.TextGen(m).generate_greedy(prompts[0], 30, pen)
        assert np.array_equal(got, port.generate(om, prompts[0], 30, greedy=True, penalty=pen)), pen
    s = G.BatchSession(m, 3)
    outs = s.generate(prompts, G.Sampling(1, 1.0, 1.3, 0, 1.0), 20)
    for p, o in zip(prompts, outs):
        assert np.array_equal(o, port.generate(om, p, 20, greedy=True, penalty=1.3))
    # argmax with ties, a NaN and a penalised maximum on caller-supplied logits
    lg = rng.standard_normal((3, vocab)).astype(np.float32)
    lg[0, 7] = lg[0, vocab - 1] = lg[0].max() + 1.0          # tie: the first index wins
    lg[1, 0] = np.nan                                          # a NaN in slot 0 stays the pick
    lg[2, 11] = lg[2].max() + 0.5                              # the maximum sits in the penalty window
    hist = [np.array([3, 5], np.int32), np.array([9], np.int32), np.array([11, 11, 4], np.int32)]
    for i, h in enumerate(hist):
        s.set_history(i, h)
    got = s.select(G.Sampling(1, 1.0, 1.7, 0, 1.0), logits=lg)
    for i, h in enumerate(hist):
        assert got[i] == port.argmax(port.apply_penalty(lg[i], h, 1.7)), i
    s.reset()
    u = rng.random((3, 4), dtype=np.float32)
    if vocab > 47000:   # the sampled stage keeps one sequence's values in one CTA's shared memory
        with pytest.raises(G.binding.GradbError) as e:
            s.generate(prompts, G.Sampling(0, 0.8, 1.0, 0, 0.9), 4, uniforms=u)
        assert "47000" in str(e.value) and all(s.position(i) == 0 for i in range(3))
    else:               # several windows of the exact scans; bit for bit on identical logits and draws
        lg = (rng.standard_normal((3, vocab)) * 1.7).astype(np.float32)
        for t, k, pp in ((0.8, 0, 0.9), (1.3, 50, 1.0), (0.7, 300, 0.95), (1.0, 0, 1.0)):
            for i in range(3):
                s.set_history(i, [])
            got, probs = s.select(G.Sampling(0, t, 1.0, k, pp), uniforms=u[:, 0], logits=lg, want_probs=True)
            for i in range(3):
                tok, want = port.sample(lg[i], t, k, pp, float(u[i, 0]), want_probs=True)
                assert got[i] == tok and np.array_equal(probs[i].view(np.uint32), want.view(np.uint32)), (t, k, pp, i)
        out = s.generate(prompts, G.Sampling(0, 0.8, 1.1, 40, 0.9), 4, uniforms=u)
        for p, o, ui in zip(prompts, out, u):
            want = port.generate(om, p, 4, greedy=False, temperature=0.8, penalty=1.1, top_k=40, top_p=0.9, draws=ui)
            assert np.array_equal(o, want)
    port.free(om)
    s.close(); m.close()
