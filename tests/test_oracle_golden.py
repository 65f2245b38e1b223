"""CPU: the plain-C restatement against fixtures produced by the reference itself.

The reference's own test for this path (tests/integration/sanity_tests.cpp:293-333)
compares two live computations with tolerance 1e-3 + 1e-3(|a|+|b|); here the
restatement is held to 1e-4 relative against recorded reference logits, and the
selection stage (penalty, argmax, top-k, top-p, draw) to exact token equality.
"""
import zlib

import numpy as np
import pytest

from conftest import GOLDEN_MODELS, sampler_logits

MODELS = list(GOLDEN_MODELS)


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


@pytest.mark.parametrize("name", MODELS)
def test_logits_match_reference(name, port, port64, golden, golden_ckpt):
    dm, path = golden_ckpt(name)
    m = port.load(path)
    got = port.logits_for(m, golden[f"{name}/tokens"])
    want = golden[f"{name}/logits"]
    assert got.shape == want.shape
    assert rel_err(got, want) < 1e-4, rel_err(got, want)
    # The double-precision witness agrees with both, so neither is drifting.
    m64 = port64.load(path)
    wit = port64.logits_for(m64, golden[f"{name}/tokens"])
    assert rel_err(wit, want) < 1e-4
    port.free(m)
    port64.free(m64)


@pytest.mark.parametrize("name", MODELS)
def test_greedy_rollouts_match_reference(name, port, golden, golden_ckpt):
    dm, path = golden_ckpt(name)
    m = port.load(path)
    prompt = golden[f"{name}/prompt"]
    for pen, key in ((1.0, "greedy_p1.0"), (1.2, "greedy_p1.2")):
        got = port.generate(m, prompt, dm.max_len, greedy=True, penalty=pen)
        want = golden[f"{name}/{key}"]
        # the rollout stops when the context is full, with the last id still emitted
        assert len(want) == dm.max_len + 1
        assert np.array_equal(got, want), (pen, got, want)
    got = port.generate(m, prompt, 3, greedy=True, penalty=1.2)
    assert np.array_equal(got, golden[f"{name}/greedy_short"])
    port.free(m)


@pytest.mark.parametrize("name", MODELS)
def test_sampled_rollouts_match_reference(name, port, golden, golden_ckpt):
    dm, path = golden_ckpt(name)
    m = port.load(path)
    prompt = golden[f"{name}/prompt"]
    for tag in "abc":
        t, pen, k, p = golden[f"{name}/sample_{tag}_params"]
        draws = golden[f"{name}/sample_{tag}_draws"]
        want = golden[f"{name}/sample_{tag}_ids"]
        got = port.generate(m, prompt, dm.max_len, greedy=False, temperature=float(t), penalty=float(pen),
                            top_k=int(k), top_p=float(p), draws=draws)
        assert np.array_equal(got, want), (tag, got, want)
    # generate_stream reports only the new ids, same selection rule
    want = golden[f"{name}/stream_ids"]
    got = port.generate(m, prompt, 6, greedy=False, temperature=0.9, penalty=1.2, top_k=0, top_p=0.95,
                        draws=golden[f"{name}/stream_draws"])
    assert np.array_equal(got[len(prompt):], want)
    port.free(m)


@pytest.mark.parametrize("name", MODELS[:2])
def test_error_codes_match_reference(name, port, golden, golden_ckpt):
    dm, path = golden_ckpt(name)
    m = port.load(path)
    s = port.session(m)
    rc_bad = port.step(s, dm.vocab, dm.vocab)[0]
    rc_neg = port.step(s, -1, dm.vocab)[0]
    for t in golden[f"{name}/tokens"]:
        assert port.step(s, int(t), dm.vocab)[0] == 0
    rc_full = port.step(s, 0, dm.vocab)[0]
    assert [rc_bad, rc_neg, rc_full] == list(golden[f"{name}/error_codes"]) == [2, 2, 1]
    port.session_free(s)
    port.free(m)


def test_sampler_matches_reference_bit_for_bit(port, golden):
    cases = golden["sampler/cases"]
    assert len(cases) >= 400
    for seed, vocab, scale, quantum, t, k, p, u, tok, crc in cases:
        lg = sampler_logits(seed, vocab, np.float32(scale), np.float32(quantum))
        assert zlib.crc32(lg.tobytes()) == int(crc), "seeded logits no longer reproduce the fixture"
        got = port.sample(lg, np.float32(t), int(k), np.float32(p), np.float32(u))
        assert got == int(tok), (seed, t, k, p, u, got, tok)


def test_sampler_quirks(port):
    """Behaviours of text_gen.cpp:135-209 that a tidy rewrite would lose."""
    lg = np.array([1.0, 3.0, 3.0, 2.0, -1.0], np.float32)
    # top-k keeps ties at the threshold: k=1 with two maxima keeps both
    _, pr = port.sample(lg, 1.0, 1, 1.0, 0.1, want_probs=True)
    assert (pr > 0).sum() == 2 and pr[1] == pr[2] == 0.5
    # p = 0 -> cutoff index 0 -> only the maximum (and its ties) survive
    _, pr = port.sample(lg, 1.0, 0, 0.0, 0.9, want_probs=True)
    assert (pr > 0).sum() == 2
    # draw above the total mass falls through to the last id
    tok = port.sample(np.array([0.0, 0.0], np.float32), 1.0, 0, 1.0, 1.0)
    assert tok in (1,)
    # penalty is applied once per occurrence within the last 50 ids
    out = port.apply_penalty(np.array([2.0, -2.0, 1.0], np.float32), [0, 0, 1], 2.0)
    assert list(out) == [0.5, -4.0, 1.0]
    ids = [2] * 10 + [0] * 50  # the 2s fall outside the window
    out = port.apply_penalty(np.array([1.0, 1.0, 1.0], np.float32), ids, 2.0)
    assert out[2] == 1.0 and out[0] == np.float32(1.0) / np.float32(2.0) ** 50
    # argmax: first index among equal maxima; NaN never wins
    assert port.argmax(np.array([1.0, 5.0, 5.0], np.float32)) == 1
    assert port.argmax(np.array([1.0, np.nan, 0.5], np.float32)) == 0
