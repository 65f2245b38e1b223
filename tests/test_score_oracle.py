"""Teacher-forced scoring (`grad eval`'s mean loss): the CPU restatement against values the
reference itself produced (tests/golden/score_golden.npz)."""
import numpy as np
import pytest

from conftest import GOLDEN_MODELS, ROOT

# The reference scores through its full-sequence forward (batched BLAS products) and a SIMD exp;
# the restatement scores through the step path and libm. Both are fp32, so they agree to rounding.
ROW_TOL = 2e-4   # absolute, on log-probabilities of magnitude 2..9
LOSS_TOL = 2e-5  # relative, on batch losses and the mean


@pytest.fixture(scope="module")
def score_golden():
    return np.load(ROOT / "tests" / "golden" / "score_golden.npz")


@pytest.mark.parametrize("name", list(GOLDEN_MODELS))
def test_port_mean_loss_matches_reference(name, port, port64, golden_ckpt, score_golden):
    dm, path = golden_ckpt(name)
    g = score_golden
    inp, tgt = g[f"{name}/inputs"], g[f"{name}/targets"]
    bw = int(g[f"{name}/batch_windows"][0])
    for P in (port, port64):
        m = P.load(path)
        mean, batch, logp = P.mean_loss(m, inp, tgt, bw)
        P.free(m)
        np.testing.assert_allclose(logp, g[f"{name}/row_logp"], rtol=0, atol=ROW_TOL)
        np.testing.assert_allclose(batch, g[f"{name}/batch_loss"], rtol=LOSS_TOL)
        assert abs(mean - float(g[f"{name}/mean"][0])) <= LOSS_TOL * abs(mean)


def test_out_of_vocabulary_targets_contribute_nothing(port, golden_ckpt, score_golden):
    dm, path = golden_ckpt("tiny_modern")
    g = score_golden
    tgt = g["tiny_modern/targets"]
    assert tgt[1, 3] == dm.vocab and tgt[4, 0] == -1
    assert g["tiny_modern/row_logp"][1, 3] == 0.0 and g["tiny_modern/row_logp"][4, 0] == 0.0
    m = port.load(path)
    _, batch, logp = port.mean_loss(m, g["tiny_modern/inputs"], tgt, 2)
    port.free(m)
    assert logp[1, 3] == 0.0 and logp[4, 0] == 0.0
    # the divisor is still the full row count (variable.cpp:553)
    S = tgt.shape[1]
    assert abs(batch[0] - (-logp[0:2].sum() / (2 * S))) < 1e-5
