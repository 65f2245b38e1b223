"""GPU: the cached-attention kernel on its own, against a float64 restatement of the
reference loop (inference.cpp:208-225): ragged contexts, context 1, the last slot of
the cache, more splits than 32-position tiles."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def reference_attention(q, K, V, pos):
    """Per sequence and head: scores over positions 0..pos, softmax, weighted sum of V rows."""
    n_seq, H, T, hs = K.shape
    out = np.zeros((n_seq, H * hs))
    for s in range(n_seq):
        ctx = int(pos[s]) + 1
        for h in range(H):
            qh = q[s, h * hs:(h + 1) * hs].astype(np.float64)
            sc = K[s, h, :ctx].astype(np.float64) @ qh / np.sqrt(hs)
            sc = np.exp(sc - sc.max())
            sc /= sc.sum()
            out[s, h * hs:(h + 1) * hs] = sc @ V[s, h, :ctx].astype(np.float64)
    return out


@pytest.fixture(scope="module")
def B(pkg):
    from grad_cpp_b200 import binding
    binding.lib()
    return binding


@pytest.mark.parametrize("n_seq,heads,max_len,splits,positions", [
    (1, 12, 256, 8, [255]),
    (3, 2, 64, 1, [0, 31, 63]),
    (5, 3, 300, 4, [0, 1, 32, 150, 299]),
    (2, 12, 2048, 16, [2047, 1000]),
    (4, 1, 40, 16, [5, 39, 0, 17]),       # more splits than tiles: some ranges are empty
])
def test_attention_matches_reference_loop(B, n_seq, heads, max_len, splits, positions):
    rng = np.random.default_rng(n_seq * 1000 + max_len)
    q = rng.standard_normal((n_seq, heads * 64)).astype(np.float32)
    K = rng.standard_normal((n_seq, heads, max_len, 64)).astype(np.float32)
    V = rng.standard_normal((n_seq, heads, max_len, 64)).astype(np.float32)
    pos = np.array(positions, np.int32)
    dq, dK, dV = (torch.from_numpy(a).cuda() for a in (q, K, V))
    dpos = torch.from_numpy(pos).cuda()
    out = torch.zeros(n_seq, heads * 64, device="cuda")
    B.attention_decode(dq, dK, dV, dpos, max_len, splits, out)
    want = reference_attention(q, K, V, pos)
    got = out.cpu().numpy()
    assert np.abs(got - want).max() < 1e-5 * max(1.0, np.abs(want).max()), np.abs(got - want).max()


def test_attention_rejects_unsupported_shapes(B):
    t = torch.zeros(1, 32, device="cuda")
    p = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(B.GradbError):
        B.lib().gradb_attention_decode  # symbol exists
        B._check(B.lib().gradb_attention_decode(t.data_ptr(), t.data_ptr(), t.data_ptr(), p.data_ptr(), 1, 1, 32, 1, 1,
                                                t.data_ptr(), 0))
