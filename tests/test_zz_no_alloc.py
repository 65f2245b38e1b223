"""GPU: the allocation-free attention entry point against the regular one.

Some callers of this library cannot allocate device memory at the moment they need attention:
hosts that hand a plugin a fixed device-memory budget at start-up, and latency-critical loops
for which cudaMalloc's unbounded blocking and cudaFree's device-wide synchronisation are not
acceptable. For them `gradb_attention_decode_static` keeps its scratch in a fixed device array.
This file is collected last on purpose: if it fails, a run that stops at the first failure has
already run every other test. It checks two calls in a row (the second with smaller shapes, so
stale scratch from the first would show), the size limit, and nothing else.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def B(pkg):
    from grad_cpp_b200 import binding
    binding.lib()
    return binding


def _case(B, seed, n_seq, heads, max_len, splits, positions):
    rng = np.random.default_rng(seed)
    q = torch.from_numpy(rng.standard_normal((n_seq, heads * 64)).astype(np.float32)).cuda()
    K = torch.from_numpy(rng.standard_normal((n_seq, heads, max_len, 64)).astype(np.float32)).cuda()
    V = torch.from_numpy(rng.standard_normal((n_seq, heads, max_len, 64)).astype(np.float32)).cuda()
    pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
    want = torch.zeros(n_seq, heads * 64, device="cuda")
    got = torch.full((n_seq, heads * 64), float("nan"), device="cuda")
    B.attention_decode(q, K, V, pos, max_len, splits, want)
    B.attention_decode(q, K, V, pos, max_len, splits, got, fn="gradb_attention_decode_static")
    torch.cuda.synchronize()
    w, g = want.cpu().numpy(), got.cpu().numpy()
    assert np.isfinite(g).all()
    # same tolerance as the stand-alone attention test uses against its reference loop
    assert np.abs(g - w).max() < 1e-5 * max(1.0, np.abs(w).max()), np.abs(g - w).max()


def test_static_scratch_attention_matches_regular_entry_point_twice(B):
    _case(B, 1, 6, 12, 512, 16, [511, 300, 17, 0, 255, 64])   # 1152 of the 4096 slots
    _case(B, 2, 3, 2, 96, 2, [95, 1, 40])                      # smaller: stale partials must not leak in


def test_static_scratch_limit_is_enforced(B):
    cap = B.lib().gradb_attention_static_capacity()
    assert cap == 4096
    t = torch.zeros(1, 64, device="cuda")
    p = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(B.GradbError, match="exceeds the fixed scratch of 4096"):
        B._check(B.lib().gradb_attention_decode_static(t.data_ptr(), t.data_ptr(), t.data_ptr(), p.data_ptr(),
                                                       100, 12, 64, 8, 4, t.data_ptr(), 0))
