"""GPU: streaming generation and the serving calls (slots admitted, decoded and vacated independently),
through the C ABI. Every sequence must come out exactly as an independent reference rollout of its prompt
(TextGen::generate_greedy / generate_sample, text_gen.cpp:37-120), whatever its neighbours do."""
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G(pkg):
    import grad_cpp_b200 as g
    g.lib()
    return g


@pytest.mark.parametrize("name", ["hs64_modern", "tiny_gpt2"])
def test_stream_hands_out_each_id_as_it_is_chosen(name, G, golden_ckpt, port):
    dm, path = golden_ckpt(name)
    rng = np.random.default_rng(41)
    prompt = rng.integers(0, dm.vocab, 5).astype(np.int32)
    n_new = dm.max_len - 5 - 2
    draws = rng.random(n_new, dtype=np.float32)
    m = G.GPTModel.load(path)
    om = port.load(path)
    want = port.generate(om, prompt, n_new, greedy=False, temperature=0.8, penalty=1.1, top_k=5, top_p=0.9, draws=draws)
    s = G.BatchSession(m, 1)
    got, asked, order = [], [], []

    def draw(seq):
        asked.append(len(got))   # ids already handed out when this draw is requested
        order.append("d")
        return draws[len(asked) - 1]

    def on_token(seq, index, token):
        assert seq == 0 and index == len(got)
        got.append(token)
        order.append("t")
        return False

    n = s.generate_stream([prompt], G.Sampling(0, 0.8, 1.1, 5, 0.9), n_new, on_token, draw)
    assert n[0] == n_new and got == list(want[5:])
    # one draw per id, each requested only after the previous id was delivered (text_gen.cpp:107-116)
    assert asked == list(range(n_new)) and "".join(order) == "dt" * n_new
    assert s.position(0) == 5 + n_new - 1

    # a callback that ends the sequence: no further ids, no further draws
    got.clear(); asked.clear(); order.clear()
    n = s.generate_stream([prompt], G.Sampling(0, 0.8, 1.1, 5, 0.9), n_new,
                          lambda seq, i, t: (got.append(t), order.append("t"), i == 3)[2], draw)
    assert n[0] == 4 and got == list(want[5:9]) and len(asked) == 4
    # an exception in the callback comes back out after the loop has been stopped
    def boom(seq, i, t):
        raise KeyError("stop here")
    with pytest.raises(KeyError):
        s.generate_stream([prompt], G.Sampling(1, 1.0, 1.2, 0, 1.0), 6, boom)
    # the session still works: greedy, context-filling prompt emits exactly one id
    full = rng.integers(0, dm.vocab, dm.max_len).astype(np.int32)
    got.clear()
    n = s.generate_stream([full], G.Sampling(1, 1.0, 1.2, 0, 1.0), 6, lambda seq, i, t: got.append(t) or False)
    assert n[0] == 1 and got == list(port.generate(om, full, 6, greedy=True, penalty=1.2)[dm.max_len:])
    assert s.generate_stream([np.zeros(0, np.int32)], G.Sampling(1, 1.0, 1.2, 0, 1.0), 6, boom)[0] == 0
    port.free(om)
    s.close(); m.close()


def test_first_id_arrives_long_before_the_last(G, ck, tmp_path):
    """Time to the first id is the prompt feed plus one selection, not the whole generation."""
    dm = ck.PRESETS["modern"]
    path = str(ck.write_synthetic(tmp_path / "modern.bin", dm, 1002))
    prompt = np.random.default_rng(42).integers(0, dm.vocab, 32).astype(np.int32)
    m = G.GPTModel.load(path)
    s = G.BatchSession(m, 1)
    stamps = []
    sp = G.Sampling(1, 1.0, 1.2, 0, 1.0)
    s.generate_stream([prompt], sp, 8, lambda seq, i, t: False)  # warm-up
    t0 = time.perf_counter()
    n = s.generate_stream([prompt], sp, 200, lambda seq, i, t: stamps.append(time.perf_counter() - t0) or False)
    total = time.perf_counter() - t0
    assert n[0] == 200 and len(stamps) == 200
    print(f"first id after {stamps[0] * 1e3:.2f} ms, last after {stamps[-1] * 1e3:.2f} ms, call {total * 1e3:.2f} ms")
    assert stamps[0] < 0.25 * stamps[-1]
    assert all(b >= a for a, b in zip(stamps, stamps[1:]))
    s.close(); m.close()


def test_batched_stream_equals_batched_generate(G, golden_ckpt):
    dm, path = golden_ckpt("hs64_modern")
    rng = np.random.default_rng(43)
    prompts = [rng.integers(0, dm.vocab, int(n)).astype(np.int32) for n in rng.integers(1, 20, 18)]
    m = G.GPTModel.load(path)
    s = G.BatchSession(m, 18)
    sp = G.Sampling(1, 1.0, 1.2, 0, 1.0)
    want = s.generate(prompts, sp, 12)
    got = [list(p) for p in prompts]
    n = s.generate_stream(prompts, sp, 12, lambda seq, i, t: got[seq].append(t) or False)
    for b in range(18):
        assert got[b] == list(want[b]) and n[b] == len(want[b]) - len(prompts[b])
    s.close(); m.close()


@pytest.mark.parametrize("name,n_slots,precision", [("hs64_modern", 6, "fp32"), ("hs64_gpt2", 20, "fp32"),
                                                    ("hs64_modern", 24, "bf16")])
def test_slots_admitted_between_decode_steps_equal_independent_rollouts(name, n_slots, precision, G, golden_ckpt, port):
    """A queue of prompts with different lengths and limits runs through a few slots: whenever slots finish, new
    prompts are admitted into them while the others keep decoding. fp32: every sequence equals the oracle's
    independent rollout; bf16: lengths equal and sequences equal those of one batched generate call."""
    dm, path = golden_ckpt(name)
    rng = np.random.default_rng(44)
    n_jobs = 3 * n_slots + 2
    prompts = [rng.integers(0, dm.vocab, int(n)).astype(np.int32) for n in rng.integers(1, dm.max_len - 4, n_jobs)]
    limits = [int(x) for x in rng.integers(1, 14, n_jobs)]
    sp = G.Sampling(1, 1.0, 1.2, 0, 1.0)
    m = G.GPTModel.load(path, 0, G.FP32 if precision == "fp32" else G.BF16)
    s = G.BatchSession(m, n_slots)
    slot_job = [-1] * n_slots
    out = [None] * n_jobs
    queue = list(range(n_jobs))
    while queue or any(j >= 0 for j in slot_job):
        free = [b for b in range(n_slots) if slot_job[b] < 0]
        take = [queue.pop(0) for _ in range(min(len(free), len(queue)))]
        if take:
            s.admit(free[:len(take)], [prompts[j] for j in take], [limits[j] for j in take])
            for b, j in zip(free, take):
                slot_job[b] = j
                out[j] = list(prompts[j])
        new, fin = s.decode(sp, 3)
        for b in range(n_slots):
            j = slot_job[b]
            if j < 0:
                assert len(new[b]) == 0
                continue
            out[j] += list(new[b])
            if fin[b]:
                assert list(s.slot_ids(b)) == out[j]
                slot_job[b] = -1
    if precision == "fp32":
        om = port.load(path)
        for j in range(n_jobs):
            want = port.generate(om, prompts[j], limits[j], greedy=True, penalty=1.2)
            assert out[j] == list(want), (j, len(prompts[j]), limits[j])
        port.free(om)
    else:
        ref = G.BatchSession(m, n_jobs)
        for j in range(n_jobs):
            want = ref.generate([prompts[j]], sp, limits[j])[0]
            assert len(out[j]) == len(want), j
        ref.close()
    s.close(); m.close()


def test_sampled_slots_stop_ids_and_prefix_reuse(G, golden_ckpt, port):
    dm, path = golden_ckpt("hs64_modern")
    rng = np.random.default_rng(45)
    m = G.GPTModel.load(path)
    om = port.load(path)
    s = G.BatchSession(m, 4)
    sp = G.Sampling(0, 0.9, 1.1, 8, 0.95)
    prompts = [rng.integers(0, dm.vocab, n).astype(np.int32) for n in (6, 3, 9, 1)]
    draws = [rng.random(12, dtype=np.float32) for _ in range(4)]
    s.admit([2, 0, 3, 1], prompts, 12, uniforms=draws)
    new, fin = s.decode(sp, 12)
    for slot, p, u in zip([2, 0, 3, 1], prompts, draws):
        want = port.generate(om, p, 12, greedy=False, temperature=0.9, penalty=1.1, top_k=8, top_p=0.95, draws=u)
        assert list(new[slot]) == list(want[len(p):]) and fin[slot]
    # a stop id ends its sequence when chosen (and is emitted); the others run on
    full = port.generate(om, prompts[0], 12, greedy=True, penalty=1.2)
    stop = int(full[len(prompts[0]) + 4])
    first_hit = next(i for i, t in enumerate(full[len(prompts[0]):]) if t == stop)
    s.admit([0, 1], [prompts[0], prompts[1]], 12)
    new, fin = s.decode(G.Sampling(1, 1.0, 1.2, 0, 1.0), 12, stop_ids=[stop, dm.vocab + 5])
    assert list(new[0]) == list(full[len(prompts[0]):len(prompts[0]) + first_hit + 1]) and fin[0]
    other = port.generate(om, prompts[1], 12, greedy=True, penalty=1.2)[len(prompts[1]):]
    cut = next((i for i, t in enumerate(other) if t == stop), len(other) - 1)
    assert list(new[1]) == list(other[:cut + 1])
    # a follow-up prompt that repeats the slot's sequence keeps those cache positions
    base = port.generate(om, prompts[2], 10, greedy=True, penalty=1.2)
    s.admit([3], [prompts[2]], 10)
    new, _ = s.decode(G.Sampling(1, 1.0, 1.2, 0, 1.0), 10)
    assert list(new[3]) == list(base[len(prompts[2]):])
    follow = np.concatenate([base, rng.integers(0, dm.vocab, 4).astype(np.int32)])
    reused = s.admit([3], [follow], 6, reuse_prefix=True)
    assert reused[0] == len(base) - 1      # every position that holds K/V: the last emitted id was never fed
    new, fin = s.decode(G.Sampling(1, 1.0, 1.2, 0, 1.0), 6)
    assert list(new[3]) == list(port.generate(om, follow, 6, greedy=True, penalty=1.2)[len(follow):]) and fin[3]
    # a prompt that shares only a few ids keeps just those
    other = follow.copy(); other[4] = (other[4] + 1) % dm.vocab
    assert s.admit([3], [other[:12]], 3, reuse_prefix=True)[0] == 4
    new, _ = s.decode(G.Sampling(1, 1.0, 1.2, 0, 1.0), 3)
    assert list(new[3]) == list(port.generate(om, other[:12], 3, greedy=True, penalty=1.2)[12:])
    # errors leave the slots alone
    with pytest.raises(IndexError):
        s.admit([1], [np.array([dm.vocab], np.int32)], 3)
    with pytest.raises(RuntimeError):
        s.admit([1], [np.zeros(dm.max_len + 1, np.int32)], 3)
    port.free(om)
    s.close(); m.close()


def test_bf16_prefix_reuse_feeds_from_a_position_inside_a_tile(G, ck, tmp_path):
    """bf16 sessions run prompt attention on the tensor-core kernel; a follow-up prompt that keeps 150 cached
    positions makes its query tile start at position 150 (not a multiple of the 128-position tile) with 100 rows.
    The K/V rows the feed writes in the last layer (which depend on every layer's attention output) must equal
    those of a fresh feed of the whole prompt up to bf16 rounding, and the greedy continuation must agree."""
    dm = ck.PRESETS["modern"]
    path = str(ck.write_synthetic(tmp_path / "modern.bin", dm, 1002))
    rng = np.random.default_rng(46)
    long = rng.integers(0, dm.vocab, 250).astype(np.int32)
    others = [rng.integers(0, dm.vocab, int(n)).astype(np.int32) for n in rng.integers(20, 200, 17)]
    greedy = G.Sampling(1, 1.0, 1.2, 0, 1.0)
    m = G.GPTModel.load(path, 0, G.BF16)
    a = G.BatchSession(m, 18, 256)
    a.admit([5], [long[:150]], 1)
    a.decode(greedy, 1)                      # slot 5 now holds the 150 prompt positions (the emitted id was never fed)
    reused = a.admit([5] + [i for i in range(18) if i != 5], [long] + others, 4, reuse_prefix=True)
    assert reused[0] == 150 and all(r == 0 for r in reused[1:])
    b = G.BatchSession(m, 18, 256)
    b.admit([5] + [i for i in range(18) if i != 5], [long] + others, 4)
    for pos in (0, 149, 150, 200, 249):
        for which in (0, 1):
            ra, rb = a.cache_row(5, dm.layers - 1, which, pos), b.cache_row(5, dm.layers - 1, which, pos)
            assert np.abs(ra - rb).max() <= 2e-2 * max(np.abs(rb).max(), 1e-6), (pos, which)
    na, _ = a.decode(greedy, 4)
    nb, _ = b.decode(greedy, 4)
    assert list(na[5]) == list(nb[5])
    a.close(); b.close(); m.close()
