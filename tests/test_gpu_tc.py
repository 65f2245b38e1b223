"""GPU: bf16-weight mode at batch >= 16, where every projection runs as a TMA-fed
tcgen05 GEMM with bf16 operands and fp32 accumulation. Not a bit-exact mode: the
error against the fp32 oracle is measured and bounded, and the greedy choices are
compared with the fp32 path."""
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


@pytest.mark.parametrize("name,n_seq", [("hs64_modern", 20), ("hs64_gpt2", 33), ("hs64_modern", 130)])
def test_tensor_core_path_tracks_fp32_oracle(name, n_seq, G, golden_ckpt, port):
    dm, path = golden_ckpt(name)
    rng = np.random.default_rng(21)
    lens = rng.integers(1, dm.max_len // 2, n_seq)
    prompts = [rng.integers(0, dm.vocab, int(n)).astype(np.int32) for n in lens]
    m16 = G.GPTModel.load(path, 0, G.BF16)
    s = G.BatchSession(m16, n_seq)
    got = s.prefill(prompts)
    om = port.load(path)
    worst = 0.0
    for i in range(0, n_seq, max(1, n_seq // 7)):
        want = port.logits_for(om, prompts[i])[-1]
        worst = max(worst, rel_err(got[i], want))
    assert worst < 4e-2, worst
    # one more decoded id per sequence, then logits again (exercises the cache written by the GEMM epilogue)
    nxt = rng.integers(0, dm.vocab, n_seq).astype(np.int32)
    lg = s.step(nxt)
    for i in (0, n_seq // 2, n_seq - 1):
        want = port.logits_for(om, list(prompts[i]) + [int(nxt[i])])[-1]
        assert rel_err(lg[i], want) < 4e-2, (i, rel_err(lg[i], want))
    # K and V rows written by the QKV epilogue (RoPE applied for the modern block)
    osess = port.session(om)
    for t in prompts[3]:
        port.step(osess, int(t), dm.vocab)
    for which in (0, 1):
        gotr = s.cache_row(3, 0, which, len(prompts[3]) - 1)
        wantr = port.cache_row(osess, 0, which, len(prompts[3]) - 1, dm.d_model)
        assert np.abs(gotr - wantr).max() < 2e-2 * max(np.abs(wantr).max(), 1e-6)
    port.session_free(osess)
    port.free(om)
    s.close()
    m16.close()


def test_batched_prompt_feed_over_several_chunks(G, golden_ckpt, port):
    """300 prompts of 30-40 ids are more rows than one pass of the batched prompt feed holds, so the
    feed runs in several position ranges; later ranges must land at their own cache positions."""
    dm, path = golden_ckpt("hs64_modern")
    n_seq = 300
    rng = np.random.default_rng(23)
    lens = rng.integers(30, dm.max_len, n_seq)
    prompts = [rng.integers(0, dm.vocab, int(n)).astype(np.int32) for n in lens]
    m16 = G.GPTModel.load(path, 0, G.BF16)
    s = G.BatchSession(m16, n_seq)
    got = s.prefill(prompts)
    om = port.load(path)
    for i in (0, 1, 149, 298, 299):
        want = port.logits_for(om, prompts[i])[-1]
        assert rel_err(got[i], want) < 4e-2, (i, rel_err(got[i], want))
        assert s.position(i) == len(prompts[i])
        osess = port.session(om)
        for t in prompts[i]:
            port.step(osess, int(t), dm.vocab)
        for pos in (0, 26, 27, len(prompts[i]) - 1):
            for which in (0, 1):
                gotr = s.cache_row(i, dm.layers - 1, which, pos)
                wantr = port.cache_row(osess, dm.layers - 1, which, pos, dm.d_model)
                assert np.abs(gotr - wantr).max() < 3e-2 * max(np.abs(wantr).max(), 1e-6), (i, pos, which)
        port.session_free(osess)
    port.free(om)
    s.close()
    m16.close()


@pytest.mark.parametrize("name,n_seq", [("hs64_modern", 40), ("odd_modern", 350), ("hs64_gpt2", 16)])
def test_tiled_prompt_attention_matches_per_position_attention(name, n_seq, G, golden_ckpt, monkeypatch):
    """The prompt feed's query-tiled attention (TF32 tensor-core products over tiles of 64 positions) against
    the same feed with every position streaming its prefix through the decode attention kernel (fp32)."""
    dm, path = golden_ckpt(name)
    rng = np.random.default_rng(24)
    lens = rng.integers(1, dm.max_len + 1, n_seq)
    lens[0], lens[1] = dm.max_len, 1
    prompts = [rng.integers(0, dm.vocab, int(n)).astype(np.int32) for n in lens]
    m16 = G.GPTModel.load(path, 0, G.BF16)
    a_s = G.BatchSession(m16, n_seq)
    a = a_s.prefill(prompts)
    monkeypatch.setenv("GRADB_NO_TILED_ATTN", "1")
    b_s = G.BatchSession(m16, n_seq)
    b = b_s.prefill(prompts)
    assert rel_err(a, b) < 1e-2, rel_err(a, b)
    a_s.close(); b_s.close(); m16.close()


def test_tensor_core_prompt_attention_on_long_ragged_prompts(G, ck, tmp_path, monkeypatch):
    """The same comparison at lengths that end just before, on and just after the 128-position tiles of the
    tcgen05 prompt attention (up to eight key tiles per query tile, partial last tiles, a one-id prompt), on the
    69.0M block with context 2048: last-position logits against the feed whose every position streams its prefix
    through the decode attention kernel in fp32."""
    dm = ck.PRESETS["modern2k"]
    path = str(ck.write_synthetic(tmp_path / "modern2k.bin", dm, 1005))
    rng = np.random.default_rng(25)
    lens = [1, 2, 63, 64, 127, 128, 129, 130, 255, 256, 257, 300, 383, 384, 385, 511, 512, 513, 700, 1023, 1024, 1025]
    prompts = [rng.integers(0, dm.vocab, n).astype(np.int32) for n in lens]
    m16 = G.GPTModel.load(path, 0, G.BF16)
    a_s = G.BatchSession(m16, len(lens), 1100)
    a = a_s.prefill(prompts)
    a_s.close()
    monkeypatch.setenv("GRADB_NO_TILED_ATTN", "1")
    b_s = G.BatchSession(m16, len(lens), 1100)
    b = b_s.prefill(prompts)
    b_s.close(); m16.close()
    for i, n in enumerate(lens):
        assert rel_err(a[i], b[i]) < 1e-2, (n, rel_err(a[i], b[i]))


def test_tensor_core_and_streaming_bf16_paths_agree(G, golden_ckpt, monkeypatch):
    dm, path = golden_ckpt("hs64_modern")
    rng = np.random.default_rng(22)
    prompts = [rng.integers(0, dm.vocab, 9).astype(np.int32) for _ in range(24)]
    m16 = G.GPTModel.load(path, 0, G.BF16)
    a = G.BatchSession(m16, 24).prefill(prompts)
    monkeypatch.setenv("GRADB_NO_TC", "1")
    b = G.BatchSession(m16, 24).prefill(prompts)
    assert rel_err(a, b) < 2e-2, rel_err(a, b)
    m16.close()


def test_benchmark_shape_greedy_agreement_with_fp32(G, ck, tmp_path):
    """modern 69.0M, 64 sequences: bf16 tensor-core decode against the fp32 path on the same weights."""
    dm = ck.PRESETS["modern"]
    path = str(ck.write_synthetic(tmp_path / "modern.bin", dm, 1004))
    rng = np.random.default_rng(2004)
    prompts = [rng.integers(0, dm.vocab, 32).astype(np.int32) for _ in range(64)]
    sp = G.Sampling(1, 1.0, 1.0, 0, 1.0)
    m32 = G.GPTModel.load(path, 0, G.FP32)
    s32 = G.BatchSession(m32, 64, 256)
    lg32 = s32.prefill(prompts)
    ids32 = s32.generate(prompts, sp, 16)
    s32.close(); m32.close()
    m16 = G.GPTModel.load(path, 0, G.BF16)
    s16 = G.BatchSession(m16, 64, 256)
    lg16 = s16.prefill(prompts)
    ids16 = s16.generate(prompts, sp, 16)
    s16.close(); m16.close()
    err = rel_err(lg16, lg32)
    # mean KL(fp32 || bf16) of the next-id distributions
    def logsm(x):
        x = x - x.max(axis=1, keepdims=True)
        return x - np.log(np.exp(x).sum(axis=1, keepdims=True))
    p32, p16 = logsm(lg32.astype(np.float64)), logsm(lg16.astype(np.float64))
    kl = float((np.exp(p32) * (p32 - p16)).sum(axis=1).mean())
    agree = float(np.mean([np.mean(a[32:] == b[32:]) for a, b in zip(ids32, ids16)]))
    first = float(np.mean([a[32] == b[32] for a, b in zip(ids32, ids16)]))
    print(f"bf16 vs fp32: logits max-abs/max {err:.3e}, mean KL {kl:.3e}, first-id agreement {first:.3f}, "
          f"16-id greedy agreement {agree:.3f}")
    assert err < 5e-2 and kl < 1e-3 and first > 0.9


@pytest.mark.parametrize("name,n_seq", [("hs64_modern", 20), ("hs64_gpt2", 40), ("odd_modern", 17)])
def test_fp32_mode_on_tensor_cores_keeps_fp32_parity(name, n_seq, G, golden_ckpt, port, monkeypatch):
    """fp32 sessions with >= 16 sequences run the projections as three TF32 MMAs per product (hi/lo operand
    pairs, fp32 accumulation). Bars are those of fp32 mode: logits within 1e-4 of the oracle (max-abs over
    max-abs), identical greedy ids, K/V rows within 1e-5."""
    dm, path = golden_ckpt(name)
    rng = np.random.default_rng(25)
    lens = rng.integers(1, dm.max_len // 2, n_seq)
    prompts = [rng.integers(0, dm.vocab, int(n)).astype(np.int32) for n in lens]
    m = G.GPTModel.load(path, 0, G.FP32)
    s = G.BatchSession(m, n_seq)
    got = s.prefill(prompts)
    om = port.load(path)
    worst = max(rel_err(got[i], port.logits_for(om, prompts[i])[-1]) for i in range(n_seq))
    assert worst < 1e-4, worst
    osess = port.session(om)
    for t in prompts[2]:
        port.step(osess, int(t), dm.vocab)
    for which in (0, 1):
        gotr = s.cache_row(2, dm.layers - 1, which, len(prompts[2]) - 1)
        wantr = port.cache_row(osess, dm.layers - 1, which, len(prompts[2]) - 1, dm.d_model)
        assert np.abs(gotr - wantr).max() < 1e-5 * max(np.abs(wantr).max(), 1.0)
    port.session_free(osess)
    sp = G.Sampling(1, 1.0, 1.2, 0, 1.0)
    n_new = dm.max_len // 2
    ids = s.generate(prompts, sp, n_new)
    for i in (0, n_seq // 2, n_seq - 1):
        assert list(ids[i]) == list(port.generate(om, prompts[i], n_new, greedy=True, penalty=1.2)), i
    # and against the streaming fp32 kernels on the same session shape
    monkeypatch.setenv("GRADB_NO_TC32", "1")
    s2 = G.BatchSession(m, n_seq)
    assert rel_err(got, s2.prefill(prompts)) < 2e-5
    port.free(om)
    s.close(); s2.close(); m.close()


def test_many_row_gemm_kernel_on_the_gpt2_block(G, ck, port, tmp_path, monkeypatch):
    """`medium` (GPT-2 block: LayerNorm, biases, GELU 3072, learned positions), 64 prompts of 64 ids in bf16
    mode: 4096 rows per projection put the prompt feed on the persistent many-tile GEMM kernel. Checked against
    the one-tile-per-CTA kernel on the same rows and, for one sequence, against the fp32 oracle."""
    dm = ck.PRESETS["medium"]
    path = str(ck.write_synthetic(tmp_path / "medium.bin", dm, 1003))
    rng = np.random.default_rng(26)
    prompts = [rng.integers(0, dm.vocab, 64).astype(np.int32) for _ in range(64)]
    m16 = G.GPTModel.load(path, 0, G.BF16)
    a_s = G.BatchSession(m16, 64, 128)
    a = a_s.prefill(prompts)
    rows_a = [a_s.cache_row(5, dm.layers - 1, which, 63) for which in (0, 1)]
    monkeypatch.setenv("GRADB_NO_WIDE_GEMM", "1")
    b_s = G.BatchSession(m16, 64, 128)
    b = b_s.prefill(prompts)
    rows_b = [b_s.cache_row(5, dm.layers - 1, which, 63) for which in (0, 1)]
    assert rel_err(a, b) < 1e-2, rel_err(a, b)
    for x, y in zip(rows_a, rows_b):
        assert np.abs(x - y).max() < 1e-2 * max(np.abs(y).max(), 1e-6)
    om = port.load(path)
    want = port.logits_for(om, prompts[5][:24])[-1]
    port.free(om)
    c_s = G.BatchSession(m16, 64, 128)
    monkeypatch.delenv("GRADB_NO_WIDE_GEMM")
    c = c_s.prefill([p[:24] for p in prompts])
    assert rel_err(c[5], want) < 4e-2, rel_err(c[5], want)
    a_s.close(); b_s.close(); c_s.close(); m16.close()


@pytest.mark.parametrize("arch", [0, 1])
def test_tensor_core_paths_with_head_size_32(arch, G, ck, port, tmp_path):
    """d_model 128 with 4 heads: the projections take the tensor-core kernels (bf16, and fp32 as TF32 pairs) while
    attention runs on the generic kernel and prompts are fed position by position (the batched feed and the
    pipelined attention kernel are for head size 64)."""
    dm = ck.ModelDims(301, 128, 2, 4, 40, arch)
    path = str(ck.write_synthetic(tmp_path / "hs32.bin", dm, 107, 0.08, True))
    rng = np.random.default_rng(27)
    n_seq = 20
    prompts = [rng.integers(0, dm.vocab, int(n)).astype(np.int32) for n in rng.integers(1, 18, n_seq)]
    om = port.load(path)
    want = [port.logits_for(om, p)[-1] for p in prompts]
    for prec, tol in ((G.FP32, 1e-4), (G.BF16, 4e-2)):
        m = G.GPTModel.load(path, 0, prec)
        s = G.BatchSession(m, n_seq)
        got = s.prefill(prompts)
        worst = max(rel_err(got[i], want[i]) for i in range(n_seq))
        assert worst < tol, (prec, worst)
        if prec == G.FP32:
            ids = s.generate(prompts, G.Sampling(1, 1.0, 1.0, 0, 1.0), 12)
            for i in (0, 7, 19):
                assert list(ids[i]) == list(port.generate(om, prompts[i], 12, greedy=True, penalty=1.0)), i
        s.close(); m.close()
    port.free(om)


@pytest.mark.parametrize("precision", ["fp32", "bf16"])
def test_batched_generation_with_empty_full_and_ragged_prompts(precision, G, golden_ckpt, port):
    """Edge cases of the batched prompt feed inside generate: an empty prompt (nothing is generated, text_gen.cpp:40),
    a one-id prompt, a prompt that fills the context (one id is still emitted, text_gen.cpp:61-63), and a stop when the
    context fills mid-way. fp32 sequences must equal the oracle's; bf16 sequences must have the oracle's lengths."""
    dm, path = golden_ckpt("hs64_modern")
    rng = np.random.default_rng(28)
    lens = [0, 1, dm.max_len, dm.max_len - 3, 7] + [int(x) for x in rng.integers(1, dm.max_len, 19)]
    prompts = [rng.integers(0, dm.vocab, n).astype(np.int32) for n in lens]
    n_new = 9
    m = G.GPTModel.load(path, 0, G.FP32 if precision == "fp32" else G.BF16)
    s = G.BatchSession(m, len(prompts))
    ids = s.generate(prompts, G.Sampling(1, 1.0, 1.2, 0, 1.0), n_new)
    om = port.load(path)
    for i, p in enumerate(prompts):
        want = port.generate(om, p, n_new, greedy=True, penalty=1.2) if len(p) else np.zeros(0, np.int32)
        assert len(ids[i]) == len(want), (i, len(p), len(ids[i]), len(want))
        assert list(ids[i][:len(p)]) == list(p)
        if precision == "fp32":
            assert list(ids[i]) == list(want), i
    port.free(om)
    s.close(); m.close()
