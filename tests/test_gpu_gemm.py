"""The tensor-core GEMM (tcgen05 + TMA, csrc/kq_gemm.cuh) behind matmul! with several activation columns
(src/matmul.jl:13-23 applied column by column) against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def rel_err(got, want64):
    return float(np.abs(got - want64).max() / max(np.abs(want64).max(), 1e-30))


@pytest.mark.parametrize("t", [12, 13])
@pytest.mark.parametrize("shape,ncols", [((256, 16), 4), ((256, 130), 21), ((4096, 512), 20), ((3072, 96), 7), ((14336, 256), 41),
                                         ((8192, 384), 64), ((1024, 64), 5)])
def test_gemm_against_oracle(pkg, orc, synth, t, shape, ncols):
    """Row counts below, at and above one 128-row tile; column counts around the 20-token block; rows of one stage, of several
    column panels and of a narrower last panel (14336 = 3.5 panels)."""
    n_in, n_out = shape
    A = synth.matrix(t, n_in, n_out, seed=n_in + 7 * n_out + t)
    X = synth.normal_f32(ncols * n_in, 5 + ncols, 1.0).reshape(ncols, n_in)
    X[ncols // 2] *= 40.0          # columns of very different magnitude keep their own scales
    X[0, :256] = 0.0               # an all-zero block (the whole column when the rows are one block long)
    Y = np.full((ncols, n_out), np.nan, dtype=np.float32)
    pkg.matmul_(Y, A, X)
    assert np.isfinite(Y).all()
    for c in range(ncols):
        assert rel_err(Y[c], orc.matmul_f64(A, X[c])) < 4e-6, c


def test_gemm_is_deterministic_and_matches_the_vector_kernel(pkg, synth):
    A = synth.matrix(12, 4096, 1024, seed=3)
    X = synth.normal_f32(8 * 4096, 4, 1.0).reshape(8, 4096)
    Y1 = np.zeros((8, 1024), np.float32)
    Y2 = np.zeros((8, 1024), np.float32)
    pkg.matmul_(Y1, A, X)
    pkg.matmul_(Y2, A, X)
    assert np.array_equal(Y1, Y2)
    y = np.zeros(1024, np.float32)
    pkg.matmul_(y, A, X[3])  # one column: the matrix-vector kernel
    assert np.abs(y - Y1[3]).max() <= 2e-6 * np.abs(y).max()


def test_gemm_many_blocks_at_once_repeated(pkg, orc, synth):
    """112 row tiles resident at the same time, several times over: unpack, MMA and epilogue warps of a block run out of step
    with one another differently on every run, so anything one of them rewrites too early shows up here."""
    A = synth.matrix(12, 4096, 14336, seed=1234)
    for ncols in (4, 20, 4, 7, 4):
        X = synth.normal_f32(ncols * 4096, 78 + ncols, 1.0).reshape(ncols, 4096)
        Y = np.zeros((ncols, 14336), dtype=np.float32)
        pkg.matmul_(Y, A, X)
        for c in (0, ncols - 1):
            assert rel_err(Y[c], orc.matmul_f64(A, X[c])) < 4e-6, (ncols, c)


def test_q6_k_columns_fall_back_to_the_vector_kernel(pkg, orc, synth):
    A = synth.matrix(14, 1024, 64, seed=9)
    X = synth.normal_f32(6 * 1024, 8, 1.0).reshape(6, 1024)
    Y = np.zeros((6, 64), np.float32)
    pkg.matmul_(Y, A, X)
    for c in range(6):
        assert rel_err(Y[c], orc.matmul_f64(A, X[c])) < 4e-6


@pytest.mark.parametrize("shape", ["llama_gqa4", "phi3_neox", "long_rows"])
def test_many_token_prompt_pass_against_oracle(pkg, orc, synth, shape):
    """A 256-token prompt through the tensor-core GEMM pass (l2b_prefill / l2b_generate): the logits of the last prompt position
    and of the positions decoded afterwards (which read the KV cache the pass wrote) against the oracle, the greedy stream, and
    the same run with the pass switched off."""
    import os
    from llama2_jl_b200 import _lib as L
    if shape == "llama_gqa4":
        cfg = pkg.ModelConfig(1024, 3584, 2, 8, 2, 2048, 320, 500000.0, False)
        types = dict(synth.ALL(12), wv=13, w2=13, output=14)
    elif shape == "phi3_neox":
        cfg = pkg.ModelConfig(768, 2048, 2, 8, 8, 1024, 320, 10000.0, True)
        types = dict(synth.ALL(13), output=14)
    else:  # rows longer than one stored column panel, with a narrower last panel (18 = 16 + 2 super-blocks)
        cfg = pkg.ModelConfig(512, 4608, 2, 4, 4, 1024, 320, 10000.0, False)
        types = dict(synth.ALL(12), output=14)
    w = synth.model_weights(cfg, types, seed=31)
    n_prompt, n_pos = 256, 264
    prompt = synth.tokens(n_prompt, 77, 3, cfg.vocab_size)
    want_tokens, want_logits = orc.OracleModel(cfg, w).sample_greedy(prompt, n_pos, want_logits=True)
    model = pkg.LanguageModel(cfg, None, w)
    got, _ = pkg.generate(model, prompt, n_pos)
    assert np.array_equal(got, want_tokens), "greedy stream after a 256-token prompt differs from the oracle"
    # l2b_prefill: the logits of the last prompt position; then one decoded position on the cache the pass left behind
    st = pkg.RunState(model)
    nxt = pkg.prefill(st, prompt, 0)
    rng = float(want_logits[n_prompt - 1].max() - want_logits[n_prompt - 1].min())
    assert np.abs(st.logits - want_logits[n_prompt - 1]).max() / rng < 5e-5
    assert nxt == int(want_tokens[n_prompt - 1])
    pkg.transformer_(nxt, n_prompt, cfg, st)
    rng = float(want_logits[n_prompt].max() - want_logits[n_prompt].min())
    assert np.abs(st.logits - want_logits[n_prompt]).max() / rng < 5e-5
    model.close()
    os.environ["L2B_PREFILL_GEMM"] = "0"
    try:
        slow = pkg.LanguageModel(cfg, None, w)
        got2, _ = pkg.generate(slow, prompt, n_pos)
    finally:
        del os.environ["L2B_PREFILL_GEMM"]
    assert np.array_equal(got2, got)
    slow.close()


@pytest.mark.parametrize("classifier", [14, 12])
def test_batched_decode_matches_single_sequences(pkg, orc, synth, classifier):
    """Seven sequences with different prompts advanced in lock step (l2b_batch_decode_next): every sequence's greedy stream
    and logits equal what the same sequence gives on its own (oracle), with a q6_K and with a q4_K classifier."""
    cfg = pkg.ModelConfig(1024, 3584, 2, 8, 2, 2048, 64, 500000.0, False)
    types = dict(synth.ALL(12), wv=13, w2=13, output=classifier)
    w = synth.model_weights(cfg, types, seed=51)
    model = pkg.LanguageModel(cfg, None, w)
    n_seq, n_prompt, n_pos = 7, 5, 24
    prompts = [synth.tokens(n_prompt, 100 + i, 3, cfg.vocab_size) for i in range(n_seq)]
    oracle = orc.OracleModel(cfg, w)
    want = [oracle.sample_greedy(p, n_pos, want_logits=True) for p in prompts]
    batch = pkg.BatchRunState(model, n_seq)
    toks = np.array([p[0] for p in prompts], dtype=np.int32)
    streams = [[] for _ in range(n_seq)]
    for pos in range(n_pos):
        nxt = batch.decode_next(toks, np.full(n_seq, pos, np.int32), want_logits=True)
        for i in range(n_seq):
            wl = want[i][1][pos]
            assert np.abs(batch.logits[i] - wl).max() / float(wl.max() - wl.min()) < 5e-5, (i, pos)
            t = int(prompts[i][pos + 1]) if pos + 1 < n_prompt else int(nxt[i])
            streams[i].append(t)
            toks[i] = t
    for i in range(n_seq):
        assert streams[i] == [int(t) for t in want[i][0]], i
    # sequences may sit at different positions: restart sequence 0 alone (its cache rows are simply overwritten)
    batch.reset()
    pos_list = np.zeros(n_seq, np.int32)
    toks = np.array([p[0] for p in prompts], dtype=np.int32)
    nxt = batch.decode_next(toks, pos_list, want_logits=True)
    assert np.abs(batch.logits[3] - want[3][1][0]).max() / float(want[3][1][0].max() - want[3][1][0].min()) < 5e-5
    from llama2_jl_b200 import _lib as L
    bad = toks.copy()
    bad[2] = cfg.vocab_size
    with pytest.raises(L.L2BError):
        batch.decode_next(bad, pos_list)
    batch.close()
    model.close()
