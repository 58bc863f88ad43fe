"""CPU checks of the host side: the C ABI library loads and exports what the header declares, argument and
no-device errors, the seeded generators, tokenizers and the two file loaders."""
import ctypes as C
import os
import re
import struct

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(pkg):
    from llama2_jl_b200 import _lib as L
    header = open(os.path.join(ROOT, "include", "llama2_b200.h")).read()
    declared = sorted(set(re.findall(r"\b(l2b_[a-z0-9_]+)\s*\(", header)))
    assert declared == L.exported_symbols()
    lib = L.lib()
    for name in declared:
        assert getattr(lib, name) is not None
    synth_header = open(os.path.join(ROOT, "include", "l2b_synth.h")).read()
    synth_declared = sorted(set(re.findall(r"\b(l2b_[a-z0-9_]+)\s*\(", synth_header)))
    assert synth_declared == sorted(L._SYNTH_SIGNATURES)
    for name in synth_declared:
        assert getattr(L.synth_lib(), name) is not None
        assert not hasattr(lib, name), "the synthetic-data generators are test support and stay out of the product library"
    assert lib.l2b_version() >= 100
    assert lib.l2b_status_string(L.ERR_TIMEOUT).decode() == "device-side wait timed out"


def test_no_device_means_error_not_fallback(pkg):
    import torch
    from llama2_jl_b200 import _lib as L
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    n = C.c_int32(-1)
    L.check(L.lib().l2b_device_count(C.byref(n)))
    assert n.value == 0
    x = np.zeros(256, dtype=np.float32)
    assert L.lib().l2b_rmsnorm(L.ptr(x), L.ptr(x), L.ptr(x), 256) == L.ERR_NO_DEVICE
    raw = np.zeros(144, dtype=np.uint8)
    assert L.lib().l2b_dequantize(12, L.ptr(raw), 256, L.ptr(x)) == L.ERR_NO_DEVICE
    with pytest.raises(L.L2BError) as e:
        pkg.matmul_(np.zeros(2, np.float32), np.zeros((2, 8), np.float32), np.zeros(8, np.float32))
    assert e.value.status == L.ERR_NO_DEVICE and "no CPU path" in str(e.value)
    cfg = L.Config(dim=64, hidden_dim=96, n_layers=1, n_heads=4, n_kv_heads=4, vocab_size=66, seq_len=16, rope_freq_base=1e4)
    m = C.c_void_p()
    assert L.lib().l2b_model_create(C.byref(cfg), C.byref(m)) == L.ERR_NO_DEVICE


def test_config_validation(pkg):
    from llama2_jl_b200 import _lib as L
    m = C.c_void_p()
    bad = L.Config(dim=65, hidden_dim=96, n_layers=1, n_heads=4, n_kv_heads=4, vocab_size=66, seq_len=16, rope_freq_base=1e4)
    assert L.lib().l2b_model_create(C.byref(bad), C.byref(m)) == L.ERR_BAD_ARG
    assert L.lib().l2b_model_create(None, C.byref(m)) == L.ERR_BAD_ARG
    assert L.lib().l2b_session_create(None, None, C.byref(m)) == L.ERR_BAD_ARG


def test_synth_is_deterministic_and_shaped(pkg, synth):
    a = synth.normal_f32(100000, 1, 0.02)
    assert np.array_equal(a, synth.normal_f32(100000, 1, 0.02)) and not np.array_equal(a, synth.normal_f32(100000, 2, 0.02))
    assert abs(a.mean()) < 3e-4 and abs(a.std() - 0.02) < 3e-4
    # a fixed known answer pins the generator across machines
    assert synth.tokens(4, 9, 3, 32000).tolist() == synth.tokens(4, 9, 3, 32000).tolist()
    t = synth.tokens(1000, 9, 3, 32000)
    assert t.min() >= 3 and t.max() < 32000
    for typ, bb, doffs in ((12, 144, (0, 2)), (13, 176, (0, 2)), (14, 210, (208,))):
        raw = synth.kquant_bytes(typ, 2000, 5).reshape(2000, bb)
        for off in doffs:
            d = raw[:, off:off + 2].copy().view(np.float16).astype(np.float32).reshape(-1)
            assert np.all(np.isfinite(d)) and np.all(d >= 0) and abs(d.mean() - 0.01 * np.sqrt(2 / np.pi)) < 1e-3
        body = np.delete(raw, [o + i for o in doffs for i in (0, 1)], axis=1)
        assert abs(body.mean() - 127.5) < 1.0  # remaining bytes uniform
    g = np.load(os.path.join(ROOT, "tests", "golden", "kquants_golden.npz"))
    assert g["q4_K_raw"].shape == (32, 144)


def test_tokenizers(pkg):
    from llama2_jl_b200.tokenizer import BPETokenizer, CharTokenizer, encode
    ct = CharTokenizer.from_text("hello world")
    assert ct.id_to_token[:3] == [" ", "d", "e"] and ct.id_to_token[-2:] == ["<s>", "</s>"]
    assert ct.bos_token_id == len(ct.id_to_token) - 2 and ct.eos_token_id == len(ct.id_to_token) - 1
    assert [ct.id_to_token[i] for i in encode("low", ct)] == ["l", "o", "w"]
    vocab = [b"<unk>", b"<s>", b"</s>", b" ", b"a", b"b", b"c", b"ab", b" a", b" ab", b"abc"]
    scores = [0, 0, 0, -1, -2, -3, -4, 5, 4, 6, 7]
    tok = BPETokenizer(vocab, {t: i for i, t in enumerate(vocab)}, scores, 1, 2)
    # " abc": best pair first: a+b (5) -> " " "ab" "c"; then "ab"+"c" = "abc" (7) beats " "+"ab" (6) -> " ", "abc"
    assert [vocab[i] for i in encode("abc", tok)] == [b" ", b"abc"]
    assert [vocab[i] for i in encode("ab", tok)] == [b" ab"]
    assert encode("", tok) == []
    assert [vocab[i] for i in encode("ba", tok, pad_input=False)] == [b"b", b"a"]


def _tiny_model(synth, pkg):
    cfg = pkg.ModelConfig(64, 96, 2, 4, 4, 66, 32, 10000.0, False)
    w = synth.model_weights(cfg, synth.ALL(0), seed=1, tied_output=True)
    return cfg, w


def test_karpathy_roundtrip(pkg, synth, tmp_path):
    from llama2_jl_b200 import load_karpathy as lk
    from llama2_jl_b200.tokenizer import BPETokenizer
    cfg, w = _tiny_model(synth, pkg)
    vocab = [bytes([65 + i % 26]) * (1 + i // 26) for i in range(cfg.vocab_size)]
    tok = BPETokenizer(vocab, {t: i for i, t in enumerate(vocab)}, [float(-i) for i in range(cfg.vocab_size)], 1, 2)
    ck, tk = str(tmp_path / "m.bin"), str(tmp_path / "t.bin")
    lk.write_karpathy_checkpoint(ck, cfg, w)
    lk.write_karpathy_tokenizer(tk, tok)
    hdr = struct.unpack("<7i", open(ck, "rb").read(28))
    assert hdr == (64, 96, 2, 4, 4, 66, 32)
    m = pkg.load_karpathy_model(ck, tk)
    assert m.config == cfg and m.tokenizer.bos_token_id == 1 and m.tokenizer.eos_token_id == 2
    assert m.tokenizer.id_to_token == vocab
    assert np.array_equal(m.weights.layers[1].w2, w.layers[1].w2) and m.weights.layers[1].w2.shape == (64, 96)
    assert np.array_equal(m.weights.output_weight, m.weights.token_embedding_table)  # tied classifier
    assert "dim            = 64" in str(m)
    # llama2.c's unshared-classifier variant (negative vocab_size in the header), grouped-query heads included
    cfg2 = pkg.ModelConfig(64, 96, 2, 4, 2, 66, 32, 10000.0, False)
    w2 = synth.model_weights(cfg2, synth.ALL(0), seed=2, tied_output=False)
    ck2 = str(tmp_path / "untied.bin")
    lk.write_karpathy_checkpoint(ck2, cfg2, w2, untied=True)
    assert struct.unpack("<7i", open(ck2, "rb").read(28))[5] == -66
    m2 = pkg.load_karpathy_model(ck2, tk)
    assert m2.config == cfg2 and m2.weights.layers[0].wk.shape == (32, 64)
    assert np.array_equal(m2.weights.output_weight, w2.output_weight)
    assert not np.array_equal(m2.weights.output_weight, m2.weights.token_embedding_table)
    assert np.array_equal(m2.weights.layers[1].w3, w2.layers[1].w3) and np.array_equal(m2.weights.rms_final_weight, w2.rms_final_weight)


def _write_gguf(path, arch, cfg, w, synth, fused=False):
    import gguf
    wr = gguf.GGUFWriter(path, arch)
    wr.add_uint32(f"{arch}.embedding_length", cfg.dim)
    wr.add_uint32(f"{arch}.feed_forward_length", cfg.hidden_dim)
    wr.add_uint32(f"{arch}.block_count", cfg.n_layers)
    wr.add_uint32(f"{arch}.attention.head_count", cfg.n_heads)
    wr.add_uint32(f"{arch}.attention.head_count_kv", cfg.n_kv_heads)
    wr.add_uint32(f"{arch}.context_length", 2048)
    wr.add_float32(f"{arch}.rope.freq_base", cfg.rope_freq_base)
    wr.add_uint64("general.some_u64", 7)  # a value type the reference cannot read
    toks = [b"<unk>", b"<s>", b"</s>", b"<0x41>"] + [("▁t%d" % i).encode() for i in range(cfg.vocab_size - 4)]
    wr.add_tokenizer_model("llama")
    wr.add_token_list(toks)
    wr.add_token_scores([0.0] * len(toks))
    wr.add_token_types([2, 3, 3, 6] + [1] * (len(toks) - 4))
    wr.add_bos_token_id(1)
    wr.add_eos_token_id(2)

    def add(name, a):
        if hasattr(a, "ggml_type"):
            bb = {12: 144, 13: 176, 14: 210}[a.ggml_type]
            wr.add_tensor(name, a.data.reshape(a.out_dim, (a.in_dim // 256) * bb), raw_dtype=gguf.GGMLQuantizationType(a.ggml_type))
        else:
            wr.add_tensor(name, np.ascontiguousarray(a, dtype=np.float32))
    add("token_embd.weight", w.token_embedding_table)
    add("output_norm.weight", w.rms_final_weight)
    add("output.weight", w.output_weight)
    for i, l in enumerate(w.layers):
        add(f"blk.{i}.attn_norm.weight", l.rms_att_weight)
        add(f"blk.{i}.ffn_norm.weight", l.rms_ffn_weight)
        if fused:
            cat = lambda ms: type(ms[0])(ms[0].ggml_type, np.concatenate([m.data for m in ms]), ms[0].in_dim, sum(m.out_dim for m in ms))
            add(f"blk.{i}.attn_qkv.weight", cat([l.wq, l.wk, l.wv]))
            add(f"blk.{i}.ffn_up.weight", cat([l.w1, l.w3]))
        else:
            add(f"blk.{i}.attn_q.weight", l.wq)
            add(f"blk.{i}.attn_k.weight", l.wk)
            add(f"blk.{i}.attn_v.weight", l.wv)
            add(f"blk.{i}.ffn_gate.weight", l.w1)
            add(f"blk.{i}.ffn_up.weight", l.w3)
        add(f"blk.{i}.attn_output.weight", l.wo)
        add(f"blk.{i}.ffn_down.weight", l.w2)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()


@pytest.mark.parametrize("arch", ["llama", "phi3"])
def test_gguf_loader(pkg, synth, tmp_path, arch):
    neox = arch == "phi3"
    n_kv = 4 if neox else 2
    cfg = pkg.ModelConfig(256, 512, 2, 4, n_kv, 40, 512, 500000.0, neox)
    types = dict(wq=12, wk=12, wv=13, wo=12, w1=12, w2=13, w3=12, token_embd=12, output=14)
    if neox:
        types = dict(synth.ALL(13), output=14)
    w = synth.model_weights(cfg, types, seed=8)
    path = str(tmp_path / f"{arch}.gguf")
    _write_gguf(path, arch, cfg, w, synth, fused=neox)
    m = pkg.load_gguf_model(path)
    assert m.config == cfg  # seq_len pinned to 512 like the reference
    assert pkg.load_gguf_model(path, seq_len=0).config.seq_len == 2048
    tk = m.tokenizer
    assert tk.bos_token_id == 1 and tk.eos_token_id == 2
    assert tk.id_to_token[3] == b"A" and tk.id_to_token[4] == b" t0"  # byte token and the ▁ -> space fix-up
    for l in range(2):
        for name in ("wq", "wk", "wv", "wo", "w1", "w2", "w3"):
            a, b = getattr(m.weights.layers[l], name), getattr(w.layers[l], name)
            assert (a.ggml_type, a.in_dim, a.out_dim) == (b.ggml_type, b.in_dim, b.out_dim)
            assert np.array_equal(np.asarray(a.data), b.data)
    assert np.array_equal(np.asarray(m.weights.output_weight.data), w.output_weight.data)
    assert np.array_equal(m.weights.layers[0].rms_att_weight, np.ones(256, np.float32))


@pytest.mark.parametrize("arch", ["llama", "phi3"])
def test_native_gguf_inspect(pkg, synth, tmp_path, arch):
    """The library's own GGUF parser (no device needed): config, architecture, tensor count, context length."""
    import ctypes as C
    from llama2_jl_b200 import _lib as L
    neox = arch == "phi3"
    cfg = pkg.ModelConfig(256, 512, 2, 4, 4 if neox else 2, 40, 512, 500000.0, neox)
    w = synth.model_weights(cfg, dict(synth.ALL(13), output=14) if neox else dict(synth.ALL(12), wv=13, w2=13, output=14), seed=8)
    path = str(tmp_path / f"{arch}.gguf")
    _write_gguf(path, arch, cfg, w, synth, fused=neox)
    out, a, n, ctx = L.Config(), C.c_int32(), C.c_int64(), C.c_int64()
    L.check(L.lib().l2b_gguf_inspect(path.encode(), C.byref(out), C.byref(a), C.byref(n), C.byref(ctx)))
    assert (out.dim, out.hidden_dim, out.n_layers, out.n_heads, out.n_kv_heads, out.vocab_size) == (256, 512, 2, 4, cfg.n_kv_heads, 40)
    assert abs(out.rope_freq_base - 500000.0) < 1e-3 and bool(out.rope_is_neox) == neox
    assert a.value == (1 if neox else 0) and ctx.value == 2048 and out.seq_len == 2048
    assert n.value == 3 + 2 * (6 if neox else 9)


def test_native_gguf_rejects_other_files(pkg, tmp_path):
    import ctypes as C
    from llama2_jl_b200 import _lib as L
    lib = L.lib()
    out = L.Config()
    cases = {"magic": b"GGML" + b"\0" * 64, "short": b"GGUF\x03", "truncated": b"GGUF" + (3).to_bytes(4, "little") + (5).to_bytes(8, "little") + (9).to_bytes(8, "little"),
             "huge_count": b"GGUF" + (3).to_bytes(4, "little") + (1 << 40).to_bytes(8, "little") + (0).to_bytes(8, "little") + b"\0" * 32}
    for name, blob in cases.items():
        p = tmp_path / f"{name}.gguf"
        p.write_bytes(blob)
        assert lib.l2b_gguf_inspect(str(p).encode(), C.byref(out), None, None, None) == L.ERR_BAD_ARG, name
        if name == "magic":
            assert b"Not a GGUF file" in lib.l2b_last_error_string()  # the reference's message (src/load_gguf.jl:89)
    assert lib.l2b_gguf_inspect(str(tmp_path / "missing.gguf").encode(), C.byref(out), None, None, None) == L.ERR_BAD_ARG


def test_gguf_rejects_other_files(pkg, tmp_path):
    p = tmp_path / "x.gguf"
    p.write_bytes(b"GGML" + b"\0" * 64)
    with pytest.raises(ValueError, match="Not a GGUF file"):
        pkg.load_gguf_model(str(p))


def test_sample_argument_check(pkg):
    with pytest.raises(ValueError, match="Prompt cannot be empty"):
        pkg.sample(pkg.LanguageModel(None, None, None), "", bos_token=False)
