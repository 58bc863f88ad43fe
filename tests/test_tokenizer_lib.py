"""The tokenizer inside the library (l2b_tokenizer_*) against the Python mirror of src/tokenizer.jl and of the vocabulary
fix-ups in src/load_gguf.jl:339-380.  Host code only: no GPU is needed."""
import ctypes as C

import numpy as np
import pytest


class LibTokenizer:
    def __init__(self, L, handle):
        self.L, self.h = L, handle

    @classmethod
    def create(cls, L, tokens, scores, types, model, bos, eos):
        flat = np.frombuffer(b"".join(tokens), dtype=np.uint8).copy() if tokens else np.zeros(0, np.uint8)
        if flat.size == 0:
            flat = np.zeros(1, np.uint8)
        off = np.zeros(len(tokens) + 1, np.int64)
        off[1:] = np.cumsum([len(t) for t in tokens])
        sc = None if scores is None else np.asarray(scores, np.float32)
        ty = None if types is None else np.asarray(types, np.int32)
        h = C.c_void_p()
        L.check(L.lib().l2b_tokenizer_create(L.ptr(flat), L.ptr(off), len(tokens), L.ptr(sc), L.ptr(ty), model, bos, eos, C.byref(h)))
        return cls(L, h)

    def encode(self, data: bytes, pad_input=True):
        buf = np.frombuffer(data, dtype=np.uint8).copy() if data else np.zeros(1, np.uint8)
        out = np.zeros(len(data) + 1, np.int32)
        n = C.c_int64()
        self.L.check(self.L.lib().l2b_tokenizer_encode(self.h, self.L.ptr(buf), len(data), int(pad_input), self.L.ptr(out), out.size, C.byref(n)))
        return [int(t) for t in out[:n.value]]

    def token(self, i):
        p, n = C.c_void_p(), C.c_int64()
        self.L.check(self.L.lib().l2b_tokenizer_token(self.h, i, C.byref(p), C.byref(n)))
        return C.string_at(p.value, n.value) if n.value else b""

    def info(self):
        a, b, c = C.c_int32(), C.c_int32(), C.c_int32()
        self.L.check(self.L.lib().l2b_tokenizer_info(self.h, C.byref(a), C.byref(b), C.byref(c)))
        return a.value, b.value, c.value

    def close(self):
        self.L.lib().l2b_tokenizer_destroy(self.h)


@pytest.fixture(scope="module")
def L(pkg):
    from llama2_jl_b200 import _lib
    return _lib


def _random_vocab(rng, n_merges):
    """All 256 single bytes plus random concatenations of existing tokens, with random scores (ties included)."""
    toks = [bytes([b]) for b in range(256)]
    seen = set(toks)
    while len(toks) < 256 + n_merges:
        a, b = toks[rng.integers(len(toks))], toks[rng.integers(len(toks))]
        if len(a + b) <= 6 and a + b not in seen:
            toks.append(a + b)
            seen.add(a + b)
    scores = rng.integers(-5, 6, size=len(toks)).astype(np.float32)  # few distinct values: many ties
    return toks, scores


def test_encode_matches_the_python_mirror_on_random_bytes(L):
    from llama2_jl_b200.tokenizer import BPETokenizer, encode
    rng = np.random.default_rng(11)
    toks, scores = _random_vocab(rng, 600)
    py = BPETokenizer(toks, {t: i for i, t in enumerate(toks)}, [float(s) for s in scores], 1, 2)
    lt = LibTokenizer.create(L, toks, scores, None, 0, 1, 2)
    assert lt.info() == (len(toks), 1, 2)
    for trial in range(200):
        n = int(rng.integers(0, 40))
        alphabet = rng.integers(0, 256, size=4) if trial % 2 else np.arange(256)  # small alphabets merge a lot
        data = bytes(int(x) for x in rng.choice(alphabet, size=n))
        for pad in (True, False):
            assert lt.encode(data, pad) == encode(data, py, pad_input=pad), (data, pad)
    assert lt.encode(b"") == []
    assert [lt.token(i) for i in (0, 65, 300)] == [toks[0], toks[65], toks[300]]
    lt.close()


def test_encode_known_case_and_errors(L):
    vocab = [b"<unk>", b"<s>", b"</s>", b" ", b"a", b"b", b"c", b"ab", b" a", b" ab", b"abc"]
    scores = [0, 0, 0, -1, -2, -3, -4, 5, 4, 6, 7]
    lt = LibTokenizer.create(L, vocab, scores, None, 0, 1, 2)
    # " abc": a+b (5) first -> " " "ab" "c"; then "ab"+"c" = "abc" (7) beats " "+"ab" (6) -> " ", "abc"
    assert [vocab[i] for i in lt.encode(b"abc")] == [b" ", b"abc"]
    assert [vocab[i] for i in lt.encode(b"ab")] == [b" ab"]
    assert [vocab[i] for i in lt.encode(b"ba", pad_input=False)] == [b"b", b"a"]
    buf = np.frombuffer(b"abz", dtype=np.uint8).copy()
    out, n = np.zeros(8, np.int32), C.c_int64()
    assert L.lib().l2b_tokenizer_encode(lt.h, L.ptr(buf), 3, 1, L.ptr(out), 8, C.byref(n)) == L.ERR_BAD_ARG  # no token for "z"
    assert b"byte 122" in L.lib().l2b_last_error_string()
    assert L.lib().l2b_tokenizer_encode(lt.h, L.ptr(buf), 2, 1, L.ptr(out), 0, C.byref(n)) == L.ERR_BAD_ARG and n.value == 1  # too small
    p, k = C.c_void_p(), C.c_int64()
    assert L.lib().l2b_tokenizer_token(lt.h, 99, C.byref(p), C.byref(k)) == L.ERR_BAD_ARG
    lt.close()
    h = C.c_void_p()
    flat, off = np.zeros(4, np.uint8), np.array([0, 2, 1], np.int64)
    assert L.lib().l2b_tokenizer_create(L.ptr(flat), L.ptr(off), 2, None, None, 0, 0, 1, C.byref(h)) == L.ERR_BAD_ARG  # offsets decrease
    assert L.lib().l2b_tokenizer_create(L.ptr(flat), L.ptr(np.array([0, 1, 2], np.int64)), 2, None, None, 0, 0, 5, C.byref(h)) == L.ERR_BAD_ARG


def test_vocabulary_fixups(L):
    from llama2_jl_b200.load_gguf import _gpt2_decoder
    # "llama": U+2581 -> space in NORMAL tokens only; <0xNN> byte tokens; other types untouched (src/load_gguf.jl:345-358)
    toks = ["<unk>".encode(), "▁the▁cat".encode(), "<0x0A>".encode(), "<0xff>".encode(), "▁ctl".encode()]
    lt = LibTokenizer.create(L, toks, None, [2, 1, 6, 6, 3], 1, 0, 0)
    assert [lt.token(i) for i in range(5)] == [b"<unk>", b" the cat", b"\n", b"\xff", "▁ctl".encode()]
    lt.close()
    # "gpt2": NORMAL tokens through the inverse byte encoder, re-encoded as characters (:359-368)
    dec = _gpt2_decoder()
    enc = {b: c for c, b in dec.items()}
    raw = bytes([32, 104, 105, 10, 200, 255])  # " hi\n" and two bytes beyond ASCII
    spelled = "".join(enc[b] for b in raw).encode("utf-8")
    lt = LibTokenizer.create(L, [spelled, "Ġ".encode(), spelled], None, [1, 1, 3], 2, 0, 0)
    want = "".join(chr(b) for b in raw).encode("utf-8")
    assert lt.token(0) == want and lt.token(1) == b" " and lt.token(2) == spelled
    lt.close()
    h = C.c_void_p()
    bad = "☃".encode()  # not in GPT-2's alphabet: a KeyError in the reference
    assert L.lib().l2b_tokenizer_create(L.ptr(np.frombuffer(bad, np.uint8).copy()), L.ptr(np.array([0, len(bad)], np.int64)), 1, None,
                                        L.ptr(np.array([1], np.int32)), 2, 0, 0, C.byref(h)) == L.ERR_BAD_ARG


def test_tokenizer_from_a_gguf_file_matches_the_python_loader(L, pkg, synth, tmp_path):
    from test_host_logic import _tiny_model, _write_gguf
    from llama2_jl_b200.tokenizer import encode
    cfg, w = _tiny_model(synth, pkg)
    path = str(tmp_path / "tok.gguf")
    _write_gguf(path, "llama", cfg, w, synth)
    py = pkg.load_gguf_model(path).tokenizer
    h = C.c_void_p()
    L.check(L.lib().l2b_tokenizer_load_gguf(path.encode(), C.byref(h)))
    lt = LibTokenizer(L, h)
    assert lt.info() == (len(py.id_to_token), py.bos_token_id, py.eos_token_id)
    assert [lt.token(i) for i in range(len(py.id_to_token))] == list(py.id_to_token)
    # the byte token <0x41> = "A" is the only single-byte token besides the pad space of " t<i>": text made of it encodes
    assert lt.encode(b"AAA", pad_input=False) == encode("AAA", py, pad_input=False)
    lt.close()
    assert L.lib().l2b_tokenizer_load_gguf(str(tmp_path / "missing.gguf").encode(), C.byref(h)) == L.ERR_BAD_ARG
