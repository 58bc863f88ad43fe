"""GGUF reader (src/load_gguf.jl).  Tensors are numpy views into a memory map of the file, so an
upload copies straight from the page cache to the device (the reference's mmap=true path,
src/load_gguf.jl:160-185)."""
import struct

import numpy as np

from . import _lib as L
from .model import LanguageModel, ModelConfig, QuantMatrix, TransformerLayerWeights, TransformerWeights
from .tokenizer import BPETokenizer

# GGUF_METADATA_VALUE_TYPE (src/load_gguf.jl:1-24).  The reference reads only STRING, UINT32, INT32,
# FLOAT32, ARRAY and BOOL (:59-77); the remaining scalar types are read here too.
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_STRING, _ARRAY = 8, 9
_TOKEN_NORMAL, _TOKEN_BYTE = 1, 6  # LLAMA_TOKEN_TYPE (src/load_gguf.jl:44-52)


class _Reader:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt):
        n = struct.calcsize(fmt)
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += n
        return v

    def string(self):  # src/load_gguf.jl:54-57
        n = self.take("<Q")
        s = bytes(self.buf[self.pos:self.pos + n])
        self.pos += n
        return s

    def value(self, vt):  # src/load_gguf.jl:59-77
        if vt == _STRING:
            return self.string()
        if vt == _ARRAY:
            et = self.take("<I")
            n = self.take("<Q")
            if et in _SCALARS and et != 7:
                fmt = _SCALARS[et]
                a = np.frombuffer(self.buf, dtype=np.dtype(fmt), count=n, offset=self.pos)
                self.pos += a.nbytes
                return a
            return [self.value(et) for _ in range(n)]
        if vt in _SCALARS:
            return self.take(_SCALARS[vt])
        raise L.L2BError(L.ERR_UNSUPPORTED_TYPE, f"reading metadata value of type {vt} is not implemented yet")


def read_gguf_header(r: _Reader):
    """magic, version (ignored), tensor_count, metadata (src/load_gguf.jl:84-105)."""
    if bytes(r.buf[0:4]) != b"GGUF":
        raise ValueError("Not a GGUF file")
    r.pos = 4
    r.take("<I")
    tensor_count = r.take("<Q")
    kv_count = r.take("<Q")
    kv = {}
    for _ in range(kv_count):
        key = r.string().decode("utf-8")
        kv[key] = r.value(r.take("<I"))
    return tensor_count, kv


def read_gguf_tensor_info(r: _Reader):
    """src/load_gguf.jl:121-129."""
    name = r.string().decode("utf-8")
    nd = r.take("<I")
    dims = [r.take("<Q") for _ in range(nd)]
    typ = r.take("<I")
    offset = r.take("<Q")
    return name, dims, typ, offset


def align_offset(offset, alignment):  # src/load_gguf.jl:131-133
    return offset + (alignment - (offset % alignment)) % alignment


def _tensor(buf, start, dims, typ):
    """read_ggml_tensor (src/load_gguf.jl:135-193): F32, Q4_K, Q5_K, Q6_K only."""
    in_dim = int(dims[0])
    out_dim = int(np.prod(dims[1:])) if len(dims) > 1 else 1
    if typ == L.TYPE_F32:
        a = np.frombuffer(buf, dtype="<f4", count=in_dim * out_dim, offset=start)
        return a.reshape(out_dim, in_dim) if len(dims) > 1 else a
    if typ in L.BLOCK_BYTES:
        if in_dim % 256 != 0:
            raise ValueError("size[1] % QK_K must be 0")
        nbytes = (in_dim // 256) * out_dim * L.BLOCK_BYTES[typ]
        return QuantMatrix(typ, np.frombuffer(buf, dtype=np.uint8, count=nbytes, offset=start), in_dim, out_dim)
    raise L.L2BError(L.ERR_UNSUPPORTED_TYPE, f"tensor type {typ} not implemented")


def _gpt2_decoder():
    """Inverse of GPT-2's byte-to-unicode table (src/load_gguf.jl:195-209)."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {chr(c): b for c, b in zip(cs, bs)}


def _rows(m, a, b):
    return m.rows(a, b) if isinstance(m, QuantMatrix) else m[a:b]


def _out_dim(m):
    return m.out_dim if isinstance(m, QuantMatrix) else m.shape[0]


def build_llama(kv, t, vocab_size, seq_len):
    """src/load_gguf.jl:211-253."""
    c = ModelConfig(dim=int(kv["llama.embedding_length"]), hidden_dim=int(kv["llama.feed_forward_length"]),
                    n_layers=int(kv["llama.block_count"]), n_heads=int(kv["llama.attention.head_count"]),
                    n_kv_heads=int(kv["llama.attention.head_count_kv"]), vocab_size=vocab_size, seq_len=seq_len,
                    rope_freq_base=float(kv.get("llama.rope.freq_base", 10000.0)), rope_is_neox=False)
    layers = []
    for i in range(c.n_layers):
        if f"blk.{i}.attn_q.weight" not in t:
            raise KeyError(f"missing blk.{i} weights")
        g = lambda n: t[f"blk.{i}.{n}.weight"]
        layers.append(TransformerLayerWeights(g("attn_norm"), g("ffn_norm"), g("attn_q"), g("attn_k"), g("attn_v"), g("attn_output"),
                                              g("ffn_gate"), g("ffn_down"), g("ffn_up")))
    return c, TransformerWeights(t["token_embd.weight"], layers, t["output_norm.weight"], t["output.weight"])


def build_phi3(kv, t, vocab_size, seq_len):
    """src/load_gguf.jl:255-315: fused attn_qkv split in three row ranges, fused ffn_up split into gate (first half)
    and up (second half); neox RoPE.  The reference asserts the qkv third is 3072 (:262); any size that splits
    evenly is accepted here."""
    c = ModelConfig(dim=int(kv["phi3.embedding_length"]), hidden_dim=int(kv["phi3.feed_forward_length"]),
                    n_layers=int(kv["phi3.block_count"]), n_heads=int(kv["phi3.attention.head_count"]),
                    n_kv_heads=int(kv["phi3.attention.head_count_kv"]), vocab_size=vocab_size, seq_len=seq_len,
                    rope_freq_base=float(kv.get("phi3.rope.freq_base", 10000.0)), rope_is_neox=True)
    layers = []
    for i in range(c.n_layers):
        if f"blk.{i}.attn_qkv.weight" not in t:
            raise KeyError(f"missing blk.{i} weights")
        g = lambda n: t[f"blk.{i}.{n}.weight"]
        qkv = g("attn_qkv")
        n = _out_dim(qkv) // 3
        gu = g("ffn_up")
        h = _out_dim(gu) // 2
        layers.append(TransformerLayerWeights(g("attn_norm"), g("ffn_norm"), _rows(qkv, 0, n), _rows(qkv, n, 2 * n), _rows(qkv, 2 * n, 3 * n),
                                              g("attn_output"), _rows(gu, 0, h), g("ffn_down"), _rows(gu, h, 2 * h)))
    return c, TransformerWeights(t["token_embd.weight"], layers, t["output_norm.weight"], t["output.weight"])


def load_gguf_model(filename: str, mmap: bool = True, seq_len: int = 512, native: bool = False, **kw) -> LanguageModel:
    """load_gguf_model(filename; mmap=true) (src/load_gguf.jl:317-394).

    seq_len defaults to the 512 the reference hard-codes (:237, :299); pass 0 to take `<arch>.context_length`
    from the file instead.  native=True lets the library read the tensors itself (l2b_model_load_gguf: its own
    parser, memory map and upload; `model.weights` is then None); the tokenizer is built here either way."""
    buf = np.memmap(filename, dtype=np.uint8, mode="r") if mmap else np.fromfile(filename, dtype=np.uint8)
    r = _Reader(buf)
    tensor_count, kv = read_gguf_header(r)
    infos = [read_gguf_tensor_info(r) for _ in range(tensor_count)]
    alignment = int(kv.get("general.alignment", 32))
    pad_offset = align_offset(r.pos, alignment)
    tensors = {} if native else {name: _tensor(buf, pad_offset + off, dims, typ) for name, dims, typ, off in infos}

    id_to_token = [bytes(s) for s in kv["tokenizer.ggml.tokens"]]
    token_types = kv["tokenizer.ggml.token_type"]
    tok_model = kv["tokenizer.ggml.model"].decode()
    if tok_model == "llama":  # src/load_gguf.jl:345-358
        for i, tt in enumerate(token_types):
            if tt == _TOKEN_NORMAL:
                id_to_token[i] = id_to_token[i].replace(b"\xe2\x96\x81", b" ")
            elif tt == _TOKEN_BYTE:
                id_to_token[i] = bytes([int(id_to_token[i][1:-1], 0)])
    elif tok_model == "gpt2":  # :359-368
        dec = _gpt2_decoder()
        for i, tt in enumerate(token_types):
            if tt == _TOKEN_NORMAL:
                # String([dict[c] for c in token]) (:365): the byte VALUES as characters, i.e. UTF-8 encoded again
                id_to_token[i] = "".join(chr(dec[ch]) for ch in id_to_token[i].decode("utf-8")).encode("utf-8")
    else:
        raise ValueError(f"unsupported tokenizer model: {tok_model}")
    token_to_id = {tok: i for i, tok in enumerate(id_to_token)}
    scores = kv.get("tokenizer.ggml.scores")
    scores = [0.0] * len(id_to_token) if scores is None else [float(s) for s in scores]
    tokenizer = BPETokenizer(id_to_token, token_to_id, scores, int(kv["tokenizer.ggml.bos_token_id"]), int(kv["tokenizer.ggml.eos_token_id"]))

    arch = kv["general.architecture"].decode()
    if native:
        from .model import _DeviceModel
        dev, config = _DeviceModel.from_gguf(filename, seq_len, kw.get("act_planes", 0), kw.get("device", -1), kw.get("stream"),
                                             kw.get("tp_size", 1), kw.get("tp_rank", 0))
        model = LanguageModel(config, tokenizer, None, **kw)
        model._dev = dev
        return model
    if seq_len == 0:
        seq_len = int(kv[f"{arch}.context_length"])
    if arch == "llama":
        config, weights = build_llama(kv, tensors, len(id_to_token), seq_len)
    elif arch == "phi3":
        config, weights = build_phi3(kv, tensors, len(id_to_token), seq_len)
    else:
        raise ValueError(f"unsupported model architecture: {arch}")
    return LanguageModel(config, tokenizer, weights, **kw)
