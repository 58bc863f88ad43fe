"""llama2.c checkpoint and tokenizer reader (src/load_karpathy.jl)."""
import struct

import numpy as np

from .model import LanguageModel, ModelConfig, TransformerLayerWeights, TransformerWeights
from .tokenizer import BPETokenizer


def read_karpathy_config(f) -> ModelConfig:
    """Seven Int32: dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len; rope base 10000,
    interleaved RoPE (src/load_karpathy.jl:1-11).  llama2.c writes a NEGATIVE vocab_size when the classifier is not shared
    with the embedding; the reference does not handle that case.  Here the config carries the absolute value and the
    attribute `untied_classifier` says which variant the file is."""
    dim, hidden, n_layers, n_heads, n_kv, vocab, seq = struct.unpack("<7i", f.read(28))
    c = ModelConfig(dim, hidden, n_layers, n_heads, n_kv, abs(vocab), seq, 10000.0, False)
    c.untied_classifier = vocab < 0
    return c


def read_karpathy_weights(f, c: ModelConfig) -> TransformerWeights:
    """f32 arrays in llama2.c order: embedding, then per kind across layers (src/load_karpathy.jl:33-59).
    The reference reads wk and wv as (dim, dim), which needs n_kv_heads == n_heads (:17-18); llama2.c stores them with
    n_kv_heads * head_size rows, which is what is read here (the same thing when the head counts are equal).
    Untied variant: after the final norm the file holds the two RoPE tables of the legacy format (seq_len * head_size / 2
    floats each, skipped: the tables are recomputed) and then the classifier (vocab_size, dim)."""
    def rd(*shape):
        n = int(np.prod(shape))
        a = np.frombuffer(f.read(4 * n), dtype="<f4")
        if a.size != n:
            raise EOFError("checkpoint truncated")
        return a.reshape(shape).copy()
    emb = rd(c.vocab_size, c.dim)
    L = c.n_layers
    rms_att = [rd(c.dim) for _ in range(L)]
    wq = [rd(c.dim, c.dim) for _ in range(L)]
    kv_dim = c.dim // c.n_heads * c.n_kv_heads
    wk = [rd(kv_dim, c.dim) for _ in range(L)]
    wv = [rd(kv_dim, c.dim) for _ in range(L)]
    wo = [rd(c.dim, c.dim) for _ in range(L)]
    rms_ffn = [rd(c.dim) for _ in range(L)]
    w1 = [rd(c.hidden_dim, c.dim) for _ in range(L)]
    w2 = [rd(c.dim, c.hidden_dim) for _ in range(L)]
    w3 = [rd(c.hidden_dim, c.dim) for _ in range(L)]
    rms_final = rd(c.dim)
    layers = [TransformerLayerWeights(rms_att[l], rms_ffn[l], wq[l], wk[l], wv[l], wo[l], w1[l], w2[l], w3[l]) for l in range(L)]
    if getattr(c, "untied_classifier", False):
        rd(c.seq_len, c.dim // c.n_heads // 2)  # freq_cis_real
        rd(c.seq_len, c.dim // c.n_heads // 2)  # freq_cis_imag
        return TransformerWeights(emb, layers, rms_final, rd(c.vocab_size, c.dim))
    return TransformerWeights(emb, layers, rms_final, emb.copy())  # output tied to the embedding (:56)


def load_karpathy_tokenizer(filename: str, vocab_size: int) -> BPETokenizer:
    """max_token_length Int32, then per token score f32, len Int32, bytes (src/load_karpathy.jl:61-78).
    BOS = 1, EOS = 2 in 0-based ids (2 and 3 in the reference)."""
    id_to_token, token_to_id, scores = [], {}, []
    with open(filename, "rb") as f:
        f.read(4)
        for i in range(vocab_size):
            score, ln = struct.unpack("<fi", f.read(8))
            word = f.read(ln)
            id_to_token.append(word)
            token_to_id[word] = i
            scores.append(score)
    return BPETokenizer(id_to_token, token_to_id, scores, 1, 2)


def load_karpathy_model(checkpoint_filename: str, tokenizer_filename: str, **kw) -> LanguageModel:
    """load_karpathy_model(checkpoint, tokenizer) (src/load_karpathy.jl:80-98)."""
    with open(checkpoint_filename, "rb") as f:
        config = read_karpathy_config(f)
        weights = read_karpathy_weights(f, config)
    tokenizer = load_karpathy_tokenizer(tokenizer_filename, config.vocab_size)
    return LanguageModel(config, tokenizer, weights, **kw)


def write_karpathy_checkpoint(filename: str, c: ModelConfig, w: TransformerWeights, untied: bool = False) -> None:
    """Writer for the same format (the reference has none); used to build fixtures and to hand a trained model over.
    untied = True writes llama2.c's unshared-classifier variant: negative vocab_size, the legacy RoPE tables, the classifier."""
    with open(filename, "wb") as f:
        f.write(struct.pack("<7i", c.dim, c.hidden_dim, c.n_layers, c.n_heads, c.n_kv_heads, -c.vocab_size if untied else c.vocab_size, c.seq_len))
        f.write(np.ascontiguousarray(w.token_embedding_table, dtype="<f4").tobytes())
        for name in ("rms_att_weight", "wq", "wk", "wv", "wo", "rms_ffn_weight", "w1", "w2", "w3"):
            for l in w.layers:
                f.write(np.ascontiguousarray(getattr(l, name), dtype="<f4").tobytes())
        f.write(np.ascontiguousarray(w.rms_final_weight, dtype="<f4").tobytes())
        if untied:
            h2 = c.dim // c.n_heads // 2
            ang = np.arange(c.seq_len, dtype=np.float64)[:, None] * (10000.0 ** (-np.arange(h2, dtype=np.float64) / h2))[None, :]
            f.write(np.cos(ang).astype("<f4").tobytes())
            f.write(np.sin(ang).astype("<f4").tobytes())
            f.write(np.ascontiguousarray(w.output_weight, dtype="<f4").tobytes())


def write_karpathy_tokenizer(filename: str, tok: BPETokenizer) -> None:
    with open(filename, "wb") as f:
        f.write(struct.pack("<i", max(len(t) for t in tok.id_to_token)))
        for t, s in zip(tok.id_to_token, tok.token_scores):
            f.write(struct.pack("<fi", s, len(t)))
            f.write(t)
