"""Seeded synthetic weights, prompts and configurations of the benchmark shapes.  All bytes come from the
counter-based generators of the test-support library (libl2b_synth.so, include/l2b_synth.h), so every machine builds the same model from a seed."""
import numpy as np

from . import _lib as L
from .model import ModelConfig, QuantMatrix, TransformerLayerWeights, TransformerWeights

Q4, Q5, Q6, F32 = L.TYPE_Q4_K, L.TYPE_Q5_K, L.TYPE_Q6_K, L.TYPE_F32


def normal_f32(n, seed, std):
    a = np.empty(int(n), dtype=np.float32)
    L.synth_check(L.synth_lib().l2b_synth_f32(L.ptr(a), a.size, int(seed), float(std), 0))
    return a


def kquant_bytes(ggml_type, n_blocks, seed):
    a = np.empty(int(n_blocks) * L.BLOCK_BYTES[ggml_type], dtype=np.uint8)
    L.synth_check(L.synth_lib().l2b_synth_kquant(ggml_type, L.ptr(a), int(n_blocks), int(seed)))
    return a


def tokens(n, seed, lo, hi):
    a = np.empty(int(n), dtype=np.int32)
    L.synth_check(L.synth_lib().l2b_synth_tokens(L.ptr(a), a.size, int(seed), int(lo), int(hi)))
    return a


def matrix(ggml_type, in_dim, out_dim, seed, std=0.02):
    """(in, out) weight matrix of the given storage type."""
    if ggml_type == F32:
        return normal_f32(in_dim * out_dim, seed, std).reshape(out_dim, in_dim)
    return QuantMatrix(ggml_type, kquant_bytes(ggml_type, (in_dim // 256) * out_dim, seed), in_dim, out_dim)


def _seed(base, layer, role):
    return (base * 1000003 + layer * 101 + role) & 0xFFFFFFFFFFFF


def model_weights(c: ModelConfig, types: dict, seed: int, tied_output=False, distinct_layers: int = 0) -> TransformerWeights:
    """types maps 'wq','wk','wv','wo','w1','w2','w3','token_embd','output' to a ggml type.  Norm gains are 1.
    distinct_layers = k > 0: only the first k layers are generated and layer l reuses the host arrays of layer l % k
    (every layer still gets its own device copy), for shapes whose full host copy would not fit in memory."""
    hs = c.dim // c.n_heads
    kv = hs * c.n_kv_heads
    ones = np.ones(c.dim, dtype=np.float32)
    layers = []
    for l in range(c.n_layers):
        if distinct_layers and l >= distinct_layers:
            layers.append(layers[l % distinct_layers])
            continue
        layers.append(TransformerLayerWeights(
            ones, ones,
            matrix(types["wq"], c.dim, c.dim, _seed(seed, l, 1)), matrix(types["wk"], c.dim, kv, _seed(seed, l, 2)),
            matrix(types["wv"], c.dim, kv, _seed(seed, l, 3)), matrix(types["wo"], c.dim, c.dim, _seed(seed, l, 4)),
            matrix(types["w1"], c.dim, c.hidden_dim, _seed(seed, l, 5)), matrix(types["w2"], c.hidden_dim, c.dim, _seed(seed, l, 6)),
            matrix(types["w3"], c.dim, c.hidden_dim, _seed(seed, l, 7))))
    emb = matrix(types["token_embd"], c.dim, c.vocab_size, _seed(seed, 999, 8))
    out = emb if tied_output else matrix(types["output"], c.dim, c.vocab_size, _seed(seed, 999, 9))
    return TransformerWeights(emb, layers, ones, out)


ALL = lambda t: {k: t for k in ("wq", "wk", "wv", "wo", "w1", "w2", "w3", "token_embd", "output")}

# the configurations the benchmark specification names
TINY_F32 = dict(config=ModelConfig(288, 768, 6, 6, 6, 32000, 256, 10000.0, False), types=ALL(F32), tied=True,
                n_prompt=16, n_decode=240)
LLAMA3_8B_Q4_K_S = dict(config=ModelConfig(4096, 14336, 32, 32, 8, 128256, 512, 500000.0, False),
                        types=dict(wq=Q4, wk=Q4, wv=Q5, wo=Q4, w1=Q4, w2=Q5, w3=Q4, token_embd=Q4, output=Q6), tied=False,
                        n_prompt=128, n_decode=256)
PHI3_MINI_Q5_K_M = dict(config=ModelConfig(3072, 8192, 32, 32, 32, 32064, 4096, 10000.0, True),
                        types=dict(ALL(Q5), output=Q6), tied=False, n_prompt=2048, n_decode=512)
LLAMA2_70B_Q4_K = dict(config=ModelConfig(8192, 28672, 80, 64, 8, 32000, 4096, 10000.0, False),
                       types=dict(ALL(Q4), output=Q6), tied=False, n_prompt=512, n_decode=256)


def scaled(spec, n_layers=None, vocab_size=None, seq_len=None):
    """The same shape with fewer layers / a smaller vocabulary / a shorter context (for parity runs the
    CPU oracle finishes in seconds)."""
    c = spec["config"]
    c2 = ModelConfig(c.dim, c.hidden_dim, n_layers or c.n_layers, c.n_heads, c.n_kv_heads, vocab_size or c.vocab_size,
                     seq_len or c.seq_len, c.rope_freq_base, c.rope_is_neox)
    return dict(spec, config=c2)


def prompt_tokens(spec, seed):
    c = spec["config"]
    return tokens(spec["n_prompt"], seed ^ 0xABCDEF, 3, c.vocab_size)
