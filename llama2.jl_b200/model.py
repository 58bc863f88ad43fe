"""Host-side mirror of the reference's inference interface (src/inference.jl), bound to the C ABI.

Names and argument meaning follow the reference: ModelConfig, TransformerLayerWeights,
TransformerWeights, LanguageModel, matmul!, transformer!, sample.  Python differences:
`!` becomes a trailing underscore, and token ids / positions are 0-based throughout (the
reference is 1-based Julia).  Weight matrices are given as the reference stores them:
`(in, out)` column-major, which is a C-contiguous numpy array of shape (out, in); k-quant
matrices are `QuantMatrix` (raw super-block bytes, out rows of in/256 blocks).
"""
import ctypes as C
import random
import sys
import time
from dataclasses import dataclass, field
from typing import List, Optional, Union

import numpy as np

from . import _lib as L


@dataclass
class ModelConfig:
    """src/inference.jl:1-11 (no defaults there either)."""
    dim: int
    hidden_dim: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    vocab_size: int
    seq_len: int
    rope_freq_base: float
    rope_is_neox: bool

    def __str__(self):  # Base.show, src/inference.jl:13-25
        rows = [("dim", self.dim), ("hidden_dim", self.hidden_dim), ("n_layers", self.n_layers), ("n_heads", self.n_heads),
                ("n_kv_heads", self.n_kv_heads), ("vocab_size", self.vocab_size), ("seq_len", self.seq_len),
                ("rope_freq_base", self.rope_freq_base), ("rope_is_neox", str(self.rope_is_neox).lower())]
        return "ModelConfig(\n" + "".join(f"  {k:<14} = {v},\n" for k, v in rows) + ")"


class QuantMatrix:
    """AbstractMatrix{block_q4_K|block_q5_K|block_q6_K} of size (in/256, out) (src/kquants.jl:7-35):
    `data` is a uint8 array of out * (in/256) * block_bytes raw bytes, rows contiguous."""

    def __init__(self, ggml_type: int, data: np.ndarray, in_dim: int, out_dim: int):
        if ggml_type not in L.BLOCK_BYTES:
            raise L.L2BError(L.ERR_UNSUPPORTED_TYPE, f"tensor type {ggml_type} not implemented")
        if in_dim % 256 != 0:
            raise ValueError("in_dim % 256 must be 0")
        self.ggml_type, self.in_dim, self.out_dim = ggml_type, in_dim, out_dim
        self.data = np.ascontiguousarray(data).reshape(-1).view(np.uint8) if not isinstance(data, np.memmap) else data
        expect = out_dim * (in_dim // 256) * L.BLOCK_BYTES[ggml_type]
        if self.data.size != expect:
            raise ValueError(f"expected {expect} bytes, got {self.data.size}")

    def rows(self, start: int, stop: int) -> "QuantMatrix":
        """view(A, :, start+1:stop): a contiguous range of output rows (src/load_gguf.jl:264-276)."""
        rb = (self.in_dim // 256) * L.BLOCK_BYTES[self.ggml_type]
        return QuantMatrix(self.ggml_type, self.data[start * rb:stop * rb], self.in_dim, stop - start)


Matrix = Union[np.ndarray, QuantMatrix]


def _matrix_info(a: Matrix):
    if isinstance(a, QuantMatrix):
        return a.ggml_type, a.data, a.in_dim, a.out_dim
    a32 = np.ascontiguousarray(a, dtype=np.float32)
    if a32.ndim != 2:
        raise ValueError("f32 weight matrices are 2-D (out, in)")
    return L.TYPE_F32, a32, a32.shape[1], a32.shape[0]


@dataclass
class TransformerLayerWeights:
    """src/inference.jl:27-40."""
    rms_att_weight: np.ndarray
    rms_ffn_weight: np.ndarray
    wq: Matrix
    wk: Matrix
    wv: Matrix
    wo: Matrix
    w1: Matrix
    w2: Matrix
    w3: Matrix


@dataclass
class TransformerWeights:
    """src/inference.jl:42-48."""
    token_embedding_table: Matrix
    layers: List[TransformerLayerWeights]
    rms_final_weight: np.ndarray
    output_weight: Matrix


class _DeviceModel:
    """Owns an l2b_model and one l2b_session (RunState)."""

    def __init__(self, config: ModelConfig, weights: TransformerWeights, act_planes=0, device=-1, stream=None, tp_size=1, tp_rank=0):
        lib = L.lib()
        cfg = L.Config(dim=config.dim, hidden_dim=config.hidden_dim, n_layers=config.n_layers, n_heads=config.n_heads,
                       n_kv_heads=config.n_kv_heads, vocab_size=config.vocab_size, seq_len=config.seq_len,
                       rope_freq_base=float(config.rope_freq_base), rope_is_neox=int(bool(config.rope_is_neox)),
                       act_planes=act_planes, device=device, tp_size=tp_size, tp_rank=tp_rank)
        self.model = C.c_void_p()
        self.session = C.c_void_p()
        L.check(lib.l2b_model_create(C.byref(cfg), C.byref(self.model)))
        try:
            def up(role, layer, a, vector=False):
                if vector:
                    v = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
                    L.check(lib.l2b_model_upload_tensor(self.model, role, layer, L.TYPE_F32, L.ptr(v), v.size, 1))
                else:
                    t, data, i, o = _matrix_info(a)
                    L.check(lib.l2b_model_upload_tensor(self.model, role, layer, t, L.ptr(data), i, o))
            up(L.ROLE_TOKEN_EMBEDDING, 0, weights.token_embedding_table)
            up(L.ROLE_OUTPUT, 0, weights.output_weight)
            up(L.ROLE_RMS_FINAL, 0, weights.rms_final_weight, vector=True)
            for l, w in enumerate(weights.layers):
                up(L.ROLE_RMS_ATT, l, w.rms_att_weight, vector=True)
                up(L.ROLE_RMS_FFN, l, w.rms_ffn_weight, vector=True)
                for role, a in ((L.ROLE_WQ, w.wq), (L.ROLE_WK, w.wk), (L.ROLE_WV, w.wv), (L.ROLE_WO, w.wo),
                                (L.ROLE_W1, w.w1), (L.ROLE_W2, w.w2), (L.ROLE_W3, w.w3)):
                    up(role, l, a)
            L.check(lib.l2b_model_finalize(self.model))
            L.check(lib.l2b_session_create(self.model, stream, C.byref(self.session)))
        except Exception:
            self.close()
            raise

    @classmethod
    def from_gguf(cls, path: str, seq_len: int, act_planes=0, device=-1, stream=None, tp_size=1, tp_rank=0):
        """Weights loaded by the library's own GGUF reader (l2b_model_load_gguf); returns (device model, ModelConfig)."""
        lib = L.lib()
        self = cls.__new__(cls)
        self.model, self.session = C.c_void_p(), C.c_void_p()
        cfg = L.Config()
        L.check(lib.l2b_model_load_gguf(path.encode(), int(seq_len), act_planes, device, tp_size, tp_rank, C.byref(cfg), C.byref(self.model)))
        try:
            L.check(lib.l2b_session_create(self.model, stream, C.byref(self.session)))
        except Exception:
            self.close()
            raise
        config = ModelConfig(cfg.dim, cfg.hidden_dim, cfg.n_layers, cfg.n_heads, cfg.n_kv_heads, cfg.vocab_size, cfg.seq_len,
                             float(cfg.rope_freq_base), bool(cfg.rope_is_neox))
        return self, config

    def close(self):
        lib = L.lib()
        if self.session:
            lib.l2b_session_destroy(self.session)
            self.session = C.c_void_p()
        if self.model:
            lib.l2b_model_destroy(self.model)
            self.model = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class LanguageModel:
    """src/inference.jl:50-54.  Constructible from plain arrays: LanguageModel(config, tokenizer, weights).

    `act_planes` (1..3, 0 = library default 3) selects how many int8 planes represent an activation in the
    k-quant integer dot products; the device copy of the weights is made on first use.
    """

    def __init__(self, config: ModelConfig, tokenizer, weights: TransformerWeights, act_planes: int = 0, device: int = -1, stream=None,
                 tp_size: int = 1, tp_rank: int = 0):
        self.config, self.tokenizer, self.weights = config, tokenizer, weights
        self.act_planes, self.device, self.stream = act_planes, device, stream
        self.tp_size, self.tp_rank = tp_size, tp_rank  # tensor parallelism: see tp.py (one process per GPU)
        self._dev: Optional[_DeviceModel] = None

    def device_model(self) -> _DeviceModel:
        if self._dev is None:
            self._dev = _DeviceModel(self.config, self.weights, self.act_planes, self.device, self.stream, self.tp_size, self.tp_rank)
        return self._dev

    def close(self):
        if self._dev is not None:
            self._dev.close()
            self._dev = None

    def __str__(self):  # src/inference.jl:56-60
        return "LanguageModel(\n" + str(self.config) + ")"

    # -- measurement helpers --------------------------------------------------------------
    def weight_bytes_per_token(self) -> int:
        n = C.c_int64()
        L.check(L.lib().l2b_model_weight_bytes(self.device_model().model, C.byref(n)))
        return n.value

    def kernels_per_token(self) -> int:
        n = C.c_int32()
        L.check(L.lib().l2b_session_kernels_per_token(self.device_model().session, C.byref(n)))
        return n.value

    def prefill_pairs(self) -> bool:
        """True when `generate` feeds prompts two positions per pass over the weights."""
        n = C.c_int32()
        L.check(L.lib().l2b_session_prefill_pairs(self.device_model().session, C.byref(n)))
        return bool(n.value)

    def prefill_gemm_min_tokens(self) -> int:
        """Smallest run of forced prompt positions that goes through the tensor-core GEMM pass (0: not available for this model)."""
        n = C.c_int32()
        L.check(L.lib().l2b_session_prefill_gemm(self.device_model().session, C.byref(n)))
        return n.value

    def last_launches(self) -> int:
        """Kernel launches the most recent forward / decode / prefill / generate call enqueued."""
        n = C.c_int64()
        L.check(L.lib().l2b_session_last_launches(self.device_model().session, C.byref(n)))
        return n.value

    def last_phase_ms(self):
        """(prompt ms, decode ms) of the most recent `generate`: positions fed prompt tokens / positions fed generated tokens."""
        a, b = C.c_float(), C.c_float()
        L.check(L.lib().l2b_session_last_phase_ms(self.device_model().session, C.byref(a), C.byref(b)))
        return a.value, b.value

    def last_device_ms(self) -> float:
        ms = C.c_float()
        L.check(L.lib().l2b_session_last_device_ms(self.device_model().session, C.byref(ms)))
        return ms.value


class RunState:
    """src/inference.jl:72-100: the per-call state.  Here it is a handle on the device session;
    creating one zeroes the KV cache exactly like `RunState(config)`."""

    def __init__(self, model: LanguageModel):
        self.model = model
        self.session = model.device_model().session
        L.check(L.lib().l2b_session_reset(self.session))
        self.logits = np.zeros(model.config.vocab_size, dtype=np.float32)


class BatchRunState:
    """Several RunStates (src/inference.jl:72-100) decoded in lock step: one zeroed KV cache per sequence, one position per call
    for all of them.  No counterpart in the reference, whose `sample` serves one prompt; the per-sequence arithmetic is
    transformer! unchanged."""

    def __init__(self, model: LanguageModel, n_seq: int):
        self.model, self.n_seq = model, n_seq
        self.batch = C.c_void_p()
        L.check(L.lib().l2b_batch_create(model.device_model().model, int(n_seq), C.byref(self.batch)))
        self.logits = np.zeros((n_seq, model.config.vocab_size), dtype=np.float32)

    def decode_next(self, tokens, positions, want_logits: bool = False) -> np.ndarray:
        """tokens[i] at position positions[i] of sequence i; returns the greedy next token of every sequence."""
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        p = np.ascontiguousarray(positions, dtype=np.int32)
        if t.size != self.n_seq or p.size != self.n_seq:
            raise ValueError("one token and one position per sequence")
        nxt = np.zeros(self.n_seq, dtype=np.int32)
        L.check(L.lib().l2b_batch_decode_next(self.batch, L.ptr(t), L.ptr(p), L.ptr(nxt), L.ptr(self.logits) if want_logits else None))
        return nxt

    def reset(self):
        L.check(L.lib().l2b_batch_reset(self.batch))

    def close(self):
        if self.batch:
            L.lib().l2b_batch_destroy(self.batch)
            self.batch = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def matmul_(y: np.ndarray, A: Matrix, x: np.ndarray, act_planes: int = 0) -> None:
    """matmul!(y, A, x): y .= A' * x (src/matmul.jl:3-23).  x may hold several columns, shape (ncols, in)."""
    t, data, i, o = _matrix_info(A)
    x32 = np.ascontiguousarray(x, dtype=np.float32)
    ncols = 1 if x32.ndim == 1 else x32.shape[0]
    if x32.size != ncols * i:
        raise ValueError("length(x) must equal the matrix input dimension")
    if y.dtype != np.float32 or not y.flags.c_contiguous or y.size != ncols * o:
        raise ValueError("y must be a contiguous float32 array of ncols * out elements")
    L.check(L.lib().l2b_matvec(t, L.ptr(data), i, o, L.ptr(x32), ncols, L.ptr(y), act_planes))


def dequantize(x: QuantMatrix) -> np.ndarray:
    """dequantize(x) (src/kquants.jl:49-53)."""
    n = x.in_dim * x.out_dim
    y = np.zeros(n, dtype=np.float32)
    L.check(L.lib().l2b_dequantize(x.ggml_type, L.ptr(x.data), n, L.ptr(y)))
    return y


def transformer_(token: int, pos: int, config: ModelConfig, s: RunState, weights: TransformerWeights = None) -> None:
    """transformer!(token, pos, config, s, weights) (src/inference.jl:222-315): fills s.logits, advances the KV cache.
    token and pos are 0-based."""
    L.check(L.lib().l2b_forward(s.session, int(token), int(pos), L.ptr(s.logits)))


def prefill(s: RunState, tokens, pos0: int = 0) -> int:
    """The prompt phase of `sample` (src/inference.jl:349-356) in one call: tokens at positions pos0.., two positions per pass
    over the weights where possible.  Returns the argmax after the last prompt position; its logits are read with
    l2b_session_logits (s.logits is filled)."""
    t = np.ascontiguousarray(tokens, dtype=np.int32)
    nxt = C.c_int32()
    L.check(L.lib().l2b_prefill(s.session, L.ptr(t), t.size, int(pos0), C.byref(nxt)))
    L.check(L.lib().l2b_session_logits(s.session, L.ptr(s.logits)))
    return nxt.value


def generate(model: LanguageModel, prompt_tokens, n_positions: int, temperature: float = 0.0, seed: int = 0):
    """The loop of `sample` without text: returns (tokens chosen after each position, device milliseconds)."""
    dev = model.device_model()
    L.check(L.lib().l2b_session_reset(dev.session))
    p = np.ascontiguousarray(prompt_tokens, dtype=np.int32)
    out = np.zeros(n_positions, dtype=np.int32)
    ms = C.c_float()
    L.check(L.lib().l2b_generate(dev.session, L.ptr(p), p.size, n_positions, float(temperature), int(seed), L.ptr(out), C.byref(ms)))
    return out, ms.value


def _text(tok) -> str:
    return tok.decode("utf-8", errors="replace") if isinstance(tok, (bytes, bytearray)) else tok


def sample(model: LanguageModel, prompt: str = "", *, temperature: float = 0.9, stop_on_special_token: bool = True,
           max_seq_len: int = sys.maxsize, bos_token: bool = True, rng: Optional[random.Random] = None, out=None) -> None:
    """sample(model, prompt; temperature, stop_on_special_token, max_seq_len, bos_token) (src/inference.jl:317-395).

    Prints the text and the achieved tok/s like the reference and returns None.  The prompt positions whose next token is
    a prompt token go through one l2b_prefill call (unless the stop condition could fire among them); every other position
    is one l2b_decode_next call (token id in, next token id out)."""
    from .tokenizer import encode
    out = out or sys.stdout
    if not bos_token and prompt == "":
        raise ValueError("Prompt cannot be empty if bos_token = false")
    config, tokenizer = model.config, model.tokenizer
    prompt_tokens = list(encode(prompt, tokenizer))
    state = RunState(model)
    rng = rng or random
    time_start = time.perf_counter_ns()
    if bos_token:
        prompt_tokens.insert(0, tokenizer.bos_token_id)
    else:
        out.write(_text(tokenizer.id_to_token[prompt_tokens[0]]))
    token = prompt_tokens[0]
    generated_seq_len = 0
    lib = L.lib()
    nxt = C.c_int32()
    limit = min(config.seq_len, max_seq_len)
    first = 0
    n_forced = len(prompt_tokens) - 1  # positions 0 .. n_forced-1 are followed by a prompt token
    specials = (tokenizer.bos_token_id, tokenizer.eos_token_id)
    if n_forced >= 2 and n_forced <= limit and not (stop_on_special_token and any(t in specials for t in prompt_tokens[1:])):
        t = np.ascontiguousarray(prompt_tokens[:n_forced], dtype=np.int32)
        L.check(lib.l2b_prefill(state.session, L.ptr(t), t.size, 0, None))
        for tok in prompt_tokens[1:]:
            out.write(_text(tokenizer.id_to_token[tok]))
        generated_seq_len = n_forced
        token = prompt_tokens[n_forced]
        first = n_forced
    for pos in range(first, limit):
        L.check(lib.l2b_decode_next(state.session, int(token), pos, float(temperature), rng.random() if temperature != 0 else 0.0,
                                    C.byref(nxt)))
        generated_seq_len += 1
        next_token = prompt_tokens[pos + 1] if pos + 1 < len(prompt_tokens) else nxt.value
        if stop_on_special_token and next_token in (tokenizer.bos_token_id, tokenizer.eos_token_id):
            break
        out.write(_text(tokenizer.id_to_token[next_token]))
        token = next_token
    out.write("\n")
    dt = time.perf_counter_ns() - time_start
    out.write("-------\nachieved tok/s: %.2f\n" % (generated_seq_len / dt * 1e9))
    return None
