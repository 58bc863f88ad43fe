"""ctypes binding of the C ABI declared in include/llama2_b200.h.

The shared library is built in-tree (see build.py).  Importing this module never falls back
to a CPU implementation: if the library is missing, `lib()` raises, and without a CUDA device
every compute entry point returns L2B_ERR_NO_DEVICE, which `check` turns into an exception.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("L2B_LIBRARY") or os.path.join(_HERE, "libllama2_b200.so")

OK, ERR_BAD_ARG, ERR_UNSUPPORTED_TYPE, ERR_CUDA, _ERR_UNUSED, ERR_TIMEOUT, ERR_OOM, ERR_STATE, ERR_NO_DEVICE = range(9)
TYPE_F32, TYPE_Q4_K, TYPE_Q5_K, TYPE_Q6_K = 0, 12, 13, 14
BLOCK_BYTES = {TYPE_Q4_K: 144, TYPE_Q5_K: 176, TYPE_Q6_K: 210}
(ROLE_TOKEN_EMBEDDING, ROLE_RMS_ATT, ROLE_WQ, ROLE_WK, ROLE_WV, ROLE_WO, ROLE_RMS_FFN, ROLE_W1, ROLE_W2, ROLE_W3,
 ROLE_RMS_FINAL, ROLE_OUTPUT) = range(12)


class L2BError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"llama2_b200 status {status}: {message}")
        self.status = status


class Config(C.Structure):
    """l2b_config: ModelConfig (src/inference.jl:1-11) field for field, then library options."""
    _fields_ = [
        ("dim", C.c_int32), ("hidden_dim", C.c_int32), ("n_layers", C.c_int32), ("n_heads", C.c_int32),
        ("n_kv_heads", C.c_int32), ("vocab_size", C.c_int32), ("seq_len", C.c_int32),
        ("rope_freq_base", C.c_float), ("rope_is_neox", C.c_int32),
        ("act_planes", C.c_int32), ("device", C.c_int32), ("tp_size", C.c_int32), ("tp_rank", C.c_int32),
        ("reserved", C.c_int32 * 7),
    ]


_P = C.c_void_p
_SIGNATURES = {
    "l2b_version": ([], C.c_int32),
    "l2b_last_error_string": ([], C.c_char_p),
    "l2b_status_string": ([C.c_int32], C.c_char_p),
    "l2b_device_count": ([C.POINTER(C.c_int32)], C.c_int32),
    "l2b_model_create": ([C.POINTER(Config), C.POINTER(_P)], C.c_int32),
    "l2b_model_upload_tensor": ([_P, C.c_int32, C.c_int32, C.c_int32, _P, C.c_int64, C.c_int64], C.c_int32),
    "l2b_model_finalize": ([_P], C.c_int32),
    "l2b_model_destroy": ([_P], C.c_int32),
    "l2b_model_weight_bytes": ([_P, C.POINTER(C.c_int64)], C.c_int32),
    "l2b_session_create": ([_P, _P, C.POINTER(_P)], C.c_int32),
    "l2b_session_reset": ([_P], C.c_int32),
    "l2b_session_destroy": ([_P], C.c_int32),
    "l2b_forward": ([_P, C.c_int32, C.c_int32, _P], C.c_int32),
    "l2b_decode_next": ([_P, C.c_int32, C.c_int32, C.c_float, C.c_double, C.POINTER(C.c_int32)], C.c_int32),
    "l2b_generate": ([_P, _P, C.c_int32, C.c_int32, C.c_float, C.c_uint64, _P, C.POINTER(C.c_float)], C.c_int32),
    "l2b_session_logits": ([_P, _P], C.c_int32),
    "l2b_session_read": ([_P, C.c_int32, _P, C.c_int64, C.POINTER(C.c_int64)], C.c_int32),
    "l2b_session_last_device_ms": ([_P, C.POINTER(C.c_float)], C.c_int32),
    "l2b_session_last_phase_ms": ([_P, C.POINTER(C.c_float), C.POINTER(C.c_float)], C.c_int32),
    "l2b_session_last_launches": ([_P, C.POINTER(C.c_int64)], C.c_int32),
    "l2b_session_kernels_per_token": ([_P, C.POINTER(C.c_int32)], C.c_int32),
    "l2b_dequantize": ([C.c_int32, _P, C.c_int64, _P], C.c_int32),
    "l2b_quantize_q8k": ([_P, C.c_int64, C.c_int32, _P, _P, _P], C.c_int32),
    "l2b_rmsnorm_quantize_q8k": ([_P, _P, C.c_int64, C.c_int32, _P, _P, _P], C.c_int32),
    "l2b_matvec": ([C.c_int32, _P, C.c_int64, C.c_int64, _P, C.c_int32, _P, C.c_int32], C.c_int32),
    "l2b_rmsnorm": ([_P, _P, _P, C.c_int64], C.c_int32),
    "l2b_rope": ([_P, C.c_int32, C.c_int32, C.c_int32, C.c_float, C.c_int32], C.c_int32),
    "l2b_attention": ([_P, _P, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32], C.c_int32),
    "l2b_model_load_gguf": ([C.c_char_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, C.POINTER(_P)], C.c_int32),
    "l2b_gguf_inspect": ([C.c_char_p, _P, C.POINTER(C.c_int32), C.POINTER(C.c_int64), C.POINTER(C.c_int64)], C.c_int32),
    "l2b_batch_create": ([_P, C.c_int32, C.POINTER(_P)], C.c_int32),
    "l2b_batch_reset": ([_P], C.c_int32),
    "l2b_batch_destroy": ([_P], C.c_int32),
    "l2b_batch_decode_next": ([_P, _P, _P, _P, _P], C.c_int32),
    "l2b_tokenizer_create": ([_P, _P, C.c_int32, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.POINTER(_P)], C.c_int32),
    "l2b_tokenizer_load_gguf": ([C.c_char_p, C.POINTER(_P)], C.c_int32),
    "l2b_tokenizer_destroy": ([_P], C.c_int32),
    "l2b_tokenizer_info": ([_P, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)], C.c_int32),
    "l2b_tokenizer_token": ([_P, C.c_int32, C.POINTER(_P), C.POINTER(C.c_int64)], C.c_int32),
    "l2b_tokenizer_encode": ([_P, _P, C.c_int64, C.c_int32, _P, C.c_int64, C.POINTER(C.c_int64)], C.c_int32),
    "l2b_prefill": ([_P, _P, C.c_int32, C.c_int32, C.POINTER(C.c_int32)], C.c_int32),
    "l2b_session_prefill_gemm": ([_P, C.POINTER(C.c_int32)], C.c_int32),
    "l2b_session_prefill_pairs": ([_P, C.POINTER(C.c_int32)], C.c_int32),
    "l2b_session_tp_handle": ([_P, _P], C.c_int32),
    "l2b_session_tp_connect": ([_P, _P, C.c_int32], C.c_int32),
    "l2b_attention_device_noalloc": ([_P, _P, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P], C.c_int32),
    "l2b_swiglu": ([_P, _P, C.c_int64], C.c_int32),
    "l2b_argmax": ([_P, C.c_int64, C.POINTER(C.c_int32)], C.c_int32),
    "l2b_sample_temperature": ([_P, C.c_int64, C.c_float, C.c_double, C.POINTER(C.c_int32)], C.c_int32),
    "l2b_matrix_create": ([C.c_int32, _P, C.c_int64, C.c_int64, C.c_int32, C.POINTER(_P)], C.c_int32),
    "l2b_matrix_destroy": ([_P], C.c_int32),
    "l2b_matrix_matvec_device": ([_P, C.c_int32, _P, _P, C.c_int32, _P], C.c_int32),
    "l2b_matrix_matmul_device": ([_P, C.c_int32, _P, C.c_int32, _P, _P], C.c_int32),
    "l2b_matrix_matvec": ([_P, _P, C.c_int32, _P, C.c_int32], C.c_int32),
}
# include/l2b_synth.h: the test-support library of seeded synthetic data (libl2b_synth.so, no CUDA)
SYNTH_LIB_PATH = os.path.join(_HERE, "libl2b_synth.so")
_SYNTH_SIGNATURES = {
    "l2b_synth_f32": ([_P, C.c_int64, C.c_uint64, C.c_float, C.c_int32], C.c_int32),
    "l2b_synth_kquant": ([C.c_int32, _P, C.c_int64, C.c_uint64], C.c_int32),
    "l2b_synth_tokens": ([_P, C.c_int64, C.c_uint64, C.c_int32, C.c_int32], C.c_int32),
}
_synth = None


def synth_lib():
    """The synthetic-data library; loading it does not load the CUDA library."""
    global _synth
    if _synth is None:
        if not os.path.exists(SYNTH_LIB_PATH):
            raise ImportError(f"{SYNTH_LIB_PATH} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()')")
        handle = C.CDLL(SYNTH_LIB_PATH)
        for name, (argtypes, restype) in _SYNTH_SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _synth = handle
    return _synth


def synth_check(status):
    if status != OK:
        raise L2BError(status, "synthetic-data generator: bad argument or unsupported tensor type")

_lib = None


def lib():
    """The loaded shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()')")
        handle = C.CDLL(LIB_PATH)
        for name, (argtypes, restype) in _SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here = the library does not export a declared symbol
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = handle
    return _lib


def exported_symbols():
    return sorted(_SIGNATURES)


def check(status):
    if status != OK:
        raise L2BError(status, lib().l2b_last_error_string().decode() or lib().l2b_status_string(status).decode())


def ptr(a):
    """Address of a contiguous numpy array (or None)."""
    return None if a is None else a.ctypes.data
