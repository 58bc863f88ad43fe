"""ctypes binding of the CPU oracle (liboracle.so, beside this file).  Test infrastructure only: imported by tests/,
by the smoke check and by the CPU-baseline leg of bench.py; the library itself never loads it."""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(HERE, "liboracle.so")
ACC_SEQ, ACC_LANES, ACC_F64 = 0, 1, 2
F32, Q4_K, Q5_K, Q6_K = 0, 12, 13, 14
BLOCK_BYTES = {Q4_K: 144, Q5_K: 176, Q6_K: 210}


class _Config(C.Structure):
    _fields_ = [("dim", C.c_int32), ("hidden_dim", C.c_int32), ("n_layers", C.c_int32), ("n_heads", C.c_int32),
                ("n_kv_heads", C.c_int32), ("vocab_size", C.c_int32), ("seq_len", C.c_int32),
                ("rope_freq_base", C.c_float), ("rope_is_neox", C.c_int32)]


def _load():
    src = os.path.join(HERE, "oracle.cpp")
    if not os.path.exists(_PATH) or os.path.getmtime(_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-s", "-C", HERE], check=True)
    lib = C.CDLL(_PATH)
    P = C.c_void_p
    sig = {
        "orc_dequantize": ([C.c_int, P, C.c_int64, P], None),
        "orc_vecdot": ([C.c_int, P, C.c_int64, P, C.c_int], C.c_double),
        "orc_matmul": ([C.c_int, P, C.c_int64, C.c_int64, P, P, C.c_int, C.c_int], None),
        "orc_matmul_f64": ([C.c_int, P, C.c_int64, C.c_int64, P, P, C.c_int], None),
        "orc_rmsnorm": ([P, P, P, C.c_int64], None),
        "orc_rope": ([P, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int], None),
        "orc_rope_table_row": ([P, C.c_int, C.c_int, C.c_float], None),
        "orc_softmax": ([P, C.c_int64], None),
        "orc_attention": ([P, P, P, P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int], None),
        "orc_swiglu": ([P, P, C.c_int64], None),
        "orc_argmax": ([P, C.c_int64], C.c_int64),
        "orc_sample_temperature": ([P, C.c_int64, C.c_float, C.c_double], C.c_int64),
        "orc_model_create": ([C.POINTER(_Config)], P),
        "orc_model_destroy": ([P], None),
        "orc_model_set_tensor": ([P, C.c_int, C.c_int, C.c_int, P, C.c_int64, C.c_int64], C.c_int),
        "orc_state_create": ([P], P),
        "orc_state_destroy": ([P], None),
        "orc_transformer": ([P, P, C.c_int, C.c_int, C.c_int, C.c_int, P], None),
        "orc_state_read": ([P, C.c_int, P, C.c_int64], C.c_int64),
        "orc_sample_greedy": ([P, P, C.c_int, C.c_int, P, P, C.c_int, C.c_int], C.c_double),
        "orc_hardware_threads": ([], C.c_int),
    }
    for name, (a, r) in sig.items():
        f = getattr(lib, name)
        f.argtypes, f.restype = a, r
    return lib


lib = _load()
NTHREADS = max(1, lib.orc_hardware_threads())


def dequantize(ggml_type, raw, n_elems):
    out = np.empty(n_elems, dtype=np.float32)
    lib.orc_dequantize(ggml_type, raw.ctypes.data, n_elems if ggml_type == F32 else n_elems // 256, out.ctypes.data)
    return out


def _minfo(a):
    """(type, contiguous buffer, in, out) of a numpy f32 (out, in) matrix or a QuantMatrix-like object."""
    if hasattr(a, "ggml_type"):
        return a.ggml_type, a.data, a.in_dim, a.out_dim
    a32 = np.ascontiguousarray(a, dtype=np.float32)
    return F32, a32, a32.shape[1], a32.shape[0]


def matmul(A, x, acc=ACC_SEQ, nthreads=None):
    t, data, i, o = _minfo(A)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(o, dtype=np.float32)
    lib.orc_matmul(t, data.ctypes.data, i, o, x.ctypes.data, y.ctypes.data, acc, nthreads or NTHREADS)
    return y


def matmul_f64(A, x, nthreads=None):
    t, data, i, o = _minfo(A)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(o, dtype=np.float64)
    lib.orc_matmul_f64(t, data.ctypes.data, i, o, x.ctypes.data, y.ctypes.data, nthreads or NTHREADS)
    return y


def rmsnorm(x, w):
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    o = np.empty_like(x)
    lib.orc_rmsnorm(o.ctypes.data, x.ctypes.data, w.ctypes.data, x.size)
    return o


def rope(x, head_size, n_heads, pos0, base, neox):
    y = np.array(x, dtype=np.float32, copy=True)
    lib.orc_rope(y.ctypes.data, head_size, n_heads, pos0, base, int(neox))
    return y


def softmax(x):
    y = np.array(x, dtype=np.float32, copy=True)
    lib.orc_softmax(y.ctypes.data, y.size)
    return y


def attention(q, k, v, n_heads, n_kv, hs):
    """q [n_heads][hs]; k, v [npos][n_kv][hs] (position-major).  The oracle wants the value cache as [kv][hs][seq]."""
    npos = k.shape[0]
    kc = np.ascontiguousarray(k, dtype=np.float32)
    vc = np.ascontiguousarray(np.transpose(v.reshape(npos, n_kv, hs), (1, 2, 0)), dtype=np.float32)
    q = np.ascontiguousarray(q, dtype=np.float32)
    out = np.empty(n_heads * hs, dtype=np.float32)
    lib.orc_attention(out.ctypes.data, q.ctypes.data, kc.ctypes.data, vc.ctypes.data, npos, npos, n_heads, n_kv, hs)
    return out


def swiglu(hb, hb2):
    a = np.array(hb, dtype=np.float32, copy=True)
    b = np.ascontiguousarray(hb2, dtype=np.float32)
    lib.orc_swiglu(a.ctypes.data, b.ctypes.data, a.size)
    return a


def argmax(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    return int(lib.orc_argmax(x.ctypes.data, x.size))


def sample_temperature(logits, temperature, u):
    x = np.array(logits, dtype=np.float32, copy=True)
    return int(lib.orc_sample_temperature(x.ctypes.data, x.size, temperature, u)), x


ROLES = dict(tok=0, rms_att=1, wq=2, wk=3, wv=4, wo=5, rms_ffn=6, w1=7, w2=8, w3=9, rms_final=10, output=11)


class OracleModel:
    """transformer! / sample of the oracle over the same host arrays the device model was built from."""

    def __init__(self, config, weights):
        self.config = config
        self._keep = []
        c = _Config(config.dim, config.hidden_dim, config.n_layers, config.n_heads, config.n_kv_heads, config.vocab_size,
                    config.seq_len, float(config.rope_freq_base), int(bool(config.rope_is_neox)))
        self.m = lib.orc_model_create(C.byref(c))
        self._set("tok", 0, weights.token_embedding_table)
        self._set("output", 0, weights.output_weight)
        self._setv("rms_final", 0, weights.rms_final_weight)
        for l, w in enumerate(weights.layers):
            self._setv("rms_att", l, w.rms_att_weight)
            self._setv("rms_ffn", l, w.rms_ffn_weight)
            for name in ("wq", "wk", "wv", "wo", "w1", "w2", "w3"):
                self._set(name, l, getattr(w, name))
        self.state = None

    def _set(self, role, layer, a):
        t, data, i, o = _minfo(a)
        self._keep.append(data)
        assert lib.orc_model_set_tensor(self.m, ROLES[role], layer, t, data.ctypes.data, i, o) == 0

    def _setv(self, role, layer, v):
        v = np.ascontiguousarray(v, dtype=np.float32)
        self._keep.append(v)
        assert lib.orc_model_set_tensor(self.m, ROLES[role], layer, F32, v.ctypes.data, v.size, 1) == 0

    def reset(self):
        if self.state:
            lib.orc_state_destroy(self.state)
        self.state = lib.orc_state_create(self.m)

    def transformer(self, token0, pos0, acc=ACC_LANES, nthreads=None):
        if self.state is None:
            self.reset()
        logits = np.empty(self.config.vocab_size, dtype=np.float32)
        lib.orc_transformer(self.m, self.state, int(token0), int(pos0), acc, nthreads or NTHREADS, logits.ctypes.data)
        return logits

    def read(self, which, n):
        out = np.empty(n, dtype=np.float32)
        lib.orc_state_read(self.state, which, out.ctypes.data, n)
        return out

    def sample_greedy(self, prompt, n_positions, want_logits=False, acc=ACC_LANES, nthreads=None):
        p = np.ascontiguousarray(prompt, dtype=np.int32)
        out = np.empty(n_positions, dtype=np.int32)
        logits = np.empty((n_positions, self.config.vocab_size), dtype=np.float32) if want_logits else None
        self.seconds = lib.orc_sample_greedy(self.m, p.ctypes.data, p.size, n_positions, out.ctypes.data,
                                             None if logits is None else logits.ctypes.data, acc, nthreads or NTHREADS)
        return (out, logits) if want_logits else out

    def __del__(self):
        try:
            if self.state:
                lib.orc_state_destroy(self.state)
            lib.orc_model_destroy(self.m)
        except Exception:
            pass
