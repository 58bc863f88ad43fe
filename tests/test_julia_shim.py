"""The Julia binding (llama2.jl_b200/julia/Llama2B200.jl) cannot be run where this repository is built (no Julia), so its
`ccall`s are checked as text: every call must name an exported entry point and carry the argument and return types of the
Python ctypes binding that the GPU tests drive, and the file must define new methods on new types only."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "llama2.jl_b200", "julia", "Llama2B200.jl")


def _julia_kind(t):
    t = t.strip()
    if t.startswith(("Ptr{", "Ref{")) or t == "Cstring":
        return "ptr"
    return {"Int32": "i32", "Int64": "i64", "Float32": "f32", "Float64": "f64", "UInt64": "u64"}[t]


def _ctypes_kind(t):
    if t in (C.c_void_p, C.c_char_p) or (isinstance(t, type) and issubclass(t, C._Pointer)):
        return "ptr"
    return {C.c_int32: "i32", C.c_int64: "i64", C.c_float: "f32", C.c_double: "f64", C.c_uint64: "u64"}[t]


def _split_top(s):
    out, depth, cur = [], 0, ""
    for ch in s:
        if ch in "{(":
            depth += 1
        elif ch in "})":
            depth -= 1
        if ch == "," and depth == 0:
            out.append(cur)
            cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur)
    return out


def test_every_ccall_matches_the_ctypes_binding(pkg):
    from llama2_jl_b200 import _lib as L
    src = open(SHIM).read()
    calls = re.findall(r"ccall\(\(:(l2b_[a-z0-9_]+), LIB\),\s*([A-Za-z0-9{}]+),\s*\(([^()]*(?:\{[^{}]*\}[^()]*)*)\)", src)
    assert len(calls) >= 12
    seen = set()
    for name, ret, args in calls:
        assert name in L._SIGNATURES, f"{name} is not an entry point of the library"
        argtypes, restype = L._SIGNATURES[name]
        got = [_julia_kind(a) for a in _split_top(args)]
        want = [_ctypes_kind(a) for a in argtypes]
        assert got == want, (name, got, want)
        assert _julia_kind(ret) == _ctypes_kind(restype), name
        seen.add(name)
    # the calls the device path of `sample` is made of
    for needed in ("l2b_model_create", "l2b_model_upload_tensor", "l2b_model_finalize", "l2b_session_create", "l2b_forward",
                   "l2b_decode_next", "l2b_prefill", "l2b_matrix_create", "l2b_matrix_matvec", "l2b_last_error_string"):
        assert needed in seen, needed


def test_shim_defines_new_methods_on_new_types_only():
    src = open(SHIM).read()
    code = "\n".join(l for l in src.splitlines() if not l.lstrip().startswith("#"))
    # methods of the package's functions must dispatch on one of the shim's own types
    assert re.search(r"function matmul!\(y::AbstractVector\{Float32\}, A::B200Matrix,", code)
    assert re.search(r"function transformer!\(token::Int, pos::Int, config::ModelConfig, s::B200RunState, weights::B200Weights\)", code)
    assert re.search(r"function sample\(\s*model::B200LanguageModel,", code)
    for fn in ("matmul!", "transformer!", "sample"):
        for sig in re.findall(r"function " + re.escape(fn) + r"\(([^)]*)\)", code):
            assert "B200" in sig, f"{fn}({sig}) would overwrite a method of the package"
    # nothing defined and never used: the loop calls prefill! and decode_next, the stop rule is there
    body = code[code.index("function sample("):]
    assert "prefill!(state" in body and "decode_next(state" in body
    assert "next == tokenizer.bos_token_id || next == tokenizer.eos_token_id" in body
    # sessions belong to run states, not to a table keyed by weights
    assert "IdDict" not in code and "l2b_session_create" in code[code.index("function B200RunState("):code.index("function transformer!(")]


def test_config_struct_matches_the_c_struct(pkg):
    from llama2_jl_b200 import _lib as L
    src = open(SHIM).read()
    body = src[src.index("struct L2BConfig"):src.index("\nend", src.index("struct L2BConfig"))]
    fields = re.findall(r"([a-z_]+)::(Int32|Float32|NTuple\{7,Int32\})", body)
    want = [(n, {C.c_int32: "Int32", C.c_float: "Float32"}.get(t, "NTuple{7,Int32}")) for n, t in L.Config._fields_]
    assert fields == want
