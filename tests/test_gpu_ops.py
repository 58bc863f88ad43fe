"""GPU parity of the isolated operators, through the C ABI, against the CPU oracle."""
import ctypes as C
import os

import numpy as np
import pytest

from test_oracle import TYPES, random_blocks

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


class QM:
    def __init__(self, t, raw, in_dim, out_dim):
        self.ggml_type, self.data, self.in_dim, self.out_dim = t, np.ascontiguousarray(raw).reshape(-1), in_dim, out_dim


@pytest.fixture(scope="module")
def L(pkg):
    from llama2_jl_b200 import _lib
    return _lib


# ---- dequantize!: bit-exact ------------------------------------------------------------------
@pytest.mark.parametrize("name", list(TYPES))
def test_dequantize_bit_exact(L, orc, synth, name):
    t, bb = TYPES[name]
    for raw in (random_blocks(name, 257, 21), synth.kquant_bytes(t, 64, 5).reshape(64, bb)):
        n = raw.shape[0] * 256
        got = np.empty(n, dtype=np.float32)
        L.check(L.lib().l2b_dequantize(t, L.ptr(raw), n, L.ptr(got)))
        assert np.array_equal(got.view(np.uint32), orc.dequantize(t, raw, n).view(np.uint32))


@pytest.mark.parametrize("name", list(TYPES))
def test_dequantize_golden_and_corners(L, orc, name):
    t, bb = TYPES[name]
    g = np.load(os.path.join(GOLDEN, "kquants_golden.npz"))
    raw = g[f"{name}_raw"]
    got = np.empty(raw.shape[0] * 256, dtype=np.float32)
    L.check(L.lib().l2b_dequantize(t, L.ptr(raw), got.size, L.ptr(got)))
    assert np.array_equal(got.view(np.uint32), g[f"{name}_dequant_bits"])
    # all-zero and all-ones blocks, and the scale bytes at their corner values
    cases = [np.zeros((1, bb), np.uint8), np.full((1, bb), 0xFF, np.uint8)]
    if name != "q6_K":
        base = random_blocks(name, 1, 3)
        for byte in (0x00, 0x3F, 0x40, 0xC0, 0xFF):
            for i in range(12):
                b = base.copy()
                b[0, 4 + i] = byte
                cases.append(b)
    raw = np.concatenate(cases)
    raw[1, (208 if name == "q6_K" else 0):(210 if name == "q6_K" else 4)] = 0  # keep d finite (0xFFFF is a NaN half)
    got = np.empty(raw.shape[0] * 256, dtype=np.float32)
    L.check(L.lib().l2b_dequantize(t, L.ptr(raw), got.size, L.ptr(got)))
    assert np.array_equal(got.view(np.uint32), orc.dequantize(t, raw, got.size).view(np.uint32))


def test_dequantize_f32_and_empty(L):
    x = np.arange(10, dtype=np.float32)
    y = np.zeros(10, dtype=np.float32)
    L.check(L.lib().l2b_dequantize(0, L.ptr(x), 10, L.ptr(y)))
    assert np.array_equal(x, y)
    L.check(L.lib().l2b_dequantize(12, L.ptr(x), 0, L.ptr(y)))  # empty input is fine
    assert L.lib().l2b_dequantize(12, L.ptr(x), 100, L.ptr(y)) == L.ERR_BAD_ARG  # ragged block count
    assert L.lib().l2b_dequantize(2, L.ptr(x), 256, L.ptr(y)) == L.ERR_UNSUPPORTED_TYPE  # Q4_0 is not implemented


# ---- activation quantisation -------------------------------------------------------------------
@pytest.mark.parametrize("planes", [1, 2, 3])
def test_quantize_q8k(L, planes):
    rng = np.random.default_rng(30)
    n = 2048
    x = rng.normal(size=n).astype(np.float32)
    x[256:512] = 0  # an all-zero block
    x[600] = 37.5   # an outlier
    q = np.zeros((planes, n), dtype=np.int8)
    d = np.zeros((planes, n // 256), dtype=np.float32)
    sums = np.zeros(n // 16, dtype=np.float32)
    L.check(L.lib().l2b_quantize_q8k(L.ptr(x), n, planes, L.ptr(q), L.ptr(d), L.ptr(sums)))
    xb = x.reshape(-1, 256)
    amax = np.abs(xb).max(1)
    assert np.allclose(d[0], amax / 127, rtol=1e-6)
    assert np.abs(q).max() <= 127
    # plane 0 is the q8_K quantisation of the block: round(x / d)
    want0 = np.rint(xb * np.where(amax > 0, 127 / np.maximum(amax, 1e-30), 0)[:, None].astype(np.float32))
    assert np.abs(q[0].reshape(-1, 256) - want0).max() <= 1
    xhat = sum(q[k].reshape(-1, 256).astype(np.float64) * d[k][:, None] for k in range(planes))
    err = np.abs(xhat - xb).max(1)
    bound = amax / 127 / 2 / (254.0 ** (planes - 1)) * 1.01 + 1e-12
    assert np.all(err <= bound), (err / np.maximum(amax, 1e-30)).max()
    assert np.allclose(sums, xhat.reshape(-1, 16).sum(1), rtol=1e-5, atol=1e-6)


# ---- matmul! -------------------------------------------------------------------------------------
def rel_err(got, want64):
    return float(np.abs(got - want64).max() / np.abs(want64).max())


@pytest.mark.parametrize("name", list(TYPES))
@pytest.mark.parametrize("shape", [(256, 16), (4096, 512), (14336, 128), (3072, 96), (1024, 64), (3584, 40)])
def test_matvec_kquant(pkg, orc, synth, name, shape):
    t, bb = TYPES[name]
    n_in, n_out = shape
    A = synth.matrix(t, n_in, n_out, seed=n_in * 31 + n_out + t)
    x = synth.normal_f32(n_in, 77, 1.0)
    want = orc.matmul_f64(A, x)
    tol = {1: 2e-2, 2: 2e-4, 3: 4e-6}
    for planes in (1, 2, 3):
        y = np.zeros(n_out, dtype=np.float32)
        pkg.matmul_(y, A, x, act_planes=planes)
        # error relative to the output scale: 8-bit activations ~1e-2, three planes = f32 reassociation noise
        assert rel_err(y, want) < tol[planes], (planes, rel_err(y, want))
    # the oracle's own f32 orders differ from the f64 sum by about the same amount as the three-plane result
    noise = rel_err(orc.matmul(A, x, acc=orc.ACC_SEQ), want)
    assert rel_err(y, want) < max(4 * noise, 2e-6)


def test_matvec_full_size_and_batch(pkg, orc, synth):
    """The isolated-operator configuration: W 14336 x 4096 q4_K, 1 and 4 activation columns."""
    A = synth.matrix(12, 4096, 14336, seed=1234)
    X = synth.normal_f32(4 * 4096, 78, 1.0).reshape(4, 4096)
    Y = np.zeros((4, 14336), dtype=np.float32)
    pkg.matmul_(Y, A, X)
    for c in range(4):
        e = rel_err(Y[c], orc.matmul_f64(A, X[c]))
        assert e < 4e-6, (c, e)
    # linearity, a size-independent property: A'(2x) == 2 A'x exactly (power-of-two scaling commutes with rounding)
    y1 = np.zeros(14336, dtype=np.float32)
    y2 = np.zeros(14336, dtype=np.float32)
    pkg.matmul_(y1, A, X[0])
    pkg.matmul_(y2, A, 2 * X[0])
    assert np.array_equal(2 * y1, y2)
    y3 = np.zeros(14336, dtype=np.float32)
    pkg.matmul_(y3, A, X[0])
    assert np.array_equal(y1, y3)  # deterministic: the same input gives the same bits
    # four columns go through the tensor-core GEMM, one column through the matrix-vector kernel: same integers, other f32 order
    assert rel_err(Y[0], y1.astype(np.float64)) < 2e-6


@pytest.mark.parametrize("shape", [(288, 288), (288, 768), (768, 288), (288, 32000), (64, 96)])
def test_matvec_f32(pkg, orc, synth, shape):
    n_in, n_out = shape
    A = synth.matrix(0, n_in, n_out, seed=9)
    x = synth.normal_f32(n_in, 79, 1.0)
    y = np.zeros(n_out, dtype=np.float32)
    pkg.matmul_(y, A, x)
    assert rel_err(y, orc.matmul_f64(A, x)) < 2e-6


def test_matvec_golden(pkg):
    g = np.load(os.path.join(GOLDEN, "kquants_golden.npz"))
    for name, (t, bb) in TYPES.items():
        raw = g[f"{name}_raw"]
        A = pkg.QuantMatrix(t, raw.reshape(-1), 1024, 8)
        y = np.zeros(8, dtype=np.float32)
        pkg.matmul_(y, A, g["x1024"])
        want = g[f"{name}_matvec_seq_bits"].view(np.float32)
        assert np.abs(y - want).max() < 4e-6 * np.abs(want).max()


def test_matvec_rejects_bad_arguments(L, pkg):
    x = np.zeros(300, dtype=np.float32)
    raw = np.zeros(144 * 2, dtype=np.uint8)
    y = np.zeros(2, dtype=np.float32)
    assert L.lib().l2b_matvec(12, L.ptr(raw), 300, 2, L.ptr(x), 1, L.ptr(y), 3) == L.ERR_BAD_ARG  # in % 256 != 0
    assert L.lib().l2b_matvec(8, L.ptr(raw), 256, 2, L.ptr(x), 1, L.ptr(y), 3) == L.ERR_UNSUPPORTED_TYPE  # Q8_0
    assert L.lib().l2b_matvec(12, None, 256, 2, L.ptr(x), 1, L.ptr(y), 3) == L.ERR_BAD_ARG
    assert b"" != L.lib().l2b_last_error_string()


# ---- small operators ------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [288, 4096, 8192, 14336])
def test_rmsnorm(L, orc, n):
    rng = np.random.default_rng(40)
    x, w = rng.normal(size=n).astype(np.float32), rng.normal(size=n).astype(np.float32)
    o = np.zeros(n, dtype=np.float32)
    L.check(L.lib().l2b_rmsnorm(L.ptr(o), L.ptr(x), L.ptr(w), n))
    want = orc.rmsnorm(x, w)
    assert np.abs(o - want).max() <= 4e-7 * np.abs(want).max() + 1e-7


@pytest.mark.parametrize("neox", [0, 1])
@pytest.mark.parametrize("hs,heads", [(48, 6), (96, 32), (128, 8)])
@pytest.mark.parametrize("pos", [0, 1, 255, 4095])
def test_rope_bit_exact(L, orc, neox, hs, heads, pos):
    x = np.random.default_rng(41).normal(size=hs * heads).astype(np.float32)
    for base in (10000.0, 500000.0):
        y = x.copy()
        L.check(L.lib().l2b_rope(L.ptr(y), hs, heads, pos, base, neox))
        assert np.array_equal(y.view(np.uint32), orc.rope(x, hs, heads, pos, base, neox).view(np.uint32))


@pytest.mark.parametrize("n_heads,n_kv,hs", [(6, 6, 48), (32, 8, 128), (32, 32, 96), (64, 8, 128), (12, 4, 64)])
@pytest.mark.parametrize("npos", [1, 2, 37, 512, 4096])
def test_attention(L, orc, n_heads, n_kv, hs, npos):
    rng = np.random.default_rng(42)
    q = rng.normal(size=(n_heads * hs)).astype(np.float32)
    k = rng.normal(size=(npos, n_kv, hs)).astype(np.float32)
    v = rng.normal(size=(npos, n_kv, hs)).astype(np.float32)
    out = np.zeros(n_heads * hs, dtype=np.float32)
    L.check(L.lib().l2b_attention(L.ptr(out), L.ptr(q), L.ptr(k), L.ptr(v), npos, n_heads, n_kv, hs))
    want = orc.attention(q, k, v, n_heads, n_kv, hs)
    assert np.abs(out - want).max() < 1e-5 * max(1.0, np.abs(want).max())


def test_swiglu_argmax_sampling(L, orc):
    rng = np.random.default_rng(43)
    a, b = (rng.normal(size=14336) * 4).astype(np.float32), rng.normal(size=14336).astype(np.float32)
    got = a.copy()
    L.check(L.lib().l2b_swiglu(L.ptr(got), L.ptr(b), a.size))
    want = orc.swiglu(a, b)
    assert np.abs(got - want).max() <= 2e-6 * np.abs(want).max()
    idx = C.c_int32()
    x = rng.normal(size=128256).astype(np.float32)
    x[[7, 100000, 90]] = x.max() + 1  # three equal maxima: the first index wins
    L.check(L.lib().l2b_argmax(L.ptr(x), x.size, C.byref(idx)))
    assert idx.value == orc.argmax(x) == 7
    logits = (rng.normal(size=32000) * 3).astype(np.float32)
    for temperature in (0.8, 1.0):
        _, p = orc.sample_temperature(logits, temperature, 0.5)
        cdf = np.cumsum(p.astype(np.float64))
        for u in (0.0, 0.01, 0.25, 0.5, 0.9, 0.999999):
            L.check(L.lib().l2b_sample_temperature(L.ptr(logits), logits.size, temperature, u, C.byref(idx)))
            want = orc.sample_temperature(logits, temperature, u)[0]
            # the index whose cumulative-probability interval holds u, up to rounding of the running sum
            assert idx.value == want or abs(cdf[idx.value] - cdf[want]) < 1e-6


@pytest.mark.parametrize("name", ["q4_K", "q5_K", "q6_K"])
def test_matvec_activation_blocks_of_tiny_values(pkg, orc, synth, name):
    """Blocks whose largest activation is tiny (down to denormals) beside blocks of ordinary size: the per-plane inverse
    scales of such a block overflow f32 and must not turn the result into NaN (SwiGLU outputs look like this when the
    gate saturates)."""
    t = {"q4_K": 12, "q5_K": 13, "q6_K": 14}[name]
    n_in, n_out = 1536, 64
    A = synth.matrix(t, n_in, n_out, seed=5)
    x = synth.normal_f32(n_in, 6, 1.0)
    for b, scale in enumerate([1.0, 1e-30, 4e-33, 1e-36, 1e-39, 0.0]):
        x[256 * b:256 * (b + 1)] *= np.float32(scale)
    x[256 + 7] = 0.0
    y = np.zeros(n_out, np.float32)
    pkg.matmul_(y, A, x)
    want = orc.matmul_f64(A, x)
    assert np.isfinite(y).all()
    assert np.abs(y - want).max() <= 4e-6 * np.abs(want).max()
