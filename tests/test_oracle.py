"""CPU checks of the oracle (the restatement of src/kquants.jl, src/matmul.jl, src/inference.jl) itself:
against the independent numpy dequantiser of the `gguf` package, against hand-computed blocks, against a
per-weight Python restatement, and against the committed golden vectors."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
TYPES = {"q4_K": (12, 144), "q5_K": (13, 176), "q6_K": (14, 210)}


def half_bits(v):
    return np.array([v], dtype=np.float16).view(np.uint8)


def py_scale_min(j, s):
    # src/kquants.jl:80-81,86-87,102-103,108-109 with 0-based indices
    if j < 4:
        return s[j] & 63, s[j + 4] & 63
    return (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4), (s[j + 4] >> 4) | ((s[j] >> 6) << 4)


def py_dequant(name, blk):
    """One block, one weight at a time, float32 arithmetic with separate roundings."""
    f = np.float32
    blk = [int(b) for b in blk]
    y = np.zeros(256, dtype=np.float32)
    if name in ("q4_K", "q5_K"):
        d = f(np.array(blk[0:2], dtype=np.uint8).view(np.float16)[0])
        dmin = f(np.array(blk[2:4], dtype=np.uint8).view(np.float16)[0])
        s = blk[4:16]
        qh = blk[16:48] if name == "q5_K" else None
        qs = blk[48:176] if name == "q5_K" else blk[16:144]
        for k in range(256):
            p, hi, l = k // 64, (k // 32) % 2, k % 32
            sc, m = py_scale_min(2 * p + hi, s)
            q = (qs[32 * p + l] >> 4) if hi else (qs[32 * p + l] & 0xF)
            if qh is not None and (qh[l] >> (2 * p + hi)) & 1:
                q += 16
            y[k] = f(f(d * f(sc)) * f(q)) - f(dmin * f(m))
    else:
        ql, qh, sc = blk[0:128], blk[128:192], blk[192:208]
        d = f(np.array(blk[208:210], dtype=np.uint8).view(np.float16)[0])
        for k in range(256):
            n, quad, l = k // 128, (k // 32) % 4, k % 32
            b = ql[64 * n + l + (32 if quad & 1 else 0)]
            nib = (b >> 4) if quad >= 2 else (b & 0xF)
            q = (nib | (((qh[32 * n + l] >> (2 * quad)) & 3) << 4)) - 32
            s8 = sc[8 * n + l // 16 + 2 * quad]
            s8 = s8 - 256 if s8 > 127 else s8
            y[k] = f(d * f(s8 * q))
    return y


def random_blocks(name, nb, seed):
    t, bb = TYPES[name]
    rng = np.random.default_rng(seed)
    raw = rng.integers(0, 256, size=(nb, bb), dtype=np.uint8)
    for off in ([208] if name == "q6_K" else [0, 2]):
        h = np.abs(rng.normal(0, 0.01, size=nb)).astype(np.float16)
        raw[:, off:off + 2] = h.view(np.uint8).reshape(nb, 2)
    return raw


@pytest.mark.parametrize("name", list(TYPES))
def test_dequant_matches_gguf_numpy(orc, name):
    """Independent cross-check: bit-identical to gguf.quants.dequantize except for the sign of zero
    (the reference multiplies d by an exact integer product, which gives +0 where gguf's (d*scale)*q gives -0)."""
    from gguf import GGMLQuantizationType as Q
    from gguf import quants
    t, bb = TYPES[name]
    raw = random_blocks(name, 300, 1)
    got = orc.dequantize(t, raw, 300 * 256)
    ref = quants.dequantize(raw.reshape(-1), getattr(Q, name.upper())).reshape(-1).astype(np.float32)
    assert np.array_equal(got, ref)  # value equality (0.0 == -0.0)
    nz = ref != 0
    assert np.array_equal(got.view(np.uint32)[nz], ref.view(np.uint32)[nz])


@pytest.mark.parametrize("name", list(TYPES))
def test_dequant_matches_per_weight_restatement(orc, name):
    t, bb = TYPES[name]
    raw = random_blocks(name, 6, 2)
    got = orc.dequantize(t, raw, 6 * 256).reshape(6, 256)
    for i in range(6):
        want = py_dequant(name, raw[i])
        assert np.array_equal(got[i].view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("name", list(TYPES))
def test_all_zero_block(orc, name):
    t, bb = TYPES[name]
    assert not orc.dequantize(t, np.zeros((1, bb), dtype=np.uint8), 256).any()


def test_q4k_hand_computed(orc):
    blk = np.zeros(144, dtype=np.uint8)
    blk[0:2] = half_bits(1.0)
    blk[2:4] = half_bits(0.5)
    blk[4 + 0] = 3      # sc of sub-block 0
    blk[4 + 4] = 2      # min of sub-block 0
    blk[16 + 0] = 0x95  # low nibble 5 -> value 0, high nibble 9 -> value 32 (sub-block 1: sc = m = 0)
    y = orc.dequantize(12, blk, 256)
    assert y[0] == np.float32(1 * 3 * 5 - 0.5 * 2)
    assert y[1] == np.float32(-1.0)  # q = 0 in sub-block 0: -dmin*m
    assert y[32] == 0.0
    # scale bytes 0xFF: every 6-bit scale and min decodes to 63, also through the high-bit paths of j >= 4
    blk[4:16] = 0xFF
    blk[16:144] = 0xFF
    blk[2:4] = half_bits(1.0)
    assert np.all(orc.dequantize(12, blk, 256) == np.float32(63 * 15 - 63))


def test_q5k_hand_computed(orc):
    blk = np.zeros(176, dtype=np.uint8)
    blk[0:2] = half_bits(2.0)
    blk[4 + 1] = 1            # sc of sub-block 1
    blk[16 + 7] = 0b10        # fifth bit of value 32+7 (sub-block 1 uses bit 1)
    blk[48 + 7] = 0x30        # high nibble 3
    y = orc.dequantize(13, blk, 256)
    assert y[32 + 7] == np.float32(2.0 * 1 * (3 + 16))
    assert y[7] == 0.0


def test_q6k_hand_computed(orc):
    blk = np.zeros(210, dtype=np.uint8)
    blk[208:210] = half_bits(0.25)
    blk[192 + 2] = np.array([-3], dtype=np.int8).view(np.uint8)[0]  # scale of values 32..47
    blk[0 + 32 + 5] = 0x07   # ql[32+5] low nibble -> q2 of l = 5
    blk[128 + 5] = 0b1100    # qh bits 2..3 = 3 -> high bits of q2
    y = orc.dequantize(14, blk, 256)
    assert y[32 + 5] == np.float32(0.25 * (-3 * ((7 | (3 << 4)) - 32)))
    assert y[0] == 0.0  # scale 0


@pytest.mark.parametrize("byte", [0x00, 0x3F, 0x40, 0xC0, 0xFF])
@pytest.mark.parametrize("name", ["q4_K", "q5_K"])
def test_scale_corner_bytes(orc, name, byte):
    """Each of the 12 packed scale bytes in turn takes a corner value; compared with the per-weight restatement."""
    t, bb = TYPES[name]
    base = random_blocks(name, 1, 3)[0]
    for i in range(12):
        blk = base.copy()
        blk[4:16] = 0x15
        blk[4 + i] = byte
        got = orc.dequantize(t, blk, 256)
        assert np.array_equal(got.view(np.uint32), py_dequant(name, blk).view(np.uint32)), (i, byte)


@pytest.mark.parametrize("name", list(TYPES))
def test_vecdot_orders_agree(orc, name):
    """The three accumulation orders differ only by f32 reassociation noise."""
    t, bb = TYPES[name]
    raw = random_blocks(name, 16 * 8, 4)
    x = np.random.default_rng(5).normal(size=4096).astype(np.float32)

    class M:
        ggml_type, data, in_dim, out_dim = t, raw.reshape(-1), 4096, 8
    y64 = orc.matmul_f64(M, x)
    w = orc.dequantize(t, raw, 8 * 4096).reshape(8, 4096).astype(np.float64)
    assert np.allclose(y64, (w * x.astype(np.float64)).sum(1), rtol=1e-6, atol=1e-6)  # products are rounded to f32 first
    for acc in (orc.ACC_SEQ, orc.ACC_LANES):
        y = orc.matmul(M, x, acc=acc)
        assert np.abs(y - y64).max() <= 2e-5 * np.abs(y64).max() + 1e-5


def test_rmsnorm_rope_softmax_against_numpy(orc):
    rng = np.random.default_rng(6)
    x = rng.normal(size=288).astype(np.float32)
    w = rng.normal(size=288).astype(np.float32)
    ss = np.float32(1.0) / np.sqrt(np.float32(np.dot(x.astype(np.float64), x.astype(np.float64))) / np.float32(288) + np.float32(1e-5))
    assert np.allclose(orc.rmsnorm(x, w), w * (ss * x), rtol=1e-6)
    # RoPE at position 0 is the identity (theta = 0); at pos 3 pair 0 rotates by 3 rad
    v = rng.normal(size=2 * 48).astype(np.float32)
    assert np.array_equal(orc.rope(v, 48, 2, 0, 10000.0, False), v)
    r = orc.rope(v, 48, 2, 3, 10000.0, False)
    c, s = np.float32(np.cos(3.0)), np.float32(np.sin(3.0))
    assert r[0] == np.float32(v[0] * c) - np.float32(v[1] * s) and r[1] == np.float32(v[0] * s) + np.float32(v[1] * c)
    rn = orc.rope(v, 48, 2, 3, 10000.0, True)
    assert rn[0] == np.float32(v[0] * c) - np.float32(v[24] * s) and rn[24] == np.float32(v[0] * s) + np.float32(v[24] * c)
    # iterated angle: theta_1 = fl(3 * fl(10000^(-1/24)))
    sc = np.float32(np.float64(10000.0) ** np.float64(np.float32(-1.0) / np.float32(24)))
    th = np.float32(3.0) * sc
    assert r[2] == np.float32(v[2] * np.float32(np.cos(np.float64(th)))) - np.float32(v[3] * np.float32(np.sin(np.float64(th))))
    p = orc.softmax(x)
    e = np.exp(x - x.max())
    assert np.allclose(p, e / e.sum(), rtol=1e-5) and abs(p.sum() - 1) < 1e-5


def test_argmax_first_index_and_sampling(orc):
    x = np.array([1, 5, 5, 2], dtype=np.float32)
    assert orc.argmax(x) == 1  # Julia argmax: first maximal element
    logits = np.log(np.array([0.1, 0.2, 0.3, 0.4], dtype=np.float32))
    for u, want in ((0.05, 0), (0.15, 1), (0.45, 2), (0.95, 3)):
        assert orc.sample_temperature(logits, 1.0, u)[0] == want


def test_attention_against_numpy(orc):
    rng = np.random.default_rng(7)
    n_heads, n_kv, hs, npos = 8, 2, 16, 9
    q = rng.normal(size=(n_heads, hs)).astype(np.float32)
    k = rng.normal(size=(npos, n_kv, hs)).astype(np.float32)
    v = rng.normal(size=(npos, n_kv, hs)).astype(np.float32)
    got = orc.attention(q.reshape(-1), k, v, n_heads, n_kv, hs).reshape(n_heads, hs)
    for h in range(n_heads):
        kvh = h // (n_heads // n_kv)
        s = (k[:, kvh, :] @ q[h]) / np.sqrt(np.float32(hs))
        p = np.exp(s - s.max())
        p /= p.sum()
        assert np.allclose(got[h], p @ v[:, kvh, :], rtol=2e-5, atol=2e-6)


def test_golden_vectors(orc):
    """The committed fixtures (tests/golden/make_golden.py) pin the oracle's outputs."""
    g = np.load(os.path.join(GOLDEN, "kquants_golden.npz"))
    for name, (t, bb) in TYPES.items():
        raw = g[f"{name}_raw"]
        assert np.array_equal(orc.dequantize(t, raw, raw.shape[0] * 256).view(np.uint32), g[f"{name}_dequant_bits"])

        class M:
            ggml_type, data, in_dim, out_dim = t, raw.reshape(-1), 1024, raw.shape[0] // 4
        assert np.array_equal(orc.matmul(M, g["x1024"], acc=orc.ACC_SEQ).view(np.uint32), g[f"{name}_matvec_seq_bits"])
