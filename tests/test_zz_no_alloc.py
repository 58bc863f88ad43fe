"""The attention entry point that allocates nothing (scratch in a fixed device array inside the library).

Collected last on purpose (file name): the entry point must give the same answer whether it is the first thing a
process runs on the GPU or follows every other test, and on two calls in a row, because its scratch array keeps the
previous call's contents.  Everything goes through the C ABI; torch only provides the device buffers.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L(pkg):
    from llama2_jl_b200 import _lib

    _lib.lib()
    return _lib


def _dev(t):
    return ctypes.c_void_p(t.data_ptr())


def _case(seed, n_heads, n_kv, hs, npos, seq_len):
    rng = np.random.default_rng(seed)
    q = rng.normal(size=(n_heads * hs)).astype(np.float32)
    k = rng.normal(size=(npos, n_kv, hs)).astype(np.float32)
    v = rng.normal(size=(npos, n_kv, hs)).astype(np.float32)
    # cache layout of the library: [kv head][seq_len][hs]; positions beyond npos hold junk that must not be read
    kc = np.full((n_kv, seq_len, hs), np.nan, dtype=np.float32)
    vc = np.full((n_kv, seq_len, hs), np.nan, dtype=np.float32)
    kc[:, :npos] = k.transpose(1, 0, 2)
    vc[:, :npos] = v.transpose(1, 0, 2)
    return q, k, v, kc, vc


def _existing(L, q, k, v, n_heads, n_kv, hs, npos):
    out = np.zeros(n_heads * hs, dtype=np.float32)
    L.check(L.lib().l2b_attention(L.ptr(out), L.ptr(q), L.ptr(k), L.ptr(v), npos, n_heads, n_kv, hs))
    return out


def _noalloc(L, torch, q, kc, vc, n_heads, n_kv, hs, npos, seq_len):
    dq, dk, dv = (torch.from_numpy(a).cuda() for a in (q, kc, vc))
    dout = torch.full((n_heads * hs,), float("nan"), device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    L.check(L.lib().l2b_attention_device_noalloc(_dev(dout), _dev(dq), _dev(dk), _dev(dv), npos, seq_len, n_heads, n_kv, hs, stream))
    torch.cuda.synchronize()
    return dout.cpu().numpy()


@pytest.mark.parametrize("n_heads,n_kv,hs,npos,seq_len", [(32, 8, 128, 300, 512), (6, 6, 48, 5, 16), (64, 8, 128, 512, 512), (12, 4, 64, 37, 64)])
def test_noalloc_matches_existing_entry_point_twice(L, orc, n_heads, n_kv, hs, npos, seq_len):
    import torch

    # two calls in a row with DIFFERENT inputs: the second must not see anything the first left in the scratch array
    for seed in (7, 8):
        q, k, v, kc, vc = _case(seed, n_heads, n_kv, hs, npos, seq_len)
        want = _existing(L, q, k, v, n_heads, n_kv, hs, npos)
        got = _noalloc(L, torch, q, kc, vc, n_heads, n_kv, hs, npos, seq_len)
        assert np.isfinite(got).all()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        # and against the CPU oracle (attention_weights!, softmax!, combine_values!), to the tolerance of the attention tests
        ref = orc.attention(q, k, v, n_heads, n_kv, hs)
        assert np.abs(got - ref).max() <= 2e-5 * max(1.0, float(np.abs(ref).max()))


def test_noalloc_leaves_device_memory_untouched(L):
    """After the first call on the device (which resolves the scratch array's address), a call must not change the amount
    of free device memory: it allocates nothing and frees nothing."""
    import torch

    n_heads, n_kv, hs, npos, seq_len = 32, 8, 128, 200, 256
    q, k, v, kc, vc = _case(3, n_heads, n_kv, hs, npos, seq_len)
    dq, dk, dv = (torch.from_numpy(a).cuda() for a in (q, kc, vc))
    dout = torch.zeros(n_heads * hs, device="cuda", dtype=torch.float32)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    call = lambda: L.check(L.lib().l2b_attention_device_noalloc(_dev(dout), _dev(dq), _dev(dk), _dev(dv), npos, seq_len, n_heads, n_kv, hs, stream))
    call()  # first call on this device in this process, or not: either way set-up is done after it
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free0 == free1


def test_noalloc_after_a_smaller_and_a_larger_shape(L):
    import torch

    # the shape changes between calls, so partial results of another geometry are lying in the array
    for (n_heads, n_kv, hs, npos, seq_len) in [(128, 16, 128, 256, 256), (8, 2, 64, 9, 32), (128, 16, 128, 256, 256)]:
        q, k, v, kc, vc = _case(n_heads + npos, n_heads, n_kv, hs, npos, seq_len)
        want = _existing(L, q, k, v, n_heads, n_kv, hs, npos)
        got = _noalloc(L, torch, q, kc, vc, n_heads, n_kv, hs, npos, seq_len)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_noalloc_rejects_what_does_not_fit(L):
    import torch

    buf = torch.zeros(1024, device="cuda", dtype=torch.float32)
    p = _dev(buf)
    lib = L.lib()
    bad = [
        (1, 1, 256, 16, 128),   # more than 128 heads
        (1, 1, 8, 8, 136),      # head size beyond 128
        (4, 2, 8, 8, 64),       # n_pos beyond seq_len
        (1, 1, 8, 3, 64),       # heads not a multiple of kv heads
        (0, 1, 8, 8, 64),       # no positions
    ]
    for (npos, seq_len, n_heads, n_kv, hs) in bad:
        rc = lib.l2b_attention_device_noalloc(p, p, p, p, npos, seq_len, n_heads, n_kv, hs, None)
        assert rc == 1, (npos, seq_len, n_heads, n_kv, hs)  # L2B_ERR_BAD_ARG
        assert lib.l2b_last_error_string()
    assert lib.l2b_attention_device_noalloc(None, p, p, p, 1, 1, 8, 8, 64, None) == 1
