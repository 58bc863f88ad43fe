"""Tensor parallelism: the partition on the CPU (gloo, two ranks, against the oracle) and, where two GPUs are
present, a two-rank greedy run against the single-GPU run.  Ranks are child processes (tp_worker.py)."""
import json
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return str(s.getsockname()[1])


def _run_ranks(mode, world, tmp_path, timeout):
    port = _free_port()
    outs = [str(tmp_path / f"rank{r}.json") for r in range(world)]
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), mode, str(r), str(world), port, outs[r]],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    logs = []
    try:
        for p in procs:
            out, _ = p.communicate(timeout=timeout)
            logs.append(out)
    finally:
        for p in procs:  # exactly the children started here
            if p.poll() is None:
                p.kill()
    for r, p in enumerate(procs):
        assert p.returncode == 0, f"rank {r} failed:\n{logs[r][-3000:]}"
    return [json.load(open(o)) for o in outs]


def test_shard_plan_covers_everything_once(pkg):
    from llama2_jl_b200 import tp
    c = pkg.ModelConfig(dim=8192, hidden_dim=28672, n_layers=80, n_heads=64, n_kv_heads=8, vocab_size=32000, seq_len=4096,
                        rope_freq_base=10000.0, rope_is_neox=False)
    for g in (1, 2, 4, 8):
        plans = [tp.shard_plan(c, g, r) for r in range(g)]
        for key, total in (("wq_rows", 8192), ("wk_rows", 1024), ("wv_rows", 1024), ("w1_rows", 28672), ("w3_rows", 28672),
                           ("wo_block_cols", 32), ("w2_block_cols", 112)):
            edges = [p[key] for p in plans]
            assert edges[0][0] == 0 and edges[-1][1] == total
            assert all(edges[i][1] == edges[i + 1][0] for i in range(g - 1))
        assert plans[0]["n_heads"] * g == 64 and plans[0]["n_kv_heads"] * g == 8
        # query heads stay with their kv head
        hs = 128
        for r, p in enumerate(plans):
            q0, k0 = p["wq_rows"][0] // hs, p["wk_rows"][0] // hs
            assert q0 // (64 // 8) == k0
    with pytest.raises(ValueError):
        tp.shard_plan(c, 3, 0)
    with pytest.raises(ValueError):
        tp.shard_plan(pkg.ModelConfig(4096, 14336, 32, 32, 8, 128256, 512, 5e5, False), 16, 0)


def test_partition_matches_oracle_two_gloo_ranks(pkg, tmp_path):
    res = _run_ranks("cpu", 2, tmp_path, timeout=300)
    for r in res:
        assert r["handles_ok"]
        assert r["errs"]["wo"] < 1e-12 and r["errs"]["w2"] < 1e-12  # f64 sums of exact products: only reassociation
        assert r["errs"]["wq"] == 0.0 and r["errs"]["wk"] == 0.0 and r["errs"]["w1"] == 0.0


def test_library_rejects_unshardable_configs(pkg):
    # argument checks run before any device is touched
    from llama2_jl_b200 import _lib as L
    import ctypes as C
    lib = L.lib()
    def create(**kw):
        base = dict(dim=512, hidden_dim=1024, n_layers=1, n_heads=8, n_kv_heads=4, vocab_size=1024, seq_len=64,
                    rope_freq_base=10000.0, rope_is_neox=0, act_planes=0, device=-1, tp_size=2, tp_rank=0)
        base.update(kw)
        m = C.c_void_p()
        rc = lib.l2b_model_create(C.byref(L.Config(**base)), C.byref(m))
        if rc == 0:
            lib.l2b_model_destroy(m)
        return rc
    assert create(tp_size=3) == L.ERR_BAD_ARG           # kv heads not divisible
    assert create(tp_rank=2) == L.ERR_BAD_ARG           # rank out of range
    assert create(dim=256, n_heads=4, n_kv_heads=4) == L.ERR_BAD_ARG   # dim / 2 is not a multiple of 256
    assert create(tp_size=16) == L.ERR_BAD_ARG


@pytest.mark.gpu
def test_two_gpu_greedy_run_matches_single_gpu(pkg, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = _run_ranks("gpu", 2, tmp_path, timeout=600)
    r0, r1 = res
    assert r0["tokens"] == r1["tokens"], "ranks disagree"
    assert r0["tokens"] == r0["tokens_again"] and r1["tokens"] == r1["tokens_again"]
    assert r0["logits_head"] == r1["logits_head"], "replicated logits must be bit-identical across ranks"
    # against one GPU: partial sums are added in another order, so logits agree to reassociation noise
    assert r0["logit_err_over_range"] < 2e-3
    assert r0["tokens"] == r0["single_tokens"]


@pytest.mark.gpu
def test_two_gpu_run_rides_out_a_second_of_host_skew(pkg, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    r0, r1 = _run_ranks("gpu_skew", 2, tmp_path, timeout=600)
    assert r0["tokens"] == r1["tokens"] == r0["single_tokens"]
    assert r0["tokens"] == r0["tokens_again"]


@pytest.mark.gpu
def test_two_gpu_peer_timeout_is_reported_not_hung(pkg, tmp_path):
    """One rank does not make the call (between steps, nothing of its own in flight): the other's bounded wait runs out."""
    import torch
    from llama2_jl_b200 import _lib as L
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    r0, r1 = _run_ranks("gpu_timeout", 2, tmp_path, timeout=600)
    assert r0["status"] == L.ERR_TIMEOUT, r0
    assert "tensor-parallel rank" in r0["message"]
    assert r0["seconds"] < 10.0
    assert r0["after"] == 0 and r0["closed"] and r1["closed"]
