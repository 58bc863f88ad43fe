"""One rank of a tensor-parallel test, run as a child process: `python tp_worker.py MODE RANK WORLD PORT OUT.json`.

MODE cpu: gloo only, no GPU -- the partition is checked against the CPU oracle (the sum over ranks of the sharded
          wo / w2 products equals the unsharded product; the handle exchange returns the handles in rank order).
MODE gpu: one GPU per rank -- a tensor-parallel greedy run is compared with the single-GPU run of the same model.
MODE gpu_skew: the same run with rank 1 entering it a second late: the waits inside the kernels must ride that out.
MODE gpu_timeout: L2B_TP_TIMEOUT_MS=50 and rank 1 does NOT make the call (it stays alive with its memory mapped, between
          steps, no kernel in flight): rank 0's wait for the peer runs out, the call returns L2B_ERR_TIMEOUT, the context
          stays usable and the session can be destroyed.  No GPU faults, traps or hangs.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def tiny_config(pkg):
    # every sharded dimension stays a multiple of 256 per rank for 2 ranks; GQA 2
    return pkg.ModelConfig(dim=512, hidden_dim=1024, n_layers=3, n_heads=8, n_kv_heads=4, vocab_size=1024, seq_len=64,
                           rope_freq_base=10000.0, rope_is_neox=False)


def main():
    mode, rank, world, port, out_path = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4], sys.argv[5]
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = port
    import datetime

    import torch
    import torch.distributed as dist

    import __graft_entry__ as g
    pkg = g.load_package()
    from llama2_jl_b200 import synth, tp

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    cfg = tiny_config(pkg)
    types = dict(synth.ALL(synth.Q4), wv=synth.Q5, w2=synth.Q5, output=synth.Q6)
    w = synth.model_weights(cfg, types, seed=11)
    res = {"rank": rank}

    if mode == "cpu":
        import oracle_binding as orc

        # handle exchange: rank-ordered
        handles = tp.exchange_handles(bytes([rank]) * 64)
        res["handles_ok"] = [h[0] for h in handles] == list(range(world))
        # partition against the oracle
        mine = tp.shard_weights(cfg, w, world, rank)
        pl = tp.shard_plan(cfg, world, rank)
        x = synth.normal_f32(cfg.dim, 5, 1.0)
        h = synth.normal_f32(cfg.hidden_dim, 6, 1.0)
        lw, ls = w.layers[1], mine.layers[1]
        errs = {}
        for name, full, shard, vec, key in (("wo", lw.wo, ls.wo, x, "wo_block_cols"), ("w2", lw.w2, ls.w2, h, "w2_block_cols")):
            lo, hi = pl[key]
            part = orc.matmul_f64(shard, vec[lo * 256:hi * 256])
            t = torch.from_numpy(part.copy())
            dist.all_reduce(t)
            want = orc.matmul_f64(full, vec)
            errs[name] = float(np.abs(t.numpy() - want).max() / max(1e-30, np.abs(want).max()))
        # row-split matrices: this rank's rows are the corresponding rows of the full product
        for name, full, shard, key in (("wq", lw.wq, ls.wq, "wq_rows"), ("wk", lw.wk, ls.wk, "wk_rows"), ("w1", lw.w1, ls.w1, "w1_rows")):
            lo, hi = pl[key]
            errs[name] = float(np.abs(orc.matmul(shard, x) - orc.matmul(full, x)[lo:hi]).max())
        res["errs"] = errs
    elif mode == "gpu_timeout":
        import ctypes as C
        from llama2_jl_b200 import _lib as L
        torch.cuda.set_device(rank)
        os.environ["L2B_TP_TIMEOUT_MS"] = "50"  # read when the token graph is captured (tp.connect)
        m = pkg.LanguageModel(cfg, None, w, device=rank, tp_size=world, tp_rank=rank)
        tp.connect(m)
        if rank == 0:
            nxt = C.c_int32(-1)
            import time
            t0 = time.perf_counter()
            res["status"] = int(L.lib().l2b_decode_next(m.device_model().session, 5, 0, 0.0, 0.0, C.byref(nxt)))
            res["seconds"] = time.perf_counter() - t0
            res["message"] = L.lib().l2b_last_error_string().decode()
            # the context is still usable: an unrelated operator runs
            x = np.arange(256, dtype=np.float32)
            y = np.zeros(256, dtype=np.float32)
            res["after"] = int(L.lib().l2b_rmsnorm(L.ptr(y), L.ptr(x), L.ptr(np.ones(256, np.float32)), 256))
        dist.barrier()  # rank 1 has made no call; nothing of rank 0 is in flight any more
        m.close()
        res["closed"] = True
    else:
        torch.cuda.set_device(rank)
        prompt = synth.tokens(8, 3, 3, cfg.vocab_size)
        n_pos = 40
        single = None
        if rank == 0:
            m1 = pkg.LanguageModel(cfg, None, w, device=0)
            toks1, _ = pkg.generate(m1, prompt, n_pos)
            st1 = pkg.RunState(m1)
            pkg.transformer_(int(prompt[0]), 0, cfg, st1)
            single = (toks1.tolist(), st1.logits.copy())
            m1.close()
        m = pkg.LanguageModel(cfg, None, w, device=rank, tp_size=world, tp_rank=rank)
        tp.connect(m)
        if mode == "gpu_skew" and rank == 1:
            import time
            time.sleep(1.0)  # host-side skew between the ranks: far beyond the kernels' short poll budget
        toks, ms = pkg.generate(m, prompt, n_pos)
        res["tokens"] = toks.tolist()
        res["ms"] = ms
        # a second run right after the first: the arrival counters keep counting across calls
        toks_b, _ = pkg.generate(m, prompt, n_pos)
        res["tokens_again"] = toks_b.tolist()
        st = pkg.RunState(m)
        pkg.transformer_(int(prompt[0]), 0, cfg, st)
        res["logits_head"] = st.logits[:8].tolist()
        if single is not None:
            res["single_tokens"] = single[0]
            rng = float(single[1].max() - single[1].min())
            res["logit_err_over_range"] = float(np.abs(st.logits - single[1]).max() / rng)
        dist.barrier()  # nobody tears its exchange memory down while a peer may still write to it
        m.close()
    with open(out_path, "w") as f:
        json.dump(res, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
