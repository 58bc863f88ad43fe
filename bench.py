#!/usr/bin/env python
"""Benchmark of the per-token decode path.

Workload (default): the Llama-3-8B shape, Q4_K_S-style mix (q4_K, attn_v / ffn_down q5_K, output q6_K), seeded synthetic
weights, a prompt of 128 random ids followed by 256 greedy tokens, batch 1, seq_len 512 -- the configuration the headline
metric is quoted on.  One "step" is that whole 384-position run through l2b_generate (the loop of `sample`).

What the printed line says:
  value     decode tok/s: the 256 positions that are fed generated tokens, CUDA events on the session stream, everything
            resident on the device;
  prefill   tok/s over the 128 positions that are fed prompt tokens (two positions per pass where both are forced), same events;
  e2e       decode tok/s through one l2b_decode_next call per position (host token id in, host token id out, wall clock),
            after the prompt has gone through l2b_prefill;
  roofline  weight + KV bytes of the decode positions / their device time, against the measured copy bandwidth;
  parity    the CUDA path against the CPU oracle at FULL depth on the first positions of the same run;
  cpu_baseline  the timing of that oracle run (the reference's CPU arithmetic; Julia itself is not installed).
On N > 1 GPUs every rank runs an independent replica of the 8B shape (it fits one GPU and has no exchange step), `value` is
the sum over ranks, and the key `tp_70b` carries the Llama-2-70B shape run tensor-parallel over the same N GPUs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload 8b|tiny|phi3|70b-tp|matvec-q4k|...]
"""
import argparse
import ctypes as C
import json
import os
import re
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
METRIC = "decode tok/s @Llama-3-8B-shape Q4_K_S, batch 1; % of HBM roofline"
PARITY_PROMPT, PARITY_POSITIONS = 8, 18  # the oracle run shared by `parity` and `cpu_baseline`: 8 prompt ids, 18 positions
REF_POSITIONS_PER_STEP = 4


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def profiled_traffic(name):
    """`traffic_bytes_per_launch: N` of a tracked ncu summary under profiles/ (None when the summary does not carry it)."""
    try:
        with open(os.path.join(ROOT, "profiles", name)) as f:
            m = re.search(r"traffic_bytes_per_launch:\s*([0-9]+)", f.read())
        return int(m.group(1)) if m else None
    except OSError:
        return None


class ClockSampler(threading.Thread):
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.rows, self.stop_flag = index, [], threading.Event()

    def run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            self.stop_flag.wait(0.2)

    def summary(self):
        self.stop_flag.set()
        self.join(timeout=6)
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        sm = sorted(float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows if len(r) > 2 + i)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": float(self.rows[0][1]) if self.rows[0][1].isdigit() else None,
                "reasons": reasons, "samples": len(self.rows)}


def workload_spec(synth, name):
    if name == "8b":
        return synth.LLAMA3_8B_Q4_K_S, "llama3-8b-shape Q4_K_S, 128 prompt ids + 256 greedy tokens, batch 1, seq_len 512"
    if name == "tiny":
        return synth.TINY_F32, "llama2.c f32 dim 288 x 6 layers, 16 prompt ids + 240 greedy tokens"
    if name == "phi3":
        return synth.PHI3_MINI_Q5_K_M, "phi3-mini-shape Q5_K_M, 2048 prompt ids + 512 greedy tokens, seq_len 4096"
    if name == "70b-tp":
        return synth.LLAMA2_70B_Q4_K, "llama2-70b-shape q4_K (q6_K output), tensor parallel, 512 prompt ids + 256 greedy tokens, batch 1, seq_len 4096"
    raise SystemExit(f"unknown workload {name}")


def shared_config(wl_name, spec, world, tp_mode):
    """The `config` both arms print: the workload and nothing specific to an implementation."""
    return {"workload": wl_name, "n_prompt": spec["n_prompt"], "n_decode": spec["n_decode"], "seq_len": spec["config"].seq_len, "batch": 1,
            "l2": "inputs larger than L2 (the weights streamed per position exceed it many times)",
            "multi_gpu": ("tensor parallel over %d GPUs" % world) if tp_mode else ("replicas only" if world > 1 else "single GPU")}


def pass_schedule(n_prompt, n_positions, pairs):
    """The passes l2b_generate makes: (first position, positions in the pass).  Two positions share a pass when both are
    followed by a prompt token (their next tokens are forced, so neither needs logits)."""
    out, i = [], 0
    while i < n_positions:
        k = 2 if (pairs and i + 2 < n_prompt and i + 1 < n_positions) else 1
        out.append((i, k))
        i += k
    return out


def kv_bytes(cfg, schedule, tp=1):
    hs = cfg.dim // cfg.n_heads
    per_pos = 2 * hs * (cfg.n_kv_heads // tp) * 4 * cfg.n_layers  # f32 keys + values of one position, all layers (this GPU's heads)
    return per_pos * sum(p + k for p, k in schedule)              # a pass reads the cache once, up to its last position


def time_matvec(ggml_type, n_in, n_out, copies, launches, steps, warmup, planes, cols=1):
    """Average device time of one fused_matvec_kernel launch (CUDA events on the launching stream), weights rotated
    through `copies` copies of the matrix so that every launch streams from HBM.  cols > 1: one call of the tensor-core GEMM
    (quantise + kq_gemm_kernel) over that many activation columns instead."""
    import torch
    import __graft_entry__ as g
    g.load_package()
    from llama2_jl_b200 import _lib as L
    from llama2_jl_b200 import synth
    A = synth.matrix(ggml_type, n_in, n_out, seed=77)
    x = torch.from_numpy(synth.normal_f32(cols * n_in, 78, 1.0)).cuda()
    y = torch.zeros(cols * n_out, dtype=torch.float32, device="cuda")
    h = C.c_void_p()
    L.check(L.lib().l2b_matrix_create(ggml_type, L.ptr(A.data), n_in, n_out, copies, C.byref(h)))
    stream = torch.cuda.current_stream().cuda_stream

    def run(n):
        for i in range(n):
            if cols > 1:
                L.check(L.lib().l2b_matrix_matmul_device(h, i % copies, x.data_ptr(), cols, y.data_ptr(), stream))
            else:
                L.check(L.lib().l2b_matrix_matvec_device(h, i % copies, x.data_ptr(), y.data_ptr(), planes, stream))
    run(warmup * copies)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ms = 0.0
    for _ in range(steps):
        e0.record()
        run(launches)
        e1.record()
        torch.cuda.synchronize()
        ms += e0.elapsed_time(e1)
    L.lib().l2b_matrix_destroy(h)
    nbytes = (n_in // 256) * n_out * L.BLOCK_BYTES[ggml_type]
    return ms, ms * 1e3 / (steps * launches), nbytes


def run_matvec(args):
    """Isolated operator: W 14336 x 4096 as k-quant super-blocks, x f32[4096] quantised on the device, batch 1.
    Eight copies of W (more than the L2) are rotated through, so every launch streams its weights from HBM."""
    import torch
    torch.cuda.set_device(0)
    t = {"matvec-q4k": 12, "matvec-q5k": 13, "matvec-q6k": 14}[args.workload]
    n_in, n_out, copies = args.matvec_in, args.matvec_out, args.matvec_copies
    planes = args.act_planes or 3
    launches = args.matvec_launches
    cols = args.matvec_cols
    ms, us, nbytes = time_matvec(t, n_in, n_out, copies, launches, args.steps, args.warmup, planes, cols)
    peak, kind = measured_peak()
    traffic = profiled_traffic("fused_matvec_kernel__q4_K_14336x4096.md") if (t, n_in, n_out, cols) == (12, 4096, 14336, 1) else None
    line = {"metric": "k-quant dequant-matvec, batch %d" % cols, "value": round(us, 3), "unit": "us per matvec" if cols == 1 else "us per %d-column product" % cols,
            "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": False, "vs_baseline": None,
            "dtype": f"int8 activation planes x k-quant integers on int8 tensor-core MMAs, f32 accumulate; {planes} int8 activation plane(s)",
            "data": "synthetic", "config": {"workload": f"{args.workload} W {n_out}x{n_in}, {cols} column(s), {copies} rotating copies, {launches} launches per step"},
            "columns_per_s": round(cols / us * 1e6, 1), "tflops": round(2.0 * n_in * n_out * cols / us / 1e6, 2),
            "gpu_launches": args.steps * launches,
            "roofline": {"bound": "hbm", "achieved": round(nbytes / us / 1e3, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(nbytes / us / 1e3 / peak, 4), "traffic": traffic, "peak_kind": kind, "bytes_per_launch": nbytes}}
    print(json.dumps(line), flush=True)


def oracle_check(pkg, synth, spec, model):
    """The CPU oracle at FULL depth on the first positions of the benchmark's own run (its first PARITY_PROMPT prompt ids, then
    greedy), timed, and the CUDA path compared with it.  Returns (parity, cpu_baseline).  The only place the GPU arm runs oracle/."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_binding as orc
    cfg = spec["config"]
    prompt = synth.prompt_tokens(spec, 2024)[:PARITY_PROMPT]
    n_pos = min(PARITY_POSITIONS, cfg.seq_len)
    oracle = orc.OracleModel(cfg, model.weights)
    oracle.sample_greedy(prompt, 1)  # touch every weight once (page faults, thread start-up)
    want_tokens, want_logits = oracle.sample_greedy(prompt, n_pos, want_logits=True)
    seconds = oracle.seconds
    got, _ = pkg.generate(model, prompt, n_pos)
    fed = np.concatenate([prompt[:1], want_tokens])
    state = pkg.RunState(model)
    worst, agree, decided = 0.0, 0, 0
    for pos in range(n_pos):
        pkg.transformer_(int(fed[pos]), pos, cfg, state)
        w = want_logits[pos]
        err = float(np.abs(state.logits - w).max())
        worst = max(worst, err / float(w.max() - w.min()))
        s = np.sort(w)
        if s[-1] - s[-2] > 2 * err:  # the oracle's margin exceeds the error: the argmax is decided
            decided += 1
            agree += int(np.argmax(state.logits)) == int(np.argmax(w))
    parity = {"against": "CPU oracle at full depth, same weights and prompt", "positions": n_pos,
              "max_logit_err_over_range": float("%.3g" % worst), "tolerance": 2e-3, "argmax_agree": f"{agree}/{decided}",
              "greedy_identical": bool(np.array_equal(got, want_tokens)),
              "ok": bool(worst < 2e-3 and agree == decided and np.array_equal(got, want_tokens))}
    baseline = {"value": round(n_pos / seconds, 3), "unit": "tok/s", "cores": orc.NTHREADS, "kind": "port",
                "sample": f"the first {n_pos} positions of the run at full depth ({cfg.n_layers} layers, full vocabulary), {orc.NTHREADS} threads"}
    return parity, baseline


def decode_roofline(cfg, wbytes, n_prompt, n_pos, decode_ms, peak, tp=1):
    sched = [(p, 1) for p in range(n_prompt, n_pos)]
    algo = wbytes * len(sched) + kv_bytes(cfg, sched, tp)
    achieved = algo / (decode_ms / 1e3) / 1e9
    return algo, achieved, achieved / peak


def run_tp_70b(args, pkg, synth, L, torch, dist, world, rank, local, steps, positions=0, layers=0, check_single=True):
    """The Llama-2-70B shape tensor-parallel over all `world` GPUs (one token stream, strong scaling); world == 1: the same
    shape on one GPU, the base of the strong-scaling curve.  Returns the result dict and the token stream."""
    from llama2_jl_b200 import tp
    spec, wl_name = workload_spec(synth, "70b-tp")
    if layers > 0:
        spec = synth.scaled(spec, n_layers=layers)
    cfg = spec["config"]
    n_prompt = spec["n_prompt"]
    n_pos = positions if positions > 0 else n_prompt + spec["n_decode"]
    # four distinct layers, reused in turn: the full host copy (38.7 GB per rank) would not fit beside the other ranks'
    weights = synth.model_weights(cfg, spec["types"], seed=2024, tied_output=spec["tied"], distinct_layers=4)
    model = pkg.LanguageModel(cfg, None, weights, act_planes=args.act_planes, device=local, tp_size=world, tp_rank=rank)
    if world > 1:
        tp.connect(model)
    prompt = synth.prompt_tokens(spec, 2024)[:min(n_prompt, n_pos)]
    wbytes = model.weight_bytes_per_token()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    toks, _ = pkg.generate(model, prompt, n_pos)  # warm-up
    barrier()
    pm = dm = 0.0
    for _ in range(steps):
        toks, _ = pkg.generate(model, prompt, n_pos)
        a, b = model.last_phase_ms()
        pm, dm = pm + a, dm + b
    barrier()
    same = True
    if world > 1:
        t = torch.tensor([pm, dm], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        pm, dm = float(t[0]), float(t[1])
        # every rank must have produced the same stream
        mine = torch.tensor(np.asarray(toks, dtype=np.int64), device="cuda")
        ref = mine.clone()
        dist.broadcast(ref, 0)
        eq = torch.tensor([int(torch.equal(mine, ref))], device="cuda")
        dist.all_reduce(eq, op=dist.ReduceOp.MIN)
        same = bool(int(eq[0]))
    peak, kind = measured_peak()
    n_dec = max(n_pos - len(prompt), 0)
    out = {"workload": wl_name + (f" [reduced to {layers} layers]" if layers else "") + (f" [shortened to {n_pos} positions]" if positions else ""),
           "n_gpus": world, "scaling": "strong", "steps": steps, "bytes_per_token_per_gpu": int(wbytes)}
    if world > 1:
        out["tokens_equal_across_ranks"] = same
    if n_dec > 0 and dm > 0:
        _, ach, frac = decode_roofline(cfg, wbytes, len(prompt), n_pos, dm / steps, peak, tp=world)
        out.update({"decode_tok_s": round(n_dec * steps / (dm / 1e3), 2), "ms_per_decode_token": round(dm / steps / n_dec, 4),
                    "roofline_per_gpu": {"achieved": round(ach, 1), "peak": peak, "unit": "GB/s", "frac": round(frac, 4), "peak_kind": kind}})
    if pm > 0:
        out["prefill_tok_s"] = round(len(prompt) * steps / (pm / 1e3), 2)
    model.close()
    del model, weights
    if world > 1 and check_single:
        # the same ranks on a 2-layer model of the shape: the tensor-parallel stream against the one-GPU stream of rank 0
        rspec = synth.scaled(spec, n_layers=2)
        rcfg = rspec["config"]
        rw = synth.model_weights(rcfg, rspec["types"], seed=2024, tied_output=rspec["tied"])
        rprompt = synth.prompt_tokens(rspec, 2024)[:16]
        tpm = pkg.LanguageModel(rcfg, None, rw, act_planes=args.act_planes, device=local, tp_size=world, tp_rank=rank)
        tp.connect(tpm)
        tp_toks, _ = pkg.generate(tpm, rprompt, 48)
        barrier()
        tpm.close()
        eq1 = 1
        if rank == 0:
            one = pkg.LanguageModel(rcfg, None, rw, act_planes=args.act_planes, device=local)
            one_toks, _ = pkg.generate(one, rprompt, 48)
            one.close()
            eq1 = int([int(x) for x in one_toks] == [int(x) for x in tp_toks])
        e = torch.tensor([eq1], device="cuda")
        dist.broadcast(e, 0)
        out["tokens_equal_single_gpu"] = {"value": bool(int(e[0])), "how": "2-layer model of the shape, 16 prompt ids + 32 greedy tokens: the %d-rank stream against rank 0 alone" % world}
    return out, [int(x) for x in toks]


def run_ours(args):
    if args.workload.startswith("matvec"):
        return run_matvec(args)
    import torch
    import torch.distributed as dist
    import __graft_entry__ as g
    pkg = g.load_package()
    from llama2_jl_b200 import _lib as L
    from llama2_jl_b200 import synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if args.workload == "70b-tp":  # the tensor-parallel run on its own line
        if world < 2:
            raise SystemExit("--workload 70b-tp needs --gpus 2, 4 or 8 (one rank per GPU under torch.distributed.run)")
        res, _ = run_tp_70b(args, pkg, synth, L, torch, dist, world, rank, local, args.steps, args.positions, args.layers)
        if rank == 0:
            spec, wl_name = workload_spec(synth, "70b-tp")
            line = {"metric": "decode tok/s @Llama-2-70B-shape q4_K, batch 1, tensor parallel; % of HBM roofline", "value": res.get("decode_tok_s"),
                    "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": 1, "higher_is_better": True, "scaling": "strong",
                    "vs_baseline": None, "data": "synthetic (seeded random weights and token ids)",
                    "config": shared_config(wl_name, spec, world, True), "tp_70b": res}
            print(json.dumps(line), flush=True)
        dist.destroy_process_group()
        return
    spec, wl_name = workload_spec(synth, args.workload)
    if args.layers > 0:
        spec = synth.scaled(spec, n_layers=args.layers)
        wl_name += f" [reduced to {args.layers} layers]"
    cfg = spec["config"]
    n_prompt = spec["n_prompt"]
    n_pos = n_prompt + spec["n_decode"]
    if args.positions > 0:  # shortened run (profiling captures); not the benchmark configuration
        n_pos = args.positions
        wl_name += f" [shortened to {n_pos} positions]"
    weights = synth.model_weights(cfg, spec["types"], seed=2024, tied_output=spec["tied"])
    model = pkg.LanguageModel(cfg, None, weights, act_planes=args.act_planes, device=local)
    prompt = synth.prompt_tokens(spec, 2024)[:n_pos]
    if args.prompt_len > 0:
        prompt = prompt[:args.prompt_len]
        wl_name += f" [prompt shortened to {len(prompt)} ids]"
    n_prompt = len(prompt)
    n_decode = n_pos - n_prompt
    wbytes = model.weight_bytes_per_token()
    kpt = model.kernels_per_token()
    pairs = model.prefill_pairs()
    sess = model.device_model().session
    lib = L.lib()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident loop (l2b_generate): prompt and decode phases timed by CUDA events inside the library --------------
    for _ in range(args.warmup):
        toks, _ = pkg.generate(model, prompt, n_pos)
    sampler = ClockSampler(local)
    sampler.start()
    barrier()
    prompt_ms = decode_ms = 0.0
    for _ in range(args.steps):
        toks, _ = pkg.generate(model, prompt, n_pos)
        a, b = model.last_phase_ms()
        prompt_ms, decode_ms = prompt_ms + a, decode_ms + b
    barrier()
    clocks = sampler.summary()

    # ---- end to end: the prompt through l2b_prefill, then one l2b_decode_next call per position ----------------------------
    nxt = C.c_int32()

    def e2e_run(timed):
        L.check(lib.l2b_session_reset(sess))
        first = C.c_int32()
        L.check(lib.l2b_prefill(sess, L.ptr(prompt), n_prompt, 0, C.byref(first)))
        out = [int(t) for t in prompt[1:]] + [first.value]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        tok = first.value
        for pos in range(n_prompt, n_pos):
            L.check(lib.l2b_decode_next(sess, tok, pos, 0.0, 0.0, C.byref(nxt)))  # 48 bytes in, 8 bytes out, a wait per token
            tok = nxt.value
            out.append(tok)
        return out, time.perf_counter() - t0
    e2e_steps = max(1, min(args.steps, 3))
    stream, _ = e2e_run(False)
    assert stream == [int(t) for t in toks], "one-step and device-loop token streams differ"
    barrier()
    percall_s = 0.0
    for _ in range(e2e_steps):
        percall_s += e2e_run(True)[1]
    # the whole loop as one call (`sample`'s replacement): host prompt in, host tokens out, wall clock, all positions
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        toks2, _ = pkg.generate(model, prompt, n_pos)
    loop_s = time.perf_counter() - t0
    assert [int(t) for t in toks2] == stream
    barrier()

    t = torch.tensor([prompt_ms, decode_ms, percall_s, loop_s], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    prompt_ms, decode_ms, percall_s, loop_s = (float(v) for v in t)
    streams = world
    peak, peak_kind = measured_peak()
    value = streams * n_decode * args.steps / (decode_ms / 1e3) if n_decode else 0.0
    algo, achieved, frac = decode_roofline(cfg, wbytes, n_prompt, n_pos, decode_ms / args.steps, peak) if n_decode else (0, 0.0, 0.0)
    launches_per_step = model.last_launches()  # of the l2b_generate call above, counted by the library as it enqueues
    forced = max(min(n_prompt - 1, n_pos), 0)  # prompt positions that are followed by a prompt token (no logits needed)
    gemm_min = model.prefill_gemm_min_tokens()
    if gemm_min and forced >= gemm_min:
        prefill_how = ("%d forced positions through the tensor-core GEMM pass (tcgen05 + TMA, 20 tokens per pass over a weight tile, "
                       "no logits for forced positions), the last prompt position through the decode kernels" % forced)
    elif pairs:
        prefill_how = "two positions per pass of the decode kernels where both are followed by a prompt token (no logits for forced positions)"
    else:
        prefill_how = "position by position"
    line = {
        "metric": METRIC if args.workload == "8b" else "decode tok/s @%s, batch 1; %% of HBM roofline" % wl_name.split(",")[0],
        "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round((prompt_ms + decode_ms) / args.steps, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 activation planes x k-quant integers on int8 tensor-core MMAs, f32 accumulate; %d int8 activation plane(s)" % (args.act_planes or 3),
        "data": "synthetic (seeded random weights and token ids)",
        "config": shared_config(wl_name, spec, world, False),
        "value_scope": "the %d decode positions (fed generated tokens) only; prompt positions are reported under `prefill`" % n_decode,
        "prefill": {"value": round(streams * n_prompt * args.steps / (prompt_ms / 1e3), 2), "unit": "tok/s", "positions": n_prompt,
                    "ms": round(prompt_ms / args.steps, 3), "how": prefill_how},
        "blended": {"value": round(streams * n_pos * args.steps / ((prompt_ms + decode_ms) / 1e3), 2), "unit": "positions/s",
                    "note": "all positions / device time: what `sample` prints (src/inference.jl:391-392)"},
        "e2e": {"value": round(streams * n_decode * e2e_steps / percall_s, 2) if n_decode else 0.0, "unit": "tok/s",
                "h2d_bytes_per_step": 48, "d2h_bytes_per_step": 8,
                "note": "decode positions through one l2b_decode_next call each (host token id in, host token id out, a wait per token), wall clock; "
                        "a step here is one position",
                "loop_call": {"value": round(streams * n_pos * e2e_steps / loop_s, 2), "unit": "positions/s", "h2d_bytes": 4 * n_prompt + 48,
                              "d2h_bytes": 4 * n_pos + 4, "note": "one l2b_generate call for all positions (host prompt in, host tokens out), wall clock"}},
        "gpu_launches": launches_per_step * args.steps,  # kernels of this library enqueued by the timed l2b_generate calls
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(frac, 4),
                     "traffic": None, "peak_kind": peak_kind, "frac_of_nominal_8000": round(achieved / 8000.0, 4),
                     "scope": "decode positions: weight + KV bytes per position / device time per position (every kernel of the token)",
                     "bytes_per_position": int(algo / max(n_decode, 1))},
        "clocks": clocks,
        "us_per_decode_token": round(decode_ms * 1e3 / args.steps / max(n_decode, 1), 2),
        "kernels_per_token": kpt,
    }
    if kpt == 1 and n_decode:
        # one token is one launch of token_kernel: the dominant kernel IS the token
        us = decode_ms * 1e3 / args.steps / n_decode
        per_launch = algo / n_decode
        tr = profiled_traffic("token_kernel__llama3-8b_Q4_K_S.md")
        line["roofline"]["traffic"] = tr
        line["roofline"]["dominant_kernel"] = {
            "kernel": "token_kernel", "workload": "one decode position of this run (one launch = one token)", "us_per_launch": round(us, 2),
            "bytes_per_launch": int(per_launch), "achieved": round(per_launch / us / 1e3, 1), "unit": "GB/s",
            "frac": round(per_launch / us / 1e3 / peak, 4), "traffic": tr,
            "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu summary under profiles/ (null when absent)"}
    if args.workload == "8b" and world == 1:
        # the isolated operator of the chain: fused_matvec_kernel on the gate/up-sized q4_K matrix (14336 x 4096), timed live
        _, k_us, k_bytes = time_matvec(12, 4096, 14336, 8, 64, 2, 3, args.act_planes or 3)
        line["roofline"]["isolated_matvec"] = {
            "kernel": "fused_matvec_kernel", "workload": "q4_K 14336x4096, batch 1, 8 rotating copies (264 MB > L2), back-to-back launches",
            "us_per_launch": round(k_us, 3), "bytes_per_launch": k_bytes, "achieved": round(k_bytes / k_us / 1e3, 1), "unit": "GB/s",
            "frac": round(k_bytes / k_us / 1e3 / peak, 4), "traffic": profiled_traffic("fused_matvec_kernel__q4_K_14336x4096.md")}
        line["roofline"]["dominant_kernel"] = line["roofline"]["isolated_matvec"]  # (the same measurement under its earlier name)
        line["roofline"]["traffic"] = line["roofline"]["isolated_matvec"]["traffic"]
        line["roofline"]["traffic_scope"] = "one launch of the dominant kernel (isolated_matvec), from its ncu summary under profiles/"
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["parity"], line["cpu_baseline"] = oracle_check(pkg, synth, spec, model)
    model.close()
    del model, weights
    if world == 1 and args.workload == "8b" and not args.no_tp and not args.positions and not args.layers:
        # the base of the tensor-parallel curve: the 70B shape on this one GPU (38.7 GB of weights)
        try:
            base, _ = run_tp_70b(args, pkg, synth, L, torch, dist, 1, 0, local, steps=1, positions=args.tp_positions)
            line["tp_70b_one_gpu"] = base
        except Exception as e:
            line["tp_70b_one_gpu"] = {"error": str(e)[:300]}
    if world > 1 and args.workload == "8b" and not args.no_tp:
        # the 70B shape over the same GPUs, tensor parallel: shortened so that the whole run stays within minutes
        try:
            full, toks_full = run_tp_70b(args, pkg, synth, L, torch, dist, world, rank, local, steps=1, positions=args.tp_positions)
            line["tp_70b"] = full
        except Exception as e:  # keep the replica line even if the tensor-parallel leg fails
            line["tp_70b"] = {"error": str(e)[:300]}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_reference(args):
    """The reference's CPU implementation of the path on this box's host cores.  Julia is not installed here, so this is the
    C++ oracle port of it, with all host threads, on the benchmark's shape at full depth and on the benchmark's own prompt;
    one step = the next REF_POSITIONS_PER_STEP positions of that run (teacher-forced while inside the prompt)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    import __graft_entry__ as g
    g.load_package()
    from llama2_jl_b200 import synth
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_binding as orc
    spec, wl_name = workload_spec(synth, args.workload if args.workload in ("8b", "tiny", "phi3") else "8b")
    cfg = spec["config"]
    w = synth.model_weights(cfg, spec["types"], seed=2024, tied_output=spec["tied"])
    m = orc.OracleModel(cfg, w)
    per_step = REF_POSITIONS_PER_STEP
    prompt = synth.prompt_tokens(spec, 2024)
    m.reset()
    pos, tok = 0, int(prompt[0])

    def step_positions(n):
        nonlocal pos, tok
        for _ in range(n):
            logits = m.transformer(tok, pos)
            pos += 1
            tok = int(prompt[pos]) if pos < len(prompt) else int(np.argmax(logits))
    step_positions(args.warmup * per_step)
    t0 = time.perf_counter()
    step_positions(args.steps * per_step)
    dt = time.perf_counter() - t0
    value = args.steps * per_step / dt
    sample = (f"{per_step} positions per step of the same run at full depth ({cfg.n_layers} layers, full vocabulary), positions "
              f"{args.warmup * per_step}..{(args.warmup + args.steps) * per_step - 1}, {orc.NTHREADS} threads")
    line = {"impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 2), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 (dequantised k-quant weights x f32 activations)", "data": "synthetic (seeded random weights and token ids)",
            "config": shared_config(wl_name, spec, world, False),
            "note": "Julia is absent on this box: C++ port of the reference's CPU arithmetic (oracle/), Threads.@threads-style row split",
            "cpu_baseline": {"value": round(value, 3), "unit": "tok/s", "cores": orc.NTHREADS, "kind": "port", "sample": sample},
            "e2e": {"value": round(value, 3), "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="8b", choices=["8b", "tiny", "phi3", "70b-tp", "matvec-q4k", "matvec-q5k", "matvec-q6k"])
    ap.add_argument("--layers", type=int, default=0, help="run the workload's shape with this many layers (0 = all)")
    ap.add_argument("--matvec-in", type=int, default=4096)
    ap.add_argument("--matvec-out", type=int, default=14336)
    ap.add_argument("--matvec-copies", type=int, default=8)
    ap.add_argument("--matvec-launches", type=int, default=64)
    ap.add_argument("--matvec-cols", type=int, default=1, help="activation columns per product (more than 1: the tensor-core GEMM)")
    ap.add_argument("--prompt-len", type=int, default=0, help="use only this many prompt ids (0 = the workload's prompt; for profiler captures)")
    ap.add_argument("--act-planes", type=int, default=0, help="int8 planes per activation (1..3; 0 = library default 3)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the oracle run (parity and cpu_baseline keys)")
    ap.add_argument("--no-tp", action="store_true", help="skip the 70B-shape leg (one GPU: the base figure; several: the tensor-parallel run)")
    ap.add_argument("--tp-positions", type=int, default=576, help="positions of the tensor-parallel 70B leg (512 prompt ids, then decode)")
    ap.add_argument("--positions", type=int, default=0, help="run only this many positions per step (for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
