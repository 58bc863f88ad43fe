#!/usr/bin/env python
"""Benchmark of the per-token decode path.

Workload (default): the Llama-3-8B shape, Q4_K_S-style mix (q4_K, attn_v / ffn_down q5_K, output q6_K),
seeded synthetic weights, a prompt of 128 random ids fed token by token followed by 256 greedy tokens,
batch 1, seq_len 512 -- the configuration the headline metric is quoted on.  One "step" is that whole
384-position run.  `value` is positions per second with everything resident on the device (CUDA events
on the session stream around the token loop); `e2e` drives the same run one l2b_decode_next call per
position with host token ids in and out.  On N > 1 GPUs every rank runs an independent replica
(the shape fits one GPU; there is no exchange step), so `value` is the sum over ranks.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload 8b|tiny|phi3]
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
METRIC = "decode tok/s @Llama-3-8B-shape Q4_K_S, batch 1; % of HBM roofline"


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


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


def pass_schedule(n_prompt, n_positions, pairs):
    """The passes l2b_generate makes: (first position, positions in the pass).  Two positions share a pass when both are
    followed by a prompt token (their next tokens are forced, so neither needs logits)."""
    out, i = [], 0
    while i < n_positions:
        k = 2 if (pairs and i + 2 < n_prompt and i + 1 < n_positions) else 1
        out.append((i, k))
        i += k
    return out


def kv_bytes_per_run(cfg, schedule, tp=1):
    hs = cfg.dim // cfg.n_heads
    per_pos = 2 * hs * (cfg.n_kv_heads // tp) * 4 * cfg.n_layers  # f32 keys + values of one position, all layers (this GPU's heads)
    return per_pos * sum(p + k for p, k in schedule)          # a pass reads the cache once, up to its last position


# dram__bytes_read.sum + dram__bytes_write.sum of one fused_matvec_kernel launch on the 14336 x 4096 q4_K matrix, from the
# ncu capture summarised in profiles/ (33 030 144 algorithmic bytes): no re-reads.
NCU_TRAFFIC_MATVEC_Q4K_14336x4096 = 33131008


def time_matvec(ggml_type, n_in, n_out, copies, launches, steps, warmup, planes):
    """Average device time of one fused_matvec_kernel launch (CUDA events on the launching stream), weights rotated
    through `copies` copies of the matrix so that every launch streams from HBM."""
    import torch
    import __graft_entry__ as g
    g.load_package()
    from llama2_jl_b200 import _lib as L
    from llama2_jl_b200 import synth
    A = synth.matrix(ggml_type, n_in, n_out, seed=77)
    x = torch.from_numpy(synth.normal_f32(n_in, 78, 1.0)).cuda()
    y = torch.zeros(n_out, dtype=torch.float32, device="cuda")
    h = C.c_void_p()
    L.check(L.lib().l2b_matrix_create(ggml_type, L.ptr(A.data), n_in, n_out, copies, C.byref(h)))
    stream = torch.cuda.current_stream().cuda_stream

    def run(n):
        for i in range(n):
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
    ms, us, nbytes = time_matvec(t, n_in, n_out, copies, launches, args.steps, args.warmup, planes)
    peak, kind = measured_peak()
    traffic = NCU_TRAFFIC_MATVEC_Q4K_14336x4096 if (t, n_in, n_out) == (12, 4096, 14336) else None
    line = {"metric": "k-quant dequant-matvec, batch 1", "value": round(us, 3), "unit": "us per matvec", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": False, "vs_baseline": None,
            "dtype": f"int8 activation planes x k-quant integers on int8 tensor-core MMAs, f32 accumulate; {planes} int8 activation plane(s)",
            "data": "synthetic", "config": {"workload": f"{args.workload} W {n_out}x{n_in}, {copies} rotating copies, {launches} launches per step"},
            "gpu_launches": args.steps * launches,
            "roofline": {"bound": "hbm", "achieved": round(nbytes / us / 1e3, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(nbytes / us / 1e3 / peak, 4), "traffic": traffic, "peak_kind": kind, "bytes_per_launch": nbytes}}
    print(json.dumps(line), flush=True)


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
    spec, wl_name = workload_spec(synth, args.workload)
    tp_mode = args.workload == "70b-tp"  # all GPUs work on ONE token stream (strong scaling); otherwise N replicas
    if tp_mode and world < 2:
        raise SystemExit("--workload 70b-tp needs --gpus 2, 4 or 8 (one rank per GPU under torch.distributed.run)")
    if args.layers > 0:
        spec = synth.scaled(spec, n_layers=args.layers)
        wl_name += f" [reduced to {args.layers} layers]"
    cfg = spec["config"]
    n_pos = spec["n_prompt"] + spec["n_decode"]
    if args.positions > 0:  # shortened run (profiling captures); not the benchmark configuration
        n_pos = args.positions
        wl_name += f" [shortened to {n_pos} positions]"
    if tp_mode:
        from llama2_jl_b200 import tp
        # four distinct layers, reused in turn: the full host copy (38.7 GB per rank) would not fit beside the other ranks'
        weights = synth.model_weights(cfg, spec["types"], seed=2024, tied_output=spec["tied"], distinct_layers=4)
        model = pkg.LanguageModel(cfg, None, weights, act_planes=args.act_planes, device=local, tp_size=world, tp_rank=rank)
        tp.connect(model)
    else:
        weights = synth.model_weights(cfg, spec["types"], seed=2024, tied_output=spec["tied"])
        model = pkg.LanguageModel(cfg, None, weights, act_planes=args.act_planes, device=local)
    prompt = synth.prompt_tokens(spec, 2024)[:n_pos]
    wbytes = model.weight_bytes_per_token()
    kpt = model.kernels_per_token()
    pairs = model.prefill_pairs()
    schedule = pass_schedule(len(prompt), n_pos, pairs)
    n_pair_passes = sum(1 for _, k in schedule if k == 2)
    # a two-position pass streams the layers once and skips the classifier (the logits of a forced position are not used)
    out_bytes = weights.output_weight.data.size if hasattr(weights.output_weight, "data") else weights.output_weight.size * 4
    sess = model.device_model().session
    lib = L.lib()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident loop ------------------------------------------------------------------
    for _ in range(args.warmup):
        toks, _ = pkg.generate(model, prompt, n_pos)
    sampler = ClockSampler(local)
    sampler.start()
    barrier()
    dev_ms = 0.0
    for _ in range(args.steps):
        toks, ms = pkg.generate(model, prompt, n_pos)
        dev_ms += ms
    barrier()
    clocks = sampler.summary()

    # ---- end to end: one C-ABI call per position, host ids in and out ------------------------
    nxt = C.c_int32()

    def e2e_run():
        L.check(lib.l2b_session_reset(sess))
        tok = int(prompt[0])
        out = []
        for pos in range(n_pos):
            L.check(lib.l2b_decode_next(sess, tok, pos, 0.0, 0.0, C.byref(nxt)))
            tok = int(prompt[pos + 1]) if pos + 1 < len(prompt) else nxt.value
            out.append(tok)
        return out
    e2e_steps = max(1, min(args.steps, 3))
    stream = e2e_run()
    assert stream == [int(t) for t in toks], "one-step and device-loop token streams differ"
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_run()
    torch.cuda.synchronize()
    percall_s = time.perf_counter() - t0
    # end to end through the loop call (`sample`'s replacement): host prompt in, host tokens out, wall clock
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        toks2, _ = pkg.generate(model, prompt, n_pos)
    e2e_s = time.perf_counter() - t0
    assert [int(t) for t in toks2] == stream
    barrier()

    t = torch.tensor([dev_ms, e2e_s, percall_s], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_s, percall_s = float(t[0]), float(t[1]), float(t[2])
    ms_per_step = dev_ms / args.steps
    streams = 1 if tp_mode else world
    value = streams * n_pos * args.steps / (dev_ms / 1e3)
    e2e_value = streams * n_pos * e2e_steps / e2e_s
    peak, peak_kind = measured_peak()
    # per step (one run) and GPU: every pass streams the layers; one-position passes also stream the classifier
    algo_bytes = (wbytes - out_bytes) * len(schedule) + out_bytes * (len(schedule) - n_pair_passes) + kv_bytes_per_run(cfg, schedule, world if tp_mode else 1)
    achieved = algo_bytes / (ms_per_step / 1e3) / 1e9
    line = {
        "metric": METRIC if not tp_mode else "decode tok/s @Llama-2-70B-shape q4_K, batch 1, tensor parallel; % of HBM roofline",
        "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "strong" if tp_mode else "weak", "vs_baseline": None,
        "dtype": "int8 activation planes x k-quant integers on int8 tensor-core MMAs, f32 accumulate; %d int8 activation plane(s)" % (args.act_planes or 3),
        "data": "synthetic (seeded random weights and token ids)",
        "config": {"workload": wl_name, "positions_per_step": n_pos, "act_planes": args.act_planes or 3,
                   "prompt": ("fed two positions per pass (%d two-position passes + %d one-position passes per step; no logits for forced positions)"
                              % (n_pair_passes, len(schedule) - n_pair_passes)) if pairs else "fed position by position",
                   "l2": "inputs larger than L2 (%.2f GB of weights streamed per pass)" % (wbytes / 1e9),
                   "multi_gpu": ("tensor parallel over %d GPUs, partial vectors exchanged by peer stores" % world) if tp_mode
                   else ("replicas only" if world > 1 else "single GPU")},
        "e2e": {"value": round(e2e_value, 2), "unit": "tok/s", "h2d_bytes_per_step": 4 * len(prompt) + 48, "d2h_bytes_per_step": 4 * n_pos + 4,
                "note": "one l2b_generate call per step (the loop of `sample`): host prompt ids in, host token ids out, wall clock",
                "per_position_calls": {"value": round(streams * n_pos * e2e_steps / percall_s, 2), "unit": "tok/s",
                                       "note": "one l2b_decode_next call per position (48 B in, 8 B out each), wall clock"}},
        "gpu_launches": kpt * len(schedule) * args.steps,  # a two-position pass has as many launches as a one-position pass
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                     "traffic": None, "peak_kind": peak_kind, "frac_of_nominal_8000": round(achieved / 8000.0, 4),
                     "scope": "whole token (all kernels): weight + KV bytes per position (of one GPU) / device time per position",
                     "bytes_per_position": int(algo_bytes / n_pos), "passes_per_step": len(schedule)},
        "clocks": clocks,
        "us_per_token": round(ms_per_step * 1e3 / n_pos, 2),
        "kernels_per_token": kpt,
    }
    if not tp_mode:
        # the dominant kernel on its own: fused_matvec_kernel on the gate/up-sized q4_K matrix (14336 x 4096), timed live
        _, k_us, k_bytes = time_matvec(12, 4096, 14336, 8, 64, 2, 3, args.act_planes or 3)
        line["roofline"]["dominant_kernel"] = {
            "kernel": "fused_matvec_kernel", "workload": "q4_K 14336x4096, batch 1, 8 rotating copies (264 MB > L2), back-to-back launches",
            "us_per_launch": round(k_us, 3), "bytes_per_launch": k_bytes, "achieved": round(k_bytes / k_us / 1e3, 1), "unit": "GB/s",
            "frac": round(k_bytes / k_us / 1e3 / peak, 4), "traffic": NCU_TRAFFIC_MATVEC_Q4K_14336x4096,
            "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch, ncu capture summarised under profiles/"}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(pkg, synth, spec, args)
    if rank == 0:
        print(json.dumps(line), flush=True)
    model.close()
    if world > 1:
        dist.destroy_process_group()


def oracle_positions_per_s(orc, synth, spec, n_layers, n_positions, seed=2024):
    cfg = synth.scaled(spec, n_layers=n_layers)["config"]
    w = synth.model_weights(cfg, spec["types"], seed=seed, tied_output=spec["tied"])
    m = orc.OracleModel(cfg, w)
    prompt = synth.tokens(n_positions, seed, 3, cfg.vocab_size)
    m.sample_greedy(prompt, 1, acc=orc.ACC_LANES)  # touch the weights once
    m.sample_greedy(prompt, n_positions, acc=orc.ACC_LANES)
    return m.seconds / n_positions


def cpu_baseline(pkg, synth, spec, args):
    """The CPU oracle (a C++ port of the reference arithmetic) on this box's host cores, on a bounded sample:
    the same shape with 2 layers and with 1 layer, a few positions each, extrapolated linearly to all layers."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_binding as orc
    full = spec["config"].n_layers
    if full <= 8:
        s = oracle_positions_per_s(orc, synth, spec, full, 16)
        sample = f"all {full} layers, 16 positions"
    else:
        s2 = oracle_positions_per_s(orc, synth, spec, 2, 4)
        s1 = oracle_positions_per_s(orc, synth, spec, 1, 4)
        per_layer = max(s2 - s1, 1e-9)
        s = s1 + per_layer * (full - 1)
        sample = f"1- and 2-layer models of the same shape (full vocabulary), 4 positions each, extrapolated linearly to {full} layers"
    return {"value": round(1.0 / s, 3), "unit": "tok/s", "cores": orc.NTHREADS, "kind": "port", "sample": sample}


def run_reference(args):
    """The reference's CPU implementation of the path.  Julia is not installed here, so this is the C++ oracle port of it,
    with all host threads, on the benchmark's shape at full depth; one step = 2 positions."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    import __graft_entry__ as g
    pkg = g.load_package()
    from llama2_jl_b200 import synth
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_binding as orc
    spec, wl_name = workload_spec(synth, args.workload)
    cfg = spec["config"]
    w = synth.model_weights(cfg, spec["types"], seed=2024, tied_output=spec["tied"])
    m = orc.OracleModel(cfg, w)
    per_step = 2
    total = per_step * (args.steps + args.warmup)
    prompt = synth.tokens(max(total, 2), 2024, 3, cfg.vocab_size)
    m.reset()
    pos = 0
    for _ in range(args.warmup * per_step):
        m.transformer(int(prompt[pos]), pos)
        pos += 1
    t0 = time.perf_counter()
    for _ in range(args.steps * per_step):
        m.transformer(int(prompt[pos]), pos)
        pos += 1
    dt = time.perf_counter() - t0
    value = args.steps * per_step / dt
    sample = f"{per_step} positions per step at full depth ({cfg.n_layers} layers), teacher-forced ids, {orc.NTHREADS} threads"
    line = {"impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 2), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 (dequantised k-quant weights x f32 activations)", "data": "synthetic (seeded random weights and token ids)",
            "config": {"workload": wl_name, "positions_per_step": per_step,
                       "note": "Julia is absent on this box: C++ port of the reference's CPU arithmetic (oracle/), Threads.@threads-style row split"},
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
    ap.add_argument("--act-planes", type=int, default=0, help="int8 planes per activation (1..3; 0 = library default 3)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--positions", type=int, default=0, help="run only this many positions per step (for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
