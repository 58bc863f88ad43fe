"""Generates the golden fixtures of this directory.  Run from the repository root:

    python tests/golden/make_golden.py

kquants_golden.npz  random super-blocks of each k-quant type with the oracle's dequantised bits and a
                    1024-input matvec (sequential f32 accumulation), cross-checked here against the numpy
                    dequantiser of the `gguf` package before being written.
tiny_f32_golden.npz the tiny f32 llama2.c-format model (dim 288, 6 layers, vocab 32000, seq 256) from seed:
                    16 random prompt ids, 240 greedy tokens and the logits of four positions.
reduced_8b_golden.npz the Llama-3-8B shape cut to 2 layers / 4096 vocabulary entries, k-quant weights from seed:
                    greedy stream and logits of four positions.
The reference itself (Julia) cannot be run where these were made, so the values come from the C++ oracle.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import __graft_entry__ as g  # noqa: E402

g.build()
pkg = g.load_package()
import oracle_binding as orc  # noqa: E402
from llama2_jl_b200 import synth  # noqa: E402
from test_oracle import TYPES, random_blocks  # noqa: E402


def kquants():
    from gguf import GGMLQuantizationType as Q
    from gguf import quants
    out = {}
    x = np.random.default_rng(10).normal(size=1024).astype(np.float32)
    out["x1024"] = x
    for name, (t, bb) in TYPES.items():
        raw = random_blocks(name, 32, 11)
        deq = orc.dequantize(t, raw, 32 * 256)
        ref = quants.dequantize(raw.reshape(-1), getattr(Q, name.upper())).reshape(-1).astype(np.float32)
        assert np.array_equal(deq, ref)

        class M:
            ggml_type, data, in_dim, out_dim = t, raw.reshape(-1), 1024, 8
        out[f"{name}_raw"] = raw
        out[f"{name}_dequant_bits"] = deq.view(np.uint32)
        out[f"{name}_matvec_seq_bits"] = orc.matmul(M, x, acc=orc.ACC_SEQ).view(np.uint32)
    np.savez_compressed(os.path.join(HERE, "kquants_golden.npz"), **out)


def model_case(spec, seed, n_prompt, n_positions, keep, fname):
    cfg = spec["config"]
    w = synth.model_weights(cfg, spec["types"], seed=seed, tied_output=spec["tied"])
    prompt = synth.tokens(n_prompt, seed + 1, 3, cfg.vocab_size)
    m = orc.OracleModel(cfg, w)
    toks, logits = m.sample_greedy(prompt, n_positions, want_logits=True, acc=orc.ACC_LANES)
    np.savez_compressed(os.path.join(HERE, fname), seed=seed, prompt=prompt, tokens=toks, positions=np.array(keep),
                        logits=logits[keep].astype(np.float32), seconds=m.seconds)
    print(fname, "oracle seconds", m.seconds)


if __name__ == "__main__":
    kquants()
    model_case(synth.TINY_F32, 42, 16, 256, [0, 15, 100, 255], "tiny_f32_golden.npz")
    model_case(synth.scaled(synth.LLAMA3_8B_Q4_K_S, n_layers=2, vocab_size=4096, seq_len=128), 43, 16, 96, [0, 15, 50, 95],
               "reduced_8b_golden.npz")
