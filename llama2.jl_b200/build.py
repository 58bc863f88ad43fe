"""In-tree build of the CUDA library for sm_100a (cross-compiles without a GPU)."""
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["csrc/api.cu", "csrc/gguf_reader.cpp", "csrc/tokenizer.cpp"]
HEADERS = ["csrc/common.cuh", "csrc/kquants.cuh", "csrc/fused_matvec.cuh", "csrc/attention.cuh", "csrc/sampling.cuh",
           "csrc/small_ops.cuh", "csrc/token_kernel.cuh", "csrc/kq_gemm.cuh", "csrc/prefill_ops.cuh", "csrc/gguf_reader.h", "../include/llama2_b200.h"]
OUTPUT = os.path.join(_HERE, "libllama2_b200.so")
SYNTH_OUTPUT = os.path.join(_HERE, "libl2b_synth.so")  # test support: seeded synthetic data, plain C++
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-shared"]


def needs_build():
    if not os.path.exists(OUTPUT):
        return True
    t = os.path.getmtime(OUTPUT)
    return any(os.path.getmtime(os.path.join(_HERE, f)) > t for f in SOURCES + HEADERS)


def build_synth(force=False):
    src = os.path.join(_HERE, "csrc/synth.cpp")
    if force or not os.path.exists(SYNTH_OUTPUT) or os.path.getmtime(src) > os.path.getmtime(SYNTH_OUTPUT):
        subprocess.run([os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-o", SYNTH_OUTPUT, src], check=True)
    return SYNTH_OUTPUT


def build_measure():
    """A second library with the measurement aids compiled in (-DL2B_MEASURE): time stamps inside the kernels, switches that
    skip parts of them.  Not the product: load it with L2B_LIBRARY=<path> for your own measurements."""
    out = os.path.join(_HERE, "libllama2_b200_measure.so")
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    subprocess.run([nvcc] + NVCC_FLAGS + ["-DL2B_MEASURE", "-o", out] + [os.path.join(_HERE, s) for s in SOURCES], check=True)
    return out


def build(force=False, verbose=False):
    build_synth(force)
    if not force and not needs_build():
        return OUTPUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", OUTPUT] + [os.path.join(_HERE, s) for s in SOURCES]
    subprocess.run(cmd, check=True)
    return OUTPUT


if __name__ == "__main__":
    print(build(force=True, verbose=True))
