/*
 * l2b_synth.h -- seeded synthetic weights, activations and token ids for tests and benchmarks.
 *
 * Test support, built as its own small library (libl2b_synth.so, plain C++, no CUDA): the product library
 * libllama2_b200.so does not contain these.  The reference has no counterpart (it has no tests); the generators
 * exist so that the CUDA path, the CPU oracle and the benchmark's two arms all see the same bytes from a seed.
 * Counter-based and integer-only: identical output on every machine and compiler.  Status codes are l2b_status values
 * (0 = ok, 1 = bad argument, 2 = unsupported tensor type).
 */
#ifndef L2B_SYNTH_H
#define L2B_SYNTH_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* n f32 values ~ N(0, std^2) (Irwin-Hall of 12 16-bit uniforms), or the constant `std` when constant != 0. */
int32_t l2b_synth_f32(float* host_out, int64_t n, uint64_t seed, float std, int32_t constant);
/* n_blocks k-quant super-blocks: fp16 d, dmin = |N(0, 0.01^2)|, every other byte uniform random. */
int32_t l2b_synth_kquant(int32_t ggml_type, void* host_out, int64_t n_blocks, uint64_t seed);
/* n token ids uniform in [lo, hi). */
int32_t l2b_synth_tokens(int32_t* host_out, int64_t n, uint64_t seed, int32_t lo, int32_t hi);

#ifdef __cplusplus
}
#endif
#endif /* L2B_SYNTH_H */
