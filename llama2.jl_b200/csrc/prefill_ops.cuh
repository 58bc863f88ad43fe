// Element-wise kernels of the many-token prompt pass (the tensor-core GEMM of kq_gemm.cuh does the matrix products):
// embedding rows, RoPE + KV-cache write, SwiGLU, bookkeeping of the loop state.  Each restates, for T tokens at once, what
// the fused epilogues of the decode path do for one (src/inference.jl:236, 251-260, 295-299, 354-356).
#pragma once
#include "fused_matvec.cuh"

namespace l2b {

// x[t] = dequantize!(token_embedding_table[:, tokens[t]]) for t < n_tok (src/inference.jl:236); grid (blocks per row, n_tok).
__global__ void embed_rows_kernel(int type, const uint8_t* __restrict__ table, const __half* __restrict__ d6, const int* __restrict__ tokens, int n, int vocab,
                                  float* __restrict__ x) {
    const int tok = __ldg(tokens + blockIdx.y);
    const bool valid = tok >= 0 && tok < vocab;
    const int nb = n / QK_K;
    float* row = x + (size_t)blockIdx.y * n;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float v = 0.f;
        if (valid) {
            const int b = i >> 8, k = i & 255;
            const uint8_t* blk = table + ((size_t)tok * nb + b) * dev_block_bytes(type);
            if (type == T_Q4_K) v = dequant_q45<false>(blk, k);
            else if (type == T_Q5_K) v = dequant_q45<true>(blk, k);
            else v = dequant_q6(blk, __half2float(d6[(size_t)tok * nb + b]), k);
        }
        row[i] = v;
    }
}

// rope!(q), rope!(k) at positions pos0 + t and the cache writes key_cache[:, :, pos] = k, value_cache[pos, :, :] = v
// (src/inference.jl:251-260) for T tokens.  q [T][q_dim] is rotated in place; k, v [T][kv_dim] go to the caches
// [kv_head][seq_len][hs].  The rotation multiplies exactly as the decode epilogue does (separately rounded products).
struct RopeKvParams {
    float* q;
    const float* k;
    const float* v;
    float* kc;
    float* vc;
    const float* rope_cs;  // [seq_len][hs/2] (cos, sin)
    int n_tok, q_dim, kv_dim, hs, seq_len, pos0, neox;
    const int* pos_list;   // batched decode: token t is at position pos_list[t] of its own sequence ...
    size_t cache_stride;   // ... whose caches start cache_stride * t elements after kc / vc (null / 0: one sequence, pos0 + t)
};
__global__ void rope_kv_kernel(const __grid_constant__ RopeKvParams p) {
    const int t = blockIdx.y, pos = p.pos_list ? __ldg(p.pos_list + t) : p.pos0 + t;
    float* const kc = p.kc + (p.pos_list ? (size_t)t * p.cache_stride : 0);
    float* const vc = p.vc + (p.pos_list ? (size_t)t * p.cache_stride : 0);
    const int h2 = p.hs >> 1;
    const int qp = p.q_dim >> 1, kp = p.kv_dim >> 1;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < qp + kp + p.kv_dim; i += gridDim.x * blockDim.x) {
        if (i < qp + kp) {
            const bool is_q = i < qp;
            const int pr = is_q ? i : i - qp;
            const int head = pr / h2, f = pr - head * h2;
            const int ia = head * p.hs + (p.neox ? f : 2 * f), ib = p.neox ? ia + h2 : ia + 1;
            const float2 cs = __ldg(reinterpret_cast<const float2*>(p.rope_cs) + (size_t)pos * h2 + f);
            const float* src = is_q ? p.q + (size_t)t * p.q_dim : p.k + (size_t)t * p.kv_dim;
            const float vA = src[ia], vB = src[ib];
            const float oa = __fsub_rn(__fmul_rn(vA, cs.x), __fmul_rn(vB, cs.y));
            const float ob = __fadd_rn(__fmul_rn(vA, cs.y), __fmul_rn(vB, cs.x));
            if (is_q) {
                p.q[(size_t)t * p.q_dim + ia] = oa;
                p.q[(size_t)t * p.q_dim + ib] = ob;
            } else {
                float* dst = kc + ((size_t)head * p.seq_len + pos) * p.hs;
                dst[ia - head * p.hs] = oa;
                dst[ib - head * p.hs] = ob;
            }
        } else {
            const int e = i - qp - kp;
            const int head = e / p.hs;
            vc[((size_t)head * p.seq_len + pos) * p.hs + (e - head * p.hs)] = p.v[(size_t)t * p.kv_dim + e];
        }
    }
}

// hb = silu(hb) .* hb2 (src/inference.jl:295-299) over T x hidden values, in place in g.
__global__ void swiglu_rows_kernel(float* __restrict__ g, const float* __restrict__ u, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = g[i];
        g[i] = (v * (1.0f / (1.0f + expf(-v)))) * u[i];
    }
}

// After a prompt pass over positions pos0 .. pos0 + n - 1, all followed by a prompt token: record the forced tokens as the
// loop's outputs (out_tokens[p] = prompt[p + 1]).
__global__ void fill_forced_kernel(const int* __restrict__ prompt, int* __restrict__ out_tokens, int pos0, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) out_tokens[pos0 + i] = prompt[pos0 + i + 1];
}

// argmax of every row of logits [n_rows][n] (first maximal index, src/inference.jl:360); one block per row.
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float* __restrict__ logits, int n, int* __restrict__ out_idx, int* status) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    const float* x = logits + (size_t)blockIdx.x * n;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < n; i += 1024) {
        const float v = x[i];
        if (v > bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) {
            bv = ov;
            bi = oi;
        }
    }
    if (lane == 0) {
        s_val[warp] = bv;
        s_idx[warp] = bi;
    }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < 32; ++w)
            if (s_val[w] > s_val[0] || (s_val[w] == s_val[0] && s_idx[w] < s_idx[0])) {
                s_val[0] = s_val[w];
                s_idx[0] = s_idx[w];
            }
        int best = s_idx[0];
        if (best < 0 || best >= n) {  // no finite maximum: all logits NaN
            if (status) atomicExch(status, DEV_ERR_BAD_INDEX);
            best = 0;
        }
        out_idx[blockIdx.x] = best;
    }
}

}  // namespace l2b
