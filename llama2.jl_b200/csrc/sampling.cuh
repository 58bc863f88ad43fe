// End-of-token step of the loop in `sample` (src/inference.jl:354-385): choose the next token
// on the device and advance the position, so that a generation loop needs no host round trip.
#pragma once
#include "common.cuh"

namespace l2b {

// Device-resident loop state; kernels read token/pos from here, so one captured graph serves
// every position.
struct Control {
    int token;          // token fed at this position
    int pos;            // 0-based position
    int n_prompt;       // prompt length; while pos+1 < n_prompt the next token is forced
    int use_seed;       // 1: uniform drawn from (seed, pos); 0: `uniform` below
    float temperature;  // 0 = greedy
    int pad;
    double uniform;
    unsigned long long seed;
};

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

struct FinalizeParams {
    const float* logits;
    int vocab;
    const float* amax_val;  // per-block maxima written by the logits kernel
    const int* amax_idx;
    int nparts;
    Control* ctl;
    const int* prompt;  // device copy of the prompt (may be null when n_prompt <= 1)
    int* out_tokens;    // out_tokens[pos] = token chosen after position pos (may be null)
    int advance;        // 1: ctl->token = next, ctl->pos += 1
    int* next_token;    // single-slot result for one-step calls
    unsigned* tp_epoch; // tensor parallelism: count of completed tokens, advanced here (null on one GPU)
    int* status;        // device status word: DEV_ERR_BAD_INDEX when no valid token could be chosen (may be null)
};

// The chosen token must be a row of the embedding table.  All-NaN logits (one NaN or Inf anywhere upstream, e.g. a corrupt
// fp16 scale in a model file) leave the argmax at its start value; the next embedding lookup would then read far outside the
// table.  Such a token is replaced by 0 and reported through the status word, so that the host call fails while every
// access of the launches already enqueued stays in bounds.
__device__ __forceinline__ int checked_token(int tok, int vocab, int* status) {
    if (tok >= 0 && tok < vocab) return tok;
    if (status) atomicExch(status, DEV_ERR_BAD_INDEX);
    return 0;
}

constexpr int FIN_THREADS = 1024;

// NT threads of one block (tid = 0 .. NT-1; `sync` is a barrier over exactly those threads).
// Greedy: argmax = first maximal index (Julia argmax, src/inference.jl:360).
// Temperature: logits ./= T; softmax!; inverse-CDF walk of StatsBase.wsample (src/inference.jl:361-368),
// with cumulative sums kept in f64.  Scratch: s_val[32], s_idx[32], s_sum[NT], s_choice in shared memory.
template <int NT, class Sync>
__device__ __forceinline__ void finalize_token_body(const FinalizeParams& p, int tid, float* s_val, int* s_idx, double* s_sum, int* s_choice_p,
                                                    Sync sync) {
    const int lane = tid & 31, warp = tid >> 5;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < p.nparts; i += NT) {
        const float v = __ldcg(p.amax_val + i);
        const int ix = __ldcg(p.amax_idx + i);
        if (v > bv || (v == bv && ix < bi)) {
            bv = v;
            bi = ix;
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
    sync();
    if (tid == 0) {
        for (int w = 1; w < NT / 32; ++w)
            if (s_val[w] > s_val[0] || (s_val[w] == s_val[0] && s_idx[w] < s_idx[0])) {
                s_val[0] = s_val[w];
                s_idx[0] = s_idx[w];
            }
        *s_choice_p = s_idx[0];
    }
    sync();
    const float T = p.ctl->temperature;
    const int pos = p.ctl->pos;
    if (T != 0.f) {
        const float mx = s_val[0] / T;  // maximum of logits ./ T  (T > 0)
        const int per = (p.vocab + NT - 1) / NT;
        const int i0 = tid * per, i1 = min(p.vocab, i0 + per);
        // pass 1: sum of exp
        float fs = 0.f;
        for (int i = i0; i < i1; ++i) fs += expf(__ldcg(p.logits + i) / T - mx);
        // total in f32 like sum(x) of the reference, order: per thread then tree
        s_sum[tid] = (double)fs;
        sync();
        for (int o = NT / 2; o > 0; o >>= 1) {
            if (tid < o) s_sum[tid] += s_sum[tid + o];
            sync();
        }
        const float denom = (float)s_sum[0];
        sync();
        // pass 2: probabilities and their f64 chunk sums
        double cs = 0.0;
        for (int i = i0; i < i1; ++i) cs += (double)(expf(__ldcg(p.logits + i) / T - mx) / denom);
        s_sum[tid] = cs;
        sync();
        if (tid == 0) {
            double u = p.ctl->uniform;
            if (p.ctl->use_seed) u = (double)(splitmix64(p.ctl->seed + (unsigned long long)pos) >> 11) * (1.0 / 9007199254740992.0);
            double total = 0.0;
            for (int t = 0; t < NT; ++t) total += s_sum[t];
            const double target = u * total;
            // find the chunk whose cumulative sum reaches the target, then walk inside it
            double cw = 0.0;
            int t = 0;
            while (t < NT - 1 && cw + s_sum[t] < target) cw += s_sum[t++];
            int c0 = t * per, c1 = min(p.vocab, c0 + per);
            if (c0 >= p.vocab) {
                c0 = p.vocab - 1;
                c1 = p.vocab;
            }
            int i = c0;
            cw += (double)(expf(__ldcg(p.logits + i) / T - mx) / denom);
            while (cw < target && i < c1 - 1) {
                ++i;
                cw += (double)(expf(__ldcg(p.logits + i) / T - mx) / denom);
            }
            *s_choice_p = i;
        }
        sync();
    }
    if (tid == 0) {
        const int choice = checked_token(*s_choice_p, p.vocab, p.status);
        int next = choice;
        if (pos + 1 < p.ctl->n_prompt && p.prompt) next = checked_token(p.prompt[pos + 1], p.vocab, p.status);
        if (p.out_tokens) p.out_tokens[pos] = next;
        if (p.next_token) *p.next_token = choice;
        if (p.advance) {
            p.ctl->token = next;
            p.ctl->pos = pos + 1;
        }
        if (p.tp_epoch) *p.tp_epoch += 1u;
    }
}

// One block of FIN_THREADS threads.
__global__ void __launch_bounds__(FIN_THREADS) finalize_token_kernel(const __grid_constant__ FinalizeParams p) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ double s_sum[FIN_THREADS];
    __shared__ int s_choice;
    finalize_token_body<FIN_THREADS>(p, (int)threadIdx.x, s_val, s_idx, s_sum, &s_choice, [] { __syncthreads(); });
}

// End of a two-position prompt pass (positions pos and pos + 1, both followed by a prompt token): nothing is sampled,
// the loop state moves on by two positions.
struct AdvanceParams {
    Control* ctl;
    const int* prompt;
    int* out_tokens;
    unsigned* epoch;
    int vocab;
    int* status;
};
__global__ void advance_pair_kernel(const __grid_constant__ AdvanceParams a) {
    Control* ctl = a.ctl;
    const int* prompt = a.prompt;
    int* out_tokens = a.out_tokens;
    unsigned* epoch = a.epoch;
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        const int pos = ctl->pos;
        const int t1 = checked_token(prompt[pos + 1], a.vocab, a.status), t2 = checked_token(prompt[pos + 2], a.vocab, a.status);
        if (out_tokens) {
            out_tokens[pos] = t1;
            out_tokens[pos + 1] = t2;
        }
        ctl->token = t2;
        ctl->pos = pos + 2;
        if (epoch) *epoch += 1u;
    }
}

// argmax over a plain vector (isolated-operator entry point): one block.
__global__ void __launch_bounds__(FIN_THREADS) argmax_kernel(const float* x, int n, float* out_val, int* out_idx) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < n; i += FIN_THREADS) {
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
        for (int w = 1; w < FIN_THREADS / 32; ++w)
            if (s_val[w] > s_val[0] || (s_val[w] == s_val[0] && s_idx[w] < s_idx[0])) {
                s_val[0] = s_val[w];
                s_idx[0] = s_idx[w];
            }
        out_val[0] = s_val[0];
        out_idx[0] = s_idx[0];
    }
}

}  // namespace l2b
