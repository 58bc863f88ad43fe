// Split-KV ("flash-decoding") attention for one query position with grouped query heads.
// Replaces attention_weights! + the 1/sqrt(head_size) division + softmax! + combine_values!
// (src/inference.jl:263-278, 169-220).
//
// Grid: (n_heads / GQ) * nsplit blocks.  Block (hg, sp) reads the keys and values of positions
// [sp*chunk, (sp+1)*chunk) of one kv head exactly once and serves GQ query heads that share
// it (GQ = n_heads / n_kv_heads when that is 1, 2, 4 or 8; otherwise GQ = 1).  Each warp walks positions with an online softmax; warps are
// merged in shared memory; the block writes (max, sum, unnormalised output) per query head.
// The merge over splits happens in the prologue of the kernel that consumes the result.
//
// Cache layout (private to the library): key and value caches are [kv_head][seq_len][head_size]
// f32 (the reference keeps values transposed, (seq, hs, kv); both are f32).
#pragma once
#include "common.cuh"

namespace l2b {

struct AttnParams {
    const float* q;   // [n_heads][hs], after RoPE
    const float* kc;  // layer's key cache
    const float* vc;  // layer's value cache
    float* part_m;    // [n_heads][nsplit]
    float* part_l;    // [n_heads][nsplit]
    float* part_acc;  // [n_heads][nsplit][hs]
    const int* pos;   // device scalar, 0-based position of the query; positions 0..pos are attended
    int n_heads, n_kv, hs, seq_len, nsplit;
    int npos_override;  // >0: attend exactly this many positions (isolated-operator entry point)
};

constexpr int ATTN_WARPS = 4;

template <int GQ>  // query heads served per block; GQ divides n_heads / n_kv
__global__ void __launch_bounds__(ATTN_WARPS * 32) attention_split_kernel(const __grid_constant__ AttnParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hg = blockIdx.x / p.nsplit, sp = blockIdx.x % p.nsplit;
    const int kvh = (hg * GQ) / (p.n_heads / p.n_kv);
    const int npos = p.npos_override > 0 ? p.npos_override : (__ldcg(p.pos) + 1);
    const int chunk = (npos + p.nsplit - 1) / p.nsplit;
    const int t0 = sp * chunk, t1 = min(npos, t0 + chunk);
    const int hs = p.hs;
    const bool active = 4 * lane < hs;  // lane owns elements 4*lane .. 4*lane+3 of the head
    const float inv_div = sqrtf((float)hs);

    float4 qv[GQ], acc[GQ];
    float m[GQ], l[GQ];
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
        const int h = hg * GQ + g;
        qv[g] = active ? __ldcg(reinterpret_cast<const float4*>(p.q + (size_t)h * hs) + lane) : make_float4(0, 0, 0, 0);
        acc[g] = make_float4(0, 0, 0, 0);
        m[g] = -INFINITY;
        l[g] = 0.f;
    }
    const float* kbase = p.kc + (size_t)kvh * p.seq_len * hs;
    const float* vbase = p.vc + (size_t)kvh * p.seq_len * hs;
    for (int t = t0 + warp; t < t1; t += ATTN_WARPS) {
        float4 kv4 = make_float4(0, 0, 0, 0), vv4 = make_float4(0, 0, 0, 0);
        if (active) {
            kv4 = __ldcg(reinterpret_cast<const float4*>(kbase + (size_t)t * hs) + lane);
            vv4 = __ldcg(reinterpret_cast<const float4*>(vbase + (size_t)t * hs) + lane);
        }
#pragma unroll
        for (int g = 0; g < GQ; ++g) {
            float s = qv[g].x * kv4.x;
            s = fmaf(qv[g].y, kv4.y, s);
            s = fmaf(qv[g].z, kv4.z, s);
            s = fmaf(qv[g].w, kv4.w, s);
            s = warp_sum(s);
            s = s / inv_div;  // att ./= sqrt(Float32(head_size))
            const float mn = fmaxf(m[g], s);
            const float corr = expf(m[g] - mn);  // 0 on the first position (m = -inf)
            const float pr = expf(s - mn);
            l[g] = fmaf(l[g], corr, pr);
            acc[g].x = fmaf(acc[g].x, corr, pr * vv4.x);
            acc[g].y = fmaf(acc[g].y, corr, pr * vv4.y);
            acc[g].z = fmaf(acc[g].z, corr, pr * vv4.z);
            acc[g].w = fmaf(acc[g].w, corr, pr * vv4.w);
            m[g] = mn;
        }
    }
    // merge the warps
    __shared__ float sm[ATTN_WARPS][GQ], sl[ATTN_WARPS][GQ];
    __shared__ float4 sacc[ATTN_WARPS][GQ][32];
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
        if (lane == 0) {
            sm[warp][g] = m[g];
            sl[warp][g] = l[g];
        }
        sacc[warp][g][lane] = acc[g];
    }
    __syncthreads();
    for (int g = warp; g < GQ; g += ATTN_WARPS) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; ++w) M = fmaxf(M, sm[w][g]);
        float L = 0.f;
        float4 a = make_float4(0, 0, 0, 0);
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; ++w) {
            const float wgt = (sm[w][g] == -INFINITY) ? 0.f : expf(sm[w][g] - M);
            L = fmaf(sl[w][g], wgt, L);
            const float4 b = sacc[w][g][lane];
            a.x = fmaf(b.x, wgt, a.x);
            a.y = fmaf(b.y, wgt, a.y);
            a.z = fmaf(b.z, wgt, a.z);
            a.w = fmaf(b.w, wgt, a.w);
        }
        const int h = hg * GQ + g;
        if (lane == 0) {
            p.part_m[(size_t)h * p.nsplit + sp] = M;
            p.part_l[(size_t)h * p.nsplit + sp] = L;
        }
        if (active) reinterpret_cast<float4*>(p.part_acc + ((size_t)h * p.nsplit + sp) * hs)[lane] = a;
    }
}

}  // namespace l2b
