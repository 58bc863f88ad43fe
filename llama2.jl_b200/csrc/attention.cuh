// Split-KV ("flash-decoding") attention with grouped query heads: one query position per launch on the decode path
// (attention_decode_kernel), several in the prompt passes and batched decode (attention_split_kernel).
// Replaces attention_weights! + the 1/sqrt(head_size) division + softmax! + combine_values!
// (src/inference.jl:263-278, 169-220).
//
// Grid: (n_heads / GQ) * nsplit blocks.  Block (hg, sp) reads the keys and values of positions
// [sp*chunk, (sp+1)*chunk) of one kv head exactly once and serves GQ query heads that share
// it (GQ = n_heads / n_kv_heads when that is 1, 2, 4 or 8; otherwise GQ = 1).  Each warp walks
// positions with an online softmax, several positions' loads in flight at a time; warps are
// merged in shared memory; the block writes (max, sum, unnormalised output) per query head to
// scratch memory.  The block that finishes last for a head group (an atomic ticket) merges the
// nsplit partial results and writes the attention output, so no further kernel is needed.
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
    float* out;       // [n_heads][hs] attention output
    // scratch (global memory beyond inputs and outputs)
    float* part_m;    // [n_heads][nsplit]
    float* part_l;    // [n_heads][nsplit]
    float* part_acc;  // [n_heads][nsplit][hs]
    int* tickets;     // [n_heads / GQ], zero before the launch; left zero after it
    const int* pos;   // device scalar, 0-based position of the (first) query; positions 0..pos are attended.  Null: pos_base
    int n_heads, n_kv, hs, seq_len, nsplit;
    int npos_override;  // >0: attend exactly this many positions (isolated-operator entry point)
    int nq;             // 2: two consecutive query positions (pos, pos + 1) per launch; 0 or 1: one
    int q_stride;       // elements between the two positions' q (and out) vectors
    int min_chunk;      // positions per split below which splitting is not worth it (0: ATTN_MIN_CHUNK)
    int pos_base;       // position of the first query when `pos` is null (launches outside the captured token graph)
    const int* pos_list;     // batched decode: query qi belongs to its own sequence, at position pos_list[qi] ...
    size_t cache_stride_q;   // ... whose caches start cache_stride_q * qi elements after kc / vc
    int late_trigger;           // measurement build only: release the dependent kernel at the end instead of at the start
    unsigned long long* trace;  // measurement build only: 16 time stamps per block of the decode kernel, or null
};

#ifdef L2B_MEASURE
#define ATTN_TRACE(i)                                                                                                   \
    do {                                                                                                                \
        if (p.trace && threadIdx.x == 0) asm volatile("{.reg .u64 t; mov.u64 t, %%globaltimer; st.global.u64 [%0], t;}" \
                                                      ::"l"(p.trace + (size_t)blockIdx.x * 16 + (i)) : "memory");          \
    } while (0)
#else
#define ATTN_TRACE(i) do {} while (0)
#endif

constexpr int ATTN_WARPS = 4;
constexpr int ATTN_UNROLL = 4;      // positions whose key/value loads a warp keeps in flight
constexpr int ATTN_MERGE_BATCH = 16;  // partial results of the splits fetched together by the merging block
constexpr int ATTN_MIN_CHUNK = 16;  // positions per split below which splitting costs more than it saves

// What follows the walk over the positions: the warps of a block are merged in shared memory; with one active split the
// block writes the attention output, otherwise (max, sum, unnormalised output) per query head go to scratch memory and the
// block that finishes last for the head group (an atomic ticket) merges the splits.
template <int GQ>
__device__ __forceinline__ void attention_merge(const AttnParams& p, const float (&m)[GQ], const float (&l)[GQ], const float4 (&acc)[GQ], int hg, int sp, int active,
                                                int hq, float* obase, int* ticket_p, bool lane_active) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hs = p.hs;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    __shared__ float sm[ATTN_WARPS][GQ], sl[ATTN_WARPS][GQ];
    __shared__ float4 sacc[ATTN_WARPS][GQ][32];
    __shared__ int s_last;
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
        float Ls = 0.f;
        float4 a = zero4;
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; ++w) {
            const float wgt = (sm[w][g] == -INFINITY) ? 0.f : exp2f(sm[w][g] - M);
            Ls = fmaf(sl[w][g], wgt, Ls);
            const float4 b = sacc[w][g][lane];
            a.x = fmaf(b.x, wgt, a.x);
            a.y = fmaf(b.y, wgt, a.y);
            a.z = fmaf(b.z, wgt, a.z);
            a.w = fmaf(b.w, wgt, a.w);
        }
        const int h = hg * GQ + g;
        if (active == 1) {  // nothing to merge across blocks
            if (lane_active) {
                const float inv = __frcp_rn(Ls);
                a.x *= inv; a.y *= inv; a.z *= inv; a.w *= inv;
                reinterpret_cast<float4*>(obase + (size_t)h * hs)[lane] = a;
            }
        } else {
            if (lane == 0) {
                p.part_m[(size_t)(hq + h) * p.nsplit + sp] = M;
                p.part_l[(size_t)(hq + h) * p.nsplit + sp] = Ls;
            }
            if (lane_active) reinterpret_cast<float4*>(p.part_acc + ((size_t)(hq + h) * p.nsplit + sp) * hs)[lane] = a;
        }
    }
    if (active == 1) return;
    // The last block of this head group merges the splits.  One thread per block publishes: the barrier orders the block's
    // partial results before its fence, and fences are cumulative, so the other threads need none.
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const int ticket = atomicAdd(ticket_p, 1);
        s_last = (ticket == active - 1);
        if (s_last) {
            *ticket_p = 0;  // ready for the next launch
            __threadfence();
        }
    }
    __syncthreads();
    if (!s_last) return;
    for (int g = warp; g < GQ; g += ATTN_WARPS) {
        const int h = hg * GQ + g;
        const float* pm = p.part_m + (size_t)(hq + h) * p.nsplit;
        const float* pl = p.part_l + (size_t)(hq + h) * p.nsplit;
        // Up to ATTN_MERGE_BATCH partial results are fetched together, and before the arithmetic on the maxima: a loop of small
        // batches would pay the L2 latency once per batch, in series, on the critical path of the token.
        float4 b[ATTN_MERGE_BATCH];
        auto fetch = [&](int s0) {
#pragma unroll
            for (int u = 0; u < ATTN_MERGE_BATCH; ++u) {
                b[u] = zero4;
                if (lane_active && s0 + u < active) b[u] = __ldcg(reinterpret_cast<const float4*>(p.part_acc + ((size_t)(hq + h) * p.nsplit + s0 + u) * hs) + lane);
            }
        };
        fetch(0);
        // lane s holds split s (nsplit <= 32)
        const float ms = lane < active ? __ldcg(pm + lane) : -INFINITY;
        const float ls = lane < active ? __ldcg(pl + lane) : 0.f;
        const float M = warp_max(ms);
        const float wgt = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
        const float Ls = warp_sum(ls * wgt);
        float4 a = zero4;
        for (int s0 = 0; s0 < active; s0 += ATTN_MERGE_BATCH) {
            if (s0) fetch(s0);
#pragma unroll
            for (int u = 0; u < ATTN_MERGE_BATCH; ++u) {
                const float wu = __shfl_sync(0xffffffffu, wgt, (s0 + u) & 31);
                if (s0 + u < active) {
                    a.x = fmaf(b[u].x, wu, a.x);
                    a.y = fmaf(b[u].y, wu, a.y);
                    a.z = fmaf(b[u].z, wu, a.z);
                    a.w = fmaf(b[u].w, wu, a.w);
                }
            }
        }
        if (lane_active) {
            const float inv = __frcp_rn(Ls);
            a.x *= inv; a.y *= inv; a.z *= inv; a.w *= inv;
            reinterpret_cast<float4*>(obase + (size_t)h * hs)[lane] = a;
        }
    }
}

// GQ: query heads served per block (divides n_heads / n_kv).  NQ = 1: one query position per launch; any other value: the grid
// holds p.nq copies of the (head group, split) blocks, copy qi serving the query at position pos + qi (2 in the two-position
// prompt passes of the decode chain, up to a few hundred in the many-token prompt pass).
template <int GQ, int NQ = 1>
__device__ __forceinline__ void attention_split_body(const AttnParams& p) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // with two query positions the grid holds two copies of the (head group, split) blocks: copy qi serves position pos + qi
    const int ngroups = p.n_heads / GQ;
    const int qi = (NQ > 1) ? (int)blockIdx.x / (ngroups * p.nsplit) : 0;  // NQ = 1: everything below folds to the one-position code
    const int bx = (int)blockIdx.x - qi * ngroups * p.nsplit;
    const int hg = bx / p.nsplit, sp = bx % p.nsplit;
    const int kvh = (hg * GQ) / (p.n_heads / p.n_kv);
    const int npos = p.npos_override > 0 ? p.npos_override
                     : (NQ != 1 && p.pos_list) ? __ldg(p.pos_list + qi) + 1
                                               : ((p.pos ? __ldcg(p.pos) : p.pos_base) + 1 + qi);
    const float* const qbase = p.q + (size_t)qi * p.q_stride;
    float* const obase = p.out + (size_t)qi * p.q_stride;
    const int hq = qi * p.n_heads;   // first row of this position in the partial-result scratch
    int* const ticket_p = p.tickets + qi * ngroups + hg;
    // Short contexts use fewer splits (at least ATTN_MIN_CHUNK positions each): blocks beyond `active` leave at
    // once, and a single active split writes its result directly, with no partials and no merge.
    const int mc = p.min_chunk > 0 ? p.min_chunk : ATTN_MIN_CHUNK;
    const int active = min(p.nsplit, (npos + mc - 1) / mc);
    if (sp >= active) return;
    const int chunk = (npos + active - 1) / active;
    const int t0 = sp * chunk, t1 = min(npos, t0 + chunk);
    const int hs = p.hs;
    const bool lane_active = 4 * lane < hs;  // lane owns elements 4*lane .. 4*lane+3 of the head
    // scores carry the factor log2(e) / sqrt(head_size) and the softmax uses exp2, as in the decode kernel: a division and two
    // natural exponentials per position and head are most of this loop's instructions otherwise
    const float scale2 = 1.4426950408889634f / sqrtf((float)hs);
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);

    float4 qv[GQ], acc[GQ];
    float m[GQ], l[GQ];
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
        const int h = hg * GQ + g;
        qv[g] = lane_active ? __ldcg(reinterpret_cast<const float4*>(qbase + (size_t)h * hs) + lane) : zero4;
        acc[g] = zero4;
        m[g] = -INFINITY;
        l[g] = 0.f;
    }
    const size_t seq_off = (NQ != 1) ? (size_t)qi * p.cache_stride_q : 0;
    const float* kbase = p.kc + seq_off + (size_t)kvh * p.seq_len * hs;
    const float* vbase = p.vc + seq_off + (size_t)kvh * p.seq_len * hs;
    for (int tb = t0 + warp * ATTN_UNROLL; tb < t1; tb += ATTN_WARPS * ATTN_UNROLL) {
        float4 kk[ATTN_UNROLL], vv[ATTN_UNROLL];
#pragma unroll
        for (int u = 0; u < ATTN_UNROLL; ++u) {
            kk[u] = vv[u] = zero4;
            if (lane_active && tb + u < t1) {
                kk[u] = __ldcg(reinterpret_cast<const float4*>(kbase + (size_t)(tb + u) * hs) + lane);
                vv[u] = __ldcg(reinterpret_cast<const float4*>(vbase + (size_t)(tb + u) * hs) + lane);
            }
        }
#pragma unroll
        for (int u = 0; u < ATTN_UNROLL; ++u) {
            if (tb + u < t1) {
#pragma unroll
                for (int g = 0; g < GQ; ++g) {
                    float s = qv[g].x * kk[u].x;
                    s = fmaf(qv[g].y, kk[u].y, s);
                    s = fmaf(qv[g].z, kk[u].z, s);
                    s = fmaf(qv[g].w, kk[u].w, s);
                    s = warp_sum(s);
                    s = s * scale2;  // att ./= sqrt(Float32(head_size)), in the log2 domain
                    const float mn = fmaxf(m[g], s);
                    const float corr = exp2f(m[g] - mn);  // 0 on the first position (m = -inf)
                    const float pr = exp2f(s - mn);
                    l[g] = fmaf(l[g], corr, pr);
                    acc[g].x = fmaf(acc[g].x, corr, pr * vv[u].x);
                    acc[g].y = fmaf(acc[g].y, corr, pr * vv[u].y);
                    acc[g].z = fmaf(acc[g].z, corr, pr * vv[u].z);
                    acc[g].w = fmaf(acc[g].w, corr, pr * vv[u].w);
                    m[g] = mn;
                }
            }
        }
    }
    attention_merge<GQ>(p, m, l, acc, hg, sp, active, hq, obase, ticket_p, lane_active);
}

// ---- decode: one query position per launch, built for latency ------------------------------------------------
// Grid: (n_heads / GQ) * nsplit blocks of ATTN_DW warps, launched as thread-block clusters of ATTN_CL consecutive blocks
// (nsplit is a multiple of ATTN_CL), so a head group is served by nsplit / ATTN_CL clusters.
//  * The keys and values of earlier positions were written by earlier tokens: the first batch of every warp is fetched
//    BEFORE the wait on the previous kernel (which writes q and this position's key and value), so the cache latency hides
//    behind that kernel's tail.
//  * A batch of ATTN_UNROLL positions is scored without branches (all dot products and their lane reductions are independent),
//    then folded into the running softmax with one maximum and one set of exponentials per batch.
//  * The blocks of a cluster merge through distributed shared memory: every block reduces its warps in its own shared memory
//    and stores each part of the result into the shared memory of the block that finishes that part of the output; one
//    cluster barrier later every block combines what it received and writes its slice.  A launch with one cluster per head
//    group (the host's choice up to 512 positions), and any launch up to ATTN_CL * ATTN_DW * ATTN_UNROLL = 256 positions, needs
//    no global scratch, fence or atomic at all.  Beyond that the clusters of a head group exchange one partial result per
//    cluster through scratch memory and a ticket.
constexpr int ATTN_CL = 8;  // blocks per cluster (the portable maximum)
constexpr int ATTN_DW = 8;  // warps per block
constexpr int ATTN_CLUSTER_POS = ATTN_CL * ATTN_DW * ATTN_UNROLL;  // positions a cluster takes in one batch per warp

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_map(const void* smem_ptr, uint32_t rank) {  // the same variable in block `rank` of the cluster
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(smem_ptr)), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) { asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ void st_cluster_f32x4(uint32_t addr, float4 v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

// PDL = false: launched without a programmatic dependency (no previous kernel to wait for).
template <int GQ, bool PDL>
__device__ __forceinline__ void attention_decode_body(const AttnParams& p) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    ATTN_TRACE(0);
    const int hg = (int)blockIdx.x / p.nsplit, sp = (int)blockIdx.x % p.nsplit;
    const int cg = sp / ATTN_CL, rank = sp % ATTN_CL;  // cluster of the head group, block of the cluster (clusters are consecutive blocks)
    const int ncl = p.nsplit / ATTN_CL;
    const int kvh = (hg * GQ) / (p.n_heads / p.n_kv);
    const int npos = p.npos_override > 0 ? p.npos_override : ((p.pos ? __ldcg(p.pos) : p.pos_base) + 1);  // the position is set before the token starts
    // clusters at work: one per ATTN_CLUSTER_POS positions (or per min_chunk); the others leave at once, whole
    const int per = p.min_chunk > 0 ? p.min_chunk : ATTN_CLUSTER_POS;
    const int ac = min(ncl, (npos + per - 1) / per);
    if (cg >= ac) return;
    const int nblk = ac * ATTN_CL;
    const int chunk = (npos + nblk - 1) / nblk;
    const int t0 = min(npos, (cg * ATTN_CL + rank) * chunk), t1 = min(npos, t0 + chunk);  // (an empty range contributes nothing)
    const int hs = p.hs;
    const bool lane_active = 4 * lane < hs;
    // A warp's own instruction stream is the critical path of this kernel (dependent instructions issue every ten cycles or so),
    // so the arithmetic is kept short: att ./= sqrt(Float32(head_size)) and the softmax's exp become one multiplication
    // by log2(e) / sqrt(head_size) and exp2 (a single special-function instruction, 2 ulp); maxima are kept in the same
    // log2 domain, in which all merges below work; normalisation multiplies by a correctly rounded reciprocal.
    const float inv_div = 1.4426950408889634f / sqrtf((float)hs);
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* kbase = p.kc + (size_t)kvh * p.seq_len * hs;
    const float* vbase = p.vc + (size_t)kvh * p.seq_len * hs;
    const int tb0 = t0 + warp * ATTN_UNROLL;

    float4 kk[ATTN_UNROLL], vv[ATTN_UNROLL];
#pragma unroll
    for (int u = 0; u < ATTN_UNROLL; ++u) {
        kk[u] = vv[u] = zero4;
        const int t = tb0 + u;
        if (lane_active && t < t1 && t < npos - 1) {
            kk[u] = __ldcg(reinterpret_cast<const float4*>(kbase + (size_t)t * hs) + lane);
            vv[u] = __ldcg(reinterpret_cast<const float4*>(vbase + (size_t)t * hs) + lane);
        }
    }
    if (PDL) pdl_wait();
    ATTN_TRACE(1);
    float4 qv[GQ], acc[GQ];
    float m[GQ], l[GQ];
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
        qv[g] = lane_active ? __ldcg(reinterpret_cast<const float4*>(p.q + (size_t)(hg * GQ + g) * hs) + lane) : zero4;
        acc[g] = zero4;
        m[g] = -INFINITY;
        l[g] = 0.f;
    }
#pragma unroll
    for (int u = 0; u < ATTN_UNROLL; ++u) {  // the position the previous kernel has just written, if it is in this batch
        const int t = tb0 + u;
        if (lane_active && t < t1 && t == npos - 1) {
            kk[u] = __ldcg(reinterpret_cast<const float4*>(kbase + (size_t)t * hs) + lane);
            vv[u] = __ldcg(reinterpret_cast<const float4*>(vbase + (size_t)t * hs) + lane);
        }
    }
    for (int tb = tb0; tb < t1; tb += ATTN_DW * ATTN_UNROLL) {
        if (tb != tb0) {
#pragma unroll
            for (int u = 0; u < ATTN_UNROLL; ++u) {
                kk[u] = vv[u] = zero4;
                if (lane_active && tb + u < t1) {
                    kk[u] = __ldcg(reinterpret_cast<const float4*>(kbase + (size_t)(tb + u) * hs) + lane);
                    vv[u] = __ldcg(reinterpret_cast<const float4*>(vbase + (size_t)(tb + u) * hs) + lane);
                }
            }
        }
        float s[ATTN_UNROLL][GQ];
#pragma unroll
        for (int u = 0; u < ATTN_UNROLL; ++u)
#pragma unroll
            for (int g = 0; g < GQ; ++g) {
                float d = qv[g].x * kk[u].x;
                d = fmaf(qv[g].y, kk[u].y, d);
                d = fmaf(qv[g].z, kk[u].z, d);
                s[u][g] = fmaf(qv[g].w, kk[u].w, d);
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < ATTN_UNROLL; ++u)
#pragma unroll
                for (int g = 0; g < GQ; ++g) s[u][g] += __shfl_xor_sync(0xffffffffu, s[u][g], o);
#pragma unroll
        for (int g = 0; g < GQ; ++g) {
            float mx = m[g];
#pragma unroll
            for (int u = 0; u < ATTN_UNROLL; ++u) {
                s[u][g] = (tb + u < t1) ? s[u][g] * inv_div : -INFINITY;  // positions beyond the range weigh nothing
                mx = fmaxf(mx, s[u][g]);
            }
            const float corr = exp2f(m[g] - mx);  // 0 for the first batch (m = -inf; the batch's first position is always in range)
            float ps = 0.f;
            float4 pv = zero4;
#pragma unroll
            for (int u = 0; u < ATTN_UNROLL; ++u) {
                const float pr = exp2f(s[u][g] - mx);
                ps += pr;
                pv.x = fmaf(pr, vv[u].x, pv.x);
                pv.y = fmaf(pr, vv[u].y, pv.y);
                pv.z = fmaf(pr, vv[u].z, pv.z);
                pv.w = fmaf(pr, vv[u].w, pv.w);
            }
            l[g] = fmaf(l[g], corr, ps);
            acc[g].x = fmaf(acc[g].x, corr, pv.x);
            acc[g].y = fmaf(acc[g].y, corr, pv.y);
            acc[g].z = fmaf(acc[g].z, corr, pv.z);
            acc[g].w = fmaf(acc[g].w, corr, pv.w);
            m[g] = mx;
        }
    }
    ATTN_TRACE(2);

    // ---- the warps of this block, in its own shared memory
    constexpr int PER_BLOCK = GQ * 32 / ATTN_CL;  // float4s of the head group's output that one block of the cluster finishes
    __shared__ float sm[ATTN_DW][GQ], sl[ATTN_DW][GQ];
    __shared__ float4 sacc[ATTN_DW][GQ][32];
    // what the blocks of the cluster send to this one: per sending block, maximum and sum of every query head and the
    // PER_BLOCK float4s of unnormalised output that this block finishes
    __shared__ float rx_m[ATTN_CL][GQ], rx_l[ATTN_CL][GQ];
    __shared__ float4 rx_a[ATTN_CL][PER_BLOCK];
    __shared__ int s_last;
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
        if (lane == 0) {
            sm[warp][g] = m[g];
            sl[warp][g] = l[g];
        }
        sacc[warp][g][lane] = acc[g];
    }
    __syncthreads();
    for (int g = warp; g < GQ; g += ATTN_DW) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATTN_DW; ++w) M = fmaxf(M, sm[w][g]);
        float Ls = 0.f;
        float4 a = zero4;
#pragma unroll
        for (int w = 0; w < ATTN_DW; ++w) {
            const float wgt = (sm[w][g] == -INFINITY) ? 0.f : exp2f(sm[w][g] - M);
            Ls = fmaf(sl[w][g], wgt, Ls);
            const float4 b = sacc[w][g][lane];
            a.x = fmaf(b.x, wgt, a.x);
            a.y = fmaf(b.y, wgt, a.y);
            a.z = fmaf(b.z, wgt, a.z);
            a.w = fmaf(b.w, wgt, a.w);
        }
        // ---- stored into the shared memory of the block that finishes this part of the output (remote stores): after ONE
        // cluster barrier every block works on its own shared memory only, so nobody has to outlive a reader
        const int item = g * 32 + lane;
        st_cluster_f32x4(cluster_map(&rx_a[rank][item % PER_BLOCK], (uint32_t)(item / PER_BLOCK)), a);
        if (lane < ATTN_CL) {
            st_cluster_f32(cluster_map(&rx_m[rank][g], (uint32_t)lane), M);
            st_cluster_f32(cluster_map(&rx_l[rank][g], (uint32_t)lane), Ls);
        }
    }
    ATTN_TRACE(5);
    cluster_sync_all();
    ATTN_TRACE(6);
    if ((int)threadIdx.x < PER_BLOCK) {
        const int item = rank * PER_BLOCK + (int)threadIdx.x;
        const int ig = item >> 5, il = item & 31;
        float M = -INFINITY;
#pragma unroll
        for (int c = 0; c < ATTN_CL; ++c) M = fmaxf(M, rx_m[c][ig]);
        float Ls = 0.f;
        float4 a = zero4;
#pragma unroll
        for (int c = 0; c < ATTN_CL; ++c) {
            const float wgt = (rx_m[c][ig] == -INFINITY) ? 0.f : exp2f(rx_m[c][ig] - M);
            Ls = fmaf(rx_l[c][ig], wgt, Ls);
            const float4 b = rx_a[c][threadIdx.x];
            a.x = fmaf(b.x, wgt, a.x);
            a.y = fmaf(b.y, wgt, a.y);
            a.z = fmaf(b.z, wgt, a.z);
            a.w = fmaf(b.w, wgt, a.w);
        }
        const int h = hg * GQ + ig;
        if (4 * il < hs) {
            if (ac == 1) {  // the cluster saw every position: this is the attention output
                const float inv = __frcp_rn(Ls);
                a.x *= inv; a.y *= inv; a.z *= inv; a.w *= inv;
                reinterpret_cast<float4*>(p.out + (size_t)h * hs)[il] = a;
            } else {
                reinterpret_cast<float4*>(p.part_acc + ((size_t)h * ncl + cg) * hs)[il] = a;
                if (il == 0) {
                    p.part_m[(size_t)h * ncl + cg] = M;
                    p.part_l[(size_t)h * ncl + cg] = Ls;
                }
            }
        }
    }
    if (ac == 1) {
        ATTN_TRACE(3);
        return;
    }
    // ---- several clusters per head group: every block publishes its part of the cluster's partial result, the cluster that
    // finishes last (a ticket counting blocks) merges the clusters' partial results
    int* const ticket_p = p.tickets + hg;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();  // cumulative: covers what the block's threads wrote before the barrier
        const int ticket = atomicAdd(ticket_p, 1);
        s_last = (ticket == ac * ATTN_CL - 1);
        if (s_last) __threadfence();
    }
    __syncthreads();
    ATTN_TRACE(3);
    if (!s_last) return;
    for (int i = (int)threadIdx.x; i < GQ * 32; i += ATTN_DW * 32) {
        const int g = i >> 5, l4 = i & 31, h = hg * GQ + g;
        float Mc[4], Lc[4];
        float4 Ac[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {  // nsplit <= 4 * ATTN_CL
            Mc[c] = -INFINITY;
            Lc[c] = 0.f;
            Ac[c] = zero4;
            if (c < ac) {
                Mc[c] = __ldcg(p.part_m + (size_t)h * ncl + c);
                Lc[c] = __ldcg(p.part_l + (size_t)h * ncl + c);
                if (4 * l4 < hs) Ac[c] = __ldcg(reinterpret_cast<const float4*>(p.part_acc + ((size_t)h * ncl + c) * hs) + l4);
            }
        }
        const float M = fmaxf(fmaxf(Mc[0], Mc[1]), fmaxf(Mc[2], Mc[3]));
        float Ls = 0.f;
        float4 a = zero4;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float wgt = (Mc[c] == -INFINITY) ? 0.f : exp2f(Mc[c] - M);
            Ls = fmaf(Lc[c], wgt, Ls);
            a.x = fmaf(Ac[c].x, wgt, a.x);
            a.y = fmaf(Ac[c].y, wgt, a.y);
            a.z = fmaf(Ac[c].z, wgt, a.z);
            a.w = fmaf(Ac[c].w, wgt, a.w);
        }
        if (4 * l4 < hs) {
            const float inv = __frcp_rn(Ls);
            a.x *= inv; a.y *= inv; a.z *= inv; a.w *= inv;
            reinterpret_cast<float4*>(p.out + (size_t)h * hs)[l4] = a;
        }
    }
    if (threadIdx.x == 0) *ticket_p = 0;  // ready for the next launch (ordered by the kernel boundary)
}

template <int GQ>
__global__ void __launch_bounds__(ATTN_DW * 32) attention_decode_kernel(const __grid_constant__ AttnParams p) {
#ifdef L2B_MEASURE
    if (p.late_trigger) {  // measurement: the next kernel's blocks start only when this one is done
        attention_decode_body<GQ, true>(p);
        pdl_launch_dependents();
        return;
    }
#endif
    pdl_launch_dependents();
    attention_decode_body<GQ, true>(p);
}

template <int GQ, int NQ = 1>
__global__ void __launch_bounds__(ATTN_WARPS * 32) attention_split_kernel(const __grid_constant__ AttnParams p) {
    pdl_launch_dependents();
    pdl_wait();
    attention_split_body<GQ, NQ>(p);
}

}  // namespace l2b
