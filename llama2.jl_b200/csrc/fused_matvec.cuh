// The fused matrix-vector kernel of the decode path: replaces matmul! (src/matmul.jl:3-23)
// together with the element-wise work around each call site in transformer!
// (src/inference.jl:236-312).
//
// One launch = prologue (build the activation vector in shared memory) + a stream of
// weight rows + an epilogue per pair of output rows.
//
//   prologue  : raw copy | rmsnorm (inference.jl:102-110) | embedding row + rmsnorm (:236,:244) |
//               merge of the split-KV attention partials; then, for k-quant weights, on-device
//               quantisation of the vector to 1..3 int8 planes (block_q8_K layout, kquants.jl:38-42)
//   weights   : every warp owns a private ring of shared-memory slots that it fills itself with
//               bulk asynchronous copies (TMA) and drains itself; a slot holds one super-block
//               for each lane and each of the two rows of a pair (64 super-blocks).  The first
//               slots are requested BEFORE the wait on the previous kernel (programmatic
//               dependent launch), so weight bytes already stream while the previous kernel
//               finishes.
//   epilogue  : store | residual add (:284,:305) | SwiGLU (:295-299) | RoPE + KV-cache write
//               (:255-260) | logits store + running argmax (:312,:360)
#pragma once
#include "kquants.cuh"

namespace l2b {

enum : int { PRO_COPY = 0, PRO_RMSNORM = 1, PRO_EMBED_RMSNORM = 2, PRO_ATTN_MERGE = 3 };
enum : int { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2, EPI_ROPE_Q = 3, EPI_ROPE_K = 4, EPI_STORE_V = 5, EPI_LOGITS = 6 };
enum : int { PAIR_ADJACENT = 0, PAIR_NEOX = 1, PAIR_DUAL = 2 };

constexpr int MV_MAX_SEG = 3;
constexpr int MV_MAX_WARPS = 16;
constexpr int MV_MAX_STAGES = 4;
constexpr int MV_REG_BLOCKS = 4;  // 256-value blocks a warp keeps in registers across the rmsnorm reduction

struct MvSegment {
    const uint8_t* w;    // rows A (for PAIR_DUAL: the gate matrix)
    const uint8_t* w2;   // rows B of PAIR_DUAL (the up matrix), else unused
    const __half* d6;    // q6_K: fp16 super-block scales of w (one per block, row-major)
    const __half* d6_2;  // same for w2
    float* out;          // destination vector / cache base
    int type;            // ggml type of the segment
    int npairs;          // number of row pairs
    int pair_mode;       // PAIR_*
    int epi;             // EPI_*
    int head_size;       // for RoPE / cache addressing
};

struct MvParams {
    MvSegment seg[MV_MAX_SEG];
    int nseg;
    int n_in;        // input length
    int lgG;         // log2 of lanes per row pair
    int nstages;     // ring depth per warp
    int planes;      // int8 activation planes (k-quant launches)
    // prologue
    int pro;
    const float* x_in;      // input vector (PRO_COPY, PRO_RMSNORM)
    const float* gain;      // rmsnorm gain
    float* x_out;           // PRO_EMBED_RMSNORM: where block 0 stores the raw embedding row (the residual stream)
    const uint8_t* emb;     // embedding table (device layout)
    const __half* emb_d6;
    int emb_type;
    const int* token;       // device scalar: current token id
    const int* pos;         // device scalar: current position (0-based)
    // PRO_ATTN_MERGE: partials of the split-KV attention
    const float* part_m;    // [n_heads][nsplit]
    const float* part_l;    // [n_heads][nsplit]
    const float* part_acc;  // [n_heads][nsplit][head_size]
    int nsplit;
    int attn_head_size;
    // epilogue extras
    const float* resid;     // EPI_RESIDUAL: vector added to the result (may alias out)
    const float* rope_cs;   // [seq_len][head_size/2][2] (cos, sin)
    int seq_len;
    float* amax_val;        // EPI_LOGITS: per-block best value   [gridDim.x]
    int* amax_idx;          // EPI_LOGITS: per-block best index   [gridDim.x]
    int* status;            // device status word
};

// ---- shared-memory carve-up (host and device agree through this helper) ------------------
struct MvSmem {
    int off_bar, off_act, off_xs, off_xf, off_ring, off_red, total;
    int plane_stride, slot_bytes;
};

__host__ __device__ inline MvSmem mv_smem_layout(int n_in, int planes, bool kquant, int warps, int nstages, int max_block_bytes) {
    MvSmem s;
    const int nb = n_in / QK_K;
    int o = 0;
    s.off_bar = o;
    o += MV_MAX_WARPS * MV_MAX_STAGES * 8;
    s.off_red = o;
    o += 64 * 4;
    o = (o + 127) & ~127;
    s.plane_stride = nb * ACT_STRIDE;
    s.off_act = o;
    if (kquant) o += planes * s.plane_stride;
    o = (o + 15) & ~15;
    s.off_xs = o;
    if (kquant) o += nb * 16 * 4;
    s.off_xf = o;
    if (!kquant) o += n_in * 4;
    o = (o + 127) & ~127;
    s.off_ring = o;
    s.slot_bytes = 64 * max_block_bytes;
    if (kquant) o += warps * nstages * s.slot_bytes;
    s.total = o;
    return s;
}

// ---- prologue pieces ---------------------------------------------------------------------

__device__ __forceinline__ float block_sum(float v, float* red, int warp, int lane, int nwarps) {
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nwarps; ++i) t += red[i];  // same order in every thread
    __syncthreads();
    return t;
}

// Quantise the 8 values a lane holds (values 8*lane .. 8*lane+7 of block b) into P planes.
template <int P>
__device__ __forceinline__ void quantise_block(const float (&v)[8], int lane, uint8_t* act, int plane_stride, float* xs16, int b) {
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
    amax = warp_max(amax);
    float d[3], id[3];
    d[0] = amax / 127.f;
    id[0] = amax > 0.f ? 127.f / amax : 0.f;
    d[1] = d[0] / 254.f;
    id[1] = id[0] * 254.f;
    d[2] = d[1] / 254.f;
    id[2] = id[1] * 254.f;
    float r[8], xh[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        r[e] = v[e];
        xh[e] = 0.f;
    }
#pragma unroll
    for (int k = 0; k < P; ++k) {
        uint32_t w0 = 0, w1 = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float q = rintf(r[e] * id[k]);
            q = fminf(127.f, fmaxf(-127.f, q));
            r[e] = fmaf(-q, d[k], r[e]);
            xh[e] = fmaf(q, d[k], xh[e]);
            const uint32_t byte = (uint32_t)((int)q) & 0xFFu;
            if (e < 4) w0 |= byte << (8 * e);
            else w1 |= byte << (8 * (e - 4));
        }
        uint8_t* rec = act + k * plane_stride + b * ACT_STRIDE;
        *reinterpret_cast<uint2*>(rec + 8 * lane) = make_uint2(w0, w1);
        if (lane == 0) *reinterpret_cast<float*>(rec + 256) = d[k];
    }
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) s += xh[e];
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    if ((lane & 1) == 0) xs16[b * 16 + (lane >> 1)] = s;
}

// Value i (0 <= i < n) of the prologue's source vector, before any normalisation.
struct ProSource {
    const MvParams* p;
    const uint8_t* emb_row;
    const __half* emb_d6_row;
    int nsplit;
};

__device__ __forceinline__ void load8(const MvParams& p, const ProSource& src, int i0, float (&v)[8]) {
    if (p.pro == PRO_COPY || p.pro == PRO_RMSNORM) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(p.x_in + i0));
        const float4 b = __ldcg(reinterpret_cast<const float4*>(p.x_in + i0 + 4));
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else if (p.pro == PRO_EMBED_RMSNORM) {
        if (p.emb_type == T_F32) {
            const float* row = reinterpret_cast<const float*>(src.emb_row);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = row[i0 + e];
        } else {
            const int b = i0 >> 8, k0 = i0 & 255;
            const uint8_t* blk = src.emb_row + (size_t)b * dev_block_bytes(p.emb_type);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                if (p.emb_type == T_Q4_K) v[e] = dequant_q45<false>(blk, k0 + e);
                else if (p.emb_type == T_Q5_K) v[e] = dequant_q45<true>(blk, k0 + e);
                else v[e] = dequant_q6(blk, __half2float(src.emb_d6_row[b]), k0 + e);
            }
        }
    } else {  // PRO_ATTN_MERGE: out[h][i] = sum_s acc_s[i] e^{m_s - M} / sum_s l_s e^{m_s - M}
        const int hs = p.attn_head_size, h = i0 / hs, i = i0 % hs, ns = p.nsplit;
        const float* pm = p.part_m + (size_t)h * ns;
        const float* pl = p.part_l + (size_t)h * ns;
        float M = -INFINITY;
        for (int s = 0; s < ns; ++s) M = fmaxf(M, __ldcg(pm + s));
        float L = 0.f, acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        for (int s = 0; s < ns; ++s) {
            const float ms = __ldcg(pm + s);
            const float wgt = (ms == -INFINITY) ? 0.f : expf(ms - M);
            L = fmaf(__ldcg(pl + s), wgt, L);
            const float* pa = p.part_acc + ((size_t)h * ns + s) * hs + i;
            const float4 a = __ldcg(reinterpret_cast<const float4*>(pa));
            const float4 b = __ldcg(reinterpret_cast<const float4*>(pa + 4));
            acc[0] = fmaf(a.x, wgt, acc[0]); acc[1] = fmaf(a.y, wgt, acc[1]); acc[2] = fmaf(a.z, wgt, acc[2]); acc[3] = fmaf(a.w, wgt, acc[3]);
            acc[4] = fmaf(b.x, wgt, acc[4]); acc[5] = fmaf(b.y, wgt, acc[5]); acc[6] = fmaf(b.z, wgt, acc[6]); acc[7] = fmaf(b.w, wgt, acc[7]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = acc[e] / L;
    }
}

// Build the activation vector in shared memory.  KQ: int8 planes + sums; else f32 copy.
template <bool KQ, int P>
__device__ __forceinline__ void build_activation(const MvParams& p, uint8_t* smem, const MvSmem& L, int warp, int lane, int nwarps) {
    ProSource src;
    src.p = &p;
    src.emb_row = nullptr;
    src.emb_d6_row = nullptr;
    const int n = p.n_in;
    if (p.pro == PRO_EMBED_RMSNORM) {
        const int tok = __ldcg(p.token);
        const size_t row_bytes = (p.emb_type == T_F32) ? (size_t)n * 4 : (size_t)(n / QK_K) * dev_block_bytes(p.emb_type);
        src.emb_row = p.emb + (size_t)tok * row_bytes;
        if (p.emb_type == T_Q6_K) src.emb_d6_row = p.emb_d6 + (size_t)tok * (n / QK_K);
    }
    float* red = reinterpret_cast<float*>(smem + L.off_red);
    uint8_t* act = smem + L.off_act;
    float* xs16 = reinterpret_cast<float*>(smem + L.off_xs);
    float* xf = reinterpret_cast<float*>(smem + L.off_xf);
    const bool norm = (p.pro == PRO_RMSNORM || p.pro == PRO_EMBED_RMSNORM);
    const int n8 = n / 8;  // groups of 8 values; a warp takes 32 consecutive groups (= one 256-value block) per turn
    const int turns = (n8 + 32 * nwarps - 1) / (32 * nwarps);

    auto fetch = [&](int turn, float (&v)[8]) {
        const int g = 32 * (warp + nwarps * turn) + lane;
        if (g < n8) load8(p, src, 8 * g, v);
        else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = 0.f;
        }
    };
    auto emit = [&](int turn, const float (&v)[8]) {
        const int g0 = 32 * (warp + nwarps * turn), g = g0 + lane;
        if (g0 >= n8) return;
        if (KQ) quantise_block<P>(v, lane, act, L.plane_stride, xs16, g0 >> 5);
        else if (g < n8) {
            *reinterpret_cast<float4*>(xf + 8 * g) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(xf + 8 * g + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
    };
    auto store_raw = [&](int turn, const float (&v)[8]) {  // the residual stream starts as the raw embedding row
        const int g = 32 * (warp + nwarps * turn) + lane;
        if (p.pro == PRO_EMBED_RMSNORM && blockIdx.x == 0 && g < n8) {
            *reinterpret_cast<float4*>(p.x_out + 8 * g) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(p.x_out + 8 * g + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
    };

    if (!norm) {
        for (int turn = 0; turn < turns; ++turn) {
            float v[8];
            fetch(turn, v);
            emit(turn, v);
        }
    } else {
        // pass 1: sum of squares; the first MV_REG_BLOCKS turns stay in registers for pass 2
        float keep[MV_REG_BLOCKS][8];
        float ss = 0.f;
#pragma unroll
        for (int turn = 0; turn < MV_REG_BLOCKS; ++turn) {
            if (turn < turns) {
                fetch(turn, keep[turn]);
                store_raw(turn, keep[turn]);
#pragma unroll
                for (int e = 0; e < 8; ++e) ss = fmaf(keep[turn][e], keep[turn][e], ss);
            }
        }
        for (int turn = MV_REG_BLOCKS; turn < turns; ++turn) {
            float v[8];
            fetch(turn, v);
            store_raw(turn, v);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(v[e], v[e], ss);
        }
        float tot = block_sum(ss, red, warp, lane, nwarps);
        tot /= (float)n;
        tot += 1e-5f;
        const float scale = 1.0f / sqrtf(tot);
        auto normalise = [&](int turn, float (&v)[8]) {
            const int g = 32 * (warp + nwarps * turn) + lane;
            if (g < n8) {
                const float4 ga = __ldg(reinterpret_cast<const float4*>(p.gain + 8 * g));
                const float4 gb = __ldg(reinterpret_cast<const float4*>(p.gain + 8 * g + 4));
                const float gw[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = gw[e] * (scale * v[e]);  // weight .* (ss .* x)
            }
        };
#pragma unroll
        for (int turn = 0; turn < MV_REG_BLOCKS; ++turn) {
            if (turn < turns) {
                normalise(turn, keep[turn]);
                emit(turn, keep[turn]);
            }
        }
        for (int turn = MV_REG_BLOCKS; turn < turns; ++turn) {
            float v[8];
            fetch(turn, v);
            normalise(turn, v);
            emit(turn, v);
        }
    }
    __syncthreads();
}

// ---- work enumeration ----------------------------------------------------------------------
// A "step" is PW = 32 >> lgG row pairs of one segment (k-quant) or one pair (f32).  Steps of all
// segments are numbered consecutively; warp gw of TW takes steps gw, gw+TW, ...
struct StepInfo {
    int seg;    // segment index, -1 = none
    int pair0;  // first pair of the step within the segment
};

__device__ __forceinline__ StepInfo find_step(const MvParams& p, int step, int pw) {
    StepInfo si;
    si.seg = -1;
    si.pair0 = 0;
    for (int s = 0; s < p.nseg; ++s) {
        const int nsteps = (p.seg[s].npairs + pw - 1) / pw;
        if (step < nsteps) {
            si.seg = s;
            si.pair0 = step * pw;
            return si;
        }
        step -= nsteps;
    }
    return si;
}

__device__ __forceinline__ void pair_rows(const MvSegment& sg, int t, int& rowA, int& rowB) {
    if (sg.pair_mode == PAIR_ADJACENT) {
        rowA = 2 * t;
        rowB = 2 * t + 1;
    } else if (sg.pair_mode == PAIR_NEOX) {
        const int h2 = sg.head_size >> 1;
        rowA = (t / h2) * sg.head_size + (t % h2);
        rowB = rowA + h2;
    } else {
        rowA = rowB = t;
    }
}

// ---- epilogue -------------------------------------------------------------------------------
struct ArgBest {
    float v;
    int i;
};
__device__ __forceinline__ void arg_update(ArgBest& b, float v, int i) {
    if (v > b.v || (v == b.v && i < b.i)) {
        b.v = v;
        b.i = i;
    }
}

__device__ __forceinline__ void epilogue_pair(const MvParams& p, const MvSegment& sg, int t, float vA, float vB, int pos, ArgBest& best) {
    int rowA, rowB;
    pair_rows(sg, t, rowA, rowB);
    switch (sg.epi) {
        case EPI_STORE:
            sg.out[rowA] = vA;
            sg.out[rowB] = vB;
            break;
        case EPI_RESIDUAL:
            sg.out[rowA] = __ldcg(p.resid + rowA) + vA;
            sg.out[rowB] = __ldcg(p.resid + rowB) + vB;
            break;
        case EPI_SWIGLU: {
            const float g = vA * (1.0f / (1.0f + expf(-vA)));
            sg.out[t] = g * vB;
            break;
        }
        case EPI_ROPE_Q:
        case EPI_ROPE_K: {
            const int hs = sg.head_size, h2 = hs >> 1;
            const int head = rowA / hs;
            const int i = (sg.pair_mode == PAIR_NEOX) ? (rowA % hs) : ((rowA % hs) >> 1);
            const float2 cs = __ldg(reinterpret_cast<const float2*>(p.rope_cs) + (size_t)pos * h2 + i);
            // (a + bi)(c + si): every product and sum rounded on its own, as the reference's complex multiply
            const float oa = __fsub_rn(__fmul_rn(vA, cs.x), __fmul_rn(vB, cs.y));
            const float ob = __fadd_rn(__fmul_rn(vA, cs.y), __fmul_rn(vB, cs.x));
            if (sg.epi == EPI_ROPE_Q) {
                sg.out[rowA] = oa;
                sg.out[rowB] = ob;
            } else {  // key cache [kv_head][seq_len][hs]
                float* dst = sg.out + ((size_t)head * p.seq_len + pos) * hs;
                dst[rowA % hs] = oa;
                dst[rowB % hs] = ob;
            }
            break;
        }
        case EPI_STORE_V: {  // value cache [kv_head][seq_len][hs]
            const int hs = sg.head_size;
            float* dst = sg.out + ((size_t)(rowA / hs) * p.seq_len + pos) * hs;
            dst[rowA % hs] = vA;
            dst[rowB % hs] = vB;
            break;
        }
        case EPI_LOGITS:
            sg.out[rowA] = vA;
            sg.out[rowB] = vB;
            arg_update(best, vA, rowA);
            arg_update(best, vB, rowB);
            break;
    }
}

// ---- the kernel --------------------------------------------------------------------------------
template <bool KQ, int P>
__global__ void __launch_bounds__(MV_MAX_WARPS * 32, 1) fused_matvec_kernel(const __grid_constant__ MvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int gw = blockIdx.x * nwarps + warp, TW = gridDim.x * nwarps;
    int max_bb = 0;
    if (KQ)
        for (int s = 0; s < p.nseg; ++s) max_bb = max(max_bb, dev_block_bytes(p.seg[s].type));
    const MvSmem L = mv_smem_layout(p.n_in, P, KQ, nwarps, p.nstages, max_bb);

    const int nb = p.n_in / QK_K;
    const int G = 1 << p.lgG, PW = KQ ? (32 >> p.lgG) : 1;
    const int nit = KQ ? (nb + G - 1) / G : 1;
    int total_steps = 0;
    for (int s = 0; s < p.nseg; ++s) total_steps += (p.seg[s].npairs + PW - 1) / PW;
    const int my_steps = (gw < total_steps) ? (total_steps - gw + TW - 1) / TW : 0;
    const int my_stages = my_steps * nit;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.off_bar) + warp * MV_MAX_STAGES;
    uint8_t* ring = smem + L.off_ring + (size_t)warp * p.nstages * L.slot_bytes;
    const int q = lane >> p.lgG, jl = lane & (G - 1);  // pair slot and block slot of this lane
    uint64_t policy = 0;

    // Issue the copies of this warp's stage s into slot s % nstages.  All lanes call it.
    auto issue_stage = [&](int s) {
        const int k = s / nit, it = s - k * nit;
        const StepInfo si = find_step(p, gw + k * TW, PW);
        const MvSegment& sg = p.seg[si.seg];
        const int bb = dev_block_bytes(sg.type);
        const int b0 = it * G, nblk = min(G, nb - b0);
        uint8_t* slot = ring + (size_t)(s % p.nstages) * L.slot_bytes;
        uint64_t* bar = bars + (s % p.nstages);
        const int npair_here = min(PW, sg.npairs - si.pair0);
        if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)(2 * npair_here * nblk * bb));
        __syncwarp();
        if (lane < 2 * PW) {
            const int qq = lane >> 1, sel = lane & 1;
            if (qq < npair_here) {
                int rowA, rowB;
                pair_rows(sg, si.pair0 + qq, rowA, rowB);
                const uint8_t* base = (sg.pair_mode == PAIR_DUAL && sel) ? sg.w2 : sg.w;
                const int row = sel ? rowB : rowA;
                const uint8_t* src = base + ((size_t)row * nb + b0) * bb;
                bulk_g2s(slot + (size_t)(sel * 32 + qq * G) * bb, src, (uint32_t)(nblk * bb), bar, policy);
            }
        }
    };

    if (KQ) {
        if (lane == 0) {
            for (int s = 0; s < p.nstages; ++s) mbar_init(bars + s, 1);
            fence_barrier_init();
            fence_proxy_async();
        }
        __syncwarp();
        policy = policy_evict_first();
        const int pre = min(p.nstages, my_stages);
        for (int s = 0; s < pre; ++s) issue_stage(s);
    }
    // Weights are constants; everything below reads what the previous kernel wrote.
    pdl_launch_dependents();
    pdl_wait();

    build_activation<KQ, P>(p, smem, L, warp, lane, nwarps);

    const int pos = p.pos ? __ldcg(p.pos) : 0;
    ArgBest best;
    best.v = -INFINITY;
    best.i = 0x7fffffff;
    const uint8_t* act = smem + L.off_act;
    const float* xs16 = reinterpret_cast<const float*>(smem + L.off_xs);
    const float* xf = reinterpret_cast<const float*>(smem + L.off_xf);
    bool dead = false;

    for (int k = 0; k < my_steps; ++k) {
        const StepInfo si = find_step(p, gw + k * TW, PW);
        const MvSegment& sg = p.seg[si.seg];
        float accA = 0.f, accB = 0.f;
        if (KQ) {
            const int bb = dev_block_bytes(sg.type);
            const int t = si.pair0 + q;
            const bool have_pair = t < sg.npairs;
            int rowA = 0, rowB = 0;
            if (have_pair) pair_rows(sg, t, rowA, rowB);
            for (int it = 0; it < nit; ++it) {
                const int s = k * nit + it;
                const int b = it * G + jl;
                // q6_K super-block scales travel outside the records: fetch them before waiting on the slot
                float dA = 0.f, dB = 0.f;
                if (sg.type == T_Q6_K && have_pair && b < nb) {
                    const __half* dsrcB = (sg.pair_mode == PAIR_DUAL) ? sg.d6_2 : sg.d6;
                    dA = __half2float(__ldg(sg.d6 + (size_t)rowA * nb + b));
                    dB = __half2float(__ldg(dsrcB + (size_t)rowB * nb + b));
                }
                if (!dead && !mbar_wait_bounded(bars + (s % p.nstages), (uint32_t)((s / p.nstages) & 1))) dead = true;
                dead = __any_sync(0xffffffffu, dead);
                if (!dead && have_pair && b < nb) {
                    const uint8_t* slot = ring + (size_t)(s % p.nstages) * L.slot_bytes;
                    const uint8_t* A = slot + (size_t)(q * G + jl) * bb;
                    const uint8_t* B = slot + (size_t)(32 + q * G + jl) * bb;
                    const uint8_t* ab = act + b * ACT_STRIDE;
                    const float* xb = xs16 + b * 16;
                    if (sg.type == T_Q4_K) dot2_q4k<P>(A, B, ab, L.plane_stride, xb, accA, accB);
                    else if (sg.type == T_Q5_K) dot2_q5k<P>(A, B, ab, L.plane_stride, xb, accA, accB);
                    else dot2_q6k<P>(A, B, dA, dB, ab, L.plane_stride, xb, accA, accB);
                }
                fence_proxy_async();  // order this lane's reads of the slot before the async-proxy refill
                __syncwarp();         // every lane is done reading the slot before it is refilled
                if (!dead && s + p.nstages < my_stages) issue_stage(s + p.nstages);
            }
            // sum over the G lanes of the pair
            for (int o = G >> 1; o > 0; o >>= 1) {
                accA += __shfl_xor_sync(0xffffffffu, accA, o);
                accB += __shfl_xor_sync(0xffffffffu, accB, o);
            }
            if (!dead && have_pair && jl == 0) epilogue_pair(p, sg, t, accA, accB, pos, best);
        } else {
            const int t = si.pair0;
            int rowA, rowB;
            pair_rows(sg, t, rowA, rowB);
            const float* baseB = reinterpret_cast<const float*>(sg.pair_mode == PAIR_DUAL ? sg.w2 : sg.w);
            const float4* wa = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(sg.w) + (size_t)rowA * p.n_in);
            const float4* wb = reinterpret_cast<const float4*>(baseB + (size_t)rowB * p.n_in);
            const float4* xv = reinterpret_cast<const float4*>(xf);
            const int n4 = p.n_in >> 2;
            for (int i = lane; i < n4; i += 32) {
                const float4 x4 = xv[i], a4 = __ldg(wa + i), b4 = __ldg(wb + i);
                accA = fmaf(a4.x, x4.x, accA); accA = fmaf(a4.y, x4.y, accA); accA = fmaf(a4.z, x4.z, accA); accA = fmaf(a4.w, x4.w, accA);
                accB = fmaf(b4.x, x4.x, accB); accB = fmaf(b4.y, x4.y, accB); accB = fmaf(b4.z, x4.z, accB); accB = fmaf(b4.w, x4.w, accB);
            }
            accA = warp_sum(accA);
            accB = warp_sum(accB);
            if (lane == 0) epilogue_pair(p, sg, t, accA, accB, pos, best);
        }
    }

    if (KQ && dead) {
        // Give copies still in flight a bounded chance to land before the block's shared memory is released.
        if (lane == 0) atomicExch(p.status, DEV_ERR_TMA_TIMEOUT);
        for (int s = 0; s < p.nstages; ++s) (void)mbar_wait_bounded(bars + s, 0), (void)mbar_wait_bounded(bars + s, 1);
    }

    if (p.amax_val) {  // EPI_LOGITS: first maximal index over this block's rows
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best.v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best.i, o);
            arg_update(best, ov, oi);
        }
        __shared__ float sv[MV_MAX_WARPS];
        __shared__ int sidx[MV_MAX_WARPS];
        if (lane == 0) {
            sv[warp] = best.v;
            sidx[warp] = best.i;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            ArgBest bb2 = {sv[0], sidx[0]};
            for (int w = 1; w < nwarps; ++w) arg_update(bb2, sv[w], sidx[w]);
            p.amax_val[blockIdx.x] = bb2.v;
            p.amax_idx[blockIdx.x] = bb2.i;
        }
    }
}

}  // namespace l2b
