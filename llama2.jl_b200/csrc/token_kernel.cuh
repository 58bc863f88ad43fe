// One persistent kernel per token: transformer! (src/inference.jl:222-315) and the end of the loop body of `sample`
// (:354-385) as ONE launch for k-quant models on one GPU.
//
// The kernel chain of fused_matvec.cuh pays a fixed cost of several microseconds per launch (hand-over between kernels,
// barrier set-up, the wait for the first weight tile) some 160 times per token.  Here one block per SM stays resident for the
// whole token and walks a table of operations (embedding row, q/k/v, attention, output projection, gate/up, down, ...,
// classifier, next-token choice) that the host built once:
//   * the producer warp never stops: weights are constants, so it streams the tiles of operation k+1 into the shared-memory
//     ring while the consumer warps are still finishing operation k or waiting for the other SMs;
//   * an operation that needs the complete result of the one before it waits on that operation's arrival counter (every
//     block adds one to an operation's counter when it has finished its part; the wait is `count == blocks`), which replaces
//     the kernel boundary.  A block arrives for its operations in order, so the counter of the operation just before
//     covers everything earlier;
//   * the consumer warps build the activation planes, multiply (the same int8 tensor-core tile functions as the chain), and
//     hand their partial sums to the finisher warp, which runs the same epilogues as the chain;
//   * a matrix whose rows are longer than the activation planes kept in shared memory and whose epilogue is a plain
//     accumulation into the residual stream (the down projection) is cut along its input into several operations that need
//     no wait between them: each adds its part to the rows its block owns.
// Attention runs on the 16 consumer warps of a block (one (head group, split) work item at a time), the partial results
// of the splits are merged by the block that finishes last for a head group, as in attention.cuh.
//
// Every wait is bounded; a wait that runs out sets the status word and a block-wide flag, after which all warps of the block
// leave their loops; other blocks see the status word in their own waits.
#pragma once
#include <cstddef>

#include "attention.cuh"
#include "fused_matvec.cuh"
#include "sampling.cuh"

namespace l2b {

enum : int { TK_EMBED = 0, TK_MATVEC = 1, TK_ATTN = 2, TK_FINAL = 3 };

constexpr int TK_CONSUMERS = 16;  // consumer warps per block, in two groups of 8 that alternate over a block's tiles
constexpr int TK_GROUPS = 2;
constexpr int TK_THREADS = (TK_CONSUMERS + 2) * 32;

struct alignas(16) TkOp {
    int kind;        // TK_*
    int wait;        // 1: needs everything before it, from every block (device-wide wait); 0: only what this block did itself
    int pad[2];
    MvParams mv;     // TK_MATVEC
    AttnParams at;   // TK_ATTN
};

struct TkEmbed {
    int type;
    const uint8_t* table;
    const __half* d6;
    int n;       // dim
    int vocab;
    float* x;    // residual stream
};

// Shared-memory carve-up, decided on the host.
struct TkSmem {
    int off_bar;     // full[8] empty[8] red_full[8] red_empty[8]
    int off_misc;    // block-wide flags and small exchange arrays
    int off_ops;     // 5 copies of a TkOp: producer (two, alternating), consumers (two, alternating), finisher
    int off_red;     // partial sums between consumer warps and the finisher warp
    int off_region;  // dpl | xs16 | activation planes; attention and next-token scratch alias it
    int off_ring;
    int region_bytes, slot_bytes, nslots, plane_stride, planes_cap, total;
};

struct TkParams {
    const TkOp* ops;
    int n_ops;
    unsigned* sync;            // arrival counters, one per operation: zero at launch, zeroed again by block 0 at the end
    unsigned long long* trace; // measurement builds: time stamps per operation (block 0), or null
    Control* ctl;
    int* status;
    unsigned timeout_ms;       // bound on a device-wide wait
    TkEmbed embed;
    FinalizeParams fin;
    TkSmem sm;
};

constexpr int TK_MAX_OPS = 1024;
struct TkMisc {
    int dead;        // a bounded wait ran out somewhere in this block
    int stop;        // the consumer warps' common decision to leave (a snapshot of `dead` taken by one thread)
    int s_last;      // attention: this block merges the splits of its head group
    int s_choice;    // next-token choice
    float ssq[32];   // sums of squares of the rmsnorm prologue, one per consumer warp
    uint8_t kinds[TK_MAX_OPS];  // kind | wait << 4 of every operation, read once at the start
};

__host__ __device__ inline int tk_op_bytes() { return (int)((sizeof(TkOp) + 15) & ~(size_t)15); }

__host__ inline TkSmem tk_smem_layout(int planes, int planes_cap, int attn_scratch, int slot_bytes, int max_total) {
    TkSmem s;
    int o = 0;
    s.off_bar = o;
    o += (2 * MV_MAX_SLOTS + 2 * MV_RED_BUFS) * 8;
    s.off_misc = o;
    o += (int)((sizeof(TkMisc) + 15) & ~(size_t)15);
    s.off_ops = o;
    o += 5 * tk_op_bytes();
    o = (o + 127) & ~127;
    s.off_red = o;
    o += MV_RED_BUFS * MV_MAX_CONSUMERS * 16 * 4;
    s.off_region = o;
    s.planes_cap = planes_cap;
    s.plane_stride = planes_cap;
    while ((s.plane_stride & 127) != 32) s.plane_stride += 16;
    const int nb = planes_cap / QK_K;
    int region = nb * 8 * 4 + nb * 16 * 4;
    region = (region + 127) & ~127;
    region += planes * s.plane_stride;
    const int fin_scratch = 32 * 4 + 32 * 4 + TK_CONSUMERS * 32 * 8 + 64;
    region = region > attn_scratch ? region : attn_scratch;
    region = region > fin_scratch ? region : fin_scratch;
    s.region_bytes = (region + 127) & ~127;
    o += s.region_bytes;
    s.off_ring = o;
    s.slot_bytes = slot_bytes;
    int ns = slot_bytes > 0 ? (max_total - o) / slot_bytes : 0;
    if (ns > MV_MAX_SLOTS) ns = MV_MAX_SLOTS;
    ns -= ns % TK_GROUPS;
    s.nslots = ns;
    s.total = o + ns * slot_bytes;
    return s;
}

// ---- device-wide arrival counter ---------------------------------------------------------------
__device__ __forceinline__ void tk_arrive(unsigned* ctr) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(ctr), "r"(1u) : "memory");
}
__device__ __forceinline__ unsigned tk_load_acquire(const unsigned* ctr) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
    return v;
}
// One thread polls.  Gives up when the count does not arrive within limit_ns, or when this block or any other has reported a
// failure.
__device__ __forceinline__ bool tk_wait_count(const unsigned* ctr, unsigned target, const int* status, volatile int* dead,
                                              unsigned long long limit_ns) {
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (tk_load_acquire(ctr) >= target) return true;
        if ((i & 63u) == 63u) {
            if (*dead || __ldcg(status) != DEV_OK) return false;
            const unsigned long long t = global_ns();
            if (t0 == 0) t0 = t;
            else if (t - t0 > limit_ns) return false;
        }
    }
}
// mbarrier wait that also gives up when the block has been declared dead
__device__ __forceinline__ bool tk_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* dead) {
    for (uint32_t i = 0; i < MBAR_MAX_POLLS; ++i) {
        if (mbar_test_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(32);
        if ((i & 255u) == 255u && *dead) return false;
    }
    return false;
}

// Copy one operation descriptor from the table in global memory into shared memory with the threads [0, nthreads) of a role.
__device__ __forceinline__ void tk_load_op(TkOp* dst, const TkOp* src, int tid, int nthreads) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int i = tid; i < tk_op_bytes() / 16; i += nthreads) d4[i] = __ldg(s4 + i);
}

// ---- attention on the consumer warps of one block ------------------------------------------------
// One (head group, split) work item: the arithmetic of attention_split_body with TK_CONSUMERS warps walking the item's
// positions.  The warps are merged head by head through two alternating scratch buffers in shared memory.
template <int GQ>
__device__ __noinline__ void tk_attention_item(const AttnParams& p, int item, int npos, int warp, int lane, uint8_t* scratch, TkMisc* misc) {
    constexpr int W = TK_CONSUMERS;
    const int hg = item / p.nsplit, sp = item % p.nsplit;
    const int kvh = (hg * GQ) / (p.n_heads / p.n_kv);
    const int mc = p.min_chunk > 0 ? p.min_chunk : ATTN_MIN_CHUNK;
    const int active = min(p.nsplit, (npos + mc - 1) / mc);
    if (sp >= active) return;  // uniform over the block
    const int chunk = (npos + active - 1) / active;
    const int t0 = sp * chunk, t1 = min(npos, t0 + chunk);
    const int hs = p.hs;
    const bool lane_active = 4 * lane < hs;
    const float div = sqrtf((float)hs);
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    int* const ticket_p = p.tickets + hg;

    float4 qv[GQ], acc[GQ];
    float m[GQ], l[GQ];
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
        const int h = hg * GQ + g;
        qv[g] = lane_active ? __ldcg(reinterpret_cast<const float4*>(p.q + (size_t)h * hs) + lane) : zero4;
        acc[g] = zero4;
        m[g] = -INFINITY;
        l[g] = 0.f;
    }
    const float* kbase = p.kc + (size_t)kvh * p.seq_len * hs;
    const float* vbase = p.vc + (size_t)kvh * p.seq_len * hs;
    for (int tb = t0 + warp * ATTN_UNROLL; tb < t1; tb += W * ATTN_UNROLL) {
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
                    s = s / div;  // att ./= sqrt(Float32(head_size))
                    const float mn = fmaxf(m[g], s);
                    const float corr = expf(m[g] - mn);
                    const float pr = expf(s - mn);
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
    // merge the warps, one query head per round; round g uses buffer g & 1, and the warp that merges round g has finished
    // before anyone passes the barrier of round g + 1, so the buffer is free again in round g + 2
    constexpr int BUF_BYTES = W * 8 + W * 32 * 16;
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
        uint8_t* buf = scratch + (g & 1) * BUF_BYTES;
        float* sm = reinterpret_cast<float*>(buf);
        float* sl = sm + W;
        float4* sacc = reinterpret_cast<float4*>(buf + W * 8);
        if (lane == 0) {
            sm[warp] = m[g];
            sl[warp] = l[g];
        }
        sacc[warp * 32 + lane] = acc[g];
        consumer_sync(W * 32);
        if (warp == (g % W)) {
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < W; ++w) M = fmaxf(M, sm[w]);
            float Ls = 0.f;
            float4 a = zero4;
#pragma unroll
            for (int w = 0; w < W; ++w) {
                const float wgt = (sm[w] == -INFINITY) ? 0.f : expf(sm[w] - M);
                Ls = fmaf(sl[w], wgt, Ls);
                const float4 b = sacc[w * 32 + lane];
                a.x = fmaf(b.x, wgt, a.x);
                a.y = fmaf(b.y, wgt, a.y);
                a.z = fmaf(b.z, wgt, a.z);
                a.w = fmaf(b.w, wgt, a.w);
            }
            const int h = hg * GQ + g;
            if (active == 1) {
                if (lane_active) {
                    a.x /= Ls; a.y /= Ls; a.z /= Ls; a.w /= Ls;
                    reinterpret_cast<float4*>(p.out + (size_t)h * hs)[lane] = a;
                }
            } else {
                if (lane == 0) {
                    p.part_m[(size_t)h * p.nsplit + sp] = M;
                    p.part_l[(size_t)h * p.nsplit + sp] = Ls;
                }
                if (lane_active) reinterpret_cast<float4*>(p.part_acc + ((size_t)h * p.nsplit + sp) * hs)[lane] = a;
            }
        }
    }
    if (active == 1) return;
    // the block that finishes last for this head group merges the splits
    __threadfence();
    consumer_sync(W * 32);
    if (threadIdx.x == 0) {
        const int ticket = atomicAdd(ticket_p, 1);
        misc->s_last = (ticket == active - 1);
        if (misc->s_last) *ticket_p = 0;
    }
    consumer_sync(W * 32);
    const bool last = misc->s_last != 0;
    consumer_sync(W * 32);  // s_last may be rewritten by the next item
    if (!last) return;
    __threadfence();
    for (int g = warp; g < GQ; g += W) {
        const int h = hg * GQ + g;
        const float* pm = p.part_m + (size_t)h * p.nsplit;
        const float* pl = p.part_l + (size_t)h * p.nsplit;
        const float ms = lane < active ? __ldcg(pm + lane) : -INFINITY;
        const float ls = lane < active ? __ldcg(pl + lane) : 0.f;
        const float M = warp_max(ms);
        const float wgt = (ms == -INFINITY) ? 0.f : expf(ms - M);
        const float Ls = warp_sum(ls * wgt);
        float4 a = zero4;
        for (int s0 = 0; s0 < active; s0 += 4) {
            float4 b[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                b[u] = zero4;
                if (lane_active && s0 + u < active) b[u] = __ldcg(reinterpret_cast<const float4*>(p.part_acc + ((size_t)h * p.nsplit + s0 + u) * hs) + lane);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
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
            a.x /= Ls; a.y /= Ls; a.z /= Ls; a.w /= Ls;
            reinterpret_cast<float4*>(p.out + (size_t)h * hs)[lane] = a;
        }
    }
}

// x = dequantize!(x, token_embedding_table[:, token]) (src/inference.jl:236) by the consumer warps of block 0.
__device__ __noinline__ void tk_embed(const TkEmbed& e, int tok, int ctid) {
    const bool valid = tok >= 0 && tok < e.vocab;
    const int nbr = e.n / QK_K;
    for (int i = ctid; i < e.n; i += TK_CONSUMERS * 32) {
        float v = 0.f;
        if (valid) {
            const int b = i >> 8, k = i & 255;
            const uint8_t* blk = e.table + ((size_t)tok * nbr + b) * dev_block_bytes(e.type);
            if (e.type == T_Q4_K) v = dequant_q45<false>(blk, k);
            else if (e.type == T_Q5_K) v = dequant_q45<true>(blk, k);
            else v = dequant_q6(blk, __half2float(e.d6[(size_t)tok * nbr + b]), k);
        }
        e.x[i] = v;
    }
    __threadfence();
}

// Next token (src/inference.jl:354-368) and advance, by the consumer warps of block 0.
__device__ __noinline__ void tk_final(const FinalizeParams& f, int ctid, uint8_t* region, int* s_choice) {
    float* s_val = reinterpret_cast<float*>(region);
    int* s_idx = reinterpret_cast<int*>(region + 128);
    double* s_sum = reinterpret_cast<double*>(region + 256);
    finalize_token_body<TK_CONSUMERS * 32>(f, ctid, s_val, s_idx, s_sum, s_choice, [] { consumer_sync(TK_CONSUMERS * 32); });
}

__device__ __noinline__ void tk_attention_op(const AttnParams& a, int npos, int warp, int lane, uint8_t* region, TkMisc* misc) {
    const int gq = a.n_heads / a.n_kv;
    const int GQ = (gq == 8 || gq == 4 || gq == 2) ? gq : 1;
    const int n_items = (a.n_heads / GQ) * a.nsplit;
    for (int item = (int)blockIdx.x; item < n_items; item += (int)gridDim.x) {
        if (GQ == 8) tk_attention_item<8>(a, item, npos, warp, lane, region, misc);
        else if (GQ == 4) tk_attention_item<4>(a, item, npos, warp, lane, region, misc);
        else if (GQ == 2) tk_attention_item<2>(a, item, npos, warp, lane, region, misc);
        else tk_attention_item<1>(a, item, npos, warp, lane, region, misc);
        consumer_sync(TK_CONSUMERS * 32);  // the scratch buffers are free again
    }
    __threadfence();
}

__host__ __device__ inline int tk_attention_scratch_bytes() { return 2 * (TK_CONSUMERS * 8 + TK_CONSUMERS * 32 * 16); }

// ---- the kernel --------------------------------------------------------------------------------------
template <int P>
__global__ void __launch_bounds__(TK_THREADS, 1) token_kernel(const __grid_constant__ TkParams tp) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int W = TK_CONSUMERS, CG = TK_GROUPS, WG = W / CG;
    const TkSmem& S = tp.sm;
    const int NS = S.nslots, NSG = NS / CG;

    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S.off_bar);
    uint64_t* empty = full + MV_MAX_SLOTS;
    uint64_t* red_full = empty + MV_MAX_SLOTS;
    uint64_t* red_empty = red_full + MV_RED_BUFS;
    TkMisc* misc = reinterpret_cast<TkMisc*>(smem + S.off_misc);
    volatile int* dead_flag = &misc->dead;
    uint8_t* ring = smem + S.off_ring;
    float* red = reinterpret_cast<float*>(smem + S.off_red);
    auto opbuf = [&](int i) { return reinterpret_cast<TkOp*>(smem + S.off_ops + i * tk_op_bytes()); };
    const unsigned nblocks = gridDim.x;
#ifdef L2B_MEASURE
#define TK_STAMP(op_index, k)                                                                                        \
    do {                                                                                                             \
        if (tp.trace && blockIdx.x == 0) tp.trace[(size_t)(op_index) * 4 + (k)] = global_ns();                       \
    } while (0)
#else
#define TK_STAMP(op_index, k) do { } while (0)
#endif

    if (threadIdx.x < NS) {
        mbar_init(full + threadIdx.x, 1);
        mbar_init(empty + threadIdx.x, WG);
    }
    if (threadIdx.x >= 32 && threadIdx.x < 32 + MV_RED_BUFS) {
        mbar_init(red_full + (threadIdx.x - 32), WG);
        mbar_init(red_empty + (threadIdx.x - 32), 1);
    }
    if (threadIdx.x == 64) {
        misc->dead = 0;
        misc->stop = 0;
        misc->s_last = 0;
    }
    for (int i = threadIdx.x; i < tp.n_ops; i += blockDim.x) misc->kinds[i] = (uint8_t)(__ldg(&tp.ops[i].kind) | (__ldg(&tp.ops[i].wait) << 4));
    if (threadIdx.x < 32 + MV_RED_BUFS) {
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();
    const int pos = __ldcg(&tp.ctl->pos);

    // ================================ producer warp =============================================
    // Lane c brings copy group c of every stage.  This warp runs serial address arithmetic on a busy SM (some 20 cycles per
    // instruction), so the source of the NEXT tile is worked out right after a tile's copies have been issued, in the shadow
    // of the wait for a free slot, and the descriptor of the next operation is fetched while this one's tiles are streamed.
    if (warp == W) {
        if (lane >= 16) return;
        const uint64_t policy = policy_evict_first();
        const int c = lane;
        int slot_g[2] = {0, NSG}, ph_g[2] = {0, 0};
        unsigned gt = 0;  // tiles of this block so far, over all operations
        bool dead = false;
        struct TileSrc {
            const uint8_t* src;  // first byte of this lane's copy (stage 0)
            uint32_t bytes0;     // bytes of this lane's copy in a full-width stage (0: nothing to copy)
            uint32_t tx0;        // bytes of the whole stage (all lanes) in a full-width stage
            int bb, nrows, nvalid, gs, row;
            size_t ps;           // bytes of one full column panel of the matrix
        };
        constexpr int OPV = (sizeof(TkOp) + 16 * 16 - 1) / (16 * 16);  // uint4 per lane that hold one descriptor
        auto next_matvec = [&](int from) {
            while (from < tp.n_ops && (misc->kinds[from] & 15) != TK_MATVEC) ++from;
            return from;
        };
        int oi = next_matvec(0), buf = 0;
        // descriptor buffers of this warp: 0 and 1 (the finisher keeps its own copy in registers-fed buffer 1 below)
        if (oi < tp.n_ops) tk_load_op(opbuf(0), tp.ops + oi, lane, 16);
        __syncwarp(0x0000ffffu);
        while (oi < tp.n_ops && !dead) {
            const TkOp* op = opbuf(buf);
            const MvParams& p = op->mv;
            const int nb = p.n_in / QK_K, nit = p.nit;
            const int my_units = p.units_lo + ((int)blockIdx.x < p.units_rem ? 1 : 0);
            const int oi_next = next_matvec(oi + 1);
            uint4 pre[OPV];  // the next operation's descriptor, on its way while this one's tiles are issued
            if (oi_next < tp.n_ops) {
#pragma unroll
                for (int k = 0; k < OPV; ++k) {
                    const int idx = lane + 16 * k;
                    pre[k] = idx < tk_op_bytes() / 16 ? __ldg(reinterpret_cast<const uint4*>(tp.ops + oi_next) + idx) : make_uint4(0u, 0u, 0u, 0u);
                }
            }
            auto tile_src = [&](int j) {
                TileSrc ts;
                ts.src = nullptr;
                ts.bytes0 = ts.tx0 = 0;
                ts.bb = ts.nrows = ts.nvalid = ts.gs = ts.row = 0;
                ts.ps = 0;
                if (j >= my_units) return ts;
                const UnitInfo u = find_unit<true>(p, (int)blockIdx.x + j * (int)gridDim.x);
                const MvSegment& sg = p.seg[u.seg];
                ts.bb = dev_block_bytes(sg.type);
                ts.gs = sg.gs;
                const int pairs_left = sg.npairs - u.pair0;  // >= 1
                ts.nvalid = 2 * min(MV_TILE_PAIRS, pairs_left);
                if (c < sg.ngroups) {
                    if (sg.rpg == 4) {  // adjacent rows 16*tile + 4c ..
                        ts.nrows = max(0, min(4, 2 * pairs_left - 4 * c));
                        ts.row = 2 * u.pair0 + 4 * c;
                        ts.src = sg.w + (size_t)ts.row * sg.rowb;
                    } else {
                        const int half = c >> 2;      // A or B rows
                        const int jp = 2 * (c & 3);   // pair of the copy's first row
                        ts.nrows = max(0, min(sg.rpg, pairs_left - jp));
                        if (ts.nrows > 0) {
                            int rowA, rowB;
                            pair_rows(p, sg, u.pair0 + jp, rowA, rowB);
                            const uint8_t* base = (sg.pair_mode == PAIR_DUAL && half) ? sg.w2 : sg.w;
                            ts.row = half ? rowB : rowA;
                            ts.src = base + (size_t)ts.row * sg.rowb;
                        }
                    }
                }
                ts.bytes0 = (uint32_t)(ts.nrows * sg.rowb);
                ts.tx0 = (uint32_t)(ts.nvalid * sg.rowb);
                ts.ps = (size_t)(sg.pair_mode == PAIR_DUAL ? sg.npairs : 2 * sg.npairs) * sg.rowb;
                return ts;
            };
            TileSrc ts = tile_src(0);
            // Fast path for the common case (one segment, adjacent or dual rows, full tiles): the next tile's source is the
            // current one plus a constant.
            const bool linear = (p.nseg == 1) && (p.seg[0].pair_mode != PAIR_NEOX);
            const int row_step = (int)gridDim.x * (p.seg[0].pair_mode == PAIR_ADJACENT ? 16 : 8);
            const size_t tile_step = linear ? (size_t)row_step * p.seg[0].rowb : 0;
            const int full_tiles = linear ? p.seg[0].npairs / MV_TILE_PAIRS : 0;
            for (int j = 0; j < my_units && !dead; ++j, ++gt) {
                const int grp = (int)(gt & 1u);
                int slot_i = grp ? slot_g[1] : slot_g[0], ph = grp ? ph_g[1] : ph_g[0];
                for (int it = 0; it < nit; ++it) {
                    if (ph > 0) {
                        int ok = 1;
                        if (c == 0) ok = tk_mbar_wait(empty + slot_i, (uint32_t)((ph & 1) ^ 1), dead_flag) ? 1 : 0;
                        ok = __shfl_sync(0x0000ffffu, ok, 0);
                        if (!ok) {
                            dead = true;
                            break;
                        }
                    }
                    uint32_t bytes = ts.bytes0, tx = ts.tx0;
                    const uint8_t* src = ts.src;
                    if (nit > 1) {  // stage `it` lives in column panel `it`, whose rows are nblk blocks wide
                        const int nblk = min(p.kb, nb - it * p.kb);
                        bytes = (uint32_t)(ts.nrows * nblk * ts.bb);
                        tx = (uint32_t)(ts.nvalid * nblk * ts.bb);
                        src += (size_t)it * ts.ps - (size_t)ts.row * ((p.kb - nblk) * ts.bb);
                    }
                    if (c == 0) mbar_arrive_expect_tx(full + slot_i, tx);
                    __syncwarp(0x0000ffffu);
                    if (bytes) bulk_g2s(ring + (size_t)slot_i * S.slot_bytes + (size_t)c * ts.gs, src, bytes, full + slot_i, policy);
                    if (++slot_i == (grp + 1) * NSG) {
                        slot_i = grp * NSG;
                        ++ph;
                    }
                }
                if (grp) {
                    slot_g[1] = slot_i;
                    ph_g[1] = ph;
                } else {
                    slot_g[0] = slot_i;
                    ph_g[0] = ph;
                }
                // source of the next tile (in the shadow of the wait for its slot)
                const int next_tile = (int)blockIdx.x + (j + 1) * (int)gridDim.x;
                if (linear && next_tile < full_tiles) {
                    ts.src += tile_step;
                    ts.row += row_step;
                } else {
                    ts = tile_src(j + 1);
                }
            }
            // the next operation's descriptor goes to the other buffer
            if (oi_next < tp.n_ops) {
                uint4* d4 = reinterpret_cast<uint4*>(opbuf(buf ^ 1));
#pragma unroll
                for (int k = 0; k < OPV; ++k) {
                    const int idx = lane + 16 * k;
                    if (idx < tk_op_bytes() / 16) d4[idx] = pre[k];
                }
            }
            __syncwarp(0x0000ffffu);
            buf ^= 1;
            oi = oi_next;
        }
        if (dead) {
            if (c == 0) {
                atomicExch(tp.status, DEV_ERR_TMA_TIMEOUT);
                misc->dead = 1;
            }
            for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // copies in flight land within microseconds
        }
        return;
    }

    // ================================ finisher warp ==============================================
    if (warp == W + 1) {
        TkOp* op = opbuf(4);
        const int fq = lane >> 4, fidx = lane & 15;
        unsigned gt = 0;
        bool dead = false;
        for (int oi = 0; oi < tp.n_ops && !dead; ++oi) {
            if ((misc->kinds[oi] & 15) != TK_MATVEC) continue;
            __syncwarp();
            tk_load_op(op, tp.ops + oi, lane, 32);
            __syncwarp();
            const MvParams& p = op->mv;
            const int my_units = p.units_lo + ((int)blockIdx.x < p.units_rem ? 1 : 0);
            ArgBest best;
            best.v = -INFINITY;
            best.i = 0x7fffffff;
            int unit = (int)blockIdx.x;
            for (int j = 0; j < my_units && !dead; ++j, ++gt, unit += (int)gridDim.x) {
                const UnitInfo u = find_unit<true>(p, unit);
                const MvSegment& sg = p.seg[u.seg];
                const int t = u.pair0 + lane;
                const bool mine = lane < MV_TILE_PAIRS && t < sg.npairs;
                EpiPre pre0;
                if (mine) pre0 = epilogue_preload(p, sg, t, pos);
                const int rb = (int)(gt & (MV_RED_BUFS - 1));
                const uint32_t par = (gt / MV_RED_BUFS) & 1u;
                if (!tk_mbar_wait(red_full + rb, par, dead_flag)) {
                    dead = true;
                    break;
                }
                const float* rbuf = red + rb * (MV_MAX_CONSUMERS * 16);
                float v = 0.f;
                for (int w = fq; w < WG; w += 2) v += rbuf[w * 16 + fidx];
                __syncwarp();
                if (lane == 0) mbar_arrive(red_empty + rb);
                v += __shfl_xor_sync(0xffffffffu, v, 16);
                const float vB = __shfl_sync(0xffffffffu, v, (lane & 7) + 8);
                if (mine) epilogue_pair<false, true>(p, sg, t, v, vB, pos, best, 0, &pre0);
            }
            if (dead) break;
            if (p.amax_val) {  // EPI_LOGITS: first maximal index over this block's rows
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, best.v, o);
                    const int oi2 = __shfl_xor_sync(0xffffffffu, best.i, o);
                    arg_update(best, ov, oi2);
                }
                if (lane == 0) {
                    p.amax_val[blockIdx.x] = best.v;
                    p.amax_idx[blockIdx.x] = best.i;
                }
            }
            // this block's part of the operation is in memory: tell everyone
            __threadfence();
            __syncwarp();
            if (lane == 0) {
                tk_arrive(tp.sync + oi);
                TK_STAMP(oi, 3);
            }
        }
        if (dead && lane == 0) {
            atomicExch(tp.status, DEV_ERR_TMA_TIMEOUT);
            misc->dead = 1;
        }
        return;
    }

    // ================================ consumer warps ============================================
    const int ctid = threadIdx.x;  // 0 .. W*32-1
    uint8_t* region = smem + S.off_region;
    const int nbcap = S.planes_cap / QK_K;
    float* dpl = reinterpret_cast<float*>(region);
    float* xs16 = dpl + nbcap * 8;
    uint8_t* act = region + (((nbcap * 8 + nbcap * 16) * 4 + 127) & ~127);
    MvSmem L;  // what build_activation needs to know about the carve-up
    L.plane_stride = S.plane_stride;
    L.off_red = S.off_misc + (int)offsetof(TkMisc, ssq);
    L.off_xf = 0;

    TileCtx cx;
    cx.act = act;
    cx.dpl = dpl;
    cx.xs16 = xs16;
    tile_ctx_columns<1, P>(cx, act, S.plane_stride, lane);
    const int pj = ((cx.g & 3) << 1) | (cx.g >> 2);
    const int grp = warp / WG, wl = warp - grp * WG;
    int slot_i = grp * NSG;
    uint32_t full_par = 0;
    unsigned gt = 0;
    bool dead = false;
    const unsigned long long limit_ns = (unsigned long long)tp.timeout_ms * 1000000ull;

    tk_load_op(opbuf(2), tp.ops, ctid, W * 32);
    for (int oi = 0; oi < tp.n_ops; ++oi) {
        // A warp whose own wait ran out (`dead`) keeps walking the loops without waiting or computing, so that it still
        // joins every barrier of the consumer warps; all of them leave together at the next operation, on `stop`.
        TkOp* op = opbuf(2 + (oi & 1));
        const int kind = misc->kinds[oi] & 15;
        if (kind == TK_FINAL && blockIdx.x != 0) break;  // the next token is chosen by block 0
        if (ctid == 0) {
            if ((misc->kinds[oi] >> 4) && !*dead_flag &&
                !tk_wait_count(tp.sync + oi - 1, nblocks, tp.status, dead_flag, limit_ns)) {
                atomicExch(tp.status, DEV_ERR_TMA_TIMEOUT);
                misc->dead = 1;
            }
            misc->stop = misc->dead;
            TK_STAMP(oi, 0);
        }
        consumer_sync(W * 32);  // also: every warp has finished the previous operation (planes, descriptor buffers are free)
        if (misc->stop) break;
        if (oi + 1 < tp.n_ops) tk_load_op(opbuf(2 + ((oi + 1) & 1)), tp.ops + oi + 1, ctid, W * 32);  // visible after the next barrier
        if (kind == TK_EMBED) {  // every block's first q/k/v prologue reads x, block 0 writes it
            if (blockIdx.x == 0) tk_embed(tp.embed, __ldcg(&tp.ctl->token), ctid);
            consumer_sync(W * 32);
            if (ctid == 0) tk_arrive(tp.sync + oi);
            continue;
        }
        if (kind == TK_ATTN) {
            tk_attention_op(op->at, pos + 1, warp, lane, region, misc);
            consumer_sync(W * 32);
            if (ctid == 0) {
                tk_arrive(tp.sync + oi);
                TK_STAMP(oi, 3);
            }
            continue;
        }
        if (kind == TK_FINAL) {  // block 0 only
            tk_final(tp.fin, ctid, region, &misc->s_choice);
            // every block has made its last arrival (this operation waited for all of them): counters back to zero
            for (int i = ctid; i < tp.n_ops; i += W * 32) tp.sync[i] = 0u;
            break;
        }
        // ---- TK_MATVEC ----
        const MvParams& p = op->mv;
        build_activation<true, P, false>(p, smem, L, warp, lane, W, p.x_in, act, dpl, xs16);
        if (ctid == 0) TK_STAMP(oi, 1);
        const int nb = p.n_in / QK_K, nit = p.nit;
        const int my_units = p.units_lo + ((int)blockIdx.x < p.units_rem ? 1 : 0);
        // tiles of this block alternate between the two groups of consumer warps by their running number
        int seg_i = -1, seg_end = 0, seg_first = 0;
        int bb = 0, offA = 0, offB = 0;
        const int j0 = (int)((gt ^ (unsigned)grp) & 1u);  // first tile of this operation that belongs to this warp's group
        for (int j = j0; j < my_units; j += CG) {
            const int unit = (int)blockIdx.x + j * (int)gridDim.x;
            if (seg_i < 0 || unit >= seg_end) {
                seg_i = find_unit<true>(p, unit).seg;
                seg_first = p.seg_start[seg_i];
                seg_end = p.seg_start[seg_i + 1];
                bb = dev_block_bytes(p.seg[seg_i].type);
                pair_offsets(p.seg[seg_i], p.seg[seg_i].rowb, pj, offA, offB);
            }
            const MvSegment& sg = p.seg[seg_i];
            const int pair0 = (unit - seg_first) * MV_TILE_PAIRS;
            const __half* d6A = nullptr;
            const __half* d6B = nullptr;
            if (sg.type == T_Q6_K) {
                const int t = min(pair0 + pj, sg.npairs - 1);
                int rowA, rowB;
                pair_rows(p, sg, t, rowA, rowB);
                const int nbrow = sg.d6_nb ? sg.d6_nb : nb;
                d6A = sg.d6 + (size_t)rowA * nbrow;
                d6B = ((sg.pair_mode == PAIR_DUAL) ? sg.d6_2 : sg.d6) + (size_t)rowB * nbrow;
            }
            float accA = 0.f, accB = 0.f;
            for (int it = 0; it < nit; ++it) {
                const int b0 = it * p.kb, nblk = min(p.kb, nb - b0);
                int oA = offA, oB = offB;
                if (nit > 1 && nblk < p.kb) pair_offsets(sg, nblk * bb, pj, oA, oB);
                float dA = 0.f, dB = 0.f;
                if (sg.type == T_Q6_K && wl < nblk) {
                    dA = __half2float(__ldg(d6A + b0 + wl));
                    dB = __half2float(__ldg(d6B + b0 + wl));
                }
                if (!dead && !tk_mbar_wait(full + slot_i, full_par, dead_flag)) dead = true;
                if (!dead) {
                    const uint8_t* slot = ring + (size_t)slot_i * S.slot_bytes;
                    for (int bl = wl; bl < nblk; bl += WG) {
                        const uint8_t* rA = slot + oA + bl * bb;
                        const uint8_t* rB = slot + oB + bl * bb;
                        if (sg.type == T_Q4_K) tile_q4k<1>(rA, rB, b0 + bl, cx, accA, accB);
                        else if (sg.type == T_Q5_K) tile_q5k<1>(rA, rB, b0 + bl, cx, accA, accB);
                        else {
                            if (bl != wl) {
                                dA = __half2float(__ldg(d6A + b0 + bl));
                                dB = __half2float(__ldg(d6B + b0 + bl));
                            }
                            tile_q6k<1>(rA, rB, dA, dB, b0 + bl, cx, accA, accB);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0 && !dead) mbar_arrive(empty + slot_i);
                if (++slot_i == (grp + 1) * NSG) {
                    slot_i = grp * NSG;
                    full_par ^= 1u;
                }
            }
            accA += __shfl_xor_sync(0xffffffffu, accA, 1);
            accB += __shfl_xor_sync(0xffffffffu, accB, 1);
            accA += __shfl_xor_sync(0xffffffffu, accA, 2);
            accB += __shfl_xor_sync(0xffffffffu, accB, 2);
            const unsigned T = gt + (unsigned)j;  // running number of this tile
            const int rb = (int)(T & (MV_RED_BUFS - 1));
            const unsigned use = T / MV_RED_BUFS;
            if (use > 0 && !dead && !tk_mbar_wait(red_empty + rb, (use - 1) & 1u, dead_flag)) dead = true;
            float* rbuf = red + rb * (MV_MAX_CONSUMERS * 16);
            if (cx.t == 0) {
                rbuf[wl * 16 + pj] = accA;
                rbuf[wl * 16 + 8 + pj] = accB;
            }
            __syncwarp();
            if (lane == 0 && !dead) mbar_arrive(red_full + rb);
        }
        gt += (unsigned)my_units;
        if (ctid == 0) TK_STAMP(oi, 2);
        if (dead && lane == 0) {
            atomicExch(tp.status, DEV_ERR_TMA_TIMEOUT);
            misc->dead = 1;
        }
    }
}

}  // namespace l2b
