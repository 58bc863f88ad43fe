// The fused matrix-vector kernel of the decode path: replaces matmul! (src/matmul.jl:3-23)
// together with the element-wise work around each call site in transformer!
// (src/inference.jl:236-312).
//
// One launch = prologue (build the activation vector in shared memory) + a stream of
// weight tiles + an epilogue per pair of output rows.
//
//   prologue  : raw copy | rmsnorm (inference.jl:102-110) of a vector in global memory; then, for
//               k-quant weights, on-device quantisation of the vector to 1..3 int8 planes
//               (block_q8_K layout, kquants.jl:38-42).  With rmsnorm the planes are built from
//               gain .* x while the sum of squares is still being collected; 1/rms scales the plane
//               scales afterwards.  A two-position launch builds the planes of both positions.
//   weights   : warp-specialised.  A tile is 16 output rows (8 row pairs) by up to 16 super-blocks (a
//               stage).  The lanes of one producer warp bring a stage into a ring of shared-memory slots
//               with a few large bulk asynchronous copies (TMA): 4 copies of 4 adjacent rows, or 8 copies
//               of 2 rows when the two rows of a pair are far apart (an SM issues only ~23 bulk copies
//               per microsecond, so 16 row-sized copies per tile would cap the stream below the HBM
//               rate).  Rows longer than a stage are stored as column panels, so every stage of theirs
//               looks like a short row.  The producer starts BEFORE the wait on the previous kernel
//               (programmatic dependent launch): weights are constants, so the ring is already full
//               when the activations arrive.  All consumer warps of a group work on the same slot, one or
//               two super-block columns each, with int8 tensor-core MMAs (kquants.cuh); their partial
//               sums go to a small ring of shared-memory buffers, where a dedicated finisher warp adds
//               them in a fixed order and runs the epilogue, so that no consumer warp ever waits for
//               another one.  The finisher fetches what the epilogue needs from global memory (residual
//               values, RoPE factors) before it waits for a tile's sums.
//   epilogue  : store | residual add (:284,:305) | SwiGLU (:295-299) | RoPE + KV-cache write
//               (:255-260) | logits store + running argmax (:312,:360) | push of a partial vector to the
//               other tensor-parallel ranks
//
// A kernel here lives for a few microseconds, so serial scalar work on the critical path matters as
// much as bandwidth: everything that can be computed on the host (tile counts, loop bounds, division
// magic) arrives in the parameter block.
#pragma once
#include "kquants.cuh"

namespace l2b {

enum : int { PRO_COPY = 0, PRO_RMSNORM = 1 };
enum : int { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2, EPI_ROPE_Q = 3, EPI_ROPE_K = 4, EPI_STORE_V = 5, EPI_LOGITS = 6, EPI_PUSH = 7 };
// Tensor parallelism (no counterpart in the reference): a row-split matrix (wo, w2) yields a PARTIAL output vector
// per GPU.  EPI_PUSH writes this GPU's partial vector into every GPU's exchange buffer with plain stores over
// NVLink, every value as 8 bytes {f32 bits, tag} with tag = the token's number + 1.  The next kernel's rmsnorm
// prologue reads those words until their tags are this token's (bounded by a time-out) and forms
// x_new = x + sum_r partial_r in rank order, so that all GPUs hold bit-identical residual streams.  No fence,
// arrival counter or separate wait is involved: a value is there when its tag is.
constexpr int MV_MAX_TP = 8;
// How the 8 row pairs (A, B) of a tile map to matrix rows.  Pair j of a tile occupies tile rows j and j+8.
//   ADJACENT: rows (2t, 2t+1)            -- plain outputs and interleaved RoPE pairs
//   NEOX    : rows (i, i + head_size/2)  -- NeoX RoPE pairs
//   DUAL    : row t of `w` and row t of `w2` -- gate and up projections feeding SwiGLU
enum : int { PAIR_ADJACENT = 0, PAIR_NEOX = 1, PAIR_DUAL = 2 };

constexpr int MV_MAX_SEG = 3;
constexpr int MV_MAX_CONSUMERS = 16;
constexpr int MV_MAX_SLOTS = 8;
constexpr int MV_TILE_PAIRS = 8;
constexpr int MV_TILE_BLOCKS = 16;  // super-blocks per row and stage
constexpr int MV_RED_BUFS = 8;      // partial-sum buffers between the consumer warps and the finisher warp
constexpr int MV_GAIN_BLOCKS = 2;   // of those, the blocks whose rmsnorm gains are loaded together with x
constexpr int MV_REG_BLOCKS = 4;    // 256-value blocks a warp keeps in registers across the rmsnorm reduction

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
    // slot geometry, filled by the host (mv_fill_geometry)
    int ngroups;         // bulk copies per stage
    int rpg;             // rows per copy
    int gs;              // bytes between copy groups inside a slot (= 32 mod 128)
    int rowb;            // bytes of one row in a full-width stage
    int out2;            // two-position launches: element offset of the second position's output vector (0: same base, e.g. caches)
    int d6_nb;           // q6_K: super-block scales per row of d6 / d6_2 when that differs from n_in / 256 (a launch over a column
                         // range of the matrix; token_kernel.cuh only); 0 = n_in / 256
};

// What a tensor-parallel launch needs to know about the other GPUs.
struct MvTp {
    int tp_size;
    unsigned tp_timeout_ms;               // bound on the wait for the other GPUs
    float* push_dst[8];                   // [r]: where this GPU's partial vector lives in GPU r's exchange buffer ({value, tag} pairs)
    const float* part_src;                // prologue: partial vectors [tp_size][n_in] of {value, tag} pairs in this GPU's exchange buffer, or null
    const unsigned* tp_epoch;             // tokens completed so far (device word, advanced once per token)
    float* x_out;                         // prologue: block 0 writes x_new here (the residual stream is double-buffered)
};

// Offsets of the regions of a block's shared memory (mv_smem_layout).
struct MvSmem {
    int off_bar, off_ss, off_red, off_dpl, off_xs, off_act, off_xf, off_ring, total;
    int plane_stride, slot_bytes;
};

struct MvParams {
    MvSegment seg[MV_MAX_SEG];
    int nseg;
    int n_in;        // input length
    int planes;      // int8 activation planes (k-quant launches)
    // schedule, precomputed on the host (plan_matvec)
    int nslots;                      // ring slots
    int row_stride;                  // bytes between tile rows inside a slot (a multiple of 16, = 32 mod 128)
    int nit;                         // stages per tile = ceil(blocks per row / kb)
    int kb;                          // super-blocks per row and stage (16, or 8 where 16-wide slots would leave fewer than 4 of them)
    int seg_start[MV_MAX_SEG + 1];   // first unit of each segment; [nseg] = total; a unit is a tile (k-quant) or a pair (f32)
    int units_lo, units_rem;         // block b runs units_lo + (b < units_rem) units: b, b + grid, ...
    int consumers;                   // consumer warps per block (k-quant: blockDim/32 - 2; f32: blockDim/32)
    int cgroups;                     // consumer groups (1 or 2): tile j is worked on by group j % cgroups, so that one
                                     // group's barrier and reduction latencies hide behind the other group's arithmetic
    int turns;                       // prologue turns per warp = ceil(n_in / (256 * consumers))
    unsigned neox_magic;             // ceil(2^32 / (head_size/2)) for PAIR_NEOX row arithmetic
    // prologue
    int pro;
    const float* x_in;      // input vector
    const float* gain;      // rmsnorm gain (PRO_RMSNORM)
    const int* pos;         // device scalar: current position (0-based)
    // epilogue extras
    const float* resid;     // EPI_RESIDUAL: vector added to the result (may alias out)
    const float* rope_cs;   // [seq_len][head_size/2][2] (cos, sin)
    int seq_len;
    float* amax_val;        // EPI_LOGITS: per-block best value   [gridDim.x]
    int* amax_idx;          // EPI_LOGITS: per-block best index   [gridDim.x]
    // tensor parallelism: descriptor in device memory (null on one GPU).  Kept out of the parameter block on purpose:
    // every byte of kernel parameters is paid for at each of the ~160 launches of a token.
    const MvTp* tp;
    int tp_push;            // this launch ends in EPI_PUSH
    int* status;            // device status word
    int debug;              // measurement aid: bit 0 = consumers skip the arithmetic, bit 1 = the producer skips the copies (results are wrong)
    unsigned long long* trace;  // optional timeline: 16 globaltimer stamps per block (debugging aid), or null
};

// ---- shared-memory carve-up (host and device agree through this helper) ------------------

__host__ __device__ inline int mv_row_stride(int blocks_per_stage, int block_bytes) {
    int rs = blocks_per_stage * block_bytes;  // a multiple of 16
    while ((rs & 127) != 32) rs += 16;        // rows g = 0..3 of a 64-bit fragment load then fall in distinct banks
    return rs;
}

// nbatch = activation vectors per launch (1, or 2 for the two-position prompt passes): planes, sums and reduction buffers double.
__host__ __device__ inline MvSmem mv_smem_layout(int n_in, int planes, bool kquant, int nslots, int row_stride, int nbatch = 1) {
    MvSmem s;
    const int nb = n_in / QK_K;
    int o = 0;
    s.off_bar = o;  // full[MV_MAX_SLOTS], empty[MV_MAX_SLOTS], red_full[MV_RED_BUFS], red_empty[MV_RED_BUFS]
    o += (2 * MV_MAX_SLOTS + 2 * MV_RED_BUFS + 1) * 8;  // ... and ss_ready (below)
    s.off_ss = o;   // [MV_MAX_CONSUMERS] f32: the consumer warps' sums of squares, for the finisher warp (deferred rmsnorm scale)
    o += MV_MAX_CONSUMERS * 4;
    o = (o + 15) & ~15;
    s.off_red = o;  // [MV_RED_BUFS][MV_MAX_CONSUMERS][16] f32 tile partials (also the block-sum scratch of the prologue)
    o += MV_RED_BUFS * MV_MAX_CONSUMERS * 16 * 4 * nbatch;
    s.off_dpl = o;
    if (kquant) o += nb * 8 * 4;
    s.off_xs = o;
    if (kquant) o += nb * 16 * 4 * nbatch;
    o = (o + 127) & ~127;
    s.plane_stride = n_in;
    while ((s.plane_stride & 127) != 32) s.plane_stride += 16;  // planes 0..2 of a fragment load fall in distinct banks
    s.off_act = o;
    if (kquant) o += planes * nbatch * s.plane_stride;
    o = (o + 15) & ~15;
    s.off_xf = o;
    if (!kquant) o += n_in * 4;
    o = (o + 127) & ~127;
    s.off_ring = o;
    s.slot_bytes = 16 * row_stride;
    if (kquant) o += nslots * s.slot_bytes;
    s.total = o;
    return s;
}

// ---- prologue pieces ---------------------------------------------------------------------

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define MV_TRACE(i)                                                                      \
    do {                                                                                 \
        if (DBG && p.trace && threadIdx.x == 0) p.trace[blockIdx.x * 16 + (i)] = global_ns();  \
    } while (0)

// Barrier over the first `nthreads` threads of the block (the consumer warps); the producer warp never joins it.
__device__ __forceinline__ void consumer_sync(int nthreads) { asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory"); }

__device__ __forceinline__ float block_sum(float v, float* red, int warp, int lane, int nwarps) {
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    consumer_sync(nwarps * 32);
    float t = 0.f;
    for (int i = 0; i < nwarps; ++i) t += red[i];  // same order in every thread
    consumer_sync(nwarps * 32);                    // `red` is reused by the tile reduction
    return t;
}

// Quantise the 8 values a lane holds (values 8*lane .. 8*lane+7 of block b) into P planes:
//   plane 0: q = round(x * 127/amax), d0 = amax/127 (this is block_q8_K, src/kquants.jl:38-42);
//   plane k: the residual of the planes before it, quantised with d_k = d_{k-1}/254.
// Rounding to nearest-even uses the 1.5*2^23 trick: the low byte of the float's bits is the int8.
// Not inlined: it is called from several places in the prologue.
template <int P, int ZHI = 8>  // columns P .. ZHI-1 of the block's scale row are zeroed (unused MMA columns)
__device__ __noinline__ void quantise_block(float4 va, float4 vb, int lane, uint8_t* act, int plane_stride, float* dpl, float* xs16, int b) {
    const float v[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
    amax = warp_max(amax);
    const float MAGIC = 12582912.f;
    float d = amax * (1.0f / 127.f);
    // Inverse scales overflow for blocks whose largest value is below ~1e-32 (id grows by 254 per plane): such a plane is
    // left empty (id = 0), which drops a residual of relative size 1e-5 or less of a block that is itself negligible.
    float id = amax > 0.f ? __fdividef(127.f, amax) : 0.f;
    if (!(id < 3.0e38f)) id = 0.f;
    float r[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) r[e] = v[e];
#pragma unroll
    for (int k = 0; k < P; ++k) {
        uint32_t tb[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float t = fmaf(r[e], id, MAGIC);
            tb[e] = __float_as_uint(t);
            r[e] = fmaf(-(t - MAGIC), d, r[e]);
        }
        const uint32_t w0 = __byte_perm(__byte_perm(tb[0], tb[1], 0x0040), __byte_perm(tb[2], tb[3], 0x0040), 0x5410);
        const uint32_t w1 = __byte_perm(__byte_perm(tb[4], tb[5], 0x0040), __byte_perm(tb[6], tb[7], 0x0040), 0x5410);
        *reinterpret_cast<uint2*>(act + k * plane_stride + 256 * b + 8 * lane) = make_uint2(w0, w1);
        if (lane == k) dpl[8 * b + k] = d;
        d *= (1.0f / 254.f);
        id *= 254.f;
        if (!(id < 3.0e38f)) id = 0.f;
    }
    if (lane >= P && lane < ZHI) dpl[8 * b + lane] = 0.f;  // unused MMA columns
    // sum of the represented values = x - final residual
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) s += v[e] - r[e];
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    if ((lane & 1) == 0) xs16[b * 16 + (lane >> 1)] = s;
}

// Build the activation vector in shared memory.  KQ: int8 planes + sums; else f32 copy.
// A warp takes 32 consecutive groups of 8 values (= one 256-value block) per turn.
// DEFER (k-quant weights behind an rmsnorm): the positive scalar 1/rms is not applied here at all.  The warps leave their sums of
// squares at L.off_ss and the caller multiplies every RESULT by 1/rms instead (W (c z) = c (W z)); the block-wide reduction,
// the square root and a second pass over the scales leave the critical path between "previous kernel done" and "first tile".
template <bool KQ, int P, bool TP = false, int ZHI = 8, bool DEFER = false>
__device__ __forceinline__ void build_activation(const MvParams& p, uint8_t* smem, const MvSmem& L, int warp, int lane, int nwarps, const float* x_in,
                                                 uint8_t* act, float* dpl, float* xs16, unsigned tp_epoch = 0) {
    const int n = p.n_in;
    float* red = reinterpret_cast<float*>(smem + L.off_red);
    float* xf = reinterpret_cast<float*>(smem + L.off_xf);
    const int n8 = n / 8;
    const int turns = p.turns;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);

    auto group_of = [&](int turn) { return 32 * (warp + nwarps * turn) + lane; };
    const MvTp* T = TP ? p.tp : nullptr;  // TP = false compiles the exchange out of single-GPU kernels
    const bool tp_sum = TP && T && T->part_src != nullptr;
    const int tp_n = tp_sum ? T->tp_size : 0;
    const float* part_src = tp_sum ? T->part_src : nullptr;
    float* x_out = tp_sum ? T->x_out : nullptr;
    // write_back: block 0 stores the summed residual stream (first pass over the vector only)
    auto fetch = [&](int turn, float4& a, float4& b, bool write_back = false) {
        const int g = group_of(turn);
        a = b = zero4;
        if (g < n8) {
            a = __ldcg(reinterpret_cast<const float4*>(x_in + 8 * g));
            b = __ldcg(reinterpret_cast<const float4*>(x_in + 8 * g + 4));
            if (tp_sum) {
                // Every value of a partial vector arrives as 8 bytes {f32 bits, tag}, tag = this token's number + 1, written by the
                // pushing GPU's finisher warps with 16-byte stores (two values).  A value is there when its tag is: no fence, no
                // arrival counter, no separate wait; each thread polls exactly what it is about to add (bounded by tp_timeout_ms).
                // Two ranks' words are in flight together (one L2 round trip per pair of ranks instead of per rank); the sums
                // are formed in rank order on every GPU: identical bits everywhere.
                const unsigned want = tp_epoch + 1u;
                const uint2* part2 = reinterpret_cast<const uint2*>(part_src);
#pragma unroll 1
                for (int r = 0; r < tp_n; r += 2) {
                    const bool two = r + 1 < tp_n;
                    const uint4* src0 = reinterpret_cast<const uint4*>(part2 + (size_t)r * n + 8 * g);
                    const uint4* src1 = reinterpret_cast<const uint4*>(part2 + (size_t)(two ? r + 1 : r) * n + 8 * g);
                    uint4 q0, q1, q2, q3, u0, u1, u2, u3;
                    unsigned long long t0 = 0;
                    for (unsigned spins = 0;; ++spins) {
                        q0 = ld_volatile_u32x4(src0);
                        q1 = ld_volatile_u32x4(src0 + 1);
                        q2 = ld_volatile_u32x4(src0 + 2);
                        q3 = ld_volatile_u32x4(src0 + 3);
                        u0 = ld_volatile_u32x4(src1);
                        u1 = ld_volatile_u32x4(src1 + 1);
                        u2 = ld_volatile_u32x4(src1 + 2);
                        u3 = ld_volatile_u32x4(src1 + 3);
                        const bool ok = q0.y == want && q0.w == want && q1.y == want && q1.w == want && q2.y == want && q2.w == want && q3.y == want && q3.w == want &&
                                        u0.y == want && u0.w == want && u1.y == want && u1.w == want && u2.y == want && u2.w == want && u3.y == want && u3.w == want;
                        if (ok) break;
                        if ((spins & 63u) == 63u) {  // not yet: look at the clock and at the status word now and then
                            const unsigned long long now = global_ns();
                            if (t0 == 0) t0 = now;
                            if (now - t0 > (unsigned long long)T->tp_timeout_ms * 1000000ull) {
                                atomicExch(p.status, DEV_ERR_PEER_TIMEOUT);
                                break;
                            }
                            if (__ldcg(p.status) != DEV_OK) break;  // somebody has given up already: the token is lost
                        }
                    }
                    a.x += __uint_as_float(q0.x); a.y += __uint_as_float(q0.z); a.z += __uint_as_float(q1.x); a.w += __uint_as_float(q1.z);
                    b.x += __uint_as_float(q2.x); b.y += __uint_as_float(q2.z); b.z += __uint_as_float(q3.x); b.w += __uint_as_float(q3.z);
                    if (two) {
                        a.x += __uint_as_float(u0.x); a.y += __uint_as_float(u0.z); a.z += __uint_as_float(u1.x); a.w += __uint_as_float(u1.z);
                        b.x += __uint_as_float(u2.x); b.y += __uint_as_float(u2.z); b.z += __uint_as_float(u3.x); b.w += __uint_as_float(u3.z);
                    }
                }
                if (write_back && blockIdx.x == 0) {
                    *reinterpret_cast<float4*>(x_out + 8 * g) = a;
                    *reinterpret_cast<float4*>(x_out + 8 * g + 4) = b;
                }
            }
        }
    };
    auto emit = [&](int turn, float4 a, float4 b) {
        const int g0 = 32 * (warp + nwarps * turn), g = g0 + lane;
        if (g0 >= n8) return;
        if (KQ) quantise_block<P, ZHI>(a, b, lane, act, L.plane_stride, dpl, xs16, g0 >> 5);
        else if (g < n8) {
            *reinterpret_cast<float4*>(xf + 8 * g) = a;
            *reinterpret_cast<float4*>(xf + 8 * g + 4) = b;
        }
    };
    auto sumsq = [](float4 a, float4 b, float ss) {
        ss = fmaf(a.x, a.x, ss); ss = fmaf(a.y, a.y, ss); ss = fmaf(a.z, a.z, ss); ss = fmaf(a.w, a.w, ss);
        ss = fmaf(b.x, b.x, ss); ss = fmaf(b.y, b.y, ss); ss = fmaf(b.z, b.z, ss); ss = fmaf(b.w, b.w, ss);
        return ss;
    };

    if (p.pro != PRO_RMSNORM) {
        // loads of up to MV_REG_BLOCKS turns are in flight together
        for (int t0 = 0; t0 < turns; t0 += MV_REG_BLOCKS) {
            float4 ka[MV_REG_BLOCKS], kb[MV_REG_BLOCKS];
#pragma unroll
            for (int u = 0; u < MV_REG_BLOCKS; ++u) fetch(t0 + u, ka[u], kb[u]);
#pragma unroll
            for (int u = 0; u < MV_REG_BLOCKS; ++u) emit(t0 + u, ka[u], kb[u]);
        }
    } else if (KQ) {
        // rmsnorm in front of k-quant weights: the int8 planes do not wait for the norm.  They are built from gain .* x at
        // once; the positive scalar 1/rms leaves them unchanged and only multiplies the plane scales and the per-16 sums,
        // which happens after the block-wide sum of squares (one barrier, whose wait the quantisation now overlaps).
        float ss = 0.f;
        const float inv_n = 1.0f / (float)n;
        for (int t0 = 0; t0 < turns; t0 += MV_GAIN_BLOCKS) {
            float4 ka[MV_GAIN_BLOCKS], kb[MV_GAIN_BLOCKS], ga[MV_GAIN_BLOCKS], gb[MV_GAIN_BLOCKS];
#pragma unroll
            for (int u = 0; u < MV_GAIN_BLOCKS; ++u) {
                fetch(t0 + u, ka[u], kb[u], true);
                const int g = group_of(t0 + u);
                ga[u] = gb[u] = zero4;
                if (g < n8) {
                    ga[u] = __ldg(reinterpret_cast<const float4*>(p.gain + 8 * g));
                    gb[u] = __ldg(reinterpret_cast<const float4*>(p.gain + 8 * g + 4));
                }
            }
#pragma unroll
            for (int u = 0; u < MV_GAIN_BLOCKS; ++u) {
                ss = sumsq(ka[u], kb[u], ss);
                float4 a = ka[u], b = kb[u];
                a.x *= ga[u].x; a.y *= ga[u].y; a.z *= ga[u].z; a.w *= ga[u].w;
                b.x *= gb[u].x; b.y *= gb[u].y; b.z *= gb[u].z; b.w *= gb[u].w;
                emit(t0 + u, a, b);
            }
        }
        ss = warp_sum(ss);
        if (DEFER) {
            if (lane == 0) {
                reinterpret_cast<float*>(smem + L.off_ss)[warp] = ss;
                mbar_arrive(reinterpret_cast<uint64_t*>(smem + L.off_bar) + 2 * MV_MAX_SLOTS + 2 * MV_RED_BUFS);  // ss_ready
            }
            consumer_sync(nwarps * 32);
            return;
        }
        if (lane == 0) red[warp] = ss;
        consumer_sync(nwarps * 32);
        float tot = 0.f;
        for (int i = 0; i < nwarps; ++i) tot += red[i];  // same order in every thread
        // 1 / sqrt(ss / n + eps) (src/inference.jl:105-107) with a multiplication by 1/n and a correctly rounded reciprocal
        // square root: two divisions and a square root are about eighty dependent instructions, on the critical path of every
        // layer twice.  The planes are an approximation of the f32 activations already (relative 1e-7); this is below it.
        tot = fmaf(tot, inv_n, 1e-5f);
        const float scale = __frsqrt_rn(tot);
        for (int turn = 0; turn < turns; ++turn) {  // this warp's blocks
            const int g0 = 32 * (warp + nwarps * turn);
            if (g0 >= n8) break;
            const int b = g0 >> 5;
            if (lane < ZHI) dpl[8 * b + lane] *= scale;
            if (lane < 16) xs16[16 * b + lane] *= scale;
        }
        // (the barrier below also keeps `red` untouched until every thread has read it)
    } else {
        // pass 1: sum of squares; the first MV_REG_BLOCKS turns stay in registers for pass 2
        float4 ka[MV_REG_BLOCKS], kb[MV_REG_BLOCKS];
        float4 ga[MV_GAIN_BLOCKS], gb[MV_GAIN_BLOCKS];  // gains of the register-held turns, loaded with x, not after the sum
        float ss = 0.f;
#pragma unroll
        for (int u = 0; u < MV_REG_BLOCKS; ++u) fetch(u, ka[u], kb[u], true);
#pragma unroll
        for (int u = 0; u < MV_GAIN_BLOCKS; ++u) {
            const int g = group_of(u);
            ga[u] = gb[u] = zero4;
            if (g < n8) {
                ga[u] = __ldg(reinterpret_cast<const float4*>(p.gain + 8 * g));
                gb[u] = __ldg(reinterpret_cast<const float4*>(p.gain + 8 * g + 4));
            }
        }
#pragma unroll
        for (int u = 0; u < MV_REG_BLOCKS; ++u) ss = sumsq(ka[u], kb[u], ss);
        for (int turn = MV_REG_BLOCKS; turn < turns; ++turn) {
            float4 a, b;
            fetch(turn, a, b, true);
            ss = sumsq(a, b, ss);
        }
        float tot = block_sum(ss, red, warp, lane, nwarps);
        tot /= (float)n;
        tot += 1e-5f;
        const float scale = 1.0f / sqrtf(tot);
        auto apply = [&](const float4& ga, const float4& gb, float4& a, float4& b) {  // weight .* (ss .* x)
            a.x = ga.x * (scale * a.x); a.y = ga.y * (scale * a.y); a.z = ga.z * (scale * a.z); a.w = ga.w * (scale * a.w);
            b.x = gb.x * (scale * b.x); b.y = gb.y * (scale * b.y); b.z = gb.z * (scale * b.z); b.w = gb.w * (scale * b.w);
        };
        auto normalise = [&](int turn, float4& a, float4& b) {
            const int g = group_of(turn);
            if (g < n8) {
                const float4 ga = __ldg(reinterpret_cast<const float4*>(p.gain + 8 * g));
                const float4 gb = __ldg(reinterpret_cast<const float4*>(p.gain + 8 * g + 4));
                apply(ga, gb, a, b);
            }
        };
#pragma unroll
        for (int u = 0; u < MV_REG_BLOCKS; ++u) {
            if (u < MV_GAIN_BLOCKS) apply(ga[u], gb[u], ka[u], kb[u]);  // lanes beyond n have x = 0 and gain = 0
            else normalise(u, ka[u], kb[u]);
            emit(u, ka[u], kb[u]);
        }
        for (int turn = MV_REG_BLOCKS; turn < turns; ++turn) {
            float4 a, b;
            fetch(turn, a, b);
            normalise(turn, a, b);
            emit(turn, a, b);
        }
    }
    consumer_sync(nwarps * 32);
}

// The same for the two vectors of a two-position launch (k-quant weights, one GPU), both in one pass: vector 0 at x_in ->
// planes 0..P-1, scale columns 0..3; vector 1 at x_in + n_in -> planes P..2P-1, scale columns 4..7, its own sums.
template <int P>
__device__ __forceinline__ void build_activation_pair(const MvParams& p, uint8_t* smem, const MvSmem& L, int warp, int lane, int nwarps) {
    const int n = p.n_in, n8 = n / 8, turns = p.turns, nb = n / QK_K;
    float* red = reinterpret_cast<float*>(smem + L.off_red);
    uint8_t* act0 = smem + L.off_act;
    uint8_t* act1 = act0 + P * L.plane_stride;
    float* dpl0 = reinterpret_cast<float*>(smem + L.off_dpl);
    float* dpl1 = dpl0 + 4;
    float* xs0 = reinterpret_cast<float*>(smem + L.off_xs);
    float* xs1 = xs0 + nb * 16;
    const bool norm = p.pro == PRO_RMSNORM;
    auto sumsq = [](float4 a, float4 b, float ss) {
        ss = fmaf(a.x, a.x, ss); ss = fmaf(a.y, a.y, ss); ss = fmaf(a.z, a.z, ss); ss = fmaf(a.w, a.w, ss);
        ss = fmaf(b.x, b.x, ss); ss = fmaf(b.y, b.y, ss); ss = fmaf(b.z, b.z, ss); ss = fmaf(b.w, b.w, ss);
        return ss;
    };
    auto mul = [](float4& a, const float4& g) { a.x *= g.x; a.y *= g.y; a.z *= g.z; a.w *= g.w; };
    float ss0 = 0.f, ss1 = 0.f;
    for (int turn = 0; turn < turns; ++turn) {
        const int g0 = 32 * (warp + nwarps * turn), g = g0 + lane;
        if (g0 >= n8) break;  // whole 256-value blocks: every lane of the warp is inside the vector
        const float* x0 = p.x_in + 8 * g;
        const float* x1 = x0 + n;
        float4 a0 = __ldcg(reinterpret_cast<const float4*>(x0)), b0 = __ldcg(reinterpret_cast<const float4*>(x0 + 4));
        float4 a1 = __ldcg(reinterpret_cast<const float4*>(x1)), b1 = __ldcg(reinterpret_cast<const float4*>(x1 + 4));
        if (norm) {  // gain .* x now, 1/rms afterwards (see build_activation)
            const float4 ga = __ldg(reinterpret_cast<const float4*>(p.gain + 8 * g));
            const float4 gb = __ldg(reinterpret_cast<const float4*>(p.gain + 8 * g + 4));
            ss0 = sumsq(a0, b0, ss0);
            ss1 = sumsq(a1, b1, ss1);
            mul(a0, ga); mul(b0, gb); mul(a1, ga); mul(b1, gb);
        }
        quantise_block<P, 4>(a0, b0, lane, act0, L.plane_stride, dpl0, xs0, g0 >> 5);
        quantise_block<P, 4>(a1, b1, lane, act1, L.plane_stride, dpl1, xs1, g0 >> 5);
    }
    if (norm) {
        ss0 = warp_sum(ss0);
        ss1 = warp_sum(ss1);
        if (lane == 0) {
            red[warp] = ss0;
            red[MV_MAX_CONSUMERS + warp] = ss1;
        }
        consumer_sync(nwarps * 32);
        float t0 = 0.f, t1 = 0.f;
        for (int i = 0; i < nwarps; ++i) {  // same order in every thread
            t0 += red[i];
            t1 += red[MV_MAX_CONSUMERS + i];
        }
        const float s0 = 1.0f / sqrtf(t0 / (float)n + 1e-5f), s1 = 1.0f / sqrtf(t1 / (float)n + 1e-5f);
        for (int turn = 0; turn < turns; ++turn) {
            const int g0 = 32 * (warp + nwarps * turn);
            if (g0 >= n8) break;
            const int b = g0 >> 5;
            if (lane < 4) {
                dpl0[8 * b + lane] *= s0;
                dpl1[8 * b + lane] *= s1;
            }
            if (lane < 16) {
                xs0[16 * b + lane] *= s0;
                xs1[16 * b + lane] *= s1;
            }
        }
    }
    consumer_sync(nwarps * 32);
}

// ---- work enumeration ----------------------------------------------------------------------
// A unit is a tile of MV_TILE_PAIRS row pairs of one segment (k-quant) or one pair (f32).  Units of all segments
// are numbered consecutively; block b takes units b, b + grid, b + 2*grid, ... so that every block streams the
// same number of bytes (+-1 unit).
struct UnitInfo {
    int seg;    // segment index
    int pair0;  // first pair of the unit within the segment
};

template <bool KQ>
__device__ __forceinline__ UnitInfo find_unit(const MvParams& p, int unit) {
    UnitInfo u;
    u.seg = 0;
    if (p.nseg > 1 && unit >= p.seg_start[1]) u.seg = 1;
    if (p.nseg > 2 && unit >= p.seg_start[2]) u.seg = 2;
    u.pair0 = (unit - p.seg_start[u.seg]) * (KQ ? MV_TILE_PAIRS : 1);
    return u;
}

// Segment descriptor number i, chosen with selects on statically indexed parameters: a dynamically indexed
// read of the kernel parameter block costs an indexed constant load of a few hundred cycles per field.
__device__ __forceinline__ MvSegment get_segment(const MvParams& p, int i) {
    MvSegment a = p.seg[0];
    if (p.nseg > 1 && i >= 1) {
        const MvSegment& b = (i == 1) ? p.seg[1] : p.seg[2];
        a = b;
    }
    return a;
}

__device__ __forceinline__ void pair_rows(const MvParams& p, const MvSegment& sg, int t, int& rowA, int& rowB) {
    if (sg.pair_mode == PAIR_ADJACENT) {
        rowA = 2 * t;
        rowB = 2 * t + 1;
    } else if (sg.pair_mode == PAIR_NEOX) {
        const int h2 = sg.head_size >> 1;
        const int head = (int)__umulhi((unsigned)t, p.neox_magic);  // t / h2
        rowA = head * sg.head_size + (t - head * h2);
        rowB = rowA + h2;
    } else {
        rowA = rowB = t;
    }
}

// ---- tile geometry in a ring slot ----------------------------------------------------------------
// Rows of a tile arrive in groups of adjacent matrix rows, one bulk copy per group.  Groups are GS bytes apart,
// GS = 32 mod 128, and lane group g works on pair PI[g] = (0,2,4,6,1,3,5,7)[g]: the four row groups g = 0..3
// (and 4..7) that a 64-bit fragment load touches together then sit in four different copy groups, i.e. in
// different shared-memory banks.  When a row is longer than one stage (nit > 1) the rows of a group are not
// contiguous in memory and every row is its own copy (16 per stage).  The grouping of a segment is fixed on the host.
__host__ __device__ inline int pad_32_mod_128(int v) {
    while ((v & 127) != 32) v += 16;
    return v;
}
// Host side: decide the copy grouping of a segment.  kb = super-blocks per row and stage, nit = stages per row.
__host__ inline void mv_fill_geometry(MvSegment& sg, int kb, int nit) {
    sg.rowb = kb * dev_block_bytes(sg.type);
    (void)nit;  // rows longer than a stage are stored as column panels (panelize_kernel): every stage looks like a short row
    if (sg.pair_mode == PAIR_ADJACENT) {
        sg.ngroups = 4; sg.rpg = 4;
    } else {
        sg.ngroups = 8; sg.rpg = 2;
    }
    sg.gs = pad_32_mod_128(sg.rpg * sg.rowb);
}
// Byte offsets of the two rows (A, B) of pair j inside a slot.
// rowb = bytes of one row in THIS stage (the last panel of a long row may be narrower than 16 blocks).
__device__ __forceinline__ void pair_offsets(const MvSegment& t, int rowb, int j, int& offA, int& offB) {
    if (t.rpg == 4) {
        offA = (j >> 1) * t.gs + 2 * (j & 1) * rowb;
        offB = offA + rowb;
    } else {
        offA = (j >> 1) * t.gs + (j & 1) * rowb;
        offB = offA + 4 * t.gs;
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

// Operands of an epilogue that come from global memory (the residual values, the RoPE factors).  The finisher warp
// loads them BEFORE it waits for a tile's sums, so that their latency is not added to the tail of the kernel.
struct EpiPre {
    int rowA, rowB;   // the pair's matrix rows
    float rA, rB;     // EPI_RESIDUAL: resid[rowA], resid[rowB]
    float2 cs;        // EPI_ROPE_*: (cos, sin)
    size_t dA, dB;    // cache epilogues: element offsets of the two destinations (the divisions by head_size are done here)
};
__device__ __forceinline__ EpiPre epilogue_preload(const MvParams& p, const MvSegment& sg, int t, int pos, int seq = 0) {
    EpiPre e;
    e.rA = e.rB = 0.f;
    e.cs = make_float2(0.f, 0.f);
    e.dA = e.dB = 0;
    pair_rows(p, sg, t, e.rowA, e.rowB);
    if (sg.epi == EPI_RESIDUAL) {
        const float* resid = p.resid + (size_t)seq * sg.out2;
        e.rA = __ldcg(resid + e.rowA);
        e.rB = __ldcg(resid + e.rowB);
    } else if (sg.epi == EPI_ROPE_Q || sg.epi == EPI_ROPE_K || sg.epi == EPI_STORE_V) {
        const int hs = sg.head_size, h2 = hs >> 1;
        const int head = e.rowA / hs, inA = e.rowA - head * hs, inB = e.rowB - head * hs;  // both rows lie in one head
        if (sg.epi != EPI_STORE_V) {
            const int i = (sg.pair_mode == PAIR_NEOX) ? inA : (inA >> 1);
            e.cs = __ldg(reinterpret_cast<const float2*>(p.rope_cs) + (size_t)pos * h2 + i);
        }
        const size_t base = ((size_t)head * p.seq_len + pos) * hs;  // cache layout [kv_head][seq_len][hs]
        e.dA = base + inA;
        e.dB = base + inB;
    }
    return e;
}

template <bool TP = false, bool PRE = false>
__device__ __forceinline__ void epilogue_pair(const MvParams& p, const MvSegment& sg, int t, float vA, float vB, int pos, ArgBest& best, int seq = 0,
                                              const EpiPre* pre = nullptr) {
    // seq = 1: the second position of a two-position launch (pos is already that position's; vectors sit out2 elements further)
    int rowA, rowB;
    if (PRE) {
        rowA = pre->rowA;
        rowB = pre->rowB;
    } else {
        pair_rows(p, sg, t, rowA, rowB);
    }
    float* const out = sg.out + (size_t)seq * sg.out2;
    switch (sg.epi) {
        case EPI_STORE:
            out[rowA] = vA;
            out[rowB] = vB;
            break;
        case EPI_RESIDUAL: {
            if (PRE) {
                out[rowA] = pre->rA + vA;
                out[rowB] = pre->rB + vB;
            } else {
                const float* resid = p.resid + (size_t)seq * sg.out2;
                out[rowA] = __ldcg(resid + rowA) + vA;
                out[rowB] = __ldcg(resid + rowB) + vB;
            }
            break;
        }
        case EPI_SWIGLU: {
            const float g = vA * (1.0f / (1.0f + expf(-vA)));
            out[t] = g * vB;
            break;
        }
        case EPI_ROPE_Q:
        case EPI_ROPE_K: {
            float2 cs;
            if (PRE) {
                cs = pre->cs;
            } else {
                const int hs = sg.head_size, h2 = hs >> 1;
                const int i = (sg.pair_mode == PAIR_NEOX) ? (rowA % hs) : ((rowA % hs) >> 1);
                cs = __ldg(reinterpret_cast<const float2*>(p.rope_cs) + (size_t)pos * h2 + i);
            }
            // (a + bi)(c + si): every product and sum rounded on its own, as the reference's complex multiply
            const float oa = __fsub_rn(__fmul_rn(vA, cs.x), __fmul_rn(vB, cs.y));
            const float ob = __fadd_rn(__fmul_rn(vA, cs.y), __fmul_rn(vB, cs.x));
            if (sg.epi == EPI_ROPE_Q) {
                out[rowA] = oa;
                out[rowB] = ob;
            } else if (PRE) {  // key cache [kv_head][seq_len][hs]
                out[pre->dA] = oa;
                out[pre->dB] = ob;
            } else {
                const int hs = sg.head_size;
                float* dst = out + ((size_t)(rowA / hs) * p.seq_len + pos) * hs;
                dst[rowA % hs] = oa;
                dst[rowB % hs] = ob;
            }
            break;
        }
        case EPI_STORE_V: {  // value cache [kv_head][seq_len][hs]
            if (PRE) {
                out[pre->dA] = vA;
                out[pre->dB] = vB;
            } else {
                const int hs = sg.head_size;
                float* dst = out + ((size_t)(rowA / hs) * p.seq_len + pos) * hs;
                dst[rowA % hs] = vA;
                dst[rowB % hs] = vB;
            }
            break;
        }
        case EPI_LOGITS:
            out[rowA] = vA;
            out[rowB] = vB;
            arg_update(best, vA, rowA);
            arg_update(best, vB, rowB);
            break;
        case EPI_PUSH:
            if (TP) {
                const MvTp* T = p.tp;
                const int g = T->tp_size;
                for (int r = 0; r < g; ++r) {
                    float* dst = T->push_dst[r];
                    dst[rowA] = vA;
                    dst[rowB] = vB;
                }
            }
            break;
    }
}

// ---- the kernel --------------------------------------------------------------------------------
// DBG = true compiles in the measurement aids (timeline stamps, skip-arithmetic / skip-copies switches); the production
// instantiations carry none of them: even a predicated-off stamp in the producer's loop cost 2 % of a token.
// NB = 2: two activation vectors (two consecutive prompt positions) per launch.  Their int8 planes occupy MMA columns
// 0..2 and 4..6, so the weights are streamed and unpacked once for both positions at no extra MMA cost.
template <bool KQ, int P, bool TP = false, bool DBG = false, int NB = 1>
__global__ void __launch_bounds__((MV_MAX_CONSUMERS + 2) * 32, 1) fused_matvec_kernel(const __grid_constant__ MvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int W = p.consumers;
    const int NS = p.nslots;
    const MvSmem L = mv_smem_layout(p.n_in, P, KQ, KQ ? NS : 0, p.row_stride, NB);
    MV_TRACE(0);

    const int nb = p.n_in / QK_K;
    const int nit = p.nit;
    const int my_units = p.units_lo + ((int)blockIdx.x < p.units_rem ? 1 : 0);

    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.off_bar);
    uint64_t* empty = full + MV_MAX_SLOTS;
    uint64_t* red_full = empty + MV_MAX_SLOTS;
    uint64_t* red_empty = red_full + MV_RED_BUFS;
    uint64_t* ss_ready = red_empty + MV_RED_BUFS;  // every consumer warp has left its sum of squares (deferred rmsnorm scale)
    uint8_t* ring = smem + L.off_ring;
    // Waits of the producer and finisher warps on the consumer warps.  With tensor parallelism the consumers may themselves
    // be waiting, legitimately and for up to tp_timeout_ms, for another GPU's partial results: those waits are then bounded
    // by that time plus a margin instead of by the short poll budget, which host-side skew between the ranks would exhaust.
    auto wait_partner = [&](uint64_t* bar, uint32_t parity) -> bool {
        if (TP && p.tp) return mbar_wait_bounded_ns(bar, parity, ((unsigned long long)p.tp->tp_timeout_ms + 1000ull) * 1000000ull);
        return mbar_wait_bounded(bar, parity);
    };

    if (KQ) {
        if (threadIdx.x < NS) {
            mbar_init(full + threadIdx.x, 1);
            mbar_init(empty + threadIdx.x, W / p.cgroups);
        }
        if (threadIdx.x >= 32 && threadIdx.x < 32 + MV_RED_BUFS) {
            mbar_init(red_full + (threadIdx.x - 32), W / p.cgroups);
            mbar_init(red_empty + (threadIdx.x - 32), 1);
        }
        if (threadIdx.x == 31) mbar_init(ss_ready, W);
        if (threadIdx.x < 32 + MV_RED_BUFS) {
            fence_barrier_init();
            fence_proxy_async();
        }
        __syncthreads();
    }
    MV_TRACE(7);

    // ================================ producer warp =============================================
    // Lane c brings copy group c of every stage.  This warp runs serial address arithmetic on a busy SM, so the
    // parameters of the NEXT tile are worked out right after a tile's copies are issued, in the shadow of the
    // wait for a free slot.
    if (KQ && warp == W) {
        pdl_launch_dependents();
        if (lane >= 16) return;
        const uint64_t policy = policy_evict_first();
        const int c = lane;
        struct TileSrc {
            const uint8_t* src;  // first byte of this lane's copy (stage 0)
            uint32_t bytes0;     // bytes of this lane's copy in a full-width stage (0: nothing to copy)
            uint32_t tx0;        // bytes of the whole stage (all lanes) in a full-width stage
            int bb, nrows, nvalid, gs;
            int row;             // matrix row of this lane's copy (panel addressing of long rows)
            size_t ps;           // bytes of one full column panel of the matrix (rows * 16 blocks)
        };
        auto tile_src = [&](int j) {
            TileSrc ts;
            ts.src = nullptr;
            ts.bytes0 = ts.tx0 = 0;
            ts.bb = ts.nrows = ts.nvalid = ts.gs = ts.row = 0;
            ts.ps = 0;
            if (j >= my_units) return ts;
            const UnitInfo u = find_unit<true>(p, (int)blockIdx.x + j * (int)gridDim.x);
            const MvSegment sg = get_segment(p, u.seg);
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
                    const int half = (sg.rpg == 2) ? (c >> 2) : (c >> 3);      // A or B rows
                    const int jp = (sg.rpg == 2) ? 2 * (c & 3) : (c & 7);      // pair of the copy's first row
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
        bool dead = false, first = true;
        // Stage counters kept as (slot, phase) per consumer group: integer division by a run-time value costs
        // hundreds of cycles here.  Group g owns slots g*NSG .. g*NSG+NSG-1 and takes tiles g, g+cgroups, ...
        const int CG = p.cgroups, NSG = NS / CG;
        int slot_g[2] = {0, NSG}, ph_g[2] = {0, 0};
        TileSrc ts = tile_src(0);
        // Fast path for the common case (one segment, adjacent or dual rows, full tiles): the next tile's source
        // is the current one plus a constant.
        const bool linear = (p.nseg == 1) && (p.seg[0].pair_mode != PAIR_NEOX);
        const int row_step = (int)gridDim.x * (p.seg[0].pair_mode == PAIR_ADJACENT ? 16 : 8);  // rows between a block's consecutive tiles
        const size_t tile_step = linear ? (size_t)row_step * p.seg[0].rowb : 0;
        const int full_tiles = linear ? p.seg[0].npairs / MV_TILE_PAIRS : 0;  // tiles below this index are complete
        for (int j = 0; j < my_units && !dead; ++j) {
            const int grp = (CG == 2) ? (j & 1) : 0;
            int slot_i = grp ? slot_g[1] : slot_g[0], ph = grp ? ph_g[1] : ph_g[0];
            for (int it = 0; it < nit; ++it) {
                // wait until every consumer warp of the group has released what this slot held before
                if (ph > 0) {
                    int ok = 1;
                    if (c == 0) ok = wait_partner(empty + slot_i, (uint32_t)((ph & 1) ^ 1)) ? 1 : 0;
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
                if (DBG && (p.debug & 2)) bytes = tx = 0;
                if (c == 0) mbar_arrive_expect_tx(full + slot_i, tx);
                __syncwarp(0x0000ffffu);
                if (bytes)
                    bulk_g2s(ring + (size_t)slot_i * L.slot_bytes + (size_t)c * ts.gs, src, bytes, full + slot_i, policy);
                if (DBG && first && p.trace && lane == 0) p.trace[blockIdx.x * 16 + 1] = global_ns();
                first = false;
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
            // parameters of the next tile (in the shadow of the wait for its slot)
            const int next_tile = (int)blockIdx.x + (j + 1) * (int)gridDim.x;
            if (linear && next_tile < full_tiles) {
                ts.src += tile_step;
                ts.row += row_step;
            }
            else ts = tile_src(j + 1);
        }
        if (dead) {
            // a consumer gave up: let copies still in flight land (bounded) before shared memory is released
            atomicExch(p.status, DEV_ERR_TMA_TIMEOUT);
            for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // copies land within microseconds; 2 ms is a generous bound
        }
        return;
    }

    // ================================ finisher warp ==============================================
    // Adds the consumer warps' partial sums of a tile in a fixed order (results do not depend on timing) and runs
    // the epilogue of its 8 row pairs.
    if (KQ && warp == W + 1) {
        pdl_launch_dependents();
        pdl_wait();
        const int pos = p.pos ? __ldcg(p.pos) : 0;
        ArgBest best;
        best.v = -INFINITY;
        best.i = 0x7fffffff;
        const float* red = reinterpret_cast<const float*>(smem + L.off_red);
        // 1/rms of the input vector (deferred by the prologue, NB == 1): worked out from the warps' sums of squares when the first
        // tile arrives, which orders their stores before these loads
        float in_scale = 1.f;
        // EPI_PUSH: where this GPU's partial vector goes on every GPU, read once (read per tile, each address would cost the
        // finisher an L2 round trip per rank and tile, in series: the stores of the previous tile may alias the descriptor)
        float* push_to[MV_MAX_TP];
#pragma unroll
        for (int r = 0; r < MV_MAX_TP; ++r) push_to[r] = (TP && p.tp_push && r < p.tp->tp_size) ? p.tp->push_dst[r] : nullptr;
        const unsigned push_tag = (TP && p.tp_push) ? __ldcg(p.tp->tp_epoch) + 1u : 0u;  // this token's number + 1 (see the summing prologue)
        // lane = 16*q + 8*half + pair: sums the partials of warps w = q, q+2, ... of row `half` of pair `pair`
        const int fq = lane >> 4, fidx = lane & 15;
        const int WGf = W / p.cgroups;  // warps that contribute to one tile
        int unit = (int)blockIdx.x, seg_i = -1, seg_end = 0, seg_first = 0, rb = 0;
        uint32_t par = 0;
        MvSegment sg = p.seg[0];
        bool dead = false;
        if (NB == 1 && p.pro == PRO_RMSNORM && my_units > 0) {  // while the consumers work on the first tile
            if (wait_partner(ss_ready, 0)) {
                const float* ssw = reinterpret_cast<const float*>(smem + L.off_ss);
                float tot = 0.f;
                for (int i = 0; i < W; ++i) tot += ssw[i];  // same order in every block
                in_scale = __frsqrt_rn(fmaf(tot, 1.0f / (float)p.n_in, 1e-5f));  // 1 / sqrt(ss / n + eps), src/inference.jl:105-107
            } else {
                dead = true;
            }
        }
        for (int j = 0; j < my_units && !dead; ++j, unit += (int)gridDim.x) {
            if (seg_i < 0 || unit >= seg_end) {
                seg_i = find_unit<true>(p, unit).seg;
                sg = get_segment(p, seg_i);
                seg_first = (seg_i == 0) ? 0 : (seg_i == 1 ? p.seg_start[1] : p.seg_start[2]);
                seg_end = (seg_i == 0) ? p.seg_start[1] : (seg_i == 1 ? p.seg_start[2] : p.seg_start[3]);
            }
            // what the epilogue needs from global memory is fetched while the consumers are still at work on the tile
            const int t = (unit - seg_first) * MV_TILE_PAIRS + lane;
            const bool mine = lane < MV_TILE_PAIRS && t < sg.npairs;
            EpiPre pre0, pre1;
            if (mine) {
                pre0 = epilogue_preload(p, sg, t, pos);
                if (NB == 2) pre1 = epilogue_preload(p, sg, t, pos + 1, 1);
            }
            if (!wait_partner(red_full + rb, par)) {
                dead = true;
                break;
            }
            const float* rbuf = red + rb * (MV_MAX_CONSUMERS * 16 * NB);
            float v = 0.f, v1 = 0.f;
            if (NB == 1) {
                for (int w = fq; w < WGf; w += 2) v += rbuf[w * 16 + fidx];
            } else {
                for (int w = fq; w < WGf; w += 2) {
                    v += rbuf[(w * 2) * 16 + fidx];
                    v1 += rbuf[(w * 2 + 1) * 16 + fidx];
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(red_empty + rb);  // the buffer may be rewritten
            v += __shfl_xor_sync(0xffffffffu, v, 16);     // (even warps) + (odd warps)
            if (NB == 1) v *= in_scale;
            const float vB = __shfl_sync(0xffffffffu, v, (lane & 7) + 8);
            if (TP && p.tp_push) {
                if (mine) {
#pragma unroll
                    for (int r = 0; r < MV_MAX_TP; ++r) {
                        if (push_to[r] == nullptr) continue;
                        uint2* dst2 = reinterpret_cast<uint2*>(push_to[r]);  // {value, tag} pairs
                        if (pre0.rowB == pre0.rowA + 1 && !(pre0.rowA & 1)) {  // adjacent rows: one 16-byte store
                            st_volatile_u32x4(reinterpret_cast<uint4*>(dst2 + pre0.rowA), make_uint4(__float_as_uint(v), push_tag, __float_as_uint(vB), push_tag));
                        } else {
                            st_volatile_u32x2(dst2 + pre0.rowA, make_uint2(__float_as_uint(v), push_tag));
                            st_volatile_u32x2(dst2 + pre0.rowB, make_uint2(__float_as_uint(vB), push_tag));
                        }
                    }
                }
            } else if (mine) {
                epilogue_pair<TP, true>(p, sg, t, v, vB, pos, best, 0, &pre0);
            }
            if (NB == 2) {  // the second position
                v1 += __shfl_xor_sync(0xffffffffu, v1, 16);
                const float v1B = __shfl_sync(0xffffffffu, v1, (lane & 7) + 8);
                if (mine) epilogue_pair<TP, true>(p, sg, t, v1, v1B, pos + 1, best, 1, &pre1);
            }
            if (++rb == MV_RED_BUFS) {
                rb = 0;
                par ^= 1u;
            }
        }
        if (dead && lane == 0) atomicExch(p.status, DEV_ERR_TMA_TIMEOUT);
        if (p.amax_val) {  // EPI_LOGITS: first maximal index over this block's rows
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best.v, o);
                const int oi = __shfl_xor_sync(0xffffffffu, best.i, o);
                arg_update(best, ov, oi);
            }
            if (lane == 0) {
                p.amax_val[blockIdx.x] = best.v;
                p.amax_idx[blockIdx.x] = best.i;
            }
        }
        if (DBG && p.trace && lane == 0) p.trace[blockIdx.x * 16 + 8] = global_ns();
        return;
    }

    // ================================ consumer warps ============================================
    // Weights are constants; everything below reads what the previous kernel wrote.
    pdl_launch_dependents();
    // The exchange descriptor and the token count do not change during a token (the count advances in the token's last
    // kernel): fetched now, behind the previous kernel's tail, instead of as two dependent round trips after the wait.
    unsigned tp_epoch = 0;
    if (TP && p.tp && p.tp->part_src != nullptr) tp_epoch = __ldcg(p.tp->tp_epoch);
    pdl_wait();
    MV_TRACE(2);

    {
        uint8_t* act = smem + L.off_act;
        float* dpl = reinterpret_cast<float*>(smem + L.off_dpl);
        float* xs16 = reinterpret_cast<float*>(smem + L.off_xs);
        if (NB == 1) {
            build_activation<KQ, P, TP, 8, KQ>(p, smem, L, warp, lane, W, p.x_in, act, dpl, xs16, tp_epoch);
        } else {
            build_activation_pair<P>(p, smem, L, warp, lane, W);
        }
    }
    MV_TRACE(3);

    const int pos = p.pos ? __ldcg(p.pos) : 0;
    ArgBest best;
    best.v = -INFINITY;
    best.i = 0x7fffffff;

    if (KQ) {
        TileCtx cx;
        cx.act = smem + L.off_act;
        cx.dpl = reinterpret_cast<const float*>(smem + L.off_dpl);
        cx.xs16 = reinterpret_cast<const float*>(smem + L.off_xs);
        tile_ctx_columns<NB, P>(cx, smem + L.off_act, L.plane_stride, lane);
        if (NB == 2) cx.xs16 = reinterpret_cast<const float*>(smem + L.off_xs) + (cx.t >> 1) * (p.n_in / QK_K) * 16;  // this lane's vector
        const int pj = ((cx.g & 3) << 1) | (cx.g >> 2);  // the pair of the tile this lane group works on: (0,2,4,6,1,3,5,7)[g]
        float* red = reinterpret_cast<float*>(smem + L.off_red);
        bool dead = false;
        // counters kept incrementally (no run-time divisions in the loop): weight slot and its phase parity,
        // reduction buffer and its phase parity, and the warp whose turn it is to finish a tile
        const int CG = p.cgroups, WG = W / CG, NSG = NS / CG;
        const int grp = warp / WG, wl = warp - grp * WG;  // this warp's group and its index inside the group
        int slot_i = grp * NSG, rb = grp, red_wrap = 0;
        uint32_t full_par = 0;
        // Per-tile bookkeeping is incremental: the segment descriptor and everything derived from it change only
        // when the unit number crosses into the next segment (serial code here runs at ~20 cycles per instruction).
        int unit = (int)blockIdx.x + grp * (int)gridDim.x, seg_i = -1, seg_end = 0, seg_first = 0;
        MvSegment sg = p.seg[0];
        int bb = 0, offA = 0, offB = 0;
        for (int j = grp; j < my_units; j += CG, unit += CG * (int)gridDim.x) {
            if (seg_i < 0 || unit >= seg_end) {
                const UnitInfo u0 = find_unit<true>(p, unit);
                seg_i = u0.seg;
                sg = get_segment(p, seg_i);
                seg_first = (seg_i == 0) ? 0 : (seg_i == 1 ? p.seg_start[1] : p.seg_start[2]);
                seg_end = (seg_i == 0) ? p.seg_start[1] : (seg_i == 1 ? p.seg_start[2] : p.seg_start[3]);
                bb = dev_block_bytes(sg.type);
                pair_offsets(sg, sg.rowb, pj, offA, offB);
            }
            UnitInfo u;
            u.seg = seg_i;
            u.pair0 = (unit - seg_first) * MV_TILE_PAIRS;
            // q6_K super-block scales travel outside the records; rows of this lane group's pair
            const __half* d6A = nullptr;
            const __half* d6B = nullptr;
            if (sg.type == T_Q6_K) {
                const int t = min(u.pair0 + pj, sg.npairs - 1);
                int rowA, rowB;
                pair_rows(p, sg, t, rowA, rowB);
                d6A = sg.d6 + (size_t)rowA * nb;
                d6B = ((sg.pair_mode == PAIR_DUAL) ? sg.d6_2 : sg.d6) + (size_t)rowB * nb;
            }
            float accA = 0.f, accB = 0.f;  // the two rows of pair pj of the tile
            for (int it = 0; it < nit; ++it) {
                const int b0 = it * p.kb, nblk = min(p.kb, nb - b0);
                int oA = offA, oB = offB;
                if (nit > 1 && nblk < p.kb) pair_offsets(sg, nblk * bb, pj, oA, oB);  // narrow last panel
                float dA = 0.f, dB = 0.f;
                if (sg.type == T_Q6_K && wl < nblk) {  // fetched before the wait so that the latency overlaps it
                    dA = __half2float(__ldg(d6A + b0 + wl));
                    dB = __half2float(__ldg(d6B + b0 + wl));
                }
                if (!dead && !mbar_wait_bounded(full + slot_i, full_par)) dead = true;  // uniform across the warp
                if (!dead && !(DBG && (p.debug & 1))) {
                    const uint8_t* slot = ring + (size_t)slot_i * L.slot_bytes;
                    for (int bl = wl; bl < nblk; bl += WG) {
                        const uint8_t* rA = slot + oA + bl * bb;
                        const uint8_t* rB = slot + oB + bl * bb;
                        if (sg.type == T_Q4_K) tile_q4k<NB>(rA, rB, b0 + bl, cx, accA, accB);
                        else if (sg.type == T_Q5_K) tile_q5k<NB>(rA, rB, b0 + bl, cx, accA, accB);
                        else {
                            if (bl != wl) {  // a second column for this warp (fewer warps than columns)
                                dA = __half2float(__ldg(d6A + b0 + bl));
                                dB = __half2float(__ldg(d6B + b0 + bl));
                            }
                            tile_q6k<NB>(rA, rB, dA, dB, b0 + bl, cx, accA, accB);
                        }
                    }
                }
                __syncwarp();  // every lane is done reading the slot
                if (lane == 0 && !dead) mbar_arrive(empty + slot_i);
                if (++slot_i == (grp + 1) * NSG) {
                    slot_i = grp * NSG;
                    full_par ^= 1u;
                }
            }
            // This warp's share of the tile: sum over the four lanes of a row group, then hand it to the finisher
            // warp through one of MV_RED_BUFS buffers (full/empty mbarriers, like the weight ring).
            accA += __shfl_xor_sync(0xffffffffu, accA, 1);
            accB += __shfl_xor_sync(0xffffffffu, accB, 1);
            if (NB == 1) {
                accA += __shfl_xor_sync(0xffffffffu, accA, 2);
                accB += __shfl_xor_sync(0xffffffffu, accB, 2);
            }
            if (red_wrap > 0 && !dead && !mbar_wait_bounded(red_empty + rb, (uint32_t)((red_wrap & 1) ^ 1))) dead = true;
            float* rbuf = red + rb * (MV_MAX_CONSUMERS * 16 * NB);
            if (NB == 1) {
                if (cx.t == 0) {
                    rbuf[wl * 16 + pj] = accA;
                    rbuf[wl * 16 + 8 + pj] = accB;
                }
            } else if ((cx.t & 1) == 0) {  // t = 0 holds vector 0's sums, t = 2 vector 1's
                rbuf[(wl * 2 + (cx.t >> 1)) * 16 + pj] = accA;
                rbuf[(wl * 2 + (cx.t >> 1)) * 16 + 8 + pj] = accB;
            }
            __syncwarp();
            if (lane == 0 && !dead) mbar_arrive(red_full + rb);
            rb += CG;  // the buffer of this group's next tile (MV_RED_BUFS is even)
            if (rb >= MV_RED_BUFS) {
                rb -= MV_RED_BUFS;
                ++red_wrap;
            }
        }
        if (dead && lane == 0) atomicExch(p.status, DEV_ERR_TMA_TIMEOUT);
    } else {
        const float* xf = reinterpret_cast<const float*>(smem + L.off_xf);
        // f32 weights: one warp per row pair, weights read straight from global memory (they are L2-sized models)
        for (int j = warp; j < my_units; j += W) {
            const UnitInfo u = find_unit<false>(p, (int)blockIdx.x + j * (int)gridDim.x);
            const MvSegment sg = get_segment(p, u.seg);
            const int t = u.pair0;
            int rowA, rowB;
            pair_rows(p, sg, t, rowA, rowB);
            const float* baseB = reinterpret_cast<const float*>(sg.pair_mode == PAIR_DUAL ? sg.w2 : sg.w);
            const float4* wa = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(sg.w) + (size_t)rowA * p.n_in);
            const float4* wb = reinterpret_cast<const float4*>(baseB + (size_t)rowB * p.n_in);
            const float4* xv = reinterpret_cast<const float4*>(xf);
            const int n4 = p.n_in >> 2;
            float accA = 0.f, accB = 0.f;
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
    MV_TRACE(6);
    if (DBG && p.trace && threadIdx.x == 0) p.trace[blockIdx.x * 16 + 14] = (unsigned long long)my_units;

    if (!KQ && p.amax_val) {  // EPI_LOGITS (f32 weights): first maximal index over this block's rows
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best.v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best.i, o);
            arg_update(best, ov, oi);
        }
        __shared__ float sv[MV_MAX_CONSUMERS];
        __shared__ int sidx[MV_MAX_CONSUMERS];
        if (lane == 0) {
            sv[warp] = best.v;
            sidx[warp] = best.i;
        }
        consumer_sync(W * 32);
        if (threadIdx.x == 0) {
            ArgBest bb2 = {sv[0], sidx[0]};
            for (int w = 1; w < W; ++w) arg_update(bb2, sv[w], sidx[w]);
            p.amax_val[blockIdx.x] = bb2.v;
            p.amax_idx[blockIdx.x] = bb2.i;
        }
    }
}

}  // namespace l2b
