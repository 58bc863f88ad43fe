// k-quant weights x many activation vectors on the 5th-generation tensor cores (tcgen05): the dense GEMM that prompt
// prefill and batched matmul! need.  The reference feeds a prompt one token at a time through matmul! (src/matmul.jl:13-23,
// src/inference.jl:349-356); here 20 tokens share one pass over the weights, with the SAME exact integer arithmetic as the
// decode path (kquants.cuh): activations as three int8 planes, weights as their stored 4/5-bit integers, s32 accumulation.
//
//   Y[t][o] = sum_b ( d_ob * sum_j sc_obj * sum_p dpl_tbp * <q_obj, a_tbpj>  -  dmin_ob * sum_j m_obj * xs_tbj )
//
// with b the 256-value super-blocks of a row, j its eight 32-value sub-blocks, p the activation planes.
//
// One block = 128 weight rows x 20 tokens, walking the row's super-blocks:
//   producer warp   one TMA tiled copy (cp.async.bulk.tensor) brings the 128 packed super-blocks of this step (a
//                   128 x 144/176-byte box of the row-major matrix) and one bulk copy brings the step's activation planes
//                   (already in the tensor core's operand layout, written by quantise_rows_kernel) plus their scales;
//   unpack warps    thread r unpacks row r's nibbles (and fifth bits) to bytes into the canonical K-major operand layout
//                   (8-row x 16-byte core matrices), and decodes the row's 6-bit scales / mins and fp16 d / dmin;
//   MMA warp        one thread issues eight tcgen05.mma.kind::i8 (M 128, N 64, K 32), one per sub-block, each into its own
//                   64 columns of tensor memory: 8 x 64 = all 512 columns;
//   epilogue warps  thread = weight row: tcgen05.ld of the row's s32 dot products, times the sub-block scale (integer),
//                   then plane scales, d, and the dmin term in f32, accumulated over the super-blocks in registers.
// The tensor-memory accumulators are handed back to the MMA warp as soon as the integer part of the epilogue has read
// them, so the next step's MMAs overlap the float part.
//
// Every mbarrier wait is bounded; a wait that runs out sets the status word, after which the block drains and still frees
// its tensor memory.
#pragma once
#include <cuda.h>

#include "fused_matvec.cuh"

namespace l2b {

constexpr int GM_ROWS = 128;    // weight rows per block = MMA M
constexpr int GM_N = 64;        // MMA N: two halves of 32 columns, each 10 tokens x 3 planes + 2 unused columns
constexpr int GM_TOK = 20;      // tokens per block
constexpr int GM_HALF_TOK = 10;
constexpr int GM_STAGES = 3;
constexpr int GM_B_BYTES = 8 * GM_N * 32;              // activation operand of one super-block: 8 sub-blocks x (64 x 32) int8 = 16 KiB
constexpr int GM_SCALE_BYTES = 1024;                   // dpl[20][3] + xs[20][8] f32 = 880 bytes, padded
constexpr int GM_ACT_BYTES = GM_B_BYTES + GM_SCALE_BYTES;  // one (token chunk, super-block) record in global memory
constexpr int GM_A_TILE = GM_ROWS * 32;                // unpacked weights of one sub-block: 4 KiB
constexpr int GM_A_BYTES = 8 * GM_A_TILE;              // of one super-block: 32 KiB
constexpr int GM_EPI_WARPS = 8, GM_UNPACK_WARPS = 4;
constexpr int GM_THREADS = (GM_EPI_WARPS + 2 + GM_UNPACK_WARPS) * 32;  // warps 0-7 epilogue, 8 producer, 9 MMA, 10-13 unpack
enum : int { GM_STORE = 0, GM_RESIDUAL = 1 };

struct GmRowHdr {  // what the epilogue needs to know about one row's super-block
    float d, dmin;
    uint8_t sc[8], m[8];
};

struct GemmParams {
    int type;         // T_Q4_K or T_Q5_K
    int rows;         // weight rows (outputs)
    int nb;           // super-blocks per row
    int kb;           // super-blocks per stored column panel (nb when the matrix is not stored as panels)
    int n_tok;        // activation vectors
    const uint8_t* act;  // [chunks][nb] records of GM_ACT_BYTES (quantise_rows_kernel)
    float* y;         // [n_tok][ldy]
    const float* resid;  // GM_RESIDUAL: y = resid + W x (same indexing as y; may alias it)
    int ldy;
    int mode;
    int* status;
};

// ---- shared memory -----------------------------------------------------------------------------
struct GmSmem {
    int off_bar, off_tmem, off_hdr, off_au, off_stage, stage_bytes, packed_bytes, total;
};
__host__ __device__ inline GmSmem gm_smem_layout(int block_bytes) {
    GmSmem s;
    int o = 0;
    s.off_bar = o;  // full[3] stage_free[3] unpacked[2] mma_done[2] tmem_free[1]
    o += 16 * 8;
    s.off_tmem = o;
    o += 16;
    o = (o + 127) & ~127;
    s.off_hdr = o;  // [GM_STAGES][128] GmRowHdr: one set per ring stage, because a stage is refilled only after the epilogue
                    // of the step that used it has finished (a set per unpack buffer would be rewritten while still being read)
    o += GM_STAGES * GM_ROWS * (int)sizeof(GmRowHdr);
    o = (o + 1023) & ~1023;
    s.off_au = o;   // [2] unpacked weights
    o += 2 * GM_A_BYTES;
    s.packed_bytes = (GM_ROWS * block_bytes + 1023) & ~1023;
    s.stage_bytes = s.packed_bytes + GM_ACT_BYTES;
    s.off_stage = o;
    o += GM_STAGES * s.stage_bytes;
    s.total = o;
    return s;
}

// ---- tcgen05 / TMA wrappers ----------------------------------------------------------------------
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
                     smem_u32(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] = A[smem] * B[smem] (accumulate = 0: overwrite), u8 x s8 -> s32
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 consecutive columns of this thread's tensor-memory lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, int (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
        "%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices; lbo = bytes between the two 16-byte
// halves of the 32-byte K extent, sbo = bytes between consecutive 8-row groups.
__device__ __forceinline__ uint64_t umma_desc(const void* smem_ptr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(smem_ptr) >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version of this architecture
    return d;                // base offset 0, layout type 0 (no swizzle)
}
// Instruction descriptor: s32 accumulators, A unsigned 8-bit, B signed 8-bit, both K-major, N and M as given.
__host__ __device__ constexpr uint32_t umma_idesc_i8(int M, int N) {
    return (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// ---- activations: f32 rows -> int8 planes in operand layout --------------------------------------------
// One block per token.  Optional rmsnorm (src/inference.jl:102-110) as in the decode prologue: planes from gain .* x, 1/rms on
// the scales.  Record (chunk c = token / 20, super-block b) at act + (c * nb + b) * GM_ACT_BYTES:
//   bytes  [0, 16384)  B operand: sub-block j at j*2048; value k (0..31) of column n at (k/16)*1024 + (n/8)*128 + (n%8)*16 + k%16;
//                      column n = 32*(t/10) + 3*(t%10) + plane, t = token % 20
//   floats [0, 60)     dpl[t][plane];   floats [60, 220) xs[t][j] = sum of the represented activations of sub-block j
// Columns and tokens that do not exist must read as zero: the caller clears the buffer first.
struct QuantRowsParams {
    const float* x;     // [n_tok][ldx]
    const float* gain;  // rmsnorm gain, or null for none
    uint8_t* act;
    int n, ldx, n_tok;
};

__global__ void __launch_bounds__(512) quantise_rows_kernel(const __grid_constant__ QuantRowsParams p) {
    __shared__ float s_red[16];
    __shared__ float s_dpl[8 * 64];    // scratch of quantise_block for the block a warp works on: [warp][8]  (only [0..2] used)
    __shared__ float s_xs[16 * 16];    // [warp][16]
    __shared__ __align__(16) uint8_t s_act[16][3][256];
    const int tok = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int nb = p.n / QK_K;
    const float* x = p.x + (size_t)tok * p.ldx;
    float scale = 1.f;
    if (p.gain) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < p.n / 4; i += blockDim.x) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(x) + i);
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) s_red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int i = 0; i < nwarps; ++i) tot += s_red[i];
        scale = 1.0f / sqrtf(tot / (float)p.n + 1e-5f);
    }
    const int c = tok / GM_TOK, t = tok % GM_TOK;
    const int col0 = 32 * (t / GM_HALF_TOK) + 3 * (t % GM_HALF_TOK);
    for (int b = warp; b < nb; b += nwarps) {
        float4 a = __ldcg(reinterpret_cast<const float4*>(x + 256 * b + 8 * lane));
        float4 bq = __ldcg(reinterpret_cast<const float4*>(x + 256 * b + 8 * lane + 4));
        if (p.gain) {
            const float4 ga = __ldg(reinterpret_cast<const float4*>(p.gain + 256 * b + 8 * lane));
            const float4 gb = __ldg(reinterpret_cast<const float4*>(p.gain + 256 * b + 8 * lane + 4));
            a.x *= ga.x; a.y *= ga.y; a.z *= ga.z; a.w *= ga.w;
            bq.x *= gb.x; bq.y *= gb.y; bq.z *= gb.z; bq.w *= gb.w;
        }
        // quantise into this warp's scratch (block index 0 of a one-block vector), then scatter into the operand layout
        quantise_block<3, 8>(a, bq, lane, &s_act[warp][0][0], 256, s_dpl + warp * 8, s_xs + warp * 16, 0);
        __syncwarp();
        uint8_t* rec = p.act + ((size_t)c * nb + b) * GM_ACT_BYTES;
        const int j = lane >> 2, kk = 8 * (lane & 3);  // this lane's 8 values: sub-block j, k = kk .. kk+7
#pragma unroll
        for (int pl = 0; pl < 3; ++pl) {
            const int n = col0 + pl;
            const uint2 v = *reinterpret_cast<const uint2*>(&s_act[warp][pl][8 * lane]);
            *reinterpret_cast<uint2*>(rec + j * 2048 + (kk >> 4) * 1024 + (n >> 3) * 128 + (n & 7) * 16 + (kk & 15)) = v;
        }
        float* sc = reinterpret_cast<float*>(rec + GM_B_BYTES);
        if (lane < 3) sc[t * 3 + lane] = s_dpl[warp * 8 + lane] * scale;
        if (lane < 8) sc[60 + t * 8 + lane] = (s_xs[warp * 16 + 2 * lane] + s_xs[warp * 16 + 2 * lane + 1]) * scale;
        __syncwarp();
    }
}

// ---- the GEMM ----------------------------------------------------------------------------------------
// Grid (row tiles, token chunks).  tmap_main: the matrix as [panels][rows][kb * block bytes] (one panel when it is stored row
// by row); tmap_tail: the last, narrower panel when nb is not a multiple of kb.
__global__ void __launch_bounds__(GM_THREADS, 1) kq_gemm_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ CUtensorMap tmap_main,
                                                                const __grid_constant__ CUtensorMap tmap_tail) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);  // the copies and operands want their alignment
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bb = dev_block_bytes(p.type);
    const GmSmem L = gm_smem_layout(bb);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.off_bar);
    uint64_t* stage_free = full + GM_STAGES;
    uint64_t* unpacked = stage_free + GM_STAGES;
    uint64_t* mma_done = unpacked + 2;
    uint64_t* tmem_free = mma_done + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L.off_tmem);
    GmRowHdr* hdr = reinterpret_cast<GmRowHdr*>(smem + L.off_hdr);
    uint8_t* au = smem + L.off_au;
    uint8_t* stages = smem + L.off_stage;
    const int row0 = blockIdx.x * GM_ROWS, chunk = blockIdx.y;
    const int nb = p.nb;

    if (threadIdx.x == 0) {
        for (int i = 0; i < GM_STAGES; ++i) {
            mbar_init(full + i, 1);
            mbar_init(stage_free + i, GM_EPI_WARPS);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(unpacked + i, GM_UNPACK_WARPS);
            mbar_init(mma_done + i, 1);
        }
        mbar_init(tmem_free, GM_EPI_WARPS);
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 9) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 8) {
        // ================= producer: one tiled copy of packed weights + one bulk copy of activations per step =================
        if (lane == 0) {
            const uint64_t policy = policy_evict_first();
            const int full_panels = nb / p.kb;
            bool ok = true;
            for (int b = 0; b < nb && ok; ++b) {
                const int s = b % GM_STAGES, use = b / GM_STAGES;
                if (use > 0 && !mbar_wait_bounded(stage_free + s, (uint32_t)((use - 1) & 1))) {
                    ok = false;
                    break;
                }
                uint8_t* st = stages + (size_t)s * L.stage_bytes;
                mbar_arrive_expect_tx(full + s, (uint32_t)(GM_ROWS * bb + GM_ACT_BYTES));
                const int panel = b / p.kb;
                if (panel < full_panels) tma_load_3d(st, &tmap_main, (b - panel * p.kb) * bb, row0, panel, full + s);
                else tma_load_3d(st, &tmap_tail, (b - panel * p.kb) * bb, row0, 0, full + s);
                bulk_g2s(st + L.packed_bytes, p.act + ((size_t)chunk * nb + b) * GM_ACT_BYTES, GM_ACT_BYTES, full + s, policy);
            }
            if (!ok) {
                atomicExch(p.status, DEV_ERR_TMA_TIMEOUT);
                for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // copies in flight land within microseconds
            }
        }
    } else if (warp == 9) {
        // ================= MMA issue: eight K = 32 products per step, one per sub-block, into 8 x 64 columns =================
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_i8(GM_ROWS, GM_N);
            bool ok = true;
            for (int b = 0; b < nb && ok; ++b) {
                const int s = b % GM_STAGES, buf = b & 1;
                if (!mbar_wait_bounded(unpacked + buf, (uint32_t)((b >> 1) & 1))) ok = false;       // weights unpacked (and the stage has landed)
                if (ok && b > 0 && !mbar_wait_bounded(tmem_free, (uint32_t)((b - 1) & 1))) ok = false;  // the epilogue has read step b-1
                if (!ok) break;
                tc_fence_after();
                const uint8_t* a_base = au + (size_t)buf * GM_A_BYTES;
                const uint8_t* b_base = stages + (size_t)s * L.stage_bytes + L.packed_bytes;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    umma_i8(tmem_base + (uint32_t)(j * GM_N), umma_desc(a_base + j * GM_A_TILE, 16 * 128, 128), umma_desc(b_base + j * 2048, 8 * 128, 128),
                            idesc, 0u);
                umma_commit(mma_done + buf);
            }
            if (!ok) atomicExch(p.status, DEV_ERR_TMA_TIMEOUT);
        }
    } else if (warp >= 10) {
        // ================= unpack: thread r turns row r's packed quants into bytes in operand layout =================
        const int r = threadIdx.x - 10 * 32;  // 0..127
        bool ok = true;
        for (int b = 0; b < nb; ++b) {
            const int s = b % GM_STAGES, buf = b & 1;
            if (ok && b >= 2 && !mbar_wait_bounded(mma_done + buf, (uint32_t)(((b - 2) >> 1) & 1))) ok = false;  // the MMAs of step b-2 have read this buffer
            if (ok && !mbar_wait_bounded(full + s, (uint32_t)((b / GM_STAGES) & 1))) ok = false;
            if (ok) {
                const uint8_t* blk = stages + (size_t)s * L.stage_bytes + (size_t)r * bb;
                const uint4 h = *reinterpret_cast<const uint4*>(blk);
                uint64_t sc8, m8;
                decode_scales_k4(h, sc8, m8);
                GmRowHdr hd;
                hd.d = half_bits_to_float(h.x & 0xFFFFu);
                hd.dmin = half_bits_to_float(h.x >> 16);
                *reinterpret_cast<uint64_t*>(hd.sc) = sc8;
                *reinterpret_cast<uint64_t*>(hd.m) = m8;
                hdr[s * GM_ROWS + r] = hd;
                uint8_t* dst = au + (size_t)buf * GM_A_BYTES + (r >> 3) * 128 + (r & 7) * 16;
                const uint8_t* qs = blk + (p.type == T_Q5_K ? 48 : 16);
                uint4 qh0 = make_uint4(0u, 0u, 0u, 0u), qh1 = qh0;
                if (p.type == T_Q5_K) {  // fifth bits of values l = 0..15 and 16..31 of every sub-block: bit j of byte qh[l]
                    qh0 = *reinterpret_cast<const uint4*>(blk + 16);
                    qh1 = *reinterpret_cast<const uint4*>(blk + 32);
                }
#pragma unroll
                for (int pr = 0; pr < 4; ++pr) {
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const uint4 v = *reinterpret_cast<const uint4*>(qs + 32 * pr + 16 * hh);
                        const uint4 q5 = hh ? qh1 : qh0;
                        uint4 lo, hi;
                        lo.x = (v.x & 0x0f0f0f0fu) | (((q5.x >> (2 * pr)) & 0x01010101u) << 4);
                        lo.y = (v.y & 0x0f0f0f0fu) | (((q5.y >> (2 * pr)) & 0x01010101u) << 4);
                        lo.z = (v.z & 0x0f0f0f0fu) | (((q5.z >> (2 * pr)) & 0x01010101u) << 4);
                        lo.w = (v.w & 0x0f0f0f0fu) | (((q5.w >> (2 * pr)) & 0x01010101u) << 4);
                        hi.x = ((v.x >> 4) & 0x0f0f0f0fu) | (((q5.x >> (2 * pr + 1)) & 0x01010101u) << 4);
                        hi.y = ((v.y >> 4) & 0x0f0f0f0fu) | (((q5.y >> (2 * pr + 1)) & 0x01010101u) << 4);
                        hi.z = ((v.z >> 4) & 0x0f0f0f0fu) | (((q5.z >> (2 * pr + 1)) & 0x01010101u) << 4);
                        hi.w = ((v.w >> 4) & 0x0f0f0f0fu) | (((q5.w >> (2 * pr + 1)) & 0x01010101u) << 4);
                        *reinterpret_cast<uint4*>(dst + (2 * pr) * GM_A_TILE + hh * (16 * 128)) = lo;      // sub-block 2*pr, values 16*hh ..
                        *reinterpret_cast<uint4*>(dst + (2 * pr + 1) * GM_A_TILE + hh * (16 * 128)) = hi;  // sub-block 2*pr + 1
                    }
                }
                fence_proxy_async();  // the tensor core reads shared memory through the asynchronous proxy
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(unpacked + buf);
        }
        if (!ok && lane == 0) atomicExch(p.status, DEV_ERR_TMA_TIMEOUT);
    } else {
        // ================= epilogue: thread = weight row; warps e and e + 4 split the tokens =================
        const int q = warp & 3, half = warp >> 2;
        const int r = 32 * q + lane;
        const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(32 * half);
        float acc[GM_HALF_TOK];
#pragma unroll
        for (int t = 0; t < GM_HALF_TOK; ++t) acc[t] = 0.f;
        bool ok = true;
        for (int b = 0; b < nb; ++b) {
            const int s = b % GM_STAGES, buf = b & 1;
            if (ok && !mbar_wait_bounded(mma_done + buf, (uint32_t)((b >> 1) & 1))) ok = false;
            if (ok) {
                tc_fence_after();
                const GmRowHdr hd = hdr[s * GM_ROWS + r];
                int S[3 * GM_HALF_TOK];
#pragma unroll
                for (int n = 0; n < 3 * GM_HALF_TOK; ++n) S[n] = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    int c[32];
                    tmem_ld32(taddr + (uint32_t)(j * GM_N), c);
                    const int sc = hd.sc[j];
#pragma unroll
                    for (int n = 0; n < 3 * GM_HALF_TOK; ++n) S[n] += sc * c[n];
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tmem_free);  // the accumulators may be overwritten by the next step
                const float* scl = reinterpret_cast<const float*>(stages + (size_t)s * L.stage_bytes + L.packed_bytes + GM_B_BYTES);
                float mf[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) mf[j] = (float)hd.m[j];
#pragma unroll
                for (int t = 0; t < GM_HALF_TOK; ++t) {
                    const int tt = GM_HALF_TOK * half + t;
                    const float f = fmaf(scl[tt * 3], (float)S[3 * t], fmaf(scl[tt * 3 + 1], (float)S[3 * t + 1], scl[tt * 3 + 2] * (float)S[3 * t + 2]));
                    float mt = 0.f;
#pragma unroll
                    for (int j = 0; j < 8; ++j) mt = fmaf(mf[j], scl[60 + tt * 8 + j], mt);
                    acc[t] += hd.d * f - hd.dmin * mt;
                }
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(stage_free + s);
        }
        if (!ok && lane == 0) atomicExch(p.status, DEV_ERR_TMA_TIMEOUT);
        const int row = row0 + r;
        if (ok && row < p.rows) {
#pragma unroll
            for (int t = 0; t < GM_HALF_TOK; ++t) {
                const int tok = chunk * GM_TOK + GM_HALF_TOK * half + t;
                if (tok < p.n_tok) {
                    const size_t o = (size_t)tok * p.ldy + row;
                    p.y[o] = p.mode == GM_RESIDUAL ? p.resid[o] + acc[t] : acc[t];
                }
            }
        }
    }
    // every path ends here; the tensor memory is freed by the warp that allocated it
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem_base, 512);
}

}  // namespace l2b
