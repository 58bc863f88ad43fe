// Small kernels behind the isolated-operator entry points and the upload path.  Dequantisation, the activation
// prologue (export_activation_kernel) and the epilogues (epilogue_probe_kernel: RoPE, SwiGLU) call the very device
// functions the fused decode kernels call, so a parity test of those entry points tests the token path's arithmetic.
#pragma once
#include "fused_matvec.cuh"

namespace l2b {

// q6_K file blocks (210 bytes: ql qh scales d) -> 208-byte records + fp16 scale array.
__global__ void repack_q6k_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ rec, __half* __restrict__ d, int64_t nblocks) {
    const int64_t total = nblocks * 105;  // 105 half-words per block
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / 105;
        const int w = (int)(i % 105);
        const uint16_t v = reinterpret_cast<const uint16_t*>(src)[b * 105 + w];  // 210*b is even
        if (w < 104) reinterpret_cast<uint16_t*>(rec)[b * 104 + w] = v;
        else d[b] = __ushort_as_half(v);
    }
}

// Matrices whose rows are longer than one stage (more than kb super-blocks, kb = 16 or 8) are stored as column panels: panel k
// holds blocks kb*k .. kb*k+kb-1 of EVERY row, rows back to back.  A tile's stage is then 16 adjacent rows of one panel, which a
// few large bulk copies bring in, instead of 16 row slices that lie a whole row apart.  Same bytes, other order.
//   address(row, block b) = (b / kb) * rows * kb * bb  +  row * w * bb  +  (b % kb) * bb,   w = width of panel b / kb
__global__ void panelize_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int nb, int64_t rows, int bb, int kb) {
    const int q = bb / 16;  // 16-byte units per block
    const int64_t total = rows * nb * q;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t blk = i / q;
        const int u = (int)(i % q);
        const int64_t r = blk / nb;
        const int b = (int)(blk % nb);
        const int k = b / kb, w = min(kb, nb - kb * k);
        const int64_t o = (int64_t)k * rows * kb + r * w + (b % kb);
        reinterpret_cast<uint4*>(dst)[o * q + u] = reinterpret_cast<const uint4*>(src)[i];
    }
}

// dequantize! of n values from device-layout blocks.
__global__ void dequantize_kernel(int type, const uint8_t* __restrict__ blocks, const __half* __restrict__ d6, int64_t n, float* __restrict__ out) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i >> 8;
        const int k = (int)(i & 255);
        const uint8_t* blk = blocks + b * dev_block_bytes(type);
        float v;
        if (type == T_Q4_K) v = dequant_q45<false>(blk, k);
        else if (type == T_Q5_K) v = dequant_q45<true>(blk, k);
        else v = dequant_q6(blk, __half2float(d6[b]), k);
        out[i] = v;
    }
}

// x = dequantize!(x, token_embedding_table[:, token]) (src/inference.jl:236): the first kernel of a token.
// `token` is a device scalar.  For f32 tables the row is copied.
// `prompt` non-null: the row of the NEXT prompt token, prompt[*pos + 1] (second position of a two-position pass).
// A token id outside [0, vocab) gives a row of zeros (the table is never read out of bounds).
__global__ void embed_row_kernel(int type, const uint8_t* __restrict__ table, const __half* __restrict__ d6, const int* token, int n, float* __restrict__ x,
                                 const int* prompt, const int* pos, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const int tok = prompt ? __ldcg(prompt + __ldcg(pos) + 1) : __ldcg(token);
    const bool valid = tok >= 0 && tok < vocab;
    const int nb = n / QK_K;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float v;
        if (!valid) {
            v = 0.f;
        } else if (type == T_F32) {
            v = reinterpret_cast<const float*>(table)[(size_t)tok * n + i];
        } else {
            const int b = i >> 8, k = i & 255;
            const uint8_t* blk = table + ((size_t)tok * nb + b) * dev_block_bytes(type);
            if (type == T_Q4_K) v = dequant_q45<false>(blk, k);
            else if (type == T_Q5_K) v = dequant_q45<true>(blk, k);
            else v = dequant_q6(blk, __half2float(d6[(size_t)tok * nb + b]), k);
        }
        x[i] = v;
    }
}

// Runs the prologue of the fused kernel on one block and exports what it built.
// KQ: planes -> q [P][n] int8, dsc [P][n/256], sums [n/16].  else: the f32 vector.
template <bool KQ, int P>
__global__ void __launch_bounds__(256) export_activation_kernel(const __grid_constant__ MvParams p, int8_t* q_out, float* d_out, float* sums_out,
                                                                 float* f_out) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const MvSmem L = mv_smem_layout(p.n_in, P, KQ, 0, 0);
    build_activation<KQ, P>(p, smem, L, warp, lane, nwarps, p.x_in, smem + L.off_act, reinterpret_cast<float*>(smem + L.off_dpl),
                            reinterpret_cast<float*>(smem + L.off_xs));
    const int n = p.n_in, nb = n / QK_K;
    if (KQ) {
        for (int i = threadIdx.x; i < P * n; i += blockDim.x) {
            const int k = i / n, e = i % n;
            q_out[i] = (int8_t)smem[L.off_act + k * L.plane_stride + e];
        }
        for (int i = threadIdx.x; i < P * nb; i += blockDim.x) {
            const int k = i / nb, b = i % nb;
            d_out[i] = reinterpret_cast<const float*>(smem + L.off_dpl)[8 * b + k];
        }
        for (int i = threadIdx.x; i < nb * 16; i += blockDim.x) sums_out[i] = reinterpret_cast<const float*>(smem + L.off_xs)[i];
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) f_out[i] = reinterpret_cast<const float*>(smem + L.off_xf)[i];
    }
}

// Runs the fused kernel's epilogue (epilogue_pair, with the operands preloaded as the finisher warp does) on given
// matvec results: pair t of segment 0 takes vin[rowA], vin[rowB] (adjacent / NeoX pairs) or vin[t], vin2[t] (gate / up).
// Behind l2b_rope (EPI_ROPE_Q) and l2b_swiglu (EPI_SWIGLU).
__global__ void epilogue_probe_kernel(const __grid_constant__ MvParams p, const float* __restrict__ vin, const float* __restrict__ vin2, int pos) {
    const MvSegment sg = p.seg[0];
    ArgBest best;
    best.v = -INFINITY;
    best.i = 0x7fffffff;
    for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < sg.npairs; t += gridDim.x * blockDim.x) {
        const EpiPre pre = epilogue_preload(p, sg, t, pos);
        const float vA = sg.pair_mode == PAIR_DUAL ? vin[t] : vin[pre.rowA];
        const float vB = sg.pair_mode == PAIR_DUAL ? vin2[t] : vin[pre.rowB];
        epilogue_pair<false, true>(p, sg, t, vA, vB, pos, best, 0, &pre);
    }
}

}  // namespace l2b
