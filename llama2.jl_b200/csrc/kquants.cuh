// k-quant super-block arithmetic on the device.
//
// Two families live here:
//  (1) exact dequantisation of one weight, bit-for-bit what the reference's dequantize!
//      produces (src/kquants.jl:70-125, 186-251, 322-363): products and the subtraction are
//      rounded separately (__fmul_rn / __fsub_rn block FMA contraction);
//  (2) integer dot products of one super-block column of a 16-row weight tile against int8
//      activation planes held in shared memory.  The algebra is the reference's vecdot
//      (src/kquants.jl:127-184, 253-320, 365-408) factorised per sub-block:
//          sum_k x_k (d sc q_k - dmin m) = d sc sum_k x_k q_k  -  dmin m sum_k x_k
//      with x_k represented as sum_p dplane_p * a_{p,k}, a int8 (1..3 planes), so that the
//      inner sums are exact integer dot products (int8 tensor-core MMA, s32 accumulate).
#pragma once
#include "common.cuh"

namespace l2b {

// ---- (1) exact dequantisation --------------------------------------------------------

// 6-bit scale and min of sub-block j of a q4_K/q5_K block; s = the 12 scale bytes.
// src/kquants.jl:80-81,86-87,102-103,108-109.
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* s, int& sc, int& m) {
    if (j < 4) {
        sc = s[j] & 63;
        m = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
        m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

// Weight k (0..255) of a q4_K (bits5 = false) or q5_K (bits5 = true) block in device layout.
template <bool bits5>
__device__ __forceinline__ float dequant_q45(const uint8_t* blk, int k) {
    const float d = half_bits_to_float(blk[0] | (blk[1] << 8));
    const float dmin = half_bits_to_float(blk[2] | (blk[3] << 8));
    const int p = k >> 6, hi = (k >> 5) & 1, l = k & 31;
    int sc, m;
    scale_min_k4(2 * p + hi, blk + 4, sc, m);
    const uint8_t* qs = blk + (bits5 ? 48 : 16);
    int q = hi ? (qs[32 * p + l] >> 4) : (qs[32 * p + l] & 0xF);
    if (bits5) q += (blk[16 + l] & (1 << (2 * p + hi))) ? 16 : 0;
    const float d1 = __fmul_rn(d, (float)sc);
    const float m1 = __fmul_rn(dmin, (float)m);
    return __fsub_rn(__fmul_rn(d1, (float)q), m1);
}

// Weight k of a q6_K block: rec = 208-byte record (ql[128] qh[64] scales[16]), d = its fp16 scale.
// src/kquants.jl:331-358: fl(d * float(scale * q)).
__device__ __forceinline__ float dequant_q6(const uint8_t* rec, float d, int k) {
    const int n = k >> 7, quad = (k >> 5) & 3, l = k & 31;
    const int is = 8 * n + (l >> 4) + 2 * quad;
    const uint8_t qlb = rec[64 * n + l + ((quad & 1) ? 32 : 0)];
    const int nib = (quad >= 2) ? (qlb >> 4) : (qlb & 0xF);
    const int hb = (rec[128 + 32 * n + l] >> (2 * quad)) & 3;
    const int q = (nib | (hb << 4)) - 32;
    const int sc = (int)(int8_t)rec[192 + is];
    return __fmul_rn(d, (float)(sc * q));
}

// ---- (2) tile dot products on the int8 tensor-core path --------------------------------------
//
// A warp multiplies one super-block column of a 16-row weight tile with the activation planes:
// the unpacked quants of 16 rows x 32 values (one sub-block) are the A operand of
// mma.sync.m16n8k32 (u8), the int8 activation planes are the columns of the B operand (s8), and
// the s32 result holds, per row and plane, the exact integer dot product of the sub-block.  The
// 6-bit sub-block scale is applied to that integer, the fp16 super-block scale and the plane scale
// afterwards in f32.  The instruction count per weight no longer grows with the number of planes.
//
// Fragment ownership (PTX ISA, mma.m16n8k32 with 8-bit operands), lane = 4*g + t:
//   A: a0 = row g,   k 4t..4t+3     a1 = row g+8, k 4t..4t+3     a2 = row g,   k 16+4t..   a3 = row g+8, k 16+4t..
//   B: b0 = k 4t..4t+3, column g    b1 = k 16+4t.., column g
//   C: c0,c1 = row g, columns 2t,2t+1    c2,c3 = row g+8, columns 2t,2t+1
// Any permutation of k is allowed if A and B use the same one: lane t takes the eight consecutive
// values 8t..8t+7 of a sub-block (one 64-bit load of quants, one of activations).
//
// Shared-memory layout of the activations (see ActLayout): plane p holds int8 value i at
// p*plane_stride + i; dpl[b*8 + c] is the f32 scale of column c (plane) for block b, 0 for unused
// columns; xs16[b*16 + j] is the f32 sum of the represented activations over values 16j..16j+15.

__device__ __forceinline__ void mma_u8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_u8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// The eight 6-bit scales and eight 6-bit mins of a q4_K / q5_K block as bytes of 64-bit words.
// src/kquants.jl:80-81,86-87 (sub-blocks 0..3) and :102-103,108-109 (4..7).
__device__ __forceinline__ void decode_scales_k4(const uint4& hd, uint64_t& sc8, uint64_t& m8) {
    const uint32_t sc_lo = hd.y & 0x3f3f3f3fu, m_lo = hd.z & 0x3f3f3f3fu;
    const uint32_t sc_hi = (hd.w & 0x0f0f0f0fu) | ((hd.y >> 2) & 0x30303030u);
    const uint32_t m_hi = ((hd.w >> 4) & 0x0f0f0f0fu) | ((hd.z >> 2) & 0x30303030u);
    sc8 = ((uint64_t)sc_hi << 32) | sc_lo;
    m8 = ((uint64_t)m_hi << 32) | m_lo;
}
__device__ __forceinline__ int byte64(uint64_t w, int i) { return (int)((w >> (8 * i)) & 0xFFull); }

struct TileCtx {
    const uint8_t* act;  // the activation plane carried by this lane's MMA column g (meaningful when colv)
    const float* dpl;    // [nb][8] plane scales
    const float* xs16;   // [nb][16]
    int g, t;            // lane = 4*g + t
    bool colv;           // this lane's column g carries an activation plane
};

// Which plane rides in which MMA column.  One vector per launch (NB = 1): plane k in column 2k, so that every lane t holds
// exactly one useful result column (2t: c[0] for row g, c[2] for row g+8) and applies the sub-block scale to two integers
// instead of four; the odd columns are zero.  Two vectors (NB = 2): planes of vector v in columns 4v .. 4v+2, lanes t = 0, 1
// collect vector 0 and t = 2, 3 vector 1.
template <int NB, int P>
__device__ __forceinline__ void tile_ctx_columns(TileCtx& cx, const uint8_t* planes, int plane_stride, int lane) {
    cx.g = lane >> 2;
    cx.t = lane & 3;
    if (NB == 1) {
        cx.colv = !(cx.g & 1) && (cx.g >> 1) < P;
        cx.act = planes + (cx.g >> 1) * plane_stride;
    } else {
        cx.colv = (cx.g & 3) < P;
        cx.act = planes + ((cx.g >> 2) * P + (cx.g & 3)) * plane_stride;
    }
}

template <int NB>
__device__ __forceinline__ void scale_add(int (&S)[4], int sa, int sb, const int (&c)[4]) {
    S[0] += sa * c[0];
    S[2] += sb * c[2];
    if (NB != 1) {
        S[1] += sa * c[1];
        S[3] += sb * c[3];
    }
}

// integer sums -> f32, times the scale of the plane(s) this lane holds
template <int NB>
__device__ __forceinline__ void plane_scale(const TileCtx& x, int b, const int (&S)[4], float& fA, float& fB) {
    if (NB == 1) {
        const float dp = x.dpl[8 * b + x.t];  // 0 for t >= planes
        fA = dp * (float)S[0];
        fB = dp * (float)S[2];
    } else {
        const float2 dp = *reinterpret_cast<const float2*>(x.dpl + 8 * b + 2 * x.t);
        fA = fmaf(dp.x, (float)S[0], dp.y * (float)S[1]);
        fB = fmaf(dp.x, (float)S[2], dp.y * (float)S[3]);
    }
}

// sum over this lane's two sub-blocks (2t, 2t+1) of m_s * sum(activations of sub-block s)
__device__ __forceinline__ float min_term_lane(uint64_t m8, const float* xs16b, int t) {
    const float4 v = *reinterpret_cast<const float4*>(xs16b + 4 * t);
    return fmaf((float)byte64(m8, 2 * t), v.x + v.y, (float)byte64(m8, 2 * t + 1) * (v.z + v.w));
}

// Two activation vectors per launch (NB = 2): lanes t = 0, 1 work for the first vector, t = 2, 3 for the second, so a
// lane covers half of the block's sub-blocks: 4h .. 4h+3 with h = t & 1 (xs16b already points at the lane's vector).
__device__ __forceinline__ float min_term_half(uint64_t m8, const float* xs16b, int h) {
    const float4 v0 = *reinterpret_cast<const float4*>(xs16b + 8 * h);
    const float4 v1 = *reinterpret_cast<const float4*>(xs16b + 8 * h + 4);
    float r = (float)byte64(m8, 4 * h) * (v0.x + v0.y);
    r = fmaf((float)byte64(m8, 4 * h + 1), v0.z + v0.w, r);
    r = fmaf((float)byte64(m8, 4 * h + 2), v1.x + v1.y, r);
    r = fmaf((float)byte64(m8, 4 * h + 3), v1.z + v1.w, r);
    return r;
}

// q4_K: rA, rB = this block of rows g and g+8 (144-byte blocks); b = block index along the row.
template <int NB = 1>
__device__ __forceinline__ void tile_q4k(const uint8_t* rA, const uint8_t* rB, int b, const TileCtx& x, float& accA, float& accB) {
    const uint4 hA = *reinterpret_cast<const uint4*>(rA);
    const uint4 hB = *reinterpret_cast<const uint4*>(rB);
    uint64_t scA, mA, scB, mB;
    decode_scales_k4(hA, scA, mA);
    decode_scales_k4(hB, scB, mB);
    const uint8_t* ap = x.act + 256 * b + 8 * x.t;
    int S[4] = {0, 0, 0, 0};
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const uint2 wA = *reinterpret_cast<const uint2*>(rA + 16 + 32 * p + 8 * x.t);
        const uint2 wB = *reinterpret_cast<const uint2*>(rB + 16 + 32 * p + 8 * x.t);
        uint2 be = make_uint2(0u, 0u), bo = make_uint2(0u, 0u);
        if (x.colv) {
            be = *reinterpret_cast<const uint2*>(ap + 64 * p);
            bo = *reinterpret_cast<const uint2*>(ap + 64 * p + 32);
        }
        int c[4];
        // sub-block 2p: low nibbles.  Its scale is taken x16 so that it matches the high nibbles left in place below.
        mma_u8s8_k32(c, wA.x & 0x0f0f0f0fu, wB.x & 0x0f0f0f0fu, wA.y & 0x0f0f0f0fu, wB.y & 0x0f0f0f0fu, be.x, be.y);
        int sa = byte64(scA, 2 * p) << 4, sb = byte64(scB, 2 * p) << 4;
        scale_add<NB>(S, sa, sb, c);
        // sub-block 2p+1: high nibbles, 16 * q
        mma_u8s8_k32(c, wA.x & 0xf0f0f0f0u, wB.x & 0xf0f0f0f0u, wA.y & 0xf0f0f0f0u, wB.y & 0xf0f0f0f0u, bo.x, bo.y);
        sa = byte64(scA, 2 * p + 1); sb = byte64(scB, 2 * p + 1);
        scale_add<NB>(S, sa, sb, c);
    }
    float fA, fB;
    plane_scale<NB>(x, b, S, fA, fB);
    const float dA = half_bits_to_float(hA.x & 0xFFFFu), dminA = half_bits_to_float(hA.x >> 16);
    const float dB = half_bits_to_float(hB.x & 0xFFFFu), dminB = half_bits_to_float(hB.x >> 16);
    if (NB == 1) {
        accA += dA * 0.0625f * fA - dminA * min_term_lane(mA, x.xs16 + 16 * b, x.t);
        accB += dB * 0.0625f * fB - dminB * min_term_lane(mB, x.xs16 + 16 * b, x.t);
    } else {
        accA += dA * 0.0625f * fA - dminA * min_term_half(mA, x.xs16 + 16 * b, x.t & 1);
        accB += dB * 0.0625f * fB - dminB * min_term_half(mB, x.xs16 + 16 * b, x.t & 1);
    }
}

// q5_K: 176-byte blocks: header 16 | qh 32 | qs 128.
template <int NB = 1>
__device__ __forceinline__ void tile_q5k(const uint8_t* rA, const uint8_t* rB, int b, const TileCtx& x, float& accA, float& accB) {
    const uint4 hA = *reinterpret_cast<const uint4*>(rA);
    const uint4 hB = *reinterpret_cast<const uint4*>(rB);
    uint64_t scA, mA, scB, mB;
    decode_scales_k4(hA, scA, mA);
    decode_scales_k4(hB, scB, mB);
    // fifth bits of values l = 8t..8t+7 of every sub-block: bit s of byte qh[l]
    const uint2 qA = *reinterpret_cast<const uint2*>(rA + 16 + 8 * x.t);
    const uint2 qB = *reinterpret_cast<const uint2*>(rB + 16 + 8 * x.t);
    const uint8_t* ap = x.act + 256 * b + 8 * x.t;
    int S[4] = {0, 0, 0, 0};
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const uint2 wA = *reinterpret_cast<const uint2*>(rA + 48 + 32 * p + 8 * x.t);
        const uint2 wB = *reinterpret_cast<const uint2*>(rB + 48 + 32 * p + 8 * x.t);
        uint2 be = make_uint2(0u, 0u), bo = make_uint2(0u, 0u);
        if (x.colv) {
            be = *reinterpret_cast<const uint2*>(ap + 64 * p);
            bo = *reinterpret_cast<const uint2*>(ap + 64 * p + 32);
        }
        int c[4];
        mma_u8s8_k32(c, (wA.x & 0x0f0f0f0fu) | (((qA.x >> (2 * p)) & 0x01010101u) << 4), (wB.x & 0x0f0f0f0fu) | (((qB.x >> (2 * p)) & 0x01010101u) << 4),
                     (wA.y & 0x0f0f0f0fu) | (((qA.y >> (2 * p)) & 0x01010101u) << 4), (wB.y & 0x0f0f0f0fu) | (((qB.y >> (2 * p)) & 0x01010101u) << 4), be.x, be.y);
        int sa = byte64(scA, 2 * p), sb = byte64(scB, 2 * p);
        scale_add<NB>(S, sa, sb, c);
        mma_u8s8_k32(c, ((wA.x >> 4) & 0x0f0f0f0fu) | (((qA.x >> (2 * p + 1)) & 0x01010101u) << 4),
                     ((wB.x >> 4) & 0x0f0f0f0fu) | (((qB.x >> (2 * p + 1)) & 0x01010101u) << 4),
                     ((wA.y >> 4) & 0x0f0f0f0fu) | (((qA.y >> (2 * p + 1)) & 0x01010101u) << 4),
                     ((wB.y >> 4) & 0x0f0f0f0fu) | (((qB.y >> (2 * p + 1)) & 0x01010101u) << 4), bo.x, bo.y);
        sa = byte64(scA, 2 * p + 1); sb = byte64(scB, 2 * p + 1);
        scale_add<NB>(S, sa, sb, c);
    }
    float fA, fB;
    plane_scale<NB>(x, b, S, fA, fB);
    const float dA = half_bits_to_float(hA.x & 0xFFFFu), dminA = half_bits_to_float(hA.x >> 16);
    const float dB = half_bits_to_float(hB.x & 0xFFFFu), dminB = half_bits_to_float(hB.x >> 16);
    if (NB == 1) {
        accA += dA * fA - dminA * min_term_lane(mA, x.xs16 + 16 * b, x.t);
        accB += dB * fB - dminB * min_term_lane(mB, x.xs16 + 16 * b, x.t);
    } else {
        accA += dA * fA - dminA * min_term_half(mA, x.xs16 + 16 * b, x.t & 1);
        accB += dB * fB - dminB * min_term_half(mB, x.xs16 + 16 * b, x.t & 1);
    }
}

// q6_K: 208-byte records (ql[128] qh[64] scales[16]); dA, dB = the blocks' fp16 scales.  Scales cover 16 values,
// so the products run on m16n8k16.  Quants stay unsigned 0..63; the -32 offset becomes -32 * scale * (sum of
// the activations of the group).  Lane t takes values l = 16c + 4t .. 16c + 4t + 3 of every group.
template <int NB = 1>
__device__ __forceinline__ void tile_q6k(const uint8_t* rA, const uint8_t* rB, float dA, float dB, int b, const TileCtx& x, float& accA, float& accB) {
    const uint4 sA4 = *reinterpret_cast<const uint4*>(rA + 192);
    const uint4 sB4 = *reinterpret_cast<const uint4*>(rB + 192);
    const uint32_t scwA[4] = {sA4.x, sA4.y, sA4.z, sA4.w}, scwB[4] = {sB4.x, sB4.y, sB4.z, sB4.w};
    // int8 scale number `is`, sign-extended by one byte permute (selector nibble 8 + i replicates the sign bit of byte i)
    // (prmt in PTX: the __byte_perm intrinsic ignores the sign-replication bit of a selector nibble)
    auto sc_of = [](const uint32_t (&w)[4], int is) -> int {
        const unsigned i = (unsigned)(is & 3), sgn = 8u + i;
        int r;
        asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w[is >> 2]), "r"(0u), "r"((sgn << 12) | (sgn << 8) | (sgn << 4) | i));
        return r;
    };
    const uint8_t* ap = x.act + 256 * b + 4 * x.t;
    int S[4] = {0, 0, 0, 0};
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
            const uint32_t Aa = *reinterpret_cast<const uint32_t*>(rA + 64 * n + 16 * cc + 4 * x.t);
            const uint32_t Ab = *reinterpret_cast<const uint32_t*>(rA + 64 * n + 32 + 16 * cc + 4 * x.t);
            const uint32_t Ah = *reinterpret_cast<const uint32_t*>(rA + 128 + 32 * n + 16 * cc + 4 * x.t);
            const uint32_t Ba = *reinterpret_cast<const uint32_t*>(rB + 64 * n + 16 * cc + 4 * x.t);
            const uint32_t Bb = *reinterpret_cast<const uint32_t*>(rB + 64 * n + 32 + 16 * cc + 4 * x.t);
            const uint32_t Bh = *reinterpret_cast<const uint32_t*>(rB + 128 + 32 * n + 16 * cc + 4 * x.t);
            const uint32_t qa[4] = {(Aa & 0x0f0f0f0fu) | ((Ah << 4) & 0x30303030u), (Ab & 0x0f0f0f0fu) | ((Ah << 2) & 0x30303030u),
                                    ((Aa >> 4) & 0x0f0f0f0fu) | (Ah & 0x30303030u), ((Ab >> 4) & 0x0f0f0f0fu) | ((Ah >> 2) & 0x30303030u)};
            const uint32_t qb[4] = {(Ba & 0x0f0f0f0fu) | ((Bh << 4) & 0x30303030u), (Bb & 0x0f0f0f0fu) | ((Bh << 2) & 0x30303030u),
                                    ((Ba >> 4) & 0x0f0f0f0fu) | (Bh & 0x30303030u), ((Bb >> 4) & 0x0f0f0f0fu) | ((Bh >> 2) & 0x30303030u)};
#pragma unroll
            for (int qd = 0; qd < 4; ++qd) {
                uint32_t bv = 0u;
                if (x.colv) bv = *reinterpret_cast<const uint32_t*>(ap + 128 * n + 32 * qd + 16 * cc);
                int c[4];
                mma_u8s8_k16(c, qa[qd], qb[qd], bv);
                const int is = 8 * n + cc + 2 * qd;
                const int sa = sc_of(scwA, is), sb = sc_of(scwB, is);
                scale_add<NB>(S, sa, sb, c);
            }
        }
    }
    float fA, fB;
    plane_scale<NB>(x, b, S, fA, fB);
    float tA = 0.f, tB = 0.f;
    if (NB == 1) {
        // offset term, this lane's four groups 4t..4t+3 (scale word t, selected without indexing the array dynamically)
        const float4 v = *reinterpret_cast<const float4*>(x.xs16 + 16 * b + 4 * x.t);
        const float vv[4] = {v.x, v.y, v.z, v.w};
        const uint32_t wA = (x.t & 2) ? ((x.t & 1) ? sA4.w : sA4.z) : ((x.t & 1) ? sA4.y : sA4.x);
        const uint32_t wB = (x.t & 2) ? ((x.t & 1) ? sB4.w : sB4.z) : ((x.t & 1) ? sB4.y : sB4.x);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            tA = fmaf((float)(((int)(wA << (24 - 8 * j))) >> 24), vv[j], tA);
            tB = fmaf((float)(((int)(wB << (24 - 8 * j))) >> 24), vv[j], tB);
        }
    } else {
        // two vectors per launch: lane half h = t & 1 takes groups 8h..8h+7 (scale words 2h, 2h+1) of its own vector
        const int h = x.t & 1;
        const float4 v0 = *reinterpret_cast<const float4*>(x.xs16 + 16 * b + 8 * h);
        const float4 v1 = *reinterpret_cast<const float4*>(x.xs16 + 16 * b + 8 * h + 4);
        const float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        const uint32_t wA0 = h ? sA4.z : sA4.x, wA1 = h ? sA4.w : sA4.y;
        const uint32_t wB0 = h ? sB4.z : sB4.x, wB1 = h ? sB4.w : sB4.y;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            tA = fmaf((float)(((int)(wA0 << (24 - 8 * j))) >> 24), vv[j], tA);
            tB = fmaf((float)(((int)(wB0 << (24 - 8 * j))) >> 24), vv[j], tB);
            tA = fmaf((float)(((int)(wA1 << (24 - 8 * j))) >> 24), vv[4 + j], tA);
            tB = fmaf((float)(((int)(wB1 << (24 - 8 * j))) >> 24), vv[4 + j], tB);
        }
    }
    accA += dA * (fA - 32.f * tA);
    accB += dB * (fB - 32.f * tB);
}

}  // namespace l2b
