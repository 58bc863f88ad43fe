// k-quant super-block arithmetic on the device.
//
// Two families live here:
//  (1) exact dequantisation of one weight, bit-for-bit what the reference's dequantize!
//      produces (src/kquants.jl:70-125, 186-251, 322-363): products and the subtraction are
//      rounded separately (__fmul_rn / __fsub_rn block FMA contraction);
//  (2) integer dot products of one super-block of TWO weight rows against int8 activation
//      planes held in shared memory.  The algebra is the reference's vecdot
//      (src/kquants.jl:127-184, 253-320, 365-408) factorised per sub-block:
//          sum_k x_k (d sc q_k - dmin m) = d sc sum_k x_k q_k  -  dmin m sum_k x_k
//      with x_k represented as sum_p dplane_p * a_{p,k}, a int8 (1..3 planes), so that the
//      inner sums are exact integer dot products (dp4a).
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

// ---- (2) two-row half-block dot products ------------------------------------------------
//
// A lane works on HALF a super-block (128 weights) of two rows at a time, so that a warp's
// shared-memory slot holds only 32 super-blocks and the unrolled body stays small enough for
// the instruction cache.  h = 0 / 1 selects weights 0..127 / 128..255.
//
// Activation record of one (plane, block) in shared memory, ACT_STRIDE = 288 bytes:
//   [0,128) int8 values 0..127 | [128,132) the plane's f32 scale | [144,272) int8 values 128..255.
// With that stride and half offset, the 16-byte reads of eight consecutive lanes (four blocks
// times two halves) fall in eight distinct bank groups.  xs16 = 16 f32 sums of the represented
// activations over groups of 16 values of this block.
constexpr int ACT_STRIDE = 288;
constexpr int ACT_HALF = 144;   // byte offset of values 128..255
constexpr int ACT_SCALE = 128;  // byte offset of the plane scale

// Unroll factor of the two-iteration loop over sub-block pairs: 1 keeps the loop body (and the
// instruction-cache footprint) small.
#ifndef L2B_DOT_UNROLL_FACTOR
#define L2B_DOT_UNROLL_FACTOR 1
#endif
constexpr int DOT_UNROLL = L2B_DOT_UNROLL_FACTOR;

// The four 6-bit scales and four 6-bit mins of sub-blocks 4h..4h+3 as bytes of two words.
// src/kquants.jl:80-81,86-87 (h = 0) and :102-103,108-109 (h = 1).
__device__ __forceinline__ void decode_scales_half(const uint4& hd, int h, uint32_t& sc4, uint32_t& m4) {
    const uint32_t sc_lo = hd.y & 0x3f3f3f3fu, m_lo = hd.z & 0x3f3f3f3fu;
    const uint32_t sc_hi = (hd.w & 0x0f0f0f0fu) | ((hd.y >> 2) & 0x30303030u);
    const uint32_t m_hi = ((hd.w >> 4) & 0x0f0f0f0fu) | ((hd.z >> 2) & 0x30303030u);
    sc4 = h ? sc_hi : sc_lo;
    m4 = h ? m_hi : m_lo;
}

// sum_s m_s * (xs16[2s] + xs16[2s+1]) over the four sub-blocks of the half; xs points at the half's 8 sums
__device__ __forceinline__ float min_term_half(uint32_t m4, const float* xs) {
    const float4 v0 = *reinterpret_cast<const float4*>(xs), v1 = *reinterpret_cast<const float4*>(xs + 4);
    float t = (float)(m4 & 0xFFu) * (v0.x + v0.y);
    t = fmaf((float)((m4 >> 8) & 0xFFu), v0.z + v0.w, t);
    t = fmaf((float)((m4 >> 16) & 0xFFu), v1.x + v1.y, t);
    t = fmaf((float)(m4 >> 24), v1.z + v1.w, t);
    return t;
}

// q4_K.  A, B: the two rows' 144-byte blocks in shared memory; act: plane 0's record of this
// block position; plane_stride: bytes between planes.  Adds the two partial dots to accA/accB.
template <int P>
__device__ __forceinline__ void dot2h_q4k(const uint8_t* A, const uint8_t* B, const uint8_t* act, int plane_stride, const float* xs16, int h,
                                          float& accA, float& accB) {
    const uint4 hA = *reinterpret_cast<const uint4*>(A);
    const uint4 hB = *reinterpret_cast<const uint4*>(B);
    uint32_t scA, mA, scB, mB;
    decode_scales_half(hA, h, scA, mA);
    decode_scales_half(hB, h, scB, mB);
    int SA[P], SB[P];
#pragma unroll
    for (int k = 0; k < P; ++k) SA[k] = SB[k] = 0;
    const uint8_t* qa = A + 16 + 64 * h;
    const uint8_t* qb = B + 16 + 64 * h;
    const uint8_t* xa = act + ACT_HALF * h;
#pragma unroll DOT_UNROLL
    for (int pp = 0; pp < 2; ++pp) {  // sub-block pair 2h + pp
        int IAl[P], IAh[P], IBl[P], IBh[P];
#pragma unroll
        for (int k = 0; k < P; ++k) IAl[k] = IAh[k] = IBl[k] = IBh[k] = 0;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const uint4 wA = *reinterpret_cast<const uint4*>(qa + 32 * pp + 16 * half);
            const uint4 wB = *reinterpret_cast<const uint4*>(qb + 32 * pp + 16 * half);
            const uint32_t a[4] = {wA.x, wA.y, wA.z, wA.w};
            const uint32_t b[4] = {wB.x, wB.y, wB.z, wB.w};
#pragma unroll
            for (int k = 0; k < P; ++k) {
                const int4 lo = *reinterpret_cast<const int4*>(xa + k * plane_stride + 64 * pp + 16 * half);
                const int4 hi = *reinterpret_cast<const int4*>(xa + k * plane_stride + 64 * pp + 32 + 16 * half);
                const int xl[4] = {lo.x, lo.y, lo.z, lo.w};
                const int xh[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    IAl[k] = dp4a_us(a[w] & 0x0f0f0f0fu, xl[w], IAl[k]);
                    IAh[k] = dp4a_us(a[w] & 0xf0f0f0f0u, xh[w], IAh[k]);  // 16 * high nibble
                    IBl[k] = dp4a_us(b[w] & 0x0f0f0f0fu, xl[w], IBl[k]);
                    IBh[k] = dp4a_us(b[w] & 0xf0f0f0f0u, xh[w], IBh[k]);
                }
            }
        }
        // even sub-block: low nibbles (scale taken x16 to match the high nibbles); odd: high nibbles
        const int se_A = (int)(((scA >> (16 * pp)) & 0xFFu) << 4), so_A = (int)((scA >> (16 * pp + 8)) & 0xFFu);
        const int se_B = (int)(((scB >> (16 * pp)) & 0xFFu) << 4), so_B = (int)((scB >> (16 * pp + 8)) & 0xFFu);
#pragma unroll
        for (int k = 0; k < P; ++k) {
            SA[k] += se_A * IAl[k] + so_A * IAh[k];
            SB[k] += se_B * IBl[k] + so_B * IBh[k];
        }
    }
    float fA = 0.f, fB = 0.f;
#pragma unroll
    for (int k = 0; k < P; ++k) {
        const float dp = *reinterpret_cast<const float*>(act + k * plane_stride + ACT_SCALE);
        fA = fmaf(dp, (float)SA[k], fA);
        fB = fmaf(dp, (float)SB[k], fB);
    }
    const float dA = half_bits_to_float(hA.x & 0xFFFFu), dminA = half_bits_to_float(hA.x >> 16);
    const float dB = half_bits_to_float(hB.x & 0xFFFFu), dminB = half_bits_to_float(hB.x >> 16);
    accA += dA * 0.0625f * fA - dminA * min_term_half(mA, xs16 + 8 * h);
    accB += dB * 0.0625f * fB - dminB * min_term_half(mB, xs16 + 8 * h);
}

// q5_K: 176-byte blocks: header 16 | qh 32 | qs 128.
template <int P>
__device__ __forceinline__ void dot2h_q5k(const uint8_t* A, const uint8_t* B, const uint8_t* act, int plane_stride, const float* xs16, int h,
                                          float& accA, float& accB) {
    const uint4 hA = *reinterpret_cast<const uint4*>(A);
    const uint4 hB = *reinterpret_cast<const uint4*>(B);
    uint32_t scA, mA, scB, mB;
    decode_scales_half(hA, h, scA, mA);
    decode_scales_half(hB, h, scB, mB);
    uint32_t qhA[8], qhB[8];
    {
        const uint4 t0 = *reinterpret_cast<const uint4*>(A + 16), t1 = *reinterpret_cast<const uint4*>(A + 32);
        const uint4 u0 = *reinterpret_cast<const uint4*>(B + 16), u1 = *reinterpret_cast<const uint4*>(B + 32);
        // bring the four fifth-bits this half uses (bits 4h .. 4h+3 of every qh byte) down to bits 0..3
        const int sh = 4 * h;
        qhA[0] = t0.x >> sh; qhA[1] = t0.y >> sh; qhA[2] = t0.z >> sh; qhA[3] = t0.w >> sh;
        qhA[4] = t1.x >> sh; qhA[5] = t1.y >> sh; qhA[6] = t1.z >> sh; qhA[7] = t1.w >> sh;
        qhB[0] = u0.x >> sh; qhB[1] = u0.y >> sh; qhB[2] = u0.z >> sh; qhB[3] = u0.w >> sh;
        qhB[4] = u1.x >> sh; qhB[5] = u1.y >> sh; qhB[6] = u1.z >> sh; qhB[7] = u1.w >> sh;
    }
    int SA[P], SB[P];
#pragma unroll
    for (int k = 0; k < P; ++k) SA[k] = SB[k] = 0;
    const uint8_t* qa = A + 48 + 64 * h;
    const uint8_t* qb = B + 48 + 64 * h;
    const uint8_t* xa = act + ACT_HALF * h;
#pragma unroll
    for (int pp = 0; pp < 2; ++pp) {  // kept unrolled: the fifth-bit words are indexed statically
        int IAl[P], IAh[P], IBl[P], IBh[P];
#pragma unroll
        for (int k = 0; k < P; ++k) IAl[k] = IAh[k] = IBl[k] = IBh[k] = 0;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const uint4 wA = *reinterpret_cast<const uint4*>(qa + 32 * pp + 16 * half);
            const uint4 wB = *reinterpret_cast<const uint4*>(qb + 32 * pp + 16 * half);
            const uint32_t a[4] = {wA.x, wA.y, wA.z, wA.w};
            const uint32_t b[4] = {wB.x, wB.y, wB.z, wB.w};
            uint32_t qAl[4], qAh[4], qBl[4], qBh[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                // fifth bit of value 64p+l is bit 2p of qh[l]; of 64p+32+l, bit 2p+1 (l = 16*half + 4w + byte)
                const uint32_t ha = qhA[4 * half + w], hb = qhB[4 * half + w];
                qAl[w] = (a[w] & 0x0f0f0f0fu) | (((ha >> (2 * pp)) & 0x01010101u) << 4);
                qAh[w] = ((a[w] >> 4) & 0x0f0f0f0fu) | (((ha >> (2 * pp + 1)) & 0x01010101u) << 4);
                qBl[w] = (b[w] & 0x0f0f0f0fu) | (((hb >> (2 * pp)) & 0x01010101u) << 4);
                qBh[w] = ((b[w] >> 4) & 0x0f0f0f0fu) | (((hb >> (2 * pp + 1)) & 0x01010101u) << 4);
            }
#pragma unroll
            for (int k = 0; k < P; ++k) {
                const int4 lo = *reinterpret_cast<const int4*>(xa + k * plane_stride + 64 * pp + 16 * half);
                const int4 hi = *reinterpret_cast<const int4*>(xa + k * plane_stride + 64 * pp + 32 + 16 * half);
                const int xl[4] = {lo.x, lo.y, lo.z, lo.w};
                const int xh[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    IAl[k] = dp4a_us(qAl[w], xl[w], IAl[k]);
                    IAh[k] = dp4a_us(qAh[w], xh[w], IAh[k]);
                    IBl[k] = dp4a_us(qBl[w], xl[w], IBl[k]);
                    IBh[k] = dp4a_us(qBh[w], xh[w], IBh[k]);
                }
            }
        }
        const int se_A = (int)((scA >> (16 * pp)) & 0xFFu), so_A = (int)((scA >> (16 * pp + 8)) & 0xFFu);
        const int se_B = (int)((scB >> (16 * pp)) & 0xFFu), so_B = (int)((scB >> (16 * pp + 8)) & 0xFFu);
#pragma unroll
        for (int k = 0; k < P; ++k) {
            SA[k] += se_A * IAl[k] + so_A * IAh[k];
            SB[k] += se_B * IBl[k] + so_B * IBh[k];
        }
    }
    float fA = 0.f, fB = 0.f;
#pragma unroll
    for (int k = 0; k < P; ++k) {
        const float dp = *reinterpret_cast<const float*>(act + k * plane_stride + ACT_SCALE);
        fA = fmaf(dp, (float)SA[k], fA);
        fB = fmaf(dp, (float)SB[k], fB);
    }
    const float dA = half_bits_to_float(hA.x & 0xFFFFu), dminA = half_bits_to_float(hA.x >> 16);
    const float dB = half_bits_to_float(hB.x & 0xFFFFu), dminB = half_bits_to_float(hB.x >> 16);
    accA += dA * fA - dminA * min_term_half(mA, xs16 + 8 * h);
    accB += dB * fB - dminB * min_term_half(mB, xs16 + 8 * h);
}

// q6_K: 208-byte records (ql[128] qh[64] scales[16]); dA, dB = the blocks' fp16 scales.  The half h is
// the reference's outer index n (src/kquants.jl:329).  Quants stay unsigned 0..63; the -32 offset
// becomes -32 * scale * (sum of activations).
template <int P>
__device__ __forceinline__ void dot2h_q6k(const uint8_t* A, const uint8_t* B, float dA, float dB, const uint8_t* act, int plane_stride,
                                          const float* xs16, int h, float& accA, float& accB) {
    int SA[P], SB[P];
#pragma unroll
    for (int k = 0; k < P; ++k) SA[k] = SB[k] = 0;
    const uint2 sA2 = *reinterpret_cast<const uint2*>(A + 192 + 8 * h);
    const uint2 sB2 = *reinterpret_cast<const uint2*>(B + 192 + 8 * h);
    const uint64_t scA = ((uint64_t)sA2.y << 32) | sA2.x, scB = ((uint64_t)sB2.y << 32) | sB2.x;  // scales 8h .. 8h+7
    auto sc_of = [](uint64_t w, int i) -> int { return (int)(int8_t)((w >> (8 * i)) & 0xFF); };
    const uint8_t* la = A + 64 * h;
    const uint8_t* lb = B + 64 * h;
    const uint8_t* ha = A + 128 + 32 * h;
    const uint8_t* hb = B + 128 + 32 * h;
    const uint8_t* xa = act + ACT_HALF * h;
#pragma unroll DOT_UNROLL
    for (int c = 0; c < 2; ++c) {  // l = 16c .. 16c+15; scale index within the half: c + 2*quad
        const uint4 Aa4 = *reinterpret_cast<const uint4*>(la + 16 * c), Ab4 = *reinterpret_cast<const uint4*>(la + 32 + 16 * c);
        const uint4 Ah4 = *reinterpret_cast<const uint4*>(ha + 16 * c);
        const uint4 Ba4 = *reinterpret_cast<const uint4*>(lb + 16 * c), Bb4 = *reinterpret_cast<const uint4*>(lb + 32 + 16 * c);
        const uint4 Bh4 = *reinterpret_cast<const uint4*>(hb + 16 * c);
        const uint32_t Aa[4] = {Aa4.x, Aa4.y, Aa4.z, Aa4.w}, Ab[4] = {Ab4.x, Ab4.y, Ab4.z, Ab4.w}, Ah[4] = {Ah4.x, Ah4.y, Ah4.z, Ah4.w};
        const uint32_t Ba[4] = {Ba4.x, Ba4.y, Ba4.z, Ba4.w}, Bb[4] = {Bb4.x, Bb4.y, Bb4.z, Bb4.w}, Bh[4] = {Bh4.x, Bh4.y, Bh4.z, Bh4.w};
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
            int IA[P], IB[P];
#pragma unroll
            for (int k = 0; k < P; ++k) IA[k] = IB[k] = 0;
            uint32_t qA[4], qB[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                if (qd == 0) {
                    qA[w] = (Aa[w] & 0x0f0f0f0fu) | ((Ah[w] << 4) & 0x30303030u);
                    qB[w] = (Ba[w] & 0x0f0f0f0fu) | ((Bh[w] << 4) & 0x30303030u);
                } else if (qd == 1) {
                    qA[w] = (Ab[w] & 0x0f0f0f0fu) | ((Ah[w] << 2) & 0x30303030u);
                    qB[w] = (Bb[w] & 0x0f0f0f0fu) | ((Bh[w] << 2) & 0x30303030u);
                } else if (qd == 2) {
                    qA[w] = ((Aa[w] >> 4) & 0x0f0f0f0fu) | (Ah[w] & 0x30303030u);
                    qB[w] = ((Ba[w] >> 4) & 0x0f0f0f0fu) | (Bh[w] & 0x30303030u);
                } else {
                    qA[w] = ((Ab[w] >> 4) & 0x0f0f0f0fu) | ((Ah[w] >> 2) & 0x30303030u);
                    qB[w] = ((Bb[w] >> 4) & 0x0f0f0f0fu) | ((Bh[w] >> 2) & 0x30303030u);
                }
            }
#pragma unroll
            for (int k = 0; k < P; ++k) {
                const int4 xv = *reinterpret_cast<const int4*>(xa + k * plane_stride + 32 * qd + 16 * c);
                const int xx[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    IA[k] = dp4a_us(qA[w], xx[w], IA[k]);
                    IB[k] = dp4a_us(qB[w], xx[w], IB[k]);
                }
            }
            const int sa = sc_of(scA, c + 2 * qd), sb = sc_of(scB, c + 2 * qd);
#pragma unroll
            for (int k = 0; k < P; ++k) {
                SA[k] += sa * IA[k];
                SB[k] += sb * IB[k];
            }
        }
    }
    float fA = 0.f, fB = 0.f;
#pragma unroll
    for (int k = 0; k < P; ++k) {
        const float dp = *reinterpret_cast<const float*>(act + k * plane_stride + ACT_SCALE);
        fA = fmaf(dp, (float)SA[k], fA);
        fB = fmaf(dp, (float)SB[k], fB);
    }
    float tA = 0.f, tB = 0.f;
    const float4 v0 = *reinterpret_cast<const float4*>(xs16 + 8 * h), v1 = *reinterpret_cast<const float4*>(xs16 + 8 * h + 4);
    const float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        tA = fmaf((float)sc_of(scA, j), vv[j], tA);
        tB = fmaf((float)sc_of(scB, j), vv[j], tB);
    }
    accA += dA * (fA - 32.f * tA);
    accB += dB * (fB - 32.f * tB);
}

}  // namespace l2b
