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

// ---- (2) two-row block dot products ---------------------------------------------------
//
// Activation record of one (plane, block) in shared memory: 256 int8, then the plane's f32
// scale at byte 256; records are ACT_STRIDE bytes apart (272: 16-byte reads by consecutive
// lanes at that stride fall in distinct banks).  xs16 = 16 f32 sums of the represented
// activations over groups of 16 values of this block.
constexpr int ACT_STRIDE = 272;

__device__ __forceinline__ uint32_t byte_of(uint32_t w, int i) { return (w >> (8 * i)) & 0xFFu; }

// Decode the 12 packed 6-bit scale bytes (words y,z,w of the 16-byte block header) into four
// words of 8-bit values: sc[0..3], sc[4..7], m[0..3], m[4..7].
__device__ __forceinline__ void decode_scales_k4(const uint4& h, uint32_t& sc_lo, uint32_t& sc_hi, uint32_t& m_lo, uint32_t& m_hi) {
    sc_lo = h.y & 0x3f3f3f3fu;
    m_lo = h.z & 0x3f3f3f3fu;
    sc_hi = (h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u);
    m_hi = ((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u);
}

// min term: sum_s m_s * xs32[s]
__device__ __forceinline__ float min_term(uint32_t m_lo, uint32_t m_hi, const float (&xs32)[8]) {
    float t = 0.f;
#pragma unroll
    for (int s = 0; s < 4; ++s) t = fmaf((float)byte_of(m_lo, s), xs32[s], t);
#pragma unroll
    for (int s = 0; s < 4; ++s) t = fmaf((float)byte_of(m_hi, s), xs32[4 + s], t);
    return t;
}

__device__ __forceinline__ void load_xs32(const float* xs16, float (&xs32)[8]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 v = *reinterpret_cast<const float4*>(xs16 + 4 * i);
        xs32[2 * i] = v.x + v.y;
        xs32[2 * i + 1] = v.z + v.w;
    }
}

// q4_K.  A, B: the two rows' 144-byte blocks in shared memory; act: plane 0's record of this
// block position; plane_stride: bytes between planes.  Adds the two partial dots to accA/accB.
template <int P>
__device__ __forceinline__ void dot2_q4k(const uint8_t* A, const uint8_t* B, const uint8_t* act, int plane_stride, const float* xs16,
                                         float& accA, float& accB) {
    const uint4 hA = *reinterpret_cast<const uint4*>(A);
    const uint4 hB = *reinterpret_cast<const uint4*>(B);
    uint32_t scA[2], mA[2], scB[2], mB[2];
    decode_scales_k4(hA, scA[0], scA[1], mA[0], mA[1]);
    decode_scales_k4(hB, scB[0], scB[1], mB[0], mB[1]);
    int SA[P], SB[P];
#pragma unroll
    for (int k = 0; k < P; ++k) SA[k] = SB[k] = 0;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        int IAl[P], IAh[P], IBl[P], IBh[P];
#pragma unroll
        for (int k = 0; k < P; ++k) IAl[k] = IAh[k] = IBl[k] = IBh[k] = 0;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const uint4 wA = *reinterpret_cast<const uint4*>(A + 16 + 32 * p + 16 * half);
            const uint4 wB = *reinterpret_cast<const uint4*>(B + 16 + 32 * p + 16 * half);
            const uint32_t a[4] = {wA.x, wA.y, wA.z, wA.w};
            const uint32_t b[4] = {wB.x, wB.y, wB.z, wB.w};
#pragma unroll
            for (int k = 0; k < P; ++k) {
                const int4 lo = *reinterpret_cast<const int4*>(act + k * plane_stride + 64 * p + 16 * half);
                const int4 hi = *reinterpret_cast<const int4*>(act + k * plane_stride + 64 * p + 32 + 16 * half);
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
        // sub-block 2p takes the low nibbles (scaled here by 16 to match the high nibbles), 2p+1 the high ones
        const int se_A = (int)(byte_of(scA[p >> 1], (2 * p) & 3) << 4), so_A = (int)byte_of(scA[p >> 1], (2 * p + 1) & 3);
        const int se_B = (int)(byte_of(scB[p >> 1], (2 * p) & 3) << 4), so_B = (int)byte_of(scB[p >> 1], (2 * p + 1) & 3);
#pragma unroll
        for (int k = 0; k < P; ++k) {
            SA[k] += se_A * IAl[k] + so_A * IAh[k];
            SB[k] += se_B * IBl[k] + so_B * IBh[k];
        }
    }
    float fA = 0.f, fB = 0.f;
#pragma unroll
    for (int k = 0; k < P; ++k) {
        const float dp = *reinterpret_cast<const float*>(act + k * plane_stride + 256);
        fA = fmaf(dp, (float)SA[k], fA);
        fB = fmaf(dp, (float)SB[k], fB);
    }
    float xs32[8];
    load_xs32(xs16, xs32);
    const float dA = half_bits_to_float(hA.x & 0xFFFFu), dminA = half_bits_to_float(hA.x >> 16);
    const float dB = half_bits_to_float(hB.x & 0xFFFFu), dminB = half_bits_to_float(hB.x >> 16);
    accA += dA * 0.0625f * fA - dminA * min_term(mA[0], mA[1], xs32);
    accB += dB * 0.0625f * fB - dminB * min_term(mB[0], mB[1], xs32);
}

// q5_K: 176-byte blocks: header 16 | qh 32 | qs 128.
template <int P>
__device__ __forceinline__ void dot2_q5k(const uint8_t* A, const uint8_t* B, const uint8_t* act, int plane_stride, const float* xs16,
                                         float& accA, float& accB) {
    const uint4 hA = *reinterpret_cast<const uint4*>(A);
    const uint4 hB = *reinterpret_cast<const uint4*>(B);
    uint32_t scA[2], mA[2], scB[2], mB[2];
    decode_scales_k4(hA, scA[0], scA[1], mA[0], mA[1]);
    decode_scales_k4(hB, scB[0], scB[1], mB[0], mB[1]);
    uint32_t qhA[8], qhB[8];
    {
        const uint4 t0 = *reinterpret_cast<const uint4*>(A + 16), t1 = *reinterpret_cast<const uint4*>(A + 32);
        qhA[0] = t0.x; qhA[1] = t0.y; qhA[2] = t0.z; qhA[3] = t0.w; qhA[4] = t1.x; qhA[5] = t1.y; qhA[6] = t1.z; qhA[7] = t1.w;
        const uint4 u0 = *reinterpret_cast<const uint4*>(B + 16), u1 = *reinterpret_cast<const uint4*>(B + 32);
        qhB[0] = u0.x; qhB[1] = u0.y; qhB[2] = u0.z; qhB[3] = u0.w; qhB[4] = u1.x; qhB[5] = u1.y; qhB[6] = u1.z; qhB[7] = u1.w;
    }
    int SA[P], SB[P];
#pragma unroll
    for (int k = 0; k < P; ++k) SA[k] = SB[k] = 0;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        int IAl[P], IAh[P], IBl[P], IBh[P];
#pragma unroll
        for (int k = 0; k < P; ++k) IAl[k] = IAh[k] = IBl[k] = IBh[k] = 0;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const uint4 wA = *reinterpret_cast<const uint4*>(A + 48 + 32 * p + 16 * half);
            const uint4 wB = *reinterpret_cast<const uint4*>(B + 48 + 32 * p + 16 * half);
            const uint32_t a[4] = {wA.x, wA.y, wA.z, wA.w};
            const uint32_t b[4] = {wB.x, wB.y, wB.z, wB.w};
            uint32_t qAl[4], qAh[4], qBl[4], qBh[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                // fifth bit of value 64p+l is bit 2p of qh[l]; of 64p+32+l, bit 2p+1 (l = 16*half + 4w + byte)
                const uint32_t ha = qhA[4 * half + w], hb = qhB[4 * half + w];
                qAl[w] = (a[w] & 0x0f0f0f0fu) | (((ha >> (2 * p)) & 0x01010101u) << 4);
                qAh[w] = ((a[w] >> 4) & 0x0f0f0f0fu) | (((ha >> (2 * p + 1)) & 0x01010101u) << 4);
                qBl[w] = (b[w] & 0x0f0f0f0fu) | (((hb >> (2 * p)) & 0x01010101u) << 4);
                qBh[w] = ((b[w] >> 4) & 0x0f0f0f0fu) | (((hb >> (2 * p + 1)) & 0x01010101u) << 4);
            }
#pragma unroll
            for (int k = 0; k < P; ++k) {
                const int4 lo = *reinterpret_cast<const int4*>(act + k * plane_stride + 64 * p + 16 * half);
                const int4 hi = *reinterpret_cast<const int4*>(act + k * plane_stride + 64 * p + 32 + 16 * half);
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
        const int se_A = (int)byte_of(scA[p >> 1], (2 * p) & 3), so_A = (int)byte_of(scA[p >> 1], (2 * p + 1) & 3);
        const int se_B = (int)byte_of(scB[p >> 1], (2 * p) & 3), so_B = (int)byte_of(scB[p >> 1], (2 * p + 1) & 3);
#pragma unroll
        for (int k = 0; k < P; ++k) {
            SA[k] += se_A * IAl[k] + so_A * IAh[k];
            SB[k] += se_B * IBl[k] + so_B * IBh[k];
        }
    }
    float fA = 0.f, fB = 0.f;
#pragma unroll
    for (int k = 0; k < P; ++k) {
        const float dp = *reinterpret_cast<const float*>(act + k * plane_stride + 256);
        fA = fmaf(dp, (float)SA[k], fA);
        fB = fmaf(dp, (float)SB[k], fB);
    }
    float xs32[8];
    load_xs32(xs16, xs32);
    const float dA = half_bits_to_float(hA.x & 0xFFFFu), dminA = half_bits_to_float(hA.x >> 16);
    const float dB = half_bits_to_float(hB.x & 0xFFFFu), dminB = half_bits_to_float(hB.x >> 16);
    accA += dA * fA - dminA * min_term(mA[0], mA[1], xs32);
    accB += dB * fB - dminB * min_term(mB[0], mB[1], xs32);
}

// q6_K: 208-byte records (ql[128] qh[64] scales[16]); dA, dB = the blocks' fp16 scales.
// Quants are kept as unsigned 0..63; the -32 offset becomes -32 * scale * (sum of activations).
template <int P>
__device__ __forceinline__ void dot2_q6k(const uint8_t* A, const uint8_t* B, float dA, float dB, const uint8_t* act, int plane_stride,
                                         const float* xs16, float& accA, float& accB) {
    int SA[P], SB[P];
#pragma unroll
    for (int k = 0; k < P; ++k) SA[k] = SB[k] = 0;
    const uint4 sA4 = *reinterpret_cast<const uint4*>(A + 192);
    const uint4 sB4 = *reinterpret_cast<const uint4*>(B + 192);
    const uint32_t scwA[4] = {sA4.x, sA4.y, sA4.z, sA4.w};
    const uint32_t scwB[4] = {sB4.x, sB4.y, sB4.z, sB4.w};
    auto sc_of = [](const uint32_t (&w)[4], int is) -> int { return (int)(int8_t)((w[is >> 2] >> (8 * (is & 3))) & 0xFF); };
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const uint4 la = *reinterpret_cast<const uint4*>(A + 64 * n + 16 * c);
            const uint4 lb = *reinterpret_cast<const uint4*>(A + 64 * n + 32 + 16 * c);
            const uint4 lh = *reinterpret_cast<const uint4*>(A + 128 + 32 * n + 16 * c);
            const uint4 ma = *reinterpret_cast<const uint4*>(B + 64 * n + 16 * c);
            const uint4 mb = *reinterpret_cast<const uint4*>(B + 64 * n + 32 + 16 * c);
            const uint4 mh = *reinterpret_cast<const uint4*>(B + 128 + 32 * n + 16 * c);
            const uint32_t Aa[4] = {la.x, la.y, la.z, la.w}, Ab[4] = {lb.x, lb.y, lb.z, lb.w}, Ah[4] = {lh.x, lh.y, lh.z, lh.w};
            const uint32_t Ba[4] = {ma.x, ma.y, ma.z, ma.w}, Bb[4] = {mb.x, mb.y, mb.z, mb.w}, Bh[4] = {mh.x, mh.y, mh.z, mh.w};
            int IA[4][P], IB[4][P];
#pragma unroll
            for (int qd = 0; qd < 4; ++qd)
#pragma unroll
                for (int k = 0; k < P; ++k) IA[qd][k] = IB[qd][k] = 0;
            uint32_t qA[4][4], qB[4][4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                qA[0][w] = (Aa[w] & 0x0f0f0f0fu) | ((Ah[w] << 4) & 0x30303030u);
                qA[1][w] = (Ab[w] & 0x0f0f0f0fu) | ((Ah[w] << 2) & 0x30303030u);
                qA[2][w] = ((Aa[w] >> 4) & 0x0f0f0f0fu) | (Ah[w] & 0x30303030u);
                qA[3][w] = ((Ab[w] >> 4) & 0x0f0f0f0fu) | ((Ah[w] >> 2) & 0x30303030u);
                qB[0][w] = (Ba[w] & 0x0f0f0f0fu) | ((Bh[w] << 4) & 0x30303030u);
                qB[1][w] = (Bb[w] & 0x0f0f0f0fu) | ((Bh[w] << 2) & 0x30303030u);
                qB[2][w] = ((Ba[w] >> 4) & 0x0f0f0f0fu) | (Bh[w] & 0x30303030u);
                qB[3][w] = ((Bb[w] >> 4) & 0x0f0f0f0fu) | ((Bh[w] >> 2) & 0x30303030u);
            }
#pragma unroll
            for (int k = 0; k < P; ++k) {
#pragma unroll
                for (int qd = 0; qd < 4; ++qd) {
                    const int4 xv = *reinterpret_cast<const int4*>(act + k * plane_stride + 128 * n + 32 * qd + 16 * c);
                    const int xx[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        IA[qd][k] = dp4a_us(qA[qd][w], xx[w], IA[qd][k]);
                        IB[qd][k] = dp4a_us(qB[qd][w], xx[w], IB[qd][k]);
                    }
                }
            }
#pragma unroll
            for (int qd = 0; qd < 4; ++qd) {
                const int is = 8 * n + c + 2 * qd;
                const int sa = sc_of(scwA, is), sb = sc_of(scwB, is);
#pragma unroll
                for (int k = 0; k < P; ++k) {
                    SA[k] += sa * IA[qd][k];
                    SB[k] += sb * IB[qd][k];
                }
            }
        }
    }
    float fA = 0.f, fB = 0.f;
#pragma unroll
    for (int k = 0; k < P; ++k) {
        const float dp = *reinterpret_cast<const float*>(act + k * plane_stride + 256);
        fA = fmaf(dp, (float)SA[k], fA);
        fB = fmaf(dp, (float)SB[k], fB);
    }
    float tA = 0.f, tB = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 v = *reinterpret_cast<const float4*>(xs16 + 4 * i);
        const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            tA = fmaf((float)sc_of(scwA, 4 * i + j), vv[j], tA);
            tB = fmaf((float)sc_of(scwB, 4 * i + j), vv[j], tB);
        }
    }
    accA += dA * (fA - 32.f * tA);
    accB += dB * (fB - 32.f * tB);
}

}  // namespace l2b
