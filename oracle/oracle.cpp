// CPU oracle: a plain C++17 restatement of the reference's per-token decode arithmetic.
//
// THIS FILE IS TEST INFRASTRUCTURE.  It is the checker the CUDA path is compared
// against and the timed CPU baseline; the shipped library never calls it.
//
// Parity status: PARITY UNPINNED.  The reference (cafaxo/Llama2.jl) ships no tests,
// fixtures or golden vectors and cannot be executed where this was written (no Julia),
// so this restatement is validated (i) line by line against the cited source,
// (ii) bit-for-bit against the independent numpy dequantiser of the `gguf` Python
// package for q4_K/q5_K/q6_K, and (iii) against hand-computed single-block cases.
//
// Every function cites the reference file:line it follows (paths are relative to the
// reference project root).  Build with -ffp-contract=off and without -ffast-math: the
// reference rounds `d*sc*q` and `- dmin*m` separately (no FMA), and so must this.
//
// Index conventions: the reference is 1-based (Julia); everything here is 0-based.
// `pos0 = pos - 1`, `token0 = token - 1`.

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

namespace {

constexpr int QK_K = 256;  // src/kquants.jl:1

enum GgmlType : int { T_F32 = 0, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14 };  // src/load_gguf.jl:26-42

// ---- block layouts (src/kquants.jl:7-42); all are packed C structs -----------------
#pragma pack(push, 1)
struct block_q4_K {      // 144 bytes, src/kquants.jl:7-12
    uint16_t d, dmin;    // fp16
    uint8_t scales[12];
    uint8_t qs[128];
};
struct block_q5_K {      // 176 bytes, src/kquants.jl:18-24
    uint16_t d, dmin;
    uint8_t scales[12];
    uint8_t qh[32];
    uint8_t qs[128];
};
struct block_q6_K {      // 210 bytes, src/kquants.jl:30-35
    uint8_t ql[128];
    uint8_t qh[64];
    int8_t scales[16];
    uint16_t d;
};
#pragma pack(pop)
static_assert(sizeof(block_q4_K) == 144, "q4_K");
static_assert(sizeof(block_q5_K) == 176, "q5_K");
static_assert(sizeof(block_q6_K) == 210, "q6_K");

inline size_t block_bytes(int type) {
    switch (type) {
        case T_Q4_K: return 144;
        case T_Q5_K: return 176;
        case T_Q6_K: return 210;
        default: return 0;
    }
}

// IEEE binary16 -> binary32, exact (what Julia's Float32(::Float16) does).
inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {  // subnormal: normalise
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// 6-bit scale / min of sub-block j (0..7) of a q4_K / q5_K super-block.
// src/kquants.jl:80-81,86-87 (j<4) and :102-103,108-109 (j>=4), indices shifted to 0-based.
inline void scale_min_k4(int j, const uint8_t* s, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = s[j] & 63;
        *m = s[j + 4] & 63;
    } else {
        *sc = (uint8_t)((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4));
        *m = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

// ---- dequantize! -----------------------------------------------------------------
// src/kquants.jl:70-125.  y = fl(fl(d*sc) * q) - fl(dmin*m): two roundings, no FMA.
void dequant_q4_K(const block_q4_K* x, int64_t nb, float* y) {
    for (int64_t i = 0; i < nb; ++i) {
        const float d = f16_to_f32(x[i].d), dmin = f16_to_f32(x[i].dmin);
        const uint8_t* q = x[i].qs;
        for (int p = 0; p < 4; ++p) {
            uint8_t sc, m;
            scale_min_k4(2 * p, x[i].scales, &sc, &m);
            const float d1 = d * (float)sc, m1 = dmin * (float)m;
            scale_min_k4(2 * p + 1, x[i].scales, &sc, &m);
            const float d2 = d * (float)sc, m2 = dmin * (float)m;
            float* yo = y + QK_K * i + 64 * p;
            for (int l = 0; l < 32; ++l) yo[l] = d1 * (float)(q[32 * p + l] & 0xF) - m1;
            for (int l = 0; l < 32; ++l) yo[32 + l] = d2 * (float)(q[32 * p + l] >> 4) - m2;
        }
    }
}

// src/kquants.jl:186-251.  The fifth bit of value 64p+l is bit 2p of qh[l]; of 64p+32+l, bit 2p+1.
void dequant_q5_K(const block_q5_K* x, int64_t nb, float* y) {
    for (int64_t i = 0; i < nb; ++i) {
        const float d = f16_to_f32(x[i].d), dmin = f16_to_f32(x[i].dmin);
        const uint8_t* ql = x[i].qs;
        const uint8_t* qh = x[i].qh;
        uint8_t u1 = 1, u2 = 2;
        for (int p = 0; p < 4; ++p) {
            uint8_t sc, m;
            scale_min_k4(2 * p, x[i].scales, &sc, &m);
            const float d1 = d * (float)sc, m1 = dmin * (float)m;
            scale_min_k4(2 * p + 1, x[i].scales, &sc, &m);
            const float d2 = d * (float)sc, m2 = dmin * (float)m;
            float* yo = y + QK_K * i + 64 * p;
            for (int l = 0; l < 32; ++l)
                yo[l] = d1 * (float)(uint8_t)((ql[32 * p + l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - m1;
            for (int l = 0; l < 32; ++l)
                yo[32 + l] = d2 * (float)(uint8_t)((ql[32 * p + l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
            u1 <<= 2;
            u2 <<= 2;
        }
    }
}

// src/kquants.jl:322-363.  y = fl(d * float(scale*q)); the integer product is exact.
void dequant_q6_K(const block_q6_K* x, int64_t nb, float* y) {
    for (int64_t i = 0; i < nb; ++i) {
        const float d = f16_to_f32(x[i].d);
        for (int n = 0; n < 2; ++n) {
            const uint8_t* ql = x[i].ql + 64 * n;
            const uint8_t* qh = x[i].qh + 32 * n;
            const int8_t* sc = x[i].scales + 8 * n;
            float* yo = y + QK_K * i + 128 * n;
            for (int l = 0; l < 32; ++l) {
                const int is = l / 16;
                const int q1 = (int)(int8_t)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                const int q2 = (int)(int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                const int q3 = (int)(int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                const int q4 = (int)(int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                yo[l + 0] = d * (float)((int)sc[is + 0] * q1);
                yo[l + 32] = d * (float)((int)sc[is + 2] * q2);
                yo[l + 64] = d * (float)((int)sc[is + 4] * q3);
                yo[l + 96] = d * (float)((int)sc[is + 6] * q4);
            }
        }
    }
}

void dequant_any(int type, const void* blocks, int64_t nb, float* y) {
    switch (type) {
        case T_F32: std::memcpy(y, blocks, (size_t)nb * sizeof(float)); break;  // src/kquants.jl:44-47 (nb = element count)
        case T_Q4_K: dequant_q4_K((const block_q4_K*)blocks, nb, y); break;
        case T_Q5_K: dequant_q5_K((const block_q5_K*)blocks, nb, y); break;
        case T_Q6_K: dequant_q6_K((const block_q6_K*)blocks, nb, y); break;
    }
}

// ---- vecdot ----------------------------------------------------------------------
// src/kquants.jl:127-184, :253-320, :365-408: sum_k x[k] * w[k] with w[k] the exact
// dequantised weight, the product a strict f32 multiply, the accumulation `add_fast`
// (order left to the compiler).  Three accumulation orders are offered:
//   ACC_SEQ   one f32 accumulator in the source's loop order,
//   ACC_LANES 16 f32 partial sums by k mod 16, folded at the end (what a vectorising
//             compiler makes of add_fast; this is the timed CPU baseline),
//   ACC_F64   one f64 accumulator (bounds the reassociation noise of the other two).
enum { ACC_SEQ = 0, ACC_LANES = 1, ACC_F64 = 2 };

template <typename Acc>
inline Acc dot_seq(const float* w, const float* x, int n, Acc s) {
    for (int k = 0; k < n; ++k) s += (Acc)(x[k] * w[k]);
    return s;
}

double vecdot_blocks(int type, const uint8_t* blocks, int64_t nb, const float* x, int acc) {
    float w[QK_K];
    const size_t bb = block_bytes(type);
    if (acc == ACC_SEQ) {
        float s = 0.f;
        for (int64_t i = 0; i < nb; ++i) {
            dequant_any(type, blocks + i * bb, 1, w);
            s = dot_seq<float>(w, x + i * QK_K, QK_K, s);
        }
        return (double)s;
    } else if (acc == ACC_F64) {
        double s = 0.0;
        for (int64_t i = 0; i < nb; ++i) {
            dequant_any(type, blocks + i * bb, 1, w);
            s = dot_seq<double>(w, x + i * QK_K, QK_K, s);
        }
        return s;
    } else {
        float lanes[16] = {0};
        for (int64_t i = 0; i < nb; ++i) {
            dequant_any(type, blocks + i * bb, 1, w);
            const float* xi = x + i * QK_K;
            for (int k = 0; k < QK_K; k += 16)
                for (int j = 0; j < 16; ++j) lanes[j] += xi[k + j] * w[k + j];
        }
        for (int w2 = 8; w2 >= 1; w2 >>= 1)
            for (int j = 0; j < w2; ++j) lanes[j] += lanes[j + w2];
        return (double)lanes[0];
    }
}

double vecdot_f32(const float* w, const float* x, int64_t n, int acc) {
    if (acc == ACC_SEQ) {
        float s = 0.f;
        for (int64_t k = 0; k < n; ++k) s += x[k] * w[k];
        return s;
    } else if (acc == ACC_F64) {
        double s = 0.0;
        for (int64_t k = 0; k < n; ++k) s += (double)(x[k] * w[k]);
        return s;
    } else {
        float lanes[16] = {0};
        int64_t k = 0;
        for (; k + 16 <= n; k += 16)
            for (int j = 0; j < 16; ++j) lanes[j] += x[k + j] * w[k + j];
        for (; k < n; ++k) lanes[k & 15] += x[k] * w[k];
        for (int w2 = 8; w2 >= 1; w2 >>= 1)
            for (int j = 0; j < w2; ++j) lanes[j] += lanes[j + w2];
        return (double)lanes[0];
    }
}

// ---- matmul! ---------------------------------------------------------------------
// src/matmul.jl:3-23: y .= A' * x with A stored (in, out) column-major, i.e. output row i
// owns `in` contiguous weights (in/256 contiguous super-blocks).  The k-quant method is a
// static partition of the output rows over threads (Threads.@threads, :18); the f32
// method is a BLAS gemv whose summation order is the library's own.
template <typename Out>
void matmul_any(int type, const void* W, int64_t in, int64_t out, const float* x, Out* y, int acc,
                int nthreads) {
    const uint8_t* base = (const uint8_t*)W;
    const size_t row_bytes = (type == T_F32) ? (size_t)in * 4 : (size_t)(in / QK_K) * block_bytes(type);
    auto work = [&](int64_t r0, int64_t r1) {
        for (int64_t i = r0; i < r1; ++i) {
            double v = (type == T_F32) ? vecdot_f32((const float*)(base + i * row_bytes), x, in, acc)
                                       : vecdot_blocks(type, base + i * row_bytes, in / QK_K, x, acc);
            y[i] = (Out)v;
        }
    };
    if (nthreads <= 1 || out < 2 * nthreads) {
        work(0, out);
        return;
    }
    std::vector<std::thread> th;
    const int64_t per = (out + nthreads - 1) / nthreads;
    for (int t = 0; t < nthreads; ++t) {
        int64_t r0 = t * per, r1 = std::min<int64_t>(out, r0 + per);
        if (r0 < r1) th.emplace_back(work, r0, r1);
    }
    for (auto& t : th) t.join();
}

// ---- small ops -------------------------------------------------------------------
// src/inference.jl:102-110.  ss = dot(x,x)/n + 1f-5; ss = 1/sqrt(ss); o = w .* (ss .* x).
// The dot is accumulated in f64 and rounded once (BLAS leaves the order unspecified).
void rmsnorm(float* o, const float* x, const float* w, int64_t n) {
    double acc = 0.0;
    for (int64_t i = 0; i < n; ++i) acc += (double)(x[i] * x[i]);
    float ss = (float)acc;
    ss /= (float)n;
    ss += 1e-5f;
    ss = 1.0f / std::sqrt(ss);
    for (int64_t i = 0; i < n; ++i) o[i] = w[i] * (ss * x[i]);
}

// theta_scale = base ^ (-(1/Float32(hs/2))) in f32 (src/inference.jl:119,140); Julia's f32
// pow evaluates in f64 and rounds once, as does this.
float rope_theta_scale(float base, int head_size_div2) {
    const float e = -(1.0f / (float)head_size_div2);
    return (float)std::pow((double)base, (double)e);
}

// (cos, sin) of the iterated f32 angle: theta_0 = Float32(pos0); theta_{i+1} = theta_i * scale
// (src/inference.jl:122-127,143-153).  cis(::Float32) is evaluated in f64 and rounded.
void rope_table_row(float* cs, int head_size_div2, int pos0, float base) {
    const float scale = rope_theta_scale(base, head_size_div2);
    float theta = 1.0f * (float)pos0;
    for (int i = 0; i < head_size_div2; ++i) {
        cs[2 * i] = (float)std::cos((double)theta);
        cs[2 * i + 1] = (float)std::sin((double)theta);
        theta *= scale;
    }
}

// src/inference.jl:112-167.  x is [n_heads][head_size].  normal: pairs (2i, 2i+1); neox: (i, i+hs/2).
// (a+bi)(c+di) = (ac - bd) + (ad + bc)i with each product and sum rounded separately.
void rope(float* x, int head_size, int n_heads, int pos0, float base, int neox) {
    const int h2 = head_size / 2;
    std::vector<float> cs(2 * h2);
    rope_table_row(cs.data(), h2, pos0, base);
    for (int h = 0; h < n_heads; ++h) {
        float* xh = x + (size_t)h * head_size;
        for (int i = 0; i < h2; ++i) {
            const int ia = neox ? i : 2 * i, ib = neox ? i + h2 : 2 * i + 1;
            const float a = xh[ia], b = xh[ib], c = cs[2 * i], s = cs[2 * i + 1];
            xh[ia] = a * c - b * s;
            xh[ib] = a * s + b * c;
        }
    }
}

// src/inference.jl:169-174.
void softmax(float* x, int64_t n) {
    float mx = x[0];
    for (int64_t i = 1; i < n; ++i) mx = std::max(mx, x[i]);
    float sum = 0.f;
    for (int64_t i = 0; i < n; ++i) {
        x[i] = std::exp(x[i] - mx);
        sum += x[i];
    }
    for (int64_t i = 0; i < n; ++i) x[i] /= sum;
}

struct Config {  // src/inference.jl:1-11
    int32_t dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len;
    float rope_freq_base;
    int32_t rope_is_neox;
};

struct Tensor {
    int type = T_F32;
    const void* data = nullptr;  // borrowed
    int64_t in = 0, out = 0;
};

enum Role { R_TOK_EMB = 0, R_RMS_ATT, R_WQ, R_WK, R_WV, R_WO, R_RMS_FFN, R_W1, R_W2, R_W3, R_RMS_FINAL, R_OUTPUT, R_COUNT };

struct Model {
    Config c;
    Tensor tok_emb, rms_final, output;
    std::vector<Tensor> per_layer[R_COUNT];
};

struct State {  // src/inference.jl:62-100; caches zero-initialised
    std::vector<float> x, xb, xb2, hb, hb2, q, k, v, att, logits;
    // key cache (head_size, n_kv, seq) -> [pos][kv][hs]; value cache (seq, hs, n_kv) -> [kv][hs][pos]
    std::vector<std::vector<float>> kc, vc;
};

// src/inference.jl:176-197: att[t,h] = sum_i q[i,h] * K[i,kvh,t]; sequential f32 over i.
void attention_weights(float* att, const float* kc, const float* q, int pos_count, int n_heads, int n_kv,
                       int hs) {
    const int n_gqa = n_heads / n_kv;
    for (int h = 0; h < n_heads; ++h) {
        const int kvh = h / n_gqa;
        for (int t = 0; t < pos_count; ++t) {
            const float* kp = kc + ((size_t)t * n_kv + kvh) * hs;
            float s = 0.f;
            for (int i = 0; i < hs; ++i) s += q[(size_t)h * hs + i] * kp[i];
            att[(size_t)h * pos_count + t] = s;
        }
    }
}

// src/inference.jl:199-220: xb[i,h] = sum_t att[t,h] * V[t,i,kvh]; sequential f32 over t.
void combine_values(float* xb, const float* vc, const float* att, int pos_count, int seq_len, int n_heads,
                    int n_kv, int hs) {
    const int n_gqa = n_heads / n_kv;
    for (int h = 0; h < n_heads; ++h) {
        const int kvh = h / n_gqa;
        for (int i = 0; i < hs; ++i) {
            const float* vp = vc + ((size_t)kvh * hs + i) * seq_len;
            float s = 0.f;
            for (int t = 0; t < pos_count; ++t) s += att[(size_t)h * pos_count + t] * vp[t];
            xb[(size_t)h * hs + i] = s;
        }
    }
}

void mm(const Tensor& t, const float* x, float* y, int acc, int nthreads) {
    matmul_any<float>(t.type, t.data, t.in, t.out, x, y, acc, nthreads);
}

// src/inference.jl:222-315.
void transformer(const Model& m, State& s, int token0, int pos0, int acc, int nthreads) {
    const Config& c = m.c;
    const int dim = c.dim, hs = dim / c.n_heads, kv_dim = hs * c.n_kv_heads;
    const int npos = pos0 + 1;
    // :236 token embedding row -> x
    if (m.tok_emb.type == T_F32)
        std::memcpy(s.x.data(), (const float*)m.tok_emb.data + (size_t)token0 * dim, (size_t)dim * 4);
    else
        dequant_any(m.tok_emb.type,
                    (const uint8_t*)m.tok_emb.data + (size_t)token0 * (dim / QK_K) * block_bytes(m.tok_emb.type),
                    dim / QK_K, s.x.data());
    for (int l = 0; l < c.n_layers; ++l) {
        rmsnorm(s.xb.data(), s.x.data(), (const float*)m.per_layer[R_RMS_ATT][l].data, dim);  // :244
        mm(m.per_layer[R_WQ][l], s.xb.data(), s.q.data(), acc, nthreads);                      // :247-249
        mm(m.per_layer[R_WK][l], s.xb.data(), s.k.data(), acc, nthreads);
        mm(m.per_layer[R_WV][l], s.xb.data(), s.v.data(), acc, nthreads);
        rope(s.q.data(), hs, c.n_heads, pos0, c.rope_freq_base, c.rope_is_neox);  // :255-256
        rope(s.k.data(), hs, c.n_kv_heads, pos0, c.rope_freq_base, c.rope_is_neox);
        std::memcpy(s.kc[l].data() + (size_t)pos0 * kv_dim, s.k.data(), (size_t)kv_dim * 4);  // :259
        for (int j = 0; j < kv_dim; ++j) s.vc[l][(size_t)j * c.seq_len + pos0] = s.v[j];       // :260
        attention_weights(s.att.data(), s.kc[l].data(), s.q.data(), npos, c.n_heads, c.n_kv_heads, hs);  // :266
        const float sq = std::sqrt((float)hs);
        for (size_t i = 0; i < (size_t)npos * c.n_heads; ++i) s.att[i] /= sq;  // :268
        for (int h = 0; h < c.n_heads; ++h) softmax(s.att.data() + (size_t)h * npos, npos);  // :270-273
        combine_values(s.xb.data(), s.vc[l].data(), s.att.data(), npos, c.seq_len, c.n_heads, c.n_kv_heads, hs);  // :278
        mm(m.per_layer[R_WO][l], s.xb.data(), s.xb2.data(), acc, nthreads);  // :281
        for (int i = 0; i < dim; ++i) s.x[i] += s.xb2[i];                      // :284
        rmsnorm(s.xb.data(), s.x.data(), (const float*)m.per_layer[R_RMS_FFN][l].data, dim);  // :287
        mm(m.per_layer[R_W1][l], s.xb.data(), s.hb.data(), acc, nthreads);   // :291-292
        mm(m.per_layer[R_W3][l], s.xb.data(), s.hb2.data(), acc, nthreads);
        for (int i = 0; i < c.hidden_dim; ++i) {  // :295-299
            s.hb[i] = s.hb[i] * (1.0f / (1.0f + std::exp(-s.hb[i])));
            s.hb[i] *= s.hb2[i];
        }
        mm(m.per_layer[R_W2][l], s.hb.data(), s.xb.data(), acc, nthreads);  // :302
        for (int i = 0; i < dim; ++i) s.x[i] += s.xb[i];                     // :305
    }
    rmsnorm(s.x.data(), s.x.data(), (const float*)m.rms_final.data, dim);  // :309
    mm(m.output, s.x.data(), s.logits.data(), acc, nthreads);              // :312
}

}  // namespace

// ---------------------------------------------------------------------------------
extern "C" {

int64_t orc_block_bytes(int type) { return (int64_t)block_bytes(type); }

void orc_dequantize(int type, const void* blocks, int64_t nblocks, float* out) { dequant_any(type, blocks, nblocks, out); }

double orc_vecdot(int type, const void* blocks, int64_t n_in, const float* x, int acc) {
    if (type == T_F32) return vecdot_f32((const float*)blocks, x, n_in, acc);
    return vecdot_blocks(type, (const uint8_t*)blocks, n_in / QK_K, x, acc);
}

void orc_matmul(int type, const void* W, int64_t in, int64_t out, const float* x, float* y, int acc, int nthreads) {
    matmul_any<float>(type, W, in, out, x, y, acc, nthreads);
}

void orc_matmul_f64(int type, const void* W, int64_t in, int64_t out, const float* x, double* y, int nthreads) {
    matmul_any<double>(type, W, in, out, x, y, ACC_F64, nthreads);
}

void orc_rmsnorm(float* o, const float* x, const float* w, int64_t n) { rmsnorm(o, x, w, n); }
void orc_rope(float* x, int head_size, int n_heads, int pos0, float base, int neox) { rope(x, head_size, n_heads, pos0, base, neox); }
void orc_rope_table_row(float* cs, int head_size_div2, int pos0, float base) { rope_table_row(cs, head_size_div2, pos0, base); }
void orc_softmax(float* x, int64_t n) { softmax(x, n); }

// One attention block as in src/inference.jl:263-278 on caller-supplied caches.
// kc: [npos][n_kv][hs]; vc: [n_kv][hs][seq_len]; q: [n_heads][hs]; out: [n_heads][hs].
void orc_attention(float* out, const float* q, const float* kc, const float* vc, int npos, int seq_len, int n_heads,
                   int n_kv, int hs) {
    std::vector<float> att((size_t)npos * n_heads);
    attention_weights(att.data(), kc, q, npos, n_heads, n_kv, hs);
    const float sq = std::sqrt((float)hs);
    for (auto& a : att) a /= sq;
    for (int h = 0; h < n_heads; ++h) softmax(att.data() + (size_t)h * npos, npos);
    combine_values(out, vc, att.data(), npos, seq_len, n_heads, n_kv, hs);
}

// hb = silu(hb) .* hb2, src/inference.jl:295-299.
void orc_swiglu(float* hb, const float* hb2, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        hb[i] = hb[i] * (1.0f / (1.0f + std::exp(-hb[i])));
        hb[i] *= hb2[i];
    }
}

// Julia argmax: first maximal index (src/inference.jl:360).  0-based here.
int64_t orc_argmax(const float* x, int64_t n) {
    int64_t best = 0;
    for (int64_t i = 1; i < n; ++i)
        if (x[i] > x[best]) best = i;
    return best;
}

// Temperature sampling, src/inference.jl:361-368: logits ./= T; softmax!; wsample(1:n, p).
// StatsBase.sample(rng, ::AbstractWeights) (third-party, version not pinned by the reference's
// Project.toml) draws t = rand()*sum(w) and walks the cumulative sum until cw >= t.  The
// uniform variate is supplied by the caller here because Julia's global RNG stream cannot
// be reproduced elsewhere.  `logits` is overwritten with the probabilities.  Returns 0-based index.
int64_t orc_sample_temperature(float* logits, int64_t n, float temperature, double u) {
    for (int64_t i = 0; i < n; ++i) logits[i] /= temperature;
    softmax(logits, n);
    double total = 0.0;
    for (int64_t i = 0; i < n; ++i) total += logits[i];
    const double t = u * total;
    int64_t i = 0;
    double cw = logits[0];
    while (cw < t && i < n - 1) {
        ++i;
        cw += logits[i];
    }
    return i;
}

void* orc_model_create(const Config* c) {
    Model* m = new Model();
    m->c = *c;
    for (int r = 0; r < R_COUNT; ++r) m->per_layer[r].resize(c->n_layers);
    return m;
}
void orc_model_destroy(void* m) { delete (Model*)m; }

// Host memory is borrowed for the model's lifetime (the oracle never copies weights).
int orc_model_set_tensor(void* mp, int role, int layer, int type, const void* data, int64_t in, int64_t out) {
    Model* m = (Model*)mp;
    Tensor t;
    t.type = type; t.data = data; t.in = in; t.out = out;
    if (role == R_TOK_EMB) m->tok_emb = t;
    else if (role == R_RMS_FINAL) m->rms_final = t;
    else if (role == R_OUTPUT) m->output = t;
    else if (role > 0 && role < R_COUNT && layer >= 0 && layer < m->c.n_layers) m->per_layer[role][layer] = t;
    else return 1;
    return 0;
}

void* orc_state_create(void* mp) {
    const Config& c = ((Model*)mp)->c;
    State* s = new State();
    const int hs = c.dim / c.n_heads, kv_dim = hs * c.n_kv_heads;
    s->x.assign(c.dim, 0.f); s->xb.assign(c.dim, 0.f); s->xb2.assign(c.dim, 0.f);
    s->hb.assign(c.hidden_dim, 0.f); s->hb2.assign(c.hidden_dim, 0.f);
    s->q.assign(c.dim, 0.f); s->k.assign(kv_dim, 0.f); s->v.assign(kv_dim, 0.f);
    s->att.assign((size_t)c.seq_len * c.n_heads, 0.f);
    s->logits.assign(c.vocab_size, 0.f);
    s->kc.resize(c.n_layers); s->vc.resize(c.n_layers);
    for (int l = 0; l < c.n_layers; ++l) {
        s->kc[l].assign((size_t)c.seq_len * kv_dim, 0.f);
        s->vc[l].assign((size_t)c.seq_len * kv_dim, 0.f);
    }
    return s;
}
void orc_state_destroy(void* s) { delete (State*)s; }

// transformer!(token, pos, ...) with 0-based token/pos; logits copied out when non-null.
void orc_transformer(void* m, void* s, int token0, int pos0, int acc, int nthreads, float* logits_out) {
    transformer(*(Model*)m, *(State*)s, token0, pos0, acc, nthreads);
    if (logits_out) std::memcpy(logits_out, ((State*)s)->logits.data(), ((State*)s)->logits.size() * 4);
}

// Copy an internal buffer for stage-by-stage comparison: 0=x 1=xb 2=q 3=k 4=v 5=hb 6=logits.
int64_t orc_state_read(void* sp, int which, float* out, int64_t cap) {
    State* s = (State*)sp;
    const std::vector<float>* v = nullptr;
    switch (which) {
        case 0: v = &s->x; break; case 1: v = &s->xb; break; case 2: v = &s->q; break; case 3: v = &s->k; break;
        case 4: v = &s->v; break; case 5: v = &s->hb; break; case 6: v = &s->logits; break; default: return -1;
    }
    const int64_t n = std::min<int64_t>(cap, (int64_t)v->size());
    std::memcpy(out, v->data(), (size_t)n * 4);
    return (int64_t)v->size();
}

// The loop of `sample` (src/inference.jl:349-385) for temperature 0, stop_on_special_token=false:
// positions 0..n_positions-1; teacher-forced while inside the prompt, argmax afterwards.
// out_tokens[pos0] = the token chosen after position pos0 (0-based ids).  If logits_out is
// non-null it receives n_positions * vocab floats.  Returns seconds spent in the loop.
double orc_sample_greedy(void* mp, const int32_t* prompt, int n_prompt, int n_positions, int32_t* out_tokens,
                         float* logits_out, int acc, int nthreads) {
    Model* m = (Model*)mp;
    State* s = (State*)orc_state_create(mp);
    auto t0 = std::chrono::steady_clock::now();
    int token = prompt[0];
    for (int pos0 = 0; pos0 < n_positions; ++pos0) {
        transformer(*m, *s, token, pos0, acc, nthreads);
        if (logits_out) std::memcpy(logits_out + (size_t)pos0 * m->c.vocab_size, s->logits.data(), (size_t)m->c.vocab_size * 4);
        int next = (pos0 + 1 < n_prompt) ? prompt[pos0 + 1] : (int)orc_argmax(s->logits.data(), m->c.vocab_size);
        out_tokens[pos0] = next;
        token = next;
    }
    double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    orc_state_destroy(s);
    return dt;
}

int orc_hardware_threads() { return (int)std::thread::hardware_concurrency(); }

}  // extern "C"
