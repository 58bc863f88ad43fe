// Seeded synthetic data for tests and benchmarks (libl2b_synth.so; not part of the product library): counter-based, integer arithmetic only, so
// the same seed gives the same bytes on every machine and compiler.
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "../../include/l2b_synth.h"
#include "../../include/llama2_b200.h"  // status and tensor-type enums only

namespace {

inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
inline uint64_t draw(uint64_t seed, uint64_t idx) { return splitmix64(splitmix64(seed) ^ (idx * 0xD1342543DE82EF95ull + 0x632BE59BD9B4E019ull)); }

// ~N(0,1): sum of twelve 16-bit uniforms, centred (Irwin-Hall); exact in f32 up to the final scaling.
inline float std_normal(uint64_t seed, uint64_t idx) {
    uint32_t s = 0;
    for (int j = 0; j < 3; ++j) {
        const uint64_t r = draw(seed, 3 * idx + j);
        s += (uint32_t)(r & 0xFFFF) + (uint32_t)((r >> 16) & 0xFFFF) + (uint32_t)((r >> 32) & 0xFFFF) + (uint32_t)((r >> 48) & 0xFFFF);
    }
    return (float)((int32_t)s - 6 * 65535) * (1.0f / 65536.0f);
}

// f32 -> f16, round to nearest even, for non-negative finite values below the f16 range limit.
inline uint16_t f32_to_f16_pos(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const int32_t e = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
    uint32_t m = x & 0x7FFFFFu;
    if (e >= 31) return 0x7BFF;  // clamp to the largest finite half
    if (e <= 0) {                // subnormal half
        if (e < -10) return 0;
        m |= 0x800000u;
        const int shift = 14 - e;
        uint32_t h = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1), halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (h & 1))) ++h;
        return (uint16_t)h;
    }
    uint32_t h = ((uint32_t)e << 10) | (m >> 13);
    const uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;
    return (uint16_t)h;
}

template <typename F>
void parallel_for(int64_t n, F f) {
    const unsigned hw = std::max(1u, std::thread::hardware_concurrency());
    const int64_t min_chunk = 1 << 16;
    const int nt = (int)std::max<int64_t>(1, std::min<int64_t>(hw, n / min_chunk));
    if (nt == 1) {
        f(0, n);
        return;
    }
    std::vector<std::thread> th;
    const int64_t per = (n + nt - 1) / nt;
    for (int t = 0; t < nt; ++t) {
        const int64_t a = t * per, b = std::min(n, a + per);
        if (a < b) th.emplace_back(f, a, b);
    }
    for (auto& t : th) t.join();
}

}  // namespace

extern "C" int32_t l2b_synth_f32(float* out, int64_t n, uint64_t seed, float std_dev, int32_t constant) {
    if (!out || n < 0) return L2B_ERR_BAD_ARG;
    parallel_for(n, [&](int64_t a, int64_t b) {
        for (int64_t i = a; i < b; ++i) out[i] = constant ? std_dev : std_normal(seed, (uint64_t)i) * std_dev;
    });
    return L2B_OK;
}

extern "C" int32_t l2b_synth_kquant(int32_t type, void* out, int64_t n_blocks, uint64_t seed) {
    if (!out || n_blocks < 0) return L2B_ERR_BAD_ARG;
    const int bb = type == L2B_TYPE_Q4_K ? 144 : type == L2B_TYPE_Q5_K ? 176 : type == L2B_TYPE_Q6_K ? 210 : 0;
    if (!bb) return L2B_ERR_UNSUPPORTED_TYPE;
    uint8_t* base = (uint8_t*)out;
    parallel_for(n_blocks, [&](int64_t a, int64_t b) {
        for (int64_t i = a; i < b; ++i) {
            uint8_t* blk = base + i * bb;
            uint8_t tmp[216];
            for (int w = 0; w < 27; ++w) {
                const uint64_t r = draw(seed, (uint64_t)i * 32 + w);
                std::memcpy(tmp + 8 * w, &r, 8);
            }
            std::memcpy(blk, tmp, bb);
            // fp16 super-block scales: |N(0, 0.01^2)|
            auto half_abs_normal = [&](int j) {
                float z = std_normal(seed ^ 0x5DEECE66Dull, (uint64_t)i * 2 + j) * 0.01f;
                if (z < 0) z = -z;
                return f32_to_f16_pos(z);
            };
            if (type == L2B_TYPE_Q6_K) {
                const uint16_t d = half_abs_normal(0);
                std::memcpy(blk + 208, &d, 2);
            } else {
                const uint16_t d = half_abs_normal(0), dm = half_abs_normal(1);
                std::memcpy(blk, &d, 2);
                std::memcpy(blk + 2, &dm, 2);
            }
        }
    });
    return L2B_OK;
}

extern "C" int32_t l2b_synth_tokens(int32_t* out, int64_t n, uint64_t seed, int32_t lo, int32_t hi) {
    if (!out || n < 0 || hi <= lo) return L2B_ERR_BAD_ARG;
    const uint64_t span = (uint64_t)(hi - lo);
    for (int64_t i = 0; i < n; ++i) out[i] = lo + (int32_t)(draw(seed, (uint64_t)i) % span);
    return L2B_OK;
}
