// Shared device helpers: PTX wrappers for bulk asynchronous copies (TMA), mbarriers,
// programmatic dependent launch, and small warp utilities.  sm_100a only.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace l2b {

constexpr int QK_K = 256;
enum : int { T_F32 = 0, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14 };

// Bytes of one super-block as stored on the DEVICE.  q4_K and q5_K keep the file layout
// (144 / 176 bytes).  q6_K is split at upload into a 208-byte record (ql[128] qh[64]
// scales[16]) and a separate fp16 array of the super-block scales `d`, because a 210-byte
// stride is only 2-byte aligned; total bytes per block are unchanged (210).
__host__ __device__ constexpr int dev_block_bytes(int type) {
    return type == T_Q4_K ? 144 : type == T_Q5_K ? 176 : type == T_Q6_K ? 208 : 0;
}
__host__ __device__ constexpr int file_block_bytes(int type) {
    return type == T_Q4_K ? 144 : type == T_Q5_K ? 176 : type == T_Q6_K ? 210 : 0;
}

// Error codes written to a session's device status word by kernels (0 = fine).
enum : int { DEV_OK = 0, DEV_ERR_TMA_TIMEOUT = 1, DEV_ERR_BAD_INDEX = 2, DEV_ERR_PEER_TIMEOUT = 3 };

// Upper bound on polls of an mbarrier before a kernel gives up.  A poll is a test plus a short sleep
// (tens of nanoseconds), so this is a few tenths of a second: far beyond any legitimate wait
// (microseconds), short enough that a protocol bug costs little.
constexpr uint32_t MBAR_MAX_POLLS = 4u * 1000u * 1000u;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: a non-blocking test in a spin loop.  (The potentially-blocking try_wait form was measured to
// wake its waiters late, about a microsecond after the phase completed, which is as long as a whole tile.)
// Returns false when the poll budget ran out.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < MBAR_MAX_POLLS; ++i) {
        if (mbar_test_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(32);
    }
    return false;
}

// The same wait bounded by TIME (nanoseconds of %globaltimer) instead of by polls: for warps whose partner may itself be
// inside a long, legitimate wait (the tensor-parallel wait for another GPU's partial results).
__device__ __forceinline__ bool mbar_wait_bounded_ns(uint64_t* bar, uint32_t parity, unsigned long long limit_ns) {
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (mbar_test_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(64);
        if ((i & 1023u) == 1023u) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > limit_ns) return false;
        }
    }
}

// Volatile vector accesses for words that another GPU writes or reads while this kernel runs (tensor-parallel exchange):
// each 8-byte half {value, tag} of a 16-byte access is written and read as a unit, so a value is valid when its tag is.
__device__ __forceinline__ uint4 ld_volatile_u32x4(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile_u32x4(uint4* p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_volatile_u32x2(uint2* p, uint2 v) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// L2 policy for weight bytes: they are read once per token, so they should not evict the
// activations and KV cache that live in L2 between kernels.
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// Bulk asynchronous copy global -> shared (the 1-D form of TMA).  dst, src 16-byte aligned,
// bytes a multiple of 16.  Completion is signalled on `bar` as transaction bytes.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// Programmatic dependent launch: let the next kernel in the stream start its prologue,
// and wait until the previous kernel's memory is visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h16) { return __half2float(__ushort_as_half((unsigned short)h16)); }

}  // namespace l2b
