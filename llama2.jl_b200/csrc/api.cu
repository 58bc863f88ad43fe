// C ABI of the library (see include/llama2_b200.h): model / session objects, the captured
// per-token CUDA graph, and the isolated-operator entry points.
#include "../../include/llama2_b200.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "gguf_reader.h"
#include "attention.cuh"
#include "fused_matvec.cuh"
#include "sampling.cuh"
#include "small_ops.cuh"
#include "kq_gemm.cuh"
#include "prefill_ops.cuh"
#include "token_kernel.cuh"

using namespace l2b;

// ---------------------------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------------------------
static thread_local std::string g_last_error;

static int32_t fail(int32_t code, const std::string& msg) {
    g_last_error = msg;
    return code;
}
// for the other translation units of the library (tokenizer.cpp)
int32_t l2b_internal_fail(int32_t code, const std::string& msg) { return fail(code, msg); }

#define CU(call)                                                                                         \
    do {                                                                                                 \
        cudaError_t e_ = (call);                                                                         \
        if (e_ != cudaSuccess) {                                                                         \
            (void)cudaGetLastError();                                                                    \
            return fail(e_ == cudaErrorMemoryAllocation ? L2B_ERR_OOM : L2B_ERR_CUDA,                    \
                        std::string(#call) + ": " + cudaGetErrorString(e_) + " (" + __FILE__ + ":" + std::to_string(__LINE__) + ")"); \
        }                                                                                                \
    } while (0)

#define L2B_TRY(expr)              \
    do {                           \
        int32_t s_ = (expr);       \
        if (s_ != L2B_OK) return s_; \
    } while (0)

static int32_t require_device() {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        (void)cudaGetLastError();
        return fail(L2B_ERR_NO_DEVICE, "no CUDA device is visible; this library has no CPU path");
    }
    return L2B_OK;
}

// ---------------------------------------------------------------------------------------------
// device matrices
// ---------------------------------------------------------------------------------------------
struct DevMatrix {
    int type = -1;
    int64_t in = 0, out = 0;
    uint8_t* data = nullptr;  // f32 rows, or block records
    __half* d6 = nullptr;     // q6_K super-block scales
    int64_t file_bytes = 0;   // bytes in the stored (file) format
    bool panels = false;      // k-quant rows longer than one stage, stored as column panels
    int kb = MV_TILE_BLOCKS;  // stage width in super-blocks this matrix is laid out for (panel width)
    bool present() const { return data != nullptr; }
};

static bool type_supported(int t) { return t == T_F32 || t == T_Q4_K || t == T_Q5_K || t == T_Q6_K; }

static void free_matrix(DevMatrix& m) {
    if (m.data) cudaFree(m.data);
    if (m.d6) cudaFree(m.d6);
    m = DevMatrix();
}

// Copy one matrix to the device (repacking q6_K).  `rows` x `in` weights.
// Rows longer than one stage (in > 4096) are re-ordered into column panels on the device (panelize_kernel) unless
// `panels` is false (matrices that are read row by row: the embedding table, plain dequantisation).
static long env_long(const char* name, long dflt);
// Stage width for a matrix: 16 super-blocks, or 8 where a row is exactly one 16-wide stage and 16-wide ring slots would leave
// fewer than four slots beside the activation planes (then only one group of consumer warps could work, on a ring three deep;
// measured on the q6_K classifier 128256 x 4096: 101.7 -> 88.3 us).  Longer rows keep 16: with 8-block stages the q5_K
// 4096 x 14336 matrix went from 16.5 to 18.5 us (twice the stages per tile, twice the per-stage synchronisation).
static int choose_stage_blocks(int type, int64_t in) {
    const int64_t nb = in / QK_K;
    if (type == T_F32 || nb != MV_TILE_BLOCKS) return MV_TILE_BLOCKS;
    const long slot16 = 4L * pad_32_mod_128(4 * MV_TILE_BLOCKS * dev_block_bytes(type));
    const long base = mv_smem_layout((int)in, 3, true, 0, 0).total;
    const long cap = std::min<long>(env_long("L2B_MV_SMEM_KB", 208) * 1024, 226 * 1024);
    if (env_long("L2B_MV_STAGE_BLOCKS", 0) == 8) return 8;
    if (env_long("L2B_MV_STAGE_BLOCKS", 0) == 16) return MV_TILE_BLOCKS;
    return (cap - base) / slot16 >= 4 ? MV_TILE_BLOCKS : 8;
}

static int32_t panelize(DevMatrix& m, cudaStream_t st) {
    const int64_t nb = m.in / QK_K;
    if (m.type == T_F32) return L2B_OK;
    m.kb = choose_stage_blocks(m.type, m.in);
    if (nb <= m.kb || m.out < 2) return L2B_OK;
    const int bb = dev_block_bytes(m.type);
    const size_t bytes = (size_t)nb * m.out * bb;
    uint8_t* dst = nullptr;
    CU(cudaMalloc(&dst, bytes));
    panelize_kernel<<<1184, 256, 0, st>>>(m.data, dst, (int)nb, m.out, bb, m.kb);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        cudaFree(dst);
        CU(e);
    }
    cudaFree(m.data);
    m.data = dst;
    m.panels = true;
    return L2B_OK;
}

static int32_t upload_matrix(DevMatrix& m, int type, const void* host, int64_t in, int64_t out, cudaStream_t st, bool panels = true) {
    if (!type_supported(type)) return fail(L2B_ERR_UNSUPPORTED_TYPE, "tensor type " + std::to_string(type) + " not implemented");
    if (!host || in <= 0 || out <= 0) return fail(L2B_ERR_BAD_ARG, "upload: null pointer or empty shape");
    if (type != T_F32 && in % QK_K != 0) return fail(L2B_ERR_BAD_ARG, "k-quant tensors need in_dim % 256 == 0");
    if (type == T_F32 && in % 8 != 0 && out > 1) return fail(L2B_ERR_BAD_ARG, "f32 matrices need in_dim % 8 == 0");
    free_matrix(m);
    m.type = type;
    m.in = in;
    m.out = out;
    if (type == T_F32) {
        m.file_bytes = in * out * 4;
        CU(cudaMalloc(&m.data, (size_t)m.file_bytes));
        CU(cudaMemcpyAsync(m.data, host, (size_t)m.file_bytes, cudaMemcpyHostToDevice, st));
        CU(cudaStreamSynchronize(st));
        return L2B_OK;
    }
    const int64_t nblocks = (in / QK_K) * out;
    m.file_bytes = nblocks * file_block_bytes(type);
    if (type != T_Q6_K) {
        CU(cudaMalloc(&m.data, (size_t)m.file_bytes));
        CU(cudaMemcpyAsync(m.data, host, (size_t)m.file_bytes, cudaMemcpyHostToDevice, st));
        CU(cudaStreamSynchronize(st));
        return panels ? panelize(m, st) : L2B_OK;
    }
    uint8_t* raw = nullptr;
    CU(cudaMalloc(&raw, (size_t)m.file_bytes));
    cudaError_t e = cudaMalloc(&m.data, (size_t)nblocks * 208);
    if (e == cudaSuccess) e = cudaMalloc(&m.d6, (size_t)nblocks * sizeof(__half));
    if (e == cudaSuccess) e = cudaMemcpyAsync(raw, host, (size_t)m.file_bytes, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) {
        repack_q6k_kernel<<<1184, 256, 0, st>>>(raw, m.data, m.d6, nblocks);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(raw);
    CU(e);
    return panels ? panelize(m, st) : L2B_OK;
}

// ---------------------------------------------------------------------------------------------
// kernel launch helpers
// ---------------------------------------------------------------------------------------------
struct DeviceInfo {
    int sms = 148;
    int max_smem_optin = 227 * 1024;
};

static int32_t query_device(DeviceInfo& di) {
    int dev = 0;
    CU(cudaGetDevice(&dev));
    CU(cudaDeviceGetAttribute(&di.sms, cudaDevAttrMultiProcessorCount, dev));
    CU(cudaDeviceGetAttribute(&di.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    return L2B_OK;
}

// cluster > 1: the grid is launched as thread-block clusters of that many consecutive blocks.
template <typename Kernel, typename Params>
static cudaError_t launch_kernel(Kernel k, dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, const Params& prm, int cluster = 1) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, k, prm);
}

static long env_long(const char* name, long dflt) {
    const char* v = getenv(name);
    return v && *v ? atol(v) : dflt;
}

// A fused matrix-vector launch, fully planned on the host.
struct MvLaunch {
    MvParams p;
    bool kq = true;
    int planes = 3;
    int nb = 1;  // activation vectors per launch (2: two prompt positions per pass)
    int kb = MV_TILE_BLOCKS;  // stage width the launch's matrices are laid out for
    int grid = 0, warps = 0;
    size_t smem = 0;
};

// Decide grid, consumer warps, ring slots and shared memory for a launch whose segments, n_in, prologue and
// epilogue fields are already filled in, and precompute the schedule constants the kernel would otherwise
// derive with serial integer arithmetic.
static int32_t plan_matvec(MvLaunch& L, const DeviceInfo& di) {
    MvParams& p = L.p;
    L.kq = p.seg[0].type != T_F32;
    for (int s = 0; s < p.nseg; ++s)
        if ((p.seg[s].type != T_F32) != L.kq) return fail(L2B_ERR_UNSUPPORTED_TYPE, "f32 and k-quant matrices cannot share one launch");
    p.planes = L.planes;
#ifdef L2B_MEASURE
    p.debug = (int)env_long("L2B_MV_DEBUG", 0);
#endif
    L.grid = di.sms;
    const int nb = p.n_in / QK_K;
    const int per_unit = L.kq ? MV_TILE_PAIRS : 1;
    int units = 0, max_bb = 0;
    for (int s = 0; s < p.nseg; ++s) {
        p.seg_start[s] = units;
        units += (p.seg[s].npairs + per_unit - 1) / per_unit;
        max_bb = std::max(max_bb, dev_block_bytes(p.seg[s].type));
        if (p.seg[s].pair_mode == PAIR_NEOX) {
            const int h2 = p.seg[s].head_size / 2;
            if (L.kq && h2 % MV_TILE_PAIRS != 0) return fail(L2B_ERR_BAD_ARG, "head_size must be a multiple of 16 for NeoX RoPE");
            p.neox_magic = (unsigned)((0x100000000ull + h2 - 1) / h2);
        }
    }
    p.seg_start[p.nseg] = units;
    if (units < L.grid) L.grid = std::max(1, units);
    p.units_lo = units / L.grid;
    p.units_rem = units % L.grid;
    if (!L.kq) {
        const int per_block = p.units_lo + (p.units_rem ? 1 : 0);
        const int W = std::max(4, std::min(MV_MAX_CONSUMERS, per_block));
        p.consumers = W;
        p.cgroups = 1;
        p.turns = (p.n_in / 8 + 32 * W - 1) / (32 * W);
        p.nit = 1;
        p.nslots = 0;
        p.row_stride = 0;
        L.warps = W;
        L.smem = mv_smem_layout(p.n_in, 1, false, 0, 0).total;
        if ((long)L.smem > di.max_smem_optin - 1024) return fail(L2B_ERR_BAD_ARG, "input vector too long for shared memory");
        return L2B_OK;
    }
    const int kb = std::min(nb, L.kb);  // super-blocks per row and stage
    p.kb = L.kb;
    p.nit = (nb + L.kb - 1) / L.kb;
    // a slot holds 16 rows of kb blocks in up to 16 copy groups, each padded to 32 mod 128 bytes
    p.row_stride = kb * max_bb + 128;
    for (int s = 0; s < p.nseg; ++s) mv_fill_geometry(p.seg[s], kb, p.nit);
    // ring: as many tile slots as the shared-memory budget allows
    long slot = 0;
    for (int s = 0; s < p.nseg; ++s) slot = std::max<long>(slot, (long)p.seg[s].ngroups * p.seg[s].gs);
    p.row_stride = (int)((slot + 15) / 16);
    p.row_stride += (16 - p.row_stride % 16) % 16;
    slot = 16L * p.row_stride;
    const long base = mv_smem_layout(p.n_in, L.planes, true, 0, p.row_stride, L.nb).total;
    const long cap = std::min<long>(env_long("L2B_MV_SMEM_KB", 208) * 1024, di.max_smem_optin - 1024);
    const long per_block_stages = (long)(p.units_lo + (p.units_rem ? 1 : 0)) * p.nit;
    long ns = std::min<long>(std::min<long>(MV_MAX_SLOTS, std::max<long>(per_block_stages, 2)), (cap - base) / slot);
    const long force = env_long("L2B_MV_SLOTS", 0);
    if (force > 0) ns = std::min<long>(std::min<long>(force, MV_MAX_SLOTS), (di.max_smem_optin - 1024 - base) / slot);
    // Two groups of consumer warps alternate over the tiles of a block (one group's waits hide behind the other's
    // arithmetic) when every group can have two slots of its own; a group has up to 8 warps, each taking one or
    // two super-block columns of a stage.
    int groups = (int)std::max<long>(1, std::min<long>(2, env_long("L2B_MV_GROUPS", 2)));
    if (ns < 4) groups = 1;
    const int WG = (int)std::min<long>(groups == 2 ? 8 : MV_MAX_CONSUMERS, std::max<long>(4, std::min<long>(kb, env_long("L2B_MV_WARPS", groups == 2 ? 8 : 16))));
    const int W = WG * groups;
    p.consumers = W;
    p.cgroups = groups;
    p.turns = (p.n_in / 8 + 32 * W - 1) / (32 * W);
    L.warps = W + 2;  // + producer warp + finisher warp
    ns -= ns % groups;  // every group owns the same number of slots
    if (ns < groups) return fail(L2B_ERR_BAD_ARG, "input dimension too large for the activation planes to fit in shared memory");
    p.nslots = (int)ns;
    L.smem = mv_smem_layout(p.n_in, L.planes, true, p.nslots, p.row_stride, L.nb).total;
    return L2B_OK;
}

static std::once_flag g_attr_once;
static cudaError_t g_attr_err = cudaSuccess;
static int32_t check_kernel_attrs();
static void set_kernel_attrs() {
    std::call_once(g_attr_once, [] {
        int dev = 0, optin = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        auto set = [&](const void* f) {  // the opt-in limit covers static + dynamic shared memory
            cudaFuncAttributes fa;
            cudaError_t e = cudaFuncGetAttributes(&fa, f);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, optin - (int)fa.sharedSizeBytes);
            if (e != cudaSuccess) g_attr_err = e;
        };
        set((const void*)fused_matvec_kernel<true, 1>);
        set((const void*)fused_matvec_kernel<true, 2>);
        set((const void*)fused_matvec_kernel<true, 3>);
        set((const void*)fused_matvec_kernel<false, 1>);
        set((const void*)fused_matvec_kernel<true, 3, false, false, 2>);
#ifdef L2B_MEASURE
        set((const void*)fused_matvec_kernel<true, 1, false, true>);
        set((const void*)fused_matvec_kernel<true, 2, false, true>);
        set((const void*)fused_matvec_kernel<true, 3, false, true>);
        set((const void*)fused_matvec_kernel<false, 1, false, true>);
#endif
        set((const void*)fused_matvec_kernel<true, 1, true>);
        set((const void*)fused_matvec_kernel<true, 2, true>);
        set((const void*)fused_matvec_kernel<true, 3, true>);
        set((const void*)kq_gemm_kernel);
        set((const void*)token_kernel<1>);
        set((const void*)token_kernel<2>);
        set((const void*)token_kernel<3>);
        set((const void*)export_activation_kernel<true, 1>);
        set((const void*)export_activation_kernel<true, 2>);
        set((const void*)export_activation_kernel<true, 3>);
        set((const void*)export_activation_kernel<false, 1>);
    });
}

static int32_t check_kernel_attrs() {
    set_kernel_attrs();
    if (g_attr_err != cudaSuccess) return fail(L2B_ERR_CUDA, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(g_attr_err));
    return L2B_OK;
}

static cudaError_t launch_matvec(const MvLaunch& L, cudaStream_t st, bool pdl) {
    const dim3 grid(L.grid), block(L.warps * 32);
#ifdef L2B_MEASURE
    if (L.p.debug || L.p.trace) {  // measurement aids (a -DL2B_MEASURE build only): the instantiations that carry them
        if (L.p.tp) return cudaErrorNotSupported;
        if (!L.kq) return launch_kernel(fused_matvec_kernel<false, 1, false, true>, grid, block, L.smem, st, pdl, L.p);
        switch (L.planes) {
            case 1: return launch_kernel(fused_matvec_kernel<true, 1, false, true>, grid, block, L.smem, st, pdl, L.p);
            case 2: return launch_kernel(fused_matvec_kernel<true, 2, false, true>, grid, block, L.smem, st, pdl, L.p);
            default: return launch_kernel(fused_matvec_kernel<true, 3, false, true>, grid, block, L.smem, st, pdl, L.p);
        }
    }
#endif
    if (L.nb == 2) {  // two prompt positions per pass: k-quant weights, three planes, one GPU only
        if (!L.kq || L.planes != 3 || L.p.tp) return cudaErrorNotSupported;
        return launch_kernel(fused_matvec_kernel<true, 3, false, false, 2>, grid, block, L.smem, st, pdl, L.p);
    }
    if (!L.kq) return launch_kernel(fused_matvec_kernel<false, 1>, grid, block, L.smem, st, pdl, L.p);
    if (L.p.tp)  // the variants that carry the tensor-parallel exchange
        switch (L.planes) {
            case 1: return launch_kernel(fused_matvec_kernel<true, 1, true>, grid, block, L.smem, st, pdl, L.p);
            case 2: return launch_kernel(fused_matvec_kernel<true, 2, true>, grid, block, L.smem, st, pdl, L.p);
            default: return launch_kernel(fused_matvec_kernel<true, 3, true>, grid, block, L.smem, st, pdl, L.p);
        }
    switch (L.planes) {
        case 1: return launch_kernel(fused_matvec_kernel<true, 1>, grid, block, L.smem, st, pdl, L.p);
        case 2: return launch_kernel(fused_matvec_kernel<true, 2>, grid, block, L.smem, st, pdl, L.p);
        default: return launch_kernel(fused_matvec_kernel<true, 3>, grid, block, L.smem, st, pdl, L.p);
    }
}

static MvSegment make_segment(const DevMatrix& m, int pair_mode, int epi, float* out, int head_size) {
    MvSegment s;
    memset(&s, 0, sizeof(s));
    s.w = m.data;
    s.d6 = m.d6;
    s.type = m.type;
    s.npairs = (int)(m.out / 2);
    s.pair_mode = pair_mode;
    s.epi = epi;
    s.out = out;
    s.head_size = head_size;
    return s;
}

static cudaError_t launch_attention(const AttnParams& a, int gq, cudaStream_t st, bool pdl) {
    const dim3 grid((a.n_heads / gq) * a.nsplit * (a.nq > 1 ? a.nq : 1)), block(ATTN_WARPS * 32);
    if (a.nq > 1) switch (gq) {
            case 8: return launch_kernel(attention_split_kernel<8, 2>, grid, block, 0, st, pdl, a);
            case 4: return launch_kernel(attention_split_kernel<4, 2>, grid, block, 0, st, pdl, a);
            case 2: return launch_kernel(attention_split_kernel<2, 2>, grid, block, 0, st, pdl, a);
            default: return launch_kernel(attention_split_kernel<1, 2>, grid, block, 0, st, pdl, a);
        }
    // one query position: clusters of ATTN_CL blocks (a.nsplit is a multiple of it, see decode_splits)
    const dim3 dblock(ATTN_DW * 32);
    switch (gq) {
        case 8: return launch_kernel(attention_decode_kernel<8>, grid, dblock, 0, st, pdl, a, ATTN_CL);
        case 4: return launch_kernel(attention_decode_kernel<4>, grid, dblock, 0, st, pdl, a, ATTN_CL);
        case 2: return launch_kernel(attention_decode_kernel<2>, grid, dblock, 0, st, pdl, a, ATTN_CL);
        default: return launch_kernel(attention_decode_kernel<1>, grid, dblock, 0, st, pdl, a, ATTN_CL);
    }
}
// Blocks per head group of the decode attention kernel for contexts of up to max_pos positions: one cluster per 512
// positions (two batches per warp; measured at the 8B shape, seq_len 512: one cluster 634 tok/s, two clusters with their
// exchange through scratch memory beyond 256 positions 630), at most four clusters (the final merge holds one partial result
// per cluster in registers).
static int decode_splits(int max_pos) {
    const int ncl = std::max(1, std::min(4, (max_pos + 2 * ATTN_CLUSTER_POS - 1) / (2 * ATTN_CLUSTER_POS)));
    return ncl * ATTN_CL;
}
static int choose_gq(int n_heads, int n_kv) {
    const int r = n_heads / n_kv;
    return (r == 8 || r == 4 || r == 2) ? r : 1;
}

// ---- tensor-core GEMM (kq_gemm.cuh): host side ----------------------------------------------------------
// cuTensorMapEncodeTiled comes from the driver; the library links the runtime only, so the entry point is looked up.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            f = nullptr;
        }
        return (EncodeTiledFn)f;
    }();
    return fn;
}

static bool gemm_supported(const DevMatrix& w) { return (w.type == T_Q4_K || w.type == T_Q5_K) && w.out >= 1; }

// The matrix as a 3-D byte tensor [panels][rows][panel row bytes]; box = one super-block of 128 rows.
static int32_t gemm_tensor_maps(const DevMatrix& w, CUtensorMap& main_map, CUtensorMap& tail_map, int& kb_eff) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(L2B_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const int bb = dev_block_bytes(w.type);
    const int64_t nb = w.in / QK_K;
    kb_eff = w.panels ? w.kb : (int)nb;
    const int64_t full_panels = nb / kb_eff, tail_blocks = nb % kb_eff;
    auto make = [&](CUtensorMap& m, uint8_t* base, int64_t blocks, int64_t panels) -> int32_t {
        const cuuint64_t dims[3] = {(cuuint64_t)(blocks * bb), (cuuint64_t)w.out, (cuuint64_t)panels};
        const cuuint64_t strides[2] = {(cuuint64_t)(blocks * bb), (cuuint64_t)(blocks * bb) * (cuuint64_t)w.out};
        const cuuint32_t box[3] = {(cuuint32_t)bb, (cuuint32_t)GM_ROWS, 1u};
        const cuuint32_t estr[3] = {1u, 1u, 1u};
        const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(L2B_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
        return L2B_OK;
    };
    if (full_panels > 0) L2B_TRY(make(main_map, w.data, kb_eff, full_panels));
    if (tail_blocks > 0) L2B_TRY(make(tail_map, w.data + (size_t)full_panels * w.out * kb_eff * bb, tail_blocks, 1));
    else tail_map = main_map;
    if (full_panels == 0) main_map = tail_map;
    return L2B_OK;
}

static size_t gemm_act_bytes(int64_t n_in, int n_tok) { return (size_t)((n_tok + GM_TOK - 1) / GM_TOK) * (size_t)(n_in / QK_K) * GM_ACT_BYTES; }

// x [n_tok][ldx] f32 (optionally rmsnorm'ed with `gain`) -> int8 planes in the GEMM's operand layout
static int32_t launch_quantise_rows(const float* x, const float* gain, uint8_t* act, int n, int ldx, int n_tok, cudaStream_t st) {
    CU(cudaMemsetAsync(act, 0, gemm_act_bytes(n, n_tok), st));  // unused columns and tokens must read as zero
    QuantRowsParams q;
    q.x = x; q.gain = gain; q.act = act; q.n = n; q.ldx = ldx; q.n_tok = n_tok;
    quantise_rows_kernel<<<n_tok, 512, 0, st>>>(q);
    CU(cudaGetLastError());
    return L2B_OK;
}

// y[t][ldy] (+= resid) = W x_t for n_tok activation vectors already quantised by launch_quantise_rows
static int32_t launch_kq_gemm(const DevMatrix& w, const uint8_t* act, int n_tok, float* y, int ldy, const float* resid, int* status, cudaStream_t st) {
    if (!gemm_supported(w)) return fail(L2B_ERR_UNSUPPORTED_TYPE, "the tensor-core GEMM takes q4_K and q5_K matrices");
    CUtensorMap mm, mt;
    int kb_eff = 0;
    L2B_TRY(gemm_tensor_maps(w, mm, mt, kb_eff));
    GemmParams g;
    memset(&g, 0, sizeof(g));
    g.type = w.type; g.rows = (int)w.out; g.nb = (int)(w.in / QK_K); g.kb = kb_eff; g.n_tok = n_tok;
    g.act = act; g.y = y; g.resid = resid; g.ldy = ldy; g.mode = resid ? GM_RESIDUAL : GM_STORE; g.status = status;
    const dim3 grid((unsigned)((w.out + GM_ROWS - 1) / GM_ROWS), (unsigned)((n_tok + GM_TOK - 1) / GM_TOK));
    const size_t smem = (size_t)gm_smem_layout(dev_block_bytes(w.type)).total + 1024;  // + room to align the base to 1024 bytes
    kq_gemm_kernel<<<grid, GM_THREADS, smem, st>>>(g, mm, mt);
    CU(cudaGetLastError());
    return L2B_OK;
}

// Buffers of a many-token pass: activations of up to PF_MAX_TOK tokens, attention scratch, quantised activations.
struct GemmBufs {
    float *x = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *g = nullptr, *u = nullptr;
    float *pm = nullptr, *pl = nullptr, *pacc = nullptr;
    int* tickets = nullptr;
    uint8_t* act = nullptr;
    int nsplit = 1;
};

static void free_gemm_bufs(GemmBufs& B) {
    void* pf[] = {B.x, B.q, B.k, B.v, B.att, B.g, B.u, B.pm, B.pl, B.pacc, B.tickets, B.act};
    for (void* b : pf)
        if (b) cudaFree(b);
    B = GemmBufs();
}

// cos/sin of the iterated f32 angle, exactly as rope_normal!/rope_neox! advance it
// (src/inference.jl:119-127, 140-153): theta_scale = base^(-1/(hs/2)) in f32 (Julia evaluates the
// f32 power in f64 and rounds once), theta_0 = Float32(pos), theta *= theta_scale; cis(theta) is
// evaluated in f64 and rounded.
static void rope_table_host(std::vector<float>& cs, int seq_len, int hs, float base) {
    const int h2 = hs / 2;
    cs.resize((size_t)seq_len * h2 * 2);
    const float e = -(1.0f / (float)h2);
    const float scale = (float)std::pow((double)base, (double)e);
    for (int pos = 0; pos < seq_len; ++pos) {
        float theta = 1.0f * (float)pos;
        for (int i = 0; i < h2; ++i) {
            cs[((size_t)pos * h2 + i) * 2] = (float)std::cos((double)theta);
            cs[((size_t)pos * h2 + i) * 2 + 1] = (float)std::sin((double)theta);
            theta *= scale;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// model
// ---------------------------------------------------------------------------------------------
struct LayerW {
    float* rms_att = nullptr;
    float* rms_ffn = nullptr;
    DevMatrix wq, wk, wv, wo, w1, w2, w3;
};

struct l2b_model {
    l2b_config cfg;
    int device = 0;
    DevMatrix tok_emb, output;
    float* rms_final = nullptr;
    std::vector<LayerW> layers;
    bool finalized = false;
    int planes = 3;
    // tensor parallelism: this process holds rank `rank` of `tp` shards.  Heads are split by kv group, the ffn by
    // hidden units; wo and w2 are split along their INPUT (block columns), so their outputs are partial sums.
    int tp = 1, rank = 0;
    int l_heads = 0, l_kv = 0, l_hidden = 0;  // this rank's query heads, kv heads and hidden units
    int l_qdim() const { return l_heads * (cfg.dim / cfg.n_heads); }
    int l_kvdim() const { return l_kv * (cfg.dim / cfg.n_heads); }
};

struct l2b_session {
    l2b_model* model = nullptr;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    DeviceInfo di;
    // activations
    float *x = nullptr, *q = nullptr, *att = nullptr, *hb = nullptr, *logits = nullptr;
    float *kc = nullptr, *vc = nullptr;  // [layer][kv_head][seq_len][hs]
    float *part_m = nullptr, *part_l = nullptr, *part_acc = nullptr;
    int* tickets = nullptr;
    float* amax_val = nullptr;
    int* amax_idx = nullptr;
    float* rope_cs = nullptr;
    Control* ctl = nullptr;
    int* status = nullptr;
    int* prompt = nullptr;
    int* out_tokens = nullptr;
    int* next_token = nullptr;
    int nsplit = 1, gq = 1;
    // host pinned mirrors
    Control* h_ctl = nullptr;
    int* h_small = nullptr;  // [0] next token, [1] status
    cudaGraphExec_t graph = nullptr;
    cudaGraphExec_t graph2 = nullptr;  // two prompt positions per pass (null when the model does not qualify)
    bool all_kquant = true;            // set while the one-position graph is built
    int kernels_per_token = 0;
    int kernels_per_pair = 0;      // launches of the two-position prompt graph
    long long last_launches = 0;   // kernel launches of the most recent forward / decode / prefill / generate call
    cudaEvent_t ev0 = nullptr, ev1 = nullptr, ev_mid = nullptr;
    float last_ms = 0.f;
    float last_prompt_ms = 0.f, last_decode_ms = 0.f;  // l2b_generate: positions inside the prompt / after it
    unsigned long long* trace = nullptr;  // L2B_TRACE_TOKEN=1: per-launch, per-block timeline stamps (debugging aid)
    unsigned long long* attn_trace = nullptr;  // the same for the decode attention kernel: [layer][1024 blocks][8]
    int trace_launches = 0;
    // tensor parallelism.  tp_mem = [n_exch][tp][dim] partial vectors of {f32, tag} pairs;
    // n_exch = 2 * n_layers (one exchange after wo, one after w2).  Peers write into it through IPC mappings.
    float* x2 = nullptr;          // second buffer of the residual stream (the summing prologue reads one, writes the other)
    uint8_t* tp_mem = nullptr;
    size_t tp_bytes = 0;
    unsigned* tp_epoch = nullptr;  // tokens completed (device word)
    uint8_t* peer_mem[MV_MAX_TP] = {nullptr};  // [r]: rank r's tp_mem as seen from this process ([rank] = own)
    // many-token prompt pass through the tensor-core GEMM (kq_gemm.cuh): buffers for PF_MAX_TOK tokens, allocated on first use
    bool pf_checked = false, pf_ok = false;
    GemmBufs pf;
    // one persistent kernel per token (token_kernel.cuh): k-quant models on one GPU
    bool tk = false;
    TkOp* tk_ops = nullptr;
    unsigned* tk_sync = nullptr;          // one arrival counter per operation
    unsigned long long* tk_trace = nullptr;  // measurement builds only
    std::vector<int> tk_kinds;               // measurement builds only: kind and input length of every operation
    TkParams tkp;
    bool tp_connected = false;
    MvTp* tp_descs = nullptr;          // device array: one descriptor per tensor-parallel launch of the token
    std::vector<MvTp> tp_descs_host;   // filled while the token graph is captured, uploaded right after
};

static size_t kv_layer_elems(const l2b_model* m) { return (size_t)m->l_kv * m->cfg.seq_len * (m->cfg.dim / m->cfg.n_heads); }

extern "C" int32_t l2b_version(void) { return 100; }
extern "C" const char* l2b_last_error_string(void) { return g_last_error.c_str(); }
extern "C" const char* l2b_status_string(int32_t s) {
    switch (s) {
        case L2B_OK: return "ok";
        case L2B_ERR_BAD_ARG: return "bad argument";
        case L2B_ERR_UNSUPPORTED_TYPE: return "unsupported tensor type";
        case L2B_ERR_CUDA: return "CUDA error";
        case L2B_ERR_TIMEOUT: return "device-side wait timed out";
        case L2B_ERR_OOM: return "out of device memory";
        case L2B_ERR_STATE: return "call made in the wrong state";
        case L2B_ERR_NO_DEVICE: return "no CUDA device";
        default: return "unknown status";
    }
}
extern "C" int32_t l2b_device_count(int32_t* count) {
    if (!count) return fail(L2B_ERR_BAD_ARG, "count is null");
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        n = 0;
    }
    *count = n;
    return L2B_OK;
}

extern "C" int32_t l2b_model_create(const l2b_config* c, l2b_model** out) {
    if (!c || !out) return fail(L2B_ERR_BAD_ARG, "null argument");
    *out = nullptr;
    if (c->dim <= 0 || c->hidden_dim <= 0 || c->n_layers <= 0 || c->n_heads <= 0 || c->n_kv_heads <= 0 || c->vocab_size <= 0 || c->seq_len <= 0)
        return fail(L2B_ERR_BAD_ARG, "ModelConfig fields must be positive");
    if (c->dim % c->n_heads != 0 || c->n_heads % c->n_kv_heads != 0) return fail(L2B_ERR_BAD_ARG, "dim % n_heads and n_heads % n_kv_heads must be 0");
    const int hs = c->dim / c->n_heads;
    if (hs % 8 != 0 || hs > 128) return fail(L2B_ERR_BAD_ARG, "head size must be a multiple of 8 and at most 128");
    if (c->dim % 8 != 0 || c->hidden_dim % 8 != 0 || c->vocab_size % 2 != 0) return fail(L2B_ERR_BAD_ARG, "dim, hidden_dim must be multiples of 8 and vocab_size even");
    if (c->act_planes < 0 || c->act_planes > 3) return fail(L2B_ERR_BAD_ARG, "act_planes must be 0..3");
    const int tp = c->tp_size <= 1 ? 1 : c->tp_size;
    if (tp > 1) {
        if (tp > MV_MAX_TP) return fail(L2B_ERR_BAD_ARG, "tp_size is at most 8");
        if (c->tp_rank < 0 || c->tp_rank >= tp) return fail(L2B_ERR_BAD_ARG, "tp_rank must lie in [0, tp_size)");
        if (c->n_kv_heads % tp != 0) return fail(L2B_ERR_BAD_ARG, "n_kv_heads must be a multiple of tp_size (heads are split by kv group)");
        if ((c->dim / tp) % QK_K != 0 || (c->hidden_dim / tp) % QK_K != 0 || c->hidden_dim % tp != 0)
            return fail(L2B_ERR_BAD_ARG, "dim / tp_size and hidden_dim / tp_size must be multiples of 256 (wo and w2 are split by super-block columns)");
    }
    L2B_TRY(require_device());
    l2b_model* m = new l2b_model();
    m->cfg = *c;
    m->tp = tp;
    m->rank = tp > 1 ? c->tp_rank : 0;
    m->l_heads = c->n_heads / tp;
    m->l_kv = c->n_kv_heads / tp;
    m->l_hidden = c->hidden_dim / tp;
    m->planes = c->act_planes == 0 ? 3 : c->act_planes;
    if (c->device >= 0) {
        cudaError_t e = cudaSetDevice(c->device);
        if (e != cudaSuccess) {
            delete m;
            return fail(L2B_ERR_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
        }
    }
    cudaGetDevice(&m->device);
    m->layers.resize(c->n_layers);
    *out = m;
    return L2B_OK;
}

static int32_t upload_vector(float*& dst, const void* host, int64_t n) {
    if (dst) cudaFree(dst), dst = nullptr;
    CU(cudaMalloc(&dst, (size_t)n * 4));
    CU(cudaMemcpy(dst, host, (size_t)n * 4, cudaMemcpyHostToDevice));
    return L2B_OK;
}

extern "C" int32_t l2b_model_upload_tensor(l2b_model* m, int32_t role, int32_t layer, int32_t type, const void* host, int64_t in_dim, int64_t out_dim) {
    if (!m || !host) return fail(L2B_ERR_BAD_ARG, "null argument");
    if (m->finalized) return fail(L2B_ERR_STATE, "model already finalized");
    CU(cudaSetDevice(m->device));
    const l2b_config& c = m->cfg;
    const int hs = c.dim / c.n_heads, kv_dim = hs * c.n_kv_heads;
    const bool per_layer = !(role == L2B_ROLE_TOKEN_EMBEDDING || role == L2B_ROLE_RMS_FINAL || role == L2B_ROLE_OUTPUT);
    if (per_layer && (layer < 0 || layer >= c.n_layers)) return fail(L2B_ERR_BAD_ARG, "layer index out of range");
    auto want = [&](int64_t in, int64_t out) -> int32_t {
        if (in_dim != in || out_dim != out)
            return fail(L2B_ERR_BAD_ARG, "tensor shape (" + std::to_string(in_dim) + "," + std::to_string(out_dim) + ") does not match the config (" +
                                             std::to_string(in) + "," + std::to_string(out) + ")");
        return L2B_OK;
    };
    auto norm = [&](float*& dst) -> int32_t {
        if (type != L2B_TYPE_F32) return fail(L2B_ERR_UNSUPPORTED_TYPE, "norm gains must be f32");
        if (in_dim * out_dim != c.dim) return fail(L2B_ERR_BAD_ARG, "norm gain length must equal dim");
        return upload_vector(dst, host, c.dim);
    };
    LayerW* lw = per_layer ? &m->layers[layer] : nullptr;
    if (m->tp > 1) {
        // The caller passes the FULL tensor on every rank; this rank keeps its shard.
        //   rows (outputs) of wq / wk / wv / w1 / w3: a contiguous range, i.e. an offset pointer;
        //   block columns (inputs) of wo / w2: the range [rank*nb/tp, (rank+1)*nb/tp) of every row, gathered on the host.
        const int64_t r = m->rank, g = m->tp;
        auto rows = [&](DevMatrix& dst, int64_t in, int64_t out) -> int32_t {
            L2B_TRY(want(in, out));
            if (!type_supported(type)) return fail(L2B_ERR_UNSUPPORTED_TYPE, "tensor type " + std::to_string(type) + " not implemented");
            const int64_t row_bytes = type == T_F32 ? in * 4 : (in / QK_K) * file_block_bytes(type);
            const int64_t lo = out / g;
            return upload_matrix(dst, type, (const uint8_t*)host + r * lo * row_bytes, in, lo, 0);
        };
        auto cols = [&](DevMatrix& dst, int64_t in, int64_t out) -> int32_t {
            L2B_TRY(want(in, out));
            if (type != T_Q4_K && type != T_Q5_K && type != T_Q6_K)
                return fail(L2B_ERR_UNSUPPORTED_TYPE, "tensor parallelism needs k-quant wo and w2 matrices");
            const int64_t bb = file_block_bytes(type), nb = in / QK_K, nbl = nb / g;
            std::vector<uint8_t> tmp((size_t)(out * nbl * bb));
            for (int64_t o = 0; o < out; ++o)
                memcpy(tmp.data() + (size_t)(o * nbl * bb), (const uint8_t*)host + (size_t)((o * nb + r * nbl) * bb), (size_t)(nbl * bb));
            return upload_matrix(dst, type, tmp.data(), in / g, out, 0);
        };
        switch (role) {
            case L2B_ROLE_WQ: return rows(lw->wq, c.dim, c.dim);
            case L2B_ROLE_WK: return rows(lw->wk, c.dim, kv_dim);
            case L2B_ROLE_WV: return rows(lw->wv, c.dim, kv_dim);
            case L2B_ROLE_W1: return rows(lw->w1, c.dim, c.hidden_dim);
            case L2B_ROLE_W3: return rows(lw->w3, c.dim, c.hidden_dim);
            case L2B_ROLE_WO: return cols(lw->wo, c.dim, c.dim);
            case L2B_ROLE_W2: return cols(lw->w2, c.hidden_dim, c.dim);
            default: break;  // embedding, norms and the classifier are replicated
        }
    }
    switch (role) {
        case L2B_ROLE_TOKEN_EMBEDDING: L2B_TRY(want(c.dim, c.vocab_size)); return upload_matrix(m->tok_emb, type, host, in_dim, out_dim, 0, false);
        case L2B_ROLE_OUTPUT: L2B_TRY(want(c.dim, c.vocab_size)); return upload_matrix(m->output, type, host, in_dim, out_dim, 0);
        case L2B_ROLE_RMS_FINAL: return norm(m->rms_final);
        case L2B_ROLE_RMS_ATT: return norm(lw->rms_att);
        case L2B_ROLE_RMS_FFN: return norm(lw->rms_ffn);
        case L2B_ROLE_WQ: L2B_TRY(want(c.dim, c.dim)); return upload_matrix(lw->wq, type, host, in_dim, out_dim, 0);
        case L2B_ROLE_WK: L2B_TRY(want(c.dim, kv_dim)); return upload_matrix(lw->wk, type, host, in_dim, out_dim, 0);
        case L2B_ROLE_WV: L2B_TRY(want(c.dim, kv_dim)); return upload_matrix(lw->wv, type, host, in_dim, out_dim, 0);
        case L2B_ROLE_WO: L2B_TRY(want(c.dim, c.dim)); return upload_matrix(lw->wo, type, host, in_dim, out_dim, 0);
        case L2B_ROLE_W1: L2B_TRY(want(c.dim, c.hidden_dim)); return upload_matrix(lw->w1, type, host, in_dim, out_dim, 0);
        case L2B_ROLE_W3: L2B_TRY(want(c.dim, c.hidden_dim)); return upload_matrix(lw->w3, type, host, in_dim, out_dim, 0);
        case L2B_ROLE_W2: L2B_TRY(want(c.hidden_dim, c.dim)); return upload_matrix(lw->w2, type, host, in_dim, out_dim, 0);
        default: return fail(L2B_ERR_BAD_ARG, "unknown tensor role " + std::to_string(role));
    }
}

extern "C" int32_t l2b_model_finalize(l2b_model* m) {
    if (!m) return fail(L2B_ERR_BAD_ARG, "null model");
    if (!m->tok_emb.present() || !m->output.present() || !m->rms_final) return fail(L2B_ERR_STATE, "token embedding, output weight or final norm missing");
    for (int l = 0; l < m->cfg.n_layers; ++l) {
        const LayerW& w = m->layers[l];
        if (!w.rms_att || !w.rms_ffn || !w.wq.present() || !w.wk.present() || !w.wv.present() || !w.wo.present() || !w.w1.present() ||
            !w.w2.present() || !w.w3.present())
            return fail(L2B_ERR_STATE, "missing blk." + std::to_string(l) + " weights");
        if (w.w1.type != w.w3.type) return fail(L2B_ERR_UNSUPPORTED_TYPE, "ffn gate and up matrices must have the same tensor type");
        if (m->tp > 1 && (w.wq.type == T_F32 || w.wk.type == T_F32 || w.wv.type == T_F32 || w.w1.type == T_F32))
            return fail(L2B_ERR_UNSUPPORTED_TYPE, "tensor parallelism needs k-quant layer matrices");
    }
    if (m->tp > 1 && m->output.type == T_F32) return fail(L2B_ERR_UNSUPPORTED_TYPE, "tensor parallelism needs a k-quant output matrix");
    m->finalized = true;
    return L2B_OK;
}

extern "C" int32_t l2b_model_destroy(l2b_model* m) {
    if (!m) return L2B_OK;
    cudaSetDevice(m->device);
    free_matrix(m->tok_emb);
    free_matrix(m->output);
    if (m->rms_final) cudaFree(m->rms_final);
    for (auto& w : m->layers) {
        if (w.rms_att) cudaFree(w.rms_att);
        if (w.rms_ffn) cudaFree(w.rms_ffn);
        free_matrix(w.wq); free_matrix(w.wk); free_matrix(w.wv); free_matrix(w.wo);
        free_matrix(w.w1); free_matrix(w.w2); free_matrix(w.w3);
    }
    delete m;
    return L2B_OK;
}

extern "C" int32_t l2b_model_weight_bytes(const l2b_model* m, int64_t* bytes) {
    if (!m || !bytes) return fail(L2B_ERR_BAD_ARG, "null argument");
    int64_t b = m->output.file_bytes + (int64_t)m->cfg.dim * 4;  // output matrix + final norm gain
    b += m->tok_emb.file_bytes / m->cfg.vocab_size;               // one embedding row
    for (const auto& w : m->layers)
        b += w.wq.file_bytes + w.wk.file_bytes + w.wv.file_bytes + w.wo.file_bytes + w.w1.file_bytes + w.w2.file_bytes + w.w3.file_bytes +
             2 * (int64_t)m->cfg.dim * 4;
    *bytes = b;
    return L2B_OK;
}

// ---------------------------------------------------------------------------------------------
// GGUF files: load_gguf_model's weight path (src/load_gguf.jl:211-336) inside the library
// ---------------------------------------------------------------------------------------------
namespace {

struct GgufModelInfo {
    l2b_config cfg;
    int arch = 0;  // 0 llama, 1 phi3
    int64_t context_length = 0;
};

int32_t gguf_describe(const GgufFile& f, GgufModelInfo& info) {
    memset(&info.cfg, 0, sizeof(info.cfg));
    const GgufValue* a = f.find("general.architecture");
    if (!a || a->type != 8) return fail(L2B_ERR_BAD_ARG, "general.architecture is missing");
    const std::string arch = a->str;
    if (arch == "llama") info.arch = 0;
    else if (arch == "phi3") info.arch = 1;
    else return fail(L2B_ERR_BAD_ARG, "unsupported model architecture: " + arch);  // src/load_gguf.jl:385-386
    auto num = [&](const char* key, double dflt, bool required, double& out) -> int32_t {
        const GgufValue* v = f.find(arch + "." + key);
        if (!v || v->type == 8 || v->type == 9) {
            if (required) return fail(L2B_ERR_BAD_ARG, "metadata key " + arch + "." + key + " is missing");
            out = dflt;
            return L2B_OK;
        }
        out = v->num;
        return L2B_OK;
    };
    double dim, hidden, layers, heads, kv_heads, base, ctx;
    L2B_TRY(num("embedding_length", 0, true, dim));
    L2B_TRY(num("feed_forward_length", 0, true, hidden));
    L2B_TRY(num("block_count", 0, true, layers));
    L2B_TRY(num("attention.head_count", 0, true, heads));
    L2B_TRY(num("attention.head_count_kv", heads, false, kv_heads));
    L2B_TRY(num("rope.freq_base", 10000.0, false, base));  // src/load_gguf.jl:238, 300
    L2B_TRY(num("context_length", 0, false, ctx));
    l2b_config& c = info.cfg;
    c.dim = (int32_t)dim; c.hidden_dim = (int32_t)hidden; c.n_layers = (int32_t)layers;
    c.n_heads = (int32_t)heads; c.n_kv_heads = (int32_t)kv_heads;
    c.rope_freq_base = (float)base;
    c.rope_is_neox = info.arch == 1;  // src/load_gguf.jl:239, 301
    info.context_length = (int64_t)ctx;
    // vocabulary = number of tokenizer tokens (src/load_gguf.jl:382), else the rows of the embedding table
    const GgufValue* toks = f.find("tokenizer.ggml.tokens");
    if (toks && toks->type == 9) c.vocab_size = (int32_t)toks->count;
    else if (const GgufTensor* e = f.tensor("token_embd.weight")) c.vocab_size = (int32_t)e->rows();
    else return fail(L2B_ERR_BAD_ARG, "neither tokenizer.ggml.tokens nor token_embd.weight is present");
    return L2B_OK;
}

}  // namespace

extern "C" int32_t l2b_gguf_inspect(const char* path, l2b_config* config_out, int32_t* arch_out, int64_t* n_tensors, int64_t* context_length) {
    if (!path || !config_out) return fail(L2B_ERR_BAD_ARG, "null argument");
    GgufFile f;
    if (!f.open(path)) return fail(L2B_ERR_BAD_ARG, f.error());
    GgufModelInfo info;
    L2B_TRY(gguf_describe(f, info));
    info.cfg.seq_len = (int32_t)std::min<int64_t>(info.context_length, 0x7fffffff);
    *config_out = info.cfg;
    if (arch_out) *arch_out = info.arch;
    if (n_tensors) *n_tensors = (int64_t)f.tensors().size();
    if (context_length) *context_length = info.context_length;
    return L2B_OK;
}

extern "C" int32_t l2b_model_load_gguf(const char* path, int32_t seq_len, int32_t act_planes, int32_t device, int32_t tp_size, int32_t tp_rank,
                                       l2b_config* config_out, l2b_model** out) {
    if (!path || !out) return fail(L2B_ERR_BAD_ARG, "null argument");
    *out = nullptr;
    GgufFile f;
    if (!f.open(path)) return fail(L2B_ERR_BAD_ARG, f.error());
    GgufModelInfo info;
    L2B_TRY(gguf_describe(f, info));
    l2b_config c = info.cfg;
    // seq_len > 0: as given; 0: the file's context_length; < 0: the 512 the reference hard-codes (src/load_gguf.jl:237, 299)
    c.seq_len = seq_len > 0 ? seq_len : (seq_len == 0 ? (int32_t)info.context_length : 512);
    c.act_planes = act_planes;
    c.device = device;
    c.tp_size = tp_size;
    c.tp_rank = tp_rank;
    l2b_model* m = nullptr;
    L2B_TRY(l2b_model_create(&c, &m));
    const int64_t hs = c.dim / c.n_heads, kv_dim = hs * c.n_kv_heads;
    auto fail_free = [&](int32_t st) {
        l2b_model_destroy(m);
        return st;
    };
    // one tensor (or a row range of it) -> one role.  Rows are contiguous, so a range is an offset pointer.
    auto up = [&](const std::string& name, int32_t role, int32_t layer, int64_t in, int64_t row0, int64_t rows, bool vector) -> int32_t {
        const GgufTensor* t = f.tensor(name);
        if (!t) return fail(L2B_ERR_STATE, "tensor " + name + " is missing");
        if (!t->data) return fail(L2B_ERR_UNSUPPORTED_TYPE, "tensor type " + std::to_string(t->type) + " not implemented (" + name + ")");  // :153
        const int64_t t_in = (int64_t)t->dims[0], t_rows = (int64_t)t->rows();
        if (vector) {
            if (t->type != T_F32 || t_in * t_rows != in) return fail(L2B_ERR_BAD_ARG, "norm tensor " + name + " must be f32 of length dim");
            return l2b_model_upload_tensor(m, role, layer, T_F32, t->data, in, 1);
        }
        if (t_in != in || row0 + rows > t_rows) return fail(L2B_ERR_BAD_ARG, "tensor " + name + " has an unexpected shape");
        const int64_t row_bytes = t->type == T_F32 ? in * 4 : in / QK_K * file_block_bytes((int)t->type);
        return l2b_model_upload_tensor(m, role, layer, (int32_t)t->type, t->data + row0 * row_bytes, in, rows);
    };
    int32_t st = up("token_embd.weight", L2B_ROLE_TOKEN_EMBEDDING, 0, c.dim, 0, c.vocab_size, false);
    // models that tie the classifier to the embedding ship no output.weight
    if (st == L2B_OK) st = up(f.tensor("output.weight") ? "output.weight" : "token_embd.weight", L2B_ROLE_OUTPUT, 0, c.dim, 0, c.vocab_size, false);
    if (st == L2B_OK) st = up("output_norm.weight", L2B_ROLE_RMS_FINAL, 0, c.dim, 0, 1, true);
    for (int l = 0; l < c.n_layers && st == L2B_OK; ++l) {
        const std::string b = "blk." + std::to_string(l) + ".";
        st = up(b + "attn_norm.weight", L2B_ROLE_RMS_ATT, l, c.dim, 0, 1, true);
        if (st == L2B_OK) st = up(b + "ffn_norm.weight", L2B_ROLE_RMS_FFN, l, c.dim, 0, 1, true);
        if (st != L2B_OK) break;
        if (info.arch == 0) {  // src/load_gguf.jl:211-253
            st = up(b + "attn_q.weight", L2B_ROLE_WQ, l, c.dim, 0, c.dim, false);
            if (st == L2B_OK) st = up(b + "attn_k.weight", L2B_ROLE_WK, l, c.dim, 0, kv_dim, false);
            if (st == L2B_OK) st = up(b + "attn_v.weight", L2B_ROLE_WV, l, c.dim, 0, kv_dim, false);
            if (st == L2B_OK) st = up(b + "ffn_gate.weight", L2B_ROLE_W1, l, c.dim, 0, c.hidden_dim, false);
            if (st == L2B_OK) st = up(b + "ffn_up.weight", L2B_ROLE_W3, l, c.dim, 0, c.hidden_dim, false);
        } else {  // phi3 (src/load_gguf.jl:255-315): q, k, v are row ranges of attn_qkv; gate and up are the halves of ffn_up
            st = up(b + "attn_qkv.weight", L2B_ROLE_WQ, l, c.dim, 0, c.dim, false);
            if (st == L2B_OK) st = up(b + "attn_qkv.weight", L2B_ROLE_WK, l, c.dim, c.dim, kv_dim, false);
            if (st == L2B_OK) st = up(b + "attn_qkv.weight", L2B_ROLE_WV, l, c.dim, c.dim + kv_dim, kv_dim, false);
            if (st == L2B_OK) st = up(b + "ffn_up.weight", L2B_ROLE_W1, l, c.dim, 0, c.hidden_dim, false);
            if (st == L2B_OK) st = up(b + "ffn_up.weight", L2B_ROLE_W3, l, c.dim, c.hidden_dim, c.hidden_dim, false);
        }
        if (st == L2B_OK) st = up(b + "attn_output.weight", L2B_ROLE_WO, l, c.dim, 0, c.dim, false);
        if (st == L2B_OK) st = up(b + "ffn_down.weight", L2B_ROLE_W2, l, c.hidden_dim, 0, c.dim, false);
    }
    if (st == L2B_OK) st = l2b_model_finalize(m);
    if (st != L2B_OK) return fail_free(st);
    if (config_out) *config_out = c;
    *out = m;
    return L2B_OK;
}

// ---------------------------------------------------------------------------------------------
// session
// ---------------------------------------------------------------------------------------------
static void session_free(l2b_session* s) {
    if (!s) return;
    if (s->graph) cudaGraphExecDestroy(s->graph);
    if (s->graph2) cudaGraphExecDestroy(s->graph2);
    void* bufs[] = {s->x, s->q, s->att, s->tickets, s->hb, s->logits, s->kc, s->vc, s->part_m, s->part_l, s->part_acc, s->amax_val, s->amax_idx,
                    s->rope_cs, s->ctl, s->prompt, s->out_tokens, s->next_token};  // (status lives behind next_token)
    for (void* b : bufs)
        if (b) cudaFree(b);
    if (s->trace) cudaFree(s->trace);
    if (s->attn_trace) cudaFree(s->attn_trace);
    if (s->model)
        for (int r = 0; r < s->model->tp; ++r)
            if (s->peer_mem[r] && r != s->model->rank) cudaIpcCloseMemHandle(s->peer_mem[r]);
    if (s->x2) cudaFree(s->x2);
    if (s->tp_mem) cudaFree(s->tp_mem);
    if (s->tp_epoch) cudaFree(s->tp_epoch);
    if (s->tp_descs) cudaFree(s->tp_descs);
    free_gemm_bufs(s->pf);
    if (s->tk_ops) cudaFree(s->tk_ops);
    if (s->tk_sync) cudaFree(s->tk_sync);
    if (s->tk_trace) cudaFree(s->tk_trace);
    if (s->h_ctl) cudaFreeHost(s->h_ctl);
    if (s->h_small) cudaFreeHost(s->h_small);
    if (s->ev0) cudaEventDestroy(s->ev0);
    if (s->ev1) cudaEventDestroy(s->ev1);
    if (s->ev_mid) cudaEventDestroy(s->ev_mid);
    if (s->own_stream && s->stream) cudaStreamDestroy(s->stream);
    delete s;
}

struct l2b_session;
static cudaError_t cudaLaunchKernelEx_embed(const l2b_model* m, l2b_session* s, int blocks, int threads, int second);

// Enqueue every kernel of one token on the session stream (this is what the graph captures).
// nb = 2: a pass over TWO consecutive prompt positions (pos, pos + 1), both of which are followed by a prompt token:
// every matrix is streamed once for both, no logits are computed and nothing is sampled.
static int32_t enqueue_token(l2b_session* s, int* nlaunch, int nb = 1) {
    const l2b_model* m = s->model;
    const l2b_config& c = m->cfg;
    const int hs = c.dim / c.n_heads;
    const size_t kvl = kv_layer_elems(m);
    int count = 0, last_grid = 0;
    bool first = true;
    auto mv = [&](MvLaunch& L) -> int32_t {
        L.planes = m->planes;
        L.nb = nb;
        L2B_TRY(plan_matvec(L, s->di));
        if (!L.kq) s->all_kquant = false;
#ifdef L2B_MEASURE
        if (s->trace) L.p.trace = s->trace + (size_t)(s->trace_launches++) * s->di.sms * 16;
#endif
        CU(launch_matvec(L, s->stream, !first));
        last_grid = L.grid;
        first = false;
        ++count;
        return L2B_OK;
    };
    auto base_params = [&](MvLaunch& L, int n_in) {
        memset(&L.p, 0, sizeof(L.p));
        L.p.n_in = n_in;
        L.p.pos = &s->ctl->pos;
        L.p.rope_cs = s->rope_cs;
        L.p.seq_len = c.seq_len;
        L.p.status = s->status;
    };
    // Tensor parallelism: the residual stream alternates between two buffers; `pending` is the exchange whose
    // partial vectors the next rmsnorm prologue has to add (-1: none).
    const int tp = m->tp;
    float* xbuf[2] = {s->x, tp > 1 ? s->x2 : s->x};
    int cur = 0, pending = -1;
    // (every value of a partial vector travels as 8 bytes {f32 bits, token tag}: 2 * dim floats per vector)
    auto xchg_vec = [&](uint8_t* base, int e, int r) { return reinterpret_cast<float*>(base) + ((size_t)e * tp + r) * c.dim * 2; };
    // rmsnorm prologue over the residual stream; with an exchange pending it first forms x + sum of the partial vectors
    // descriptors live in device memory; their contents are uploaded after the capture (capture_token_graph)
    auto new_desc = [&](MvLaunch& L) -> MvTp& {
        MvTp d;
        memset(&d, 0, sizeof(d));
        d.tp_size = tp;
        s->tp_descs_host.push_back(d);
        L.p.tp = s->tp_descs + (s->tp_descs_host.size() - 1);
        return s->tp_descs_host.back();
    };
    auto norm_input = [&](MvLaunch& L, const float* gain) {
        L.p.pro = PRO_RMSNORM;
        L.p.gain = gain;
        L.p.x_in = xbuf[cur];
        if (pending >= 0) {
            MvTp& d = new_desc(L);
            d.part_src = xchg_vec(s->tp_mem, pending, 0);
            d.tp_epoch = s->tp_epoch;
            d.tp_timeout_ms = (unsigned)env_long("L2B_TP_TIMEOUT_MS", 10000);
            d.x_out = xbuf[cur ^ 1];
        }
    };
    auto norm_done = [&]() {  // after the launch(es) that consumed the pending exchange
        if (pending >= 0) cur ^= 1;
        pending = -1;
    };
    // output of a row-split matrix: residual add on one GPU, push of the partial vector with several
    auto partial_output = [&](MvLaunch& L, const DevMatrix& w, int e) {
        if (tp == 1) {
            L.p.seg[L.p.nseg++] = make_segment(w, PAIR_ADJACENT, EPI_RESIDUAL, s->x, hs);
            L.p.seg[L.p.nseg - 1].out2 = c.dim;
            L.kb = w.kb;
            L.p.resid = s->x;
            return;
        }
        L.p.seg[L.p.nseg++] = make_segment(w, PAIR_ADJACENT, EPI_PUSH, nullptr, hs);
        L.kb = w.kb;
        L.p.tp_push = 1;
        MvTp& d = new_desc(L);
        d.tp_epoch = s->tp_epoch;  // the pushed values carry the token's number as their tag
        d.tp_timeout_ms = (unsigned)env_long("L2B_TP_TIMEOUT_MS", 10000);
        for (int r = 0; r < tp; ++r) {
            d.push_dst[r] = xchg_vec(s->peer_mem[r], e, m->rank);
        }
    };
    const int rope_mode = c.rope_is_neox ? PAIR_NEOX : PAIR_ADJACENT;
    // --- token embedding row -> residual stream (inference.jl:236)
    {
        const int threads = 256, blocks = std::max(1, std::min(32, c.dim / 256));
        CU(cudaLaunchKernelEx_embed(m, s, blocks, threads, 0));
        first = false;
        ++count;
        if (nb == 2) {
            CU(cudaLaunchKernelEx_embed(m, s, blocks, threads, 1));
            ++count;
        }
    }
    for (int l = 0; l < c.n_layers; ++l) {
        const LayerW& w = m->layers[l];
        float* kcl = s->kc + (size_t)l * kvl;
        float* vcl = s->vc + (size_t)l * kvl;
        // --- attention rmsnorm + q/k/v projections + RoPE + cache write (inference.jl:236-260)
        {
            MvSegment segs[3] = {make_segment(w.wq, rope_mode, EPI_ROPE_Q, s->q, hs), make_segment(w.wk, rope_mode, EPI_ROPE_K, kcl, hs),
                                 make_segment(w.wv, PAIR_ADJACENT, EPI_STORE_V, vcl, hs)};
            segs[0].out2 = m->l_qdim();  // the caches take both positions at their own rows: out2 = 0
            // matrices of one storage class (f32, k-quant laid out for 16-block stages, k-quant laid out for 8-block
            // stages) share a launch
            const DevMatrix* mats[3] = {&w.wq, &w.wk, &w.wv};
            for (int cls = 0; cls < 3; ++cls) {
                MvLaunch L;
                base_params(L, c.dim);
                for (int i = 0; i < 3; ++i) {
                    const int ci = segs[i].type == T_F32 ? 0 : (mats[i]->kb == MV_TILE_BLOCKS ? 1 : 2);
                    if (ci == cls) L.p.seg[L.p.nseg++] = segs[i];
                }
                if (L.p.nseg == 0) continue;
                L.kb = cls == 2 ? 8 : MV_TILE_BLOCKS;
                norm_input(L, w.rms_att);
                L2B_TRY(mv(L));
            }
            norm_done();
        }
        // --- attention over the cache (inference.jl:263-278)
        {
            AttnParams a;
            memset(&a, 0, sizeof(a));
            a.q = s->q; a.kc = kcl; a.vc = vcl; a.out = s->att; a.tickets = s->tickets;
            a.part_m = s->part_m; a.part_l = s->part_l; a.part_acc = s->part_acc;
            a.pos = &s->ctl->pos;
            a.n_heads = m->l_heads; a.n_kv = m->l_kv; a.hs = hs; a.seq_len = c.seq_len; a.nsplit = s->nsplit;
            a.nq = nb; a.q_stride = m->l_qdim();
            a.min_chunk = (int)env_long("L2B_ATTN_MIN_CHUNK", 0);
#ifdef L2B_MEASURE
            if (s->attn_trace) a.trace = s->attn_trace + (size_t)l * 1024 * 16;
            a.late_trigger = (int)env_long("L2B_ATTN_LATE_TRIGGER", 0);
#endif
            CU(launch_attention(a, s->gq, s->stream, true));
#ifdef L2B_MEASURE
            if (env_long("L2B_ATTN_TWICE", 0)) CU(launch_attention(a, s->gq, s->stream, true));  // the second launch finds its instructions cached
#endif
            ++count;
        }
        // --- output projection + residual (inference.jl:281-284)
        {
            MvLaunch L;
            base_params(L, m->l_qdim());
            partial_output(L, w.wo, 2 * l);
            L.p.pro = PRO_COPY;
            L.p.x_in = s->att;
            L2B_TRY(mv(L));
            if (tp > 1) pending = 2 * l;
        }
        // --- ffn rmsnorm + gate/up + SwiGLU (inference.jl:287-299)
        {
            MvLaunch L;
            base_params(L, c.dim);
            MvSegment g = make_segment(w.w1, PAIR_DUAL, EPI_SWIGLU, s->hb, hs);
            g.npairs = (int)w.w1.out;
            g.w2 = w.w3.data;
            g.d6_2 = w.w3.d6;
            g.out2 = m->l_hidden;
            L.kb = w.w1.kb;
            L.p.seg[L.p.nseg++] = g;
            norm_input(L, w.rms_ffn);
            L2B_TRY(mv(L));
            norm_done();
        }
        // --- down projection + residual (inference.jl:302-305)
        {
            MvLaunch L;
            base_params(L, m->l_hidden);
            partial_output(L, w.w2, 2 * l + 1);
            L.p.pro = PRO_COPY;
            L.p.x_in = s->hb;
            L2B_TRY(mv(L));
            if (tp > 1) pending = 2 * l + 1;
        }
    }
    if (nb == 2) {  // both positions are followed by prompt tokens: no classifier, no sampling, move on by two
        AdvanceParams ap;
        ap.ctl = s->ctl; ap.prompt = s->prompt; ap.out_tokens = s->out_tokens; ap.epoch = s->tp_epoch;
        ap.vocab = c.vocab_size; ap.status = s->status;
        CU(launch_kernel(advance_pair_kernel, dim3(1), dim3(32), 0, s->stream, true, ap));
        ++count;
        if (nlaunch) *nlaunch = count;
        return L2B_OK;
    }
    // --- final rmsnorm + classifier + per-block argmax (inference.jl:309-312)
    {
        MvLaunch L;
        base_params(L, c.dim);
        L.p.seg[L.p.nseg++] = make_segment(m->output, PAIR_ADJACENT, EPI_LOGITS, s->logits, hs);
        L.kb = m->output.kb;
        norm_input(L, m->rms_final);
        L.p.amax_val = s->amax_val;
        L.p.amax_idx = s->amax_idx;
        L2B_TRY(mv(L));
        norm_done();
    }
    // --- next token (inference.jl:354-368) and advance
    {
        FinalizeParams f;
        memset(&f, 0, sizeof(f));
        f.logits = s->logits; f.vocab = c.vocab_size;
        f.amax_val = s->amax_val; f.amax_idx = s->amax_idx; f.nparts = last_grid;
        f.ctl = s->ctl; f.prompt = s->prompt; f.out_tokens = s->out_tokens; f.advance = 1; f.next_token = s->next_token;
        f.tp_epoch = s->tp_epoch;
        f.status = s->status;
        CU(launch_kernel(finalize_token_kernel, dim3(1), dim3(FIN_THREADS), 0, s->stream, true, f));
        ++count;
    }
    if (nlaunch) *nlaunch = count;
    return L2B_OK;
}

static cudaError_t cudaLaunchKernelEx_embed(const l2b_model* m, l2b_session* s, int blocks, int threads, int second) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(threads);
    cfg.stream = s->stream;
    return cudaLaunchKernelEx(&cfg, embed_row_kernel, m->tok_emb.type, (const uint8_t*)m->tok_emb.data, (const __half*)m->tok_emb.d6,
                              (const int*)&s->ctl->token, (int)m->cfg.dim, s->x + (second ? m->cfg.dim : 0), (const int*)(second ? s->prompt : nullptr),
                              (const int*)&s->ctl->pos, (int)m->cfg.vocab_size);
}


// ---- one persistent kernel per token (token_kernel.cuh) --------------------------------------------------
// Fill the schedule of one matrix-vector operation of the token kernel (the counterpart of plan_matvec: the grid is always
// one block per SM, 16 consumer warps in two groups).  Returns the bytes one ring slot must hold for it.
static int32_t tk_plan(MvParams& p, int planes, int kb_layout, int sms, int& slot_bytes) {
    p.planes = planes;
    const int nb = p.n_in / QK_K;
    int units = 0;
    for (int i = 0; i < p.nseg; ++i) {
        if (p.seg[i].type == T_F32) return fail(L2B_ERR_UNSUPPORTED_TYPE, "the token kernel takes k-quant matrices only");
        p.seg_start[i] = units;
        units += (p.seg[i].npairs + MV_TILE_PAIRS - 1) / MV_TILE_PAIRS;
        if (p.seg[i].pair_mode == PAIR_NEOX) {
            const int h2 = p.seg[i].head_size / 2;
            if (h2 % MV_TILE_PAIRS != 0) return fail(L2B_ERR_BAD_ARG, "head_size must be a multiple of 16 for NeoX RoPE");
            p.neox_magic = (unsigned)((0x100000000ull + h2 - 1) / h2);
        }
    }
    for (int i = p.nseg; i <= MV_MAX_SEG; ++i) p.seg_start[i] = units;
    p.units_lo = units / sms;
    p.units_rem = units % sms;
    p.kb = kb_layout;
    p.nit = (nb + kb_layout - 1) / kb_layout;
    const int kb = std::min(nb, kb_layout);
    slot_bytes = 0;
    for (int i = 0; i < p.nseg; ++i) {
        mv_fill_geometry(p.seg[i], kb, p.nit);
        slot_bytes = std::max(slot_bytes, p.seg[i].ngroups * p.seg[i].gs);
    }
    p.consumers = TK_CONSUMERS;
    p.cgroups = TK_GROUPS;
    p.turns = (p.n_in / 8 + 32 * TK_CONSUMERS - 1) / (32 * TK_CONSUMERS);
    return L2B_OK;
}

// Build the operation table of a token and decide whether the token kernel can run this model (sets s->tk).
static int32_t build_token_kernel(l2b_session* s) {
    const l2b_model* m = s->model;
    const l2b_config& c = m->cfg;
    s->tk = false;
    // Opt-in (L2B_TOKEN_KERNEL=1): measured on a B200 the single launch is not faster than the chain of launches yet (the
    // consumer warps, not the hand-over between kernels, bound the token), so the chain stays the default.
    if (m->tp != 1 || env_long("L2B_TOKEN_KERNEL", 0) == 0) return L2B_OK;
    const DevMatrix* all[] = {&m->tok_emb, &m->output};
    for (const DevMatrix* w : all)
        if (w->type == T_F32) return L2B_OK;
    for (const LayerW& w : m->layers) {
        const DevMatrix* ms[] = {&w.wq, &w.wk, &w.wv, &w.wo, &w.w1, &w.w2, &w.w3};
        for (const DevMatrix* x : ms)
            if (x->type == T_F32) return L2B_OK;
    }
    const int hs = c.dim / c.n_heads, sms = s->di.sms;
    const size_t kvl = kv_layer_elems(m);
    // activation planes kept in shared memory: the longest input of an operation that cannot be cut along its input
    auto up256 = [](int v) { return (v + QK_K - 1) / QK_K * QK_K; };
    int cap = up256(std::max(c.dim, m->l_qdim()));
    auto chunk_of = [&](const DevMatrix& w) -> int {  // input values per operation for a residual matrix
        if (!w.panels) return (int)w.in;
        const int pw = w.kb * QK_K;  // a stored column panel
        return std::max(pw, cap / pw * pw);
    };
    for (const LayerW& w : m->layers) cap = std::max(cap, std::max(up256(std::min<int>((int)w.wo.in, chunk_of(w.wo))), up256(std::min<int>((int)w.w2.in, chunk_of(w.w2)))));
    std::vector<TkOp> ops;
    int slot_bytes = 0;
    auto new_op = [&](int kind, int wait) -> TkOp& {
        TkOp o;
        memset(&o, 0, sizeof(o));
        o.kind = kind;
        o.wait = wait;
        ops.push_back(o);
        return ops.back();
    };
    auto finish_mv = [&](TkOp& o, int kb_layout) -> int32_t {
        int sb = 0;
        L2B_TRY(tk_plan(o.mv, m->planes, kb_layout, sms, sb));
        slot_bytes = std::max(slot_bytes, sb);
        return L2B_OK;
    };
    auto base_mv = [&](TkOp& o, int n_in) {
        o.mv.n_in = n_in;
        o.mv.rope_cs = s->rope_cs;
        o.mv.seq_len = c.seq_len;
    };
    // a matrix whose result is added to the residual stream; cut along its input when the input is longer than the planes
    auto residual_ops = [&](const DevMatrix& w, const float* x_in) -> int32_t {
        const int chunk = std::min<int>((int)w.in, chunk_of(w));
        const int nb = (int)(w.in / QK_K), cb = chunk / QK_K, bb = dev_block_bytes(w.type);
        const size_t panel_bytes = (size_t)w.out * w.kb * bb;
        int first = 1;
        for (int b0 = 0; b0 < nb; b0 += cb, first = 0) {
            const int nbl = std::min(cb, nb - b0);
            TkOp& o = new_op(TK_MATVEC, first);
            base_mv(o, nbl * QK_K);
            MvSegment sg = make_segment(w, PAIR_ADJACENT, EPI_RESIDUAL, s->x, hs);
            if (b0 > 0) {
                sg.w = w.data + (size_t)(b0 / w.kb) * panel_bytes;
                if (sg.d6) sg.d6 = w.d6 + b0;
            }
            sg.d6_nb = nb;
            o.mv.seg[o.mv.nseg++] = sg;
            o.mv.resid = s->x;
            o.mv.pro = PRO_COPY;
            o.mv.x_in = x_in + (size_t)b0 * QK_K;
            L2B_TRY(finish_mv(o, w.kb));
        }
        return L2B_OK;
    };
    const int rope_mode = c.rope_is_neox ? PAIR_NEOX : PAIR_ADJACENT;
    const int gq = choose_gq(m->l_heads, m->l_kv);
    const int groups = m->l_heads / gq;
    const int tk_nsplit = std::max(1, std::min(32, std::min(std::max(1, sms / groups), (c.seq_len + 7) / 8)));
    new_op(TK_EMBED, 0);
    for (int l = 0; l < c.n_layers; ++l) {
        const LayerW& w = m->layers[l];
        float* kcl = s->kc + (size_t)l * kvl;
        float* vcl = s->vc + (size_t)l * kvl;
        {   // attention rmsnorm + q/k/v + RoPE + cache write; matrices laid out for different stage widths go to operations of their own
            MvSegment segs[3] = {make_segment(w.wq, rope_mode, EPI_ROPE_Q, s->q, hs), make_segment(w.wk, rope_mode, EPI_ROPE_K, kcl, hs),
                                 make_segment(w.wv, PAIR_ADJACENT, EPI_STORE_V, vcl, hs)};
            const DevMatrix* mats[3] = {&w.wq, &w.wk, &w.wv};
            int first = 1;
            for (int cls = 0; cls < 2; ++cls) {
                const int kb_layout = cls == 0 ? MV_TILE_BLOCKS : 8;
                int n = 0;
                for (int i = 0; i < 3; ++i) n += mats[i]->kb == kb_layout;
                if (!n) continue;
                TkOp& o = new_op(TK_MATVEC, first);
                first = 0;
                base_mv(o, c.dim);
                for (int i = 0; i < 3; ++i)
                    if (mats[i]->kb == kb_layout) o.mv.seg[o.mv.nseg++] = segs[i];
                o.mv.pro = PRO_RMSNORM;
                o.mv.gain = w.rms_att;
                o.mv.x_in = s->x;
                L2B_TRY(finish_mv(o, kb_layout));
            }
        }
        {
            TkOp& o = new_op(TK_ATTN, 1);
            AttnParams& a = o.at;
            a.q = s->q; a.kc = kcl; a.vc = vcl; a.out = s->att; a.tickets = s->tickets;
            a.part_m = s->part_m; a.part_l = s->part_l; a.part_acc = s->part_acc;
            a.n_heads = m->l_heads; a.n_kv = m->l_kv; a.hs = hs; a.seq_len = c.seq_len; a.nsplit = tk_nsplit;
            a.min_chunk = (int)env_long("L2B_ATTN_MIN_CHUNK", 0);
        }
        L2B_TRY(residual_ops(w.wo, s->att));
        {
            TkOp& o = new_op(TK_MATVEC, 1);
            base_mv(o, c.dim);
            MvSegment g = make_segment(w.w1, PAIR_DUAL, EPI_SWIGLU, s->hb, hs);
            g.npairs = (int)w.w1.out;
            g.w2 = w.w3.data;
            g.d6_2 = w.w3.d6;
            o.mv.seg[o.mv.nseg++] = g;
            o.mv.pro = PRO_RMSNORM;
            o.mv.gain = w.rms_ffn;
            o.mv.x_in = s->x;
            if (w.w1.kb != w.w3.kb) return L2B_OK;
            L2B_TRY(finish_mv(o, w.w1.kb));
        }
        L2B_TRY(residual_ops(w.w2, s->hb));
    }
    {
        TkOp& o = new_op(TK_MATVEC, 1);
        base_mv(o, c.dim);
        o.mv.seg[o.mv.nseg++] = make_segment(m->output, PAIR_ADJACENT, EPI_LOGITS, s->logits, hs);
        o.mv.pro = PRO_RMSNORM;
        o.mv.gain = m->rms_final;
        o.mv.x_in = s->x;
        o.mv.amax_val = s->amax_val;
        o.mv.amax_idx = s->amax_idx;
        L2B_TRY(finish_mv(o, m->output.kb));
    }
    new_op(TK_FINAL, 1);
    if ((int)ops.size() > TK_MAX_OPS) return L2B_OK;
    const int max_total = std::min<int>((int)env_long("L2B_TK_SMEM_KB", 227) * 1024, s->di.max_smem_optin);
    TkSmem sm = tk_smem_layout(m->planes, cap, tk_attention_scratch_bytes(), slot_bytes, max_total);
    if (sm.nslots < 2 * TK_GROUPS) return L2B_OK;  // the ring would be too shallow: the kernel chain runs instead
    TkParams& P = s->tkp;
    memset(&P, 0, sizeof(P));
    if (!s->tk_ops) CU(cudaMalloc(&s->tk_ops, ops.size() * sizeof(TkOp)));
    if (!s->tk_sync) CU(cudaMalloc(&s->tk_sync, TK_MAX_OPS * sizeof(unsigned)));
    CU(cudaMemcpy(s->tk_ops, ops.data(), ops.size() * sizeof(TkOp), cudaMemcpyHostToDevice));
    CU(cudaMemset(s->tk_sync, 0, TK_MAX_OPS * sizeof(unsigned)));
#ifdef L2B_MEASURE
    if (env_long("L2B_TK_TRACE", 0)) {
        if (!s->tk_trace) CU(cudaMalloc(&s->tk_trace, ops.size() * 4 * 8));
        CU(cudaMemset(s->tk_trace, 0, ops.size() * 4 * 8));
        P.trace = s->tk_trace;
        s->tk_kinds.clear();
        for (const TkOp& o : ops) s->tk_kinds.push_back(o.kind * 1000000 + (o.kind == TK_MATVEC ? o.mv.n_in : 0) + (o.wait ? 500000 : 0));
    }
#endif
    P.ops = s->tk_ops;
    P.n_ops = (int)ops.size();
    P.sync = s->tk_sync;
    P.ctl = s->ctl;
    P.status = s->status;
    P.timeout_ms = (unsigned)env_long("L2B_TK_TIMEOUT_MS", 2000);
    P.embed.type = m->tok_emb.type; P.embed.table = m->tok_emb.data; P.embed.d6 = m->tok_emb.d6;
    P.embed.n = c.dim; P.embed.vocab = c.vocab_size; P.embed.x = s->x;
    FinalizeParams& f = P.fin;
    f.logits = s->logits; f.vocab = c.vocab_size;
    f.amax_val = s->amax_val; f.amax_idx = s->amax_idx; f.nparts = sms;
    f.ctl = s->ctl; f.prompt = s->prompt; f.out_tokens = s->out_tokens; f.advance = 1; f.next_token = s->next_token;
    f.status = s->status;
    P.sm = sm;
    s->tk = true;
    return L2B_OK;
}

static cudaError_t launch_token_kernel(l2b_session* s, bool cooperative) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(s->di.sms);
    cfg.blockDim = dim3(TK_THREADS);
    cfg.dynamicSmemBytes = (size_t)s->tkp.sm.total;
    cfg.stream = s->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all blocks resident at once: they wait for one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = cooperative ? 1 : 0;
    switch (s->model->planes) {
        case 1: return cudaLaunchKernelEx(&cfg, token_kernel<1>, s->tkp);
        case 2: return cudaLaunchKernelEx(&cfg, token_kernel<2>, s->tkp);
        default: return cudaLaunchKernelEx(&cfg, token_kernel<3>, s->tkp);
    }
}

// Capture the token kernel as the one-position graph.  Returns false (and leaves no graph) when that is not possible.
static bool capture_token_kernel_graph(l2b_session* s) {
    for (int coop = 1; coop >= 0; --coop) {
        cudaGraph_t g = nullptr;
        if (cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) break;
        cudaError_t le = launch_token_kernel(s, coop != 0);
        cudaError_t ce = cudaStreamEndCapture(s->stream, &g);
        cudaError_t ie = cudaErrorUnknown;
        if (le == cudaSuccess && ce == cudaSuccess && g) ie = cudaGraphInstantiate(&s->graph, g, 0);
        if (g) cudaGraphDestroy(g);
        if (ie == cudaSuccess) {
            s->kernels_per_token = 1;
            return true;
        }
        (void)cudaGetLastError();
        s->graph = nullptr;
    }
    return false;
}

static int32_t capture_token_graph(l2b_session* s) {
    cudaGraph_t g = nullptr;
    const size_t max_descs = 4 * (size_t)s->model->cfg.n_layers + 2;  // <= 2 pushes + 2 summing prologues per layer, + logits
    if (s->model->tp > 1 && !s->tp_descs) CU(cudaMalloc(&s->tp_descs, max_descs * sizeof(MvTp)));
    s->tp_descs_host.clear();
    s->tp_descs_host.reserve(max_descs + 8);
    L2B_TRY(build_token_kernel(s));
    int32_t es = L2B_OK;
    cudaError_t ce = cudaSuccess;
    if (s->tk && capture_token_kernel_graph(s)) {
        // the one-position graph is the token kernel; the two-position prompt graph below still uses the kernel chain
    } else {
    s->tk = false;
    CU(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
    es = enqueue_token(s, &s->kernels_per_token);
    ce = cudaStreamEndCapture(s->stream, &g);
    if (es == L2B_OK && ce == cudaSuccess && !s->tp_descs_host.empty()) {
        if (s->tp_descs_host.size() > max_descs) es = fail(L2B_ERR_STATE, "more tensor-parallel launches than descriptors");
        else ce = cudaMemcpy(s->tp_descs, s->tp_descs_host.data(), s->tp_descs_host.size() * sizeof(MvTp), cudaMemcpyHostToDevice);
    }
    if (es != L2B_OK) {
        if (g) cudaGraphDestroy(g);
        return es;
    }
    CU(ce);
    {
        cudaError_t ie = cudaGraphInstantiate(&s->graph, g, 0);
        cudaGraphDestroy(g);
        CU(ie);
    }
    }
    // Second graph: two prompt positions per pass.  Needs k-quant matrices throughout, three planes, one GPU.
    if (s->model->tp == 1 && s->model->planes == 3 && s->all_kquant && !s->trace && env_long("L2B_PREFILL_PAIRS", 1) != 0) {
        cudaGraph_t g2 = nullptr;
        int n2 = 0;
        CU(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
        es = enqueue_token(s, &n2, 2);
        s->kernels_per_pair = n2;
        ce = cudaStreamEndCapture(s->stream, &g2);
        if (es != L2B_OK || ce != cudaSuccess) {
            // e.g. two sets of activation planes of a very long input do not fit in shared memory: prompts then
            // go through the one-position graph, as they do for f32 models
            (void)cudaGetLastError();
            if (g2) cudaGraphDestroy(g2);
            g_last_error.clear();
        } else {
            cudaError_t ie = cudaGraphInstantiate(&s->graph2, g2, 0);
            cudaGraphDestroy(g2);
            CU(ie);
        }
    }
    return L2B_OK;
}

extern "C" int32_t l2b_session_create(l2b_model* m, void* stream, l2b_session** out) {
    if (!m || !out) return fail(L2B_ERR_BAD_ARG, "null argument");
    *out = nullptr;
    if (!m->finalized) return fail(L2B_ERR_STATE, "l2b_model_finalize has not been called");
    CU(cudaSetDevice(m->device));
    L2B_TRY(check_kernel_attrs());
    const l2b_config& c = m->cfg;
    const int hs = c.dim / c.n_heads;
    l2b_session* s = new l2b_session();
    s->model = m;
    int32_t st = L2B_OK;
    auto guard = [&](int32_t code) {
        if (code != L2B_OK && st == L2B_OK) st = code;
        return code == L2B_OK;
    };
    auto run = [&]() -> int32_t {
        L2B_TRY(query_device(s->di));
        if (stream) s->stream = (cudaStream_t)stream;
        else {
            CU(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking));
            s->own_stream = true;
        }
        s->gq = choose_gq(m->l_heads, m->l_kv);
        // blocks per head group in the attention launches: whole clusters for the decode kernel (L2B_ATTN_SPLITS is rounded up)
        // Enough clusters for the longest context, but no more blocks than about 1.75 per SM: with many head groups (Phi-3-mini
        // shape, 32 groups, seq_len 4096) one cluster per group gave 631 tok/s, two 564, four 543.
        {
            const int groups = m->l_heads / s->gq;
            const int by_sms = std::max(1, s->di.sms * 7 / 4 / (groups * ATTN_CL));
            const long want = env_long("L2B_ATTN_SPLITS", std::min(decode_splits(c.seq_len), by_sms * ATTN_CL));
            s->nsplit = (int)std::max<long>(ATTN_CL, std::min<long>(4 * ATTN_CL, (want + ATTN_CL - 1) / ATTN_CL * ATTN_CL));
        }
        const size_t kvl = kv_layer_elems(m);
        // q, att, hb and the caches hold this rank's heads / hidden units only (everything, on one GPU)
        // (two of each vector: the two-position prompt passes keep both positions' activations side by side)
        CU(cudaMalloc(&s->x, (size_t)c.dim * 4 * 2));
        CU(cudaMalloc(&s->q, (size_t)m->l_qdim() * 4 * 2));
        CU(cudaMalloc(&s->att, (size_t)m->l_qdim() * 4 * 2));
        CU(cudaMalloc(&s->tickets, (size_t)c.n_heads * 4 * 2));
        CU(cudaMalloc(&s->hb, (size_t)m->l_hidden * 4 * 2));
        CU(cudaMalloc(&s->logits, (size_t)c.vocab_size * 4));
        CU(cudaMalloc(&s->kc, kvl * c.n_layers * 4));
        CU(cudaMalloc(&s->vc, kvl * c.n_layers * 4));
        // (room for 32 splits, the most any launch uses: the token kernel chooses its own split count)
        CU(cudaMalloc(&s->part_m, (size_t)m->l_heads * 32 * 4 * 2));
        CU(cudaMalloc(&s->part_l, (size_t)m->l_heads * 32 * 4 * 2));
        CU(cudaMalloc(&s->part_acc, (size_t)m->l_heads * 32 * hs * 4 * 2));
        CU(cudaMalloc(&s->amax_val, (size_t)s->di.sms * 4));
        CU(cudaMalloc(&s->amax_idx, (size_t)s->di.sms * 4));
        CU(cudaMalloc(&s->ctl, sizeof(Control)));
        CU(cudaMalloc(&s->next_token, 8));  // next token and status word side by side: one copy brings both back
        s->status = s->next_token + 1;
        CU(cudaMalloc(&s->prompt, (size_t)c.seq_len * 4));
        CU(cudaMalloc(&s->out_tokens, (size_t)c.seq_len * 4));
        CU(cudaMallocHost(&s->h_ctl, sizeof(Control)));
        CU(cudaMallocHost(&s->h_small, 16));
        CU(cudaEventCreate(&s->ev0));
        CU(cudaEventCreate(&s->ev1));
        CU(cudaEventCreate(&s->ev_mid));
        CU(cudaMemsetAsync(s->kc, 0, kvl * c.n_layers * 4, s->stream));
        CU(cudaMemsetAsync(s->vc, 0, kvl * c.n_layers * 4, s->stream));
        CU(cudaMemsetAsync(s->status, 0, 4, s->stream));
        CU(cudaMemsetAsync(s->tickets, 0, (size_t)c.n_heads * 4 * 2, s->stream));
        CU(cudaMemsetAsync(s->ctl, 0, sizeof(Control), s->stream));
        CU(cudaMemsetAsync(s->prompt, 0, (size_t)c.seq_len * 4, s->stream));
        std::vector<float> cs;
        rope_table_host(cs, c.seq_len, hs, c.rope_freq_base);
        CU(cudaMalloc(&s->rope_cs, cs.size() * 4));
        CU(cudaMemcpyAsync(s->rope_cs, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice, s->stream));
        CU(cudaStreamSynchronize(s->stream));
#ifdef L2B_MEASURE
        if (env_long("L2B_TRACE_TOKEN", 0)) {
            const size_t n = (size_t)(4 * c.n_layers + 1) * s->di.sms * 16;
            CU(cudaMalloc(&s->trace, n * 8));
            CU(cudaMemset(s->trace, 0, n * 8));
            CU(cudaMalloc(&s->attn_trace, (size_t)c.n_layers * 1024 * 16 * 8));
            CU(cudaMemset(s->attn_trace, 0, (size_t)c.n_layers * 1024 * 16 * 8));
        }
#endif
        if (m->tp > 1) {
            // exchange memory; the token graph is captured by l2b_session_tp_connect, once the peers' mappings exist
            const size_t n_exch = 2 * (size_t)c.n_layers;
            s->tp_bytes = n_exch * m->tp * c.dim * 8;
            CU(cudaMalloc(&s->tp_mem, s->tp_bytes));
            CU(cudaMemset(s->tp_mem, 0, s->tp_bytes));
            CU(cudaMalloc(&s->x2, (size_t)c.dim * 4));
            CU(cudaMalloc(&s->tp_epoch, 4));
            CU(cudaMemset(s->tp_epoch, 0, 4));
            s->peer_mem[m->rank] = s->tp_mem;
            return L2B_OK;
        }
        return capture_token_graph(s);
    };
    guard(run());
    if (st != L2B_OK) {
        session_free(s);
        return st;
    }
    *out = s;
    return L2B_OK;
}

extern "C" int32_t l2b_session_reset(l2b_session* s) {
    if (!s) return fail(L2B_ERR_BAD_ARG, "null session");
    CU(cudaSetDevice(s->model->device));
    const size_t bytes = kv_layer_elems(s->model) * s->model->cfg.n_layers * 4;
    CU(cudaMemsetAsync(s->kc, 0, bytes, s->stream));
    CU(cudaMemsetAsync(s->vc, 0, bytes, s->stream));
    CU(cudaStreamSynchronize(s->stream));
    return L2B_OK;
}

extern "C" int32_t l2b_session_destroy(l2b_session* s) {
    if (!s) return L2B_OK;
    cudaSetDevice(s->model->device);
    if (s->stream) cudaStreamSynchronize(s->stream);
    session_free(s);
    return L2B_OK;
}

// ---- tensor-parallel wiring --------------------------------------------------------------------
// One process per GPU.  Each rank exports an IPC handle of its exchange memory; the host moves the handles between
// the processes (any transport: torch.distributed, MPI, a file) and hands every rank the full list.
extern "C" int32_t l2b_session_tp_handle(l2b_session* s, void* handle64) {
    if (!s || !handle64) return fail(L2B_ERR_BAD_ARG, "null argument");
    if (s->model->tp <= 1) return fail(L2B_ERR_STATE, "the model was created with tp_size <= 1");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    CU(cudaSetDevice(s->model->device));
    cudaIpcMemHandle_t h;
    CU(cudaIpcGetMemHandle(&h, s->tp_mem));
    memcpy(handle64, &h, 64);
    return L2B_OK;
}

extern "C" int32_t l2b_session_tp_connect(l2b_session* s, const void* handles, int32_t count) {
    if (!s || !handles) return fail(L2B_ERR_BAD_ARG, "null argument");
    const l2b_model* m = s->model;
    if (m->tp <= 1) return fail(L2B_ERR_STATE, "the model was created with tp_size <= 1");
    if (count != m->tp) return fail(L2B_ERR_BAD_ARG, "one handle per rank is needed, ordered by rank");
    if (s->tp_connected) return fail(L2B_ERR_STATE, "the session is connected already");
    CU(cudaSetDevice(m->device));
    for (int r = 0; r < m->tp; ++r) {
        if (r == m->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t*)handles + (size_t)r * 64, 64);
        void* ptr = nullptr;
        CU(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        s->peer_mem[r] = (uint8_t*)ptr;
    }
    L2B_TRY(capture_token_graph(s));
    s->tp_connected = true;
    return L2B_OK;
}

static int32_t check_status_word(l2b_session* s) {
    if (s->h_small[1] != DEV_OK && s->tk_sync) cudaMemsetAsync(s->tk_sync, 0, TK_MAX_OPS * sizeof(unsigned), s->stream);  // an abandoned token leaves the arrival counter anywhere
    if (s->h_small[1] == DEV_ERR_TMA_TIMEOUT) {
        cudaMemsetAsync(s->status, 0, 4, s->stream);
        return fail(L2B_ERR_TIMEOUT, "a bounded wait on a weight copy ran out inside a kernel");
    }
    if (s->h_small[1] == DEV_ERR_PEER_TIMEOUT) {
        cudaMemsetAsync(s->status, 0, 4, s->stream);
        return fail(L2B_ERR_TIMEOUT, "the partial results of another tensor-parallel rank did not arrive in time");
    }
    if (s->h_small[1] == DEV_ERR_BAD_INDEX) {
        cudaMemsetAsync(s->status, 0, 4, s->stream);
        return fail(L2B_ERR_CUDA, "no valid token could be chosen (the logits are not finite); token 0 was substituted");
    }
    if (s->h_small[1] != DEV_OK) {
        cudaMemsetAsync(s->status, 0, 4, s->stream);
        return fail(L2B_ERR_CUDA, "kernel reported device status " + std::to_string(s->h_small[1]));
    }
    return L2B_OK;
}

// One graph launch with the control block set from the host.
static int32_t run_one(l2b_session* s, int token, int pos, float temperature, double uniform) {
    const l2b_config& c = s->model->cfg;
    if (token < 0 || token >= c.vocab_size) return fail(L2B_ERR_BAD_ARG, "token id out of range");
    if (pos < 0 || pos >= c.seq_len) return fail(L2B_ERR_BAD_ARG, "position out of range (seq_len)");
    if (temperature < 0.f) return fail(L2B_ERR_BAD_ARG, "temperature must be >= 0");
    if (!s->graph) return fail(L2B_ERR_STATE, "tensor-parallel session: call l2b_session_tp_connect first");
    CU(cudaSetDevice(s->model->device));
    Control& h = *s->h_ctl;
    memset(&h, 0, sizeof(h));
    h.token = token;
    h.pos = pos;
    h.n_prompt = 0;
    h.temperature = temperature;
    h.uniform = uniform;
    CU(cudaEventRecord(s->ev0, s->stream));
    CU(cudaMemcpyAsync(s->ctl, s->h_ctl, sizeof(Control), cudaMemcpyHostToDevice, s->stream));
    CU(cudaGraphLaunch(s->graph, s->stream));
    s->last_launches = s->kernels_per_token;
    CU(cudaMemcpyAsync(&s->h_small[0], s->next_token, 8, cudaMemcpyDeviceToHost, s->stream));  // [0] next token, [1] status
    CU(cudaEventRecord(s->ev1, s->stream));
    CU(cudaStreamSynchronize(s->stream));
    CU(cudaEventElapsedTime(&s->last_ms, s->ev0, s->ev1));
    return check_status_word(s);
}

// ---- many-token prompt pass ---------------------------------------------------------------------------------
// The reference runs transformer! once per prompt token (src/inference.jl:349-356).  For prompt positions that are all followed
// by a prompt token (no logits needed) the layers are run for up to PF_MAX_TOK tokens at once: every matrix product is one
// launch of the tensor-core GEMM (20 tokens per pass over a weight tile), the element-wise steps are small kernels over
// [tokens][dim] arrays, attention serves every token's query against the cache (causal: token t sees positions <= pos0 + t).
// Needs q4_K / q5_K layer matrices, three activation planes, one GPU; otherwise the caller uses the decode passes.
constexpr int PF_MAX_TOK = 240;
constexpr int PF_MIN_TOK = 12;

// Every layer for n tokens whose residual-stream rows are in B.x.  One sequence: token t sits at position pos0 + t and the
// layer's caches are kc / vc + l * layer_stride.  Batched decode (pos_list non-null): token t is the next position pos_list[t]
// of sequence t, whose caches lie seq_stride * t further.
static int32_t enqueue_layers_gemm(const l2b_model* m, const GemmBufs& B, int n, float* kc, float* vc, size_t layer_stride, int pos0, const int* pos_list,
                                   size_t seq_stride, const float* rope_cs, int gq, int* status, cudaStream_t st) {
    const l2b_config& c = m->cfg;
    const int hs = c.dim / c.n_heads, kv_dim = hs * c.n_kv_heads;
    for (int l = 0; l < c.n_layers; ++l) {
        const LayerW& w = m->layers[l];
        float* kcl = kc + (size_t)l * layer_stride;
        float* vcl = vc + (size_t)l * layer_stride;
        L2B_TRY(launch_quantise_rows(B.x, w.rms_att, B.act, c.dim, c.dim, n, st));
        L2B_TRY(launch_kq_gemm(w.wq, B.act, n, B.q, c.dim, nullptr, status, st));
        L2B_TRY(launch_kq_gemm(w.wk, B.act, n, B.k, kv_dim, nullptr, status, st));
        L2B_TRY(launch_kq_gemm(w.wv, B.act, n, B.v, kv_dim, nullptr, status, st));
        RopeKvParams r;
        memset(&r, 0, sizeof(r));
        r.q = B.q; r.k = B.k; r.v = B.v; r.kc = kcl; r.vc = vcl; r.rope_cs = rope_cs;
        r.n_tok = n; r.q_dim = c.dim; r.kv_dim = kv_dim; r.hs = hs; r.seq_len = c.seq_len; r.pos0 = pos0; r.neox = c.rope_is_neox;
        r.pos_list = pos_list; r.cache_stride = seq_stride;
        rope_kv_kernel<<<dim3(8, n), 256, 0, st>>>(r);
        CU(cudaGetLastError());
        AttnParams a;
        memset(&a, 0, sizeof(a));
        a.q = B.q; a.kc = kcl; a.vc = vcl; a.out = B.att; a.tickets = B.tickets;
        a.part_m = B.pm; a.part_l = B.pl; a.part_acc = B.pacc;
        a.pos = nullptr; a.pos_base = pos0; a.pos_list = pos_list; a.cache_stride_q = seq_stride;
        a.n_heads = c.n_heads; a.n_kv = c.n_kv_heads; a.hs = hs; a.seq_len = c.seq_len; a.nsplit = B.nsplit;
        a.nq = std::max(n, 2);  // (a one-token pass takes the many-query form of the kernel too: the second query copy leaves at once)
        a.q_stride = c.dim;
        a.min_chunk = 256;  // many queries already fill the GPU: split a query's positions only when there are many
        if (n < 2) return fail(L2B_ERR_BAD_ARG, "a many-token pass needs at least two tokens");
        CU(launch_attention(a, gq, st, false));
        L2B_TRY(launch_quantise_rows(B.att, nullptr, B.act, c.dim, c.dim, n, st));
        L2B_TRY(launch_kq_gemm(w.wo, B.act, n, B.x, c.dim, B.x, status, st));
        L2B_TRY(launch_quantise_rows(B.x, w.rms_ffn, B.act, c.dim, c.dim, n, st));
        L2B_TRY(launch_kq_gemm(w.w1, B.act, n, B.g, c.hidden_dim, nullptr, status, st));
        L2B_TRY(launch_kq_gemm(w.w3, B.act, n, B.u, c.hidden_dim, nullptr, status, st));
        swiglu_rows_kernel<<<1184, 256, 0, st>>>(B.g, B.u, (size_t)n * c.hidden_dim);
        CU(cudaGetLastError());
        L2B_TRY(launch_quantise_rows(B.g, nullptr, B.act, c.hidden_dim, c.hidden_dim, n, st));
        L2B_TRY(launch_kq_gemm(w.w2, B.act, n, B.x, c.dim, B.x, status, st));
    }
    return L2B_OK;
}

static bool gemm_layers_supported(const l2b_model* m) {
    if (m->tp != 1 || m->planes != 3 || !encode_tiled_fn() || m->tok_emb.type == T_F32) return false;
    for (const LayerW& w : m->layers) {
        const DevMatrix* ms[] = {&w.wq, &w.wk, &w.wv, &w.wo, &w.w1, &w.w2, &w.w3};
        for (const DevMatrix* x : ms)
            if (!gemm_supported(*x)) return false;
    }
    return true;
}

static bool alloc_gemm_bufs(const l2b_model* m, GemmBufs& B, size_t T) {
    const l2b_config& c = m->cfg;
    const int hs = c.dim / c.n_heads, kv_dim = hs * c.n_kv_heads;
    B.nsplit = c.seq_len >= 2048 ? 4 : 1;
    auto alloc = [&](auto*& ptr, size_t bytes) { return cudaMalloc((void**)&ptr, bytes) == cudaSuccess; };
    bool ok = alloc(B.x, T * c.dim * 4) && alloc(B.q, T * c.dim * 4) && alloc(B.k, T * kv_dim * 4) && alloc(B.v, T * kv_dim * 4) &&
              alloc(B.att, T * c.dim * 4) && alloc(B.g, T * c.hidden_dim * 4) && alloc(B.u, T * c.hidden_dim * 4) &&
              alloc(B.pm, T * c.n_heads * B.nsplit * 4) && alloc(B.pl, T * c.n_heads * B.nsplit * 4) &&
              alloc(B.pacc, T * c.n_heads * B.nsplit * hs * 4) && alloc(B.tickets, T * c.n_heads * 4) &&
              alloc(B.act, gemm_act_bytes(std::max(c.dim, c.hidden_dim), (int)T));
    if (ok) ok = cudaMemset(B.tickets, 0, T * c.n_heads * 4) == cudaSuccess;
    if (!ok) {
        (void)cudaGetLastError();
        free_gemm_bufs(B);
    }
    return ok;
}

static bool prefill_gemm_eligible(l2b_session* s) {
    if (s->pf_checked) return s->pf_ok;
    s->pf_checked = true;
    // (a pass that cannot get its buffers leaves prompts to the decode passes)
    s->pf_ok = env_long("L2B_PREFILL_GEMM", 1) != 0 && gemm_layers_supported(s->model) && alloc_gemm_bufs(s->model, s->pf, PF_MAX_TOK);
    return s->pf_ok;
}

// Positions pos0 .. pos0 + n - 1 of the prompt already in s->prompt (device), 2 <= n <= PF_MAX_TOK; all enqueued on the session stream.
static int32_t enqueue_prefill_gemm(l2b_session* s, int pos0, int n) {
    const l2b_model* m = s->model;
    const l2b_config& c = m->cfg;
    cudaStream_t st = s->stream;
    embed_rows_kernel<<<dim3(std::max(1, std::min(16, c.dim / 256)), n), 256, 0, st>>>(m->tok_emb.type, m->tok_emb.data, m->tok_emb.d6, s->prompt + pos0, c.dim,
                                                                                      c.vocab_size, s->pf.x);
    CU(cudaGetLastError());
    L2B_TRY(enqueue_layers_gemm(m, s->pf, n, s->kc, s->vc, kv_layer_elems(m), pos0, nullptr, 0, s->rope_cs, s->gq, s->status, st));
    fill_forced_kernel<<<1, 256, 0, st>>>(s->prompt, s->out_tokens, pos0, n);
    CU(cudaGetLastError());
    s->last_launches += 2 + 14LL * c.n_layers;  // per layer: 4 quantise, 7 GEMM, RoPE + cache write, attention, SwiGLU
    return L2B_OK;
}

// Feed the forced positions [from, to) (each followed by a prompt token) and leave the loop state at position `to`, whose
// token is host_tokens[to - base].  Many-token passes where possible, the decode graphs for the rest.
static int32_t enqueue_forced_positions(l2b_session* s, int from, int to, const int32_t* host_prompt_at_from) {
    int i = from;
    if (to - from >= PF_MIN_TOK && prefill_gemm_eligible(s)) {
        while (i < to) {
            const int n = std::min(PF_MAX_TOK, to - i);
            L2B_TRY(enqueue_prefill_gemm(s, i, n));
            i += n;
        }
        // the decode graphs read the loop state from the device: move it to position i
        Control& h = *s->h_ctl;
        h.token = host_prompt_at_from[i - from];
        h.pos = i;
        CU(cudaMemcpyAsync(s->ctl, s->h_ctl, sizeof(Control), cudaMemcpyHostToDevice, s->stream));
    }
    while (i < to) {
        const bool pair = s->graph2 && i + 2 <= to;
        CU(cudaGraphLaunch(pair ? s->graph2 : s->graph, s->stream));
        s->last_launches += pair ? s->kernels_per_pair : s->kernels_per_token;
        i += pair ? 2 : 1;
    }
    return L2B_OK;
}

#ifdef L2B_MEASURE
static void dump_token_trace(l2b_session* s) {
    const int nl = s->trace_launches, sms = s->di.sms;
    std::vector<unsigned long long> h((size_t)nl * sms * 16);
    if (cudaMemcpy(h.data(), s->trace, h.size() * 8, cudaMemcpyDeviceToHost) != cudaSuccess) return;
    unsigned long long t0 = ~0ull;
    for (int b = 0; b < sms; ++b)
        if (h[b * 16]) t0 = std::min(t0, h[b * 16]);
    fprintf(stderr, "[l2b token trace] per fused launch, us after the previous fused launch's last block ended: block start min/avg/max | first copy issued avg/max | "
                    "wait over min/avg/max | planes built avg/max | consumers done min/avg/max | finisher done avg/max | blocks\n");
    double prev_end = 0;
    for (int k = 0; k < nl; ++k) {
        double mn[8], mx[8], av[8];
        for (int i = 0; i < 8; ++i) mn[i] = 1e30, mx[i] = -1e30, av[i] = 0;
        int nb = 0;
        for (int b = 0; b < sms; ++b) {
            const unsigned long long* r = &h[((size_t)k * sms + b) * 16];
            if (!r[0]) continue;
            ++nb;
            for (int i : {0, 1, 2, 3, 6, 7}) {
                const int src = i == 7 ? 8 : i;  // slot 7 of the statistics: the finisher warp's end (stamp 8)
                const double v = r[src] ? (double)(r[src] - t0) / 1e3 : 0.0;
                mn[i] = std::min(mn[i], v); mx[i] = std::max(mx[i], v); av[i] += v;
            }
        }
        if (!nb) continue;
        auto rel = [&](double v) { return v - prev_end; };
        if (k < 16 || k >= nl - 3)
            fprintf(stderr, "  launch %3d: start %6.2f %6.2f %6.2f | copy %6.2f %6.2f | wait %6.2f %6.2f %6.2f | planes %6.2f %6.2f | end %6.2f %6.2f %6.2f | fin %6.2f %6.2f | %d  (abs %.2f)\n", k,
                    rel(mn[0]), rel(av[0] / nb), rel(mx[0]), rel(av[1] / nb), rel(mx[1]), rel(mn[2]), rel(av[2] / nb), rel(mx[2]), rel(av[3] / nb), rel(mx[3]),
                    rel(mn[6]), rel(av[6] / nb), rel(mx[6]), rel(av[7] / nb), rel(mx[7]), nb, mx[7]);
        prev_end = std::max(mx[6], mx[7]);
        if (s->attn_trace && k % 4 == 0 && k / 4 < s->model->cfg.n_layers && k < 16) {  // the attention launch that follows this layer's qkv launch
            std::vector<unsigned long long> a((size_t)1024 * 16);
            if (cudaMemcpy(a.data(), s->attn_trace + (size_t)(k / 4) * 1024 * 16, a.size() * 8, cudaMemcpyDeviceToHost) != cudaSuccess) continue;
            double amn[16], amx[16], aav[16];
            int cnt[16];
            for (int i = 0; i < 16; ++i) amn[i] = 1e30, amx[i] = -1e30, aav[i] = 0, cnt[i] = 0;
            for (int b = 0; b < 1024; ++b)
                for (int i = 0; i < 16; ++i) {
                    if (!a[(size_t)b * 16 + i]) continue;
                    const double v = (double)(a[(size_t)b * 16 + i] - t0) / 1e3 - prev_end;
                    amn[i] = std::min(amn[i], v); amx[i] = std::max(amx[i], v); aav[i] += v; ++cnt[i];
                }
            fprintf(stderr, "     attention: blocks %d | start %6.2f %6.2f %6.2f | wait over %6.2f %6.2f %6.2f | positions done %6.2f %6.2f %6.2f | merged %6.2f %6.2f %6.2f\n", cnt[0],
                    amn[0], aav[0] / std::max(cnt[0], 1), amx[0], amn[1], aav[1] / std::max(cnt[1], 1), amx[1], amn[2], aav[2] / std::max(cnt[2], 1), amx[2],
                    amn[3], aav[3] / std::max(cnt[3], 1), amx[3]);
            fprintf(stderr, "                block barrier %6.2f %6.2f | pushed %6.2f %6.2f | cluster barrier over %6.2f %6.2f (avg, max)\n", aav[4] / std::max(cnt[4], 1), amx[4],
                    aav[5] / std::max(cnt[5], 1), amx[5], aav[6] / std::max(cnt[6], 1), amx[6]);
            fprintf(stderr, "                averages: block max known %6.2f | block sums done %6.2f | output pushed %6.2f | received max known %6.2f | received sums done %6.2f\n",
                    aav[7] / std::max(cnt[7], 1), aav[8] / std::max(cnt[8], 1), aav[9] / std::max(cnt[9], 1), aav[10] / std::max(cnt[10], 1), aav[11] / std::max(cnt[11], 1));
        }
    }
}
#endif

extern "C" int32_t l2b_forward(l2b_session* s, int32_t token, int32_t pos, float* host_logits) {
    if (!s) return fail(L2B_ERR_BAD_ARG, "null session");
    L2B_TRY(run_one(s, token, pos, 0.f, 0.0));
#ifdef L2B_MEASURE
    if (s->trace) dump_token_trace(s);
    if (s->tk_trace && s->tk) {  // per-operation timeline of block 0 of the token kernel
        const size_t n = s->tk_kinds.size();
        std::vector<unsigned long long> h(n * 4);
        if (cudaMemcpy(h.data(), s->tk_trace, n * 32, cudaMemcpyDeviceToHost) == cudaSuccess) {
            const unsigned long long t0 = h[0];
            fprintf(stderr, "[l2b token kernel trace] block 0, us since its first stamp: op kind wait n_in | wait-over  planes-built  tiles-done  arrived\n");
            for (size_t i = 0; i < n; ++i) {
                if (i > 26 && i + 6 < n) continue;
                auto us = [&](int k) { return h[i * 4 + k] ? (double)(h[i * 4 + k] - t0) / 1e3 : 0.0; };
                fprintf(stderr, "  %3zu %d %d %6d | %9.2f %9.2f %9.2f %9.2f\n", i, s->tk_kinds[i] / 1000000, (s->tk_kinds[i] / 500000) & 1, s->tk_kinds[i] % 500000,
                        us(0), us(1), us(2), us(3));
            }
        }
    }
#endif
    if (host_logits) CU(cudaMemcpy(host_logits, s->logits, (size_t)s->model->cfg.vocab_size * 4, cudaMemcpyDeviceToHost));
    return L2B_OK;
}

extern "C" int32_t l2b_decode_next(l2b_session* s, int32_t token, int32_t pos, float temperature, double uniform, int32_t* next) {
    if (!s || !next) return fail(L2B_ERR_BAD_ARG, "null argument");
    if (!(uniform >= 0.0 && uniform < 1.0)) return fail(L2B_ERR_BAD_ARG, "uniform must lie in [0,1)");
    L2B_TRY(run_one(s, token, pos, temperature, uniform));
    *next = s->h_small[0];
    return L2B_OK;
}

// Feed n prompt tokens at positions pos0 .. pos0+n-1 (teacher-forced; two positions per pass where both are followed by a
// prompt token).  The last position goes through the one-position graph, so its logits are in the session afterwards and
// *next (if given) is their argmax; the caller continues with l2b_decode_next(session, chosen token, pos0 + n, ...).
extern "C" int32_t l2b_prefill(l2b_session* s, const int32_t* tokens, int32_t n, int32_t pos0, int32_t* next) {
    if (!s || !tokens) return fail(L2B_ERR_BAD_ARG, "null argument");
    const l2b_config& c = s->model->cfg;
    if (n < 1 || pos0 < 0 || (int64_t)pos0 + n > c.seq_len) return fail(L2B_ERR_BAD_ARG, "positions pos0 .. pos0+n-1 must lie in 0..seq_len-1");
    for (int i = 0; i < n; ++i)
        if (tokens[i] < 0 || tokens[i] >= c.vocab_size) return fail(L2B_ERR_BAD_ARG, "prompt token id out of range");
    if (!s->graph) return fail(L2B_ERR_STATE, "tensor-parallel session: call l2b_session_tp_connect first");
    CU(cudaSetDevice(s->model->device));
    Control& h = *s->h_ctl;
    memset(&h, 0, sizeof(h));
    h.token = tokens[0];
    h.pos = pos0;
    h.n_prompt = pos0 + n;  // positions are absolute: prompt[pos] is the token fed at position pos
    CU(cudaEventRecord(s->ev0, s->stream));
    CU(cudaMemcpyAsync(s->prompt + pos0, tokens, (size_t)n * 4, cudaMemcpyHostToDevice, s->stream));
    CU(cudaMemcpyAsync(s->ctl, s->h_ctl, sizeof(Control), cudaMemcpyHostToDevice, s->stream));
    const int end = pos0 + n;
    s->last_launches = 0;
    L2B_TRY(enqueue_forced_positions(s, pos0, end - 1, tokens));  // every position but the last is followed by a prompt token
    CU(cudaGraphLaunch(s->graph, s->stream));                     // the last one: its logits are wanted
    s->last_launches += s->kernels_per_token;
    CU(cudaMemcpyAsync(&s->h_small[0], s->next_token, 4, cudaMemcpyDeviceToHost, s->stream));
    CU(cudaMemcpyAsync(&s->h_small[1], s->status, 4, cudaMemcpyDeviceToHost, s->stream));
    CU(cudaEventRecord(s->ev1, s->stream));
    CU(cudaStreamSynchronize(s->stream));
    CU(cudaEventElapsedTime(&s->last_ms, s->ev0, s->ev1));
    if (next) *next = s->h_small[0];
    return check_status_word(s);
}

extern "C" int32_t l2b_session_prefill_gemm(l2b_session* s, int32_t* min_tokens) {
    if (!s || !min_tokens) return fail(L2B_ERR_BAD_ARG, "null argument");
    CU(cudaSetDevice(s->model->device));
    *min_tokens = prefill_gemm_eligible(s) ? PF_MIN_TOK : 0;
    return L2B_OK;
}

extern "C" int32_t l2b_session_prefill_pairs(l2b_session* s, int32_t* enabled) {
    if (!s || !enabled) return fail(L2B_ERR_BAD_ARG, "null argument");
    *enabled = s->graph2 ? 1 : 0;
    return L2B_OK;
}

extern "C" int32_t l2b_generate(l2b_session* s, const int32_t* prompt, int32_t n_prompt, int32_t n_positions, float temperature, uint64_t seed,
                                int32_t* out_tokens, float* device_ms) {
    if (!s || !prompt || !out_tokens) return fail(L2B_ERR_BAD_ARG, "null argument");
    const l2b_config& c = s->model->cfg;
    if (n_prompt < 1 || n_prompt > c.seq_len) return fail(L2B_ERR_BAD_ARG, "prompt length must be in 1..seq_len");
    if (n_positions < 1 || n_positions > c.seq_len) return fail(L2B_ERR_BAD_ARG, "n_positions must be in 1..seq_len");
    if (temperature < 0.f) return fail(L2B_ERR_BAD_ARG, "temperature must be >= 0");
    for (int i = 0; i < n_prompt; ++i)
        if (prompt[i] < 0 || prompt[i] >= c.vocab_size) return fail(L2B_ERR_BAD_ARG, "prompt token id out of range");
    if (!s->graph) return fail(L2B_ERR_STATE, "tensor-parallel session: call l2b_session_tp_connect first");
    CU(cudaSetDevice(s->model->device));
    Control& h = *s->h_ctl;
    memset(&h, 0, sizeof(h));
    h.token = prompt[0];
    h.pos = 0;
    h.n_prompt = n_prompt;
    h.temperature = temperature;
    h.use_seed = 1;
    h.seed = seed;
    CU(cudaMemcpyAsync(s->prompt, prompt, (size_t)n_prompt * 4, cudaMemcpyHostToDevice, s->stream));
    CU(cudaMemcpyAsync(s->ctl, s->h_ctl, sizeof(Control), cudaMemcpyHostToDevice, s->stream));
    CU(cudaEventRecord(s->ev0, s->stream));  // the timed region is the token loop itself: inputs are resident
    // Positions p and p + 1 go through one two-position pass when both are followed by a prompt token (their next
    // tokens are forced, so neither needs logits); everything else takes the one-position graph.
    bool mid = false;
    const int forced_end = std::min(n_prompt - 1, n_positions);  // positions below this are followed by a prompt token
    s->last_launches = 0;
    L2B_TRY(enqueue_forced_positions(s, 0, forced_end, prompt));
    s->last_launches += (long long)(n_positions - forced_end) * s->kernels_per_token;
    for (int i = forced_end; i < n_positions; ++i) {
        if (i >= n_prompt && !mid) {  // the first position that is fed a generated token
            CU(cudaEventRecord(s->ev_mid, s->stream));
            mid = true;
        }
        CU(cudaGraphLaunch(s->graph, s->stream));
    }
    if (!mid) CU(cudaEventRecord(s->ev_mid, s->stream));
    CU(cudaEventRecord(s->ev1, s->stream));
    CU(cudaMemcpyAsync(out_tokens, s->out_tokens, (size_t)n_positions * 4, cudaMemcpyDeviceToHost, s->stream));
    CU(cudaMemcpyAsync(&s->h_small[1], s->status, 4, cudaMemcpyDeviceToHost, s->stream));
    CU(cudaStreamSynchronize(s->stream));
    CU(cudaEventElapsedTime(&s->last_ms, s->ev0, s->ev1));
    CU(cudaEventElapsedTime(&s->last_prompt_ms, s->ev0, s->ev_mid));
    CU(cudaEventElapsedTime(&s->last_decode_ms, s->ev_mid, s->ev1));
    if (device_ms) *device_ms = s->last_ms;
    return check_status_word(s);
}

extern "C" int32_t l2b_session_logits(l2b_session* s, float* host_logits) {
    if (!s || !host_logits) return fail(L2B_ERR_BAD_ARG, "null argument");
    CU(cudaSetDevice(s->model->device));
    CU(cudaStreamSynchronize(s->stream));
    CU(cudaMemcpy(host_logits, s->logits, (size_t)s->model->cfg.vocab_size * 4, cudaMemcpyDeviceToHost));
    return L2B_OK;
}

extern "C" int32_t l2b_session_read(l2b_session* s, int32_t which, float* host_out, int64_t cap, int64_t* n) {
    if (!s || !host_out) return fail(L2B_ERR_BAD_ARG, "null argument");
    const l2b_config& c = s->model->cfg;
    const float* src = nullptr;
    int64_t len = 0;
    switch (which) {
        case 0: src = s->x; len = c.dim; break;
        case 2: src = s->q; len = c.dim; break;
        case 5: src = s->hb; len = c.hidden_dim; break;
        case 6: src = s->logits; len = c.vocab_size; break;
        default: return fail(L2B_ERR_BAD_ARG, "unknown buffer id");
    }
    CU(cudaSetDevice(s->model->device));
    CU(cudaStreamSynchronize(s->stream));
    CU(cudaMemcpy(host_out, src, (size_t)std::min(cap, len) * 4, cudaMemcpyDeviceToHost));
    if (n) *n = len;
    return L2B_OK;
}

extern "C" int32_t l2b_session_last_device_ms(l2b_session* s, float* ms) {
    if (!s || !ms) return fail(L2B_ERR_BAD_ARG, "null argument");
    *ms = s->last_ms;
    return L2B_OK;
}
extern "C" int32_t l2b_session_last_phase_ms(l2b_session* s, float* prompt_ms, float* decode_ms) {
    if (!s || !prompt_ms || !decode_ms) return fail(L2B_ERR_BAD_ARG, "null argument");
    *prompt_ms = s->last_prompt_ms;
    *decode_ms = s->last_decode_ms;
    return L2B_OK;
}
extern "C" int32_t l2b_session_last_launches(l2b_session* s, int64_t* n) {
    if (!s || !n) return fail(L2B_ERR_BAD_ARG, "null argument");
    *n = s->last_launches;
    return L2B_OK;
}
extern "C" int32_t l2b_session_kernels_per_token(l2b_session* s, int32_t* n) {
    if (!s || !n) return fail(L2B_ERR_BAD_ARG, "null argument");
    *n = s->kernels_per_token;
    return L2B_OK;
}

// ---------------------------------------------------------------------------------------------
// batched decode: several independent sequences in lock step (no counterpart in the reference,
// whose `sample` serves one prompt)
// ---------------------------------------------------------------------------------------------
struct l2b_batch {
    l2b_model* model = nullptr;
    int n_seq = 0;
    cudaStream_t stream = nullptr;
    DeviceInfo di;
    GemmBufs B;
    float *kc = nullptr, *vc = nullptr;  // [layer][sequence][kv_head][seq_len][hs]
    float* rope_cs = nullptr;
    float* logits = nullptr;             // [n_seq][vocab]
    int *tokens = nullptr, *pos = nullptr, *next = nullptr, *status = nullptr;
    int* h_io = nullptr;                 // pinned: tokens, positions, next tokens, status
    int gq = 1;
};

static void batch_free(l2b_batch* b) {
    if (!b) return;
    free_gemm_bufs(b->B);
    void* bufs[] = {b->kc, b->vc, b->rope_cs, b->logits, b->tokens, b->pos, b->next, b->status};
    for (void* p : bufs)
        if (p) cudaFree(p);
    if (b->h_io) cudaFreeHost(b->h_io);
    if (b->stream) cudaStreamDestroy(b->stream);
    delete b;
}

extern "C" int32_t l2b_batch_create(l2b_model* m, int32_t n_seq, l2b_batch** out) {
    if (!m || !out) return fail(L2B_ERR_BAD_ARG, "null argument");
    *out = nullptr;
    if (!m->finalized) return fail(L2B_ERR_STATE, "l2b_model_finalize has not been called");
    if (n_seq < 2 || n_seq > PF_MAX_TOK) return fail(L2B_ERR_BAD_ARG, "a batch holds 2 .. " + std::to_string(PF_MAX_TOK) + " sequences");
    CU(cudaSetDevice(m->device));
    L2B_TRY(check_kernel_attrs());
    if (!gemm_layers_supported(m))
        return fail(L2B_ERR_UNSUPPORTED_TYPE, "batched decode needs q4_K / q5_K layer matrices, three activation planes and one GPU");
    const l2b_config& c = m->cfg;
    const int hs = c.dim / c.n_heads;
    l2b_batch* b = new l2b_batch();
    b->model = m;
    b->n_seq = n_seq;
    auto run = [&]() -> int32_t {
        L2B_TRY(query_device(b->di));
        CU(cudaStreamCreateWithFlags(&b->stream, cudaStreamNonBlocking));
        b->gq = choose_gq(c.n_heads, c.n_kv_heads);
        if (!alloc_gemm_bufs(m, b->B, (size_t)n_seq)) return fail(L2B_ERR_OOM, "out of device memory for the batch buffers");
        const size_t cache = kv_layer_elems(m) * c.n_layers * (size_t)n_seq * 4;
        CU(cudaMalloc(&b->kc, cache));
        CU(cudaMalloc(&b->vc, cache));
        CU(cudaMemsetAsync(b->kc, 0, cache, b->stream));
        CU(cudaMemsetAsync(b->vc, 0, cache, b->stream));
        CU(cudaMalloc(&b->logits, (size_t)n_seq * c.vocab_size * 4));
        CU(cudaMalloc(&b->tokens, (size_t)n_seq * 4));
        CU(cudaMalloc(&b->pos, (size_t)n_seq * 4));
        CU(cudaMalloc(&b->next, (size_t)n_seq * 4));
        CU(cudaMalloc(&b->status, 4));
        CU(cudaMemsetAsync(b->status, 0, 4, b->stream));
        CU(cudaMallocHost(&b->h_io, (size_t)(3 * n_seq + 1) * 4));
        std::vector<float> cs;
        rope_table_host(cs, c.seq_len, hs, c.rope_freq_base);
        CU(cudaMalloc(&b->rope_cs, cs.size() * 4));
        CU(cudaMemcpyAsync(b->rope_cs, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice, b->stream));
        CU(cudaStreamSynchronize(b->stream));
        return L2B_OK;
    };
    const int32_t st = run();
    if (st != L2B_OK) {
        batch_free(b);
        return st;
    }
    *out = b;
    return L2B_OK;
}

extern "C" int32_t l2b_batch_destroy(l2b_batch* b) {
    if (!b) return L2B_OK;
    cudaSetDevice(b->model->device);
    if (b->stream) cudaStreamSynchronize(b->stream);
    batch_free(b);
    return L2B_OK;
}

extern "C" int32_t l2b_batch_reset(l2b_batch* b) {
    if (!b) return fail(L2B_ERR_BAD_ARG, "null batch");
    CU(cudaSetDevice(b->model->device));
    const size_t cache = kv_layer_elems(b->model) * b->model->cfg.n_layers * (size_t)b->n_seq * 4;
    CU(cudaMemsetAsync(b->kc, 0, cache, b->stream));
    CU(cudaMemsetAsync(b->vc, 0, cache, b->stream));
    CU(cudaStreamSynchronize(b->stream));
    return L2B_OK;
}

extern "C" int32_t l2b_batch_decode_next(l2b_batch* b, const int32_t* tokens, const int32_t* positions, int32_t* next_tokens, float* host_logits) {
    if (!b || !tokens || !positions || !next_tokens) return fail(L2B_ERR_BAD_ARG, "null argument");
    const l2b_model* m = b->model;
    const l2b_config& c = m->cfg;
    const int n = b->n_seq;
    for (int i = 0; i < n; ++i) {
        if (tokens[i] < 0 || tokens[i] >= c.vocab_size) return fail(L2B_ERR_BAD_ARG, "token id out of range");
        if (positions[i] < 0 || positions[i] >= c.seq_len) return fail(L2B_ERR_BAD_ARG, "position out of range (seq_len)");
    }
    CU(cudaSetDevice(m->device));
    cudaStream_t st = b->stream;
    memcpy(b->h_io, tokens, (size_t)n * 4);
    memcpy(b->h_io + n, positions, (size_t)n * 4);
    CU(cudaMemcpyAsync(b->tokens, b->h_io, (size_t)n * 4, cudaMemcpyHostToDevice, st));
    CU(cudaMemcpyAsync(b->pos, b->h_io + n, (size_t)n * 4, cudaMemcpyHostToDevice, st));
    embed_rows_kernel<<<dim3(std::max(1, std::min(16, c.dim / 256)), n), 256, 0, st>>>(m->tok_emb.type, m->tok_emb.data, m->tok_emb.d6, b->tokens, c.dim,
                                                                                      c.vocab_size, b->B.x);
    CU(cudaGetLastError());
    const size_t kvl = kv_layer_elems(m);
    L2B_TRY(enqueue_layers_gemm(m, b->B, n, b->kc, b->vc, kvl * (size_t)n, 0, b->pos, kvl, b->rope_cs, b->gq, b->status, st));
    // final rmsnorm + classifier (src/inference.jl:309-312) for every sequence, then argmax (:360)
    if (gemm_supported(m->output)) {
        L2B_TRY(launch_quantise_rows(b->B.x, m->rms_final, b->B.act, c.dim, c.dim, n, st));
        L2B_TRY(launch_kq_gemm(m->output, b->B.act, n, b->logits, c.vocab_size, nullptr, b->status, st));
    } else {  // a q6_K classifier: one pass of the matrix-vector kernel per sequence
        for (int i = 0; i < n; ++i) {
            MvLaunch L;
            memset(&L.p, 0, sizeof(L.p));
            L.planes = m->planes;
            L.p.n_in = c.dim;
            L.p.seg[L.p.nseg++] = make_segment(m->output, PAIR_ADJACENT, EPI_STORE, b->logits + (size_t)i * c.vocab_size, 0);
            L.kb = m->output.kb;
            L.p.pro = PRO_RMSNORM;
            L.p.gain = m->rms_final;
            L.p.x_in = b->B.x + (size_t)i * c.dim;
            L.p.status = b->status;
            L2B_TRY(plan_matvec(L, b->di));
            CU(launch_matvec(L, st, false));
        }
    }
    argmax_rows_kernel<<<n, 1024, 0, st>>>(b->logits, c.vocab_size, b->next, b->status);
    CU(cudaGetLastError());
    CU(cudaMemcpyAsync(b->h_io + 2 * n, b->next, (size_t)n * 4, cudaMemcpyDeviceToHost, st));
    CU(cudaMemcpyAsync(b->h_io + 3 * n, b->status, 4, cudaMemcpyDeviceToHost, st));
    if (host_logits) CU(cudaMemcpyAsync(host_logits, b->logits, (size_t)n * c.vocab_size * 4, cudaMemcpyDeviceToHost, st));
    CU(cudaStreamSynchronize(st));
    const int dev_status = b->h_io[3 * n];
    if (dev_status != DEV_OK) {
        cudaMemsetAsync(b->status, 0, 4, st);
        if (dev_status == DEV_ERR_BAD_INDEX) return fail(L2B_ERR_CUDA, "no valid token could be chosen (the logits are not finite); token 0 was substituted");
        return fail(dev_status == DEV_ERR_TMA_TIMEOUT ? L2B_ERR_TIMEOUT : L2B_ERR_CUDA, "kernel reported device status " + std::to_string(dev_status));
    }
    memcpy(next_tokens, b->h_io + 2 * n, (size_t)n * 4);
    return L2B_OK;
}

// ---------------------------------------------------------------------------------------------
// isolated operators
// ---------------------------------------------------------------------------------------------
struct DevBuf {
    void* p = nullptr;
    ~DevBuf() {
        if (p) cudaFree(p);
    }
    template <typename T>
    T* as() { return (T*)p; }
};
static int32_t dev_alloc(DevBuf& b, size_t bytes) {
    CU(cudaMalloc(&b.p, bytes ? bytes : 16));
    return L2B_OK;
}
static int32_t dev_upload(DevBuf& b, const void* host, size_t bytes) {
    L2B_TRY(dev_alloc(b, bytes));
    CU(cudaMemcpy(b.p, host, bytes, cudaMemcpyHostToDevice));
    return L2B_OK;
}

extern "C" int32_t l2b_dequantize(int32_t type, const void* host_blocks, int64_t n, float* host_out) {
    if (!host_blocks || !host_out || n < 0) return fail(L2B_ERR_BAD_ARG, "null argument");
    if (!type_supported(type)) return fail(L2B_ERR_UNSUPPORTED_TYPE, "tensor type " + std::to_string(type) + " not implemented");
    L2B_TRY(require_device());
    if (n == 0) return L2B_OK;
    if (type == T_F32) {  // dequantize!(y, x::Vector{Float32}) is a copy; it still goes through the device
        DevBuf b;
        L2B_TRY(dev_upload(b, host_blocks, (size_t)n * 4));
        CU(cudaMemcpy(host_out, b.p, (size_t)n * 4, cudaMemcpyDeviceToHost));
        return L2B_OK;
    }
    if (n % QK_K != 0) return fail(L2B_ERR_BAD_ARG, "element count must be a multiple of 256");
    DevMatrix m;
    int32_t st = upload_matrix(m, type, host_blocks, n, 1, 0, false);
    if (st != L2B_OK) return st;
    DevBuf out;
    st = dev_alloc(out, (size_t)n * 4);
    if (st == L2B_OK) {
        const int grid = (int)std::min<int64_t>(4096, (n + 255) / 256);
        dequantize_kernel<<<grid, 256>>>(type, m.data, m.d6, n, out.as<float>());
        cudaError_t e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaMemcpy(host_out, out.p, (size_t)n * 4, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) st = fail(L2B_ERR_CUDA, cudaGetErrorString(e));
    }
    free_matrix(m);
    return st;
}

// Run the fused kernel's prologue on one block and export what it built.
static int32_t run_export(MvParams& p, bool kq, int planes, int8_t* q_out, float* d_out, float* sums_out, float* f_out) {
    L2B_TRY(check_kernel_attrs());
    const int warps = 8;
    const size_t smem = mv_smem_layout(p.n_in, planes, kq, 0, 0).total;
    p.consumers = warps;
    p.turns = (p.n_in / 8 + 32 * warps - 1) / (32 * warps);
    int optin = 0, dev = 0;
    CU(cudaGetDevice(&dev));
    CU(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    if ((long)smem > optin - 1024) return fail(L2B_ERR_BAD_ARG, "vector too long for one block's shared memory");
    if (!kq) export_activation_kernel<false, 1><<<1, warps * 32, smem>>>(p, q_out, d_out, sums_out, f_out);
    else if (planes == 1) export_activation_kernel<true, 1><<<1, warps * 32, smem>>>(p, q_out, d_out, sums_out, f_out);
    else if (planes == 2) export_activation_kernel<true, 2><<<1, warps * 32, smem>>>(p, q_out, d_out, sums_out, f_out);
    else export_activation_kernel<true, 3><<<1, warps * 32, smem>>>(p, q_out, d_out, sums_out, f_out);
    CU(cudaGetLastError());
    CU(cudaDeviceSynchronize());
    return L2B_OK;
}

static int32_t quantize_planes(const float* host_x, const float* host_w, int64_t n, int32_t planes, int8_t* host_q, float* host_d, float* host_sums) {
    if (!host_x || !host_q || !host_d || !host_sums) return fail(L2B_ERR_BAD_ARG, "null argument");
    if (n <= 0 || n % QK_K != 0) return fail(L2B_ERR_BAD_ARG, "n must be a positive multiple of 256");
    if (planes < 1 || planes > 3) return fail(L2B_ERR_BAD_ARG, "planes must be 1..3");
    L2B_TRY(require_device());
    DevBuf x, w, q, d, sums;
    L2B_TRY(dev_upload(x, host_x, (size_t)n * 4));
    if (host_w) L2B_TRY(dev_upload(w, host_w, (size_t)n * 4));
    L2B_TRY(dev_alloc(q, (size_t)planes * n));
    L2B_TRY(dev_alloc(d, (size_t)planes * (n / QK_K) * 4));
    L2B_TRY(dev_alloc(sums, (size_t)(n / 16) * 4));
    MvParams p;
    memset(&p, 0, sizeof(p));
    p.n_in = (int)n;
    p.pro = host_w ? PRO_RMSNORM : PRO_COPY;
    p.x_in = x.as<float>();
    p.gain = host_w ? w.as<float>() : nullptr;
    L2B_TRY(run_export(p, true, planes, q.as<int8_t>(), d.as<float>(), sums.as<float>(), nullptr));
    CU(cudaMemcpy(host_q, q.p, (size_t)planes * n, cudaMemcpyDeviceToHost));
    CU(cudaMemcpy(host_d, d.p, (size_t)planes * (n / QK_K) * 4, cudaMemcpyDeviceToHost));
    CU(cudaMemcpy(host_sums, sums.p, (size_t)(n / 16) * 4, cudaMemcpyDeviceToHost));
    return L2B_OK;
}

extern "C" int32_t l2b_quantize_q8k(const float* host_x, int64_t n, int32_t planes, int8_t* host_q, float* host_d, float* host_sums) {
    return quantize_planes(host_x, nullptr, n, planes, host_q, host_d, host_sums);
}

extern "C" int32_t l2b_rmsnorm_quantize_q8k(const float* host_x, const float* host_w, int64_t n, int32_t planes, int8_t* host_q, float* host_d,
                                            float* host_sums) {
    if (!host_w) return fail(L2B_ERR_BAD_ARG, "null argument");
    return quantize_planes(host_x, host_w, n, planes, host_q, host_d, host_sums);
}

extern "C" int32_t l2b_rmsnorm(float* host_o, const float* host_x, const float* host_w, int64_t n) {
    if (!host_o || !host_x || !host_w) return fail(L2B_ERR_BAD_ARG, "null argument");
    if (n <= 0 || n % 8 != 0) return fail(L2B_ERR_BAD_ARG, "n must be a positive multiple of 8");
    L2B_TRY(require_device());
    DevBuf x, w, o;
    L2B_TRY(dev_upload(x, host_x, (size_t)n * 4));
    L2B_TRY(dev_upload(w, host_w, (size_t)n * 4));
    L2B_TRY(dev_alloc(o, (size_t)n * 4));
    MvParams p;
    memset(&p, 0, sizeof(p));
    p.n_in = (int)n;
    p.pro = PRO_RMSNORM;
    p.x_in = x.as<float>();
    p.gain = w.as<float>();
    L2B_TRY(run_export(p, false, 1, nullptr, nullptr, nullptr, o.as<float>()));
    CU(cudaMemcpy(host_o, o.p, (size_t)n * 4, cudaMemcpyDeviceToHost));
    return L2B_OK;
}

extern "C" int32_t l2b_rope(float* host_x, int32_t hs, int32_t n_heads, int32_t pos, float base, int32_t neox) {
    if (!host_x) return fail(L2B_ERR_BAD_ARG, "null argument");
    if (hs <= 0 || hs % 2 != 0 || n_heads <= 0 || pos < 0) return fail(L2B_ERR_BAD_ARG, "bad head size / head count / position");
    L2B_TRY(require_device());
    std::vector<float> cs;
    rope_table_host(cs, pos + 1, hs, base);
    DevBuf x, y, table;
    const size_t n = (size_t)hs * n_heads;
    L2B_TRY(dev_upload(x, host_x, n * 4));
    L2B_TRY(dev_alloc(y, n * 4));
    L2B_TRY(dev_upload(table, cs.data(), cs.size() * 4));
    // the token path's own epilogue (EPI_ROPE_Q of the q projection) on the given vector
    MvParams p;
    memset(&p, 0, sizeof(p));
    p.nseg = 1;
    p.seg[0].npairs = (int)(n / 2);
    p.seg[0].pair_mode = neox ? PAIR_NEOX : PAIR_ADJACENT;
    p.seg[0].epi = EPI_ROPE_Q;
    p.seg[0].out = y.as<float>();
    p.seg[0].head_size = hs;
    p.neox_magic = (unsigned)((0x100000000ull + hs / 2 - 1) / (hs / 2));
    p.rope_cs = table.as<float>();
    p.seq_len = pos + 1;
    epilogue_probe_kernel<<<(int)std::min<size_t>(1024, (n / 2 + 255) / 256), 256>>>(p, x.as<float>(), nullptr, pos);
    CU(cudaGetLastError());
    CU(cudaMemcpy(host_x, y.p, n * 4, cudaMemcpyDeviceToHost));
    return L2B_OK;
}

extern "C" int32_t l2b_attention(float* host_out, const float* host_q, const float* host_k, const float* host_v, int32_t n_pos, int32_t n_heads,
                                 int32_t n_kv, int32_t hs) {
    if (!host_out || !host_q || !host_k || !host_v) return fail(L2B_ERR_BAD_ARG, "null argument");
    if (n_pos <= 0 || n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || hs % 8 != 0 || hs > 128 || hs <= 0)
        return fail(L2B_ERR_BAD_ARG, "bad attention shape");
    L2B_TRY(require_device());
    // position-major input -> cache layout [kv][pos][hs]
    std::vector<float> kc((size_t)n_kv * n_pos * hs), vc(kc.size());
    for (int t = 0; t < n_pos; ++t)
        for (int h = 0; h < n_kv; ++h) {
            memcpy(&kc[((size_t)h * n_pos + t) * hs], host_k + ((size_t)t * n_kv + h) * hs, (size_t)hs * 4);
            memcpy(&vc[((size_t)h * n_pos + t) * hs], host_v + ((size_t)t * n_kv + h) * hs, (size_t)hs * 4);
        }
    const int gq = choose_gq(n_heads, n_kv);
    const int nsplit = decode_splits(n_pos);
    DevBuf q, k, v, pm, pl, pa, out, tickets;
    L2B_TRY(dev_upload(q, host_q, (size_t)n_heads * hs * 4));
    L2B_TRY(dev_upload(k, kc.data(), kc.size() * 4));
    L2B_TRY(dev_upload(v, vc.data(), vc.size() * 4));
    L2B_TRY(dev_alloc(pm, (size_t)n_heads * nsplit * 4));
    L2B_TRY(dev_alloc(pl, (size_t)n_heads * nsplit * 4));
    L2B_TRY(dev_alloc(pa, (size_t)n_heads * nsplit * hs * 4));
    L2B_TRY(dev_alloc(out, (size_t)n_heads * hs * 4));
    L2B_TRY(dev_alloc(tickets, (size_t)n_heads * 4));
    CU(cudaMemset(tickets.p, 0, (size_t)n_heads * 4));
    AttnParams a;
    memset(&a, 0, sizeof(a));
    a.q = q.as<float>(); a.kc = k.as<float>(); a.vc = v.as<float>(); a.out = out.as<float>();
    a.part_m = pm.as<float>(); a.part_l = pl.as<float>(); a.part_acc = pa.as<float>(); a.tickets = tickets.as<int>();
    a.n_heads = n_heads; a.n_kv = n_kv; a.hs = hs; a.seq_len = n_pos; a.nsplit = nsplit; a.npos_override = n_pos;
    CU(launch_attention(a, gq, 0, false));
    CU(cudaDeviceSynchronize());
    CU(cudaMemcpy(host_out, out.p, (size_t)n_heads * hs * 4, cudaMemcpyDeviceToHost));
    return L2B_OK;
}

extern "C" int32_t l2b_swiglu(float* host_hb, const float* host_hb2, int64_t n) {
    if (!host_hb || !host_hb2 || n < 0 || n > 0x7fffffff) return fail(L2B_ERR_BAD_ARG, "null argument or bad length");
    L2B_TRY(require_device());
    if (n == 0) return L2B_OK;
    DevBuf a, b, o;
    L2B_TRY(dev_upload(a, host_hb, (size_t)n * 4));
    L2B_TRY(dev_upload(b, host_hb2, (size_t)n * 4));
    L2B_TRY(dev_alloc(o, (size_t)n * 4));
    // the token path's own epilogue (EPI_SWIGLU of the gate / up projections) on the given vectors
    MvParams p;
    memset(&p, 0, sizeof(p));
    p.nseg = 1;
    p.seg[0].npairs = (int)n;
    p.seg[0].pair_mode = PAIR_DUAL;
    p.seg[0].epi = EPI_SWIGLU;
    p.seg[0].out = o.as<float>();
    epilogue_probe_kernel<<<(int)std::min<int64_t>(1024, (n + 255) / 256), 256>>>(p, a.as<float>(), b.as<float>(), 0);
    CU(cudaGetLastError());
    CU(cudaMemcpy(host_hb, o.p, (size_t)n * 4, cudaMemcpyDeviceToHost));
    return L2B_OK;
}

extern "C" int32_t l2b_argmax(const float* host_logits, int64_t n, int32_t* index) {
    if (!host_logits || !index || n <= 0 || n > 0x7fffffff) return fail(L2B_ERR_BAD_ARG, "bad argument");
    L2B_TRY(require_device());
    DevBuf x, v, i;
    L2B_TRY(dev_upload(x, host_logits, (size_t)n * 4));
    L2B_TRY(dev_alloc(v, 4));
    L2B_TRY(dev_alloc(i, 4));
    argmax_kernel<<<1, FIN_THREADS>>>(x.as<float>(), (int)n, v.as<float>(), i.as<int>());
    CU(cudaGetLastError());
    CU(cudaMemcpy(index, i.p, 4, cudaMemcpyDeviceToHost));
    return L2B_OK;
}

extern "C" int32_t l2b_sample_temperature(const float* host_logits, int64_t n, float temperature, double uniform, int32_t* index) {
    if (!host_logits || !index || n <= 0 || n > 0x7fffffff) return fail(L2B_ERR_BAD_ARG, "bad argument");
    if (!(temperature > 0.f)) return fail(L2B_ERR_BAD_ARG, "temperature must be > 0");
    if (!(uniform >= 0.0 && uniform < 1.0)) return fail(L2B_ERR_BAD_ARG, "uniform must lie in [0,1)");
    L2B_TRY(require_device());
    DevBuf x, v, i, ctl, nt;
    L2B_TRY(dev_upload(x, host_logits, (size_t)n * 4));
    L2B_TRY(dev_alloc(v, 4));
    L2B_TRY(dev_alloc(i, 4));
    L2B_TRY(dev_alloc(nt, 4));
    argmax_kernel<<<1, FIN_THREADS>>>(x.as<float>(), (int)n, v.as<float>(), i.as<int>());
    CU(cudaGetLastError());
    Control h;
    memset(&h, 0, sizeof(h));
    h.temperature = temperature;
    h.uniform = uniform;
    L2B_TRY(dev_upload(ctl, &h, sizeof(h)));
    FinalizeParams f;
    memset(&f, 0, sizeof(f));
    f.logits = x.as<float>(); f.vocab = (int)n;
    f.amax_val = v.as<float>(); f.amax_idx = i.as<int>(); f.nparts = 1;
    f.ctl = ctl.as<Control>(); f.next_token = nt.as<int>();
    finalize_token_kernel<<<1, FIN_THREADS>>>(f);
    CU(cudaGetLastError());
    CU(cudaMemcpy(index, nt.p, 4, cudaMemcpyDeviceToHost));
    return L2B_OK;
}

// ---------------------------------------------------------------------------------------------
// resident matrices
// ---------------------------------------------------------------------------------------------
#ifdef L2B_MEASURE
static unsigned long long* g_trace = nullptr;  // set only by the L2B_MV_TRACE measurement path
#endif

struct l2b_matrix {
    std::vector<DevMatrix> copies;
    int device = 0;
    DeviceInfo di;
    int* status = nullptr;
    uint8_t* act = nullptr;  // quantised activation columns of l2b_matrix_matmul_device (grown on demand)
    size_t act_bytes = 0;
};

extern "C" int32_t l2b_matrix_create(int32_t type, const void* host_W, int64_t in_dim, int64_t out_dim, int32_t copies, l2b_matrix** out) {
    if (!host_W || !out || copies < 1) return fail(L2B_ERR_BAD_ARG, "bad argument");
    *out = nullptr;
    if (out_dim % 2 != 0) return fail(L2B_ERR_BAD_ARG, "out_dim must be even");
    L2B_TRY(require_device());
    L2B_TRY(check_kernel_attrs());
    l2b_matrix* m = new l2b_matrix();
    cudaGetDevice(&m->device);
    int32_t st = query_device(m->di);
    m->copies.resize(copies);
    for (int i = 0; i < copies && st == L2B_OK; ++i) st = upload_matrix(m->copies[i], type, host_W, in_dim, out_dim, 0);
    if (st == L2B_OK && cudaMalloc(&m->status, 4) != cudaSuccess) st = fail(L2B_ERR_OOM, "cudaMalloc status");
    if (st == L2B_OK) cudaMemset(m->status, 0, 4);
    if (st != L2B_OK) {
        for (auto& c : m->copies) free_matrix(c);
        delete m;
        return st;
    }
    *out = m;
    return L2B_OK;
}

extern "C" int32_t l2b_matrix_destroy(l2b_matrix* m) {
    if (!m) return L2B_OK;
    cudaSetDevice(m->device);
    for (auto& c : m->copies) free_matrix(c);
    if (m->status) cudaFree(m->status);
    if (m->act) cudaFree(m->act);
    delete m;
    return L2B_OK;
}

// y[c] = A' x[c] for ncols columns on device pointers (x: [ncols][in], y: [ncols][out]) through the tensor-core GEMM:
// the columns are quantised once, then every weight tile is unpacked once per 20 columns.
extern "C" int32_t l2b_matrix_matmul_device(l2b_matrix* m, int32_t copy, const float* dev_x, int32_t ncols, float* dev_y, void* stream) {
    if (!m || !dev_x || !dev_y || ncols < 1) return fail(L2B_ERR_BAD_ARG, "bad argument");
    if (copy < 0 || copy >= (int)m->copies.size()) return fail(L2B_ERR_BAD_ARG, "copy index out of range");
    const DevMatrix& w = m->copies[copy];
    if (!gemm_supported(w)) return fail(L2B_ERR_UNSUPPORTED_TYPE, "the tensor-core GEMM takes q4_K and q5_K matrices");
    CU(cudaSetDevice(m->device));
    const size_t need = gemm_act_bytes(w.in, ncols);
    if (need > m->act_bytes) {
        if (m->act) cudaFree(m->act);
        m->act = nullptr;
        m->act_bytes = 0;
        CU(cudaMalloc(&m->act, need));
        m->act_bytes = need;
    }
    L2B_TRY(launch_quantise_rows(dev_x, nullptr, m->act, (int)w.in, (int)w.in, ncols, (cudaStream_t)stream));
    return launch_kq_gemm(w, m->act, ncols, dev_y, (int)w.out, nullptr, m->status, (cudaStream_t)stream);
}

extern "C" int32_t l2b_matrix_matvec_device(l2b_matrix* m, int32_t copy, const float* dev_x, float* dev_y, int32_t planes, void* stream) {
    if (!m || !dev_x || !dev_y) return fail(L2B_ERR_BAD_ARG, "null argument");
    if (copy < 0 || copy >= (int)m->copies.size()) return fail(L2B_ERR_BAD_ARG, "copy index out of range");
    if (planes < 0 || planes > 3) return fail(L2B_ERR_BAD_ARG, "act_planes must be 0..3");
    const DevMatrix& w = m->copies[copy];
    MvLaunch L;
    memset(&L.p, 0, sizeof(L.p));
    L.planes = planes == 0 ? 3 : planes;
    L.p.n_in = (int)w.in;
    L.p.seg[L.p.nseg++] = make_segment(w, PAIR_ADJACENT, EPI_STORE, dev_y, 0);
    L.kb = w.kb;
    L.p.pro = PRO_COPY;
    L.p.x_in = dev_x;
    L.p.status = m->status;
#ifdef L2B_MEASURE
    L.p.trace = g_trace;
#endif
    L2B_TRY(plan_matvec(L, m->di));
    CU(launch_matvec(L, (cudaStream_t)stream, false));
    return L2B_OK;
}

extern "C" int32_t l2b_matrix_matvec(l2b_matrix* m, const float* host_x, int32_t ncols, float* host_y, int32_t planes) {
    if (!m || !host_x || !host_y || ncols < 1) return fail(L2B_ERR_BAD_ARG, "bad argument");
    CU(cudaSetDevice(m->device));
    const DevMatrix& w = m->copies[0];
    DevBuf x, y;
    L2B_TRY(dev_upload(x, host_x, (size_t)ncols * w.in * 4));
    L2B_TRY(dev_alloc(y, (size_t)ncols * w.out * 4));
    // Several columns: one pass of the tensor-core GEMM per 20 columns (every weight is unpacked once for all of them)
    // instead of one matrix-vector pass per column.  L2B_GEMM_MIN_COLS sets the threshold (default 4; 0 switches it off).
    const long gemm_min = env_long("L2B_GEMM_MIN_COLS", 4);
    if (gemm_min > 0 && ncols >= gemm_min && (planes == 0 || planes == 3) && gemm_supported(w)) {
        DevBuf act;
        L2B_TRY(dev_alloc(act, gemm_act_bytes(w.in, ncols)));
        L2B_TRY(launch_quantise_rows(x.as<float>(), nullptr, act.as<uint8_t>(), (int)w.in, (int)w.in, ncols, nullptr));
        L2B_TRY(launch_kq_gemm(w, act.as<uint8_t>(), ncols, y.as<float>(), (int)w.out, nullptr, m->status, nullptr));
    } else {
        for (int c = 0; c < ncols; ++c)
            L2B_TRY(l2b_matrix_matvec_device(m, 0, x.as<float>() + (size_t)c * w.in, y.as<float>() + (size_t)c * w.out, planes, nullptr));
    }
    CU(cudaDeviceSynchronize());
#ifdef L2B_MEASURE
    if (env_long("L2B_MV_TRACE", 0)) {  // measurement aid: per-block timeline of one more launch, printed to stderr
        DevBuf tr;
        const int NT = 16;
        L2B_TRY(dev_alloc(tr, (size_t)m->di.sms * NT * 8));
        CU(cudaMemset(tr.p, 0, (size_t)m->di.sms * NT * 8));
        g_trace = tr.as<unsigned long long>();
        for (int rep = 0; rep < 3; ++rep) L2B_TRY(l2b_matrix_matvec_device(m, 0, x.as<float>(), y.as<float>(), planes, nullptr));
        g_trace = nullptr;
        CU(cudaDeviceSynchronize());
        std::vector<unsigned long long> h((size_t)m->di.sms * NT);
        CU(cudaMemcpy(h.data(), tr.p, h.size() * 8, cudaMemcpyDeviceToHost));
        unsigned long long t0 = ~0ull;
        for (int b = 0; b < m->di.sms; ++b) t0 = std::min(t0, h[b * NT]);
        double mx[NT] = {0}, av[NT] = {0};
        for (int b = 0; b < m->di.sms; ++b)
            for (int i = 0; i < 14; ++i) {
                const double v = h[b * NT + i] ? (double)(h[b * NT + i] - t0) : 0.0;
                mx[i] = std::max(mx[i], v);
                av[i] += v / m->di.sms;
            }
        fprintf(stderr, "[l2b trace] ns since first block start (avg/max): start %.0f/%.0f barriers-ready %.0f issued %.0f/%.0f waited %.0f/%.0f act %.0f/%.0f end %.0f/%.0f | tiles/block %llu\n",
                av[0], mx[0], av[7], av[1], mx[1], av[2], mx[2], av[3], mx[3], av[6], mx[6], h[14]);
    }
#endif
    int hst = 0;
    CU(cudaMemcpy(&hst, m->status, 4, cudaMemcpyDeviceToHost));
    if (hst != DEV_OK) {
        cudaMemset(m->status, 0, 4);
        return fail(hst == DEV_ERR_TMA_TIMEOUT ? L2B_ERR_TIMEOUT : L2B_ERR_CUDA, "kernel reported device status " + std::to_string(hst));
    }
    CU(cudaMemcpy(host_y, y.p, (size_t)ncols * w.out * 4, cudaMemcpyDeviceToHost));
    return L2B_OK;
}

extern "C" int32_t l2b_matvec(int32_t type, const void* host_W, int64_t in_dim, int64_t out_dim, const float* host_x, int32_t ncols, float* host_y,
                              int32_t planes) {
    l2b_matrix* m = nullptr;
    L2B_TRY(l2b_matrix_create(type, host_W, in_dim, out_dim, 1, &m));
    int32_t st = l2b_matrix_matvec(m, host_x, ncols, host_y, planes);
    l2b_matrix_destroy(m);
    return st;
}

// ---------------------------------------------------------------------------------------------
// Attention on device pointers that allocates nothing
// ---------------------------------------------------------------------------------------------
// For contexts of more than 256 positions the decode attention kernel needs scratch memory: one partial result per
// cluster of blocks and the tickets that elect the merging cluster.  l2b_attention allocates that scratch per call; this entry point keeps it in one
// file-scope device array of fixed size instead, so the call makes no device, pinned or managed allocation and
// frees nothing.  Consequences, all of them the caller's to respect:
//   * the first call on each device looks the array's address up (cudaGetSymbolAddress) and must therefore be
//     made outside any stream capture; later calls on that device reuse the address;
//   * the array is shared by every call on the device and keeps what the last call left in it; the tickets,
//     which must be zero when the kernel starts, are cleared on the caller's stream before every launch;
//   * two calls whose execution overlaps (different streams, or two host threads) race on the array: callers
//     serialise their calls per device;
//   * shapes whose scratch exceeds the array are rejected with L2B_ERR_BAD_ARG.
namespace {

constexpr int NA_MAX_HEADS = 128;   // query heads
constexpr int NA_MAX_HS = 128;      // head size
constexpr int NA_MAX_CLUSTERS = 4;  // clusters per head group (decode_splits): one scratch row each
constexpr int NA_MAX_DEVICES = 64;
constexpr size_t NA_ACC_FLOATS = (size_t)NA_MAX_HEADS * NA_MAX_CLUSTERS * NA_MAX_HS;  // 65536 floats = 256 KiB
constexpr size_t NA_ML_FLOATS = (size_t)NA_MAX_HEADS * NA_MAX_CLUSTERS;               // 512 floats each for max and sum
constexpr size_t NA_SCRATCH_FLOATS = NA_ACC_FLOATS + 2 * NA_ML_FLOATS + NA_MAX_HEADS;  // + tickets (int32)

// 256 KiB + 4.5 KiB of scratch per device, inside the module's global memory (no allocation at run time).
static __device__ __align__(256) float g_attn_static_scratch[NA_SCRATCH_FLOATS];

std::mutex g_na_mutex;
float* g_na_scratch_addr[NA_MAX_DEVICES] = {nullptr};

template <int GQ>
__global__ void __launch_bounds__(ATTN_DW * 32) attention_static_scratch_kernel(const __grid_constant__ AttnParams p) {
    attention_decode_body<GQ, false>(p);  // the arithmetic of l2b_attention, in the same order
}

}  // namespace

extern "C" int32_t l2b_attention_device_noalloc(float* dev_out, const float* dev_q, const float* dev_kcache, const float* dev_vcache,
                                                int32_t n_pos, int32_t seq_len, int32_t n_heads, int32_t n_kv, int32_t hs,
                                                void* stream) {
    if (!dev_out || !dev_q || !dev_kcache || !dev_vcache) return fail(L2B_ERR_BAD_ARG, "null argument");
    if (n_pos <= 0 || seq_len < n_pos || n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || hs % 8 != 0 || hs <= 0)
        return fail(L2B_ERR_BAD_ARG, "bad attention shape");
    if (n_heads > NA_MAX_HEADS || hs > NA_MAX_HS)
        return fail(L2B_ERR_BAD_ARG, "l2b_attention_device_noalloc: at most 128 heads of at most 128 values fit the static scratch array");
    L2B_TRY(require_device());
    int dev = 0;
    CU(cudaGetDevice(&dev));
    if (dev < 0 || dev >= NA_MAX_DEVICES) return fail(L2B_ERR_BAD_ARG, "l2b_attention_device_noalloc: device ordinal beyond 63");
    float* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_na_mutex);
        if (!g_na_scratch_addr[dev]) {
            float* ptr = nullptr;
            CU(cudaGetSymbolAddress((void**)&ptr, g_attn_static_scratch));
            g_na_scratch_addr[dev] = ptr;
        }
        scratch = g_na_scratch_addr[dev];
    }
    const int gq = choose_gq(n_heads, n_kv);
    // the same split rule as l2b_attention, so that both entry points add in the same order
    const int nsplit = decode_splits(n_pos);
    if ((size_t)n_heads * (nsplit / ATTN_CL) * hs > NA_ACC_FLOATS || (size_t)n_heads * (nsplit / ATTN_CL) > NA_ML_FLOATS)
        return fail(L2B_ERR_BAD_ARG, "l2b_attention_device_noalloc: shape exceeds the static scratch array");
    cudaStream_t st = (cudaStream_t)stream;
    AttnParams a;
    memset(&a, 0, sizeof(a));
    a.q = dev_q; a.kc = dev_kcache; a.vc = dev_vcache; a.out = dev_out;
    a.part_acc = scratch;
    a.part_m = scratch + NA_ACC_FLOATS;
    a.part_l = scratch + NA_ACC_FLOATS + NA_ML_FLOATS;
    a.tickets = reinterpret_cast<int*>(scratch + NA_ACC_FLOATS + 2 * NA_ML_FLOATS);
    a.n_heads = n_heads; a.n_kv = n_kv; a.hs = hs; a.seq_len = seq_len; a.nsplit = nsplit; a.npos_override = n_pos;
    // the array keeps the last call's contents: the tickets must be zero when the kernel starts
    CU(cudaMemsetAsync(a.tickets, 0, (size_t)NA_MAX_HEADS * sizeof(int), st));
    const dim3 grid((n_heads / gq) * nsplit), block(ATTN_DW * 32);
    switch (gq) {
        case 8: CU(launch_kernel(attention_static_scratch_kernel<8>, grid, block, 0, st, false, a, ATTN_CL)); break;
        case 4: CU(launch_kernel(attention_static_scratch_kernel<4>, grid, block, 0, st, false, a, ATTN_CL)); break;
        case 2: CU(launch_kernel(attention_static_scratch_kernel<2>, grid, block, 0, st, false, a, ATTN_CL)); break;
        default: CU(launch_kernel(attention_static_scratch_kernel<1>, grid, block, 0, st, false, a, ATTN_CL)); break;
    }
    CU(cudaGetLastError());
    return L2B_OK;
}
