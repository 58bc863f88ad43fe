# Llama2B200.jl -- the binding a Llama2.jl maintainer adds to run the per-token decode path on a B200.
#
# It leaves the public API of the package alone (load_gguf_model / load_karpathy_model / LanguageModel /
# sample, src/Llama2.jl:12-14) and replaces three internals with `ccall`s into libllama2_b200.so
# (include/llama2_b200.h):
#
#   matmul!(y, A, x)                 src/matmul.jl:3-23        -> l2b_matvec
#   transformer!(token, pos, ...)    src/inference.jl:222-315  -> l2b_forward
#   the loop body of sample          src/inference.jl:349-385  -> l2b_decode_next (one call per position)
#
# Token ids and positions are 1-based in Julia and 0-based at the C ABI: the shim subtracts 1.
# Host arrays are borrowed for the duration of a call only, so mmap'ed tensors (load_gguf.jl:160-185) upload
# straight from the page cache; every call that passes a pointer is wrapped in GC.@preserve.
#
# This file cannot be executed where it was written (no Julia there); tests/ exercise the same entry points
# through Python ctypes, call for call.
module Llama2B200

using ..Llama2: ModelConfig, TransformerWeights, TransformerLayerWeights, LanguageModel, RunState,
                block_q4_K, block_q5_K, block_q6_K, QK_K, encode
import ..Llama2: matmul!, transformer!, sample

const LIB = get(ENV, "LLAMA2_B200_LIB", "libllama2_b200.so")

const L2B_TYPE_F32, L2B_TYPE_Q4_K, L2B_TYPE_Q5_K, L2B_TYPE_Q6_K = Int32(0), Int32(12), Int32(13), Int32(14)
@enum Role::Int32 TOKEN_EMBEDDING=0 RMS_ATT WQ WK WV WO RMS_FFN W1 W2 W3 RMS_FINAL OUTPUT

# l2b_config: ModelConfig field for field, then library options (include/llama2_b200.h)
struct L2BConfig
    dim::Int32; hidden_dim::Int32; n_layers::Int32; n_heads::Int32; n_kv_heads::Int32; vocab_size::Int32; seq_len::Int32
    rope_freq_base::Float32; rope_is_neox::Int32
    act_planes::Int32; device::Int32; tp_size::Int32; tp_rank::Int32
    reserved::NTuple{7,Int32}
end
L2BConfig(c::ModelConfig; act_planes=0, device=-1) = L2BConfig(c.dim, c.hidden_dim, c.n_layers, c.n_heads, c.n_kv_heads, c.vocab_size,
    c.seq_len, c.rope_freq_base, c.rope_is_neox, act_planes, device, 1, 0, ntuple(_ -> Int32(0), 7))

function check(status::Int32)
    status == 0 && return nothing
    error("llama2_b200: " * unsafe_string(ccall((:l2b_last_error_string, LIB), Cstring, ())))
end

ggml_type(::AbstractMatrix{Float32}) = L2B_TYPE_F32
ggml_type(::AbstractMatrix{block_q4_K}) = L2B_TYPE_Q4_K
ggml_type(::AbstractMatrix{block_q5_K}) = L2B_TYPE_Q5_K
ggml_type(::AbstractMatrix{block_q6_K}) = L2B_TYPE_Q6_K
in_dim(A::AbstractMatrix{Float32}) = size(A, 1)
in_dim(A::AbstractMatrix) = size(A, 1) * QK_K          # (in/256, out) super-blocks

# ---- matmul! -------------------------------------------------------------------------------------
# Column views of one fused tensor (phi3, load_gguf.jl:264-276) are contiguous, so `pointer(A)` is enough.
function matmul!(y::AbstractVector{Float32}, A::AbstractMatrix, x::AbstractVector{Float32})
    GC.@preserve y A x begin
        check(ccall((:l2b_matvec, LIB), Int32,
                    (Int32, Ptr{Cvoid}, Int64, Int64, Ptr{Float32}, Int32, Ptr{Float32}, Int32),
                    ggml_type(A), pointer(A), in_dim(A), size(A, 2), pointer(x), 1, pointer(y), 0))
    end
    return nothing
end

# ---- model / session handles -------------------------------------------------------------------
mutable struct DeviceModel
    model::Ptr{Cvoid}
    session::Ptr{Cvoid}
end

function upload!(m::Ptr{Cvoid}, role::Role, layer::Int, A::AbstractMatrix)
    GC.@preserve A check(ccall((:l2b_model_upload_tensor, LIB), Int32,
        (Ptr{Cvoid}, Int32, Int32, Int32, Ptr{Cvoid}, Int64, Int64),
        m, Int32(role), layer - 1, ggml_type(A), pointer(A), in_dim(A), size(A, 2)))
end
function upload!(m::Ptr{Cvoid}, role::Role, layer::Int, v::Vector{Float32})
    GC.@preserve v check(ccall((:l2b_model_upload_tensor, LIB), Int32,
        (Ptr{Cvoid}, Int32, Int32, Int32, Ptr{Cvoid}, Int64, Int64),
        m, Int32(role), layer - 1, L2B_TYPE_F32, pointer(v), length(v), 1))
end

function DeviceModel(config::ModelConfig, w::TransformerWeights; act_planes=0)
    cfg = Ref(L2BConfig(config; act_planes))
    model = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:l2b_model_create, LIB), Int32, (Ref{L2BConfig}, Ref{Ptr{Cvoid}}), cfg, model))
    m = model[]
    upload!(m, TOKEN_EMBEDDING, 1, w.token_embedding_table)
    upload!(m, OUTPUT, 1, w.output_weight)
    upload!(m, RMS_FINAL, 1, w.rms_final_weight)
    for (l, lw) in enumerate(w.layers)
        upload!(m, RMS_ATT, l, lw.rms_att_weight); upload!(m, RMS_FFN, l, lw.rms_ffn_weight)
        upload!(m, WQ, l, lw.wq); upload!(m, WK, l, lw.wk); upload!(m, WV, l, lw.wv); upload!(m, WO, l, lw.wo)
        upload!(m, W1, l, lw.w1); upload!(m, W2, l, lw.w2); upload!(m, W3, l, lw.w3)
    end
    check(ccall((:l2b_model_finalize, LIB), Int32, (Ptr{Cvoid},), m))
    session = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:l2b_session_create, LIB), Int32, (Ptr{Cvoid}, Ptr{Cvoid}, Ref{Ptr{Cvoid}}), m, C_NULL, session))
    dm = DeviceModel(m, session[])
    finalizer(dm) do d
        ccall((:l2b_session_destroy, LIB), Int32, (Ptr{Cvoid},), d.session)
        ccall((:l2b_model_destroy, LIB), Int32, (Ptr{Cvoid},), d.model)
    end
    return dm
end

const DEVICE_MODELS = IdDict{TransformerWeights,DeviceModel}()
device_model(config, weights) = get!(() -> DeviceModel(config, weights), DEVICE_MODELS, weights)

# ---- transformer! ------------------------------------------------------------------------------
# RunState keeps its host logits buffer; activations and the KV cache live in the session.
function transformer!(token::Int, pos::Int, config::ModelConfig, s::RunState, weights::TransformerWeights)
    dm = device_model(config, weights)
    pos == 1 && check(ccall((:l2b_session_reset, LIB), Int32, (Ptr{Cvoid},), dm.session))   # a fresh RunState has a zeroed cache
    GC.@preserve s check(ccall((:l2b_forward, LIB), Int32, (Ptr{Cvoid}, Int32, Int32, Ptr{Float32}),
                               dm.session, token - 1, pos - 1, pointer(s.logits)))
    return nothing
end

# ---- the sampling step of `sample` ---------------------------------------------------------------
# Replaces lines 351-368 of src/inference.jl: forward + argmax / temperature sampling in one call, so that a
# single Int32 crosses PCIe per position.  rand() supplies the uniform that StatsBase.wsample would draw.
function decode_next(config::ModelConfig, weights::TransformerWeights, token::Int, pos::Int, temperature::Float32)
    dm = device_model(config, weights)
    pos == 1 && check(ccall((:l2b_session_reset, LIB), Int32, (Ptr{Cvoid},), dm.session))
    next = Ref{Int32}(0)
    check(ccall((:l2b_decode_next, LIB), Int32, (Ptr{Cvoid}, Int32, Int32, Float32, Float64, Ref{Int32}),
                dm.session, token - 1, pos - 1, temperature, temperature == 0f0 ? 0.0 : rand(), next))
    return Int(next[]) + 1
end

# ---- the prompt phase of `sample` ----------------------------------------------------------------
# Replaces the iterations of the loop in src/inference.jl:349-356 whose next token is a prompt token: all prompt tokens
# in one call (the library streams the weights once for two positions where it can).  Returns the greedy choice after the
# last prompt token; for temperature sampling the caller reads the logits of that position and draws from them as before.
function prefill!(config::ModelConfig, weights::TransformerWeights, prompt_tokens::Vector{Int})
    dm = device_model(config, weights)
    check(ccall((:l2b_session_reset, LIB), Int32, (Ptr{Cvoid},), dm.session))
    toks = Int32.(prompt_tokens .- 1)
    next = Ref{Int32}(0)
    GC.@preserve toks check(ccall((:l2b_prefill, LIB), Int32, (Ptr{Cvoid}, Ptr{Int32}, Int32, Int32, Ref{Int32}),
                                  dm.session, pointer(toks), length(toks), 0, next))
    return Int(next[]) + 1
end

end # module
