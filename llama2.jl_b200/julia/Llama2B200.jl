# Llama2B200.jl -- the binding a Llama2.jl maintainer adds to run the per-token decode path on a B200.
#
# Included at the end of src/Llama2.jl (`include("Llama2B200.jl")`).  It OVERWRITES NOTHING: every method below is a new
# method on a new type, selected by dispatch, so the package still precompiles and the CPU path stays what it was.
#
#   reference (CPU)                                              this file (B200, through libllama2_b200.so)
#   LanguageModel{TOK}           src/inference.jl:50-54          B200LanguageModel{TOK}   = to_b200(model)
#   RunState(config)             src/inference.jl:88-100         B200RunState(model)      one l2b_session per state
#   matmul!(y, A, x)             src/matmul.jl:3-23              matmul!(y, A::B200Matrix, x)
#   transformer!(token, pos, config, s, weights)  inference.jl:222-315   transformer!(token, pos, config, s::B200RunState, w::B200Weights)
#   sample(model, prompt; ...)   src/inference.jl:317-395        sample(model::B200LanguageModel, prompt; ...)  same keywords, same output
#
# `sample(to_b200(load_gguf_model(path)), "prompt"; temperature = 0.0f0)` prints what `sample(load_gguf_model(path), ...)`
# prints.  To make the unchanged call `sample(model::LanguageModel, ...)` itself run on the GPU, the maintainer replaces the
# body of that method in src/inference.jl by `sample(to_b200(model), prompt; kwargs...)` (an edit of the package's own method,
# not a second definition from here).
#
# Token ids and positions are 1-based in Julia and 0-based at the C ABI: the shim subtracts 1.  Host arrays are borrowed for
# the duration of a call only, so mmap'ed tensors (src/load_gguf.jl:160-185) upload straight from the page cache; every call
# that passes a pointer is wrapped in GC.@preserve.
#
# This file has never been run: Julia is not installed where it was written.  Every ccall below is mirrored, argument type
# for argument type, by the Python ctypes binding that the tests drive (a CPU test parses the tuples in this file and compares
# them with that binding).
module Llama2B200

using Printf
using ..Llama2: ModelConfig, TransformerWeights, TransformerLayerWeights, LanguageModel, Tokenizer,
                block_q4_K, block_q5_K, block_q6_K, QK_K, encode
import ..Llama2: matmul!, transformer!, sample

export to_b200, B200LanguageModel, B200RunState, B200Weights, B200Matrix

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

# ---- matmul! on a matrix resident on the device ------------------------------------------------------
# B200Matrix(A) uploads a host matrix once; matmul!(y, ::B200Matrix, x) is then a new, more specific method than both
# methods of src/matmul.jl (which take AbstractMatrix{Float32} and AbstractMatrix{<:block}).
# Column views of one fused tensor (phi3, src/load_gguf.jl:264-276) are contiguous, so `pointer(A)` is enough.
mutable struct B200Matrix <: AbstractMatrix{Float32}
    handle::Ptr{Cvoid}
    in_dim::Int
    out_dim::Int
end
Base.size(A::B200Matrix) = (A.in_dim, A.out_dim)
Base.getindex(::B200Matrix, ::Int...) = error("a B200Matrix lives on the device; dequantize the host matrix instead")

function B200Matrix(A::AbstractMatrix)
    h = Ref{Ptr{Cvoid}}(C_NULL)
    GC.@preserve A check(ccall((:l2b_matrix_create, LIB), Int32, (Int32, Ptr{Cvoid}, Int64, Int64, Int32, Ref{Ptr{Cvoid}}),
                               ggml_type(A), pointer(A), in_dim(A), size(A, 2), 1, h))
    m = B200Matrix(h[], in_dim(A), size(A, 2))
    finalizer(x -> ccall((:l2b_matrix_destroy, LIB), Int32, (Ptr{Cvoid},), x.handle), m)
    return m
end

function matmul!(y::AbstractVector{Float32}, A::B200Matrix, x::AbstractVector{Float32})
    GC.@preserve y x check(ccall((:l2b_matrix_matvec, LIB), Int32, (Ptr{Cvoid}, Ptr{Float32}, Int32, Ptr{Float32}, Int32),
                                 A.handle, pointer(x), 1, pointer(y), 0))
    return nothing
end

# ---- weights on the device ---------------------------------------------------------------------------
# B200Weights plays the role of TransformerWeights (src/inference.jl:42-48) for the device path: one l2b_model handle.
mutable struct B200Weights
    model::Ptr{Cvoid}
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

function B200Weights(config::ModelConfig, w::TransformerWeights; act_planes=0, device=-1)
    cfg = Ref(L2BConfig(config; act_planes, device))
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
    bw = B200Weights(m)
    finalizer(x -> ccall((:l2b_model_destroy, LIB), Int32, (Ptr{Cvoid},), x.model), bw)
    return bw
end

# ---- the model and its per-call state ------------------------------------------------------------------
struct B200LanguageModel{TOK<:Tokenizer}
    config::ModelConfig
    tokenizer::TOK
    weights::B200Weights
end
to_b200(model::LanguageModel; act_planes=0, device=-1) =
    B200LanguageModel(model.config, model.tokenizer, B200Weights(model.config, model.weights; act_planes, device))

# RunState (src/inference.jl:72-100): activations, logits and a zeroed KV cache -- here one l2b_session, created per state
# (two states on the same weights have two sessions) plus the host copy of the logits.
mutable struct B200RunState
    session::Ptr{Cvoid}
    logits::Vector{Float32}
end
function B200RunState(model::B200LanguageModel)
    session = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:l2b_session_create, LIB), Int32, (Ptr{Cvoid}, Ptr{Cvoid}, Ref{Ptr{Cvoid}}), model.weights.model, C_NULL, session))
    s = B200RunState(session[], zeros(Float32, model.config.vocab_size))
    finalizer(x -> ccall((:l2b_session_destroy, LIB), Int32, (Ptr{Cvoid},), x.session), s)
    return s
end

# ---- transformer! ----------------------------------------------------------------------------------------
function transformer!(token::Int, pos::Int, config::ModelConfig, s::B200RunState, weights::B200Weights)
    GC.@preserve s check(ccall((:l2b_forward, LIB), Int32, (Ptr{Cvoid}, Int32, Int32, Ptr{Float32}),
                               s.session, token - 1, pos - 1, pointer(s.logits)))
    return nothing
end

# One iteration of the loop of `sample` (src/inference.jl:351-368): forward + argmax / temperature sampling in one call, so
# that a single Int32 crosses PCIe per position.  rand() supplies the uniform that StatsBase.wsample would draw.
function decode_next(s::B200RunState, token::Int, pos::Int, temperature::Float32)
    next = Ref{Int32}(0)
    check(ccall((:l2b_decode_next, LIB), Int32, (Ptr{Cvoid}, Int32, Int32, Float32, Float64, Ref{Int32}),
                s.session, token - 1, pos - 1, temperature, temperature == 0f0 ? 0.0 : rand(), next))
    return Int(next[]) + 1
end

# The iterations of that loop whose next token is a prompt token (src/inference.jl:349-356), as one call: tokens at
# positions 1..length(tokens) (the library streams the weights once for two positions where it can).
function prefill!(s::B200RunState, tokens::Vector{Int})
    toks = Int32.(tokens .- 1)
    GC.@preserve toks check(ccall((:l2b_prefill, LIB), Int32, (Ptr{Cvoid}, Ptr{Int32}, Int32, Int32, Ptr{Int32}),
                                  s.session, pointer(toks), length(toks), 0, C_NULL))
    return nothing
end

# ---- sample ------------------------------------------------------------------------------------------------
# src/inference.jl:317-395, statement for statement where the device does not change it: same keywords, same printing, same
# stop rule (a BOS or EOS as the next token ends the loop, prompt tokens included, :371-373), same tok/s line (:391-392).
function sample(
        model::B200LanguageModel,
        prompt::String = "";
        temperature::Float32 = 0.9f0,
        stop_on_special_token = true,
        max_seq_len = typemax(Int),
        bos_token = true,
    )
    if !bos_token && isempty(prompt)
        error("Prompt cannot be empty if bos_token = false")
    end
    (; config, tokenizer) = model
    prompt_tokens = encode(prompt, tokenizer)
    state = B200RunState(model)
    time_start = time_ns()
    if bos_token
        pushfirst!(prompt_tokens, tokenizer.bos_token_id)
    end
    if !bos_token
        print(tokenizer.id_to_token[prompt_tokens[1]])
    end
    token = prompt_tokens[1]
    generated_seq_len = 0
    limit = min(config.seq_len, max_seq_len)
    first_pos = 1
    # positions 1..n_forced are followed by a prompt token: one prefill call, unless the stop rule could fire among them
    n_forced = length(prompt_tokens) - 1
    specials = (tokenizer.bos_token_id, tokenizer.eos_token_id)
    if n_forced >= 2 && n_forced <= limit && !(stop_on_special_token && any(in(specials), prompt_tokens[2:end]))
        prefill!(state, prompt_tokens[1:n_forced])
        for t in prompt_tokens[2:end]
            print(tokenizer.id_to_token[t])
        end
        generated_seq_len = n_forced
        token = prompt_tokens[n_forced + 1]
        first_pos = n_forced + 1
    end
    for pos in first_pos:limit
        next = decode_next(state, token, pos, temperature)
        generated_seq_len += 1
        if pos + 1 <= length(prompt_tokens)
            next = prompt_tokens[pos + 1]
        end
        if stop_on_special_token && (next == tokenizer.bos_token_id || next == tokenizer.eos_token_id)
            break
        end
        print(tokenizer.id_to_token[next])
        token = next
    end
    println()
    time_end = time_ns()
    @printf "-------\nachieved tok/s: %.2f\n" generated_seq_len / (time_end - time_start) * 1e9
    return nothing
end

end # module
