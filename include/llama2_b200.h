/*
 * llama2_b200.h -- C ABI of the B200 (sm_100a) per-token decode library.
 *
 * This is the boundary a Llama2.jl maintainer binds with `ccall`.  The reference has no
 * FFI of its own; each entry point below names the reference function or type it
 * replaces (paths relative to the reference project root).
 *
 * Conventions
 *   - every function returns an int32 status (L2B_OK == 0); no exception, abort or exit
 *     crosses the boundary; l2b_last_error_string() gives the text of the last failure
 *     on the calling thread;
 *   - token ids and positions are 0-BASED here (the Julia shim subtracts 1);
 *   - pointers named host_* are host memory, borrowed for the duration of the call only
 *     (they may point into a read-only mmap, as src/load_gguf.jl:160-185 produces);
 *   - matrices are given exactly as the reference stores them: `in` contiguous weights
 *     (or in/256 contiguous super-blocks) per output row, `out` rows
 *     (src/inference.jl:32-47, src/matmul.jl:1);
 *   - a session is used by one host thread at a time; different sessions may be used
 *     concurrently;
 *   - there is no CPU fallback: without a CUDA device every compute entry point returns
 *     L2B_ERR_NO_DEVICE.
 */
#ifndef LLAMA2_B200_H
#define LLAMA2_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct l2b_model l2b_model;     /* TransformerWeights + ModelConfig on the device */
typedef struct l2b_session l2b_session; /* RunState: activations, KV cache, captured token graph */
typedef struct l2b_matrix l2b_matrix;   /* one weight matrix resident on the device */
typedef struct l2b_batch l2b_batch;     /* several RunStates decoded in lock step (batched decode) */
typedef struct l2b_tokenizer l2b_tokenizer; /* BPETokenizer (src/tokenizer.jl:3-9), host memory only */

enum l2b_status {
    L2B_OK = 0,
    L2B_ERR_BAD_ARG = 1,
    L2B_ERR_UNSUPPORTED_TYPE = 2, /* src/load_gguf.jl:153,179 "tensor type ... not implemented" */
    L2B_ERR_CUDA = 3,
    /* 4 is not used */
    L2B_ERR_TIMEOUT = 5, /* a bounded device-side wait ran out */
    L2B_ERR_OOM = 6,
    L2B_ERR_STATE = 7, /* call order: e.g. forward before finalize */
    L2B_ERR_NO_DEVICE = 8
};

/* GGML tensor types the reference can load (src/load_gguf.jl:26-42,135-154). */
enum l2b_ggml_type { L2B_TYPE_F32 = 0, L2B_TYPE_Q4_K = 12, L2B_TYPE_Q5_K = 13, L2B_TYPE_Q6_K = 14 };

/* Tensor roles = the fields of TransformerWeights / TransformerLayerWeights
 * (src/inference.jl:27-48). */
enum l2b_role {
    L2B_ROLE_TOKEN_EMBEDDING = 0, /* token_embedding_table (dim, vocab) */
    L2B_ROLE_RMS_ATT = 1,         /* rms_att_weight (dim,)  f32 */
    L2B_ROLE_WQ = 2,
    L2B_ROLE_WK = 3,
    L2B_ROLE_WV = 4,
    L2B_ROLE_WO = 5,
    L2B_ROLE_RMS_FFN = 6, /* rms_ffn_weight (dim,) f32 */
    L2B_ROLE_W1 = 7,      /* ffn gate */
    L2B_ROLE_W2 = 8,      /* ffn down */
    L2B_ROLE_W3 = 9,      /* ffn up */
    L2B_ROLE_RMS_FINAL = 10,
    L2B_ROLE_OUTPUT = 11 /* output_weight (dim, vocab) */
};

/* ModelConfig (src/inference.jl:1-11), field for field, followed by library options. */
typedef struct l2b_config {
    int32_t dim;
    int32_t hidden_dim;
    int32_t n_layers;
    int32_t n_heads;
    int32_t n_kv_heads;
    int32_t vocab_size;
    int32_t seq_len; /* the reference pins GGUF models to 512 (src/load_gguf.jl:237); any value is accepted here */
    float rope_freq_base;
    int32_t rope_is_neox;
    /* ---- options with no counterpart in the reference ---- */
    int32_t act_planes; /* int8 planes per activation value fed to the k-quant integer dot products:
                           1 = one q8_K plane (8-bit activations), 2 = two (~15 bit), 3 = three (~23 bit,
                           indistinguishable from the reference's f32 activations); 0 selects 3 */
    int32_t device;     /* CUDA device ordinal; -1 = current device */
    int32_t tp_size;    /* tensor-parallel world size (1 = single GPU) */
    int32_t tp_rank;
    int32_t reserved[7];
} l2b_config;

/* ---- library ------------------------------------------------------------------ */
int32_t l2b_version(void);
const char* l2b_last_error_string(void);
const char* l2b_status_string(int32_t status);
int32_t l2b_device_count(int32_t* count);

/* ---- model: replaces the TransformerWeights the loaders build
 *      (src/load_gguf.jl:229-253,291-315; src/load_karpathy.jl:36-56) ------------- */
int32_t l2b_model_create(const l2b_config* config, l2b_model** model);
/* Upload one tensor.  `layer` is 0-based and ignored for the three model-level roles.
 * ggml_type is one of l2b_ggml_type; in_dim % 256 == 0 is required for k-quants
 * (src/load_gguf.jl:141,145,149).  Norm gains are f32 with out_dim == 1. */
int32_t l2b_model_upload_tensor(l2b_model* model, int32_t role, int32_t layer, int32_t ggml_type, const void* host_data,
                                int64_t in_dim, int64_t out_dim);
int32_t l2b_model_finalize(l2b_model* model); /* checks that every tensor is present and shapes agree */
int32_t l2b_model_destroy(l2b_model* model);
int32_t l2b_model_weight_bytes(const l2b_model* model, int64_t* bytes_per_token); /* bytes a decoded token streams from HBM */

/* ---- session: replaces RunState / KVCache (src/inference.jl:62-100) ----------------
 * `stream` is a cudaStream_t passed as a pointer (NULL = the library creates its own). */
int32_t l2b_session_create(l2b_model* model, void* stream, l2b_session** session);
int32_t l2b_session_reset(l2b_session* session); /* zero the KV cache, as a fresh RunState */
/* ---- GGUF files --------------------------------------------------------------------- */
/* The file walk of load_gguf_model (src/load_gguf.jl:317-336: header, metadata, tensor directory, alignment) and the model
 * construction of build_llama / build_phi3 (:211-315) inside the library: the file is memory-mapped and every tensor is
 * uploaded straight from the map.  Every metadata value type of the format is read (the reference reads six, :59-77); a
 * missing output.weight means a classifier tied to the embedding.  The tokenizer metadata stays with the host.
 *   seq_len > 0: as given; 0: the file's <arch>.context_length; < 0: the 512 the reference hard-codes (:237, :299). */
int32_t l2b_model_load_gguf(const char* path, int32_t seq_len, int32_t act_planes, int32_t device, int32_t tp_size, int32_t tp_rank,
                            l2b_config* config_out, l2b_model** model);
/* The same parse without a device: ModelConfig fields (seq_len = context_length), architecture (0 llama, 1 phi3),
 * number of tensors, context length.  Fails with L2B_ERR_BAD_ARG ("Not a GGUF file", :89) on anything else. */
int32_t l2b_gguf_inspect(const char* path, l2b_config* config_out, int32_t* arch_out, int64_t* n_tensors, int64_t* context_length);

/* ---- tokenizer (host only; ids are 0-based here, bos / eos included) ------------------------------------
 * BPETokenizer (src/tokenizer.jl:3-9) from a vocabulary as a file stores it: token i is
 * token_bytes[offsets[i] .. offsets[i+1]); scores may be NULL (all 0); token_types (LLAMA_TOKEN_TYPE, src/load_gguf.jl:44-52)
 * may be NULL when model == 0.  model selects the fix-ups load_gguf_model applies (src/load_gguf.jl:345-368):
 *   0 none (a llama2.c tokenizer.bin, src/load_karpathy.jl:58-78); 1 "llama": U+2581 becomes a space in NORMAL tokens and
 *   BYTE tokens "<0xNN>" become the byte; 2 "gpt2": NORMAL tokens go through the inverse of GPT-2's byte encoder (:196-209). */
int32_t l2b_tokenizer_create(const uint8_t* token_bytes, const int64_t* offsets, int32_t n_tokens, const float* scores,
                             const int32_t* token_types, int32_t model, int32_t bos_id, int32_t eos_id, l2b_tokenizer** tokenizer);
/* The tokenizer part of load_gguf_model (src/load_gguf.jl:339-380): tokenizer.ggml.{tokens,token_type,model,scores,
 * bos_token_id,eos_token_id} read from the file by the library's own GGUF parser. */
int32_t l2b_tokenizer_load_gguf(const char* path, l2b_tokenizer** tokenizer);
int32_t l2b_tokenizer_destroy(l2b_tokenizer* tokenizer);
int32_t l2b_tokenizer_info(const l2b_tokenizer* tokenizer, int32_t* n_tokens, int32_t* bos_id, int32_t* eos_id);
/* id_to_token[id] after the fix-ups (what `sample` prints, src/inference.jl:375-382): a pointer into the tokenizer, valid
 * until it is destroyed; tokens may hold any bytes. */
int32_t l2b_tokenizer_token(const l2b_tokenizer* tokenizer, int32_t id, const uint8_t** bytes, int64_t* n_bytes);
/* encode(text, tokenizer; pad_input) (src/tokenizer.jl:11-57).  *n_out receives the number of tokens; when that exceeds
 * `capacity` nothing is written and L2B_ERR_BAD_ARG is returned (n_bytes + 1 always suffices).  A byte of the text (or the
 * space of pad_input) without a token of its own is L2B_ERR_BAD_ARG, where the reference raises a KeyError. */
int32_t l2b_tokenizer_encode(const l2b_tokenizer* tokenizer, const uint8_t* text, int64_t n_bytes, int32_t pad_input,
                             int32_t* ids_out, int64_t capacity, int64_t* n_out);

/* ---- tensor parallelism (no counterpart in the reference, which runs on one CPU) ------
 * One process per GPU; every rank creates its model with the same l2b_config except tp_rank, uploads the FULL tensors
 * (the library keeps its shard: whole kv groups of wq/wk/wv, hidden units of w1/w3, super-block columns of wo/w2; needs
 * n_kv_heads, dim/256 and hidden_dim/256 divisible by tp_size and k-quant wo/w2), and creates a session.  Then:
 *   l2b_session_tp_handle  writes a 64-byte handle of this rank's exchange memory;
 *   the host moves the handles between the processes (any transport) ...
 *   l2b_session_tp_connect takes all tp_size handles ordered by rank, maps the peers' memory and captures the token graph.
 * After that l2b_forward / l2b_decode_next / l2b_generate must be called by ALL ranks with the same arguments; every rank
 * returns the same logits and tokens.  A rank whose peers do not deliver within L2B_TP_TIMEOUT_MS (default 10000) gets
 * L2B_ERR_TIMEOUT.  All ranks must have finished their calls before any of them destroys its session. */
int32_t l2b_session_tp_handle(l2b_session* session, void* handle64);
int32_t l2b_session_tp_connect(l2b_session* session, const void* handles, int32_t count);

int32_t l2b_session_destroy(l2b_session* session);

/* transformer!(token, pos, config, s, weights) (src/inference.jl:222-315): one token
 * through every layer; the KV cache advances; logits (vocab_size floats) are copied to
 * host_logits when it is non-NULL. */
int32_t l2b_forward(l2b_session* session, int32_t token, int32_t pos, float* host_logits);

/* One iteration of the loop in `sample` (src/inference.jl:349-385): forward, then
 * temperature == 0 ? argmax (first maximal index) : softmax(logits / temperature) sampled
 * by inverse CDF with the caller's uniform variate in [0,1) (StatsBase.wsample draws its
 * own from Julia's global RNG; that stream cannot be reproduced outside Julia). */
int32_t l2b_decode_next(l2b_session* session, int32_t token, int32_t pos, float temperature, double uniform, int32_t* next_token);

/* The whole loop of `sample` on the device: positions 0 .. n_positions-1, teacher-forced
 * while inside the prompt, then greedy (temperature 0) or sampled with uniforms drawn from
 * a counter-based generator seeded by `seed`.  host_out_tokens[p] = token chosen after
 * position p.  No stop on BOS/EOS (stop_on_special_token=false); the shim truncates.
 * device_ms (optional) = CUDA-event time of the loop. */
int32_t l2b_generate(l2b_session* session, const int32_t* host_prompt, int32_t n_prompt, int32_t n_positions,
                     float temperature, uint64_t seed, int32_t* host_out_tokens, float* device_ms);

/* Copy the logits of the most recent position to the host (state.logits). */
int32_t l2b_session_logits(l2b_session* session, float* host_logits);
/* Copy an activation buffer of the most recent forward for stage-wise checks:
 * which: 0 = x (residual stream after the last layer, before the final norm is applied in place),
 *        2 = q (after RoPE, last layer), 5 = hb (SwiGLU output, last layer).  Returns element count in *n. */
int32_t l2b_session_read(l2b_session* session, int32_t which, float* host_out, int64_t capacity, int64_t* n);
/* Device time (ms, CUDA events on the session stream) of the most recent forward/decode/generate call. */
int32_t l2b_session_last_device_ms(l2b_session* session, float* ms);
/* The same for the most recent l2b_generate call, split where the loop of `sample` stops being teacher-forced
 * (src/inference.jl:354-356): positions 0 .. n_prompt-1 (fed prompt tokens) and positions n_prompt .. (fed generated tokens). */
int32_t l2b_session_last_phase_ms(l2b_session* session, float* prompt_ms, float* decode_ms);
/* The prompt phase of `sample` (src/inference.jl:349-356, where the reference runs transformer! once per prompt token) as one
 * call: feeds tokens[0..n-1] at positions pos0 .. pos0+n-1, two positions per pass where both are followed by a prompt token.
 * Afterwards the session holds the logits of the last prompt position (l2b_session_logits); *next (may be NULL) is their argmax.
 * Continue with l2b_decode_next(session, chosen_token, pos0 + n, ...). */
int32_t l2b_prefill(l2b_session* session, const int32_t* tokens, int32_t n, int32_t pos0, int32_t* next);
/* *min_tokens > 0: runs of at least that many prompt positions that are all followed by a prompt token go through the
 * many-token pass (every matrix product one launch of the tensor-core GEMM, tcgen05 + TMA, 20 tokens per pass over a weight
 * tile; up to 240 tokens per pass over the layers).  0: not available for this model (needs q4_K / q5_K layer matrices, three
 * activation planes, one GPU; L2B_PREFILL_GEMM=0 switches it off) -- prompts then go through the decode kernels.  The reference
 * feeds prompts token by token (src/inference.jl:349-356). */
int32_t l2b_session_prefill_gemm(l2b_session* session, int32_t* min_tokens);
/* 1 when l2b_generate feeds prompts two positions per pass (k-quant model, three activation planes, one GPU, everything fits in
 * shared memory; switch off with L2B_PREFILL_PAIRS=0): positions p, p+1 that are both followed by a prompt token share one pass
 * over the weights, and no logits are computed for them.  The reference feeds prompts token by token (src/inference.jl:349-356). */
int32_t l2b_session_prefill_pairs(l2b_session* session, int32_t* enabled);
/* Kernel launches the most recent l2b_forward / l2b_decode_next / l2b_prefill / l2b_generate call enqueued. */
int32_t l2b_session_last_launches(l2b_session* session, int64_t* n);
/* Number of kernel launches per token: 1 when the whole token is one persistent kernel (k-quant model on one GPU), else
 * 5 per layer + 3. */
int32_t l2b_session_kernels_per_token(l2b_session* session, int32_t* n);

/* ---- batched decode (no counterpart in the reference, whose `sample` serves one prompt) ----------------------
 * n_seq independent sequences (2 .. 240), each with its own zeroed KV cache of seq_len positions, advanced one position per
 * call: every matrix is streamed once per 20 sequences by the tensor-core GEMM instead of once per sequence.  Needs q4_K /
 * q5_K layer matrices (the classifier may be q6_K), three activation planes, one GPU; otherwise L2B_ERR_UNSUPPORTED_TYPE.
 * l2b_batch_decode_next: tokens[i] is fed at position positions[i] of sequence i (transformer!, src/inference.jl:222-315, for
 * each); next_tokens[i] = argmax of its logits (src/inference.jl:360); host_logits (optional) receives [n_seq][vocab_size]. */
int32_t l2b_batch_create(l2b_model* model, int32_t n_seq, l2b_batch** batch);
int32_t l2b_batch_reset(l2b_batch* batch);
int32_t l2b_batch_destroy(l2b_batch* batch);
int32_t l2b_batch_decode_next(l2b_batch* batch, const int32_t* tokens, const int32_t* positions, int32_t* next_tokens, float* host_logits);

/* ---- isolated operators (host buffers in, host buffers out) ------------------------ */
/* dequantize! (src/kquants.jl:44-47,70-125,186-251,322-363); bit-exact. n_elems % 256 == 0 for k-quants. */
int32_t l2b_dequantize(int32_t ggml_type, const void* host_blocks, int64_t n_elems, float* host_out);
/* Quantise f32 activations to `planes` int8 planes in the layout of block_q8_K (src/kquants.jl:38-42):
 * host_q[p][n] int8, host_d[p][n/256] f32 (scale of plane p), host_sums[n/16] f32 = sums of the represented
 * values over groups of 16 (the role of bsums).  The reference declares block_q8_K but has no quantiser. */
int32_t l2b_quantize_q8k(const float* host_x, int64_t n, int32_t planes, int8_t* host_q, float* host_d, float* host_sums);
/* rmsnorm! (src/inference.jl:102-110) fused with that quantisation, as it runs in front of every k-quant matrix of the
 * token path: the planes represent w .* (x / rms(x)).  Same outputs as l2b_quantize_q8k. */
int32_t l2b_rmsnorm_quantize_q8k(const float* host_x, const float* host_w, int64_t n, int32_t planes, int8_t* host_q, float* host_d,
                                 float* host_sums);
/* matmul!(y, A, x) (src/matmul.jl:3-23) for ncols activation columns: x is [ncols][in], y is [ncols][out]. */
int32_t l2b_matvec(int32_t ggml_type, const void* host_W, int64_t in_dim, int64_t out_dim, const float* host_x,
                   int32_t ncols, float* host_y, int32_t act_planes);
/* rmsnorm!(o, x, w) (src/inference.jl:102-110). */
int32_t l2b_rmsnorm(float* host_o, const float* host_x, const float* host_w, int64_t n);
/* rope!(x, pos, config) (src/inference.jl:112-167); x is [n_heads][head_size], rotated in place. */
int32_t l2b_rope(float* host_x, int32_t head_size, int32_t n_heads, int32_t pos, float freq_base, int32_t is_neox);
/* attention_weights! + scale + softmax! + combine_values! (src/inference.jl:263-278) for one layer:
 * q [n_heads][hs]; k, v [n_pos][n_kv_heads][hs] (position-major); out [n_heads][hs]. */
int32_t l2b_attention(float* host_out, const float* host_q, const float* host_k, const float* host_v, int32_t n_pos,
                      int32_t n_heads, int32_t n_kv_heads, int32_t head_size);
/* The same attention on DEVICE pointers, making no allocation of any kind.  This entry point has no counterpart in
 * the reference (which has no device memory to manage); it exists for callers that must not allocate, e.g. inside a
 * region where the CUDA allocator may not be entered.
 *   dev_q [n_heads][hs], dev_out [n_heads][hs]; dev_kcache, dev_vcache [n_kv_heads][seq_len][hs] f32, of which
 *   positions 0..n_pos-1 are attended.  The launch is asynchronous on `stream` (cudaStream_t; NULL = default).
 * Scratch for the partial results lives in one fixed device array inside the library (about 0.26 MiB per device), so:
 *   - limits: n_heads <= 128, head_size <= 128 (a multiple of 8); larger shapes are rejected with L2B_ERR_BAD_ARG
 *     (the scratch holds one partial result per cluster of blocks, at most four per head group);
 *   - the first call on each device resolves the array's address and must be made outside any stream capture;
 *   - the array is shared by all calls on a device and keeps the previous call's contents (the words that must be
 *     zero are cleared on `stream` before each launch); calls whose execution overlaps race on it, so callers
 *     serialise their calls per device. */
int32_t l2b_attention_device_noalloc(float* dev_out, const float* dev_q, const float* dev_kcache, const float* dev_vcache,
                                     int32_t n_pos, int32_t seq_len, int32_t n_heads, int32_t n_kv_heads, int32_t head_size,
                                     void* stream);
/* hb = silu(hb) .* hb2 (src/inference.jl:295-299); written to host_hb. */
int32_t l2b_swiglu(float* host_hb, const float* host_hb2, int64_t n);
/* argmax(logits) (src/inference.jl:360), first maximal index, 0-based. */
int32_t l2b_argmax(const float* host_logits, int64_t n, int32_t* index);
/* logits ./= T; softmax!; wsample (src/inference.jl:361-368) with a supplied uniform in [0,1). */
int32_t l2b_sample_temperature(const float* host_logits, int64_t n, float temperature, double uniform, int32_t* index);

/* ---- resident matrices (for measurement with inputs already in HBM) ----------------- */
/* Upload `copies` identical copies of one matrix (copies > 1 lets a benchmark rotate through more than the L2). */
int32_t l2b_matrix_create(int32_t ggml_type, const void* host_W, int64_t in_dim, int64_t out_dim, int32_t copies, l2b_matrix** m);
int32_t l2b_matrix_destroy(l2b_matrix* m);
/* y = A' x on device pointers (x: [in] f32, y: [out] f32), copy index `copy`, on `stream` (cudaStream_t; NULL = default). */
int32_t l2b_matrix_matvec_device(l2b_matrix* m, int32_t copy, const float* dev_x, float* dev_y, int32_t act_planes, void* stream);
/* ncols columns at once on device pointers (x: [ncols][in], y: [ncols][out]) through the tensor-core GEMM (q4_K / q5_K): the
 * weights are streamed once per 20 columns.  The first call (and any call with more columns than before) allocates the buffer
 * of quantised columns. */
int32_t l2b_matrix_matmul_device(l2b_matrix* m, int32_t copy, const float* dev_x, int32_t ncols, float* dev_y, void* stream);
/* The same through host buffers (x: [ncols][in], y: [ncols][out]); 4 or more columns of a q4_K / q5_K matrix take the GEMM. */
int32_t l2b_matrix_matvec(l2b_matrix* m, const float* host_x, int32_t ncols, float* host_y, int32_t act_planes);

#ifdef __cplusplus
}
#endif
#endif /* LLAMA2_B200_H */
