// The BPE tokenizer of the reference inside the library: encode (src/tokenizer.jl:11-57) and the vocabulary fix-ups its
// GGUF loader applies (src/load_gguf.jl:196-209, 339-380).  Host code only; token ids are 0-based at this boundary.
#include <cstring>
#include <limits>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/llama2_b200.h"
#include "gguf_reader.h"

using namespace l2b;

// defined in api.cu: records the message l2b_last_error_string() returns and hands the code back
int32_t l2b_internal_fail(int32_t code, const std::string& msg);

struct l2b_tokenizer {
    std::vector<std::string> id_to_token;            // after the fix-ups: what `sample` prints
    std::unordered_map<std::string, int32_t> token_to_id;  // the LAST id wins for duplicate strings, as in a Julia Dict built in order
    std::vector<float> scores;
    int32_t bos = 0, eos = 0;
};

namespace {

enum : int { TOKEN_NORMAL = 1, TOKEN_BYTE = 6 };  // LLAMA_TOKEN_TYPE (src/load_gguf.jl:44-52)

// One UTF-8 encoded character starting at s[i]; advances i.  Malformed input yields the byte itself.
uint32_t next_char(const std::string& s, size_t& i) {
    const unsigned char c = (unsigned char)s[i];
    const int n = c < 0x80 ? 0 : (c >> 5) == 6 ? 1 : (c >> 4) == 14 ? 2 : (c >> 3) == 30 ? 3 : 0;
    bool ok = n > 0 && i + (size_t)n < s.size();
    for (int k = 1; ok && k <= n; ++k) ok = ((unsigned char)s[i + k] & 0xC0) == 0x80;
    if (!ok) {
        ++i;
        return c;
    }
    uint32_t cp = c & (0xFFu >> (n + 2));
    for (int k = 1; k <= n; ++k) cp = (cp << 6) | ((unsigned char)s[i + k] & 0x3F);
    i += (size_t)n + 1;
    return cp;
}

void put_char(std::string& out, uint32_t cp) {
    if (cp < 0x80) out.push_back((char)cp);
    else if (cp < 0x800) {
        out.push_back((char)(0xC0 | (cp >> 6)));
        out.push_back((char)(0x80 | (cp & 0x3F)));
    } else if (cp < 0x10000) {
        out.push_back((char)(0xE0 | (cp >> 12)));
        out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
        out.push_back((char)(0x80 | (cp & 0x3F)));
    } else {
        out.push_back((char)(0xF0 | (cp >> 18)));
        out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
        out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
        out.push_back((char)(0x80 | (cp & 0x3F)));
    }
}

// gpt2_decoder() (src/load_gguf.jl:196-209): the printable stand-in characters of GPT-2's byte encoder, back to byte values.
std::unordered_map<uint32_t, uint32_t> gpt2_decoder() {
    std::vector<uint32_t> bs, cs;
    auto range = [&](uint32_t a, uint32_t b) {
        for (uint32_t v = a; v <= b; ++v) bs.push_back(v);
    };
    range('!', '~');
    range(0xA1, 0xAC);
    range(0xAE, 0xFF);
    cs = bs;
    uint32_t n = 0;
    for (uint32_t b = 0; b < 256; ++b) {
        bool in = false;
        for (uint32_t v : bs) in |= (v == b);
        if (!in) {
            bs.push_back(b);
            cs.push_back(256 + n);
            ++n;
        }
    }
    std::unordered_map<uint32_t, uint32_t> d;
    for (size_t i = 0; i < bs.size(); ++i) d[cs[i]] = bs[i];
    return d;
}

// The fix-ups of load_gguf_model (src/load_gguf.jl:345-368).  model: 0 none, 1 "llama", 2 "gpt2".
int32_t fix_vocabulary(std::vector<std::string>& toks, const int32_t* types, int32_t model) {
    if (model == 0) return L2B_OK;
    if (!types) return l2b_internal_fail(L2B_ERR_BAD_ARG, "token types are needed for the llama and gpt2 vocabulary fix-ups");
    if (model == 1) {
        for (size_t i = 0; i < toks.size(); ++i) {
            if (types[i] == TOKEN_NORMAL) {  // the SentencePiece space marker U+2581 becomes a space
                std::string& t = toks[i];
                std::string out;
                for (size_t k = 0; k < t.size();) {
                    if (k + 2 < t.size() && (unsigned char)t[k] == 0xE2 && (unsigned char)t[k + 1] == 0x96 && (unsigned char)t[k + 2] == 0x81) {
                        out.push_back(' ');
                        k += 3;
                    } else {
                        out.push_back(t[k++]);
                    }
                }
                t.swap(out);
            } else if (types[i] == TOKEN_BYTE) {  // "<0xNN>" -> the byte NN
                const std::string& t = toks[i];
                if (t.size() < 3) return l2b_internal_fail(L2B_ERR_BAD_ARG, "malformed byte token " + t);
                char* end = nullptr;
                const std::string inner = t.substr(1, t.size() - 2);
                const long v = strtol(inner.c_str(), &end, 0);
                if (!end || *end != 0 || v < 0 || v > 255) return l2b_internal_fail(L2B_ERR_BAD_ARG, "malformed byte token " + t);
                toks[i] = std::string(1, (char)v);
            }
        }
        return L2B_OK;
    }
    if (model == 2) {
        const auto dec = gpt2_decoder();
        for (size_t i = 0; i < toks.size(); ++i) {
            if (types[i] != TOKEN_NORMAL) continue;
            std::string out;
            for (size_t k = 0; k < toks[i].size();) {
                const uint32_t cp = next_char(toks[i], k);
                auto it = dec.find(cp);
                if (it == dec.end()) return l2b_internal_fail(L2B_ERR_BAD_ARG, "token " + std::to_string(i) + " holds a character outside GPT-2's byte alphabet");
                put_char(out, it->second);  // String(::Vector{Char}): the byte value as a character, UTF-8 encoded
            }
            toks[i].swap(out);
        }
        return L2B_OK;
    }
    return l2b_internal_fail(L2B_ERR_BAD_ARG, "unsupported tokenizer model");  // src/load_gguf.jl:370
}

int32_t finish(l2b_tokenizer* t, const int32_t* types, int32_t model, l2b_tokenizer** out) {
    int32_t st = fix_vocabulary(t->id_to_token, types, model);
    if (st == L2B_OK && (t->bos < 0 || t->eos < 0 || t->bos >= (int32_t)t->id_to_token.size() || t->eos >= (int32_t)t->id_to_token.size()))
        st = l2b_internal_fail(L2B_ERR_BAD_ARG, "bos / eos token id outside the vocabulary");
    if (st != L2B_OK) {
        delete t;
        return st;
    }
    t->token_to_id.reserve(t->id_to_token.size() * 2);
    for (size_t i = 0; i < t->id_to_token.size(); ++i) t->token_to_id[t->id_to_token[i]] = (int32_t)i;
    *out = t;
    return L2B_OK;
}

}  // namespace

extern "C" int32_t l2b_tokenizer_create(const uint8_t* token_bytes, const int64_t* offsets, int32_t n_tokens, const float* scores,
                                        const int32_t* token_types, int32_t model, int32_t bos_id, int32_t eos_id, l2b_tokenizer** out) {
    if (!token_bytes || !offsets || !out || n_tokens <= 0) return l2b_internal_fail(L2B_ERR_BAD_ARG, "null argument or empty vocabulary");
    *out = nullptr;
    if (model < 0 || model > 2) return l2b_internal_fail(L2B_ERR_BAD_ARG, "unsupported tokenizer model");
    l2b_tokenizer* t = new l2b_tokenizer();
    t->id_to_token.resize(n_tokens);
    for (int32_t i = 0; i < n_tokens; ++i) {
        if (offsets[i + 1] < offsets[i]) {
            delete t;
            return l2b_internal_fail(L2B_ERR_BAD_ARG, "token offsets must not decrease");
        }
        t->id_to_token[i].assign(reinterpret_cast<const char*>(token_bytes) + offsets[i], (size_t)(offsets[i + 1] - offsets[i]));
    }
    t->scores.assign(n_tokens, 0.f);
    if (scores) memcpy(t->scores.data(), scores, (size_t)n_tokens * 4);
    t->bos = bos_id;
    t->eos = eos_id;
    return finish(t, token_types, model, out);
}

extern "C" int32_t l2b_tokenizer_load_gguf(const char* path, l2b_tokenizer** out) {
    if (!path || !out) return l2b_internal_fail(L2B_ERR_BAD_ARG, "null argument");
    *out = nullptr;
    GgufFile f;
    if (!f.open(path)) return l2b_internal_fail(L2B_ERR_BAD_ARG, f.error());
    const GgufValue* toks = f.find("tokenizer.ggml.tokens");
    const GgufValue* types = f.find("tokenizer.ggml.token_type");
    const GgufValue* model = f.find("tokenizer.ggml.model");
    const GgufValue* scores = f.find("tokenizer.ggml.scores");
    const GgufValue* bos = f.find("tokenizer.ggml.bos_token_id");
    const GgufValue* eos = f.find("tokenizer.ggml.eos_token_id");
    if (!toks || toks->type != 9 || toks->elem_type != 8 || !types || types->type != 9 || !model || model->type != 8 || !bos || !eos)
        return l2b_internal_fail(L2B_ERR_BAD_ARG, "the file has no complete tokenizer.ggml.* metadata");
    if (types->count != toks->count || (types->elem_type != 4 && types->elem_type != 5))
        return l2b_internal_fail(L2B_ERR_BAD_ARG, "tokenizer.ggml.token_type must hold one 32-bit integer per token");
    int32_t mid;
    if (model->str == "llama") mid = 1;
    else if (model->str == "gpt2") mid = 2;
    else return l2b_internal_fail(L2B_ERR_BAD_ARG, "unsupported tokenizer model: " + model->str);  // src/load_gguf.jl:370
    l2b_tokenizer* t = new l2b_tokenizer();
    t->id_to_token.resize((size_t)toks->count);
    const uint8_t* p = toks->elems;
    for (uint64_t i = 0; i < toks->count; ++i) {  // bounds were checked when the file was opened
        uint64_t n;
        memcpy(&n, p, 8);
        t->id_to_token[i].assign(reinterpret_cast<const char*>(p + 8), (size_t)n);
        p += 8 + n;
    }
    t->scores.assign((size_t)toks->count, 0.f);
    if (scores && scores->type == 9 && scores->elem_type == 6 && scores->count == toks->count) memcpy(t->scores.data(), scores->elems, (size_t)toks->count * 4);
    std::vector<int32_t> ty((size_t)toks->count);
    memcpy(ty.data(), types->elems, (size_t)toks->count * 4);
    t->bos = (int32_t)bos->inum;
    t->eos = (int32_t)eos->inum;
    return finish(t, ty.data(), mid, out);
}

extern "C" int32_t l2b_tokenizer_destroy(l2b_tokenizer* t) {
    delete t;
    return L2B_OK;
}

extern "C" int32_t l2b_tokenizer_info(const l2b_tokenizer* t, int32_t* n_tokens, int32_t* bos_id, int32_t* eos_id) {
    if (!t) return l2b_internal_fail(L2B_ERR_BAD_ARG, "null tokenizer");
    if (n_tokens) *n_tokens = (int32_t)t->id_to_token.size();
    if (bos_id) *bos_id = t->bos;
    if (eos_id) *eos_id = t->eos;
    return L2B_OK;
}

extern "C" int32_t l2b_tokenizer_token(const l2b_tokenizer* t, int32_t id, const uint8_t** bytes, int64_t* n_bytes) {
    if (!t || !bytes || !n_bytes) return l2b_internal_fail(L2B_ERR_BAD_ARG, "null argument");
    if (id < 0 || id >= (int32_t)t->id_to_token.size()) return l2b_internal_fail(L2B_ERR_BAD_ARG, "token id out of range");
    *bytes = reinterpret_cast<const uint8_t*>(t->id_to_token[id].data());
    *n_bytes = (int64_t)t->id_to_token[id].size();
    return L2B_OK;
}

// encode(text, tokenizer; pad_input) (src/tokenizer.jl:11-57): a space token in front (pad_input), one token per byte of the
// text, then repeatedly merge the adjacent pair whose concatenation is a token with the highest score (the first such pair
// on ties, since the comparison is strict) until no pair is a token.
extern "C" int32_t l2b_tokenizer_encode(const l2b_tokenizer* t, const uint8_t* text, int64_t n_bytes, int32_t pad_input, int32_t* ids_out,
                                        int64_t capacity, int64_t* n_out) {
    if (!t || (!text && n_bytes > 0) || !n_out || n_bytes < 0 || (!ids_out && capacity > 0)) return l2b_internal_fail(L2B_ERR_BAD_ARG, "null argument");
    *n_out = 0;
    if (n_bytes == 0) return L2B_OK;
    std::vector<int32_t> tokens;
    tokens.reserve((size_t)n_bytes + 1);
    auto lookup = [&](const std::string& s) -> int32_t {
        auto it = t->token_to_id.find(s);
        return it == t->token_to_id.end() ? -1 : it->second;
    };
    if (pad_input) {
        const int32_t sp = lookup(" ");
        if (sp < 0) return l2b_internal_fail(L2B_ERR_BAD_ARG, "the vocabulary has no token for a single space");  // KeyError in the reference
        tokens.push_back(sp);
    }
    for (int64_t i = 0; i < n_bytes; ++i) {
        const int32_t id = lookup(std::string(1, (char)text[i]));
        if (id < 0) return l2b_internal_fail(L2B_ERR_BAD_ARG, "the vocabulary has no token for byte " + std::to_string((int)text[i]));
        tokens.push_back(id);
    }
    std::string cat;
    for (;;) {
        float best_score = -std::numeric_limits<float>::infinity();
        int32_t best_id = -1;
        int64_t best_idx = -1;
        for (size_t i = 0; i + 1 < tokens.size(); ++i) {
            cat.assign(t->id_to_token[tokens[i]]);
            cat.append(t->id_to_token[tokens[i + 1]]);
            const int32_t id = lookup(cat);
            if (id >= 0 && t->scores[id] > best_score) {
                best_score = t->scores[id];
                best_id = id;
                best_idx = (int64_t)i;
            }
        }
        if (best_idx < 0) break;
        tokens[(size_t)best_idx] = best_id;
        tokens.erase(tokens.begin() + best_idx + 1);
    }
    *n_out = (int64_t)tokens.size();
    if ((int64_t)tokens.size() > capacity) return l2b_internal_fail(L2B_ERR_BAD_ARG, "ids_out is too small: " + std::to_string(tokens.size()) + " tokens");
    memcpy(ids_out, tokens.data(), tokens.size() * 4);
    return L2B_OK;
}
