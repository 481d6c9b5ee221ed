// Tokenizer of the reference (src/tokenizer.rs:22-108, src/util.rs:29-37,116-123): loads
// tokenizer.bin and encodes text by greedy best-score pair merging.  Host only; it is not
// on the data-parallel path and exists so that text prompts work through the same API.
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "host_common.h"

struct l2_tokenizer {
    std::vector<std::string> vocab;
    std::vector<float> scores;
    int max_token_length = 0;
    // str_lookup (src/util.rs:29-37): the first match at index >= 260 wins, else the first match.
    std::unordered_map<std::string, int> first_ge260, first_any;
    int lookup(const std::string& s) const {
        auto a = first_ge260.find(s);
        if (a != first_ge260.end()) return a->second;
        auto b = first_any.find(s);
        return b == first_any.end() ? -1 : b->second;
    }
};

using namespace l2;

extern "C" int l2_tokenizer_open(const char* filename, int vocab_size, l2_tokenizer** out) {
    clear_error();
    if (!filename || !out || vocab_size <= 0) return fail(L2_EINVAL, "l2_tokenizer_open: bad argument");
    FILE* f = fopen(filename, "rb");
    if (!f) return fail(L2_EIO, "Failed to open %s", filename);
    l2_tokenizer* t = new l2_tokenizer;
    bool ok = true;
    int32_t v = 0;
    ok = fread(&v, 4, 1, f) == 1;  // src/tokenizer.rs:29
    t->max_token_length = v;
    for (int i = 0; i < vocab_size && ok; i++) {
        float score;
        int32_t len;
        ok = fread(&score, 4, 1, f) == 1 && fread(&len, 4, 1, f) == 1 && len >= 0 && len < (1 << 20);
        if (!ok) break;
        std::string s((size_t)len, '\0');
        ok = len == 0 || fread(&s[0], 1, (size_t)len, f) == (size_t)len;
        t->scores.push_back(score);
        t->vocab.push_back(s);
    }
    fclose(f);
    if (!ok) {
        delete t;
        return fail(L2_EFORMAT, "%s is not a tokenizer file with %d entries", filename, vocab_size);
    }
    for (int i = 0; i < vocab_size; i++) {
        t->first_any.emplace(t->vocab[i], i);
        if (i >= 260) t->first_ge260.emplace(t->vocab[i], i);
    }
    *out = t;
    return L2_OK;
}

extern "C" void l2_tokenizer_free(l2_tokenizer* t) { delete t; }

extern "C" int l2_tokenizer_encode(const l2_tokenizer* t, const char* text, int32_t* ids, int cap) {
    clear_error();
    if (!t || !text || (!ids && cap > 0)) return fail(L2_EINVAL, "l2_tokenizer_encode: null argument");
    std::vector<int> tokens;
    // one token per Unicode scalar value (src/tokenizer.rs:53-60)
    const unsigned char* p = reinterpret_cast<const unsigned char*>(text);
    while (*p) {
        int n = 1;
        if (*p >= 0xF0) n = 4; else if (*p >= 0xE0) n = 3; else if (*p >= 0xC0) n = 2;
        std::string ch;
        for (int i = 0; i < n && p[i]; i++) ch.push_back((char)p[i]);
        const int id = t->lookup(ch);
        if (id < 0) return fail(L2_EINVAL, "character at byte %ld is not in the vocabulary", (long)(p - reinterpret_cast<const unsigned char*>(text)));
        tokens.push_back(id);
        p += ch.size();
    }
    std::string buf;
    while (tokens.size() >= 2) {  // src/tokenizer.rs:63-107
        float best_score = -1e10f;
        int best_id = 0, best_idx = -1;
        for (size_t i = 0; i + 1 < tokens.size(); i++) {
            buf = t->vocab[tokens[i]];
            buf += t->vocab[tokens[i + 1]];
            const int id = t->lookup(buf);
            if (id >= 0 && t->scores[id] > best_score) {
                best_score = t->scores[id];
                best_id = id;
                best_idx = (int)i;
            }
        }
        if (best_idx < 0) break;
        tokens[best_idx] = best_id;
        tokens.erase(tokens.begin() + best_idx + 1);
    }
    for (size_t i = 0; i < tokens.size() && (int)i < cap; i++) ids[i] = tokens[i];
    return (int)tokens.size();
}

extern "C" const char* l2_tokenizer_vocab(const l2_tokenizer* t, int32_t id) {
    if (!t || id < 0 || id >= (int)t->vocab.size()) return nullptr;
    return t->vocab[id].c_str();
}

extern "C" const char* l2_tokenizer_piece(const l2_tokenizer* t, int32_t prev, int32_t next) {
    const char* s = l2_tokenizer_vocab(t, next);
    if (!s) return nullptr;
    return (prev == 1 && s[0] == ' ') ? s + 1 : s;  // src/util.rs:116-123
}
