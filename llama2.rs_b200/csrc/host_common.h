// Host-side definitions shared by the loader, the synthetic checkpoint generator and
// the C ABI: checkpoint layout, error reporting, tensor sources.
#pragma once

#include <cstddef>
#include <cstdint>
#include <algorithm>
#include <string>
#include <thread>
#include <vector>

#include "../../include/llama2_b200.h"

namespace l2 {

constexpr int BITS = 4;  // src/constants.rs:5

int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
void clear_error();

// Tensors of QTransformerWeights in file order (src/gptq.rs:36-65, export.py:94-119).
enum Tensor : int {
    T_RMS_EPS = 0, T_TOK_EMB, T_RMS_ATT, T_WQ, T_WK, T_WV, T_WO, T_RMS_FFN,
    T_W1, T_W2, T_W3, T_RMS_FINAL, T_FREQ_REAL, T_FREQ_IMAG, T_WCLS, T_COUNT
};
// Fields of one QLinear record in file order (src/gptq.rs:75-83).
enum Sub : int { S_QWEIGHT = 0, S_QZEROS, S_SCALES, S_GINDEX, S_DENSE };

inline bool is_qlinear(int t) { return t == T_WQ || t == T_WK || t == T_WV || t == T_WO || t == T_W1 || t == T_W2 || t == T_W3; }

struct Shape {
    l2_config c;
    int head_size() const { return c.dim / c.n_heads; }
    int kv_dim() const { return head_size() * c.n_kv_heads; }
    int attn_groups() const { return c.n_heads / c.n_kv_heads; }
    // (IN, OUT) of a QLinear tensor.
    void qdims(int t, int* in, int* out) const;
    static size_t groups(size_t in, size_t gs) { return in / gs + (in % gs ? 1 : 0); }  // int_div_up, src/gptq.rs:18-20
    // Words (4 bytes) of one field of one layer's record / of a dense tensor (all layers).
    size_t sub_words(int t, int sub) const;
    size_t qlinear_words(int t) const;
    size_t tensor_words(int t) const;  // whole tensor incl. all layers
    size_t tensor_offset_words(int t) const;
    size_t total_words() const;
    // Offset of field `sub` of layer `layer` of tensor `t`, in words from the payload start.
    size_t offset_words(int t, int layer, int sub) const;
};

int validate_config(const l2_config& c);

// Where the loader takes tensor data from: a mapped payload or the generator.
struct Source {
    virtual ~Source() {}
    // Returns a pointer to `words` words of (t, layer, sub); may use `scratch` as backing store.
    virtual const uint32_t* get(int t, int layer, int sub, std::vector<uint32_t>& scratch) = 0;
    // Rows rows[0..n) of QLinear tensor t, compactly: qw [n][in/8], sc [n][groups], zn [n][groups] (zero nibbles).
    virtual void get_rows(int t, int layer, const int32_t* rows, int n, uint32_t* qw, float* sc, uint8_t* zn) = 0;
};

struct BlobSource : Source {
    Shape shape;
    const uint32_t* base;
    BlobSource(const Shape& s, const void* payload) : shape(s), base(static_cast<const uint32_t*>(payload)) {}
    const uint32_t* get(int t, int layer, int sub, std::vector<uint32_t>&) override {
        return base + shape.offset_words(t, layer, sub);
    }
    void get_rows(int t, int layer, const int32_t* rows, int n, uint32_t* qw, float* sc, uint8_t* zn) override;
};

struct SynthSource : Source {
    Shape shape;
    uint64_t seed;
    int threads;
    SynthSource(const Shape& s, uint64_t sd, int th) : shape(s), seed(sd), threads(th) {}
    const uint32_t* get(int t, int layer, int sub, std::vector<uint32_t>& scratch) override;
    // generates only the requested rows (a tensor-parallel rank needs 1/T of every matrix)
    void get_rows(int t, int layer, const int32_t* rows, int n, uint32_t* qw, float* sc, uint8_t* zn) override;
};

// Fills `dst` with field `sub` of layer `layer` of tensor `t` of the seeded synthetic checkpoint.
void synth_tensor(const Shape& s, uint64_t seed, int t, int layer, int sub, uint32_t* dst, int threads);
// Words [first, first + count) of a QLinear field (S_QWEIGHT, S_QZEROS or S_SCALES), single-threaded.
void synth_range(const Shape& s, uint64_t seed, int t, int layer, int sub, size_t first, size_t count, uint32_t* dst);
int default_threads();

// Splits [0, n) into contiguous ranges and runs fn(begin, end) on `threads` host threads.
template <class F>
void parallel_for(size_t n, int threads, F fn) {
    if (threads <= 1 || n < 4096) { fn(size_t(0), n); return; }
    std::vector<std::thread> pool;
    size_t per = (n + threads - 1) / threads;
    for (int i = 0; i < threads; i++) {
        size_t b = std::min(n, per * i), e = std::min(n, per * (i + 1));
        if (b < e) pool.emplace_back([=] { fn(b, e); });
    }
    for (auto& t : pool) t.join();
}

}  // namespace l2
