// Seeded synthetic checkpoint in the export.py layout.  Stands in for real GPTQ weights:
// qweight nibbles U{0..15}, zero nibbles U{6..9}, scales U[0.002,0.02], act-order g_index
// from a seeded permutation, embeddings/classifier N(0,0.02), norm weights 1+N(0,0.02).
// Every value is a pure function of (seed, tensor, layer, field, index), so any tensor can
// be produced on its own and in parallel.  Host only.
#include <cmath>
#include <cstdio>
#include <cstring>

#include "host_common.h"
#include "repack.h"

namespace l2 {

static inline uint64_t mix64(uint64_t z) {  // splitmix64 finaliser
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

static inline uint64_t stream_key(uint64_t seed, int t, int layer, int sub) {
    return mix64(mix64(seed) ^ mix64(((uint64_t)t << 48) | ((uint64_t)sub << 40) | (uint64_t)(uint32_t)layer));
}
static inline uint64_t draw(uint64_t key, uint64_t idx) { return mix64(key + idx * 0xD1342543DE82EF95ull); }

static inline double normal(uint64_t key, uint64_t idx) {  // Box-Muller, one value per index
    const uint64_t h1 = draw(key, idx), h2 = mix64(h1);
    const double u1 = ((double)(h1 >> 11) + 1.0) * (1.0 / 9007199254740992.0);
    const double u2 = (double)(h2 >> 11) * (1.0 / 9007199254740992.0);
    return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586476925 * u2);
}

static void fill_normal(float* dst, size_t n, uint64_t key, double mean, double std_, int threads) {
    parallel_for(n, threads, [=](size_t b, size_t e) {
        for (size_t i = b; i < e; i++) dst[i] = (float)(mean + std_ * normal(key, i));
    });
}

// g_idx[k] = perm[k] / GS for a seeded permutation; the file stores stable_argsort(g_idx)
// (export.py:52,65): positions k listed group by group, ascending inside a group.
static void fill_gindex(int32_t* dst, int in, int gs, uint64_t key) {
    std::vector<int32_t> perm(in);
    for (int i = 0; i < in; i++) perm[i] = i;
    for (int i = in - 1; i > 0; i--) {  // Fisher-Yates
        int j = (int)(draw(key, (uint64_t)i) % (uint64_t)(i + 1));
        std::swap(perm[i], perm[j]);
    }
    const int groups = (int)Shape::groups(in, gs);
    std::vector<int> count(groups + 1, 0);
    for (int k = 0; k < in; k++) count[perm[k] / gs + 1]++;
    for (int g = 0; g < groups; g++) count[g + 1] += count[g];
    for (int k = 0; k < in; k++) dst[count[perm[k] / gs]++] = k;
}

void synth_range(const Shape& s, uint64_t seed, int t, int layer, int sub, size_t first, size_t count, uint32_t* dst) {
    (void)s;
    const uint64_t key = stream_key(seed, t, layer, sub);
    float* f = reinterpret_cast<float*>(dst);
    switch (sub) {
        case S_QWEIGHT:  // 8 i.i.d. nibbles per word
            for (size_t i = 0; i < count; i++) dst[i] = (uint32_t)(draw(key, first + i) >> 16);
            break;
        case S_QZEROS:
            for (size_t i = 0; i < count; i++) {
                const uint64_t h = draw(key, first + i);
                uint32_t w = 0;
                for (int j = 0; j < 8; j++) w |= (uint32_t)(6 + ((h >> (2 * j + 20)) & 3)) << (4 * j);
                dst[i] = w;
            }
            break;
        case S_SCALES:
            for (size_t i = 0; i < count; i++) {
                const float u = (float)(draw(key, first + i) >> 40) * (1.0f / 16777216.0f);
                f[i] = 0.002f + 0.018f * u;
            }
            break;
    }
}

void synth_tensor(const Shape& s, uint64_t seed, int t, int layer, int sub, uint32_t* dst, int threads) {
    const size_t n = s.sub_words(t, is_qlinear(t) ? sub : S_DENSE);
    const uint64_t key = stream_key(seed, t, layer, sub);
    float* f = reinterpret_cast<float*>(dst);
    if (is_qlinear(t)) {
        int in, out;
        s.qdims(t, &in, &out);
        switch (sub) {
            case S_QWEIGHT: case S_QZEROS: case S_SCALES:
                parallel_for(n, threads, [=, &s](size_t b, size_t e) { synth_range(s, seed, t, layer, sub, b, e - b, dst + b); });
                break;
            case S_GINDEX:
                fill_gindex(reinterpret_cast<int32_t*>(dst), in, s.c.group_size, key);
                break;
        }
        return;
    }
    switch (t) {
        case T_RMS_EPS: f[0] = 1e-5f; break;
        case T_TOK_EMB: case T_WCLS: fill_normal(f, n, key, 0.0, 0.02, threads); break;
        case T_RMS_ATT: case T_RMS_FFN: {
            // one stream per tensor: `layer` selects a row of [L][DIM] when a single layer is asked for
            const uint64_t k0 = stream_key(seed, t, 0, sub);
            fill_normal(f, n, k0, 1.0, 0.02, threads);
            break;
        }
        case T_RMS_FINAL: fill_normal(f, n, key, 1.0, 0.02, threads); break;
        case T_FREQ_REAL: case T_FREQ_IMAG: {  // export.py:15-21; present in the file, never read
            const int hs = s.head_size(), half = hs / 2;
            for (int p = 0; p < s.c.seq_len; p++)
                for (int i = 0; i < half; i++) {
                    const float freq = 1.0f / std::pow(10000.0f, (float)(2 * i) / (float)hs);
                    const float a = (float)p * freq;
                    f[(size_t)p * half + i] = t == T_FREQ_REAL ? std::cos(a) : std::sin(a);
                }
            break;
        }
    }
}

const uint32_t* SynthSource::get(int t, int layer, int sub, std::vector<uint32_t>& scratch) {
    const bool q = is_qlinear(t);
    const size_t n = shape.sub_words(t, q ? sub : S_DENSE);
    scratch.resize(n);
    synth_tensor(shape, seed, t, q ? layer : 0, q ? sub : S_DENSE, scratch.data(), threads);
    if (!q && (t == T_RMS_ATT || t == T_RMS_FFN)) {
        // callers ask for one layer's row; hand back a pointer into the full tensor
        return scratch.data() + (size_t)layer * shape.c.dim;
    }
    return scratch.data();
}

void BlobSource::get_rows(int t, int layer, const int32_t* rows, int n, uint32_t* qw, float* sc, uint8_t* zn) {
    int in, out;
    shape.qdims(t, &in, &out);
    gather_rows(in, shape.c.group_size, base + shape.offset_words(t, layer, S_QWEIGHT), base + shape.offset_words(t, layer, S_QZEROS),
                reinterpret_cast<const float*>(base + shape.offset_words(t, layer, S_SCALES)), rows, n, qw, sc, zn);
}

void SynthSource::get_rows(int t, int layer, const int32_t* rows, int n, uint32_t* qw, float* sc, uint8_t* zn) {
    int in, out;
    shape.qdims(t, &in, &out);
    const size_t g = Shape::groups(in, shape.c.group_size), wpr = in / 8;
    parallel_for((size_t)n, n * wpr >= 65536 ? threads : 1, [=](size_t b, size_t e) {
        std::vector<uint32_t> zw(g);
        for (size_t j = b; j < e; j++) {
            const size_t src = (size_t)rows[j];
            synth_range(shape, seed, t, layer, S_QWEIGHT, src * wpr, wpr, qw + j * wpr);
            synth_range(shape, seed, t, layer, S_SCALES, src * g, g, reinterpret_cast<uint32_t*>(sc + j * g));
            synth_range(shape, seed, t, layer, S_QZEROS, (src / 8) * g, g, zw.data());
            for (size_t k = 0; k < g; k++) zn[j * g + k] = (uint8_t)((zw[k] >> (4 * (src % 8))) & 15u);
        }
    });
}

}  // namespace l2

using namespace l2;

extern "C" int l2_synth_fill(const l2_config* c, uint64_t seed, void* payload, size_t nbytes, int threads) {
    clear_error();
    if (!c || !payload) return fail(L2_EINVAL, "l2_synth_fill: null argument");
    if (int rc = validate_config(*c)) return rc;
    Shape s{*c};
    if (nbytes != s.total_words() * 4)
        return fail(L2_EFORMAT, "l2_synth_fill: buffer is %zu bytes, checkpoint payload is %zu", nbytes, s.total_words() * 4);
    if (threads <= 0) threads = default_threads();
    uint32_t* base = static_cast<uint32_t*>(payload);
    for (int t = 0; t < T_COUNT; t++) {
        if (is_qlinear(t)) {
            for (int l = 0; l < c->n_layers; l++)
                for (int sub = S_QWEIGHT; sub <= S_GINDEX; sub++)
                    synth_tensor(s, seed, t, l, sub, base + s.offset_words(t, l, sub), threads);
        } else {
            synth_tensor(s, seed, t, 0, S_DENSE, base + s.tensor_offset_words(t), threads);
        }
    }
    return L2_OK;
}

extern "C" int l2_synth_write_file(const l2_config* c, uint64_t seed, const char* path, int threads) {
    clear_error();
    if (!c || !path) return fail(L2_EINVAL, "l2_synth_write_file: null argument");
    if (int rc = validate_config(*c)) return rc;
    Shape s{*c};
    if (threads <= 0) threads = default_threads();
    FILE* f = fopen(path, "wb");
    if (!f) return fail(L2_EIO, "cannot create %s", path);
    // Header as export.py:83-87 writes it: n_kv_heads repeats n_heads, vocab is negative.
    const int32_t header[7] = {c->dim, c->hidden_dim, c->n_layers, c->n_heads, c->n_heads, -c->vocab_size, c->seq_len};
    bool ok = fwrite(header, sizeof header, 1, f) == 1;
    std::vector<uint32_t> buf;
    auto put = [&](int t, int l, int sub, size_t n) {
        buf.resize(n);
        synth_tensor(s, seed, t, l, sub, buf.data(), threads);
        ok = ok && fwrite(buf.data(), 4, n, f) == n;
    };
    for (int t = 0; t < T_COUNT && ok; t++) {
        if (is_qlinear(t)) {
            for (int l = 0; l < c->n_layers && ok; l++)
                for (int sub = S_QWEIGHT; sub <= S_GINDEX; sub++) put(t, l, sub, s.sub_words(t, sub));
        } else {
            put(t, 0, S_DENSE, s.sub_words(t, S_DENSE));
        }
    }
    ok = (fclose(f) == 0) && ok;
    return ok ? L2_OK : fail(L2_EIO, "short write to %s", path);
}
