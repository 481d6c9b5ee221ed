/*
 * CPU oracle for the llama2.rs token loop -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * See llama2_oracle.h for scope and parity status ("parity unpinned" by reference
 * golden vectors; pinned by derived known-answer cases).
 *
 * Arithmetic rules kept from the reference so that the only difference from the Rust
 * binary is the platform libm:
 *   - every multiply and add is a separate IEEE f32 operation (build with
 *     -ffp-contract=off; rustc never contracts to FMA),
 *   - QLinear keeps eight independent partial sums (lane j holds k = j mod 8) and adds
 *     the lanes once per output row, lane 0 first (std::simd reduce_sum on floats is an
 *     ordered reduction starting from 0.0),
 *   - every other reduction is a sequential left fold in index order.
 * Rows/heads are spread over OpenMP threads exactly where the reference uses rayon;
 * this does not change any result because no reduction crosses a thread.
 */
#define _GNU_SOURCE
#include "llama2_oracle.h"

#include <fcntl.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef float v8f __attribute__((vector_size(32)));
typedef int32_t v8i __attribute__((vector_size(32)));

#define BITS 4 /* src/constants.rs:5 */

typedef struct qlinear_view {
    const int32_t* qweight; /* [OUT][IN/8] */
    const int32_t* qzeros;  /* [OUT/8][GROUPS] */
    const float* scales;    /* [OUT][GROUPS] */
    const int32_t* g_index; /* [IN] */
    int in, out;
} qlinear_view;

struct orc_model {
    orc_config c;
    float rms_eps;
    const float* token_embedding_table;
    const float* rms_att_weight;
    qlinear_view *wq, *wk, *wv, *wo;
    const float* rms_ffn_weight;
    qlinear_view *w1, *w2, *w3;
    const float* rms_final_weight;
    const float* wcls;
    void* mapping; /* non-NULL when the model owns an mmap */
    size_t mapping_len;
};

struct orc_state {
    float* key_cache;
    float* value_cache;
    size_t n;
};

static double now_ms(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec * 1e3 + ts.tv_nsec * 1e-6;
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---- layout: src/gptq.rs:17-32 (int_div_up, bit_div) and :68-84 (QLinear) ---- */
static size_t int_div_up(size_t x, size_t y) { return x / y + (x % y == 0 ? 0 : 1); }
static size_t bit_div(size_t x) { return x / 32 * BITS; }

static size_t qlinear_words(size_t in, size_t out, size_t gs) {
    size_t groups = int_div_up(in, gs);
    return out * bit_div(in) + bit_div(out) * groups + out * groups + in;
}

static int head_size(const orc_config* c) { return c->dim / c->n_heads; }
static int kv_dim(const orc_config* c) { return head_size(c) * c->n_kv_heads; }

size_t orc_weights_bytes(const orc_config* c) {
    size_t D = c->dim, H = c->hidden_dim, L = c->n_layers, V = c->vocab_size, S = c->seq_len;
    size_t KV = kv_dim(c), G = c->group_size, HS = head_size(c);
    size_t w = 1;                                             /* rms_eps */
    w += V * D;                                               /* token_embedding_table */
    w += L * D;                                               /* rms_att_weight */
    w += L * (2 * qlinear_words(D, D, G) + 2 * qlinear_words(D, KV, G)); /* wq wk wv wo */
    w += L * D;                                               /* rms_ffn_weight */
    w += L * (2 * qlinear_words(D, H, G) + qlinear_words(H, D, G));      /* w1 w2 w3 */
    w += D;                                                   /* rms_final_weight */
    w += 2 * S * (HS / 2);                                    /* _freq_cis_real/imag */
    w += V * D;                                               /* wcls */
    return w * 4;
}

static const int32_t* take_qlinear(const int32_t* p, qlinear_view* q, size_t in, size_t out, size_t gs) {
    size_t groups = int_div_up(in, gs);
    q->in = (int)in;
    q->out = (int)out;
    q->qweight = p;
    p += out * bit_div(in);
    q->qzeros = p;
    p += bit_div(out) * groups;
    q->scales = (const float*)p;
    p += out * groups;
    q->g_index = p;
    p += in;
    return p;
}

orc_model* orc_model_map(const orc_config* c, const void* blob, size_t nbytes) {
    if (nbytes != orc_weights_bytes(c)) return NULL; /* src/lib.rs:97 */
    orc_model* m = (orc_model*)calloc(1, sizeof(orc_model));
    m->c = *c;
    size_t D = c->dim, H = c->hidden_dim, L = c->n_layers, V = c->vocab_size, S = c->seq_len;
    size_t KV = kv_dim(c), G = c->group_size, HS = head_size(c);
    qlinear_view* all = (qlinear_view*)calloc(7 * L, sizeof(qlinear_view));
    m->wq = all; m->wk = all + L; m->wv = all + 2 * L; m->wo = all + 3 * L;
    m->w1 = all + 4 * L; m->w2 = all + 5 * L; m->w3 = all + 6 * L;
    const int32_t* p = (const int32_t*)blob;
    m->rms_eps = *(const float*)p; p += 1;
    m->token_embedding_table = (const float*)p; p += V * D;
    m->rms_att_weight = (const float*)p; p += L * D;
    for (size_t l = 0; l < L; l++) p = take_qlinear(p, &m->wq[l], D, D, G);
    for (size_t l = 0; l < L; l++) p = take_qlinear(p, &m->wk[l], D, KV, G);
    for (size_t l = 0; l < L; l++) p = take_qlinear(p, &m->wv[l], D, KV, G);
    for (size_t l = 0; l < L; l++) p = take_qlinear(p, &m->wo[l], D, D, G);
    m->rms_ffn_weight = (const float*)p; p += L * D;
    for (size_t l = 0; l < L; l++) p = take_qlinear(p, &m->w1[l], D, H, G);
    for (size_t l = 0; l < L; l++) p = take_qlinear(p, &m->w2[l], H, D, G);
    for (size_t l = 0; l < L; l++) p = take_qlinear(p, &m->w3[l], D, H, G);
    m->rms_final_weight = (const float*)p; p += D;
    p += 2 * S * (HS / 2); /* _freq_cis_*: present, unused (src/gptq.rs:60-62) */
    m->wcls = (const float*)p; p += V * D;
    if ((size_t)((const char*)p - (const char*)blob) != nbytes) { orc_model_close(m); return NULL; }
    return m;
}

orc_model* orc_model_open(const char* path, int attn_groups, int group_size) {
    int fd = open(path, O_RDONLY);
    if (fd < 0) return NULL;
    struct stat st;
    int32_t h[7];
    if (fstat(fd, &st) != 0 || read(fd, h, sizeof h) != (ssize_t)sizeof h) { close(fd); return NULL; }
    /* Config::load: dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab(abs), seq_len.
     * The file's n_kv_heads field is ignored, as in the reference (src/constants.rs:94-100). */
    orc_config c;
    c.dim = h[0]; c.hidden_dim = h[1]; c.n_layers = h[2]; c.n_heads = h[3];
    c.n_kv_heads = h[3] / attn_groups;
    c.vocab_size = h[5] < 0 ? -h[5] : h[5];
    c.seq_len = h[6];
    c.group_size = group_size;
    size_t len = (size_t)st.st_size - sizeof h;
    void* map = mmap(NULL, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) return NULL;
    orc_model* m = orc_model_map(&c, (const char*)map + sizeof h, len);
    if (!m) { munmap(map, (size_t)st.st_size); return NULL; }
    m->mapping = map;
    m->mapping_len = (size_t)st.st_size;
    return m;
}

void orc_model_close(orc_model* m) {
    if (!m) return;
    if (m->mapping) munmap(m->mapping, m->mapping_len);
    free(m->wq);
    free(m);
}

const orc_config* orc_model_config(const orc_model* m) { return &m->c; }

orc_state* orc_state_new(const orc_model* m) {
    orc_state* s = (orc_state*)calloc(1, sizeof(orc_state));
    s->n = (size_t)m->c.n_layers * m->c.seq_len * kv_dim(&m->c);
    s->key_cache = (float*)calloc(s->n, sizeof(float));
    s->value_cache = (float*)calloc(s->n, sizeof(float));
    return s;
}
void orc_state_free(orc_state* s) {
    if (!s) return;
    free(s->key_cache);
    free(s->value_cache);
    free(s);
}
float* orc_state_key_cache(orc_state* s) { return s->key_cache; }
float* orc_state_value_cache(orc_state* s) { return s->value_cache; }

/* ---- QLinear::matvec<B>, src/gptq.rs:94-176 ---- */
#define MAX_B 64
void orc_qlinear_matvec(int in, int out, int group_size, const int32_t* qweight,
                        const int32_t* qzeros, const float* scales, const int32_t* g_index,
                        int B, const float* x, float* xout) {
    const int ing = in / 32 * BITS;          /* words per row */
    const int groups = (int)int_div_up(in, group_size);
    const int ipg = group_size / 32 * BITS;  /* words per group, :127 */
    const int elems_per_i32 = 32 / BITS;
    const int mask = (1 << BITS) - 1;
    /* :110-122 gather by g_index, then lay out as [IN/8][B] vectors of 8 consecutive k */
    v8f* x_temp = (v8f*)aligned_alloc(32, (size_t)(in / 8) * B * sizeof(v8f));
    for (int i = 0; i < in / 8; i++)
        for (int b = 0; b < B; b++) {
            v8f v;
            for (int j = 0; j < 8; j++) v[j] = x[(size_t)b * in + g_index[i * 8 + j]];
            x_temp[(size_t)i * B + b] = v;
        }
    const v8i shift_right = {0, 4, 8, 12, 16, 20, 24, 28};
#pragma omp parallel for schedule(static)
    for (int oi = 0; oi < out; oi++) { /* :132 */
        const int32_t* qz_row = qzeros + (size_t)(oi / elems_per_i32) * groups;
        const int out_elem = oi % elems_per_i32;
        const int32_t* qw_row = qweight + (size_t)oi * ing;
        v8f sum[MAX_B];
        for (int b = 0; b < B; b++) sum[b] = (v8f){0, 0, 0, 0, 0, 0, 0, 0};
        const int ngroups = ing / ipg < groups ? ing / ipg : groups; /* zip stops at the shortest */
        for (int g = 0; g < ngroups; g++) {
            const int qz = ((qz_row[g] >> (BITS * out_elem)) & mask) + 1; /* :148 */
            const float scale = scales[(size_t)oi * groups + g];
            const v8f scale_simd = {scale, scale, scale, scale, scale, scale, scale, scale};
            const v8i zero_simd = {qz, qz, qz, qz, qz, qz, qz, qz};
            for (int i = 0; i < ipg; i++) { /* :152 */
                const int32_t v = qw_row[g * ipg + i];
                const v8i num = {v, v, v, v, v, v, v, v};
                const v8i qw = (num >> shift_right) & mask; /* arithmetic shift, then mask */
                const v8f combine = __builtin_convertvector(qw - zero_simd, v8f);
                const v8f weight = scale_simd * combine;
                const v8f* xs = x_temp + (size_t)(g * ipg + i) * B;
                for (int b = 0; b < B; b++) sum[b] = sum[b] + weight * xs[b]; /* :160-162 */
            }
        }
        for (int b = 0; b < B; b++) { /* :166-168, ordered lane sum from 0.0 */
            float r = 0.0f;
            for (int j = 0; j < 8; j++) r = r + sum[b][j];
            xout[(size_t)b * out + oi] = 0.0f + r;
        }
    }
    free(x_temp);
}

/* ---- Linear::matvec<B>, src/model.rs:22-31 ---- */
void orc_linear_matvec(int in, int out, const float* w, int B, const float* x, float* xout) {
    for (int b = 0; b < B; b++) {
        const float* xb = x + (size_t)b * in;
#pragma omp parallel for schedule(static)
        for (int i = 0; i < out; i++) {
            const float* wr = w + (size_t)i * in;
            float acc = 0.0f;
            for (int k = 0; k < in; k++) acc = acc + wr[k] * xb[k];
            xout[(size_t)b * out + i] = acc;
        }
    }
}

/* ---- src/models.rs:47-98 ---- */
static void accum(float* a, const float* b, int n) { /* :47-51 */
    for (int i = 0; i < n; i++) a[i] += b[i];
}

void orc_rmsnorm(float* o, const float* x, const float* weight, int n, float eps) { /* :53-66 */
    float ss = 0.0f;
    for (int i = 0; i < n; i++) ss = ss + x[i] * x[i];
    ss /= (float)n;
    ss += eps;
    ss = 1.0f / sqrtf(ss);
    for (int j = 0; j < n; j++) o[j] = weight[j] * ss * x[j];
}

void orc_softmax(float* x, int n) { /* :68-81 */
    float max_val = x[0];
    for (int i = 0; i < n; i++) max_val = fmaxf(max_val, x[i]);
    float sum = 0.0f;
    for (int i = 0; i < n; i++) {
        x[i] = expf(x[i] - max_val);
        sum += x[i];
    }
    for (int i = 0; i < n; i++) x[i] /= sum;
}

static float dot(const float* q, const float* k, int n) { /* :83-89 */
    float s = 0.0f;
    for (int i = 0; i < n; i++) s = s + q[i] * k[i];
    return s;
}

void orc_silu(float* s, const float* s2, int n) { /* :92-98 */
    for (int i = 0; i < n; i++) {
        s[i] = s[i] * (1.0f / (1.0f + expf(-s[i])));
        s[i] = s[i] * s2[i];
    }
}

/* ---- rope, src/models.rs:100-129.  Rotate-half, updated in place: the second half
 * of each head reads the already rotated first half. ---- */
void orc_rope(float* queries, float* keys, int pos, int n_heads, int n_kv_heads, int hs) {
    for (int h = 0; h < n_heads; h++) {
        float* q = queries + (size_t)h * hs;
        for (int i = 0; i < hs; i++) {
            float freq = 1.0f / powf(10000.0f, ((float)(2 * i % hs)) / (float)hs);
            float val = (float)pos * freq;
            float fcr = cosf(val);
            float fci = sinf(val);
            if (i < hs / 2) q[i] = q[i] * fcr - q[hs / 2 + i] * fci;
            else            q[i] = q[i] * fcr + q[i - hs / 2] * fci;
            if (h < n_kv_heads) {
                float* k = keys + (size_t)h * hs;
                if (i < hs / 2) k[i] = k[i] * fcr - k[hs / 2 + i] * fci;
                else            k[i] = k[i] * fcr + k[i - hs / 2] * fci;
            }
        }
    }
}

/* ---- multihead_attention for one batch row, src/models.rs:131-176 ---- */
void orc_attention(float* out, const float* queries, const float* value_cache,
                   const float* key_cache, int pos, int n_heads, int n_kv_heads, int hs) {
    const int attn_groups = n_heads / n_kv_heads;
    const size_t row = (size_t)n_kv_heads * hs;
#pragma omp parallel for schedule(static)
    for (int h = 0; h < n_heads; h++) {
        const float* q = queries + (size_t)h * hs;
        float* xb = out + (size_t)h * hs;
        float* att = (float*)malloc(sizeof(float) * (size_t)(pos + 1));
        const float div = sqrtf((float)hs);
        for (int t = 0; t <= pos; t++) {
            const float* k = key_cache + (size_t)t * row + (size_t)(h / attn_groups) * hs;
            att[t] = dot(q, k, hs) / div; /* :158 */
        }
        orc_softmax(att, pos + 1);
        for (int i = 0; i < hs; i++) xb[i] = 0.0f;
        for (int t = 0; t <= pos; t++) {
            const float* v = value_cache + (size_t)t * row + (size_t)(h / attn_groups) * hs;
            for (int i = 0; i < hs; i++) xb[i] += att[t] * v[i];
        }
        free(att);
    }
}

static void qmatvec(const qlinear_view* w, int gs, int B, const float* x, float* xout) {
    orc_qlinear_matvec(w->in, w->out, gs, w->qweight, w->qzeros, w->scales, w->g_index, B, x, xout);
}

/* ---- transformer<B>, src/models.rs:178-298 ---- */
void orc_transformer(const orc_model* m, orc_state* s, int B, const int32_t* tokens,
                     const int32_t* pos, float* logits) {
    const orc_config* c = &m->c;
    const int D = c->dim, H = c->hidden_dim, KV = kv_dim(c), HS = head_size(c), G = c->group_size;
    const size_t layer_stride = (size_t)c->seq_len * KV;
    float* x = (float*)malloc(sizeof(float) * (size_t)B * D);
    float* xb = (float*)malloc(sizeof(float) * (size_t)B * D);
    float* xb2 = (float*)malloc(sizeof(float) * (size_t)B * D);
    float* q = (float*)malloc(sizeof(float) * (size_t)B * D);
    float* k = (float*)malloc(sizeof(float) * (size_t)B * KV);
    float* v = (float*)malloc(sizeof(float) * (size_t)B * KV);
    float* hb = (float*)malloc(sizeof(float) * (size_t)B * H);
    float* hb2 = (float*)malloc(sizeof(float) * (size_t)B * H);
    for (int b = 0; b < B; b++) /* :189-191 */
        memcpy(x + (size_t)b * D, m->token_embedding_table + (size_t)tokens[b] * D, sizeof(float) * D);
    for (int l = 0; l < c->n_layers; l++) {
        for (int b = 0; b < B; b++) /* :217-219 */
            orc_rmsnorm(xb + (size_t)b * D, x + (size_t)b * D, m->rms_att_weight + (size_t)l * D, D, m->rms_eps);
        qmatvec(&m->wq[l], G, B, xb, q); /* :224-226 */
        qmatvec(&m->wk[l], G, B, xb, k);
        qmatvec(&m->wv[l], G, B, xb, v);
        for (int b = 0; b < B; b++) /* :228-230 */
            orc_rope(q + (size_t)b * D, k + (size_t)b * KV, pos[b], c->n_heads, c->n_kv_heads, HS);
        float* kc = s->key_cache + (size_t)l * layer_stride;
        float* vc = s->value_cache + (size_t)l * layer_stride;
        for (int b = 0; b < B; b++) { /* :236-249, all rows stored before any attention */
            memcpy(kc + (size_t)pos[b] * KV, k + (size_t)b * KV, sizeof(float) * KV);
            memcpy(vc + (size_t)pos[b] * KV, v + (size_t)b * KV, sizeof(float) * KV);
        }
        for (int b = 0; b < B; b++) /* :250-256 */
            orc_attention(xb + (size_t)b * D, q + (size_t)b * D, vc, kc, pos[b], c->n_heads, c->n_kv_heads, HS);
        qmatvec(&m->wo[l], G, B, xb, xb2); /* :260 */
        for (int b = 0; b < B; b++) {      /* :263-267 */
            accum(x + (size_t)b * D, xb2 + (size_t)b * D, D);
            orc_rmsnorm(xb + (size_t)b * D, x + (size_t)b * D, m->rms_ffn_weight + (size_t)l * D, D, m->rms_eps);
        }
        qmatvec(&m->w1[l], G, B, xb, hb); /* :271-272 */
        qmatvec(&m->w3[l], G, B, xb, hb2);
        for (int b = 0; b < B; b++) orc_silu(hb + (size_t)b * H, hb2 + (size_t)b * H, H); /* :274-276 */
        qmatvec(&m->w2[l], G, B, hb, xb); /* :279 */
        for (int b = 0; b < B; b++) accum(x + (size_t)b * D, xb + (size_t)b * D, D); /* :283-285 */
    }
    if (B == 1) { /* :288-297 */
        orc_rmsnorm(xb, x, m->rms_final_weight, D, m->rms_eps);
        orc_linear_matvec(D, c->vocab_size, m->wcls, 1, xb, logits);
    }
    free(x); free(xb); free(xb2); free(q); free(k); free(v); free(hb); free(hb2);
}

/* ---- src/util.rs ---- */
int32_t orc_argmax(const float* v, int n) { /* :39-46: reduce keeps a only when a > b, so the last maximum wins */
    int best = 0;
    for (int i = 1; i < n; i++)
        if (!(v[best] > v[i])) best = i;
    return best;
}

uint32_t orc_random_u32(uint64_t* seed) { /* :71-77 xorshift* */
    uint64_t s = *seed;
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    *seed = s;
    return (uint32_t)((s * 0x2545F4914F6CDD1Dull) >> 32);
}

float orc_random_f32(uint64_t* seed) { /* :79-82 */
    return (float)(orc_random_u32(seed) >> 8) / 16777216.0f;
}

int32_t orc_sample(uint64_t* seed, const float* probabilities, int n) { /* :102-113 */
    float r = orc_random_f32(seed);
    float cdf = 0.0f;
    for (int i = 0; i < n; i++) {
        cdf += probabilities[i];
        if (r < cdf) return i;
    }
    return n - 1;
}

/* ---- prefill<A>, src/inference.rs:16-44 ---- */
static void prefill(int A, int* pos, orc_state* st, const int32_t* prompt, int n_prompt, const orc_model* m) {
    int32_t tokens[MAX_B], positions[MAX_B];
    while (*pos + A < n_prompt) {
        for (int i = 0; i < A; i++) {
            int32_t next = (*pos == 0) ? 1 /* START */ : prompt[*pos - 1];
            positions[i] = *pos;
            tokens[i] = next;
            *pos += 1;
        }
        orc_transformer(m, st, A, tokens, positions, NULL);
    }
}

/* ---- generate, src/inference.rs:49-193 ---- */
int orc_generate_ids(const orc_model* m, const int32_t* prompt, int n_prompt, int steps,
                     float temperature, uint64_t* rng_seed, int use_prefill,
                     int32_t* out_tokens, int32_t* out_pos0, float* logits_trace,
                     double* elapsed_ms, double* prefill_ms) {
    if (steps > m->c.seq_len) return -1;
    const int V = m->c.vocab_size;
    orc_state* st = orc_state_new(m); /* :59 fresh RunState per call */
    float* logits = (float*)malloc(sizeof(float) * (size_t)V);
    double start = now_ms(); /* :72 */
    int pos = 0;
    if (use_prefill) { /* :78-127 */
        static const int ladder[6] = {64, 32, 16, 8, 4, 2};
        for (int i = 0; i < 6; i++) prefill(ladder[i], &pos, st, prompt, n_prompt, m);
    }
    if (prefill_ms) *prefill_ms = now_ms() - start;
    if (out_pos0) *out_pos0 = pos;
    int32_t token = (pos == 0) ? 1 : prompt[pos - 1]; /* :128-132 */
    int n_out = 0;
    while (pos < steps) { /* :141 */
        int32_t p32 = pos;
        orc_transformer(m, st, 1, &token, &p32, logits);
        if (logits_trace) memcpy(logits_trace + (size_t)n_out * V, logits, sizeof(float) * (size_t)V);
        int32_t next;
        if (pos < n_prompt) {
            next = prompt[pos]; /* :154-156 */
        } else if (temperature == 0.0f) {
            next = orc_argmax(logits, V); /* :160-162 */
        } else {
            for (int q = 0; q < V; q++) logits[q] /= temperature; /* :164-173 */
            orc_softmax(logits, V);
            next = orc_sample(rng_seed, logits, V);
        }
        out_tokens[n_out++] = next;
        token = next;
        pos += 1;
    }
    if (elapsed_ms) *elapsed_ms = now_ms() - start;
    free(logits);
    orc_state_free(st);
    return n_out;
}
