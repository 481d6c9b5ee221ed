/*
 * CPU oracle for the llama2.rs token loop -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the reference's CPU arithmetic (rayon + portable_simd in
 * the original; OpenMP + GCC 8-lane vectors here).  It is the checker the CUDA path
 * is compared against and the timed CPU baseline.  Only the test-suite, the smoke
 * check and the benchmark's CPU-baseline leg may load it; the product library never
 * links or calls it.
 *
 * Parity status: the reference's own tests assert nothing about this path and the
 * reference (nightly Rust) cannot be compiled in this environment, so the oracle is
 * pinned only by known-answer vectors derived from the constant fixtures in the
 * reference's src/gptq_test.rs:40-62 and src/kernel.py:100-103 and by an independent
 * dequantise-then-matmul check: "parity unpinned" by reference golden vectors.
 *
 * Every function cites the reference file:line it follows.
 */
#ifndef LLAMA2_ORACLE_H
#define LLAMA2_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* src/constants.rs:7-74 -- the compile-time constants of the reference, as a run-time record. */
typedef struct orc_config {
    int32_t dim;        /* DIM */
    int32_t hidden_dim; /* HIDDEN_DIM */
    int32_t n_layers;   /* N_LAYERS */
    int32_t n_heads;    /* N_HEADS */
    int32_t n_kv_heads; /* N_HEADS / ATTN_GROUPS */
    int32_t vocab_size; /* VOCAB_SIZE */
    int32_t seq_len;    /* SEQ_LEN */
    int32_t group_size; /* GROUPSIZE */
} orc_config;

typedef struct orc_model orc_model; /* view over a weights blob (src/gptq.rs:34-66) */
typedef struct orc_state orc_state; /* RunState (src/models.rs:29-42) */

/* size_of::<QTransformerWeights>() for this configuration (src/gptq.rs:34-84). */
size_t orc_weights_bytes(const orc_config* c);

/* LlamaModel::from_file's pointer cast (src/lib.rs:95-98): the blob is the file
 * contents after the 28-byte header.  Returns NULL when nbytes != orc_weights_bytes. */
orc_model* orc_model_map(const orc_config* c, const void* blob, size_t nbytes);

/* LlamaModel::from_file (src/lib.rs:88-104) + Config::load (src/constants.rs:102-119).
 * attn_groups and group_size are compile-time features in the reference and are not
 * stored in the file, so the caller supplies them. Returns NULL on any mismatch. */
orc_model* orc_model_open(const char* path, int attn_groups, int group_size);
void orc_model_close(orc_model* m);
const orc_config* orc_model_config(const orc_model* m);

orc_state* orc_state_new(const orc_model* m); /* RunState::new, zeroed caches */
void orc_state_free(orc_state* s);
float* orc_state_key_cache(orc_state* s);   /* [L][SEQ][KVH][HS] */
float* orc_state_value_cache(orc_state* s); /* [L][SEQ][KVH][HS] */

/* QLinear::matvec<B> (src/gptq.rs:94-176). x [B][IN], xout [B][OUT]. */
void orc_qlinear_matvec(int in, int out, int group_size, const int32_t* qweight,
                        const int32_t* qzeros, const float* scales, const int32_t* g_index,
                        int B, const float* x, float* xout);
/* Linear::matvec<B> (src/model.rs:22-31). w [OUT][IN]. */
void orc_linear_matvec(int in, int out, const float* w, int B, const float* x, float* xout);

void orc_rmsnorm(float* o, const float* x, const float* weight, int n, float eps); /* src/models.rs:53-66 */
void orc_softmax(float* x, int n);                                                  /* src/models.rs:68-81 */
void orc_silu(float* s, const float* s2, int n);                                    /* src/models.rs:92-98 */
void orc_rope(float* q, float* k, int pos, int n_heads, int n_kv_heads, int head_size); /* src/models.rs:100-129 */
/* multihead_attention for one batch row (src/models.rs:131-176). caches are one layer: [SEQ][KVH][HS]. */
void orc_attention(float* out, const float* q, const float* value_cache, const float* key_cache,
                   int pos, int n_heads, int n_kv_heads, int head_size);

/* transformer<B> (src/models.rs:178-298). logits [VOCAB] written only when B == 1. */
void orc_transformer(const orc_model* m, orc_state* s, int B, const int32_t* tokens,
                     const int32_t* pos, float* logits);

int32_t orc_argmax(const float* v, int n);                             /* src/util.rs:39-46 */
uint32_t orc_random_u32(uint64_t* seed);                               /* src/util.rs:71-77 */
float orc_random_f32(uint64_t* seed);                                  /* src/util.rs:79-82 */
int32_t orc_sample(uint64_t* seed, const float* probabilities, int n); /* src/util.rs:102-113 */

/* generate (src/inference.rs:49-193) on token ids instead of text: the prompt ids
 * stand where `bpe_encode(" " + prompt)` stands in the reference.  out_tokens
 * receives the `next` token of every B=1 loop iteration (teacher-forced ones too),
 * out_pos0 the position of the first such iteration; logits_trace (may be NULL) gets
 * the raw logits of every B=1 iteration, [n_out][VOCAB].  use_prefill selects
 * LlamaModel::prefill() (src/lib.rs:84-86).  Returns the number of tokens written,
 * or -1 when steps exceeds SEQ_LEN (the reference would index out of bounds). */
int orc_generate_ids(const orc_model* m, const int32_t* prompt, int n_prompt, int steps,
                     float temperature, uint64_t* rng_seed, int use_prefill,
                     int32_t* out_tokens, int32_t* out_pos0, float* logits_trace,
                     double* elapsed_ms, double* prefill_ms);

int orc_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif
