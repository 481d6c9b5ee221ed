/*
 * llama2_b200 -- C ABI of the B200-native llama2.rs token loop.
 *
 * Every entry point replaces one seam of the reference crate (file:line given per
 * declaration, paths relative to the reference project).  All functions return 0 on
 * success and a negative L2_E* code on failure; l2_last_error() gives the message of
 * the calling thread's last failure.  No exception or abort crosses this boundary.
 *
 * There is no CPU fallback: every compute entry point fails with L2_ECUDA when no
 * CUDA device is usable.
 *
 * Threading: one host thread per model handle; all device work of a handle runs on
 * one CUDA stream; calls on one handle are not re-entrant.
 */
#ifndef LLAMA2_B200_H
#define LLAMA2_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define L2_OK 0
#define L2_EINVAL (-1)   /* bad argument */
#define L2_EFORMAT (-2)  /* checkpoint header / size mismatch (check_static, mmap length assert) */
#define L2_ECUDA (-3)    /* CUDA runtime failure or no device */
#define L2_EIO (-4)      /* file could not be opened / read / written */
#define L2_ERANGE (-5)   /* position / steps beyond SEQ_LEN, token beyond VOCAB_SIZE */
#define L2_ESTATUS (-6)  /* a device-side bounded wait gave up (status word set): the launch left early, its results are not
                            valid, and the run state refuses further calls until l2_state_reset (which also evens out the
                            kernel's barrier count).  Under tensor parallelism every rank of the group must reset. */

#define L2_START 1 /* src/tokenizer.rs:10 */
#define L2_RET 13  /* src/tokenizer.rs:11 */

/* The reference's compile-time constants (src/constants.rs:7-74) as a run-time record. */
typedef struct l2_config {
    int32_t dim;        /* DIM */
    int32_t hidden_dim; /* HIDDEN_DIM */
    int32_t n_layers;   /* N_LAYERS */
    int32_t n_heads;    /* N_HEADS */
    int32_t n_kv_heads; /* N_HEADS / ATTN_GROUPS */
    int32_t vocab_size; /* VOCAB_SIZE */
    int32_t seq_len;    /* SEQ_LEN */
    int32_t group_size; /* GROUPSIZE: 32 | 64 | 128 */
} l2_config;

/* What the reference fixes with cargo features (Cargo.toml:28-43, build.rs:5-43). */
typedef struct l2_options {
    const char* model_size; /* "7B" | "13B" | "70B"; NULL = take the shape from the file header and attn_groups below */
    int32_t group_size;     /* group_32 | group_64 | group_128 */
    int32_t attn_groups;    /* ATTN_GROUPS when model_size is NULL (1 = no GQA) */
    int32_t device;         /* CUDA device ordinal, -1 = current device */
    int32_t debug;          /* print the configuration, as LlamaModel::from_file(debug=true) does */
    int32_t max_batch;      /* largest B accepted by l2_forward / prefill chunk (0 = default 64) */
    int32_t flags;          /* L2_FLAG_* */
    int32_t tp_rank;        /* tensor parallelism: this process's rank ... */
    int32_t tp_world;       /* ... of tp_world processes, one per GPU of the box (0 or 1 = single GPU) */
    int32_t poll_limit_log2; /* one-kernel-per-token path: log2 of the polls of an input another CTA (or rank) writes before the
                                kernel gives up and the call returns L2_ESTATUS; 0 = default (20, about a second); 8..30.
                                One value per device and process: the model opened last sets it. */
} l2_options;

#define L2_FLAG_NO_GRAPH 1 /* launch kernels directly instead of replaying the per-token CUDA graph */
#define L2_FLAG_NO_PDL 2   /* do not use programmatic dependent launch between the kernels of a token */
#define L2_FLAG_NO_L2_PREFETCH 4 /* do not prefetch the next kernel's weights into L2 */
#define L2_FLAG_NO_TOKEN_KERNEL 8 /* one launch per operator instead of one persistent kernel per token */

typedef struct l2_model l2_model;     /* LlamaModel (src/lib.rs:28-36, 68-77) */
typedef struct l2_state l2_state;     /* RunState (src/models.rs:29-42) */
typedef struct l2_qlinear l2_qlinear; /* QLinearCuda (src/gptq_cuda.rs:93-110) */
typedef struct l2_tokenizer l2_tokenizer; /* Tokenizer (src/tokenizer.rs:13-19) */

const char* l2_last_error(void);
/* Kernels launched by this library in this process so far (graph replays count their nodes). */
uint64_t l2_launch_count(void);

/* ---- shapes and checkpoint format ------------------------------------------------ */

/* The constants module selected by the 7B/13B/70B features (src/constants.rs:7-41). */
int l2_preset_config(const char* model_size, int group_size, l2_config* out);
/* size_of::<QTransformerWeights>() (src/gptq.rs:34-84): payload bytes after the 28-byte header. */
size_t l2_checkpoint_bytes(const l2_config* c);

/* Seeded synthetic checkpoint in the export.py layout (export.py:83-119): nibbles U{0..15},
 * zero nibbles U{6..9}, scales U[0.002,0.02], act-order g_index from a seeded permutation,
 * embeddings/classifier N(0,0.02), norm weights 1+N(0,0.02).  Host only. */
int l2_synth_fill(const l2_config* c, uint64_t seed, void* payload, size_t nbytes, int threads);
int l2_synth_write_file(const l2_config* c, uint64_t seed, const char* path, int threads);

/* ---- model handle: LlamaModel::from_file (src/lib.rs:45-63, 88-104) ----------------- */

int l2_model_open(const char* checkpoint, const l2_options* opt, l2_model** out);
/* The same on the bytes that follow the header (what the reference mmaps at offset 28). */
int l2_model_open_blob(const l2_config* c, const void* payload, size_t nbytes,
                       const l2_options* opt, l2_model** out);
/* Generates the l2_synth_fill checkpoint tensor by tensor straight into device memory. */
int l2_model_open_synthetic(const l2_config* c, uint64_t seed, const l2_options* opt, l2_model** out);
void l2_model_close(l2_model* m);
int l2_model_config(const l2_model* m, l2_config* out);
/* LlamaModel::prefill() (src/lib.rs:41-43, 84-86): 1, batched prefill is supported. */
int l2_model_prefill(const l2_model* m);
/* Run this handle's device work on a caller-owned cudaStream_t (NULL = the handle's own). */
int l2_model_set_stream(l2_model* m, void* cuda_stream);
/* Packed weight bytes one decode token must stream: all QLinear qweight+qzeros+scales,
 * the f32 classifier and the norm weights. */
uint64_t l2_model_decode_bytes(const l2_model* m);

/* ---- tensor parallelism (no counterpart in the reference, which is single-device) ------------
 * One process per GPU.  Every QLinear is split by output rows (tp_world must divide the kv heads
 * and leave whole 16-row tiles); vectors are re-assembled with NCCL all-gathers inside the token
 * graph.  Rank 0 makes an id with l2_tp_unique_id, the host program hands the 128 bytes to every
 * rank (torch.distributed, MPI, a file ...), and every rank calls l2_model_tp_connect on its model
 * (opened with tp_rank / tp_world set) before the first forward. */
int l2_tp_unique_id(void* id128);
int l2_model_tp_connect(l2_model* m, const void* id128);
/* Rows [row0, row0 + nrows) of a matrix of total_rows rows owned by `rank`. */
int l2_tp_rows(int total_rows, int rank, int world, int* row0, int* nrows);
/* Tensor parallelism without NCCL on the token path: every rank makes a pool for the activations that cross
 * ranks (l2_model_tp_pool_handle returns its 64-byte CUDA IPC handle), the host hands every rank's handle to
 * every other rank, and each rank maps them with l2_model_tp_pool_attach(rank, handle).  Once all tp_world
 * pools are attached, the first run state of the model runs its B=1 forwards as the one-kernel-per-token
 * path, whose epilogues store straight into every rank's pool over NVLink (no collective, no barrier); all
 * ranks must make the same calls in the same order.  Without this the NCCL path above is used.
 * No counterpart in the reference (which has no multi-GPU path). */
int l2_model_tp_pool_handle(l2_model* m, void* handle64);
int l2_model_tp_pool_attach(l2_model* m, int rank, const void* handle64);
/* Bytes of a rank's pool, and attaching a pool by device pointer instead of by IPC handle: for a rank whose pool lives in
 * this process (several GPUs driven by one process with peer access enabled by the caller, or a buffer that stands in for a
 * rank that never runs, as the bounded-wait tests use).  The memory must stay valid until the model is closed. */
size_t l2_model_tp_pool_bytes(const l2_model* m);
int l2_model_tp_pool_attach_ptr(l2_model* m, int rank, void* device_ptr);

/* ---- run state: RunState::new (src/models.rs:36-41) --------------------------------- */

int l2_state_new(l2_model* m, l2_state** out); /* device-resident KV cache, zeroed */
int l2_state_reset(l2_state* s);               /* zero the caches and rewind to position 0 */
void l2_state_free(l2_state* s);
/* Debug read-back of one layer's caches, [SEQ][KVH][HS] each (either pointer may be NULL). */
int l2_state_read_kv(l2_state* s, int layer, float* key_cache, float* value_cache);

/* ---- forward pass: transformer<B> (src/models.rs:178-298) ---------------------------- */

/* tokens[B], pos[B] host arrays; logits (host, VOCAB floats) is written only when B == 1
 * and may be NULL. */
int l2_forward(l2_model* m, l2_state* s, const int32_t* tokens, const int32_t* pos, int B, float* logits);

/* ---- token loop: prefill<A> + generate (src/inference.rs:16-193) --------------------- */

/* The prefill ladder (src/inference.rs:78-127): feeds [START, prompt...] positions in
 * chunks while pos + chunk < n_prompt and returns the first position left to the B=1
 * loop.  The ladder 64/32/16/8/4/2 is used when chunk == 0. */
int l2_prefill(l2_model* m, l2_state* s, const int32_t* prompt, int n_prompt, int chunk, int32_t* pos_out);

/* One iteration of the decode loop (src/inference.rs:141-190) with the host in the loop:
 * forward at `pos`, then next = forced_next if >= 0, else argmax (temperature == 0) or
 * a temperature sample drawn with *rng_seed (src/util.rs:71-113). */
int l2_decode_step(l2_model* m, l2_state* s, int32_t token, int32_t pos, float temperature,
                   uint64_t* rng_seed, int32_t forced_next, int32_t* next, float* logits);

/* Positions [pos0, steps) of the decode loop without host round trips: token selection
 * stays on the device and the per-token graph is replayed back to back.  out_tokens gets
 * steps - pos0 ids (teacher-forced ones included). */
int l2_decode_run(l2_model* m, l2_state* s, const int32_t* prompt, int n_prompt, int32_t pos0,
                  int32_t steps, float temperature, uint64_t* rng_seed, int32_t* out_tokens);

/* generate() on token ids (the reference takes text and encodes it, src/inference.rs:62-67).
 * A fresh RunState is used, as in the reference (src/inference.rs:59).  logits_trace
 * (NULL or [n_out][VOCAB]) forces one host round trip per token.  elapsed/prefill/decode
 * times are device times in ms.  Returns the number of tokens written or a negative code. */
int l2_generate_ids(l2_model* m, const int32_t* prompt, int n_prompt, int steps, float temperature,
                    uint64_t* rng_seed, int use_prefill, int32_t* out_tokens, int32_t* out_pos0,
                    float* logits_trace, double* elapsed_ms, double* prefill_ms, double* decode_ms);

/* ---- one quantised linear layer: QLinear::matvec<B> (src/gptq.rs:94-176,
 *      src/gptq_cuda.rs:50-90, 120-179) ---------------------------------------------- */

/* Arrays are host pointers in the checkpoint layout: qweight [OUT][IN/8] i32,
 * qzeros [OUT/8][GROUPS] i32, scales [OUT][GROUPS] f32, g_index [IN] i32. */
int l2_qlinear_create(int in, int out, int group_size, const int32_t* qweight, const int32_t* qzeros,
                      const float* scales, const int32_t* g_index, int device, l2_qlinear** h);
/* x [B][IN] -> xout [B][OUT], host f32 buffers; copies to and from the device inside the call. */
int l2_qlinear_matvec(l2_qlinear* h, const float* x, float* xout, int B);
/* The same on device buffers, enqueued on cuda_stream (no copies, no synchronisation). */
int l2_qlinear_matvec_dev(l2_qlinear* h, const float* x_dev, float* xout_dev, int B, void* cuda_stream);
void l2_qlinear_free(l2_qlinear* h);

/* ---- attention of one position (src/models.rs:100-176, 236-249) on device buffers --------- */

/* The RoPE cos/sin table of the reference's formula (src/models.rs:107-110), [seq_len][64] each; host. */
int l2_rope_table(int seq_len, float* cos_out, float* sin_out);
/* Bytes of device scratch l2_attention_decode_dev needs (split partials and arrival tickets). */
size_t l2_attention_workspace_bytes(int n_heads, int n_kv_heads);
/* rope(q, k, pos); key_cache[pos] = k; value_cache[pos] = v; out = multihead_attention(q, caches, pos)
 * for head size 128.  All pointers are device memory: q/out [n_heads*128], k/v [n_kv_heads*128],
 * caches [SEQ][n_kv_heads][128] of one layer, rope tables from l2_rope_table, workspace from the
 * caller (contents need not be kept between calls).  Enqueued on cuda_stream, no synchronisation. */
int l2_attention_decode_dev(int n_heads, int n_kv_heads, int pos, const float* q, const float* k, const float* v,
                            float* key_cache, float* value_cache, const float* rope_cos, const float* rope_sin,
                            float* out, void* workspace, size_t workspace_bytes, void* cuda_stream);

/* The same computation for callers that cannot allocate device memory (no counterpart in the
 * reference).  Takes no workspace: the split-sequence scratch is a fixed array inside the library
 * (about 1.1 MB held on every GPU that loads it, until the process exits), which limits it to
 * 64 query heads and 64 kv heads; larger shapes are rejected with L2_EINVAL.  Calls no cudaMalloc,
 * cudaFree or other allocating routine.  The device is the current one.  The first call on a
 * device looks up the array's address: make it before any stream capture.  All calls on a device
 * share the array: calls that overlap on the GPU race and must be serialised by the caller. */
int l2_attention_decode_noalloc(int n_heads, int n_kv_heads, int pos, const float* q, const float* k, const float* v,
                                float* key_cache, float* value_cache, const float* rope_cos, const float* rope_sin,
                                float* out, void* cuda_stream);

/* ---- measurement hooks (no counterpart in the reference, which times whole runs only,
 *      src/main.rs:61-65) --------------------------------------------------------------- */
/* Enqueue `count` launches of one projection kernel of the token forward, cycling through the
 * layers from layer0, on the model's stream; the caller brackets them with events.
 * which: 0 wq/wk/wv, 1 wo, 2 w1/w3+SwiGLU, 3 w2, 4 classifier, 5 attention. */
int l2_bench_projection(l2_model* m, l2_state* s, int which, int layer0, int count);
/* Algorithmic bytes one such launch streams (qweight+qzeros+scales, or the f32 classifier). */
uint64_t l2_projection_bytes(const l2_model* m, int which);

/* Debug: per-CTA clock stamps of the GEMV kernels (8 per CTA); enable != 0 turns tracing on for
 * launches planned afterwards, host_out (may be NULL) receives the stamps of the last launch. */
int l2_debug_trace(int enable, unsigned long long* host_out, int n_ctas);

/* Debug: clock stamps of the one-kernel-per-token path; they are written only by a library built
 * with -DL2_TK_TRACE (L2_TK_TRACE=1 for build.py), a default build leaves the buffer zero.
 * enable = 1 arms recording into a device buffer of `count` stamps (needs SMs x phases x 16);
 * enable = 0 copies the first `count` stamps to host_out, laid out [CTA][phase][16]: SM clock at
 * phase start, inputs staged, main loop done, phase left; global nanosecond timer at phase start,
 * phase end, phase left; SM clock at phase end; the rest are per-phase details.
 * No counterpart in the reference. */
int l2_debug_token_trace(l2_state* s, int enable, unsigned long long* host_out, size_t count);

/* ---- sampling helpers (src/util.rs:39-46, 71-113) ----------------------------------- */
uint32_t l2_random_u32(uint64_t* seed);
float l2_random_f32(uint64_t* seed);

/* ---- tokenizer (src/tokenizer.rs:22-108, src/util.rs:29-37,116-123); host only ------- */
int l2_tokenizer_open(const char* filename, int vocab_size, l2_tokenizer** out);
void l2_tokenizer_free(l2_tokenizer* t);
/* bpe_encode: returns the number of ids (written up to cap), or a negative code. */
int l2_tokenizer_encode(const l2_tokenizer* t, const char* text, int32_t* ids, int cap);
/* vocab[id] as a NUL-terminated UTF-8 string owned by the tokenizer. */
const char* l2_tokenizer_vocab(const l2_tokenizer* t, int32_t id);
/* get_token (src/util.rs:116-123): strips one leading space after START. */
const char* l2_tokenizer_piece(const l2_tokenizer* t, int32_t prev, int32_t next);

/* ---- host-side repack, exposed so that it can be checked without a GPU --------------- */
/* Device layout of one QLinear as built at load time: [tiles][groups] unit records of unit_words
 * 32-bit words each (tiles of 16 rows, one quantisation group): 2*32*(GS/32) weight words in lane
 * order, 16 f32 scales, 2 words of zero nibbles, 2 words of padding.  Returns a malloc'ed array the
 * caller frees with l2_host_free.  rows_order (NULL or [OUT]) re-orders output rows. */
int l2_debug_repack(int in, int out, int group_size, const int32_t* qweight, const int32_t* qzeros,
                    const float* scales, const int32_t* rows_order, uint32_t** rec_dev, int* tiles,
                    int* unit_words);
void l2_host_free(void* p);

#ifdef __cplusplus
}
#endif
#endif
