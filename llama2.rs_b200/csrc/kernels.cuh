// Device-side parameter records and launch wrappers of the per-token kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

namespace l2 {

constexpr int HS = 128;  // head size of every Llama-2 model (src/constants.rs:70)

// Loop state of the token loop kept on the device so that the captured per-token graph
// can be replayed without host involvement (src/inference.rs:134-190: token, pos, next).
struct Ctl {
    int pos;                  // position fed to the next forward
    int token;                // token fed to the next forward
    int n_prompt;             // teacher-forced while pos < n_prompt (src/inference.rs:154-156)
    int force;                // >= 0: the next token is this one regardless of the logits
    float temperature;        // 0 = greedy
    int status;               // non-zero when a device-side check failed
    unsigned long long rng;   // Random.seed (src/util.rs:56-58)
    int last_next;            // last selected token
    int pad;
};

enum : int { EPI_STORE = 0, EPI_RESID = 1, EPI_SWIGLU = 2 };

constexpr int SK_THREADS = 512;            // one CTA per SM
constexpr int SK_WARPS = SK_THREADS / 32;
constexpr int SK_MAX_SLOTS = 16;           // ring slots of a CTA (upper bound)

// One 4-bit matrix in device layout (see repack.cpp) with its input vector.
struct SkSeg {
    const uint32_t* rec;  // [tile][group] unit records of 64*W + 20 words (see repack.cpp)
    const float* x;       // input in this matrix's K order (the producer scatters it); token kernel: tagged, see perm
    const float* nw;      // rmsnorm weight in the matrix's K order, or null
    const int* perm;      // token kernel: x is in natural order, element i of it belongs at position perm[i] of the K order (perm as packed
                          // 16-bit indices), and nw is in natural order too (null: x is in K order already)
};

// One fused dequant+GEMV problem of a launch.  nseg == 2 pairs w1 with w3 for SwiGLU.
struct SkJob {
    SkSeg seg[2];
    float* out;            // STORE/SWIGLU: result vector; RESID: residual stream, natural order
    float* sdst[3];        // RESID: copies of the new residual value ...
    const int* sidx[3];    // ... written at these positions (inverse act-order permutations)
    int rows, tiles, in, G;
    int cta0, ncta;        // CTAs [cta0, cta0+ncta) of the launch work on this job
    int tq, trem;          // tiles / ncta and tiles % ncta
    float rGs;             // 1 / (nseg * G)
    int epi, nscatter;
    // token kernel only: x / out / sdst point to (value, tag) pairs; the phases (indices into the phase
    // table) that write this job's inputs and the residual it adds to
    int in_phase[2], resid_phase;
    int bcast;  // tensor parallel token kernel: the results are stored into every rank's buffers, not only this one's
    int gather; // token kernel, two matrices on one input (w1, w3): seg[].perm are FORWARD 16-bit indices (position p of the K order reads
                // input perm[p]); the input is kept once in natural order and each matrix's digits are gathered from it
    int pad1;
};

struct alignas(16) SkParams {
    SkJob job[3];
    int njobs;
    float eps;
    // weights of the kernel that runs after this one: fetched into L2 while this one computes
    const void* next_ptr[6];
    size_t next_bytes[6];
    size_t next_slice[6];   // bytes of each range one CTA asks for (multiple of 16)
    int n_next;
    unsigned long long* trace;  // debug: 8 clock stamps per CTA, or null
    int* status;                // set non-zero when a bounded wait gives up, or null
    int chunk, slots;           // units per ring slot, ring slots per warp
    int debug_skip;             // debug: wait for the copies but skip the arithmetic
    int ptiles;                 // tiles the per-CTA sum buffer holds
};

// Batched QLinear on tcgen05 (gemm_tc.cu): out[m][o] for m < M tokens, 128 output rows per CTA.
struct TcParams {
    const uint32_t* rec;   // unit records of the matrix (see repack.cpp)
    const uint8_t* bimg;   // [G] blocks of [n][gs] signed digit bytes of the activations, swizzled, followed by [mpad] digit sums
                           // per token (f32): one contiguous block per group (act_quant_kernel)
    const float* oscale;   // [mpad] factor of the integer result per token
    float* out;            // [M][ldo]
    int* status;
    int tiles16, G, gs, rows;
    int m, mpad, n;        // tokens, tokens padded to a multiple of 16, n = 3 * mpad (three digits per token)
    int ldo, epi;
    int ksplit;            // > 1: the groups are split over gridDim.y CTAs; slice k stores part + k * kstride [m][rows]
    size_t kstride;
    float* part;
};

struct QuantParams {
    const float* x;        // [M][ldx] activations, natural order
    const int* perm;       // consumer's K order (g_index) or null
    const float* nw;       // rmsnorm weight in the consumer's K order, or null (no norm)
    uint8_t* bimg;         // [G] blocks of [n][gs] digit bytes + [mpad] digit sums (f32)
    float* oscale;         // [mpad]
    int in, gs, ldx, mpad, n;
    float eps;
};

struct RopeParams {
    float* q; const float* k; const float* v;   // [M][ldq], [M][ldkv]
    float* kc; float* vc;                        // this layer's caches
    const float* rope_cos; const float* rope_sin;
    const int* pos;                              // [M]
    int n_kv_heads, ldq, ldkv;
    int kv_stride;                               // floats between cache rows of consecutive positions (all kv heads of the model); 0 = n_kv_heads * 128
};

struct AttnBatchParams {
    const float* q; const float* kc; const float* vc;
    const int* pos;
    float* out;                                  // [M][ldo], natural order
    int n_kv_heads, ag, ldq, ldo;
    int kv_stride;                               // as in RopeParams
};

// Batched forward under tensor parallelism: a rank has computed columns [col0, col0 + ncols) of a [M][ld] buffer that every
// rank keeps at the same offset of its pool; the kernel stores them into every peer's copy, tells the peers and waits for theirs.
struct TpGatherParams {
    char* pool[8];              // every rank's pool (this rank's own included)
    size_t buf_off;             // the buffer inside a pool
    size_t flag_off;            // [world] 64-bit arrival counters inside a pool: flag[r] of rank q's pool is written by rank r
    unsigned long long* seq;    // device counter of exchanges made: the kernel takes the next number (the same on every rank, never repeated)
    unsigned* done;             // CTAs of this launch that have stored their part (left at zero)
    int* status;
    int rank, world, M, ld, col0, ncols;
};

struct EmbedParams {
    const float* table;   // [VOCAB][DIM]
    const Ctl* ctl;
    const int* prompt;    // device copy of the prompt ids
    float* x;             // residual stream, natural order
    float* sdst[3];
    const int* sidx[3];
    int dim, nscatter;
    int feed_prompt;      // 1: token = START at pos 0 else prompt[pos-1] (src/inference.rs:29-35)
    int vocab;
};

struct AttnParams {
    const float* q; const float* k; const float* v;  // raw projections of this position
    float* kc; float* vc;                            // this layer's caches [SEQ][KVH][HS]
    const float* rope_cos; const float* rope_sin;    // [SEQ][HS/2]
    const Ctl* ctl;
    float* part;                                     // [n_heads][max_split][HS+2] split partials
    unsigned* counter;                               // [n_kv_heads] arrival tickets
    float* out; const int* oidx;                     // attention output scattered into wo's K order (null: natural order)
    int n_kv_heads, ag, max_split, split_min;
    int pos_fixed;                                   // >= 0: use this position instead of ctl->pos
    int kvh0, n_kv_local;                            // tensor parallelism: this launch covers kv heads [kvh0, kvh0 + n_kv_local); 0 local = all
    int in_phase;                                    // token kernel only: q/k/v/out are (value, tag) pairs, written by this phase
    int bcast;                                       // tensor parallel token kernel: out goes to every rank
};

struct ClsParams {
    const float* w;       // [VOCAB][DIM] f32 (src/gptq.rs:65)
    const float* x;       // residual stream, natural order
    const float* nw;      // rms_final_weight
    float* logits;
    int rows, in;
    float eps;
    int in_phase;         // token kernel only: x is (value, tag) pairs written by this phase
    // Tensor parallelism over peer memory (token kernel only): this rank computes the logits of vocabulary rows
    // [row0, row0 + rows) and stores them as (value, tag) pairs into every rank's `tagged` array; null = all rows, plain floats.
    unsigned long long* tagged;
    int row0, pad;
};

struct SelectParams {
    const float* logits;
    Ctl* ctl;
    const int* prompt;
    int* out_tokens;      // [SEQ] next token chosen at each position
    int vocab;
    // Vocabulary-parallel classifier: the logits arrive as (value, tag) pairs from every rank; the selecting CTA polls
    // them and writes the plain array first (which the selection, and the host, then read).  null = plain already.
    const unsigned long long* tagged;
    int tagged_phase;     // phase that wrote them
    int collect_only;     // no selection: only the plain array (a forward pass that returns logits)
};

// ---- the whole token as one persistent kernel (token_kernel.cu) --------------------------------
// A token is a list of phases; all CTAs run every phase.  A phase polls the tagged values of the
// phases it depends on; only where barrier_after is set do the CTAs meet at a grid-wide barrier.
// A phase record is what the stand-alone kernel of the same name takes as parameters.
enum : int { PH_EMBED = 0, PH_GEMV1, PH_GEMV2, PH_ATTN, PH_CLS, PH_SELECT, PH_ADVANCE };

struct alignas(16) PhaseRec {
    int type;
    int barrier_after;   // all CTAs meet at a grid barrier after this phase (else the next phase polls its tagged inputs)
    int pad[2];
    union {
        SkParams sk;     // PH_GEMV1 (one matrix per job) / PH_GEMV2 (w1 with w3 + SwiGLU)
        AttnParams at;
        EmbedParams em;
        ClsParams cl;
        SelectParams se; // PH_SELECT; PH_ADVANCE uses se.ctl only
    } u;
};

constexpr int TK_TRACE_W = 32;  // debugging clock stamps per (CTA, phase)

struct TokenParams {
    const PhaseRec* phases;     // device table
    int nphases;
    unsigned* bar;              // bar[0]: arrivals at grid barriers (never reset), bar[32]: launches so far (tag epoch), bar[33]: barriers so far
    int* status;                // set non-zero when a bounded wait gives up
    const Ctl* ctl;             // loop state: the position of this token
    unsigned long long* trace;  // debug: [grid][nphases][TK_TRACE_W] stamps, or null
    int chunk, slots;           // ring geometry: unit records per slot, slots
    unsigned fixed_bytes;       // shared memory in front of the ring (digits, sums, scratch of the other phases)
    int skip;                   // debug: stream the weights but skip the GEMV arithmetic (results are wrong)
    // tensor parallelism over peer memory: every rank's pool of tagged activations (same layout everywhere, this
    // rank's own at pool[rank]); a phase that broadcasts stores at the same offset into each of them
    char* pool[8];
    int world, rank;
};

cudaError_t launch_token(const TokenParams& tk, int group_size, int attn_groups, int grid, size_t smem, cudaStream_t st);
cudaError_t token_set_poll_limit(unsigned polls);  // polls of a tagged input before giving up; 0 = default
cudaError_t token_init(int max_optin);     // max_optin: opt-in shared memory per block of the device
size_t token_attn_scratch_bytes(int ag);   // shared memory the attention phase needs
size_t token_gemv_smem(int in, int G, int nseg, int ptiles, bool natural, bool gather);  // shared memory a GEMV phase of the token kernel needs in front of the ring

void launch_embed(const EmbedParams& p, cudaStream_t st, bool pdl);
// `p` points to device memory: the kernel copies the record into shared memory with one cooperative load
cudaError_t launch_sk(const SkParams* p, int group_size, int nseg, int grid, size_t smem, cudaStream_t st, bool pdl);
size_t sk_smem_fixed(int in, int G, int nseg, int ptiles);  // digits, group sums, tile sums
size_t sk_slot_bytes(int group_size, int chunk);           // one ring slot of one warp
cudaError_t sk_init(int max_smem);
void launch_embed_batch(const float* table, const int* tokens, float* x, int dim, int M, cudaStream_t st);
void launch_act_quant(const QuantParams& p, int M, cudaStream_t st);
void launch_rope_append(const RopeParams& p, int n_heads, int M, cudaStream_t st);
void launch_attn_batch(const AttnBatchParams& p, int n_heads, int M, bool tiled, cudaStream_t st);
void launch_tp_gather(const TpGatherParams& p, cudaStream_t st);
void launch_swiglu(const float* h1, const float* h3, float* hb, int n, int ld, int M, cudaStream_t st);
// out[m][o] (+)= sum over the K slices, in slice order: finishes a GEMM whose groups were split over several CTAs
cudaError_t launch_gemm_tc(const TcParams& p, cudaStream_t st);
cudaError_t gemm_tc_init(int max_smem);
cudaError_t attn_batch_init();
void launch_ksum(const float* part, size_t kstride, int ksplit, float* out, int ldo, int rows, int M, int epi, cudaStream_t st);
size_t gemm_tc_smem_bytes(int gs, int n);
int gemm_tc_mpad(int tokens);  // tokens of a pass, padded to the granularity of the kernel's drain (16)
size_t gemm_tc_image_bytes(int in, int gs, int tokens);  // digit image of `tokens` activations rows for a matrix with IN = in
extern unsigned long long* g_sk_trace;  // device buffer for SkParams::trace when tracing is on
void launch_attn(const AttnParams& p, cudaStream_t st, bool pdl);
void launch_cls(const ClsParams& p, int grid, cudaStream_t st, bool pdl);
void launch_select(const SelectParams& p, cudaStream_t st, bool pdl);
void launch_advance(Ctl* ctl, cudaStream_t st, bool pdl);
// dst_i[idx_i[j]] = src[j] for j < n and up to three destinations (copies of a vector in consumers' K orders)
void launch_scatter(const float* src, int n, float* const* dst, const int* const* idx, int ndst, cudaStream_t st, bool pdl);
cudaError_t kernels_init();  // opt-in shared memory sizes; call once per device

extern unsigned long long g_launches;

}  // namespace l2
