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

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;
constexpr int GEMV_R = 4;  // output rows a warp accumulates at once (x registers are shared by them)

// One fused dequant+GEMV problem: out = W x for a 4-bit act-order QLinear in device layout.
// The input vector is already in the layer's permuted K order (the producer scatters it).
struct GemvJob {
    const uint4* qw;  const float* sc;  const uint32_t* zr;   // matrix A
    const uint4* qw2; const float* sc2; const uint32_t* zr2;  // matrix B (w3 of the SwiGLU pair) or null
    const float* x;   const float* nw;   // A's input in A's K order; rmsnorm weight in the same order or null
    const float* x2;  const float* nw2;  // B's input / norm weight in B's K order
    float* out;                          // STORE/SWIGLU: result vector; RESID: residual stream, natural order
    float* sdst[3];                      // RESID: copies of the new residual value ...
    const int* sidx[3];                  // ... written at these positions (inverse act-order permutations)
    int rows, in, gp, gshift;            // gshift = log2(group_size / 32)
    int cta0, ncta;                      // CTAs [cta0, cta0+ncta) of the launch work on this job
    int epi, nscatter;
    int ks;                              // warps that split K of one row block (power of two <= 8)
};

struct GemvParams {
    GemvJob job[3];
    int njobs;
    float eps;
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
};

struct ClsParams {
    const float* w;       // [VOCAB][DIM] f32 (src/gptq.rs:65)
    const float* x;       // residual stream, natural order
    const float* nw;      // rms_final_weight
    float* logits;
    int rows, in;
    float eps;
};

struct SelectParams {
    const float* logits;
    Ctl* ctl;
    const int* prompt;
    int* out_tokens;      // [SEQ] next token chosen at each position
    int vocab;
};

void launch_embed(const EmbedParams& p, cudaStream_t st, bool pdl);
void launch_gemv(const GemvParams& p, int grid, size_t smem, bool dual, cudaStream_t st, bool pdl);
size_t gemv_smem_bytes(int in, bool dual);
int gemv_ctas_per_sm(int in, bool dual);
void launch_attn(const AttnParams& p, cudaStream_t st, bool pdl);
void launch_cls(const ClsParams& p, int grid, cudaStream_t st, bool pdl);
void launch_select(const SelectParams& p, cudaStream_t st, bool pdl);
void launch_advance(Ctl* ctl, cudaStream_t st, bool pdl);
cudaError_t kernels_init();  // opt-in shared memory sizes; call once per device

extern unsigned long long g_launches;

}  // namespace l2
