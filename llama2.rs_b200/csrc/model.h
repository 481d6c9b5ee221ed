// Host-side model / run-state records behind the C ABI handles.
#pragma once

#include <cuda_runtime.h>

#include <memory>
#include <vector>

#include "host_common.h"
#include "kernels.cuh"
#include "repack.h"

namespace l2 {

#define L2_CUDA(expr)                                                                              \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess)                                                                     \
            return ::l2::fail(L2_ECUDA, "%s: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
    } while (0)

// One QLinear in device layout (see repack.cpp) plus what its producers/consumers need.
struct DevQ {
    uint32_t* rec = nullptr;   // [tiles][G] unit records: weights, scales, zero nibbles (see repack.cpp)
    int* perm = nullptr;  // g_index: permuted position j reads input perm[j]
    int* inv = nullptr;   // inverse: input o is written to permuted position inv[o]
    uint16_t* perm16 = nullptr;  // perm as 16-bit indices
    uint16_t* inv16 = nullptr;   // inv as 16-bit indices (IN < 65536): where the token kernel puts input o when it brings a vector into K order
    int in = 0, out = 0, tiles = 0, G = 0, gs = 0;  // out / tiles: the rows held by this process
    int row0 = 0;                                   // first row held (tensor parallelism), else 0
};

// A planned GEMV launch: parameters, grid and shared memory.
struct SkLaunch {
    SkParams p{};
    int grid = 0, nseg = 1, gs = 128;
    size_t smem = 0;
};

struct DevLayer {
    DevQ wq, wk, wv, wo, w1, w2, w3;
    float *nw_q = nullptr, *nw_k = nullptr, *nw_v = nullptr;  // rms_att_weight in each consumer's K order
    float *nw_1 = nullptr, *nw_3 = nullptr;                   // rms_ffn_weight likewise
    float *rms_att = nullptr, *rms_ffn = nullptr;             // the two norm weights in natural order (token kernel)
};

constexpr int CTL_RING = 128;
constexpr int L2_MAX_TP = 8;   // ranks of a tensor-parallel group (the GPUs of one box)
constexpr int MAX_BATCH = 64;  // tokens of one batched forward (one tcgen05 accumulator holds 3 digits x 64 tokens = 192 columns)

// Device buffers of the batched forward pass (transformer<B>, B >= 2).
struct BatchBuffers {
    float *x = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *h1 = nullptr, *h3 = nullptr, *hb = nullptr;
    float* kpart[3] = {nullptr, nullptr, nullptr};  // [4][tokens][rows] partial results of GEMMs whose groups are split over CTAs, one per stream
    uint8_t* img[3] = {nullptr, nullptr, nullptr};  // digit images (with the digit sums) of up to three consumers
    float* osc[3] = {nullptr, nullptr, nullptr};
    int *tok = nullptr, *pos = nullptr;             // device token ids / positions of the batch
    int* h_stage = nullptr;                         // pinned ring for their upload
    int stage_slot = 0;
    // independent projections of a layer (wq/wk/wv, w1/w3) run side by side on two more streams
    cudaStream_t aux[2] = {nullptr, nullptr};
    cudaEvent_t fork = nullptr, join[2] = {nullptr, nullptr};
    bool tp = false;          // tensor parallel over peer memory: x, att and hb live in the model's pool, the other buffers hold this rank's columns
    unsigned* tp_done = nullptr;  // completion counter of the gather kernel
    cudaGraphExec_t graph[2][MAX_BATCH + 1] = {};  // the pass as a CUDA graph, per (short / long context, batch size)
    int graph_nodes[2][MAX_BATCH + 1] = {};
};

enum GraphKind : int { G_DECODE = 0, G_FEED, G_FWD_CLS, G_FWD, G_COUNT };

}  // namespace l2

struct l2_model {
    l2::Shape shape;
    l2_options opt{};
    int device = 0;
    int sms = 148;
    float eps = 1e-5f;
    cudaStream_t own_stream = nullptr, stream = nullptr;
    std::vector<l2::DevLayer> layers;
    float* tok_emb = nullptr;
    float* wcls = nullptr;
    float* rms_final = nullptr;
    float* rope_cos = nullptr;
    float* rope_sin = nullptr;
    std::vector<void*> allocs;
    uint64_t decode_bytes = 0;
    size_t device_bytes = 0;
    l2_state* gen_state = nullptr;  // reused by l2_generate_ids
    bool use_graph = true, use_pdl = true;
    bool use_token_kernel = true;    // B=1 forward as one persistent kernel (single GPU only)
    int tp_rank = 0, tp_world = 1;   // tensor parallelism: this process owns 1/tp_world of every matrix's rows
    void* nccl_comm = nullptr;
    // tensor parallelism over peer memory (token kernel): one pool of tagged activations per rank, the peers'
    // pools mapped through CUDA IPC; the first run state of the model works in the pool
    char* tp_pool = nullptr;
    char* tp_peers[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    size_t tp_batch_off[3] = {0, 0, 0};   // batched forward under tensor parallelism: x, att, hb ([MAX_BATCH][dim or hidden] f32) inside the pool
    size_t tp_flag_off = 0;               // [8] arrival counters of its exchanges; at + 128 bytes this rank's count of exchanges made
    bool tp_peer_borrowed[8] = {false, false, false, false, false, false, false, false};  // attached by pointer: not an IPC mapping to close
    bool tp_direct = false;          // every rank's pool is attached
    l2_state* tp_pool_owner = nullptr;
};

struct l2_state {
    l2_model* m = nullptr;
    float *kc = nullptr, *vc = nullptr;  // [L][SEQ][KVH][HS]
    float *x = nullptr, *xq = nullptr, *xk = nullptr, *xv = nullptr;
    float *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr;
    float* att_nat = nullptr;  // tensor parallelism: attention output in natural order before it is gathered
    float *x1 = nullptr, *x3 = nullptr, *hb = nullptr, *logits = nullptr;
    float* part = nullptr;
    unsigned* counter = nullptr;
    l2::Ctl* ctl = nullptr;
    l2::Ctl* h_ctl = nullptr;  // pinned ring of CTL_RING records; h_ctl[0] also receives read-backs
    int ctl_slot = 0;
    int* prompt = nullptr;
    int* out_tokens = nullptr;
    int max_split = 1;
    int failed_status = 0;              // device status of a launch that gave up; cleared by l2_state_reset
    std::vector<l2::SkLaunch> plans;     // [layer][4] GEMV launches, planned once
    l2::SkParams* d_plans = nullptr;     // their parameter records on the device
    l2::BatchBuffers* batch = nullptr;   // activations of the batched forward, allocated on first use
    l2::PhaseRec* d_phases[l2::G_COUNT] = {nullptr, nullptr, nullptr, nullptr};  // phase tables of the token kernel
    int n_phases[l2::G_COUNT] = {0, 0, 0, 0};
    l2::TokenParams tk{};                // ring geometry and barrier of the token kernel
    size_t tk_smem = 0;
    // activations of the token kernel as (value, tag) pairs, 8 bytes per element (see token_kernel.cu)
    unsigned long long *t_x = nullptr, *t_xq = nullptr, *t_xk = nullptr, *t_xv = nullptr, *t_q = nullptr, *t_k = nullptr, *t_v = nullptr;
    unsigned long long *t_att = nullptr, *t_x1 = nullptr, *t_x3 = nullptr, *t_hb = nullptr;
    unsigned long long* t_logits = nullptr;  // [VOCAB] tagged logits, tensor parallel over peer memory only (every rank computes a slice of the rows)
    unsigned long long* t_part = nullptr;  // [n_heads][tk_max_split][HS + 2] partial attention results of the sequence splits, tagged
    int tk_max_split = 1;
    unsigned long long* tk_trace = nullptr;
    size_t tk_trace_count = 0;
    cudaGraphExec_t graphs[l2::G_COUNT] = {nullptr, nullptr, nullptr, nullptr};
    int graph_nodes[l2::G_COUNT] = {0, 0, 0, 0};
    std::vector<void*> allocs;
};

struct l2_qlinear {
    l2::DevQ q;
    int device = 0;
    int sms = 148;
    int group_size = 128;
    float *x_dev = nullptr, *xp_dev = nullptr, *y_dev = nullptr;
    l2::SkParams* d_plan = nullptr;
    uint8_t* img = nullptr;   // batched path: digit image with the digit sums, and the factors
    float* osc = nullptr;
    float* kpart = nullptr;   // [4][MAX_BATCH][out] partial results when the groups of a tile are split over CTAs
    int* status = nullptr;
    int cap_b = 0;
    cudaStream_t stream = nullptr;
    std::vector<void*> allocs;
};

namespace l2 {
int upload_qlinear(const PackedQ& p, const int32_t* g_index, DevQ& d, std::vector<void*>& allocs, size_t* bytes);
void launch_permute(const float* x, const int* perm, float* xp, int n, cudaStream_t st);
int check_attention_args(int n_heads, int n_kv_heads, int pos, const void* q, const void* k, const void* v, const void* kc,
                         const void* vc, const void* rc, const void* rs, const void* out);
int device_sm_count();
int attention_max_split(int n_kv_heads);
int run_gemv_single(const DevQ& q, const float* xp, float* y, int sms, SkParams* d_plan, cudaStream_t st);
int sk_plan(SkLaunch& L, int sms);
void sk_prefetch_next(SkLaunch& L, const DevQ& q);
int forward_batch(l2_state* s, int M, const int32_t* tokens, const int32_t* pos);
struct NcclId { char bytes[128]; };  // ncclUniqueId
int tp_all_gather(l2_model* m, float* buf, size_t count, cudaStream_t st);
void tp_disconnect(l2_model* m);
void tp_rows(int total_rows, int rank, int world, int* row0, int* nrows);
int gemm_batched(const DevQ& q, const float* x, int ldx, bool gather, const float* nw, float eps, int M, uint8_t* img, float* osc,
                 float* out, int ldo, int epi, int* status, cudaStream_t st, float* kpart = nullptr, int sms = 148, int side_tiles = 0);
int dev_alloc_bytes(void** p, size_t bytes, std::vector<void*>& allocs);
void sk_set_matrix(SkJob& j, int seg, const DevQ& q, const float* x, const float* nw);
}  // namespace l2
