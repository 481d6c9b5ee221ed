// Host side of the batched forward pass transformer<B>, B >= 2 (src/models.rs:178-298): the
// sequence of launches for a chunk of M <= 64 tokens.  Every QLinear is a tcgen05 GEMM on exact
// integer digits of the activations (gemm_tc.cu); no logits are produced, as in the reference.
#include <cstring>

#include "model.h"

namespace l2 {

int dev_alloc_bytes(void** p, size_t bytes, std::vector<void*>& allocs) {
    L2_CUDA(cudaMalloc(p, bytes ? bytes : 16));
    allocs.push_back(*p);
    return L2_OK;
}

// out[m][:] = QLinear(x[m][:]) for m < M.  gather: x is in natural order and is brought into the
// matrix's K order through its g_index; nw (K order) folds an rmsnorm in.
int gemm_batched(const DevQ& q, const float* x, int ldx, bool gather, const float* nw, float eps, int M, uint8_t* img,
                 float* osc, float* out, int ldo, int epi, int* status, cudaStream_t st, float* kpart, int sms, int side_tiles) {
    const int mpad = gemm_tc_mpad(M);
    QuantParams a{};
    a.x = x; a.perm = gather ? q.perm : nullptr; a.nw = nw;
    a.bimg = img; a.oscale = osc;
    a.in = q.in; a.gs = q.gs; a.ldx = ldx; a.mpad = mpad; a.n = 3 * mpad; a.eps = eps;
    launch_act_quant(a, M, st);
    TcParams t{};
    t.rec = q.rec; t.bimg = img; t.oscale = osc; t.out = out; t.status = status;
    t.tiles16 = q.tiles; t.G = q.G; t.gs = q.gs; t.rows = q.out;
    t.m = M; t.mpad = mpad; t.n = 3 * mpad; t.ldo = ldo; t.epi = epi;
    // A matrix with few 128-row tiles would leave most SMs idle: its groups are split over several CTAs
    // per tile, which store partial results that a small kernel adds up in slice order.
    // (side_tiles: 128-row tiles of the GEMMs that run side by side with this one on other streams)
    const int tiles128 = (q.tiles + 7) / 8;
    int ks = 1;
    if (kpart) {  // cost in group times: waves x (groups per CTA + about four to fill the CTA's pipeline) + about five for the sum kernel
        long best = -1;
        for (int k = 1; k <= 4 && k * 4 <= q.G; k++) {
            const long waves = ((long)(tiles128 + side_tiles) * k + sms - 1) / sms;
            const long cost = waves * ((q.G + k - 1) / k + 4) + (k > 1 ? 5 : 0);
            if (best < 0 || cost < best) { best = cost; ks = k; }
        }
    }
    if (ks > 1) {
        t.ksplit = ks;
        t.kstride = (size_t)M * q.out;
        t.part = kpart;
    }
    L2_CUDA(launch_gemm_tc(t, st));
    if (ks > 1) launch_ksum(kpart, t.kstride, ks, out, ldo, q.out, M, epi, st);
    return L2_OK;
}

static int ensure_batch(l2_state* s) {
    if (s->batch) return L2_OK;
    l2_model* m = s->m;
    const l2_config& c = m->shape.c;
    const size_t B = MAX_BATCH, D = c.dim, KV = m->shape.kv_dim(), H = c.hidden_dim;
    const size_t kmax = std::max(D, H);
    BatchBuffers* b = new BatchBuffers;
    int rc = 0;
    auto F = [&](float** p, size_t n) { return dev_alloc_bytes(reinterpret_cast<void**>(p), n * sizeof(float), s->allocs); };
    // Tensor parallel over peer memory: the vectors that every rank needs in full (x, the attention output, the SwiGLU
    // output) live in the model's pool, where the peers store their columns; q, k, v, h1, h3 hold this rank's columns only.
    b->tp = m->tp_world > 1;
    const size_t T = b->tp ? (size_t)m->tp_world : 1;
    if (b->tp) {
        if (!m->tp_direct || !m->tp_pool) { delete b; return fail(L2_EINVAL, "batched forward under tensor parallelism needs the peers' pools attached"); }
        if (!m->tp_pool_owner) m->tp_pool_owner = s;
        if (m->tp_pool_owner != s) { delete b; return fail(L2_EINVAL, "batched forward under tensor parallelism: another run state of this model works in the pool"); }
        b->x = reinterpret_cast<float*>(m->tp_pool + m->tp_batch_off[0]);
        b->att = reinterpret_cast<float*>(m->tp_pool + m->tp_batch_off[1]);
        b->hb = reinterpret_cast<float*>(m->tp_pool + m->tp_batch_off[2]);
        if ((rc = dev_alloc_bytes(reinterpret_cast<void**>(&b->tp_done), 256, s->allocs))) { delete b; return rc; }
        L2_CUDA(cudaMemset(b->tp_done, 0, 256));
    } else if ((rc = F(&b->x, B * D)) || (rc = F(&b->att, B * D)) || (rc = F(&b->hb, B * H))) { delete b; return rc; }
    if ((rc = F(&b->q, B * D / T)) || (rc = F(&b->k, B * KV / T)) || (rc = F(&b->v, B * KV / T)) ||
        (rc = F(&b->h1, B * H / T)) || (rc = F(&b->h3, B * H / T)) ||
        (rc = F(&b->kpart[0], 4 * B * kmax)) || (rc = F(&b->kpart[1], 4 * B * kmax)) || (rc = F(&b->kpart[2], 4 * B * kmax))) { delete b; return rc; }
    for (int i = 0; i < 3; i++) {
        const size_t img_bytes = gemm_tc_image_bytes((int)kmax, c.group_size, (int)B);
        if ((rc = dev_alloc_bytes(reinterpret_cast<void**>(&b->img[i]), img_bytes, s->allocs)) ||
            (rc = F(&b->osc[i], B))) { delete b; return rc; }
        L2_CUDA(cudaMemset(b->img[i], 0, img_bytes));
    }
    if ((rc = dev_alloc_bytes(reinterpret_cast<void**>(&b->tok), B * sizeof(int), s->allocs)) ||
        (rc = dev_alloc_bytes(reinterpret_cast<void**>(&b->pos), B * sizeof(int), s->allocs))) { delete b; return rc; }
    if (cudaMallocHost(reinterpret_cast<void**>(&b->h_stage), sizeof(int) * 2 * B * CTL_RING) != cudaSuccess) { delete b; return fail(L2_ECUDA, "cudaMallocHost failed"); }
    for (int i = 0; i < 2; i++) {
        L2_CUDA(cudaStreamCreateWithFlags(&b->aux[i], cudaStreamNonBlocking));
        L2_CUDA(cudaEventCreateWithFlags(&b->join[i], cudaEventDisableTiming));
    }
    L2_CUDA(cudaEventCreateWithFlags(&b->fork, cudaEventDisableTiming));
    s->batch = b;
    return L2_OK;
}

// The kernels of one batched forward of M tokens (their ids and positions already in b->tok / b->pos), enqueued on `st`
// and, for the projections that run side by side, on the two auxiliary streams forked from it and joined back.
static int enqueue_batch(l2_state* s, int M, bool long_context, cudaStream_t st) {
    l2_model* m = s->m;
    const l2_config& c = m->shape.c;
    BatchBuffers* b = s->batch;
    const int D = c.dim, KV = m->shape.kv_dim(), H = c.hidden_dim;
    // this rank's share (everything on one GPU): rows of wq / wo (= heads), of wk / wv (= kv heads), of w1 / w3 / w2's inputs
    const int T = b->tp ? m->tp_world : 1, R = b->tp ? m->tp_rank : 0;
    const int Dl = D / T, KVl = KV / T, Hl = H / T, heads_l = c.n_heads / T, kvh_l = c.n_kv_heads / T;
    int* status = &s->ctl->status;
    // After a stage whose result every rank needs in full, this rank's columns go to the peers (stores over NVLink into their
    // pools) and the peers' columns are waited for: the same data flow as the tagged exchanges of the token kernel.  The
    // exchanges are numbered by a counter on the device (every rank makes the same exchanges in the same order), so that
    // the launch parameters do not change from call to call and the pass can be replayed as a CUDA graph.
    auto gather = [&](int which, int ld, int col0, int ncols) {
        if (!b->tp) return;
        TpGatherParams g{};
        for (int r = 0; r < 8; r++) g.pool[r] = r < T ? m->tp_peers[r] : nullptr;
        g.buf_off = m->tp_batch_off[which]; g.flag_off = m->tp_flag_off; g.seq = reinterpret_cast<unsigned long long*>(m->tp_pool + m->tp_flag_off + 128);  // in the pool: it outlives run states, like the peers' counters
        g.done = b->tp_done; g.status = status; g.rank = R; g.world = T; g.M = M; g.ld = ld; g.col0 = col0; g.ncols = ncols;
        launch_tp_gather(g, st);
    };
    launch_embed_batch(m->tok_emb, b->tok, b->x, D, M, st);  // src/models.rs:189-191 (every rank holds the table: no exchange)
    const size_t ls = (size_t)c.seq_len * KV;
    for (int l = 0; l < c.n_layers; l++) {
        const DevLayer& y = m->layers[l];
        int rc;
        // rmsnorm + wq/wk/wv (:217-226): three independent GEMMs, side by side on three streams
        L2_CUDA(cudaEventRecord(b->fork, st));
        L2_CUDA(cudaStreamWaitEvent(b->aux[0], b->fork, 0));
        L2_CUDA(cudaStreamWaitEvent(b->aux[1], b->fork, 0));
        if ((rc = gemm_batched(y.wq, b->x, D, true, y.nw_q, m->eps, M, b->img[0], b->osc[0], b->q, Dl, EPI_STORE, status, st, b->kpart[0], m->sms, (y.wk.tiles + 7) / 8 + (y.wv.tiles + 7) / 8))) return rc;
        if ((rc = gemm_batched(y.wk, b->x, D, true, y.nw_k, m->eps, M, b->img[1], b->osc[1], b->k, KVl, EPI_STORE, status, b->aux[0], b->kpart[1], m->sms, (y.wq.tiles + 7) / 8 + (y.wv.tiles + 7) / 8))) return rc;
        if ((rc = gemm_batched(y.wv, b->x, D, true, y.nw_v, m->eps, M, b->img[2], b->osc[2], b->v, KVl, EPI_STORE, status, b->aux[1], b->kpart[2], m->sms, (y.wq.tiles + 7) / 8 + (y.wk.tiles + 7) / 8))) return rc;
        for (int i = 0; i < 2; i++) {
            L2_CUDA(cudaEventRecord(b->join[i], b->aux[i]));
            L2_CUDA(cudaStreamWaitEvent(st, b->join[i], 0));
        }
        // rope, all rows into the cache (this rank's kv heads of the full-width cache rows), then attention (:228-256)
        RopeParams r{};
        r.q = b->q; r.k = b->k; r.v = b->v;
        r.kc = s->kc + (size_t)l * ls + (size_t)R * KVl; r.vc = s->vc + (size_t)l * ls + (size_t)R * KVl;
        r.rope_cos = m->rope_cos; r.rope_sin = m->rope_sin; r.pos = b->pos;
        r.n_kv_heads = kvh_l; r.ldq = Dl; r.ldkv = KVl; r.kv_stride = KV;
        launch_rope_append(r, heads_l, M, st);
        AttnBatchParams a{};
        a.q = b->q; a.kc = r.kc; a.vc = r.vc; a.pos = b->pos; a.out = b->att + (size_t)R * Dl;
        a.n_kv_heads = kvh_l; a.ag = m->shape.attn_groups(); a.ldq = Dl; a.ldo = D; a.kv_stride = KV;
        launch_attn_batch(a, heads_l, M, long_context, st);
        gather(1, D, R * Dl, Dl);
        // wo + residual (:260-264): this rank's rows of wo update its columns of x
        if ((rc = gemm_batched(y.wo, b->att, D, true, nullptr, m->eps, M, b->img[0], b->osc[0], b->x + y.wo.row0, D, EPI_RESID, status, st, b->kpart[0], m->sms, 0))) return rc;
        gather(0, D, y.wo.row0, y.wo.out);
        // rmsnorm + w1/w3 + SwiGLU (:266-276); their rows are stored in w2's K order
        L2_CUDA(cudaEventRecord(b->fork, st));
        L2_CUDA(cudaStreamWaitEvent(b->aux[0], b->fork, 0));
        if ((rc = gemm_batched(y.w1, b->x, D, true, y.nw_1, m->eps, M, b->img[0], b->osc[0], b->h1, Hl, EPI_STORE, status, st, b->kpart[0], m->sms, (y.w3.tiles + 7) / 8))) return rc;
        if ((rc = gemm_batched(y.w3, b->x, D, true, y.nw_3, m->eps, M, b->img[1], b->osc[1], b->h3, Hl, EPI_STORE, status, b->aux[0], b->kpart[1], m->sms, (y.w1.tiles + 7) / 8))) return rc;
        L2_CUDA(cudaEventRecord(b->join[0], b->aux[0]));
        L2_CUDA(cudaStreamWaitEvent(st, b->join[0], 0));
        launch_swiglu(b->h1, b->h3, b->hb + y.w1.row0, Hl, H, M, st);
        gather(2, H, y.w1.row0, y.w1.out);
        // w2 + residual (:279-285)
        if ((rc = gemm_batched(y.w2, b->hb, H, false, nullptr, m->eps, M, b->img[0], b->osc[0], b->x + y.w2.row0, D, EPI_RESID, status, st, b->kpart[0], m->sms, 0))) return rc;
        gather(0, D, y.w2.row0, y.w2.out);
    }
    L2_CUDA(cudaGetLastError());
    return L2_OK;
}

// One batched forward.  The ids and positions travel through a pinned ring; the kernels of the pass (about 25 per layer,
// most of them a few microseconds long: launched one by one the host cannot keep up with the GPU) are captured once per
// batch size into a CUDA graph and replayed.
int forward_batch(l2_state* s, int M, const int32_t* tokens, const int32_t* pos) {
    if (int rc = ensure_batch(s)) return rc;
    l2_model* m = s->m;
    BatchBuffers* b = s->batch;
    cudaStream_t st = m->stream;
    if (M < 1 || M > MAX_BATCH) return fail(L2_EINVAL, "forward_batch: %d tokens", M);
    // token ids and positions: own pinned slot per call until the copy has run
    if (++b->stage_slot >= CTL_RING) { L2_CUDA(cudaStreamSynchronize(st)); b->stage_slot = 0; }
    int* hs = b->h_stage + (size_t)b->stage_slot * 2 * MAX_BATCH;
    memcpy(hs, tokens, sizeof(int) * M);
    memcpy(hs + MAX_BATCH, pos, sizeof(int) * M);
    L2_CUDA(cudaMemcpyAsync(b->tok, hs, sizeof(int) * M, cudaMemcpyHostToDevice, st));
    L2_CUDA(cudaMemcpyAsync(b->pos, hs + MAX_BATCH, sizeof(int) * M, cudaMemcpyHostToDevice, st));
    // two graphs per batch size: the attention kernel differs between short and long contexts
    int last = 0;
    for (int i = 0; i < M; i++) last = std::max(last, (int)pos[i]);
    const int lc = last >= 192 ? 1 : 0;
    if (!m->use_graph) return enqueue_batch(s, M, lc != 0, st);
    if (!b->graph[lc][M]) {
        cudaStream_t cap;
        L2_CUDA(cudaStreamCreateWithFlags(&cap, cudaStreamNonBlocking));
        const unsigned long long before = g_launches;
        L2_CUDA(cudaStreamBeginCapture(cap, cudaStreamCaptureModeThreadLocal));
        const int rc = enqueue_batch(s, M, lc != 0, cap);
        cudaGraph_t graph = nullptr;
        const cudaError_t e = cudaStreamEndCapture(cap, &graph);
        b->graph_nodes[lc][M] = (int)(g_launches - before);
        g_launches = before;  // captured launches have not run
        cudaStreamDestroy(cap);
        if (rc != L2_OK) { if (graph) cudaGraphDestroy(graph); return rc; }
        if (e != cudaSuccess) return fail(L2_ECUDA, "batched forward: graph capture failed: %s", cudaGetErrorString(e));
        const cudaError_t e2 = cudaGraphInstantiate(&b->graph[lc][M], graph, 0);
        cudaGraphDestroy(graph);
        if (e2 != cudaSuccess) { b->graph[lc][M] = nullptr; return fail(L2_ECUDA, "batched forward: graph instantiate failed: %s", cudaGetErrorString(e2)); }
    }
    L2_CUDA(cudaGraphLaunch(b->graph[lc][M], st));
    g_launches += b->graph_nodes[lc][M];
    return L2_OK;
}

}  // namespace l2
