// Model handle, run state and token loop behind the C ABI: loads a checkpoint into the
// device layout, captures the per-token forward (src/models.rs:178-298) into CUDA graphs
// and drives prefill / decode (src/inference.rs:16-193).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "model.h"

using namespace l2;

extern "C" void l2_model_close(l2_model* m);

namespace l2 {

static int dev_alloc(void** p, size_t bytes, std::vector<void*>& allocs, size_t* total = nullptr) {
    L2_CUDA(cudaMalloc(p, bytes ? bytes : 16));
    allocs.push_back(*p);
    if (total) *total += bytes;
    return L2_OK;
}

// Host -> device copies of a checkpoint load: the bytes go through two pinned staging buffers in chunks, one
// cudaMemcpyAsync per chunk, so that reading the next chunk from the mmap (page faults, disk) or repacking the next
// matrix overlaps the DMA of the previous one and 70B does not stage 41 GB synchronously (the reference maps the
// file and "loads instantly", README.md:12; here the file is streamed once onto the device).
class Uploader {
public:
    static constexpr size_t CHUNK = (size_t)16 << 20;
    ~Uploader() { release(); }
    int copy(void* dst, const void* src, size_t bytes) {
        if (int rc = init()) return rc;
        const char* s = static_cast<const char*>(src);
        char* d = static_cast<char*>(dst);
        for (size_t off = 0; off < bytes; off += CHUNK) {
            const size_t n = std::min(CHUNK, bytes - off);
            L2_CUDA(cudaEventSynchronize(done_[cur_]));  // the copy that used this buffer last has finished
            memcpy(pinned_[cur_], s + off, n);
            L2_CUDA(cudaMemcpyAsync(d + off, pinned_[cur_], n, cudaMemcpyHostToDevice, stream_));
            L2_CUDA(cudaEventRecord(done_[cur_], stream_));
            cur_ ^= 1;
        }
        return L2_OK;
    }
    int finish() {
        if (stream_) L2_CUDA(cudaStreamSynchronize(stream_));
        return L2_OK;
    }
private:
    int init() {
        if (stream_) return L2_OK;
        L2_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
        for (int i = 0; i < 2; i++) {
            L2_CUDA(cudaMallocHost(reinterpret_cast<void**>(&pinned_[i]), CHUNK));
            L2_CUDA(cudaEventCreateWithFlags(&done_[i], cudaEventDisableTiming));
        }
        return L2_OK;
    }
    void release() {
        if (stream_) cudaStreamSynchronize(stream_);
        for (int i = 0; i < 2; i++) {
            if (pinned_[i]) cudaFreeHost(pinned_[i]);
            if (done_[i]) cudaEventDestroy(done_[i]);
        }
        if (stream_) cudaStreamDestroy(stream_);
    }
    cudaStream_t stream_ = nullptr;
    char* pinned_[2] = {nullptr, nullptr};
    cudaEvent_t done_[2] = {nullptr, nullptr};
    int cur_ = 0;
};
static thread_local Uploader* g_uploader = nullptr;  // set while build_model runs: its uploads go through it

template <class T>
static int dev_upload(T** p, const void* src, size_t count, std::vector<void*>& allocs, size_t* total = nullptr) {
    if (int rc = dev_alloc(reinterpret_cast<void**>(p), count * sizeof(T), allocs, total)) return rc;
    if (g_uploader) return g_uploader->copy(*p, src, count * sizeof(T));  // the source may be reused as soon as this returns
    L2_CUDA(cudaMemcpy(*p, src, count * sizeof(T), cudaMemcpyHostToDevice));
    return L2_OK;
}

int upload_qlinear(const PackedQ& p, const int32_t* g_index, DevQ& d, std::vector<void*>& allocs, size_t* bytes) {
    d.in = p.in; d.out = p.out; d.tiles = p.tiles; d.G = p.groups; d.gs = p.w * 32;
    if (int rc = dev_upload(&d.rec, p.rec.data(), p.rec.size(), allocs, bytes)) return rc;
    if (g_index) {
        if (int rc = dev_upload(&d.perm, g_index, (size_t)p.in, allocs, bytes)) return rc;
        std::vector<int32_t> inv = inverse_permutation(g_index, p.in);
        if (int rc = dev_upload(&d.inv, inv.data(), (size_t)p.in, allocs, bytes)) return rc;
        if (p.in < 65536) {
            std::vector<uint16_t> i16(inv.begin(), inv.end());
            if (int rc = dev_upload(&d.inv16, i16.data(), (size_t)p.in, allocs, bytes)) return rc;
            std::vector<uint16_t> p16(g_index, g_index + p.in);
            if (int rc = dev_upload(&d.perm16, p16.data(), (size_t)p.in, allocs, bytes)) return rc;
        }
    }
    return L2_OK;
}

__global__ void permute_kernel(const float* __restrict__ x, const int* __restrict__ perm, float* __restrict__ xp, int n) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < n) xp[j] = x[perm[j]];
}

void launch_permute(const float* x, const int* perm, float* xp, int n, cudaStream_t st) {
    permute_kernel<<<(n + 255) / 256, 256, 0, st>>>(x, perm, xp, n);
    g_launches++;
}

void sk_set_matrix(SkJob& j, int seg, const DevQ& q, const float* x, const float* nw) {
    j.seg[seg].rec = q.rec;
    j.seg[seg].x = x; j.seg[seg].nw = nw;
    j.rows = q.out; j.tiles = q.tiles; j.in = q.in; j.G = q.G;
}

// Deals the CTAs of a launch to its jobs in proportion to their tiles (every CTA owns whole tiles;
// inside a job the first tiles % ncta CTAs own one tile more) and sizes the shared memory.
int sk_plan(SkLaunch& L, int sms) {
    SkParams& p = L.p;
    long long total = 0;
    for (int i = 0; i < p.njobs; i++) total += p.job[i].tiles;
    const int want = (int)std::min<long long>(sms, total);
    int used = 0, ptiles = 1, max_g = 0;
    for (int i = 0; i < p.njobs; i++) {
        SkJob& j = p.job[i];
        long long n = i + 1 == p.njobs ? want - used : (long long)want * j.tiles / total;
        n = std::max<long long>(1, std::min<long long>(n, j.tiles));
        j.cta0 = used;
        j.ncta = (int)n;
        used += (int)n;
        j.tq = j.tiles / j.ncta;
        j.trem = j.tiles % j.ncta;
        j.rGs = 1.0f / (float)(L.nseg * j.G);
        ptiles = std::max(ptiles, (j.tiles + j.ncta - 1) / j.ncta);
        max_g = std::max(max_g, j.G);
    }
    L.grid = used;
    for (int i = 0; i < p.n_next; i++) p.next_slice[i] = ((p.next_bytes[i] / used) + 15) & ~(size_t)15;
    // shared memory: digits, group sums and tile sums are fixed; the rest goes to the weight rings
    const size_t fixed = (sk_smem_fixed(p.job[0].in, max_g, L.nseg, ptiles) + 127) & ~(size_t)127;
    const size_t budget = 224 * 1024;
    if (fixed >= budget) return fail(L2_EINVAL, "IN %d needs %zu bytes of shared memory before the weight rings", p.job[0].in, fixed);
    // ring geometry: large slots (the copy engine spends a fixed time per request), as many as fit,
    // no more than the longest CTA range needs
    int su = 32;
    if (const char* e = getenv("L2_SK_CHUNK")) su = std::max(2, atoi(e) & ~1);  // tuning knob
    long long max_units = 0;
    for (int i = 0; i < p.njobs; i++)
        max_units = std::max<long long>(max_units, (long long)((p.job[i].tiles + p.job[i].ncta - 1) / p.job[i].ncta) * L.nseg * p.job[i].G);
    int slots = 0;
    for (; su >= 2; su /= 2) {
        slots = (int)std::min<size_t>(SK_MAX_SLOTS, (budget - fixed) / sk_slot_bytes(L.gs, su));
        if (slots >= 2) break;
    }
    if (slots < 2) return fail(L2_EINVAL, "IN %d leaves no shared memory for the weight ring", p.job[0].in);
    slots = std::max(2, std::min<int>(slots, (int)((max_units + su - 1) / su)));
    const int chunk = su;
    if (const char* e = getenv("L2_SK_SLOTS")) slots = std::max(2, std::min(slots, atoi(e)));
    p.debug_skip = getenv("L2_SK_SKIP") ? 1 : 0;
    p.chunk = chunk;
    p.slots = slots;
    p.ptiles = ptiles;
    L.smem = fixed + (size_t)slots * sk_slot_bytes(L.gs, chunk);
    return L2_OK;
}

// Registers the weights of `q` as the next kernel's, to be fetched into L2 by launch L.
void sk_prefetch_next(SkLaunch& L, const DevQ& q) {
    SkParams& p = L.p;
    if (p.n_next + 1 > 6) return;
    p.next_ptr[p.n_next] = q.rec;
    p.next_bytes[p.n_next++] = (size_t)q.tiles * q.G * ((q.gs / 32) * 256 + 80);
}

int run_gemv_single(const DevQ& q, const float* xp, float* y, int sms, SkParams* d_plan, cudaStream_t st) {
    SkLaunch L;
    L.p.njobs = 1;
    L.nseg = 1;
    L.gs = q.gs;
    sk_set_matrix(L.p.job[0], 0, q, xp, nullptr);
    L.p.job[0].out = y;
    L.p.job[0].epi = EPI_STORE;
    if (int rc = sk_plan(L, sms)) return rc;
    L.p.trace = g_sk_trace;
    L2_CUDA(cudaMemcpyAsync(d_plan, &L.p, sizeof(SkParams), cudaMemcpyHostToDevice, st));  // pageable source: staged before return
    L2_CUDA(launch_sk(d_plan, L.gs, 1, L.grid, L.smem, st, false));
    return L2_OK;
}

static int check_device(int device, int* out_dev, int* sms) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0)
        return fail(L2_ECUDA, "no usable CUDA device (%s); this library has no CPU fallback", cudaGetErrorString(e));
    int dev = device;
    if (dev < 0) L2_CUDA(cudaGetDevice(&dev));
    if (dev >= n) return fail(L2_EINVAL, "device %d out of range (%d devices)", dev, n);
    L2_CUDA(cudaSetDevice(dev));
    cudaDeviceProp prop;
    L2_CUDA(cudaGetDeviceProperties(&prop, dev));
    if (prop.major < 10) return fail(L2_ECUDA, "device %d is sm_%d%d; this library is built for sm_100a only", dev, prop.major, prop.minor);
    *out_dev = dev;
    *sms = prop.multiProcessorCount;
    L2_CUDA(kernels_init());
    return L2_OK;
}

// Builds the device model from a tensor source.
// Frees what a partly built model holds when the open fails (device allocations, the stream).
struct ModelDeleter { void operator()(l2_model* m) const { l2_model_close(m); } };

static int build_model(const Shape& shape, Source& src, const l2_options* opt, l2_model** out) {
    std::unique_ptr<l2_model, ModelDeleter> m(new l2_model);
    Uploader uploader;
    struct Scope { Scope(Uploader* u) { g_uploader = u; } ~Scope() { g_uploader = nullptr; } } scope(&uploader);
    m->shape = shape;
    if (opt) m->opt = *opt;
    if (int rc = check_device(opt ? opt->device : -1, &m->device, &m->sms)) return rc;
    m->tp_world = m->opt.tp_world > 1 ? m->opt.tp_world : 1;
    m->tp_rank = m->tp_world > 1 ? m->opt.tp_rank : 0;
    if (m->tp_world > L2_MAX_TP) return fail(L2_EINVAL, "tp_world %d exceeds the %d ranks of one box", m->tp_world, L2_MAX_TP);
    if (m->tp_rank < 0 || m->tp_rank >= m->tp_world) return fail(L2_EINVAL, "tp_rank %d outside 0..%d", m->tp_rank, m->tp_world - 1);
    if (shape.c.n_kv_heads % m->tp_world || (shape.c.dim / m->tp_world) % 16 || (shape.c.hidden_dim / m->tp_world) % 16 || shape.c.hidden_dim % m->tp_world)
        return fail(L2_EINVAL, "tp_world %d does not divide the kv heads / leave whole 16-row tiles", m->tp_world);
    m->use_graph = !(m->opt.flags & L2_FLAG_NO_GRAPH);
    m->use_pdl = !(m->opt.flags & L2_FLAG_NO_PDL);
    m->use_token_kernel = !(m->opt.flags & L2_FLAG_NO_TOKEN_KERNEL) && !getenv("L2_NO_TOKEN_KERNEL");
    L2_CUDA(cudaStreamCreateWithFlags(&m->own_stream, cudaStreamNonBlocking));
    m->stream = m->own_stream;
    const l2_config& c = shape.c;
    const int D = c.dim, L = c.n_layers, V = c.vocab_size, G = c.group_size;
    std::vector<uint32_t> s0, s1, s2, s3;
    size_t* tot = &m->device_bytes;

    m->eps = *reinterpret_cast<const float*>(src.get(T_RMS_EPS, 0, S_DENSE, s0));
    if (int rc = dev_upload(&m->tok_emb, src.get(T_TOK_EMB, 0, S_DENSE, s0), (size_t)V * D, m->allocs, tot)) return rc;
    if (int rc = dev_upload(&m->wcls, src.get(T_WCLS, 0, S_DENSE, s0), (size_t)V * D, m->allocs, tot)) return rc;
    if (int rc = dev_upload(&m->rms_final, src.get(T_RMS_FINAL, 0, S_DENSE, s0), (size_t)D, m->allocs, tot)) return rc;
    {   // RoPE table with the reference's f32 formula (src/models.rs:107-110)
        const int half = HS / 2;
        std::vector<float> co((size_t)c.seq_len * half), si((size_t)c.seq_len * half);
        for (int p = 0; p < c.seq_len; p++)
            for (int i = 0; i < half; i++) {
                const float freq = 1.0f / powf(10000.0f, (float)(2 * i % HS) / (float)HS);
                const float val = (float)p * freq;
                co[(size_t)p * half + i] = cosf(val);
                si[(size_t)p * half + i] = sinf(val);
            }
        if (int rc = dev_upload(&m->rope_cos, co.data(), co.size(), m->allocs, tot)) return rc;
        if (int rc = dev_upload(&m->rope_sin, si.data(), si.size(), m->allocs, tot)) return rc;
    }

    m->layers.resize(L);
    uint64_t qbytes = 0;
    std::vector<int32_t> gi, gi2;
    std::vector<float> nw, nwp;
    auto load_q = [&](int t, int l, DevQ& d, const int32_t* rows_order, std::vector<int32_t>* keep_gi) -> int {
        int in, outn;
        shape.qdims(t, &in, &outn);
        const uint32_t* gx = src.get(t, l, S_GINDEX, s3);
        const int32_t* gidx = reinterpret_cast<const int32_t*>(gx);
        if (!is_permutation(gidx, in)) return fail(L2_EFORMAT, "tensor %d layer %d: g_index is not a permutation of 0..%d", t, l, in - 1);
        // tensor parallelism: this process keeps rows [row0, row0 + nrows) of the (re-ordered) matrix
        int row0 = 0, nrows = outn;
        tp_rows(outn, m->tp_rank, m->tp_world, &row0, &nrows);
        std::vector<int32_t> order(nrows);
        for (int j = 0; j < nrows; j++) order[j] = rows_order ? rows_order[row0 + j] : row0 + j;
        const size_t g = Shape::groups(in, G);
        s0.resize((size_t)nrows * (in / 8));
        s1.resize((size_t)nrows * g);
        std::vector<uint8_t> zn((size_t)nrows * g);
        src.get_rows(t, l, order.data(), nrows, s0.data(), reinterpret_cast<float*>(s1.data()), zn.data());
        PackedQ p;
        repack_compact(in, nrows, G, s0.data(), reinterpret_cast<const float*>(s1.data()), zn.data(), p);
        if (keep_gi) keep_gi->assign(gidx, gidx + in);
        qbytes += (shape.sub_words(t, S_QWEIGHT) + shape.sub_words(t, S_QZEROS) + shape.sub_words(t, S_SCALES)) * 4 / m->tp_world;
        d.row0 = row0;
        return upload_qlinear(p, gidx, d, m->allocs, tot);
    };
    auto permuted_norm = [&](const float* w, const std::vector<int32_t>& g, float** dst) -> int {
        nwp.resize(g.size());
        for (size_t j = 0; j < g.size(); j++) nwp[j] = w[g[j]];
        return dev_upload(dst, nwp.data(), nwp.size(), m->allocs, tot);
    };
    std::vector<uint32_t> sn;
    for (int l = 0; l < L; l++) {
        DevLayer& y = m->layers[l];
        const float* att = reinterpret_cast<const float*>(src.get(T_RMS_ATT, l, S_DENSE, sn));
        nw.assign(att, att + D);
        if (int rc = dev_upload(&y.rms_att, nw.data(), (size_t)D, m->allocs, tot)) return rc;
        if (int rc = load_q(T_WQ, l, y.wq, nullptr, &gi)) return rc;
        if (int rc = permuted_norm(nw.data(), gi, &y.nw_q)) return rc;
        if (int rc = load_q(T_WK, l, y.wk, nullptr, &gi)) return rc;
        if (int rc = permuted_norm(nw.data(), gi, &y.nw_k)) return rc;
        if (int rc = load_q(T_WV, l, y.wv, nullptr, &gi)) return rc;
        if (int rc = permuted_norm(nw.data(), gi, &y.nw_v)) return rc;
        if (int rc = load_q(T_WO, l, y.wo, nullptr, nullptr)) return rc;
        const float* ffn = reinterpret_cast<const float*>(src.get(T_RMS_FFN, l, S_DENSE, sn));
        nw.assign(ffn, ffn + D);
        if (int rc = dev_upload(&y.rms_ffn, nw.data(), (size_t)D, m->allocs, tot)) return rc;
        // w2 first: its act-order permutation becomes the row order of w1 and w3, so that the
        // SwiGLU output is produced directly in w2's K order.
        if (int rc = load_q(T_W2, l, y.w2, nullptr, &gi2)) return rc;
        if (int rc = load_q(T_W1, l, y.w1, gi2.data(), &gi)) return rc;
        if (int rc = permuted_norm(nw.data(), gi, &y.nw_1)) return rc;
        if (int rc = load_q(T_W3, l, y.w3, gi2.data(), &gi)) return rc;
        if (int rc = permuted_norm(nw.data(), gi, &y.nw_3)) return rc;
    }
    if (int rc = uploader.finish()) return rc;
    m->decode_bytes = qbytes + (uint64_t)V * D * 4 + (uint64_t)(2 * L + 1) * D * 4;
    if (m->opt.debug) {
        printf("Configuration: Config { dim: %d, hidden_dim: %d, n_layers: %d, n_heads: %d, n_kv_heads: %d, vocab_size: %d, seq_len: %d, group_size: %d }\n",
               c.dim, c.hidden_dim, c.n_layers, c.n_heads, c.n_kv_heads, c.vocab_size, c.seq_len, c.group_size);
        printf("CUDA device %d, %d SMs, %.2f GB of weights on device\n", m->device, m->sms, m->device_bytes / 1e9);
    }
    *out = m.release();
    return L2_OK;
}

static void free_allocs(std::vector<void*>& a) {
    for (void* p : a) cudaFree(p);
    a.clear();
}

// ---- the forward pass as a sequence of launches ------------------------------------------------

static void set_scatter3(float** sdst, const int** sidx, int* n, l2_state* s, const DevLayer* next) {
    if (!next) { *n = 0; return; }
    sdst[0] = s->xq; sidx[0] = next->wq.inv;
    sdst[1] = s->xk; sidx[1] = next->wk.inv;
    sdst[2] = s->xv; sidx[2] = next->wv.inv;
    *n = 3;
}

// The four GEMV launches of a layer; each also prefetches the next GEMV's weights into L2.
static int plan_layer_gemv(l2_state* s, int l, int which, SkLaunch& L, bool direct = false) {
    l2_model* m = s->m;
    const l2_config& c = m->shape.c;
    const DevLayer& y = m->layers[l];
    L = SkLaunch{};
    L.gs = c.group_size;
    L.p.eps = m->eps;
    SkJob* j = L.p.job;
    const bool tp = m->tp_world > 1 && !direct;  // direct: the token kernel stores into every rank's buffers itself
    switch (which) {
        case 0:  // rmsnorm + wq/wk/wv (src/models.rs:217-226)
            L.p.njobs = 3;
            sk_set_matrix(j[0], 0, y.wq, s->xq, y.nw_q); j[0].out = s->q + y.wq.row0; j[0].epi = EPI_STORE;
            sk_set_matrix(j[1], 0, y.wk, s->xk, y.nw_k); j[1].out = s->k + y.wk.row0; j[1].epi = EPI_STORE;
            sk_set_matrix(j[2], 0, y.wv, s->xv, y.nw_v); j[2].out = s->v + y.wv.row0; j[2].epi = EPI_STORE;
            sk_prefetch_next(L, y.wo);
            break;
        case 1:  // wo + residual (:260-264); the new x goes to w1's and w3's K order as well
            L.p.njobs = 1;
            sk_set_matrix(j[0], 0, y.wo, s->att, nullptr); j[0].out = s->x + y.wo.row0; j[0].epi = EPI_RESID;
            if (!tp) {  // with tensor parallelism the copies are made after the all-gather of x
                j[0].sdst[0] = s->x1; j[0].sidx[0] = y.w1.inv + y.wo.row0;  // indexed by the rows this process holds
                j[0].sdst[1] = s->x3; j[0].sidx[1] = y.w3.inv + y.wo.row0;
                j[0].nscatter = 2;
            }
            sk_prefetch_next(L, y.w1);
            sk_prefetch_next(L, y.w3);
            break;
        case 2:  // rmsnorm + w1/w3 + SwiGLU (:266-276); rows are in w2's K order
            L.p.njobs = 1;
            L.nseg = 2;
            sk_set_matrix(j[0], 0, y.w1, s->x1, y.nw_1);
            sk_set_matrix(j[0], 1, y.w3, s->x3, y.nw_3);
            j[0].out = s->hb + y.w1.row0; j[0].epi = EPI_SWIGLU;
            sk_prefetch_next(L, y.w2);
            break;
        default:  // w2 + residual (:279-285); the new x goes to the next layer's q/k/v K orders
            L.p.njobs = 1;
            sk_set_matrix(j[0], 0, y.w2, s->hb, nullptr); j[0].out = s->x + y.w2.row0; j[0].epi = EPI_RESID;
            if (!tp) {
                set_scatter3(j[0].sdst, j[0].sidx, &j[0].nscatter, s, l + 1 < c.n_layers ? &m->layers[l + 1] : nullptr);
                for (int i = 0; i < j[0].nscatter; i++) j[0].sidx[i] += y.w2.row0;
            }
            if (l + 1 < c.n_layers) {
                sk_prefetch_next(L, m->layers[l + 1].wq);
                sk_prefetch_next(L, m->layers[l + 1].wk);
                sk_prefetch_next(L, m->layers[l + 1].wv);
            }
            break;
    }
    if (m->opt.flags & L2_FLAG_NO_L2_PREFETCH) L.p.n_next = 0;
    L.p.trace = g_sk_trace;
    L.p.status = &s->ctl->status;
    return sk_plan(L, m->sms);
}

static void launch_layer_gemv(l2_state* s, int l, int which, cudaStream_t st, bool pdl) {
    const SkLaunch& L = s->plans[(size_t)l * 4 + which];
    launch_sk(s->d_plans + (size_t)l * 4 + which, L.gs, L.nseg, L.grid, L.smem, st, pdl);
}
static void launch_qkv(l2_state* s, int l, cudaStream_t st, bool pdl) { launch_layer_gemv(s, l, 0, st, pdl); }
static void launch_wo(l2_state* s, int l, cudaStream_t st, bool pdl) { launch_layer_gemv(s, l, 1, st, pdl); }
static void launch_w13(l2_state* s, int l, cudaStream_t st, bool pdl) { launch_layer_gemv(s, l, 2, st, pdl); }
static void launch_w2(l2_state* s, int l, cudaStream_t st, bool pdl) { launch_layer_gemv(s, l, 3, st, pdl); }

// rope + cache append + attention (src/models.rs:228-256)
static AttnParams attention_params(l2_state* s, int l, bool direct = false) {
    l2_model* m = s->m;
    const l2_config& c = m->shape.c;
    const DevLayer& y = m->layers[l];
    AttnParams a{};
    a.q = s->q; a.k = s->k; a.v = s->v;
    const size_t ls = (size_t)c.seq_len * m->shape.kv_dim();
    a.kc = s->kc + (size_t)l * ls; a.vc = s->vc + (size_t)l * ls;
    a.rope_cos = m->rope_cos; a.rope_sin = m->rope_sin;
    a.ctl = s->ctl; a.part = s->part; a.counter = s->counter;
    const bool gathered = m->tp_world > 1 && !direct;  // tensor parallel over NCCL: natural order, gathered and permuted afterwards
    a.out = gathered ? s->att_nat : s->att; a.oidx = gathered ? nullptr : y.wo.inv;
    a.n_kv_heads = c.n_kv_heads; a.ag = m->shape.attn_groups();
    a.n_kv_local = c.n_kv_heads / m->tp_world; a.kvh0 = m->tp_rank * a.n_kv_local;
    a.max_split = s->max_split; a.split_min = 64;
    a.pos_fixed = -1;
    return a;
}

static void launch_attention(l2_state* s, int l, cudaStream_t st, bool pdl) { launch_attn(attention_params(s, l), st, pdl); }

static ClsParams classifier_params(l2_state* s) {
    l2_model* m = s->m;
    const l2_config& c = m->shape.c;
    ClsParams cp{};
    cp.w = m->wcls; cp.x = s->x; cp.nw = m->rms_final; cp.logits = s->logits;
    cp.rows = c.vocab_size; cp.in = c.dim; cp.eps = m->eps;
    return cp;
}

static void launch_classifier(l2_state* s, cudaStream_t st, bool pdl) { launch_cls(classifier_params(s), s->m->sms * 2, st, pdl); }

static EmbedParams embed_params(l2_state* s, int kind) {
    l2_model* m = s->m;
    const l2_config& c = m->shape.c;
    EmbedParams e{};
    e.table = m->tok_emb; e.ctl = s->ctl; e.prompt = s->prompt; e.x = s->x;
    e.dim = c.dim; e.vocab = c.vocab_size; e.feed_prompt = kind == G_FEED;
    set_scatter3(e.sdst, e.sidx, &e.nscatter, s, &m->layers[0]);
    return e;
}

// ---- the forward pass as one persistent kernel ---------------------------------------------------

// The tagged activation vectors of the token kernel live in one pool with the same layout on every rank,
// so that a rank can store into a peer's pool at the offset it uses in its own.
struct TaggedLayout { size_t off[12], n[12], total; size_t batch_off[3], flag_off; };
static TaggedLayout tagged_layout(const l2_model* m) {
    const l2_config& c = m->shape.c;
    const size_t D = c.dim, KV = m->shape.kv_dim(), H = c.hidden_dim;
    // x, xq, xk, xv, q, k, v, att, x1, x3, hb; under tensor parallelism also the logits (each rank computes a slice of the vocabulary)
    const size_t n[12] = {D, D, D, D, D, KV, KV, D, D, D, H, m->tp_world > 1 ? (size_t)c.vocab_size : 0};
    TaggedLayout t{};
    size_t at = 0;
    for (int i = 0; i < 12; i++) { t.off[i] = at; t.n[i] = n[i]; at += (n[i] * 8 + 255) & ~(size_t)255; }
    if (m->tp_world > 1) {  // batched forward: the vectors every rank needs in full (plain f32 rows of MAX_BATCH tokens) and the exchange counters
        const size_t bn[3] = {D, D, H};  // x, att, hb
        for (int i = 0; i < 3; i++) { t.batch_off[i] = at; at += (MAX_BATCH * bn[i] * 4 + 255) & ~(size_t)255; }
        t.flag_off = at; at += 256;
    }
    t.total = at;
    return t;
}

// The forward of this state runs as the token kernel: always on one GPU; under tensor parallelism when the
// peers' pools are attached and this state is the one that works in the model's pool.
static bool token_path(const l2_state* s) {
    const l2_model* m = s->m;
    if (!m->use_token_kernel) return false;
    return m->tp_world == 1 || (m->tp_direct && m->tp_pool_owner == s);
}

// Shared memory in front of the ring (the largest need of any phase) and the ring slots that fit behind it.  The next
// smaller carve-out (196 KB) leaves 60 KB of L1 instead of 28 KB, which the kernel's local memory (stack, the few spilled
// registers of 544 threads) and read-only operands need more than a fourth or fifth ring slot (measured: 3 slots of 35 KB beat
// 5 on the 7B model); the largest carve-out only where the ring would otherwise be shorter than three slots.
static size_t tk_fixed_bytes(const l2_state* s, bool gather13) {
    const l2_model* m = s->m;
    const l2_config& c = m->shape.c;
    size_t fixed = std::max<size_t>(token_attn_scratch_bytes(m->shape.attn_groups()), (size_t)c.dim * 4);
    for (int which = 0; which < 4; which++) {
        const SkLaunch& L = s->plans[which];  // every layer has the same shapes
        int max_g = 0;
        for (int i = 0; i < L.p.njobs; i++) max_g = std::max(max_g, L.p.job[i].G);
        // all inputs but w2's arrive in natural order
        fixed = std::max(fixed, token_gemv_smem(L.p.job[0].in, max_g, L.nseg, L.p.ptiles, which != 3, which == 2 && gather13));
    }
    return (fixed + 127) & ~(size_t)127;
}
static int tk_slots(const l2_state* s, size_t fixed, int su) {
    int slots = 0;
    size_t budget = 190 * 1024;
    if (const char* e = getenv("L2_TK_SMEM_KB")) budget = (size_t)std::max(64, std::min(222, atoi(e))) * 1024;  // tuning knob
    for (int attempt = 0; attempt < 2; attempt++, budget = 222 * 1024) {
        slots = fixed < budget ? (int)std::min<size_t>(SK_MAX_SLOTS, (budget - fixed) / sk_slot_bytes(s->m->shape.c.group_size, su)) : 0;
        if (slots >= 3) break;
    }
    return slots;
}
// w1 and w3 read one input through two different g_index orders.  Keeping the input once in natural order and gathering each
// matrix's blocks from it saves 4 * dim bytes of shared memory against two K-ordered copies, at the price of scattered
// shared-memory reads while the digits are cut.  It is used where it lets three ring slots fit into the smaller carve-out
// (13B and 70B shapes; measured on the 70B shapes: + 3 %, the same with three slots and 60 KB of L1 as with four slots and
// 28 KB), or where it buys a slot at all.
static bool tk_gather13(const l2_state* s) {
    const int su = 2 * SK_WARPS;
    if (const char* e = getenv("L2_TK_GATHER13")) return atoi(e) != 0;  // tuning knob
    // under tensor parallelism staging is a larger share of a token (the weight stream shrinks, the vectors do not) and the
    // gathered staging costs more than the larger L1 returns (70B on 4 GPUs: 148 tok/s without, 145 with)
    if (s->m->tp_world > 1) return false;
    const size_t with = tk_fixed_bytes(s, true), without = tk_fixed_bytes(s, false);
    const size_t three = 3 * sk_slot_bytes(s->m->shape.c.group_size, su), small = 190 * 1024;
    if (without + three > small && with + three <= small) return true;
    return tk_slots(s, with, su) > tk_slots(s, without, su);
}

// Ring geometry and shared-memory carve-up shared by every phase of the token kernel.
static int plan_token(l2_state* s) {
    l2_model* m = s->m;
    const l2_config& c = m->shape.c;
    const int su = 2 * SK_WARPS;  // unit records per slot fill: every consumer warp takes one pair
    const size_t fixed = tk_fixed_bytes(s, tk_gather13(s));
    int slots = tk_slots(s, fixed, su);
    if (slots < 2) return fail(L2_EINVAL, "the token kernel needs %zu bytes of shared memory before its weight ring", fixed);
    if (const char* e = getenv("L2_SK_SLOTS")) slots = std::max(2, std::min(slots, atoi(e)));
    s->tk = TokenParams{};
    s->tk.chunk = su;
    s->tk.slots = slots;
    s->tk.fixed_bytes = (unsigned)fixed;
    s->tk.status = &s->ctl->status;
    s->tk.ctl = s->ctl;
    s->tk.skip = (getenv("L2_SK_SKIP") ? 1 : 0) | (getenv("L2_SK_NOCOPY") ? 2 : 0);  // debugging: no arithmetic / no weight copies (results are wrong)
    s->tk_smem = fixed + (size_t)slots * sk_slot_bytes(c.group_size, su);
    {
        const int lg = m->opt.poll_limit_log2;
        if (lg && (lg < 8 || lg > 30)) return fail(L2_EINVAL, "poll_limit_log2 %d outside 8..30", lg);
        L2_CUDA(token_set_poll_limit(lg ? 1u << lg : 0u));
    }
    if (int rc = dev_alloc(reinterpret_cast<void**>(&s->tk.bar), 256, s->allocs)) return rc;
    L2_CUDA(cudaMemset(s->tk.bar, 0, 256));
    {   // tagged activations, zeroed once: tag 0 is never expected
        const TaggedLayout lay = tagged_layout(m);
        char* pool = nullptr;
        if (m->tp_world > 1) {
            pool = m->tp_pool;  // made (and zeroed) by l2_model_tp_pool_handle, known to the peers
        } else {
            if (int rc = dev_alloc(reinterpret_cast<void**>(&pool), lay.total, s->allocs)) return rc;
            L2_CUDA(cudaMemset(pool, 0, lay.total));
        }
        if (!pool) return fail(L2_EINVAL, "token kernel: no activation pool");
        unsigned long long** bufs[11] = {&s->t_x, &s->t_xq, &s->t_xk, &s->t_xv, &s->t_q, &s->t_k, &s->t_v, &s->t_att, &s->t_x1, &s->t_x3, &s->t_hb};
        for (int i = 0; i < 11; i++) *bufs[i] = reinterpret_cast<unsigned long long*>(pool + lay.off[i]);
        s->t_logits = lay.n[11] ? reinterpret_cast<unsigned long long*>(pool + lay.off[11]) : nullptr;
        // attention: the sequence of a kv head is split over the CTAs (one item per CTA at most); partial results per head and split
        s->tk_max_split = std::max(1, std::min(32, m->sms / std::max(1, c.n_kv_heads / m->tp_world)));
        const size_t part_bytes = (size_t)c.n_heads * s->tk_max_split * (HS + 2) * 8;
        if (int rc = dev_alloc(reinterpret_cast<void**>(&s->t_part), part_bytes, s->allocs)) return rc;
        L2_CUDA(cudaMemset(s->t_part, 0, part_bytes));
        s->tk.world = m->tp_world;
        s->tk.rank = m->tp_rank;
        for (int r = 0; r < 8; r++) s->tk.pool[r] = r < m->tp_world ? (m->tp_world > 1 ? m->tp_peers[r] : pool) : nullptr;
    }
    return L2_OK;
}

static int build_phase_table(l2_state* s, int kind) {
    l2_model* m = s->m;
    const l2_config& c = m->shape.c;
    std::vector<PhaseRec> t;
    auto add = [&](int type) -> PhaseRec& {
        t.emplace_back();
        memset(&t.back(), 0, sizeof(PhaseRec));
        t.back().type = type;
        return t.back();
    };
    // the token kernel's copies of the activation vectors: (value, tag) pairs instead of floats
    const TaggedLayout lay = tagged_layout(m);
    auto tg = [&](const float* plain) -> float* {  // a pointer into a plain vector -> the same element of its tagged copy
        const struct { const float* f; unsigned long long* t; } map[11] = {{s->x, s->t_x}, {s->xq, s->t_xq}, {s->xk, s->t_xk}, {s->xv, s->t_xv},
                                                                            {s->q, s->t_q}, {s->k, s->t_k}, {s->v, s->t_v}, {s->att, s->t_att},
                                                                            {s->x1, s->t_x1}, {s->x3, s->t_x3}, {s->hb, s->t_hb}};
        for (int i = 0; i < 11; i++)
            if (plain >= map[i].f && plain < map[i].f + lay.n[i]) return reinterpret_cast<float*>(map[i].t + (plain - map[i].f));
        return nullptr;
    };
    const bool direct = m->tp_world > 1;
    bool bad = false;
    auto must = [&](float* p) { if (!p) bad = true; return p; };
    {
        EmbedParams e = embed_params(s, kind);
        e.x = must(tg(e.x));
        e.nscatter = 0;
        add(PH_EMBED).u.em = e;
    }
    int x_phase = 0;  // the phase that last wrote the residual stream (and its copies for the next consumer)
    for (int l = 0; l < c.n_layers; l++) {
        int qkv_phase = 0, attn_phase = 0, w13_phase = 0;
        for (int which = 0; which < 4; which++) {
            SkLaunch L;
            if (int rc = plan_layer_gemv(s, l, which, L, direct)) return rc;
            const int me = (int)t.size();
            PhaseRec& r = add(L.nseg == 2 ? PH_GEMV2 : PH_GEMV1);
            r.u.sk = L.p;
            r.u.sk.trace = nullptr;
            r.u.sk.n_next = 0;
            const int in_phase = which == 0 ? x_phase : which == 1 ? attn_phase : which == 2 ? x_phase : w13_phase;
            // Inputs travel in natural order (one writer per 128-byte line) and are gathered into each matrix's K order by
            // the consumer through its g_index; only w2 reads a vector that its producers (w1/w3, whose rows are stored in
            // w2's K order) already write in the right order.
            const DevLayer& y = m->layers[l];
            auto p16 = [](const DevQ& q) { return reinterpret_cast<const int*>(q.inv16); };
            auto f16 = [](const DevQ& q) { return reinterpret_cast<const int*>(q.perm16); };
            const bool g13 = tk_gather13(s);
            const int* perms[4][3] = {{p16(y.wq), p16(y.wk), p16(y.wv)}, {p16(y.wo), nullptr, nullptr},
                                      {g13 ? f16(y.w1) : p16(y.w1), g13 ? f16(y.w3) : p16(y.w3), nullptr}, {nullptr, nullptr, nullptr}};
            const float* norms[4] = {y.rms_att, nullptr, y.rms_ffn, nullptr};
            if (c.dim >= 65536) return fail(L2_EINVAL, "token kernel: DIM %d does not fit 16-bit gather indices", c.dim);
            float* inputs[4] = {reinterpret_cast<float*>(s->t_x), reinterpret_cast<float*>(s->t_att), reinterpret_cast<float*>(s->t_x), reinterpret_cast<float*>(s->t_hb)};
            for (int j = 0; j < r.u.sk.njobs; j++) {
                SkJob& J = r.u.sk.job[j];
                for (int sg = 0; sg < L.nseg; sg++) {
                    J.seg[sg].x = inputs[which];
                    J.seg[sg].perm = perms[which][which == 2 ? sg : j];
                    J.gather = which == 2 && g13 ? 1 : 0;
                    J.seg[sg].nw = norms[which];
                    J.in_phase[sg] = in_phase;
                }
                J.out = must(tg(J.out));
                J.nscatter = 0;
                J.resid_phase = x_phase;
                J.bcast = direct && which != 0;  // q/k/v stay with the rank that owns the heads; everything else every rank needs
            }
            if (which == 0) {
                qkv_phase = me;
                attn_phase = (int)t.size();
                AttnParams a = attention_params(s, l, direct);
                a.q = must(tg(a.q)); a.k = must(tg(a.k)); a.v = must(tg(a.v));
                a.out = reinterpret_cast<float*>(s->t_att);  // natural order: wo gathers it through its g_index
                a.oidx = nullptr;
                a.in_phase = qkv_phase;
                a.bcast = direct;
                a.part = reinterpret_cast<float*>(s->t_part);
                a.max_split = s->tk_max_split;
                a.split_min = 32;  // positions a split holds at least (measured: 16..32 is best, a split costs a second exchange)
                if (const char* e = getenv("L2_TK_SPLIT_MIN")) a.split_min = std::max(1, atoi(e));  // tuning knob
                add(PH_ATTN).u.at = a;
            } else if (which == 1) {
                x_phase = me;  // wo wrote x (+ copies for w1/w3)
            } else if (which == 2) {
                w13_phase = me;
            } else {
                x_phase = me;  // w2 wrote x (+ copies for the next layer's q/k/v)
            }
        }
    }
    int cls_phase_index = -1;
    if (kind == G_DECODE || kind == G_FWD_CLS) {
        ClsParams cp = classifier_params(s);
        cp.x = must(tg(cp.x));
        cp.in_phase = x_phase;
        if (direct && s->t_logits) {  // vocabulary-parallel: this rank's slice of the rows, results to every rank as tagged values
            int row0 = 0, nrows = c.vocab_size;
            row0 = (int)((long long)c.vocab_size * m->tp_rank / m->tp_world);
            nrows = (int)((long long)c.vocab_size * (m->tp_rank + 1) / m->tp_world) - row0;
            cp.row0 = row0; cp.rows = nrows; cp.tagged = s->t_logits;
        }
        cls_phase_index = (int)t.size();
        PhaseRec& r = add(PH_CLS);
        r.u.cl = cp;
        r.barrier_after = 1;  // the selection reads every logit
    }
    if (kind == G_DECODE || (kind == G_FWD_CLS && direct && s->t_logits)) {
        SelectParams sp{};
        sp.logits = s->logits; sp.ctl = s->ctl; sp.prompt = s->prompt; sp.out_tokens = s->out_tokens; sp.vocab = c.vocab_size;
        if (direct && s->t_logits) { sp.tagged = s->t_logits; sp.tagged_phase = cls_phase_index; }
        sp.collect_only = kind == G_FWD_CLS ? 1 : 0;
        add(PH_SELECT).u.se = sp;
    } else if (kind == G_FEED) {
        add(PH_ADVANCE).u.se.ctl = s->ctl;
    }
    if (bad) return fail(L2_EINVAL, "token kernel: an activation buffer of the launch plan has no tagged counterpart");
    if (t.size() >= 1024) return fail(L2_EINVAL, "token kernel: %zu phases do not fit the 10-bit phase field of a tag", t.size());
    if (int rc = dev_alloc(reinterpret_cast<void**>(&s->d_phases[kind]), sizeof(PhaseRec) * t.size(), s->allocs)) return rc;
    L2_CUDA(cudaMemcpy(s->d_phases[kind], t.data(), sizeof(PhaseRec) * t.size(), cudaMemcpyHostToDevice));
    s->n_phases[kind] = (int)t.size();
    return L2_OK;
}

static int enqueue_token(l2_state* s, int kind, cudaStream_t st) {
    l2_model* m = s->m;
    TokenParams tk = s->tk;
    tk.phases = s->d_phases[kind];
    tk.nphases = s->n_phases[kind];
    tk.trace = s->tk_trace && (size_t)m->sms * tk.nphases * TK_TRACE_W <= s->tk_trace_count ? s->tk_trace : nullptr;
    L2_CUDA(launch_token(tk, m->shape.c.group_size, m->shape.attn_groups(), m->sms, s->tk_smem, st));
    return L2_OK;
}

static int enqueue_forward(l2_state* s, int kind, cudaStream_t st) {
    l2_model* m = s->m;
    const l2_config& c = m->shape.c;
    if (token_path(s)) return enqueue_token(s, kind, st);
    const bool pdl = m->use_pdl;
    const int L = c.n_layers, D = c.dim;
    launch_embed(embed_params(s, kind), st, false);  // first node of the token: plain stream order
    const int T = m->tp_world;
    for (int l = 0; l < L; l++) {
        const DevLayer& y = m->layers[l];
        launch_qkv(s, l, st, pdl);
        launch_attention(s, l, st, pdl);
        if (T > 1) {  // every rank holds its heads' outputs: gather, then bring into wo's K order
            if (int rc = tp_all_gather(m, s->att_nat, (size_t)D / T, st)) return rc;
            float* dst[1] = {s->att};
            const int* idx[1] = {y.wo.inv};
            launch_scatter(s->att_nat, D, dst, idx, 1, st, false);
        }
        launch_wo(s, l, st, pdl);
        if (T > 1) {
            if (int rc = tp_all_gather(m, s->x, (size_t)D / T, st)) return rc;
            float* dst[2] = {s->x1, s->x3};
            const int* idx[2] = {y.w1.inv, y.w3.inv};
            launch_scatter(s->x, D, dst, idx, 2, st, false);
        }
        launch_w13(s, l, st, pdl);
        if (T > 1) {
            if (int rc = tp_all_gather(m, s->hb, (size_t)c.hidden_dim / T, st)) return rc;
        }
        launch_w2(s, l, st, T > 1 ? false : pdl);
        if (T > 1) {
            if (int rc = tp_all_gather(m, s->x, (size_t)D / T, st)) return rc;
            if (l + 1 < L) {
                const DevLayer& nx = m->layers[l + 1];
                float* dst[3] = {s->xq, s->xk, s->xv};
                const int* idx[3] = {nx.wq.inv, nx.wk.inv, nx.wv.inv};
                launch_scatter(s->x, D, dst, idx, 3, st, false);
            }
        }
    }
    if (kind == G_DECODE || kind == G_FWD_CLS) launch_classifier(s, st, pdl);  // final rmsnorm + classifier (:288-297)
    if (kind == G_DECODE) {
        SelectParams sp{};
        sp.logits = s->logits; sp.ctl = s->ctl; sp.prompt = s->prompt; sp.out_tokens = s->out_tokens; sp.vocab = c.vocab_size;
        launch_select(sp, st, pdl);
    } else if (kind == G_FEED) {
        launch_advance(s->ctl, st, pdl);
    }
    L2_CUDA(cudaGetLastError());
    return L2_OK;
}

static int nodes_per_forward(const l2_state* s, int kind) {
    const l2_model* m = s->m;
    if (token_path(s)) return 1;
    const int L = m->shape.c.n_layers;
    int n = 1 + 5 * L;
    if (m->tp_world > 1) n += 3 * L - 1;  // the copies into the consumers' K orders after each all-gather
    if (kind == G_DECODE) n += 2;
    if (kind == G_FWD_CLS || kind == G_FEED) n += 1;
    return n;
}

// Runs one forward of the given kind on the model's stream (graph replay unless disabled).
static int run_forward(l2_state* s, int kind) {
    l2_model* m = s->m;
    if (m->tp_direct && !m->tp_pool_owner) m->tp_pool_owner = s;  // the first state that runs works in the model's pool
    if (token_path(s) && !s->d_phases[kind]) {
        if (!s->tk.bar)
            if (int rc = plan_token(s)) return rc;
        if (int rc = build_phase_table(s, kind)) return rc;
    }
    if (!m->use_graph) return enqueue_forward(s, kind, m->stream);
    if (!s->graphs[kind]) {
        cudaStream_t cap;
        L2_CUDA(cudaStreamCreateWithFlags(&cap, cudaStreamNonBlocking));
        const unsigned long long before = g_launches;
        L2_CUDA(cudaStreamBeginCapture(cap, cudaStreamCaptureModeThreadLocal));
        int rc = enqueue_forward(s, kind, cap);
        cudaGraph_t graph = nullptr;
        cudaError_t e = cudaStreamEndCapture(cap, &graph);
        g_launches = before;  // captured launches have not run
        if (rc != L2_OK) { if (graph) cudaGraphDestroy(graph); cudaStreamDestroy(cap); return rc; }
        if (e != cudaSuccess) { cudaStreamDestroy(cap); return fail(L2_ECUDA, "graph capture failed: %s", cudaGetErrorString(e)); }
        e = cudaGraphInstantiate(&s->graphs[kind], graph, 0);
        cudaGraphDestroy(graph);
        cudaStreamDestroy(cap);
        if (e != cudaSuccess) return fail(L2_ECUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
        s->graph_nodes[kind] = nodes_per_forward(s, kind);
    }
    L2_CUDA(cudaGraphLaunch(s->graphs[kind], m->stream));
    g_launches += s->graph_nodes[kind];
    return L2_OK;
}

static int write_ctl(l2_state* s, int pos, int token, int n_prompt, int force, float temperature, uint64_t rng) {
    // Each upload needs its own pinned record until the copy has run: cycle through a ring
    // (slot 0 is kept for read-backs) and drain the stream when it wraps.
    if (++s->ctl_slot >= CTL_RING) {
        L2_CUDA(cudaStreamSynchronize(s->m->stream));
        s->ctl_slot = 1;
    }
    Ctl* h = s->h_ctl + s->ctl_slot;
    memset(h, 0, sizeof(Ctl));
    h->pos = pos; h->token = token; h->n_prompt = n_prompt; h->force = force;
    h->temperature = temperature; h->rng = rng; h->last_next = -1;
    L2_CUDA(cudaMemcpyAsync(s->ctl, h, sizeof(Ctl), cudaMemcpyHostToDevice, s->m->stream));
    return L2_OK;
}

static int upload_prompt(l2_state* s, const int32_t* prompt, int n_prompt) {
    const l2_config& c = s->m->shape.c;
    if (n_prompt < 0 || n_prompt > c.seq_len) return fail(L2_ERANGE, "prompt of %d tokens exceeds SEQ_LEN %d", n_prompt, c.seq_len);
    for (int i = 0; i < n_prompt; i++)
        if (prompt[i] < 0 || prompt[i] >= c.vocab_size) return fail(L2_ERANGE, "prompt token %d out of range", prompt[i]);
    if (n_prompt) L2_CUDA(cudaMemcpyAsync(s->prompt, prompt, sizeof(int) * n_prompt, cudaMemcpyHostToDevice, s->m->stream));
    return L2_OK;
}

}  // namespace l2

// ---- C ABI: model -------------------------------------------------------------------------------

extern "C" uint64_t l2_launch_count(void) { return g_launches; }

static int resolve_shape(const l2_options* opt, const int32_t* header, Shape* out) {
    // Config::load + check_static (src/constants.rs:94-119); n_kv_heads in the file is ignored.
    l2_config c{};
    c.dim = header[0]; c.hidden_dim = header[1]; c.n_layers = header[2]; c.n_heads = header[3];
    c.vocab_size = header[5] < 0 ? -header[5] : header[5];
    c.seq_len = header[6];
    c.group_size = opt && opt->group_size ? opt->group_size : 128;
    if (opt && opt->model_size) {
        l2_config p;
        if (int rc = l2_preset_config(opt->model_size, c.group_size, &p)) return rc;
        if (p.dim != c.dim || p.hidden_dim != c.hidden_dim || p.n_layers != c.n_layers || p.n_heads != c.n_heads || p.vocab_size != c.vocab_size)
            return fail(L2_EFORMAT, "checkpoint header (dim %d, hidden %d, layers %d, heads %d, vocab %d) does not match model size %s",
                        c.dim, c.hidden_dim, c.n_layers, c.n_heads, c.vocab_size, opt->model_size);
        c.n_kv_heads = p.n_kv_heads;
    } else {
        const int ag = opt && opt->attn_groups > 0 ? opt->attn_groups : 1;
        if (c.n_heads <= 0 || c.n_heads % ag) return fail(L2_EFORMAT, "attn_groups %d does not divide n_heads %d", ag, c.n_heads);
        c.n_kv_heads = c.n_heads / ag;
    }
    if (int rc = validate_config(c)) return rc;
    out->c = c;
    return L2_OK;
}

extern "C" int l2_model_open_blob(const l2_config* c, const void* payload, size_t nbytes, const l2_options* opt, l2_model** out) {
    clear_error();
    if (!c || !payload || !out) return fail(L2_EINVAL, "l2_model_open_blob: null argument");
    if (int rc = validate_config(*c)) return rc;
    Shape s{*c};
    if (nbytes != s.total_words() * 4)  // src/lib.rs:97
        return fail(L2_EFORMAT, "payload is %zu bytes, QTransformerWeights for this configuration is %zu", nbytes, s.total_words() * 4);
    BlobSource src(s, payload);
    return build_model(s, src, opt, out);
}

extern "C" int l2_model_open(const char* checkpoint, const l2_options* opt, l2_model** out) {
    clear_error();
    if (!checkpoint || !out) return fail(L2_EINVAL, "l2_model_open: null argument");
    int fd = open(checkpoint, O_RDONLY);
    if (fd < 0) return fail(L2_EIO, "cannot open %s", checkpoint);
    struct stat st;
    int32_t header[7];
    if (fstat(fd, &st) != 0 || st.st_size < (off_t)sizeof header || read(fd, header, sizeof header) != (ssize_t)sizeof header) {
        close(fd);
        return fail(L2_EIO, "cannot read the header of %s", checkpoint);
    }
    Shape s;
    if (int rc = resolve_shape(opt, header, &s)) { close(fd); return rc; }
    const size_t payload = (size_t)st.st_size - sizeof header;
    if (payload != s.total_words() * 4) {
        close(fd);
        return fail(L2_EFORMAT, "%s holds %zu payload bytes, QTransformerWeights for this configuration is %zu", checkpoint, payload, s.total_words() * 4);
    }
    void* map = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) return fail(L2_EIO, "mmap of %s failed", checkpoint);
    BlobSource src(s, static_cast<const char*>(map) + sizeof header);
    int rc = build_model(s, src, opt, out);
    munmap(map, (size_t)st.st_size);  // everything lives on the device now
    return rc;
}

extern "C" int l2_model_open_synthetic(const l2_config* c, uint64_t seed, const l2_options* opt, l2_model** out) {
    clear_error();
    if (!c || !out) return fail(L2_EINVAL, "l2_model_open_synthetic: null argument");
    if (int rc = validate_config(*c)) return rc;
    Shape s{*c};
    const int world = opt && opt->tp_world > 1 ? opt->tp_world : 1;
    SynthSource src(s, seed, std::max(1, default_threads() / world));  // ranks of one box share the host cores
    return build_model(s, src, opt, out);
}

extern "C" void l2_model_close(l2_model* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    if (m->gen_state) l2_state_free(m->gen_state);
    for (int r = 0; r < 8; r++)
        if (m->tp_peers[r] && r != m->tp_rank && !m->tp_peer_borrowed[r]) cudaIpcCloseMemHandle(m->tp_peers[r]);
    if (m->tp_pool) cudaFree(m->tp_pool);
    tp_disconnect(m);
    free_allocs(m->allocs);
    if (m->own_stream) cudaStreamDestroy(m->own_stream);
    delete m;
}

// ---- tensor parallelism over peer memory ----------------------------------------------------------
extern "C" int l2_model_tp_pool_handle(l2_model* m, void* handle64) {
    clear_error();
    if (!m || !handle64) return fail(L2_EINVAL, "l2_model_tp_pool_handle: null argument");
    if (m->tp_world <= 1) return fail(L2_EINVAL, "l2_model_tp_pool_handle: the model is not tensor parallel");
    L2_CUDA(cudaSetDevice(m->device));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
    if (!m->tp_pool) {
        const TaggedLayout lay = tagged_layout(m);
        L2_CUDA(cudaMalloc(reinterpret_cast<void**>(&m->tp_pool), lay.total));
        L2_CUDA(cudaMemset(m->tp_pool, 0, lay.total));
        m->tp_peers[m->tp_rank] = m->tp_pool;
        for (int i = 0; i < 3; i++) m->tp_batch_off[i] = lay.batch_off[i];
        m->tp_flag_off = lay.flag_off;
    }
    cudaIpcMemHandle_t h;
    L2_CUDA(cudaIpcGetMemHandle(&h, m->tp_pool));
    memcpy(handle64, &h, sizeof h);
    return L2_OK;
}

extern "C" int l2_model_tp_pool_attach(l2_model* m, int rank, const void* handle64) {
    clear_error();
    if (!m || !handle64) return fail(L2_EINVAL, "l2_model_tp_pool_attach: null argument");
    if (rank < 0 || rank >= m->tp_world || m->tp_world > 8) return fail(L2_EINVAL, "l2_model_tp_pool_attach: rank %d outside 0..%d", rank, m->tp_world - 1);
    if (!m->tp_pool) return fail(L2_EINVAL, "l2_model_tp_pool_attach: call l2_model_tp_pool_handle first");
    L2_CUDA(cudaSetDevice(m->device));
    if (rank != m->tp_rank && !m->tp_peers[rank]) {
        cudaIpcMemHandle_t h;
        memcpy(&h, handle64, sizeof h);
        void* p = nullptr;
        L2_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        m->tp_peers[rank] = static_cast<char*>(p);
    }
    bool all = true;
    for (int r = 0; r < m->tp_world; r++) all = all && m->tp_peers[r];
    m->tp_direct = all;
    return L2_OK;
}

extern "C" size_t l2_model_tp_pool_bytes(const l2_model* m) { return m && m->tp_world > 1 ? tagged_layout(m).total : 0; }

extern "C" int l2_model_tp_pool_attach_ptr(l2_model* m, int rank, void* device_ptr) {
    clear_error();
    if (!m || !device_ptr) return fail(L2_EINVAL, "l2_model_tp_pool_attach_ptr: null argument");
    if (rank < 0 || rank >= m->tp_world || rank == m->tp_rank) return fail(L2_EINVAL, "l2_model_tp_pool_attach_ptr: rank %d is not a peer (0..%d, own rank %d)", rank, m->tp_world - 1, m->tp_rank);
    if (!m->tp_pool) return fail(L2_EINVAL, "l2_model_tp_pool_attach_ptr: call l2_model_tp_pool_handle first");
    if (m->tp_peers[rank]) return fail(L2_EINVAL, "l2_model_tp_pool_attach_ptr: rank %d is attached already", rank);
    m->tp_peers[rank] = static_cast<char*>(device_ptr);
    m->tp_peer_borrowed[rank] = true;
    bool all = true;
    for (int r = 0; r < m->tp_world; r++) all = all && m->tp_peers[r];
    m->tp_direct = all;
    return L2_OK;
}

extern "C" int l2_model_config(const l2_model* m, l2_config* out) {
    if (!m || !out) return fail(L2_EINVAL, "l2_model_config: null argument");
    *out = m->shape.c;
    return L2_OK;
}

extern "C" int l2_model_prefill(const l2_model*) { return 1; }

extern "C" int l2_model_set_stream(l2_model* m, void* cuda_stream) {
    if (!m) return fail(L2_EINVAL, "l2_model_set_stream: null model");
    m->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : m->own_stream;
    return L2_OK;
}

extern "C" uint64_t l2_model_decode_bytes(const l2_model* m) {
    if (!m) return 0;
    uint64_t b = m->decode_bytes;
    if (m->tp_world > 1 && m->tp_direct) {  // vocabulary-parallel classifier: this rank streams its slice of the rows only
        const l2_config& c = m->shape.c;
        const long long row0 = (long long)c.vocab_size * m->tp_rank / m->tp_world, row1 = (long long)c.vocab_size * (m->tp_rank + 1) / m->tp_world;
        b -= (uint64_t)(c.vocab_size - (row1 - row0)) * c.dim * 4;
    }
    return b;
}

// ---- C ABI: run state ---------------------------------------------------------------------------

extern "C" int l2_state_new(l2_model* m, l2_state** out) {
    clear_error();
    if (!m || !out) return fail(L2_EINVAL, "l2_state_new: null argument");
    L2_CUDA(cudaSetDevice(m->device));
    std::unique_ptr<l2_state> s(new l2_state);
    s->m = m;
    const l2_config& c = m->shape.c;
    const size_t kvn = (size_t)c.n_layers * c.seq_len * m->shape.kv_dim();
    const int D = c.dim, KV = m->shape.kv_dim(), H = c.hidden_dim;
    auto A = [&](float** p, size_t n) { return dev_alloc(reinterpret_cast<void**>(p), n * sizeof(float), s->allocs); };
    int rc = 0;
    if ((rc = A(&s->kc, kvn)) || (rc = A(&s->vc, kvn)) || (rc = A(&s->x, D)) || (rc = A(&s->xq, D)) || (rc = A(&s->xk, D)) ||
        (rc = A(&s->xv, D)) || (rc = A(&s->q, D)) || (rc = A(&s->k, KV)) || (rc = A(&s->v, KV)) || (rc = A(&s->att, D)) || (rc = A(&s->att_nat, D)) ||
        (rc = A(&s->x1, D)) || (rc = A(&s->x3, D)) || (rc = A(&s->hb, H)) || (rc = A(&s->logits, c.vocab_size))) {
        free_allocs(s->allocs);
        return rc;
    }
    // enough (kv head, split) CTAs to cover the SMs about twice
    s->max_split = std::max(1, std::min(32, (2 * m->sms + c.n_kv_heads - 1) / c.n_kv_heads));
    if ((rc = A(&s->part, (size_t)c.n_heads * s->max_split * (HS + 2))) ||
        (rc = dev_alloc(reinterpret_cast<void**>(&s->counter), sizeof(unsigned) * c.n_kv_heads, s->allocs)) ||
        (rc = dev_alloc(reinterpret_cast<void**>(&s->ctl), sizeof(Ctl), s->allocs)) ||
        (rc = dev_alloc(reinterpret_cast<void**>(&s->prompt), sizeof(int) * c.seq_len, s->allocs)) ||
        (rc = dev_alloc(reinterpret_cast<void**>(&s->out_tokens), sizeof(int) * c.seq_len, s->allocs))) {
        free_allocs(s->allocs);
        return rc;
    }
    {   // plan the four GEMV launches of every layer once and keep their records on the device
        const int L = c.n_layers;
        s->plans.resize((size_t)L * 4);
        std::vector<SkParams> host((size_t)L * 4);
        if ((rc = dev_alloc(reinterpret_cast<void**>(&s->d_plans), sizeof(SkParams) * L * 4, s->allocs))) { free_allocs(s->allocs); return rc; }
        for (int l = 0; l < L; l++)
            for (int which = 0; which < 4; which++) {
                if ((rc = plan_layer_gemv(s.get(), l, which, s->plans[(size_t)l * 4 + which]))) { free_allocs(s->allocs); return rc; }
                host[(size_t)l * 4 + which] = s->plans[(size_t)l * 4 + which].p;
            }
        if (cudaMemcpy(s->d_plans, host.data(), sizeof(SkParams) * host.size(), cudaMemcpyHostToDevice) != cudaSuccess) {
            free_allocs(s->allocs);
            return fail(L2_ECUDA, "uploading the launch records failed");
        }
    }
    if (cudaMallocHost(reinterpret_cast<void**>(&s->h_ctl), sizeof(Ctl) * CTL_RING) != cudaSuccess) {
        free_allocs(s->allocs);
        return fail(L2_ECUDA, "cudaMallocHost failed");
    }
    l2_state* sp = s.release();
    if ((rc = l2_state_reset(sp))) { l2_state_free(sp); return rc; }
    *out = sp;
    return L2_OK;
}

extern "C" int l2_state_reset(l2_state* s) {
    if (!s) return fail(L2_EINVAL, "l2_state_reset: null state");
    l2_model* m = s->m;
    const l2_config& c = m->shape.c;
    const size_t kvn = (size_t)c.n_layers * c.seq_len * m->shape.kv_dim();
    L2_CUDA(cudaMemsetAsync(s->kc, 0, kvn * sizeof(float), m->stream));
    L2_CUDA(cudaMemsetAsync(s->vc, 0, kvn * sizeof(float), m->stream));
    L2_CUDA(cudaMemsetAsync(s->counter, 0, sizeof(unsigned) * c.n_kv_heads, m->stream));
    L2_CUDA(cudaMemsetAsync(s->ctl, 0, sizeof(Ctl), m->stream));
    L2_CUDA(cudaMemsetAsync(s->prompt, 0, sizeof(int) * c.seq_len, m->stream));
    L2_CUDA(cudaMemsetAsync(s->out_tokens, 0, sizeof(int) * c.seq_len, m->stream));
    if (s->tk.bar) {
        // grid-barrier bookkeeping of the token kernel (a launch that gave up may have left it uneven);
        // the launch count behind the tags keeps running, so stale activations can never match
        L2_CUDA(cudaMemsetAsync(s->tk.bar, 0, sizeof(unsigned), m->stream));
        L2_CUDA(cudaMemsetAsync(s->tk.bar + 33, 0, sizeof(unsigned), m->stream));
    }
    L2_CUDA(cudaStreamSynchronize(m->stream));
    s->failed_status = 0;
    return L2_OK;
}

extern "C" void l2_state_free(l2_state* s) {
    if (!s) return;
    cudaSetDevice(s->m->device);
    for (auto& g : s->graphs) if (g) cudaGraphExecDestroy(g);
    free_allocs(s->allocs);
    if (s->h_ctl) cudaFreeHost(s->h_ctl);
    if (s->batch) {
        if (s->batch->h_stage) cudaFreeHost(s->batch->h_stage);
        for (int i = 0; i < 2; i++) {
            if (s->batch->aux[i]) cudaStreamDestroy(s->batch->aux[i]);
            if (s->batch->join[i]) cudaEventDestroy(s->batch->join[i]);
        }
        if (s->batch->fork) cudaEventDestroy(s->batch->fork);
        for (auto& row : s->batch->graph)
            for (cudaGraphExec_t g : row)
                if (g) cudaGraphExecDestroy(g);
        delete s->batch;
    }
    if (s->m->gen_state == s) s->m->gen_state = nullptr;
    if (s->m->tp_pool_owner == s) s->m->tp_pool_owner = nullptr;
    delete s;
}

extern "C" int l2_state_read_kv(l2_state* s, int layer, float* key_cache, float* value_cache) {
    if (!s) return fail(L2_EINVAL, "l2_state_read_kv: null state");
    const l2_config& c = s->m->shape.c;
    if (layer < 0 || layer >= c.n_layers) return fail(L2_ERANGE, "layer %d out of range", layer);
    const size_t ls = (size_t)c.seq_len * s->m->shape.kv_dim();
    L2_CUDA(cudaStreamSynchronize(s->m->stream));
    if (key_cache) L2_CUDA(cudaMemcpy(key_cache, s->kc + layer * ls, ls * sizeof(float), cudaMemcpyDeviceToHost));
    if (value_cache) L2_CUDA(cudaMemcpy(value_cache, s->vc + layer * ls, ls * sizeof(float), cudaMemcpyDeviceToHost));
    return L2_OK;
}

// ---- C ABI: forward, prefill, decode --------------------------------------------------------------

static int check_state(l2_model* m, l2_state* s, const char* who) {
    if (!m || !s) return fail(L2_EINVAL, "%s: null handle", who);
    if (s->m != m) return fail(L2_EINVAL, "%s: the state belongs to another model", who);
    if (s->failed_status) return fail(L2_ESTATUS, "%s: an earlier call on this state ended with device status %d; call l2_state_reset first", who, s->failed_status);
    L2_CUDA(cudaSetDevice(m->device));
    return L2_OK;
}

static int check_status(l2_state* s);
static int report_status(l2_state* s);

extern "C" int l2_forward(l2_model* m, l2_state* s, const int32_t* tokens, const int32_t* pos, int B, float* logits) {
    clear_error();
    if (int rc = check_state(m, s, "l2_forward")) return rc;
    const l2_config& c = m->shape.c;
    const int maxb = m->opt.max_batch > 0 ? std::min(m->opt.max_batch, (int)MAX_BATCH) : (int)MAX_BATCH;
    if (!tokens || !pos || B < 1 || B > maxb) return fail(L2_EINVAL, "l2_forward: bad batch (B=%d, max %d)", B, maxb);
    for (int b = 0; b < B; b++) {
        if (pos[b] < 0 || pos[b] >= c.seq_len) return fail(L2_ERANGE, "l2_forward: position %d outside 0..%d", pos[b], c.seq_len - 1);
        if (tokens[b] < 0 || tokens[b] >= c.vocab_size) return fail(L2_ERANGE, "l2_forward: token %d outside the vocabulary", tokens[b]);
        for (int a = 0; a < b; a++)
            if (pos[a] == pos[b]) return fail(L2_EINVAL, "l2_forward: two rows of a batch share position %d", pos[b]);
    }
    if (B == 1) {
        if (int rc = write_ctl(s, pos[0], tokens[0], 0, -1, 0.f, 0)) return rc;
        if (int rc = run_forward(s, logits ? G_FWD_CLS : G_FWD)) return rc;
    } else if (m->tp_world > 1) {
        // one row at a time, each seeing the rows before it: equal to the reference when positions ascend
        for (int b = 0; b < B; b++) {
            if (b && pos[b] <= pos[b - 1]) return fail(L2_EINVAL, "l2_forward: tensor parallel batches need ascending positions");
            if (int rc = write_ctl(s, pos[b], tokens[b], 0, -1, 0.f, 0)) return rc;
            if (int rc = run_forward(s, G_FWD)) return rc;
        }
    } else if (int rc = forward_batch(s, B, tokens, pos)) {  // all rows stored, then attention over 0..=pos[b]
        return rc;
    }
    if (B == 1 && logits) L2_CUDA(cudaMemcpyAsync(logits, s->logits, sizeof(float) * c.vocab_size, cudaMemcpyDeviceToHost, m->stream));
    if (B > 1) return check_status(s);
    L2_CUDA(cudaStreamSynchronize(m->stream));
    return L2_OK;
}

static int prefill_async(l2_model* m, l2_state* s, const int32_t* prompt, int n_prompt, int chunk, int32_t* pos_out) {
    if (int rc = upload_prompt(s, prompt, n_prompt)) return rc;
    // Positions the reference's ladder 64/32/16/8/4/2 covers (src/inference.rs:24, 78-127): the B=1 loop
    // must start where it starts there.  How those positions are cut into batches does not change the
    // cache ("should lead to identical results", src/inference.rs:12-15), so they go in batches of up to
    // MAX_BATCH rows.
    static const int ladder[6] = {64, 32, 16, 8, 4, 2};
    int target = 0;
    if (chunk > 0) { while (target + chunk < n_prompt) target += chunk; }
    else for (int a : ladder) while (target + a < n_prompt) target += a;
    int pos = 0;
    int32_t tokens[MAX_BATCH], positions[MAX_BATCH];
    while (pos < target) {
        // tensor parallel models run the batched path when the ranks are connected through peer memory (the exchanges are
        // stores into the peers' pools) and this state is the one that works in the pool; otherwise one position at a time
        if (m->tp_direct && !m->tp_pool_owner) m->tp_pool_owner = s;
        const bool batched = m->tp_world == 1 || (m->tp_direct && token_path(s));
        const int A = batched ? std::min<int>(MAX_BATCH, target - pos) : 1;
        for (int i = 0; i < A; i++) {
            tokens[i] = pos == 0 ? L2_START : prompt[pos - 1];  // src/inference.rs:29-35
            positions[i] = pos++;
        }
        if (A == 1) {
            if (int rc = write_ctl(s, positions[0], tokens[0], 0, -1, 0.f, 0)) return rc;
            if (int rc = run_forward(s, G_FWD)) return rc;
        } else if (int rc = forward_batch(s, A, tokens, positions)) {
            return rc;
        }
    }
    *pos_out = pos;
    return L2_OK;
}

// A device-side bounded wait gave up (h_ctl holds the record read back).  The launch left early: the
// grid-barrier count of the token kernel is uneven and, under tensor parallelism, the ranks' launch
// counts may differ.  The state refuses further forwards until l2_state_reset.
static int report_status(l2_state* s) {
    s->failed_status = s->h_ctl->status;
    return fail(L2_ESTATUS, "device status %d (a bounded wait on the device gave up); reset the state before using it again", s->h_ctl->status);
}

// Synchronises the stream and reports a device-side bounded wait that gave up.
static int check_status(l2_state* s) {
    L2_CUDA(cudaMemcpyAsync(s->h_ctl, s->ctl, sizeof(Ctl), cudaMemcpyDeviceToHost, s->m->stream));
    L2_CUDA(cudaStreamSynchronize(s->m->stream));
    if (s->h_ctl->status) return report_status(s);
    return L2_OK;
}

extern "C" int l2_prefill(l2_model* m, l2_state* s, const int32_t* prompt, int n_prompt, int chunk, int32_t* pos_out) {
    clear_error();
    if (int rc = check_state(m, s, "l2_prefill")) return rc;
    if ((!prompt && n_prompt) || !pos_out || chunk < 0) return fail(L2_EINVAL, "l2_prefill: bad argument");
    if (int rc = prefill_async(m, s, prompt, n_prompt, chunk, pos_out)) return rc;
    return check_status(s);
}

extern "C" int l2_decode_step(l2_model* m, l2_state* s, int32_t token, int32_t pos, float temperature, uint64_t* rng_seed,
                              int32_t forced_next, int32_t* next, float* logits) {
    clear_error();
    if (int rc = check_state(m, s, "l2_decode_step")) return rc;
    const l2_config& c = m->shape.c;
    if (pos < 0 || pos >= c.seq_len) return fail(L2_ERANGE, "l2_decode_step: position %d outside 0..%d", pos, c.seq_len - 1);
    if (token < 0 || token >= c.vocab_size) return fail(L2_ERANGE, "l2_decode_step: token %d outside the vocabulary", token);
    if (forced_next >= c.vocab_size) return fail(L2_ERANGE, "l2_decode_step: forced token outside the vocabulary");
    if (int rc = write_ctl(s, pos, token, 0, forced_next < 0 ? -1 : forced_next, temperature, rng_seed ? *rng_seed : 0)) return rc;
    if (int rc = run_forward(s, G_DECODE)) return rc;
    L2_CUDA(cudaMemcpyAsync(s->h_ctl, s->ctl, sizeof(Ctl), cudaMemcpyDeviceToHost, m->stream));
    if (logits) L2_CUDA(cudaMemcpyAsync(logits, s->logits, sizeof(float) * c.vocab_size, cudaMemcpyDeviceToHost, m->stream));
    L2_CUDA(cudaStreamSynchronize(m->stream));
    if (s->h_ctl->status) return report_status(s);
    if (next) *next = s->h_ctl->last_next;
    if (rng_seed) *rng_seed = s->h_ctl->rng;
    return L2_OK;
}

static int decode_run_async(l2_model* m, l2_state* s, const int32_t* prompt, int n_prompt, int pos0, int steps,
                            float temperature, uint64_t rng) {
    const int token = pos0 == 0 ? L2_START : prompt[pos0 - 1];  // src/inference.rs:128-132
    if (int rc = write_ctl(s, pos0, token, n_prompt, -1, temperature, rng)) return rc;
    for (int p = pos0; p < steps; p++)
        if (int rc = run_forward(s, G_DECODE)) return rc;
    return L2_OK;
}

extern "C" int l2_decode_run(l2_model* m, l2_state* s, const int32_t* prompt, int n_prompt, int32_t pos0, int32_t steps,
                             float temperature, uint64_t* rng_seed, int32_t* out_tokens) {
    clear_error();
    if (int rc = check_state(m, s, "l2_decode_run")) return rc;
    const l2_config& c = m->shape.c;
    if (steps > c.seq_len) return fail(L2_ERANGE, "steps %d exceeds SEQ_LEN %d", steps, c.seq_len);
    if (pos0 < 0 || pos0 > n_prompt || (!prompt && n_prompt)) return fail(L2_EINVAL, "l2_decode_run: bad prompt / start position");
    if (int rc = upload_prompt(s, prompt, n_prompt)) return rc;
    if (int rc = decode_run_async(m, s, prompt, n_prompt, pos0, steps, temperature, rng_seed ? *rng_seed : 0)) return rc;
    const int n = steps > pos0 ? steps - pos0 : 0;
    if (n && out_tokens) L2_CUDA(cudaMemcpyAsync(out_tokens, s->out_tokens + pos0, sizeof(int) * n, cudaMemcpyDeviceToHost, m->stream));
    L2_CUDA(cudaMemcpyAsync(s->h_ctl, s->ctl, sizeof(Ctl), cudaMemcpyDeviceToHost, m->stream));
    L2_CUDA(cudaStreamSynchronize(m->stream));
    if (s->h_ctl->status) return report_status(s);
    if (rng_seed) *rng_seed = s->h_ctl->rng;
    return L2_OK;
}

extern "C" int l2_generate_ids(l2_model* m, const int32_t* prompt, int n_prompt, int steps, float temperature,
                               uint64_t* rng_seed, int use_prefill, int32_t* out_tokens, int32_t* out_pos0,
                               float* logits_trace, double* elapsed_ms, double* prefill_ms, double* decode_ms) {
    clear_error();
    if (!m || !out_tokens || (!prompt && n_prompt)) return fail(L2_EINVAL, "l2_generate_ids: null argument");
    L2_CUDA(cudaSetDevice(m->device));
    const l2_config& c = m->shape.c;
    if (steps > c.seq_len) return fail(L2_ERANGE, "steps %d exceeds SEQ_LEN %d", steps, c.seq_len);
    if (!m->gen_state) {
        if (int rc = l2_state_new(m, &m->gen_state)) return rc;
    } else if (int rc = l2_state_reset(m->gen_state)) {  // fresh RunState per call (src/inference.rs:59)
        return rc;
    }
    l2_state* s = m->gen_state;
    cudaEvent_t e0, e1, e2;
    L2_CUDA(cudaEventCreate(&e0));
    L2_CUDA(cudaEventCreate(&e1));
    L2_CUDA(cudaEventCreate(&e2));
    int rc = L2_OK, pos0 = 0, n_out = 0;
    uint64_t rng = rng_seed ? *rng_seed : 0;
    do {
        if ((rc = upload_prompt(s, prompt, n_prompt))) break;
        cudaEventRecord(e0, m->stream);  // src/inference.rs:72
        if (use_prefill && ((rc = prefill_async(m, s, prompt, n_prompt, 0, &pos0)) || (pos0 > 0 && (rc = check_status(s))))) break;
        cudaEventRecord(e1, m->stream);
        n_out = steps > pos0 ? steps - pos0 : 0;
        if (!logits_trace) {
            if ((rc = decode_run_async(m, s, prompt, n_prompt, pos0, steps, temperature, rng))) break;
            if (n_out) cudaMemcpyAsync(out_tokens, s->out_tokens + pos0, sizeof(int) * n_out, cudaMemcpyDeviceToHost, m->stream);
            cudaMemcpyAsync(s->h_ctl, s->ctl, sizeof(Ctl), cudaMemcpyDeviceToHost, m->stream);
            cudaEventRecord(e2, m->stream);
            if (cudaStreamSynchronize(m->stream) != cudaSuccess) { rc = fail(L2_ECUDA, "decode failed: %s", cudaGetErrorString(cudaGetLastError())); break; }
            if (s->h_ctl->status) { rc = report_status(s); break; }  // a bounded wait gave up: the tokens are not valid
            rng = s->h_ctl->rng;
        } else {
            int token = pos0 == 0 ? L2_START : prompt[pos0 - 1];
            for (int p = pos0; p < steps; p++) {
                int next = 0;
                const int forced = p < n_prompt ? prompt[p] : -1;
                if ((rc = l2_decode_step(m, s, token, p, temperature, &rng, forced, &next, logits_trace + (size_t)(p - pos0) * c.vocab_size))) break;
                out_tokens[p - pos0] = next;
                token = next;
            }
            if (rc) break;
            cudaEventRecord(e2, m->stream);
            cudaStreamSynchronize(m->stream);
        }
        float a = 0.f, b = 0.f;
        cudaEventElapsedTime(&a, e0, e1);
        cudaEventElapsedTime(&b, e1, e2);
        if (prefill_ms) *prefill_ms = a;
        if (decode_ms) *decode_ms = b;
        if (elapsed_ms) *elapsed_ms = (double)a + b;
    } while (0);
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaEventDestroy(e2);
    if (rc) return rc;
    if (out_pos0) *out_pos0 = pos0;
    if (rng_seed) *rng_seed = rng;
    return n_out;
}

// Enqueues, for every layer in [layer0, layer0+count), the launch of one projection kernel of the
// token forward on the model's stream, so that a caller can time that kernel alone with events.
// which: 0 wq/wk/wv, 1 wo, 2 w1/w3+SwiGLU, 3 w2, 4 classifier (count launches), 5 attention.
extern "C" int l2_bench_projection(l2_model* m, l2_state* s, int which, int layer0, int count) {
    clear_error();
    if (int rc = check_state(m, s, "l2_bench_projection")) return rc;
    const int L = m->shape.c.n_layers;
    if (which < 0 || which > 5 || count < 0) return fail(L2_EINVAL, "l2_bench_projection: bad argument");
    for (int i = 0; i < count; i++) {
        const int l = (layer0 + i) % L;
        switch (which) {
            case 0: launch_qkv(s, l, m->stream, false); break;
            case 1: launch_wo(s, l, m->stream, false); break;
            case 2: launch_w13(s, l, m->stream, false); break;
            case 3: launch_w2(s, l, m->stream, false); break;
            case 4: launch_classifier(s, m->stream, false); break;
            default: launch_attention(s, l, m->stream, false); break;
        }
    }
    L2_CUDA(cudaGetLastError());
    return L2_OK;
}

// Debug: turns on per-CTA clock stamps in the GEMV kernels (n_ctas * 8 values: kernel entry, loads
// issued, dependency wait over, digits staged, main loop done, barrier passed, exit) or reads them back.
extern "C" int l2_debug_trace(int enable, unsigned long long* host_out, int n_ctas) {
    if (enable && !g_sk_trace) {
        L2_CUDA(cudaMalloc(&g_sk_trace, sizeof(unsigned long long) * 8 * 1024));
        L2_CUDA(cudaMemset(g_sk_trace, 0, sizeof(unsigned long long) * 8 * 1024));
    }
    if (host_out && g_sk_trace) {
        L2_CUDA(cudaDeviceSynchronize());
        L2_CUDA(cudaMemcpy(host_out, g_sk_trace, sizeof(unsigned long long) * 8 * std::min(n_ctas, 1024), cudaMemcpyDeviceToHost));
    }
    return L2_OK;
}

// Algorithmic bytes one launch of l2_bench_projection's kernel streams: the checkpoint's
// qweight + qzeros + scales of the projection(s), or the f32 classifier matrix.
extern "C" int l2_debug_token_trace(l2_state* s, int enable, unsigned long long* host_out, size_t count) {
    clear_error();
    if (!s) return fail(L2_EINVAL, "l2_debug_token_trace: null state");
    L2_CUDA(cudaSetDevice(s->m->device));
    L2_CUDA(cudaStreamSynchronize(s->m->stream));
    if (enable) {
        if (!s->tk_trace) {
            s->tk_trace_count = count;
            if (int rc = dev_alloc(reinterpret_cast<void**>(&s->tk_trace), count * 8, s->allocs)) return rc;
        }
        if (count > s->tk_trace_count) return fail(L2_EINVAL, "l2_debug_token_trace: the buffer holds %zu stamps", s->tk_trace_count);
        L2_CUDA(cudaMemset(s->tk_trace, 0, s->tk_trace_count * 8));
        for (auto& g : s->graphs)  // captured launches carry the old setting
            if (g) { cudaGraphExecDestroy(g); g = nullptr; }
        return L2_OK;
    }
    if (!s->tk_trace || !host_out || count > s->tk_trace_count) return fail(L2_EINVAL, "l2_debug_token_trace: nothing recorded");
    L2_CUDA(cudaMemcpy(host_out, s->tk_trace, count * 8, cudaMemcpyDeviceToHost));
    return L2_OK;
}

extern "C" uint64_t l2_projection_bytes(const l2_model* m, int which) {
    if (!m) return 0;
    const Shape& sh = m->shape;
    auto q = [&](int t) { return (uint64_t)(sh.sub_words(t, S_QWEIGHT) + sh.sub_words(t, S_QZEROS) + sh.sub_words(t, S_SCALES)) * 4 / m->tp_world; };  // this process's rows
    switch (which) {
        case 0: return q(T_WQ) + q(T_WK) + q(T_WV);
        case 1: return q(T_WO);
        case 2: return q(T_W1) + q(T_W3);
        case 3: return q(T_W2);
        case 4: return (uint64_t)sh.c.vocab_size * sh.c.dim * 4;
    }
    return 0;
}

// ---- C ABI: attention of one position on caller-owned device buffers ------------------------------

// Splits per kv head of the stand-alone attention entry points: enough (kv head, split) CTAs to cover the
// SMs of the current device about twice.  The SM count is read once per device.
int l2::device_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
        cached[dev] = n;
    }
    return cached[dev];
}
int l2::attention_max_split(int n_kv_heads) { return std::max(1, std::min(32, (2 * device_sm_count() + n_kv_heads - 1) / n_kv_heads)); }

extern "C" int l2_rope_table(int seq_len, float* cos_out, float* sin_out) {
    clear_error();
    if (seq_len <= 0 || !cos_out || !sin_out) return fail(L2_EINVAL, "l2_rope_table: bad argument");
    const int half = HS / 2;
    for (int p = 0; p < seq_len; p++)
        for (int i = 0; i < half; i++) {  // src/models.rs:107-110
            const float freq = 1.0f / powf(10000.0f, (float)(2 * i % HS) / (float)HS);
            const float val = (float)p * freq;
            cos_out[(size_t)p * half + i] = cosf(val);
            sin_out[(size_t)p * half + i] = sinf(val);
        }
    return L2_OK;
}

extern "C" size_t l2_attention_workspace_bytes(int n_heads, int n_kv_heads) {
    if (n_heads <= 0 || n_kv_heads <= 0) return 0;
    return 256 + (size_t)n_heads * attention_max_split(n_kv_heads) * (HS + 2) * sizeof(float);
}

int l2::check_attention_args(int n_heads, int n_kv_heads, int pos, const void* q, const void* k, const void* v, const void* kc,
                             const void* vc, const void* rc, const void* rs, const void* out) {
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return fail(L2_EINVAL, "attention: kv heads must divide heads");
    const int ag = n_heads / n_kv_heads;
    if (ag != 1 && ag != 2 && ag != 4 && ag != 8) return fail(L2_EINVAL, "attention: %d query heads per kv head unsupported (1, 2, 4 or 8)", ag);
    if (pos < 0) return fail(L2_ERANGE, "attention: negative position");
    if (!q || !k || !v || !kc || !vc || !rc || !rs || !out) return fail(L2_EINVAL, "attention: null device pointer");
    return L2_OK;
}

extern "C" int l2_attention_decode_dev(int n_heads, int n_kv_heads, int pos, const float* q, const float* k, const float* v,
                                       float* key_cache, float* value_cache, const float* rope_cos, const float* rope_sin,
                                       float* out, void* workspace, size_t workspace_bytes, void* cuda_stream) {
    clear_error();
    if (int rc = check_attention_args(n_heads, n_kv_heads, pos, q, k, v, key_cache, value_cache, rope_cos, rope_sin, out)) return rc;
    if (!workspace || workspace_bytes < l2_attention_workspace_bytes(n_heads, n_kv_heads))
        return fail(L2_EINVAL, "attention: workspace of %zu bytes needed", l2_attention_workspace_bytes(n_heads, n_kv_heads));
    if (n_kv_heads * sizeof(unsigned) > 256) return fail(L2_EINVAL, "attention: more than 64 kv heads");
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    L2_CUDA(cudaMemsetAsync(workspace, 0, 256, st));  // arrival tickets start at zero
    AttnParams a{};
    a.q = q; a.k = k; a.v = v; a.kc = key_cache; a.vc = value_cache;
    a.rope_cos = rope_cos; a.rope_sin = rope_sin;
    a.ctl = nullptr; a.pos_fixed = pos;
    a.counter = static_cast<unsigned*>(workspace);
    a.part = reinterpret_cast<float*>(static_cast<char*>(workspace) + 256);
    a.out = out; a.oidx = nullptr;
    a.n_kv_heads = n_kv_heads; a.ag = n_heads / n_kv_heads;
    a.max_split = attention_max_split(n_kv_heads); a.split_min = 64;
    launch_attn(a, st, false);
    L2_CUDA(cudaGetLastError());
    return L2_OK;
}

// ---- C ABI: one QLinear ---------------------------------------------------------------------------

extern "C" int l2_qlinear_create(int in, int out, int group_size, const int32_t* qweight, const int32_t* qzeros,
                                 const float* scales, const int32_t* g_index, int device, l2_qlinear** h) {
    clear_error();
    if (!qweight || !qzeros || !scales || !g_index || !h) return fail(L2_EINVAL, "l2_qlinear_create: null argument");
    if (in <= 0 || out <= 0 || in % 32 || out % 8) return fail(L2_EINVAL, "l2_qlinear_create: IN must be a multiple of 32 and OUT of 8");
    if (group_size != 32 && group_size != 64 && group_size != 128) return fail(L2_EINVAL, "group_size %d is not 32, 64 or 128", group_size);
    if (in % group_size) return fail(L2_EINVAL, "group size must divide IN");
    if ((size_t)in * 4 > 200 * 1024) return fail(L2_EINVAL, "IN %d does not fit the shared-memory staging", in);
    if (!is_permutation(g_index, in)) return fail(L2_EFORMAT, "g_index is not a permutation of 0..%d", in - 1);
    std::unique_ptr<l2_qlinear> q(new l2_qlinear);
    if (int rc = check_device(device, &q->device, &q->sms)) return rc;
    q->group_size = group_size;
    PackedQ p;
    repack_qlinear(in, out, group_size, qweight, qzeros, scales, nullptr, p);
    if (int rc = upload_qlinear(p, g_index, q->q, q->allocs, nullptr)) { free_allocs(q->allocs); return rc; }
    if (int rc = dev_alloc(reinterpret_cast<void**>(&q->d_plan), sizeof(SkParams), q->allocs)) { free_allocs(q->allocs); return rc; }
    L2_CUDA(cudaStreamCreateWithFlags(&q->stream, cudaStreamNonBlocking));
    *h = q.release();
    return L2_OK;
}

static int qlinear_reserve(l2_qlinear* h, int B) {
    if (B <= h->cap_b) return L2_OK;
    int rc;
    if ((rc = dev_alloc(reinterpret_cast<void**>(&h->x_dev), sizeof(float) * h->q.in * B, h->allocs))) return rc;
    if ((rc = dev_alloc(reinterpret_cast<void**>(&h->xp_dev), sizeof(float) * h->q.in * B, h->allocs))) return rc;
    if ((rc = dev_alloc(reinterpret_cast<void**>(&h->y_dev), sizeof(float) * h->q.out * B, h->allocs))) return rc;
    if (!h->img) {  // buffers of the batched (tcgen05) path, one chunk of MAX_BATCH tokens
        if ((rc = dev_alloc(reinterpret_cast<void**>(&h->img), gemm_tc_image_bytes(h->q.in, h->q.gs, MAX_BATCH), h->allocs))) return rc;
        if ((rc = dev_alloc(reinterpret_cast<void**>(&h->osc), sizeof(float) * MAX_BATCH, h->allocs))) return rc;
        if ((rc = dev_alloc(reinterpret_cast<void**>(&h->kpart), sizeof(float) * 4 * MAX_BATCH * h->q.out, h->allocs))) return rc;
        if ((rc = dev_alloc(reinterpret_cast<void**>(&h->status), sizeof(int), h->allocs))) return rc;
        L2_CUDA(cudaMemset(h->status, 0, sizeof(int)));
    }
    h->cap_b = B;
    return L2_OK;
}

extern "C" int l2_qlinear_matvec_dev(l2_qlinear* h, const float* x_dev, float* xout_dev, int B, void* cuda_stream) {
    clear_error();
    if (!h || !x_dev || !xout_dev || B < 1) return fail(L2_EINVAL, "l2_qlinear_matvec_dev: bad argument");
    L2_CUDA(cudaSetDevice(h->device));
    cudaStream_t st = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : h->stream;
    if (int rc = qlinear_reserve(h, B)) return rc;
    if (B >= 2) {  // batched: tensor-core GEMM, MAX_BATCH tokens at a time
        for (int b0 = 0; b0 < B; b0 += MAX_BATCH) {
            const int M = std::min<int>(MAX_BATCH, B - b0);
            if (int rc = gemm_batched(h->q, x_dev + (size_t)b0 * h->q.in, h->q.in, true, nullptr, 0.f, M, h->img, h->osc,
                                      xout_dev + (size_t)b0 * h->q.out, h->q.out, EPI_STORE, h->status, st, h->kpart, h->sms)) return rc;
        }
        return L2_OK;
    }
    for (int b = 0; b < B; b++) {
        launch_permute(x_dev + (size_t)b * h->q.in, h->q.perm, h->xp_dev + (size_t)b * h->q.in, h->q.in, st);
        if (int rc = run_gemv_single(h->q, h->xp_dev + (size_t)b * h->q.in, xout_dev + (size_t)b * h->q.out, h->sms, h->d_plan, st)) return rc;
    }
    return L2_OK;
}

extern "C" int l2_qlinear_matvec(l2_qlinear* h, const float* x, float* xout, int B) {
    clear_error();
    if (!h || !x || !xout || B < 1) return fail(L2_EINVAL, "l2_qlinear_matvec: bad argument");
    L2_CUDA(cudaSetDevice(h->device));
    if (int rc = qlinear_reserve(h, B)) return rc;
    L2_CUDA(cudaMemcpyAsync(h->x_dev, x, sizeof(float) * h->q.in * B, cudaMemcpyHostToDevice, h->stream));
    if (int rc = l2_qlinear_matvec_dev(h, h->x_dev, h->y_dev, B, h->stream)) return rc;
    L2_CUDA(cudaMemcpyAsync(xout, h->y_dev, sizeof(float) * h->q.out * B, cudaMemcpyDeviceToHost, h->stream));
    int status = 0;
    if (h->status) L2_CUDA(cudaMemcpyAsync(&status, h->status, sizeof(int), cudaMemcpyDeviceToHost, h->stream));
    L2_CUDA(cudaStreamSynchronize(h->stream));
    if (status) return fail(L2_ESTATUS, "device status %d", status);
    return L2_OK;
}

extern "C" void l2_qlinear_free(l2_qlinear* h) {
    if (!h) return;
    cudaSetDevice(h->device);
    free_allocs(h->allocs);
    if (h->stream) cudaStreamDestroy(h->stream);
    delete h;
}

extern "C" uint32_t l2_random_u32(uint64_t* seed) {  // src/util.rs:71-77
    uint64_t s = *seed;
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    *seed = s;
    return (uint32_t)((s * 0x2545F4914F6CDD1Dull) >> 32);
}
extern "C" float l2_random_f32(uint64_t* seed) { return (float)(l2_random_u32(seed) >> 8) / 16777216.0f; }
