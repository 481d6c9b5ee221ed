// Per-token kernels of the B=1 forward pass (src/models.rs:178-298), hand-written for sm_100a.
//
//   embed    token embedding row -> residual stream (+ copies in each consumer's K order)
//   (the fused rmsnorm + 4-bit dequant + GEMV for QLinear::matvec lives in gemv_kernels.cu)
//   attn     RoPE (src/models.rs:100-129) + KV append (:236-249) + GQA attention
//            (:131-176) with split-K over the sequence
//   cls      final rmsnorm + dense f32 classifier GEMV (src/model.rs:22-31)
//   select   forced / argmax / temperature sample (src/inference.rs:154-173, src/util.rs:39-113)
//
// All of them are HBM-bound streaming kernels: weights and caches are read once with 128-bit
// loads, activations live in shared memory, reductions are warp shuffles in a fixed order
// (results are bit-reproducible from run to run).
#include <cfloat>
#include <cmath>

#include "kernels.cuh"

namespace l2 {

unsigned long long g_launches = 0;

// ---- small device helpers --------------------------------------------------------------

// Programmatic dependent launch: wait until the kernels this one depends on have finished
// and their writes are visible (a no-op for a kernel launched without the attribute).
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Let the next kernel in the stream begin its own prologue.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Streaming 128-bit load: read-only path, do not keep the line in L1 (weights are read once).
__device__ __forceinline__ float4 ld_stream_f4(const float4* p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum of squares of n floats (n % 4 == 0) over the whole block, the same value in every thread.
__device__ float block_sum_sq(const float* x, int n, float* scratch /* >= 33 floats */) {
    float s = 0.f;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
        const float4 v = x4[i];
        s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    s = warp_sum(s);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (lane == 0) scratch[warp] = s;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// ---- embed -------------------------------------------------------------------------------

__global__ void __launch_bounds__(256) embed_kernel(const __grid_constant__ EmbedParams p) {
    grid_dependency_wait();
    grid_launch_dependents();
    const int pos = p.ctl->pos;
    int token = p.ctl->token;
    if (p.feed_prompt) token = pos == 0 ? 1 : p.prompt[pos - 1];
    if (token < 0 || token >= p.vocab) token = 0;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < p.dim) {
        const float v = p.table[(size_t)token * p.dim + i];
        p.x[i] = v;
        for (int s = 0; s < p.nscatter; s++) p.sdst[s][p.sidx[s][i]] = v;
    }
}

static void launch_cfg(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, dim3 grid, dim3 block, size_t smem,
                cudaStream_t st, bool pdl) {
    cfg = cudaLaunchConfig_t{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cfg.numAttrs = 0;
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    g_launches++;
}

void launch_embed(const EmbedParams& p, cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    launch_cfg(cfg, attr, dim3((p.dim + 255) / 256), dim3(256), 0, st, pdl);
    cudaLaunchKernelEx(&cfg, embed_kernel, p);
}

// ---- RoPE + KV append + attention, split over the sequence ----------------------------------

constexpr int ATT_THREADS = 128;
constexpr int ATT_WARPS = ATT_THREADS / 32;

template <int AG>
__global__ void __launch_bounds__(ATT_THREADS) attn_decode_kernel(const __grid_constant__ AttnParams p) {
    __shared__ __align__(16) float qs[AG][HS];
    __shared__ __align__(16) float sm_acc[ATT_WARPS][AG][HS];
    __shared__ float sm_m[ATT_WARPS][AG], sm_l[ATT_WARPS][AG];
    __shared__ int sm_last;

    grid_dependency_wait();
    grid_launch_dependents();
    const int kvh = blockIdx.x + p.kvh0, split = blockIdx.y;
    const int pos = p.pos_fixed >= 0 ? p.pos_fixed : p.ctl->pos;
    const int T = pos + 1;
    int nsplit = (T + p.split_min - 1) / p.split_min;
    nsplit = nsplit < 1 ? 1 : (nsplit > p.max_split ? p.max_split : nsplit);
    const int chunk = (T + nsplit - 1) / nsplit;
    nsplit = (T + chunk - 1) / chunk;
    if (split >= nsplit) return;
    const int t0 = split * chunk, t1 = min(T, t0 + chunk);
    const int KV = p.n_kv_heads * HS;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // RoPE, rotate-half and updated in place: the second half is rotated with the already
    // rotated first half (src/models.rs:106-116).  cos/sin come from a host table built with
    // the reference's f32 formula.
    for (int idx = tid; idx < AG * (HS / 2); idx += ATT_THREADS) {
        const int g = idx / (HS / 2), i = idx % (HS / 2);
        const int h = kvh * AG + g;
        const float c = p.rope_cos[(size_t)pos * (HS / 2) + i], s = p.rope_sin[(size_t)pos * (HS / 2) + i];
        const float a = p.q[(size_t)h * HS + i], b = p.q[(size_t)h * HS + HS / 2 + i];
        const float na = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
        const float nb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(na, s));
        qs[g][i] = na;
        qs[g][HS / 2 + i] = nb;
    }
    if (split == nsplit - 1) {  // this CTA owns position `pos`: append k (rotated) and v to the cache
        if (tid < HS / 2) {
            const int i = tid;
            const float c = p.rope_cos[(size_t)pos * (HS / 2) + i], s = p.rope_sin[(size_t)pos * (HS / 2) + i];
            const float a = p.k[(size_t)kvh * HS + i], b = p.k[(size_t)kvh * HS + HS / 2 + i];
            const float na = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
            const float nb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(na, s));
            p.kc[(size_t)pos * KV + kvh * HS + i] = na;
            p.kc[(size_t)pos * KV + kvh * HS + HS / 2 + i] = nb;
        }
        p.vc[(size_t)pos * KV + kvh * HS + tid] = p.v[(size_t)kvh * HS + tid];
    }
    __syncthreads();

    float4 qr[AG];
    float m[AG], l[AG];
    float4 acc[AG];
#pragma unroll
    for (int g = 0; g < AG; g++) {
        qr[g] = reinterpret_cast<const float4*>(qs[g])[lane];
        m[g] = -INFINITY;
        l[g] = 0.f;
        acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float inv_div = sqrtf((float)HS);
    const float4* kc4 = reinterpret_cast<const float4*>(p.kc) + (size_t)kvh * (HS / 4) + lane;
    const float4* vc4 = reinterpret_cast<const float4*>(p.vc) + (size_t)kvh * (HS / 4) + lane;
    const size_t rs = (size_t)KV / 4;
    constexpr int U = 4;
    for (int tb = t0 + warp * U; tb < t1; tb += ATT_WARPS * U) {
        float4 kk[U], vv[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int t = min(tb + u, t1 - 1);
            kk[u] = kc4[(size_t)t * rs];
            vv[u] = vc4[(size_t)t * rs];
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (tb + u < t1) {
#pragma unroll
                for (int g = 0; g < AG; g++) {
                    float d = qr[g].x * kk[u].x + qr[g].y * kk[u].y + qr[g].z * kk[u].z + qr[g].w * kk[u].w;
                    d = warp_sum(d);
                    const float sc = __fdiv_rn(d, inv_div);  // src/models.rs:158
                    const float mn = fmaxf(m[g], sc);
                    const float corr = expf(m[g] - mn), pr = expf(sc - mn);
                    l[g] = l[g] * corr + pr;
                    acc[g].x = acc[g].x * corr + pr * vv[u].x;
                    acc[g].y = acc[g].y * corr + pr * vv[u].y;
                    acc[g].z = acc[g].z * corr + pr * vv[u].z;
                    acc[g].w = acc[g].w * corr + pr * vv[u].w;
                    m[g] = mn;
                }
            }
        }
    }
#pragma unroll
    for (int g = 0; g < AG; g++) {
        reinterpret_cast<float4*>(sm_acc[warp][g])[lane] = acc[g];
        if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
    }
    __syncthreads();

    // combine the warps; thread i owns element i of every head of the group
    const int i = tid;
    float M[AG], L[AG], A[AG];
#pragma unroll
    for (int g = 0; g < AG; g++) {
        float mm = -INFINITY;
        for (int w = 0; w < ATT_WARPS; w++) mm = fmaxf(mm, sm_m[w][g]);
        float ll = 0.f, aa = 0.f;
        for (int w = 0; w < ATT_WARPS; w++) {
            const float e = sm_m[w][g] == -INFINITY ? 0.f : expf(sm_m[w][g] - mm);
            ll += sm_l[w][g] * e;
            aa += sm_acc[w][g][i] * e;
        }
        M[g] = mm; L[g] = ll; A[g] = aa;
    }
    if (nsplit == 1) {
#pragma unroll
        for (int g = 0; g < AG; g++) {
            const int o = (kvh * AG + g) * HS + i;
            p.out[p.oidx ? p.oidx[o] : o] = A[g] / L[g];
        }
        return;
    }
#pragma unroll
    for (int g = 0; g < AG; g++) {
        float* dst = p.part + ((size_t)(kvh * AG + g) * p.max_split + split) * (HS + 2);
        dst[i] = A[g];
        if (i == 0) { dst[HS] = M[g]; dst[HS + 1] = L[g]; }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned ticket = atomicAdd(p.counter + kvh, 1u);
        sm_last = (ticket == (unsigned)nsplit - 1u);
        if (sm_last) p.counter[kvh] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!sm_last) return;
    __threadfence();
    // the last CTA of this kv head merges the splits in split order
#pragma unroll
    for (int g = 0; g < AG; g++) {
        const float* src = p.part + (size_t)(kvh * AG + g) * p.max_split * (HS + 2);
        float mm = -INFINITY;
        for (int s = 0; s < nsplit; s++) mm = fmaxf(mm, __ldcg(src + (size_t)s * (HS + 2) + HS));
        float ll = 0.f, aa = 0.f;
        for (int s = 0; s < nsplit; s++) {
            const float e = expf(__ldcg(src + (size_t)s * (HS + 2) + HS) - mm);
            ll += __ldcg(src + (size_t)s * (HS + 2) + HS + 1) * e;
            aa += __ldcg(src + (size_t)s * (HS + 2) + i) * e;
        }
        const int o = (kvh * AG + g) * HS + i;
        p.out[p.oidx ? p.oidx[o] : o] = aa / ll;
    }
}

void launch_attn(const AttnParams& p, cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    launch_cfg(cfg, attr, dim3(p.n_kv_local > 0 ? p.n_kv_local : p.n_kv_heads, p.max_split), dim3(ATT_THREADS), 0, st, pdl);
    switch (p.ag) {
        case 1: cudaLaunchKernelEx(&cfg, attn_decode_kernel<1>, p); break;
        case 2: cudaLaunchKernelEx(&cfg, attn_decode_kernel<2>, p); break;
        case 4: cudaLaunchKernelEx(&cfg, attn_decode_kernel<4>, p); break;
        default: cudaLaunchKernelEx(&cfg, attn_decode_kernel<8>, p); break;
    }
}

// ---- final rmsnorm + dense f32 classifier ---------------------------------------------------

constexpr int CLS_THREADS = 256;

__global__ void __launch_bounds__(CLS_THREADS, 2) cls_kernel(const __grid_constant__ ClsParams p) {
    extern __shared__ float4 smem4[];
    __shared__ float scratch[34];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r0 = (int)(((long long)blockIdx.x * p.rows) / gridDim.x);
    const int r1 = (int)(((long long)(blockIdx.x + 1) * p.rows) / gridDim.x);
    const int n4 = p.in / 4;
    grid_dependency_wait();
    grid_launch_dependents();
    {
        const float sum = block_sum_sq(p.x, p.in, scratch);
        const float ss = 1.0f / sqrtf(sum / (float)p.in + p.eps);
        const float4* x4 = reinterpret_cast<const float4*>(p.x);
        const float4* w4 = reinterpret_cast<const float4*>(p.nw);
        for (int i = threadIdx.x; i < n4; i += CLS_THREADS) {
            float4 v = x4[i];
            const float4 w = w4[i];
            v.x = (w.x * ss) * v.x; v.y = (w.y * ss) * v.y; v.z = (w.z * ss) * v.z; v.w = (w.w * ss) * v.w;
            smem4[i] = v;
        }
        __syncthreads();
    }
    for (int row = r0 + warp * 2; row < r1; row += (CLS_THREADS / 32) * 2) {
        const bool two = row + 1 < r1;
        const float4* wa = reinterpret_cast<const float4*>(p.w + (size_t)row * p.in);
        const float4* wb = reinterpret_cast<const float4*>(p.w + (size_t)(two ? row + 1 : row) * p.in);
        float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll 4
        for (int i = lane; i < n4; i += 32) {
            const float4 x = smem4[i];
            const float4 u = ld_stream_f4(wa + i);
            const float4 v = ld_stream_f4(wb + i);
            a0 = fmaf(u.x, x.x, a0); a1 = fmaf(u.y, x.y, a1); a0 = fmaf(u.z, x.z, a0); a1 = fmaf(u.w, x.w, a1);
            b0 = fmaf(v.x, x.x, b0); b1 = fmaf(v.y, x.y, b1); b0 = fmaf(v.z, x.z, b0); b1 = fmaf(v.w, x.w, b1);
        }
        const float ya = warp_sum(a0 + a1), yb = warp_sum(b0 + b1);
        if (lane == 0) {
            p.logits[row] = ya;
            if (two) p.logits[row + 1] = yb;
        }
    }
}

void launch_cls(const ClsParams& p, int grid, cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    launch_cfg(cfg, attr, dim3(grid), dim3(CLS_THREADS), (size_t)p.in * 4, st, pdl);
    cudaLaunchKernelEx(&cfg, cls_kernel, p);
}

// ---- next-token selection ---------------------------------------------------------------------

constexpr int SEL_THREADS = 1024;

__device__ __forceinline__ unsigned random_u32(unsigned long long& s) {  // src/util.rs:71-77
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    return (unsigned)((s * 0x2545F4914F6CDD1Dull) >> 32);
}

__global__ void __launch_bounds__(SEL_THREADS) select_kernel(const __grid_constant__ SelectParams p) {
    __shared__ float s_val[SEL_THREADS / 32];
    __shared__ int s_idx[SEL_THREADS / 32];
    __shared__ float s_f[SEL_THREADS / 32 + 2];
    __shared__ int s_choice;
    grid_dependency_wait();
    grid_launch_dependents();
    Ctl* ctl = p.ctl;
    const int pos = ctl->pos, force = ctl->force, n_prompt = ctl->n_prompt;
    const float T = ctl->temperature;
    unsigned long long rng = ctl->rng;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int V = p.vocab;
    __syncthreads();  // every thread has read the loop state before thread 0 rewrites it
    int chosen;
    if (force >= 0) {
        chosen = force;
    } else if (pos < n_prompt) {
        chosen = p.prompt[pos];  // src/inference.rs:154-156
    } else {
        // argmax; among equal maxima the last index wins (src/util.rs:39-46)
        float bv = -INFINITY;
        int bi = V - 1;
        bool any = false;
        for (int i = tid; i < V; i += SEL_THREADS) {
            const float v = p.logits[i];
            if (!any || v >= bv) { bv = v; bi = i; any = true; }
        }
        if (!any) { bv = -INFINITY; bi = -1; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi > bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { s_val[warp] = bv; s_idx[warp] = bi; }
        __syncthreads();
        if (warp == 0) {
            bv = s_val[lane];
            bi = s_idx[lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi > bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0) { s_val[0] = bv; s_idx[0] = bi; }
        }
        __syncthreads();
        const float maxv = s_val[0];
        chosen = s_idx[0];
        if (T != 0.0f) {
            // softmax(logits / T), then the first index whose running sum exceeds r
            // (src/inference.rs:164-173, src/util.rs:102-113).  Each thread owns a
            // contiguous segment so that the running sum is taken in index order.
            const float mx = maxv / T;
            const int seg = (V + SEL_THREADS - 1) / SEL_THREADS;
            const int b = tid * seg, e = min(V, b + seg);
            float loc = 0.f;
            for (int i = b; i < e; i++) loc += expf(p.logits[i] / T - mx);
            // block-wide inclusive scan of the segment sums
            float incl = loc;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            if (lane == 31) s_f[warp] = incl;
            __syncthreads();
            if (warp == 0) {
                float w = s_f[lane];
                float wi = w;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float t = __shfl_up_sync(0xffffffffu, wi, o);
                    if (lane >= o) wi += t;
                }
                s_f[lane] = wi - w;  // exclusive prefix of the warp totals
                if (lane == 31) s_f[32] = wi;
            }
            if (tid == 0) s_choice = V - 1;  // "in case of rounding errors" (src/util.rs:112)
            __syncthreads();
            const float total = s_f[32];
            const float r = (float)(random_u32(rng) >> 8) / 16777216.0f;
            float cdf = (s_f[warp] + incl - loc) / total;
            for (int i = b; i < e; i++) {
                cdf += expf(p.logits[i] / T - mx) / total;
                if (r < cdf) { atomicMin(&s_choice, i); break; }
            }
            __syncthreads();
            chosen = s_choice;
            if (tid == 0) ctl->rng = rng;
        }
    }
    if (tid == 0) {
        p.out_tokens[pos] = chosen;
        ctl->last_next = chosen;
        ctl->token = chosen;
        ctl->pos = pos + 1;
    }
}

void launch_select(const SelectParams& p, cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    launch_cfg(cfg, attr, dim3(1), dim3(SEL_THREADS), 0, st, pdl);
    cudaLaunchKernelEx(&cfg, select_kernel, p);
}

struct ScatterParams { const float* src; float* dst[3]; const int* idx[3]; int n, ndst; };

__global__ void __launch_bounds__(256) scatter_kernel(const __grid_constant__ ScatterParams p) {
    grid_dependency_wait();
    grid_launch_dependents();
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < p.n) {
        const float v = p.src[j];
        for (int s = 0; s < p.ndst; s++) p.dst[s][p.idx[s][j]] = v;
    }
}

void launch_scatter(const float* src, int n, float* const* dst, const int* const* idx, int ndst, cudaStream_t st, bool pdl) {
    ScatterParams p{};
    p.src = src; p.n = n; p.ndst = ndst;
    for (int i = 0; i < ndst; i++) { p.dst[i] = dst[i]; p.idx[i] = idx[i]; }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    launch_cfg(cfg, attr, dim3((n + 255) / 256), dim3(256), 0, st, pdl);
    cudaLaunchKernelEx(&cfg, scatter_kernel, p);
}

__global__ void advance_kernel(Ctl* ctl) {
    grid_dependency_wait();
    grid_launch_dependents();
    if (threadIdx.x == 0) ctl->pos = ctl->pos + 1;
}

void launch_advance(Ctl* ctl, cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    launch_cfg(cfg, attr, dim3(1), dim3(32), 0, st, pdl);
    cudaLaunchKernelEx(&cfg, advance_kernel, ctl);
}

cudaError_t kernels_init() {
    cudaError_t e;
    int dev = 0, max_optin = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&max_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) return e;
    if ((e = sk_init(max_optin - 2048)) != cudaSuccess) return e;
    if ((e = gemm_tc_init(max_optin - 2048)) != cudaSuccess) return e;
    if ((e = attn_batch_init()) != cudaSuccess) return e;
    if ((e = token_init(max_optin)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(cls_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_optin - 2048)) != cudaSuccess) return e;
    return cudaSuccess;
}

}  // namespace l2
