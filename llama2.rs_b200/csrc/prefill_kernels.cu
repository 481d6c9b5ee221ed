// Kernels of the batched forward pass transformer<B>, B >= 2 (src/models.rs:178-298), around the
// tcgen05 GEMM of gemm_tc.cu: embedding rows, activation quantiser (rmsnorm folded in), RoPE +
// cache append, causal attention over the cache, SwiGLU.  One CTA per token (and head).
#include <algorithm>
#include <cfloat>
#include <cmath>

#include "kernels.cuh"

namespace l2 {

namespace {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t kbyte, uint32_t gs) {
    const uint32_t off = row * gs + kbyte;
    return off ^ (((off >> 7) & ((gs >> 4) - 1)) << 4);
}

}  // namespace

// ---- x[m] = token_embedding_table[tokens[m]] (src/models.rs:189-191) ---------------------------
__global__ void embed_batch_kernel(const float* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ x, int dim) {
    const int m = blockIdx.x;
    const float4* src = reinterpret_cast<const float4*>(table + (size_t)tokens[m] * dim);
    float4* dst = reinterpret_cast<float4*>(x + (size_t)m * dim);
    for (int i = threadIdx.x; i < dim / 4; i += blockDim.x) dst[i] = src[i];
}

// ---- activation quantiser ---------------------------------------------------------------------
// Token m of x (natural order) is gathered into the consumer's K order, multiplied by the rmsnorm
// weight (linearity: the 1/sqrt(mean(x^2)+eps) factor goes into oscale), scaled by a power of two
// so that |X| <= 2^22 (23 of the 24 bits of an f32 mantissa for the token's largest element) and written
// as three balanced base-256 digits (-128..127 each) into the K-major, swizzled byte image the GEMM
// copies into shared memory: row digit * mpad + m (most significant digit first), inside a block of
// 8 inputs the order (0,2,4,6,1,3,5,7) in which a weight word separates into nibbles.
constexpr int AQ_THREADS = 256;
constexpr int AQ_CACHE = 2;        // rounds of a CTA's own slice kept in registers between the two passes

__global__ void __launch_bounds__(AQ_THREADS) act_quant_kernel(const __grid_constant__ QuantParams P) {
    __shared__ float red[2 * (AQ_THREADS / 32) + 2];
    // the GEMM behind this kernel is launched programmatically: it may start now (its loaders need nothing from here) and
    // waits inside for this grid to finish before it reads the image
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int m = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const float* x = P.x + (size_t)m * P.ldx;
    const int nblk = P.in / 8;
    const uint32_t gs = P.gs, lanes_per_group = gs / 8;
    auto fetch = [&](int blk, float (&v)[8], float& sq) {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int k = blk * 8 + j;
            const float xv = x[P.perm ? P.perm[k] : k];
            sq += xv * xv;
            v[j] = P.nw ? xv * P.nw[k] : xv;
        }
    };
    // The row is cut into gridDim.y slices of whole groups; every slice's CTA takes the statistics of the whole row (the
    // row is 16 to 112 KB and sits in the L2) and writes the digits of its own slice.  It walks the row starting at its
    // slice and keeps what it fetched there (AQ_CACHE rounds), so its slice is gathered once.
    const int G = P.in / (int)gs, S = (int)gridDim.y, slice = (int)blockIdx.y;
    const int b0 = (slice * G / S) * (int)lanes_per_group, nslice = ((slice + 1) * G / S) * (int)lanes_per_group - b0;
    float cache[AQ_CACHE][8];
    float mx = 0.f, sq = 0.f;
    const int rounds = (nblk + AQ_THREADS - 1) / AQ_THREADS;
#pragma unroll
    for (int k = 0; k < AQ_CACHE; k++) {
        const int idx = tid + k * AQ_THREADS;
        if (idx < nblk) {
            fetch(b0 + idx < nblk ? b0 + idx : b0 + idx - nblk, cache[k], sq);
#pragma unroll
            for (int j = 0; j < 8; j++) mx = fmaxf(mx, fabsf(cache[k][j]));
        }
    }
    for (int k = AQ_CACHE; k < rounds; k++) {
        const int idx = tid + k * AQ_THREADS;
        if (idx >= nblk) break;
        float v[8];
        fetch(b0 + idx < nblk ? b0 + idx : b0 + idx - nblk, v, sq);
#pragma unroll
        for (int j = 0; j < 8; j++) mx = fmaxf(mx, fabsf(v[j]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
    }
    if (lane == 0) { red[warp] = mx; red[AQ_THREADS / 32 + warp] = sq; }
    __syncthreads();
    if (tid == 0) {
        float a = 0.f, b = 0.f;
        for (int w = 0; w < AQ_THREADS / 32; w++) { a = fmaxf(a, red[w]); b += red[AQ_THREADS / 32 + w]; }
        red[2 * (AQ_THREADS / 32)] = a;
        red[2 * (AQ_THREADS / 32) + 1] = b;
    }
    __syncthreads();
    mx = red[2 * (AQ_THREADS / 32)];
    const float total = red[2 * (AQ_THREADS / 32) + 1];
    const float rs = P.nw ? 1.0f / sqrtf(total / (float)P.in + P.eps) : 1.0f;  // src/models.rs:58-60
    int e = 0;
    // |x| * scale < 2^22: three balanced digits reach from -0x808080 to 0x7F7F7F, a little short of 2^23
    if (mx > 0.f && mx < INFINITY) e = 21 - (int)((__float_as_uint(mx) >> 23) & 255u) + 127;
    e = max(-100, min(100, e));
    const float scale = __uint_as_float((uint32_t)(127 + e) << 23);
    if (tid == 0 && slice == 0) P.oscale[m] = rs / scale;

    const size_t img_group = (size_t)P.n * gs + (size_t)P.mpad * 4;  // bytes of one group's block: the digit image, then the tokens' digit sums
    const int erounds = (nslice + AQ_THREADS - 1) / AQ_THREADS;
#pragma unroll 1
    for (int k = 0; k < erounds; k++) {
        const int idx = tid + k * AQ_THREADS;
        if ((idx & ~31) >= nslice) break;  // warp-uniform
        const bool valid = idx < nslice;   // a group is 4 to 16 adjacent lanes and nslice a multiple of that: valid for all lanes of a group or none
        const int blk = b0 + idx;
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (valid) {
            static_assert(AQ_CACHE == 2, "the rounds kept in registers are picked by name");
            if (k == 0) {
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = cache[0][j];
            } else if (k == 1) {
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = cache[1][j];
            } else {
                float dummy = 0.f;
                fetch(blk, v, dummy);
            }
        }
        uint32_t E[8];  // per element: bytes d2, d1, d0 (least significant digit first), balanced: X = d0 2^16 + d1 2^8 + d2, d in -128..127
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int X = __float2int_rn(v[j] * scale);
            E[j] = ((uint32_t)X + 0x00808080u) ^ 0x00808080u;
        }
        // 4x4 byte transposes: words of one digit for inputs (0,2,4,6) and (1,3,5,7), the order in which the nibbles of a
        // weight word separate into its low and high halves; index 0 = most significant digit
        uint32_t lo[3], hi[3];
        {
            const uint32_t a = __byte_perm(E[0], E[2], 0x5140), b = __byte_perm(E[0], E[2], 0x7362);
            const uint32_t c = __byte_perm(E[4], E[6], 0x5140), d = __byte_perm(E[4], E[6], 0x7362);
            lo[2] = __byte_perm(a, c, 0x5410); lo[1] = __byte_perm(a, c, 0x7632);
            lo[0] = __byte_perm(b, d, 0x5410);
        }
        {
            const uint32_t a = __byte_perm(E[1], E[3], 0x5140), b = __byte_perm(E[1], E[3], 0x7362);
            const uint32_t c = __byte_perm(E[5], E[7], 0x5140), d = __byte_perm(E[5], E[7], 0x7362);
            hi[2] = __byte_perm(a, c, 0x5410); hi[1] = __byte_perm(a, c, 0x7632);
            hi[0] = __byte_perm(b, d, 0x5410);
        }
        const int g = valid ? (int)((uint32_t)(blk * 8) / gs) : 0;
        const uint32_t kb = (uint32_t)(blk * 8) % gs;
        int sum[3];
#pragma unroll
        for (int p = 0; p < 3; p++) {
            if (valid)
                *reinterpret_cast<uint2*>(P.bimg + (size_t)g * img_group + swz((uint32_t)(p * P.mpad + m), kb, gs)) = make_uint2(lo[p], hi[p]);
            sum[p] = __dp4a((int)lo[p], 0x01010101, __dp4a((int)hi[p], 0x01010101, 0));
        }
        int s01 = 256 * sum[0] + sum[1], s2 = sum[2];
        for (uint32_t o = 1; o < lanes_per_group; o <<= 1) {
            s01 += __shfl_xor_sync(0xffffffffu, s01, o);
            s2 += __shfl_xor_sync(0xffffffffu, s2, o);
        }
        if (valid && (tid & (lanes_per_group - 1)) == 0) {
            // the sum of the token's integers over the group, as the f32 nearest to it (|s01| < 2^23 and |s2| < 2^15 are exact)
            *reinterpret_cast<float*>(P.bimg + (size_t)g * img_group + (size_t)P.n * gs + (size_t)m * 4) = fmaf((float)s01, 256.0f, (float)s2);
        }
    }
}

// ---- RoPE + cache append for M tokens (src/models.rs:100-129, 236-249) ----------------------------
// grid (n_heads, M), 64 threads.  q is rotated in place; k (rotated) and v go to the cache rows.
__global__ void __launch_bounds__(64) rope_append_kernel(const __grid_constant__ RopeParams P) {
    const int h = blockIdx.x, m = blockIdx.y, i = threadIdx.x;
    const int pos = P.pos[m];
    const float c = P.rope_cos[(size_t)pos * (HS / 2) + i], s = P.rope_sin[(size_t)pos * (HS / 2) + i];
    float* q = P.q + (size_t)m * P.ldq + (size_t)h * HS;
    {
        const float a = q[i], b = q[HS / 2 + i];
        const float na = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
        const float nb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(na, s));  // second half uses the rotated first half
        q[i] = na;
        q[HS / 2 + i] = nb;
    }
    if (h < P.n_kv_heads) {
        const int KV = P.kv_stride ? P.kv_stride : P.n_kv_heads * HS;
        const float* k = P.k + (size_t)m * P.ldkv + (size_t)h * HS;
        const float* v = P.v + (size_t)m * P.ldkv + (size_t)h * HS;
        const float a = k[i], b = k[HS / 2 + i];
        const float na = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
        const float nb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(na, s));
        float* kc = P.kc + (size_t)pos * KV + (size_t)h * HS;
        float* vc = P.vc + (size_t)pos * KV + (size_t)h * HS;
        kc[i] = na;
        kc[HS / 2 + i] = nb;
        vc[i] = v[i];
        vc[HS / 2 + i] = v[HS / 2 + i];
    }
}

// ---- attention of M tokens over the cache, causal through 0..=pos[m] (src/models.rs:131-176) ------
// grid (n_heads, M), 128 threads: each warp walks the time steps t = warp, warp + 4, ... with an
// online softmax; the four warps are merged in shared memory.
__global__ void __launch_bounds__(128) attn_batch_kernel(const __grid_constant__ AttnBatchParams P) {
    __shared__ __align__(16) float sm_acc[4][HS];
    __shared__ float sm_m[4], sm_l[4];
    const int h = blockIdx.x, m = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = h / P.ag, KV = P.kv_stride ? P.kv_stride : P.n_kv_heads * HS;
    const int T = P.pos[m] + 1;
    const float4 q = reinterpret_cast<const float4*>(P.q + (size_t)m * P.ldq + (size_t)h * HS)[lane];
    const float4* kc = reinterpret_cast<const float4*>(P.kc) + (size_t)kvh * (HS / 4) + lane;
    const float4* vc = reinterpret_cast<const float4*>(P.vc) + (size_t)kvh * (HS / 4) + lane;
    const size_t rs = (size_t)KV / 4;
    const float div = sqrtf((float)HS);
    float mx = -INFINITY, l = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int t = warp; t < T; t += 4) {
        const float4 k = kc[(size_t)t * rs], v = vc[(size_t)t * rs];
        float d = warp_sum_f(q.x * k.x + q.y * k.y + q.z * k.z + q.w * k.w);
        const float sc = __fdiv_rn(d, div);  // src/models.rs:158
        const float mn = fmaxf(mx, sc);
        const float corr = expf(mx - mn), pr = expf(sc - mn);
        l = l * corr + pr;
        acc.x = acc.x * corr + pr * v.x; acc.y = acc.y * corr + pr * v.y;
        acc.z = acc.z * corr + pr * v.z; acc.w = acc.w * corr + pr * v.w;
        mx = mn;
    }
    reinterpret_cast<float4*>(sm_acc[warp])[lane] = acc;
    if (lane == 0) { sm_m[warp] = mx; sm_l[warp] = l; }
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < 4; w++) M = fmaxf(M, sm_m[w]);
    float L = 0.f, A = 0.f;
    for (int w = 0; w < 4; w++) {
        const float e = sm_m[w] == -INFINITY ? 0.f : expf(sm_m[w] - M);
        L += sm_l[w] * e;
        A += sm_acc[w][tid] * e;
    }
    P.out[(size_t)m * P.ldo + (size_t)h * HS + tid] = A / L;
}

// ---- hb = silu(h1) * h3 (src/models.rs:92-98) --------------------------------------------------------
// h1, h3: [M][n] (this process's columns); hb: [M][ld] with those columns at the pointer given
__global__ void swiglu_kernel(const float* __restrict__ h1, const float* __restrict__ h3, float* __restrict__ hb, int n, int ld, int M) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < (size_t)M * n) {
        const float a = h1[i];
        hb[(i / n) * ld + i % n] = (a * (1.0f / (1.0f + expf(-a)))) * h3[i];
    }
}

void launch_embed_batch(const float* table, const int* tokens, float* x, int dim, int M, cudaStream_t st) {
    g_launches++;
    embed_batch_kernel<<<M, 256, 0, st>>>(table, tokens, x, dim);
}
void launch_act_quant(const QuantParams& p, int M, cudaStream_t st) {
    g_launches++;
    // slices of about one round of the CTA's threads (256 blocks of 8 inputs), whole groups each
    const int G = p.in / p.gs;
    const int S = std::max(1, std::min(std::min(4, G), p.in / 8 / AQ_THREADS));
    act_quant_kernel<<<dim3(M, S), AQ_THREADS, 0, st>>>(p);
}
void launch_rope_append(const RopeParams& p, int n_heads, int M, cudaStream_t st) {
    g_launches++;
    rope_append_kernel<<<dim3(n_heads, M), 64, 0, st>>>(p);
}

// ---- the same attention with the cache rows shared by the queries that need them ---------------------------------------
// One CTA takes a kv head and a block of tokens: all their queries (AG heads per token) walk the cache together, 32
// positions at a time.  A tile of K and V rows is brought into shared memory once and used by up to 64 queries, instead of
// once per (head, token) as above — at a context of 1500 that kernel moved 64 times the cache through the L2 per kv head
// and was a fifth of a long prompt's prefill.  Scores: lane = position, the query comes as broadcast loads from shared
// memory; softmax state per query (online, one rescale per tile); values: lane = four of the 128 dimensions, the
// probabilities come by shuffle.  Plain f32 FMAs: the arithmetic is the reference's, only the order of the sums differs.
constexpr int AT_WARPS = 8, AT_TILE = 32, AT_KPAD = HS + 4;  // K rows padded: a lane reads "its" row without bank conflicts
template <int AG, int NQW>  // query heads per kv head; queries per warp (NQW / AG tokens)
__global__ void __launch_bounds__(32 * AT_WARPS) attn_batch_tiled_kernel(const __grid_constant__ AttnBatchParams P, int M) {
    extern __shared__ __align__(16) float at_smem[];
    constexpr int TPW = NQW / AG;                       // tokens per warp
    constexpr int QB = AT_WARPS * TPW;                  // tokens per CTA
    float* Qs = at_smem;                                // [AT_WARPS * NQW][HS]
    float* Ks = Qs + AT_WARPS * NQW * HS;               // [AT_TILE][AT_KPAD]
    float* Vs = Ks + AT_TILE * AT_KPAD;                 // [AT_TILE][HS]
    const int kvh = blockIdx.x, m0 = blockIdx.y * QB, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int KV = P.kv_stride ? P.kv_stride : P.n_kv_heads * HS;
    const float div = sqrtf((float)HS);
    // queries of this CTA: query i = (token m0 + i / AG, head kvh * AG + i % AG)
    for (int i = tid; i < AT_WARPS * NQW * (HS / 4); i += 32 * AT_WARPS) {
        const int qi = i / (HS / 4), c = i % (HS / 4), m = m0 + qi / AG;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m < M) v = reinterpret_cast<const float4*>(P.q + (size_t)m * P.ldq + (size_t)(kvh * AG + qi % AG) * HS)[c];
        reinterpret_cast<float4*>(Qs)[i] = v;
    }
    int last[TPW];   // last position each of this warp's tokens attends to (-1: no such token)
    int tmax = -1;   // over the CTA
#pragma unroll
    for (int j = 0; j < TPW; j++) {
        const int m = m0 + warp * TPW + j;
        last[j] = m < M ? P.pos[m] : -1;
    }
    for (int m = m0; m < min(M, m0 + QB); m++) tmax = max(tmax, P.pos[m]);
    float mx[NQW], l[NQW];
    float4 acc[NQW];
#pragma unroll
    for (int q = 0; q < NQW; q++) { mx[q] = -INFINITY; l[q] = 0.f; acc[q] = make_float4(0.f, 0.f, 0.f, 0.f); }
    const float4* kc = reinterpret_cast<const float4*>(P.kc) + (size_t)kvh * (HS / 4);
    const float4* vc = reinterpret_cast<const float4*>(P.vc) + (size_t)kvh * (HS / 4);
    const size_t rs = (size_t)KV / 4;
    for (int t0 = 0; t0 <= tmax; t0 += AT_TILE) {
        __syncthreads();  // the previous tile has been used (and Qs is complete)
        for (int i = tid; i < AT_TILE * (HS / 4); i += 32 * AT_WARPS) {
            const int r = i / (HS / 4), c = i % (HS / 4), t = t0 + r;
            float4 k = make_float4(0.f, 0.f, 0.f, 0.f), v = k;
            if (t <= tmax) { k = kc[(size_t)t * rs + c]; v = vc[(size_t)t * rs + c]; }
            reinterpret_cast<float4*>(Ks + r * AT_KPAD)[c] = k;
            reinterpret_cast<float4*>(Vs + r * HS)[c] = v;
        }
        __syncthreads();
        // scores of position t0 + lane for this warp's queries
        float s[NQW];
#pragma unroll
        for (int q = 0; q < NQW; q++) s[q] = 0.f;
        const float4* krow = reinterpret_cast<const float4*>(Ks + lane * AT_KPAD);
        const float4* qrow = reinterpret_cast<const float4*>(Qs + (size_t)warp * NQW * HS);
#pragma unroll 4
        for (int c = 0; c < HS / 4; c++) {
            const float4 k = krow[c];
#pragma unroll
            for (int q = 0; q < NQW; q++) {
                const float4 qq = qrow[q * (HS / 4) + c];
                s[q] = fmaf(qq.x, k.x, s[q]); s[q] = fmaf(qq.y, k.y, s[q]); s[q] = fmaf(qq.z, k.z, s[q]); s[q] = fmaf(qq.w, k.w, s[q]);
            }
        }
        // online softmax per query, then the values
        float p[NQW];
#pragma unroll
        for (int q = 0; q < NQW; q++) {
            const bool valid = t0 + lane <= last[q / AG];
            const float sc = valid ? __fdiv_rn(s[q], div) : -INFINITY;  // src/models.rs:158
            float tm = sc;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
            const float mn = fmaxf(mx[q], tm);
            const float corr = mn == -INFINITY ? 1.f : expf(mx[q] - mn);
            p[q] = valid ? expf(sc - mn) : 0.f;
            const float ps = warp_sum_f(p[q]);
            l[q] = l[q] * corr + ps;
            acc[q].x *= corr; acc[q].y *= corr; acc[q].z *= corr; acc[q].w *= corr;
            mx[q] = mn;
        }
        const float4* vcol = reinterpret_cast<const float4*>(Vs) + lane;
#pragma unroll 4
        for (int t = 0; t < AT_TILE; t++) {
            const float4 v = vcol[t * (HS / 4)];
#pragma unroll
            for (int q = 0; q < NQW; q++) {
                const float pq = __shfl_sync(0xffffffffu, p[q], t);
                acc[q].x = fmaf(pq, v.x, acc[q].x); acc[q].y = fmaf(pq, v.y, acc[q].y);
                acc[q].z = fmaf(pq, v.z, acc[q].z); acc[q].w = fmaf(pq, v.w, acc[q].w);
            }
        }
    }
#pragma unroll
    for (int q = 0; q < NQW; q++) {
        const int qi = warp * NQW + q, m = m0 + qi / AG;
        if (m < M) {
            const float inv = 1.0f / l[q];
            reinterpret_cast<float4*>(P.out + (size_t)m * P.ldo + (size_t)(kvh * AG + qi % AG) * HS)[lane] =
                make_float4(acc[q].x * inv, acc[q].y * inv, acc[q].z * inv, acc[q].w * inv);
        }
    }
}

template <int AG, int NQW>
static void launch_attn_tiled(const AttnBatchParams& p, int M, cudaStream_t st) {
    constexpr int QB = AT_WARPS * (NQW / AG);
    const size_t smem = (size_t)(AT_WARPS * NQW * HS + AT_TILE * AT_KPAD + AT_TILE * HS) * sizeof(float);
    attn_batch_tiled_kernel<AG, NQW><<<dim3(p.n_kv_heads, (M + QB - 1) / QB), 32 * AT_WARPS, smem, st>>>(p, M);
}

// the tiled kernel's shared memory (65 KB at most) is above the default limit: once per device, at start-up
cudaError_t attn_batch_init() {
    const int smem = (AT_WARPS * 8 * HS + AT_TILE * AT_KPAD + AT_TILE * HS) * (int)sizeof(float);
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(attn_batch_tiled_kernel<1, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(attn_batch_tiled_kernel<2, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(attn_batch_tiled_kernel<4, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess) return e;
    return cudaFuncSetAttribute(attn_batch_tiled_kernel<8, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
}

// tiled: the kernel that shares cache tiles among queries (long contexts); otherwise one CTA per (head, token), which has
// more CTAs and less set-up (short contexts: the cache is small and sits in the L2 anyway)
void launch_attn_batch(const AttnBatchParams& p, int n_heads, int M, bool tiled, cudaStream_t st) {
    g_launches++;
    switch (tiled ? p.ag : 0) {
        case 1: launch_attn_tiled<1, 4>(p, M, st); break;
        case 2: launch_attn_tiled<2, 8>(p, M, st); break;
        case 4: launch_attn_tiled<4, 8>(p, M, st); break;
        case 8: launch_attn_tiled<8, 8>(p, M, st); break;
        default: attn_batch_kernel<<<dim3(n_heads, M), 128, 0, st>>>(p); break;
    }
}
// ---- all-gather of a column slice over peer memory (batched forward under tensor parallelism) ----------------------------
// Every CTA copies rows of this rank's columns into the peers' buffers with plain stores.  The CTA that finishes last
// (completion counter behind a system-wide fence) then tells every peer "my part of exchange seq is in your memory" and waits,
// bounded, until every peer has said the same: after this kernel the whole buffer is valid on this rank.
constexpr uint32_t TPG_WAIT_LIMIT = 1u << 22;
__global__ void __launch_bounds__(256) tp_gather_kernel(const __grid_constant__ TpGatherParams P) {
    __shared__ unsigned last;
    __shared__ unsigned long long seq_s;
    const int n4 = P.ncols / 4;
    for (int m = blockIdx.x; m < P.M; m += gridDim.x) {
        const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(P.pool[P.rank] + P.buf_off) + (size_t)m * P.ld + P.col0);
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 v = src[i];
            for (int r = 0; r < P.world; r++)
                if (r != P.rank) reinterpret_cast<float4*>(reinterpret_cast<float*>(P.pool[r] + P.buf_off) + (size_t)m * P.ld + P.col0)[i] = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(P.done, 1u) == gridDim.x - 1 ? 1u : 0u;
    __syncthreads();
    if (!last) return;
    if (threadIdx.x == 0) { *P.done = 0; seq_s = ++*P.seq; }  // ready for the next launch; this exchange's number
    __threadfence_system();
    __syncthreads();
    const unsigned long long seq = seq_s;
    const int r = threadIdx.x;
    if (r < P.world && r != P.rank) {
        unsigned long long* theirs = reinterpret_cast<unsigned long long*>(P.pool[r] + P.flag_off) + P.rank;
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(theirs), "l"(seq) : "memory");
        const unsigned long long* mine = reinterpret_cast<const unsigned long long*>(P.pool[P.rank] + P.flag_off) + r;
        bool ok = false;
#pragma unroll 1
        for (uint32_t it = 0; it < TPG_WAIT_LIMIT; it++) {
            unsigned long long v;
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(mine) : "memory");
            if (v >= seq) { ok = true; break; }
            __nanosleep(200);
        }
        if (!ok && P.status) atomicCAS(P.status, 0, 3001);
    }
}
void launch_tp_gather(const TpGatherParams& p, cudaStream_t st) {
    g_launches++;
    tp_gather_kernel<<<std::min(p.M, 64), 256, 0, st>>>(p);
}

void launch_swiglu(const float* h1, const float* h3, float* hb, int n, int ld, int M, cudaStream_t st) {
    g_launches++;
    swiglu_kernel<<<(unsigned)(((size_t)M * n + 255) / 256), 256, 0, st>>>(h1, h3, hb, n, ld, M);
}

__global__ void __launch_bounds__(256) ksum_kernel(const float* __restrict__ part, size_t kstride, int ksplit, float* __restrict__ out,
                                                   int ldo, int rows, int M, int epi) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)M * rows) return;
    const int m = (int)(i / rows), o = (int)(i % rows);
    float v = 0.f;
    for (int k = 0; k < ksplit; k++) v += part[(size_t)k * kstride + (size_t)m * rows + o];  // slice order: reproducible
    float* dst = out + (size_t)m * ldo + o;
    *dst = epi == EPI_RESID ? *dst + v : v;
}

void launch_ksum(const float* part, size_t kstride, int ksplit, float* out, int ldo, int rows, int M, int epi, cudaStream_t st) {
    const size_t n = (size_t)M * rows;
    g_launches++;
    ksum_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(part, kstride, ksplit, out, ldo, rows, M, epi);
}

}  // namespace l2
