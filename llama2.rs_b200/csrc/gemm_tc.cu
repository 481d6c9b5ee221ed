// Batched QLinear::matvec<B> (src/gptq.rs:94-176) for B >= 2 as a dense contraction on the
// 5th-generation tensor cores: tcgen05.mma kind::i8 with accumulators in tensor memory.
//
//   out[m][o] = f[m] * sum_g scale[o][g] * sum_{k in g} (q[o][k] - z[o][g]) * X[m][k]
//
// X[m][k] is the activation of token m as an exact 28-bit integer (four 7-bit digits, see
// act_quant_kernel in prefill_kernels.cu), so every product and every sum inside a quantisation
// group is exact integer arithmetic; f[m] carries the block exponent and the rmsnorm factor.
//
// One CTA owns 128 output rows and walks the quantisation groups.  Per group:
//   A  128 rows x GS weights, unpacked from nibbles to unsigned bytes in shared memory (3 bit
//      operations per 8 weights), K-major with the 128/64/32-byte swizzle the MMA unit expects;
//   B  N = 4 digits x M tokens rows x GS signed bytes, copied by one bulk copy from the image the
//      quantiser wrote (already swizzled);
//   D  128 x N s32 in tensor memory, overwritten by the first MMA of the group (GS/32 MMAs of K = 32).
// While the tensor core works on group g, all 16 warps drain group g-1 from the other accumulator:
// tcgen05.ld, zero point via the group's digit sums, one f32 FMA per (row, token) with the scale.
// Two shared-memory stages and two accumulators; every wait on an mbarrier is bounded.
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels.cuh"

namespace l2 {

namespace {

constexpr int TC_THREADS = 512;            // 16 warps: four per quadrant of tensor-memory lanes, each draining a quarter of the columns
constexpr int TC_CHUNKS = TC_THREADS / 128;  // column chunks of the drain
constexpr int TC_UNPACK = 512 / TC_THREADS;  // (record, half, lane) items of a group's A tile per thread
constexpr int TC_ACC = 64 / TC_CHUNKS;       // tokens per thread at most
constexpr int TC_AHEAD = 4;  // groups whose weights are in flight in registers
constexpr int MAX_TOKENS = 64;  // tokens of one pass (N = 4 * tokens <= 256 columns)
constexpr uint32_t TC_WAIT_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// bounded: returns false after TC_WAIT_LIMIT polls
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < TC_WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}

// K-major operand descriptor: rows of GS bytes, 8-row swizzle atoms of 8*GS bytes
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t gs) {
    const uint64_t layout = gs == 128 ? 2 : (gs == 64 ? 4 : 6);  // SWIZZLE_128B / 64B / 32B
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)((8u * gs) >> 4) << 32) | (1ull << 46) | (layout << 61);
}
// byte offset of (row, k) inside a K-major tile with rows of gs bytes, swizzled
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t kbyte, uint32_t gs) {
    const uint32_t off = row * gs + kbyte;
    return off ^ (((off >> 7) & ((gs >> 4) - 1)) << 4);
}

}  // namespace

__global__ void __launch_bounds__(TC_THREADS, 1) gemm_q4_tc_kernel(const __grid_constant__ TcParams P) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t mma_done[2], b_full[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int failed;
    __shared__ int2 sv_s[3][MAX_TOKENS];  // digit sums of a group: written in its own iteration, read in the next, reused two later

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t GS = P.gs, W = GS / 32, N = P.n;
    const int tile = blockIdx.x;                 // 128 output rows
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t a_bytes = 128 * GS, b_bytes = N * GS;
    const uint32_t stage_bytes = (a_bytes + b_bytes + 1023) & ~1023u;
    uint8_t* stage_a[2] = {smem, smem + stage_bytes};
    uint8_t* stage_b[2] = {smem + a_bytes, smem + stage_bytes + a_bytes};

    if (tid == 0) {
        mbar_init(&mma_done[0], 1); mbar_init(&mma_done[1], 1);
        mbar_init(&b_full[0], 1); mbar_init(&b_full[1], 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {  // 512 columns of tensor memory: two accumulators of up to 256 columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_addr(&tmem_base_s)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;

    // instruction descriptor: D s32, A u8, B s8, both K-major, N, M = 128
    const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((N >> 3) << 17) | ((128u >> 4) << 24);

    // epilogue ownership: warp w reads tensor-memory lanes 32*(w%4).. (= rows), column half w/4
    const int row = 32 * (warp & 3) + lane;                 // row inside the 128-row tile
    const int orow = tile * 128 + row;                       // output row
    const int rec16 = orow >> 4;                             // 16-row record the row lives in
    const bool row_ok = rec16 < P.tiles16;
    const int chalf = warp >> 2;                             // which chunk of the token range
    const int tok_per = (int)(N / 4) / TC_CHUNKS;            // tokens per column chunk (N = 4 * Mpad, Mpad % 4 == 0)
    float acc[TC_ACC];
#pragma unroll
    for (int i = 0; i < TC_ACC; i++) acc[i] = 0.f;
    const uint32_t UW = 64 * W + 20;                         // words per unit record

    bool ok = true;
    // split K: blockIdx.y takes groups [gb, gb + G) of the matrix's Gfull and writes its partial result
    const int Gfull = P.G;
    const int gper = (Gfull + (int)gridDim.y - 1) / (int)gridDim.y;
    const int gb = (int)blockIdx.y * gper;
    const int G = min(gper, Gfull - gb);  // groups of this CTA (at least one: the host never launches empty slices)
    // Software pipeline over the groups: the weight words and the row's scale / zero point of group
    // g + TC_AHEAD are requested while group g is unpacked and multiplied and group g - 1 drained, so that
    // a trip to HBM is hidden behind several iterations.  The register sets are indexed statically: the
    // group loop below is unrolled by TC_AHEAD.
    uint32_t wreg[TC_AHEAD][TC_UNPACK][4];
    float sc_set[TC_AHEAD];
    int z_set[TC_AHEAD];
    auto load_group = [&](int g, uint32_t (&w)[TC_UNPACK][4], float& sc_next, int& z_next) {
#pragma unroll
        for (int it = 0; it < TC_UNPACK; it++) {
            const int idx = tid + it * TC_THREADS, sub = idx >> 6, hl = idx & 63;
            const int rec = tile * 8 + sub;
            w[it][0] = w[it][1] = w[it][2] = w[it][3] = 0;
            if (rec < P.tiles16) {
                const uint32_t* src = P.rec + ((size_t)rec * Gfull + gb + g) * UW + (size_t)hl * W;
                if (W == 4) { const uint4 v = __ldg(reinterpret_cast<const uint4*>(src)); w[it][0] = v.x; w[it][1] = v.y; w[it][2] = v.z; w[it][3] = v.w; }
                else if (W == 2) { const uint2 v = __ldg(reinterpret_cast<const uint2*>(src)); w[it][0] = v.x; w[it][1] = v.y; }
                else w[it][0] = __ldg(src);
            }
        }
        sc_next = 0.f;
        z_next = 1;
        if (row_ok) {
            const uint32_t* meta = P.rec + ((size_t)rec16 * Gfull + gb + g) * UW + 64 * W;
            sc_next = __uint_as_float(__ldg(meta + (orow & 15)));
            z_next = (int)((__ldg(meta + 16 + ((orow & 15) >> 3)) >> (4 * (orow & 7))) & 15u) + 1;  // src/gptq.rs:148
        }
    };
    if (tid == 0) {
        mbar_expect_tx(&b_full[0], b_bytes);
        bulk_g2s(stage_b[0], P.bimg + (size_t)gb * b_bytes, b_bytes, &b_full[0]);
    }
    if (tid == 0 && G > 1) {  // the second stage is free from the start
        mbar_expect_tx(&b_full[1], b_bytes);
        bulk_g2s(stage_b[1], P.bimg + (size_t)(gb + 1) * b_bytes, b_bytes, &b_full[1]);
    }
#pragma unroll
    for (int j = 0; j < TC_AHEAD; j++) {
        sc_set[j] = 0.f;
        z_set[j] = 1;
#pragma unroll
        for (int it = 0; it < TC_UNPACK; it++) wreg[j][it][0] = wreg[j][it][1] = wreg[j][it][2] = wreg[j][it][3] = 0;
        if (j < G) load_group(j, wreg[j], sc_set[j], z_set[j]);
    }
    float sc_cur = 0.f, sc_prev = 0.f;
    int z_cur = 1, z_prev = 1;
    // digit sums: group g's are loaded into a register in iteration g - 1, parked in shared memory in
    // iteration g (before its barrier) and read by the drain of group g in iteration g + 1
    const int2* sv_g = reinterpret_cast<const int2*>(P.sv);
    int2 sv_reg = make_int2(0, 0);
    if (tid < P.mpad) sv_reg = __ldg(sv_g + (size_t)gb * P.mpad + tid);
    for (int g0 = 0; g0 <= G; g0 += TC_AHEAD) {
#pragma unroll
    for (int jj = 0; jj < TC_AHEAD; jj++) {
        const int g = g0 + jj;
        if (g > G) break;
        const int s = g & 1;
        sc_prev = sc_cur; z_prev = z_cur;
        if (g < G && tid < P.mpad) {
            sv_s[g % 3][tid] = sv_reg;
            if (g + 1 < G) sv_reg = __ldg(sv_g + (size_t)(gb + g + 1) * P.mpad + tid);
        }
        if (g < G) {
            // ---- A of group g: registers -> unsigned bytes in shared memory (lane layout of a record:
            // half h, lane L = (r, t): W words of row 8h + r, inputs 8 * (t*W + j) ..)
            sc_cur = sc_set[jj]; z_cur = z_set[jj];
#pragma unroll
            for (int it = 0; it < TC_UNPACK; it++) {
                const int idx = tid + it * TC_THREADS, sub = idx >> 6, hl = idx & 63;
                const int h = hl >> 5, L = hl & 31, r = L >> 2, t = L & 3;
                const uint32_t arow = sub * 16 + h * 8 + r;
#pragma unroll
                for (uint32_t j = 0; j < 4; j++) {
                    if (j < W) {
                        // 8 weights -> 8 bytes in the block order (0,2,4,6,1,3,5,7), the order of the digit image
                        const uint2 b = make_uint2(wreg[jj][it][j] & 0x0F0F0F0Fu, (wreg[jj][it][j] >> 4) & 0x0F0F0F0Fu);
                        *reinterpret_cast<uint2*>(stage_a[s] + swz(arow, (t * W + j) * 8, GS)) = b;
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the MMA unit
            if (g + TC_AHEAD < G) load_group(g + TC_AHEAD, wreg[jj], sc_set[jj], z_set[jj]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (g < G && tid == 0) {
            // ---- issue the MMAs of group g (one thread), completion arrives on mma_done[s]
            if (mbar_wait(&b_full[s], (uint32_t)(g >> 1) & 1u)) {
                const uint32_t d = tmem_base + (uint32_t)s * 256u;
                const uint32_t a0 = smem_addr(stage_a[s]), b0 = smem_addr(stage_b[s]);
                for (uint32_t k = 0; k < W; k++) {
                    const uint64_t da = umma_desc(a0 + 32 * k, GS), db = umma_desc(b0 + 32 * k, GS);
                    const uint32_t accumulate = k ? 1u : 0u;
                    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
                                 ::"r"(d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(&mma_done[s])) : "memory");
            } else {
                failed = 1;
                if (P.status) atomicExch(P.status, 2001);
                // release the waiters of this stage
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&mma_done[s])) : "memory");
            }
        }
        if (g > 0) {
            // ---- drain group g-1 from the other accumulator
            const int ps = (g - 1) & 1;
            if (ok && !mbar_wait(&mma_done[ps], (uint32_t)((g - 1) >> 1) & 1u)) {
                ok = false;
                failed = 1;
                if (P.status) atomicExch(P.status, 2002);
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (tid == 0 && g + 1 < G && ok && !failed) {
                // the MMAs of group g-1 are done: their stage is free for the digits of group g+1
                mbar_expect_tx(&b_full[ps], b_bytes);
                bulk_g2s(stage_b[ps], P.bimg + (size_t)(gb + g + 1) * b_bytes, b_bytes, &b_full[ps]);
            }
            if (ok && !failed) {
                const float sc = sc_prev;
                const int z = z_prev;
                const int2* sv = sv_s[(g - 1) % 3] + chalf * tok_per;
                const uint32_t tbase = tmem_base + (uint32_t)ps * 256u + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(chalf * tok_per * 4);
#pragma unroll
                for (int c0 = 0; c0 < TC_ACC * 4; c0 += 32) {  // 32 columns = 8 tokens per load
                    if (c0 >= tok_per * 4) break;  // warp-uniform
                    uint32_t v[32];
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                                 : "r"(tbase + (uint32_t)c0) : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        const int tk = c0 / 4 + q;  // token inside this half
                        if (tk < tok_per) {
                            const int2 s2 = sv[tk];
                            const int hi = (int)v[4 * q] * 128 + (int)v[4 * q + 1] - z * s2.x;
                            const int lo = (int)v[4 * q + 2] * 128 + (int)v[4 * q + 3] - z * s2.y;
                            acc[tk] = fmaf(sc, fmaf((float)hi, 16384.0f, (float)lo), acc[tk]);
                        }
                    }
                }
            }
        }
    }
    }

    // ---- output: out[m][orow] (+= for the residual epilogue), scaled per token
    if (ok && !failed && row_ok && orow < P.rows) {
#pragma unroll
        for (int tk = 0; tk < TC_ACC; tk++) {
            const int m = chalf * tok_per + tk;
            if (tk < tok_per && m < P.m) {
                const float y = acc[tk] * __ldg(P.oscale + m);
                float* dst = P.out + (size_t)blockIdx.y * P.kstride + (size_t)m * P.ldo + orow;
                *dst = P.epi == EPI_RESID ? *dst + y : y;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
}

// at least 120 KB so that only one CTA (one owner of the tensor memory) is resident per SM
size_t gemm_tc_smem_bytes(int gs, int n) {
    const size_t need = 2 * (((size_t)128 * gs + (size_t)n * gs + 1023) & ~(size_t)1023) + 1024;
    return need < 120 * 1024 ? 120 * 1024 : need;
}

cudaError_t gemm_tc_init(int max_smem) {
    return cudaFuncSetAttribute(gemm_q4_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
}

cudaError_t launch_gemm_tc(const TcParams& p, cudaStream_t st) {
    const int grid = (p.tiles16 + 7) / 8;
    const int ks = p.ksplit > 1 ? p.ksplit : 1;
    g_launches++;
    gemm_q4_tc_kernel<<<dim3(grid, ks), TC_THREADS, gemm_tc_smem_bytes(p.gs, p.n), st>>>(p);
    return cudaGetLastError();
}

}  // namespace l2
