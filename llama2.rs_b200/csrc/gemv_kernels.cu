// Fused rmsnorm + 4-bit dequant + GEMV for QLinear::matvec at batch 1 (src/gptq.rs:94-176),
// hand-written for sm_100a.
//
// The kernel is bound by HBM only if it spends about one instruction per 4-bit weight, so the
// inner product runs on the tensor cores with exact integer arithmetic:
//
//   * the activation vector is turned, once per CTA, into four 7-bit digits per element:
//     X = round(v * 2^e) with |X| < 2^27, X = d0*2^21 + d1*2^14 + d2*2^7 + d3 with d0 = X >> 21 signed
//     and d1..d3 in 0..127 (block floating point over the whole vector; the error is below 2^-27 of
//     the largest element, finer than f32);
//   * weights stay packed nibbles in HBM; in registers a word becomes two MMA operands with three
//     bit operations (lo = w & 0x0F0F0F0F, hi = (w >> 4) & 0x0F0F0F0F), no int->float conversion;
//   * mma.sync.m16n8k32 (u8 x s8 -> s32) multiplies 16 rows x 32 weights by the four digit columns;
//     the sums over one quantisation group are exact integers, the zero point is removed with the
//     group's digit sums, and one f32 FMA per row and group applies the scale;
//   * work split: every CTA owns a contiguous run of whole 16-row tiles, i.e. one contiguous byte
//     range of (tile, group) unit records; tiles are summed over the warps through shared memory in
//     warp order, so results are bit-reproducible and no CTA ever waits for another;
//   * weights never pass through registers on their way in: a producer warp streams the CTA's range
//     into a ring of shared-memory slots with large bulk asynchronous copies (cp.async.bulk,
//     completion counted on an mbarrier per slot, every wait bounded); the first copies are issued
//     before the kernel waits for its predecessor and keep HBM streaming while the activations are
//     staged; the 16 consumer warps take the units of a slot two at a time;
//   * every CTA also asks the L2 to fetch its share of the next kernel's weights
//     (cp.async.bulk.prefetch.L2).
//
// rmsnorm is folded in by linearity: the digits are those of (norm weight * x) and the output is
// multiplied by 1/sqrt(mean(x^2)+eps) at the end.  Epilogues: store, residual add + scatter into
// the next consumers' K orders, or SwiGLU (w1 and w3 rows of a tile are processed together).
#include <cfloat>
#include <cmath>

#include "gemv_device.cuh"
#include "kernels.cuh"

namespace l2 {

unsigned long long* g_sk_trace = nullptr;

#define SK_STAMP(i) do { if (P.trace && threadIdx.x == 0) P.trace[blockIdx.x * 8 + (i)] = clock64(); } while (0)
#define SK_STAMP0() do { if (threadIdx.x == 0) t_entry = clock64(); } while (0)


template <int W, int NSEG>
__global__ void __launch_bounds__(SK_THREADS + 32, 1) gemv_sk_kernel(const SkParams* __restrict__ gp) {
    constexpr int GS = 32 * W;
    constexpr int ROWS = 16 * NSEG;  // rows of a (super) tile
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ float red[2 * SK_WARPS + 2];
    __shared__ float oscale[2];
    __shared__ __align__(8) uint64_t full[SK_MAX_SLOTS], empty[SK_MAX_SLOTS];
    __shared__ volatile int abort_flag;
    __shared__ SkParams sp;

    // The launch record lives in global memory: one cooperative 128-bit load per thread brings it into
    // shared memory (kernel arguments this large would cost a chain of constant-cache misses).
    long long t_entry = 0;
    SK_STAMP0();
    static_assert(sizeof(SkParams) % 16 == 0, "SkParams is copied in 16-byte pieces");
    if (threadIdx.x < sizeof(SkParams) / 16)
        reinterpret_cast<uint4*>(&sp)[threadIdx.x] = __ldg(reinterpret_cast<const uint4*>(gp) + threadIdx.x);
    __syncthreads();
    const SkParams& P = sp;
    if (P.trace && threadIdx.x == 0) P.trace[blockIdx.x * 8] = t_entry;

    int ji = 0;
    for (int j = 1; j < P.njobs; j++)
        if ((int)blockIdx.x >= P.job[j].cta0) ji = j;
    const SkJob& J = P.job[ji];
    const int cta = blockIdx.x - J.cta0;
    const int G = J.G, Gs = NSEG * G;
    // whole tiles per CTA: the first `trem` CTAs own tq + 1 tiles, the others tq
    const int tau_first = cta * J.tq + min(cta, J.trem);
    const int nt = J.tq + (cta < J.trem ? 1 : 0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = nt * Gs;                      // units of this CTA

    // shared memory carve-up
    const int dstride = J.in + 16;
    uint8_t* digits = smem;                                              // [NSEG][4][in + 16]
    int* ss = reinterpret_cast<int*>(smem + (size_t)NSEG * 4 * dstride);  // [NSEG][G][2]
    float* partial = reinterpret_cast<float*>(ss + NSEG * G * 2);        // [ptiles][SK_WARPS][ROWS]
    constexpr uint32_t UB = 256u * W + 80u;  // bytes of one unit record
    const int SU = P.chunk, NS = P.slots;    // units per ring slot, ring slots
    const uint32_t slot_bytes = (uint32_t)SU * UB;
    const size_t fixed_bytes = ((size_t)NSEG * 4 * dstride + (size_t)NSEG * G * 8 + (size_t)P.ptiles * SK_WARPS * ROWS * 4 + 127) & ~(size_t)127;
    uint8_t* ring = smem + fixed_bytes;      // 128-byte aligned (bulk copies need 16)
    const int nslots = (n + SU - 1) / SU;    // slot fills this CTA goes through

    if (threadIdx.x == 0) {
        for (int i = 0; i < NS; i++) { mbar_init(full + i, 1); mbar_init(empty + i, SK_WARPS); }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // ================= producer warp: streams the CTA's units through the ring ===================
    // Slot fill k holds units [k*SU, min((k+1)*SU, n)) of the CTA's range.  Units are contiguous in
    // memory inside one (tile, segment) run, and from tile to tile when there is a single segment, so
    // a fill is one large bulk copy (or one per run it touches).  Large copies matter: the copy
    // engine spends a fixed time per request.  The first fills do not depend on the previous kernel
    // and are issued before the dependency wait.
    if (warp == SK_WARPS) {
        if (lane == 0) {
            // the next kernel's weights: every CTA asks the L2 for an equal slice of each range
            for (int i = 0; i < P.n_next; i++) {
                const size_t per = P.next_slice[i], off = per * blockIdx.x;
                if (off < P.next_bytes[i]) prefetch_l2(static_cast<const char*>(P.next_ptr[i]) + off, (uint32_t)min(per, P.next_bytes[i] - off));
            }
            int tl = 0, seg = 0, g = 0;  // position of the next unit to copy
            for (int k = 0; k < nslots; k++) {
                const int slot = k % NS;
                if (k >= NS && !mbar_wait(empty + slot, (uint32_t)(k / NS - 1) & 1u)) {
                    if (P.status) atomicExch(P.status, 1002);
                    abort_flag = 1;
                    break;
                }
                if (abort_flag) break;
                int left = min(SU, n - k * SU);
                mbar_expect_tx(full + slot, (uint32_t)left * UB);
                uint8_t* dst = ring + (size_t)slot * slot_bytes;
                while (left > 0) {
                    // NSEG == 1: consecutive tiles are consecutive in memory, one copy covers them all
                    const int run = NSEG == 1 ? left : min(left, G - g);
                    const SkSeg& S = J.seg[NSEG == 1 ? 0 : seg];
                    const size_t mu = (size_t)(tau_first + tl) * G + g;
                    bulk_g2s(dst, S.rec + mu * (UB / 4), (uint32_t)run * UB, full + slot);
                    dst += (size_t)run * UB;
                    left -= run;
                    g += run;
                    while (g >= G) { g -= G; if (++seg == NSEG) { seg = 0; tl++; } }
                }
            }
        }
        grid_launch_dependents();
        return;
    }

    // ================= consumer warps ================================================================
    // epilogue operands of this warp's first tile that do not depend on the previous kernel
    const int e_row = (tau_first + warp) * 16 + (lane & 15);
    const bool e_pre = NSEG == 1 && warp < nt && lane < 16 && e_row < J.rows && J.epi == EPI_RESID;
    int e_idx[3] = {0, 0, 0};
    if (e_pre)
        for (int s = 0; s < 3; s++)
            if (s < J.nscatter) e_idx[s] = __ldg(J.sidx[s] + e_row);
    for (int i = threadIdx.x; i < nt * SK_WARPS * ROWS; i += SK_THREADS) partial[i] = 0.f;

    SK_STAMP(1);
    grid_dependency_wait();
    grid_launch_dependents();
    SK_STAMP(2);
    float e_out = 0.f;
    if (e_pre) e_out = J.out[e_row];

    // ---- stage the activation digits (its first barrier also orders the zeroing of `partial`)
    if (n > 0) {
#pragma unroll
        for (int s = 0; s < NSEG; s++) {
            const float f = stage_digits<W>(J.seg[s], J.in, P.eps, digits + (size_t)s * 4 * dstride, ss + s * G * 2, red);
            if (threadIdx.x == 0) oscale[s] = f;
        }
    }
    consumer_sync();

    SK_STAMP(3);
    // ---- main loop: in every slot fill this warp takes units 2*warp and 2*warp + 1 (+ 2*SK_WARPS ...)
    const int r = lane >> 2, t = lane & 3;
    float tot0 = 0.f, tot1 = 0.f;
    int cur_tl = -1, cur_seg = 0;  // (tile, segment) the row sums belong to
    bool ok = true;
    auto flush = [&]() {
        if (cur_tl >= 0) {
            // lanes t = 0 hold digits 0,1 (weight 2^14 relative to digits 2,3 held by lanes t = 1)
            float a = t == 0 ? tot0 * 16384.0f : tot0, b = t == 0 ? tot1 * 16384.0f : tot1;
            a += __shfl_xor_sync(0xffffffffu, a, 1);
            b += __shfl_xor_sync(0xffffffffu, b, 1);
            if (t == 0) {
                float* dst = partial + ((size_t)cur_tl * SK_WARPS + warp) * ROWS + cur_seg * 16;
                dst[r] = a;
                dst[r + 8] = b;
            }
        }
        tot0 = tot1 = 0.f;
    };
    // scale, zero point and digit sums of one finished unit (exact integers up to the final FMA)
    auto unit_finish = [&](const uint8_t* rec, int tl, int seg, int g, const int (&c)[4]) {
        if (tl != cur_tl || seg != cur_seg) { flush(); cur_tl = tl; cur_seg = seg; }  // warp-uniform
        if (t < 2) {
            const uint32_t* mt = reinterpret_cast<const uint32_t*>(rec + 256 * W);
            const float s0 = __uint_as_float(mt[r]), s1 = __uint_as_float(mt[8 + r]);
            const int z0 = (int)((mt[16] >> (4 * r)) & 15u) + 1, z1 = (int)((mt[17] >> (4 * r)) & 15u) + 1;  // src/gptq.rs:148
            const int sv = ss[((NSEG == 1 ? 0 : seg) * G + g) * 2 + t];
            tot0 = fmaf(s0, (float)(c[0] * 128 + c[1] - z0 * sv), tot0);
            tot1 = fmaf(s1, (float)(c[2] * 128 + c[3] - z1 * sv), tot1);
        }
    };
    constexpr uint32_t M = 0x0F0F0F0Fu;
    // MMAs of one unit whose record starts at rec; dg points at this lane's digits of the unit's group
    auto unit_mma = [&](const uint8_t* rec, const uint8_t* dg, int (&c)[4]) {
        c[0] = c[1] = c[2] = c[3] = 0;
        if constexpr (W == 4) {
            const uint4 a = *reinterpret_cast<const uint4*>(rec + lane * 16), b = *reinterpret_cast<const uint4*>(rec + 512 + lane * 16);
            uint4 d0 = make_uint4(0, 0, 0, 0), d1 = d0;
            if (r < 4) { d0 = reinterpret_cast<const uint4*>(dg)[0]; d1 = reinterpret_cast<const uint4*>(dg)[1]; }
            mma_u8s8(c, a.x & M, b.x & M, (a.x >> 4) & M, (b.x >> 4) & M, d0.x, d0.y);
            mma_u8s8(c, a.y & M, b.y & M, (a.y >> 4) & M, (b.y >> 4) & M, d0.z, d0.w);
            mma_u8s8(c, a.z & M, b.z & M, (a.z >> 4) & M, (b.z >> 4) & M, d1.x, d1.y);
            mma_u8s8(c, a.w & M, b.w & M, (a.w >> 4) & M, (b.w >> 4) & M, d1.z, d1.w);
        } else {
#pragma unroll
            for (int j = 0; j < W; j++) {
                const uint32_t a = *reinterpret_cast<const uint32_t*>(rec + lane * 4 * W + 4 * j);
                const uint32_t b = *reinterpret_cast<const uint32_t*>(rec + 128 * W + lane * 4 * W + 4 * j);
                uint2 bb = make_uint2(0u, 0u);
                if (r < 4) bb = *reinterpret_cast<const uint2*>(dg + 8 * j);
                mma_u8s8(c, a & M, b & M, (a >> 4) & M, (b >> 4) & M, bb.x, bb.y);
            }
        }
    };
    auto locate = [&](int u, int& tl, int& seg, int& g) {  // unit index in the CTA -> tile, segment, group
        tl = (int)((float)u * J.rGs);
        if (tl * Gs > u) tl--; else if ((tl + 1) * Gs <= u) tl++;
        g = u - tl * Gs;
        seg = 0;
        if (NSEG == 2 && g >= G) { seg = 1; g -= G; }
    };
    auto digits_of = [&](int seg, int g) {
        return digits + (size_t)(NSEG == 1 ? 0 : seg) * 4 * dstride + (size_t)r * dstride + g * GS + t * (8 * W);
    };
    for (int k = 0; k < nslots; k++) {
        const int slot = k % NS;
        const int m = min(SU, n - k * SU);  // units in this fill
        if (ok && (abort_flag || !mbar_wait(full + slot, (uint32_t)(k / NS) & 1u))) {
            ok = false;
            if (P.status) atomicExch(P.status, 1001);
            abort_flag = 1;
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (!P.debug_skip) {
            const uint8_t* base = ring + (size_t)slot * slot_bytes;
            for (int j = 2 * warp; j < m; j += 2 * SK_WARPS) {
                const bool two = j + 1 < m;
                int tl0, seg0, g0, tl1 = 0, seg1 = 0, g1 = 0;
                locate(k * SU + j, tl0, seg0, g0);
                if (two) { g1 = g0 + 1; seg1 = seg0; tl1 = tl0; if (g1 == G) locate(k * SU + j + 1, tl1, seg1, g1); }
                int c0[4], c1[4];
                const uint8_t* rec0 = base + (size_t)j * UB;
                unit_mma(rec0, digits_of(seg0, g0), c0);
                if (two) unit_mma(rec0 + UB, digits_of(seg1, g1), c1);
                unit_finish(rec0, tl0, seg0, g0, c0);
                if (two) unit_finish(rec0 + UB, tl1, seg1, g1, c1);
            }
        }
        __syncwarp();  // every lane has read the slot
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(empty + slot)) : "memory");
    }
    flush();
    if (!ok) {
        // copies may still be in flight into this CTA's shared memory: give them a bounded time to land
        // before the CTA exits, without using their data
        for (int i = 0; i < NS; i++) { mbar_wait(full + i, 0, 1u << 8); mbar_wait(full + i, 1, 1u << 8); }
    }
    SK_STAMP(4);
    consumer_sync();
    SK_STAMP(5);

    // ---- per tile: sum the warps in order, then the epilogue
    for (int tl = warp; tl < nt; tl += SK_WARPS) {
        const int tau = tau_first + tl;
        float v = 0.f;
        if (lane < ROWS)
            for (int w = 0; w < SK_WARPS; w++) v += partial[((size_t)tl * SK_WARPS + w) * ROWS + lane];
        const float y = v * oscale[lane >> 4 & (NSEG - 1)];
        const int row = tau * 16 + (lane & 15);
        if (NSEG == 2) {  // SwiGLU: lanes 0-15 hold w1 rows, lanes 16-31 the same rows of w3 (src/models.rs:92-98)
            const float y3 = __shfl_down_sync(0xffffffffu, y, 16);
            if (lane < 16 && row < J.rows) {
                const float sg = y * (1.0f / (1.0f + expf(-y)));
                J.out[row] = sg * y3;
            }
        } else if (lane < 16 && row < J.rows) {
            if (J.epi == EPI_STORE) {
                J.out[row] = y;
            } else {  // residual add (src/models.rs:47-51) + copies in the next consumers' K orders
                const bool pre = e_pre && tl == warp;
                const float xv = (pre ? e_out : J.out[row]) + y;
                J.out[row] = xv;
                for (int s = 0; s < 3; s++)
                    if (s < J.nscatter) J.sdst[s][pre ? e_idx[s] : J.sidx[s][row]] = xv;
            }
        }
    }
    SK_STAMP(6);
}

size_t sk_smem_fixed(int in, int G, int nseg, int ptiles) {
    return (size_t)nseg * 4 * (in + 16) + (size_t)nseg * G * 2 * 4 + (size_t)ptiles * SK_WARPS * 16 * nseg * 4;
}

size_t sk_slot_bytes(int group_size, int chunk) { return (size_t)chunk * (8 * (size_t)group_size + 80); }

template <int W, int NSEG>
static cudaError_t launch_sk_t(const SkParams* p, int grid, size_t smem, cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(SK_THREADS + 32);  // 16 consumer warps + 1 producer warp
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    g_launches++;
    return cudaLaunchKernelEx(&cfg, gemv_sk_kernel<W, NSEG>, p);
}

cudaError_t launch_sk(const SkParams* p, int group_size, int nseg, int grid, size_t smem, cudaStream_t st, bool pdl) {
    const int w = group_size / 32;
    if (nseg == 1) {
        if (w == 4) return launch_sk_t<4, 1>(p, grid, smem, st, pdl);
        if (w == 2) return launch_sk_t<2, 1>(p, grid, smem, st, pdl);
        return launch_sk_t<1, 1>(p, grid, smem, st, pdl);
    }
    if (w == 4) return launch_sk_t<4, 2>(p, grid, smem, st, pdl);
    if (w == 2) return launch_sk_t<2, 2>(p, grid, smem, st, pdl);
    return launch_sk_t<1, 2>(p, grid, smem, st, pdl);
}

cudaError_t sk_init(int max_smem) {
    cudaError_t e;
#define L2_SK_ATTR(W, N) \
    if ((e = cudaFuncSetAttribute(gemv_sk_kernel<W, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem)) != cudaSuccess) return e;
    L2_SK_ATTR(4, 1) L2_SK_ATTR(2, 1) L2_SK_ATTR(1, 1) L2_SK_ATTR(4, 2) L2_SK_ATTR(2, 2) L2_SK_ATTR(1, 2)
#undef L2_SK_ATTR
    return cudaSuccess;
}

}  // namespace l2
