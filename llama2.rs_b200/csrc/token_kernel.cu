// One token of the B=1 forward pass (src/models.rs:178-298, src/inference.rs:134-190) as ONE
// persistent kernel for sm_100a: one CTA per SM, every CTA walks the same list of phases
//
//   embed | per layer: wq/wk/wv GEMV | rope + KV append + attention | wo GEMV + residual |
//   w1/w3 GEMV + SwiGLU | w2 GEMV + residual | final rmsnorm + classifier | select
//
// and all CTAs meet at a grid-wide barrier between two phases.  Compared with one launch per phase
// this removes the launch gaps and, above all, lets the weights stream without a break: warp 16 of
// every CTA is a producer that walks the phase list ahead of the 16 consumer warps and keeps a ring
// of shared-memory slots filled with the CTA's next unit records (large cp.async.bulk copies,
// mbarrier per slot), across phase boundaries, while the consumers are still in the previous
// phase, at the grid barrier, or staging the next activation vector.
//
// Waits are bounded everywhere (mbarriers, the grid barrier, the producer's wait for a free record
// buffer): a wait that gives up writes a status word, raises the CTA's abort flag, lets copies in
// flight land and leaves; the other CTAs see the status word at their next barrier and leave too.
// The launch is cooperative, so all CTAs are resident together.
#include "gemv_device.cuh"
#include "kernels.cuh"

namespace l2 {

constexpr int TK_NREC = 4;                    // phase records buffered in shared memory
constexpr uint32_t TK_BAR_LIMIT = 1u << 22;   // polls of the grid barrier before giving up (about a second)

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TK_STAMP_NS(p, i) do { if (tk.trace && threadIdx.x == 0) tk.trace[((size_t)blockIdx.x * tk.nphases + (p)) * 16 + (i)] = global_ns(); } while (0)
#define TK_STAMP(p, i) do { if (tk.trace && threadIdx.x == 0) tk.trace[((size_t)blockIdx.x * tk.nphases + (p)) * 16 + (i)] = clock64(); } while (0)

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

struct CtaRange { int ji, tau_first, nt; };

// Tiles of the launch record `P` that this CTA owns (the same split as the stand-alone kernel; CTAs
// beyond the last job own nothing).
__device__ __forceinline__ CtaRange sk_cta_range(const SkParams& P) {
    CtaRange c;
    c.ji = 0;
    for (int j = 1; j < P.njobs; j++)
        if ((int)blockIdx.x >= P.job[j].cta0) c.ji = j;
    const SkJob& J = P.job[c.ji];
    const int cta = blockIdx.x - J.cta0;
    if (cta >= J.ncta) { c.tau_first = 0; c.nt = 0; return c; }
    c.tau_first = cta * J.tq + min(cta, J.trem);
    c.nt = J.tq + (cta < J.trem ? 1 : 0);
    return c;
}

struct Ring {
    uint8_t* base;
    uint64_t *full, *empty;
    uint32_t slot_bytes;
    int SU, NS;
    volatile int* abort_flag;
    int* status;
    const uint8_t* zeros;  // 32 bytes of zeros in shared memory
};

// Producer side of one GEMV phase (one thread): streams this CTA's unit records through the ring.
// `kfill` counts slot fills since the start of the kernel.
template <int W>
__device__ bool produce_units(const SkParams& P, int NSEG, const Ring& R, uint32_t& kfill) {
    constexpr uint32_t UB = 256u * W + 80u;
    const CtaRange c = sk_cta_range(P);
    const SkJob& J = P.job[c.ji];
    const int G = J.G, n = c.nt * NSEG * G;
    const int nslots = (n + R.SU - 1) / R.SU;
    // A later phase's weights: every CTA asks the L2 for an equal slice of them, one piece with each
    // of its own slot fills, so that the requests are paced with the demand instead of queueing in
    // front of it.
    const int pieces = max(nslots, 1);
    const char* pf_ptr[6];
    uint32_t pf_mine[6], pf_piece[6];
    for (int i = 0; i < 6; i++) {
        pf_ptr[i] = nullptr; pf_mine[i] = 0; pf_piece[i] = 0;
        if (i < P.n_next) {
            const size_t per = P.next_slice[i], off = per * blockIdx.x;
            if (off < P.next_bytes[i]) {
                pf_ptr[i] = static_cast<const char*>(P.next_ptr[i]) + off;
                pf_mine[i] = (uint32_t)min(per, P.next_bytes[i] - off);
                pf_piece[i] = ((pf_mine[i] + (uint32_t)pieces - 1u) / (uint32_t)pieces + 127u) & ~127u;
            }
        }
    }
    auto prefetch_piece = [&](int k) {
#pragma unroll
        for (int i = 0; i < 6; i++) {
            const uint32_t b = pf_piece[i] * (uint32_t)k;
            if (b < pf_mine[i]) prefetch_l2(pf_ptr[i] + b, min(pf_piece[i], pf_mine[i] - b));
        }
    };
    if (nslots == 0) prefetch_piece(0);
    int tl = 0, seg = 0, g = 0;
    for (int k = 0; k < nslots; k++) {
        prefetch_piece(k);
        const uint32_t f = kfill + (uint32_t)k;
        const int slot = (int)(f % (uint32_t)R.NS);
        if (f >= (uint32_t)R.NS && !mbar_wait(R.empty + slot, (f / (uint32_t)R.NS - 1u) & 1u)) {
            if (R.status) atomicExch(R.status, 1002);
            *R.abort_flag = 1;
            return false;
        }
        if (*R.abort_flag) return false;
        int left = min(R.SU, n - k * R.SU);
        mbar_expect_tx(R.full + slot, (uint32_t)left * UB);
        uint8_t* dst = R.base + (size_t)slot * R.slot_bytes;
        while (left > 0) {
            const int run = NSEG == 1 ? left : min(left, G - g);  // one matrix: tiles follow one another in memory
            const SkSeg& S = J.seg[NSEG == 1 ? 0 : seg];
            const size_t mu = (size_t)(c.tau_first + tl) * G + g;
            bulk_g2s(dst, S.rec + mu * (UB / 4), (uint32_t)run * UB, R.full + slot);
            dst += (size_t)run * UB;
            left -= run;
            g += run;
            while (g >= G) { g -= G; if (++seg == NSEG) { seg = 0; tl++; } }
        }
    }
    kfill += (uint32_t)nslots;
    return true;
}

__device__ __forceinline__ void prefetch_line_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Producer warp, ahead of the consumers: asks the L2 for the small operands of a GEMV phase that do
// not depend on the previous phase (norm weights, spread over the CTAs; the scatter indices and the
// residual rows of this CTA), so that the consumers' dependent loads do not go to HBM.
__device__ void warm_operands(const SkParams& P, int NSEG) {
    const int lane = threadIdx.x & 31;
    const CtaRange c = sk_cta_range(P);
    const SkJob& J = P.job[c.ji];
    const int lines = J.in / 32;  // 128-byte lines of a norm weight vector
    for (int s = 0; s < NSEG; s++)
        if (J.seg[s].nw)
            for (int i = blockIdx.x + lane * gridDim.x; i < lines; i += 32 * gridDim.x) prefetch_line_l2(J.seg[s].nw + (size_t)i * 32);
    if (J.epi == EPI_RESID && c.nt > 0) {
        const int row0 = c.tau_first * 16, nrows = min(c.nt * 16, J.rows - row0);
        for (int i = lane * 32; i < nrows; i += 32 * 32) {
            prefetch_line_l2(J.out + row0 + i);
            for (int sc = 0; sc < J.nscatter; sc++) prefetch_line_l2(J.sidx[sc] + row0 + i);
        }
    }
}

// Consumer side of one GEMV phase: stage the digits, multiply, reduce, epilogue.  Returns false
// when a wait gave up.  `kbase` is the number of slot fills consumed before this phase.
template <int W, int NSEG>
__device__ __forceinline__ bool gemv_phase(const SkParams& P, uint8_t* smem, const Ring& R, float* red, float* oscale, uint32_t& kbase,
                           unsigned long long* stamp) {
    constexpr int GS = 32 * W;
    constexpr int ROWS = 16 * NSEG;
    constexpr uint32_t UB = 256u * W + 80u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const CtaRange cr = sk_cta_range(P);
    const SkJob& J = P.job[cr.ji];
    const int G = J.G, Gs = NSEG * G, nt = cr.nt, tau_first = cr.tau_first;
    const int n = nt * Gs;
    const int SU = R.SU, NS = R.NS;
    const int nslots = (n + SU - 1) / SU;

    const int dstride = J.in + 16;
    uint8_t* digits = smem;                                               // [NSEG][4][in + 16]
    int* ss = reinterpret_cast<int*>(smem + (size_t)NSEG * 4 * dstride);   // [NSEG][G][2]
    float* partial = reinterpret_cast<float*>(ss + NSEG * G * 2);         // [nt][SK_WARPS][ROWS]

    for (int i = threadIdx.x; i < nt * SK_WARPS * ROWS; i += SK_THREADS) partial[i] = 0.f;
    if (n > 0) {  // the first barrier inside also orders the zeroing of `partial`
        if (NSEG == 2 && J.in <= 2 * 8 * SK_THREADS) {
            // w1 and w3 read the same x, each in its own K order: one pass over the statistics
            const float f = stage_digits_pair<W>(J.seg[0], J.seg[NSEG - 1], J.in, P.eps, digits, digits + (size_t)4 * dstride, ss, ss + G * 2, red);
            if (threadIdx.x == 0) oscale[0] = oscale[1] = f;
        } else {
#pragma unroll
            for (int s = 0; s < NSEG; s++) {
                const float f = stage_digits<W>(J.seg[s], J.in, P.eps, digits + (size_t)s * 4 * dstride, ss + s * G * 2, red);
                if (threadIdx.x == 0) oscale[s] = f;
            }
        }
    }
    consumer_sync();
    if (stamp && threadIdx.x == 0) stamp[1] = clock64();

    // ---- main loop.  In every slot fill this warp owns units 2*warp and 2*warp + 1.  With four warps
    // per scheduler the loop lives on instruction count and on the length of its dependent chain, so
    //  * the common case (a full slot: every warp has its pair) is straight-line code without
    //    data-dependent branches: all lanes run the scale / zero-point step (lanes t >= 2 hold the
    //    unused MMA columns and are ignored when the sums are flushed), lanes r >= 4 read their digits
    //    from a block of zeros instead of skipping the load;
    //  * tile and group are carried from fill to fill instead of being recomputed;
    //  * the loop is software-pipelined by hand: the MMAs of the current pair are issued, then the
    //    scale / zero-point step of the previous pair runs while they are in flight, and only then is
    //    the previous slot handed back to the producer.
    const int r = lane >> 2, t = lane & 3;
    float tot0 = 0.f, tot1 = 0.f;
    int cur_key = -1;  // 2 * tile + segment the row sums belong to
    bool ok = true;
    auto flush = [&]() {
        if (cur_key >= 0) {
            // lanes t = 0 hold digits 0,1 (weight 2^14 relative to digits 2,3 held by lanes t = 1)
            float a = t == 0 ? tot0 * 16384.0f : tot0, b = t == 0 ? tot1 * 16384.0f : tot1;
            a += __shfl_xor_sync(0xffffffffu, a, 1);
            b += __shfl_xor_sync(0xffffffffu, b, 1);
            if (t == 0) {
                float* dst = partial + ((size_t)(cur_key >> 1) * SK_WARPS + warp) * ROWS + (cur_key & 1) * 16;
                dst[r] = a;
                dst[r + 8] = b;
            }
        }
        tot0 = tot1 = 0.f;
    };
    const int zshift = 4 * r;
    const int* ss_lane = ss + (t & 1);
    // scale, zero point and digit sums of one finished unit (exact integers up to the final FMA);
    // gg = position of the unit inside its (super) tile: segment * G + group
    auto unit_finish = [&](const uint8_t* rec, int tl, int gg, const int (&c)[4]) {
        const int key = 2 * tl + (NSEG == 2 && gg >= G ? 1 : 0);
        if (key != cur_key) { flush(); cur_key = key; }  // warp-uniform
        const uint32_t* mt = reinterpret_cast<const uint32_t*>(rec + 256 * W);
        const float s0 = __uint_as_float(mt[r]), s1 = __uint_as_float(mt[8 + r]);
        const uint2 zz = *reinterpret_cast<const uint2*>(mt + 16);
        const int z0 = (int)((zz.x >> zshift) & 15u) + 1, z1 = (int)((zz.y >> zshift) & 15u) + 1;  // src/gptq.rs:148
        const int sv = ss_lane[gg * 2];
        tot0 = fmaf(s0, (float)(c[0] * 128 + c[1] - z0 * sv), tot0);
        tot1 = fmaf(s1, (float)(c[2] * 128 + c[3] - z1 * sv), tot1);
    };
    constexpr uint32_t M = 0x0F0F0F0Fu;
    // this lane's digits of the group at position gg; lanes r >= 4 (MMA columns 4..7) read zeros
    const uint8_t* dg_lane = r < 4 ? digits + (size_t)r * dstride + t * (8 * W) : R.zeros;
    const int dmul = r < 4 ? 1 : 0;
    auto digits_of = [&](int gg) {
        const int seg = NSEG == 2 && gg >= G ? 1 : 0;
        return dg_lane + (seg * 4 * dstride + (gg - seg * G) * GS) * dmul;
    };
    // loads and MMAs of one unit whose record starts at rec
    auto unit_mma = [&](const uint8_t* rec, const uint8_t* dg, int (&c)[4]) {
        if constexpr (W == 4) {
            const uint4 a = *reinterpret_cast<const uint4*>(rec + lane * 16), b = *reinterpret_cast<const uint4*>(rec + 512 + lane * 16);
            const uint4 d0 = reinterpret_cast<const uint4*>(dg)[0], d1 = reinterpret_cast<const uint4*>(dg)[1];
            mma_u8s8_first(c, a.x & M, b.x & M, (a.x >> 4) & M, (b.x >> 4) & M, d0.x, d0.y);
            mma_u8s8(c, a.y & M, b.y & M, (a.y >> 4) & M, (b.y >> 4) & M, d0.z, d0.w);
            mma_u8s8(c, a.z & M, b.z & M, (a.z >> 4) & M, (b.z >> 4) & M, d1.x, d1.y);
            mma_u8s8(c, a.w & M, b.w & M, (a.w >> 4) & M, (b.w >> 4) & M, d1.z, d1.w);
        } else if constexpr (W == 2) {
            const uint2 a = *reinterpret_cast<const uint2*>(rec + lane * 8), b = *reinterpret_cast<const uint2*>(rec + 256 + lane * 8);
            const uint4 d0 = reinterpret_cast<const uint4*>(dg)[0];
            mma_u8s8_first(c, a.x & M, b.x & M, (a.x >> 4) & M, (b.x >> 4) & M, d0.x, d0.y);
            mma_u8s8(c, a.y & M, b.y & M, (a.y >> 4) & M, (b.y >> 4) & M, d0.z, d0.w);
        } else {
            const uint32_t a = *reinterpret_cast<const uint32_t*>(rec + lane * 4);
            const uint32_t b = *reinterpret_cast<const uint32_t*>(rec + 128 + lane * 4);
            const uint2 bb = *reinterpret_cast<const uint2*>(dg);
            mma_u8s8_first(c, a & M, b & M, (a >> 4) & M, (b >> 4) & M, bb.x, bb.y);
        }
    };
    auto release = [&](int slot) {
        __syncwarp();  // every lane has read the slot
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(R.empty + slot)) : "memory");
    };
    // position of this warp's first unit of the current fill; advanced by SU units per fill
    int tl0 = (2 * warp) / Gs, gg0 = (2 * warp) % Gs;
    // the pair of the previous fill, finished one iteration later
    int pc0[4] = {0, 0, 0, 0}, pc1[4] = {0, 0, 0, 0};
    const uint8_t* p_rec = nullptr;
    int p_tl0 = 0, p_gg0 = 0, p_tl1 = 0, p_gg1 = 0, p_n = 0, p_slot = -1;
    uint32_t fslot = kbase % (uint32_t)NS, fpar = (kbase / (uint32_t)NS) & 1u;  // slot and parity of the next fill
    const uint8_t* rec_lane = R.base + (uint32_t)(2 * warp) * UB;
    for (int k = 0; k < nslots; k++) {
        const int slot = (int)fslot;
        const int m = min(SU, n - k * SU);
        bool got = mbar_try_wait(R.full + slot, fpar);
        if (!__all_sync(0xffffffffu, got)) {  // not there yet: the bounded wait
            got = !*R.abort_flag && mbar_wait(R.full + slot, fpar);
            if (!__all_sync(0xffffffffu, got)) {
                if (!*R.abort_flag) { if (R.status) atomicExch(R.status, 1001); *R.abort_flag = 1; }
                ok = false;
                break;
            }
        }
        const uint8_t* rec0 = rec_lane + (uint32_t)slot * R.slot_bytes;
        int tl1 = tl0, gg1 = gg0 + 1;
        if (gg1 == Gs) { gg1 = 0; tl1++; }
        int c0[4], c1[4];
        if (m == 2 * SK_WARPS) {  // a full slot: straight-line
            unit_mma(rec0, digits_of(gg0), c0);
            unit_mma(rec0 + UB, digits_of(gg1), c1);
            if (k > 0) {  // the previous fill was a full one as well; runs while the MMAs above are in flight
                unit_finish(p_rec, p_tl0, p_gg0, pc0);
                unit_finish(p_rec + UB, p_tl1, p_gg1, pc1);
                release(p_slot);
            }
            p_n = 2;
        } else {  // the last, partial fill
            const int j = 2 * warp;
            const int nu = j + 1 < m ? 2 : (j < m ? 1 : 0);
            c0[0] = c0[1] = c0[2] = c0[3] = c1[0] = c1[1] = c1[2] = c1[3] = 0;
            if (nu > 0) unit_mma(rec0, digits_of(gg0), c0);
            if (nu > 1) unit_mma(rec0 + UB, digits_of(gg1), c1);
            if (k > 0) {
                unit_finish(p_rec, p_tl0, p_gg0, pc0);
                unit_finish(p_rec + UB, p_tl1, p_gg1, pc1);
                release(p_slot);
            }
            p_n = nu;
        }
        p_rec = rec0; p_slot = slot;
        p_tl0 = tl0; p_gg0 = gg0; p_tl1 = tl1; p_gg1 = gg1;
#pragma unroll
        for (int i = 0; i < 4; i++) { pc0[i] = c0[i]; pc1[i] = c1[i]; }
        gg0 += SU;
        while (gg0 >= Gs) { gg0 -= Gs; tl0++; }
        if (++fslot == (uint32_t)NS) { fslot = 0; fpar ^= 1u; }
    }
    if (ok && p_slot >= 0) {
        if (p_n > 0) unit_finish(p_rec, p_tl0, p_gg0, pc0);
        if (p_n > 1) unit_finish(p_rec + UB, p_tl1, p_gg1, pc1);
        release(p_slot);
    }
    kbase += (uint32_t)nslots;
    flush();
    // epilogue operands of this warp's first tile, fetched while the other warps finish
    const int e_row = (tau_first + warp) * 16 + (lane & 15);
    const bool e_pre = NSEG == 1 && warp < nt && lane < 16 && e_row < J.rows && J.epi == EPI_RESID;
    int e_idx[3] = {0, 0, 0};
    float e_out = 0.f;
    if (e_pre) {
#pragma unroll
        for (int s = 0; s < 3; s++)
            if (s < J.nscatter) e_idx[s] = __ldg(J.sidx[s] + e_row);
        e_out = __ldcg(J.out + e_row);
    }
    if (stamp && threadIdx.x == 0) { stamp[2] = clock64(); stamp[9] = (unsigned long long)nslots; }
    consumer_sync();
    if (*R.abort_flag) return false;

    for (int tl = warp; tl < nt; tl += SK_WARPS) {
        const int tau = tau_first + tl;
        float v = 0.f;
        if (lane < ROWS)
            for (int w = 0; w < SK_WARPS; w++) v += partial[((size_t)tl * SK_WARPS + w) * ROWS + lane];
        const float y = v * oscale[lane >> 4 & (NSEG - 1)];
        const int row = tau * 16 + (lane & 15);
        if (NSEG == 2) {  // SwiGLU (src/models.rs:92-98)
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
                int idx[3] = {e_idx[0], e_idx[1], e_idx[2]};
                if (!pre) {
#pragma unroll
                    for (int s = 0; s < 3; s++)
                        if (s < J.nscatter) idx[s] = __ldg(J.sidx[s] + row);
                }
                const float xv = (pre ? e_out : __ldcg(J.out + row)) + y;
                J.out[row] = xv;
#pragma unroll
                for (int s = 0; s < 3; s++)
                    if (s < J.nscatter) J.sdst[s][idx[s]] = xv;
            }
        }
    }
    return true;
}

// ---- the other phases ------------------------------------------------------------------------------

__device__ __forceinline__ float tk_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __noinline__ void embed_phase(const EmbedParams& p) {
    const int pos = p.ctl->pos;
    int token = p.ctl->token;
    if (p.feed_prompt) token = pos == 0 ? 1 : p.prompt[pos - 1];  // src/inference.rs:29-35
    if (token < 0 || token >= p.vocab) token = 0;
    for (int i = blockIdx.x * SK_THREADS + threadIdx.x; i < p.dim; i += gridDim.x * SK_THREADS) {
        const float v = __ldg(p.table + (size_t)token * p.dim + i);
        p.x[i] = v;
        for (int s = 0; s < p.nscatter; s++) p.sdst[s][__ldg(p.sidx[s] + i)] = v;
    }
}

// RoPE + KV append + attention (src/models.rs:100-176, 228-256).  A CTA (16 consumer warps) takes
// (kv head, sequence split) items; short sequences are not split at all, so that the common case has
// no cross-CTA merge; otherwise the CTA that finishes the last split of a kv head merges the splits
// in split order.
constexpr int TK_ATT_WARPS = SK_WARPS;

__host__ __device__ constexpr size_t tk_att_bytes(int ag) {
    return ((size_t)ag * HS + (size_t)TK_ATT_WARPS * ag * HS + 2 * (size_t)TK_ATT_WARPS * ag + 4) * 4;
}

template <int AG>
__device__ __noinline__ void attn_phase(const AttnParams& p, uint8_t* scratch) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float* base = reinterpret_cast<float*>(scratch);
    float(*qs)[HS] = reinterpret_cast<float(*)[HS]>(base);
    float(*sm_acc)[AG][HS] = reinterpret_cast<float(*)[AG][HS]>(base + AG * HS);
    float(*sm_m)[AG] = reinterpret_cast<float(*)[AG]>(base + AG * HS + TK_ATT_WARPS * AG * HS);
    float(*sm_l)[AG] = reinterpret_cast<float(*)[AG]>(base + AG * HS + TK_ATT_WARPS * AG * HS + TK_ATT_WARPS * AG);
    volatile int* sm_last = reinterpret_cast<volatile int*>(base + AG * HS + TK_ATT_WARPS * AG * HS + 2 * TK_ATT_WARPS * AG);

    const int pos = p.pos_fixed >= 0 ? p.pos_fixed : p.ctl->pos;
    const int T = pos + 1;
    const int nkv = p.n_kv_local > 0 ? p.n_kv_local : p.n_kv_heads;
    // splits: about 256 positions each, no more than the CTAs can take in one round
    int nsplit = (T + 255) / 256;
    nsplit = min(nsplit, min(p.max_split, max(1, (int)gridDim.x / nkv)));
    const int chunk = (T + nsplit - 1) / nsplit;
    nsplit = (T + chunk - 1) / chunk;
    const int nitems = nkv * nsplit;
    const int KV = p.n_kv_heads * HS;
    const float inv_div = sqrtf((float)HS);

    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        const int kvh = item % nkv + p.kvh0, split = item / nkv;
        const int t0 = split * chunk, t1 = min(T, t0 + chunk);
        // rotate-half RoPE updated in place: the second half uses the already rotated first half (src/models.rs:106-116)
        for (int idx = tid; idx < AG * (HS / 2); idx += SK_THREADS) {
            const int g = idx / (HS / 2), i = idx % (HS / 2);
            const int h = kvh * AG + g;
            const float c = __ldg(p.rope_cos + (size_t)pos * (HS / 2) + i), s = __ldg(p.rope_sin + (size_t)pos * (HS / 2) + i);
            const float a = __ldcg(p.q + (size_t)h * HS + i), b = __ldcg(p.q + (size_t)h * HS + HS / 2 + i);
            const float na = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
            const float nb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(na, s));
            qs[g][i] = na;
            qs[g][HS / 2 + i] = nb;
        }
        if (split == nsplit - 1 && warp >= SK_WARPS - 6) {  // this CTA owns position `pos`: append k (rotated) and v
            const int u = tid - (SK_WARPS - 6) * 32;          // 0..191, taken from the warps the RoPE of q uses last
            if (u < HS / 2) {
                const int i = u;
                const float c = __ldg(p.rope_cos + (size_t)pos * (HS / 2) + i), s = __ldg(p.rope_sin + (size_t)pos * (HS / 2) + i);
                const float a = __ldcg(p.k + (size_t)kvh * HS + i), b = __ldcg(p.k + (size_t)kvh * HS + HS / 2 + i);
                const float na = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
                const float nb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(na, s));
                p.kc[(size_t)pos * KV + kvh * HS + i] = na;
                p.kc[(size_t)pos * KV + kvh * HS + HS / 2 + i] = nb;
            } else {
                const int i = u - HS / 2;  // 0..127
                p.vc[(size_t)pos * KV + kvh * HS + i] = __ldcg(p.v + (size_t)kvh * HS + i);
            }
        }
        consumer_sync();

        float4 qr[AG], acc[AG];
        float m[AG], l[AG];
#pragma unroll
        for (int g = 0; g < AG; g++) {
            qr[g] = reinterpret_cast<const float4*>(qs[g])[lane];
            m[g] = -INFINITY;
            l[g] = 0.f;
            acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        const float4* kc4 = reinterpret_cast<const float4*>(p.kc) + (size_t)kvh * (HS / 4) + lane;
        const float4* vc4 = reinterpret_cast<const float4*>(p.vc) + (size_t)kvh * (HS / 4) + lane;
        const size_t rs = (size_t)KV / 4;
        constexpr int U = AG >= 8 ? 2 : 4;
        for (int tb = t0 + warp * U; tb < t1; tb += TK_ATT_WARPS * U) {
            float4 kk[U], vv[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int tt = min(tb + u, t1 - 1);
                kk[u] = kc4[(size_t)tt * rs];
                vv[u] = vc4[(size_t)tt * rs];
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                if (tb + u < t1) {
#pragma unroll
                    for (int g = 0; g < AG; g++) {
                        float d = qr[g].x * kk[u].x + qr[g].y * kk[u].y + qr[g].z * kk[u].z + qr[g].w * kk[u].w;
                        d = tk_warp_sum(d);
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
        consumer_sync();

        // combine the warps in warp order: thread (j, i) owns element i of heads j, j + 4, ...
        const int i = tid & (HS - 1), j0 = tid >> 7;
        if (nsplit > 1) {
            for (int g = j0; g < AG; g += SK_THREADS / HS) {
                float mm = -INFINITY;
                for (int w = 0; w < TK_ATT_WARPS; w++) mm = fmaxf(mm, sm_m[w][g]);
                float ll = 0.f, aa = 0.f;
                for (int w = 0; w < TK_ATT_WARPS; w++) {
                    const float e = sm_m[w][g] == -INFINITY ? 0.f : expf(sm_m[w][g] - mm);
                    ll += sm_l[w][g] * e;
                    aa += sm_acc[w][g][i] * e;
                }
                float* dst = p.part + ((size_t)(kvh * AG + g) * p.max_split + split) * (HS + 2);
                dst[i] = aa;
                if (i == 0) { dst[HS] = mm; dst[HS + 1] = ll; }
            }
            __threadfence();
            consumer_sync();
            if (tid == 0) {
                const unsigned ticket = atomicAdd(p.counter + kvh, 1u);
                const int last = ticket == (unsigned)nsplit - 1u;
                if (last) p.counter[kvh] = 0;  // ready for the next use
                *sm_last = last;
            }
            consumer_sync();
            if (*sm_last) {
                __threadfence();
                for (int g = j0; g < AG; g += SK_THREADS / HS) {
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
                    p.out[p.oidx ? __ldg(p.oidx + o) : o] = aa / ll;
                }
            }
        } else {
            for (int g = j0; g < AG; g += SK_THREADS / HS) {
                float mm = -INFINITY;
                for (int w = 0; w < TK_ATT_WARPS; w++) mm = fmaxf(mm, sm_m[w][g]);
                float ll = 0.f, aa = 0.f;
                for (int w = 0; w < TK_ATT_WARPS; w++) {
                    const float e = sm_m[w][g] == -INFINITY ? 0.f : expf(sm_m[w][g] - mm);
                    ll += sm_l[w][g] * e;
                    aa += sm_acc[w][g][i] * e;
                }
                const int o = (kvh * AG + g) * HS + i;
                p.out[p.oidx ? __ldg(p.oidx + o) : o] = aa / ll;
            }
        }
        consumer_sync();  // the scratch is reused by the next item
    }
}

// final rmsnorm + dense f32 classifier (src/models.rs:288-297, src/model.rs:22-31)
__device__ __noinline__ void cls_phase(const ClsParams& p, float* xs, float* red) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r0 = (int)(((long long)blockIdx.x * p.rows) / gridDim.x);
    const int r1 = (int)(((long long)(blockIdx.x + 1) * p.rows) / gridDim.x);
    const int n4 = p.in / 4;
    const float4* x4 = reinterpret_cast<const float4*>(p.x);
    float s = 0.f;
    for (int i = threadIdx.x; i < n4; i += SK_THREADS) {
        const float4 v = __ldcg(x4 + i);
        s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    s = tk_warp_sum(s);
    if (lane == 0) red[warp] = s;
    consumer_sync();
    float sum = 0.f;
    for (int w = 0; w < SK_WARPS; w++) sum += red[w];
    const float ss = 1.0f / sqrtf(sum / (float)p.in + p.eps);
    const float4* w4 = reinterpret_cast<const float4*>(p.nw);
    float4* xs4 = reinterpret_cast<float4*>(xs);
    for (int i = threadIdx.x; i < n4; i += SK_THREADS) {
        float4 v = __ldcg(x4 + i);
        const float4 w = __ldg(w4 + i);
        v.x = (w.x * ss) * v.x; v.y = (w.y * ss) * v.y; v.z = (w.z * ss) * v.z; v.w = (w.w * ss) * v.w;
        xs4[i] = v;
    }
    consumer_sync();
    for (int row = r0 + warp * 2; row < r1; row += SK_WARPS * 2) {
        const bool two = row + 1 < r1;
        const float4* wa = reinterpret_cast<const float4*>(p.w + (size_t)row * p.in);
        const float4* wb = reinterpret_cast<const float4*>(p.w + (size_t)(two ? row + 1 : row) * p.in);
        float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll 4
        for (int i = lane; i < n4; i += 32) {
            const float4 x = xs4[i];
            float4 u, v;
            asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(u.x), "=f"(u.y), "=f"(u.z), "=f"(u.w) : "l"(wa + i));
            asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(wb + i));
            a0 = fmaf(u.x, x.x, a0); a1 = fmaf(u.y, x.y, a1); a0 = fmaf(u.z, x.z, a0); a1 = fmaf(u.w, x.w, a1);
            b0 = fmaf(v.x, x.x, b0); b1 = fmaf(v.y, x.y, b1); b0 = fmaf(v.z, x.z, b0); b1 = fmaf(v.w, x.w, b1);
        }
        const float ya = tk_warp_sum(a0 + a1), yb = tk_warp_sum(b0 + b1);
        if (lane == 0) {
            p.logits[row] = ya;
            if (two) p.logits[row + 1] = yb;
        }
    }
}

__device__ __forceinline__ unsigned tk_random_u32(unsigned long long& s) {  // src/util.rs:71-77
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    return (unsigned)((s * 0x2545F4914F6CDD1Dull) >> 32);
}

// Next-token selection by the consumer threads of one CTA: forced / prompt / argmax (last maximum
// wins, src/util.rs:39-46) / temperature sample (src/inference.rs:164-173, src/util.rs:102-113).
__device__ __noinline__ void select_phase(const SelectParams& p, float* scratch) {
    float* s_val = scratch;                                   // [SK_WARPS]
    int* s_idx = reinterpret_cast<int*>(scratch + SK_WARPS);   // [SK_WARPS]
    float* s_f = scratch + 2 * SK_WARPS;                       // [SK_WARPS + 2]
    int* s_choice = reinterpret_cast<int*>(scratch + 3 * SK_WARPS + 2);
    Ctl* ctl = p.ctl;
    const int pos = ctl->pos, force = ctl->force, n_prompt = ctl->n_prompt;
    const float T = ctl->temperature;
    unsigned long long rng = ctl->rng;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int V = p.vocab;
    consumer_sync();  // every thread has read the loop state before thread 0 rewrites it
    int chosen;
    if (force >= 0) {
        chosen = force;
    } else if (pos < n_prompt) {
        chosen = p.prompt[pos];  // src/inference.rs:154-156
    } else {
        float bv = -INFINITY;
        int bi = -1;
        for (int i = tid; i < V; i += SK_THREADS) {
            const float v = __ldcg(p.logits + i);
            if (bi < 0 || v >= bv) { bv = v; bi = i; }
        }
        auto merge = [&](float ov, int oi) {
            if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi > bi))) { bv = ov; bi = oi; }
        };
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            merge(ov, oi);
        }
        if (lane == 0) { s_val[warp] = bv; s_idx[warp] = bi; }
        consumer_sync();
        if (warp == 0) {
            bv = lane < SK_WARPS ? s_val[lane] : -INFINITY;
            bi = lane < SK_WARPS ? s_idx[lane] : -1;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                merge(ov, oi);
            }
            if (lane == 0) { s_val[0] = bv; s_idx[0] = bi; }
        }
        consumer_sync();
        const float maxv = s_val[0];
        chosen = s_idx[0];
        if (T != 0.0f) {
            // every thread owns a contiguous segment so that the running sum is taken in index order
            const float mx = maxv / T;
            const int seg = (V + SK_THREADS - 1) / SK_THREADS;
            const int b = min(V, tid * seg), e = min(V, b + seg);
            float loc = 0.f;
            for (int i = b; i < e; i++) loc += expf(__ldcg(p.logits + i) / T - mx);
            float incl = loc;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            if (lane == 31) s_f[warp] = incl;
            consumer_sync();
            if (warp == 0) {
                const float w = lane < SK_WARPS ? s_f[lane] : 0.f;
                float wi = w;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float v = __shfl_up_sync(0xffffffffu, wi, o);
                    if (lane >= o) wi += v;
                }
                if (lane < SK_WARPS) s_f[lane] = wi - w;  // exclusive prefix of the warp totals
                if (lane == 31) s_f[SK_WARPS] = wi;
            }
            if (tid == 0) *s_choice = V - 1;  // "in case of rounding errors" (src/util.rs:112)
            consumer_sync();
            const float total = s_f[SK_WARPS];
            const float r = (float)(tk_random_u32(rng) >> 8) / 16777216.0f;
            float cdf = (s_f[warp] + incl - loc) / total;
            for (int i = b; i < e; i++) {
                cdf += expf(__ldcg(p.logits + i) / T - mx) / total;
                if (r < cdf) { atomicMin(s_choice, i); break; }
            }
            consumer_sync();
            chosen = *s_choice;
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

// ---- the kernel ------------------------------------------------------------------------------------

template <int W>
__global__ void __launch_bounds__(SK_THREADS + 32, 1) token_kernel(const __grid_constant__ TokenParams tk) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(16) PhaseRec recs[TK_NREC];
    __shared__ __align__(8) uint64_t full[SK_MAX_SLOTS], empty[SK_MAX_SLOTS], rec_full[TK_NREC];
    __shared__ float red[4 * SK_WARPS + 8];
    __shared__ float oscale[2];
    __shared__ volatile int abort_flag;
    __shared__ volatile int consumer_phase;  // phases the consumer warps have finished
    __shared__ __align__(16) uint32_t zeros[8];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < tk.slots; i++) { mbar_init(full + i, 1); mbar_init(empty + i, SK_WARPS); }
        for (int i = 0; i < TK_NREC; i++) mbar_init(rec_full + i, 1);
        abort_flag = 0;
        consumer_phase = 0;
        for (int i = 0; i < 8; i++) zeros[i] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    Ring R;
    R.base = smem + tk.fixed_bytes;
    R.full = full; R.empty = empty;
    R.SU = tk.chunk; R.NS = tk.slots;
    R.slot_bytes = (uint32_t)tk.chunk * (256u * W + 80u);
    R.abort_flag = &abort_flag;
    R.status = tk.status;
    R.zeros = reinterpret_cast<const uint8_t*>(zeros);

    // ================= producer warp ================================================================
    if (warp == SK_WARPS) {
        uint32_t kfill = 0;
        for (int p = 0; p < tk.nphases; p++) {
            bool okp = true;
            if (p >= TK_NREC) {  // its record buffer is free once the consumers have finished phase p - TK_NREC
                uint32_t it = 0;
                while (consumer_phase < p - TK_NREC + 1) {
                    if (abort_flag || ++it > (1u << 24)) { okp = false; break; }
                    __nanosleep(64);
                }
            }
            okp = __all_sync(0xffffffffu, okp);
            if (!okp) {
                if (lane == 0 && !abort_flag) { if (tk.status) atomicExch(tk.status, 1003); abort_flag = 1; }
                break;
            }
            const uint4* src = reinterpret_cast<const uint4*>(tk.phases + p);
            uint4* dst = reinterpret_cast<uint4*>(&recs[p % TK_NREC]);
            for (int i = lane; i < (int)(sizeof(PhaseRec) / 16); i += 32) dst[i] = __ldg(src + i);
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(rec_full + p % TK_NREC)) : "memory");
            __syncwarp();
            const PhaseRec& rec = recs[p % TK_NREC];
            if (rec.type == PH_GEMV1 || rec.type == PH_GEMV2) {
                warm_operands(rec.u.sk, rec.type == PH_GEMV2 ? 2 : 1);
                int good = 1;
                if (lane == 0) good = produce_units<W>(rec.u.sk, rec.type == PH_GEMV2 ? 2 : 1, R, kfill) ? 1 : 0;
                good = __shfl_sync(0xffffffffu, good, 0);
                if (!good) break;
            }
        }
        return;
    }

    // ================= consumer warps ===============================================================
    uint32_t kbase = 0;
    unsigned bar_target = 0;
    bool ok = true;
    for (int p = 0; p < tk.nphases && ok; p++) {
        if (!mbar_wait(rec_full + p % TK_NREC, (uint32_t)(p / TK_NREC) & 1u)) {
            if (tk.status) atomicExch(tk.status, 1005);
            abort_flag = 1;
        }
        consumer_sync();
        if (abort_flag) { ok = false; break; }
        const PhaseRec& rec = recs[p % TK_NREC];
        unsigned long long* stamp = tk.trace ? tk.trace + ((size_t)blockIdx.x * tk.nphases + p) * 16 : nullptr;
        TK_STAMP(p, 0);
        TK_STAMP_NS(p, 4);
        switch (rec.type) {
            case PH_EMBED: embed_phase(rec.u.em); break;
            case PH_GEMV1: ok = gemv_phase<W, 1>(rec.u.sk, smem, R, red, oscale, kbase, stamp); break;
            case PH_GEMV2: ok = gemv_phase<W, 2>(rec.u.sk, smem, R, red, oscale, kbase, stamp); break;
            case PH_ATTN:
                switch (rec.u.at.ag) {
                    case 1: attn_phase<1>(rec.u.at, smem); break;
                    case 2: attn_phase<2>(rec.u.at, smem); break;
                    case 4: attn_phase<4>(rec.u.at, smem); break;
                    default: attn_phase<8>(rec.u.at, smem); break;
                }
                break;
            case PH_CLS: cls_phase(rec.u.cl, reinterpret_cast<float*>(smem), red); break;
            case PH_SELECT: if (blockIdx.x == 0) select_phase(rec.u.se, red); break;
            case PH_ADVANCE: if (blockIdx.x == 0 && threadIdx.x == 0) rec.u.se.ctl->pos = rec.u.se.ctl->pos + 1; break;
            default: break;
        }
        if (!ok) break;
        if (p + 1 < tk.nphases) {
            // grid barrier: this CTA's writes are published by thread 0's fence after the CTA barrier
            consumer_sync();
            TK_STAMP(p, 7);
            TK_STAMP_NS(p, 5);
            if (threadIdx.x == 0) {
                bar_target += gridDim.x;
                __threadfence();
                atomicAdd(tk.bar, 1u);
                uint32_t it = 0;
                while (ld_acquire_u32(tk.bar) < bar_target) {
                    if (++it > TK_BAR_LIMIT || ((it & 255u) == 0 && tk.status && *reinterpret_cast<volatile int*>(tk.status) != 0)) {
                        if (tk.status) atomicCAS(tk.status, 0, 1004);
                        abort_flag = 1;
                        break;
                    }
                }
                __threadfence();
            }
            consumer_sync();
            if (abort_flag) { ok = false; break; }
        }
        TK_STAMP(p, 3);
        TK_STAMP_NS(p, 6);
        if (threadIdx.x == 0) consumer_phase = p + 1;
    }
    if (!ok) {
        // copies may still be in flight into this CTA's shared memory: give them a bounded time to land
        for (int i = 0; i < tk.slots; i++) { mbar_wait(full + i, 0, 1u << 8); mbar_wait(full + i, 1, 1u << 8); }
    }
}

size_t token_attn_scratch_bytes(int ag) { return tk_att_bytes(ag); }

template <int W>
static cudaError_t launch_token_t(const TokenParams& tk, int grid, size_t smem, cudaStream_t st) {
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(SK_THREADS + 32);  // 16 consumer warps + the producer warp
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident together: the grid barrier relies on it
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    g_launches++;
    return cudaLaunchKernelEx(&cfg, token_kernel<W>, tk);
}

cudaError_t launch_token(const TokenParams& tk, int group_size, int grid, size_t smem, cudaStream_t st) {
    switch (group_size) {
        case 128: return launch_token_t<4>(tk, grid, smem, st);
        case 64: return launch_token_t<2>(tk, grid, smem, st);
        default: return launch_token_t<1>(tk, grid, smem, st);
    }
}

// Opt in to as much dynamic shared memory as the device offers beside the kernel's static part.
cudaError_t token_init(int max_optin) {
    cudaError_t e;
    cudaFuncAttributes fa;
#define L2_TK_ATTR(W)                                                                                     \
    if ((e = cudaFuncGetAttributes(&fa, token_kernel<W>)) != cudaSuccess) return e;                       \
    if ((e = cudaFuncSetAttribute(token_kernel<W>, cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                                  max_optin - (int)fa.sharedSizeBytes)) != cudaSuccess) return e;
    L2_TK_ATTR(4) L2_TK_ATTR(2) L2_TK_ATTR(1)
#undef L2_TK_ATTR
    return cudaSuccess;
}

}  // namespace l2
