// One token of the B=1 forward pass (src/models.rs:178-298, src/inference.rs:134-190) as ONE
// persistent kernel for sm_100a: one CTA per SM, every CTA walks the same list of phases
//
//   embed | per layer: wq/wk/wv GEMV | rope + KV append + attention | wo GEMV + residual |
//   w1/w3 GEMV + SwiGLU | w2 GEMV + residual | final rmsnorm + classifier | select
//
// Compared with one launch per phase this removes the launch gaps and lets the weights stream
// without a break: warp 16 of every CTA is a producer that walks the phase list ahead of the 16
// consumer warps and keeps a ring of shared-memory slots filled with the CTA's next unit records
// (large cp.async.bulk copies, one mbarrier per slot), across phase boundaries, while the consumers
// are still in the previous phase's epilogue or staging the next activation vector.
//
// There is no grid-wide barrier between phases.  Values that cross CTAs travel as (value, tag)
// pairs that the reader polls (see gemv_device.cuh); one grid barrier per token remains, between the
// classifier and the selection of the next token, which reads every logit.
//
// The kernel is bound by instruction issue and by the latency of each exchange, not by HBM: every
// phase's code runs once per layer, so it is kept small (one GEMV phase for all four projections,
// no unrolled polling loops) and each exchange is arranged so that everything that does not depend
// on the awaited values (norm weights, scatter positions, K/V rows) is already in flight.
//
// Waits are bounded everywhere (mbarriers, tag polls, the grid barrier, the producer's wait for a
// free slot or record buffer): a wait that gives up writes a status word, raises the CTA's abort
// flag, lets copies in flight land and leaves; the other CTAs run into their own limits or see the
// flag at their next wait and leave too.  The launch is cooperative, so all CTAs are resident together.
#include "gemv_device.cuh"
#include "kernels.cuh"

namespace l2 {

// The phase functions have one call site each: inlined, they share the kernel's register allocation and no
// registers are saved to local memory around a call (with most of the L1 given to shared memory that is a trip to the L2).
#ifndef L2_TK_PHASE_INLINE
#define L2_TK_PHASE_INLINE __forceinline__
#endif
constexpr int TK_BLOCK = SK_THREADS + 32;  // 16 consumer warps + the producer warp
constexpr int TK_NREC = 4;                    // phase records buffered in shared memory
static_assert(sizeof(PhaseRec) % 16 == 0, "phase records travel as bulk copies");
constexpr uint32_t TK_BAR_LIMIT = 1u << 22;   // polls of the grid barrier before giving up (about a second)

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#ifdef L2_TK_TRACE
#define TK_STAMP_NS(p, i) do { if (tk.trace && threadIdx.x == 0) tk.trace[((size_t)blockIdx.x * tk.nphases + (p)) * TK_TRACE_W + (i)] = global_ns(); } while (0)
#define TK_STAMP(p, i) do { if (tk.trace && threadIdx.x == 0) tk.trace[((size_t)blockIdx.x * tk.nphases + (p)) * TK_TRACE_W + (i)] = clock64(); } while (0)
#else
#define TK_STAMP_NS(p, i) do { } while (0)
#define TK_STAMP(p, i) do { } while (0)
#endif

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ float tk_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
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

// Everything about the weight ring that the phases need, as 32-bit shared-space addresses: the record
// is alive across the whole phase loop, and generic pointers would cost two registers each.
struct Ring {
    uint32_t base, full, empty, zeros;  // slot 0; full[] / empty[] barriers; 32 bytes of zeros
    uint32_t abort_flag;                // int: raised when a bounded wait gave up
    uint32_t slot_bytes;
    int SU, NS;
    int* status;
    int skip;  // debug: consume the slot fills without doing the arithmetic
};
__device__ __forceinline__ bool ring_aborted(const Ring& R) { return lds_volatile_i32(R.abort_flag) != 0; }
__device__ __forceinline__ void ring_abort(const Ring& R, int code) {
    if (R.status) atomicCAS(R.status, 0, code);
    sts_volatile_i32(R.abort_flag, 1);
}

// A result that other ranks need as well (tensor parallelism): stored into this rank's buffer and at the
// same offset into every peer's pool.  The consumers on every rank poll their own memory only.
__device__ __forceinline__ void store_tagged_all(const TokenParams& tk, bool bcast, void* base, size_t index, float v, uint32_t tag) {
    store_tagged(base, index, v, tag);
    if (bcast && tk.world > 1) {
        const size_t off = static_cast<char*>(base) - tk.pool[tk.rank];
        for (int r = 0; r < tk.world; r++)
            if (r != tk.rank) store_tagged_peer(tk.pool[r] + off, index, v, tag);
    }
}

__device__ __forceinline__ void prefetch_line_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Producer side of one GEMV phase (called by the whole producer warp, lane 0 issues): streams this
// CTA's unit records through the ring.  `kfill` counts slot fills since the start of the kernel.
// Nothing beyond the ring is requested ahead of time.  Asking the L2 for the next phase's weights
// (cp.async.bulk.prefetch.L2, issued one GEMV phase ahead) does make slot fills faster in isolation
// (32-42 against 25 bytes per clock and SM), but in the kernel it was measured to cost more than it
// gains, twice: the exchanges between phases are trips to the L2, and they slow down when HBM
// traffic is poured into the L2 in exactly the windows in which they happen.
template <int W>
__device__ __forceinline__ bool produce_units(const SkParams& P, int NSEG, const Ring& R, uint32_t& kfill, unsigned long long* pstamp = nullptr) {
    constexpr uint32_t UB = 256u * W + 80u;
    const uint32_t r_base = R.base, r_full = R.full, r_empty = R.empty;
    const int r_NS = R.NS, r_skip = R.skip;
    const int lane = threadIdx.x & 31;
    const CtaRange c = sk_cta_range(P);
    const SkJob& J = P.job[c.ji];
    const int G = J.G, n = c.nt * NSEG * G;
    constexpr int SU = 2 * SK_WARPS;
    const int nslots = (n + SU - 1) / SU;
    struct Cur { int tl, seg, g; };
    // visits the runs of records (contiguous in memory) that the next `count` units consist of
    auto walk = [&](Cur& cu, int count, auto&& visit) {
        while (count > 0) {
            const int run = NSEG == 1 ? count : min(count, G - cu.g);  // one matrix: tiles follow one another in memory
            const SkSeg& S = J.seg[NSEG == 1 ? 0 : cu.seg];
            const size_t mu = (size_t)(c.tau_first + cu.tl) * G + cu.g;
            visit(S.rec + mu * (UB / 4), (uint32_t)run * UB);
            count -= run;
            cu.g += run;
            while (cu.g >= G) { cu.g -= G; if (++cu.seg == NSEG) { cu.seg = 0; cu.tl++; } }
        }
    };
    Cur cf{0, 0, 0};
    unsigned long long waited = 0;
    if (pstamp && lane == 0) pstamp[10] = clock64();
    // kfill: slot of the next fill in the low half, its round (how often the ring has wrapped) in the high half
    uint32_t slot = kfill & 0xFFFFu, round = kfill >> 16;
#pragma unroll 1
    for (int k = 0; k < nslots; k++) {
        int good = 1;
        const unsigned long long w0 = pstamp ? clock64() : 0;
        if (lane == 0) {
            if (round > 0) {  // in short pieces: an abort raised by the consumers is seen within a millisecond
                bool free_now = false;
#pragma unroll 1
                for (uint32_t piece = 0; piece < SK_WAIT_LIMIT / 32u && !free_now && !ring_aborted(R); piece++)
                    free_now = mbar_wait_u32(r_empty + 8u * slot, (round - 1u) & 1u, 32u);
                if (!free_now) {
                    if (!ring_aborted(R)) ring_abort(R, 1002);
                    good = 0;
                }
            }
            if (ring_aborted(R)) good = 0;
        }
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) return false;
        const int left = min(SU, n - k * SU);
        if (pstamp && lane == 0) { waited += clock64() - w0; if (k == 0) pstamp[11] = clock64(); pstamp[12] = clock64(); pstamp[13] = waited; }
        if (r_skip & 2) {  // debug: no copies at all, the consumers multiply whatever the slot holds
            if (lane == 0) mbar_arrive_u32(r_full + 8u * slot);
        } else {
            if (lane == 0) mbar_expect_tx_u32(r_full + 8u * slot, (uint32_t)left * UB);
            uint32_t dst = r_base + slot * ((uint32_t)SU * UB);
            walk(cf, left, [&](const uint32_t* src, uint32_t bytes) {
                if (lane == 0) bulk_g2s_u32(dst, src, bytes, r_full + 8u * slot);
                dst += bytes;
            });
        }
        if (++slot == (uint32_t)r_NS) { slot = 0; round++; }
    }
    kfill = slot | (round << 16);
    return true;
}


// Producer warp, ahead of the consumers: asks the L2 for the small operands of a GEMV phase that do
// not depend on the previous phase (norm weights, spread over the CTAs; the scatter indices and the
// residual rows of this CTA), so that the consumers' dependent loads do not go to HBM.
__device__ __forceinline__ void warm_operands(const SkParams& P, int NSEG) {
    const int lane = threadIdx.x & 31;
    const CtaRange c = sk_cta_range(P);
    const SkJob& J = P.job[c.ji];
    const int lines = J.in / 32;  // 128-byte lines of a norm weight vector
    for (int s = 0; s < NSEG; s++)
        if (J.seg[s].nw)
            for (int i = blockIdx.x + lane * gridDim.x; i < lines; i += 32 * gridDim.x) prefetch_line_l2(J.seg[s].nw + (size_t)i * 32);

}

// Consumer side of one GEMV phase: stage the digits, multiply, reduce, epilogue.  Returns false
// when a wait gave up.  `kbase` is the number of slot fills consumed before this phase.  nseg = 2
// pairs w1 with w3 (SwiGLU).  One copy of this code serves every GEMV phase of the token (the kernel
// runs each phase's code once per layer, so what is not shared is fetched from the L2 every time:
// the instruction cache of an SM holds far less than an unrolled copy per phase type would need).
// Shared memory in front of the weight ring that a GEMV phase needs (host side of the carve-up in gemv_phase).
size_t token_gemv_smem(int in, int G, int nseg, int ptiles, bool natural, bool gather) {
    size_t b = (size_t)4 * ((size_t)nseg * in + 16);       // digit planes
    b += (size_t)nseg * G * 16;                            // group records
    if (natural) b += (size_t)(gather ? 1 : nseg) * in * 4;  // the vector as plain floats: in each matrix's K order, or once in natural order
    b += (size_t)ptiles * SK_WARPS * 32 * 4;               // tile sums per warp
    return b;
}

template <int W>
__device__ L2_TK_PHASE_INLINE bool gemv_phase(const TokenParams& tk, const SkParams& P, const int nseg, uint8_t* smem, const Ring& R, float* red, float* oscale,
                                              uint32_t& kbase, unsigned long long* stamp, uint32_t tagbase, int phase) {
    constexpr int GS = 32 * W;
    constexpr uint32_t UB = 256u * W + 80u;
    constexpr int SU = 2 * SK_WARPS;  // units per slot fill: a pair per warp
    constexpr uint32_t SLOT_BYTES = (uint32_t)SU * UB;
    constexpr int PROWS = 32;         // tile sums per (tile, warp): 16 rows of up to two matrices
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const CtaRange cr = sk_cta_range(P);
    const SkJob& J = P.job[cr.ji];
    const int G = J.G, Gs = nseg * G, nt = cr.nt, tau_first = cr.tau_first;
    const int n = nt * Gs;
    const int nslots = (n + SU - 1) / SU;
    // the ring's constants as plain values: the record itself may live in local memory, and a load from it inside the
    // main loop would cost a trip to the L2 whenever the small L1 has dropped the line
    const uint32_t r_base = R.base, r_full = R.full, r_empty = R.empty, r_zeros = R.zeros, r_abort = R.abort_flag;
    const int NS = R.NS, skip = R.skip;
    auto aborted = [&]() { return lds_volatile_i32(r_abort) != 0; };

    const int pstride = nseg * J.in + 16;
    uint8_t* digits = smem;                                              // [4][nseg * in + 16]
    uint4* sp = reinterpret_cast<uint4*>(smem + (size_t)4 * pstride);    // [nseg * G] group records
    const bool natural = J.seg[0].perm != nullptr;                       // the input arrives in natural order and is gathered into the K order
    float* xs = reinterpret_cast<float*>(sp + Gs);                       // [nseg][in] the vector in each matrix's K order as plain floats (only then)
    float* partial = xs + (natural ? (J.gather ? 1 : nseg) * J.in : 0);  // [nt][SK_WARPS][PROWS]

    for (int i = threadIdx.x; i < nt * SK_WARPS * PROWS; i += SK_THREADS) partial[i] = 0.f;
    bool stage_failed = false;  // a poll for a tagged input gave up
    if (stamp && threadIdx.x == 0) stamp[16] = clock64();
    if (n > 0) {
        float sq;
        if (natural)  // w1 and w3 read the same x, each through its own g_index
            sq = stage_natural<W>(J.seg, nseg, J.in, G, digits, pstride, sp, xs, tagbase | (uint32_t)J.in_phase[0], &stage_failed, J.gather != 0, stamp);
        else          // the producer's row order is this matrix's K order (w2 after w1/w3)
            sq = stage_direct<W>(J.seg[0].x, J.in, digits, pstride, sp, tagbase | (uint32_t)J.in_phase[0], &stage_failed, stamp);
        if (stamp && threadIdx.x == 0) stamp[17] = clock64();
        sq = tk_warp_sum(sq);
        if (lane == 0) red[warp] = sq;
    }
    if (stage_failed) ring_abort(R, 1010);
    consumer_sync();  // digits and group records are in place; so are the zeroed tile sums
    if (warp == 0) {  // rmsnorm factor of the input (src/models.rs:58-60), read by the epilogue; the digit scaling is already in the sums
        float total = tk_warp_sum(lane < SK_WARPS ? red[lane] : 0.f);
        if (lane == 0) oscale[0] = J.seg[0].nw ? 1.0f / sqrtf(total / (float)J.in + P.eps) : 1.0f;
    }
    if (stamp && threadIdx.x == 0) stamp[1] = clock64();

    // The residual value of this warp's first tile was written phases ago: requested now, so that its trip
    // to the L2 overlaps the main loop.
    const int e_row = (tau_first + warp) * 16 + (lane & 15);
    const bool e_pre = nseg == 1 && warp < nt && lane < 16 && e_row < J.rows && J.epi == EPI_RESID;
    unsigned long long e_res = 0;
    if (e_pre) {
        asm volatile(L2_POLL_LD ".u64 %0, [%1];" : "=l"(e_res) : "l"(reinterpret_cast<const unsigned long long*>(J.out) + e_row) : "memory");
    }

    // ---- main loop.  In every slot fill this warp owns units 2*warp and 2*warp + 1; unit u of the CTA is group
    // u % Gs of tile u / Gs (the groups of w1 and of w3 of a tile follow one another).  The loop is bound by
    // instruction issue (16 warps run it on 4 schedulers), so it is straight-line code on 32-bit shared-space
    // addresses: all lanes run the scale / zero-point step (lanes t >= 2 hold the unused MMA columns and are ignored
    // when the sums are written), lanes r >= 4 read their digits from a block of zeros instead of skipping the load;
    // in the last, partial fill of a phase the units beyond the end are multiplied all the same (the slot holds older
    // records there) and only their sums are left out.  Row sums stay in registers while consecutive units belong to
    // the same (tile, matrix) and go to shared memory when that changes.
    const int r = lane >> 2, t = lane & 3;
    const uint32_t zshift = 4u * (uint32_t)r;
    const uint32_t w_lane = r_base + (uint32_t)(2 * warp) * UB + (uint32_t)lane * 16u;            // this lane's weights of unit 0 in slot 0
    const uint32_t m_lane = r_base + (uint32_t)(2 * warp) * UB + 256u * W + 4u * (uint32_t)r;     // its two scales (and, + 64 - 4r, the zero-point words)
    const uint32_t z_warp = r_base + (uint32_t)(2 * warp) * UB + 256u * W + 64u;
    const uint32_t dg_lane = r < 4 ? smem_u32(digits) + (uint32_t)(r * pstride + t * (8 * W)) : r_zeros;
    const uint32_t dstep = r < 4 ? (uint32_t)GS : 0u;
    const uint32_t sp_lane = smem_u32(sp) + 8u * (uint32_t)(t & 1);
    const uint32_t part_lane = smem_u32(partial) + 4u * (uint32_t)(warp * PROWS + r);
    float tot0 = 0.f, tot1 = 0.f;
    uint32_t cur_dst = 0;  // where the running row sums belong (0: nothing accumulated yet)
    auto flush = [&]() {   // lanes t = 0 hold digits 0,1 (already scaled by 2^16), lanes t = 1 digits 2,3
        const float a = tot0 + __shfl_xor_sync(0xffffffffu, tot0, 1), b = tot1 + __shfl_xor_sync(0xffffffffu, tot1, 1);
        if (t == 0) {
            asm volatile("st.shared.f32 [%0], %1;" ::"r"(cur_dst), "f"(a) : "memory");
            asm volatile("st.shared.f32 [%0], %1;" ::"r"(cur_dst + 32u), "f"(b) : "memory");
        }
    };
    constexpr uint32_t M = 0x0F0F0F0Fu;
    // position of this warp's first unit of the current fill: group f0 of the tile's Gs, tile tile0
    int f0 = 2 * warp, tile0 = 0;
    while (f0 >= Gs) { f0 -= Gs; tile0++; }
    int rem = n - 2 * warp;  // units of this warp's stride that are left, counted from its first of the current fill
    uint32_t fslot = kbase & 0xFFFFu, fpar = kbase >> 16;  // slot and parity of the next fill, carried from phase to phase
    bool ok = true;
#pragma unroll 1
    for (int k = 0; k < nslots; k++) {
        bool got = mbar_try_wait_u32(r_full + 8u * fslot, fpar);
        if (!__all_sync(0xffffffffu, got)) {  // not there yet: the bounded wait
            got = !aborted() && mbar_wait_u32(r_full + 8u * fslot, fpar);
            if (!__all_sync(0xffffffffu, got)) {
                if (!aborted()) ring_abort(R, 1001);
                ok = false;
                break;
            }
        }
        if (!(skip & 1)) {
            const uint32_t so = fslot * SLOT_BYTES;
            int f1 = f0 + 1, tile1 = tile0;
            if (f1 == Gs) { f1 = 0; tile1++; }
            // operands of both units: weights (two 16-row halves), digits, scales, zero points, group record
            uint32_t a0[W], b0[W], a1[W], b1[W], d0[2 * W], d1[2 * W];
            const uint32_t dg0 = dg_lane + (uint32_t)f0 * dstep, dg1 = dg_lane + (uint32_t)f1 * dstep;
            if constexpr (W == 4) {
                const uint4 x0 = lds128(w_lane + so), y0 = lds128(w_lane + so + 512), x1 = lds128(w_lane + so + UB), y1 = lds128(w_lane + so + UB + 512);
                const uint4 p0 = lds128(dg0), q0 = lds128(dg0 + 16), p1 = lds128(dg1), q1 = lds128(dg1 + 16);
                a0[0] = x0.x; a0[1] = x0.y; a0[2] = x0.z; a0[3] = x0.w; b0[0] = y0.x; b0[1] = y0.y; b0[2] = y0.z; b0[3] = y0.w;
                a1[0] = x1.x; a1[1] = x1.y; a1[2] = x1.z; a1[3] = x1.w; b1[0] = y1.x; b1[1] = y1.y; b1[2] = y1.z; b1[3] = y1.w;
                d0[0] = p0.x; d0[1] = p0.y; d0[2] = p0.z; d0[3] = p0.w; d0[4] = q0.x; d0[5] = q0.y; d0[6] = q0.z; d0[7] = q0.w;
                d1[0] = p1.x; d1[1] = p1.y; d1[2] = p1.z; d1[3] = p1.w; d1[4] = q1.x; d1[5] = q1.y; d1[6] = q1.z; d1[7] = q1.w;
            } else if constexpr (W == 2) {
                const uint32_t wl = w_lane - (uint32_t)lane * 8u;  // 8 bytes per lane and half
                const uint2 x0 = lds64(wl + so), y0 = lds64(wl + so + 256), x1 = lds64(wl + so + UB), y1 = lds64(wl + so + UB + 256);
                const uint4 p0 = lds128(dg0), p1 = lds128(dg1);
                a0[0] = x0.x; a0[1] = x0.y; b0[0] = y0.x; b0[1] = y0.y; a1[0] = x1.x; a1[1] = x1.y; b1[0] = y1.x; b1[1] = y1.y;
                d0[0] = p0.x; d0[1] = p0.y; d0[2] = p0.z; d0[3] = p0.w; d1[0] = p1.x; d1[1] = p1.y; d1[2] = p1.z; d1[3] = p1.w;
            } else {
                const uint32_t wl = w_lane - (uint32_t)lane * 12u;  // 4 bytes per lane and half
                a0[0] = lds32(wl + so); b0[0] = lds32(wl + so + 128); a1[0] = lds32(wl + so + UB); b1[0] = lds32(wl + so + UB + 128);
                const uint2 p0 = lds64(dg0), p1 = lds64(dg1);
                d0[0] = p0.x; d0[1] = p0.y; d1[0] = p1.x; d1[1] = p1.y;
            }
            const uint32_t s00 = lds32(m_lane + so), s01 = lds32(m_lane + so + 32), s10 = lds32(m_lane + so + UB), s11 = lds32(m_lane + so + UB + 32);
            const uint2 zz0 = lds64(z_warp + so), zz1 = lds64(z_warp + so + UB);
            const uint2 g0 = lds64(sp_lane + 16u * (uint32_t)f0), g1 = lds64(sp_lane + 16u * (uint32_t)f1);  // {digit sums of this lane's columns, their factor}
            // The MMAs of the pair are independent instructions issued back to back (even and odd K steps of a unit have
            // their own accumulators): an integer mma.sync that depends on the previous one of its warp occupies the
            // tensor pipe about four times as long as one that follows an independent one.
            int c0[4], c1[4];
            if constexpr (W == 1) {
                mma_u8s8_first(c0, a0[0] & M, b0[0] & M, (a0[0] >> 4) & M, (b0[0] >> 4) & M, d0[0], d0[1]);
                mma_u8s8_first(c1, a1[0] & M, b1[0] & M, (a1[0] >> 4) & M, (b1[0] >> 4) & M, d1[0], d1[1]);
            } else {
                int e0[4], e1[4];
                mma_u8s8_first(c0, a0[0] & M, b0[0] & M, (a0[0] >> 4) & M, (b0[0] >> 4) & M, d0[0], d0[1]);
                mma_u8s8_first(e0, a0[1] & M, b0[1] & M, (a0[1] >> 4) & M, (b0[1] >> 4) & M, d0[2], d0[3]);
                mma_u8s8_first(c1, a1[0] & M, b1[0] & M, (a1[0] >> 4) & M, (b1[0] >> 4) & M, d1[0], d1[1]);
                mma_u8s8_first(e1, a1[1] & M, b1[1] & M, (a1[1] >> 4) & M, (b1[1] >> 4) & M, d1[2], d1[3]);
#pragma unroll
                for (int i = 2; i < W; i += 2) {
                    mma_u8s8(c0, a0[i] & M, b0[i] & M, (a0[i] >> 4) & M, (b0[i] >> 4) & M, d0[2 * i], d0[2 * i + 1]);
                    mma_u8s8(e0, a0[i + 1] & M, b0[i + 1] & M, (a0[i + 1] >> 4) & M, (b0[i + 1] >> 4) & M, d0[2 * i + 2], d0[2 * i + 3]);
                    mma_u8s8(c1, a1[i] & M, b1[i] & M, (a1[i] >> 4) & M, (b1[i] >> 4) & M, d1[2 * i], d1[2 * i + 1]);
                    mma_u8s8(e1, a1[i + 1] & M, b1[i + 1] & M, (a1[i + 1] >> 4) & M, (b1[i + 1] >> 4) & M, d1[2 * i + 2], d1[2 * i + 3]);
                }
#pragma unroll
                for (int j = 0; j < 4; j++) { c0[j] += e0[j]; c1[j] += e1[j]; }
            }
            // scale, zero point and digit sums of the finished units (exact integers up to the final FMA)
            if (rem > 0) {
                const uint32_t dst = part_lane + (uint32_t)tile0 * (SK_WARPS * PROWS * 4u) + (f0 >= G ? 64u : 0u);
                if (dst != cur_dst) {  // warp-uniform
                    if (cur_dst) flush();
                    cur_dst = dst;
                    tot0 = tot1 = 0.f;
                }
                const int za = (int)((zz0.x >> zshift) & 15u) + 1, zb = (int)((zz0.y >> zshift) & 15u) + 1;  // src/gptq.rs:148
                const float pf = __uint_as_float(g0.y);  // a power of two: the products below are exact scalings
                tot0 = fmaf(__uint_as_float(s00) * pf, (float)(c0[0] * 256 + c0[1] - za * (int)g0.x), tot0);
                tot1 = fmaf(__uint_as_float(s01) * pf, (float)(c0[2] * 256 + c0[3] - zb * (int)g0.x), tot1);
            }
            if (rem > 1) {
                const uint32_t dst = part_lane + (uint32_t)tile1 * (SK_WARPS * PROWS * 4u) + (f1 >= G ? 64u : 0u);
                if (dst != cur_dst) {
                    if (cur_dst) flush();
                    cur_dst = dst;
                    tot0 = tot1 = 0.f;
                }
                const int za = (int)((zz1.x >> zshift) & 15u) + 1, zb = (int)((zz1.y >> zshift) & 15u) + 1;
                const float pf = __uint_as_float(g1.y);
                tot0 = fmaf(__uint_as_float(s10) * pf, (float)(c1[0] * 256 + c1[1] - za * (int)g1.x), tot0);
                tot1 = fmaf(__uint_as_float(s11) * pf, (float)(c1[2] * 256 + c1[3] - zb * (int)g1.x), tot1);
            }
        }
        __syncwarp();  // every lane has read the slot
        if (lane == 0) mbar_arrive_u32(r_empty + 8u * fslot);
        rem -= SU;
        f0 += SU;
        while (f0 >= Gs) { f0 -= Gs; tile0++; }
        if (++fslot == (uint32_t)NS) { fslot = 0; fpar ^= 1u; }
    }
    kbase = fslot | (fpar << 16);
    if (cur_dst) flush();
    if (stamp && threadIdx.x == 0) { stamp[2] = clock64(); stamp[9] = (unsigned long long)nslots; }
    consumer_sync();
    if (stamp && threadIdx.x == 0) stamp[18] = clock64();
    if (!ok || aborted()) return false;

    const float rs = oscale[0];
    // Results leave as (value, tag) pairs: whoever needs them polls for the tag of this phase.
    const uint32_t out_tag = tagbase | (uint32_t)phase;
    bool fine = true;
#pragma unroll 1
    for (int tl = warp; tl < nt; tl += SK_WARPS) {
        float v = 0.f;
        for (int w = 0; w < SK_WARPS; w++) v += partial[(tl * SK_WARPS + w) * PROWS + lane];
        float y = v * rs;
        if (stamp && threadIdx.x == 0) stamp[19] = clock64() + (y == 1.2345f ? 1 : 0);
        const int row = (tau_first + tl) * 16 + (lane & 15);
        if (nseg == 2) {  // SwiGLU (src/models.rs:92-98)
            const float y3 = __shfl_down_sync(0xffffffffu, y, 16);
            y = y * (1.0f / (1.0f + expf(-y))) * y3;
        }
        if (lane >= 16 || row >= J.rows) continue;
        if (nseg == 1 && J.epi == EPI_RESID) {  // residual add (src/models.rs:47-51)
            const bool pre = e_pre && tl == warp;
            float res = __uint_as_float((uint32_t)e_res);
            if (!pre || (uint32_t)(e_res >> 32) != (tagbase | (uint32_t)J.resid_phase))  // not the early copy: poll
                fine = load_tagged(J.out, row, tagbase | (uint32_t)J.resid_phase, res) && fine;
            y += res;
        }
        store_tagged_all(tk, J.bcast, J.out, row, y, out_tag);  // a tile is one 128-byte line: one writer per line
    }
    if (stamp && threadIdx.x == 0) stamp[20] = clock64();
    if (!fine) ring_abort(R, 1008);
    return true;
}

// ---- the other phases ------------------------------------------------------------------------------

__device__ __forceinline__ void embed_phase(const EmbedParams& p, uint32_t out_tag) {
    const int pos = p.ctl->pos;
    int token = p.ctl->token;
    if (p.feed_prompt) token = pos == 0 ? 1 : p.prompt[pos - 1];  // src/inference.rs:29-35
    if (token < 0 || token >= p.vocab) token = 0;
    for (int i = blockIdx.x * SK_THREADS + threadIdx.x; i < p.dim; i += gridDim.x * SK_THREADS) {
        const float v = __ldg(p.table + (size_t)token * p.dim + i);
        store_tagged(p.x, i, v, out_tag);
    }
}

// RoPE + KV append + attention (src/models.rs:100-176, 228-256).  A CTA (16 consumer warps) takes one
// (kv head, sequence split) item; the sequence is split over as many CTAs as there are (so that a CTA
// reads its K/V rows in one or two rounds of loads, all requested before q has arrived), and the partial
// results (unnormalised sums with their maximum and denominator) travel as tagged values to the CTA
// that merges the head's splits in split order.  A short sequence is not split: no second exchange.
constexpr int TK_ATT_WARPS = SK_WARPS;

__host__ __device__ constexpr size_t tk_att_bytes(int ag) {
    const size_t work = ((size_t)ag * HS + (size_t)TK_ATT_WARPS * ag * HS + 2 * (size_t)TK_ATT_WARPS * ag + 4 + 2 * HS + ag) * 4;
    const size_t merge = (size_t)32 * (HS + 2) * 4;  // up to 32 splits of one head
    return work > merge ? work : merge;
}

struct AttSplit { int nsplit, chunk; };
// How the T positions of a token are cut: rows_min positions per split at least, no more splits than the
// CTAs can take in one round (or than the partial buffer holds).
__device__ __forceinline__ AttSplit att_split(const AttnParams& p, int T, int nkv) {
    AttSplit a;
    int ns = T / max(1, p.split_min);
    ns = max(1, min(ns, min(p.max_split, max(1, (int)gridDim.x / nkv))));
    a.chunk = (T + ns - 1) / ns;
    a.nsplit = (T + a.chunk - 1) / a.chunk;
    return a;
}

// Producer warp, ahead of the consumers: brings the K/V rows this CTA will read in an attention phase
// (the same item split as attn_phase) and the output positions of its heads into the L2.  These are
// real loads, not prefetch hints: hints were found to leave the rows in HBM, and the attention phase
// has nothing to hide that latency behind.  The values are folded into a word that is stored only
// if it has a value it cannot have.
__device__ __noinline__ void warm_attention(const AttnParams& p, int pos_now, int* sink) {
    const int lane = threadIdx.x & 31;
    const int pos = p.pos_fixed >= 0 ? p.pos_fixed : pos_now;
    const int T = pos + 1;
    const int nkv = p.n_kv_local > 0 ? p.n_kv_local : p.n_kv_heads;
    const AttSplit sp = att_split(p, T, nkv);
    const int KV = p.n_kv_heads * HS;
    float fold = 0.f;
#pragma unroll 1
    for (int item = blockIdx.x; item < nkv * sp.nsplit; item += gridDim.x) {
        const int kvh = item % nkv + p.kvh0, split = item / nkv;
        const int t0 = split * sp.chunk, t1 = min(pos, t0 + sp.chunk);  // row `pos` is written by the phase itself
        const float4* kc4 = reinterpret_cast<const float4*>(p.kc) + (size_t)kvh * (HS / 4) + lane;
        const float4* vc4 = reinterpret_cast<const float4*>(p.vc) + (size_t)kvh * (HS / 4) + lane;
        const size_t rs = (size_t)KV / 4;
#pragma unroll 1
        for (int tb = t0; tb < t1; tb += 8) {  // only one word of every 512-byte row is needed to bring the row's lines in
            float a[8], b[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int tt = min(tb + u, t1 - 1);
                a[u] = __ldcg(reinterpret_cast<const float*>(kc4 + (size_t)tt * rs));
                b[u] = __ldcg(reinterpret_cast<const float*>(vc4 + (size_t)tt * rs));
            }
#pragma unroll
            for (int u = 0; u < 8; u++) fold += a[u] + b[u];
        }
    }
    if (fold == 1.2345678e38f && sink) *sink = 1;  // never true in practice; keeps the loads alive
}

// Three tagged words that become valid together (an element of a partial sum with the split's maximum
// and denominator): one trip to the L2 once they are there.
__device__ __forceinline__ bool load_tagged3(const unsigned long long* pa, const unsigned long long* pm, const unsigned long long* pl, uint32_t tag,
                                             float& a, float& m, float& l) {
#pragma unroll 1
    for (uint32_t it = 0; it < TAG_POLL_LIMIT; it++) {
        unsigned long long wa, wm, wl;
        asm volatile(L2_POLL_LD ".u64 %0, [%1];" : "=l"(wa) : "l"(pa) : "memory");
        asm volatile(L2_POLL_LD ".u64 %0, [%1];" : "=l"(wm) : "l"(pm) : "memory");
        asm volatile(L2_POLL_LD ".u64 %0, [%1];" : "=l"(wl) : "l"(pl) : "memory");
        if ((uint32_t)(wa >> 32) == tag && (uint32_t)(wm >> 32) == tag && (uint32_t)(wl >> 32) == tag) {
            a = __uint_as_float((uint32_t)wa); m = __uint_as_float((uint32_t)wm); l = __uint_as_float((uint32_t)wl);
            return true;
        }
    }
    a = 0.f; m = 0.f; l = 1.f;
    return false;
}

template <int AG>
__device__ L2_TK_PHASE_INLINE bool attn_phase(const TokenParams& tk, const AttnParams& p, uint8_t* scratch, int pos, unsigned long long* stamp, uint32_t in_tag,
                                        uint32_t out_tag) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float* base = reinterpret_cast<float*>(scratch);
    float(*qs)[HS] = reinterpret_cast<float(*)[HS]>(base);
    float(*sm_acc)[AG][HS] = reinterpret_cast<float(*)[AG][HS]>(base + AG * HS);
    float(*sm_m)[AG] = reinterpret_cast<float(*)[AG]>(base + AG * HS + TK_ATT_WARPS * AG * HS);
    float(*sm_l)[AG] = reinterpret_cast<float(*)[AG]>(base + AG * HS + TK_ATT_WARPS * AG * HS + TK_ATT_WARPS * AG);
    float* new_k = base + AG * HS + TK_ATT_WARPS * AG * HS + 2 * TK_ATT_WARPS * AG + 4;  // the row of `pos`: k (rotated), then v
    float* new_v = new_k + HS;
    float* sm_mx = new_v + HS;  // [AG] maximum over the warps
    unsigned long long* part = reinterpret_cast<unsigned long long*>(p.part);  // [head][max_split][HS + 2] tagged

    if (p.pos_fixed >= 0) pos = p.pos_fixed;
    const int T = pos + 1;
    const int nkv = p.n_kv_local > 0 ? p.n_kv_local : p.n_kv_heads;
    const AttSplit sp = att_split(p, T, nkv);
    const int nsplit = sp.nsplit, chunk = sp.chunk;
    const int nitems = nkv * nsplit;
    const int KV = p.n_kv_heads * HS;
    const float rdiv = 1.0f / sqrtf((float)HS);  // the reference divides by sqrt(head_size) (src/models.rs:158); the product differs by at most one ulp
    bool fine = true;  // false when a poll for a tagged input gave up
    constexpr int U = AG >= 4 ? 2 : 4;
    // combine: thread (j0, i) owns element i of heads j0, j0 + 4, ...
    const int i = tid & (HS - 1), j0 = tid >> 7;

#pragma unroll 1
    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        const int kvh = item % nkv + p.kvh0, split = item / nkv;
        const int t0 = split * chunk, t1 = min(T, t0 + chunk);
        const int nwarps = min(TK_ATT_WARPS, (t1 - t0 + U - 1) / U);  // warps that have rows in the first round
        // Loads that do not depend on this token's projections are issued first, so that their latency
        // overlaps the loads of q/k/v and the RoPE below: the first round of K/V rows (except the row
        // of `pos` itself).
        const float4* kc4 = reinterpret_cast<const float4*>(p.kc) + (size_t)kvh * (HS / 4) + lane;
        const float4* vc4 = reinterpret_cast<const float4*>(p.vc) + (size_t)kvh * (HS / 4) + lane;
        const size_t rs = (size_t)KV / 4;
        float4 kk[U], vv[U];
        const int tb0 = t0 + warp * U;
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int tt = min(tb0 + u, t1 - 1);
            if (tt != pos && tb0 < t1) {
                kk[u] = kc4[(size_t)tt * rs];
                vv[u] = vc4[(size_t)tt * rs];
            } else {
                kk[u] = vv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        if (stamp && tid == 0) stamp[10] = clock64();
        // rotate-half RoPE updated in place: the second half uses the already rotated first half (src/models.rs:106-116)
#pragma unroll 1
        for (int idx = tid; idx < AG * (HS / 2); idx += SK_THREADS) {
            const int g = idx / (HS / 2), e = idx % (HS / 2);
            const int h = kvh * AG + g;
            const float c = __ldg(p.rope_cos + (size_t)pos * (HS / 2) + e), s = __ldg(p.rope_sin + (size_t)pos * (HS / 2) + e);
            float a, b;
            fine = load_tagged(p.q, (size_t)h * HS + e, in_tag, a) && fine;
            fine = load_tagged(p.q, (size_t)h * HS + HS / 2 + e, in_tag, b) && fine;
            const float na = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
            const float nb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(na, s));
            qs[g][e] = na;
            qs[g][HS / 2 + e] = nb;
        }
        if (split == nsplit - 1 && warp >= SK_WARPS - 6) {  // this CTA owns position `pos`: append k (rotated) and v
            const int u = tid - (SK_WARPS - 6) * 32;          // 0..191, taken from the warps the RoPE of q uses last
            if (u < HS / 2) {
                const int e = u;
                const float c = __ldg(p.rope_cos + (size_t)pos * (HS / 2) + e), s = __ldg(p.rope_sin + (size_t)pos * (HS / 2) + e);
                float a, b;
                fine = load_tagged(p.k, (size_t)kvh * HS + e, in_tag, a) && fine;
                fine = load_tagged(p.k, (size_t)kvh * HS + HS / 2 + e, in_tag, b) && fine;
                const float na = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
                const float nb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(na, s));
                p.kc[(size_t)pos * KV + kvh * HS + e] = na;
                p.kc[(size_t)pos * KV + kvh * HS + HS / 2 + e] = nb;
                new_k[e] = na;
                new_k[HS / 2 + e] = nb;
            } else {
                const int e = u - HS / 2;  // 0..127
                float vv0;
                fine = load_tagged(p.v, (size_t)kvh * HS + e, in_tag, vv0) && fine;
                p.vc[(size_t)pos * KV + kvh * HS + e] = vv0;
                new_v[e] = vv0;
            }
        }
        consumer_sync();
        if (stamp && tid == 0) stamp[11] = clock64();

        float4 qr[AG], acc[AG];
        float m[AG], l[AG];
#pragma unroll
        for (int g = 0; g < AG; g++) {
            qr[g] = reinterpret_cast<const float4*>(qs[g])[lane];
            m[g] = -INFINITY;
            l[g] = 0.f;
            acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        // the row this phase has just written comes from shared memory, not through the L2
        auto load_k = [&](int tt, float4& k) { k = tt == pos ? reinterpret_cast<const float4*>(new_k)[lane] : kc4[(size_t)tt * rs]; };
        auto load_v = [&](int tt, float4& v) { v = tt == pos ? reinterpret_cast<const float4*>(new_v)[lane] : vc4[(size_t)tt * rs]; };
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int tt = min(tb0 + u, t1 - 1);
            if (tt == pos && tb0 < t1) { load_k(tt, kk[u]); load_v(tt, vv[u]); }
        }
#pragma unroll 1
        for (int tb = tb0; tb < t1; tb += TK_ATT_WARPS * U) {
            const int tbn = tb + TK_ATT_WARPS * U;  // the next round's rows are requested as soon as a register is free
            // all scores of the round first (independent warp reductions), then the running softmax in row order
            float sc[U][AG];
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int g = 0; g < AG; g++)
                    sc[u][g] = qr[g].x * kk[u].x + qr[g].y * kk[u].y + qr[g].z * kk[u].z + qr[g].w * kk[u].w;
            if (tbn < t1) {
#pragma unroll
                for (int u = 0; u < U; u++) load_k(min(tbn + u, t1 - 1), kk[u]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int u = 0; u < U; u++)
#pragma unroll
                    for (int g = 0; g < AG; g++) sc[u][g] += __shfl_xor_sync(0xffffffffu, sc[u][g], o);
            // one rescale per round: the exponentials of the round's rows are independent of one another
#pragma unroll
            for (int g = 0; g < AG; g++) {
                float mr = -INFINITY;
#pragma unroll
                for (int u = 0; u < U; u++) {
                    sc[u][g] *= rdiv;
                    if (tb + u < t1) mr = fmaxf(mr, sc[u][g]);
                }
                const float mn = fmaxf(m[g], mr);
                const float corr = __expf(m[g] - mn);  // exp(-inf) = 0 on the first round
                float pr[U];
#pragma unroll
                for (int u = 0; u < U; u++) pr[u] = tb + u < t1 ? __expf(sc[u][g] - mn) : 0.f;
                float ls = 0.f;
                float4 as = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < U; u++) {
                    ls += pr[u];
                    as.x += pr[u] * vv[u].x; as.y += pr[u] * vv[u].y; as.z += pr[u] * vv[u].z; as.w += pr[u] * vv[u].w;
                }
                l[g] = l[g] * corr + ls;
                acc[g].x = acc[g].x * corr + as.x; acc[g].y = acc[g].y * corr + as.y;
                acc[g].z = acc[g].z * corr + as.z; acc[g].w = acc[g].w * corr + as.w;
                m[g] = mn;
            }
            if (tbn < t1) {
#pragma unroll
                for (int u = 0; u < U; u++) load_v(min(tbn + u, t1 - 1), vv[u]);
            }
        }
        if (stamp && tid == 0) stamp[12] = clock64() + (acc[0].x == 1.2345f ? 1 : 0);
        if (warp < nwarps) {
#pragma unroll
            for (int g = 0; g < AG; g++) {
                reinterpret_cast<float4*>(sm_acc[warp][g])[lane] = acc[g];
                if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
            }
        }
        consumer_sync();

        // combine the warps that had rows, in warp order.  The factor exp(m_w - max) of a warp is the same
        // for all 128 elements: thread (w, g) computes it once and leaves it where the warp's maximum was.
        float fmax_g = -INFINITY;
        if (tid < TK_ATT_WARPS * AG) {
            const int g = tid % AG;
            float mm = -INFINITY;
            for (int w2 = 0; w2 < nwarps; w2++) mm = fmaxf(mm, sm_m[w2][g]);
            fmax_g = mm;
        }
        consumer_sync();
        if (tid < TK_ATT_WARPS * AG) {
            const int w = tid / AG, g = tid % AG;
            if (w < nwarps) {
                const float mw = sm_m[w][g];
                sm_m[w][g] = mw == -INFINITY ? 0.f : __expf(mw - fmax_g);
            }
            if (w == 0) sm_mx[g] = fmax_g;
        }
        consumer_sync();
#pragma unroll 1
        for (int g = j0; g < AG; g += 4) {
            float ll = 0.f, aa = 0.f;
            for (int w = 0; w < nwarps; w++) {
                const float e = sm_m[w][g];
                ll += sm_l[w][g] * e;
                aa += sm_acc[w][g][i] * e;
            }
            const int o = (kvh * AG + g) * HS + i;
            if (nsplit == 1) {
                store_tagged_all(tk, p.bcast, p.out, p.oidx ? __ldg(p.oidx + o) : o, aa / ll, out_tag);
            } else {  // this rank's own partial buffer: the merging CTA is on this GPU
                unsigned long long* dst = part + ((size_t)(kvh * AG + g) * p.max_split + split) * (HS + 2);
                store_tagged(dst, i, aa, out_tag);
                if (i == 0) { store_tagged(dst, HS, sm_mx[g], out_tag); store_tagged(dst, HS + 1, ll, out_tag); }
            }
        }
        consumer_sync();  // the scratch is reused by the next item
        if (stamp && tid == 0) stamp[13] = clock64();
    }
    if (nsplit > 1) {
        // ---- merge: CTA c takes the local heads c, c + grid, ...; the splits are combined in split order
        float* mg_a = base;                                  // [nsplit][HS]
        float* mg_m = base + 32 * HS;                        // [nsplit]
        float* mg_l = mg_m + 32;
        const int sgrp = tid >> 7;                           // thread (sgrp, i) fetches element i of splits sgrp, sgrp + 4, ...
#pragma unroll 1
        for (int hl = blockIdx.x; hl < nkv * AG; hl += gridDim.x) {
            const int h = p.kvh0 * AG + hl;
            const unsigned long long* src = part + (size_t)h * p.max_split * (HS + 2);
#pragma unroll 1
            for (int s = sgrp; s < nsplit; s += 4) {
                float a, mm, ll;
                fine = load_tagged3(src + (size_t)s * (HS + 2) + i, src + (size_t)s * (HS + 2) + HS, src + (size_t)s * (HS + 2) + HS + 1, out_tag, a, mm, ll) && fine;
                mg_a[s * HS + i] = a;
                if (i == 0) { mg_m[s] = mm; mg_l[s] = ll; }
            }
            consumer_sync();
            if (tid < HS) {
                float mm = -INFINITY;
                for (int s = 0; s < nsplit; s++) mm = fmaxf(mm, mg_m[s]);
                float ll = 0.f, aa = 0.f;
                for (int s = 0; s < nsplit; s++) {
                    const float e = __expf(mg_m[s] - mm);
                    ll += mg_l[s] * e;
                    aa += mg_a[s * HS + i] * e;
                }
                const int o = h * HS + i;
                store_tagged_all(tk, p.bcast, p.out, p.oidx ? __ldg(p.oidx + o) : o, aa / ll, out_tag);
            }
            consumer_sync();
        }
    }
    return fine;
}

// final rmsnorm + dense f32 classifier (src/models.rs:288-297, src/model.rs:22-31)
__device__ __forceinline__ bool cls_phase(const TokenParams& tk, const ClsParams& p, float* xs, float* red, uint32_t in_tag, uint32_t out_tag) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r0 = p.row0 + (int)(((long long)blockIdx.x * p.rows) / gridDim.x);  // this rank's rows, dealt out over its CTAs
    const int r1 = p.row0 + (int)(((long long)(blockIdx.x + 1) * p.rows) / gridDim.x);
    const int n4 = p.in / 4;
    // the residual stream arrives as tagged pairs; the raw values are parked in xs for the second pass
    float4* xs4 = reinterpret_cast<float4*>(xs);
    bool fine = true;
    float s = 0.f;
    for (int i = threadIdx.x; i < n4 / 2; i += SK_THREADS) {
        float4 v0, v1;
        fine = load_tagged8(p.x, (size_t)i * 8, in_tag, v0, v1) && fine;
        s += v0.x * v0.x + v0.y * v0.y + v0.z * v0.z + v0.w * v0.w + v1.x * v1.x + v1.y * v1.y + v1.z * v1.z + v1.w * v1.w;
        xs4[2 * i] = v0;
        xs4[2 * i + 1] = v1;
    }
    s = tk_warp_sum(s);
    if (lane == 0) red[warp] = s;
    consumer_sync();
    float sum = 0.f;
    for (int w = 0; w < SK_WARPS; w++) sum += red[w];
    const float ss = 1.0f / sqrtf(sum / (float)p.in + p.eps);
    const float4* w4 = reinterpret_cast<const float4*>(p.nw);
    for (int i = threadIdx.x; i < n4 / 2; i += SK_THREADS) {  // the elements this thread parked above
#pragma unroll
        for (int h = 0; h < 2; h++) {
            float4 v = xs4[2 * i + h];
            const float4 w = __ldg(w4 + 2 * i + h);
            v.x = (w.x * ss) * v.x; v.y = (w.y * ss) * v.y; v.z = (w.z * ss) * v.z; v.w = (w.w * ss) * v.w;
            xs4[2 * i + h] = v;
        }
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
            if (p.tagged) {  // vocabulary-parallel: every rank gets this rank's logits
                store_tagged_all(tk, true, p.tagged, (size_t)row, ya, out_tag);
                if (two) store_tagged_all(tk, true, p.tagged, (size_t)row + 1, yb, out_tag);
            } else {
                p.logits[row] = ya;
                if (two) p.logits[row + 1] = yb;
            }
        }
    }
    return fine;
}

__device__ __forceinline__ unsigned tk_random_u32(unsigned long long& s) {  // src/util.rs:71-77
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    return (unsigned)((s * 0x2545F4914F6CDD1Dull) >> 32);
}

// Next-token selection by the consumer threads of one CTA: forced / prompt / argmax (last maximum
// wins, src/util.rs:39-46) / temperature sample (src/inference.rs:164-173, src/util.rs:102-113).
__device__ __forceinline__ bool select_phase(const SelectParams& p, float* scratch, uint32_t tagbase) {
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
    bool fine = true;
    if (p.tagged) {  // logits from every rank: poll them, keep the plain array (the host reads it too)
        float* plain = const_cast<float*>(p.logits);
        const uint32_t tag = tagbase | (uint32_t)p.tagged_phase;
        for (int i = tid; i < V; i += SK_THREADS) {
            float v;
            fine = load_tagged(p.tagged, (size_t)i, tag, v) && fine;
            plain[i] = v;
        }
    }
    consumer_sync();  // every thread has read the loop state before thread 0 rewrites it; the plain logits are in place
    if (p.collect_only) return fine;
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
    return fine;
}

// ---- the kernel ------------------------------------------------------------------------------------

template <int W, int AG>
__global__ void __launch_bounds__(TK_BLOCK, 1) token_kernel(const __grid_constant__ TokenParams tk) {
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
    R.base = smem_u32(smem) + tk.fixed_bytes;
    R.full = smem_u32(full); R.empty = smem_u32(empty);
    R.SU = tk.chunk; R.NS = tk.slots;
    R.slot_bytes = (uint32_t)tk.chunk * (256u * W + 80u);
    R.abort_flag = smem_u32(const_cast<int*>(&abort_flag));
    R.status = tk.status;
    R.zeros = smem_u32(zeros);
    R.skip = tk.skip;

    // ================= producer warp ================================================================
    if (warp == SK_WARPS) {
        uint32_t kfill = 0;
        const int prod_pos = tk.ctl->pos;  // read before any CTA can have advanced it
        // Phase records travel into their shared-memory buffers as bulk copies that complete on
        // rec_full[]; they are requested two phases ahead so that the switch from one phase to the
        // next costs no trip to global memory.
        bool okp = true;
        auto request_record = [&](int q) {
            if (q >= TK_NREC) {  // the buffer is free once the consumers have finished phase q - TK_NREC
                uint32_t it = 0;
                while (consumer_phase < q - TK_NREC + 1) {
                    if (abort_flag || ++it > (1u << 24)) { okp = false; break; }
                    __nanosleep(64);
                }
            }
            okp = __all_sync(0xffffffffu, okp);
            if (!okp) {
                if (lane == 0 && !abort_flag) { if (tk.status) atomicExch(tk.status, 1003); abort_flag = 1; }
                return;
            }
            if (lane == 0) {
                mbar_expect_tx(rec_full + q % TK_NREC, (uint32_t)sizeof(PhaseRec));
                bulk_g2s(&recs[q % TK_NREC], tk.phases + q, (uint32_t)sizeof(PhaseRec), rec_full + q % TK_NREC);
            }
        };
        for (int q = 0; q < 2 && q < tk.nphases && okp; q++) request_record(q);
        for (int p = 0; p < tk.nphases && okp; p++) {
            if (p + 2 < tk.nphases) request_record(p + 2);
            if (!okp) break;
            bool got = mbar_wait(rec_full + p % TK_NREC, (uint32_t)(p / TK_NREC) & 1u);
            got = __all_sync(0xffffffffu, got);
            if (!got) {
                if (lane == 0 && !abort_flag) { if (tk.status) atomicExch(tk.status, 1006); abort_flag = 1; }
                break;
            }
            const PhaseRec& rec = recs[p % TK_NREC];
            if (rec.type == PH_GEMV1 || rec.type == PH_GEMV2) {
                // An attention phase that follows is warmed up first, a whole phase early: once this
                // phase's weights are on their way its loads would queue behind them.
                if (p + 1 < tk.nphases) {
                    bool got1 = mbar_wait(rec_full + (p + 1) % TK_NREC, (uint32_t)((p + 1) / TK_NREC) & 1u);
                    got1 = __all_sync(0xffffffffu, got1);
                    if (got1 && recs[(p + 1) % TK_NREC].type == PH_ATTN) warm_attention(recs[(p + 1) % TK_NREC].u.at, prod_pos, nullptr);
                }
                warm_operands(rec.u.sk, rec.type == PH_GEMV2 ? 2 : 1);
                #ifdef L2_TK_TRACE
                unsigned long long* pstamp = tk.trace ? tk.trace + ((size_t)blockIdx.x * tk.nphases + p) * TK_TRACE_W : nullptr;
#else
                unsigned long long* const pstamp = nullptr;
#endif
                if (!produce_units<W>(rec.u.sk, rec.type == PH_GEMV2 ? 2 : 1, R, kfill, pstamp)) break;
            }
        }
        return;
    }

    // ================= consumer warps ===============================================================
    const int tok_pos = tk.ctl->pos;  // read once: the attention phases would pay a trip to the L2 each
    // Tags of this launch: (launches so far + 1) in the upper bits, the writing phase in the lower ten.
    const uint32_t epoch = tk.bar[32];
    const uint32_t tagbase = (epoch % 4194303u + 1u) << 10;  // 22 bits, never zero (zero means "not tagged")
    uint32_t kbase = 0;
    unsigned bar_target = tk.bar[33] * gridDim.x;  // arrivals of the grid barriers of earlier launches (the counter is never reset)
    unsigned bars_done = 0;
    bool ok = true;
    // The record of a phase is waited for before the CTA barrier that ends the previous phase (the copy was requested two
    // phases earlier), so that a phase boundary costs one barrier, not two.
    auto await_record = [&](int q) {
        if (q < tk.nphases && !mbar_wait(rec_full + q % TK_NREC, (uint32_t)(q / TK_NREC) & 1u)) {
            if (tk.status) atomicExch(tk.status, 1005);
            abort_flag = 1;
        }
    };
    await_record(0);
    consumer_sync();
    for (int p = 0; p < tk.nphases && ok; p++) {
        if (abort_flag) { ok = false; break; }
        const PhaseRec& rec = recs[p % TK_NREC];
#ifdef L2_TK_TRACE
        unsigned long long* stamp = tk.trace ? tk.trace + ((size_t)blockIdx.x * tk.nphases + p) * TK_TRACE_W : nullptr;
#else
        unsigned long long* const stamp = nullptr;  // clock stamps are compiled in with -DL2_TK_TRACE only: they cost registers
#endif
        TK_STAMP(p, 0);
        TK_STAMP_NS(p, 4);
        const uint32_t out_tag = tagbase | (uint32_t)p;
        bool fine = true;
        switch (rec.type) {
            case PH_EMBED: embed_phase(rec.u.em, out_tag); break;
            case PH_GEMV1:
            case PH_GEMV2: ok = gemv_phase<W>(tk, rec.u.sk, rec.type == PH_GEMV2 ? 2 : 1, smem, R, red, oscale, kbase, stamp, tagbase, p); break;
            case PH_ATTN: fine = attn_phase<AG>(tk, rec.u.at, smem, tok_pos, stamp, tagbase | (uint32_t)rec.u.at.in_phase, out_tag); break;
            case PH_CLS: fine = cls_phase(tk, rec.u.cl, reinterpret_cast<float*>(smem), red, tagbase | (uint32_t)rec.u.cl.in_phase, out_tag); break;
            case PH_SELECT: if (blockIdx.x == 0) fine = select_phase(rec.u.se, red, tagbase); break;
            case PH_ADVANCE: if (blockIdx.x == 0 && threadIdx.x == 0) rec.u.se.ctl->pos = rec.u.se.ctl->pos + 1; break;
            default: break;
        }
        if (!fine) {  // a poll for a tagged input gave up
            if (tk.status) atomicCAS(tk.status, 0, 1009);
            abort_flag = 1;
        }
        if (!ok) break;
        TK_STAMP(p, 7);
        TK_STAMP_NS(p, 5);
        if (rec.barrier_after && p + 1 < tk.nphases) {
            // Grid barrier (only where the next phase cannot poll its inputs: the selection reads every
            // logit).  This CTA's writes are published by thread 0's fence after the CTA barrier.
            consumer_sync();
            bars_done++;
            if (threadIdx.x == 0) {
                bar_target += gridDim.x;
                __threadfence();
                atomicAdd(tk.bar, 1u);
                uint32_t it = 0;
                while ((int)(ld_acquire_u32(tk.bar) - bar_target) < 0) {
                    if (++it > TK_BAR_LIMIT || ((it & 255u) == 0 && tk.status && *reinterpret_cast<volatile int*>(tk.status) != 0)) {
                        if (tk.status) atomicCAS(tk.status, 0, 1004);
                        abort_flag = 1;
                        break;
                    }
                }
                __threadfence();
            }
        }
        await_record(p + 1);
        consumer_sync();  // the next phase reuses this phase's shared memory
        if (abort_flag) { ok = false; break; }
        TK_STAMP(p, 3);
        TK_STAMP_NS(p, 6);
        if (threadIdx.x == 0) consumer_phase = p + 1;
    }
    // the next launch uses new tags; every CTA has read the count long before CTA 0 gets here
    if (ok && blockIdx.x == 0 && threadIdx.x == 0) { tk.bar[32] = epoch + 1u; tk.bar[33] += bars_done; }
    if (!ok) {
        // copies may still be in flight into this CTA's shared memory: give them a bounded time to land
        for (int i = 0; i < tk.slots; i++) { mbar_wait(full + i, 0, 1u << 8); mbar_wait(full + i, 1, 1u << 8); }
    }
}

size_t token_attn_scratch_bytes(int ag) { return tk_att_bytes(ag); }

// Polls of a tagged input before the token kernel gives up (0 = the default, about a second).
cudaError_t token_set_poll_limit(unsigned polls) {
    const uint32_t v = polls ? polls : TAG_POLL_LIMIT_DEFAULT;
    return cudaMemcpyToSymbol(c_tag_poll_limit, &v, sizeof v);
}

template <int W, int AG>
static cudaError_t launch_token_t(const TokenParams& tk, int grid, size_t smem, cudaStream_t st) {
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(TK_BLOCK);  // 16 consumer warps + the producer warp
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident together: the grid barrier relies on it
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    g_launches++;
    return cudaLaunchKernelEx(&cfg, token_kernel<W, AG>, tk);
}

template <int W>
static cudaError_t launch_token_w(const TokenParams& tk, int ag, int grid, size_t smem, cudaStream_t st) {
    switch (ag) {
        case 1: return launch_token_t<W, 1>(tk, grid, smem, st);
#ifndef L2_TK_ONE
        case 2: return launch_token_t<W, 2>(tk, grid, smem, st);
        case 4: return launch_token_t<W, 4>(tk, grid, smem, st);
        case 8: return launch_token_t<W, 8>(tk, grid, smem, st);
#endif
        default: return cudaErrorInvalidValue;
    }
}

// One instantiation per (group size, query heads per kv head): everything is inlined into the kernel,
// which keeps its working set in registers (local memory is close to uncached here, almost all of the
// L1 being configured as shared memory).
cudaError_t launch_token(const TokenParams& tk, int group_size, int ag, int grid, size_t smem, cudaStream_t st) {
    switch (group_size) {
        case 128: return launch_token_w<4>(tk, ag, grid, smem, st);
#ifndef L2_TK_ONE
        case 64: return launch_token_w<2>(tk, ag, grid, smem, st);
        default: return launch_token_w<1>(tk, ag, grid, smem, st);
#else
        default: return cudaErrorInvalidValue;  // a development build that holds the 128-wide, one-head-per-kv-head kernel only
#endif
    }
}

// Opt in to as much dynamic shared memory as the device offers beside the kernel's static part.
cudaError_t token_init(int max_optin) {
    cudaError_t e;
    cudaFuncAttributes fa;
#define L2_TK_ATTR(W, AG)                                                                                 \
    if ((e = cudaFuncGetAttributes(&fa, token_kernel<W, AG>)) != cudaSuccess) return e;                   \
    if ((e = cudaFuncSetAttribute(token_kernel<W, AG>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                                  max_optin - (int)fa.sharedSizeBytes)) != cudaSuccess) return e;
#ifndef L2_TK_ONE
#define L2_TK_ATTR_W(W) L2_TK_ATTR(W, 1) L2_TK_ATTR(W, 2) L2_TK_ATTR(W, 4) L2_TK_ATTR(W, 8)
    L2_TK_ATTR_W(4) L2_TK_ATTR_W(2) L2_TK_ATTR_W(1)
#else
#define L2_TK_ATTR_W(W) L2_TK_ATTR(W, 1)
    L2_TK_ATTR_W(4)
#endif
#undef L2_TK_ATTR_W
#undef L2_TK_ATTR
    return cudaSuccess;
}

}  // namespace l2
