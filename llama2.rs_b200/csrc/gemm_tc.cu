// Batched QLinear::matvec<B> (src/gptq.rs:94-176) for B >= 2 as a dense contraction on the
// 5th-generation tensor cores: tcgen05.mma kind::i8 with accumulators in tensor memory.
//
//   out[m][o] = f[m] * sum_g scale[o][g] * sum_{k in g} (q[o][k] - z[o][g]) * X[m][k]
//
// X[m][k] is the activation of token m as a 23-bit signed integer (three balanced base-256 digits, see
// act_quant_kernel in prefill_kernels.cu), so every product and every sum inside a quantisation
// group is exact integer arithmetic; f[m] carries the block exponent and the rmsnorm factor.
//
// One CTA owns 128 output rows and a slice of the quantisation groups (grid.y slices).  Per group:
//   A  128 rows x GS weights, unpacked from nibbles to unsigned bytes in shared memory (3 bit
//      operations per 8 weights), K-major with the 128/64/32-byte swizzle the MMA unit expects;
//   B  N = 3 digits x M tokens rows x GS signed bytes, one bulk copy from the image the quantiser
//      wrote (already swizzled);
//   D  128 x N s32 in tensor memory, overwritten by the first MMA of the group (GS/32 MMAs of K = 32).
//
// Roles (they meet only through mbarriers):
//   warps 0-3   loaders.  A thread owns four 16-byte pieces of a group's packed weights (GS = 128): it asks for the
//               pieces of group g + 7 (cp.async into a ring of raw slots) and unpacks those of group g into one
//               of three A stages.
//   warps 4-11  drain: tcgen05.ld of the finished accumulator (a warp reads the 32 tensor-memory lanes of its
//               quadrant and half of the token columns), zero point through the tokens' digit sums, one f32 FMA
//               per (row, token) with the scale.  The group's scales, zero points and digit sums arrive in a side
//               ring that the drain warps fill themselves, seven groups ahead.
//   warp 12     one thread issues the MMAs of a group into one of two accumulators and commits once: the
//               commit frees the A and B stages and tells the drain that the accumulator is complete.
//   warp 13     one thread keeps three B stages filled, up to three groups ahead.
// While the drain works on group g the tensor cores work on group g + 1 and the loaders on group g + 2.  The kernel
// is bound by instruction issue, so ring positions are carried along instead of being computed from the group
// number, and the work is cut so that the bookkeeping of a group is paid by few warps.
// Split K: the CTAs of a tile whose groups are divided among several (grid.y) store partial results, which
// ksum_kernel adds in slice order (measured: letting the last CTA of a tile add them cost more than the extra launch).
// The kernel is launched programmatically behind the activation quantiser: everything that does not read the quantiser's
// output (set-up, tensor-memory allocation, the loaders' first requests) runs while that kernel still does.  Extending the
// chain (slice sum behind this kernel, the next quantiser behind the slice sum) was measured slower: the early-resident
// kernels of the next projection take issue slots and bandwidth from the one that is running (1.13 -> 1.32 ms for eight
// 7B layers at 30 tokens).
// Every wait on an mbarrier is bounded; a wait that gives up raises a flag that ends every loop.
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels.cuh"

namespace l2 {

namespace {

constexpr int TC_LOAD_WARPS = 4, TC_DRAIN_WARPS = 8;
constexpr int TC_LOADERS = 32 * TC_LOAD_WARPS;     // 128
constexpr int TC_DRAINERS = 32 * TC_DRAIN_WARPS;   // 256
constexpr int TC_THREADS = TC_LOADERS + TC_DRAINERS + 64;  // + the MMA warp and the B warp: 448
constexpr int TC_MMA_WARP = TC_LOAD_WARPS + TC_DRAIN_WARPS;
constexpr int TC_STAGES = 3;     // A and B stages
constexpr int TC_RING = 4;       // barrier ring of groups in flight (full / done)
constexpr int TC_RAW = 8;        // raw ring: groups whose packed weight words are in shared memory or on their way there
constexpr int TC_SIDE = 12;      // side ring (scales, zero points, digit sums)
constexpr int TC_AHEAD = TC_RAW - 1;  // groups between a request and the step that makes it (both rings)
constexpr int MAX_TOKENS = 64;   // tokens of one pass (N = 3 * tokens <= 192 columns)
constexpr int TC_HALF = MAX_TOKENS / 2;   // tokens a drain thread holds at most
constexpr int TC_META = 8 * 80;  // bytes of a group's scales and zero points: 20 words of each of the 8 records
constexpr uint32_t TC_WAIT_LIMIT = 1u << 20;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// One poll of a barrier phase with a time hint: the hardware parks the thread until the phase completes or the time has
// passed.  A warp that polls in a tight loop instead takes issue slots and shared-memory bandwidth from the warps that
// share its scheduler, and this kernel's warps wait a lot (measured: every role ran three to four times slower).
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity), "r"(2000u) : "memory");
    return ok != 0;
}
// bounded: gives up after TC_WAIT_LIMIT polls or as soon as another thread has given up.  A poll that fails is followed
// by a short sleep: barrier polls share the shared-memory pipe with every store, copy and MMA issue of the CTA, and
// hundreds of waiting threads polling back to back made each of those take 200 to 300 cycles (measured).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* failed) {
#pragma unroll 1
    for (uint32_t i = 0; i < TC_WAIT_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*failed) return false;
        __nanosleep(40);
    }
    return false;
}
// the same for a whole warp: lane 0 polls, the others sleep at the shuffle and then look at the barrier once themselves
// (one successful poll each, which also orders their reads behind the arrivals)
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* failed) {
    bool ok = true;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, failed);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    return ok && mbar_try_wait(bar, parity);
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void commit_to(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// (float)i for |i| < 2^22 without a conversion instruction: 1.5 * 2^23 + i is exact in f32
__device__ __forceinline__ float magic_float(int i) { return __int_as_float(0x4B400000 + i) - 12582912.0f; }

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


// the same, first with one poll by every lane (the usual case: the phase is complete or completes while the hardware parks the warp)
__device__ __forceinline__ bool mbar_wait_fast(uint64_t* bar, uint32_t parity, volatile int* failed) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_warp(bar, parity, failed);
}

}  // namespace

template <int W>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_q4_tc_kernel(const __grid_constant__ TcParams P) {
    constexpr uint32_t GS = 32 * W, A_BYTES = 128 * GS, RAW_BYTES = 8 * 64 * W * 4, UW = 64 * W + 20;  // UW: words per unit record
    constexpr int ITEMS = 512 / TC_LOADERS;      // (record, half, lane) items of a group's A tile per loader thread
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t ab_full[TC_RING], mma_done[TC_RING], acc_free[2], raw_full[TC_RAW], side_full[TC_SIDE];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t N = P.n;
    const int tile = blockIdx.x;                 // 128 output rows
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t b_bytes = N * GS, sv_bytes = (uint32_t)P.mpad * 4u;
    const uint32_t b_stage = (b_bytes + 1023) & ~1023u;
    const uint32_t side_bytes = TC_META + sv_bytes;
    uint8_t* stage_a = smem;                                 // [TC_STAGES][A_BYTES]
    uint8_t* stage_b = smem + TC_STAGES * A_BYTES;           // [TC_STAGES][b_stage]
    uint8_t* raw = stage_b + TC_STAGES * b_stage;            // [TC_RAW][8 records][64 W words]
    uint8_t* side = raw + TC_RAW * RAW_BYTES;                // [TC_SIDE][8 records x 20 words | mpad floats]

    if (tid == 0) {
        for (int i = 0; i < TC_RING; i++) { mbar_init(&ab_full[i], TC_LOADERS + 1); mbar_init(&mma_done[i], 1); }
        for (int i = 0; i < 2; i++) mbar_init(&acc_free[i], TC_DRAINERS);
        for (int i = 0; i < TC_RAW; i++) mbar_init(&raw_full[i], TC_LOADERS);
        for (int i = 0; i < TC_SIDE; i++) mbar_init(&side_full[i], TC_DRAINERS);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_MMA_WARP) {  // 512 columns of tensor memory: two accumulators of up to 256 columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_addr(&tmem_base_s)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;

    // split K: blockIdx.y takes groups [gb, gb + G) of the matrix's Gfull
    const int Gfull = P.G;
    const int gper = (Gfull + (int)gridDim.y - 1) / (int)gridDim.y;
    const int gb = (int)blockIdx.y * gper;
    const int G = min(gper, Gfull - gb);  // groups of this CTA (at least one: the host never launches empty slices)
    const size_t img_group = (size_t)b_bytes + sv_bytes;  // a group's block of the digit image: digits, then digit sums

    if (warp < TC_LOAD_WARPS) {
        // ================= loaders ==================================================================================
        // item (record sub, half h, lane (r, t)) = W words of row 8h + r, inputs 8 (t W + j) ..; thread tid owns the items
        // tid + 128 it: its own 16-byte piece of records sub0 + 2 it (GS = 128; smaller groups have fewer pieces, and a
        // thread then unpacks words that another thread asked for: the barrier of the raw slot covers all of them)
        constexpr int NW16 = 8 * 16 * W;                          // 16-byte pieces of a group's weight words
        // A request overwrites the raw slot of an earlier group.  With GS = 128 a thread reads only pieces it asked for itself, so
        // the slot of the group it unpacked last is free; otherwise the slot must be one that every loader warp has left: the
        // warps are at most two groups apart (a warp passes group g only after all have delivered group g - 3).
        constexpr int AHEAD = W == 4 ? TC_RAW - 1 : TC_RAW - 3;
        const uint32_t* rq_w[ITEMS];
        bool has_w[ITEMS];
#pragma unroll
        for (int it = 0; it < ITEMS; it++) {
            const int piece = tid + it * TC_LOADERS;
            has_w[it] = W == 4 || piece < NW16;
            rq_w[it] = P.rec + ((size_t)min(tile * 8 + piece / (16 * W), P.tiles16 - 1) * Gfull + gb) * UW + (size_t)(piece % (16 * W)) * 4;  // rows beyond the matrix read the last record (results dropped)
        }
        const uint32_t raw_s = smem_addr(raw) + (uint32_t)tid * 16u, rawfull_s = smem_addr(&raw_full[0]);
        int rq_g = 0;
        uint32_t rq_raw = 0;
        auto request = [&]() {
            if (rq_g < G) {
#pragma unroll
                for (int it = 0; it < ITEMS; it++) {
                    if (has_w[it]) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(raw_s + rq_raw * RAW_BYTES + (uint32_t)(it * TC_LOADERS * 16)), "l"(rq_w[it]) : "memory");
                    rq_w[it] += UW;
                }
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(rawfull_s + rq_raw * 8u) : "memory");
            }
            rq_g++;
            rq_raw = (rq_raw + 1) & (TC_RAW - 1);
        };
        const uint8_t* up_src[ITEMS];
        uint8_t *up_dst0[ITEMS], *up_dst1[ITEMS];
#pragma unroll
        for (int it = 0; it < ITEMS; it++) {
            const int idx = tid + it * TC_LOADERS, sub = idx >> 6, hl = idx & 63, uh = hl >> 5, ur = (hl & 31) >> 2, ut = hl & 3;
            const uint32_t arow = sub * 16 + uh * 8 + ur;
            up_src[it] = raw + ((size_t)sub * 64 + hl) * W * 4;
            up_dst0[it] = stage_a + (W == 4 ? arow * 128u + ((((uint32_t)ut * 2u) ^ (uint32_t)ur) << 4) : swz(arow, (uint32_t)ut * W * 8, GS));
            up_dst1[it] = stage_a + (W == 4 ? arow * 128u + ((((uint32_t)ut * 2u + 1u) ^ (uint32_t)ur) << 4) : swz(arow, ((uint32_t)ut * W + 1) * 8, GS));
        }
#pragma unroll 1
        for (int j = 0; j < AHEAD; j++) request();
        bool ok = true;
        uint32_t up_raw = 0, up_rawph = 0, up_a = 0;
#pragma unroll 1
        for (int g = 0; g < G; g++) {
            request();  // group g + AHEAD
            if (!mbar_wait_fast(&raw_full[up_raw], up_rawph, &failed)) { ok = false; break; }
            // the A stage was read by the MMAs of group g - 3
            if (g >= TC_STAGES && !mbar_wait_fast(&mma_done[(g - TC_STAGES) & (TC_RING - 1)], ((uint32_t)(g - TC_STAGES) >> 2) & 1u, &failed)) { ok = false; break; }
            // 8 weights -> 8 bytes in the block order (0,2,4,6,1,3,5,7), the order of the digit image
            if (W == 4) {  // two words share a 16-byte piece of the swizzled row: an item is two 16-byte stores
                uint4 v[ITEMS];
#pragma unroll
                for (int it = 0; it < ITEMS; it++) v[it] = *reinterpret_cast<const uint4*>(up_src[it] + up_raw * RAW_BYTES);
#pragma unroll
                for (int it = 0; it < ITEMS; it++) {
                    *reinterpret_cast<uint4*>(up_dst0[it] + up_a * A_BYTES) = make_uint4(v[it].x & 0x0F0F0F0Fu, (v[it].x >> 4) & 0x0F0F0F0Fu, v[it].y & 0x0F0F0F0Fu, (v[it].y >> 4) & 0x0F0F0F0Fu);
                    *reinterpret_cast<uint4*>(up_dst1[it] + up_a * A_BYTES) = make_uint4(v[it].z & 0x0F0F0F0Fu, (v[it].z >> 4) & 0x0F0F0F0Fu, v[it].w & 0x0F0F0F0Fu, (v[it].w >> 4) & 0x0F0F0F0Fu);
                }
            } else if (W == 2) {
#pragma unroll
                for (int it = 0; it < ITEMS; it++) {
                    const uint2 v = *reinterpret_cast<const uint2*>(up_src[it] + up_raw * RAW_BYTES);
                    *reinterpret_cast<uint2*>(up_dst0[it] + up_a * A_BYTES) = make_uint2(v.x & 0x0F0F0F0Fu, (v.x >> 4) & 0x0F0F0F0Fu);
                    *reinterpret_cast<uint2*>(up_dst1[it] + up_a * A_BYTES) = make_uint2(v.y & 0x0F0F0F0Fu, (v.y >> 4) & 0x0F0F0F0Fu);
                }
            } else {
#pragma unroll
                for (int it = 0; it < ITEMS; it++) {
                    const uint32_t v = *reinterpret_cast<const uint32_t*>(up_src[it] + up_raw * RAW_BYTES);
                    *reinterpret_cast<uint2*>(up_dst0[it] + up_a * A_BYTES) = make_uint2(v & 0x0F0F0F0Fu, (v >> 4) & 0x0F0F0F0Fu);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the MMA unit
            mbar_arrive(&ab_full[g & (TC_RING - 1)]);
            up_raw = (up_raw + 1) & (TC_RAW - 1);
            up_rawph ^= up_raw == 0 ? 1u : 0u;
            up_a = up_a == TC_STAGES - 1 ? 0 : up_a + 1;
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        if (!ok && lane == 0) { failed = 1; if (P.status) atomicExch(P.status, 2003); }
    } else if (warp < TC_MMA_WARP) {
        // ================= drain warps ==================================================================================
        // a warp may read the 32 tensor-memory lanes (= rows) of the quadrant given by its index in the CTA modulo 4;
        // the first four drain warps take the first half of the token columns, the other four the second half
        const int dt = tid - TC_LOADERS;                         // 0 .. 255
        const int quad = warp & 3, half = (warp - TC_LOAD_WARPS) >> 2;
        const int row = 32 * quad + lane;                        // row inside the 128-row tile
        const int orow = tile * 128 + row;                       // output row
        const bool row_ok = (orow >> 4) < P.tiles16;
        const int tq = P.mpad / 2;                               // tokens per column half, a multiple of 8 (mpad % 16 == 0)
        const uint32_t moff_s = (uint32_t)(row >> 4) * 20u + (uint32_t)(orow & 15), moff_z = (uint32_t)(row >> 4) * 20u + 16u + (uint32_t)((orow & 15) >> 3);
        const uint32_t zsh = 4 * (orow & 7);
        const uint32_t tcol = tmem_base + ((uint32_t)(32 * quad) << 16) + (uint32_t)(half * tq);  // column of digit p, token t: p * mpad + t
        // ---- side ring: 16-byte pieces of the 8 records' scales and zero points (40) and of the tokens' digit sums (mpad / 4)
        // the tokens' digit sums are written by the quantiser that runs in front of this kernel; with a programmatic launch
        // this kernel may have started before that one finished (the loaders need nothing of it): wait for it here
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const bool has_m = dt < 40, has_s = dt >= 64 && dt < 64 + (int)(sv_bytes / 16);
        const uint32_t* rq_m = P.rec + ((size_t)min(tile * 8 + dt / 5, P.tiles16 - 1) * Gfull + gb) * UW + 64 * W + (size_t)(dt % 5) * 4;
        const uint8_t* rq_s = P.bimg + (size_t)gb * img_group + b_bytes + (size_t)(dt - 64) * 16;
        const uint32_t side_dst = smem_addr(side) + (has_m ? (uint32_t)dt * 16u : TC_META + (uint32_t)(dt - 64) * 16u), sidefull_s = smem_addr(&side_full[0]);
        int rq_g = 0;
        uint32_t rq_side = 0;
        auto request = [&]() {
            if (rq_g < G) {
                if (has_m) asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(side_dst + rq_side * side_bytes), "l"(rq_m) : "memory");
                if (has_s) asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(side_dst + rq_side * side_bytes), "l"(rq_s) : "memory");
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(sidefull_s + rq_side * 8u) : "memory");
                rq_m += UW; rq_s += img_group;
            }
            rq_g++;
            rq_side = rq_side == TC_SIDE - 1 ? 0 : rq_side + 1;
        };
        float acc[TC_HALF];
#pragma unroll
        for (int i = 0; i < TC_HALF; i++) acc[i] = 0.f;
#pragma unroll 1
        for (int j = 0; j < TC_AHEAD; j++) request();
        bool ok = true;
        uint32_t dr_side = 0, dr_sideph = 0;
#pragma unroll 1
        for (int g = 0; g < G; g++) {
            request();  // group g + 7
            const uint32_t b = (uint32_t)g & 1u;
            if (!mbar_wait_fast(&side_full[dr_side], dr_sideph, &failed)) { ok = false; break; }
            const uint32_t* meta = reinterpret_cast<const uint32_t*>(side + dr_side * side_bytes);
            const float* sv = reinterpret_cast<const float*>(meta + TC_META / 4) + half * tq;
            const float zf = (float)((int)((meta[moff_z] >> zsh) & 15u) + 1);  // src/gptq.rs:148
            const float scf = row_ok ? __uint_as_float(meta[moff_s]) : 0.f;
            const float nzs = -zf * scf;
            if (!mbar_wait_fast(&mma_done[g & (TC_RING - 1)], ((uint32_t)g >> 2) & 1u, &failed)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tbase = tcol + b * 256u;
#pragma unroll
            for (int t0 = 0; t0 < TC_HALF; t0 += 16) {  // 16 tokens per step: one 16-column load per digit
                if (t0 >= tq) break;  // warp-uniform: tq is a multiple of 8
                uint32_t v[3][16];
#pragma unroll
                for (int p = 0; p < 3; p++)
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                 : "=r"(v[p][0]), "=r"(v[p][1]), "=r"(v[p][2]), "=r"(v[p][3]), "=r"(v[p][4]), "=r"(v[p][5]), "=r"(v[p][6]), "=r"(v[p][7]),
                                   "=r"(v[p][8]), "=r"(v[p][9]), "=r"(v[p][10]), "=r"(v[p][11]), "=r"(v[p][12]), "=r"(v[p][13]), "=r"(v[p][14]), "=r"(v[p][15])
                                 : "r"(tbase + (uint32_t)(p * P.mpad + t0)) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (t0 + 16 >= tq) {  // the last columns of this accumulator have been read: the MMAs of group g + 2 may overwrite it
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    mbar_arrive(&acc_free[b]);
                }
#pragma unroll
                for (int q8 = 0; q8 < 16; q8 += 8) {
                    if (t0 + q8 < tq) {  // warp-uniform
#pragma unroll
                        for (int q = q8; q < q8 + 8; q++) {
                            // c0 2^16 + c1 2^8 + c2 (|c| < 2^18): the upper two as an integer through the conversion unit (quarter
                            // rate, but one issue slot; rounded once to f32), the lowest through floats: an integer below 2^22 becomes
                            // a float exactly with one integer add and one float add.  The zero point enters through the token's sum
                            // of integers over the group (a float).
                            const int tk = t0 + q;  // token inside this half
                            const float fh = (float)((int)v[0][q] * 256 + (int)v[1][q]);
                            acc[tk] = fmaf(nzs, sv[tk], fmaf(scf, fmaf(fh, 256.0f, magic_float((int)v[2][q])), acc[tk]));
                        }
                    }
                }
            }
            dr_side = dr_side == TC_SIDE - 1 ? 0 : dr_side + 1;
            dr_sideph ^= dr_side == 0 ? 1u : 0u;
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        if (!ok && lane == 0) { failed = 1; if (P.status) atomicExch(P.status, 2002); }
        // ---- output: out[m][orow] (+= for the residual epilogue), scaled per token; a slice of a split tile stores its part
        //      instead ([slice][m][rows]), and ksum_kernel adds the parts in slice order
        if (ok && !failed && row_ok && orow < P.rows) {
            const bool split = gridDim.y > 1;
#pragma unroll
            for (int tk = 0; tk < TC_HALF; tk++) {
                const int m = half * tq + tk;
                if (tk < tq && m < P.m) {
                    const float y = acc[tk] * __ldg(P.oscale + m);
                    if (split) P.part[(size_t)blockIdx.y * P.kstride + (size_t)m * P.rows + orow] = y;
                    else {
                        float* dst = P.out + (size_t)m * P.ldo + orow;
                        *dst = P.epi == EPI_RESID ? *dst + y : y;
                    }
                }
            }
        }
    } else if (warp == TC_MMA_WARP) {
        // ================= MMA issue: one thread ===================================================================
        if (lane == 0) {
            // instruction descriptor: D s32, A u8, B s8, both K-major, N, M = 128
            const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((N >> 3) << 17) | ((128u >> 4) << 24);
            const uint64_t desc_a0 = umma_desc(smem_addr(stage_a), GS), desc_b0 = umma_desc(smem_addr(stage_b), GS);  // stage 0, K step 0
            uint32_t s = 0;
#pragma unroll 1
            for (int g = 0; g < G; g++) {
                const uint32_t b = (uint32_t)g & 1u, ring = (uint32_t)g & (TC_RING - 1);
                bool ok = mbar_wait(&ab_full[ring], ((uint32_t)g >> 2) & 1u, &failed);
                if (ok && g >= 2) ok = mbar_wait(&acc_free[b], (((uint32_t)g >> 1) - 1u) & 1u, &failed);
                if (!ok) { failed = 1; if (P.status) atomicExch(P.status, 2001); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d = tmem_base + b * 256u;
                const uint64_t da0 = desc_a0 + (uint64_t)(s * (A_BYTES >> 4)), db0 = desc_b0 + (uint64_t)(s * (b_stage >> 4));
#pragma unroll
                for (uint32_t k = 0; k < (uint32_t)W; k++) {
                    const uint64_t da = da0 + 2 * k, db = db0 + 2 * k;  // 32 bytes further along K: the address field counts 16-byte units
                    const uint32_t accumulate = k ? 1u : 0u;
                    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
                                 ::"r"(d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
                }
                commit_to(&mma_done[ring]);  // the accumulator of group g is complete, its A and B stages may be refilled
                s = s == TC_STAGES - 1 ? 0 : s + 1;
            }
        }
    } else {
        // ================= B stages: one thread ========================================================================
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");  // the digit image is the output of the kernel in front of this one
            uint32_t s = 0;
            const uint8_t* src = P.bimg + (size_t)gb * img_group;
#pragma unroll 1
            for (int g = 0; g < G; g++) {
                bool ok = true;
                if (g >= TC_STAGES) ok = mbar_wait(&mma_done[(g - TC_STAGES) & (TC_RING - 1)], ((uint32_t)(g - TC_STAGES) >> 2) & 1u, &failed);  // the MMAs of group g - 3 have read the stage
                if (!ok) { failed = 1; if (P.status) atomicExch(P.status, 2004); break; }
                uint64_t* full = &ab_full[g & (TC_RING - 1)];
                mbar_expect_tx(full, b_bytes);
                bulk_g2s(stage_b + (size_t)s * b_stage, src, b_bytes, full);
                src += img_group;
                s = s == TC_STAGES - 1 ? 0 : s + 1;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == TC_MMA_WARP) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
}

// at least 120 KB so that only one CTA (one owner of the tensor memory) is resident per SM
size_t gemm_tc_smem_bytes(int gs, int n) {
    const size_t need = (size_t)TC_STAGES * ((size_t)128 * gs + (((size_t)n * gs + 1023) & ~(size_t)1023)) + (size_t)TC_RAW * 8 * 64 * (gs / 32) * 4 +
                        (size_t)TC_SIDE * (TC_META + (size_t)n / 3 * 4) + 1024;  // digit sums: 4 bytes per token, n = 3 tokens
    return need < 120 * 1024 ? 120 * 1024 : need;
}

int gemm_tc_mpad(int tokens) { return (tokens + 15) & ~15; }

size_t gemm_tc_image_bytes(int in, int gs, int tokens) {
    const size_t mpad = (size_t)gemm_tc_mpad(tokens);
    return (size_t)(in / gs) * (3 * mpad * gs + mpad * 4);
}

cudaError_t gemm_tc_init(int max_smem) {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(gemm_q4_tc_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(gemm_q4_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem)) != cudaSuccess) return e;
    return cudaFuncSetAttribute(gemm_q4_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
}

// Launched programmatically after the activation quantiser: set-up, tensor-memory allocation and the first weight requests
// of this kernel overlap the quantiser's run (about a third of a short GEMM is the time to fill its pipeline); the two
// roles that read the quantiser's output wait for it inside the kernel.
cudaError_t launch_gemm_tc(const TcParams& p, cudaStream_t st) {
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3((p.tiles16 + 7) / 8, p.ksplit > 1 ? p.ksplit : 1);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = gemm_tc_smem_bytes(p.gs, p.n);
    cfg.stream = st;
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    g_launches++;
    if (p.gs == 128) return cudaLaunchKernelEx(&cfg, gemm_q4_tc_kernel<4>, p);
    if (p.gs == 64) return cudaLaunchKernelEx(&cfg, gemm_q4_tc_kernel<2>, p);
    return cudaLaunchKernelEx(&cfg, gemm_q4_tc_kernel<1>, p);
}

}  // namespace l2
