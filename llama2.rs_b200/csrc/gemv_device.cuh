// Device-side building blocks shared by the stand-alone GEMV kernel (gemv_kernels.cu) and the
// one-kernel-per-token path (token_kernel.cu): integer MMA, mbarriers, bulk copies, the barrier of
// the consumer warps, and the staging of an activation vector as signed byte digits (per-operator kernels: 7-bit digits).
#pragma once

#include <cfloat>
#include <cmath>

#include "kernels.cuh"

namespace l2 {

__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The first MMA of a chain: the accumulator input is the constant zero, no register has to be cleared.
__device__ __forceinline__ void mma_u8s8_first(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One poll of a barrier phase.  The time hint lets the hardware park the thread until the phase
// completes (or the time has passed) instead of returning at once: a warp that polls in a tight
// loop floods the shared-memory pipe and slows every other warp of the SM down.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity, uint32_t hint_ns = 0) {
    uint32_t ok;
    if (hint_ns)
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns) : "memory");
    else
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Waits for a phase of the barrier, but never forever: after `limit` polls (each parked for up to
// 20 microseconds, with a pause between two) it gives up and reports failure; the caller records
// it in the status word and stops using the data.
constexpr uint32_t SK_WAIT_LIMIT = 1u << 17;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = SK_WAIT_LIMIT) {
#pragma unroll 1
    for (uint32_t i = 0; i < limit; i++) {
        if (mbar_try_wait(bar, parity, 20000u)) return true;
        __nanosleep(200);
    }
    return false;
}
// Bulk asynchronous copy global -> shared of this CTA; bytes and both addresses are multiples of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Shared-memory loads and barrier operations on 32-bit shared-space addresses.  The hot loops keep
// their addresses in this form: generic 64-bit pointers cost two registers each and a chain of
// wide integer operations per access.  The loads are volatile so that they stay in program order
// with the barrier operations around them.
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ bool mbar_try_wait_u32(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_u32(uint32_t bar, uint32_t parity, uint32_t limit = SK_WAIT_LIMIT) {
#pragma unroll 1
    for (uint32_t i = 0; i < limit; i++) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity), "r"(20000u) : "memory");
        if (ok) return true;
        __nanosleep(200);
    }
    return false;
}
__device__ __forceinline__ void mbar_expect_tx_u32(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s_u32(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ int lds_volatile_i32(uint32_t a) {
    int v;
    asm volatile("ld.volatile.shared.s32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ void sts_volatile_i32(uint32_t a, int v) { asm volatile("st.volatile.shared.s32 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }
__device__ __forceinline__ void mbar_arrive_u32(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// barrier of the SK_THREADS consumer threads only (the producer warp runs on its own)
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(SK_THREADS) : "memory"); }

__device__ __forceinline__ float block_reduce_2(float& mx, float sq, float* red /* 2*SK_WARPS+2 floats */) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
    }
    if (lane == 0) { red[warp] = mx; red[SK_WARPS + warp] = sq; }
    consumer_sync();
    if (warp == 0) {
        float m = lane < SK_WARPS ? red[lane] : 0.f;
        float s = lane < SK_WARPS ? red[SK_WARPS + lane] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            s += __shfl_xor_sync(0xffffffffu, s, o);
        }
        if (lane == 0) { red[2 * SK_WARPS] = m; red[2 * SK_WARPS + 1] = s; }
    }
    consumer_sync();
    mx = red[2 * SK_WARPS];
    const float total = red[2 * SK_WARPS + 1];
    consumer_sync();
    return total;
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 255) | ((uint32_t)(b & 255) << 8) | ((uint32_t)(c & 255) << 16) | ((uint32_t)(d & 255) << 24);
}

// ---- staging of an activation vector as digits ------------------------------------------------------
// Thread i owns the 8-input blocks i, i + 512, ...; the first SK_KEEP of them stay in registers
// between the two passes (max / sum of squares, then digits).
constexpr int SK_KEEP = 3;

// Loads block `blk` of the segment's vector times its norm weight; with `stats` also folds the block
// into the running max |v| and sum of x^2.
// Values that travel from CTA to CTA inside one kernel without a barrier in between are stored as
// (value, tag) pairs, one 64-bit word each: the reader polls until the tag is the one it expects (the
// tag names the launch and the phase that writes the value), so no fence, flag or barrier has to
// order the two sides.  Polls are bounded: after TAG_POLL_LIMIT tries the reader gives up.
constexpr uint32_t TAG_POLL_LIMIT_DEFAULT = 1u << 20;
// The limit lives in constant memory so that a host can shorten it (l2_options.poll_limit_log2): one value per
// device and translation unit, set when a launch plan is made.
static __constant__ uint32_t c_tag_poll_limit = TAG_POLL_LIMIT_DEFAULT;
#define TAG_POLL_LIMIT c_tag_poll_limit

__device__ __forceinline__ void store_tagged(void* base, size_t index, float v, uint32_t tag) {
    const unsigned long long w = (unsigned long long)__float_as_uint(v) | ((unsigned long long)tag << 32);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(static_cast<unsigned long long*>(base) + index), "l"(w) : "memory");
}
// The same word into a peer GPU's memory (over NVLink): system scope.
__device__ __forceinline__ void store_tagged_peer(void* base, size_t index, float v, uint32_t tag) {
    const unsigned long long w = (unsigned long long)__float_as_uint(v) | ((unsigned long long)tag << 32);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(static_cast<unsigned long long*>(base) + index), "l"(w) : "memory");
}
// The polls are system-scope loads: under tensor parallelism a value may have been stored by another GPU
// (st.relaxed.sys over NVLink into this GPU's memory), and a load only synchronises with a store whose
// scope it shares.  Device memory is served by this GPU's L2 either way.
#ifdef L2_POLL_GPU_SCOPE  // development switch: device-scope polls (single-GPU timing comparisons only)
#define L2_POLL_LD "ld.relaxed.gpu.global"
#else
#define L2_POLL_LD "ld.relaxed.sys.global"
#endif
// One tagged value; returns false when the poll limit is reached.
__device__ __forceinline__ bool load_tagged(const void* base, size_t index, uint32_t tag, float& v) {
    const unsigned long long* p = static_cast<const unsigned long long*>(base) + index;
#pragma unroll 1
    for (uint32_t it = 0; it < TAG_POLL_LIMIT; it++) {
        unsigned long long w;
        asm volatile(L2_POLL_LD ".u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
        if ((uint32_t)(w >> 32) == tag) { v = __uint_as_float((uint32_t)w); return true; }
    }
    v = 0.f;
    return false;
}
// Eight consecutive tagged values (64 bytes, 64-byte aligned).
__device__ __forceinline__ bool load_tagged8(const void* base, size_t index, uint32_t tag, float4& v0, float4& v1) {
    const uint4* p = reinterpret_cast<const uint4*>(static_cast<const unsigned long long*>(base) + index);
#pragma unroll 1
    for (uint32_t it = 0; it < TAG_POLL_LIMIT; it++) {
        uint4 a, b, c, d;
        asm volatile(L2_POLL_LD ".v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(p) : "memory");
        asm volatile(L2_POLL_LD ".v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p + 1) : "memory");
        asm volatile(L2_POLL_LD ".v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(c.x), "=r"(c.y), "=r"(c.z), "=r"(c.w) : "l"(p + 2) : "memory");
        asm volatile(L2_POLL_LD ".v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(d.x), "=r"(d.y), "=r"(d.z), "=r"(d.w) : "l"(p + 3) : "memory");
        if (a.y == tag && a.w == tag && b.y == tag && b.w == tag && c.y == tag && c.w == tag && d.y == tag && d.w == tag) {
            v0 = make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
            v1 = make_float4(__uint_as_float(c.x), __uint_as_float(c.z), __uint_as_float(d.x), __uint_as_float(d.z));
            return true;
        }
    }
    v0 = v1 = make_float4(0.f, 0.f, 0.f, 0.f);
    return false;
}

// Loads block `blk` of the segment's vector times its norm weight; with `stats` also folds the block
// into the running max |v| and sum of x^2.  tag != 0: the vector is stored as tagged pairs.
__device__ __forceinline__ void stage_fetch(const SkSeg& sg, int blk, float4& v0, float4& v1, bool stats, float& mx, float& sq,
                                            uint32_t tag = 0, bool* fail = nullptr) {
    const float4* x4 = reinterpret_cast<const float4*>(sg.x);
    const float4* n4 = reinterpret_cast<const float4*>(sg.nw);
    if (tag) {
        if (!load_tagged8(sg.x, (size_t)blk * 8, tag, v0, v1) && fail) *fail = true;
    } else {
        v0 = __ldcg(x4 + 2 * blk);  // written by other CTAs shortly before: read at the L2, never from a stale L1 line
        v1 = __ldcg(x4 + 2 * blk + 1);
    }
    if (stats) sq += v0.x * v0.x + v0.y * v0.y + v0.z * v0.z + v0.w * v0.w + v1.x * v1.x + v1.y * v1.y + v1.z * v1.z + v1.w * v1.w;
    if (sg.nw) {
        const float4 w0 = __ldg(n4 + 2 * blk), w1 = __ldg(n4 + 2 * blk + 1);
        v0.x *= w0.x; v0.y *= w0.y; v0.z *= w0.z; v0.w *= w0.w;
        v1.x *= w1.x; v1.y *= w1.y; v1.z *= w1.z; v1.w *= w1.w;
    }
    if (stats) {
        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))));
        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
    }
}

// P = 2^(26 - E) with 2^E <= mx < 2^(E+1): |v * P| < 2^27 for every |v| <= mx
__device__ __forceinline__ float stage_scale(float mx) {
    int e = 0;
    if (mx > 0.f && mx < INFINITY) e = 26 - (int)((__float_as_uint(mx) >> 23) & 255u) + 127;
    e = max(-100, min(100, e));
    return __uint_as_float((uint32_t)(127 + e) << 23);
}

// Writes the digits of block `blk` (8 values v0, v1 scaled by P) and adds them to the group sums.
// Called by whole warps; lanes whose block lies beyond the vector pass zeros and valid = false.
template <int W>
__device__ __forceinline__ void stage_emit(uint8_t* digits, int* ss, int stride, int blk, const float4& v0, const float4& v1, bool valid, float P) {
    const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    uint32_t E[8];  // per element: bytes d3, d2, d1, d0 (d0 signed, the others 0..127)
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const uint32_t X = (uint32_t)__float2int_rn(v[j] * P);
        E[j] = (X & 0x7Fu) | ((X << 1) & 0x7F00u) | ((X << 2) & 0x7F0000u) | ((X << 3) & 0xFF000000u);
    }
    // 4x4 byte transposes: words of one digit for inputs (0,2,4,6) and (1,3,5,7), the order in
    // which the nibbles of a weight word separate into its low and high halves
    uint32_t lo[4], hi[4];
    {
        const uint32_t a = __byte_perm(E[0], E[2], 0x5140), b2 = __byte_perm(E[0], E[2], 0x7362);
        const uint32_t c = __byte_perm(E[4], E[6], 0x5140), d = __byte_perm(E[4], E[6], 0x7362);
        lo[3] = __byte_perm(a, c, 0x5410); lo[2] = __byte_perm(a, c, 0x7632);
        lo[1] = __byte_perm(b2, d, 0x5410); lo[0] = __byte_perm(b2, d, 0x7632);
    }
    {
        const uint32_t a = __byte_perm(E[1], E[3], 0x5140), b2 = __byte_perm(E[1], E[3], 0x7362);
        const uint32_t c = __byte_perm(E[5], E[7], 0x5140), d = __byte_perm(E[5], E[7], 0x7362);
        hi[3] = __byte_perm(a, c, 0x5410); hi[2] = __byte_perm(a, c, 0x7632);
        hi[1] = __byte_perm(b2, d, 0x5410); hi[0] = __byte_perm(b2, d, 0x7632);
    }
    int sum[4];
#pragma unroll
    for (int p = 0; p < 4; p++) {
        if (valid) *reinterpret_cast<uint2*>(digits + (size_t)p * stride + (size_t)blk * 8) = make_uint2(lo[p], hi[p]);
        sum[p] = __dp4a((int)lo[p], 0x01010101, __dp4a((int)hi[p], 0x01010101, 0));
    }
    // a group is 4*W consecutive blocks = 4*W consecutive lanes: sum them with shuffles
    int s01 = 128 * sum[0] + sum[1], s23 = 128 * sum[2] + sum[3];
#pragma unroll
    for (int o = 1; o < 4 * W; o <<= 1) {
        s01 += __shfl_xor_sync(0xffffffffu, s01, o);
        s23 += __shfl_xor_sync(0xffffffffu, s23, o);
    }
    if (valid && (threadIdx.x & (4 * W - 1)) == 0) {
        const int g = blk / (4 * W);
        ss[2 * g] = s01;
        ss[2 * g + 1] = s23;
    }
}

// Turns the vector of one segment into digits and per-group digit sums in shared memory.
// Returns (in every thread) the factor the integer result has to be multiplied with.
template <int W>
__device__ float stage_digits(const SkSeg& sg, int in, float eps, uint8_t* digits, int* ss, float* red, unsigned long long* dbg = nullptr,
                              uint32_t tag = 0, bool* fail = nullptr) {
    const int nblk = in / 8;
    float mx = 0.f, sq = 0.f;
    float4 keep[SK_KEEP][2];
#pragma unroll
    for (int k = 0; k < SK_KEEP; k++) keep[k][0] = keep[k][1] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < SK_KEEP; k++) {
        const int blk = threadIdx.x + k * SK_THREADS;
        if (blk < nblk) stage_fetch(sg, blk, keep[k][0], keep[k][1], true, mx, sq, tag, fail);
    }
    for (int blk = threadIdx.x + SK_KEEP * SK_THREADS; blk < nblk; blk += SK_THREADS) {
        float4 a, b;
        stage_fetch(sg, blk, a, b, true, mx, sq, tag, fail);
    }
    if (dbg && threadIdx.x == 0) dbg[0] = clock64() + (mx > 1e30f ? 1 : 0);
    const float total = block_reduce_2(mx, sq, red);
    if (dbg && threadIdx.x == 0) dbg[1] = clock64();
    const float rs = sg.nw ? 1.0f / sqrtf(total / (float)in + eps) : 1.0f;  // src/models.rs:58-60
    const float P = stage_scale(mx);
    const int stride = in + 16;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const int rounds = (nblk + SK_THREADS - 1) / SK_THREADS;
#pragma unroll
    for (int k = 0; k < SK_KEEP; k++) {
        const int blk = threadIdx.x + k * SK_THREADS;
        if (k < rounds && (blk & ~31) < nblk) {  // warp-uniform
            const bool valid = blk < nblk;
            stage_emit<W>(digits, ss, stride, blk, valid ? keep[k][0] : zero4, valid ? keep[k][1] : zero4, valid, P);
        }
    }
    for (int k = SK_KEEP; k < rounds; k++) {
        const int blk = threadIdx.x + k * SK_THREADS;
        if ((blk & ~31) < nblk) {
            const bool valid = blk < nblk;
            float4 a = zero4, b = zero4;
            float m2 = 0.f, s2 = 0.f;
            if (valid) stage_fetch(sg, blk, a, b, false, m2, s2, tag, fail);
            stage_emit<W>(digits, ss, stride, blk, a, b, valid, P);
        }
    }
    if (dbg && threadIdx.x == 0) dbg[2] = clock64();
    return rs / P;
}

// Two segments whose vectors are two orderings of the same values (w1 and w3 read the same x, each
// in its own K order, with the norm weight ordered alike): the maximum and the sum of squares are
// taken once, from the first, and both are turned into digits with the same scale.  Needs
// in <= 2 * 8 * SK_THREADS.  Returns the common output factor.
template <int W>
__device__ float stage_digits_pair(const SkSeg& sa, const SkSeg& sb, int in, float eps, uint8_t* da, uint8_t* db, int* ssa, int* ssb, float* red,
                                   unsigned long long* dbg = nullptr, uint32_t tag = 0, bool* fail = nullptr) {
    const int nblk = in / 8;
    float mx = 0.f, sq = 0.f, m2 = 0.f, s2 = 0.f;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 ka[2][2], kb[2][2];
#pragma unroll
    for (int k = 0; k < 2; k++) {
        ka[k][0] = ka[k][1] = kb[k][0] = kb[k][1] = zero4;
        const int blk = threadIdx.x + k * SK_THREADS;
        if (blk < nblk) {
            stage_fetch(sa, blk, ka[k][0], ka[k][1], true, mx, sq, tag, fail);
            stage_fetch(sb, blk, kb[k][0], kb[k][1], false, m2, s2, tag, fail);
        }
    }
    if (dbg && threadIdx.x == 0) dbg[0] = clock64() + (mx > 1e30f ? 1 : 0);
    const float total = block_reduce_2(mx, sq, red);
    if (dbg && threadIdx.x == 0) dbg[1] = clock64();
    const float rs = sa.nw ? 1.0f / sqrtf(total / (float)in + eps) : 1.0f;
    const float P = stage_scale(mx);
    const int stride = in + 16;
#pragma unroll
    for (int k = 0; k < 2; k++) {
        const int blk = threadIdx.x + k * SK_THREADS;
        if ((blk & ~31) < nblk) {
            const bool valid = blk < nblk;
            stage_emit<W>(da, ssa, stride, blk, ka[k][0], ka[k][1], valid, P);
            stage_emit<W>(db, ssb, stride, blk, kb[k][0], kb[k][1], valid, P);
        }
    }
    if (dbg && threadIdx.x == 0) dbg[2] = clock64();
    return rs / P;
}

// ---- one-pass staging with one exponent per quantisation group (token kernel) --------------------
// X[k] = round(x[k] * nw[k] * 2^(26 - E_g)) with E_g the exponent of the largest |x * nw| of group g, so
// every group uses the full 28 bits and no statistic of the whole vector has to be known before the
// first digit is written: the vector is read once, a group is finished by the 4 * W lanes that hold it
// (shuffles only), and the factor 2^-(26 - E_g) goes into the per-(row, group) scale of the GEMV.
// The sum of squares for the rmsnorm is only needed by the epilogue and is collected on the side.
//
// Digits: X is written in balanced base 256, X = sum_j d_j 256^j with -128 <= d_j <= 127, which is two
// integer operations per value: the bytes of (X + 0x80808080) ^ 0x80808080.  All four are legal s8
// operands of the integer MMA.
//
// Layout in shared memory: digits [4 planes][pstride], plane 0 the most significant digit, a plane holding
// the K orders of the phase's matrices one after the other; sp [groups] records of four words
// {256 * S0 + S1, f * 2^16, 256 * S2 + S3, f}: the digit sums of the upper and of the lower digit pair, each
// followed by the factor its MMA columns are scaled with (f = 2^-(26 - E_g); the upper pair weighs 2^16 more).

// Turns 8 values of K-order block `blk` into digits and finishes the group's record.
template <int W>
__device__ __forceinline__ void stage_emit8(float (&v)[8], bool valid, int blk, uint8_t* digits, int pstride, uint4* sp) {
    float mx = fmaxf(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))),
                     fmaxf(fmaxf(fabsf(v[4]), fabsf(v[5])), fmaxf(fabsf(v[6]), fabsf(v[7]))));
    // (a group's 4 * W lanes reduce with shuffles: redux.sync on a part of the warp was measured slower here)
#pragma unroll
    for (int o = 1; o < 4 * W; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float P = stage_scale(mx);
    uint32_t E[8];  // per element: bytes d3, d2, d1, d0 (least significant digit first)
#pragma unroll
    for (int j = 0; j < 8; j++) E[j] = ((uint32_t)__float2int_rn(v[j] * P) + 0x80808080u) ^ 0x80808080u;
    // 4x4 byte transposes: words of one digit for inputs (0,2,4,6) and (1,3,5,7), the order in
    // which the nibbles of a weight word separate into its low and high halves
    uint32_t lo[4], hi[4];
    {
        const uint32_t a = __byte_perm(E[0], E[2], 0x5140), b2 = __byte_perm(E[0], E[2], 0x7362);
        const uint32_t c = __byte_perm(E[4], E[6], 0x5140), d = __byte_perm(E[4], E[6], 0x7362);
        lo[3] = __byte_perm(a, c, 0x5410); lo[2] = __byte_perm(a, c, 0x7632);
        lo[1] = __byte_perm(b2, d, 0x5410); lo[0] = __byte_perm(b2, d, 0x7632);
    }
    {
        const uint32_t a = __byte_perm(E[1], E[3], 0x5140), b2 = __byte_perm(E[1], E[3], 0x7362);
        const uint32_t c = __byte_perm(E[5], E[7], 0x5140), d = __byte_perm(E[5], E[7], 0x7362);
        hi[3] = __byte_perm(a, c, 0x5410); hi[2] = __byte_perm(a, c, 0x7632);
        hi[1] = __byte_perm(b2, d, 0x5410); hi[0] = __byte_perm(b2, d, 0x7632);
    }
    int sum[4];
#pragma unroll
    for (int p = 0; p < 4; p++) {
        if (valid) *reinterpret_cast<uint2*>(digits + (size_t)p * pstride + (size_t)blk * 8) = make_uint2(lo[p], hi[p]);
        sum[p] = __dp4a((int)lo[p], 0x01010101, __dp4a((int)hi[p], 0x01010101, 0));
    }
    // a group is 4*W consecutive blocks = 4*W consecutive lanes: sum them with shuffles
    int s01 = 256 * sum[0] + sum[1], s23 = 256 * sum[2] + sum[3];
#pragma unroll
    for (int o = 1; o < 4 * W; o <<= 1) {
        s01 += __shfl_xor_sync(0xffffffffu, s01, o);
        s23 += __shfl_xor_sync(0xffffffffu, s23, o);
    }
    if (valid && (threadIdx.x & (4 * W - 1)) == 0) {
        const uint32_t f = (254u << 23) - __float_as_uint(P);  // 1 / P, exact (P is a power of two)
        sp[blk / (4 * W)] = make_uint4((uint32_t)s01, f + (16u << 23), (uint32_t)s23, f);
    }
}

// A vector that its producers already write in this matrix's K order (w2 after w1/w3): polled block by block and
// turned into digits at once.  Returns this thread's share of the sum of squares.
template <int W>
__device__ __forceinline__ float stage_direct(const void* x_tagged, int in, uint8_t* digits, int pstride, uint4* sp, uint32_t tag, bool* fail,
                                              unsigned long long* stamp = nullptr) {
    const int nblk = in / 8;
    float sq = 0.f;
#pragma unroll 1
    for (int blk = threadIdx.x; (blk & ~31) < nblk; blk += SK_THREADS) {
        const bool valid = blk < nblk;
        float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
        if (valid && !load_tagged8(x_tagged, (size_t)blk * 8, tag, v0, v1)) *fail = true;
        if (stamp && threadIdx.x == 0 && blk == 0) stamp[21] = clock64();
        float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        sq += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3] + v[4] * v[4] + v[5] * v[5] + v[6] * v[6] + v[7] * v[7];
        stage_emit8<W>(v, valid, blk, digits, pstride, sp);
    }
    if (stamp && threadIdx.x == 0) stamp[23] = clock64();
    return sq;
}

// ---- staging of a vector that arrives in natural order and is consumed in a matrix's K order -------
// Values cross CTAs fastest when every 128-byte line has one writer: a vector whose elements are scattered
// by their producers into a consumer's K order (eight writers per line polled) takes about three times as
// long to arrive as the same vector written tile by tile.  So producers store in natural order, and the
// consumer (1) polls the natural vector, applies the norm weight, takes the sum of squares and scatters the
// values into the matrix's K order in shared memory (plain floats; the bank conflicts of the scattered stores
// are paid while other values are still awaited), and (2) turns the K-order floats into digits block by block.
// seg[s].perm holds 16-bit indices: natural element i belongs at position perm[i] of matrix s's K order.

template <int W>
__device__ __forceinline__ float stage_natural(const SkSeg* seg, int nseg, int in, int G, uint8_t* digits, int pstride, uint4* sp, float* xs, uint32_t tag,
                                               bool* fail, bool gather, unsigned long long* stamp = nullptr) {
    const int nblk = in / 8;
    float* xs1 = xs + in;  // the second matrix's K order (w3 beside w1)
    float sq = 0.f;
    if (gather) {
        // Two matrices on a long input (w1 and w3 of the 70B shapes): two K-ordered copies of the vector would take the
        // shared memory of a ring slot or two, and the ring's depth is what the weight stream of these shapes is short of.
        // The vector is kept once, in natural order, and each matrix's blocks are gathered from it through its g_index
        // (seg[s].perm: forward 16-bit indices) when the digits are cut.
#pragma unroll 1
        for (int blk = threadIdx.x; blk < nblk; blk += SK_THREADS) {
            float4 w0 = make_float4(1.f, 1.f, 1.f, 1.f), w1 = w0;
            if (seg[0].nw) {
                w0 = __ldg(reinterpret_cast<const float4*>(seg[0].nw) + 2 * blk);
                w1 = __ldg(reinterpret_cast<const float4*>(seg[0].nw) + 2 * blk + 1);
            }
            float4 v0, v1;
            if (!load_tagged8(seg[0].x, (size_t)blk * 8, tag, v0, v1)) *fail = true;
            sq += v0.x * v0.x + v0.y * v0.y + v0.z * v0.z + v0.w * v0.w + v1.x * v1.x + v1.y * v1.y + v1.z * v1.z + v1.w * v1.w;
            v0.x *= w0.x; v0.y *= w0.y; v0.z *= w0.z; v0.w *= w0.w;
            v1.x *= w1.x; v1.y *= w1.y; v1.z *= w1.z; v1.w *= w1.w;
            reinterpret_cast<float4*>(xs)[2 * blk] = v0;
            reinterpret_cast<float4*>(xs)[2 * blk + 1] = v1;
        }
        if (stamp && threadIdx.x == 0) stamp[21] = clock64();
        consumer_sync();
        if (stamp && threadIdx.x == 0) stamp[22] = clock64();
#pragma unroll 1
        for (int s = 0; s < nseg; s++) {
#pragma unroll 1
            for (int blk = threadIdx.x; (blk & ~31) < nblk; blk += SK_THREADS) {
                const bool valid = blk < nblk;
                float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (valid) {
                    const uint4 ix = __ldg(reinterpret_cast<const uint4*>(seg[s].perm) + blk);
                    v[0] = xs[ix.x & 0xFFFFu]; v[1] = xs[ix.x >> 16]; v[2] = xs[ix.y & 0xFFFFu]; v[3] = xs[ix.y >> 16];
                    v[4] = xs[ix.z & 0xFFFFu]; v[5] = xs[ix.z >> 16]; v[6] = xs[ix.w & 0xFFFFu]; v[7] = xs[ix.w >> 16];
                }
                stage_emit8<W>(v, valid, blk, digits + (size_t)s * in, pstride, sp + s * G);
            }
        }
        if (stamp && threadIdx.x == 0) stamp[23] = clock64();
        return sq;
    }
    // (1) everything that does not depend on the awaited values is requested first: positions and norm weights
#pragma unroll 1
    for (int blk = threadIdx.x; blk < nblk; blk += SK_THREADS) {
        const uint4 i0 = __ldg(reinterpret_cast<const uint4*>(seg[0].perm) + blk);
        uint4 i1 = make_uint4(0, 0, 0, 0);
        if (nseg == 2) i1 = __ldg(reinterpret_cast<const uint4*>(seg[1].perm) + blk);
        float4 w0 = make_float4(1.f, 1.f, 1.f, 1.f), w1 = w0;
        if (seg[0].nw) {
            w0 = __ldg(reinterpret_cast<const float4*>(seg[0].nw) + 2 * blk);
            w1 = __ldg(reinterpret_cast<const float4*>(seg[0].nw) + 2 * blk + 1);
        }
        float4 v0, v1;
        if (!load_tagged8(seg[0].x, (size_t)blk * 8, tag, v0, v1)) *fail = true;
        sq += v0.x * v0.x + v0.y * v0.y + v0.z * v0.z + v0.w * v0.w + v1.x * v1.x + v1.y * v1.y + v1.z * v1.z + v1.w * v1.w;
        v0.x *= w0.x; v0.y *= w0.y; v0.z *= w0.z; v0.w *= w0.w;
        v1.x *= w1.x; v1.y *= w1.y; v1.z *= w1.z; v1.w *= w1.w;
        xs[i0.x & 0xFFFFu] = v0.x; xs[i0.x >> 16] = v0.y; xs[i0.y & 0xFFFFu] = v0.z; xs[i0.y >> 16] = v0.w;
        xs[i0.z & 0xFFFFu] = v1.x; xs[i0.z >> 16] = v1.y; xs[i0.w & 0xFFFFu] = v1.z; xs[i0.w >> 16] = v1.w;
        if (nseg == 2) {
            xs1[i1.x & 0xFFFFu] = v0.x; xs1[i1.x >> 16] = v0.y; xs1[i1.y & 0xFFFFu] = v0.z; xs1[i1.y >> 16] = v0.w;
            xs1[i1.z & 0xFFFFu] = v1.x; xs1[i1.z >> 16] = v1.y; xs1[i1.w & 0xFFFFu] = v1.z; xs1[i1.w >> 16] = v1.w;
        }
    }
    if (stamp && threadIdx.x == 0) stamp[21] = clock64();
    consumer_sync();
    if (stamp && threadIdx.x == 0) stamp[22] = clock64();
    // (2) digits, block by block of each matrix's K order
#pragma unroll 1
    for (int s = 0; s < nseg; s++) {
        const float4* src = reinterpret_cast<const float4*>(xs + (size_t)s * in);
#pragma unroll 1
        for (int blk = threadIdx.x; (blk & ~31) < nblk; blk += SK_THREADS) {
            const bool valid = blk < nblk;
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
            if (valid) { a = src[2 * blk]; b = src[2 * blk + 1]; }
            float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            stage_emit8<W>(v, valid, blk, digits + (size_t)s * in, pstride, sp + s * G);
        }
    }
    if (stamp && threadIdx.x == 0) stamp[23] = clock64();
    return sq;
}

// Asks the L2 to fetch [p, p + bytes) from HBM; nothing waits on it.
__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
    const char* c = static_cast<const char*>(p);
    for (uint32_t off = 0; off < bytes; off += 32768u) {
        const uint32_t n = min(32768u, bytes - off) & ~15u;
        if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(c + off), "r"(n) : "memory");
    }
}
}  // namespace l2
