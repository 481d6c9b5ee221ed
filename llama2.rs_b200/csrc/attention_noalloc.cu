// Attention of one position for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need attention:
// code running inside a latency-critical serving loop that has handed all device memory to its
// own pool, plug-ins that are only given pointers into such a pool, and callers that hold locks
// under which the CUDA allocator (which may synchronise the device) must not run.  For them the
// split-sequence scratch of the attention kernel (per-split partial sums and arrival tickets)
// lives in a fixed array inside the library image instead of a caller workspace.
//
// Limits and rules, all checked or documented at the entry point below:
//   * at most L2_NOALLOC_MAX_HEADS query heads and L2_NOALLOC_MAX_KV_HEADS kv heads;
//   * every GPU that loads the library keeps the array (about 1.1 MB) until the process exits;
//   * all calls on a device share the array, and it keeps the last call's contents: the tickets
//     are cleared at the start of every call, and two calls that overlap on the GPU (different
//     streams, or different host threads) race on it and must be serialised by the caller;
//   * the first call on a device looks up the array's device address; make that first call
//     before starting any stream capture.
#include <cuda_runtime.h>

#include <atomic>

#include "host_common.h"
#include "kernels.cuh"
#include "model.h"

#define L2_NOALLOC_MAX_HEADS 64
#define L2_NOALLOC_MAX_KV_HEADS 64
#define L2_NOALLOC_MAX_SPLIT 32
#define L2_NOALLOC_TICKET_BYTES 256
#define L2_NOALLOC_SCRATCH_BYTES \
    (L2_NOALLOC_TICKET_BYTES + L2_NOALLOC_MAX_HEADS * L2_NOALLOC_MAX_SPLIT * (128 + 2) * 4)

// In host code this name is only a stand-in for the device array: it is never passed to a
// kernel; its device address is taken with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_attention_scratch[L2_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::atomic<void*> g_scratch_addr[kMaxDevices];  // device address of g_attention_scratch, per device (zero-initialised: static storage)
}

using namespace l2;

extern "C" int l2_attention_decode_noalloc(int n_heads, int n_kv_heads, int pos, const float* q, const float* k,
                                           const float* v, float* key_cache, float* value_cache, const float* rope_cos,
                                           const float* rope_sin, float* out, void* cuda_stream) {
    clear_error();
    if (int rc = check_attention_args(n_heads, n_kv_heads, pos, q, k, v, key_cache, value_cache, rope_cos, rope_sin, out)) return rc;
    if (n_heads > L2_NOALLOC_MAX_HEADS || n_kv_heads > L2_NOALLOC_MAX_KV_HEADS)
        return fail(L2_EINVAL, "l2_attention_decode_noalloc: %d heads / %d kv heads exceed the built-in scratch (max %d / %d); "
                    "use l2_attention_decode_dev with a caller workspace", n_heads, n_kv_heads, L2_NOALLOC_MAX_HEADS, L2_NOALLOC_MAX_KV_HEADS);
    int dev = 0;
    L2_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(L2_EINVAL, "l2_attention_decode_noalloc: device ordinal %d unsupported", dev);
    void* addr = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (!addr) {  // set-up, once per device, with that device current (two threads racing here store the same value)
        L2_CUDA(cudaGetSymbolAddress(&addr, g_attention_scratch));
        g_scratch_addr[dev].store(addr, std::memory_order_release);
    }
    char* base = static_cast<char*>(addr);
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    // Same split geometry as l2_attention_decode_dev, capped by what the array holds.
    int max_split = attention_max_split(n_kv_heads);  // from the SM count of the current device (an attribute query, no allocation)
    if (max_split > L2_NOALLOC_MAX_SPLIT) max_split = L2_NOALLOC_MAX_SPLIT;
    L2_CUDA(cudaMemsetAsync(base, 0, L2_NOALLOC_TICKET_BYTES, st));  // the tickets must start at zero
    AttnParams a{};
    a.q = q; a.k = k; a.v = v; a.kc = key_cache; a.vc = value_cache;
    a.rope_cos = rope_cos; a.rope_sin = rope_sin;
    a.ctl = nullptr; a.pos_fixed = pos;
    a.counter = reinterpret_cast<unsigned*>(base);
    a.part = reinterpret_cast<float*>(base + L2_NOALLOC_TICKET_BYTES);
    a.out = out; a.oidx = nullptr;
    a.n_kv_heads = n_kv_heads; a.ag = n_heads / n_kv_heads;
    a.max_split = max_split; a.split_min = 64;
    launch_attn(a, st, false);
    L2_CUDA(cudaGetLastError());
    return L2_OK;
}
