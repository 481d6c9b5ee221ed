// Tensor parallelism over the GPUs of one box (one process per GPU): NCCL plumbing.
// The reference has no multi-GPU code; this is the sharding of the 70B model described in
// include/llama2_b200.h (l2_options::tp_rank / tp_world, l2_tp_unique_id, l2_model_tp_connect).
//
// Every QLinear is split by output rows (whole 16-row tiles), so a rank streams 1/T of every
// matrix; the vectors its rows produce are put together again with an in-place all-gather
// (4 per layer: attention output, x after wo, SwiGLU output, x after w2).  Results are bit-identical
// on all ranks and identical to the single-GPU run, because no sum is split across ranks.
//
// NCCL is opened with dlopen at first use: a process that already loaded a libnccl.so.2 (for
// example through torch) shares that copy, and a single-GPU user never needs the library.
#include <dlfcn.h>

#include <cstring>

#include "model.h"

namespace l2 {

namespace {
typedef int (*fn_get_unique_id)(void*);
typedef int (*fn_comm_init_rank)(void**, int, NcclId, int);
typedef int (*fn_all_gather)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*fn_comm_destroy)(void*);
typedef const char* (*fn_error_string)(int);
struct Api {
    void* lib = nullptr;
    fn_get_unique_id get_unique_id = nullptr;
    fn_comm_init_rank comm_init_rank = nullptr;
    fn_all_gather all_gather = nullptr;
    fn_comm_destroy comm_destroy = nullptr;
    fn_error_string error_string = nullptr;
} api;

int load_api() {
    if (api.lib) return L2_OK;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail(L2_ECUDA, "cannot load libnccl.so.2: %s", dlerror());
    api.get_unique_id = (fn_get_unique_id)dlsym(h, "ncclGetUniqueId");
    api.comm_init_rank = (fn_comm_init_rank)dlsym(h, "ncclCommInitRank");
    api.all_gather = (fn_all_gather)dlsym(h, "ncclAllGather");
    api.comm_destroy = (fn_comm_destroy)dlsym(h, "ncclCommDestroy");
    api.error_string = (fn_error_string)dlsym(h, "ncclGetErrorString");
    if (!api.get_unique_id || !api.comm_init_rank || !api.all_gather || !api.comm_destroy)
        return fail(L2_ECUDA, "libnccl.so.2 lacks an expected symbol");
    api.lib = h;
    return L2_OK;
}
const char* err(int rc) { return api.error_string ? api.error_string(rc) : "nccl error"; }
}  // namespace

// In-place all-gather of `count` floats per rank: rank r's part sits at buf + r * count.
int tp_all_gather(l2_model* m, float* buf, size_t count, cudaStream_t st) {
    if (m->tp_world == 1) return L2_OK;
    if (!m->nccl_comm) return fail(L2_EINVAL, "tensor-parallel model used before l2_model_tp_connect");
    const int rc = api.all_gather(buf + (size_t)m->tp_rank * count, buf, count, 7 /* ncclFloat32 */, m->nccl_comm, st);
    if (rc != 0) return fail(L2_ECUDA, "ncclAllGather: %s", err(rc));
    return L2_OK;
}

void tp_disconnect(l2_model* m) {
    if (m->nccl_comm && api.comm_destroy) api.comm_destroy(m->nccl_comm);
    m->nccl_comm = nullptr;
}

void tp_rows(int total_rows, int rank, int world, int* row0, int* nrows) {
    const int per = total_rows / world;
    *row0 = rank * per;
    *nrows = per;
}

}  // namespace l2

using namespace l2;

extern "C" int l2_tp_unique_id(void* id128) {
    clear_error();
    if (!id128) return fail(L2_EINVAL, "l2_tp_unique_id: null argument");
    if (int rc = load_api()) return rc;
    NcclId id;
    const int rc = api.get_unique_id(&id);
    if (rc != 0) return fail(L2_ECUDA, "ncclGetUniqueId: %s", err(rc));
    memcpy(id128, &id, sizeof id);
    return L2_OK;
}

extern "C" int l2_model_tp_connect(l2_model* m, const void* id128) {
    clear_error();
    if (!m || !id128) return fail(L2_EINVAL, "l2_model_tp_connect: null argument");
    if (m->tp_world == 1) return L2_OK;
    if (int rc = load_api()) return rc;
    L2_CUDA(cudaSetDevice(m->device));
    NcclId id;
    memcpy(&id, id128, sizeof id);
    void* comm = nullptr;
    const int rc = api.comm_init_rank(&comm, m->tp_world, id, m->tp_rank);
    if (rc != 0) return fail(L2_ECUDA, "ncclCommInitRank: %s", err(rc));
    m->nccl_comm = comm;
    return L2_OK;
}

extern "C" int l2_tp_rows(int total_rows, int rank, int world, int* row0, int* nrows) {
    if (!row0 || !nrows || world < 1 || rank < 0 || rank >= world || total_rows % (16 * world))
        return fail(L2_EINVAL, "l2_tp_rows: %d rows cannot be cut into %d parts of whole 16-row tiles", total_rows, world);
    tp_rows(total_rows, rank, world, row0, nrows);
    return L2_OK;
}
