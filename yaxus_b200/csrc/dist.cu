// Long-context decode with the keys split across GPUs: every rank computes the (m, l, o)
// triples of its own page range, the triples are exchanged with one NCCL all-gather over
// NVLink, and every rank merges them with the log-sum-exp combine.  The reference has no
// multi-GPU path; the triple format is the one its split attention already uses
// (crates/yaxus-backend-gpu/src/shaders.rs:1466-1637).
//
// NCCL is loaded at run time (dlopen) so that the library itself has no link-time dependency
// on it; a process that already loaded a libnccl.so.2 (PyTorch's) shares that copy.
#include <dlfcn.h>
#include <string.h>

#include "yx_internal.h"

namespace yx {
namespace {

typedef struct { char internal[128]; } nccl_id;
typedef int (*fn_get_id)(nccl_id *);
typedef int (*fn_init_rank)(ncclComm **, int, nccl_id, int);
typedef int (*fn_destroy)(ncclComm *);
typedef int (*fn_all_gather)(const void *, void *, size_t, int, ncclComm *, cudaStream_t);
typedef const char *(*fn_err)(int);
constexpr int NCCL_FLOAT32 = 7;

struct Nccl {
    void *lib = nullptr;
    fn_get_id get_id = nullptr;
    fn_init_rank init_rank = nullptr;
    fn_destroy destroy = nullptr;
    fn_all_gather all_gather = nullptr;
    fn_err err = nullptr;
    bool ok = false;
};

Nccl &nccl() {
    static Nccl n;
    if (n.lib) return n;
    n.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!n.lib) n.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!n.lib) return n;
    n.get_id = (fn_get_id)dlsym(n.lib, "ncclGetUniqueId");
    n.init_rank = (fn_init_rank)dlsym(n.lib, "ncclCommInitRank");
    n.destroy = (fn_destroy)dlsym(n.lib, "ncclCommDestroy");
    n.all_gather = (fn_all_gather)dlsym(n.lib, "ncclAllGather");
    n.err = (fn_err)dlsym(n.lib, "ncclGetErrorString");
    n.ok = n.get_id && n.init_rank && n.destroy && n.all_gather && n.err;
    return n;
}

int nccl_fail(yx_ctx *ctx, int rc, const char *what) {
    Nccl &n = nccl();
    return fail(ctx, YX_ERR_NCCL, std::string(what) + ": " + (n.err ? n.err(rc) : "NCCL error"));
}

}  // namespace
}  // namespace yx

using namespace yx;

extern "C" {

int yx_comm_unique_id(void *out_id128) {
    if (!out_id128) return YX_ERR_INVALID;
    Nccl &n = nccl();
    if (!n.ok) return YX_ERR_NCCL;
    nccl_id id;
    memset(&id, 0, sizeof id);
    if (n.get_id(&id) != 0) return YX_ERR_NCCL;
    memcpy(out_id128, &id, sizeof id);
    return YX_OK;
}

int yx_comm_create(yx_ctx *ctx, int n_ranks, int rank, const void *id128) {
    if (!ctx) return YX_ERR_INVALID;
    if (n_ranks < 1 || rank < 0 || rank >= n_ranks) return fail(ctx, YX_ERR_INVALID, "comm_create: bad rank");
    if (ctx->comm) return fail(ctx, YX_ERR_STATE, "comm_create: the context already has a communicator");
    ctx->n_ranks = n_ranks;
    ctx->rank = rank;
    if (n_ranks == 1) return YX_OK;   // nothing to exchange
    if (!id128) return fail(ctx, YX_ERR_INVALID, "comm_create: null id");
    Nccl &n = nccl();
    if (!n.ok) return fail(ctx, YX_ERR_NCCL, "comm_create: libnccl.so.2 could not be loaded");
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(ctx->device);
    nccl_id id;
    memcpy(&id, id128, sizeof id);
    int rc = n.init_rank(&ctx->comm, n_ranks, id, rank);
    if (prev >= 0 && prev != ctx->device) cudaSetDevice(prev);
    if (rc != 0) {
        ctx->comm = nullptr;
        return nccl_fail(ctx, rc, "ncclCommInitRank");
    }
    return YX_OK;
}

int yx_comm_destroy(yx_ctx *ctx) {
    if (!ctx) return YX_ERR_INVALID;
    if (ctx->comm) {
        Nccl &n = nccl();
        if (n.ok) n.destroy(ctx->comm);
        ctx->comm = nullptr;
    }
    ctx->n_ranks = 1;
    ctx->rank = 0;
    return YX_OK;
}

int yx_attend_allgather(yx_ctx *ctx, yx_kv *kv, int layer, const void *q, int q_dtype, int hq, int64_t window,
                        uint64_t key_lo, uint64_t key_hi, void *out, int out_dtype) {
    if (!ctx || !kv) return YX_ERR_INVALID;
    if (ctx->status != YX_OK) return ctx->status;
    if (!ctx->have_pass) return fail(ctx, YX_ERR_STATE, "attention without begin_pass");
    if (!out) return fail(ctx, YX_ERR_INVALID, "null tensor");
    if (ctx->n_ranks > 1 && !ctx->comm) return fail(ctx, YX_ERR_STATE, "attend_allgather without a communicator");
    const size_t n = (size_t)ctx->pass.rows * hq;
    if (n == 0) return YX_OK;
    // One rank has nothing to exchange: the split-key kernel's merge writes the output itself.
    if (ctx->n_ranks <= 1) return attend_key_range(ctx, kv, layer, q, q_dtype, hq, window, key_lo, key_hi, out, out_dtype);
    const size_t block = n * (D + 2);   // floats per rank: m | l | o
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(ctx->device);
    int rc = ensure_buffer(ctx, (void **)&ctx->gather_buf, &ctx->gather_cap, block * sizeof(float) * (ctx->n_ranks + 1));
    float *mine = ctx->gather_buf;                 // this rank's block
    float *all = ctx->gather_buf + block;          // [rank][block]
    if (!rc) rc = yx_attend_partial(ctx, kv, layer, q, q_dtype, hq, window, key_lo, key_hi, mine, mine + n, mine + 2 * n);
    int launches = ctx->last_plan.launches;
    if (!rc) {
        if (ctx->n_ranks > 1) {
            int e = nccl().all_gather(mine, all, block, NCCL_FLOAT32, ctx->comm, ctx->stream);
            if (e != 0) rc = nccl_fail(ctx, e, "ncclAllGather");
            launches++;
        } else {
            all = mine;
        }
    }
    if (!rc) rc = launch_combine_strided(ctx, ctx->n_ranks, all, all + n, all + 2 * n, block, block, block, n, out, out_dtype);
    ctx->last_plan.launches = launches + 1;
    if (prev >= 0 && prev != ctx->device) cudaSetDevice(prev);
    return rc;
}

}  // extern "C"
