// NCCL communicator: the B200 stand-in for the reference's HCCL transport
// (rust-ascend-driver/src/tensor/runtime/hccl.rs:79-85,133-307,386-548).
//
// Like the reference, the collective library is loaded at run time (dlopen, never linked): RUDA_NCCL_LIBRARY or
// "libnccl.so.2".  One process drives one GPU; the 128-byte ncclUniqueId plays the role of HcclRootInfo and
// travels over the caller's control plane.  Collectives run on the communicator's own stream: each call first
// makes that stream wait for everything already enqueued on the context's compute stream, and, unless the caller
// asks for a deferred fence, makes the compute stream wait for the collective.  With deferred fences a caller can
// keep issuing GEMMs for the next row chunk while the all-reduce of the previous chunk crosses NVLink.
#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>

#include "common.cuh"

namespace {

struct NcclApi {
    void* library = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*GetVersion)(int*) = nullptr;
};

NcclApi g_api;

int32_t load_api() {
    if (g_api.library) return RB_OK;
    const char* name = getenv("RUDA_NCCL_LIBRARY");
    if (!name || !*name) name = "libnccl.so.2";
    void* lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
    if (!lib) return rb::fail(RB_LIBRARY, "cannot load the NCCL library '%s': %s", name, dlerror());
#define RB_SYM(field, symbol) \
    *reinterpret_cast<void**>(&g_api.field) = dlsym(lib, symbol); \
    if (!g_api.field) { dlclose(lib); return rb::fail(RB_SYMBOL, "NCCL library '%s' lacks symbol %s", name, symbol); }
    RB_SYM(GetUniqueId, "ncclGetUniqueId") RB_SYM(CommInitRank, "ncclCommInitRank") RB_SYM(CommDestroy, "ncclCommDestroy")
    RB_SYM(CommAbort, "ncclCommAbort") RB_SYM(CommGetAsyncError, "ncclCommGetAsyncError") RB_SYM(AllReduce, "ncclAllReduce")
    RB_SYM(Broadcast, "ncclBroadcast") RB_SYM(AllGather, "ncclAllGather") RB_SYM(ReduceScatter, "ncclReduceScatter")
    RB_SYM(GetErrorString, "ncclGetErrorString") RB_SYM(GetVersion, "ncclGetVersion")
#undef RB_SYM
    *reinterpret_cast<void**>(&g_api.CommInitRankConfig) = dlsym(lib, "ncclCommInitRankConfig");  // optional
    g_api.library = lib;
    return RB_OK;
}

int32_t nccl_fail(const char* operation, ncclResult_t r) {
    return rb::fail(RB_STATUS, "%s failed with NCCL status %d (%s)", operation, (int)r, g_api.GetErrorString ? g_api.GetErrorString(r) : "?");
}

// hccl.rs:97-111 accepts F32/F16/BF16/I32/I64 and bytes.
int32_t nccl_dtype(uint32_t dtype, ncclDataType_t* out) {
    switch (dtype) {
        case RB_F32: *out = ncclFloat32; return RB_OK;
        case RB_F16: *out = ncclFloat16; return RB_OK;
        case RB_BF16: *out = ncclBfloat16; return RB_OK;
        case RB_I32: *out = ncclInt32; return RB_OK;
        case RB_I64: *out = ncclInt64; return RB_OK;
        case RB_U8: *out = ncclUint8; return RB_OK;
        default: return rb::fail(RB_INVALID_TENSOR, "NCCL tensor requires FP32/FP16/BF16/I32/I64 or bytes");
    }
}
int32_t nccl_op(int32_t op, ncclRedOp_t* out) {
    switch (op) {
        case RB_SUM: *out = ncclSum; return RB_OK;
        case RB_PROD: *out = ncclProd; return RB_OK;
        case RB_MAX: *out = ncclMax; return RB_OK;
        case RB_MIN: *out = ncclMin; return RB_OK;
        default: return rb::fail(RB_INVALID_TENSOR, "unknown reduction");
    }
}

}  // namespace

struct rb_comm {
    rb_ctx* ctx = nullptr;
    ncclComm_t comm = nullptr;
    uint32_t rank = 0, world = 1;
    cudaStream_t stream = nullptr;
    cudaEvent_t before = nullptr, after = nullptr;
    static constexpr int TICKETS = 32;
    cudaEvent_t done[TICKETS] = {};   // completion event of collective number n lives in slot n % TICKETS
    uint64_t issued = 0;              // collectives issued so far; the ticket of the latest one
    bool poisoned = false;
};

using namespace rb;

namespace {

int32_t check_comm(rb_comm* c) {
    if (!c || !c->comm) return fail(RB_NULL_HANDLE, "null communicator");
    if (c->poisoned) return fail(RB_SERVER_UNHEALTHY, "communicator is poisoned by an earlier failed collective");
    return check_ctx(c->ctx);
}

// Orders the collective after the compute stream's earlier work.
int32_t enter(rb_comm* c) {
    RB_CUDA(c->ctx, "cudaEventRecord", cudaEventRecord(c->before, c->ctx->stream));
    RB_CUDA(c->ctx, "cudaStreamWaitEvent", cudaStreamWaitEvent(c->stream, c->before, 0));
    return RB_OK;
}
// Orders later compute after the collective unless the caller defers the fence to rb_comm_fence.
int32_t leave(rb_comm* c, const char* operation, ncclResult_t r, int32_t deferred) {
    c->ctx->stats.launches++;
    if (r != ncclSuccess) { c->poisoned = true; return nccl_fail(operation, r); }
    RB_CUDA(c->ctx, "cudaEventRecord", cudaEventRecord(c->after, c->stream));
    c->issued++;
    RB_CUDA(c->ctx, "cudaEventRecord", cudaEventRecord(c->done[c->issued % rb_comm::TICKETS], c->stream));
    if (!deferred) RB_CUDA(c->ctx, "cudaStreamWaitEvent", cudaStreamWaitEvent(c->ctx->stream, c->after, 0));
    if (c->ctx->synchronous) {  // the reference synchronises after every collective (hccl.rs:290-305)
        c->ctx->stats.synchronizations++;
        cudaError_t e = cudaStreamSynchronize(c->stream);
        if (e != cudaSuccess) { c->poisoned = true; return fail(RB_COMPLETION, "%s completion failed with CUDA status %d (%s)", operation, (int)e, cudaGetErrorString(e)); }
    }
    return RB_OK;
}

}  // namespace

extern "C" {

int32_t rb_comm_unique_id(uint8_t* id_128_bytes) {
    if (!id_128_bytes) return fail(RB_NULL_HANDLE, "null id buffer");
    RB_TRY(load_api());
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
    ncclUniqueId id;
    ncclResult_t r = g_api.GetUniqueId(&id);
    if (r != ncclSuccess) return nccl_fail("ncclGetUniqueId", r);
    memcpy(id_128_bytes, &id, 128);
    return RB_OK;
}

int32_t rb_comm_init(rb_ctx* ctx, const uint8_t* id_128_bytes, uint32_t rank, uint32_t world_size, rb_comm** out) {
    RB_TRY(check_ctx(ctx));
    if (!id_128_bytes || !out) return fail(RB_NULL_HANDLE, "null pointer");
    if (world_size == 0 || rank >= world_size) return fail(RB_INVALID_TENSOR, "rank %u is outside a world of %u", rank, world_size);
    RB_TRY(load_api());
    RB_CUDA(ctx, "cudaSetDevice", cudaSetDevice(ctx->device));
    ncclUniqueId id; memcpy(&id, id_128_bytes, 128);
    rb_comm* c = new rb_comm();
    c->ctx = ctx; c->rank = rank; c->world = world_size;
    // RUDA_NCCL_MAX_CTAS bounds the SMs a collective may occupy, so that it can run beside a GEMM that leaves
    // that many SMs free (rb_set_sm_limit).
    const char* max_ctas = getenv("RUDA_NCCL_MAX_CTAS");
    ncclResult_t r;
    if (max_ctas && atoi(max_ctas) > 0 && g_api.CommInitRankConfig) {
        ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
        config.maxCTAs = atoi(max_ctas);
        config.minCTAs = 1;
        r = g_api.CommInitRankConfig(&c->comm, (int)world_size, id, (int)rank, &config);
    } else {
        r = g_api.CommInitRank(&c->comm, (int)world_size, id, (int)rank);
    }
    if (r != ncclSuccess) { delete c; return nccl_fail("ncclCommInitRank", r); }
    // Highest priority: when an SM frees up, a waiting collective block is placed before a compute block.
    int least = 0, greatest = 0;
    cudaDeviceGetStreamPriorityRange(&least, &greatest);
    cudaError_t e = cudaStreamCreateWithPriority(&c->stream, cudaStreamNonBlocking, greatest);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->before, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->after, cudaEventDisableTiming);
    for (int i = 0; e == cudaSuccess && i < rb_comm::TICKETS; ++i) e = cudaEventCreateWithFlags(&c->done[i], cudaEventDisableTiming);
    if (e != cudaSuccess) { g_api.CommAbort(c->comm); delete c; return fail(RB_STATUS, "communicator stream/event creation failed with CUDA status %d", (int)e); }
    *out = c;
    return RB_OK;
}

int32_t rb_comm_destroy(rb_comm* c) {
    if (!c) return fail(RB_NULL_HANDLE, "null communicator");
    // Drain first; if the work cannot be drained the communicator is aborted and its objects are leaked rather than
    // destroyed under running kernels (hccl.rs:119-131).
    bool drained = cudaStreamSynchronize(c->stream) == cudaSuccess && !c->poisoned;
    // Recorded graphs may hold collectives of this communicator, and NCCL does not finish destroying a communicator
    // while such a graph exists: drop every graph of the context first.
    {
        std::lock_guard<std::mutex> lk(c->ctx->lock);
        for (auto& kv : c->ctx->graphs) cudaGraphExecDestroy(kv.second);
        c->ctx->graphs.clear();
    }
    if (drained) {
        g_api.CommDestroy(c->comm);
        cudaEventDestroy(c->before); cudaEventDestroy(c->after);
        for (int i = 0; i < rb_comm::TICKETS; ++i) if (c->done[i]) cudaEventDestroy(c->done[i]);
        cudaStreamDestroy(c->stream);
    } else if (c->comm) {
        g_api.CommAbort(c->comm);
    }
    delete c;
    return RB_OK;
}

int32_t rb_comm_info(rb_comm* c, uint32_t* rank, uint32_t* world_size, int32_t* nccl_version) {
    if (!c) return fail(RB_NULL_HANDLE, "null communicator");
    if (rank) *rank = c->rank;
    if (world_size) *world_size = c->world;
    if (nccl_version) { int v = 0; g_api.GetVersion(&v); *nccl_version = v; }
    return RB_OK;
}

int32_t rb_comm_fence(rb_comm* c) {
    RB_TRY(check_comm(c));
    RB_CUDA(c->ctx, "cudaStreamWaitEvent", cudaStreamWaitEvent(c->ctx->stream, c->after, 0));
    ncclResult_t async = ncclSuccess;
    ncclResult_t r = g_api.CommGetAsyncError(c->comm, &async);
    if (r != ncclSuccess || async != ncclSuccess) { c->poisoned = true; return nccl_fail("asynchronous NCCL error", r != ncclSuccess ? r : async); }
    return RB_OK;
}

int32_t rb_comm_ticket(rb_comm* c, uint64_t* ticket) {
    if (!c || !ticket) return fail(RB_NULL_HANDLE, "null pointer");
    *ticket = c->issued;
    return RB_OK;
}

int32_t rb_comm_wait_ticket(rb_comm* c, uint64_t ticket) {
    RB_TRY(check_comm(c));
    if (ticket == 0) return RB_OK;
    if (ticket > c->issued) return fail(RB_INVALID_TENSOR, "ticket %llu has not been issued", (unsigned long long)ticket);
    // Events are recycled after TICKETS further collectives; an older ticket is already covered by a newer one in
    // the same slot because collectives of one communicator complete in issue order.
    RB_CUDA(c->ctx, "cudaStreamWaitEvent", cudaStreamWaitEvent(c->ctx->stream, c->done[ticket % rb_comm::TICKETS], 0));
    return RB_OK;
}

int32_t rb_all_reduce(rb_comm* c, const rb_tensor* in, int32_t op, const rb_tensor* out, int32_t deferred_fence) {
    RB_TRY(check_comm(c));
    void *pi, *po; ncclDataType_t dt; ncclRedOp_t ro;
    RB_TRY(resolve(c->ctx, in, "all_reduce input", &pi)); RB_TRY(resolve(c->ctx, out, "all_reduce output", &po));
    if (!same_shape(in, out) || in->dtype != out->dtype) return fail(RB_INVALID_TENSOR, "all_reduce output must match the input shape and dtype");
    RB_TRY(nccl_dtype(in->dtype, &dt)); RB_TRY(nccl_op(op, &ro));
    if (in->dtype == RB_U8) return fail(RB_INVALID_TENSOR, "all_reduce requires a numeric dtype");
    uint64_t n = elements(in);
    if (pi != po) RB_TRY(no_overlap(po, n * dtype_size(out->dtype), pi, n * dtype_size(in->dtype), "all_reduce"));
    if (n == 0) return empty_call(c->ctx);
    RB_TRY(enter(c));
    return leave(c, "ncclAllReduce", g_api.AllReduce(pi, po, n, dt, ro, c->comm, c->stream), deferred_fence);
}

int32_t rb_broadcast(rb_comm* c, const rb_tensor* in, uint32_t root, const rb_tensor* out) {
    RB_TRY(check_comm(c));
    if (root >= c->world) return fail(RB_INVALID_TENSOR, "broadcast root is outside the world");
    void *pi, *po; ncclDataType_t dt;
    RB_TRY(resolve(c->ctx, in, "broadcast input", &pi)); RB_TRY(resolve(c->ctx, out, "broadcast output", &po));
    if (!same_shape(in, out) || in->dtype != out->dtype) return fail(RB_INVALID_TENSOR, "broadcast output must match the input shape and dtype");
    RB_TRY(nccl_dtype(in->dtype, &dt));
    uint64_t n = elements(in);
    if (n == 0) return empty_call(c->ctx);
    RB_TRY(enter(c));
    return leave(c, "ncclBroadcast", g_api.Broadcast(pi, po, n, dt, (int)root, c->comm, c->stream), 0);
}

int32_t rb_all_gather(rb_comm* c, const rb_tensor* in, const rb_tensor* out) {
    RB_TRY(check_comm(c));
    void *pi, *po; ncclDataType_t dt;
    RB_TRY(resolve(c->ctx, in, "all_gather input", &pi)); RB_TRY(resolve(c->ctx, out, "all_gather output", &po));
    RB_TRY(nccl_dtype(in->dtype, &dt));
    // Rank-ordered concatenation along the leading axis (hccl.rs:398-422).
    bool ok = in->rank == out->rank && in->dtype == out->dtype && out->shape[0] == in->shape[0] * c->world;
    for (uint32_t i = 1; ok && i < in->rank; ++i) ok = in->shape[i] == out->shape[i];
    if (!ok) return fail(RB_INVALID_TENSOR, "all_gather output must be the input with its leading axis multiplied by the world size");
    uint64_t n = elements(in);
    RB_TRY(no_overlap(po, n * c->world * dtype_size(out->dtype), pi, n * dtype_size(in->dtype), "all_gather"));
    if (n == 0) return empty_call(c->ctx);
    RB_TRY(enter(c));
    return leave(c, "ncclAllGather", g_api.AllGather(pi, po, n, dt, c->comm, c->stream), 0);
}

int32_t rb_reduce_scatter(rb_comm* c, const rb_tensor* in, int32_t op, const rb_tensor* out) {
    RB_TRY(check_comm(c));
    void *pi, *po; ncclDataType_t dt; ncclRedOp_t ro;
    RB_TRY(resolve(c->ctx, in, "reduce_scatter input", &pi)); RB_TRY(resolve(c->ctx, out, "reduce_scatter output", &po));
    RB_TRY(nccl_dtype(in->dtype, &dt)); RB_TRY(nccl_op(op, &ro));
    if (in->dtype == RB_U8) return fail(RB_INVALID_TENSOR, "reduce_scatter requires a numeric dtype");
    bool ok = in->rank == out->rank && in->dtype == out->dtype && in->shape[0] % c->world == 0 && out->shape[0] == in->shape[0] / c->world;
    for (uint32_t i = 1; ok && i < in->rank; ++i) ok = in->shape[i] == out->shape[i];
    if (!ok) return fail(RB_INVALID_TENSOR, "reduce_scatter needs a leading axis divisible by the world size and an output holding one shard");
    uint64_t n = elements(out);
    RB_TRY(no_overlap(po, n * dtype_size(out->dtype), pi, n * c->world * dtype_size(in->dtype), "reduce_scatter"));
    if (n == 0) return empty_call(c->ctx);
    RB_TRY(enter(c));
    return leave(c, "ncclReduceScatter", g_api.ReduceScatter(pi, po, n, dt, ro, c->comm, c->stream), 0);
}

// Row-parallel Linear followed by all-reduce(sum) in one call: out [T, H] = sum over ranks of x_r [T, K/world] w_r [H, K/world]^T.
// overlap_mode 0: one GEMM, one all-reduce.  overlap_mode 1: the rows are cut into up to four chunks of whole 128-row tiles;
// the all-reduce of chunk i runs on the communicator's stream while the GEMM of chunk i+1 runs on the compute stream
// (deferred fences), and later compute is ordered after the last chunk.
int32_t rb_row_parallel_linear_allreduce(rb_comm* c, const rb_tensor* x, const rb_tensor* w_shard, const rb_tensor* out, int32_t overlap_mode) {
    RB_TRY(check_comm(c));
    if (!x || !w_shard || !out) return fail(RB_NULL_HANDLE, "null tensor");
    if (overlap_mode != 0 && overlap_mode != 1) return fail(RB_INVALID_TENSOR, "overlap mode is 0 (sequential) or 1 (row chunks)");
    if (x->rank != 2 || w_shard->rank != 2 || out->rank != 2 || out->shape[0] != x->shape[0] || out->shape[1] != w_shard->shape[0] || x->shape[1] != w_shard->shape[1])
        return fail(RB_INVALID_TENSOR, "row-parallel linear takes x [T, K/world], w [H, K/world] and out [T, H]");
    const uint64_t rows = x->shape[0], k = x->shape[1], n = out->shape[1];
    uint64_t chunks = 1;
    if (overlap_mode == 1 && c->world > 1) {
        const uint64_t tiles = rows / 128;
        chunks = tiles >= 4 && rows % 128 == 0 ? 4 : (tiles >= 2 && rows % 128 == 0 ? 2 : 1);
        while (chunks > 1 && tiles % chunks) chunks /= 2;
    }
    const uint64_t chunk_rows = rows / chunks;
    for (uint64_t i = 0; i < chunks; ++i) {
        rb_tensor xi = *x, oi = *out;
        xi.shape[0] = chunk_rows; xi.offset = x->offset + i * chunk_rows * k * dtype_size(x->dtype);
        oi.shape[0] = chunk_rows; oi.offset = out->offset + i * chunk_rows * n * dtype_size(out->dtype);
        RB_TRY(rb_gemm(c->ctx, &xi, w_shard, RB_NO_TRANSPOSE, RB_TRANSPOSE, nullptr, nullptr, RB_EPILOGUE_NONE, &oi));
        RB_TRY(rb_all_reduce(c, &oi, RB_SUM, &oi, chunks > 1 ? 1 : 0));
    }
    if (chunks > 1) RB_TRY(rb_comm_fence(c));
    return RB_OK;
}

}  // extern "C"
