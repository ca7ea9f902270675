// Peer memory between the processes of one node: a storage of this process is exported as an opaque 64-byte token, the
// other ranks open the token and get a storage handle whose device address is the exporter's memory reached over NVLink.
// The fused tensor-parallel kernels (fused_tp.cu) store partial tiles and flags straight into such memory.
//
// The reference has no counterpart: its collectives always go through the vendor library (runtime/hccl.rs:386-548).
// Tokens travel over the same control plane that carries the communicator's root id (src/distributed.rs:74-110).
#include "common.cuh"

#include <map>

namespace {

struct Opened { void* base; };
std::mutex g_lock;
std::map<std::pair<rb_ctx*, uint64_t>, Opened> g_opened;   // storage handles that came from rb_peer_open

static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the exported token is a 64-byte IPC handle");

}  // namespace

using namespace rb;

extern "C" {

int32_t rb_peer_export(rb_ctx* ctx, uint64_t handle, uint8_t token[64]) {
    RB_TRY(check_ctx(ctx));
    if (!token) return fail(RB_NULL_HANDLE, "null token buffer");
    void* p = nullptr; uint64_t bytes = 0;
    RB_TRY(rb_resource(ctx, handle, &p, &bytes));
    {
        std::lock_guard<std::mutex> g(g_lock);
        if (g_opened.count({ctx, handle})) return fail(RB_INVALID_TENSOR, "a storage opened from another rank cannot be exported again");
    }
    cudaIpcMemHandle_t h;
    RB_CUDA(ctx, "cudaIpcGetMemHandle", cudaIpcGetMemHandle(&h, p));
    std::memcpy(token, &h, 64);
    return RB_OK;
}

int32_t rb_peer_open(rb_ctx* ctx, const uint8_t token[64], uint64_t bytes, uint64_t* handle) {
    RB_TRY(check_ctx(ctx));
    if (!token || !handle) return fail(RB_NULL_HANDLE, "null token or handle pointer");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, token, 64);
    void* p = nullptr;
    RB_CUDA(ctx, "cudaIpcOpenMemHandle", cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    int32_t rc = rb_import(ctx, p, bytes, handle);
    if (rc != RB_OK) { cudaIpcCloseMemHandle(p); return rc; }
    std::lock_guard<std::mutex> g(g_lock);
    g_opened[{ctx, *handle}] = Opened{p};
    return RB_OK;
}

int32_t rb_peer_close(rb_ctx* ctx, uint64_t handle) {
    RB_TRY(check_ctx(ctx));
    Opened o{};
    {
        std::lock_guard<std::mutex> g(g_lock);
        auto it = g_opened.find({ctx, handle});
        if (it == g_opened.end()) return fail(RB_NULL_HANDLE, "storage handle %llu was not opened from a peer token", (unsigned long long)handle);
        o = it->second;
        g_opened.erase(it);
    }
    RB_TRY(rb_sync(ctx));                         // nothing of this process may still be writing through the mapping
    RB_TRY(rb_free(ctx, handle));                 // drops the table entry; the memory belongs to the exporter
    RB_CUDA(ctx, "cudaIpcCloseMemHandle", cudaIpcCloseMemHandle(o.base));
    return RB_OK;
}

}  // extern "C"
