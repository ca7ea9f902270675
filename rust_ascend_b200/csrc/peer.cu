// Peer memory between the processes of one node: a storage of this process is exported as an opaque token, the other ranks
// open the token and get a storage handle whose device address is the exporter's memory reached over NVLink.  The fused
// tensor-parallel kernels (fused_tp.cu) store partial tiles and flags straight into such memory.
//
// The reference has no counterpart: its collectives always go through the vendor library (runtime/hccl.rs:386-548).
// Tokens travel over the same control plane that carries the communicator's root id (src/distributed.rs:74-110).
//
// A CUDA IPC handle names a whole cudaMalloc allocation, and the allocator may carve several small storages out of one
// allocation.  So a token is the allocation's IPC handle plus the storage's byte offset inside it, and an allocation that
// several tokens name is mapped once per process and reference-counted (mapping it twice is an error in CUDA IPC).
#include "common.cuh"

#include <cuda.h>

#include <map>

namespace {

constexpr size_t HANDLE_BYTES = sizeof(cudaIpcMemHandle_t);
static_assert(HANDLE_BYTES == 64 && RB_PEER_TOKEN_BYTES == HANDLE_BYTES + 16, "token = 64-byte IPC handle + 8-byte offset + 8-byte length");

struct Mapping { void* base = nullptr; int refs = 0; };
struct Opened { std::string key; };
std::mutex g_lock;
std::map<std::string, Mapping> g_mappings;                        // IPC handle bytes -> mapped allocation
std::map<std::pair<rb_ctx*, uint64_t>, Opened> g_opened;           // storage handles that came from rb_peer_open

typedef CUresult (*AddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
AddressRangeFn address_range_fn() {
    static AddressRangeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return (AddressRangeFn)p;
    }();
    return fn;
}

}  // namespace

using namespace rb;

extern "C" {

int32_t rb_peer_export(rb_ctx* ctx, uint64_t handle, uint8_t token[RB_PEER_TOKEN_BYTES]) {
    RB_TRY(check_ctx(ctx));
    if (!token) return fail(RB_NULL_HANDLE, "null token buffer");
    void* p = nullptr; uint64_t bytes = 0;
    RB_TRY(rb_resource(ctx, handle, &p, &bytes));
    {
        std::lock_guard<std::mutex> g(g_lock);
        if (g_opened.count({ctx, handle})) return fail(RB_INVALID_TENSOR, "a storage opened from another rank cannot be exported again");
    }
    AddressRangeFn range = address_range_fn();
    if (!range) return fail(RB_SYMBOL, "cuMemGetAddressRange is not available from the driver");
    CUdeviceptr base = 0; size_t span = 0;
    CUresult r = range(&base, &span, (CUdeviceptr)(uintptr_t)p);
    if (r != CUDA_SUCCESS) return fail(RB_STATUS, "cuMemGetAddressRange failed with driver status %d", (int)r);
    cudaIpcMemHandle_t h;
    RB_CUDA(ctx, "cudaIpcGetMemHandle", cudaIpcGetMemHandle(&h, (void*)(uintptr_t)base));
    const uint64_t offset = (uint64_t)((uintptr_t)p - (uintptr_t)base);
    std::memcpy(token, &h, HANDLE_BYTES);
    std::memcpy(token + HANDLE_BYTES, &offset, 8);
    std::memcpy(token + HANDLE_BYTES + 8, &bytes, 8);        // the opener may not claim more than the exporter owns
    return RB_OK;
}

int32_t rb_peer_open(rb_ctx* ctx, const uint8_t token[RB_PEER_TOKEN_BYTES], uint64_t bytes, uint64_t* handle) {
    RB_TRY(check_ctx(ctx));
    if (!token || !handle) return fail(RB_NULL_HANDLE, "null token or handle pointer");
    cudaIpcMemHandle_t h;
    uint64_t offset = 0;
    std::memcpy(&h, token, HANDLE_BYTES);
    std::memcpy(&offset, token + HANDLE_BYTES, 8);
    uint64_t exported = 0;
    std::memcpy(&exported, token + HANDLE_BYTES + 8, 8);
    if (bytes > exported) return fail(RB_INVALID_TENSOR, "the token names a storage of %llu bytes; %llu were asked for", (unsigned long long)exported, (unsigned long long)bytes);
    const std::string key(reinterpret_cast<const char*>(token), HANDLE_BYTES);
    std::lock_guard<std::mutex> g(g_lock);
    Mapping& m = g_mappings[key];
    if (m.refs == 0) {
        void* base = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            g_mappings.erase(key);
            return fail(RB_STATUS, "cudaIpcOpenMemHandle failed with CUDA status %d (%s)", (int)e, cudaGetErrorString(e));
        }
        m.base = base;
    }
    int32_t rc = rb_import(ctx, static_cast<uint8_t*>(m.base) + offset, bytes, handle);
    if (rc != RB_OK) {
        if (m.refs == 0) { cudaIpcCloseMemHandle(m.base); g_mappings.erase(key); }
        return rc;
    }
    ++m.refs;
    g_opened[{ctx, *handle}] = Opened{key};
    return RB_OK;
}

int32_t rb_peer_close(rb_ctx* ctx, uint64_t handle) {
    RB_TRY(check_ctx(ctx));
    {
        std::lock_guard<std::mutex> g(g_lock);
        if (!g_opened.count({ctx, handle})) return fail(RB_NULL_HANDLE, "storage handle %llu was not opened from a peer token", (unsigned long long)handle);
    }
    RB_TRY(rb_sync(ctx));                         // nothing of this process may still be writing through the mapping
    RB_TRY(rb_free(ctx, handle));                 // drops the table entry; the memory belongs to the exporter
    std::lock_guard<std::mutex> g(g_lock);
    auto it = g_opened.find({ctx, handle});
    const std::string key = it->second.key;
    g_opened.erase(it);
    auto mi = g_mappings.find(key);
    if (mi != g_mappings.end() && --mi->second.refs == 0) {
        cudaError_t e = cudaIpcCloseMemHandle(mi->second.base);
        g_mappings.erase(mi);
        if (e != cudaSuccess) return fail(RB_STATUS, "cudaIpcCloseMemHandle failed with CUDA status %d (%s)", (int)e, cudaGetErrorString(e));
    }
    return RB_OK;
}

}  // extern "C"
