// Context, storage and server entry points of libruda_b200 (the ComputeServer / ComputeStorage role of
// rust-ascend-driver/src/tensor/runtime/mod.rs:485-877).
#include "common.cuh"

#include <cstdlib>

namespace rb {

static thread_local char g_error[1024] = "";

int32_t fail(rb_status code, const char* fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_error, sizeof(g_error), fmt, ap); va_end(ap);
    return (int32_t)code;
}

size_t dtype_size(uint32_t dtype) {
    switch (dtype) {
        case RB_F32: case RB_I32: return 4;
        case RB_F16: case RB_BF16: return 2;
        case RB_I64: return 8;
        case RB_U8: return 1;
        default: return 0;
    }
}
const char* dtype_name(uint32_t dtype) {
    switch (dtype) {
        case RB_F32: return "F32"; case RB_F16: return "F16"; case RB_BF16: return "BF16";
        case RB_I32: return "I32"; case RB_I64: return "I64"; case RB_U8: return "U8";
        default: return "unknown";
    }
}
uint64_t elements(const rb_tensor* t) {
    uint64_t n = 1;
    for (uint32_t i = 0; i < t->rank; ++i) n *= t->shape[i];
    return n;
}
bool contiguous(const rb_tensor* t) {
    // Same rule as runtime/mod.rs:907-925: row-major strides; axes of extent <= 1 may carry any stride.
    uint64_t stride = 1;
    for (int i = (int)t->rank - 1; i >= 0; --i) {
        if (t->shape[i] > 1 && t->strides[i] != stride) return false;
        stride *= t->shape[i];
    }
    return true;
}
bool same_shape(const rb_tensor* a, const rb_tensor* b) {
    if (a->rank != b->rank) return false;
    for (uint32_t i = 0; i < a->rank; ++i) if (a->shape[i] != b->shape[i]) return false;
    return true;
}
void rows_width(const rb_tensor* t, uint64_t* rows, uint64_t* width) {
    *width = t->rank ? t->shape[t->rank - 1] : 0;
    uint64_t r = 1;
    for (uint32_t i = 0; i + 1 < t->rank; ++i) r *= t->shape[i];
    *rows = r;
}

int32_t check_ctx(rb_ctx* ctx) {
    if (!ctx) return fail(RB_NULL_HANDLE, "null runtime context");
    if (ctx->poisoned) return fail(RB_SERVER_UNHEALTHY, "runtime is poisoned by an earlier failed launch or synchronisation");
    return RB_OK;
}

int32_t resolve(rb_ctx* ctx, const rb_tensor* t, const char* what, void** out, bool allow_null) {
    *out = nullptr;
    if (!t) return allow_null ? RB_OK : fail(RB_INVALID_TENSOR, "%s: missing tensor", what);
    if (t->rank == 0 || t->rank > 8) return fail(RB_INVALID_TENSOR, "%s: rank must be within 1..8", what);
    size_t es = dtype_size(t->dtype);
    if (!es) return fail(RB_INVALID_TENSOR, "%s: unsupported dtype %u", what, t->dtype);
    if (!contiguous(t)) return fail(RB_INVALID_TENSOR, "%s: requires a contiguous row-major tensor", what);
    Storage s;
    {
        std::lock_guard<std::mutex> g(ctx->lock);
        auto it = ctx->storage.find(t->handle);
        if (it == ctx->storage.end()) return fail(RB_NULL_HANDLE, "%s: unknown storage handle %llu", what, (unsigned long long)t->handle);
        s = it->second;
    }
    uint64_t bytes = elements(t) * es;
    if (t->offset > s.bytes || bytes > s.bytes - t->offset)
        return fail(RB_INVALID_TENSOR, "%s: buffer shape, stride, dtype or byte length mismatch (%llu bytes at offset %llu in a %llu byte storage)",
                    what, (unsigned long long)bytes, (unsigned long long)t->offset, (unsigned long long)s.bytes);
    char* p = (char*)s.ptr + t->offset;
    if (((uintptr_t)p & 15u) != 0) return fail(RB_INVALID_TENSOR, "%s: device address must be 16-byte aligned", what);
    *out = p;
    return RB_OK;
}

int32_t no_overlap(const void* out, uint64_t out_bytes, const void* in, uint64_t in_bytes, const char* what) {
    if (!out || !in || !out_bytes || !in_bytes) return RB_OK;
    uintptr_t a = (uintptr_t)out, b = (uintptr_t)in;
    if (a < b + in_bytes && b < a + out_bytes) return fail(RB_INVALID_TENSOR, "%s: output storage overlaps an input", what);
    return RB_OK;
}

int32_t after_launch(rb_ctx* ctx, const char* operation) {
    cudaError_t e = cudaGetLastError();
    ctx->stats.launches++;
    if (e != cudaSuccess) {
        char msg[256];
        snprintf(msg, sizeof(msg), "%s launch failed with CUDA status %d (%s)", operation, (int)e, cudaGetErrorString(e));
        std::lock_guard<std::mutex> g(ctx->lock);
        ctx->sticky.emplace_back(msg);
        return fail(RB_COMPLETION, "%s", msg);
    }
    if (ctx->synchronous) {
        ctx->stats.synchronizations++;
        e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) {
            ctx->poisoned = true;
            return fail(RB_COMPLETION, "%s completion failed with CUDA status %d (%s)", operation, (int)e, cudaGetErrorString(e));
        }
    }
    return RB_OK;
}

int32_t empty_call(rb_ctx* ctx) { ctx->stats.empty_calls++; return RB_OK; }

int32_t ensure_workspace(rb_ctx* ctx, uint64_t bytes) {
    if (bytes <= ctx->workspace_bytes) return RB_OK;
    if (ctx->workspace) { cudaStreamSynchronize(ctx->stream); cudaFree(ctx->workspace); ctx->workspace = nullptr; ctx->workspace_bytes = 0; }
    uint64_t want = (bytes + ((1u << 20) - 1)) & ~uint64_t((1u << 20) - 1);
    cudaError_t e = cudaMalloc(&ctx->workspace, want);
    if (e != cudaSuccess) return fail(RB_STATUS, "workspace allocation of %llu bytes failed with CUDA status %d", (unsigned long long)want, (int)e);
    ctx->workspace_bytes = want;
    return RB_OK;
}

static std::mutex g_init_lock;
static rb_ctx* g_ctx = nullptr;

}  // namespace rb

using namespace rb;

namespace {

constexpr int GUARD_PATTERN = 0xA5;

// Reads both guard bands of an allocation back and compares them with the pattern (the stream has been drained by the caller).
bool guards_damaged(const Storage& s) {
    const uint64_t body = ((s.bytes ? s.bytes : 1) + 255) & ~uint64_t(255);
    std::vector<unsigned char> host(2ull * s.guard);
    if (cudaMemcpy(host.data(), static_cast<const char*>(s.ptr) - s.guard, s.guard, cudaMemcpyDeviceToHost) != cudaSuccess) return true;
    if (cudaMemcpy(host.data() + s.guard, static_cast<const char*>(s.ptr) + body, s.guard, cudaMemcpyDeviceToHost) != cudaSuccess) return true;
    for (unsigned char c : host) if (c != GUARD_PATTERN) return true;
    return false;
}

}  // namespace

extern "C" {

const char* rb_last_error(void) { return g_error; }

int32_t rb_init_exclusive(const rb_options* options, rb_ctx** out) {
    if (!out) return fail(RB_NULL_HANDLE, "null output pointer");
    std::lock_guard<std::mutex> g(g_init_lock);
    if (g_ctx) return fail(RB_INVALID_DEVICE, "B200 runtime already initialized");
    int device = options ? options->device : 0;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(RB_INVALID_DEVICE, "no CUDA device is available (status %d: %s); this backend has no CPU fallback", (int)e, cudaGetErrorString(e));
    if (device < 0 || device >= count) return fail(RB_INVALID_DEVICE, "device ordinal %d is outside 0..%d", device, count - 1);
    RB_CUDA(nullptr, "cudaSetDevice", cudaSetDevice(device));
    cudaDeviceProp prop;
    RB_CUDA(nullptr, "cudaGetDeviceProperties", cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(RB_INVALID_DEVICE, "device %d is sm_%d%d; this library carries sm_100a code only", device, prop.major, prop.minor);
    rb_ctx* ctx = new rb_ctx();
    ctx->device = device;
    ctx->synchronous = options && options->synchronous;
    { const char* env = std::getenv("RUDA_GUARD_BANDS"); ctx->guard_bytes = env && env[0] == '1' ? 256u : 0u; }
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = prop.sharedMemPerBlockOptin;
    e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreate(&ctx->profile_start);
    if (e == cudaSuccess) e = cudaEventCreate(&ctx->profile_stop);
    if (e != cudaSuccess) { delete ctx; return fail(RB_STATUS, "stream/event creation failed with CUDA status %d", (int)e); }
    g_ctx = ctx;
    *out = ctx;
    return RB_OK;
}

int32_t rb_shutdown(rb_ctx* ctx) {
    std::lock_guard<std::mutex> g(g_init_lock);
    if (!ctx || ctx != g_ctx) return fail(RB_NULL_HANDLE, "unknown runtime context");
    cudaSetDevice(ctx->device);
    // If work cannot be drained, device memory is leaked rather than freed under a running kernel
    // (the reference's rule, tensor/mod.rs:258-268).
    bool drained = cudaStreamSynchronize(ctx->stream) == cudaSuccess;
    if (drained) {
        for (auto& kv : ctx->storage) if (kv.second.owned && kv.second.ptr) cudaFree(kv.second.ptr);
        if (ctx->workspace) cudaFree(ctx->workspace);
        cudaEventDestroy(ctx->profile_start); cudaEventDestroy(ctx->profile_stop);
        cudaStreamDestroy(ctx->stream);
    }
    g_ctx = nullptr;
    delete ctx;
    return RB_OK;
}

int32_t rb_device_properties(rb_ctx* ctx, char* name, size_t name_bytes, int32_t* sm_count, uint64_t* memory_bytes) {
    if (!ctx) return fail(RB_NULL_HANDLE, "null runtime context");
    cudaDeviceProp prop;
    RB_CUDA(ctx, "cudaGetDeviceProperties", cudaGetDeviceProperties(&prop, ctx->device));
    if (name && name_bytes) { strncpy(name, prop.name, name_bytes - 1); name[name_bytes - 1] = 0; }
    if (sm_count) *sm_count = prop.multiProcessorCount;
    if (memory_bytes) *memory_bytes = prop.totalGlobalMem;
    return RB_OK;
}

int32_t rb_check_guards(rb_ctx* ctx, uint64_t* damaged) {
    RB_TRY(check_ctx(ctx));
    if (!damaged) return fail(RB_NULL_HANDLE, "null pointer");
    *damaged = 0;
    if (!ctx->guard_bytes) return RB_OK;
    ctx->stats.synchronizations++;
    RB_CUDA(ctx, "cudaStreamSynchronize", cudaStreamSynchronize(ctx->stream));
    std::vector<Storage> owned;
    {
        std::lock_guard<std::mutex> g(ctx->lock);
        for (auto& kv : ctx->storage) if (kv.second.owned && kv.second.guard) owned.push_back(kv.second);
    }
    for (const Storage& s : owned) if (guards_damaged(s)) ++*damaged;
    return RB_OK;
}

int32_t rb_alloc(rb_ctx* ctx, uint64_t bytes, uint64_t* handle) {
    RB_TRY(check_ctx(ctx));
    if (!handle) return fail(RB_NULL_HANDLE, "null handle pointer");
    void* p = nullptr;
    uint64_t real = bytes ? bytes : 1;  // empty tensors still own an allocation
    const uint32_t guard = ctx->guard_bytes;
    if (guard) {
        // Debug option: [guard | body rounded up to 256 B | guard].  The guards hold a fixed pattern that rb_check_guards and
        // rb_free verify; the body starts as all-ones bytes (NaN in every float format), so an output element that a kernel
        // never wrote shows up in any comparison.
        const uint64_t body = (real + 255) & ~uint64_t(255);
        RB_CUDA(ctx, "cudaMalloc", cudaMalloc(&p, body + 2ull * guard));
        RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(p, GUARD_PATTERN, guard, ctx->stream));
        RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(static_cast<char*>(p) + guard, 0xFF, body, ctx->stream));
        RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(static_cast<char*>(p) + guard + body, GUARD_PATTERN, guard, ctx->stream));
        p = static_cast<char*>(p) + guard;
    } else {
        RB_CUDA(ctx, "cudaMalloc", cudaMalloc(&p, real));
    }
    std::lock_guard<std::mutex> g(ctx->lock);
    uint64_t id = ctx->next_handle++;
    ctx->storage[id] = Storage{p, bytes, true, guard};
    ctx->stats.bytes_in_use += bytes; ctx->stats.allocations++;
    *handle = id;
    return RB_OK;
}

int32_t rb_import(rb_ctx* ctx, void* device_pointer, uint64_t bytes, uint64_t* handle) {
    RB_TRY(check_ctx(ctx));
    if (!handle || !device_pointer) return fail(RB_NULL_HANDLE, "null pointer");
    std::lock_guard<std::mutex> g(ctx->lock);
    uint64_t id = ctx->next_handle++;
    ctx->storage[id] = Storage{device_pointer, bytes, false};
    *handle = id;
    return RB_OK;
}

int32_t rb_free(rb_ctx* ctx, uint64_t handle) {
    if (!ctx) return fail(RB_NULL_HANDLE, "null runtime context");
    Storage s;
    {
        std::lock_guard<std::mutex> g(ctx->lock);
        auto it = ctx->storage.find(handle);
        if (it == ctx->storage.end()) return fail(RB_NULL_HANDLE, "unknown storage handle %llu", (unsigned long long)handle);
        s = it->second;
        ctx->storage.erase(it);
        if (s.owned) { ctx->stats.bytes_in_use -= s.bytes; ctx->stats.allocations--; }
    }
    if (!s.owned) return RB_OK;
    ctx->stats.synchronizations++;
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) { ctx->poisoned = true; return fail(RB_COMPLETION, "dealloc: stream did not drain (CUDA status %d); memory is leaked, not freed", (int)e); }
    if (s.guard) {
        if (guards_damaged(s)) {
            std::lock_guard<std::mutex> g(ctx->lock);
            char msg[160]; snprintf(msg, sizeof(msg), "a kernel wrote outside storage %llu (%llu bytes): its guard band is damaged", (unsigned long long)handle, (unsigned long long)s.bytes);
            ctx->sticky.emplace_back(msg);
        }
        RB_CUDA(ctx, "cudaFree", cudaFree(static_cast<char*>(s.ptr) - s.guard));
        return RB_OK;
    }
    RB_CUDA(ctx, "cudaFree", cudaFree(s.ptr));
    return RB_OK;
}

int32_t rb_resource(rb_ctx* ctx, uint64_t handle, void** device_pointer, uint64_t* bytes) {
    if (!ctx) return fail(RB_NULL_HANDLE, "null runtime context");
    std::lock_guard<std::mutex> g(ctx->lock);
    auto it = ctx->storage.find(handle);
    if (it == ctx->storage.end()) return fail(RB_NULL_HANDLE, "unknown storage handle %llu", (unsigned long long)handle);
    if (device_pointer) *device_pointer = it->second.ptr;
    if (bytes) *bytes = it->second.bytes;
    return RB_OK;
}

static int32_t range(rb_ctx* ctx, uint64_t handle, uint64_t offset, uint64_t bytes, char** p) {
    std::lock_guard<std::mutex> g(ctx->lock);
    auto it = ctx->storage.find(handle);
    if (it == ctx->storage.end()) return fail(RB_NULL_HANDLE, "unknown storage handle %llu", (unsigned long long)handle);
    if (offset > it->second.bytes || bytes > it->second.bytes - offset)
        return fail(RB_INVALID_TENSOR, "byte range %llu+%llu is outside a %llu byte storage", (unsigned long long)offset,
                    (unsigned long long)bytes, (unsigned long long)it->second.bytes);
    *p = (char*)it->second.ptr + offset;
    return RB_OK;
}

int32_t rb_write(rb_ctx* ctx, uint64_t handle, uint64_t offset, const void* host, uint64_t bytes) {
    RB_TRY(check_ctx(ctx));
    char* p; RB_TRY(range(ctx, handle, offset, bytes, &p));
    if (!bytes) return RB_OK;
    if (!host) return fail(RB_NULL_HANDLE, "null host pointer");
    RB_CUDA(ctx, "cudaMemcpyAsync(H2D)", cudaMemcpyAsync(p, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return RB_OK;
}

static int32_t raise_sticky(rb_ctx* ctx) {
    std::lock_guard<std::mutex> g(ctx->lock);
    if (ctx->sticky.empty()) return RB_OK;
    std::string all;
    for (auto& s : ctx->sticky) { if (!all.empty()) all += "; "; all += s; }
    return fail(RB_SERVER_UNHEALTHY, "server unhealthy: %s", all.c_str());
}

int32_t rb_sync(rb_ctx* ctx) {
    if (!ctx) return fail(RB_NULL_HANDLE, "null runtime context");
    ctx->stats.synchronizations++;
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        ctx->poisoned = true;
        std::lock_guard<std::mutex> g(ctx->lock);
        char msg[200]; snprintf(msg, sizeof(msg), "stream synchronisation failed with CUDA status %d (%s)", (int)e, cudaGetErrorString(e));
        ctx->sticky.emplace_back(msg);
    } else {
        poll_kernel_status(ctx);
    }
    return raise_sticky(ctx);
}

int32_t rb_read(rb_ctx* ctx, uint64_t handle, uint64_t offset, void* host, uint64_t bytes) {
    if (!ctx) return fail(RB_NULL_HANDLE, "null runtime context");
    RB_TRY(raise_sticky(ctx));
    char* p; RB_TRY(range(ctx, handle, offset, bytes, &p));
    if (bytes) {
        if (!host) return fail(RB_NULL_HANDLE, "null host pointer");
        RB_CUDA(ctx, "cudaMemcpyAsync(D2H)", cudaMemcpyAsync(host, p, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    }
    return rb_sync(ctx);
}

int32_t rb_memset(rb_ctx* ctx, uint64_t handle, uint64_t offset, int32_t value, uint64_t bytes) {
    RB_TRY(check_ctx(ctx));
    char* p; RB_TRY(range(ctx, handle, offset, bytes, &p));
    if (bytes) RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(p, value, bytes, ctx->stream));
    return RB_OK;
}

int32_t rb_take_errors(rb_ctx* ctx, char* buf, size_t buf_bytes, uint32_t* count) {
    if (!ctx) return fail(RB_NULL_HANDLE, "null runtime context");
    std::lock_guard<std::mutex> g(ctx->lock);
    if (count) *count = (uint32_t)ctx->sticky.size();
    if (buf && buf_bytes) {
        std::string all;
        for (auto& s : ctx->sticky) { all += s; all += "\n"; }
        strncpy(buf, all.c_str(), buf_bytes - 1); buf[buf_bytes - 1] = 0;
    }
    ctx->sticky.clear();
    return RB_OK;
}

int32_t rb_get_stats(rb_ctx* ctx, rb_stats* out) {
    if (!ctx || !out) return fail(RB_NULL_HANDLE, "null pointer");
    *out = ctx->stats;
    return RB_OK;
}

int32_t rb_host_alloc(rb_ctx* ctx, uint64_t bytes, void** host) {
    RB_TRY(check_ctx(ctx));
    if (!host) return fail(RB_NULL_HANDLE, "null pointer");
    RB_CUDA(ctx, "cudaHostAlloc", cudaHostAlloc(host, bytes ? bytes : 1, cudaHostAllocDefault));
    return RB_OK;
}
int32_t rb_host_free(rb_ctx* ctx, void* host) {
    if (!ctx) return fail(RB_NULL_HANDLE, "null runtime context");
    if (host) RB_CUDA(ctx, "cudaFreeHost", cudaFreeHost(host));
    return RB_OK;
}

int32_t rb_profile_begin(rb_ctx* ctx) {
    RB_TRY(check_ctx(ctx));
    RB_CUDA(ctx, "cudaEventRecord", cudaEventRecord(ctx->profile_start, ctx->stream));
    return RB_OK;
}
int32_t rb_profile_end(rb_ctx* ctx, float* milliseconds) {
    RB_TRY(check_ctx(ctx));
    RB_CUDA(ctx, "cudaEventRecord", cudaEventRecord(ctx->profile_stop, ctx->stream));
    ctx->stats.synchronizations++;
    cudaError_t e = cudaEventSynchronize(ctx->profile_stop);
    if (e != cudaSuccess) { ctx->poisoned = true; return fail(RB_COMPLETION, "profile: event synchronisation failed with CUDA status %d (%s)", (int)e, cudaGetErrorString(e)); }
    float ms = 0;
    RB_CUDA(ctx, "cudaEventElapsedTime", cudaEventElapsedTime(&ms, ctx->profile_start, ctx->profile_stop));
    if (milliseconds) *milliseconds = ms;
    return raise_sticky(ctx);
}

int32_t rb_set_sm_limit(rb_ctx* ctx, int32_t sm_limit) {
    if (!ctx) return fail(RB_NULL_HANDLE, "null runtime context");
    if (sm_limit < 0 || sm_limit > ctx->sm_count) return fail(RB_INVALID_TENSOR, "SM limit must be within 0..%d", ctx->sm_count);
    ctx->sm_limit = sm_limit;
    return RB_OK;
}

int32_t rb_graph_begin(rb_ctx* ctx) {
    RB_TRY(check_ctx(ctx));
    if (ctx->capturing) return fail(RB_INVALID_TENSOR, "a graph is already being recorded");
    if (ctx->synchronous) return fail(RB_INVALID_TENSOR, "graphs cannot be recorded in synchronous mode");
    RB_CUDA(ctx, "cudaStreamBeginCapture", cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
    ctx->capturing = true;
    return RB_OK;
}

int32_t rb_graph_end(rb_ctx* ctx, uint64_t* graph) {
    if (!ctx || !graph) return fail(RB_NULL_HANDLE, "null pointer");
    if (!ctx->capturing) return fail(RB_INVALID_TENSOR, "no graph is being recorded");
    ctx->capturing = false;
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
    if (e != cudaSuccess || !g) return fail(RB_STATUS, "cudaStreamEndCapture failed with CUDA status %d (%s)", (int)e, cudaGetErrorString(e));
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return fail(RB_STATUS, "cudaGraphInstantiate failed with CUDA status %d (%s)", (int)e, cudaGetErrorString(e));
    std::lock_guard<std::mutex> lk(ctx->lock);
    *graph = ctx->next_graph++;
    ctx->graphs[*graph] = exec;
    return RB_OK;
}

int32_t rb_graph_launch(rb_ctx* ctx, uint64_t graph) {
    RB_TRY(check_ctx(ctx));
    cudaGraphExec_t exec;
    {
        std::lock_guard<std::mutex> lk(ctx->lock);
        auto it = ctx->graphs.find(graph);
        if (it == ctx->graphs.end()) return fail(RB_NULL_HANDLE, "unknown graph %llu", (unsigned long long)graph);
        exec = it->second;
    }
    RB_CUDA(ctx, "cudaGraphLaunch", cudaGraphLaunch(exec, ctx->stream));
    ctx->stats.launches++;
    return RB_OK;
}

int32_t rb_graph_destroy(rb_ctx* ctx, uint64_t graph) {
    if (!ctx) return fail(RB_NULL_HANDLE, "null runtime context");
    std::lock_guard<std::mutex> lk(ctx->lock);
    auto it = ctx->graphs.find(graph);
    if (it == ctx->graphs.end()) return fail(RB_NULL_HANDLE, "unknown graph %llu", (unsigned long long)graph);
    cudaGraphExecDestroy(it->second);
    ctx->graphs.erase(it);
    return RB_OK;
}

int32_t rb_stream(rb_ctx* ctx, void** stream) {
    if (!ctx || !stream) return fail(RB_NULL_HANDLE, "null pointer");
    *stream = (void*)ctx->stream;
    return RB_OK;
}

}  // extern "C"
