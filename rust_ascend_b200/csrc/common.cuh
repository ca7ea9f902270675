// Shared host-side plumbing of libruda_b200: the process context, storage table, sticky errors,
// tensor validation and the launch epilogue.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <initializer_list>
#include <vector>

#include "ruda_b200.h"

namespace rb {

int32_t fail(rb_status code, const char* fmt, ...);

struct Storage {
    void* ptr = nullptr;
    uint64_t bytes = 0;
    bool owned = false;
    uint32_t guard = 0;      // bytes of guard band in front of and behind `ptr` (debug option), 0 when off
};

}  // namespace rb

struct rb_ctx {
    int device = 0;
    bool synchronous = false;
    cudaStream_t stream = nullptr;
    cudaEvent_t profile_start = nullptr, profile_stop = nullptr;
    std::mutex lock;
    std::unordered_map<uint64_t, rb::Storage> storage;
    uint64_t next_handle = 1;
    std::vector<std::string> sticky;   // failures raised by the next read / sync
    bool poisoned = false;             // set after a failed launch or synchronisation
    rb_stats stats{};
    int sm_count = 0;
    int sm_limit = 0;                  // 0: persistent kernels use every SM
    std::unordered_map<uint64_t, cudaGraphExec_t> graphs;
    uint64_t next_graph = 1;
    bool capturing = false;
    size_t smem_optin = 0;
    void* workspace = nullptr;         // lazily grown scratch owned by the context
    uint64_t workspace_bytes = 0;
    uint32_t guard_bytes = 0;          // RUDA_GUARD_BANDS=1: every allocation gets guard bands and starts filled with NaN patterns
    void* gemm_state = nullptr;        // tensor-map cache owned by the GEMM translation unit
    void* attention_state = nullptr;
};

namespace rb {

size_t dtype_size(uint32_t dtype);
const char* dtype_name(uint32_t dtype);
uint64_t elements(const rb_tensor* t);
bool contiguous(const rb_tensor* t);

// Resolves a tensor to its device address after the checks the reference performs before a launch:
// known handle, contiguous layout, byte range inside the storage, 16-byte alignment.
int32_t resolve(rb_ctx* ctx, const rb_tensor* t, const char* what, void** out, bool allow_null = false);
// Rejects an output that overlaps an input in device memory.
int32_t no_overlap(const void* out, uint64_t out_bytes, const void* in, uint64_t in_bytes, const char* what);
bool same_shape(const rb_tensor* a, const rb_tensor* b);
// Rows and width of a last-axis operation.
void rows_width(const rb_tensor* t, uint64_t* rows, uint64_t* width);

// Called after every kernel launch: records launch failures on the sticky list, counts the launch
// and synchronises when the context runs in the reference's synchronous mode.
int32_t after_launch(rb_ctx* ctx, const char* operation);
int32_t ensure_workspace(rb_ctx* ctx, uint64_t bytes);
int32_t check_ctx(rb_ctx* ctx);
int32_t empty_call(rb_ctx* ctx);
int32_t poll_kernel_status(rb_ctx* ctx);
int32_t kernel_status_word(rb_ctx* ctx, uint32_t** out);
// True between rb_aux_begin and rb_aux_end: launches are going to the side stream, beside the compute stream's kernels.
bool aux_active(rb_ctx* ctx);
// One launch of the tensor-core GEMM on K-major operands (A [.., m, k], B [.., n, k], both 16-bit), with every option the
// kernel has.  Operands that were split into parts store the parts as consecutive batch entries (z = batch * parts + part).
struct GemmCall {
    const void* a = nullptr; const void* b = nullptr; const void* b_up = nullptr;
    uint32_t batches = 1, m = 0, n = 0, k = 0;
    uint32_t a_rows = 0, b_rows = 0;                   // rows each batch entry of A / B occupies in memory (0: m / n); more when padded
    int epilogue = 0; const void* bias = nullptr; bool bias_bf16 = false;
    void* out = nullptr; uint32_t out_kind = 0;        // 0 BF16, 1 FP32, 2 FP16
    bool f16_operands = false;                         // operands are FP16 bit patterns instead of BF16
    bool ragged = false;                               // n * element size is not a multiple of 16 bytes
    uint32_t nseg = 1, parts_a = 1, parts_b = 1;
    uint32_t seg_a[6] = {0, 0, 0, 0, 0, 0}, seg_b[6] = {0, 0, 0, 0, 0, 0};
    bool a_bcast = false, b_bcast = false;             // the operand has one batch entry used by every output batch
    const int32_t* group_ends = nullptr; uint32_t groups = 0;   // M-grouped NT: B is [groups, n, k], device array of row prefix sums
};
int32_t gemm_run(rb_ctx* ctx, const GemmCall& call);
int32_t gemm_kmajor(rb_ctx* ctx, const void* a, const void* b, const void* b_up, uint32_t batches, uint32_t m, uint32_t n, uint32_t k,
                    int epilogue, const void* bias, bool bias_bf16, void* out, bool out_f32);

}  // namespace rb

namespace rb {

// Device temporaries of one call.  Each is registered as a non-owning storage so that the other entry points can be called on
// it through an ordinary tensor descriptor; the destructor drops the registrations and queues the frees behind the work.
struct Scratch {
    rb_ctx* ctx;
    struct Item { void* ptr; uint64_t handle; };
    std::vector<Item> items;
    explicit Scratch(rb_ctx* c) : ctx(c) {}
    ~Scratch() {
        for (auto& it : items) { rb_free(ctx, it.handle); cudaFreeAsync(it.ptr, ctx->stream); }
    }
    int32_t tensor(uint32_t dtype, std::initializer_list<uint64_t> shape, rb_tensor* out, void** ptr_out = nullptr) {
        *out = rb_tensor{};
        out->dtype = dtype; out->rank = (uint32_t)shape.size();
        uint64_t n = 1; int i = 0;
        for (uint64_t d : shape) { out->shape[i++] = d; n *= d; }
        uint64_t stride = 1;
        for (int a = (int)out->rank - 1; a >= 0; --a) { out->strides[a] = stride; stride *= out->shape[a]; }
        const uint64_t bytes = n * dtype_size(dtype);
        void* p = nullptr;
        cudaError_t e = cudaMallocAsync(&p, bytes ? bytes : 16, ctx->stream);
        if (e != cudaSuccess) return fail(RB_STATUS, "temporary of %llu bytes: cudaMallocAsync failed with CUDA status %d (%s)", (unsigned long long)bytes, (int)e, cudaGetErrorString(e));
        uint64_t h = 0;
        int32_t rc = rb_import(ctx, p, bytes ? bytes : 16, &h);
        if (rc != RB_OK) { cudaFreeAsync(p, ctx->stream); return rc; }
        items.push_back({p, h});
        out->handle = h;
        if (ptr_out) *ptr_out = p;
        return RB_OK;
    }
};

// The same storage seen with another shape (contiguous).
inline rb_tensor view(const rb_tensor& t, std::initializer_list<uint64_t> shape) {
    rb_tensor v = t;
    v.rank = (uint32_t)shape.size();
    int i = 0;
    for (uint64_t d : shape) v.shape[i++] = d;
    uint64_t stride = 1;
    for (int a = (int)v.rank - 1; a >= 0; --a) { v.strides[a] = stride; stride *= v.shape[a]; }
    return v;
}

}  // namespace rb

#define RB_TRY(expr) do { int32_t _s = (expr); if (_s != RB_OK) return _s; } while (0)
#define RB_CUDA(ctx, op, expr) do { cudaError_t _e = (expr); if (_e != cudaSuccess) \
    return rb::fail(RB_STATUS, "%s failed with CUDA status %d (%s)", op, (int)_e, cudaGetErrorString(_e)); } while (0)
