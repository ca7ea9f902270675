// Linear on host buffers with the copies pipelined against the tensor cores.
//
// The reference serves a host-side caller as write -> launch -> read through its ComputeServer, each step synchronous
// (rust-ascend-driver/src/tensor/runtime/mod.rs:767-845 for write/read, worker.rs:404-415 for launch + stream sync), so
// the upload, the GEMM and the read-back of one call never overlap.  Here the rows of X are cut into chunks that walk
// through three streams: chunk c uploads on the copy-in stream while chunk c-1 multiplies on the context's stream and
// chunk c-2 downloads on the copy-out stream.  PCIe is full duplex, so the call approaches the time of the larger of the
// two transfers instead of their sum plus the GEMM.
//
// Arithmetic is rb_gemm's (A [M,K] BF16, B [N,K] BF16, FP32 accumulate, optional bias, BF16 or FP32 out): each chunk is
// an independent set of output rows, so the result is bit-identical to one rb_gemm over all rows.
#include "common.cuh"

#include <map>

namespace {

constexpr int MAX_CHUNKS = 32;
struct Pipe {
    cudaStream_t up = nullptr, down = nullptr;
    cudaEvent_t entered = nullptr, drained = nullptr;
    cudaEvent_t uploaded[MAX_CHUNKS] = {}, computed[MAX_CHUNKS] = {};
};
std::mutex g_lock;
std::map<rb_ctx*, Pipe> g_pipes;

int32_t pipe_for(rb_ctx* ctx, Pipe** out) {
    std::lock_guard<std::mutex> g(g_lock);
    Pipe& p = g_pipes[ctx];
    if (!p.up) {
        RB_CUDA(ctx, "cudaStreamCreateWithFlags", cudaStreamCreateWithFlags(&p.up, cudaStreamNonBlocking));
        RB_CUDA(ctx, "cudaStreamCreateWithFlags", cudaStreamCreateWithFlags(&p.down, cudaStreamNonBlocking));
        RB_CUDA(ctx, "cudaEventCreateWithFlags", cudaEventCreateWithFlags(&p.entered, cudaEventDisableTiming));
        RB_CUDA(ctx, "cudaEventCreateWithFlags", cudaEventCreateWithFlags(&p.drained, cudaEventDisableTiming));
        for (int c = 0; c < MAX_CHUNKS; ++c) {
            RB_CUDA(ctx, "cudaEventCreateWithFlags", cudaEventCreateWithFlags(&p.uploaded[c], cudaEventDisableTiming));
            RB_CUDA(ctx, "cudaEventCreateWithFlags", cudaEventCreateWithFlags(&p.computed[c], cudaEventDisableTiming));
        }
    }
    *out = &p;
    return RB_OK;
}

}  // namespace

using namespace rb;

extern "C" {

int32_t rb_linear_host(rb_ctx* ctx, const void* host_x, const rb_tensor* x, const rb_tensor* w, const rb_tensor* bias,
                       const rb_tensor* y, void* host_y, uint32_t row_chunks) {
    RB_TRY(check_ctx(ctx));
    if (ctx->capturing) return fail(RB_INVALID_TENSOR, "rb_linear_host copies from and to host memory and cannot run while rb_graph_begin is recording");
    if (!host_x || !host_y) return fail(RB_NULL_HANDLE, "null host pointer");
    void *px, *pw, *py, *pb = nullptr;
    RB_TRY(resolve(ctx, x, "host Linear X staging", &px)); RB_TRY(resolve(ctx, w, "host Linear weight", &pw)); RB_TRY(resolve(ctx, y, "host Linear Y staging", &py));
    if (x->rank != 2 || w->rank != 2 || y->rank != 2 || x->dtype != RB_BF16 || w->dtype != RB_BF16 || (y->dtype != RB_BF16 && y->dtype != RB_F32))
        return fail(RB_INVALID_TENSOR, "host Linear takes BF16 X [M,K] and W [N,K] and a BF16 or FP32 Y [M,N]");
    const uint64_t m = x->shape[0], k = x->shape[1], n = w->shape[0];
    if (w->shape[1] != k || y->shape[0] != m || y->shape[1] != n) return fail(RB_INVALID_TENSOR, "host Linear shapes do not agree");
    if (m == 0 || n == 0 || k == 0 || m % 16 || n % 16 || k % 16 || m > 0x7fffffffull || n > 0x7fffffffull || k > 0x7fffffffull)
        return fail(RB_INVALID_TENSOR, "GEMM M/N/K must be positive multiples of 16 within INT32_MAX");
    if (bias) {
        RB_TRY(resolve(ctx, bias, "host Linear bias", &pb));
        if (elements(bias) != n || (bias->dtype != RB_F32 && bias->dtype != RB_BF16)) return fail(RB_INVALID_TENSOR, "GEMM bias must hold N FP32 or BF16 values");
    }
    const uint64_t ys = dtype_size(y->dtype);
    RB_TRY(no_overlap(py, m * n * ys, px, m * k * 2, "host Linear")); RB_TRY(no_overlap(py, m * n * ys, pw, n * k * 2, "host Linear"));
    if (row_chunks == 0) row_chunks = 1;
    if (row_chunks > MAX_CHUNKS) row_chunks = MAX_CHUNKS;
    // chunk height: a multiple of 128 rows (one tile row) unless the matrix is smaller than that
    uint64_t rows = (m + row_chunks - 1) / row_chunks;
    rows = rows >= 128 ? (rows + 127) / 128 * 128 : (rows + 15) / 16 * 16;
    Pipe* p = nullptr;
    RB_TRY(pipe_for(ctx, &p));
    // Uploads may not overwrite X while earlier work on the context's stream still reads it.
    RB_CUDA(ctx, "cudaEventRecord", cudaEventRecord(p->entered, ctx->stream));
    RB_CUDA(ctx, "cudaStreamWaitEvent", cudaStreamWaitEvent(p->up, p->entered, 0));
    RB_CUDA(ctx, "cudaStreamWaitEvent", cudaStreamWaitEvent(p->down, p->entered, 0));
    int c = 0;
    for (uint64_t r0 = 0; r0 < m; r0 += rows, ++c) {
        const uint64_t r = m - r0 < rows ? m - r0 : rows;
        RB_CUDA(ctx, "cudaMemcpyAsync(H2D)", cudaMemcpyAsync(static_cast<char*>(px) + r0 * k * 2, static_cast<const char*>(host_x) + r0 * k * 2, r * k * 2,
                                                            cudaMemcpyHostToDevice, p->up));
        RB_CUDA(ctx, "cudaEventRecord", cudaEventRecord(p->uploaded[c], p->up));
        RB_CUDA(ctx, "cudaStreamWaitEvent", cudaStreamWaitEvent(ctx->stream, p->uploaded[c], 0));
        RB_TRY(gemm_kmajor(ctx, static_cast<char*>(px) + r0 * k * 2, pw, nullptr, 1, (uint32_t)r, (uint32_t)n, (uint32_t)k,
                           bias ? RB_EPILOGUE_BIAS : RB_EPILOGUE_NONE, pb, bias && bias->dtype == RB_BF16,
                           static_cast<char*>(py) + r0 * n * ys, y->dtype == RB_F32));
        RB_CUDA(ctx, "cudaEventRecord", cudaEventRecord(p->computed[c], ctx->stream));
        RB_CUDA(ctx, "cudaStreamWaitEvent", cudaStreamWaitEvent(p->down, p->computed[c], 0));
        RB_CUDA(ctx, "cudaMemcpyAsync(D2H)", cudaMemcpyAsync(static_cast<char*>(host_y) + r0 * n * ys, static_cast<char*>(py) + r0 * n * ys, r * n * ys,
                                                            cudaMemcpyDeviceToHost, p->down));
    }
    // The call returns when Y is in host memory, like rb_read; later work on the context's stream is ordered behind it.
    RB_CUDA(ctx, "cudaEventRecord", cudaEventRecord(p->drained, p->down));
    RB_CUDA(ctx, "cudaStreamWaitEvent", cudaStreamWaitEvent(ctx->stream, p->drained, 0));
    return rb_sync(ctx);
}

}  // extern "C"
