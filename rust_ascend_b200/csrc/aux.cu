// A second, higher-priority stream beside the context's compute stream, for work that should run under the compute
// stream's kernels instead of between them (the owner-side reduce + push of the fused tensor-parallel exchange, which is
// bound by the peer links and needs only a few SMs).  rb_aux_begin forks: everything enqueued until rb_aux_end goes to the
// side stream, ordered after what the compute stream held at the fork.  rb_aux_end records the side stream's position in one
// of 32 slots; rb_aux_wait makes the compute stream wait for a slot.  Forks and joins are stream/event operations only, so a
// CUDA graph recorded on the compute stream captures them as branches.
//
// The reference has no counterpart: every operation there is launch + stream synchronisation (runtime/worker.rs:404-415).
#include "common.cuh"

#include <map>

namespace {

constexpr int SLOTS = 32;
struct Aux {
    cudaStream_t side = nullptr, main = nullptr;
    cudaEvent_t fork = nullptr;
    cudaEvent_t done[SLOTS] = {};
    bool recorded[SLOTS] = {};
    bool active = false;
};
std::mutex g_lock;
std::map<rb_ctx*, Aux> g_aux;

}  // namespace

namespace rb {

bool aux_active(rb_ctx* ctx) {
    std::lock_guard<std::mutex> g(g_lock);
    auto it = g_aux.find(ctx);
    return it != g_aux.end() && it->second.active;
}

}  // namespace rb

using namespace rb;

extern "C" {

int32_t rb_aux_begin(rb_ctx* ctx) {
    RB_TRY(check_ctx(ctx));
    std::lock_guard<std::mutex> g(g_lock);
    Aux& a = g_aux[ctx];
    if (a.active) return fail(RB_INVALID_TENSOR, "the side stream is already open");
    if (!a.side) {
        int least = 0, greatest = 0;
        RB_CUDA(ctx, "cudaDeviceGetStreamPriorityRange", cudaDeviceGetStreamPriorityRange(&least, &greatest));
        RB_CUDA(ctx, "cudaStreamCreateWithPriority", cudaStreamCreateWithPriority(&a.side, cudaStreamNonBlocking, greatest));
        RB_CUDA(ctx, "cudaEventCreateWithFlags", cudaEventCreateWithFlags(&a.fork, cudaEventDisableTiming));
        for (int s = 0; s < SLOTS; ++s) RB_CUDA(ctx, "cudaEventCreateWithFlags", cudaEventCreateWithFlags(&a.done[s], cudaEventDisableTiming));
    }
    RB_CUDA(ctx, "cudaEventRecord", cudaEventRecord(a.fork, ctx->stream));
    RB_CUDA(ctx, "cudaStreamWaitEvent", cudaStreamWaitEvent(a.side, a.fork, 0));
    a.main = ctx->stream;
    ctx->stream = a.side;
    a.active = true;
    return RB_OK;
}

int32_t rb_aux_end(rb_ctx* ctx, uint32_t slot) {
    RB_TRY(check_ctx(ctx));
    std::lock_guard<std::mutex> g(g_lock);
    auto it = g_aux.find(ctx);
    if (it == g_aux.end() || !it->second.active) return fail(RB_INVALID_TENSOR, "the side stream is not open");
    Aux& a = it->second;
    ctx->stream = a.main;                          // restored whatever happens below
    a.active = false;
    if (slot >= SLOTS) return fail(RB_INVALID_TENSOR, "side-stream slots are 0..%d", SLOTS - 1);
    RB_CUDA(ctx, "cudaEventRecord", cudaEventRecord(a.done[slot], a.side));
    a.recorded[slot] = true;
    return RB_OK;
}

int32_t rb_aux_wait(rb_ctx* ctx, uint32_t slot) {
    RB_TRY(check_ctx(ctx));
    std::lock_guard<std::mutex> g(g_lock);
    auto it = g_aux.find(ctx);
    if (it == g_aux.end() || slot >= SLOTS || !it->second.recorded[slot]) return fail(RB_INVALID_TENSOR, "nothing was recorded in side-stream slot %u", slot);
    if (it->second.active) return fail(RB_INVALID_TENSOR, "close the side stream before waiting for it");
    RB_CUDA(ctx, "cudaStreamWaitEvent", cudaStreamWaitEvent(ctx->stream, it->second.done[slot], 0));
    return RB_OK;
}

}  // extern "C"
