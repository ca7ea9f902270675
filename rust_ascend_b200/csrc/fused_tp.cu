// Tensor-parallel row-parallel projection with its exchange step fused in, over peer memory (NVLink / NVSwitch).
//
// The reference runs the row-parallel Linear and then one all-reduce of the [T, H] result through the vendor library
// (runtime/hccl.rs:386-548; src/distributed.rs:139-156 for reduce-scatter).  Here the exchange is split into the two halves
// an all-reduce consists of and each half is fused into the kernel next to it:
//
//   1. gemm_scatter_kernel: Y_partial = A[T, K/N] * B[H, K/N]^T on the tensor cores (same pipeline as the plain GEMM: TMA
//      producer warp, tcgen05.mma issuer warp, four epilogue warps, two TMEM accumulators).  The epilogue does not write a
//      local [T, H]: rows [o*R, (o+1)*R) belong to rank o (R = T / world), and every finished 32-row slice is stored
//      straight into rank o's staging area slot [this rank]; when a CTA has stored all its tiles, each epilogue warp
//      fences once and adds the number of slices it stored for rank o to rank o's flag word [this rank].  The transfer of tile i overlaps the main loop of tile i+1.  (reduce-scatter, fused tile by tile)
//   2. reduce_norm_push_kernel, on the R rows a rank owns: sums the `world` staged partials in rank order in FP32 (one
//      rounding to BF16, as an all-reduce result would have), adds the residual stream, applies RMSNorm, and stores the
//      normalised rows into every rank's activation buffer at the owner's row offset, then announces them with one
//      release-add per destination.  (all-gather, fused into the norm; the residual stream stays sharded by rows)
//   3. peer_wait_kernel: one warp that waits, with a time limit, until the local flag words have reached their running
//      target.  It runs on this GPU and waits only for kernels on OTHER GPUs, which never wait for it.
//
// Flags only ever count up; the running target lives in device memory next to them, so the same launches can be
// replayed from a CUDA graph.  Staging and activation buffers are reused by consecutive projections; that is safe
// because a rank can only reach the next scatter after it has seen every owner's push of the step before, and the next
// push after it has seen every rank's scatter (each owner reads its staging area before it pushes).
//
// No load here uses cluster broadcast; peers are reached by plain stores and red operations only.
#include "common.cuh"

#include <cmath>
#include <cstdlib>

#include "schedule.h"
#include "sm100.cuh"

namespace {

using namespace sm100;
using bf = __nv_bfloat16;

constexpr int BM = 128, BK = 64, UMMA_K = 16, GROUP_M = 8, THREADS = 192;
constexpr int MAX_PEERS = RB_MAX_PEERS;
constexpr int CHUNK = 64;                       // output columns moved through shared memory at a time
constexpr int PITCH = CHUNK * 2 + 16;           // bytes per staged row: 128 payload + 16 pad (conflict-free 16-byte accesses)

struct ScatterParams {
    uint32_t m, n, k;               // m = world * rows_per_owner
    uint32_t tiles_m, tiles_n;
    uint32_t rows_per_owner;
    uint32_t world;
    uint32_t tile_shift;            // tile rows this rank starts ahead of rank order, so that at any moment the ranks write to
                                    // different owners instead of all to the same one
    const float* bias;              // FP32 [n] added to this rank's partial product before it is rounded and stored, or null
    uint8_t* dst[MAX_PEERS];        // owner o's staging slot for this rank: [rows_per_owner, n] BF16
    uint32_t* flag[MAX_PEERS];      // owner o's flag word for this rank
    uint32_t* status;
};

template <int BN> struct Config {
    static constexpr int STAGES = BN == 256 ? 4 : 6;
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int OUT_BYTES = 4 * 32 * PITCH;   // one 32-row x CHUNK-column slice per epilogue warp
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + OUT_BYTES;
    static constexpr int TMEM_COLS = 2 * BN;
};

__device__ __forceinline__ void scatter_coords(uint32_t t, const ScatterParams& p, uint32_t& tm, uint32_t& tn) {
    rb_scatter_tile(t, p.tiles_m, p.tiles_n, GROUP_M, p.tile_shift, tm, tn);
}

__device__ __forceinline__ void signal_release_sys(uint32_t* flag, uint32_t count = 1u) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(flag), "r"(count) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_scatter_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const ScatterParams p) {
    using C = Config<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + C::STAGES;
    uint64_t* tmem_full = empty_bar + C::STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;
    uint8_t* out_smem = smem + C::STAGES * C::STAGE_BYTES + 256;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t num_kb = (p.k + BK - 1) / BK;
    const uint32_t num_tiles = p.tiles_m * p.tiles_n;
    // An earlier kernel of this stream gave up on a bounded wait: the step is lost, store and announce nothing.  One thread
    // reads the word so that the whole CTA takes the same branch.
    __shared__ uint32_t step_lost;
    if (threadIdx.x == 0) step_lost = *reinterpret_cast<volatile uint32_t*>(p.status);
    __syncthreads();
    if (step_lost) return;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 128); }
        *abort_word = 0;
        fence_barrier_init();
        prefetch_tmap(&map_a); prefetch_tmap(&map_b);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (elect_one()) {
            uint32_t stage = 0, phase = 0, armed = 0, armed_parity = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
                uint32_t tm, tn; scatter_coords(t, p, tm, tn);
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_word))) break;
                    uint8_t* sa = smem + stage * C::STAGE_BYTES; uint8_t* sb = sa + C::A_BYTES;
                    mbar_expect_tx(&full_bar[stage], C::STAGE_BYTES);
                    armed |= 1u << stage; armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
                    tma_load_3d(sa, &map_a, &full_bar[stage], (int32_t)(kb * BK), (int32_t)(tm * BM), 0);
                    tma_load_3d(sb, &map_b, &full_bar[stage], (int32_t)(kb * BK), (int32_t)(tn * BN), 0);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // A wait expired somewhere: let the copies this thread issued land before the CTA retires.
                for (int s = 0; s < C::STAGES; ++s)
                    if (armed & (1u << s))
                        for (uint32_t i = 0; i < (1u << 20) && !mbar_try_wait(&full_bar[s], (armed_parity >> s) & 1u); ++i) {}
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (elect_one()) {
            const uint32_t idesc = make_idesc_bf16(BM, BN);
            uint32_t stage = 0, phase = 0, iter = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x, ++iter) {
                const uint32_t acc = iter & 1, acc_phase = (iter >> 1) & 1;
                if (!(ok = mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_word))) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(&full_bar[stage], phase, abort_word))) break;
                    tc_fence_after();
                    uint8_t* sa = smem + stage * C::STAGE_BYTES;
                    const uint64_t da = make_kmajor_sw128_desc(smem_u32(sa)), db = make_kmajor_sw128_desc(smem_u32(sa + C::A_BYTES));
#pragma unroll
                    for (uint32_t k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_ss(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    umma_commit(&empty_bar[stage]);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit(&tmem_full[acc]);
            }
        }
    } else {
        // ---------------- epilogue: 4 warps; TMEM lane = output row; rows leave through shared memory so that every
        // global store instruction covers whole 128-byte row segments (what a peer link moves efficiently) ------------
        const uint32_t quarter = warp & 3;
        uint8_t* my_smem = out_smem + quarter * 32 * PITCH;
        uint32_t iter = 0;
        uint32_t slices = 0;                 // lane o counts the slices this warp stored for owner o
        bool ok = true;
        for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x, ++iter) {
            const uint32_t acc = iter & 1, acc_phase = (iter >> 1) & 1;
            uint32_t tm, tn; scatter_coords(t, p, tm, tn);
            ok = mbar_wait(&tmem_full[acc], acc_phase, abort_word);
            if (!(ok = __all_sync(0xffffffffu, ok))) break;  // keep the warp converged
            tc_fence_after();
            const uint32_t row0 = tm * BM + quarter * 32;             // first of this warp's 32 rows
            uint32_t owner, local_row0;                               // a 128-row tile never straddles two owners
            rb_scatter_owner(row0, p.rows_per_owner, owner, local_row0);
            const uint32_t col0 = tn * BN;
            const uint32_t taddr = tmem_base + acc * BN + ((quarter * 32) << 16);
            uint8_t* dst = p.dst[owner] + ((size_t)local_row0 * p.n + col0) * 2;
            for (uint32_t c = 0; c < BN; c += CHUNK) {
                if (col0 + c >= p.n) break;  // warp-uniform (n is a multiple of CHUNK)
                uint32_t r0[32], r1[32];
                tmem_ld_32x32(taddr + c, r0);
                tmem_ld_32x32(taddr + c + 32, r1);
                tmem_wait_ld();
                if (p.bias) {
                    // the bias of a row-parallel Linear is added once: the rank that is given it folds it into its partial product
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        r0[j] = __float_as_uint(__fadd_rn(__uint_as_float(r0[j]), __ldg(p.bias + col0 + c + j)));
                        r1[j] = __float_as_uint(__fadd_rn(__uint_as_float(r1[j]), __ldg(p.bias + col0 + c + 32 + j)));
                    }
                }
                if (c + CHUNK >= BN || col0 + c + CHUNK >= p.n) {    // last read of this accumulator: hand it back early
                    tc_fence_before();
                    mbar_arrive(&tmem_empty[acc]);
                }
                uint4* mine = reinterpret_cast<uint4*>(my_smem + lane * PITCH);
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    __nv_bfloat162 q0 = __floats2bfloat162_rn(__uint_as_float(r0[j]), __uint_as_float(r0[j + 1]));
                    __nv_bfloat162 q1 = __floats2bfloat162_rn(__uint_as_float(r0[j + 2]), __uint_as_float(r0[j + 3]));
                    __nv_bfloat162 q2 = __floats2bfloat162_rn(__uint_as_float(r0[j + 4]), __uint_as_float(r0[j + 5]));
                    __nv_bfloat162 q3 = __floats2bfloat162_rn(__uint_as_float(r0[j + 6]), __uint_as_float(r0[j + 7]));
                    uint4 w;
                    w.x = *reinterpret_cast<uint32_t*>(&q0); w.y = *reinterpret_cast<uint32_t*>(&q1);
                    w.z = *reinterpret_cast<uint32_t*>(&q2); w.w = *reinterpret_cast<uint32_t*>(&q3);
                    mine[j / 8] = w;
                }
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    __nv_bfloat162 q0 = __floats2bfloat162_rn(__uint_as_float(r1[j]), __uint_as_float(r1[j + 1]));
                    __nv_bfloat162 q1 = __floats2bfloat162_rn(__uint_as_float(r1[j + 2]), __uint_as_float(r1[j + 3]));
                    __nv_bfloat162 q2 = __floats2bfloat162_rn(__uint_as_float(r1[j + 4]), __uint_as_float(r1[j + 5]));
                    __nv_bfloat162 q3 = __floats2bfloat162_rn(__uint_as_float(r1[j + 6]), __uint_as_float(r1[j + 7]));
                    uint4 w;
                    w.x = *reinterpret_cast<uint32_t*>(&q0); w.y = *reinterpret_cast<uint32_t*>(&q1);
                    w.z = *reinterpret_cast<uint32_t*>(&q2); w.w = *reinterpret_cast<uint32_t*>(&q3);
                    mine[4 + j / 8] = w;
                }
                __syncwarp();
                // 32 rows x 128 bytes = 256 16-byte words; lane l moves words l, l+32, ...: 8 lanes per row segment.
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    uint32_t r, j; rb_scatter_word(it, lane, r, j);
                    const uint4 w = *reinterpret_cast<const uint4*>(my_smem + r * PITCH + j * 16);
                    *reinterpret_cast<uint4*>(dst + ((size_t)r * p.n + c) * 2 + j * 16) = w;
                }
                __syncwarp();
            }
            slices += lane == owner;
        }
        // One fence for everything this warp stored, then its announcements: waiting for the link's acknowledgements once
        // per CTA instead of once per tile keeps the epilogue shorter than the next tile's main loop.  Slices of a tile
        // that was abandoned after an expired wait are not announced, so the owner's wait runs out instead of passing.
        __threadfence_system();
        __syncwarp();
        if (lane < p.world && slices) signal_release_sys(p.flag[lane], slices);
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_word) atomicExch(p.status, 1u);
    if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, C::TMEM_COLS); }
}

// The scatter GEMM on pairs of CTAs (cluster of two, tcgen05 cta_group::2), for outputs wider than 128 columns and T a multiple of
// 256: the pipeline of gemm_bf16_pair_kernel (each CTA loads its 128 rows of A and half of the 256 B rows, the leader issues the
// MMAs, completions are broadcast to both CTAs) with the epilogue above: every CTA scatters its own 128 rows of the 256 x 256 tile.
constexpr int SP_BN = 256, SP_STAGES = 6;
constexpr int SP_A_BYTES = BM * BK * 2, SP_B_BYTES = (SP_BN / 2) * BK * 2, SP_STAGE_BYTES = SP_A_BYTES + SP_B_BYTES;
constexpr int SP_SMEM_BYTES = SP_STAGES * SP_STAGE_BYTES + 1024 + 256 + 4 * 32 * PITCH;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_scatter_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const ScatterParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + SP_STAGES * SP_STAGE_BYTES);   // used in the leader only
    uint64_t* empty_bar = full_bar + SP_STAGES;
    uint64_t* tmem_full = empty_bar + SP_STAGES;
    uint64_t* tmem_empty = tmem_full + 2;                                                   // leader only: 256 arrivals
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;
    uint32_t* step_lost = tmem_slot + 2;
    uint8_t* out_smem = smem + SP_STAGES * SP_STAGE_BYTES + 256;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const uint32_t num_kb = (p.k + BK - 1) / BK;
    const uint32_t num_tiles = p.tiles_m * p.tiles_n;
    // An earlier kernel of this stream gave up on a bounded wait: the step is lost, store and announce nothing.  Both CTAs of a
    // pair must take the same branch, so the leader's reading decides for both (the peer reads it after the cluster barrier).
    if (threadIdx.x == 0) *step_lost = *reinterpret_cast<volatile uint32_t*>(p.status);

    if (threadIdx.x == 0) {
        for (int s = 0; s < SP_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 256); }
        *abort_word = 0;
        fence_barrier_init();
        prefetch_tmap(&map_a); prefetch_tmap(&map_b);
    }
    if (warp == 1) { tmem_alloc_pair(tmem_slot, 2 * SP_BN); tmem_relinquish_pair(); }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    uint32_t lost;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(lost) : "r"(mapa_shared(smem_u32(step_lost), 0)) : "memory");
    const bool run = lost == 0;

    if (run && warp == 0) {
        if (elect_one()) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t t = pair; ok && t < num_tiles; t += pairs) {
                uint32_t tm, tn; scatter_coords(t, p, tm, tn);
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_word))) break;
                    uint8_t* sa = smem + stage * SP_STAGE_BYTES; uint8_t* sb = sa + SP_A_BYTES;
                    const uint32_t leader_full = mapa_shared(smem_u32(&full_bar[stage]), 0);
                    if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * SP_STAGE_BYTES);
                    tma_load_3d_pair(sa, &map_a, leader_full, (int32_t)(kb * BK), (int32_t)(tm * 2 * BM + rank * BM), 0);
                    tma_load_3d_pair(sb, &map_b, leader_full, (int32_t)(kb * BK), (int32_t)(tn * SP_BN + rank * (SP_BN / 2)), 0);
                    if (++stage == SP_STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) for (uint32_t i = 0; i < (1u << 22); ++i) __nanosleep(32);   // let the copies in flight land
        }
    } else if (run && warp == 1) {
        if (rank == 0 && elect_one()) {
            const uint32_t idesc = make_idesc_bf16(2 * BM, SP_BN);
            uint32_t stage = 0, phase = 0, iter = 0;
            bool ok = true;
            for (uint32_t t = pair; ok && t < num_tiles; t += pairs, ++iter) {
                const uint32_t acc = iter & 1, acc_phase = (iter >> 1) & 1;
                if (!(ok = mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_word))) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * SP_BN;
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(&full_bar[stage], phase, abort_word))) break;
                    tc_fence_after();
                    uint8_t* sa = smem + stage * SP_STAGE_BYTES;
                    const uint64_t da = make_kmajor_sw128_desc(smem_u32(sa)), db = make_kmajor_sw128_desc(smem_u32(sa + SP_A_BYTES));
#pragma unroll
                    for (uint32_t k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_ss_pair(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    umma_commit_pair(&empty_bar[stage]);
                    if (++stage == SP_STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit_pair(&tmem_full[acc]);
            }
        }
    } else if (run) {
        const uint32_t quarter = warp & 3;
        uint8_t* my_smem = out_smem + quarter * 32 * PITCH;
        const uint32_t leader_empty0 = mapa_shared(smem_u32(&tmem_empty[0]), 0), leader_empty1 = mapa_shared(smem_u32(&tmem_empty[1]), 0);
        uint32_t iter = 0, slices = 0;       // lane o counts the slices this warp stored for owner o
        bool ok = true;
        for (uint32_t t = pair; ok && t < num_tiles; t += pairs, ++iter) {
            const uint32_t acc = iter & 1, acc_phase = (iter >> 1) & 1;
            uint32_t tm, tn; scatter_coords(t, p, tm, tn);
            ok = mbar_wait(&tmem_full[acc], acc_phase, abort_word);
            if (!(ok = __all_sync(0xffffffffu, ok))) break;
            tc_fence_after();
            const uint32_t row0 = tm * 2 * BM + rank * BM + quarter * 32;    // first of this warp's 32 rows
            uint32_t owner, local_row0;
            rb_scatter_owner(row0, p.rows_per_owner, owner, local_row0);
            const uint32_t col0 = tn * SP_BN;
            const uint32_t taddr = tmem_base + acc * SP_BN + ((quarter * 32) << 16);
            uint8_t* dst = p.dst[owner] + ((size_t)local_row0 * p.n + col0) * 2;
            for (uint32_t c = 0; c < (uint32_t)SP_BN; c += CHUNK) {
                if (col0 + c >= p.n) break;  // warp-uniform (n is a multiple of CHUNK)
                uint32_t r0[32], r1[32];
                tmem_ld_32x32(taddr + c, r0);
                tmem_ld_32x32(taddr + c + 32, r1);
                tmem_wait_ld();
                if (p.bias) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        r0[j] = __float_as_uint(__fadd_rn(__uint_as_float(r0[j]), __ldg(p.bias + col0 + c + j)));
                        r1[j] = __float_as_uint(__fadd_rn(__uint_as_float(r1[j]), __ldg(p.bias + col0 + c + 32 + j)));
                    }
                }
                if (c + CHUNK >= (uint32_t)SP_BN || col0 + c + CHUNK >= p.n) {    // last read of this accumulator: hand it back early
                    tc_fence_before();
                    mbar_arrive_cluster(acc ? leader_empty1 : leader_empty0);
                }
                uint4* mine = reinterpret_cast<uint4*>(my_smem + lane * PITCH);
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    uint4 w;
                    __nv_bfloat162 q0 = __floats2bfloat162_rn(__uint_as_float(r0[j]), __uint_as_float(r0[j + 1]));
                    __nv_bfloat162 q1 = __floats2bfloat162_rn(__uint_as_float(r0[j + 2]), __uint_as_float(r0[j + 3]));
                    __nv_bfloat162 q2 = __floats2bfloat162_rn(__uint_as_float(r0[j + 4]), __uint_as_float(r0[j + 5]));
                    __nv_bfloat162 q3 = __floats2bfloat162_rn(__uint_as_float(r0[j + 6]), __uint_as_float(r0[j + 7]));
                    w.x = *reinterpret_cast<uint32_t*>(&q0); w.y = *reinterpret_cast<uint32_t*>(&q1);
                    w.z = *reinterpret_cast<uint32_t*>(&q2); w.w = *reinterpret_cast<uint32_t*>(&q3);
                    mine[j / 8] = w;
                    q0 = __floats2bfloat162_rn(__uint_as_float(r1[j]), __uint_as_float(r1[j + 1]));
                    q1 = __floats2bfloat162_rn(__uint_as_float(r1[j + 2]), __uint_as_float(r1[j + 3]));
                    q2 = __floats2bfloat162_rn(__uint_as_float(r1[j + 4]), __uint_as_float(r1[j + 5]));
                    q3 = __floats2bfloat162_rn(__uint_as_float(r1[j + 6]), __uint_as_float(r1[j + 7]));
                    w.x = *reinterpret_cast<uint32_t*>(&q0); w.y = *reinterpret_cast<uint32_t*>(&q1);
                    w.z = *reinterpret_cast<uint32_t*>(&q2); w.w = *reinterpret_cast<uint32_t*>(&q3);
                    mine[4 + j / 8] = w;
                }
                __syncwarp();
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    uint32_t r, j; rb_scatter_word(it, lane, r, j);
                    const uint4 w = *reinterpret_cast<const uint4*>(my_smem + r * PITCH + j * 16);
                    *reinterpret_cast<uint4*>(dst + ((size_t)r * p.n + c) * 2 + j * 16) = w;
                }
                __syncwarp();
            }
            slices += lane == owner;
        }
        __threadfence_system();
        __syncwarp();
        if (lane < p.world && slices) signal_release_sys(p.flag[lane], slices);
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_word) atomicExch(p.status, 1u);
    cluster_sync_all();
    if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc_pair(tmem_base, 2 * SP_BN); }
}

// flags[0..world) count up as peers announce their stores; flags[world] is the running target.  Lane i waits until
// flags[i] has reached target + count (wrap-safe), with a time limit after which the status word is raised and the wait
// ends, so the context stays usable.  Then the target moves on.
__global__ void __launch_bounds__(32) peer_wait_kernel(uint32_t* flags, uint32_t world, uint32_t count, uint32_t* status, uint64_t limit_ns) {
    const uint32_t lane = threadIdx.x;
    const uint32_t target = flags[world] + count;
    bool expired = false;
    // A wait that already ran out (here or in an earlier kernel of this stream) ends the step: the waits queued behind it
    // return at once instead of each spending its own limit, so a lost rank costs about one limit in total.
    const bool give_up = *reinterpret_cast<volatile uint32_t*>(status) != 0;
    if (lane < world && !give_up) {
        const uint64_t start = global_timer_ns();
        while ((int32_t)(load_acquire_sys(flags + lane) - target) < 0) {
            if (global_timer_ns() - start > limit_ns) { expired = true; break; }
            __nanosleep(64);
        }
    }
    if (__any_sync(0xffffffffu, expired) && lane == 0) atomicExch(status, 2u);
    __syncwarp();
    if (lane == 0) flags[world] = target;
}

struct SignalParams { uint32_t world; uint32_t* flag[MAX_PEERS]; };

// Adds 1 to this rank's word at every destination, after everything earlier in the stream (a stream-ordered barrier's
// arrival half; rb_peer_wait is the other half).
__global__ void __launch_bounds__(32) peer_signal_kernel(const SignalParams p) {
    __threadfence_system();
    if (threadIdx.x < p.world) signal_release_sys(p.flag[threadIdx.x]);
}

// The scatter as a kernel of its own, for a row-parallel Linear that ran as a plain GEMM: every row of the local partial
// product goes to slot [this rank] of the staging area of the rank that owns it.  All link traffic is posted stores (16 bytes
// per thread, a warp covers 512 contiguous bytes), which a few SMs keep flowing without holding anything in flight the way
// remote reads must.  Blocks walk the rows starting with the owner after this rank, so the ranks write to different owners at
// any moment.  The last block to finish tells every owner once.
struct ScatterRowsParams {
    const bf* src;                  // [world * rows, width] local
    uint32_t rows, width, world, rank;
    bf* dst[MAX_PEERS];             // owner o's staging slot for this rank: [rows, width]
    uint32_t* flag[MAX_PEERS];      // owner o's flag word for this rank
    uint32_t* done;                 // local block counter, zero between launches
    const uint32_t* status;
};

__global__ void __launch_bounds__(256) scatter_rows_kernel(const ScatterRowsParams p) {
    __shared__ bool last;
    __shared__ uint32_t step_lost;
    if (threadIdx.x == 0) step_lost = *reinterpret_cast<const volatile uint32_t*>(p.status);
    __syncthreads();
    if (step_lost) return;
    const uint32_t vecs = p.width / 8, total = p.rows * p.world;
    const uint32_t first = ((p.rank + 1) % p.world) * p.rows;      // rotation of the row order
    for (uint32_t i = blockIdx.x; i < total; i += gridDim.x) {
        uint32_t row = i + first; if (row >= total) row -= total;
        const uint32_t owner = row / p.rows, local = row - owner * p.rows;
        const uint4* src = reinterpret_cast<const uint4*>(p.src + (size_t)row * p.width);
        uint4* dst = reinterpret_cast<uint4*>(p.dst[owner] + (size_t)local * p.width);
        for (uint32_t vi = threadIdx.x; vi < vecs; vi += 256) dst[vi] = __ldcs(src + vi);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t ticket = atomicAdd(p.done, 1u);
        __threadfence_system();
        last = ticket == gridDim.x - 1;
    }
    __syncthreads();
    if (last) {
        if (threadIdx.x == 0) *p.done = 0;
        if (threadIdx.x < p.world) signal_release_sys(p.flag[threadIdx.x]);
    }
}

struct PushParams {
    const bf* staging;              // [partials, rows, width] or null
    const bf* pull[MAX_PEERS];      // pull form: rank s's partial product, at the first of the rows this rank owns ([rows, width])
    uint32_t partials;
    const bf* x_in;                 // [rows, width] residual stream (owned rows) or null
    bf* x_out;                      // [rows, width] or null
    const bf* weight;               // [width], or null: no normalisation, the summed rows are pushed as they are
    float eps;
    uint32_t rows, width, world;
    uint64_t dst_row0;              // first row of this rank's block inside every destination buffer
    bf* dst[MAX_PEERS];             // destination activation buffers [world * rows (or more), width]
    uint32_t* flag[MAX_PEERS];      // destination d's flag word for this rank
    uint32_t* done;                 // local block counter, zero between launches
    uint32_t* status;               // device status word: non-zero once a bounded wait has run out
    uint32_t stages;                // pull form: rows in flight per block (1..PULL_STAGES)
};

constexpr int PUSH_THREADS = 256;
constexpr int PUSH_MAXV = 4;        // 16-byte vectors per thread: width <= 256 * 4 * 8 = 8192

// What follows the sum of the partials for one row: round it once to BF16 (as the result of an all-reduce would be), add the
// residual stream, store the new residual row, normalise, and store the row into every rank's activation buffer.
// v[i][0..8) is the FP32 sum of 16-byte vector i * PUSH_THREADS + threadIdx.x of the row.  Called by all threads of the block.
// xin[i] is the same vector of the residual stream's row (read when p.x_in is set).
// SYNC_BEFORE_RED: a block-wide barrier separates this row's write of the reduction scratch from the previous row's reads; a
// caller whose own loop already has a barrier between the rows passes false.
template <bool SYNC_BEFORE_RED, int NV>
__device__ __forceinline__ void push_row(const PushParams& p, uint32_t row, const uint4 (&xin)[NV], float (&v)[NV][8], const bool (&have)[NV], float* red) {
    if (p.partials) {
#pragma unroll
        for (int i = 0; i < NV; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j]));
    }
    if (p.x_in) {
#pragma unroll
        for (int i = 0; i < NV; ++i) if (have[i]) {
            const uint4 w = xin[i];
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f = __bfloat1622float2(h2[j]);
                // residual update rounded to the storage type first, as the separate add+norm kernel does
                v[i][2 * j] = __bfloat162float(__float2bfloat16_rn(__fadd_rn(f.x, v[i][2 * j])));
                v[i][2 * j + 1] = __bfloat162float(__float2bfloat16_rn(__fadd_rn(f.y, v[i][2 * j + 1])));
            }
        }
    }
    if (p.x_out) {
        uint4* dstx = reinterpret_cast<uint4*>(p.x_out + (size_t)row * p.width);
#pragma unroll
        for (int i = 0; i < NV; ++i) if (have[i]) {
            uint4 w; __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
            for (int j = 0; j < 4; ++j) h2[j] = __floats2bfloat162_rn(v[i][2 * j], v[i][2 * j + 1]);
            dstx[i * PUSH_THREADS + threadIdx.x] = w;
        }
    }
    if (!p.weight) {
        // plain all-reduce: the reduced rows themselves go to every destination
#pragma unroll
        for (int i = 0; i < NV; ++i) if (have[i]) {
            const uint32_t vi = i * PUSH_THREADS + threadIdx.x;
            uint4 o; __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(v[i][2 * j], v[i][2 * j + 1]);
            for (uint32_t d = 0; d < p.world; ++d)
                reinterpret_cast<uint4*>(p.dst[d] + (p.dst_row0 + row) * p.width)[vi] = o;
        }
        return;
    }
    // RMSNorm (row_programs.rs:144-151): r = rsqrt(mean(x^2) + eps); y = (x * r) * w
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc = acc + __fmul_rn(v[i][j], v[i][j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (SYNC_BEFORE_RED) __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    float sum = red[0];
#pragma unroll
    for (int w = 1; w < PUSH_THREADS / 32; ++w) sum += red[w];
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)p.width), p.eps)));
#pragma unroll
    for (int i = 0; i < NV; ++i) if (have[i]) {
        const uint32_t vi = i * PUSH_THREADS + threadIdx.x;
        const uint4 ww = __ldg(reinterpret_cast<const uint4*>(p.weight) + vi);
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&ww);
        uint4 o; __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 wf = __bfloat1622float2(w2[j]);
            o2[j] = __floats2bfloat162_rn(__fmul_rn(__fmul_rn(v[i][2 * j], r), wf.x), __fmul_rn(__fmul_rn(v[i][2 * j + 1], r), wf.y));
        }
        for (uint32_t d = 0; d < p.world; ++d)
            reinterpret_cast<uint4*>(p.dst[d] + (p.dst_row0 + row) * p.width)[vi] = o;
    }
}

// The last block of the grid to finish announces this rank's rows to every destination.
__device__ __forceinline__ void push_announce(const PushParams& p, bool* last) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t ticket = atomicAdd(p.done, 1u);
        __threadfence_system();          // what the other blocks stored before their tickets is ordered before the signals below
        *last = ticket == gridDim.x - 1;
    }
    __syncthreads();
    if (*last) {
        if (threadIdx.x == 0) *p.done = 0;
        if (threadIdx.x < p.world) signal_release_sys(p.flag[threadIdx.x]);
    }
}

__global__ void __launch_bounds__(PUSH_THREADS) reduce_norm_push_kernel(const PushParams p) {
    __shared__ float red[PUSH_THREADS / 32];
    __shared__ bool last;
    const uint32_t vecs = p.width / 8;  // 16-byte vectors per row
    __shared__ uint32_t step_lost;      // read by one thread so that the whole block takes the same branch
    if (threadIdx.x == 0) step_lost = *reinterpret_cast<const volatile uint32_t*>(p.status);
    __syncthreads();
    if (step_lost) return;              // a bounded wait already ran out: push and announce nothing
    for (uint32_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
        float v[PUSH_MAXV][8];
        bool have[PUSH_MAXV];
#pragma unroll
        for (int i = 0; i < PUSH_MAXV; ++i) {
            const uint32_t vi = i * PUSH_THREADS + threadIdx.x;
            have[i] = vi < vecs;
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
        }
        // fixed rank order, FP32: every rank computes bit-identical sums for the rows it owns
        for (uint32_t s = 0; s < p.partials; ++s) {
            const uint4* src = reinterpret_cast<const uint4*>(p.staging + ((size_t)s * p.rows + row) * p.width);
#pragma unroll
            for (int i = 0; i < PUSH_MAXV; ++i) if (have[i]) {
                const uint4 w = __ldcg(src + i * PUSH_THREADS + threadIdx.x);   // written by peers: read through L2
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
                for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(h2[j]); v[i][2 * j] += f.x; v[i][2 * j + 1] += f.y; }
            }
        }
        uint4 xin[PUSH_MAXV];
        if (p.x_in) {
            const uint4* src = reinterpret_cast<const uint4*>(p.x_in + (size_t)row * p.width);
#pragma unroll
            for (int i = 0; i < PUSH_MAXV; ++i) if (have[i]) xin[i] = src[i * PUSH_THREADS + threadIdx.x];
        }
        push_row<true, PUSH_MAXV>(p, row, xin, v, have, red);
    }
    push_announce(p, &last);
}

// The pull form of the owner-side step: the partial products stay where the plain GEMM of each rank wrote them, and the owner
// fetches its rows of all of them itself.  Remote reads have microseconds of latency, so the rows come in as bulk asynchronous
// copies (one per source and row, straight into shared memory, completion counted by an mbarrier) that keep PULL_STAGES rows
// of `world` sources in flight per block without holding them in registers; the row of the residual stream travels the same
// way, so that no thread waits for a load from global memory.  The copies name one GPU's memory each and are not cluster
// broadcasts.  Everything after the sum is push_row, so both forms give the same bits.
constexpr int PULL_STAGES = 3;

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

template <int NV>      // 16-byte vectors per thread: 2 for rows of up to 4096 values, else NV
__global__ void __launch_bounds__(PUSH_THREADS) pull_reduce_norm_push_kernel(const PushParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    __shared__ uint64_t full[PULL_STAGES];
    __shared__ float red[PUSH_THREADS / 32];
    __shared__ bool last;
    __shared__ uint32_t step_lost, abort_word_s;
    volatile uint32_t* abort_word = &abort_word_s;
    const uint32_t vecs = p.width / 8, row_bytes = p.width * 2, stage_bytes = (p.partials + (p.x_in ? 1u : 0u)) * row_bytes;
    if (threadIdx.x == 0) {
        step_lost = *reinterpret_cast<const volatile uint32_t*>(p.status);
        abort_word_s = 0;
        for (int s = 0; s < PULL_STAGES; ++s) mbar_init(&full[s], 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (step_lost) return;
    const uint32_t my_rows = blockIdx.x < p.rows ? (p.rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    // Row number `it` of this block into stage it % stages: thread 0 arms the barrier with the stage's byte count (arm), then,
    // behind a block-wide barrier, thread s issues the copy of source s (copy), so that the issue cost of world + 1 copies is
    // not one thread's.
    auto arm = [&](uint32_t it) { mbar_expect_tx(&full[it % p.stages], stage_bytes); };
    auto copy = [&](uint32_t it) {
        const uint32_t st = it % p.stages, row = blockIdx.x + it * gridDim.x, s = threadIdx.x;
        if (s < p.partials)
            bulk_load(smem + (size_t)st * stage_bytes + (size_t)s * row_bytes, p.pull[s] + (size_t)row * p.width, row_bytes, &full[st]);
        else if (s == p.partials && p.x_in)
            bulk_load(smem + (size_t)st * stage_bytes + (size_t)s * row_bytes, p.x_in + (size_t)row * p.width, row_bytes, &full[st]);
    };
    if (threadIdx.x == 0)
        for (uint32_t it = 0; it < my_rows && it < p.stages; ++it) arm(it);
    __syncthreads();
    for (uint32_t it = 0; it < my_rows && it < p.stages; ++it) copy(it);
    bool ok = true;
    uint32_t landed = 0;                 // rows whose copies are known to have completed
    for (uint32_t it = 0; it < my_rows; ++it) {
        const uint32_t st = it % p.stages, row = blockIdx.x + it * gridDim.x;
        // every thread waits for the row itself (no barrier needed before reading it); a thread whose wait ran out has raised
        // the abort word, which all threads read after the barrier below
        mbar_wait(&full[st], (it / p.stages) & 1, abort_word);
        float v[NV][8];
        bool have[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const uint32_t vi = i * PUSH_THREADS + threadIdx.x;
            have[i] = vi < vecs;
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
        }
        // fixed rank order, FP32: every rank computes bit-identical sums for the rows it owns
        for (uint32_t s = 0; s < p.partials; ++s) {
            const uint4* src = reinterpret_cast<const uint4*>(smem + (size_t)st * stage_bytes + (size_t)s * row_bytes);
#pragma unroll
            for (int i = 0; i < NV; ++i) if (have[i]) {
                const uint4 w = src[i * PUSH_THREADS + threadIdx.x];
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
                for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(h2[j]); v[i][2 * j] += f.x; v[i][2 * j + 1] += f.y; }
            }
        }
        // the residual row moves to registers before the stage is handed back
        uint4 xin[NV];
        if (p.x_in) {
            const uint4* src = reinterpret_cast<const uint4*>(smem + (size_t)st * stage_bytes + (size_t)p.partials * row_bytes);
#pragma unroll
            for (int i = 0; i < NV; ++i) if (have[i]) xin[i] = src[i * PUSH_THREADS + threadIdx.x];
        }
        if (threadIdx.x == 0 && it + p.stages < my_rows) arm(it + p.stages);   // this phase of the barrier is over: arm the next
        __syncthreads();                 // every thread has read the stage: it may be filled again (also orders the rows' uses of `red`)
        if (*abort_word) { ok = false; break; }
        landed = it + 1;
        if (it + p.stages < my_rows) copy(it + p.stages);
        push_row<false, NV>(p, row, xin, v, have, red);
    }
    if (!ok) {
        // A copy did not arrive within the bound (a peer's memory went away): raise the status word, give the copies that
        // are still in flight a bounded time to land, and announce nothing.
        if (threadIdx.x == 0) {
            atomicExch(p.status, 1u);
            const uint32_t issued = my_rows < landed + p.stages ? my_rows : landed + p.stages;
            for (uint32_t it = landed; it < issued; ++it)
                for (uint32_t i = 0; i < (1u << 20) && !mbar_try_wait(&full[it % p.stages], (it / p.stages) & 1); ++i) {}
        }
        __syncthreads();
        return;
    }
    push_announce(p, &last);
}

template <int BN>
int32_t launch_scatter(rb_ctx* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const ScatterParams& p) {
    using C = Config<BN>;
    // raised once per process and template instance; std::call_once makes the first use safe from any thread
    static std::once_flag once;
    static cudaError_t configured = cudaSuccess;
    std::call_once(once, [] { configured = cudaFuncSetAttribute(gemm_scatter_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES); });
    if (configured != cudaSuccess) return rb::fail(RB_STATUS, "cudaFuncSetAttribute(scatter GEMM) failed with CUDA status %d (%s)", (int)configured, cudaGetErrorString(configured));
    const uint32_t tiles = p.tiles_m * p.tiles_n;
    const uint32_t sms = ctx->sm_limit > 0 ? (uint32_t)ctx->sm_limit : (uint32_t)ctx->sm_count;
    gemm_scatter_kernel<BN><<<tiles < sms ? tiles : sms, THREADS, C::SMEM_BYTES, ctx->stream>>>(ma, mb, p);
    return rb::after_launch(ctx, "gemm_scatter");
}

// The pair kernel's launch: as many pairs as the occupancy query for clusters of two allows (not every SM can be paired),
// capped by the context's SM limit.
int32_t launch_scatter_pair(rb_ctx* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const ScatterParams& p) {
    static std::once_flag once;
    static cudaError_t configured = cudaSuccess;
    static int max_pairs = 0;
    std::call_once(once, [ctx] {
        configured = cudaFuncSetAttribute(gemm_scatter_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SP_SMEM_BYTES);
        if (configured != cudaSuccess) return;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(2 * (unsigned)ctx->sm_count, 1, 1); cfg.blockDim = dim3(THREADS, 1, 1); cfg.dynamicSmemBytes = SP_SMEM_BYTES;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeClusterDimension; attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr; cfg.numAttrs = 1;
        configured = cudaOccupancyMaxActiveClusters(&max_pairs, gemm_scatter_pair_kernel, &cfg);
    });
    if (configured != cudaSuccess || max_pairs < 1)
        return rb::fail(RB_STATUS, "configuring the scatter GEMM on CTA pairs failed with CUDA status %d (%s)", (int)configured, cudaGetErrorString(configured));
    uint32_t pairs = (uint32_t)max_pairs;
    if (ctx->sm_limit > 0 && (uint32_t)ctx->sm_limit / 2 < pairs) pairs = (uint32_t)ctx->sm_limit / 2;
    if (pairs == 0) pairs = 1;
    const uint32_t tiles = p.tiles_m * p.tiles_n;
    if (tiles < pairs) pairs = tiles;
    gemm_scatter_pair_kernel<<<2 * pairs, THREADS, SP_SMEM_BYTES, ctx->stream>>>(ma, mb, p);
    return rb::after_launch(ctx, "gemm_scatter (CTA pairs)");
}

bool operand_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t k, uint32_t box_rows) {
    uint64_t dims[3] = {k, rows, 1};
    uint64_t strides[2] = {k * 2, rows * k * 2};
    uint32_t box[3] = {BK, box_rows, 1};
    return encode_bf16_map(map, base, 3, dims, strides, box, true);
}

using namespace rb;

int32_t resolve_flags(rb_ctx* ctx, const rb_tensor* t, uint32_t world, const char* what, uint32_t** out);

// Host side of both forms of the owner-side step.  `staging` (push form: [world, rows, width] in local memory, written by the
// scatter GEMMs of all ranks) or `pulls` (pull form: every rank's [world * rows, width] partial product, peers' memory mapped
// here) names the partials; neither means "no partials, normalise the residual stream only".
// `local_out` (with destinations and flags null) selects the form that keeps everything on this GPU: the rows go to local_out
// [rows, width] only and the closing announcement lands in word 1 of `done`.
int32_t reduce_norm_push_impl(rb_ctx* ctx, const rb_tensor* staging, const rb_tensor* const* pulls, const rb_tensor* x_in, const rb_tensor* weight,
                              double epsilon, const rb_tensor* x_out, uint32_t rank, uint32_t world, const rb_tensor* const* destinations,
                              const rb_tensor* const* flags, const rb_tensor* done, const rb_tensor* local_out = nullptr) {
    RB_TRY(check_ctx(ctx));
    if (world < 1 || world > MAX_PEERS || rank >= world || (!local_out && (!destinations || !flags)))
        return fail(RB_INVALID_TENSOR, "reduce+norm+push needs 1..%d ranks and their activation and flag tensors", MAX_PEERS);
    void *ps = nullptr, *pxi = nullptr, *pxo = nullptr, *pw = nullptr, *pd = nullptr;
    RB_TRY(resolve(ctx, staging, "reduce+norm+push staging area", &ps, true)); RB_TRY(resolve(ctx, x_in, "reduce+norm+push residual", &pxi, true));
    RB_TRY(resolve(ctx, x_out, "reduce+norm+push residual output", &pxo, true)); RB_TRY(resolve(ctx, weight, "reduce+norm+push weight", &pw, true));
    RB_TRY(resolve(ctx, done, "reduce+norm+push block counter", &pd));
    if (!staging && !pulls && !x_in) return fail(RB_INVALID_TENSOR, "reduce+norm+push needs partial products, a residual stream, or both");
    if (weight && (!(epsilon > 0.0) || !std::isfinite(epsilon))) return fail(RB_INVALID_TENSOR, "RMSNorm epsilon must be finite and positive");
    const rb_tensor* shape_of = x_in ? x_in : x_out;
    uint64_t rows, width;
    if (staging) {
        if (staging->rank != 3 || staging->dtype != RB_BF16 || staging->shape[0] != world) return fail(RB_INVALID_TENSOR, "staging area is BF16 [world, rows, width]");
        rows = staging->shape[1]; width = staging->shape[2];
    } else if (pulls) {
        if (!pulls[0] || pulls[0]->rank != 2 || pulls[0]->shape[0] % world) return fail(RB_INVALID_TENSOR, "partial products are BF16 [world * rows, width]");
        rows = pulls[0]->shape[0] / world; width = pulls[0]->shape[1];
    } else {
        if (!shape_of || shape_of->rank != 2) return fail(RB_INVALID_TENSOR, "residual stream is BF16 [rows, width]");
        rows = shape_of->shape[0]; width = shape_of->shape[1];
    }
    for (const rb_tensor* t : {x_in, x_out})
        if (t && (t->rank != 2 || t->dtype != RB_BF16 || t->shape[0] != rows || t->shape[1] != width)) return fail(RB_INVALID_TENSOR, "residual stream is BF16 [rows, width]");
    if (weight && (weight->dtype != RB_BF16 || elements(weight) != width)) return fail(RB_INVALID_TENSOR, "RMSNorm weight is BF16 [width]");
    if (done->dtype != RB_I32 || elements(done) < (local_out ? 2u : 1u)) return fail(RB_INVALID_TENSOR, "block counter is one INT32 word (two for the local form)");
    if (rows == 0 || width == 0 || width % 8 || width > (uint64_t)PUSH_THREADS * PUSH_MAXV * 8 || rows > 0x7fffffffull)
        return fail(RB_INVALID_TENSOR, "reduce+norm+push needs a positive width that is a multiple of 8 and at most 8192");
    PushParams p{};
    p.staging = static_cast<const bf*>(ps); p.partials = staging || pulls ? world : 0;
    p.x_in = static_cast<const bf*>(pxi); p.x_out = static_cast<bf*>(pxo); p.weight = static_cast<const bf*>(pw);
    p.eps = (float)epsilon; p.rows = (uint32_t)rows; p.width = (uint32_t)width; p.world = world; p.dst_row0 = (uint64_t)rank * rows;
    p.done = static_cast<uint32_t*>(pd);
    RB_TRY(kernel_status_word(ctx, &p.status));
    if (local_out) {
        void* po = nullptr;
        RB_TRY(resolve(ctx, local_out, "reduce+norm output rows", &po));
        if (local_out->dtype != RB_BF16 || local_out->rank != 2 || local_out->shape[0] != rows || local_out->shape[1] != width)
            return fail(RB_INVALID_TENSOR, "output rows are BF16 [rows, width]");
        p.world = 1; p.dst_row0 = 0;
        p.dst[0] = static_cast<bf*>(po);
        p.flag[0] = p.done + 1;
    }
    for (uint32_t d = 0; d < world && !local_out; ++d) {
        void* pdst = nullptr; uint32_t* pf = nullptr;
        RB_TRY(resolve(ctx, destinations[d], "reduce+norm+push destination", &pdst));
        RB_TRY(resolve_flags(ctx, flags[d], world, "reduce+norm+push flags", &pf));
        const rb_tensor* t = destinations[d];
        if (t->dtype != RB_BF16 || t->rank != 2 || t->shape[1] != width || t->shape[0] != rows * world)
            return fail(RB_INVALID_TENSOR, "destinations are BF16 [world * rows, width]");
        p.dst[d] = static_cast<bf*>(pdst);
        p.flag[d] = pf + rank;
        if (pulls) {
            void* pp = nullptr;
            RB_TRY(resolve(ctx, pulls[d], "reduce+norm+push partial product", &pp));
            const rb_tensor* q = pulls[d];
            if (q->dtype != RB_BF16 || q->rank != 2 || q->shape[1] != width || q->shape[0] != rows * world)
                return fail(RB_INVALID_TENSOR, "partial products are BF16 [world * rows, width]");
            p.pull[d] = static_cast<const bf*>(pp) + (uint64_t)rank * rows * width;
            if (reinterpret_cast<uintptr_t>(p.pull[d]) % 16) return fail(RB_INVALID_TENSOR, "partial products must start on a 16-byte boundary");
        }
    }
    // Beside the compute stream's persistent GEMMs this kernel gets the SMs they leave free; alone it gets them all.
    const int sms = ctx->sm_limit > 0 ? (aux_active(ctx) ? ctx->sm_count - ctx->sm_limit : ctx->sm_limit) : ctx->sm_count;
    if (pulls) {
        // Every block keeps up to three rows of (world partial products + the residual row) in flight in shared memory, and an
        // SM takes as many blocks as fit, so that the stores of one row overlap the sum of another.  Measured against it at two
        // ranks and kept out: one block per SM with eight rows in flight (a pipelined Linear step took 229 us instead of
        // 128-167); two rows per block and more blocks, with the loads of all sources issued before the adds (the unpipelined
        // Linear step took 185 us instead of 172, the decoder forward 28.7 ms instead of 27.4-28.1).
        const uint64_t stage_bytes = (uint64_t)(world + (x_in ? 1 : 0)) * width * 2;
        const uint64_t budget = 222 * 1024;
        uint32_t stages = (uint32_t)(budget / stage_bytes);
        if (stages > 3u) stages = 3u;
        if (stages == 0) return fail(RB_INVALID_TENSOR, "pull form: one row of every rank's partial product (%llu bytes) does not fit shared memory", (unsigned long long)stage_bytes);
        p.stages = stages;
        const uint32_t smem = (uint32_t)(stages * stage_bytes + 128);
        uint64_t per_sm = budget / (smem + 1024);
        per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
        static std::once_flag once;
        static cudaError_t configured = cudaSuccess;
        std::call_once(once, [] {
            configured = cudaFuncSetAttribute(pull_reduce_norm_push_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 222 * 1024 + 128);
            if (configured == cudaSuccess) configured = cudaFuncSetAttribute(pull_reduce_norm_push_kernel<PUSH_MAXV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 222 * 1024 + 128);
        });
        if (configured != cudaSuccess) return fail(RB_STATUS, "cudaFuncSetAttribute(pull reduce+norm+push) failed with CUDA status %d (%s)", (int)configured, cudaGetErrorString(configured));
        const uint64_t cap = (uint64_t)(sms > 0 ? sms : 1) * per_sm;
        if (width <= (uint64_t)PUSH_THREADS * 2 * 8) pull_reduce_norm_push_kernel<2><<<(unsigned)(rows < cap ? rows : cap), PUSH_THREADS, smem, ctx->stream>>>(p);
        else pull_reduce_norm_push_kernel<PUSH_MAXV><<<(unsigned)(rows < cap ? rows : cap), PUSH_THREADS, smem, ctx->stream>>>(p);
        return after_launch(ctx, "reduce_norm_push (pull)");
    }
    const uint64_t cap = (uint64_t)(sms > 0 ? sms : 1) * 8;
    reduce_norm_push_kernel<<<(unsigned)(rows < cap ? rows : cap), PUSH_THREADS, 0, ctx->stream>>>(p);
    return after_launch(ctx, "reduce_norm_push");
}

}  // namespace

using namespace rb;

namespace {

// flags tensors are U8/I32 storage of (world + 1) 32-bit words; returns the device address.
int32_t resolve_flags(rb_ctx* ctx, const rb_tensor* t, uint32_t world, const char* what, uint32_t** out) {
    void* p = nullptr;
    RB_TRY(resolve(ctx, t, what, &p));
    if (t->dtype != RB_I32 || elements(t) < (uint64_t)world + 1) return fail(RB_INVALID_TENSOR, "%s must hold world + 1 INT32 words", what);
    *out = static_cast<uint32_t*>(p);
    return RB_OK;
}

}  // namespace

extern "C" {

int32_t rb_gemm_scatter(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* b, uint32_t rank, uint32_t world,
                        const rb_tensor* const* staging, const rb_tensor* const* flags) {
    return rb_gemm_scatter_bias(ctx, a, b, nullptr, rank, world, staging, flags);
}

int32_t rb_gemm_scatter_bias(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* b, const rb_tensor* bias, uint32_t rank, uint32_t world,
                             const rb_tensor* const* staging, const rb_tensor* const* flags) {
    RB_TRY(check_ctx(ctx));
    if (world < 1 || world > MAX_PEERS || rank >= world || !staging || !flags) return fail(RB_INVALID_TENSOR, "scatter GEMM needs 1..%d ranks and their staging and flag tensors", MAX_PEERS);
    void *pa, *pb;
    RB_TRY(resolve(ctx, a, "scatter GEMM A", &pa)); RB_TRY(resolve(ctx, b, "scatter GEMM B", &pb));
    if (a->rank != 2 || b->rank != 2 || a->dtype != RB_BF16 || b->dtype != RB_BF16 || a->shape[1] != b->shape[1])
        return fail(RB_INVALID_TENSOR, "scatter GEMM takes BF16 A [T, K] and B [H, K] (Linear layout)");
    const uint64_t m = a->shape[0], n = b->shape[0], k = a->shape[1];
    if (m == 0 || n == 0 || k == 0 || k % 16 || n % CHUNK || m % ((uint64_t)world * BM) || m > 0x7fffffffull || n > 0x7fffffffull || k > 0x7fffffffull)
        return fail(RB_INVALID_TENSOR, "scatter GEMM needs T a multiple of 128 * world, H a multiple of 64 and K a multiple of 16");
    ScatterParams p{};
    if (bias) {
        void* pbias = nullptr;
        RB_TRY(resolve(ctx, bias, "scatter GEMM bias", &pbias));
        if (bias->dtype != RB_F32 || elements(bias) != n) return fail(RB_INVALID_TENSOR, "scatter GEMM bias is FP32 [H]");
        p.bias = static_cast<const float*>(pbias);
    }
    p.m = (uint32_t)m; p.n = (uint32_t)n; p.k = (uint32_t)k; p.world = world; p.rows_per_owner = (uint32_t)(m / world);
    const uint64_t slot = (uint64_t)p.rows_per_owner * n * 2;
    for (uint32_t o = 0; o < world; ++o) {
        void* ps = nullptr; uint32_t* pf = nullptr;
        RB_TRY(resolve(ctx, staging[o], "scatter GEMM staging area", &ps));
        RB_TRY(resolve_flags(ctx, flags[o], world, "scatter GEMM flags", &pf));
        const rb_tensor* s = staging[o];
        if (s->dtype != RB_BF16 || s->rank != 3 || s->shape[0] != world || s->shape[1] != p.rows_per_owner || s->shape[2] != n)
            return fail(RB_INVALID_TENSOR, "scatter GEMM staging areas are BF16 [world, T / world, H]");
        p.dst[o] = static_cast<uint8_t*>(ps) + (uint64_t)rank * slot;
        p.flag[o] = pf + rank;
    }
    RB_TRY(kernel_status_word(ctx, &p.status));
    const int bn = n > 128 ? 256 : 128;
    CUtensorMap ma, mb;
    // Pairs of CTAs take 256 x 256 tiles; RUDA_GEMM_PAIRS=0 keeps every GEMM of the library on single CTAs.
    const char* pairs_env = std::getenv("RUDA_GEMM_PAIRS");
    if (bn == 256 && m % (2 * BM) == 0 && !(pairs_env && pairs_env[0] == '0')) {
        p.tiles_m = (uint32_t)(m / (2 * BM)); p.tiles_n = (uint32_t)((n + bn - 1) / bn);
        p.tile_shift = rb_scatter_shift(rank, world, p.rows_per_owner, 2 * BM);
        if (!operand_map(&ma, pa, m, k, BM) || !operand_map(&mb, pb, n, k, SP_BN / 2))
            return fail(RB_STATUS, "cuTensorMapEncodeTiled failed for a scatter GEMM operand (m=%u n=%u k=%u)", p.m, p.n, p.k);
        return launch_scatter_pair(ctx, ma, mb, p);
    }
    p.tiles_m = (uint32_t)(m / BM); p.tiles_n = (uint32_t)((n + bn - 1) / bn);
    p.tile_shift = rb_scatter_shift(rank, world, p.rows_per_owner, BM);
    if (!operand_map(&ma, pa, m, k, BM) || !operand_map(&mb, pb, n, k, bn))
        return fail(RB_STATUS, "cuTensorMapEncodeTiled failed for a scatter GEMM operand (m=%u n=%u k=%u)", p.m, p.n, p.k);
    return bn == 256 ? launch_scatter<256>(ctx, ma, mb, p) : launch_scatter<128>(ctx, ma, mb, p);
}

uint32_t rb_gemm_scatter_signals(uint64_t tokens, uint64_t hidden, uint32_t world) {
    if (world == 0 || tokens % ((uint64_t)world * BM)) return 0;
    const uint64_t bn = hidden > 128 ? 256 : 128;
    return (uint32_t)(tokens / world / BM * ((hidden + bn - 1) / bn) * 4);
}

int32_t rb_peer_wait(rb_ctx* ctx, const rb_tensor* flags, uint32_t world, uint32_t count) {
    RB_TRY(check_ctx(ctx));
    if (world < 1 || world > MAX_PEERS) return fail(RB_INVALID_TENSOR, "peer wait covers 1..%d ranks", MAX_PEERS);
    uint32_t* pf = nullptr; uint32_t* status = nullptr;
    RB_TRY(resolve_flags(ctx, flags, world, "peer wait flags", &pf));
    RB_TRY(kernel_status_word(ctx, &status));
    // Long enough for a peer whose host thread is late with its launch, short enough that a lost rank ends as an error.
    uint64_t limit_ms = 5000;
    if (const char* env = std::getenv("RUDA_PEER_WAIT_MS")) { const long v = std::atol(env); if (v > 0 && v <= 60000) limit_ms = (uint64_t)v; }
    peer_wait_kernel<<<1, 32, 0, ctx->stream>>>(pf, world, count, status, limit_ms * 1000000ull);
    return after_launch(ctx, "peer_wait");
}

int32_t rb_peer_signal(rb_ctx* ctx, uint32_t rank, uint32_t world, const rb_tensor* const* flags) {
    RB_TRY(check_ctx(ctx));
    if (world < 1 || world > MAX_PEERS || rank >= world || !flags) return fail(RB_INVALID_TENSOR, "peer signal covers 1..%d ranks", MAX_PEERS);
    SignalParams p{};
    p.world = world;
    for (uint32_t d = 0; d < world; ++d) {
        uint32_t* pf = nullptr;
        RB_TRY(resolve_flags(ctx, flags[d], world, "peer signal flags", &pf));
        p.flag[d] = pf + rank;
    }
    peer_signal_kernel<<<1, 32, 0, ctx->stream>>>(p);
    return after_launch(ctx, "peer_signal");
}

int32_t rb_scatter_rows(rb_ctx* ctx, const rb_tensor* partial, uint32_t rank, uint32_t world, const rb_tensor* const* staging,
                        const rb_tensor* const* flags, const rb_tensor* done) {
    RB_TRY(check_ctx(ctx));
    if (world < 1 || world > MAX_PEERS || rank >= world || !staging || !flags) return fail(RB_INVALID_TENSOR, "row scatter covers 1..%d ranks and needs their staging and flag tensors", MAX_PEERS);
    void *pp = nullptr, *pd = nullptr;
    RB_TRY(resolve(ctx, partial, "row scatter partial product", &pp)); RB_TRY(resolve(ctx, done, "row scatter block counter", &pd));
    if (partial->rank != 2 || partial->dtype != RB_BF16 || partial->shape[0] % world || partial->shape[1] % 8 || partial->shape[0] == 0 || partial->shape[0] > 0x7fffffffull)
        return fail(RB_INVALID_TENSOR, "row scatter takes a BF16 [world * rows, width] partial product with a width that is a multiple of 8");
    if (done->dtype != RB_I32 || elements(done) < 1) return fail(RB_INVALID_TENSOR, "block counter is one INT32 word");
    ScatterRowsParams p{};
    p.src = static_cast<const bf*>(pp);
    p.rows = (uint32_t)(partial->shape[0] / world); p.width = (uint32_t)partial->shape[1]; p.world = world; p.rank = rank;
    p.done = static_cast<uint32_t*>(pd);
    { uint32_t* st = nullptr; RB_TRY(kernel_status_word(ctx, &st)); p.status = st; }
    for (uint32_t o = 0; o < world; ++o) {
        void* ps = nullptr; uint32_t* pf = nullptr;
        RB_TRY(resolve(ctx, staging[o], "row scatter staging area", &ps));
        RB_TRY(resolve_flags(ctx, flags[o], world, "row scatter flags", &pf));
        const rb_tensor* t = staging[o];
        if (t->dtype != RB_BF16 || t->rank != 3 || t->shape[0] != world || t->shape[1] != p.rows || t->shape[2] != p.width)
            return fail(RB_INVALID_TENSOR, "staging areas are BF16 [world, rows, width]");
        p.dst[o] = static_cast<bf*>(ps) + (uint64_t)rank * p.rows * p.width;
        p.flag[o] = pf + rank;
    }
    // Beside the compute stream's persistent GEMMs this kernel gets the SMs they leave free; alone it gets them all.
    const int sms = ctx->sm_limit > 0 ? (aux_active(ctx) ? ctx->sm_count - ctx->sm_limit : ctx->sm_limit) : ctx->sm_count;
    const uint64_t cap = (uint64_t)(sms > 0 ? sms : 1) * 8, total = (uint64_t)p.rows * world;
    scatter_rows_kernel<<<(unsigned)(total < cap ? total : cap), 256, 0, ctx->stream>>>(p);
    return after_launch(ctx, "scatter_rows");
}

int32_t rb_reduce_norm_push(rb_ctx* ctx, const rb_tensor* staging, const rb_tensor* x_in, const rb_tensor* weight, double epsilon,
                            const rb_tensor* x_out, uint32_t rank, uint32_t world, const rb_tensor* const* destinations,
                            const rb_tensor* const* flags, const rb_tensor* done) {
    return reduce_norm_push_impl(ctx, staging, nullptr, x_in, weight, epsilon, x_out, rank, world, destinations, flags, done);
}

int32_t rb_reduce_norm_rows(rb_ctx* ctx, const rb_tensor* staging, const rb_tensor* x_in, const rb_tensor* weight, double epsilon,
                            const rb_tensor* x_out, const rb_tensor* out, const rb_tensor* done) {
    if (!staging || !out) return fail(RB_NULL_HANDLE, "reduce+norm of local rows needs the gathered partial products and an output");
    if (staging->rank != 3 || staging->shape[0] < 1 || staging->shape[0] > (uint64_t)MAX_PEERS) return fail(RB_INVALID_TENSOR, "staging area is BF16 [world, rows, width]");
    return reduce_norm_push_impl(ctx, staging, nullptr, x_in, weight, epsilon, x_out, 0, (uint32_t)staging->shape[0], nullptr, nullptr, done, out);
}

int32_t rb_reduce_norm_push_pull(rb_ctx* ctx, const rb_tensor* const* partials, const rb_tensor* x_in, const rb_tensor* weight, double epsilon,
                                 const rb_tensor* x_out, uint32_t rank, uint32_t world, const rb_tensor* const* destinations,
                                 const rb_tensor* const* flags, const rb_tensor* done) {
    if (!partials) return fail(RB_NULL_HANDLE, "pull form of reduce+norm+push needs every rank's partial product");
    return reduce_norm_push_impl(ctx, nullptr, partials, x_in, weight, epsilon, x_out, rank, world, destinations, flags, done);
}

}  // extern "C"
