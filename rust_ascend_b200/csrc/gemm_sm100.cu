// BF16 GEMM with FP32 accumulation on Blackwell tensor cores (tcgen05 + TMEM), fed by a multi-stage TMA ring.
//
// Replaces the reference's generated matrix program (rust-ascend-kernels/src/kernel.rs:11-76, persistent
// scheduler scheduler.rs:5-79, tile constants layout.rs:4-12) and its runtime entry points
// (rust-ascend-driver/src/tensor/runtime/matrix.rs:47-59).  The contract is the reference's
// (deepgemm/plan.rs:49-80): contiguous row-major BF16 operands, rank 2 or equal-batch rank 3, M/N/K positive
// multiples of 16, all four transpose combinations, BF16 or FP32 output.
//
// Design: one persistent CTA per SM walks output tiles of 128 x BN in a grouped raster.  Warp 0 is the TMA
// producer, warp 1 issues tcgen05.mma (UMMA 128 x BN x 16, operands K-major in 128-byte-swizzled shared
// memory), warps 2..5 are the epilogue.  Two TMEM accumulators let the epilogue of tile i overlap the
// main loop of tile i+1.  The epilogue is fused: identity, + bias[n], or SiLU(gate)*up where the gate and
// up projections are accumulated side by side in one UMMA of N = BN from two weight matrices.
// Tail wave: when the tiles left for the last round of the persistent loop would occupy at most half of the CTAs, each
// of them is cut into two half-width tiles (UMMA N = BN/2, loaded through half-height B boxes), so that the last round
// takes about half a tile's time on twice as many SMs instead of a full tile's time on a few (4096^3: 512 tiles on 148
// CTAs = 3 rounds + 68 tiles -> 136 half tiles).  No partial sums are exchanged; every output element is still the
// result of one accumulator in one fixed K order.
// Operands that are not K-major (A transposed, B not transposed) are first rewritten K-major by a tiled
// transpose kernel; the hot Linear layout (X [M,K], W [N,K]) needs no rewrite.
#include "common.cuh"

#include <cstdlib>
#include "schedule.h"
#include "sm100.cuh"

namespace {

using namespace sm100;
using bf = __nv_bfloat16;

constexpr int BM = 128;      // UMMA M (TMEM lanes)
constexpr int BK = 64;       // K per stage: 64 BF16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int GROUP_M = 8;   // raster group height in tiles
constexpr int THREADS = 192;

struct GemmParams {
    uint32_t m, n, k, batches;      // n = output columns
    uint32_t tiles_m, tiles_n;
    uint32_t split;                 // work items below this index are whole tiles; from it on, item = half of tile split + (i - split) / 2
    uint32_t items;                 // whole tiles + half tiles
    uint32_t epilogue;              // rb_epilogue
    uint32_t out_f32;               // output storage: 0 BF16, 1 FP32, 2 FP16
    uint32_t bias_bf16;             // bias storage: 1 BF16, 0 FP32
    uint32_t f16_operands;          // 1: the 16-bit operands are FP16 instead of BF16 (UMMA operand format)
    uint32_t ragged;                // 1: output rows are not multiples of 16 bytes, stored element by element
    // K passes: pass s multiplies part seg_a[s] of A with part seg_b[s] of B into the same accumulator (an FP32 operand
    // split into BF16 parts); an operand with `parts` parts stores them as consecutive batch entries: z = batch * parts + part
    uint32_t nseg, parts_a, parts_b;
    uint32_t seg_a[6], seg_b[6];
    uint32_t a_bcast, b_bcast;      // 1: the operand has one batch entry that every output batch uses
    const int32_t* group_ends;      // M-grouped NT: B's batch entry is the group that owns the tile's rows (row prefix sums); else null
    uint32_t groups;
    void* out;
    const void* bias;
    uint32_t* status;               // device status word: non-zero when a bounded wait expired
};

template <int BN> struct Config {
    static constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BIAS_BYTES = 4 * 2 * 256 * 4;  // per epilogue warp: two staged bias rows, one per accumulator in flight
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + BIAS_BYTES;
    static constexpr int TMEM_COLS = 2 * BN;
};

// Work item -> tile coordinates; `half` is 0 or 1 for a half-width tile and 2 for a whole tile.
__device__ __forceinline__ void tile_coords(uint32_t item, const GemmParams& p, uint32_t& batch, uint32_t& tm, uint32_t& tn, uint32_t& half) {
    uint32_t t; rb_gemm_item(item, p.split, t, half);
    rb_tile_coords(t, p.tiles_m, p.tiles_n, GROUP_M, batch, tm, tn);
}

__device__ __forceinline__ float bias_at(const GemmParams& p, uint32_t col) {
    return p.bias_bf16 ? __bfloat162float(static_cast<const bf*>(p.bias)[col]) : static_cast<const float*>(p.bias)[col];
}

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_b2, const __grid_constant__ CUtensorMap map_bh,
                 const __grid_constant__ CUtensorMap map_b2h, const GemmParams p) {
    using C = Config<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + C::STAGES;
    uint64_t* tmem_full = empty_bar + C::STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;
    float* bias_smem = reinterpret_cast<float*>(smem + C::STAGES * C::STAGE_BYTES + 256);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool swiglu = p.epilogue == RB_EPILOGUE_SWIGLU;
    const uint32_t bn_out = swiglu ? BN / 2 : BN;      // output columns of a whole tile
    const uint32_t num_kb = (p.k + BK - 1) / BK;
    const uint32_t total_kb = num_kb * p.nseg;          // K blocks of all passes
    const uint32_t num_tiles = p.items;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 128); }
        *abort_word = 0;
        fence_barrier_init();
        prefetch_tmap(&map_a); prefetch_tmap(&map_b); if (swiglu) prefetch_tmap(&map_b2);
        if (p.items > p.split) { prefetch_tmap(&map_bh); if (swiglu) prefetch_tmap(&map_b2h); }
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
                uint32_t batch, tm, tn, half; tile_coords(t, p, batch, tm, tn, half);
                const bool whole = half == 2;
                // B rows of this item: a whole tile takes bn_out rows of each weight, a half tile half as many, starting
                // in the middle of the tile's range for the second half.
                const uint32_t b_rows = whole ? bn_out : bn_out / 2;
                const int32_t b_row0 = (int32_t)(tn * bn_out + (whole ? 0 : half * b_rows));
                const uint32_t b_bytes = b_rows * BK * 2;
                const CUtensorMap* mb = whole ? &map_b : &map_bh;
                const CUtensorMap* mb2 = whole ? &map_b2 : &map_b2h;
                const uint32_t za0 = (p.a_bcast ? 0u : batch) * p.parts_a;
                uint32_t zb0 = (p.b_bcast ? 0u : batch) * p.parts_b;
                if (p.group_ends) zb0 = rb_group_of(p.group_ends, p.groups, tm * BM);
                for (uint32_t kt = 0; kt < total_kb; ++kt) {
                    const uint32_t seg = kt / num_kb, kb = kt - seg * num_kb;
                    const int32_t za = (int32_t)(za0 + p.seg_a[seg]), zb = (int32_t)(zb0 + p.seg_b[seg]);
                    if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_word))) break;
                    uint8_t* sa = smem + stage * C::STAGE_BYTES; uint8_t* sb = sa + C::A_BYTES;
                    mbar_expect_tx(&full_bar[stage], C::A_BYTES + (swiglu ? 2 * b_bytes : b_bytes));
                    armed |= 1u << stage; armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
                    tma_load_3d(sa, &map_a, &full_bar[stage], (int32_t)(kb * BK), (int32_t)(tm * BM), za);
                    tma_load_3d(sb, mb, &full_bar[stage], (int32_t)(kb * BK), b_row0, zb);
                    if (swiglu) tma_load_3d(sb + b_bytes, mb2, &full_bar[stage], (int32_t)(kb * BK), b_row0, zb);
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
            // FP16 operands clear the two operand-format fields (bits 7-9 and 10-12: 1 = BF16, 0 = FP16)
            const uint32_t fmt_mask = p.f16_operands ? ~((1u << 7) | (1u << 10)) : ~0u;
            const uint32_t idesc_whole = make_idesc_bf16(BM, BN) & fmt_mask, idesc_half = make_idesc_bf16(BM, BN / 2) & fmt_mask;
            uint32_t stage = 0, phase = 0, iter = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x, ++iter) {
                const uint32_t acc = iter & 1, acc_phase = (iter >> 1) & 1;
                const uint32_t idesc = t < p.split ? idesc_whole : idesc_half;
                if (!(ok = mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_word))) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (uint32_t kb = 0; kb < total_kb; ++kb) {
                    if (!(ok = mbar_wait(&full_bar[stage], phase, abort_word))) break;
                    tc_fence_after();
                    uint8_t* sa = smem + stage * C::STAGE_BYTES;
                    const uint64_t da = make_kmajor_sw128_desc(smem_u32(sa)), db = make_kmajor_sw128_desc(smem_u32(sa + C::A_BYTES));
#pragma unroll
                    for (uint32_t k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_ss(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);  // +32 bytes per K step
                    umma_commit(&empty_bar[stage]);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit(&tmem_full[acc]);
            }
        }
    } else {
        // ---------------- epilogue: 4 warps, one TMEM lane (= output row) per thread ----------------
        const uint32_t quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are the ones this warp may read
        uint32_t iter = 0;
        bool ok = true;
        for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x, ++iter) {
            const uint32_t acc = iter & 1, acc_phase = (iter >> 1) & 1;
            uint32_t batch, tm, tn, half; tile_coords(t, p, batch, tm, tn, half);
            const uint32_t width = half == 2 ? bn_out : bn_out / 2;                    // output columns of this item
            const uint32_t col0 = tn * bn_out + (half == 2 ? 0 : half * width);
            const uint32_t up_at = half == 2 ? BN / 2 : BN / 4;                         // TMEM column where the up half starts (SwiGLU)
            float* sbias = bias_smem + (quarter * 2 + acc) * 256;
            if (p.epilogue == RB_EPILOGUE_BIAS) {
                // Each warp stages this tile's bias row for itself (warp-level sync only, so no CTA barrier can
                // be left waiting if a bounded wait expires).
                for (uint32_t j = lane; j < width; j += 32) sbias[j] = col0 + j < p.n ? bias_at(p, col0 + j) : 0.f;
                __syncwarp();
            }
            ok = mbar_wait(&tmem_full[acc], acc_phase, abort_word);
            if (!(ok = __all_sync(0xffffffffu, ok))) break;  // keep the warp converged
            tc_fence_after();
            const uint32_t row = tm * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + acc * BN + ((quarter * 32) << 16);
            const size_t out_off = ((size_t)batch * p.m + row) * p.n;
            for (uint32_t c = 0; c < width; c += 32) {
                if (col0 + c >= p.n) break;  // warp-uniform
                uint32_t r[32];
                tmem_ld_32x32(taddr + c, r);
                float v[32];
                if (swiglu) {
                    uint32_t u[32];
                    tmem_ld_32x32(taddr + up_at + c, u);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float g = __uint_as_float(r[j]);
                        float s = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)));
                        v[j] = __fmul_rn(__fmul_rn(g, s), __uint_as_float(u[j]));
                    }
                } else {
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    if (p.epilogue == RB_EPILOGUE_BIAS) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __fadd_rn(v[j], sbias[c + j]);
                    }
                }
                if (row < p.m && p.ragged) {
                    // rows that are not multiples of 16 bytes: one element per store
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (col0 + c + j < p.n) {
                            const size_t at = out_off + col0 + c + j;
                            if (p.out_f32 == 1) static_cast<float*>(p.out)[at] = v[j];
                            else if (p.out_f32 == 2) static_cast<__half*>(p.out)[at] = __float2half_rn(v[j]);
                            else static_cast<bf*>(p.out)[at] = __float2bfloat16_rn(v[j]);
                        }
                    }
                } else if (row < p.m) {
                    if (p.out_f32 == 2) {
                        __half* o = static_cast<__half*>(p.out) + out_off + col0 + c;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            if (col0 + c + j < p.n) {
                                __half2 q0 = __floats2half2_rn(v[j], v[j + 1]), q1 = __floats2half2_rn(v[j + 2], v[j + 3]);
                                __half2 q2 = __floats2half2_rn(v[j + 4], v[j + 5]), q3 = __floats2half2_rn(v[j + 6], v[j + 7]);
                                uint4 w;
                                w.x = *reinterpret_cast<uint32_t*>(&q0); w.y = *reinterpret_cast<uint32_t*>(&q1);
                                w.z = *reinterpret_cast<uint32_t*>(&q2); w.w = *reinterpret_cast<uint32_t*>(&q3);
                                *reinterpret_cast<uint4*>(o + j) = w;
                            }
                        }
                    } else if (p.out_f32) {
                        float* o = static_cast<float*>(p.out) + out_off + col0 + c;
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            if (col0 + c + j < p.n) *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    } else {
                        bf* o = static_cast<bf*>(p.out) + out_off + col0 + c;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            if (col0 + c + j < p.n) {
                                __nv_bfloat162 q0 = __floats2bfloat162_rn(v[j], v[j + 1]), q1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                                __nv_bfloat162 q2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), q3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                                uint4 w;
                                w.x = *reinterpret_cast<uint32_t*>(&q0); w.y = *reinterpret_cast<uint32_t*>(&q1);
                                w.z = *reinterpret_cast<uint32_t*>(&q2); w.w = *reinterpret_cast<uint32_t*>(&q3);
                                *reinterpret_cast<uint4*>(o + j) = w;
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&tmem_empty[acc]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_word) atomicExch(p.status, 1u);
    if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, C::TMEM_COLS); }
}

// ---------------------------------------------------------------------------------------------------------------------
// The same GEMM on pairs of CTAs (cluster of two, tcgen05 cta_group::2): one MMA covers a 256 x BN tile, each CTA of the pair
// keeps 128 of its rows in its own TMEM and loads its own half of A and only HALF of B, since the tensor core reads the two
// halves of B from the two CTAs' shared memory.  Per output tile that is a third less traffic from L2 into shared memory than
// two independent 128 x BN tiles, and 32 KiB instead of 48 KiB per stage, so the ring is six stages deep instead of four.
// Rank 0 of the pair (the leader) issues the MMAs; every completion is broadcast to the barriers of both CTAs.  Every CTA
// fetches its own tiles (no cluster-broadcast load); it only reports their arrival to the leader's barrier.
// Tail round: as above, a last round that would use at most half of the pairs runs as tiles of half the width.
constexpr int PAIR_BN = 256;
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_A_BYTES = BM * BK * 2;                 // this CTA's 128 rows of A
constexpr int PAIR_B_BYTES = (PAIR_BN / 2) * BK * 2;      // this CTA's half of B
constexpr int PAIR_STAGE_BYTES = PAIR_A_BYTES + PAIR_B_BYTES;
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256 + 4 * 2 * 256 * 4;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_b2, const __grid_constant__ CUtensorMap map_bh,
                      const __grid_constant__ CUtensorMap map_b2h, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + PAIR_STAGES * PAIR_STAGE_BYTES);   // used in the leader only
    uint64_t* empty_bar = full_bar + PAIR_STAGES;                                               // one copy per CTA
    uint64_t* tmem_full = empty_bar + PAIR_STAGES;                                              // one copy per CTA
    uint64_t* tmem_empty = tmem_full + 2;                                                       // used in the leader only: 256 arrivals
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;
    float* bias_smem = reinterpret_cast<float*>(smem + PAIR_STAGES * PAIR_STAGE_BYTES + 256);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();               // 0: leader
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const bool swiglu = p.epilogue == RB_EPILOGUE_SWIGLU;
    const uint32_t bn_out = swiglu ? PAIR_BN / 2 : PAIR_BN;   // output columns of a whole tile
    const uint32_t num_kb = (p.k + BK - 1) / BK;
    const uint32_t num_tiles = p.items;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 256); }
        *abort_word = 0;
        fence_barrier_init();
        prefetch_tmap(&map_a); prefetch_tmap(&map_b); if (swiglu) prefetch_tmap(&map_b2);
        if (p.items > p.split) { prefetch_tmap(&map_bh); if (swiglu) prefetch_tmap(&map_b2h); }
    }
    if (warp == 1) { tmem_alloc_pair(tmem_slot, 2 * PAIR_BN); tmem_relinquish_pair(); }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();            // both CTAs' barriers exist before either reports to, or broadcasts into, the other
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer (one per CTA) ----------------
        if (elect_one()) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t t = pair; ok && t < num_tiles; t += pairs) {
                uint32_t batch, tm, tn, half; tile_coords(t, p, batch, tm, tn, half);
                const bool whole = half == 2;
                // this CTA's rows of B: whole tile 128, half tile 64; with SwiGLU rank 0 holds gate rows and rank 1 up rows
                const uint32_t b_rows = whole ? PAIR_BN / 2 : PAIR_BN / 4;
                const uint32_t out_w = whole ? bn_out : bn_out / 2;          // output columns of this item
                const uint32_t col0 = tn * bn_out + (whole ? 0 : half * out_w);
                const int32_t b_row0 = (int32_t)(swiglu ? col0 : col0 + rank * b_rows);
                const uint32_t b_bytes = b_rows * BK * 2;
                const CUtensorMap* mb = swiglu && rank == 1 ? (whole ? &map_b2 : &map_b2h) : (whole ? &map_b : &map_bh);
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_word))) break;
                    uint8_t* sa = smem + stage * PAIR_STAGE_BYTES; uint8_t* sb = sa + PAIR_A_BYTES;
                    const uint32_t leader_full = mapa_shared(smem_u32(&full_bar[stage]), 0);
                    if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * (PAIR_A_BYTES + b_bytes));   // the bytes of both CTAs
                    tma_load_3d_pair(sa, &map_a, leader_full, (int32_t)(kb * BK), (int32_t)(tm * 2 * BM + rank * BM), (int32_t)batch);
                    tma_load_3d_pair(sb, mb, leader_full, (int32_t)(kb * BK), b_row0, (int32_t)batch);
                    if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // A wait expired somewhere: give the copies in flight a bounded time to land before the CTA retires.
                for (uint32_t i = 0; i < (1u << 22); ++i) __nanosleep(32);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader only) ----------------
        if (rank == 0 && elect_one()) {
            const uint32_t idesc_whole = make_idesc_bf16(2 * BM, PAIR_BN), idesc_half = make_idesc_bf16(2 * BM, PAIR_BN / 2);
            uint32_t stage = 0, phase = 0, iter = 0;
            bool ok = true;
            for (uint32_t t = pair; ok && t < num_tiles; t += pairs, ++iter) {
                const uint32_t acc = iter & 1, acc_phase = (iter >> 1) & 1;
                const uint32_t idesc = t < p.split ? idesc_whole : idesc_half;
                if (!(ok = mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_word))) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * PAIR_BN;
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(&full_bar[stage], phase, abort_word))) break;
                    tc_fence_after();
                    uint8_t* sa = smem + stage * PAIR_STAGE_BYTES;
                    const uint64_t da = make_kmajor_sw128_desc(smem_u32(sa)), db = make_kmajor_sw128_desc(smem_u32(sa + PAIR_A_BYTES));
#pragma unroll
                    for (uint32_t k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_ss_pair(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    umma_commit_pair(&empty_bar[stage]);       // frees the stage in both CTAs
                    if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit_pair(&tmem_full[acc]);     // wakes the epilogue warps of both CTAs
            }
        }
    } else {
        // ---------------- epilogue: 4 warps per CTA, one TMEM lane (= output row) per thread ----------------
        const uint32_t quarter = warp & 3;
        uint32_t iter = 0;
        bool ok = true;
        for (uint32_t t = pair; ok && t < num_tiles; t += pairs, ++iter) {
            const uint32_t acc = iter & 1, acc_phase = (iter >> 1) & 1;
            uint32_t batch, tm, tn, half; tile_coords(t, p, batch, tm, tn, half);
            const bool whole = half == 2;
            const uint32_t width = whole ? bn_out : bn_out / 2;
            const uint32_t col0 = tn * bn_out + (whole ? 0 : half * width);
            const uint32_t up_at = whole ? PAIR_BN / 2 : PAIR_BN / 4;     // TMEM column where the up half starts (SwiGLU)
            float* sbias = bias_smem + (quarter * 2 + acc) * 256;
            if (p.epilogue == RB_EPILOGUE_BIAS) {
                for (uint32_t j = lane; j < width; j += 32) sbias[j] = col0 + j < p.n ? bias_at(p, col0 + j) : 0.f;
                __syncwarp();
            }
            ok = mbar_wait(&tmem_full[acc], acc_phase, abort_word);
            if (!(ok = __all_sync(0xffffffffu, ok))) break;
            tc_fence_after();
            const uint32_t row = tm * 2 * BM + rank * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + acc * PAIR_BN + ((quarter * 32) << 16);
            const size_t out_off = ((size_t)batch * p.m + row) * p.n;
            for (uint32_t c = 0; c < width; c += 32) {
                if (col0 + c >= p.n) break;  // warp-uniform
                uint32_t r[32];
                tmem_ld_32x32(taddr + c, r);
                float v[32];
                if (swiglu) {
                    uint32_t u[32];
                    tmem_ld_32x32(taddr + up_at + c, u);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float g = __uint_as_float(r[j]);
                        float sg = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)));
                        v[j] = __fmul_rn(__fmul_rn(g, sg), __uint_as_float(u[j]));
                    }
                } else {
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    if (p.epilogue == RB_EPILOGUE_BIAS) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __fadd_rn(v[j], sbias[c + j]);
                    }
                }
                if (row < p.m) {
                    if (p.out_f32) {
                        float* o = static_cast<float*>(p.out) + out_off + col0 + c;
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            if (col0 + c + j < p.n) *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    } else {
                        bf* o = static_cast<bf*>(p.out) + out_off + col0 + c;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            if (col0 + c + j < p.n) {
                                __nv_bfloat162 q0 = __floats2bfloat162_rn(v[j], v[j + 1]), q1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                                __nv_bfloat162 q2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), q3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                                uint4 w;
                                w.x = *reinterpret_cast<uint32_t*>(&q0); w.y = *reinterpret_cast<uint32_t*>(&q1);
                                w.z = *reinterpret_cast<uint32_t*>(&q2); w.w = *reinterpret_cast<uint32_t*>(&q3);
                                *reinterpret_cast<uint4*>(o + j) = w;
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            // hand the accumulator back to the leader's MMA thread: 128 arrivals from each CTA of the pair
            mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty[acc]), 0));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_word) atomicExch(p.status, 1u);
    cluster_sync_all();            // nothing may still be reporting to this CTA's barriers when its shared memory goes away
    if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc_pair(tmem_base, 2 * PAIR_BN); }
}

// Batched BF16 transpose [batches, R, C] -> [batches, C, R] through a padded shared-memory tile.
__global__ void __launch_bounds__(256) transpose_bf16_kernel(const uint16_t* in, uint16_t* out, uint32_t rows, uint32_t cols) {
    __shared__ uint16_t tile[64][66];
    const size_t base = (size_t)blockIdx.z * rows * cols;
    const uint32_t r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    for (uint32_t i = threadIdx.x; i < 64 * 64; i += 256) {
        uint32_t r = i / 64, c = i % 64;
        if (r0 + r < rows && c0 + c < cols) tile[r][c] = in[base + (size_t)(r0 + r) * cols + c0 + c];
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < 64 * 64; i += 256) {
        uint32_t c = i / 64, r = i % 64;
        if (r0 + r < rows && c0 + c < cols) out[base + (size_t)(c0 + c) * rows + r0 + r] = tile[r][c];
    }
}

struct GemmState { uint32_t* status = nullptr; bool attrs_set = false; bool pair_configured = false; uint32_t max_pairs = 0; int use_pairs = -1; };

template <int BN>
int32_t launch(rb_ctx* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2, const CUtensorMap& mbh,
               const CUtensorMap& mb2h, GemmParams& p) {
    using C = Config<BN>;
    // raised once per process and template instance; std::call_once makes the first use safe from any thread
    static std::once_flag once;
    static cudaError_t configured = cudaSuccess;
    std::call_once(once, [] { configured = cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES); });
    if (configured != cudaSuccess) return rb::fail(RB_STATUS, "cudaFuncSetAttribute(GEMM) failed with CUDA status %d (%s)", (int)configured, cudaGetErrorString(configured));
    const uint32_t sms = ctx->sm_limit > 0 ? (uint32_t)ctx->sm_limit : (uint32_t)ctx->sm_count;
    const uint32_t grid = p.items < sms ? p.items : sms;
    gemm_bf16_kernel<BN><<<grid, THREADS, C::SMEM_BYTES, ctx->stream>>>(ma, mb, mb2, mbh, mb2h, p);
    return rb::after_launch(ctx, "gemm");
}

// Decides whether the last round of the persistent loop runs as half-width tiles (see the note at the top of the file).
void plan_tail(rb_ctx* ctx, GemmParams& p, uint32_t bn_out) {
    const uint32_t sms = ctx->sm_limit > 0 ? (uint32_t)ctx->sm_limit : (uint32_t)ctx->sm_count;
    rb_gemm_plan(p.tiles_m * p.tiles_n * p.batches, sms, (bn_out / 2) % 32 == 0, p.split, p.items);
}

// Launch on CTA pairs.  The number of pairs that can be resident at once comes from the occupancy query for clusters (not
// every SM of the chip can be paired), capped by the context's SM limit.
int32_t launch_pair(rb_ctx* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2, const CUtensorMap& mbh,
                    const CUtensorMap& mb2h, GemmParams& p, uint32_t bn_out) {
    GemmState* st = static_cast<GemmState*>(ctx->gemm_state);
    if (!st->pair_configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES);
        if (e != cudaSuccess) return rb::fail(RB_STATUS, "cudaFuncSetAttribute(pair GEMM) failed with CUDA status %d (%s)", (int)e, cudaGetErrorString(e));
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(2 * (unsigned)ctx->sm_count, 1, 1); cfg.blockDim = dim3(THREADS, 1, 1); cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeClusterDimension; attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr; cfg.numAttrs = 1;
        int clusters = 0;
        e = cudaOccupancyMaxActiveClusters(&clusters, gemm_bf16_pair_kernel, &cfg);
        if (e != cudaSuccess || clusters < 1) return rb::fail(RB_STATUS, "cudaOccupancyMaxActiveClusters(pair GEMM) failed with CUDA status %d (%s)", (int)e, cudaGetErrorString(e));
        st->max_pairs = (uint32_t)clusters;
        st->pair_configured = true;
    }
    uint32_t pairs = st->max_pairs;
    if (ctx->sm_limit > 0 && (uint32_t)ctx->sm_limit / 2 < pairs) pairs = (uint32_t)ctx->sm_limit / 2;
    if (pairs == 0) pairs = 1;
    rb_gemm_plan(p.tiles_m * p.tiles_n * p.batches, pairs, (bn_out / 2) % 32 == 0, p.split, p.items);
    if (p.items < pairs) pairs = p.items;
    gemm_bf16_pair_kernel<<<2 * pairs, THREADS, PAIR_SMEM_BYTES, ctx->stream>>>(ma, mb, mb2, mbh, mb2h, p);
    return rb::after_launch(ctx, "gemm (CTA pairs)");
}

bool make_operand_map(CUtensorMap* map, const void* base, uint64_t batches, uint64_t rows, uint64_t k, uint32_t box_rows) {
    uint64_t dims[3] = {k, rows, batches};
    uint64_t strides[2] = {k * 2, rows * k * 2};
    uint32_t box[3] = {BK, box_rows, 1};
    return encode_bf16_map(map, base, 3, dims, strides, box, true);
}

}  // namespace

using namespace rb;

namespace rb {

// Device status word shared by the tensor-core kernels; non-zero after a bounded wait expired.
int32_t kernel_status_word(rb_ctx* ctx, uint32_t** out) {
    GemmState* st = static_cast<GemmState*>(ctx->gemm_state);
    if (!st) { st = new GemmState(); ctx->gemm_state = st; }
    if (!st->status) {
        cudaError_t e = cudaMalloc(&st->status, 256);
        if (e == cudaSuccess) e = cudaMemset(st->status, 0, 256);
        if (e != cudaSuccess) return fail(RB_STATUS, "status word allocation failed with CUDA status %d", (int)e);
    }
    *out = st->status;
    return RB_OK;
}

// Reads the status word after the stream has drained; a non-zero value becomes a sticky error.
int32_t poll_kernel_status(rb_ctx* ctx) {
    GemmState* st = static_cast<GemmState*>(ctx->gemm_state);
    if (!st || !st->status) return RB_OK;
    uint32_t h = 0;
    if (cudaMemcpy(&h, st->status, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return RB_OK;
    if (h) {
        cudaMemset(st->status, 0, sizeof(h));
        std::lock_guard<std::mutex> g(ctx->lock);
        ctx->sticky.emplace_back(h == 2 ? std::string("a bounded wait ran out (status word = 2: a peer's announcement never arrived, or a barrier inside the "
                                                      "attention kernel was never completed); the outputs of this step are invalid")
                                        : std::string("a tensor-core kernel gave up on a bounded barrier wait (status word = 1); its output is invalid"));
    }
    return RB_OK;
}

int32_t gemm_run(rb_ctx* ctx, const GemmCall& c) {
    GemmParams p{};
    p.m = c.m; p.n = c.n; p.k = c.k; p.batches = c.batches; p.epilogue = (uint32_t)c.epilogue; p.out_f32 = c.out_kind; p.bias_bf16 = c.bias_bf16;
    p.out = c.out; p.bias = c.bias;
    p.f16_operands = c.f16_operands; p.ragged = c.ragged; p.nseg = c.nseg; p.parts_a = c.parts_a; p.parts_b = c.parts_b;
    for (int i = 0; i < 6; ++i) { p.seg_a[i] = c.seg_a[i]; p.seg_b[i] = c.seg_b[i]; }
    p.a_bcast = c.a_bcast; p.b_bcast = c.b_bcast; p.group_ends = c.group_ends; p.groups = c.groups;
    RB_TRY(kernel_status_word(ctx, &p.status));
    const bool swiglu = c.epilogue == RB_EPILOGUE_SWIGLU;
    // Tile width: the widest accumulator that does not leave most of the tile empty.
    int bn = c.n > 128 || swiglu ? 256 : (c.n > 64 ? 128 : 64);
    if (swiglu && c.n <= 64) bn = 128;
    const uint32_t bn_out = swiglu ? bn / 2 : bn;
    GemmState* st = static_cast<GemmState*>(ctx->gemm_state);
    { const char* env = std::getenv("RUDA_GEMM_PAIRS"); st->use_pairs = env && env[0] == '0' ? 0 : 1; }   // RUDA_GEMM_PAIRS=0 keeps every GEMM on single CTAs
    // CTA pairs take the plain shapes of the hot path: wide outputs, one K pass, BF16 operands, 16-byte rows.
    const bool pairs_ok = st->use_pairs == 1 && bn == 256 && c.m >= 256 && c.nseg == 1 && !c.group_ends && !c.f16_operands && !c.ragged &&
                          c.out_kind <= 1 && !c.a_bcast && !c.b_bcast && c.parts_a == 1 && c.parts_b == 1;
    if (pairs_ok) {
        p.tiles_m = (c.m + 2 * BM - 1) / (2 * BM); p.tiles_n = (c.n + bn_out - 1) / bn_out;
        const uint64_t ar2 = c.a_rows ? c.a_rows : c.m, br2 = c.b_rows ? c.b_rows : c.n;
        CUtensorMap ma, mb, mb2, mbh, mb2h;
        if (!make_operand_map(&ma, c.a, c.batches, ar2, c.k, BM) || !make_operand_map(&mb, c.b, c.batches, br2, c.k, PAIR_BN / 2) ||
            !make_operand_map(&mb2, swiglu ? c.b_up : c.b, c.batches, br2, c.k, PAIR_BN / 2) || !make_operand_map(&mbh, c.b, c.batches, br2, c.k, PAIR_BN / 4) ||
            !make_operand_map(&mb2h, swiglu ? c.b_up : c.b, c.batches, br2, c.k, PAIR_BN / 4))
            return fail(RB_STATUS, "cuTensorMapEncodeTiled failed for a GEMM operand (m=%u n=%u k=%u)", c.m, c.n, c.k);
        return launch_pair(ctx, ma, mb, mb2, mbh, mb2h, p, bn_out);
    }
    p.tiles_m = (c.m + BM - 1) / BM; p.tiles_n = (c.n + bn_out - 1) / bn_out;
    plan_tail(ctx, p, bn_out);
    const uint64_t za = (uint64_t)(c.a_bcast ? 1 : c.batches) * c.parts_a;
    const uint64_t zb = c.group_ends ? c.groups : (uint64_t)(c.b_bcast ? 1 : c.batches) * c.parts_b;
    const uint64_t ar = c.a_rows ? c.a_rows : c.m, br = c.b_rows ? c.b_rows : c.n;
    CUtensorMap ma, mb, mb2, mbh, mb2h;
    if (!make_operand_map(&ma, c.a, za, ar, c.k, BM) || !make_operand_map(&mb, c.b, zb, br, c.k, bn_out) ||
        !make_operand_map(&mb2, swiglu ? c.b_up : c.b, zb, br, c.k, bn_out) || !make_operand_map(&mbh, c.b, zb, br, c.k, bn_out / 2) ||
        !make_operand_map(&mb2h, swiglu ? c.b_up : c.b, zb, br, c.k, bn_out / 2))
        return fail(RB_STATUS, "cuTensorMapEncodeTiled failed for a GEMM operand (m=%u n=%u k=%u)", c.m, c.n, c.k);
    if (bn == 256) return launch<256>(ctx, ma, mb, mb2, mbh, mb2h, p);
    if (bn == 128) return launch<128>(ctx, ma, mb, mb2, mbh, mb2h, p);
    return launch<64>(ctx, ma, mb, mb2, mbh, mb2h, p);
}

// C[batches, m, n] = A_k[batches, m, k] * B_k[batches, n, k]^T with both operands already K-major.
int32_t gemm_kmajor(rb_ctx* ctx, const void* a, const void* b, const void* b_up, uint32_t batches, uint32_t m, uint32_t n, uint32_t k,
                    int epilogue, const void* bias, bool bias_bf16, void* out, bool out_f32) {
    GemmCall c;
    c.a = a; c.b = b; c.b_up = b_up; c.batches = batches; c.m = m; c.n = n; c.k = k; c.epilogue = epilogue; c.bias = bias; c.bias_bf16 = bias_bf16;
    c.out = out; c.out_kind = out_f32 ? 1 : 0;
    return gemm_run(ctx, c);
}

}  // namespace rb

namespace {

int32_t matrix_dims(const rb_tensor* t, const char* what, uint64_t* batches, uint64_t* rows, uint64_t* cols) {
    if (t->rank != 2 && t->rank != 3) return fail(RB_INVALID_TENSOR, "%s: GEMM operands are rank 2 or equal-batch rank 3", what);
    *batches = t->rank == 3 ? t->shape[0] : 1; *rows = t->shape[t->rank - 2]; *cols = t->shape[t->rank - 1];
    return RB_OK;
}

}  // namespace

extern "C" {

int32_t rb_gemm(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* b, int32_t transpose_a, int32_t transpose_b,
                const rb_tensor* bias, const rb_tensor* b_up, int32_t epilogue, const rb_tensor* out) {
    RB_TRY(check_ctx(ctx));
    void *pa, *pb, *pbias = nullptr, *pup = nullptr, *po;
    RB_TRY(resolve(ctx, a, "GEMM A", &pa)); RB_TRY(resolve(ctx, b, "GEMM B", &pb)); RB_TRY(resolve(ctx, out, "GEMM output", &po));
    if (a->dtype != RB_BF16 || b->dtype != RB_BF16) return fail(RB_INVALID_TENSOR, "native GEMM requires BF16 operands");
    if (out->dtype != RB_BF16 && out->dtype != RB_F32) return fail(RB_INVALID_TENSOR, "GEMM output must be BF16 or FP32");
    uint64_t ba, ra, ca, bb, rbw, cb, bo, ro, co;
    RB_TRY(matrix_dims(a, "GEMM A", &ba, &ra, &ca)); RB_TRY(matrix_dims(b, "GEMM B", &bb, &rbw, &cb)); RB_TRY(matrix_dims(out, "GEMM output", &bo, &ro, &co));
    const uint64_t m = transpose_a ? ca : ra, k = transpose_a ? ra : ca;
    const uint64_t n = transpose_b ? rbw : cb, kb = transpose_b ? cb : rbw;
    if (a->rank != b->rank || a->rank != out->rank || ba != bb || ba != bo || k != kb || ro != m || co != n)
        return fail(RB_INVALID_TENSOR, "GEMM shapes do not agree: A gives M=%llu K=%llu, B gives N=%llu K=%llu, output is %llux%llu",
                    (unsigned long long)m, (unsigned long long)k, (unsigned long long)n, (unsigned long long)kb, (unsigned long long)ro, (unsigned long long)co);
    if (m == 0 || n == 0 || k == 0 || m % 16 || n % 16 || k % 16 || m > 0x7fffffffull || n > 0x7fffffffull || k > 0x7fffffffull)
        return fail(RB_INVALID_TENSOR, "GEMM M/N/K must be positive multiples of 16 within INT32_MAX");
    if (ba == 0 || ba > 4096) return fail(RB_INVALID_TENSOR, "GEMM batch count must be within 1..4096");
    if (epilogue != RB_EPILOGUE_NONE && epilogue != RB_EPILOGUE_BIAS && epilogue != RB_EPILOGUE_SWIGLU) return fail(RB_INVALID_TENSOR, "unknown GEMM epilogue");
    if (epilogue == RB_EPILOGUE_BIAS) {
        RB_TRY(resolve(ctx, bias, "GEMM bias", &pbias));
        if (elements(bias) != n || (bias->dtype != RB_F32 && bias->dtype != RB_BF16)) return fail(RB_INVALID_TENSOR, "GEMM bias must hold N FP32 or BF16 values");
    }
    if (epilogue == RB_EPILOGUE_SWIGLU) {
        RB_TRY(resolve(ctx, b_up, "GEMM up weight", &pup));
        if (!same_shape(b, b_up) || b_up->dtype != RB_BF16) return fail(RB_INVALID_TENSOR, "SwiGLU epilogue needs an up weight with the gate weight's shape and dtype");
    }
    const uint64_t a_bytes = ba * m * k * 2, b_bytes = ba * n * k * 2, o_bytes = ba * m * n * dtype_size(out->dtype);
    RB_TRY(no_overlap(po, o_bytes, pa, a_bytes, "GEMM")); RB_TRY(no_overlap(po, o_bytes, pb, b_bytes, "GEMM"));
    if (pup) RB_TRY(no_overlap(po, o_bytes, pup, b_bytes, "GEMM"));
    // Operands that are not K-major are rewritten K-major in the context workspace.
    const bool fix_a = transpose_a != 0, fix_b = transpose_b == 0;
    uint64_t need = (fix_a ? a_bytes : 0) + (fix_b ? b_bytes * (pup ? 2 : 1) : 0);
    if (need) RB_TRY(ensure_workspace(ctx, need + 1024));
    uint8_t* ws = static_cast<uint8_t*>(ctx->workspace) + 256;  // the first 256 bytes hold small flags
    const void *ka = pa, *kbp = pb, *kup = pup;
    if (fix_a) {  // stored [K, M] -> [M, K]
        dim3 grid((unsigned)((m + 63) / 64), (unsigned)((k + 63) / 64), (unsigned)ba);
        transpose_bf16_kernel<<<grid, 256, 0, ctx->stream>>>((const uint16_t*)pa, (uint16_t*)ws, (uint32_t)k, (uint32_t)m);
        RB_TRY(after_launch(ctx, "gemm operand transpose")); ka = ws; ws += a_bytes;
    }
    if (fix_b) {  // stored [K, N] -> [N, K]
        dim3 grid((unsigned)((n + 63) / 64), (unsigned)((k + 63) / 64), (unsigned)ba);
        transpose_bf16_kernel<<<grid, 256, 0, ctx->stream>>>((const uint16_t*)pb, (uint16_t*)ws, (uint32_t)k, (uint32_t)n);
        RB_TRY(after_launch(ctx, "gemm operand transpose")); kbp = ws; ws += b_bytes;
        if (pup) {
            transpose_bf16_kernel<<<grid, 256, 0, ctx->stream>>>((const uint16_t*)pup, (uint16_t*)ws, (uint32_t)k, (uint32_t)n);
            RB_TRY(after_launch(ctx, "gemm operand transpose")); kup = ws;
        }
    }
    return gemm_kmajor(ctx, ka, kbp, kup, (uint32_t)ba, (uint32_t)m, (uint32_t)n, (uint32_t)k, epilogue, pbias,
                       bias && bias->dtype == RB_BF16, po, out->dtype == RB_F32);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------
// Allocation-free GEMM entry point.
//
// Some hosts of this library may not allocate device memory once they are running: an inference server whose
// memory budget is fixed and audited at start-up, a real-time loop that cannot afford the device-wide
// synchronisation hidden in cudaMalloc/cudaFree, or a process that hands all remaining memory to another pool
// and would simply get an out-of-memory error.  rb_gemm needs scratch memory in two places (the K-major rewrite
// of an operand stored the other way round, and the status word the kernel raises when a bounded wait expires)
// and takes both from cudaMalloc.  rb_gemm_no_alloc takes them from the array below instead, which is part of
// the loaded module: every GPU that loads the library holds these 16 MiB + 256 B until the process exits.
// ---------------------------------------------------------------------------------------------------------
#define RB_NO_ALLOC_SCRATCH_BYTES (16ull << 20)
static __device__ __align__(256) uint8_t g_no_alloc_scratch[256 + RB_NO_ALLOC_SCRATCH_BYTES];
// Device address of g_no_alloc_scratch per CUDA ordinal.  In host code the array's name is only a stand-in
// for the symbol, not an address a kernel can use; the real address comes from cudaGetSymbolAddress.
static uint8_t* g_no_alloc_scratch_address[64] = {};

extern "C" int32_t rb_gemm_no_alloc(rb_ctx* ctx, const rb_tensor* a, const rb_tensor* b, int32_t transpose_a, int32_t transpose_b,
                                    const rb_tensor* out) {
    RB_TRY(check_ctx(ctx));
    // This call drains the stream and reads the status word back; while rb_graph_begin is recording that would break the
    // recording and leave the context unusable, so it is refused up front.
    if (ctx->capturing) return fail(RB_INVALID_TENSOR, "rb_gemm_no_alloc synchronises the stream and cannot run while rb_graph_begin is recording");
    int current = -1;
    RB_CUDA(ctx, "cudaGetDevice", cudaGetDevice(&current));
    if (current != ctx->device || current < 0 || current >= 64)
        return fail(RB_INVALID_DEVICE, "rb_gemm_no_alloc: make the context's device (%d) current on the calling thread (current is %d)", ctx->device, current);
    // One-time set-up per device, with that device current: resolve the symbol to its device address.
    if (!g_no_alloc_scratch_address[current]) {
        void* address = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&address, g_no_alloc_scratch);
        if (e != cudaSuccess || !address)
            return fail(RB_STATUS, "rb_gemm_no_alloc: cudaGetSymbolAddress failed with CUDA status %d (%s)", (int)e, cudaGetErrorString(e));
        g_no_alloc_scratch_address[current] = static_cast<uint8_t*>(address);
    }
    uint8_t* scratch = g_no_alloc_scratch_address[current];

    void *pa, *pb, *po;
    RB_TRY(resolve(ctx, a, "GEMM A", &pa)); RB_TRY(resolve(ctx, b, "GEMM B", &pb)); RB_TRY(resolve(ctx, out, "GEMM output", &po));
    if (a->dtype != RB_BF16 || b->dtype != RB_BF16) return fail(RB_INVALID_TENSOR, "native GEMM requires BF16 operands");
    if (out->dtype != RB_BF16 && out->dtype != RB_F32) return fail(RB_INVALID_TENSOR, "GEMM output must be BF16 or FP32");
    uint64_t ba, ra, ca, bb, rbw, cb, bo, ro, co;
    RB_TRY(matrix_dims(a, "GEMM A", &ba, &ra, &ca)); RB_TRY(matrix_dims(b, "GEMM B", &bb, &rbw, &cb)); RB_TRY(matrix_dims(out, "GEMM output", &bo, &ro, &co));
    const uint64_t m = transpose_a ? ca : ra, k = transpose_a ? ra : ca;
    const uint64_t n = transpose_b ? rbw : cb, kb = transpose_b ? cb : rbw;
    if (a->rank != b->rank || a->rank != out->rank || ba != bb || ba != bo || k != kb || ro != m || co != n)
        return fail(RB_INVALID_TENSOR, "GEMM shapes do not agree");
    if (m == 0 || n == 0 || k == 0 || m % 16 || n % 16 || k % 16 || m > 0x7fffffffull || n > 0x7fffffffull || k > 0x7fffffffull)
        return fail(RB_INVALID_TENSOR, "GEMM M/N/K must be positive multiples of 16 within INT32_MAX");
    if (ba == 0 || ba > 4096) return fail(RB_INVALID_TENSOR, "GEMM batch count must be within 1..4096");
    const uint64_t a_bytes = ba * m * k * 2, b_bytes = ba * n * k * 2, o_bytes = ba * m * n * dtype_size(out->dtype);
    RB_TRY(no_overlap(po, o_bytes, pa, a_bytes, "GEMM")); RB_TRY(no_overlap(po, o_bytes, pb, b_bytes, "GEMM"));
    const bool fix_a = transpose_a != 0, fix_b = transpose_b == 0;
    const uint64_t need = (fix_a ? a_bytes : 0) + (fix_b ? b_bytes : 0);
    if (need > RB_NO_ALLOC_SCRATCH_BYTES)
        return fail(RB_INVALID_TENSOR, "rb_gemm_no_alloc: the operands stored against the K-major layout need %llu bytes of scratch, the built-in "
                    "array holds %llu; use rb_gemm, or store A as [M,K] and B as [N,K]", (unsigned long long)need, (unsigned long long)RB_NO_ALLOC_SCRATCH_BYTES);

    // The array keeps whatever the previous call left in it.  Only the status word must start at zero; the
    // operand rewrites below overwrite every byte they later read.
    uint32_t* status = reinterpret_cast<uint32_t*>(scratch);
    RB_CUDA(ctx, "cudaMemsetAsync", cudaMemsetAsync(status, 0, 256, ctx->stream));
    uint8_t* ws = scratch + 256;
    const void *ka = pa, *kbp = pb;
    if (fix_a) {
        dim3 grid((unsigned)((m + 63) / 64), (unsigned)((k + 63) / 64), (unsigned)ba);
        transpose_bf16_kernel<<<grid, 256, 0, ctx->stream>>>((const uint16_t*)pa, (uint16_t*)ws, (uint32_t)k, (uint32_t)m);
        RB_TRY(after_launch(ctx, "gemm operand transpose")); ka = ws; ws += a_bytes;
    }
    if (fix_b) {
        dim3 grid((unsigned)((n + 63) / 64), (unsigned)((k + 63) / 64), (unsigned)ba);
        transpose_bf16_kernel<<<grid, 256, 0, ctx->stream>>>((const uint16_t*)pb, (uint16_t*)ws, (uint32_t)k, (uint32_t)n);
        RB_TRY(after_launch(ctx, "gemm operand transpose")); kbp = ws;
    }
    GemmParams p{};
    p.m = (uint32_t)m; p.n = (uint32_t)n; p.k = (uint32_t)k; p.batches = (uint32_t)ba; p.epilogue = RB_EPILOGUE_NONE;
    p.out_f32 = out->dtype == RB_F32; p.out = po; p.status = status;
    p.nseg = 1; p.parts_a = 1; p.parts_b = 1;
    const int bn = n > 128 ? 256 : (n > 64 ? 128 : 64);
    p.tiles_m = (p.m + BM - 1) / BM; p.tiles_n = (p.n + bn - 1) / bn;
    plan_tail(ctx, p, (uint32_t)bn);
    CUtensorMap ma, mb, mbh;
    if (!make_operand_map(&ma, ka, ba, m, k, BM) || !make_operand_map(&mb, kbp, ba, n, k, (uint32_t)bn) || !make_operand_map(&mbh, kbp, ba, n, k, (uint32_t)bn / 2))
        return fail(RB_STATUS, "cuTensorMapEncodeTiled failed for a GEMM operand");
    int32_t launched = bn == 256 ? launch<256>(ctx, ma, mb, mb, mbh, mbh, p) : (bn == 128 ? launch<128>(ctx, ma, mb, mb, mbh, mbh, p) : launch<64>(ctx, ma, mb, mb, mbh, mbh, p));
    RB_TRY(launched);
    // Report an expired wait without any state outside the array: drain the stream and read the status word.
    ctx->stats.synchronizations++;
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) { ctx->poisoned = true; return fail(RB_COMPLETION, "rb_gemm_no_alloc: completion failed with CUDA status %d (%s)", (int)e, cudaGetErrorString(e)); }
    uint32_t raised = 0;
    RB_CUDA(ctx, "cudaMemcpy(status)", cudaMemcpy(&raised, status, sizeof(raised), cudaMemcpyDeviceToHost));
    if (raised) return fail(RB_COMPLETION, "rb_gemm_no_alloc: the kernel gave up on a bounded barrier wait; the output is invalid");
    return RB_OK;
}
