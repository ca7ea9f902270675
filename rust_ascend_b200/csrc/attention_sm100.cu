// Flash-style attention forward on Blackwell tensor cores (tcgen05 + TMEM), head dim 128, BF16 in/out.
//
// Stands in for the reference's composed attention (src/nn/attention.rs:10-80): S = scale * bf16(Q) bf16(K)^T,
// causal predicate key_start+k > query_start+q (mask_programs.rs:30-37), softmax in FP32, O = bf16(P) bf16(V),
// grouped-query mapping kv_head = q_head / (Hq/Hkv) (heads_programs.rs:48-52).  Nothing is materialised: no
// score matrix, no mask tensor, no repeated KV heads.
//
// Persistent kernel, one CTA per SM.  A work item is 256 query rows of one (batch, head), handled as two 128-row tiles
// that ping-pong on the tensor core; items are numbered heaviest first (under a causal mask the last query blocks see the
// most keys); see schedule.h for the order in which the CTAs take them.  Roles (384 threads, twelve warps: four control warps and
// two softmax warpgroups; the order of the groups is a build option):
//   softmax warps    four for tile 0, four for tile 1: one query row per thread, running max and sum in FP32, exp2 with the
//                    scale folded in, P written back to TMEM as BF16 over the scores, handed to the MMA warp in two halves;
//                    at the end of an item the same warps normalise O and store it, while the TMA and MMA warps already
//                    load and multiply the first key block of the next item
//   TMA warp          Q of the next item as soon as the last score GEMM of this one has read it, K and V
//                    tiles of 128 keys through two 2-stage rings
//   MMA warp         issues tcgen05.mma:  S_t = Q_t K^T (operands in shared memory),  O_t += P_t V (P from TMEM, V consumed
//                    as stored, Dv-contiguous)
//   two more warps   idle; they only donate their registers to the softmax warps (setmaxnreg)
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_t aliases the first 64 columns of S_t.
// The running maximum is only refreshed when it grows by more than 2^8 (the accumulator and the sum are then rescaled),
// so most key blocks need no pass over O.  A key block that the causal rule or the end of the keys cuts is processed in
// 32-key chunks whose class (all visible / partly / none) is the same for the whole warp, so that only the partly visible
// chunk runs predicated code and hidden chunks cost no exponentials.
#include "common.cuh"
#include "schedule.h"
#include "sm100.cuh"

namespace {

using namespace sm100;
using bf = __nv_bfloat16;

constexpr int D = 128;            // head dim (Q/K) and value dim
constexpr int TQ = 128;           // query rows per tile
constexpr int TK = 128;           // keys per block
constexpr int KV_STAGES = 2;
constexpr int THREADS = 384;
// Warp roles.  The warp that issues the MMAs is a single thread with a long dependent instruction stream; which warp slot it
// sits in decides how often the scheduler lets it issue beside the two busy softmax warps of its SM sub-partition
// (-DRB_ATTN_MMA_LAST puts the control warps behind the softmax warps instead of in front of them).
#ifdef RB_ATTN_MMA_LAST
constexpr uint32_t W_SOFTMAX = 0, W_CONTROL = 8;
#else
constexpr uint32_t W_SOFTMAX = 4, W_CONTROL = 0;
#endif
constexpr uint32_t W_MMA = W_CONTROL, W_TMA = W_CONTROL + 1;   // the other two control warps only donate registers
constexpr int TILE_BYTES = 128 * D * 2;       // 32 KiB: one [128 x 128] BF16 tile = two 64-wide swizzle slabs
constexpr int SLAB_BYTES = 128 * 64 * 2;      // 16 KiB
constexpr int ITEM_TAB = 512;                 // steps whose items are tabulated in shared memory; later steps compute theirs
constexpr int SMEM_BYTES = 2 * TILE_BYTES + 2 * KV_STAGES * TILE_BYTES + 1024 + 256 + ITEM_TAB * 16;
#ifdef RB_ATTN_TILE0_FIRST
constexpr uint32_t FIRST_TILE = 0;
#else
constexpr uint32_t FIRST_TILE = 1;
#endif                                        // tile served first in every round of the ping-pong: under a causal mask tile 1 has one key
                                              // block more than tile 0, so it leads and its extra block overlaps tile 0's lag

struct AttnParams {
    uint32_t B, Hq, Hkv, M, N;
    uint32_t items, heads_total;  // work items = query block pairs x B x Hq; heads_total = B * Hq
    uint32_t q_blocks;            // 256-row query blocks per head
    uint32_t wave_heads;          // heads per wave of the item order
    float scale_log2;             // scale * log2(e)
    int32_t causal;
    int64_t delta;                // query_start - key_start (saturated): key k is masked iff k > q + delta
    void* out; uint64_t o_stride_b, o_stride_h, o_stride_m;  // BF16 or FP32 (kernel template); strides in elements
    const float* mask;            // additive FP32 [B*Hq, M, N] or null (kernel template)
    uint32_t* status;
};

constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r;
}

// Number of key blocks tile rows [row0, row_end) must visit.
__device__ __forceinline__ uint32_t blocks_for(const AttnParams& p, uint32_t row0, uint32_t row_end) {
    return rb_attention_blocks(p.M, p.N, p.causal, p.delta, row0, row_end, TK);
}
// Work item -> (query block, head, batch): heaviest query blocks first, heads of one KV group next to each other.
// One work item of this CTA: (query block | valid << 31, head | batch << 16, key blocks of tile 0, key blocks of tile 1).
__device__ __forceinline__ uint4 make_item(const AttnParams& p, uint32_t step) {
    uint32_t qb = 0, h = 0, b = 0;
    const bool valid = rb_attention_item(step, blockIdx.x, gridDim.x, p.q_blocks, p.heads_total, p.Hq, p.wave_heads, qb, h, b);
    const uint32_t row0 = qb * 2 * TQ;
    return make_uint4(qb | (valid ? 0x80000000u : 0u), h | (b << 16), valid ? blocks_for(p, row0, row0 + TQ) : 0u,
                      valid ? blocks_for(p, row0 + TQ, row0 + 2 * TQ) : 0u);
}
// The same item for a step beyond the table: a real call, so that the index arithmetic (divisions, 64-bit compares) does not
// become part of the roles' loops, whose single issuing threads have few registers.  Only very large problems get here.
__device__ __noinline__ uint4 make_item_late(uint32_t step, uint32_t q_blocks, uint32_t heads_total, uint32_t Hq, uint32_t wave_heads,
                                             uint32_t M, uint32_t N, int32_t causal, int64_t delta) {
    uint32_t qb = 0, h = 0, b = 0;
    const bool valid = rb_attention_item(step, blockIdx.x, gridDim.x, q_blocks, heads_total, Hq, wave_heads, qb, h, b);
    const uint32_t row0 = qb * 2 * TQ;
    return make_uint4(qb | (valid ? 0x80000000u : 0u), h | (b << 16), valid ? rb_attention_blocks(M, N, causal, delta, row0, row0 + TQ, TK) : 0u,
                      valid ? rb_attention_blocks(M, N, causal, delta, row0 + TQ, row0 + 2 * TQ, TK) : 0u);
}
// `round` is the CTA's step number; returns false when the CTA has no item in that step.  nb0 / nb1 are the key blocks the
// item's two tiles visit.
__device__ __forceinline__ bool item_coords(const AttnParams& p, const uint4* item_tab, uint32_t round, uint32_t& qb, uint32_t& h, uint32_t& b,
                                            uint32_t& nb0, uint32_t& nb1) {
    const uint4 e = round < ITEM_TAB ? item_tab[round] : make_item_late(round, p.q_blocks, p.heads_total, p.Hq, p.wave_heads, p.M, p.N, p.causal, p.delta);
    qb = e.x & 0x7fffffffu; h = e.y & 0xffffu; b = e.y >> 16; nb0 = e.z; nb1 = e.w;
    return (e.x >> 31) != 0;
}

// The MMA warp's two issue sequences.  (As functions that are really called, so that every call site shares one copy of the
// instructions, they measured 30 % slower on B200 than inlined: the call sequence costs the single issuing thread more than
// the shared copy saves in instruction fetches.)
__device__ __forceinline__ void issue_scores(uint32_t tmem_s, uint32_t qa, uint32_t ka, uint32_t idesc, uint64_t* done) {
#pragma unroll
    for (uint32_t kk = 0; kk < D / 16; ++kk) {
        const uint32_t off = ((kk >> 2) * SLAB_BYTES + (kk & 3) * 32) >> 4;  // 16 head-dim elements per step
        umma_bf16_ss_lo(tmem_s, qa + off, ka + off, idesc, kk != 0);
    }
    umma_commit(done);
}
// Half of O += P V: keys [64 * half, 64 * half + 64) of the block.  16 keys per step: 8 TMEM columns of packed BF16 pairs, 2048 B of V.
__device__ __forceinline__ void issue_pv_half(uint32_t tmem_o, uint32_t tmem_p, uint32_t va, uint32_t idesc, uint32_t accumulate_first) {
#pragma unroll
    for (uint32_t kk = 0; kk < TK / 32; ++kk)
        umma_bf16_ts_lo(tmem_o, tmem_p + kk * 8, va + kk * (2048 >> 4), idesc, kk != 0 ? 1u : accumulate_first);
}

// Packed FP32 pairs (fma.rn.f32x2 / add.rn.f32x2) and the three-input max halve the issue slots of the softmax.
__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi)); return r; }
__device__ __forceinline__ uint64_t pack2f(float lo, float hi) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void unpack2f(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) { uint64_t d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) { uint64_t d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ float max3(float a, float b, float c) { float d; asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }

// Waits on the three hand-offs of the per-tile chain (scores ready, P half ready, P ready).  The suspending wait measured
// 1.5-2 % faster than polling with test_wait on B200 (the pollers take issue slots from the softmax warps of the other
// tile); -DRB_ATTN_SPIN selects polling.
__device__ __forceinline__ bool wait_handoff(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_word) {
#ifdef RB_ATTN_SPIN
    return mbar_wait_spin(bar, parity, abort_word);
#else
    return mbar_wait(bar, parity, abort_word);
#endif
}

// Part of the exponentials can run on the FMA pipe instead of the 16-per-clock exp2 unit: 2^x = 2^n * p(f) with n = round(x),
// f = x - n in [-0.5, 0.5] and a cubic p (relative error 7.5e-5, far below the BF16 rounding P gets next).  RB_ATTN_POLY
// is the number of element pairs per 32-key chunk (0..16) computed this way.
#ifndef RB_ATTN_POLY
#define RB_ATTN_POLY 0
#endif
__device__ __forceinline__ void ex2_poly_pair(float x0, float x1, float& p0, float& p1) {
    x0 = fmaxf(x0, -120.f); x1 = fmaxf(x1, -120.f);
    const uint64_t x2 = pack2f(x0, x1);
    const uint64_t t2 = add2(x2, pack2f(12582912.f, 12582912.f));                 // 1.5 * 2^23: the integer part lands in the low mantissa bits
    const uint64_t n2 = add2(t2, pack2f(-12582912.f, -12582912.f));
    const uint64_t f2 = fma2(n2, pack2f(-1.f, -1.f), x2);
    uint64_t q2 = fma2(f2, pack2f(0.055171650f, 0.055171650f), pack2f(0.24261113f, 0.24261113f));
    q2 = fma2(q2, f2, pack2f(0.69326097f, 0.69326097f));
    q2 = fma2(q2, f2, pack2f(0.99992806f, 0.99992806f));
    float q0, q1, t0, t1; unpack2f(q2, q0, q1); unpack2f(t2, t0, t1);
    p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
    p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
}

// Optional cycle trace of one CTA (developer builds only, -DRB_ATTN_TRACE): slot = ((role * 64 + block) * 8 + event).
#ifdef RB_ATTN_TRACE
__device__ unsigned long long g_attn_trace[5 * 64 * 8];
#define RB_TR(on, role, j, e) do { if ((on) && (j) < 64u) g_attn_trace[(((role) * 64u + (j)) * 8u) + (e)] = clock64(); } while (0)
#else
#define RB_TR(on, role, j, e) do { } while (0)
#endif

// Row maximum of one 32-score chunk.  CLS: 2 = every key visible, 1 = keys [0, vis) of the chunk visible (per lane),
// 0 = none (nothing to do).
template <int CLS>
__device__ __forceinline__ void chunk_max(const uint32_t (&r)[32], int32_t vis, float& m) {
    if (CLS == 2) {
        float a = __uint_as_float(r[0]), b = __uint_as_float(r[1]);
#pragma unroll
        for (int i = 2; i < 32; i += 4) {
            a = max3(a, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
            if (i + 3 < 32) b = max3(b, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
        }
        m = max3(m, a, b);
    } else if (CLS == 1) {
#pragma unroll
        for (int i = 0; i < 32; ++i) if (i < vis) m = fmaxf(m, __uint_as_float(r[i]));
    }
}
// P = exp2(s * sc - m) of one chunk as BF16 pairs into `packed`; the FP32 values are added to the row sum.
template <int CLS>
__device__ __forceinline__ void chunk_exp(const uint32_t (&r)[32], int32_t vis, float sc, float neg_m, uint32_t (&packed)[16], uint64_t& acc_a, uint64_t& acc_b) {
    if (CLS == 2) {
        const uint64_t sc2 = pack2f(sc, sc), nm2 = pack2f(neg_m, neg_m);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            float x0, x1; unpack2f(fma2(pack2(r[i], r[i + 1]), sc2, nm2), x0, x1);
            float p0, p1;
            // the pairs handed to the polynomial are spread evenly over the chunk
            if (RB_ATTN_POLY > 0 && ((i >> 1) * RB_ATTN_POLY) % 16 < RB_ATTN_POLY) ex2_poly_pair(x0, x1, p0, p1);
            else { p0 = ex2(x0); p1 = ex2(x1); }
            if (i & 2) acc_b = add2(acc_b, pack2f(p0, p1)); else acc_a = add2(acc_a, pack2f(p0, p1));
            packed[i >> 1] = pack_bf16(p0, p1);
        }
    } else if (CLS == 1) {
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            float p0 = ex2(__fmaf_rn(__uint_as_float(r[i]), sc, neg_m)), p1 = ex2(__fmaf_rn(__uint_as_float(r[i + 1]), sc, neg_m));
            if (i >= vis) p0 = 0.f;
            if (i + 1 >= vis) p1 = 0.f;
            s0 += p0; s1 += p1;
            packed[i >> 1] = pack_bf16(p0, p1);
        }
        acc_a = add2(acc_a, pack2f(s0, s1));
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) packed[i] = 0u;
    }
}

// Class of the 32-key chunk c of a block for the whole warp: lane l sees keys [0, min(v0 + l, nk)) of the block.
__device__ __forceinline__ int chunk_class(int32_t v0, int32_t nk, int c) {
    const int32_t least = v0 < nk ? v0 : nk, most = v0 + 31 < nk ? v0 + 31 : nk;   // visible keys of lane 0 / lane 31
    if (least >= 32 * c + 32) return 2;
    if (most <= 32 * c) return 0;
    return 1;
}

// One key block of the online softmax for one query row (= one thread, one TMEM lane).  The 128 scores are read from
// TMEM once (four loads in flight, one wait) and stay in registers; P goes back to TMEM as BF16 pairs over the scores
// already consumed, and the MMA warp is told after the first 64 keys and again after all 128 so that P V can start
// early.  MASKED is false for blocks entirely below the causal diagonal and inside the key range.
// r = r * sc + mask * log2(e) for one 32-key chunk: the additive mask joins the scores before the row maximum is taken.
__device__ __forceinline__ void chunk_add_mask(uint32_t (&r)[32], float sc, const float* mask_row) {
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        const float4 mk = __ldg(reinterpret_cast<const float4*>(mask_row + i));
        r[i] = __float_as_uint(__fmaf_rn(__uint_as_float(r[i]), sc, mk.x * LOG2E));
        r[i + 1] = __float_as_uint(__fmaf_rn(__uint_as_float(r[i + 1]), sc, mk.y * LOG2E));
        r[i + 2] = __float_as_uint(__fmaf_rn(__uint_as_float(r[i + 2]), sc, mk.z * LOG2E));
        r[i + 3] = __float_as_uint(__fmaf_rn(__uint_as_float(r[i + 3]), sc, mk.w * LOG2E));
    }
}

template <bool MASKED, bool HAS_MASK>
__device__ __forceinline__ void softmax_block(uint32_t tmem_s, uint32_t tmem_o, float sc, int32_t visible, int32_t v0, int32_t nk, bool first,
                                              float& m_used, float& l, uint64_t* p_half, uint64_t* p_full, const float* mask_row,
                                              bool tr, uint32_t tr_role, uint32_t tr_j) {
    uint32_t r0[32], r1[32], r2[32], r3[32];
    tmem_ld_32x32(tmem_s, r0); tmem_ld_32x32(tmem_s + 32, r1); tmem_ld_32x32(tmem_s + 64, r2); tmem_ld_32x32(tmem_s + 96, r3);
    tmem_wait_ld();
    RB_TR(tr, tr_role, tr_j, 1);
    int c0 = 2, c1 = 2, c2 = 2, c3 = 2;
    if (MASKED) { c0 = chunk_class(v0, nk, 0); c1 = chunk_class(v0, nk, 1); c2 = chunk_class(v0, nk, 2); c3 = chunk_class(v0, nk, 3); }
    if (HAS_MASK) {
        // chunks that exist (the key count is a multiple of 32) take their mask values now; from here on the scores are final
        // and already in the exp2 domain, so the scale that follows is 1
        if (c0) chunk_add_mask(r0, sc, mask_row);
        if (c1) chunk_add_mask(r1, sc, mask_row + 32);
        if (c2) chunk_add_mask(r2, sc, mask_row + 64);
        if (c3) chunk_add_mask(r3, sc, mask_row + 96);
        sc = 1.0f;
    }
    float mx = -INFINITY;
#define RB_MAX(R, CLS, BASE) { if (!MASKED || CLS == 2) chunk_max<2>(R, 32, mx); else if (CLS == 1) chunk_max<1>(R, visible - BASE, mx); }
    RB_MAX(r0, c0, 0) RB_MAX(r1, c1, 32) RB_MAX(r2, c2, 64) RB_MAX(r3, c3, 96)
#undef RB_MAX
    RB_TR(tr, tr_role, tr_j, 2);
    float m_blk = mx * sc;                      // -inf when every key of the block is masked for this row
    if (!(m_blk > -INFINITY)) m_blk = -INFINITY;
    // Refresh the reference maximum only when it grew by more than 8 (a factor 256 in P).
    const bool grow = first ? true : (m_blk > m_used + 8.f);
    if (__any_sync(0xffffffffu, grow)) {
        const float m_new = first ? (m_blk > -INFINITY ? m_blk : 0.f) : (grow ? m_blk : m_used);
        if (!first) {
            const float alpha = ex2(m_used - m_new);   // 1 for lanes that keep their maximum
            l *= alpha;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t o[32];
                tmem_ld_32x32(tmem_o + c * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                tmem_st_32x32(tmem_o + c * 32, o);
            }
            tmem_wait_st();
        }
        m_used = m_new;
    }
    const float neg_m = -m_used;
    RB_TR(tr, tr_role, tr_j, 3);
    uint64_t acc_a = pack2f(0.f, 0.f), acc_b = acc_a;
#define RB_EXP(R, CLS, BASE) { uint32_t packed[16]; \
        if (!MASKED || CLS == 2) chunk_exp<2>(R, 32, sc, neg_m, packed, acc_a, acc_b); \
        else if (CLS == 1) chunk_exp<1>(R, visible - BASE, sc, neg_m, packed, acc_a, acc_b); \
        else chunk_exp<0>(R, 0, sc, neg_m, packed, acc_a, acc_b); \
        tmem_st_32x16(tmem_s + BASE / 2, packed); }
    RB_EXP(r0, c0, 0) RB_EXP(r1, c1, 32)
    tmem_wait_st();
    tc_fence_before();
    mbar_arrive(p_half);
    RB_TR(tr, tr_role, tr_j, 4);
    RB_EXP(r2, c2, 64) RB_EXP(r3, c3, 96)
#undef RB_EXP
    tmem_wait_st();
    tc_fence_before();
    mbar_arrive(p_full);
    RB_TR(tr, tr_role, tr_j, 5);
    float s0, s1; unpack2f(add2(acc_a, acc_b), s0, s1);
    l += s0 + s1;
}

template <bool HAS_MASK, bool OUT_F32>
__global__ void __launch_bounds__(THREADS, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sq = smem;                                   // [2 tiles][2 slabs][128][64]
    uint8_t* sk = smem + 2 * TILE_BYTES;                  // [stages][2 slabs][128 keys][64 d]
    uint8_t* sv = sk + KV_STAGES * TILE_BYTES;            // [stages][2 slabs][128 keys][64 dv]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sv + KV_STAGES * TILE_BYTES);
    uint64_t* q_full = bars;                    // [1]  TMA -> MMA: Q of the item has landed
    uint64_t* q_empty = bars + 1;               // [1]  MMA -> TMA: the item's last score GEMM has read Q
    uint64_t* k_full = bars + 2;                // [stages]
    uint64_t* k_empty = k_full + KV_STAGES;
    uint64_t* v_full = k_empty + KV_STAGES;
    uint64_t* v_empty = v_full + KV_STAGES;
    uint64_t* s_full = v_empty + KV_STAGES;     // [2 tiles]  MMA -> softmax: scores of a block are in TMEM
    uint64_t* p_half = s_full + 2;              // [2 tiles]  softmax -> MMA: P of the first 64 keys is in TMEM
    uint64_t* p_full = p_half + 2;              // [2 tiles]  softmax -> MMA: all of P
    uint64_t* o_full = p_full + 2;              // [2 tiles]  MMA -> softmax warps: the item's last P V has completed
    uint64_t* o_free = o_full + 2;              // [2 tiles]  softmax warps -> MMA: O has been read out of TMEM
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_free + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;
    // this CTA's work items, one entry per step (see make_item).  Filled by all threads at once
    // before the roles part, so that no role spends its own (single-thread) instruction stream on the index arithmetic.
    uint4* item_tab = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(bars) + 256);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rounds = rb_attention_steps(p.q_blocks, p.heads_total, p.wave_heads, gridDim.x);
    for (uint32_t step = threadIdx.x; step < rounds && step < ITEM_TAB; step += THREADS) item_tab[step] = make_item(p, step);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1); mbar_init(q_empty, 1);
        for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&s_full[t], 1); mbar_init(&p_half[t], 128); mbar_init(&p_full[t], 128); mbar_init(&o_full[t], 1);
            mbar_init(&o_free[t], 128);
        }
        *abort_word = 0;
        fence_barrier_init();
        prefetch_tmap(&map_q); prefetch_tmap(&map_k); prefetch_tmap(&map_v);
    }
    if (warp == W_MMA) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
#ifdef RB_ATTN_TRACE
    const bool trace_cta = blockIdx.x == 0;
#else
    const bool trace_cta = false;
#endif

    // Register budget: the two softmax warpgroups keep a whole score row in registers, the third warpgroup (TMA, MMA and
    // two idle warps) needs few.  256 * 224 + 128 * 56 = 64512 registers.
    if (warp >= W_CONTROL && warp < W_CONTROL + 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        if (warp == W_TMA && elect_one()) {
            // ---------------- TMA producer ----------------
            bool ok = true;
            uint32_t kv_it = 0, q_it = 0;
            uint32_t armed = 0, armed_parity = 0;      // bit 0: Q, bits 1-2: K stages, bits 3-4: V stages
            auto arm = [&](uint32_t bit, uint32_t parity) { armed |= 1u << bit; armed_parity = (armed_parity & ~(1u << bit)) | (parity << bit); };
            for (uint32_t round = 0; ok && round < rounds; ++round) {
                uint32_t qb, h, b, nb0, nb1;
                if (!item_coords(p, item_tab, round, qb, h, b, nb0, nb1)) continue;
                const uint32_t kvh = h / (p.Hq / p.Hkv), row0 = qb * 2 * TQ;
                const uint32_t n_max = nb0 > nb1 ? nb0 : nb1;
                if (n_max == 0) continue;
                if (q_it > 0 && !(ok = mbar_wait(q_empty, (q_it - 1) & 1, abort_word))) break;
                mbar_expect_tx(q_full, 2 * TILE_BYTES); arm(0, q_it & 1);
                for (int t = 0; t < 2; ++t)
                    for (int s = 0; s < 2; ++s)
                        tma_load_4d(sq + t * TILE_BYTES + s * SLAB_BYTES, &map_q, q_full, s * 64, (int32_t)(row0 + t * TQ), (int32_t)h, (int32_t)b);
                for (uint32_t j = 0; ok && j < n_max; ++j) {
                    const uint32_t st = (kv_it + j) % KV_STAGES, ph = ((kv_it + j) / KV_STAGES) & 1;
                    if (!(ok = mbar_wait(&k_empty[st], ph ^ 1, abort_word))) break;
                    mbar_expect_tx(&k_full[st], TILE_BYTES); arm(1 + st, ph);
                    for (int s = 0; s < 2; ++s)
                        tma_load_4d(sk + st * TILE_BYTES + s * SLAB_BYTES, &map_k, &k_full[st], s * 64, (int32_t)(j * TK), (int32_t)kvh, (int32_t)b);
                    if (!(ok = mbar_wait(&v_empty[st], ph ^ 1, abort_word))) break;
                    mbar_expect_tx(&v_full[st], TILE_BYTES); arm(3 + st, ph);
                    for (int s = 0; s < 2; ++s)
                        tma_load_4d(sv + st * TILE_BYTES + s * SLAB_BYTES, &map_v, &v_full[st], s * 64, (int32_t)(j * TK), (int32_t)kvh, (int32_t)b);
                }
                kv_it += n_max; ++q_it;
            }
            if (!ok) {
                // A wait expired: give the copies already issued a bounded time to land before the CTA retires.
                for (uint32_t bit = 0; bit < 5; ++bit) {
                    if (!(armed & (1u << bit))) continue;
                    uint64_t* bar = bit == 0 ? q_full : (bit < 3 ? &k_full[bit - 1] : &v_full[bit - 3]);
                    for (uint32_t i = 0; i < (1u << 20) && !mbar_try_wait(bar, (armed_parity >> bit) & 1u); ++i) {}
                }
            }
        } else if (warp == W_MMA && elect_one()) {
            // ---------------- MMA issuer ----------------
            // This single thread's instruction stream is the scarcest resource of the kernel (every instruction costs it about
            // 15 cycles beside two busy softmax warps on the same scheduler), so the per-tile step exists once, with the tile
            // index as a variable and the per-tile counters packed into two registers: unrolled over the two tiles it measured
            // 3 % slower, with rolled MMA loops 15 % slower.
            const uint32_t idesc_qk = make_idesc_bf16(TQ, TK, 0, 0);   // A = Q (K-major), B = K tile (K-major)
            const uint32_t idesc_pv = make_idesc_bf16(TQ, D, 0, 1);    // A = P (TMEM), B = V tile, Dv-contiguous (MN-major)
            bool ok = true;
            uint32_t kv_it = 0, q_it = 0;
            uint32_t bpar = 0;             // bit t: parity of the key blocks served for tile t (s_full / p_half / p_full)
            uint32_t usedp = 0;            // 16 bits per tile: items served so far (parity of o_full / o_free)
            const uint32_t q_lo = desc_lo_kmajor(smem_u32(sq)), k_lo = desc_lo_kmajor(smem_u32(sk)), v_lo = desc_lo_mnmajor(smem_u32(sv), SLAB_BYTES);
            auto issue_s = [&](uint32_t t, uint32_t st) {
                uint32_t qa = q_lo + t * (TILE_BYTES >> 4);
                asm volatile("" : "+r"(qa));
                uint32_t ka = k_lo + st * (TILE_BYTES >> 4);
                asm volatile("" : "+r"(ka));
                issue_scores(tmem_base + t * TK, qa, ka, idesc_qk, &s_full[t]);
            };
            for (uint32_t round = 0; ok && round < rounds; ++round) {
                uint32_t qb, h, b, nb0, nb1;
                if (!item_coords(p, item_tab, round, qb, h, b, nb0, nb1)) continue;
                const uint32_t nbp = nb0 | (nb1 << 16);
                const uint32_t n_max = nb0 > nb1 ? nb0 : nb1;
                if (n_max == 0) continue;
                uint32_t s_left = nb0 + nb1;
                if (!(ok = mbar_wait(q_full, q_it & 1, abort_word))) break;
                {
                    const uint32_t st = kv_it % KV_STAGES, ph = (kv_it / KV_STAGES) & 1;
                    if (!(ok = mbar_wait(&k_full[st], ph, abort_word))) break;
                    tc_fence_after();
#pragma unroll 1
                    for (uint32_t ti = 0; ti < 2; ++ti) { const uint32_t t = ti ^ FIRST_TILE; if (((nbp >> (16 * t)) & 0xffffu) > 0) { issue_s(t, st); --s_left; } }
                    umma_commit(&k_empty[st]);
                    if (s_left == 0) umma_commit(q_empty);
                }
                for (uint32_t j = 0; ok && j < n_max; ++j) {
                    const uint32_t st = (kv_it + j) % KV_STAGES, ph = ((kv_it + j) / KV_STAGES) & 1;
#pragma unroll 1
                    for (uint32_t ti = 0; ti < 2; ++ti) {
                        const uint32_t t = ti ^ FIRST_TILE;
                        const uint32_t nbt = (nbp >> (16 * t)) & 0xffffu, nbo = (nbp >> (16 * (t ^ 1u))) & 0xffffu;
                        if (!ok || j >= nbt) continue;
                        const uint32_t par = (bpar >> t) & 1u;
                        if (!(ok = wait_handoff(&p_half[t], par, abort_word))) continue;
                        // the first P V of an item overwrites O: the epilogue must have read the previous item's O
                        const uint32_t used_t = (usedp >> (16 * t)) & 0xffffu;
                        if (j == 0 && used_t > 0 && !(ok = mbar_wait(&o_free[t], (used_t - 1) & 1, abort_word))) continue;
                        if (!(ok = mbar_wait(&v_full[st], ph, abort_word))) continue;
                        tc_fence_after();
                        uint32_t va = v_lo + st * (TILE_BYTES >> 4);
                        asm volatile("" : "+r"(va));
                        const uint32_t tmem_o = tmem_base + 256 + t * D, tmem_p = tmem_base + t * TK;
                        issue_pv_half(tmem_o, tmem_p, va, idesc_pv, j);
                        if (!(ok = wait_handoff(&p_full[t], par, abort_word))) continue;
                        tc_fence_after();
                        issue_pv_half(tmem_o, tmem_p + 32, va + 4 * (2048 >> 4), idesc_pv, 1u);
                        bpar ^= 1u << t;
                        // the stage is released by the tile served second, or by this one when the other tile does not use the block
                        if (ti == 1 || j >= nbo) umma_commit(&v_empty[st]);
                        if (j + 1 < nbt) {
                            const uint32_t st1 = (kv_it + j + 1) % KV_STAGES, ph1 = ((kv_it + j + 1) / KV_STAGES) & 1;
                            if (!(ok = mbar_wait(&k_full[st1], ph1, abort_word))) continue;
                            tc_fence_after();
                            issue_s(t, st1); --s_left;
                            if (ti == 1 || j + 1 >= nbo) umma_commit(&k_empty[st1]);
                            if (s_left == 0) umma_commit(q_empty);
                        } else {
                            umma_commit(&o_full[t]);
                            usedp += 1u << (16 * t);
                        }
                    }
                }
                kv_it += n_max; ++q_it;
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
        // ---------------- softmax + epilogue: warps 0-3 own tile 0, warps 4-7 own tile 1 ----------------
        const uint32_t t = (warp - W_SOFTMAX) >> 2, quarter = warp & 3;
        const uint32_t row_in_tile = quarter * 32 + lane;
        const uint32_t lane_base = (quarter * 32) << 16;
        const uint32_t tmem_s = tmem_base + t * TK + lane_base;
        const uint32_t tmem_o = tmem_base + 256 + t * D + lane_base;
        uint32_t blk = 0, used = 0;
        bool ok = true;
        for (uint32_t round = 0; ok && round < rounds; ++round) {
            uint32_t qb, h, b, nb0, nb1;
            if (!item_coords(p, item_tab, round, qb, h, b, nb0, nb1)) continue;
            const uint32_t tile_row0 = qb * 2 * TQ + t * TQ;
            if (tile_row0 >= p.M) continue;
            const uint32_t nb = t ? nb1 : nb0;
            const uint32_t row = tile_row0 + row_in_tile;                  // query index inside the sequence
            const uint64_t o_at = (uint64_t)b * p.o_stride_b + (uint64_t)h * p.o_stride_h + (uint64_t)row * p.o_stride_m;
            // row of the additive mask [B*Hq, M, N]; rows past M are never dereferenced beyond the mask because their loads are
            // clamped to row M - 1
            const float* mask_row = HAS_MASK ? p.mask + ((uint64_t)(b * p.Hq + h) * p.M + (row < p.M ? row : p.M - 1)) * p.N : nullptr;
            if (nb == 0) {
                // No visible key for this tile: a softmax over an empty set has no value.  The reference's composition gives NaN
                // there (its mask is -inf everywhere in the row, mask_programs.rs:5), and so does this kernel.
                if (row < p.M) {
                    if (OUT_F32) { float* o = static_cast<float*>(p.out) + o_at; for (int i = 0; i < D / 4; ++i) reinterpret_cast<uint4*>(o)[i] = make_uint4(0x7fc00000u, 0x7fc00000u, 0x7fc00000u, 0x7fc00000u); }
                    else { bf* o = static_cast<bf*>(p.out) + o_at; for (int i = 0; i < D / 8; ++i) reinterpret_cast<uint4*>(o)[i] = make_uint4(0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u); }
                }
                continue;
            }
            const bool tr = trace_cta && round == 0 && quarter == 0 && lane == 0;
            const int64_t q_limit0 = (int64_t)(tile_row0 + quarter * 32) + p.delta;   // last visible key of this warp's first row (causal)
            float m_used = 0.f, l = 0.f;
            const bool tri = trace_cta && t == 0 && quarter == 0 && lane == 0;
            RB_TR(tri, 4, round, 4);                                 // softmax tile 0: item starts
            for (uint32_t j = 0; j < nb; ++j, ++blk) {
                ok = wait_handoff(&s_full[t], blk & 1, abort_word);
                if (!(ok = __all_sync(0xffffffffu, ok))) break;
                tc_fence_after();
                RB_TR(tr, t, j, 0);
                const uint32_t k0 = j * TK;
                const bool partial = k0 + TK > p.N;
                const bool diagonal = p.causal && (int64_t)(k0 + TK - 1) > (int64_t)tile_row0 + p.delta;  // CTA-tile-uniform
                if (partial || diagonal) {
                    // keys [0, nk) of the block exist; lane l of this warp sees keys [0, v0 + l) of them under the causal rule
                    const int64_t nk64 = (int64_t)p.N - (int64_t)k0;
                    const int32_t nk = (int32_t)(nk64 > TK ? TK : nk64);
                    int32_t v0 = TK;   // without a causal rule every lane sees the whole block
                    if (p.causal) {
                        const int64_t v64 = q_limit0 - (int64_t)k0 + 1;
                        v0 = (int32_t)(v64 > 2 * TK ? 2 * TK : (v64 < -TK ? -TK : v64));
                    }
                    int32_t visible = p.causal ? v0 + (int32_t)lane : TK;
                    visible = visible > nk ? nk : (visible < 0 ? 0 : visible);
                    softmax_block<true, HAS_MASK>(tmem_s, tmem_o, p.scale_log2, visible, v0, nk, j == 0, m_used, l, &p_half[t], &p_full[t], mask_row + k0, tr, t, j);
                } else {
                    softmax_block<false, HAS_MASK>(tmem_s, tmem_o, p.scale_log2, TK, TK, TK, j == 0, m_used, l, &p_half[t], &p_full[t], mask_row + k0, tr, t, j);
                }
            }
            if (!ok) break;
            RB_TR(tri, 4, round, 5);                                 // softmax tile 0: last P handed over
            // ---- epilogue of the item: O / l -> BF16 -> global ----
            ok = mbar_wait(&o_full[t], used & 1, abort_word);
            if (!(ok = __all_sync(0xffffffffu, ok))) break;
            RB_TR(tri, 4, round, 6);                                 // softmax tile 0: O complete
            tc_fence_after();
            // a row that saw no key at all (every key hidden by the causal rule or by -inf mask values) has no value: NaN, as the
            // reference's softmax of a row of -inf gives
            const float inv = l > 0.f ? __fdiv_rn(1.0f, l) : __uint_as_float(0x7fc00000u);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_o + c * 32, r);
                tmem_wait_ld();
                if (c == 3) { tc_fence_before(); mbar_arrive(&o_free[t]); }   // O is in registers: the next item may overwrite it
                if (row < p.M) {
                    if (OUT_F32) {
                        float* o = static_cast<float*>(p.out) + o_at + c * 32;
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4*>(o + i) = make_float4(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv,
                                                                           __uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
                    } else {
                        bf* o = static_cast<bf*>(p.out) + o_at + c * 32;
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 w;
                            w.x = pack_bf16(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
                            w.y = pack_bf16(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
                            w.z = pack_bf16(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
                            w.w = pack_bf16(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
                            *reinterpret_cast<uint4*>(o + i) = w;
                        }
                    }
                }
            }
            ++used;
            RB_TR(tri, 4, round, 7);                                 // softmax tile 0: epilogue stored
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_word) atomicExch(p.status, 2u);
    if (warp == W_MMA) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// Rotary encoding of a BF16 [B,H,S,128] tensor (any strides with a contiguous last axis) into a contiguous
// [B,H,S,128] buffer, SplitHalf or Interleaved, FP32 math with the reference's operation order
// (rotary_programs.rs:63-93); tables are FP32 [positions, 64], row = sequence index + position_offset.
__global__ void __launch_bounds__(256) rope_bf16_kernel(const bf* x, uint64_t sb, uint64_t sh, uint64_t ss, const float* cs, const float* sn,
                                                       bf* y, uint32_t H, uint32_t S, uint64_t total_rows, uint32_t position_offset, int layout) {
    // one thread per 8 pairs: 8 rows of the table, 16 input values
    const uint64_t idx = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    const uint64_t rowi = idx / 8; const uint32_t g = (uint32_t)(idx % 8);
    if (rowi >= total_rows) return;
    const uint32_t s = (uint32_t)(rowi % S); const uint64_t bh = rowi / S; const uint32_t hh = (uint32_t)(bh % H); const uint64_t bb = bh / H;
    const bf* xr = x + bb * sb + hh * sh + (uint64_t)s * ss;
    bf* yr = y + rowi * D;
    const float* c = cs + (uint64_t)(s + position_offset) * 64 + g * 8;
    const float* sv = sn + (uint64_t)(s + position_offset) * 64 + g * 8;
    // 16-byte loads and stores: eight pairs per thread (rows are 256 B apart at least and 16-byte aligned)
    float a[8], bq[8];
    const uint4 u0 = *reinterpret_cast<const uint4*>(xr + (layout == RB_ROTARY_SPLIT_HALF ? g * 8 : g * 16));
    const uint4 u1 = *reinterpret_cast<const uint4*>(xr + (layout == RB_ROTARY_SPLIT_HALF ? 64 + g * 8 : g * 16 + 8));
    const bf* h0 = reinterpret_cast<const bf*>(&u0); const bf* h1 = reinterpret_cast<const bf*>(&u1);
    if (layout == RB_ROTARY_SPLIT_HALF) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { a[i] = __bfloat162float(h0[i]); bq[i] = __bfloat162float(h1[i]); }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            a[i] = __bfloat162float(h0[2 * i]); bq[i] = __bfloat162float(h0[2 * i + 1]);
            a[4 + i] = __bfloat162float(h1[2 * i]); bq[4 + i] = __bfloat162float(h1[2 * i + 1]);
        }
    }
    float cc[8], sn8[8];
    *reinterpret_cast<float4*>(cc) = __ldg(reinterpret_cast<const float4*>(c)); *reinterpret_cast<float4*>(cc + 4) = __ldg(reinterpret_cast<const float4*>(c) + 1);
    *reinterpret_cast<float4*>(sn8) = __ldg(reinterpret_cast<const float4*>(sv)); *reinterpret_cast<float4*>(sn8 + 4) = __ldg(reinterpret_cast<const float4*>(sv) + 1);
    uint4 o0, o1;
    bf* w0 = reinterpret_cast<bf*>(&o0); bf* w1 = reinterpret_cast<bf*>(&o1);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        // first of the pair: x*cos + (pair*sin)*(-1); second: x*cos + (pair*sin)*(+1)
        const float ya = __fadd_rn(__fmul_rn(a[i], cc[i]), __fmul_rn(__fmul_rn(bq[i], sn8[i]), -1.0f));
        const float yb = __fadd_rn(__fmul_rn(bq[i], cc[i]), __fmul_rn(__fmul_rn(a[i], sn8[i]), 1.0f));
        if (layout == RB_ROTARY_SPLIT_HALF) { w0[i] = __float2bfloat16_rn(ya); w1[i] = __float2bfloat16_rn(yb); }
        else if (i < 4) { w0[2 * i] = __float2bfloat16_rn(ya); w0[2 * i + 1] = __float2bfloat16_rn(yb); }
        else { w1[2 * (i - 4)] = __float2bfloat16_rn(ya); w1[2 * (i - 4) + 1] = __float2bfloat16_rn(yb); }
    }
    *reinterpret_cast<uint4*>(yr + (layout == RB_ROTARY_SPLIT_HALF ? g * 8 : g * 16)) = o0;
    *reinterpret_cast<uint4*>(yr + (layout == RB_ROTARY_SPLIT_HALF ? 64 + g * 8 : g * 16 + 8)) = o1;
}

// General attention for shapes the tensor-core kernel does not take (head dims other than 128, FP32 storage,
// additive masks).  One CTA per query row; it follows the reference's materialised algorithm literally:
// scores in FP32 from BF16-rounded operands, + mask, row softmax by division, P rounded to BF16, P V in FP32.
template <typename T>
__global__ void __launch_bounds__(128) attention_rows_kernel(const T* q, const T* k, const T* v, const float* mask, T* out,
                                                            uint32_t Hq, uint32_t Hkv, uint32_t M, uint32_t N, uint32_t Dq, uint32_t Dv,
                                                            float scale, int causal, int64_t delta,
                                                            uint64_t o_stride_b, uint64_t o_stride_h, uint64_t o_stride_m) {
    extern __shared__ float sc[];   // [N] scores, then probabilities
    __shared__ float red[4];
    __shared__ float qs[256];
    const uint64_t r = blockIdx.x;  // flat (b, h, i)
    const uint32_t i = (uint32_t)(r % M); const uint64_t bh = r / M; const uint32_t h = (uint32_t)(bh % Hq); const uint64_t b = bh / Hq;
    const uint32_t kvh = h / (Hq / Hkv);
    auto ldf = [](const T* ptr, uint64_t idx) -> float {
        if constexpr (sizeof(T) == 4) return __bfloat162float(__float2bfloat16_rn(ptr[idx]));  // BF16-rounded operand
        else return __bfloat162float(ptr[idx]);
    };
    const T* qr = q + r * Dq; const T* kb = k + (b * Hkv + kvh) * (uint64_t)N * Dq; const T* vb = v + (b * Hkv + kvh) * (uint64_t)N * Dv;
    for (uint32_t c = threadIdx.x; c < Dq; c += 128) qs[c] = ldf(qr, c);
    __syncthreads();
    float mx = -INFINITY;
    for (uint32_t j = threadIdx.x; j < N; j += 128) {
        float acc = 0.f;
        for (uint32_t c = 0; c < Dq; ++c) acc = __fmaf_rn(qs[c], ldf(kb, (uint64_t)j * Dq + c), acc);
        float s = __fmul_rn(acc, scale);
        if (mask) s = __fadd_rn(s, mask[r * N + j]);
        if (causal && (int64_t)j > (int64_t)i + delta) s = -INFINITY;
        sc[j] = s; mx = fmaxf(mx, s);
    }
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    __syncthreads();
    float sum = 0.f;
    for (uint32_t j = threadIdx.x; j < N; j += 128) { float e = expf(__fsub_rn(sc[j], mx)); sc[j] = e; sum += e; }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    sum = (red[0] + red[1]) + (red[2] + red[3]);
    for (uint32_t j = threadIdx.x; j < N; j += 128) sc[j] = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(sc[j], sum)));
    __syncthreads();
    T* o = out + b * o_stride_b + (uint64_t)h * o_stride_h + (uint64_t)i * o_stride_m;
    for (uint32_t c = threadIdx.x; c < Dv; c += 128) {
        float acc = 0.f;
        for (uint32_t j = 0; j < N; ++j) acc = __fmaf_rn(sc[j], ldf(vb, (uint64_t)j * Dv + c), acc);
        if constexpr (sizeof(T) == 4) o[c] = acc; else o[c] = __float2bfloat16_rn(acc);
    }
}

// Per-context bookkeeping of this translation unit: which kernels have had their shared-memory limit raised, and how many
// calls took each path (read by rb_attention_launch_counts).
struct AttnState {
    bool configured[4] = {false, false, false, false};
    bool rows_f32 = false, rows_bf16 = false;
    uint64_t tensor_core_launches = 0, general_launches = 0;
};

bool make_qkv_map(CUtensorMap* map, const void* base, const rb_tensor* t) {
    // logical [B, H, S, 128] with element strides; TMA dims innermost first: {d, s, h, b}
    uint64_t dims[4] = {t->shape[3], t->shape[2], t->shape[1], t->shape[0]};
    uint64_t strides[3] = {t->strides[2] * 2, t->strides[1] * 2, t->strides[0] * 2};
    uint32_t box[4] = {64, 128, 1, 1};
    return encode_bf16_map(map, base, 4, dims, strides, box, true);
}

// Address and validity of a rank-4 tensor whose last axis is contiguous and whose other strides are multiples
// of 8 elements (16 bytes for BF16); the byte range reached through the strides must lie inside the storage.
int32_t resolve_strided4(rb_ctx* ctx, const rb_tensor* t, const char* what, void** out) {
    *out = nullptr;
    if (!t) return rb::fail(RB_INVALID_TENSOR, "%s: missing tensor", what);
    if (t->rank != 4) return rb::fail(RB_INVALID_TENSOR, "%s: attention tensors are rank 4 [B,H,S,D]", what);
    size_t es = rb::dtype_size(t->dtype);
    if (!es) return rb::fail(RB_INVALID_TENSOR, "%s: unsupported dtype", what);
    if (t->shape[3] > 1 && t->strides[3] != 1) return rb::fail(RB_INVALID_TENSOR, "%s: the last axis must be contiguous", what);
    uint64_t span = 1;
    for (int i = 0; i < 4; ++i) {
        if (t->shape[i] == 0) { span = 0; break; }
        span += (t->shape[i] - 1) * t->strides[i];
    }
    void* base; uint64_t bytes;
    if (rb_resource(ctx, t->handle, &base, &bytes) != RB_OK) return RB_NULL_HANDLE;
    if (t->offset > bytes || span * es > bytes - t->offset) return rb::fail(RB_INVALID_TENSOR, "%s: strides reach outside the storage", what);
    char* ptr = (char*)base + t->offset;
    if (((uintptr_t)ptr & 15u) != 0) return rb::fail(RB_INVALID_TENSOR, "%s: device address must be 16-byte aligned", what);
    *out = ptr;
    return RB_OK;
}

bool is_contiguous4(const rb_tensor* t) { return rb::contiguous(t); }

}  // namespace

using namespace rb;

extern "C" {

int32_t rb_attention(rb_ctx* ctx, const rb_tensor* q, const rb_tensor* k, const rb_tensor* v, const rb_tensor* additive_mask,
                     float scale, int32_t causal, uint64_t query_start, uint64_t key_start,
                     const rb_tensor* cos, const rb_tensor* sin, int32_t rotary_layout, int32_t out_layout, const rb_tensor* out) {
    RB_TRY(check_ctx(ctx));
    void *pq, *pk, *pv, *po, *pm = nullptr, *pc = nullptr, *ps = nullptr;
    RB_TRY(resolve_strided4(ctx, q, "attention Q", &pq)); RB_TRY(resolve_strided4(ctx, k, "attention K", &pk));
    RB_TRY(resolve_strided4(ctx, v, "attention V", &pv)); RB_TRY(resolve(ctx, out, "attention output", &po));
    const uint64_t B = q->shape[0], Hq = q->shape[1], M = q->shape[2], Dq = q->shape[3];
    const uint64_t Hkv = k->shape[1], N = k->shape[2], Dv = v->shape[3];
    // Domain of src/nn/attention.rs:81-104.
    if (Hq == 0 || Hkv == 0 || Hq % Hkv != 0 || k->shape[0] != B || v->shape[0] != B || v->shape[1] != Hkv || k->shape[3] != Dq || v->shape[2] != N)
        return fail(RB_INVALID_TENSOR, "GQA requires matching batches, positive divisible Q/KV heads and matching K/V lengths and Q/K widths");
    const uint64_t flat = B * Hq;
    if (flat == 0 || flat > 4096 || M == 0 || Dq == 0 || Dv == 0 || M % 16 || Dq % 16 || Dv % 16 || N == 0 || N % 32 || N > 0x7fffffffull ||
        M > 0x7fffffffull || !(scale - scale == 0.0f) || flat * M * N > 0xffffffffull)
        return fail(RB_INVALID_TENSOR, "attention requires matching batches/contractions, aligned positive matrix dimensions, positive N divisible by 32 "
                                       "within INT32_MAX, a finite FP32 scale and scores within u32");
    if (q->dtype != k->dtype || q->dtype != v->dtype || q->dtype != out->dtype || (q->dtype != RB_BF16 && q->dtype != RB_F32))
        return fail(RB_INVALID_TENSOR, "attention requires Q/K/V and the output in one dtype, BF16 or FP32");
    if (causal && (query_start + (M - 1) < query_start || key_start + (N - 1) < key_start)) return fail(RB_INVALID_TENSOR, "causal absolute position overflow");
    if (out->rank != 4) return fail(RB_INVALID_TENSOR, "attention output is rank 4");
    const bool bmhd = out_layout == RB_LAYOUT_BMHD;
    const uint64_t want[4] = {B, bmhd ? M : Hq, bmhd ? Hq : M, Dv};
    for (int i = 0; i < 4; ++i) if (out->shape[i] != want[i]) return fail(RB_INVALID_TENSOR, "attention output shape does not match the requested layout");
    const uint64_t o_stride_b = Hq * M * Dv, o_stride_h = bmhd ? Dv : M * Dv, o_stride_m = bmhd ? Hq * Dv : Dv;
    if (additive_mask) {
        RB_TRY(resolve(ctx, additive_mask, "attention mask", &pm));
        if (additive_mask->dtype != RB_F32 || elements(additive_mask) != flat * M * N) return fail(RB_INVALID_TENSOR, "attention additive mask must be FP32 [B,Hq,M,N]");
    }
    const bool rope = cos != nullptr || sin != nullptr;
    int64_t delta;
    {
        const uint64_t cap = 1ull << 40;
        if (query_start >= key_start) delta = (int64_t)(query_start - key_start < cap ? query_start - key_start : cap);
        else delta = -(int64_t)(key_start - query_start < cap ? key_start - query_start : cap);
    }
    if (rope) {
        if (!cos || !sin) return fail(RB_INVALID_TENSOR, "fused rotary needs both tables");
        RB_TRY(resolve(ctx, cos, "attention cos table", &pc)); RB_TRY(resolve(ctx, sin, "attention sin table", &ps));
        const int64_t q_off = delta;
        if (cos->dtype != RB_F32 || sin->dtype != RB_F32 || !same_shape(cos, sin) || cos->shape[cos->rank - 1] != 64 || Dq != 128 ||
            q_off < 0 || elements(cos) / 64 < N || elements(cos) / 64 < M + (uint64_t)q_off)
            return fail(RB_INVALID_TENSOR, "fused rotary needs head dim 128 and FP32 tables [positions >= max(N, M + query_start - key_start), 64]");
        if (rotary_layout != RB_ROTARY_SPLIT_HALF && rotary_layout != RB_ROTARY_INTERLEAVED) return fail(RB_INVALID_TENSOR, "unknown rotary layout");
    }

    AttnState* state = static_cast<AttnState*>(ctx->attention_state);
    if (!state) { state = new AttnState(); ctx->attention_state = state; }
    const bool f32 = q->dtype == RB_F32;
    // The tensor-core kernel takes head dim 128 and a positive scale (it takes row maxima before scaling); FP32 tensors, the
    // reference's own contract (src/nn/attention.rs:10-80), are rounded to BF16 on the way in, which is where the reference
    // rounds them too, and leave as FP32.
    const bool fast = Dq == 128 && Dv == 128 && scale > 0.0f && (!f32 || (is_contiguous4(q) && is_contiguous4(k) && is_contiguous4(v)));
    if (!fast) {
        if (rope) return fail(RB_INVALID_TENSOR, "fused rotary is only available on the head-dim-128 path");
        if (!is_contiguous4(q) || !is_contiguous4(k) || !is_contiguous4(v)) return fail(RB_INVALID_TENSOR, "general attention path requires contiguous [B,H,S,D] tensors");
        if (Dq > 256) return fail(RB_INVALID_TENSOR, "general attention path supports head dims up to 256");
        const size_t smem = N * sizeof(float);
        if (smem > 200 * 1024) return fail(RB_INVALID_TENSOR, "general attention path supports up to 51200 keys; use head dim 128 for longer sequences");
        const uint64_t rows = flat * M;
        if (f32) {
            if (!state->rows_f32) { cudaFuncSetAttribute(attention_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); state->rows_f32 = true; }
            attention_rows_kernel<float><<<(unsigned)rows, 128, smem, ctx->stream>>>((const float*)pq, (const float*)pk, (const float*)pv, (const float*)pm, (float*)po,
                (uint32_t)Hq, (uint32_t)Hkv, (uint32_t)M, (uint32_t)N, (uint32_t)Dq, (uint32_t)Dv, scale, causal, delta, o_stride_b, o_stride_h, o_stride_m);
        } else {
            if (!state->rows_bf16) { cudaFuncSetAttribute(attention_rows_kernel<bf>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); state->rows_bf16 = true; }
            attention_rows_kernel<bf><<<(unsigned)rows, 128, smem, ctx->stream>>>((const bf*)pq, (const bf*)pk, (const bf*)pv, (const float*)pm, (bf*)po,
                (uint32_t)Hq, (uint32_t)Hkv, (uint32_t)M, (uint32_t)N, (uint32_t)Dq, (uint32_t)Dv, scale, causal, delta, o_stride_b, o_stride_h, o_stride_m);
        }
        state->general_launches++;
        return after_launch(ctx, "attention (general path)");
    }

    // ---- tensor-core path ----
    Scratch scratch(ctx);
    rb_tensor qt = *q, kt = *k, vt = *v;
    if (f32) {
        // FP32 Q/K/V -> BF16 copies (Cast, as the reference's composition does before its two GEMMs)
        rb_tensor q16, k16, v16; void *c16q, *c16k, *c16v;
        RB_TRY(scratch.tensor(RB_BF16, {B, Hq, M, 128}, &q16, &c16q)); RB_TRY(scratch.tensor(RB_BF16, {B, Hkv, N, 128}, &k16, &c16k));
        RB_TRY(scratch.tensor(RB_BF16, {B, Hkv, N, 128}, &v16, &c16v));
        RB_TRY(rb_cast(ctx, q, &q16)); RB_TRY(rb_cast(ctx, k, &k16)); RB_TRY(rb_cast(ctx, v, &v16));
        qt = q16; kt = k16; vt = v16; pq = c16q; pk = c16k; pv = c16v;
    }
    if (rope) {
        // K is rotated once per KV head and Q once per query head into temporaries; doing it inside the attention CTAs
        // would repeat the K rotation for every query head of the group and every query block.
        rb_tensor rq, rk; void *wq, *wk;
        RB_TRY(scratch.tensor(RB_BF16, {B, Hq, M, 128}, &rq, &wq)); RB_TRY(scratch.tensor(RB_BF16, {B, Hkv, N, 128}, &rk, &wk));
        const uint32_t q_off = (uint32_t)delta;
        rope_bf16_kernel<<<(unsigned)((flat * M * 8 + 255) / 256), 256, 0, ctx->stream>>>((const bf*)pq, qt.strides[0], qt.strides[1], qt.strides[2], (const float*)pc,
            (const float*)ps, (bf*)wq, (uint32_t)Hq, (uint32_t)M, flat * M, q_off, rotary_layout);
        RB_TRY(after_launch(ctx, "attention rotary(Q)"));
        rope_bf16_kernel<<<(unsigned)((B * Hkv * N * 8 + 255) / 256), 256, 0, ctx->stream>>>((const bf*)pk, kt.strides[0], kt.strides[1], kt.strides[2], (const float*)pc,
            (const float*)ps, (bf*)wk, (uint32_t)Hkv, (uint32_t)N, B * Hkv * N, 0, rotary_layout);
        RB_TRY(after_launch(ctx, "attention rotary(K)"));
        pq = wq; pk = wk; qt = rq; kt = rk;
    }
    const rb_tensor* operands[3] = {&qt, &kt, &vt};
    for (const rb_tensor* t : operands)
        for (int i = 0; i < 3; ++i)
            if (t->strides[i] % 8 != 0) return fail(RB_INVALID_TENSOR, "attention strides must be multiples of 8 elements");
    AttnParams p{};
    p.B = (uint32_t)B; p.Hq = (uint32_t)Hq; p.Hkv = (uint32_t)Hkv; p.M = (uint32_t)M; p.N = (uint32_t)N;
    p.scale_log2 = scale * LOG2E; p.causal = causal ? 1 : 0; p.delta = causal ? delta : 0;
    p.q_blocks = (uint32_t)((M + 2 * TQ - 1) / (2 * TQ)); p.heads_total = (uint32_t)flat; p.items = p.q_blocks * p.heads_total;
    const uint32_t sms = ctx->sm_limit > 0 ? (uint32_t)ctx->sm_limit : (uint32_t)ctx->sm_count;
    const uint32_t grid = p.items < sms ? p.items : sms;
    p.wave_heads = rb_attention_wave_heads(p.q_blocks, p.heads_total, grid);
    p.out = po; p.o_stride_b = o_stride_b; p.o_stride_h = o_stride_h; p.o_stride_m = o_stride_m;
    p.mask = static_cast<const float*>(pm);
    RB_TRY(kernel_status_word(ctx, &p.status));
    CUtensorMap mq, mk, mv;
    if (!make_qkv_map(&mq, pq, &qt) || !make_qkv_map(&mk, pk, &kt) || !make_qkv_map(&mv, pv, &vt))
        return fail(RB_STATUS, "cuTensorMapEncodeTiled failed for an attention operand");
    const int variant = (pm ? 2 : 0) | (f32 ? 1 : 0);
    auto launch = [&](auto kernel) -> int32_t {
        if (!state->configured[variant]) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
            if (e != cudaSuccess) return fail(RB_STATUS, "cudaFuncSetAttribute(attention) failed with CUDA status %d (%s)", (int)e, cudaGetErrorString(e));
            state->configured[variant] = true;
        }
        kernel<<<grid, THREADS, SMEM_BYTES, ctx->stream>>>(mq, mk, mv, p);
        return RB_OK;
    };
    switch (variant) {
        case 0: RB_TRY(launch(attention_fwd_kernel<false, false>)); break;
        case 1: RB_TRY(launch(attention_fwd_kernel<false, true>)); break;
        case 2: RB_TRY(launch(attention_fwd_kernel<true, false>)); break;
        default: RB_TRY(launch(attention_fwd_kernel<true, true>)); break;
    }
    state->tensor_core_launches++;
    return after_launch(ctx, "attention");
}

int32_t rb_attention_launch_counts(rb_ctx* ctx, uint64_t* tensor_core, uint64_t* general) {
    RB_TRY(check_ctx(ctx));
    const AttnState* state = static_cast<const AttnState*>(ctx->attention_state);
    if (tensor_core) *tensor_core = state ? state->tensor_core_launches : 0;
    if (general) *general = state ? state->general_launches : 0;
    return RB_OK;
}

#ifdef RB_ATTN_TRACE
// Developer builds only: copies the cycle trace of the last attention launch to the host.
__attribute__((visibility("default"))) int32_t rb_debug_attention_trace(unsigned long long* out, uint64_t words) {
    if (words > 5 * 64 * 8) words = 5 * 64 * 8;
    return cudaMemcpyFromSymbol(out, g_attn_trace, words * 8) == cudaSuccess ? 0 : 3;
}
#endif

}  // extern "C"
