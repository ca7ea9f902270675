// Index arithmetic shared by the kernels and by host-side tests: the GEMM tile raster and the number of key blocks an
// attention tile visits.  Plain C++ (no CUDA headers) so that the same code compiles for the device and for a host test.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define RB_HD __host__ __device__ __forceinline__
#else
#define RB_HD inline
#endif

// Grouped raster of output tiles, the role scheduler.rs:45-79 plays in the reference: tiles are numbered so that
// `group_m` consecutive tile rows are walked column by column, which keeps the A rows and B columns of the tiles in
// flight inside L2.  Every t in [0, batches*tiles_m*tiles_n) maps to exactly one (batch, tm, tn).
RB_HD void rb_tile_coords(uint32_t t, uint32_t tiles_m, uint32_t tiles_n, uint32_t group_m, uint32_t& batch, uint32_t& tm, uint32_t& tn) {
    const uint32_t per_batch = tiles_m * tiles_n;
    batch = t / per_batch; t -= batch * per_batch;
    const uint32_t group_size = group_m * tiles_n;
    const uint32_t group = t / group_size, first_m = group * group_m;
    const uint32_t rows = tiles_m - first_m < group_m ? tiles_m - first_m : group_m;
    const uint32_t r = t - group * group_size;
    tm = first_m + r % rows; tn = r / rows;
}

// Tail wave of the persistent GEMM.  `tiles` whole tiles are walked by `ctas` persistent CTAs in rounds; when the last
// round would hold r tiles with 0 < 2r <= ctas, those r tiles become 2r half-width work items so that the last round takes
// about half a tile's time.  Items [0, split) are whole tiles (item == tile), item split + i is half (i & 1) of tile
// split + i / 2.  `allow_halves` is false where half a tile would not be a whole number of 32-column epilogue chunks.
RB_HD void rb_gemm_plan(uint32_t tiles, uint32_t ctas, bool allow_halves, uint32_t& split, uint32_t& items) {
    split = tiles; items = tiles;
    if (!allow_halves || ctas == 0 || tiles == 0) return;
    const uint32_t r = tiles % ctas;
    if (r == 0 || 2 * r > ctas) return;
    split = tiles - r; items = split + 2 * r;
}
// `half` = 2 for a whole tile, else which half (0: left columns, 1: right columns).
RB_HD void rb_gemm_item(uint32_t item, uint32_t split, uint32_t& tile, uint32_t& half) {
    if (item < split) { tile = item; half = 2; return; }
    const uint32_t i = item - split;
    tile = split + (i >> 1); half = i & 1u;
}

// M-grouped GEMM (GroupEnds, deepgemm/plan.rs:15-29): `ends` are nondecreasing row prefix sums, group g owns rows
// [ends[g-1], ends[g]).  Returns the group that owns `row` (the first g with row < ends[g]); empty groups own nothing.
RB_HD uint32_t rb_group_of(const int32_t* ends, uint32_t groups, uint32_t row) {
    uint32_t lo = 0, hi = groups;            // invariant: the answer is in [lo, hi)
    while (lo + 1 < hi) {
        const uint32_t mid = (lo + hi) / 2;
        if ((uint32_t)ends[mid - 1] <= row) lo = mid; else hi = mid;
    }
    return lo;
}

// Key blocks of `block` keys that query rows [row0, row_end) of an M-row, N-key problem must visit.  Under the causal
// rule of mask_programs.rs:30-37 key k is hidden from query q iff k > q + delta (delta = query_start - key_start), so
// the last visible key of the tile is (min(row_end, M) - 1) + delta.
RB_HD uint32_t rb_attention_blocks(uint32_t M, uint32_t N, int causal, int64_t delta, uint32_t row0, uint32_t row_end, uint32_t block) {
    if (row0 >= M) return 0;
    const uint32_t all = (N + block - 1) / block;
    if (!causal) return all;
    const int64_t last_q = (int64_t)(row_end < M ? row_end : M) - 1 + delta;
    if (last_q < 0) return 0;
    const int64_t need = last_q / block + 1;
    return need < (int64_t)all ? (uint32_t)need : all;
}

// Work items of the persistent attention kernel: one item = one block of query rows of one (batch, head).  The order serves
// two ends.  Cache reuse: the heads are taken in waves of a few neighbouring heads (about two rounds of work for the grid), so
// the K and V tiles of a head are read from DRAM once and then found in L2 by the other query blocks of that head and by the
// other query heads of its KV group.  Load balance: inside a wave the items are sorted by cost (under a causal mask the last
// query blocks see the most keys, so they come first) and the CTAs walk the wave's list in a zigzag: place r * G + c in even
// rounds r, r * G + (G - 1 - c) in odd rounds, so a CTA that drew an expensive item in one round draws a cheap one in the next.
// Heads per wave: at most two rounds of work, and the same number in every wave (a short last wave would leave the CTAs that drew
// its expensive items without cheap ones to pair them with).
RB_HD uint32_t rb_attention_wave_heads(uint32_t q_blocks, uint32_t heads_total, uint32_t ctas) {
    uint32_t most = (2 * ctas) / (q_blocks ? q_blocks : 1);
    if (most == 0) most = 1;
    if (heads_total == 0) return 1;
    const uint32_t waves = (heads_total + most - 1) / most;
    return (heads_total + waves - 1) / waves;
}
// Steps every CTA of the grid walks: waves x rounds per (full) wave.
RB_HD uint32_t rb_attention_steps(uint32_t q_blocks, uint32_t heads_total, uint32_t wave_heads, uint32_t ctas) {
    const uint32_t waves = (heads_total + wave_heads - 1) / wave_heads;
    const uint32_t in_wave = wave_heads < heads_total ? wave_heads : heads_total;
    return waves * ((in_wave * q_blocks + ctas - 1) / ctas);
}
// Item of CTA `cta` in step `step`; false when the CTA has nothing to do in that step (the end of a wave's list).
RB_HD bool rb_attention_item(uint32_t step, uint32_t cta, uint32_t ctas, uint32_t q_blocks, uint32_t heads_total, uint32_t heads, uint32_t wave_heads,
                             uint32_t& qb, uint32_t& h, uint32_t& b) {
    const uint32_t in_full = wave_heads < heads_total ? wave_heads : heads_total;
    const uint32_t rounds = (in_full * q_blocks + ctas - 1) / ctas;
    const uint32_t wave = step / rounds, r = step - wave * rounds;
    const uint32_t first = wave * wave_heads;
    if (first >= heads_total) return false;
    const uint32_t in_wave = heads_total - first < wave_heads ? heads_total - first : wave_heads;   // the last wave may be short
    const uint32_t place = r * ctas + ((r & 1u) ? ctas - 1 - cta : cta);
    if (place >= in_wave * q_blocks) return false;
    qb = q_blocks - 1 - place / in_wave;
    const uint32_t head = first + place % in_wave;
    h = head % heads; b = head / heads;
    return true;
}

// Scatter GEMM (row-parallel projection whose output rows belong to `world` owners of rows_per_owner rows each).
// Tile t of a rank is the raster tile shifted by `tile_shift` tile rows, so that rank r starts in the rows of owner r + 1 and
// the ranks write to different owners at any moment instead of all to the same one.
RB_HD void rb_scatter_tile(uint32_t t, uint32_t tiles_m, uint32_t tiles_n, uint32_t group_m, uint32_t tile_shift, uint32_t& tm, uint32_t& tn) {
    uint32_t batch;
    rb_tile_coords(t, tiles_m, tiles_n, group_m, batch, tm, tn);
    tm += tile_shift;
    if (tm >= tiles_m) tm -= tiles_m;
}
RB_HD uint32_t rb_scatter_shift(uint32_t rank, uint32_t world, uint32_t rows_per_owner, uint32_t tile_rows) {
    return ((rank + 1) % world) * (rows_per_owner / tile_rows);
}
// Owner of output row `row` and the row's index inside the owner's block.
RB_HD void rb_scatter_owner(uint32_t row, uint32_t rows_per_owner, uint32_t& owner, uint32_t& local_row) {
    owner = row / rows_per_owner;
    local_row = row - owner * rows_per_owner;
}
// A warp's copy-out of a 32-row x 64-column BF16 slice (256 words of 16 bytes): in step `it` lane `lane` moves word `j` of
// row `r`, so that eight neighbouring lanes cover one 128-byte row segment.
RB_HD void rb_scatter_word(uint32_t it, uint32_t lane, uint32_t& r, uint32_t& j) {
    const uint32_t idx = it * 32 + lane;
    r = idx >> 3; j = idx & 7;
}
