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

// Work items of the persistent attention kernel: one item = one block of query rows of one (batch, head).  Items are numbered
// so that the query blocks with the most visible keys (the last ones under a causal mask) come first and the heads of one
// batch entry, and therefore of one KV group, are neighbours; CTA c of a grid of G takes items c, c + G, c + 2G, ...
RB_HD void rb_attention_item(uint32_t item, uint32_t q_blocks, uint32_t heads_total, uint32_t heads, uint32_t& qb, uint32_t& h, uint32_t& b) {
    qb = q_blocks - 1 - item / heads_total;
    const uint32_t r = item % heads_total;
    h = r % heads; b = r / heads;
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
