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
