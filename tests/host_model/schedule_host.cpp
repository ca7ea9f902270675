// Host build of the kernels' shared index arithmetic (rust_ascend_b200/csrc/schedule.h) for CPU tests.
#include "schedule.h"
extern "C" {
void host_tile_coords(uint32_t t, uint32_t tiles_m, uint32_t tiles_n, uint32_t group_m, uint32_t* out3) {
    rb_tile_coords(t, tiles_m, tiles_n, group_m, out3[0], out3[1], out3[2]);
}
void host_scatter_tile(uint32_t t, uint32_t tiles_m, uint32_t tiles_n, uint32_t group_m, uint32_t shift, uint32_t* out2) {
    rb_scatter_tile(t, tiles_m, tiles_n, group_m, shift, out2[0], out2[1]);
}
uint32_t host_scatter_shift(uint32_t rank, uint32_t world, uint32_t rows_per_owner, uint32_t tile_rows) {
    return rb_scatter_shift(rank, world, rows_per_owner, tile_rows);
}
void host_scatter_owner(uint32_t row, uint32_t rows_per_owner, uint32_t* out2) { rb_scatter_owner(row, rows_per_owner, out2[0], out2[1]); }
void host_scatter_word(uint32_t it, uint32_t lane, uint32_t* out2) { rb_scatter_word(it, lane, out2[0], out2[1]); }
void host_gemm_plan(uint32_t tiles, uint32_t ctas, int allow_halves, uint32_t* out2) { rb_gemm_plan(tiles, ctas, allow_halves != 0, out2[0], out2[1]); }
void host_gemm_item(uint32_t item, uint32_t split, uint32_t* out2) { rb_gemm_item(item, split, out2[0], out2[1]); }
uint32_t host_attention_wave_heads(uint32_t q_blocks, uint32_t heads_total, uint32_t ctas) { return rb_attention_wave_heads(q_blocks, heads_total, ctas); }
uint32_t host_attention_steps(uint32_t q_blocks, uint32_t heads_total, uint32_t wave_heads, uint32_t ctas) { return rb_attention_steps(q_blocks, heads_total, wave_heads, ctas); }
int host_attention_item(uint32_t step, uint32_t cta, uint32_t ctas, uint32_t q_blocks, uint32_t heads_total, uint32_t heads, uint32_t wave_heads, uint32_t* out3) {
    return rb_attention_item(step, cta, ctas, q_blocks, heads_total, heads, wave_heads, out3[0], out3[1], out3[2]) ? 1 : 0;
}
uint32_t host_group_of(const int32_t* ends, uint32_t groups, uint32_t row) { return rb_group_of(ends, groups, row); }
uint32_t host_attention_blocks(uint32_t M, uint32_t N, int causal, int64_t delta, uint32_t row0, uint32_t row_end, uint32_t block) {
    return rb_attention_blocks(M, N, causal, delta, row0, row_end, block);
}
}
