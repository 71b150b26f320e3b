// One LoRA projection ("problem") of a step, as the batched kernels see it.
// A step plan is an array of these in device memory, built on the host once
// per set of buffers and reused every step.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vlr {

// Tensor maps of one (activation, weight) pair.  All boxes are 64 columns (128
// bytes, the swizzle span) wide; several box heights exist so that a tile is
// fetched with few, large copies: activations 32 / 64 / 128 rows, weights
// 16 / 32 / 64 / 128 rows.
struct alignas(128) MapSet {
  CUtensorMap act[3];   // boxes of 32 / 64 / 128 activation rows x 64 columns
  CUtensorMap w[4];     // boxes of 16 / 32 / 64 / 128 pool cells x 64 columns
  CUtensorMap row;      // one activation row x 64 columns (gathered rows)
  CUtensorMap row3[3];  // one activation row x 2 / 4 / 8 consecutive 64-column blocks, as a 3-D view
                        // [rows][cols / 64][64] of the activations (cols a multiple of 64, else unset):
                        // the blocks land as consecutive 128-byte lines
  CUtensorMap w3[3][4]; // [i][b]: 16 << b pool cells x (2 << i) consecutive 64-column blocks of the same 3-D view
                        // of the pool (set where cells x blocks <= 256, in step plans' shrink side only):
                        // a cell's blocks land as consecutive lines, cell after cell
  CUtensorMap wb3[4][3];// [b][i]: 16 << b pool cells x (2 << i) 64-column blocks (8 blocks: 16 / 32 cells only) with the block as the OUTER
                        // dimension (view [cols / 64][cells][64]): the blocks land one after the other, each
                        // [cells][64] - what one box per block gives, requested as one copy (step plans'
                        // expand side only)
  CUtensorMap act3;     // 128 activation rows x two 64-column blocks, block-major like wb3 (same side)
};

struct alignas(128) StepProblem {
  MapSet shrink;        // act = x [max_rows, h_in],  w = A-side pool [cells_a, h_in]
  MapSet expand;        // act = y [max_rows, h_out], w = B-side pool [cells_b, h_out]
  const void* x;
  void* y;
  const void* wa;       // A-side pool: cell = one rank row of length h_in
  const void* wb;       // B-side pool: cell = one row of B, length h_out
  const int64_t* a_start_a;
  const int64_t* a_loc_a;
  const int64_t* a_start_b;
  const int64_t* a_loc_b;
  int32_t h_in;
  int32_t h_out;
  int32_t slot_a;
  int32_t slot_b;
  int32_t layout_b;
  int32_t pad_[3];
};

// ---- groups of rows for the gather mat-vec kernels
struct BgmvGroups {
  // gather mode (tiles != nullptr)
  const int32_t* tiles;
  const int32_t* gather_rows;
  const int32_t* counts;      // device counts written by the packer
  // token mode
  const int64_t* indicies;
  int64_t batch;
  // adapter tables (single-problem calls; a step plan carries its own per problem)
  const int64_t* a_start;
  const int64_t* a_len;       // 4 * rank
  const int64_t* a_loc;
  int64_t qkvo;
  // step mode: problem blockIdx.z of the plan; the shrink result of problem p
  // lives at vbuf + p * vstride elements, row pitch kMaxRank
  const StepProblem* plan;
  void* vbuf;
  int64_t vstride;
};

// ---- where a CTA's tile comes from
struct TileSource {
  // mode 0: the reference's problem table (int64, device)
  const int64_t* output_counts;
  const int64_t* rank_counts;
  const int64_t* lora_ids;
  const int64_t* start_ids;
  int64_t num_problems;
  // mode 1: packed schedule (int32 tile records + device counts)
  const int32_t* tiles;
  const int32_t* counts;
  const int32_t* gather_rows;
  int gather_mma;                    // 1: gather tiles are work items of the tensor-core kernels too
  int wide_below_rank;               // expand: gather tiles of adapters below this rank use wide stages.  The
                                     // caller presets 0 (none), 1 (the tile table's threshold) or -1 (all tiles);
                                     // the launcher resolves it
  // A step may run a kernel twice, once per rank class, so that each launch cuts its operand
  // ring for the ranks it meets.  A launch of a class works on class_list[0 .. *class_count):
  // the indices of its tiles in `tiles`, in order (written on the device ahead of the
  // launches).  null = every tile.
  const int32_t* class_list;
  const int32_t* class_count;
  // adapter tables
  const int64_t* a_start;
  const int64_t* a_loc;
  int64_t slot;                      // qkvo
  int mode;
  // step mode: problem blockIdx.z of the plan supplies tensor maps, pointers and
  // index tables; the shrink result of problem p is vbuf + p * vstride elements
  // (row pitch kMaxRank)
  const StepProblem* plan;
  void* vbuf;
  int64_t vstride;
  // debug builds: timing trace of CTA 0 (clock64 stamps, 8 per pipeline stage); null = off
  long long* trace;
  int64_t trace_cap;
  // device status word of this launch (see raise_status); null = the process-wide one
  int* status;
  // shrink only: per-adapter scales (launch dtype) applied in fp32 before the single rounding
  // of the result, for callers that consume a pre-scaled V' (the fused projection); null = none
  const void* shrink_scales;
  // work distribution: null = item k of a CTA is blockIdx.x + k * gridDim.x; else a
  // zeroed device counter from which the CTAs draw their next item (after the first)
  unsigned int* item_counter;
  // work decomposition, filled by the launcher
  int64_t max_tiles;                 // mode 0: upper bound of the tile count
  int tile_rows;                     // mode 0, shrink: rows per tile (32 or 128; 0 = 128)
  int n_problems;
  int nsplit;                        // expand: work items per tile (column shares)
  // operand rings, sized by the launcher from the largest rank the launch may meet - or, where
  // set, from ring_rank: the largest rank among the tiles whose stages need the ring cut for
  // them (consecutive-row tiles; the stages of a gather tile fit a 48 KB stage at every rank)
  int max_rank;
  int ring_rank;
  int shrink_stages, shrink_stage_bytes;
  int exp_stages, exp_stage_bytes;
};

int sm_count();

// launchers shared between the single-problem entry points and the step entry point
int make_map_2d(CUtensorMap* map, const void* ptr, int dtype, int64_t rows, int64_t cols, int box_rows);
int make_map_set(MapSet* set, const void* act, int64_t act_rows, const void* w, int64_t w_rows,
                 int64_t cols, int dtype, int gather_weight_maps = 0);   // 1: w3 (shrink side), 2: wb3 (expand side)
int bgmv_gather_launch(void* y, const void* x, const void* w, const void* scales,
                       const BgmvGroups& groups, int64_t max_groups, int h_in, int h_out,
                       int layout, int dtype, cudaStream_t stream, int n_problems);
int bgmv_decode_launch(void* y, const void* x, const void* w, const void* scales,
                       const int64_t* indicies, int64_t batch, const int64_t* a_start,
                       const int64_t* a_len, const int64_t* a_loc, int64_t qkvo, int h_in, int h_out,
                       int dtype, cudaStream_t stream);
int bgmv_decode_status(int reset);
void bgmv_decode_set_trace(long long* dev_buffer, long long n);
int atmm_launch(void* y, const void* x, const void* w, const void* scales, const TileSource& src,
                int64_t max_tiles, int64_t T_rows, int h_in, int h_out, int64_t w_cells, int dtype,
                int flags, cudaStream_t stream, int n_problems);

}  // namespace vlr
