/*
 * libvlr - C ABI of the B200 (sm_100a) multi-LoRA batching operator.
 *
 * Plain pointers and sizes only.  Every pointer named "device" must be device
 * memory of the CURRENT CUDA device of the calling thread, and the stream must
 * belong to it (vlr_set_device binds a thread).  The library allocates no
 * device memory.  State it keeps between calls: a cached driver entry point
 * for tensor-map encoding, per-device flags for kernel attributes, the
 * process-wide device status word (vlr_device_status), and the per-device
 * address of the built-in scratch of vlr_pack_static.  All work is enqueued on
 * the stream passed in (a cudaStream_t cast to void*; NULL = the legacy default
 * stream) and the calls return without synchronising.
 *
 * Return value: 0 on success, a negative VLR_ERR_* code when host-side argument
 * validation fails (nothing was launched), or a positive cudaError_t value
 * when a launch failed.  vlr_error_string() explains either.
 *
 * The citations give the reference interface each entry point replaces
 * (paths relative to the reference project root).
 */
#ifndef VLR_H_
#define VLR_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VLR_OK 0
#define VLR_ERR_NULL -1          /* a required pointer is NULL */
#define VLR_ERR_SHAPE -2         /* unsupported feature sizes / ranks */
#define VLR_ERR_DTYPE -3         /* dtype is neither VLR_F16 nor VLR_BF16 */
#define VLR_ERR_ALIGN -4         /* a pointer or row pitch is not 16-byte aligned */
#define VLR_ERR_WORKSPACE -5     /* workspace too small */
#define VLR_ERR_RANGE -6         /* a count or capacity is out of range */
#define VLR_ERR_DRIVER -7        /* tensor-map encoding is unavailable or failed */
#define VLR_ERR_UNSUPPORTED -8   /* valid request this build does not implement */
#define VLR_ERR_STATIC_LIMIT -9  /* batch larger than the built-in scratch of vlr_pack_static */

#define VLR_F16 0
#define VLR_BF16 1

/* Layout of the B side of an adapter slot in the pool. */
#define VLR_LAYOUT_PUNICA 0 /* the slot's r cells hold the flat bytes of [H_out, r]
                               (valora/csrc/bgmv/bgmv_impl.cuh:174-179) */
#define VLR_LAYOUT_ROWS 1   /* cell k of the slot is row k of B [r, H_out]
                               (atmm/valora/csrc/bgmv/bgmv_impl.cuh:114-123) */

/* flags of vlr_atmm */
#define VLR_ATMM_ACCUMULATE_SHRINK 1 /* shrink adds into y (reference epilogue beta = 1,
                                        atmm/valora/csrc/bgmv/bgmv_impl.cuh:174); default overwrites */
#define VLR_ATMM_APPLY_SCALE 2       /* the call multiplies its result by lora_scales[adapter] in fp32
                                        before the single rounding (an expand: the update; a shrink:
                                        V' = s X A, what vlr_fused_proj consumes); the reference
                                        epilogue uses alpha = 1 (same file :174, :236) */
#define VLR_ATMM_FULL_TILES 4        /* shrink: always cut segments into 128-row tiles.  Without it a
                                        call with few rows (T/128 + num_problems <= half the SMs) uses
                                        32-row tiles: more CTAs, each walking K in fewer, fuller stages */

/* kinds in the tile schedule written by vlr_pack */
#define VLR_TILE_MMA 0
#define VLR_TILE_GATHER 1
#define VLR_TILE_INTS 8   /* int32 per tile: kind, adapter, rank, first, nrows, segment, sorted_pos, 0 */

/* indices into the counts array written by vlr_pack */
#define VLR_COUNT_SEGMENTS 0
#define VLR_COUNT_MMA_TILES 1
#define VLR_COUNT_GATHER_TILES 2
#define VLR_COUNT_GATHER_ROWS 3
#define VLR_COUNT_STATUS 4     /* 0 ok, 1 an adapter id was out of range (served as adapter 0),
                                  2 tile capacity exceeded */
#define VLR_COUNT_INTS 8

int vlr_version(void);
const char* vlr_error_string(int code);

/*
 * Decode gather mat-vec.  Replaces valora._kernels.dispatch_bgmv
 * (valora/csrc/lora_ops.cc:76-126; kernels valora/csrc/bgmv/bgmv_impl.cuh:14-241).
 *
 * h_in >= h_out selects the shrink: for token b with adapter a = indicies[b],
 * r = a_len[a] / 4, and j < r:
 *     y[b, j] = sum_k x[b, k] * w[a_loc[a_start[a] + r*qkvo + j], k]     (overwrites)
 * h_in < h_out selects the expand (x is [batch, h_in] with h_in = the buffer's
 * rank width; only the first r columns are read):
 *     y[b, o] += scale[a] * sum_{k<r} x[b, k] * B_a[k, o]
 * with B_a addressed per `layout`.  fp32 accumulation, one rounding to dtype.
 * w is [cells, H] with H = max(h_in, h_out) elements per cell.  r must be a
 * multiple of 8 and at most 128; H a multiple of 8.
 * All pointers device.  lora_scales has dtype `dtype`, one entry per adapter.
 */
int vlr_bgmv(void* y, const void* x, const void* w,
             const int64_t* a_start, const int64_t* a_len, const int64_t* a_loc,
             const int64_t* indicies, int64_t qkvo, const void* lora_scales,
             int64_t batch, int64_t h_in, int64_t h_out, int dtype, int layout, void* stream);

/*
 * Ragged grouped shrink / expand on the tensor cores.  Replaces
 * atmm_ops.dispatch_bgmv (atmm/valora/csrc/lora_ops.cc:115-186; host driver and
 * problem table atmm/valora/csrc/bgmv/bgmv_impl.cuh:76-125, 269-383).
 *
 * Problem i (i < num_problems): m = output_counts[i] rows starting at row
 * start_ids[i], rank r = rank_counts[i], adapter lora_ids[i]; the slot's r
 * weight rows are the r CONSECUTIVE cells from a_loc[a_start[adapter] + r*qkvo].
 * h_in >= h_out: shrink  y[rows, :r]  = x[rows, :] * W^T      (y is [T, h_out])
 * h_in <  h_out: expand  y[rows, :]  += x[rows, :r] * W       (x is [T, h_in])
 * fp32 accumulation in tensor memory, one rounding to dtype.  Ranks must be
 * multiples of 8 and at most 128.  a_len, indicies and tmp are accepted for
 * signature parity and not read; tmp may be NULL.  w is [w_cells, H].
 */
int vlr_atmm(void* y, const void* x, const void* w,
             const int64_t* a_start, const int64_t* a_len, const int64_t* a_loc,
             const int64_t* indicies, int64_t qkvo, const void* lora_scales,
             const int64_t* output_counts, const int64_t* rank_counts,
             const int64_t* lora_ids, const int64_t* start_ids,
             void* tmp, int64_t tmp_bytes, int64_t num_problems,
             int64_t T, int64_t h_in, int64_t h_out, int64_t w_cells,
             int dtype, int flags, void* stream);

/*
 * On-device ragged-batch packing.  Replaces the host metadata build
 * ModelRpcServer.set_sgmm_args (valora/server/router/model_infer/model_rpc.py:265-374)
 * and implements what count_consecutive_requests
 * (atmm/valora/csrc/bgmv/bgmv_impl.cuh:39-72) was meant to do.
 *
 * tok_adapter[T] is the adapter id of every token in batch order; a_len[a] is
 * 4 * rank(a) as in the reference's index tables.  sort != 0: perm = stable
 * argsort(tok_adapter); sort == 0: perm = identity (reference order).  The run
 * length encoding of tok_adapter[perm] gives the segments:
 *   seg_len = output_counts, seg_rank = rank_counts, seg_adapter = lora_ids,
 *   seg_start = start_ids (P+1 entries, last = T).
 * The tile schedule (see VLR_TILE_*) cuts runs of consecutive original rows of
 * at least mma_min_rows rows into tiles of tile_m rows and groups the other
 * rows per adapter, gather_rows_per_tile at a time, listing their original
 * rows in gather_rows.  counts[VLR_COUNT_INTS] receives the totals.
 * Capacities: perm, gather_rows: T; seg_*: min(T, n_adapters or T) + 1;
 * tiles: tiles_cap tiles of VLR_TILE_INTS int32.
 * Limits: tile_m <= 128 (one MMA tile), gather_rows_per_tile <= 32, else
 * VLR_ERR_RANGE.  Four small launches; counts is written in full every call.
 */
size_t vlr_pack_workspace_bytes(int64_t T, int64_t n_adapters);
int vlr_pack(const int64_t* tok_adapter, int64_t T, const int64_t* a_len, int64_t n_adapters,
             int sort, int tile_m, int mma_min_rows, int gather_rows_per_tile,
             int32_t* perm, int64_t* seg_len, int64_t* seg_rank, int64_t* seg_adapter,
             int64_t* seg_start, int32_t* tiles, int64_t tiles_cap, int32_t* gather_rows,
             int32_t* counts, void* workspace, size_t workspace_bytes, void* stream);

/*
 * vlr_pack with no scratch argument.  No counterpart in the reference (there
 * the metadata buffers are module-level CUDA tensors that reset_sgmm re-creates
 * for every forward, valora/server/router/req_queue.py:35-42).
 *
 * For callers that cannot supply device scratch: a step that runs after the
 * serving pool has claimed the GPU's remaining memory, or host code behind an
 * FFI that has no allocator and must not provoke the device synchronisation an
 * allocation implies.  The scratch is a 1 MiB array inside the library's device
 * image (every GPU that loads the library carries it until the process ends).
 * Same arguments, outputs and results as vlr_pack, bit for bit.
 * Limits: T <= 8192 and n_adapters <= 1024, else VLR_ERR_STATIC_LIMIT.
 * The array is shared by all calls on a device and not cleared between them
 * (the packer writes everything before reading it); calls whose kernels overlap
 * on the GPU race on it - keep them on one stream.  The first call on a device
 * resolves the array's address (cudaGetSymbolAddress) and should be made before
 * any stream capture starts.  The call allocates nothing.
 */
int vlr_pack_static(const int64_t* tok_adapter, int64_t T, const int64_t* a_len, int64_t n_adapters,
                    int sort, int tile_m, int mma_min_rows, int gather_rows_per_tile,
                    int32_t* perm, int64_t* seg_len, int64_t* seg_rank, int64_t* seg_adapter,
                    int64_t* seg_start, int32_t* tiles, int64_t tiles_cap, int32_t* gather_rows,
                    int32_t* counts, void* stream);

/*
 * Index-table compaction after adapters are offloaded.  Replaces
 * var_len_copy_kernel_triton (valora/server/router/model_infer/infer_adapter.py:263-282):
 * new_loc[new_start[i] + k] = old_loc[old_start[i] + k] for k < len[i], i < n.
 */
int vlr_var_len_copy(const int64_t* old_start, const int64_t* len, const int64_t* old_loc,
                     const int64_t* new_start, int64_t* new_loc, int64_t n, void* stream);

/*
 * Base projection with the LoRA update folded into the same accumulator:
 *     y[rows, :] = x[rows, :] W  +  v[rows, :r] B_a
 * for the rows of the consecutive-row tiles of a packed batch (tiles / counts from
 * vlr_pack: up to 128 rows of one adapter each), 256 output columns per work
 * item.  v is the pre-scaled shrink result V' = s X A (vlr_atmm or the step's
 * shrink with the scale applied), [T, v_pitch]; W is the base weight [h_in,
 * h_out] row-major; B_a the adapter's r rows in the B-side pool (consecutive
 * cells from a_loc_b[a_start_b[a] + r * slot_b]).  y is WRITTEN, never read:
 * the read-modify-write of y that the expand needs disappears, and with it two
 * thirds of the operator's HBM bytes.  Rows outside the consecutive-row tiles
 * (gather rows, i.e. decode tokens) are not touched; they go through a plain
 * base projection plus the gather expand.  h_in and h_out multiples of 64.
 * In the reference the two halves are a torch.mm that writes q / k / v / o and
 * dispatch_sgmm calls that read them back and add
 * (valora/models/peft/lora_unordered_batch_infer.py:885, :967-988, :1568,
 * :1611-1622; base weights valora/models/llama/layer_infer/
 * transformer_layer_infer.py:42-50).  dev_status as in vlr_lora_step.
 */
int vlr_fused_proj(void* y, const void* x, const void* w_base, const void* v, int64_t v_pitch,
                   const void* wb_pool, int64_t cells_b, const int64_t* a_start_b,
                   const int64_t* a_loc_b, int64_t slot_b, const int32_t* tiles,
                   const int32_t* counts, int64_t max_mma_tiles, int64_t T, int64_t h_in,
                   int64_t h_out, int dtype, int32_t* dev_status, void* stream);

/*
 * The tile table: what a launch of the tensor-core kernels is shaped like, per
 * kind of call and rank bound.  Replaces the reference's table of six CUTLASS
 * tile integers per (adapters, first sequence length, K, N), measured on an
 * Ampere part (valora/models/peft/lora_unordered_batch_infer.py:25-172,216-236;
 * search space atmm/valora/csrc/bgmv/bgmv_config.h:11-31).  Here the MMA tile
 * is fixed by the instruction (128 rows); what is chosen is how the 192 KB
 * operand ring is cut into stages - which sets how many K blocks (shrink) or
 * 64-column blocks (expand) of a tile travel together, i.e. how long the
 * contiguous piece of every row is that one stage requests - and the row count
 * of the tiles of a drop-in shrink with few rows.  An entry applies to launches
 * whose rank bound is <= max_rank (the entry with the smallest such max_rank
 * wins).  The table is process-wide; set it before launching, not concurrently
 * with launches.  valora_b200/tile_table.json holds the measured table and the
 * autotuner that writes it is `python -m valora_b200.autotune`.
 */
typedef struct {
  int32_t max_rank;        /* 8..128 */
  int32_t step;            /* 1: launches of vlr_lora_step, 0: single vlr_atmm calls */
  int32_t shrink_stages;   /* 2, 3 or 4 stages of 96 / 64 / 48 KB; ranks above 64 need <= 3 */
  int32_t expand_stages;   /* 3 or 4 stages of 64 / 48 KB; ranks above 64 need 3 */
  int32_t small_call_rows; /* vlr_atmm shrink with T/128 + num_problems <= half the SMs: 32, 64 or 128 */
  int32_t wide_gather_below_rank; /* expand: gather tiles of adapters below this rank use wide stages (0: none) */
} vlr_tile_choice_t;
int vlr_set_tile_table(const vlr_tile_choice_t* entries, int n);   /* n <= 16; n = 0: built-in rules */
int vlr_get_tile_choice(int step, int max_rank, vlr_tile_choice_t* out);

/* Bind the calling thread's CUDA runtime state to a device (cudaSetDevice). */
int vlr_set_device(int device);

/* Process-wide device status word, a bit set: 1 a bounded wait inside a kernel
 * gave up (the kernel returned early and its output is incomplete), 2 a tile
 * record was outside what its launch supports and was skipped (rank above the
 * launch's max_rank or not a multiple of 8, too many rows).  0 = ok.
 * Synchronises the device.  reset != 0 clears it.  vlr_lora_step can be given
 * a status word of its own instead (dev_status), which the caller reads when
 * and how it likes (no synchronisation here, usable under stream capture). */
int vlr_device_status(int reset);

/* Self-test of the bounded waits: one thread waits on a barrier nothing ever
 * completes, gives up after budget_cycles (1 .. 2e9) and raises status bit 1 in
 * *dev_status (NULL: the process-wide word).  dev_waited_cycles (may be NULL)
 * receives the cycles the wait took.  The kernel returns normally; nothing
 * faults and the context stays usable.  No counterpart in the reference, whose
 * kernels have no waits of this kind and whose launch failures are printed and
 * swallowed (atmm/valora/csrc/bgmv/bgmv_impl.cuh:185-198). */
int vlr_selftest_bounded_wait(int64_t budget_cycles, int32_t* dev_status,
                              int64_t* dev_waited_cycles, void* stream);

/*
 * One step over many projections: shrink then expand of every (layer, projection)
 * problem of a packed batch, enqueued as batched launches that cover all problems
 * at once: tensor-core shrink and expand, plus (unless
 * VLR_STEP_GATHER_ON_TENSOR_CORES is set) a SIMT gather shrink and expand.  No counterpart in the reference, which issues 6-8 calls per
 * layer from Python with a host synchronisation after each
 * (valora/models/peft/lora_unordered_batch_infer.py:946-988).
 *
 * A problem is y[T, h_out] += scale[a] * (x[T, h_in] A_a) B_a over the packed
 * batch.  A rows live in pool wa ([cells_a, h_in], cell = one rank row), B rows
 * in pool wb ([cells_b, h_out], cell = one row of B; the r cells of a slot are
 * consecutive for tensor-core tiles).  The slot of adapter a starts at cell
 * a_loc[a_start[a] + rank(a) * slot].
 *
 * vlr_step_plan_build fills plan_host (vlr_step_plan_bytes(n) bytes, host memory)
 * from the problem list; the caller copies it to 128-byte aligned device memory
 * and passes that to vlr_lora_step.  A plan stays valid while the buffers it
 * names stay allocated; max_rows is the row capacity of every x / y buffer.
 */
typedef struct {
  const void* x;            /* device [max_rows, h_in] */
  void* y;                  /* device [max_rows, h_out] */
  const void* wa;           /* device A-side pool */
  const void* wb;           /* device B-side pool */
  const int64_t* a_start_a; /* device index tables of the A-side pool */
  const int64_t* a_loc_a;
  const int64_t* a_start_b; /* device index tables of the B-side pool */
  const int64_t* a_loc_b;
  int64_t cells_a;
  int64_t cells_b;
  int32_t h_in;
  int32_t h_out;
  int32_t slot_a;
  int32_t slot_b;
} vlr_problem_t;

size_t vlr_step_plan_bytes(int n_problems);
int vlr_step_plan_build(const vlr_problem_t* problems, int n_problems, int64_t max_rows, int dtype,
                        void* plan_host);
/* workspace: the shrink results (n_problems * T * 128 elements), the work-item counters and
 * the tile lists of the two rank classes (16 T bytes) */
size_t vlr_lora_step_workspace_bytes(int64_t T, int n_problems);
/*
 * plan_dev: device copy of the plan.  tiles / gather_rows / counts: device
 * outputs of vlr_pack for this step's batch.  max_mma_tiles / max_gather_tiles:
 * host-side upper bounds used to size the grids (surplus CTAs exit at once);
 * pass <= 0 for the safe bounds derived from T.  scales: dtype[n_adapters].
 * max_h_in / max_h_out: the largest h_in / h_out over the plan's problems.
 * max_rank: the largest adapter rank the batch can contain (<= 0 or > 128 means 128).
 * A bound of 64 or less lets the kernels run deeper operand rings; tiles whose rank
 * exceeds the bound are skipped.
 * phase_mask: which of the four launches to enqueue (VLR_PHASE_ALL for a step;
 * single phases let a harness time each kernel on its own).
 * dev_status: device int32 the step's kernels OR their status bits into (see
 * vlr_device_status for the bits), or NULL for the process-wide word.  The
 * caller clears it and reads it (e.g. with the step's results).
 */
#define VLR_PHASE_SHRINK_MMA 1
#define VLR_PHASE_SHRINK_GATHER 2
#define VLR_PHASE_EXPAND_MMA 4
#define VLR_PHASE_EXPAND_GATHER 8
#define VLR_PHASE_ALL 15
/* or-ed into phase_mask: the gather tiles (rows that are not consecutive in the
 * batch, e.g. decode tokens) are processed by the two tensor-core launches, their
 * rows fetched with 128-byte 1-D bulk copies instead of tiled bulk copies; the
 * two SIMT gather launches are skipped.  gather_rows_per_tile must be <= 32 with
 * this flag and <= 8 without it.  Plans need h_in and h_out multiples of 64. */
#define VLR_STEP_GATHER_ON_TENSOR_CORES 16
/* or-ed into phase_mask together with VLR_STEP_GATHER_ON_TENSOR_CORES.  A gather
 * stage of the expand carries four 64-column blocks (two above rank 64), or - the
 * wide form - as many as the stage holds (up to 1024 columns), which pays for
 * small ranks whose weight rows fill a fraction of a stage otherwise.
 * VLR_STEP_WIDE_GATHER_STAGES: adapters of small rank may be in the batch; the form
 * is then chosen per tile, wide for adapters below the tile table's
 * wide_gather_below_rank.  Without it every gather tile takes the plain form (and
 * the kernel that runs has no per-tile choice to make, which the consecutive-row
 * tiles of the same launch gain from).  VLR_STEP_ALL_WIDE_GATHER_STAGES, with the
 * first: every gather tile takes the wide form (measurements, tests). */
#define VLR_STEP_WIDE_GATHER_STAGES 32
#define VLR_STEP_ALL_WIDE_GATHER_STAGES 64
/* or-ed into phase_mask.  With max_rank above 64: each tensor-core kernel is launched twice,
 * once over the consecutive-row tiles of adapters above rank 64, which need the 192 KB operand
 * ring cut into three stages, and once over all other tiles (consecutive rows up to rank 64,
 * gather tiles of any rank), which fit four stages and ran 18-34 % slower on three.  A small kernel ahead of them lists each class's
 * tiles in the workspace; the second class runs on a library-owned side stream, forked from
 * and joined to `stream` inside the call.  Same results bit for bit. */
#define VLR_STEP_SPLIT_RANK_CLASSES 128
int vlr_lora_step(const void* plan_dev, int n_problems, int64_t T, const int32_t* tiles,
                  const int32_t* gather_rows, int64_t max_mma_tiles, int64_t max_gather_tiles,
                  const int32_t* counts, const void* scales, int max_h_in, int max_h_out,
                  int max_rank, int dtype, int phase_mask, void* workspace, size_t workspace_bytes,
                  int32_t* dev_status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VLR_H_ */
