// Ragged grouped LoRA shrink (V = X A) and expand (Y += s V B) on the sm_100a
// tensor cores: tcgen05.mma with accumulators in tensor memory, operands staged
// in shared memory by tiled bulk tensor copies (TMA) behind an mbarrier ring.
//
// Persistent CTAs, one per SM, working through (problem, tile) items: a tile is up to 128
// consecutive rows of one segment, or up to 16 gathered rows of one adapter.  Roles
//   shrink: warps 0-2 TMA producers, 3 MMA issue + tensor-memory allocation,
//           4-7 epilogue (one TMEM lane quarter each), 8 work-item fetch
//   expand: warps 0-7 epilogue (lane quarter x 64-column block), 8-9 TMA producers,
//           10 MMA issue, 11 work-item fetch
// No cluster launch, no multicast copies, no peer memory.
//
// Shrink: A operand = X tile [128 x 64] (K-major), B operand = the adapter's A
// rows [r_pad x 64] (K-major: a pool cell is one rank row of length H_in);
// K loop over H_in.  Expand: A operand = V tile [128 x r_pad] (K-major, written
// to shared memory by the epilogue warps with the 128-byte swizzle), B operand
// = r_pad rows of B, 128 columns at a time (N contiguous = MN-major); the
// epilogue adds the caller's Y tile, which TMA staged beside B, rounds once and
// writes the rows of the segment back with coalesced 128-bit stores.
#include <cuda.h>

#include <string.h>

#include <type_traits>

#include "common.cuh"
#include "problem.cuh"
#include "sm100_ptx.cuh"

namespace vlr {

using namespace ptx;

constexpr int kTileM = 128;
// Warp roles.  Issuing a stage (barrier wait, expect_tx, two to four bulk copies)
// costs one thread several hundred cycles, so stages are dealt round-robin to
// several producer warps.  Epilogue warps start at a multiple of 4 so that
// warp % 4 is the tensor-memory lane quarter a warp may read.
constexpr int kShrinkProducers = 3;                    // warps 0..2, MMA = warp 3, epilogue = 4..7
constexpr int kShrinkMmaWarp = kShrinkProducers;
constexpr int kShrinkEpiWarp0 = 4;
constexpr int kShrinkFetchWarp = kShrinkEpiWarp0 + 4;   // warp 8: draws work items
constexpr int kThreads = 32 * (kShrinkFetchWarp + 1);
constexpr int kBoxRowsW = 16;        // weight rows per TMA box
constexpr int kBoxCols = 64;         // 64 two-byte elements = 128 bytes = swizzle span
constexpr int kGatherRows = 32;      // rows of a gather tile, at most (one producer lane per row)
// Tiles of 16 rows or fewer are laid out for 16 (N = 16 in the expand's transposed product, twice
// the K blocks per row copy in the shrink), the others for 32.
__device__ __forceinline__ int gather_cap(int rows) { return rows <= 16 ? 16 : 32; }

struct TileInfo {
  int valid;
  int row0;          // first row of the tile in x / y
  int rows;          // rows of the segment in this tile (1..128)
  int rank;          // true rank
  int adapter;
  int problem;       // index into the step plan (0 outside step mode)
  int split;         // expand: which share of the output columns
  int gather;        // 1: the rows are gather_rows[row0 .. row0+rows), not consecutive.
                     //    Row i of such a tile (at most 16 rows) goes to lane quarter i % 4 of the
                     //    128-row MMA tile, so that all four SM sub-partitions (each reads only its
                     //    own quarter of tensor memory) share the epilogue:
                     //    shrink: slot (i%4)*32 + (i/4)*8 - the first row of a swizzle atom, where
                     //            the 128-byte swizzle is the identity, so a plain 128-byte bulk
                     //            copy of the activation row lands in the right layout;
                     //    expand: the product is formed transposed, D^T = B^T V^T: the 128 output
                     //            columns of a block are the M side (tensor-memory lanes), the
                     //            gathered rows, dense in slots 0..15, are N = 16.  Every lane of
                     //            every epilogue warp then carries useful outputs.
  int64_t wrow0;     // first pool cell of the slot
};

// Consecutive activation rows [row0, row0 + rows) as one to two boxes (32 / 64 /
// 128 rows): the copy covers rows rounded up to 32.  dst is the tile's first row.
__device__ __forceinline__ int act_rows_loaded(int rows) { return (rows + 31) & ~31; }
__device__ __forceinline__ void load_act_rows(uint32_t dst, const MapSet* ms, int c0, int row0,
                                              int rows, uint32_t bar) {
  const int n32 = (rows + 31) >> 5;                  // 1..4
  if (n32 == 4) {
    tma_load_2d(dst, &ms->act[2], c0, row0, bar);
  } else if (n32 == 1) {
    tma_load_2d(dst, &ms->act[0], c0, row0, bar);
  } else {
    tma_load_2d(dst, &ms->act[1], c0, row0, bar);
    if (n32 == 3) tma_load_2d(dst + 64 * 128, &ms->act[0], c0, row0 + 64, bar);
  }
}
// n_pad (multiple of 16, <= 128) consecutive pool cells as at most four boxes
__device__ __forceinline__ void load_w_rows(uint32_t dst, const MapSet* ms, int c0, int row0,
                                            int n_pad, uint32_t bar) {
  int done = 0;
#pragma unroll
  for (int b = 3; b >= 0; --b) {
    const int h = 16 << b;
    if (n_pad - done >= h) {
      tma_load_2d(dst + done * 128, &ms->w[b], c0, row0 + done, bar);
      done += h;
    }
  }
}

// The gather form of the shrink: n_pad consecutive pool cells x g K blocks as at most four 3-D
// boxes; cell c's blocks land as the lines (c * g + j), j < g, behind one another.
__device__ __forceinline__ void load_w3_rows(uint32_t dst, const MapSet* ms, int gsel, int g, int kb0, int row0,
                                             int n_pad, uint32_t bar) {
  int done = 0;
#pragma unroll
  for (int b = 3; b >= 0; --b) {
    const int h = 16 << b;
    if (h * g <= 256 && n_pad - done >= h) {
      tma_load_3d(dst + (uint32_t)(done * g) * 128u, &ms->w3[gsel][b], 0, kb0, row0 + done, bar);
      done += h;
    }
  }
}

// Device-side status: bit 0 (1) a bounded wait gave up and the kernel returned early, bit 1
// (2) a tile record was outside what the launch supports (rank above the launch's bound or not
// a multiple of 8, more rows than a tile holds) and was skipped.  A step may name its own
// status word (TileSource::status); the other entry points use this process-wide one.
__device__ int g_status;
__device__ __forceinline__ void raise_status(const TileSource& src, int bits) {
  atomicOr(src.status != nullptr ? src.status : &g_status, bits);
}

// Item -> tile.  Warp-collective: all 32 lanes call it and all get the result.
// mode 1: item = (problem * n_tiles + tile) * nsplit + split, n_tiles on the device.
// mode 0: item = tile * nsplit + split over the reference's problem table; tiles
//         beyond the table's last one come back invalid.
__device__ __forceinline__ TileInfo get_tile(const TileSource& src, int64_t item, bool expand) {
  const int lane = threadIdx.x & 31;
  TileInfo ti;
  ti.valid = 0;
  ti.problem = 0;
  ti.gather = 0;
  ti.split = (int)(item % src.nsplit);
  const int64_t tb = item / src.nsplit;
  if (src.mode == 1) {
    const int n_tiles = src.class_list != nullptr
                            ? *src.class_count
                            : src.counts[VLR_COUNT_MMA_TILES] + (src.gather_mma ? src.counts[VLR_COUNT_GATHER_TILES] : 0);
    int b = (int)(tb % n_tiles);
    if (src.class_list != nullptr) b = __ldg(src.class_list + b);
    ti.problem = (int)(tb / n_tiles);
    // the records are the same for every problem of the step: read-only path, so that after a
    // CTA's first problem they come from L1
    const int32_t* t = src.tiles + (int64_t)b * VLR_TILE_INTS;
    const int4 r0 = __ldg(reinterpret_cast<const int4*>(t));
    ti.valid = 1;
    ti.gather = r0.x == VLR_TILE_GATHER;
    ti.adapter = r0.y;
    ti.rank = r0.z;
    ti.row0 = r0.w;
    ti.rows = __ldg(t + 4);
  } else {
    const int b = (int)tb;
    const int tm = (!expand && src.tile_rows > 0) ? src.tile_rows : kTileM;
    int base = 0;
    for (int64_t p0 = 0; p0 < src.num_problems; p0 += 32) {
      const int64_t p = p0 + lane;
      const int m = p < src.num_problems ? (int)src.output_counts[p] : 0;
      const int nt = m > 0 ? (m + tm - 1) / tm : 0;
      int inc = nt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
      }
      const int excl = base + inc - nt;
      const bool mine = nt > 0 && b >= excl && b < excl + nt;
      const unsigned who = __ballot_sync(0xffffffffu, mine);
      if (who) {
        const int srcl = __ffs(who) - 1;
        const int m0 = (b - __shfl_sync(0xffffffffu, excl, srcl)) * tm;
        const int64_t pp = p0 + srcl;
        ti.valid = 1;
        ti.adapter = (int)src.lora_ids[pp];
        ti.rank = (int)src.rank_counts[pp];
        ti.row0 = (int)src.start_ids[pp] + m0;
        ti.rows = min(tm, (int)src.output_counts[pp] - m0);
        break;
      }
      base += __shfl_sync(0xffffffffu, inc, 31);
    }
  }
  if (ti.valid) {
    if (ti.rank <= 0 || ti.rank > src.max_rank || (ti.rank & 7) || ti.rows <= 0 ||
        ti.rows > (ti.gather ? kGatherRows : kTileM)) {
      ti.valid = 0;                  // host validated what it could; skip bad entries, and say so
      if (lane == 0) raise_status(src, 2);
    } else {
      const int64_t* a_start = src.a_start;
      const int64_t* a_loc = src.a_loc;
      int64_t slot = src.slot;
      if (src.plan != nullptr) {
        const StepProblem& sp = src.plan[ti.problem];
        a_start = expand ? sp.a_start_b : sp.a_start_a;
        a_loc = expand ? sp.a_loc_b : sp.a_loc_a;
        slot = expand ? sp.slot_b : sp.slot_a;
      }
      ti.wrow0 = a_loc[a_start[ti.adapter] + (int64_t)ti.rank * slot];
    }
  }
  return ti;
}

__device__ __forceinline__ int64_t total_items(const TileSource& src) {
  if (src.mode == 1 && src.class_list != nullptr) return (int64_t)*src.class_count * src.n_problems * src.nsplit;
  if (src.mode == 1)
    return (int64_t)(src.counts[VLR_COUNT_MMA_TILES] +
                     (src.gather_mma ? src.counts[VLR_COUNT_GATHER_TILES] : 0)) *
           src.n_problems * src.nsplit;
  return src.max_tiles * src.nsplit;
}


// ---- which items a CTA works on
// With a device counter the CTAs draw items as they go (the first one is blockIdx.x, the
// k-th draw yields gridDim.x + k), which evens out tiles of very different sizes; without
// one, item k of a CTA is blockIdx.x + k * gridDim.x.  A fetch warp resolves each item -
// tile record, problem width, first pool cell, rows of a gather tile: a chain of three
// dependent global loads - one item ahead of the other roles and publishes the result in
// a small ring in shared memory (a full and an empty mbarrier per slot).  Every other
// warp reads the ring in order, so all roles see the same sequence and none of them waits
// for global memory at an item boundary.
constexpr int kItemRing = 2;
constexpr int kItemSlotBytes = 1024;                   // shared memory for the ring's slots
struct ItemSlot {
  TileInfo ti;                                         // ti.valid: 1 work, 0 skip, -1 end of the sequence
  int h;                                               // shrink: the problem's h_in; expand: its h_out
  int pad_;
  const void* ybase;                                   // expand: the problem's Y
  int grow[kGatherRows];                               // rows of a gather tile
};
static_assert(sizeof(ItemSlot) * kItemRing <= kItemSlotBytes, "item slots outgrow their shared memory");
struct ItemFeed {
  uint32_t full0, empty0;                              // shared-memory addresses of the barriers
  ItemSlot* slots;
};
// Consumer side; all 32 lanes call these.  tile_wait returns the slot of item k (null if a
// bounded wait gave up); the caller copies what it needs and hands the slot back.
__device__ __forceinline__ const ItemSlot* tile_wait(const ItemFeed& f, uint32_t k,
                                                     volatile int* abort_flag) {
  const uint32_t s = k % kItemRing;
  bool ok = true;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(f.full0 + 8u * s, (k / kItemRing) & 1, abort_flag);
  ok = __shfl_sync(0xffffffffu, ok, 0);
  __syncwarp();
  return ok ? f.slots + s : nullptr;
}
__device__ __forceinline__ void tile_release(const ItemFeed& f, uint32_t k) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(f.empty0 + 8u * (k % kItemRing));
}
__device__ __forceinline__ bool next_tile(const ItemFeed& f, uint32_t k, volatile int* abort_flag,
                                          TileInfo& ti, int& h, const void*& ybase, int& grow_lane) {
  const ItemSlot* sl = tile_wait(f, k, abort_flag);
  if (sl == nullptr) return false;
  ti = sl->ti;
  h = sl->h;
  ybase = sl->ybase;
  grow_lane = sl->grow[threadIdx.x & (kGatherRows - 1)];
  tile_release(f, k);
  return ti.valid >= 0;
}
// The fetch warp's loop (all 32 lanes: get_tile is warp-collective).
__device__ __forceinline__ void feed_tiles(const TileSource& src, const ItemFeed& f, int64_t total,
                                           bool expand, int h_arg, const void* y_arg,
                                           volatile int* abort_flag) {
  const int lane = threadIdx.x & 31;
  // (A ring of four slots and drawing the next item one iteration ahead of its use were measured:
  // a CTA then sits on more undistributed items at the end of a launch - config 2's expand 1.25 ->
  // 1.41 ms, config 3 +3 % - and batches of small tiles gained nothing.)
  for (uint32_t k = 0;; ++k) {
    const uint32_t s = k % kItemRing;
    bool ok = true;
    if (lane == 0) ok = mbar_wait(f.empty0 + 8u * s, ((k / kItemRing) & 1) ^ 1, abort_flag);
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) return;
    long long item = 0;
    if (lane == 0) {
      if (src.item_counter == nullptr) item = (long long)blockIdx.x + (long long)k * gridDim.x;
      else item = k == 0 ? (long long)blockIdx.x
                         : (long long)gridDim.x + (long long)atomicAdd(src.item_counter, 1u);
      if (item >= total) item = -1;
    }
    item = __shfl_sync(0xffffffffu, item, 0);
    TileInfo ti;
    ti.valid = -1;
    ti.gather = 0;
    ti.rows = 0;
    ti.row0 = 0;
    ti.problem = 0;
    if (item >= 0) ti = get_tile(src, item, expand);
    int h = h_arg;
    const void* yb = y_arg;
    int g = 0;
    if (ti.valid > 0) {
      if (src.plan != nullptr) {
        const StepProblem& sp = src.plan[ti.problem];
        h = expand ? sp.h_out : sp.h_in;
        yb = sp.y;
      }
      if (ti.gather && lane < ti.rows) g = src.gather_rows[ti.row0 + lane];
    }
    ItemSlot* sl = f.slots + s;
    if (lane == 0) {
      sl->ti = ti;
      sl->h = h;
      sl->ybase = yb;
    }
    if (lane < kGatherRows) sl->grow[lane] = g;
    __syncwarp();
    if (lane == 0) mbar_arrive(f.full0 + 8u * s);
    if (item < 0) return;
  }
}

// Debug aid, compiled in with -DVLR_TRACE only: CTA 0 stamps clock64 into src.trace, slot
// `what` of stage `k`.
__device__ __forceinline__ void trace_stamp(const TileSource& src, uint32_t k, int what) {
#ifdef VLR_TRACE
  if (src.trace != nullptr && blockIdx.x == 0 && (int64_t)k * 8 + what < src.trace_cap)
    src.trace[(int64_t)k * 8 + what] = clock64();
#else
  (void)src; (void)k; (void)what;
#endif
}

// ============================================================================
// shrink: persistent CTAs, TMA ring over K, two tile buffers in tensor memory so
// the epilogue of one tile overlaps the main loop of the next.
// ============================================================================
// The operand ring is 192 KB.  A K block of a full tile is the X tile (16 KB) plus
// the adapter's rank rows (8 KB at rank 64, 16 KB at rank 128); a stage holds two of
// them (4 stages of 48 KB when the launch cannot meet a rank above 64, else 3 of
// 64 KB), shorter tiles up to four.  Stages of one K block each (8 x 24 KB) were 10 %
// slower: per-stage costs (copy issue, barrier round trips) are paid per stage, and a
// row's two 128-byte pieces are then requested together.  What bounds these kernels
// is bytes in flight per SM against a memory latency of roughly 2 us under load.
constexpr int kRingBytes = 192 * 1024;
constexpr int kShrinkMaxStages = 12;
constexpr int kShrinkMaxSub = 16;                      // K blocks per stage, at most
// The A operand of an MMA is a window of 128 rows (16 KB) from where a block's
// activation rows start, whatever was loaded there: the window of the ring's last
// block runs past the ring, so that much shared memory is allocated behind it.
constexpr int kShrinkSmem = 1024 + kRingBytes + 512 + kItemSlotBytes + kTileM * 128;   // + barriers, item slots, window slack

// A stage holds as many K blocks as fit: a block = the tile's activation rows
// (2 KB for gathered rows, 4..16 KB for consecutive ones) then the adapter's rank
// rows, both 64 columns wide.  Short tiles so keep as many bytes in flight as full ones.
struct SubLayout { uint32_t xbytes, sub; int kbs; };
__device__ __forceinline__ SubLayout sub_layout(const TileInfo& ti, int n_pad, uint32_t stage_bytes) {
  SubLayout sl;
  sl.xbytes = (uint32_t)(ti.gather ? gather_cap(ti.rows) : act_rows_loaded(ti.rows)) * 128u;
  sl.sub = sl.xbytes + (uint32_t)n_pad * 128u;
  const int k = (int)(stage_bytes / sl.sub);
  sl.kbs = k < 1 ? 1 : (k > kShrinkMaxSub ? kShrinkMaxSub : k);
  return sl;
}

// Gather tiles, where the activations are at least eight K blocks wide: a gathered row is
// fetched g K blocks at a time with ONE copy (a [1 row x g blocks x 64 columns] box of the 3-D
// view of the activations), which lands as g consecutive 128-byte lines.  Token i then owns
// the lines i*g .. i*g+g-1 of the stage's X region, line i*g+j holding its K block j.  The
// adapter's weights come the same way, as [cells x g blocks x 64 columns] boxes of the pool: rank
// row c's K block j is line c*g+j of the W region, so every weight row is read in pieces of
// g * 128 contiguous bytes (with one [cells x 64 columns] box per K block they were 128-byte
// pieces 8 KB apart, and a stage of such pieces took about 6000 cycles to land).  The W region
// is ONE K-major operand of n_pad*g rows, and one MMA per 16-column K slice (M = 128 lines,
// N = n_pad*g <= 256) multiplies the whole X region with it: accumulator column c*g+j pairs
// every line with rank row c of K block j.  Of those only the lines L with L % g == j mean
// anything (the others paired a token's block with another block's weights); the epilogue picks
// them and adds the g of them that belong to a token.  Four MMAs per stage instead of 4 g: at
// 60-80 cycles per MMA for the issuing thread, 256 narrow MMAs per tile had been what bounded
// these tiles below rank 128.
//   g = 8 K blocks per stage (rank <= 32), 4 (rank <= 64), 2 above - and no more than the 128
//   lines of the operand allow: 8 for tiles of up to 16 rows, else 4
// Stage: [X region, cap * g lines][W region, n_pad * g lines]
struct GatherLayout { int g, gsel; uint32_t xbytes, wbytes; };
__device__ __forceinline__ GatherLayout gather_layout(int n_pad, int rows) {
  GatherLayout gl;
  const int cap = gather_cap(rows);
  gl.g = min(n_pad <= 32 ? 8 : (n_pad <= 64 ? 4 : 2), kTileM / cap);
  gl.gsel = gl.g == 8 ? 2 : (gl.g == 4 ? 1 : 0);
  gl.xbytes = (uint32_t)(cap * gl.g) * 128u;
  gl.wbytes = (uint32_t)(n_pad * gl.g) * 128u;        // the whole W region
  return gl;
}
// Epilogue of such a tile: the 16 rank rows c0 .. c0+15 of this lane's line, which holds K block
// jj: accumulator columns (c0 + c) * G + jj.  G loads of 16 consecutive columns, each covering
// 16 / G rank rows with all their blocks.
template <int G>
__device__ __forceinline__ void gather_collect(uint32_t tcol0, int jj, uint32_t (&r)[16]) {
  constexpr int kPer = 16 / G;
#pragma unroll
  for (int a = 0; a < G; ++a) {
    uint32_t p[16];
    ptx::tmem_ld_32x16(tcol0 + (uint32_t)(a * 16), p);
    ptx::tmem_ld_wait();
#pragma unroll
    for (int k = 0; k < kPer; ++k) {
      uint32_t v = p[k * G];
#pragma unroll
      for (int j = 1; j < G; ++j) v = (jj == j) ? p[k * G + j] : v;
      r[a * kPer + k] = v;
    }
  }
}
constexpr int kGather3MinBlocks = 8;                   // K blocks an activation row must have for this form

template <typename T, int NST>
__global__ void __launch_bounds__(kThreads, 1)
atmm_shrink_kernel(const __grid_constant__ MapSet maps_,
                   T* __restrict__ v_, const T* __restrict__ x_, TileSource src, int h_in_,
                   int v_pitch_, int accumulate) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ volatile int abort_s;
  __shared__ uint32_t tmem_base_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t total = total_items(src);
  if ((int64_t)blockIdx.x >= total) return;            // nothing for this CTA: no TMEM taken

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr int nst = NST;                             // 4 stages of 48 KB or 3 of 64 KB
  constexpr uint32_t stage_bytes = kRingBytes / NST;
  const uint32_t bars = base + kRingBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kShrinkMaxStages + s); };
  auto tfull_bar = [&](int ab) { return bars + 8u * (2 * kShrinkMaxStages + ab); };
  auto tempty_bar = [&](int ab) { return bars + 8u * (2 * kShrinkMaxStages + 2 + ab); };
  ItemFeed feed;
  feed.full0 = bars + 8u * (2 * kShrinkMaxStages + 4);
  feed.empty0 = feed.full0 + 8u * kItemRing;
  feed.slots = reinterpret_cast<ItemSlot*>(smem_raw + (bars + 512u - smem_u32(smem_raw)));
  auto x_stage = [&](int s) { return base + (uint32_t)s * stage_bytes; };

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < nst; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int ab = 0; ab < 2; ++ab) {
      mbar_init(tfull_bar(ab), 1);
      mbar_init(tempty_bar(ab), 4);
    }
    for (int i = 0; i < kItemRing; ++i) {
      mbar_init(feed.full0 + 8u * i, 1);
      mbar_init(feed.empty0 + 8u * i, kShrinkFetchWarp);   // every other warp reads every item
    }
    fence_barrier_init();
  }
  if (warp == kShrinkMmaWarp) {
    tmem_alloc(smem_u32(&tmem_base_s), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  // Tensor memory: two tile buffers of 256 columns.  A buffer holds 256 / n_pad'
  // (n_pad' = 64 or 128) partial accumulators; the K slices of a stage go to them in
  // turn, so consecutive MMAs do not wait on each other's accumulator, and the
  // epilogue adds the partial sums.
  auto acc_stride = [](int n_pad) { return n_pad <= 64 ? 64 : 128; };

  if (warp < kShrinkProducers) {
    // ------------------------------------------------------------ producers (stage k -> warp k % 3)
    // lane 0: TMA boxes (weights; consecutive activation rows).  Gather tiles: lane i
    // fetches row i with a one-row box into row slot i; the copy engine applies the
    // 128-byte swizzle from the address bits, so the slots form a dense tile.
    // A producer waits for the release of the stage it is about to refill by phase parity, so
    // it must never get more than one round of the ring ahead of the release it waits for:
    // no more producers than stages (with two stages warp 2 only follows the item sequence).
    constexpr int nprod = NST < kShrinkProducers ? NST : kShrinkProducers;
    uint32_t kiter = 0;
    bool ok = true;
    for (uint32_t ik = 0; ok; ++ik) {
      TileInfo ti;
      int hw, grow_l;
      const void* yb;
      if (!next_tile(feed, ik, &abort_s, ti, hw, yb, grow_l)) break;
      if (!ti.valid) continue;
      const MapSet* ms = src.plan ? &src.plan[ti.problem].shrink : &maps_;
      const int h_in = hw;
      const int n_pad = (ti.rank + 15) & ~15;
      const int kblocks = (h_in + kBoxCols - 1) / kBoxCols;
      const bool mine = ti.gather && lane < ti.rows;
      const int grow = mine ? grow_l : 0;
      if (lane < 8) prefetch_tensormap(lane < 3 ? &ms->act[lane] : lane < 7 ? &ms->w[lane - 3] : &ms->row);
      if (lane >= 8 && lane < 11 && kblocks >= kGather3MinBlocks) prefetch_tensormap(&ms->row3[lane - 8]);
      if (ti.gather && kblocks >= kGather3MinBlocks) {
        // ---- gathered rows, g K blocks per copy (see gather_layout)
        const GatherLayout gl = gather_layout(n_pad, ti.rows);
        const int nstages = (kblocks + gl.g - 1) / gl.g;
        for (int st = 0; st < nstages; ++st, ++kiter) {
          if ((int)(kiter % nprod) != warp) continue;
          const int s = kiter % nst;
          const int kb0 = st * gl.g;
          if (lane == 0) {
            ok = mbar_wait(empty_bar(s), ((kiter / nst) & 1) ^ 1, &abort_s);
            if (ok) {
              trace_stamp(src, kiter, 0);
              // a box counts its full size, also where it reaches past the last K block (zero fill)
              mbar_expect_tx(full_bar(s), (uint32_t)ti.rows * (uint32_t)gl.g * 128u + gl.wbytes);
              load_w3_rows(x_stage(s) + gl.xbytes, ms, gl.gsel, gl.g, kb0, (int)ti.wrow0, n_pad, full_bar(s));
              trace_stamp(src, kiter, 3);
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);          // also orders expect_tx before the copies
          if (!ok) break;
          if (mine)
            tma_load_3d(x_stage(s) + (uint32_t)(lane * gl.g) * 128u, &ms->row3[gl.gsel], 0, kb0, grow, full_bar(s));
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        continue;
      }
      const SubLayout sl = sub_layout(ti, n_pad, stage_bytes);
      const int nstages = (kblocks + sl.kbs - 1) / sl.kbs;
      const uint32_t blk_bytes =
          (uint32_t)((ti.gather ? ti.rows : act_rows_loaded(ti.rows)) + n_pad) * 128u;
      for (int st = 0; st < nstages; ++st, ++kiter) {
        if ((int)(kiter % nprod) != warp) continue;              // another producer's stage
        const int s = kiter % nst;
        const int kb0 = st * sl.kbs;
        const int nsub = min(sl.kbs, kblocks - kb0);
        if (lane == 0) {
          ok = mbar_wait(empty_bar(s), ((kiter / nst) & 1) ^ 1, &abort_s);
          if (ok) {
            trace_stamp(src, kiter, 0);
            mbar_expect_tx(full_bar(s), blk_bytes * nsub);
            for (int j = 0; j < nsub; ++j) {
              const uint32_t sb = x_stage(s) + j * sl.sub;
              const int c0 = (kb0 + j) * kBoxCols;
              if (!ti.gather) load_act_rows(sb, ms, c0, ti.row0, ti.rows, full_bar(s));
              load_w_rows(sb + sl.xbytes, ms, c0, (int)ti.wrow0, n_pad, full_bar(s));
            }
            trace_stamp(src, kiter, 3);
          }
        }
        if (lane == 0 && !ok && !ti.gather) break;
        if (ti.gather) {
          ok = __shfl_sync(0xffffffffu, ok, 0);        // also orders expect_tx before the copies
          if (!ok) break;
          if (mine)
            for (int j = 0; j < nsub; ++j)
              tma_load_2d(x_stage(s) + j * sl.sub + lane * 128, &ms->row, (kb0 + j) * kBoxCols, grow,
                          full_bar(s));
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
    }
    __syncwarp();
    if (warp == 0 && lane == 0 && abort_s) {
      // drain: let every copy that was issued land before the CTA retires
      volatile int none = 0;
      const uint32_t first = kiter > (uint32_t)nst ? kiter - nst : 0;
      for (uint32_t k = first; k < kiter; ++k)
        mbar_wait(full_bar(k % nst), (k / nst) & 1, &none);
    }
  } else if (warp == kShrinkMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    uint32_t kiter = 0, li = 0;
    bool ok = true;
    for (uint32_t ik = 0; ok; ++ik) {
      TileInfo ti;
      int hw, grow_l;
      const void* yb;
      if (!next_tile(feed, ik, &abort_s, ti, hw, yb, grow_l)) break;
      if (!ti.valid) continue;
      if (lane == 0) {
        const int n_pad = (ti.rank + 15) & ~15;
        const int kblocks = (hw + kBoxCols - 1) / kBoxCols;
        const uint32_t idesc = instr_desc_f16(std::is_same<T, __nv_bfloat16>::value, n_pad, 0);
        const int ab = li & 1;
        const uint32_t tacc = tmem_base + ab * 256;
        const int astr = acc_stride(n_pad), nacc = 256 / astr;
        ok = mbar_wait(tempty_bar(ab), ((li >> 1) & 1) ^ 1, &abort_s);
        if (ok) tc_fence_after();
        if (ti.gather && kblocks >= kGather3MinBlocks) {
          // one MMA per K slice: the whole X region against the stage's W region (N = n_pad * g;
          // K blocks past the activations' width arrive as zeros on both sides)
          const GatherLayout gl = gather_layout(n_pad, ti.rows);
          const int nstages = (kblocks + gl.g - 1) / gl.g;
          const bool bf = std::is_same<T, __nv_bfloat16>::value;
          const int n_all = n_pad * gl.g;
          // above rank 64 (g = 2) as two MMAs of half the rank rows each: measured 6 % faster than one of N = 256
          const int n_mma = n_pad <= 64 ? n_all : n_all / 2;
          const uint32_t idesc_g = instr_desc_f16(bf, n_mma, 0);
          for (int st = 0; st < nstages && ok; ++st, ++kiter) {
            const int s = kiter % nst;
            ok = mbar_wait(full_bar(s), (kiter / nst) & 1, &abort_s);
            if (!ok) break;
            trace_stamp(src, kiter, 1);
            tc_fence_after();
            const uint64_t ad = smem_desc_sw128(x_stage(s), 16, 1024);
            const uint64_t bd = smem_desc_sw128(x_stage(s) + gl.xbytes, 16, 1024);
            for (int hN = 0; hN < n_all; hN += n_mma) {
              const uint64_t bh = bd + (uint64_t)((hN * 128) >> 4);
#pragma unroll
              for (int k = 0; k < kBoxCols / 16; ++k)
                umma_f16(tacc + (uint32_t)hN, ad + (uint64_t)(2 * k), bh + (uint64_t)(2 * k), idesc_g,
                         (st > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(empty_bar(s));
            trace_stamp(src, kiter, 2);
          }
        } else {
        const SubLayout sl = sub_layout(ti, n_pad, stage_bytes);
        const int nstages = (kblocks + sl.kbs - 1) / sl.kbs;
        uint32_t aoff = 0, first = (uint32_t)nacc;     // next accumulator chain; chains not yet started
        for (int st = 0; st < nstages && ok; ++st, ++kiter) {
          const int s = kiter % nst;
          ok = mbar_wait(full_bar(s), (kiter / nst) & 1, &abort_s);
          if (!ok) break;
          trace_stamp(src, kiter, 1);
          tc_fence_after();
          const int nsub = min(sl.kbs, kblocks - st * sl.kbs);
          // One thread issues at most one MMA per 55-60 cycles, and with N <= 64 that, not the
          // tensor pipe (about 48 cycles), is what a short tile's 256 MMAs cost: so nothing but
          // additions per instruction.  The address field of a descriptor counts 16-byte units:
          // + 2 per 16-column K slice, + sub / 16 per K block.
          uint64_t ad = smem_desc_sw128(x_stage(s), 16, 1024);
          uint64_t bd = smem_desc_sw128(x_stage(s) + sl.xbytes, 16, 1024);
          const uint64_t dstep = (uint64_t)(sl.sub >> 4);
          for (int j = 0; j < nsub; ++j) {
#pragma unroll
            for (int k = 0; k < kBoxCols / 16; ++k) {
              umma_f16(tacc + aoff, ad + (uint64_t)(2 * k), bd + (uint64_t)(2 * k), idesc, first == 0);
              aoff = (aoff + (uint32_t)astr) & 255u;
              first = first > 0 ? first - 1 : 0;
            }
            ad += dstep;
            bd += dstep;
          }
          umma_commit(empty_bar(s));
          trace_stamp(src, kiter, 2);
        }
        }
        if (ok) umma_commit(tfull_bar(ab));
        ++li;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
    }
  } else if (warp < kShrinkFetchWarp) {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const int row = q * 32 + lane;
    uint32_t li = 0;
    for (uint32_t ik = 0;; ++ik) {
      TileInfo ti;
      int hw, grow_l;
      const void* yb;
      if (!next_tile(feed, ik, &abort_s, ti, hw, yb, grow_l)) break;
      if (!ti.valid) continue;
      const int ab = li & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(tfull_bar(ab), (li >> 1) & 1, &abort_s))) break;
      tc_fence_after();
      T* v = v_;
      int v_pitch = v_pitch_;
      if (src.plan != nullptr) {
        v = reinterpret_cast<T*>(src.vbuf) + (int64_t)ti.problem * src.vstride;
        v_pitch = kMaxRank;
      }
      const int n_pad = (ti.rank + 15) & ~15;
      // 16 finished sums of one row, columns c .. c+15, rounded once and stored (columns >= rank stay)
      const float vscale = src.shrink_scales != nullptr
                               ? Elem<T>::to_float(reinterpret_cast<const T*>(src.shrink_scales)[ti.adapter])
                               : 1.f;
      auto store16 = [&](T* vrow, int c, const uint32_t (&r)[16]) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int col = c + h * 8;
          if (col < ti.rank) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = vscale * __uint_as_float(r[h * 8 + e]);
            if (accumulate) {
              float old[8];
              unpack8<T>(ldg128(vrow + col), old);
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] += old[e];
            }
            stg128(vrow + col, pack8<T>(f));
          }
        }
      };
      const uint32_t tbuf = tmem_base + ((uint32_t)(q * 32) << 16) + ab * 256;
      if (ti.gather && (hw + kBoxCols - 1) / kBoxCols >= kGather3MinBlocks) {
        // gathered rows fetched g K blocks per copy: this lane holds line L of the X region =
        // K block jj of token tok; of accumulator a only the lines with jj == a count, and a
        // token's result is the sum over its g lines (see gather_layout)
        const GatherLayout gl = gather_layout(n_pad, ti.rows);
        const int tok = row >> (gl.gsel + 1), jj = row & (gl.g - 1);
        const int my_row = __shfl_sync(0xffffffffu, grow_l, tok & (kGatherRows - 1));
        if (q * 32 < ti.rows * gl.g) {
          T* vrow = v + (int64_t)(tok < ti.rows ? my_row : 0) * v_pitch;
          for (int c = 0; c < n_pad; c += 16) {
            uint32_t r[16];
            const uint32_t tcol0 = tbuf + (uint32_t)(c * gl.g);
            if (gl.g == 8) gather_collect<8>(tcol0, jj, r);
            else if (gl.g == 4) gather_collect<4>(tcol0, jj, r);
            else gather_collect<2>(tcol0, jj, r);
            for (int o = 1; o < gl.g; o <<= 1) {
#pragma unroll
              for (int e = 0; e < 16; ++e)
                r[e] = __float_as_uint(__uint_as_float(r[e]) +
                                       __uint_as_float(__shfl_xor_sync(0xffffffffu, r[e], o)));
            }
            if (jj == 0 && tok < ti.rows) store16(vrow, c, r);
          }
        }
      } else {
        // tile row held by this lane (gathered rows sit in slots 0..15: lane quarter 0)
        const int trow = ti.gather ? (q == 0 && lane < kGatherRows ? lane : kTileM) : row;
        const bool warp_live = ti.gather ? q == 0 : q * 32 < ti.rows;
        if (warp_live) {
          T* vrow = v + (int64_t)(trow < ti.rows ? (ti.gather ? grow_l : ti.row0 + trow) : 0) * v_pitch;
          const int astr = acc_stride(n_pad), nacc = 256 / astr;
          for (int c = 0; c < n_pad; c += 16) {
            uint32_t r[16];
            tmem_ld_32x16(tbuf + c, r);
            for (int a = 1; a < nacc; ++a) {
              uint32_t p[16];
              tmem_ld_32x16(tbuf + a * astr + c, p);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 16; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) + __uint_as_float(p[e]));
            }
            tmem_ld_wait();
            if (trow < ti.rows) store16(vrow, c, r);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(ab));
      ++li;
    }
    tc_fence_before();
  } else {
    // ------------------------------------------------------------ work items
    feed_tiles(src, feed, total, false, h_in_, nullptr, &abort_s);
  }
  __syncthreads();
  if (warp == kShrinkMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && abort_s) raise_status(src, 1);
}

// ============================================================================
// expand: persistent CTAs; per tile the V rows are staged once as the A operand,
// then the ring streams (B tile, Y tile) pairs, 128 output columns each (more for
// gather tiles).
// ============================================================================
constexpr int kExpMaxStages = 4;
constexpr int kExpEpiWarps = 8;                        // 2 per TMEM lane quarter, 64 columns each
constexpr int kExpEpiWarp0 = 0;                        // epilogue = warps 0..7
constexpr int kExpProducers = 2;                       // producers = warps 8..9
constexpr int kExpProdWarp0 = kExpEpiWarps;
constexpr int kExpMmaWarp = kExpProdWarp0 + kExpProducers;   // warp 10
constexpr int kExpFetchWarp = kExpMmaWarp + 1;           // warp 11: draws work items
constexpr int kExpThreads = 32 * (kExpFetchWarp + 1);
constexpr int kExpTileN = 128;
constexpr int kExpABytes = 2 * kTileM * 128;           // V tile, two 64-column K blocks: 32 KB
// A stage holds the B rows of its columns (64-column blocks k_pad * 128 bytes apart)
// followed by the Y rows: 16 + 32 KB for a 128-row tile of rank <= 64, 32 + 32 KB at
// rank 128, 32 + 8 KB for a 256-column gather tile.  Launches that cannot meet a rank
// above 64 run four 48 KB stages, the others three 64 KB stages.
constexpr int kExpAccBufs = 4;                         // accumulators of 128 TMEM columns
constexpr int kExpSmem = 1024 + kExpABytes + kRingBytes + 512 + kItemSlotBytes;      // + barriers, item slots

// A work item's output tiles.  Consecutive-row tiles use 128 columns per stage
// (B 64-column blocks 16 KB apart).  Gather tiles stream almost only weights, so
// with rank <= 64 they take 256 columns per stage (blocks 8 KB apart): twice the
// bytes in flight per stage.
struct ExpRange { int nt_begin, nt_count, h_out, ncbt, tile_n; uint32_t bstride, yoff; };

// Wide gather stages: a gather tile of an adapter below the launch's rank threshold
// (TileSource::wide_below_rank, from the tile table) takes as many 64-column blocks (weights
// + the rows' pieces) as the stage holds - an even number, at most 256 / row slots - instead
// of four: a small rank's weight rows would fill a fraction of a stage otherwise.  Decided
// per tile, so a pool of mixed ranks gets the better shape for each of its adapters - in the
// WIDE instantiation only, which a launch uses when such adapters may be in the batch: the
// other one keeps the stage shape a compile-time matter, and the consecutive-row path of a
// rank-64 step is 8-18 % faster for it (config 3's expand 5.24 against 6.20 ms).
template <bool WIDE>
__device__ __forceinline__ ExpRange exp_range(const TileSource& src, const TileInfo& ti, int h_out) {
  ExpRange r;
  r.h_out = h_out;
  r.bstride = (uint32_t)(((ti.rank + 15) & ~15) * 128);
  r.ncbt = (ti.gather && ti.rank <= 64) ? 4 : 2;
  if (WIDE && ti.gather && ti.rank < src.wide_below_rank) {
    const int cap = gather_cap(ti.rows);
    const int n = (int)((uint32_t)src.exp_stage_bytes / (r.bstride + cap * 128)) & ~1;
    const int most = 256 / cap;
    r.ncbt = n < 2 ? 2 : (n > most ? most : n);
  }
  r.tile_n = r.ncbt * kBoxCols;
  r.yoff = (uint32_t)r.ncbt * r.bstride;
  const int ntiles = (r.h_out + r.tile_n - 1) / r.tile_n;
  const int per = (ntiles + src.nsplit - 1) / src.nsplit;
  r.nt_begin = ti.split * per;
  r.nt_count = max(0, min(per, ntiles - r.nt_begin));
  return r;
}

template <typename T, int NST, bool WIDE>
__global__ void __launch_bounds__(kExpThreads, 1)
atmm_expand_kernel(const __grid_constant__ MapSet maps_,
                   T* __restrict__ y_, const T* __restrict__ v_, const T* __restrict__ scales,
                   TileSource src, int h_out_, int v_pitch_, int apply_scale) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ volatile int abort_s;
  __shared__ uint32_t tmem_base_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t total = total_items(src);
  if ((int64_t)blockIdx.x >= total) return;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_tile = base;
  constexpr int nst = NST;                             // 3 stages of 64 KB or 4 of 48 KB
  constexpr uint32_t stage_bytes = kRingBytes / NST;
  constexpr int nacc = kExpAccBufs;                    // accumulators in tensor memory, 128 columns each
  constexpr uint32_t acc_cols = 512 / nacc;
  auto b_stage = [&](int s) { return base + kExpABytes + (uint32_t)s * stage_bytes; };
  const uint32_t bars = base + kExpABytes + kRingBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kExpMaxStages + s); };
  auto tfull_bar = [&](int ab) { return bars + 8u * (2 * kExpMaxStages + ab); };
  auto tempty_bar = [&](int ab) { return bars + 8u * (2 * kExpMaxStages + kExpAccBufs + ab); };
  const uint32_t a_ready_bar = bars + 8u * (2 * kExpMaxStages + 2 * kExpAccBufs);
  const uint32_t a_free_bar = bars + 8u * (2 * kExpMaxStages + 2 * kExpAccBufs + 1);
  ItemFeed feed;
  feed.full0 = bars + 8u * (2 * kExpMaxStages + 2 * kExpAccBufs + 2);
  feed.empty0 = feed.full0 + 8u * kItemRing;
  feed.slots = reinterpret_cast<ItemSlot*>(smem_raw + (bars + 512u - smem_u32(smem_raw)));

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < nst; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), kExpEpiWarps);
    }
    for (int ab = 0; ab < kExpAccBufs; ++ab) {
      mbar_init(tfull_bar(ab), 1);
      mbar_init(tempty_bar(ab), kExpEpiWarps);
    }
    mbar_init(a_ready_bar, 32 * kExpEpiWarps);
    mbar_init(a_free_bar, 1);
    for (int i = 0; i < kItemRing; ++i) {
      mbar_init(feed.full0 + 8u * i, 1);
      mbar_init(feed.empty0 + 8u * i, kExpFetchWarp);      // every other warp reads every item
    }
    fence_barrier_init();
  }
  if (warp == kExpMmaWarp) {
    tmem_alloc(smem_u32(&tmem_base_s), 512);           // two accumulators of up to 256 columns
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp >= kExpProdWarp0 && warp < kExpMmaWarp) {
    // ------------------------------------------------------------ producers (stage k -> warp k % 2)
    const int pw = warp - kExpProdWarp0;
    // lane 0: TMA boxes (B rows; consecutive Y rows).  Gather tiles: lane i copies the
    // stage's columns of Y row i with one 1-D bulk copy, rows packed row-major (read back
    // by the epilogue only, so no swizzle).
    uint32_t it = 0;
    bool ok = true;
    for (uint32_t ik = 0; ok; ++ik) {
      TileInfo ti;
      int hw, grow_l;
      const void* yb;
      if (!next_tile(feed, ik, &abort_s, ti, hw, yb, grow_l)) break;
      if (!ti.valid) continue;
      const ExpRange er = exp_range<WIDE>(src, ti, hw);
      const MapSet* ms = src.plan ? &src.plan[ti.problem].expand : &maps_;
      const T* yg = reinterpret_cast<const T*>(yb);
      const int k_pad = (ti.rank + 15) & ~15;
      const int y_rows = ti.gather ? ti.rows : act_rows_loaded(ti.rows);
      const bool mine = ti.gather && lane < ti.rows;
      const T* yrow = mine ? yg + (int64_t)grow_l * er.h_out : yg;
      if (lane < 7) prefetch_tensormap(lane < 3 ? &ms->act[lane] : &ms->w[lane - 3]);
      // tiles of a step whose rank rows are one box (16 / 32 / 64 / 128): the stage's column
      // blocks come as ONE copy of eight, four or two blocks - the same bytes to the same places as one
      // box per block, but the pieces of a weight row are then requested close together
      const int wb = (k_pad == 16) ? 0 : (k_pad == 32) ? 1 : (k_pad == 64) ? 2 : (k_pad == 128) ? 3 : -1;
      const bool blocks3 = src.plan != nullptr && wb >= 0 && (er.h_out & (kBoxCols - 1)) == 0;
      if (blocks3 && lane >= 8 && lane < (wb < 2 ? 11 : 10)) prefetch_tensormap(&ms->wb3[wb][lane - 8]);
      if (src.plan != nullptr && lane == 11) prefetch_tensormap(&ms->act3);
      for (int t = 0; t < er.nt_count; ++t, ++it) {
        if ((int)(it % kExpProducers) != pw) continue;            // the other producer's stage
        const int s = it % nst;
        const int n0 = (er.nt_begin + t) * er.tile_n;
        const int ncb = min(er.ncbt, (er.h_out - n0 + kBoxCols - 1) / kBoxCols);
        if (lane == 0) {
          ok = mbar_wait(empty_bar(s), ((it / nst) & 1) ^ 1, &abort_s);
          if (ok) {
            trace_stamp(src, it, 0);
            uint32_t bytes = (uint32_t)ncb * (uint32_t)(k_pad + y_rows) * 128u;
            if (ti.gather)
              bytes = (uint32_t)ncb * (uint32_t)k_pad * 128u +
                      (uint32_t)y_rows * (uint32_t)min(er.tile_n, er.h_out - n0) * 2u;
            mbar_expect_tx(full_bar(s), bytes);
            int cb = 0;
            if (blocks3) {
              if (wb < 2)
                for (; ncb - cb >= 8; cb += 8)
                  tma_load_3d(b_stage(s) + cb * er.bstride, &ms->wb3[wb][2], 0, (int)ti.wrow0, n0 / kBoxCols + cb,
                              full_bar(s));
              for (; ncb - cb >= 4; cb += 4)
                tma_load_3d(b_stage(s) + cb * er.bstride, &ms->wb3[wb][1], 0, (int)ti.wrow0, n0 / kBoxCols + cb,
                            full_bar(s));
              for (; ncb - cb >= 2; cb += 2)
                tma_load_3d(b_stage(s) + cb * er.bstride, &ms->wb3[wb][0], 0, (int)ti.wrow0, n0 / kBoxCols + cb,
                            full_bar(s));
            }
            for (; cb < ncb; ++cb)
              load_w_rows(b_stage(s) + cb * er.bstride, ms, n0 + cb * kBoxCols, (int)ti.wrow0,
                          k_pad, full_bar(s));
            if (!ti.gather) {
              // a full tile's two Y blocks as one copy where the plan has the map for it
              if (src.plan != nullptr && y_rows == kTileM && ncb == 2 && (er.h_out & (kBoxCols - 1)) == 0)
                tma_load_3d(b_stage(s) + er.yoff, &ms->act3, 0, ti.row0, n0 / kBoxCols, full_bar(s));
              else
                for (int cb2 = 0; cb2 < ncb; ++cb2)
                  load_act_rows((b_stage(s) + er.yoff) + cb2 * (kTileM * 128), ms, n0 + cb2 * kBoxCols, ti.row0,
                                ti.rows, full_bar(s));
            }
          }
        }
        if (lane == 0 && !ok && !ti.gather) break;
        if (ti.gather) {
          ok = __shfl_sync(0xffffffffu, ok, 0);        // also orders expect_tx before the copies
          if (!ok) break;
          // one copy per row: the stage's columns of Y row i, row-major behind the weights
          if (mine)
            bulk_load_1d((b_stage(s) + er.yoff) + lane * (er.tile_n * 2), yrow + n0,
                         (uint32_t)min(er.tile_n, er.h_out - n0) * 2u, full_bar(s));
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
    }
    __syncwarp();
    if (pw == 0 && lane == 0 && abort_s) {
      volatile int none = 0;
      const uint32_t first = it > (uint32_t)nst ? it - nst : 0;
      for (uint32_t k = first; k < it; ++k)
        mbar_wait(full_bar(k % nst), (k / nst) & 1, &none);
    }
  } else if (warp == kExpMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    uint32_t it = 0, li = 0;
    bool ok = true;
    for (uint32_t ik = 0; ok; ++ik) {
      TileInfo ti;
      int hw, grow_l;
      const void* yb;
      if (!next_tile(feed, ik, &abort_s, ti, hw, yb, grow_l)) break;
      if (!ti.valid) continue;
      const ExpRange er = exp_range<WIDE>(src, ti, hw);
      if (er.nt_count <= 0) continue;
      const int k_pad = (ti.rank + 15) & ~15;
      const int ksteps = k_pad / 16;
      const uint32_t idesc = instr_desc_f16(std::is_same<T, __nv_bfloat16>::value, er.tile_n, 1);
      const int gcap = gather_cap(ti.rows);            // N of the transposed product = row slots
      const uint32_t idesc_g = instr_desc_f16(std::is_same<T, __nv_bfloat16>::value, gcap, 0, 1);
      ok = __all_sync(0xffffffffu, mbar_wait(a_ready_bar, li & 1, &abort_s));
      for (int t = 0; t < er.nt_count && ok; ++t, ++it) {
        const int s = it % nst, ab = it & (nacc - 1);
        bool got = mbar_wait(full_bar(s), (it / nst) & 1, &abort_s);
        if (got) got = mbar_wait(tempty_bar(ab), ((it / nacc) & 1) ^ 1, &abort_s);
        ok = __all_sync(0xffffffffu, got);             // the whole warp goes on or gives up
        if (!ok) break;
        if (k_pad != ti.rank) {
          // rank % 16 == 8: rows rank..k_pad-1 of the B tile belong to the next slot.
          // The matching V columns are zero, but 0 * Inf/NaN would poison the sum.
          const int nrow = k_pad - ti.rank;            // 8
          for (int i = lane; i < er.ncbt * nrow * 8; i += 32) {
            const int cb = i / (nrow * 8), rr = (i / 8) % nrow, ch = i % 8;
            sts128(b_stage(s) + cb * er.bstride + (ti.rank + rr) * 128 + ch * 16,
                   make_uint4(0, 0, 0, 0));
          }
          fence_proxy_async_smem();
          __syncwarp();
        }
        tc_fence_after();
        if (lane == 0) {
          trace_stamp(src, it, 1);
          if (ti.gather) {
            // D^T[128 cols x N rows] = B^T[128 x k] * V^T[k x N], one chain per 128 columns:
            // A operand = the staged B tile read MN-major (two 64-column blocks bstride
            // apart), B operand = the V rows, K-major, N = 16 or 32 row slots; a chain takes N
            // accumulator columns
            const int kChainCols = gcap;
            for (int mt = 0; mt < (er.ncbt >> 1); ++mt)
              for (int j = 0; j < ksteps; ++j) {
                const uint64_t ad = smem_desc_sw128(b_stage(s) + mt * 2 * er.bstride + j * (kBoxRowsW * 128),
                                                    er.bstride, 1024);
                const uint64_t bd = smem_desc_sw128(a_tile + (j >> 2) * (kTileM * 128) + (j & 3) * 32, 16, 1024);
                umma_f16(tmem_base + ab * acc_cols + mt * kChainCols, ad, bd, idesc_g, j != 0);
              }
          } else {
            for (int j = 0; j < ksteps; ++j) {
              const uint64_t ad = smem_desc_sw128(a_tile + (j >> 2) * (kTileM * 128) + (j & 3) * 32, 16, 1024);
              const uint64_t bd = smem_desc_sw128(b_stage(s) + j * (kBoxRowsW * 128), er.bstride, 1024);
              umma_f16(tmem_base + ab * acc_cols, ad, bd, idesc, j != 0);
            }
          }
          umma_commit(tfull_bar(ab));
        }
        __syncwarp();
      }
      if (ok && lane == 0) umma_commit(a_free_bar);    // V tile may be overwritten once these retire
      __syncwarp();
      ++li;
    }
  } else if (warp < kExpEpiWarps) {
    // ------------------------------------------------------------ V staging + epilogue
    // 8 warps: warp (q, j) owns TMEM lanes 32q..32q+31 (rows) and the 64-column block j
    // (and j + 2 of a 256-column gather tile) of every output tile.  With few warps each
    // has registers to spare: both 32-column accumulator chunks and the eight Y pieces
    // of a block are fetched before the first result is needed.
    const int q = warp & 3;                            // the lane quarter a warp may read
    const int j = (warp - kExpEpiWarp0) >> 2;          // its 64-column block
    const int row = q * 32 + lane;
    const int et = threadIdx.x - 32 * kExpEpiWarp0;    // 0..255
    uint32_t it = 0, li = 0;
    bool ok = true;
    for (uint32_t ik = 0; ok; ++ik) {
      TileInfo ti;
      int hw, grow_l;
      const void* yb;
      {
        const ItemSlot* sl = tile_wait(feed, ik, &abort_s);
        if (sl == nullptr) break;
        ti = sl->ti;
        hw = sl->h;
        yb = sl->ybase;
        grow_l = sl->grow[lane & (kGatherRows - 1)];   // lane i keeps row i of a gather tile
        tile_release(feed, ik);
      }
      if (ti.valid < 0) break;
      if (!ti.valid) continue;
      const ExpRange er = exp_range<WIDE>(src, ti, hw);
      if (er.nt_count <= 0) continue;
      T* y = reinterpret_cast<T*>(const_cast<void*>(yb));
      const T* v = v_;
      int v_pitch = v_pitch_;
      if (src.plan != nullptr) {
        v = reinterpret_cast<const T*>(src.vbuf) + (int64_t)ti.problem * src.vstride;
        v_pitch = kMaxRank;
      }
      const int h_out = er.h_out;
      const int k_pad = (ti.rank + 15) & ~15;
      // consecutive rows: lane = row.  Gather tiles: lane = output column (see the
      // epilogue), warp j takes the j-th 128-column half of a stage.
      const bool warp_live = ti.gather ? j < (er.ncbt >> 1) : q * 32 < ti.rows;
      // ---- stage V as the K-major, 128-byte-swizzled A operand (zeros beyond rank / rows)
      ok = __all_sync(0xffffffffu, mbar_wait(a_free_bar, (li & 1) ^ 1, &abort_s));
      if (!ok) break;
      {
        const int vr = et & 127;                       // row slot
        const int vt = vr;                             // gathered rows sit densely in slots 0..15
        const T* vrow = v + (int64_t)(vt < ti.rows ? (ti.gather ? grow_l : ti.row0 + vt) : 0) * v_pitch;
        for (int c8 = et >> 7; c8 < k_pad / 8; c8 += kExpEpiWarps / 4) {
          uint4 val = make_uint4(0, 0, 0, 0);
          if (vt < ti.rows && c8 * 8 < ti.rank) val = ldg128(vrow + c8 * 8);
          sts128(a_tile + (c8 >> 3) * (kTileM * 128) + vr * 128 + (((c8 & 7) ^ (vr & 7)) << 4), val);
        }
        fence_proxy_async_smem();
        mbar_arrive(a_ready_bar);
      }
      const float scale = apply_scale ? Elem<T>::to_float(scales[ti.adapter]) : 1.f;
      for (int t = 0; t < er.nt_count; ++t, ++it) {
        const int s = it % nst, ab = it & (nacc - 1);
        bool got = mbar_wait(full_bar(s), (it / nst) & 1, &abort_s);
        if (got) got = mbar_wait(tfull_bar(ab), (it / nacc) & 1, &abort_s);
        ok = __all_sync(0xffffffffu, got);
        if (!ok) break;
        tc_fence_after();
        if (warp == kExpEpiWarp0 && lane == 0) trace_stamp(src, it, 2);
        const int n0 = (er.nt_begin + t) * er.tile_n;
        const uint32_t tacc = tmem_base + ((uint32_t)(q * 32) << 16) + ab * acc_cols;
        if (ti.gather) {
          // gathered rows, transposed product: warp (q, j) takes the chains j, j + 2, ... of 128
          // columns; within a chain this lane owns column q * 32 + lane and gets the row values
          // of that column from tensor memory, 16 rows at a time.  Row-major Y tile, tile_n
          // columns wide.
          // Phase 1: out = y0 + scale * acc, rounded once, written back in place.  The
          // accumulator is handed back once this warp's last chunk is in registers.
          const int nhalf = gather_cap(ti.rows) >> 4;
          const int cs = 16 * nhalf;                   // accumulator columns per chain
          const int nchains = er.ncbt >> 1;
          const uint32_t ytile = b_stage(s) + er.yoff;
          const uint32_t ypitch = (uint32_t)er.tile_n * 2u;
          for (int mt = j; mt < nchains; mt += 2) {
            const uint32_t ycol = ytile + (uint32_t)(mt * 128 + q * 32 + lane) * 2u;
            for (int half = 0; half < nhalf; ++half) {
              uint32_t r[16];
              tmem_ld_32x16(tacc + mt * cs + half * 16, r);
              tmem_ld_wait();
              if (mt + 2 >= nchains && half == nhalf - 1) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(ab));
              }
              // four rows at a time, straight-line (a row slot past the tile's last row holds
              // nothing that is stored later): the loads of a group go out together and the
              // four chains of conversions overlap
              const int nh = ti.rows - half * 16;      // rows of this half (the same for every lane)
              uint32_t a = ycol + (uint32_t)(half * 16) * ypitch;
#pragma unroll
              for (int g4 = 0; g4 < 4; ++g4) {
                if (g4 * 4 < nh) {
                  uint32_t yv[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e) yv[e] = lds16(a + (uint32_t)e * ypitch);
#pragma unroll
                  for (int e = 0; e < 4; ++e)
                    sts16(a + (uint32_t)e * ypitch,
                          Elem<T>::float_to_bits(fmaf(scale, __uint_as_float(r[g4 * 4 + e]), Elem<T>::bits_to_float(yv[e]))));
                  a += 4u * ypitch;
                }
              }
            }
          }
          if (j >= nchains) {                          // a warp without a chain in this stage
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(ab));
          }
          __syncwarp();
          // Phase 2: the warp's own 64-byte pieces go out as 16-byte vectors, 8 rows per
          // instruction; a chain's pieces are all read before the first one is stored
          const int my_row = lane >> 2;
          int gi[kGatherRows / 8];
#pragma unroll
          for (int g = 0; g < kGatherRows / 8; ++g) gi[g] = __shfl_sync(0xffffffffu, grow_l, g * 8 + my_row);
          for (int mt = j; mt < nchains; mt += 2) {
            const int colw = mt * 128 + q * 32 + (lane & 3) * 8;
            const bool col_ok = n0 + colw < h_out;
            const uint32_t src0 = ytile + (uint32_t)my_row * ypitch + (uint32_t)colw * 2u;
            uint4 ov[kGatherRows / 8];
#pragma unroll
            for (int g = 0; g < kGatherRows / 8; ++g)
              if (g * 8 < ti.rows) ov[g] = lds128(src0 + (uint32_t)(g * 8) * ypitch);
#pragma unroll
            for (int g = 0; g < kGatherRows / 8; ++g)
              if (g * 8 + my_row < ti.rows && col_ok) stg128(y + (int64_t)gi[g] * h_out + n0 + colw, ov[g]);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(empty_bar(s));
          if (warp == kExpEpiWarp0 && lane == 0) trace_stamp(src, it, 3);
          continue;
        }
        // consecutive rows: this warp's 32 rows x 64 columns = block j of the staged Y tile
        const uint32_t blk = (b_stage(s) + er.yoff) + j * (kTileM * 128);
        if (warp_live) {
          // phase 1: lane = row.  out = y0 + scale * acc, rounded once, written back in place.
          // The block's 64 accumulator columns come in four chunks of 16, each fetched while
          // the previous one is combined with its two Y pieces: 32 accumulator registers live
          // instead of 64 (with 64 the kernel sat on its register cap and spilled).
          const uint32_t rowaddr = blk + row * 128;
          uint32_t ra[16], rb[16];
          auto combine = [&](const uint32_t (&r)[16], int c16) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int c = c16 * 2 + h;
              const uint32_t a = rowaddr + ((c ^ (row & 7)) << 4);
              float f[8];
              unpack8<T>(lds128(a), f);
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = fmaf(scale, __uint_as_float(r[h * 8 + e]), f[e]);
              sts128(a, pack8<T>(f));
            }
          };
          tmem_ld_32x16(tacc + j * 64, ra);
          tmem_ld_wait();
          tmem_ld_32x16(tacc + j * 64 + 16, rb);
          combine(ra, 0);
          tmem_ld_wait();
          tmem_ld_32x16(tacc + j * 64 + 32, ra);
          combine(rb, 1);
          tmem_ld_wait();
          tmem_ld_32x16(tacc + j * 64 + 48, rb);
          combine(ra, 2);
          tmem_ld_wait();
          combine(rb, 3);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(ab));
        // phase 2: 4 rows x 128 bytes per instruction, rows of this segment only.  The stage
        // is handed back as soon as its bytes are in registers; the second half of the global
        // stores (which the SM's store path throttles) drains afterwards.  (Two alternatives
        // measured slower on the mixed step: a tensor store of whole 32-row blocks - the copy
        // engine reads the tile only after the loads queued ahead of it, and the stage cannot
        // be reused before that - and handing phase 2 to one, two or four dedicated store
        // warps, +3 %, with more than 12 warps also costing registers.)
        const int ch = lane & 7;
        const int col = n0 + j * kBoxCols + ch * 8;
        uint4 ov[4];
        if (warp_live) {
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const int rr = q * 32 + p * 4 + (lane >> 3);
            ov[p] = lds128(blk + rr * 128 + ((ch ^ (rr & 7)) << 4));
          }
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const int rr = q * 32 + p * 4 + (lane >> 3);
            if (rr < ti.rows && col < h_out) stg128(y + (int64_t)(ti.row0 + rr) * h_out + col, ov[p]);
          }
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const int rr = q * 32 + (4 + p) * 4 + (lane >> 3);
            ov[p] = lds128(blk + rr * 128 + ((ch ^ (rr & 7)) << 4));
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(s));
        if (warp_live) {
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const int rr = q * 32 + (4 + p) * 4 + (lane >> 3);
            if (rr < ti.rows && col < h_out) stg128(y + (int64_t)(ti.row0 + rr) * h_out + col, ov[p]);
          }
        }
        if (warp == kExpEpiWarp0 && lane == 0) trace_stamp(src, it, 3);
      }
      ++li;
    }
    tc_fence_before();
  } else if (warp == kExpFetchWarp) {
    // ------------------------------------------------------------ work items
    feed_tiles(src, feed, total, true, h_out_, y_, &abort_s);
  }
  __syncthreads();
  if (warp == kExpMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && abort_s) raise_status(src, 1);
}

#include "fused_proj.cuh"

// One CTA, one thread: wait on an mbarrier that nothing ever arrives on, with a budget of
// `budget_cycles`, and report the give-up like the kernels above do.  Exercises the bounded
// wait and the status path without any kernel having to go wrong.
__global__ void bounded_wait_selftest_kernel(long long budget_cycles, int* status, long long* waited) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ volatile int abort_s;
  if (threadIdx.x == 0) {
    abort_s = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_barrier_init();
    const long long t0 = clock64();
    const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_s, budget_cycles);
    if (waited != nullptr) *waited = clock64() - t0;
    if (!ok && abort_s) atomicOr(status != nullptr ? status : &g_status, 1);
  }
}

// ============================================================================
// host side
// ============================================================================
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 2-D row-major [rows, cols] tensor of 2-byte elements, box = box_rows x 64 columns
int make_map_2d(CUtensorMap* map, const void* ptr, int dtype, int64_t rows, int64_t cols,
                int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return VLR_ERR_DRIVER;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBoxCols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype == VLR_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                  2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? VLR_OK : VLR_ERR_DRIVER;
}

// [rows][cols / 64][64] view of a row-major [rows, cols] tensor (cols % 64 == 0), box = one
// row x kblocks consecutive 64-column blocks
static int make_map_row3(CUtensorMap* map, const void* ptr, int dtype, int64_t rows, int64_t cols, int kblocks,
                         int box_rows = 1) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return VLR_ERR_DRIVER;
  cuuint64_t dims[3] = {(cuuint64_t)kBoxCols, (cuuint64_t)(cols / kBoxCols), (cuuint64_t)rows};
  cuuint64_t strides[2] = {(cuuint64_t)kBoxCols * 2, (cuuint64_t)cols * 2};
  cuuint32_t box[3] = {(cuuint32_t)kBoxCols, (cuuint32_t)kblocks, (cuuint32_t)box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dtype == VLR_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                  3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? VLR_OK : VLR_ERR_DRIVER;
}

// [cols / 64][rows][64] view of a row-major [rows, cols] tensor: box = nblocks 64-column blocks x box_rows rows
static int make_map_blocks3(CUtensorMap* map, const void* ptr, int dtype, int64_t rows, int64_t cols, int nblocks,
                            int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return VLR_ERR_DRIVER;
  cuuint64_t dims[3] = {(cuuint64_t)kBoxCols, (cuuint64_t)rows, (cuuint64_t)(cols / kBoxCols)};
  cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)kBoxCols * 2};
  cuuint32_t box[3] = {(cuuint32_t)kBoxCols, (cuuint32_t)box_rows, (cuuint32_t)nblocks};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dtype == VLR_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                  3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? VLR_OK : VLR_ERR_DRIVER;
}

int make_map_set(MapSet* set, const void* act, int64_t act_rows, const void* w, int64_t w_rows,
                 int64_t cols, int dtype, int gather_weight_maps) {
  int rc;
  if (gather_weight_maps == 2 && cols % kBoxCols == 0 &&
      (rc = make_map_blocks3(&set->act3, act, dtype, act_rows, cols, 2, kTileM)) != VLR_OK)
    return rc;
  if (gather_weight_maps == 2 && cols % kBoxCols == 0)
    for (int b = 0; b < 4; ++b)
      for (int i = 0; i < 3; ++i)
        if ((i < 2 || b < 2) &&
            (rc = make_map_blocks3(&set->wb3[b][i], w, dtype, w_rows, cols, 2 << i, 16 << b)) != VLR_OK)
          return rc;
  if (cols % kBoxCols == 0 && cols / kBoxCols >= 8)
    for (int i = 0; i < 3; ++i) {
      if ((rc = make_map_row3(&set->row3[i], act, dtype, act_rows, cols, 2 << i)) != VLR_OK) return rc;
      for (int b = 0; b < 4 && gather_weight_maps == 1; ++b)
        if ((16 << b) * (2 << i) <= 256 &&
            (rc = make_map_row3(&set->w3[i][b], w, dtype, w_rows, cols, 2 << i, 16 << b)) != VLR_OK)
          return rc;
    }
  for (int i = 0; i < 3; ++i)
    if ((rc = make_map_2d(&set->act[i], act, dtype, act_rows, cols, 32 << i)) != VLR_OK) return rc;
  for (int i = 0; i < 4; ++i)
    if ((rc = make_map_2d(&set->w[i], w, dtype, w_rows, cols, 16 << i)) != VLR_OK) return rc;
  return make_map_2d(&set->row, act, dtype, act_rows, cols, 1);
}

// Split the output columns of a tile over several work items when there are too
// few tiles to give every SM a few items.
static int expand_splits(int64_t tiles, int h_out) {
  const int ntiles = (h_out + kExpTileN - 1) / kExpTileN;
  int64_t want = (4 * (int64_t)sm_count() + tiles - 1) / tiles;
  if (want < 1) want = 1;
  if (want > ntiles) want = ntiles;
  return (int)want;
}

#ifdef VLR_TRACE
static long long* g_trace_ptr = nullptr;
static int64_t g_trace_cap = 0;
#endif

// ---- the tile table: launch-level choices per (kind of call, rank bound), measured on the
// part and loaded by the host side (vlr_set_tile_table); the built-in defaults below are what
// the table holds for a B200.  What follows from a tile's own rows and rank (copy box shapes,
// K blocks or column blocks per stage) is derived in the kernels from the stage size.
constexpr int kMaxTileChoices = 16;
static vlr_tile_choice_t g_choices[kMaxTileChoices] = {
    {64, 1, 4, 4, 32, 33}, {128, 1, 3, 3, 32, 33}, {64, 0, 4, 4, 32, 33}, {128, 0, 3, 3, 32, 33}};
static int g_n_choices = 4;

static bool choice_ok(const vlr_tile_choice_t& c) {
  const bool stages_ok = c.shrink_stages >= 2 && c.shrink_stages <= 4 && c.expand_stages >= 3 &&
                         c.expand_stages <= 4;
  // a shrink stage must hold one K block of a full tile at the entry's largest rank, an expand
  // stage two 64-column blocks (weights + Y rows)
  const int pad = (c.max_rank + 15) & ~15;
  const bool fits = kRingBytes / c.shrink_stages >= (kTileM + pad) * 128 &&
                    kRingBytes / c.expand_stages >= 2 * (kTileM + pad) * 128;
  const bool rows_ok = c.small_call_rows == 32 || c.small_call_rows == 64 || c.small_call_rows == 128;
  return c.max_rank >= 8 && c.max_rank <= kMaxRank && (c.step == 0 || c.step == 1) && stages_ok && fits &&
         rows_ok && c.wide_gather_below_rank >= 0 && c.wide_gather_below_rank <= kMaxRank + 1;
}

static const vlr_tile_choice_t* find_choice(int step, int max_rank) {
  const vlr_tile_choice_t* best = nullptr;
  for (int i = 0; i < g_n_choices; ++i) {
    const vlr_tile_choice_t& c = g_choices[i];
    if (c.step == step && c.max_rank >= max_rank && (best == nullptr || c.max_rank < best->max_rank)) best = &c;
  }
  return best;
}

static void size_rings(TileSource& src, int max_rank, bool step, int ring_rank = 0) {
  if (max_rank <= 0 || max_rank > kMaxRank) max_rank = kMaxRank;
  src.max_rank = max_rank;
  if (ring_rank > 0 && ring_rank < max_rank) max_rank = ring_rank;      // what the ring is cut for
  const int pad = (max_rank + 15) & ~15;
  const vlr_tile_choice_t* c = find_choice(step ? 1 : 0, max_rank);
  // without an entry: 48 KB stages while a full tile's two K blocks fit, else 64 KB
  src.shrink_stages = c ? c->shrink_stages : (pad <= 64 ? 4 : 3);
  src.exp_stages = c ? c->expand_stages : (pad <= 64 ? 4 : 3);
  src.shrink_stage_bytes = kRingBytes / src.shrink_stages;
  src.exp_stage_bytes = kRingBytes / src.exp_stages;
  // wide gather stages (expand): the caller says whether adapters of small rank may be in the
  // batch (1: the table's threshold decides per tile, -1: every gather tile), else none
  if (src.wide_below_rank == -1) src.wide_below_rank = kMaxRank + 1;
  else if (src.wide_below_rank == 1) src.wide_below_rank = c ? c->wide_gather_below_rank : 33;
  else src.wide_below_rank = 0;
}

static int small_call_rows(int max_rank) {
  const vlr_tile_choice_t* c = find_choice(0, max_rank);
  return c ? c->small_call_rows : 32;
}

template <typename T>
static int launch_atmm(void* y, const void* x, const void* w, const void* scales, TileSource src,
                       int64_t max_tiles, int64_t T_rows, int h_in, int h_out, int64_t w_cells,
                       int dtype, int flags, cudaStream_t stream, int n_problems) {
  // the shared-memory opt-in is per device: one flag per device this process has launched on
  static bool attr_done_dev[64];
  int cur_dev = 0;
  if (cudaGetDevice(&cur_dev) != cudaSuccess || cur_dev < 0 || cur_dev >= 64) return VLR_ERR_RANGE;
  bool& attr_done = attr_done_dev[cur_dev];
  if (!attr_done) {
    cudaError_t e = cudaSuccess;
    auto set = [&](const void* f, int bytes) {
      cudaError_t r = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
      if (e == cudaSuccess) e = r;
    };
    set((const void*)atmm_shrink_kernel<__half, 2>, kShrinkSmem);
    set((const void*)atmm_shrink_kernel<__nv_bfloat16, 2>, kShrinkSmem);
    set((const void*)atmm_shrink_kernel<__half, 3>, kShrinkSmem);
    set((const void*)atmm_shrink_kernel<__half, 4>, kShrinkSmem);
    set((const void*)atmm_shrink_kernel<__nv_bfloat16, 3>, kShrinkSmem);
    set((const void*)atmm_shrink_kernel<__nv_bfloat16, 4>, kShrinkSmem);
    set((const void*)atmm_expand_kernel<__half, 3, false>, kExpSmem);
    set((const void*)atmm_expand_kernel<__half, 3, true>, kExpSmem);
    set((const void*)atmm_expand_kernel<__half, 4, false>, kExpSmem);
    set((const void*)atmm_expand_kernel<__half, 4, true>, kExpSmem);
    set((const void*)atmm_expand_kernel<__nv_bfloat16, 3, false>, kExpSmem);
    set((const void*)atmm_expand_kernel<__nv_bfloat16, 3, true>, kExpSmem);
    set((const void*)atmm_expand_kernel<__nv_bfloat16, 4, false>, kExpSmem);
    set((const void*)atmm_expand_kernel<__nv_bfloat16, 4, true>, kExpSmem);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return (int)e;
    }
    attr_done = true;
  }
  if (max_tiles <= 0 || n_problems <= 0) return VLR_OK;
  // In step mode (src.plan set) the tensor maps come from the plan in device
  // memory, h_in / h_out are maxima over its problems and only size the grid.
  MapSet maps;
  memset(&maps, 0, sizeof(maps));
#ifdef VLR_TRACE
  src.trace = g_trace_ptr;
  src.trace_cap = g_trace_cap;
#endif
  const bool step = src.plan != nullptr;
  // rank bound: the caller's hint in a step, the width of the rank-side buffer otherwise
  size_rings(src, step ? src.max_rank : (h_in >= h_out ? h_out : h_in), step, step ? src.ring_rank : 0);
  int rc;
  if (h_in >= h_out) {
    if (!step && (rc = make_map_set(&maps, x, T_rows, w, w_cells, h_in, dtype)) != VLR_OK) return rc;
    src.max_tiles = max_tiles;
    src.n_problems = n_problems;
    src.nsplit = 1;
    const int64_t items = max_tiles * n_problems;
    const unsigned grid = (unsigned)(items < sm_count() ? items : sm_count());
    const int acc = (flags & VLR_ATMM_ACCUMULATE_SHRINK) ? 1 : 0;
    if (src.shrink_stages == 4)
      atmm_shrink_kernel<T, 4><<<grid, kThreads, kShrinkSmem, stream>>>(maps, (T*)y, (const T*)x, src,
                                                                        h_in, h_out, acc);
    else if (src.shrink_stages == 3)
      atmm_shrink_kernel<T, 3><<<grid, kThreads, kShrinkSmem, stream>>>(maps, (T*)y, (const T*)x, src,
                                                                        h_in, h_out, acc);
    else
      atmm_shrink_kernel<T, 2><<<grid, kThreads, kShrinkSmem, stream>>>(maps, (T*)y, (const T*)x, src,
                                                                        h_in, h_out, acc);
  } else {
    if (!step && (rc = make_map_set(&maps, y, T_rows, w, w_cells, h_out, dtype)) != VLR_OK) return rc;
    src.max_tiles = max_tiles;
    src.n_problems = n_problems;
    // in step mode the tile count lives on the device; with many problems no split is needed
    src.nsplit = step ? (n_problems >= 8 ? 1 : expand_splits((max_tiles / 8 + 1) * n_problems, h_out))
                      : expand_splits(max_tiles, h_out);
    const int64_t items = max_tiles * n_problems * src.nsplit;
    const unsigned grid = (unsigned)(items < sm_count() ? items : sm_count());
    const int sc = (flags & VLR_ATMM_APPLY_SCALE) ? 1 : 0;
#define VLR_EXPAND_LAUNCH(NST, WIDE)                                                  \
  atmm_expand_kernel<T, NST, WIDE><<<grid, kExpThreads, kExpSmem, stream>>>(           \
      maps, (T*)y, (const T*)x, (const T*)scales, src, h_out, h_in, sc)
    const bool wide = src.wide_below_rank > 0;         // some tile of this launch may take the wide form
    if (src.exp_stages == 4) {
      if (wide) VLR_EXPAND_LAUNCH(4, true); else VLR_EXPAND_LAUNCH(4, false);
    } else {
      if (wide) VLR_EXPAND_LAUNCH(3, true); else VLR_EXPAND_LAUNCH(3, false);
    }
#undef VLR_EXPAND_LAUNCH
  }
  return launch_status();
}

int atmm_launch(void* y, const void* x, const void* w, const void* scales, const TileSource& src,
                int64_t max_tiles, int64_t T_rows, int h_in, int h_out, int64_t w_cells, int dtype,
                int flags, cudaStream_t stream, int n_problems) {
  if (dtype == VLR_F16)
    return launch_atmm<__half>(y, x, w, scales, src, max_tiles, T_rows, h_in, h_out, w_cells, dtype, flags, stream, n_problems);
  return launch_atmm<__nv_bfloat16>(y, x, w, scales, src, max_tiles, T_rows, h_in, h_out, w_cells, dtype, flags, stream, n_problems);
}

}  // namespace vlr

extern "C" int vlr_atmm(void* y, const void* x, const void* w, const int64_t* a_start,
                        const int64_t* a_len, const int64_t* a_loc, const int64_t* indicies,
                        int64_t qkvo, const void* lora_scales, const int64_t* output_counts,
                        const int64_t* rank_counts, const int64_t* lora_ids,
                        const int64_t* start_ids, void* tmp, int64_t tmp_bytes,
                        int64_t num_problems, int64_t T, int64_t h_in, int64_t h_out,
                        int64_t w_cells, int dtype, int flags, void* stream) {
  using namespace vlr;
  (void)a_len; (void)indicies; (void)tmp; (void)tmp_bytes;
  if (num_problems == 0 || T == 0) return VLR_OK;
  if (!y || !x || !w || !a_start || !a_loc || !output_counts || !rank_counts || !lora_ids || !start_ids)
    return VLR_ERR_NULL;
  if (dtype != VLR_F16 && dtype != VLR_BF16) return VLR_ERR_DTYPE;
  if (num_problems < 0 || T < 0 || T > 0x7fffffff || qkvo < 0 || w_cells <= 0) return VLR_ERR_RANGE;
  if (h_in <= 0 || h_out <= 0 || h_in >= 65536 || h_out >= 65536) return VLR_ERR_SHAPE;
  const bool expand = h_in < h_out;
  const int64_t narrow = expand ? h_in : h_out, wide = expand ? h_out : h_in;
  if (wide % 8 != 0 || narrow % 8 != 0 || narrow > kMaxRank) return VLR_ERR_SHAPE;
  if ((flags & VLR_ATMM_APPLY_SCALE) && !lora_scales) return VLR_ERR_NULL;
  if (!aligned16(x) || !aligned16(y) || !aligned16(w)) return VLR_ERR_ALIGN;
  TileSource src{};
  src.output_counts = output_counts;
  src.rank_counts = rank_counts;
  src.lora_ids = lora_ids;
  src.start_ids = start_ids;
  src.num_problems = num_problems;
  src.a_start = a_start;
  src.a_loc = a_loc;
  src.slot = qkvo;
  src.mode = 0;
  if (!expand && (flags & VLR_ATMM_APPLY_SCALE)) src.shrink_scales = lora_scales;
  // every problem with m rows has ceil(m / tile rows) tiles; sum <= T / tile rows + num_problems.
  // A shrink with few rows is a few CTAs each walking all of K at the latency of a stage; cut
  // into 32-row tiles it occupies four times as many SMs, and a stage holds several K blocks.
  src.tile_rows = kTileM;
  if (!expand && !(flags & VLR_ATMM_FULL_TILES) && T / kTileM + num_problems <= sm_count() / 2)
    src.tile_rows = small_call_rows((int)narrow);
  const int64_t max_tiles = T / src.tile_rows + num_problems;
  return atmm_launch(y, x, w, lora_scales, src, max_tiles, T, (int)h_in, (int)h_out, w_cells, dtype,
                     flags, (cudaStream_t)stream, 1);
}

extern "C" int vlr_device_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, vlr::g_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v) {
    int z = 0;
    cudaMemcpyToSymbol(vlr::g_status, &z, sizeof(int));
  }
  const int d = vlr::bgmv_decode_status(reset);
  if (d < 0) return -1;
  return v | d;
}

extern "C" int vlr_fused_proj(void* y, const void* x, const void* w_base, const void* v, int64_t v_pitch,
                              const void* wb_pool, int64_t cells_b, const int64_t* a_start_b,
                              const int64_t* a_loc_b, int64_t slot_b, const int32_t* tiles,
                              const int32_t* counts, int64_t max_mma_tiles, int64_t T, int64_t h_in,
                              int64_t h_out, int dtype, int32_t* dev_status, void* stream) {
  using namespace vlr;
  if (T == 0) return VLR_OK;
  if (!y || !x || !w_base || !v || !wb_pool || !a_start_b || !a_loc_b || !tiles || !counts) return VLR_ERR_NULL;
  if (dtype != VLR_F16 && dtype != VLR_BF16) return VLR_ERR_DTYPE;
  if (T < 0 || T > 0x7fffffff || cells_b <= 0 || slot_b < 0) return VLR_ERR_RANGE;
  if (h_in < 64 || h_out < 64 || h_in >= 65536 || h_out >= 65536 || (h_in & 63) || (h_out & 63)) return VLR_ERR_SHAPE;
  if (v_pitch < 8 || v_pitch > kMaxRank || (v_pitch & 7)) return VLR_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(y) || !aligned16(w_base) || !aligned16(v) || !aligned16(wb_pool)) return VLR_ERR_ALIGN;
  static bool attr_done_dev[64];
  int cur_dev = 0;
  if (cudaGetDevice(&cur_dev) != cudaSuccess || cur_dev < 0 || cur_dev >= 64) return VLR_ERR_RANGE;
  if (!attr_done_dev[cur_dev]) {
    cudaError_t e = cudaFuncSetAttribute((const void*)fused_proj_kernel<__half>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kFpSmem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute((const void*)fused_proj_kernel<__nv_bfloat16>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, kFpSmem);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return (int)e;
    }
    attr_done_dev[cur_dev] = true;
  }
  if (max_mma_tiles <= 0 || max_mma_tiles > T) max_mma_tiles = T;
  FusedArgs fa;
  memset(&fa, 0, sizeof(fa));
  fa.v = v;
  fa.v_pitch = (int)v_pitch;
  fa.h_in = (int)h_in;
  fa.h_out = (int)h_out;
  int rc;
  for (int i = 0; i < 3; ++i)                          // X [T, h_in]: boxes of 32 / 64 / 128 rows
    if ((rc = make_map_2d(&fa.xw.act[i], x, dtype, T, h_in, 32 << i)) != VLR_OK) return rc;
  // W [h_in, h_out]: boxes of 64 rows (K) x 64 columns (N)
  if ((rc = make_map_2d(&fa.xw.w[2], w_base, dtype, h_in, h_out, 64)) != VLR_OK) return rc;
  for (int i = 0; i < 4; ++i)                          // B-side pool [cells, h_out]: 16 .. 128 rows
    if ((rc = make_map_2d(&fa.yb.w[i], wb_pool, dtype, cells_b, h_out, 16 << i)) != VLR_OK) return rc;
  TileSource src{};
  src.mode = 1;
  src.tiles = tiles;
  src.counts = counts;
  src.gather_mma = 0;                                  // consecutive-row tiles only
  src.a_start = a_start_b;
  src.a_loc = a_loc_b;
  src.slot = slot_b;
  src.status = dev_status;
  src.max_rank = kMaxRank;
  src.n_problems = 1;
  src.nsplit = (int)((h_out + kFpTileN - 1) / kFpTileN);
  src.max_tiles = max_mma_tiles;
  const int64_t items = max_mma_tiles * src.nsplit;
  const unsigned grid = (unsigned)(items < sm_count() ? items : sm_count());
  if (dtype == VLR_F16)
    fused_proj_kernel<__half><<<grid, kExpThreads, kFpSmem, (cudaStream_t)stream>>>(fa, (__half*)y, src);
  else
    fused_proj_kernel<__nv_bfloat16><<<grid, kExpThreads, kFpSmem, (cudaStream_t)stream>>>(fa, (__nv_bfloat16*)y, src);
  return launch_status();
}

extern "C" int vlr_set_tile_table(const vlr_tile_choice_t* entries, int n) {
  if (n < 0 || n > vlr::kMaxTileChoices) return VLR_ERR_RANGE;
  if (n > 0 && !entries) return VLR_ERR_NULL;
  for (int i = 0; i < n; ++i)
    if (!vlr::choice_ok(entries[i])) return VLR_ERR_RANGE;
  for (int i = 0; i < n; ++i) vlr::g_choices[i] = entries[i];
  vlr::g_n_choices = n;
  return VLR_OK;
}

extern "C" int vlr_get_tile_choice(int step, int max_rank, vlr_tile_choice_t* out) {
  if (!out) return VLR_ERR_NULL;
  if (max_rank <= 0 || max_rank > vlr::kMaxRank) max_rank = vlr::kMaxRank;
  vlr::TileSource src{};
  vlr::size_rings(src, max_rank, step != 0);
  const vlr_tile_choice_t* c = vlr::find_choice(step ? 1 : 0, max_rank);
  out->max_rank = c ? c->max_rank : max_rank;
  out->step = step ? 1 : 0;
  out->shrink_stages = src.shrink_stages;
  out->expand_stages = src.exp_stages;
  out->small_call_rows = c ? c->small_call_rows : 32;
  out->wide_gather_below_rank = c ? c->wide_gather_below_rank : 33;
  return VLR_OK;
}

extern "C" int vlr_selftest_bounded_wait(int64_t budget_cycles, int32_t* dev_status,
                                         int64_t* dev_waited_cycles, void* stream) {
  if (budget_cycles <= 0 || budget_cycles > 2000000000LL) return VLR_ERR_RANGE;
  vlr::bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(
      (long long)budget_cycles, dev_status, reinterpret_cast<long long*>(dev_waited_cycles));
  return vlr::launch_status();
}

#ifdef VLR_TRACE
// Debug builds (-DVLR_TRACE) only: while a device buffer is set, CTA 0 of the tensor-core
// kernels writes clock64 stamps into it (8 int64 per pipeline stage: stage issued, operands
// seen by the MMA thread, MMAs issued / epilogue started, stage released).
extern "C" int vlr_debug_set_trace(void* dev_buffer, int64_t n_int64) {
  vlr::g_trace_ptr = reinterpret_cast<long long*>(dev_buffer);
  vlr::g_trace_cap = dev_buffer ? n_int64 : 0;
  vlr::bgmv_decode_set_trace(vlr::g_trace_ptr, vlr::g_trace_cap);
  return VLR_OK;
}
#endif
