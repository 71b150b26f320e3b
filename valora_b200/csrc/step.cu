// One step over many LoRA projections: the step plan (per-problem tensor maps
// and pointers in device memory) and the batched launches that run the shrink
// and the expand of every problem of a packed batch.
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "problem.cuh"

using namespace vlr;

namespace {
// A second stream per device for the steps that run their kernels once per rank class, with
// the two events that fork it from and join it to the caller's stream.  Created on first use.
struct SideStream {
  cudaStream_t stream;
  cudaEvent_t fork, join;
  std::mutex pair;      // a record and the wait on it are one step for concurrent callers: the wait
                        // takes the event's latest record
};
SideStream* side_stream() {
  constexpr int kMaxDev = 64;
  static std::mutex mu;
  static SideStream slots[kMaxDev];
  static bool made[kMaxDev];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!made[dev]) {
    SideStream& ss = slots[dev];
    if (cudaStreamCreateWithFlags(&ss.stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&ss.fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&ss.join, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    made[dev] = true;
  }
  return &slots[dev];
}

// The step's tiles in two classes: list2 gets the indices of the consecutive-row tiles of rank >
// split_rank, list1 those of every other tile (consecutive rows up to that rank, and gather tiles
// of any rank: their stages fit the deeper ring's 48 KB at every rank), each in the order of
// `tiles`; the two counts in cls_count[0] and cls_count[16] (64 bytes apart).  One CTA; n is a
// few thousand at most.
__global__ void __launch_bounds__(1024)
classify_tiles_kernel(const int32_t* __restrict__ tiles, const int32_t* __restrict__ counts, int gather_mma,
                      int split_rank, int cap, int32_t* cls_count, int32_t* list1, int32_t* list2) {
  __shared__ int w1[32], w2[32];
  __shared__ int base1_s, base2_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int n = counts[VLR_COUNT_MMA_TILES] + (gather_mma ? counts[VLR_COUNT_GATHER_TILES] : 0);
  n = n < cap ? n : cap;
  if (tid == 0) { base1_s = 0; base2_s = 0; }
  __syncthreads();
  for (int b0 = 0; b0 < n; b0 += 1024) {
    const int b = b0 + tid;
    const bool in = b < n;
    const bool c2 = in && tiles[(int64_t)b * VLR_TILE_INTS] == VLR_TILE_MMA &&
                    tiles[(int64_t)b * VLR_TILE_INTS + 2] > split_rank;
    const bool c1 = in && !c2;
    const unsigned m1 = __ballot_sync(0xffffffffu, c1), m2 = __ballot_sync(0xffffffffu, c2);
    if (lane == 0) { w1[warp] = __popc(m1); w2[warp] = __popc(m2); }
    __syncthreads();
    int o1 = base1_s, o2 = base2_s;                   // offsets of this warp: the warps before it
    for (int w = 0; w < warp; ++w) { o1 += w1[w]; o2 += w2[w]; }
    const unsigned below = (1u << lane) - 1u;
    if (c1) list1[o1 + __popc(m1 & below)] = b;
    if (c2) list2[o2 + __popc(m2 & below)] = b;
    __syncthreads();
    if (tid == 0) {
      int t1 = 0, t2 = 0;
      for (int w = 0; w < 32; ++w) { t1 += w1[w]; t2 += w2[w]; }
      base1_s += t1;
      base2_s += t2;
    }
    __syncthreads();
  }
  if (tid == 0) { cls_count[0] = base1_s; cls_count[16] = base2_s; }
}
}  // namespace

extern "C" size_t vlr_step_plan_bytes(int n_problems) {
  return n_problems > 0 ? (size_t)n_problems * sizeof(StepProblem) : 0;
}

extern "C" int vlr_step_plan_build(const vlr_problem_t* problems, int n_problems, int64_t max_rows,
                                   int dtype, void* plan_host) {
  if (!problems || !plan_host) return VLR_ERR_NULL;
  if (n_problems <= 0 || n_problems > 65535 || max_rows <= 0 || max_rows > 0x7fffffff) return VLR_ERR_RANGE;
  if (dtype != VLR_F16 && dtype != VLR_BF16) return VLR_ERR_DTYPE;
  StepProblem* out = reinterpret_cast<StepProblem*>(plan_host);
  for (int i = 0; i < n_problems; ++i) {
    const vlr_problem_t& p = problems[i];
    if (!p.x || !p.y || !p.wa || !p.wb || !p.a_start_a || !p.a_loc_a || !p.a_start_b || !p.a_loc_b)
      return VLR_ERR_NULL;
    // 64-column (128-byte) granularity: gathered rows are fetched in 128-byte pieces
    if (p.h_in <= 0 || p.h_out <= 0 || p.h_in >= 65536 || p.h_out >= 65536 || (p.h_in & 63) ||
        (p.h_out & 63))
      return VLR_ERR_SHAPE;
    if (p.cells_a <= 0 || p.cells_b <= 0 || p.slot_a < 0 || p.slot_b < 0) return VLR_ERR_RANGE;
    if (!aligned16(p.x) || !aligned16(p.y) || !aligned16(p.wa) || !aligned16(p.wb)) return VLR_ERR_ALIGN;
    StepProblem sp;
    memset(&sp, 0, sizeof(sp));
    int rc;
    if ((rc = make_map_set(&sp.shrink, p.x, max_rows, p.wa, p.cells_a, p.h_in, dtype, 1)) != VLR_OK) return rc;
    if ((rc = make_map_set(&sp.expand, p.y, max_rows, p.wb, p.cells_b, p.h_out, dtype, 2)) != VLR_OK) return rc;
    sp.x = p.x; sp.y = p.y; sp.wa = p.wa; sp.wb = p.wb;
    sp.a_start_a = p.a_start_a; sp.a_loc_a = p.a_loc_a;
    sp.a_start_b = p.a_start_b; sp.a_loc_b = p.a_loc_b;
    sp.h_in = p.h_in; sp.h_out = p.h_out; sp.slot_a = p.slot_a; sp.slot_b = p.slot_b;
    sp.layout_b = VLR_LAYOUT_ROWS;
    memcpy(&out[i], &sp, sizeof(sp));
  }
  return VLR_OK;
}

extern "C" size_t vlr_lora_step_workspace_bytes(int64_t T, int n_problems) {
  if (T <= 0 || n_problems <= 0) return 256;
  // V buffers, alignment, work-item counters; the two rank classes' counts and tile lists (2 T entries each)
  return (size_t)n_problems * (size_t)T * kMaxRank * 2 + 256 + 512 + 256 + (size_t)T * 16;
}

extern "C" int vlr_lora_step(const void* plan_dev, int n_problems, int64_t T, const int32_t* tiles,
                             const int32_t* gather_rows, int64_t max_mma_tiles,
                             int64_t max_gather_tiles, const int32_t* counts, const void* scales,
                             int max_h_in, int max_h_out, int max_rank, int dtype, int phase_mask,
                             void* workspace, size_t workspace_bytes, int32_t* dev_status, void* stream) {
  if (T == 0 || n_problems == 0) return VLR_OK;
  if (!plan_dev || !tiles || !gather_rows || !counts || !scales || !workspace) return VLR_ERR_NULL;
  if (dtype != VLR_F16 && dtype != VLR_BF16) return VLR_ERR_DTYPE;
  if (T < 0 || T > 0x7fffffff || n_problems < 0 || n_problems > 65535) return VLR_ERR_RANGE;
  if (max_h_in <= 0 || max_h_out <= 0 || max_h_in >= 65536 || max_h_out >= 65536) return VLR_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(plan_dev) & 127u) != 0) return VLR_ERR_ALIGN;
  char* vb = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(workspace) + 255u) & ~uintptr_t(255));
  const size_t need = (size_t)n_problems * (size_t)T * kMaxRank * 2;
  // + four work-item counters, 64 bytes apart; + class counts and the two class lists
  const size_t need_all = ((need + 255) & ~size_t(255)) + 256 + 256 + (size_t)T * 16;
  if ((size_t)(vb - reinterpret_cast<char*>(workspace)) + need_all > workspace_bytes) return VLR_ERR_WORKSPACE;
  unsigned int* counters = reinterpret_cast<unsigned int*>(vb + ((need + 255) & ~size_t(255)));
  int32_t* cls_count = reinterpret_cast<int32_t*>(counters + 64);
  int32_t* cls_list1 = cls_count + 64;
  int32_t* cls_list2 = cls_list1 + 2 * T;
  // every tile holds at least one row
  if (max_mma_tiles <= 0 || max_mma_tiles > T) max_mma_tiles = T;
  if (max_gather_tiles <= 0 || max_gather_tiles > T) max_gather_tiles = T;
  cudaStream_t s = (cudaStream_t)stream;
  const StepProblem* plan = reinterpret_cast<const StepProblem*>(plan_dev);

  TileSource src{};
  src.mode = 1;
  src.tiles = tiles;
  src.counts = counts;
  src.plan = plan;
  src.vbuf = vb;
  src.vstride = T * kMaxRank;
  src.gather_rows = gather_rows;
  src.status = dev_status;
  src.max_rank = (max_rank > 0 && max_rank <= kMaxRank) ? max_rank : kMaxRank;
  src.gather_mma = (phase_mask & VLR_STEP_GATHER_ON_TENSOR_CORES) ? 1 : 0;
  src.wide_below_rank = !(phase_mask & VLR_STEP_WIDE_GATHER_STAGES) ? 0
                        : (phase_mask & VLR_STEP_ALL_WIDE_GATHER_STAGES) ? -1 : 1;
  if (src.gather_mma) {
    // gather tiles are work items of the two tensor-core launches
    max_mma_tiles = T;
    phase_mask &= ~(VLR_PHASE_SHRINK_GATHER | VLR_PHASE_EXPAND_GATHER);
  }
  BgmvGroups g{};
  g.tiles = tiles;
  g.gather_rows = gather_rows;
  g.counts = counts;
  g.plan = plan;
  g.vbuf = vb;
  g.vstride = T * kMaxRank;

  int rc = VLR_OK;
  // the tensor-core kernels draw their work items from these (tiles differ a lot in size)
  cudaError_t ce = cudaMemsetAsync(counters, 0, 256, s);
  if (ce != cudaSuccess) return (int)ce;
  // The launchers pick the direction from h_in >= h_out, and in step mode use the two
  // widths only to size grids (every problem brings its own).  Plans whose widest
  // projection is narrower than the rank buffer must still go the right way.
  const int shrink_h_in = (int)max_h_in > kMaxRank ? (int)max_h_in : kMaxRank;
  const int expand_h_out = (int)max_h_out > kMaxRank ? (int)max_h_out : kMaxRank + 8;
  // With adapters above rank 64 resident, a kernel runs once per class of tiles: consecutive-row
  // tiles above rank 64 need the three-stage ring (64 KB stages); every other tile - consecutive
  // rows up to rank 64, gather tiles of any rank - runs on the four-stage ring, on which they are
  // 18-34 % faster.  A row belongs to one tile, so shrink and expand of one class read and write
  // nothing of the other: the second class runs on a side stream, its CTAs moving onto the SMs as the first class's kernels
  // run out of tiles (one tail per step instead of one per launch - with two tails config 2's
  // large prefill tiles lost more than the deeper ring gained).
  const bool split = (phase_mask & VLR_STEP_SPLIT_RANK_CLASSES) && src.max_rank > 64 &&
                     (phase_mask & (VLR_PHASE_SHRINK_MMA | VLR_PHASE_EXPAND_MMA));
  auto run = [&](bool expand, int cls, cudaStream_t st) -> int {
    const int h_in = expand ? kMaxRank : shrink_h_in, h_out = expand ? expand_h_out : kMaxRank;
    const int flags = expand ? VLR_ATMM_APPLY_SCALE : 0;
    TileSource a = src;
    a.item_counter = counters + (expand ? 32 : 0) + (cls == 2 ? 16 : 0);
    if (cls == 1) {                                    // consecutive rows up to rank 64, gather tiles of any rank
      a.ring_rank = 64;
      a.class_list = cls_list1;
      a.class_count = cls_count;
    } else if (cls == 2) {                             // consecutive rows above rank 64
      a.class_list = cls_list2;
      a.class_count = cls_count + 16;
      a.wide_below_rank = 0;                           // wide stages are for small ranks
    }
    return atmm_launch(nullptr, nullptr, nullptr, scales, a, max_mma_tiles, T, h_in, h_out, 0, dtype, flags, st, n_problems);
  };
  SideStream* side = nullptr;
  if (split) {
    side = side_stream();
    if (side == nullptr) return VLR_ERR_DRIVER;
    // which tiles belong to which class (a rank the kernels do not support lands in one of the two
    // and is reported by that launch)
    classify_tiles_kernel<<<1, 1024, 0, s>>>(tiles, counts, src.gather_mma, 64, (int)(2 * T), cls_count, cls_list1, cls_list2);
    if ((rc = launch_status()) != VLR_OK) return rc;
    {
      std::lock_guard<std::mutex> lock(side->pair);
      if ((ce = cudaEventRecord(side->fork, s)) != cudaSuccess) return (int)ce;
      if ((ce = cudaStreamWaitEvent(side->stream, side->fork, 0)) != cudaSuccess) return (int)ce;
    }
    if (phase_mask & VLR_PHASE_SHRINK_MMA) rc = run(false, 2, side->stream);
    if (rc == VLR_OK && (phase_mask & VLR_PHASE_EXPAND_MMA)) rc = run(true, 2, side->stream);
  }
  auto join = [&]() -> int {                           // in any case: a capture or the caller's stream is never left forked
    if (side == nullptr) return VLR_OK;
    std::lock_guard<std::mutex> lock(side->pair);
    cudaError_t je = cudaEventRecord(side->join, side->stream);
    if (je == cudaSuccess) je = cudaStreamWaitEvent(s, side->join, 0);
    return je == cudaSuccess ? VLR_OK : (int)je;
  };
  if (rc != VLR_OK) {
    join();
    return rc;
  }
  const int cls = split ? 1 : 0;
  // shrink
  if (phase_mask & VLR_PHASE_SHRINK_MMA) rc = run(false, cls, s);
  if (rc == VLR_OK && (phase_mask & VLR_PHASE_SHRINK_GATHER))
    rc = bgmv_gather_launch(nullptr, nullptr, nullptr, scales, g, max_gather_tiles, shrink_h_in,
                            kMaxRank, VLR_LAYOUT_ROWS, dtype, s, n_problems);
  // expand
  if (rc == VLR_OK && (phase_mask & VLR_PHASE_EXPAND_MMA)) rc = run(true, cls, s);
  const int jrc = join();
  if (rc != VLR_OK) return rc;
  if (jrc != VLR_OK) return jrc;
  if (phase_mask & VLR_PHASE_EXPAND_GATHER)
    rc = bgmv_gather_launch(nullptr, nullptr, nullptr, scales, g, max_gather_tiles, kMaxRank,
                            expand_h_out, VLR_LAYOUT_ROWS, dtype, s, n_problems);
  return rc;
}
