// Ragged grouped LoRA shrink (V = X A) and expand (Y += s V B) on the sm_100a
// tensor cores: tcgen05.mma with accumulators in tensor memory, operands staged
// in shared memory by tiled bulk tensor copies (TMA) behind an mbarrier ring.
//
// One CTA = one tile of up to 128 consecutive rows of one segment.
//   warp 0      TMA producer (one lane)
//   warp 1      tensor-memory allocation, MMA issue (one lane)
//   warps 2..5  epilogue, one TMEM lane quarter each
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
constexpr int kThreads = 192;
constexpr int kBoxRowsAct = 32;      // activation rows per TMA box
constexpr int kBoxRowsW = 16;        // weight rows per TMA box
constexpr int kBoxCols = 64;         // 64 two-byte elements = 128 bytes = swizzle span

struct TileInfo {
  int valid;
  int row0;          // first row of the tile in x / y
  int rows;          // rows of the segment in this tile (1..128)
  int rank;          // true rank
  int adapter;
  int problem;       // index into the step plan (0 outside step mode)
  int split;         // expand: which share of the output columns
  int64_t wrow0;     // first pool cell of the slot
};

// Item -> tile.  Warp-collective: all 32 lanes call it and all get the result.
// mode 1: item = (problem * n_tiles + tile) * nsplit + split, n_tiles on the device.
// mode 0: item = tile * nsplit + split over the reference's problem table; tiles
//         beyond the table's last one come back invalid.
__device__ __forceinline__ TileInfo get_tile(const TileSource& src, int64_t item, bool expand) {
  const int lane = threadIdx.x & 31;
  TileInfo ti;
  ti.valid = 0;
  ti.problem = 0;
  ti.split = (int)(item % src.nsplit);
  const int64_t tb = item / src.nsplit;
  if (src.mode == 1) {
    const int n_tiles = src.counts[VLR_COUNT_MMA_TILES];
    const int b = (int)(tb % n_tiles);
    ti.problem = (int)(tb / n_tiles);
    const int32_t* t = src.tiles + (int64_t)b * VLR_TILE_INTS;
    ti.valid = 1;
    ti.adapter = t[1];
    ti.rank = t[2];
    ti.row0 = t[3];
    ti.rows = t[4];
  } else {
    const int b = (int)tb;
    int base = 0;
    for (int64_t p0 = 0; p0 < src.num_problems; p0 += 32) {
      const int64_t p = p0 + lane;
      const int m = p < src.num_problems ? (int)src.output_counts[p] : 0;
      const int nt = m > 0 ? (m + kTileM - 1) / kTileM : 0;
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
        const int m0 = (b - __shfl_sync(0xffffffffu, excl, srcl)) * kTileM;
        const int64_t pp = p0 + srcl;
        ti.valid = 1;
        ti.adapter = (int)src.lora_ids[pp];
        ti.rank = (int)src.rank_counts[pp];
        ti.row0 = (int)src.start_ids[pp] + m0;
        ti.rows = min(kTileM, (int)src.output_counts[pp] - m0);
        break;
      }
      base += __shfl_sync(0xffffffffu, inc, 31);
    }
  }
  if (ti.valid) {
    if (ti.rank <= 0 || ti.rank > kMaxRank || (ti.rank & 7) || ti.rows <= 0 || ti.rows > kTileM) {
      ti.valid = 0;                  // host validated what it could; skip bad entries
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
  if (src.mode == 1)
    return (int64_t)src.counts[VLR_COUNT_MMA_TILES] * src.n_problems * src.nsplit;
  return src.max_tiles * src.nsplit;
}

__device__ int g_status;             // 0 ok, 1 a bounded wait gave up

// ============================================================================
// shrink: persistent CTAs, 6-stage TMA ring over K, two accumulators in tensor
// memory so the epilogue of one tile overlaps the main loop of the next.
// ============================================================================
constexpr int kShrinkStages = 6;
constexpr int kShrinkXBytes = kTileM * 128;            // 16 KB
constexpr int kShrinkWBytes = kMaxRank * 128;          // 16 KB
constexpr int kShrinkStageBytes = kShrinkXBytes + kShrinkWBytes;
constexpr int kShrinkSmem = 1024 + kShrinkStages * kShrinkStageBytes + 256;

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
atmm_shrink_kernel(const __grid_constant__ CUtensorMap map_x_, const __grid_constant__ CUtensorMap map_w_,
                   T* __restrict__ v_, TileSource src, int h_in_, int v_pitch_, int accumulate) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ volatile int abort_s;
  __shared__ uint32_t tmem_base_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t total = total_items(src);
  if ((int64_t)blockIdx.x >= total) return;            // nothing for this CTA: no TMEM taken

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + kShrinkStages * kShrinkStageBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kShrinkStages + s); };
  auto tfull_bar = [&](int ab) { return bars + 8u * (2 * kShrinkStages + ab); };
  auto tempty_bar = [&](int ab) { return bars + 8u * (2 * kShrinkStages + 2 + ab); };
  auto x_stage = [&](int s) { return base + (uint32_t)s * kShrinkStageBytes; };
  auto w_stage = [&](int s) { return base + (uint32_t)s * kShrinkStageBytes + kShrinkXBytes; };

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < kShrinkStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int ab = 0; ab < 2; ++ab) {
      mbar_init(tfull_bar(ab), 1);
      mbar_init(tempty_bar(ab), 4);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  // per-item problem view
  auto h_in_of = [&](const TileInfo& ti) { return src.plan ? src.plan[ti.problem].h_in : h_in_; };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    uint32_t kiter = 0;
    bool ok = true;
    for (int64_t item = blockIdx.x; item < total && ok; item += gridDim.x) {
      const TileInfo ti = get_tile(src, item, false);
      if (!ti.valid) continue;
      if (lane == 0) {
        const CUtensorMap* pmap_x = src.plan ? &src.plan[ti.problem].map_x : &map_x_;
        const CUtensorMap* pmap_w = src.plan ? &src.plan[ti.problem].map_wa : &map_w_;
        const int n_pad = (ti.rank + 15) & ~15;
        const int nbox_x = (ti.rows + kBoxRowsAct - 1) / kBoxRowsAct;
        const int nbox_w = n_pad / kBoxRowsW;
        const int kblocks = (h_in_of(ti) + kBoxCols - 1) / kBoxCols;
        const uint32_t bytes = (uint32_t)(nbox_x * kBoxRowsAct + nbox_w * kBoxRowsW) * 128u;
        for (int kb = 0; kb < kblocks; ++kb, ++kiter) {
          const int s = kiter % kShrinkStages;
          if (!mbar_wait(empty_bar(s), ((kiter / kShrinkStages) & 1) ^ 1, &abort_s)) { ok = false; break; }
          mbar_expect_tx(full_bar(s), bytes);
          for (int i = 0; i < nbox_x; ++i)
            tma_load_2d(x_stage(s) + i * (kBoxRowsAct * 128), pmap_x, kb * kBoxCols,
                        ti.row0 + i * kBoxRowsAct, full_bar(s));
          for (int i = 0; i < nbox_w; ++i)
            tma_load_2d(w_stage(s) + i * (kBoxRowsW * 128), pmap_w, kb * kBoxCols,
                        (int)ti.wrow0 + i * kBoxRowsW, full_bar(s));
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
    }
    if (lane == 0 && abort_s) {
      // drain: let every copy that was issued land before the CTA retires
      volatile int none = 0;
      const uint32_t first = kiter > (uint32_t)kShrinkStages ? kiter - kShrinkStages : 0;
      for (uint32_t k = first; k < kiter; ++k)
        mbar_wait(full_bar(k % kShrinkStages), (k / kShrinkStages) & 1, &none);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    uint32_t kiter = 0, li = 0;
    bool ok = true;
    for (int64_t item = blockIdx.x; item < total && ok; item += gridDim.x) {
      const TileInfo ti = get_tile(src, item, false);
      if (!ti.valid) continue;
      if (lane == 0) {
        const int n_pad = (ti.rank + 15) & ~15;
        const int kblocks = (h_in_of(ti) + kBoxCols - 1) / kBoxCols;
        const uint32_t idesc = instr_desc_f16(std::is_same<T, __nv_bfloat16>::value, n_pad, 0);
        const int ab = li & 1;
        const uint32_t tacc = tmem_base + ab * kMaxRank;
        ok = mbar_wait(tempty_bar(ab), ((li >> 1) & 1) ^ 1, &abort_s);
        if (ok) tc_fence_after();
        for (int kb = 0; kb < kblocks && ok; ++kb, ++kiter) {
          const int s = kiter % kShrinkStages;
          ok = mbar_wait(full_bar(s), (kiter / kShrinkStages) & 1, &abort_s);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < kBoxCols / 16; ++k) {
            const uint64_t ad = smem_desc_sw128(x_stage(s) + k * 32, 16, 1024);
            const uint64_t bd = smem_desc_sw128(w_stage(s) + k * 32, 16, 1024);
            umma_f16(tacc, ad, bd, idesc, (kb | k) != 0);
          }
          umma_commit(empty_bar(s));
        }
        if (ok) umma_commit(tfull_bar(ab));
        ++li;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const int row = q * 32 + lane;
    uint32_t li = 0;
    for (int64_t item = blockIdx.x; item < total; item += gridDim.x) {
      const TileInfo ti = get_tile(src, item, false);
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
      if (q * 32 < ti.rows) {
        T* vrow = v + (int64_t)(ti.row0 + row) * v_pitch;
        for (int c = 0; c < n_pad; c += 16) {
          uint32_t r[16];
          tmem_ld_32x16(tmem_base + ((uint32_t)(q * 32) << 16) + ab * kMaxRank + c, r);
          tmem_ld_wait();
          if (row < ti.rows) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int col = c + h * 8;
              if (col < ti.rank) {
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[h * 8 + e]);
                if (accumulate) {
                  float old[8];
                  unpack8<T>(ldg128(vrow + col), old);
#pragma unroll
                  for (int e = 0; e < 8; ++e) f[e] += old[e];
                }
                stg128(vrow + col, pack8<T>(f));
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(ab));
      ++li;
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
  if (threadIdx.x == 0 && abort_s) g_status = 1;
}

// ============================================================================
// expand: persistent CTAs; per tile the V rows are staged once as the A operand,
// then a 3-stage ring streams (B tile, Y tile) pairs, 128 output columns each.
// ============================================================================
constexpr int kExpStages = 3;
constexpr int kExpTileN = 128;
constexpr int kExpABytes = 2 * kTileM * 128;           // V tile, two 64-column K blocks: 32 KB
constexpr int kExpBBytes = 2 * kMaxRank * 128;         // two 64-column N blocks x 128 rows: 32 KB
constexpr int kExpYBytes = 2 * kTileM * 128;           // two 64-column blocks x 128 rows: 32 KB
constexpr int kExpStageBytes = kExpBBytes + kExpYBytes;
constexpr int kExpSmem = 1024 + kExpABytes + kExpStages * kExpStageBytes + 256;

struct ExpRange { int nt_begin, nt_count, h_out; };

__device__ __forceinline__ ExpRange exp_range(const TileSource& src, const TileInfo& ti, int h_out_) {
  ExpRange r;
  r.h_out = src.plan ? src.plan[ti.problem].h_out : h_out_;
  const int ntiles = (r.h_out + kExpTileN - 1) / kExpTileN;
  const int per = (ntiles + src.nsplit - 1) / src.nsplit;
  r.nt_begin = ti.split * per;
  r.nt_count = max(0, min(per, ntiles - r.nt_begin));
  return r;
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
atmm_expand_kernel(const __grid_constant__ CUtensorMap map_y_, const __grid_constant__ CUtensorMap map_w_,
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
  auto b_stage = [&](int s) { return base + kExpABytes + (uint32_t)s * kExpStageBytes; };
  auto y_stage = [&](int s) { return base + kExpABytes + (uint32_t)s * kExpStageBytes + kExpBBytes; };
  const uint32_t bars = base + kExpABytes + kExpStages * kExpStageBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kExpStages + s); };
  auto tfull_bar = [&](int ab) { return bars + 8u * (2 * kExpStages + ab); };
  auto tempty_bar = [&](int ab) { return bars + 8u * (2 * kExpStages + 2 + ab); };
  const uint32_t a_ready_bar = bars + 8u * (2 * kExpStages + 4);
  const uint32_t a_free_bar = bars + 8u * (2 * kExpStages + 5);

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < kExpStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 4);
    }
    for (int ab = 0; ab < 2; ++ab) {
      mbar_init(tfull_bar(ab), 1);
      mbar_init(tempty_bar(ab), 4);
    }
    mbar_init(a_ready_bar, 128);
    mbar_init(a_free_bar, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    uint32_t it = 0;
    bool ok = true;
    for (int64_t item = blockIdx.x; item < total && ok; item += gridDim.x) {
      const TileInfo ti = get_tile(src, item, true);
      if (!ti.valid) continue;
      const ExpRange er = exp_range(src, ti, h_out_);
      if (lane == 0) {
        const CUtensorMap* pmap_y = src.plan ? &src.plan[ti.problem].map_y : &map_y_;
        const CUtensorMap* pmap_w = src.plan ? &src.plan[ti.problem].map_wb : &map_w_;
        const int k_pad = (ti.rank + 15) & ~15;
        const int ksteps = k_pad / 16;
        const int nbox_y = (ti.rows + kBoxRowsAct - 1) / kBoxRowsAct;
        for (int t = 0; t < er.nt_count; ++t, ++it) {
          const int s = it % kExpStages;
          if (!mbar_wait(empty_bar(s), ((it / kExpStages) & 1) ^ 1, &abort_s)) { ok = false; break; }
          const int n0 = (er.nt_begin + t) * kExpTileN;
          const int ncb = min(2, (er.h_out - n0 + kBoxCols - 1) / kBoxCols);
          const uint32_t bytes = (uint32_t)ncb * (uint32_t)(k_pad + nbox_y * kBoxRowsAct) * 128u;
          mbar_expect_tx(full_bar(s), bytes);
          for (int cb = 0; cb < ncb; ++cb)
            for (int j = 0; j < ksteps; ++j)
              tma_load_2d(b_stage(s) + cb * (kMaxRank * 128) + j * (kBoxRowsW * 128), pmap_w,
                          n0 + cb * kBoxCols, (int)ti.wrow0 + j * kBoxRowsW, full_bar(s));
          for (int cb = 0; cb < ncb; ++cb)
            for (int i = 0; i < nbox_y; ++i)
              tma_load_2d(y_stage(s) + cb * (kTileM * 128) + i * (kBoxRowsAct * 128), pmap_y,
                          n0 + cb * kBoxCols, ti.row0 + i * kBoxRowsAct, full_bar(s));
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
    }
    if (lane == 0 && abort_s) {
      volatile int none = 0;
      const uint32_t first = it > (uint32_t)kExpStages ? it - kExpStages : 0;
      for (uint32_t k = first; k < it; ++k)
        mbar_wait(full_bar(k % kExpStages), (k / kExpStages) & 1, &none);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    const uint32_t idesc = instr_desc_f16(std::is_same<T, __nv_bfloat16>::value, kExpTileN, 1);
    uint32_t it = 0, li = 0;
    bool ok = true;
    for (int64_t item = blockIdx.x; item < total && ok; item += gridDim.x) {
      const TileInfo ti = get_tile(src, item, true);
      if (!ti.valid) continue;
      const ExpRange er = exp_range(src, ti, h_out_);
      if (er.nt_count <= 0) continue;
      const int k_pad = (ti.rank + 15) & ~15;
      const int ksteps = k_pad / 16;
      ok = __all_sync(0xffffffffu, mbar_wait(a_ready_bar, li & 1, &abort_s));
      for (int t = 0; t < er.nt_count && ok; ++t, ++it) {
        const int s = it % kExpStages, ab = it & 1;
        bool got = mbar_wait(full_bar(s), (it / kExpStages) & 1, &abort_s);
        if (got) got = mbar_wait(tempty_bar(ab), ((it >> 1) & 1) ^ 1, &abort_s);
        ok = __all_sync(0xffffffffu, got);             // the whole warp goes on or gives up
        if (!ok) break;
        if (k_pad != ti.rank) {
          // rank % 16 == 8: rows rank..k_pad-1 of the B tile belong to the next slot.
          // The matching V columns are zero, but 0 * Inf/NaN would poison the sum.
          const int nrow = k_pad - ti.rank;            // 8
          for (int i = lane; i < 2 * nrow * 8; i += 32) {
            const int cb = i / (nrow * 8), rr = (i / 8) % nrow, ch = i % 8;
            sts128(b_stage(s) + cb * (kMaxRank * 128) + (ti.rank + rr) * 128 + ch * 16,
                   make_uint4(0, 0, 0, 0));
          }
          fence_proxy_async_smem();
          __syncwarp();
        }
        tc_fence_after();
        if (lane == 0) {
          for (int j = 0; j < ksteps; ++j) {
            const uint64_t ad = smem_desc_sw128(a_tile + (j >> 2) * (kTileM * 128) + (j & 3) * 32, 16, 1024);
            const uint64_t bd = smem_desc_sw128(b_stage(s) + j * (kBoxRowsW * 128), kMaxRank * 128, 1024);
            umma_f16(tmem_base + ab * kExpTileN, ad, bd, idesc, j != 0);
          }
          umma_commit(tfull_bar(ab));
        }
        __syncwarp();
      }
      if (ok && lane == 0) umma_commit(a_free_bar);    // V tile may be overwritten once these retire
      __syncwarp();
      ++li;
    }
  } else {
    // ------------------------------------------------------------ V staging + epilogue
    const int q = warp & 3;
    const int row = q * 32 + lane;
    uint32_t it = 0, li = 0;
    bool ok = true;
    for (int64_t item = blockIdx.x; item < total && ok; item += gridDim.x) {
      const TileInfo ti = get_tile(src, item, true);
      if (!ti.valid) continue;
      const ExpRange er = exp_range(src, ti, h_out_);
      if (er.nt_count <= 0) continue;
      T* y = y_;
      const T* v = v_;
      int v_pitch = v_pitch_;
      if (src.plan != nullptr) {
        y = reinterpret_cast<T*>(src.plan[ti.problem].y);
        v = reinterpret_cast<const T*>(src.vbuf) + (int64_t)ti.problem * src.vstride;
        v_pitch = kMaxRank;
      }
      const int h_out = er.h_out;
      const int k_pad = (ti.rank + 15) & ~15;
      const bool warp_live = q * 32 < ti.rows;
      // ---- stage V as the K-major, 128-byte-swizzled A operand (zeros beyond rank / rows)
      ok = __all_sync(0xffffffffu, mbar_wait(a_free_bar, (li & 1) ^ 1, &abort_s));
      if (!ok) break;
      {
        const T* vrow = v + (int64_t)(ti.row0 + row) * v_pitch;
        for (int c8 = 0; c8 < k_pad / 8; ++c8) {
          uint4 val = make_uint4(0, 0, 0, 0);
          if (row < ti.rows && c8 * 8 < ti.rank) val = ldg128(vrow + c8 * 8);
          sts128(a_tile + (c8 >> 3) * (kTileM * 128) + row * 128 + (((c8 & 7) ^ (row & 7)) << 4), val);
        }
        fence_proxy_async_smem();
        mbar_arrive(a_ready_bar);
      }
      const float scale = apply_scale ? Elem<T>::to_float(scales[ti.adapter]) : 1.f;
      for (int t = 0; t < er.nt_count; ++t, ++it) {
        const int s = it % kExpStages, ab = it & 1;
        bool got = mbar_wait(full_bar(s), (it / kExpStages) & 1, &abort_s);
        if (got) got = mbar_wait(tfull_bar(ab), (it >> 1) & 1, &abort_s);
        ok = __all_sync(0xffffffffu, got);
        if (!ok) break;
        tc_fence_after();
        const int n0 = (er.nt_begin + t) * kExpTileN;
        const uint32_t ys = y_stage(s);
        if (warp_live) {
          // phase 1: lane = row.  out = y0 + scale * acc, rounded once, written back in place
#pragma unroll 1
          for (int c = 0; c < kExpTileN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + ab * kExpTileN + c * 32, r);
            tmem_ld_wait();
            const uint32_t rowaddr = ys + (c >> 1) * (kTileM * 128) + row * 128;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int ch = (c & 1) * 4 + j;
              const uint32_t addr = rowaddr + ((ch ^ (row & 7)) << 4);
              float f[8];
              unpack8<T>(lds128(addr), f);
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = fmaf(scale, __uint_as_float(r[j * 8 + e]), f[e]);
              sts128(addr, pack8<T>(f));
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(ab));
        if (warp_live) {
          // phase 2: 4 rows x 128 bytes per instruction, rows of this segment only
#pragma unroll
          for (int cb = 0; cb < 2; ++cb) {
            const int col = n0 + cb * kBoxCols + (lane & 7) * 8;
#pragma unroll
            for (int p = 0; p < 8; ++p) {
              const int rr = q * 32 + p * 4 + (lane >> 3);
              if (rr < ti.rows && col < h_out) {
                const uint4 val = lds128(ys + cb * (kTileM * 128) + rr * 128 + (((lane & 7) ^ (rr & 7)) << 4));
                stg128(y + (int64_t)(ti.row0 + rr) * h_out + col, val);
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(s));
      }
      ++li;
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
  if (threadIdx.x == 0 && abort_s) g_status = 1;
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

// Split the output columns of a tile over several work items when there are too
// few tiles to give every SM a few items.
static int expand_splits(int64_t tiles, int h_out) {
  const int ntiles = (h_out + kExpTileN - 1) / kExpTileN;
  int64_t want = (4 * (int64_t)sm_count() + tiles - 1) / tiles;
  if (want < 1) want = 1;
  if (want > ntiles) want = ntiles;
  return (int)want;
}

template <typename T>
static int launch_atmm(void* y, const void* x, const void* w, const void* scales, TileSource src,
                       int64_t max_tiles, int64_t T_rows, int h_in, int h_out, int64_t w_cells,
                       int dtype, int flags, cudaStream_t stream, int n_problems) {
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e1 = cudaFuncSetAttribute(atmm_shrink_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kShrinkSmem);
    cudaError_t e2 = cudaFuncSetAttribute(atmm_shrink_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kShrinkSmem);
    cudaError_t e3 = cudaFuncSetAttribute(atmm_expand_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kExpSmem);
    cudaError_t e4 = cudaFuncSetAttribute(atmm_expand_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kExpSmem);
    if (e1 != cudaSuccess || e2 != cudaSuccess || e3 != cudaSuccess || e4 != cudaSuccess) {
      cudaGetLastError();
      return (int)(e1 != cudaSuccess ? e1 : e2 != cudaSuccess ? e2 : e3 != cudaSuccess ? e3 : e4);
    }
    attr_done = true;
  }
  if (max_tiles <= 0 || n_problems <= 0) return VLR_OK;
  // In step mode (src.plan set) the tensor maps come from the plan in device
  // memory, h_in / h_out are maxima over its problems and only size the grid.
  CUtensorMap map_act, map_w;
  memset(&map_act, 0, sizeof(map_act));
  memset(&map_w, 0, sizeof(map_w));
  const bool step = src.plan != nullptr;
  int rc;
  if (h_in >= h_out) {
    if (!step) {
      if ((rc = make_map_2d(&map_act, x, dtype, T_rows, h_in, kBoxRowsAct)) != VLR_OK) return rc;
      if ((rc = make_map_2d(&map_w, w, dtype, w_cells, h_in, kBoxRowsW)) != VLR_OK) return rc;
    }
    src.max_tiles = max_tiles;
    src.n_problems = n_problems;
    src.nsplit = 1;
    const int64_t items = max_tiles * n_problems;
    const unsigned grid = (unsigned)(items < sm_count() ? items : sm_count());
    atmm_shrink_kernel<T><<<grid, kThreads, kShrinkSmem, stream>>>(
        map_act, map_w, (T*)y, src, h_in, h_out, (flags & VLR_ATMM_ACCUMULATE_SHRINK) ? 1 : 0);
  } else {
    if (!step) {
      if ((rc = make_map_2d(&map_act, y, dtype, T_rows, h_out, kBoxRowsAct)) != VLR_OK) return rc;
      if ((rc = make_map_2d(&map_w, w, dtype, w_cells, h_out, kBoxRowsW)) != VLR_OK) return rc;
    }
    src.max_tiles = max_tiles;
    src.n_problems = n_problems;
    // in step mode the tile count lives on the device; with many problems no split is needed
    src.nsplit = step ? (n_problems >= 8 ? 1 : expand_splits((max_tiles / 8 + 1) * n_problems, h_out))
                      : expand_splits(max_tiles, h_out);
    const int64_t items = max_tiles * n_problems * src.nsplit;
    const unsigned grid = (unsigned)(items < sm_count() ? items : sm_count());
    atmm_expand_kernel<T><<<grid, kThreads, kExpSmem, stream>>>(
        map_act, map_w, (T*)y, (const T*)x, (const T*)scales, src, h_out, h_in,
        (flags & VLR_ATMM_APPLY_SCALE) ? 1 : 0);
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
  // every problem with m rows has ceil(m/128) tiles; sum <= T/128 + num_problems
  const int64_t max_tiles = T / kTileM + num_problems;
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
  return v;
}
