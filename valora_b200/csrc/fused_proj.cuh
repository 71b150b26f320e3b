// Base projection with the LoRA expand folded into the same accumulator:
//     Y[rows, :] = X[rows, :] W  +  V'[rows, :r] B_a            (V' = s * X A, from the shrink)
// for the consecutive-row tiles of a packed batch (up to 128 rows of one adapter).  The update
// is r more steps of the K loop - [X | V'] [W ; B_a] - so Y is written once and never read:
// the expand's read-modify-write of Y (two thirds of its HBM bytes) disappears, and what is
// left is a compute-bound GEMM.  In the reference the two halves are a torch.mm followed by
// dispatch_sgmm calls that read q / k / v / o back and add to them
// (valora/models/peft/lora_unordered_batch_infer.py:885 then :967-988; base projections
// valora/models/llama/layer_infer/transformer_layer_infer.py:42-50).
//
// Included by atmm_sm100.cu (inside namespace vlr), whose tile source, work-item ring and
// copy helpers it shares.  Persistent CTAs, 384 threads: warps 0-7 epilogue + V' staging,
// 8-9 TMA producers, 10 MMA issue, 11 work items.  A work item is (tile, 256 output columns).
//   stage (48 KB) = X tile [128 x 64] K-major + W tile [64 x 256] (four [64 x 64] boxes, N
//   contiguous = MN-major B operand); after the K / 64 base stages come one or two stages with
//   the adapter's B rows [<= 64 x 256], multiplied with the V' tile the epilogue warps staged.
//   accumulators: two of 256 tensor-memory columns (the epilogue of one item overlaps the main
//   loop of the next); results leave through a per-warp staging tile in shared memory so that
//   Y is written in 128-byte row pieces.
#pragma once

constexpr int kFpStages = 3;
constexpr int kFpStageBytes = 48 * 1024;
constexpr int kFpTileN = 256;
constexpr int kFpWBlock = 64 * 128;                    // one [64 x 64] box of W: 8 KB
constexpr int kFpOutBytes = kExpEpiWarps * 32 * 128;   // per-warp staging [32 rows x 64 columns]
constexpr int kFpSmem = 1024 + kExpABytes + kFpStages * kFpStageBytes + kFpOutBytes + 512 + kItemSlotBytes;

struct FusedArgs {
  const void* v;            // V' [T, v_pitch], scaled shrink result
  int v_pitch;
  int h_in, h_out;
  MapSet xw;                // act = X [T, h_in] (consecutive-row boxes), w[2] = W [h_in, h_out] (64-row boxes)
  MapSet yb;                // w = B-side pool [cells, h_out]
};

template <typename T>
__global__ void __launch_bounds__(kExpThreads, 1)
fused_proj_kernel(const __grid_constant__ FusedArgs fa, T* __restrict__ y, TileSource src) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ volatile int abort_s;
  __shared__ uint32_t tmem_base_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t total = total_items(src);
  if ((int64_t)blockIdx.x >= total) return;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_tile = base;                                        // V' tile, two 64-column K blocks
  auto stage = [&](int s) { return base + kExpABytes + (uint32_t)s * kFpStageBytes; };
  const uint32_t out0 = base + kExpABytes + kFpStages * kFpStageBytes;  // epilogue staging
  const uint32_t bars = out0 + kFpOutBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (4 + s); };
  auto tfull_bar = [&](int ab) { return bars + 8u * (8 + ab); };
  auto tempty_bar = [&](int ab) { return bars + 8u * (10 + ab); };
  const uint32_t a_ready_bar = bars + 8u * 12;
  const uint32_t a_free_bar = bars + 8u * 13;
  ItemFeed feed;
  feed.full0 = bars + 8u * 14;
  feed.empty0 = feed.full0 + 8u * kItemRing;
  feed.slots = reinterpret_cast<ItemSlot*>(smem_raw + (bars + 512u - smem_u32(smem_raw)));

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < kFpStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);                      // released by the MMA thread's commit
    }
    for (int ab = 0; ab < 2; ++ab) {
      mbar_init(tfull_bar(ab), 1);
      mbar_init(tempty_bar(ab), kExpEpiWarps);
    }
    mbar_init(a_ready_bar, 32 * kExpEpiWarps);
    mbar_init(a_free_bar, 1);
    for (int i = 0; i < kItemRing; ++i) {
      mbar_init(feed.full0 + 8u * i, 1);
      mbar_init(feed.empty0 + 8u * i, kExpFetchWarp);
    }
    fence_barrier_init();
  }
  if (warp == kExpMmaWarp) {
    tmem_alloc(smem_u32(&tmem_base_s), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  const int kblocks = fa.h_in / kBoxCols;
  const int ntiles_n = (fa.h_out + kFpTileN - 1) / kFpTileN;

  if (warp >= kExpProdWarp0 && warp < kExpMmaWarp) {
    // ------------------------------------------------------------ producers (stage k -> warp k % 2)
    const int pw = warp - kExpProdWarp0;
    uint32_t it = 0;
    bool ok = true;
    for (uint32_t ik = 0; ok; ++ik) {
      TileInfo ti;
      int hw, grow_l;
      const void* yb;
      if (!next_tile(feed, ik, &abort_s, ti, hw, yb, grow_l)) break;
      if (!ti.valid || ti.split >= ntiles_n) continue;
      const int n0 = ti.split * kFpTileN;
      const int ncb = min(4, (fa.h_out - n0 + kBoxCols - 1) / kBoxCols);
      const int k_pad = (ti.rank + 15) & ~15;
      const int lstages = (k_pad + 63) / 64;
      const int xrows = act_rows_loaded(ti.rows);
      if (lane == 0) {
        for (int st = 0; st < kblocks + lstages && ok; ++st, ++it) {
          if ((int)(it % kExpProducers) != pw) continue;
          const int s = it % kFpStages;
          ok = mbar_wait(empty_bar(s), ((it / kFpStages) & 1) ^ 1, &abort_s);
          if (!ok) break;
          if (st < kblocks) {
            mbar_expect_tx(full_bar(s), (uint32_t)(xrows + ncb * 64) * 128u);
            load_act_rows(stage(s), &fa.xw, st * kBoxCols, ti.row0, ti.rows, full_bar(s));
            for (int cb = 0; cb < ncb; ++cb)
              tma_load_2d(stage(s) + kTileM * 128 + cb * kFpWBlock, &fa.xw.w[2], n0 + cb * kBoxCols,
                          st * kBoxCols, full_bar(s));
          } else {
            // rank rows [64 j, 64 j + nr) of the adapter's B, the tile's 256 columns
            const int j = st - kblocks;
            const int nr = min(64, k_pad - 64 * j);
            mbar_expect_tx(full_bar(s), (uint32_t)(ncb * nr) * 128u);
            for (int cb = 0; cb < ncb; ++cb)
              load_w_rows(stage(s) + cb * (nr * 128), &fa.yb, n0 + cb * kBoxCols, (int)ti.wrow0 + 64 * j, nr,
                          full_bar(s));
          }
        }
      } else {
        it += kblocks + lstages;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      it = __shfl_sync(0xffffffffu, it, 0);
    }
    __syncwarp();
    if (pw == 0 && lane == 0 && abort_s) {
      volatile int none = 0;
      const uint32_t first = it > (uint32_t)kFpStages ? it - kFpStages : 0;
      for (uint32_t k = first; k < it; ++k) mbar_wait(full_bar(k % kFpStages), (k / kFpStages) & 1, &none);
    }
  } else if (warp == kExpMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    uint32_t it = 0, li = 0;
    bool ok = true;
    const bool bf = std::is_same<T, __nv_bfloat16>::value;
    const uint32_t idesc = instr_desc_f16(bf, kFpTileN, 1);
    for (uint32_t ik = 0; ok; ++ik) {
      TileInfo ti;
      int hw, grow_l;
      const void* yb;
      if (!next_tile(feed, ik, &abort_s, ti, hw, yb, grow_l)) break;
      if (!ti.valid || ti.split >= ntiles_n) continue;
      const int k_pad = (ti.rank + 15) & ~15;
      const int lstages = (k_pad + 63) / 64;
      const int ab = li & 1;
      const uint32_t tacc = tmem_base + ab * 256;
      if (lane == 0) {
        ok = mbar_wait(tempty_bar(ab), ((li >> 1) & 1) ^ 1, &abort_s);
        if (ok) tc_fence_after();
        for (int st = 0; st < kblocks + lstages && ok; ++st, ++it) {
          const int s = it % kFpStages;
          ok = mbar_wait(full_bar(s), (it / kFpStages) & 1, &abort_s);
          if (!ok) break;
          if (st == kblocks) ok = mbar_wait(a_ready_bar, li & 1, &abort_s);   // V' tile staged
          if (!ok) break;
          tc_fence_after();
          if (st < kblocks) {
            const uint64_t ad = smem_desc_sw128(stage(s), 16, 1024);
            const uint64_t bd = smem_desc_sw128(stage(s) + kTileM * 128, kFpWBlock, 1024);
#pragma unroll
            for (int k = 0; k < kBoxCols / 16; ++k)
              umma_f16(tacc, ad + (uint64_t)(2 * k), bd + (uint64_t)(k * (kBoxRowsW * 128 >> 4)), idesc,
                       (st > 0 || k > 0) ? 1u : 0u);
          } else {
            const int j = st - kblocks;
            const int nr = min(64, k_pad - 64 * j);
            const uint64_t ad = smem_desc_sw128(a_tile + j * (kTileM * 128), 16, 1024);
            const uint64_t bd = smem_desc_sw128(stage(s), (uint32_t)nr * 128u, 1024);
            for (int k = 0; k < nr / 16; ++k)
              umma_f16(tacc, ad + (uint64_t)(2 * k), bd + (uint64_t)(k * (kBoxRowsW * 128 >> 4)), idesc, 1u);
          }
          umma_commit(empty_bar(s));
        }
        if (ok) {
          umma_commit(tfull_bar(ab));
          umma_commit(a_free_bar);                     // the V' tile may be overwritten once these retire
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      it = __shfl_sync(0xffffffffu, it, 0);
      ++li;
    }
  } else if (warp < kExpEpiWarps) {
    // ------------------------------------------------------------ V' staging + epilogue
    const int q = warp & 3;                            // tensor-memory lane quarter = rows 32 q ..
    const int hh = warp >> 2;                          // which 128 of the tile's 256 columns
    const int et = threadIdx.x;                        // 0..255
    const uint32_t mine = out0 + warp * (32 * 128);    // this warp's staging tile: 32 rows x 64 columns
    uint32_t li = 0;
    bool ok = true;
    for (uint32_t ik = 0; ok; ++ik) {
      TileInfo ti;
      int hw, grow_l;
      const void* yb;
      if (!next_tile(feed, ik, &abort_s, ti, hw, yb, grow_l)) break;
      if (!ti.valid || ti.split >= ntiles_n) continue;
      const int n0 = ti.split * kFpTileN;
      const int k_pad = (ti.rank + 15) & ~15;
      const T* v = reinterpret_cast<const T*>(fa.v);
      // ---- stage V' as the K-major, 128-byte-swizzled A operand (zeros beyond rank / rows)
      ok = __all_sync(0xffffffffu, mbar_wait(a_free_bar, (li & 1) ^ 1, &abort_s));
      if (!ok) break;
      {
        const int vr = et & 127;
        const T* vrow = v + (int64_t)(vr < ti.rows ? ti.row0 + vr : 0) * fa.v_pitch;
        for (int c8 = et >> 7; c8 < k_pad / 8; c8 += kExpEpiWarps / 4) {
          uint4 val = make_uint4(0, 0, 0, 0);
          if (vr < ti.rows && c8 * 8 < ti.rank) val = ldg128(vrow + c8 * 8);
          sts128(a_tile + (c8 >> 3) * (kTileM * 128) + vr * 128 + (((c8 & 7) ^ (vr & 7)) << 4), val);
        }
        fence_proxy_async_smem();
        mbar_arrive(a_ready_bar);
      }
      const int ab = li & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(tfull_bar(ab), (li >> 1) & 1, &abort_s));
      if (!ok) break;
      tc_fence_after();
      const uint32_t tacc = tmem_base + ((uint32_t)(q * 32) << 16) + ab * 256 + hh * 128;
      const bool live = q * 32 < ti.rows;
#pragma unroll 1
      for (int pass = 0; pass < 2; ++pass) {
        if (live) {
          // lane = row: 64 accumulator columns -> 16-bit -> the staging tile (row-major, swizzled)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld_32x32(tacc + pass * 64 + h * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[c * 8 + e]);
              sts128(mine + lane * 128 + ((((h * 4 + c)) ^ (lane & 7)) << 4), pack8<T>(f));
            }
          }
        }
        if (pass == 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(ab));  // accumulator read out
        }
        __syncwarp();
        if (live) {
          // 4 rows x 128 bytes per instruction, rows of the tile only
          const int ch = lane & 7;
          const int col = n0 + hh * 128 + pass * 64 + ch * 8;
#pragma unroll
          for (int p = 0; p < 8; ++p) {
            const int rl = p * 4 + (lane >> 3);
            const int rr = q * 32 + rl;
            const uint4 ov = lds128(mine + rl * 128 + ((ch ^ (rl & 7)) << 4));
            if (rr < ti.rows && col < fa.h_out) stg128(y + (int64_t)(ti.row0 + rr) * fa.h_out + col, ov);
          }
        }
        __syncwarp();
      }
      ++li;
    }
    tc_fence_before();
  } else if (warp == kExpFetchWarp) {
    feed_tiles(src, feed, total, true, fa.h_out, y, &abort_s);
  }
  __syncthreads();
  if (warp == kExpMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && abort_s) raise_status(src, 1);
}
