// Decode gather mat-vec in its drop-in form (one adapter index per token, no
// packed schedule) for sm_100a: SIMT arithmetic fed by the bulk-copy engine.
//
// The reference's BGMV reads an adapter's rows once per token.  Here every CTA
// first groups the tokens of a window of the batch by adapter in shared memory
// (hash table + prefix sums; every CTA builds the same table), so that a work
// item is (group of up to 8 tokens of one adapter, slice of the output) and an
// adapter's rows are fetched once per group.  Inside a CTA one producer warp
// streams the rows - 1-D bulk copies straight from the paged pool cells, any
// a_loc order - into a ring of shared-memory stages armed with mbarriers, and
// eight consumer warps do the fp32 multiply-adds from shared memory, so the
// bytes in flight do not depend on registers or occupancy.  Each output is
// accumulated in fp32 and rounded once.
#include "common.cuh"
#include "problem.cuh"
#include "sm100_ptx.cuh"

namespace vlr {

using namespace ptx;

namespace {

constexpr int kG = 8;                          // tokens per group
constexpr int kWindow = 1024;                  // tokens grouped at a time
constexpr int kProducers = 2;                  // warps 0..1 issue the copies, stage k by warp k % 2
constexpr int kConsumers = 8;                  // warps 2..9 do the arithmetic
constexpr int kDecThreads = 32 * (kProducers + kConsumers);

__device__ int g_decode_status;                // 1: a bounded wait gave up

// Debug aid: while a buffer is set, CTA 0 writes clock64 stamps into it - slots 0..7:
// kernel start, grouping done, roles done, four points inside the grouping; then 4 per pipeline stage: copies issued
// (begin, end), stage seen by consumer warp 0, stage released by it.
__device__ long long* g_decode_trace;
__device__ long long g_decode_trace_cap;
__device__ __forceinline__ void dec_stamp(long long slot) {
#ifdef VLR_TRACE
  if (g_decode_trace != nullptr && blockIdx.x == 0 && slot < g_decode_trace_cap) g_decode_trace[slot] = clock64();
#else
  (void)slot;
#endif
}

// Groups of one window, in shared memory for the whole CTA.
struct GroupTable {
  int32_t adapter[kWindow];
  int32_t gbase[kWindow];                      // a_start[adapter] + rank * qkvo
  int16_t rank[kWindow];
  int16_t start[kWindow];                      // first position in sorted[]
  int16_t n[kWindow];                          // tokens in the group (1..8)
  int16_t sorted[kWindow];                     // window-relative token ids, grouped by adapter
  int n_groups;
};

constexpr int kBins = 2048;                    // adapter ids grouped by direct indexing
constexpr int kRanges = 8;                     // the window is cut into 8 token ranges of 128
constexpr int kTokPerThread = (kWindow + kDecThreads - 1) / kDecThreads;
// scratch (in the idle ring): counts [ranges][bins] u16, totals/bases [3][bins] i32,
// per-token rank-in-range i16 and adapter id i32
constexpr int kScratchBytes = kRanges * kBins * 2 + 3 * kBins * 4 + kWindow * 2 + kWindow * 4;

// All threads of the CTA.  A stable counting sort of the window's tokens by adapter
// id, so that every CTA derives the same groups: warp r ranks the tokens of range r
// among the same-adapter tokens of its range (peer masks + running counts), the
// ranges' counts are prefix-summed per adapter, the adapters are prefix-summed in
// id order, and a group is 8 consecutive tokens of an adapter's run.  Tokens with a
// negative adapter index join no group.  If an id does not fit the bins every token
// becomes a group of its own.  Each thread fetches rank and pool base of its own
// tokens' adapters right after the ids, so that round trip overlaps the sorting.
__device__ void build_groups(const int64_t* __restrict__ indicies, int64_t w0, int wn,
                             const int64_t* __restrict__ a_start, const int64_t* __restrict__ a_len,
                             int64_t qkvo, bool rank_mult8, GroupTable* gt, uint8_t* scratch) {
  __shared__ int wsum_t[8], wsum_g[8];
  __shared__ int amax_s;
  uint16_t* cntr = reinterpret_cast<uint16_t*>(scratch);            // [kRanges][kBins]
  int32_t* tot = reinterpret_cast<int32_t*>(cntr + kRanges * kBins);
  int32_t* tokbase = tot + kBins;
  int32_t* grpbase = tokbase + kBins;
  int16_t* trank = reinterpret_cast<int16_t*>(grpbase + kBins);     // rank of a token in (range, adapter)
  int32_t* ids = reinterpret_cast<int32_t*>(trank + kWindow);       // the window's adapter ids (-1: none)
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  if (tid == 0) amax_s = -1;
  int my_a[kTokPerThread], my_r[kTokPerThread];
  int64_t my_b[kTokPerThread];
  int amax = -1;
#pragma unroll
  for (int k = 0; k < kTokPerThread; ++k) {
    const int t = tid + k * kDecThreads;
    my_a[k] = t < wn ? (int)max(min(indicies[w0 + t], (int64_t)0x7fffffff), (int64_t)-1) : -1;
    if (t < kWindow) ids[t] = my_a[k];
    amax = max(amax, my_a[k]);
  }
#pragma unroll
  for (int k = 0; k < kTokPerThread; ++k) {
    my_r[k] = 0;
    my_b[k] = 0;
    if (my_a[k] >= 0) {
      my_r[k] = (int)(a_len[my_a[k]] / 4);
      my_b[k] = a_start[my_a[k]];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  __syncthreads();
  if (lane == 0) atomicMax(&amax_s, amax);
  __syncthreads();
  amax = amax_s;
  if (tid == 0) dec_stamp(3);
  // my_r / my_b are first touched where the records are written: their loads stay in flight
  auto finish_rank = [&](int k) {
    if (my_r[k] < 0 || my_r[k] > kMaxRank || (rank_mult8 && (my_r[k] & 7))) my_r[k] = 0;
    my_b[k] += (int64_t)my_r[k] * qkvo;
  };
  if (amax >= kBins) {
#pragma unroll
    for (int k = 0; k < kTokPerThread; ++k) {
      const int t = tid + k * kDecThreads;
      if (t < wn) {
        finish_rank(k);
        gt->adapter[t] = max(my_a[k], 0);
        gt->rank[t] = (int16_t)my_r[k];
        gt->gbase[t] = (int32_t)my_b[k];
        gt->start[t] = (int16_t)t;
        gt->n[t] = 1;
        gt->sorted[t] = (int16_t)t;
      }
    }
    if (tid == 0) gt->n_groups = wn;
    fence_proxy_async_smem();
    __syncthreads();
    return;
  }
  const int nb = (amax + 256) & ~255;                                // bins in use, a multiple of 256
  for (int r = 0; r < kRanges; ++r)
    for (int i = tid; i < nb; i += kDecThreads) cntr[r * kBins + i] = 0;
  __syncthreads();
  if (warp < kRanges) {
    // tokens [128 * warp, +128) in order, 32 at a time
    for (int c = 0; c < 4; ++c) {
      const int t = warp * 128 + c * 32 + lane;
      const int a = ids[t];
      // lanes holding the same adapter id: every lane reads the chunk's 32 ids (eight
      // broadcast 16-byte loads; 32 shuffles or match.any cost several times more here)
      unsigned peers = 0;
      const int4* chunk = reinterpret_cast<const int4*>(ids + warp * 128 + c * 32);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int4 v = chunk[i];
        peers |= (v.x == a ? 1u : 0u) << (4 * i) | (v.y == a ? 1u : 0u) << (4 * i + 1) |
                 (v.z == a ? 1u : 0u) << (4 * i + 2) | (v.w == a ? 1u : 0u) << (4 * i + 3);
      }
      // the lowest peer reads and bumps the running count; everybody fetches it from there
      // (one full-mask shuffle with a per-lane source: a shuffle per peer group would be
      // issued once per distinct mask)
      const int leader = __ffs(peers) - 1;
      int before = 0;
      if (a >= 0 && lane == leader) {
        before = cntr[warp * kBins + a];
        cntr[warp * kBins + a] = (uint16_t)(before + __popc(peers));
      }
      before = __shfl_sync(0xffffffffu, before, leader);
      if (a >= 0) trank[t] = (int16_t)(before + __popc(peers & ((1u << lane) - 1u)));
      __syncwarp();
    }
  }
  __syncthreads();
  if (tid == 0) dec_stamp(4);
  // per adapter: exclusive prefix over the ranges (in place) and the total
  for (int bin = tid; bin < nb; bin += kDecThreads) {
    int run = 0;
#pragma unroll
    for (int r = 0; r < kRanges; ++r) {
      const int v = cntr[r * kBins + bin];
      cntr[r * kBins + bin] = (uint16_t)run;
      run += v;
    }
    tot[bin] = run;
  }
  __syncthreads();
  if (tid == 0) dec_stamp(5);
  // exclusive prefix sums over the adapters (tokens and groups): threads 0..255, 8 bins each
  int c8[8], ts = 0, gs = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int bin = tid * 8 + i;
    c8[i] = (tid < 256 && bin < nb) ? tot[bin] : 0;
    ts += c8[i];
    gs += (c8[i] + kG - 1) / kG;
  }
  int its = ts, igs = gs;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, its, o), b = __shfl_up_sync(0xffffffffu, igs, o);
    if (lane >= o) {
      its += a;
      igs += b;
    }
  }
  if (tid < 256 && lane == 31) {
    wsum_t[warp] = its;
    wsum_g[warp] = igs;
  }
  __syncthreads();
  if (tid < 256) {
    int tb = its - ts, gb = igs - gs;
    for (int w = 0; w < warp; ++w) {
      tb += wsum_t[w];
      gb += wsum_g[w];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int bin = tid * 8 + i;
      if (bin < nb) {
        tokbase[bin] = tb;
        grpbase[bin] = gb;
        tb += c8[i];
        gb += (c8[i] + kG - 1) / kG;
      }
    }
    if (tid == 255) gt->n_groups = gb;
  }
  __syncthreads();
  if (tid == 0) dec_stamp(6);
  // place every token; the first token of a group also writes the group's record
#pragma unroll
  for (int k = 0; k < kTokPerThread; ++k) {
    const int t = tid + k * kDecThreads, a = my_a[k];
    if (t < wn && a >= 0) {
      const int within = cntr[(t >> 7) * kBins + a] + trank[t];      // position in the adapter's run
      gt->sorted[tokbase[a] + within] = (int16_t)t;
      if ((within & (kG - 1)) == 0) {
        finish_rank(k);
        const int gid = grpbase[a] + within / kG;
        gt->adapter[gid] = a;
        gt->rank[gid] = (int16_t)my_r[k];
        gt->gbase[gid] = (int32_t)my_b[k];
        gt->start[gid] = (int16_t)(tokbase[a] + within);
        gt->n[gid] = (int16_t)min(kG, tot[a] - within);
      }
    }
  }
  fence_proxy_async_smem();                            // scratch is about to be written by bulk copies
  __syncthreads();
}

// ----------------------------------------------------------------------------
// shrink: v[token, j] = sum_k x[token, k] * W[cell(j), k]   (overwrites, j < rank)
// item = (group, slice of 8 rank rows); a stage = 2048 columns of the group's
// activation rows (8 x 4 KB) and of the slice's 8 pool cells (8 x 4 KB).
// The 256 consumer lanes split the columns: a lane owns one 16-byte piece of every
// row of a stage, keeps the group's activations of that piece in registers and
// runs them against the 8 weight rows (64 accumulators per lane, 64 multiply-adds
// per 16-byte shared-memory load).  At the end of an item the partial sums are
// combined: a reduce-scatter inside each warp, then a fixed-order sum over the
// warps through shared memory, so results do not depend on timing.
// ----------------------------------------------------------------------------
constexpr int kShrSlice = 8;                            // rank rows per item
constexpr int kShrChunk = 256 * 8;                      // columns per stage
constexpr int kShrRowBytes = kShrChunk * 2;             // 4 KB
constexpr int kShrStageBytes = (kG + kShrSlice) * kShrRowBytes;   // 64 KB
constexpr int kShrStages = 3;
constexpr int kShrSmem = kShrStages * kShrStageBytes + 128;
static_assert(kScratchBytes <= kShrStages * kShrStageBytes, "grouping scratch must fit in the ring");

struct ShrinkInfo {
  int valid, first, last, nrows, nlive, slice0, cb, pad;
  int rows[kG];
};

__device__ __forceinline__ void consumer_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(32 * kConsumers) : "memory");
}

// v[0..N): keep the half chosen by lane bit d, add the partner's copy of it
template <int N>
__device__ __forceinline__ void halve(float (&v)[kShrSlice * kG], int lane, int d) {
  const bool up = lane & d;
#pragma unroll
  for (int i = 0; i < N / 2; ++i) {
    const float send = up ? v[i] : v[i + N / 2], keep = up ? v[i + N / 2] : v[i];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, d);
  }
}

// One lane's 16-byte piece of a stage: the activations of NG tokens against up to 8
// weight rows.  The multiply-adds of one weight element run over the tokens, so
// consecutive instructions never depend on each other.  Rows of absent tokens hold
// stale bytes; their sums are never stored.
template <typename T, int NG>
__device__ __forceinline__ void shrink_piece(uint32_t xaddr, uint32_t waddr, int nlive,
                                             float2 (&acc)[kShrSlice][kG / 2]) {
  // tokens in pairs: one packed fp32 multiply-add (fma.rn.f32x2) serves two tokens
  float2 xf[NG / 2][8];
#pragma unroll
  for (int h = 0; h < NG / 2; ++h) {
    float a[8], b[8];
    unpack8<T>(lds128(xaddr + (2 * h) * kShrRowBytes), a);
    unpack8<T>(lds128(xaddr + (2 * h + 1) * kShrRowBytes), b);
#pragma unroll
    for (int e = 0; e < 8; ++e) xf[h][e] = make_float2(a[e], b[e]);
  }
#pragma unroll
  for (int j = 0; j < kShrSlice; ++j) {
    if (j < nlive) {
      float wf[8];
      unpack8<T>(lds128(waddr + j * kShrRowBytes), wf);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float2 w2 = make_float2(wf[e], wf[e]);
#pragma unroll
        for (int h = 0; h < NG / 2; ++h) acc[j][h] = __ffma2_rn(w2, xf[h][e], acc[j][h]);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kDecThreads, 1)
bgmv_decode_shrink_kernel(T* __restrict__ v, const T* __restrict__ x, const T* __restrict__ w,
                          const int64_t* __restrict__ indicies, int64_t batch,
                          const int64_t* __restrict__ a_start, const int64_t* __restrict__ a_len,
                          const int64_t* __restrict__ a_loc, int64_t qkvo, int h_in, int v_pitch) {
  extern __shared__ uint8_t dec_smem[];
  __shared__ GroupTable gt;
  __shared__ ShrinkInfo infos[kShrStages];
  __shared__ float redw[2][kConsumers][kShrSlice * kG];   // alternating per item: one barrier per item
  __shared__ __align__(8) uint64_t bar_mem[2 * kShrStages];
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t ring = (smem_u32(dec_smem) + 127u) & ~127u;
  uint8_t* ring_ptr = dec_smem + (ring - smem_u32(dec_smem));
  auto full_bar = [&](int s) { return smem_u32(&bar_mem[s]); };
  auto empty_bar = [&](int s) { return smem_u32(&bar_mem[kShrStages + s]); };
  auto stage = [&](int s) { return ring + (uint32_t)s * kShrStageBytes; };

  if (tid == 0) {
    abort_s = 0;
    for (int s = 0; s < kShrStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), kConsumers);
    }
    fence_barrier_init();
  }
  __syncthreads();

  const int n_slices = (v_pitch + kShrSlice - 1) / kShrSlice;
  const int nchunks = (h_in + kShrChunk - 1) / kShrChunk;
  uint32_t it = 0;                                     // stages used so far: same count in every role
  if (tid == 0) dec_stamp(0);

  for (int64_t w0 = 0; w0 < batch; w0 += kWindow) {
    const int wn = (int)min((int64_t)kWindow, batch - w0);
    build_groups(indicies, w0, wn, a_start, a_len, qkvo, false, &gt, ring_ptr);
    const int64_t total = (int64_t)gt.n_groups * n_slices;
    if (tid == 0) dec_stamp(1);

    if (warp < kProducers) {
      // -------------------------------------------------------------- producers (stage k -> warp k % 2)
      bool ok = true;
      for (int64_t item = blockIdx.x; item < total && ok; item += gridDim.x) {
        const int g = (int)(item / n_slices), slice0 = (int)(item % n_slices) * kShrSlice;
        const int rank = gt.rank[g];
        if (slice0 >= rank) continue;
        const int nrows = gt.n[g], nlive = min(kShrSlice, min(rank, v_pitch) - slice0);
        // lanes 0..7: one pool cell each; lanes 8..15: one activation row each
        const T* src = nullptr;
        int myrow = -1;
        if (lane < nlive) {
          src = w + a_loc[gt.gbase[g] + slice0 + lane] * (int64_t)h_in;
        } else if (lane >= kShrSlice && lane - kShrSlice < nrows) {
          myrow = (int)w0 + gt.sorted[gt.start[g] + lane - kShrSlice];
          src = x + (int64_t)myrow * h_in;
        }
        const uint32_t slot = (uint32_t)(lane < kShrSlice ? kG + lane : lane - kShrSlice) * kShrRowBytes;
        for (int c = 0; c < nchunks; ++c, ++it) {
          if ((int)(it % kProducers) != warp) continue;
          const int s = it % kShrStages;
          if (lane == 0) ok = mbar_wait(empty_bar(s), ((it / kShrStages) & 1) ^ 1, &abort_s);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
          const int cb = min(kShrChunk, h_in - c * kShrChunk) * 2;
          if (lane == 0) dec_stamp(8 + 4 * (long long)it);
          if (lane == 0) {
            ShrinkInfo& in = infos[s];
            in.valid = 1; in.first = c == 0; in.last = c == nchunks - 1;
            in.nrows = nrows; in.nlive = nlive; in.slice0 = slice0; in.cb = cb;
          }
          if (lane >= kShrSlice && lane < kShrSlice + kG) infos[s].rows[lane - kShrSlice] = myrow;
          __syncwarp();
          if (lane == 0) mbar_expect_tx(full_bar(s), (uint32_t)(nlive + nrows) * cb);
          __syncwarp();
          if (src != nullptr) bulk_load_1d(stage(s) + slot, src + (int64_t)c * kShrChunk, cb, full_bar(s));
          if (lane == 0) dec_stamp(8 + 4 * (long long)it + 1);
        }
      }
      // end of the window: a stage that carries no work, armed by the warp whose turn it is
      if (ok) {
        if ((int)(it % kProducers) == warp) {
          const int s = it % kShrStages;
          if (lane == 0) ok = mbar_wait(empty_bar(s), ((it / kShrStages) & 1) ^ 1, &abort_s);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (ok && lane == 0) {
            infos[s].valid = 0;
            mbar_arrive(full_bar(s));
          }
        }
        ++it;
      }
      if (!ok && warp == 0 && lane == 0) {
        // gave up: let every copy that was issued land before the CTA retires
        volatile int none = 0;
        const uint32_t first = it > (uint32_t)kShrStages ? it - kShrStages : 0;
        for (uint32_t k = first; k < it; ++k) mbar_wait(full_bar(k % kShrStages), (k / kShrStages) & 1, &none);
      }
    } else {
      // -------------------------------------------------------------- consumers
      const int cw = warp - kProducers;
      const int piece = (cw * 32 + lane) * 16;          // this lane's bytes of every row of a stage
      float2 acc[kShrSlice][kG / 2];                      // [rank row][token pair]
      int rb = 0;
      while (true) {
        const int s = it % kShrStages;
        if (!mbar_wait(full_bar(s), (it / kShrStages) & 1, &abort_s)) break;
        if (cw == 0 && lane == 0) dec_stamp(8 + 4 * (long long)it + 2);
        const uint32_t it_now = it;
        ++it;
        const ShrinkInfo& in = infos[s];
        const int valid = in.valid, nrows = in.nrows, nlive = in.nlive;
        if (valid) {
          if (in.first) {
#pragma unroll
            for (int j = 0; j < kShrSlice; ++j)
#pragma unroll
              for (int h = 0; h < kG / 2; ++h) acc[j][h] = make_float2(0.f, 0.f);
          }
          if (piece < in.cb) {
            const uint32_t xa = stage(s) + piece, wa = xa + kG * kShrRowBytes;
            if (nrows <= 4) shrink_piece<T, 4>(xa, wa, nlive, acc);
            else shrink_piece<T, 8>(xa, wa, nlive, acc);
          }
          if (in.last) {
            // 64 partial sums per lane -> 2 per lane -> per-warp rows in shared memory
            float fl[kShrSlice * kG];                    // [rank row * 8 + token]
#pragma unroll
            for (int j = 0; j < kShrSlice; ++j)
#pragma unroll
              for (int h = 0; h < kG / 2; ++h) {
                fl[j * kG + 2 * h] = acc[j][h].x;
                fl[j * kG + 2 * h + 1] = acc[j][h].y;
              }
            halve<64>(fl, lane, 16);
            halve<32>(fl, lane, 8);
            halve<16>(fl, lane, 4);
            halve<8>(fl, lane, 2);
            halve<4>(fl, lane, 1);
            const int idx = ((lane & 16) ? 32 : 0) + ((lane & 8) ? 16 : 0) + ((lane & 4) ? 8 : 0) +
                            ((lane & 2) ? 4 : 0) + ((lane & 1) ? 2 : 0);
            redw[rb][cw][idx] = fl[0];
            redw[rb][cw][idx + 1] = fl[1];
            consumer_barrier();
            const int ct = cw * 32 + lane;              // 0..255
            if (ct < kShrSlice * kG) {
              const int g = ct / kShrSlice, j = ct % kShrSlice;
              float sum = 0.f;
#pragma unroll
              for (int wv = 0; wv < kConsumers; ++wv) sum += redw[rb][wv][j * kG + g];
              if (g < nrows && j < nlive)
                v[(int64_t)in.rows[g] * v_pitch + in.slice0 + j] = Elem<T>::from_float(sum);
            }
            rb ^= 1;                                  // the other buffer is free: its readers passed this item's barrier
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(s));
        if (cw == 0 && lane == 0) dec_stamp(8 + 4 * (long long)it_now + 3);
        if (!valid) break;
      }
    }
    __syncthreads();                                   // ring drained; its memory is scratch again
    if (tid == 0) dec_stamp(2);
    if (abort_s) break;
  }
  if (tid == 0 && abort_s) g_decode_status = 1;
}

// ----------------------------------------------------------------------------
// expand, punica weight layout: the r cells of a slot hold the flat bytes of
// Bt [h_out, r], so the r weights of output column o are contiguous (flat element
// o * r) and may run across a cell boundary.
//   y[token, o] += scale[adapter] * sum_k v[token, k] * Bt[o, k]
// item = (group, slice of 1024 output columns); a stage = the weights of `cps`
// columns (at most 16 KB, copied cell run by cell run) and, in an item's first
// stage, the group's V rows.
// A lane owns one 16-byte piece (8 of the r weights) of a column: cpo = r / 8
// lanes (rounded up to a power of two) share a column and combine their partial
// sums of the 8 tokens with a reduce-scatter, after which each holds the finished
// sums of 8 / cpo tokens.  The sums go through a small per-warp tile in shared
// memory so that Y is read and written in 16-byte pieces (fetched before the
// arithmetic of the stage starts), with one rounding per output.
// ----------------------------------------------------------------------------
constexpr int kExpSlice = 1024;                        // output columns per item
constexpr int kExpMaxCps = 512;                        // columns per stage, at most
constexpr int kExpWBytes = 16 * 1024;
constexpr int kExpVBytes = kG * kMaxRank * 2;          // 2 KB
constexpr int kExpStageBytes = kExpWBytes + kExpVBytes;   // 18 KB
constexpr int kExpStages = 9;
constexpr int kTileFloats = kG * 68;                   // one warp's tile
constexpr int kExpSmem = kExpStages * kExpStageBytes + 2 * kConsumers * kTileFloats * 4 + 128;
constexpr int kTilePitch = 68;                         // floats; rows of a warp's tile fall in different banks
static_assert(kTileFloats == kG * kTilePitch, "tile size");
static_assert(kScratchBytes <= kExpStages * kExpStageBytes, "grouping scratch must fit in the ring");

struct ExpandInfo {
  int valid, first, nrows, rank, cpo, o0, ncol, vk;     // vk: columns of a V row that exist, min(rank, v_pitch)
  float scale;
  int pad[3];
  int rows[kG];
};

// part[rd][i] (i < 8): partial sums of tokens 0..7 of round rd's column on each of its
// CPO lanes.  After the call the lane holds in part[rd][0 .. 8/CPO) (one value if
// CPO >= 8) the full sums of tokens g0, g0 + 1, ...  The steps run across all rounds
// so that the shuffles of one step are independent of each other.
template <int CPO, int R>
__device__ __forceinline__ int reduce_scatter(float (&v)[R][kG], int lane) {
  int g0 = 0;
  if (CPO >= 2) {
    const int d = CPO / 2;
    const bool up = lane & d;
#pragma unroll
    for (int rd = 0; rd < R; ++rd)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float send = up ? v[rd][i] : v[rd][i + 4], keep = up ? v[rd][i + 4] : v[rd][i];
        v[rd][i] = keep + __shfl_xor_sync(0xffffffffu, send, d);
      }
    g0 += up ? 4 : 0;
  }
  if (CPO >= 4) {
    const int d = CPO / 4;
    const bool up = lane & d;
#pragma unroll
    for (int rd = 0; rd < R; ++rd)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float send = up ? v[rd][i] : v[rd][i + 2], keep = up ? v[rd][i + 2] : v[rd][i];
        v[rd][i] = keep + __shfl_xor_sync(0xffffffffu, send, d);
      }
    g0 += up ? 2 : 0;
  }
  if (CPO >= 8) {
    const int d = CPO / 8;
    const bool up = lane & d;
#pragma unroll
    for (int rd = 0; rd < R; ++rd) {
      const float send = up ? v[rd][0] : v[rd][1], keep = up ? v[rd][1] : v[rd][0];
      v[rd][0] = keep + __shfl_xor_sync(0xffffffffu, send, d);
    }
    g0 += up ? 1 : 0;
  }
  if (CPO >= 16) {
#pragma unroll
    for (int rd = 0; rd < R; ++rd) v[rd][0] += __shfl_xor_sync(0xffffffffu, v[rd][0], 1);
  }
  return g0;
}

// The 16-byte pieces of Y a lane adds a stage's sums to: fetched when the stage is
// taken up, written one stage later, so the loads have a whole stage to arrive.
template <typename T>
struct PendingY {
  T* yp[2];
  uint4 y0v[2];
  int off[2];                                          // where the 8 sums sit in the warp's tile
};

template <typename T>
__device__ __forceinline__ void fetch_y(PendingY<T>& p, const ExpandInfo& in, int cw, int lane,
                                        T* __restrict__ y, int h_out) {
  const int cps = min(kExpMaxCps, 1024 / in.cpo), cols_w = cps / kConsumers, ppr = cols_w / 8;
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const int pc = lane + 32 * q, g = pc / ppr, c8 = (pc % ppr) * 8, col = cw * cols_w + c8;
    p.yp[q] = nullptr;
    if (pc < kG * ppr && g < in.nrows && col < in.ncol) {
      p.yp[q] = y + (int64_t)in.rows[g] * h_out + in.o0 + col;
      p.y0v[q] = ldg128(p.yp[q]);
      p.off[q] = g * kTilePitch + c8;
    }
  }
}

template <typename T>
__device__ __forceinline__ void flush_y(PendingY<T>& p, const float* __restrict__ tile) {
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    if (p.yp[q] != nullptr) {
      const float4 s0 = *reinterpret_cast<const float4*>(&tile[p.off[q]]);
      const float4 s1 = *reinterpret_cast<const float4*>(&tile[p.off[q] + 4]);
      float f[8];
      unpack8<T>(p.y0v[q], f);
      f[0] += s0.x; f[1] += s0.y; f[2] += s0.z; f[3] += s0.w;
      f[4] += s1.x; f[5] += s1.y; f[6] += s1.z; f[7] += s1.w;
      stg128(p.yp[q], pack8<T>(f));
      p.yp[q] = nullptr;
    }
  }
}

// One consumer warp's share of a stage, columns [cw * cols_w, (cw + 1) * cols_w):
// the scaled sums of every (token, column) go to the warp's tile.
template <typename T, int CPO, int NG>
__device__ __forceinline__ void expand_stage(const ExpandInfo& in, uint32_t st, float* __restrict__ tile,
                                             int cw, int lane, const float2 (&vs)[kG / 2][8]) {
  constexpr int opw = 32 / CPO;                        // columns per warp instruction
  constexpr int cps = (1024 / CPO) < kExpMaxCps ? (1024 / CPO) : kExpMaxCps;
  constexpr int cols_w = cps / kConsumers;             // 64, 64, 32, 16, 8
  constexpr int rounds = cols_w / opw;                 // 2, 4, 4, 4, 4
  const int rank = in.rank, ncol = in.ncol;
  const int kc = lane % CPO, ol = lane / CPO;
  float part[rounds][kG];
#pragma unroll
  for (int rd = 0; rd < rounds; ++rd) {
    const int col = cw * cols_w + rd * opw + ol;
    float2 p2[kG / 2];
#pragma unroll
    for (int h = 0; h < kG / 2; ++h) p2[h] = make_float2(0.f, 0.f);
    float wf[8];
    unpack8<T>(col < ncol && kc * 8 < rank ? lds128(st + (uint32_t)(col * rank + kc * 8) * 2)
                                            : make_uint4(0, 0, 0, 0), wf);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float2 w2 = make_float2(wf[e], wf[e]);
#pragma unroll
      for (int h = 0; h < NG / 2; ++h) p2[h] = __ffma2_rn(vs[h][e], w2, p2[h]);
    }
#pragma unroll
    for (int h = 0; h < kG / 2; ++h) {
      part[rd][2 * h] = p2[h].x;
      part[rd][2 * h + 1] = p2[h].y;
    }
  }
  const int g0 = reduce_scatter<CPO, rounds>(part, lane);
  constexpr int nval = CPO >= 8 ? 1 : kG / CPO;
  if (CPO < 16 || (lane & 1) == 0) {
#pragma unroll
    for (int rd = 0; rd < rounds; ++rd)
#pragma unroll
      for (int i = 0; i < nval; ++i) tile[(g0 + i) * kTilePitch + rd * opw + ol] = part[rd][i];
  }
  __syncwarp();
}

template <typename T>
__global__ void __launch_bounds__(kDecThreads, 1)
bgmv_decode_expand_kernel(T* __restrict__ y, const T* __restrict__ v, const T* __restrict__ w,
                          const T* __restrict__ scales, const int64_t* __restrict__ indicies,
                          int64_t batch, const int64_t* __restrict__ a_start,
                          const int64_t* __restrict__ a_len, const int64_t* __restrict__ a_loc,
                          int64_t qkvo, int h_out, int v_pitch) {
  extern __shared__ uint8_t dec_smem[];
  __shared__ GroupTable gt;
  __shared__ ExpandInfo infos[kExpStages];
  __shared__ int32_t cells_s[kProducers][kMaxRank];
  __shared__ __align__(8) uint64_t bar_mem[2 * kExpStages];
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t ring = (smem_u32(dec_smem) + 127u) & ~127u;
  uint8_t* ring_ptr = dec_smem + (ring - smem_u32(dec_smem));
  auto full_bar = [&](int s) { return smem_u32(&bar_mem[s]); };
  auto empty_bar = [&](int s) { return smem_u32(&bar_mem[kExpStages + s]); };
  auto stage = [&](int s) { return ring + (uint32_t)s * kExpStageBytes; };
  // two tiles per consumer warp, behind the ring
  float* tiles = reinterpret_cast<float*>(ring_ptr + kExpStages * kExpStageBytes);
  auto tile_of = [&](int b, int cw) { return tiles + (b * kConsumers + cw) * kTileFloats; };

  if (tid == 0) {
    abort_s = 0;
    for (int s = 0; s < kExpStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), kConsumers);
    }
    fence_barrier_init();
  }
  __syncthreads();

  const int n_slices = (h_out + kExpSlice - 1) / kExpSlice;
  uint32_t it = 0;
  if (tid == 0) dec_stamp(0);

  for (int64_t w0 = 0; w0 < batch; w0 += kWindow) {
    const int wn = (int)min((int64_t)kWindow, batch - w0);
    build_groups(indicies, w0, wn, a_start, a_len, qkvo, true, &gt, ring_ptr);
    const int64_t total = (int64_t)gt.n_groups * n_slices;
    if (tid == 0) dec_stamp(1);

    if (warp < kProducers) {
      // -------------------------------------------------------------- producers (stage k -> warp k % 2)
      bool ok = true;
      for (int64_t item = blockIdx.x; item < total && ok; item += gridDim.x) {
        const int g = (int)(item / n_slices), o_begin = (int)(item % n_slices) * kExpSlice;
        const int rank = gt.rank[g];
        if (rank <= 0) continue;
        const int vk = min(rank, v_pitch);
        const int nrows = gt.n[g];
        int cpo = 1;
        while (cpo * 8 < rank) cpo <<= 1;              // 1, 2, 4, 8, 16
        const int cps = min(kExpMaxCps, 1024 / cpo);
        const int o_end = min(h_out, o_begin + kExpSlice);
        const int myrow = lane < nrows ? (int)w0 + gt.sorted[gt.start[g] + lane] : -1;
        const float scale = Elem<T>::to_float(scales[gt.adapter[g]]);
        // the slot's pool cells
        __syncwarp();
#pragma unroll
        for (int q = 0; q < 4; ++q)
          if (q * 32 + lane < rank) cells_s[warp][q * 32 + lane] = (int32_t)a_loc[gt.gbase[g] + q * 32 + lane];
        __syncwarp();
        for (int o0 = o_begin; o0 < o_end; o0 += cps, ++it) {
          if ((int)(it % kProducers) != warp) continue;
          const int s = it % kExpStages;
          if (lane == 0) ok = mbar_wait(empty_bar(s), ((it / kExpStages) & 1) ^ 1, &abort_s);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
          const int ncol = min(cps, o_end - o0);
          const bool first = o0 == o_begin;
          if (lane == 0) dec_stamp(8 + 4 * (long long)it);
          if (lane == 0) {
            ExpandInfo& in = infos[s];
            in.valid = 1; in.first = first; in.nrows = nrows; in.rank = rank; in.cpo = cpo;
            in.o0 = o0; in.ncol = ncol; in.scale = scale; in.vk = vk;
          }
          if (lane < kG) infos[s].rows[lane] = myrow;
          __syncwarp();
          if (lane == 0)
            mbar_expect_tx(full_bar(s), (uint32_t)(ncol * rank + (first ? nrows * vk : 0)) * 2u);
          __syncwarp();
          // weights: the flat elements from f0 on, in pieces of 1 KB (one per lane, so many
          // copies stream at once), each cut where it crosses into the next pool cell
          const int f0 = o0 * rank, nbytes = ncol * rank * 2;
          for (int lo = lane * 1024; lo < nbytes; lo += 32 * 1024) {
            int b = lo;
            const int hi = min(lo + 1024, nbytes);
            while (b < hi) {
              const int f = f0 + (b >> 1), c = f / h_out, off = f - c * h_out;
              const int n = min(hi - b, (h_out - off) * 2);
              bulk_load_1d(stage(s) + (uint32_t)b, w + (int64_t)cells_s[warp][c] * h_out + off, (uint32_t)n,
                           full_bar(s));
              b += n;
            }
          }
          if (first && myrow >= 0)
            bulk_load_1d(stage(s) + kExpWBytes + lane * (kMaxRank * 2), v + (int64_t)myrow * v_pitch,
                         (uint32_t)vk * 2u, full_bar(s));
          if (lane == 0) dec_stamp(8 + 4 * (long long)it + 1);
        }
      }
      if (ok) {
        if ((int)(it % kProducers) == warp) {
          const int s = it % kExpStages;
          if (lane == 0) ok = mbar_wait(empty_bar(s), ((it / kExpStages) & 1) ^ 1, &abort_s);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (ok && lane == 0) {
            infos[s].valid = 0;
            mbar_arrive(full_bar(s));
          }
        }
        ++it;
      }
      if (!ok && warp == 0 && lane == 0) {
        volatile int none = 0;
        const uint32_t first = it > (uint32_t)kExpStages ? it - kExpStages : 0;
        for (uint32_t k = first; k < it; ++k) mbar_wait(full_bar(k % kExpStages), (k / kExpStages) & 1, &none);
      }
    } else {
      // -------------------------------------------------------------- consumers
      const int cw = warp - kProducers;
      float2 vs[kG / 2][8];                              // [token pair][element]: packed for fma.rn.f32x2
      PendingY<T> pend;
      pend.yp[0] = pend.yp[1] = nullptr;
      int buf = 0;
      while (true) {
        const int s = it % kExpStages;
        if (!mbar_wait(full_bar(s), (it / kExpStages) & 1, &abort_s)) break;
        if (cw == 0 && lane == 0) dec_stamp(8 + 4 * (long long)it + 2);
        const uint32_t it_now = it;
        ++it;
        const ExpandInfo& in = infos[s];
        const int valid = in.valid;
        if (valid) {
          const int cpo = in.cpo;
          if (in.first) {
            // this lane's 8 of the r values of every token's V row, scaled
            const int kc = lane % cpo;
            const float scale = in.scale;
#pragma unroll
            for (int h = 0; h < kG / 2; ++h) {
              float a[8], b[8];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const int g = 2 * h + u;
                uint4 raw = make_uint4(0, 0, 0, 0);
                if (g < in.nrows && kc * 8 < in.vk)
                  raw = lds128(stage(s) + kExpWBytes + g * (kMaxRank * 2) + kc * 16);
                unpack8<T>(raw, u == 0 ? a : b);
              }
#pragma unroll
              for (int e = 0; e < 8; ++e) vs[h][e] = make_float2(a[e] * scale, b[e] * scale);
            }
          }
          PendingY<T> cur;
          fetch_y<T>(cur, in, cw, lane, y, h_out);
#define VLR_EXPAND_STAGE(CPO)                                                           \
  if (in.nrows <= 4) expand_stage<T, CPO, 4>(in, stage(s), tile_of(buf, cw), cw, lane, vs); \
  else expand_stage<T, CPO, 8>(in, stage(s), tile_of(buf, cw), cw, lane, vs)
          switch (cpo) {
            case 1: VLR_EXPAND_STAGE(1); break;
            case 2: VLR_EXPAND_STAGE(2); break;
            case 4: VLR_EXPAND_STAGE(4); break;
            case 8: VLR_EXPAND_STAGE(8); break;
            default: VLR_EXPAND_STAGE(16); break;
          }
#undef VLR_EXPAND_STAGE
          // the previous stage's sums meet their Y pieces (requested one stage ago)
          flush_y<T>(pend, tile_of(buf ^ 1, cw));
          pend = cur;
          buf ^= 1;
        } else {
          flush_y<T>(pend, tile_of(buf ^ 1, cw));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(s));
        if (cw == 0 && lane == 0) dec_stamp(8 + 4 * (long long)it_now + 3);
        if (!valid) break;
      }
    }
    __syncthreads();
    if (tid == 0) dec_stamp(2);
    if (abort_s) break;
  }
  if (tid == 0 && abort_s) g_decode_status = 1;
}

}  // namespace

// Drop-in decode call (token mode).  h_in >= h_out: shrink; else expand with the
// punica weight layout.  Arguments were validated by the caller.
int bgmv_decode_launch(void* y, const void* x, const void* w, const void* scales,
                       const int64_t* indicies, int64_t batch, const int64_t* a_start,
                       const int64_t* a_len, const int64_t* a_loc, int64_t qkvo, int h_in, int h_out,
                       int dtype, cudaStream_t stream) {
  // the shared-memory opt-in is per device: one flag per device this process has launched on
  static bool attr_done_dev[64];
  int cur_dev = 0;
  if (cudaGetDevice(&cur_dev) != cudaSuccess || cur_dev < 0 || cur_dev >= 64) return VLR_ERR_RANGE;
  bool& attr_done = attr_done_dev[cur_dev];
  if (!attr_done) {
    cudaError_t e = cudaSuccess;
    auto set = [&](const void* f, int bytes) {
      if (e == cudaSuccess) e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    };
    set((const void*)bgmv_decode_shrink_kernel<__half>, kShrSmem);
    set((const void*)bgmv_decode_shrink_kernel<__nv_bfloat16>, kShrSmem);
    set((const void*)bgmv_decode_expand_kernel<__half>, kExpSmem);
    set((const void*)bgmv_decode_expand_kernel<__nv_bfloat16>, kExpSmem);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_done = true;
  }
  const bool shrink = h_in >= h_out;
  const int64_t n_slices = shrink ? (h_out + kShrSlice - 1) / kShrSlice : (h_out + kExpSlice - 1) / kExpSlice;
  const int64_t items = batch * n_slices;              // upper bound: one group per token
  const unsigned grid = (unsigned)(items < sm_count() ? items : sm_count());
  if (shrink) {
    if (dtype == VLR_F16)
      bgmv_decode_shrink_kernel<__half><<<grid, kDecThreads, kShrSmem, stream>>>(
          (__half*)y, (const __half*)x, (const __half*)w, indicies, batch, a_start, a_len, a_loc, qkvo,
          h_in, h_out);
    else
      bgmv_decode_shrink_kernel<__nv_bfloat16><<<grid, kDecThreads, kShrSmem, stream>>>(
          (__nv_bfloat16*)y, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, indicies, batch, a_start,
          a_len, a_loc, qkvo, h_in, h_out);
  } else {
    if (dtype == VLR_F16)
      bgmv_decode_expand_kernel<__half><<<grid, kDecThreads, kExpSmem, stream>>>(
          (__half*)y, (const __half*)x, (const __half*)w, (const __half*)scales, indicies, batch, a_start,
          a_len, a_loc, qkvo, h_out, h_in);
    else
      bgmv_decode_expand_kernel<__nv_bfloat16><<<grid, kDecThreads, kExpSmem, stream>>>(
          (__nv_bfloat16*)y, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
          (const __nv_bfloat16*)scales, indicies, batch, a_start, a_len, a_loc, qkvo, h_out, h_in);
  }
  return launch_status();
}

void bgmv_decode_set_trace(long long* dev_buffer, long long n) {
  cudaMemcpyToSymbol(g_decode_trace, &dev_buffer, sizeof(dev_buffer));
  cudaMemcpyToSymbol(g_decode_trace_cap, &n, sizeof(n));
}

// 1 if a bounded wait inside a decode kernel gave up since the last reset.
int bgmv_decode_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v) {
    int z = 0;
    cudaMemcpyToSymbol(g_decode_status, &z, sizeof(int));
  }
  return v;
}

}  // namespace vlr
