// On-device ragged-batch packing: stable sort of tokens by adapter, run-length
// segments, exclusive-scan offsets and the tile schedule.  Integer work only;
// every output is a pure function of the inputs (no atomics decide an order).
//
// Batches of up to 1024 rows: ONE launch (pack_tiles sorts in shared memory first).  Larger
// ones: four small launches on one stream (nothing has to be cleared ahead of them):
//   1. pack_hist     per-block adapter histograms (blocks of kPackBlock tokens)
//   2. pack_scan     per-adapter exclusive prefix over blocks + adapter bases
//   3. pack_scatter  stable placement: perm and the sorted key array
//   4. pack_tiles    segments, chunks and the tile schedule (one CTA; its working arrays in shared
//                    memory up to 16384 rows, in the workspace above)
// In reference order (sort = 0) only the last one runs.
#include <mutex>

#include "common.cuh"

namespace vlr {

constexpr int kPackBlock = 256;      // tokens per histogram block
constexpr int kPackMaxAdapters = 8192;
constexpr int kScanThreads = 1024;
constexpr int kMaxDevices = 64;
// One CTA does the scans, so every pass over global memory costs the thread a full round trip per
// dependent load: the passes load this many elements ahead of using them (registers: 64 per thread).
constexpr int kScanAhead = 16;                         // pack_scan: blocks per adapter
constexpr int kPosAhead = 8;                           // pack_tiles: sorted positions
constexpr int kChunkAhead = 4;                         // pack_tiles: chunks
constexpr int kPackFusedBits = 13;                     // row index bits of a sort key
constexpr int kPackFusedTokens = 1024;                 // batches up to this size are packed by ONE launch
constexpr int kPackSmemTokens = 16384;                 // up to this size pack_tiles works in shared memory (2-byte indices)
static_assert(kPackFusedTokens <= (1 << kPackFusedBits) && kPackMaxAdapters <= (1 << (32 - kPackFusedBits - 1)),
              "adapter id and row index must fit one 32-bit sort key below the padding value");

struct PackWs {
  int32_t* hist;        // [nblk][n_adapters]
  int32_t* abase;       // [n_adapters]
  int32_t* key;         // [T] sorted keys
  int32_t* chunk_start; // [T+1]
  int32_t* chunk_seg;   // [T]
  int32_t* seg_short;   // [T+1] exclusive short-row prefix per segment
  int32_t* gpos;        // [T] sorted position of each gather row
};

__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static size_t pack_ws_layout(int64_t T, int64_t n_adapters, PackWs* ws, char* base) {
  const int64_t nblk = (T + kPackBlock - 1) / kPackBlock;
  size_t off = 0;
  auto take = [&](int64_t n) {
    int32_t* p = reinterpret_cast<int32_t*>(base + off);
    off = align_up(off + (size_t)n * sizeof(int32_t), 256);
    return p;
  };
  int32_t* hist = take(nblk * n_adapters);
  int32_t* abase = take(n_adapters);
  int32_t* key = take(T);
  int32_t* cs = take(T + 1);
  int32_t* cg = take(T);
  int32_t* ssh = take(T + 1);
  int32_t* gp = take(T);
  if (ws) *ws = PackWs{hist, abase, key, cs, cg, ssh, gp};
  return off;
}

// Ids outside [0, n_adapters) are served as adapter 0; pack_tiles reports them in the status.
__device__ __forceinline__ int clamp_id(int64_t id, int n_adapters) {
  return (id < 0 || id >= n_adapters) ? 0 : (int)id;
}

__global__ void __launch_bounds__(kPackBlock)
pack_hist_kernel(const int64_t* __restrict__ tok, int T, int n_adapters, int32_t* hist) {
  extern __shared__ int32_t sh[];
  for (int a = threadIdx.x; a < n_adapters; a += kPackBlock) sh[a] = 0;
  __syncthreads();
  const int i = blockIdx.x * kPackBlock + threadIdx.x;
  if (i < T) atomicAdd(&sh[clamp_id(tok[i], n_adapters)], 1);
  __syncthreads();
  int32_t* row = hist + (int64_t)blockIdx.x * n_adapters;
  for (int a = threadIdx.x; a < n_adapters; a += kPackBlock) row[a] = sh[a];
}

// Exclusive scan of one int per thread across a 1024-thread block.
__device__ __forceinline__ int block_exscan(int v, int* total, int* warp_sums /*[33]*/) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();                       // protect warp_sums from a previous call
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = lane < (int)(blockDim.x >> 5) ? warp_sums[lane] : 0;
    int winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += n;
    }
    warp_sums[lane] = winc - w;
    if (lane == 31) warp_sums[32] = winc;
  }
  __syncthreads();
  *total = warp_sums[32];
  return warp_sums[warp] + inc - v;
}

__global__ void __launch_bounds__(kScanThreads)
pack_scan_kernel(int nblk, int n_adapters, int32_t* hist, int32_t* abase) {
  __shared__ int warp_sums[33];
  // per-adapter exclusive prefix over blocks; the adapter's total lands in abase
  for (int a = threadIdx.x; a < n_adapters; a += kScanThreads) {
    int run = 0;
    for (int b0 = 0; b0 < nblk; b0 += kScanAhead) {
      int c[kScanAhead];
#pragma unroll
      for (int j = 0; j < kScanAhead; ++j)
        c[j] = b0 + j < nblk ? hist[(int64_t)(b0 + j) * n_adapters + a] : 0;
#pragma unroll
      for (int j = 0; j < kScanAhead; ++j) {
        if (b0 + j < nblk) hist[(int64_t)(b0 + j) * n_adapters + a] = run;
        run += c[j];
      }
    }
    abase[a] = run;
  }
  __syncthreads();
  // exclusive scan of the totals over adapters
  const int per = (n_adapters + kScanThreads - 1) / kScanThreads;
  const int lo = min(threadIdx.x * per, n_adapters), hi = min(lo + per, n_adapters);
  int sum = 0;
  for (int a = lo; a < hi; ++a) sum += abase[a];
  int total;
  int run = block_exscan(sum, &total, warp_sums);
  for (int a = lo; a < hi; ++a) {
    const int c = abase[a];
    abase[a] = run;
    run += c;
  }
}

__global__ void __launch_bounds__(kPackBlock)
pack_scatter_kernel(const int64_t* __restrict__ tok, int T, int n_adapters,
                    const int32_t* __restrict__ hist, const int32_t* __restrict__ abase,
                    int32_t* perm, int32_t* key) {
  __shared__ int keys[kPackBlock];
  const int i = blockIdx.x * kPackBlock + threadIdx.x;
  const int k = i < T ? clamp_id(tok[i], n_adapters) : -1;
  keys[threadIdx.x] = k;
  __syncthreads();
  if (i >= T) return;
  int rank = 0;
  for (int j = 0; j < (int)threadIdx.x; ++j) rank += keys[j] == k;
  const int pos = abase[k] + hist[(int64_t)blockIdx.x * n_adapters + k] + rank;
  perm[pos] = i;
  key[pos] = k;
}

struct PackOut {
  int32_t* perm;
  int64_t* seg_len;
  int64_t* seg_rank;
  int64_t* seg_adapter;
  int64_t* seg_start;
  int32_t* tiles;
  int64_t tiles_cap;
  int32_t* gather_rows;
  int32_t* counts;
};

// One CTA.  Thread t owns the contiguous index range [t*per, (t+1)*per) of
// whatever is being scanned (sorted positions, chunks, segments).
// I = the type of the arrays the passes write and read again (sorted keys and rows, chunk
// starts, chunk segments, short-row prefixes, gather positions).  uint16_t: batches of up to
// kPackSmemTokens rows keep them in shared memory - this one CTA is their only reader, so no
// pass waits for a round trip to L2 (at 16384 rows the kernel took 63 us on the workspace, 43 us so).
// int32_t: larger batches keep them in the workspace.
// An array of pack_tiles.  In shared memory (2-byte elements) thread t walks the elements
// t*per .. t*per+per-1, so at 16 elements per thread the lanes of a warp are 32 bytes apart and
// eight of them meet in every bank: one word of padding per 16 elements spreads them over
// all banks (the tile pass 48 -> 43 us at 16384 rows).
template <typename I>
struct PackArr {
  I* p;
  __device__ __forceinline__ I& operator[](int i) const { return p[sizeof(I) == 2 ? i + ((i >> 4) << 1) : i]; }
};
__host__ __device__ inline int pack_arr_len(int n) { return n + ((n >> 4) << 1) + 2; }

template <typename I>
__global__ void __launch_bounds__(kScanThreads)
pack_tiles_kernel(const int64_t* __restrict__ tok, const int64_t* __restrict__ a_len, int T,
                  int n_adapters, int sorted, int tile_m, int mma_min, int grp, PackWs ws,
                  PackOut out) {
  constexpr bool kSmem = sizeof(I) == 2;
  __shared__ int warp_sums[33];
  __shared__ int s_P, s_C;
  const int tid = threadIdx.x;
  extern __shared__ uint32_t sort_keys[];              // sorted == 2: the batch's (adapter, row) keys come first
  int n2 = 0;
  if (sorted == 2) {
    n2 = 32;
    while (n2 < T) n2 <<= 1;
  }
  PackArr<I> key_a, row_a, cs_a, cg_a, ssh_a, gp_a;
  if constexpr (kSmem) {
    I* sm = reinterpret_cast<I*>(sort_keys + n2);
    const int cap = pack_arr_len(T + 1);
    key_a.p = sm;
    row_a.p = sm + cap;
    cs_a.p = sm + 2 * cap;
    cg_a.p = sm + 3 * cap;
    ssh_a.p = sm + 4 * cap;
    gp_a.p = sm + 5 * cap;
  } else {
    key_a.p = ws.key;
    row_a.p = out.perm;
    cs_a.p = ws.chunk_start;
    cg_a.p = ws.chunk_seg;
    ssh_a.p = ws.seg_short;
    gp_a.p = ws.gpos;
  }

  // every count is written by this kernel (nothing has to be cleared ahead of it); the
  // status starts from the ids themselves
  int bad = 0;
  for (int i = tid; i < T; i += kScanThreads) {
    const int64_t id = tok[i];
    bad |= (id < 0 || id >= n_adapters) ? 1 : 0;
    if (sorted == 0) {                                 // reference order: identity permutation
      out.perm[i] = i;
      key_a[i] = (I)clamp_id(id, n_adapters);
      if constexpr (kSmem) row_a[i] = (I)i;
    } else if (kSmem && sorted == 1) {                 // what pack_scatter placed, brought on chip
      key_a[i] = (I)ws.key[i];
      row_a[i] = (I)out.perm[i];
    }
  }
  bad = __syncthreads_or(bad);
  if (sorted == 2) {
    // Batches of up to kPackFusedTokens rows (decode steps) are sorted right here instead of by
    // the three launches ahead of this one - larger ones are not: at 4096 rows this sort alone
    // takes longer than those launches.  A bitonic sort in shared memory of (adapter << 13 | row),
    // which orders by adapter and keeps the batch order inside an adapter - the same
    // permutation as the stable counting sort, bit for bit.
    for (int i = tid; i < n2; i += kScanThreads)
      sort_keys[i] = i < T ? ((uint32_t)clamp_id(tok[i], n_adapters) << kPackFusedBits) | (uint32_t)i : 0xffffffffu;
    __syncthreads();
    for (int k = 2; k <= n2; k <<= 1) {
      for (int j = k >> 1; j > 0; j >>= 1) {
        for (int i = tid; i < n2; i += kScanThreads) {
          const int p = i ^ j;
          if (p > i) {
            const uint32_t a = sort_keys[i], b = sort_keys[p];
            if ((a > b) == ((i & k) == 0)) {
              sort_keys[i] = b;
              sort_keys[p] = a;
            }
          }
        }
        __syncthreads();
      }
    }
    for (int i = tid; i < T; i += kScanThreads) {
      const int32_t r = (int32_t)(sort_keys[i] & ((1u << kPackFusedBits) - 1u));
      out.perm[i] = r;
      if constexpr (kSmem) row_a[i] = (I)r;
      key_a[i] = (I)(sort_keys[i] >> kPackFusedBits);
    }
    __syncthreads();
  }
  const PackArr<I> key = key_a, row = row_a;

  // ---- pass 1: segment and chunk boundaries over sorted positions.  A chunk is a maximal run of
  // consecutive batch rows inside a segment.
  {
    const int per = (T + kScanThreads - 1) / kScanThreads;
    const int lo = min(tid * per, T), hi = min(lo + per, T);
    // keys and rows of positions b0-1 .. b0+kPosAhead-1 (position -1 reads as "no adapter")
    auto load = [&](int b0, int (&kk)[kPosAhead + 1], int (&rr)[kPosAhead + 1]) {
#pragma unroll
      for (int j = 0; j <= kPosAhead; ++j) {
        const int i = b0 - 1 + j;
        const bool ok = i >= 0 && i < hi;
        kk[j] = ok ? key[i] : -1;
        rr[j] = ok ? row[i] : -2;
      }
    };
    int nseg = 0, nchunk = 0;
    for (int b0 = lo; b0 < hi; b0 += kPosAhead) {
      int kk[kPosAhead + 1], rr[kPosAhead + 1];
      load(b0, kk, rr);
#pragma unroll
      for (int j = 1; j <= kPosAhead; ++j) {
        if (b0 - 1 + j < hi) {
          const bool sflag = kk[j] != kk[j - 1];
          nseg += sflag;
          nchunk += sflag || rr[j] != rr[j - 1] + 1;
        }
      }
    }
    int P, C;
    int sbase = block_exscan(nseg, &P, warp_sums);
    int cbase = block_exscan(nchunk, &C, warp_sums);
    if (tid == 0) { s_P = P; s_C = C; }
    for (int b0 = lo; b0 < hi; b0 += kPosAhead) {
      int kk[kPosAhead + 1], rr[kPosAhead + 1];
      load(b0, kk, rr);
#pragma unroll
      for (int j = 1; j <= kPosAhead; ++j) {
        const int i = b0 - 1 + j;
        if (i < hi) {
          const bool sflag = kk[j] != kk[j - 1];
          const bool cflag = sflag || rr[j] != rr[j - 1] + 1;
          if (sflag) {
            const int a = kk[j];
            out.seg_start[sbase] = i;
            out.seg_adapter[sbase] = a;
            out.seg_rank[sbase] = a_len[a] / 4;
            ++sbase;
          }
          if (cflag) {
            cs_a[cbase] = i;
            cg_a[cbase] = sbase - 1;
            ++cbase;
          }
        }
      }
    }
  }
  __syncthreads();
  const int P = s_P, C = s_C;
  if (tid == 0) {
    out.seg_start[P] = T;
    cs_a[C] = T;
  }
  __syncthreads();
  for (int s = tid; s < P; s += kScanThreads) out.seg_len[s] = out.seg_start[s + 1] - out.seg_start[s];

  // ---- pass 2: per chunk, tensor-core tiles and short (gather) rows
  int n_mma, n_short;
  {
    const int per = (C + kScanThreads - 1) / kScanThreads;
    const int lo = min(tid * per, C), hi = min(lo + per, C);
    int nt = 0, ns = 0;
    for (int b0 = lo; b0 < hi; b0 += kChunkAhead) {
      int cs[kChunkAhead + 1];
#pragma unroll
      for (int j = 0; j <= kChunkAhead; ++j) cs[j] = cs_a[min(b0 + j, hi)];
#pragma unroll
      for (int j = 0; j < kChunkAhead; ++j) {
        const int len = cs[j + 1] - cs[j];           // 0 past the thread's range
        if (len >= mma_min) nt += (len + tile_m - 1) / tile_m; else ns += len;
      }
    }
    int tbase = block_exscan(nt, &n_mma, warp_sums);
    int shbase = block_exscan(ns, &n_short, warp_sums);
    for (int b0 = lo; b0 < hi; b0 += kChunkAhead) {
      int cs[kChunkAhead + 1], sg[kChunkAhead + 1], ka[kChunkAhead], r0[kChunkAhead];
#pragma unroll
      for (int j = 0; j <= kChunkAhead; ++j) cs[j] = cs_a[min(b0 + j, hi)];
#pragma unroll
      for (int j = 0; j <= kChunkAhead; ++j) {       // sg[j]: segment of chunk b0 + j - 1
        const int c = b0 + j - 1;
        sg[j] = (c >= 0 && c < hi) ? cg_a[c] : -1;
      }
#pragma unroll
      for (int j = 0; j < kChunkAhead; ++j) {
        const bool ok = b0 + j < hi;
        ka[j] = ok ? key[cs[j]] : 0;
        r0[j] = ok ? row[cs[j]] : 0;
      }
#pragma unroll
      for (int j = 0; j < kChunkAhead; ++j) {
        if (b0 + j < hi) {
          const int start = cs[j], len = cs[j + 1] - cs[j], seg = sg[j + 1], a = ka[j];
          if (seg != sg[j]) ssh_a[seg] = shbase;   // first chunk of its segment
          if (len >= mma_min) {
            const int rank = (int)(a_len[a] / 4);
            for (int m0 = 0; m0 < len; m0 += tile_m, ++tbase) {
              if (tbase < out.tiles_cap) {
                int32_t* t = out.tiles + (int64_t)tbase * VLR_TILE_INTS;
                t[0] = VLR_TILE_MMA; t[1] = a; t[2] = rank; t[3] = r0[j] + m0;   // a chunk's rows are consecutive
                t[4] = min(tile_m, len - m0); t[5] = seg; t[6] = start + m0; t[7] = 0;
              }
            }
          } else {
            for (int k = 0; k < len; ++k, ++shbase) {
              out.gather_rows[shbase] = r0[j] + k;
              gp_a[shbase] = start + k;
            }
          }
        }
      }
    }
    if (tid == 0) ssh_a[P] = n_short;
  }
  __syncthreads();

  // ---- pass 3: per segment, gather tiles over its (contiguous) short rows
  int n_gather;
  {
    const int per = (P + kScanThreads - 1) / kScanThreads;
    const int lo = min(tid * per, P), hi = min(lo + per, P);
    int ng = 0;
    for (int s = lo; s < hi; ++s) ng += (ssh_a[s + 1] - ssh_a[s] + grp - 1) / grp;
    int gbase = block_exscan(ng, &n_gather, warp_sums);
    for (int s = lo; s < hi; ++s) {
      const int first = ssh_a[s];
      const int cnt = ssh_a[s + 1] - first;
      const int a = (int)out.seg_adapter[s];
      const int rank = (int)out.seg_rank[s];
      for (int g0 = 0; g0 < cnt; g0 += grp, ++gbase) {
        const int64_t ti = (int64_t)n_mma + gbase;
        if (ti < out.tiles_cap) {
          int32_t* t = out.tiles + ti * VLR_TILE_INTS;
          t[0] = VLR_TILE_GATHER; t[1] = a; t[2] = rank; t[3] = first + g0;
          t[4] = min(grp, cnt - g0); t[5] = s; t[6] = gp_a[first + g0]; t[7] = 0;
        }
      }
    }
  }
  if (tid == 0) {
    out.counts[VLR_COUNT_SEGMENTS] = P;
    out.counts[VLR_COUNT_MMA_TILES] = n_mma;
    out.counts[VLR_COUNT_GATHER_TILES] = n_gather;
    out.counts[VLR_COUNT_GATHER_ROWS] = n_short;
    out.counts[VLR_COUNT_STATUS] = ((int64_t)n_mma + n_gather > out.tiles_cap) ? 2 : (bad ? 1 : 0);
    for (int i = VLR_COUNT_STATUS + 1; i < VLR_COUNT_INTS; ++i) out.counts[i] = 0;
  }
}

// The packer's launches on scratch `ws` (caller workspace or the built-in array).
static int pack_launch(const int64_t* tok_adapter, int64_t T, const int64_t* a_len, int64_t n_adapters,
                       int sort, int tile_m, int mma_min_rows, int gather_rows_per_tile,
                       const PackWs& ws, const PackOut& out, cudaStream_t s) {
  const int nblk = (int)((T + kPackBlock - 1) / kPackBlock);
  // the on-chip form of pack_tiles needs more than the default 48 KB of dynamic shared memory
  const size_t smem_arrays = (size_t)6 * pack_arr_len((int)T + 1) * sizeof(uint16_t);
  if (T <= kPackSmemTokens) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDevices) return VLR_ERR_RANGE;
    static std::mutex mu;
    static bool raised[kMaxDevices];
    std::lock_guard<std::mutex> lock(mu);
    if (!raised[dev]) {
      e = cudaFuncSetAttribute((const void*)pack_tiles_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)(6 * pack_arr_len(kPackSmemTokens + 1) * sizeof(uint16_t) + 4 * kPackFusedTokens));
      if (e != cudaSuccess) return static_cast<int>(e);
      raised[dev] = true;
    }
  }
  if (sort && T > 0 && T <= kPackFusedTokens) {
    int n2 = 32;
    while (n2 < T) n2 <<= 1;
    pack_tiles_kernel<uint16_t><<<1, kScanThreads, n2 * sizeof(uint32_t) + smem_arrays, s>>>(
        tok_adapter, a_len, (int)T, (int)n_adapters, 2, tile_m, mma_min_rows, gather_rows_per_tile, ws, out);
    return launch_status();
  }
  if (sort && T > 0) {
    pack_hist_kernel<<<nblk, kPackBlock, n_adapters * sizeof(int32_t), s>>>(
        tok_adapter, (int)T, (int)n_adapters, ws.hist);
    pack_scan_kernel<<<1, kScanThreads, 0, s>>>(nblk, (int)n_adapters, ws.hist, ws.abase);
    pack_scatter_kernel<<<nblk, kPackBlock, 0, s>>>(tok_adapter, (int)T, (int)n_adapters, ws.hist,
                                                    ws.abase, out.perm, ws.key);
  }
  if (T <= kPackSmemTokens)
    pack_tiles_kernel<uint16_t><<<1, kScanThreads, smem_arrays, s>>>(
        tok_adapter, a_len, (int)T, (int)n_adapters, sort && T > 0, tile_m, mma_min_rows, gather_rows_per_tile, ws, out);
  else
    pack_tiles_kernel<int32_t><<<1, kScanThreads, 0, s>>>(
        tok_adapter, a_len, (int)T, (int)n_adapters, sort && T > 0, tile_m, mma_min_rows, gather_rows_per_tile, ws, out);
  return launch_status();
}

// Argument checks shared by the two packer entry points.
static int pack_check(const int64_t* tok_adapter, int64_t T, const int64_t* a_len, int64_t n_adapters,
                      int tile_m, int mma_min_rows, int gather_rows_per_tile, const PackOut& o) {
  if (!a_len || !o.perm || !o.seg_len || !o.seg_rank || !o.seg_adapter || !o.seg_start || !o.tiles ||
      !o.gather_rows || !o.counts)
    return VLR_ERR_NULL;
  if (T > 0 && !tok_adapter) return VLR_ERR_NULL;
  if (T < 0 || T > (1 << 24) || n_adapters <= 0 || n_adapters > kPackMaxAdapters || o.tiles_cap < 0)
    return VLR_ERR_RANGE;
  // a tile is at most one 128-row MMA tile, or 32 gathered rows
  if (tile_m <= 0 || tile_m > 128 || mma_min_rows <= 0 || gather_rows_per_tile <= 0 ||
      gather_rows_per_tile > 32)
    return VLR_ERR_RANGE;
  return VLR_OK;
}

__global__ void var_len_copy_kernel(const int64_t* __restrict__ old_start,
                                    const int64_t* __restrict__ len,
                                    const int64_t* __restrict__ old_loc,
                                    const int64_t* __restrict__ new_start,
                                    int64_t* __restrict__ new_loc) {
  const int64_t i = blockIdx.x;
  const int64_t n = len[i], s = old_start[i], d = new_start[i];
  for (int64_t k = threadIdx.x; k < n; k += blockDim.x) new_loc[d + k] = old_loc[s + k];
}

}  // namespace vlr

extern "C" size_t vlr_pack_workspace_bytes(int64_t T, int64_t n_adapters) {
  if (T < 0 || n_adapters < 0) return 0;
  return vlr::pack_ws_layout(T, n_adapters, nullptr, nullptr) + 256;
}

extern "C" int vlr_pack(const int64_t* tok_adapter, int64_t T, const int64_t* a_len,
                        int64_t n_adapters, int sort, int tile_m, int mma_min_rows,
                        int gather_rows_per_tile, int32_t* perm, int64_t* seg_len,
                        int64_t* seg_rank, int64_t* seg_adapter, int64_t* seg_start,
                        int32_t* tiles, int64_t tiles_cap, int32_t* gather_rows, int32_t* counts,
                        void* workspace, size_t workspace_bytes, void* stream) {
  using namespace vlr;
  PackOut out{perm, seg_len, seg_rank, seg_adapter, seg_start, tiles, tiles_cap, gather_rows, counts};
  int rc = pack_check(tok_adapter, T, a_len, n_adapters, tile_m, mma_min_rows, gather_rows_per_tile, out);
  if (rc != VLR_OK) return rc;
  if (!workspace) return VLR_ERR_NULL;
  char* base = reinterpret_cast<char*>(align_up(reinterpret_cast<uintptr_t>(workspace), 256));
  const size_t slack = base - reinterpret_cast<char*>(workspace);
  PackWs ws;
  const size_t need = pack_ws_layout(T, n_adapters, &ws, base);
  if (need + slack > workspace_bytes) return VLR_ERR_WORKSPACE;
  return pack_launch(tok_adapter, T, a_len, n_adapters, sort, tile_m, mma_min_rows,
                     gather_rows_per_tile, ws, out, (cudaStream_t)stream);
}

extern "C" int vlr_var_len_copy(const int64_t* old_start, const int64_t* len,
                                const int64_t* old_loc, const int64_t* new_start,
                                int64_t* new_loc, int64_t n, void* stream) {
  if (n == 0) return VLR_OK;
  if (!old_start || !len || !old_loc || !new_start || !new_loc) return VLR_ERR_NULL;
  if (n < 0 || n > 0x7fffffff) return VLR_ERR_RANGE;
  vlr::var_len_copy_kernel<<<(unsigned)n, 256, 0, (cudaStream_t)stream>>>(old_start, len, old_loc,
                                                                         new_start, new_loc);
  return vlr::launch_status();
}

// ----------------------------------------------------------------------------
// vlr_pack_static: the packer for callers that cannot hand over scratch memory.
//
// Who that is: a serving step that runs after its memory pool has claimed the
// device's free HBM (the reference sizes its unified KV/adapter pool from what
// is left on the GPU, so a later cudaMalloc can simply fail), and host code
// reached through an FFI that owns no allocator handle and must not trigger the
// device-wide synchronisation cudaMalloc / cudaFree imply in the middle of a
// step.  For them the packer's scratch lives in this library's image: one
// 1 MiB array per GPU that loads the library, held until the process exits.
//
// Limits: T <= 8192 tokens and n_adapters <= 1024 per call (larger batches are
// refused with VLR_ERR_STATIC_LIMIT; use vlr_pack with a caller workspace).
// The array is shared by every call on the device and keeps the previous
// call's bytes.  Nothing in it has to start at zero: the histogram rows are
// written in full before they are read, every other array is written before it
// is read within the call.  Two calls whose kernels overlap on the GPU (two
// streams, two threads) race on the array; serialise them on one stream.
// The first call on each device looks the array's device address up
// (cudaGetSymbolAddress) and caches it; make that first call before any
// stream capture begins.  No cudaMalloc, cudaFree or other allocating call
// is made here.
namespace vlr {

constexpr int64_t kStaticMaxTokens = 8192;
constexpr int64_t kStaticMaxAdapters = 1024;
constexpr size_t kStaticScratchBytes = 1u << 20;

static __device__ __align__(256) unsigned char g_pack_scratch[kStaticScratchBytes];

static std::mutex g_scratch_mu;
static unsigned char* g_scratch_ptr[kMaxDevices];   // device address of g_pack_scratch, per device

// In host code `g_pack_scratch` is only a handle for the runtime, not a device
// address: the address is asked for once per device, with that device current.
static int static_scratch(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return VLR_ERR_RANGE;
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_pack_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (p == nullptr) return VLR_ERR_DRIVER;
    g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_ptr[dev];
  return VLR_OK;
}

}  // namespace vlr

extern "C" int vlr_pack_static(const int64_t* tok_adapter, int64_t T, const int64_t* a_len,
                               int64_t n_adapters, int sort, int tile_m, int mma_min_rows,
                               int gather_rows_per_tile, int32_t* perm, int64_t* seg_len,
                               int64_t* seg_rank, int64_t* seg_adapter, int64_t* seg_start,
                               int32_t* tiles, int64_t tiles_cap, int32_t* gather_rows,
                               int32_t* counts, void* stream) {
  using namespace vlr;
  PackOut out{perm, seg_len, seg_rank, seg_adapter, seg_start, tiles, tiles_cap, gather_rows, counts};
  int rc = pack_check(tok_adapter, T, a_len, n_adapters, tile_m, mma_min_rows, gather_rows_per_tile, out);
  if (rc != VLR_OK) return rc;
  if (T > kStaticMaxTokens || n_adapters > kStaticMaxAdapters) return VLR_ERR_STATIC_LIMIT;
  unsigned char* scratch = nullptr;
  rc = static_scratch(&scratch);
  if (rc != VLR_OK) return rc;
  PackWs ws;
  const size_t need = pack_ws_layout(T, n_adapters, &ws, reinterpret_cast<char*>(scratch));
  if (need > kStaticScratchBytes) return VLR_ERR_STATIC_LIMIT;
  return pack_launch(tok_adapter, T, a_len, n_adapters, sort, tile_m, mma_min_rows,
                     gather_rows_per_tile, ws, out, (cudaStream_t)stream);
}
