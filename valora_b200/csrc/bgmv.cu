// Decode gather mat-vec (BGMV) for sm_100a: bandwidth-bound SIMT kernels.
//
// Two addressing modes share the kernels:
//  * token mode  - the drop-in call: adapter = indicies[token].  The tokens of one
//    adapter inside a window of 1024 tokens are served G at a time by the work
//    item of the first of them (the other tokens' items return at once), so an
//    adapter's rows cross L2 -> SM once per G tokens and not once per token;
//  * gather mode - group g is a gather tile of the packed schedule: up to G rows
//    of one adapter, listed in gather_rows, so the adapter's rows are fetched
//    from HBM once per group instead of once per token.
// Every kernel is a persistent loop over work items (problem, group, slice):
// the item count may live on the device (the packer's counts), so the grid is
// sized for the machine, not for the batch.
// Adapter rows are read with 128-bit loads that bypass L1; partial dot products
// are reduced with warp shuffles; accumulation is fp32 with a single rounding.
#include "common.cuh"
#include "problem.cuh"

namespace vlr {

// The tensors one work item touches, from the direct arguments or from the plan.
template <typename T>
struct ProbView {
  T* y;
  const T* x;
  const T* w;
  const int64_t* a_start;
  const int64_t* a_loc;
  int64_t slot;
  int h_in, h_out;
};

template <typename T>
__device__ __forceinline__ ProbView<T> problem_view(const BgmvGroups& g, int problem, T* y,
                                                    const T* x, const T* w, int h_in, int h_out,
                                                    bool expand) {
  ProbView<T> pv;
  if (g.plan != nullptr) {
    const StepProblem& sp = g.plan[problem];
    T* vb = reinterpret_cast<T*>(g.vbuf) + (int64_t)problem * g.vstride;
    if (expand) {
      pv.y = reinterpret_cast<T*>(sp.y); pv.x = vb; pv.w = reinterpret_cast<const T*>(sp.wb);
      pv.a_start = sp.a_start_b; pv.a_loc = sp.a_loc_b; pv.slot = sp.slot_b;
      pv.h_in = kMaxRank; pv.h_out = sp.h_out;
    } else {
      pv.y = vb; pv.x = reinterpret_cast<const T*>(sp.x); pv.w = reinterpret_cast<const T*>(sp.wa);
      pv.a_start = sp.a_start_a; pv.a_loc = sp.a_loc_a; pv.slot = sp.slot_a;
      pv.h_in = sp.h_in; pv.h_out = kMaxRank;
    }
  } else {
    pv.y = y; pv.x = x; pv.w = w; pv.a_start = g.a_start; pv.a_loc = g.a_loc; pv.slot = g.qkvo;
    pv.h_in = h_in; pv.h_out = h_out;
  }
  return pv;
}

// What one CTA needs to know about its current item; filled by thread 0.
template <typename T, int G>
struct Item {
  ProbView<T> pv;
  int adapter, rank, nrows, slice;
  int64_t gbase;                 // a_start[adapter] + rank * slot
  int rows[G];
};

__device__ __forceinline__ int64_t n_groups_of(const BgmvGroups& g) {
  return g.tiles != nullptr ? (int64_t)g.counts[VLR_COUNT_GATHER_TILES] : g.batch;
}

// item -> (problem, group, slice); slices vary fastest so that the CTAs working
// on one group at the same time share its activation rows in L2.
template <typename T, int G>
__device__ __forceinline__ void resolve_item(const BgmvGroups& g, int64_t item, int64_t n_groups,
                                             int n_slices, T* y, const T* x, const T* w, int h_in,
                                             int h_out, bool expand, Item<T, G>* out) {
  Item<T, G> it;
  it.slice = (int)(item % n_slices);
  const int64_t pg = item / n_slices;
  const int gid = (int)(pg % n_groups);
  const int problem = (int)(pg / n_groups);
  it.pv = problem_view<T>(g, problem, y, x, w, h_in, h_out, expand);
  if (g.tiles != nullptr) {
    const int32_t* t = g.tiles + (int64_t)(g.counts[VLR_COUNT_MMA_TILES] + gid) * VLR_TILE_INTS;
    it.adapter = t[1];
    it.rank = t[2];
    it.nrows = min(t[4], G);
    const int first = t[3];
#pragma unroll
    for (int i = 0; i < G; ++i) it.rows[i] = i < it.nrows ? g.gather_rows[first + i] : -1;
  } else {
    it.adapter = (int)g.indicies[gid];
    it.rank = (int)(g.a_len[it.adapter] / 4);
    it.nrows = 1;
#pragma unroll
    for (int i = 0; i < G; ++i) it.rows[i] = i == 0 ? gid : -1;
  }
  if (it.rank < 0 || it.rank > kMaxRank) it.rank = 0;
  it.gbase = it.pv.a_start[it.adapter] + (int64_t)it.rank * it.pv.slot;
  *out = it;
}

constexpr int kThreadsBgmv = 256;
constexpr int kGroupWindow = 1024;                    // tokens searched for same-adapter peers

// Block-wide form of resolve_item; every thread calls it and the result is in
// *out after it returns.  Token mode with G > 1 groups tokens by adapter: the
// block marks the tokens of its window that share the item token's adapter
// (one ballot per 32 tokens), then thread 0 counts those before the token -
// the token leads a group iff that count is a multiple of G - and lists the
// group's rows, in batch order.  Items of tokens that lead no group get nrows 0.
template <typename T, int G>
__device__ __forceinline__ void resolve_block(const BgmvGroups& g, int64_t item, int64_t n_groups,
                                              int n_slices, T* y, const T* x, const T* w, int h_in,
                                              int h_out, bool expand, Item<T, G>* out,
                                              uint32_t* mask_s) {
  const int tid = threadIdx.x, lane = tid & 31;
  if (G == 1 || g.tiles != nullptr) {
    if (tid == 0) resolve_item<T, G>(g, item, n_groups, n_slices, y, x, w, h_in, h_out, expand, out);
    __syncthreads();
    return;
  }
  const int64_t t = (item / n_slices) % n_groups;
  const int64_t w0 = t - t % kGroupWindow;
  const int wn = (int)min((int64_t)kGroupWindow, g.batch - w0);
  const int64_t a = g.indicies[t];
  for (int c0 = tid & ~31; c0 < kGroupWindow; c0 += kThreadsBgmv) {
    const int u = c0 + lane;
    const bool m = u < wn && g.indicies[w0 + u] == a;
    const unsigned b = __ballot_sync(0xffffffffu, m);
    if (lane == 0) mask_s[c0 >> 5] = b;
  }
  __syncthreads();
  if (tid == 0) {
    resolve_item<T, G>(g, item, n_groups, n_slices, y, x, w, h_in, h_out, expand, out);
    const int pos = (int)(t - w0);
    int before = __popc(mask_s[pos >> 5] & ((1u << (pos & 31)) - 1u));
    for (int i = 0; i < (pos >> 5); ++i) before += __popc(mask_s[i]);
    int n = 0;
    if (before % G == 0) {
      int wd = pos >> 5;
      uint32_t bits = mask_s[wd] & ~((1u << (pos & 31)) - 1u);
      while (n < G) {
        while (bits == 0 && ++wd < kGroupWindow / 32) bits = mask_s[wd];
        if (bits == 0) break;
        const int b = __ffs(bits) - 1;
        bits &= bits - 1;
        out->rows[n++] = (int)(w0 + wd * 32 + b);
      }
    }
    for (int i = n; i < G; ++i) out->rows[i] = -1;
    out->nrows = n;
  }
  __syncthreads();
}

constexpr int kWarpsBgmv = kThreadsBgmv / 32;
constexpr int kShrinkKB = 2048;                       // activation elements staged per pass

// y[row, j] = sum_k x[row, k] * W[cell(j), k]   for j < rank        (overwrites)
// R = rank rows per warp; a slice is 8 * R rank rows.
template <typename T, int G, int R>
__global__ void __launch_bounds__(kThreadsBgmv)
bgmv_shrink_kernel(T* __restrict__ y_, const T* __restrict__ x_, const T* __restrict__ w_,
                   BgmvGroups groups, int h_in_, int y_pitch_, int n_slices, int n_problems) {
  __shared__ __align__(16) T xs[G][kShrinkKB];
  __shared__ Item<T, G> item_s;
  __shared__ uint32_t mask_s[kGroupWindow / 32];
  constexpr int kSlice = kWarpsBgmv * R;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t n_groups = n_groups_of(groups);
  const int64_t total = n_groups * n_slices * n_problems;

  for (int64_t item = blockIdx.x; item < total; item += gridDim.x) {
    __syncthreads();                                   // previous item done with item_s / xs
    resolve_block<T, G>(groups, item, n_groups, n_slices, y_, x_, w_, h_in_, y_pitch_, false, &item_s, mask_s);
    const int rank = item_s.rank, nrows = item_s.nrows;
    const int slice0 = item_s.slice * kSlice;
    if (nrows == 0 || slice0 >= rank) continue;
    const T* __restrict__ x = item_s.pv.x;
    const T* __restrict__ w = item_s.pv.w;
    const int h_in = item_s.pv.h_in;

    const T* wrow[R];
    bool live[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int j = slice0 + warp * R + r;
      live[r] = j < rank;
      const int64_t cell = live[r] ? item_s.pv.a_loc[item_s.gbase + j] : 0;
      wrow[r] = w + cell * (int64_t)h_in;
    }
    float acc[R][G];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int g = 0; g < G; ++g) acc[r][g] = 0.f;

    for (int kb = 0; kb < h_in; kb += kShrinkKB) {
      const int kn = min(kShrinkKB, h_in - kb);        // multiple of 8
      if (kb) __syncthreads();
      for (int c = tid; c < G * (kShrinkKB / 8); c += kThreadsBgmv) {
        const int g = c / (kShrinkKB / 8), cc = c % (kShrinkKB / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        const int row = item_s.rows[g];
        if (row >= 0 && cc * 8 < kn) v = ldg128_stream(x + (int64_t)row * h_in + kb + cc * 8);
        *reinterpret_cast<uint4*>(&xs[g][cc * 8]) = v;
      }
      __syncthreads();
      if (live[0]) {
        const int nchunk = kn / 8;
#pragma unroll 2
        for (int c = lane; c < nchunk; c += 32) {
          uint4 wv[R];
#pragma unroll
          for (int r = 0; r < R; ++r)
            wv[r] = live[r] ? ldg128_stream(wrow[r] + kb + c * 8) : make_uint4(0, 0, 0, 0);
          float xf[G][8];
#pragma unroll
          for (int g = 0; g < G; ++g) unpack8<T>(*reinterpret_cast<const uint4*>(&xs[g][c * 8]), xf[g]);
#pragma unroll
          for (int r = 0; r < R; ++r) {
            float wf[8];
            unpack8<T>(wv[r], wf);
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[r][g] = fmaf(wf[e], xf[g][e], acc[r][g]);
          }
        }
      }
    }
    T* __restrict__ y = item_s.pv.y;
    const int y_pitch = item_s.pv.h_out;
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float s = warp_sum(acc[r][g]);
        if (lane == 0 && live[r] && g < nrows) {
          const int j = slice0 + warp * R + r;
          y[(int64_t)item_s.rows[g] * y_pitch + j] = Elem<T>::from_float(s);
        }
      }
  }
}

constexpr int kExpandCols = kThreadsBgmv * 8;         // outputs per item, rows layout

// rows layout: y[row, o] += scale * sum_{k<rank} v[row, k] * B[cell(k), o]
template <typename T, int G>
__global__ void __launch_bounds__(kThreadsBgmv)
bgmv_expand_rows_kernel(T* __restrict__ y_, const T* __restrict__ v_, const T* __restrict__ w_,
                        const T* __restrict__ scales, BgmvGroups groups, int h_out_, int v_pitch_,
                        int n_slices, int n_problems) {
  __shared__ float vs[G][kMaxRank];
  __shared__ int64_t rowoff[kMaxRank];
  __shared__ Item<T, G> item_s;
  __shared__ uint32_t mask_s[kGroupWindow / 32];

  const int tid = threadIdx.x;
  const int64_t n_groups = n_groups_of(groups);
  const int64_t total = n_groups * n_slices * n_problems;

  for (int64_t item = blockIdx.x; item < total; item += gridDim.x) {
    __syncthreads();
    resolve_block<T, G>(groups, item, n_groups, n_slices, y_, v_, w_, v_pitch_, h_out_, true, &item_s, mask_s);
    const int rank = item_s.rank, nrows = item_s.nrows;
    const int h_out = item_s.pv.h_out, v_pitch = item_s.pv.h_in;
    const int o = (item_s.slice * kThreadsBgmv + tid) * 8;
    if (nrows == 0 || rank == 0 || item_s.slice * kExpandCols >= h_out) continue;
    const T* __restrict__ v = item_s.pv.x;
    const T* __restrict__ w = item_s.pv.w;
    const float scale = Elem<T>::to_float(scales[item_s.adapter]);
    for (int i = tid; i < G * kMaxRank; i += kThreadsBgmv) {
      const int g = i / kMaxRank, k = i % kMaxRank;
      float val = 0.f;
      if (g < nrows && k < rank) val = Elem<T>::to_float(v[(int64_t)item_s.rows[g] * v_pitch + k]) * scale;
      vs[g][k] = val;
    }
    for (int k = tid; k < rank; k += kThreadsBgmv)
      rowoff[k] = item_s.pv.a_loc[item_s.gbase + k] * (int64_t)h_out;
    __syncthreads();
    if (o >= h_out) continue;

    float acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;

    for (int k0 = 0; k0 < rank; k0 += 8) {             // rank is a multiple of 8
      uint4 wv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) wv[u] = ldg128_stream(w + rowoff[k0 + u] + o);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        float wf[8];
        unpack8<T>(wv[u], wf);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float vv = vs[g][k0 + u];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(vv, wf[e], acc[g][e]);
        }
      }
    }
    T* __restrict__ y = item_s.pv.y;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (g < nrows) {
        T* yp = y + (int64_t)item_s.rows[g] * h_out + o;
        float yf[8];
        unpack8<T>(ldg128(yp), yf);
#pragma unroll
        for (int e = 0; e < 8; ++e) yf[e] += acc[g][e];
        stg128(yp, pack8<T>(yf));
      }
    }
  }
}

constexpr int kPunicaCols = 256;                      // outputs per item, punica layout

// punica layout: the slot's cells hold the flat bytes of Bt [h_out, rank]:
// element (o, k) is flat f = o*rank + k, in cell f / h_out at offset f % h_out.
template <typename T, int G>
__global__ void __launch_bounds__(kThreadsBgmv)
bgmv_expand_punica_kernel(T* __restrict__ y_, const T* __restrict__ v_, const T* __restrict__ w_,
                          const T* __restrict__ scales, BgmvGroups groups, int h_out_, int v_pitch_,
                          int n_slices, int n_problems) {
  __shared__ float vs[G][kMaxRank];
  __shared__ int64_t rowoff[kMaxRank];
  __shared__ Item<T, G> item_s;
  __shared__ uint32_t mask_s[kGroupWindow / 32];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t n_groups = n_groups_of(groups);
  const int64_t total = n_groups * n_slices * n_problems;

  for (int64_t item = blockIdx.x; item < total; item += gridDim.x) {
    __syncthreads();
    resolve_block<T, G>(groups, item, n_groups, n_slices, y_, v_, w_, v_pitch_, h_out_, true, &item_s, mask_s);
    const int rank = item_s.rank, nrows = item_s.nrows;
    const int h_out = item_s.pv.h_out, v_pitch = item_s.pv.h_in;
    const int o_begin = item_s.slice * kPunicaCols;
    if (nrows == 0 || rank == 0 || o_begin >= h_out) continue;
    const T* __restrict__ v = item_s.pv.x;
    const T* __restrict__ w = item_s.pv.w;
    const float scale = Elem<T>::to_float(scales[item_s.adapter]);
    for (int i = tid; i < G * kMaxRank; i += kThreadsBgmv) {
      const int g = i / kMaxRank, k = i % kMaxRank;
      float val = 0.f;
      if (g < nrows && k < rank) val = Elem<T>::to_float(v[(int64_t)item_s.rows[g] * v_pitch + k]) * scale;
      vs[g][k] = val;
    }
    for (int k = tid; k < rank; k += kThreadsBgmv)
      rowoff[k] = item_s.pv.a_loc[item_s.gbase + k] * (int64_t)h_out;
    __syncthreads();

    // lanes per output: next power of two of rank/8 (1..16)
    const int chunks = rank / 8;
    int lpo = 1;
    while (lpo < chunks) lpo <<= 1;
    const int opw = 32 / lpo;                         // outputs per warp pass
    const int kc = lane % lpo, ol = lane / lpo;
    const bool kvalid = kc < chunks;
    const int o_end = min(o_begin + kPunicaCols, h_out);
    T* __restrict__ y = item_s.pv.y;

    for (int o = o_begin + warp * opw + ol; o - ol < o_end; o += kWarpsBgmv * opw) {
      const bool valid = kvalid && o < o_end;
      float part[G];
#pragma unroll
      for (int g = 0; g < G; ++g) part[g] = 0.f;
      if (valid) {
        const int64_t f = (int64_t)o * rank + kc * 8;
        const int bin = (int)(f / h_out), off = (int)(f % h_out);
        float wf[8];
        unpack8<T>(ldg128_stream(w + rowoff[bin] + off), wf);
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
          for (int e = 0; e < 8; ++e) part[g] = fmaf(vs[g][kc * 8 + e], wf[e], part[g]);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float s = part[g];
        for (int d = lpo >> 1; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
        if (kc == 0 && o < o_end && g < nrows) {
          T* yp = y + (int64_t)item_s.rows[g] * h_out + o;
          *yp = Elem<T>::from_float(Elem<T>::to_float(*yp) + s);
        }
      }
    }
  }
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

// max_groups is a host-side upper bound of the group count (exact in token
// mode); in step mode (groups.plan set) h_in / h_out are maxima over the plan.
template <typename T, int G, int R>
int launch_bgmv(T* y, const T* x, const T* w, const T* scales, const BgmvGroups& groups,
                int64_t max_groups, int h_in, int h_out, int layout, cudaStream_t stream,
                int n_problems) {
  if (max_groups <= 0 || n_problems <= 0) return VLR_OK;
  const int64_t cap = (int64_t)sm_count() * 8;
  auto grid_for = [&](int n_slices) {
    const int64_t items = max_groups * n_slices * n_problems;
    return (unsigned)(items < cap ? items : cap);
  };
  if (h_in >= h_out) {
    const int n_slices = (h_out + kWarpsBgmv * R - 1) / (kWarpsBgmv * R);
    bgmv_shrink_kernel<T, G, R><<<grid_for(n_slices), kThreadsBgmv, 0, stream>>>(
        y, x, w, groups, h_in, h_out, n_slices, n_problems);
  } else if (layout == VLR_LAYOUT_ROWS) {
    const int n_slices = (h_out + kExpandCols - 1) / kExpandCols;
    bgmv_expand_rows_kernel<T, G><<<grid_for(n_slices), kThreadsBgmv, 0, stream>>>(
        y, x, w, scales, groups, h_out, h_in, n_slices, n_problems);
  } else {
    const int n_slices = (h_out + kPunicaCols - 1) / kPunicaCols;
    bgmv_expand_punica_kernel<T, G><<<grid_for(n_slices), kThreadsBgmv, 0, stream>>>(
        y, x, w, scales, groups, h_out, h_in, n_slices, n_problems);
  }
  return launch_status();
}

// Used by the step-level entry point (gather mode, 8 rows per group, 64-row slices).
int bgmv_gather_launch(void* y, const void* x, const void* w, const void* scales,
                       const BgmvGroups& groups, int64_t max_groups, int h_in, int h_out,
                       int layout, int dtype, cudaStream_t stream, int n_problems) {
  if (dtype == VLR_F16)
    return launch_bgmv<__half, 8, 8>((__half*)y, (const __half*)x, (const __half*)w,
                                     (const __half*)scales, groups, max_groups, h_in, h_out,
                                     layout, stream, n_problems);
  return launch_bgmv<__nv_bfloat16, 8, 8>((__nv_bfloat16*)y, (const __nv_bfloat16*)x,
                                          (const __nv_bfloat16*)w, (const __nv_bfloat16*)scales,
                                          groups, max_groups, h_in, h_out, layout, stream,
                                          n_problems);
}

}  // namespace vlr

extern "C" int vlr_bgmv(void* y, const void* x, const void* w, const int64_t* a_start,
                        const int64_t* a_len, const int64_t* a_loc, const int64_t* indicies,
                        int64_t qkvo, const void* lora_scales, int64_t batch, int64_t h_in,
                        int64_t h_out, int dtype, int layout, void* stream) {
  using namespace vlr;
  if (batch == 0) return VLR_OK;
  if (!y || !x || !w || !a_start || !a_len || !a_loc || !indicies) return VLR_ERR_NULL;
  if (dtype != VLR_F16 && dtype != VLR_BF16) return VLR_ERR_DTYPE;
  if (batch < 0 || batch > 0x7fffffff || qkvo < 0) return VLR_ERR_RANGE;
  if (h_in <= 0 || h_out <= 0 || h_in >= 65536 || h_out >= 65536) return VLR_ERR_SHAPE;
  const bool expand = h_in < h_out;
  const int64_t narrow = expand ? h_in : h_out, wide = expand ? h_out : h_in;
  if (wide % 8 != 0 || narrow > kMaxRank) return VLR_ERR_SHAPE;
  if (expand && narrow % 8 != 0) return VLR_ERR_SHAPE;
  if (expand && !lora_scales) return VLR_ERR_NULL;
  if (layout != VLR_LAYOUT_PUNICA && layout != VLR_LAYOUT_ROWS) return VLR_ERR_RANGE;
  if (!aligned16(x) || !aligned16(w) || (expand && !aligned16(y))) return VLR_ERR_ALIGN;
  cudaStream_t s = (cudaStream_t)stream;
  // adapter index per token: the ring kernels group the tokens by adapter themselves
  if (!expand || layout == VLR_LAYOUT_PUNICA)
    return bgmv_decode_launch(y, x, w, lora_scales, indicies, batch, a_start, a_len, a_loc, qkvo,
                              (int)h_in, (int)h_out, dtype, s);
  BgmvGroups g{};
  g.indicies = indicies;
  g.batch = batch;
  g.a_start = a_start;
  g.a_len = a_len;
  g.a_loc = a_loc;
  g.qkvo = qkvo;
  if (dtype == VLR_F16)
    return launch_bgmv<__half, 8, 2>((__half*)y, (const __half*)x, (const __half*)w,
                                     (const __half*)lora_scales, g, batch, (int)h_in, (int)h_out,
                                     layout, s, 1);
  return launch_bgmv<__nv_bfloat16, 8, 2>((__nv_bfloat16*)y, (const __nv_bfloat16*)x,
                                          (const __nv_bfloat16*)w,
                                          (const __nv_bfloat16*)lora_scales, g, batch, (int)h_in,
                                          (int)h_out, layout, s, 1);
}
