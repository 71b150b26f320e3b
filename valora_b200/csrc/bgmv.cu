// Decode gather mat-vec (BGMV) for sm_100a: bandwidth-bound SIMT kernels.
//
// Two addressing modes share the kernels:
//  * token mode  - group g is token g, adapter = indicies[g] (the drop-in call);
//  * gather mode - group g is a gather tile of the packed schedule: up to G rows
//    of one adapter, listed in gather_rows, so the adapter's rows are fetched
//    from HBM once per group instead of once per token.
// Adapter rows are read with 128-bit loads that bypass L1; partial dot products
// are reduced with warp shuffles; accumulation is fp32 with a single rounding.
#include "common.cuh"
#include "problem.cuh"

namespace vlr {

// The tensors one CTA works on, from the direct arguments or from the plan.
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
__device__ __forceinline__ ProbView<T> problem_view(const BgmvGroups& g, T* y, const T* x, const T* w,
                                                    int h_in, int h_out, bool expand) {
  ProbView<T> pv;
  if (g.plan != nullptr) {
    const StepProblem& sp = g.plan[blockIdx.z];
    T* vb = reinterpret_cast<T*>(g.vbuf) + (int64_t)blockIdx.z * g.vstride;
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

template <int G>
struct Group {
  int adapter, rank, nrows;
};

// Resolve the calling CTA's group into shared memory.  Returns false if the CTA
// has no work.  rows[] receives the token rows (G entries, -1 padded).
template <int G>
__device__ __forceinline__ bool resolve_group(const BgmvGroups& g, int gid, Group<G>& out,
                                              int* rows) {
  if (g.tiles != nullptr) {
    const int n_gather = g.counts[VLR_COUNT_GATHER_TILES];
    if (gid >= n_gather) return false;
    const int32_t* t = g.tiles + (int64_t)(g.counts[VLR_COUNT_MMA_TILES] + gid) * VLR_TILE_INTS;
    out.adapter = t[1];
    out.rank = t[2];
    out.nrows = min(t[4], G);
    const int first = t[3];
#pragma unroll
    for (int i = 0; i < G; ++i) rows[i] = i < out.nrows ? g.gather_rows[first + i] : -1;
  } else {
    if (gid >= g.batch) return false;
    out.adapter = (int)g.indicies[gid];
    out.rank = (int)(g.a_len[out.adapter] / 4);
    out.nrows = 1;
#pragma unroll
    for (int i = 0; i < G; ++i) rows[i] = i == 0 ? gid : -1;
  }
  return true;
}

constexpr int kShrinkThreads = 256;
constexpr int kShrinkWarps = kShrinkThreads / 32;
constexpr int kShrinkRows = 2;                        // rank rows per warp
constexpr int kShrinkSlice = kShrinkWarps * kShrinkRows;
constexpr int kShrinkKB = 2048;                       // activation elements staged per pass

// y[row, j] = sum_k x[row, k] * W[cell(j), k]   for j < rank        (overwrites)
template <typename T, int G>
__global__ void __launch_bounds__(kShrinkThreads)
bgmv_shrink_kernel(T* __restrict__ y_, const T* __restrict__ x_, const T* __restrict__ w_,
                   BgmvGroups groups, int h_in_, int y_pitch_) {
  const ProbView<T> pv = problem_view<T>(groups, y_, x_, w_, h_in_, y_pitch_, false);
  T* __restrict__ y = pv.y;
  const T* __restrict__ x = pv.x;
  const T* __restrict__ w = pv.w;
  const int h_in = pv.h_in, y_pitch = pv.h_out;
  __shared__ __align__(16) T xs[G][kShrinkKB];
  __shared__ int rows_s[G];
  __shared__ Group<G> grp_s;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    Group<G> gr;
    int rows[G];
    bool ok = resolve_group<G>(groups, blockIdx.x, gr, rows);
    if (!ok) gr.nrows = 0;
    grp_s = gr;
#pragma unroll
    for (int i = 0; i < G; ++i) rows_s[i] = rows[i];
  }
  __syncthreads();
  const Group<G> gr = grp_s;
  const int slice0 = blockIdx.y * kShrinkSlice;
  if (gr.nrows == 0 || slice0 >= gr.rank) return;
  const int64_t gbase = pv.a_start[gr.adapter] + (int64_t)gr.rank * pv.slot;

  // this warp's rank rows
  const T* wrow[kShrinkRows];
  bool live[kShrinkRows];
#pragma unroll
  for (int r = 0; r < kShrinkRows; ++r) {
    const int j = slice0 + warp * kShrinkRows + r;
    live[r] = j < gr.rank;
    const int64_t cell = live[r] ? pv.a_loc[gbase + j] : 0;
    wrow[r] = w + cell * (int64_t)h_in;
  }

  float acc[kShrinkRows][G];
#pragma unroll
  for (int r = 0; r < kShrinkRows; ++r)
#pragma unroll
    for (int g = 0; g < G; ++g) acc[r][g] = 0.f;

  for (int kb = 0; kb < h_in; kb += kShrinkKB) {
    const int kn = min(kShrinkKB, h_in - kb);          // multiple of 8
    // stage the group's activation rows
    for (int c = tid; c < G * (kShrinkKB / 8); c += kShrinkThreads) {
      const int g = c / (kShrinkKB / 8), cc = c % (kShrinkKB / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      const int row = rows_s[g];
      if (row >= 0 && cc * 8 < kn) v = ldg128_stream(x + (int64_t)row * h_in + kb + cc * 8);
      *reinterpret_cast<uint4*>(&xs[g][cc * 8]) = v;
    }
    __syncthreads();
    if (live[0]) {
      const int nchunk = kn / 8;
#pragma unroll 4
      for (int c = lane; c < nchunk; c += 32) {
        uint4 wv[kShrinkRows];
#pragma unroll
        for (int r = 0; r < kShrinkRows; ++r)
          wv[r] = live[r] ? ldg128_stream(wrow[r] + kb + c * 8) : make_uint4(0, 0, 0, 0);
        float wf[kShrinkRows][8];
#pragma unroll
        for (int r = 0; r < kShrinkRows; ++r) unpack8<T>(wv[r], wf[r]);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float xf[8];
          unpack8<T>(*reinterpret_cast<const uint4*>(&xs[g][c * 8]), xf);
#pragma unroll
          for (int r = 0; r < kShrinkRows; ++r)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[r][g] = fmaf(wf[r][e], xf[e], acc[r][g]);
        }
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int r = 0; r < kShrinkRows; ++r)
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float s = warp_sum(acc[r][g]);
      if (lane == 0 && live[r] && g < gr.nrows) {
        const int j = slice0 + warp * kShrinkRows + r;
        y[(int64_t)rows_s[g] * y_pitch + j] = Elem<T>::from_float(s);
      }
    }
}

constexpr int kExpandThreads = 256;
constexpr int kExpandCols = kExpandThreads * 8;       // outputs per CTA, rows layout

// rows layout: y[row, o] += scale * sum_{k<rank} v[row, k] * B[cell(k), o]
template <typename T, int G>
__global__ void __launch_bounds__(kExpandThreads)
bgmv_expand_rows_kernel(T* __restrict__ y_, const T* __restrict__ v_, const T* __restrict__ w_,
    const T* __restrict__ scales, BgmvGroups groups, int h_out_, int v_pitch_) {
  const ProbView<T> pv = problem_view<T>(groups, y_, v_, w_, v_pitch_, h_out_, true);
  T* __restrict__ y = pv.y;
  const T* __restrict__ v = pv.x;
  const T* __restrict__ w = pv.w;
  const int h_out = pv.h_out, v_pitch = pv.h_in;
  __shared__ float vs[G][kMaxRank];
  __shared__ int64_t rowoff[kMaxRank];
  __shared__ int rows_s[G];
  __shared__ Group<G> grp_s;

  const int tid = threadIdx.x;
  if (tid == 0) {
    Group<G> gr;
    int rows[G];
    bool ok = resolve_group<G>(groups, blockIdx.x, gr, rows);
    if (!ok) gr.nrows = 0;
    grp_s = gr;
#pragma unroll
    for (int i = 0; i < G; ++i) rows_s[i] = rows[i];
  }
  __syncthreads();
  const Group<G> gr = grp_s;
  if (gr.nrows == 0 || gr.rank == 0) return;
  const int64_t gbase = pv.a_start[gr.adapter] + (int64_t)gr.rank * pv.slot;
  const float scale = Elem<T>::to_float(scales[gr.adapter]);
  for (int i = tid; i < G * kMaxRank; i += kExpandThreads) {
    const int g = i / kMaxRank, k = i % kMaxRank;
    float val = 0.f;
    if (g < gr.nrows && k < gr.rank)
      val = Elem<T>::to_float(v[(int64_t)rows_s[g] * v_pitch + k]) * scale;
    vs[g][k] = val;
  }
  for (int k = tid; k < gr.rank; k += kExpandThreads)
    rowoff[k] = pv.a_loc[gbase + k] * (int64_t)h_out;
  __syncthreads();

  const int o = (blockIdx.y * kExpandThreads + tid) * 8;
  if (o >= h_out) return;

  float acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;

  for (int k0 = 0; k0 < gr.rank; k0 += 8) {           // rank is a multiple of 8
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
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (g < gr.nrows) {
      T* yp = y + (int64_t)rows_s[g] * h_out + o;
      float yf[8];
      unpack8<T>(ldg128(yp), yf);
#pragma unroll
      for (int e = 0; e < 8; ++e) yf[e] += acc[g][e];
      stg128(yp, pack8<T>(yf));
    }
  }
}

constexpr int kPunicaCols = 256;                      // outputs per CTA, punica layout

// punica layout: the slot's cells hold the flat bytes of Bt [h_out, rank]:
// element (o, k) is flat f = o*rank + k, in cell f / h_out at offset f % h_out.
template <typename T, int G>
__global__ void __launch_bounds__(kExpandThreads)
bgmv_expand_punica_kernel(T* __restrict__ y_, const T* __restrict__ v_, const T* __restrict__ w_,
    const T* __restrict__ scales, BgmvGroups groups, int h_out_, int v_pitch_) {
  const ProbView<T> pv = problem_view<T>(groups, y_, v_, w_, v_pitch_, h_out_, true);
  T* __restrict__ y = pv.y;
  const T* __restrict__ v = pv.x;
  const T* __restrict__ w = pv.w;
  const int h_out = pv.h_out, v_pitch = pv.h_in;
  __shared__ float vs[G][kMaxRank];
  __shared__ int64_t rowoff[kMaxRank];
  __shared__ int rows_s[G];
  __shared__ Group<G> grp_s;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    Group<G> gr;
    int rows[G];
    bool ok = resolve_group<G>(groups, blockIdx.x, gr, rows);
    if (!ok) gr.nrows = 0;
    grp_s = gr;
#pragma unroll
    for (int i = 0; i < G; ++i) rows_s[i] = rows[i];
  }
  __syncthreads();
  const Group<G> gr = grp_s;
  if (gr.nrows == 0 || gr.rank == 0) return;
  const int64_t gbase = pv.a_start[gr.adapter] + (int64_t)gr.rank * pv.slot;
  const float scale = Elem<T>::to_float(scales[gr.adapter]);
  for (int i = tid; i < G * kMaxRank; i += kExpandThreads) {
    const int g = i / kMaxRank, k = i % kMaxRank;
    float val = 0.f;
    if (g < gr.nrows && k < gr.rank)
      val = Elem<T>::to_float(v[(int64_t)rows_s[g] * v_pitch + k]) * scale;
    vs[g][k] = val;
  }
  for (int k = tid; k < gr.rank; k += kExpandThreads)
    rowoff[k] = pv.a_loc[gbase + k] * (int64_t)h_out;
  __syncthreads();

  // lanes per output: next power of two of rank/8 (1..16)
  const int chunks = gr.rank / 8;
  int lpo = 1;
  while (lpo < chunks) lpo <<= 1;
  const int opw = 32 / lpo;                           // outputs per warp pass
  const int kc = lane % lpo, ol = lane / lpo;
  const bool kvalid = kc < chunks;
  const int o_begin = blockIdx.y * kPunicaCols;
  const int o_end = min(o_begin + kPunicaCols, h_out);

  for (int o = o_begin + warp * opw + ol; o - ol < o_end; o += (kExpandThreads / 32) * opw) {
    const bool valid = kvalid && o < o_end;
    float part[G];
#pragma unroll
    for (int g = 0; g < G; ++g) part[g] = 0.f;
    if (valid) {
      const int64_t f = (int64_t)o * gr.rank + kc * 8;
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
      if (kc == 0 && o < o_end && g < gr.nrows) {
        T* yp = y + (int64_t)rows_s[g] * h_out + o;
        *yp = Elem<T>::from_float(Elem<T>::to_float(*yp) + s);
      }
    }
  }
}

// In step mode (groups.plan set) h_in / h_out are the maxima over the plan's
// problems (they size grid.y) and n_problems is grid.z.
template <typename T, int G>
int launch_bgmv(T* y, const T* x, const T* w, const T* scales, const BgmvGroups& groups,
                int64_t n_groups, int h_in, int h_out, int layout, cudaStream_t stream,
                int n_problems = 1) {
  if (n_groups <= 0 || n_problems <= 0) return VLR_OK;
  if (h_in >= h_out) {
    dim3 grid((unsigned)n_groups, (h_out + kShrinkSlice - 1) / kShrinkSlice, n_problems);
    bgmv_shrink_kernel<T, G><<<grid, kShrinkThreads, 0, stream>>>(y, x, w, groups, h_in, h_out);
  } else if (layout == VLR_LAYOUT_ROWS) {
    dim3 grid((unsigned)n_groups, (h_out + kExpandCols - 1) / kExpandCols, n_problems);
    bgmv_expand_rows_kernel<T, G><<<grid, kExpandThreads, 0, stream>>>(y, x, w, scales, groups,
                                                                      h_out, h_in);
  } else {
    dim3 grid((unsigned)n_groups, (h_out + kPunicaCols - 1) / kPunicaCols, n_problems);
    bgmv_expand_punica_kernel<T, G><<<grid, kExpandThreads, 0, stream>>>(y, x, w, scales, groups,
                                                                        h_out, h_in);
  }
  return launch_status();
}

// Used by the step-level entry point (gather mode, G = 8).
int bgmv_gather_launch(void* y, const void* x, const void* w, const void* scales,
                       const BgmvGroups& groups, int64_t max_groups, int h_in, int h_out,
                       int layout, int dtype, cudaStream_t stream, int n_problems) {
  if (dtype == VLR_F16)
    return launch_bgmv<__half, 8>((__half*)y, (const __half*)x, (const __half*)w,
                                  (const __half*)scales, groups, max_groups, h_in, h_out, layout,
                                  stream, n_problems);
  return launch_bgmv<__nv_bfloat16, 8>((__nv_bfloat16*)y, (const __nv_bfloat16*)x,
                                       (const __nv_bfloat16*)w, (const __nv_bfloat16*)scales,
                                       groups, max_groups, h_in, h_out, layout, stream, n_problems);
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
  BgmvGroups g{};
  g.indicies = indicies;
  g.batch = batch;
  g.a_start = a_start;
  g.a_len = a_len;
  g.a_loc = a_loc;
  g.qkvo = qkvo;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == VLR_F16)
    return launch_bgmv<__half, 1>((__half*)y, (const __half*)x, (const __half*)w,
                                  (const __half*)lora_scales, g, batch, (int)h_in, (int)h_out,
                                  layout, s);
  return launch_bgmv<__nv_bfloat16, 1>((__nv_bfloat16*)y, (const __nv_bfloat16*)x,
                                       (const __nv_bfloat16*)w, (const __nv_bfloat16*)lora_scales,
                                       g, batch, (int)h_in, (int)h_out, layout, s);
}
