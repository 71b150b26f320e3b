// Shared device helpers for the sm_100a multi-LoRA kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/vlr.h"

namespace vlr {

constexpr int kMaxRank = 128;

template <typename T>
struct Elem;

template <>
struct Elem<__half> {
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<const __half2*>(&u));
  }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
  // one element as the low 16 bits of a register
  static __device__ __forceinline__ float bits_to_float(uint32_t u) { return __half2float(__ushort_as_half((unsigned short)u)); }
  static __device__ __forceinline__ uint32_t float_to_bits(float v) { return __half_as_ushort(__float2half_rn(v)); }
};

template <>
struct Elem<__nv_bfloat16> {
  // bf16 -> fp32 is a 16-bit shift of the bit pattern
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    float2 r;
    r.x = __uint_as_float(u << 16);
    r.y = __uint_as_float(u & 0xffff0000u);
    return r;
  }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float bits_to_float(uint32_t u) { return __uint_as_float(u << 16); }
  static __device__ __forceinline__ uint32_t float_to_bits(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }
};

// 128-bit global load through the read-only path, no L1 allocation: adapter
// rows and activations are streamed once per CTA.
__device__ __forceinline__ uint4 ldg128_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint4 ldg128(const void* p) {
  return *reinterpret_cast<const uint4*>(p);
}

__device__ __forceinline__ void stg128(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

template <typename T>
__device__ __forceinline__ void unpack8(uint4 v, float (&f)[8]) {
  float2 a = Elem<T>::unpack(v.x), b = Elem<T>::unpack(v.y), c = Elem<T>::unpack(v.z),
         d = Elem<T>::unpack(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  v.x = Elem<T>::pack(f[0], f[1]);
  v.y = Elem<T>::pack(f[2], f[3]);
  v.z = Elem<T>::pack(f[4], f[5]);
  v.w = Elem<T>::pack(f[6], f[7]);
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? VLR_OK : static_cast<int>(e);
}

}  // namespace vlr
