// Shared device helpers for the sm_100a kernels of this engine.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "status.h"

namespace lse {

typedef __nv_bfloat16 bf16;

// Fixed-point sums (LSE_FIXED64 in kernels.h): value * 2^24 in a 64-bit integer.
typedef long long fixed64;
constexpr float kFixedScale = 16777216.f;
constexpr float kFixedInverse = 1.f / 16777216.f;
__device__ __forceinline__ float fixed_to_float(fixed64 v) { return (float)v * kFixedInverse; }

template <typename T>
struct Num;

template <>
struct Num<float> {
  static constexpr int kVec = 4;  // elements in a 16-byte vector
  __device__ __forceinline__ static float to_float(float v) { return v; }
  __device__ __forceinline__ static float from_float(float v) { return v; }
};

template <>
struct Num<bf16> {
  static constexpr int kVec = 8;
  __device__ __forceinline__ static float to_float(bf16 v) { return __bfloat162float(v); }
  __device__ __forceinline__ static bf16 from_float(float v) { return __float2bfloat16_rn(v); }
};

template <>
struct Num<fixed64> {
  static constexpr int kVec = 2;
  __device__ __forceinline__ static float to_float(fixed64 v) { return fixed_to_float(v); }
  __device__ __forceinline__ static fixed64 from_float(float v) { return __float2ll_rn(v * kFixedScale); }
};

// 16-byte vector of T, read and written as one transaction.
template <typename T>
struct alignas(16) Vec16 {
  T v[Num<T>::kVec];
};

template <typename T>
__device__ __forceinline__ Vec16<T> load16(const T* p) {
  Vec16<T> r;
  *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
  return r;
}

template <typename T>
__device__ __forceinline__ void store16(T* p, const Vec16<T>& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}

// Four consecutive elements as floats (the address a multiple of four elements' size).
template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void load4<bf16>(const bf16* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
// Fixed-point sums are taken: read, converted, and zeros left behind for the next sums.
template <>
__device__ __forceinline__ void load4<fixed64>(const fixed64* p, float (&v)[4]) {
  longlong2* q = reinterpret_cast<longlong2*>(const_cast<fixed64*>(p));
  const longlong2 a = q[0], b = q[1];
  q[0] = make_longlong2(0, 0);
  q[1] = make_longlong2(0, 0);
  v[0] = fixed_to_float(a.x); v[1] = fixed_to_float(a.y);
  v[2] = fixed_to_float(b.x); v[3] = fixed_to_float(b.y);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<bf16>(bf16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<uint32_t*>(&a);
  t.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a thread block. `scratch` holds at least 32 floats of shared memory. Every thread gets
// the result. The order of the additions depends only on blockDim, never on the data.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  return warp_sum(t);
}

// Page and offset of a token position. page_shift >= 0 when page_tokens is a power of two.
__device__ __forceinline__ void page_of(int pos, int page_tokens, int page_shift, int& idx, int& off) {
  if (page_shift >= 0) {
    idx = pos >> page_shift;
    off = pos & (page_tokens - 1);
  } else {
    idx = pos / page_tokens;
    off = pos - idx * page_tokens;
  }
}

// Programmatic dependent launch. A kernel launched through lse::launch may be scheduled while
// the kernel before it in the stream is still running; it must call pdl_wait() before it touches
// anything that kernel (or any earlier one) wrote, and may do work that depends on nothing first.
// pdl_trigger() lets the *next* kernel in the stream be scheduled early in the same way.
__device__ __forceinline__ void pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

#ifdef __CUDACC__
inline bool pdl_enabled() {
  static const bool on = (getenv("LSE_NO_PDL") == nullptr);
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

}  // namespace lse
