// Shared device helpers for the sm_100a kernels: 16-byte vector I/O, dtype packing, reductions,
// host-side launch bookkeeping.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "../../include/mdy_kernels.h"
#include "tunables.h"

namespace mdy {

// ---------------------------------------------------------------------------------------------
// host-side bookkeeping (defined in api.cu)
// ---------------------------------------------------------------------------------------------
void count_launch(int n = 1);
int tunable(int id);
int num_sms();

inline int finish_launch(int nlaunch = 1) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  count_launch(nlaunch);
  return MDY_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename F>
inline int dispatch_dtype(int dtype, F&& f) {
  switch (dtype) {
    case MDY_F32: return f(float{});
    case MDY_F16: return f(__half{});
    case MDY_BF16: return f(__nv_bfloat16{});
    default: return MDY_ERR_DTYPE;
  }
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int next_pow2(int64_t v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

// ---------------------------------------------------------------------------------------------
// element <-> float conversion
// ---------------------------------------------------------------------------------------------
template <typename T> struct VecInfo { static constexpr int kElems = 16 / sizeof(T); };

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Unpack one 16-byte vector into VecInfo<T>::kElems floats.
template <typename T> __device__ __forceinline__ void unpack(const uint4& v, float* f);
template <> __device__ __forceinline__ void unpack<float>(const uint4& v, float* f) {
  f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
  f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}
template <> __device__ __forceinline__ void unpack<__nv_bfloat16>(const uint4& v, float* f) {
  // bf16 -> f32 is a 16-bit shift: the low half of each word is the even element.
  f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
  f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
  f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
template <> __device__ __forceinline__ void unpack<__half>(const uint4& v, float* f) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __half22float2(h[i]);
    f[2 * i] = t.x; f[2 * i + 1] = t.y;
  }
}

// Pack VecInfo<T>::kElems floats (round-to-nearest-even) into one 16-byte vector.
template <typename T> __device__ __forceinline__ uint4 pack(const float* f);
template <> __device__ __forceinline__ uint4 pack<float>(const float* f) {
  return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                    __float_as_uint(f[3]));
}
template <> __device__ __forceinline__ uint4 pack<__nv_bfloat16>(const float* f) {
  uint4 v;
  __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]);
  __nv_bfloat162 b = __floats2bfloat162_rn(f[2], f[3]);
  __nv_bfloat162 c = __floats2bfloat162_rn(f[4], f[5]);
  __nv_bfloat162 d = __floats2bfloat162_rn(f[6], f[7]);
  v.x = *reinterpret_cast<uint32_t*>(&a); v.y = *reinterpret_cast<uint32_t*>(&b);
  v.z = *reinterpret_cast<uint32_t*>(&c); v.w = *reinterpret_cast<uint32_t*>(&d);
  return v;
}
template <> __device__ __forceinline__ uint4 pack<__half>(const float* f) {
  uint4 v;
  __half2 a = __floats2half2_rn(f[0], f[1]);
  __half2 b = __floats2half2_rn(f[2], f[3]);
  __half2 c = __floats2half2_rn(f[4], f[5]);
  __half2 d = __floats2half2_rn(f[6], f[7]);
  v.x = *reinterpret_cast<uint32_t*>(&a); v.y = *reinterpret_cast<uint32_t*>(&b);
  v.z = *reinterpret_cast<uint32_t*>(&c); v.w = *reinterpret_cast<uint32_t*>(&d);
  return v;
}

// ---------------------------------------------------------------------------------------------
// 16-byte global memory access with cache hints
// ---------------------------------------------------------------------------------------------
// Streaming read: data touched once per kernel (evict-first in L2, not kept in L1).
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  return __ldcs(reinterpret_cast<const uint4*>(p));
}
// Read-only data reused by many threads (weights, cos/sin): keep in L1/L2.
__device__ __forceinline__ uint4 ld_reuse(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}
// Plain cached read (default policy).
__device__ __forceinline__ uint4 ld_plain(const void* p) {
  return *reinterpret_cast<const uint4*>(p);
}
// Streaming write (evict-first).
__device__ __forceinline__ void st_stream(void* p, const uint4& v) {
  __stcs(reinterpret_cast<uint4*>(p), v);
}
__device__ __forceinline__ void st_plain(void* p, const uint4& v) {
  *reinterpret_cast<uint4*>(p) = v;
}

// ---------------------------------------------------------------------------------------------
// reductions
// ---------------------------------------------------------------------------------------------
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

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace mdy
