// Row-wise max / min with indices for sm_100a.
//
// One pass over HBM.  A row is scanned by a group of G lanes (G = 4..32, several rows per warp when rows
// are short) or by a whole 256-thread CTA (rows longer than 8192 elements), with U 16-byte loads in
// flight per thread.  The hot loop only reduces each vector to its extreme with packed, NaN-propagating
// max/min instructions and keeps, branch-free, the first vector that beats the thread's best so far; that
// one vector is looked at again after the loop to find the element.
// Lanes and warps are combined with a "better" rule that prefers the smaller index on ties, so the
// result is the first position of the extreme; a NaN counts as the extreme for both max and min
// (what torch.max / torch.min return).
#include <math.h>
#include "common.cuh"

namespace mdy {
namespace {

__device__ __forceinline__ float max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float min_nan(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// extreme of the elements of one vector; NaN if any element is NaN
template <typename T, bool MIN> __device__ __forceinline__ float vec_extreme(const uint4& q);
template <> __device__ __forceinline__ float vec_extreme<float, false>(const uint4& q) {
  return max_nan(max_nan(__uint_as_float(q.x), __uint_as_float(q.y)), max_nan(__uint_as_float(q.z), __uint_as_float(q.w)));
}
template <> __device__ __forceinline__ float vec_extreme<float, true>(const uint4& q) {
  return min_nan(min_nan(__uint_as_float(q.x), __uint_as_float(q.y)), min_nan(__uint_as_float(q.z), __uint_as_float(q.w)));
}
template <> __device__ __forceinline__ float vec_extreme<__nv_bfloat16, false>(const uint4& q) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
  const __nv_bfloat162 a = __hmax2_nan(__hmax2_nan(h[0], h[1]), __hmax2_nan(h[2], h[3]));
  return max_nan(__low2float(a), __high2float(a));
}
template <> __device__ __forceinline__ float vec_extreme<__nv_bfloat16, true>(const uint4& q) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
  const __nv_bfloat162 a = __hmin2_nan(__hmin2_nan(h[0], h[1]), __hmin2_nan(h[2], h[3]));
  return min_nan(__low2float(a), __high2float(a));
}
template <> __device__ __forceinline__ float vec_extreme<__half, false>(const uint4& q) {
  const __half2* h = reinterpret_cast<const __half2*>(&q);
  const __half2 a = __hmax2_nan(__hmax2_nan(h[0], h[1]), __hmax2_nan(h[2], h[3]));
  return max_nan(__low2float(a), __high2float(a));
}
template <> __device__ __forceinline__ float vec_extreme<__half, true>(const uint4& q) {
  const __half2* h = reinterpret_cast<const __half2*>(&q);
  const __half2 a = __hmin2_nan(__hmin2_nan(h[0], h[1]), __hmin2_nan(h[2], h[3]));
  return min_nan(__low2float(a), __high2float(a));
}

// is (a, ia) to be preferred over (b, ib)?  NaN beats numbers, ties go to the smaller index
template <bool MIN>
__device__ __forceinline__ bool better(float a, int ia, float b, int ib) {
  const bool an = a != a, bn = b != b;
  if (an || bn) return an && (!bn || ia < ib);
  if (a == b) return ia < ib;
  return MIN ? a < b : a > b;
}

// combine over groups of W adjacent lanes; every lane of a group ends with the group's result
template <bool MIN, int W>
__device__ __forceinline__ void group_best(float& v, int& i) {
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (better<MIN>(ov, oi, v, i)) { v = ov; i = oi; }
  }
}

// Scan elements [0, N) of one row with `nthr` cooperating threads (this thread is number `t`).  A
// thread visits its vectors in increasing index order and remembers, without branching, the first vector
// whose extreme beats everything before it; afterwards it re-reads that one vector (an L1/L2 hit) to find
// the element.  Elements past the last whole vector, and rows that cannot be read as vectors, go
// through the scalar rule.
template <typename T, bool MIN, int U>
__device__ __forceinline__ void scan_row(const T* __restrict__ x, int N, bool vec_ok, int t, int nthr, float& best,
                                         int& bidx) {
  constexpr int VE = VecInfo<T>::kElems;
  best = MIN ? INFINITY : -INFINITY;
  bidx = INT_MAX;
  int tail = 0;
  if (vec_ok) {
    const int nvec = N / VE;
    int bvec = -1;
    for (int i0 = t; i0 < nvec; i0 += nthr * U) {
      uint4 v[U];
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const int i = i0 + k * nthr;
        if (i < nvec) v[k] = ld_stream(x + (int64_t)i * VE);
      }
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const int i = i0 + k * nthr;
        if (i < nvec) {
          const float e = vec_extreme<T, MIN>(v[k]);
          // a NaN once found stays; otherwise a strictly better vector (or a NaN, or the first one) is taken
          const bool take = best == best && (!(MIN ? e >= best : e <= best) || bvec < 0);
          best = take ? e : best;
          bvec = take ? i : bvec;
        }
      }
    }
    if (bvec >= 0) {
      float f[VE];
      unpack<T>(ld_plain(x + (int64_t)bvec * VE), f);
      const bool want_nan = best != best;
      float hit = best;  // the element itself (keeps the sign of a zero)
#pragma unroll
      for (int j = VE - 1; j >= 0; --j)
        if (want_nan ? f[j] != f[j] : f[j] == best) { bidx = bvec * VE + j; hit = f[j]; }
      best = hit;
    }
    tail = nvec * VE;
  }
  for (int i = tail + t; i < N; i += nthr) {
    const float f = to_float(x[i]);
    if (best == best && (f != f || (MIN ? f < best : f > best) || bidx == INT_MAX)) { best = f; bidx = i; }
  }
}

// G lanes per row, 256 / G rows per CTA pass, grid-stride over row groups.
template <typename T, bool MIN, int G>
__global__ void __launch_bounds__(256) extreme_group_rows(const T* __restrict__ x, T* __restrict__ values,
                                                         int64_t* __restrict__ indices, int64_t M, int N,
                                                         int64_t rs, int vec_ok) {
  constexpr int RPC = 256 / G;
  const int t = threadIdx.x % G, r = threadIdx.x / G;
  // all lanes of a warp stay in the loop together (the shuffles need them): rows past M are skipped inside
  for (int64_t base = (int64_t)blockIdx.x * RPC; base < M; base += (int64_t)gridDim.x * RPC) {
    const int64_t row = base + r;
    float best = MIN ? INFINITY : -INFINITY;
    int bidx = INT_MAX;
    if (row < M) scan_row<T, MIN, 4>(x + row * rs, N, vec_ok != 0, t, G, best, bidx);
    group_best<MIN, G>(best, bidx);
    if (row < M && t == 0) { values[row] = from_float<T>(best); indices[row] = bidx; }
  }
}

template <typename T, bool MIN>
__global__ void __launch_bounds__(256) extreme_cta_rows(const T* __restrict__ x, T* __restrict__ values,
                                                       int64_t* __restrict__ indices, int64_t M, int N,
                                                       int64_t rs, int vec_ok) {
  __shared__ float sv[8];
  __shared__ int si[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    float best;
    int bidx;
    scan_row<T, MIN, 8>(x + row * rs, N, vec_ok != 0, threadIdx.x, 256, best, bidx);
    group_best<MIN, 32>(best, bidx);
    if (lane == 0) { sv[warp] = best; si[warp] = bidx; }
    __syncthreads();
    if (warp == 0) {
      best = lane < 8 ? sv[lane] : (MIN ? INFINITY : -INFINITY);
      bidx = lane < 8 ? si[lane] : INT_MAX;
      group_best<MIN, 8>(best, bidx);
      if (lane == 0) { values[row] = from_float<T>(best); indices[row] = bidx; }
    }
    __syncthreads();
  }
}

template <typename T, bool MIN>
int launch_extreme(const T* x, T* values, int64_t* indices, int64_t M, int N, int64_t rs, int vec_ok, cudaStream_t st) {
  constexpr int VE = VecInfo<T>::kElems;
  const int64_t cap = (int64_t)num_sms() * 8;
  if (N > 8192) {
    const unsigned grid = (unsigned)(M < cap ? M : cap);
    extreme_cta_rows<T, MIN><<<grid, 256, 0, st>>>(x, values, indices, M, N, rs, vec_ok);
    return finish_launch(1);
  }
  // lanes per row: about eight vectors per lane, at least 4 lanes
  const int nvec = vec_ok ? N / VE : N / 4;
  const int g = nvec > 128 ? 32 : nvec > 64 ? 16 : nvec > 32 ? 8 : 4;
  const int64_t groups = ceil_div(M, 256 / g);
  const unsigned grid = (unsigned)(groups < cap ? groups : cap);
  switch (g) {
    case 32: extreme_group_rows<T, MIN, 32><<<grid, 256, 0, st>>>(x, values, indices, M, N, rs, vec_ok); break;
    case 16: extreme_group_rows<T, MIN, 16><<<grid, 256, 0, st>>>(x, values, indices, M, N, rs, vec_ok); break;
    case 8: extreme_group_rows<T, MIN, 8><<<grid, 256, 0, st>>>(x, values, indices, M, N, rs, vec_ok); break;
    default: extreme_group_rows<T, MIN, 4><<<grid, 256, 0, st>>>(x, values, indices, M, N, rs, vec_ok); break;
  }
  return finish_launch(1);
}

}  // namespace
}  // namespace mdy

using namespace mdy;

extern "C" int mdy_rowwise_extreme(const void* x, void* values, int64_t* indices, int64_t M, int64_t N,
                                   int64_t row_stride, int take_min, int dtype, void* stream) {
  if (M < 0 || N < 1 || N > INT_MAX - 64 || row_stride < N) return MDY_ERR_SIZE;
  if (M == 0) return MDY_OK;
  if (!x || !values || !indices) return MDY_ERR_NULL;
  cudaStream_t st = (cudaStream_t)stream;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VE = VecInfo<T>::kElems;
    const int vec_ok = aligned16(x) && row_stride % VE == 0;
    if (take_min) return launch_extreme<T, true>((const T*)x, (T*)values, indices, M, (int)N, row_stride, vec_ok, st);
    return launch_extreme<T, false>((const T*)x, (T*)values, indices, M, (int)N, row_stride, vec_ok, st);
  });
}
