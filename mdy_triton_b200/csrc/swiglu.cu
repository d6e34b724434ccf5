// SwiGLU  y = up * gate * sigmoid(gate)  and its backward, for sm_100a.
//
// Pure streaming: every thread issues U independent 16-byte loads per input stream before the first
// use (U*32 B forward, U*48 B backward in flight per thread), computes in float32, and writes with
// streaming stores.  Inputs are addressed as [M, N] with per-tensor row strides, so the same kernels
// serve separate up/gate tensors and the two halves of a fused [M, 2N] projection; when every stride
// equals N the problem is collapsed to a single flat row and the per-vector divide disappears.
#include "common.cuh"

namespace mdy {
namespace {

template <typename T> __device__ __forceinline__ float sigmoidf_t(float g) {
  // exp(-g) overflows to +inf for g < -88 and the quotient becomes 0, the right limit.
  return __fdividef(1.f, 1.f + __expf(-g));
}
template <> __device__ __forceinline__ float sigmoidf_t<float>(float g) { return 1.f / (1.f + expf(-g)); }

struct Addr {
  int64_t rows, nvec;      // vectors per row
  bool flat;               // all tensors contiguous: treat as one row of rows*nvec vectors
};

template <int VE>
__device__ __forceinline__ void locate(const Addr& a, int64_t i, int64_t& row, int64_t& col) {
  if (a.flat) { row = 0; col = i * VE; }
  else { row = i / a.nvec; col = (i - row * a.nvec) * VE; }
}

template <typename T, int U>
__global__ void __launch_bounds__(256)
swiglu_fwd_vec(const T* __restrict__ up, const T* __restrict__ gate, T* __restrict__ y, Addr a,
               int64_t up_rs, int64_t gate_rs, int64_t y_rs) {
  constexpr int VE = VecInfo<T>::kElems;
  const int64_t total = a.rows * a.nvec;
  const int64_t base = ((int64_t)blockIdx.x * U) * blockDim.x + threadIdx.x;
  uint4 uv[U], gv[U];
  int64_t yo[U];
  bool on[U];
#pragma unroll
  for (int k = 0; k < U; ++k) {
    const int64_t i = base + (int64_t)k * blockDim.x;
    on[k] = i < total;
    if (on[k]) {
      int64_t r, c;
      locate<VE>(a, i, r, c);
      uv[k] = ld_stream(up + r * up_rs + c);
      gv[k] = ld_stream(gate + r * gate_rs + c);
      yo[k] = r * y_rs + c;
    }
  }
#pragma unroll
  for (int k = 0; k < U; ++k) {
    if (on[k]) {
      float u[VE], g[VE];
      unpack<T>(uv[k], u);
      unpack<T>(gv[k], g);
#pragma unroll
      for (int e = 0; e < VE; ++e) u[e] = g[e] * sigmoidf_t<T>(g[e]) * u[e];
      st_stream(y + yo[k], pack<T>(u));
    }
  }
}

template <typename T, int U>
__global__ void __launch_bounds__(256)
swiglu_bwd_vec(const T* __restrict__ dy, const T* __restrict__ up, const T* __restrict__ gate,
               T* __restrict__ dup, T* __restrict__ dgate, Addr a, int64_t dy_rs, int64_t up_rs,
               int64_t gate_rs, int64_t dup_rs, int64_t dgate_rs) {
  constexpr int VE = VecInfo<T>::kElems;
  const int64_t total = a.rows * a.nvec;
  const int64_t base = ((int64_t)blockIdx.x * U) * blockDim.x + threadIdx.x;
  uint4 dv[U], uv[U], gv[U];
  int64_t o1[U], o2[U];
  bool on[U];
#pragma unroll
  for (int k = 0; k < U; ++k) {
    const int64_t i = base + (int64_t)k * blockDim.x;
    on[k] = i < total;
    if (on[k]) {
      int64_t r, c;
      locate<VE>(a, i, r, c);
      dv[k] = ld_stream(dy + r * dy_rs + c);
      uv[k] = ld_stream(up + r * up_rs + c);
      gv[k] = ld_stream(gate + r * gate_rs + c);
      o1[k] = r * dup_rs + c;
      o2[k] = r * dgate_rs + c;
    }
  }
#pragma unroll
  for (int k = 0; k < U; ++k) {
    if (on[k]) {
      float d[VE], u[VE], g[VE];
      unpack<T>(dv[k], d);
      unpack<T>(uv[k], u);
      unpack<T>(gv[k], g);
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        const float s = sigmoidf_t<T>(g[e]);
        const float act = s * g[e];
        const float dact = u[e] * d[e];
        u[e] = act * d[e];                       // dup
        g[e] = (s + act * (1.f - s)) * dact;     // dgate
      }
      st_stream(dup + o1[k], pack<T>(u));
      st_stream(dgate + o2[k], pack<T>(g));
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_fwd_scalar(const T* __restrict__ up, const T* __restrict__ gate, T* __restrict__ y, int64_t M,
                  int64_t N, int64_t up_rs, int64_t gate_rs, int64_t y_rs) {
  const int64_t total = M * N;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / N, c = i - r * N;
    const float g = to_float(gate[r * gate_rs + c]);
    const float u = to_float(up[r * up_rs + c]);
    y[r * y_rs + c] = from_float<T>(g * sigmoidf_t<T>(g) * u);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_bwd_scalar(const T* __restrict__ dy, const T* __restrict__ up, const T* __restrict__ gate,
                  T* __restrict__ dup, T* __restrict__ dgate, int64_t M, int64_t N, int64_t dy_rs,
                  int64_t up_rs, int64_t gate_rs, int64_t dup_rs, int64_t dgate_rs) {
  const int64_t total = M * N;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / N, c = i - r * N;
    const float g = to_float(gate[r * gate_rs + c]);
    const float u = to_float(up[r * up_rs + c]);
    const float d = to_float(dy[r * dy_rs + c]);
    const float s = sigmoidf_t<T>(g);
    const float act = s * g;
    dup[r * dup_rs + c] = from_float<T>(act * d);
    dgate[r * dgate_rs + c] = from_float<T>((s + act * (1.f - s)) * (u * d));
  }
}

inline int pick_unroll(int dflt) {
  int u = tunable(MDY_TUNE_SWIGLU_UNROLL);
  return (u == 1 || u == 2 || u == 4) ? u : dflt;
}

inline int64_t scalar_grid(int64_t total) {
  int64_t g = ceil_div(total, 256);
  const int64_t cap = (int64_t)(num_sms() > 0 ? num_sms() : 1) * 32;
  return g > cap ? cap : (g > 0 ? g : 1);
}

template <typename T>
int launch_fwd(const void* up_, const void* gate_, void* y_, int64_t M, int64_t N, int64_t up_rs,
               int64_t gate_rs, int64_t y_rs, cudaStream_t st) {
  constexpr int VE = VecInfo<T>::kElems;
  const T* up = (const T*)up_; const T* gate = (const T*)gate_; T* y = (T*)y_;
  const bool contiguous = up_rs == N && gate_rs == N && y_rs == N;
  const bool vec = aligned16(up) && aligned16(gate) && aligned16(y) &&
                   (contiguous ? (M * N) % VE == 0
                               : (N % VE == 0 && up_rs % VE == 0 && gate_rs % VE == 0 && y_rs % VE == 0));
  if (!vec) {
    swiglu_fwd_scalar<T><<<(unsigned)scalar_grid(M * N), 256, 0, st>>>(up, gate, y, M, N, up_rs,
                                                                      gate_rs, y_rs);
    return finish_launch(1);
  }
  Addr a;
  a.flat = contiguous;
  a.rows = contiguous ? 1 : M;
  a.nvec = contiguous ? (M * N) / VE : N / VE;
  const int64_t total = a.rows * a.nvec;
  const int U = pick_unroll(4);
  const int64_t grid = ceil_div(total, (int64_t)256 * U);
  if (grid > INT32_MAX) return MDY_ERR_UNSUPPORTED;
  switch (U) {
    case 1: swiglu_fwd_vec<T, 1><<<(unsigned)grid, 256, 0, st>>>(up, gate, y, a, up_rs, gate_rs, y_rs); break;
    case 2: swiglu_fwd_vec<T, 2><<<(unsigned)grid, 256, 0, st>>>(up, gate, y, a, up_rs, gate_rs, y_rs); break;
    default: swiglu_fwd_vec<T, 4><<<(unsigned)grid, 256, 0, st>>>(up, gate, y, a, up_rs, gate_rs, y_rs); break;
  }
  return finish_launch(1);
}

template <typename T>
int launch_bwd(const void* dy_, const void* up_, const void* gate_, void* dup_, void* dgate_, int64_t M,
               int64_t N, int64_t dy_rs, int64_t up_rs, int64_t gate_rs, int64_t dup_rs,
               int64_t dgate_rs, cudaStream_t st) {
  constexpr int VE = VecInfo<T>::kElems;
  const T* dy = (const T*)dy_; const T* up = (const T*)up_; const T* gate = (const T*)gate_;
  T* dup = (T*)dup_; T* dgate = (T*)dgate_;
  const bool contiguous = dy_rs == N && up_rs == N && gate_rs == N && dup_rs == N && dgate_rs == N;
  const bool vec = aligned16(dy) && aligned16(up) && aligned16(gate) && aligned16(dup) &&
                   aligned16(dgate) &&
                   (contiguous ? (M * N) % VE == 0
                               : (N % VE == 0 && dy_rs % VE == 0 && up_rs % VE == 0 &&
                                  gate_rs % VE == 0 && dup_rs % VE == 0 && dgate_rs % VE == 0));
  if (!vec) {
    swiglu_bwd_scalar<T><<<(unsigned)scalar_grid(M * N), 256, 0, st>>>(dy, up, gate, dup, dgate, M, N,
                                                                      dy_rs, up_rs, gate_rs, dup_rs,
                                                                      dgate_rs);
    return finish_launch(1);
  }
  Addr a;
  a.flat = contiguous;
  a.rows = contiguous ? 1 : M;
  a.nvec = contiguous ? (M * N) / VE : N / VE;
  const int64_t total = a.rows * a.nvec;
  const int U = pick_unroll(2);
  const int64_t grid = ceil_div(total, (int64_t)256 * U);
  if (grid > INT32_MAX) return MDY_ERR_UNSUPPORTED;
#define MDY_SB(UU)                                                                                 \
  swiglu_bwd_vec<T, UU><<<(unsigned)grid, 256, 0, st>>>(dy, up, gate, dup, dgate, a, dy_rs, up_rs, \
                                                        gate_rs, dup_rs, dgate_rs)
  switch (U) {
    case 1: MDY_SB(1); break;
    case 2: MDY_SB(2); break;
    default: MDY_SB(4); break;
  }
#undef MDY_SB
  return finish_launch(1);
}

}  // namespace
}  // namespace mdy

using namespace mdy;

extern "C" {

int mdy_swiglu_fwd(const void* up, const void* gate, void* y, int64_t M, int64_t N,
                   int64_t up_row_stride, int64_t gate_row_stride, int64_t y_row_stride, int dtype,
                   void* stream) {
  if (M < 0 || N < 0) return MDY_ERR_SIZE;
  if (M == 0 || N == 0) return MDY_OK;
  if (!up || !gate || !y) return MDY_ERR_NULL;
  if (up_row_stride < 0 || gate_row_stride < 0 || y_row_stride < N) return MDY_ERR_SIZE;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    return launch_fwd<T>(up, gate, y, M, N, up_row_stride, gate_row_stride, y_row_stride,
                         (cudaStream_t)stream);
  });
}

int mdy_swiglu_bwd(const void* dy, const void* up, const void* gate, void* dup, void* dgate, int64_t M,
                   int64_t N, int64_t dy_row_stride, int64_t up_row_stride, int64_t gate_row_stride,
                   int64_t dup_row_stride, int64_t dgate_row_stride, int dtype, void* stream) {
  if (M < 0 || N < 0) return MDY_ERR_SIZE;
  if (M == 0 || N == 0) return MDY_OK;
  if (!dy || !up || !gate || !dup || !dgate) return MDY_ERR_NULL;
  if (dy_row_stride < 0 || up_row_stride < 0 || gate_row_stride < 0 || dup_row_stride < N ||
      dgate_row_stride < N)
    return MDY_ERR_SIZE;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    return launch_bwd<T>(dy, up, gate, dup, dgate, M, N, dy_row_stride, up_row_stride, gate_row_stride,
                         dup_row_stride, dgate_row_stride, (cudaStream_t)stream);
  });
}

}  // extern "C"
