// Large-vocab cross-entropy for sm_100a: loss/lse sweep, gradient sweep, and the one-pass kernel
// that does both while the row is still on chip (in L2).
//
// One CTA owns one row of [M, V].  Sweep 1 keeps a per-thread (max, sum-exp) pair, updating the max
// once per 16-byte vector (one rescale per vector instead of per element), with U independent
// 16-byte loads in flight per thread; the pairs are merged by warp shuffles and one shared-memory
// exchange.  Sweep 2 recomputes exp(x - lse) and writes (p - onehot) * g with streaming stores.  In
// the fused kernel sweep 2 re-reads the row the same CTA has just pulled through L2, so HBM sees one
// read and one write per element.  Rows labelled MDY_IGNORE_INDEX are never read.
#include <math.h>
#include "common.cuh"

namespace mdy {
namespace {

constexpr int kU = 4;  // 16-byte loads in flight per thread per sweep

__device__ __forceinline__ void stat_merge(float& m, float& s, float om, float os) {
  // (m, s) <- merge of two (max, sum of exp(x - max)) pairs with ONE exp; -inf maxima carry s == 0.
  if (om > m) {
    s = ((m == -INFINITY) ? 0.f : s * fast_exp2((m - om) * kLog2e)) + os;
    m = om;
  } else if (om != -INFINITY) {
    s += os * fast_exp2((om - m) * kLog2e);
  }
}

template <int VE>
__device__ __forceinline__ void stat_update(float& m, float& s, const float* f) {
  float vm = f[0];
#pragma unroll
  for (int e = 1; e < VE; ++e) vm = fmaxf(vm, f[e]);
  if (vm > m) {
    s *= fast_exp2((m - vm) * kLog2e);  // m == -inf: s == 0 and exp2(-inf) == 0
    m = vm;
  }
  const float nm2 = (m == -INFINITY) ? 0.f : -m * kLog2e;
#pragma unroll
  for (int e = 0; e < VE; ++e) s += fast_exp2(fmaf(f[e], kLog2e, nm2));
}

// Block-wide (max, sum-exp) of x[0, V).  Result valid in every thread.  sm must hold 66 floats.
template <typename T>
__device__ __forceinline__ void row_stats(const T* x, int64_t V, bool vec_ok, float& m_out, float& s_out,
                                          float* sm) {
  constexpr int VE = VecInfo<T>::kElems;
  const int tid = threadIdx.x, BT = blockDim.x;
  const int64_t nvec = vec_ok ? V / VE : 0;
  float m = -INFINITY, s = 0.f;
  for (int64_t i0 = tid; i0 < nvec; i0 += (int64_t)BT * kU) {
    uint4 v[kU];
#pragma unroll
    for (int k = 0; k < kU; ++k) {
      const int64_t i = i0 + (int64_t)k * BT;
      if (i < nvec) v[k] = ld_plain(x + i * VE);
    }
#pragma unroll
    for (int k = 0; k < kU; ++k) {
      const int64_t i = i0 + (int64_t)k * BT;
      if (i < nvec) {
        float f[VE];
        unpack<T>(v[k], f);
        stat_update<VE>(m, s, f);
      }
    }
  }
  for (int64_t c = nvec * VE + tid; c < V; c += BT) {
    const float f = to_float(x[c]);
    stat_update<1>(m, s, &f);
  }
  // merge across the warp, then across warps
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float os = __shfl_xor_sync(0xffffffffu, s, o);
    stat_merge(m, s, om, os);
  }
  // across warps: warp 0 merges the per-warp pairs (one per lane) and broadcasts through shared memory,
  // so the exp work of the merge is paid by 32 threads, not by the whole CTA
  const int warp = tid >> 5, lane = tid & 31, nwarp = (BT + 31) >> 5;
  if (lane == 0) { sm[warp] = m; sm[32 + warp] = s; }
  __syncthreads();
  if (warp == 0) {
    m = lane < nwarp ? sm[lane] : -INFINITY;
    s = lane < nwarp ? sm[32 + lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const float os = __shfl_xor_sync(0xffffffffu, s, o);
      stat_merge(m, s, om, os);
    }
    if (lane == 0) { sm[64] = m; sm[65] = s; }
  }
  __syncthreads();
  m_out = sm[64];
  s_out = sm[65];
}

// dx[c] = (exp(x[c] - lse) - [c == loc]) * g for c in [0, V).  x may alias dx.
template <typename T>
__device__ __forceinline__ void write_grad(const T* x, T* dx, int64_t V, bool vec_ok, float lse, float g,
                                           int64_t loc) {
  constexpr int VE = VecInfo<T>::kElems;
  const int tid = threadIdx.x, BT = blockDim.x;
  const int64_t nvec = vec_ok ? V / VE : 0;
  const float nl2 = -lse * kLog2e;
  for (int64_t i0 = tid; i0 < nvec; i0 += (int64_t)BT * kU) {
    uint4 v[kU];
#pragma unroll
    for (int k = 0; k < kU; ++k) {
      const int64_t i = i0 + (int64_t)k * BT;
      if (i < nvec) v[k] = ld_plain(x + i * VE);
    }
#pragma unroll
    for (int k = 0; k < kU; ++k) {
      const int64_t i = i0 + (int64_t)k * BT;
      if (i < nvec) {
        float f[VE];
        unpack<T>(v[k], f);
#pragma unroll
        for (int e = 0; e < VE; ++e) f[e] = fast_exp2(fmaf(f[e], kLog2e, nl2));
        const int64_t c0 = i * VE;
        if (loc >= c0 && loc < c0 + VE) {
#pragma unroll
          for (int e = 0; e < VE; ++e)
            if (c0 + e == loc) f[e] -= 1.f;
        }
#pragma unroll
        for (int e = 0; e < VE; ++e) f[e] *= g;
        st_stream(dx + i * VE, pack<T>(f));
      }
    }
  }
  for (int64_t c = nvec * VE + tid; c < V; c += BT) {
    float p = fast_exp2(fmaf(to_float(x[c]), kLog2e, nl2));
    if (c == loc) p -= 1.f;
    dx[c] = from_float<T>(p * g);
  }
}

template <typename T>
__device__ __forceinline__ void zero_row(T* dx, int64_t V, bool vec_ok) {
  constexpr int VE = VecInfo<T>::kElems;
  const int64_t nvec = vec_ok ? V / VE : 0;
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (int64_t i = threadIdx.x; i < nvec; i += blockDim.x) st_stream(dx + i * VE, z);
  for (int64_t c = nvec * VE + threadIdx.x; c < V; c += blockDim.x) dx[c] = from_float<T>(0.f);
}

__device__ __forceinline__ float load_scalar(const void* p, int64_t idx, int dtype) {
  if (dtype == MDY_F32) return ((const float*)p)[idx];
  if (dtype == MDY_F16) return __half2float(((const __half*)p)[idx]);
  return __bfloat162float(((const __nv_bfloat16*)p)[idx]);
}

template <typename T>
__global__ void __launch_bounds__(1024)
ce_fwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ labels, float* __restrict__ losses,
              float* __restrict__ lse_out, int64_t V, int64_t rs, int64_t vocab_start, int split,
              int vec_ok) {
  __shared__ float sm[66];
  const int64_t row = blockIdx.x;
  const int64_t label = labels[row];
  if (label == MDY_IGNORE_INDEX) {
    if (threadIdx.x == 0) { losses[row] = 0.f; lse_out[row] = 0.f; }
    return;
  }
  const T* x = logits + row * rs;
  float m, s;
  row_stats<T>(x, V, vec_ok != 0, m, s, sm);
  if (threadIdx.x == 0) {
    const float lse = m + logf(s);
    const int64_t loc = label - vocab_start;
    float loss = 0.f;
    if (loc >= 0 && loc < V) {
      const float xl = to_float(x[loc]);
      loss = split ? -xl : lse - xl;
    }
    losses[row] = loss;
    lse_out[row] = lse;
  }
}

template <typename T>
__global__ void __launch_bounds__(1024)
ce_bwd_kernel(const void* __restrict__ dlosses, int64_t dl_stride, int dl_dtype, const T* logits,
              T* dlogits, const int64_t* __restrict__ labels, const float* __restrict__ lse, int64_t V,
              int64_t rs, int64_t vocab_start, int fill_ignored, int vec_ok) {
  const int64_t row = blockIdx.x;
  const int64_t label = labels[row];
  T* dx = dlogits + row * rs;
  if (label == MDY_IGNORE_INDEX) {
    if (fill_ignored) zero_row<T>(dx, V, vec_ok != 0);
    return;
  }
  const float g = load_scalar(dlosses, row * dl_stride, dl_dtype);
  int64_t loc = label - vocab_start;
  if (loc < 0 || loc >= V) loc = -1;
  write_grad<T>(logits + row * rs, dx, V, vec_ok != 0, lse[row], g, loc);
}

template <typename T>
__global__ void __launch_bounds__(1024)
ce_fused_kernel(const T* logits, T* dlogits, const int64_t* __restrict__ labels,
                float* __restrict__ losses, float* __restrict__ lse_out,
                const float* __restrict__ gdev, float ghost, int64_t V, int64_t rs, int vec_ok) {
  __shared__ float sm[66];
  const int64_t row = blockIdx.x;
  const int64_t label = labels[row];
  T* dx = dlogits + row * rs;
  if (label == MDY_IGNORE_INDEX) {
    if (threadIdx.x == 0) { losses[row] = 0.f; lse_out[row] = 0.f; }
    zero_row<T>(dx, V, vec_ok != 0);
    return;
  }
  const T* x = logits + row * rs;
  float m, s;
  row_stats<T>(x, V, vec_ok != 0, m, s, sm);
  const float lse = m + logf(s);
  const int64_t loc = (label >= 0 && label < V) ? label : -1;
  if (threadIdx.x == 0) {
    losses[row] = loc >= 0 ? lse - to_float(x[loc]) : 0.f;
    lse_out[row] = lse;
  }
  const float g = ghost * (gdev ? *gdev : 1.f);
  // every thread must have consumed x[loc] before an in-place sweep 2 may overwrite it
  __syncthreads();
  write_grad<T>(x, dx, V, vec_ok != 0, lse, g, loc);
}

template <typename T>
__global__ void __launch_bounds__(256)
scale_kernel(T* buf, int64_t n, const float* __restrict__ scale, int vec_ok) {
  constexpr int VE = VecInfo<T>::kElems;
  const float sc = *scale;
  if (sc == 1.f) return;
  const int64_t nvec = vec_ok ? n / VE : 0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (int64_t i = t0; i < nvec; i += stride) {
    float f[VE];
    unpack<T>(ld_plain(buf + i * VE), f);
#pragma unroll
    for (int e = 0; e < VE; ++e) f[e] *= sc;
    st_plain(buf + i * VE, pack<T>(f));
  }
  for (int64_t c = nvec * VE + t0; c < n; c += stride) buf[c] = from_float<T>(to_float(buf[c]) * sc);
}

__global__ void __launch_bounds__(256)
vp_combine_kernel(const float* __restrict__ gathered, const int64_t* __restrict__ labels,
                  float* __restrict__ losses, float* __restrict__ lse_out, int tp, int64_t M) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= M) return;
  if (labels[r] == MDY_IGNORE_INDEX) {
    losses[r] = 0.f;
    lse_out[r] = 0.f;
    return;
  }
  // gathered is [tp, 2, M]: plane 0 = per-rank local lse, plane 1 = -x_label on the owning rank
  float m = -INFINITY;
  for (int t = 0; t < tp; ++t) m = fmaxf(m, gathered[(int64_t)t * 2 * M + r]);
  float s = 0.f, xl = 0.f;
  for (int t = 0; t < tp; ++t) {
    const float l = gathered[(int64_t)t * 2 * M + r];
    s += (l == -INFINITY) ? 0.f : expf(l - m);
    xl += gathered[((int64_t)t * 2 + 1) * M + r];
  }
  const float lse = m + logf(s);
  lse_out[r] = lse;
  losses[r] = lse + xl;
}

inline int ce_threads() {
  int t = tunable(MDY_TUNE_CE_THREADS);
  if (t < 64 || t > 1024 || (t & 31)) t = 512;
  return t;
}

// CTA sizes of the two-phase kernels when the tunable leaves the choice open (measured at 16384 rows,
// bf16, V from 2000 to 256000).  The statistics sweep runs best with many small CTAs per SM whatever the
// row length (V = 128256: 6380 GB/s with 128 threads, 5290 with 512; V = 4000: 3300 against 790); the
// gradient sweep wants small CTAs only for short rows (V = 4000: 5540 against 2110 GB/s) and 512
// threads for long ones.
inline int ce_fwd_threads(int64_t row_bytes) {
  const int t = tunable(MDY_TUNE_CE_THREADS);
  if (t >= 64 && t <= 1024 && !(t & 31)) return t;
  return row_bytes <= 32 * 1024 ? 64 : 128;
}
inline int ce_bwd_threads(int64_t row_bytes) {
  const int t = tunable(MDY_TUNE_CE_THREADS);
  if (t >= 64 && t <= 1024 && !(t & 31)) return t;
  return row_bytes <= 16 * 1024 ? 64 : row_bytes <= 32 * 1024 ? 128 : row_bytes <= 64 * 1024 ? 256 : 512;
}

template <typename T>
inline bool rows_vec_ok(const void* a, const void* b, int64_t rs) {
  constexpr int VE = VecInfo<T>::kElems;
  return aligned16(a) && (b == nullptr || aligned16(b)) && rs % VE == 0;
}

}  // namespace

// defined in ce_cluster.cu: shared-memory/cluster one-pass kernel.  Returns MDY_ERR_UNSUPPORTED when
// the shape does not fit it (the caller then uses the L2-resident row kernel).
int ce_fused_cluster(const void* logits, void* dlogits, const int64_t* labels, float* losses, float* lse,
                     const float* gdev, float ghost, int64_t M, int64_t V, int64_t rs, int dtype,
                     cudaStream_t st);

}  // namespace mdy

using namespace mdy;

extern "C" {

int mdy_ce_fwd(const void* logits, const int64_t* labels, float* losses, float* lse, int64_t M, int64_t V,
               int64_t row_stride, int64_t vocab_start, int split, int dtype, void* stream) {
  if (M < 0 || V <= 0 || row_stride < V) return MDY_ERR_SIZE;
  if (M > INT32_MAX) return MDY_ERR_UNSUPPORTED;
  if (M == 0) return MDY_OK;
  if (!logits || !labels || !losses || !lse) return MDY_ERR_NULL;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    ce_fwd_kernel<T><<<(unsigned)M, ce_fwd_threads(V * (int64_t)sizeof(T)), 0, (cudaStream_t)stream>>>(
        (const T*)logits, labels, losses, lse, V, row_stride, vocab_start, split,
        rows_vec_ok<T>(logits, nullptr, row_stride));
    return finish_launch(1);
  });
}

int mdy_ce_bwd(const void* dlosses, int64_t dloss_stride, int dloss_dtype, const void* logits,
               void* dlogits, const int64_t* labels, const float* lse, int64_t M, int64_t V,
               int64_t row_stride, int64_t vocab_start, int fill_ignored, int dtype, void* stream) {
  if (M < 0 || V <= 0 || row_stride < V || dloss_stride < 0) return MDY_ERR_SIZE;
  if (M > INT32_MAX) return MDY_ERR_UNSUPPORTED;
  if (dloss_dtype != MDY_F32 && dloss_dtype != MDY_F16 && dloss_dtype != MDY_BF16) return MDY_ERR_DTYPE;
  if (M == 0) return MDY_OK;
  if (!dlosses || !logits || !dlogits || !labels || !lse) return MDY_ERR_NULL;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    ce_bwd_kernel<T><<<(unsigned)M, ce_bwd_threads(V * (int64_t)sizeof(T)), 0, (cudaStream_t)stream>>>(
        dlosses, dloss_stride, dloss_dtype, (const T*)logits, (T*)dlogits, labels, lse, V, row_stride,
        vocab_start, fill_ignored, rows_vec_ok<T>(logits, dlogits, row_stride));
    return finish_launch(1);
  });
}

int mdy_ce_fused(const void* logits, void* dlogits, const int64_t* labels, float* losses, float* lse,
                 const float* grad_scale_dev, float grad_scale_host, int64_t M, int64_t V,
                 int64_t row_stride, int dtype, void* stream) {
  if (M < 0 || V <= 0 || row_stride < V) return MDY_ERR_SIZE;
  if (M > INT32_MAX) return MDY_ERR_UNSUPPORTED;
  if (dtype != MDY_F32 && dtype != MDY_F16 && dtype != MDY_BF16) return MDY_ERR_DTYPE;
  if (M == 0) return MDY_OK;
  if (!logits || !dlogits || !labels || !losses || !lse) return MDY_ERR_NULL;
  const int impl = tunable(MDY_TUNE_CE_FUSED_IMPL);
  if (impl != 1) {
    int rc = ce_fused_cluster(logits, dlogits, labels, losses, lse, grad_scale_dev, grad_scale_host, M, V,
                              row_stride, dtype, (cudaStream_t)stream);
    if (rc != MDY_ERR_UNSUPPORTED) return rc;
  }
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    // Optional residency cap: asking for 1/k of the SM's shared memory keeps at most k CTAs (rows) per
    // SM in flight, which bounds the L2 footprint of the rows between their two sweeps.
    size_t pad = 0;
    const int per_sm = tunable(MDY_TUNE_CE_FUSED_CTAS_PER_SM);
    if (per_sm > 0) {
      pad = (size_t)(227 * 1024) / per_sm - 2048;
      if (cudaFuncSetAttribute(ce_fused_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pad) != cudaSuccess) {
        (void)cudaGetLastError();
        pad = 0;
      }
    }
    ce_fused_kernel<T><<<(unsigned)M, ce_threads(), pad, (cudaStream_t)stream>>>(
        (const T*)logits, (T*)dlogits, labels, losses, lse, grad_scale_dev, grad_scale_host, V,
        row_stride, rows_vec_ok<T>(logits, dlogits, row_stride));
    return finish_launch(1);
  });
}

int mdy_scale_inplace(void* buf, int64_t n, const float* scale, int dtype, void* stream) {
  if (n < 0) return MDY_ERR_SIZE;
  if (n == 0) return MDY_OK;
  if (!buf || !scale) return MDY_ERR_NULL;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    int64_t grid = ceil_div(n, (int64_t)256 * VecInfo<T>::kElems * 4);
    const int64_t cap = (int64_t)(num_sms() > 0 ? num_sms() : 1) * 32;
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    scale_kernel<T><<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>((T*)buf, n, scale, aligned16(buf));
    return finish_launch(1);
  });
}

int mdy_ce_vp_combine(const float* gathered, const int64_t* labels, float* losses, float* lse, int64_t tp,
                      int64_t M, void* stream) {
  if (M < 0 || tp <= 0 || tp > 4096) return MDY_ERR_SIZE;
  if (M == 0) return MDY_OK;
  if (!gathered || !labels || !losses || !lse) return MDY_ERR_NULL;
  vp_combine_kernel<<<(unsigned)ceil_div(M, 256), 256, 0, (cudaStream_t)stream>>>(gathered, labels, losses,
                                                                                 lse, (int)tp, M);
  return finish_launch(1);
}

}  // extern "C"
