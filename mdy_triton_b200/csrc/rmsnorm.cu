// RMSNorm and fused add+RMSNorm, forward and backward, for sm_100a.
//
// Layout: activations are [M, N] row-major with a row stride.  A row is owned by a GROUP of G
// threads (G = 32..1024, a multiple of 32 chosen so that G * VPT covers the row with as few idle
// lanes as possible: 448 vectors -> 224 x 2); each thread keeps VPT 16-byte vectors of the row in
// registers, so the row is read from HBM exactly once in forward (sum of squares and scaling use
// the same registers) and x/dy exactly once in backward.  A CTA holds blockDim/G groups and walks a
// persistent row loop; the weight vector stays in registers across the loop.  The in-group reduction
// is warp shuffles plus one shared-memory exchange (double-buffered: one __syncthreads per row).
// Backward accumulates dw in float registers, folds the groups of a CTA through shared memory and
// writes one float partial row per CTA; a second small kernel sums the partials and casts.
#include <atomic>
#include "common.cuh"

namespace mdy {
namespace {

struct RowPlan {
  int vpt;   // 16-byte vectors per thread (1, 2, 4, 8); 0 = no vector plan
  int G;     // threads per row
  int BT;    // threads per CTA
  int gpc;   // rows (groups) per CTA
};

// `group` > 0 forces the threads per row (rounded up to a warp multiple); 0 = choose.
inline RowPlan plan_rows(int64_t nvec, int min_bt, int pref_vpt, int group) {
  RowPlan p{0, 0, 0, 0};
  if (nvec <= 0 || nvec > 8192) return p;
  if (pref_vpt != 1 && pref_vpt != 4) pref_vpt = 2;
  int64_t G;
  if (group > 0) {
    G = ceil_div(group, 32) * 32;
  } else if (tunable(MDY_TUNE_NORM_POW2_GROUPS) > 0) {
    G = next_pow2(ceil_div(nvec, pref_vpt));
  } else {
    // smallest warp multiple that covers the row with pref_vpt vectors per thread
    G = ceil_div(ceil_div(nvec, pref_vpt), 32) * 32;
  }
  if (G < 32) G = 32;
  if (G > 1024) G = 1024;
  int64_t need = ceil_div(nvec, G);
  p.vpt = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
  p.G = (int)G;
  // as many rows per CTA as fit the CTA size asked for (at least one, never more than 1024 threads)
  if (G < 1024 && need > 4) return plan_rows(nvec, min_bt, pref_vpt, 0);  // a forced group too small for the row
  // as many rows per CTA as come closest to the CTA size asked for; CTAs of more than 512 threads only
  // where one row needs them (they are limited to 64 registers per thread)
  p.gpc = G >= min_bt ? 1 : (int)((min_bt + G / 2) / G);
  if (p.gpc < 1) p.gpc = 1;
  while (p.gpc > 1 && p.G * p.gpc > 512) --p.gpc;
  p.BT = p.G * p.gpc;
  return p;
}

// Sum `v` over the G threads of the caller's group.  `buf` has one float per warp of the CTA.
// All threads of the CTA must call it the same number of times (it contains a __syncthreads when
// a group spans several warps).
__device__ __forceinline__ float group_sum(float v, float* buf, int G, int gid, int warp, int lane) {
  v = warp_sum(v);
  const int wpg = G >> 5;
  if (wpg > 1) {
    if (lane == 0) buf[warp] = v;
    __syncthreads();
    float s = 0.f;
    const float* b = buf + gid * wpg;
    for (int k = 0; k < wpg; ++k) s += b[k];
    v = s;
  }
  return v;
}

// The weight may have a different element type than the activations (fp32 master weights with
// bf16 activations); it is converted to float registers once per CTA.
__device__ __forceinline__ float load_w(const void* w, int64_t idx, int w_dtype) {
  if (w_dtype == MDY_F32) return __ldg((const float*)w + idx);
  if (w_dtype == MDY_F16) return __half2float(__ldg((const __half*)w + idx));
  return __bfloat162float(__ldg((const __nv_bfloat16*)w + idx));
}

// The VE weights of 16-byte activation vector `v` as floats.  `wvec`: the weight base is 16-byte
// aligned, so they come in one or two vector loads instead of VE scalar ones (the weight load is the
// head of every CTA's dependency chain, which is what short launches are made of).
template <int VE>
__device__ __forceinline__ void load_w_vec(const void* w, int v, int w_dtype, bool wvec, float* out) {
  if (wvec && w_dtype == MDY_F32) {
#pragma unroll
    for (int h = 0; h < VE / 4; ++h) {
      const uint4 q = ld_reuse((const float*)w + (int64_t)v * VE + h * 4);
      unpack<float>(q, out + h * 4);
    }
  } else if (wvec && VE == 8) {
    const uint4 q = ld_reuse((const uint16_t*)w + (int64_t)v * VE);
    if (w_dtype == MDY_F16) unpack<__half>(q, out); else unpack<__nv_bfloat16>(q, out);
  } else {
#pragma unroll
    for (int e = 0; e < VE; ++e) out[e] = load_w(w, (int64_t)v * VE + e, w_dtype);
  }
}

}  // namespace
}  // namespace mdy
#include "rmsnorm_staged.cuh"
namespace mdy {
namespace {

template <typename T, int VPT, bool ADD, int MAXT>
__global__ void __launch_bounds__(MAXT)
norm_fwd_vec(const T* __restrict__ x, const T* __restrict__ res, const void* __restrict__ w,
             int w_dtype, T* __restrict__ y, T* __restrict__ new_res, float* __restrict__ rstd_out,
             int64_t M, int N, int64_t x_rs, int64_t res_rs, int64_t y_rs, int64_t nres_rs,
             float eps, int G, bool wvec) {
  constexpr int VE = VecInfo<T>::kElems;
  extern __shared__ float smem[];
  const int nvec = N / VE;
  const int gpc = blockDim.x / G;
  const int gid = threadIdx.x / G;
  const int t = threadIdx.x - gid * G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarp = blockDim.x >> 5;
  const float inv_n = 1.f / (float)N;

  float wf[VPT][VE];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = t + i * G;
    if (v < nvec) {
      load_w_vec<VE>(w, v, w_dtype, wvec, wf[i]);
    } else {
#pragma unroll
      for (int e = 0; e < VE; ++e) wf[i][e] = 0.f;
    }
  }

  // Software pipeline (CTAs of up to 512 threads): the next row's loads are issued before the current
  // row's reduction and stores, so read requests stay in flight across the barrier.
  constexpr bool PF = MAXT <= 512 && !ADD;   // the add variant already has four streams in flight
  const int64_t step = (int64_t)gridDim.x * gpc;
  uint4 xv[VPT], rv[ADD ? VPT : 1];
  uint4 nx[VPT], nr[ADD ? VPT : 1];
  auto fetch = [&](int64_t row, uint4* px, uint4* pr) {
    const bool valid = row < M;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = t + i * G;
      const bool on = valid && v < nvec;
      px[i] = on ? ld_stream(x + row * x_rs + (int64_t)v * VE) : make_uint4(0, 0, 0, 0);
      if (ADD) pr[i] = on ? ld_stream(res + row * res_rs + (int64_t)v * VE) : make_uint4(0, 0, 0, 0);
    }
  };
  fetch((int64_t)blockIdx.x * gpc + gid, xv, rv);
  int it = 0;
  for (int64_t base = (int64_t)blockIdx.x * gpc; base < M; base += step, ++it) {
    const int64_t row = base + gid;
    const bool valid = row < M;
    if (PF && base + step < M) fetch(row + step, nx, nr);
    float f[VPT][VE];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      unpack<T>(xv[i], f[i]);
      if (ADD) {
        float r[VE];
        unpack<T>(rv[i], r);
#pragma unroll
        for (int e = 0; e < VE; ++e) f[i][e] += r[e];
        const int v = t + i * G;
        if (valid && v < nvec) st_plain(new_res + row * nres_rs + (int64_t)v * VE, pack<T>(f[i]));
      }
#pragma unroll
      for (int e = 0; e < VE; ++e) ss = fmaf(f[i][e], f[i][e], ss);
    }
    ss = group_sum(ss, smem + (it & 1) * nwarp, G, gid, warp, lane);
    const float rstd = 1.f / sqrtf(ss * inv_n + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = t + i * G;
#pragma unroll
      for (int e = 0; e < VE; ++e) f[i][e] = f[i][e] * rstd * wf[i][e];
      if (valid && v < nvec) st_plain(y + row * y_rs + (int64_t)v * VE, pack<T>(f[i]));
    }
    if (valid && t == 0) rstd_out[row] = rstd;
    if (PF) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        xv[i] = nx[i];
        if (ADD) rv[i] = nr[i];
      }
    } else if (base + step < M) {
      fetch(row + step, xv, rv);
    }
  }
}

__device__ __forceinline__ float block_sum(float v, float* buf) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // buf may still be read from a previous call
  if (lane == 0) buf[warp] = v;
  __syncthreads();
  float s = 0.f;
  for (int k = 0; k < nwarp; ++k) s += buf[k];
  return s;
}

// Any N, any alignment: one CTA per row, two sweeps (the second is served by L1/L2).
template <typename T, bool ADD>
__global__ void __launch_bounds__(256)
norm_fwd_scalar(const T* __restrict__ x, const T* __restrict__ res, const void* __restrict__ w,
                int w_dtype, T* __restrict__ y, T* __restrict__ new_res, float* __restrict__ rstd_out,
                int64_t M, int64_t N, int64_t x_rs, int64_t res_rs, int64_t y_rs, int64_t nres_rs,
                float eps) {
  __shared__ float buf[32];
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    float ss = 0.f;
    for (int64_t c = threadIdx.x; c < N; c += blockDim.x) {
      float v = to_float(x[row * x_rs + c]);
      if (ADD) {
        v += to_float(res[row * res_rs + c]);
        new_res[row * nres_rs + c] = from_float<T>(v);
      }
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, buf);
    const float rstd = 1.f / sqrtf(ss / (float)N + eps);
    for (int64_t c = threadIdx.x; c < N; c += blockDim.x) {
      float v = to_float(x[row * x_rs + c]);
      if (ADD) v += to_float(res[row * res_rs + c]);
      y[row * y_rs + c] = from_float<T>(v * rstd * load_w(w, c, w_dtype));
    }
    if (threadIdx.x == 0) rstd_out[row] = rstd;
  }
}

template <typename T, int VPT, bool ADD, int MAXT>
__global__ void __launch_bounds__(MAXT)
norm_bwd_vec(const T* __restrict__ dy, const T* __restrict__ x, const void* __restrict__ w,
             int w_dtype, const float* __restrict__ rstd_in, const T* __restrict__ dres, T* __restrict__ dx,
             float* __restrict__ dw_partial, int64_t M, int N, int64_t dy_rs, int64_t x_rs,
             int64_t dres_rs, int64_t dx_rs, int G, bool wvec) {
  constexpr int VE = VecInfo<T>::kElems;
  extern __shared__ float smem[];
  const int nvec = N / VE;
  const int gpc = blockDim.x / G;
  const int gid = threadIdx.x / G;
  const int t = threadIdx.x - gid * G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarp = blockDim.x >> 5;
  const float inv_n = 1.f / (float)N;
  const bool has_dres = ADD && dres != nullptr;

  float wf[VPT][VE];
  float acc[VPT][VE];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = t + i * G;
    if (v < nvec) load_w_vec<VE>(w, v, w_dtype, wvec, wf[i]);
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      if (v >= nvec) wf[i][e] = 0.f;
      acc[i][e] = 0.f;
    }
  }

  // Software pipeline: the loads of the CTA's next row are issued before the current row's reduction
  // (which contains a __syncthreads), so HBM requests stay in flight across the barrier.  Only where the
  // register budget allows it (CTAs of up to 512 threads).
  constexpr bool PF = MAXT <= 512;
  uint4 xv[VPT], gv[VPT], dv[ADD ? VPT : 1];
  uint4 nx[VPT], ng[VPT], nd[ADD ? VPT : 1];
  float rstd = 0.f, nrstd = 0.f;
  const int64_t step = (int64_t)gridDim.x * gpc;
  auto fetch = [&](int64_t row, uint4* px, uint4* pg, uint4* pd, float& r) {
    const bool valid = row < M;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = t + i * G;
      const bool on = valid && v < nvec;
      px[i] = on ? ld_stream(x + row * x_rs + (int64_t)v * VE) : make_uint4(0, 0, 0, 0);
      pg[i] = on ? ld_stream(dy + row * dy_rs + (int64_t)v * VE) : make_uint4(0, 0, 0, 0);
      if (ADD) pd[i] = (on && has_dres) ? ld_stream(dres + row * dres_rs + (int64_t)v * VE)
                                        : make_uint4(0, 0, 0, 0);
    }
    r = valid ? rstd_in[row] : 0.f;
  };
  fetch((int64_t)blockIdx.x * gpc + gid, xv, gv, dv, rstd);
  int it = 0;
  for (int64_t base = (int64_t)blockIdx.x * gpc; base < M; base += step, ++it) {
    const int64_t row = base + gid;
    const bool valid = row < M;
    if (PF && base + step < M) fetch(row + step, nx, ng, nd, nrstd);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      float xf[VE], gf[VE];
      unpack<T>(xv[i], xf);
      unpack<T>(gv[i], gf);
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        const float xhat = xf[e] * rstd;
        acc[i][e] = fmaf(xhat, gf[e], acc[i][e]);
        dot = fmaf(xhat, wf[i][e] * gf[e], dot);
      }
    }
    dot = group_sum(dot, smem + (it & 1) * nwarp, G, gid, warp, lane);
    const float c = dot * inv_n;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = t + i * G;
      float xf[VE], gf[VE], o[VE];
      unpack<T>(xv[i], xf);
      unpack<T>(gv[i], gf);
#pragma unroll
      for (int e = 0; e < VE; ++e) o[e] = (wf[i][e] * gf[e] - xf[e] * rstd * c) * rstd;
      if (ADD) {
        float df[VE];
        unpack<T>(dv[i], df);
#pragma unroll
        for (int e = 0; e < VE; ++e) o[e] += df[e];
      }
      if (valid && v < nvec) st_stream(dx + row * dx_rs + (int64_t)v * VE, pack<T>(o));
    }
    if (PF) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        xv[i] = nx[i]; gv[i] = ng[i];
        if (ADD) dv[i] = nd[i];
      }
      rstd = nrstd;
    } else if (base + step < M) {
      fetch(row + step, xv, gv, dv, rstd);
    }
  }

  float* out = dw_partial + (int64_t)blockIdx.x * N;
  if (gpc > 1) {
    float* colsum = smem + 2 * nwarp;
    for (int g = 0; g < gpc; ++g) {
      __syncthreads();
      if (gid == g) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = t + i * G;
          if (v < nvec) {
#pragma unroll
            for (int e = 0; e < VE; ++e) {
              if (g == 0) colsum[v * VE + e] = acc[i][e];
              else colsum[v * VE + e] += acc[i][e];
            }
          }
        }
      }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < N; c += blockDim.x) out[c] = colsum[c];
  } else {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = t + i * G;
      if (v < nvec) {
#pragma unroll
        for (int e = 0; e < VE; ++e) out[v * VE + e] = acc[i][e];
      }
    }
  }
}

// Any N / alignment.  Column c of a CTA's partial row is always touched by the same thread, so the
// read-modify-write on the partial row needs no atomics.
template <typename T, bool ADD>
__global__ void __launch_bounds__(256)
norm_bwd_scalar(const T* __restrict__ dy, const T* __restrict__ x, const void* __restrict__ w,
                int w_dtype, const float* __restrict__ rstd_in, const T* __restrict__ dres, T* __restrict__ dx,
                float* __restrict__ dw_partial, int64_t M, int64_t N, int64_t dy_rs, int64_t x_rs,
                int64_t dres_rs, int64_t dx_rs) {
  __shared__ float buf[32];
  float* out = dw_partial + (int64_t)blockIdx.x * N;
  for (int64_t c = threadIdx.x; c < N; c += blockDim.x) out[c] = 0.f;
  const bool has_dres = ADD && dres != nullptr;
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int64_t c = threadIdx.x; c < N; c += blockDim.x) {
      const float xhat = to_float(x[row * x_rs + c]) * rstd;
      const float g = to_float(dy[row * dy_rs + c]);
      dot = fmaf(xhat, load_w(w, c, w_dtype) * g, dot);
      out[c] = fmaf(xhat, g, out[c]);
    }
    dot = block_sum(dot, buf);
    const float cc = dot / (float)N;
    for (int64_t c = threadIdx.x; c < N; c += blockDim.x) {
      const float xhat = to_float(x[row * x_rs + c]) * rstd;
      const float g = to_float(dy[row * dy_rs + c]);
      float o = (load_w(w, c, w_dtype) * g - xhat * cc) * rstd;
      if (has_dres) o += to_float(dres[row * dres_rs + c]);
      dx[row * dx_rs + c] = from_float<T>(o);
    }
  }
}

// dw[c] = sum_p partial[p, c], cast to T.  CTA = 32 columns x 32 row-lanes.
template <typename T>
__global__ void __launch_bounds__(1024)
dw_reduce(const float* __restrict__ partial, T* __restrict__ dw, int P, int64_t N) {
  __shared__ float s[32][33];
  const int64_t c = (int64_t)blockIdx.x * 32 + threadIdx.x;
  float a = 0.f;
  if (c < N) {
    for (int p = threadIdx.y; p < P; p += 32) a += partial[(int64_t)p * N + c];
  }
  s[threadIdx.y][threadIdx.x] = a;
  __syncthreads();
  if (threadIdx.y == 0 && c < N) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) t += s[k][threadIdx.x];
    dw[c] = from_float<T>(t);
  }
}

inline int norm_ctas_per_sm() {
  int v = tunable(MDY_TUNE_NORM_CTAS_PER_SM);
  return v > 0 ? v : 2;   // x (1024 / CTA threads) CTAs per SM: 8 CTAs of 256 threads measured best
}

inline int64_t vec_grid(int64_t M, const RowPlan& p, int per_sm_scale) {
  int64_t need = ceil_div(M, p.gpc);
  int64_t cap = (int64_t)num_sms() * per_sm_scale;
  if (cap < 1) cap = 1;
  return need < cap ? need : cap;
}

// Resident-CTA budget for the backward kernels: they are persistent (one partial row per CTA), so
// the grid is sized to about one wave of 512-thread CTAs.
inline int bwd_per_sm(const RowPlan& p) {
  int t = tunable(MDY_TUNE_NORM_CTAS_PER_SM);
  if (t > 0) return t;
  // measured (hidden 4096, bf16): one 512-thread CTA per SM with the next row prefetched is fastest
  return p.BT >= 512 ? 1 : 2;
}

// CTA size the backward kernels aim for (a row group of more threads gets a CTA of its own)
inline int bwd_min_threads() {
  const int t = tunable(MDY_TUNE_NORM_BWD_THREADS);
  return (t == 128 || t == 256 || t == 512) ? t : 512;
}
inline int fwd_min_threads() {
  const int t = tunable(MDY_TUNE_NORM_FWD_THREADS);
  return (t == 128 || t == 256 || t == 512) ? t : 256;
}

inline int64_t scalar_grid(int64_t M) {
  int64_t cap = (int64_t)num_sms() * 2;
  if (cap < 1) cap = 1;
  return M < cap ? (M > 0 ? M : 1) : cap;
}

// Everything the backward launch derives from the problem size and the knobs, computed ONCE per call:
// the entry point that checks a scratch size and the launch that follows must see the same grid.
struct BwdPlan {
  RowPlan p;      // p.vpt == 0: scalar kernel
  int64_t grid;   // CTAs = partial rows written
  StagedPlan sp;  // sp.ok: the shared-memory-staged kernel runs instead, with `vpl` vectors per lane
  int vpl;
};

// Which backward kernel serves a shape: 0 = choose (staged for rows of 6 KB and more with enough of them to
// fill the GPU), 1 = register-resident kernels always, 2 = staged wherever it has a geometry.
inline bool want_staged(int64_t M, int64_t row_bytes, int rows_per_block) {
  const int impl = tunable(MDY_TUNE_NORM_IMPL);
  if (impl == 1) return false;
  if (impl == 2) return true;
  return row_bytes >= 6 * 1024 && M >= (int64_t)rows_per_block * num_sms();
}

inline int64_t staged_grid(int64_t M, const StagedPlan& sp) {
  const int64_t blocks = ceil_div(M, (int64_t)(kStagedWarps / sp.team));
  int per_sm = tunable(MDY_TUNE_NORM_CTAS_PER_SM);
  if (per_sm <= 0 || per_sm > sp.ctas_per_sm) per_sm = sp.ctas_per_sm;
  const int64_t cap = (int64_t)num_sms() * per_sm;
  return blocks < cap ? blocks : (cap > 0 ? cap : 1);
}

template <typename T>
inline BwdPlan plan_bwd(int64_t M, int64_t N, bool vec_ok, int streams) {
  constexpr int VE = VecInfo<T>::kElems;
  BwdPlan b{RowPlan{0, 0, 0, 0}, 0, StagedPlan{false, 0, 0, 0, 0, 0}, 0};
  if (vec_ok && N % VE == 0) {
    b.p = plan_rows(N / VE, bwd_min_threads(), tunable(MDY_TUNE_NORM_BWD_VPT), tunable(MDY_TUNE_NORM_BWD_GROUP));
    if (M > 0 && sizeof(T) == 2) {   // the staged kernels are built for the 16-bit activation types
      StagedPlan sp = plan_staged(N * (int64_t)sizeof(T), streams, tunable(MDY_TUNE_NORM_TEAM));
      const int64_t need = sp.ok ? ceil_div(N / VE, 32 * sp.team) : 99;
      if (sp.ok && need <= 16 && want_staged(M, N * (int64_t)sizeof(T), kStagedWarps / sp.team)) {
        b.sp = sp;
        b.vpl = need <= 2 ? 2 : need <= 4 ? 4 : need <= 8 ? 8 : 16;
      }
    }
  }
  if (M == 0) b.grid = 0;
  else if (b.sp.ok) b.grid = staged_grid(M, b.sp);
  else b.grid = b.p.vpt ? vec_grid(M, b.p, bwd_per_sm(b.p)) : scalar_grid(M);
  return b;
}

// Upper bound over the kernels that may serve the shape (the caller sizes its scratch before alignment
// and the number of gradient streams are known).
template <typename T>
inline int64_t partial_rows(int64_t M, int64_t N) {
  int64_t rows = plan_bwd<T>(M, N, false, 2).grid;
  for (int streams = 2; streams <= 3; ++streams) {
    const int64_t g = plan_bwd<T>(M, N, true, streams).grid;
    if (g > rows) rows = g;
  }
  // the register-resident kernels, should a launch not get the staged one
  if (N % VecInfo<T>::kElems == 0 && M > 0) {
    RowPlan p = plan_rows(N / VecInfo<T>::kElems, bwd_min_threads(), tunable(MDY_TUNE_NORM_BWD_VPT), tunable(MDY_TUNE_NORM_BWD_GROUP));
    if (p.vpt) {
      const int64_t g = vec_grid(M, p, bwd_per_sm(p));
      if (g > rows) rows = g;
    }
  }
  return rows;
}

template <typename T, bool ADD>
int launch_fwd(const void* x_, const void* res_, const void* w, int w_dtype, void* y_, void* nres_,
               float* rstd, int64_t M, int64_t N, int64_t x_rs, int64_t res_rs, int64_t y_rs,
               int64_t nres_rs, float eps, cudaStream_t st) {
  constexpr int VE = VecInfo<T>::kElems;
  const T* x = (const T*)x_; const T* res = (const T*)res_;
  T* y = (T*)y_; T* nres = (T*)nres_;
  bool vec = N % VE == 0 && aligned16(x) && aligned16(y) && x_rs % VE == 0 && y_rs % VE == 0;
  if (ADD) vec = vec && aligned16(res) && aligned16(nres) && res_rs % VE == 0 && nres_rs % VE == 0;
  RowPlan p = vec ? plan_rows(N / VE, fwd_min_threads(), tunable(MDY_TUNE_NORM_FWD_VPT), tunable(MDY_TUNE_NORM_FWD_GROUP))
                  : RowPlan{0, 0, 0, 0};
  const bool wvec = aligned16(w);
  if (p.vpt) {
    const int64_t grid = vec_grid(M, p, norm_ctas_per_sm() * (1024 / p.BT));
    const size_t sh = 2 * (p.BT / 32) * sizeof(float);
    // VPT 4 and 8 only occur with G == 1024 (one 1024-thread CTA per row); CTAs of up to 512
    // threads are compiled with a 128-register budget.
#define MDY_FWD(V, MT)                                                                           \
  norm_fwd_vec<T, V, ADD, MT><<<(unsigned)grid, p.BT, sh, st>>>(x, res, w, w_dtype, y, nres, rstd, \
                                                                M, (int)N, x_rs, res_rs, y_rs,   \
                                                                nres_rs, eps, p.G, wvec)
    if (p.BT <= 512) {
      if (p.vpt == 1) MDY_FWD(1, 512); else if (p.vpt == 2) MDY_FWD(2, 512); else MDY_FWD(4, 512);
    } else {
      switch (p.vpt) {
        case 1: case 2: MDY_FWD(2, 1024); break;
        case 4: MDY_FWD(4, 1024); break;
        default: MDY_FWD(8, 1024); break;
      }
    }
#undef MDY_FWD
  } else {
    norm_fwd_scalar<T, ADD><<<(unsigned)scalar_grid(M), 256, 0, st>>>(
        x, res, w, w_dtype, y, nres, rstd, M, N, x_rs, res_rs, y_rs, nres_rs, eps);
  }
  return finish_launch(1);
}

// Whether the 16-byte kernels can serve these buffers.
template <typename T>
inline bool bwd_vec_ok(const void* dy, const void* x, const void* dres, const void* dx, int64_t N, int64_t dy_rs,
                       int64_t x_rs, int64_t dres_rs, int64_t dx_rs) {
  constexpr int VE = VecInfo<T>::kElems;
  bool vec = N % VE == 0 && aligned16(dy) && aligned16(x) && aligned16(dx) && dy_rs % VE == 0 &&
             x_rs % VE == 0 && dx_rs % VE == 0;
  if (dres) vec = vec && aligned16(dres) && dres_rs % VE == 0;
  return vec;
}

template <typename T, bool ADD>
int launch_bwd(const BwdPlan& plan, const void* dy_, const void* x_, const void* w, int w_dtype, const float* rstd,
               const void* dres_, void* dx_, void* dw, float* dw_partial, int64_t M, int64_t N,
               int64_t dy_rs, int64_t x_rs, int64_t dres_rs, int64_t dx_rs, cudaStream_t st) {
  const T* dy = (const T*)dy_; const T* x = (const T*)x_;
  const T* dres = (const T*)dres_; T* dx = (T*)dx_;
  const RowPlan& p = plan.p;
  const int64_t grid = plan.grid;
  const bool wvec = aligned16(w);
  if (M == 0) {
    // nothing to sweep: the reduce below writes dw = 0
  } else if (plan.sp.ok) {
    if constexpr (sizeof(T) == 2) {
      StagedBwdArgs a;
      a.dy = dy; a.x = x; a.dres = ADD ? dres : nullptr; a.w = w; a.w_dtype = w_dtype; a.rstd = rstd; a.dx = dx;
      a.dw_partial = dw_partial; a.M = M; a.N = (int)N; a.dy_rs = dy_rs; a.x_rs = x_rs; a.dres_rs = dres_rs; a.dx_rs = dx_rs;
      a.team = plan.sp.team; a.stage_bytes = (int)plan.sp.stage_bytes; a.wait_tries = 1 << 20;
#define MDY_SBWD(V)                                                                                          \
  {                                                                                                          \
    auto kern = norm_bwd_staged<T, V, ADD>;                                                                  \
    cudaError_t e_ = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.sp.smem); \
    if (e_ != cudaSuccess) return (int)e_;                                                                   \
    kern<<<(unsigned)grid, kStagedThreads, plan.sp.smem, st>>>(a);                                           \
  }
      switch (plan.vpl) {
        case 2: MDY_SBWD(2) break;
        case 4: MDY_SBWD(4) break;
        case 8: MDY_SBWD(8) break;
        default: MDY_SBWD(16) break;
      }
#undef MDY_SBWD
    }
  } else if (p.vpt) {
    const size_t sh = (2 * (p.BT / 32) + (p.gpc > 1 ? N : 0)) * sizeof(float);
#define MDY_BWD(V, MT)                                                                          \
  norm_bwd_vec<T, V, ADD, MT><<<(unsigned)grid, p.BT, sh, st>>>(dy, x, w, w_dtype, rstd, dres,  \
                                                                dx, dw_partial, M, (int)N,      \
                                                                dy_rs, x_rs, dres_rs, dx_rs, p.G, wvec)
    if (p.BT <= 512) {
      if (p.vpt == 1) MDY_BWD(1, 512); else if (p.vpt == 2) MDY_BWD(2, 512); else MDY_BWD(4, 512);
    } else {
      switch (p.vpt) {
        case 1: case 2: MDY_BWD(2, 1024); break;
        case 4: MDY_BWD(4, 1024); break;
        default: MDY_BWD(8, 1024); break;
      }
    }
#undef MDY_BWD
  } else {
    norm_bwd_scalar<T, ADD><<<(unsigned)grid, 256, 0, st>>>(dy, x, w, w_dtype, rstd, dres, dx,
                                                           dw_partial, M, N, dy_rs, x_rs, dres_rs,
                                                           dx_rs);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  const int P = (int)grid;
  int rc = dispatch_dtype(w_dtype, [&](auto wtag) {
    using TW = decltype(wtag);
    dw_reduce<TW><<<(unsigned)ceil_div(N, 32), dim3(32, 32), 0, st>>>(dw_partial, (TW*)dw, P, N);
    return MDY_OK;
  });
  if (rc != MDY_OK) return rc;
  return finish_launch(M == 0 ? 1 : 2);
}

inline int check_mn(int64_t M, int64_t N) {
  if (M < 0 || N <= 0) return MDY_ERR_SIZE;
  if (N > (int64_t)1 << 30) return MDY_ERR_UNSUPPORTED;
  return MDY_OK;
}

inline bool dtype_ok(int d) { return d == MDY_F32 || d == MDY_F16 || d == MDY_BF16; }

// ---- scratch for mdy_rmsnorm_bwd_noalloc --------------------------------------------------------
// Lives in the library's device image: every GPU that loads the library holds these 16 MiB until the
// process exits.  In host code the NAME below is only a handle for the runtime, not a device address;
// the address a kernel can use comes from cudaGetSymbolAddress, asked once per device.
constexpr int64_t kNoAllocFloats = (int64_t)4 << 20;
static __device__ __align__(256) float g_noalloc_partials[kNoAllocFloats];

// Device address of the scratch on the current device (resolved on first use per device), or nullptr
// with *err set.  Not an allocation: the array already exists in the loaded module.
inline float* noalloc_scratch(cudaError_t* err) {
  static std::atomic<float*> ptrs[64];
  *err = cudaSuccess;
  int dev = 0;
  if ((*err = cudaGetDevice(&dev)) != cudaSuccess) return nullptr;
  if (dev < 0 || dev >= 64) { *err = cudaErrorInvalidDevice; return nullptr; }
  float* p = ptrs[dev].load(std::memory_order_acquire);
  if (p) return p;
  void* sym = nullptr;
  if ((*err = cudaGetSymbolAddress(&sym, g_noalloc_partials)) != cudaSuccess) return nullptr;
  p = static_cast<float*>(sym);
  ptrs[dev].store(p, std::memory_order_release);
  return p;
}

}  // namespace
}  // namespace mdy

namespace mdy {
int norm_dev_error(bool clear) { return read_dev_error(clear); }
}  // namespace mdy

using namespace mdy;

extern "C" {

int64_t mdy_rmsnorm_bwd_partial_rows(int64_t M, int64_t N, int dtype) {
  if (M <= 0 || N <= 0) return 1;
  int64_t rows = 1;
  int rc = dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    rows = partial_rows<T>(M, N);
    return MDY_OK;
  });
  return rc == MDY_OK ? rows : 1;
}

int mdy_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int64_t M, int64_t N,
                    int64_t x_row_stride, int64_t y_row_stride, float eps, int dtype, int w_dtype,
                    void* stream) {
  if (int rc = check_mn(M, N)) return rc;
  if (!dtype_ok(w_dtype)) return MDY_ERR_DTYPE;
  if (M == 0) return dtype_ok(dtype) ? MDY_OK : MDY_ERR_DTYPE;
  if (!x || !w || !y || !rstd) return MDY_ERR_NULL;
  if (x_row_stride < N || y_row_stride < N) return MDY_ERR_SIZE;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    return launch_fwd<T, false>(x, nullptr, w, w_dtype, y, nullptr, rstd, M, N, x_row_stride, 0,
                                y_row_stride, 0, eps, (cudaStream_t)stream);
  });
}

int mdy_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                    void* dw, float* dw_partial, int64_t M, int64_t N, int64_t dy_row_stride,
                    int64_t x_row_stride, int64_t dx_row_stride, int dtype, int w_dtype, void* stream) {
  if (int rc = check_mn(M, N)) return rc;
  if (!dtype_ok(w_dtype)) return MDY_ERR_DTYPE;
  if (!dw || !dw_partial || !w) return MDY_ERR_NULL;
  if (M > 0 && (!dy || !x || !rstd || !dx)) return MDY_ERR_NULL;
  if (dy_row_stride < 0 || x_row_stride < N || dx_row_stride < N) return MDY_ERR_SIZE;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    const BwdPlan plan = plan_bwd<T>(M, N, bwd_vec_ok<T>(dy, x, nullptr, dx, N, dy_row_stride, x_row_stride, 0, dx_row_stride), 2);
    return launch_bwd<T, false>(plan, dy, x, w, w_dtype, rstd, nullptr, dx, dw, dw_partial, M, N,
                                dy_row_stride, x_row_stride, 0, dx_row_stride, (cudaStream_t)stream);
  });
}

int mdy_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                            void* dw, int64_t M, int64_t N, int64_t dy_row_stride,
                            int64_t x_row_stride, int64_t dx_row_stride, int dtype, int w_dtype,
                            void* stream) {
  if (int rc = check_mn(M, N)) return rc;
  if (!dtype_ok(w_dtype) || !dtype_ok(dtype)) return MDY_ERR_DTYPE;
  if (!dw || !w) return MDY_ERR_NULL;
  if (M > 0 && (!dy || !x || !rstd || !dx)) return MDY_ERR_NULL;
  if (dy_row_stride < 0 || x_row_stride < N || dx_row_stride < N) return MDY_ERR_SIZE;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    // the grid is fixed here, once, and the same value is checked against the scratch and launched
    const BwdPlan plan = plan_bwd<T>(M, N, bwd_vec_ok<T>(dy, x, nullptr, dx, N, dy_row_stride, x_row_stride, 0, dx_row_stride), 2);
    if (plan.grid * N > kNoAllocFloats) return (int)MDY_ERR_UNSUPPORTED;  // would not fit the fixed scratch
    cudaError_t err;
    float* scratch = noalloc_scratch(&err);
    if (!scratch) {
      (void)cudaGetLastError();
      return err != cudaSuccess ? (int)err : (int)MDY_ERR_ARG;
    }
    return launch_bwd<T, false>(plan, dy, x, w, w_dtype, rstd, nullptr, dx, dw, scratch, M, N, dy_row_stride,
                                x_row_stride, 0, dx_row_stride, (cudaStream_t)stream);
  });
}

int mdy_add_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* new_res,
                        float* rstd, int64_t M, int64_t N, int64_t row_stride, float eps, int dtype,
                        int w_dtype, void* stream) {
  if (int rc = check_mn(M, N)) return rc;
  if (!dtype_ok(w_dtype)) return MDY_ERR_DTYPE;
  if (M == 0) return dtype_ok(dtype) ? MDY_OK : MDY_ERR_DTYPE;
  if (!x || !res || !w || !y || !new_res || !rstd) return MDY_ERR_NULL;
  if (row_stride < N) return MDY_ERR_SIZE;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    return launch_fwd<T, true>(x, res, w, w_dtype, y, new_res, rstd, M, N, row_stride, row_stride,
                               row_stride, row_stride, eps, (cudaStream_t)stream);
  });
}

int mdy_add_rmsnorm_bwd(const void* dy, const void* dnew_res, const void* new_res, const void* w,
                        const float* rstd, void* dx, void* dw, float* dw_partial, int64_t M, int64_t N,
                        int64_t row_stride, int dtype, int w_dtype, void* stream) {
  if (int rc = check_mn(M, N)) return rc;
  if (!dtype_ok(w_dtype)) return MDY_ERR_DTYPE;
  if (!dw || !dw_partial || !w) return MDY_ERR_NULL;
  if (M > 0 && (!dy || !new_res || !rstd || !dx)) return MDY_ERR_NULL;
  if (row_stride < N) return MDY_ERR_SIZE;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    const BwdPlan plan = plan_bwd<T>(M, N, bwd_vec_ok<T>(dy, new_res, dnew_res, dx, N, row_stride, row_stride, row_stride, row_stride), dnew_res ? 3 : 2);
    return launch_bwd<T, true>(plan, dy, new_res, w, w_dtype, rstd, dnew_res, dx, dw, dw_partial, M, N,
                               row_stride, row_stride, row_stride, row_stride, (cudaStream_t)stream);
  });
}

}  // extern "C"
