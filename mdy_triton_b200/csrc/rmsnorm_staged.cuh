// RMSNorm / add+RMSNorm backward with the rows staged in shared memory by the bulk-copy engine.
//
// The register-resident kernels in rmsnorm.cu keep a row in registers, so the bytes a thread has in
// flight are bounded by its registers: one row ahead at most.  For the backward of long rows (two or
// three input streams, 127 registers, one CTA per SM) that leaves HBM short of requests: 0.69-0.76 of
// the copy bandwidth at hidden 3584-4096.  Here the loads are issued by ONE thread as bulk copies
// (cp.async.bulk, completion on an mbarrier) into two stages of shared memory, each holding one row per
// team for every input stream: while the CTA computes on one stage the copy engine fills the other, so
// the bytes in flight are set by shared memory (a 56-112 KB stage per SM), not by registers
// (measured: 131 against 156 us at [32768, 3584], 143 against 163 us at [32768, 4096]).
// The forward (one or two streams) gains nothing from staging (91 us either way at [32768, 3584]) and
// short rows lose, so both stay with the register-resident kernels.
//
// A row is owned by a TEAM of 2 or 4 warps (lane l of warp t holds vectors t*32 + l, then every
// 32*TEAM-th): row reductions are warp shuffles plus one named barrier of the team.  The CTA (8 warps)
// meets at ONE __syncthreads per stage, to hand the stage back to the copy engine.  Rows are read twice
// from shared memory (statistics, then output); each lane keeps its slice of the weight and of dw in
// registers (VPL vectors); the CTA's teams are folded through shared memory at the end into one partial
// row per CTA.
#pragma once
#include "ce_common.cuh"

namespace mdy {
namespace {

constexpr int kStagedWarps = 8;
constexpr int kStagedThreads = kStagedWarps * 32;

struct StagedPlan {
  bool ok;
  int team;          // warps per row: 2 or 4
  int streams;       // input streams staged per row
  int64_t stage_bytes;
  size_t smem;
  int ctas_per_sm;
};

// Team width and stage size for rows of `row_bytes` bytes with `streams` input streams: two warps per
// row where two stages of four rows fit (measured best at hidden 3584 and 4096), else four.
inline StagedPlan plan_staged(int64_t row_bytes, int streams, int force_team) {
  const int64_t budget = 225 * 1024;
  for (int team = 2; team <= 4; team <<= 1) {
    if (force_team > 0 && team != force_team) continue;
    const int64_t stage = row_bytes * streams * (kStagedWarps / team);
    const int64_t smem = 2 * stage + 256;
    if (smem > budget) continue;
    int per_sm = (int)(budget / (smem + 1024));
    if (per_sm > 4) per_sm = 4;
    return StagedPlan{true, team, streams, stage, (size_t)smem, per_sm};
  }
  return StagedPlan{false, 0, streams, 0, 0, 0};
}

// Sum over the team that owns a row.  tred: [2][kStagedWarps] floats, `parity` alternates per row.
__device__ __forceinline__ float team_sum(float v, float* tred, int team_w, int team_id, int warp, int parity) {
  v = warp_sum(v);
  if (team_w == 1) return v;
  float* slot = tred + parity * kStagedWarps;
  if ((threadIdx.x & 31) == 0) slot[warp] = v;
  asm volatile("bar.sync %0, %1;" ::"r"(1 + team_id), "r"(32 * team_w) : "memory");
  float s = 0.f;
  for (int k = 0; k < team_w; ++k) s += slot[team_id * team_w + k];
  return s;
}

struct StagedBwdArgs {
  const void* dy; const void* x; const void* dres; const void* w; int w_dtype; const float* rstd;
  void* dx; float* dw_partial;
  int64_t M; int N; int64_t dy_rs, x_rs, dres_rs, dx_rs;
  int team; int stage_bytes; int wait_tries;
};

// VPL: vectors per lane (compile time: each lane's dw slice lives in VPL * VE float registers).
template <typename T, int VPL, bool ADD>
__global__ void __launch_bounds__(kStagedThreads) norm_bwd_staged(StagedBwdArgs a) {
  constexpr int VE = VecInfo<T>::kElems;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int N = a.N, nvec = N / VE;
  const int row_bytes = N * (int)sizeof(T);
  unsigned char* stages = smem_raw;
  uint64_t* full = reinterpret_cast<uint64_t*>(stages + 2 * (size_t)a.stage_bytes);
  float* tred = reinterpret_cast<float*>(full + 2);
  const uint32_t full_s = smem_u32(full), stages_s = smem_u32(stages);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int TW = a.team, RB = kStagedWarps / TW;
  const int team_id = warp / TW, wt = warp - team_id * TW;
  const int lane_t = wt * 32 + lane, stride_v = 32 * TW;
  const T* x = reinterpret_cast<const T*>(a.x);
  const T* dy = reinterpret_cast<const T*>(a.dy);
  const T* dres = reinterpret_cast<const T*>(a.dres);
  T* dx = reinterpret_cast<T*>(a.dx);
  const bool has_dres = ADD && a.dres != nullptr;
  const uint32_t nstreams = has_dres ? 3u : 2u;
  const bool wvec = (reinterpret_cast<uintptr_t>(a.w) & 15u) == 0;

  if (tid == 0) {
    mbar_init(full_s, 1); mbar_init(full_s + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  auto copy_rows = [&](uint32_t dst, const T* src, int64_t rs, int64_t row0, int nrows, uint32_t bar) {
    if (rs == N) {
      bulk_g2s(dst, src + row0 * rs, (uint32_t)nrows * row_bytes, bar);
    } else {
      for (int r = 0; r < nrows; ++r) bulk_g2s(dst + (uint32_t)r * row_bytes, src + (row0 + r) * rs, row_bytes, bar);
    }
  };
  auto issue_block = [&](int kl) {
    const int64_t row0 = ((int64_t)blockIdx.x + (int64_t)kl * gridDim.x) * RB;
    if (row0 >= a.M) return;
    const int nrows = (int)(a.M - row0 < RB ? a.M - row0 : RB);
    const int s = kl & 1;
    const uint32_t bar = full_s + 8 * s;
    const uint32_t dst = stages_s + (uint32_t)s * a.stage_bytes;
    mbar_expect_tx(bar, (uint32_t)nrows * row_bytes * nstreams);
    copy_rows(dst, x, a.x_rs, row0, nrows, bar);
    copy_rows(dst + (uint32_t)RB * row_bytes, dy, a.dy_rs, row0, nrows, bar);
    if (has_dres) copy_rows(dst + 2u * RB * row_bytes, dres, a.dres_rs, row0, nrows, bar);
  };
  if (tid == 0) { issue_block(0); issue_block(1); }

  // the weight slice of this lane stays in registers across the rows
  float wf[VPL][VE], acc[VPL][VE];
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int v = lane_t + stride_v * j;
    if (v < nvec) load_w_vec<VE>(a.w, v, a.w_dtype, wvec, wf[j]);
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      if (v >= nvec) wf[j][e] = 0.f;
      acc[j][e] = 0.f;
    }
  }
  const float inv_n = 1.f / (float)N;
  bool dead = false;
  // rstd of this team's row one block ahead, so the load is never waited for
  float rs_next = 0.f;
  {
    const int64_t row = (int64_t)blockIdx.x * RB + team_id;
    if (row < a.M) rs_next = a.rstd[row];
  }
  for (int kl = 0;; ++kl) {
    const int64_t row0 = ((int64_t)blockIdx.x + (int64_t)kl * gridDim.x) * RB;
    if (row0 >= a.M) break;
    const float rstd = rs_next;
    const int s = kl & 1;
    mbar_wait(full_s + 8 * s, (uint32_t)(kl >> 1) & 1u, dead, a.wait_tries);
    {
      // issued after the wait: a global load in flight delays a poll of an mbarrier by its whole latency
      const int64_t nrow = row0 + (int64_t)gridDim.x * RB + team_id;
      rs_next = nrow < a.M ? a.rstd[nrow] : 0.f;
    }
    const int64_t row = row0 + team_id;
    if (row < a.M) {
      const uint4* xr = reinterpret_cast<const uint4*>(stages + (size_t)s * a.stage_bytes + (size_t)team_id * row_bytes) + lane_t;
      const uint4* gr = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(xr) + (size_t)RB * row_bytes);
      const uint4* dr = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(gr) + (size_t)RB * row_bytes);
      // two vectors at a time (x and dy of both loaded before either is used), the row dot product in four
      // independent chains
      float dot4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j0 = 0; j0 < VPL; j0 += 2) {
        uint4 qx[2], qg[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const bool on = j0 + u < VPL && lane_t + stride_v * (j0 + u) < nvec;
          qx[u] = on ? xr[stride_v * (j0 + u)] : make_uint4(0, 0, 0, 0);
          qg[u] = on ? gr[stride_v * (j0 + u)] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (j0 + u < VPL) {
            float xf[VE], gf[VE];
            unpack<T>(qx[u], xf);
            unpack<T>(qg[u], gf);
#pragma unroll
            for (int e = 0; e < VE; ++e) {
              const float xhat = xf[e] * rstd;
              acc[j0 + u][e] = fmaf(xhat, gf[e], acc[j0 + u][e]);
              dot4[(u * 2 + (e & 1)) & 3] = fmaf(xhat, wf[j0 + u][e] * gf[e], dot4[(u * 2 + (e & 1)) & 3]);
            }
          }
        }
      }
      const float dot = team_sum((dot4[0] + dot4[1]) + (dot4[2] + dot4[3]), tred, TW, team_id, warp, kl & 1);
      const float c = dot * inv_n;
#pragma unroll
      for (int j0 = 0; j0 < VPL; j0 += 2) {
        uint4 qx[2], qg[2], qd[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const bool on = j0 + u < VPL && lane_t + stride_v * (j0 + u) < nvec;
          qx[u] = on ? xr[stride_v * (j0 + u)] : make_uint4(0, 0, 0, 0);
          qg[u] = on ? gr[stride_v * (j0 + u)] : make_uint4(0, 0, 0, 0);
          qd[u] = (on && has_dres) ? dr[stride_v * (j0 + u)] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int v = lane_t + stride_v * (j0 + u);
          if (j0 + u < VPL && v < nvec) {
            float xf[VE], gf[VE], o[VE];
            unpack<T>(qx[u], xf);
            unpack<T>(qg[u], gf);
#pragma unroll
            for (int e = 0; e < VE; ++e) o[e] = (wf[j0 + u][e] * gf[e] - xf[e] * rstd * c) * rstd;
            if (ADD) {
              float df[VE];
              unpack<T>(qd[u], df);
#pragma unroll
              for (int e = 0; e < VE; ++e) o[e] += df[e];
            }
            st_stream(dx + row * a.dx_rs + (int64_t)v * VE, pack<T>(o));
          }
        }
      }
    }
    __syncthreads();
    if (tid == 0) issue_block(kl + 2);
  }
  if (dead) {
    for (int k = 0; k < 100; ++k) __nanosleep(1000);
  }
  // fold the teams' dw slices through shared memory (the stages are free now) into one partial row
  __syncthreads();
  float* colsum = reinterpret_cast<float*>(stages);
  for (int tsel = 0; tsel < RB; ++tsel) {
    if (team_id == tsel) {
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        const int v = lane_t + stride_v * j;
        if (v < nvec) {
#pragma unroll
          for (int e = 0; e < VE; ++e) {
            if (tsel == 0) colsum[v * VE + e] = acc[j][e];
            else colsum[v * VE + e] += acc[j][e];
          }
        }
      }
    }
    __syncthreads();
  }
  float* out = a.dw_partial + (int64_t)blockIdx.x * N;
  for (int cidx = tid; cidx < N; cidx += kStagedThreads) out[cidx] = colsum[cidx];
}

}  // namespace
}  // namespace mdy
