// One-pass cross-entropy with the row staged in shared memory across a thread-block cluster.
//
// A row of V logits (256 KB at V = 128256 in bf16) does not fit one SM's shared memory, so a cluster
// of C CTAs (C = 1..8, chosen so a slice is <= 200 KB) owns a row: CTA c keeps slice c of the row in
// its shared memory.  The slice is fetched by the bulk-copy engine (cp.async.bulk, one mbarrier per
// chunk) so HBM reads run ahead of the math without occupying registers.
//   sweep 1: as each chunk lands, every thread folds its 16 bytes into a running (max, sum-exp);
//            the CTA reduces through warp shuffles + shared memory, the CTAs of the cluster exchange
//            their partial (max, sum, label logit) through distributed shared memory.
//   sweep 2: the slice is read again FROM SHARED MEMORY, (softmax - onehot) * g is written to global
//            memory with streaming stores; as soon as a chunk has been consumed, the bulk copy of the
//            same chunk of the cluster's NEXT row is issued into it, so loads of row i+1 overlap the
//            exp/store work of row i.
// HBM therefore sees exactly one read and one write per logit, independent of L2 residency.
// Clusters are persistent and take rows round-robin; rows labelled MDY_IGNORE_INDEX are zero-filled
// without being read.  No multicast copy is used anywhere.
//
// Every wait on an mbarrier is bounded.  If one expires, the thread records a code in a device flag
// (mdy_last_device_error), stops waiting for the rest of the launch and keeps walking its rows, so its
// cluster peers still get every exchange message; the rows it touches from then on get NaN as loss and
// lse (the scalar loss of the batch becomes NaN, which a training loop notices without a sync), and
// before leaving it gives its own bulk copies time to land.  A logic error therefore shows up as a
// flagged NaN result, never as a hang and never as a finite wrong number.
#include <math.h>
#include "common.cuh"
#include "ce_common.cuh"

namespace mdy {
namespace {

constexpr int kMaxChunks = 32;
constexpr int kMaxCluster = 8;

thread_local int t_geometry[4] = {0, 0, 0, 0};  // cluster CTAs, clusters, threads, shared memory of the last launch

struct ClusterArgs {
  const void* logits; void* dlogits; const int64_t* labels; float* losses; float* lse;
  const float* gdev; float ghost;
  int M; int64_t V; int64_t rs;
  int C;        // CTAs per cluster
  int vpc;      // 16-byte vectors per CTA slice
  int slice_bytes_aligned;
  int slice_limit;    // largest slice in bytes (0: the knob or 200 KB)
  int wait_tries;     // tries of one bounded mbarrier wait
  int skip_clusters;  // test hook: the first chunk of the first row of this many clusters is never requested
};

#ifdef MDY_CE_TIMING
#define MDY_TICK(i) { const long long t_ = clock64(); tacc[i] += t_ - tlast; tlast = t_; }
#else
#define MDY_TICK(i)
#endif

// NT threads per CTA, VPC vectors per thread per chunk: a chunk is NT*VPC*16 bytes.
// FOLD: the gradient scale g is positive and finite, so (p - onehot)*g is computed as
// exp2(x*log2e - lse*log2e + log2 g) - onehot*g and costs no multiply per element.
template <typename T, int NT, int VPC, bool FOLD>
__device__ __forceinline__ void cluster_rows(const ClusterArgs& a, unsigned char* smem_raw, float g) {
  constexpr int VE = VecInfo<T>::kElems;
  constexpr int CV = NT * VPC;            // vectors per chunk
  constexpr int NW = NT / 32;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + a.slice_bytes_aligned);
  float* xchg = reinterpret_cast<float*>(full + kMaxChunks + 2);  // [2][kMaxCluster][4]; full[] is followed by xbar[2]
  float* red = xchg + 2 * kMaxCluster * 4;                         // [64]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t crank = cluster_ctarank();
  const int C = a.C;
  const int cid = blockIdx.x / C, ncl = gridDim.x / C;
  const int64_t nvec_total = a.V / VE;
  const int64_t v0 = (int64_t)crank * a.vpc;
  int my_nvec = (int)(nvec_total - v0 < a.vpc ? nvec_total - v0 : a.vpc);
  if (my_nvec < 0) my_nvec = 0;
  // chunks this CTA owns (the last CTA of a cluster may own fewer vectors than a.vpc); the first
  // `nfull` of them are complete, so their inner loops carry no bounds checks
  const int nchunk = (my_nvec + CV - 1) / CV;
  const int nfull = my_nvec / CV;
  const uint32_t slice_s = smem_u32(smem_raw);
  const uint32_t full_s = smem_u32(full);
  const T* logits = reinterpret_cast<const T*>(a.logits);
  T* dlogits = reinterpret_cast<T*>(a.dlogits);
  const float log2g = FOLD ? log2f(g) : 0.f;
  const int slice_elem0 = (int)(v0 * VE);   // first column of this CTA's slice

  // issue the bulk copy of chunk k of `row` into this CTA's slice (thread 0 only)
  auto issue_chunk = [&](int64_t row, int k) {
    const int first = k * CV;
    int nv = my_nvec - first;
    if (nv <= 0) return;
    if (nv > CV) nv = CV;
    const uint32_t bytes = (uint32_t)nv * 16u;
    const char* src = reinterpret_cast<const char*>(logits + row * a.rs) + (v0 + first) * 16;
    mbar_expect_tx(full_s + 8 * k, bytes);
    bulk_g2s(slice_s + (uint32_t)first * 16u, src, bytes, full_s + 8 * k);
  };

  int64_t row = cid;
  if (row < a.M && tid == 0 && a.labels[row] != MDY_IGNORE_INDEX) {
    for (int k = (crank == 0 && cid < a.skip_clusters) ? 1 : 0; k < nchunk; ++k) issue_chunk(row, k);
  }
  // rows that carried a label so far: selects the mbarrier phase and the exchange slot (two slots, so
  // a CTA that runs ahead cannot overwrite a slot its peer is still reading: it would first have to
  // pass the cluster barrier of the row in between)
  uint32_t nloaded = 0;
  bool dead = false;
  bool ready0 = false;  // early poll of the next row's first chunk
  const uint32_t my_s = slice_s + (uint32_t)tid * 16u;
#ifdef MDY_CE_TIMING
  long long tacc[6] = {0, 0, 0, 0, 0, 0};
  long long tlast = clock64();
#endif
  // labels are fetched two rows ahead, so the global load is never on the row's critical path
  int64_t label_after = MDY_IGNORE_INDEX;
  int64_t label = row < a.M ? a.labels[row] : MDY_IGNORE_INDEX;
  int64_t label_next = row + ncl < a.M ? a.labels[row + ncl] : MDY_IGNORE_INDEX;
  for (; row < a.M; row += ncl, label = label_next, label_next = label_after) {
    const bool cur_valid = label != MDY_IGNORE_INDEX;
    const int64_t nrow = row + ncl;
    const bool next_valid = nrow < a.M && label_next != MDY_IGNORE_INDEX;
    T* dst = dlogits + row * a.rs + (int64_t)slice_elem0 + (int64_t)tid * VE;

    if (!cur_valid) {
      // ignored row: nothing was loaded; zero-fill the slice and start fetching the next row
      label_after = nrow + ncl < a.M ? a.labels[nrow + ncl] : MDY_IGNORE_INDEX;
      if (crank == 0 && tid == 0) { a.losses[row] = 0.f; a.lse[row] = 0.f; }
      if (tid == 0 && next_valid) {
        for (int k = 0; k < nchunk; ++k) issue_chunk(nrow, k);
      }
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int v = tid; v < my_nvec; v += NT) st_stream(dst + (int64_t)(v - tid) * VE, z);
      ready0 = false;
      continue;
    }

    MDY_TICK(0)
    // ---- sweep 1: (max, sum-exp) of the slice as its chunks land ----
    const uint32_t parity = nloaded & 1u;
    float m = -INFINITY, s0 = 0.f, s1 = 0.f;
    // every chunk barrier is polled one chunk ahead (the first one at the end of the previous row), so
    // the poll's latency overlaps the exponentials; the blocking wait only runs if that poll failed
    bool ready = ready0;
    for (int k = 0; k < nfull; ++k) {
      if (!ready) mbar_wait(full_s + 8 * k, parity, dead, a.wait_tries);
      uint4 q[VPC];
#pragma unroll
      for (int j = 0; j < VPC; ++j) q[j] = lds128(my_s + (uint32_t)(k * CV + j * NT) * 16u);
      ready = k + 1 < nchunk && mbar_test(full_s + 8 * (k + 1), parity);
      stats_chunk<T, VPC>(q, m, s0, s1);
    }
    if (nfull < nchunk) {
      if (!ready) mbar_wait(full_s + 8 * nfull, parity, dead, a.wait_tries);
      uint4 q[VPC];
#pragma unroll
      for (int j = 0; j < VPC; ++j) {
        const int vb = nfull * CV + j * NT;
        q[j] = vb + tid < my_nvec ? lds128(my_s + (uint32_t)vb * 16u) : neg_inf_vec<T>();
      }
      stats_chunk<T, VPC>(q, m, s0, s1);
    }
    MDY_TICK(1)
    float s = s0 + s1;
    group_merge<32>(m, s);
    if (lane == 0) { red[warp] = m; red[32 + warp] = s; }
    int loc = -1;  // label position inside this CTA's slice, in elements
    if (label >= 0 && label < a.V) {
      const int64_t l = label - slice_elem0;
      if (l >= 0 && l < (int64_t)my_nvec * VE) loc = (int)l;
    }
    // warp 0 waits for every warp's partial, the others only signal and move on
    if (warp == 0) {
      named_sync(NT);
      MDY_TICK(2)
      m = lane < NW ? red[lane] : -INFINITY;
      s = lane < NW ? red[32 + lane] : 0.f;
      group_merge<(NW <= 8 ? 8 : NW <= 16 ? 16 : 32)>(m, s);
      if (lane == 0) {
        // (max, sum, label logit) to every CTA of the cluster, itself included: 16 bytes that complete
        // 16 tx bytes on the receiver's exchange barrier (no cluster-wide barrier or fence per row)
        const float xl = loc >= 0 ? to_float(reinterpret_cast<const T*>(smem_raw)[loc]) : 0.f;
        const uint32_t xb = full_s + 8 * (kMaxChunks + (nloaded & 1u));
        const uint32_t slot = smem_u32(xchg + ((int)(nloaded & 1u) * kMaxCluster + (int)crank) * 4);
        mbar_expect_tx(xb, (uint32_t)C * 16u);
        for (int p = 0; p < C; ++p) st_async_v4(slot, xb, (uint32_t)p, m, s, xl, dead ? NAN : 0.f);
      }
    } else {
      named_arrive(NT);
      MDY_TICK(2)
    }
    // two exchange slots suffice: a peer cannot send for row n+2 before it has this CTA's message for
    // row n+1, which leaves only after the reads of row n below
    mbar_wait(full_s + 8 * (kMaxChunks + (nloaded & 1u)), (nloaded >> 1) & 1u, dead, a.wait_tries);
    MDY_TICK(3)
    float gm = -INFINITY, gs = 0.f, xl = 0.f;
    float poison = dead ? NAN : 0.f;  // NaN once a wait of this thread or of a sending peer has expired
    {
      const float* x = xchg + (int)(nloaded & 1u) * kMaxCluster * 4;
      for (int p = 0; p < C; ++p) {
        merge_nb(gm, gs, x[p * 4], x[p * 4 + 1]);
        xl += x[p * 4 + 2];
        poison += x[p * 4 + 3];
      }
    }
    const float lse = gm + logf(gs) + poison;
    if (crank == 0 && tid == 0) {
      a.losses[row] = (label >= 0 && label < a.V) ? lse - xl : 0.f;
      a.lse[row] = lse;
    }
    ++nloaded;
    // the label two rows ahead is fetched here: a global load in flight when sweep 1 polls its chunk
    // barriers was measured to delay those polls by its whole latency
    label_after = nrow + ncl < a.M ? a.labels[nrow + ncl] : MDY_IGNORE_INDEX;

    // ---- sweep 2: gradient from the staged slice; refill each chunk as soon as it is consumed ----
    const float c2 = -lse * kLog2e + log2g;
    for (int k = 0; k < nfull; ++k) {
      uint4 q[VPC];
#pragma unroll
      for (int j = 0; j < VPC; ++j) q[j] = lds128(my_s + (uint32_t)(k * CV + j * NT) * 16u);
      __syncthreads();  // chunk k is now in registers everywhere: its buffer may be refilled
      if (tid == 0 && next_valid) issue_chunk(nrow, k);
#pragma unroll
      for (int j = 0; j < VPC; ++j) st_stream(dst + (int64_t)(k * CV + j * NT) * VE, grad_vec<T, FOLD>(q[j], c2, g));
    }
    if (nfull < nchunk) {
      uint4 q[VPC];
#pragma unroll
      for (int j = 0; j < VPC; ++j) {
        const int vb = nfull * CV + j * NT;
        q[j] = vb + tid < my_nvec ? lds128(my_s + (uint32_t)vb * 16u) : make_uint4(0, 0, 0, 0);
      }
      __syncthreads();
      if (tid == 0 && next_valid) issue_chunk(nrow, nfull);
#pragma unroll
      for (int j = 0; j < VPC; ++j) {
        const int vb = nfull * CV + j * NT;
        if (vb + tid < my_nvec) st_stream(dst + (int64_t)vb * VE, grad_vec<T, FOLD>(q[j], c2, g));
      }
    }
    // the label's element is (p - 1)*g: the thread that stored its vector overwrites that one element
    // (same thread, same address: program order keeps the later store)
    if (loc >= 0 && ((loc / VE) % NT) == tid) {
      const float p = fast_exp2(fmaf(xl, kLog2e, -lse * kLog2e));
      dlogits[row * a.rs + slice_elem0 + loc] = from_float<T>((p - 1.f) * g);
    }
    ready0 = next_valid && mbar_test(full_s, nloaded & 1u);
    MDY_TICK(4)
  }
  if (dead) {
    // this thread no longer follows the chunk barriers: idle long enough (about 100 us) for any bulk copy
    // still in flight into this CTA's shared memory to land before the CTA may leave
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  }
#ifdef MDY_CE_TIMING
  if (blockIdx.x < 8 && (tid == 0 || tid == 40 || tid == NT - 1)) {
    float* o = a.lse + a.M + (blockIdx.x * 3 + (tid == 0 ? 0 : tid == 40 ? 1 : 2)) * 8;
    for (int i = 0; i < 5; ++i) o[i] = (float)tacc[i];
    o[5] = (float)nloaded;
  }
#endif
}

template <typename T, int NT, int VPC, int MINB>
__global__ void __launch_bounds__(NT, MINB) ce_cluster_kernel(ClusterArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const uint32_t full_s = smem_u32(smem_raw + a.slice_bytes_aligned);
  if (threadIdx.x == 0) {
    for (int k = 0; k < kMaxChunks + 2; ++k) mbar_init(full_s + 8 * k, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // every CTA of the cluster must be running before anyone writes into a peer's shared memory
  cluster_sync_all();
  const float g = a.ghost * (a.gdev ? *a.gdev : 1.f);
  if (g > 0.f && g < INFINITY) cluster_rows<T, NT, VPC, true>(a, smem_raw, g);
  else cluster_rows<T, NT, VPC, false>(a, smem_raw, g);
  // No CTA leaves while a peer may still send it an exchange message: in a healthy run every CTA has
  // received all of them by now; a CTA whose waits expired stopped waiting for them and would otherwise
  // exit early.  All CTAs of a cluster walk the same rows, so the barrier is reached by all.
  cluster_sync_all();
}

inline int cluster_slice_limit() {
  int kb = tunable(MDY_TUNE_CE_CLUSTER_SLICE_KB);
  if (kb < 8 || kb > 220) kb = 200;
  return kb * 1024;
}

template <typename T, int NT, int VPC, int MINB>
int launch_cluster_nt(ClusterArgs a, cudaStream_t st) {
  constexpr int VE = VecInfo<T>::kElems;
  const int64_t row_bytes = a.V * (int64_t)sizeof(T);
  const int64_t nvec = a.V / VE;
  int C = (int)ceil_div(row_bytes, a.slice_limit > 0 ? a.slice_limit : cluster_slice_limit());
  if (C > kMaxCluster) {
    // rows too long for 8 small slices: grow the slice up to what one CTA per SM can hold
    C = kMaxCluster;
    if (ceil_div(row_bytes, C) > 200 * 1024) return MDY_ERR_UNSUPPORTED;
  }
  const int64_t vpc = ceil_div(nvec, C);
  if ((int64_t)(C - 1) * vpc >= nvec) return MDY_ERR_UNSUPPORTED;  // a CTA would own nothing
  a.C = C;
  a.vpc = (int)vpc;
  const int hook = tunable(MDY_TUNE_CE_WAIT_TEST);
  a.wait_tries = hook > 0 ? (1 << 10) : (1 << 20);
  a.skip_clusters = hook > 0 ? hook : 0;
  if (ceil_div(vpc, NT * VPC) > kMaxChunks) return MDY_ERR_UNSUPPORTED;
  a.slice_bytes_aligned = (int)((vpc * 16 + 127) / 128 * 128);
  const size_t smem = (size_t)a.slice_bytes_aligned + (kMaxChunks + 2) * 8 + 2 * kMaxCluster * 4 * 4 + 64 * 4;

  auto kern = ce_cluster_kernel<T, NT, VPC, MINB>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return MDY_ERR_UNSUPPORTED; }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = C; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(NT, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(C, 1, 1);
  // co-resident clusters for this (device, kernel, cluster size, shared memory) — queried once and reused
  static thread_local int c_dev = -1, c_C = 0, c_max = 0;
  static thread_local size_t c_smem = 0;
  int dev = 0;
  (void)cudaGetDevice(&dev);
  int max_clusters = 0;
  if (dev == c_dev && C == c_C && smem == c_smem) {
    max_clusters = c_max;
  } else {
    e = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);
    if (e != cudaSuccess || max_clusters < 1) { (void)cudaGetLastError(); return MDY_ERR_UNSUPPORTED; }
    c_dev = dev; c_C = C; c_smem = smem; c_max = max_clusters;
  }
  int64_t ncl = a.M < max_clusters ? a.M : max_clusters;
  cfg.gridDim = dim3((unsigned)(ncl * C), 1, 1);
  e = cudaLaunchKernelEx(&cfg, kern, a);
  if (e != cudaSuccess) return (int)e;
  t_geometry[0] = C; t_geometry[1] = (int)ncl; t_geometry[2] = NT; t_geometry[3] = (int)smem;
  return finish_launch(1);
}

template <typename T>
int launch_cluster(const ClusterArgs& a, cudaStream_t st) {
  constexpr int VE = VecInfo<T>::kElems;
  if (a.V % VE != 0 || a.rs % VE != 0 || !aligned16(a.logits) || !aligned16(a.dlogits)) return MDY_ERR_UNSUPPORTED;
  if (a.V >= ((int64_t)1 << 27)) return MDY_ERR_UNSUPPORTED;
  const int nt = tunable(MDY_TUNE_CE_CLUSTER_THREADS);
  const int vpc = tunable(MDY_TUNE_CE_CLUSTER_VPC);
  int minb = tunable(MDY_TUNE_CE_CLUSTER_MINB);
  if (minb < 1) minb = 1;
#define MDY_CL(NT_, VPC_, MINB_) \
  if (nt == NT_ && vpc == VPC_ && minb == MINB_) return launch_cluster_nt<T, NT_, VPC_, MINB_>(a, st);
  MDY_CL(256, 4, 3) MDY_CL(256, 8, 2) MDY_CL(512, 2, 2) MDY_CL(512, 4, 1) MDY_CL(1024, 2, 1)
#undef MDY_CL
  // defaults (measured at 32768 rows, bf16).  Rows of which two or three fit in one SM's shared memory:
  // small CTAs, several per SM, so one row's reduction and exchange overlap another row's sweeps
  // (V = 32000: 6000 GB/s against 4360 with one large CTA).  Longer rows: one 512-thread CTA per SM with
  // up to 128 registers per thread and 32 KB chunks (V = 128256: 6040 GB/s; 1024 threads: 5440).
  if (a.V * (int64_t)sizeof(T) <= 112 * 1024 && tunable(MDY_TUNE_CE_CLUSTER_SLICE_KB) == 0)
    return launch_cluster_nt<T, 256, 4, 3>(a, st);
  // Rows so long that they need clusters of three or more 200 KB slices (V = 256000: 500 KB) leave SMs idle,
  // because such clusters do not tile the GPU (45 clusters of 3 = 135 of 148 SMs).  Clusters of 8 CTAs with
  // 64 KB slices, three 256-thread CTAs per SM, fill it better (48 clusters; V = 256000: 5276 against 5180 GB/s).
  if (a.V * (int64_t)sizeof(T) > 400 * 1024 && tunable(MDY_TUNE_CE_CLUSTER_SLICE_KB) == 0) {
    ClusterArgs b = a;
    b.slice_limit = 64 * 1024;
    const int rc = launch_cluster_nt<T, 256, 4, 3>(b, st);
    if (rc != MDY_ERR_UNSUPPORTED) return rc;
  }
  return launch_cluster_nt<T, 512, 4, 1>(a, st);
}

}  // namespace

int ce_fused_cluster(const void* logits, void* dlogits, const int64_t* labels, float* losses, float* lse,
                     const float* gdev, float ghost, int64_t M, int64_t V, int64_t rs, int dtype,
                     cudaStream_t st) {
  ClusterArgs a;
  a.logits = logits; a.dlogits = dlogits; a.labels = labels; a.losses = losses; a.lse = lse;
  a.gdev = gdev; a.ghost = ghost; a.M = (int)M; a.V = V; a.rs = rs;
  a.C = 0; a.vpc = 0; a.slice_bytes_aligned = 0; a.slice_limit = 0; a.wait_tries = 1 << 20; a.skip_clusters = 0;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    return launch_cluster<T>(a, st);
  });
}

}  // namespace mdy

extern "C" int mdy_ce_last_geometry(int* cluster_ctas, int* clusters, int* threads, int* smem_bytes) {
  if (mdy::t_geometry[0] == 0) return MDY_ERR_ARG;
  if (cluster_ctas) *cluster_ctas = mdy::t_geometry[0];
  if (clusters) *clusters = mdy::t_geometry[1];
  if (threads) *threads = mdy::t_geometry[2];
  if (smem_bytes) *smem_bytes = mdy::t_geometry[3];
  return MDY_OK;
}

namespace mdy {
int ce_cluster_dev_error(bool clear) { return read_dev_error(clear); }
int ce_vp_dev_error(bool clear);  // ce_vp_fused.cu
int ce_vp_dev_detail(int k, bool clear);
int norm_dev_error(bool clear);   // rmsnorm.cu
}  // namespace mdy

extern "C" int mdy_device_error_of(int source, int clear) {
  switch (source) {
    case 0: return mdy::ce_cluster_dev_error(clear != 0);
    case 1: return mdy::ce_vp_dev_error(clear != 0);
    case 2: return mdy::norm_dev_error(clear != 0);
    case 16: case 17: case 18: case 19: return mdy::ce_vp_dev_detail(source - 16, clear != 0);
    default: return MDY_ERR_ARG;
  }
}

extern "C" int mdy_last_device_error(int clear) {
  const int a = mdy::ce_cluster_dev_error(clear != 0);
  const int b = mdy::ce_vp_dev_error(clear != 0);
  const int c = mdy::norm_dev_error(clear != 0);
  if (a < 0 || b < 0 || c < 0) return -1;
  return a > b ? (a > c ? a : c) : (b > c ? b : c);
}
