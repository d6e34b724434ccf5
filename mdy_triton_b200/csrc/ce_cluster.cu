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
// Every wait on an mbarrier is bounded: if it expires the kernel records a code in a device flag
// (mdy_last_device_error) and carries on, so a logic error shows up as a flagged wrong result, never
// as a hang.
#include <math.h>
#include "common.cuh"

namespace mdy {
namespace {

constexpr int kMaxChunks = 32;
constexpr int kMaxCluster = 8;

__device__ int g_dev_error = 0;
thread_local int t_geometry[4] = {0, 0, 0, 0};  // cluster CTAs, clusters, threads, shared memory of the last launch

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// `dead` is per-thread state: after one wait has expired the thread stops waiting altogether, so a
// broken pipeline costs one bounded wait in total, not one per chunk and row.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, bool& dead) {
  if (dead) return;
  // each try_wait may suspend for up to ~1 us; 2^20 tries bound the wait to about a second
  for (int i = 0; i < (1 << 20); ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(1000u)
        : "memory");
    if (ok) return;
  }
  dead = true;
  atomicExch(&g_dev_error, 1);
}
// Non-blocking poll: true once the phase with this parity has completed.  Issued well before its result
// is needed, its latency (about 200 cycles, measured) overlaps other work.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// global -> this CTA's shared memory, completion signalled on `bar` (non-multicast bulk copy)
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// 16 bytes into CTA `rank`'s shared memory at the same offset as `local_addr`, completing 16 tx bytes
// on that CTA's mbarrier at the same offset as `local_bar`: data and signal travel together, so the
// receiver needs no cluster-wide barrier or fence (a release fence would also wait for the sender's
// outstanding gradient stores to global memory).
__device__ __forceinline__ void st_async_v4(uint32_t local_addr, uint32_t local_bar, uint32_t rank, float a, float b,
                                            float c, float d) {
  uint32_t ra, rb;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local_addr), "r"(rank));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rb) : "r"(local_bar), "r"(rank));
  asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(ra),
               "f"(a), "f"(b), "f"(c), "f"(d), "r"(rb)
               : "memory");
}

// Named barrier 1 as a producer/consumer pair: `named_arrive` signals without waiting, `named_sync`
// waits until `count` threads have arrived or synced; writes made before the arrive are visible after
// the sync.
__device__ __forceinline__ void named_arrive(int count) {
  asm volatile("bar.arrive 1, %0;" ::"r"(count) : "memory");
}
__device__ __forceinline__ void named_sync(int count) {
  asm volatile("bar.sync 1, %0;" ::"r"(count) : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// A 16-byte vector whose every element is -inf: padding that changes neither a max nor a sum of exps.
template <typename T> __device__ __forceinline__ uint4 neg_inf_vec();
template <> __device__ __forceinline__ uint4 neg_inf_vec<float>() { return make_uint4(0xff800000u, 0xff800000u, 0xff800000u, 0xff800000u); }
template <> __device__ __forceinline__ uint4 neg_inf_vec<__nv_bfloat16>() { return make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u); }
template <> __device__ __forceinline__ uint4 neg_inf_vec<__half>() { return make_uint4(0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u); }

// max of the elements of one vector, using packed 16-bit max where the type allows (4 instead of 7
// float max operations per 8 elements)
template <typename T> __device__ __forceinline__ float vec_max(const uint4& q);
template <> __device__ __forceinline__ float vec_max<float>(const uint4& q) {
  return fmaxf(fmaxf(__uint_as_float(q.x), __uint_as_float(q.y)), fmaxf(__uint_as_float(q.z), __uint_as_float(q.w)));
}
template <> __device__ __forceinline__ float vec_max<__nv_bfloat16>(const uint4& q) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
  const __nv_bfloat162 a = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
  const uint32_t w = *reinterpret_cast<const uint32_t*>(&a);
  return fmaxf(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float vec_max<__half>(const uint4& q) {
  const __half2* h = reinterpret_cast<const __half2*>(&q);
  const __half2 a = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
  return fmaxf(__low2float(a), __high2float(a));
}

struct ClusterArgs {
  const void* logits; void* dlogits; const int64_t* labels; float* losses; float* lse;
  const float* gdev; float ghost;
  int M; int64_t V; int64_t rs;
  int C;        // CTAs per cluster
  int vpc;      // 16-byte vectors per CTA slice
  int slice_bytes_aligned;
};

#ifdef MDY_CE_TIMING
#define MDY_TICK(i) { const long long t_ = clock64(); tacc[i] += t_ - tlast; tlast = t_; }
#else
#define MDY_TICK(i)
#endif

// Branch-free merge of (m, s) with (om, os): one exp, no divergence.  Maxima are clamped to -1e37 so
// two empty operands (-inf, 0) do not produce inf - inf.
__device__ __forceinline__ void merge_nb(float& m, float& s, float om, float os) {
  const float a = fmaxf(m, -1e37f), b = fmaxf(om, -1e37f);
  const float e = fast_exp2(-fabsf(a - b) * kLog2e);
  s = (a >= b) ? fmaf(os, e, s) : fmaf(s, e, os);
  m = fmaxf(m, om);
}

// (max, sum-exp) over groups of W adjacent lanes, left in every lane of the group: a max butterfly, ONE
// rescale per lane, a sum butterfly (a shorter dependency chain than log2(W) merges with an exp each).
template <int W>
__device__ __forceinline__ void group_merge(float& m, float& s) {
  float gm = m;
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, o));
  s *= fast_exp2((fmaxf(m, -1e37f) - fmaxf(gm, -1e37f)) * kLog2e);  // an empty lane's s == 0 stays 0
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  m = gm;
}

// Sweep-1 work on VPC vectors already in registers: one max/rescale per call, then 8*VPC exps
// accumulated in two independent sums.
template <typename T, int VPC>
__device__ __forceinline__ void stats_chunk(const uint4 (&q)[VPC], float& m, float& s0, float& s1) {
  constexpr int VE = VecInfo<T>::kElems;
  float vm = vec_max<T>(q[0]);
#pragma unroll
  for (int j = 1; j < VPC; ++j) vm = fmaxf(vm, vec_max<T>(q[j]));
  if (vm > m) {  // rare after the first chunks
    const float r = fast_exp2((fmaxf(m, -1e37f) - vm) * kLog2e);  // empty so far: s == 0, r == 0
    s0 *= r; s1 *= r;
    m = vm;
  }
  const float nm2 = -fmaxf(m, -1e37f) * kLog2e;  // finite even when everything so far is -inf
#pragma unroll
  for (int j = 0; j < VPC; ++j) {
    float f[VE];
    unpack<T>(q[j], f);
#pragma unroll
    for (int e = 0; e < VE; e += 2) {
      s0 += fast_exp2(fmaf(f[e], kLog2e, nm2));
      s1 += fast_exp2(fmaf(f[e + 1], kLog2e, nm2));
    }
  }
}

// Sweep-2 work on one vector: exp2(x*log2e + c) for every element, packed for the store.  With FOLD
// the gradient scale g is already inside c; otherwise it is multiplied in.
template <typename T, bool FOLD>
__device__ __forceinline__ uint4 grad_vec(const uint4& q, float c, float g) {
  constexpr int VE = VecInfo<T>::kElems;
  float f[VE];
  unpack<T>(q, f);
#pragma unroll
  for (int e = 0; e < VE; ++e) {
    f[e] = fast_exp2(fmaf(f[e], kLog2e, c));
    if (!FOLD) f[e] *= g;
  }
  return pack<T>(f);
}

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
    for (int k = 0; k < nchunk; ++k) issue_chunk(row, k);
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
      if (!ready) mbar_wait(full_s + 8 * k, parity, dead);
      uint4 q[VPC];
#pragma unroll
      for (int j = 0; j < VPC; ++j) q[j] = lds128(my_s + (uint32_t)(k * CV + j * NT) * 16u);
      ready = k + 1 < nchunk && mbar_test(full_s + 8 * (k + 1), parity);
      stats_chunk<T, VPC>(q, m, s0, s1);
    }
    if (nfull < nchunk) {
      if (!ready) mbar_wait(full_s + 8 * nfull, parity, dead);
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
        for (int p = 0; p < C; ++p) st_async_v4(slot, xb, (uint32_t)p, m, s, xl, 0.f);
      }
    } else {
      named_arrive(NT);
      MDY_TICK(2)
    }
    // two exchange slots suffice: a peer cannot send for row n+2 before it has this CTA's message for
    // row n+1, which leaves only after the reads of row n below
    mbar_wait(full_s + 8 * (kMaxChunks + (nloaded & 1u)), (nloaded >> 1) & 1u, dead);
    MDY_TICK(3)
    float gm = -INFINITY, gs = 0.f, xl = 0.f;
    {
      const float* x = xchg + (int)(nloaded & 1u) * kMaxCluster * 4;
      for (int p = 0; p < C; ++p) {
        merge_nb(gm, gs, x[p * 4], x[p * 4 + 1]);
        xl += x[p * 4 + 2];
      }
    }
    const float lse = gm + logf(gs);
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
  int C = (int)ceil_div(row_bytes, cluster_slice_limit());
  if (C > kMaxCluster) {
    // rows too long for 8 small slices: grow the slice up to what one CTA per SM can hold
    C = kMaxCluster;
    if (ceil_div(row_bytes, C) > 200 * 1024) return MDY_ERR_UNSUPPORTED;
  }
  const int64_t vpc = ceil_div(nvec, C);
  if ((int64_t)(C - 1) * vpc >= nvec) return MDY_ERR_UNSUPPORTED;  // a CTA would own nothing
  a.C = C;
  a.vpc = (int)vpc;
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
  return launch_cluster_nt<T, 512, 4, 1>(a, st);
}


// =================================================================================================
// Register-resident variant.
//
// Each thread keeps the exponentials of its NVEC vectors of the row in float registers between the
// two sweeps, so every logit costs ONE exp: sweep 1 stores e = exp2(x*log2e - ref*log2e) (ref = the
// thread's running max when the chunk was processed), sweep 2 multiplies by one per-chunk factor
// exp2((ref - lse)*log2e) * g, packs and stores.  Shared memory only holds a ring of bulk-copy
// buffers two rows deep (one "full" and one "empty" mbarrier per buffer): a buffer is released as
// soon as its 16 bytes per thread are in registers, and thread 0 refills it with the same chunk of
// the row two positions ahead, so loads run a whole row ahead of the math.
// =================================================================================================
template <typename T, int NT, int NVEC>
__global__ void __launch_bounds__(NT, (NT * NVEC <= 2048 ? 2 : 1)) ce_regrow_kernel(ClusterArgs a) {
  constexpr int VE = VecInfo<T>::kElems;
  constexpr int NW = NT / 32;
  constexpr int NSLOT = 2 * NVEC;
  constexpr uint32_t SLOT_BYTES = NT * 16;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)NSLOT * SLOT_BYTES);  // full[NSLOT], empty[NSLOT], xbar[2]
  float* xchg = reinterpret_cast<float*>(bars + 2 * NSLOT + 2);                         // [2][kMaxCluster][4]
  float* red = xchg + 2 * kMaxCluster * 4;                                               // [72]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t crank = cluster_ctarank();
  const int C = a.C;
  const int cid = blockIdx.x / C, ncl = gridDim.x / C;
  const int64_t nvec_total = a.V / VE;
  const int64_t v0 = (int64_t)crank * a.vpc;
  int my_nvec = (int)(nvec_total - v0 < a.vpc ? nvec_total - v0 : a.vpc);
  if (my_nvec < 0) my_nvec = 0;
  const int nj = (my_nvec + NT - 1) / NT;   // chunks of this CTA's slice, <= NVEC
  const uint32_t ring_s = smem_u32(smem_raw);
  const uint32_t full_s = smem_u32(bars);
  const uint32_t empty_s = full_s + 8 * NSLOT;
  const uint32_t xbar_s = empty_s + 8 * NSLOT;   // exchange barriers, one per parity of the row count
  const T* logits = reinterpret_cast<const T*>(a.logits);
  T* dlogits = reinterpret_cast<T*>(a.dlogits);
  const int slice_elem0 = (int)(v0 * VE);

  if (tid == 0) {
    for (int k = 0; k < NSLOT; ++k) {
      mbar_init(full_s + 8 * k, 1);
      mbar_init(empty_s + 8 * k, NW);
    }
    mbar_init(xbar_s, 1);
    mbar_init(xbar_s + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  cluster_sync_all();  // all CTAs of the cluster run before anyone writes a peer's shared memory
  const float g = a.ghost * (a.gdev ? *a.gdev : 1.f);

  // ---- producer state, used by thread 0 only ----
  int64_t prow = cid;  // next row of this cluster's sequence that has not been looked at for issue
  auto next_labelled_row = [&]() -> int64_t {
    while (prow < a.M && a.labels[prow] == MDY_IGNORE_INDEX) prow += ncl;
    const int64_t r = prow;
    if (prow < a.M) prow += ncl;
    return r;  // >= M: none left
  };
  // bulk copy of chunk j of `row` into ring position `pos` (position parity selects the buffer group)
  auto issue = [&](int64_t row, uint32_t pos, int j) {
    const int first = j * NT;
    int nv = my_nvec - first;
    if (nv <= 0) return;
    if (nv > NT) nv = NT;
    const uint32_t slot = (pos & 1u) * NVEC + (uint32_t)j;
    const char* src = reinterpret_cast<const char*>(logits + row * a.rs) + (v0 + first) * 16;
    mbar_expect_tx(full_s + 8 * slot, (uint32_t)nv * 16u);
    bulk_g2s(ring_s + slot * SLOT_BYTES, src, (uint32_t)nv * 16u, full_s + 8 * slot);
  };
  if (tid == 0) {
    for (uint32_t pos = 0; pos < 2; ++pos) {
      const int64_t r = next_labelled_row();
      if (r < a.M)
        for (int j = 0; j < nj; ++j) issue(r, pos, j);
    }
  }

  uint32_t n_cons = 0;  // labelled rows consumed so far == ring position of the current one
  bool dead = false;
#ifdef MDY_CE_TIMING
  long long tacc[6] = {0, 0, 0, 0, 0, 0};
  long long tlast = clock64();
#endif
  for (int64_t row = cid; row < a.M; row += ncl) {
    const int64_t label = a.labels[row];
    T* dst = dlogits + row * a.rs + (int64_t)slice_elem0 + (int64_t)tid * VE;
    MDY_TICK(0)
    if (label == MDY_IGNORE_INDEX) {
      if (crank == 0 && tid == 0) { a.losses[row] = 0.f; a.lse[row] = 0.f; }
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int v = tid; v < my_nvec; v += NT) st_stream(dst + (int64_t)(v - tid) * VE, z);
      continue;
    }
    // the row that will take this row's buffers (ring position n_cons + 2)
    int64_t r2 = a.M;
    if (tid == 0) r2 = next_labelled_row();
    const uint32_t slotbase = (n_cons & 1u) * NVEC;
    const uint32_t par = (n_cons >> 1) & 1u;
    int loc = -1;
    if (label >= 0 && label < a.V) {
      const int64_t l = label - slice_elem0;
      if (l >= 0 && l < (int64_t)my_nvec * VE) loc = (int)l;
    }
    const int loc_vec = loc >= 0 ? loc / VE : -1;

    // ---- sweep 1 ----
    float e[NVEC][VE];
    float ref[NVEC];
    float m = -INFINITY, s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int j = 0; j < NVEC; ++j) {
      if (j < nj) {
        const uint32_t slot = slotbase + (uint32_t)j;
        mbar_wait(full_s + 8 * slot, par, dead);
        const int v = j * NT + tid;
        const uint4 q = v < my_nvec ? lds128(ring_s + slot * SLOT_BYTES + (uint32_t)tid * 16u) : neg_inf_vec<T>();
        float f[VE];
        unpack<T>(q, f);
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_s + 8 * slot);   // this warp holds its part of the buffer in registers
        if (tid == 0 && r2 < a.M && j >= 1) {             // refill the buffer released one step ago
          mbar_wait(empty_s + 8 * (slot - 1), par, dead);
          issue(r2, n_cons + 2, j - 1);
        }
        const float vm = vec_max<T>(q);
        if (vm > m) {
          const float r = fast_exp2((fmaxf(m, -1e37f) - vm) * kLog2e);
          s0 *= r; s1 *= r;
          m = vm;
        }
        ref[j] = m;
        const float nm2 = -fmaxf(m, -1e37f) * kLog2e;
        if (v == loc_vec) {  // the label's logit, for the loss
          float xl = 0.f;
#pragma unroll
          for (int k = 0; k < VE; ++k)
            if (k == loc - loc_vec * VE) xl = f[k];
          red[70] = xl;
        }
#pragma unroll
        for (int k = 0; k < VE; k += 2) {
          e[j][k] = fast_exp2(fmaf(f[k], kLog2e, nm2));
          e[j][k + 1] = fast_exp2(fmaf(f[k + 1], kLog2e, nm2));
          s0 += e[j][k];
          s1 += e[j][k + 1];
        }
      }
    }
    MDY_TICK(1)
    if (tid == 0 && r2 < a.M) {
      mbar_wait(empty_s + 8 * (slotbase + (uint32_t)nj - 1), par, dead);
      issue(r2, n_cons + 2, nj - 1);
    }
    float s = s0 + s1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const float os = __shfl_xor_sync(0xffffffffu, s, o);
      merge_nb(m, s, om, os);
    }
    // m, s now hold the warp's pair; keep the thread's own history in ref[]
    if (lane == 0) { red[warp] = m; red[32 + warp] = s; }
    __syncthreads();
    MDY_TICK(2)
    if (warp == 0) {
      float wm = lane < NW ? red[lane] : -INFINITY;
      float ws = lane < NW ? red[32 + lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, wm, o);
        const float os = __shfl_xor_sync(0xffffffffu, ws, o);
        merge_nb(wm, ws, om, os);
      }
      if (lane == 0) {
        // send this CTA's (max, sum, label logit) to every CTA of the cluster, itself included; each
        // receiver's barrier completes when all C messages (16 bytes each) have landed
        const float xl = loc >= 0 ? red[70] : 0.f;
        const uint32_t xb = xbar_s + 8 * (n_cons & 1u);
        const uint32_t slotx = smem_u32(xchg + ((int)(n_cons & 1u) * kMaxCluster + (int)crank) * 4);
        mbar_expect_tx(xb, (uint32_t)C * 16u);
        for (int p = 0; p < C; ++p) st_async_v4(slotx, xb, (uint32_t)p, wm, ws, xl, 0.f);
      }
    }
    // Two exchange slots suffice: a peer needs this CTA's message for row n+1 before it can send
    // anything for row n+2, and that message is sent only after the reads of row n below.
    mbar_wait(xbar_s + 8 * (n_cons & 1u), par, dead);
    MDY_TICK(3)
    float gm = -INFINITY, gs = 0.f, xl = 0.f;
    {
      const float* x = xchg + (int)(n_cons & 1u) * kMaxCluster * 4;
      for (int p = 0; p < C; ++p) {
        merge_nb(gm, gs, x[p * 4], x[p * 4 + 1]);
        xl += x[p * 4 + 2];
      }
    }
    const float lse = gm + logf(gs);
    if (crank == 0 && tid == 0) {
      a.losses[row] = (label >= 0 && label < a.V) ? lse - xl : 0.f;
      a.lse[row] = lse;
    }

    // ---- sweep 2: from registers ----
#pragma unroll
    for (int j = 0; j < NVEC; ++j) {
      if (j < nj) {
        const int v = j * NT + tid;
        if (v < my_nvec) {
          const float fac = fast_exp2((ref[j] - lse) * kLog2e) * g;
          float o[VE];
#pragma unroll
          for (int k = 0; k < VE; ++k) o[k] = e[j][k] * fac;
          st_stream(dst + (int64_t)(j * NT) * VE, pack<T>(o));
        }
      }
    }
    if (loc >= 0 && (loc_vec % NT) == tid) {
      const float p = fast_exp2((xl - lse) * kLog2e);
      dlogits[row * a.rs + slice_elem0 + loc] = from_float<T>((p - 1.f) * g);
    }
    ++n_cons;
    MDY_TICK(4)
  }
#ifdef MDY_CE_TIMING
  if (blockIdx.x < 8 && (tid == 0 || tid == 40 || tid == NT - 1)) {
    float* o = a.lse + a.M + (blockIdx.x * 3 + (tid == 0 ? 0 : tid == 40 ? 1 : 2)) * 8;
    for (int i = 0; i < 5; ++i) o[i] = (float)tacc[i];
    o[5] = (float)n_cons;
  }
#endif
}

template <typename T, int NT, int NVEC>
int launch_regrow_nt(ClusterArgs a, cudaStream_t st) {
  constexpr int VE = VecInfo<T>::kElems;
  const int64_t nvec = a.V / VE;
  const int C = (int)ceil_div(nvec, (int64_t)NT * NVEC);
  if (C > kMaxCluster) return MDY_ERR_UNSUPPORTED;
  const int64_t vpc = ceil_div(nvec, C);
  if ((int64_t)(C - 1) * vpc >= nvec) return MDY_ERR_UNSUPPORTED;
  a.C = C;
  a.vpc = (int)vpc;
  a.slice_bytes_aligned = 0;
  const size_t smem = (size_t)2 * NVEC * NT * 16 + (size_t)(4 * NVEC + 2) * 8 + 2 * kMaxCluster * 4 * 4 + 72 * 4;
  auto kern = ce_regrow_kernel<T, NT, NVEC>;
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
  static thread_local int c_dev = -1, c_C = 0, c_max = 0;
  int dev = 0;
  (void)cudaGetDevice(&dev);
  int max_clusters = 0;
  if (dev == c_dev && C == c_C) {
    max_clusters = c_max;
  } else {
    e = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);
    if (e != cudaSuccess || max_clusters < 1) { (void)cudaGetLastError(); return MDY_ERR_UNSUPPORTED; }
    c_dev = dev; c_C = C; c_max = max_clusters;
  }
  int64_t ncl = a.M < max_clusters ? a.M : max_clusters;
  cfg.gridDim = dim3((unsigned)(ncl * C), 1, 1);
  e = cudaLaunchKernelEx(&cfg, kern, a);
  if (e != cudaSuccess) return (int)e;
  return finish_launch(1);
}

template <typename T>
int launch_regrow(const ClusterArgs& a, cudaStream_t st) {
  constexpr int VE = VecInfo<T>::kElems;
  if (a.V % VE != 0 || a.rs % VE != 0 || !aligned16(a.logits) || !aligned16(a.dlogits)) return MDY_ERR_UNSUPPORTED;
  if (a.V >= ((int64_t)1 << 27)) return MDY_ERR_UNSUPPORTED;
  switch (tunable(MDY_TUNE_CE_REG_SHAPE)) {
    case 1: return launch_regrow_nt<T, 256, 8>(a, st);
    case 2: return launch_regrow_nt<T, 512, 4>(a, st);
    case 4: return launch_regrow_nt<T, 1024, 4>(a, st);
    default: return launch_regrow_nt<T, 512, 8>(a, st);
  }
}


// =================================================================================================
// Exp-cache variant (the default where the row fits): one exp per logit with 16-32 warps per SM.
//
// Sweep 1 computes e = exp2(x*log2e - ref*log2e) (ref = the thread's running max when it processed
// the chunk) and parks it as float32 in a per-CTA shared-memory buffer; sweep 2 reads it back,
// multiplies by one factor per (thread, chunk), exp2((ref - lse)*log2e) * g, packs and stores.  The
// bf16 logits only pass through a ring of NVEC bulk-copy buffers (one row deep): a buffer is released
// the moment its 16 bytes per thread are in registers and is refilled with the same chunk of the
// cluster's next row, so the next row streams in while the current one is still being processed.
// A thread reads in sweep 2 exactly the shared-memory words it wrote in sweep 1, so the float32
// buffer needs no barrier at all.  The buffer is split into 16-byte planes so that both the stores
// and the loads of a warp are conflict-free.
//   NT = 512 : up to 2048 vectors per CTA, 96 KB of shared memory -> two CTAs per SM (a CTA's
//              reduction and exchange overlap the other's sweeps); rows up to 8 * 2048 vectors.
//   NT = 1024: up to 4096 vectors per CTA, 192 KB -> one CTA per SM; rows up to 8 * 4096 vectors.
// =================================================================================================
template <typename T, int NT>
__global__ void __launch_bounds__(NT, (NT <= 512 ? 2 : 1)) ce_expcache_kernel(ClusterArgs a) {
  constexpr int VE = VecInfo<T>::kElems;
  constexpr int NW = NT / 32;
  constexpr int NVEC = 4;
  constexpr int EPV = VE / 4;                       // 16-byte planes of float32 per vector
  constexpr uint32_t SLOT_BYTES = NT * 16;
  constexpr uint32_t PLANE_BYTES = NVEC * NT * 16;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)NVEC * SLOT_BYTES + (size_t)EPV * PLANE_BYTES);
  float* xchg = reinterpret_cast<float*>(bars + 2 * NVEC + 2);   // full[NVEC], empty[NVEC], xbar[2] | [2][kMaxCluster][4]
  float* red = xchg + 2 * kMaxCluster * 4;                       // [72]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t crank = cluster_ctarank();
  const int C = a.C;
  const int cid = blockIdx.x / C, ncl = gridDim.x / C;
  const int64_t nvec_total = a.V / VE;
  const int64_t v0 = (int64_t)crank * a.vpc;
  int my_nvec = (int)(nvec_total - v0 < a.vpc ? nvec_total - v0 : a.vpc);
  if (my_nvec < 0) my_nvec = 0;
  const int nj = (my_nvec + NT - 1) / NT;   // chunks of this CTA's slice, <= NVEC
  const uint32_t ring_s = smem_u32(smem_raw);
  const uint32_t ebuf_s = ring_s + NVEC * SLOT_BYTES + (uint32_t)tid * 16u;   // this thread's column of the planes
  const uint32_t full_s = smem_u32(bars);
  const uint32_t empty_s = full_s + 8 * NVEC;
  const uint32_t xbar_s = empty_s + 8 * NVEC;
  const T* logits = reinterpret_cast<const T*>(a.logits);
  T* dlogits = reinterpret_cast<T*>(a.dlogits);
  const int slice_elem0 = (int)(v0 * VE);

  if (tid == 0) {
    for (int k = 0; k < NVEC; ++k) {
      mbar_init(full_s + 8 * k, 1);
      mbar_init(empty_s + 8 * k, NW);
    }
    mbar_init(xbar_s, 1);
    mbar_init(xbar_s + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  cluster_sync_all();  // all CTAs of the cluster run before anyone writes a peer's shared memory
  const float g = a.ghost * (a.gdev ? *a.gdev : 1.f);

  // ---- producer state, used by thread 0 only ----
  int64_t prow = cid;
  auto next_labelled_row = [&]() -> int64_t {
    while (prow < a.M && a.labels[prow] == MDY_IGNORE_INDEX) prow += ncl;
    const int64_t r = prow;
    if (prow < a.M) prow += ncl;
    return r;  // >= M: none left
  };
  auto issue = [&](int64_t row, int j) {
    const int first = j * NT;
    int nv = my_nvec - first;
    if (nv <= 0) return;
    if (nv > NT) nv = NT;
    const char* src = reinterpret_cast<const char*>(logits + row * a.rs) + (v0 + first) * 16;
    mbar_expect_tx(full_s + 8 * j, (uint32_t)nv * 16u);
    bulk_g2s(ring_s + (uint32_t)j * SLOT_BYTES, src, (uint32_t)nv * 16u, full_s + 8 * j);
  };
  int64_t r_next = a.M;  // thread 0: the labelled row after the one currently in the ring
  if (tid == 0) {
    const int64_t r = next_labelled_row();
    if (r < a.M)
      for (int j = 0; j < nj; ++j) issue(r, j);
    r_next = next_labelled_row();
  }

  uint32_t n_cons = 0;  // labelled rows consumed so far
  bool dead = false;
  int64_t label = cid < a.M ? a.labels[cid] : MDY_IGNORE_INDEX;
#ifdef MDY_CE_TIMING
  long long tacc[6] = {0, 0, 0, 0, 0, 0};
  long long tlast = clock64();
#endif
  for (int64_t row = cid; row < a.M; row += ncl) {
    // the next row's label is fetched a whole row ahead of its use
    const int64_t label_next = row + ncl < a.M ? a.labels[row + ncl] : MDY_IGNORE_INDEX;
    T* dst = dlogits + row * a.rs + (int64_t)slice_elem0 + (int64_t)tid * VE;
    if (label == MDY_IGNORE_INDEX) {
      if (crank == 0 && tid == 0) { a.losses[row] = 0.f; a.lse[row] = 0.f; }
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int v = tid; v < my_nvec; v += NT) st_stream(dst + (int64_t)(v - tid) * VE, z);
      label = label_next;
      continue;
    }
    MDY_TICK(0)
    const uint32_t par = n_cons & 1u;
    int loc = -1;
    if (label >= 0 && label < a.V) {
      const int64_t l = label - slice_elem0;
      if (l >= 0 && l < (int64_t)my_nvec * VE) loc = (int)l;
    }
    const int loc_vec = loc >= 0 ? loc / VE : -1;

    // ---- sweep 1 ----
    float ref[NVEC];
    float m = -INFINITY, s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int j = 0; j < NVEC; ++j) {
      if (j < nj) {
        mbar_wait(full_s + 8 * j, par, dead);
        const int v = j * NT + tid;
        const uint4 q = v < my_nvec ? lds128(ring_s + (uint32_t)j * SLOT_BYTES + (uint32_t)tid * 16u) : neg_inf_vec<T>();
        float f[VE];
        unpack<T>(q, f);
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_s + 8 * j);       // this warp's part of the buffer is in registers
        if (tid == 0 && r_next < a.M && j >= 1) {          // refill the buffer released one step ago
          mbar_wait(empty_s + 8 * (j - 1), par, dead);
          issue(r_next, j - 1);
        }
        const float vm = vec_max<T>(q);
        if (vm > m) {
          const float r = fast_exp2((fmaxf(m, -1e37f) - vm) * kLog2e);
          s0 *= r; s1 *= r;
          m = vm;
        }
        ref[j] = m;
        const float nm2 = -fmaxf(m, -1e37f) * kLog2e;
        if (v == loc_vec) {  // the label's logit, for the loss
          float xl = 0.f;
#pragma unroll
          for (int k = 0; k < VE; ++k)
            if (k == loc - loc_vec * VE) xl = f[k];
          red[70] = xl;
        }
#pragma unroll
        for (int k = 0; k < VE; ++k) f[k] = fast_exp2(fmaf(f[k], kLog2e, nm2));
#pragma unroll
        for (int k = 0; k < VE; k += 2) { s0 += f[k]; s1 += f[k + 1]; }
#pragma unroll
        for (int pl = 0; pl < EPV; ++pl) {
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(ebuf_s + (uint32_t)pl * PLANE_BYTES + (uint32_t)j * SLOT_BYTES),
                       "f"(f[4 * pl]), "f"(f[4 * pl + 1]), "f"(f[4 * pl + 2]), "f"(f[4 * pl + 3])
                       : "memory");
        }
      }
    }
    MDY_TICK(1)
    if (tid == 0) {
      if (r_next < a.M) {
        mbar_wait(empty_s + 8 * (nj - 1), par, dead);
        issue(r_next, nj - 1);
      }
      r_next = next_labelled_row();
    }
    float s = s0 + s1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const float os = __shfl_xor_sync(0xffffffffu, s, o);
      merge_nb(m, s, om, os);
    }
    if (lane == 0) { red[warp] = m; red[32 + warp] = s; }
    __syncthreads();
    MDY_TICK(2)
    if (warp == 0) {
      float wm = lane < NW ? red[lane] : -INFINITY;
      float ws = lane < NW ? red[32 + lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, wm, o);
        const float os = __shfl_xor_sync(0xffffffffu, ws, o);
        merge_nb(wm, ws, om, os);
      }
      if (lane == 0) {
        // this CTA's (max, sum, label logit) to every CTA of the cluster, itself included
        const float xl = loc >= 0 ? red[70] : 0.f;
        const uint32_t xb = xbar_s + 8 * (n_cons & 1u);
        const uint32_t slotx = smem_u32(xchg + ((int)(n_cons & 1u) * kMaxCluster + (int)crank) * 4);
        mbar_expect_tx(xb, (uint32_t)C * 16u);
        for (int p = 0; p < C; ++p) st_async_v4(slotx, xb, (uint32_t)p, wm, ws, xl, 0.f);
      }
    }
    // two exchange slots suffice: a peer cannot send for row n+2 before it has this CTA's message for
    // row n+1, which leaves only after the reads of row n below
    mbar_wait(xbar_s + 8 * (n_cons & 1u), (n_cons >> 1) & 1u, dead);
    MDY_TICK(3)
    float gm = -INFINITY, gs = 0.f, xl = 0.f;
    {
      const float* x = xchg + (int)(n_cons & 1u) * kMaxCluster * 4;
      for (int p = 0; p < C; ++p) {
        merge_nb(gm, gs, x[p * 4], x[p * 4 + 1]);
        xl += x[p * 4 + 2];
      }
    }
    const float lse = gm + logf(gs);
    if (crank == 0 && tid == 0) {
      a.losses[row] = (label >= 0 && label < a.V) ? lse - xl : 0.f;
      a.lse[row] = lse;
    }

    // ---- sweep 2: from the float32 buffer this thread filled ----
#pragma unroll
    for (int j = 0; j < NVEC; ++j) {
      if (j < nj) {
        const int v = j * NT + tid;
        if (v < my_nvec) {
          const float fac = fast_exp2((ref[j] - lse) * kLog2e) * g;
          float o[VE];
#pragma unroll
          for (int pl = 0; pl < EPV; ++pl) {
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(o[4 * pl]), "=f"(o[4 * pl + 1]), "=f"(o[4 * pl + 2]), "=f"(o[4 * pl + 3])
                         : "r"(ebuf_s + (uint32_t)pl * PLANE_BYTES + (uint32_t)j * SLOT_BYTES)
                         : "memory");
          }
#pragma unroll
          for (int k = 0; k < VE; ++k) o[k] *= fac;
          st_stream(dst + (int64_t)(j * NT) * VE, pack<T>(o));
        }
      }
    }
    if (loc >= 0 && (loc_vec % NT) == tid) {
      const float p = fast_exp2((xl - lse) * kLog2e);
      dlogits[row * a.rs + slice_elem0 + loc] = from_float<T>((p - 1.f) * g);
    }
    ++n_cons;
    label = label_next;
    MDY_TICK(4)
  }
#ifdef MDY_CE_TIMING
  if (blockIdx.x < 8 && (tid == 0 || tid == 40 || tid == NT - 1)) {
    float* o = a.lse + a.M + (blockIdx.x * 3 + (tid == 0 ? 0 : tid == 40 ? 1 : 2)) * 8;
    for (int i = 0; i < 5; ++i) o[i] = (float)tacc[i];
    o[5] = (float)n_cons;
  }
#endif
}

template <typename T, int NT>
int launch_expcache_nt(ClusterArgs a, cudaStream_t st) {
  constexpr int VE = VecInfo<T>::kElems;
  constexpr int NVEC = 4, EPV = VE / 4;
  const int64_t nvec = a.V / VE;
  const int C = (int)ceil_div(nvec, (int64_t)NT * NVEC);
  if (C > kMaxCluster) return MDY_ERR_UNSUPPORTED;
  const int64_t vpc = ceil_div(nvec, C);
  if ((int64_t)(C - 1) * vpc >= nvec) return MDY_ERR_UNSUPPORTED;
  a.C = C;
  a.vpc = (int)vpc;
  a.slice_bytes_aligned = 0;
  const size_t smem = (size_t)NVEC * NT * 16 * (1 + EPV) + (size_t)(2 * NVEC + 2) * 8 + 2 * kMaxCluster * 4 * 4 + 72 * 4;
  auto kern = ce_expcache_kernel<T, NT>;
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
  static thread_local int c_dev = -1, c_C = 0, c_max = 0;
  int dev = 0;
  (void)cudaGetDevice(&dev);
  int max_clusters = 0;
  if (dev == c_dev && C == c_C) {
    max_clusters = c_max;
  } else {
    e = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);
    if (e != cudaSuccess || max_clusters < 1) { (void)cudaGetLastError(); return MDY_ERR_UNSUPPORTED; }
    c_dev = dev; c_C = C; c_max = max_clusters;
  }
  int64_t ncl = a.M < max_clusters ? a.M : max_clusters;
  cfg.gridDim = dim3((unsigned)(ncl * C), 1, 1);
  e = cudaLaunchKernelEx(&cfg, kern, a);
  if (e != cudaSuccess) return (int)e;
  return finish_launch(1);
}

// shape: 0 = smallest CTA that fits the row in <= 8 CTAs, 1 = 512 threads, 2 = 1024 threads
template <typename T>
int launch_expcache(const ClusterArgs& a, cudaStream_t st, int shape) {
  constexpr int VE = VecInfo<T>::kElems;
  if (a.V % VE != 0 || a.rs % VE != 0 || !aligned16(a.logits) || !aligned16(a.dlogits)) return MDY_ERR_UNSUPPORTED;
  if (a.V >= ((int64_t)1 << 27)) return MDY_ERR_UNSUPPORTED;
  if (shape != 2) {
    const int rc = launch_expcache_nt<T, 512>(a, st);
    if (rc != MDY_ERR_UNSUPPORTED || shape == 1) return rc;
  }
  return launch_expcache_nt<T, 1024>(a, st);
}

}  // namespace

int ce_fused_cluster(const void* logits, void* dlogits, const int64_t* labels, float* losses, float* lse,
                     const float* gdev, float ghost, int64_t M, int64_t V, int64_t rs, int dtype,
                     cudaStream_t st) {
  ClusterArgs a;
  a.logits = logits; a.dlogits = dlogits; a.labels = labels; a.losses = losses; a.lse = lse;
  a.gdev = gdev; a.ghost = ghost; a.M = (int)M; a.V = V; a.rs = rs;
  a.C = 0; a.vpc = 0; a.slice_bytes_aligned = 0;
  const int impl = tunable(MDY_TUNE_CE_FUSED_IMPL);
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    // Default: the kernel that stages the whole slice in shared memory and recomputes the exp — big
    // CTAs (one per SM, 64 K logits per CTA and row) amortise the per-row reduction and exchange best.
    // The one-exp variants (3: exponentials in registers, 4: cached in shared memory) split a row over
    // more, smaller CTAs; on-device timing showed their per-row exchange latency dominating, so they
    // are kept selectable for experiments only.
    if (impl == 3) return launch_regrow<T>(a, st);
    if (impl == 4) return launch_expcache<T>(a, st, tunable(MDY_TUNE_CE_REG_SHAPE));
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

extern "C" int mdy_last_device_error(int clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, mdy::g_dev_error, sizeof(int)) != cudaSuccess) {
    (void)cudaGetLastError();
    return -1;
  }
  if (clear && v != 0) {
    const int z = 0;
    (void)cudaMemcpyToSymbol(mdy::g_dev_error, &z, sizeof(int));
  }
  return v;
}
