// Device helpers shared by the shared-memory-staged cross-entropy kernels: mbarrier and bulk-copy
// wrappers with bounded waits, distributed-shared-memory stores, and the per-vector arithmetic of the two
// sweeps (online max / sum-exp, gradient).
#pragma once
#include <math.h>
#include "common.cuh"

namespace mdy {

namespace {

// Set to a non-zero code by a kernel of the including source file whose bounded wait expired.  Each
// source file that includes this header gets its own flag (device symbols are not shared between
// separately compiled files); mdy_last_device_error reads them all through read_dev_error.
__device__ int g_dev_error = 0;

// Synchronises with the device; returns the including file's flag (-1 if it cannot be read) and clears it
// when asked to.
inline int read_dev_error(bool clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_dev_error, sizeof(int)) != cudaSuccess) {
    (void)cudaGetLastError();
    return -1;
  }
  if (clear && v != 0) {
    const int z = 0;
    (void)cudaMemcpyToSymbol(g_dev_error, &z, sizeof(int));
  }
  return v;
}

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
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, bool& dead, int tries) {
  if (dead) return;
  // each try_wait may suspend for up to ~1 us; the default 2^20 tries bound the wait to about a second
  for (int i = 0; i < tries; ++i) {
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

}  // namespace
}  // namespace mdy
