// Vocab-parallel cross-entropy as ONE kernel per GPU: local statistics, the exchange between the ranks
// and the gradient sweep fused, with the exchange done by plain stores into the peers' memory.
//
// Every rank holds logits[:, r*Vs:(r+1)*Vs] and all labels.  The two-kernel path (statistics sweep ->
// NCCL all-gather -> gradient sweep) reads the shard twice and exposes the collective's latency.  Here a
// CTA keeps the row slices it works on in a ring of shared-memory slots (filled by the bulk-copy engine),
// so HBM sees one read and one write per logit, and the exchange overlaps the rows in between:
//
//   A(row):  wait for the slice, fold it into (max, sum-exp), publish (local lse, -logit[label] if the
//            label lies in this slice) as ONE 16-byte record {lse, epoch, negx, epoch} into the exchange
//            buffer of EVERY rank (its own included) — a store over NVLink into peer memory;
//   B(row):  `lag` rows later, poll this rank's own exchange buffer until the records of all
//            participants of the row carry the current epoch, combine them into the global lse and the
//            loss, then write (softmax - onehot) * g from the slice still in shared memory and refill
//            the slot with a later row.
//
// A shard row longer than a slot is cut into `nsub` column slices handled by different CTAs; they are
// participants of the exchange like the peers' CTAs (through this GPU's own buffer), so a row has
// P = ranks * nsub participants.  Each 8-byte half of a record carries its own epoch tag, so the record
// needs no fence and no atomicity beyond that of an aligned 64-bit vector element.  Buffers are double-buffered by
// epoch parity: a rank can be at most one call ahead of a peer that still reads the previous call.
//
// Inside a CTA the work is split between compute warps, which only stream (statistics sweep of row i,
// gradient sweep of row i - lag), and ONE exchange warp, which does everything that is latency: the end of
// the CTA's reduction, the publish, the poll, the combine.  They hand rows to each other through mbarriers.
//
// Every wait is bounded.  The poll of the exchange gives up after `wait_tries` rounds (a few seconds by
// default), the mbarrier waits likewise: the thread then raises the device flag (mdy_last_device_error),
// publishes and reports NaN from then on and keeps walking its rows, so the peers never wait for it and the
// loss of the batch is NaN, not a finite wrong number.
//
// All CTAs of a launch have to be resident at once (they wait for one another): the grid is sized from the
// occupancy query and launched cooperatively, so the runtime refuses it rather than run a part of it, on
// every participating GPU; with fewer GPUs than ranks the same kernel runs all ranks as "virtual ranks" of
// one launch (nvr > 1), which is how the protocol is tested on a single GPU.
// No multicast copy and no remote LOAD is used: peers' memory is only ever written.
#include <math.h>
#include <string.h>
#include <mutex>
#include "common.cuh"
#include "ce_common.cuh"

namespace mdy {
namespace {

constexpr int kVpMaxRanks = 8;
constexpr int kVpMaxParts = 32;   // participants of a row: one warp polls them, one lane each
constexpr int kVpMaxSlots = 8;
constexpr int kVpMaxChunks = 4;
constexpr int kLabRing = 64;      // labels kept in shared memory per CTA (a ring over its rows)
constexpr int kLabAhead = 40;     // how many rows ahead of the statistics sweep a label is fetched

struct VpArgs {
  const void* logits[kVpMaxRanks];  // shard of virtual rank v of this launch
  void* dlogits[kVpMaxRanks];
  float* losses[kVpMaxRanks];
  float* lse[kVpMaxRanks];
  uint4* xbuf[kVpMaxRanks];         // exchange buffer of RANK r as addressable from this GPU (all tp ranks)
  const int64_t* labels;
  const float* gdev; float ghost;
  int M; int64_t vs; int64_t rs;    // rows, columns of a shard, row stride in elements
  int tp, nvr, rank0;               // ranks; virtual ranks in this launch; rank of virtual rank 0
  int nsub, G;                      // column slices per shard row; CTAs per virtual rank (a multiple of nsub)
  int vps;                          // 16-byte vectors per slice
  int slot_bytes, nslots, lag;
  int xrows;                        // rows an exchange buffer holds per parity
  uint32_t epoch;
  int wait_tries;
  int mute_part;                    // test hook: participant `mute_part - 1` never publishes row 0 (0 = off)
};

// Where the first bounded wait of a launch expired: {kind (1 slot data, 3 lse hand-off, 4 statistics hand-off, 2 a
// peer's record), CTA, row index of the CTA, thread}.  Diagnosis only (mdy_device_error_of, sources 16-19).
__device__ int g_vp_detail[4] = {0, 0, 0, 0};

__device__ __forceinline__ void note_expiry(int kind, int i) {
  if (atomicCAS(&g_vp_detail[0], 0, kind) == 0) {
    g_vp_detail[1] = (int)blockIdx.x; g_vp_detail[2] = i; g_vp_detail[3] = (int)threadIdx.x;
  }
}
__device__ __forceinline__ void vp_wait(int kind, int i, uint32_t bar, uint32_t parity, bool& dead, int tries) {
  const bool was = dead;
  mbar_wait(bar, parity, dead, tries);
  if (!was && dead) note_expiry(kind, i);
}

// A record is two 64-bit words {value, tag}: written and read as vectors of 64-bit ELEMENTS, the unit the memory
// model keeps whole in a vector access, so a word is never seen with a new tag and an old value.
__device__ __forceinline__ void st_volatile_v4(uint4* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  const unsigned long long lo = ((unsigned long long)b << 32) | a, hi = ((unsigned long long)d << 32) | c;
  asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(lo), "l"(hi) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
  unsigned long long lo, hi;
  asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(lo), "=l"(hi) : "l"(p) : "memory");
  return make_uint4((uint32_t)lo, (uint32_t)(lo >> 32), (uint32_t)hi, (uint32_t)(hi >> 32));
}

__device__ __forceinline__ void bar_sync_id(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
// Hand-offs inside a CTA.  Between the compute warps and the exchange warp they are mbarriers, waited for
// with the same bounded try_wait as the bulk copies, so that a slip in the protocol would show up as an
// expired wait (flag, NaN loss), never as a hang:
//   stats[i & 7]  one arrival per compute warp: row i's per-warp statistics are in shared memory
//   lse[jb & 3]   one arrival by the exchange warp: the global lse of gradient row jb is in shared memory
// The compute warps can be at most lag + 1 <= 4 rows ahead of the exchange warp's statistics waits and the
// exchange warp at most two rows ahead of their lse waits, so rings of 4 and 2 barriers would do; they are
// twice that, so that a barrier is never re-armed while anyone could still be waiting for its previous phase.
// Among the compute warps only, hardware barrier kBarSlot: the slice has left shared memory, refill its slot.
constexpr int kBarSlot = 1;
constexpr int kStatsRing = 8, kLseRing = 4;
constexpr int kVpBarriers = 24;   // 8-byte mbarrier slots reserved: kVpMaxSlots for the ring, the two rings above

// A CTA is NTC compute threads plus ONE exchange warp (warp 0).  The compute warps stream: statistics
// sweep of row i, gradient sweep of row i - lag, both from shared memory, never waiting for the exchange
// unless it is late.  The exchange warp does everything that is latency and not bandwidth: it finishes
// the CTA's reduction, publishes the record to every rank, polls this rank's buffer for the records of the
// row whose gradient comes next, combines them, and keeps the label ring filled.  The two sides meet at
// named barriers only.
// CTAs per SM each shape is compiled for (its register budget): one 544-thread CTA may use 120 registers a
// thread; without the hint the compiler aimed for two and spilled.
constexpr int vp_min_blocks(int ntc) { return ntc >= 512 ? 1 : ntc >= 256 ? 2 : ntc >= 128 ? 4 : 8; }

// PV: the last, partial chunk of the statistics sweep is swept one vector at a time, so that a thread does only
// the vectors it really has.  It costs registers (1-2 % on shapes whose last chunk is nearly full) and wins 5 %
// where a whole vector per thread would be empty (seven vectors per thread in two chunks of four), so it is a
// compile-time variant the launcher picks by the slice length.
template <typename T, int NTC, int VPC, bool PV, int MINB = vp_min_blocks(NTC)>
__global__ void __launch_bounds__(NTC + 32, MINB) ce_vp_fused_kernel(VpArgs a) {
  constexpr int VE = VecInfo<T>::kElems;
  constexpr int CV = NTC * VPC;  // vectors per chunk
  constexpr int NWC = NTC / 32;  // compute warps
  constexpr int NTA = NTC + 32;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + (size_t)a.nslots * a.slot_bytes);
  float* red = reinterpret_cast<float*>(full + kVpBarriers);  // [kStatsRing][64]: per-warp (max, sum) of a row
  float* bcast = red + kStatsRing * 64;                        // [kLseRing][4]: global lse of a gradient row
  // labels of this CTA's rows, fetched kLabAhead rows ahead by the exchange warp into a ring: a label is
  // never waited for by a compute warp
  long long* lab_s = reinterpret_cast<long long*>(bcast + kLseRing * 4);  // [kLabRing]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vr = blockIdx.x / a.G, c = blockIdx.x % a.G;
  const int sl = c % a.nsub, rl = c / a.nsub, lanes = a.G / a.nsub;
  const int rank = a.rank0 + vr;
  const int P = a.tp * a.nsub, part = rank * a.nsub + sl;
  const int64_t nvec_total = a.vs / VE;
  const int64_t v0 = (int64_t)sl * a.vps;
  int my_nvec = (int)(nvec_total - v0 < a.vps ? nvec_total - v0 : a.vps);
  if (my_nvec < 0) my_nvec = 0;
  const int nchunk = (my_nvec + CV - 1) / CV, nfull = my_nvec / CV;
  const int slice_elem0 = (int)(v0 * VE);
  const int64_t col0 = (int64_t)rank * a.vs + slice_elem0;  // vocabulary id of the slice's first column
  const T* logits = reinterpret_cast<const T*>(a.logits[vr]);
  T* dlogits = reinterpret_cast<T*>(a.dlogits[vr]);
  const uint32_t slots_s = smem_u32(smem_raw), full_s = smem_u32(full);
  const uint32_t stats_s = full_s + 8 * kVpMaxSlots, lse_s = stats_s + 8 * kStatsRing;
  const uint32_t parity_x = a.epoch & 1u;
  const int R = rl < a.M ? (a.M - rl + lanes - 1) / lanes : 0;  // rows of this CTA: rl, rl + lanes, ...
  const int nslots = a.nslots, lag = a.lag;

  if (tid == 32) {
    for (int k = 0; k < nslots; ++k) mbar_init(full_s + 8 * k, 1);
    for (int k = 0; k < kStatsRing; ++k) mbar_init(stats_s + 8 * k, NWC);
    for (int k = 0; k < kLseRing; ++k) mbar_init(lse_s + 8 * k, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < kLabAhead && tid < R) lab_s[tid] = a.labels[(int64_t)rl + (int64_t)tid * lanes];
  __syncthreads();

  // bulk copy of a row's slice into a slot (one compute thread); ignored rows are never loaded
  auto issue_load = [&](int slot, int64_t row, int64_t label) {
    if (label == MDY_IGNORE_INDEX || my_nvec == 0) return;
    const uint32_t bar = full_s + 8 * slot;
    const char* src = reinterpret_cast<const char*>(logits + row * a.rs) + v0 * 16;
    mbar_expect_tx(bar, (uint32_t)my_nvec * 16u);
    for (int k = 0; k < nchunk; ++k) {
      int nv = my_nvec - k * CV;
      if (nv > CV) nv = CV;
      bulk_g2s(slots_s + (uint32_t)slot * a.slot_bytes + (uint32_t)k * CV * 16u, src + (size_t)k * CV * 16, (uint32_t)nv * 16u, bar);
    }
  };

  if (warp == 0) {
    // =============================================================== exchange warp
    bool dead = false;
    long long lab_new = MDY_IGNORE_INDEX;
    int lab_new_j = -1;
    int slot_a = 0;
    int64_t row_a = rl, row_b = rl;
    for (int i = 0; i < R + lag; ++i) {
      if (lane == 0) {
        if (lab_new_j >= 0) lab_s[lab_new_j & (kLabRing - 1)] = lab_new;
        const int jf = i + kLabAhead;
        if (jf < R) { lab_new = a.labels[(int64_t)rl + (int64_t)jf * lanes]; lab_new_j = jf; } else { lab_new_j = -1; }
      }
      // ---- gradient row jb = i - lag: its records were published lag rows ago; combine them now, while the
      // ---- compute warps are in their statistics sweep, so that they find the lse ready
      const int jb = i - lag;
      if (jb >= 0) {
        if (lab_s[jb & (kLabRing - 1)] != MDY_IGNORE_INDEX) {
          const uint4* rec_src = a.xbuf[rank] + ((size_t)parity_x * a.xrows + row_b) * P + lane;
          uint4 v = make_uint4(0, 0, 0, 0);
          bool ok = lane >= P;
          if (!dead) {
            int tries = 0;
            for (;;) {
              if (!ok) {
                v = ld_volatile_v4(rec_src);
                ok = v.y == a.epoch && v.w == a.epoch;
              }
              if (__all_sync(0xffffffffu, ok)) break;
              if (++tries >= a.wait_tries) {
                dead = true;
                atomicExch(&g_dev_error, 2);
                note_expiry(2, jb);
                break;
              }
              if (tries > 64) __nanosleep(200);
            }
          }
          const float pl = (lane < P && ok) ? __uint_as_float(v.x) : -INFINITY;
          const float nx = (lane < P && ok) ? __uint_as_float(v.z) : 0.f;
          const float gm = warp_max(pl);
          float e = (pl == -INFINITY) ? 0.f : fast_exp2((pl - gm) * kLog2e);
          e = warp_sum(e);
          float lse_g = gm + logf(e);
          const float xs = warp_sum(nx);
          if (dead) lse_g = NAN;
          if (lane == 0) {
            bcast[(jb & (kLseRing - 1)) * 4] = lse_g;
            if (sl == 0) { a.losses[vr][row_b] = lse_g + xs; a.lse[vr][row_b] = lse_g; }
          }
        } else if (lane == 0 && sl == 0) {
          a.losses[vr][row_b] = 0.f; a.lse[vr][row_b] = 0.f;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(lse_s + 8 * (jb & (kLseRing - 1)));
        row_b += lanes;
      }
      // ---- statistics row i: finish the CTA's reduction and publish the record to every rank
      if (i < R) {
        const int64_t label = lab_s[i & (kLabRing - 1)];
        vp_wait(4, i, stats_s + 8 * (i & (kStatsRing - 1)), (uint32_t)(i >> 3) & 1u, dead, a.wait_tries);
        if (label != MDY_IGNORE_INDEX) {
          const float* rd = red + (i & (kStatsRing - 1)) * 64;
          float m = lane < NWC ? rd[lane] : -INFINITY;
          float s = lane < NWC ? rd[32 + lane] : 0.f;
          group_merge<32>(m, s);   // every lane ends up with the slice's (max, sum): lane r publishes to rank r
          float part_lse = m + logf(s);  // -inf for an empty or all -inf slice
          float negx = 0.f;
          const int64_t l = label - col0;
          if (l >= 0 && l < (int64_t)my_nvec * VE)
            negx = -to_float(reinterpret_cast<const T*>(smem_raw + (size_t)slot_a * a.slot_bytes)[l]);
          if (dead) part_lse = NAN;
          const bool muted = a.mute_part > 0 && part == a.mute_part - 1 && row_a == 0;
          if (lane < a.tp && !muted) {
            uint4* dst = a.xbuf[lane] + ((size_t)parity_x * a.xrows + row_a) * P + part;
            st_volatile_v4(dst, __float_as_uint(part_lse), a.epoch, __float_as_uint(negx), a.epoch);
          }
        }
        slot_a = slot_a + 1 == nslots ? 0 : slot_a + 1;
        row_a += lanes;
      }
    }
    return;
  }

  // ================================================================= compute warps
  const int ct = tid - 32, cw = warp - 1;
  const float g = a.ghost * (a.gdev ? *a.gdev : 1.f);
  const bool fold = g > 0.f && g < INFINITY;
  const float log2g = fold ? log2f(g) : 0.f;
  if (ct == 0) {
    for (int j = 0; j < nslots && j < R; ++j) issue_load(j, (int64_t)rl + (int64_t)j * lanes, lab_s[j]);
  }
  uint32_t phase_bits = 0;  // bit k: parity of the next wait on slot k's barrier
  bool dead = false;
  const uint32_t my_off = (uint32_t)ct * 16u;
  int slot_a = 0, slot_b = 0;
  int64_t row_b = rl;
  for (int i = 0; i < R + lag; ++i) {
    // ---------------------------------------------------------------- A(i): statistics of row i
    if (i < R) {
      const int64_t label = lab_s[i & (kLabRing - 1)];
      if (label != MDY_IGNORE_INDEX) {
        const uint32_t base = slots_s + (uint32_t)slot_a * a.slot_bytes + my_off;
        float m = -INFINITY, s0 = 0.f, s1 = 0.f;
        if (my_nvec > 0) {
          vp_wait(1, i, full_s + 8 * slot_a, (phase_bits >> slot_a) & 1u, dead, a.wait_tries);
          phase_bits ^= 1u << slot_a;
          for (int k = 0; k < nfull; ++k) {
            uint4 q[VPC];
#pragma unroll
            for (int jv = 0; jv < VPC; ++jv) q[jv] = lds128(base + (uint32_t)(k * CV + jv * NTC) * 16u);
            stats_chunk<T, VPC>(q, m, s0, s1);
          }
          if (nfull < nchunk) {
            if constexpr (PV) {
#pragma unroll 1
              for (int vb = nfull * CV; vb + ct < my_nvec; vb += NTC) {
                uint4 q[1];
                q[0] = lds128(base + (uint32_t)vb * 16u);
                stats_chunk<T, 1>(q, m, s0, s1);
              }
            } else {
              uint4 q[VPC];
#pragma unroll
              for (int jv = 0; jv < VPC; ++jv) {
                const int vb = nfull * CV + jv * NTC;
                q[jv] = vb + ct < my_nvec ? lds128(base + (uint32_t)vb * 16u) : neg_inf_vec<T>();
              }
              stats_chunk<T, VPC>(q, m, s0, s1);
            }
          }
        }
        float s = s0 + s1;
        group_merge<32>(m, s);
        if (dead) m = NAN;  // the slice never arrived: the row's record and loss become NaN
        float* rd = red + (i & (kStatsRing - 1)) * 64;
        if (lane == 0) { rd[cw] = m; rd[32 + cw] = s; }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(stats_s + 8 * (i & (kStatsRing - 1)));
      slot_a = slot_a + 1 == nslots ? 0 : slot_a + 1;
    }
    // ------------------------------------------------- B(i - lag): gradient of row i - lag, refill
    const int jb = i - lag;
    if (jb >= 0) {
      const int64_t row = row_b;
      const int64_t label = lab_s[jb & (kLabRing - 1)];
      T* dst = dlogits + row * a.rs + (int64_t)slice_elem0 + (int64_t)ct * VE;
      const int jn = jb + nslots;  // the row that takes over this slot
      const int64_t label_n = jn < R ? lab_s[jn & (kLabRing - 1)] : MDY_IGNORE_INDEX;
      const int64_t row_n = row + (int64_t)nslots * lanes;
      // the exchange warp is done with row jb (usually long since): its lse is in shared memory
      vp_wait(3, jb, lse_s + 8 * (jb & (kLseRing - 1)), (uint32_t)(jb >> 2) & 1u, dead, a.wait_tries);
      if (label == MDY_IGNORE_INDEX) {
        if (ct == 0) issue_load(slot_b, row_n, label_n);  // the slot was never used by this row
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (int v = ct; v < my_nvec; v += NTC) st_stream(dst + (int64_t)(v - ct) * VE, z);
      } else {
        const float lse_g = bcast[(jb & (kLseRing - 1)) * 4];
        const float c2 = -lse_g * kLog2e + log2g;
        const uint32_t base = slots_s + (uint32_t)slot_b * a.slot_bytes + my_off;
        // the label's own element, if it lies in this slice: (p - 1) * g, written after the vector store
        int loc = -1;
        {
          const int64_t l = label - col0;
          if (l >= 0 && l < (int64_t)my_nvec * VE) loc = (int)l;
        }
        const bool mine = loc >= 0 && ((loc / VE) % NTC) == ct;
        float xl = 0.f;
        if (mine) xl = to_float(reinterpret_cast<const T*>(smem_raw + (size_t)slot_b * a.slot_bytes)[loc]);
        for (int k = 0; k < nchunk; ++k) {
          uint4 q[VPC];
          const bool whole = k < nfull;
#pragma unroll
          for (int jv = 0; jv < VPC; ++jv) {
            const int vb = k * CV + jv * NTC;
            q[jv] = (whole || vb + ct < my_nvec) ? lds128(base + (uint32_t)vb * 16u) : make_uint4(0, 0, 0, 0);
          }
          if (k == nchunk - 1) {
            bar_sync_id(kBarSlot, NTC);  // the whole slice is in registers or already written: refill the slot
            if (ct == 0) issue_load(slot_b, row_n, label_n);
          }
          if (fold) {
#pragma unroll
            for (int jv = 0; jv < VPC; ++jv) {
              const int vb = k * CV + jv * NTC;
              if (whole || vb + ct < my_nvec) st_stream(dst + (int64_t)vb * VE, grad_vec<T, true>(q[jv], c2, g));
            }
          } else {
#pragma unroll
            for (int jv = 0; jv < VPC; ++jv) {
              const int vb = k * CV + jv * NTC;
              if (whole || vb + ct < my_nvec) st_stream(dst + (int64_t)vb * VE, grad_vec<T, false>(q[jv], c2, g));
            }
          }
        }
        if (mine) {
          const float p = fast_exp2(fmaf(xl, kLog2e, -lse_g * kLog2e));
          dlogits[row * a.rs + slice_elem0 + loc] = from_float<T>((p - 1.f) * g);
        }
      }
      slot_b = slot_b + 1 == nslots ? 0 : slot_b + 1;
      row_b += lanes;
    }
  }
  if (dead) {
    // the thread stopped following the slot barriers: give bulk copies still in flight time to land
    for (int k = 0; k < 100; ++k) __nanosleep(1000);
  }
}

struct VpGeometry { int nsub, vps, slot_bytes, nslots, lag, nt, vpc, per_sm; size_t smem; };

// Slice, ring and CTA shape for shard rows of `vs` elements of `esize` bytes.
inline bool vp_geometry(int64_t vs, int esize, int tp, VpGeometry* out) {
  const int ve = 16 / esize;
  if (vs <= 0 || vs % ve != 0) return false;
  const int64_t nvec = vs / ve;
  const int64_t row_bytes = nvec * 16;
  VpGeometry g;
  // Column slices of at most 32 KB (256 compute threads, two CTAs per SM), or 64 KB for shard rows above 96 KB
  // (512 compute threads, one CTA per SM: the per-row work that does not scale with the slice is amortised
  // over twice the logits; measured 0.81 against 0.77 of the copy bandwidth at 250 KB rows).
  int slice_kb = tunable(MDY_TUNE_CE_VP_SLICE_KB);
  if (slice_kb < 4 || slice_kb > 96) slice_kb = row_bytes > 96 * 1024 ? 64 : 32;
  g.nsub = (int)ceil_div(row_bytes, (int64_t)slice_kb * 1024);
  if (g.nsub * tp > kVpMaxParts) return false;
  g.vps = (int)ceil_div(nvec, g.nsub);
  if ((int64_t)(g.nsub - 1) * g.vps >= nvec) return false;  // a slice would be empty
  const int64_t slice_bytes = (int64_t)g.vps * 16;
  // Compute threads per CTA (plus one exchange warp), 16-byte vectors per thread and chunk, CTAs per SM.  A row's
  // reduction, publish and hand-offs are a serial chain of a few microseconds inside its CTA: short slices need
  // many CTAs per SM to cover it (8 KB of logits are 0.4 us of HBM time per SM), long ones amortise it.
  if (slice_bytes <= 8704) { g.nt = 64; g.vpc = 8; g.per_sm = 8; }
  else if (slice_bytes <= 17408) { g.nt = 128; g.vpc = 8; g.per_sm = 4; }
  else if (slice_bytes <= 40 * 1024) { g.nt = 256; g.vpc = 4; g.per_sm = 2; }
  else { g.nt = 512; g.vpc = 4; g.per_sm = 1; }
  // 16-bit logits: the chunk width (4, 5 or 6 vectors per thread) that leaves the fewest empty lanes in the last
  // chunk.  A 19 KB slice is swept as one chunk of five or six instead of a full chunk of four and a mostly empty
  // second one (0.61 against 0.55 of the copy bandwidth), a 37 KB slice as two of five instead of three of four.
  // Eight per thread in one chunk measured slower than two chunks of four (32 KB slices: 0.72 against 0.75).
  if (esize == 2 && g.nt >= 256) {
    const int64_t need = ceil_div(g.vps, g.nt);
    int64_t best = ceil_div(need, 4) * 4;
    for (int c = 5; c <= 6; ++c) {
      const int64_t padded = ceil_div(need, c) * c;
      if (padded < best) { best = padded; g.vpc = c; }
    }
    // a slice swept as ONE chunk of five or six and short enough for three slots in a third of the shared memory:
    // three CTAs per SM (27 warps instead of 18; the kernel is compiled for 72 registers there)
    if (g.nt == 256 && need <= g.vpc && slice_bytes <= 23 * 1024) g.per_sm = 3;
  }
  if (ceil_div(g.vps, g.nt * g.vpc) > kVpMaxChunks) return false;
  if (tunable(MDY_TUNE_CE_VP_CTAS_PER_SM) > 0) g.per_sm = tunable(MDY_TUNE_CE_VP_CTAS_PER_SM);
  g.slot_bytes = (int)((slice_bytes + 127) / 128 * 128);
  const int fixed = kVpBarriers * 8 + (kStatsRing * 64 + kLseRing * 4) * 4 + kLabRing * 8;
  // at least three slots: fewer CTAs per SM where the asked-for number leaves too little shared memory each
  for (;; --g.per_sm) {
    const int budget = (227 * 1024) / g.per_sm - 1024 - fixed;
    g.nslots = budget / g.slot_bytes;
    if (g.nslots >= 3 || g.per_sm == 1) break;
  }
  if (g.nslots > 5) g.nslots = 5;
  if (tunable(MDY_TUNE_CE_VP_SLOTS) > 0 && tunable(MDY_TUNE_CE_VP_SLOTS) <= g.nslots) g.nslots = tunable(MDY_TUNE_CE_VP_SLOTS);
  if (g.nslots < 3) return false;
  // rows between a row's publish and its poll: what hides the exchange's latency; loads run the other
  // two slots ahead.  At most 3 (the hand-off rings are sized for it).
  g.lag = g.nslots - 2;
  g.smem = (size_t)g.nslots * g.slot_bytes + fixed;
  *out = g;
  return true;
}

template <typename T, int NTC, int VPC, bool PV = false, int MINB = vp_min_blocks(NTC)>
int launch_vp(VpArgs a, const VpGeometry& g, cudaStream_t st) {
  constexpr int NT = NTC + 32;
  auto kern = ce_vp_fused_kernel<T, NTC, VPC, PV, MINB>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return MDY_ERR_UNSUPPORTED; }
  // The occupancy figure below assumes the largest shared-memory carve-out; ask for it, so that the SMs are
  // not left configured with a smaller one in which fewer CTAs fit than the grid counts on.
  (void)cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
  (void)cudaGetLastError();
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NT, g.smem);
  if (e != cudaSuccess || per_sm < 1) { (void)cudaGetLastError(); return MDY_ERR_UNSUPPORTED; }
  if (per_sm > g.per_sm) per_sm = g.per_sm;
  // every CTA of the launch must be resident at once: they wait for one another
  const int resident = per_sm * num_sms();
  int G = resident / a.nvr / a.nsub * a.nsub;
  const int64_t useful = ceil_div(a.M, 1) * a.nsub;        // one row lane per row at most
  if (G > useful) G = (int)useful;
  if (G < a.nsub) return MDY_ERR_UNSUPPORTED;
  a.G = G;
  // A cooperative launch: the runtime either makes every CTA of the grid resident at once or refuses the
  // launch (cudaErrorCooperativeLaunchTooLarge).  The CTAs wait for one another's records, so a grid of which
  // only a part is resident would leave the resident part waiting (bounded, but seconds) for CTAs that cannot
  // start until it is done.
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.gridDim = dim3((unsigned)(G * a.nvr), 1, 1);
  cfg.blockDim = dim3(NT, 1, 1);
  cfg.dynamicSmemBytes = g.smem;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kern, a);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
  return finish_launch(1);
}

std::mutex g_peer_mu;

}  // namespace

int ce_vp_dev_error(bool clear) { return read_dev_error(clear); }

int ce_vp_dev_detail(int k, bool clear) {
  int v[4] = {0, 0, 0, 0};
  if (k < 0 || k > 3 || cudaMemcpyFromSymbol(v, g_vp_detail, sizeof(v)) != cudaSuccess) {
    (void)cudaGetLastError();
    return -1;
  }
  if (clear) {
    const int z[4] = {0, 0, 0, 0};
    (void)cudaMemcpyToSymbol(g_vp_detail, z, sizeof(z));
  }
  return v[k];
}

}  // namespace mdy

using namespace mdy;

extern "C" {

int64_t mdy_ce_vp_exchange_bytes(int64_t max_rows, int64_t shard_cols, int tp, int dtype) {
  if (max_rows <= 0 || tp <= 0 || tp > kVpMaxRanks) return MDY_ERR_SIZE;
  const int esize = dtype == MDY_F32 ? 4 : (dtype == MDY_F16 || dtype == MDY_BF16) ? 2 : 0;
  if (!esize) return MDY_ERR_DTYPE;
  VpGeometry g;
  if (!vp_geometry(shard_cols, esize, tp, &g)) return MDY_ERR_UNSUPPORTED;
  return (int64_t)2 * max_rows * tp * g.nsub * 16;
}

int mdy_ce_vp_geometry(int64_t shard_cols, int tp, int dtype, int32_t* out8) {
  if (!out8) return MDY_ERR_NULL;
  if (shard_cols <= 0 || tp <= 0 || tp > kVpMaxRanks) return MDY_ERR_SIZE;
  const int esize = dtype == MDY_F32 ? 4 : (dtype == MDY_F16 || dtype == MDY_BF16) ? 2 : 0;
  if (!esize) return MDY_ERR_DTYPE;
  VpGeometry g;
  if (!vp_geometry(shard_cols, esize, tp, &g)) return MDY_ERR_UNSUPPORTED;
  const int v[8] = {g.nsub, g.vps, g.slot_bytes, g.nslots, g.lag, g.nt, g.vpc, g.per_sm};
  for (int k = 0; k < 8; ++k) out8[k] = v[k];
  return MDY_OK;
}

int mdy_ce_vp_fused(const void* const* logits, void* const* dlogits, float* const* losses, float* const* lse,
                    void* const* exchange, const int64_t* labels, const float* grad_scale_dev,
                    float grad_scale_host, int64_t M, int64_t shard_cols, int64_t row_stride, int tp,
                    int first_rank, int n_local_ranks, int64_t exchange_rows, uint32_t epoch, int dtype,
                    void* stream) {
  if (M < 0 || shard_cols <= 0 || row_stride < shard_cols || exchange_rows < M) return MDY_ERR_SIZE;
  if (tp <= 0 || tp > kVpMaxRanks || n_local_ranks <= 0 || first_rank < 0 || first_rank + n_local_ranks > tp)
    return MDY_ERR_ARG;
  if (M > INT32_MAX || epoch == 0) return MDY_ERR_ARG;
  if (dtype != MDY_F32 && dtype != MDY_F16 && dtype != MDY_BF16) return MDY_ERR_DTYPE;
  if (M == 0) return MDY_OK;
  if (!logits || !dlogits || !losses || !lse || !exchange || !labels) return MDY_ERR_NULL;
  VpArgs a = {};
  for (int v = 0; v < n_local_ranks; ++v) {
    if (!logits[v] || !dlogits[v] || !losses[v] || !lse[v]) return MDY_ERR_NULL;
    if (!aligned16(logits[v]) || !aligned16(dlogits[v])) return MDY_ERR_UNSUPPORTED;
    a.logits[v] = logits[v]; a.dlogits[v] = dlogits[v]; a.losses[v] = losses[v]; a.lse[v] = lse[v];
  }
  for (int r = 0; r < tp; ++r) {
    if (!exchange[r]) return MDY_ERR_NULL;
    if (!aligned16(exchange[r])) return MDY_ERR_ARG;
    a.xbuf[r] = reinterpret_cast<uint4*>(exchange[r]);
  }
  a.labels = labels; a.gdev = grad_scale_dev; a.ghost = grad_scale_host;
  a.M = (int)M; a.vs = shard_cols; a.rs = row_stride;
  a.tp = tp; a.nvr = n_local_ranks; a.rank0 = first_rank;
  a.xrows = (int)exchange_rows; a.epoch = epoch;
  const int hook = tunable(MDY_TUNE_CE_WAIT_TEST);
  a.wait_tries = hook > 0 ? (1 << 12) : (1 << 22);
  a.mute_part = hook > 0 ? hook : 0;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VE = VecInfo<T>::kElems;
    if (row_stride % VE != 0) return (int)MDY_ERR_UNSUPPORTED;
    VpGeometry g;
    if (!vp_geometry(shard_cols, (int)sizeof(T), tp, &g)) return (int)MDY_ERR_UNSUPPORTED;
    a.nsub = g.nsub; a.vps = g.vps; a.slot_bytes = g.slot_bytes; a.nslots = g.nslots; a.lag = g.lag;
    // a whole vector per thread (or more) of the last chunk is empty: sweep that chunk vector by vector
    const int64_t need = ceil_div(g.vps, g.nt);
    const bool pv = ceil_div(need, g.vpc) * g.vpc > need;
    if (pv) {
      if (g.nt == 64) return launch_vp<T, 64, 8, true>(a, g, (cudaStream_t)stream);
      if (g.nt == 128) return launch_vp<T, 128, 8, true>(a, g, (cudaStream_t)stream);
      if (g.nt == 256 && g.vpc == 4) return launch_vp<T, 256, 4, true>(a, g, (cudaStream_t)stream);
      if (g.nt == 512 && g.vpc == 4) return launch_vp<T, 512, 4, true>(a, g, (cudaStream_t)stream);
    }
    if (g.nt == 64) return launch_vp<T, 64, 8>(a, g, (cudaStream_t)stream);
    if (g.nt == 128) return launch_vp<T, 128, 8>(a, g, (cudaStream_t)stream);
    if constexpr (sizeof(T) == 2) {
      if (g.nt == 256 && g.per_sm == 3 && g.vpc == 5) return launch_vp<T, 256, 5, false, 3>(a, g, (cudaStream_t)stream);
      if (g.nt == 256 && g.per_sm == 3 && g.vpc == 6) return launch_vp<T, 256, 6, false, 3>(a, g, (cudaStream_t)stream);
      if (g.nt == 256 && g.vpc == 5) return launch_vp<T, 256, 5>(a, g, (cudaStream_t)stream);
      if (g.nt == 512 && g.vpc == 5) return launch_vp<T, 512, 5>(a, g, (cudaStream_t)stream);
      if (g.nt == 256 && g.vpc == 6) return launch_vp<T, 256, 6>(a, g, (cudaStream_t)stream);
      if (g.nt == 512 && g.vpc == 6) return launch_vp<T, 512, 6>(a, g, (cudaStream_t)stream);
    }
    if (g.nt == 256) return launch_vp<T, 256, 4>(a, g, (cudaStream_t)stream);
    return launch_vp<T, 512, 4>(a, g, (cudaStream_t)stream);
  });
}

// ---- set-up of the exchange buffers (not on the hot path) ---------------------------------------
// The buffer a rank's peers write into has to be device memory another process can map, so it is the
// one thing this library allocates itself: cudaMalloc, zero-filled (epoch tags start at 1), exported as
// a CUDA IPC handle the caller passes to its peers through any channel it likes.

int mdy_peer_buffer_create(int64_t bytes, void** ptr, void* ipc_handle_64_bytes) {
  if (bytes <= 0 || !ptr || !ipc_handle_64_bytes) return MDY_ERR_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  std::lock_guard<std::mutex> lock(g_peer_mu);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { (void)cudaGetLastError(); (void)cudaFree(p); return (int)e; }
  memcpy(ipc_handle_64_bytes, &h, 64);
  *ptr = p;
  return MDY_OK;
}

int mdy_peer_buffer_open(const void* ipc_handle_64_bytes, void** ptr) {
  if (!ipc_handle_64_bytes || !ptr) return MDY_ERR_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle_64_bytes, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
  *ptr = p;
  return MDY_OK;
}

int mdy_peer_buffer_close(void* ptr) {
  if (!ptr) return MDY_OK;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
  return MDY_OK;
}

int mdy_peer_buffer_destroy(void* ptr) {
  if (!ptr) return MDY_OK;
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
  return MDY_OK;
}

}  // extern "C"
