// Rotate-half RoPE on q and k in one launch, forward and backward, for sm_100a.
//
// Work item = (token, chunk of HPT heads, 16-byte column j of the first half of the head).  The
// thread that owns column j of the first half also owns column j of the second half, so the rotation
// is register-local.  The four cos/sin vectors of the token are loaded once per item (they stay in
// L1/L2 across the heads of a token) and reused for the HPT heads of the chunk; all 2*HPT activation
// loads are issued before the first use.  HPT = 1 by default: fewest registers, most threads in flight.  q heads
// and k heads of a token are addressed as one list of QH+KH heads, so one launch covers both tensors.
// Input and output take independent (batch, head, position) strides: forward runs in place on the
// [B, L, H, D] projection output, backward can read an arbitrarily strided gradient and write it in
// the layout the projection's backward wants.
#include "common.cuh"

namespace mdy {
namespace {

struct RopeArgs {
  const void* qi; void* qo; const void* ki; void* ko;
  const void* cos; const void* sin;
  int64_t qi_sb, qi_sh, qi_sl, qo_sb, qo_sh, qo_sl;
  int64_t ki_sb, ki_sh, ki_sl, ko_sb, ko_sh, ko_sl;
  int64_t cos_sb;  // 0 when cos/sin are broadcast over batch, else L*D
  int B, L, QH, KH, D;
};

template <bool BWD>
__device__ __forceinline__ void rotate(float& a, float& b, float c1, float c2, float s1, float s2) {
  // forward : o1 = x1*c1 - x2*s1 ; o2 = x2*c2 + x1*s2
  // backward: d1 = g1*c1 + g2*s2 ; d2 = g2*c2 - g1*s1
  const float x1 = a, x2 = b;
  if (!BWD) {
    a = x1 * c1 - x2 * s1;
    b = x2 * c2 + x1 * s2;
  } else {
    a = x1 * c1 + x2 * s2;
    b = x2 * c2 - x1 * s1;
  }
}

// IDX is the type of the flat work-item index: uint32_t whenever the item count fits (the usual case;
// 32-bit divisions cost a fraction of the emulated 64-bit ones and this kernel is issue-bound), else int64_t.
template <typename T, bool BWD, int HPT, typename IDX>
__global__ void __launch_bounds__(256)
rope_vec(RopeArgs a) {
  constexpr int VE = VecInfo<T>::kElems;
  const int half = a.D >> 1;
  const int hv = half / VE;                      // vectors per half head
  const int H = a.QH + a.KH;
  const int nchunk = (H + HPT - 1) / HPT;
  const IDX per_tok = (IDX)hv * (IDX)nchunk;
  const IDX total = (IDX)a.B * (IDX)a.L * per_tok;
  const T* cosp = (const T*)a.cos;
  const T* sinp = (const T*)a.sin;

  for (IDX idx = (IDX)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (IDX)gridDim.x * blockDim.x) {
    const IDX tok = idx / per_tok;
    const int rem = (int)(idx - tok * per_tok);
    const int chunk = (int)((unsigned)rem / (unsigned)hv);
    const int j = rem - chunk * hv;
    const int b = (int)(tok / (IDX)a.L);
    const int l = (int)(tok - (IDX)b * (IDX)a.L);

    const int64_t cs_off = (int64_t)b * a.cos_sb + (int64_t)l * a.D + (int64_t)j * VE;
    const uint4 c1v = ld_reuse(cosp + cs_off);
    const uint4 c2v = ld_reuse(cosp + cs_off + half);
    const uint4 s1v = ld_reuse(sinp + cs_off);
    const uint4 s2v = ld_reuse(sinp + cs_off + half);

    const T* src[HPT];
    T* dst[HPT];
    uint4 v1[HPT], v2[HPT];
#pragma unroll
    for (int u = 0; u < HPT; ++u) {
      const int h = chunk * HPT + u;
      if (h < a.QH) {
        src[u] = (const T*)a.qi + b * a.qi_sb + h * a.qi_sh + l * a.qi_sl + (int64_t)j * VE;
        dst[u] = (T*)a.qo + b * a.qo_sb + h * a.qo_sh + l * a.qo_sl + (int64_t)j * VE;
      } else if (h < H) {
        const int hk = h - a.QH;
        src[u] = (const T*)a.ki + b * a.ki_sb + hk * a.ki_sh + l * a.ki_sl + (int64_t)j * VE;
        dst[u] = (T*)a.ko + b * a.ko_sb + hk * a.ko_sh + l * a.ko_sl + (int64_t)j * VE;
      } else {
        src[u] = nullptr;
        dst[u] = nullptr;
      }
    }
#pragma unroll
    for (int u = 0; u < HPT; ++u) {
      if (src[u]) {
        v1[u] = ld_stream(src[u]);
        v2[u] = ld_stream(src[u] + half);
      }
    }
    float c1[VE], c2[VE], s1[VE], s2[VE];
    unpack<T>(c1v, c1); unpack<T>(c2v, c2); unpack<T>(s1v, s1); unpack<T>(s2v, s2);
#pragma unroll
    for (int u = 0; u < HPT; ++u) {
      if (src[u]) {
        float x1[VE], x2[VE];
        unpack<T>(v1[u], x1);
        unpack<T>(v2[u], x2);
#pragma unroll
        for (int e = 0; e < VE; ++e) rotate<BWD>(x1[e], x2[e], c1[e], c2[e], s1[e], s2[e]);
        st_plain(dst[u], pack<T>(x1));
        st_plain(dst[u] + half, pack<T>(x2));
      }
    }
  }
}

// Any even D / any alignment: one thread per (token, head, column pair).
template <typename T, bool BWD>
__global__ void __launch_bounds__(256)
rope_scalar(RopeArgs a) {
  const int half = a.D >> 1;
  const int H = a.QH + a.KH;
  const int64_t total = (int64_t)a.B * a.L * H * half;
  const T* cosp = (const T*)a.cos;
  const T* sinp = (const T*)a.sin;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int j = (int)(idx % half);
    const int64_t r = idx / half;
    const int h = (int)(r % H);
    const int64_t tok = r / H;
    const int b = (int)(tok / a.L);
    const int l = (int)(tok - (int64_t)b * a.L);
    const int64_t cs_off = (int64_t)b * a.cos_sb + (int64_t)l * a.D + j;
    const float c1 = to_float(cosp[cs_off]), c2 = to_float(cosp[cs_off + half]);
    const float s1 = to_float(sinp[cs_off]), s2 = to_float(sinp[cs_off + half]);
    const T* src;
    T* dst;
    if (h < a.QH) {
      src = (const T*)a.qi + b * a.qi_sb + h * a.qi_sh + l * a.qi_sl + j;
      dst = (T*)a.qo + b * a.qo_sb + h * a.qo_sh + l * a.qo_sl + j;
    } else {
      const int hk = h - a.QH;
      src = (const T*)a.ki + b * a.ki_sb + hk * a.ki_sh + l * a.ki_sl + j;
      dst = (T*)a.ko + b * a.ko_sb + hk * a.ko_sh + l * a.ko_sl + j;
    }
    float x1 = to_float(src[0]), x2 = to_float(src[half]);
    rotate<BWD>(x1, x2, c1, c2, s1, s2);
    dst[0] = from_float<T>(x1);
    dst[half] = from_float<T>(x2);
  }
}

template <typename T, int HPT>
int launch_rope_h(const RopeArgs& a, bool bwd, cudaStream_t st) {
  constexpr int VE = VecInfo<T>::kElems;
  const int half = a.D / 2;
  auto ok = [&](int64_t s) { return s % VE == 0; };
  bool vec = half % VE == 0 && aligned16(a.cos) && aligned16(a.sin) &&
             (a.QH == 0 || (aligned16(a.qi) && aligned16(a.qo))) &&
             (a.KH == 0 || (aligned16(a.ki) && aligned16(a.ko))) &&
             ok(a.qi_sb) && ok(a.qi_sh) && ok(a.qi_sl) && ok(a.qo_sb) && ok(a.qo_sh) && ok(a.qo_sl) &&
             ok(a.ki_sb) && ok(a.ki_sh) && ok(a.ki_sl) && ok(a.ko_sb) && ok(a.ko_sh) && ok(a.ko_sl) &&
             ok(a.cos_sb);
  int threads = tunable(MDY_TUNE_ROPE_THREADS);
  if (threads < 32 || threads > 256 || (threads & 31)) threads = 128;
  const int H = a.QH + a.KH;
  int64_t items;
  if (vec) items = (int64_t)a.B * a.L * (half / VE) * ((H + HPT - 1) / HPT);
  else items = (int64_t)a.B * a.L * H * half;
  if (items == 0) return MDY_OK;
  int64_t grid = ceil_div(items, threads);
  int waves = tunable(MDY_TUNE_ROPE_GRID_PER_SM);
  if (waves <= 0) waves = 64;
  const int64_t cap = (int64_t)(num_sms() > 0 ? num_sms() : 1) * waves;
  if (grid > cap) grid = cap;
  if (vec) {
    // the grid-stride loop adds at most grid*threads to an index below `items`
    const bool small = items + grid * threads < ((int64_t)1 << 32);
    if (small) {
      if (bwd) rope_vec<T, true, HPT, uint32_t><<<(unsigned)grid, threads, 0, st>>>(a);
      else rope_vec<T, false, HPT, uint32_t><<<(unsigned)grid, threads, 0, st>>>(a);
    } else {
      if (bwd) rope_vec<T, true, HPT, int64_t><<<(unsigned)grid, threads, 0, st>>>(a);
      else rope_vec<T, false, HPT, int64_t><<<(unsigned)grid, threads, 0, st>>>(a);
    }
  } else {
    if (bwd) rope_scalar<T, true><<<(unsigned)grid, threads, 0, st>>>(a);
    else rope_scalar<T, false><<<(unsigned)grid, threads, 0, st>>>(a);
  }
  return finish_launch(1);
}

template <typename T>
int launch_rope(const RopeArgs& a, bool bwd, cudaStream_t st) {
  // default from an on-device sweep (32q/8kv heads x 128, bf16): one head per item and 128-thread CTAs
  // (44 registers, full occupancy) beat 2 or 4 heads per item (75-115 registers) by 12 %
  switch (tunable(MDY_TUNE_ROPE_HEADS_PER_THREAD)) {
    case 2: return launch_rope_h<T, 2>(a, bwd, st);
    case 4: return launch_rope_h<T, 4>(a, bwd, st);
    default: return launch_rope_h<T, 1>(a, bwd, st);
  }
}

}  // namespace
}  // namespace mdy

using namespace mdy;

extern "C" int mdy_rope(const void* q_in, void* q_out, const void* k_in, void* k_out, const void* cos,
                        const void* sin, int64_t B, int64_t L, int64_t QH, int64_t KH, int64_t D,
                        int64_t cos_b, int64_t qi_sb, int64_t qi_sh, int64_t qi_sl, int64_t qo_sb,
                        int64_t qo_sh, int64_t qo_sl, int64_t ki_sb, int64_t ki_sh, int64_t ki_sl,
                        int64_t ko_sb, int64_t ko_sh, int64_t ko_sl, int backward, int dtype,
                        void* stream) {
  if (B < 0 || L < 0 || QH < 0 || KH < 0 || D <= 0 || (D & 1)) return MDY_ERR_SIZE;
  if (B > INT32_MAX || L > INT32_MAX || QH > 65535 || KH > 65535 || D > 65536) return MDY_ERR_UNSUPPORTED;
  if (cos_b != 1 && cos_b != B) return MDY_ERR_ARG;
  if (B == 0 || L == 0 || QH + KH == 0) return MDY_OK;
  if (!cos || !sin) return MDY_ERR_NULL;
  if (QH > 0 && (!q_in || !q_out)) return MDY_ERR_NULL;
  if (KH > 0 && (!k_in || !k_out)) return MDY_ERR_NULL;
  RopeArgs a;
  a.qi = q_in; a.qo = q_out; a.ki = k_in; a.ko = k_out; a.cos = cos; a.sin = sin;
  a.qi_sb = qi_sb; a.qi_sh = qi_sh; a.qi_sl = qi_sl; a.qo_sb = qo_sb; a.qo_sh = qo_sh; a.qo_sl = qo_sl;
  a.ki_sb = ki_sb; a.ki_sh = ki_sh; a.ki_sl = ki_sl; a.ko_sb = ko_sb; a.ko_sh = ko_sh; a.ko_sl = ko_sl;
  a.cos_sb = (cos_b == 1 && B != 1) ? 0 : L * D;
  a.B = (int)B; a.L = (int)L; a.QH = (int)QH; a.KH = (int)KH; a.D = (int)D;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    return launch_rope<T>(a, backward != 0, (cudaStream_t)stream);
  });
}
