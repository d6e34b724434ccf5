// Library-level entry points: version, SM count, launch counter, tunables, status text.
#include <atomic>
#include "common.cuh"

namespace mdy {

static std::atomic<int64_t> g_launches{0};
static std::atomic<int> g_tunables[MDY_TUNE_COUNT];
static std::atomic<int> g_sms[64];

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int tunable(int id) {
  if (id < 0 || id >= MDY_TUNE_COUNT) return 0;
  return g_tunables[id].load(std::memory_order_relaxed);
}

int num_sms() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  if (dev >= 0 && dev < 64) {
    int c = g_sms[dev].load(std::memory_order_relaxed);
    if (c > 0) return c;
  }
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  if (dev >= 0 && dev < 64) g_sms[dev].store(n, std::memory_order_relaxed);
  return n;
}

}  // namespace mdy

extern "C" {

int mdy_version(void) { return 1; }

int mdy_num_sms(void) { return mdy::num_sms(); }

int64_t mdy_launch_count(void) { return mdy::g_launches.load(std::memory_order_relaxed); }

const char* mdy_status_string(int status) {
  switch (status) {
    case MDY_OK: return "ok";
    case MDY_ERR_NULL: return "a required pointer is NULL";
    case MDY_ERR_DTYPE: return "unsupported dtype code";
    case MDY_ERR_SIZE: return "invalid size or stride";
    case MDY_ERR_UNSUPPORTED: return "size above a compiled limit";
    case MDY_ERR_ARG: return "inconsistent argument";
    default: break;
  }
  if (status > 0) return cudaGetErrorString((cudaError_t)status);
  return "unknown status";
}

int mdy_set_tunable(int id, int value) {
  if (id < 0 || id >= MDY_TUNE_COUNT) return MDY_ERR_ARG;
  mdy::g_tunables[id].store(value > 0 ? value : 0, std::memory_order_relaxed);
  return MDY_OK;
}

int mdy_get_tunable(int id) {
  if (id < 0 || id >= MDY_TUNE_COUNT) return MDY_ERR_ARG;
  return mdy::g_tunables[id].load(std::memory_order_relaxed);
}

}  // extern "C"
