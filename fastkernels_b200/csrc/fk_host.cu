// Host-side plumbing shared by every entry point: error text, launch counter,
// device properties, driver entry point for tensor-map encoding.
#include "fk_common.cuh"

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace fk {

static thread_local char g_err[512] = {0};
static std::atomic<int64_t> g_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int sm_count() {
  static int cached[64];
  static std::once_flag once;
  std::call_once(once, [] { memset(cached, 0, sizeof(cached)); });
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) !=
            cudaSuccess ||
        n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static std::atomic<int> g_pdl{-1};
bool pdl_enabled() {
  int v = g_pdl.load(std::memory_order_relaxed);
  if (v < 0) {
    const char* e = getenv("FK_B200_PDL");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
    g_pdl.store(v, std::memory_order_relaxed);
  }
  return v != 0;
}

tensormap_encode_fn get_tensormap_encode() {
  static tensormap_encode_fn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault,
                                &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<tensormap_encode_fn>(p);
  });
  return fn;
}

}  // namespace fk

extern "C" {

int fk_version(void) { return 100; /* 0.1.0 */ }

const char* fk_last_error(void) { return fk::g_err; }

int fk_set_pdl(int enabled) {
  const int prev = fk::pdl_enabled() ? 1 : 0;
  fk::g_pdl.store(enabled ? 1 : 0, std::memory_order_relaxed);
  return prev;
}

int64_t fk_launch_count(void) {
  return fk::g_launches.load(std::memory_order_relaxed);
}

}  // extern "C"
