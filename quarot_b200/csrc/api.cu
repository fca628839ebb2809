// Library-wide host utilities: error strings, device status word, tuning knobs.
#include "common.cuh"

#include <map>
#include <mutex>
#include <string>
#include <string.h>

namespace qr {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_err, sizeof(g_err), "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  return (int)e;
}

// One status word per device, in that device's global memory.  Kernels write a
// non-zero code into it when a bounded wait gives up.
__device__ int g_kernel_status = 0;

int* kernel_status_ptr() {
  static std::mutex mu;
  static std::map<int, int*> cache;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lk(mu);
  auto it = cache.find(dev);
  if (it != cache.end()) return it->second;
  int* p = nullptr;
  if (cudaGetSymbolAddress((void**)&p, g_kernel_status) != cudaSuccess) return nullptr;
  cache[dev] = p;
  return p;
}

int num_sms() {
  static std::mutex mu;
  static std::map<int, int> cache;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  std::lock_guard<std::mutex> lk(mu);
  auto it = cache.find(dev);
  if (it != cache.end()) return it->second;
  int n = 148;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  cache[dev] = n;
  return n;
}

static void* g_trace_ptr = nullptr;   // set through qr_debug_set_trace (debugging aid)
void* debug_trace_ptr() { return g_trace_ptr; }

static std::mutex g_tune_mu;
static std::map<std::string, int> g_tune;

int tuning(const char* key, int dflt) {
  std::lock_guard<std::mutex> lk(g_tune_mu);
  auto it = g_tune.find(key);
  return it == g_tune.end() ? dflt : it->second;
}

}  // namespace qr

extern "C" {

int qr_version(void) { return QR_VERSION; }

const char* qr_last_error(void) { return qr::g_err; }

int qr_kernel_status(int* status_out) {
  if (!status_out) return qr::fail(QR_EINVAL, "qr_kernel_status: null output");
  int* p = qr::kernel_status_ptr();
  if (!p) return qr::fail(QR_ENOTREADY, "qr_kernel_status: no CUDA device");
  QR_CUDA(cudaDeviceSynchronize());
  QR_CUDA(cudaMemcpy(status_out, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status_out != 0) {
    int zero = 0;
    QR_CUDA(cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice));
  }
  return QR_OK;
}

int qr_debug_set_trace(void* device_buffer) {
  qr::g_trace_ptr = device_buffer;
  return QR_OK;
}

int qr_set_tuning(const char* key, int value) {
  static const char* known[] = {"gemm_bn", "gemm_pst", "gemm_ist", "gemm_acc", "gemm_grid",
                                "gemm_swap_max_m", "gemm_splitk", "gemm_2sm", "gemm_ts", "gemm_sync", "gemm_debug", "gemm_tma_out", "gemv_max_m", "pdl", "hadq_debug", "hadq_path", "hadq_tc", nullptr};
  if (!key) return qr::fail(QR_EINVAL, "qr_set_tuning: null key");
  for (int i = 0; known[i]; ++i) {
    if (strcmp(known[i], key) == 0) {
      std::lock_guard<std::mutex> lk(qr::g_tune_mu);
      qr::g_tune[key] = value;
      return QR_OK;
    }
  }
  return qr::fail(QR_EINVAL, "qr_set_tuning: unknown key '%s'", key);
}

}  // extern "C"
