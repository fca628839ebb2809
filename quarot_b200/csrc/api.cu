// Library-wide host utilities: error strings, device status word, tuning knobs.
#include "common.cuh"

#include <map>
#include <mutex>
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

// Tuning knobs: plain ints that qr_set_tuning overwrites; the launch path reads them without a lock or a lookup.
Tuning g_tuning;

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

int qr_set_tuning(const char* key, int value) {
  static const struct { const char* name; int qr::Tuning::*field; } known[] = {
      {"gemm_bn", &qr::Tuning::gemm_bn},           {"gemm_pst", &qr::Tuning::gemm_pst},
      {"gemm_grid", &qr::Tuning::gemm_grid},       {"gemm_decode_max_m", &qr::Tuning::gemm_decode_max_m},
      {"gemm_splitk", &qr::Tuning::gemm_splitk},   {"gemm_2sm", &qr::Tuning::gemm_2sm},
      {"gemm_tma_out", &qr::Tuning::gemm_tma_out}, {"gemv_max_m", &qr::Tuning::gemv_max_m},
      {"pdl", &qr::Tuning::pdl},                   {"hadq_path", &qr::Tuning::hadq_path},
      {"hadq_tc", &qr::Tuning::hadq_tc},           {"gemm_decode", &qr::Tuning::gemm_decode},
      {"gemm_bn2", &qr::Tuning::gemm_bn2},         {"hadq_walsh", &qr::Tuning::hadq_walsh},
      {"gemv_mma_max_m", &qr::Tuning::gemv_mma_max_m}, {"gemv_mma_halves", &qr::Tuning::gemv_mma_halves}, {"gemv_mma_two_pass", &qr::Tuning::gemv_mma_two_pass}, {"hadq_split", &qr::Tuning::hadq_split}, {"hadq_heads", &qr::Tuning::hadq_heads}, {"gemm_tail_help", &qr::Tuning::gemm_tail_help},
  };
  if (!key) return qr::fail(QR_EINVAL, "qr_set_tuning: null key");
  for (const auto& k : known) {
    if (strcmp(k.name, key) == 0) {
      qr::g_tuning.*(k.field) = value;
      return QR_OK;
    }
  }
  return qr::fail(QR_EINVAL, "qr_set_tuning: unknown key '%s'", key);
}

}  // extern "C"
