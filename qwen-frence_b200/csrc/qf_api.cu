// Library-wide plumbing of libqf_hotpath.so: ABI version, per-thread error
// text, the per-device status word kernels write when they meet a bad page id,
// and the tuning switches.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "qf_common.cuh"

namespace qf {

namespace {
thread_local char g_error[512] = "";
__device__ int g_status_word = 0;
int g_dependent_launch = 1;
int g_ordered_launch = 0;
}  // namespace

void request_ordered_launch() { g_ordered_launch = 1; }
int take_ordered_launch() {
  const int taken = g_ordered_launch;
  g_ordered_launch = 0;
  return taken;
}

int dependent_launch_enabled() { return g_dependent_launch; }
void disable_dependent_launch() { g_dependent_launch = 0; }

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t err, const char* what) {
  return fail(QF_ECUDA, "%s failed: %s (%s)", what, cudaGetErrorName(err), cudaGetErrorString(err));
}

int* device_status_word() {
  int* ptr = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_status_word) != cudaSuccess) {
    return nullptr;
  }
  return ptr;
}

}  // namespace qf

extern "C" {

int qf_abi_version(void) { return QF_ABI_VERSION; }

const char* qf_last_error(void) { return qf::g_error; }

int qf_set_dependent_launch(int32_t enabled) {
  qf::g_dependent_launch = enabled ? 1 : 0;
  return QF_OK;
}

int qf_order_next_launch(void) {
  qf::request_ordered_launch();
  return QF_OK;
}

int qf_device_status(int32_t* status, int32_t reset) {
  QF_REQUIRE(status != nullptr, "status must not be null");
  int value = 0;
  QF_CUDA(cudaMemcpyFromSymbol(&value, qf::g_status_word, sizeof(int)));
  *status = value;
  if (reset) {
    const int zero = 0;
    QF_CUDA(cudaMemcpyToSymbol(qf::g_status_word, &zero, sizeof(int)));
  }
  return QF_OK;
}

}  // extern "C"
