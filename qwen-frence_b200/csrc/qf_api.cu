// Library-wide plumbing of libqf_hotpath.so: ABI version, per-thread error
// text, the per-device status word kernels write when they meet a bad page id,
// and the tuning switches.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "qf_common.cuh"

namespace qf {

namespace {
thread_local char g_error[512] = "";
__device__ int g_status_word = 0;
// Process-wide switches.  They are atomics, so concurrent calls cannot tear them, but they
// are still ONE switch each: the pending ordered launch is consumed by the next chained
// launch of the process, whichever thread or stream makes it.  A host that drives several
// streams from several threads must make the request and the launch it is meant for from the
// same thread with no other launch of this library in between (the reference's loop is one
// thread and one stream, engine/cpp/include/iteration_loop.hpp:157-161).
std::atomic<int> g_dependent_launch{1};
std::atomic<int> g_ordered_launch{0};
}  // namespace

void request_ordered_launch() { g_ordered_launch.store(1, std::memory_order_release); }
int take_ordered_launch() { return g_ordered_launch.exchange(0, std::memory_order_acq_rel); }

int dependent_launch_enabled() { return g_dependent_launch.load(std::memory_order_acquire); }
void disable_dependent_launch() { g_dependent_launch.store(0, std::memory_order_release); }

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
  qf::g_dependent_launch.store(enabled ? 1 : 0, std::memory_order_release);
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
