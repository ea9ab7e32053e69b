// Shared helpers for the libqf_hotpath.so translation units: error reporting,
// element-type conversion and metadata loads.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qf_hotpath.h"

namespace qf {

// ---- host side -----------------------------------------------------------
int fail(int code, const char* fmt, ...);  // records the message, returns code
int cuda_fail(cudaError_t err, const char* what);

#define QF_REQUIRE(cond, ...)                              \
  do {                                                     \
    if (!(cond)) return ::qf::fail(QF_EINVAL, __VA_ARGS__); \
  } while (0)

#define QF_CUDA(expr)                                         \
  do {                                                        \
    cudaError_t qf_err__ = (expr);                            \
    if (qf_err__ != cudaSuccess) return ::qf::cuda_fail(qf_err__, #expr); \
  } while (0)

// Address of the per-device status word (file-scope __device__ int).
int* device_status_word();

// Whether launch_chained() asks for programmatic stream serialization (1, default) or
// launches the ordinary way (0); see qf_set_dependent_launch.
int dependent_launch_enabled();
void disable_dependent_launch();
// qf_order_next_launch(): the next launch_chained() launches the ordinary way.
void request_ordered_launch();
int take_ordered_launch();  // 1 once after a request, else 0

// Status codes kernels may record (1 is reserved).
constexpr int kStatusBadPageId = QF_STATUS_BAD_PAGE_ID;
constexpr int kStatusMergeTimeout = QF_STATUS_MERGE_TIMEOUT;  // a warp gave up waiting for an earlier piece's merge
constexpr int kStatusPositionPastTable = QF_STATUS_POSITION_PAST_TABLE;
constexpr int kStatusPipelineTimeout = QF_STATUS_PIPELINE_TIMEOUT;  // a bounded barrier wait of the GEMM ran out

// ---- device side ---------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T>
__device__ __forceinline__ T from_float(float x);
template <>
__device__ __forceinline__ __half from_float<__half>(float x) {
  return __float2half_rn(x);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

// Two packed 16-bit elements (one 32-bit register) -> float2.
template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t bits);
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t bits) {
  __half2 h = *reinterpret_cast<__half2*>(&bits);
  return __half22float2(h);
}
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t bits) {
  float2 r;
  r.x = __uint_as_float(bits << 16);
  r.y = __uint_as_float(bits & 0xffff0000u);
  return r;
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Two e4m3 bytes (low 16 bits) -> float2 (exact: every e4m3 value is an fp16 value).
__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t bits) {
  __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(bits, __NV_E4M3);
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}

__device__ __forceinline__ int64_t load_index(const void* base, int dtype, int64_t offset) {
  if (dtype == QF_INDEX_I64) return static_cast<const int64_t*>(base)[offset];
  return static_cast<const int32_t*>(base)[offset];
}

__device__ __forceinline__ void store_index(void* base, int dtype, int64_t offset, int64_t value) {
  if (dtype == QF_INDEX_I64) {
    static_cast<int64_t*>(base)[offset] = value;
  } else {
    static_cast<int32_t*>(base)[offset] = static_cast<int32_t>(value);
  }
}

__device__ __forceinline__ float load_position(const void* base, int dtype, int64_t offset) {
  if (dtype == QF_INDEX_F32) return static_cast<const float*>(base)[offset];
  if (dtype == QF_INDEX_I64) return static_cast<float>(static_cast<const int64_t*>(base)[offset]);
  return static_cast<float>(static_cast<const int32_t*>(base)[offset]);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Programmatic dependent launch (the kernels of one decode layer run back to back
// on one stream): a kernel launched through launch_chained() may become resident
// while its predecessor still runs.  It must call dependency_wait() before it reads
// anything an earlier kernel wrote and before its own first global write; what it
// does earlier (index arithmetic, reads of step metadata that no kernel writes)
// overlaps the predecessor's tail.  release_dependents() lets the next kernel of the
// stream be scheduled as soon as resources free up.  Both are no-ops in a kernel
// launched the ordinary way.
__device__ __forceinline__ void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void release_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Launch `kernel` so that it may overlap the tail of the previous kernel of `stream`
// (the kernel itself orders its memory accesses with dependency_wait()).  Falls back
// to an ordinary launch, for good, if the driver refuses the attribute.  With a
// ClusterShape as the first kernel argument slot the grid is launched as thread-block
// clusters of that shape.
struct ClusterShape {
  unsigned x, y, z;
};

template <typename... Params, typename... Args>
inline cudaError_t launch_chained_impl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                       cudaStream_t stream, const ClusterShape* cluster, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid, config.blockDim = block;
  config.dynamicSmemBytes = smem, config.stream = stream;
  cudaLaunchAttribute attribute[2];
  unsigned count = 0;
  if (cluster != nullptr) {
    attribute[count].id = cudaLaunchAttributeClusterDimension;
    attribute[count].val.clusterDim.x = cluster->x;
    attribute[count].val.clusterDim.y = cluster->y;
    attribute[count].val.clusterDim.z = cluster->z;
    ++count;
  }
  const bool ordered = take_ordered_launch() != 0;
  const bool chained = dependent_launch_enabled() && !ordered;
  attribute[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[count].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = count + (chained ? 1 : 0);
  cudaError_t err = cudaLaunchKernelEx(&config, kernel, args...);
  if (err == cudaErrorNotSupported && chained) {
    (void)cudaGetLastError();
    disable_dependent_launch();
    config.numAttrs = count;
    err = cudaLaunchKernelEx(&config, kernel, args...);
  }
  return err;
}

template <typename... Params, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t stream, ClusterShape cluster, Args... args) {
  return launch_chained_impl(kernel, grid, block, smem, stream, &cluster, args...);
}

template <typename... Params, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t stream, Args... args) {
  return launch_chained_impl(kernel, grid, block, smem, stream, static_cast<const ClusterShape*>(nullptr),
                             args...);
}

#endif  // __CUDACC__
}  // namespace qf
