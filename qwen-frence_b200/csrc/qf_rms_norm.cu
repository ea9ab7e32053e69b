// RMSNorm and residual-add + RMSNorm over rows of a 16-bit activation matrix: the two
// steps either side of attention in a decode layer (the residual stream is summed once,
// stored rounded to the model dtype, and normalised from that rounded value).
// Restates fused_rms_norm / _residual_add_rms_norm_kernel of the reference
// (custom_kernels/fused_rms.py:8-49, :78-104):
//   summed     = T(residual + branch)                         (one rounding, as fp16/bf16 add)
//   rms        = sqrtf(sum(float(summed)^2) / N + epsilon)    (fp32)
//   normalized = T((float(weight) * float(summed)) / rms)
// One CTA per row.  A thread holds its 16-byte chunks of the row in registers between the
// sum of squares and the scaling, so a row of up to kHeld * 8 * blockDim elements (8192 at
// 256 threads) is read exactly once; longer rows re-read what the same thread stored.
// HBM bound for many long rows (2 reads + 2 writes of rows x N x 2 bytes), pure launch
// latency at decode batch sizes -- there the kernel chains onto its predecessor and loads
// its weights before the dependency wait.
#include "qf_common.cuh"

namespace qf {
namespace {

struct NormParams {
  const void* x;       // residual (or the only input)
  const void* branch;  // RESIDUAL only
  const void* weight;
  void* summed;        // RESIDUAL only
  void* normalized;
  int64_t x_stride, branch_stride, summed_stride, norm_stride;  // row strides, elements
  int hidden;
  float epsilon;
};

constexpr int kMaxNormThreads = 256;
constexpr int kHeld = 4;  // chunks per thread kept in registers

template <typename T>
__device__ __forceinline__ uint32_t add_pairs(uint32_t a, uint32_t b);
template <>
__device__ __forceinline__ uint32_t add_pairs<__half>(uint32_t a, uint32_t b) {
  __half2 r = __hadd2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
template <>
__device__ __forceinline__ uint32_t add_pairs<__nv_bfloat16>(uint32_t a, uint32_t b) {
  // fp32 add, one rounding to bf16: the exact sum of two bf16 values fits fp32's
  // significand whenever it matters for that rounding (24 >= 2 * 8 + 2)
  const float2 x = unpack2<__nv_bfloat16>(a), y = unpack2<__nv_bfloat16>(b);
  return pack2<__nv_bfloat16>(x.x + y.x, x.y + y.y);
}

// A chunk is VEC elements: one uint4 (8 elements) on the vector path, one element otherwise.
template <typename T, int VEC>
struct Chunk;
template <typename T>
struct Chunk<T, 8> {
  uint4 bits;
  __device__ __forceinline__ void load(const void* base, int64_t element) {
    bits = *reinterpret_cast<const uint4*>(static_cast<const T*>(base) + element);
  }
  __device__ __forceinline__ void store(void* base, int64_t element) const {
    *reinterpret_cast<uint4*>(static_cast<T*>(base) + element) = bits;
  }
  __device__ __forceinline__ void add(const Chunk& other) {
    bits.x = add_pairs<T>(bits.x, other.bits.x), bits.y = add_pairs<T>(bits.y, other.bits.y);
    bits.z = add_pairs<T>(bits.z, other.bits.z), bits.w = add_pairs<T>(bits.w, other.bits.w);
  }
  __device__ __forceinline__ float squares() const {
    const uint32_t words[4] = {bits.x, bits.y, bits.z, bits.w};
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = unpack2<T>(words[i]);
      total = fmaf(v.x, v.x, total);
      total = fmaf(v.y, v.y, total);
    }
    return total;
  }
  __device__ __forceinline__ Chunk scaled(const Chunk& weight, float rms) const {
    const uint32_t xs[4] = {bits.x, bits.y, bits.z, bits.w};
    const uint32_t ws[4] = {weight.bits.x, weight.bits.y, weight.bits.z, weight.bits.w};
    uint32_t out[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = unpack2<T>(xs[i]), w = unpack2<T>(ws[i]);
      out[i] = pack2<T>(__fdiv_rn(w.x * v.x, rms), __fdiv_rn(w.y * v.y, rms));
    }
    Chunk r;
    r.bits = make_uint4(out[0], out[1], out[2], out[3]);
    return r;
  }
};
template <typename T>
struct Chunk<T, 1> {
  T value;
  __device__ __forceinline__ void load(const void* base, int64_t element) {
    value = static_cast<const T*>(base)[element];
  }
  __device__ __forceinline__ void store(void* base, int64_t element) const {
    static_cast<T*>(base)[element] = value;
  }
  __device__ __forceinline__ void add(const Chunk& other) {
    value = from_float<T>(to_float(value) + to_float(other.value));
  }
  __device__ __forceinline__ float squares() const { return to_float(value) * to_float(value); }
  __device__ __forceinline__ Chunk scaled(const Chunk& weight, float rms) const {
    Chunk r;
    r.value = from_float<T>(__fdiv_rn(to_float(weight.value) * to_float(value), rms));
    return r;
  }
};

template <typename T, int VEC, bool RESIDUAL>
__global__ void __launch_bounds__(kMaxNormThreads, 5) rms_norm_kernel(NormParams p) {
  release_dependents();
  using Piece = Chunk<T, VEC>;
  __shared__ float warp_sums[kMaxNormThreads / 32];

  const int64_t row = blockIdx.x;
  const int chunks = p.hidden / VEC;
  const int threads = blockDim.x;

  // Weights belong to the model: no kernel of the step writes them, so they may be
  // fetched while the previous kernel is still running.
  // (Only the thread's first chunk: at decode widths that is all it has, and for wide
  // rows the registers are better spent on residency; the rest comes from L2 later.)
  Piece first_weight;
  if (threadIdx.x < chunks) first_weight.load(p.weight, static_cast<int64_t>(threadIdx.x) * VEC);
  dependency_wait();

  const T* x_row = static_cast<const T*>(p.x) + row * p.x_stride;
  const T* branch_row = RESIDUAL ? static_cast<const T*>(p.branch) + row * p.branch_stride : nullptr;
  T* summed_row = RESIDUAL ? static_cast<T*>(p.summed) + row * p.summed_stride : nullptr;
  T* norm_row = static_cast<T*>(p.normalized) + row * p.norm_stride;

  Piece held[kHeld];
  float squares = 0.f;
  auto fetch = [&](int c) {
    Piece value;
    value.load(x_row, c * VEC);
    if (RESIDUAL) {
      Piece other;
      other.load(branch_row, c * VEC);
      value.add(other);
      value.store(summed_row, c * VEC);
    }
    return value;
  };
#pragma unroll
  for (int i = 0; i < kHeld; ++i) {
    const int c = threadIdx.x + i * threads;
    if (c < chunks) {
      held[i] = fetch(c);
      squares += held[i].squares();
    }
  }
  for (int c = threadIdx.x + kHeld * threads; c < chunks; c += threads) squares += fetch(c).squares();

  // Block sum in a fixed order: lanes by butterfly, then the warps' sums one after another.
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) squares += __shfl_xor_sync(0xffffffffu, squares, offset);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = squares;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < (threads + 31) / 32; ++w) total += warp_sums[w];
  const float rms = __fsqrt_rn(__fdiv_rn(total, static_cast<float>(p.hidden)) + p.epsilon);

#pragma unroll
  for (int i = 0; i < kHeld; ++i) {
    const int c = threadIdx.x + i * threads;
    if (c < chunks) {
      Piece w = first_weight;
      if (i > 0) w.load(p.weight, c * VEC);
      held[i].scaled(w, rms).store(norm_row, c * VEC);
    }
  }
  for (int c = threadIdx.x + kHeld * threads; c < chunks; c += threads) {
    // the rounded sum this same thread stored above (or the input itself)
    Piece value, w;
    value.load(RESIDUAL ? summed_row : x_row, c * VEC);
    w.load(p.weight, c * VEC);
    value.scaled(w, rms).store(norm_row, c * VEC);
  }
}

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; }

template <typename T, bool RESIDUAL>
cudaError_t launch_norm(const NormParams& p, int64_t rows, bool vector, cudaStream_t stream) {
  const int chunks = vector ? p.hidden / 8 : p.hidden;
  int threads = ((chunks + 31) / 32) * 32;
  threads = threads < 32 ? 32 : (threads > kMaxNormThreads ? kMaxNormThreads : threads);
  const dim3 grid(static_cast<unsigned>(rows));
  if (vector) return launch_chained(rms_norm_kernel<T, 8, RESIDUAL>, grid, dim3(threads), 0, stream, p);
  return launch_chained(rms_norm_kernel<T, 1, RESIDUAL>, grid, dim3(threads), 0, stream, p);
}

int run_norm(const NormParams& p, int64_t rows, int32_t dtype, bool residual, void* stream) {
  QF_REQUIRE(dtype == QF_DTYPE_F16 || dtype == QF_DTYPE_BF16, "dtype must be fp16 or bf16");
  QF_REQUIRE(rows >= 0 && rows <= 0x7fffffff, "row count out of range");
  QF_REQUIRE(p.hidden > 0, "hidden size must be positive");
  if (rows == 0) return QF_OK;
  QF_REQUIRE(p.x && p.weight && p.normalized, "input, weight and output must not be null");
  QF_REQUIRE(!residual || (p.branch && p.summed), "branch and summed must not be null");
  bool vector = p.hidden % 8 == 0 && aligned16(p.x) && aligned16(p.weight) && aligned16(p.normalized) &&
                p.x_stride % 8 == 0 && p.norm_stride % 8 == 0;
  if (residual) {
    vector = vector && aligned16(p.branch) && aligned16(p.summed) && p.branch_stride % 8 == 0 &&
             p.summed_stride % 8 == 0;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err;
  if (dtype == QF_DTYPE_F16) {
    err = residual ? launch_norm<__half, true>(p, rows, vector, s) : launch_norm<__half, false>(p, rows, vector, s);
  } else {
    err = residual ? launch_norm<__nv_bfloat16, true>(p, rows, vector, s)
                   : launch_norm<__nv_bfloat16, false>(p, rows, vector, s);
  }
  QF_CUDA(err);
  return QF_OK;
}

}  // namespace
}  // namespace qf

extern "C" int qf_rms_norm(const void* x, int64_t x_row_stride, const void* weight, void* out,
                           int64_t out_row_stride, int64_t rows, int32_t hidden, int32_t dtype,
                           float epsilon, void* stream) {
  qf::NormParams p = {};
  p.x = x, p.weight = weight, p.normalized = out;
  p.x_stride = x_row_stride, p.norm_stride = out_row_stride;
  p.hidden = hidden, p.epsilon = epsilon;
  return qf::run_norm(p, rows, dtype, false, stream);
}

extern "C" int qf_residual_add_rms_norm(const void* residual, int64_t residual_row_stride,
                                        const void* branch, int64_t branch_row_stride,
                                        const void* weight, void* summed, int64_t summed_row_stride,
                                        void* normalized, int64_t normalized_row_stride, int64_t rows,
                                        int32_t hidden, int32_t dtype, float epsilon, void* stream) {
  qf::NormParams p = {};
  p.x = residual, p.branch = branch, p.weight = weight, p.summed = summed, p.normalized = normalized;
  p.x_stride = residual_row_stride, p.branch_stride = branch_row_stride;
  p.summed_stride = summed_row_stride, p.norm_stride = normalized_row_stride;
  p.hidden = hidden, p.epsilon = epsilon;
  return qf::run_norm(p, rows, dtype, true, stream);
}
