// GQA paged decode attention over block tables: split-K partial pass, combine,
// and the host entry points.
//
// The fast partial kernels (sm_100a, cp.async ring, Qwen geometry) live in
// qf_decode_partial.cuh (one CTA per partition, the reference's balanced
// partitions), qf_decode_stream.cuh (persistent CTAs that share the batch's
// pages equally, CUDA-core math; kept for comparison) and qf_decode_mma.cuh (the
// same scheduling with tensor-core math; the fused entry point's kernel for
// fp16 / bf16 and for FP8 pools).
//
// A stride-generic kernel covers every other layout and geometry the
// reference accepts (custom_kernels/paged_decode_grouped_splitk.py:228-334):
// arbitrary strides, other page sizes, head dims and group sizes.
#include <cmath>
#include <mutex>

#include "qf_common.cuh"
#include "qf_decode_partial.cuh"
#include "qf_decode_stream.cuh"
#include "qf_decode_mma.cuh"
#include "qf_rope_math.cuh"

namespace qf {
namespace {

int g_tuned_stages = 0;
int g_force_generic = 0;

// ---------------------------------------------------------------------------
// Stride-generic partial kernel: any strides, page size, head dim <= 256 and
// group size.  One CTA of four warps per (sequence, query head, split); warp w
// takes tokens w, w+4, ... of the partition; a lane holds dims lane + 32*i.
// Exact running maximum, natural-log units (expf), as the reference kernels.
// ---------------------------------------------------------------------------
struct GenericParams {
  const void* q;
  int64_t q_sb, q_sh, q_sd;
  const void* k_pool;
  const void* v_pool;
  int64_t k_sp, k_st, k_sh, k_sd;
  int64_t v_sp, v_st, v_sh, v_sd;
  const void* block_table;
  int64_t bt_sb, bt_sp;
  const void* seq_lens;
  int64_t lens_stride;
  const float* k_scale;
  const float* v_scale;
  float* partial_out;
  float* partial_max;
  float* partial_sum;
  void* out;
  int64_t o_sb, o_sh, o_sd;
  int64_t num_pages;
  int* status;
  int table_dtype, lens_dtype;
  int batch, q_heads, kv_heads, head_dim, page_size, split_k;
  int64_t max_tokens;  // table_width * page_size: a longer sequence length is cut to this
  float scale;
};

template <typename KV>
__device__ __forceinline__ float kv_to_float(KV x) {
  return to_float(x);
}
template <>
__device__ __forceinline__ float kv_to_float<uint8_t>(uint8_t x) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(x, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

constexpr int kGenericWarps = 4;
constexpr int kGenericMaxPerLane = 8;  // head_dim <= 256

template <typename T, typename KV>
__global__ void __launch_bounds__(kGenericWarps * 32)
    decode_partial_generic_kernel(const GenericParams p) {
  __shared__ float s_max[kGenericWarps];
  __shared__ float s_sum[kGenericWarps];
  __shared__ float s_acc[kGenericWarps][256];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x % p.split_k;
  const int head = (blockIdx.x / p.split_k) % p.q_heads;
  const int sequence = blockIdx.x / (p.split_k * p.q_heads);
  const int group = p.q_heads / p.kv_heads;
  const int kv_head = head / group;

  int64_t seq_len = load_index(p.seq_lens, p.lens_dtype, sequence * p.lens_stride);
  if (seq_len < 0) seq_len = 0;
  if (seq_len > p.max_tokens) seq_len = p.max_tokens;  // never read past the table row
  const int64_t total_pages = (seq_len + p.page_size - 1) / p.page_size;
  const int64_t start_page = split * total_pages / p.split_k;
  const int64_t end_page = (static_cast<int64_t>(split) + 1) * total_pages / p.split_k;
  const int64_t tok_begin = start_page * p.page_size;
  int64_t tok_end = end_page * p.page_size;
  if (tok_end > seq_len) tok_end = seq_len;

  float q[kGenericMaxPerLane], acc[kGenericMaxPerLane];
  const T* qrow = static_cast<const T*>(p.q) + sequence * p.q_sb + head * p.q_sh;
#pragma unroll
  for (int i = 0; i < kGenericMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    q[i] = d < p.head_dim ? to_float(qrow[d * p.q_sd]) : 0.f;
    acc[i] = 0.f;
  }
  float run_max = -INFINITY, run_sum = 0.f;

  for (int64_t tok = tok_begin + warp; tok < tok_end; tok += kGenericWarps) {
    const int64_t logical = tok / p.page_size;
    const int in_page = static_cast<int>(tok - logical * p.page_size);
    const int64_t page_id =
        load_index(p.block_table, p.table_dtype, sequence * p.bt_sb + logical * p.bt_sp);
    if (page_id < 0 || page_id >= p.num_pages) {
      if (lane == 0) atomicMax(p.status, kStatusBadPageId);
      continue;
    }
    const KV* krow = static_cast<const KV*>(p.k_pool) + page_id * p.k_sp + in_page * p.k_st +
                     kv_head * p.k_sh;
    const KV* vrow = static_cast<const KV*>(p.v_pool) + page_id * p.v_sp + in_page * p.v_st +
                     kv_head * p.v_sh;
    float k_mul = 1.f, v_mul = 1.f;
    if (p.k_scale != nullptr) {
      k_mul = p.k_scale[page_id * p.kv_heads + kv_head];
      v_mul = p.v_scale[page_id * p.kv_heads + kv_head];
    }
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kGenericMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < p.head_dim) dot += q[i] * (kv_to_float<KV>(krow[d * p.k_sd]) * k_mul);
    }
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    const float score = dot * p.scale;
    const float new_max = fmaxf(run_max, score);
    const float corr = run_max == -INFINITY ? 0.f : expf(run_max - new_max);
    const float prob = expf(score - new_max);
    run_sum = run_sum * corr + prob;
#pragma unroll
    for (int i = 0; i < kGenericMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < p.head_dim) acc[i] = acc[i] * corr + prob * (kv_to_float<KV>(vrow[d * p.v_sd]) * v_mul);
    }
    run_max = new_max;
  }

  if (lane == 0) s_max[warp] = run_max, s_sum[warp] = run_sum;
  __syncthreads();
  float cta_max = -INFINITY;
  for (int w = 0; w < kGenericWarps; ++w) cta_max = fmaxf(cta_max, s_max[w]);
  const float factor = run_max == -INFINITY ? 0.f : expf(run_max - cta_max);
#pragma unroll
  for (int i = 0; i < kGenericMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < p.head_dim) s_acc[warp][d] = acc[i] * factor;
  }
  __syncthreads();
  float cta_total = 0.f;
  for (int w = 0; w < kGenericWarps; ++w) {
    if (s_max[w] != -INFINITY) cta_total += s_sum[w] * expf(s_max[w] - cta_max);
  }
  const int64_t partial_row = (static_cast<int64_t>(sequence) * p.split_k + split) * p.q_heads + head;
  for (int d = threadIdx.x; d < p.head_dim; d += blockDim.x) {
    float value = 0.f;
    for (int w = 0; w < kGenericWarps; ++w) value += s_acc[w][d];
    if (p.partial_out != nullptr) p.partial_out[partial_row * p.head_dim + d] = value;
    if (p.out != nullptr) {
      static_cast<T*>(p.out)[sequence * p.o_sb + head * p.o_sh + d * p.o_sd] =
          from_float<T>(value / (cta_total > 0.f ? cta_total : 1.f));
    }
  }
  if (threadIdx.x == 0 && p.partial_max != nullptr) {
    p.partial_max[partial_row] = cta_max;
    p.partial_sum[partial_row] = cta_total;
  }
}

// ---------------------------------------------------------------------------
// Combine: one CTA per (sequence, query head); a thread per head dimension.
// Partitions whose sum is zero are skipped, so an empty first partition is
// harmless (custom_kernels/paged_decode_grouped_splitk.py:210-218).
// ---------------------------------------------------------------------------
struct ReduceParams {
  const float* po;
  const float* pm;
  const float* ps;
  int64_t po_sb, po_sk, po_sh, po_sd;
  int64_t pm_sb, pm_sk, pm_sh;
  void* out;
  int64_t o_sb, o_sh, o_sd;
  int q_heads, head_dim, split_k;
  // Only for partials written by the streamed kernel:
  const void* seq_lens;
  int64_t lens_stride;
  int lens_dtype;
  int64_t max_tokens;  // as in the partial pass: lengths are cut to the table's capacity
};

constexpr int kReduceChunk = 256;  // partitions whose weights are staged at a time

// STREAMED: the partials come from decode_stream_kernel.  A sequence then fills
// only its first few split slots, the slot after the last one holds sum = -1
// (unless all slots are used), and a sequence without tokens has no slot at all.
template <typename T, bool STREAMED>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const ReduceParams p) {
  __shared__ float s_weight[kReduceChunk];   // exp(offset_k - top), 0 for an empty partition
  __shared__ float s_red[8];
  __shared__ int s_first[8];
  __shared__ float s_top;
  const int sequence = blockIdx.x / p.q_heads;
  const int head = blockIdx.x - sequence * p.q_heads;
  const int tid = threadIdx.x;
  const float* pm = p.pm + sequence * p.pm_sb + head * p.pm_sh;
  const float* ps = p.ps + sequence * p.pm_sb + head * p.pm_sh;
  const float* po = p.po + sequence * p.po_sb + head * p.po_sh + tid * p.po_sd;

  int split_k = p.split_k;
  if (STREAMED) {
    if (min(load_index(p.seq_lens, p.lens_dtype, sequence * p.lens_stride), p.max_tokens) <= 0) {
      if (tid < p.head_dim) {
        static_cast<T*>(p.out)[sequence * p.o_sb + head * p.o_sh + tid * p.o_sd] = from_float<T>(0.f);
      }
      return;
    }
    int first = p.split_k;  // the first slot marked "no further pieces"
    for (int k = tid; k < p.split_k; k += blockDim.x) {
      if (ps[k * p.pm_sk] < 0.f) first = min(first, k);
    }
    for (int off = 16; off > 0; off >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, off));
    if ((tid & 31) == 0) s_first[tid >> 5] = first;
    __syncthreads();
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) split_k = min(split_k, s_first[w]);
  }

  // Pass 1: the largest offset among non-empty partitions; every thread takes a
  // strided share of the partitions, so the loads are issued together.
  float top = -INFINITY;
  for (int k = tid; k < split_k; k += blockDim.x) {
    if (ps[k * p.pm_sk] > 0.f) top = fmaxf(top, pm[k * p.pm_sk]);
  }
  for (int off = 16; off > 0; off >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, off));
  if ((tid & 31) == 0) s_red[tid >> 5] = top;
  __syncthreads();
  if (tid == 0) {
    float m = -INFINITY;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) m = fmaxf(m, s_red[w]);
    s_top = m;
  }
  __syncthreads();
  top = s_top;

  // Pass 2: weights of a chunk of partitions go to shared memory (one exp per
  // partition, computed in parallel), then every thread accumulates its head
  // dimension over the chunk with independent loads.
  float acc = 0.f, total = 0.f;
  for (int first = 0; first < split_k; first += kReduceChunk) {
    const int count = min(kReduceChunk, split_k - first);
    for (int k = tid; k < count; k += blockDim.x) {
      const float sum = ps[(first + k) * p.pm_sk];
      s_weight[k] = sum > 0.f ? expf(pm[(first + k) * p.pm_sk] - top) : 0.f;
    }
    __syncthreads();
    if (tid < p.head_dim) {
#pragma unroll 4
      for (int k = 0; k < count; ++k) {
        const float w = s_weight[k];
        if (w != 0.f) acc += po[(first + k) * p.po_sk] * w;
      }
    }
    if (tid == 0) {
      for (int k = 0; k < count; ++k) {
        const float w = s_weight[k];
        if (w != 0.f) total += ps[(first + k) * p.pm_sk] * w;
      }
      s_red[0] = total;
    }
    __syncthreads();
  }
  total = s_red[0];
  if (tid < p.head_dim) {
    const float result = acc / (total > 0.f ? total : 1.f);
    static_cast<T*>(p.out)[sequence * p.o_sb + head * p.o_sh + tid * p.o_sd] = from_float<T>(result);
  }
}

// Combine for split_k <= 32: two memory round trips and no block-wide barrier.
// Every warp reads the split_k statistics once (lane k holds slot k), derives the
// number of filled slots, the top offset, the weights and the total with warp
// shuffles, and then each thread sums its head dimension over the filled slots
// with independent loads.
constexpr int kSmallReduceSlots = 32;

template <typename T, bool STREAMED>
__global__ void __launch_bounds__(256) splitk_reduce_small_kernel(const ReduceParams p) {
  constexpr unsigned kFull = 0xffffffffu;
  release_dependents();
  dependency_wait();  // the partials come from the kernel before this one
  const int sequence = blockIdx.x / p.q_heads;
  const int head = blockIdx.x - sequence * p.q_heads;
  const int tid = threadIdx.x, lane = tid & 31;
  const float* pm = p.pm + sequence * p.pm_sb + head * p.pm_sh;
  const float* ps = p.ps + sequence * p.pm_sb + head * p.pm_sh;
  const float* po = p.po + sequence * p.po_sb + head * p.po_sh + tid * p.po_sd;
  T* out = static_cast<T*>(p.out) + sequence * p.o_sb + head * p.o_sh + tid * p.o_sd;

  // round trip 1: length (streamed partials only) and the statistics, all independent
  int64_t length = 1;
  if (STREAMED) length = min(load_index(p.seq_lens, p.lens_dtype, sequence * p.lens_stride), p.max_tokens);
  float sum = 0.f, offset = -INFINITY;
  if (lane < p.split_k) sum = ps[lane * p.pm_sk], offset = pm[lane * p.pm_sk];
  if (STREAMED && length <= 0) {
    if (tid < p.head_dim) *out = from_float<T>(0.f);  // no tokens: no slot was written
    return;
  }
  int filled = p.split_k;
  if (STREAMED) {
    // the slot after a sequence's last piece carries sum = -1
    const unsigned marks = __ballot_sync(kFull, lane < p.split_k && sum < 0.f);
    if (marks != 0) filled = __ffs(marks) - 1;
  }
  const bool used = lane < filled && sum > 0.f;
  float top = used ? offset : -INFINITY;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) top = fmaxf(top, __shfl_xor_sync(kFull, top, off));
  const float weight = used ? expf(offset - top) : 0.f;
  float total = sum * weight;  // 0 for unused slots (weight 0; sum finite or, unused, ignored)
  if (!used) total = 0.f;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) total += __shfl_xor_sync(kFull, total, off);

  // round trip 2: this thread's head dimension of every filled slot
  float acc = 0.f;
  if (tid < p.head_dim) {
#pragma unroll 4
    for (int k = 0; k < filled; ++k) {
      const float w = __shfl_sync(kFull, weight, k);
      if (w != 0.f) acc += po[k * p.po_sk] * w;
    }
    *out = from_float<T>(acc / (total > 0.f ? total : 1.f));
  }
}

// The same combine with one WARP per (sequence, head) row instead of one CTA: eight rows per
// CTA, a lane four dimensions (one 16-byte load per slot).  Same operations in the same order
// as the kernel above, so the same bits; needs head_dim 128, unit dimension strides and
// 16-byte aligned rows, and is then used for every batch: at 512 sequences the one-CTA-per-row
// grid is 6 144 CTAs and took 7.6 us per layer against 3.4 (1 024 sequences: 14 against 5),
// and at 64 sequences with ten filled slots per row a step of 28 layers went from 0.837 to
// 0.829 ms.

template <typename T, bool STREAMED>
__global__ void __launch_bounds__(256) splitk_reduce_rows_kernel(const ReduceParams p, int rows) {
  constexpr unsigned kFull = 0xffffffffu;
  release_dependents();
  dependency_wait();  // the partials come from the kernel before this one
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int sequence = row / p.q_heads;
  const int head = row - sequence * p.q_heads;
  const float* pm = p.pm + sequence * p.pm_sb + head * p.pm_sh;
  const float* ps = p.ps + sequence * p.pm_sb + head * p.pm_sh;
  const float* po = p.po + sequence * p.po_sb + head * p.po_sh + 4 * lane;
  T* out = static_cast<T*>(p.out) + sequence * p.o_sb + head * p.o_sh + 4 * lane;
  auto store = [&](float a, float b, float c, float d) {
    __align__(8) T packed[4] = {from_float<T>(a), from_float<T>(b), from_float<T>(c), from_float<T>(d)};
    *reinterpret_cast<uint2*>(out) = *reinterpret_cast<const uint2*>(packed);
  };

  int64_t length = 1;
  if (STREAMED) length = min(load_index(p.seq_lens, p.lens_dtype, sequence * p.lens_stride), p.max_tokens);
  float sum = 0.f, offset = -INFINITY;
  if (lane < p.split_k) sum = ps[lane * p.pm_sk], offset = pm[lane * p.pm_sk];
  if (STREAMED && length <= 0) {
    store(0.f, 0.f, 0.f, 0.f);  // no tokens: no slot was written
    return;
  }
  int filled = p.split_k;
  if (STREAMED) {
    const unsigned marks = __ballot_sync(kFull, lane < p.split_k && sum < 0.f);
    if (marks != 0) filled = __ffs(marks) - 1;
  }
  const bool used = lane < filled && sum > 0.f;
  float top = used ? offset : -INFINITY;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) top = fmaxf(top, __shfl_xor_sync(kFull, top, off));
  const float weight = used ? expf(offset - top) : 0.f;
  float total = sum * weight;
  if (!used) total = 0.f;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) total += __shfl_xor_sync(kFull, total, off);

  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
  for (int k = 0; k < filled; ++k) {
    const float w = __shfl_sync(kFull, weight, k);
    if (w != 0.f) {
      const float4 part = *reinterpret_cast<const float4*>(po + k * p.po_sk);
      acc.x += part.x * w, acc.y += part.y * w, acc.z += part.z * w, acc.w += part.w * w;
    }
  }
  const float divisor = total > 0.f ? total : 1.f;
  store(acc.x / divisor, acc.y / divisor, acc.z / divisor, acc.w / divisor);
}

// Combine for 32 < split_k <= 256 (few long sequences cut into many pieces): the small
// kernel's scheme with up to eight slots per lane.  Every warp reads all statistics in one
// trip (lane l holds slots l, l + 32, ...), finds the filled slots, the top offset, the
// weights and the total with shuffles; warp 0 leaves the weights in shared memory (the one
// block barrier), and each thread then sums its head dimension over the filled slots
// sixteen independent loads at a time.  Chained to the partial pass like the small kernel.
constexpr int kMediumReduceSlots = 256;
constexpr int kMediumSlotsPerLane = kMediumReduceSlots / 32;

template <typename T, bool STREAMED>
__global__ void __launch_bounds__(256) splitk_reduce_medium_kernel(const ReduceParams p) {
  constexpr unsigned kFull = 0xffffffffu;
  __shared__ float s_weight[kMediumReduceSlots];
  release_dependents();
  dependency_wait();  // the partials come from the kernel before this one
  const int sequence = blockIdx.x / p.q_heads;
  const int head = blockIdx.x - sequence * p.q_heads;
  const int tid = threadIdx.x, lane = tid & 31;
  const float* pm = p.pm + sequence * p.pm_sb + head * p.pm_sh;
  const float* ps = p.ps + sequence * p.pm_sb + head * p.pm_sh;
  const float* po = p.po + sequence * p.po_sb + head * p.po_sh + tid * p.po_sd;
  T* out = static_cast<T*>(p.out) + sequence * p.o_sb + head * p.o_sh + tid * p.o_sd;

  int64_t length = 1;
  if (STREAMED) length = min(load_index(p.seq_lens, p.lens_dtype, sequence * p.lens_stride), p.max_tokens);
  float sum[kMediumSlotsPerLane], offset[kMediumSlotsPerLane];
#pragma unroll
  for (int j = 0; j < kMediumSlotsPerLane; ++j) {
    const int k = lane + 32 * j;
    sum[j] = 0.f, offset[j] = -INFINITY;
    if (k < p.split_k) sum[j] = ps[k * p.pm_sk], offset[j] = pm[k * p.pm_sk];
  }
  if (STREAMED && length <= 0) {
    if (tid < p.head_dim) *out = from_float<T>(0.f);  // no tokens: no slot was written
    return;
  }
  int filled = p.split_k;
  if (STREAMED) {
    // the slot after a sequence's last piece carries sum = -1
#pragma unroll
    for (int j = kMediumSlotsPerLane - 1; j >= 0; --j) {
      const unsigned marks = __ballot_sync(kFull, lane + 32 * j < p.split_k && sum[j] < 0.f);
      if (marks != 0) filled = 32 * j + __ffs(marks) - 1;
    }
  }
  float top = -INFINITY;
#pragma unroll
  for (int j = 0; j < kMediumSlotsPerLane; ++j) {
    if (lane + 32 * j < filled && sum[j] > 0.f) top = fmaxf(top, offset[j]);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) top = fmaxf(top, __shfl_xor_sync(kFull, top, off));
  float total = 0.f;
#pragma unroll
  for (int j = 0; j < kMediumSlotsPerLane; ++j) {
    const bool used = lane + 32 * j < filled && sum[j] > 0.f;
    const float weight = used ? expf(offset[j] - top) : 0.f;
    if (used) total += sum[j] * weight;
    if (tid < 32) s_weight[lane + 32 * j] = weight;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) total += __shfl_xor_sync(kFull, total, off);
  __syncthreads();

  if (tid < p.head_dim) {
    float acc = 0.f;
    for (int first = 0; first < filled; first += 16) {
      float part[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int k = first + i;
        part[i] = (k < filled && s_weight[k] != 0.f) ? po[k * p.po_sk] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int k = first + i;
        if (k < filled && s_weight[k] != 0.f) acc += part[i] * s_weight[k];
      }
    }
    *out = from_float<T>(acc / (total > 0.f ? total : 1.f));
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
int* status_word_for_current_device() {
  static std::mutex mutex;
  static int* cache[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mutex);
  if (cache[device] == nullptr) cache[device] = device_status_word();
  return cache[device];
}

size_t fast_smem_bytes(bool fp8) {
  const size_t ring = static_cast<size_t>(kSlots) * (fp8 ? 8192 : 16384);
  const size_t merge = kMergeFloats * sizeof(float);
  return ring > merge ? ring : merge;
}

template <typename T, bool FP8, bool PROFILE>
int launch_fast(const FastParams& p, cudaStream_t stream) {
  auto kernel = decode_partial_kernel<T, FP8, PROFILE>;
  const size_t smem = fast_smem_bytes(FP8);
  QF_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem)));
  const int64_t blocks = static_cast<int64_t>(p.batch) * p.kv_heads * p.split_k;
  kernel<<<static_cast<unsigned>(blocks), kFastThreads, smem, stream>>>(p);
  QF_CUDA(cudaGetLastError());
  return QF_OK;
}

// Resident CTAs of the streamed kernel on the current device: two per SM.
int stream_ctas_on_current_device() {
  static std::mutex mutex;
  static int cache[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  std::lock_guard<std::mutex> lock(mutex);
  if (cache[device] == 0) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    cache[device] = sms * QF_MIN_CTAS;
  }
  return cache[device];
}

size_t stream_smem_bytes(bool fp8) {
  return static_cast<size_t>(kSlots) * (fp8 ? 8192 : 16384) + kMergeFloats * sizeof(float);
}

template <typename T, bool FP8>
int launch_stream(const FastParams& p, cudaStream_t stream) {
  auto kernel = decode_stream_kernel<T, FP8>;
  const size_t smem = stream_smem_bytes(FP8);
  QF_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem)));
  const int resident = stream_ctas_on_current_device();
  QF_REQUIRE(resident >= p.kv_heads, "could not size the streamed kernel for this device");
  StreamParams sp{p, resident / p.kv_heads, 0};
  kernel<<<static_cast<unsigned>(sp.ctas_per_head * p.kv_heads), kFastThreads, smem, stream>>>(sp);
  QF_CUDA(cudaGetLastError());
  return QF_OK;
}

// Resident CTAs of the tensor-core kernel on the current device.
int mma_ctas_on_current_device(bool fp8) {
  const int sms = stream_ctas_on_current_device() / QF_MIN_CTAS;
  return sms * (fp8 ? RingShape<true>::kCtasPerSm : RingShape<false>::kCtasPerSm);
}

size_t mma_smem_bytes(bool fp8) {
  const size_t ring = fp8 ? RingShape<true>::kWarpBytes : RingShape<false>::kWarpBytes;
  return static_cast<size_t>(kMmaWarps) * ring + kMmaMergeFloats * sizeof(float);
}

// One CTA per SM for 16-bit pools (its rings take most of the shared memory), two for FP8.
template <typename T, bool FP8, bool PROFILE, bool ROPE = false, bool SOLO = false>
int launch_mma(const FastParams& p, cudaStream_t stream, const RopeInputs& rope = RopeInputs{}) {
  auto kernel = decode_mma_kernel<T, FP8, PROFILE, ROPE, SOLO>;
  const size_t smem = mma_smem_bytes(FP8);
  QF_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem)));
  const int resident = mma_ctas_on_current_device(FP8);
  QF_REQUIRE(resident >= p.kv_heads, "could not size the tensor-core kernel for this device");
  // The fused step is a decode step by contract: one new token per sequence, stored by this
  // very kernel, and every older K / V row written before the step began.  Its kernel may
  // therefore request tiles of the older pages before its dependency wait.  The plain
  // attention call makes no such promise about the kernel in front of it.
  StreamParams sp{p, resident / p.kv_heads, ROPE ? 1 : 0};
  QF_CUDA(launch_chained(kernel, dim3(static_cast<unsigned>(sp.ctas_per_head * p.kv_heads)),
                         dim3(kFastThreads), smem, stream, sp, rope));
  QF_CUDA(cudaGetLastError());
  return QF_OK;
}

template <typename T, bool PROFILE>
int launch_mma_for_pools(const FastParams& p, bool fp8, cudaStream_t stream) {
  return fp8 ? launch_mma<T, true, PROFILE>(p, stream) : launch_mma<T, false, PROFILE>(p, stream);
}
// the variant in which every warp keeps its pieces to itself
template <typename T>
int launch_mma_solo(const FastParams& p, bool fp8, cudaStream_t stream) {
  return fp8 ? launch_mma<T, true, false, false, true>(p, stream) : launch_mma<T, false, false, false, true>(p, stream);
}

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; }

// (cos, sin) of position * inv_freq[f] for every position and rotary frequency: the very
// expressions of the RoPE / KV-write kernel, so a kernel that reads the table rotates to the
// same bits as that kernel.
__global__ void rope_table_kernel(float2* table, int positions, const __grid_constant__ InvFreqTable freq) {
  const int64_t entry = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (entry >= static_cast<int64_t>(positions) * (QF_HEAD_DIM / 2)) return;
  const int position = static_cast<int>(entry / (QF_HEAD_DIM / 2)), f = static_cast<int>(entry % (QF_HEAD_DIM / 2));
  const float angle = __fmul_rn(static_cast<float>(position), freq.v[f]);
  table[entry] = make_float2(cosf(angle), sinf(angle));
}

int validate(const qf_decode_attention_args* a, bool need_out) {
  QF_REQUIRE(a != nullptr, "args must not be null");
  QF_REQUIRE(a->batch >= 0 && a->q_heads >= 1 && a->kv_heads >= 1, "invalid batch or head counts");
  QF_REQUIRE(a->q_heads % a->kv_heads == 0, "query heads must be divisible by KV heads");
  QF_REQUIRE(a->head_dim >= 1 && a->head_dim <= 256 && (a->head_dim & (a->head_dim - 1)) == 0 &&
                 a->page_size >= 1 && (a->page_size & (a->page_size - 1)) == 0,
             "head dimension and page size must be powers of two (head_dim <= 256)");
  QF_REQUIRE(a->dtype == QF_DTYPE_F16 || a->dtype == QF_DTYPE_BF16,
             "Q/K/V must be float16 or bfloat16");
  QF_REQUIRE(a->table_dtype == QF_INDEX_I32 || a->table_dtype == QF_INDEX_I64,
             "page table must use an integer dtype");
  QF_REQUIRE(a->lens_dtype == QF_INDEX_I32 || a->lens_dtype == QF_INDEX_I64,
             "sequence lengths must use an integer dtype");
  QF_REQUIRE(a->split_k >= 1 && a->split_k <= 65535, "split_k must be in [1, 65535]");
  QF_REQUIRE(a->num_pages >= 0 && a->num_pages < (1LL << 31), "num_pages out of range");
  if (a->batch == 0) return QF_OK;
  QF_REQUIRE(a->q && a->seq_lens, "q and seq_lens must not be null");
  QF_REQUIRE(a->table_width == 0 || a->block_table, "block_table must not be null");
  QF_REQUIRE(a->num_pages == 0 || (a->k_pool && a->v_pool), "K/V pools must not be null");
  if (a->kv_fp8) QF_REQUIRE(a->k_scale && a->v_scale, "fp8 pools need k_scale and v_scale");
  if (need_out) QF_REQUIRE(a->out != nullptr, "out must not be null");
  if (a->split_k > 1 || a->out == nullptr) {
    QF_REQUIRE(a->partial_out && a->partial_max && a->partial_sum,
               "partial buffers must not be null");
  }
  const int64_t blocks = static_cast<int64_t>(a->batch) * a->q_heads * a->split_k;
  QF_REQUIRE(blocks < (1LL << 31), "batch * heads * split_k exceeds the grid limit");
  return QF_OK;
}

bool fast_path_ok(const qf_decode_attention_args* a) {
  if (g_force_generic == 1) return false;
  if (a->head_dim != QF_HEAD_DIM || a->page_size != QF_PAGE_SIZE) return false;
  if (a->q_heads != a->kv_heads * QF_GQA_GROUP) return false;
  if (a->num_pages < 1 || a->kv_heads > 65535) return false;
  if (a->q_stride_d != 1 || !aligned16(a->q) || (a->q_stride_b & 7) || (a->q_stride_h & 7)) return false;
  if (a->k_stride_d != 1 || a->v_stride_d != 1) return false;
  if (!aligned16(a->k_pool) || !aligned16(a->v_pool)) return false;
  const int64_t unit = a->kv_fp8 ? 16 : 8;  // elements per 16 bytes
  const int64_t strides[6] = {a->k_stride_page, a->k_stride_tok, a->k_stride_head,
                              a->v_stride_page, a->v_stride_tok, a->v_stride_head};
  for (int64_t s : strides) {
    if (s <= 0 || (s % unit) != 0) return false;
  }
  return true;
}

FastParams fast_params(const qf_decode_attention_args* a, void* out, long long* cycles, int* status) {
  FastParams p{};
  p.q = a->q, p.q_sb = a->q_stride_b, p.q_sh = a->q_stride_h;
  const int64_t elem = a->kv_fp8 ? 1 : 2;
  p.k_pool = static_cast<const unsigned char*>(a->k_pool);
  p.v_pool = static_cast<const unsigned char*>(a->v_pool);
  p.k_page_bytes = a->k_stride_page * elem, p.k_tok_bytes = a->k_stride_tok * elem;
  p.k_head_bytes = a->k_stride_head * elem;
  p.v_page_bytes = a->v_stride_page * elem, p.v_tok_bytes = a->v_stride_tok * elem;
  p.v_head_bytes = a->v_stride_head * elem;
  p.block_table = a->block_table, p.bt_sb = a->table_stride_b, p.bt_sp = a->table_stride_p;
  p.seq_lens = a->seq_lens, p.lens_stride = a->lens_stride;
  p.k_scale = a->k_scale, p.v_scale = a->v_scale;
  p.partial_out = a->partial_out, p.partial_max = a->partial_max, p.partial_sum = a->partial_sum;
  p.out = out, p.o_sb = a->o_stride_b, p.o_sh = a->o_stride_h, p.o_sd = a->o_stride_d;
  p.num_pages = a->num_pages;
  p.cycles = cycles;
  p.status = status;
  p.table_dtype = a->table_dtype, p.lens_dtype = a->lens_dtype;
  p.batch = a->batch, p.q_heads = a->q_heads, p.kv_heads = a->kv_heads, p.split_k = a->split_k;
  const int64_t capacity = a->table_width * a->page_size;
  p.max_tokens = static_cast<int>(capacity > kMaxStreamLen ? kMaxStreamLen : capacity);
  p.scale_log2 = a->scale * kLog2e;
  return p;
}

// The tensor-core persistent kernel serves the fused attention entry point whenever
// the layout is the fast one, split_k >= 2, the batch's prefix fits in its shared
// memory, both pools share their strides and the partial buffer is 16-byte aligned.  A
// sequence may be cut into at most split_k pieces, so a CTA's share is at least
// longest / (split_k - 1) units and a batch of few sequences with few slots leaves
// resident CTAs without work; the per-partition kernel has the same limit (split_k CTAs
// per sequence and head) and half the speed per page, so the persistent one is used
// regardless (measured from batch 1 x 4096 tokens, split_k 22: 9.3 us against 12.3 us,
// upwards).  Pools whose K and V strides differ (a view of a larger allocation on one
// side) and partial buffers carved out at a 4-byte offset take the CUDA-core persistent
// kernel, which keeps separate strides and stores partials element by element.
enum class FusedKernel { kPartitioned, kStreamed, kTensorCore, kTensorCoreSolo };

FusedKernel choose_fused_kernel(const qf_decode_attention_args* a) {
  const int mode = g_force_generic;  // 0 automatic, 3 / 4 / 5 force a persistent kernel (tests)
  if ((mode != 0 && mode != 3 && mode != 4 && mode != 5) || !fast_path_ok(a) || a->split_k < 2) {
    return FusedKernel::kPartitioned;
  }
  if (a->batch > kMaxStreamBatch || a->kv_heads > 64) return FusedKernel::kPartitioned;
  const int resident = stream_ctas_on_current_device();  // two per SM
  if (resident / QF_MIN_CTAS < a->kv_heads) return FusedKernel::kPartitioned;
  // the tensor-core kernel uses one set of row offsets for both pools
  const bool same_strides = a->k_stride_page == a->v_stride_page && a->k_stride_tok == a->v_stride_tok &&
                            a->k_stride_head == a->v_stride_head &&
                            a->k_stride_tok * (a->kv_fp8 ? 1 : 2) * QF_PAGE_SIZE < (1LL << 31);
  // ... and stores a piece's partial rows as 16-byte vectors
  const bool tensor_core = mode != 3 && same_strides && aligned16(a->partial_out);
  if ((mode == 4 || mode == 5) && !tensor_core) return FusedKernel::kPartitioned;
  // The solo variant (every warp streams a block of consecutive pages on its own; what a CTA's
  // warps hold of one sequence is merged once, at the CTA's end) is the tensor-core kernel of
  // every call; the variant whose warps interleave over the pages and merge piece by piece
  // remains as the instrumented kernel and behind mode 4.  Measured step times, solo against
  // interleaved, same split counts: 64 x U[128, 4096] tokens 0.782 against 0.824 ms, 256 x
  // log-uniform [64, 8192] 2.120 against 2.346, 4 sequences of up to 32 768 tokens 0.530 against
  // 0.531, FP8 128 x 2 048 1.022 against 1.032, 8 x 513 tokens (one layer) 14.6 against 14.5 us;
  // 512 x 100 tokens: partial pass 11.8 against 24.7 us.
  if (tensor_core && mode != 4) return FusedKernel::kTensorCoreSolo;
  return tensor_core ? FusedKernel::kTensorCore : FusedKernel::kStreamed;
}

int launch_persistent_partial(const qf_decode_attention_args* a, FusedKernel kind, cudaStream_t stream,
                              long long* timeline = nullptr) {
  int* status = status_word_for_current_device();
  QF_REQUIRE(status != nullptr, "could not resolve the device status word");
  const FastParams p = fast_params(a, nullptr, timeline, status);
  if (timeline != nullptr) {
    QF_REQUIRE(kind == FusedKernel::kTensorCore || kind == FusedKernel::kTensorCoreSolo,
               "only the tensor-core kernel has a timeline variant");
    if (kind == FusedKernel::kTensorCoreSolo) {
      QF_REQUIRE(!a->kv_fp8, "the instrumented solo variant is built for 16-bit pools");
      return a->dtype == QF_DTYPE_F16 ? launch_mma<__half, false, true, false, true>(p, stream)
                                      : launch_mma<__nv_bfloat16, false, true, false, true>(p, stream);
    }
    return a->dtype == QF_DTYPE_F16 ? launch_mma_for_pools<__half, true>(p, a->kv_fp8 != 0, stream)
                                    : launch_mma_for_pools<__nv_bfloat16, true>(p, a->kv_fp8 != 0, stream);
  }
  if (kind == FusedKernel::kTensorCoreSolo) {
    return a->dtype == QF_DTYPE_F16 ? launch_mma_solo<__half>(p, a->kv_fp8 != 0, stream)
                                    : launch_mma_solo<__nv_bfloat16>(p, a->kv_fp8 != 0, stream);
  }
  if (kind == FusedKernel::kTensorCore) {
    return a->dtype == QF_DTYPE_F16 ? launch_mma_for_pools<__half, false>(p, a->kv_fp8 != 0, stream)
                                    : launch_mma_for_pools<__nv_bfloat16, false>(p, a->kv_fp8 != 0, stream);
  }
  if (a->kv_fp8) {
    return a->dtype == QF_DTYPE_F16 ? launch_stream<__half, true>(p, stream)
                                    : launch_stream<__nv_bfloat16, true>(p, stream);
  }
  return a->dtype == QF_DTYPE_F16 ? launch_stream<__half, false>(p, stream)
                                  : launch_stream<__nv_bfloat16, false>(p, stream);
}

template <bool PROFILE>
int launch_partial(const qf_decode_attention_args* a, bool direct_out, long long* cycles,
                   cudaStream_t stream) {
  if (a->batch == 0) return QF_OK;
  int* status = status_word_for_current_device();
  QF_REQUIRE(status != nullptr, "could not resolve the device status word");
  void* out = direct_out ? a->out : nullptr;

  if (fast_path_ok(a)) {
    const FastParams p = fast_params(a, out, cycles, status);
    if (a->kv_fp8) {
      return a->dtype == QF_DTYPE_F16
                 ? launch_fast<__half, true, PROFILE>(p, stream)
                 : launch_fast<__nv_bfloat16, true, PROFILE>(p, stream);
    }
    return a->dtype == QF_DTYPE_F16
               ? launch_fast<__half, false, PROFILE>(p, stream)
               : launch_fast<__nv_bfloat16, false, PROFILE>(p, stream);
  }

  QF_REQUIRE(!PROFILE, "stage profiling requires the native grouped-decode layout");
  GenericParams g{};
  g.q = a->q, g.q_sb = a->q_stride_b, g.q_sh = a->q_stride_h, g.q_sd = a->q_stride_d;
  g.k_pool = a->k_pool, g.v_pool = a->v_pool;
  g.k_sp = a->k_stride_page, g.k_st = a->k_stride_tok, g.k_sh = a->k_stride_head, g.k_sd = a->k_stride_d;
  g.v_sp = a->v_stride_page, g.v_st = a->v_stride_tok, g.v_sh = a->v_stride_head, g.v_sd = a->v_stride_d;
  g.block_table = a->block_table, g.bt_sb = a->table_stride_b, g.bt_sp = a->table_stride_p;
  g.seq_lens = a->seq_lens, g.lens_stride = a->lens_stride;
  g.k_scale = a->kv_fp8 ? a->k_scale : nullptr, g.v_scale = a->kv_fp8 ? a->v_scale : nullptr;
  g.partial_out = a->partial_out, g.partial_max = a->partial_max, g.partial_sum = a->partial_sum;
  g.out = out, g.o_sb = a->o_stride_b, g.o_sh = a->o_stride_h, g.o_sd = a->o_stride_d;
  g.num_pages = a->num_pages;
  g.status = status;
  g.table_dtype = a->table_dtype, g.lens_dtype = a->lens_dtype;
  g.batch = a->batch, g.q_heads = a->q_heads, g.kv_heads = a->kv_heads, g.head_dim = a->head_dim;
  g.page_size = a->page_size, g.split_k = a->split_k;
  g.max_tokens = a->table_width * a->page_size;
  g.scale = a->scale;
  const unsigned blocks = static_cast<unsigned>(static_cast<int64_t>(a->batch) * a->q_heads * a->split_k);
  const int threads = kGenericWarps * 32;
  if (a->kv_fp8) {
    if (a->dtype == QF_DTYPE_F16)
      decode_partial_generic_kernel<__half, uint8_t><<<blocks, threads, 0, stream>>>(g);
    else
      decode_partial_generic_kernel<__nv_bfloat16, uint8_t><<<blocks, threads, 0, stream>>>(g);
  } else if (a->dtype == QF_DTYPE_F16) {
    decode_partial_generic_kernel<__half, __half><<<blocks, threads, 0, stream>>>(g);
  } else {
    decode_partial_generic_kernel<__nv_bfloat16, __nv_bfloat16><<<blocks, threads, 0, stream>>>(g);
  }
  QF_CUDA(cudaGetLastError());
  return QF_OK;
}

template <typename T>
void launch_reduce_typed(const ReduceParams& r, unsigned blocks, int threads, bool streamed,
                         cudaStream_t stream) {
  // head_dim is a multiple of 32 on this path, so whole warps take part in the shuffles
  const bool small = r.split_k <= kSmallReduceSlots && (r.head_dim & 31) == 0;
  const bool medium = !small && r.split_k <= kMediumReduceSlots && (r.head_dim & 31) == 0;
  const bool vector_rows = r.head_dim == 128 && r.po_sd == 1 && r.o_sd == 1 && aligned16(r.po) &&
                           ((r.po_sb | r.po_sk | r.po_sh | r.o_sb | r.o_sh) & 3) == 0 &&
                           (reinterpret_cast<uintptr_t>(r.out) & 7) == 0;
  if (small && vector_rows) {
    const int rows = static_cast<int>(blocks);
    const dim3 grid((blocks + 7) / 8), cta(256);
    if (streamed) {
      (void)launch_chained(splitk_reduce_rows_kernel<T, true>, grid, cta, 0, stream, r, rows);
    } else {
      (void)launch_chained(splitk_reduce_rows_kernel<T, false>, grid, cta, 0, stream, r, rows);
    }
  } else if (medium && streamed) {
    (void)launch_chained(splitk_reduce_medium_kernel<T, true>, dim3(blocks), dim3(threads), 0, stream, r);
  } else if (medium) {
    (void)launch_chained(splitk_reduce_medium_kernel<T, false>, dim3(blocks), dim3(threads), 0, stream, r);
  } else if (small && streamed) {
    (void)launch_chained(splitk_reduce_small_kernel<T, true>, dim3(blocks), dim3(threads), 0, stream, r);
  } else if (small) {
    (void)launch_chained(splitk_reduce_small_kernel<T, false>, dim3(blocks), dim3(threads), 0, stream, r);
  } else if (streamed) {
    splitk_reduce_kernel<T, true><<<blocks, threads, 0, stream>>>(r);
  } else {
    splitk_reduce_kernel<T, false><<<blocks, threads, 0, stream>>>(r);
  }
}

int launch_reduce(const ReduceParams& r, int batch, int dtype, bool streamed, cudaStream_t stream) {
  if (batch == 0) return QF_OK;
  const unsigned blocks = static_cast<unsigned>(static_cast<int64_t>(batch) * r.q_heads);
  const int threads = ((r.head_dim + 31) / 32) * 32;
  if (dtype == QF_DTYPE_F16) {
    launch_reduce_typed<__half>(r, blocks, threads, streamed, stream);
  } else {
    launch_reduce_typed<__nv_bfloat16>(r, blocks, threads, streamed, stream);
  }
  QF_CUDA(cudaGetLastError());
  return QF_OK;
}

}  // namespace
}  // namespace qf

extern "C" {

int qf_grouped_gqa_splitk_partial_out(const qf_decode_attention_args* args, void* stream) {
  const int rc = qf::validate(args, false);
  if (rc != QF_OK) return rc;
  const bool direct = args->split_k == 1 && args->out != nullptr;
  return qf::launch_partial<false>(args, direct, nullptr, static_cast<cudaStream_t>(stream));
}

int qf_grouped_gqa_splitk_profile_out(const qf_decode_attention_args* args, int64_t* cycles,
                                      void* stream) {
  const int rc = qf::validate(args, false);
  if (rc != QF_OK) return rc;
  QF_REQUIRE(cycles != nullptr, "cycles must not be null");
  const bool direct = args->split_k == 1 && args->out != nullptr;
  return qf::launch_partial<true>(args, direct, reinterpret_cast<long long*>(cycles),
                                  static_cast<cudaStream_t>(stream));
}

int qf_splitk_reduce(const float* partial_out, const float* partial_max, const float* partial_sum,
                     int64_t po_stride_b, int64_t po_stride_k, int64_t po_stride_h,
                     int64_t po_stride_d, int64_t pm_stride_b, int64_t pm_stride_k,
                     int64_t pm_stride_h, void* out, int64_t o_stride_b, int64_t o_stride_h,
                     int64_t o_stride_d, int32_t batch, int32_t q_heads, int32_t head_dim,
                     int32_t split_k, int32_t dtype, void* stream) {
  QF_REQUIRE(batch >= 0 && q_heads >= 1 && split_k >= 1, "invalid batch, head or split count");
  QF_REQUIRE(head_dim >= 1 && head_dim <= 256, "head_dim must be in [1, 256]");
  QF_REQUIRE(dtype == QF_DTYPE_F16 || dtype == QF_DTYPE_BF16, "out must be float16 or bfloat16");
  if (batch == 0) return QF_OK;
  QF_REQUIRE(partial_out && partial_max && partial_sum && out, "buffers must not be null");
  qf::ReduceParams r{};
  r.po = partial_out, r.pm = partial_max, r.ps = partial_sum;
  r.po_sb = po_stride_b, r.po_sk = po_stride_k, r.po_sh = po_stride_h, r.po_sd = po_stride_d;
  r.pm_sb = pm_stride_b, r.pm_sk = pm_stride_k, r.pm_sh = pm_stride_h;
  r.out = out, r.o_sb = o_stride_b, r.o_sh = o_stride_h, r.o_sd = o_stride_d;
  r.q_heads = q_heads, r.head_dim = head_dim, r.split_k = split_k;
  return qf::launch_reduce(r, batch, dtype, false, static_cast<cudaStream_t>(stream));
}

int qf_grouped_splitk_decode_attention_stages(const qf_decode_attention_args* args, int32_t stages,
                                              void* stream) {
  int rc = qf::validate(args, true);
  if (rc != QF_OK) return rc;
  QF_REQUIRE(stages >= 1 && stages <= (QF_STAGE_PARTIAL | QF_STAGE_COMBINE),
             "stages must be QF_STAGE_PARTIAL, QF_STAGE_COMBINE or both");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (args->split_k == 1) {
    return (stages & QF_STAGE_PARTIAL) ? qf::launch_partial<false>(args, true, nullptr, s) : QF_OK;
  }
  if (args->batch == 0) return QF_OK;
  const qf::FusedKernel kind = qf::choose_fused_kernel(args);
  const bool streamed = kind != qf::FusedKernel::kPartitioned;
  if (stages & QF_STAGE_PARTIAL) {
    rc = streamed ? qf::launch_persistent_partial(args, kind, s)
                  : qf::launch_partial<false>(args, false, nullptr, s);
    if (rc != QF_OK) return rc;
  }
  if (!(stages & QF_STAGE_COMBINE)) return QF_OK;
  qf::ReduceParams r{};
  r.po = args->partial_out, r.pm = args->partial_max, r.ps = args->partial_sum;
  const int64_t hq = args->q_heads, d = args->head_dim, k = args->split_k;
  r.po_sb = k * hq * d, r.po_sk = hq * d, r.po_sh = d, r.po_sd = 1;
  r.pm_sb = k * hq, r.pm_sk = hq, r.pm_sh = 1;
  r.out = args->out, r.o_sb = args->o_stride_b, r.o_sh = args->o_stride_h, r.o_sd = args->o_stride_d;
  r.q_heads = args->q_heads, r.head_dim = args->head_dim, r.split_k = args->split_k;
  r.seq_lens = args->seq_lens, r.lens_stride = args->lens_stride, r.lens_dtype = args->lens_dtype;
  r.max_tokens = args->table_width * args->page_size;
  return qf::launch_reduce(r, args->batch, args->dtype, streamed, s);
}

int qf_grouped_splitk_decode_attention_plan(const qf_decode_attention_args* args, int32_t* kernel,
                                            int32_t* ctas_per_head) {
  const int rc = qf::validate(args, false);
  if (rc != QF_OK) return rc;
  QF_REQUIRE(kernel != nullptr && ctas_per_head != nullptr, "outputs must not be null");
  *kernel = QF_KERNEL_PARTITIONED, *ctas_per_head = 0;
  if (args->split_k == 1 || args->batch == 0) return QF_OK;
  const qf::FusedKernel kind = qf::choose_fused_kernel(args);
  if (kind == qf::FusedKernel::kPartitioned) return QF_OK;
  const int resident = qf::stream_ctas_on_current_device();
  const bool mma = kind == qf::FusedKernel::kTensorCore || kind == qf::FusedKernel::kTensorCoreSolo;
  *kernel = mma ? QF_KERNEL_PERSISTENT_MMA : QF_KERNEL_PERSISTENT;
  if (kind == qf::FusedKernel::kTensorCoreSolo) *kernel = QF_KERNEL_PERSISTENT_MMA_SOLO;
  *ctas_per_head = (mma ? qf::mma_ctas_on_current_device(args->kv_fp8 != 0) : resident) / args->kv_heads;
  return QF_OK;
}

int qf_grouped_splitk_persistent_timeline(const qf_decode_attention_args* args, int64_t* timeline,
                                          void* stream) {
  const int rc = qf::validate(args, true);
  if (rc != QF_OK) return rc;
  QF_REQUIRE(timeline != nullptr, "timeline must not be null");
  QF_REQUIRE(args->split_k >= 2 && args->batch >= 1, "the persistent kernels need split_k >= 2 and a batch");
  qf::FusedKernel kind = qf::choose_fused_kernel(args);
  // FP8 pools: the instrumented kernel is the variant whose warps interleave over the pages
  if (kind == qf::FusedKernel::kTensorCoreSolo && args->kv_fp8) kind = qf::FusedKernel::kTensorCore;
  QF_REQUIRE(kind == qf::FusedKernel::kTensorCore || kind == qf::FusedKernel::kTensorCoreSolo,
             "these arguments do not select the tensor-core persistent kernel");
  return qf::launch_persistent_partial(args, kind, static_cast<cudaStream_t>(stream),
                                       reinterpret_cast<long long*>(timeline));
}

int qf_build_rope_table(float* table, int32_t positions, double base, void* stream) {
  QF_REQUIRE(positions >= 0, "the number of positions must not be negative");
  if (positions == 0) return QF_OK;
  QF_REQUIRE(table != nullptr && qf::aligned16(table), "the table must be a 16-byte aligned device buffer");
  const qf::InvFreqTable freq = qf::make_inv_freq(base, QF_HEAD_DIM / 2);
  const int64_t entries = static_cast<int64_t>(positions) * (QF_HEAD_DIM / 2);
  const unsigned blocks = static_cast<unsigned>((entries + 255) / 256);
  qf::rope_table_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<float2*>(table),
                                                                             positions, freq);
  QF_CUDA(cudaGetLastError());
  return QF_OK;
}

int qf_packed_rope_decode_attention(const qf_decode_attention_args* args, const void* positions,
                                    int32_t positions_dtype, int64_t positions_stride, const float* rope_table,
                                    int32_t table_positions, int32_t stages, void* stream) {
  int rc = qf::validate(args, true);
  QF_REQUIRE(stages >= 1 && stages <= (QF_STAGE_PARTIAL | QF_STAGE_COMBINE),
             "stages must be QF_STAGE_PARTIAL, QF_STAGE_COMBINE or both");
  if (rc != QF_OK) return rc;
  QF_REQUIRE(positions != nullptr || args->batch == 0, "positions must not be null");
  QF_REQUIRE(positions_dtype == QF_INDEX_I32 || positions_dtype == QF_INDEX_I64,
             "positions must be int32 or int64");
  QF_REQUIRE(rope_table != nullptr && table_positions >= 1 && qf::aligned16(rope_table),
             "the rotation table must be a 16-byte aligned device buffer of at least one position");
  if (args->batch == 0) return QF_OK;
  // q points at the packed rows: 16 segments of 128, the query heads first
  const qf::FusedKernel kind = qf::choose_fused_kernel(args);
  // (FP8 pools: the solo variant only, i.e. not behind qf_set_tuning mode 4)
  if (args->q_heads != 12 || args->kv_heads != 2 || args->q_stride_h != QF_HEAD_DIM ||
      args->q_stride_b < 16 * QF_HEAD_DIM || args->split_k < 2 ||
      (kind != qf::FusedKernel::kTensorCoreSolo && (kind != qf::FusedKernel::kTensorCore || args->kv_fp8))) {
    return qf::fail(QF_EUNSUPPORTED,
                    "the fused step needs the packed 12 + 2 + 2 head layout, split_k >= 2 and a layout the "
                    "tensor-core kernel takes; run the RoPE / KV write and the attention separately");
  }
  int* status = qf::status_word_for_current_device();
  QF_REQUIRE(status != nullptr, "could not resolve the device status word");
  const qf::FastParams p = qf::fast_params(args, nullptr, nullptr, status);
  qf::RopeInputs rope{};
  rope.packed = static_cast<const unsigned char*>(args->q);
  rope.row_bytes = args->q_stride_b * 2;
  rope.positions = positions, rope.pos_stride = positions_stride, rope.pos_dtype = positions_dtype;
  rope.table = reinterpret_cast<const float2*>(rope_table), rope.table_positions = table_positions;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (stages & QF_STAGE_PARTIAL) {
    if (args->kv_fp8) {
      rc = args->dtype == QF_DTYPE_F16 ? qf::launch_mma<__half, true, false, true, true>(p, s, rope)
                                       : qf::launch_mma<__nv_bfloat16, true, false, true, true>(p, s, rope);
    } else if (kind == qf::FusedKernel::kTensorCoreSolo) {
      rc = args->dtype == QF_DTYPE_F16 ? qf::launch_mma<__half, false, false, true, true>(p, s, rope)
                                       : qf::launch_mma<__nv_bfloat16, false, false, true, true>(p, s, rope);
    } else {
      rc = args->dtype == QF_DTYPE_F16 ? qf::launch_mma<__half, false, false, true>(p, s, rope)
                                       : qf::launch_mma<__nv_bfloat16, false, false, true>(p, s, rope);
    }
    if (rc != QF_OK) return rc;
  }
  if (!(stages & QF_STAGE_COMBINE)) return QF_OK;
  return qf_grouped_splitk_decode_attention_stages(args, QF_STAGE_COMBINE, stream);
}

int qf_grouped_splitk_decode_attention(const qf_decode_attention_args* args, void* stream) {
  return qf_grouped_splitk_decode_attention_stages(args, QF_STAGE_PARTIAL | QF_STAGE_COMBINE, stream);
}

int qf_grouped_gqa_splitk_diagnostics(int32_t device, int32_t dtype, int32_t kv_fp8, int64_t* info) {
  QF_REQUIRE(info != nullptr, "info must not be null");
  QF_REQUIRE(dtype == QF_DTYPE_F16 || dtype == QF_DTYPE_BF16, "dtype must be float16 or bfloat16");
  const void* kernel;
  if (kv_fp8) {
    kernel = dtype == QF_DTYPE_F16
                 ? reinterpret_cast<const void*>(qf::decode_partial_kernel<__half, true, false>)
                 : reinterpret_cast<const void*>(qf::decode_partial_kernel<__nv_bfloat16, true, false>);
  } else {
    kernel = dtype == QF_DTYPE_F16
                 ? reinterpret_cast<const void*>(qf::decode_partial_kernel<__half, false, false>)
                 : reinterpret_cast<const void*>(qf::decode_partial_kernel<__nv_bfloat16, false, false>);
  }
  int previous = 0;
  QF_CUDA(cudaGetDevice(&previous));
  QF_CUDA(cudaSetDevice(device));
  const size_t smem = qf::fast_smem_bytes(kv_fp8 != 0);
  cudaFuncAttributes attr{};
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
  if (err == cudaSuccess) err = cudaFuncGetAttributes(&attr, kernel);
  int active = 0;
  if (err == cudaSuccess) {
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&active, kernel, qf::kFastThreads, smem);
  }
  cudaDeviceProp prop{};
  if (err == cudaSuccess) err = cudaGetDeviceProperties(&prop, device);
  cudaSetDevice(previous);
  if (err != cudaSuccess) return qf::cuda_fail(err, "kernel diagnostics");
  info[0] = attr.numRegs;
  info[1] = static_cast<int64_t>(attr.sharedSizeBytes);
  info[2] = static_cast<int64_t>(smem);
  info[3] = static_cast<int64_t>(attr.localSizeBytes);
  info[4] = attr.maxThreadsPerBlock;
  info[5] = attr.binaryVersion;
  info[6] = attr.ptxVersion;
  info[7] = qf::kFastThreads;
  info[8] = active;
  info[9] = prop.maxThreadsPerMultiProcessor / 32;
  info[10] = 2 * qf::kSlots;  // pages resident in the ring
  info[11] = prop.multiProcessorCount;
  return QF_OK;
}

int qf_set_tuning(int32_t stages, int32_t force_generic) {
  QF_REQUIRE(stages >= 0 && stages <= 64, "stages must be in [0, 64]");
  QF_REQUIRE(force_generic >= 0 && force_generic <= 5, "force_generic must be in [0, 5]");
  qf::g_tuned_stages = stages;
  qf::g_force_generic = force_generic;
  return QF_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Split-K attention whose partial buffers live in a static device array.
//
// Some hosts of this library cannot hand it scratch memory: a C++ serving loop
// that binds the C ABI directly has no caching allocator to draw the partial
// buffers from, and a raw cudaMalloc / cudaFree per decode step synchronises
// the device and stalls the step; other processes give all device memory to
// their own allocator up front, so a later cudaMalloc simply fails.  For them
// the partials of this one entry point come from the array below, which every
// GPU that loads the library holds (kStaticScratchBytes) until the process ends.
// ---------------------------------------------------------------------------
namespace qf {
namespace {

constexpr size_t kStaticScratchBytes = QF_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device
// address: the address is looked up once per device, with that device current.
int static_scratch_on_current_device(float** out) {
  static std::mutex mutex;
  static void* resolved[64] = {};
  int device = 0;
  QF_CUDA(cudaGetDevice(&device));
  QF_REQUIRE(device >= 0 && device < 64, "device ordinal %d is out of range", device);
  std::lock_guard<std::mutex> lock(mutex);
  if (resolved[device] == nullptr) {
    void* address = nullptr;
    QF_CUDA(cudaGetSymbolAddress(&address, g_static_scratch));
    QF_REQUIRE(address != nullptr, "the static scratch array has no device address");
    resolved[device] = address;
  }
  *out = static_cast<float*>(resolved[device]);
  return QF_OK;
}

}  // namespace
}  // namespace qf

extern "C" int qf_grouped_splitk_decode_attention_static(const qf_decode_attention_args* args,
                                                         void* stream) {
  QF_REQUIRE(args != nullptr, "args must not be null");
  QF_REQUIRE(args->batch >= 0 && args->split_k >= 1 && args->q_heads >= 1 && args->head_dim >= 1,
             "invalid batch, split or head counts");
  // the factors are bounded one by one, so that the byte count below cannot wrap
  QF_REQUIRE(args->split_k <= 65535 && args->head_dim <= 256, "split_k must be <= 65535 and head_dim <= 256");
  QF_REQUIRE(static_cast<long long>(args->batch) * args->q_heads < (1LL << 31),
             "batch * q_heads exceeds the grid limit");
  const unsigned long long rows = static_cast<unsigned long long>(args->batch) *
                                  static_cast<unsigned long long>(args->split_k) *
                                  static_cast<unsigned long long>(args->q_heads);
  const unsigned long long needed = rows * (static_cast<unsigned long long>(args->head_dim) + 2ull) * sizeof(float);
  QF_REQUIRE(needed <= qf::kStaticScratchBytes,
             "batch * split_k * q_heads * (head_dim + 2) fp32 partials need %llu bytes; the static scratch "
             "holds %llu (QF_STATIC_SCRATCH_BYTES): lower split_k or pass your own buffers to "
             "qf_grouped_splitk_decode_attention",
             needed, static_cast<unsigned long long>(qf::kStaticScratchBytes));
  float* scratch = nullptr;
  const int rc = qf::static_scratch_on_current_device(&scratch);
  if (rc != QF_OK) return rc;
  // Every (sequence, split, head) row of the three partial tensors is written by the
  // partial pass before the combine reads it, so nothing has to start at zero.
  qf_decode_attention_args local = *args;
  local.partial_out = scratch;
  local.partial_max = scratch + rows * static_cast<unsigned long long>(args->head_dim);
  local.partial_sum = local.partial_max + rows;
  return qf_grouped_splitk_decode_attention(&local, stream);
}
