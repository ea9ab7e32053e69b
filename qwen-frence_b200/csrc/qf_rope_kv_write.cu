// Fused rotate-half RoPE on Q/K plus placement of rotated K and raw V into
// paged cache slots, for 16-bit pools and for FP8-e4m3 pools with per-page
// scales.  Restates the arithmetic of the three reference kernels
// (custom_kernels/rope_kv_write.py:12-86, :165-220 and
// custom_kernels/packed_qkv_rope_cache.py:12-88) as one CUDA kernel
// parameterised by strides.
//
// Launch shape: one CTA per row (token).  Phase 1: the first D/2 threads
// compute cos/sin of position * inv_freq[i] once per row into shared memory
// (the reference recomputes them in each of its 12-16 programs per row).
// Phase 2: each (q_heads + 2*kv_heads) segment of D elements is handled by
// D/16 threads, each loading 8 elements of the first half and the matching 8
// of the second half as two 16-byte vectors when the layout allows, or element
// by element for arbitrary strides.
//
// This file is compiled WITHOUT fast-math: cosf/sinf are the accurate
// versions and the rotation is evaluated as separate fp32 multiplies and a
// subtract/add, as PyTorch's fp32 reference does.
#include <cmath>

#include "qf_common.cuh"
#include "qf_rope_math.cuh"

namespace qf {
namespace {

struct RopeParams {
  const void* q;
  const void* k;
  const void* v;
  void* q_out;
  int64_t q_sr, q_sh, q_sd;
  int64_t k_sr, k_sh, k_sd;
  int64_t v_sr, v_sh, v_sd;
  int64_t o_sr, o_sh, o_sd;
  const void* positions;
  int64_t pos_stride;
  const void* slots;
  int64_t slot_stride;
  void* k_pool;
  void* v_pool;
  int64_t kp_ss, kp_sh, kp_sd;
  int64_t vp_ss, vp_sh, vp_sd;
  int64_t num_slots;
  const int32_t* valid_tokens;
  const float* k_scale;  // fp8 only
  const float* v_scale;
  int rows, q_heads, kv_heads, head_dim;
  int pos_dtype, slot_dtype;
  int rotate_q;
  int page_size;  // fp8 only
};

__device__ __forceinline__ uint8_t encode_e4m3(float x, float scale) {
  // clamp(x / scale, +-448) then round-to-nearest-even, saturating: the codec of
  // experiments/quant/attention.py:27-41.
  float y = __fdiv_rn(x, scale);
  y = fminf(fmaxf(y, -448.f), 448.f);
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3));
}

// T: element type of q/k/v/q_out (and of the pools unless FP8).
// VEC: every d-stride is 1 and every row/head base is 16-byte aligned.
template <typename T, bool VEC, bool FP8>
__global__ void __launch_bounds__(256) rope_kv_write_kernel(const RopeParams p,
                                                           const __grid_constant__ InvFreqTable freq) {
  __shared__ float s_cos[kMaxHalf];
  __shared__ float s_sin[kMaxHalf];

  // The rows come from the kernel before this one (the QKV projection), so nothing is
  // read ahead of it; the attention kernel after this one may start its set-up now.
  release_dependents();
  dependency_wait();
  const int row = blockIdx.x;
  const int half = p.head_dim >> 1;
  const int live_rows = p.valid_tokens ? min(*p.valid_tokens, p.rows) : p.rows;
  const bool live = row < live_rows;

  const int lanes_per_segment = p.head_dim >> 4;  // 8 + 8 elements per thread
  const int segments = (p.rotate_q ? p.q_heads : 0) + 2 * p.kv_heads;
  const int work = segments * lanes_per_segment;

  // Which segment (Q head, K head or V head) and which 8 + 8 elements an item covers.
  enum Kind { kQ, kK, kV };
  struct Item {
    Kind kind;
    int head, d0;  // first-half element offset; the second half starts at d0 + half
    const T* src;
    int64_t src_sd;
  };
  auto locate = [&](int item) {
    Item it;
    int segment = item / lanes_per_segment;
    it.d0 = (item - segment * lanes_per_segment) * 8;
    if (p.rotate_q && segment < p.q_heads) {
      it.kind = kQ;
      it.head = segment;
    } else {
      if (p.rotate_q) segment -= p.q_heads;
      it.kind = segment < p.kv_heads ? kK : kV;
      it.head = segment < p.kv_heads ? segment : segment - p.kv_heads;
    }
    if (it.kind == kQ) {
      it.src = static_cast<const T*>(p.q) + row * p.q_sr + it.head * p.q_sh;
      it.src_sd = p.q_sd;
    } else if (it.kind == kK) {
      it.src = static_cast<const T*>(p.k) + row * p.k_sr + it.head * p.k_sh;
      it.src_sd = p.k_sd;
    } else {
      it.src = static_cast<const T*>(p.v) + row * p.v_sr + it.head * p.v_sh;
      it.src_sd = p.v_sd;
    }
    return it;
  };

  // Everything the row needs from memory is requested before the sin / cos phase,
  // so that its latency overlaps that arithmetic: the slot, the position (below),
  // and, on the vector path, this thread's first item.
  int64_t slot = 0;
  bool slot_ok = false;
  if (live) {
    slot = load_index(p.slots, p.slot_dtype, row * p.slot_stride);
    slot_ok = slot >= 0 && slot < p.num_slots;
  }
  uint32_t early_first[4] = {0u, 0u, 0u, 0u}, early_second[4] = {0u, 0u, 0u, 0u};
  const bool early = VEC && live && static_cast<int>(threadIdx.x) < work;
  if constexpr (VEC) {
    if (early) {
      const Item it = locate(threadIdx.x);
      *reinterpret_cast<uint4*>(early_first) = *reinterpret_cast<const uint4*>(it.src + it.d0);
      *reinterpret_cast<uint4*>(early_second) = *reinterpret_cast<const uint4*>(it.src + it.d0 + half);
    }
  }

  if (live && threadIdx.x < half) {
    const float position = load_position(p.positions, p.pos_dtype, row * p.pos_stride);
    const float angle = __fmul_rn(position, freq.v[threadIdx.x]);
    s_cos[threadIdx.x] = cosf(angle);
    s_sin[threadIdx.x] = sinf(angle);
  }
  __syncthreads();

  for (int item = threadIdx.x; item < work; item += blockDim.x) {
    const Item it = locate(item);
    const Kind kind = it.kind;
    const int head = it.head, d0 = it.d0;

    if (!live) {
      // Padded rows of a captured token bucket: deterministic zero queries,
      // never a cache write (packed_qkv_rope_cache.py:69-71).
      if (kind == kQ && row < p.rows) {
        T* dst = static_cast<T*>(p.q_out) + row * p.o_sr + head * p.o_sh;
        for (int j = 0; j < 8; ++j) {
          dst[(d0 + j) * p.o_sd] = from_float<T>(0.f);
          dst[(d0 + half + j) * p.o_sd] = from_float<T>(0.f);
        }
      }
      continue;
    }
    if (kind != kQ && !slot_ok) continue;

    const T* src = it.src;
    const int64_t src_sd = it.src_sd;
    uint32_t first[4], second[4];  // 8 + 8 packed 16-bit elements
    if constexpr (VEC) {
      if (early && item == static_cast<int>(threadIdx.x)) {
#pragma unroll
        for (int j = 0; j < 4; ++j) first[j] = early_first[j], second[j] = early_second[j];
      } else {
        *reinterpret_cast<uint4*>(first) = *reinterpret_cast<const uint4*>(src + d0);
        *reinterpret_cast<uint4*>(second) = *reinterpret_cast<const uint4*>(src + d0 + half);
      }
    } else {
      T* f = reinterpret_cast<T*>(first);
      T* s = reinterpret_cast<T*>(second);
      for (int j = 0; j < 8; ++j) {
        f[j] = src[(d0 + j) * src_sd];
        s[j] = src[(d0 + half + j) * src_sd];
      }
    }

    float out1[8], out2[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack2<T>(first[j]);
      const float2 b = unpack2<T>(second[j]);
      if (kind == kV) {
        out1[2 * j] = a.x, out1[2 * j + 1] = a.y;
        out2[2 * j] = b.x, out2[2 * j + 1] = b.y;
      } else {
        const float c0 = s_cos[d0 + 2 * j], s0 = s_sin[d0 + 2 * j];
        const float c1 = s_cos[d0 + 2 * j + 1], s1 = s_sin[d0 + 2 * j + 1];
        out1[2 * j] = __fsub_rn(__fmul_rn(a.x, c0), __fmul_rn(b.x, s0));
        out1[2 * j + 1] = __fsub_rn(__fmul_rn(a.y, c1), __fmul_rn(b.y, s1));
        out2[2 * j] = __fadd_rn(__fmul_rn(b.x, c0), __fmul_rn(a.x, s0));
        out2[2 * j + 1] = __fadd_rn(__fmul_rn(b.y, c1), __fmul_rn(a.y, s1));
      }
    }

    if (kind == kQ || !FP8) {
      T* dst;
      int64_t dst_sd;
      if (kind == kQ) {
        dst = static_cast<T*>(p.q_out) + row * p.o_sr + head * p.o_sh;
        dst_sd = p.o_sd;
      } else if (kind == kK) {
        dst = static_cast<T*>(p.k_pool) + slot * p.kp_ss + head * p.kp_sh;
        dst_sd = p.kp_sd;
      } else {
        dst = static_cast<T*>(p.v_pool) + slot * p.vp_ss + head * p.vp_sh;
        dst_sd = p.vp_sd;
      }
      if (kind == kV) {
        // Bit-exact copy: no float round trip (keeps NaN payloads and -0).
        if constexpr (VEC) {
          *reinterpret_cast<uint4*>(dst + d0) = *reinterpret_cast<uint4*>(first);
          *reinterpret_cast<uint4*>(dst + d0 + half) = *reinterpret_cast<uint4*>(second);
        } else {
          const T* f = reinterpret_cast<const T*>(first);
          const T* s = reinterpret_cast<const T*>(second);
          for (int j = 0; j < 8; ++j) {
            dst[(d0 + j) * dst_sd] = f[j];
            dst[(d0 + half + j) * dst_sd] = s[j];
          }
        }
      } else if constexpr (VEC) {
        uint4 w1, w2;
        w1.x = pack2<T>(out1[0], out1[1]), w1.y = pack2<T>(out1[2], out1[3]);
        w1.z = pack2<T>(out1[4], out1[5]), w1.w = pack2<T>(out1[6], out1[7]);
        w2.x = pack2<T>(out2[0], out2[1]), w2.y = pack2<T>(out2[2], out2[3]);
        w2.z = pack2<T>(out2[4], out2[5]), w2.w = pack2<T>(out2[6], out2[7]);
        *reinterpret_cast<uint4*>(dst + d0) = w1;
        *reinterpret_cast<uint4*>(dst + d0 + half) = w2;
      } else {
        for (int j = 0; j < 8; ++j) {
          dst[(d0 + j) * dst_sd] = from_float<T>(out1[j]);
          dst[(d0 + half + j) * dst_sd] = from_float<T>(out2[j]);
        }
      }
    } else {
      // FP8 pools: one byte per element, fixed per-(page, head) scale.
      const int64_t page = slot / p.page_size;
      const float scale =
          (kind == kK ? p.k_scale : p.v_scale)[page * p.kv_heads + head];
      uint8_t* dst = static_cast<uint8_t*>(kind == kK ? p.k_pool : p.v_pool) +
                     (kind == kK ? slot * p.kp_ss + head * p.kp_sh
                                 : slot * p.vp_ss + head * p.vp_sh);
      const int64_t dst_sd = kind == kK ? p.kp_sd : p.vp_sd;
      if (dst_sd == 1 && (reinterpret_cast<uintptr_t>(dst + d0) & 7) == 0 && (half & 7) == 0) {
        uint8_t b1[8], b2[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          b1[j] = encode_e4m3(out1[j], scale);
          b2[j] = encode_e4m3(out2[j], scale);
        }
        *reinterpret_cast<uint2*>(dst + d0) = *reinterpret_cast<uint2*>(b1);
        *reinterpret_cast<uint2*>(dst + d0 + half) = *reinterpret_cast<uint2*>(b2);
      } else {
        for (int j = 0; j < 8; ++j) {
          dst[(d0 + j) * dst_sd] = encode_e4m3(out1[j], scale);
          dst[(d0 + half + j) * dst_sd] = encode_e4m3(out2[j], scale);
        }
      }
    }
  }
}

// One CTA per (page, kv head): amax over the page's tokens, scale =
// max(amax/448, 1e-12), then encode.  Restates quantize()
// (experiments/quant/attention.py:27-41) at page granularity.
template <typename T>
__global__ void __launch_bounds__(256) quantize_pages_kernel(const T* __restrict__ pool,
                                                            uint8_t* __restrict__ pool8,
                                                            float* __restrict__ scales,
                                                            int page_size, int kv_heads,
                                                            int head_dim) {
  __shared__ float s_red[8];
  __shared__ float s_scale;
  const int64_t page = blockIdx.x;
  const int head = blockIdx.y;
  const int per_page = page_size * head_dim;
  const int64_t page_base = page * static_cast<int64_t>(page_size) * kv_heads * head_dim;

  float amax = 0.f;
  for (int i = threadIdx.x; i < per_page; i += blockDim.x) {
    const int tok = i / head_dim, d = i - tok * head_dim;
    const float x = to_float(pool[page_base + (static_cast<int64_t>(tok) * kv_heads + head) * head_dim + d]);
    amax = fmaxf(amax, fabsf(x));
  }
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) m = fmaxf(m, s_red[w]);
    const float scale = fmaxf(__fdiv_rn(m, 448.f), 1e-12f);
    s_scale = scale;
    scales[page * kv_heads + head] = scale;
  }
  __syncthreads();
  const float scale = s_scale;
  for (int i = threadIdx.x; i < per_page; i += blockDim.x) {
    const int tok = i / head_dim, d = i - tok * head_dim;
    const int64_t off = page_base + (static_cast<int64_t>(tok) * kv_heads + head) * head_dim + d;
    pool8[off] = encode_e4m3(to_float(pool[off]), scale);
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int launch_rope(const qf_rope_kv_write_args* a, const float* k_scale, const float* v_scale,
                int page_size, bool fp8, cudaStream_t stream) {
  QF_REQUIRE(a != nullptr, "args must not be null");
  QF_REQUIRE(a->rows >= 0, "rows must be non-negative");
  QF_REQUIRE(a->dtype == QF_DTYPE_F16 || a->dtype == QF_DTYPE_BF16,
             "q, k, and v must use float16 or bfloat16");
  QF_REQUIRE(a->head_dim >= 16 && a->head_dim <= 2 * kMaxHalf && a->head_dim % 16 == 0,
             "head dimension must be a multiple of 16 no larger than %d", 2 * kMaxHalf);
  QF_REQUIRE(a->kv_heads >= 1 && a->q_heads >= 0, "head counts must be positive");
  QF_REQUIRE(a->positions_dtype == QF_INDEX_I32 || a->positions_dtype == QF_INDEX_I64 ||
                 a->positions_dtype == QF_INDEX_F32,
             "positions must be int32, int64, or float32");
  QF_REQUIRE(a->slot_dtype == QF_INDEX_I32 || a->slot_dtype == QF_INDEX_I64,
             "slot mapping must use an integer dtype");
  QF_REQUIRE(a->k && a->v && a->k_pool && a->v_pool && a->positions && a->slot_mapping,
             "k, v, pools, positions and slot mapping must not be null");
  QF_REQUIRE(!a->rotate_q || (a->q && a->q_out), "q and q_out are required when rotate_q is set");
  QF_REQUIRE(a->base > 0.0, "rope base must be positive");
  if (fp8) {
    QF_REQUIRE(k_scale && v_scale, "fp8 pools need k_scale and v_scale");
    QF_REQUIRE(page_size >= 1, "page_size must be positive");
  }
  if (a->rows == 0) return QF_OK;

  RopeParams p{};
  p.q = a->q, p.k = a->k, p.v = a->v, p.q_out = a->q_out;
  p.q_sr = a->q_stride_row, p.q_sh = a->q_stride_head, p.q_sd = a->q_stride_d;
  p.k_sr = a->k_stride_row, p.k_sh = a->k_stride_head, p.k_sd = a->k_stride_d;
  p.v_sr = a->v_stride_row, p.v_sh = a->v_stride_head, p.v_sd = a->v_stride_d;
  p.o_sr = a->o_stride_row, p.o_sh = a->o_stride_head, p.o_sd = a->o_stride_d;
  p.positions = a->positions, p.pos_stride = a->positions_stride;
  p.slots = a->slot_mapping, p.slot_stride = a->slot_stride;
  p.k_pool = a->k_pool, p.v_pool = a->v_pool;
  p.kp_ss = a->kp_stride_slot, p.kp_sh = a->kp_stride_head, p.kp_sd = a->kp_stride_d;
  p.vp_ss = a->vp_stride_slot, p.vp_sh = a->vp_stride_head, p.vp_sd = a->vp_stride_d;
  p.num_slots = a->num_slots;
  p.valid_tokens = a->valid_tokens;
  p.k_scale = k_scale, p.v_scale = v_scale;
  p.rows = a->rows, p.q_heads = a->rotate_q ? a->q_heads : 0, p.kv_heads = a->kv_heads;
  p.head_dim = a->head_dim;
  p.pos_dtype = a->positions_dtype, p.slot_dtype = a->slot_dtype;
  p.rotate_q = a->rotate_q ? 1 : 0;
  p.page_size = page_size;

  // inv_freq[i] = expf(i * (-(float)log(base) / half)): the kernels' formula
  // (custom_kernels/rope_kv_write.py:190-191), evaluated once on the host in
  // fp32 and handed to the kernel by value.
  const int half = a->head_dim / 2;
  const InvFreqTable freq = make_inv_freq(a->base, half);

  // 16-byte vectors need unit d-strides and 8-element-aligned bases/strides.
  auto mult8 = [](int64_t s) { return (s & 7) == 0; };
  bool vec = a->k_stride_d == 1 && a->v_stride_d == 1 && aligned16(a->k) && aligned16(a->v) &&
             mult8(a->k_stride_row) && mult8(a->k_stride_head) && mult8(a->v_stride_row) &&
             mult8(a->v_stride_head) && (half % 8 == 0);
  if (a->rotate_q) {
    vec = vec && a->q_stride_d == 1 && a->o_stride_d == 1 && aligned16(a->q) &&
          aligned16(a->q_out) && mult8(a->q_stride_row) && mult8(a->q_stride_head) &&
          mult8(a->o_stride_row) && mult8(a->o_stride_head);
  }
  if (!fp8) {
    vec = vec && a->kp_stride_d == 1 && a->vp_stride_d == 1 && aligned16(a->k_pool) &&
          aligned16(a->v_pool) && mult8(a->kp_stride_slot) && mult8(a->kp_stride_head) &&
          mult8(a->vp_stride_slot) && mult8(a->vp_stride_head);
  }

  const int segments = p.q_heads + 2 * p.kv_heads;
  int threads = segments * (a->head_dim / 16);
  threads = ((threads + 31) / 32) * 32;
  if (threads < half) threads = ((half + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  const dim3 grid(a->rows);

  cudaError_t err = cudaSuccess;
#define QF_LAUNCH_ROPE(T)                                                                   \
  do {                                                                                      \
    if (fp8) {                                                                              \
      if (vec)                                                                              \
        err = launch_chained(rope_kv_write_kernel<T, true, true>, grid, dim3(threads), 0, stream, p, freq);   \
      else                                                                                  \
        err = launch_chained(rope_kv_write_kernel<T, false, true>, grid, dim3(threads), 0, stream, p, freq);  \
    } else {                                                                                \
      if (vec)                                                                              \
        err = launch_chained(rope_kv_write_kernel<T, true, false>, grid, dim3(threads), 0, stream, p, freq);  \
      else                                                                                  \
        err = launch_chained(rope_kv_write_kernel<T, false, false>, grid, dim3(threads), 0, stream, p, freq); \
    }                                                                                       \
  } while (0)

  if (a->dtype == QF_DTYPE_F16) {
    QF_LAUNCH_ROPE(__half);
  } else {
    QF_LAUNCH_ROPE(__nv_bfloat16);
  }
#undef QF_LAUNCH_ROPE
  QF_CUDA(err);
  QF_CUDA(cudaGetLastError());
  return QF_OK;
}

}  // namespace
}  // namespace qf

extern "C" {

int qf_rope_kv_write(const qf_rope_kv_write_args* args, void* stream) {
  return qf::launch_rope(args, nullptr, nullptr, 0, false, static_cast<cudaStream_t>(stream));
}

int qf_rope_kv_write_fp8(const qf_rope_kv_write_args* args, const float* k_scale,
                         const float* v_scale, int32_t page_size, void* stream) {
  return qf::launch_rope(args, k_scale, v_scale, page_size, true,
                         static_cast<cudaStream_t>(stream));
}

int qf_quantize_kv_pages_e4m3(const void* pool, int32_t dtype, int64_t num_pages,
                              int32_t page_size, int32_t kv_heads, int32_t head_dim,
                              void* pool8, float* scales, void* stream) {
  QF_REQUIRE(pool && pool8 && scales, "pool, pool8 and scales must not be null");
  QF_REQUIRE(dtype == QF_DTYPE_F16 || dtype == QF_DTYPE_BF16, "pool must be float16 or bfloat16");
  QF_REQUIRE(num_pages >= 0 && num_pages < (1LL << 31), "num_pages out of range");
  QF_REQUIRE(page_size >= 1 && kv_heads >= 1 && kv_heads <= 65535 && head_dim >= 1,
             "invalid pool geometry");
  if (num_pages == 0) return QF_OK;
  const dim3 grid(static_cast<unsigned>(num_pages), kv_heads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == QF_DTYPE_F16) {
    qf::quantize_pages_kernel<__half><<<grid, 256, 0, s>>>(
        static_cast<const __half*>(pool), static_cast<uint8_t*>(pool8), scales, page_size,
        kv_heads, head_dim);
  } else {
    qf::quantize_pages_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(pool), static_cast<uint8_t*>(pool8), scales, page_size,
        kv_heads, head_dim);
  }
  QF_CUDA(cudaGetLastError());
  return QF_OK;
}

}  // extern "C"
