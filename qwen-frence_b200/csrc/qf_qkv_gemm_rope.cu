// QKV projection with the RoPE + paged KV-cache write as its epilogue, for decode batches:
//   packed = T(hidden @ weight^T + bias)            [rows, 2048], fp32 accumulate, one rounding
//   q, k   = rope(packed)  (fp32, one rounding);  v = packed;  k, v -> cache slot of the row
// i.e. exactly packed_qkv_rope_cache applied to the model-dtype output of the projection, as
// the reference's CUTLASS epilogue does (custom_kernels/gemm_epilogue/fused_gemm.cu:223-310),
// without the packed tensor ever reaching memory.
//
// Shape of the work: rows <= a few hundred, N = 2048, K = 1536 -- the 6.3 MB weight matrix is
// streamed once; tensor-core time is negligible, so the kernel is built to keep many TMA
// loads in flight per SM and to finish in about one weight-read time.
//   * CTA tile: 128 rows x 64 columns = columns [32j, 32j+32) of one head and their rotation
//     partners [64+32j, 64+32j+32), j = 0/1 -> 32 column tiles, so RoPE needs no exchange.
//   * Operands travel by tiled TMA (cp.async.bulk.tensor.2d, 128-byte swizzle, no multicast)
//     into a 6-stage ring: A = 128 x 64 of hidden (rows beyond the batch are zero-filled or
//     ignored), B = 2 x (32 x 64) of weight.  One thread issues the copies, one thread issues
//     tcgen05.mma (M 128, N 64, K 16, fp32 accumulator in 64 TMEM columns); a stage is
//     released by tcgen05.commit on its "empty" barrier.
//   * Four epilogue warps compute their row's sin / cos while the ring runs, then read the
//     accumulator with tcgen05.ld (32 lanes x 32 columns per warp and half), add the bias,
//     round, rotate and store to q / the cache.
//   * 32 tiles would leave most of the 148 SMs idle and each CTA waiting on its own ring, so
//     for up to 256 rows K is split four ways over a thread-block cluster (128 - 256 CTAs, a
//     whole K slice in flight per CTA): the four partial accumulators are exchanged through
//     distributed shared memory as a reduce-scatter, after which each CTA owns 8 columns and
//     their 8 partners of the tile and finishes those (sums taken in rank order).
// Every barrier wait is bounded: when one runs out, the CTA records status 5, stops issuing,
// waits (bounded) for copies and MMAs in flight, frees its TMEM and returns.
#include <cuda.h>

#include <cmath>
#include <type_traits>

#include "qf_common.cuh"
#include "qf_rope_math.cuh"

namespace qf {
namespace {

constexpr int kTileM = 128;
constexpr int kTileN = 64;   // 32 columns + their 32 rotation partners
constexpr int kTileK = 64;   // 128 bytes per row: one swizzle atom wide
constexpr int kStages = 6;
constexpr int kBytesA = kTileM * kTileK * 2;  // 16 KB
constexpr int kBytesB = kTileN * kTileK * 2;  // 8 KB
constexpr int kStageBytes = kBytesA + kBytesB;
constexpr int kGemmThreads = 192;             // warps 0-3 epilogue, 4 copies, 5 MMA + TMEM
constexpr int kTmemColumns = 64;
constexpr int kQkvWidth = 2048;
constexpr int kSpinLimit = 1 << 21;
constexpr int kGemmTimelineColumns = QF_GEMM_TIMELINE_COLUMNS;
constexpr size_t kGemmSmemBytes = kStages * kStageBytes + 1024;  // + room to align to 1 KB

struct GemmParams {
  const void* bias;  // [2048] or null
  void* q_out;
  int64_t q_stride_row;
  const void* positions;
  const void* slots;
  void* k_cache;     // flat [slots, 2, 128]
  void* v_cache;
  int64_t num_slots;
  const int* valid_tokens;
  int* status;
  long long* timeline;  // [CTAs][kGemmTimelineColumns] %globaltimer stamps, or null
  int rows, k_blocks, a_box_rows;
  int pos_dtype, slot_dtype;
};

__device__ __forceinline__ long long nanoseconds_now() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait; gives up for the whole CTA (abort flag in shared memory) when it runs out.
__device__ __forceinline__ bool wait_barrier(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (int spin = 0; spin < kSpinLimit; ++spin) {
    if (try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (spin > 128) __nanosleep(64);
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// K-major operand tile in 128-byte-swizzled shared memory: rows of 128 bytes, groups of
// eight rows 1024 bytes apart (descriptor version 1, layout type 2 = SWIZZLE_128B).
__device__ __forceinline__ uint64_t operand_descriptor(uint32_t smem_address) {
  uint64_t desc = (smem_address >> 4) & 0x3fffu;
  desc |= uint64_t(1) << 16;            // leading byte offset (unused for swizzled K-major)
  desc |= uint64_t(1024 >> 4) << 32;    // stride between 8-row groups
  desc |= uint64_t(1) << 46;            // descriptor version
  desc |= uint64_t(2) << 61;            // SWIZZLE_128B
  return desc;
}

template <typename T>
__device__ __forceinline__ float round_to_storage(float x) {
  return to_float(from_float<T>(x));
}

// Cluster helpers (SPLIT > 1: the CTAs of a cluster share one output tile and split K).
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive_relaxed() {  // nothing to publish: presence only
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_shared_address(uint32_t local_address, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_address), "r"(rank));
  return remote;
}
__device__ __forceinline__ void store_peer_v4(uint32_t address, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(address), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

// SPLIT = 1: one CTA per tile walks all of K.  SPLIT = 4: a cluster of four CTAs per tile,
// each accumulates a quarter of K, then the four exchange partial sums through distributed
// shared memory so that each ends up with (and finishes) a quarter of the tile's columns.
template <typename T, int SPLIT>
__global__ void __launch_bounds__(kGemmThreads, 1)
    qkv_gemm_rope_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const GemmParams p, const __grid_constant__ InvFreqTable freq) {
  constexpr int kOwn = 32 / SPLIT;  // columns (and as many partners) this CTA finishes
  extern __shared__ unsigned char smem_raw[];
  __shared__ uint64_t full_bar[kStages], empty_bar[kStages], acc_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ float s_bias[kTileN];

  release_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x, m_tile = blockIdx.y;
  long long* stamps = p.timeline == nullptr ? nullptr
                                            : p.timeline + ((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x +
                                                            blockIdx.x) * kGemmTimelineColumns;
  auto stamp = [&](int column) {
    if (stamps != nullptr) stamps[column] = nanoseconds_now();
  };
  if (threadIdx.x == 0) stamp(0);  // entry
  const int rank = SPLIT > 1 ? static_cast<int>(cluster_rank()) : 0;
  const int head = n_tile >> 1, j = n_tile & 1;  // 16 heads: 12 Q, 2 K, 2 V
  const int column0 = head * 128 + j * 32;       // partners at column0 + 64
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t exchange = ring + kStages * kStageBytes;  // [source rank][2 * kOwn / 4 groups][128 rows][4] fp32
  const int my_blocks = p.k_blocks / SPLIT, first_block = rank * my_blocks;
  volatile int* aborted = &abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&full_bar[s])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&empty_bar[s])));
    }
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&acc_bar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the copies' completions use the async proxy
    abort_flag = 0;
  }
  if (threadIdx.x == 4 * 32) {  // the copy thread fetches its two descriptors while the others set up
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
  }
  if (threadIdx.x < kTileN) {  // the model's bias: no kernel writes it
    const int column = column0 + (threadIdx.x & 31) + (threadIdx.x >> 5) * 64;
    s_bias[threadIdx.x] = p.bias ? to_float(static_cast<const T*>(p.bias)[column]) : 0.f;
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(kTmemColumns));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  if (threadIdx.x == 0) stamp(1);  // barriers and TMEM ready
  // Phase 1 of the cluster barrier: its wait (before the first remote store) proves that
  // every CTA of the cluster is resident.
  if (SPLIT > 1) cluster_arrive_relaxed();

  uint32_t lo[32], hi[32];  // this row's accumulators (epilogue warps)
  bool ready = false;
  if (warp == 4) {
    const uint32_t bytes = static_cast<uint32_t>(p.a_box_rows) * kTileK * 2 + kBytesB;
    auto load_weights = [&](int i) {
      const uint32_t b = ring + (i % kStages) * kStageBytes + kBytesA, full = smem_u32(&full_bar[i % kStages]);
      tma_load_2d(b, &map_b, (first_block + i) * kTileK, column0, full);
      tma_load_2d(b + kBytesB / 2, &map_b, (first_block + i) * kTileK, column0 + 64, full);
    };
    auto load_rows = [&](int i) {
      tma_load_2d(ring + (i % kStages) * kStageBytes, &map_a, (first_block + i) * kTileK, m_tile * kTileM,
                  smem_u32(&full_bar[i % kStages]));
    };
    // The weights belong to the model (no kernel writes them): the first ring-full of weight
    // tiles is requested while the previous kernel is still running; the rows of `hidden`
    // follow once that kernel has completed.  One lane per stage: a thread issues a tensor
    // copy every 70 ns or so, which in one thread would stagger the ring by a microsecond.
    const int early = my_blocks < kStages ? my_blocks : kStages;
    if (lane < early) {
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&full_bar[lane])), "r"(bytes)
                   : "memory");
      load_weights(lane);
    }
    dependency_wait();
    if (lane == 0) stamp(2);  // previous kernel complete
    if (lane < early) load_rows(lane);
    if (lane == 0) {
      int issued = early;
      for (int i = early; i < my_blocks; ++i, ++issued) {
        const int s = i % kStages;
        if (!wait_barrier(smem_u32(&empty_bar[s]), ((i / kStages) & 1) ^ 1, aborted)) break;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&full_bar[s])), "r"(bytes)
                     : "memory");
        load_rows(i);
        load_weights(i);
      }
      if (*aborted) {
        // copies already issued still land in this CTA's shared memory: wait for them
        for (int i = issued > kStages ? issued - kStages : 0; i < issued; ++i) {
          for (int spin = 0; spin < kSpinLimit; ++spin) {
            if (try_wait(smem_u32(&full_bar[i % kStages]), (i / kStages) & 1)) break;
            __nanosleep(64);
          }
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      dependency_wait();
      // instruction descriptor: fp32 accumulate, A and B K-major, N = 64, M = 128
      const uint32_t format = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;  // operand type code
      const uint32_t idesc = (1u << 4) | (format << 7) | (format << 10) | (uint32_t(kTileN >> 3) << 17) |
                             (uint32_t(kTileM >> 4) << 24);
      for (int i = 0; i < my_blocks; ++i) {
        const int s = i % kStages;
        if (!wait_barrier(smem_u32(&full_bar[s]), (i / kStages) & 1, aborted)) break;
        if (i == 0) stamp(3);  // first operand tiles landed
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a = ring + s * kStageBytes, b = a + kBytesA;
        const uint64_t desc_a = operand_descriptor(a), desc_b = operand_descriptor(b);
#pragma unroll
        for (int k = 0; k < kTileK / 16; ++k) {
          const uint32_t accumulate = (i | k) != 0 ? 1u : 0u;
          // 16 elements of K = 32 bytes further along the swizzled row
          asm volatile(
              "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
              :
              : "r"(tmem_base), "l"(desc_a + uint64_t(k * 2)), "l"(desc_b + uint64_t(k * 2)), "r"(idesc),
                "r"(accumulate)
              : "memory");
        }
        // frees the stage once the MMAs that read it have completed
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                         smem_u32(&empty_bar[s]))
                     : "memory");
      }
      stamp(4);  // last MMA issued
      // always: the epilogue and the TMEM release wait on this
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                       smem_u32(&acc_bar))
                   : "memory");
    }
  }

  // ---- epilogue warps: row m of the batch <-> TMEM lane 32 * warp + lane ----
  const int row = warp * 32 + lane;  // meaningful for warps 0-3
  const int m = m_tile * kTileM + row;
  const bool is_q = head < 12, is_v = head >= 14;
  bool in_batch = false, live = false;
  int64_t slot = -1;
  float cosine[kOwn], sine[kOwn];
  if (warp < 4) {
    dependency_wait();  // positions, slots and valid_tokens may come from the kernel before
    const int live_rows = p.valid_tokens ? min(*p.valid_tokens, p.rows) : p.rows;
    in_batch = m < p.rows, live = m < live_rows;
    if (live) {
      if (!is_q) {
        slot = load_index(p.slots, p.slot_dtype, m);
        if (slot < 0 || slot >= p.num_slots) {
          if (rank == 0) atomicMax(p.status, kStatusBadPageId);
          slot = -1;
        }
      }
      if (!is_v) {
        const float position = load_position(p.positions, p.pos_dtype, m);
#pragma unroll
        for (int c = 0; c < kOwn; ++c) {
          const float angle = __fmul_rn(position, freq.v[j * 32 + rank * kOwn + c]);
          cosine[c] = cosf(angle);
          sine[c] = sinf(angle);
        }
      }
    }
    // warp-uniform: tcgen05.ld is a warp-wide instruction
    ready = __all_sync(0xffffffffu, wait_barrier(smem_u32(&acc_bar), 0, aborted) && !*aborted);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (threadIdx.x == 0) stamp(5);  // accumulator complete
    if (ready) {
      const uint32_t address = tmem_base + (uint32_t(warp * 32) << 16);
#define QF_TMEM_LOAD_32(dst, addr)                                                                        \
  asm volatile(                                                                                           \
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                            \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                            \
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"            \
      : "=r"(dst[0]), "=r"(dst[1]), "=r"(dst[2]), "=r"(dst[3]), "=r"(dst[4]), "=r"(dst[5]), "=r"(dst[6]),  \
        "=r"(dst[7]), "=r"(dst[8]), "=r"(dst[9]), "=r"(dst[10]), "=r"(dst[11]), "=r"(dst[12]),             \
        "=r"(dst[13]), "=r"(dst[14]), "=r"(dst[15]), "=r"(dst[16]), "=r"(dst[17]), "=r"(dst[18]),          \
        "=r"(dst[19]), "=r"(dst[20]), "=r"(dst[21]), "=r"(dst[22]), "=r"(dst[23]), "=r"(dst[24]),          \
        "=r"(dst[25]), "=r"(dst[26]), "=r"(dst[27]), "=r"(dst[28]), "=r"(dst[29]), "=r"(dst[30]),          \
        "=r"(dst[31])                                                                                      \
      : "r"(addr))
      QF_TMEM_LOAD_32(lo, address);
      QF_TMEM_LOAD_32(hi, address + 32);
#undef QF_TMEM_LOAD_32
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (SPLIT > 1) {
        cluster_wait();  // phase 1: the peers are resident
        // reduce-scatter: the partial sums of columns [kOwn * d, kOwn * (d + 1)) and of their
        // partners go to CTA d, into the slot of this CTA's rank (its own share included)
#pragma unroll
        for (int d = 0; d < SPLIT; ++d) {
          // [source rank][group of four values][row][4]: 16-byte stores, the lanes of a warp
          // (consecutive rows) side by side, so a store covers 512 contiguous bytes
          const uint32_t group0 =
              peer_shared_address(exchange + uint32_t((rank * (2 * kOwn / 4)) * kTileM + row) * 16, uint32_t(d));
#pragma unroll
          for (int c = 0; c < kOwn; c += 4) {
            store_peer_v4(group0 + uint32_t((c / 4) * kTileM) * 16, lo[d * kOwn + c], lo[d * kOwn + c + 1],
                          lo[d * kOwn + c + 2], lo[d * kOwn + c + 3]);
            store_peer_v4(group0 + uint32_t(((kOwn + c) / 4) * kTileM) * 16, hi[d * kOwn + c], hi[d * kOwn + c + 1],
                          hi[d * kOwn + c + 2], hi[d * kOwn + c + 3]);
          }
        }
      }
    }
  }
  __syncwarp();
  if (SPLIT > 1) {
    // every thread passes phase 1 exactly once, then phase 2: the partial sums have
    // arrived (release / acquire at cluster scope)
    if (!(warp < 4 && ready)) cluster_wait();
    if (threadIdx.x == 0) stamp(6);  // partial sums sent
    cluster_arrive();
    cluster_wait();
  }
  if (threadIdx.x == 0) stamp(7);  // partial sums of the peers arrived

  if (warp < 4 && ready) {
    float sum_lo[kOwn], sum_hi[kOwn];
    if (SPLIT > 1) {
      const float4* parts = reinterpret_cast<const float4*>(smem_raw + (exchange - smem_u32(smem_raw)));
#pragma unroll
      for (int c = 0; c < kOwn; ++c) sum_lo[c] = 0.f, sum_hi[c] = 0.f;
#pragma unroll
      for (int source = 0; source < SPLIT; ++source) {  // always in rank order: deterministic
        const float4* group0 = parts + (source * (2 * kOwn / 4)) * kTileM + row;
#pragma unroll
        for (int c = 0; c < kOwn; c += 4) {
          const float4 a = group0[(c / 4) * kTileM], b = group0[((kOwn + c) / 4) * kTileM];
          sum_lo[c] = __fadd_rn(sum_lo[c], a.x), sum_lo[c + 1] = __fadd_rn(sum_lo[c + 1], a.y);
          sum_lo[c + 2] = __fadd_rn(sum_lo[c + 2], a.z), sum_lo[c + 3] = __fadd_rn(sum_lo[c + 3], a.w);
          sum_hi[c] = __fadd_rn(sum_hi[c], b.x), sum_hi[c + 1] = __fadd_rn(sum_hi[c + 1], b.y);
          sum_hi[c + 2] = __fadd_rn(sum_hi[c + 2], b.z), sum_hi[c + 3] = __fadd_rn(sum_hi[c + 3], b.w);
        }
      }
    } else {
#pragma unroll
      for (int c = 0; c < kOwn; ++c) sum_lo[c] = __uint_as_float(lo[c]), sum_hi[c] = __uint_as_float(hi[c]);
    }

    const int own0 = rank * kOwn;  // first own column inside the 32-column run
    T* first = nullptr;            // kOwn elements here, their partners 64 elements further
    if (is_q) {
      if (in_batch) first = static_cast<T*>(p.q_out) + m * p.q_stride_row + column0 + own0;
    } else if (live && slot >= 0) {
      const int kv_head = (head - 12) & 1;
      first = static_cast<T*>(is_v ? p.v_cache : p.k_cache) + (slot * 2 + kv_head) * 128 + j * 32 + own0;
    }
    if (first != nullptr) {
      uint32_t out_lo[kOwn / 2], out_hi[kOwn / 2];
#pragma unroll
      for (int c = 0; c < kOwn; c += 2) {
        float a[2], b[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          // the projection's output in the model dtype, then the rotation in fp32
          a[e] = round_to_storage<T>(__fadd_rn(sum_lo[c + e], s_bias[own0 + c + e]));
          b[e] = round_to_storage<T>(__fadd_rn(sum_hi[c + e], s_bias[32 + own0 + c + e]));
          if (!is_v) {
            const float x = a[e], y = b[e];
            a[e] = __fsub_rn(__fmul_rn(x, cosine[c + e]), __fmul_rn(y, sine[c + e]));
            b[e] = __fadd_rn(__fmul_rn(y, cosine[c + e]), __fmul_rn(x, sine[c + e]));
          }
          if (is_q && !live) a[e] = 0.f, b[e] = 0.f;  // padded rows of a token bucket
        }
        out_lo[c >> 1] = pack2<T>(a[0], a[1]);
        out_hi[c >> 1] = pack2<T>(b[0], b[1]);
      }
#pragma unroll
      for (int v = 0; v < kOwn / 8; ++v) {
        reinterpret_cast<uint4*>(first)[v] =
            make_uint4(out_lo[4 * v], out_lo[4 * v + 1], out_lo[4 * v + 2], out_lo[4 * v + 3]);
        reinterpret_cast<uint4*>(first + 64)[v] =
            make_uint4(out_hi[4 * v], out_hi[4 * v + 1], out_hi[4 * v + 2], out_hi[4 * v + 3]);
      }
    }
  }

  if (threadIdx.x == 0) stamp(8);  // outputs stored
  __syncwarp();
  // ---- teardown: nobody touches TMEM after this barrier; MMAs have completed (or the
  // bounded wait on the accumulator barrier has run out) before it is freed ----
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 5) {
    if (*aborted) {
      for (int spin = 0; spin < kSpinLimit; ++spin) {
        if (try_wait(smem_u32(&acc_bar), 0)) break;
        __nanosleep(64);
      }
      if (lane == 0) atomicMax(p.status, kStatusPipelineTimeout);
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns));
    if (lane == 0) stamp(9);  // TMEM released
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      entry = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(entry);
  }();
  return fn;
}

// [rows, columns] 16-bit matrix, unit stride inside a row; box = box_rows x 64 columns, 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t columns, int64_t row_stride, int box_rows,
              bool bf16) {
  EncodeTiledFn encode = encode_tiled();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(columns), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_stride) * 2};
  const cuuint32_t box[2] = {kTileK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t element_strides[2] = {1, 1};
  return encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                const_cast<void*>(base), dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; }

constexpr size_t kExchangeBytes = 2 * 32 * kTileM * 4;  // [SPLIT][2 * 32 / SPLIT][128] fp32 = 32 KB

template <typename T, int SPLIT>
cudaError_t launch_split(const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmParams& p,
                         const InvFreqTable& freq, unsigned m_tiles, cudaStream_t stream) {
  auto kernel = qkv_gemm_rope_kernel<T, SPLIT>;
  const size_t smem = kGemmSmemBytes + (SPLIT > 1 ? kExchangeBytes : 0);
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (err != cudaSuccess) return err;
  const dim3 grid(kQkvWidth / kTileN, m_tiles, SPLIT);
  if (SPLIT == 1) return launch_chained(kernel, grid, dim3(kGemmThreads), smem, stream, map_a, map_b, p, freq);
  return launch_chained(kernel, grid, dim3(kGemmThreads), smem, stream, ClusterShape{1, 1, SPLIT}, map_a, map_b, p,
                        freq);
}

template <typename T>
cudaError_t launch_gemm(const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmParams& p,
                        const InvFreqTable& freq, cudaStream_t stream) {
  const unsigned m_tiles = static_cast<unsigned>((p.rows + kTileM - 1) / kTileM);
  // 32 column tiles per 128 rows: split K over a cluster while the grid still fits the
  // SMs in one wave (one CTA per SM), and K divides into slices of at least two blocks.
  auto fits = [&](int split) { return p.k_blocks % split == 0 && p.k_blocks >= 2 * split && m_tiles * split <= 4; };
  if (fits(4)) return launch_split<T, 4>(map_a, map_b, p, freq, m_tiles, stream);
  if (fits(2)) return launch_split<T, 2>(map_a, map_b, p, freq, m_tiles, stream);
  return launch_split<T, 1>(map_a, map_b, p, freq, m_tiles, stream);
}

}  // namespace
}  // namespace qf

namespace qf {
namespace {
int run_qkv_rope_cache(const qf_qkv_rope_cache_args* a, long long* timeline, void* stream);
}
}  // namespace qf

extern "C" int qf_qkv_rope_cache(const qf_qkv_rope_cache_args* a, void* stream) {
  return qf::run_qkv_rope_cache(a, nullptr, stream);
}

extern "C" int qf_qkv_rope_cache_timeline(const qf_qkv_rope_cache_args* a, int64_t* timeline, void* stream) {
  QF_REQUIRE(timeline != nullptr, "timeline must not be null");
  return qf::run_qkv_rope_cache(a, reinterpret_cast<long long*>(timeline), stream);
}

namespace qf {
namespace {
int run_qkv_rope_cache(const qf_qkv_rope_cache_args* a, long long* timeline, void* stream) {
  QF_REQUIRE(a != nullptr, "args must not be null");
  QF_REQUIRE(a->dtype == QF_DTYPE_F16 || a->dtype == QF_DTYPE_BF16, "dtype must be fp16 or bf16");
  QF_REQUIRE(a->rows >= 0, "row count must not be negative");
  QF_REQUIRE(a->in_features > 0 && a->in_features % kTileK == 0,
             "the input width must be a positive multiple of 64");
  QF_REQUIRE(a->positions_dtype == QF_INDEX_I32 || a->positions_dtype == QF_INDEX_I64 ||
                 a->positions_dtype == QF_INDEX_F32,
             "positions must be int32, int64 or float32");
  QF_REQUIRE(a->slot_dtype == QF_INDEX_I32 || a->slot_dtype == QF_INDEX_I64,
             "slot mapping must use an integer dtype");
  if (a->rows == 0) return QF_OK;
  QF_REQUIRE(a->hidden && a->weight && a->q_out && a->positions && a->slot_mapping && a->k_pool && a->v_pool,
             "hidden, weight, q_out, positions, slot mapping and pools must not be null");
  QF_REQUIRE(aligned16(a->hidden) && aligned16(a->weight) && aligned16(a->q_out) && aligned16(a->k_pool) &&
                 aligned16(a->v_pool) && a->hidden_stride_row % 8 == 0 && a->weight_stride_row % 8 == 0 &&
                 a->q_stride_row % 8 == 0,
             "tensors must be 16-byte aligned with row strides that are multiples of 8 elements");
  QF_REQUIRE(a->hidden_stride_row >= a->in_features && a->weight_stride_row >= a->in_features &&
                 a->q_stride_row >= 12 * 128,
             "row strides are shorter than the rows");
  QF_REQUIRE(a->num_slots > 0, "the pools must hold at least one slot");

  const bool bf16 = a->dtype == QF_DTYPE_BF16;
  const int box_rows = a->rows < kTileM ? a->rows : kTileM;
  CUtensorMap map_a, map_b;
  if (!make_map(&map_a, a->hidden, a->rows, a->in_features, a->hidden_stride_row, box_rows, bf16) ||
      !make_map(&map_b, a->weight, kQkvWidth, a->in_features, a->weight_stride_row, kTileN / 2, bf16)) {
    return fail(QF_ECUDA, "cuTensorMapEncodeTiled failed or is unavailable");
  }
  GemmParams p;
  p.bias = a->bias, p.q_out = a->q_out, p.q_stride_row = a->q_stride_row;
  p.positions = a->positions, p.slots = a->slot_mapping;
  p.k_cache = a->k_pool, p.v_cache = a->v_pool, p.num_slots = a->num_slots;
  p.valid_tokens = static_cast<const int*>(a->valid_tokens);
  p.status = device_status_word();
  p.timeline = timeline;
  QF_REQUIRE(p.status != nullptr, "device status word is unavailable");
  p.rows = a->rows, p.k_blocks = a->in_features / kTileK, p.a_box_rows = box_rows;
  p.pos_dtype = a->positions_dtype, p.slot_dtype = a->slot_dtype;
  const InvFreqTable freq = make_inv_freq(a->base, 64);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  QF_CUDA(bf16 ? launch_gemm<__nv_bfloat16>(map_a, map_b, p, freq, s) : launch_gemm<__half>(map_a, map_b, p, freq, s));
  return QF_OK;
}
}  // namespace
}  // namespace qf
