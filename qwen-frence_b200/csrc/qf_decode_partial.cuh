// Fast split-K partial kernel of GQA paged decode attention for sm_100a,
// geometry D=128, page=16, 6 query heads per KV head
// (baseline/naive_forward.py:17-26).  Included by qf_decode_attention.cu.
//
// Work split
//   * one CTA of eight warps per (sequence, KV head, split): the six query heads
//     of the GQA group share every K/V page load
//     (same CTA grid as native_grouped_decode.cu:62-67);
//   * pages stream through a ring of shared-memory stages guarded by full/empty
//     mbarriers and filled by 4-D tiled TMA loads ([pages,16,kv,128] tensor map,
//     box [1,16,1,128]) that lane 0 of warp 0 issues `stages - 2` pages ahead of
//     the math; page ids are fetched 32 at a time, one batch ahead;
//   * warps 0-3 compute heads 0-2 of the group, warps 4-7 heads 3-5.  Inside a
//     head group, thread (r, c) owns head dims [8c, 8c+8) of FOUR tokens per
//     iteration: rows r and r+8 of two consecutive pages.  Q (3 heads x 8 dims)
//     and the accumulators (3 heads x 8 dims) take 48 registers, so four
//     independent token chains fit without spilling and the per-iteration costs
//     (barrier waits, score reduction, softmax, address arithmetic) are spread
//     over four tokens;
//   * the twelve per-thread partial dots (4 tokens x 3 heads) are reduce-scattered
//     over the 16 lanes that share those tokens with 12 shuffles, leaving one
//     (token, head) score per lane; probabilities go back through shared memory
//     as ready-made (p, p) operands of the packed FMAs;
//   * the exponent offset is kept per (16-lane group, head) and only moves when a
//     score exceeds it by 2^8, so rescaling the accumulators is off the common
//     path; (out, offset, sum) stays self-consistent for the combine;
//   * the per-group states merge once per CTA through shared memory.
//
// No tensor-core MMA: with M=6 the op is a bandwidth-bound GEMV.  No load here
// names a cluster-multicast qualifier.  Every wait is bounded.
#pragma once

#include "qf_common.cuh"

namespace qf {
namespace {

constexpr int kConsumerWarps = 8;
constexpr int kFastThreads = kConsumerWarps * 32;
constexpr int kMaxStages = 12;
constexpr int kMinStages = 3;
constexpr int kDefaultStagesF16 = 8;
constexpr int kDefaultStagesFp8 = 12;
constexpr int kHeadsPerThread = 3;   // half of the GQA group
constexpr int kTokensPerThread = 4;  // rows r, r+8 of two pages
constexpr int kGroupRows = 8;        // 16-lane groups per head group
constexpr int kMergeFloats = kConsumerWarps * kHeadsPerThread * QF_HEAD_DIM;  // 12 KB
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
// The exponent offset follows the running maximum only when a score exceeds it
// by more than this many powers of two; probabilities stay below 2^kOffsetSlack.
constexpr float kOffsetSlack = 8.f;

struct FastParams {
  const void* q;
  int64_t q_sb, q_sh;
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
  long long* cycles;
  int* status;
  int table_dtype, lens_dtype;
  int batch, q_heads, kv_heads, split_k, stages;
  float scale_log2;  // softmax scale * log2(e)
};

template <typename T, bool FP8>
struct TileTraits {
  static constexpr int kChunkBytes = FP8 ? 8 : 16;  // one thread's 8 elements
  static constexpr int kTileBytes = QF_PAGE_SIZE * 16 * kChunkBytes;  // K or V of a page and KV head
  static constexpr int kStageBytes = 2 * kTileBytes;
};

// This thread's 8 elements of one token row, as stored (16 bytes, 8 for FP8).
template <bool FP8>
struct RawChunk {
  uint32_t w[FP8 ? 2 : 4];
};

template <bool FP8>
__device__ __forceinline__ RawChunk<FP8> load_raw(const unsigned char* at) {
  RawChunk<FP8> r;
  if constexpr (FP8) {
    const uint2 v = *reinterpret_cast<const uint2*>(at);
    r.w[0] = v.x, r.w[1] = v.y;
  } else {
    const uint4 v = *reinterpret_cast<const uint4*>(at);
    r.w[0] = v.x, r.w[1] = v.y, r.w[2] = v.z, r.w[3] = v.w;
  }
  return r;
}

template <typename T, bool FP8>
__device__ __forceinline__ void to_pairs(const RawChunk<FP8>& raw, float2 (&r)[4]) {
  if constexpr (FP8) {
    r[0] = e4m3x2_to_float2(static_cast<uint16_t>(raw.w[0] & 0xffffu));
    r[1] = e4m3x2_to_float2(static_cast<uint16_t>(raw.w[0] >> 16));
    r[2] = e4m3x2_to_float2(static_cast<uint16_t>(raw.w[1] & 0xffffu));
    r[3] = e4m3x2_to_float2(static_cast<uint16_t>(raw.w[1] >> 16));
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) r[j] = unpack2<T>(raw.w[j]);
  }
}

// Slow side of a barrier wait: poll until the phase completes, the cycle limit
// passes, or another thread of the CTA has already given up.  Giving up raises
// the CTA's abort flag and the device status word; the caller carries on with
// whatever is in shared memory, so control flow never diverges and every later
// wait returns at once.
__device__ __forceinline__ void wait_slow(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status) {
  if (*abort_flag) return;
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return;
    if (clock64() - start > kWaitCycleLimit) {
      *abort_flag = 1;
      atomicExch(status, kStatusWaitTimeout);
      return;
    }
  }
}

__device__ __forceinline__ void wait_phase(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                           int* status) {
  if (!mbar_try_wait(bar, parity)) wait_slow(bar, parity, abort_flag, status);
}

// Reduce twelve per-thread partial dots v[token*3 + head] over the 16 lanes that
// hold the same four tokens, so that each lane ends with the full dot product of
// ONE (token, head).  With lane bits b3 b2 b1 b0:
//   token = 2*b3 + b2,   head = b0 ? 2 : b1
// (head 2 is held twice, by b1 = 0 and b1 = 1).  12 shuffles, 12 adds.
__device__ __forceinline__ float reduce_scatter12(const float (&v)[12], int sub) {
  constexpr unsigned kFull = 0xffffffffu;
  const bool b3 = sub & 8, b2 = sub & 4, b1 = sub & 2, b0 = sub & 1;
  float six[6];
#pragma unroll
  for (int i = 0; i < 6; ++i) {
    const float keep = b3 ? v[6 + i] : v[i];
    const float send = b3 ? v[i] : v[6 + i];
    six[i] = keep + __shfl_xor_sync(kFull, send, 8);
  }
  float three[3];
#pragma unroll
  for (int h = 0; h < 3; ++h) {
    const float keep = b2 ? six[3 + h] : six[h];
    const float send = b2 ? six[h] : six[3 + h];
    three[h] = keep + __shfl_xor_sync(kFull, send, 4);
  }
  float a = b1 ? three[1] : three[0];
  const float send_a = b1 ? three[0] : three[1];
  a += __shfl_xor_sync(kFull, send_a, 2);
  const float c = three[2] + __shfl_xor_sync(kFull, three[2], 2);
  float x = b0 ? c : a;
  const float send_x = b0 ? a : c;
  x += __shfl_xor_sync(kFull, send_x, 1);
  return x;
}

// Lane (within a 16-lane group) that holds head h of token 0 after reduce_scatter12.
__device__ __forceinline__ constexpr int head_lane(int h) { return h == 0 ? 0 : h == 1 ? 2 : 1; }


template <typename T, bool FP8, bool PROFILE>
__global__ void __launch_bounds__(kFastThreads, 2)
    decode_partial_tma_kernel(const __grid_constant__ CUtensorMap k_map,
                              const __grid_constant__ CUtensorMap v_map, const FastParams p) {
  using Traits = TileTraits<T, FP8>;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ uint64_t full_bar[kMaxStages];
  __shared__ uint64_t empty_bar[kMaxStages];
  __shared__ float stage_scale[kMaxStages][2];
  __shared__ int batch_ids[32];
  __shared__ float batch_scale[32][2];
  // Probabilities of one iteration as (p, p) operands: [parity][warp][half-warp][token*3 + head]
  __shared__ __align__(16) float2 prob_pairs[2][kConsumerWarps][2][12];
  __shared__ float group_offset[2][kGroupRows][kHeadsPerThread];  // [head group][row][head]
  __shared__ float group_sum[2][kGroupRows][kHeadsPerThread];
  __shared__ float cta_offset[QF_GQA_GROUP];
  __shared__ float cta_sum[QF_GQA_GROUP];
  __shared__ int abort_word;
  __shared__ int issued_loads;  // iterations (pages) whose loads have been issued

  constexpr unsigned kFull = 0xffffffffu;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int sub = lane & 15;                          // dim chunk, and lane in the 16-lane group
  const int head_group = warp >> 2;                   // heads 3*head_group .. +2 of the GQA group
  const int row = ((warp & 3) << 1) | (lane >> 4);    // token rows `row` and `row + 8` of a page
  const int stages = p.stages;
  const int lookahead = stages - 2;                   // pages in flight ahead of the math
  volatile int* abort_flag = &abort_word;

  // blockIdx.x = (sequence * kv_heads + kv_head) * split_k + split
  const int split = blockIdx.x % p.split_k;
  const int kv_head = (blockIdx.x / p.split_k) % p.kv_heads;
  const int sequence = blockIdx.x / (p.split_k * p.kv_heads);

  int seq_len;
  {
    int64_t raw = load_index(p.seq_lens, p.lens_dtype, sequence * p.lens_stride);
    raw = raw < 0 ? 0 : raw;
    seq_len = static_cast<int>(raw > 0x7ffffff0 ? 0x7ffffff0 : raw);
  }
  const int total_pages = (seq_len + QF_PAGE_SIZE - 1) / QF_PAGE_SIZE;
  const int start_page = static_cast<int>(static_cast<int64_t>(split) * total_pages / p.split_k);
  const int end_page = static_cast<int>((static_cast<int64_t>(split) + 1) * total_pages / p.split_k);
  const int num_iters = end_page - start_page;  // pages of this partition
  // Tokens of this partition that exist, counted from its first page: every token
  // index below this is inside the sequence.
  const int tokens_here = min(seq_len - start_page * QF_PAGE_SIZE, num_iters * QF_PAGE_SIZE);

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kConsumerWarps);
    }
    abort_word = 0;
    issued_loads = 0;
    fence_barrier_init();
    if (num_iters > 0) {
      tma_prefetch_descriptor(&k_map);
      tma_prefetch_descriptor(&v_map);
    }
  }
  __syncthreads();

  // ---- producer role (warp 0 only; every lane runs it, lane 0 issues) ----
  // Page ids (and FP8 scales) are fetched 32 at a time into registers, one batch
  // ahead, and parked in shared memory when their batch becomes current.
  const int num_pages = static_cast<int>(p.num_pages);
  int ids_next = -1;
  float ks_next = 1.f, vs_next = 1.f;
  auto fetch_batch = [&](int first_iter) {
    const int idx = start_page + first_iter + lane;
    ids_next = -1;
    if (idx < end_page) {
      const int64_t raw = load_index(p.block_table, p.table_dtype,
                                     sequence * p.bt_sb + static_cast<int64_t>(idx) * p.bt_sp);
      ids_next = raw >= 0 && raw < num_pages ? static_cast<int>(raw) : -1;  // -1: outside the pool
    }
    if (FP8) {
      ks_next = ids_next >= 0 ? p.k_scale[static_cast<int64_t>(ids_next) * p.kv_heads + kv_head] : 1.f;
      vs_next = ids_next >= 0 ? p.v_scale[static_cast<int64_t>(ids_next) * p.kv_heads + kv_head] : 1.f;
    }
  };
  // Issues the loads of page `index` (0-based in this partition; called with
  // index = 0, 1, 2, ...) into the next stage of the ring, once the previous
  // occupant of that stage has been released.  A fresh barrier reports the phase
  // of parity 1 complete, so the first lap never waits.
  int pstage = 0;
  uint32_t pparity = 1u;
  auto produce = [&](int index) {
    if ((index & 31) == 0) {
      if (index == 0) fetch_batch(0);
      __syncwarp();
      batch_ids[lane] = ids_next;
      if (FP8) batch_scale[lane][0] = ks_next, batch_scale[lane][1] = vs_next;
      __syncwarp();
      if (index + 32 < num_iters) fetch_batch(index + 32);
    }
    if (lane == 0) {
      wait_phase(&empty_bar[pstage], pparity, abort_flag, p.status);
      const int page_id = batch_ids[index & 31];
      if (page_id < 0) atomicExch(p.status, kStatusBadPageId);
      if (FP8) {
        stage_scale[pstage][0] = batch_scale[index & 31][0];
        stage_scale[pstage][1] = batch_scale[index & 31][1];
      }
      unsigned char* dst = smem + pstage * Traits::kStageBytes;
      mbar_arrive_expect_tx(&full_bar[pstage], Traits::kStageBytes);
      // A page id outside the pool reads as zeros (TMA out-of-bounds fill).
      tma_load_4d(dst, &k_map, &full_bar[pstage], 0, kv_head, 0, page_id);
      tma_load_4d(dst + Traits::kTileBytes, &v_map, &full_bar[pstage], 0, kv_head, 0, page_id);
      issued_loads = index + 1;
    }
    if (++pstage == stages) pstage = 0, pparity ^= 1u;
    __syncwarp();
  };

  if (warp == 0) {
    for (int i = 0; i < lookahead && i < num_iters; ++i) produce(i);
  }

  // ---- per-thread state: 3 heads x 8 dims of Q (pre-scaled) and of the output ----
  float2 q2[kHeadsPerThread][4];
  float2 acc[kHeadsPerThread][4];
#pragma unroll
  for (int h = 0; h < kHeadsPerThread; ++h)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[h][j] = make_float2(0.f, 0.f);
  if (num_iters > 0) {
    const T* qbase = static_cast<const T*>(p.q) + sequence * p.q_sb +
                     (static_cast<int64_t>(kv_head) * QF_GQA_GROUP + head_group * kHeadsPerThread) * p.q_sh +
                     sub * 8;
    const float2 s2 = make_float2(p.scale_log2, p.scale_log2);
#pragma unroll
    for (int h = 0; h < kHeadsPerThread; ++h) {
      const uint4 raw = *reinterpret_cast<const uint4*>(qbase + h * p.q_sh);
      q2[h][0] = __fmul2_rn(unpack2<T>(raw.x), s2);
      q2[h][1] = __fmul2_rn(unpack2<T>(raw.y), s2);
      q2[h][2] = __fmul2_rn(unpack2<T>(raw.z), s2);
      q2[h][3] = __fmul2_rn(unpack2<T>(raw.w), s2);
    }
  }
  // After the reduce-scatter this lane owns one (token, head) of its group:
  const int my_token = ((sub >> 3) & 1) * 2 + ((sub >> 2) & 1);  // 0: (page A,row) 1: (A,row+8) 2: (B,row) 3: (B,row+8)
  const int my_head = (sub & 1) ? 2 : ((sub >> 1) & 1);
  float my_offset = -INFINITY;  // exponent offset of my head, shared by the group (log2 units)
  float my_sum = 0.f;           // sum of p over my token stream
  // Byte offset of this thread's chunk of token row `row` inside a K or V tile.
  const int chunk_offset = (((warp & 3) << 5) | lane) * Traits::kChunkBytes;
  constexpr int kRowPlus8 = 8 * 16 * Traits::kChunkBytes;
  float2* prob_slot = &prob_pairs[0][warp][lane >> 4][0];
  constexpr int kProbParityStride = kConsumerWarps * 2 * 12;  // float2 elements

  // ------------------------------ main loop -------------------------------
  // One iteration = two pages (A, B) = four tokens per thread.  A missing page B
  // (odd page count) and the sequence's partial last page are handled by one
  // rule: token t of the partition exists iff t < tokens_here.
  long long t_wait = 0, t_total = 0, t_mark = 0;
  if (PROFILE) t_total = clock64();
  int stage_a = 0;
  uint32_t phase_a = 0;
  int produce_next = lookahead < num_iters ? lookahead : num_iters;  // next page index to issue (warp 0)
  for (int page_a = 0; page_a < num_iters; page_a += 2) {
    int stage_b = stage_a + 1;
    uint32_t phase_b = phase_a;
    if (stage_b == stages) stage_b = 0, phase_b ^= 1u;
    const bool has_b = page_a + 1 < num_iters;
    if (warp == 0) {
      // keep the ring `lookahead` pages ahead of the pair being computed
      for (int n = 0; n < 2 && produce_next < num_iters; ++n) produce(produce_next++);
    }
    const unsigned char* tile_a = smem + stage_a * Traits::kStageBytes + chunk_offset;
    const unsigned char* tile_b = smem + stage_b * Traits::kStageBytes + chunk_offset;
    if (PROFILE) t_mark = clock64();
    wait_phase(&full_bar[stage_a], phase_a, abort_flag, p.status);
    if (has_b) wait_phase(&full_bar[stage_b], phase_b, abort_flag, p.status);
    if (PROFILE) t_wait += clock64() - t_mark;

    // ---- scores: q . k for 3 heads x 4 tokens over this thread's 8 dims ----
    float dots[12];
    auto score_token = [&](const unsigned char* at, int base) {
      float2 kreg[4];
      to_pairs<T, FP8>(load_raw<FP8>(at), kreg);
#pragma unroll
      for (int h = 0; h < kHeadsPerThread; ++h) {
        float2 d = __fmul2_rn(q2[h][0], kreg[0]);
#pragma unroll
        for (int j = 1; j < 4; ++j) d = __ffma2_rn(q2[h][j], kreg[j], d);
        dots[base + h] = d.x + d.y;
      }
    };
    score_token(tile_a, 0);
    score_token(tile_a + kRowPlus8, 3);
    if (has_b) {
      score_token(tile_b, 6);
      score_token(tile_b + kRowPlus8, 9);
    } else {
#pragma unroll
      for (int i = 6; i < 12; ++i) dots[i] = 0.f;
    }
    float score = reduce_scatter12(dots, sub);
    const int token_base = page_a * QF_PAGE_SIZE + row;  // partition-relative index of token 0
    const bool my_valid = token_base + (my_token >> 1) * QF_PAGE_SIZE + (my_token & 1) * 8 < tokens_here;
    if (FP8) score *= stage_scale[(my_token >> 1) ? stage_b : stage_a][0];
    if (!my_valid) score = -INFINITY;

    // ---- online softmax; the offset of a head is shared by its four token lanes ----
    const bool grow = score > my_offset + kOffsetSlack;  // also the first valid token (offset -inf)
    if (__any_sync(kFull, grow)) {
      float target = fmaxf(my_offset, score);
      target = fmaxf(target, __shfl_xor_sync(kFull, target, 8));
      target = fmaxf(target, __shfl_xor_sync(kFull, target, 4));
      const float corr = my_offset == -INFINITY ? 0.f : fast_exp2(my_offset - target);
      my_sum *= corr;
      my_offset = target;
#pragma unroll
      for (int h = 0; h < kHeadsPerThread; ++h) {
        const float ch = __shfl_sync(kFull, corr, head_lane(h), 16);
        const float2 c2 = make_float2(ch, ch);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[h][j] = __fmul2_rn(acc[h][j], c2);
      }
    }
    float prob = fast_exp2(score - my_offset);
    if (!my_valid) prob = 0.f;  // also covers offset == -inf (NaN from inf - inf)
    my_sum += prob;
    if (FP8) prob *= stage_scale[(my_token >> 1) ? stage_b : stage_a][1];

    // ---- publish the twelve probabilities of this group as (p, p) pairs ----
    float2* probs = prob_slot + ((page_a >> 1) & 1) * kProbParityStride;
    probs[my_token * 3 + my_head] = make_float2(prob, prob);  // head 2 is written twice, same value
    __syncwarp();
    float4 pp[6];
#pragma unroll
    for (int i = 0; i < 6; ++i) pp[i] = reinterpret_cast<const float4*>(probs)[i];

    // ---- values: acc[h] += p[token][h] * v[token] ----
    auto add_token = [&](const unsigned char* at, int k) {
      float2 vreg[4];
      to_pairs<T, FP8>(load_raw<FP8>(at + Traits::kTileBytes), vreg);
#pragma unroll
      for (int h = 0; h < kHeadsPerThread; ++h) {
        const int i = k * 3 + h;  // compile-time after unrolling
        const float2 p2 = (i & 1) ? make_float2(pp[i >> 1].z, pp[i >> 1].w)
                                  : make_float2(pp[i >> 1].x, pp[i >> 1].y);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[h][j] = __ffma2_rn(p2, vreg[j], acc[h][j]);
      }
    };
    if (token_base + 8 + QF_PAGE_SIZE < tokens_here) {
      // all four tokens exist (the common case)
      add_token(tile_a, 0);
      add_token(tile_a + kRowPlus8, 1);
      add_token(tile_b, 2);
      add_token(tile_b + kRowPlus8, 3);
    } else {
      if (token_base < tokens_here) add_token(tile_a, 0);
      if (token_base + 8 < tokens_here) add_token(tile_a + kRowPlus8, 1);
      if (token_base + QF_PAGE_SIZE < tokens_here) add_token(tile_b, 2);
      if (token_base + QF_PAGE_SIZE + 8 < tokens_here) add_token(tile_b + kRowPlus8, 3);
    }

    // ---- both stages are in registers: hand them back to the producer ----
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(&empty_bar[stage_a]);
      if (has_b) mbar_arrive(&empty_bar[stage_b]);
    }
    stage_a = stage_b + 1, phase_a = phase_b;
    if (stage_a == stages) stage_a = 0, phase_a ^= 1u;
  }
  if (PROFILE && p.cycles != nullptr && tid == 32) {
    // One pure-consumer warp per CTA reports {waiting for pages, whole loop, 0, 0}.
    long long* dst = p.cycles + static_cast<int64_t>(blockIdx.x) * 4;
    dst[0] = t_wait, dst[1] = clock64() - t_total, dst[2] = 0, dst[3] = 0;
  }

  // ------------------------------ CTA merge -------------------------------
  // Barrier: every stage has been read, so the ring is free for the merge.
  __syncthreads();
  if (*abort_flag) {
    // A wait ran out somewhere in this CTA.  Give the loads already issued a
    // bounded chance to land before their shared memory is reused or released.
    if (tid == 0) {
      abort_word = 0;  // let the waits below poll again
      const int issued = issued_loads;
      for (int s = 0; s < stages && s < issued; ++s) {
        const int last = ((issued - 1 - s) / stages) * stages + s;  // last page that used stage s
        wait_phase(&full_bar[s], static_cast<uint32_t>(last / stages) & 1u, abort_flag, p.status);
      }
    }
    __syncthreads();
  }
  float* merge = reinterpret_cast<float*>(smem);  // [8 warps][3 heads][128]
  {
    // sum of a head over the group's four token streams (lanes differing in bits 3, 2)
    float total = my_sum + __shfl_xor_sync(kFull, my_sum, 8);
    total += __shfl_xor_sync(kFull, total, 4);
    if (my_token == 0 && sub == head_lane(my_head)) {
      group_offset[head_group][row][my_head] = my_offset;
      group_sum[head_group][row][my_head] = total;
    }
  }
  __syncthreads();
  if (tid < QF_GQA_GROUP) {
    const int g = tid / kHeadsPerThread, h = tid - g * kHeadsPerThread;
    float m = -INFINITY;
    for (int r = 0; r < kGroupRows; ++r) m = fmaxf(m, group_offset[g][r][h]);
    float total = 0.f;
    for (int r = 0; r < kGroupRows; ++r) {
      const float mg = group_offset[g][r][h];
      if (mg != -INFINITY) total += group_sum[g][r][h] * fast_exp2(mg - m);
    }
    cta_offset[tid] = m;
    cta_sum[tid] = total;
  }
  __syncthreads();
#pragma unroll
  for (int h = 0; h < kHeadsPerThread; ++h) {
    const float mg = group_offset[head_group][row][h];
    const float f = mg == -INFINITY ? 0.f : fast_exp2(mg - cta_offset[head_group * kHeadsPerThread + h]);
    const float2 f2 = make_float2(f, f);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = __fmul2_rn(acc[h][j], f2);
      a.x += __shfl_xor_sync(kFull, a.x, 16);
      a.y += __shfl_xor_sync(kFull, a.y, 16);
      acc[h][j] = a;
    }
    if (lane < 16) {
      float4* dst =
          reinterpret_cast<float4*>(merge + (warp * kHeadsPerThread + h) * QF_HEAD_DIM + sub * 8);
      dst[0] = make_float4(acc[h][0].x, acc[h][0].y, acc[h][1].x, acc[h][1].y);
      dst[1] = make_float4(acc[h][2].x, acc[h][2].y, acc[h][3].x, acc[h][3].y);
    }
  }
  __syncthreads();
  const int64_t head0 = static_cast<int64_t>(kv_head) * QF_GQA_GROUP;
  const int64_t partial_row =
      (static_cast<int64_t>(sequence) * p.split_k + split) * p.q_heads + head0;
#pragma unroll
  for (int i = 0; i < (QF_GQA_GROUP * QF_HEAD_DIM) / kFastThreads; ++i) {
    const int e = tid + i * kFastThreads;  // (head, dim) flattened
    const int head = e >> 7, d = e & 127;
    const int g = head / kHeadsPerThread, h = head - g * kHeadsPerThread;
    float value = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) value += merge[((g * 4 + w) * kHeadsPerThread + h) * QF_HEAD_DIM + d];
    if (p.partial_out != nullptr) p.partial_out[partial_row * QF_HEAD_DIM + e] = value;
    if (p.out != nullptr) {
      const float total = cta_sum[head];
      const float norm = value / (total > 0.f ? total : 1.f);
      static_cast<T*>(p.out)[sequence * p.o_sb + (head0 + head) * p.o_sh + d * p.o_sd] =
          from_float<T>(norm);
    }
  }
  if (tid < QF_GQA_GROUP && p.partial_max != nullptr) {
    // natural-log units, as the combine and the reference's reduce expect
    p.partial_max[partial_row + tid] = cta_offset[tid] * kLn2;
    p.partial_sum[partial_row + tid] = cta_sum[tid];
  }
}

}  // namespace
}  // namespace qf
