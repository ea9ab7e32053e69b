// Fast split-K partial kernel of GQA paged decode attention for sm_100a,
// geometry D=128, page=16, 6 query heads per KV head
// (baseline/naive_forward.py:17-26).  Included by qf_decode_attention.cu.
//
// Work split
//   * one CTA of eight warps per (sequence, KV head, split): the six query heads
//     of the GQA group share every K/V page load
//     (same CTA grid as native_grouped_decode.cu:62-67);
//   * warps 0-3 compute heads 0-2 of the group, warps 4-7 heads 3-5.  Inside a
//     head group, thread (r, c) owns head dims [8c, 8c+8) of FOUR tokens per
//     iteration: rows r and r+8 of two consecutive pages.  Q (3 heads x 8 dims)
//     and the accumulators (3 heads x 8 dims) take 48 registers, so four
//     independent token chains fit without spilling and the per-iteration costs
//     are spread over four tokens;
//   * loads: 16-byte cp.async (global -> shared, no registers) into a ring of
//     page-pair slots, three pairs ahead of the math.  A thread and its twin in
//     the other head group need the same eight chunks; the twin in group 0
//     copies the four K chunks, the one in group 1 the four V chunks, and the
//     two warps meet at a 64-thread named barrier once per iteration.  Each
//     16-byte chunk of a page is fetched exactly once, a warp's copies cover
//     whole 256-byte rows, and nothing spins: the only waits are
//     cp.async.wait_group and bar.sync.  (A 4-D tiled TMA box of one KV head is
//     16 rows of 256 B at a 512 B pitch; streaming such boxes with no math reached
//     3.7 TB/s on B200 against 6.7 - 6.9 TB/s for 16-byte loads that cover whole
//     rows warp-wide, and 6.5 - 6.8 TB/s for a box that spans both KV heads.)
//   * the twelve per-thread partial dots (4 tokens x 3 heads) are reduce-scattered
//     over the 16 lanes that share those tokens with 12 shuffles, leaving one
//     (token, head) score per lane; probabilities go back through shared memory
//     as ready-made (p, p) operands of the packed FMAs (fma.rn.f32x2);
//   * the exponent offset is kept per (16-lane group, head) and only moves when a
//     score exceeds it by 2^8, so rescaling the accumulators is off the common
//     path; (out, offset, sum) stays self-consistent for the combine;
//   * the per-group states merge once per CTA through shared memory.
//
// No tensor-core MMA: with M=6 the op is a bandwidth-bound GEMV.
#pragma once

#include "qf_common.cuh"

namespace qf {
namespace {

constexpr int kConsumerWarps = 8;
constexpr int kFastThreads = kConsumerWarps * 32;
constexpr int kDepth = 3;             // page pairs in flight ahead of the math
constexpr int kSlots = kDepth + 1;    // page-pair slots in the ring (a power of two)
constexpr int kHeadsPerThread = 3;    // half of the GQA group
constexpr int kTokensPerThread = 4;   // rows r, r+8 of two pages
constexpr int kGroupRows = 8;         // 16-lane groups per head group
constexpr int kMergeFloats = kConsumerWarps * kHeadsPerThread * QF_HEAD_DIM;  // 12 KB
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
// The exponent offset follows the running maximum only when a score exceeds it
// by more than this many powers of two; probabilities stay below 2^kOffsetSlack.
constexpr float kOffsetSlack = 8.f;

struct FastParams {
  const void* q;
  int64_t q_sb, q_sh;
  const unsigned char* k_pool;
  const unsigned char* v_pool;
  int64_t k_page_bytes, k_tok_bytes, k_head_bytes;  // pool strides in bytes
  int64_t v_page_bytes, v_tok_bytes, v_head_bytes;
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
  int batch, q_heads, kv_heads, split_k;
  int max_tokens;    // table_width * page size: a longer sequence length is cut to this
  float scale_log2;  // softmax scale * log2(e)
};

template <typename T, bool FP8>
struct TileTraits {
  static constexpr int kChunkBytes = FP8 ? 8 : 16;                    // one thread's 8 elements
  static constexpr int kTileBytes = QF_PAGE_SIZE * 16 * kChunkBytes;  // K or V of a page and KV head
  static constexpr int kSlotBytes = 4 * kTileBytes;                   // K(A) K(B) V(A) V(B)
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

// Asynchronous global -> shared copy of one chunk (16 bytes, 8 for FP8), L2 only.
template <bool FP8>
__device__ __forceinline__ void copy_chunk_async(unsigned char* smem_dst, const unsigned char* src) {
  if constexpr (FP8) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(smem_dst)), "l"(src) : "memory");
  } else {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(src) : "memory");
  }
}
__device__ __forceinline__ void commit_copies() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Wait until at most kDepth - 1 of this thread's committed groups are in flight,
// i.e. until the oldest of the kDepth pairs it keeps in flight has landed.
__device__ __forceinline__ void wait_oldest_pair() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kDepth - 1) : "memory");
}
__device__ __forceinline__ void wait_all_copies() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
// Barrier among the 64 threads of a warp and its twin in the other head group.
__device__ __forceinline__ void twin_barrier(int pair) {
  asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory");
}

// Reduce twelve per-thread partial dots over the 16 lanes that hold the same four
// tokens, so that each lane ends with the full dot product of ONE (token, head).
// With lane bits b3 b2 b1 b0 the lane ends up owning
//   token = 2*b3 + b2  (0: page A,row  1: A,row+8  2: B,row  3: B,row+8),  head = b0 ? 2 : b1.
// The caller hands the dots in a LANE-DEPENDENT order, v[(2*P + R)*3 + head], where
// P = 0 is the page this lane keeps (A if b3 = 0, else B) and R = 0 the row it keeps
// (row if b2 = 0, else row+8): the exchange partner at distance 8 (4) keeps the other
// page (row), so "keep the first half, send the second half" needs no selects.
// (head 2 is held twice, by b1 = 0 and b1 = 1).  12 shuffles, 12 adds.
__device__ __forceinline__ float reduce_scatter12(const float (&v)[12], int sub) {
  constexpr unsigned kFull = 0xffffffffu;
  const bool b1 = sub & 2, b0 = sub & 1;
  float six[6];
#pragma unroll
  for (int i = 0; i < 6; ++i) six[i] = v[i] + __shfl_xor_sync(kFull, v[6 + i], 8);
  float three[3];
#pragma unroll
  for (int h = 0; h < 3; ++h) three[h] = six[h] + __shfl_xor_sync(kFull, six[3 + h], 4);
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


// What a lane does inside its 16-lane group, fixed for the kernel's lifetime.
template <typename T, bool FP8>
struct LaneRole {
  int sub;        // dim chunk, and lane within the 16-lane group
  int row;        // token rows `row` and `row + 8` of a page
  int my_token;   // after the reduce-scatter this lane owns one (token, head):
  int my_head;    //   token 0: (page A, row)  1: (A, row+8)  2: (B, row)  3: (B, row+8)
  int keep_page, send_page;  // byte offsets, inside a slot's K region, of the page / row
  int keep_row, send_row;    //   this lane keeps and sends in the reduce-scatter
  __device__ __forceinline__ LaneRole(int sub_, int row_) : sub(sub_), row(row_) {
    using Traits = TileTraits<T, FP8>;
    constexpr int kRowPlus8 = 8 * 16 * Traits::kChunkBytes;
    my_token = ((sub >> 3) & 1) * 2 + ((sub >> 2) & 1);
    my_head = (sub & 1) ? 2 : ((sub >> 1) & 1);
    keep_page = (sub & 8) ? Traits::kTileBytes : 0, send_page = Traits::kTileBytes - keep_page;
    keep_row = (sub & 4) ? kRowPlus8 : 0, send_row = kRowPlus8 - keep_row;
  }
};

// One page pair (A, B) = four tokens per thread: scores of 3 heads x 4 tokens,
// online softmax with the lazily moving offset, probabilities through shared
// memory, accumulate p * V.  `slot` points at this thread's chunk of token row
// `row` in the pair's K(A) tile; `token_base` is the index, counted from the first
// token of the range `tokens_here` is measured in, of token 0; a token exists iff
// its index is below `tokens_here`, and `all_valid` promises that all 32 do.
template <typename T, bool FP8>
__device__ __forceinline__ void attend_pair(const unsigned char* slot, float2* probs,
                                            const LaneRole<T, FP8>& role,
                                            const float2 (&q2)[kHeadsPerThread][4],
                                            float2 (&acc)[kHeadsPerThread][4], float& my_offset,
                                            float& my_sum, bool all_valid, int token_base,
                                            int tokens_here, float k_mul, float v_mul) {
  using Traits = TileTraits<T, FP8>;
  constexpr unsigned kFull = 0xffffffffu;
  constexpr int kRowPlus8 = 8 * 16 * Traits::kChunkBytes;
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
  // lane-dependent order: kept page / kept row first (see reduce_scatter12)
  score_token(slot + role.keep_page + role.keep_row, 0);
  score_token(slot + role.keep_page + role.send_row, 3);
  score_token(slot + role.send_page + role.keep_row, 6);
  score_token(slot + role.send_page + role.send_row, 9);
  float score = reduce_scatter12(dots, role.sub);
  bool my_valid = true;
  if (FP8) score *= k_mul;
  if (!all_valid) {
    my_valid = token_base + (role.my_token >> 1) * QF_PAGE_SIZE + (role.my_token & 1) * 8 < tokens_here;
    if (!my_valid) score = -INFINITY;
  }

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
  if (!all_valid && !my_valid) prob = 0.f;  // also covers offset == -inf (NaN from inf - inf)
  my_sum += prob;
  if (FP8) prob *= v_mul;

  // ---- publish the twelve probabilities of this group as (p, p) pairs ----
  probs[role.my_token * 3 + role.my_head] = make_float2(prob, prob);  // head 2 is written twice, same value
  __syncwarp();

  // ---- values: acc[h] += p[token][h] * v[token] ----
  auto add_token = [&](const unsigned char* at, int k) {
    float2 vreg[4];
    to_pairs<T, FP8>(load_raw<FP8>(at), vreg);
#pragma unroll
    for (int h = 0; h < kHeadsPerThread; ++h) {
      const float2 p2 = probs[k * 3 + h];
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[h][j] = __ffma2_rn(p2, vreg[j], acc[h][j]);
    }
  };
  const unsigned char* values = slot + 2 * Traits::kTileBytes;
  if (all_valid) {
    // all four tokens exist (the common case)
    add_token(values, 0);
    add_token(values + kRowPlus8, 1);
    add_token(values + Traits::kTileBytes, 2);
    add_token(values + Traits::kTileBytes + kRowPlus8, 3);
  } else {
    // a token that does not exist may hold anything (NaN included): skip it
    if (token_base < tokens_here) add_token(values, 0);
    if (token_base + 8 < tokens_here) add_token(values + kRowPlus8, 1);
    if (token_base + QF_PAGE_SIZE < tokens_here) add_token(values + Traits::kTileBytes, 2);
    if (token_base + QF_PAGE_SIZE + 8 < tokens_here) add_token(values + Traits::kTileBytes + kRowPlus8, 3);
  }
}

// Shared-memory state of the once-per-partition merge of the sixteen 16-lane groups.
struct MergeShared {
  float group_offset[2][kGroupRows][kHeadsPerThread];  // [head group][row][head]
  float group_sum[2][kGroupRows][kHeadsPerThread];
  float cta_offset[QF_GQA_GROUP];
  float cta_sum[QF_GQA_GROUP];
};

// Merge the per-group (accumulator, offset, sum) states of a CTA and store the
// result: the unnormalised fp32 partial of the six heads (`partial_out_row`,
// [6][128]) with its offset in natural-log units and its sum, and / or the
// normalised output (`out_row`, head stride o_sh, dim stride o_sd).  `merge` is
// kMergeFloats of shared memory nobody else touches until the call returns.  Every
// thread of the CTA calls this; it contains three CTA-wide barriers.
template <typename T>
__device__ __forceinline__ void merge_and_store(MergeShared& ms, float* merge,
                                                float2 (&acc)[kHeadsPerThread][4], float my_offset,
                                                float my_sum, int my_token, int my_head,
                                                float* partial_out_row, float* partial_max_row,
                                                float* partial_sum_row, T* out_row, int64_t o_sh,
                                                int64_t o_sd) {
  constexpr unsigned kFull = 0xffffffffu;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, sub = lane & 15;
  const int head_group = warp >> 2;
  const int row = ((warp & 3) << 1) | (lane >> 4);
  {
    // sum of a head over the group's four token streams (lanes differing in bits 3, 2)
    float total = my_sum + __shfl_xor_sync(kFull, my_sum, 8);
    total += __shfl_xor_sync(kFull, total, 4);
    if (my_token == 0 && sub == head_lane(my_head)) {
      ms.group_offset[head_group][row][my_head] = my_offset;
      ms.group_sum[head_group][row][my_head] = total;
    }
  }
  __syncthreads();
  if (tid < QF_GQA_GROUP) {
    const int g = tid / kHeadsPerThread, h = tid - g * kHeadsPerThread;
    float m = -INFINITY;
    for (int r = 0; r < kGroupRows; ++r) m = fmaxf(m, ms.group_offset[g][r][h]);
    float total = 0.f;
    for (int r = 0; r < kGroupRows; ++r) {
      const float mg = ms.group_offset[g][r][h];
      if (mg != -INFINITY) total += ms.group_sum[g][r][h] * fast_exp2(mg - m);
    }
    ms.cta_offset[tid] = m;
    ms.cta_sum[tid] = total;
  }
  __syncthreads();
#pragma unroll
  for (int h = 0; h < kHeadsPerThread; ++h) {
    const float mg = ms.group_offset[head_group][row][h];
    const float f = mg == -INFINITY ? 0.f : fast_exp2(mg - ms.cta_offset[head_group * kHeadsPerThread + h]);
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
#pragma unroll
  for (int i = 0; i < (QF_GQA_GROUP * QF_HEAD_DIM) / kFastThreads; ++i) {
    const int e = tid + i * kFastThreads;  // (head, dim) flattened
    const int head = e >> 7, d = e & 127;
    const int g = head / kHeadsPerThread, h = head - g * kHeadsPerThread;
    float value = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) value += merge[((g * 4 + w) * kHeadsPerThread + h) * QF_HEAD_DIM + d];
    if (partial_out_row != nullptr) partial_out_row[e] = value;
    if (out_row != nullptr) {
      const float total = ms.cta_sum[head];
      out_row[head * o_sh + d * o_sd] = from_float<T>(value / (total > 0.f ? total : 1.f));
    }
  }
  if (tid < QF_GQA_GROUP && partial_max_row != nullptr) {
    // natural-log units, as the combine and the reference's reduce expect
    partial_max_row[tid] = ms.cta_offset[tid] * kLn2;
    partial_sum_row[tid] = ms.cta_sum[tid];
  }
}

#ifndef QF_MIN_CTAS
#define QF_MIN_CTAS 2
#endif
template <typename T, bool FP8, bool PROFILE>
__global__ void __launch_bounds__(kFastThreads, QF_MIN_CTAS)
    decode_partial_kernel(const FastParams p) {
  using Traits = TileTraits<T, FP8>;
  extern __shared__ __align__(1024) unsigned char smem[];  // ring of page-pair slots; merge scratch later
  // Probabilities of one iteration as (p, p) operands: [parity][warp][half-warp][token*3 + head]
  __shared__ __align__(16) float2 prob_pairs[2][kConsumerWarps][2][12];
  __shared__ MergeShared merge_state;

  long long t_entry = 0;
  if (PROFILE) t_entry = clock64();
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int sub = lane & 15;                        // dim chunk, and lane in the 16-lane group
  const int head_group = warp >> 2;                 // heads 3*head_group .. +2 of the GQA group
  const int row = ((warp & 3) << 1) | (lane >> 4);  // token rows `row` and `row + 8` of a page

  // blockIdx.x = (sequence * kv_heads + kv_head) * split_k + split
  const int split = blockIdx.x % p.split_k;
  const int kv_head = (blockIdx.x / p.split_k) % p.kv_heads;
  const int sequence = blockIdx.x / (p.split_k * p.kv_heads);

  int seq_len;
  {
    int64_t raw = load_index(p.seq_lens, p.lens_dtype, sequence * p.lens_stride);
    raw = raw < 0 ? 0 : raw;
    seq_len = static_cast<int>(raw > p.max_tokens ? p.max_tokens : raw);  // never read past the table row
  }
  const int total_pages = (seq_len + QF_PAGE_SIZE - 1) / QF_PAGE_SIZE;
  const int start_page = static_cast<int>(static_cast<int64_t>(split) * total_pages / p.split_k);
  const int end_page = static_cast<int>((static_cast<int64_t>(split) + 1) * total_pages / p.split_k);
  const int num_pages_here = end_page - start_page;  // pages of this partition
  const int num_pairs = (num_pages_here + 1) >> 1;
  // Tokens of this partition that exist, counted from its first page.
  const int tokens_here = min(seq_len - start_page * QF_PAGE_SIZE, num_pages_here * QF_PAGE_SIZE);

  // ---- loads -------------------------------------------------------------
  // This thread copies four chunks per page pair: rows `row`, `row+8` of pages A and
  // B, of K when it is in head group 0 and of V when it is in head group 1.
  const int pool_pages = static_cast<int>(p.num_pages);
  const unsigned char* pool = head_group == 0 ? p.k_pool : p.v_pool;
  const int64_t page_bytes = head_group == 0 ? p.k_page_bytes : p.v_page_bytes;
  const int64_t tok_bytes = head_group == 0 ? p.k_tok_bytes : p.v_tok_bytes;
  const unsigned char* pool_row =
      pool + row * tok_bytes + kv_head * (head_group == 0 ? p.k_head_bytes : p.v_head_bytes) +
      sub * Traits::kChunkBytes;
  // Byte offset of this thread's chunk of token row `row` inside a K or V tile.
  const int chunk_offset = (((warp & 3) << 5) | lane) * Traits::kChunkBytes;
  constexpr int kRowPlus8 = 8 * 16 * Traits::kChunkBytes;
  const int fill_offset = head_group * 2 * Traits::kTileBytes + chunk_offset;  // K tiles first, then V tiles
  // The partition's block-table entries: byte pointer to the next unread entry.
  const int table_elem = p.table_dtype == QF_INDEX_I64 ? 8 : 4;
  const int64_t table_step = p.bt_sp * table_elem;
  const unsigned char* table_first =
      static_cast<const unsigned char*>(p.block_table) +
      (sequence * p.bt_sb + static_cast<int64_t>(start_page) * p.bt_sp) * table_elem;
  const unsigned char* table_next = table_first;
  // Page id stored at `at`, or -1 when the page does not exist or lies outside
  // the pool (recorded in the status word, never dereferenced).
  auto read_id = [&](const unsigned char* at, bool exists) -> int {
    if (!exists) return -1;
    const int64_t raw = table_elem == 8 ? *reinterpret_cast<const int64_t*>(at)
                                        : static_cast<int64_t>(*reinterpret_cast<const int32_t*>(at));
    if (static_cast<uint64_t>(raw) >= static_cast<uint64_t>(pool_pages)) {
      atomicMax(p.status, kStatusBadPageId);
      return -1;
    }
    return static_cast<int>(raw);
  };
  auto copy_page = [&](unsigned char* dst, int page_id) {
    if (page_id >= 0) {
      const unsigned char* src = pool_row + static_cast<int64_t>(page_id) * page_bytes;
      copy_chunk_async<FP8>(dst, src);
      copy_chunk_async<FP8>(dst + kRowPlus8, src + 8 * tok_bytes);
    } else {
      // no such page: zeros, so that nothing stale or non-finite is ever multiplied
      if constexpr (FP8) {
        *reinterpret_cast<uint2*>(dst) = make_uint2(0u, 0u);
        *reinterpret_cast<uint2*>(dst + kRowPlus8) = make_uint2(0u, 0u);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(dst + kRowPlus8) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };
  // Page ids of the pair to be issued next are fetched one iteration early.
  int pages_left = num_pages_here;  // pages whose ids have not been fetched yet
  int next_id_a = -1, next_id_b = -1;
  auto fetch_ids = [&]() {
    next_id_a = read_id(table_next, pages_left > 0);
    next_id_b = read_id(table_next + table_step, pages_left > 1);
    table_next += 2 * table_step;
    pages_left -= 2;
  };
  int pairs_to_issue = num_pairs;
  int fill_slot = 0;
  auto issue_pair = [&]() {
    if (pairs_to_issue > 0) {
      unsigned char* dst = smem + fill_slot * Traits::kSlotBytes + fill_offset;
      copy_page(dst, next_id_a);
      copy_page(dst + Traits::kTileBytes, next_id_b);
      --pairs_to_issue;
      fetch_ids();
    }
    commit_copies();  // always, so that group counting stays uniform
    fill_slot = (fill_slot + 1) & (kSlots - 1);
  };
  {
    // Prologue: the ids of the first kDepth + 1 pairs are read in ONE round trip
    // (independent loads), then the first kDepth pairs are put in flight.
    int first_ids[2 * kDepth + 2];
#pragma unroll
    for (int i = 0; i < 2 * kDepth + 2; ++i) first_ids[i] = read_id(table_first + i * table_step, i < num_pages_here);
#pragma unroll
    for (int i = 0; i < kDepth; ++i) {
      if (i < num_pairs) {
        unsigned char* dst = smem + i * Traits::kSlotBytes + fill_offset;
        copy_page(dst, first_ids[2 * i]);
        copy_page(dst + Traits::kTileBytes, first_ids[2 * i + 1]);
      }
      commit_copies();
    }
    fill_slot = kDepth & (kSlots - 1);
    pairs_to_issue = max(num_pairs - kDepth, 0);
    next_id_a = first_ids[2 * kDepth];
    next_id_b = first_ids[2 * kDepth + 1];
    table_next = table_first + (2 * kDepth + 2) * table_step;
    pages_left = num_pages_here - (2 * kDepth + 2);
  }

  // ---- per-thread state: 3 heads x 8 dims of Q (pre-scaled) and of the output ----
  float2 q2[kHeadsPerThread][4];
  float2 acc[kHeadsPerThread][4];
#pragma unroll
  for (int h = 0; h < kHeadsPerThread; ++h)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[h][j] = make_float2(0.f, 0.f);
  if (num_pairs > 0) {
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
  const LaneRole<T, FP8> role(sub, row);
  const int my_token = role.my_token, my_head = role.my_head;
  float my_offset = -INFINITY;  // exponent offset of my head, shared by the group (log2 units)
  float my_sum = 0.f;           // sum of p over my token stream
  float2* prob_slot = &prob_pairs[0][warp][lane >> 4][0];
  constexpr int kProbParityStride = kConsumerWarps * 2 * 12;  // float2 elements

  // ------------------------------ main loop -------------------------------
  // One iteration = one page pair (A, B) = four tokens per thread.  A missing page B
  // (odd page count) and the sequence's partial last page are handled by one
  // rule: token t of the partition exists iff t < tokens_here.
  long long t_wait = 0, t_total = 0, t_mark = 0;
  if (PROFILE) t_total = clock64();
  // FP8: dequantisation scales of the page that holds this lane's token, fetched an
  // iteration ahead (the lane that owns a score only needs its own page's scales).
  float k_mul = 1.f, v_mul = 1.f, k_mul_next = 1.f, v_mul_next = 1.f;
  auto fetch_scales = [&](int pair) {
    const int index = 2 * pair + (my_token >> 1);
    k_mul_next = v_mul_next = 1.f;
    if (index < num_pages_here) {
      const unsigned char* at = table_first + index * table_step;
      const int64_t raw = table_elem == 8 ? *reinterpret_cast<const int64_t*>(at)
                                          : static_cast<int64_t>(*reinterpret_cast<const int32_t*>(at));
      if (static_cast<uint64_t>(raw) < static_cast<uint64_t>(pool_pages)) {
        k_mul_next = p.k_scale[raw * p.kv_heads + kv_head];
        v_mul_next = p.v_scale[raw * p.kv_heads + kv_head];
      }
    }
  };
  if (FP8) fetch_scales(0);
  int read_slot = 0;
  const int full_pairs = tokens_here >> 5;
  for (int pair = 0; pair < num_pairs; ++pair) {
    if (PROFILE) t_mark = clock64();
    wait_oldest_pair();      // this thread's copies of `pair` have landed
    twin_barrier(warp & 3);  // so have the twin's; and the twin is done with the previous slot
    if (PROFILE) t_wait += clock64() - t_mark;
    issue_pair();            // refill the slot both twins have just left
    if (FP8) {
      k_mul = k_mul_next, v_mul = v_mul_next;
      fetch_scales(pair + 1);
    }
    const unsigned char* slot = smem + read_slot * Traits::kSlotBytes + chunk_offset;
    read_slot = (read_slot + 1) & (kSlots - 1);

    // Pairs below `full_pairs` hold 32 existing tokens; only the partition's last
    // pair can hold tokens past the sequence end or lack its second page.
    attend_pair<T, FP8>(slot, prob_slot + (pair & 1) * kProbParityStride, role, q2, acc, my_offset,
                        my_sum, pair < full_pairs, pair * 2 * QF_PAGE_SIZE + row, tokens_here, k_mul,
                        v_mul);
  }
  long long t_loop_end = 0;
  if (PROFILE) t_loop_end = clock64();

  // ------------------------------ CTA merge -------------------------------
  // Barrier: every slot has been read, so the ring is free for the merge.
  wait_all_copies();
  __syncthreads();
  const int64_t head0 = static_cast<int64_t>(kv_head) * QF_GQA_GROUP;
  const int64_t partial_row =
      (static_cast<int64_t>(sequence) * p.split_k + split) * p.q_heads + head0;
  merge_and_store<T>(
      merge_state, reinterpret_cast<float*>(smem), acc, my_offset, my_sum, my_token, my_head,
      p.partial_out != nullptr ? p.partial_out + partial_row * QF_HEAD_DIM : nullptr,
      p.partial_max != nullptr ? p.partial_max + partial_row : nullptr,
      p.partial_max != nullptr ? p.partial_sum + partial_row : nullptr,
      p.out != nullptr ? static_cast<T*>(p.out) + sequence * p.o_sb + head0 * p.o_sh : nullptr, p.o_sh,
      p.o_sd);
  if (PROFILE && p.cycles != nullptr && tid == 32) {
    // One warp per CTA reports {waiting for pages, page loop, set-up before it, merge after it}.
    long long* dst = p.cycles + static_cast<int64_t>(blockIdx.x) * 4;
    dst[0] = t_wait, dst[1] = t_loop_end - t_total, dst[2] = t_total - t_entry, dst[3] = clock64() - t_loop_end;
  }
}

}  // namespace
}  // namespace qf
