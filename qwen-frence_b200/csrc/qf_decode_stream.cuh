// Persistent ("streamed") split-K partial kernel of GQA paged decode attention for
// sm_100a, same geometry and per-pair math as qf_decode_partial.cuh.
//
// Why a second kernel.  With one CTA per (sequence, KV head, split) a decode batch
// of mixed lengths becomes thousands of short CTAs, and each of them pays a chain
// of dependent global reads before its first page arrives (sequence length ->
// page ids -> pages, about a microsecond each under load) plus a merge at the
// end; on 2K-token sequences split ten ways that is a third of a CTA's life.
// Here the launch has a fixed number of resident CTAs per KV head, and the CTAs of
// a head cut the concatenated page-pair list of ALL sequences into equal
// contiguous shares:
//
//   * every CTA reads all sequence lengths once, builds the exclusive prefix of
//     page pairs in shared memory and finds its own share [begin, begin + count);
//     the dependent chain is paid once per CTA, not once per partition;
//   * the share is walked pair by pair across sequence boundaries; the copy ring
//     never drains: while the math finishes one sequence, the copies (and page
//     ids) of the next are already in flight, and so are its Q rows during the
//     merge;
//   * a stretch of one sequence inside one share is a "piece".  Piece j of a
//     sequence (counted from the CTA that holds its first pair) is stored in
//     split slot j of the caller's partial buffers; the share is never smaller
//     than ceil(longest sequence / (split_k - 1)) pairs, so no sequence has more
//     than split_k pieces.  The CTA that finishes a sequence marks the next slot
//     (if any) with sum = -1; the combine stops there;
//   * CTA c of KV head 0 and CTA c of KV head 1 walk the same pages at the same
//     pace, so the two 256-byte halves of a 512-byte token row are fetched close
//     together in time.
//
// Split boundaries therefore depend on the whole batch, not only on the sequence
// (results agree with the per-partition kernel to fp32 rounding, not bit for bit),
// and the partial buffers hold pieces, not the reference's balanced partitions:
// callers that want those use the per-partition kernel.
#pragma once

#include "qf_decode_partial.cuh"

namespace qf {
namespace {

constexpr int kMaxStreamBatch = 1024;                            // sequences whose prefix fits in shared memory
constexpr int kScanPerThread = kMaxStreamBatch / kFastThreads;   // consecutive sequences a thread scans
constexpr int kMaxStreamLen = 0x7fffff00;                        // keeps (len + 31) inside int

struct StreamParams {
  FastParams f;
  int ctas_per_head;  // resident CTAs that share one KV head's pair list
  // Tensor-core kernel only.  Nonzero: the caller promises that, of the pages this launch
  // reads, only each sequence's last one (the page of its newest token) can be written by a
  // kernel still in flight when this one starts; K / V tiles of the other pages may then be
  // requested before the dependency wait.
  int early_tiles;
};

// The launch-wide work list in shared memory: sequences in units of
// `kUnitTokens` tokens (a page pair here, a page in the tensor-core kernel).
struct WorkList {
  int first_unit[kMaxStreamBatch + 1];  // exclusive prefix of units over sequences; [kMaxStreamBatch] = total
  int length[kMaxStreamBatch];          // clamped sequence lengths
  int warp_total[kFastThreads / 32];
  int warp_longest[kFastThreads / 32];
};

// Every thread of a kFastThreads-wide CTA calls this once (it has two CTA-wide
// barriers); returns the longest sequence in units.  The total is
// list.first_unit[kMaxStreamBatch].  A sequence with tokens counts
// sequence_overhead<kOverheadUnits>(data units) extra units in front of its data
// units: they stand for the fixed cost a CTA pays per sequence, so that equal shares
// of units are equal shares of time.
// Empty units in front of a sequence of `data_units`: kOverheadUnits, but at most a
// quarter of the sequence (short sequences cost less than the flat figure, and a
// run of mostly empty units would leave some warps of a CTA without pages).
template <int kOverheadUnits>
__host__ __device__ __forceinline__ int sequence_overhead(int data_units) {
  return kOverheadUnits < data_units / 4 ? kOverheadUnits : data_units / 4;
}

template <int kUnitTokens, int kOverheadUnits = 0>
__device__ __forceinline__ int build_work_list(WorkList& list, const void* seq_lens, int lens_dtype,
                                               int64_t lens_stride, int batch, int max_tokens) {
  constexpr unsigned kFull = 0xffffffffu;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int running = 0, longest = 0;
  int before[kScanPerThread];
#pragma unroll
  for (int i = 0; i < kScanPerThread; ++i) {
    const int b = tid * kScanPerThread + i;
    int len = 0;
    if (b < batch) {
      int64_t raw = load_index(seq_lens, lens_dtype, b * lens_stride);
      raw = raw < 0 ? 0 : raw;
      len = static_cast<int>(raw > max_tokens ? max_tokens : raw);  // never read past the table row
    }
    list.length[b] = len;
    const int data_units = (len + kUnitTokens - 1) / kUnitTokens;
    const int units = data_units + sequence_overhead<kOverheadUnits>(data_units);
    before[i] = running;
    running += units;
    longest = max(longest, units);
  }
  int inclusive = running;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int up = __shfl_up_sync(kFull, inclusive, off);
    if (lane >= off) inclusive += up;
    longest = max(longest, __shfl_xor_sync(kFull, longest, off));
  }
  if (lane == 31) list.warp_total[warp] = inclusive, list.warp_longest[warp] = longest;
  __syncthreads();
  int base = inclusive - running;  // units of earlier threads of this warp
  for (int w = 0; w < warp; ++w) base += list.warp_total[w];
#pragma unroll
  for (int i = 0; i < kScanPerThread; ++i) list.first_unit[tid * kScanPerThread + i] = base + before[i];
  if (tid == kFastThreads - 1) list.first_unit[kMaxStreamBatch] = base + running;
  __syncthreads();
  longest = 0;
#pragma unroll
  for (int w = 0; w < kFastThreads / 32; ++w) longest = max(longest, list.warp_longest[w]);
  return longest;
}

// The last sequence whose first unit is <= `unit` (it is not empty when `unit` is
// below the total, because the next prefix is larger).
__device__ __forceinline__ int sequence_of_unit(const WorkList& list, int batch, int unit) {
  int lo = 0, hi = batch - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (list.first_unit[mid] <= unit) lo = mid; else hi = mid - 1;
  }
  return lo;
}

template <typename T, bool FP8>
__global__ void __launch_bounds__(kFastThreads, QF_MIN_CTAS)
    decode_stream_kernel(const StreamParams sp) {
  using Traits = TileTraits<T, FP8>;
  const FastParams& p = sp.f;
  // ring of page-pair slots, then kMergeFloats of merge scratch
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(16) float2 prob_pairs[2][kConsumerWarps][2][12];
  __shared__ MergeShared merge_state;
  __shared__ WorkList work;  // units are page pairs

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int sub = lane & 15;
  const int head_group = warp >> 2;
  const int row = ((warp & 3) << 1) | (lane >> 4);
  const int kv_head = blockIdx.x / sp.ctas_per_head;
  const int cta = blockIdx.x - kv_head * sp.ctas_per_head;

  // ---- the pair list of this launch: prefix over sequences, total, longest ----
  const int longest =
      build_work_list<2 * QF_PAGE_SIZE>(work, p.seq_lens, p.lens_dtype, p.lens_stride, p.batch, p.max_tokens);
  const int* first_pair = work.first_unit;
  const int* length = work.length;
  const int total = first_pair[kMaxStreamBatch];
  if (total == 0) return;
  // Pairs per CTA: an equal share, but never so small that a sequence would be cut
  // into more pieces than there are split slots.
  const int share = max((total + sp.ctas_per_head - 1) / sp.ctas_per_head,
                        (longest + p.split_k - 2) / (p.split_k - 1));
  const int begin = cta * share;
  if (begin >= total) return;
  const int count = min(share, total - begin);

  const int start_seq = sequence_of_unit(work, p.batch, begin);  // holds pair `begin`
  const int start_pair = begin - first_pair[start_seq];  // first pair of the share, within its sequence

  // ---- loads: as in the per-partition kernel, but the fetch cursor crosses sequences ----
  const int pool_pages = static_cast<int>(p.num_pages);
  const unsigned char* pool = head_group == 0 ? p.k_pool : p.v_pool;
  const int64_t page_bytes = head_group == 0 ? p.k_page_bytes : p.v_page_bytes;
  const int64_t tok_bytes = head_group == 0 ? p.k_tok_bytes : p.v_tok_bytes;
  const unsigned char* pool_row =
      pool + row * tok_bytes + kv_head * (head_group == 0 ? p.k_head_bytes : p.v_head_bytes) +
      sub * Traits::kChunkBytes;
  const int chunk_offset = (((warp & 3) << 5) | lane) * Traits::kChunkBytes;
  constexpr int kRowPlus8 = 8 * 16 * Traits::kChunkBytes;
  const int fill_offset = head_group * 2 * Traits::kTileBytes + chunk_offset;
  const int table_elem = p.table_dtype == QF_INDEX_I64 ? 8 : 4;
  const int64_t table_step = p.bt_sp * table_elem;
  const int64_t table_row_step = p.bt_sb * table_elem;
  const unsigned char* table_base = static_cast<const unsigned char*>(p.block_table);

  // Page id stored at `at`: -1 when the page does not exist, -2 when the id lies
  // outside the pool (reported when the pair is issued, never dereferenced).
  auto read_id = [&](const unsigned char* at, bool exists) -> int {
    if (!exists) return -1;
    const int64_t raw = table_elem == 8 ? *reinterpret_cast<const int64_t*>(at)
                                        : static_cast<int64_t>(*reinterpret_cast<const int32_t*>(at));
    return static_cast<uint64_t>(raw) < static_cast<uint64_t>(pool_pages) ? static_cast<int>(raw) : -2;
  };
  auto copy_page = [&](unsigned char* dst, int page_id) {
    if (page_id >= 0) {
      const unsigned char* src = pool_row + static_cast<int64_t>(page_id) * page_bytes;
      copy_chunk_async<FP8>(dst, src);
      copy_chunk_async<FP8>(dst + kRowPlus8, src + 8 * tok_bytes);
    } else {
      if (page_id == -2) atomicMax(p.status, kStatusBadPageId);
      if constexpr (FP8) {
        *reinterpret_cast<uint2*>(dst) = make_uint2(0u, 0u);
        *reinterpret_cast<uint2*>(dst + kRowPlus8) = make_uint2(0u, 0u);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(dst + kRowPlus8) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };

  // Fetch cursor: the pair whose page ids are read next.
  int fetch_seq = start_seq;
  int fetch_in_piece;  // pairs of the current piece whose ids have not been read
  int fetch_after;     // pairs of the share after the current piece
  int fetch_pages;     // pages of the current sequence from the next pair on
  const unsigned char* table_next;
  {
    const int in_sequence = first_pair[start_seq + 1] - first_pair[start_seq] - start_pair;
    fetch_in_piece = min(in_sequence, count);
    fetch_after = count - fetch_in_piece;
    fetch_pages = (length[start_seq] + QF_PAGE_SIZE - 1) / QF_PAGE_SIZE - 2 * start_pair;
    table_next = table_base + start_seq * table_row_step + 2 * start_pair * table_step;
  }
  int next_id_a = -1, next_id_b = -1;
  auto fetch_ids = [&]() {
    if (fetch_in_piece <= 0 && fetch_after > 0) {
      // the next sequence that has pages (one exists, because pairs remain)
      do {
        ++fetch_seq;
      } while (fetch_seq < p.batch - 1 && first_pair[fetch_seq + 1] == first_pair[fetch_seq]);
      const int pairs = first_pair[fetch_seq + 1] - first_pair[fetch_seq];
      fetch_in_piece = min(pairs, fetch_after);
      fetch_after -= fetch_in_piece;
      fetch_pages = (length[fetch_seq] + QF_PAGE_SIZE - 1) / QF_PAGE_SIZE;
      table_next = table_base + fetch_seq * table_row_step;
    }
    const bool any = fetch_in_piece > 0;
    next_id_a = read_id(table_next, any && fetch_pages > 0);
    next_id_b = read_id(table_next + table_step, any && fetch_pages > 1);
    table_next += 2 * table_step;
    fetch_pages -= 2;
    --fetch_in_piece;
  };
  int pairs_to_issue = count;
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
    // Prologue: ids of the first kDepth + 1 pairs in one round trip, then kDepth pairs in flight.
    int ids_a[kDepth + 1], ids_b[kDepth + 1];
#pragma unroll
    for (int i = 0; i <= kDepth; ++i) {
      fetch_ids();
      ids_a[i] = next_id_a, ids_b[i] = next_id_b;
    }
#pragma unroll
    for (int i = 0; i < kDepth; ++i) {
      if (i < count) {
        unsigned char* dst = smem + i * Traits::kSlotBytes + fill_offset;
        copy_page(dst, ids_a[i]);
        copy_page(dst + Traits::kTileBytes, ids_b[i]);
      }
      commit_copies();
    }
    fill_slot = kDepth & (kSlots - 1);
    pairs_to_issue = max(count - kDepth, 0);
    next_id_a = ids_a[kDepth], next_id_b = ids_b[kDepth];
  }

  // ---- per-thread state ----
  float2 q2[kHeadsPerThread][4];
  float2 acc[kHeadsPerThread][4];
  uint4 q_raw[kHeadsPerThread];
  auto load_q = [&](int sequence) {
    const T* qbase = static_cast<const T*>(p.q) + sequence * p.q_sb +
                     (static_cast<int64_t>(kv_head) * QF_GQA_GROUP + head_group * kHeadsPerThread) * p.q_sh +
                     sub * 8;
#pragma unroll
    for (int h = 0; h < kHeadsPerThread; ++h) q_raw[h] = *reinterpret_cast<const uint4*>(qbase + h * p.q_sh);
  };
  auto scale_q = [&]() {
    const float2 s2 = make_float2(p.scale_log2, p.scale_log2);
#pragma unroll
    for (int h = 0; h < kHeadsPerThread; ++h) {
      q2[h][0] = __fmul2_rn(unpack2<T>(q_raw[h].x), s2);
      q2[h][1] = __fmul2_rn(unpack2<T>(q_raw[h].y), s2);
      q2[h][2] = __fmul2_rn(unpack2<T>(q_raw[h].z), s2);
      q2[h][3] = __fmul2_rn(unpack2<T>(q_raw[h].w), s2);
    }
  };
  const LaneRole<T, FP8> role(sub, row);
  float2* prob_slot = &prob_pairs[0][warp][lane >> 4][0];
  constexpr int kProbParityStride = kConsumerWarps * 2 * 12;  // float2 elements
  float* merge = reinterpret_cast<float*>(smem + kSlots * Traits::kSlotBytes);

  // Math cursor: the piece being computed.
  int piece_seq = start_seq;
  int piece_first = start_pair;  // first pair of the piece within its sequence
  int piece_pairs = min(first_pair[start_seq + 1] - first_pair[start_seq] - start_pair, count);
  int pairs_after = count - piece_pairs;
  int read_slot = 0;
  load_q(piece_seq);

  while (true) {
    scale_q();
#pragma unroll
    for (int h = 0; h < kHeadsPerThread; ++h)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[h][j] = make_float2(0.f, 0.f);
    float my_offset = -INFINITY, my_sum = 0.f;
    // Tokens of the sequence from the piece's first pair on; pairs below
    // `full_pairs` hold 32 existing tokens.
    const int tokens_here = length[piece_seq] - piece_first * 2 * QF_PAGE_SIZE;
    const int full_pairs = tokens_here >> 5;

    // FP8: scales of the page that holds this lane's token, fetched a pair ahead.
    float k_mul = 1.f, v_mul = 1.f, k_mul_next = 1.f, v_mul_next = 1.f;
    const unsigned char* piece_table =
        table_base + piece_seq * table_row_step + 2 * piece_first * table_step;
    const int piece_pages = (tokens_here + QF_PAGE_SIZE - 1) / QF_PAGE_SIZE;
    auto fetch_scales = [&](int pair) {
      const int index = 2 * pair + (role.my_token >> 1);
      k_mul_next = v_mul_next = 1.f;
      if (pair < piece_pairs && index < piece_pages) {
        const int id = read_id(piece_table + index * table_step, true);
        if (id >= 0) {
          k_mul_next = p.k_scale[static_cast<int64_t>(id) * p.kv_heads + kv_head];
          v_mul_next = p.v_scale[static_cast<int64_t>(id) * p.kv_heads + kv_head];
        }
      }
    };
    if (FP8) fetch_scales(0);

    for (int pair = 0; pair < piece_pairs; ++pair) {
      wait_oldest_pair();      // this thread's copies of the pair have landed
      twin_barrier(warp & 3);  // so have the twin's; and the twin is done with the previous slot
      issue_pair();            // refill the slot both twins have just left
      if (FP8) {
        k_mul = k_mul_next, v_mul = v_mul_next;
        fetch_scales(pair + 1);
      }
      const unsigned char* slot = smem + read_slot * Traits::kSlotBytes + chunk_offset;
      attend_pair<T, FP8>(slot, prob_slot + (read_slot & 1) * kProbParityStride, role, q2, acc,
                          my_offset, my_sum, pair < full_pairs, pair * 2 * QF_PAGE_SIZE + row,
                          tokens_here, k_mul, v_mul);
      read_slot = (read_slot + 1) & (kSlots - 1);
    }

    // ---- the piece is done: where it goes, what comes next ----
    const int done_seq = piece_seq;
    const int sequence_pairs = first_pair[done_seq + 1] - first_pair[done_seq];
    const bool sequence_ends = piece_first + piece_pairs >= sequence_pairs;
    const int split_slot = cta - first_pair[done_seq] / share;
    bool more = pairs_after > 0;
    if (more) {
      do {
        ++piece_seq;
      } while (piece_seq < p.batch - 1 && first_pair[piece_seq + 1] == first_pair[piece_seq]);
      piece_first = 0;
      piece_pairs = min(first_pair[piece_seq + 1] - first_pair[piece_seq], pairs_after);
      pairs_after -= piece_pairs;
      // A sequence without pairs cannot come up while pairs remain; the test keeps
      // the loop bounded whatever the prefix holds.
      more = piece_pairs > 0;
    }
    if (more) load_q(piece_seq);  // in flight during the merge
    const int64_t partial_row =
        (static_cast<int64_t>(done_seq) * p.split_k + split_slot) * p.q_heads +
        static_cast<int64_t>(kv_head) * QF_GQA_GROUP;
    const bool slot_ok = split_slot >= 0 && split_slot < p.split_k;  // holds by the choice of `share`
    merge_and_store<T>(merge_state, merge, acc, my_offset, my_sum, role.my_token, role.my_head,
                       slot_ok ? p.partial_out + partial_row * QF_HEAD_DIM : nullptr,
                       slot_ok ? p.partial_max + partial_row : nullptr,
                       slot_ok ? p.partial_sum + partial_row : nullptr, static_cast<T*>(nullptr), 0, 0);
    if (sequence_ends && split_slot + 1 < p.split_k && slot_ok && tid < QF_GQA_GROUP) {
      p.partial_sum[partial_row + p.q_heads + tid] = -1.f;  // no further pieces of this sequence
    }
    if (!more) break;
  }
  wait_all_copies();
}

}  // namespace
}  // namespace qf
