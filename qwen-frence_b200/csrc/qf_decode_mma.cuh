// Tensor-core split-K partial kernel of GQA paged decode attention for sm_100a:
// persistent CTAs over the batch's page list (the scheduling of
// qf_decode_stream.cuh, in units of pages), warp-level MMA for the math.
//
// Why tensor cores for a bandwidth-bound op.  On CUDA cores one page pair costs
// about 3 400 warp instructions (fp16 -> fp32 conversions, packed FMAs, the
// shuffle reduction), and once the per-partition set-up latencies are gone that
// instruction stream, not HBM, is the limit.  Here a page of one KV head costs
// about a hundred: the arithmetic intensity is still 6 flop/byte, the MMA only
// takes the conversions and FMAs off the issue slots.
//
// Shapes.  The GQA group has 6 query heads, so heads cannot fill an MMA's M = 16;
// tokens can.  A warp computes, for one page (16 tokens) at a time,
//     S^T [16 tokens x 8 heads]  = K [16 x 128] . Q^T [128 x 8]      (8 x m16n8k16)
//     O^T [128 dims x 8 heads]  += V^T [128 x 16] . P^T [16 x 8]     (8 x m16n8k16)
// with heads 6, 7 zero padding (6/8 of the MMA useful).  K is the A operand
// straight from shared memory (ldmatrix), Q^T the B operand held in 16 registers
// for the whole piece, V^T the A operand through ldmatrix.trans, and P^T becomes
// a B operand with two movmatrix transposes of the packed probabilities.  The
// accumulators of S^T and O^T both give a thread heads (2q, 2q+1), q = lane % 4,
// so the online softmax rescale needs no shuffle; its offset only moves when a
// score exceeds it by 2^8, as in the CUDA-core kernels.
//
// Loads.  Every warp owns pages begin + warp, begin + warp + 8, ... of the CTA's
// share and a private ring of five 4 KB tiles (K and V tiles of consecutive pages
// alternate), filled by 16-byte cp.async with an XOR swizzle so that ldmatrix is
// bank-conflict free; four tiles (16 KB per warp, 128 KB per SM) are in flight
// ahead of the math, and nothing but cp.async.wait_group and __syncwarp orders
// them: no barrier inside a piece, no spin wait anywhere.  Rows past the end of a
// sequence are written as zeros instead of copied, so that no NaN from an unused
// cache row reaches an MMA.  Page ids, and the rows a page holds, sit in lane
// registers, 32 pages per warp at a time, fetched a chunk ahead.
//
// Pieces, split slots and the end-of-sequence mark are those of the streamed
// CUDA-core kernel, and so is the combine.
#pragma once

#include "qf_decode_stream.cuh"

namespace qf {
namespace {

constexpr int kMmaWarps = kFastThreads / 32;                   // 8
constexpr int kTileBytes16 = QF_PAGE_SIZE * QF_HEAD_DIM * 2;   // K or V of one page and KV head: 4 KB
constexpr int kRingTiles = 5;                                  // per warp
constexpr int kTilesAhead = 4;                                 // in flight ahead of the math
constexpr int kPaddedHeads = 8;
constexpr int kMmaMergeFloats = kMmaWarps * QF_HEAD_DIM * kPaddedHeads;  // 32 KB

template <typename T>
struct MmaOps;
template <>
struct MmaOps<__half> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};
template <>
struct MmaOps<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}
// Transpose an 8x8 matrix of 16-bit elements held one 32-bit pair per lane.
__device__ __forceinline__ uint32_t transpose_8x8(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ void wait_tiles_ahead() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kTilesAhead - 1) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kFastThreads, 1) decode_mma_kernel(const StreamParams sp) {
  using Ops = MmaOps<T>;
  const FastParams& p = sp.f;
  // [kMmaWarps][kRingTiles] tiles of 4 KB, then kMmaMergeFloats of merge scratch
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ WorkList work;  // units are pages
  __shared__ float warp_offset[kMmaWarps][kPaddedHeads];
  __shared__ float warp_sum[kMmaWarps][kPaddedHeads];

  constexpr unsigned kFull = 0xffffffffu;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int g = lane >> 2;  // MMA fragment row group
  const int q = lane & 3;   // MMA fragment column pair: heads 2q, 2q + 1
  const int kv_head = blockIdx.x / sp.ctas_per_head;
  const int cta = blockIdx.x - kv_head * sp.ctas_per_head;

  // ---- the page list of this launch and this CTA's share of it ----
  const int longest = build_work_list<QF_PAGE_SIZE>(work, p.seq_lens, p.lens_dtype, p.lens_stride, p.batch);
  const int* first_page = work.first_unit;
  const int total = first_page[kMaxStreamBatch];
  if (total == 0) return;
  const int share = max((total + sp.ctas_per_head - 1) / sp.ctas_per_head,
                        (longest + p.split_k - 2) / (p.split_k - 1));
  const int begin = cta * share;
  if (begin >= total) return;
  const int count = min(share, total - begin);
  const int end = begin + count;
  // This warp's pages: begin + warp + 8 k, k = 0 .. my_pages - 1.
  const int my_pages = count > warp ? (count - warp + kMmaWarps - 1) / kMmaWarps : 0;

  // ---- loads ----
  const int pool_pages = static_cast<int>(p.num_pages);
  const int table_elem = p.table_dtype == QF_INDEX_I64 ? 8 : 4;
  const unsigned char* table_base = static_cast<const unsigned char*>(p.block_table);
  const unsigned char* k_base = p.k_pool + kv_head * p.k_head_bytes + (lane & 15) * 16;
  const unsigned char* v_base = p.v_pool + kv_head * p.v_head_bytes + (lane & 15) * 16;
  unsigned char* ring = smem + warp * (kRingTiles * kTileBytes16);
  // A lane copies the 16-byte chunk (lane % 16) of rows 2j + lane / 16, j = 0..7; chunk c
  // of row r is stored at chunk c ^ (r % 8) of the row's 256 bytes.
  int fill_offset[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int r = 2 * j + (lane >> 4);
    fill_offset[j] = r * 256 + (((lane & 15) ^ (r & 7)) << 4);
  }

  // Page ids and row counts of 32 of this warp's pages at a time, one per lane.
  auto describe = [&](int chunk, int& id, int& rows) {
    const int k = chunk * 32 + lane;
    id = -1, rows = 0;
    if (k < my_pages) {
      const int page = begin + warp + kMmaWarps * k;
      const int sequence = sequence_of_unit(work, p.batch, page);
      const int in_sequence = page - first_page[sequence];
      const unsigned char* at =
          table_base + (sequence * p.bt_sb + static_cast<int64_t>(in_sequence) * p.bt_sp) * table_elem;
      const int64_t raw = table_elem == 8 ? *reinterpret_cast<const int64_t*>(at)
                                          : static_cast<int64_t>(*reinterpret_cast<const int32_t*>(at));
      id = static_cast<uint64_t>(raw) < static_cast<uint64_t>(pool_pages) ? static_cast<int>(raw) : -2;
      rows = min(QF_PAGE_SIZE, work.length[sequence] - in_sequence * QF_PAGE_SIZE);
    }
  };
  int id_now, rows_now, id_next, rows_next;
  describe(0, id_now, rows_now);
  describe(1, id_next, rows_next);

  // Tile t of this warp is K (t even) or V (t odd) of its page t / 2, in ring slot t % 5.
  int fill_tile = 0, fill_slot = 0;
  auto issue_tile = [&]() {
    const int k = fill_tile >> 1;
    if (k < my_pages) {
      if ((fill_tile & 1) == 0 && (k & 31) == 0 && k > 0) {
        id_now = id_next, rows_now = rows_next;
        describe((k >> 5) + 1, id_next, rows_next);
      }
      const int id = __shfl_sync(kFull, id_now, k & 31);
      int rows = __shfl_sync(kFull, rows_now, k & 31);
      if (id < 0) {
        rows = 0;  // bad or missing id: the page reads as zeros
        if (id == -2 && lane == 0) atomicExch(p.status, kStatusBadPageId);
      }
      const bool is_v = fill_tile & 1;
      const unsigned char* src = (is_v ? v_base : k_base) +
                                 static_cast<int64_t>(id < 0 ? 0 : id) * (is_v ? p.v_page_bytes : p.k_page_bytes);
      const int64_t tok_bytes = is_v ? p.v_tok_bytes : p.k_tok_bytes;
      unsigned char* dst = ring + fill_slot * kTileBytes16;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int r = 2 * j + (lane >> 4);
        unsigned char* to = dst + fill_offset[j & 3] + (j >> 2) * (8 * 256);
        if (r < rows) {
          copy_chunk_async<false>(to, src + r * tok_bytes);
        } else {
          *reinterpret_cast<uint4*>(to) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
    commit_copies();  // always, so that group counting stays uniform
    ++fill_tile;
    fill_slot = fill_slot == kRingTiles - 1 ? 0 : fill_slot + 1;
  };
#pragma unroll
  for (int i = 0; i < kTilesAhead; ++i) issue_tile();

  // ---- fragments ----
  // ldmatrix row addresses inside a tile.  K (A = K tile, k-step s covers dims 16 s ..):
  // matrix i = lane / 8 holds rows 8 (i & 1) .., chunk 2 s + (i >> 1).  V (A = V^T, m-tile j
  // covers dims 16 j ..): matrix i holds token rows 8 (i >> 1) .., chunk 2 j + (i & 1).
  const int mat = lane >> 3;
  const uint32_t k_row_offset = ((lane & 7) + 8 * (mat & 1)) * 256;
  const uint32_t k_chunk_xor = ((mat >> 1) ^ (lane & 7)) << 4;
  const uint32_t v_row_offset = ((lane & 7) + 8 * (mat >> 1)) * 256;
  const uint32_t v_chunk_xor = ((mat & 1) ^ (lane & 7)) << 4;
  const uint32_t ring_addr = smem_u32(ring);

  uint32_t q_frag[8][2];  // B operand Q^T: [k-step][dims 2q.. | dims 8 + 2q..] of head g (0 for g >= 6)
  auto load_q = [&](int sequence) {
    const T* row = static_cast<const T*>(p.q) + sequence * p.q_sb +
                   (static_cast<int64_t>(kv_head) * QF_GQA_GROUP + (g < QF_GQA_GROUP ? g : 0)) * p.q_sh + 2 * q;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const uint32_t lo = *reinterpret_cast<const uint32_t*>(row + 16 * s);
      const uint32_t hi = *reinterpret_cast<const uint32_t*>(row + 16 * s + 8);
      q_frag[s][0] = g < QF_GQA_GROUP ? lo : 0u;
      q_frag[s][1] = g < QF_GQA_GROUP ? hi : 0u;
    }
  };

  float* merge = reinterpret_cast<float*>(smem + kMmaWarps * kRingTiles * kTileBytes16);
  float acc[8][4];  // O^T: [m-tile j][(dim 16j+g, head 2q) (16j+g, 2q+1) (16j+g+8, 2q) (16j+g+8, 2q+1)]

  int piece_seq = sequence_of_unit(work, p.batch, begin);
  int page = begin + warp;  // global index of this warp's next page
  int read_slot = 0;
  load_q(piece_seq);

  while (true) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
    float offset[2] = {-INFINITY, -INFINITY};  // of heads 2q, 2q+1 (log2 units), equal in all lanes of a q
    float sum[2] = {0.f, 0.f};                 // over this lane's tokens
    const int seq_first = first_page[piece_seq];
    const int seq_len = work.length[piece_seq];
    const int piece_end = min(first_page[piece_seq + 1], end);

    for (; page < piece_end; page += kMmaWarps) {
      // ---- scores S^T = K Q^T ----
      wait_tiles_ahead();
      __syncwarp();
      issue_tile();
      const uint32_t k_tile = ring_addr + read_slot * kTileBytes16 + k_row_offset;
      read_slot = read_slot == kRingTiles - 1 ? 0 : read_slot + 1;
      float s_even[4] = {0.f, 0.f, 0.f, 0.f}, s_odd[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        uint32_t a[4];
        ldmatrix_x4(a, k_tile + ((32u * s) ^ k_chunk_xor));
        Ops::mma((s & 1) ? s_odd : s_even, a, q_frag[s][0], q_frag[s][1]);
      }
      // score[i]: i = 0 (token g, head 2q), 1 (g, 2q+1), 2 (g+8, 2q), 3 (g+8, 2q+1)
      float score[4];
      const int rows = seq_len - (page - seq_first) * QF_PAGE_SIZE;  // tokens of the page that exist (>= 1)
      const bool valid_lo = g < rows, valid_hi = g + 8 < rows;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        score[i] = (s_even[i] + s_odd[i]) * p.scale_log2;
        if (!(i < 2 ? valid_lo : valid_hi)) score[i] = -INFINITY;
      }
      const bool grow = fmaxf(score[0], score[2]) > offset[0] + kOffsetSlack ||
                        fmaxf(score[1], score[3]) > offset[1] + kOffsetSlack;
      if (__any_sync(kFull, grow)) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float top = fmaxf(score[h], score[h + 2]);
          top = fmaxf(top, __shfl_xor_sync(kFull, top, 4));
          top = fmaxf(top, __shfl_xor_sync(kFull, top, 8));
          top = fmaxf(top, __shfl_xor_sync(kFull, top, 16));
          const float target = fmaxf(offset[h], top);
          const float corr = offset[h] == -INFINITY ? 0.f : fast_exp2(offset[h] - target);
          offset[h] = target;
          sum[h] *= corr;
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j][h] *= corr, acc[j][h + 2] *= corr;
        }
      }
      float prob[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        prob[i] = (i < 2 ? valid_lo : valid_hi) ? fast_exp2(score[i] - offset[i & 1]) : 0.f;
        sum[i & 1] += prob[i];
      }
      // P^T as B operand: [k = tokens 2q.. | 8 + 2q..][n = head g]
      const uint32_t p_lo = transpose_8x8(Ops::pack(prob[0], prob[1]));
      const uint32_t p_hi = transpose_8x8(Ops::pack(prob[2], prob[3]));

      // ---- values O^T += V^T P^T ----
      wait_tiles_ahead();
      __syncwarp();
      issue_tile();
      const uint32_t v_tile = ring_addr + read_slot * kTileBytes16 + v_row_offset;
      read_slot = read_slot == kRingTiles - 1 ? 0 : read_slot + 1;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t a[4];
        ldmatrix_x4_trans(a, v_tile + ((32u * j) ^ v_chunk_xor));
        Ops::mma(acc[j], a, p_lo, p_hi);
      }
    }

    // ---- the piece is done: where it goes, what comes next ----
    const int done_seq = piece_seq;
    const bool sequence_ends = first_page[done_seq + 1] <= end;
    const int split_slot = cta - seq_first / share;
    bool more = piece_end < end;
    if (more) {
      do {
        ++piece_seq;
      } while (piece_seq < p.batch - 1 && first_page[piece_seq + 1] == first_page[piece_seq]);
      // A sequence without pages cannot come up while pages remain; the test keeps
      // the loop bounded whatever the prefix holds.
      more = first_page[piece_seq + 1] > first_page[piece_seq] && first_page[piece_seq] >= piece_end;
    }
    if (more) load_q(piece_seq);  // in flight during the merge

    // ---- merge the eight warps' states and store the piece ----
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float total = sum[h];
      total += __shfl_xor_sync(kFull, total, 4);
      total += __shfl_xor_sync(kFull, total, 8);
      total += __shfl_xor_sync(kFull, total, 16);
      if (g == 0) warp_offset[warp][2 * q + h] = offset[h], warp_sum[warp][2 * q + h] = total;
    }
    __syncthreads();
    float piece_offset[2], factor[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float top = -INFINITY;
#pragma unroll
      for (int w = 0; w < kMmaWarps; ++w) top = fmaxf(top, warp_offset[w][2 * q + h]);
      piece_offset[h] = top;
      factor[h] = offset[h] == -INFINITY ? 0.f : fast_exp2(offset[h] - top);
    }
    // scratch [warp][dim][8 heads]: a lane stores heads (2q, 2q+1) of dims 16j+g, 16j+g+8
    float* mine = merge + warp * (QF_HEAD_DIM * kPaddedHeads);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      *reinterpret_cast<float2*>(mine + (16 * j + g) * kPaddedHeads + 2 * q) =
          make_float2(acc[j][0] * factor[0], acc[j][1] * factor[1]);
      *reinterpret_cast<float2*>(mine + (16 * j + g + 8) * kPaddedHeads + 2 * q) =
          make_float2(acc[j][2] * factor[0], acc[j][3] * factor[1]);
    }
    __syncthreads();
    const bool slot_ok = split_slot >= 0 && split_slot < p.split_k;  // holds by the choice of `share`
    const int64_t partial_row =
        (static_cast<int64_t>(done_seq) * p.split_k + split_slot) * p.q_heads +
        static_cast<int64_t>(kv_head) * QF_GQA_GROUP;
    if (slot_ok) {
#pragma unroll
      for (int i = 0; i < (QF_GQA_GROUP * QF_HEAD_DIM) / kFastThreads; ++i) {
        const int e = tid + i * kFastThreads;  // (head, dim) flattened
        const int head = e >> 7, d = e & 127;
        float value = 0.f;
#pragma unroll
        for (int w = 0; w < kMmaWarps; ++w) value += merge[(w * QF_HEAD_DIM + d) * kPaddedHeads + head];
        p.partial_out[partial_row * QF_HEAD_DIM + e] = value;
      }
      if (tid < QF_GQA_GROUP) {
        float top = -INFINITY;
        for (int w = 0; w < kMmaWarps; ++w) top = fmaxf(top, warp_offset[w][tid]);
        float total = 0.f;
        for (int w = 0; w < kMmaWarps; ++w) {
          const float mw = warp_offset[w][tid];
          if (mw != -INFINITY) total += warp_sum[w][tid] * fast_exp2(mw - top);
        }
        // natural-log units, as the combine expects
        p.partial_max[partial_row + tid] = top * kLn2;
        p.partial_sum[partial_row + tid] = total;
        if (sequence_ends && split_slot + 1 < p.split_k) {
          p.partial_sum[partial_row + p.q_heads + tid] = -1.f;  // no further pieces of this sequence
        }
      }
    }
    if (!more) break;
    __syncthreads();  // warp_offset / warp_sum / scratch are rewritten by the next piece
  }
  wait_all_copies();
}

}  // namespace
}  // namespace qf
