// Tensor-core split-K partial kernel of GQA paged decode attention for sm_100a:
// persistent CTAs over the batch's page list (the scheduling of
// qf_decode_stream.cuh, in units of pages), warp-level MMA for the math.  Serves
// fp16 / bf16 pools and FP8-e4m3 pools with per-page scales.
//
// Why tensor cores for a bandwidth-bound op.  On CUDA cores one page pair costs
// about 3 400 warp instructions (fp16 -> fp32 conversions, packed FMAs, the
// shuffle reduction), and once the per-partition set-up latencies are gone that
// instruction stream, not HBM, is the limit.  Here a page of one KV head costs
// about 430, most of them copy issue and address arithmetic: the arithmetic
// intensity is still 6 flop/byte, the MMA only takes the conversions and FMAs off
// the issue slots.
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
// Work.  The list the CTAs of a KV head share is in "units": a sequence is up to
// kPieceOverhead empty units followed by its pages, so a CTA whose share holds
// many short sequences gets fewer pages than one whose share is a stretch of one
// long sequence, and they finish together (with equal page counts the former
// finished up to 10 us later: every sequence costs a Q tile, deposits, a merge
// and a store).  Warp w owns units begin + w, begin + w + 8, ... of the CTA's share
// and skips the empty ones.  Pieces, split slots and the end-of-sequence mark are
// those of the streamed CUDA-core kernel, and so is the combine.
//
// Loads.  Every warp has a private ring of five 4 KB tiles (K and V tiles of its
// consecutive pages alternate), filled by 16-byte cp.async with an XOR swizzle so
// that ldmatrix is bank-conflict free; four tiles (16 KB per warp, 128 KB per SM)
// are in flight ahead of the math, and nothing but cp.async.wait_group and
// __syncwarp orders them: no barrier inside a piece.  Rows past the end of a
// sequence are written as zeros instead of copied, so that no NaN from an unused
// cache row reaches an MMA.  Page ids, and the rows a page holds, sit in lane
// registers, 32 units per warp at a time, fetched a chunk ahead.  The Q rows of a
// sequence travel through the same ring, as one more tile in front of the warp's
// first page of that sequence: a plain global load of Q at a sequence boundary
// would queue behind the 128 KB of page traffic the SM has in flight.
//
// Merging a piece has no CTA-wide barrier (a barrier at every sequence boundary
// stalls all eight copy pipelines for the spread between the fastest and the
// slowest warp, measured at 2.2 - 2.7 us per piece): a warp that has finished its
// pages of a piece deposits (accumulator, offset, sum) in shared memory, bumps the
// piece's arrival counter and goes on with the next piece; the warp whose arrival
// completes the count merges the deposits and stores the piece.  Deposits are
// double-buffered by piece parity; before depositing piece r a warp checks that
// piece r - 2 has been merged.  That check can only fail when the warp is two
// sequences ahead of the slowest one; it then polls, for a bounded number of
// rounds, a flag that only depends on warps behind it (the warp that is furthest
// behind never waits, so the poll cannot deadlock); running out of rounds raises
// status 3 and goes on.
//
// The kernel is launched chained to its predecessor (launch_chained): everything up
// to dependency_wait() - the work list, the share, the page ids - runs while the
// RoPE / KV-write kernel before it is still running.
#pragma once

#include <type_traits>

#include "qf_decode_stream.cuh"

namespace qf {
namespace {

constexpr int kMmaWarps = kFastThreads / 32;                   // 8
// Ring geometry.  16-bit pools: K or V of one page and KV head is 4 KB, five slots per
// warp, four tiles in flight, one CTA per SM.  FP8 pools: a tile is 2 KB plus its fp32
// scale (the slot keeps 64 more bytes for it), three slots, two tiles in flight, and
// TWO CTAs per SM: with e4m3 tiles the kernel is bound by instruction latency (the
// conversions make a page cost more instructions, and a page is half the bytes), and
// sixteen warps per SM hide it where eight could not; the FP8 variant compiles to 128
// registers, and 2 x (8 x 3 slots + deposits) fits the shared memory.
template <bool FP8>
struct RingShape {
  static constexpr int kRowBytes = FP8 ? QF_HEAD_DIM : 2 * QF_HEAD_DIM;
  static constexpr int kTileBytes = QF_PAGE_SIZE * kRowBytes;
  // (FP8: the tile's scale rides behind it; the fused step's Q tile and its cos / sin row,
  // 1 632 + 512 bytes, need the slot a little larger than a tile as well)
  static constexpr int kSlotBytes = FP8 ? kTileBytes + 128 : kTileBytes;
  static constexpr int kSlots = FP8 ? 3 : 5;
  static constexpr int kCtasPerSm = FP8 ? 2 : 1;
  static constexpr int kAhead = kSlots - 1;
  static constexpr int kWarpBytes = ((kSlots * kSlotBytes + 127) / 128) * 128;
};
constexpr int kPaddedHeads = 8;
// What a sequence costs a CTA besides its pages (Q tile, deposit, merge, store),
// in pages: shares are equal in pages + min(kPieceOverhead, pages / 4) per sequence.
#ifndef QF_PIECE_OVERHEAD
#define QF_PIECE_OVERHEAD 6
#endif
constexpr int kPieceOverhead = QF_PIECE_OVERHEAD;
constexpr int kQTileBytes = QF_GQA_GROUP * (QF_HEAD_DIM * 2 + 16);  // six padded rows; cos / sin may follow
constexpr int kQRowBytes = QF_HEAD_DIM * 2 + 16;                        // Q tile: head stride, padded against bank conflicts
constexpr int kDepositHeadStride = QF_HEAD_DIM + 8;                      // floats; the pad spreads the heads over banks
constexpr int kDepositFloats = QF_GQA_GROUP * kDepositHeadStride;        // one warp's O^T of a piece: 3.2 KB
constexpr int kMmaMergeFloats = 2 * kMmaWarps * kDepositFloats;          // two piece parities: 48 KB
constexpr int kMergePollRounds = 1 << 22;                                // bound of the (rare) wait for piece r - 2

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
template <int kAhead>
__device__ __forceinline__ void wait_tiles_ahead() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kAhead - 1) : "memory");
}
// Four e4m3 bytes -> 2 x two f16: `lo` from bytes 0, 1 and `hi` from bytes 2, 3 (one
// conversion instruction each).
__device__ __forceinline__ void e4m3x4_to_f16x2x2(uint32_t x, uint32_t& lo, uint32_t& hi) {
  asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}"
      : "=r"(lo), "=r"(hi)
      : "r"(x));
}
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t x) {
  const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x));
  const __half2 h = __floats2half2_rn(f.x, f.y);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Shared-memory flag operations with CTA-scope release / acquire semantics.
__device__ __forceinline__ int add_acq_rel(int* counter, int value) {
  int old;
  asm volatile("atom.acq_rel.cta.shared.add.u32 %0, [%1], %2;"
               : "=r"(old) : "r"(smem_u32(counter)), "r"(value) : "memory");
  return old;
}
__device__ __forceinline__ int load_acquire(const int* flag) {
  int value;
  asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(value) : "r"(smem_u32(flag)) : "memory");
  return value;
}
__device__ __forceinline__ void store_release(int* flag, int value) {
  asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(flag)), "r"(value) : "memory");
}

__device__ __forceinline__ long long global_nanoseconds() {
  long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// PROFILE: thread 0 of every CTA with work also writes kTimelineColumns values to
// p.cycles[kTimelineColumns * blockIdx.x ..]: ns (%globaltimer, one clock for all
// SMs) at entry, when the work list was built, when its page ids were known, when
// its first tile had landed, at exit (of its last warp); then the pages of its
// share, the pieces that held pages of warp 0, the ns warp 0 spent depositing its
// piece states, the ns it spent merging pieces, and the pieces it merged.
constexpr int kTimelineColumns = 10;
// FP8: the pools are e4m3 bytes with one fp32 scale per (page, KV head).  A tile is
// converted to f16 in registers after ldmatrix and the MMAs are the f16 ones whatever
// T is (bf16 queries are converted once per piece; they are exact in f16 unless
// beyond its range).  The K scale multiplies the scores, the V scale the
// probabilities (relative to the scale of the warp's first page of the piece, which
// multiplies the accumulator once at the end, so that probabilities keep their
// magnitude in f16; the reference moves up when a page's scale exceeds it 16 times).
// What the ROPE variant needs on top: the packed QKV rows of the step ([Q0..Q11 | K0 K1 |
// V0 V1] x 128 per sequence), their positions and a table of (cos, sin) per position and
// rotary frequency (qf_build_rope_table: the same fp32 expressions as the RoPE / KV-write
// kernel, so the same bits).  With ROPE the kernel is the whole layer step: `f.q` points at
// the packed rows, so the Q tile of a piece arrives unrotated, its position's 512 bytes of
// the table ride behind it as one more 16-byte copy per lane, and every warp rotates its
// copy of the six heads in shared memory; the warp that owns a sequence's last page rotates
// the new K row, copies the new V row and stores both into the pools before it copies that
// page -- so no separate RoPE / KV-write kernel runs.  No sin / cos and no call in this
// kernel: with them (inlined or out of line) the page loop ran 4 to 10 us slower.
struct RopeInputs {
  const unsigned char* packed;  // row b at packed + b * row_bytes
  int64_t row_bytes;
  const void* positions;        // integer positions
  int64_t pos_stride;
  const float2* table;          // [table_positions][64] (cos, sin)
  int pos_dtype;
  int table_positions;
};

//
// SOLO (the variant every call runs): warp w owns the CONSECUTIVE units begin + block_start(w) ..
// of the CTA's share (eight blocks of share / 8 units, the first share % 8 of them one more)
// instead of every eighth (the list keeps its empty units: they make a block that holds many
// sequence starts shorter in pages).  Every
// stretch of one sequence inside a warp's block is a piece the warp computes on its own: one Q
// tile, its pages, no deposits, arrival counters or polls on the way.  A piece whose sequence
// neither began in the block of the warp before nor goes on in the block of the warp after is
// stored straight to its split slot.  The others -- at most a warp's first and last -- stay in
// the warp's two deposit buffers until the CTA's end, where, after the kernel's only CTA-wide
// barrier past the work list, a sequence's consecutive pieces (a "chain") are summed and stored
// as ONE piece per CTA and sequence -- by the warp that holds the first of them when the chain
// is short (many chains: all at once), by six warps, a query head each, when it is long -- so
// the slots, the bound share >= longest / (split_k - 1) and the end-of-sequence mark are exactly
// those of the variant above, and so is what the combine reads.  What a sequence
// boundary costs is one Q tile and one store for one warp instead of a Q tile and a deposit for
// each of eight plus a merge in the middle of the stream.
template <typename T, bool FP8, bool PROFILE, bool ROPE = false, bool SOLO = false>
__global__ void __launch_bounds__(kFastThreads, RingShape<FP8>::kCtasPerSm)
    decode_mma_kernel(const StreamParams sp, const __grid_constant__ RopeInputs rope) {
  static_assert(!(ROPE && FP8) || SOLO, "the fused RoPE / KV write on FP8 pools is built for the solo variant");
  static_assert(kQTileBytes + (ROPE ? 512 : 0) <= RingShape<FP8>::kSlotBytes, "the Q tile must fit a ring slot");
  // empty units in front of a sequence: both variants weigh the shares with them (the solo
  // variant, where a sequence costs one warp a Q tile and a store, measured per 28-layer step
  // with 0 / 3 / 6: 64 x U[128, 4096] tokens 0.790 / 0.771 / 0.767 ms, 256 x log-uniform
  // [64, 8192] 2.072 / 2.005 / 2.012, FP8 128 x 2 048 1.039 / 1.000 / 0.995)
  constexpr int kOverhead = kPieceOverhead;
  constexpr int kStep = SOLO ? 1 : kMmaWarps;          // distance between a warp's units
  using Ops = MmaOps<typename std::conditional<FP8, __half, T>::type>;
  using Ring = RingShape<FP8>;
  constexpr int kAhead = Ring::kAhead;
  const FastParams& p = sp.f;
  // [kMmaWarps] rings of Ring::kSlots slots, then kMmaMergeFloats of merge scratch
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ WorkList work;  // units are pages
  // per piece parity: the warps' softmax states, the weights the merging warp gives
  // them, how many warps have deposited, and the last piece merged
  __shared__ float warp_offset[2][kMmaWarps][kPaddedHeads];
  __shared__ float warp_sum[2][kMmaWarps][kPaddedHeads];
  __shared__ float warp_weight[2][kMmaWarps][kPaddedHeads];
  __shared__ int arrived[2];
  __shared__ int merged[2];
  __shared__ int chain_of[kMmaWarps][3];  // SOLO: per warp, the chain it heads: sequence (-1: none), buffer, warps

  constexpr unsigned kFull = 0xffffffffu;
  long long t_entry = 0, t_list = 0, t_ids = 0, t_first = 0, t_deposit = 0, t_merge = 0;
  int pieces = 0, merges = 0;
  if (PROFILE) t_entry = global_nanoseconds();
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int g = lane >> 2;  // MMA fragment row group
  const int q = lane & 3;   // MMA fragment column pair: heads 2q, 2q + 1
  const int kv_head = blockIdx.x / sp.ctas_per_head;
  const int cta = blockIdx.x - kv_head * sp.ctas_per_head;

  // The combine after this kernel may be scheduled as CTAs exit.  Until
  // dependency_wait() below, only step metadata that no kernel of the layer writes is
  // read (the sequence lengths, the block table and, ROPE, the positions) and -- when
  // sp.early_tiles says the caller vouches for them -- K / V tiles of pages other than
  // each sequence's last; nothing is written.
  release_dependents();
  if (tid < 2) arrived[tid] = 0, merged[tid] = tid - 2;  // pieces -2 and -1 count as merged
  // ---- the page list of this launch and this CTA's share of it (two CTA-wide barriers) ----
  const int longest =
      build_work_list<QF_PAGE_SIZE, kOverhead>(work, p.seq_lens, p.lens_dtype, p.lens_stride, p.batch,
                                               p.max_tokens);
  const int* first_page = work.first_unit;  // first unit of a sequence; its pages follow its empty units
  const int total = first_page[kMaxStreamBatch];
  if (PROFILE) t_list = global_nanoseconds();
  if (total == 0) {
    dependency_wait();  // keeps the chain of completions intact even without work
    return;
  }
  const int share = max((total + sp.ctas_per_head - 1) / sp.ctas_per_head,
                        (longest + p.split_k - 2) / (p.split_k - 1));
  // SOLO: warp w's block is base + 1 units for w < extra, base units otherwise, and starts at
  // block_start(w) units into the share; unit o of the share lies in the block of warp_of(o).
  const int base = share / kMmaWarps, extra = share - base * kMmaWarps;
  auto block_start = [&](int w) { return w * base + min(w, extra); };
  auto warp_of = [&](int o) { return o < extra * (base + 1) ? o / (base + 1) : extra + (o - extra * (base + 1)) / max(base, 1); };
  const int begin = cta * share;
  if (begin >= total) {
    dependency_wait();
    return;
  }
  const int count = min(share, total - begin);
  const int end = begin + count;
  // This warp's units: begin + warp + 8 k, k = 0 .. my_pages - 1 (pages, or empty units);
  // SOLO: begin + block_start(warp) + k.
  const int my_first = SOLO ? begin + block_start(warp) : begin + warp;
  const int my_pages = SOLO ? min(max(count - block_start(warp), 0), base + (warp < extra ? 1 : 0))
                            : (count > warp ? (count - warp + kMmaWarps - 1) / kMmaWarps : 0);

  // ---- loads ----
  const int pool_pages = static_cast<int>(p.num_pages);
  const int table_elem = p.table_dtype == QF_INDEX_I64 ? 8 : 4;
  const unsigned char* table_base = static_cast<const unsigned char*>(p.block_table);
  // A row is 16 chunks of 16 bytes (8 for FP8): a lane copies chunk lane % 16 (lane % 8)
  // of rows 2j + lane / 16, j = 0..7 (4j + lane / 8, j = 0..3); chunk c of row r is
  // stored at chunk c ^ (r % 8) of the row.
  constexpr int kChunksPerRow = Ring::kRowBytes / 16;
  constexpr int kRowsPerPass = 32 / kChunksPerRow;
  const int copy_chunk = lane & (kChunksPerRow - 1), copy_row = lane / kChunksPerRow;
  const unsigned char* k_base = p.k_pool + kv_head * p.k_head_bytes + copy_chunk * 16;
  const unsigned char* v_base = p.v_pool + kv_head * p.v_head_bytes + copy_chunk * 16;
  unsigned char* ring = smem + warp * Ring::kWarpBytes;
  int fill_offset[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int r = kRowsPerPass * j + copy_row;
    fill_offset[j] = r * Ring::kRowBytes + ((copy_chunk ^ (r & 7)) << 4);
  }
  // Byte offset, inside a page, of the row each of the lane's copies reads (K and V
  // pools share their strides), and the page stride.
  int row_source[FP8 ? 4 : 8];
#pragma unroll
  for (int j = 0; j < (FP8 ? 4 : 8); ++j) row_source[j] = (kRowsPerPass * j + copy_row) * static_cast<int>(p.k_tok_bytes);
  const int64_t page_bytes = p.k_page_bytes;

  // Page ids and row counts of 32 of this warp's units at a time, one per lane (id -3:
  // an empty unit, nothing to load), and the sequence whose Q rows must precede the
  // page (-1 unless it is the warp's first page of the sequence in this share).
  auto describe = [&](int chunk, int& id, int& rows, int& q_of, int& last_of, int& pos) {
    const int k = chunk * 32 + lane;
    id = -1, rows = 0, q_of = -1, last_of = -1, pos = 0;
    if (k < my_pages) {
      const int unit = my_first + kStep * k;
      const int sequence = sequence_of_unit(work, p.batch, unit);
      const int in_sequence = unit - first_page[sequence] -
                              sequence_overhead<kOverhead>((work.length[sequence] + QF_PAGE_SIZE - 1) / QF_PAGE_SIZE);
      // page index within the sequence; < 0: an empty unit
      if (in_sequence < 0) {
        id = -3;
        return;
      }
      const unsigned char* at =
          table_base + (sequence * p.bt_sb + static_cast<int64_t>(in_sequence) * p.bt_sp) * table_elem;
      const int64_t raw = table_elem == 8 ? *reinterpret_cast<const int64_t*>(at)
                                          : static_cast<int64_t>(*reinterpret_cast<const int32_t*>(at));
      id = static_cast<uint64_t>(raw) < static_cast<uint64_t>(pool_pages) ? static_cast<int>(raw) : -2;
      rows = min(QF_PAGE_SIZE, work.length[sequence] - in_sequence * QF_PAGE_SIZE);
      // the page that takes the step's new token (the last token of the sequence): ROPE stores
      // that token's row itself; no variant copies this page before the dependency wait
      if (in_sequence == (work.length[sequence] - 1) / QF_PAGE_SIZE) last_of = sequence;
      // ... and the sequence's rotation position, fetched here (32 units ahead of its use)
      if (ROPE) {
        const int64_t at = load_index(rope.positions, rope.pos_dtype, sequence * rope.pos_stride);
        if (at < 0 || at >= rope.table_positions) atomicMax(p.status, kStatusPositionPastTable);
        pos = static_cast<int>(at < 0 ? 0 : (at >= rope.table_positions ? rope.table_positions - 1 : at));
      }
      if (k == 0 || in_sequence < kStep) q_of = sequence;  // the warp's previous unit is no page of this sequence
    }
  };
  int id_now, rows_now, q_now, last_now, id_next, rows_next, q_next, last_next;
  int pos_now, pos_next;  // ROPE: row of the (cos, sin) table
  describe(0, id_now, rows_now, q_now, last_now, pos_now);
  describe(1, id_next, rows_next, q_next, last_next, pos_next);
  // Bit k: unit k of the chunk is a "plain" page -- a valid id, all sixteen rows, no Q tile
  // in front of it.  Such pages (all but a sequence's first few and its last) take a short
  // path through issue_tile.
  auto plain_units = [&](int id, int rows, int q_of) {
    return __ballot_sync(kFull, id >= 0 && rows >= QF_PAGE_SIZE && q_of < 0);
  };
  unsigned plain_now = 0, plain_next = 0;
  if constexpr (FP8) plain_now = plain_units(id_now, rows_now, q_now), plain_next = plain_units(id_next, rows_next, q_next);
  if (PROFILE) t_ids = id_now + id_next > -100 ? global_nanoseconds() : 0;  // after the ids have arrived

  // The warp's tiles, in ring order: for each of its pages [Q rows, if the page is its
  // first of a sequence,] K, V.  Tile n sits in ring slot n % 5.
  const unsigned char* q_base = static_cast<const unsigned char*>(p.q) +
                                (static_cast<int64_t>(kv_head) * QF_GQA_GROUP * p.q_sh) * 2;
  int fill_page = 0, fill_stage = 0, fill_slot = 0;  // stage 0: Q, 1: K, 2: V
  // ROPE: the step's new token of `sequence` is row rows - 1 of page `id`: store it (K
  // rotated, V as it is) so that the copy of the page brings it along.
  struct NewRow {  // what one lane holds of a new token between its loads and its stores
    float2 cs_lo, cs_hi;
    float x1, x2, y1, y2;
    uint4 v_bits;
    int64_t row;  // byte offset of the pool row (the same in both pools)
    float k_scale, v_scale;  // FP8 pools: the page's scales, by which the new row is divided
    bool write;   // false: the sequence's length was cut to the table's capacity
  };
  auto load_new_row = [&](int sequence, int id, int rows, int position) {
    NewRow r;
    // Not when the length was cut to the table's capacity: the token's slot is then outside
    // the table, and nothing is written for it.  Only a length equal to the capacity can have
    // been cut, and only then is the given length looked at again.
    r.write = work.length[sequence] < p.max_tokens ||
              load_index(p.seq_lens, p.lens_dtype, sequence * p.lens_stride) == work.length[sequence];
    if (!r.write && lane == 0) atomicMax(p.status, kStatusPositionPastTable);
    r.row = static_cast<int64_t>(id) * page_bytes + static_cast<int64_t>(rows - 1) * p.k_tok_bytes +
            kv_head * p.k_head_bytes;
    const unsigned char* row_in = rope.packed + static_cast<int64_t>(sequence) * rope.row_bytes;
    const T* from = reinterpret_cast<const T*>(row_in + (12 + kv_head) * QF_HEAD_DIM * 2);
    const float2* cs = rope.table + static_cast<int64_t>(position) * (QF_HEAD_DIM / 2);
    // every load at once: one trip to memory for the whole row
    r.cs_lo = cs[lane], r.cs_hi = cs[lane + 32];
    r.x1 = to_float(from[lane]), r.x2 = to_float(from[lane + 64]);
    r.y1 = to_float(from[lane + 32]), r.y2 = to_float(from[lane + 96]);
    r.v_bits = make_uint4(0u, 0u, 0u, 0u);
    if (lane < 16) r.v_bits = reinterpret_cast<const uint4*>(row_in + (14 + kv_head) * QF_HEAD_DIM * 2)[lane];
    r.k_scale = r.v_scale = 1.f;
    if constexpr (FP8) {
      r.k_scale = p.k_scale[static_cast<int64_t>(id) * p.kv_heads + kv_head];
      r.v_scale = p.v_scale[static_cast<int64_t>(id) * p.kv_heads + kv_head];
    }
    return r;
  };
  auto finish_new_row = [&](const NewRow& r) {
    if (!r.write) return;  // the same for every lane
    if constexpr (FP8) {
      // e4m3 bytes at the page's fixed scales: clamp(x / scale, +-448), round to nearest even,
      // saturating -- the expressions of the RoPE / KV-write kernel, so the same bytes
      auto encode = [](float x, float scale) {
        const float y = fminf(fmaxf(__fdiv_rn(x, scale), -448.f), 448.f);
        return static_cast<unsigned char>(__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3));
      };
      unsigned char* to = const_cast<unsigned char*>(p.k_pool) + r.row;
      to[lane] = encode(__fsub_rn(__fmul_rn(r.x1, r.cs_lo.x), __fmul_rn(r.x2, r.cs_lo.y)), r.k_scale);
      to[lane + 64] = encode(__fadd_rn(__fmul_rn(r.x2, r.cs_lo.x), __fmul_rn(r.x1, r.cs_lo.y)), r.k_scale);
      to[lane + 32] = encode(__fsub_rn(__fmul_rn(r.y1, r.cs_hi.x), __fmul_rn(r.y2, r.cs_hi.y)), r.k_scale);
      to[lane + 96] = encode(__fadd_rn(__fmul_rn(r.y2, r.cs_hi.x), __fmul_rn(r.y1, r.cs_hi.y)), r.k_scale);
      if (lane < 16) {
        const float2 a = unpack2<T>(r.v_bits.x), b = unpack2<T>(r.v_bits.y), c = unpack2<T>(r.v_bits.z),
                     d = unpack2<T>(r.v_bits.w);
        __align__(8) unsigned char bytes[8] = {encode(a.x, r.v_scale), encode(a.y, r.v_scale), encode(b.x, r.v_scale),
                                               encode(b.y, r.v_scale), encode(c.x, r.v_scale), encode(c.y, r.v_scale),
                                               encode(d.x, r.v_scale), encode(d.y, r.v_scale)};
        reinterpret_cast<uint2*>(const_cast<unsigned char*>(p.v_pool) + r.row)[lane] = *reinterpret_cast<const uint2*>(bytes);
      }
      __syncwarp();  // the lanes' stores are ordered before the lanes' copies of the rows
      return;
    }
    T* to = reinterpret_cast<T*>(const_cast<unsigned char*>(p.k_pool) + r.row);
    to[lane] = from_float<T>(__fsub_rn(__fmul_rn(r.x1, r.cs_lo.x), __fmul_rn(r.x2, r.cs_lo.y)));
    to[lane + 64] = from_float<T>(__fadd_rn(__fmul_rn(r.x2, r.cs_lo.x), __fmul_rn(r.x1, r.cs_lo.y)));
    to[lane + 32] = from_float<T>(__fsub_rn(__fmul_rn(r.y1, r.cs_hi.x), __fmul_rn(r.y2, r.cs_hi.y)));
    to[lane + 96] = from_float<T>(__fadd_rn(__fmul_rn(r.y2, r.cs_hi.x), __fmul_rn(r.y1, r.cs_hi.y)));
    if (lane < 16) reinterpret_cast<uint4*>(const_cast<unsigned char*>(p.v_pool) + r.row)[lane] = r.v_bits;
    __syncwarp();  // the lanes' stores are ordered before the lanes' copies of the rows
  };
  auto store_new_row = [&](int sequence, int id, int rows, int position) {
    finish_new_row(load_new_row(sequence, id, rows, position));
  };
  // New rows are stored when their units are described, 32 units at a time: those among the
  // warp's first 64 units up front (past its first two pages in the shadow of the first
  // tiles' latency), later ones
  // when the descriptors are refreshed.  Stored from inside the page loop, next to the copy
  // of its page, a row cost its warp the contents of its ring (a third of the kernel's time).
  auto store_new_rows_of = [&](int& id_of, int& rows_of, int& last_of, int& pos_of, unsigned lanes) {
    unsigned pending = __ballot_sync(kFull, last_of >= 0 && id_of >= 0) & lanes;
    while (pending != 0) {
      const int source = __ffs(pending) - 1;
      pending &= pending - 1;
      store_new_row(__shfl_sync(kFull, last_of, source), __shfl_sync(kFull, id_of, source),
                    __shfl_sync(kFull, rows_of, source), __shfl_sync(kFull, pos_of, source));
      if (lane == source) last_of = -1;
    }
  };
  // The Q rows of sequence `q_of` (and, ROPE, its position's cos / sin) into ring slot `dst`.
  auto copy_q_tile = [&](unsigned char* dst, int q_of, int position) {
    // 6 heads x 256 bytes = 96 chunks: three per lane
    const unsigned char* src = q_base + static_cast<int64_t>(q_of) * p.q_sb * 2;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const int chunk = lane + 32 * j, head = chunk >> 4, c = chunk & 15;
      copy_chunk_async<false>(dst + head * kQRowBytes + c * 16, src + head * p.q_sh * 2 + c * 16);
    }
    if constexpr (ROPE) {
      // the position's (cos, sin) of all 64 frequencies ride behind the tile: 32 chunks
      copy_chunk_async<false>(dst + kQTileBytes + lane * 16,
                              reinterpret_cast<const unsigned char*>(
                                  rope.table + static_cast<int64_t>(position) * (QF_HEAD_DIM / 2)) + lane * 16);
    }
  };
  // early: called before the dependency wait.  Only tiles of pages that no kernel of this
  // step writes may be copied then: K and V of pages that do not hold a sequence's newest
  // token.  The warp's first Q tile (ring slot 0) is left for later (`deferred_q`); the call
  // returns false, without having issued anything, at the first tile that has to wait.
  int deferred_q = -1, deferred_pos = 0;
  // All sixteen rows of a (page, KV head) tile at `src` into ring slot `dst`.
  auto copy_full_tile = [&](unsigned char* dst, const unsigned char* src) {
    constexpr int kPasses = FP8 ? 4 : 8;
#pragma unroll
    for (int j = 0; j < kPasses; ++j) {
      copy_chunk_async<false>(dst + fill_offset[j & 3] + (FP8 ? 0 : (j >> 2) * (8 * 256)), src + row_source[j]);
    }
  };
  // FP8: the tile's scale rides behind it (one 4-byte copy by lane 0).
  auto copy_scale = [&](unsigned char* dst, int id, bool value_tile) {
    if (lane == 0) {
      const float* scale = (value_tile ? p.v_scale : p.k_scale) + static_cast<int64_t>(id) * p.kv_heads + kv_head;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst + Ring::kTileBytes)), "l"(scale)
                   : "memory");
    }
  };
  bool new_rows_described = false;  // ROPE: the descriptors just fetched may hold new rows to store
  bool plain_v_pending = false;  // the last call issued the K tile of a plain page; its V tile is next
  int64_t plain_page_offset = 0;
  int plain_id = 0;
  auto issue_tile = [&](bool early = false) -> bool {
    // FP8 only: that variant is bound by its instruction stream (31.5 -> 28.7 us per launch on
    // 128 x 2048 tokens); the 16-bit variants are bound by HBM and ran 2 to 7 % slower with the
    // extra code in their page loop.
    if (FP8 && !early) {
      // The common case, kept short (the general path below costs about 85 instructions per
      // tile, most of them deciding what the tile is): K then V of a plain page.
      unsigned char* dst = ring + fill_slot * Ring::kSlotBytes;
      if (fill_stage == 2 && plain_v_pending) {
        copy_full_tile(dst, v_base + plain_page_offset);
        if constexpr (FP8) copy_scale(dst, plain_id, true);
        plain_v_pending = false, fill_stage = 0, ++fill_page;
        commit_copies();
        fill_slot = fill_slot == Ring::kSlots - 1 ? 0 : fill_slot + 1;
        return true;
      }
      // (unit 0 of a 32-unit chunk goes the general way: that is where the descriptors move on)
      if (fill_stage == 0 && fill_page < my_pages && (fill_page & 31) != 0 && ((plain_now >> (fill_page & 31)) & 1u)) {
        plain_id = __shfl_sync(kFull, id_now, fill_page & 31);
        plain_page_offset = static_cast<int64_t>(plain_id) * page_bytes;
        copy_full_tile(dst, k_base + plain_page_offset);
        if constexpr (FP8) copy_scale(dst, plain_id, false);
        plain_v_pending = true, fill_stage = 2;
        commit_copies();
        fill_slot = fill_slot == Ring::kSlots - 1 ? 0 : fill_slot + 1;
        return true;
      }
    }
    int id = -3;
    while (fill_page < my_pages) {
      if (fill_stage == 0 && (fill_page & 31) == 0 && fill_page > 0) {
        if (early) return false;
        id_now = id_next, rows_now = rows_next, q_now = q_next, last_now = last_next, pos_now = pos_next;
        plain_now = plain_next;
        describe((fill_page >> 5) + 1, id_next, rows_next, q_next, last_next, pos_next);
        if constexpr (FP8) plain_next = plain_units(id_next, rows_next, q_next);
        // ROPE: the new rows of the 32 units just described, well before their pages are copied
        // (which happens after the next 32 units have been issued).  FP8 pools: at the top of the
        // next page instead, in one place -- this code is inlined wherever a tile is issued, and
        // with the quantisation in every copy that instantiation grew to 145 KB (120 KB so; the
        // step of 128 x 2 048 tokens 0.944 -> 0.924 ms)
        if constexpr (ROPE && !FP8) store_new_rows_of(id_next, rows_next, last_next, pos_next, kFull);
        if constexpr (ROPE && FP8) new_rows_described = true;
      }
      id = __shfl_sync(kFull, id_now, fill_page & 31);
      if (id != -3) break;
      ++fill_page;  // an empty unit (only met at stage 0): nothing to load
    }
    if (early && fill_page >= my_pages) return false;
    if (fill_page < my_pages) {
      int rows = __shfl_sync(kFull, rows_now, fill_page & 31);
      const int q_of = __shfl_sync(kFull, q_now, fill_page & 31);
      if (fill_stage == 0 && q_of < 0) fill_stage = 1;
      if (early) {
        if (fill_stage == 0) {
          if (fill_slot != 0 || deferred_q >= 0) return false;  // a later sequence's Q rows
          deferred_q = q_of, deferred_pos = __shfl_sync(kFull, pos_now, fill_page & 31);
          fill_stage = 1, fill_slot = 1;  // slot 0 is filled after the wait
        }
        if (id < 0 || __shfl_sync(kFull, last_now, fill_page & 31) >= 0) return false;
      }
      unsigned char* dst = ring + fill_slot * Ring::kSlotBytes;
      if (fill_stage == 0) {
        copy_q_tile(dst, q_of, ROPE ? __shfl_sync(kFull, pos_now, fill_page & 31) : 0);
      } else {
        if (id < 0) {
          rows = 0;  // bad or missing id: the page reads as zeros
          if (id == -2 && lane == 0) atomicMax(p.status, kStatusBadPageId);
        }
        // K and V pools have the same strides here (the host checks), so one set of row
        // offsets serves both.  A page whose 16 rows all exist (every page but a
        // sequence's last) takes the branch-free copies.
        const unsigned char* src = (fill_stage == 2 ? v_base : k_base) + static_cast<int64_t>(id < 0 ? 0 : id) * page_bytes;
        constexpr int kPasses = FP8 ? 4 : 8;
        if (rows >= QF_PAGE_SIZE) {
#pragma unroll
          for (int j = 0; j < kPasses; ++j) {
            copy_chunk_async<false>(dst + fill_offset[j & 3] + (FP8 ? 0 : (j >> 2) * (8 * 256)), src + row_source[j]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < kPasses; ++j) {
            const int r = kRowsPerPass * j + copy_row;
            unsigned char* to = dst + fill_offset[j & 3] + (FP8 ? 0 : (j >> 2) * (8 * 256));
            if (r < rows) {
              copy_chunk_async<false>(to, src + row_source[j]);
            } else {
              *reinterpret_cast<uint4*>(to) = make_uint4(0u, 0u, 0u, 0u);
            }
          }
        }
        if constexpr (FP8) {
          if (lane == 0) {
            // the tile's scale rides behind it
            float* scale_slot = reinterpret_cast<float*>(dst + Ring::kTileBytes);
            if (id >= 0) {
              const float* scale =
                  (fill_stage == 2 ? p.v_scale : p.k_scale) + static_cast<int64_t>(id) * p.kv_heads + kv_head;
              asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(scale_slot)), "l"(scale)
                           : "memory");
            } else {
              *scale_slot = 1.f;
            }
          }
        }
      }
      if (++fill_stage > 2) fill_stage = 0, ++fill_page;
    }
    commit_copies();  // always, so that group counting stays uniform
    fill_slot = fill_slot == Ring::kSlots - 1 ? 0 : fill_slot + 1;
    return true;
  };
  // Before the wait: up to kAhead - 1 K / V tiles of pages that nothing in flight can write
  // (the caller's promise, see StreamParams::early_tiles) start their trip to shared memory
  // while the kernels before this one drain.
  int issued = 0;
  if constexpr (ROPE && !FP8) {
    // (not for FP8 pools: one early tile per warp is all their ring has room for, and the copy
    // of the tile-issue code it needs makes the largest instantiation of the family larger still)
    if (sp.early_tiles) {
#pragma unroll 1
      while (issued < kAhead - 1 && issue_tile(true)) ++issued;
    }
  }
  bool first_tiles_out_of_order = issued > 0;  // groups: early tiles first, then the Q tile
  // From here on the kernel reads what the RoPE / KV-write kernel stored (Q rows, the
  // newest K/V rows) and writes the partial buffers the previous combine read.
  dependency_wait();
  auto issue_first_tiles = [&]() {
    if (deferred_q >= 0) {
      copy_q_tile(ring, deferred_q, deferred_pos);
      commit_copies();
      ++issued;
    }
#pragma unroll 1
    for (; issued < kAhead; ++issued) issue_tile();
  };
  if constexpr (ROPE) {
    // the first four tiles (Q K V of a page, then Q or K of the next) touch the warp's first
    // two units that are pages: only their new rows have to be in place before any copy
    unsigned first_two = __ballot_sync(kFull, id_now != -3);
    first_two &= ~((first_two & (first_two - 1)) & ((first_two & (first_two - 1)) - 1));
    store_new_rows_of(id_now, rows_now, last_now, pos_now, first_two);
    // The warp's next new row (usually its only one): its loads go out ahead of the first
    // tiles' copies -- behind them they would queue after the whole GPU's opening burst --
    // and it is stored once those copies are on their way.
    const unsigned pending = __ballot_sync(kFull, last_now >= 0 && id_now >= 0);
    NewRow early;
    const int source = pending != 0 ? __ffs(pending) - 1 : -1;
    if (source >= 0) {
      early = load_new_row(__shfl_sync(kFull, last_now, source), __shfl_sync(kFull, id_now, source),
                           __shfl_sync(kFull, rows_now, source), __shfl_sync(kFull, pos_now, source));
      if (lane == source) last_now = -1;
    }
    issue_first_tiles();
    if (source >= 0) finish_new_row(early);
    store_new_rows_of(id_now, rows_now, last_now, pos_now, kFull);
    store_new_rows_of(id_next, rows_next, last_next, pos_next, kFull);
  } else {
    issue_first_tiles();
  }

  // ---- fragments ----
  // ldmatrix row addresses inside a tile; matrix i = lane / 8.
  // 16-bit pools.  K (A = K tile, k-step s covers dims 16 s ..): matrix i holds rows
  // 8 (i & 1) .., chunk 2 s + (i >> 1).  V (A = V^T, m-tile j covers dims 16 j ..): matrix
  // i holds token rows 8 (i >> 1) .., chunk 2 j + (i & 1).
  // FP8 pools (a 16-byte chunk is 16 dims): for K and for V alike matrix i holds token
  // rows 8 (i & 1) .., chunk 2 s + (i >> 1); one ldmatrix.x4 feeds two k-steps (m-tiles).
  const int mat = lane >> 3;
  const uint32_t k_row_offset = ((lane & 7) + 8 * (mat & 1)) * Ring::kRowBytes;
  const uint32_t k_chunk_xor = ((mat >> 1) ^ (lane & 7)) << 4;
  const uint32_t v_row_offset = FP8 ? k_row_offset : ((lane & 7) + 8 * (mat >> 1)) * Ring::kRowBytes;
  const uint32_t v_chunk_xor = FP8 ? k_chunk_xor : ((mat & 1) ^ (lane & 7)) << 4;
  const uint32_t ring_addr = smem_u32(ring);

  // B operand Q^T of head g (0 for g >= 6), read from the Q tile at the head of each
  // piece.  16-bit pools: [k-step s][dims 16 s + 2q, +1 | 16 s + 8 + 2q, +1].  FP8 pools:
  // [k-step s][dims 16 s + 4q, +1 | 16 s + 4q + 2, +3], the order in which ldmatrix on
  // the byte view hands out a row's dims; an MMA does not care which dim sits at
  // which k as long as both operands agree.
  uint32_t q_frag[8][2];
  const uint32_t q_lane_offset = (g < QF_GQA_GROUP ? g : 0) * kQRowBytes + (FP8 ? 8 : 4) * q;

  float* deposits = reinterpret_cast<float*>(smem + kMmaWarps * Ring::kWarpBytes);
  // O^T: [m-tile j][(dim a, head 2q) (a, 2q+1) (b, 2q) (b, 2q+1)] with (a, b) = (16j + g,
  // 16j + g + 8) for 16-bit pools and (16j + 2g, 16j + 2g + 1) for FP8 pools
  float acc[8][4];

  // Pieces are numbered by `rank` in the order of the sequences; every warp walks
  // the same list but only stops at pieces that hold some of its pages.
  int piece_seq = sequence_of_unit(work, p.batch, begin);
  int rank = 0;
  int page = my_first;  // this warp's next unit
  const int my_end = SOLO ? my_first + my_pages : end;  // end of this warp's units
  int chain_seq = -1, chain_buffer = 0;  // SOLO: the sequence whose pieces this warp merges at the CTA's end
  int read_slot = 0;
  // Move (piece_seq, rank) forward to the sequence that holds unit `target` (< end).  Only
  // sequences with a page inside the share count as pieces.
  auto first_data_unit = [&](int sequence) {
    return first_page[sequence] +
           sequence_overhead<kOverhead>((work.length[sequence] + QF_PAGE_SIZE - 1) / QF_PAGE_SIZE);
  };
  auto advance_to = [&](int target) {
    while (piece_seq < p.batch - 1 && first_page[piece_seq + 1] <= target) {
      ++piece_seq;
      if (first_page[piece_seq + 1] > first_page[piece_seq] && first_data_unit(piece_seq) < end) ++rank;
    }
  };

  while (page < my_end) {
    advance_to(page);
    const int seq_first = first_data_unit(piece_seq);  // unit of the sequence's first page
    if (page < seq_first) {
      // empty units: on to this warp's first unit that is a page (maybe of a later sequence)
      page += ((seq_first - page + kStep - 1) / kStep) * kStep;
      continue;
    }
    {
      // ---- the piece's Q tile ----
      if (first_tiles_out_of_order) {
        wait_all_copies();  // the warp's first Q tile was issued behind the early tiles
        first_tiles_out_of_order = false;
      } else {
        wait_tiles_ahead<kAhead>();
      }
      __syncwarp();
      if (PROFILE && t_first == 0) t_first = global_nanoseconds();
      issue_tile();
      if constexpr (ROPE) {
        // the tile holds the six unrotated query heads of the group: rotate them in place,
        // each lane the frequencies 2 lane and 2 lane + 1 of every head (one 32-bit word of
        // each half of a head; their cos / sin are the 16 bytes this lane copied)
        unsigned char* tile = ring + read_slot * Ring::kSlotBytes;
        const float4 cs = reinterpret_cast<const float4*>(tile + kQTileBytes)[lane];  // c0 s0 c1 s1
#pragma unroll
        for (int head = 0; head < QF_GQA_GROUP; ++head) {
          uint32_t* row = reinterpret_cast<uint32_t*>(tile + head * kQRowBytes);
          const float2 x1 = unpack2<T>(row[lane]), x2 = unpack2<T>(row[lane + 32]);
          row[lane] = pack2<T>(__fsub_rn(__fmul_rn(x1.x, cs.x), __fmul_rn(x2.x, cs.y)),
                               __fsub_rn(__fmul_rn(x1.y, cs.z), __fmul_rn(x2.y, cs.w)));
          row[lane + 32] = pack2<T>(__fadd_rn(__fmul_rn(x2.x, cs.x), __fmul_rn(x1.x, cs.y)),
                                    __fadd_rn(__fmul_rn(x2.y, cs.z), __fmul_rn(x1.y, cs.w)));
        }
        __syncwarp();
      }
      const unsigned char* q_tile = ring + read_slot * Ring::kSlotBytes + q_lane_offset;
      read_slot = read_slot == Ring::kSlots - 1 ? 0 : read_slot + 1;
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        uint32_t lo, hi;
        if constexpr (FP8) {
          const uint2 both = *reinterpret_cast<const uint2*>(q_tile + 32 * s);
          lo = both.x, hi = both.y;
          if constexpr (std::is_same<T, __nv_bfloat16>::value) lo = bf16x2_to_f16x2(lo), hi = bf16x2_to_f16x2(hi);
        } else {
          lo = *reinterpret_cast<const uint32_t*>(q_tile + 32 * s);
          hi = *reinterpret_cast<const uint32_t*>(q_tile + 32 * s + 16);
        }
        q_frag[s][0] = g < QF_GQA_GROUP ? lo : 0u;
        q_frag[s][1] = g < QF_GQA_GROUP ? hi : 0u;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
    float offset[2] = {-INFINITY, -INFINITY};  // of heads 2q, 2q+1 (log2 units), equal in all lanes of a q
    float sum[2] = {0.f, 0.f};                 // over this lane's tokens
    float v_reference = 0.f, v_reference_inverse = 0.f;  // FP8: V scale of the warp's first page of the piece
    const int seq_len = work.length[piece_seq];
    const int piece_begin = max(seq_first, begin);  // first page of the piece (as a unit)
    const int piece_end = min(first_page[piece_seq + 1], my_end);
    const int done_seq = piece_seq, done_rank = rank;

    for (; page < piece_end; page += kStep) {
      if constexpr (ROPE && FP8) {
        if (new_rows_described) {
          store_new_rows_of(id_next, rows_next, last_next, pos_next, kFull);
          new_rows_described = false;
        }
      }
      // ---- scores S^T = K Q^T ----
      wait_tiles_ahead<kAhead>();
      __syncwarp();
      issue_tile();
      const uint32_t k_tile = ring_addr + read_slot * Ring::kSlotBytes + k_row_offset;
      float k_scale = 1.f;
      if constexpr (FP8) {
        k_scale = *reinterpret_cast<const float*>(ring + read_slot * Ring::kSlotBytes + Ring::kTileBytes);
      }
      read_slot = read_slot == Ring::kSlots - 1 ? 0 : read_slot + 1;
      float s_even[4] = {0.f, 0.f, 0.f, 0.f}, s_odd[4] = {0.f, 0.f, 0.f, 0.f};
      if constexpr (FP8) {
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          // bytes of r[.]: this lane's dims 4q .. 4q+3 of the 16-dim chunk; r[0], r[1]: tokens
          // g, g + 8 of chunk 2s; r[2], r[3]: of chunk 2s + 1
          uint32_t r[4];
          ldmatrix_x4(r, k_tile + ((32u * s) ^ k_chunk_xor));
          uint32_t first[4], second[4];  // a0 a1 a2 a3 of the two k-steps
          e4m3x4_to_f16x2x2(r[0], first[0], first[2]);
          e4m3x4_to_f16x2x2(r[1], first[1], first[3]);
          e4m3x4_to_f16x2x2(r[2], second[0], second[2]);
          e4m3x4_to_f16x2x2(r[3], second[1], second[3]);
          Ops::mma(s_even, first, q_frag[2 * s][0], q_frag[2 * s][1]);
          Ops::mma(s_odd, second, q_frag[2 * s + 1][0], q_frag[2 * s + 1][1]);
        }
      } else {
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          uint32_t a[4];
          ldmatrix_x4(a, k_tile + ((32u * s) ^ k_chunk_xor));
          Ops::mma((s & 1) ? s_odd : s_even, a, q_frag[s][0], q_frag[s][1]);
        }
      }
      // score[i]: i = 0 (token g, head 2q), 1 (g, 2q+1), 2 (g+8, 2q), 3 (g+8, 2q+1)
      float score[4];
      const int rows = seq_len - (page - seq_first) * QF_PAGE_SIZE;  // tokens of the page that exist (>= 1)
      const bool valid_lo = g < rows, valid_hi = g + 8 < rows;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        score[i] = (s_even[i] + s_odd[i]) * (FP8 ? p.scale_log2 * k_scale : p.scale_log2);
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
      // ---- values O^T += V^T P^T ----
      wait_tiles_ahead<kAhead>();
      __syncwarp();
      issue_tile();
      const uint32_t v_tile = ring_addr + read_slot * Ring::kSlotBytes + v_row_offset;
      float v_weight = 1.f;
      if constexpr (FP8) {
        const float v_scale = *reinterpret_cast<const float*>(ring + read_slot * Ring::kSlotBytes + Ring::kTileBytes);
        if (v_reference == 0.f) {
          v_reference = v_scale, v_reference_inverse = 1.f / v_scale;
        } else if (v_scale > 16.f * v_reference) {
          // a page far larger than the reference: move the reference up (rare; the same
          // for all lanes), so that weighted probabilities stay well inside f16
          const float down = v_reference * (1.f / v_scale);
#pragma unroll
          for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[j][i] *= down;
          v_reference = v_scale, v_reference_inverse = 1.f / v_scale;
        }
        v_weight = v_scale * v_reference_inverse;
      }
      read_slot = read_slot == Ring::kSlots - 1 ? 0 : read_slot + 1;
      // P^T as B operand: [k = tokens 2q.. | 8 + 2q..][n = head g]
      const uint32_t p_lo = transpose_8x8(Ops::pack(prob[0] * v_weight, prob[1] * v_weight));
      const uint32_t p_hi = transpose_8x8(Ops::pack(prob[2] * v_weight, prob[3] * v_weight));
      if constexpr (FP8) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // r[.] after the transpose: bytes (token 2q: dims 2g, 2g+1 | token 2q+1: dims 2g,
          // 2g+1) of a 16-dim chunk; r[0], r[1]: tokens 0-7, 8-15 of chunk 2j; r[2], r[3]: of
          // chunk 2j + 1.  Bytes (0, 2) are dim 2g of both tokens, bytes (1, 3) dim 2g + 1.
          uint32_t r[4];
          ldmatrix_x4_trans(r, v_tile + ((32u * j) ^ v_chunk_xor));
          // one byte permute per register puts (dim 2g: tokens 2q, 2q+1) in the low half and
          // (dim 2g+1: tokens 2q, 2q+1) in the high half
          uint32_t first[4], second[4];
          e4m3x4_to_f16x2x2(__byte_perm(r[0], 0u, 0x3120), first[0], first[1]);
          e4m3x4_to_f16x2x2(__byte_perm(r[1], 0u, 0x3120), first[2], first[3]);
          e4m3x4_to_f16x2x2(__byte_perm(r[2], 0u, 0x3120), second[0], second[1]);
          e4m3x4_to_f16x2x2(__byte_perm(r[3], 0u, 0x3120), second[2], second[3]);
          Ops::mma(acc[2 * j], first, p_lo, p_hi);
          Ops::mma(acc[2 * j + 1], second, p_lo, p_hi);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint32_t a[4];
          ldmatrix_x4_trans(a, v_tile + ((32u * j) ^ v_chunk_xor));
          Ops::mma(acc[j], a, p_lo, p_hi);
        }
      }
    }
    if constexpr (FP8) {
      // back to absolute V scale (v_reference is 0 only if the warp had no page, and
      // then the accumulator is 0 too)
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] *= v_reference;
    }

    if constexpr (SOLO) {
      // ---- the piece is this warp's alone.  If the sequence neither reaches into the block of
      // the warp before nor into that of the warp after (within this CTA), it goes to its split
      // slot now; otherwise its state is left in shared memory for the merge at the CTA's end.
      // Buffer 0 of a warp holds its first piece, buffer 1 stages the others (the last one, if
      // it reaches into the next block, stays there). ----
      if (PROFILE) ++pieces;
      const bool first_piece = max(seq_first, my_first) == my_first;
      const bool open_left = first_piece && seq_first < my_first && my_first > begin;
      const bool open_right = first_page[done_seq + 1] > my_end && my_end < end;
      const int buffer = first_piece ? 0 : 1;
      float* mine = deposits + (buffer * kMmaWarps + warp) * kDepositFloats;  // [6 heads][dim]
      if (q < QF_GQA_GROUP / 2) {
        float* even = mine + (2 * q) * kDepositHeadStride + (FP8 ? 2 * g : g);
        float* odd = even + kDepositHeadStride;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          even[16 * j] = acc[j][0], odd[16 * j] = acc[j][1];
          even[16 * j + (FP8 ? 1 : 8)] = acc[j][2], odd[16 * j + (FP8 ? 1 : 8)] = acc[j][3];
        }
      }
      float total[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        total[h] = sum[h];
        total[h] += __shfl_xor_sync(kFull, total[h], 4);
        total[h] += __shfl_xor_sync(kFull, total[h], 8);
        total[h] += __shfl_xor_sync(kFull, total[h], 16);
      }
      if (open_left || open_right) {
        if (g == 0) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            warp_offset[buffer][warp][2 * q + h] = offset[h], warp_sum[buffer][warp][2 * q + h] = total[h];
          }
        }
        if (open_right && !open_left) chain_seq = done_seq, chain_buffer = buffer;  // this warp merges the chain
        __syncwarp();
        continue;
      }
      __syncwarp();
      const int split_slot = cta - seq_first / share;
      const bool slot_ok = split_slot >= 0 && split_slot < p.split_k;  // holds by the choice of `share`
      if (slot_ok) {
        const int64_t partial_row =
            (static_cast<int64_t>(done_seq) * p.split_k + split_slot) * p.q_heads +
            static_cast<int64_t>(kv_head) * QF_GQA_GROUP;
        float4* row = reinterpret_cast<float4*>(p.partial_out + partial_row * QF_HEAD_DIM) + lane;
#pragma unroll
        for (int head = 0; head < QF_GQA_GROUP; ++head) {
          row[head * (QF_HEAD_DIM / 4)] = *reinterpret_cast<const float4*>(mine + head * kDepositHeadStride + 4 * lane);
        }
        if (g == 0 && q < QF_GQA_GROUP / 2) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            p.partial_max[partial_row + 2 * q + h] = offset[h] * kLn2;  // natural-log units for the combine
            p.partial_sum[partial_row + 2 * q + h] = total[h];
            if (first_page[done_seq + 1] <= end && split_slot + 1 < p.split_k) {
              p.partial_sum[partial_row + p.q_heads + 2 * q + h] = -1.f;  // no further pieces of this sequence
            }
          }
        }
      }
      __syncwarp();  // the buffer is read before the next piece overwrites it
      continue;
    }
    // ---- deposit this warp's state of the piece; the last warp to arrive merges ----
    long long t_piece = 0;
    if (PROFILE) t_piece = global_nanoseconds(), ++pieces;
    const int parity = done_rank & 1;
    if (lane == 0) {
      // Piece done_rank - 2 used the same buffers: they are free once it is merged.
      int rounds = 0;
      while (load_acquire(&merged[parity]) < done_rank - 2) {
        if (++rounds > kMergePollRounds) {
          atomicMax(p.status, kStatusMergeTimeout);
          break;
        }
        __nanosleep(64);
      }
    }
    __syncwarp();
    float* mine = deposits + (parity * kMmaWarps + warp) * kDepositFloats;  // [6 heads][dim]
    if (q < QF_GQA_GROUP / 2) {
      float* even = mine + (2 * q) * kDepositHeadStride + (FP8 ? 2 * g : g);
      float* odd = even + kDepositHeadStride;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        even[16 * j] = acc[j][0], odd[16 * j] = acc[j][1];
        even[16 * j + (FP8 ? 1 : 8)] = acc[j][2], odd[16 * j + (FP8 ? 1 : 8)] = acc[j][3];
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float total = sum[h];
      total += __shfl_xor_sync(kFull, total, 4);
      total += __shfl_xor_sync(kFull, total, 8);
      total += __shfl_xor_sync(kFull, total, 16);
      if (g == 0) warp_offset[parity][warp][2 * q + h] = offset[h], warp_sum[parity][warp][2 * q + h] = total;
    }
    __syncwarp();
    // Warps with pages in the piece: consecutive pages go to consecutive warps.
    const int piece_pages = piece_end - piece_begin;
    const int first_warp = (piece_begin - begin) & (kMmaWarps - 1);
    const int participants = min(piece_pages, kMmaWarps);
    int last = 0;
    if (lane == 0) last = add_acq_rel(&arrived[parity], 1) == participants - 1;
    last = __shfl_sync(kFull, last, 0);
    long long t_arrived = 0;
    if (PROFILE) t_arrived = global_nanoseconds(), t_deposit += t_arrived - t_piece;
    if (last) {
      // lane = (warp w = lane / 4, head pair q): weight of w's deposit, per head
      const int w = lane >> 2;
      const bool took_part = ((w - first_warp) & (kMmaWarps - 1)) < piece_pages;
      float top[2], total[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float mw = took_part ? warp_offset[parity][w][2 * q + h] : -INFINITY;
        float best = mw;
        best = fmaxf(best, __shfl_xor_sync(kFull, best, 4));
        best = fmaxf(best, __shfl_xor_sync(kFull, best, 8));
        best = fmaxf(best, __shfl_xor_sync(kFull, best, 16));
        const float weight = mw == -INFINITY ? 0.f : fast_exp2(mw - best);
        warp_weight[parity][w][2 * q + h] = weight;
        float part = took_part ? warp_sum[parity][w][2 * q + h] * weight : 0.f;
        part += __shfl_xor_sync(kFull, part, 4);
        part += __shfl_xor_sync(kFull, part, 8);
        part += __shfl_xor_sync(kFull, part, 16);
        top[h] = best, total[h] = part;
      }
      __syncwarp();
      const int split_slot = cta - seq_first / share;
      const bool slot_ok = split_slot >= 0 && split_slot < p.split_k;  // holds by the choice of `share`
      const int64_t partial_row =
          (static_cast<int64_t>(done_seq) * p.split_k + split_slot) * p.q_heads +
          static_cast<int64_t>(kv_head) * QF_GQA_GROUP;
      if (slot_ok) {
        // A lane sums four dims (4 lane .. 4 lane + 3) of each head over the deposits.
        const float* base = deposits + parity * kMmaWarps * kDepositFloats + 4 * lane;
        float4 value[QF_GQA_GROUP];
#pragma unroll
        for (int head = 0; head < QF_GQA_GROUP; ++head) value[head] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < participants; ++k) {
          const int ww = (first_warp + k) & (kMmaWarps - 1);
#pragma unroll
          for (int head = 0; head < QF_GQA_GROUP; ++head) {
            const float weight = warp_weight[parity][ww][head];
            const float4 part =
                *reinterpret_cast<const float4*>(base + ww * kDepositFloats + head * kDepositHeadStride);
            value[head].x += part.x * weight, value[head].y += part.y * weight;
            value[head].z += part.z * weight, value[head].w += part.w * weight;
          }
        }
        float4* row = reinterpret_cast<float4*>(p.partial_out + partial_row * QF_HEAD_DIM) + lane;
#pragma unroll
        for (int head = 0; head < QF_GQA_GROUP; ++head) row[head * (QF_HEAD_DIM / 4)] = value[head];
        if (w == 0 && q < QF_GQA_GROUP / 2) {
          // lanes 0..2 hold (top, total) of heads (2q, 2q+1); natural-log units for the combine
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            p.partial_max[partial_row + 2 * q + h] = top[h] * kLn2;
            p.partial_sum[partial_row + 2 * q + h] = total[h];
            if (first_page[done_seq + 1] <= end && split_slot + 1 < p.split_k) {
              p.partial_sum[partial_row + p.q_heads + 2 * q + h] = -1.f;  // no further pieces of this sequence
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) {
        arrived[parity] = 0;
        store_release(&merged[parity], done_rank);
      }
    }
    if (PROFILE && last) t_merge += global_nanoseconds() - t_arrived, ++merges;
  }
  wait_all_copies();
  if constexpr (SOLO) {
    // ---- pieces of one sequence in consecutive blocks of this CTA become one piece.  The warp
    // whose block holds the first of them (chain_seq) announces the chain; after the CTA's only
    // barrier past the work list, the warps share the (chain, query head) pairs: one of them
    // sums that head over the deposits of the warps up to the one that holds the sequence's (or
    // the share's) end, a lane four dims, the weights recomputed by every lane from the offsets. ----
    // A chain of up to kSoloOwnChain warps is summed by its first warp alone (many short chains:
    // all of them at once); a longer one is announced and its six heads are shared out (few long
    // chains).  Measured per 28-layer step, first warp alone / all shared / this rule: 64 x
    // U[128, 4096] tokens 0.800 / 0.786 ms, 256 x log-uniform [64, 8192] 2.142 / 2.158 ms.
    constexpr int kSoloOwnChain = 3;
    const int chain_warps = chain_seq >= 0 ? warp_of(min(first_page[chain_seq + 1], end) - 1 - begin) - warp + 1 : 0;
    const bool own_chain = chain_warps > 0 && chain_warps <= kSoloOwnChain;
    if (lane == 0) {
      chain_of[warp][0] = own_chain ? -1 : chain_seq, chain_of[warp][1] = chain_buffer, chain_of[warp][2] = chain_warps;
    }
    long long t_loop_end = 0, t_barrier = 0;
    if (PROFILE) t_loop_end = global_nanoseconds();
    __syncthreads();
    if (PROFILE) t_barrier = global_nanoseconds(), t_deposit = t_barrier - t_loop_end;  // warp 0's wait at the barrier
    if (own_chain) {
      const int seq_first = first_data_unit(chain_seq);
      const int chain_end = min(first_page[chain_seq + 1], end);         // unit after the chain's last page
      const int participants = chain_warps;                              // this warp and the ones after it
      // lane = (member m = lane / 4, head pair q): weight of m's deposit, per head
      const int m = lane >> 2;
      const bool took_part = m < participants;
      const int member_buffer = m == 0 ? chain_buffer : 0;
      float top[2], total[2], weight[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float mw = took_part ? warp_offset[member_buffer][warp + m][2 * q + h] : -INFINITY;
        float best = mw;
        best = fmaxf(best, __shfl_xor_sync(kFull, best, 4));
        best = fmaxf(best, __shfl_xor_sync(kFull, best, 8));
        best = fmaxf(best, __shfl_xor_sync(kFull, best, 16));
        weight[h] = mw == -INFINITY ? 0.f : fast_exp2(mw - best);
        float part = took_part ? warp_sum[member_buffer][warp + m][2 * q + h] * weight[h] : 0.f;
        part += __shfl_xor_sync(kFull, part, 4);
        part += __shfl_xor_sync(kFull, part, 8);
        part += __shfl_xor_sync(kFull, part, 16);
        top[h] = best, total[h] = part;
      }
      const int split_slot = cta - seq_first / share;
      if (split_slot >= 0 && split_slot < p.split_k) {  // holds by the choice of `share`
        const int64_t partial_row =
            (static_cast<int64_t>(chain_seq) * p.split_k + split_slot) * p.q_heads +
            static_cast<int64_t>(kv_head) * QF_GQA_GROUP;
        // A lane sums four dims (4 lane .. 4 lane + 3) of each head over the deposits.
        float4 value[QF_GQA_GROUP];
#pragma unroll
        for (int head = 0; head < QF_GQA_GROUP; ++head) value[head] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < participants; ++k) {
          const float* from = deposits + (((k == 0 ? chain_buffer : 0) * kMmaWarps) + warp + k) * kDepositFloats + 4 * lane;
#pragma unroll
          for (int head = 0; head < QF_GQA_GROUP; ++head) {
            const float even = __shfl_sync(kFull, weight[0], 4 * k + (head >> 1));
            const float odd = __shfl_sync(kFull, weight[1], 4 * k + (head >> 1));
            const float w = (head & 1) ? odd : even;
            const float4 part = *reinterpret_cast<const float4*>(from + head * kDepositHeadStride);
            value[head].x += part.x * w, value[head].y += part.y * w;
            value[head].z += part.z * w, value[head].w += part.w * w;
          }
        }
        float4* row = reinterpret_cast<float4*>(p.partial_out + partial_row * QF_HEAD_DIM) + lane;
#pragma unroll
        for (int head = 0; head < QF_GQA_GROUP; ++head) row[head * (QF_HEAD_DIM / 4)] = value[head];
        if (m == 0 && q < QF_GQA_GROUP / 2) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            p.partial_max[partial_row + 2 * q + h] = top[h] * kLn2;
            p.partial_sum[partial_row + 2 * q + h] = total[h];
            if (first_page[chain_seq + 1] <= end && split_slot + 1 < p.split_k) {
              p.partial_sum[partial_row + p.q_heads + 2 * q + h] = -1.f;  // no further pieces of this sequence
            }
          }
        }
      }
    }
    // items (chain headed by warp `first`, query head): item t goes to warp t % 8, so the six
    // heads of a chain are summed by six warps at once
    for (int t = warp; t < kMmaWarps * QF_GQA_GROUP; t += kMmaWarps) {
      const int first = t / QF_GQA_GROUP, head = t - first * QF_GQA_GROUP;
      const int sequence = chain_of[first][0];
      if (sequence < 0) continue;
      if (PROFILE) ++merges;
      const int first_buffer = chain_of[first][1], participants = chain_of[first][2];
      // every load unconditional (of a member that exists in shared memory, whether or not it
      // belongs to the chain) and independent of the others; what does not belong is selected away
      float member_offset[kMmaWarps], member_sum[kMmaWarps], best = -INFINITY;
      float4 part[kMmaWarps];
#pragma unroll
      for (int k = 0; k < kMmaWarps; ++k) {
        const int member = min(first + k, kMmaWarps - 1), buffer = k == 0 ? first_buffer : 0;
        member_offset[k] = warp_offset[buffer][member][head];
        member_sum[k] = warp_sum[buffer][member][head];
        part[k] = *reinterpret_cast<const float4*>(deposits + (buffer * kMmaWarps + member) * kDepositFloats +
                                                   head * kDepositHeadStride + 4 * lane);
        if (k >= participants) member_offset[k] = -INFINITY;
        best = fmaxf(best, member_offset[k]);
      }
      float total = 0.f;
      float4 value = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int k = 0; k < kMmaWarps; ++k) {
        const bool in = k < participants && member_offset[k] != -INFINITY;
        const float w = in ? fast_exp2(member_offset[k] - best) : 0.f;
        total += in ? member_sum[k] * w : 0.f;
        value.x += in ? part[k].x * w : 0.f, value.y += in ? part[k].y * w : 0.f;
        value.z += in ? part[k].z * w : 0.f, value.w += in ? part[k].w * w : 0.f;
      }
      const int split_slot = cta - first_data_unit(sequence) / share;
      if (split_slot >= 0 && split_slot < p.split_k) {  // holds by the choice of `share`
        const int64_t partial_row =
            (static_cast<int64_t>(sequence) * p.split_k + split_slot) * p.q_heads +
            static_cast<int64_t>(kv_head) * QF_GQA_GROUP + head;
        reinterpret_cast<float4*>(p.partial_out + partial_row * QF_HEAD_DIM)[lane] = value;
        if (lane == 0) {
          p.partial_max[partial_row] = best * kLn2;  // natural-log units for the combine
          p.partial_sum[partial_row] = total;
          if (first_page[sequence + 1] <= end && split_slot + 1 < p.split_k) {
            p.partial_sum[partial_row + p.q_heads] = -1.f;  // no further pieces of this sequence
          }
        }
      }
    }
    if (PROFILE) t_merge = global_nanoseconds() - t_barrier;  // warp 0's share of the merges
  }
  if (PROFILE) {
    __syncthreads();  // the CTA's exit time is that of its last warp
    if (p.cycles != nullptr && tid == 0) {
      long long* dst = p.cycles + static_cast<int64_t>(blockIdx.x) * kTimelineColumns;
      // (warp 0 stamps the first tile; in the solo variant its block may hold empty units only)
      dst[0] = t_entry, dst[1] = t_list, dst[2] = t_ids, dst[3] = t_first != 0 ? t_first : t_ids;
      dst[4] = global_nanoseconds();
      dst[5] = count, dst[6] = pieces, dst[7] = t_deposit, dst[8] = t_merge, dst[9] = merges;
    }
  }
}

}  // namespace
}  // namespace qf
