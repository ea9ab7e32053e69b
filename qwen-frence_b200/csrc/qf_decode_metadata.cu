// Device-side advance of the decode-step metadata of a stable cohort: positions
// and lengths move on by one token and the slot of the new position is looked up
// in the (immutable) block table.  One thread per sequence; the whole batch is a
// few hundred bytes, so this kernel is pure launch latency and exists to take the
// host rebuild and the host-to-device copy out of consecutive decode steps.
// Restates IterationLoop::advance_decode_state
// (engine/cpp/src/iteration_loop.cpp:500-528), which does the same with six torch
// ops.
#include "qf_common.cuh"

namespace qf {
namespace {

struct AdvanceParams {
  void* positions;
  void* seq_lens;
  void* slots;
  const void* table;
  int64_t table_stride_b, table_stride_p, table_width, num_pages;
  int* status;
  int pos_dtype, lens_dtype, slot_dtype, table_dtype;
  int batch, page_size;
};

constexpr int kAdvanceThreads = 128;

__global__ void __launch_bounds__(kAdvanceThreads) advance_metadata_kernel(AdvanceParams p) {
  // Chained onto the previous kernel of the stream: resident early, but every kernel that
  // read the old metadata has completed once this wait returns.
  dependency_wait();
  const int b = blockIdx.x * kAdvanceThreads + threadIdx.x;
  if (b >= p.batch) return;
  const int64_t position = load_index(p.positions, p.pos_dtype, b) + 1;
  const int64_t length = load_index(p.seq_lens, p.lens_dtype, b) + 1;
  const int64_t logical_page = position / p.page_size;
  int64_t slot = -1;  // the KV-write kernel skips a row whose slot is out of range
  if (position < 0 || logical_page >= p.table_width) {
    atomicMax(p.status, kStatusPositionPastTable);
  } else {
    const int64_t page =
        load_index(p.table, p.table_dtype, b * p.table_stride_b + logical_page * p.table_stride_p);
    if (page < 0 || page >= p.num_pages) {
      atomicMax(p.status, kStatusBadPageId);
    } else {
      slot = page * p.page_size + position % p.page_size;
    }
  }
  store_index(p.positions, p.pos_dtype, b, position);
  store_index(p.seq_lens, p.lens_dtype, b, length);
  store_index(p.slots, p.slot_dtype, b, slot);
}

bool integer_dtype(int dtype) { return dtype == QF_INDEX_I32 || dtype == QF_INDEX_I64; }

}  // namespace
}  // namespace qf

extern "C" int qf_advance_decode_metadata(void* positions, int32_t positions_dtype, void* seq_lens,
                                          int32_t lens_dtype, void* slot_mapping, int32_t slot_dtype,
                                          const void* block_table, int32_t table_dtype,
                                          int64_t table_stride_b, int64_t table_stride_p,
                                          int64_t table_width, int64_t num_pages, int32_t batch,
                                          int32_t page_size, void* stream) {
  using namespace qf;
  QF_REQUIRE(batch >= 0, "batch must not be negative");
  QF_REQUIRE(page_size > 0, "page size must be positive");
  QF_REQUIRE(table_width >= 0 && num_pages >= 0, "table width and pool size must not be negative");
  QF_REQUIRE(integer_dtype(positions_dtype) && integer_dtype(lens_dtype) && integer_dtype(slot_dtype) &&
                 integer_dtype(table_dtype),
             "positions, lengths, slot mapping and block table must use an integer dtype");
  if (batch == 0) return QF_OK;
  QF_REQUIRE(positions && seq_lens && slot_mapping, "positions, lengths and slot mapping must not be null");
  QF_REQUIRE(block_table != nullptr || table_width == 0, "block table must not be null");
  AdvanceParams p;
  p.positions = positions, p.seq_lens = seq_lens, p.slots = slot_mapping, p.table = block_table;
  p.table_stride_b = table_stride_b, p.table_stride_p = table_stride_p;
  p.table_width = table_width, p.num_pages = num_pages;
  p.status = device_status_word();
  QF_REQUIRE(p.status != nullptr, "device status word is unavailable");
  p.pos_dtype = positions_dtype, p.lens_dtype = lens_dtype, p.slot_dtype = slot_dtype;
  p.table_dtype = table_dtype;
  p.batch = batch, p.page_size = page_size;
  const unsigned blocks = static_cast<unsigned>((batch + kAdvanceThreads - 1) / kAdvanceThreads);
  QF_CUDA(launch_chained(advance_metadata_kernel, dim3(blocks), dim3(kAdvanceThreads), 0,
                         static_cast<cudaStream_t>(stream), p));
  // The kernel that follows must not start early: the partial pass reads lengths and
  // table before its own dependency wait, and may become resident as soon as the kernel
  // before it has started.
  request_ordered_launch();
  return QF_OK;
}
