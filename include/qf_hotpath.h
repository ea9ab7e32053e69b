/*
 * qf_hotpath.h -- C ABI of libqf_hotpath.so: the decode-step attention hot path
 * of Qwen-frence (fused RoPE + paged KV-cache write, GQA paged decode attention
 * with split-K partial softmax and combine, optional FP8-e4m3 KV cache) as
 * hand-written sm_100a CUDA kernels.
 *
 * Conventions
 *   - Every pointer marked "device" is a CUDA device pointer owned by the
 *     caller.  The library allocates no device memory, ever, and keeps no
 *     per-pool state.
 *   - `stream` is a cudaStream_t passed as void*.  Every call only enqueues
 *     work on that stream: no host synchronisation, no device->host read, so
 *     every call may be recorded into a CUDA graph.
 *   - Strides are in ELEMENTS of the tensor's dtype, like torch's.
 *   - Return value: 0 on success, a negative QF_E* code otherwise;
 *     qf_last_error() then returns a message for the calling thread.
 *   - Threads: every call may be made from any thread, and calls on different
 *     streams may run concurrently; the error text is per thread.  Three switches
 *     are process-wide (atomic, but one switch each): qf_set_tuning,
 *     qf_set_dependent_launch, and the one-shot request of qf_order_next_launch,
 *     which is consumed by the NEXT chained launch of the process whichever thread
 *     or stream makes it.  A host with several launching threads must make that
 *     request and the launch it is meant for on one thread with no other launch of
 *     this library in between.  The reference engine is driven by a single host
 *     thread on one stream (engine/cpp/include/iteration_loop.hpp:157-161).
 *
 * Each entry point cites the reference interface it replaces, by path inside
 * the benjaminW2025/qwen-frence tree.
 */
#ifndef QF_HOTPATH_H_
#define QF_HOTPATH_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QF_ABI_VERSION 1

/* element types of Q/K/V and the pools */
#define QF_DTYPE_F16 0
#define QF_DTYPE_BF16 1
/* element types of metadata tensors (positions, slots, block table, lengths) */
#define QF_INDEX_I32 0
#define QF_INDEX_I64 1
#define QF_INDEX_F32 2 /* positions only */

#define QF_OK 0
#define QF_EINVAL (-1)   /* bad argument (shape, dtype, alignment, null) */
#define QF_ECUDA (-2)    /* a CUDA runtime/driver call failed */
#define QF_EUNSUPPORTED (-3)

/* Fixed geometry of the fast kernels (baseline/naive_forward.py:17-26). */
#define QF_HEAD_DIM 128
#define QF_PAGE_SIZE 16
#define QF_GQA_GROUP 6

int qf_abi_version(void);
const char* qf_last_error(void);

/* ------------------------------------------------------------------------
 * Fused RoPE + paged KV-cache write.
 *
 * One generic entry point; the three reference functions differ only in the
 * strides they pass:
 *   rope_kv_write                 custom_kernels/rope_kv_write.py:89-162
 *       q (1,Hq,T,D): row stride = stride(2), head stride = stride(1)
 *   native_decode_rope_kv_write   custom_kernels/rope_kv_write.py:223-276
 *       q (B,Hq,1,D): row stride = stride(0), head stride = stride(1)
 *   packed_qkv_rope_cache         custom_kernels/packed_qkv_rope_cache.py:91-133
 *       packed (rows,2048): q = packed, k = packed+1536*sd, v = packed+1792*sd,
 *       head stride = 128*sd, row stride = stride(0), d stride = sd = stride(1)
 *
 * For every row r < rows and every rotary pair (i, i+D/2):
 *   inv_freq[i] = expf(i * (-(float)log(base) / (D/2)))      (host, fp32)
 *   angle = (float)positions[r] * inv_freq[i];  c = cosf(angle); s = sinf(angle)
 *   out[i] = x[i]*c - x[i+D/2]*s;  out[i+D/2] = x[i+D/2]*c + x[i]*s   (fp32,
 *   one rounding to the element type on store)
 * Q heads go to q_out (skipped when rotate_q == 0); K heads (rotated) and V
 * heads (bit-exact copy) go to pool row `slot_mapping[r]` of the flat
 * [slots, kv_heads, D] view of k_pool / v_pool.
 * `valid_tokens` (device int32 scalar, may be NULL): rows >= *valid_tokens
 * write zeros to q_out and do not touch the pools.
 * ------------------------------------------------------------------------ */
typedef struct qf_rope_kv_write_args {
  const void* q;  /* device, may be NULL when rotate_q == 0 */
  const void* k;  /* device */
  const void* v;  /* device */
  void* q_out;    /* device, may be NULL when rotate_q == 0 */
  int64_t q_stride_row, q_stride_head, q_stride_d;
  int64_t k_stride_row, k_stride_head, k_stride_d;
  int64_t v_stride_row, v_stride_head, v_stride_d;
  int64_t o_stride_row, o_stride_head, o_stride_d;
  const void* positions;    /* device, [rows] */
  int32_t positions_dtype;  /* QF_INDEX_* */
  int64_t positions_stride;
  const void* slot_mapping; /* device, [rows] */
  int32_t slot_dtype;       /* QF_INDEX_I32 / I64 */
  int64_t slot_stride;
  void* k_pool; /* device, flat [slots, kv_heads, D] view */
  void* v_pool; /* device */
  int64_t kp_stride_slot, kp_stride_head, kp_stride_d;
  int64_t vp_stride_slot, vp_stride_head, vp_stride_d;
  int64_t num_slots;           /* pool rows; slots outside [0,num_slots) are skipped */
  const int32_t* valid_tokens; /* device scalar or NULL */
  int32_t rows, q_heads, kv_heads, head_dim;
  int32_t dtype;    /* QF_DTYPE_* of q/k/v/q_out/pools */
  int32_t rotate_q; /* 0: only the kv_heads K/V segments are processed */
  double base;      /* rope theta */
} qf_rope_kv_write_args;

int qf_rope_kv_write(const qf_rope_kv_write_args* args, void* stream);

/* Same, but the pools are FP8-e4m3 bytes with one fp32 scale per
 * (page, kv head): byte = e4m3_rn_satfinite(clamp(x / scale, +-448)) where
 * scale = {k,v}_scale[(slot / page_size) * kv_heads + head].  The scales are
 * read, never written (fixed-scale write; nearest reference:
 * experiments/quant/kernels/staged_cache.py:39-55, codec
 * experiments/quant/attention.py:27-50).  The reference has no per-page-scale
 * paged cache; this layout is defined here.  k_pool/v_pool strides are in
 * bytes == elements. */
int qf_rope_kv_write_fp8(const qf_rope_kv_write_args* args, const float* k_scale,
                         const float* v_scale, int32_t page_size, void* stream);

/* Quantise whole fp16/bf16 pools [pages, page_size, kv_heads, D] (contiguous)
 * to e4m3 pools of the same shape plus scales [pages, kv_heads]:
 * scale = max(amax(page, head)/448, 1e-12)
 * (experiments/quant/attention.py:27-41, page granularity instead of token). */
int qf_quantize_kv_pages_e4m3(const void* pool, int32_t dtype, int64_t num_pages,
                              int32_t page_size, int32_t kv_heads, int32_t head_dim,
                              void* pool8, float* scales, void* stream);

/* ------------------------------------------------------------------------
 * GQA paged decode attention, split-K partial pass.
 * Replaces grouped_gqa_splitk_partial_out
 * (custom_kernels/native_grouped_decode/native_grouped_decode.cu:329-403) and
 * _grouped_splitk_kernel (custom_kernels/paged_decode_grouped_splitk.py:28-158).
 *
 * Partition `s` of sequence `b` covers logical pages
 * [s*P/split_k, (s+1)*P/split_k), P = ceil(seq_lens[b]/page_size).
 * Outputs (fp32, contiguous):
 *   partial_out [batch, split_k, q_heads, D]  un-normalised sum of p*V
 *   partial_max [batch, split_k, q_heads]     exponent offset m (natural-log
 *                                             units of score*scale); -inf if empty
 *   partial_sum [batch, split_k, q_heads]     sum of exp(score*scale - m); 0 if empty
 * with p = exp(score*scale - m).  m is an upper-bounded running offset, not
 * necessarily the exact maximum: (out, m, sum) is self-consistent, which is
 * all the combine needs.
 * When split_k == 1 and out != NULL the kernel also writes the normalised
 * result to `out` in the q dtype (rows with seq_len 0 give zeros) and the
 * partial pointers may be NULL.
 * k_scale/v_scale: NULL for 16-bit pools; for FP8-e4m3 pools (kv_fp8 != 0)
 * device fp32 [num_pages, kv_heads].
 * ------------------------------------------------------------------------ */
typedef struct qf_decode_attention_args {
  const void* q; /* device [batch, q_heads, D] */
  int64_t q_stride_b, q_stride_h, q_stride_d;
  const void* k_pool; /* device [num_pages, page_size, kv_heads, D] */
  const void* v_pool;
  int64_t k_stride_page, k_stride_tok, k_stride_head, k_stride_d;
  int64_t v_stride_page, v_stride_tok, v_stride_head, v_stride_d;
  const void* block_table; /* device [batch, table_width]; a seq_lens entry beyond
                              table_width * page_size tokens is cut to that, so no
                              kernel reads past a table row */
  int32_t table_dtype;     /* QF_INDEX_I32 / I64 */
  int64_t table_stride_b, table_stride_p;
  int64_t table_width;
  const void* seq_lens; /* device [batch] */
  int32_t lens_dtype;
  int64_t lens_stride;
  const float* k_scale; /* device or NULL */
  const float* v_scale;
  float* partial_out; /* device, see above */
  float* partial_max;
  float* partial_sum;
  void* out; /* device [batch, q_heads, D] in q dtype, or NULL */
  int64_t o_stride_b, o_stride_h, o_stride_d;
  int64_t num_pages;
  int32_t batch, q_heads, kv_heads, head_dim, page_size;
  int32_t split_k;
  int32_t dtype;  /* QF_DTYPE_* of q/out (and of the pools unless kv_fp8) */
  int32_t kv_fp8; /* 0: pools in `dtype`; 1: pools are e4m3 bytes */
  float scale;    /* softmax scale */
} qf_decode_attention_args;

int qf_grouped_gqa_splitk_partial_out(const qf_decode_attention_args* args, void* stream);

/* Split-K combine.  Replaces _splitk_reduce_kernel
 * (custom_kernels/paged_decode_grouped_splitk.py:165-226): log-sum-exp merge of
 * the partitions with partial_sum > 0, out = acc / (sum > 0 ? sum : 1).
 * Partial strides are in fp32 elements; `out` is in `dtype`. */
int qf_splitk_reduce(const float* partial_out, const float* partial_max,
                     const float* partial_sum, int64_t po_stride_b, int64_t po_stride_k,
                     int64_t po_stride_h, int64_t po_stride_d, int64_t pm_stride_b,
                     int64_t pm_stride_k, int64_t pm_stride_h, void* out,
                     int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_d,
                     int32_t batch, int32_t q_heads, int32_t head_dim, int32_t split_k,
                     int32_t dtype, void* stream);

/* Partial pass + combine in one call (two launches; one when split_k == 1).
 * Replaces grouped_splitk_decode_attention
 * (custom_kernels/paged_decode_grouped_splitk.py:228-334) and
 * native_grouped_splitk_decode_attention
 * (custom_kernels/paged_decode_native_grouped.py:30-88).  `out` is required.
 *
 * The partial buffers are scratch of this call: for the Qwen geometry
 * (D = 128, page 16, six query heads per KV head, unit inner strides, K and V pools
 * with equal strides) with split_k >= 2 and batch <= 1024 the partial pass is a
 * persistent kernel whose CTAs share the batch's pages equally; a sequence then
 * fills only its first few split slots (one per CTA that holds some of its pages),
 * the slot after them carries partial_sum = -1, and split boundaries depend on the
 * whole batch.
 * Callers that need the reference's partitions call
 * qf_grouped_gqa_splitk_partial_out and qf_splitk_reduce instead. */
int qf_grouped_splitk_decode_attention(const qf_decode_attention_args* args, void* stream);

/* The two launches of qf_grouped_splitk_decode_attention separately, for callers
 * that time or schedule them apart (no counterpart in the reference):
 * QF_STAGE_PARTIAL runs only the partial pass, QF_STAGE_COMBINE only the combine
 * of partials left by an earlier QF_STAGE_PARTIAL call with the same arguments;
 * both bits are the fused call.  split_k == 1 has a single launch, which belongs
 * to QF_STAGE_PARTIAL. */
#define QF_STAGE_PARTIAL 1
#define QF_STAGE_COMBINE 2
int qf_grouped_splitk_decode_attention_stages(const qf_decode_attention_args* args, int32_t stages,
                                              void* stream);

/* Which partial kernel qf_grouped_splitk_decode_attention would launch for these
 * arguments on the current device, without launching anything: *kernel is
 * QF_KERNEL_PARTITIONED (one CTA per sequence, KV head and split; also the
 * stride-generic kernel), QF_KERNEL_PERSISTENT (CUDA-core math; only when forced
 * with qf_set_tuning), QF_KERNEL_PERSISTENT_MMA (tensor-core math, 16-bit and FP8
 * pools; only behind qf_set_tuning mode 4 and as the instrumented kernel) or
 * QF_KERNEL_PERSISTENT_MMA_SOLO (the tensor-core kernel of every call whose layout allows
 * it: each warp streams a block of consecutive pages on its own, and what a CTA's warps hold
 * of one sequence is merged once, at the CTA's end); *ctas_per_head
 * is the number of resident CTAs that share one KV head's pages (0 for
 * QF_KERNEL_PARTITIONED). */
#define QF_KERNEL_PARTITIONED 0
#define QF_KERNEL_PERSISTENT 1
#define QF_KERNEL_PERSISTENT_MMA 2
#define QF_KERNEL_PERSISTENT_MMA_SOLO 3
int qf_grouped_splitk_decode_attention_plan(const qf_decode_attention_args* args, int32_t* kernel,
                                            int32_t* ctas_per_head);

/* Instrumented run of the tensor-core persistent partial pass, 16-bit or FP8 pools
 * (QF_EINVAL when the arguments select another kernel): timeline [kv_heads * ctas_per_head][10] int64,
 * per CTA {ns at entry, ns when the work list was built, ns when its page ids were
 * known, ns when its first K tile had landed, ns at exit (of its last warp), units
 * in its share (pages plus up to six empty units per sequence), pieces that held pages of its warp 0, ns warp 0 spent depositing
 * its piece states, ns warp 0 spent merging pieces, pieces warp 0 merged}; times
 * from %globaltimer (one clock for all SMs, 256 ns steps on B200);
 * CTAs without work leave their row untouched.  Plays the role of
 * grouped_gqa_splitk_profile_out
 * (custom_kernels/native_grouped_decode/native_grouped_decode.cu:405-459) for
 * this kernel, whose CTAs are not tied to a (sequence, head, split). */
int qf_grouped_splitk_persistent_timeline(const qf_decode_attention_args* args, int64_t* timeline,
                                          void* stream);

/* The same computation as qf_grouped_splitk_decode_attention, for callers that
 * cannot provide (or allocate) the split-K partial buffers.  No counterpart in
 * the reference: its wrappers always allocate partials with torch.  Meant for
 * hosts without a caching allocator (a C++ serving loop bound straight to this
 * ABI, where a cudaMalloc/cudaFree per decode step would synchronise the device)
 * and for processes that gave all device memory to their own allocator at start,
 * where a later cudaMalloc fails.
 *   - args->partial_out / partial_max / partial_sum are IGNORED; the partials
 *     live in a static device array of QF_STATIC_SCRATCH_BYTES that every GPU
 *     loading this library holds until the process exits.  q, pools, tables and
 *     `out` are still the caller's.
 *   - Limit: batch * split_k * q_heads * (head_dim + 2) * 4 bytes must fit; a
 *     larger request returns QF_EINVAL with the numbers in qf_last_error().
 *   - The call allocates nothing (no cudaMalloc, cudaFree or allocating library
 *     routine).  The FIRST call on each device looks up the array's device
 *     address (cudaGetSymbolAddress, with that device current): make that first
 *     call before any stream capture begins.
 *   - All calls on a device share the one array and it keeps the previous
 *     call's contents.  Nothing in it needs clearing (the partial pass rewrites
 *     every row the combine reads), but two calls whose kernels overlap on the
 *     GPU (different streams, or several host threads) race on it: keep them on
 *     one stream or order them with events. */
#define QF_STATIC_SCRATCH_BYTES (16u << 20)
int qf_grouped_splitk_decode_attention_static(const qf_decode_attention_args* args, void* stream);

/* Compiled resources and occupancy of the fast partial kernel for `dtype` /
 * `kv_fp8` on `device`.  Replaces grouped_gqa_splitk_diagnostics
 * (native_grouped_decode.cu:310-327).  Fills
 *   info[0] registers_per_thread   info[1] static_shared_bytes
 *   info[2] dynamic_shared_bytes   info[3] local_bytes_per_thread
 *   info[4] max_threads_per_block  info[5] binary_version
 *   info[6] ptx_version            info[7] threads_per_block
 *   info[8] active_blocks_per_sm   info[9] max_warps_per_sm
 *   info[10] pipeline_stages       info[11] multiprocessor_count */
#define QF_KERNEL_INFO_FIELDS 12
int qf_grouped_gqa_splitk_diagnostics(int32_t device, int32_t dtype, int32_t kv_fp8,
                                      int64_t* info);

/* Instrumented partial pass.  Replaces grouped_gqa_splitk_profile_out
 * (native_grouped_decode.cu:405-459): same outputs as the partial pass plus
 * cycles [batch, kv_heads, split_k, 4] (device int64): clock64() cycles one
 * warp of each CTA of the per-partition kernel spent {waiting for pages, in the
 * whole page loop, in the set-up before it, in the merge after it} (loads overlap
 * the math, so there is no separate QK / softmax / PV stage to time). */
int qf_grouped_gqa_splitk_profile_out(const qf_decode_attention_args* args,
                                      int64_t* cycles, void* stream);

/* Device-side status word of the kernels on the current device: the LARGEST code any
 * kernel has recorded since the last reset (kernels record with an atomic maximum, so
 * a later, smaller code does not hide an earlier, larger one).  0: nothing; 2 when a
 * kernel met a page id outside the pool (such a page is never dereferenced; it
 * reads as zeros); 3 when a warp of the tensor-core persistent kernel gave up its
 * bounded poll for an earlier sequence's merge (the one wait in the library that
 * is not a hardware wait_group or barrier; the result of that call is then
 * unreliable); 4 when qf_advance_decode_metadata moved a position beyond its block
 * table; 5 when a bounded barrier wait of qf_qkv_rope_cache ran out.  Synchronises
 * the device; for tests and debugging only.  `reset` != 0 clears it after reading. */
int qf_device_status(int32_t* status, int32_t reset);

/* Programmatic dependent launch (on by default).  The RoPE / KV-write kernel, the
 * tensor-core partial pass and the combine for split_k <= 256 are launched with
 * cudaLaunchAttributeProgrammaticStreamSerialization: each may become resident
 * while the previous kernel of the stream is still running, does its index set-up
 * then, and waits (griddepcontrol.wait) for that kernel to complete and flush
 * before it reads any tensor or writes anything.  The exceptions: during that set-up
 * the partial pass reads seq_lens and the block table -- and, in
 * qf_packed_rope_decode_attention, the positions, and it requests K / V tiles of pages
 * that do not hold a sequence's newest token (see there) -- i.e. possibly before the
 * kernel launched two places earlier on the stream has flushed.  Step metadata
 * that arrives by a copy (the usual case) is ordered as usual; metadata that a
 * KERNEL updates in place on the same stream must be followed by
 * qf_order_next_launch() (qf_advance_decode_metadata does that itself).
 * enabled == 0 launches everything the ordinary way (process-wide, read at launch
 * and capture time). */
int qf_set_dependent_launch(int32_t enabled);

/* The next kernel this library launches from the calling process is launched the
 * ordinary way (it starts after everything earlier on its stream has completed and
 * flushed), whatever qf_set_dependent_launch says; later launches chain again.
 * Call it after a kernel of your own has written positions, seq_lens, the slot
 * mapping or the block table in place on the stream. */
int qf_order_next_launch(void);

/* ------------------------------------------------------------------------
 * Device-side advance of the step metadata of a stable decode cohort, in place,
 * so that consecutive decode steps (or the K steps of an unrolled graph) need no
 * host rebuild and no host-to-device copy.  Replaces the torch ops of
 * IterationLoop::advance_decode_state (engine/cpp/src/iteration_loop.cpp:500-528;
 * the per-step tensors of engine/graph/unrolled_graph_decoder.py:92-130 are its
 * K-fold application).  For every b < batch:
 *   positions[b] += 1;  seq_lens[b] += 1;
 *   slot_mapping[b] = block_table[b, positions[b] / page_size] * page_size
 *                     + positions[b] % page_size          (the NEW position)
 * The table is immutable for the cohort (requests reserve their whole page
 * sequence at admission).  A position whose logical page lies beyond table_width,
 * or whose page id is outside [0, num_pages), gets slot -1 -- which the KV-write
 * kernel skips -- and the device status word becomes 4 / 2; the reference's
 * gather would fault there.  positions, seq_lens, slot_mapping: int32 or int64,
 * contiguous; block_table int32 or int64 with strides in elements.
 * Ends with qf_order_next_launch(). */
#define QF_STATUS_BAD_PAGE_ID 2
#define QF_STATUS_MERGE_TIMEOUT 3
#define QF_STATUS_POSITION_PAST_TABLE 4
#define QF_STATUS_PIPELINE_TIMEOUT 5
int qf_advance_decode_metadata(void* positions, int32_t positions_dtype,
                               void* seq_lens, int32_t lens_dtype,
                               void* slot_mapping, int32_t slot_dtype,
                               const void* block_table, int32_t table_dtype,
                               int64_t table_stride_b, int64_t table_stride_p,
                               int64_t table_width, int64_t num_pages,
                               int32_t batch, int32_t page_size, void* stream);

/* ------------------------------------------------------------------------
 * RMSNorm and residual-add + RMSNorm, the steps either side of attention in a
 * decode layer.  Replace rms_norm (custom_kernels/fused_rms.py:52-75) and
 * residual_add_rms_norm (custom_kernels/fused_rms.py:107-135; caller
 * engine/graph/paged_graph_decoder.py:303-309, :325-331).  Per row of `hidden`
 * fp16 / bf16 elements (row strides in elements, unit stride inside a row):
 *   summed     = T(residual + branch)                      (stored; residual form only)
 *   rms        = sqrtf(sum(float(summed)^2) / hidden + epsilon)
 *   normalized = T(float(weight) * float(summed) / rms)
 * `summed` is the exact fp16 / bf16 sum; the normalisation reads that rounded
 * value, as the reference does.  Inputs and outputs may alias row for row
 * (summed == residual, out == x).  rows == 0 is a no-op. */
int qf_rms_norm(const void* x, int64_t x_row_stride, const void* weight, void* out,
                int64_t out_row_stride, int64_t rows, int32_t hidden, int32_t dtype,
                float epsilon, void* stream);
int qf_residual_add_rms_norm(const void* residual, int64_t residual_row_stride,
                             const void* branch, int64_t branch_row_stride,
                             const void* weight, void* summed, int64_t summed_row_stride,
                             void* normalized, int64_t normalized_row_stride, int64_t rows,
                             int32_t hidden, int32_t dtype, float epsilon, void* stream);

/* ------------------------------------------------------------------------
 * QKV projection with RoPE + paged KV-cache write as its epilogue (decode).
 * Replaces qkv_rope_cache of the reference's CUTLASS extension
 * (custom_kernels/fused_gemm.py:271-278, custom_kernels/gemm_epilogue/
 * fused_gemm.cu:223-310; caller engine/graph/paged_graph_decoder.py:218-224),
 * without its norm-folding row scale:
 *   packed[r, n] = T(sum_k hidden[r, k] * weight[n, k] + bias[n])   n < 2048, fp32 sum
 *   then exactly qf_rope_kv_write on the packed row: Q heads 0-11 rotated into
 *   q_out [rows, 12 * 128]; K heads rotated, V heads as they are, into row
 *   slot_mapping[r] of the flat [slots, 2, 128] view of the pools.
 * Rows >= *valid_tokens (device int32 scalar, may be NULL) get zero queries and no
 * cache write.  A slot outside [0, num_slots) is skipped and recorded (status 2).
 * hidden [rows, in_features] and weight [2048, in_features] (nn.Linear layout):
 * unit stride inside a row, 16-byte aligned, row strides multiples of 8 elements;
 * in_features a multiple of 64; pools contiguous.  An sm_100a tensor-core kernel
 * (TMA operand loads, tcgen05.mma into TMEM); if one of its bounded barrier waits
 * ever ran out the device status word would read 5 and the outputs be unreliable. */
typedef struct qf_qkv_rope_cache_args {
  const void* hidden;        /* device */
  int64_t hidden_stride_row; /* elements */
  const void* weight;        /* device */
  int64_t weight_stride_row;
  const void* bias;          /* device [2048], may be NULL */
  void* q_out;               /* device [rows, >= 1536] */
  int64_t q_stride_row;
  const void* positions;     /* device [rows] */
  int32_t positions_dtype;   /* QF_INDEX_* */
  const void* slot_mapping;  /* device [rows] */
  int32_t slot_dtype;
  void* k_pool;              /* device, flat [num_slots, 2, 128] */
  void* v_pool;
  int64_t num_slots;
  const void* valid_tokens;  /* device int32 scalar or NULL */
  int32_t rows;
  int32_t in_features;
  int32_t dtype;             /* QF_DTYPE_* of hidden, weight, bias, q_out, pools */
  double base;               /* RoPE theta */
} qf_qkv_rope_cache_args;
int qf_qkv_rope_cache(const qf_qkv_rope_cache_args* args, void* stream);

/* The same call with a per-CTA timeline: timeline [CTAs][QF_GEMM_TIMELINE_COLUMNS] (device
 * int64, CTAs = 32 column tiles x ceil(rows / 128) x K split, at most 32 * ceil(rows/128) * 4)
 * receives %globaltimer nanoseconds at {entry, barriers and TMEM ready, previous kernel
 * complete, first operand tiles landed, last MMA issued, accumulator complete, partial sums
 * sent, peers' sums arrived, outputs stored, TMEM released}.  For profiling. */
#define QF_GEMM_TIMELINE_COLUMNS 10
int qf_qkv_rope_cache_timeline(const qf_qkv_rope_cache_args* args, int64_t* timeline, void* stream);

/* ------------------------------------------------------------------------
 * The whole layer step in two launches instead of three: RoPE + KV write folded into
 * the attention partial pass, then the combine.  No counterpart in the reference (it
 * runs packed_qkv_rope_cache, custom_kernels/packed_qkv_rope_cache.py:91-133, and then
 * grouped_splitk_decode_attention, custom_kernels/paged_decode_grouped_splitk.py:228-334);
 * the results are those of that pair, bit for bit in the pools.
 *   args->q            the packed rows [batch, 2048] = [Q0..Q11 | K0 K1 | V0 V1] x 128
 *                      (q_stride_b = row stride, q_stride_h = 128, q_stride_d = 1)
 *   positions          [batch] int32 / int64: rotation position of the row (the engine's
 *                      seq_len - 1), an index into rope_table
 *   rope_table         [table_positions][64] (cos, sin) fp32 pairs from qf_build_rope_table;
 *                      a position outside it is clamped and recorded (status 4)
 * Every warp that works on a sequence rotates its own copy of the six query heads in
 * shared memory (the position's row of the table travels with the Q tile); the warp that
 * owns the sequence's last page stores the rotated K row and the V row at token
 * seq_len - 1 of that page -- the slot the engine's slot mapping names
 * (engine/graph/paged_graph_decoder.py:392-417) -- before it copies the page.  Sequences of
 * length 0 write nothing.  No rotated Q is returned.
 * The slot mapping is NOT an argument: the row goes where block_table and seq_lens say.
 * A caller whose slot mapping names another place (or -1, "skip this row") for a row of
 * the batch must use the operator pair; rows duplicated as padding (the reference's
 * bucketed decoder) are fine, they store identical bytes twice.
 * Contract on the pools (what makes this a decode step): when the call is enqueued, every
 * K / V row of the attended tokens EXCEPT each sequence's newest is already in the pools,
 * written by work that completed before the kernel in front of this call on the stream
 * started (an earlier step, a prefill).  The kernel relies on it: it requests tiles of
 * those older pages before its dependency wait, while the kernels before it drain.  The
 * newest token's page is only copied after this kernel itself has stored the new row.
 * FP8 pools (args->kv_fp8 with k_scale / v_scale): the new K / V rows are stored as e4m3
 * bytes at their page's fixed scales, byte for byte what qf_rope_kv_write_fp8 stores.
 * QF_EUNSUPPORTED unless: 12 + 2 heads, split_k >= 2, and arguments for which
 * qf_grouped_splitk_decode_attention_plan reports QF_KERNEL_PERSISTENT_MMA_SOLO (or, for
 * 16-bit pools, QF_KERNEL_PERSISTENT_MMA: the fused step runs the same variant); callers
 * then run qf_rope_kv_write(_fp8) and qf_grouped_splitk_decode_attention.
 * `stages`: QF_STAGE_PARTIAL | QF_STAGE_COMBINE for the whole step; one of them alone
 * launches only that kernel (timing). */
int qf_packed_rope_decode_attention(const qf_decode_attention_args* args, const void* positions,
                                    int32_t positions_dtype, int64_t positions_stride,
                                    const float* rope_table, int32_t table_positions, int32_t stages,
                                    void* stream);

/* table[position][f] = (cosf(a), sinf(a)), a = (float)position * inv_freq[f], f < 64,
 * inv_freq as in qf_rope_kv_write: the cos / sin cache the model's own RoPE keeps
 * (engine/kvcache/paged_forward.py build_rope_from_positions), in fp32 and with the fused
 * kernels' formula.  `table` holds positions * 64 * 2 floats. */
int qf_build_rope_table(float* table, int32_t positions, double base, void* stream);

/* Switches for tests and experiments (process-wide, read at launch time).
 * force_generic: 0 automatic choice; 1 every attention call goes through the
 * stride-generic kernel; 2 fast per-partition kernel only, no persistent kernel;
 * 3 / 4 the persistent CUDA-core / tensor-core kernel whenever the layout allows,
 * whatever the number of split slots; 5 the tensor-core kernel's solo variant whenever the
 * layout allows (4 never picks that variant).  `stages` is accepted and recorded but the
 * kernels' shared-memory rings have fixed depths chosen at compile time. */
int qf_set_tuning(int32_t stages, int32_t force_generic);

#ifdef __cplusplus
}
#endif
#endif /* QF_HOTPATH_H_ */
