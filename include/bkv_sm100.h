/*
 * bkv_sm100.h — C ABI of the B200 (sm_100a) packed-KV hot path.
 *
 * One shared library, libbkv_sm100.so, exports the entry points below.  They take
 * raw device pointers, sizes, element strides and a CUDA stream handle; they never
 * allocate (bkv_kv_exchange_alloc, a set-up call, is the one exception), never synchronise
 * and never throw: every call returns BKV_OK or a negative status (see bkv_status_string).  Launch errors reported by the CUDA
 * runtime are returned as BKV_ERR_CUDA and the message is kept per thread
 * (bkv_last_cuda_error).
 *
 * Every entry point names the reference interface (wsxhjnb1/Beyond-KV-Cache,
 * path:line inside that project) that it replaces.
 *
 * Packed page ABI (identical to the reference, quant/beyond_cute.py:675-765):
 * the cache is `int32 [num_pages][page_stride_i32]`; one page holds, in order,
 * K codes, K statistics, V codes, V statistics for `block_size` tokens and
 * `heads_kv` heads of 128 scalars each, quantised in groups of 32 to 4-bit codes
 * (8 codes per 32-bit word, code i in bits 4*(i%8)) with one statistics word per
 * group (low 16 bits = scale, high 16 bits = minimum, both fp16 or bf16).
 */
#ifndef BKV_SM100_H_
#define BKV_SM100_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BKV_ABI_VERSION 2

/* status codes */
#define BKV_OK 0
#define BKV_ERR_ARG (-1)         /* null pointer / negative size / bad enum          */
#define BKV_ERR_UNSUPPORTED (-2) /* a shape or layout this library does not handle   */
#define BKV_ERR_ALIGN (-3)       /* pointer or stride not aligned as documented      */
#define BKV_ERR_CUDA (-4)        /* CUDA runtime reported an error at launch         */
#define BKV_ERR_LIMIT (-5)       /* size beyond a documented maximum                 */

/* element types */
#define BKV_F16 0
#define BKV_BF16 1
#define BKV_F32 2

/* code layouts of the page (quant/beyond_cute.py:56-58) */
#define BKV_LAYOUT_HEAD_WORD_TOKEN 1 /* ABI v1: word-major, token-minor */
#define BKV_LAYOUT_HND_TOKEN_WORD 2  /* ABI v2: token-major (production) */

/* flags */
#define BKV_FLAG_PDL_TRIGGER 0x1   /* encode: signal dependent launch early          */
#define BKV_FLAG_PDL_WAIT 0x2      /* decode: launched as a programmatic dependent of the
                                      immediately preceding kernel, which must be the cache
                                      writer: sequence lengths, block table and queries are
                                      read before the wait and must come from older launches.
                                      encode: likewise launched as a programmatic dependent of
                                      whatever kernel precedes it on the stream; only the
                                      threshold / level tables are read before the wait (rows,
                                      slots and cache after it), so the predecessor may be the
                                      producer of K and V or an earlier chunk of the same write */
#define BKV_FLAG_LINEAR_SEARCH 0x4 /* encode: count thresholds linearly (unsorted tables) */
#define BKV_FLAG_KLEVELS_LANE_MAJOR 0x8 /* decode: K levels given as (Hkv,16,4)      */
#define BKV_FLAG_BINNED_TABLES 0x10 /* encode: the caller has checked, for both threshold tensors,
                                      that every table is ascending, every threshold positive with
                                      the low four bits of its float32 pattern clear (any 16-bit
                                      value), and that every interval [e/512, (e+1)/512),
                                      e = 0..511, holds at most one threshold of a table (true
                                      when neighbouring thresholds are 2^-9 or more apart): large
                                      writes then replace the search by one indexed look-up.  A
                                      wrong claim gives wrong codes, never a bad access.       */

typedef void* bkv_stream_t; /* a cudaStream_t / CUstream */

int bkv_abi_version(void);
const char* bkv_status_string(int status);
const char* bkv_last_cuda_error(void);

/*
 * Encode-on-write.  Replaces write_tokens_to_paged_cache ->
 * _try_write_tokens_to_paged_cache_triton -> _write_packed_kv_cache_group_head128_kernel
 * (quant/beyond_cute.py:2147-2207, :1556-1700, :934-1164); bit-exact with the
 * reference quantiser quantize_k / quantize_v (:439-486, :525-584).
 *
 * k, v ........ [num_tokens][heads_kv][128] of in_dtype, innermost stride 1,
 *               token/head strides in elements; rows 16-byte aligned.
 * slots ....... int32 or int64 flat slot ids (page*block_size + offset); a
 *               negative slot writes nothing to the cache.
 * thr_*, lvl_*  15 thresholds / 16 levels of table_dtype, either one shared table
 *               (grouped_* = 0) or heads_kv*4 tables indexed head*4+group.
 * k_dq, v_dq .. optional (may be NULL, may alias k / v): reconstruction
 *               level*stored_scale + stored_min rounded to in_dtype
 *               (reference :1042-1079), written for every row, also slot < 0.
 */
int bkv_encode_sm100(const void* k, const void* v, int64_t k_stride_t, int64_t k_stride_h,
                     int64_t v_stride_t, int64_t v_stride_h, int in_dtype, const void* slots,
                     int slot_is_i64, int64_t slot_stride, int64_t num_tokens, int heads_kv,
                     void* cache, int64_t num_pages, int64_t page_stride_i32, int block_size,
                     int code_layout, int stat_dtype, const void* thr_k, const void* thr_v,
                     const void* lvl_k, const void* lvl_v, int table_dtype, int grouped_k,
                     int grouped_v, void* k_dq, void* v_dq, int64_t kdq_stride_t,
                     int64_t kdq_stride_h, int64_t vdq_stride_t, int64_t vdq_stride_h, int flags,
                     bkv_stream_t stream);

/*
 * Fused paged split-KV decode attention over the packed cache, general form: a
 * (split, kv head, request) grid on CUDA cores that takes any page size and any supported
 * head ratio.  Replaces run_nonuniform_decode -> MixedInputFusedMultiHeadAttentionDecode
 * (+ reducer) (quant/fa4_cute/beyond_mixed_decode_runtime.py:520-612,
 *  quant/fa4_cute/beyond_mixed_decode_sm100.py:930-3214) for an explicit split count.
 * The production path is bkv_decode_stream_sm100 below (tensor cores, no split count).
 *
 * q ............. [batch][heads_q][128] q_dtype, head stride 128, batch stride given.
 * block_table ... int32 [batch][>= ceil(max seq_len / block_size)], row stride given.
 * seq_lens ...... int32 [batch]; 0 gives a zero output row.
 * lvl_k, lvl_v .. heads_kv*4 tables of 16 levels (table_dtype); K may be given in
 *                 the launcher's (Hkv,16,4) order with BKV_FLAG_KLEVELS_LANE_MAJOR.
 * out ........... [batch][heads_q][128] out_dtype, contiguous.
 * out_f32 ....... optional float32 copy of the un-rounded result (may be NULL).
 * o/m/l_partial . float32 workspaces [num_splits][batch][heads_q]([128]); only read
 *                 and written when num_splits > 1.
 * softmax_scale . must be positive.
 * Split s of a request covers pages s, s+num_splits, ... of its block table row.
 */
int bkv_decode_sm100(const void* q, int64_t q_batch_stride, int q_dtype, const void* cache,
                     int64_t num_pages, int64_t page_stride_i32, int block_size, int heads_kv,
                     int stat_dtype, const int32_t* block_table, int64_t block_table_stride,
                     const int32_t* seq_lens, const void* lvl_k, const void* lvl_v,
                     int table_dtype, void* out, int out_dtype, float* out_f32, float* o_partial,
                     float* m_partial, float* l_partial, int num_splits, int batch, int heads_q,
                     int max_seq_len, float softmax_scale, int flags, bkv_stream_t stream);

/*
 * Test hook (no counterpart in the reference): the encoder divides by the group scale with
 * a reciprocal shared by the 8 scalars of a lane and an exact-remainder correction; this
 * entry point runs that division next to the IEEE division (__fdiv_rn) on `count`
 * pseudo-random operand pairs and ADDS the number of bitwise mismatches to *mismatches
 * (device memory, 64-bit, zeroed by the caller).  mode 0: the quantiser's domain
 * (divisor in [2^-20, 2^6), dividend in [0, divisor]); mode 1: any finite positive pair.
 * The expected count is 0 in both modes.
 */
int bkv_selftest_division_sm100(uint64_t seed, int64_t count, int mode, unsigned long long* mismatches,
                                bkv_stream_t stream);

/*
 * The production decode kernel: tensor cores, one persistent CTA per SM.
 *
 * Replaces the same reference launcher as bkv_decode_sm100
 * (quant/fa4_cute/beyond_mixed_decode_runtime.py:520-612 run_nonuniform_decode ->
 * compiled split kernel + reducer, quant/fa4_cute/beyond_mixed_decode_sm100.py:930-3214).
 * Instead of a (split, head, request) grid whose split count comes from a launch policy,
 * one CTA per SM takes an equal share of all (head, request, 16-token tile) work, so
 * requests of any length mix keep every SM busy.  A request that ends up cut between workers
 * leaves partials in `workspace`; the worker that finishes last merges them inside the same
 * kernel.  There is no split count and no second launch.
 *
 * workspace / workspace_bytes: device scratch of at least
 * bkv_decode_stream_workspace_bytes() bytes (the bound depends on the current device only).
 * Before its FIRST use it must be prepared with bkv_decode_stream_workspace_init (or be
 * zero-filled); the kernels leave it prepared, so one call per allocation is enough.  Two
 * calls that may overlap on the GPU need separate workspaces.  If
 * bkv_decode_device_status ever reports a non-zero status, prepare the workspace again.
 * byte_tables: NULL, or the buffer filled by bkv_decode_tables_sm100 for these lvl_k /
 * lvl_v (once per layer): the kernel then copies its look-up tables instead of building them.
 * lvl_k / lvl_v must be 16-bit tables here (BKV_F16 or BKV_BF16; bf16 levels of magnitude
 * 2^-14 .. 1 are exact in the kernel's fp16 tables); float32 tables return
 * BKV_ERR_UNSUPPORTED.
 * Returns BKV_ERR_UNSUPPORTED (launches nothing) for batch > 16384, more than 2^26 pages,
 * more than 2^20 (kv head, request) pairs or a page size that is not 16 * 2^k; use
 * bkv_decode_sm100 then.
 * loader: 0 = 16-byte asynchronous copies (default), 1 = tensor copies of whole tile parts.
 */
int64_t bkv_decode_stream_workspace_bytes(void);
int bkv_decode_stream_workspace_init(void* workspace, int64_t workspace_bytes, bkv_stream_t stream);
int bkv_decode_stream_sm100(const void* q, int64_t q_batch_stride, int q_dtype, const void* cache,
                            int64_t num_pages, int64_t page_stride_i32, int block_size,
                            int heads_kv, int stat_dtype, const int32_t* block_table,
                            int64_t block_table_stride, const int32_t* seq_lens,
                            const void* lvl_k, const void* lvl_v, int table_dtype, void* out,
                            int out_dtype, float* out_f32, void* workspace,
                            int64_t workspace_bytes, const void* byte_tables, int batch,
                            int heads_q, int max_seq_len, float softmax_scale, int flags,
                            int loader, bkv_stream_t stream);

/*
 * Decode-side table preparation, once per layer: expands the 16-level tables of every kv
 * head into the byte-indexed look-up tables of bkv_decode_stream_sm100 (128 KiB per kv head,
 * bkv_decode_tables_bytes(heads_kv) in all).  Takes the place of the per-launch table
 * staging of the reference kernel (prepare_runtime_qpoints,
 * quant/fa4_cute/beyond_mixed_decode_runtime.py:92-134, is likewise "once per layer").
 * lvl_k / lvl_v / table_dtype / flags as for the decode call.
 */
int64_t bkv_decode_tables_bytes(int heads_kv);
int bkv_decode_tables_sm100(const void* lvl_k, const void* lvl_v, int table_dtype, int heads_kv,
                            int flags, void* tables, int64_t tables_bytes, bkv_stream_t stream);

/*
 * Host-only check of the persistent kernel's work partition (no device access; no counterpart
 * in the reference): for `batch` requests of `tiles[b]` 16-token tiles each and
 * `virtual_heads` heads on `sm_count` SMs it walks every worker's run the way the kernel does
 * and compares where the parts of every cut request go with the list the merging worker
 * derives.  Returns the number of requests that disagree (expected 0), -1 for bad arguments.
 */
int bkv_selftest_partition(const int32_t* tiles, int batch, int virtual_heads, int sm_count,
                           int max_tiles_per_request);

/*
 * bkv_combine_sm100 over packed records: split s is the block of rows*130 floats at
 * records + s*rows*130 laid out as o (rows x 128) | m (rows) | l (rows) - the form in which
 * one rank's partials travel in a single all-gather (no counterpart in the reference).
 */
int bkv_combine_packed_sm100(const float* records, int num_splits, int64_t rows, void* out,
                             int out_dtype, float* out_f32, bkv_stream_t stream);

/*
 * bkv_decode_range_sm100 under the persistent schedule of bkv_decode_stream_sm100: the
 * un-normalised partials (o, m natural-log, l) of every (request, query head) over the
 * positions [token_lo, min(token_hi, seq_len)), with all SMs busy even for one request
 * (the range call above runs one CTA per request and head).  No counterpart in the
 * reference, which has no KV-range sharding.  workspace, byte_tables and loader as for
 * bkv_decode_stream_sm100; token_lo must be a multiple of block_size.
 */
int bkv_decode_range_stream_sm100(const void* q, int64_t q_batch_stride, int q_dtype,
                                  const void* cache, int64_t num_pages, int64_t page_stride_i32,
                                  int block_size, int heads_kv, int stat_dtype,
                                  const int32_t* block_table, int64_t block_table_stride,
                                  const int32_t* seq_lens, const void* lvl_k, const void* lvl_v,
                                  int table_dtype, float* o_partial, float* m_partial,
                                  float* l_partial, void* workspace, int64_t workspace_bytes,
                                  const void* byte_tables, int batch, int heads_q, int token_lo,
                                  int token_hi, float softmax_scale, int flags, int loader,
                                  bkv_stream_t stream);

/*
 * Exchange step of the KV-range split without a collective on the data path (no counterpart in
 * the reference, which has no multi-GPU decode).  Every rank owns a receive buffer of
 * bkv_kv_exchange_bytes(world, rows) bytes - [2][world] records of rows*130 floats followed by
 * [2][world] flag words - that all other ranks of the node map through CUDA IPC:
 *   bkv_kv_exchange_alloc  allocates and zero-fills the buffer (set-up time: this is the one
 *                          entry point of the library that allocates) and returns its 64-byte
 *                          IPC handle, which the caller hands to the other ranks by any means;
 *   bkv_kv_exchange_open / _close  map / unmap a peer's buffer from its handle;
 *   bkv_kv_exchange_free   releases the own buffer (after every peer has closed it).
 * bkv_kv_exchange_merge_sm100 is the per-step call, one kernel: it stores this rank's record
 * (o | m | l as written by bkv_decode_range_stream_sm100 into one contiguous block) into slot
 * `rank` of every peer's buffer with plain peer stores, publishes `step` in the peer's flag word,
 * waits until the `world` flags of its own buffer show `step`, and merges the records by
 * log-sum-exp into `out` ([rows][128]).  peer_buffers: host array of `world` device addresses,
 * entry `rank` being the own buffer.  step: 1, 2, 3, ... the same sequence on every rank, or 0
 * on every call: the kernel then numbers the steps itself with a counter kept in the rank's own
 * buffer, which makes the launch identical from step to step (a captured CUDA graph can replay
 * it); use one of the two forms for the lifetime of a buffer.
 * The wait is bounded: after timeout_ns nanoseconds without the flags the kernel sets *status
 * (device int, never cleared by the library) to 1, leaves `out` untouched and returns; nothing
 * hangs when a peer is gone.  world <= 16.
 */
int64_t bkv_kv_exchange_bytes(int world, int64_t rows);
int bkv_kv_exchange_alloc(int64_t bytes, void** buffer_out, unsigned char* handle64_out);
int bkv_kv_exchange_open(const unsigned char* handle64, void** peer_out);
int bkv_kv_exchange_close(void* peer);
int bkv_kv_exchange_free(void* buffer);
int bkv_kv_exchange_merge_sm100(const float* record, int64_t rows, const uint64_t* peer_buffers, int world,
                                int rank, int step, int64_t timeout_ns, void* out, int out_dtype,
                                float* out_f32, int* status, bkv_stream_t stream);

/*
 * bkv_decode_sm100 for callers that cannot allocate device memory (no counterpart in
 * the reference, whose launcher always receives a caller-allocated workspace).
 *
 * Some callers have no way to provide the split workspace: code that already runs inside
 * a stream capture, a plugin that must not touch its host's allocator, an embedder with a
 * fixed arena.  Here the partials go to a fixed array inside the library image, so the
 * call performs no cudaMalloc / cudaFree and calls no allocating library routine.
 *
 * Limits and rules:
 *  - num_splits * batch * heads_q must not exceed BKV_NOALLOC_MAX_SPLIT_ROWS; larger
 *    launches are refused with BKV_ERR_LIMIT.  The array costs
 *    BKV_NOALLOC_MAX_SPLIT_ROWS * 520 bytes (about 4.1 MiB) of device memory on every GPU
 *    that loads the library, until the process exits.
 *  - The first call on a device looks up the array's device address (once per device, with
 *    that device current).  Make that first call before starting any stream capture.
 *  - All calls on one GPU share the array, which keeps the previous call's contents.  Each
 *    call rewrites every slot it later reads, so nothing needs clearing; but two calls
 *    whose kernels may overlap on the GPU (different streams) race on it - serialise them.
 * Arguments and results are those of bkv_decode_sm100 without the three workspace pointers.
 */
#define BKV_NOALLOC_MAX_SPLIT_ROWS 8192
int bkv_decode_noalloc_sm100(const void* q, int64_t q_batch_stride, int q_dtype, const void* cache,
                             int64_t num_pages, int64_t page_stride_i32, int block_size,
                             int heads_kv, int stat_dtype, const int32_t* block_table,
                             int64_t block_table_stride, const int32_t* seq_lens,
                             const void* lvl_k, const void* lvl_v, int table_dtype, void* out,
                             int out_dtype, float* out_f32, int num_splits, int batch, int heads_q,
                             int max_seq_len, float softmax_scale, int flags, bkv_stream_t stream);

/*
 * Diagnostic: reads and clears the device-side status word of the decode kernels
 * (0 = fine; 2 = a bounded wait inside the tensor-core kernel gave up after 2 s instead of
 * spinning forever; 3 = the kernel found an unexpected shared-memory layout and did nothing).  Synchronises the device.  No counterpart in the
 * reference.
 */
int bkv_decode_device_status(int* status_out);

/*
 * Log-sum-exp merge of split partials.  Replaces reduction_parallel_weights /
 * reduction_cta4_weights / reduction_warp_parallel_weights
 * (quant/fa4_cute/beyond_mixed_decode_sm100.py:2935-3214).  m_partial is in the
 * natural-log domain of the scaled scores.  rows = batch*heads_q.
 */
int bkv_combine_sm100(const float* o_partial, const float* m_partial, const float* l_partial,
                      int num_splits, int64_t rows, void* out, int out_dtype, float* out_f32,
                      bkv_stream_t stream);

/*
 * Partial (un-normalised) decode over pages [page_lo, page_hi) of every request:
 * writes o/m/l for ONE split slot; used for the KV-range split across GPUs, whose
 * partials are exchanged and merged with bkv_combine_sm100.  No counterpart in the
 * reference (it has no multi-GPU decode); the arithmetic is that of bkv_decode_sm100.
 */
int bkv_decode_range_sm100(const void* q, int64_t q_batch_stride, int q_dtype, const void* cache,
                           int64_t num_pages, int64_t page_stride_i32, int block_size,
                           int heads_kv, int stat_dtype, const int32_t* block_table,
                           int64_t block_table_stride, const int32_t* seq_lens, const void* lvl_k,
                           const void* lvl_v, int table_dtype, float* o_partial, float* m_partial,
                           float* l_partial, int batch, int heads_q, int token_lo, int token_hi,
                           float softmax_scale, int flags, bkv_stream_t stream);

/*
 * Paged read-back to dense varlen K/V.  Replaces dequantize_paged_kv_to_dense and
 * its two Triton kernels (quant/beyond_cute.py:1703-1856, :1166-1476); bit-exact
 * with read_request_from_paged_cache (:2210-2395).
 * out_k/out_v: [total_tokens][heads_kv][128] out_dtype, contiguous; request r
 * writes rows seq_start[r] .. seq_start[r]+seq_lens[r]-1.
 */
int bkv_readback_sm100(const void* cache, int64_t num_pages, int64_t page_stride_i32,
                       int block_size, int heads_kv, int stat_dtype, const int32_t* block_table,
                       int64_t block_table_stride, int64_t block_table_width,
                       const int32_t* seq_lens, const int32_t* seq_start, int batch,
                       int max_seq_len, const void* lvl_k, const void* lvl_v, int table_dtype,
                       int grouped_k, int grouped_v, void* out_k, void* out_v, int out_dtype,
                       bkv_stream_t stream);

/*
 * bf16/fp16-KV paged decode attention of the same shape and split policy: the
 * full-precision baseline the packed kernel is measured against.  K and V pages:
 * [num_pages][block_size][heads_kv][128] kv_dtype.  No counterpart in the
 * reference repository (it compares against FlashAttention-4).
 */
int bkv_decode_dense_sm100(const void* q, int64_t q_batch_stride, int q_dtype, const void* k_pages,
                           const void* v_pages, int kv_dtype, int64_t num_pages, int block_size,
                           int heads_kv, const int32_t* block_table, int64_t block_table_stride,
                           const int32_t* seq_lens, void* out, int out_dtype, float* o_partial,
                           float* m_partial, float* l_partial, int num_splits, int batch,
                           int heads_q, int max_seq_len, float softmax_scale,
                           bkv_stream_t stream);

/*
 * Last-token slot derivation for graph-safe decode:
 * slot[b] = block_table[b][(len-1)/BS]*BS + (len-1)%BS, or -1 when len <= 0 or the
 * page id is negative.  Replaces _derive_dense_decode_slot_mapping_kernel
 * (src/beyond/runtime/vllm/packed_backend.py:2251-2283).
 */
int bkv_derive_slots_sm100(const int32_t* seq_lens, const int32_t* block_table,
                           int64_t block_table_stride, int64_t block_table_width, int block_size,
                           int batch, int32_t* slots_out, bkv_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* BKV_SM100_H_ */
