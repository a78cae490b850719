// C ABI glue: status strings, launch-error capture and the decode entry points.
#include <math_constants.h>

#include <climits>
#include <cstdio>

#include "bkv_decode_common.cuh"

namespace bkv {

static thread_local char g_last_error[256] = "";

void set_last_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", where, cudaGetErrorString(e),
           cudaGetErrorName(e));
}

int check_launch(const char* where) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return BKV_OK;
  set_last_cuda_error(e, where);
  return BKV_ERR_CUDA;
}

static int fill_decode_params(DecodeParams& p, const void* q, int64_t q_batch_stride, int q_dtype,
                              const void* cache, int64_t num_pages, int64_t page_stride_i32,
                              int block_size, int heads_kv, int stat_dtype,
                              const int32_t* block_table, int64_t block_table_stride,
                              const int32_t* seq_lens, const void* lvl_k, const void* lvl_v,
                              int table_dtype, int batch, int heads_q, float softmax_scale,
                              int flags) {
  if (batch < 0 || heads_q <= 0 || heads_kv <= 0 || block_size <= 0 || num_pages < 0)
    return BKV_ERR_ARG;
  if (!q || !cache || !block_table || !seq_lens || !lvl_k || !lvl_v) return BKV_ERR_ARG;
  if (q_dtype != BKV_F16 && q_dtype != BKV_BF16 && q_dtype != BKV_F32) return BKV_ERR_ARG;
  if (stat_dtype != BKV_F16 && stat_dtype != BKV_BF16) return BKV_ERR_ARG;
  if (table_dtype != BKV_F16 && table_dtype != BKV_BF16 && table_dtype != BKV_F32)
    return BKV_ERR_ARG;
  if (heads_q % heads_kv) return BKV_ERR_ARG;
  const int gqa = heads_q / heads_kv;
  if (gqa != 1 && gqa != 2 && gqa != 4 && gqa != 8) return BKV_ERR_UNSUPPORTED;
  if (page_stride_i32 < make_geom(block_size, heads_kv).block_i32) return BKV_ERR_ARG;
  if (q_batch_stride < static_cast<int64_t>(heads_q) * kHeadDim) return BKV_ERR_ARG;
  if (!(softmax_scale > 0.f)) return BKV_ERR_ARG;  // the kernels take the maximum before scaling
  p.q = q; p.q_batch_stride = q_batch_stride; p.q_dtype = q_dtype;
  p.cache = static_cast<const uint32_t*>(cache);
  p.num_pages = num_pages; p.page_stride = page_stride_i32; p.block_size = block_size;
  p.heads_kv = heads_kv; p.heads_q = heads_q; p.batch = batch;
  p.stat_bf16 = stat_dtype == BKV_BF16;
  p.block_table = block_table; p.bt_stride = block_table_stride; p.seq_lens = seq_lens;
  p.lvl_k = lvl_k; p.lvl_v = lvl_v; p.table_dtype = table_dtype;
  p.klevels_lane_major = (flags & BKV_FLAG_KLEVELS_LANE_MAJOR) != 0;
  p.out = nullptr; p.out_dtype = BKV_F32; p.out_f32 = nullptr;
  p.o_partial = nullptr; p.m_partial = nullptr; p.l_partial = nullptr;
  p.num_splits = 1; p.token_lo = 0; p.token_hi = INT_MAX; p.force_partial = 0;
  p.scale_log2 = softmax_scale * kLog2e;
  p.flags = flags;
  return BKV_OK;
}

}  // namespace bkv

extern "C" int bkv_abi_version(void) { return BKV_ABI_VERSION; }

extern "C" const char* bkv_status_string(int status) {
  switch (status) {
    case BKV_OK: return "ok";
    case BKV_ERR_ARG: return "invalid argument (null pointer, negative size or unknown enum)";
    case BKV_ERR_UNSUPPORTED: return "shape or layout not supported by the sm_100a kernels";
    case BKV_ERR_ALIGN: return "pointer or stride is not 16-byte aligned";
    case BKV_ERR_CUDA: return "CUDA runtime error at launch (see bkv_last_cuda_error)";
    case BKV_ERR_LIMIT: return "size exceeds a documented maximum";
    default: return "unknown status";
  }
}

extern "C" const char* bkv_last_cuda_error(void) { return bkv::g_last_error; }

extern "C" int bkv_decode_sm100(const void* q, int64_t q_batch_stride, int q_dtype,
                                const void* cache, int64_t num_pages, int64_t page_stride_i32,
                                int block_size, int heads_kv, int stat_dtype,
                                const int32_t* block_table, int64_t block_table_stride,
                                const int32_t* seq_lens, const void* lvl_k, const void* lvl_v,
                                int table_dtype, void* out, int out_dtype, float* out_f32,
                                float* o_partial, float* m_partial, float* l_partial,
                                int num_splits, int batch, int heads_q, int max_seq_len,
                                float softmax_scale, int flags, bkv_stream_t stream) {
  using namespace bkv;
  DecodeParams p;
  const int rc = fill_decode_params(p, q, q_batch_stride, q_dtype, cache, num_pages,
                                    page_stride_i32, block_size, heads_kv, stat_dtype, block_table,
                                    block_table_stride, seq_lens, lvl_k, lvl_v, table_dtype, batch,
                                    heads_q, softmax_scale, flags);
  if (rc != BKV_OK) return rc;
  if (batch == 0) return BKV_OK;
  if (!out) return BKV_ERR_ARG;
  if (out_dtype != BKV_F16 && out_dtype != BKV_BF16 && out_dtype != BKV_F32) return BKV_ERR_ARG;
  if (num_splits < 1 || num_splits > 64) return BKV_ERR_ARG;
  if (num_splits > 1 && (!o_partial || !m_partial || !l_partial)) return BKV_ERR_ARG;
  if (max_seq_len <= 0) return BKV_ERR_ARG;
  p.out = out; p.out_dtype = out_dtype; p.out_f32 = out_f32;
  p.o_partial = o_partial; p.m_partial = m_partial; p.l_partial = l_partial;
  p.num_splits = num_splits;
  p.token_hi = max_seq_len;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int launched = launch_decode_scalar(p, s);
  if (launched != BKV_OK) return launched;
  if (num_splits > 1)
    return launch_combine(o_partial, m_partial, l_partial, num_splits,
                          static_cast<int64_t>(batch) * heads_q, out, out_dtype, out_f32, s);
  return BKV_OK;
}

extern "C" int64_t bkv_decode_stream_workspace_bytes(void) { return bkv::stream_workspace_bytes(); }

extern "C" int bkv_decode_stream_workspace_init(void* workspace, int64_t workspace_bytes, bkv_stream_t stream) {
  return bkv::init_stream_workspace(workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int64_t bkv_decode_tables_bytes(int heads_kv) { return heads_kv > 0 ? bkv::byte_table_bytes(heads_kv) : 0; }

extern "C" int bkv_decode_tables_sm100(const void* lvl_k, const void* lvl_v, int table_dtype, int heads_kv,
                                       int flags, void* tables, int64_t tables_bytes, bkv_stream_t stream) {
  using namespace bkv;
  if (!lvl_k || !lvl_v || !tables || heads_kv <= 0) return BKV_ERR_ARG;
  if (table_dtype != BKV_F16 && table_dtype != BKV_BF16) return BKV_ERR_UNSUPPORTED;
  if (tables_bytes < byte_table_bytes(heads_kv)) return BKV_ERR_ARG;
  DecodeParams p = {};
  p.lvl_k = lvl_k; p.lvl_v = lvl_v; p.table_dtype = table_dtype; p.heads_kv = heads_kv;
  p.klevels_lane_major = (flags & BKV_FLAG_KLEVELS_LANE_MAJOR) != 0;
  return launch_build_byte_tables(p, tables, static_cast<cudaStream_t>(stream));
}

extern "C" int bkv_selftest_partition(const int32_t* tiles, int batch, int virtual_heads, int sm_count,
                                      int max_tiles_per_request) {
  return bkv::check_partition(tiles, batch, virtual_heads, sm_count, max_tiles_per_request);
}

extern "C" int bkv_decode_stream_sm100(const void* q, int64_t q_batch_stride, int q_dtype,
                                       const void* cache, int64_t num_pages,
                                       int64_t page_stride_i32, int block_size, int heads_kv,
                                       int stat_dtype, const int32_t* block_table,
                                       int64_t block_table_stride, const int32_t* seq_lens,
                                       const void* lvl_k, const void* lvl_v, int table_dtype,
                                       void* out, int out_dtype, float* out_f32, void* workspace,
                                       int64_t workspace_bytes, const void* byte_tables, int batch,
                                       int heads_q, int max_seq_len, float softmax_scale, int flags,
                                       int loader, bkv_stream_t stream) {
  using namespace bkv;
  DecodeParams p;
  const int rc = fill_decode_params(p, q, q_batch_stride, q_dtype, cache, num_pages,
                                    page_stride_i32, block_size, heads_kv, stat_dtype, block_table,
                                    block_table_stride, seq_lens, lvl_k, lvl_v, table_dtype, batch,
                                    heads_q, softmax_scale, flags);
  if (rc != BKV_OK) return rc;
  if (batch == 0) return BKV_OK;
  if (!out || !workspace) return BKV_ERR_ARG;
  if (out_dtype != BKV_F16 && out_dtype != BKV_BF16 && out_dtype != BKV_F32) return BKV_ERR_ARG;
  if (max_seq_len <= 0) return BKV_ERR_ARG;
  p.out = out; p.out_dtype = out_dtype; p.out_f32 = out_f32;
  p.num_splits = 1;
  p.token_hi = max_seq_len;
  if (loader != 0 && loader != 1) return BKV_ERR_ARG;
  return launch_decode_stream(p, workspace, workspace_bytes, byte_tables, max_seq_len,
                              static_cast<cudaStream_t>(stream), loader);
}

extern "C" int bkv_decode_device_status(int* status_out) {
  if (!status_out) return BKV_ERR_ARG;
  *status_out = bkv::read_stream_status();
  return bkv::check_launch("bkv_decode_device_status");
}

extern "C" int bkv_combine_sm100(const float* o_partial, const float* m_partial,
                                 const float* l_partial, int num_splits, int64_t rows, void* out,
                                 int out_dtype, float* out_f32, bkv_stream_t stream) {
  using namespace bkv;
  if (num_splits < 1 || rows < 0) return BKV_ERR_ARG;
  if (rows == 0) return BKV_OK;
  if (!o_partial || !m_partial || !l_partial || !out) return BKV_ERR_ARG;
  if (out_dtype != BKV_F16 && out_dtype != BKV_BF16 && out_dtype != BKV_F32) return BKV_ERR_ARG;
  return launch_combine(o_partial, m_partial, l_partial, num_splits, rows, out, out_dtype, out_f32,
                        static_cast<cudaStream_t>(stream));
}

extern "C" int bkv_combine_packed_sm100(const float* records, int num_splits, int64_t rows, void* out,
                                        int out_dtype, float* out_f32, bkv_stream_t stream) {
  using namespace bkv;
  if (num_splits < 1 || rows < 0) return BKV_ERR_ARG;
  if (rows == 0) return BKV_OK;
  if (!records || !out) return BKV_ERR_ARG;
  if (out_dtype != BKV_F16 && out_dtype != BKV_BF16 && out_dtype != BKV_F32) return BKV_ERR_ARG;
  return launch_combine_packed(records, num_splits, rows, out, out_dtype, out_f32,
                               static_cast<cudaStream_t>(stream));
}

extern "C" int bkv_decode_range_stream_sm100(const void* q, int64_t q_batch_stride, int q_dtype,
                                             const void* cache, int64_t num_pages,
                                             int64_t page_stride_i32, int block_size, int heads_kv,
                                             int stat_dtype, const int32_t* block_table,
                                             int64_t block_table_stride, const int32_t* seq_lens,
                                             const void* lvl_k, const void* lvl_v, int table_dtype,
                                             float* o_partial, float* m_partial, float* l_partial,
                                             void* workspace, int64_t workspace_bytes,
                                             const void* byte_tables, int batch, int heads_q,
                                             int token_lo, int token_hi, float softmax_scale,
                                             int flags, int loader, bkv_stream_t stream) {
  using namespace bkv;
  DecodeParams p;
  const int rc = fill_decode_params(p, q, q_batch_stride, q_dtype, cache, num_pages,
                                    page_stride_i32, block_size, heads_kv, stat_dtype, block_table,
                                    block_table_stride, seq_lens, lvl_k, lvl_v, table_dtype, batch,
                                    heads_q, softmax_scale, flags);
  if (rc != BKV_OK) return rc;
  if (batch == 0) return BKV_OK;
  if (!o_partial || !m_partial || !l_partial || !workspace) return BKV_ERR_ARG;
  if (token_lo < 0 || token_hi < token_lo) return BKV_ERR_ARG;
  if (token_lo % block_size) return BKV_ERR_ARG;  // ranges start on a page boundary
  p.o_partial = o_partial; p.m_partial = m_partial; p.l_partial = l_partial;
  p.num_splits = 1; p.force_partial = 1;
  p.token_lo = token_lo; p.token_hi = token_hi;
  if (loader != 0 && loader != 1) return BKV_ERR_ARG;
  return launch_decode_stream(p, workspace, workspace_bytes, byte_tables, token_hi - token_lo,
                              static_cast<cudaStream_t>(stream), loader);
}

extern "C" int bkv_decode_range_sm100(const void* q, int64_t q_batch_stride, int q_dtype,
                                      const void* cache, int64_t num_pages,
                                      int64_t page_stride_i32, int block_size, int heads_kv,
                                      int stat_dtype, const int32_t* block_table,
                                      int64_t block_table_stride, const int32_t* seq_lens,
                                      const void* lvl_k, const void* lvl_v, int table_dtype,
                                      float* o_partial, float* m_partial, float* l_partial,
                                      int batch, int heads_q, int token_lo, int token_hi,
                                      float softmax_scale, int flags, bkv_stream_t stream) {
  using namespace bkv;
  DecodeParams p;
  const int rc = fill_decode_params(p, q, q_batch_stride, q_dtype, cache, num_pages,
                                    page_stride_i32, block_size, heads_kv, stat_dtype, block_table,
                                    block_table_stride, seq_lens, lvl_k, lvl_v, table_dtype, batch,
                                    heads_q, softmax_scale, flags);
  if (rc != BKV_OK) return rc;
  if (batch == 0) return BKV_OK;
  if (!o_partial || !m_partial || !l_partial) return BKV_ERR_ARG;
  if (token_lo < 0 || token_hi < token_lo) return BKV_ERR_ARG;
  if (token_lo % block_size) return BKV_ERR_ARG;  // ranges start on a page boundary
  p.o_partial = o_partial; p.m_partial = m_partial; p.l_partial = l_partial;
  p.num_splits = 1; p.force_partial = 1;
  p.token_lo = token_lo; p.token_hi = token_hi;
  return launch_decode_scalar(p, static_cast<cudaStream_t>(stream));
}
