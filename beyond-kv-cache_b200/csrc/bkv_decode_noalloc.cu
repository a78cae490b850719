// Packed decode attention for callers that cannot allocate device memory.
//
// The split-KV decode needs scratch for the per-split partial outputs.  Callers such as
// code running inside a CUDA-graph capture region, plugins that are handed tensors by a
// host framework whose allocator they may not touch, or embedders that run with a fixed
// memory arena normally pre-allocate that workspace; this entry point serves the ones
// that have no way to do so.  The scratch lives in a fixed-size array inside the library
// image, so the call allocates nothing: no cudaMalloc / cudaFree and no allocating library
// routine.  The price is a hard size limit and one shared buffer per GPU.
#include <mutex>

#include "bkv_common.cuh"

namespace {

// partial outputs [split*row][128] followed by the running maxima and sums [split*row] each
constexpr int64_t kMaxSplitRows = BKV_NOALLOC_MAX_SPLIT_ROWS;
constexpr int64_t kScratchFloats = kMaxSplitRows * (bkv::kHeadDim + 2);
static __device__ __align__(256) float g_split_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
float* g_scratch_addr[kMaxDevices] = {};  // device address of g_split_scratch, per device

// In host code `g_split_scratch` is only a handle for the device symbol, not a pointer a
// kernel can use; the real address is asked for once per device, with that device current.
int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    bkv::set_last_cuda_error(e, "bkv_decode_noalloc_sm100: cudaGetDevice");
    return BKV_ERR_CUDA;
  }
  if (dev < 0 || dev >= kMaxDevices) return BKV_ERR_LIMIT;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* addr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&addr), g_split_scratch);
    if (e != cudaSuccess || addr == nullptr) {
      bkv::set_last_cuda_error(e, "bkv_decode_noalloc_sm100: cudaGetSymbolAddress");
      return BKV_ERR_CUDA;
    }
    g_scratch_addr[dev] = addr;
  }
  *out = g_scratch_addr[dev];
  return BKV_OK;
}

}  // namespace

extern "C" int bkv_decode_noalloc_sm100(const void* q, int64_t q_batch_stride, int q_dtype,
                                        const void* cache, int64_t num_pages,
                                        int64_t page_stride_i32, int block_size, int heads_kv,
                                        int stat_dtype, const int32_t* block_table,
                                        int64_t block_table_stride, const int32_t* seq_lens,
                                        const void* lvl_k, const void* lvl_v, int table_dtype,
                                        void* out, int out_dtype, float* out_f32, int num_splits,
                                        int batch, int heads_q, int max_seq_len,
                                        float softmax_scale, int flags, bkv_stream_t stream) {
  if (num_splits < 1 || batch < 0 || heads_q <= 0) return BKV_ERR_ARG;
  const int64_t split_rows = static_cast<int64_t>(num_splits) * batch * heads_q;
  if (split_rows > kMaxSplitRows) return BKV_ERR_LIMIT;  // scratch is a fixed-size array
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != BKV_OK) return rc;
  // Every (split, row) slot the merge reads is rewritten by the decode kernel of the same
  // call (empty splits write a zero weight), so nothing has to be cleared between calls.
  float* o_partial = scratch;
  float* m_partial = scratch + split_rows * bkv::kHeadDim;
  float* l_partial = m_partial + split_rows;
  return bkv_decode_sm100(q, q_batch_stride, q_dtype, cache, num_pages, page_stride_i32, block_size,
                          heads_kv, stat_dtype, block_table, block_table_stride, seq_lens, lvl_k,
                          lvl_v, table_dtype, out, out_dtype, out_f32, o_partial, m_partial,
                          l_partial, num_splits, batch, heads_q, max_seq_len, softmax_scale, flags,
                          stream);
}
