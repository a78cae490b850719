// Parameters shared by the packed decode kernels and the combine kernel.
#pragma once

#include "bkv_common.cuh"

namespace bkv {

struct DecodeParams {
  const void* q;
  int64_t q_batch_stride;
  int q_dtype;
  const uint32_t* cache;
  int64_t num_pages;
  int64_t page_stride;
  int block_size;
  int heads_kv;
  int heads_q;
  int batch;
  int stat_bf16;
  const int32_t* block_table;
  int64_t bt_stride;
  const int32_t* seq_lens;
  const void* lvl_k;
  const void* lvl_v;
  int table_dtype;
  int klevels_lane_major;  // K levels stored (Hkv,16,4) instead of (Hkv*4,16)
  void* out;
  int out_dtype;
  float* out_f32;
  float* o_partial;  // [splits][batch][heads_q][128]
  float* m_partial;  // [splits][batch][heads_q]   natural-log domain
  float* l_partial;  // [splits][batch][heads_q]
  int num_splits;
  int token_lo;      // attend positions token_lo <= t < min(token_hi, seq_len)
  int token_hi;
  int force_partial; // write partials even when num_splits == 1
  float scale_log2;  // softmax_scale * log2(e)
  int flags;
};

constexpr float kLn2 = 0.6931471805599453f;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float load_q(const void* q, int64_t idx, int dtype) {
  if (dtype == BKV_F32) return static_cast<const float*>(q)[idx];
  const uint32_t bits = static_cast<const unsigned short*>(q)[idx];
  return dtype == BKV_BF16 ? bf16_bits_to_f32(bits) : f16_bits_to_f32(bits);
}

__device__ __forceinline__ void store_out(void* out, int64_t idx, int dtype, float v) {
  if (dtype == BKV_F32) static_cast<float*>(out)[idx] = v;
  else if (dtype == BKV_BF16) static_cast<unsigned short*>(out)[idx] = static_cast<unsigned short>(f32_to_bf16_bits(v));
  else static_cast<unsigned short*>(out)[idx] = static_cast<unsigned short>(f32_to_f16_bits(v));
}

// K level of table (head, group), entry code, honouring the optional (Hkv,16,4) order
// produced by prepare_runtime_qpoints (quant/fa4_cute/beyond_mixed_decode_runtime.py:126-130).
__device__ __forceinline__ float load_k_level(const DecodeParams& p, int head, int group, int code) {
  const int idx = p.klevels_lane_major ? (head * 16 + code) * kGroupsPerHead + group
                                       : (head * kGroupsPerHead + group) * 16 + code;
  return load_table_f32(p.lvl_k, idx, p.table_dtype);
}
__device__ __forceinline__ float load_v_level(const DecodeParams& p, int head, int group, int code) {
  return load_table_f32(p.lvl_v, (head * kGroupsPerHead + group) * 16 + code, p.table_dtype);
}

int launch_decode_scalar(const DecodeParams& p, cudaStream_t stream);
int launch_combine_packed(const float* records, int num_splits, int64_t rows, void* out, int out_dtype,
                          float* out_f32, cudaStream_t stream);
int launch_decode_stream(const DecodeParams& p, void* workspace, int64_t workspace_bytes, const void* byte_tables,
                         int max_seq_len, cudaStream_t stream, int config);
int64_t stream_workspace_bytes();
int init_stream_workspace(void* workspace, int64_t workspace_bytes, cudaStream_t stream);
int64_t byte_table_bytes(int heads_kv);
int launch_build_byte_tables(const DecodeParams& p, void* out, cudaStream_t stream);
int check_partition(const int* tiles, int batch, int hv, int sm_count, int max_tiles_per_request);
int read_stream_status();
int launch_combine(const float* o_partial, const float* m_partial, const float* l_partial,
                   int num_splits, int64_t rows, void* out, int out_dtype, float* out_f32,
                   cudaStream_t stream);

}  // namespace bkv
