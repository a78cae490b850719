// Paged read-back of the packed cache to dense varlen K/V, and the last-token
// slot derivation used by graph-safe decode (sm_100a).
//
// Read-back mirrors the encode mapping: one warp per (request position, kv-head);
// lanes 0-15 expand the 16 K code words (8 scalars each), lanes 16-31 the V words.
// Reconstruction is level * stored_scale + stored_min as two separately rounded
// float32 operations followed by one rounding to the output type, which is what
// read_request_from_paged_cache of the reference evaluates
// (quant/beyond_cute.py:2322-2326, :2390-2393), so the result is bit-identical.
#include "bkv_common.cuh"

namespace bkv {

namespace {

struct ReadbackParams {
  const uint32_t* cache;
  int64_t num_pages, page_stride;
  int block_size, heads, stat_bf16;
  const int32_t* block_table;
  int64_t bt_stride, bt_width;
  const int32_t* seq_lens;
  const int32_t* seq_start;
  int batch, max_seq_len;
  const void* lvl_k;
  const void* lvl_v;
  int table_dtype, grouped_k, grouped_v;
  void* out_k;
  void* out_v;
  int out_dtype;
};

__global__ void __launch_bounds__(256) readback_kernel(const ReadbackParams p) {
  extern __shared__ float s_lvl[];  // [K tables | V tables], heads*4 tables of 16
  const int tables = p.heads * kGroupsPerHead;
  for (int i = threadIdx.x; i < tables * 16; i += blockDim.x) {
    const int t = i >> 4, j = i & 15;
    s_lvl[i] = load_table_f32(p.lvl_k, (p.grouped_k ? t * 16 : 0) + j, p.table_dtype);
    s_lvl[tables * 16 + i] = load_table_f32(p.lvl_v, (p.grouped_v ? t * 16 : 0) + j, p.table_dtype);
  }
  __syncthreads();

  const int lane = threadIdx.x & 31, is_v = lane >> 4, sub = lane & 15, grp = sub >> 2;
  const int warps_per_block = blockDim.x >> 5;
  const int BS = p.block_size;
  const PageGeom g = make_geom(BS, p.heads);
  const bool bf16 = p.stat_bf16 != 0;
  const int64_t per_req = static_cast<int64_t>(p.max_seq_len) * p.heads;
  const int64_t items = per_req * p.batch;
  for (int64_t item = static_cast<int64_t>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
       item < items; item += static_cast<int64_t>(gridDim.x) * warps_per_block) {
    const int b = static_cast<int>(item / per_req);
    const int64_t rem = item - b * per_req;
    const int pos = static_cast<int>(rem / p.heads);
    const int head = static_cast<int>(rem - static_cast<int64_t>(pos) * p.heads);
    if (pos >= p.seq_lens[b]) continue;
    const int lp = pos / BS, tok = pos - lp * BS;
    if (lp >= p.bt_width) continue;
    const int64_t phys = p.block_table[b * p.bt_stride + lp];
    if (phys < 0 || phys >= p.num_pages) continue;
    const uint32_t* pg = p.cache + phys * p.page_stride;
    const uint32_t word = pg[(is_v ? g.v_code_off : g.k_code_off) + head * (BS * kWordsPerHead) +
                             tok * kWordsPerHead + sub];
    const uint32_t st = is_v ? pg[g.v_stat_off + head * (4 * BS) + grp * BS + tok]
                             : pg[g.k_stat_off + head * (BS * 4) + tok * 4 + grp];
    const float sc = stat_bits_to_f32(st, bf16), mn = stat_bits_to_f32(st >> 16, bf16);
    const float* lvl = s_lvl + (is_v ? tables * 16 : 0) + (head * kGroupsPerHead + grp) * 16;
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = __fadd_rn(__fmul_rn(lvl[(word >> (4 * i)) & 15], sc), mn);
    const int64_t o = (static_cast<int64_t>(p.seq_start[b]) + pos) * p.heads * kHeadDim +
                      head * kHeadDim + sub * 8;
    void* dst = is_v ? p.out_v : p.out_k;
    if (p.out_dtype == BKV_F32) {
      float4* d4 = reinterpret_cast<float4*>(static_cast<float*>(dst) + o);
      d4[0] = make_float4(y[0], y[1], y[2], y[3]);
      d4[1] = make_float4(y[4], y[5], y[6], y[7]);
    } else {
      uint4 raw;
      uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        w[i] = p.out_dtype == BKV_BF16
                   ? (f32_to_bf16_bits(y[2 * i]) | (f32_to_bf16_bits(y[2 * i + 1]) << 16))
                   : (f32_to_f16_bits(y[2 * i]) | (f32_to_f16_bits(y[2 * i + 1]) << 16));
      *reinterpret_cast<uint4*>(static_cast<unsigned short*>(dst) + o) = raw;
    }
  }
}

__global__ void derive_slots_kernel(const int32_t* seq_lens, const int32_t* block_table,
                                    int64_t bt_stride, int64_t bt_width, int block_size, int batch,
                                    int32_t* slots) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const int len = seq_lens[b];
  int32_t slot = -1;
  if (len > 0) {
    const int last = len - 1;
    const int lp = last / block_size;
    if (lp < bt_width) {
      const int32_t phys = block_table[b * bt_stride + lp];
      if (phys >= 0) slot = phys * block_size + (last - lp * block_size);
    }
  }
  slots[b] = slot;
}

}  // namespace
}  // namespace bkv

extern "C" int bkv_readback_sm100(const void* cache, int64_t num_pages, int64_t page_stride_i32,
                                  int block_size, int heads_kv, int stat_dtype,
                                  const int32_t* block_table, int64_t block_table_stride,
                                  int64_t block_table_width, const int32_t* seq_lens,
                                  const int32_t* seq_start, int batch, int max_seq_len,
                                  const void* lvl_k, const void* lvl_v, int table_dtype,
                                  int grouped_k, int grouped_v, void* out_k, void* out_v,
                                  int out_dtype, bkv_stream_t stream) {
  using namespace bkv;
  if (batch < 0 || max_seq_len < 0 || heads_kv <= 0 || block_size <= 0) return BKV_ERR_ARG;
  if (batch == 0 || max_seq_len == 0) return BKV_OK;
  if (!cache || !block_table || !seq_lens || !seq_start || !lvl_k || !lvl_v || !out_k || !out_v)
    return BKV_ERR_ARG;
  if (stat_dtype != BKV_F16 && stat_dtype != BKV_BF16) return BKV_ERR_ARG;
  if (out_dtype != BKV_F16 && out_dtype != BKV_BF16 && out_dtype != BKV_F32) return BKV_ERR_ARG;
  if (heads_kv > 64) return BKV_ERR_LIMIT;
  if (!aligned16(out_k) || !aligned16(out_v)) return BKV_ERR_ALIGN;
  if (page_stride_i32 < make_geom(block_size, heads_kv).block_i32) return BKV_ERR_ARG;
  ReadbackParams p;
  p.cache = static_cast<const uint32_t*>(cache);
  p.num_pages = num_pages; p.page_stride = page_stride_i32;
  p.block_size = block_size; p.heads = heads_kv; p.stat_bf16 = stat_dtype == BKV_BF16;
  p.block_table = block_table; p.bt_stride = block_table_stride; p.bt_width = block_table_width;
  p.seq_lens = seq_lens; p.seq_start = seq_start; p.batch = batch; p.max_seq_len = max_seq_len;
  p.lvl_k = lvl_k; p.lvl_v = lvl_v; p.table_dtype = table_dtype;
  p.grouped_k = grouped_k; p.grouped_v = grouped_v;
  p.out_k = out_k; p.out_v = out_v; p.out_dtype = out_dtype;
  const int64_t items = static_cast<int64_t>(batch) * max_seq_len * heads_kv;
  int64_t blocks = (items + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  const size_t smem = static_cast<size_t>(heads_kv) * kGroupsPerHead * 16 * sizeof(float) * 2;
  readback_kernel<<<static_cast<unsigned>(blocks), 256, smem, static_cast<cudaStream_t>(stream)>>>(p);
  return check_launch("bkv_readback_sm100");
}

extern "C" int bkv_derive_slots_sm100(const int32_t* seq_lens, const int32_t* block_table,
                                      int64_t block_table_stride, int64_t block_table_width,
                                      int block_size, int batch, int32_t* slots_out,
                                      bkv_stream_t stream) {
  using namespace bkv;
  if (batch < 0 || block_size <= 0) return BKV_ERR_ARG;
  if (batch == 0) return BKV_OK;
  if (!seq_lens || !block_table || !slots_out) return BKV_ERR_ARG;
  derive_slots_kernel<<<(batch + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      seq_lens, block_table, block_table_stride, block_table_width, block_size, batch, slots_out);
  return check_launch("bkv_derive_slots_sm100");
}
