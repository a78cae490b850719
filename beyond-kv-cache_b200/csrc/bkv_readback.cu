// Paged read-back of the packed cache to dense varlen K/V, and the last-token
// slot derivation used by graph-safe decode (sm_100a).
//
// Read-back mirrors the encode mapping: one warp per request position, walking the kv-heads;
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

// store eight reconstructed scalars of one lane as kOut (BKV_F32 / BKV_BF16 / BKV_F16)
template <int kOut>
__device__ __forceinline__ void store_row8(void* dst, int64_t o, const float (&y)[8]) {
  if (kOut == BKV_F32) {
    float4* d4 = reinterpret_cast<float4*>(static_cast<float*>(dst) + o);
    d4[0] = make_float4(y[0], y[1], y[2], y[3]);
    d4[1] = make_float4(y[4], y[5], y[6], y[7]);
  } else {
    uint4 raw;
    uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      w[i] = kOut == BKV_BF16 ? (f32_to_bf16_bits(y[2 * i]) | (f32_to_bf16_bits(y[2 * i + 1]) << 16))
                              : (f32_to_f16_bits(y[2 * i]) | (f32_to_f16_bits(y[2 * i + 1]) << 16));
    *reinterpret_cast<uint4*>(static_cast<unsigned short*>(dst) + o) = raw;
  }
}

// A warp owns one (request, position) and walks its KV heads; the page is located once per
// token and the code word and statistic of the next head are in flight while this one is
// expanded.  Level tables in shared memory: entry j of the table lane l needs for head h at
// [h][j][l] (bank l: the data-dependent look-ups of a warp never collide; 2 KB per head), or,
// with kCompact (more than 32 heads), one copy per table.
template <int kOut, bool kCompact>
__global__ void __launch_bounds__(256) readback_kernel(const ReadbackParams p) {
  extern __shared__ float s_lvl[];
  const int tables = p.heads * kGroupsPerHead;
  if (kCompact) {
    for (int i = threadIdx.x; i < tables * 16; i += blockDim.x) {
      const int t = i >> 4, j = i & 15;
      s_lvl[i] = load_table_f32(p.lvl_k, (p.grouped_k ? t * 16 : 0) + j, p.table_dtype);
      s_lvl[tables * 16 + i] = load_table_f32(p.lvl_v, (p.grouped_v ? t * 16 : 0) + j, p.table_dtype);
    }
  } else {
    for (int i = threadIdx.x; i < p.heads * 16 * 32; i += blockDim.x) {
      const int l = i & 31, j = (i >> 5) & 15, h = i >> 9;
      const int t = h * kGroupsPerHead + ((l & 15) >> 2);
      const bool v = l >= 16;
      const int grouped = v ? p.grouped_v : p.grouped_k;
      s_lvl[i] = load_table_f32(v ? p.lvl_v : p.lvl_k, (grouped ? t * 16 : 0) + j, p.table_dtype);
    }
  }
  __syncthreads();

  const int lane = threadIdx.x & 31, is_v = lane >> 4, sub = lane & 15, grp = sub >> 2;
  const uint32_t warps_per_block = blockDim.x >> 5;
  const int BS = p.block_size;
  const PageGeom g = make_geom(BS, p.heads);
  const bool bf16 = p.stat_bf16 != 0;
  constexpr int kEntryStride = kCompact ? 1 : 32;
  const int head_stride = kCompact ? kGroupsPerHead * 16 : 16 * 32;
  const float* const lvl_base = kCompact ? s_lvl + (is_v ? tables * 16 : 0) + grp * 16 : s_lvl + lane;
  void* const dst = is_v ? p.out_v : p.out_k;
  const uint32_t lvl_a = static_cast<uint32_t>(__cvta_generic_to_shared(s_lvl));
  const uint32_t lane4 = lane * 4;
  const uint32_t max_len = static_cast<uint32_t>(p.max_seq_len);
  const uint32_t tokens = static_cast<uint32_t>(p.batch) * max_len;  // < 2^31, checked by the launcher
  const uint32_t step = gridDim.x * warps_per_block;
  // what locates a token: its page id (negative: nothing to read) and position; read one token
  // ahead so that the chain sequence length -> block table -> page is off the critical path
  struct Located {
    int64_t phys;
    int pos;
    uint32_t b;
  };
  auto locate = [&](const uint32_t item) -> Located {
    Located t;
    t.b = item / max_len;
    t.pos = static_cast<int>(item - t.b * max_len);
    t.phys = -1;
    const int lp = t.pos / BS;
    if (t.pos < p.seq_lens[t.b] && lp < p.bt_width) t.phys = p.block_table[t.b * p.bt_stride + lp];
    return t;
  };
  constexpr int kDepth = 4;  // heads whose code word and statistic are in flight per lane
  const int code_step = BS * kWordsPerHead, stat_step = BS * 4;
  uint32_t item = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (item >= tokens) return;
  Located cur = locate(item);
  for (; item < tokens; item += step) {
    const uint32_t next_item = item + step;
    Located nxt = cur;
    if (next_item < tokens) nxt = locate(next_item);
    if (cur.phys >= 0 && cur.phys < p.num_pages) {
      const int tok = cur.pos % BS;
      const uint32_t* const pg = p.cache + cur.phys * p.page_stride;
      // this lane's code word and statistic of head 0; every further head adds a constant
      const uint32_t* code_ptr = pg + (is_v ? g.v_code_off : g.k_code_off) + tok * kWordsPerHead + sub;
      const uint32_t* stat_ptr = is_v ? pg + g.v_stat_off + grp * BS + tok : pg + g.k_stat_off + tok * 4 + grp;
      int64_t o = (static_cast<int64_t>(p.seq_start[cur.b]) + cur.pos) * p.heads * kHeadDim + sub * 8;
      uint32_t word[kDepth], st[kDepth];
#pragma unroll
      for (int d = 0; d < kDepth; ++d) {
        if (d < p.heads) {
          word[d] = code_ptr[d * code_step];
          st[d] = stat_ptr[d * stat_step];
        }
      }
      for (int head0 = 0; head0 < p.heads; head0 += kDepth) {
#pragma unroll
        for (int d = 0; d < kDepth; ++d) {
          const int head = head0 + d;
          if (head >= p.heads) break;
          const uint32_t w = word[d];
          const float sc = stat_bits_to_f32(st[d], bf16), mn = stat_bits_to_f32(st[d] >> 16, bf16);
          if (head + kDepth < p.heads) {
            word[d] = code_ptr[(head + kDepth) * code_step];
            st[d] = stat_ptr[(head + kDepth) * stat_step];
          }
          float y[8];
          if (kCompact) {
            const float* const lvl = lvl_base + head * head_stride;
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = __fadd_rn(__fmul_rn(lvl[(w >> (4 * i)) & 15], sc), mn);
          } else {
            // entry j of this lane's table sits at head_a + j * 128 + lane * 4: the nibble is moved
            // to bits 7-10 and merged with the lane's bits in one logic operation
            const uint32_t head_a = lvl_a + static_cast<uint32_t>(head) * (16 * 32 * sizeof(float));
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint32_t moved = 4 * i < 7 ? w << (7 - 4 * i) : w >> (4 * i - 7);
              y[i] = __fadd_rn(__fmul_rn(shared_f32(head_a + ((moved & 0x780u) | lane4)), sc), mn);
            }
          }
          store_row8<kOut>(dst, o, y);
          o += kHeadDim;
        }
      }
    }
    cur = nxt;
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
  const int64_t tokens = static_cast<int64_t>(batch) * max_seq_len;
  if (tokens >= (1ll << 31)) return BKV_ERR_LIMIT;
  int64_t blocks = (tokens + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const bool compact = heads_kv > 32;
  const size_t smem = compact ? static_cast<size_t>(heads_kv) * kGroupsPerHead * 16 * sizeof(float) * 2
                              : static_cast<size_t>(heads_kv) * 16 * 32 * sizeof(float);
#define BKV_READBACK_PICK(C) \
  (out_dtype == BKV_F32 ? readback_kernel<BKV_F32, C> : out_dtype == BKV_BF16 ? readback_kernel<BKV_BF16, C> : readback_kernel<BKV_F16, C>)
  auto kern = compact ? BKV_READBACK_PICK(true) : BKV_READBACK_PICK(false);
#undef BKV_READBACK_PICK
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) {
      set_last_cuda_error(e, "cudaFuncSetAttribute(readback_kernel)");
      return BKV_ERR_CUDA;
    }
  }
  if (blocks >= 148 * 8) {  // persistent grid: the blocks that are resident at once
    int dev = 0, sms = 148, resident = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, 256, smem) == cudaSuccess && resident > 0)
      blocks = static_cast<int64_t>(sms) * resident;
  }
  kern<<<static_cast<unsigned>(blocks), 256, smem, static_cast<cudaStream_t>(stream)>>>(p);
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
