// 16-bit-KV paged decode attention of the same shape and split policy as the packed
// kernel: the full-precision baseline that the packed path is timed against.
// K and V pages are [num_pages][block_size][heads_kv][128] fp16/bf16.
#include <math_constants.h>

#include "bkv_decode_common.cuh"

namespace bkv {

namespace {

struct DenseParams {
  const void* q;
  int64_t q_batch_stride;
  int q_dtype;
  const unsigned short* k_pages;
  const unsigned short* v_pages;
  int kv_bf16;
  int64_t num_pages;
  int block_size, heads_kv, heads_q, batch;
  const int32_t* block_table;
  int64_t bt_stride;
  const int32_t* seq_lens;
  void* out;
  int out_dtype;
  float* o_partial;
  float* m_partial;
  float* l_partial;
  int num_splits;
  int max_seq_len;
  float scale_log2;
};

constexpr int kDenseWarps = 4;

__device__ __forceinline__ void unpack4(uint2 raw, bool bf16, float (&x)[4]) {
  if (bf16) {
    x[0] = __uint_as_float(raw.x << 16);
    x[1] = __uint_as_float(raw.x & 0xFFFF0000u);
    x[2] = __uint_as_float(raw.y << 16);
    x[3] = __uint_as_float(raw.y & 0xFFFF0000u);
  } else {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
  }
}

template <int GQA>
__global__ void __launch_bounds__(kDenseWarps * 32) decode_dense_kernel(const DenseParams p) {
  __shared__ float s_o[kDenseWarps][GQA][kHeadDim];
  __shared__ float s_m[kDenseWarps][GQA];
  __shared__ float s_l[kDenseWarps][GQA];
  const int split = blockIdx.x, head = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool bf16 = p.kv_bf16 != 0;

  float qv[GQA][4];
#pragma unroll
  for (int h = 0; h < GQA; ++h)
#pragma unroll
    for (int i = 0; i < 4; ++i)
      qv[h][i] = load_q(p.q, b * p.q_batch_stride + (head * GQA + h) * kHeadDim + lane * 4 + i, p.q_dtype) *
                 p.scale_log2;
  float acc[GQA][4], m2[GQA], l[GQA];
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    m2[h] = -CUDART_INF_F;
    l[h] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[h][i] = 0.f;
  }
  const int BS = p.block_size;
  const int hi = min(p.max_seq_len, p.seq_lens[b]);
  const int page_hi = (hi + BS - 1) / BS;
  const int64_t tok_stride = static_cast<int64_t>(p.heads_kv) * kHeadDim;
  for (int page = split + p.num_splits * warp; page < page_hi; page += p.num_splits * kDenseWarps) {
    const int64_t phys = p.block_table[b * p.bt_stride + page];
    if (phys < 0 || phys >= p.num_pages) continue;
    const int64_t base = phys * BS * tok_stride + head * kHeadDim + lane * 4;
    const int tok_hi = min(hi - page * BS, BS);
    for (int tok = 0; tok < tok_hi; ++tok) {
      float kh[4], vh[4];
      unpack4(*reinterpret_cast<const uint2*>(p.k_pages + base + tok * tok_stride), bf16, kh);
      unpack4(*reinterpret_cast<const uint2*>(p.v_pages + base + tok * tok_stride), bf16, vh);
#pragma unroll
      for (int h = 0; h < GQA; ++h) {
        float s = qv[h][0] * kh[0] + qv[h][1] * kh[1] + qv[h][2] * kh[2] + qv[h][3] * kh[3];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float m_new = fmaxf(m2[h], s);
        const float corr = exp2f(m2[h] - m_new);
        const float pr = exp2f(s - m_new);
        l[h] = l[h] * corr + pr;
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[h][i] = acc[h][i] * corr + pr * vh[i];
        m2[h] = m_new;
      }
    }
  }
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
#pragma unroll
    for (int i = 0; i < 4; ++i) s_o[warp][h][lane * 4 + i] = acc[h][i];
    if (lane == 0) {
      s_m[warp][h] = m2[h];
      s_l[warp][h] = l[h];
    }
  }
  __syncthreads();
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    float M = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < kDenseWarps; ++w)
      if (s_l[w][h] > 0.f) M = fmaxf(M, s_m[w][h]);
    float den = 0.f, num = 0.f;
#pragma unroll
    for (int w = 0; w < kDenseWarps; ++w) {
      const float wt = s_l[w][h] > 0.f ? exp2f(s_m[w][h] - M) : 0.f;
      den += wt * s_l[w][h];
      num += wt * s_o[w][h][tid];
    }
    const int64_t row = static_cast<int64_t>(b) * p.heads_q + head * GQA + h;
    if (p.num_splits == 1) {
      store_out(p.out, row * kHeadDim + tid, p.out_dtype, den > 0.f ? num / den : 0.f);
    } else {
      const int64_t prow = static_cast<int64_t>(split) * p.batch * p.heads_q + row;
      p.o_partial[prow * kHeadDim + tid] = num;
      if (tid == 0) {
        p.m_partial[prow] = den > 0.f ? M * kLn2 : -CUDART_INF_F;
        p.l_partial[prow] = den;
      }
    }
  }
}

}  // namespace
}  // namespace bkv

extern "C" int bkv_decode_dense_sm100(const void* q, int64_t q_batch_stride, int q_dtype,
                                      const void* k_pages, const void* v_pages, int kv_dtype,
                                      int64_t num_pages, int block_size, int heads_kv,
                                      const int32_t* block_table, int64_t block_table_stride,
                                      const int32_t* seq_lens, void* out, int out_dtype,
                                      float* o_partial, float* m_partial, float* l_partial,
                                      int num_splits, int batch, int heads_q, int max_seq_len,
                                      float softmax_scale, bkv_stream_t stream) {
  using namespace bkv;
  if (batch < 0 || heads_q <= 0 || heads_kv <= 0 || block_size <= 0 || max_seq_len <= 0)
    return BKV_ERR_ARG;
  if (batch == 0) return BKV_OK;
  if (!q || !k_pages || !v_pages || !block_table || !seq_lens || !out) return BKV_ERR_ARG;
  if (kv_dtype != BKV_F16 && kv_dtype != BKV_BF16) return BKV_ERR_ARG;
  if (heads_q % heads_kv) return BKV_ERR_ARG;
  if (num_splits < 1 || num_splits > 64) return BKV_ERR_ARG;
  if (num_splits > 1 && (!o_partial || !m_partial || !l_partial)) return BKV_ERR_ARG;
  if (!aligned16(k_pages) || !aligned16(v_pages)) return BKV_ERR_ALIGN;
  DenseParams p;
  p.q = q; p.q_batch_stride = q_batch_stride; p.q_dtype = q_dtype;
  p.k_pages = static_cast<const unsigned short*>(k_pages);
  p.v_pages = static_cast<const unsigned short*>(v_pages);
  p.kv_bf16 = kv_dtype == BKV_BF16;
  p.num_pages = num_pages; p.block_size = block_size; p.heads_kv = heads_kv; p.heads_q = heads_q;
  p.batch = batch; p.block_table = block_table; p.bt_stride = block_table_stride;
  p.seq_lens = seq_lens; p.out = out; p.out_dtype = out_dtype;
  p.o_partial = o_partial; p.m_partial = m_partial; p.l_partial = l_partial;
  p.num_splits = num_splits; p.max_seq_len = max_seq_len;
  p.scale_log2 = softmax_scale * kLog2e;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(num_splits, heads_kv, batch);
  switch (heads_q / heads_kv) {
    case 1: decode_dense_kernel<1><<<grid, kDenseWarps * 32, 0, s>>>(p); break;
    case 2: decode_dense_kernel<2><<<grid, kDenseWarps * 32, 0, s>>>(p); break;
    case 4: decode_dense_kernel<4><<<grid, kDenseWarps * 32, 0, s>>>(p); break;
    case 8: decode_dense_kernel<8><<<grid, kDenseWarps * 32, 0, s>>>(p); break;
    default: return BKV_ERR_UNSUPPORTED;
  }
  int rc = check_launch("bkv_decode_dense_sm100");
  if (rc != BKV_OK) return rc;
  if (num_splits > 1)
    return launch_combine(o_partial, m_partial, l_partial, num_splits,
                          static_cast<int64_t>(batch) * heads_q, out, out_dtype, nullptr, s);
  return BKV_OK;
}
