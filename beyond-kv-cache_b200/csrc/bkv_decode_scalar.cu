// Plain CUDA-core packed decode attention and the log-sum-exp combine kernel.
//
// decode_scalar_kernel is the simple, obviously-correct form of the fused paged
// split-KV decode: every lane owns 4 of the 128 head dimensions, dequantises its
// 4 K and 4 V scalars of a token in registers (nibble -> level -> *scale + min) and
// the warp reduces the dot products by shuffle.  It accepts any page size and GQA
// ratio up to 8 and is the kernel used for shapes the tensor-core kernel does not
// take; it is not the bandwidth-optimised path.
#include <math_constants.h>

#include "bkv_decode_common.cuh"

namespace bkv {

namespace {

constexpr int kScalarWarps = 4;

template <int GQA>
__global__ void __launch_bounds__(kScalarWarps * 32) decode_scalar_kernel(const DecodeParams p) {
  __shared__ float s_lk[kGroupsPerHead][16];
  __shared__ float s_lv[kGroupsPerHead][16];
  __shared__ float s_o[kScalarWarps][GQA][kHeadDim];
  __shared__ float s_m[kScalarWarps][GQA];
  __shared__ float s_l[kScalarWarps][GQA];

  const int split = blockIdx.x, head = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int grp = lane >> 3;
  if (p.flags & BKV_FLAG_PDL_WAIT) pdl_wait();

  if (tid < 64) {
    const int g = tid >> 4, c = tid & 15;
    s_lk[g][c] = load_k_level(p, head, g, c);
  } else {
    const int g = (tid - 64) >> 4, c = tid & 15;
    s_lv[g][c] = load_v_level(p, head, g, c);
  }

  float qv[GQA][4];
#pragma unroll
  for (int h = 0; h < GQA; ++h)
#pragma unroll
    for (int i = 0; i < 4; ++i)
      qv[h][i] = load_q(p.q, b * p.q_batch_stride + (head * GQA + h) * kHeadDim + lane * 4 + i, p.q_dtype) *
                 p.scale_log2;
  __syncthreads();

  float acc[GQA][4], m2[GQA], l[GQA];
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    m2[h] = -CUDART_INF_F;
    l[h] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[h][i] = 0.f;
  }

  const int BS = p.block_size;
  const PageGeom g = make_geom(BS, p.heads_kv);
  const int seq_len = p.seq_lens[b];
  const int lo = max(p.token_lo, 0);
  const int hi = min(p.token_hi, seq_len);
  const bool bf16 = p.stat_bf16 != 0;
  if (hi > lo) {
    const int page_lo = lo / BS;
    const int page_hi = (hi + BS - 1) / BS;
    for (int page = page_lo + split + p.num_splits * warp; page < page_hi;
         page += p.num_splits * kScalarWarps) {
      const int64_t phys = p.block_table[b * p.bt_stride + page];
      if (phys < 0 || phys >= p.num_pages) continue;
      const uint32_t* pg = p.cache + phys * p.page_stride;
      const uint32_t* kc = pg + g.k_code_off + head * (BS * kWordsPerHead) + (lane >> 1);
      const uint32_t* vc = pg + g.v_code_off + head * (BS * kWordsPerHead) + (lane >> 1);
      const uint32_t* ks = pg + g.k_stat_off + head * (BS * 4) + grp;
      const uint32_t* vs = pg + g.v_stat_off + head * (4 * BS) + grp * BS;
      const int t0 = page * BS;
      const int tok_lo = max(lo - t0, 0), tok_hi = min(hi - t0, BS);
      for (int tok = tok_lo; tok < tok_hi; ++tok) {
        const uint32_t kw = kc[tok * kWordsPerHead] >> ((lane & 1) * 16);
        const uint32_t vw = vc[tok * kWordsPerHead] >> ((lane & 1) * 16);
        const uint32_t kst = ks[tok * 4];
        const uint32_t vst = vs[tok];
        const float ksc = stat_bits_to_f32(kst, bf16), kmn = stat_bits_to_f32(kst >> 16, bf16);
        const float vsc = stat_bits_to_f32(vst, bf16), vmn = stat_bits_to_f32(vst >> 16, bf16);
        float kh[4], vh[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          kh[i] = fmaf(s_lk[grp][(kw >> (4 * i)) & 15], ksc, kmn);
          vh[i] = fmaf(s_lv[grp][(vw >> (4 * i)) & 15], vsc, vmn);
        }
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

  // merge the warps of this CTA; thread tid owns dimension tid of every head
  const bool direct = p.num_splits == 1 && !p.force_partial;
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    float M = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < kScalarWarps; ++w)
      if (s_l[w][h] > 0.f) M = fmaxf(M, s_m[w][h]);
    float den = 0.f, num = 0.f;
#pragma unroll
    for (int w = 0; w < kScalarWarps; ++w) {
      const float wt = s_l[w][h] > 0.f ? exp2f(s_m[w][h] - M) : 0.f;
      den += wt * s_l[w][h];
      num += wt * s_o[w][h][tid];
    }
    const int hq = head * GQA + h;
    const int64_t row = static_cast<int64_t>(b) * p.heads_q + hq;
    if (direct) {
      const float o = den > 0.f ? num / den : 0.f;
      store_out(p.out, row * kHeadDim + tid, p.out_dtype, o);
      if (p.out_f32) p.out_f32[row * kHeadDim + tid] = o;
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

// One CTA of 128 threads merges the splits of one (request, query head) row.
__global__ void __launch_bounds__(kHeadDim) combine_strided_kernel(const float* __restrict__ o_partial,
                                                                   const float* __restrict__ m_partial,
                                                                   const float* __restrict__ l_partial,
                                                                   int num_splits, int64_t rows, int64_t split_stride,
                                                                   void* out, int out_dtype, float* out_f32) {
  // split s: o at o_partial + s*split_stride (rows x 128), m and l at m/l_partial + s*split_stride
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int d = threadIdx.x;
  float M = -CUDART_INF_F;
  for (int s = 0; s < num_splits; ++s)
    if (l_partial[s * split_stride + row] > 0.f) M = fmaxf(M, m_partial[s * split_stride + row]);
  float den = 0.f, num = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float ls = l_partial[s * split_stride + row];
    const float w = ls > 0.f ? __expf(m_partial[s * split_stride + row] - M) : 0.f;
    den += w * ls;
    num += w * o_partial[s * split_stride + row * kHeadDim + d];
  }
  const float o = den > 0.f ? num / den : 0.f;
  store_out(out, row * kHeadDim + d, out_dtype, o);
  if (out_f32) out_f32[row * kHeadDim + d] = o;
}

}  // namespace

// Dense partials ([splits][rows][128], [splits][rows], [splits][rows]) have split strides of
// rows*128 and rows elements; a packed per-rank record (o | m | l) has one stride for all three.
__global__ void __launch_bounds__(kHeadDim) combine_dense_kernel(const float* __restrict__ o_partial,
                                                                 const float* __restrict__ m_partial,
                                                                 const float* __restrict__ l_partial,
                                                                 int num_splits, int64_t rows, void* out,
                                                                 int out_dtype, float* out_f32) {
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int d = threadIdx.x;
  float M = -CUDART_INF_F;
  for (int s = 0; s < num_splits; ++s)
    if (l_partial[s * rows + row] > 0.f) M = fmaxf(M, m_partial[s * rows + row]);
  float den = 0.f, num = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float ls = l_partial[s * rows + row];
    const float w = ls > 0.f ? __expf(m_partial[s * rows + row] - M) : 0.f;
    den += w * ls;
    num += w * o_partial[(s * rows + row) * kHeadDim + d];
  }
  const float o = den > 0.f ? num / den : 0.f;
  store_out(out, row * kHeadDim + d, out_dtype, o);
  if (out_f32) out_f32[row * kHeadDim + d] = o;
}

int launch_combine(const float* o_partial, const float* m_partial, const float* l_partial,
                   int num_splits, int64_t rows, void* out, int out_dtype, float* out_f32,
                   cudaStream_t stream) {
  if (rows <= 0) return BKV_OK;
  combine_dense_kernel<<<static_cast<unsigned>(rows), kHeadDim, 0, stream>>>(
      o_partial, m_partial, l_partial, num_splits, rows, out, out_dtype, out_f32);
  return check_launch("bkv_combine_sm100");
}

int launch_combine_packed(const float* records, int num_splits, int64_t rows, void* out, int out_dtype,
                          float* out_f32, cudaStream_t stream) {
  if (rows <= 0) return BKV_OK;
  const int64_t stride = rows * (kHeadDim + 2);  // one record: o (rows x 128) | m (rows) | l (rows)
  combine_strided_kernel<<<static_cast<unsigned>(rows), kHeadDim, 0, stream>>>(
      records, records + rows * kHeadDim, records + rows * (kHeadDim + 1), num_splits, rows, stride, out, out_dtype,
      out_f32);
  return check_launch("bkv_combine_packed_sm100");
}

int launch_decode_scalar(const DecodeParams& p, cudaStream_t stream) {
  const dim3 grid(p.num_splits, p.heads_kv, p.batch);
  const int gqa = p.heads_q / p.heads_kv;
  switch (gqa) {
    case 1: decode_scalar_kernel<1><<<grid, kScalarWarps * 32, 0, stream>>>(p); break;
    case 2: decode_scalar_kernel<2><<<grid, kScalarWarps * 32, 0, stream>>>(p); break;
    case 4: decode_scalar_kernel<4><<<grid, kScalarWarps * 32, 0, stream>>>(p); break;
    case 8: decode_scalar_kernel<8><<<grid, kScalarWarps * 32, 0, stream>>>(p); break;
    default: return BKV_ERR_UNSUPPORTED;
  }
  return check_launch("bkv_decode_sm100(scalar)");
}

}  // namespace bkv
