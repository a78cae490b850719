// Tensor-core fused paged split-KV decode attention over the packed 4-bit cache (sm_100a).
//
// One CTA serves one (split, kv-head [, query-head quad], request).  NW consumer warps
// each own a private ring of 16-token tiles that a producer warp fills with 1-D bulk
// copies (cp.async.bulk + mbarrier); a warp keeps its own online-softmax state, so
// there is no cross-warp synchronisation inside the main loop.  Warp partials are
// merged through shared memory at the end, split partials by the combine kernel.
//
// Dequantisation never materialises K or V.  A 256-entry table indexed by a whole
// code BYTE returns the two fp16 levels of its two nibbles as one MMA operand
// register; the per-(token, group) scale and minimum are applied outside the MMAs:
//   s[t,h]  = sum_g  scale_k[t,g] * (sum_{d in g} q[h,d] * Lk_g[code_k[t,d]]) + min_k[t,g] * sum_{d in g} q[h,d]
//   o[h,d]  = sum_t (p[t,h] * scale_v[t,g(d)]) * Lv_g(d)[code_v[t,d]]  +  sum_t p[t,h] * min_v[t,g(d)]
// The byte table is replicated so that lane l only ever reads shared-memory bank l
// (bank l holds a copy of the table of K group l%4, and of V group l/8): every table
// look-up is conflict-free.  MMA fragments are laid out so that each lane only needs
// levels of "its" group:
//   QK : S^T[(h,g), token] = Q_blockdiag[(h,g), d] * Lk[d, token]   (k-slots of lane tig belong to group tig)
//   PV : O[d, (h,g')]      = Lv^T[d, token] * (p*scale_v)[token, (h,g')]   (rows of lane gid belong to group gid/2)
// Products whose row group and column group differ are computed and discarded.
#include <math_constants.h>

#include "bkv_decode_common.cuh"

namespace bkv {

__device__ int g_decode_status = 0;  // non-zero: a bounded wait gave up (1 producer, 2 consumer)

namespace {

constexpr int kTile = 16;
constexpr int kTileBytes = 2560;
constexpr int kOffKCode = 0;
constexpr int kOffKStat = 1024;
constexpr int kOffVCode = 1280;
constexpr int kOffVStat = 2304;
constexpr int kLutBytes = 65536;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // a wait that lasts 2 s gives up
constexpr float kRescaleThreshold = 8.f;  // log2 units: p stays below 2^8

// ---- PTX helpers --------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait bookkeeping: returns true once `limit` nanoseconds have passed since the
// first failed poll (the clock is only read every 256 polls).
struct WaitBudget {
  uint32_t polls = 0;
  unsigned long long start = 0;
  __device__ __forceinline__ bool expired() {
    if ((++polls & 255u) != 0) return false;
    const unsigned long long now = global_timer_ns();
    if (start == 0) {
      start = now;
      return false;
    }
    return now - start > kWaitLimitNs;
  }
  __device__ __forceinline__ void reset() {
    polls = 0;
    start = 0;
  }
};
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void consumer_bar_sync(int threads) {
  asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ float lo16_to_f32(uint32_t w, bool bf16) {
  return bf16 ? __uint_as_float(w << 16) : __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xFFFFu)));
}
__device__ __forceinline__ float hi16_to_f32(uint32_t w, bool bf16) {
  return bf16 ? __uint_as_float(w & 0xFFFF0000u) : __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16)));
}

template <int NW, int STAGES>
struct SmemLayout {
  static constexpr int kRing = kLutBytes;
  static constexpr int kRingBytes = NW * STAGES * kTileBytes;
  static constexpr int kFullBar = kRing + kRingBytes;
  static constexpr int kEmptyBar = kFullBar + NW * STAGES * 8;
  static constexpr int kNValid = kEmptyBar + NW * STAGES * 8;
  static constexpr int kLevels = kNValid + NW * STAGES * 4;  // fp16 [K|V][4][16]
  static constexpr int kTotal = kLevels + 2 * 4 * 16 * 2;
  // epilogue overlay on the ring: O partials [NW][4][128] f32, then m, l [NW][4]
  static constexpr int kMergeO = kRing;
  static constexpr int kMergeM = kMergeO + NW * 4 * kHeadDim * 4;
  static constexpr int kMergeL = kMergeM + NW * 4 * 4;
  static_assert(kMergeL + NW * 4 * 4 <= kFullBar, "merge overlay must fit in the ring");
};

template <int NW, int STAGES, bool STAT_BF16>
__global__ void __launch_bounds__((NW + 1) * 32, 1) decode_mma_kernel(const DecodeParams p, const int quads) {
  using L = SmemLayout<NW, STAGES>;
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t smem_base = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gid = lane >> 2, tig = lane & 3;

  const int split = blockIdx.x;
  const int head = blockIdx.y / quads, quad = blockIdx.y - head * quads;
  const int b = blockIdx.z;
  const int gqa = p.heads_q / p.heads_kv;
  const int hq0 = head * gqa + quad * 4;
  const int nh = min(4, gqa - quad * 4);
  const int S = p.num_splits;
  const int BS = p.block_size;
  const int tiles_per_page = BS / kTile;

  if (p.flags & BKV_FLAG_PDL_WAIT) pdl_wait();

  // ---- which tiles does this CTA own ------------------------------------------------
  const int seq_len = p.seq_lens[b];
  const int lo = max(p.token_lo, 0);
  const int hi = min(p.token_hi, seq_len);
  int n_tiles = 0;
  const int page_lo = lo / BS;
  if (hi > lo) {
    const int page_hi = (hi + BS - 1) / BS;
    const int span = page_hi - page_lo - split;
    if (span > 0) {
      const int n_pages = (span + S - 1) / S;
      const int last_page = page_lo + split + S * (n_pages - 1);
      n_tiles = n_pages * tiles_per_page;
      if (last_page == page_hi - 1) {
        const int in_last = (hi - last_page * BS + kTile - 1) / kTile;
        n_tiles -= tiles_per_page - in_last;
      }
    }
  }

  if (tid == 0) {
    for (int i = 0; i < NW * STAGES; ++i) {
      mbar_init(smem_base + L::kFullBar + 8 * i, 1);
      mbar_init(smem_base + L::kEmptyBar + 8 * i, 1);
    }
    fence_barrier_init();
  }
  __syncthreads();

  // =====================================================================================
  // Producer warp: lane w feeds consumer warp w.  The lanes run in lock step; a lane whose
  // next ring slot is still in use simply sits the round out.
  // =====================================================================================
  if (warp == NW) {
    const int w = lane;
    const int my_tiles = (w < NW && n_tiles > w) ? (n_tiles - w + NW - 1) / NW : 0;
    const PageGeom g = make_geom(BS, p.heads_kv);
    const int32_t* bt_row = p.block_table + static_cast<int64_t>(b) * p.bt_stride;
    const char* cache_bytes = reinterpret_cast<const char*>(p.cache);
    constexpr int PF = 4;
    int32_t phys_next[PF];
    auto page_of = [&](int k) {
      const int j = w + k * NW;
      return page_lo + split + S * (j / tiles_per_page);
    };
#pragma unroll
    for (int i = 0; i < PF; ++i) phys_next[i] = i < my_tiles ? bt_row[page_of(i)] : 0;
    int32_t phys_cur[PF] = {0, 0, 0, 0};
    int k = 0;
    WaitBudget idle;
    while (true) {
      const bool active = k < my_tiles;
      if (!__any_sync(0xffffffffu, active)) break;
      bool can = false;
      if (active) {
        const int use = k / STAGES;
        const int stage = k - use * STAGES;
        can = use == 0 || mbar_try_wait(smem_base + L::kEmptyBar + 8 * (w * STAGES + stage), (use - 1) & 1);
      }
      if (can) {
        if ((k & (PF - 1)) == 0) {
#pragma unroll
          for (int i = 0; i < PF; ++i) {
            phys_cur[i] = phys_next[i];
            phys_next[i] = (k + PF + i) < my_tiles ? bt_row[page_of(k + PF + i)] : 0;
          }
        }
        int64_t phys = phys_cur[0];
#pragma unroll
        for (int i = 1; i < PF; ++i)
          if ((k & (PF - 1)) == i) phys = phys_cur[i];
        const int stage = k % STAGES;
        const int slot = w * STAGES + stage;
        const int j = w + k * NW;
        const int sub = j % tiles_per_page;
        const int tok0 = page_of(k) * BS + sub * kTile;
        const uint32_t full = smem_base + L::kFullBar + 8 * slot;
        int* nvalid = reinterpret_cast<int*>(smem + L::kNValid) + slot;
        if (phys < 0 || phys >= p.num_pages) {
          *nvalid = 0;  // unmapped page: the consumer skips the tile
          mbar_arrive(full);
        } else {
          *nvalid = min(kTile, hi - tok0);
          const uint32_t dst = smem_base + L::kRing + slot * kTileBytes;
          const char* pg = cache_bytes + phys * p.page_stride * 4;
          mbar_arrive_expect_tx(full, kTileBytes);
          const int code_off = head * (BS * kWordsPerHead) + sub * (kTile * kWordsPerHead);
          bulk_copy_g2s(dst + kOffKCode, pg + 4 * (g.k_code_off + code_off), 1024, full);
          bulk_copy_g2s(dst + kOffKStat, pg + 4 * (g.k_stat_off + head * (BS * 4) + sub * (kTile * 4)), 256, full);
          bulk_copy_g2s(dst + kOffVCode, pg + 4 * (g.v_code_off + code_off), 1024, full);
          const char* vs = pg + 4 * (g.v_stat_off + head * (4 * BS) + sub * kTile);
          if (tiles_per_page == 1) {
            bulk_copy_g2s(dst + kOffVStat, vs, 256, full);
          } else {
#pragma unroll
            for (int gg = 0; gg < 4; ++gg) bulk_copy_g2s(dst + kOffVStat + gg * 64, vs + 4 * gg * BS, 64, full);
          }
        }
        ++k;
      }
      if (!__any_sync(0xffffffffu, can)) {
        if (__any_sync(0xffffffffu, idle.expired())) {
          atomicExch(&g_decode_status, 1);
          break;
        }
        __nanosleep(40);
      } else {
        idle.reset();
      }
    }
    return;
  }

  // =====================================================================================
  // Consumer warps
  // =====================================================================================
  const int cthreads = NW * 32;
  {  // level tables -> fp16 in shared memory
    __half* lv = reinterpret_cast<__half*>(smem + L::kLevels);
    for (int i = tid; i < 128; i += cthreads) {
      const int which = i >> 6, g = (i >> 4) & 3, c = i & 15;
      lv[i] = __float2half_rn(which ? load_v_level(p, head, g, c) : load_k_level(p, head, g, c));
    }
  }
  consumer_bar_sync(cthreads);
  {  // byte -> (level[low nibble], level[high nibble]) table, one copy per bank
    const unsigned short* lv = reinterpret_cast<const unsigned short*>(smem + L::kLevels);
    const int kg = lane & 3, vg = lane >> 3;
    for (int e = warp; e < 256; e += NW) {
      const uint32_t kval = lv[kg * 16 + (e & 15)] | (static_cast<uint32_t>(lv[kg * 16 + (e >> 4)]) << 16);
      const uint32_t vval = lv[64 + vg * 16 + (e & 15)] | (static_cast<uint32_t>(lv[64 + vg * 16 + (e >> 4)]) << 16);
      uint32_t* row = reinterpret_cast<uint32_t*>(smem + e * 256);
      row[lane] = kval;
      row[32 + lane] = vval;
    }
  }

  // ---- query fragments (A operand of QK), pre-scaled by softmax_scale * log2(e) --------
  const int hsel = gid & 3;          // query head of this lane's score / B columns
  const int grow = 2 * (gid >> 2);   // K group of MMA row gid (row gid+8 is group grow+1)
  uint32_t qa[8][4];
  float qs0, qs1;
  {
    const bool live = hsel < nh;
    const int64_t qoff = static_cast<int64_t>(b) * p.q_batch_stride + static_cast<int64_t>(hq0 + hsel) * kHeadDim;
    const bool m0 = tig == grow, m1 = tig == grow + 1;
    float qsum = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float f[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) f[i] = live ? load_q(p.q, qoff + 32 * tig + 4 * j + i, p.q_dtype) * p.scale_log2 : 0.f;
      const uint32_t lo2 = pack_half2(f[0], f[1]), hi2 = pack_half2(f[2], f[3]);
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo2));
      const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&hi2));
      qsum += (a.x + a.y) + (c.x + c.y);
      qa[j][0] = m0 ? lo2 : 0u;
      qa[j][1] = m1 ? lo2 : 0u;
      qa[j][2] = m0 ? hi2 : 0u;
      qa[j][3] = m1 ? hi2 : 0u;
    }
    qs0 = __shfl_sync(0xffffffffu, qsum, gid * 4 + grow);
    qs1 = __shfl_sync(0xffffffffu, qsum, gid * 4 + grow + 1);
  }
  consumer_bar_sync(cthreads);  // table complete

  const int gv = gid >> 1, vu = gid & 1;  // V group / nibble parity of this lane's MMA rows
  const uint32_t klane = lane * 4, vlane = lane * 4 + 128;
  const unsigned char* lut = smem;

  float oacc[8][2][4];
  float cmin[2][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int jn = 0; jn < 2; ++jn)
#pragma unroll
      for (int c = 0; c < 4; ++c) oacc[i][jn][c] = 0.f;
#pragma unroll
  for (int jn = 0; jn < 2; ++jn)
#pragma unroll
    for (int c = 0; c < 4; ++c) cmin[jn][c] = 0.f;
  float m_used = -CUDART_INF_F, l_run = 0.f;
  bool gave_up = false;

  int k = 0;
  for (int j = warp; j < n_tiles && !gave_up; j += NW, ++k) {
    const int use = k / STAGES;
    const int stage = k - use * STAGES;
    const int slot = warp * STAGES + stage;
    {
      const uint32_t full = smem_base + L::kFullBar + 8 * slot;
      WaitBudget budget;
      while (!mbar_try_wait(full, use & 1)) {
        if (__any_sync(0xffffffffu, budget.expired())) {
          gave_up = true;
          break;
        }
      }
      if (gave_up) {
        atomicExch(&g_decode_status, 2);
        break;
      }
    }
    const int nv = reinterpret_cast<const int*>(smem + L::kNValid)[slot];
    const unsigned char* st = smem + L::kRing + slot * kTileBytes;
    if (nv > 0) {
      // ------------------------------ S^T = Q * Lk^T -------------------------------------
      float sacc[2][4];
#pragma unroll
      for (int o = 0; o < 2; ++o) {
#pragma unroll
        for (int c = 0; c < 4; ++c) sacc[o][c] = 0.f;
        const uint4 kw = *reinterpret_cast<const uint4*>(st + kOffKCode + (8 * o + gid) * 64 + tig * 16);
        const uint32_t w4[4] = {kw.x, kw.y, kw.z, kw.w};
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const uint32_t wd = w4[jj >> 1];
          const uint32_t off0 = __byte_perm(wd, klane, (jj & 1) ? 0x5524 : 0x5504);
          const uint32_t off1 = __byte_perm(wd, klane, (jj & 1) ? 0x5534 : 0x5514);
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(lut + off0);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(lut + off1);
          mma16816(sacc[o], qa[jj][0], qa[jj][1], qa[jj][2], qa[jj][3], b0, b1);
        }
      }
      // ------------------------------ scores of this lane ---------------------------------
      float s[2][2];
#pragma unroll
      for (int o = 0; o < 2; ++o) {
        const int t0 = 8 * o + 2 * tig;
        const uint2 st0 = *reinterpret_cast<const uint2*>(st + kOffKStat + t0 * 16 + grow * 4);
        const uint2 st1 = *reinterpret_cast<const uint2*>(st + kOffKStat + (t0 + 1) * 16 + grow * 4);
        float p0 = lo16_to_f32(st0.x, STAT_BF16) * sacc[o][0];
        p0 = fmaf(hi16_to_f32(st0.x, STAT_BF16), qs0, p0);
        p0 = fmaf(lo16_to_f32(st0.y, STAT_BF16), sacc[o][2], p0);
        p0 = fmaf(hi16_to_f32(st0.y, STAT_BF16), qs1, p0);
        float p1 = lo16_to_f32(st1.x, STAT_BF16) * sacc[o][1];
        p1 = fmaf(hi16_to_f32(st1.x, STAT_BF16), qs0, p1);
        p1 = fmaf(lo16_to_f32(st1.y, STAT_BF16), sacc[o][3], p1);
        p1 = fmaf(hi16_to_f32(st1.y, STAT_BF16), qs1, p1);
        p0 += __shfl_xor_sync(0xffffffffu, p0, 16);
        p1 += __shfl_xor_sync(0xffffffffu, p1, 16);
        s[o][0] = (t0 < nv) ? p0 : -CUDART_INF_F;
        s[o][1] = (t0 + 1 < nv) ? p1 : -CUDART_INF_F;
      }
      // ------------------------------ online softmax --------------------------------------
      float tmax = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
      const bool need = tmax > m_used + kRescaleThreshold;
      if (__any_sync(0xffffffffu, need)) {
        const float m_new = need ? tmax : m_used;
        const float corr = (m_new == -CUDART_INF_F) ? 1.f : exp2f(m_used - m_new);
        m_used = m_new;
        l_run *= corr;
        const float ce = __shfl_sync(0xffffffffu, corr, ((2 * tig) & 3) * 4);
        const float co = __shfl_sync(0xffffffffu, corr, ((2 * tig + 1) & 3) * 4);
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int jn = 0; jn < 2; ++jn) {
            oacc[i][jn][0] *= ce;
            oacc[i][jn][1] *= co;
            oacc[i][jn][2] *= ce;
            oacc[i][jn][3] *= co;
          }
#pragma unroll
        for (int jn = 0; jn < 2; ++jn) {
          cmin[jn][0] *= ce;
          cmin[jn][1] *= co;
          cmin[jn][2] *= ce;
          cmin[jn][3] *= co;
        }
      }
      uint32_t ph[2];
#pragma unroll
      for (int o = 0; o < 2; ++o) {
        const float e0 = exp2f(s[o][0] - m_used), e1 = exp2f(s[o][1] - m_used);
        l_run += e0 + e1;
        ph[o] = pack_half2(e0, e1);
      }
      // ------------------------------ W = p * scale_v, p * min_v ---------------------------
      uint32_t wb[2][2], mb[2][2];
#pragma unroll
      for (int jn = 0; jn < 2; ++jn) {
        const int gp = 2 * jn + (gid >> 2);
#pragma unroll
        for (int o = 0; o < 2; ++o) {
          const int t0 = 8 * o + 2 * tig;
          const uint2 vs = *reinterpret_cast<const uint2*>(st + kOffVStat + (gp * kTile + t0) * 4);
          uint32_t sc2, mn2;
          if (STAT_BF16) {
            sc2 = pack_half2(__uint_as_float(vs.x << 16), __uint_as_float(vs.y << 16));
            mn2 = pack_half2(__uint_as_float(vs.x & 0xFFFF0000u), __uint_as_float(vs.y & 0xFFFF0000u));
          } else {
            sc2 = __byte_perm(vs.x, vs.y, 0x5410);
            mn2 = __byte_perm(vs.x, vs.y, 0x7632);
          }
          uint32_t wv = hmul2_u32(ph[o], sc2), mv = hmul2_u32(ph[o], mn2);
          if (nv < kTile) {  // stale statistics behind the last token may be NaN/Inf
            const uint32_t keep = (t0 < nv ? 0x0000FFFFu : 0u) | (t0 + 1 < nv ? 0xFFFF0000u : 0u);
            wv &= keep;
            mv &= keep;
          }
          wb[jn][o] = wv;
          mb[jn][o] = mv;
        }
      }
      // ------------------------------ O += Lv^T * W ---------------------------------------
      {
        const unsigned char* vc = st + kOffVCode + gv * 16;
        const uint4 x00 = *reinterpret_cast<const uint4*>(vc + (2 * tig) * 64);
        const uint4 x01 = *reinterpret_cast<const uint4*>(vc + (2 * tig + 1) * 64);
        const uint4 x10 = *reinterpret_cast<const uint4*>(vc + (8 + 2 * tig) * 64);
        const uint4 x11 = *reinterpret_cast<const uint4*>(vc + (9 + 2 * tig) * 64);
        const uint32_t a00[4] = {x00.x, x00.y, x00.z, x00.w}, a01[4] = {x01.x, x01.y, x01.z, x01.w};
        const uint32_t a10[4] = {x10.x, x10.y, x10.z, x10.w}, a11[4] = {x11.x, x11.y, x11.z, x11.w};
        const int sh0 = 4 * vu, sh1 = 4 - 4 * vu;
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          const uint32_t m0 = ((a00[wi] >> sh0) & 0x0F0F0F0Fu) | ((a01[wi] << sh1) & 0xF0F0F0F0u);
          const uint32_t m1 = ((a10[wi] >> sh0) & 0x0F0F0F0Fu) | ((a11[wi] << sh1) & 0xF0F0F0F0u);
          uint32_t av[2][4];
          av[0][0] = *reinterpret_cast<const uint32_t*>(lut + __byte_perm(m0, vlane, 0x5504));
          av[0][1] = *reinterpret_cast<const uint32_t*>(lut + __byte_perm(m0, vlane, 0x5514));
          av[1][0] = *reinterpret_cast<const uint32_t*>(lut + __byte_perm(m0, vlane, 0x5524));
          av[1][1] = *reinterpret_cast<const uint32_t*>(lut + __byte_perm(m0, vlane, 0x5534));
          av[0][2] = *reinterpret_cast<const uint32_t*>(lut + __byte_perm(m1, vlane, 0x5504));
          av[0][3] = *reinterpret_cast<const uint32_t*>(lut + __byte_perm(m1, vlane, 0x5514));
          av[1][2] = *reinterpret_cast<const uint32_t*>(lut + __byte_perm(m1, vlane, 0x5524));
          av[1][3] = *reinterpret_cast<const uint32_t*>(lut + __byte_perm(m1, vlane, 0x5534));
#pragma unroll
          for (int e = 0; e < 2; ++e)
#pragma unroll
            for (int jn = 0; jn < 2; ++jn)
              mma16816(oacc[2 * wi + e][jn], av[e][0], av[e][1], av[e][2], av[e][3], wb[jn][0], wb[jn][1]);
        }
        const uint32_t ones = 0x3C003C00u;
#pragma unroll
        for (int jn = 0; jn < 2; ++jn) mma16816(cmin[jn], ones, ones, ones, ones, mb[jn][0], mb[jn][1]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_base + L::kEmptyBar + 8 * slot);
  }

  // ---- epilogue: warp partials -> shared memory -> CTA result ---------------------------
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  consumer_bar_sync(cthreads);  // every tile of every warp has been consumed: the ring is free
  float* mo = reinterpret_cast<float*>(smem + L::kMergeO);
  float* mm = reinterpret_cast<float*>(smem + L::kMergeM);
  float* ml = reinterpret_cast<float*>(smem + L::kMergeL);
  if ((tig >> 1) == (gv & 1)) {
    const bool hi_tile = (gv >> 1) != 0;
    const int h0 = (2 * tig) & 3;
    const float c0 = hi_tile ? cmin[1][0] : cmin[0][0];
    const float c1 = hi_tile ? cmin[1][1] : cmin[0][1];
    float* base0 = mo + (warp * 4 + h0) * kHeadDim;
    float* base1 = base0 + kHeadDim;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int d0 = 32 * gv + 4 * i + vu;
      base0[d0] = (hi_tile ? oacc[i][1][0] : oacc[i][0][0]) + c0;
      base1[d0] = (hi_tile ? oacc[i][1][1] : oacc[i][0][1]) + c1;
      base0[d0 + 2] = (hi_tile ? oacc[i][1][2] : oacc[i][0][2]) + c0;
      base1[d0 + 2] = (hi_tile ? oacc[i][1][3] : oacc[i][0][3]) + c1;
    }
  }
  if (tig == 0 && gid < 4) {
    mm[warp * 4 + gid] = m_used;
    ml[warp * 4 + gid] = l_run;
  }
  consumer_bar_sync(cthreads);
  const bool direct = S == 1 && !p.force_partial;
  for (int idx = tid; idx < 4 * kHeadDim; idx += cthreads) {
    const int h = idx >> 7, d = idx & 127;
    if (h >= nh) continue;
    float M = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < NW; ++w)
      if (ml[w * 4 + h] > 0.f) M = fmaxf(M, mm[w * 4 + h]);
    float den = 0.f, num = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float lw = ml[w * 4 + h];
      const float wt = lw > 0.f ? exp2f(mm[w * 4 + h] - M) : 0.f;
      den += wt * lw;
      num += wt * mo[(w * 4 + h) * kHeadDim + d];
    }
    const int64_t row = static_cast<int64_t>(b) * p.heads_q + hq0 + h;
    if (direct) {
      const float o = den > 0.f ? num / den : 0.f;
      store_out(p.out, row * kHeadDim + d, p.out_dtype, o);
      if (p.out_f32) p.out_f32[row * kHeadDim + d] = o;
    } else {
      const int64_t prow = static_cast<int64_t>(split) * p.batch * p.heads_q + row;
      p.o_partial[prow * kHeadDim + d] = den > 0.f ? num : 0.f;
      if (d == 0) {
        p.m_partial[prow] = den > 0.f ? M * kLn2 : -CUDART_INF_F;
        p.l_partial[prow] = den;
      }
    }
  }
}

template <int NW, int STAGES>
int launch_variant(const DecodeParams& p, cudaStream_t stream) {
  using L = SmemLayout<NW, STAGES>;
  const int gqa = p.heads_q / p.heads_kv;
  const int quads = gqa == 8 ? 2 : 1;
  const dim3 grid(p.num_splits, p.heads_kv * quads, p.batch);
  const dim3 block((NW + 1) * 32);
  auto kern = p.stat_bf16 ? decode_mma_kernel<NW, STAGES, true> : decode_mma_kernel<NW, STAGES, false>;
  static bool configured[2][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[p.stat_bf16 ? 1 : 0][dev]) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) {
      set_last_cuda_error(e, "cudaFuncSetAttribute(decode_mma_kernel)");
      return BKV_ERR_CUDA;
    }
    configured[p.stat_bf16 ? 1 : 0][dev] = true;
  }
  kern<<<grid, block, L::kTotal, stream>>>(p, quads);
  return check_launch("bkv_decode_sm100(mma)");
}

}  // namespace

int launch_decode_mma(const DecodeParams& p, cudaStream_t stream) {
  if (p.block_size % kTile != 0 || p.block_size > 1024) return BKV_ERR_UNSUPPORTED;
  if ((p.page_stride * 4) % 16 != 0 || !aligned16(p.cache)) return BKV_ERR_UNSUPPORTED;
  if (p.token_lo % p.block_size != 0) return BKV_ERR_UNSUPPORTED;
  return launch_variant<8, 4>(p, stream);
}

int read_decode_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(int));
  const int zero = 0;
  cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int));
  return v;
}

}  // namespace bkv
