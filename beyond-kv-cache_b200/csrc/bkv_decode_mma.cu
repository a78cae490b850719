// Tensor-core fused paged split-KV decode attention over the packed 4-bit cache (sm_100a).
//
// One CTA serves one (split, kv-head [, query-head quad], request).  Each of its NW warps
// owns a private ring of 16-token tiles which it fills itself with 1-D bulk copies
// (cp.async.bulk + mbarrier, five lanes issue the five chunks of a tile in parallel) and
// keeps its own online-softmax state, so there is no cross-warp synchronisation inside
// the main loop.  Warp partials are merged through shared memory at the end, split
// partials by the combine kernel.
//
// Dequantisation never materialises K or V.  A 256-entry table indexed by a whole
// code BYTE returns the two fp16 levels of its two nibbles as one MMA operand
// register; the per-(token, group) scale and minimum are applied outside the MMAs:
//   s[t,h]  = sum_g  scale_k[t,g] * (sum_{d in g} q[h,d] * Lk_g[code_k[t,d]]) + min_k[t,g] * sum_{d in g} q[h,d]
//   o[h,d]  = sum_t (p[t,h] * scale_v[t,g(d)]) * Lv_g(d)[code_v[t,d]]  +  sum_t p[t,h] * min_v[t,g(d)]
// The byte tables are replicated so that lane l only ever reads shared-memory bank l, which
// makes every look-up conflict-free.  An MMA works on one PAIR of groups {P, P+2} (P = 0, 1);
// bank l of table block P holds the K table of the group lane l feeds into the QK MMAs of
// pair P, and the V table of the group lane l feeds into the PV MMAs of pair P:
//   QK : S[token, (h, g)]  = Lk[token, d] * Q_blockdiag[d, (h, g)]        (k-slots of lane tig: group 2*(tig/2)+P)
//   PV : O[d, (h, g')]     = Lv^T[d, token] * (p*scale_v)[token, (h, g')]  (rows of lane gid:  group 2*(gid/4)+P)
// Half of the products pair a d with a column of the other group of the pair and are discarded.
// The probabilities leave the QK accumulators with tokens spread over gid and are handed to the
// PV operand layout (tokens spread over tig) with two shuffles per tile.
//
// The tables sit at the fixed shared-memory addresses 0x10000 / 0x20000, so a look-up address
// is a single byte-permute of (code word, lane constant) with no addition.  Tokens of a tile are
// assigned to MMA rows / k-slots through fixed permutations (kTokOfSlot, kRowSlot) which,
// together with a 16-byte skew of the second half of the code chunks, make every 64-bit code
// load of a half-warp conflict-free.
#include <math_constants.h>

#include <type_traits>

#include "bkv_decode_common.cuh"
#include "bkv_mma_ptx.cuh"

namespace bkv {

__device__ int g_decode_status = 0;  // non-zero: 1/2 a bounded wait gave up, 3 unexpected smem base

namespace {

using namespace mma;

constexpr int kHiSlots = (kSmemEnd - kRingHi) / kTileBytes;

constexpr int BKV_FLAG_DEBUG_NOLOAD = 0x100;  // timing experiment: reuse the first ring fill
constexpr int BKV_FLAG_DEBUG_NOCOPY = 0x400;  // timing experiment: run the issue logic without the copies
constexpr int BKV_FLAG_DEBUG_NOWAIT = 0x200;  // timing experiment: issue loads but never wait for them

__device__ __forceinline__ uint32_t slot_addr(int slot) {
  return slot < kLoSlots ? kRingLo + slot * kTileBytes : kRingHi + (slot - kLoSlots) * kTileBytes;
}

template <int NW, int STAGES>
struct Smem {
  static constexpr int kSlots = NW * STAGES;
  static_assert(kSlots <= kLoSlots + kHiSlots, "ring does not fit next to the two table blocks");
  static_assert(kSlots <= 64, "control block holds at most 64 barriers");
  static constexpr uint32_t kFullBar = kSmemBase;        // 8 B each
  static constexpr uint32_t kLevels = kSmemBase + 1280;  // fp16 [K|V][4][16]
  static constexpr int kDynBytes = static_cast<int>(kSmemEnd - kSmemBase);
  // epilogue overlay in the high region (all ring traffic has drained by then)
  static constexpr uint32_t kMergeO = kRingHi;
  static constexpr uint32_t kMergeM = kMergeO + NW * 4 * kHeadDim * 4;
  static constexpr uint32_t kMergeL = kMergeM + NW * 4 * 4;
  static_assert(kMergeL + NW * 4 * 4 <= kSmemEnd, "merge overlay must fit in the high region");
};

template <int NW, int STAGES, bool STAT_BF16, int ABL = 0>
__global__ void __maxnreg__(max_regs_for(NW)) decode_mma_kernel(const DecodeParams p, const int quads) {
  using L = Smem<NW, STAGES>;
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t smem_base = smem_u32(smem);
  if (smem_base != kSmemBase) {  // the fixed-address tables need the documented layout
    if (threadIdx.x == 0) atomicExch(&g_decode_status, 3);
    return;
  }
  auto gptr = [&](uint32_t shared_addr) { return smem + (shared_addr - kSmemBase); };
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
  const int log2r = 31 - __clz(BS / kTile);  // tiles per page is a power of two
  const int tiles_per_page = 1 << log2r;
  const bool noload = (p.flags & BKV_FLAG_DEBUG_NOLOAD) != 0;
  const bool nocopy = (p.flags & BKV_FLAG_DEBUG_NOCOPY) != 0;
  const bool nowait = (p.flags & BKV_FLAG_DEBUG_NOWAIT) != 0 || nocopy;

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
  const int my_tiles = n_tiles > warp ? (n_tiles - warp + NW - 1) / NW : 0;  // tiles warp, warp+NW, ...

  if (tid == 0) {
    for (int i = 0; i < L::kSlots; ++i) mbar_init(L::kFullBar + 8 * i, 1);
    fence_barrier_init();
  }
  __syncthreads();

  // ---- this warp's loader: lane c issues chunk c of a tile --------------------------------
  // chunks: 0/1 K codes of tokens 0-7 / 8-15 (512 B each), 2 K statistics (256), 3/4 V codes
  // (512 each), then V statistics: one 256 B chunk for 16-token pages, else 64 B per group.
  const PageGeom geo = make_geom(BS, p.heads_kv);
  const int n_chunks = tiles_per_page == 1 ? 6 : 9;
  uint32_t ch_src = 0, ch_sub = 0, ch_dst = 0, ch_bytes = 0;
  {
    const uint32_t code_head = head * (BS * kWordsPerHead) * 4;
    if (lane == 0) { ch_src = geo.k_code_off * 4 + code_head; ch_sub = 1024; ch_dst = kOffKLo; ch_bytes = 512; }
    if (lane == 1) { ch_src = geo.k_code_off * 4 + code_head + 512; ch_sub = 1024; ch_dst = kOffKHi; ch_bytes = 512; }
    if (lane == 2) { ch_src = (geo.k_stat_off + head * (BS * 4)) * 4; ch_sub = 256; ch_dst = kOffKStat; ch_bytes = 256; }
    if (lane == 3) { ch_src = geo.v_code_off * 4 + code_head; ch_sub = 1024; ch_dst = kOffVLo; ch_bytes = 512; }
    if (lane == 4) { ch_src = geo.v_code_off * 4 + code_head + 512; ch_sub = 1024; ch_dst = kOffVHi; ch_bytes = 512; }
    if (lane >= 5 && lane < n_chunks) {
      const int gg = lane - 5;
      ch_src = (geo.v_stat_off + head * (4 * BS) + gg * BS) * 4;
      ch_sub = 64;
      ch_dst = kOffVStat + gg * 64;
      ch_bytes = tiles_per_page == 1 ? 256 : 64;
    }
  }
  const int32_t* bt_row = p.block_table + static_cast<int64_t>(b) * p.bt_stride;
  const char* src_base = reinterpret_cast<const char*>(p.cache) + ch_src;  // this lane's chunk inside page 0
  const int64_t page_bytes = p.page_stride * 4;
  const uint32_t num_pages_u = static_cast<uint32_t>(min(p.num_pages, static_cast<int64_t>(0x7fffffff)));
  auto page_of = [&](int ki) { return page_lo + split + S * ((warp + ki * NW) >> log2r); };
  // lane l holds the physical page of tile (base + l); the next 32 are fetched one batch ahead
  int32_t phys_cur = lane < my_tiles ? bt_row[page_of(lane)] : 0;
  int32_t phys_nxt = 32 + lane < my_tiles ? bt_row[page_of(32 + lane)] : 0;
  uint32_t bad_slots = 0;  // bit s: the tile now in ring stage s maps to no page
  auto issue_tile = [&](int ki) {
    if (ki != 0 && (ki & 31) == 0) {
      phys_cur = phys_nxt;
      phys_nxt = ki + 32 + lane < my_tiles ? bt_row[page_of(ki + 32 + lane)] : 0;
    }
    uint32_t phys = static_cast<uint32_t>(__shfl_sync(0xffffffffu, phys_cur, ki & 31));
    const int stage = ki % STAGES;
    const int slot = warp * STAGES + stage;
    const bool bad = phys >= num_pages_u;  // also catches negative ids
    bad_slots = bad ? (bad_slots | (1u << stage)) : (bad_slots & ~(1u << stage));
    if (bad) phys = 0;
    const uint32_t sub = (warp + ki * NW) & (tiles_per_page - 1);
    const uint32_t full = L::kFullBar + 8 * slot;
    if (lane == 0 && !(nocopy && ki >= STAGES)) mbar_arrive_expect_tx(full, 2560);
    __syncwarp();
    if (lane < n_chunks && !(nocopy && ki >= STAGES))
      bulk_copy_g2s(slot_addr(slot) + ch_dst, src_base + phys * page_bytes + sub * ch_sub, ch_bytes, full);
  };
  for (int ki = 0; ki < min(my_tiles, STAGES); ++ki) issue_tile(ki);

  {  // level tables -> fp16 in shared memory
    __half* lv = reinterpret_cast<__half*>(gptr(L::kLevels));
    for (int i = tid; i < 128; i += NW * 32) {
      const int which = i >> 6, g = (i >> 4) & 3, c = i & 15;
      lv[i] = __float2half_rn(which ? load_v_level(p, head, g, c) : load_k_level(p, head, g, c));
    }
  }
  __syncthreads();
  {  // byte -> (level[low nibble], level[high nibble]) tables, one copy per bank.
     // Block P (P = 0, 1) holds, in bank l, the K table of group 2*((l>>1)&1)+P and the
     // V table of group 2*(l>>4)+P: the groups lane l needs when an MMA works on pair P.
    const unsigned short* lv = reinterpret_cast<const unsigned short*>(gptr(L::kLevels));
    for (int e = warp; e < 512; e += NW) {
      const int P = e >> 8, byte = e & 255;
      const int kg = 2 * ((lane >> 1) & 1) + P, vg = 2 * (lane >> 4) + P;
      const uint32_t kval = lv[kg * 16 + (byte & 15)] | (static_cast<uint32_t>(lv[kg * 16 + (byte >> 4)]) << 16);
      const uint32_t vval = lv[64 + vg * 16 + (byte & 15)] | (static_cast<uint32_t>(lv[64 + vg * 16 + (byte >> 4)]) << 16);
      uint32_t* row = reinterpret_cast<uint32_t*>(gptr(kLutAddr + P * kLutBlock + byte * 256));
      row[lane] = kval;
      row[32 + lane] = vval;
    }
  }

  // ---- per-lane roles ---------------------------------------------------------------------
  // QK (S[token, (head, group)] = Lk[token, d] * Qblock[d, (head, group)], pair P at a time):
  //   A rows gid / gid+8 are tokens tq0 / tq1; this lane's k-slots carry half `khalf` of group 2*ksel+P.
  //   B column gid is (head gid&3, group 2*(gid>>2)+P); C columns 2tig, 2tig+1 are heads hA, hA+1 of group 2*ksel+P.
  const int ksel = tig >> 1, khalf = tig & 1;
  const int hA = (2 * tig) & 3;
  const int prow = (kRowSlot >> (4 * gid)) & 15;  // k-slot of the PV stage that A row gid corresponds to
  const int tq0 = static_cast<int>((kTokOfSlot >> (4 * prow)) & 15), tq1 = static_cast<int>((kTokOfSlot >> (4 * (prow + 8))) & 15);
  auto code_off = [](int t) { return t * 64 + (t >= 8 ? kCodeSkew : 0); };
  const uint32_t kc_off0 = kOffKLo + code_off(tq0) + (2 * ksel) * 16 + khalf * 8;  // pair 1: +16
  const uint32_t kc_off1 = kOffKLo + code_off(tq1) + (2 * ksel) * 16 + khalf * 8;
  const uint32_t ks_off0 = kOffKStat + tq0 * 16 + ksel * 8, ks_off1 = kOffKStat + tq1 * 16 + ksel * 8;
  // PV (O[d, (head, group)] = Lv^T[d, token] * W[token, (head, group)], pair P at a time):
  //   A rows gid / gid+8 are d's of group 2*vsel+P; k-slots 2tig, 2tig+1 (+8) are tokens tk[o][0..1];
  //   B column gid is (head gid&3, group 2*vsel+P).
  const int vsel = gid >> 2, vu = gid & 3;
  int tk[2][2];
#pragma unroll
  for (int o = 0; o < 2; ++o)
#pragma unroll
    for (int e = 0; e < 2; ++e) tk[o][e] = static_cast<int>((kTokOfSlot >> (4 * (2 * tig + e + 8 * o))) & 15);
  uint32_t vc_off[2][2], vs_off[2];
#pragma unroll
  for (int o = 0; o < 2; ++o) {
#pragma unroll
    for (int e = 0; e < 2; ++e) vc_off[o][e] = kOffVLo + code_off(tk[o][e]) + (2 * vsel) * 16 + (vu >> 1) * 8;  // pair 1: +16
    vs_off[o] = kOffVStat + ((2 * vsel) * kTile + min(tk[o][0], tk[o][1])) * 4;                                  // pair 1: +64
  }
  const bool pair_swapped = tk[0][0] > tk[0][1];  // odd tig: the pair sits in memory as (second, first)
  const uint32_t sel_scale = pair_swapped ? 0x1054u : 0x5410u, sel_min = pair_swapped ? 0x3276u : 0x7632u;
  const int sh0 = 4 * (vu & 1), sh1 = 4 - sh0;
  const uint32_t klane0 = kLutAddr | (lane * 4), klane1 = klane0 + kLutBlock;
  const uint32_t vlane0 = kLutAddr | (lane * 4 + 128), vlane1 = vlane0 + kLutBlock;
  // probabilities travel from the QK layout (token by gid, head by tig) to the PV layout (token by tig, head by gid)
  const int hsrc = gid & 3;  // head of this lane's W column
  const int src_tig = (hsrc >> 1) | ((hsrc & 1) << 1);
  const int src_lane0 = ((kRowSlot >> (4 * (2 * tig))) & 15) * 4 + src_tig;      // row holding k-slots 2tig, 2tig+8
  const int src_lane1 = ((kRowSlot >> (4 * (2 * tig + 1))) & 15) * 4 + src_tig;  // row holding k-slots 2tig+1, 2tig+9

  // ---- query fragments (B operand of QK), pre-scaled by softmax_scale * log2(e) ------------
  uint32_t qb[2][4][2];
  float qs[2][2];  // sum over d of the rounded q for (head hA+e, group 2*ksel+P)
  {
    const int hq = gid & 3;
    const bool live = hq < nh && ksel == (gid >> 2);
    const int64_t qoff = static_cast<int64_t>(b) * p.q_batch_stride + static_cast<int64_t>(hq0 + hq) * kHeadDim;
    float part[2] = {0.f, 0.f};
#pragma unroll
    for (int P = 0; P < 2; ++P)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int d0 = 32 * (2 * ksel + P) + 16 * khalf + 4 * j;
        float f[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = live ? load_q(p.q, qoff + d0 + i, p.q_dtype) * p.scale_log2 : 0.f;
        const uint32_t lo2 = pack_half2(f[0], f[1]), hi2 = pack_half2(f[2], f[3]);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo2));
        const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&hi2));
        part[P] += (a.x + a.y) + (c.x + c.y);
        qb[P][j][0] = lo2;
        qb[P][j][1] = hi2;
      }
#pragma unroll
    for (int P = 0; P < 2; ++P) {
      part[P] += __shfl_xor_sync(0xffffffffu, part[P], 1);  // both halves of the group
#pragma unroll
      for (int e = 0; e < 2; ++e) qs[e][P] = __shfl_sync(0xffffffffu, part[P], (ksel * 4 + hA + e) * 4 + tig);
    }
  }
  __syncthreads();  // tables complete

  float oacc[2][4][4];
  float cmin[2][4];
#pragma unroll
  for (int P = 0; P < 2; ++P) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) oacc[P][i][c] = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) cmin[P][c] = 0.f;
  }
  float m_used[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.f, 0.f};  // heads hA, hA+1

  // ---- main loop: two ring tiles (32 tokens) per iteration -------------------------------
  auto wait_tile = [&](int k) -> bool {  // false: the bounded wait gave up
    const int use = k / STAGES, stage = k - use * STAGES;
    if ((noload || nowait) && use > 0) return true;
    const uint32_t full = L::kFullBar + 8 * (warp * STAGES + stage);
    WaitBudget budget;
    while (!mbar_try_wait(full, use & 1)) {
      if (__any_sync(0xffffffffu, budget.expired())) {
        atomicExch(&g_decode_status, 2);
        return false;
      }
    }
    return true;
  };
  auto tile_len = [&](int k) -> int {  // valid tokens of ring tile k (0: none / unmapped page)
    if (k >= my_tiles) return 0;
    const int j = warp + k * NW;
    const int tok0 = (page_lo + split + S * (j >> log2r)) * BS + (j & (tiles_per_page - 1)) * kTile;
    return (bad_slots >> (k % STAGES)) & 1 ? 0 : min(kTile, hi - tok0);
  };

  // timing ablations (ABL): bit 0 drops the MMAs, bit 1 replaces table look-ups by their address
#define BKV_MMA(c, a0, a1, a2, a3, b0, b1)                                                      \
  do {                                                                                          \
    if (ABL & 1) {                                                                              \
      asm volatile("" ::"r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));                  \
    } else {                                                                                    \
      mma16816(c, a0, a1, a2, a3, b0, b1);                                                      \
    }                                                                                           \
  } while (0)
#define BKV_LUT(a) ((ABL & 2) ? (a) : lut_load(a))
  auto process_pair = [&](auto partial_tag, const uint32_t sbA, const uint32_t sbB, const int nvA, const int nvB) {
    constexpr bool PARTIAL = decltype(partial_tag)::value;
    const uint32_t sb[2] = {sbA, sbB};
    const int nv[2] = {nvA, nvB};
    // ------------------------------ S = Lk * Qblock (one accumulator per tile and pair) ------
    float sacc[2][2][4] = {};
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int P = 0; P < 2; ++P) {
        const uint2 k0 = P ? ring_load64<16>(sb[t] + kc_off0) : ring_load64<0>(sb[t] + kc_off0);
        const uint2 k1 = P ? ring_load64<16>(sb[t] + kc_off1) : ring_load64<0>(sb[t] + kc_off1);
        const uint32_t w0[2] = {k0.x, k0.y}, w1[2] = {k1.x, k1.y};
        const uint32_t kl = P ? klane1 : klane0;
        uint32_t av[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          av[j][0] = BKV_LUT(__byte_perm(w0[j >> 1], kl, (j & 1) ? 0x7624 : 0x7604));
          av[j][1] = BKV_LUT(__byte_perm(w1[j >> 1], kl, (j & 1) ? 0x7624 : 0x7604));
          av[j][2] = BKV_LUT(__byte_perm(w0[j >> 1], kl, (j & 1) ? 0x7634 : 0x7614));
          av[j][3] = BKV_LUT(__byte_perm(w1[j >> 1], kl, (j & 1) ? 0x7634 : 0x7614));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          BKV_MMA(sacc[t][P], av[j][0], av[j][1], av[j][2], av[j][3], qb[P][j][0], qb[P][j][1]);
      }
    // ------------------------------ V index bytes (token pair -> one table index) -----------
    // Independent of the softmax below, so issued here to overlap with its latency.
    uint32_t vidx[2][2][2][2];  // [tile][pair][token pair][word: row gid / row gid+8]
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int P = 0; P < 2; ++P)
#pragma unroll
        for (int o = 0; o < 2; ++o) {
          const uint2 xf = P ? ring_load64<16>(sb[t] + vc_off[o][0]) : ring_load64<0>(sb[t] + vc_off[o][0]);
          const uint2 xs = P ? ring_load64<16>(sb[t] + vc_off[o][1]) : ring_load64<0>(sb[t] + vc_off[o][1]);
          vidx[t][P][o][0] = ((xf.x >> sh0) & 0x0F0F0F0Fu) | ((xs.x << sh1) & 0xF0F0F0F0u);
          vidx[t][P][o][1] = ((xf.y >> sh0) & 0x0F0F0F0Fu) | ((xs.y << sh1) & 0xF0F0F0F0u);
        }
    // ------------------------------ scores: tokens tq0, tq1 x heads hA, hA+1 ----------------
    float s[2][2][2];  // [tile][row][head]
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const uint2 st = ring_load64<0>(sb[t] + (r ? ks_off1 : ks_off0));  // groups 2*ksel, 2*ksel+1
        const float2 g0 = stat_word_to_f32<STAT_BF16>(st.x), g1 = stat_word_to_f32<STAT_BF16>(st.y);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float v = g0.x * sacc[t][0][2 * r + e];
          v = fmaf(g0.y, qs[e][0], v);
          v = fmaf(g1.x, sacc[t][1][2 * r + e], v);
          v = fmaf(g1.y, qs[e][1], v);
          v += __shfl_xor_sync(0xffffffffu, v, 2);  // the other two groups
          if (PARTIAL) {                            // behind the end of the sequence (statistics may be NaN)
            if ((r ? tq1 : tq0) >= nv[t]) v = -CUDART_INF_F;
          }
          s[t][r][e] = v;
        }
      }
    // ------------------------------ online softmax over the 32 tokens -----------------------
    float tmax[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float m = fmaxf(fmaxf(s[0][0][e], s[0][1][e]), fmaxf(s[1][0][e], s[1][1][e]));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
      tmax[e] = m;
    }
    const bool need0 = tmax[0] > m_used[0] + kRescaleThreshold, need1 = tmax[1] > m_used[1] + kRescaleThreshold;
    if (__any_sync(0xffffffffu, need0 || need1)) {
      float corr[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float m_new = (e ? need1 : need0) ? tmax[e] : m_used[e];
        corr[e] = (m_new == -CUDART_INF_F) ? 1.f : fast_exp2(m_used[e] - m_new);
        m_used[e] = m_new;
        l_run[e] *= corr[e];
      }
#pragma unroll
      for (int P = 0; P < 2; ++P) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          oacc[P][i][0] *= corr[0];
          oacc[P][i][1] *= corr[1];
          oacc[P][i][2] *= corr[0];
          oacc[P][i][3] *= corr[1];
        }
        cmin[P][0] *= corr[0];
        cmin[P][1] *= corr[1];
        cmin[P][2] *= corr[0];
        cmin[P][3] *= corr[1];
      }
    }
    uint32_t ph[2][2];  // [tile][token pair]: probabilities of this lane's W column head, tokens tk[o][0..1]
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      float pe[2][2];
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          pe[r][e] = fast_exp2(s[t][r][e] - m_used[e]);
          l_run[e] += pe[r][e];
        }
      // this lane serves head hA + ksel to the PV layout: (token tq0, token tq1) packed
      const uint32_t mine = ksel ? pack_half2(pe[0][1], pe[1][1]) : pack_half2(pe[0][0], pe[1][0]);
      const uint32_t fromA = __shfl_sync(0xffffffffu, mine, src_lane0);  // tokens of k-slots 2tig, 2tig+8
      const uint32_t fromB = __shfl_sync(0xffffffffu, mine, src_lane1);  // tokens of k-slots 2tig+1, 2tig+9
      ph[t][0] = __byte_perm(fromA, fromB, 0x5410);
      ph[t][1] = __byte_perm(fromA, fromB, 0x7632);
    }
    // ------------------------------ per tile: W = p*scale_v, p*min_v, then O += Lv^T * W ----
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int P = 0; P < 2; ++P) {
        uint32_t wb[2], mb[2];
#pragma unroll
        for (int o = 0; o < 2; ++o) {
          const uint2 vs = P ? ring_load64<kTile * 4>(sb[t] + vs_off[o]) : ring_load64<0>(sb[t] + vs_off[o]);
          uint32_t sc2, mn2;
          if (STAT_BF16) {
            const uint32_t first = pair_swapped ? vs.y : vs.x, second = pair_swapped ? vs.x : vs.y;
            sc2 = pack_half2(__uint_as_float(first << 16), __uint_as_float(second << 16));
            mn2 = pack_half2(__uint_as_float(first & 0xFFFF0000u), __uint_as_float(second & 0xFFFF0000u));
          } else {
            sc2 = __byte_perm(vs.x, vs.y, sel_scale);
            mn2 = __byte_perm(vs.x, vs.y, sel_min);
          }
          uint32_t wv = hmul2_u32(ph[t][o], sc2), mv = hmul2_u32(ph[t][o], mn2);
          if (PARTIAL) {  // 0 * NaN would poison the accumulators
            const uint32_t keep = (tk[o][0] < nv[t] ? 0x0000FFFFu : 0u) | (tk[o][1] < nv[t] ? 0xFFFF0000u : 0u);
            wv &= keep;
            mv &= keep;
          }
          wb[o] = wv;
          mb[o] = mv;
        }
        const uint32_t vl = P ? vlane1 : vlane0;
        uint32_t av[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t sel = i == 0 ? 0x7604 : i == 1 ? 0x7614 : i == 2 ? 0x7624 : 0x7634;
          av[i][0] = BKV_LUT(__byte_perm(vidx[t][P][0][0], vl, sel));
          av[i][1] = BKV_LUT(__byte_perm(vidx[t][P][0][1], vl, sel));
          av[i][2] = BKV_LUT(__byte_perm(vidx[t][P][1][0], vl, sel));
          av[i][3] = BKV_LUT(__byte_perm(vidx[t][P][1][1], vl, sel));
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) BKV_MMA(oacc[P][i], av[i][0], av[i][1], av[i][2], av[i][3], wb[0], wb[1]);
        const uint32_t ones = 0x3C003C00u;
        BKV_MMA(cmin[P], ones, ones, ones, ones, mb[0], mb[1]);
      }
  };

  for (int k = 0; k < my_tiles; k += 2) {
    if (!wait_tile(k)) break;
    const bool has_b = k + 1 < my_tiles;
    if (has_b && !wait_tile(k + 1)) break;
    const int nvA = tile_len(k), nvB = tile_len(k + 1);
    const uint32_t sbA = slot_addr(warp * STAGES + k % STAGES);
    const uint32_t sbB = slot_addr(warp * STAGES + (k + 1) % STAGES);
    if (nvA == kTile && nvB == kTile) process_pair(std::false_type{}, sbA, sbB, nvA, nvB);
    else if (nvA > 0 || nvB > 0) process_pair(std::true_type{}, sbA, sbB, nvA, nvB);
    // both stages are free again: refill them with the tiles STAGES ahead
    if (!noload && k + STAGES < my_tiles) {
      __syncwarp();
      fence_proxy_async();
      issue_tile(k + STAGES);
      if (k + 1 + STAGES < my_tiles) issue_tile(k + 1 + STAGES);
    }
  }
#undef BKV_MMA
#undef BKV_LUT

  // ---- epilogue: warp partials -> shared memory -> CTA result ---------------------------
#pragma unroll
  for (int e = 0; e < 2; ++e) {  // tokens were spread over gid
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 4);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 8);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 16);
  }
  __syncthreads();  // every tile of every warp has been consumed: the ring is free
  float* mo = reinterpret_cast<float*>(gptr(L::kMergeO));
  float* mm = reinterpret_cast<float*>(gptr(L::kMergeM));
  float* ml = reinterpret_cast<float*>(gptr(L::kMergeL));
  if (ksel == vsel) {  // accumulator columns of this lane match the group of its rows
    float* base0 = mo + (warp * 4 + hA) * kHeadDim;
    float* base1 = base0 + kHeadDim;
#pragma unroll
    for (int P = 0; P < 2; ++P)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int d0 = 32 * (2 * vsel + P) + 16 * (vu >> 1) + 2 * i + (vu & 1);
        base0[d0] = oacc[P][i][0] + cmin[P][0];
        base1[d0] = oacc[P][i][1] + cmin[P][1];
        base0[d0 + 8] = oacc[P][i][2] + cmin[P][0];
        base1[d0 + 8] = oacc[P][i][3] + cmin[P][1];
      }
  }
  if (gid == 0 && ksel == 0) {  // tig 0 holds heads 0,1; tig 1 holds heads 2,3
    mm[warp * 4 + hA] = m_used[0];
    mm[warp * 4 + hA + 1] = m_used[1];
    ml[warp * 4 + hA] = l_run[0];
    ml[warp * 4 + hA + 1] = l_run[1];
  }
  __syncthreads();
  const bool direct = S == 1 && !p.force_partial;
  for (int idx = tid; idx < 4 * kHeadDim; idx += NW * 32) {
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

template <int NW, int STAGES, int ABL = 0>
int launch_variant(const DecodeParams& p, cudaStream_t stream) {
  using L = Smem<NW, STAGES>;
  const int gqa = p.heads_q / p.heads_kv;
  const int quads = gqa == 8 ? 2 : 1;
  const dim3 grid(p.num_splits, p.heads_kv * quads, p.batch);
  const dim3 block(NW * 32);
  auto kern = p.stat_bf16 ? decode_mma_kernel<NW, STAGES, true, ABL> : decode_mma_kernel<NW, STAGES, false, ABL>;
  static bool configured[2][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[p.stat_bf16 ? 1 : 0][dev]) {
    int reserved = 0;
    cudaDeviceGetAttribute(&reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev);
    if (reserved != static_cast<int>(kSmemBase)) return BKV_ERR_UNSUPPORTED;
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynBytes);
    if (e != cudaSuccess) {
      set_last_cuda_error(e, "cudaFuncSetAttribute(decode_mma_kernel)");
      return BKV_ERR_CUDA;
    }
    configured[p.stat_bf16 ? 1 : 0][dev] = true;
  }
  kern<<<grid, block, L::kDynBytes, stream>>>(p, quads);
  return check_launch("bkv_decode_sm100(mma)");
}

}  // namespace

int launch_decode_mma(const DecodeParams& p, cudaStream_t stream, int config) {
  const int r = p.block_size / kTile;
  if (p.block_size % kTile != 0 || (r & (r - 1)) != 0 || p.block_size > 1024) return BKV_ERR_UNSUPPORTED;
  if ((p.page_stride * 4) % 16 != 0 || !aligned16(p.cache)) return BKV_ERR_UNSUPPORTED;
  if (p.token_lo % p.block_size != 0) return BKV_ERR_UNSUPPORTED;
  switch (config) {
    case 1: return launch_variant<8, 4>(p, stream);
    case 2: return launch_variant<12, 3>(p, stream);
    case 3: return launch_variant<16, 2>(p, stream);
    case 4: return launch_variant<9, 4>(p, stream);
    case 10: return launch_variant<12, 3, 1>(p, stream);
    case 11: return launch_variant<12, 3, 2>(p, stream);
    default: return launch_variant<12, 3>(p, stream);
  }
}

int read_decode_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(int));
  const int zero = 0;
  cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int));
  return v;
}

}  // namespace bkv
