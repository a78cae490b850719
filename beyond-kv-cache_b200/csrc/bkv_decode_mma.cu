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
// The byte table is replicated so that lane l only ever reads shared-memory bank l
// (bank l holds a copy of the table of K group l%4, and of V group l/8): every table
// look-up is conflict-free.  MMA fragments are laid out so that each lane only needs
// levels of "its" group:
//   QK : S^T[(h,g), token] = Q_blockdiag[(h,g), d] * Lk[d, token]   (k-slots of lane tig belong to group tig)
//   PV : O[d, (h,g')]      = Lv^T[d, token] * (p*scale_v)[token, (h,g')]   (rows of lane gid belong to group gid/2)
// Products whose row group and column group differ are computed and discarded.
//
// The table sits at the fixed shared-memory address 0x10000, so a look-up address is a
// single byte-permute of (code word, lane constant) with no addition.  Tokens of a tile
// are assigned to MMA columns / k-slots through a fixed permutation (kTok0 / kTok1) that
// makes every 128-bit code load of a quarter-warp hit eight distinct bank groups.
#include <math_constants.h>

#include <type_traits>

#include "bkv_decode_common.cuh"

namespace bkv {

__device__ int g_decode_status = 0;  // non-zero: 1/2 a bounded wait gave up, 3 unexpected smem base

namespace {

constexpr int kTile = 16;
constexpr int kTileBytes = 2592;
constexpr int kOffKCode = 0;
constexpr int kOffKStat = 1024;
constexpr int kOffVCode = 1280;   // tokens 0-7; tokens 8-15 start 32 bytes later than contiguous
constexpr int kVCodeSkew = 32;
constexpr int kOffVStat = 2336;
constexpr uint32_t kSmemBase = 0x400;   // dynamic shared memory starts after the 1 KB the system reserves
constexpr uint32_t kLutAddr = 0x10000;  // 64 KB table, 64 KB aligned: address = 0x10000 | byte << 8 | slot
constexpr uint32_t kRingHi = 0x20000;
constexpr int kCtrlBytes = 2048;        // barriers, tile lengths, fp16 level tables
constexpr uint32_t kRingLo = kSmemBase + kCtrlBytes;
constexpr int kLoSlots = (kLutAddr - kRingLo) / kTileBytes;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // a wait that lasts 2 s gives up
constexpr float kRescaleThreshold = 8.f;                     // log2 units: p stays below 2^8
// token held by MMA column / k-slot n of the first (kTok0) and second (kTok1) half of a tile
constexpr uint32_t kTok0 = 0xEFDC2310u;  // 0,1,3,2,12,13,15,14
constexpr uint32_t kTok1 = 0x6754AB98u;  // 8,9,11,10,4,5,7,6

constexpr int BKV_FLAG_DEBUG_NOLOAD = 0x100;  // timing experiment: reuse the first ring fill
constexpr int BKV_FLAG_DEBUG_NOCOPY = 0x400;  // timing experiment: run the issue logic without the copies
constexpr int BKV_FLAG_DEBUG_NOWAIT = 0x200;  // timing experiment: issue loads but never wait for them

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
// Bounded wait bookkeeping: true once kWaitLimitNs have passed since the first failed
// poll (the clock is only read every 256 polls).
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
__device__ __forceinline__ float fast_exp2(float x) {  // ex2.approx: 2 ulp, exp2(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void mma16816_zero(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {  // c = a*b (no accumulator input)
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// Table look-up: the address is complete, no base is added.  Not volatile: the table is
// constant once built, so the compiler may schedule these freely.
__device__ __forceinline__ uint32_t lut_load(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
// Ring loads are volatile: they stay, in program order, between the full-barrier wait of
// their tile and the bulk copies that later refill the same ring stage.
__device__ __forceinline__ uint4 ring_load128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
template <int IMM>
__device__ __forceinline__ uint2 ring_load64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.b32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(IMM));
  return v;
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
template <bool BF16>
__device__ __forceinline__ float2 stat_word_to_f32(uint32_t w) {  // (scale, minimum)
  if (BF16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
__device__ __forceinline__ uint32_t slot_addr(int slot) {
  return slot < kLoSlots ? kRingLo + slot * kTileBytes : kRingHi + (slot - kLoSlots) * kTileBytes;
}

template <int NW, int STAGES>
struct Smem {
  static constexpr int kSlots = NW * STAGES;
  static_assert(kSlots <= 64, "control block holds at most 64 ring slots");
  static constexpr uint32_t kFullBar = kSmemBase;        // 8 B each
  static constexpr uint32_t kLevels = kSmemBase + 1280;  // fp16 [K|V][4][16]
  static constexpr int kMergeBytes = NW * 4 * kHeadDim * 4 + NW * 4 * 4 * 2;
  static constexpr int kHiSlots = kSlots > kLoSlots ? kSlots - kLoSlots : 0;
  static constexpr int kHiBytes = kHiSlots * kTileBytes > kMergeBytes ? kHiSlots * kTileBytes : kMergeBytes;
  static constexpr int kDynBytes = static_cast<int>(kRingHi - kSmemBase) + kHiBytes;
  static_assert(kDynBytes <= 232448, "exceeds the 227 KB a CTA can opt into");
  // epilogue overlay in the high region (all ring traffic has drained by then)
  static constexpr uint32_t kMergeO = kRingHi;
  static constexpr uint32_t kMergeM = kMergeO + NW * 4 * kHeadDim * 4;
  static constexpr uint32_t kMergeL = kMergeM + NW * 4 * 4;
};

// registers a thread may use when one CTA of NW warps owns the SM (64 K registers, allocated in eights)
constexpr int max_regs_for(int nw) {
  // the register file is split over the four schedulers (16 K registers each) and a CTA's
  // warps are dealt to them round-robin
  const int per_thread = 16384 / (((nw + 3) / 4) * 32) / 8 * 8;
  return per_thread > 255 ? 255 : per_thread;
}

template <int NW, int STAGES, bool STAT_BF16, int ABL = 0>
__global__ void __maxnreg__(max_regs_for(NW)) decode_mma_kernel(const DecodeParams p, const int quads) {
  using L = Smem<NW, STAGES>;
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t smem_base = smem_u32(smem);
  if (smem_base != kSmemBase) {  // the fixed-address table needs the documented layout
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
  // chunks: 0 K codes (1024 B), 1 K statistics (256), 2/3 V codes of tokens 0-7 / 8-15 (512 each),
  // then V statistics: one 256 B chunk for 16-token pages, else one 64 B chunk per group.
  const PageGeom geo = make_geom(BS, p.heads_kv);
  const int n_chunks = tiles_per_page == 1 ? 5 : 8;
  uint32_t ch_src = 0, ch_sub = 0, ch_dst = 0, ch_bytes = 0;
  {
    const uint32_t code_head = head * (BS * kWordsPerHead) * 4;
    if (lane == 0) { ch_src = geo.k_code_off * 4 + code_head; ch_sub = 1024; ch_dst = kOffKCode; ch_bytes = 1024; }
    if (lane == 1) { ch_src = (geo.k_stat_off + head * (BS * 4)) * 4; ch_sub = 256; ch_dst = kOffKStat; ch_bytes = 256; }
    if (lane == 2) { ch_src = geo.v_code_off * 4 + code_head; ch_sub = 1024; ch_dst = kOffVCode; ch_bytes = 512; }
    if (lane == 3) { ch_src = geo.v_code_off * 4 + code_head + 512; ch_sub = 1024; ch_dst = kOffVCode + 512 + kVCodeSkew; ch_bytes = 512; }
    if (lane >= 4 && lane < n_chunks) {
      const int gg = lane - 4;
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
  {
    const int first = noload ? min(my_tiles, STAGES) : min(my_tiles, STAGES);
    for (int ki = 0; ki < first; ++ki) issue_tile(ki);
  }

  {  // level tables -> fp16 in shared memory
    __half* lv = reinterpret_cast<__half*>(gptr(L::kLevels));
    for (int i = tid; i < 128; i += NW * 32) {
      const int which = i >> 6, g = (i >> 4) & 3, c = i & 15;
      lv[i] = __float2half_rn(which ? load_v_level(p, head, g, c) : load_k_level(p, head, g, c));
    }
  }
  __syncthreads();
  {  // byte -> (level[low nibble], level[high nibble]) table, one copy per bank
    const unsigned short* lv = reinterpret_cast<const unsigned short*>(gptr(L::kLevels));
    const int kg = lane & 3, vg = lane >> 3;
    for (int e = warp; e < 256; e += NW) {
      const uint32_t kval = lv[kg * 16 + (e & 15)] | (static_cast<uint32_t>(lv[kg * 16 + (e >> 4)]) << 16);
      const uint32_t vval = lv[64 + vg * 16 + (e & 15)] | (static_cast<uint32_t>(lv[64 + vg * 16 + (e >> 4)]) << 16);
      uint32_t* row = reinterpret_cast<uint32_t*>(gptr(kLutAddr + e * 256));
      row[lane] = kval;
      row[32 + lane] = vval;
    }
  }

  // ---- query fragments (A operand of QK), pre-scaled by softmax_scale * log2(e) --------
  const int hsel = gid & 3;         // query head of this lane's scores / B columns
  const int grow = 2 * (gid >> 2);  // K group of MMA row gid (row gid+8 is group grow+1)
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
  __syncthreads();  // table complete

  // ---- per-lane constants ---------------------------------------------------------------
  const int gv = gid >> 1, vu = gid & 1;  // V group / nibble parity of this lane's MMA rows
  const uint32_t klane = kLutAddr | (lane * 4), vlane = kLutAddr | (lane * 4 + 128);
  // token whose K codes this lane feeds into column gid of the two QK halves
  const int kprov0 = (kTok0 >> (4 * gid)) & 15, kprov1 = (kTok1 >> (4 * gid)) & 15;
  const uint32_t kc_off0 = kOffKCode + kprov0 * 64 + tig * 16, kc_off1 = kOffKCode + kprov1 * 64 + tig * 16;
  // tokens of this lane's columns / k-slots 2tig, 2tig+1 in the two halves
  int tk[2][2];
  tk[0][0] = (kTok0 >> (8 * tig)) & 15;
  tk[0][1] = (kTok0 >> (8 * tig + 4)) & 15;
  tk[1][0] = (kTok1 >> (8 * tig)) & 15;
  tk[1][1] = (kTok1 >> (8 * tig + 4)) & 15;
  uint32_t ks_off[2][2], vc_off[2][2], vs_off[2];
#pragma unroll
  for (int o = 0; o < 2; ++o) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      ks_off[o][e] = kOffKStat + tk[o][e] * 16 + grow * 4;
      vc_off[o][e] = kOffVCode + tk[o][e] * 64 + (tk[o][e] >= 8 ? kVCodeSkew : 0) + gv * 16;
    }
    vs_off[o] = kOffVStat + ((gid >> 2) * kTile + min(tk[o][0], tk[o][1])) * 4;
  }
  const bool pair_swapped = tk[0][0] > tk[0][1];  // odd tig: the pair sits in memory as (second, first)
  const uint32_t sel_scale = pair_swapped ? 0x1054u : 0x5410u, sel_min = pair_swapped ? 0x3276u : 0x7632u;
  const int sh0 = 4 * vu, sh1 = 4 - 4 * vu;

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
#define BKV_MMA(c, a0, a1, a2, a3, b0, b1) \
  do { if (ABL & 1) { asm volatile("" ::"r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1)); } else { mma16816(c, a0, a1, a2, a3, b0, b1); } } while (0)
#define BKV_LUT(a) ((ABL & 2) ? (a) : lut_load(a))
  auto process_pair = [&](auto partial_tag, const uint32_t sbA, const uint32_t sbB, const int nvA, const int nvB) {
    constexpr bool PARTIAL = decltype(partial_tag)::value;
    const uint32_t sb[2] = {sbA, sbB};
    const int nv[2] = {nvA, nvB};
    // ------------------------------ S^T = Q * Lk^T (4 independent accumulator chains) ------
    float sacc[2][2][4] = {};
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int o = 0; o < 2; ++o) {
        const uint4 kw = ring_load128(sb[t] + (o ? kc_off1 : kc_off0));
        const uint32_t w4[4] = {kw.x, kw.y, kw.z, kw.w};
        // all 16 look-up addresses first, then the 16 look-ups, then the 8 dependent MMAs
        uint32_t ad[8][2], bv[8][2];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          ad[jj][0] = __byte_perm(w4[jj >> 1], klane, (jj & 1) ? 0x7624 : 0x7604);
          ad[jj][1] = __byte_perm(w4[jj >> 1], klane, (jj & 1) ? 0x7634 : 0x7614);
        }
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          bv[jj][0] = BKV_LUT(ad[jj][0]);
          bv[jj][1] = BKV_LUT(ad[jj][1]);
        }
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          if (jj == 0 && !(ABL & 1)) mma16816_zero(sacc[t][o], qa[jj][0], qa[jj][1], qa[jj][2], qa[jj][3], bv[jj][0], bv[jj][1]);
          else BKV_MMA(sacc[t][o], qa[jj][0], qa[jj][1], qa[jj][2], qa[jj][3], bv[jj][0], bv[jj][1]);
        }
      }
    // ------------------------------ V index bytes (token pair -> one table index) -----------
    // Independent of the softmax below, so issued here to overlap with its latency.
    uint32_t vidx[2][2][4];
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int o = 0; o < 2; ++o) {
        const uint4 xf = ring_load128(sb[t] + vc_off[o][0]);
        const uint4 xs = ring_load128(sb[t] + vc_off[o][1]);
        vidx[t][o][0] = ((xf.x >> sh0) & 0x0F0F0F0Fu) | ((xs.x << sh1) & 0xF0F0F0F0u);
        vidx[t][o][1] = ((xf.y >> sh0) & 0x0F0F0F0Fu) | ((xs.y << sh1) & 0xF0F0F0F0u);
        vidx[t][o][2] = ((xf.z >> sh0) & 0x0F0F0F0Fu) | ((xs.z << sh1) & 0xF0F0F0F0u);
        vidx[t][o][3] = ((xf.w >> sh0) & 0x0F0F0F0Fu) | ((xs.w << sh1) & 0xF0F0F0F0u);
      }
    // ------------------------------ scores of this lane -------------------------------------
    float s[2][2][2];
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int o = 0; o < 2; ++o) {
        const uint2 st0 = ring_load64<0>(sb[t] + ks_off[o][0]);
        const uint2 st1 = ring_load64<0>(sb[t] + ks_off[o][1]);
        const float2 a0 = stat_word_to_f32<STAT_BF16>(st0.x), b0 = stat_word_to_f32<STAT_BF16>(st0.y);
        const float2 a1 = stat_word_to_f32<STAT_BF16>(st1.x), b1 = stat_word_to_f32<STAT_BF16>(st1.y);
        float p0 = a0.x * sacc[t][o][0];
        p0 = fmaf(a0.y, qs0, p0);
        p0 = fmaf(b0.x, sacc[t][o][2], p0);
        p0 = fmaf(b0.y, qs1, p0);
        float p1 = a1.x * sacc[t][o][1];
        p1 = fmaf(a1.y, qs0, p1);
        p1 = fmaf(b1.x, sacc[t][o][3], p1);
        p1 = fmaf(b1.y, qs1, p1);
        p0 += __shfl_xor_sync(0xffffffffu, p0, 16);
        p1 += __shfl_xor_sync(0xffffffffu, p1, 16);
        if (PARTIAL) {  // tokens behind the end of the sequence (their statistics may be NaN)
          if (tk[o][0] >= nv[t]) p0 = -CUDART_INF_F;
          if (tk[o][1] >= nv[t]) p1 = -CUDART_INF_F;
        }
        s[t][o][0] = p0;
        s[t][o][1] = p1;
      }
    // ------------------------------ online softmax over the 32 tokens -----------------------
    float tmax = fmaxf(fmaxf(fmaxf(s[0][0][0], s[0][0][1]), fmaxf(s[0][1][0], s[0][1][1])),
                       fmaxf(fmaxf(s[1][0][0], s[1][0][1]), fmaxf(s[1][1][0], s[1][1][1])));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
    const bool need = tmax > m_used + kRescaleThreshold;
    if (__any_sync(0xffffffffu, need)) {
      const float m_new = need ? tmax : m_used;
      const float corr = (m_new == -CUDART_INF_F) ? 1.f : fast_exp2(m_used - m_new);
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
    uint32_t ph[2][2];
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int o = 0; o < 2; ++o) {
        const float e0 = fast_exp2(s[t][o][0] - m_used), e1 = fast_exp2(s[t][o][1] - m_used);
        l_run += e0 + e1;
        ph[t][o] = pack_half2(e0, e1);
      }
    // ------------------------------ per tile: W = p*scale_v, p*min_v, then O += Lv^T * W ----
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      uint32_t wb[2][2], mb[2][2];
#pragma unroll
      for (int jn = 0; jn < 2; ++jn)
#pragma unroll
        for (int o = 0; o < 2; ++o) {
          const uint2 vs = jn ? ring_load64<2 * kTile * 4>(sb[t] + vs_off[o]) : ring_load64<0>(sb[t] + vs_off[o]);
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
          wb[jn][o] = wv;
          mb[jn][o] = mv;
        }
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) {
        const uint32_t m0 = vidx[t][0][wi], m1 = vidx[t][1][wi];
        uint32_t aa[8], av[2][4];
        aa[0] = __byte_perm(m0, vlane, 0x7604);
        aa[1] = __byte_perm(m0, vlane, 0x7614);
        aa[2] = __byte_perm(m0, vlane, 0x7624);
        aa[3] = __byte_perm(m0, vlane, 0x7634);
        aa[4] = __byte_perm(m1, vlane, 0x7604);
        aa[5] = __byte_perm(m1, vlane, 0x7614);
        aa[6] = __byte_perm(m1, vlane, 0x7624);
        aa[7] = __byte_perm(m1, vlane, 0x7634);
        av[0][0] = BKV_LUT(aa[0]);
        av[0][1] = BKV_LUT(aa[1]);
        av[1][0] = BKV_LUT(aa[2]);
        av[1][1] = BKV_LUT(aa[3]);
        av[0][2] = BKV_LUT(aa[4]);
        av[0][3] = BKV_LUT(aa[5]);
        av[1][2] = BKV_LUT(aa[6]);
        av[1][3] = BKV_LUT(aa[7]);
#pragma unroll
        for (int e = 0; e < 2; ++e)
#pragma unroll
          for (int jn = 0; jn < 2; ++jn)
            BKV_MMA(oacc[2 * wi + e][jn], av[e][0], av[e][1], av[e][2], av[e][3], wb[jn][0], wb[jn][1]);
      }
      const uint32_t ones = 0x3C003C00u;
#pragma unroll
      for (int jn = 0; jn < 2; ++jn) BKV_MMA(cmin[jn], ones, ones, ones, ones, mb[jn][0], mb[jn][1]);
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

  // ---- epilogue: warp partials -> shared memory -> CTA result ---------------------------
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  __syncthreads();  // every tile of every warp has been consumed: the ring is free
  float* mo = reinterpret_cast<float*>(gptr(L::kMergeO));
  float* mm = reinterpret_cast<float*>(gptr(L::kMergeM));
  float* ml = reinterpret_cast<float*>(gptr(L::kMergeL));
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
    case 2: return launch_variant<8, 6>(p, stream);
    case 3: return launch_variant<12, 5>(p, stream);
    case 4: return launch_variant<16, 3>(p, stream);
    case 5: return launch_variant<12, 4>(p, stream);
    case 10: return launch_variant<8, 4, 1>(p, stream);
    case 11: return launch_variant<8, 4, 2>(p, stream);
    case 12: return launch_variant<8, 4, 3>(p, stream);
    default: return launch_variant<8, 4>(p, stream);
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
