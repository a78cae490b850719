// Persistent, warp-granular form of the tensor-core decode attention over the packed cache.
//
// The (kv-head, request, 16-token tile) space is one long line, head-major.  The grid is one
// CTA per SM; CTA c owns the c-th equal share of the line and every warp of it an equal,
// contiguous share of that.  A warp therefore streams through a run of consecutive tiles that
// may start in the middle of one request and end in the middle of another; the byte tables are
// built once per CTA (twice when its share straddles two heads) instead of once per split.
//
// A warp keeps a private ring of tiles which it fills itself with asynchronous copies (16-byte
// cp.async pieces or tensor copies, see LOADER), running STAGES tiles ahead across request
// boundaries, and a private online-softmax state; no block barrier is executed while it works.
// When it leaves a request it either
//   * owns the whole request: normalises and writes the attention output, or
//   * owns a part of it:      writes an un-normalised partial (o, m, l) into one of the two
//     slots of its range (slot 0: the request began before the range, slot 1: it goes on
//     behind it) together with a header word naming the request.
// The fix-up kernel walks the ranges in order, collects the chain of partials of every
// request that was cut, and merges them by log-sum-exp.  When one request covers a CTA's whole
// share, its warps merge in shared memory first and the CTA leaves a single partial.
//
// Arithmetic and operand layouts (byte tables, group pairs) are those of bkv_decode_mma.cu with
// three changes that remove shuffles, shared-memory traffic and padding:
//   * tokens sit in natural order in the QK rows (row g / g+8 = token g / g+8) and as
//     (t, t+4) pairs in the PV k-slots; the ring slot is swizzled instead of padded;
//   * MMA column n stands for (query head n/2, group n%2 of the pair), so a lane's two QK
//     accumulator columns are the two groups of ONE head and its scores need no exchange;
//   * PV row g / g+8 of MMA i hold the even / odd dimension 8*(g%4)+2i(+1) of a group, so
//     a lane reads each V code word exactly once and uses both nibbles of every byte.
#include <math_constants.h>

#include <type_traits>

#include <cuda.h>

#include <mutex>

#include "bkv_decode_common.cuh"
#include "bkv_mma_ptx.cuh"

namespace bkv {

__device__ int g_stream_status = 0;  // non-zero: 2 a bounded wait gave up, 3 unexpected smem base

namespace {

using namespace mma;

constexpr int kMaxBatch = 1024;        // the per-request tile counts of larger batches do not fit in shared memory:
constexpr int kMaxBatchPlanned = 16384;  // a one-CTA kernel then leaves their prefix sums in the workspace
constexpr int kMaxPagesLog2 = 26;  // a page id and the tile's position in its page share one word
// Ring slot of this kernel: K codes, V codes (16 tokens x 64 B each), K statistics (16 tokens x
// 16 B), V statistics (4 groups x 16 tokens x 4 B), all as 64-byte rows.  Inside the slot the
// 16-byte chunk at byte offset o is stored at o ^ (((o >> 7) & 3) << 4): the 64-byte swizzle of
// the tensor copy unit, which the cp.async loader reproduces.  It makes every per-lane load of the
// MMA layouts conflict-free without padding, so one tensor copy moves one part of a tile.
constexpr int kSwKCode = 0;
constexpr int kSwVCode = 1024;
constexpr int kSwKStat = 2048;
constexpr int kSwVStat = 2304;
constexpr int kSlotBytes = 2560;
__host__ __device__ constexpr uint32_t swz(uint32_t off) { return off ^ (((off >> 7) & 3u) << 4); }
constexpr uint32_t kRingLoS = kSmemBase + 2048;  // 512-aligned, like every slot; control data ends at 1536
static_assert(kRingLoS % 512 == 0 && kRingHi % 512 == 0 && kSlotBytes % 512 == 0, "the swizzle follows address bits 7-8");
constexpr int kLoSlotsS = (kLutAddr - kRingLoS) / kSlotBytes;
constexpr uint32_t kPrefixAddr = kSmemEnd - 4224;  // int[kMaxBatch + 1] tiles before request b
constexpr int kHiSlots = (kPrefixAddr - kRingHi) / kSlotBytes;
constexpr uint32_t kFullBar = kSmemBase;          // 8 B each
constexpr uint32_t kChunkTot = kSmemBase + 512;   // int[32] scan scratch
constexpr uint32_t kLevels = kSmemBase + 1280;    // fp16 [K|V][4][16]
constexpr int kHdrNone = -1;

constexpr int BKV_FLAG_DEBUG_NOLOAD = 0x100;  // timing experiment: reuse the first ring fill
constexpr int BKV_FLAG_DEBUG_NOWAIT = 0x200;  // timing experiment (cp.async loader): consume tiles without waiting for them
constexpr int BKV_FLAG_DEBUG_EQUAL_SHARES = 0x800;     // experiment: force equal shares
constexpr int BKV_FLAG_DEBUG_ALIGNED_SHARES = 0x1000;  // experiment: force head-aligned shares

struct StreamParams {
  DecodeParams d;
  float* ws_o;   // [slots][4][128]
  float* ws_m;   // [slots][4]  log2 domain
  float* ws_l;   // [slots][4]
  int* ws_hdr;   // [slots]  (virtual head * batch + request) * 2 + (1: last part), or kHdrNone
  int* ws_prefix;  // [batch + 1] tiles before request b, written by stream_prefix_kernel when batch > kMaxBatch
  int quads;     // query-head quads per kv head
  int aligned;   // 1: every CTA's share lies inside one head (heads get floor or ceil of C / heads CTAs)
  int straddle_tiles;  // equal shares: tiles by which a share that straddles two heads is shortened
  int q_vec;           // 16-bit queries whose rows can be read in 8-byte pieces
};

// one box of the packed cache, seen as [page][64-byte row][64 bytes], into a ring slot
// the V statistics of the four groups of one head for one 16-token tile: the region is seen as
// [page][head*4+group][tile of the page][64 bytes]
__device__ __forceinline__ void tensor_copy_4d(uint32_t dst, const CUtensorMap* map, int tile, int row, int page,
                                               uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(map), "r"(0), "r"(tile), "r"(row), "r"(page), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tensor_copy_3d(uint32_t dst, const CUtensorMap* map, int row, int page, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
      "l"(map), "r"(0), "r"(row), "r"(page), "r"(bar)
      : "memory");
}

template <int NW, int STAGES>
struct Ring {
  static_assert(NW * STAGES <= 64, "control block holds at most 64 barriers");
  static constexpr int kWarpsLo = kLoSlotsS / STAGES;
  static_assert((NW - kWarpsLo) * STAGES <= kHiSlots, "ring does not fit next to the two table blocks");
  static constexpr int kDynBytes = static_cast<int>(kSmemEnd - kSmemBase);
  __device__ static uint32_t base(int warp) {
    return warp < kWarpsLo ? kRingLoS + warp * (STAGES * kSlotBytes)
                           : kRingHi + (warp - kWarpsLo) * (STAGES * kSlotBytes);
  }
};

// LOADER 1: every lane moves 16-byte pieces with cp.async, one commit group per tile.
// LOADER 3: an elected lane issues one tensor copy (cp.async.bulk.tensor) per part of a tile,
// completing on one mbarrier per ring stage; the copies bypass the load/store pipe.
template <int NW, int STAGES, bool STAT_BF16, int LOADER, int PAIR = 2>
__global__ void __maxnreg__(max_regs_for(NW))
    decode_stream_kernel(const StreamParams sp, const __grid_constant__ CUtensorMap map16,
                         const __grid_constant__ CUtensorMap map4, const __grid_constant__ CUtensorMap mapvs) {
  static_assert(STAGES <= 4, "cp_async_wait_pending handles up to three groups in flight");
  using R = Ring<NW, STAGES>;
  const DecodeParams& p = sp.d;
  extern __shared__ __align__(1024) unsigned char smem[];
  if (smem_u32(smem) != kSmemBase) {  // the fixed-address tables need the documented layout
    if (threadIdx.x == 0) atomicExch(&g_stream_status, 3);
    return;
  }
  auto gptr = [&](uint32_t shared_addr) { return smem + (shared_addr - kSmemBase); };
  constexpr uint32_t kFull = 0xffffffffu;
  const int tid = threadIdx.x, lane = tid & 31;
  // a warp-wide reduction leaves its result in a uniform register, so the compiler knows the
  // warp index (and all the loop state derived from it) to be uniform across the warp
  const int warp = __reduce_max_sync(kFull, tid >> 5);
  const int gid = lane >> 2, tig = lane & 3;
  const int C = gridDim.x, cta = blockIdx.x;
  const int B = p.batch;
  const int quads = sp.quads;
  const int gqa = p.heads_q / p.heads_kv;
  const int BS = p.block_size;
  const int log2r = 31 - __clz(BS / kTile);  // tiles per page is a power of two
  const int tiles_per_page = 1 << log2r;
  const int lo = max(p.token_lo, 0);
  const int page_lo = lo / BS;
  const bool noload = (p.flags & BKV_FLAG_DEBUG_NOLOAD) != 0;
  const bool nowait = (p.flags & BKV_FLAG_DEBUG_NOWAIT) != 0;

  pdl_launch_dependents();  // the fix-up grid may be set up now; it waits for this grid to finish

  if (tid == 0) {
    for (int i = 0; i < NW * STAGES; ++i) mbar_init(kFullBar + 8 * i, 1);
    fence_barrier_init();
  }

  // ---- tiles before every request (exclusive prefix sum over the batch) ------------------
  const bool planned = B > kMaxBatch;
  const int* const prefix = planned ? sp.ws_prefix : reinterpret_cast<const int*>(gptr(kPrefixAddr));
  if (!planned) {
    int* const prefix = reinterpret_cast<int*>(gptr(kPrefixAddr));
    int* tot = reinterpret_cast<int*>(gptr(kChunkTot));
    const int nchunks = (B + 31) >> 5;
    for (int c = warp; c < nchunks; c += NW) {
      const int b = 32 * c + lane;
      int n = 0;
      if (b < B) {
        const int hi_b = min(p.token_hi, p.seq_lens[b]);
        n = hi_b > lo ? (hi_b - lo + kTile - 1) / kTile : 0;
      }
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(kFull, n, o);
        if (lane >= o) n += y;
      }
      if (b < B) prefix[1 + b] = n;
      if (lane == 31) tot[c] = n;
    }
    if (tid == 0) prefix[0] = 0;
    __syncthreads();
    if (warp == 0) {
      const int v = lane < nchunks ? tot[lane] : 0;
      int n = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(kFull, n, o);
        if (lane >= o) n += y;
      }
      tot[lane] = n - v;
    }
    __syncthreads();
    for (int b = tid; b < B; b += NW * 32) prefix[1 + b] += tot[b >> 5];
    __syncthreads();
  }
  const int Tb = prefix[B];  // tiles of one head
  // requests without any position to attend are nobody's tiles: their output rows are zeros
  for (int b = cta; b < B; b += C) {
    if (prefix[b + 1] != prefix[b]) continue;
    const int64_t row0 = static_cast<int64_t>(b) * p.heads_q * kHeadDim;
    for (int i = tid; i < p.heads_q * kHeadDim; i += NW * 32) {
      if (p.force_partial) {
        p.o_partial[row0 + i] = 0.f;
        if ((i & (kHeadDim - 1)) == 0) {
          p.m_partial[(row0 + i) / kHeadDim] = -CUDART_INF_F;
          p.l_partial[(row0 + i) / kHeadDim] = 0.f;
        }
      } else {
        store_out(p.out, row0 + i, p.out_dtype, 0.f);
        if (p.out_f32) p.out_f32[row0 + i] = 0.f;
      }
    }
  }
  const int64_t G = static_cast<int64_t>(p.heads_kv * quads) * Tb;
  int64_t ga, gb;  // this CTA's share of the line
  if (sp.aligned) {
    // heads 0..extra-1 are served by base+1 CTAs, the others by base; no share straddles two
    // heads, so the tables are built once, at the price of unequal shares
    const int hv = p.heads_kv * quads;
    const int base = C / hv, extra = C - base * hv;
    int h, idx, cnt;
    if (cta < extra * (base + 1)) {
      h = cta / (base + 1);
      idx = cta - h * (base + 1);
      cnt = base + 1;
    } else {
      const int c2 = cta - extra * (base + 1);
      h = extra + c2 / base;
      idx = c2 - (c2 / base) * base;
      cnt = base;
    }
    ga = static_cast<int64_t>(h) * Tb + static_cast<int64_t>(Tb) * idx / cnt;
    gb = static_cast<int64_t>(h) * Tb + static_cast<int64_t>(Tb) * (idx + 1) / cnt;
  } else {
    // Equal shares of COST: a CTA whose share straddles two heads builds the tables twice and
    // restarts its pipelines, which is worth `straddle_tiles` tiles.  The cost line is the tile
    // line with a gap of that length at every head boundary; a share that contains a gap is
    // that much shorter in tiles, one that ends inside a gap ends at the head boundary.
    const int hv = p.heads_kv * quads;
    const int64_t gap = sp.straddle_tiles;
    const int64_t L = G + (hv - 1) * gap;
    auto to_tile = [&](int64_t x) {
      int64_t shift = 0;
      for (int h = 1; h < hv; ++h) {
        const int64_t start = static_cast<int64_t>(h) * Tb + (h - 1) * gap;
        if (x >= start + gap) shift += gap;
        else if (x > start) return static_cast<int64_t>(h) * Tb;
        else break;
      }
      return x - shift;
    };
    ga = to_tile(L * cta / C);
    gb = to_tile(L * (cta + 1) / C);
  }

  // ---- per-lane roles (see the file comment) ----------------------------------------------
  const int ksel = tig >> 1, khalf = tig & 1;     // QK: this lane's k-slots carry half khalf of group 2*ksel+P
  const int tq0 = gid;                            // QK rows gid / gid+8 carry tokens gid / gid+8
  const uint32_t kc_off0 = swz(kSwKCode + tq0 * 64 + (2 * ksel) * 16) + khalf * 8;      // pair 0; +512: row gid+8
  const uint32_t kc_off1 = swz(kSwKCode + tq0 * 64 + (2 * ksel + 1) * 16) + khalf * 8;  // pair 1
  const uint32_t ks_off0 = swz(kSwKStat + tq0 * 16), ks_off1 = swz(kSwKStat + (tq0 + 8) * 16);
  const int vsel = gid >> 2, vu = gid & 3;        // PV: rows gid/gid+8 are dims 8*vu+2i(+1) of group 2*vsel+P
  const int hcol = gid >> 1, gsel = gid & 1;      // B column gid: query head hcol, group 2*gsel+P
  // PV k-slots 2tig, 2tig+1 (+8) carry tokens tig, tig+4 (+8): four consecutive tokens per load
  uint32_t vc_off[2][2];                          // [token tig / tig+4][pair]; +512: tokens +8
#pragma unroll
  for (int e = 0; e < 2; ++e)
#pragma unroll
    for (int P = 0; P < 2; ++P) vc_off[e][P] = swz(kSwVCode + (tig + 4 * e) * 64 + (2 * vsel + P) * 16) + vu * 4;
  // V statistic word of (group 2*gsel+P, token tig+4e+8o): +64 for pair 1, +32 for o = 0 (the
  // swizzle of this part flips the bit that o sets)
  const uint32_t vs_off0 = swz(kSwVStat + (2 * gsel) * 64 + (tig + 8) * 4);
  const uint32_t vs_off1 = swz(kSwVStat + (2 * gsel) * 64 + (tig + 4 + 8) * 4);
  const uint32_t klane0 = kLutAddr | (lane * 4), klane1 = klane0 + kLutBlock;
  const uint32_t vlane0 = kLutAddr | (lane * 4 + 128), vlane1 = vlane0 + kLutBlock;
  // probabilities travel from the QK layout (token by gid, head by tig) to the PV layout (token by tig, head by gid)
  const int src_lane0 = tig * 4 + hcol;        // row holding tokens tig, tig+8     (k-slots 2tig, 2tig+8)
  const int src_lane1 = (tig + 4) * 4 + hcol;  // row holding tokens tig+4, tig+12  (k-slots 2tig+1, 2tig+9)

  // ---- ring state of this warp: tile number g of its lifetime lives in stage g % STAGES ----
  const uint32_t ring_base = R::base(warp);
  const uint32_t bar_base = kFullBar + 8 * (warp * STAGES);
  int s = 0;           // stage of the next tile to consume
  uint32_t phase = 0;  // parity of that stage's current use
  int n_issued = 0, n_done = 0;
  uint32_t bad_mask = 0;  // bit s: the tile now in stage s maps to no page
  bool dead = false;      // a bounded wait gave up: stop working, keep walking to the barriers

  const PageGeom geo = make_geom(BS, p.heads_kv);
  const int64_t page_bytes = p.page_stride * 4;
  const uint32_t num_pages_u = static_cast<uint32_t>(p.num_pages);

  auto wait_full = [&](uint32_t bar, uint32_t parity) -> bool {  // false: the bounded wait gave up
    bool ok = mbar_try_wait(bar, parity);
    if (!ok) {
      WaitBudget budget;
      do {
        ok = mbar_try_wait(bar, parity);
      } while (!ok && !budget.expired());
    }
    ok = __all_sync(kFull, ok);
    if (!ok) atomicExch(&g_stream_status, 2);
    return ok;
  };

  // Launched behind a cache writer that lets its dependents start early: everything above read
  // only what older launches produced (sequence lengths); the cache is read from here on.  (In
  // a grid that was launched the ordinary way this returns at once.)
  if (p.flags & BKV_FLAG_PDL_WAIT) pdl_wait();

  for (int ph = 0; ph < 2; ++ph) {
    // ---- the part of this CTA's share that lies in its ph-th head (CTA-uniform) ------------
    int vh = 0, span = 0, first = 0;
    if (Tb > 0 && gb > ga) {
      vh = static_cast<int>(ga / Tb) + ph;
      const int64_t h0 = static_cast<int64_t>(vh) * Tb;
      const int64_t a = max(ga, h0), e = min(gb, h0 + Tb);
      span = e > a ? static_cast<int>(e - a) : 0;
      first = static_cast<int>(a - h0);
    }
    const int range = (cta * 2 + ph) * NW + warp;
    if (lane == 0) {
      sp.ws_hdr[2 * range] = kHdrNone;
      sp.ws_hdr[2 * range + 1] = kHdrNone;
    }
    if (span == 0) continue;
    const int head = vh / quads, quad = vh - head * quads;
    const int hq0 = head * gqa + quad * 4;
    const int nh = min(4, gqa - quad * 4);

    // ---- this warp's run of tiles [wa, wb) inside the head ---------------------------------
    const int wa = first + static_cast<int>(static_cast<int64_t>(span) * warp / NW);
    const int wb = first + static_cast<int>(static_cast<int64_t>(span) * (warp + 1) / NW);
    const int total = wb - wa;
    const bool work = total > 0 && !dead;
    // this head's level tables: requested now, stored to shared memory after the first ring fill
    // has been issued, so the read overlaps the page-id read below
    float level_early = 0.f;
    if (tid < 128) {
      const int which = tid >> 6, g = (tid >> 4) & 3, c = tid & 15;
      level_early = which ? load_v_level(p, head, g, c) : load_k_level(p, head, g, c);
    }

    // cp.async loader: lane l moves the l-th 16 bytes of each 512-byte half of the K and V
    // codes (tokens 0-7 / 8-15); lanes 0-15 move the K statistics, lanes 16-31 the V statistics
    const uint32_t code_head = head * (BS * kWordsPerHead) * 4;
    const uint32_t ld_kcode = geo.k_code_off * 4 + code_head + lane * 16;
    const uint32_t ld_vcode = geo.v_code_off * 4 + code_head + lane * 16;
    const uint32_t ld_code_dst = swz(lane * 16);  // the swizzle repeats every 512 bytes
    uint32_t ld_stat_src, ld_stat_dst, ld_stat_sub;
    if (lane < 16) {
      ld_stat_src = (geo.k_stat_off + head * (BS * 4)) * 4 + lane * 16;
      ld_stat_dst = swz(kSwKStat + lane * 16);
      ld_stat_sub = 256;
    } else {
      const int g = (lane - 16) >> 2, c = (lane - 16) & 3;  // 64 bytes per group and tile
      ld_stat_src = (geo.v_stat_off + head * (4 * BS) + g * BS) * 4 + c * 16;
      ld_stat_dst = swz(kSwVStat + g * 64 + c * 16);
      ld_stat_sub = 64;
    }
    // tensor-copy loader: 64-byte rows of the four parts inside a page
    const int row_kcode = (geo.k_code_off * 4 + code_head) >> 6;
    const int row_kstat = ((geo.k_stat_off + head * (BS * 4)) * 4) >> 6;
    const int row_vcode = (geo.v_code_off * 4 + code_head) >> 6;

    // request that holds tile x of the head (prefix[b] <= x < prefix[b+1])
    auto request_of = [&](int x) {
      int l = 0, h = B;
      while (h - l > 1) {
        const int mid = (l + h) >> 1;
        if (prefix[mid] <= x) l = mid;
        else h = mid;
      }
      return l;
    };
    // lane l: physical page and position in it of the (base+l)-th tile of the run
    auto fetch_meta = [&](int base) -> uint32_t {
      const int i = base + lane;
      if (i >= total) return 0xFFFFFFFFu;
      const int x = wa + i;
      const int b = request_of(x);
      const int k = x - prefix[b];
      const uint32_t phys =
          static_cast<uint32_t>(p.block_table[static_cast<int64_t>(b) * p.bt_stride + page_lo + (k >> log2r)]);
      if (phys >= num_pages_u) return 0xFFFFFFFFu;  // also catches negative ids
      return phys | (static_cast<uint32_t>(k & (tiles_per_page - 1)) << kMaxPagesLog2);
    };
    uint32_t meta_cur = fetch_meta(0), meta_nxt = fetch_meta(32);
    auto issue = [&](int j, int stage) {  // j-th tile of the run into ring stage `stage`
      if (j != 0 && (j & 31) == 0) {
        meta_cur = meta_nxt;
        meta_nxt = fetch_meta(j + 32);
      }
      // (a reduction rather than a shuffle: the result is uniform for the compiler, so the
      // address arithmetic of the copies runs on the uniform datapath)
      const uint32_t meta = __reduce_or_sync(kFull, lane == (j & 31) ? meta_cur : 0u);
      const bool bad = meta == 0xFFFFFFFFu;
      bad_mask = bad ? (bad_mask | (1u << stage)) : (bad_mask & ~(1u << stage));
      const uint32_t phys = bad ? 0u : (meta & ((1u << kMaxPagesLog2) - 1));
      const uint32_t sub = bad ? 0u : (meta >> kMaxPagesLog2);
      const uint32_t dst = ring_base + stage * kSlotBytes;
      if (LOADER == 1) {
        if (!bad) {
          const char* const page = reinterpret_cast<const char*>(p.cache) + phys * page_bytes;
          const char* const kp = page + (ld_kcode + sub * 1024);
          const char* const vp = page + (ld_vcode + sub * 1024);
          const uint32_t dl = dst + ld_code_dst;
          cp_async16(dl + kSwKCode, kp);
          cp_async16(dl + kSwKCode + 512, kp + 512);
          cp_async16(dst + ld_stat_dst, page + (ld_stat_src + sub * ld_stat_sub));
          cp_async16(dl + kSwVCode, vp);
          cp_async16(dl + kSwVCode + 512, vp + 512);
        }
        cp_async_commit();
      } else {
        const uint32_t bar = bar_base + 8 * stage;
        if (elect_one_sync()) {
          mbar_arrive_expect_tx(bar, kSlotBytes);
          tensor_copy_3d(dst + kSwKCode, &map16, row_kcode + sub * 16, phys, bar);
          tensor_copy_3d(dst + kSwVCode, &map16, row_vcode + sub * 16, phys, bar);
          tensor_copy_3d(dst + kSwKStat, &map4, row_kstat + sub * 4, phys, bar);
          tensor_copy_4d(dst + kSwVStat, &mapvs, sub, head * 4, phys, bar);
        }
      }
      ++n_issued;
    };
    if (work && (!noload || n_issued == 0)) {  // first ring fill: in flight while the tables are built
      int st = s;
      for (int j = 0; j < min(total, STAGES); ++j) {
        issue(j, st);
        st = st + 1 == STAGES ? 0 : st + 1;
      }
    }

    __syncthreads();  // the previous head's tables are no longer read
    if (tid < 128) reinterpret_cast<__half*>(gptr(kLevels))[tid] = __float2half_rn(level_early);  // fp16 [K|V][4][16]
    __syncthreads();
    {  // byte -> (level[low nibble], level[high nibble]) tables, one copy per bank.
       // Block P (P = 0, 1) holds, in bank l, the K table of group 2*((l>>1)&1)+P and the
       // V table of group 2*(l>>4)+P: the groups lane l needs when an MMA works on pair P.
      const unsigned short* lv = reinterpret_cast<const unsigned short*>(gptr(kLevels));
#pragma unroll 4
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
    __syncthreads();

    // One request covers this CTA's whole share (few, long requests): the warps do not leave a
    // partial each; they merge in shared memory and the CTA leaves one, so a request's chain of
    // partials has one link per CTA instead of one per warp.  (CTA-uniform.)
    int solo_b = request_of(first);
    const bool solo = prefix[solo_b + 1] >= first + span;

    // ---- attention state of the request being streamed ------------------------------------
    uint32_t qb[2][4][2];  // B operand of QK: q of head hcol, pre-scaled by softmax_scale * log2(e)
    float qs[4];           // sum over the dims of group g of the rounded q of head tig
    float oacc[2][4][4], cmin[2][4];
    float m_used = -CUDART_INF_F, l_run = 0.f;  // head tig

    // `before_second` runs before the first read of the second tile (its wait), `after_reads(t)`
    // after the last read of tile t from the ring (its stage is refilled while its V part is
    // still being multiplied): the tile that was issued last gets the most time to arrive.
    auto process = [&](auto nt_tag, auto partial_tag, const uint32_t sbA, const uint32_t sbB, const int nvA,
                       const int nvB, auto&& before_second, auto&& after_reads) {
      constexpr int NT = decltype(nt_tag)::value;
      constexpr bool PARTIAL = decltype(partial_tag)::value;
      const uint32_t sb[2] = {sbA, sbB};
      const int nv[2] = {nvA, nvB};
      // ------------------------------ S = Lk * Qblock (one accumulator per tile and pair) ----
      float sacc[NT][2][4];
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        if (t == 1) before_second();
#pragma unroll
        for (int P = 0; P < 2; ++P) {
          const uint32_t ka = sb[t] + (P ? kc_off1 : kc_off0);
          const uint2 k0 = ring_load64<0>(ka);    // token gid
          const uint2 k1 = ring_load64<512>(ka);  // token gid+8
          const uint32_t w0[2] = {k0.x, k0.y}, w1[2] = {k1.x, k1.y};
          const uint32_t kl = P ? klane1 : klane0;
          uint32_t av[4][4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            av[j][0] = lut_load(__byte_perm(w0[j >> 1], kl, (j & 1) ? 0x7624 : 0x7604));
            av[j][1] = lut_load(__byte_perm(w1[j >> 1], kl, (j & 1) ? 0x7624 : 0x7604));
            av[j][2] = lut_load(__byte_perm(w0[j >> 1], kl, (j & 1) ? 0x7634 : 0x7614));
            av[j][3] = lut_load(__byte_perm(w1[j >> 1], kl, (j & 1) ? 0x7634 : 0x7614));
          }
          mma16816_zero(sacc[t][P], av[0][0], av[0][1], av[0][2], av[0][3], qb[P][0][0], qb[P][0][1]);
#pragma unroll
          for (int j = 1; j < 4; ++j)
            mma16816(sacc[t][P], av[j][0], av[j][1], av[j][2], av[j][3], qb[P][j][0], qb[P][j][1]);
        }
      }
      // ------------------------------ V index bytes (token pair -> one table index) ---------
      // Independent of the softmax below, so issued here to overlap with its latency.
      uint32_t vidx[NT][2][2][2];  // [tile][pair][k-slots 2tig.. / 2tig+8..][row gid / row gid+8]
#pragma unroll
      for (int t = 0; t < NT; ++t) {
#pragma unroll
        for (int P = 0; P < 2; ++P)
#pragma unroll
          for (int o = 0; o < 2; ++o) {
            const uint32_t va = sb[t] + vc_off[0][P], vb = sb[t] + vc_off[1][P];
            const uint32_t xa = o ? ring_load32<512>(va) : ring_load32<0>(va);  // token tig (+8)
            const uint32_t xb = o ? ring_load32<512>(vb) : ring_load32<0>(vb);  // token tig+4 (+8)
            vidx[t][P][o][0] = (xa & 0x0F0F0F0Fu) | ((xb << 4) & 0xF0F0F0F0u);
            vidx[t][P][o][1] = ((xa >> 4) & 0x0F0F0F0Fu) | (xb & 0xF0F0F0F0u);
          }
      }
      // ------------------------------ scores of head tig for tokens tq0, tq0+4 ---------------
      float sc[NT][2];
#pragma unroll
      for (int t = 0; t < NT; ++t) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const uint4 st = ring_load128i<0>(sb[t] + (r ? ks_off1 : ks_off0));  // groups 0..3
          const float2 g0 = stat_word_to_f32<STAT_BF16>(st.x), g1 = stat_word_to_f32<STAT_BF16>(st.y);
          const float2 g2 = stat_word_to_f32<STAT_BF16>(st.z), g3 = stat_word_to_f32<STAT_BF16>(st.w);
          float u = g0.x * sacc[t][0][2 * r];       // column 2tig: group P, column 2tig+1: group P+2
          float v = g1.x * sacc[t][1][2 * r];
          u = fmaf(g2.x, sacc[t][0][2 * r + 1], u);
          v = fmaf(g3.x, sacc[t][1][2 * r + 1], v);
          u = fmaf(g0.y, qs[0], u);
          v = fmaf(g1.y, qs[1], v);
          u = fmaf(g2.y, qs[2], u);
          v = fmaf(g3.y, qs[3], v);
          float x = u + v;
          if (PARTIAL) {  // behind the end of the sequence (statistics may be NaN)
            if (tq0 + 8 * r >= nv[t]) x = -CUDART_INF_F;
          }
          sc[t][r] = x;
        }
      }
      // ------------------------------ online softmax over the tile(s) -------------------------
      float tmax = fmaxf(sc[0][0], sc[0][1]);
      if (NT == 2) tmax = fmaxf(tmax, fmaxf(sc[NT - 1][0], sc[NT - 1][1]));
      tmax = fmaxf(tmax, __shfl_xor_sync(kFull, tmax, 4));
      tmax = fmaxf(tmax, __shfl_xor_sync(kFull, tmax, 8));
      tmax = fmaxf(tmax, __shfl_xor_sync(kFull, tmax, 16));
      const bool need = tmax > m_used + kRescaleThreshold;
      if (__any_sync(kFull, need)) {
        const float m_new = need ? tmax : m_used;
        const float corr = (m_new == -CUDART_INF_F) ? 1.f : fast_exp2(m_used - m_new);
        m_used = m_new;
        l_run *= corr;
#pragma unroll
        for (int P = 0; P < 2; ++P) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) oacc[P][i][c] *= corr;
#pragma unroll
          for (int c = 0; c < 4; ++c) cmin[P][c] *= corr;
        }
      }
      uint32_t ph2[NT][2];  // [tile][k-slots 2tig.. / 2tig+8..]: probabilities of head hcol, two tokens each
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const float e0 = fast_exp2(sc[t][0] - m_used), e1 = fast_exp2(sc[t][1] - m_used);
        l_run += e0 + e1;
        const uint32_t mine = pack_half2(e0, e1);  // head tig: (token gid, token gid+8)
        const uint32_t fromA = __shfl_sync(kFull, mine, src_lane0);  // tokens of k-slots 2tig, 2tig+8
        const uint32_t fromB = __shfl_sync(kFull, mine, src_lane1);  // tokens of k-slots 2tig+1, 2tig+9
        ph2[t][0] = __byte_perm(fromA, fromB, 0x5410);
        ph2[t][1] = __byte_perm(fromA, fromB, 0x7632);
      }
      // ------------------------------ per tile: W = p*scale_v, p*min_v, then O += Lv^T * W ----
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const uint32_t sa0 = sb[t] + vs_off0, sa1 = sb[t] + vs_off1;
        uint32_t wb2[2][2], mb2[2][2];  // [pair][k-slots 2tig.. / 2tig+8..]
#pragma unroll
        for (int P = 0; P < 2; ++P) {
#pragma unroll
          for (int o = 0; o < 2; ++o) {
            // statistic words of tokens tig+8o and tig+4+8o
            const uint32_t fst = P ? (o ? ring_load32<64>(sa0) : ring_load32<64 + 32>(sa0))
                                   : (o ? ring_load32<0>(sa0) : ring_load32<32>(sa0));
            const uint32_t snd = P ? (o ? ring_load32<64>(sa1) : ring_load32<64 + 32>(sa1))
                                   : (o ? ring_load32<0>(sa1) : ring_load32<32>(sa1));
            uint32_t sc2, mn2;
            if (STAT_BF16) {
              sc2 = pack_half2(__uint_as_float(fst << 16), __uint_as_float(snd << 16));
              mn2 = pack_half2(__uint_as_float(fst & 0xFFFF0000u), __uint_as_float(snd & 0xFFFF0000u));
            } else {
              sc2 = __byte_perm(fst, snd, 0x5410);
              mn2 = __byte_perm(fst, snd, 0x7632);
            }
            uint32_t wv = hmul2_u32(ph2[t][o], sc2), mv = hmul2_u32(ph2[t][o], mn2);
            if (PARTIAL) {  // 0 * NaN would poison the accumulators
              const uint32_t keep = (tig + 8 * o < nv[t] ? 0x0000FFFFu : 0u) | (tig + 4 + 8 * o < nv[t] ? 0xFFFF0000u : 0u);
              wv &= keep;
              mv &= keep;
            }
            wb2[P][o] = wv;
            mb2[P][o] = mv;
          }
        }
        after_reads(t);  // nothing of this tile is read from the ring any more
#pragma unroll
        for (int P = 0; P < 2; ++P) {
          const uint32_t vl = P ? vlane1 : vlane0;
          uint32_t av[4][4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t sel = i == 0 ? 0x7604 : i == 1 ? 0x7614 : i == 2 ? 0x7624 : 0x7634;
            av[i][0] = lut_load(__byte_perm(vidx[t][P][0][0], vl, sel));
            av[i][1] = lut_load(__byte_perm(vidx[t][P][0][1], vl, sel));
            av[i][2] = lut_load(__byte_perm(vidx[t][P][1][0], vl, sel));
            av[i][3] = lut_load(__byte_perm(vidx[t][P][1][1], vl, sel));
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) mma16816(oacc[P][i], av[i][0], av[i][1], av[i][2], av[i][3], wb2[P][0], wb2[P][1]);
          const uint32_t ones = 0x3C003C00u;
          mma16816(cmin[P], ones, ones, ones, ones, mb2[P][0], mb2[P][1]);
        }
      }
    };

    // ---- stream through the run, request by request ----------------------------------------
    int x = wa;
    int b = work ? request_of(wa) : 0;
    int run_done = 0;  // tiles of this run consumed so far
    while (work && run_done < total && !dead) {
      while (prefix[b + 1] <= x) ++b;
      const int pb = prefix[b];
      const int nb = prefix[b + 1] - pb;
      const int k0 = x - pb, kend = min(nb, wb - pb);
      const int ntok = min(p.token_hi, p.seq_lens[b]) - lo;
      {  // query fragments and group sums of request b
        const bool live_h = hcol < nh;
        const int64_t qoff = static_cast<int64_t>(b) * p.q_batch_stride + static_cast<int64_t>(hq0 + hcol) * kHeadDim;
        float part[2] = {0.f, 0.f};
#pragma unroll
        for (int P = 0; P < 2; ++P)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int d0 = 32 * (2 * ksel + P) + 16 * khalf + 4 * j;
            float f[4];
            if (sp.q_vec) {
              const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const unsigned short*>(p.q) + qoff + d0);
              const uint32_t w[2] = {raw.x, raw.y};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const uint32_t bits = (i & 1) ? (w[i >> 1] >> 16) : (w[i >> 1] & 0xFFFFu);
                const float v = p.q_dtype == BKV_BF16 ? bf16_bits_to_f32(bits) : f16_bits_to_f32(bits);
                f[i] = live_h ? v * p.scale_log2 : 0.f;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i) f[i] = live_h ? load_q(p.q, qoff + d0 + i, p.q_dtype) * p.scale_log2 : 0.f;
            }
            const uint32_t lo2 = pack_half2(f[0], f[1]), hi2 = pack_half2(f[2], f[3]);
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo2));
            const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&hi2));
            part[P] += (a.x + a.y) + (c.x + c.y);
            qb[P][j][0] = ksel == gsel ? lo2 : 0u;  // the other group of the pair meets zeros
            qb[P][j][1] = ksel == gsel ? hi2 : 0u;
          }
#pragma unroll
        for (int P = 0; P < 2; ++P) {
          part[P] += __shfl_xor_sync(kFull, part[P], 1);  // both halves of the group
#pragma unroll
          for (int e = 0; e < 2; ++e) qs[2 * e + P] = __shfl_sync(kFull, part[P], (2 * tig) * 4 + 2 * e);
        }
      }
#pragma unroll
      for (int P = 0; P < 2; ++P) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int c = 0; c < 4; ++c) oacc[P][i][c] = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) cmin[P][c] = 0.f;
      }
      m_used = -CUDART_INF_F;
      l_run = 0.f;

      for (int k = k0; k < kend;) {
        const int cnt = min(PAIR, kend - k);
        const int sB = s + 1 == STAGES ? 0 : s + 1;
        const uint32_t phaseB = s + 1 == STAGES ? phase ^ 1u : phase;
        // (the timing experiment stops issuing after the first fill and so stops waiting too)
        auto wait_tile = [&](int ahead, int stage, uint32_t parity) {  // tile n_done + ahead of this warp
          if (n_done + ahead >= n_issued) return;
          if (LOADER == 1) {
            if (nowait) return;
            cp_async_wait_pending(n_issued - n_done - ahead - 1);  // this thread's pieces of the tile ...
            __syncwarp();                                           // ... and every other lane's
          } else if (!wait_full(bar_base + 8 * stage, parity)) {
            dead = true;
          }
        };
        auto refill = [&](int ahead, int stage) {  // the stage of tile n_done + ahead is free again
          if (noload) return;
          __syncwarp();
          if (LOADER != 1) fence_proxy_async();  // reads of the generic proxy before writes of the async proxy
          if (run_done + ahead + STAGES < total) issue(run_done + ahead + STAGES, stage);
        };
        wait_tile(0, s, phase);
        if (dead) break;
        const int rem = ntok - kTile * k;
        const int nvA = (bad_mask >> s) & 1 ? 0 : min(kTile, rem);
        const int nvB = cnt == 2 ? ((bad_mask >> sB) & 1 ? 0 : min(kTile, rem - kTile)) : 0;
        const uint32_t sbA = ring_base + s * kSlotBytes, sbB = ring_base + sB * kSlotBytes;
        auto wait_second = [&] { wait_tile(1, sB, phaseB); };
        auto refill_tile = [&](int t) { refill(t, t ? sB : s); };
        if (cnt == 2) {
          if (nvA == kTile && nvB == kTile) {
            process(std::integral_constant<int, 2>{}, std::false_type{}, sbA, sbB, nvA, nvB, wait_second, refill_tile);
          } else if (nvA > 0 || nvB > 0) {
            process(std::integral_constant<int, 2>{}, std::true_type{}, sbA, sbB, nvA, nvB, wait_second, refill_tile);
          } else {  // two unmapped pages: nothing to compute, the ring still turns
            wait_second();
            refill_tile(0);
            refill_tile(1);
          }
        } else if (nvA > 0) {
          process(std::integral_constant<int, 1>{}, std::true_type{}, sbA, sbA, nvA, 0, [] {}, refill_tile);
        } else {
          refill_tile(0);
        }
        if (dead) break;
        k += cnt;
        run_done += cnt;
        n_done += cnt;
        if (cnt == 2) {
          s = sB + 1 == STAGES ? 0 : sB + 1;
          phase = sB + 1 == STAGES ? phaseB ^ 1u : phaseB;
        } else {
          s = sB;
          phase = phaseB;
        }
      }
      if (dead) break;
      if (solo) break;  // the only request of this run: merged with the other warps below

      // ---- leave request b: final output or a partial ---------------------------------------
      float l_tot = l_run;  // tokens were spread over gid
      l_tot += __shfl_xor_sync(kFull, l_tot, 4);
      l_tot += __shfl_xor_sync(kFull, l_tot, 8);
      l_tot += __shfl_xor_sync(kFull, l_tot, 16);
      const bool whole = k0 == 0 && kend == nb;
      if (tig < nh) {
        if (whole && p.force_partial) {  // the caller merges across ranks: un-normalised (o, m, l)
          const int64_t row = static_cast<int64_t>(b) * p.heads_q + hq0 + tig;
          float2* dst = reinterpret_cast<float2*>(p.o_partial + row * kHeadDim);
#pragma unroll
          for (int P = 0; P < 2; ++P)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int d = 32 * (2 * vsel + P) + 8 * vu + 2 * i;
              const float mn = vsel ? cmin[P][1] : cmin[P][0];
              dst[d >> 1] = l_tot > 0.f ? make_float2((vsel ? oacc[P][i][1] : oacc[P][i][0]) + mn,
                                                      (vsel ? oacc[P][i][3] : oacc[P][i][2]) + mn)
                                        : make_float2(0.f, 0.f);
            }
          if (gid == 0) {
            p.m_partial[row] = l_tot > 0.f ? m_used * kLn2 : -CUDART_INF_F;
            p.l_partial[row] = l_tot;
          }
        } else if (whole) {
          const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
          const int64_t row = static_cast<int64_t>(b) * p.heads_q + hq0 + tig;
#pragma unroll
          for (int P = 0; P < 2; ++P)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int d = 32 * (2 * vsel + P) + 8 * vu + 2 * i;
              const float mn = vsel ? cmin[P][1] : cmin[P][0];
              const float ve = ((vsel ? oacc[P][i][1] : oacc[P][i][0]) + mn) * inv;
              const float vo = ((vsel ? oacc[P][i][3] : oacc[P][i][2]) + mn) * inv;
              store_out(p.out, row * kHeadDim + d, p.out_dtype, ve);
              store_out(p.out, row * kHeadDim + d + 1, p.out_dtype, vo);
              if (p.out_f32) {
                p.out_f32[row * kHeadDim + d] = ve;
                p.out_f32[row * kHeadDim + d + 1] = vo;
              }
            }
        } else {
          const int64_t row = static_cast<int64_t>(2 * range + (k0 > 0 ? 0 : 1)) * 4 + tig;
          float2* dst = reinterpret_cast<float2*>(sp.ws_o + row * kHeadDim);
#pragma unroll
          for (int P = 0; P < 2; ++P)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int d = 32 * (2 * vsel + P) + 8 * vu + 2 * i;
              const float mn = vsel ? cmin[P][1] : cmin[P][0];
              dst[d >> 1] = make_float2((vsel ? oacc[P][i][1] : oacc[P][i][0]) + mn,
                                        (vsel ? oacc[P][i][3] : oacc[P][i][2]) + mn);
            }
          if (gid == 0) {
            sp.ws_m[row] = m_used;
            sp.ws_l[row] = l_tot;
          }
        }
      }
      if (!whole && lane == 0)
        sp.ws_hdr[2 * range + (k0 > 0 ? 0 : 1)] = ((vh * B + b) << 1) | (kend == nb ? 1 : 0);
      x += kend - k0;
    }

    if (solo) {
      // ---- merge the warps of the CTA (all of them worked on request solo_b) ------------------
      __syncthreads();  // every tile of every warp has been consumed: the rings are free
      float* const mo = reinterpret_cast<float*>(gptr(kRingLoS));  // [NW][4][128]
      float* const mm = mo + NW * 4 * kHeadDim;
      float* const ml = mm + NW * 4;
      const bool mine = work && !dead;
      float l_tot = mine ? l_run : 0.f;  // tokens were spread over gid
      l_tot += __shfl_xor_sync(kFull, l_tot, 4);
      l_tot += __shfl_xor_sync(kFull, l_tot, 8);
      l_tot += __shfl_xor_sync(kFull, l_tot, 16);
      if (mine) {
        float2* dst = reinterpret_cast<float2*>(mo + (warp * 4 + tig) * kHeadDim);
#pragma unroll
        for (int P = 0; P < 2; ++P)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int d = 32 * (2 * vsel + P) + 8 * vu + 2 * i;
            const float mn = vsel ? cmin[P][1] : cmin[P][0];
            dst[d >> 1] = make_float2((vsel ? oacc[P][i][1] : oacc[P][i][0]) + mn,
                                      (vsel ? oacc[P][i][3] : oacc[P][i][2]) + mn);
          }
      }
      if (gid == 0) {
        mm[warp * 4 + tig] = mine ? m_used : -CUDART_INF_F;
        ml[warp * 4 + tig] = l_tot;
      }
      __syncthreads();
      const int k0c = first - prefix[solo_b];
      const bool ends = first + span == prefix[solo_b + 1];
      const bool whole = k0c == 0 && ends;
      const int slot = 2 * ((cta * 2 + ph) * NW) + (k0c > 0 ? 0 : 1);  // of the CTA's first range
      for (int idx = tid; idx < 4 * kHeadDim; idx += NW * 32) {
        const int h = idx >> 7, d = idx & (kHeadDim - 1);
        if (h >= nh) continue;
        float M = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < NW; ++w)
          if (ml[w * 4 + h] > 0.f) M = fmaxf(M, mm[w * 4 + h]);
        float den = 0.f, num = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          const float lw = ml[w * 4 + h];
          if (!(lw > 0.f)) continue;
          const float wt = exp2f(mm[w * 4 + h] - M);
          den += wt * lw;
          num += wt * mo[(w * 4 + h) * kHeadDim + d];
        }
        const int64_t row = static_cast<int64_t>(solo_b) * p.heads_q + hq0 + h;
        if (!whole) {
          const int64_t prow = static_cast<int64_t>(slot) * 4 + h;
          sp.ws_o[prow * kHeadDim + d] = num;
          if (d == 0) {
            sp.ws_m[prow] = M;
            sp.ws_l[prow] = den;
          }
        } else if (p.force_partial) {
          p.o_partial[row * kHeadDim + d] = den > 0.f ? num : 0.f;
          if (d == 0) {
            p.m_partial[row] = den > 0.f ? M * kLn2 : -CUDART_INF_F;
            p.l_partial[row] = den;
          }
        } else {
          const float o = den > 0.f ? num / den : 0.f;
          store_out(p.out, row * kHeadDim + d, p.out_dtype, o);
          if (p.out_f32) p.out_f32[row * kHeadDim + d] = o;
        }
      }
      if (!whole && tid == 0) sp.ws_hdr[slot] = ((vh * B + solo_b) << 1) | (ends ? 1 : 0);
      __syncthreads();  // the scratch is ring space again
    }
  }

  if (LOADER == 1) cp_async_wait_group<0>();
  if (LOADER != 1 && dead) {  // let the copies still in flight land before the shared memory is given back
    for (int g = n_done; g < n_issued; ++g) {
      const int st = g % STAGES;
      WaitBudget budget;
      while (!mbar_try_wait(bar_base + 8 * st, (g / STAGES) & 1) && !budget.expired()) {
      }
    }
  }
}

// ---- fix-up: merge the chains of partials of the requests that were cut ---------------------
// One CTA per decode CTA looks at the 2*NW ranges of that CTA.  A range OWNS the request whose
// first part is its slot 1; the chain continues through slot 0 of the following ranges up to
// the part flagged last.  The four 128-thread groups of the CTA each take one owner at a time
// (thread = output dimension, the four query heads in registers).
constexpr int kFixThreads = 512;
constexpr int kFixGroup = 128;
constexpr int kFixBatch = 4;

__device__ __forceinline__ void group_sync(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "n"(kFixGroup) : "memory");
}

__global__ void __launch_bounds__(kFixThreads) stream_fixup_kernel(const StreamParams sp, const int ranges_per_cta,
                                                                  const int num_ranges) {
  const DecodeParams& p = sp.d;
  pdl_wait();  // launched while the decode grid still runs: its writes are visible from here on
  __shared__ int s_owner[32];
  __shared__ int s_nown;
  __shared__ int s_hdr[4][kFixGroup];
  __shared__ int s_list[4][kFixGroup];
  __shared__ int s_cnt[4], s_done[4];
  __shared__ float s_red[3][4][4][kFixGroup];  // [M, num, den][group][head][dim]: cooperative mode only
  const int tid = threadIdx.x, g = tid >> 7, d = tid & (kFixGroup - 1);
  const int r0 = blockIdx.x * ranges_per_cta;
  if (tid < 32) {  // ranges_per_cta <= 32
    const int hd = tid < ranges_per_cta ? sp.ws_hdr[2 * (r0 + tid) + 1] : kHdrNone;
    const unsigned mask = __ballot_sync(0xffffffffu, hd >= 0);
    if (hd >= 0) s_owner[__popc(mask & ((1u << tid) - 1))] = r0 + tid;
    if (tid == 0) s_nown = __popc(mask);
  }
  __syncthreads();
  const int nown = s_nown;
  const int gqa = p.heads_q / p.heads_kv;
  // One owner in this CTA (few, long requests): all four groups share its chain, group g taking
  // every fourth part, and the four results are merged through shared memory.  Several owners:
  // one group per owner.
  const bool coop = nown == 1;
  for (int oi = coop ? 0 : g; oi < nown; oi += 4) {
    const int range = s_owner[oi];
    const int hd = sp.ws_hdr[2 * range + 1];
    const int item = hd >> 1;
    const int vh = item / p.batch, b = item - vh * p.batch;
    const int head = vh / sp.quads, quad = vh - head * sp.quads;
    const int nh = min(4, gqa - quad * 4);
    float M[4], num[4], den[4];
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      M[h] = -CUDART_INF_F;
      num[h] = 0.f;
      den[h] = 0.f;
    }
    auto merge = [&](int h, float m2, float l2, float o2) {
      if (!(l2 > 0.f)) return;
      const float Mn = fmaxf(M[h], m2);
      const float a = (M[h] == -CUDART_INF_F) ? 0.f : exp2f(M[h] - Mn);
      const float w = exp2f(m2 - Mn);
      num[h] = num[h] * a + o2 * w;
      den[h] = den[h] * a + l2 * w;
      M[h] = Mn;
    };
    auto merge_slots = [&](const int64_t slot0, const int64_t slot1, const int64_t slot2, const int64_t slot3, int n) {
      const int64_t slots[kFixBatch] = {slot0, slot1, slot2, slot3};
      float m2[kFixBatch][4], l2[kFixBatch][4], o2[kFixBatch][4];
#pragma unroll
      for (int u = 0; u < kFixBatch; ++u)
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const bool on = u < n && h < nh;
          const int64_t row = slots[u] * 4 + h;
          m2[u][h] = on ? sp.ws_m[row] : 0.f;
          l2[u][h] = on ? sp.ws_l[row] : 0.f;
          o2[u][h] = on ? sp.ws_o[row * kHeadDim + d] : 0.f;
        }
#pragma unroll
      for (int u = 0; u < kFixBatch; ++u)
#pragma unroll
        for (int h = 0; h < 4; ++h) merge(h, m2[u][h], l2[u][h], o2[u][h]);
    };
    if (!coop || g == 0) merge_slots(2ll * range + 1, 0, 0, 0, 1);
    const bool chain_open = (hd & 1) == 0;
    for (int base = range + 1; chain_open && base < num_ranges; base += kFixGroup) {
      const int r = base + d;
      s_hdr[g][d] = r < num_ranges ? sp.ws_hdr[2 * r] : kHdrNone;
      group_sync(g);
      if (d == 0) {
        int cnt = 0, done = base + kFixGroup >= num_ranges ? 1 : 0;
        for (int j = 0; j < kFixGroup; ++j) {
          const int hj = s_hdr[g][j];
          if (hj < 0) continue;                        // an empty range
          if ((hj >> 1) != item) { done = 1; break; }  // cannot happen: the chain is contiguous
          s_list[g][cnt++] = base + j;
          if (hj & 1) { done = 1; break; }
        }
        s_cnt[g] = cnt;
        s_done[g] = done;
      }
      group_sync(g);
      const int cnt = s_cnt[g];
      const int first = coop ? g * kFixBatch : 0, stride = coop ? 4 * kFixBatch : kFixBatch;
      for (int c0 = first; c0 < cnt; c0 += stride) {
        const int n = min(kFixBatch, cnt - c0);
        merge_slots(2ll * s_list[g][c0], 2ll * s_list[g][min(c0 + 1, cnt - 1)], 2ll * s_list[g][min(c0 + 2, cnt - 1)],
                    2ll * s_list[g][min(c0 + 3, cnt - 1)], n);
      }
      const int done = s_done[g];
      group_sync(g);
      if (done) break;
    }
    if (coop) {  // fold the four groups' results (uniform over the CTA: one owner)
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        s_red[0][g][h][d] = M[h];
        s_red[1][g][h][d] = num[h];
        s_red[2][g][h][d] = den[h];
      }
      __syncthreads();
      if (g != 0) continue;
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        M[h] = -CUDART_INF_F;
        num[h] = 0.f;
        den[h] = 0.f;
#pragma unroll
        for (int gg = 0; gg < 4; ++gg) {
          const float m2 = s_red[0][gg][h][d], l2 = s_red[2][gg][h][d], o2 = s_red[1][gg][h][d];
          if (!(l2 > 0.f)) continue;
          const float Mn = fmaxf(M[h], m2);
          const float a = (M[h] == -CUDART_INF_F) ? 0.f : exp2f(M[h] - Mn);
          const float w = exp2f(m2 - Mn);
          num[h] = num[h] * a + o2 * w;
          den[h] = den[h] * a + l2 * w;
          M[h] = Mn;
        }
      }
    }
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      if (h >= nh) continue;
      const int64_t row = static_cast<int64_t>(b) * p.heads_q + head * gqa + quad * 4 + h;
      if (p.force_partial) {
        p.o_partial[row * kHeadDim + d] = den[h] > 0.f ? num[h] : 0.f;
        if (d == 0) {
          p.m_partial[row] = den[h] > 0.f ? M[h] * kLn2 : -CUDART_INF_F;
          p.l_partial[row] = den[h];
        }
      } else {
        const float o = den[h] > 0.f ? num[h] / den[h] : 0.f;
        store_out(p.out, row * kHeadDim + d, p.out_dtype, o);
        if (p.out_f32) p.out_f32[row * kHeadDim + d] = o;
      }
    }
  }
}

// tiles before every request for batches beyond kMaxBatch (one CTA, inclusive scan by chunks)
__global__ void __launch_bounds__(1024) stream_prefix_kernel(const DecodeParams p, int* __restrict__ prefix) {
  __shared__ int s_warp[32];
  __shared__ int s_carry;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int lo = max(p.token_lo, 0);
  if (tid == 0) {
    s_carry = 0;
    prefix[0] = 0;
  }
  __syncthreads();
  for (int base = 0; base < p.batch; base += 1024) {
    const int b = base + tid;
    int n = 0;
    if (b < p.batch) {
      const int hi_b = min(p.token_hi, p.seq_lens[b]);
      n = hi_b > lo ? (hi_b - lo + kTile - 1) / kTile : 0;
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, n, o);
      if (lane >= o) n += y;
    }
    if (lane == 31) s_warp[warp] = n;
    __syncthreads();
    if (warp == 0) {
      const int v = s_warp[lane];
      int w = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += y;
      }
      s_warp[lane] = w - v;
    }
    __syncthreads();
    const int incl = s_carry + s_warp[warp] + n;
    if (b < p.batch) prefix[1 + b] = incl;
    __syncthreads();
    if (tid == 1023) s_carry = incl;
    __syncthreads();
  }
}

constexpr int64_t kPartialBytes = 4 * kHeadDim * 4 + 16 + 16 + 4;  // o, m, l of four heads and the header
constexpr int64_t kPlannedPrefixBytes = (kMaxBatchPlanned + 64) * 4;  // a multiple of 256

// ---- tensor maps of the packed cache ------------------------------------------------------------
// The cache is described as uint8 [page][64-byte row][64]; a box is `rows` rows of one page,
// stored with the 64-byte swizzle.  Maps are cached per (cache, geometry, box).
struct CacheMaps {
  CUtensorMap map16, map4, mapvs;
};
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      sym = nullptr;
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

bool make_cache_map(CUtensorMap* out, const DecodeParams& p, int rows) {
  const EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return false;
  const PageGeom geo = make_geom(p.block_size, p.heads_kv);
  const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(geo.block_i32) * 4 / 64, static_cast<cuuint64_t>(p.num_pages)};
  const cuuint64_t strides[2] = {64, static_cast<cuuint64_t>(p.page_stride) * 4};
  const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(rows), 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint32_t*>(p.cache), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_vstat_map(CUtensorMap* out, const DecodeParams& p) {
  const EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return false;
  const PageGeom geo = make_geom(p.block_size, p.heads_kv);
  const cuuint64_t dims[4] = {64, static_cast<cuuint64_t>(p.block_size / 16), static_cast<cuuint64_t>(p.heads_kv) * 4,
                              static_cast<cuuint64_t>(p.num_pages)};
  const cuuint64_t strides[3] = {64, static_cast<cuuint64_t>(p.block_size) * 4, static_cast<cuuint64_t>(p.page_stride) * 4};
  const cuuint32_t box[4] = {64, 1, 4, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  void* base = const_cast<uint32_t*>(p.cache) + geo.v_stat_off;
  return enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// false: the driver offers no tensor maps for this cache (then the cp.async loader is used)
bool cache_maps_for(const DecodeParams& p, CacheMaps* out) {
  struct Entry {
    const void* cache;
    int64_t pages, stride;
    int block, heads, dev;
    CacheMaps maps;
    bool ok;
  };
  static std::mutex mu;
  static Entry slots[8] = {};
  static int next = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  for (const Entry& e : slots)
    if (e.cache == p.cache && e.pages == p.num_pages && e.stride == p.page_stride && e.block == p.block_size &&
        e.heads == p.heads_kv && e.dev == dev && e.cache != nullptr) {
      *out = e.maps;
      return e.ok;
    }
  Entry& e = slots[next];
  next = (next + 1) % 8;
  e = Entry{p.cache, p.num_pages, p.page_stride, p.block_size, p.heads_kv, dev, {}, false};
  e.ok = (p.page_stride * 4) % 64 == 0 && make_cache_map(&e.maps.map16, p, 16) && make_cache_map(&e.maps.map4, p, 4) &&
         make_vstat_map(&e.maps.mapvs, p);
  *out = e.maps;
  return e.ok;
}

template <int NW, int STAGES, int LOADER, int PAIR = 2>
int launch_variant(const DecodeParams& p, void* ws, int64_t ws_bytes, int max_seq_len, int sm_count,
                   cudaStream_t stream) {
  using R = Ring<NW, STAGES>;
  StreamParams sp;
  sp.d = p;
  const int gqa = p.heads_q / p.heads_kv;
  sp.quads = (gqa + 3) / 4;
  sp.q_vec = (p.q_dtype == BKV_BF16 || p.q_dtype == BKV_F16) && reinterpret_cast<uintptr_t>(p.q) % 8 == 0 &&
             p.q_batch_stride % 4 == 0;
  const int hv = p.heads_kv * sp.quads;
  if (hv > sm_count) return BKV_ERR_UNSUPPORTED;
  const int64_t tiles_max = static_cast<int64_t>(hv) * p.batch * ((max_seq_len + kTile - 1) / kTile);
  int64_t ctas = (tiles_max + 2 * NW - 1) / (2 * NW);
  if (ctas < hv) ctas = hv;  // a share never spans more than two heads
  if (ctas > sm_count) ctas = sm_count;
  const int C = static_cast<int>(ctas);
  // Equal shares make the CTAs whose share straddles two heads build the tables twice and
  // restart their pipelines (a few us, which the share computation takes off their tile
  // count); head-aligned shares avoid that but the heads served by fewer CTAs finish later.
  // Take the cheaper of the two estimates (0.1 us per tile and SM).
  {
    const int base = C / hv;
    const double per_cta_us = static_cast<double>(tiles_max) / C * 0.1;
    const double aligned_loss_us = per_cta_us * (static_cast<double>(C) / hv / base - 1.0);
    sp.straddle_tiles = 40;  // ~4 us: with 100 the straddling CTAs were measured to finish 7 us early
    // compensated equal shares lose about (heads - 1) gaps spread over all CTAs
    const double equal_loss_us = 4.0 * (hv - 1) / C + 1.0;
    sp.aligned = (C % hv == 0 || aligned_loss_us < equal_loss_us) ? 1 : 0;
    if (p.flags & BKV_FLAG_DEBUG_EQUAL_SHARES) sp.aligned = 0;
    if (p.flags & BKV_FLAG_DEBUG_ALIGNED_SHARES) sp.aligned = 1;
  }
  const int num_ranges = C * 2 * NW;
  const int64_t slots = 2ll * num_ranges;
  if (!ws || ws_bytes < slots * kPartialBytes + kPlannedPrefixBytes) return BKV_ERR_ARG;
  char* w = static_cast<char*>(ws) + kPlannedPrefixBytes;  // the prefix sums come first
  sp.ws_o = reinterpret_cast<float*>(w);
  sp.ws_m = reinterpret_cast<float*>(w + slots * (4 * kHeadDim * 4));
  sp.ws_l = sp.ws_m + slots * 4;
  sp.ws_hdr = reinterpret_cast<int*>(sp.ws_l + slots * 4);
  sp.ws_prefix = static_cast<int*>(ws);
  if (p.batch > kMaxBatch) {
    stream_prefix_kernel<<<1, 1024, 0, stream>>>(p, sp.ws_prefix);
    const int rcp = check_launch("bkv_decode_stream_sm100(prefix)");
    if (rcp != BKV_OK) return rcp;
  }

  CacheMaps maps = {};
  if (LOADER == 3 && !cache_maps_for(p, &maps)) return BKV_ERR_UNSUPPORTED;
  auto kern = p.stat_bf16 ? decode_stream_kernel<NW, STAGES, true, LOADER, PAIR>
                          : decode_stream_kernel<NW, STAGES, false, LOADER, PAIR>;
  static bool configured[2][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[p.stat_bf16 ? 1 : 0][dev]) {
    int reserved = 0;
    cudaDeviceGetAttribute(&reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev);
    if (reserved != static_cast<int>(kSmemBase)) return BKV_ERR_UNSUPPORTED;
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, R::kDynBytes);
    if (e != cudaSuccess) {
      set_last_cuda_error(e, "cudaFuncSetAttribute(decode_stream_kernel)");
      return BKV_ERR_CUDA;
    }
    // the small kernels around the decode grid ask for the same shared-memory carve-out, so the
    // SMs are not reconfigured between the launches of a step
    cudaFuncSetAttribute(stream_fixup_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(stream_prefix_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    configured[p.stat_bf16 ? 1 : 0][dev] = true;
  }
  if ((sp.d.flags & BKV_FLAG_PDL_WAIT) && sp.d.batch <= kMaxBatch) {
    // programmatic dependent launch behind the cache writer: this grid's set-up (prefix sums,
    // shares, page ids) runs while the writer drains; it waits before its first cache read.
    // (With the prefix sums planned by a kernel of their own that kernel is the predecessor
    // and the set-up reads its output, so the launch stays ordinary.)
    cudaLaunchConfig_t dcfg = {};
    dcfg.gridDim = dim3(C);
    dcfg.blockDim = dim3(NW * 32);
    dcfg.dynamicSmemBytes = R::kDynBytes;
    dcfg.stream = stream;
    cudaLaunchAttribute dattr[1];
    dattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    dattr[0].val.programmaticStreamSerializationAllowed = 1;
    dcfg.attrs = dattr;
    dcfg.numAttrs = 1;
    const cudaError_t de = cudaLaunchKernelEx(&dcfg, kern, sp, maps.map16, maps.map4, maps.mapvs);
    if (de != cudaSuccess) {
      set_last_cuda_error(de, "bkv_decode_stream_sm100(decode, dependent launch)");
      return BKV_ERR_CUDA;
    }
  } else {
    kern<<<C, NW * 32, R::kDynBytes, stream>>>(sp, maps.map16, maps.map4, maps.mapvs);
  }
  int rc = check_launch("bkv_decode_stream_sm100(decode)");
  if (rc != BKV_OK) return rc;
  // programmatic dependent launch: the fix-up grid is set up while the decode grid drains
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(C);
  cfg.blockDim = dim3(kFixThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, stream_fixup_kernel, sp, 2 * NW, num_ranges);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "bkv_decode_stream_sm100(fixup)");
    return BKV_ERR_CUDA;
  }
  return BKV_OK;
}

int device_sm_count() {
  static int cached[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && cached[dev]) return cached[dev];
  int n = 0;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (dev < 64) cached[dev] = n;
  return n;
}

}  // namespace

int64_t stream_workspace_bytes() {
  const int64_t sms = device_sm_count();
  // the prefix sums, then the ranges of the widest configuration (16 warps), two slots each
  return kPlannedPrefixBytes + sms * 2 * 16 * 2 * kPartialBytes;
}

int launch_decode_stream(const DecodeParams& p, void* ws, int64_t ws_bytes, int max_seq_len, cudaStream_t stream,
                         int config) {
  const int r = p.block_size / kTile;
  if (p.block_size % kTile != 0 || (r & (r - 1)) != 0 || p.block_size > 1024) return BKV_ERR_UNSUPPORTED;
  if ((p.page_stride * 4) % 16 != 0 || !aligned16(p.cache)) return BKV_ERR_UNSUPPORTED;
  if (p.token_lo % p.block_size != 0) return BKV_ERR_UNSUPPORTED;
  if (p.batch > kMaxBatchPlanned || p.num_pages > (1ll << kMaxPagesLog2)) return BKV_ERR_UNSUPPORTED;
  const int sms = device_sm_count();
  if (sms <= 0) return BKV_ERR_CUDA;
  switch (config) {
    case 1: return launch_variant<8, 4, 3>(p, ws, ws_bytes, max_seq_len, sms, stream);
    case 2: return launch_variant<12, 3, 3>(p, ws, ws_bytes, max_seq_len, sms, stream);
    case 3: return launch_variant<16, 2, 3>(p, ws, ws_bytes, max_seq_len, sms, stream);
    case 5: return launch_variant<12, 3, 1>(p, ws, ws_bytes, max_seq_len, sms, stream);
    case 6: return launch_variant<8, 4, 1>(p, ws, ws_bytes, max_seq_len, sms, stream);
    case 7: return launch_variant<16, 2, 1>(p, ws, ws_bytes, max_seq_len, sms, stream);
    default: return launch_variant<12, 3, 1>(p, ws, ws_bytes, max_seq_len, sms, stream);
  }
}

int read_stream_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_stream_status, sizeof(int));
  const int zero = 0;
  cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int));
  return v;
}

}  // namespace bkv
