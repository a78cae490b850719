// Persistent, warp-granular form of the tensor-core decode attention over the packed cache.
//
// The (kv-head, request, 16-token tile) space is one long line, head-major.  The grid is one
// CTA per SM; CTA c owns the c-th equal share of the line and every warp of it an equal,
// contiguous share of that (bkv_stream_partition.h).  A warp therefore streams through a run of
// consecutive tiles that may start in the middle of one request and end in the middle of another;
// the byte tables are set up once per CTA (twice when its share straddles two heads) instead of
// once per split.
//
// A warp keeps a private ring of tiles which it fills itself with asynchronous copies (16-byte
// cp.async pieces or tensor copies, see LOADER), running STAGES tiles ahead across request
// boundaries, and a private online-softmax state; no block barrier is executed while it works.
// When it leaves a request it either
//   * owns the whole request: normalises and writes the attention output, or
//   * owns a part of it:      writes an un-normalised partial (o, m, l) into one of the two
//     slots of its range and adds its tile count to the request's counter.  The warp whose
//     addition completes the count is the last of the request: it recomputes, from the
//     partition alone, where the other parts lie, merges them by log-sum-exp and writes the
//     output.  Nobody waits for anybody, and no second kernel is needed.
// When one request covers a CTA's whole share, its warps merge in shared memory first and the
// CTA leaves a single partial (and, if it is the last, merges the chain with all its warps).
//
// Arithmetic: a 256-entry table indexed by a whole code BYTE returns the two fp16 levels of its
// two nibbles as one MMA operand register, replicated so that lane l only reads bank l; the
// per-(token, group) scale and minimum are applied outside the MMAs:
//   s[t,h]  = c * sum_g ( scale_k[t,g] * (sum_{d in g} q[h,d] * Lk_g[code_k[t,d]]) + min_k[t,g] * sum_{d in g} q[h,d] )
//   o[h,d]  = sum_t (p[t,h] * scale_v[t,g(d)]) * Lv_g(d)[code_v[t,d]]  +  sum_t p[t,h] * min_v[t,g(d)]
// (fp16 statistics: the K-minimum term of s is one more MMA - A = the minima as they lie in the
// statistic words, B = the per-group sums of q as exact (high, low) fp16 pairs; bf16 statistics
// use fp32 FMAs.)
// The queries enter the MMAs un-scaled (a bf16 or fp16 query is exact as an fp16 operand; the
// softmax scale c is applied to the fp32 score), the probabilities are rounded to fp16 once and
// the softmax denominator sums the rounded values, so that rounding cancels in the quotient.
// An MMA works on one PAIR of groups {P, P+2}:
//   * tokens sit in natural order in the QK rows (row g / g+8 = token g / g+8) and as
//     (t, t+4) pairs in the PV k-slots; the ring slot is swizzled instead of padded;
//   * MMA column n stands for (query head n/2, group n%2 of the pair), so a lane's two QK
//     accumulator columns are the two groups of ONE head and its scores need no exchange;
//   * PV row g / g+8 of MMA i hold the even / odd dimension 8*(g%4)+2i(+1) of a group, so
//     a lane reads each V code word exactly once and uses both nibbles of every byte.
// A tile that is processed alone (the odd last tile of a request, and every tile of a request of
// at most four tiles) carries p*scale_v and p*min_v as an exact fp16 (high, low) pair: with a
// handful of tokens nothing averages the rounding of that product.
//
// The steady state - pairs of complete tiles, ring full, a refill behind every tile - is a loop of
// its own without per-tile case analysis; the ends of a run, ragged tails, unmapped pages and
// short requests take a general loop that computes the same values.  The per-lane shared-memory
// offsets of the MMA layouts are kept in registers as opaque values (keep_in_register): left as
// expressions of the lane index they are recomputed inside the tile loop.
#include <math_constants.h>

#include <type_traits>

#include <cuda.h>

#include <algorithm>
#include <climits>
#include <mutex>
#include <vector>

#include "bkv_decode_common.cuh"
#include "bkv_mma_ptx.cuh"
#include "bkv_stream_partition.h"

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
constexpr uint32_t kBoundAddr = kRingHi + kHiSlots * kSlotBytes;  // int64[CTAs + 1]: where every CTA's share begins
constexpr int kMaxCtas = (kPrefixAddr - kBoundAddr) / 8 - 1;
static_assert(kMaxCtas >= 148, "the share boundaries of a full B200 grid fit behind the ring");
constexpr uint32_t kFullBar = kSmemBase;          // 8 B each
constexpr uint32_t kChunkTot = kSmemBase + 512;   // int[32] scan scratch
constexpr uint32_t kPendList = kSmemBase + 640;   // int[64]: cut requests whose last part a warp of this CTA wrote
constexpr uint32_t kPendCount = kSmemBase + 896;  // int: entries of the list
constexpr uint32_t kPendCta = kSmemBase + 960;    // int[2]: the same for the CTA as a whole, one per phase (-1: none)
constexpr uint32_t kLevels = kSmemBase + 1280;    // fp16 [K|V][4][16]
constexpr int kTableBarIndex = 63;               // the last of the 64 barrier words: byte tables landed
constexpr int kMaxCounters = 1 << 20;            // virtual heads x batch of one launch (see launch_variant)

struct StreamParams {
  DecodeParams d;
  float* ws_o;   // [slots][4][128]
  float* ws_m;   // [slots][4]  log2 domain
  float* ws_l;   // [slots][4]
  int* ws_cnt;   // [virtual heads * batch] tiles of a cut request that have been turned into partials;
                 // zero between launches (the warp that completes a count puts it back to zero)
  int* ws_prefix;  // [batch + 1] tiles before request b, written by stream_prefix_kernel when batch > kMaxBatch
  const uint32_t* byte_tables;  // optional [heads_kv][2][256][64]: the two table blocks of every head, ready to copy
  int quads;     // query-head quads per kv head
  int aligned;   // 1: every CTA's share lies inside one head (heads get floor or ceil of C / heads CTAs)
  int straddle_tiles;  // equal shares: tiles by which a share that straddles two heads is shortened
  int q_vec;           // 16-bit queries whose rows can be read in 8-byte pieces
};

// Tensor copies of the packed cache.  A page is two halves of the same shape - K codes + K
// statistics | V codes + V statistics - so the cache is described as uint8
// [page][half][64-byte row][64]: one copy with a box of two halves brings the K and the V
// rows of a tile in together.  The V statistics of pages longer than one tile are group-major
// and get a view of their own: [page][head*4+group][tile of the page][64].
__device__ __forceinline__ void tensor_copy_4d(uint32_t dst, const CUtensorMap* map, int c1, int c2, int c3,
                                               uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(map), "r"(0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
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

// 16 consecutive floats of a result row, rounded to the output type
__device__ __forceinline__ void store_out16(void* out, int64_t idx, int dtype, const float (&v)[16]) {
  if (dtype == BKV_F32) {
    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(out) + idx);
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    return;
  }
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t lo2 = dtype == BKV_BF16 ? f32_to_bf16_bits(v[2 * i]) : f32_to_f16_bits(v[2 * i]);
    const uint32_t hi2 = dtype == BKV_BF16 ? f32_to_bf16_bits(v[2 * i + 1]) : f32_to_f16_bits(v[2 * i + 1]);
    w[i] = lo2 | (hi2 << 16);
  }
  uint4* dst = reinterpret_cast<uint4*>(static_cast<unsigned short*>(out) + idx);
  dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
  dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
}

// Where the merged result of a cut request goes.  Everything is passed BY VALUE to the
// (deliberately not inlined) merge routine: handing it a reference to the kernel's parameter
// block would force that block into local memory for the whole kernel.
struct MergeIo {
  const int64_t* bounds;  // shared memory: tile at which the share of CTA c begins, c = 0 .. CTAs
  const float* ws_o;  // partial slots [slot][4][128], [slot][4], [slot][4]
  const float* ws_m;
  const float* ws_l;
  float* stage;       // not null: the caller's [4][128 | m | l] staging record in shared memory (CTA-level merge)
  void* out;          // else: final result rows ...
  float* out_f32;
  float* o_partial;   // ... or, with force_partial, un-normalised rows for a merge across ranks
  float* m_partial;
  float* l_partial;
  int out_dtype;
  int force_partial;
  int64_t row0;       // result row of query head 0 of the quad
  int nh;             // live query heads of the quad
};

// Log-sum-exp merge of parts of the cut request whose tiles are [pb, pe) of virtual head vh.
// Where the parts lie follows from the partition alone (bkv_stream_partition.h): lane i of the
// warp works out what CTA c0+i leaves, a scan numbers the parts, and the warp then loads them
// six at a time.  The calling warp takes the batches begin, begin+step, ...; lane l accumulates
// query head l>>3 of the quad, dimensions 16*(l&7) .. +15.  The partials were written by other
// SMs, so they are read from L2.
template <int NW>
__device__ __noinline__ void merge_parts(const MergeIo io, const part::Plan pl, const int vh, const int pb, const int pe,
                                         const int begin, const int step) {
  constexpr uint32_t kAll = 0xffffffffu;
  const int lane = threadIdx.x & 31;
  const int h = lane >> 3, dc = lane & 7;
  float M = -CUDART_INF_F, den = 0.f, num[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) num[i] = 0.f;
  constexpr int kBatch = 6;  // parts loaded at once (one L2 round trip)
  int batch = 0;
  const int64_t g0 = static_cast<int64_t>(vh) * pl.Tb + pb, g1 = static_cast<int64_t>(vh) * pl.Tb + pe;
  int c_lo, c_hi;
  part::ctas_near_head(pl, vh, &c_lo, &c_hi);  // the CTAs that can hold tiles of this head: usually one round of 32
  for (int c0 = c_lo; c0 <= c_hi; c0 += 32) {
    // which of these 32 CTAs hold tiles of the request at all: two loads and two compares per lane
    int64_t ga = 0, gb = 0;
    if (c0 + lane <= c_hi) {
      ga = io.bounds[c0 + lane];
      gb = io.bounds[c0 + lane + 1];
    }
    const bool meets = ga < g1 && gb > g0;
    if (!__any_sync(kAll, meets)) continue;
    part::CtaParts cp = {0u, 0, 0, 0};
    if (meets) cp = part::cta_parts<NW>(pl, ga, gb, vh, pb, pe);
    const int cnt = __popc(cp.mask);
    int incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(kAll, incl, o);
      if (lane >= o) incl += y;
    }
    const int total = __shfl_sync(kAll, incl, 31);
    const int pre = incl - cnt;  // parts of this round before those of this lane's CTA
    const uint32_t info = cp.mask | (static_cast<uint32_t>(cp.ph) << 16) | (static_cast<uint32_t>(cp.solo) << 17) |
                          (static_cast<uint32_t>(cp.starts) << 18);
    for (int j0 = 0; j0 < total; j0 += kBatch, ++batch) {
      if (batch < begin || (batch - begin) % step != 0) continue;
      float o2[kBatch][16], m2[kBatch], l2[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int j = j0 + u;
        m2[u] = 0.f;
        l2[u] = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) o2[u][i] = 0.f;
        if (j < total) {  // uniform over the warp
          const int owner = 31 - __clz(__ballot_sync(kAll, pre <= j));  // pre is non-decreasing over the lanes
          const uint32_t oi = __shfl_sync(kAll, info, owner);
          const int nth = j - __shfl_sync(kAll, pre, owner);  // which of the owner's parts
          uint32_t mk = oi & 0xFFFFu;
          for (int i = 0; i < nth; ++i) mk &= mk - 1;
          const int w = __ffs(mk) - 1;
          const bool solo = (oi >> 17) & 1u;
          const int starts = ((oi >> 18) & 1u) && nth == 0;
          const int64_t row = static_cast<int64_t>(part::part_slot(pl, c0 + owner, (oi >> 16) & 1, solo ? 0 : w, starts)) * 4 + h;
          m2[u] = __ldcg(io.ws_m + row);
          l2[u] = __ldcg(io.ws_l + row);
          const float4* src = reinterpret_cast<const float4*>(io.ws_o + row * kHeadDim + dc * 16);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 v = __ldcg(src + i);
            o2[u][4 * i] = v.x;
            o2[u][4 * i + 1] = v.y;
            o2[u][4 * i + 2] = v.z;
            o2[u][4 * i + 3] = v.w;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        if (!(l2[u] > 0.f)) continue;
        const float Mn = fmaxf(M, m2[u]);
        const float a = fast_exp2(M - Mn), wgt = fast_exp2(m2[u] - Mn);  // exp2(-inf) = 0: the first part
        den = den * a + l2[u] * wgt;
#pragma unroll
        for (int i = 0; i < 16; ++i) num[i] = num[i] * a + o2[u][i] * wgt;
        M = Mn;
      }
    }
  }
  if (io.stage) {  // one warp's share of a CTA-level merge: the CTA folds the warps' records
    float4* dst = reinterpret_cast<float4*>(io.stage + h * kHeadDim + dc * 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] = make_float4(num[4 * i], num[4 * i + 1], num[4 * i + 2], num[4 * i + 3]);
    if (dc == 0) {
      io.stage[4 * kHeadDim + h] = M;
      io.stage[4 * kHeadDim + 4 + h] = den;
    }
    return;
  }
  if (h >= io.nh) return;
  const int64_t row = io.row0 + h;
  if (io.force_partial) {
#pragma unroll
    for (int i = 0; i < 16; ++i) io.o_partial[row * kHeadDim + dc * 16 + i] = den > 0.f ? num[i] : 0.f;
    if (dc == 0) {
      io.m_partial[row] = den > 0.f ? M * kLn2 : -CUDART_INF_F;
      io.l_partial[row] = den;
    }
    return;
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) num[i] *= inv;
  store_out16(io.out, row * kHeadDim + dc * 16, io.out_dtype, num);
  if (io.out_f32) store_out16(io.out_f32, row * kHeadDim + dc * 16, BKV_F32, num);
}

// LOADER 1: every lane moves 16-byte pieces with cp.async, one commit group per tile.
// LOADER 3: an elected lane issues two (16-token pages) or three tensor copies
// (cp.async.bulk.tensor) per tile, completing on one mbarrier per ring stage; the copies bypass
// the load/store pipe.
template <int NW, int STAGES, bool STAT_BF16, int LOADER, int PAIR = 2>
__global__ void __maxnreg__(max_regs_for(NW))
    decode_stream_kernel(const StreamParams sp, const __grid_constant__ CUtensorMap map_code,
                         const __grid_constant__ CUtensorMap map_stat, const __grid_constant__ CUtensorMap map_vstat) {
  static_assert(STAGES >= 2 && STAGES <= 4, "a tile pair needs two stages; cp.async groups in flight are counted up to three");
  static_assert(NW * STAGES < kTableBarIndex, "the last barrier word belongs to the byte tables");
  static_assert(4 * NW <= 64, "every warp can be the last of two cut requests in each of the two phases");
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

  pdl_launch_dependents();  // a kernel launched as this grid's programmatic dependent may be set up now
  if (tid == 0) {
    for (int i = 0; i < NW * STAGES; ++i) mbar_init(kFullBar + 8 * i, 1);
    mbar_init(kFullBar + 8 * kTableBarIndex, 1);
    fence_barrier_init();
    reinterpret_cast<int*>(gptr(kPendCta))[0] = -1;
    reinterpret_cast<int*>(gptr(kPendCta))[1] = -1;
  }
  if (tid == 0) reinterpret_cast<int*>(gptr(kPendCount))[0] = 0;

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
  // (rebuilt where it is needed: nothing of it has to stay in registers through the tile loop)
  auto make_plan = [&] {
    part::Plan pl;
    pl.C = gridDim.x;
    pl.NW = NW;
    pl.hv = p.heads_kv * sp.quads;
    pl.Tb = prefix[p.batch];
    pl.aligned = sp.aligned;
    pl.gap = sp.straddle_tiles;
    return pl;
  };
  int64_t* const bounds = reinterpret_cast<int64_t*>(gptr(kBoundAddr));
  auto make_io = [&](float* stage, int64_t row0, int nh) {
    MergeIo io;
    io.bounds = bounds;
    io.ws_o = sp.ws_o;
    io.ws_m = sp.ws_m;
    io.ws_l = sp.ws_l;
    io.stage = stage;
    io.out = p.out;
    io.out_f32 = p.out_f32;
    io.o_partial = p.o_partial;
    io.m_partial = p.m_partial;
    io.l_partial = p.l_partial;
    io.out_dtype = p.out_dtype;
    io.force_partial = p.force_partial;
    io.row0 = row0;
    io.nh = nh;
    return io;
  };
  // where every CTA's share of the line begins (the merges at the end look the shares up here)
  for (int c = tid; c <= C; c += NW * 32) {
    int64_t a, e;
    part::share_of(make_plan(), min(c, C - 1), &a, &e);
    bounds[c] = c < C ? a : e;
  }
  __syncthreads();
  const int64_t ga = bounds[cta], gb = bounds[cta + 1];  // this CTA's share

  // ---- per-lane roles (see the file comment) ----------------------------------------------
  const int ksel = tig >> 1, khalf = tig & 1;     // QK: this lane's k-slots carry half khalf of group 2*ksel+P
  const int tq0 = gid;                            // QK rows gid / gid+8 carry tokens gid / gid+8
  uint32_t kc_off0 = swz(kSwKCode + tq0 * 64 + (2 * ksel) * 16) + khalf * 8;      // pair 0; +512: row gid+8
  uint32_t kc_off1 = swz(kSwKCode + tq0 * 64 + (2 * ksel + 1) * 16) + khalf * 8;  // pair 1
  uint32_t ks_off0 = swz(kSwKStat + tq0 * 16), ks_off1 = swz(kSwKStat + (tq0 + 8) * 16);
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
  uint32_t vs_off0 = swz(kSwVStat + (2 * gsel) * 64 + (tig + 8) * 4);
  uint32_t vs_off1 = swz(kSwVStat + (2 * gsel) * 64 + (tig + 4 + 8) * 4);
  uint32_t klane0 = kLutAddr | (lane * 4), klane1 = klane0 + kLutBlock;
  uint32_t vlane0 = kLutAddr | (lane * 4 + 128), vlane1 = vlane0 + kLutBlock;
  // probabilities travel from the QK layout (token by gid, head by tig) to the PV layout (token by tig, head by gid)
  const int src_lane0 = tig * 4 + hcol;        // row holding tokens tig, tig+8     (k-slots 2tig, 2tig+8)
  const int src_lane1 = (tig + 4) * 4 + hcol;  // row holding tokens tig+4, tig+12  (k-slots 2tig+1, 2tig+9)
  // These per-lane offsets are used by every tile.  Left as plain expressions of the lane index
  // the compiler recomputes them inside the tile loop (dozens of integer instructions per tile);
  // passed through an empty asm statement they are opaque values that stay in registers.
  keep_in_register(kc_off0), keep_in_register(kc_off1), keep_in_register(ks_off0), keep_in_register(ks_off1);
  keep_in_register(vc_off[0][0]), keep_in_register(vc_off[0][1]), keep_in_register(vc_off[1][0]), keep_in_register(vc_off[1][1]);
  keep_in_register(vs_off0), keep_in_register(vs_off1);
  keep_in_register(klane0), keep_in_register(klane1), keep_in_register(vlane0), keep_in_register(vlane1);

  // ---- ring state of this warp: tile number g of its lifetime lives in stage g % STAGES ----
  uint32_t ring_base = R::base(warp);
  keep_in_register(ring_base);
  const uint32_t bar_base = kFullBar + 8 * (warp * STAGES);
  int s = 0;           // stage of the next tile to consume
  uint32_t phase = 0;  // parity of that stage's current use
  int n_issued = 0, n_done = 0;
  uint32_t bad_mask = 0;  // bit s: the tile now in stage s maps to no page
  bool dead = false;      // a bounded wait gave up: stop working, keep walking to the barriers
  uint32_t table_parity = 0;

  const PageGeom geo = make_geom(BS, p.heads_kv);
  const uint32_t page_bytes = static_cast<uint32_t>(p.page_stride * 4);  // (a page is far below 4 GiB)
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
    const part::Span sh = part::phase_span(make_plan(), ga, gb, ph);
    const int vh = sh.vh, span = sh.span, first = sh.first;
    const int range = (cta * 2 + ph) * NW + warp;
    if (span == 0) continue;
    const int head = vh / quads, quad = vh - head * quads;
    const int hq0 = head * gqa + quad * 4;
    const int nh = min(4, gqa - quad * 4);

    // ---- this warp's run of tiles [wa, wb) inside the head ---------------------------------
    const int wa = part::run_begin(sh, NW, warp), wb = part::run_begin(sh, NW, warp + 1);
    const int total = wb - wa;
    const bool work = total > 0 && !dead;
    // The CTA's first head: nothing reads the table space yet, so the two bulk copies of its byte
    // tables are requested before the page ids and the first ring fill instead of behind them.
    if (ph == 0 && sp.byte_tables && tid == 0) {
      const uint32_t bar = kFullBar + 8 * kTableBarIndex;
      mbar_arrive_expect_tx(bar, 2 * kLutBlock);
      const char* const src = reinterpret_cast<const char*>(sp.byte_tables) + static_cast<int64_t>(head) * (2 * kLutBlock);
      bulk_copy_g2s(kLutAddr, src, kLutBlock, bar);
      bulk_copy_g2s(kLutAddr + kLutBlock, src + kLutBlock, kLutBlock, bar);
    }
    // this head's level tables: requested now, stored to shared memory after the first ring fill
    // has been issued, so the read overlaps the page-id read below
    float level_early = 0.f;
    if (tid < 128 && !sp.byte_tables) {
      const int which = tid >> 6, g = (tid >> 4) & 3, c = tid & 15;
      level_early = which ? load_v_level(p, head, g, c) : load_k_level(p, head, g, c);
    }

    // cp.async loader: lane l moves the l-th 16 bytes of each 512-byte half of the K and V
    // codes (tokens 0-7 / 8-15); lanes 0-15 move the K statistics, lanes 16-31 the V statistics
    const uint32_t code_head = head * (BS * kWordsPerHead) * 4;
    uint32_t ld_kcode = geo.k_code_off * 4 + code_head + lane * 16;
    uint32_t ld_vcode = geo.v_code_off * 4 + code_head + lane * 16;
    uint32_t ld_code_dst = swz(lane * 16);  // the swizzle repeats every 512 bytes
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
    keep_in_register(ld_kcode), keep_in_register(ld_vcode), keep_in_register(ld_code_dst);
    keep_in_register(ld_stat_src), keep_in_register(ld_stat_dst), keep_in_register(ld_stat_sub);
    // tensor-copy loader: 64-byte rows of the code and the statistic part inside each half of a page
    const int row_code = code_head >> 6;
    const int row_stat = ((geo.k_stat_off + head * (BS * 4)) * 4) >> 6;

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
    if (work) {  // the queries of the run's first request: under way while the tables are set up
      const int esize = p.q_dtype == BKV_F32 ? 4 : 2;
      const char* const fq = reinterpret_cast<const char*>(p.q) +
                             (static_cast<int64_t>(request_of(wa)) * p.q_batch_stride + static_cast<int64_t>(hq0) * kHeadDim) * esize;
      if (lane * 128 < nh * kHeadDim * esize) asm volatile("prefetch.global.L2 [%0];" ::"l"(fq + lane * 128));
    }
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
          const char* const page = reinterpret_cast<const char*>(p.cache) + static_cast<uint64_t>(phys) * page_bytes;
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
          // K and V codes in one copy: rows row_code.. of both halves of the page
          tensor_copy_4d(dst + kSwKCode, &map_code, row_code + sub * 16, 0, phys, bar);
          if (tiles_per_page == 1) {  // the statistics of both halves likewise
            tensor_copy_4d(dst + kSwKStat, &map_stat, row_stat, 0, phys, bar);
          } else {
            tensor_copy_4d(dst + kSwKStat, &map_stat, row_stat + sub * 4, 0, phys, bar);
            tensor_copy_4d(dst + kSwVStat, &map_vstat, sub, head * 4, phys, bar);
          }
        }
      }
      ++n_issued;
    };
    if (work) {  // first ring fill: in flight while the tables are set up
      int st = s;
      for (int j = 0; j < min(total, STAGES); ++j) {
        issue(j, st);
        st = st + 1 == STAGES ? 0 : st + 1;
      }
    }

    __syncthreads();  // the previous head's tables are no longer read
    if (sp.byte_tables) {
      // the two table blocks of this head were laid out once per layer: two bulk copies
      const uint32_t bar = kFullBar + 8 * kTableBarIndex;
      if (tid == 0 && ph != 0) {
        fence_proxy_async();  // the reads of the old tables before the writes of the copy unit
        mbar_arrive_expect_tx(bar, 2 * kLutBlock);
        const char* const src = reinterpret_cast<const char*>(sp.byte_tables) + static_cast<int64_t>(head) * (2 * kLutBlock);
        bulk_copy_g2s(kLutAddr, src, kLutBlock, bar);
        bulk_copy_g2s(kLutAddr + kLutBlock, src + kLutBlock, kLutBlock, bar);
      }
      if (!wait_full(bar, table_parity)) dead = true;
      table_parity ^= 1u;
    } else {
      if (tid < 128) reinterpret_cast<__half*>(gptr(kLevels))[tid] = __float2half_rn(level_early);  // fp16 [K|V][4][16]
      __syncthreads();
      // byte -> (level[low nibble], level[high nibble]) tables, one copy per bank.
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
      __syncthreads();
    }

    // One request covers this CTA's whole share (few, long requests): the warps do not leave a
    // partial each; they merge in shared memory and the CTA leaves one, so a request's chain of
    // partials has one link per CTA instead of one per warp.  (CTA-uniform.)
    int solo_b = request_of(first);
    const bool solo = prefix[solo_b + 1] >= first + span;

    // ---- attention state of the request being streamed ------------------------------------
    uint32_t qb[2][4][2];  // B operand of QK: q of head hcol as fp16 (exact for 16-bit queries)
    float qs[4];           // sum over the dims of group g of the fp16 q of head tig (bf16 statistics)
    uint32_t qmin_b[2];    // fp16 statistics: B operand that multiplies the K minima by those sums
    float oacc[2][4][4], cmin[2][4];
    float m_used = -CUDART_INF_F, l_run = 0.f;  // head tig

    // `before_second` runs before the first read of the second tile (its wait), `after_reads(t)`
    // after the last read of tile t from the ring (its stage is refilled while its V part is
    // still being multiplied): the tile that was issued last gets the most time to arrive.
    auto process = [&](auto nt_tag, auto partial_tag, const uint32_t sbA, const uint32_t sbB, const int nvA,
                       const int nvB, auto&& before_second, auto&& after_reads) {
      constexpr int NT = decltype(nt_tag)::value;
      constexpr bool PARTIAL = decltype(partial_tag)::value;
      constexpr bool PRECISE = NT == 1;  // p*scale_v and p*min_v as exact (high, low) fp16 pairs
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
        // statistic words (scale low, minimum high) of groups 0..3 for tokens gid (s0) and gid+8 (s1)
        const uint4 s0 = ring_load128i<0>(sb[t] + ks_off0), s1 = ring_load128i<0>(sb[t] + ks_off1);
        float mm[4] = {0.f, 0.f, 0.f, 0.f};
        if (!STAT_BF16) {
          // fp16 minima go to the tensor cores as they are: sum_g min[token][g] * qsum[g][head] is one
          // more MMA.  A = the high halves of the words (in every lane: groups 0,1 in k-slots 2tig..,
          // groups 2,3 in k-slots 2tig+8..; B is zero outside the k rows of lane 0), B = the sums as
          // (high, low) fp16 parts in columns 2*head, 2*head+1; the two columns are added below.
          mma16816_zero(mm, __byte_perm(s0.x, s0.y, 0x7632), __byte_perm(s1.x, s1.y, 0x7632), __byte_perm(s0.z, s0.w, 0x7632),
                        __byte_perm(s1.z, s1.w, 0x7632), qmin_b[0], qmin_b[1]);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const uint4 st = r ? s1 : s0;
          float u, v;  // column 2tig of an accumulator: group P, column 2tig+1: group P+2
          if (!STAT_BF16) {
            u = fmaf(f16_bits_to_f32(st.x & 0xFFFFu), sacc[t][0][2 * r], mm[2 * r]);
            v = fmaf(f16_bits_to_f32(st.y & 0xFFFFu), sacc[t][1][2 * r], mm[2 * r + 1]);
            u = fmaf(f16_bits_to_f32(st.z & 0xFFFFu), sacc[t][0][2 * r + 1], u);
            v = fmaf(f16_bits_to_f32(st.w & 0xFFFFu), sacc[t][1][2 * r + 1], v);
          } else {
            const float2 g0 = stat_word_to_f32<true>(st.x), g1 = stat_word_to_f32<true>(st.y);
            const float2 g2 = stat_word_to_f32<true>(st.z), g3 = stat_word_to_f32<true>(st.w);
            u = g0.x * sacc[t][0][2 * r];
            v = g1.x * sacc[t][1][2 * r];
            u = fmaf(g2.x, sacc[t][0][2 * r + 1], u);
            v = fmaf(g3.x, sacc[t][1][2 * r + 1], v);
            u = fmaf(g0.y, qs[0], u);
            v = fmaf(g1.y, qs[1], v);
            u = fmaf(g2.y, qs[2], u);
            v = fmaf(g3.y, qs[3], v);
          }
          float x = u + v;
          if (PARTIAL) {  // behind the end of the sequence (statistics may be NaN)
            if (tq0 + 8 * r >= nv[t]) x = -CUDART_INF_F;
          }
          sc[t][r] = x;
        }
      }
      // ------------------------------ online softmax over the tile(s) -------------------------
      // (the scores are still un-scaled; the scale is positive, so the maximum commutes with it)
      // Most tiles leave the running maximum alone: every lane tests its own scores against it,
      // and only when some lane of the warp is beyond the threshold are the maxima of the heads
      // reduced over the lanes (the same decision per head as reducing first).
      float tmax = fmaxf(sc[0][0], sc[0][1]);
      if (NT == 2) tmax = fmaxf(tmax, fmaxf(sc[NT - 1][0], sc[NT - 1][1]));
      if (__any_sync(kFull, tmax * p.scale_log2 > m_used + kRescaleThreshold)) {
        tmax = fmaxf(tmax, __shfl_xor_sync(kFull, tmax, 4));
        tmax = fmaxf(tmax, __shfl_xor_sync(kFull, tmax, 8));
        tmax = fmaxf(tmax, __shfl_xor_sync(kFull, tmax, 16));
        tmax *= p.scale_log2;
        const bool need = tmax > m_used + kRescaleThreshold;
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
        const float e0 = fast_exp2(fmaf(sc[t][0], p.scale_log2, -m_used)), e1 = fast_exp2(fmaf(sc[t][1], p.scale_log2, -m_used));
        const uint32_t mine = pack_half2(e0, e1);  // head tig: (token gid, token gid+8)
        // the denominator sums what the PV product will use: the rounding of p cancels in o / l
        const float2 er = __half22float2(*reinterpret_cast<const __half2*>(&mine));
        l_run += er.x + er.y;
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
        uint32_t wl2[2][2], ml2[2][2];  // PRECISE: what the fp16 rounding of the two products dropped
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
            uint32_t wl = 0u, ml = 0u;
            if (PRECISE) {  // p*s - round(p*s) is exact in fp16 (a fused multiply-add rounds once)
              wl = hfma2_u32(ph2[t][o], sc2, wv ^ 0x80008000u);
              ml = hfma2_u32(ph2[t][o], mn2, mv ^ 0x80008000u);
            }
            if (PARTIAL) {  // 0 * NaN would poison the accumulators
              const uint32_t keep = (tig + 8 * o < nv[t] ? 0x0000FFFFu : 0u) | (tig + 4 + 8 * o < nv[t] ? 0xFFFF0000u : 0u);
              wv &= keep;
              mv &= keep;
              wl &= keep;
              ml &= keep;
            }
            wb2[P][o] = wv;
            mb2[P][o] = mv;
            wl2[P][o] = wl;
            ml2[P][o] = ml;
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
          if (PRECISE) {
#pragma unroll
            for (int i = 0; i < 4; ++i) mma16816(oacc[P][i], av[i][0], av[i][1], av[i][2], av[i][3], wl2[P][0], wl2[P][1]);
            mma16816(cmin[P], ones, ones, ones, ones, ml2[P][0], ml2[P][1]);
          }
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
        float qsum[2] = {0.f, 0.f};
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
                f[i] = live_h ? v : 0.f;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i) f[i] = live_h ? load_q(p.q, qoff + d0 + i, p.q_dtype) : 0.f;
            }
            const uint32_t lo2 = pack_half2(f[0], f[1]), hi2 = pack_half2(f[2], f[3]);
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo2));
            const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&hi2));
            qsum[P] += (a.x + a.y) + (c.x + c.y);
            qb[P][j][0] = ksel == gsel ? lo2 : 0u;  // the other group of the pair meets zeros
            qb[P][j][1] = ksel == gsel ? hi2 : 0u;
          }
#pragma unroll
        for (int P = 0; P < 2; ++P) {
          qsum[P] += __shfl_xor_sync(kFull, qsum[P], 1);  // both halves of the group
#pragma unroll
          for (int e = 0; e < 2; ++e) qs[2 * e + P] = __shfl_sync(kFull, qsum[P], (2 * tig) * 4 + 2 * e);
        }
        if (!STAT_BF16) {
          // this lane holds the sums of groups 2*ksel, 2*ksel+1 of head hcol; lane (gid, 0) gathers all four
          const float g2s = __shfl_sync(kFull, qsum[0], gid * 4 + 2), g3s = __shfl_sync(kFull, qsum[1], gid * 4 + 2);
          const float four[4] = {qsum[0], qsum[1], g2s, g3s};
          float part[4];
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const float hi = __half2float(__float2half_rn(four[g]));
            part[g] = (gid & 1) ? four[g] - hi : hi;  // column 2*head: high part, 2*head+1: what it dropped
          }
          qmin_b[0] = tig == 0 ? pack_half2(part[0], part[1]) : 0u;
          qmin_b[1] = tig == 0 ? pack_half2(part[2], part[3]) : 0u;
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

      if (x + (kend - k0) < wb && b + 1 < B) {  // the next request's queries: on their way to L2 meanwhile
        const int esize = p.q_dtype == BKV_F32 ? 4 : 2;
        const char* const nq = reinterpret_cast<const char*>(p.q) +
                               (static_cast<int64_t>(b + 1) * p.q_batch_stride + static_cast<int64_t>(hq0) * kHeadDim) * esize;
        if (lane * 128 < nh * kHeadDim * esize) asm volatile("prefetch.global.L2 [%0];" ::"l"(nq + lane * 128));
      }
      int k = k0;
      // ---- steady state: pairs of complete tiles with the ring full and a refill behind each ----
      // (no per-tile case analysis: the conditions below are checked once per pair, and everything
      // that fails them - the ends of a run, ragged tails, unmapped pages, short requests - takes
      // the general loop further down, which computes the same values for complete tiles)
      if (PAIR == 2 && nb > 4) {
        const int k_fast = min(kend, ntok / kTile);  // complete tiles of this part
        while (k + 2 <= k_fast && run_done + 2 + STAGES <= total && bad_mask == 0 && n_issued - n_done == STAGES && !dead) {
          const int sB = s + 1 == STAGES ? 0 : s + 1;
          const uint32_t phaseB = s + 1 == STAGES ? phase ^ 1u : phase;
          if (LOADER == 1) {
            cp_async_wait_group<STAGES - 1>();
            __syncwarp();
          } else if (!wait_full(bar_base + 8 * s, phase)) {
            dead = true;
            break;
          }
          process(std::integral_constant<int, 2>{}, std::false_type{}, ring_base + s * kSlotBytes, ring_base + sB * kSlotBytes,
                  kTile, kTile,
                  [&] {
                    if (LOADER == 1) {
                      cp_async_wait_group<STAGES - 2>();
                      __syncwarp();
                    } else if (!wait_full(bar_base + 8 * sB, phaseB)) {
                      dead = true;
                    }
                  },
                  [&](int t) {
                    __syncwarp();
                    if (LOADER != 1) fence_proxy_async();  // reads of the generic proxy before writes of the async proxy
                    issue(run_done + t + STAGES, t ? sB : s);
                  });
          if (dead) break;
          k += 2;
          run_done += 2;
          n_done += 2;
          s = sB + 1 == STAGES ? 0 : sB + 1;
          phase = sB + 1 == STAGES ? phaseB ^ 1u : phaseB;
        }
      }
      for (; k < kend;) {
        // a request of a few tiles is processed one tile at a time, i.e. by the precise form
        const int cnt = nb <= 4 ? 1 : min(PAIR, kend - k);
        const int sB = s + 1 == STAGES ? 0 : s + 1;
        const uint32_t phaseB = s + 1 == STAGES ? phase ^ 1u : phase;
        auto wait_tile = [&](auto ahead_tag, int stage, uint32_t parity) {  // tile n_done + ahead of this warp
          constexpr int kAhead = decltype(ahead_tag)::value;
          const int in_flight = n_issued - n_done;  // tiles issued and not yet consumed
          if (in_flight <= kAhead) return;
          if (LOADER == 1) {
            // this thread's pieces of the tile: with a full ring the newer STAGES - 1 - kAhead groups may
            // still be under way; near the end of a run simply everything is awaited ...
            if (in_flight == STAGES) cp_async_wait_group<STAGES - 1 - kAhead>();
            else cp_async_wait_group<0>();
            __syncwarp();  // ... and every other lane's
          } else if (!wait_full(bar_base + 8 * stage, parity)) {
            dead = true;
          }
        };
        auto refill = [&](int ahead, int stage) {  // the stage of tile n_done + ahead is free again
          __syncwarp();
          if (LOADER != 1) fence_proxy_async();  // reads of the generic proxy before writes of the async proxy
          if (run_done + ahead + STAGES < total) issue(run_done + ahead + STAGES, stage);
        };
        wait_tile(std::integral_constant<int, 0>{}, s, phase);
        if (dead) break;
        const int rem = ntok - kTile * k;
        const int nvA = (bad_mask >> s) & 1 ? 0 : min(kTile, rem);
        const int nvB = cnt == 2 ? ((bad_mask >> sB) & 1 ? 0 : min(kTile, rem - kTile)) : 0;
        const uint32_t sbA = ring_base + s * kSlotBytes, sbB = ring_base + sB * kSlotBytes;
        auto wait_second = [&] { wait_tile(std::integral_constant<int, 1>{}, sB, phaseB); };
        auto refill_tile = [&](int t) { refill(t, t ? sB : s); };
        if (cnt == 2) {
          if (nvA > 0 || nvB > 0) {
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
      if (!whole) {
        // This part is in place: count its tiles.  The warp whose tiles complete the request merges
        // all its parts (its own included) and writes the result; the others just go on.
        // (the warp's barrier orders every lane's stores before lane 0's fence: one fence, not thirty-two)
        __syncwarp();
        if (lane == 0) {
          __threadfence();
          int* const cnt_b = sp.ws_cnt + (static_cast<int64_t>(vh) * B + b);
          if (atomicAdd(cnt_b, kend - k0) + (kend - k0) == nb) {
            *cnt_b = 0;  // nobody else touches it any more: ready for the next launch
            // the merge itself waits until the CTA has streamed all its tiles and is then dealt to
            // whichever warp is next (at most two cut requests per warp and phase end up here): no
            // call, and nothing a call would clobber, in this loop
            const int at = atomicAdd(reinterpret_cast<int*>(gptr(kPendCount)), 1);
            reinterpret_cast<int*>(gptr(kPendList))[at] = vh * B + b;
          }
        }
      }
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
      const int pb = prefix[solo_b], pe = prefix[solo_b + 1];
      const int k0c = first - pb;
      const bool whole = k0c == 0 && first + span == pe;
      const int slot = 2 * ((cta * 2 + ph) * NW) + (k0c > 0 ? 0 : 1);  // of the CTA's first range
      // fold the NW records in shared memory; `final`: the result is the request's, else this CTA's part
      auto fold = [&](const bool final) {
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
          if (!final) {
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
      };
      fold(whole);
      if (!whole) {
        // count this CTA's tiles; the CTA that completes the request merges its parts, every warp
        // taking every NW-th batch of four, and folds the NW results like above
        __syncthreads();  // orders every thread's stores before thread 0's fence
        if (tid == 0) {
          __threadfence();
          int* const cnt_b = sp.ws_cnt + (static_cast<int64_t>(vh) * B + solo_b);
          if (atomicAdd(cnt_b, span) + span == pe - pb) {
            *cnt_b = 0;
            reinterpret_cast<int*>(gptr(kPendCta))[ph] = vh * B + solo_b;  // merged by all warps at the end
          }
        }
      }
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

  // ---- the cut requests this warp / this CTA was the last to finish -------------------------
  // Every part of them is in the workspace by now (their counters were complete).  The tile loop is
  // over, so the call clobbers nothing that matters and the ring space is free.
  {
    const int hvq = quads;
    __syncthreads();  // every warp is through with its tiles: the list is complete, the ring space is free
    const int n_pend = reinterpret_cast<const int*>(gptr(kPendCount))[0];
    for (int e = warp; e < n_pend; e += NW) {
      const int item = reinterpret_cast<const int*>(gptr(kPendList))[e];
      const int vh = item / B, b = item - vh * B;
      const int head = vh / hvq, quad = vh - head * hvq;
      merge_parts<NW>(make_io(nullptr, static_cast<int64_t>(b) * p.heads_q + head * gqa + quad * 4, min(4, gqa - quad * 4)),
                      make_plan(), vh, prefix[b], prefix[b + 1], 0, 1);
    }
    for (int ph = 0; ph < 2; ++ph) {
      const int item = reinterpret_cast<const int*>(gptr(kPendCta))[ph];
      if (item < 0) continue;  // uniform over the CTA
      const int vh = item / B, b = item - vh * B;
      const int head = vh / hvq, quad = vh - head * hvq;
      const int hq0 = head * gqa + quad * 4, nh = min(4, gqa - quad * 4);
      // every warp merges every NW-th batch of four parts into a record o | m | l of its own ...
      float* const rec = reinterpret_cast<float*>(gptr(kRingLoS));
      constexpr int kRec = 4 * kHeadDim + 8;
      __syncthreads();
      merge_parts<NW>(make_io(rec + warp * kRec, 0, nh), make_plan(), vh, prefix[b], prefix[b + 1], warp, NW);
      __syncthreads();
      // ... and the CTA folds the NW records
      for (int idx = tid; idx < 4 * kHeadDim; idx += NW * 32) {
        const int h = idx >> 7, d = idx & (kHeadDim - 1);
        if (h >= nh) continue;
        float M = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < NW; ++w)
          if (rec[w * kRec + 4 * kHeadDim + 4 + h] > 0.f) M = fmaxf(M, rec[w * kRec + 4 * kHeadDim + h]);
        float den = 0.f, num = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          const float lw = rec[w * kRec + 4 * kHeadDim + 4 + h];
          if (!(lw > 0.f)) continue;
          const float wt = exp2f(rec[w * kRec + 4 * kHeadDim + h] - M);
          den += wt * lw;
          num += wt * rec[w * kRec + h * kHeadDim + d];
        }
        const int64_t row = static_cast<int64_t>(b) * p.heads_q + hq0 + h;
        if (p.force_partial) {
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

constexpr int64_t kPartialBytes = 4 * kHeadDim * 4 + 16 + 16;  // o, m, l of four heads
constexpr int64_t kPlannedPrefixBytes = (kMaxBatchPlanned + 64) * 4;  // a multiple of 256
constexpr int64_t kCounterBytes = static_cast<int64_t>(kMaxCounters) * 4;
constexpr int kStreamWarps = 12, kStreamStages = 3;

// Byte tables of every kv head in the layout the decode kernel keeps in shared memory: block P
// (P = 0, 1) of a head is 256 rows (one per code byte) of 64 words; word l < 32 of a row is
// (level[low nibble], level[high nibble]) of the K group lane l uses in the QK MMAs of pair P,
// word 32 + l the same for the V group lane l uses in the PV MMAs.
__global__ void __launch_bounds__(256) build_byte_tables_kernel(const DecodeParams p, uint32_t* __restrict__ out) {
  __shared__ unsigned short lv[128];  // fp16 [K|V][4][16]
  const int head = blockIdx.x, tid = threadIdx.x;
  if (tid < 128) {
    const int which = tid >> 6, g = (tid >> 4) & 3, c = tid & 15;
    lv[tid] = __half_as_ushort(__float2half_rn(which ? load_v_level(p, head, g, c) : load_k_level(p, head, g, c)));
  }
  __syncthreads();
  uint32_t* const dst = out + static_cast<int64_t>(head) * (2 * kLutBlock / 4);
  for (int e = tid; e < 2 * 256 * 64; e += 256) {
    const int P = e >> 14, byte = (e >> 6) & 255, word = e & 63, l = word & 31;
    const int g = word < 32 ? 2 * ((l >> 1) & 1) + P : 2 * (l >> 4) + P;
    const unsigned short* t = lv + (word < 32 ? 0 : 64) + g * 16;
    dst[e] = t[byte & 15] | (static_cast<uint32_t>(t[byte >> 4]) << 16);
  }
}

// ---- tensor maps of the packed cache ------------------------------------------------------------
// uint8 [page][half][64-byte row][64] with the 64-byte swizzle; a box is `rows` rows of `halves`
// halves of one page.  Maps are cached per (cache, geometry).
struct CacheMaps {
  CUtensorMap code, stat, vstat;
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

bool make_half_map(CUtensorMap* out, const DecodeParams& p, int rows, int halves) {
  const EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return false;
  const PageGeom geo = make_geom(p.block_size, p.heads_kv);
  const cuuint64_t half_bytes = static_cast<cuuint64_t>(geo.block_i32) * 2;  // K codes + K statistics
  const cuuint64_t dims[4] = {64, half_bytes / 64, 2, static_cast<cuuint64_t>(p.num_pages)};
  const cuuint64_t strides[3] = {64, half_bytes, static_cast<cuuint64_t>(p.page_stride) * 4};
  const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(rows), static_cast<cuuint32_t>(halves), 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<uint32_t*>(p.cache), dims, strides, box, estr,
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

// false: the driver offers no tensor maps for this cache
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
  const bool one_tile_pages = p.block_size == kTile;
  // half a page must be a whole number of 64-byte rows and start on a 16-byte boundary
  e.ok = (p.page_stride * 4) % 64 == 0 && (static_cast<int64_t>(p.heads_kv) * p.block_size) % 4 == 0 &&
         make_half_map(&e.maps.code, p, 16, 2) && make_half_map(&e.maps.stat, p, 4, one_tile_pages ? 2 : 1) &&
         make_vstat_map(&e.maps.vstat, p);
  *out = e.maps;
  return e.ok;
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

// grid size and share policy of a launch: the same numbers on the host (launch, self-test) and,
// through StreamParams, on the device
void plan_launch(int hv, int batch, int max_seq_len, int sm_count, part::Plan* pl) {
  const int NW = kStreamWarps;
  const int64_t tiles_max = static_cast<int64_t>(hv) * batch * ((max_seq_len + kTile - 1) / kTile);
  int64_t ctas = (tiles_max + 2 * NW - 1) / (2 * NW);
  if (ctas < hv) ctas = hv;  // a share never spans more than two heads
  if (ctas > sm_count) ctas = sm_count;
  const int C = static_cast<int>(ctas);
  // Equal shares make the CTAs whose share straddles two heads set up twice and restart their
  // pipelines (a few us, which the share computation takes off their tile count); head-aligned
  // shares avoid that but the heads served by fewer CTAs finish later.  Take the cheaper of the
  // two estimates (0.1 us per tile and SM).
  const int base = C / hv;
  const double per_cta_us = static_cast<double>(tiles_max) / C * 0.1;
  const double aligned_loss_us = per_cta_us * (static_cast<double>(C) / hv / base - 1.0);
  // A CTA whose share straddles two heads drains its rings, waits for its warps, brings in the
  // second head's 128 KiB of tables and restarts its pipelines: about 12 us, i.e. the time of 160
  // tiles, by which its share is shortened (per-CTA time stamps on batch 64 x 8 K: with 40 the four
  // straddling CTAs finished 7 us behind the median and set the end of the kernel; 160 to 250
  // measure alike, 149 against 155 us per step).  Compensated equal shares lose about
  // (heads - 1) such gaps spread over all CTAs.
  constexpr int kStraddleTiles = 160;
  const double equal_loss_us = 0.08 * kStraddleTiles * (hv - 1) / C + 1.0;
  pl->C = C;
  pl->NW = NW;
  pl->hv = hv;
  pl->Tb = 0;  // known on the device only
  pl->gap = kStraddleTiles;
  pl->aligned = (C % hv == 0 || aligned_loss_us < equal_loss_us) ? 1 : 0;
}

template <int LOADER>
int launch_variant(const DecodeParams& p, void* ws, int64_t ws_bytes, const void* byte_tables, int max_seq_len,
                   int sm_count, cudaStream_t stream) {
  constexpr int NW = kStreamWarps, STAGES = kStreamStages;
  using R = Ring<NW, STAGES>;
  StreamParams sp;
  sp.d = p;
  const int gqa = p.heads_q / p.heads_kv;
  sp.quads = (gqa + 3) / 4;
  sp.q_vec = (p.q_dtype == BKV_BF16 || p.q_dtype == BKV_F16) && reinterpret_cast<uintptr_t>(p.q) % 8 == 0 &&
             p.q_batch_stride % 4 == 0;
  const int hv = p.heads_kv * sp.quads;
  if (hv > sm_count || sm_count > kMaxCtas) return BKV_ERR_UNSUPPORTED;
  if (static_cast<int64_t>(hv) * p.batch > kMaxCounters) return BKV_ERR_UNSUPPORTED;
  part::Plan pl;
  plan_launch(hv, p.batch, max_seq_len, sm_count, &pl);
  const int C = pl.C;
  sp.aligned = pl.aligned;
  sp.straddle_tiles = pl.gap;
  sp.byte_tables = static_cast<const uint32_t*>(byte_tables);
  const int64_t slots = 2ll * C * 2 * NW;
  if (!ws || ws_bytes < kPlannedPrefixBytes + kCounterBytes + slots * kPartialBytes) return BKV_ERR_ARG;
  char* w = static_cast<char*>(ws);  // the prefix sums come first, then the counters, then the partials
  sp.ws_prefix = reinterpret_cast<int*>(w);
  sp.ws_cnt = reinterpret_cast<int*>(w + kPlannedPrefixBytes);
  w += kPlannedPrefixBytes + kCounterBytes;
  sp.ws_o = reinterpret_cast<float*>(w);
  sp.ws_m = reinterpret_cast<float*>(w + slots * (4 * kHeadDim * 4));
  sp.ws_l = sp.ws_m + slots * 4;
  if (p.batch > kMaxBatch) {
    stream_prefix_kernel<<<1, 1024, 0, stream>>>(p, sp.ws_prefix);
    const int rcp = check_launch("bkv_decode_stream_sm100(prefix)");
    if (rcp != BKV_OK) return rcp;
  }

  CacheMaps maps = {};
  if (LOADER == 3 && !cache_maps_for(p, &maps)) return BKV_ERR_UNSUPPORTED;
  auto kern = p.stat_bf16 ? decode_stream_kernel<NW, STAGES, true, LOADER> : decode_stream_kernel<NW, STAGES, false, LOADER>;
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
    // the planning kernel asks for the same shared-memory carve-out, so the SMs are not
    // reconfigured between the launches of a step
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
    const cudaError_t de = cudaLaunchKernelEx(&dcfg, kern, sp, maps.code, maps.stat, maps.vstat);
    if (de != cudaSuccess) {
      set_last_cuda_error(de, "bkv_decode_stream_sm100(decode, dependent launch)");
      return BKV_ERR_CUDA;
    }
  } else {
    kern<<<C, NW * 32, R::kDynBytes, stream>>>(sp, maps.code, maps.stat, maps.vstat);
  }
  return check_launch("bkv_decode_stream_sm100(decode)");
}

}  // namespace

int64_t stream_workspace_bytes() {
  const int64_t sms = device_sm_count();
  // the prefix sums, the request counters, then two slots for each of the 2 * warps ranges of a CTA
  return kPlannedPrefixBytes + kCounterBytes + sms * 2 * kStreamWarps * 2 * kPartialBytes;
}

int init_stream_workspace(void* ws, int64_t ws_bytes, cudaStream_t stream) {
  if (!ws || ws_bytes < kPlannedPrefixBytes + kCounterBytes) return BKV_ERR_ARG;
  const cudaError_t e = cudaMemsetAsync(static_cast<char*>(ws) + kPlannedPrefixBytes, 0, kCounterBytes, stream);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "bkv_decode_stream_workspace_init");
    return BKV_ERR_CUDA;
  }
  return BKV_OK;
}

int64_t byte_table_bytes(int heads_kv) { return static_cast<int64_t>(heads_kv) * 2 * kLutBlock; }

int launch_build_byte_tables(const DecodeParams& p, void* out, cudaStream_t stream) {
  if (!aligned16(out)) return BKV_ERR_ALIGN;
  build_byte_tables_kernel<<<p.heads_kv, 256, 0, stream>>>(p, static_cast<uint32_t*>(out));
  return check_launch("bkv_decode_tables_sm100");
}

int launch_decode_stream(const DecodeParams& p, void* ws, int64_t ws_bytes, const void* byte_tables, int max_seq_len,
                         cudaStream_t stream, int config) {
  const int r = p.block_size / kTile;
  if (p.block_size % kTile != 0 || (r & (r - 1)) != 0 || p.block_size > 1024) return BKV_ERR_UNSUPPORTED;
  if ((p.page_stride * 4) % 16 != 0 || !aligned16(p.cache)) return BKV_ERR_UNSUPPORTED;
  if (p.page_stride * 4 >= (1ll << 32)) return BKV_ERR_UNSUPPORTED;  // the kernel multiplies page ids by a 32-bit stride
  if (p.token_lo % p.block_size != 0) return BKV_ERR_UNSUPPORTED;
  if (p.batch > kMaxBatchPlanned || p.num_pages > (1ll << kMaxPagesLog2)) return BKV_ERR_UNSUPPORTED;
  // the byte tables hold fp16 levels: 16-bit level tables convert exactly, float32 ones would be rounded
  if (p.table_dtype == BKV_F32) return BKV_ERR_UNSUPPORTED;
  if (byte_tables && !aligned16(byte_tables)) return BKV_ERR_ALIGN;
  // merged results leave in 16-byte pieces; the partials are read back in 16-byte pieces
  if (!aligned16(ws) || (p.out && !aligned16(p.out)) || (p.out_f32 && !aligned16(p.out_f32))) return BKV_ERR_ALIGN;
  const int sms = device_sm_count();
  if (sms <= 0) return BKV_ERR_CUDA;
  if (config == 1) return launch_variant<3>(p, ws, ws_bytes, byte_tables, max_seq_len, sms, stream);
  return launch_variant<1>(p, ws, ws_bytes, byte_tables, max_seq_len, sms, stream);
}

// Host-side check of the work partition (no device access): for `batch` requests of the given tile
// counts, walk every warp's run exactly as the kernel does, note which slot every part of every cut
// request goes to, and compare that with the list the merging warp derives.  Returns the number of
// requests whose lists differ, or -1 for unusable arguments.
int check_partition(const int* tiles, int batch, int hv, int sm_count, int max_tiles_per_request) {
  if (!tiles || batch <= 0 || hv <= 0 || sm_count < hv || max_tiles_per_request <= 0) return -1;
  part::Plan pl;
  plan_launch(hv, batch, max_tiles_per_request * kTile, sm_count, &pl);
  std::vector<int64_t> prefix(batch + 1, 0);
  for (int b = 0; b < batch; ++b) {
    if (tiles[b] < 0 || tiles[b] > max_tiles_per_request) return -1;
    prefix[b + 1] = prefix[b] + tiles[b];
  }
  if (prefix[batch] > INT32_MAX) return -1;
  pl.Tb = static_cast<int>(prefix[batch]);
  // what the kernel writes: (virtual head, request) -> slots, tiles counted
  std::vector<std::vector<int>> written(static_cast<size_t>(hv) * batch);
  std::vector<int64_t> counted(static_cast<size_t>(hv) * batch, 0);
  int64_t covered = 0;
  for (int c = 0; c < pl.C; ++c) {
    int64_t ga, gb;
    part::share_of(pl, c, &ga, &gb);
    covered += gb - ga;
    for (int ph = 0; ph < 2; ++ph) {
      const part::Span s = part::phase_span(pl, ga, gb, ph);
      if (s.span == 0) continue;
      if (s.vh >= hv) return -1;
      auto request_of = [&](int x) {
        int l = 0, h = batch;
        while (h - l > 1) {
          const int mid = (l + h) >> 1;
          if (prefix[mid] <= x) l = mid; else h = mid;
        }
        return l;
      };
      const int solo_b = request_of(s.first);
      if (prefix[solo_b + 1] >= s.first + s.span) {  // one partial for the CTA
        const bool whole = s.first == prefix[solo_b] && s.first + s.span == prefix[solo_b + 1];
        if (!whole) {
          written[static_cast<size_t>(s.vh) * batch + solo_b].push_back(2 * ((c * 2 + ph) * pl.NW) + (s.first > prefix[solo_b] ? 0 : 1));
          counted[static_cast<size_t>(s.vh) * batch + solo_b] += s.span;
        }
        continue;
      }
      for (int w = 0; w < pl.NW; ++w) {
        const int wa = part::run_begin(s, pl.NW, w), wb = part::run_begin(s, pl.NW, w + 1);
        int x = wa;
        int b = wb > wa ? request_of(wa) : 0;
        while (x < wb) {
          while (prefix[b + 1] <= x) ++b;
          const int pb = static_cast<int>(prefix[b]), nb = static_cast<int>(prefix[b + 1] - prefix[b]);
          const int k0 = x - pb, kend = std::min(nb, wb - pb);
          if (!(k0 == 0 && kend == nb)) {
            written[static_cast<size_t>(s.vh) * batch + b].push_back(2 * ((c * 2 + ph) * pl.NW + w) + (k0 > 0 ? 0 : 1));
            counted[static_cast<size_t>(s.vh) * batch + b] += kend - k0;
          }
          x += kend - k0;
        }
      }
    }
  }
  int bad = covered == static_cast<int64_t>(hv) * pl.Tb ? 0 : 1;
  for (int vh = 0; vh < hv; ++vh)
    for (int b = 0; b < batch; ++b) {
      const std::vector<int>& w = written[static_cast<size_t>(vh) * batch + b];
      if (w.empty()) continue;
      const int pb = static_cast<int>(prefix[b]), pe = static_cast<int>(prefix[b + 1]);
      std::vector<int> derived;
      int c_lo, c_hi;
      part::ctas_near_head(pl, vh, &c_lo, &c_hi);
      for (int c = c_lo; c <= c_hi; ++c) {
        int64_t sa, sb;
        part::share_of(pl, c, &sa, &sb);
        const part::CtaParts cp = part::cta_parts(pl, sa, sb, vh, pb, pe);
        bool first_of_cta = true;
        for (int wi = 0; wi < pl.NW; ++wi) {
          if (!((cp.mask >> wi) & 1u)) continue;
          derived.push_back(part::part_slot(pl, c, cp.ph, cp.solo ? 0 : wi, cp.starts && first_of_cta));
          first_of_cta = false;
        }
      }
      if (derived != w || counted[static_cast<size_t>(vh) * batch + b] != pe - pb) ++bad;
    }
  return bad;
}

int read_stream_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_stream_status, sizeof(int));
  const int zero = 0;
  cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int));
  return v;
}

}  // namespace bkv
