// Exchange step of the KV-range split of one long sequence across GPUs, without a collective
// library on the data path.
//
// Every rank attends its own range of positions and is left with one record of un-normalised
// partials, o (rows x 128) | m (rows, natural log) | l (rows).  The ranks hold a receive buffer
// each, mapped into all the others through CUDA IPC: [2 parities][world][record] floats followed
// by [2][world] flag words and four control words (steps done, CTAs arrived, two unused).  ONE
// kernel per step then
//   1. pushes this rank's record into slot `rank` of every peer's buffer with plain peer stores
//      (CTA r writes to rank r, one peer at a time), makes it visible system-wide and publishes the
//      step number in the peer's flag word;
//   2. waits - with a time limit - until all `world` flags of its own buffer show this step;
//   3. merges the `world` records by log-sum-exp into the attention output, as
//      bkv_combine_packed_sm100 does.
// Buffers alternate with the parity of the step: a rank can only be one step ahead of a peer
// (its own step needs the peer's record), so a slot is never overwritten while it is read.
// Nothing spins without a limit: when the wait runs out the kernel records it in a status word,
// leaves the output alone and returns.
// The step number either comes from the caller (step > 0) or is kept in the rank's own buffer
// (step = 0): the launch is then the same every time, so a captured graph can replay it.  The CTA
// that is the last of its grid to finish writes the new count, after every CTA has read the old.
#include <math_constants.h>

#include <cstring>

#include "bkv_decode_common.cuh"

namespace bkv {
namespace {

constexpr int kMaxWorld = 16;

struct ExchangeParams {
  const float* record;        // this rank's record (device-local)
  int64_t record_floats;      // rows * 130
  float* peer_recv[kMaxWorld];  // base of every rank's receive buffer (own entry: local pointer)
  int world, rank;
  int64_t rows;
  int step;                   // > 0: the same on every rank, +1 per call; 0: counted in the rank's own buffer
  long long timeout_ns;
  void* out;
  int out_dtype;
  float* out_f32;
  int* status;                // device word, set to 1 when the wait ran out
};

__device__ __forceinline__ int load_flag(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store_flag(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__global__ void __launch_bounds__(kHeadDim) kv_exchange_merge_kernel(const ExchangeParams p) {
  __shared__ int s_ok, s_step;
  pdl_wait();  // launched while the range decode still drains: its record is complete from here on
  const int tid = threadIdx.x;
  const int64_t slot_floats = p.record_floats;
  const int64_t flags_at = 2 * static_cast<int64_t>(p.world) * slot_floats;  // floats before the flag words
  int* const control = reinterpret_cast<int*>(p.peer_recv[p.rank] + flags_at) + 2 * p.world;  // [steps done, CTAs arrived]
  if (tid == 0) s_step = p.step > 0 ? p.step : __ldcg(control) + 1;
  __syncthreads();
  const int step = s_step;
  const int parity = step & 1;
  // (step = 0) every CTA counts itself out; the last one publishes the step for the next launch
  auto leave = [&] {
    if (p.step > 0) return;
    __syncthreads();
    if (tid == 0 && atomicAdd(control + 1, 1) == static_cast<int>(gridDim.x) - 1) {
      control[1] = 0;
      __threadfence();
      atomicExch(control, step);
    }
  };
  // ---- 1. push: CTA r delivers this rank's record to rank r ---------------------------------
  for (int r = blockIdx.x; r < p.world; r += gridDim.x) {
    float* const dst = p.peer_recv[r] + (static_cast<int64_t>(parity) * p.world + p.rank) * slot_floats;
    const float4* const src4 = reinterpret_cast<const float4*>(p.record);
    float4* const dst4 = reinterpret_cast<float4*>(dst);
    // 16-byte pieces when every slot starts on a 16-byte boundary (rows * 130 floats: an even row count)
    const int64_t n4 = slot_floats % 4 == 0 ? slot_floats / 4 : 0;
    for (int64_t i = tid; i < n4; i += blockDim.x) dst4[i] = src4[i];
    for (int64_t i = n4 * 4 + tid; i < slot_floats; i += blockDim.x) dst[i] = p.record[i];
    __syncthreads();  // orders every thread's peer stores before the release (system scope) below
    if (tid == 0) {
      int* const flag = reinterpret_cast<int*>(p.peer_recv[r] + flags_at) + parity * p.world + p.rank;
      store_flag(flag, step);
    }
  }
  // ---- 2. wait for every rank's record of this step (bounded) -------------------------------
  const float* const mine = p.peer_recv[p.rank];
  const int* const flags = reinterpret_cast<const int*>(mine + flags_at) + parity * p.world;
  if (tid == 0) s_ok = 1;
  __syncthreads();
  if (tid < p.world) {
    const unsigned long long t0 = timer_ns();
    bool ok = load_flag(flags + tid) >= step;
    unsigned polls = 0;
    while (!ok) {
      ok = load_flag(flags + tid) >= step;
      if (!ok && (++polls & 63u) == 0 && timer_ns() - t0 > static_cast<unsigned long long>(p.timeout_ns)) break;
    }
    if (!ok) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) {
    if (tid == 0) atomicExch(p.status, 1);
    leave();
    return;
  }
  // ---- 3. merge the records (row = blockIdx.x, thread = dimension) --------------------------
  const float* const recs = mine + static_cast<int64_t>(parity) * p.world * slot_floats;
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    float M = -CUDART_INF_F;
    for (int s = 0; s < p.world; ++s) {
      const float* rec = recs + s * slot_floats;
      if (__ldcg(rec + p.rows * (kHeadDim + 1) + row) > 0.f) M = fmaxf(M, __ldcg(rec + p.rows * kHeadDim + row));
    }
    float den = 0.f, num = 0.f;
    for (int s = 0; s < p.world; ++s) {
      const float* rec = recs + s * slot_floats;
      const float ls = __ldcg(rec + p.rows * (kHeadDim + 1) + row);
      const float w = ls > 0.f ? __expf(__ldcg(rec + p.rows * kHeadDim + row) - M) : 0.f;
      den += w * ls;
      num += w * __ldcg(rec + row * kHeadDim + tid);
    }
    const float o = den > 0.f ? num / den : 0.f;
    store_out(p.out, row * kHeadDim + tid, p.out_dtype, o);
    if (p.out_f32) p.out_f32[row * kHeadDim + tid] = o;
  }
  leave();
}

}  // namespace
}  // namespace bkv

extern "C" int64_t bkv_kv_exchange_bytes(int world, int64_t rows) {
  if (world < 1 || world > bkv::kMaxWorld || rows < 0) return 0;
  const int64_t slot = rows * (bkv::kHeadDim + 2);
  return (2 * world * slot + 2 * world + 4) * 4;
}

extern "C" int bkv_kv_exchange_alloc(int64_t bytes, void** buffer_out, unsigned char* handle64_out) {
  if (bytes <= 0 || !buffer_out || !handle64_out) return BKV_ERR_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
  void* ptr = nullptr;
  cudaError_t e = cudaMalloc(&ptr, static_cast<size_t>(bytes));
  if (e == cudaSuccess) e = cudaMemset(ptr, 0, static_cast<size_t>(bytes));  // flags start at step 0
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) {
    bkv::set_last_cuda_error(e, "bkv_kv_exchange_alloc");
    if (ptr) cudaFree(ptr);
    return BKV_ERR_CUDA;
  }
  memcpy(handle64_out, &h, 64);
  *buffer_out = ptr;
  return BKV_OK;
}

extern "C" int bkv_kv_exchange_open(const unsigned char* handle64, void** peer_out) {
  if (!handle64 || !peer_out) return BKV_ERR_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* ptr = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    bkv::set_last_cuda_error(e, "bkv_kv_exchange_open");
    return BKV_ERR_CUDA;
  }
  *peer_out = ptr;
  return BKV_OK;
}

extern "C" int bkv_kv_exchange_close(void* peer) {
  if (!peer) return BKV_ERR_ARG;
  const cudaError_t e = cudaIpcCloseMemHandle(peer);
  if (e != cudaSuccess) {
    bkv::set_last_cuda_error(e, "bkv_kv_exchange_close");
    return BKV_ERR_CUDA;
  }
  return BKV_OK;
}

extern "C" int bkv_kv_exchange_free(void* buffer) {
  if (!buffer) return BKV_ERR_ARG;
  const cudaError_t e = cudaFree(buffer);
  if (e != cudaSuccess) {
    bkv::set_last_cuda_error(e, "bkv_kv_exchange_free");
    return BKV_ERR_CUDA;
  }
  return BKV_OK;
}

extern "C" int bkv_kv_exchange_merge_sm100(const float* record, int64_t rows, const uint64_t* peer_buffers, int world,
                                           int rank, int step, int64_t timeout_ns, void* out, int out_dtype,
                                           float* out_f32, int* status, bkv_stream_t stream) {
  using namespace bkv;
  if (!record || !peer_buffers || !out || !status) return BKV_ERR_ARG;
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || rows < 0 || step < 0 || timeout_ns <= 0) return BKV_ERR_ARG;
  if (out_dtype != BKV_F16 && out_dtype != BKV_BF16 && out_dtype != BKV_F32) return BKV_ERR_ARG;
  if (rows == 0) return BKV_OK;
  if (!aligned16(record)) return BKV_ERR_ALIGN;
  ExchangeParams p = {};
  p.record = record;
  p.record_floats = rows * (kHeadDim + 2);
  for (int r = 0; r < world; ++r) {
    p.peer_recv[r] = reinterpret_cast<float*>(peer_buffers[r]);
    if (!p.peer_recv[r] || !aligned16(p.peer_recv[r])) return BKV_ERR_ALIGN;
  }
  p.world = world; p.rank = rank; p.rows = rows; p.step = step; p.timeout_ns = timeout_ns;
  p.out = out; p.out_dtype = out_dtype; p.out_f32 = out_f32; p.status = status;
  int64_t ctas = rows > world ? rows : world;
  if (ctas > 128) ctas = 128;  // every CTA is resident: none of them waits for another CTA of this grid
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(ctas));
  cfg.blockDim = dim3(kHeadDim);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kv_exchange_merge_kernel, p);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "bkv_kv_exchange_merge_sm100");
    return BKV_ERR_CUDA;
  }
  return BKV_OK;
}
