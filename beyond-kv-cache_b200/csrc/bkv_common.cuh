// Shared helpers for the sm_100a packed-KV kernels: page geometry, 16-bit
// conversions with explicit rounding, small PTX wrappers and launch-error capture.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/bkv_sm100.h"

namespace bkv {

constexpr int kHeadDim = 128;
constexpr int kGroup = 32;
constexpr int kGroupsPerHead = kHeadDim / kGroup;  // 4
constexpr int kWordsPerHead = kHeadDim / 8;        // 16 code words per (token, head)

// Word offsets of the four regions of one page (reference PagedLayout.build,
// quant/beyond_cute.py:708-734, expressed in int32 words instead of halves).
struct PageGeom {
  int block_size;
  int heads;
  int k_code_off;
  int k_stat_off;
  int v_code_off;
  int v_stat_off;
  int block_i32;
};

__host__ __device__ inline PageGeom make_geom(int block_size, int heads) {
  PageGeom g;
  g.block_size = block_size;
  g.heads = heads;
  const int code_words = heads * block_size * kWordsPerHead;
  const int stat_words = heads * block_size * kGroupsPerHead;
  g.k_code_off = 0;
  g.k_stat_off = code_words;
  g.v_code_off = code_words + stat_words;
  g.v_stat_off = 2 * code_words + stat_words;
  g.block_i32 = 2 * code_words + 2 * stat_words;
  return g;
}

// ---- 16-bit <-> float32 -------------------------------------------------------
__device__ __forceinline__ float f16_bits_to_f32(uint32_t bits) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(bits)));
}
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits) {
  return __uint_as_float(bits << 16);
}
__device__ __forceinline__ float stat_bits_to_f32(uint32_t bits, bool bf16) {
  return bf16 ? bf16_bits_to_f32(bits & 0xFFFFu) : f16_bits_to_f32(bits & 0xFFFFu);
}
__device__ __forceinline__ uint32_t f32_to_f16_bits(float x) {
  return static_cast<uint32_t>(__half_as_ushort(__float2half_rn(x)));
}
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float x) {
  return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(x)));
}
__device__ __forceinline__ uint32_t f32_to_stat_bits(float x, bool bf16) {
  return bf16 ? f32_to_bf16_bits(x) : f32_to_f16_bits(x);
}

// Table element (levels / thresholds) of dtype BKV_F16 / BKV_BF16 / BKV_F32 -> float32.
__device__ __forceinline__ float load_table_f32(const void* base, int idx, int dtype) {
  if (dtype == BKV_F32) return static_cast<const float*>(base)[idx];
  const uint32_t bits = static_cast<const unsigned short*>(base)[idx];
  return dtype == BKV_BF16 ? bf16_bits_to_f32(bits) : f16_bits_to_f32(bits);
}

// an ordinary load through a shared-memory window address
__device__ __forceinline__ float shared_f32(uint32_t addr) {
  return *static_cast<const float*>(__cvta_shared_to_generic(addr));
}
__device__ __forceinline__ uint32_t shared_u32(uint32_t addr) {
  return *static_cast<const uint32_t*>(__cvta_shared_to_generic(addr));
}

// ---- PTX wrappers -------------------------------------------------------------
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- host side ----------------------------------------------------------------
void set_last_cuda_error(cudaError_t e, const char* where);
int check_launch(const char* where);  // returns BKV_OK or BKV_ERR_CUDA

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace bkv
