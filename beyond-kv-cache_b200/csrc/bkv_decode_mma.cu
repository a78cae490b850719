// Tensor-core packed decode attention (sm_100a) — placeholder until the kernel lands.
#include "bkv_decode_common.cuh"

namespace bkv {

int launch_decode_mma(const DecodeParams&, cudaStream_t) { return BKV_ERR_UNSUPPORTED; }

}  // namespace bkv
