// W4A16 prefill GEMM on tcgen05 tensor cores (placeholder until the kernel lands).
#pragma once
#include "common.cuh"
namespace lcq {
namespace gemm_tc {
inline bool supported(int, int, int, int, int, int) { return false; }
inline size_t workspace_bytes(int, int, int) { return 0; }
inline int launch(const void*, const void*, const void*, void*, int, int, int, int, int, void*, size_t, int,
                  cudaStream_t) {
  set_error("GEMM_TC is not built");
  return LCQ_ERR_UNSUPPORTED;
}
}  // namespace gemm_tc
}  // namespace lcq
