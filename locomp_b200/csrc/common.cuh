// Shared device/host helpers for the locomp_b200 kernels (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/locomp_b200.h"

namespace lcq {

// ------------------------------------------------------------------ host-side error plumbing
void set_error(const char* fmt, ...);          // stores a thread-local message (defined in lib.cu)
int cuda_fail(cudaError_t e, const char* what); // stores the message, returns LCQ_ERR_CUDA

#define LCQ_CUDA_TRY(expr)                                            \
  do {                                                                \
    cudaError_t _e = (expr);                                          \
    if (_e != cudaSuccess) return ::lcq::cuda_fail(_e, #expr);        \
  } while (0)

// Every workspace starts with this many bytes of counters that must be zero between calls;
// whatever follows is scratch that calls may leave dirty.
constexpr size_t kWorkspaceCounterBytes = 512 * 1024;

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Device status word: set to a non-zero code by a kernel whose bounded wait expired.
// Defined here because the library is one translation unit (no relocatable device code).
__device__ int g_device_status = 0;

// Programmatic dependent launch can be switched off with LCQ_NO_PDL=1 (read once).
inline bool pdl_enabled() {
  static const bool on = [] { const char* e = getenv("LCQ_NO_PDL"); return !(e && e[0] == '1'); }();
  return on;
}

// ------------------------------------------------------------------ dtype helpers
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// float(q) for an integer 0 <= q < 2^23 without an int->float conversion instruction.
__device__ __forceinline__ float small_uint_to_f32(uint32_t q) {
  return __uint_as_float(0x4B000000u | q) - 8388608.0f;
}

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: returns false (and the caller must unwind) if the phase does not complete
// within the wait limit (two seconds of wall-clock time unless lcq_set_wait_limit_ns changed
// it).  try_wait itself suspends the thread for a hardware-defined interval, so the loop is
// not a hot spin; the limit is read from device memory only on the slow path.
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ unsigned long long g_wait_limit_ns = 2000000000ull;
__device__ __forceinline__ uint64_t wait_limit_ns() { return *reinterpret_cast<volatile unsigned long long*>(&g_wait_limit_ns); }
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  const uint64_t limit = wait_limit_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (global_timer_ns() - t0 > limit) return false;
  }
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// 2-D tiled TMA load (no multicast): global -> shared::cta, completion on an mbarrier.
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tmap, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// Programmatic dependent launch (no-ops when the kernel was launched without the attribute).
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// D(16x8,f32) = A(16x16,f16,row) * B(16x8,f16,col) + C
__device__ __forceinline__ void mma_m16n8k16_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                  uint32_t b0, uint32_t b1, const float (&c)[4]) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// Four float zeros the optimiser cannot see through: kept live in one register quad, they can
// be fed to an MMA as its C operand without being re-materialised before every use.
__device__ __forceinline__ void opaque_zero4(float (&z)[4]) {
  asm volatile("mov.f32 %0, 0f00000000;\n\tmov.f32 %1, 0f00000000;\n\tmov.f32 %2, 0f00000000;\n\tmov.f32 %3, 0f00000000;"
               : "=f"(z[0]), "=f"(z[1]), "=f"(z[2]), "=f"(z[3]));
}

// ------------------------------------------------------------------ tensor-map encoding (host)
// Encodes a 2-D row-major tensor map through the driver entry point obtained at run time,
// so the library has no link-time dependency on libcuda.
int encode_tmap_2d(void* out_map /*CUtensorMap, 128 B*/, int dtype_code /*0=u8,1=f16,2=bf16*/,
                   const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                   uint32_t box_inner, uint32_t box_outer, int swizzle_code /*0 none,1=32B,2=64B,3=128B*/);

}  // namespace lcq
