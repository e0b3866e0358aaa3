// Weight quantisers: float weights -> packed int4 (or int8) + per-group float32 scales, with the
// reference's arithmetic reproduced bit for bit.
//
// Reference behaviour (Zyora-Dev/locomp v1.0.0), all in float32:
//   style 0  examples/38_quantized_matmul.py:248-271 (quantize_int4), :274-293 (quantize_int8)
//            amax  = max |w| over the group
//            scale = amax / 7  (int8: / 127), or 1.0 when the group is all zero
//            q     = clip(rint(w / scale) + 8, 0, 15)          (int8: clip(rint(w / scale), -128, 127))
//   style 1  examples/52_dequantize.py:110-126 (quantize_int4_ref), :162-165 (int8 self-check)
//            amax  = max(max |w|, 1e-10)   (int8: no floor)
//            scale = amax / 7  (int8: / 127)
//            q     = clip(rint(w / (scale + 1e-10)) + 8, 0, 15)
//   packing  byte j of a row = q[2j] | q[2j+1] << 4  (low nibble = even k)
// rint is round-half-to-even (np.round); both divisions are IEEE float32 divisions.
//
// Streaming kernel, HBM-bound: 4 B read per weight (float32 input), 0.5 B + 4/G B written.
// One thread owns 8 consecutive weights (one packed 32-bit word); the G/8 threads of a group
// combine their maxima with warp shuffles, so loads are 32 B per thread and stores 4 B per
// thread, both coalesced.  Group sizes that are not 8, 16, 32, 64, 128 or 256 take a generic
// kernel with one thread per group.
#pragma once
#include "common.cuh"
#include "gemv_simt.cuh"

namespace lcq {
namespace quant {

__device__ __forceinline__ float group_scale(float amax, float qmax, int style, int wbits) {
  if (style == 0) return amax > 0.0f ? __fdiv_rn(amax, qmax) : 1.0f;
  if (wbits == 4) amax = fmaxf(amax, 1e-10f);
  return __fdiv_rn(amax, qmax);
}
__device__ __forceinline__ float group_denom(float scale, int style) {
  return style == 0 ? scale : __fadd_rn(scale, 1e-10f);
}
__device__ __forceinline__ uint32_t q4(float w, float denom) {
  const float r = rintf(__fdiv_rn(w, denom)) + 8.0f;
  return static_cast<uint32_t>(fminf(fmaxf(r, 0.0f), 15.0f));
}
__device__ __forceinline__ int q8(float w, float denom) {
  const float r = rintf(__fdiv_rn(w, denom));
  return static_cast<int>(fminf(fmaxf(r, -128.0f), 127.0f));
}

// Fast path: G in {8, ..., 256} (a power of two), K % 8 == 0, rows 16-byte aligned.
// total_oct = N*K/8 octets; octet e belongs to group e / (G/8).
template <typename XT, int WBITS>
__global__ void __launch_bounds__(256) quantize_octets_kernel(const XT* __restrict__ w, uint8_t* __restrict__ q,
                                                              float* __restrict__ scales, long long total_oct,
                                                              int lanes_per_group, int style) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  // whole warps iterate together so the shuffles below are convergent
  const long long n_iter = (total_oct + stride - 1) / stride;
  long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (long long it = 0; it < n_iter; ++it, e += stride) {
    const bool ok = e < total_oct;
    float v[8];
    if (ok) load8<XT>(w + e * 8, v);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    for (int off = 1; off < lanes_per_group; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float scale = group_scale(amax, WBITS == 4 ? 7.0f : 127.0f, style, WBITS);
    const float denom = group_denom(scale, style);
    if (!ok) continue;
    if ((e % lanes_per_group) == 0) scales[e / lanes_per_group] = scale;
    if (WBITS == 4) {
      uint32_t word = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) word |= q4(v[i], denom) << (4 * i);
      reinterpret_cast<uint32_t*>(q)[e] = word;
    } else {
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        lo |= (static_cast<uint32_t>(q8(v[i], denom)) & 0xFFu) << (8 * i);
        hi |= (static_cast<uint32_t>(q8(v[4 + i], denom)) & 0xFFu) << (8 * i);
      }
      reinterpret_cast<uint2*>(q)[e] = make_uint2(lo, hi);
    }
  }
}

// Generic path: one thread per group, any G dividing K (G even for int4).
template <typename XT, int WBITS>
__global__ void __launch_bounds__(256) quantize_groups_kernel(const XT* __restrict__ w, uint8_t* __restrict__ q,
                                                              float* __restrict__ scales, long long total_groups,
                                                              int G, int style) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long g = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; g < total_groups; g += stride) {
    const XT* src = w + g * G;
    float amax = 0.0f;
    for (int i = 0; i < G; ++i) amax = fmaxf(amax, fabsf(to_f32<XT>(src[i])));
    const float scale = group_scale(amax, WBITS == 4 ? 7.0f : 127.0f, style, WBITS);
    const float denom = group_denom(scale, style);
    scales[g] = scale;
    if (WBITS == 4) {
      uint8_t* dst = q + g * (G / 2);
      for (int i = 0; i < G; i += 2)
        dst[i / 2] = static_cast<uint8_t>(q4(to_f32<XT>(src[i]), denom) | (q4(to_f32<XT>(src[i + 1]), denom) << 4));
    } else {
      int8_t* dst = reinterpret_cast<int8_t*>(q) + g * G;
      for (int i = 0; i < G; ++i) dst[i] = static_cast<int8_t>(q8(to_f32<XT>(src[i]), denom));
    }
  }
}

template <typename XT, int WBITS>
int launch_quantize(const void* w, void* q, void* scales, long long N, long long K, int G, int style, int sm_count,
                    cudaStream_t st) {
  const long long total = N * K;
  if (total == 0) return LCQ_OK;
  const bool pow2 = G >= 8 && G <= 256 && (G & (G - 1)) == 0;
  const bool fast = pow2 && aligned(w, 16) && aligned(q, 8) && ((K * sizeof(XT)) % 16 == 0);
  if (fast) {
    const long long oct = total / 8;
    long long blocks = (oct + 255) / 256;
    if (blocks > static_cast<long long>(sm_count) * 16) blocks = static_cast<long long>(sm_count) * 16;
    quantize_octets_kernel<XT, WBITS><<<static_cast<int>(blocks), 256, 0, st>>>(
        static_cast<const XT*>(w), static_cast<uint8_t*>(q), static_cast<float*>(scales), oct, G / 8, style);
  } else {
    const long long groups = total / G;
    long long blocks = (groups + 255) / 256;
    if (blocks > static_cast<long long>(sm_count) * 16) blocks = static_cast<long long>(sm_count) * 16;
    quantize_groups_kernel<XT, WBITS><<<static_cast<int>(blocks), 256, 0, st>>>(
        static_cast<const XT*>(w), static_cast<uint8_t*>(q), static_cast<float*>(scales), groups, G, style);
  }
  LCQ_CUDA_TRY(cudaGetLastError());
  return LCQ_OK;
}

}  // namespace quant
}  // namespace lcq
