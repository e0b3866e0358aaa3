// Streaming dequantize kernels: packed int4 / int8 weights -> f32 / f16 / bf16.
//
// Reference behaviour: examples/52_dequantize.py:27-53 (int4) and :60-74 (int8):
//   out[r, 2j]   = (float(b & 15) - 8) * scales[r, 2j / G]
//   out[r, 2j+1] = (float(b >> 4) - 8) * scales[r, (2j+1) / G]
// Because K % G == 0, the scale of flat element e = r*K + k is scales_flat[e / G], so the
// fast paths index everything flat and never need the row.
//
// HBM-bound (write dominated: 4 B out per 0.5 B in for f32).  The fast int4 path reads one
// 32-bit word per lane (128 B per warp, coalesced), redistributes nibbles with two warp
// shuffles so that every store instruction writes 32 x 16 B = 512 contiguous bytes.
#pragma once
#include "common.cuh"

namespace lcq {

template <typename OT> struct Out4;   // 4 consecutive outputs, one vector store
template <> struct Out4<float> {
  static __device__ __forceinline__ void store(float* p, float a, float b, float c, float d) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(a, b, c, d));
  }
};
template <> struct Out4<__half> {
  static __device__ __forceinline__ void store(__half* p, float a, float b, float c, float d) {
    __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
    uint2 v = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    __stcs(reinterpret_cast<uint2*>(p), v);
  }
};
template <> struct Out4<__nv_bfloat16> {
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    __stcs(reinterpret_cast<uint2*>(p), v);
  }
};

// Index of the scale of flat element e: a shift when G is a power of two (gshift >= 0), else a division.
__device__ __forceinline__ long long scale_index(long long e, int G, int gshift) {
  return gshift >= 0 ? (e >> gshift) : (e / G);
}

template <typename OT> struct Out8;   // 8 consecutive 16-bit outputs, one 16-byte store
template <> struct Out8<__half> {
  static __device__ __forceinline__ void store(__half* p, const float (&f)[8]) {
    __half2 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(h));
  }
};
template <> struct Out8<__nv_bfloat16> {
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
    __nv_bfloat162 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(h));
  }
};

template <> struct Out8<float> {
  static __device__ __forceinline__ void store(float*, const float (&)[8]) {}   // never taken: float32 goes through Out4
};

// Independent 128-byte warp loads in flight per warp, as measured best on a 4096 x 14336 weight:
// int4 -> f32 4, int4 -> 16-bit 2, int8 1 (more only costs registers, hence resident blocks).
template <typename OT> __host__ __device__ constexpr int dq4_unroll() { return sizeof(OT) == 4 ? 4 : 2; }
constexpr int DQ8_UNROLL = 1;

// ---- int4 fast path: K % 8 == 0, G % 8 == 0, w 4-byte aligned, out 16-byte aligned.
// total_words = N*K/8.  A warp iteration covers dq4_unroll<OT>() blocks of 32 words (256 weights each): all
// loads of weights and scales are issued before the first store.  float32 output: two shuffles hand
// every lane 4 consecutive weights per store, so a store instruction writes 512 contiguous bytes.
// 16-bit output: a lane's own word is 8 outputs = 16 bytes, contiguous across the warp as it is.
template <typename ST, typename OT>
__global__ void __launch_bounds__(256) dequant_w4_words_kernel(const uint32_t* __restrict__ w,
                                                               const ST* __restrict__ scales,
                                                               OT* __restrict__ out,
                                                               long long total_words, int G, int gshift) {
  constexpr bool WIDE = sizeof(OT) == 4;
  constexpr int DQ_UNROLL = dq4_unroll<OT>();
  constexpr int NS = WIDE ? 2 : 1;              // stores (and scales) per lane and block
  const int lane = threadIdx.x & 31;
  const long long warp_id = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long n_blocks = (total_words + 31) >> 5;
  for (long long it = warp_id * DQ_UNROLL; it < n_blocks; it += n_warps * DQ_UNROLL) {
    uint32_t word[DQ_UNROLL];
    float sc[DQ_UNROLL][NS];
#pragma unroll
    for (int u = 0; u < DQ_UNROLL; ++u) {
      const long long wi = ((it + u) << 5) + lane;
      word[u] = (wi < total_words) ? __ldg(w + wi) : 0u;
#pragma unroll
      for (int j = 0; j < NS; ++j) {
        // WIDE: store j of lane l covers half (l & 1) of word 16j + l/2 of the block; else the lane's own word
        const long long src_word = WIDE ? (((it + u) << 5) + 16 * j + (lane >> 1)) : wi;
        const long long e0 = src_word * 8 + (WIDE ? 4 * (lane & 1) : 0);
        sc[u][j] = (src_word < total_words) ? to_f32<ST>(__ldg(scales + scale_index(e0, G, gshift))) : 0.0f;
      }
    }
#pragma unroll
    for (int u = 0; u < DQ_UNROLL; ++u) {
      if (WIDE) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint32_t wj = __shfl_sync(0xffffffffu, word[u], 16 * j + (lane >> 1));
          const long long src_word = ((it + u) << 5) + 16 * j + (lane >> 1);
          if (src_word < total_words) {
            const uint32_t nib = (wj >> (16 * (lane & 1))) & 0xFFFFu;
            const long long e0 = src_word * 8 + 4 * (lane & 1);
            const float s = sc[u][j];
            const float f0 = (small_uint_to_f32(nib & 15u) - 8.0f) * s;
            const float f1 = (small_uint_to_f32((nib >> 4) & 15u) - 8.0f) * s;
            const float f2 = (small_uint_to_f32((nib >> 8) & 15u) - 8.0f) * s;
            const float f3 = (small_uint_to_f32((nib >> 12) & 15u) - 8.0f) * s;
            Out4<OT>::store(out + e0, f0, f1, f2, f3);
          }
        }
      } else {
        const long long wi = ((it + u) << 5) + lane;
        if (wi < total_words) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = (small_uint_to_f32((word[u] >> (4 * i)) & 15u) - 8.0f) * sc[u][0];
          Out8<OT>::store(out + wi * 8, f);
        }
      }
    }
  }
}

// ---- int4 generic path: one thread per packed byte; any even K, any G dividing K.
template <typename ST, typename OT>
__global__ void __launch_bounds__(256) dequant_w4_bytes_kernel(const uint8_t* __restrict__ w,
                                                               const ST* __restrict__ scales,
                                                               OT* __restrict__ out,
                                                               long long total_bytes, int K, int G) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const int half_k = K >> 1, ns = K / G;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total_bytes; i += stride) {
    const long long r = i / half_k;
    const int j = static_cast<int>(i - r * half_k);
    const uint32_t b = __ldg(w + i);
    const int k0 = 2 * j, k1 = 2 * j + 1;
    const float s0 = to_f32<ST>(__ldg(scales + r * ns + k0 / G));
    const float s1 = to_f32<ST>(__ldg(scales + r * ns + k1 / G));
    out[r * K + k0] = from_f32<OT>((small_uint_to_f32(b & 15u) - 8.0f) * s0);
    out[r * K + k1] = from_f32<OT>((small_uint_to_f32(b >> 4) - 8.0f) * s1);
  }
}

// float(int8) for the 4 bytes of a word without conversion instructions.
__device__ __forceinline__ void int8x4_to_f32(uint32_t v, float (&f)[4]) {
  v ^= 0x80808080u;  // bias to unsigned: b + 128
  f[0] = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7540)) - 8388736.0f;
  f[1] = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7541)) - 8388736.0f;
  f[2] = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7542)) - 8388736.0f;
  f[3] = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7543)) - 8388736.0f;
}

// ---- int8 fast path: K % 4 == 0, G % 4 == 0; one 32-bit word (4 weights) per thread and load,
// DQ8_UNROLL loads in flight.
template <typename ST, typename OT>
__global__ void __launch_bounds__(256) dequant_w8_words_kernel(const uint32_t* __restrict__ w,
                                                               const ST* __restrict__ scales,
                                                               OT* __restrict__ out,
                                                               long long total_words, int G, int gshift) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total_words; i0 += stride * DQ8_UNROLL) {
    uint32_t word[DQ8_UNROLL];
    float sc[DQ8_UNROLL];
#pragma unroll
    for (int u = 0; u < DQ8_UNROLL; ++u) {
      const long long i = i0 + u * stride;
      const bool ok = i < total_words;
      word[u] = ok ? __ldg(w + i) : 0u;
      sc[u] = ok ? to_f32<ST>(__ldg(scales + scale_index(i * 4, G, gshift))) : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < DQ8_UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i < total_words) {
        float f[4];
        int8x4_to_f32(word[u], f);
        Out4<OT>::store(out + i * 4, f[0] * sc[u], f[1] * sc[u], f[2] * sc[u], f[3] * sc[u]);
      }
    }
  }
}

// ---- int8 generic path: one thread per weight.
template <typename ST, typename OT>
__global__ void __launch_bounds__(256) dequant_w8_elems_kernel(const int8_t* __restrict__ w,
                                                               const ST* __restrict__ scales,
                                                               OT* __restrict__ out,
                                                               long long total, int K, int G) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const int ns = K / G;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / K;
    const int k = static_cast<int>(i - r * K);
    const float sc = to_f32<ST>(__ldg(scales + r * ns + k / G));
    out[i] = from_f32<OT>(static_cast<float>(__ldg(w + i)) * sc);
  }
}

// Blocks of `kern` (256 threads, no dynamic shared memory) that are resident on the whole GPU at
// once: the grid-stride kernels are launched with exactly one wave, never more blocks than work.
template <auto kern>
int one_wave_grid(long long work_items, int per_block, int sm_count) {
  static thread_local int per_sm = 0;      // per (thread, kernel): the kernel is a template VALUE, not its type
  if (per_sm == 0) {
    int nb = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kern, 256, 0) != cudaSuccess || nb < 1) nb = 4;
    per_sm = nb;
  }
  long long need = (work_items + per_block - 1) / per_block;
  const long long cap = static_cast<long long>(sm_count) * per_sm;
  if (need < 1) need = 1;
  return static_cast<int>(need < cap ? need : cap);
}

template <typename ST, typename OT>
int launch_dequant(int wbits, const void* w, const void* scales, void* out, long long N, long long K, int G,
                   int sm_count, cudaStream_t stream) {
  const long long total = N * K;
  if (total == 0) return LCQ_OK;
  const size_t out_vec_align = 4 * sizeof(OT);
  int gshift = -1;
  if (G > 0 && (G & (G - 1)) == 0) { gshift = 0; while ((1 << gshift) < G) ++gshift; }
  if (wbits == 4) {
    const bool fast = (K % 8 == 0) && (G % 8 == 0) && aligned(w, 4) && aligned(out, 16);
    if (fast) {
      const long long words = total / 8;
      // 8 warps per block, each taking dq4_unroll<OT>() blocks of 32 words per iteration
      const int grid = one_wave_grid<dequant_w4_words_kernel<ST, OT>>((words + 31) / 32, 8 * dq4_unroll<OT>(), sm_count);
      dequant_w4_words_kernel<ST, OT><<<grid, 256, 0, stream>>>(
          static_cast<const uint32_t*>(w), static_cast<const ST*>(scales), static_cast<OT*>(out), words, G, gshift);
    } else {
      const long long bytes = total / 2;
      const int grid = one_wave_grid<dequant_w4_bytes_kernel<ST, OT>>(bytes, 256, sm_count);
      dequant_w4_bytes_kernel<ST, OT><<<grid, 256, 0, stream>>>(
          static_cast<const uint8_t*>(w), static_cast<const ST*>(scales), static_cast<OT*>(out), bytes,
          static_cast<int>(K), G);
    }
  } else {
    const bool fast = (K % 4 == 0) && (G % 4 == 0) && aligned(w, 4) && aligned(out, out_vec_align);
    if (fast) {
      const long long words = total / 4;
      const int grid = one_wave_grid<dequant_w8_words_kernel<ST, OT>>(words, 256 * DQ8_UNROLL, sm_count);
      dequant_w8_words_kernel<ST, OT><<<grid, 256, 0, stream>>>(
          static_cast<const uint32_t*>(w), static_cast<const ST*>(scales), static_cast<OT*>(out), words, G, gshift);
    } else {
      const int grid = one_wave_grid<dequant_w8_elems_kernel<ST, OT>>(total, 256, sm_count);
      dequant_w8_elems_kernel<ST, OT><<<grid, 256, 0, stream>>>(
          static_cast<const int8_t*>(w), static_cast<const ST*>(scales), static_cast<OT*>(out), total,
          static_cast<int>(K), G);
    }
  }
  LCQ_CUDA_TRY(cudaGetLastError());
  return LCQ_OK;
}

}  // namespace lcq
