// Warp-per-row quantized matmul on CUDA cores: the general kernel (any K % G == 0, any
// dtype combination, float32 math end to end).  It is the path for the reference's own
// dtypes -- float32 x / scales / out, M = 1 (examples/38_quantized_matmul.py:30-134) --
// and the fallback for shapes the tensor-core kernels do not take.
//
//   out[m, n] = sum_k x[m, k] * wq(n, k) * scales[n, k / G]
//   wq = nibble - 8 (int4, low nibble = even k)  or  int8 value
//
// One warp owns one output row n and MT rows of x; lanes stride over K in chunks of 8
// weights (vector path) or single bytes (scalar path), accumulate in float32 and combine
// with a shuffle tree.  Within a chunk the scale is factored out of the 8 products.
#pragma once
#include "common.cuh"
#include "dequant.cuh"

namespace lcq {

template <typename XT> __device__ __forceinline__ void load8(const XT* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__half>(const __half* p, float (&v)[8]) {
  const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
  const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t* u = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(u[i] << 16);
    v[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
  }
}

template <int WBITS, typename XT, typename ST, typename OT, int MT, bool VEC>
__global__ void __launch_bounds__(256) gemv_simt_kernel(const XT* __restrict__ x, const uint8_t* __restrict__ w,
                                                        const ST* __restrict__ scales, OT* __restrict__ out,
                                                        int M, int N, int K, int G) {
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int m0 = blockIdx.y * MT;
  // Programmatic dependent launch.  Weights and scales are constants, so a lane fetches its first
  // chunk of them BEFORE waiting for the kernel ahead of it on the stream: that DRAM round trip then
  // runs under the other kernel's tail.  x (possibly that kernel's output) and out are touched only
  // after the wait.  A grid that fits on the machine at once lets the next kernel in right away
  // (its launch and its own weight prefetch then overlap this kernel entirely); a larger grid does so
  // only once its loads are issued, so that resident-but-waiting CTAs of the next kernel do not take
  // SM slots from this grid's later waves.
  const bool small_grid = gridDim.x * gridDim.y <= 296u;
  if (small_grid) griddep_launch_dependents();
  const bool row_ok = n < N;
  const int ns = K / G;
  const ST* srow = scales + static_cast<long long>(row_ok ? n : 0) * ns;
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0.0f;

  if (VEC) {
    // K % 8 == 0, G % 8 == 0, all rows 16-byte (x) / 4- or 8-byte (w) aligned.
    const int nchunks = K >> 3;
    const uint8_t* wrow8 = w + static_cast<long long>(row_ok ? n : 0) * (WBITS == 4 ? (K >> 1) : K);
    constexpr int PRE = 4;       // chunks per lane fetched ahead of the wait (K <= 1024 is covered whole)
    uint32_t pre_w0[PRE], pre_w1[PRE];
    float pre_sc[PRE];
#pragma unroll
    for (int j = 0; j < PRE; ++j) {
      const int c = lane + 32 * j;
      pre_w0[j] = 0u; pre_w1[j] = 0u; pre_sc[j] = 0.0f;
      if (row_ok && c < nchunks) {
        if (WBITS == 4) {
          pre_w0[j] = __ldg(reinterpret_cast<const uint32_t*>(wrow8) + c);
        } else {
          const uint2 two = __ldg(reinterpret_cast<const uint2*>(wrow8) + c);
          pre_w0[j] = two.x; pre_w1[j] = two.y;
        }
        pre_sc[j] = to_f32<ST>(__ldg(srow + (c << 3) / G));
      }
    }
    griddep_wait();
    if (!row_ok) { if (!small_grid) griddep_launch_dependents(); return; }
    auto chunk = [&](int c, uint32_t w0, uint32_t w1, float sc) {
      const int k0 = c << 3;
      float wq[8];
      if (WBITS == 4) {
#pragma unroll
        for (int i = 0; i < 8; ++i) wq[i] = small_uint_to_f32((w0 >> (4 * i)) & 15u) - 8.0f;
      } else {
        float f[4];
        int8x4_to_f32(w0, f); wq[0] = f[0]; wq[1] = f[1]; wq[2] = f[2]; wq[3] = f[3];
        int8x4_to_f32(w1, f); wq[4] = f[0]; wq[5] = f[1]; wq[6] = f[2]; wq[7] = f[3];
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m0 + m < M) {
          float xv[8];
          load8<XT>(x + static_cast<long long>(m0 + m) * K + k0, xv);
          float p = 0.0f;
#pragma unroll
          for (int i = 0; i < 8; ++i) p = fmaf(xv[i], wq[i], p);
          acc[m] = fmaf(sc, p, acc[m]);
        }
      }
    };
#pragma unroll
    for (int j = 0; j < PRE; ++j) {
      const int c = lane + 32 * j;
      if (c < nchunks) chunk(c, pre_w0[j], pre_w1[j], pre_sc[j]);
    }
#pragma unroll 4
    for (int c = lane + 32 * PRE; c < nchunks; c += 32) {
      uint32_t w0, w1 = 0u;
      if (WBITS == 4) {
        w0 = __ldg(reinterpret_cast<const uint32_t*>(wrow8) + c);
      } else {
        const uint2 two = __ldg(reinterpret_cast<const uint2*>(wrow8) + c);
        w0 = two.x; w1 = two.y;
      }
      chunk(c, w0, w1, to_f32<ST>(__ldg(srow + (c << 3) / G)));
    }
    if (!small_grid) griddep_launch_dependents();
  } else {
    griddep_wait();
    if (!small_grid) griddep_launch_dependents();
    if (!row_ok) return;
    if (WBITS == 4) {
      const uint8_t* wrow = w + static_cast<long long>(n) * (K >> 1);
      for (int j = lane; j < (K >> 1); j += 32) {
        const uint32_t b = __ldg(wrow + j);
        const int k0 = 2 * j, k1 = 2 * j + 1;
        const float w0 = (small_uint_to_f32(b & 15u) - 8.0f) * to_f32<ST>(__ldg(srow + k0 / G));
        const float w1 = (small_uint_to_f32(b >> 4) - 8.0f) * to_f32<ST>(__ldg(srow + k1 / G));
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if (m0 + m < M) {
            const XT* xr = x + static_cast<long long>(m0 + m) * K;
            acc[m] = fmaf(to_f32<XT>(xr[k0]), w0, acc[m]);
            acc[m] = fmaf(to_f32<XT>(xr[k1]), w1, acc[m]);
          }
        }
      }
    } else {
      const int8_t* wrow = reinterpret_cast<const int8_t*>(w) + static_cast<long long>(n) * K;
      for (int k = lane; k < K; k += 32) {
        const float wv = static_cast<float>(__ldg(wrow + k)) * to_f32<ST>(__ldg(srow + k / G));
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if (m0 + m < M) acc[m] = fmaf(to_f32<XT>(x[static_cast<long long>(m0 + m) * K + k]), wv, acc[m]);
        }
      }
    }
  }

#pragma unroll
  for (int m = 0; m < MT; ++m) {
    float v = acc[m];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if (lane == 0 && m0 + m < M) out[static_cast<long long>(m0 + m) * N + n] = from_f32<OT>(v);
  }
}

template <int WBITS, typename XT, typename ST, typename OT>
int launch_gemv_simt(const void* x, const void* w, const void* s, void* out, int M, int N, int K, int G,
                     cudaStream_t stream) {
  if (M == 0 || N == 0) return LCQ_OK;
  const bool vec = (K % 8 == 0) && (G % 8 == 0) && aligned(x, 16) && aligned(w, WBITS == 4 ? 4 : 8);
  const XT* xp = static_cast<const XT*>(x);
  const uint8_t* wp = static_cast<const uint8_t*>(w);
  const ST* sp = static_cast<const ST*>(s);
  OT* op = static_cast<OT*>(out);
  const int rows_per_block = 8;
  const unsigned gx = (N + rows_per_block - 1) / rows_per_block;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
#define LCQ_SIMT_LAUNCH(MT_, VEC_)                                                                   \
  do {                                                                                               \
    cfg.gridDim = dim3(gx, (M + MT_ - 1) / MT_);                                                     \
    LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_simt_kernel<WBITS, XT, ST, OT, MT_, VEC_>, xp, wp, sp, \
                                    op, M, N, K, G));                                                \
  } while (0)
  if (vec) {
    if (M == 1) LCQ_SIMT_LAUNCH(1, true);
    else if (M == 2) LCQ_SIMT_LAUNCH(2, true);
    else LCQ_SIMT_LAUNCH(4, true);
  } else {
    if (M == 1) LCQ_SIMT_LAUNCH(1, false);
    else LCQ_SIMT_LAUNCH(4, false);
  }
#undef LCQ_SIMT_LAUNCH
  return LCQ_OK;
}

}  // namespace lcq
