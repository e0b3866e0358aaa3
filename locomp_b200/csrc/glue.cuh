// Decode-step kernels on either side of the quantized linears: RMS norm, SiLU * up, residual
// add, the residual add fused with the following RMS norm, embedding lookup and greedy argmax.
//
// Reference behaviour (Zyora-Dev/locomp v1.0.0):
//   rms_norm      examples/54_smollm2_inference.py:40-73     o = x * rsqrt(mean(x^2) + eps) * w
//   silu_mul      examples/54_smollm2_inference.py:113-120   o = g * sigmoid(g) * u
//   add_inplace   examples/54_smollm2_inference.py:164-167   a += b
//   residual+norm examples/34_fused_residual_norm.py:18-60   h = r + x ; o = rms_norm(h) * w
//   embed_lookup  locomp/_builtin_kernels.py:8-25, locomp/api.py:1025-1038   out[i] = table[ids[i]]
//   argmax        host-side np.argmax in examples/54_smollm2_inference.py:606 (first maximum wins)
// All arithmetic is float32 whatever the storage type; results are rounded once (to nearest
// even) into the output type.  Every kernel takes part in programmatic dependent launch: it
// lets the next kernel of the stream become resident at once and touches memory only after
// the kernel before it has completed.
//
// HBM/L2-bound elementwise work of a few KB per call: the cost is launch latency, which is why
// the fused form exists.
#pragma once
#include "common.cuh"

namespace lcq {
namespace glue {

constexpr int NORM_THREADS = 256;

template <typename T> __device__ __forceinline__ void load_vec8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void load_vec8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load_vec8<__half>(const __half* p, float (&v)[8]) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
template <> __device__ __forceinline__ void load_vec8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const uint32_t* u = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(u[i] << 16); v[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u); }
}
template <typename T> __device__ __forceinline__ void store_vec8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void store_vec8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *(reinterpret_cast<float4*>(p) + 1) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store_vec8<__half>(__half* p, const float (&v)[8]) {
  __half2 h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(h);
}
template <> __device__ __forceinline__ void store_vec8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  __nv_bfloat162 h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(h);
}

// Sum over the CTA; every thread gets the total.  `red` holds one float per warp (+1).
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.0f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// One CTA per row.  ADD: h = resid + x is formed first, written back to `resid` (in place, as the
// reference's add_inplace does) and normalised; without ADD, `resid` is unused.
// VEC: n % 8 == 0 and all row starts 16-byte aligned.
template <typename T, bool ADD, bool VEC>
__global__ void __launch_bounds__(NORM_THREADS) rms_norm_kernel(const T* __restrict__ x, T* __restrict__ resid,
                                                                const T* __restrict__ w, T* __restrict__ out,
                                                                int n, float eps) {
  __shared__ float red[33];
  griddep_launch_dependents();
  griddep_wait();
  const long long row = blockIdx.x;
  const T* xr = x + row * n;
  T* rr = ADD ? resid + row * n : nullptr;
  T* orow = out + row * n;
  float ss = 0.0f;
  if (VEC) {
    for (int i = threadIdx.x * 8; i < n; i += NORM_THREADS * 8) {
      float v[8];
      load_vec8<T>(xr + i, v);
      if (ADD) {
        float r[8];
        load_vec8<T>(rr + i, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = to_f32<T>(from_f32<T>(r[j] + v[j]));   // the value the in-place add stores
        store_vec8<T>(rr + i, v);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
    }
  } else {
    for (int i = threadIdx.x; i < n; i += NORM_THREADS) {
      float v = to_f32<T>(xr[i]);
      if (ADD) {
        const T h = from_f32<T>(to_f32<T>(rr[i]) + v);
        rr[i] = h;
        v = to_f32<T>(h);
      }
      ss = fmaf(v, v, ss);
    }
  }
  const float total = block_sum(ss, red);           // also orders the in-place stores before the reads below
  const float rms = rsqrtf(total / static_cast<float>(n) + eps);
  const T* src = ADD ? rr : xr;
  if (VEC) {
    for (int i = threadIdx.x * 8; i < n; i += NORM_THREADS * 8) {
      float v[8], g[8];
      load_vec8<T>(src + i, v);
      load_vec8<T>(w + i, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = v[j] * rms * g[j];
      store_vec8<T>(orow + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < n; i += NORM_THREADS) orow[i] = from_f32<T>(to_f32<T>(src[i]) * rms * to_f32<T>(w[i]));
  }
}

// MODE 0: out = silu(a) * b      MODE 1: a += b (out == a)
template <typename T, int MODE>
__global__ void __launch_bounds__(256) elementwise_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                          T* __restrict__ out, long long n, int vec) {
  griddep_launch_dependents();
  griddep_wait();
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (vec) {
    for (long long i = tid * 8; i < n; i += stride * 8) {
      float x[8], y[8];
      load_vec8<T>(a + i, x);
      load_vec8<T>(b + i, y);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        x[j] = MODE == 0 ? (x[j] * (1.0f / (1.0f + expf(-x[j])))) * y[j] : x[j] + y[j];
      store_vec8<T>(out + i, x);
    }
  } else {
    for (long long i = tid; i < n; i += stride) {
      const float x = to_f32<T>(a[i]), y = to_f32<T>(b[i]);
      out[i] = from_f32<T>(MODE == 0 ? (x * (1.0f / (1.0f + expf(-x)))) * y : x + y);
    }
  }
}

// out[i, :] = table[ids[i], :]; one CTA per token.  An id outside [0, vocab) yields a row of
// zeros and sets the device status word (code 40) instead of reading out of bounds.
__global__ void __launch_bounds__(128) embed_lookup_kernel(const int* __restrict__ ids, const uint8_t* __restrict__ table,
                                                           uint8_t* __restrict__ out, int vocab, long long row_bytes, int vec) {
  griddep_launch_dependents();
  griddep_wait();
  const long long t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0) atomicExch(&g_device_status, 40);
  const uint8_t* src = table + static_cast<long long>(ok ? id : 0) * row_bytes;
  uint8_t* dst = out + t * row_bytes;
  if (vec) {
    for (long long i = threadIdx.x * 16LL; i < row_bytes; i += 128 * 16)
      *reinterpret_cast<uint4*>(dst + i) = ok ? __ldg(reinterpret_cast<const uint4*>(src + i)) : make_uint4(0u, 0u, 0u, 0u);
  } else {
    for (long long i = threadIdx.x; i < row_bytes; i += 128) dst[i] = ok ? src[i] : 0;
  }
}

// out[r] = index of the first maximum of x[r, :] (np.argmax: ties go to the lowest index, a NaN
// counts as the maximum).  One CTA per row.
constexpr int ARGMAX_THREADS = 1024;
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  // NaN beats everything; among equals the lower index wins
  const bool vn = v != v, bn = bv != bv;
  if (vn != bn) return vn;
  if (!vn && v != bv) return v > bv;
  return i < bi;
}
template <typename T>
__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_kernel(const T* __restrict__ x, int* __restrict__ out, int n, int vec) {
  __shared__ float sv[32];
  __shared__ int si[32];
  griddep_launch_dependents();
  griddep_wait();
  const T* xr = x + static_cast<long long>(blockIdx.x) * n;
  float bv = -INFINITY;
  int bi = 0x7FFFFFFF;
  if (vec) {
    for (int i = threadIdx.x * 8; i < n; i += ARGMAX_THREADS * 8) {
      float v[8];
      load_vec8<T>(xr + i, v);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (better(v[j], i + j, bv, bi)) { bv = v[j]; bi = i + j; }
    }
  } else {
    for (int i = threadIdx.x; i < n; i += ARGMAX_THREADS) {
      const float v = to_f32<T>(xr[i]);
      if (better(v, i, bv, bi)) { bv = v; bi = i; }
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = sv[lane]; bi = si[lane];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out[blockIdx.x] = bi;
  }
}

// ---------------------------------------------------------------------------- host side
inline void pdl_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, dim3 grid, dim3 block, cudaStream_t stream) {
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = stream;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
}

template <typename T>
int launch_rms_norm(const void* x, void* resid, const void* w, void* out, long long rows, int n, float eps, cudaStream_t st) {
  if (rows == 0 || n == 0) return LCQ_OK;
  if (rows > 2147483647LL) { set_error("rms_norm: too many rows"); return LCQ_ERR_UNSUPPORTED; }
  const bool vec = (n % 8 == 0) && aligned(x, 16) && aligned(w, 16) && aligned(out, 16) && (!resid || aligned(resid, 16)) &&
                   ((static_cast<long long>(n) * sizeof(T)) % 16 == 0);
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  pdl_config(cfg, attr, dim3(static_cast<unsigned>(rows)), dim3(NORM_THREADS), st);
  const T* xp = static_cast<const T*>(x);
  T* rp = static_cast<T*>(resid);
  const T* wp = static_cast<const T*>(w);
  T* op = static_cast<T*>(out);
  if (resid) {
    if (vec) LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, rms_norm_kernel<T, true, true>, xp, rp, wp, op, n, eps));
    else LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, rms_norm_kernel<T, true, false>, xp, rp, wp, op, n, eps));
  } else {
    if (vec) LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, rms_norm_kernel<T, false, true>, xp, rp, wp, op, n, eps));
    else LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, rms_norm_kernel<T, false, false>, xp, rp, wp, op, n, eps));
  }
  return LCQ_OK;
}

template <typename T, int MODE>
int launch_elementwise(const void* a, const void* b, void* out, long long n, int sm_count, cudaStream_t st) {
  if (n == 0) return LCQ_OK;
  const int vec = (n % 8 == 0) && aligned(a, 16) && aligned(b, 16) && aligned(out, 16);
  long long blocks = ((vec ? n / 8 : n) + 255) / 256;
  if (blocks > static_cast<long long>(sm_count) * 8) blocks = static_cast<long long>(sm_count) * 8;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  pdl_config(cfg, attr, dim3(static_cast<unsigned>(blocks)), dim3(256), st);
  LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, elementwise_kernel<T, MODE>, static_cast<const T*>(a), static_cast<const T*>(b),
                                  static_cast<T*>(out), n, vec));
  return LCQ_OK;
}

inline int launch_embed(const void* ids, const void* table, void* out, long long tokens, int vocab, long long row_bytes,
                        cudaStream_t st) {
  if (tokens == 0 || row_bytes == 0) return LCQ_OK;
  if (tokens > 2147483647LL) { set_error("embed_lookup: too many tokens"); return LCQ_ERR_UNSUPPORTED; }
  const int vec = (row_bytes % 16 == 0) && aligned(table, 16) && aligned(out, 16);
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  pdl_config(cfg, attr, dim3(static_cast<unsigned>(tokens)), dim3(128), st);
  LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, embed_lookup_kernel, static_cast<const int*>(ids), static_cast<const uint8_t*>(table),
                                  static_cast<uint8_t*>(out), vocab, row_bytes, vec));
  return LCQ_OK;
}

template <typename T>
int launch_argmax(const void* x, void* out, long long rows, int n, cudaStream_t st) {
  if (rows == 0) return LCQ_OK;
  if (n <= 0) { set_error("argmax: empty rows have no maximum"); return LCQ_ERR_BAD_ARG; }
  if (rows > 2147483647LL) { set_error("argmax: too many rows"); return LCQ_ERR_UNSUPPORTED; }
  const int vec = (n % 8 == 0) && aligned(x, 16) && ((static_cast<long long>(n) * sizeof(T)) % 16 == 0);
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  pdl_config(cfg, attr, dim3(static_cast<unsigned>(rows)), dim3(ARGMAX_THREADS), st);
  LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, argmax_kernel<T>, static_cast<const T*>(x), static_cast<int*>(out), n, vec));
  return LCQ_OK;
}

}  // namespace glue
}  // namespace lcq
