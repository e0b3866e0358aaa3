// W8 decode kernel (M <= 8): int8 weights streamed from HBM by 2-D TMA into a multi-stage
// shared-memory ring, read back 128 bits per lane, dequantised and contracted in float32.
//
// It computes the reference's dequant_matvec_int8 (examples/38_quantized_matmul.py:94-134)
// and its batched form:
//   out[m, n] = sum_g scales[n, g] * sum_{k in group g} x[m, k] * float(w[n, k])
// with float32 arithmetic end to end, so it serves the reference's own dtypes (float32 x,
// scales and out at 1e-4 relative) as well as 16-bit activations.
//
// Work decomposition.  A CTA owns 16 output rows and walks all of K in tiles of 16 rows x 256
// bytes (one TMA box, 4 KB; K need only be a multiple of 16: the last box is filled with
// zeros).  A producer warp keeps an 8-stage ring full; it starts before the kernel ahead of it
// on the stream has finished (weights are constants), while the four consumer warps wait for
// that kernel before touching x.  Consumer warp w takes rows 4w .. 4w+3: a 256-byte tile row is
// 16 lanes x 16 bytes, so one 128-bit shared load serves two rows per warp instruction and a
// lane holds 16 consecutive weights of one group (group_size % 16 == 0).  Per-lane partial sums
// are combined with a 16-lane shuffle tree once, after the last tile.  No scratch memory, no
// reduction between CTAs.
//
// HBM-bound: algorithmic bytes per call = N*K + N*(K/G)*sizeof(scale) (+ x and out).
#pragma once
#include "common.cuh"
#include "dequant.cuh"
#include "gemv_simt.cuh"

namespace lcq {
namespace gemv_w8 {

constexpr int RB = 16;                       // rows per CTA and tile
constexpr int KB = 256;                      // weight bytes (= k) per tile row
constexpr int STAGE_BYTES = RB * KB;         // 4096
constexpr int NSTAGES = 8;
constexpr int NCW = 4;                       // consumer warps, 4 rows each
constexpr int RPW = RB / NCW / 2;            // 128-bit loads (two rows each) per warp and tile
constexpr int NTHREADS = (NCW + 1) * 32;

__device__ __forceinline__ uint4 lds128_w8(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}

template <typename XT> __device__ __forceinline__ void load16(const XT* p, float (&v)[16]) {
  float a[8], b[8];
  load8<XT>(p, a);
  load8<XT>(p + 8, b);
#pragma unroll
  for (int i = 0; i < 8; ++i) { v[i] = a[i]; v[8 + i] = b[i]; }
}

__device__ __forceinline__ float load_scale(const void* s, int dtype, long long i) {
  if (dtype == LCQ_F16) return __half2float(__ldg(static_cast<const __half*>(s) + i));
  if (dtype == LCQ_BF16) return __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(s) + i));
  return __ldg(static_cast<const float*>(s) + i);
}
__device__ __forceinline__ void store_result(void* out, int dtype, long long i, float v) {
  if (dtype == LCQ_F16) static_cast<__half*>(out)[i] = __float2half_rn(v);
  else if (dtype == LCQ_BF16) static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
  else static_cast<float*>(out)[i] = v;
}

// XT: activation type.  MM: rows of x the accumulators are sized for (>= M; 1, 2, 4 or 8).
// Scale and output types are run-time codes (one scale load per 16 weights, one store per output).
template <typename XT, int MM>
__global__ void __launch_bounds__(NTHREADS) w8_gemv_kernel(const __grid_constant__ CUtensorMap tmap_w,
                                                           const XT* __restrict__ x, const void* __restrict__ scales,
                                                           void* __restrict__ out, int M, int N, int K, int G,
                                                           int s_dtype, int o_dtype) {
  __shared__ __align__(128) uint8_t stages[NSTAGES * STAGE_BYTES];
  __shared__ __align__(8) uint64_t full_bar[NSTAGES];
  __shared__ __align__(8) uint64_t empty_bar[NSTAGES];
  __shared__ int flag_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (K + KB - 1) / KB;
  const int row0 = blockIdx.x * RB;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], NCW); }
    flag_abort = 0;
    fence_barrier_init();
    griddep_launch_dependents();     // the next kernel of the stream may become resident as our CTAs retire
  }
  __syncthreads();

  if (warp == NCW) {
    // ------------------------------------------------------------ producer (weights are constants: no dependency wait)
    if (lane == 0) {
      tma_prefetch_desc(&tmap_w);
      for (int it = 0; it < n_tiles; ++it) {
        const int s = it % NSTAGES;
        const uint32_t ph = (it / NSTAGES) & 1;
        if (*reinterpret_cast<volatile int*>(&flag_abort) || !mbar_wait_bounded(&empty_bar[s], ph ^ 1)) {
          flag_abort = 1; atomicExch(&g_device_status, 5);
          break;
        }
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        tma_load_2d(stages + s * STAGE_BYTES, &tmap_w, &full_bar[s], it * KB, row0);
      }
    }
  } else {
    // ------------------------------------------------------------ consumers
    const int half = lane >> 4, seg = lane & 15;       // which of the two rows of a load; 16-byte segment of the tile row
    const int ns = K / G;
    float acc[RPW][MM];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
#pragma unroll
      for (int m = 0; m < MM; ++m) acc[i][m] = 0.0f;
    }
    const uint32_t lane_addr = smem_u32(stages) + static_cast<uint32_t>((warp * (2 * RPW) + half) * KB + seg * 16);
    griddep_wait();                  // x may be the output of the kernel ahead of us; out may still be in its use
    bool dead = false;
    // x and the scales of a tile come from global memory (L1 / L2): those of tile it+1 are fetched
    // before the math of tile it, so their latency hides behind it.
    float xn[MM <= 2 ? MM : 1][16];
    float scn[RPW];
    auto fetch = [&](int it) {
      const int k0 = it * KB + seg * 16;
      if (it < n_tiles && k0 < K) {
        if (MM <= 2) {
#pragma unroll
          for (int m = 0; m < MM; ++m) {
            if (m < M) load16<XT>(x + static_cast<long long>(m) * K + k0, xn[m]);
          }
        }
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
          const int row = row0 + warp * (2 * RPW) + 2 * i + half;
          scn[i] = row < N ? load_scale(scales, s_dtype, static_cast<long long>(row) * ns + k0 / G) : 0.0f;
        }
      }
    };
    fetch(0);
    for (int it = 0; it < n_tiles; ++it) {
      const int s = it % NSTAGES;
      const uint32_t ph = (it / NSTAGES) & 1;
      float xr[MM <= 2 ? MM : 1][16];
      float sc[RPW];
#pragma unroll
      for (int m = 0; m < (MM <= 2 ? MM : 1); ++m) {
#pragma unroll
        for (int e = 0; e < 16; ++e) xr[m][e] = xn[m][e];
      }
#pragma unroll
      for (int i = 0; i < RPW; ++i) sc[i] = scn[i];
      fetch(it + 1);
      if (!dead && (*reinterpret_cast<volatile int*>(&flag_abort) || !mbar_wait_bounded(&full_bar[s], ph))) {
        dead = true; flag_abort = 1; atomicExch(&g_device_status, 6);
      }
      const int k0 = it * KB + seg * 16;               // this lane's 16 consecutive k
      if (!dead && k0 < K) {
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
          const uint4 wv = lds128_w8(lane_addr + static_cast<uint32_t>(s * STAGE_BYTES + 2 * i * KB));
          float wf[16];
          {
            float f[4];
            int8x4_to_f32(wv.x, f); wf[0] = f[0]; wf[1] = f[1]; wf[2] = f[2]; wf[3] = f[3];
            int8x4_to_f32(wv.y, f); wf[4] = f[0]; wf[5] = f[1]; wf[6] = f[2]; wf[7] = f[3];
            int8x4_to_f32(wv.z, f); wf[8] = f[0]; wf[9] = f[1]; wf[10] = f[2]; wf[11] = f[3];
            int8x4_to_f32(wv.w, f); wf[12] = f[0]; wf[13] = f[1]; wf[14] = f[2]; wf[15] = f[3];
          }
#pragma unroll
          for (int m = 0; m < MM; ++m) {
            if (m < M) {
              float dot = 0.0f;
              if (MM <= 2) {
#pragma unroll
                for (int e = 0; e < 16; ++e) dot = fmaf(xr[m][e], wf[e], dot);
              } else {
                float xv[16];
                load16<XT>(x + static_cast<long long>(m) * K + k0, xv);
#pragma unroll
                for (int e = 0; e < 16; ++e) dot = fmaf(xv[e], wf[e], dot);
              }
              acc[i][m] = fmaf(sc[i], dot, acc[i][m]);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);       // also in the dead state, so the producer never stalls on us
    }
    // 16-lane tree: lanes 0-15 hold row (2i), lanes 16-31 row (2i+1) of the warp's 8 rows
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
#pragma unroll
      for (int m = 0; m < MM; ++m) {
        float v = acc[i][m];
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        const int row = row0 + warp * (2 * RPW) + 2 * i + half;
        if (seg == 0 && m < M && row < N) store_result(out, o_dtype, static_cast<long long>(m) * N + row, v);
      }
    }
  }
  __syncthreads();
}

inline bool supported(int M, int N, int K, int G) {
  return M >= 1 && M <= 8 && N >= 1 && K >= 16 && (K % 16) == 0 && G >= 16 && (G % 16) == 0;
}

template <typename XT>
int launch(const void* x, const void* w, const void* s, void* out, int M, int N, int K, int G, int s_dtype, int o_dtype,
           cudaStream_t stream) {
  if (!aligned(w, 16) || !aligned(x, 16) || (static_cast<long long>(K) * sizeof(XT)) % 16 != 0) {
    set_error("w8 gemv: x rows and w_int8 must be 16-byte aligned");
    return LCQ_ERR_BAD_ARG;
  }
  CUtensorMap tw;
  int rc = encode_tmap_2d(&tw, 0, w, static_cast<uint64_t>(K), static_cast<uint64_t>(N), static_cast<uint64_t>(K), KB, RB, 0);
  if (rc != LCQ_OK) return rc;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((N + RB - 1) / RB);
  cfg.blockDim = dim3(NTHREADS);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  const XT* xp = static_cast<const XT*>(x);
  if (M == 1) LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, w8_gemv_kernel<XT, 1>, tw, xp, s, out, M, N, K, G, s_dtype, o_dtype));
  else if (M == 2) LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, w8_gemv_kernel<XT, 2>, tw, xp, s, out, M, N, K, G, s_dtype, o_dtype));
  else if (M <= 4) LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, w8_gemv_kernel<XT, 4>, tw, xp, s, out, M, N, K, G, s_dtype, o_dtype));
  else LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, w8_gemv_kernel<XT, 8>, tw, xp, s, out, M, N, K, G, s_dtype, o_dtype));
  return LCQ_OK;
}

}  // namespace gemv_w8
}  // namespace lcq
