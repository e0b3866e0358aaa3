// W4A16 decode kernel (M <= 16): int4 weights streamed from HBM by 2-D TMA into a
// multi-stage shared-memory ring, dequantised for free, contracted on warp-level tensor
// cores with float32 accumulation, split along K with a deterministic last-arriver reduce.
//
// It computes the batched form of the reference's dequant_matvec_int4
// (examples/38_quantized_matmul.py:30-87) for 16-bit activations:
//   out[m, n] = sum_g scales[n, g] * sum_{k in group g} x[m, k] * (nib(n, k) - 8)
//
// How the dequantisation becomes free.  A stored nibble q sitting in bits 0-3 of a 16-bit
// lane *is* the fp16 subnormal q * 2^-24; in bits 4-7 it is q * 2^-20.  So
//   word & 0x000F000F, word & 0x00F000F0, (word>>8) & 0x000F000F, (word>>8) & 0x00F000F0
// are four ready-made half2 A-operands holding elements (0,4) (1,5) (2,6) (3,7) of the 8
// nibbles of a 32-bit word.  The activations are staged once per CTA into shared memory in
// exactly that element order, with the (1,5) and (3,7) slots pre-divided by 16, so both
// nibble positions come out scaled by 2^-24.  The zero point is folded in through the
// accumulator input:  C = -8 * 2^-24 * sum_{k in g} x[m, k].  One 32-wide group is two
// m16n8k16 MMAs, after which  acc += scale * D  (float32); the final result is acc * 2^24.
//
// Work decomposition.  A tile is 128 rows x 256 k (16 KB of packed weights + 2 KB of
// scales, one TMA box each).  K is cut into n_kr ranges so that one range of x fits in
// shared memory; the CTAs of a range split its tile sequence (row-block major) evenly,
// stream-K style, so the last wave is never ragged.  A row block whose tiles were produced
// by more than one CTA is combined through scratch: every contributor writes its float32
// partial, bumps a per-row-block counter, and the last one sums all partials in a fixed
// order, writes the output and resets the counter.  Nobody spins.
//
// HBM-bound: algorithmic bytes per call = N*K/2 + N*(K/32)*2 (+ 2*M*(K+N)).
#pragma once
#include "common.cuh"
#include "gemv_simt.cuh"

namespace lcq {
namespace gemv_tc {

constexpr int ROWS = 128;                    // rows per tile
constexpr int KT = 256;                      // k per tile
constexpr int GT = KT / 32;                  // groups per tile
constexpr int W_BYTES = ROWS * (KT / 2);     // 16384, 128B-swizzled rows of 128 B
constexpr int S_BYTES = ROWS * GT * 2;       // 2048, rows of 8 fp16 scales
constexpr int STAGE_BYTES = W_BYTES + S_BYTES;
constexpr int NSTAGES = 6;
constexpr int NCW = 8;                       // consumer warps, 16 rows each
constexpr int NTHREADS = (NCW + 1) * 32;     // + 1 producer warp
constexpr int X_SMEM_BYTES = 64 * 1024;      // budget for one k-range of activations
constexpr int BAR_CONSUMERS = 1;             // named barrier id for the consumer warps
// The workspace starts with a counter region of FIXED size so that it sits at the same place
// for every problem: only the counters must be zero on entry (and are zero again on exit);
// the partials behind them are scratch that successive calls may leave dirty.
constexpr int MAX_ROW_BLOCKS = 16384;
constexpr size_t COUNTER_BYTES = MAX_ROW_BLOCKS * sizeof(int);

struct Params {
  const void* x;        // [M, K] fp16 or bf16
  void* out;            // [M, N]
  float* partials;      // [n_rb][n_kr * max_split][M][ROWS]
  int* counters;        // [n_rb], zero on entry, zero on exit
  int M, N, K;
  int x_is_bf16;
  int n_rb;             // ceil(N / ROWS)
  int n_kr;             // k ranges
  int S;                // tiles (of 256 k) per k-range; the last range may hold fewer
  int nst;              // K / 256
  int ctas_per_kr;      // CTAs working on one k-range
  int max_split;        // scratch slots per (row block, k-range)
};

struct Sched {          // the share of one k-range's tile sequence owned by one CTA
  int S_kr;             // tiles per row block in this k-range
  long long T;          // n_rb * S_kr
  int G;                // CTAs on this k-range (<= T)
};

__host__ __device__ inline Sched make_sched(const Params& p, int kr) {
  Sched s;
  const int left = p.nst - kr * p.S;
  s.S_kr = left < p.S ? left : p.S;
  s.T = static_cast<long long>(p.n_rb) * s.S_kr;
  s.G = p.ctas_per_kr < s.T ? p.ctas_per_kr : static_cast<int>(s.T);
  return s;
}
__host__ __device__ inline long long tile_begin(const Sched& s, int j) { return (static_cast<long long>(j) * s.T) / s.G; }
__host__ __device__ inline int owner_of(const Sched& s, long long t) {
  return static_cast<int>(((t + 1) * s.G - 1) / s.T);
}
// CTAs j0..j1 (inclusive) of this k-range contribute to row block rb.
__host__ __device__ inline void cover(const Sched& s, int rb, int& j0, int& j1) {
  j0 = owner_of(s, static_cast<long long>(rb) * s.S_kr);
  j1 = owner_of(s, static_cast<long long>(rb + 1) * s.S_kr - 1);
}
__host__ __device__ inline int contributors(const Params& p, int rb) {
  int total = 0;
  for (int kr = 0; kr < p.n_kr; ++kr) {
    const Sched s = make_sched(p, kr);
    int j0, j1;
    cover(s, rb, j0, j1);
    total += j1 - j0 + 1;
  }
  return total;
}

struct SmemLayout {
  // offsets from the 1024-byte aligned base
  int stages;   // NSTAGES * STAGE_BYTES
  int xs;       // staged activations: [group][M][4] x 16 B
  int cz;       // accumulator inputs: [group][MP] float
  int bars;     // full[NSTAGES], empty[NSTAGES]
  int flags;    // abort flag, last-arriver flag
  int total;
};
__host__ __device__ inline SmemLayout smem_layout(int M, int MP, int S) {
  SmemLayout L;
  L.stages = 0;
  L.xs = NSTAGES * STAGE_BYTES;
  const int groups = S * GT;
  L.cz = L.xs + groups * M * 64;
  L.bars = L.cz + groups * MP * 4;
  L.bars = (L.bars + 15) & ~15;
  L.flags = L.bars + 2 * NSTAGES * 8;
  L.total = L.flags + 16;
  return L;
}

template <typename T> __device__ __forceinline__ void store_out(T* out, long long idx, float v) { out[idx] = from_f32<T>(v); }

template <int MT, typename OT>
__global__ void __launch_bounds__(NTHREADS, 1)
w4a16_gemv_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_s,
                  const Params p) {
  constexpr int MP = 8 * MT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

  const int kr = blockIdx.x % p.n_kr;
  const int j = blockIdx.x / p.n_kr;
  const Sched sch = make_sched(p, kr);
  if (j >= sch.G) return;  // whole CTA leaves together; nothing was started
  const long long t0 = tile_begin(sch, j), t1 = tile_begin(sch, j + 1);

  const SmemLayout L = smem_layout(p.M, MP, p.S);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L.bars);
  uint64_t* empty_bar = full_bar + NSTAGES;
  volatile int* flag_abort = reinterpret_cast<volatile int*>(smem + L.flags);
  volatile int* flag_last = flag_abort + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], NCW); }
    *flag_abort = 0;
    *flag_last = 0;
    fence_barrier_init();
  }
  __syncthreads();

  if (warp == NCW) {
    // ------------------------------------------------------------ producer warp
    if (lane == 0) {
      tma_prefetch_desc(&tmap_w);
      tma_prefetch_desc(&tmap_s);
      bool dead = false;
      int it = 0;
      int rb = static_cast<int>(t0 / sch.S_kr);
      int ks = static_cast<int>(t0 - static_cast<long long>(rb) * sch.S_kr);
      for (long long t = t0; t < t1; ++t, ++it) {
        const int s = it % NSTAGES;
        const uint32_t ph = (it / NSTAGES) & 1;
        if (!dead && *flag_abort) dead = true;
        if (!dead && !mbar_wait_bounded(&empty_bar[s], ph ^ 1)) {
          dead = true; *flag_abort = 1; atomicExch(&g_device_status, 1);
        }
        if (dead) break;
        const int kt = kr * p.S + ks;  // absolute k tile
        uint8_t* dst = smem + s * STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        tma_load_2d(dst, &tmap_w, &full_bar[s], kt * (KT / 2), rb * ROWS);
        tma_load_2d(dst + W_BYTES, &tmap_s, &full_bar[s], kt * GT, rb * ROWS);
        if (++ks == sch.S_kr) { ks = 0; ++rb; }
      }
    }
  } else {
    // ------------------------------------------------------------ consumer warps
    const int ctid = threadIdx.x;            // 0..255
    const int g = lane >> 2, t4 = lane & 3;
    uint4* xs = reinterpret_cast<uint4*>(smem + L.xs);
    float* cz = reinterpret_cast<float*>(smem + L.cz);

    // ---- stage this k-range of x: permuted element order, fp16, high-nibble slots / 16
    {
      const int oct_per_row = sch.S_kr * (KT / 8);
      const int total = p.M * oct_per_row;
      const long long kbase = static_cast<long long>(kr) * p.S * KT;
      for (int i = ctid; i < sch.S_kr * GT * MP; i += NCW * 32) cz[i] = 0.0f;
      named_bar_sync(BAR_CONSUMERS, NCW * 32);
      for (int base = 0; base < total; base += NCW * 32) {
        const int idx = base + ctid;
        const bool valid = idx < total;
        const int m = valid ? idx / oct_per_row : 0;
        const int o = valid ? idx - m * oct_per_row : 0;
        float v[8];
        if (valid) {
          const long long off = static_cast<long long>(m) * p.K + kbase + 8 * o;
          if (p.x_is_bf16) load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(p.x) + off, v);
          else load8<__half>(static_cast<const __half*>(p.x) + off, v);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = 0.0f;
        }
        float sum = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (valid) {
          const __half2 h0 = __floats2half2_rn(v[0], v[4]);
          const __half2 h1 = __floats2half2_rn(v[1] * 0.0625f, v[5] * 0.0625f);
          const __half2 h2 = __floats2half2_rn(v[2], v[6]);
          const __half2 h3 = __floats2half2_rn(v[3] * 0.0625f, v[7] * 0.0625f);
          uint4 q;
          q.x = *reinterpret_cast<const uint32_t*>(&h0); q.y = *reinterpret_cast<const uint32_t*>(&h1);
          q.z = *reinterpret_cast<const uint32_t*>(&h2); q.w = *reinterpret_cast<const uint32_t*>(&h3);
          const int grp = o >> 2;
          xs[(grp * p.M + m) * 4 + (o & 3)] = q;
          if ((o & 3) == 0) cz[grp * MP + m] = -sum * 4.76837158203125e-07f;  // -8 * 2^-24
        }
      }
      named_bar_sync(BAR_CONSUMERS, NCW * 32);
    }

    float acc[MT][4];
#pragma unroll
    for (int jm = 0; jm < MT; ++jm) { acc[jm][0] = acc[jm][1] = acc[jm][2] = acc[jm][3] = 0.0f; }

    const int r0 = warp * 16 + g;
    const int swz = g & 7;
    bool has_m[MT];
    const uint4* xs_lane[MT];
    const float2* cz_lane[MT];
#pragma unroll
    for (int jm = 0; jm < MT; ++jm) {
      has_m[jm] = (8 * jm + g) < p.M;
      xs_lane[jm] = xs + (has_m[jm] ? (8 * jm + g) * 4 + t4 : 0);
      cz_lane[jm] = reinterpret_cast<const float2*>(cz + 8 * jm + 2 * t4);
    }

    bool dead = false;
    int it = 0;
    int rb = static_cast<int>(t0 / sch.S_kr);
    int ks = static_cast<int>(t0 - static_cast<long long>(rb) * sch.S_kr);
    for (long long t = t0; t < t1; ++t, ++it) {
      const int s = it % NSTAGES;
      const uint32_t ph = (it / NSTAGES) & 1;

      if (!dead && *flag_abort) dead = true;
      if (!dead && !mbar_wait_bounded(&full_bar[s], ph)) {
        dead = true; *flag_abort = 1; atomicExch(&g_device_status, 2);
      }
      if (!dead) {
        const uint8_t* ws = smem + s * STAGE_BYTES;
        const uint32_t* rowA = reinterpret_cast<const uint32_t*>(ws + r0 * 128) + t4;
        const uint32_t* rowB = reinterpret_cast<const uint32_t*>(ws + (r0 + 8) * 128) + t4;
        const uint4 sA = *reinterpret_cast<const uint4*>(ws + W_BYTES + r0 * 16);
        const uint4 sB = *reinterpret_cast<const uint4*>(ws + W_BYTES + (r0 + 8) * 16);
        const __half* hA = reinterpret_cast<const __half*>(&sA);
        const __half* hB = reinterpret_cast<const __half*>(&sB);
        const int gbase = ks * GT;
#pragma unroll
        for (int c = 0; c < GT; ++c) {
          const int cs = (c ^ swz) * 4;
          const uint32_t wa = rowA[cs], wb = rowB[cs];
          const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
          const float s_a = __half2float(hA[c]), s_b = __half2float(hB[c]);
#pragma unroll
          for (int jm = 0; jm < MT; ++jm) {
            uint4 bx = make_uint4(0u, 0u, 0u, 0u);
            if (has_m[jm]) bx = xs_lane[jm][(gbase + c) * p.M * 4];
            const float2 ci = cz_lane[jm][(gbase + c) * (MP / 2)];
            const float cin[4] = {ci.x, ci.y, ci.x, ci.y};
            float d[4];
            mma_m16n8k16_f16(d, wa & 0x000F000Fu, wb & 0x000F000Fu, wa & 0x00F000F0u, wb & 0x00F000F0u,
                             bx.x, bx.y, cin);
            mma_m16n8k16_f16(d, wa8 & 0x000F000Fu, wb8 & 0x000F000Fu, wa8 & 0x00F000F0u, wb8 & 0x00F000F0u,
                             bx.z, bx.w, d);
            acc[jm][0] = fmaf(s_a, d[0], acc[jm][0]);
            acc[jm][1] = fmaf(s_a, d[1], acc[jm][1]);
            acc[jm][2] = fmaf(s_b, d[2], acc[jm][2]);
            acc[jm][3] = fmaf(s_b, d[3], acc[jm][3]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);  // also in the dead state, so the producer never stalls on us

      // ---- end of this CTA's share of row block rb: flush
      if (ks == sch.S_kr - 1 || t == t1 - 1) {
        const int n_contrib = contributors(p, rb);
        const int nA = rb * ROWS + r0, nB = nA + 8;
        if (n_contrib == 1) {
          OT* out = static_cast<OT*>(p.out);
#pragma unroll
          for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int m = 8 * jm + 2 * t4 + e;
              if (m < p.M) {
                if (nA < p.N) store_out(out, static_cast<long long>(m) * p.N + nA, acc[jm][e] * 16777216.0f);
                if (nB < p.N) store_out(out, static_cast<long long>(m) * p.N + nB, acc[jm][2 + e] * 16777216.0f);
              }
            }
          }
        } else {
          int j0, j1;
          cover(sch, rb, j0, j1);
          const int slot = kr * p.max_split + (j - j0);
          float* part = p.partials + (static_cast<long long>(rb) * p.n_kr * p.max_split + slot) * p.M * ROWS;
#pragma unroll
          for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int m = 8 * jm + 2 * t4 + e;
              if (m < p.M) {
                __stcg(part + m * ROWS + r0, acc[jm][e] * 16777216.0f);
                __stcg(part + m * ROWS + r0 + 8, acc[jm][2 + e] * 16777216.0f);
              }
            }
          }
          __threadfence();
          named_bar_sync(BAR_CONSUMERS, NCW * 32);
          if (ctid == 0) {
            const int old = atomicAdd(p.counters + rb, 1);
            *flag_last = (old == n_contrib - 1) ? 1 : 0;
          }
          named_bar_sync(BAR_CONSUMERS, NCW * 32);
          if (*flag_last) {
            __threadfence();
            OT* out = static_cast<OT*>(p.out);
            const float* rb_part = p.partials + static_cast<long long>(rb) * p.n_kr * p.max_split * p.M * ROWS;
            for (int idx = ctid; idx < p.M * ROWS; idx += NCW * 32) {
              const int m = idx / ROWS, r = idx - m * ROWS;
              float sum = 0.0f;
              for (int kk = 0; kk < p.n_kr; ++kk) {
                const Sched s2 = make_sched(p, kk);
                int a0, a1;
                cover(s2, rb, a0, a1);
                for (int c = 0; c <= a1 - a0; ++c)
                  sum += __ldcg(rb_part + (static_cast<long long>(kk) * p.max_split + c) * p.M * ROWS + idx);
              }
              const int n = rb * ROWS + r;
              if (n < p.N) store_out(out, static_cast<long long>(m) * p.N + n, sum);
            }
            if (ctid == 0) p.counters[rb] = 0;
          }
          named_bar_sync(BAR_CONSUMERS, NCW * 32);  // flag_last is reused by the next flush
        }
#pragma unroll
        for (int jm = 0; jm < MT; ++jm) { acc[jm][0] = acc[jm][1] = acc[jm][2] = acc[jm][3] = 0.0f; }
      }
      if (++ks == sch.S_kr) { ks = 0; ++rb; }
    }
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------- host side
struct Plan {
  Params p;
  int grid;
  int MT;
  size_t smem_bytes;
  size_t counters_bytes;   // COUNTER_BYTES, the same for every problem
  size_t workspace_bytes;  // counters + partials
};

inline bool supported(int M, int N, int K, int G, int x_dtype, int scale_dtype) {
  return M >= 1 && M <= 16 && N >= 1 && N <= MAX_ROW_BLOCKS * ROWS && K >= KT && (K % KT) == 0 && G == 32 &&
         (x_dtype == LCQ_F16 || x_dtype == LCQ_BF16) && scale_dtype == LCQ_F16;
}

inline Plan make_plan(int M, int N, int K, int sm_count) {
  Plan pl;
  memset(&pl, 0, sizeof(pl));
  Params& p = pl.p;
  p.M = M; p.N = N; p.K = K;
  p.n_rb = (N + ROWS - 1) / ROWS;
  p.nst = K / KT;
  const int s_max = X_SMEM_BYTES / (M * KT * 2);
  p.n_kr = (p.nst + s_max - 1) / s_max;
  p.S = (p.nst + p.n_kr - 1) / p.n_kr;
  p.n_kr = (p.nst + p.S - 1) / p.S;           // drop empty trailing ranges
  p.ctas_per_kr = sm_count / p.n_kr;
  if (p.ctas_per_kr < 1) p.ctas_per_kr = 1;
  const long long T = static_cast<long long>(p.n_rb) * p.S;
  if (p.ctas_per_kr > T) p.ctas_per_kr = static_cast<int>(T);
  // a row block of S tiles can straddle at most S / min_tiles_per_cta + 2 CTAs of a k-range;
  // the last (shorter) range has its own, smaller T -- bound with the worst of the two
  int max_split = 1;
  for (int kr = 0; kr < p.n_kr; ++kr) {
    const Sched s = make_sched(p, kr);
    const long long min_tiles = s.T / s.G;
    const int b = static_cast<int>(s.S_kr / (min_tiles > 0 ? min_tiles : 1)) + 2;
    if (b > max_split) max_split = b;
  }
  p.max_split = max_split;
  pl.grid = p.n_kr * p.ctas_per_kr;
  pl.MT = M <= 8 ? 1 : 2;
  pl.smem_bytes = smem_layout(M, 8 * pl.MT, p.S).total + 1024;
  pl.counters_bytes = COUNTER_BYTES;
  pl.workspace_bytes = pl.counters_bytes +
                       static_cast<size_t>(p.n_rb) * p.n_kr * p.max_split * M * ROWS * sizeof(float);
  return pl;
}

template <int MT, typename OT>
int launch_t(const Plan& pl, const CUtensorMap& tw, const CUtensorMap& ts, cudaStream_t stream) {
  auto kern = w4a16_gemv_kernel<MT, OT>;
  static thread_local int configured_device = -1;  // per (thread, template instance)
  int dev = 0;
  LCQ_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_device != dev) {
    LCQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured_device = dev;
  }
  kern<<<pl.grid, NTHREADS, pl.smem_bytes, stream>>>(tw, ts, pl.p);
  LCQ_CUDA_TRY(cudaGetLastError());
  return LCQ_OK;
}

inline int launch(const void* x, const void* w, const void* s, void* out, int M, int N, int K, int x_dtype,
                  int out_dtype, void* workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream) {
  Plan pl = make_plan(M, N, K, sm_count);
  if (workspace == nullptr || workspace_bytes < pl.workspace_bytes || !aligned(workspace, 256)) {
    set_error("w4a16 gemv: workspace of %zu bytes (256-byte aligned) required, got %zu", pl.workspace_bytes,
              workspace_bytes);
    return LCQ_ERR_WORKSPACE;
  }
  if (!aligned(w, 16) || !aligned(s, 16) || !aligned(x, 16)) {
    set_error("w4a16 gemv: x, w_packed and scales must be 16-byte aligned");
    return LCQ_ERR_BAD_ARG;
  }
  pl.p.x = x;
  pl.p.out = out;
  pl.p.x_is_bf16 = (x_dtype == LCQ_BF16);
  pl.p.counters = static_cast<int*>(workspace);
  pl.p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + pl.counters_bytes);
  CUtensorMap tw, ts;
  int rc = encode_tmap_2d(&tw, 0, w, static_cast<uint64_t>(K) / 2, static_cast<uint64_t>(N),
                          static_cast<uint64_t>(K) / 2, KT / 2, ROWS, 3);
  if (rc != LCQ_OK) return rc;
  rc = encode_tmap_2d(&ts, 1, s, static_cast<uint64_t>(K) / 32, static_cast<uint64_t>(N),
                      static_cast<uint64_t>(K) / 16, GT, ROWS, 0);
  if (rc != LCQ_OK) return rc;
#define LCQ_GEMV_TC_CASE(MT_)                                                                 \
  switch (out_dtype) {                                                                        \
    case LCQ_F32: return launch_t<MT_, float>(pl, tw, ts, stream);                            \
    case LCQ_F16: return launch_t<MT_, __half>(pl, tw, ts, stream);                           \
    case LCQ_BF16: return launch_t<MT_, __nv_bfloat16>(pl, tw, ts, stream);                   \
    default: break;                                                                           \
  }
  if (pl.MT == 1) { LCQ_GEMV_TC_CASE(1) } else { LCQ_GEMV_TC_CASE(2) }
#undef LCQ_GEMV_TC_CASE
  set_error("w4a16 gemv: bad out_dtype %d", out_dtype);
  return LCQ_ERR_BAD_ARG;
}

}  // namespace gemv_tc
}  // namespace lcq
