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
// nibble positions come out scaled by 2^-24.  One 32-wide group is two m16n8k16 MMAs
// giving D = 2^-24 * sum x*q, after which  acc += scale * D  in float32.
//
// The zero point (-8) is a separate, tiny contraction:  -8 * sum_g scale[n,g] * xsum[g,m]
// with xsum[g,m] = sum_{k in g} x[m,k].  Per 256-wide tile that is ONE more MMA whose
// A operand is the tile's 8 fp16 scales per row and whose B operand is -8*xsum split into
// an fp16 high part (k slots 0-7) and an fp16 residual (k slots 8-15), accumulated in its
// own float32 registers (B carries -8*xsum*2^-9 so it cannot overflow fp16).
// Result: out = acc * 2^24 + corr * 2^9.
//
// Work decomposition.  A tile is 128 rows x 256 k (16 KB of packed weights + 2 KB of
// scales, one TMA box each).  K is cut into n_kr ranges so that one range of x fits in
// shared memory; the CTAs of a range split its tile sequence (row-block major) evenly,
// stream-K style, so the last wave is never ragged.  A row block whose tiles were produced
// by more than one CTA is combined through scratch: every contributor writes its float32
// partial, bumps a counter (one per row block and 16-row warp slab, so warps never wait for
// each other), and the last one sums all partials in a fixed order, writes the output and
// resets the counter.  Nobody spins.
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
constexpr int NCW = 8;                       // consumer warps, 16 rows each
constexpr int NTHREADS = (NCW + 1) * 32;     // + 1 producer warp
constexpr int BAR_CONSUMERS = 1;             // named barrier id for the consumer warps
// The workspace starts with a counter region of FIXED size so that it sits at the same place
// for every problem: only the counters must be zero on entry (and are zero again on exit);
// the partials behind them are scratch that successive calls may leave dirty.
constexpr int MAX_ROW_BLOCKS = 16384;
constexpr size_t COUNTER_BYTES = kWorkspaceCounterBytes;  // one int per (row block, 16-row slab)
static_assert(static_cast<size_t>(MAX_ROW_BLOCKS) * NCW * sizeof(int) <= COUNTER_BYTES, "counter region too small");

// Per m-tile-count configuration: M <= 8 runs two CTAs per SM (16 consumer warps hide the
// shared-memory and MMA latencies), M <= 16 one CTA with a deeper ring.
template <int MT> struct Cfg;
// XC_BYTES: shared memory left for the staged activations and zero-point operands.
template <> struct Cfg<1> { static constexpr int NSTAGES = 4, CTAS_PER_SM = 2, XC_BYTES = 40000; };
template <> struct Cfg<2> { static constexpr int NSTAGES = 6, CTAS_PER_SM = 1, XC_BYTES = 118000; };
// bytes of x (M rows, exact) + zero-point operands (padded to 8*MT columns) per 256-wide tile
__host__ __device__ inline int xc_bytes_per_tile(int M, int MT) { return GT * M * 64 + MT * 256; }

struct Params {
  const void* x;        // [M, K] fp16 or bf16
  void* out;            // [M, N]
  float* partials;      // [n_rb][n_kr * max_split][M][ROWS]
  int* counters;        // [n_rb][NCW], zero on entry, zero on exit
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

struct SmemLayout {     // offsets from the 1024-byte aligned base
  int xs;       // staged activations: [group][M][4] x 16 B (+ 64 spare bytes)
  int corr;     // zero-point operands: [tile][MT][8 m][4 t] x 8 B  (hi pair, lo pair)
  int bars;     // full[NSTAGES], empty[NSTAGES]
  int flags;    // abort flag
  int total;
};
__host__ __device__ inline SmemLayout smem_layout(int nstages, int M, int MT, int S) {
  SmemLayout L;
  L.xs = nstages * STAGE_BYTES;
  L.corr = L.xs + S * GT * M * 64 + 64;
  L.bars = L.corr + S * MT * 8 * 4 * 8;
  L.flags = L.bars + 2 * nstages * 8;
  L.total = L.flags + 16;
  return L;
}

template <typename T> __device__ __forceinline__ void store_out(T* out, long long idx, float v) { out[idx] = from_f32<T>(v); }

// MT: 8-wide m tiles (1 or 2).  NC: output columns each lane keeps per m tile (1 when M == 1,
// where only column 0 exists, else 2).
template <int MT, int NC, typename OT>
__global__ void __launch_bounds__(NTHREADS, Cfg<MT>::CTAS_PER_SM)
w4a16_gemv_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_s,
                  const Params p) {
  constexpr int NSTAGES = Cfg<MT>::NSTAGES;
  // Declared 1024-byte aligned (the 128-byte TMA swizzle needs it) and used directly, so the
  // compiler keeps every access in the shared address space with 32-bit addressing.
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicExch(&g_device_status, 3);
    return;
  }

  const int kr = blockIdx.x % p.n_kr;
  const int j = blockIdx.x / p.n_kr;
  const Sched sch = make_sched(p, kr);
  if (j >= sch.G) return;  // whole CTA leaves together; nothing was started
  const long long t0 = tile_begin(sch, j), t1 = tile_begin(sch, j + 1);

  const SmemLayout L = smem_layout(NSTAGES, p.M, MT, p.S);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L.bars);
  uint64_t* empty_bar = full_bar + NSTAGES;
  volatile int* flag_abort = reinterpret_cast<volatile int*>(smem + L.flags);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], NCW); }
    *flag_abort = 0;
    fence_barrier_init();
    // Programmatic dependent launch: let the next kernel on the stream become resident as our
    // CTAs retire.  Its producer warp may then prefetch weights (constants) while we finish;
    // everything that reads activations or touches out / workspace waits for us below.
    griddep_launch_dependents();
  }
  __syncthreads();

  if (warp == NCW) {
    // ------------------------------------------------------------ producer warp
    // (weights and scales only: they are not produced by the preceding kernel, so no dependency wait)
    if (lane == 0) {
      tma_prefetch_desc(&tmap_w);
      tma_prefetch_desc(&tmap_s);
      int it = 0;
      int rb = static_cast<int>(t0 / sch.S_kr);
      int ks = static_cast<int>(t0 - static_cast<long long>(rb) * sch.S_kr);
      for (long long t = t0; t < t1; ++t, ++it) {
        const int s = it % NSTAGES;
        const uint32_t ph = (it / NSTAGES) & 1;
        if (*flag_abort) break;
        if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1)) {
          *flag_abort = 1; atomicExch(&g_device_status, 1);
          break;
        }
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
    uint8_t* corr = smem + L.corr;

    // ---- stage this k-range of x: permuted element order, fp16, high-nibble slots / 16;
    //      and the zero-point operands -8 * xsum * 2^-9 as fp16 (high part, residual)
    griddep_wait();   // x may be the previous kernel's output; out / workspace may still be in its use
    {
      // Only the k tiles this CTA will actually visit are staged: its tile range starts at tile
      // ks0 of a row block and wraps around the k-range, so it touches min(n_tiles, S_kr) tiles.
      const int ks0 = static_cast<int>(t0 % sch.S_kr);
      const long long span = t1 - t0;
      const int need_tiles = span < sch.S_kr ? static_cast<int>(span) : sch.S_kr;
      const int oct_per_row = need_tiles * (KT / 8);
      const int total = p.M * oct_per_row;
      const long long kbase = static_cast<long long>(kr) * p.S * KT;
      // zero the zero-point operands (rows m >= M stay zero)
      {
        uint4* z = reinterpret_cast<uint4*>(smem + L.corr - 64);
        const int zero16 = (L.bars - (L.corr - 64)) / 16;
        for (int i = ctid; i < zero16; i += NCW * 32) z[i] = make_uint4(0u, 0u, 0u, 0u);
      }
      named_bar_sync(BAR_CONSUMERS, NCW * 32);
      constexpr int U = 4;   // independent 16-byte loads in flight per thread
      for (int base = 0; base < total; base += U * NCW * 32) {
        uint4 raw[U];
        int mm[U], oo[U];
        bool ok[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int idx = base + u * NCW * 32 + ctid;
          ok[u] = idx < total;
          mm[u] = ok[u] ? idx / oct_per_row : 0;
          {
            const int ol = ok[u] ? idx - mm[u] * oct_per_row : 0;       // octet within the visited tiles
            int ks = ks0 + (ol >> 5);                                    // 32 octets per 256-k tile
            if (ks >= sch.S_kr) ks -= sch.S_kr;
            oo[u] = ks * (KT / 8) + (ol & 31);
          }
          raw[u] = make_uint4(0u, 0u, 0u, 0u);
          if (ok[u]) {
            const long long off = static_cast<long long>(mm[u]) * p.K + kbase + 8 * oo[u];
            raw[u] = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.x) + off));
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          float v[8];
          const uint32_t* rw = reinterpret_cast<const uint32_t*>(&raw[u]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (p.x_is_bf16) {
              v[2 * e] = __uint_as_float(rw[e] << 16);
              v[2 * e + 1] = __uint_as_float(rw[e] & 0xFFFF0000u);
            } else {
              const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&rw[e]));
              v[2 * e] = f.x; v[2 * e + 1] = f.y;
            }
          }
          float sum = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          if (ok[u]) {
            const int m = mm[u], o = oo[u];
            const __half2 h0 = __floats2half2_rn(v[0], v[4]);
            const __half2 h1 = __floats2half2_rn(v[1] * 0.0625f, v[5] * 0.0625f);
            const __half2 h2 = __floats2half2_rn(v[2], v[6]);
            const __half2 h3 = __floats2half2_rn(v[3] * 0.0625f, v[7] * 0.0625f);
            uint4 q;
            q.x = *reinterpret_cast<const uint32_t*>(&h0); q.y = *reinterpret_cast<const uint32_t*>(&h1);
            q.z = *reinterpret_cast<const uint32_t*>(&h2); q.w = *reinterpret_cast<const uint32_t*>(&h3);
            const int grp = o >> 2;
            xs[(grp * p.M + m) * 4 + (o & 3)] = q;
            if ((o & 3) == 0) {
              const float zp = -0.015625f * sum;   // -8 * xsum * 2^-9: stays inside fp16 range for any fp16 x
              const __half hi = __float2half_rn(zp);
              const __half lo = __float2half_rn(zp - __half2float(hi));
              const int tile = grp >> 3, gi = grp & 7;
              uint8_t* cp = corr + ((((tile * MT + (m >> 3)) * 8 + (m & 7)) * 4 + (gi >> 1)) * 8) + (gi & 1) * 2;
              *reinterpret_cast<__half*>(cp) = hi;
              *reinterpret_cast<__half*>(cp + 4) = lo;
            }
          }
        }
      }
      named_bar_sync(BAR_CONSUMERS, NCW * 32);
    }

    float acc[MT][4], cor[MT][4];
#pragma unroll
    for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
      for (int e = 0; e < 4; ++e) { acc[jm][e] = 0.0f; cor[jm][e] = 0.0f; }
    }

    float zero4[4];
    opaque_zero4(zero4);

    const int r0 = warp * 16 + g;
    // byte offset of (row r0, word t4) inside a stage with the row's swizzle folded in:
    // chunk c of that row sits at  lane_off ^ (c << 4)   (rows r0 and r0+8 share r & 7)
    const uint32_t lane_off = static_cast<uint32_t>(r0 * 128 + 4 * t4) ^ (static_cast<uint32_t>(g & 7) << 4);
    // x fragment of lane (g, t4) for m tile jm: row m = 8*jm + g of group grp sits at
    // xs[(grp*M + m)*4 + t4].  A lane whose m does not exist reads row M-1 instead: B column m only
    // feeds D column m, and columns >= M are never stored.
    const uint4* xs_lane[MT];
#pragma unroll
    for (int jm = 0; jm < MT; ++jm) {
      const int m = (8 * jm + g) < p.M ? (8 * jm + g) : p.M - 1;
      xs_lane[jm] = xs + m * 4 + t4;
    }
    const int xs_stride = (NC == 1) ? 4 : p.M * 4;     // uint4 per group; NC == 1 means M == 1
    const uint2* corr_lane = reinterpret_cast<const uint2*>(corr) + g * 4 + t4;  // + (tile*MT + jm)*32

    bool dead = false;
    int rb = static_cast<int>(t0 / sch.S_kr);
    int ks = static_cast<int>(t0 - static_cast<long long>(rb) * sch.S_kr);
    const int n_tiles = static_cast<int>(t1 - t0);
    int s = 0;
    uint32_t ph = 0;
    for (int ti = 0; ti < n_tiles; ++ti) {
      const long long t = t0 + ti;
      if (!dead) {
        if (*flag_abort || !mbar_wait_bounded(&full_bar[s], ph)) {
          dead = true; *flag_abort = 1; atomicExch(&g_device_status, 2);
        }
      }
      if (!dead) {
        const uint8_t* ws = smem + s * STAGE_BYTES;
        const uint32_t* srA = reinterpret_cast<const uint32_t*>(ws + W_BYTES + r0 * 16);
        const uint32_t* srB = reinterpret_cast<const uint32_t*>(ws + W_BYTES + (r0 + 8) * 16);
        const uint4 sA = *reinterpret_cast<const uint4*>(srA);
        const uint4 sB = *reinterpret_cast<const uint4*>(srB);
        float scA[GT], scB[GT];   // the tile's 8 scales of rows r0 and r0+8
        {
          const uint32_t wA[4] = {sA.x, sA.y, sA.z, sA.w}, wB[4] = {sB.x, sB.y, sB.z, sB.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&wA[i]));
            const float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&wB[i]));
            scA[2 * i] = fa.x; scA[2 * i + 1] = fa.y; scB[2 * i] = fb.x; scB[2 * i + 1] = fb.y;
          }
        }
        const uint4* xp[MT];
#pragma unroll
        for (int jm = 0; jm < MT; ++jm) xp[jm] = xs_lane[jm] + ks * GT * xs_stride;
        const uint32_t tile_off = static_cast<uint32_t>(s * STAGE_BYTES) + lane_off;   // stage bases are 1024-aligned: the XOR below only flips chunk bits
#pragma unroll
        for (int c = 0; c < GT; ++c) {
          const uint32_t off = tile_off ^ (static_cast<uint32_t>(c) << 4);
          const uint32_t wa = *reinterpret_cast<const uint32_t*>(smem + off);
          const uint32_t wb = *reinterpret_cast<const uint32_t*>(smem + off + 1024);
          const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
#pragma unroll
          for (int jm = 0; jm < MT; ++jm) {
            const uint4 bx = xp[jm][c * xs_stride];
            float d[4];
            mma_m16n8k16_f16(d, wa & 0x000F000Fu, wb & 0x000F000Fu, wa & 0x00F000F0u, wb & 0x00F000F0u,
                             bx.x, bx.y, zero4);
            mma_m16n8k16_f16(d, wa8 & 0x000F000Fu, wb8 & 0x000F000Fu, wa8 & 0x00F000F0u, wb8 & 0x00F000F0u,
                             bx.z, bx.w, d);
            acc[jm][0] = fmaf(scA[c], d[0], acc[jm][0]);
            acc[jm][2] = fmaf(scB[c], d[2], acc[jm][2]);
            if (NC == 2) {
              acc[jm][1] = fmaf(scA[c], d[1], acc[jm][1]);
              acc[jm][3] = fmaf(scB[c], d[3], acc[jm][3]);
            }
          }
        }
        // zero point of the whole tile: A = the rows' 8 scales (k slots 0-7 and again 8-15),
        // B = (-8*xsum*2^-9) high parts | residuals
        const uint32_t sa_w = srA[t4], sb_w = srB[t4];
#pragma unroll
        for (int jm = 0; jm < MT; ++jm) {
          const uint2 cb = corr_lane[(ks * MT + jm) * 32];
          mma_m16n8k16_f16(cor[jm], sa_w, sb_w, sa_w, sb_w, cb.x, cb.y, cor[jm]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);  // also in the dead state, so the producer never stalls on us
      if (++s == NSTAGES) { s = 0; ph ^= 1; }

      // ---- end of this CTA's share of row block rb: flush.  Each warp settles its own
      //      16-row slab, so no CTA-wide barrier is needed and the other warps keep streaming.
      if (ks == sch.S_kr - 1 || t == t1 - 1) {
        const int nA = rb * ROWS + r0, nB = nA + 8;
        float y[MT][4];
#pragma unroll
        for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
          for (int e = 0; e < 4; ++e) y[jm][e] = fmaf(acc[jm][e], 16777216.0f, cor[jm][e] * 512.0f);
        }
        const long long rb_t0 = static_cast<long long>(rb) * sch.S_kr;
        const bool whole = p.n_kr == 1 && rb_t0 >= t0 && rb_t0 + sch.S_kr <= t1;
        if (whole) {
          OT* out = static_cast<OT*>(p.out);
#pragma unroll
          for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
            for (int e = 0; e < NC; ++e) {
              const int m = 8 * jm + 2 * t4 + e;
              if (m < p.M) {
                if (nA < p.N) store_out(out, static_cast<long long>(m) * p.N + nA, y[jm][e]);
                if (nB < p.N) store_out(out, static_cast<long long>(m) * p.N + nB, y[jm][2 + e]);
              }
            }
          }
        } else {
          // contributors: identical for every full-length k-range, the last range may differ
          int j0, j1, c_full, c_last;
          cover(sch, rb, j0, j1);
          {
            int a0, a1;
            const Sched sf = make_sched(p, 0);
            cover(sf, rb, a0, a1);
            c_full = a1 - a0 + 1;
            const Sched sl = make_sched(p, p.n_kr - 1);
            cover(sl, rb, a0, a1);
            c_last = a1 - a0 + 1;
          }
          const int n_contrib = (p.n_kr - 1) * c_full + c_last;
          const int slot = kr * p.max_split + (j - j0);
          const long long slot_elems = static_cast<long long>(p.M) * ROWS;
          float* rb_part = p.partials + static_cast<long long>(rb) * p.n_kr * p.max_split * slot_elems;
          float* part = rb_part + slot * slot_elems;
          int* counter = p.counters + rb * NCW + warp;
          // Shortcut: if every other contributor has already published its partial, this warp is
          // the one that completes the slab -- add the others to the values still in registers and
          // write the output, without publishing (no global round trip at the kernel's tail).
          int seen = 0;
          if (lane == 0) seen = *reinterpret_cast<volatile int*>(counter);
          seen = __shfl_sync(0xffffffffu, seen, 0);
          if (seen == n_contrib - 1) {
            __threadfence();
            OT* out = static_cast<OT*>(p.out);
#pragma unroll
            for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
              for (int e = 0; e < NC; ++e) {
                const int m = 8 * jm + 2 * t4 + e;
                if (m < p.M) {
                  float sa = 0.0f, sb = 0.0f;      // same slot order as the reducer below: bit-identical result
                  for (int kk = 0; kk < p.n_kr; ++kk) {
                    const int cnt = (kk == p.n_kr - 1) ? c_last : c_full;
                    for (int c = 0; c < cnt; ++c) {
                      const int os = kk * p.max_split + c;
                      const float* src = rb_part + os * slot_elems + m * ROWS + r0;
                      sa += (os == slot) ? y[jm][e] : __ldcg(src);
                      sb += (os == slot) ? y[jm][2 + e] : __ldcg(src + 8);
                    }
                  }
                  if (nA < p.N) store_out(out, static_cast<long long>(m) * p.N + nA, sa);
                  if (nB < p.N) store_out(out, static_cast<long long>(m) * p.N + nB, sb);
                }
              }
            }
            __syncwarp();
            if (lane == 0) *counter = 0;
          } else {
#pragma unroll
          for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
            for (int e = 0; e < NC; ++e) {
              const int m = 8 * jm + 2 * t4 + e;
              if (m < p.M) {
                __stcg(part + m * ROWS + r0, y[jm][e]);
                __stcg(part + m * ROWS + r0 + 8, y[jm][2 + e]);
              }
            }
          }
          __threadfence();
          __syncwarp();
          int last = 0;
          if (lane == 0) last = (atomicAdd(counter, 1) == n_contrib - 1) ? 1 : 0;
          last = __shfl_sync(0xffffffffu, last, 0);
          if (last) {
            __threadfence();
            OT* out = static_cast<OT*>(p.out);
            for (int idx = lane; idx < p.M * 16; idx += 32) {
              const int m = idx >> 4, r = warp * 16 + (idx & 15);
              const float* src = rb_part + m * ROWS + r;
              float sum = 0.0f;
              for (int kk = 0; kk < p.n_kr; ++kk) {
                const int cnt = (kk == p.n_kr - 1) ? c_last : c_full;
                for (int c = 0; c < cnt; ++c) sum += __ldcg(src + (kk * p.max_split + c) * slot_elems);
              }
              const int n = rb * ROWS + r;
              if (n < p.N) store_out(out, static_cast<long long>(m) * p.N + n, sum);
            }
            if (lane == 0) p.counters[rb * NCW + warp] = 0;
          }
          }   // published path
        }
#pragma unroll
        for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
          for (int e = 0; e < 4; ++e) { acc[jm][e] = 0.0f; cor[jm][e] = 0.0f; }
        }
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
  pl.MT = M <= 8 ? 1 : 2;
  const int nstages = pl.MT == 1 ? Cfg<1>::NSTAGES : Cfg<2>::NSTAGES;
  const int ctas_per_sm = pl.MT == 1 ? Cfg<1>::CTAS_PER_SM : Cfg<2>::CTAS_PER_SM;
  const int xc_bytes = pl.MT == 1 ? Cfg<1>::XC_BYTES : Cfg<2>::XC_BYTES;
  p.n_rb = (N + ROWS - 1) / ROWS;
  p.nst = K / KT;
  const int s_max = xc_bytes / xc_bytes_per_tile(M, pl.MT);
  p.n_kr = (p.nst + s_max - 1) / s_max;
  p.S = (p.nst + p.n_kr - 1) / p.n_kr;
  p.n_kr = (p.nst + p.S - 1) / p.S;           // drop empty trailing ranges
  p.ctas_per_kr = (sm_count * ctas_per_sm) / p.n_kr;
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
  pl.smem_bytes = smem_layout(nstages, M, pl.MT, p.S).total;
  pl.counters_bytes = COUNTER_BYTES;
  pl.workspace_bytes = pl.counters_bytes +
                       static_cast<size_t>(p.n_rb) * p.n_kr * p.max_split * M * ROWS * sizeof(float);
  return pl;
}

template <int MT, int NC, typename OT>
int launch_t(const Plan& pl, const CUtensorMap& tw, const CUtensorMap& ts, bool allow_pdl, cudaStream_t stream) {
  auto kern = w4a16_gemv_kernel<MT, NC, OT>;
  static thread_local int configured_device = -1;  // per (thread, template instance)
  int dev = 0;
  LCQ_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_device != dev) {
    LCQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (227 * 1024) / Cfg<MT>::CTAS_PER_SM - 1024));
    LCQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                                      cudaSharedmemCarveoutMaxShared));
    configured_device = dev;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(pl.grid);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = pl.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (allow_pdl && pdl_enabled()) ? 1 : 0;
  LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tw, ts, pl.p));
  return LCQ_OK;
}

template <typename OT>
int launch_o(const Plan& pl, const CUtensorMap& tw, const CUtensorMap& ts, bool allow_pdl, cudaStream_t stream) {
  if (pl.MT == 2) return launch_t<2, 2, OT>(pl, tw, ts, allow_pdl, stream);
  if (pl.p.M == 1) return launch_t<1, 1, OT>(pl, tw, ts, allow_pdl, stream);
  return launch_t<1, 2, OT>(pl, tw, ts, allow_pdl, stream);
}

inline int launch(const void* x, const void* w, const void* s, void* out, int M, int N, int K, int x_dtype,
                  int out_dtype, void* workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream,
                  bool allow_pdl = true) {
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
  switch (out_dtype) {
    case LCQ_F32: return launch_o<float>(pl, tw, ts, allow_pdl, stream);
    case LCQ_F16: return launch_o<__half>(pl, tw, ts, allow_pdl, stream);
    case LCQ_BF16: return launch_o<__nv_bfloat16>(pl, tw, ts, allow_pdl, stream);
    default: break;
  }
  set_error("w4a16 gemv: bad out_dtype %d", out_dtype);
  return LCQ_ERR_BAD_ARG;
}

}  // namespace gemv_tc
}  // namespace lcq
