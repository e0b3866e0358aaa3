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
// The zero point (-8) rides in the MMA's accumulator input:  -8 * sum_{k in g} x[m,k] =
// -8 * xsum[g,m] is the same for every weight row, so the first MMA of a group starts from
// C[n, m] = -8 * xsum[g,m] * 2^-24 (float32, staged next to the activations) instead of zero.
// Result: out = acc * 2^24.
//
// Work decomposition.  A tile is 128 rows x 256 k (16 KB of packed weights + 2 KB of
// scales).  Inside a CTA the consumer warps split a tile as 4 row groups of 32 rows x PARTS
// slices of the tile's 8 groups; a warp loads an activation fragment once and uses it for
// both 16-row slabs of its row group (shared-memory bandwidth, not issue rate, bounds the
// M = 16 case), and the slices of a row group are added through shared memory when a row
// block ends.  K is cut into n_kr ranges so that one range of x fits in shared memory; the
// CTAs of a range split its tile sequence (row-block major) stream-K style.  A row block
// whose tiles were produced by more than one CTA is combined through scratch: every
// contributor writes its float32 partial, bumps a counter (one per row block and row
// group), and the last one sums all partials in a fixed order, writes the output and resets
// the counter.  Nobody spins on another CTA.  At M > 8 (two m tiles) the zero point is
// taken off the weights instead (see MAGIC in the kernel): shared-memory bandwidth bounds
// that case, and it saves the fetch of the zero-point quads.
//
// Small problems (fewer than ~4 tiles per CTA) run in cluster mode: a thread-block cluster
// of 2, 4 or 8 CTAs owns a row block, every CTA streams its share of the k tiles, and the
// partial sums meet in the first CTA's shared memory (remote stores + remote mbarrier
// arrivals over distributed shared memory) -- no scratch, no counters, no global round trip.
//
// Any K that is a multiple of 64: the last k tile may be partial (TMA fills the missing
// bytes with zeros).  When K is not a multiple of 256 the scale rows are not 16-byte
// multiples and no tensor map can describe them; the producer warp then fetches the tile's
// scales with 4-byte cp.async copies that arrive on the same mbarrier.
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
constexpr int NRG = 4;                       // row groups of 32 rows per tile
constexpr int BAR_CONSUMERS = 1;             // named barrier ids: consumers; slice hand-over per row group
constexpr int BAR_FULL0 = 2, BAR_FREE0 = 6;
// The workspace starts with a counter region of FIXED size so that it sits at the same place
// for every problem: only the counters must be zero on entry (and are zero again on exit);
// the partials behind them are scratch that successive calls may leave dirty.
constexpr int MAX_ROW_BLOCKS = 16384;
constexpr int COUNTERS_PER_RB = 8;
constexpr size_t COUNTER_BYTES = kWorkspaceCounterBytes;  // ints per (row block, row group)
static_assert(static_cast<size_t>(MAX_ROW_BLOCKS) * COUNTERS_PER_RB * sizeof(int) <= COUNTER_BYTES, "counter region too small");

// Per m-tile-count configuration.  M <= 8: 8 consumer warps, two CTAs per SM (the second CTA of
// an SM is also what lets the next kernel of a stream become resident early).  M <= 16: the
// activations of a k range take 8 KB per tile, so one CTA owns the SM, with 16 consumer warps.
template <int MT> struct Cfg;
template <> struct Cfg<1> { static constexpr int NCW = 8, NSTAGES = 4, CTAS_PER_SM = 2; };
template <> struct Cfg<2> { static constexpr int NCW = 16, NSTAGES = 6, CTAS_PER_SM = 1; };
// Ring depth.  In cluster mode a CTA owns at most S / cluster tiles of one row block, so a short ring
// holds (nearly) all of them and leaves room for the reduction buffer.
__host__ __device__ constexpr int nstages_for(int MT, bool CL) { return MT == 1 ? (CL ? 3 : Cfg<1>::NSTAGES) : (CL ? 4 : Cfg<2>::NSTAGES); }
// bytes one CTA hands to its cluster leader per row group: 2 slabs x MT x 4 values x 32 lanes x 4 B
__host__ __device__ constexpr int red_slot_bytes(int MT) { return 2 * MT * 4 * 32 * 4; }
__host__ __device__ constexpr int max_dynamic_smem(int ctas_per_sm) { return (227 * 1024) / ctas_per_sm - (ctas_per_sm > 1 ? 1024 : 0); }
// bytes of the slice hand-over buffer: (PARTS - 1) writers x 4 row groups x 2 slabs x MT x 4 values x 32 lanes
__host__ __device__ constexpr int comb_bytes(int MT) { return ((MT == 1 ? 8 : 16) / NRG - 1) * NRG * 2 * MT * 4 * 32 * 4; }
// bytes of the zero-point quads of one group: one 16-byte quad per pair of x rows (a single quad at MPAD = 1)
__host__ __device__ constexpr int zq_group_bytes(int MPAD) { return MPAD == 1 ? 16 : MPAD * 8; }
// bytes of staged x (MPAD rows) + zero-point quads per 256-wide tile
__host__ __device__ inline int xc_bytes_per_tile(int MPAD, int MT) { (void)MT; return GT * MPAD * 64 + GT * zq_group_bytes(MPAD); }

struct Params {
  const void* x;        // [M, K] fp16 or bf16
  void* out;            // [M, N]
  const void* scales;   // [N, K/32] fp16 (read directly when K % 256 != 0)
  float* partials;      // [n_rb][n_kr * max_split][M][ROWS]
  int* counters;        // [n_rb][COUNTERS_PER_RB], zero on entry, zero on exit
  int M, N, K;
  int x_is_bf16;
  int out_dtype;        // LCQ_F32 / LCQ_F16 / LCQ_BF16
  int n_rb;             // ceil(N / ROWS)
  int n_kr;             // k ranges
  int S;                // tiles (of 256 k) per k-range; the last range may hold fewer
  int nst;              // ceil(K / 256)
  int ctas_per_kr;      // CTAs working on one k-range
  int max_split;        // scratch slots per (row block, k-range)
  int x_tiles;          // k tiles of x a CTA keeps in shared memory (S, or ceil(S / cluster) in cluster mode)
  int cluster;          // CTAs per row block that reduce through distributed shared memory (1 = none)
};

// The share of one k-range's tile sequence owned by one CTA.  Tile counts are 32-bit: the plan
// refuses problems where (T + 1) * G would not fit in 32 bits (see make_plan).
struct Sched {
  int S_kr;             // tiles per row block in this k-range
  unsigned T;           // n_rb * S_kr
  int G;                // CTAs on this k-range (<= T)
};

__host__ __device__ inline Sched make_sched(const Params& p, int kr) {
  Sched s;
  const int left = p.nst - kr * p.S;
  s.S_kr = left < p.S ? left : p.S;
  s.T = static_cast<unsigned>(p.n_rb) * static_cast<unsigned>(s.S_kr);
  s.G = static_cast<unsigned>(p.ctas_per_kr) < s.T ? p.ctas_per_kr : static_cast<int>(s.T);
  return s;
}
__host__ __device__ inline unsigned tile_begin(const Sched& s, int j) { return (static_cast<unsigned>(j) * s.T) / static_cast<unsigned>(s.G); }
__host__ __device__ inline int owner_of(const Sched& s, unsigned t) {
  return static_cast<int>(((t + 1u) * static_cast<unsigned>(s.G) - 1u) / s.T);
}
// CTAs j0..j1 (inclusive) of this k-range contribute to row block rb.
__host__ __device__ inline void cover(const Sched& s, int rb, int& j0, int& j1) {
  j0 = owner_of(s, static_cast<unsigned>(rb) * s.S_kr);
  j1 = owner_of(s, static_cast<unsigned>(rb + 1) * s.S_kr - 1u);
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
  int comb;     // slice hand-over buffer
  int xs;       // staged activations: [visited tile][group][MPAD][4] x 16 B (+ 64 spare bytes)
  int zps;      // zero-point quads: [visited tile][group][row pair] x {z(m0), z(m1), z(m0), z(m1)}, z = -8 * xsum * 2^-24 (+ 64 spare bytes)
  int bars;     // full[NSTAGES], empty[NSTAGES], red[NRG]
  int flags;    // CtaInfo (abort flag first)
  int red;      // cluster mode, read by the leader only: [rank - 1][row group] slots of red_slot_bytes(MT)
  int total;
};
__host__ __device__ inline SmemLayout smem_layout(int nstages, int MPAD, int MT, int x_tiles, int cluster) {
  SmemLayout L;
  L.comb = nstages * STAGE_BYTES;
  L.xs = L.comb + comb_bytes(MT);
  L.zps = L.xs + x_tiles * GT * MPAD * 64 + 64;
  L.bars = L.zps + x_tiles * GT * zq_group_bytes(MPAD) + 64;
  L.flags = L.bars + (2 * nstages + NRG) * 8;
  L.red = L.flags + 64;
  L.total = L.red + (cluster > 1 ? (cluster - 1) * NRG * red_slot_bytes(MT) : 0);
  return L;
}

__device__ __forceinline__ void store_out(void* out, int dtype, long long idx, float v) {
  if (dtype == LCQ_F16) static_cast<__half*>(out)[idx] = __float2half_rn(v);
  else if (dtype == LCQ_BF16) static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
  else static_cast<float*>(out)[idx] = v;
}

__device__ __forceinline__ void named_bar_arrive(int id, int nthreads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// 4-byte asynchronous copy global -> shared; src_bytes = 0 writes zeros instead.
__device__ __forceinline__ void cp_async_4(uint32_t dst_smem, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes) : "memory");
}
// The mbarrier receives one arrival from this thread once all its earlier cp.async copies have landed.
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Shared-memory loads and mbarrier operations on 32-bit shared-space addresses.
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ void mbar_arrive_a(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_a(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Slow path of a bounded wait, out of line: polls in batches, gives up when the CTA's abort flag
// is set or the library's wait limit has passed.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, uint32_t abort_addr) {
#pragma unroll 1
  for (int i = 0; i < 64; ++i) {
    if (mbar_try_wait_a(bar, parity)) return true;
  }
  const uint64_t t0 = global_timer_ns();
  const uint64_t limit = wait_limit_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait_a(bar, parity)) return true;
    }
    if (lds32(abort_addr) != 0u) return false;
    if (global_timer_ns() - t0 > limit) return false;
  }
}
__device__ __forceinline__ bool mbar_wait_bounded_a(uint32_t bar, uint32_t parity, uint32_t abort_addr) {
  if (mbar_try_wait_a(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_addr);
}

// ---- thread-block cluster helpers (cluster mode: the CTAs of a row block add their partial
//      results in the leader's shared memory instead of going through global scratch)
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Hardware cluster barrier, used once: arrive at kernel entry, wait before the first remote access
// (shared memory of another CTA may only be touched once that CTA has started).
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
// shared::cluster address of `local_addr` (a shared::cta address) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_addr), "r"(rank));
  return a;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// Arrival on another CTA's mbarrier; the release makes this thread's earlier remote stores visible
// to whoever acquires the barrier's phase.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_acq_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded like every other wait of the kernel: gives up at the library's wait limit.
__device__ __noinline__ bool mbar_wait_cluster_bounded(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait_acq_cluster(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  const uint64_t limit = wait_limit_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait_acq_cluster(bar, parity)) return true;
    }
    if (global_timer_ns() - t0 > limit) return false;
  }
}

// q - 8 as fp16 pairs without a conversion: (word & 0x000F000F) | 0x64006400 is {1024 + q, 1024 + q'},
// minus {1032, 1032}; for nibbles in bits 4-7, {1024 + 16 q, ...} minus {1152, 1152} = 16 (q - 8).
__device__ __forceinline__ uint32_t magic_lo(uint32_t w) {
  uint32_t r;
  asm("{\n\t.reg .b32 t;\n\tlop3.b32 t, %1, 0x000F000F, 0x64006400, 0xEA;\n\tsub.f16x2 %0, t, %2;\n\t}" : "=r"(r) : "r"(w), "r"(0x64086408u));
  return r;
}
__device__ __forceinline__ uint32_t magic_hi(uint32_t w) {
  uint32_t r;
  asm("{\n\t.reg .b32 t;\n\tlop3.b32 t, %1, 0x00F000F0, 0x64006400, 0xEA;\n\tsub.f16x2 %0, t, %2;\n\t}" : "=r"(r) : "r"(w), "r"(0x64806480u));
  return r;
}

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// What one thread works out for the whole CTA before the first barrier (schedule arithmetic needs
// several integer divisions; the other threads read the results from shared memory).
struct CtaInfo {
  int abort;            // set when a bounded wait gave up
  int leave;            // this CTA has no tiles
  unsigned t0;          // first tile of the CTA's share
  int n_tiles;
  int rb0, ks0;         // row block and k tile (inside the k-range) of tile t0
  int kr, j;            // k-range and index of the CTA inside it
  int S_kr;
  unsigned T;
  int G;
  int pad;
};
static_assert(sizeof(CtaInfo) == 48, "CtaInfo layout");

// Walks the scratch slots of a row block in slot order: k-range kk holds its contributors in slots
// kk * max_split .. kk * max_split + cnt(kk) - 1.  next() returns -1 when all have been visited.
struct SlotIter {
  int n_kr, c_full, c_last, max_split, kk, c;
  __device__ SlotIter(int n_kr_, int c_full_, int c_last_, int max_split_)
      : n_kr(n_kr_), c_full(c_full_), c_last(c_last_), max_split(max_split_), kk(0), c(0) {}
  __device__ __forceinline__ int next() {
    if (kk >= n_kr) return -1;
    const int os = kk * max_split + c;
    const int cnt = (kk == n_kr - 1) ? c_last : c_full;
    if (++c >= cnt) { c = 0; ++kk; }
    return os;
  }
};

// The row group's values are the outputs (this CTA, or this cluster, produced the whole row block):
// store them.  Inline on purpose: an out-of-line call parks the caller's registers on the stack, and
// with nearly all of L1 carved out as shared memory that round trip goes to L2 (about a microsecond
// per call, measured); typed pointers keep the address arithmetic to one multiply per column.
template <typename OT, int MT, int NC>
__device__ __forceinline__ void store_row_group_t(OT* out, const Params& p, const float (&y)[2][MT][4], int n0, int t4) {
  const bool rows_inside = n0 - (n0 & 7) + 32 <= p.N;      // the row group's 32 rows all exist
#pragma unroll
  for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
    for (int e = 0; e < NC; ++e) {
      const int m = 8 * jm + 2 * t4 + e;
      if (m < p.M) {
        OT* col = out + static_cast<long long>(m) * p.N + n0;
#pragma unroll
        for (int sl = 0; sl < 2; ++sl) {
          if (rows_inside || n0 + 16 * sl < p.N) col[16 * sl] = from_f32<OT>(y[sl][jm][e]);
          if (rows_inside || n0 + 16 * sl + 8 < p.N) col[16 * sl + 8] = from_f32<OT>(y[sl][jm][2 + e]);
        }
      }
    }
  }
}
template <int MT, int NC>
__device__ __forceinline__ void store_row_group(const Params& p, const float (&y)[2][MT][4], int rb, int rg, int g, int t4) {
  const int n0 = rb * ROWS + rg * 32 + g;               // rows n0 + 16*sl and n0 + 16*sl + 8
  if (p.out_dtype == LCQ_F16) store_row_group_t<__half, MT, NC>(static_cast<__half*>(p.out), p, y, n0, t4);
  else if (p.out_dtype == LCQ_BF16) store_row_group_t<__nv_bfloat16, MT, NC>(static_cast<__nv_bfloat16*>(p.out), p, y, n0, t4);
  else store_row_group_t<float, MT, NC>(static_cast<float*>(p.out), p, y, n0, t4);
}

// Settles the 32 rows of one row group of a row block that has several contributors (other CTAs of
// this k-range and / or other k-ranges); called by the row group's slice-0 warp with the slices
// already added up in y: publish the partial, count, and let the last contributor sum all partials
// in slot order -- or, if the counter shows that everybody else has already published, add their
// partials to the values still in registers and write the output without publishing.  `seen_lane0` is the counter value
// lane 0 read (with an acquire load) a tile earlier.  Inline on purpose: an out-of-line call parks
// the caller's registers on the stack, and with nearly all of L1 carved out as shared memory that
// round trip goes to L2 (about a microsecond per call, measured).
template <int MT, int NC>
__device__ __forceinline__ void flush_row_group(const Params& p, const float (&y)[2][MT][4], int rb, int rg, int g, int t4,
                                             int lane, int seen_lane0, const CtaInfo* info) {
  Sched sch;
  sch.S_kr = info->S_kr; sch.T = info->T; sch.G = info->G;
  const int kr = info->kr, j = info->j;
  // contributors: identical for every full-length k-range, the last range may differ
  int j0, j1, c_full, c_last;
  cover(sch, rb, j0, j1);
  c_full = c_last = j1 - j0 + 1;
  if (p.n_kr > 1) {
    int a0, a1;
    if (kr == p.n_kr - 1) {
      const Sched sf = make_sched(p, 0);
      cover(sf, rb, a0, a1);
      c_full = a1 - a0 + 1;
    } else {
      const Sched sl = make_sched(p, p.n_kr - 1);
      cover(sl, rb, a0, a1);
      c_last = a1 - a0 + 1;
    }
  }
  const int n_contrib = (p.n_kr - 1) * c_full + c_last;
  const int slot = kr * p.max_split + (j - j0);
  const long long slot_elems = static_cast<long long>(p.M) * ROWS;
  float* rb_part = p.partials + static_cast<long long>(rb) * p.n_kr * p.max_split * slot_elems;
  float* part_out = rb_part + slot * slot_elems;
  int* counter = p.counters + rb * COUNTERS_PER_RB + rg;
  const int r0 = rg * 32 + g;                           // row inside the row block (slab 0, first half)
  // Shortcut: if every other contributor had already published its partial, this warp is the one
  // that completes the row group -- add the others to the values still in registers and write the
  // output, without publishing (no global round trip at the kernel's tail).
  const int seen = __shfl_sync(0xffffffffu, seen_lane0, 0);
  if (seen == n_contrib - 1) {
    // (no fence here: lane 0 read the counter with an acquire load a tile ago, and the shuffle above
    // orders the other lanes' loads after it)
    __syncwarp();
    // One pass per contributor, in slot order (the reducer below uses the same order, so both paths
    // give the same bits); all of a pass's loads are independent and in flight together.
    float sum[2][MT][NC][2];
#pragma unroll
    for (int sl = 0; sl < 2; ++sl)
#pragma unroll
      for (int jm = 0; jm < MT; ++jm)
#pragma unroll
        for (int e = 0; e < NC; ++e) { sum[sl][jm][e][0] = 0.0f; sum[sl][jm][e][1] = 0.0f; }
    // CU contributors per pass: all loads of a pass are independent and in flight together; the
    // additions follow slot order (the reducer below uses the same order, so both paths give the same bits).
    constexpr int CU = (MT == 1 && NC == 1) ? 8 : (MT == 1 ? 4 : 2);
    SlotIter iter(p.n_kr, c_full, c_last, p.max_split);
    for (int done = 0; done < n_contrib; done += CU) {
      float v[CU][2][MT][NC][2];
      bool mine[CU];
#pragma unroll
      for (int u = 0; u < CU; ++u) {
        const int os = iter.next();                      // -1 past the end
        mine[u] = os == slot;
        const float* src = rb_part + (os < 0 ? 0 : os) * slot_elems + r0;
        const bool live = os >= 0 && !mine[u];
#pragma unroll
        for (int sl = 0; sl < 2; ++sl)
#pragma unroll
          for (int jm = 0; jm < MT; ++jm)
#pragma unroll
            for (int e = 0; e < NC; ++e) {
              const int m = 8 * jm + 2 * t4 + e;
              const bool ok = live && m < p.M;
              v[u][sl][jm][e][0] = ok ? __ldcg(src + m * ROWS + 16 * sl) : 0.0f;
              v[u][sl][jm][e][1] = ok ? __ldcg(src + m * ROWS + 16 * sl + 8) : 0.0f;
            }
      }
#pragma unroll
      for (int u = 0; u < CU; ++u)
#pragma unroll
        for (int sl = 0; sl < 2; ++sl)
#pragma unroll
          for (int jm = 0; jm < MT; ++jm)
#pragma unroll
            for (int e = 0; e < NC; ++e) {
              sum[sl][jm][e][0] += mine[u] ? y[sl][jm][e] : v[u][sl][jm][e][0];
              sum[sl][jm][e][1] += mine[u] ? y[sl][jm][2 + e] : v[u][sl][jm][e][1];
            }
    }
    float out_y[2][MT][4];
#pragma unroll
    for (int sl = 0; sl < 2; ++sl)
#pragma unroll
      for (int jm = 0; jm < MT; ++jm)
#pragma unroll
        for (int e = 0; e < NC; ++e) { out_y[sl][jm][e] = sum[sl][jm][e][0]; out_y[sl][jm][2 + e] = sum[sl][jm][e][1]; }
    store_row_group<MT, NC>(p, out_y, rb, rg, g, t4);
    __syncwarp();
    if (lane == 0) *counter = 0;
    return;
  }
#pragma unroll
  for (int sl = 0; sl < 2; ++sl) {
#pragma unroll
    for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
      for (int e = 0; e < NC; ++e) {
        const int m = 8 * jm + 2 * t4 + e;
        if (m < p.M) {
          __stcg(part_out + m * ROWS + r0 + 16 * sl, y[sl][jm][e]);
          __stcg(part_out + m * ROWS + r0 + 16 * sl + 8, y[sl][jm][2 + e]);
        }
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
    // lane = row of the row group; one pass per contributor in slot order, the (up to 8 * MT) rows of
    // x of a pass loaded together
    constexpr int MR = 8 * MT;
    const float* src = rb_part + rg * 32 + lane;
    float sum[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) sum[m] = 0.0f;
    constexpr int CU = MT == 1 ? 4 : 2;      // contributors per pass, their loads in flight together
    SlotIter iter(p.n_kr, c_full, c_last, p.max_split);
    for (int done = 0; done < n_contrib; done += CU) {
      float v[CU][MR];
#pragma unroll
      for (int u = 0; u < CU; ++u) {
        const int os = iter.next();
        const float* sp = src + (os < 0 ? 0 : os) * slot_elems;
#pragma unroll
        for (int m = 0; m < MR; ++m) v[u][m] = (os >= 0 && m < p.M) ? __ldcg(sp + m * ROWS) : 0.0f;
      }
#pragma unroll
      for (int u = 0; u < CU; ++u)
#pragma unroll
        for (int m = 0; m < MR; ++m) sum[m] += v[u][m];
    }
    const int n = rb * ROWS + rg * 32 + lane;
    if (n < p.N) {
#pragma unroll
      for (int m = 0; m < MR; ++m)
        if (m < p.M) store_out(p.out, p.out_dtype, static_cast<long long>(m) * p.N + n, sum[m]);
    }
    if (lane == 0) *counter = 0;
  }
}

// MT: 8-wide m tiles (1 or 2).  MPAD: rows of x per group in shared memory (>= M; 1, 2, 4, 8 or 16),
// a compile-time stride.  RAGGED: K % 256 != 0 (scales by cp.async, activations beyond K staged as zeros).
//
// CL: cluster mode, for problems too small to give every CTA several tiles.  A row block belongs
// to a cluster of p.cluster CTAs; CTA r of the cluster streams the r-th share of the row block's k
// tiles, then hands its 128 x M partial to the cluster's first CTA through distributed shared
// memory (remote stores + one remote mbarrier arrival per lane), and that CTA adds the shares in
// rank order and writes the output.  No global scratch, no counters, no atomics.
template <int MT, int MPAD, bool RAGGED, bool CL>
__global__ void __launch_bounds__((Cfg<MT>::NCW + 1) * 32, Cfg<MT>::CTAS_PER_SM)
w4a16_gemv_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_s,
                  const __grid_constant__ Params p) {
  constexpr int NSTAGES = nstages_for(MT, CL);
  constexpr int NCW = Cfg<MT>::NCW;
  constexpr int PARTS = NCW / NRG;            // slices of a tile's 8 groups (2 or 4)
  constexpr int CPW = GT / PARTS;             // groups per warp and tile (4 or 2)
  constexpr int NC = MPAD == 1 ? 1 : 2;       // output columns a lane keeps per m tile (only column 0 exists at M == 1)
  constexpr int ZQB = zq_group_bytes(MPAD);
  // MAGIC: the zero point is taken off the weights, not the accumulator.  (word & mask) | 0x6400 in a
  // 16-bit lane is the fp16 number 1024 + q (1024 + 16 q for a nibble in bits 4-7); subtracting 1032
  // (1152) leaves q - 8 (16 (q - 8)) exactly.  One more instruction per operand register, but no
  // zero-point quad to fetch from shared memory per (group, m tile): worth it where shared-memory
  // bandwidth, not issue rate, is the bound (two m tiles).
  constexpr bool MAGIC = MT == 2;
  // Declared 1024-byte aligned (the 128-byte TMA swizzle needs it) and used directly, so the
  // compiler keeps every access in the shared address space with 32-bit addressing.
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicExch(&g_device_status, 3);
    return;
  }
  const SmemLayout L = smem_layout(NSTAGES, MPAD, MT, p.x_tiles, CL ? p.cluster : 1);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar_addr = sbase + static_cast<uint32_t>(L.bars);      // full[s] at +8*s, empty[s] at +8*(NSTAGES+s)
  const uint32_t abort_addr = sbase + static_cast<uint32_t>(L.flags);   // CtaInfo::abort
  CtaInfo* info = reinterpret_cast<CtaInfo*>(smem + L.flags);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    CtaInfo ci;
    ci.abort = 0;
    ci.kr = blockIdx.x % p.n_kr;
    ci.j = blockIdx.x / p.n_kr;
    const Sched sch = make_sched(p, ci.kr);
    ci.leave = ci.j >= sch.G;
    ci.S_kr = sch.S_kr; ci.T = sch.T; ci.G = sch.G;
    ci.t0 = 0; ci.n_tiles = 0; ci.rb0 = 0; ci.ks0 = 0; ci.pad = 0;
    if (!ci.leave) {
      ci.t0 = tile_begin(sch, ci.j);
      ci.n_tiles = static_cast<int>(tile_begin(sch, ci.j + 1) - ci.t0);
      ci.rb0 = static_cast<int>(ci.t0 / static_cast<unsigned>(sch.S_kr));
      ci.ks0 = static_cast<int>(ci.t0 - static_cast<unsigned>(ci.rb0) * sch.S_kr);
    }
    if (CL && ci.leave) ci.rb0 = ci.j / p.cluster;   // (never planned) it would hand zeros to its own leader
    if (CL || !ci.leave) {   // a cluster CTA always runs to the hand-over, tiles or not
      for (int s = 0; s < NSTAGES; ++s) {
        mbar_init(reinterpret_cast<uint64_t*>(smem + L.bars) + s, RAGGED ? 33 : 1);
        mbar_init(reinterpret_cast<uint64_t*>(smem + L.bars) + NSTAGES + s, NCW);
      }
      if (CL) {   // one arrival per lane of each other CTA's row-group warp
        for (int r = 0; r < NRG; ++r) mbar_init(reinterpret_cast<uint64_t*>(smem + L.bars) + 2 * NSTAGES + r, (p.cluster - 1) * 32);
      }
      fence_barrier_init();
    }
    *info = ci;
    // Programmatic dependent launch: let the next kernel on the stream become resident as our
    // CTAs retire.  Its producer warp may then prefetch weights (constants) while we finish;
    // everything that reads activations or touches out / workspace waits for us below.
    griddep_launch_dependents();
  }
  __syncthreads();
  if (CL) cluster_arrive();   // "this CTA runs and its barriers exist"; no CTA leaves early in cluster mode
  if (!CL && info->leave) return;  // whole CTA leaves together; nothing was started
  const unsigned t0 = info->t0;
  const int n_tiles = info->n_tiles;
  const int rb0 = info->rb0, ks0 = info->ks0, kr = info->kr, S_kr = info->S_kr;

  if (warp == NCW) {
    // ------------------------------------------------------------ producer warp
    // (weights and scales only: they are not produced by the preceding kernel, so no dependency wait)
    if (lane == 0) {
      tma_prefetch_desc(&tmap_w);
      if (!RAGGED) tma_prefetch_desc(&tmap_s);
    }
    if (RAGGED || lane == 0) {
      int rb = rb0, ks = ks0;
      const int n_groups = p.K >> 5;
      const long long srow_bytes = static_cast<long long>(n_groups) * 2;
      for (int it = 0; it < n_tiles; ++it) {
        const int s = it % NSTAGES;
        const uint32_t ph = (it / NSTAGES) & 1;
        bool ok = mbar_wait_bounded_a(bar_addr + 8 * (NSTAGES + s), ph ^ 1, abort_addr);
        if (RAGGED) ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) { info->abort = 1; atomicExch(&g_device_status, 1); }
          break;
        }
        const int kt = kr * p.S + ks;  // absolute k tile
        uint8_t* dst = smem + s * STAGE_BYTES;
        uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars) + s;
        if (lane == 0) {
          mbar_expect_tx(full, RAGGED ? W_BYTES : STAGE_BYTES);
          tma_load_2d(dst, &tmap_w, full, kt * (KT / 2), rb * ROWS);
          if (!RAGGED) tma_load_2d(dst + W_BYTES, &tmap_s, full, kt * GT, rb * ROWS);
        }
        if (RAGGED) {
          // the tile's scales, 128 rows x 16 bytes, as 4-byte pieces: lane l copies pieces l, l+32, ...
          const uint32_t sdst = smem_u32(dst + W_BYTES);
#pragma unroll
          for (int i = 0; i < (ROWS * 4) / 32; ++i) {
            const int piece = i * 32 + lane;
            const int r = piece >> 2, wq = piece & 3;
            const long long row = static_cast<long long>(rb) * ROWS + r;
            const int grp = kt * GT + wq * 2;
            const bool valid = row < p.N && grp < n_groups;
            const uint8_t* src = static_cast<const uint8_t*>(p.scales) + (valid ? row * srow_bytes + grp * 2 : 0);
            cp_async_4(sdst + r * 16 + wq * 4, src, valid ? 4u : 0u);
          }
          cp_async_arrive_noinc(full);
        }
        if (++ks == S_kr) { ks = 0; ++rb; }
      }
    }
  } else {
    // ------------------------------------------------------------ consumer warps
    const int g = lane >> 2, t4 = lane & 3;
    const int rg = warp & (NRG - 1);         // row group: rows 32*rg .. 32*rg+31 of the tile
    const int part = warp / NRG;             // slice: groups part*CPW .. part*CPW+CPW-1 of the tile
    float* comb = reinterpret_cast<float*>(smem + L.comb);

    if (part == 0) named_bar_arrive(BAR_FREE0 + rg, PARTS * 32);   // the hand-over buffer starts out free

    // ---- stage this k-range of x: permuted element order, fp16, high-nibble slots / 16;
    //      and the zero-point terms -8 * xsum * 2^-24 as float32
    griddep_wait();   // x may be the previous kernel's output; out / workspace may still be in its use
    // Only the k tiles this CTA will actually visit are staged, in visiting order: its tile range
    // starts at tile ks0 of a row block and wraps around the k-range, so it touches
    // min(n_tiles, S_kr) tiles and the i-th tile it streams uses slot i mod that.
    const int need_tiles = n_tiles < S_kr ? n_tiles : S_kr;
    {
      // One warp instruction covers one (visited tile, row m): lane = octet (8 consecutive k) of the tile.
      uint4* xs = reinterpret_cast<uint4*>(smem + L.xs);
      float* zps = reinterpret_cast<float*>(smem + L.zps);
      const long long kbase = static_cast<long long>(kr) * p.S * KT;
      int tile_i = 0, m = warp;
      while (m >= p.M) { m -= p.M; ++tile_i; }
      constexpr int U = MT == 2 ? 8 : 4;   // independent 16-byte loads in flight per lane
      while (tile_i < need_tiles) {
        uint4 raw[U];
        int mm[U], kk[U];
        bool ok[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          ok[u] = tile_i < need_tiles;
          int ks = ks0 + tile_i;
          if (ks >= S_kr) ks -= S_kr;
          mm[u] = m; kk[u] = tile_i;
          raw[u] = make_uint4(0u, 0u, 0u, 0u);
          const long long kpos = kbase + static_cast<long long>(ks) * KT + 8 * lane;
          if (ok[u] && (!RAGGED || kpos < p.K))
            raw[u] = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.x) + static_cast<long long>(m) * p.K + kpos));
          m += NCW;
          while (m >= p.M) { m -= p.M; ++tile_i; }
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
          if (ok[u]) {                                       // warp-uniform
            const __half2 h0 = __floats2half2_rn(v[0], v[4]);
            const __half2 h1 = __floats2half2_rn(v[1] * 0.0625f, v[5] * 0.0625f);
            const __half2 h2 = __floats2half2_rn(v[2], v[6]);
            const __half2 h3 = __floats2half2_rn(v[3] * 0.0625f, v[7] * 0.0625f);
            uint4 q;
            q.x = *reinterpret_cast<const uint32_t*>(&h0); q.y = *reinterpret_cast<const uint32_t*>(&h1);
            q.z = *reinterpret_cast<const uint32_t*>(&h2); q.w = *reinterpret_cast<const uint32_t*>(&h3);
            const int grp = kk[u] * GT + (lane >> 2);
            xs[(grp * MPAD + mm[u]) * 4 + (lane & 3)] = q;
            if (!MAGIC && (lane & 3) == 0) {
              // the MMA's accumulator-input quad of rows (g, g+8) x columns (m0, m1) is {z(m0), z(m1), z(m0), z(m1)}
              const float z = sum * -4.76837158203125e-7f;   // -8 * xsum * 2^-24
              if (MPAD == 1) {
                *reinterpret_cast<float4*>(zps + grp * 4) = make_float4(z, z, z, z);
              } else {
                float* q4 = zps + (grp * (MPAD / 2) + (mm[u] >> 1)) * 4 + (mm[u] & 1);
                q4[0] = z; q4[2] = z;
              }
            }
          }
        }
      }
      named_bar_sync(BAR_CONSUMERS, NCW * 32);
    }

    float acc[2][MT][4];                     // [16-row slab of the row group][m tile][fragment element]
#pragma unroll
    for (int sl = 0; sl < 2; ++sl) {
#pragma unroll
      for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[sl][jm][e] = 0.0f;
      }
    }

    float zero4[4];
    opaque_zero4(zero4);
    // All hot-loop operands are read with explicit shared-space loads from 32-bit addresses.
    // Word t4 of row (32*rg + g), this warp's group c, inside a stage: every row a lane reads has
    // (row & 7) == g, so the 128-byte swizzle is the same XOR for all four of them; the other three
    // rows sit 1024, 2048 and 3072 bytes further on.
    uint32_t w_addr[CPW];
#pragma unroll
    for (int c = 0; c < CPW; ++c)
      w_addr[c] = sbase + static_cast<uint32_t>((rg * 32 + g) * 128 + 4 * t4) + (static_cast<uint32_t>((part * CPW + c) ^ g) << 4);
    // scales of row (32*rg + g): this warp's CPW groups
    const uint32_t s_addr = sbase + static_cast<uint32_t>(W_BYTES + (rg * 32 + g) * 16 + part * CPW * 2);
    // x fragment of lane (g, t4) for m tile jm: row m = 8*jm + g of group grp sits at
    // xs[(grp*MPAD + m)*4 + t4].  A lane whose m does not exist reads row M-1 instead: B column m only
    // feeds D column m, and columns >= M are never stored.
    uint32_t x_addr[MT];
#pragma unroll
    for (int jm = 0; jm < MT; ++jm) {
      const int m = (8 * jm + g) < p.M ? (8 * jm + g) : p.M - 1;
      x_addr[jm] = sbase + static_cast<uint32_t>(L.xs + ((part * CPW * MPAD + m) * 4 + t4) * 16);
    }
    // zero-point quad of the lane's output columns m = 8*jm + 2*t4 (+1); columns that do not exist
    // read whatever lies there (spare bytes follow the array) and are never stored
    const uint32_t zq_addr = sbase + static_cast<uint32_t>(L.zps + part * CPW * ZQB + (NC == 2 ? t4 * 16 : 0));

    // The CTA's tiles come in segments, one per row block it touches; a segment is streamed with no
    // bookkeeping beyond the ring, then flushed.
    bool dead = false;
    int rb = rb0;
    int seg = S_kr - ks0;                    // tiles until the end of row block rb (inside this k-range)
    uint32_t x_off = 0, z_off = 0;           // byte offsets of the current k tile's slot in xs / zps
    const uint32_t x_wrap = static_cast<uint32_t>(need_tiles * (GT * MPAD * 64));
    uint32_t so = 0;                         // byte offset of the current stage
    uint32_t full_a = bar_addr, empty_a = bar_addr + 8 * NSTAGES;
    uint32_t ph = 0;
    int remaining = n_tiles;
    while (remaining > 0) {
      if (seg > remaining) seg = remaining;
      remaining -= seg;
      // the row block is written directly if this CTA produces all of it
      const unsigned rb_t0 = static_cast<unsigned>(rb) * S_kr;
      const bool whole = p.n_kr == 1 && rb_t0 >= t0 && rb_t0 + S_kr <= t0 + n_tiles;
      // Ahead of a flush through scratch: read the row group's counter while the segment's last tile
      // is still to be computed, so the round trip to L2 runs under that tile's math and the value is
      // as fresh as it can be for free.  (A value read early stays valid: the counter only grows until
      // the last contributor resets it.)
      int seen = -1;
      const bool want_seen = !CL && part == 0 && !whole && lane == 0;
#pragma unroll 1
      for (int i = 0; i < seg; ++i) {
        if (want_seen && i == seg - 1)
          seen = ld_acquire_gpu(p.counters + rb * COUNTERS_PER_RB + rg);
        const bool ok = !dead && (mbar_try_wait_a(full_a, ph) || mbar_wait_slow(full_a, ph, abort_addr));
        if (ok) {
          // scales of the lane's four rows (slab 0: g, g+8; slab 1: g+16, g+24) for the warp's groups
          float sc[2][2][CPW];
          const uint32_t sa0 = s_addr + so;
#pragma unroll
          for (int sl = 0; sl < 2; ++sl) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint32_t sa = sa0 + (sl * 16 + h * 8) * 16;
              if (CPW == 4) {
                const uint2 v = lds64(sa);
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
                const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
                sc[sl][h][0] = f0.x; sc[sl][h][1] = f0.y; sc[sl][h][2 % CPW] = f1.x; sc[sl][h][3 % CPW] = f1.y;
              } else {
                const uint32_t v = lds32(sa);
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&v));
                sc[sl][h][0] = f0.x; sc[sl][h][1] = f0.y;
              }
            }
          }
          uint32_t xa[MT];
#pragma unroll
          for (int jm = 0; jm < MT; ++jm) xa[jm] = x_addr[jm] + x_off;
          const uint32_t za = zq_addr + z_off;
#pragma unroll
          for (int c = 0; c < CPW; ++c) {
            uint4 bx[MT];
            float zc[MT][4];                   // accumulator input of the group's first MMA, loaded as one register quad
#pragma unroll
            for (int jm = 0; jm < MT; ++jm) {
              bx[jm] = lds128(xa[jm] + c * (MPAD * 64));
              if (MAGIC) {
                zc[jm][0] = zero4[0]; zc[jm][1] = zero4[1]; zc[jm][2] = zero4[2]; zc[jm][3] = zero4[3];
              } else {
                const uint4 z = lds128(za + c * ZQB + jm * 64);
                zc[jm][0] = __uint_as_float(z.x); zc[jm][1] = __uint_as_float(z.y);
                zc[jm][2] = __uint_as_float(z.z); zc[jm][3] = __uint_as_float(z.w);
              }
            }
            const uint32_t wp = w_addr[c] + so;
#pragma unroll
            for (int sl = 0; sl < 2; ++sl) {
              const uint32_t wa = lds32(wp + sl * 2048);
              const uint32_t wb = lds32(wp + sl * 2048 + 1024);
              const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
              uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
              if (MAGIC) {
                a0 = magic_lo(wa); a1 = magic_lo(wb); a2 = magic_hi(wa); a3 = magic_hi(wb);
                b0 = magic_lo(wa8); b1 = magic_lo(wb8); b2 = magic_hi(wa8); b3 = magic_hi(wb8);
              } else {
                a0 = wa & 0x000F000Fu; a1 = wb & 0x000F000Fu; a2 = wa & 0x00F000F0u; a3 = wb & 0x00F000F0u;
                b0 = wa8 & 0x000F000Fu; b1 = wb8 & 0x000F000Fu; b2 = wa8 & 0x00F000F0u; b3 = wb8 & 0x00F000F0u;
              }
#pragma unroll
              for (int jm = 0; jm < MT; ++jm) {
                float d[4];
                mma_m16n8k16_f16(d, a0, a1, a2, a3, bx[jm].x, bx[jm].y, zc[jm]);
                mma_m16n8k16_f16(d, b0, b1, b2, b3, bx[jm].z, bx[jm].w, d);
                acc[sl][jm][0] = fmaf(sc[sl][0][c], d[0], acc[sl][jm][0]);
                acc[sl][jm][2] = fmaf(sc[sl][1][c], d[2], acc[sl][jm][2]);
                if (NC == 2) {
                  acc[sl][jm][1] = fmaf(sc[sl][0][c], d[1], acc[sl][jm][1]);
                  acc[sl][jm][3] = fmaf(sc[sl][1][c], d[3], acc[sl][jm][3]);
                }
              }
            }
          }
        } else if (!dead) {
          dead = true; info->abort = 1; atomicExch(&g_device_status, 2);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_a(empty_a);   // also in the dead state, so the producer never stalls on us
        x_off += GT * MPAD * 64;
        z_off += GT * ZQB;
        if (x_off == x_wrap) { x_off = 0; z_off = 0; }
        so += STAGE_BYTES; full_a += 8; empty_a += 8;
        if (so == NSTAGES * STAGE_BYTES) { so = 0; full_a = bar_addr; empty_a = bar_addr + 8 * NSTAGES; ph ^= 1; }
      }

      // ---- end of this CTA's share of row block rb: flush.  The slices of a row group are added
      //      through shared memory (slice 0 collects), then slice 0 settles the row group's 32 rows;
      //      row groups never wait for each other.  Runs in the dead state too (the barriers pair up).
      {
        float y[2][MT][4];
#pragma unroll
        for (int sl = 0; sl < 2; ++sl) {
#pragma unroll
          for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
            for (int e = 0; e < 4; ++e) { y[sl][jm][e] = MAGIC ? acc[sl][jm][e] : acc[sl][jm][e] * 16777216.0f; acc[sl][jm][e] = 0.0f; }
          }
        }
        if (part != 0) {
          named_bar_sync(BAR_FREE0 + rg, PARTS * 32);          // slice 0 has read the previous hand-over
          float* dst = comb + (((part - 1) * NRG + rg) * 2 * MT * 4) * 32 + lane;
#pragma unroll
          for (int sl = 0; sl < 2; ++sl) {
#pragma unroll
            for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                if (NC == 2 || (e & 1) == 0) dst[((sl * MT + jm) * 4 + e) * 32] = y[sl][jm][e];
              }
            }
          }
          __threadfence_block();
          named_bar_arrive(BAR_FULL0 + rg, PARTS * 32);
        } else {
          named_bar_sync(BAR_FULL0 + rg, PARTS * 32);
#pragma unroll
          for (int pp = 1; pp < PARTS; ++pp) {
            const float* src = comb + (((pp - 1) * NRG + rg) * 2 * MT * 4) * 32 + lane;
#pragma unroll
            for (int sl = 0; sl < 2; ++sl) {
#pragma unroll
              for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  if (NC == 2 || (e & 1) == 0) y[sl][jm][e] += src[((sl * MT + jm) * 4 + e) * 32];
                }
              }
            }
          }
          __threadfence_block();
          named_bar_arrive(BAR_FREE0 + rg, PARTS * 32);
          if (CL) {
            const uint32_t crank = cluster_ctarank();
            const uint32_t red_bar = bar_addr + 8 * (2 * NSTAGES + rg);
            constexpr int SLOT = red_slot_bytes(MT);
            if (crank != 0) {
              cluster_wait();                                   // the leader runs and its barriers exist
              const uint32_t local = sbase + static_cast<uint32_t>(L.red + ((crank - 1) * NRG + rg) * SLOT + lane * 4);
              const uint32_t dst = map_to_rank(local, 0);
#pragma unroll
              for (int sl = 0; sl < 2; ++sl) {
#pragma unroll
                for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    if (NC == 2 || (e & 1) == 0) st_cluster_f32(dst + ((sl * MT + jm) * 4 + e) * 128, y[sl][jm][e]);
                  }
                }
              }
              mbar_arrive_remote(map_to_rank(red_bar, 0));
            } else {
              if (!mbar_wait_cluster_bounded(red_bar, 0)) {
                if (lane == 0) { info->abort = 1; atomicExch(&g_device_status, 4); }
              } else {
                for (int r = 1; r < p.cluster; ++r) {          // rank order: the same bits every run
                  const uint32_t src = sbase + static_cast<uint32_t>(L.red + ((r - 1) * NRG + rg) * SLOT + lane * 4);
#pragma unroll
                  for (int sl = 0; sl < 2; ++sl) {
#pragma unroll
                    for (int jm = 0; jm < MT; ++jm) {
#pragma unroll
                      for (int e = 0; e < 4; ++e) {
                        if (NC == 2 || (e & 1) == 0) y[sl][jm][e] += __uint_as_float(lds32(src + ((sl * MT + jm) * 4 + e) * 128));
                      }
                    }
                  }
                }
                store_row_group<MT, NC>(p, y, rb, rg, g, t4);
              }
            }
          } else {
            if (whole) store_row_group<MT, NC>(p, y, rb, rg, g, t4);
            else flush_row_group<MT, NC>(p, y, rb, rg, g, t4, lane, seen, info);
          }
        }
      }
      ++rb; seg = S_kr;   // the next segment starts a row block
    }
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------- host side
struct Plan {
  Params p;
  int grid;
  int MT, MPAD;
  bool ragged;
  bool cluster;             // cluster mode (p.cluster CTAs per row block), no scratch
  bool fits_32bit;          // the device-side schedule arithmetic is 32-bit
  size_t smem_bytes;
  size_t counters_bytes;   // COUNTER_BYTES, the same for every problem
  size_t workspace_bytes;  // counters + partials
};

inline bool supported(int M, int N, int K, int G, int x_dtype, int scale_dtype) {
  return M >= 1 && M <= 16 && N >= 1 && N <= MAX_ROW_BLOCKS * ROWS && K >= 64 && (K % 64) == 0 && G == 32 &&
         (x_dtype == LCQ_F16 || x_dtype == LCQ_BF16) && scale_dtype == LCQ_F16;
}

inline int mpad_for(int M) { return M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : 16; }

// Tiles one CTA may take from ONE row block before the row block is cut between CTAs, for
// problems too small to give every CTA several tiles: below it a row block stays whole and its
// CTA writes the output directly (no scratch round trip, which costs more than a few tiles).
inline int whole_row_block_tiles() {
  static const int v = [] {
    const char* e = getenv("LCQ_GEMV_WHOLE_RB_TILES");
    const int n = e ? atoi(e) : 0;
    return n > 0 ? n : 12;
  }();
  return v;
}

// Cluster mode can be switched off with LCQ_GEMV_CLUSTER=0 (read once).
inline bool cluster_mode_enabled() {
  static const bool on = [] { const char* e = getenv("LCQ_GEMV_CLUSTER"); return !(e && e[0] == '0'); }();
  return on;
}

// Largest cluster tried, per m-tile count: 8 with two CTAs per SM; 4 with one CTA per SM, where a
// cluster of 8 needs 8 free SMs of one GPC at once and measured 1.5 - 1.8 x slower than clusters of 4.
// (LCQ_GEMV_MAX_CLUSTER / LCQ_GEMV_MAX_CLUSTER2 override, read once.)
inline int max_cluster_for(int MT) {
  static const int v1 = [] { const char* e = getenv("LCQ_GEMV_MAX_CLUSTER"); const int n = e ? atoi(e) : 0; return (n == 1 || n == 2 || n == 4 || n == 8) ? n : 8; }();
  static const int v2 = [] { const char* e = getenv("LCQ_GEMV_MAX_CLUSTER2"); const int n = e ? atoi(e) : 0; return (n == 1 || n == 2 || n == 4 || n == 8) ? n : 4; }();
  return MT == 1 ? v1 : v2;
}

inline Plan make_plan(int M, int N, int K, int sm_count) {
  Plan pl;
  memset(&pl, 0, sizeof(pl));
  Params& p = pl.p;
  p.M = M; p.N = N; p.K = K;
  pl.MT = M <= 8 ? 1 : 2;
  pl.MPAD = mpad_for(M);
  pl.ragged = (K % KT) != 0;
  const int nstages = pl.MT == 1 ? Cfg<1>::NSTAGES : Cfg<2>::NSTAGES;
  const int ctas_per_sm = pl.MT == 1 ? Cfg<1>::CTAS_PER_SM : Cfg<2>::CTAS_PER_SM;
  const int fixed = smem_layout(nstages, pl.MPAD, pl.MT, 0, 1).total;
  const int xc_bytes = max_dynamic_smem(ctas_per_sm) - fixed - 64;
  p.n_rb = (N + ROWS - 1) / ROWS;
  p.nst = (K + KT - 1) / KT;
  const int s_max = xc_bytes / xc_bytes_per_tile(pl.MPAD, pl.MT);
  p.n_kr = (p.nst + s_max - 1) / s_max;
  p.S = (p.nst + p.n_kr - 1) / p.n_kr;
  p.n_kr = (p.nst + p.S - 1) / p.S;           // drop empty trailing ranges
  p.ctas_per_kr = (sm_count * ctas_per_sm) / p.n_kr;
  if (p.ctas_per_kr < 1) p.ctas_per_kr = 1;
  long long T = static_cast<long long>(p.n_rb) * p.S;
  if (p.ctas_per_kr > T) p.ctas_per_kr = static_cast<int>(T);
  p.x_tiles = p.S;
  p.cluster = 1;
  // Small problems (fewer than a few tiles per CTA): a cluster of c CTAs per row block, c the
  // largest power of two (<= 8) that keeps every cluster resident at once, gives every CTA a tile and
  // fits in shared memory.  A CTA then stages only its own share of x, so K needs no ranges.
  const long long capacity = static_cast<long long>(sm_count) * ctas_per_sm;
  if (static_cast<long long>(p.n_rb) * p.nst < 4LL * capacity && cluster_mode_enabled()) {
    const int nst_cl = nstages_for(pl.MT, true);
    int c = max_cluster_for(pl.MT);
    while (c > 1) {
      // clusters of 8 do not pack the GPCs completely: leave a quarter of the CTA slots unused
      const bool resident = static_cast<long long>(p.n_rb) * c <= (c == 8 ? capacity * 3 / 4 : capacity);
      const int xt = (p.nst + c - 1) / c;
      if (c <= p.nst && resident && smem_layout(nst_cl, pl.MPAD, pl.MT, xt, c).total <= max_dynamic_smem(ctas_per_sm)) break;
      c >>= 1;
    }
    if (c > 1) {
      pl.cluster = true;
      p.cluster = c;
      p.n_kr = 1;
      p.S = p.nst;
      p.x_tiles = (p.nst + c - 1) / c;
      p.ctas_per_kr = p.n_rb * c;
    }
  }
  T = static_cast<long long>(p.n_rb) * p.S;
  // Otherwise: give each row block to c CTAs, c as small as keeps a CTA's share of a row block within
  // whole_row_block_tiles(); c = 1 means no scratch at all.
  if (!pl.cluster && T < 4LL * p.ctas_per_kr) {
    const int lim = whole_row_block_tiles();
    int c = (p.S + lim - 1) / lim;
    long long want = static_cast<long long>(p.n_rb) * c;
    if (want < p.ctas_per_kr) p.ctas_per_kr = static_cast<int>(want);
  }
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
  pl.fits_32bit = (T + 1) * static_cast<long long>(p.ctas_per_kr) < (1LL << 32);
  pl.smem_bytes = smem_layout(nstages_for(pl.MT, pl.cluster), pl.MPAD, pl.MT, p.x_tiles, p.cluster).total;
  pl.counters_bytes = COUNTER_BYTES;
  pl.workspace_bytes = pl.counters_bytes +
                       static_cast<size_t>(p.n_rb) * p.n_kr * p.max_split * M * ROWS * sizeof(float);
  return pl;
}

template <int MT, int MPAD, bool RAGGED, bool CL>
int launch_c(const Plan& pl, const CUtensorMap& tw, const CUtensorMap& ts, bool allow_pdl, cudaStream_t stream) {
  auto kern = w4a16_gemv_kernel<MT, MPAD, RAGGED, CL>;
  static thread_local int configured_device = -1;  // per (thread, template instance)
  int dev = 0;
  LCQ_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_device != dev) {
    LCQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      max_dynamic_smem(Cfg<MT>::CTAS_PER_SM)));
    LCQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                                      cudaSharedmemCarveoutMaxShared));
    configured_device = dev;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(pl.grid);
  cfg.blockDim = dim3((Cfg<MT>::NCW + 1) * 32);
  cfg.dynamicSmemBytes = pl.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (CL) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = pl.p.cluster;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  if (allow_pdl && pdl_enabled()) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tw, ts, pl.p));
  return LCQ_OK;
}

template <int MT, int MPAD, bool RAGGED>
int launch_t(const Plan& pl, const CUtensorMap& tw, const CUtensorMap& ts, bool allow_pdl, cudaStream_t stream) {
  return pl.cluster ? launch_c<MT, MPAD, RAGGED, true>(pl, tw, ts, allow_pdl, stream)
                    : launch_c<MT, MPAD, RAGGED, false>(pl, tw, ts, allow_pdl, stream);
}

template <bool RAGGED>
int launch_r(const Plan& pl, const CUtensorMap& tw, const CUtensorMap& ts, bool allow_pdl, cudaStream_t stream) {
  switch (pl.MPAD) {
    case 1: return launch_t<1, 1, RAGGED>(pl, tw, ts, allow_pdl, stream);
    case 2: return launch_t<1, 2, RAGGED>(pl, tw, ts, allow_pdl, stream);
    case 4: return launch_t<1, 4, RAGGED>(pl, tw, ts, allow_pdl, stream);
    case 8: return launch_t<1, 8, RAGGED>(pl, tw, ts, allow_pdl, stream);
    default: return launch_t<2, 16, RAGGED>(pl, tw, ts, allow_pdl, stream);
  }
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
  if (out_dtype != LCQ_F32 && out_dtype != LCQ_F16 && out_dtype != LCQ_BF16) {
    set_error("w4a16 gemv: bad out_dtype %d", out_dtype);
    return LCQ_ERR_BAD_ARG;
  }
  if (!pl.fits_32bit) {
    set_error("w4a16 gemv: problem too large for the 32-bit tile schedule");
    return LCQ_ERR_UNSUPPORTED;
  }
  if (pl.smem_bytes > static_cast<size_t>(max_dynamic_smem(pl.MT == 1 ? Cfg<1>::CTAS_PER_SM : Cfg<2>::CTAS_PER_SM))) {
    set_error("w4a16 gemv: plan needs %zu bytes of shared memory", pl.smem_bytes);
    return LCQ_ERR_UNSUPPORTED;
  }
  pl.p.x = x;
  pl.p.out = out;
  pl.p.scales = s;
  pl.p.x_is_bf16 = (x_dtype == LCQ_BF16);
  pl.p.out_dtype = out_dtype;
  pl.p.counters = static_cast<int*>(workspace);
  pl.p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + pl.counters_bytes);
  CUtensorMap tw, ts;
  memset(&ts, 0, sizeof(ts));
  int rc = encode_tmap_2d(&tw, 0, w, static_cast<uint64_t>(K) / 2, static_cast<uint64_t>(N),
                          static_cast<uint64_t>(K) / 2, KT / 2, ROWS, 3);
  if (rc != LCQ_OK) return rc;
  if (!pl.ragged) {
    rc = encode_tmap_2d(&ts, 1, s, static_cast<uint64_t>(K) / 32, static_cast<uint64_t>(N),
                        static_cast<uint64_t>(K) / 16, GT, ROWS, 0);
    if (rc != LCQ_OK) return rc;
    return launch_r<false>(pl, tw, ts, allow_pdl, stream);
  }
  return launch_r<true>(pl, tw, ts, allow_pdl, stream);
}

}  // namespace gemv_tc
}  // namespace lcq
