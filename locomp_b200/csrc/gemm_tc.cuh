// W4A16 prefill GEMM (M > 16) on 5th-generation tensor cores: tcgen05.mma with the
// accumulator AND the dequantised weight operand in tensor memory.
//
//   out[m, n] = sum_k x[m, k] * (nib(n, k) - 8) * scales[n, k / 32]      (float32 accumulate)
//
// Orientation ("swap A/B"): the MMA's M dimension is the weight row n, its N dimension the
// activation row m:   D[128 n x BM m] += Wdq[128 n x 64 k] * X^T[64 k x BM m].
//   * X tiles [BM x 64] fp16 arrive by TMA (128-byte swizzle) and are the shared-memory B operand.
//   * Packed int4 tiles [128 n x 256 k] (+ their fp16 scales) arrive by TMA; eight dequant
//     warps turn them into fp16 (exactly RN((q - 8) * s)) in registers and write them with
//     tcgen05.st into a ring of TMEM slots that the MMA reads as its A operand.  The packed
//     weights therefore cross shared memory once (0.5 B/weight) and never as 2-byte values.
//   * One thread issues the MMAs; tcgen05.commit releases X stages and TMEM slots and, after
//     the last k tile, hands the accumulator to four epilogue warps (tcgen05.ld -> global).
// TMEM map (512 columns): [0, 256) accumulator, [256, 512) eight A slots of 32 columns
// (64 k as packed fp16 pairs).  Weight tiles are fp16 because bf16's 8-bit significand
// cannot hold (q-8)*s within the 1e-2 output tolerance; bf16 activations are converted to
// fp16 by a small pre-pass into the caller's workspace.
//
// Tensor-bound: 2*M*N*K flops per call against the dense 16-bit tensor peak.
// Every mbarrier wait is bounded; on expiry the kernel records a status code and unwinds.
#pragma once
#include "common.cuh"

namespace lcq {
namespace gemm_tc {

constexpr int BN = 128;                 // weight rows per tile (MMA M)
constexpr int BK = 64;                  // k per MMA stage (one 128-byte swizzle row of fp16)
constexpr int WK = 256;                 // k per packed-weight stage
constexpr int W_STAGE = BN * (WK / 2);  // 16384
constexpr int S_STAGE = BN * (WK / 32) * 2;   // 2048
constexpr int WS_STAGE = W_STAGE + S_STAGE;
constexpr int NXS = 4;                  // X stages
constexpr int NWS = 2;                  // packed-weight stages
constexpr int NAS = 8;                  // TMEM A slots
constexpr int A_COL0 = 256;             // first TMEM column of the A ring
constexpr int A_SLOT_COLS = 32;
constexpr int TMEM_COLS = 512;
constexpr int WARP_TMA = 4, WARP_MMA = 5, WARP_DQ0 = 8;
constexpr int N_DQ_WARPS = 8;                 // 8 or 16 (16: two sets of warps take alternate 64-k tiles)
constexpr int DQ_PAR = N_DQ_WARPS / 8;
constexpr int NTHREADS = (WARP_DQ0 + N_DQ_WARPS) * 32;

// ---------------------------------------------------------------- tcgen05 wrappers
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor]
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
}

// Shared-memory matrix descriptor: K-major tile of 128-byte rows, 128-byte swizzle,
// 1024 bytes between 8-row groups.
__device__ __forceinline__ uint64_t make_b_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);   // start address
  d |= static_cast<uint64_t>(1) << 16;                        // leading byte offset (unused for swizzled K-major)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                        // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                        // 128-byte swizzle
  return d;
}
// kind::f16 instruction descriptor: D=f32, A=B=f16, both K-major, M=128, N=bm.
__host__ __device__ inline uint32_t make_idesc(int bm) {
  return (1u << 4) | (static_cast<uint32_t>(bm >> 3) << 17) | (static_cast<uint32_t>(BN >> 4) << 24);
}

struct Params {
  void* out;            // [M, N]
  int M, N, K;
  int bm;               // activation rows per tile (MMA N): multiple of 32, <= 256
  int n_tiles_n, n_tiles_m;
  int splits;           // split-K factor (1 = none); with > 1 `out` is float scratch [splits][M][N]
  int k_tiles_per_split;  // 64-k tiles per split, a multiple of 4
  int out_dtype;
  int vec_store;        // N and out allow 16-byte stores
};

struct Smem {           // offsets from the 1024-byte aligned dynamic shared memory base
  int x;                // NXS stages of bm x 128 B
  int w;                // NWS stages of WS_STAGE
  int bars;
  int tmem_slot;
  int flags;
  int stage;            // epilogue staging: 2 x [32 m][128 n] of the output type (sized for float)
  int total;
};
__host__ __device__ inline Smem smem_map(int bm) {
  Smem s;
  s.x = 0;
  s.w = NXS * bm * 128;
  s.bars = s.w + NWS * WS_STAGE;
  // full_x, empty_x [NXS]; full_w, empty_w [NWS]; full_a, empty_a [NAS]; full_d, empty_d
  s.tmem_slot = s.bars + (2 * NXS + 2 * NWS + 2 * NAS + 2) * 8;
  s.flags = s.tmem_slot + 8;
  s.stage = (s.flags + 8 + 15) & ~15;
  s.total = s.stage + 2 * 32 * BN * 4;
  return s;
}

// RN((q - 8) * s) for the 8 nibbles of a word, as 4 half2 in natural k order.
// PERM = true leaves them in the order the masks deliver -- (e0,e4) (e1,e5) (e2,e6) (e3,e7) --
// for activations whose k order was permuted the same way by the pre-pass (saves 4 PRMT).
template <bool PERM>
__device__ __forceinline__ void dequant_word(uint32_t w, __half2 s2, uint32_t (&o)[4]) {
  const __half2 k1032 = __half2half2(__ushort_as_half(0x6408));   // 1032.0
  const __half2 k16th = __half2half2(__ushort_as_half(0x2C00));   // 1/16
  const __half2 km72 = __half2half2(__ushort_as_half(0xD480));    // -72.0
  const uint32_t w8 = w >> 8;
  uint32_t l0 = (w & 0x000F000Fu) | 0x64006400u;     // 1024 + (e0, e4)
  uint32_t h0 = (w & 0x00F000F0u) | 0x64006400u;     // 1024 + 16*(e1, e5)
  uint32_t l1 = (w8 & 0x000F000Fu) | 0x64006400u;    // 1024 + (e2, e6)
  uint32_t h1 = (w8 & 0x00F000F0u) | 0x64006400u;    // 1024 + 16*(e3, e7)
  __half2 p0 = __hsub2(*reinterpret_cast<__half2*>(&l0), k1032);
  __half2 p1 = __hfma2(*reinterpret_cast<__half2*>(&h0), k16th, km72);
  __half2 p2 = __hsub2(*reinterpret_cast<__half2*>(&l1), k1032);
  __half2 p3 = __hfma2(*reinterpret_cast<__half2*>(&h1), k16th, km72);
  p0 = __hmul2(p0, s2); p1 = __hmul2(p1, s2); p2 = __hmul2(p2, s2); p3 = __hmul2(p3, s2);
  const uint32_t u0 = *reinterpret_cast<uint32_t*>(&p0), u1 = *reinterpret_cast<uint32_t*>(&p1);
  const uint32_t u2 = *reinterpret_cast<uint32_t*>(&p2), u3 = *reinterpret_cast<uint32_t*>(&p3);
  if (PERM) {
    o[0] = u0; o[1] = u1; o[2] = u2; o[3] = u3;
  } else {
    o[0] = __byte_perm(u0, u1, 0x5410);   // (e0, e1)
    o[1] = __byte_perm(u2, u3, 0x5410);   // (e2, e3)
    o[2] = __byte_perm(u0, u1, 0x7632);   // (e4, e5)
    o[3] = __byte_perm(u2, u3, 0x7632);   // (e6, e7)
  }
}

// Bounded wait whose verdict is the same in every lane, so warp-aligned instructions that
// follow it never run with a partial warp.
__device__ __forceinline__ bool warp_wait(volatile int* flag_abort, uint64_t* bar, uint32_t parity) {
  const bool ok = (*flag_abort == 0) && mbar_wait_bounded(bar, parity);
  return __all_sync(0xffffffffu, ok);
}

template <typename OT, bool PERM>
__global__ void __launch_bounds__(NTHREADS, 1)
w4a16_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                  const __grid_constant__ CUtensorMap tmap_s, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicExch(&g_device_status, 13);
    return;
  }
  const Smem L = smem_map(p.bm);
  uint64_t* full_x = reinterpret_cast<uint64_t*>(smem + L.bars);
  uint64_t* empty_x = full_x + NXS;
  uint64_t* full_w = empty_x + NXS;
  uint64_t* empty_w = full_w + NWS;
  uint64_t* full_a = empty_w + NWS;
  uint64_t* empty_a = full_a + NAS;
  uint64_t* full_d = empty_a + NAS;
  uint64_t* empty_d = full_d + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L.tmem_slot);
  volatile int* flag_abort = reinterpret_cast<volatile int*>(smem + L.flags);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int x_stage_bytes = p.bm * 128;
  // a work item is (output tile, k split); k_tiles counts the 64-k tiles of one item
  const int k_tiles = p.k_tiles_per_split;
  const int total_tiles = p.n_tiles_n * p.n_tiles_m * p.splits;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NXS; ++i) { mbar_init(&full_x[i], 1); mbar_init(&empty_x[i], 1); }
    for (int i = 0; i < NWS; ++i) { mbar_init(&full_w[i], 1); mbar_init(&empty_w[i], N_DQ_WARPS); }
    for (int i = 0; i < NAS; ++i) { mbar_init(&full_a[i], 8); mbar_init(&empty_a[i], 1); }
    mbar_init(full_d, 1);
    mbar_init(empty_d, 4);
    *flag_abort = 0;
    fence_barrier_init();
  }
  if (warp == WARP_MMA) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

#define LCQ_GIVE_UP(code) do { *flag_abort = 1; atomicExch(&g_device_status, (code)); } while (0)

  if (warp == WARP_TMA) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_x); tma_prefetch_desc(&tmap_w); tma_prefetch_desc(&tmap_s);
      uint32_t xi = 0, wi = 0;   // running stage counters
      bool ok = true;
      for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x) {
        const int tile = item / p.splits, kt0 = (item % p.splits) * k_tiles;
        const int m0 = (tile / p.n_tiles_n) * p.bm, n0 = (tile % p.n_tiles_n) * BN;
        for (int kt = 0; kt < k_tiles && ok; ++kt) {
          if ((kt & 3) == 0) {
            const uint32_t s = wi % NWS, ph = (wi / NWS) & 1;
            if (*flag_abort || !mbar_wait_bounded(&empty_w[s], ph ^ 1)) { LCQ_GIVE_UP(10); ok = false; break; }
            uint8_t* dst = smem + L.w + s * WS_STAGE;
            mbar_expect_tx(&full_w[s], WS_STAGE);
            tma_load_2d(dst, &tmap_w, &full_w[s], ((kt0 + kt) / 4) * (WK / 2), n0);
            tma_load_2d(dst + W_STAGE, &tmap_s, &full_w[s], ((kt0 + kt) / 4) * (WK / 32), n0);
            ++wi;
          }
          const uint32_t s = xi % NXS, ph = (xi / NXS) & 1;
          if (*flag_abort || !mbar_wait_bounded(&empty_x[s], ph ^ 1)) { LCQ_GIVE_UP(11); ok = false; break; }
          mbar_expect_tx(&full_x[s], x_stage_bytes);
          tma_load_2d(smem + L.x + s * x_stage_bytes, &tmap_x, &full_x[s], (kt0 + kt) * BK, m0);
          ++xi;
        }
      }
    }
  } else if (warp == WARP_MMA) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(p.bm);
      uint32_t xi = 0, ai = 0, di = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++di) {
        if (*flag_abort || !mbar_wait_bounded(empty_d, (di & 1) ^ 1)) { LCQ_GIVE_UP(12); ok = false; break; }
        tc_fence_after();
        for (int kt = 0; kt < k_tiles && ok; ++kt, ++xi, ++ai) {
          const uint32_t sx = xi % NXS, phx = (xi / NXS) & 1;
          const uint32_t sa = ai % NAS, pha = (ai / NAS) & 1;
          if (*flag_abort || !mbar_wait_bounded(&full_x[sx], phx) || !mbar_wait_bounded(&full_a[sa], pha)) {
            LCQ_GIVE_UP(14); ok = false; break;
          }
          tc_fence_after();
          const uint64_t bdesc = make_b_desc(smem_u32(smem + L.x + sx * x_stage_bytes));
          const uint32_t a_t = tmem_base + A_COL0 + sa * A_SLOT_COLS;
#pragma unroll
          for (int j = 0; j < BK / 16; ++j)
            umma_f16_ts(tmem_base, a_t + j * 8, bdesc + static_cast<uint64_t>(2 * j), idesc, (kt | j) != 0 ? 1u : 0u);
          umma_commit(&empty_x[sx]);
          umma_commit(&empty_a[sa]);
        }
        if (ok) umma_commit(full_d);
      }
    }
  } else if (warp >= WARP_DQ0) {
    // ------------------------------------------------------------ dequant warps: smem int4 -> TMEM fp16
    // Thread = weight row = TMEM lane; warpgroup bit 0 picks the 32-wide half of a 64-k tile.  With
    // 16 warps the second pair of warpgroups takes the odd tiles (DQ_PAR = 2).  Software-pipelined
    // by one tile: the registers of a warp's next tile are computed while the tcgen05.st of its
    // current one is in flight; only then is that store waited for and the slot handed to the MMA.
    const int q4 = warp & 3;                    // TMEM lane quarter this warp may touch
    const int wg = (warp - WARP_DQ0) >> 2;      // 0..3
    const int h = wg & 1;                       // which 32-wide half of the 64-k tile
    const int par = wg >> 1;                    // which tiles: kt % 2 == par
    const int r = q4 * 32 + lane;               // weight row inside the tile = TMEM lane
    const uint32_t lane_taddr = tmem_base + (static_cast<uint32_t>(q4 * 32) << 16) + A_COL0 + h * 16;
    const int my_tiles = (total_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
    const long long n_steps = static_cast<long long>(my_tiles) * k_tiles;   // 64-k tiles this CTA processes (even)
    bool ok = true;
    uint32_t v[16];

    // registers of step `st` (packed tile q = st % 4 of weight stage st / 4)
    auto produce = [&](long long st) -> bool {
      const int q = static_cast<int>(st & 3);
      const uint32_t wi = static_cast<uint32_t>(st >> 2);
      const uint32_t sw = wi % NWS;
      if (q < DQ_PAR) {                         // this warp's first tile in the weight stage
        if (!warp_wait(flag_abort, &full_w[sw], (wi / NWS) & 1)) return false;
      }
      const uint8_t* wst = smem + L.w + sw * WS_STAGE;
      const int c = q * 2 + h;                  // 16-byte chunk (= one 32-wide group) of the 128-byte row
      const uint4 pk = *reinterpret_cast<const uint4*>(wst + r * 128 + ((c ^ (r & 7)) << 4));
      const __half2 s2 = __half2half2(*reinterpret_cast<const __half*>(wst + W_STAGE + r * 16 + c * 2));
      uint32_t o[4];
      dequant_word<PERM>(pk.x, s2, o); v[0] = o[0]; v[1] = o[1]; v[2] = o[2]; v[3] = o[3];
      dequant_word<PERM>(pk.y, s2, o); v[4] = o[0]; v[5] = o[1]; v[6] = o[2]; v[7] = o[3];
      dequant_word<PERM>(pk.z, s2, o); v[8] = o[0]; v[9] = o[1]; v[10] = o[2]; v[11] = o[3];
      dequant_word<PERM>(pk.w, s2, o); v[12] = o[0]; v[13] = o[1]; v[14] = o[2]; v[15] = o[3];
      __syncwarp();
      if (q >= 4 - DQ_PAR && lane == 0) mbar_arrive(&empty_w[sw]);   // this warp's last read of the weight stage
      return true;
    };

    if (n_steps > par && !produce(par)) { LCQ_GIVE_UP(15); ok = false; }
    for (long long st = par; st < n_steps && ok; st += DQ_PAR) {
      const uint32_t ai = static_cast<uint32_t>(st);
      const uint32_t sa = ai % NAS;
      if (!warp_wait(flag_abort, &empty_a[sa], ((ai / NAS) & 1) ^ 1)) { LCQ_GIVE_UP(16); ok = false; break; }
      tc_fence_after();
      tmem_st16(lane_taddr + sa * A_SLOT_COLS, v);         // registers are read at issue
      if (st + DQ_PAR < n_steps) {
        if (!produce(st + DQ_PAR)) { LCQ_GIVE_UP(15); ok = false; }   // overlaps the store in flight
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_a[sa]);
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------ epilogue warps: TMEM -> smem -> global
    // The accumulator is n-major (lane = n, column = m) while out is [M, N]: 32 columns at a
    // time are converted and transposed through a double-buffered staging tile [32 m][128 n],
    // then written with 16-byte stores, 256 contiguous bytes (128 n) per output row.
    OT* out_base = static_cast<OT*>(p.out);
    OT* stage = reinterpret_cast<OT*>(smem + L.stage);
    constexpr int VEC = 16 / sizeof(OT);                 // outputs per 16-byte store
    constexpr int ROW_VECS = BN / VEC;                   // 16-byte pieces per staged row
    const int et = warp * 32 + lane;                     // 0..127
    uint32_t di = 0, chunk = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x, ++di) {
      const int tile = item / p.splits;
      const int m0 = (tile / p.n_tiles_n) * p.bm, n0 = (tile % p.n_tiles_n) * BN;
      OT* out = out_base + static_cast<long long>(item % p.splits) * p.M * p.N;   // split-K: this split's partial
      if (!warp_wait(flag_abort, full_d, di & 1)) { LCQ_GIVE_UP(17); ok = false; break; }
      tc_fence_after();
      const int n_cb = p.bm / 32;
      for (int cb = 0; cb < n_cb; ++cb, ++chunk) {
        uint32_t v[32];
        tmem_ld32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + cb * 32, v);
        tmem_wait_ld();
        if (cb == n_cb - 1) {                            // accumulator fully read: the next tile's MMAs may start
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(empty_d);
        }
        OT* sb = stage + (chunk & 1) * (32 * BN);
#pragma unroll
        for (int i = 0; i < 32; ++i) sb[i * BN + et] = from_f32<OT>(__uint_as_float(v[i]));
        named_bar_sync(2, 128);
        {
          if (p.vec_store) {
#pragma unroll
            for (int j = 0; j < (32 * ROW_VECS) / 128; ++j) {
              const int idx = j * 128 + et;
              const int mi = idx / ROW_VECS, cv = idx - mi * ROW_VECS;
              const int m = m0 + cb * 32 + mi, n = n0 + cv * VEC;
              if (m < p.M && n < p.N) {
                const uint4 val = *reinterpret_cast<const uint4*>(sb + mi * BN + cv * VEC);
                *reinterpret_cast<uint4*>(out + static_cast<long long>(m) * p.N + n) = val;
              }
            }
          } else {
            const int n = n0 + et;
            if (n < p.N) {
              for (int i = 0; i < 32; ++i) {
                const int m = m0 + cb * 32 + i;
                if (m < p.M) out[static_cast<long long>(m) * p.N + n] = sb[i * BN + et];
              }
            }
          }
        }
      }
    }
  }
#undef LCQ_GIVE_UP

  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// bf16 -> fp16 copy of the activations (exact for |x| in fp16's normal range) with the 8 values
// of every 16-byte piece reordered to (0,4,1,5,2,6,3,7): the order in which the nibble masks
// deliver the weights, so the dequant warps need no re-pairing.
__global__ void __launch_bounds__(256) bf16_to_f16_perm_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, long long n16) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += stride) {
    const uint4 a = __ldg(in + i);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { f[2 * j] = __uint_as_float(w[j] << 16); f[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u); }
    const __half2 h0 = __floats2half2_rn(f[0], f[4]), h1 = __floats2half2_rn(f[1], f[5]);
    const __half2 h2 = __floats2half2_rn(f[2], f[6]), h3 = __floats2half2_rn(f[3], f[7]);
    out[i] = make_uint4(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1),
                        *reinterpret_cast<const uint32_t*>(&h2), *reinterpret_cast<const uint32_t*>(&h3));
  }
}

// out[i] = sum over splits of partial[s][i], rounded once to the output type
template <typename OT>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part, OT* __restrict__ out,
                                                            long long n, int splits) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    float acc = 0.0f;
    for (int s = 0; s < splits; ++s) acc += __ldcs(part + static_cast<long long>(s) * n + i);
    out[i] = from_f32<OT>(acc);
  }
}

// ---------------------------------------------------------------------------- host side
struct Tiling { int bm, n_tiles_n, n_tiles_m, splits, k_tiles_per_split; };

// Tile shape and split-K factor.  Few output tiles (small M and modest N) would leave most SMs
// idle, so K is cut into `splits` ranges (multiples of 256 k) whose float partials are summed by
// a small second kernel.
inline Tiling choose_tiling(int M, int N, int K, int sm_count) {
  Tiling t;
  t.n_tiles_n = (N + BN - 1) / BN;
  if (M < 256) {
    t.bm = ((M + 31) / 32) * 32;
  } else {
    double best = -1.0;
    t.bm = 256;
    for (int bm : {256, 128}) {
      const long long tiles = static_cast<long long>(t.n_tiles_n) * ((M + bm - 1) / bm);
      const long long waves = (tiles + sm_count - 1) / sm_count;
      const double fill = static_cast<double>(tiles) / static_cast<double>(waves * sm_count);
      const double score = fill * (bm == 256 ? 1.0 : 0.8);
      if (score > best) { best = score; t.bm = bm; }
    }
  }
  t.n_tiles_m = (M + t.bm - 1) / t.bm;
  const long long tiles = static_cast<long long>(t.n_tiles_n) * t.n_tiles_m;
  const int w_stages = K / WK;                       // 256-k weight stages
  t.splits = 1;
  if (tiles * 2 <= sm_count && w_stages >= 2) {
    int s = static_cast<int>(sm_count / tiles);
    if (s > w_stages) s = w_stages;
    if (s > 16) s = 16;
    while (s > 1 && w_stages % s != 0) --s;            // equal ranges only
    t.splits = s < 1 ? 1 : s;
  }
  t.k_tiles_per_split = (w_stages / t.splits) * (WK / BK);
  return t;
}

inline bool supported(int M, int N, int K, int G, int x_dtype, int scale_dtype) {
  return M >= 1 && N >= 1 && K >= WK && (K % WK) == 0 && G == 32 &&
         (x_dtype == LCQ_F16 || x_dtype == LCQ_BF16) && scale_dtype == LCQ_F16;
}

inline size_t x_copy_bytes(int M, int K, int x_dtype) {
  return x_dtype == LCQ_BF16 ? ((static_cast<size_t>(M) * K * 2 + 255) & ~static_cast<size_t>(255)) : 0;
}
// [shared counter region][fp16 copy of bf16 activations][split-K float partials]
inline size_t workspace_bytes(int M, int N, int K, int x_dtype, int sm_count = 148) {
  const Tiling t = choose_tiling(M, N, K, sm_count);
  const size_t part = t.splits > 1 ? static_cast<size_t>(t.splits) * M * N * sizeof(float) : 0;
  const size_t xc = x_copy_bytes(M, K, x_dtype);
  return (xc + part) ? kWorkspaceCounterBytes + xc + part : 0;
}

template <typename OT, bool PERM>
int launch_t(const CUtensorMap& tx, const CUtensorMap& tw, const CUtensorMap& ts, const Params& p, int grid,
             size_t smem_bytes, cudaStream_t stream) {
  auto kern = w4a16_gemm_kernel<OT, PERM>;
  static thread_local int configured_device = -1;
  int dev = 0;
  LCQ_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_device != dev) {
    LCQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured_device = dev;
  }
  kern<<<grid, NTHREADS, smem_bytes, stream>>>(tx, tw, ts, p);
  LCQ_CUDA_TRY(cudaGetLastError());
  return LCQ_OK;
}

template <bool PERM>
int launch_by_out(int out_dtype, const CUtensorMap& tx, const CUtensorMap& tw, const CUtensorMap& ts, const Params& p,
                  int grid, size_t smem_bytes, cudaStream_t stream) {
  switch (out_dtype) {
    case LCQ_F32: return launch_t<float, PERM>(tx, tw, ts, p, grid, smem_bytes, stream);
    case LCQ_F16: return launch_t<__half, PERM>(tx, tw, ts, p, grid, smem_bytes, stream);
    case LCQ_BF16: return launch_t<__nv_bfloat16, PERM>(tx, tw, ts, p, grid, smem_bytes, stream);
    default: break;
  }
  set_error("w4a16 gemm: bad out_dtype %d", out_dtype);
  return LCQ_ERR_BAD_ARG;
}

inline int launch(const void* x, const void* w, const void* s, void* out, int M, int N, int K, int x_dtype,
                  int out_dtype, void* workspace, size_t ws_bytes, int sm_count, cudaStream_t stream) {
  if (!aligned(w, 16) || !aligned(s, 16) || !aligned(x, 16)) {
    set_error("w4a16 gemm: x, w_packed and scales must be 16-byte aligned");
    return LCQ_ERR_BAD_ARG;
  }
  const Tiling t = choose_tiling(M, N, K, sm_count);
  const size_t need = workspace_bytes(M, N, K, x_dtype, sm_count);
  if (need && (workspace == nullptr || ws_bytes < need || !aligned(workspace, 256))) {
    set_error("w4a16 gemm: workspace of %zu bytes (256-byte aligned) required, got %zu", need, ws_bytes);
    return LCQ_ERR_WORKSPACE;
  }
  uint8_t* scratch = need ? static_cast<uint8_t*>(workspace) + kWorkspaceCounterBytes : nullptr;
  const void* xh = x;
  // kind::f16 wants both operands in one 16-bit format and the weight tiles must be fp16, so bf16
  // activations are converted once into the workspace.
  if (x_dtype == LCQ_BF16) {
    const long long n16 = static_cast<long long>(M) * K / 8;
    long long blocks = (n16 + 255) / 256;
    if (blocks > static_cast<long long>(sm_count) * 8) blocks = static_cast<long long>(sm_count) * 8;
    bf16_to_f16_perm_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<const uint4*>(x),
                                                                          reinterpret_cast<uint4*>(scratch), n16);
    LCQ_CUDA_TRY(cudaGetLastError());
    xh = scratch;
  }
  float* partials = reinterpret_cast<float*>(scratch + x_copy_bytes(M, K, x_dtype));
  Params p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K;
  p.bm = t.bm; p.n_tiles_n = t.n_tiles_n; p.n_tiles_m = t.n_tiles_m;
  p.splits = t.splits; p.k_tiles_per_split = t.k_tiles_per_split;
  const int kernel_out_dtype = t.splits > 1 ? LCQ_F32 : out_dtype;
  p.out = t.splits > 1 ? static_cast<void*>(partials) : out;
  p.out_dtype = kernel_out_dtype;
  {
    const int vec = kernel_out_dtype == LCQ_F32 ? 4 : 8;
    p.vec_store = (N % vec == 0) && aligned(p.out, 16) && ((static_cast<long long>(M) * N) % vec == 0);
  }
  const long long items = static_cast<long long>(p.n_tiles_n) * p.n_tiles_m * p.splits;
  const int grid = static_cast<int>(items < sm_count ? items : sm_count);
  CUtensorMap tx, tw, ts;
  int rc = encode_tmap_2d(&tx, 1, xh, static_cast<uint64_t>(K), static_cast<uint64_t>(M),
                          static_cast<uint64_t>(K) * 2, BK, p.bm, 3);
  if (rc != LCQ_OK) return rc;
  rc = encode_tmap_2d(&tw, 0, w, static_cast<uint64_t>(K) / 2, static_cast<uint64_t>(N),
                      static_cast<uint64_t>(K) / 2, WK / 2, BN, 3);
  if (rc != LCQ_OK) return rc;
  rc = encode_tmap_2d(&ts, 1, s, static_cast<uint64_t>(K) / 32, static_cast<uint64_t>(N),
                      static_cast<uint64_t>(K) / 16, WK / 32, BN, 0);
  if (rc != LCQ_OK) return rc;
  const size_t smem_bytes = smem_map(p.bm).total;
  const bool perm = (x_dtype == LCQ_BF16);   // the pre-pass already permuted k inside every 8-block
  rc = perm ? launch_by_out<true>(kernel_out_dtype, tx, tw, ts, p, grid, smem_bytes, stream)
            : launch_by_out<false>(kernel_out_dtype, tx, tw, ts, p, grid, smem_bytes, stream);
  if (rc != LCQ_OK || t.splits == 1) return rc;
  const long long n = static_cast<long long>(M) * N;
  long long blocks = (n + 255) / 256;
  if (blocks > static_cast<long long>(sm_count) * 8) blocks = static_cast<long long>(sm_count) * 8;
  switch (out_dtype) {
    case LCQ_F32: splitk_reduce_kernel<float><<<static_cast<int>(blocks), 256, 0, stream>>>(partials, static_cast<float*>(out), n, t.splits); break;
    case LCQ_F16: splitk_reduce_kernel<__half><<<static_cast<int>(blocks), 256, 0, stream>>>(partials, static_cast<__half*>(out), n, t.splits); break;
    case LCQ_BF16: splitk_reduce_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, stream>>>(partials, static_cast<__nv_bfloat16*>(out), n, t.splits); break;
    default: set_error("w4a16 gemm: bad out_dtype %d", out_dtype); return LCQ_ERR_BAD_ARG;
  }
  LCQ_CUDA_TRY(cudaGetLastError());
  return LCQ_OK;
}

}  // namespace gemm_tc
}  // namespace lcq
