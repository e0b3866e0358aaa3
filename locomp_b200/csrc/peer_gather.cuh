// All-gather over NVLink peer memory for the N-column sharded linears: one kernel per rank
// PUSHES its output slice into every rank's region with plain peer stores and unpacks what the
// peers pushed.  No loads from peer memory, no multicast, no NCCL on this path.
//
// Every rank owns one region allocated with cudaMalloc and exported with a CUDA IPC handle; peers
// map it (cudaIpcOpenMemHandle).  The sequence number of a region lives in device memory and is
// advanced by the kernel itself, so a CUDA graph that captured the launch can be replayed.  Ranks
// run on different GPUs (one process per GPU); the wait is on other GPUs' kernels, never on
// another launch of the same GPU, and it is bounded by the library's wait limit.
//
// Reuse rule: the data area a push fills is read by the kernels that follow it on the stream; the
// next push to the same region overwrites it, so those readers must be enqueued ahead of that push
// (stream order does the rest).  A peer can run one call ahead of this rank, never two.  Large slices
// take the bulk form below, whose stores land in the data area itself: there, callers alternate
// between two regions.
#pragma once
#include "common.cuh"

namespace lcq {
namespace peer {

constexpr int MAX_RANKS = 8;
constexpr int FLAG_BYTES = 256;

struct PushArgs {
  uint4* data[MAX_RANKS];        // data area (followed by the staging area) of every rank's region, peer-mapped
  int* flags[MAX_RANKS];         // first 256 bytes of every rank's region: one sequence flag per rank (bulk form)
  const uint4* src;
  long long n16;                 // 16-byte pieces per rank slice
  int rank, world;
  int* state;                    // local: [0] sequence number, [1] CTA arrival counter
};

// Low-latency form: every 4-byte word travels as an 8-byte {word, sequence number} pair, so the
// receiver needs no flag, no fence and no barrier -- it polls the pair itself until the number of
// the current call appears (8-byte stores arrive whole).  Each rank stores its slice, in that
// form, into the staging area of every peer's region (peer stores only), then unpacks what the
// peers stored into its own region's data area.  Two staging buffers alternate by call parity: a
// peer can start call n+1 while this rank still reads call n, but cannot start call n+2 before
// this rank has started n+1 (it needs this rank's slice of n+1 to finish), so two are enough.
// Region layout:  [ 256 B of flags (bulk form) | data: world x slice | staging: 2 x world x 2*slice ].
__device__ __forceinline__ void st_volatile_v4(uint4* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(256) allgather_push_kernel(const PushArgs a) {
  // Programmatic dependent launch: the next kernel on the stream may become resident now (a
  // following decode kernel then prefetches its weights while this all-gather is in flight; it
  // touches activations, outputs and scratch only after this grid has completed).
  griddep_launch_dependents();
  griddep_wait();                // src is the output of the kernel before us on the stream
  const uint32_t seq = static_cast<uint32_t>(*reinterpret_cast<volatile int*>(&a.state[0])) + 1u;
  const long long buf = static_cast<long long>(seq & 1u) * a.world;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long first = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  // send
  for (long long i = first; i < a.n16; i += stride) {
    const uint4 v = a.src[i];
    const uint4 lo = make_uint4(v.x, seq, v.y, seq), hi = make_uint4(v.z, seq, v.w, seq);
#pragma unroll
    for (int g = 0; g < MAX_RANKS; ++g) {
      if (g < a.world && g != a.rank) {
        uint4* dst = a.data[g] + static_cast<long long>(a.world) * a.n16 + ((buf + a.rank) * a.n16 + i) * 2;
        st_volatile_v4(dst, lo);
        st_volatile_v4(dst + 1, hi);
      }
    }
    a.data[a.rank][static_cast<long long>(a.rank) * a.n16 + i] = v;
  }
  // receive: bounded polling on this rank's own staging area.  For each of its elements a thread polls
  // the pairs of ALL peers together (their loads are in flight at the same time), so a call costs about
  // one round trip to L2 per retry, not one per peer.
  const uint64_t t0 = global_timer_ns();
  const uint64_t limit = wait_limit_ns();
  bool gave_up = false;
  const uint4* stage0 = a.data[a.rank] + static_cast<long long>(a.world) * a.n16 + buf * a.n16 * 2;
  for (long long i = first; i < a.n16 && !gave_up; i += stride) {
    unsigned pending = ((1u << a.world) - 1u) & ~(1u << a.rank);
    int spins = 0;
    while (pending != 0u) {
      uint4 lo[MAX_RANKS], hi[MAX_RANKS];
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r) {
        if ((pending >> r) & 1u) {
          const uint4* stage = stage0 + static_cast<long long>(r) * a.n16 * 2;
          lo[r] = ld_volatile_v4(stage + 2 * i);
          hi[r] = ld_volatile_v4(stage + 2 * i + 1);
        }
      }
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r) {
        if (((pending >> r) & 1u) && lo[r].y == seq && lo[r].w == seq && hi[r].y == seq && hi[r].w == seq) {
          a.data[a.rank][static_cast<long long>(r) * a.n16 + i] = make_uint4(lo[r].x, lo[r].z, hi[r].x, hi[r].z);
          pending &= ~(1u << r);
        }
      }
      if (pending != 0u && (++spins & 63) == 0 && global_timer_ns() - t0 > limit) {
        atomicExch(&g_device_status, 30 + (__ffs(pending) - 1));
        gave_up = true;
        break;
      }
    }
  }
  // the last CTA to finish advances the sequence number (every CTA has read it by then)
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(&a.state[1], 1);
    if (prev == static_cast<int>(gridDim.x) - 1) {
      a.state[1] = 0;
      a.state[0] = static_cast<int>(seq);
      __threadfence();
    }
  }
}

// Bulk form, for slices large enough that doubling the bytes costs more than two fences: plain
// stores of the slice into slot `rank` of every region's data area, a system-wide fence after the
// last CTA's stores, this rank's sequence number into flags[rank] of every region, then a bounded
// wait until the own region shows the number from every rank.  Because peers write straight into
// the data area, a region must not be pushed to again while any rank may still read its previous
// contents: callers alternate between two regions.
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(256) allgather_bulk_kernel(const PushArgs a) {
  griddep_launch_dependents();
  griddep_wait();                // src is the output of the kernel before us on the stream
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  // four 16-byte pieces per thread and step: all four loads in flight before the first peer store
  for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < a.n16; i0 += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * stride;
      v[u] = i < a.n16 ? a.src[i] : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * stride;
      if (i < a.n16) {
        const long long o = static_cast<long long>(a.rank) * a.n16 + i;
#pragma unroll
        for (int g = 0; g < MAX_RANKS; ++g)
          if (g < a.world) a.data[g][o] = v[u];
      }
    }
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  __threadfence_system();        // one fence per CTA, after the barrier: covers every thread's slice stores
  if (gridDim.x > 1) {
    const int prev = atomicAdd(&a.state[1], 1);
    if (prev != static_cast<int>(gridDim.x) - 1) return;
    a.state[1] = 0;
    __threadfence_system();      // last CTA: the other CTAs' fenced stores are ordered before the flags below
  }
  const int seq = a.state[0] + 1;
  a.state[0] = seq;
  for (int g = 0; g < a.world; ++g) st_release_sys(a.flags[g] + a.rank, seq);
  const uint64_t t0 = global_timer_ns();
  const uint64_t limit = wait_limit_ns();
  const int* mine = a.flags[a.rank];
  for (int r = 0; r < a.world; ++r) {
    while (ld_acquire_sys(mine + r) - seq < 0) {                     // wrap-safe "not yet"
      if (global_timer_ns() - t0 > limit) { atomicExch(&g_device_status, 30 + r); return; }
    }
  }
}

// The pair form doubles the bytes on the wire and saves two fences (a few microseconds): it is used
// while the extra bytes to all peers stay under 1 MiB.  Every rank takes the same decision.
inline long long pair_limit_bytes() {     // LCQ_GATHER_PAIR_LIMIT_KIB overrides (read once)
  static const long long v = [] {
    const char* e = getenv("LCQ_GATHER_PAIR_LIMIT_KIB");
    const long long n = e ? atoll(e) : 0;
    return n > 0 ? n * 1024 : (1LL << 20);
  }();
  return v;
}
inline bool use_pairs(long long bytes_per_rank, int world) { return bytes_per_rank * (world - 1) <= pair_limit_bytes(); }

inline int launch_push(const PushArgs& a, cudaStream_t stream) {
  const bool pairs = use_pairs(a.n16 * 16, a.world);
  static const int bulk_cap = [] { const char* e = getenv("LCQ_GATHER_BULK_CTAS"); const int n = e ? atoi(e) : 0; return n > 0 ? n : 148; }();
  long long blocks = (a.n16 + 255) / 256;
  if (blocks > (pairs ? 64 : bulk_cap)) blocks = pairs ? 64 : bulk_cap;
  if (blocks < 1) blocks = 1;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(static_cast<unsigned>(blocks));
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  if (pairs) LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, allgather_push_kernel, a));
  else LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, allgather_bulk_kernel, a));
  return LCQ_OK;
}

}  // namespace peer
}  // namespace lcq
