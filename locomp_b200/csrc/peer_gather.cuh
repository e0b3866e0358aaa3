// All-gather over NVLink peer memory for the N-column sharded linears: one kernel per rank
// PUSHES its output slice into every rank's gathered buffer with plain peer stores, then signals
// and waits on flags.  No loads from peer memory, no multicast, no NCCL on this path.
//
// Every rank owns one region  [ flags: 64 ints | data: world x bytes_per_rank ]  allocated with
// cudaMalloc and exported with a CUDA IPC handle; peers map it (cudaIpcOpenMemHandle).  A call
//   1. copies this rank's slice into slot `rank` of every region (its own included),
//   2. after the last CTA's stores are fenced system-wide, writes the call's sequence number
//      into flags[rank] of every region,
//   3. waits -- bounded by the library's wait limit -- until its own region shows that sequence number from every
//      rank, so kernels that follow on the stream see the complete gathered buffer.
// The sequence number lives in device memory and is advanced by the kernel itself, so a CUDA
// graph that captured the launch can be replayed.  Ranks run on different GPUs (one process per
// GPU); the wait is on other GPUs' kernels, never on another launch of the same GPU.
//
// Reuse rule: a rank's push overwrites slot `rank` of EVERY rank's region as soon as it runs, so
// a region may be pushed to again only when no rank can still be reading its previous contents.
// A rank leaves push k only after it has seen every rank's flag of push k, i.e. every rank has
// at least started push k; it has not necessarily finished reading the data of push k-1 on the
// same region.  So between two pushes to one region there must be (a) the readers of the first,
// enqueued ahead of the second push on every rank's stream, and (b) one complete push/wait round
// on a DIFFERENT region, which proves that every rank's stream has passed those readers.  A
// layer called back to back therefore alternates between two regions.
#pragma once
#include "common.cuh"

namespace lcq {
namespace peer {

constexpr int MAX_RANKS = 8;
constexpr int FLAG_BYTES = 256;

struct PushArgs {
  uint4* data[MAX_RANKS];        // data area of every rank's region (peer-mapped, own included)
  int* flags[MAX_RANKS];         // flag area of every rank's region
  const uint4* src;
  long long n16;                 // 16-byte pieces per rank slice
  int rank, world;
  int* state;                    // local: [0] sequence number, [1] CTA arrival counter
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(256) allgather_push_kernel(const PushArgs a) {
  // Programmatic dependent launch: the next kernel on the stream may become resident now (a
  // following decode kernel then prefetches its weights while this all-gather is in flight; it
  // touches activations, outputs and scratch only after this grid has completed).
  griddep_launch_dependents();
  griddep_wait();                // src is the output of the kernel before us on the stream
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < a.n16; i += stride) {
    const uint4 v = a.src[i];
    const long long o = static_cast<long long>(a.rank) * a.n16 + i;
#pragma unroll
    for (int g = 0; g < MAX_RANKS; ++g)
      if (g < a.world) a.data[g][o] = v;
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
  // every slice store of this rank is visible system-wide: publish, then wait for the peers
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

inline int launch_push(const PushArgs& a, cudaStream_t stream) {
  long long blocks = (a.n16 + 255) / 256;
  if (blocks > 32) blocks = 32;
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
  LCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, allgather_push_kernel, a));
  return LCQ_OK;
}

}  // namespace peer
}  // namespace lcq
