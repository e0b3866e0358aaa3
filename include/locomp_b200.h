/*
 * locomp_b200 -- C ABI of the B200 (sm_100a) weight-quantized matmul / dequantize library.
 *
 * The library replaces, for NVIDIA B200, the four operators that the reference project
 * (Zyora-Dev/locomp v1.0.0) JIT-generates from examples/38_quantized_matmul.py and
 * examples/52_dequantize.py.  The reference has no fixed C ABI for them: it emits one
 * `extern "C" void locomp_launch_<kernel>(int,int,int,int,void** args)` per kernel AND per
 * constexpr tuple (locomp/backends/cuda_codegen.py:349-389), called through ctypes
 * (locomp/api.py:805-851).  The entry points below are what a fixed binding for the same
 * operators binds instead; each comment names the reference interface it stands in for.
 *
 * Conventions
 *   - All pointers are DEVICE pointers unless the name says host.  Row-major, contiguous.
 *   - w_packed : uint8 [N, K/2], low nibble = even k, high nibble = odd k, stored value = q + 8
 *   - w_int8   : int8  [N, K]
 *   - scales   : [N, K/group_size], dtype given by scale_dtype
 *   - x        : [M, K]   (M = 1 is the reference's matvec),  out : [M, N]
 *   - stream   : a cudaStream_t passed as void* (NULL = legacy default stream).  Calls are
 *                stream-ordered and never synchronise the device.
 *   - Every function returns an lcq_status (0 = ok, negative = error) and never throws,
 *     exits, traps the device or allocates device memory unless its comment says so.
 */
#ifndef LOCOMP_B200_H
#define LOCOMP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define LCQ_OK               0
#define LCQ_ERR_BAD_ARG     (-1)  /* null pointer, non-positive size, K % group_size != 0, ...   */
#define LCQ_ERR_UNSUPPORTED (-2)  /* dtype / shape combination no kernel covers                  */
#define LCQ_ERR_CUDA        (-3)  /* a CUDA runtime/driver call failed; see lcq_last_error()     */
#define LCQ_ERR_WORKSPACE   (-4)  /* workspace missing, misaligned or too small                  */
#define LCQ_ERR_TIMEOUT     (-5)  /* a bounded device-side wait expired (reported by lcq_check_device_status) */

/* dtype codes for x_dtype / scale_dtype / out_dtype */
#define LCQ_F32  0
#define LCQ_F16  1
#define LCQ_BF16 2

/* algorithm selector for lcq_matmul_int4/int8 */
#define LCQ_ALGO_AUTO    0   /* pick by shape and dtype                                         */
#define LCQ_ALGO_SIMT    1   /* warp-per-row CUDA-core kernel; any K % group_size == 0           */
#define LCQ_ALGO_GEMV_TC 2   /* int4, M <= 16, K % 64 == 0: TMA-staged int4 stream + warp-level MMA, split-K */
#define LCQ_ALGO_GEMM_TC 3   /* M >= 17: TMA + in-kernel dequant + tcgen05 MMA, TMEM accumulators */
#define LCQ_ALGO_GEMV_W8 4   /* int8, M <= 8: TMA-staged int8 stream, 128-bit shared loads, float32 math */

int         lcq_version(void);
const char* lcq_status_string(int status);
/* Text of the last error raised on the calling thread ("" if none). */
const char* lcq_last_error(void);

/* Name, SM count and L2 size of a device; any out pointer may be NULL. */
int lcq_device_info(int device, char* name, size_t name_len, int* sm_count, int* l2_bytes,
                    int* cc_major, int* cc_minor);

/*
 * Dequantize int4 -> float.  out[r, k] = (float(nibble) - 8) * float(scales[r, k / group_size]),
 * one rounding in float32; out_dtype F16/BF16 round that float32 value to nearest-even.
 * Replaces the generated kernel `dequant_int4` (examples/52_dequantize.py:27-53), i.e.
 * locomp_launch_dequant_int4(grid,..., args = {W, SCALES, OUT}) with K, HALF_K, NUM_SCALES and
 * GROUP_SIZE baked in.  Requires K % 2 == 0 and K % group_size == 0 (the reference kernel
 * silently truncates K to a multiple of 256; this one covers all of K).
 */
int lcq_dequant_int4(const void* w_packed, const void* scales, void* out,
                     int64_t N, int64_t K, int group_size,
                     int scale_dtype, int out_dtype, void* stream);

/* Dequantize int8 -> float: out[r, k] = float(w[r, k]) * scales[r, k / group_size].
 * Replaces `dequant_int8` (examples/52_dequantize.py:60-74). */
int lcq_dequant_int8(const void* w_int8, const void* scales, void* out,
                     int64_t N, int64_t K, int group_size,
                     int scale_dtype, int out_dtype, void* stream);

/*
 * Quantized matmul, int4 weights: out[m, n] = sum_k x[m, k] * (nibble(n, k) - 8) * scales[n, k / G],
 * float32 accumulation, out rounded to out_dtype.  M = 1 with F32 everywhere is the reference's
 * `dequant_matvec_int4` (examples/38_quantized_matmul.py:30-87; launch wrapper
 * locomp_launch_dequant_matvec_int4, args = {X, W, scales, O}); M > 1 and 16-bit dtypes are the
 * batched generalisation X @ dequant(W)^T.  The reference kernel asserts K % 256 == 0
 * (examples/38_quantized_matmul.py:145); this one needs only K % group_size == 0, K % 2 == 0.
 *
 * workspace: device scratch of at least lcq_matmul_workspace_bytes(...) bytes, 256-byte aligned,
 * ZERO-FILLED before its first use; the kernels leave it zeroed again, so one buffer can be
 * reused by consecutive calls on one stream.  Calls that may overlap on the GPU need separate
 * workspaces.  May be NULL when the size query returns 0.
 *
 * Preconditions.  (1) The kernels are launched with programmatic stream serialisation and fetch
 * w_packed / scales BEFORE the kernel ahead of them on the stream has finished: both must be complete
 * before that kernel starts (weights written on the same stream need one synchronisation before the
 * first matmul), or set LCQ_NO_PDL=1 in the environment.  x, out and workspace are touched only after
 * that kernel has completed.  (2) With F16/BF16 activations the tensor-core kernels compute in fp16:
 * |x| must not exceed 65504, and |x| below about 1e-3 loses precision in the M <= 16 kernel (it divides
 * half of the activations by 16, into fp16's subnormal range).  F32 activations take a float32 kernel.
 */
int lcq_matmul_int4(const void* x, const void* w_packed, const void* scales, void* out,
                    int M, int N, int K, int group_size,
                    int x_dtype, int scale_dtype, int out_dtype, int algo,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Quantized matmul, int8 weights; M = 1 / F32 is `dequant_matvec_int8`
 * (examples/38_quantized_matmul.py:94-134).  Per-output-channel scales are group_size = K. */
int lcq_matmul_int8(const void* x, const void* w_int8, const void* scales, void* out,
                    int M, int N, int K, int group_size,
                    int x_dtype, int scale_dtype, int out_dtype, int algo,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Bytes of workspace lcq_matmul_int4 / lcq_matmul_int8 need for this problem on the current
 * device (0 if none).  wbits is 4 or 8.  Returns (size_t)-1 for an invalid problem. */
size_t lcq_matmul_workspace_bytes(int wbits, int M, int N, int K, int group_size,
                                  int x_dtype, int scale_dtype, int out_dtype, int algo);

/* Which algorithm LCQ_ALGO_AUTO resolves to for this problem (one of LCQ_ALGO_*), or a
 * negative status. */
int lcq_matmul_select_algo(int wbits, int M, int N, int K, int group_size,
                           int x_dtype, int scale_dtype, int out_dtype);

/*
 * Decode matmul that allocates nothing.  No counterpart in the reference.
 *
 * Same computation and same kernel as lcq_matmul_int4 with LCQ_ALGO_GEMV_TC (M <= 16,
 * group_size 32, K % 64 == 0, f16 scales, f16/bf16 x), but the split-K scratch is a fixed array
 * inside the library instead of a caller-provided workspace.  It exists for callers that cannot
 * obtain device memory at the point of the call: a serving loop whose framework has taken the
 * whole device into its own pool (so cudaMalloc fails or is forbidden), or a host that must not
 * make a call that synchronises the device.  This function, and everything under it, calls no
 * cudaMalloc / cudaFree and no allocating library routine; the caller still passes x, weights,
 * scales and out.
 *
 * Limits and rules
 *   - The scratch holds lcq_noalloc_scratch_bytes() bytes (8 MiB); every GPU that loads the
 *     library keeps that much memory until the process exits.  A problem whose plan needs more
 *     is refused with LCQ_ERR_WORKSPACE (the message says how much) -- use lcq_matmul_int4.
 *   - The first call on each device looks up the array's device address and sets kernel
 *     attributes; make that first call before any stream capture.
 *   - All calls on a device share the one array, which keeps the previous call's contents; each
 *     call clears the counters it needs (a cudaMemsetAsync on `stream`).  Two calls that overlap
 *     on the GPU -- different streams, no ordering between them -- race on it and give wrong
 *     results; order them, or use lcq_matmul_int4 with separate workspaces.
 */
int lcq_matmul_int4_noalloc(const void* x, const void* w_packed, const void* scales, void* out,
                            int M, int N, int K, int group_size,
                            int x_dtype, int scale_dtype, int out_dtype, void* stream);

/* Size in bytes of the built-in scratch of lcq_matmul_int4_noalloc.  No counterpart in the reference. */
size_t lcq_noalloc_scratch_bytes(void);

/*
 * Decode-step kernels on either side of the quantized linears.  `dtype` (LCQ_F32 / F16 / BF16) is
 * the storage type of every tensor of the call; arithmetic is float32, results are rounded once.
 * All are stream-ordered single kernels that take part in programmatic dependent launch.
 *
 * lcq_rms_norm: out[r, i] = x[r, i] * rsqrt(mean_i(x[r, :]^2) + eps) * weight[i], x and out [rows, n].
 *   Replaces `rms_norm_kernel` (examples/54_smollm2_inference.py:40-73, launched [(rows,),(128,)] with
 *   N and EPS_X1000 baked in; eps = EPS_X1000 * 1e-6).
 * lcq_residual_rms_norm: hidden[r, :] += delta[r, :] (in place), then out = rms_norm(hidden) as above:
 *   `add_inplace_kernel` followed by `rms_norm_kernel` (examples/54_smollm2_inference.py:529-534) in one
 *   launch; the reference's own fused form is examples/34_fused_residual_norm.py:18-60.
 * lcq_silu_mul: out[i] = gate[i] * sigmoid(gate[i]) * up[i].  Replaces `silu_mul_kernel`
 *   (examples/54_smollm2_inference.py:113-120).
 * lcq_add_inplace: a[i] += b[i].  Replaces `add_inplace_kernel` (examples/54_smollm2_inference.py:164-167).
 */
int lcq_rms_norm(const void* x, const void* weight, void* out, int64_t rows, int n, float eps, int dtype, void* stream);
int lcq_residual_rms_norm(void* hidden, const void* delta, const void* weight, void* out, int64_t rows, int n,
                          float eps, int dtype, void* stream);
int lcq_silu_mul(const void* gate, const void* up, void* out, int64_t n, int dtype, void* stream);
int lcq_add_inplace(void* a, const void* b, int64_t n, int dtype, void* stream);

/*
 * Embedding lookup: out[t, :] = table[token_ids[t], :]; token_ids int32 [tokens], table [vocab, dim],
 * out [tokens, dim], both of `dtype`.  Replaces `_embed_fp32` / `_embed_fp16`
 * (locomp/_builtin_kernels.py:8-25) behind locomp.embed_lookup (locomp/api.py:1025-1038).  An id
 * outside [0, vocab) gives a row of zeros and is reported by lcq_check_device_status (the reference
 * reads out of bounds).
 */
int lcq_embed_lookup(const void* token_ids, const void* table, void* out, int64_t tokens, int vocab, int dim,
                     int dtype, void* stream);

/*
 * Greedy sampling on the device: out[r] (int32) = index of the first maximum of x[r, 0..n), so a
 * decode loop copies back 4 bytes per token instead of the logits.  Same result as the host-side
 * np.argmax the reference applies to the downloaded logits (examples/54_smollm2_inference.py:606):
 * ties go to the lowest index, a NaN counts as the maximum.
 */
int lcq_argmax(const void* x, void* out, int64_t rows, int n, int dtype, void* stream);

/*
 * Weight quantisers with the reference's arithmetic, bit for bit: w [N, K] of `w_dtype` ->
 * w_packed uint8 [N, K/2] (or w_int8 int8 [N, K]) and scales float32 [N, K/group_size].
 * style 0 = quantize_int4 / quantize_int8 of examples/38_quantized_matmul.py:248-293
 *           (scale = amax/7 resp. amax/127, 1.0 for an all-zero group; q = clip(rint(w/scale) [+8]));
 * style 1 = quantize_int4_ref of examples/52_dequantize.py:110-126 and the int8 form of its self-check
 *           (:162-165): amax floored at 1e-10 (int4 only), q = clip(rint(w/(scale + 1e-10)) [+8]).
 * Both are O(N*K) Python loops / NumPy passes in the reference.
 */
int lcq_quantize_int4(const void* w, void* w_packed, void* scales, int64_t N, int64_t K, int group_size,
                      int w_dtype, int style, void* stream);
int lcq_quantize_int8(const void* w, void* w_int8, void* scales, int64_t N, int64_t K, int group_size,
                      int w_dtype, int style, void* stream);

/*
 * All-gather over NVLink peer memory for N-column sharded linears (one process per GPU).  No
 * counterpart in the reference, which has no multi-GPU code.
 *
 * Each rank owns one region of lcq_peer_region_bytes(bytes_per_rank, world) bytes:
 * [256 bytes][data: world slices][staging: 2 x world x 2 slices].  lcq_peer_alloc allocates it
 * (cudaMalloc, zero-filled -- a set-up call, not for the hot path) and returns a 64-byte CUDA IPC
 * handle to hand to the other ranks; lcq_peer_open maps a peer's region from its handle.
 * lcq_allgather_push(src, ..., regions[0..world-1], rank, world, state, stream) enqueues ONE kernel
 * that stores this rank's slice, as {word, sequence number} pairs, into the staging area of every
 * peer's region (peer stores only, never peer loads; no fence, no flag: the receiver polls the pairs
 * themselves) and unpacks the peers' slices into the data area of its own region, which then holds
 * every rank's slice of the call at byte offset 256 + r * bytes_per_rank.  (Slices so large that the
 * pairs would add more than 1 MiB per call are instead stored plainly into the peers' data areas,
 * followed by a system-wide fence and per-rank sequence flags; with such slices, alternate between
 * two regions, because peers then write into the area the previous call's readers use.)  The wait is bounded; on
 * expiry lcq_check_device_status reports it.  `state`: 2 zero-initialised ints of local device memory
 * per region.  All ranks must issue the same sequence of pushes per region.  world <= 8; slices are
 * multiples of 16 bytes.
 */
int lcq_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64);
int lcq_peer_open(const unsigned char* handle64, void** ptr);
int lcq_peer_close(void* ptr);
int lcq_peer_free(void* ptr);
int lcq_allgather_push(const void* src, size_t bytes_per_rank, void* const* regions, int rank, int world,
                       void* state, void* stream);
size_t lcq_peer_region_bytes(size_t bytes_per_rank, int world);

/*
 * Sharding context for a host that is not Python: one per rank (one process per GPU), for linears
 * whose output columns are split across the GPUs of one box.  No counterpart in the reference.
 *   lcq_shard_ctx_create   allocates this rank's two gather regions (for slices of up to
 *                          max_slice_bytes = M * N/world * sizeof(out)), its scratch, and returns two
 *                          64-byte IPC handles (128 bytes) to hand to the other ranks by any means.
 *   lcq_shard_ctx_connect  maps the peers' regions: all_handles = world x 128 bytes, rank-major.
 *                          Every rank must have created its context before any rank connects.
 *   lcq_sharded_matmul_int4  runs lcq_matmul_int4 on this rank's row block (w_local [N_total/world, K/2],
 *                          scales_local [N_total/world, K/G]) with the replicated x [M, K], then the
 *                          peer all-gather, both on `stream`; *gathered = device pointer to
 *                          [world, M, N_total/world] of out_dtype (row-major [1, N_total] when M = 1),
 *                          valid until the call after next on this context (two regions alternate).
 *                          The first call of a problem size allocates its workspace (cudaMalloc,
 *                          synchronises the device); later calls allocate nothing.
 *   lcq_shard_ctx_destroy  synchronises the device and frees everything; every rank, after its last call.
 * Set-up and tear-down are not for the hot path.  All ranks must issue the same sequence of calls.
 */
typedef struct lcq_shard_ctx lcq_shard_ctx;
int lcq_shard_ctx_create(int rank, int world, size_t max_slice_bytes, lcq_shard_ctx** ctx, unsigned char* handles128);
int lcq_shard_ctx_connect(lcq_shard_ctx* ctx, const unsigned char* all_handles);
int lcq_sharded_matmul_int4(lcq_shard_ctx* ctx, const void* x, const void* w_local, const void* scales_local,
                            void** gathered, int M, int N_total, int K, int group_size,
                            int x_dtype, int scale_dtype, int out_dtype, int algo, void* stream);
int lcq_shard_ctx_destroy(lcq_shard_ctx* ctx);

/*
 * Device-side status word.  Kernels that wait on an mbarrier do so with an iteration limit;
 * when a wait gives up the kernel records it here and returns instead of hanging.  Reads the
 * word of the current device (synchronising `stream` first), clears it and returns LCQ_OK or
 * LCQ_ERR_TIMEOUT.  No counterpart in the reference, whose launch wrapper never checks errors.
 */
int lcq_check_device_status(void* stream);

/*
 * Sets, for the CURRENT device, how long a kernel of this library waits (on an mbarrier or on a
 * peer's flag) before it gives up, records the failure for lcq_check_device_status and returns.
 * Default 2,000,000,000 ns.  Synchronises the device (it writes a device variable); a set-up call.
 * No counterpart in the reference.
 */
int lcq_set_wait_limit_ns(unsigned long long limit_ns);

/*
 * Diagnostic, host only: builds the work plan the GEMV_TC kernel would use for (M, N, K) on a
 * device with sm_count SMs and replays its device-side schedule on the CPU, checking that
 * every (row block, k tile) is produced exactly once and that scratch slots and contributor
 * counts agree.  fields (may be NULL) receives {grid, row blocks, k ranges, tiles per range,
 * CTAs per range, max split, shared-memory bytes, m tiles}.  No counterpart in the reference.
 */
int lcq_gemv_tc_plan_check(int M, int N, int K, int sm_count, int* fields);

/*
 * Host-only: CTAs per thread-block cluster the decode kernel would use for this problem on a GPU
 * with sm_count SMs (1 = no clusters: stream-K with scratch, or whole row blocks per CTA; 2, 4 or 8 =
 * cluster mode, partial sums meet in the first CTA's shared memory).  Negative: status code.
 */
int lcq_gemv_tc_plan_cluster(int M, int N, int K, int sm_count);

#ifdef __cplusplus
}
#endif
#endif /* LOCOMP_B200_H */
