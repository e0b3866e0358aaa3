// locomp_b200 shared library: the extern "C" boundary declared in include/locomp_b200.h.
// Single translation unit (the kernel headers are included here) so the device status word
// and the kernels link without relocatable device code.
#include <stdarg.h>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "dequant.cuh"
#include "gemv_simt.cuh"
#include "gemv_tc.cuh"
#include "gemv_w8.cuh"
#include "gemm_tc.cuh"
#include "peer_gather.cuh"
#include "glue.cuh"
#include "quantize.cuh"

namespace lcq {

static thread_local char t_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) in %s", static_cast<int>(e), cudaGetErrorString(e), what);
  return LCQ_ERR_CUDA;
}

// ---------------------------------------------------------------- tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int encode_tmap_2d(void* out_map, int dtype_code, const void* base, uint64_t inner, uint64_t outer,
                   uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle_code) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return LCQ_ERR_CUDA;
  }
  CUtensorMapDataType dt = dtype_code == 0 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                          : dtype_code == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                            : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMapSwizzle sw = swizzle_code == 0 ? CU_TENSOR_MAP_SWIZZLE_NONE
                         : swizzle_code == 1 ? CU_TENSOR_MAP_SWIZZLE_32B
                         : swizzle_code == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                                             : CU_TENSOR_MAP_SWIZZLE_128B;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(static_cast<CUtensorMap*>(out_map), dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (inner=%llu outer=%llu stride=%llu box=%ux%u)",
              static_cast<int>(r), static_cast<unsigned long long>(inner), static_cast<unsigned long long>(outer),
              static_cast<unsigned long long>(row_stride_bytes), box_inner, box_outer);
    return LCQ_ERR_CUDA;
  }
  return LCQ_OK;
}

// ---------------------------------------------------------------- device properties (cached per device)
struct DevInfo { int sm_count = 0; int l2 = 0; int major = 0; int minor = 0; bool ok = false; };
static DevInfo g_dev[64];
static std::mutex g_dev_mu;

static int current_dev_info(DevInfo& out) {
  int dev = 0;
  LCQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) { set_error("device index %d out of range", dev); return LCQ_ERR_BAD_ARG; }
  std::lock_guard<std::mutex> lk(g_dev_mu);
  if (!g_dev[dev].ok) {
    LCQ_CUDA_TRY(cudaDeviceGetAttribute(&g_dev[dev].sm_count, cudaDevAttrMultiProcessorCount, dev));
    LCQ_CUDA_TRY(cudaDeviceGetAttribute(&g_dev[dev].l2, cudaDevAttrL2CacheSize, dev));
    LCQ_CUDA_TRY(cudaDeviceGetAttribute(&g_dev[dev].major, cudaDevAttrComputeCapabilityMajor, dev));
    LCQ_CUDA_TRY(cudaDeviceGetAttribute(&g_dev[dev].minor, cudaDevAttrComputeCapabilityMinor, dev));
    g_dev[dev].ok = true;
  }
  out = g_dev[dev];
  return LCQ_OK;
}

static bool dtype_ok(int d) { return d == LCQ_F32 || d == LCQ_F16 || d == LCQ_BF16; }

static int check_problem(int wbits, long long M, long long N, long long K, int G) {
  if (wbits != 4 && wbits != 8) { set_error("wbits must be 4 or 8, got %d", wbits); return LCQ_ERR_BAD_ARG; }
  if (M < 0 || N < 0 || K <= 0 || G <= 0) {
    set_error("bad sizes M=%lld N=%lld K=%lld group_size=%d", M, N, K, G);
    return LCQ_ERR_BAD_ARG;
  }
  if (K % G != 0) { set_error("K=%lld is not a multiple of group_size=%d", K, G); return LCQ_ERR_BAD_ARG; }
  if (wbits == 4 && (K % 2) != 0) { set_error("int4 weights need an even K, got %lld", K); return LCQ_ERR_BAD_ARG; }
  if (M > 2000000000LL / 4 || N > 2000000000LL || K > 2000000000LL) {
    set_error("sizes beyond 32-bit indexing are not supported");
    return LCQ_ERR_UNSUPPORTED;
  }
  return LCQ_OK;
}

// ---------------------------------------------------------------- dispatch helpers
template <typename ST>
static int dequant_by_out(int wbits, const void* w, const void* s, void* out, long long N, long long K, int G,
                          int out_dtype, int sm, cudaStream_t st) {
  switch (out_dtype) {
    case LCQ_F32: return launch_dequant<ST, float>(wbits, w, s, out, N, K, G, sm, st);
    case LCQ_F16: return launch_dequant<ST, __half>(wbits, w, s, out, N, K, G, sm, st);
    case LCQ_BF16: return launch_dequant<ST, __nv_bfloat16>(wbits, w, s, out, N, K, G, sm, st);
  }
  return LCQ_ERR_BAD_ARG;
}

static int dequant_entry(int wbits, const void* w, const void* s, void* out, int64_t N, int64_t K, int G,
                         int scale_dtype, int out_dtype, void* stream) {
  int rc = check_problem(wbits, 1, N, K, G);
  if (rc != LCQ_OK) return rc;
  if (!dtype_ok(scale_dtype) || !dtype_ok(out_dtype)) { set_error("bad dtype code"); return LCQ_ERR_BAD_ARG; }
  if (N == 0) return LCQ_OK;
  if (!w || !s || !out) { set_error("null pointer argument"); return LCQ_ERR_BAD_ARG; }
  DevInfo di;
  rc = current_dev_info(di);
  if (rc != LCQ_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (scale_dtype) {
    case LCQ_F32: return dequant_by_out<float>(wbits, w, s, out, N, K, G, out_dtype, di.sm_count, st);
    case LCQ_F16: return dequant_by_out<__half>(wbits, w, s, out, N, K, G, out_dtype, di.sm_count, st);
    case LCQ_BF16: return dequant_by_out<__nv_bfloat16>(wbits, w, s, out, N, K, G, out_dtype, di.sm_count, st);
  }
  return LCQ_ERR_BAD_ARG;
}

template <int WBITS, typename XT, typename ST>
static int simt_by_out(const void* x, const void* w, const void* s, void* out, int M, int N, int K, int G,
                       int out_dtype, cudaStream_t st) {
  switch (out_dtype) {
    case LCQ_F32: return launch_gemv_simt<WBITS, XT, ST, float>(x, w, s, out, M, N, K, G, st);
    case LCQ_F16: return launch_gemv_simt<WBITS, XT, ST, __half>(x, w, s, out, M, N, K, G, st);
    case LCQ_BF16: return launch_gemv_simt<WBITS, XT, ST, __nv_bfloat16>(x, w, s, out, M, N, K, G, st);
  }
  return LCQ_ERR_BAD_ARG;
}
template <int WBITS, typename XT>
static int simt_by_scale(const void* x, const void* w, const void* s, void* out, int M, int N, int K, int G,
                         int scale_dtype, int out_dtype, cudaStream_t st) {
  switch (scale_dtype) {
    case LCQ_F32: return simt_by_out<WBITS, XT, float>(x, w, s, out, M, N, K, G, out_dtype, st);
    case LCQ_F16: return simt_by_out<WBITS, XT, __half>(x, w, s, out, M, N, K, G, out_dtype, st);
    case LCQ_BF16: return simt_by_out<WBITS, XT, __nv_bfloat16>(x, w, s, out, M, N, K, G, out_dtype, st);
  }
  return LCQ_ERR_BAD_ARG;
}
template <int WBITS>
static int simt_entry(const void* x, const void* w, const void* s, void* out, int M, int N, int K, int G,
                      int x_dtype, int scale_dtype, int out_dtype, cudaStream_t st) {
  if (M > 4 * 65535) { set_error("SIMT path supports M <= 262140"); return LCQ_ERR_UNSUPPORTED; }
  switch (x_dtype) {
    case LCQ_F32: return simt_by_scale<WBITS, float>(x, w, s, out, M, N, K, G, scale_dtype, out_dtype, st);
    case LCQ_F16: return simt_by_scale<WBITS, __half>(x, w, s, out, M, N, K, G, scale_dtype, out_dtype, st);
    case LCQ_BF16: return simt_by_scale<WBITS, __nv_bfloat16>(x, w, s, out, M, N, K, G, scale_dtype, out_dtype, st);
  }
  return LCQ_ERR_BAD_ARG;
}

// Scratch the decode kernel needs for M rows: the call runs in chunks of 16 rows plus one tail
// chunk of M % 16 rows, and the tail's plan can need more scratch than a full chunk's.
static size_t gemv_tc_workspace_bytes(int M, int N, int K, int sm_count) {
  size_t need = gemv_tc::make_plan(M < 16 ? M : 16, N, K, sm_count).workspace_bytes;
  if (M > 16 && (M % 16) != 0) {
    const size_t tail = gemv_tc::make_plan(M % 16, N, K, sm_count).workspace_bytes;
    if (tail > need) need = tail;
  }
  return need;
}

static int select_algo(int wbits, int M, int N, int K, int G, int x_dtype, int scale_dtype, int out_dtype) {
  (void)out_dtype;
  // The prefill kernel rounds each dequantised weight to fp16 (relative error 2^-12); summed over
  // K > 16384 that error alone reaches the 1e-2 absolute output tolerance in a few outputs per
  // million, so long-K problems with few rows stay on the decode kernel, whose products are exact.
  const bool long_k_few_rows = K > 16384 && M <= 64;
  if (wbits == 4 && M > 16 && !long_k_few_rows && gemm_tc::supported(M, N, K, G, x_dtype, scale_dtype))
    return LCQ_ALGO_GEMM_TC;
  // A single activation row against a weight of at most 2 Mi weights (1 MiB packed) is pure latency:
  // the warp-per-row kernel has no ring to fill and no activations to stage, and measures
  // ~2 us per call in a chain of dependent launches against ~4 us for the TMA-staged kernel.
  const bool tiny_matvec = M == 1 && static_cast<long long>(N) * K <= (1LL << 21);
  if (wbits == 4 && !tiny_matvec && gemv_tc::supported(M < 16 ? M : 16, N, K, G, x_dtype, scale_dtype)) return LCQ_ALGO_GEMV_TC;
  // int8: the TMA-staged kernel has one CTA per 16 rows and no split along K; it pays off once that is
  // several CTAs per SM, below that the warp-per-row kernel (8 rows per CTA) is faster
  if (wbits == 8 && N >= 16384 && gemv_w8::supported(M, N, K, G)) return LCQ_ALGO_GEMV_W8;
  return LCQ_ALGO_SIMT;
}

static int matmul_entry(int wbits, const void* x, const void* w, const void* s, void* out, int M, int N, int K,
                        int G, int x_dtype, int scale_dtype, int out_dtype, int algo, void* workspace,
                        size_t workspace_bytes, void* stream) {
  int rc = check_problem(wbits, M, N, K, G);
  if (rc != LCQ_OK) return rc;
  if (!dtype_ok(x_dtype) || !dtype_ok(scale_dtype) || !dtype_ok(out_dtype)) {
    set_error("bad dtype code");
    return LCQ_ERR_BAD_ARG;
  }
  if (M == 0 || N == 0) return LCQ_OK;
  if (!x || !w || !s || !out) { set_error("null pointer argument"); return LCQ_ERR_BAD_ARG; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (algo == LCQ_ALGO_AUTO) algo = select_algo(wbits, M, N, K, G, x_dtype, scale_dtype, out_dtype);
  DevInfo di;
  rc = current_dev_info(di);
  if (rc != LCQ_OK) return rc;
  if (algo != LCQ_ALGO_SIMT && (di.major != 10)) {
    set_error("tensor-core kernels are built for sm_100a only; device is sm_%d%d", di.major, di.minor);
    return LCQ_ERR_UNSUPPORTED;
  }
  switch (algo) {
    case LCQ_ALGO_SIMT:
      return wbits == 4 ? simt_entry<4>(x, w, s, out, M, N, K, G, x_dtype, scale_dtype, out_dtype, st)
                        : simt_entry<8>(x, w, s, out, M, N, K, G, x_dtype, scale_dtype, out_dtype, st);
    case LCQ_ALGO_GEMV_TC: {
      if (wbits != 4 || !gemv_tc::supported(M < 16 ? M : 16, N, K, G, x_dtype, scale_dtype)) {
        set_error("GEMV_TC needs int4, group_size 32, K %% 64 == 0, f16 scales, f16/bf16 x");
        return LCQ_ERR_UNSUPPORTED;
      }
      // M > 16: rows of x in chunks of 16 (each chunk re-streams the weights).  Every chunk's plan
      // is checked against the workspace before the first launch, so a call either runs whole
      // or not at all.
      const size_t xe = 2, oe = out_dtype == LCQ_F32 ? 4 : 2;
      {
        const size_t need = gemv_tc_workspace_bytes(M, N, K, di.sm_count);
        if (workspace == nullptr || workspace_bytes < need) {
          set_error("w4a16 gemv: workspace of %zu bytes (256-byte aligned) required, got %zu", need, workspace_bytes);
          return LCQ_ERR_WORKSPACE;
        }
      }
      for (int m0 = 0; m0 < M; m0 += 16) {
        const int mc = M - m0 < 16 ? M - m0 : 16;
        rc = gemv_tc::launch(static_cast<const uint8_t*>(x) + static_cast<size_t>(m0) * K * xe, w, s,
                             static_cast<uint8_t*>(out) + static_cast<size_t>(m0) * N * oe, mc, N, K, x_dtype,
                             out_dtype, workspace, workspace_bytes, di.sm_count, st);
        if (rc != LCQ_OK) return rc;
      }
      return LCQ_OK;
    }
    case LCQ_ALGO_GEMV_W8:
      if (wbits != 8 || !gemv_w8::supported(M, N, K, G)) {
        set_error("GEMV_W8 needs int8 weights, M <= 8, K %% 16 == 0, group_size %% 16 == 0");
        return LCQ_ERR_UNSUPPORTED;
      }
      switch (x_dtype) {
        case LCQ_F32: return gemv_w8::launch<float>(x, w, s, out, M, N, K, G, scale_dtype, out_dtype, st);
        case LCQ_F16: return gemv_w8::launch<__half>(x, w, s, out, M, N, K, G, scale_dtype, out_dtype, st);
        default: return gemv_w8::launch<__nv_bfloat16>(x, w, s, out, M, N, K, G, scale_dtype, out_dtype, st);
      }
    case LCQ_ALGO_GEMM_TC:
      if (wbits != 4 || !gemm_tc::supported(M, N, K, G, x_dtype, scale_dtype)) {
        set_error("GEMM_TC needs int4, group_size 32, K %% 256 == 0, f16 scales, f16/bf16 x");
        return LCQ_ERR_UNSUPPORTED;
      }
      return gemm_tc::launch(x, w, s, out, M, N, K, x_dtype, out_dtype, workspace, workspace_bytes, di.sm_count, st);
    default:
      set_error("unknown algo %d", algo);
      return LCQ_ERR_BAD_ARG;
  }
}

}  // namespace lcq

// =================================================================== extern "C"
using namespace lcq;

extern "C" {

int lcq_version(void) { return 100; }

const char* lcq_status_string(int status) {
  switch (status) {
    case LCQ_OK: return "ok";
    case LCQ_ERR_BAD_ARG: return "bad argument";
    case LCQ_ERR_UNSUPPORTED: return "unsupported dtype/shape";
    case LCQ_ERR_CUDA: return "CUDA error";
    case LCQ_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case LCQ_ERR_TIMEOUT: return "device-side wait timed out";
    default: return "unknown status";
  }
}

const char* lcq_last_error(void) { return t_error; }

int lcq_device_info(int device, char* name, size_t name_len, int* sm_count, int* l2_bytes, int* cc_major,
                    int* cc_minor) {
  cudaDeviceProp prop;
  LCQ_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
  if (name && name_len) { strncpy(name, prop.name, name_len - 1); name[name_len - 1] = 0; }
  if (sm_count) *sm_count = prop.multiProcessorCount;
  if (l2_bytes) *l2_bytes = prop.l2CacheSize;
  if (cc_major) *cc_major = prop.major;
  if (cc_minor) *cc_minor = prop.minor;
  return LCQ_OK;
}

int lcq_dequant_int4(const void* w_packed, const void* scales, void* out, int64_t N, int64_t K, int group_size,
                     int scale_dtype, int out_dtype, void* stream) {
  return dequant_entry(4, w_packed, scales, out, N, K, group_size, scale_dtype, out_dtype, stream);
}

int lcq_dequant_int8(const void* w_int8, const void* scales, void* out, int64_t N, int64_t K, int group_size,
                     int scale_dtype, int out_dtype, void* stream) {
  return dequant_entry(8, w_int8, scales, out, N, K, group_size, scale_dtype, out_dtype, stream);
}

int lcq_matmul_int4(const void* x, const void* w_packed, const void* scales, void* out, int M, int N, int K,
                    int group_size, int x_dtype, int scale_dtype, int out_dtype, int algo, void* workspace,
                    size_t workspace_bytes, void* stream) {
  return matmul_entry(4, x, w_packed, scales, out, M, N, K, group_size, x_dtype, scale_dtype, out_dtype, algo,
                      workspace, workspace_bytes, stream);
}

int lcq_matmul_int8(const void* x, const void* w_int8, const void* scales, void* out, int M, int N, int K,
                    int group_size, int x_dtype, int scale_dtype, int out_dtype, int algo, void* workspace,
                    size_t workspace_bytes, void* stream) {
  return matmul_entry(8, x, w_int8, scales, out, M, N, K, group_size, x_dtype, scale_dtype, out_dtype, algo,
                      workspace, workspace_bytes, stream);
}

int lcq_matmul_select_algo(int wbits, int M, int N, int K, int group_size, int x_dtype, int scale_dtype,
                           int out_dtype) {
  int rc = check_problem(wbits, M, N, K, group_size);
  if (rc != LCQ_OK) return rc;
  return select_algo(wbits, M, N, K, group_size, x_dtype, scale_dtype, out_dtype);
}

size_t lcq_matmul_workspace_bytes(int wbits, int M, int N, int K, int group_size, int x_dtype, int scale_dtype,
                                  int out_dtype, int algo) {
  if (check_problem(wbits, M, N, K, group_size) != LCQ_OK) return static_cast<size_t>(-1);
  if (M == 0 || N == 0) return 0;
  if (algo == LCQ_ALGO_AUTO) algo = select_algo(wbits, M, N, K, group_size, x_dtype, scale_dtype, out_dtype);
  if (algo == LCQ_ALGO_SIMT) return 0;
  if (algo == LCQ_ALGO_GEMV_W8) return (wbits == 8 && gemv_w8::supported(M, N, K, group_size)) ? 0 : static_cast<size_t>(-1);
  int sm = 148;  // B200; refined from the device when one is present
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) sm = v;
  } else {
    (void)cudaGetLastError();
  }
  if (algo == LCQ_ALGO_GEMV_TC) {
    if (wbits != 4 || !gemv_tc::supported(M < 16 ? M : 16, N, K, group_size, x_dtype, scale_dtype))
      return static_cast<size_t>(-1);
    return gemv_tc_workspace_bytes(M, N, K, sm);
  }
  if (algo == LCQ_ALGO_GEMM_TC) {
    if (wbits != 4 || !gemm_tc::supported(M, N, K, group_size, x_dtype, scale_dtype)) return static_cast<size_t>(-1);
    return gemm_tc::workspace_bytes(M, N, K, x_dtype, sm);
  }
  return static_cast<size_t>(-1);
}

int lcq_gemv_tc_plan_check(int M, int N, int K, int sm_count, int* fields) {
  if (!gemv_tc::supported(M, N, K, 32, LCQ_F16, LCQ_F16) || sm_count < 1) {
    set_error("plan check: problem not covered by GEMV_TC");
    return LCQ_ERR_UNSUPPORTED;
  }
  const gemv_tc::Plan pl = gemv_tc::make_plan(M, N, K, sm_count);
  const gemv_tc::Params& p = pl.p;
  if (fields) {
    fields[0] = pl.grid; fields[1] = p.n_rb; fields[2] = p.n_kr; fields[3] = p.S; fields[4] = p.ctas_per_kr;
    fields[5] = p.max_split; fields[6] = static_cast<int>(pl.smem_bytes); fields[7] = pl.MT;
  }
  if (pl.smem_bytes > 227 * 1024) { set_error("plan check: %zu bytes of shared memory", pl.smem_bytes); return LCQ_ERR_UNSUPPORTED; }
  // Replay the device-side schedule on the host: every (row block, k tile) exactly once,
  // slots within bounds and unique, contributor counts consistent.
  std::vector<int> seen(static_cast<size_t>(p.n_rb) * p.nst, 0);
  std::vector<int> contrib(p.n_rb, 0);
  std::vector<int> slot_used(static_cast<size_t>(p.n_rb) * p.n_kr * p.max_split, 0);
  for (int b = 0; b < pl.grid; ++b) {
    const int kr = b % p.n_kr, j = b / p.n_kr;
    const gemv_tc::Sched s = gemv_tc::make_sched(p, kr);
    if (j >= s.G) continue;
    const long long t0 = gemv_tc::tile_begin(s, j), t1 = gemv_tc::tile_begin(s, j + 1);
    if (!pl.fits_32bit) { set_error("plan check: schedule does not fit 32 bits"); return LCQ_ERR_UNSUPPORTED; }
    if (t1 <= t0) { set_error("plan check: CTA %d has no tiles", b); return LCQ_ERR_BAD_ARG; }
    if (pl.cluster) {
      // cluster mode: the c CTAs of a cluster share one row block, nobody idles, a share fits the x slots
      if (s.G != pl.grid || pl.grid % p.cluster != 0 || t0 / s.S_kr != b / p.cluster || (t1 - 1) / s.S_kr != b / p.cluster ||
          t1 - t0 > p.x_tiles) {
        set_error("plan check: CTA %d breaks the cluster layout", b);
        return LCQ_ERR_BAD_ARG;
      }
    }
    int last_rb = -1;
    for (long long t = t0; t < t1; ++t) {
      const int rb = static_cast<int>(t / s.S_kr), ks = static_cast<int>(t % s.S_kr);
      const int kt = kr * p.S + ks;
      if (rb >= p.n_rb || kt >= p.nst) { set_error("plan check: tile out of range"); return LCQ_ERR_BAD_ARG; }
      seen[static_cast<size_t>(rb) * p.nst + kt]++;
      if (rb != last_rb) {
        int j0, j1;
        gemv_tc::cover(s, rb, j0, j1);
        if (j < j0 || j > j1) { set_error("plan check: CTA outside cover"); return LCQ_ERR_BAD_ARG; }
        const int slot = kr * p.max_split + (j - j0);
        if (j - j0 >= p.max_split) { set_error("plan check: slot %d >= max_split %d", j - j0, p.max_split); return LCQ_ERR_BAD_ARG; }
        if (slot_used[(static_cast<size_t>(rb) * p.n_kr * p.max_split) + slot]++) { set_error("plan check: slot reused"); return LCQ_ERR_BAD_ARG; }
        contrib[rb]++;
        last_rb = rb;
      }
    }
  }
  for (size_t i = 0; i < seen.size(); ++i)
    if (seen[i] != 1) { set_error("plan check: tile %zu covered %d times", i, seen[i]); return LCQ_ERR_BAD_ARG; }
  for (int rb = 0; rb < p.n_rb; ++rb)
    if (contrib[rb] != gemv_tc::contributors(p, rb)) {
      set_error("plan check: row block %d has %d contributors, kernel expects %d", rb, contrib[rb], gemv_tc::contributors(p, rb));
      return LCQ_ERR_BAD_ARG;
    }
  return LCQ_OK;
}

int lcq_gemv_tc_plan_cluster(int M, int N, int K, int sm_count) {
  if (!gemv_tc::supported(M, N, K, 32, LCQ_F16, LCQ_F16) || sm_count < 1) {
    set_error("plan: problem not covered by GEMV_TC");
    return LCQ_ERR_UNSUPPORTED;
  }
  return gemv_tc::make_plan(M, N, K, sm_count).p.cluster;
}

// ---------------------------------------------------------------- allocation-free decode entry
// Scratch for lcq_matmul_int4_noalloc: lives in the library image, so every GPU that loads the
// library holds these bytes until the process exits.  Zero at load time.
#define LCQ_NOALLOC_SCRATCH_BYTES (8u * 1024u * 1024u)
static __device__ __align__(256) unsigned char g_noalloc_scratch[LCQ_NOALLOC_SCRATCH_BYTES];
static void* g_noalloc_ptr[64];          // device address of the array, per device
static std::mutex g_noalloc_mu;

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address; the
// address a kernel can use has to be asked for, once per device, with that device current.
static int noalloc_scratch_address(void** out) {
  int dev = 0;
  LCQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) { set_error("device index %d out of range", dev); return LCQ_ERR_BAD_ARG; }
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    LCQ_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    if (ptr == nullptr) { set_error("cudaGetSymbolAddress returned a null address"); return LCQ_ERR_CUDA; }
    g_noalloc_ptr[dev] = ptr;
  }
  *out = g_noalloc_ptr[dev];
  return LCQ_OK;
}

int lcq_matmul_int4_noalloc(const void* x, const void* w_packed, const void* scales, void* out, int M, int N, int K,
                            int group_size, int x_dtype, int scale_dtype, int out_dtype, void* stream) {
  int rc = check_problem(4, M, N, K, group_size);
  if (rc != LCQ_OK) return rc;
  if (!dtype_ok(x_dtype) || !dtype_ok(scale_dtype) || !dtype_ok(out_dtype)) { set_error("bad dtype code"); return LCQ_ERR_BAD_ARG; }
  if (M == 0 || N == 0) return LCQ_OK;
  if (!x || !w_packed || !scales || !out) { set_error("null pointer argument"); return LCQ_ERR_BAD_ARG; }
  if (!gemv_tc::supported(M, N, K, group_size, x_dtype, scale_dtype)) {
    set_error("lcq_matmul_int4_noalloc covers M <= 16, group_size 32, K %% 64 == 0, f16 scales, f16/bf16 x");
    return LCQ_ERR_UNSUPPORTED;
  }
  DevInfo di;
  rc = current_dev_info(di);
  if (rc != LCQ_OK) return rc;
  if (di.major != 10) { set_error("built for sm_100a only; device is sm_%d%d", di.major, di.minor); return LCQ_ERR_UNSUPPORTED; }
  const gemv_tc::Plan pl = gemv_tc::make_plan(M, N, K, di.sm_count);
  if (pl.workspace_bytes > LCQ_NOALLOC_SCRATCH_BYTES) {
    set_error("problem M=%d N=%d K=%d needs %zu bytes of scratch; the built-in scratch holds %u bytes -- "
              "use lcq_matmul_int4 with a caller-provided workspace", M, N, K, pl.workspace_bytes,
              LCQ_NOALLOC_SCRATCH_BYTES);
    return LCQ_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  rc = noalloc_scratch_address(&scratch);
  if (rc != LCQ_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the array keeps whatever the previous call (possibly an aborted one) left: the counters must start at zero
  LCQ_CUDA_TRY(cudaMemsetAsync(scratch, 0, kWorkspaceCounterBytes, st));
  // no programmatic overlap here: the kernel must not start before the memset above has finished
  return gemv_tc::launch(x, w_packed, scales, out, M, N, K, x_dtype, out_dtype, scratch, LCQ_NOALLOC_SCRATCH_BYTES,
                         di.sm_count, st, /*allow_pdl=*/false);
}

size_t lcq_noalloc_scratch_bytes(void) { return LCQ_NOALLOC_SCRATCH_BYTES; }

// ---------------------------------------------------------------- NVLink peer all-gather
int lcq_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
  if (!ptr || !handle64 || bytes == 0) { set_error("lcq_peer_alloc: bad argument"); return LCQ_ERR_BAD_ARG; }
  void* p = nullptr;
  LCQ_CUDA_TRY(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { cudaFree(p); return cuda_fail(e, "lcq_peer_alloc"); }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  *ptr = p;
  return LCQ_OK;
}

int lcq_peer_open(const unsigned char* handle64, void** ptr) {
  if (!ptr || !handle64) { set_error("lcq_peer_open: bad argument"); return LCQ_ERR_BAD_ARG; }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  LCQ_CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return LCQ_OK;
}

int lcq_peer_close(void* ptr) {
  LCQ_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return LCQ_OK;
}

int lcq_peer_free(void* ptr) {
  LCQ_CUDA_TRY(cudaFree(ptr));
  return LCQ_OK;
}

int lcq_allgather_push(const void* src, size_t bytes_per_rank, void* const* regions, int rank, int world,
                       void* state, void* stream) {
  if (!src || !regions || !state || world < 1 || world > peer::MAX_RANKS || rank < 0 || rank >= world) {
    set_error("lcq_allgather_push: bad argument (world must be 1..%d)", peer::MAX_RANKS);
    return LCQ_ERR_BAD_ARG;
  }
  if (bytes_per_rank == 0 || bytes_per_rank % 16 != 0 || !aligned(src, 16)) {
    set_error("lcq_allgather_push: slices must be 16-byte aligned multiples of 16 bytes");
    return LCQ_ERR_BAD_ARG;
  }
  peer::PushArgs a;
  memset(&a, 0, sizeof(a));
  for (int g = 0; g < world; ++g) {
    if (!regions[g]) { set_error("lcq_allgather_push: region %d is null", g); return LCQ_ERR_BAD_ARG; }
    a.flags[g] = static_cast<int*>(regions[g]);
    a.data[g] = reinterpret_cast<uint4*>(static_cast<uint8_t*>(regions[g]) + peer::FLAG_BYTES);
  }
  a.src = static_cast<const uint4*>(src);
  a.n16 = static_cast<long long>(bytes_per_rank / 16);
  a.rank = rank;
  a.world = world;
  a.state = static_cast<int*>(state);
  return peer::launch_push(a, static_cast<cudaStream_t>(stream));
}

size_t lcq_peer_region_bytes(size_t bytes_per_rank, int world) {
  return peer::FLAG_BYTES + 5 * bytes_per_rank * static_cast<size_t>(world);   // data + two staging buffers of twice the size
}

// ---------------------------------------------------------------- decode-step glue, embedding, argmax
#define LCQ_BY_DTYPE(dtype, CALL)                                   \
  switch (dtype) {                                                  \
    case LCQ_F32: { typedef float T; return CALL; }                 \
    case LCQ_F16: { typedef __half T; return CALL; }                \
    case LCQ_BF16: { typedef __nv_bfloat16 T; return CALL; }        \
    default: set_error("bad dtype code %d", dtype); return LCQ_ERR_BAD_ARG; \
  }

int lcq_rms_norm(const void* x, const void* weight, void* out, int64_t rows, int n, float eps, int dtype, void* stream) {
  if (rows < 0 || n < 0) { set_error("rms_norm: negative size"); return LCQ_ERR_BAD_ARG; }
  if (rows == 0 || n == 0) return LCQ_OK;
  if (!x || !weight || !out) { set_error("null pointer argument"); return LCQ_ERR_BAD_ARG; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LCQ_BY_DTYPE(dtype, (glue::launch_rms_norm<T>(x, nullptr, weight, out, rows, n, eps, st)))
}

int lcq_residual_rms_norm(void* hidden, const void* delta, const void* weight, void* out, int64_t rows, int n, float eps,
                          int dtype, void* stream) {
  if (rows < 0 || n < 0) { set_error("residual_rms_norm: negative size"); return LCQ_ERR_BAD_ARG; }
  if (rows == 0 || n == 0) return LCQ_OK;
  if (!hidden || !delta || !weight || !out) { set_error("null pointer argument"); return LCQ_ERR_BAD_ARG; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LCQ_BY_DTYPE(dtype, (glue::launch_rms_norm<T>(delta, hidden, weight, out, rows, n, eps, st)))
}

int lcq_silu_mul(const void* gate, const void* up, void* out, int64_t n, int dtype, void* stream) {
  if (n < 0) { set_error("silu_mul: negative size"); return LCQ_ERR_BAD_ARG; }
  if (n == 0) return LCQ_OK;
  if (!gate || !up || !out) { set_error("null pointer argument"); return LCQ_ERR_BAD_ARG; }
  DevInfo di;
  int rc = current_dev_info(di);
  if (rc != LCQ_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LCQ_BY_DTYPE(dtype, (glue::launch_elementwise<T, 0>(gate, up, out, n, di.sm_count, st)))
}

int lcq_add_inplace(void* a, const void* b, int64_t n, int dtype, void* stream) {
  if (n < 0) { set_error("add_inplace: negative size"); return LCQ_ERR_BAD_ARG; }
  if (n == 0) return LCQ_OK;
  if (!a || !b) { set_error("null pointer argument"); return LCQ_ERR_BAD_ARG; }
  DevInfo di;
  int rc = current_dev_info(di);
  if (rc != LCQ_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LCQ_BY_DTYPE(dtype, (glue::launch_elementwise<T, 1>(a, b, a, n, di.sm_count, st)))
}

int lcq_embed_lookup(const void* token_ids, const void* table, void* out, int64_t tokens, int vocab, int dim, int dtype,
                     void* stream) {
  if (tokens < 0 || vocab <= 0 || dim < 0 || !dtype_ok(dtype)) { set_error("embed_lookup: bad size or dtype"); return LCQ_ERR_BAD_ARG; }
  if (tokens == 0 || dim == 0) return LCQ_OK;
  if (!token_ids || !table || !out) { set_error("null pointer argument"); return LCQ_ERR_BAD_ARG; }
  const long long row_bytes = static_cast<long long>(dim) * (dtype == LCQ_F32 ? 4 : 2);
  return glue::launch_embed(token_ids, table, out, tokens, vocab, row_bytes, static_cast<cudaStream_t>(stream));
}

int lcq_argmax(const void* x, void* out, int64_t rows, int n, int dtype, void* stream) {
  if (rows < 0) { set_error("argmax: negative size"); return LCQ_ERR_BAD_ARG; }
  if (rows == 0) return LCQ_OK;
  if (!x || !out) { set_error("null pointer argument"); return LCQ_ERR_BAD_ARG; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LCQ_BY_DTYPE(dtype, (glue::launch_argmax<T>(x, out, rows, n, st)))
}

// ---------------------------------------------------------------- quantisers
static int quantize_entry(int wbits, const void* w, void* q, void* scales, int64_t N, int64_t K, int G, int w_dtype,
                          int style, void* stream) {
  int rc = check_problem(wbits, 1, N, K, G);
  if (rc != LCQ_OK) return rc;
  if (wbits == 4 && (G % 2) != 0) { set_error("int4 quantiser needs an even group_size, got %d", G); return LCQ_ERR_BAD_ARG; }
  if (style != 0 && style != 1) { set_error("quantiser style must be 0 or 1, got %d", style); return LCQ_ERR_BAD_ARG; }
  if (N == 0) return LCQ_OK;
  if (!w || !q || !scales) { set_error("null pointer argument"); return LCQ_ERR_BAD_ARG; }
  DevInfo di;
  rc = current_dev_info(di);
  if (rc != LCQ_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (wbits == 4) { LCQ_BY_DTYPE(w_dtype, (quant::launch_quantize<T, 4>(w, q, scales, N, K, G, style, di.sm_count, st))) }
  LCQ_BY_DTYPE(w_dtype, (quant::launch_quantize<T, 8>(w, q, scales, N, K, G, style, di.sm_count, st)))
}

int lcq_quantize_int4(const void* w, void* w_packed, void* scales, int64_t N, int64_t K, int group_size, int w_dtype,
                      int style, void* stream) {
  return quantize_entry(4, w, w_packed, scales, N, K, group_size, w_dtype, style, stream);
}

int lcq_quantize_int8(const void* w, void* w_int8, void* scales, int64_t N, int64_t K, int group_size, int w_dtype,
                      int style, void* stream) {
  return quantize_entry(8, w, w_int8, scales, N, K, group_size, w_dtype, style, stream);
}

int lcq_set_wait_limit_ns(unsigned long long limit_ns) {
  if (limit_ns == 0) { set_error("lcq_set_wait_limit_ns: the limit must be positive"); return LCQ_ERR_BAD_ARG; }
  LCQ_CUDA_TRY(cudaMemcpyToSymbol(g_wait_limit_ns, &limit_ns, sizeof(limit_ns)));
  return LCQ_OK;
}

// ---------------------------------------------------------------- sharding context (one per rank)
struct lcq_shard_ctx {
  int rank, world, device;
  size_t max_slice_bytes;
  void* mine[2];                         // this rank's two regions (used alternately)
  void* regions[2][peer::MAX_RANKS];     // every rank's regions as mapped here
  int* state;                            // 2 x 2 ints
  void* y_local;                         // this rank's [M, N/world] before the gather
  void* workspace;
  size_t workspace_bytes;
  unsigned next;                         // which region the next call uses
  bool connected;
};

int lcq_shard_ctx_create(int rank, int world, size_t max_slice_bytes, lcq_shard_ctx** out, unsigned char* handles128) {
  if (!out || !handles128 || world < 1 || world > peer::MAX_RANKS || rank < 0 || rank >= world || max_slice_bytes == 0) {
    set_error("lcq_shard_ctx_create: bad argument (world must be 1..%d)", peer::MAX_RANKS);
    return LCQ_ERR_BAD_ARG;
  }
  max_slice_bytes = (max_slice_bytes + 15) & ~static_cast<size_t>(15);
  lcq_shard_ctx* c = new lcq_shard_ctx();
  memset(c, 0, sizeof(*c));
  c->rank = rank; c->world = world; c->max_slice_bytes = max_slice_bytes;
  LCQ_CUDA_TRY(cudaGetDevice(&c->device));
  const size_t region_bytes = lcq_peer_region_bytes(max_slice_bytes, world);
  for (int i = 0; i < 2; ++i) {
    int rc = lcq_peer_alloc(region_bytes, &c->mine[i], handles128 + 64 * i);
    if (rc != LCQ_OK) { lcq_shard_ctx_destroy(c); return rc; }
    c->regions[i][rank] = c->mine[i];
  }
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&c->state), 4 * sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(c->state, 0, 4 * sizeof(int));
  if (e == cudaSuccess) e = cudaMalloc(&c->y_local, max_slice_bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { lcq_shard_ctx_destroy(c); return cuda_fail(e, "lcq_shard_ctx_create"); }
  c->connected = world == 1;
  *out = c;
  return LCQ_OK;
}

int lcq_shard_ctx_connect(lcq_shard_ctx* c, const unsigned char* all_handles) {
  if (!c || !all_handles) { set_error("lcq_shard_ctx_connect: bad argument"); return LCQ_ERR_BAD_ARG; }
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    for (int i = 0; i < 2; ++i) {
      int rc = lcq_peer_open(all_handles + (static_cast<size_t>(r) * 2 + i) * 64, &c->regions[i][r]);
      if (rc != LCQ_OK) return rc;
    }
  }
  c->connected = true;
  return LCQ_OK;
}

int lcq_sharded_matmul_int4(lcq_shard_ctx* c, const void* x, const void* w_local, const void* scales_local, void** gathered,
                            int M, int N_total, int K, int group_size, int x_dtype, int scale_dtype, int out_dtype,
                            int algo, void* stream) {
  if (!c || !gathered) { set_error("lcq_sharded_matmul_int4: bad argument"); return LCQ_ERR_BAD_ARG; }
  if (!c->connected) { set_error("lcq_sharded_matmul_int4: call lcq_shard_ctx_connect first"); return LCQ_ERR_BAD_ARG; }
  if (N_total <= 0 || N_total % c->world != 0 || M <= 0) {
    set_error("lcq_sharded_matmul_int4: N_total=%d must be a positive multiple of the %d ranks", N_total, c->world);
    return LCQ_ERR_BAD_ARG;
  }
  const int n_local = N_total / c->world;
  const size_t slice = static_cast<size_t>(M) * n_local * (out_dtype == LCQ_F32 ? 4 : 2);
  if (slice > c->max_slice_bytes || slice % 16 != 0) {
    set_error("lcq_sharded_matmul_int4: slice of %zu bytes (limit %zu, must be a multiple of 16)", slice, c->max_slice_bytes);
    return LCQ_ERR_BAD_ARG;
  }
  const size_t need = lcq_matmul_workspace_bytes(4, M, n_local, K, group_size, x_dtype, scale_dtype, out_dtype, algo);
  if (need == static_cast<size_t>(-1)) { set_error("lcq_sharded_matmul_int4: no kernel covers this problem"); return LCQ_ERR_UNSUPPORTED; }
  if (need > c->workspace_bytes) {       // first call of this size only: allocates and synchronises the device
    LCQ_CUDA_TRY(cudaDeviceSynchronize());
    if (c->workspace) LCQ_CUDA_TRY(cudaFree(c->workspace));
    c->workspace = nullptr; c->workspace_bytes = 0;
    LCQ_CUDA_TRY(cudaMalloc(&c->workspace, need));
    LCQ_CUDA_TRY(cudaMemset(c->workspace, 0, need));
    LCQ_CUDA_TRY(cudaDeviceSynchronize());
    c->workspace_bytes = need;
  }
  const unsigned i = c->next & 1u;
  uint8_t* data = static_cast<uint8_t*>(c->mine[i]) + peer::FLAG_BYTES;
  void* y = c->world == 1 ? static_cast<void*>(data) : c->y_local;
  int rc = lcq_matmul_int4(x, w_local, scales_local, y, M, n_local, K, group_size, x_dtype, scale_dtype, out_dtype, algo,
                           c->workspace, c->workspace_bytes, stream);
  if (rc != LCQ_OK) return rc;
  if (c->world > 1) {
    rc = lcq_allgather_push(y, slice, c->regions[i], c->rank, c->world, c->state + 2 * i, stream);
    if (rc != LCQ_OK) return rc;
  }
  c->next++;
  *gathered = data;
  return LCQ_OK;
}

int lcq_shard_ctx_destroy(lcq_shard_ctx* c) {
  if (!c) return LCQ_OK;
  cudaDeviceSynchronize();
  for (int i = 0; i < 2; ++i) {
    for (int r = 0; r < c->world; ++r)
      if (r != c->rank && c->regions[i][r]) cudaIpcCloseMemHandle(c->regions[i][r]);
    if (c->mine[i]) cudaFree(c->mine[i]);
  }
  if (c->state) cudaFree(c->state);
  if (c->y_local) cudaFree(c->y_local);
  if (c->workspace) cudaFree(c->workspace);
  (void)cudaGetLastError();
  delete c;
  return LCQ_OK;
}

int lcq_check_device_status(void* stream) {
  LCQ_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  int v = 0;
  LCQ_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    LCQ_CUDA_TRY(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
    if (v == 40) set_error("a kernel reported a failure (code 40): embed_lookup met a token id outside the table");
    else set_error("a kernel gave up a bounded wait (code %d)", v);
    return LCQ_ERR_TIMEOUT;
  }
  return LCQ_OK;
}

}  // extern "C"
