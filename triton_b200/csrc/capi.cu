// C ABI of the library (include/triton_b200.h): argument validation, per-device context,
// error strings, TMA tensor-map encoding.  The kernels live in gemm.cu / attn_fwd.cu / attn_bwd.cu.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "host.h"

namespace tb {

// Status word read by b200_status(); kernels receive its device address as a parameter.
// Word 0: the status; words 2-3: device-visible address of this device's word in the pinned host
// mirror below (0 when the page could not be registered).
#ifdef B200_TRACE
__device__ __align__(16) unsigned g_status_word[4 + 2 * tb::kTraceRegions * tb::kTraceEvents];  // + trace buffer
#else
__device__ __align__(16) unsigned g_status_word[4];
#endif
// Work counters of the persistent attention kernels.  A counter is zero between launches: the CTA
// that takes the last ticket of a launch puts the zero back, so no reset precedes a launch.
// Eager launches take the next word of a ring, so launches in flight on different streams do not
// share one (more than kSchedRing attention launches in flight at once on one device would).
// Launches captured into a CUDA graph keep their counter for as long as the graph may be
// replayed, so they take words of a pool that is never recycled: a replay can then never meet
// an eager launch, or another graph, on its counter.
constexpr unsigned kSchedRing = 256, kSchedGraphPool = 4096;
__device__ int g_sched_ring[kSchedRing + kSchedGraphPool];

namespace {
thread_local char g_err[512] = "";
thread_local int g_err_code = B200_OK;  // code of the last fail() on this thread
std::mutex g_mu;
DeviceCtx g_ctx[64];
// One word per device (64 bytes apart) in a page of the library's own static memory, pinned and
// mapped on first use (cudaHostRegister: nothing is allocated).  A kernel whose bounded wait runs
// out stores its failure code here as well as in the device status word.
alignas(4096) unsigned g_host_status[1024];
bool g_host_status_registered = false, g_host_status_tried = false;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  g_err_code = code;
  return code;
}

DeviceCtx* current_ctx() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    fail(B200_ERR_DEVICE, "no CUDA device current: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return nullptr;
  }
  // Bind the device's primary context to THIS thread: the driver entry point used for tensor maps
  // needs a current context, and a thread that has made no runtime call yet (an autograd worker
  // calling the backward, say) does not have one.
  e = cudaSetDevice(dev);
  if (e != cudaSuccess) {
    fail(B200_ERR_CUDA, "cudaSetDevice(%d): %s", dev, cudaGetErrorString(e));
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceCtx& c = g_ctx[dev];
  if (c.device == dev) return &c;
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, dev);
  if (e != cudaSuccess) {
    fail(B200_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    return nullptr;
  }
  if (prop.major != 10) {
    fail(B200_ERR_DEVICE, "device %d is sm_%d%d; this library contains sm_100a code only", dev, prop.major,
         prop.minor);
    return nullptr;
  }
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
      fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled not available from the driver");
      return nullptr;
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  void* st = nullptr;
  e = cudaGetSymbolAddress(&st, g_status_word);
  if (e != cudaSuccess) {
    fail(B200_ERR_CUDA, "cudaGetSymbolAddress(status): %s", cudaGetErrorString(e));
    return nullptr;
  }
  c.status = static_cast<unsigned*>(st);
  // host mirror of the status word (optional: without it a failure is still seen by b200_status)
  c.host_status = nullptr;
  if (!g_host_status_tried) {
    g_host_status_tried = true;
    g_host_status_registered =
        cudaHostRegister(g_host_status, sizeof(g_host_status), cudaHostRegisterPortable | cudaHostRegisterMapped) == cudaSuccess;
    if (!g_host_status_registered) cudaGetLastError();
  }
  if (g_host_status_registered) {
    void* dptr = nullptr;
    unsigned* hword = &g_host_status[dev * 16];
    if (cudaHostGetDevicePointer(&dptr, hword, 0) == cudaSuccess && dptr) {
      *hword = 0;
      unsigned long long addr = reinterpret_cast<unsigned long long>(dptr);
      if (cudaMemcpy(c.status + 2, &addr, sizeof(addr), cudaMemcpyHostToDevice) == cudaSuccess) c.host_status = hword;
    }
    if (!c.host_status) cudaGetLastError();
  }
  c.sm_count = prop.multiProcessorCount;
  c.max_smem_optin = (int)prop.sharedMemPerBlockOptin;
  c.device = dev;
  return &c;
}

DeviceCtx* ready_ctx() {
  DeviceCtx* ctx = current_ctx();
  if (!ctx) return nullptr;
  if (ctx->host_status) {
    const unsigned v = *reinterpret_cast<volatile unsigned*>(ctx->host_status);
    if (v != 0) {
      fail(B200_ERR_KERNEL,
           "an earlier kernel on device %d gave up a bounded wait (status 0x%08x: site %u, block %u); results "
           "since then are invalid and nothing more is launched until b200_status(&v, 1) clears it",
           ctx->device, v, v & 0xFFu, v >> 16);
      return nullptr;
    }
  }
  return ctx;
}

int* next_sched_counter(DeviceCtx* ctx, cudaStream_t stream) {
  static int* base[64] = {};
  static unsigned next_eager[64] = {}, next_graph[64] = {};
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  cudaError_t e = cudaStreamIsCapturing(stream, &cap);
  if (e != cudaSuccess) {
    fail(B200_ERR_CUDA, "cudaStreamIsCapturing: %s", cudaGetErrorString(e));
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  if (!base[ctx->device]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_sched_ring);
    if (e != cudaSuccess) {
      fail(B200_ERR_CUDA, "cudaGetSymbolAddress(scheduler ring): %s", cudaGetErrorString(e));
      return nullptr;
    }
    base[ctx->device] = static_cast<int*>(ptr);
  }
  if (cap == cudaStreamCaptureStatusNone) return base[ctx->device] + (next_eager[ctx->device]++ % kSchedRing);
  if (next_graph[ctx->device] >= kSchedGraphPool) {
    fail(B200_ERR_UNSUPPORTED,
         "this process has captured %u attention launches into CUDA graphs on device %d; each keeps its work "
         "counter for the life of the process and the pool holds no more",
         kSchedGraphPool, ctx->device);
    return nullptr;
  }
  return base[ctx->device] + kSchedRing + next_graph[ctx->device]++;
}

bool encode_tmap(CUtensorMap* out, int dtype, int rank, const void* base, const uint64_t* dims,
                 const uint64_t* strides_bytes, const uint32_t* box, int swizzle) {
  CUtensorMapDataType dt;
  switch (dtype) {
    case B200_F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
    case B200_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
    case B200_E4M3:
    case B200_E5M2: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    case B200_F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
    default: fail(B200_ERR_ARG, "bad dtype %d", dtype); return false;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) {
    fail(B200_ERR_UNSUPPORTED, "tensor base address %p is not 16-byte aligned", base);
    return false;
  }
  cuuint64_t d[5], s[4];
  cuuint32_t b[5], es[5];
  const int eb = dtype_bytes(dtype);
  uint64_t extent = dims[0] * eb;
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    es[i] = 1;
    if (i > 0) {
      uint64_t st = strides_bytes[i - 1];
      if (dims[i] == 1) st = (extent + 15) & ~15ull;  // stride of a size-1 dimension is never used
      if (st % 16 != 0) {
        fail(B200_ERR_UNSUPPORTED, "stride of dimension %d (%llu bytes) is not a multiple of 16 bytes", i,
             (unsigned long long)st);
        return false;
      }
      s[i - 1] = st;
      extent = st * dims[i];
    }
    if (dims[i] == 0) {
      fail(B200_ERR_ARG, "empty tensor dimension");
      return false;
    }
  }
  CUresult r = g_encode(out, dt, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_128B : (swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE),
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fail(B200_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu x %llu)", (int)r,
         rank, (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 1));
    return false;
  }
  return true;
}

// b200_selftest_wait_timeout: the give-up path of the kernels' bounded waits, on a barrier that
// nothing ever arrives on.  Same shape as the real kernels: TMEM is allocated, one thread waits
// (with the limit passed in instead of the kernels' 250 ms), the failure is recorded, the CTA
// tears down in the usual order and frees its TMEM.  It faults nothing and returns by itself.
__global__ void __launch_bounds__(64, 1) wait_timeout_selftest_kernel(unsigned* status, unsigned long long limit_ns) {
  __shared__ uint64_t never;  // an mbarrier with one expected arrival that never comes
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&never, 1);
    fence_barrier_init();
    cta_wait_flag_clear();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_slot, 32);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_slot);
  if (warp == 1 && lane == 0) {
    if (!mbar_try_wait(&never, 0)) mbar_wait_slow(&never, 0, status, SITE_SELFTEST, limit_ns);
  }
  __syncwarp();
  cta_linger_after_failure();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 32);
  }
}

}  // namespace tb

using namespace tb;

extern "C" {

int b200_version(void) { return 100; }

const char* b200_last_error(void) { return g_err; }

#ifdef B200_TRACE
// trace builds only: copies the (tag, clock) pairs of all regions to `dst` and clears them
extern "C" B200_API int b200_trace_read(void* dst, size_t bytes) {
  const size_t all = sizeof(unsigned) * 2 * tb::kTraceRegions * tb::kTraceEvents;
  if (!dst || bytes < all) return fail(B200_ERR_ARG, "trace buffer too small");
  if (!current_ctx()) return B200_ERR_DEVICE;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(dst, g_status_word, all, sizeof(unsigned) * tb::kTraceOffset);
  if (e == cudaSuccess) {
    void* sym = nullptr;
    e = cudaGetSymbolAddress(&sym, g_status_word);
    if (e == cudaSuccess) e = cudaMemset(static_cast<unsigned*>(sym) + tb::kTraceOffset, 0, all);
  }
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "trace read: %s", cudaGetErrorString(e));
  return B200_OK;
}
#endif

int b200_status(unsigned* value, int clear) {
  DeviceCtx* ctx = current_ctx();
  if (!ctx) return g_err_code;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
  unsigned v = 0;
  e = cudaMemcpy(&v, ctx->status, sizeof(v), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "status read: %s", cudaGetErrorString(e));
  if (value) *value = v;
  if (clear && v != 0) {
    e = cudaMemset(ctx->status, 0, sizeof(unsigned));
    if (e != cudaSuccess) return fail(B200_ERR_CUDA, "status clear: %s", cudaGetErrorString(e));
    if (ctx->host_status) *reinterpret_cast<volatile unsigned*>(ctx->host_status) = 0;
    // a kernel that gave up may have left its work counter non-zero
    void* ring = nullptr;
    e = cudaGetSymbolAddress(&ring, g_sched_ring);
    if (e == cudaSuccess) e = cudaMemset(ring, 0, sizeof(int) * (kSchedRing + kSchedGraphPool));
    if (e != cudaSuccess) return fail(B200_ERR_CUDA, "work counter clear: %s", cudaGetErrorString(e));
  }
  return B200_OK;
}

int b200_selftest_wait_timeout(b200_stream_t stream, unsigned limit_us) {
  if (limit_us == 0 || limit_us > 250000u) return fail(B200_ERR_ARG, "limit_us must be in [1, 250000]");
  DeviceCtx* ctx = ready_ctx();
  if (!ctx) return g_err_code;
  wait_timeout_selftest_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(ctx->status, 1000ull * limit_us);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "self-test launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

int b200_matmul(b200_stream_t stream, const void* a, const void* b, void* c, int M, int N, int K, int64_t stride_am,
                int64_t stride_ak, int64_t stride_bk, int64_t stride_bn, int64_t stride_cm, int64_t stride_cn,
                int in_dtype, int out_dtype, int activation, const float* scale_a, const float* scale_b) {
  return b200_matmul_splitk(stream, a, b, c, M, N, K, stride_am, stride_ak, stride_bk, stride_bn, stride_cm, stride_cn,
                            in_dtype, out_dtype, activation, scale_a, scale_b, 1, nullptr);
}

int b200_matmul_plan(int M, int N, int K, int in_dtype, int* splits, size_t* workspace_bytes) {
  if (M < 0 || N < 0 || K < 0 || !splits || !workspace_bytes) return fail(B200_ERR_ARG, "bad argument");
  if (in_dtype != B200_F16 && in_dtype != B200_BF16 && in_dtype != B200_E4M3)
    return fail(B200_ERR_ARG, "in_dtype must be F16, BF16 or E4M3");
  DeviceCtx* ctx = current_ctx();
  if (!ctx) return g_err_code;
  *splits = (M == 0 || N == 0 || K == 0) ? 1 : gemm_plan_splits(ctx, M, N, K, in_dtype);
  *workspace_bytes = *splits > 1 ? (size_t)*splits * M * N * sizeof(float) : 0;
  return B200_OK;
}

int b200_matmul_splitk(b200_stream_t stream, const void* a, const void* b, void* c, int M, int N, int K,
                       int64_t stride_am, int64_t stride_ak, int64_t stride_bk, int64_t stride_bn, int64_t stride_cm,
                       int64_t stride_cn, int in_dtype, int out_dtype, int activation, const float* scale_a,
                       const float* scale_b, int splits, float* workspace) {
  return b200_matmul_bias(stream, a, b, c, M, N, K, stride_am, stride_ak, stride_bk, stride_bn, stride_cm, stride_cn,
                          in_dtype, out_dtype, activation, scale_a, scale_b, nullptr, B200_BIAS_NONE, 0, 0, splits,
                          workspace);
}

int b200_matmul_chain(b200_stream_t stream, const void* a, const void* b, const void* w, void* c, int M, int N, int K,
                      int N2, int64_t stride_am, int64_t stride_ak, int64_t stride_bk, int64_t stride_bn,
                      int64_t stride_wk, int64_t stride_wn, int64_t stride_cm, int64_t stride_cn, int in_dtype,
                      int out_dtype) {
  if (M < 0 || N < 0 || K < 0 || N2 < 0) return fail(B200_ERR_ARG, "negative dimension");
  if (in_dtype != B200_F16 && in_dtype != B200_BF16) return fail(B200_ERR_ARG, "chain-dot: in_dtype must be F16 or BF16");
  if (out_dtype != B200_F16 && out_dtype != B200_BF16 && out_dtype != B200_F32)
    return fail(B200_ERR_ARG, "chain-dot: out_dtype must be F16, BF16 or F32");
  if (N > 128 || N2 > 128)
    return fail(B200_ERR_UNSUPPORTED, "chain-dot keeps a whole row of A B in one tile: N and N2 must be at most 128");
  DeviceCtx* ctx = ready_ctx();
  if (!ctx) return g_err_code;
  if (M == 0 || N2 == 0) return B200_OK;
  if (!c || (N > 0 && !w) || (N > 0 && K > 0 && (!a || !b))) return fail(B200_ERR_ARG, "null pointer");
  if (stride_cn != 1 && N2 != 1) return fail(B200_ERR_UNSUPPORTED, "C must have stride_cn == 1");
  if (K == 0 || N == 0) {  // an empty sum in either product: zeros
    const int es = dtype_bytes(out_dtype);
    cudaError_t e = cudaMemset2DAsync(c, (size_t)stride_cm * es, 0, (size_t)N2 * es, (size_t)M,
                                      reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(B200_ERR_CUDA, "memset: %s", cudaGetErrorString(e));
    return B200_OK;
  }
  return launch_gemm_chain(ctx, reinterpret_cast<cudaStream_t>(stream), a, b, w, c, M, N, K, N2, stride_am, stride_ak,
                           stride_bk, stride_bn, stride_wk, stride_wn, stride_cm, in_dtype, out_dtype);
}

int b200_matmul_bias(b200_stream_t stream, const void* a, const void* b, void* c, int M, int N, int K,
                     int64_t stride_am, int64_t stride_ak, int64_t stride_bk, int64_t stride_bn, int64_t stride_cm,
                     int64_t stride_cn, int in_dtype, int out_dtype, int activation, const float* scale_a,
                     const float* scale_b, const void* bias, int bias_mode, int64_t bias_stride_m,
                     int64_t bias_stride_n, int splits, float* workspace) {
  if (bias_mode < B200_BIAS_NONE || bias_mode > B200_BIAS_COLS) return fail(B200_ERR_ARG, "bad bias mode");
  if (bias_mode != B200_BIAS_NONE && !bias) return fail(B200_ERR_ARG, "null bias pointer");
  if (bias_mode != B200_BIAS_NONE && out_dtype == B200_E4M3)
    return fail(B200_ERR_ARG, "no bias epilogue with an e4m3 output");
  if (splits < 1 || splits > 64) return fail(B200_ERR_ARG, "splits must be in [1, 64]");
  if (splits > 1 && (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15)))
    return fail(B200_ERR_ARG, "split-K needs a 16-byte aligned workspace of splits * M * N floats");
  if (M < 0 || N < 0 || K < 0) return fail(B200_ERR_ARG, "negative dimension");
  if (in_dtype != B200_F16 && in_dtype != B200_BF16 && in_dtype != B200_E4M3)
    return fail(B200_ERR_ARG, "in_dtype must be F16, BF16 or E4M3");
  if (out_dtype != B200_F16 && out_dtype != B200_BF16 && out_dtype != B200_F32 && out_dtype != B200_E4M3)
    return fail(B200_ERR_ARG, "out_dtype must be F16, BF16, F32 or E4M3");
  if (activation != B200_ACT_NONE && activation != B200_ACT_LEAKY_RELU && activation != B200_ACT_SOFTMAX)
    return fail(B200_ERR_ARG, "bad activation");
  if (activation == B200_ACT_SOFTMAX) {
    if (N > 256) return fail(B200_ERR_UNSUPPORTED, "the softmax epilogue needs N <= 256 (one tile spans the row)");
    if (bias_mode != B200_BIAS_NONE || splits != 1 || out_dtype == B200_E4M3)
      return fail(B200_ERR_ARG, "the softmax epilogue takes no bias, no split-K and a 16- or 32-bit output");
    if (K == 0) return fail(B200_ERR_UNSUPPORTED, "softmax epilogue with K == 0");
  }
  DeviceCtx* ctx = ready_ctx();
  if (!ctx) return g_err_code;
  if (M == 0 || N == 0) return B200_OK;
  if (!c || (K > 0 && (!a || !b))) return fail(B200_ERR_ARG, "null pointer");
  if (stride_cn != 1 && N != 1) return fail(B200_ERR_UNSUPPORTED, "C must have stride_cn == 1");
  if (K == 0 && bias_mode != B200_BIAS_NONE) return fail(B200_ERR_UNSUPPORTED, "bias epilogue with K == 0");
  if (K == 0) {
    // an empty sum: the reference's K loop does not run and the zero accumulator is stored
    const int es = dtype_bytes(out_dtype);
    cudaError_t e = cudaMemset2DAsync(c, (size_t)stride_cm * es, 0, (size_t)N * es, (size_t)M,
                                      reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(B200_ERR_CUDA, "memset: %s", cudaGetErrorString(e));
    return B200_OK;
  }
  return launch_gemm(ctx, reinterpret_cast<cudaStream_t>(stream), a, b, c, M, N, K, stride_am, stride_ak, stride_bk,
                     stride_bn, stride_cm, in_dtype, out_dtype, activation, scale_a, scale_b, bias, bias_mode, bias_stride_m,
                     bias_stride_n, splits, workspace);
}

size_t b200_grouped_matmul_workspace(int group_count) { return gemm_grouped_workspace_bytes(group_count); }

static int grouped_args_ok(int in_dtype, int out_dtype) {
  if (in_dtype != B200_F16 && in_dtype != B200_BF16) return fail(B200_ERR_ARG, "grouped matmul takes F16 or BF16 inputs");
  if (out_dtype != B200_F16 && out_dtype != B200_BF16 && out_dtype != B200_F32)
    return fail(B200_ERR_ARG, "out_dtype must be F16, BF16 or F32");
  return B200_OK;
}

int b200_grouped_matmul_prepare(b200_stream_t stream, int group_count, const void* const* a, const void* const* b,
                                void* const* c, const int* sizes, const int* lds, int in_dtype, int out_dtype,
                                void* workspace, int* total_tiles) {
  if (!total_tiles) return fail(B200_ERR_ARG, "null total_tiles");
  *total_tiles = 0;
  if (group_count < 0) return fail(B200_ERR_ARG, "negative group count");
  if (group_count == 0) return B200_OK;
  if (!a || !b || !c || !sizes || !lds) return fail(B200_ERR_ARG, "null array");
  if (int rc = grouped_args_ok(in_dtype, out_dtype)) return rc;
  DeviceCtx* ctx = ready_ctx();
  if (!ctx) return g_err_code;
  return prepare_gemm_grouped(ctx, reinterpret_cast<cudaStream_t>(stream), group_count, a, b, c, sizes, lds, in_dtype,
                              out_dtype, workspace, total_tiles);
}

int b200_grouped_matmul_run(b200_stream_t stream, const void* workspace, int total_tiles, int in_dtype, int out_dtype) {
  if (total_tiles < 0) return fail(B200_ERR_ARG, "negative tile count");
  if (total_tiles == 0) return B200_OK;
  if (!workspace) return fail(B200_ERR_ARG, "null workspace");
  if (int rc = grouped_args_ok(in_dtype, out_dtype)) return rc;
  DeviceCtx* ctx = ready_ctx();
  if (!ctx) return g_err_code;
  return launch_gemm_grouped(ctx, reinterpret_cast<cudaStream_t>(stream), workspace, total_tiles, in_dtype, out_dtype);
}

int b200_grouped_matmul(b200_stream_t stream, int group_count, const void* const* a, const void* const* b,
                        void* const* c, const int* sizes, const int* lds, int in_dtype, int out_dtype,
                        void* workspace) {
  int total_tiles = 0;
  int rc = b200_grouped_matmul_prepare(stream, group_count, a, b, c, sizes, lds, in_dtype, out_dtype, workspace,
                                       &total_tiles);
  if (rc) return rc;
  return b200_grouped_matmul_run(stream, workspace, total_tiles, in_dtype, out_dtype);
}

int b200_attention_fwd_stats(b200_stream_t stream, const void* q, const void* k, const void* v, void* o, float* m,
                             float* row_max, int Z, int H, int N, int D, const int64_t stride_q[4],
                             const int64_t stride_k[4], const int64_t stride_v[4], const int64_t stride_o[4],
                             float sm_scale, int causal, int dtype) {
  if (Z < 0 || H < 0 || N < 0) return fail(B200_ERR_ARG, "negative dimension");
  if (dtype != B200_F16 && dtype != B200_BF16 && dtype != B200_E5M2)
    return fail(B200_ERR_ARG, "forward attention dtype must be F16, BF16 or E5M2");
  if (D != 64 && D != 128 && D != 256)
    return fail(B200_ERR_UNSUPPORTED, "head dim %d: the forward has kernels for 64, 128 and 256", D);
  if (D == 256 && dtype == B200_E5M2) return fail(B200_ERR_UNSUPPORTED, "the 8-bit forward has kernels for head dims 64 and 128");
  if (!(sm_scale > 0.f)) return fail(B200_ERR_ARG, "sm_scale must be positive");
  if (!stride_q || !stride_k || !stride_v || !stride_o) return fail(B200_ERR_ARG, "null stride array");
  if (dtype != B200_E5M2 && (stride_q[3] != 1 || stride_k[3] != 1 || stride_v[3] != 1 || stride_o[3] != 1))
    return fail(B200_ERR_UNSUPPORTED, "the head dimension must be contiguous");
  DeviceCtx* ctx = ready_ctx();
  if (!ctx) return g_err_code;
  if (Z == 0 || H == 0 || N == 0) return B200_OK;
  if (!q || !k || !v || !o || !m) return fail(B200_ERR_ARG, "null pointer");
  if ((long long)Z * H * ((N + 127) / 128) > 0x7fffffffLL) return fail(B200_ERR_UNSUPPORTED, "too many work items");
  return launch_attn_fwd(ctx, reinterpret_cast<cudaStream_t>(stream), q, k, v, o, m, row_max, Z, H, N, D, stride_q,
                         stride_k, stride_v, stride_o, sm_scale, causal, dtype);
}

int b200_attention_fwd(b200_stream_t stream, const void* q, const void* k, const void* v, void* o, float* m, int Z,
                       int H, int N, int D, const int64_t stride_q[4], const int64_t stride_k[4],
                       const int64_t stride_v[4], const int64_t stride_o[4], float sm_scale, int causal, int dtype) {
  return b200_attention_fwd_stats(stream, q, k, v, o, m, nullptr, Z, H, N, D, stride_q, stride_k, stride_v, stride_o,
                                  sm_scale, causal, dtype);
}

int b200_attention_bwd(b200_stream_t stream, const void* q, const void* k, const void* v, const void* o,
                       const void* d_o, const float* m, float* delta, void* dq, void* dk, void* dv, int Z, int H, int N,
                       int D, const int64_t stride_q[4], const int64_t stride_k[4], const int64_t stride_v[4],
                       const int64_t stride_o[4], const int64_t stride_do[4], const int64_t stride_dq[4],
                       const int64_t stride_dk[4], const int64_t stride_dv[4], float sm_scale, int causal, int dtype) {
  if (Z < 0 || H < 0 || N < 0) return fail(B200_ERR_ARG, "negative dimension");
  if (dtype != B200_F16 && dtype != B200_BF16) return fail(B200_ERR_ARG, "attention dtype must be F16 or BF16");
  if (D == 256)
    return fail(B200_ERR_UNSUPPORTED,
                "head dim 256: the backward needs [N, N] scratch at this head dim; call b200_attention_bwd_wide with a "
                "workspace of b200_attention_bwd_wide_workspace(N) bytes");
  if (D != 64 && D != 128) return fail(B200_ERR_UNSUPPORTED, "head dim %d: the backward has kernels for 64, 128 and (b200_attention_bwd_wide) 256", D);
  if (!(sm_scale > 0.f)) return fail(B200_ERR_ARG, "sm_scale must be positive");
  if (N % 128 != 0) return fail(B200_ERR_ARG, "backward needs N to be a multiple of 128 (N = %d)", N);
  const int64_t* all[8] = {stride_q, stride_k, stride_v, stride_o, stride_do, stride_dq, stride_dk, stride_dv};
  for (const int64_t* st : all) {
    if (!st) return fail(B200_ERR_ARG, "null stride array");
    if (st[3] != 1) return fail(B200_ERR_UNSUPPORTED, "the head dimension must be contiguous");
  }
  DeviceCtx* ctx = ready_ctx();
  if (!ctx) return g_err_code;
  if (Z == 0 || H == 0 || N == 0) return B200_OK;
  if (!q || !k || !v || !o || !d_o || !m || !delta || !dq || !dk || !dv) return fail(B200_ERR_ARG, "null pointer");
  if ((long long)Z * H * ((N + 127) / 128) > 0x7fffffffLL) return fail(B200_ERR_UNSUPPORTED, "too many work items");
  if ((reinterpret_cast<uintptr_t>(m) & 15) || (reinterpret_cast<uintptr_t>(delta) & 15))
    return fail(B200_ERR_UNSUPPORTED, "m and delta must be 16-byte aligned");
  return launch_attn_bwd(ctx, reinterpret_cast<cudaStream_t>(stream), q, k, v, o, d_o, m, delta, dq, dk, dv, Z, H, N, D,
                         stride_q, stride_k, stride_v, stride_o, stride_do, stride_dq, stride_dk, stride_dv, sm_scale,
                         causal, dtype);
}

size_t b200_attention_bwd_onepass_workspace(int Z, int H, int N, int D) {
  return (Z > 0 && H > 0 && N > 0 && D > 0) ? attn_bwd_fused_workspace_bytes(Z, H, N, D) : 0;
}

int b200_attention_bwd_onepass(b200_stream_t stream, const void* q, const void* k, const void* v, const void* o,
                               const void* d_o, const float* m, float* delta, float* dq_accum, void* dq, void* dk,
                               void* dv, int Z, int H, int N, int D, const int64_t stride_q[4],
                               const int64_t stride_k[4], const int64_t stride_v[4], const int64_t stride_o[4],
                               const int64_t stride_do[4], const int64_t stride_dq[4], const int64_t stride_dk[4],
                               const int64_t stride_dv[4], float sm_scale, int causal, int dtype) {
  if (Z < 0 || H < 0 || N < 0) return fail(B200_ERR_ARG, "negative dimension");
  if (dtype != B200_F16 && dtype != B200_BF16) return fail(B200_ERR_ARG, "attention dtype must be F16 or BF16");
  if (D != 64) return fail(B200_ERR_UNSUPPORTED, "the one-pass backward has a kernel for head dim 64 only (head dim %d)", D);
  if (!(sm_scale > 0.f)) return fail(B200_ERR_ARG, "sm_scale must be positive");
  if (N % 128 != 0) return fail(B200_ERR_ARG, "backward needs N to be a multiple of 128 (N = %d)", N);
  const int64_t* all[8] = {stride_q, stride_k, stride_v, stride_o, stride_do, stride_dq, stride_dk, stride_dv};
  for (const int64_t* st : all) {
    if (!st) return fail(B200_ERR_ARG, "null stride array");
    if (st[3] != 1) return fail(B200_ERR_UNSUPPORTED, "the head dimension must be contiguous");
  }
  DeviceCtx* ctx = ready_ctx();
  if (!ctx) return g_err_code;
  if (Z == 0 || H == 0 || N == 0) return B200_OK;
  if (!q || !k || !v || !o || !d_o || !m || !delta || !dq_accum || !dq || !dk || !dv) return fail(B200_ERR_ARG, "null pointer");
  if ((long long)Z * H * (N / 128) > 0x7fffffffLL) return fail(B200_ERR_UNSUPPORTED, "too many work items");
  for (const int64_t* s : {stride_o, stride_do})
    if ((s[0] & 7) || (s[1] & 7) || (s[2] & 7)) return fail(B200_ERR_UNSUPPORTED, "O / dO strides must be multiples of 8 elements");
  if ((reinterpret_cast<uintptr_t>(o) & 15) || (reinterpret_cast<uintptr_t>(d_o) & 15))
    return fail(B200_ERR_UNSUPPORTED, "O / dO must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(m) & 15) || (reinterpret_cast<uintptr_t>(delta) & 15) ||
      (reinterpret_cast<uintptr_t>(dq_accum) & 15))
    return fail(B200_ERR_UNSUPPORTED, "m, delta and dq_accum must be 16-byte aligned");
  return launch_attn_bwd_fused(ctx, reinterpret_cast<cudaStream_t>(stream), q, k, v, o, d_o, m, delta, dq_accum, dq, dk, dv,
                               Z, H, N, D, stride_q, stride_k, stride_v, stride_o, stride_do, stride_dq, stride_dk,
                               stride_dv, sm_scale, causal, dtype);
}

size_t b200_attention_bwd_wide_workspace(int N) { return N > 0 ? attn_bwd_wide_workspace_bytes(N) : 0; }

int b200_attention_bwd_wide(b200_stream_t stream, const void* q, const void* k, const void* v, const void* o,
                            const void* d_o, const float* m, float* delta, void* dq, void* dk, void* dv, int Z, int H,
                            int N, int D, const int64_t stride_q[4], const int64_t stride_k[4],
                            const int64_t stride_v[4], const int64_t stride_o[4], const int64_t stride_do[4],
                            const int64_t stride_dq[4], const int64_t stride_dk[4], const int64_t stride_dv[4],
                            float sm_scale, int causal, int dtype, void* workspace) {
  if (D != 256)  // the fused kernels serve the other head dims; same arguments minus the workspace
    return b200_attention_bwd(stream, q, k, v, o, d_o, m, delta, dq, dk, dv, Z, H, N, D, stride_q, stride_k, stride_v,
                              stride_o, stride_do, stride_dq, stride_dk, stride_dv, sm_scale, causal, dtype);
  if (Z < 0 || H < 0 || N < 0) return fail(B200_ERR_ARG, "negative dimension");
  if (dtype != B200_F16 && dtype != B200_BF16) return fail(B200_ERR_ARG, "attention dtype must be F16 or BF16");
  if (!(sm_scale > 0.f)) return fail(B200_ERR_ARG, "sm_scale must be positive");
  if (N % 128 != 0) return fail(B200_ERR_ARG, "backward needs N to be a multiple of 128 (N = %d)", N);
  const int64_t* all[8] = {stride_q, stride_k, stride_v, stride_o, stride_do, stride_dq, stride_dk, stride_dv};
  for (const int64_t* st : all) {
    if (!st) return fail(B200_ERR_ARG, "null stride array");
    if (st[3] != 1) return fail(B200_ERR_UNSUPPORTED, "the head dimension must be contiguous");
    if ((st[0] & 7) || (st[1] & 7) || (st[2] & 7)) return fail(B200_ERR_UNSUPPORTED, "strides must be multiples of 8 elements");
  }
  DeviceCtx* ctx = ready_ctx();
  if (!ctx) return g_err_code;
  if (Z == 0 || H == 0 || N == 0) return B200_OK;
  if (!q || !k || !v || !o || !d_o || !m || !delta || !dq || !dk || !dv) return fail(B200_ERR_ARG, "null pointer");
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return fail(B200_ERR_ARG, "head dim 256 needs a 256-byte aligned workspace of b200_attention_bwd_wide_workspace(N) bytes");
  for (const void* ptr : {q, k, v, o, d_o, (const void*)dq, (const void*)dk, (const void*)dv})
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return fail(B200_ERR_UNSUPPORTED, "tensors must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(m) & 15) || (reinterpret_cast<uintptr_t>(delta) & 15))
    return fail(B200_ERR_UNSUPPORTED, "m and delta must be 16-byte aligned");
  return launch_attn_bwd_wide(ctx, reinterpret_cast<cudaStream_t>(stream), q, k, v, o, d_o, m, delta, dq, dk, dv, Z, H, N,
                              D, stride_q, stride_k, stride_v, stride_o, stride_do, stride_dq, stride_dk, stride_dv,
                              sm_scale, causal, dtype, workspace);
}

long long b200_attention_bwd_noalloc_capacity(void) { return attn_bwd_scratch_capacity(); }

int b200_attention_bwd_noalloc(b200_stream_t stream, const void* q, const void* k, const void* v, const void* o,
                               const void* d_o, const float* m, void* dq, void* dk, void* dv, int Z, int H, int N,
                               int D, const int64_t stride_q[4], const int64_t stride_k[4], const int64_t stride_v[4],
                               const int64_t stride_o[4], const int64_t stride_do[4], const int64_t stride_dq[4],
                               const int64_t stride_dk[4], const int64_t stride_dv[4], float sm_scale, int causal,
                               int dtype) {
  if (Z < 0 || H < 0 || N < 0) return fail(B200_ERR_ARG, "negative dimension");
  // Z*H is checked first so that the row count cannot overflow: Z*H <= 2^20 and N < 2^31
  const long long cap = attn_bwd_scratch_capacity(), zh = (long long)Z * H;
  const long long rows = (zh > cap) ? cap + 1 : zh * N;
  if (rows > cap)
    return fail(B200_ERR_UNSUPPORTED,
                "Z*H*N = %lld * %d rows exceed the built-in scratch of %lld rows; use b200_attention_bwd with caller "
                "scratch for this size",
                zh, N, cap);
  float* delta = nullptr;
  if (rows > 0) {  // (an empty problem still goes through the same argument validation below)
    DeviceCtx* ctx = ready_ctx();
    if (!ctx) return g_err_code;
    delta = attn_bwd_scratch(ctx);
    if (!delta) return B200_ERR_CUDA;
  }
  // same validation and launches as the caller-scratch entry point, on the built-in array
  return b200_attention_bwd(stream, q, k, v, o, d_o, m, delta, dq, dk, dv, Z, H, N, D, stride_q, stride_k, stride_v,
                            stride_o, stride_do, stride_dq, stride_dk, stride_dv, sm_scale, causal, dtype);
}

}  // extern "C"
