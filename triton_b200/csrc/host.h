// Host-side helpers shared by the launchers: per-device context, error reporting and
// TMA tensor-map encoding.  Internal to the library (the public surface is include/triton_b200.h).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/triton_b200.h"
#include "trace.h"

namespace tb {

struct DeviceCtx {
  int device = -1;
  int sm_count = 0;
  int max_smem_optin = 0;
  unsigned* status = nullptr;  // device address of the status word (a __device__ symbol, never cudaMalloc'd)
  unsigned* host_status = nullptr;  // pinned host mirror of the status word (nullptr: none), written by a failing kernel
};

// Context of the CURRENT device; created on first use.  Returns nullptr (and sets the error
// string) when no usable sm_100 device is current.
DeviceCtx* current_ctx();

// current_ctx() for an entry point that launches: additionally refuses (B200_ERR_KERNEL, nullptr)
// while the device's status word records a bounded wait that ran out.  Reads the pinned host
// mirror, so it costs no device synchronisation.
DeviceCtx* ready_ctx();

// A work counter (zero between launches: the kernel restores it) for one launch of a persistent kernel on
// `stream`; launches under stream capture get counters that are never handed out again (nullptr + error
// string on failure).
int* next_sched_counter(DeviceCtx* ctx, cudaStream_t stream);

// Record an error message for b200_last_error() and return `code`.
int fail(int code, const char* fmt, ...);

// Encode a tiled tensor map.  dims/strides innermost first; strides_bytes[0] is the stride of
// dimension 1 (dimension 0 is contiguous).  swizzle: 0 none, 1 (or true) 128-byte, 2 64-byte swizzle.
bool encode_tmap(CUtensorMap* out, int dtype, int rank, const void* base, const uint64_t* dims,
                 const uint64_t* strides_bytes, const uint32_t* box, int swizzle);

// cudaFuncAttributeMaxDynamicSharedMemorySize of `kernel`, set once per device; `done` is the
// launcher's static per-device flag array.  Host threads may race here: setting the attribute twice
// is harmless, the flags are atomics.
template <typename Kernel>
inline int ensure_dynamic_smem(Kernel kernel, size_t smem, int device, std::atomic<bool>* done, const char* what) {
  if (done[device].load(std::memory_order_acquire)) return B200_OK;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "cudaFuncSetAttribute(%s): %s", what, cudaGetErrorString(e));
  done[device].store(true, std::memory_order_release);
  return B200_OK;
}

inline int dtype_bytes(int dt) {
  switch (dt) {
    case B200_F16:
    case B200_BF16: return 2;
    case B200_E4M3:
    case B200_E5M2: return 1;
    case B200_F32: return 4;
    default: return 0;
  }
}

// launchers implemented in the kernel translation units
int launch_gemm_chain(DeviceCtx* ctx, cudaStream_t stream, const void* a, const void* b, const void* w, void* c, int M,
                      int N, int K, int N2, int64_t sam, int64_t sak, int64_t sbk, int64_t sbn, int64_t swk, int64_t swn,
                      int64_t scm, int in_dtype, int out_dtype);
int launch_gemm(DeviceCtx* ctx, cudaStream_t stream, const void* a, const void* b, void* c, int M, int N, int K,
                int64_t sam, int64_t sak, int64_t sbk, int64_t sbn, int64_t scm, int in_dtype, int out_dtype,
                int activation, const float* scale_a, const float* scale_b, const void* bias, int bias_mode,
                int64_t bias_sm, int64_t bias_sn, int splits, float* ws);
int gemm_plan_splits(DeviceCtx* ctx, int M, int N, int K, int in_dtype);
size_t gemm_grouped_workspace_bytes(int group_count);
int prepare_gemm_grouped(DeviceCtx* ctx, cudaStream_t stream, int group_count, const void* const* a,
                         const void* const* b, void* const* c, const int* sizes, const int* lds, int in_dtype,
                         int out_dtype, void* workspace, int* total_tiles_out);
int launch_gemm_grouped(DeviceCtx* ctx, cudaStream_t stream, const void* workspace, int total_tiles, int in_dtype,
                        int out_dtype);

int launch_attn_fwd(DeviceCtx* ctx, cudaStream_t stream, const void* q, const void* k, const void* v, void* o,
                    float* m, float* row_max, int Z, int H, int N, int D, const int64_t* sq, const int64_t* sk, const int64_t* sv,
                    const int64_t* so, float sm_scale, int causal, int dtype);

int launch_attn_bwd(DeviceCtx* ctx, cudaStream_t stream, const void* q, const void* k, const void* v, const void* o,
                    const void* dout, const float* m, float* delta, void* dq, void* dk, void* dv, int Z, int H, int N,
                    int D, const int64_t* sq, const int64_t* sk, const int64_t* sv, const int64_t* so,
                    const int64_t* sdo, const int64_t* sdq, const int64_t* sdk, const int64_t* sdv, float sm_scale,
                    int causal, int dtype);

// the backward's pre-pass on its own: delta[z, h, n] = sum_d O * dO (head dims 64, 128, 256)
int launch_attn_bwd_delta(DeviceCtx* ctx, cudaStream_t stream, const void* o, const void* dout, float* delta, int Z,
                          int H, int N, int D, const int64_t* so, const int64_t* sdo, int dtype,
                          float* zero_rows = nullptr);

// head dim 256 backward, composed of matmul launches per head (attn_bwd_wide.cu)
size_t attn_bwd_wide_workspace_bytes(int N);
int launch_attn_bwd_wide(DeviceCtx* ctx, cudaStream_t stream, const void* q, const void* k, const void* v,
                         const void* o, const void* dout, const float* m, float* delta, void* dq, void* dk, void* dv,
                         int Z, int H, int N, int D, const int64_t* sq, const int64_t* sk, const int64_t* sv,
                         const int64_t* so, const int64_t* sdo, const int64_t* sdq, const int64_t* sdk,
                         const int64_t* sdv, float sm_scale, int causal, int dtype, void* workspace);

// head dim 64 backward in one pass (attn_bwd_fused.cu); dq_acc: Z*H*N*64 floats of caller scratch
size_t attn_bwd_fused_workspace_bytes(int Z, int H, int N, int D);
int launch_attn_bwd_fused(DeviceCtx* ctx, cudaStream_t stream, const void* q, const void* k, const void* v, const void* o,
                          const void* dout, const float* m, float* delta, float* dq_acc, void* dq, void* dk, void* dv, int Z,
                          int H, int N, int D, const int64_t* sq, const int64_t* sk, const int64_t* sv, const int64_t* so,
                          const int64_t* sdo, const int64_t* sdq, const int64_t* sdk, const int64_t* sdv, float sm_scale,
                          int causal, int dtype);

// built-in scratch of the no-allocation backward entry point (attn_bwd.cu)
long long attn_bwd_scratch_capacity();
float* attn_bwd_scratch(DeviceCtx* ctx);

// 4-D tensor map over [Z, H, N, D] (D contiguous): boxes of 64 columns x box_rows rows, 128-byte swizzle
// 4-D map over a [Z, H, N, D] tensor (D contiguous) with boxes of box_cols x box_rows elements
bool encode_rows_map(CUtensorMap* out, int dtype, const void* base, int Z, int H, int N, int D, int64_t sz, int64_t sh,
                     int64_t sn, int box_cols, int box_rows, int swizzle);
bool encode_qkv_map(CUtensorMap* out, int dtype, const void* base, int Z, int H, int N, int D, int64_t sz, int64_t sh,
                    int64_t sn, int box_rows);

}  // namespace tb
