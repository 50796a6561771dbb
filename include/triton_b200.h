/* triton_b200 — C ABI of the B200 (sm_100a) dense hot path: tiled matmul and flash attention.
 *
 * These entry points are what a host-language binding of the reference's op wrappers would
 * call instead of the reference's JIT launcher.  Conventions (they mirror the reference's
 * launcher, third_party/nvidia/backend/driver.py:274-325, and its ahead-of-time C template,
 * python/triton/tools/compile.h:12-14 — `CUresult kernel(CUstream stream, args...)`):
 *   - every pointer is a DEVICE pointer on the current device; the caller owns all memory,
 *     the library allocates nothing and keeps no pointer after the call returns;
 *   - launches are asynchronous on the given stream of the current device;
 *   - strides are in ELEMENTS, as in the reference kernels' argument lists;
 *   - the return value is 0 on success or a B200_ERR_* code; b200_last_error() gives the text
 *     (the reference raises RuntimeError / assert at this point, driver.py:154-169).
 * There is no CPU fallback: on a machine without an sm_100 device every compute entry point
 * returns B200_ERR_DEVICE.
 */
#ifndef TRITON_B200_H_
#define TRITON_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200_API __attribute__((visibility("default")))
#else
#define B200_API
#endif

typedef struct CUstream_st* b200_stream_t; /* a cudaStream_t / CUstream */

enum b200_dtype { B200_F16 = 0, B200_BF16 = 1, B200_E4M3 = 2, B200_F32 = 3, B200_E5M2 = 4 };
enum b200_activation { B200_ACT_NONE = 0, B200_ACT_LEAKY_RELU = 1, B200_ACT_SOFTMAX = 2 };
enum b200_bias { B200_BIAS_NONE = 0, B200_BIAS_MATRIX = 1, B200_BIAS_ROWS = 2, B200_BIAS_COLS = 3 };
enum b200_error {
  B200_OK = 0,
  B200_ERR_ARG = 1,         /* shapes / dtypes / null pointers (the reference's Python asserts) */
  B200_ERR_UNSUPPORTED = 2, /* layout the TMA path cannot address (alignment, stride) */
  B200_ERR_CUDA = 3,        /* a CUDA runtime or driver call failed */
  B200_ERR_DEVICE = 4,      /* no sm_100 device current */
  B200_ERR_KERNEL = 5       /* a bounded device-side wait ran out (see b200_status) */
};

/* Library version, and the text of the last error on the calling thread. */
B200_API int b200_version(void);
B200_API const char* b200_last_error(void);

/* Device status word of the current device: 0 when every kernel since the last clear ran
 * to completion normally; otherwise the code of the first bounded wait that gave up
 * (site | parity << 8 | block << 16).  Synchronises the device.  `clear` != 0 resets it.
 * Every wait inside the kernels has a time limit (250 ms); a kernel whose wait runs out records
 * the code, finishes without faulting and leaves its outputs incomplete.  The code is mirrored
 * into pinned host memory, and from then on every entry point that would launch work on that
 * device returns B200_ERR_KERNEL without launching, until b200_status(&v, 1) has cleared it
 * (no device synchronisation is involved in that check). */
B200_API int b200_status(unsigned* value, int clear);

/* Exercises the give-up path described above without any faulty input: launches one small
 * kernel that allocates tensor memory and waits, for at most `limit_us` microseconds (1 ..
 * 250000), on a barrier that nothing arrives on.  The kernel records its failure code
 * (site 99), frees what it holds and exits normally; afterwards the device is in the state
 * b200_status documents (compute entry points return B200_ERR_KERNEL until it is cleared).
 * No counterpart in the reference, whose kernels wait without limits. */
B200_API int b200_selftest_wait_timeout(b200_stream_t stream, unsigned limit_us);

/* C[M,N] = act(A[M,K] @ B[K,N]) with fp32 accumulation.
 * Replaces matmul_kernel + its launch in python/tutorials/03-matrix-multiplication.py:241-348
 * (pointer, size and stride arguments in the same order; ACTIVATION becomes `activation`), and
 * the fp8 matmul_kernel of python/test/unit/language/test_core.py:5110-5140 when in_dtype is
 * B200_E4M3.  scale_a / scale_b are optional DEVICE pointers to one fp32 each: the epilogue
 * multiplies the accumulator by (*scale_a) * (*scale_b) before the activation and the single
 * rounding to out_dtype (per-tensor fp8 scaling; pass NULL for 1.0).
 * A and B may have any strides; C must have stride_cn == 1.  The tensor-core path needs one unit
 * stride per operand, 16-byte aligned base addresses and non-unit strides that are multiples of
 * 16 bytes (what TMA can address); other layouts run on a plain CUDA-core kernel, correct but slow.
 * in_dtype: F16, BF16 or E4M3 (both operands); out_dtype: F16, BF16, F32 or E4M3 (see b200_matmul_bias). */
B200_API int b200_matmul(b200_stream_t stream, const void* a, const void* b, void* c, int M, int N, int K,
                int64_t stride_am, int64_t stride_ak, int64_t stride_bk, int64_t stride_bn,
                int64_t stride_cm, int64_t stride_cn, int in_dtype, int out_dtype, int activation,
                const float* scale_a, const float* scale_b);

/* Split-K variant for skinny problems (few output tiles, long K; the tall-skinny shapes of
 * python/test/regression/test_performance.py:36-46).  b200_matmul_plan says how many K splits pay
 * off for a shape on the current device and how large the fp32 workspace must be (0 when splits
 * is 1); b200_matmul_splitk computes exactly what b200_matmul computes, with the K range cut in
 * `splits` parts whose fp32 partial tiles go to `workspace` ([splits][M][N] floats, caller's
 * scratch) and are summed in a fixed order by a second kernel (deterministic).  splits == 1 is
 * b200_matmul.  The reference has no counterpart (its kernels do not split K); the library still
 * allocates nothing. */
B200_API int b200_matmul_plan(int M, int N, int K, int in_dtype, int* splits, size_t* workspace_bytes);
B200_API int b200_matmul_splitk(b200_stream_t stream, const void* a, const void* b, void* c, int M, int N, int K,
                                int64_t stride_am, int64_t stride_ak, int64_t stride_bk, int64_t stride_bn,
                                int64_t stride_cm, int64_t stride_cn, int in_dtype, int out_dtype, int activation,
                                const float* scale_a, const float* scale_b, int splits, float* workspace);

/* The reference's 'chain-dot' epilogue (python/test/unit/hopper/test_gemm.py:229-232: `w = tl.load(w_tile_ptr);
 * z = tl.dot(z.to(w.dtype), w); z = z.to(out_dtype)`, case list :269-284) as one launch:
 * c[M,N2] = out_type( in_type(out_type(a[M,K] @ b[K,N])) @ w[N,N2] ), fp32 accumulation in both
 * products, the intermediate rounded to the output type and then to the input type as the reference
 * does.  a, b, w: F16 or BF16 (one type), element strides as in b200_matmul (w[k * stride_wk +
 * n * stride_wn]); a row of a @ b stays in one tile, so N and N2 are at most 128
 * (B200_ERR_UNSUPPORTED beyond; the reference's test uses BLOCK_N == N); operands must be
 * addressable by TMA (16-byte aligned base and rows). */
B200_API int b200_matmul_chain(b200_stream_t stream, const void* a, const void* b, const void* w, void* c, int M, int N,
                               int K, int N2, int64_t stride_am, int64_t stride_ak, int64_t stride_bk,
                               int64_t stride_bn, int64_t stride_wk, int64_t stride_wn, int64_t stride_cm,
                               int64_t stride_cn, int in_dtype, int out_dtype);

/* Matmul with the reference's bias epilogues (python/test/unit/hopper/test_gemm.py:213-222, cases
 * 'add-matrix', 'add-rows', 'add-cols' at :281): c = out_type(act(scale * a @ b)) + bias, the sum
 * formed in the output type as the reference does (`z = z.to(out_dtype); z += bias`).  `bias` has
 * the output type (F16, BF16 or F32) and is indexed bias[m * bias_stride_m + n * bias_stride_n];
 * B200_BIAS_ROWS reads one value per output row (n ignored), B200_BIAS_COLS one per column
 * (m ignored), B200_BIAS_NONE makes this b200_matmul_splitk.  out_dtype B200_E4M3 (8-bit output,
 * python/tutorials/09-persistent-matmul.py: `c = accumulator.to(tl.float8e4nv)`, round to nearest
 * even, saturating) is accepted here, by b200_matmul and by b200_matmul_splitk, without a bias.
 * activation B200_ACT_SOFTMAX is the reference's 'softmax' epilogue (test_gemm.py:223-228): a
 * softmax over every output row, computed like the reference in the output type (F16, BF16 or
 * F32); it needs N <= 256 (one tile spans the row), no bias, splits == 1 and TMA-addressable
 * operands. */
B200_API int b200_matmul_bias(b200_stream_t stream, const void* a, const void* b, void* c, int M, int N, int K,
                              int64_t stride_am, int64_t stride_ak, int64_t stride_bk, int64_t stride_bn,
                              int64_t stride_cm, int64_t stride_cn, int in_dtype, int out_dtype, int activation,
                              const float* scale_a, const float* scale_b, const void* bias, int bias_mode,
                              int64_t bias_stride_m, int64_t bias_stride_n, int splits, float* workspace);

/* Grouped matmul: c[g] = a[g] @ b[g] for group_count independent problems in one persistent launch
 * (python/tutorials/08-grouped-gemm.py:64-141 grouped_matmul_kernel, :144-191 group_gemm_fn).
 * a, b, c are HOST arrays of device pointers; sizes = {M, N, K} and lds = {lda, ldb, ldc} per group
 * are host arrays laid out like the reference's `group_gemm_sizes` and `g_lds` tensors ([group][3]).
 * A[g] is [M, K] row-major with leading dimension lda, B[g] is [K, N] row-major (ldb), C[g] is
 * [M, N] row-major (ldc), as in the reference; in_dtype F16 or BF16, out_dtype F16, BF16 or F32,
 * fp32 accumulation, one rounding.  Partial tiles are handled (the reference assumes full tiles).
 * Operands must be addressable by TMA (16-byte aligned base, lda and ldb multiples of 8 elements),
 * else B200_ERR_UNSUPPORTED.  `workspace`: b200_grouped_matmul_workspace(group_count) bytes of
 * device memory, 128-byte aligned, owned by the caller; the call writes the groups' descriptors
 * there (asynchronously, on `stream`) and the kernel reads them, so it must stay untouched until
 * the work on `stream` has finished. */
B200_API size_t b200_grouped_matmul_workspace(int group_count);
B200_API int b200_grouped_matmul(b200_stream_t stream, int group_count, const void* const* a, const void* const* b,
                                 void* const* c, const int* sizes, const int* lds, int in_dtype, int out_dtype,
                                 void* workspace);
/* The two halves of b200_grouped_matmul, for callers that run the same groups repeatedly (the
 * reference times `triton_perf_fn`, which launches on device tensors prepared once,
 * 08-grouped-gemm.py:218-229): _prepare writes the descriptors (pointers, sizes, tensor maps) to
 * `workspace` and returns the tile count; _run launches on a prepared workspace and can be called
 * any number of times while the operands stay where they were.  Groups with K == 0 are zeroed by
 * _prepare only. */
B200_API int b200_grouped_matmul_prepare(b200_stream_t stream, int group_count, const void* const* a,
                                         const void* const* b, void* const* c, const int* sizes, const int* lds,
                                         int in_dtype, int out_dtype, void* workspace, int* total_tiles);
B200_API int b200_grouped_matmul_run(b200_stream_t stream, const void* workspace, int total_tiles, int in_dtype,
                                     int out_dtype);

/* Flash-attention forward: O = softmax(Q K^T * sm_scale, causal mask optional) V, and per-row
 * statistics M[Z,H,N] (fp32) = base-2 log-sum-exp of the scores scaled by sm_scale * log2(e)
 * (natural-log LSE = M * ln 2).
 * Replaces _attn_fwd and its launch in _attention.forward,
 * python/tutorials/06-fused-attention.py:98-187, 441-475 (Q, K, V, sm_scale, M, Out, the four
 * stride quadruples, Z, H, N_CTX, HEAD_DIM, STAGE -> causal).
 * q, k, v, o: [Z, H, N, D] of `dtype` (F16 or BF16) with element strides {z, h, n, d} each; the d
 * stride must be 1 and the others multiples of 8 elements; D is 64, 128 or 256; sm_scale > 0.
 * (The reference's set is {16, 32, 64, 128, 256}, 06-fused-attention.py:447: 16 and 32 are served by
 * the host wrapper, which appends zero columns up to 64 - they change neither Q K^T nor the kept
 * columns of O.)
 * m: contiguous [Z, H, N] fp32.
 * dtype E5M2 is the reference's 8-bit forward (06-fused-attention.py:38-40, 66-69, 127, 609-615):
 * q, k, v and o are e5m2, both products run on 8-bit MMAs, P is converted to e5m2 (round to
 * nearest even, saturating) before the second product and O is stored as e5m2.  D must be 64 (the
 * reference's own fp8 benchmark shape, :570) or 128;
 * q, k, o need a d stride of 1 and other strides that are multiples of 16 elements; v must have its
 * KEY dimension contiguous (stride_v[2] == 1, the `v.permute(0, 1, 3, 2).contiguous().permute(0,
 * 1, 3, 2)` layout the reference gives an fp8 V) and stride_v[3] a multiple of 16. */
B200_API int b200_attention_fwd(b200_stream_t stream, const void* q, const void* k, const void* v, void* o, float* m,
                                int Z, int H, int N, int D, const int64_t stride_q[4], const int64_t stride_k[4],
                                const int64_t stride_v[4], const int64_t stride_o[4], float sm_scale, int causal,
                                int dtype);

/* b200_attention_fwd that also returns the row maximum: row_max[Z,H,N] (fp32, contiguous, may be
 * NULL) = max over the (unmasked) keys of q.k * sm_scale * log2(e), the base-2 counterpart of `m`.
 * The reference's older forward kernel (python/test/unit/hopper/test_flashattention.py:36-131)
 * stores its statistics as two tensors, the row maximum M and the row sum L of exp(score - M)
 * (:128-131); they follow from the two outputs here as M = row_max * ln 2 and
 * L = 2^(m - row_max). */
B200_API int b200_attention_fwd_stats(b200_stream_t stream, const void* q, const void* k, const void* v, void* o,
                                      float* m, float* row_max, int Z, int H, int N, int D,
                                      const int64_t stride_q[4], const int64_t stride_k[4],
                                      const int64_t stride_v[4], const int64_t stride_o[4], float sm_scale,
                                      int causal, int dtype);

/* Flash-attention backward: dQ, dK, dV from Q, K, V, O, dO and the forward's statistics M.
 * Replaces _attn_bwd_preprocess, _attn_bwd and their launches in _attention.backward,
 * python/tutorials/06-fused-attention.py:190-435, 478-517 (Q, K, V, sm_scale, DO, DQ, DK, DV, M, D
 * -> delta, strides, H, N_CTX; the host-side pre-scaling of K at :491-492 is folded into the kernels).
 * All tensors [Z, H, N, D] of `dtype` with their own element strides {z, h, n, d} (d stride 1, the
 * others multiples of 8); m and delta are contiguous [Z, H, N] fp32.  `delta` is SCRATCH memory the
 * caller provides (Z*H*N floats): the pre-pass writes rowsum(O * dO) there and the main kernels
 * read it; its contents after the call are that intermediate.  N must be a multiple of 128 (the
 * reference asserts the same, :494).  `causal` selects the mask for both kernels (the reference's
 * backward always applies the causal mask; pass the flag the forward was run with). */
B200_API int b200_attention_bwd(b200_stream_t stream, const void* q, const void* k, const void* v, const void* o,
                                const void* d_o, const float* m, float* delta, void* dq, void* dk, void* dv, int Z,
                                int H, int N, int D, const int64_t stride_q[4], const int64_t stride_k[4],
                                const int64_t stride_v[4], const int64_t stride_o[4], const int64_t stride_do[4],
                                const int64_t stride_dq[4], const int64_t stride_dk[4], const int64_t stride_dv[4],
                                float sm_scale, int causal, int dtype);

/* The backward at head dim 64 in one pass: same results as b200_attention_bwd up to the rounding of
 * dQ described below, about 1.6x faster.  b200_attention_bwd runs two kernels (dK/dV per K/V block,
 * dQ per Q block, the reference's layout, 06-fused-attention.py:308-435) and each recomputes the
 * scores, the exponentials and dS; here one kernel walks the (K/V block, Q block) pairs once,
 * accumulates dK and dV as before and adds every 128 x 64 partial of dQ into `dq_accum` - fp32
 * [Z, H, N, 64], b200_attention_bwd_onepass_workspace(Z, H, N, D) bytes of caller scratch, 16-byte
 * aligned, cleared by the call - with TMA reduce-adds; a last kernel scales the sums by sm_scale and
 * rounds them into dq.  This is the reference's older `sequence_parallel` backward
 * (python/test/regression/test_performance.py:174, 194: partial dQ per K/V block, summed
 * afterwards).  The partials of one Q block arrive in no fixed order, so the last bit of dQ may
 * differ from run to run (dK, dV are deterministic); callers that need bitwise repeatability use
 * b200_attention_bwd.  D must be 64 (B200_ERR_UNSUPPORTED otherwise, also for dK / dV / dQ layouts
 * that TMA cannot address); all other arguments as for b200_attention_bwd. */
B200_API size_t b200_attention_bwd_onepass_workspace(int Z, int H, int N, int D);
B200_API int b200_attention_bwd_onepass(b200_stream_t stream, const void* q, const void* k, const void* v,
                                        const void* o, const void* d_o, const float* m, float* delta,
                                        float* dq_accum, void* dq, void* dk, void* dv, int Z, int H, int N, int D,
                                        const int64_t stride_q[4], const int64_t stride_k[4],
                                        const int64_t stride_v[4], const int64_t stride_o[4],
                                        const int64_t stride_do[4], const int64_t stride_dq[4],
                                        const int64_t stride_dk[4], const int64_t stride_dv[4], float sm_scale,
                                        int causal, int dtype);

/* b200_attention_bwd for every head dim of the reference's set, 256 included (06-fused-attention.py:447).
 * The fused backward kernels hold four 128 x D operand tiles in shared memory, which fits for D = 64
 * and 128.  At D = 256 the same arithmetic (same roundings of P and dS to the storage type) is laid
 * out per (batch, head) as matmuls of this library - S = Q K^T and dP = dO V^T into fp32 [N, N], one
 * element-wise pass for P and dS, then dV = P^T dO, dK = sm_scale dS^T Q, dQ = sm_scale dS K - and
 * needs `workspace`: b200_attention_bwd_wide_workspace(N) bytes (12 N^2 + 256) of caller-owned device
 * memory, 256-byte aligned, reused head after head.  Other head dims ignore the workspace and run the
 * fused kernels.  All tensors 16-byte aligned, strides multiples of 8 elements. */
B200_API size_t b200_attention_bwd_wide_workspace(int N);
B200_API int b200_attention_bwd_wide(b200_stream_t stream, const void* q, const void* k, const void* v, const void* o,
                                     const void* d_o, const float* m, float* delta, void* dq, void* dk, void* dv,
                                     int Z, int H, int N, int D, const int64_t stride_q[4], const int64_t stride_k[4],
                                     const int64_t stride_v[4], const int64_t stride_o[4],
                                     const int64_t stride_do[4], const int64_t stride_dq[4],
                                     const int64_t stride_dk[4], const int64_t stride_dv[4], float sm_scale,
                                     int causal, int dtype, void* workspace);

/* Same computation as b200_attention_bwd, for callers that may not allocate device memory.
 * (No counterpart in the reference, whose Python wrapper allocates `delta` with torch.empty_like.)
 * Some hosts of this library hand every byte of device memory to their own arena or planner at
 * start-up - an inference server with a fixed memory plan, a runtime that forbids allocation on
 * its hot path - and have nowhere to take the Z*H*N-float `delta` scratch from without going back
 * to the allocator.  Here that scratch is a fixed array built into the library image: 2^20 floats
 * (4 MiB), held by every GPU that loads the library until the process exits.  The call makes no
 * cudaMalloc / cudaFree and uses no allocating library routine; inputs and outputs are still the
 * caller's.
 *   - Z*H*N must not exceed b200_attention_bwd_noalloc_capacity() (2^20); larger problems are
 *     rejected with B200_ERR_UNSUPPORTED and a message.
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call outside any stream capture.
 *   - All calls on a device share the one array.  It keeps whatever the previous call left there;
 *     nothing in it needs to start at zero because the pre-pass overwrites every row the main
 *     kernels read.  Two calls whose kernels overlap on the GPU (different streams) race on it:
 *     serialise them. */
B200_API int b200_attention_bwd_noalloc(b200_stream_t stream, const void* q, const void* k, const void* v,
                                        const void* o, const void* d_o, const float* m, void* dq, void* dk, void* dv,
                                        int Z, int H, int N, int D, const int64_t stride_q[4],
                                        const int64_t stride_k[4], const int64_t stride_v[4],
                                        const int64_t stride_o[4], const int64_t stride_do[4],
                                        const int64_t stride_dq[4], const int64_t stride_dk[4],
                                        const int64_t stride_dv[4], float sm_scale, int causal, int dtype);
B200_API long long b200_attention_bwd_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
#endif /* TRITON_B200_H_ */
