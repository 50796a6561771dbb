// Flash-attention backward at head dim 256, composed of this library's matmul kernel.
//
// The reference's backward takes head dims up to 256 (python/tutorials/06-fused-attention.py:447,
// 478-517).  The fused backward kernels of attn_bwd.cu keep four 128 x D operand tiles in shared
// memory, which fits for D = 64 and 128 only; at D = 256 the same arithmetic is laid out per
// (batch, head) as
//     S  = Q K^T,  dP = dO V^T                      two matmuls into fp32 [N, N]
//     P  = exp2(S * sm_scale * log2 e - M) masked,  dS = P * (dP - delta)      one element-wise pass,
//                                                    both rounded to the storage type (:244, :251, :297)
//     dV = P^T dO,  dK = sm_scale * dS^T Q,  dQ = sm_scale * dS K               three matmuls
// with the [N, N] intermediates in a workspace the caller provides (12 * N^2 bytes, reused head after
// head).  Same roundings as the fused path; O(N^2) scratch and no overlap between the steps, so it is
// the slow path of a head dim the reference's own benchmarks do not use.
#include "common.cuh"
#include "host.h"

namespace tb {

namespace {

// eight consecutive keys of one query row per thread
template <bool BF16>
__global__ void __launch_bounds__(256)
attn_bwd_wide_pointwise_kernel(const float* __restrict__ s, const float* __restrict__ dp, const float* __restrict__ m,
                               const float* __restrict__ delta, uint16_t* __restrict__ p16, uint16_t* __restrict__ ds16,
                               int N, float scale_log2, int causal) {
  const int row = blockIdx.y;
  const int col0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (col0 >= N) return;
  const long long base = (long long)row * N + col0;
  const float mr = m[row], dr = delta[row];
  const float4 s0 = *reinterpret_cast<const float4*>(s + base), s1 = *reinterpret_cast<const float4*>(s + base + 4);
  const float4 d0 = *reinterpret_cast<const float4*>(dp + base), d1 = *reinterpret_cast<const float4*>(dp + base + 4);
  const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  const float dv[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
  float pv[8], dsv[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    float p = ex2(fmaf(sv[k], scale_log2, -mr));
    if (causal && col0 + k > row) p = 0.f;  // keys after the query contribute exactly 0
    pv[k] = p;
    dsv[k] = p * (dv[k] - dr);
  }
  uint32_t pw[4], dw[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    pw[k] = pack2<BF16>(pv[2 * k], pv[2 * k + 1]);
    dw[k] = pack2<BF16>(dsv[2 * k], dsv[2 * k + 1]);
  }
  *reinterpret_cast<uint4*>(p16 + base) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
  *reinterpret_cast<uint4*>(ds16 + base) = make_uint4(dw[0], dw[1], dw[2], dw[3]);
}

__global__ void write_scalar_kernel(float* dst, float v) { *dst = v; }

}  // namespace

size_t attn_bwd_wide_workspace_bytes(int N) { return (size_t)12 * N * N + 256; }

int launch_attn_bwd_wide(DeviceCtx* ctx, cudaStream_t stream, const void* q, const void* k, const void* v,
                         const void* o, const void* dout, const float* m, float* delta, void* dq, void* dk, void* dv,
                         int Z, int H, int N, int D, const int64_t* sq, const int64_t* sk, const int64_t* sv,
                         const int64_t* so, const int64_t* sdo, const int64_t* sdq, const int64_t* sdk,
                         const int64_t* sdv, float sm_scale, int causal, int dtype, void* workspace) {
  if (int rc = launch_attn_bwd_delta(ctx, stream, o, dout, delta, Z, H, N, D, so, sdo, dtype)) return rc;
  const size_t nn = (size_t)N * N;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float* s_ws = reinterpret_cast<float*>(ws);
  float* dp_ws = reinterpret_cast<float*>(ws + 4 * nn);
  uint16_t* p_ws = reinterpret_cast<uint16_t*>(ws + 8 * nn);
  uint16_t* ds_ws = reinterpret_cast<uint16_t*>(ws + 10 * nn);
  float* scale_dev = reinterpret_cast<float*>(ws + 12 * nn);
  write_scalar_kernel<<<1, 1, 0, stream>>>(scale_dev, sm_scale);
  const float scale_log2 = sm_scale * 1.44269504f;
  const int eb = 2;
  auto at = [&](const void* base, const int64_t* st, int z, int h) {
    return static_cast<const uint8_t*>(base) + ((long long)z * st[0] + (long long)h * st[1]) * eb;
  };
  for (int z = 0; z < Z; ++z) {
    for (int h = 0; h < H; ++h) {
      const void *qh = at(q, sq, z, h), *kh = at(k, sk, z, h), *vh = at(v, sv, z, h), *doh = at(dout, sdo, z, h);
      void* dqh = const_cast<uint8_t*>(at(dq, sdq, z, h));
      void* dkh = const_cast<uint8_t*>(at(dk, sdk, z, h));
      void* dvh = const_cast<uint8_t*>(at(dv, sdv, z, h));
      const float* mh = m + ((long long)z * H + h) * N;
      const float* dh = delta + ((long long)z * H + h) * N;
      // S = Q K^T and dP = dO V^T: the second operand is read as B[d][key] = X[key][d]
      int rc = launch_gemm(ctx, stream, qh, kh, s_ws, N, N, D, sq[2], 1, 1, sk[2], N, dtype, B200_F32, B200_ACT_NONE, nullptr,
                           nullptr, nullptr, B200_BIAS_NONE, 0, 0, 1, nullptr);
      if (rc) return rc;
      rc = launch_gemm(ctx, stream, doh, vh, dp_ws, N, N, D, sdo[2], 1, 1, sv[2], N, dtype, B200_F32, B200_ACT_NONE, nullptr,
                       nullptr, nullptr, B200_BIAS_NONE, 0, 0, 1, nullptr);
      if (rc) return rc;
      dim3 grid((N / 8 + 255) / 256, N, 1);
      if (dtype == B200_BF16)
        attn_bwd_wide_pointwise_kernel<true><<<grid, 256, 0, stream>>>(s_ws, dp_ws, mh, dh, p_ws, ds_ws, N, scale_log2, causal);
      else
        attn_bwd_wide_pointwise_kernel<false><<<grid, 256, 0, stream>>>(s_ws, dp_ws, mh, dh, p_ws, ds_ws, N, scale_log2, causal);
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return fail(B200_ERR_CUDA, "attn bwd (head dim 256) pointwise launch: %s", cudaGetErrorString(e));
      // dV = P^T dO, dK = sm_scale * dS^T Q: the first operand is read as A[key][query] = X[query][key]
      rc = launch_gemm(ctx, stream, p_ws, doh, dvh, N, D, N, 1, N, sdo[2], 1, sdv[2], dtype, dtype, B200_ACT_NONE, nullptr,
                       nullptr, nullptr, B200_BIAS_NONE, 0, 0, 1, nullptr);
      if (rc) return rc;
      rc = launch_gemm(ctx, stream, ds_ws, qh, dkh, N, D, N, 1, N, sq[2], 1, sdk[2], dtype, dtype, B200_ACT_NONE, scale_dev,
                       nullptr, nullptr, B200_BIAS_NONE, 0, 0, 1, nullptr);
      if (rc) return rc;
      // dQ = sm_scale * dS K
      rc = launch_gemm(ctx, stream, ds_ws, kh, dqh, N, D, N, N, 1, sk[2], 1, sdq[2], dtype, dtype, B200_ACT_NONE, scale_dev,
                       nullptr, nullptr, B200_BIAS_NONE, 0, 0, 1, nullptr);
      if (rc) return rc;
    }
  }
  return B200_OK;
}

}  // namespace tb
