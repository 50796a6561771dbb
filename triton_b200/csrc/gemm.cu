// Persistent, warp-specialised tiled matmul for sm_100a.
//
// Computes what the reference's matmul_kernel computes (python/tutorials/03-matrix-
// multiplication.py:241-316; fp8 variant python/test/unit/language/test_core.py:5110-5140):
// C = act(scale * A @ B), fp32 accumulation, one rounding to the output type, program ids
// mapped to tiles in groups of 8 tile-rows (03-...py:265-273).  The reference's persistent
// variants (python/tutorials/09-persistent-matmul.py:141-309) are the model for the structure:
// one CTA per SM walks tiles `tile += gridDim.x`.
//
// Structure of one CTA (192 threads):
//   warp 0      TMA producer: fills a ring of shared-memory stages (A 128 x 128 B, B BN x 128 B,
//               128-byte swizzle) and signals `full[s]` through the copy's byte count
//   warp 1      MMA issuer: one thread issues tcgen05.mma (128 x BN x 32 B per instruction) into
//               one of two TMEM accumulators; tcgen05.commit releases the stage (`empty[s]`)
//               and, after the last K block, publishes the accumulator (`tmem_full[acc]`)
//   warps 2-5   epilogue: tcgen05.ld the accumulator (each warp owns 32 TMEM lanes = 32 rows),
//               scale / activation / convert, store C, then hand the accumulator back
//               (`tmem_empty[acc]`), so the epilogue of tile i overlaps the main loop of tile i+1
// Out-of-range rows / columns / K are zero-filled by TMA, which is the masked load of the
// reference (03-...py:297-298); stores are bounds-checked.
#include "common.cuh"
#include "host.h"

namespace tb {

namespace {

constexpr int BM = 128;
constexpr int KBYTES = 128;  // bytes of K per stage row = swizzle span
constexpr int GEMM_THREADS = 192;
constexpr int GROUP_M = 8;

struct OperandGeom {
  uint32_t mn_major;     // 0: K contiguous, 1: M/N contiguous
  uint32_t nbox;         // TMA boxes per stage
  uint32_t box_bytes;    // bytes of one box in shared memory
  uint32_t box_mn;       // extent of one box along M/N, elements (MN-major only)
  uint32_t lbo, sbo;     // descriptor offsets
  uint32_t kstep_bytes;  // start-address advance per MMA K step (32 bytes of K)
};

struct GemmParams {
  void* c;
  int M, N, K;
  long long ldc;
  int out_dtype, activation, fp8;
  const float* scale_a;
  const float* scale_b;
  unsigned* status;
  int num_pid_m, num_pid_n, num_tiles, num_k, bk_elems;
  uint32_t idesc;
  OperandGeom ga, gb;
};

__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& pid_m, int& pid_n) {
  const int in_group = GROUP_M * p.num_pid_n;
  const int group_id = tile / in_group;
  const int first_m = group_id * GROUP_M;
  const int gsz = min(p.num_pid_m - first_m, GROUP_M);
  pid_m = first_m + ((tile % in_group) % gsz);
  pid_n = (tile % in_group) / gsz;
}

__device__ __forceinline__ float apply_act(float v, int act) {
  return (act == B200_ACT_LEAKY_RELU) ? (v >= 0.f ? v : 0.01f * v) : v;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
            const GemmParams p) {
  constexpr uint32_t A_BYTES = BM * KBYTES, B_BYTES = BN * KBYTES, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 128);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
        int pid_m, pid_n;
        tile_coords(p, tile, pid_m, pid_n);
        const int m0 = pid_m * BM, n0 = pid_n * BN;
        for (int kb = 0; kb < p.num_k; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
          mbar_wait(&empty[s], ph ^ 1u, p.status, SITE_GEMM_EMPTY);
          mbar_expect_tx(&full[s], STAGE_BYTES);
          uint8_t* a_dst = smem + s * STAGE_BYTES;
          uint8_t* b_dst = a_dst + A_BYTES;
          const int k0 = kb * p.bk_elems;
          if (!p.ga.mn_major) {
            tma_load_2d(a_dst, &tma_a, &full[s], k0, m0);
          } else {
            for (uint32_t b = 0; b < p.ga.nbox; ++b)
              tma_load_2d(a_dst + b * p.ga.box_bytes, &tma_a, &full[s], m0 + b * p.ga.box_mn, k0);
          }
          if (!p.gb.mn_major) {
            tma_load_2d(b_dst, &tma_b, &full[s], k0, n0);
          } else {
            for (uint32_t b = 0; b < p.gb.nbox; ++b)
              tma_load_2d(b_dst + b * p.gb.box_bytes, &tma_b, &full[s], n0 + b * p.gb.box_mn, k0);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, ti = 0;
      for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++ti) {
        const uint32_t acc = ti & 1u;
        mbar_wait(&tmem_empty[acc], ((ti >> 1) & 1u) ^ 1u, p.status, SITE_GEMM_TMEM_EMPTY);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.num_k; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
          mbar_wait(&full[s], ph, p.status, SITE_GEMM_FULL);
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < KBYTES / 32; ++k) {
            const uint64_t da = smem_desc_sw128(a_addr + k * p.ga.kstep_bytes, p.ga.lbo, p.ga.sbo);
            const uint64_t db = smem_desc_sw128(b_addr + k * p.gb.kstep_bytes, p.gb.lbo, p.gb.sbo);
            const uint32_t accum = (kb | k) != 0 ? 1u : 0u;
            if (p.fp8)
              umma_ss<true>(d_tmem, da, db, p.idesc, accum);
            else
              umma_ss<false>(d_tmem, da, db, p.idesc, accum);
          }
          tc_commit(&empty[s]);
        }
        tc_commit(&tmem_full[acc]);
      }
    }
    __syncwarp();
  } else {
    const uint32_t quarter = warp & 3u;  // TMEM lanes this warp may read: [32*quarter, 32*quarter+32)
    float scale = 1.f;
    if (p.scale_a) scale *= __ldg(p.scale_a);
    if (p.scale_b) scale *= __ldg(p.scale_b);
    const int esize = (p.out_dtype == B200_F32) ? 4 : 2;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0) && (((p.ldc * esize) & 15) == 0);
    uint32_t ti = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++ti) {
      int pid_m, pid_n;
      tile_coords(p, tile, pid_m, pid_n);
      const uint32_t acc = ti & 1u;
      mbar_wait(&tmem_full[acc], (ti >> 1) & 1u, p.status, SITE_GEMM_TMEM_FULL);
      tc_fence_after();
      const int row = pid_m * BM + quarter * 32 + lane;
      const int n0 = pid_n * BN;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((quarter * 32u) << 16) + acc * BN + c0, r);
        tmem_ld_wait();
        if (row < p.M) {
          const int col = n0 + c0;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = apply_act(__uint_as_float(r[j]) * scale, p.activation);
          if (p.out_dtype == B200_F32) {
            float* dst = reinterpret_cast<float*>(p.c) + (long long)row * p.ldc + col;
            if (vec_ok && col + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                reinterpret_cast<float4*>(dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            } else {
              for (int j = 0; j < 32; ++j)
                if (col + j < p.N) dst[j] = v[j];
            }
          } else {
            uint32_t w[16];
            if (p.out_dtype == B200_BF16) {
#pragma unroll
              for (int j = 0; j < 16; ++j) w[j] = pack2<true>(v[2 * j], v[2 * j + 1]);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) w[j] = pack2<false>(v[2 * j], v[2 * j + 1]);
            }
            uint16_t* dst = reinterpret_cast<uint16_t*>(p.c) + (long long)row * p.ldc + col;
            if (vec_ok && col + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                reinterpret_cast<uint4*>(dst)[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
            } else {
              for (int j = 0; j < 32; ++j)
                if (col + j < p.N) dst[j] = (uint16_t)((j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xFFFFu));
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tmem_empty[acc]);
    }
  }

  // teardown: after a recorded failure give copies in flight time to land before the CTA exits
  if (*(volatile unsigned*)p.status != 0) __nanosleep(100000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, int STAGES>
constexpr size_t gemm_smem_bytes() {
  return (size_t)STAGES * (BM * KBYTES + BN * KBYTES) + (2 * STAGES + 4) * 8 + 16 + 1024;
}

OperandGeom make_geom(bool mn_major, int rows, int elt, int bk_elems) {
  OperandGeom g{};
  g.mn_major = mn_major ? 1u : 0u;
  if (!mn_major) {
    g.nbox = 1;
    g.box_bytes = rows * KBYTES;
    g.box_mn = rows;
    g.lbo = 0;
    g.sbo = 1024;
    g.kstep_bytes = 32;
  } else {
    g.box_mn = 128 / elt;
    g.nbox = rows / g.box_mn;
    g.box_bytes = bk_elems * 128;
    g.lbo = g.box_bytes;
    g.sbo = 1024;
    g.kstep_bytes = (32 / elt) * 128;
  }
  return g;
}

template <int BN, int STAGES>
int launch_bn(DeviceCtx* ctx, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb_, GemmParams& p) {
  static bool attr_done[64] = {};
  constexpr size_t smem = gemm_smem_bytes<BN, STAGES>();
  if (ctx->device < 64 && !attr_done[ctx->device]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(B200_ERR_CUDA, "cudaFuncSetAttribute(gemm): %s", cudaGetErrorString(e));
    attr_done[ctx->device] = true;
  }
  const int grid = p.num_tiles < ctx->sm_count ? p.num_tiles : ctx->sm_count;
  gemm_kernel<BN, STAGES><<<grid, GEMM_THREADS, smem, stream>>>(ta, tb_, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "gemm launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

}  // namespace

int launch_gemm(DeviceCtx* ctx, cudaStream_t stream, const void* a, const void* b, void* c, int M, int N, int K,
                int64_t sam, int64_t sak, int64_t sbk, int64_t sbn, int64_t scm, int in_dtype, int out_dtype,
                int activation, const float* scale_a, const float* scale_b) {
  const int elt = dtype_bytes(in_dtype);
  const int bk_elems = KBYTES / elt;
  const bool a_mn = !(sak == 1 || K == 1) ? true : false;   // K contiguous preferred
  const bool b_mn = !(sbk == 1 || K == 1) ? true : false;
  if (a_mn && sam != 1 && M != 1) return fail(B200_ERR_UNSUPPORTED, "A must have a unit stride in M or K");
  if (b_mn && sbn != 1 && N != 1) return fail(B200_ERR_UNSUPPORTED, "B must have a unit stride in K or N");

  // tile width: the widest whose tile count still fills the SMs
  const int num_pid_m = (M + BM - 1) / BM;
  int bn = 64;
  for (int cand : {256, 128}) {
    if ((long long)num_pid_m * ((N + cand - 1) / cand) >= ctx->sm_count) { bn = cand; break; }
  }
  if (elt == 1 && b_mn && bn < 128) bn = 128;  // an MN-major box is 128 columns of 1-byte elements

  GemmParams p{};
  p.c = c; p.M = M; p.N = N; p.K = K; p.ldc = scm;
  p.out_dtype = out_dtype; p.activation = activation; p.fp8 = (in_dtype == B200_E4M3);
  p.scale_a = scale_a; p.scale_b = scale_b; p.status = ctx->status;
  p.num_pid_m = num_pid_m; p.num_pid_n = (N + bn - 1) / bn;
  p.num_tiles = p.num_pid_m * p.num_pid_n;
  p.num_k = (K + bk_elems - 1) / bk_elems;
  p.bk_elems = bk_elems;
  const int fmt = (in_dtype == B200_BF16) ? 1 : 0;  // kind::f16: f16 = 0, bf16 = 1; kind::f8f6f4: e4m3 = 0
  p.idesc = make_idesc(fmt, fmt, a_mn, b_mn, BM, bn);
  p.ga = make_geom(a_mn, BM, elt, bk_elems);
  p.gb = make_geom(b_mn, bn, elt, bk_elems);

  CUtensorMap ta, tbm;
  {
    uint64_t dims[2], strides[1];
    uint32_t box[2];
    if (!a_mn) { dims[0] = K; dims[1] = M; strides[0] = (uint64_t)sam * elt; box[0] = bk_elems; box[1] = BM; }
    else       { dims[0] = M; dims[1] = K; strides[0] = (uint64_t)sak * elt; box[0] = p.ga.box_mn; box[1] = bk_elems; }
    if (dims[1] == 1) strides[0] = (uint64_t)dims[0] * elt;
    if (!encode_tmap(&ta, in_dtype, 2, a, dims, strides, box, true)) return B200_ERR_UNSUPPORTED;
    if (!b_mn) { dims[0] = K; dims[1] = N; strides[0] = (uint64_t)sbn * elt; box[0] = bk_elems; box[1] = bn; }
    else       { dims[0] = N; dims[1] = K; strides[0] = (uint64_t)sbk * elt; box[0] = p.gb.box_mn; box[1] = bk_elems; }
    if (dims[1] == 1) strides[0] = (uint64_t)dims[0] * elt;
    if (!encode_tmap(&tbm, in_dtype, 2, b, dims, strides, box, true)) return B200_ERR_UNSUPPORTED;
  }
  switch (bn) {
    case 256: return launch_bn<256, 4>(ctx, stream, ta, tbm, p);
    case 128: return launch_bn<128, 6>(ctx, stream, ta, tbm, p);
    default: return launch_bn<64, 8>(ctx, stream, ta, tbm, p);
  }
}

}  // namespace tb
