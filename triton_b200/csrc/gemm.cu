// Persistent, warp-specialised tiled matmul for sm_100a.
//
// Computes what the reference's matmul_kernel computes (python/tutorials/03-matrix-
// multiplication.py:241-316; fp8 variant python/test/unit/language/test_core.py:5110-5140):
// C = act(scale * A @ B), fp32 accumulation, one rounding to the output type, program ids
// mapped to tiles in groups of tile-rows (03-...py:265-273).  The reference's persistent
// variants (python/tutorials/09-persistent-matmul.py:141-309) are the model for the structure:
// one CTA per SM walks tiles `tile += gridDim.x`.
//
// Tile shapes
//   128 x {64,128,256}   one CTA, two TMEM accumulators: the epilogue of tile i overlaps the main
//                        loop of tile i+1
//   256 x 256            one CTA, two 128-row MMAs per K step sharing the B stage, one accumulator
//                        set; a third less shared-memory fill traffic per flop (the default for
//                        large problems)
//   256 x 256 / 256 x 512 (pair)  two CTAs of a cluster (cta_group::2): each stages 128 rows of A
//                        and 128 columns of B per 256-column MMA, the leader issues 256 x 256 MMAs
//                        that read both CTAs' shared memory; selectable with B200_GEMM_TILE
// What bounds the big shapes is the L2 -> shared-memory fill (bytes per flop), not the tensor
// pipe, hence the preference for 256-row tiles when the problem has enough of them.
//
// Structure of one CTA (64 + 128 threads per 128 tile rows, plus one warp for the 256-row tile):
//   warp 0      TMA producer: fills a ring of shared-memory stages (128-byte swizzle) and signals
//               `full[s]` through the copy's byte count
//   warp 1      MMA issuer: one thread issues tcgen05.mma (32 bytes of K per instruction) into a
//               TMEM accumulator; tcgen05.commit releases the stage (`empty[s]`) and, after the
//               last K block, publishes the accumulator (`tmem_full[acc]`).  The 256-row tile has
//               a second issuing thread (last warp) for its lower 128 rows
//   warps 2..   epilogue: tcgen05.ld the accumulator (each warp owns 32 TMEM lanes = 32 rows),
//               scale / activation / convert, store C, then hand the accumulator back
//               (`tmem_empty[acc]`)
// Out-of-range rows / columns / K are zero-filled by TMA, which is the masked load of the
// reference (03-...py:297-298); stores are bounds-checked.
#include <cuda_fp8.h>

#include <cstdlib>
#include <type_traits>
#include <vector>

#include "common.cuh"
#include "host.h"

namespace tb {

namespace {

constexpr int KBYTES = 128;  // bytes of K per stage row = swizzle span

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
  int group_m;  // tile rows per rasterisation group (the reference's GROUP_SIZE_M)
  int c_tma;    // C is written through shared-memory staging + TMA stores (16-bit outputs TMA can address)
  int splits;   // split-K: work items = tiles x splits, each writes an fp32 partial tile to `ws`
  int kb_per_split;
  float* ws;    // [splits][M][N] fp32 partial sums (caller's workspace), reduced by splitk_reduce_kernel
  const void* bias;  // epilogue addend of the output type: [M,N] matrix, one value per row, or one per column
  int bias_mode;     // b200_bias
  long long bias_sm, bias_sn;
  uint32_t idesc;
  OperandGeom ga, gb;
  // chain-dot (gemm_chain_kernel): second product with W
  int in_bf16;       // 16-bit input type: 0 fp16, 1 bf16
  uint32_t idesc2;   // Z (TMEM) x W
  OperandGeom gw;
};

__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& pid_m, int& pid_n) {
  const int in_group = p.group_m * p.num_pid_n;
  const int group_id = tile / in_group;
  const int first_m = group_id * p.group_m;
  const int gsz = min(p.num_pid_m - first_m, p.group_m);
  pid_m = first_m + ((tile % in_group) % gsz);
  pid_n = (tile % in_group) / gsz;
}

__device__ __forceinline__ float apply_act(float v, int act) {
  return (act == B200_ACT_LEAKY_RELU) ? (v >= 0.f ? v : 0.01f * v) : v;
}

// value -> nearest value of the output type, as fp32
__device__ __forceinline__ float round_out(float v, int out_dtype) {
  if (out_dtype == B200_F16) return __half2float(__float2half_rn(v));
  if (out_dtype == B200_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  return v;
}
// The reference's bias epilogues (python/test/unit/hopper/test_gemm.py:213-222) convert the
// accumulator to the output type first and add the bias in that type: round, add, round again
// (the second rounding is the caller's final conversion).
__device__ __forceinline__ float add_bias(const GemmParams& p, float v, int row, int col) {
  if (row >= p.M || col >= p.N) return v;  // lanes past the edge compute values that are never stored
  long long i = 0;
  if (p.bias_mode != B200_BIAS_COLS) i += (long long)row * p.bias_sm;
  if (p.bias_mode != B200_BIAS_ROWS) i += (long long)col * p.bias_sn;
  float b;
  if (p.out_dtype == B200_F16) b = __half2float(reinterpret_cast<const __half*>(p.bias)[i]);
  else if (p.out_dtype == B200_BF16) b = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[i]);
  else b = reinterpret_cast<const float*>(p.bias)[i];
  return round_out(v, p.out_dtype) + b;
}
// accumulator -> scale, activation, bias: the fp32 value that is rounded once to the output type.
// BIAS is a template parameter so that the code without a bias is exactly the plain epilogue.
template <bool BIAS>
__device__ __forceinline__ float finish(const GemmParams& p, float acc, float scale, int row, int col) {
  const float v = apply_act(acc * scale, p.activation);
  if constexpr (BIAS) return add_bias(p, v, row, col);
  else return v;
}
// four fp32 -> four e4m3 bytes (round to nearest even, saturating at +-448 like the reference's
// cvt.rn.satfinite lowering of `.to(tl.float8e4nv)`)
__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// one thread's 32 consecutive accumulator columns -> scale, activation, one rounding, store
// EXT: the instantiation also knows the 8-bit output (kept out of the plain kernels, whose register
// allocation and speed it would otherwise change)
template <bool BIAS, bool EXT>
__device__ __forceinline__ void store_chunk32(const GemmParams& p, int row, int col, const uint32_t* r, float scale,
                                              bool vec_ok) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = finish<BIAS>(p, __uint_as_float(r[j]), scale, row, col + j);
  if (EXT && p.out_dtype == B200_E4M3) {
    uint8_t* dst = reinterpret_cast<uint8_t*>(p.c) + (long long)row * p.ldc + col;
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j] = pack4_e4m3(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    if (vec_ok && col + 32 <= p.N) {
      reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
      reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
      for (int j = 0; j < 32; ++j)
        if (col + j < p.N) dst[j] = (uint8_t)(w[j >> 2] >> (8 * (j & 3)));
    }
  } else if (p.out_dtype == B200_F32) {
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


constexpr int STG_BYTES = 32 * 128;  // staging of one epilogue warp: 32 rows x 64 columns of 16 bit
constexpr int kMaxSmem = 232448;     // dynamic shared memory one CTA can opt in to on sm_100
// epilogue staging buffers of the pair kernel: only where they fit beside the stages (the 7-stage
// 256 x 256 configuration keeps direct stores; its two accumulators hide the epilogue anyway)
constexpr int pair_staging_warps(int stages, int nb) {
  return (stages * (128 + 128 * nb) * 128 + 4 * STG_BYTES + 2048 <= kMaxSmem) ? 4 : 0;
}

// One epilogue warp drains `ncols` accumulator columns of its 32 TMEM lanes (rows row0 .. row0+31 of C,
// columns col0 ..).  Fast path: 64 columns at a time are converted, written to the warp's swizzled
// staging buffer and stored by TMA (full 128-byte lines, clipped at the matrix edge by the hardware);
// a warp-wide store of one row each would touch 32 separate lines per instruction and made the
// epilogue cost 9 % of a 256 x 256 tile.  Other outputs (fp32, or a C that TMA cannot address) take
// direct stores.
template <bool BIAS, bool EXT, class Release>
__device__ __forceinline__ void drain_accumulator_t(const GemmParams& p, const CUtensorMap* tma_c, uint8_t* stg,
                                                    uint32_t taddr, int ncols, int row0, int col0, int lane,
                                                    float scale, bool vec_ok, Release&& release_accumulator) {
  if (p.c_tma) {
    // The conversions dominate this path (256 values per thread and tile, two epilogue warps per
    // scheduler), so the activation and the output type are compile-time constants inside it: scale,
    // (activation,) convert, nothing else per value.
    auto tma_path = [&](auto leaky_tag, auto bf16_tag) {
    constexpr bool LEAKY = decltype(leaky_tag)::value, OUT_BF16 = decltype(bf16_tag)::value;
    // one TMA store of 32 rows x 64 columns through the warp's staging buffer; `word(j)` gives packed
    // word j (columns 2j, 2j+1) of this lane's row
    auto emit = [&](auto&& word, int c0) {
      if (lane == 0) tma_store_wait_read<0>();  // the previous store has read the staging buffer
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(stg + sw128_offset(lane, c)) = make_uint4(word(4 * c), word(4 * c + 1), word(4 * c + 2), word(4 * c + 3));
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && row0 < p.M && col0 + c0 < p.N) {
        tma_store_2d(tma_c, stg, col0 + c0, row0);
        tma_store_commit();
      }
    };
    // packed word j of the 64 fp32 columns in r that start at column c0 of the tile
    auto pack_word = [&](const uint32_t* r, int c0, int j) {
      float v0 = __uint_as_float(r[2 * j]) * scale, v1 = __uint_as_float(r[2 * j + 1]) * scale;
      if constexpr (LEAKY) {
        v0 = v0 >= 0.f ? v0 : 0.01f * v0;
        v1 = v1 >= 0.f ? v1 : 0.01f * v1;
      }
      if constexpr (BIAS) {
        v0 = add_bias(p, v0, row0 + lane, col0 + c0 + 2 * j);
        v1 = add_bias(p, v1, row0 + lane, col0 + c0 + 2 * j + 1);
      }
      return pack2<OUT_BF16>(v0, v1);
    };
    if (ncols == 256) {
      // A 256-column accumulator has no second buffer, so the MMA warps wait for this drain, and a
      // store cannot reuse the staging buffer before the previous one has read it.  So the
      // accumulator is emptied into registers first: three of the four 64-column groups are packed
      // to the output type and kept (96 registers, 32 columns in flight at a time), the fourth goes
      // to the staging buffer, and the accumulator is released after its last TMEM load; the
      // stores run under the next tile's MMAs.
      uint32_t k1[32], k2[32], k3[32];
      auto load_pack = [&](int c0, uint32_t* k) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          tmem_ld32(taddr + c0 + 32 * h, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) k[16 * h + j] = pack_word(r, c0 + 32 * h, j);
        }
      };
      load_pack(64, k1);
      load_pack(128, k2);
      load_pack(192, k3);
      {
        uint32_t r[32];
        tmem_ld32(taddr, r);
        tmem_ld_wait();
        if (lane == 0) tma_store_wait_read<0>();  // the previous tile's last store has read the staging buffer
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<uint4*>(stg + sw128_offset(lane, c)) =
              make_uint4(pack_word(r, 0, 4 * c), pack_word(r, 0, 4 * c + 1), pack_word(r, 0, 4 * c + 2), pack_word(r, 0, 4 * c + 3));
        tmem_ld32(taddr + 32, r);
        tmem_ld_wait();
        release_accumulator();
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<uint4*>(stg + sw128_offset(lane, 4 + c)) =
              make_uint4(pack_word(r, 32, 4 * c), pack_word(r, 32, 4 * c + 1), pack_word(r, 32, 4 * c + 2), pack_word(r, 32, 4 * c + 3));
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && row0 < p.M && col0 < p.N) {
          tma_store_2d(tma_c, stg, col0, row0);
          tma_store_commit();
        }
      }
      emit([&](int j) { return k1[j]; }, 64);
      emit([&](int j) { return k2[j]; }, 128);
      emit([&](int j) { return k3[j]; }, 192);
      return;
    }
#pragma unroll 1
    for (int c0 = 0; c0 < ncols; c0 += 64) {
      uint32_t r[64];
      tmem_ld32(taddr + c0, r);
      tmem_ld32(taddr + c0 + 32, r + 32);
      tmem_ld_wait();
      if (c0 + 64 >= ncols) release_accumulator();
      emit([&](int j) { return pack_word(r, c0, j); }, c0);
    }
    };
    const bool leaky = p.activation == B200_ACT_LEAKY_RELU, bf = p.out_dtype == B200_BF16;
    if (leaky) {
      if (bf) tma_path(std::true_type{}, std::true_type{});
      else tma_path(std::true_type{}, std::false_type{});
    } else {
      if (bf) tma_path(std::false_type{}, std::true_type{});
      else tma_path(std::false_type{}, std::false_type{});
    }
  } else {
    const int row = row0 + lane;
#pragma unroll 1
    for (int c0 = 0; c0 < ncols; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(taddr + c0, r);
      tmem_ld_wait();
      if (row < p.M) store_chunk32<BIAS, EXT>(p, row, col0 + c0, r, scale, vec_ok);
    }
    release_accumulator();
  }
}

// Drains one warp's part of an accumulator and calls `release` (every thread, once) as soon as the
// last TMEM load has completed, which on the TMA-store path is before the last stores: the caller
// passes what tells the MMA warp that the accumulator may be overwritten.
template <bool EXT, class Release>
__device__ __forceinline__ void drain_accumulator(const GemmParams& p, const CUtensorMap* tma_c, uint8_t* stg,
                                                  uint32_t taddr, int ncols, int row0, int col0, int lane,
                                                  float scale, bool vec_ok, Release&& release) {
  if constexpr (EXT) {
    if (p.bias_mode) drain_accumulator_t<true, true>(p, tma_c, stg, taddr, ncols, row0, col0, lane, scale, vec_ok, release);
    else drain_accumulator_t<false, true>(p, tma_c, stg, taddr, ncols, row0, col0, lane, scale, vec_ok, release);
  } else {
    drain_accumulator_t<false, false>(p, tma_c, stg, taddr, ncols, row0, col0, lane, scale, vec_ok, release);
  }
}

// Row-softmax epilogue (python/test/unit/hopper/test_gemm.py:223-228, 'softmax'): the whole row is
// in this tile (N <= tile width), one thread per row.  As the reference: z = out_type(acc);
// z -= max(z) in the output type; num = out_type(exp(fp32(z))); z = num / sum(num).  Three passes
// over the accumulator in TMEM (maximum, sum, write).
__device__ __forceinline__ void drain_softmax(const GemmParams& p, uint32_t taddr, int row0, int lane, float scale) {
  const int row = row0 + lane;
  const int nchunks = (p.N + 31) / 32;
  float mx = -INFINITY;
  for (int ch = 0; ch < nchunks; ++ch) {
    uint32_t r[32];
    tmem_ld32(taddr + ch * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (ch * 32 + j < p.N) mx = fmaxf(mx, round_out(__uint_as_float(r[j]) * scale, p.out_dtype));
  }
  float den = 0.f;
  for (int ch = 0; ch < nchunks; ++ch) {
    uint32_t r[32];
    tmem_ld32(taddr + ch * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (ch * 32 + j < p.N) {
        const float z = round_out(round_out(__uint_as_float(r[j]) * scale, p.out_dtype) - mx, p.out_dtype);
        den += round_out(__expf(z), p.out_dtype);
      }
  }
  den = round_out(den, p.out_dtype);
  for (int ch = 0; ch < nchunks; ++ch) {
    uint32_t r[32];
    tmem_ld32(taddr + ch * 32, r);
    tmem_ld_wait();
    if (row >= p.M) continue;
#pragma unroll 4
    for (int j = 0; j < 32; ++j) {
      const int col = ch * 32 + j;
      if (col >= p.N) break;
      const float z = round_out(round_out(__uint_as_float(r[j]) * scale, p.out_dtype) - mx, p.out_dtype);
      const float v = round_out(__expf(z), p.out_dtype) / den;
      const long long o = (long long)row * p.ldc + col;
      if (p.out_dtype == B200_F32) reinterpret_cast<float*>(p.c)[o] = v;
      else if (p.out_dtype == B200_BF16) reinterpret_cast<__nv_bfloat16*>(p.c)[o] = __float2bfloat16_rn(v);
      else reinterpret_cast<__half*>(p.c)[o] = __float2half_rn(v);
    }
  }
}

// split-K: one epilogue warp writes its 32 rows of raw fp32 partial sums to a dense [M][N] slice
__device__ __forceinline__ void drain_partial(float* ws, int M, int N, uint32_t taddr, int ncols, int row0, int col0,
                                              int lane) {
  const int row = row0 + lane;
  const bool vec_ok = (N & 3) == 0;  // the slice base is 16-byte aligned (checked on the host)
#pragma unroll 1
  for (int c0 = 0; c0 < ncols; c0 += 32) {
    uint32_t r[32];
    tmem_ld32(taddr + c0, r);
    tmem_ld_wait();
    if (row >= M) continue;
    const int col = col0 + c0;
    float* dst = ws + (long long)row * N + col;
    if (vec_ok && col + 32 <= N) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        reinterpret_cast<uint4*>(dst)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    } else {
      for (int j = 0; j < 32; ++j)
        if (col + j < N) dst[j] = __uint_as_float(r[j]);
    }
  }
}

// TMA boxes of one operand stage (2-D maps: K-major {k, row}; MN-major {row, k} in 128-byte column blocks)
template <bool PAIR>
__device__ __forceinline__ void load_operand(const OperandGeom& g, const CUtensorMap* map, uint8_t* dst, uint64_t* bar,
                                             int k0, int mn0) {
  if (!g.mn_major) {
    if constexpr (PAIR) tma_load_2d_pair(dst, map, bar, k0, mn0);
    else tma_load_2d(dst, map, bar, k0, mn0);
  } else {
    for (uint32_t b = 0; b < g.nbox; ++b) {
      if constexpr (PAIR) tma_load_2d_pair(dst + b * g.box_bytes, map, bar, mn0 + b * g.box_mn, k0);
      else tma_load_2d(dst + b * g.box_bytes, map, bar, mn0 + b * g.box_mn, k0);
    }
  }
}

// ------------------------------------------------------------------------------- single CTA
template <int BM, int BN, int STAGES, bool EXT>
__global__ void __launch_bounds__(64 + BM + (BM == 256 ? 32 : 0), 1)
gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
            const __grid_constant__ CUtensorMap tma_c, const GemmParams p) {
  constexpr uint32_t A_BYTES = BM * KBYTES, B_BYTES = BN * KBYTES, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));  // a power of two
  constexpr int MH = BM / 128;                  // 128-row MMAs per K step
  constexpr uint32_t NACC = (MH == 1) ? 2 : 1;  // accumulator sets in TMEM

  extern __shared__ uint8_t smem_raw[];
  const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  uint8_t* staging = smem + STAGES * STAGE_BYTES;  // one 4 KiB buffer per epilogue warp
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + (BM / 32) * STG_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  B200_TRACE_DECL;  // trace builds: region 0 = TMA warp, 1 / 2 = the issuing warps, 3 = first epilogue warp

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], MH);  // one commit per issuing thread
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], MH);
      mbar_init(&tmem_empty[i], BM);
    }
    if (p.c_tma) tma_prefetch_desc(&tma_c);
    fence_barrier_init();
    cta_wait_flag_clear();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  // The TMA warp initialised the barriers itself and needs nothing from the others (not the TMEM
  // base either): it only arrives at the CTA's start-up barrier and goes on to its first loads, which
  // are then in flight while TMEM is allocated and the other warps wait here.
  tc_fence_before();
  if (warp == 0) {
    __syncwarp();
    asm volatile("bar.arrive 1, %0;" ::"r"((int)blockDim.x) : "memory");
  } else {
    asm volatile("bar.sync 1, %0;" ::"r"((int)blockDim.x) : "memory");
  }
  tc_fence_after();
  const uint32_t tmem_base = (warp == 0) ? 0u : *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    // TMA producer.  The warp stays converged and every box of a stage has a lane of its own (K-major
    // operand: one box; MN-major: one per 128 bytes of M / N), so the loads of a stage go out as one
    // instruction instead of one after the other from a lone lane: the issue loop of this warp, not
    // the data, was what a short K loop waited for (one-wave problems: 0.33 us per K block).
    const uint32_t n_a = p.ga.mn_major ? p.ga.nbox : 1u, n_b = p.gb.mn_major ? p.gb.nbox : 1u;
    const bool has_box = (uint32_t)lane < n_a + n_b, is_b = (uint32_t)lane >= n_a;
    const uint32_t box = is_b ? lane - n_a : lane;
    const uint32_t mn_major = is_b ? p.gb.mn_major : p.ga.mn_major;
    const uint32_t dst_off = (is_b ? A_BYTES : 0u) + (mn_major ? box * (is_b ? p.gb.box_bytes : p.ga.box_bytes) : 0u);
    const int mn_off = mn_major ? (int)(box * (is_b ? p.gb.box_mn : p.ga.box_mn)) : 0;
    const CUtensorMap* map = is_b ? &tma_b : &tma_a;
    uint32_t s = 0, ph = 0;
    for (int work = blockIdx.x; work < p.num_tiles * p.splits; work += gridDim.x) {
      const int tile = work % p.num_tiles, split = work / p.num_tiles;
      int pid_m, pid_n;
      tile_coords(p, tile, pid_m, pid_n);
      const int mn0 = (is_b ? pid_n * BN : pid_m * BM) + mn_off;
      const int kb_end = min(p.num_k, (split + 1) * p.kb_per_split);
      for (int kb = split * p.kb_per_split; kb < kb_end; ++kb) {
        if (lane == 0) B200_TRACE_EVENT(p.status, 0, 1);
        mbar_wait(&empty[s], ph ^ 1u, p.status, SITE_GEMM_EMPTY);
        if (lane == 0) B200_TRACE_EVENT(p.status, 0, 2);
        if (lane == 0) mbar_expect_tx(&full[s], STAGE_BYTES);
        if (has_box) {
          const int k0 = kb * p.bk_elems;
          tma_load_2d(smem + s * STAGE_BYTES + dst_off, map, &full[s], mn_major ? mn0 : k0, mn_major ? k0 : mn0);
        }
        if (++s == STAGES) { s = 0; ph ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1 || (MH == 2 && warp == 2 + BM / 32)) {
    // One issuing thread per 128-row half of the tile (warp 1: rows 0-127, the last warp: rows
    // 128-255).  The halves have separate accumulators and share the B stage; while one thread
    // does its per-stage bookkeeping the other keeps the pipe fed (+3 % fp16, +4 % fp8 measured).
    const int h = (__shfl_sync(0xffffffffu, warp, 0) == 1) ? 0 : 1;  // warp-uniform for the compiler too
    {
      // The issue loop is kept lean (the tensor pipe queues only about one MMA ahead of the
      // issuer): the warp stays converged and an elected lane issues, so the descriptor
      // arithmetic is warp-uniform; a descriptor is a constant plus (address >> 4) in its low
      // bits, and stage / phase are running counters.
      const uint64_t da0 = smem_desc_sw128(smem_u32(smem), p.ga.lbo, p.ga.sbo);
      const uint64_t db0 = smem_desc_sw128(smem_u32(smem) + A_BYTES, p.gb.lbo, p.gb.sbo);
      const uint32_t ka = p.ga.kstep_bytes >> 4, kb16 = p.gb.kstep_bytes >> 4;
      const uint32_t idesc = p.idesc;
      const bool fp8 = p.fp8 != 0;
      uint32_t a_off[KBYTES / 32], b_off[KBYTES / 32];  // descriptor advance of the four K steps of a stage
#pragma unroll
      for (int k = 0; k < KBYTES / 32; ++k) {
        a_off[k] = h * ((128 * KBYTES) >> 4) + k * ka;
        b_off[k] = k * kb16;
      }
      uint32_t s = 0, ph = 0, ti = 0;
      for (int work = blockIdx.x; work < p.num_tiles * p.splits; work += gridDim.x, ++ti) {
        const int split = work / p.num_tiles;
        const int kb_cnt = min(p.num_k, (split + 1) * p.kb_per_split) - split * p.kb_per_split;
        const uint32_t acc = ti % NACC;
        if (lane == 0) B200_TRACE_EVENT(p.status, 1 + h, 0x10);
        mbar_wait(&tmem_empty[acc], ((ti / NACC) & 1u) ^ 1u, p.status, SITE_GEMM_TMEM_EMPTY);
        if (lane == 0) B200_TRACE_EVENT(p.status, 1 + h, 0x20);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN + h * BN;
        // the operand type is fixed outside the K loop: nothing between two MMAs but the descriptor sums
        auto k_loop = [&](auto fp8_tag) {
          constexpr bool F8 = decltype(fp8_tag)::value;
          uint32_t accum = 0;
          for (int kb = 0; kb < kb_cnt; ++kb) {
            if (lane == 0) B200_TRACE_EVENT(p.status, 1 + h, 1);
            mbar_wait(&full[s], ph, p.status, SITE_GEMM_FULL);  // TMA bytes landed
            if (lane == 0) B200_TRACE_EVENT(p.status, 1 + h, 2);
            const uint64_t das = da0 + s * (STAGE_BYTES >> 4), dbs = db0 + s * (STAGE_BYTES >> 4);
#pragma unroll
            for (int k = 0; k < KBYTES / 32; ++k)  // rows [128h, 128h+128) of A: 16 KiB apart
              umma_ss_elect<F8>(d_tmem, das + a_off[k], dbs + b_off[k], idesc, k == 0 ? accum : 1u);
            accum = 1;
            tc_commit_elect(&empty[s]);
            if (++s == STAGES) { s = 0; ph ^= 1u; }
          }
        };
        if (fp8) k_loop(std::true_type{});
        else k_loop(std::false_type{});
        tc_commit_elect(&tmem_full[acc]);
      }
    }
    __syncwarp();
  } else {
    const uint32_t quarter = warp & 3u;     // TMEM lanes this warp may read: [32*quarter, 32*quarter+32)
    const uint32_t half = (warp - 2) >> 2;  // which 128-row MMA of the tile this warp drains
    float scale = 1.f;
    if (p.scale_a) scale *= __ldg(p.scale_a);
    if (p.scale_b) scale *= __ldg(p.scale_b);
    const int esize = (p.out_dtype == B200_F32) ? 4 : (p.out_dtype == B200_E4M3 ? 1 : 2);
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0) && (((p.ldc * esize) & 15) == 0);
    uint32_t ti = 0;
    for (int work = blockIdx.x; work < p.num_tiles * p.splits; work += gridDim.x, ++ti) {
      const int tile = work % p.num_tiles, split = work / p.num_tiles;
      int pid_m, pid_n;
      tile_coords(p, tile, pid_m, pid_n);
      const uint32_t acc = ti % NACC;
      if (warp == 2 && lane == 0) B200_TRACE_EVENT(p.status, 3, 1);
      mbar_wait(&tmem_full[acc], (ti / NACC) & 1u, p.status, SITE_GEMM_TMEM_FULL);
      if (warp == 2 && lane == 0) B200_TRACE_EVENT(p.status, 3, 2);
      tc_fence_after();
      if (p.splits > 1) {
        // split-K: the raw fp32 partial sums go to this split's slice of the workspace
        drain_partial(p.ws + (long long)split * p.M * p.N, p.M, p.N,
                      tmem_base + ((quarter * 32u) << 16) + (acc + half) * BN, BN,
                      pid_m * BM + half * 128 + quarter * 32, pid_n * BN, lane);
      } else if (EXT && p.activation == B200_ACT_SOFTMAX) {
        drain_softmax(p, tmem_base + ((quarter * 32u) << 16) + (acc + half) * BN,
                      pid_m * BM + half * 128 + quarter * 32, lane, scale);
      } else
      {
        drain_accumulator<EXT>(p, &tma_c, staging + (warp - 2) * STG_BYTES,
                          tmem_base + ((quarter * 32u) << 16) + (acc + half) * BN, BN,
                          pid_m * BM + half * 128 + quarter * 32, pid_n * BN, lane, scale, vec_ok, [&]() {
                            tc_fence_before();
                            mbar_arrive(&tmem_empty[acc]);
                            if (warp == 2 && lane == 0) B200_TRACE_EVENT(p.status, 3, 3);
                          });
        continue;
      }
      tc_fence_before();
      mbar_arrive(&tmem_empty[acc]);
      if (warp == 2 && lane == 0) B200_TRACE_EVENT(p.status, 3, 3);
    }
    if (p.c_tma && lane == 0) tma_store_wait_read<0>();  // the staging buffer has been read: the CTA may exit, the writes land on their own
  }

  // teardown: after a recorded failure give copies in flight time to land before the CTA exits
  cta_linger_after_failure();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------- chain-dot
// C = out_type( in_type(out_type(A B)) W ), the reference's 'chain-dot' epilogue
// (python/test/unit/hopper/test_gemm.py:229-232): one 128-row tile per CTA spans all N <= 128
// columns of A B, whose rounded values go back into TMEM as the 16-bit A operand of a second
// product with W [N, N2 <= 128] (shared memory, loaded once), as P does in the attention kernels.
// TMEM: columns [0,128) A B, [128,192) Z (two values per column), [256,384) Z W.
// warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 conversion and epilogue.
template <int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_chain_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                  const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_c,
                  const GemmParams p) {
  constexpr int BM = 128, BN = 128;
  constexpr uint32_t A_BYTES = BM * KBYTES, B_BYTES = BN * KBYTES, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TM_ACC1 = 0, TM_Z = 128, TM_ACC2 = 256;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  uint8_t* sw = smem + STAGES * STAGE_BYTES;       // W: two K blocks of 64 rows
  uint8_t* staging = sw + 2 * B_BYTES;             // one 4 KiB buffer per epilogue warp
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + 4 * STG_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* w_full = empty + STAGES;
  uint64_t* acc1_full = w_full + 1;
  uint64_t* z_full = acc1_full + 1;
  uint64_t* acc2_full = z_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc2_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(w_full, 1);
    mbar_init(acc1_full, 1);
    mbar_init(z_full, 4);  // one arrival per conversion warp
    mbar_init(acc2_full, 1);
    fence_barrier_init();
    cta_wait_flag_clear();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    tma_prefetch_desc(&tma_w);
    if (p.c_tma) tma_prefetch_desc(&tma_c);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(w_full, 2 * B_BYTES);
      for (int kb = 0; kb < 2; ++kb) load_operand<false>(p.gw, &tma_w, sw + kb * B_BYTES, w_full, kb * p.bk_elems, 0);
      uint32_t s = 0, ph = 0;
      for (int kb = 0; kb < p.num_k; ++kb) {
        mbar_wait(&empty[s], ph ^ 1u, p.status, SITE_GEMM_EMPTY);
        mbar_expect_tx(&full[s], STAGE_BYTES);
        uint8_t* a_dst = smem + s * STAGE_BYTES;
        load_operand<false>(p.ga, &tma_a, a_dst, &full[s], kb * p.bk_elems, m0);
        load_operand<false>(p.gb, &tma_b, a_dst + A_BYTES, &full[s], kb * p.bk_elems, 0);
        if (++s == STAGES) { s = 0; ph ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    const uint64_t da0 = smem_desc_sw128(smem_u32(smem), p.ga.lbo, p.ga.sbo);
    const uint64_t db0 = smem_desc_sw128(smem_u32(smem) + A_BYTES, p.gb.lbo, p.gb.sbo);
    const uint64_t dw0 = smem_desc_sw128(smem_u32(sw), p.gw.lbo, p.gw.sbo);
    const uint32_t ka = p.ga.kstep_bytes >> 4, kb16 = p.gb.kstep_bytes >> 4, kw = p.gw.kstep_bytes >> 4;
    uint32_t s = 0, ph = 0, accum = 0;
    for (int kb = 0; kb < p.num_k; ++kb) {
      mbar_wait(&full[s], ph, p.status, SITE_GEMM_FULL);
      const uint64_t das = da0 + s * (STAGE_BYTES >> 4), dbs = db0 + s * (STAGE_BYTES >> 4);
#pragma unroll
      for (int k = 0; k < KBYTES / 32; ++k) {
        umma_ss_elect<false>(tmem_base + TM_ACC1, das + k * ka, dbs + k * kb16, p.idesc, accum);
        accum = 1;
      }
      tc_commit_elect(&empty[s]);
      if (++s == STAGES) { s = 0; ph ^= 1u; }
    }
    tc_commit_elect(acc1_full);
    // second product: Z (TMEM, 8 columns per 16 values of K) x W
    mbar_wait(w_full, 0, p.status, SITE_GEMM_FULL);
    mbar_wait(z_full, 0, p.status, SITE_GEMM_TMEM_EMPTY);
    tc_fence_after();
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)
      umma_ts_f16_elect(tmem_base + TM_ACC2, tmem_base + TM_Z + kk * 8, dw0 + (kk >> 2) * (B_BYTES >> 4) + (kk & 3) * kw,
                        p.idesc2, kk != 0);
    tc_commit_elect(acc2_full);
    __syncwarp();
  } else {
    const uint32_t quarter = warp & 3u;  // TMEM lanes this warp may access: [32*quarter, +32)
    const uint32_t lane_addr = (quarter * 32u) << 16;
    const int esize = (p.out_dtype == B200_F32) ? 4 : 2;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0) && (((p.ldc * esize) & 15) == 0);
    mbar_wait(acc1_full, 0, p.status, SITE_GEMM_TMEM_FULL);
    tc_fence_after();
    // z = out_type(acc), then the input type: the two roundings of the reference, in its order
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      uint32_t r[32], wv[16];
      tmem_ld32(tmem_base + TM_ACC1 + lane_addr + c, r);
      tmem_ld_wait();
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const float z0 = round_out(__uint_as_float(r[2 * k]), p.out_dtype);
        const float z1 = round_out(__uint_as_float(r[2 * k + 1]), p.out_dtype);
        wv[k] = p.in_bf16 ? pack2<true>(z0, z1) : pack2<false>(z0, z1);
      }
      tmem_st16(tmem_base + TM_Z + lane_addr + (c >> 1), wv);
    }
    tmem_st_wait();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(z_full);
    mbar_wait(acc2_full, 0, p.status, SITE_GEMM_TMEM_FULL);
    tc_fence_after();
    drain_accumulator<false>(p, &tma_c, staging + (warp - 2) * STG_BYTES, tmem_base + TM_ACC2 + lane_addr, BN,
                             m0 + quarter * 32, 0, lane, 1.f, vec_ok, []() {});
    if (p.c_tma && lane == 0) tma_store_wait_read<0>();
  }

  cta_linger_after_failure();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// --------------------------------------------------------------------------------- CTA pair
// Barriers: both producers credit the LEADER's full[s] (the peer through the leader's cluster
// address); the leader's tcgen05.commit is multicast to both CTAs' empty[s] / tmem_full[acc];
// the peer's epilogue warps arrive remotely on the leader's tmem_empty[acc].
template <int STAGES, int NB, bool EXT>
__global__ void __launch_bounds__(192, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_c, const GemmParams p) {
  // The pair's tile is 256 x (256 * NB).  Per K block each CTA stages its 128 rows of A and, for
  // each of the NB 256-column MMAs, its 128 columns of B.  NB = 2 needs a quarter less fill
  // traffic per flop and amortises the per-stage bookkeeping over eight MMAs, but its
  // accumulators fill TMEM, so the epilogue is not overlapped with the next tile.
  constexpr int BN = 256 * NB, HALF_N = 128;
  constexpr uint32_t A_BYTES = 128 * KBYTES, B_BYTES = NB * HALF_N * KBYTES, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t NACC = (NB == 1) ? 2 : 1;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  uint8_t* staging = smem + STAGES * STAGE_BYTES;  // one 4 KiB buffer per epilogue warp
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + pair_staging_warps(STAGES, NB) * STG_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  B200_TRACE_DECL;  // trace builds (leader of pair 0): region 0 = TMA warp, 1 = issuing warp, 3 = first epilogue warp

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);   // the leader's expect_tx arrival; bytes of both CTAs
      mbar_init(&empty[s], 1);  // one multicast commit
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 8);  // one arrival per epilogue warp of both CTAs
    }
    fence_barrier_init();
    cta_wait_flag_clear();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    if (p.c_tma) tma_prefetch_desc(&tma_c);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      for (int tile = pair; tile < p.num_tiles; tile += num_pairs) {
        int pid_m, pid_n;
        tile_coords(p, tile, pid_m, pid_n);
        const int m0 = pid_m * 256 + rank * 128, n0 = pid_n * BN + rank * HALF_N;
        for (int kb = 0; kb < p.num_k; ++kb) {
          B200_TRACE_EVENT(p.status, 0, 1);
          mbar_wait(&empty[s], ph ^ 1u, p.status, SITE_GEMM_EMPTY);
          B200_TRACE_EVENT(p.status, 0, 2);
          if (rank == 0) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
          uint8_t* a_dst = smem + s * STAGE_BYTES;
          load_operand<true>(p.ga, &tma_a, a_dst, &full[s], kb * p.bk_elems, m0);
#pragma unroll
          for (int j = 0; j < NB; ++j)  // this CTA's 128 columns of the j-th 256-column MMA
            load_operand<true>(p.gb, &tma_b, a_dst + A_BYTES + j * (HALF_N * KBYTES), &full[s], kb * p.bk_elems,
                               n0 + j * 256);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (rank == 0) {  // the leader CTA's warp issues for the pair: converged, one elected lane
      const uint64_t da0 = smem_desc_sw128(smem_u32(smem), p.ga.lbo, p.ga.sbo);
      const uint64_t db0 = smem_desc_sw128(smem_u32(smem) + A_BYTES, p.gb.lbo, p.gb.sbo);
      const uint32_t ka = p.ga.kstep_bytes >> 4, kb16 = p.gb.kstep_bytes >> 4;
      const uint32_t idesc = p.idesc;
      const bool fp8 = p.fp8 != 0;
      uint32_t s = 0, ph = 0, ti = 0;
      for (int tile = pair; tile < p.num_tiles; tile += num_pairs, ++ti) {
        const uint32_t acc = ti % NACC;
        if (lane == 0) B200_TRACE_EVENT(p.status, 1, 0x10);
        mbar_wait(&tmem_empty[acc], ((ti / NACC) & 1u) ^ 1u, p.status, SITE_GEMM_TMEM_EMPTY);
        if (lane == 0) B200_TRACE_EVENT(p.status, 1, 0x20);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * 256;
        uint32_t accum = 0;
        for (int kb = 0; kb < p.num_k; ++kb) {
          if (lane == 0) B200_TRACE_EVENT(p.status, 1, 1);
          mbar_wait(&full[s], ph, p.status, SITE_GEMM_FULL);
          if (lane == 0) B200_TRACE_EVENT(p.status, 1, 2);
          const uint64_t das = da0 + s * (STAGE_BYTES >> 4), dbs = db0 + s * (STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < KBYTES / 32; ++k) {
#pragma unroll
            for (int j = 0; j < NB; ++j) {
              const uint64_t db = dbs + (j * ((HALF_N * KBYTES) >> 4) + k * kb16);
              if (fp8)
                umma_ss_pair_elect<true>(d_tmem + j * 256, das + k * ka, db, idesc, accum);
              else
                umma_ss_pair_elect<false>(d_tmem + j * 256, das + k * ka, db, idesc, accum);
            }
            accum = 1;
          }
          tc_commit_pair_elect(&empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        tc_commit_pair_elect(&tmem_full[acc]);
      }
    }
    __syncwarp();
  } else {
    const uint32_t quarter = warp & 3u;
    float scale = 1.f;
    if (p.scale_a) scale *= __ldg(p.scale_a);
    if (p.scale_b) scale *= __ldg(p.scale_b);
    const int esize = (p.out_dtype == B200_F32) ? 4 : (p.out_dtype == B200_E4M3 ? 1 : 2);
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0) && (((p.ldc * esize) & 15) == 0);
    uint32_t ti = 0;
    for (int tile = pair; tile < p.num_tiles; tile += num_pairs, ++ti) {
      int pid_m, pid_n;
      tile_coords(p, tile, pid_m, pid_n);
      const uint32_t acc = ti % NACC;
      if (warp == 2 && lane == 0) B200_TRACE_EVENT(p.status, 3, 1);
      mbar_wait(&tmem_full[acc], (ti / NACC) & 1u, p.status, SITE_GEMM_TMEM_FULL);
      if (warp == 2 && lane == 0) B200_TRACE_EVENT(p.status, 3, 2);
      tc_fence_after();
      drain_accumulator<EXT>(p, &tma_c, staging + (warp - 2) * STG_BYTES,
                        tmem_base + ((quarter * 32u) << 16) + acc * 256, BN,
                        pid_m * 256 + rank * 128 + quarter * 32, pid_n * BN, lane, scale, vec_ok, [&]() {
                          tc_fence_before();
                          __syncwarp();
                          if (lane == 0) mbar_arrive_cluster(&tmem_empty[acc], 0);  // the leader's barrier
                          if (warp == 2 && lane == 0) B200_TRACE_EVENT(p.status, 3, 3);
                        });
    }
    if (p.c_tma && lane == 0) tma_store_wait_read<0>();
  }

  cta_linger_after_failure();
  tc_fence_before();
  cluster_sync();  // neither CTA may exit (or free TMEM) while its peer can still reach it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------ layouts TMA cannot address
// A base address that is not 16-byte aligned or a row stride that is not a multiple of 16 bytes
// (N = 257 fp16 columns, say) cannot be described by a tensor map.  The reference accepts any
// strides, so such calls take this plain CUDA-core kernel: same arithmetic (fp32 accumulation in
// K order per 16-wide slab, scale, activation, one rounding), no tensor cores, no speed claim.
__device__ __forceinline__ float load_elem(const void* base, long long idx, int dtype) {
  if (dtype == B200_F16) return __half2float(reinterpret_cast<const __half*>(base)[idx]);
  if (dtype == B200_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  // e4m3: sign, 4 exponent bits (bias 7), 3 mantissa bits; 0x7f / 0xff are NaN
  const uint32_t b = reinterpret_cast<const uint8_t*>(base)[idx];
  const uint32_t e = (b >> 3) & 0xFu, m = b & 7u;
  float v;
  if (e == 0) v = (float)m * 0.001953125f;                       // m / 8 * 2^-6
  else if (e == 15 && m == 7) v = __int_as_float(0x7fc00000);
  else v = __int_as_float(((e + 120u) << 23) | (m << 20));        // (1 + m/8) * 2^(e-7)
  return (b & 0x80u) ? -v : v;
}

__global__ void __launch_bounds__(256)
gemm_plain_kernel(const void* a, const void* b, GemmParams p, long long sam, long long sak, long long sbk,
                  long long sbn, int in_dtype) {
  __shared__ float sa[16][64 + 1], sb[16][64 + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < p.K; k0 += 16) {
    for (int i = threadIdx.x; i < 16 * 64; i += 256) {
      const int kk = i & 15, mn = i >> 4;
      const int gm = m0 + mn, gn = n0 + mn, gk = k0 + kk;
      sa[kk][mn] = (gm < p.M && gk < p.K) ? load_elem(a, gm * sam + gk * sak, in_dtype) : 0.f;
      sb[kk][mn] = (gn < p.N && gk < p.K) ? load_elem(b, gk * sbk + gn * sbn, in_dtype) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { av[i] = sa[kk][ty * 4 + i]; bv[i] = sb[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  float scale = 1.f;
  if (p.scale_a) scale *= __ldg(p.scale_a);
  if (p.scale_b) scale *= __ldg(p.scale_b);
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= p.M) continue;
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= p.N) continue;
      const float v = p.bias_mode ? finish<true>(p, acc[i][j], scale, gm, gn) : finish<false>(p, acc[i][j], scale, gm, gn);
      const long long o = (long long)gm * p.ldc + gn;
      if (p.out_dtype == B200_E4M3) reinterpret_cast<uint8_t*>(p.c)[o] = (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
      else if (p.out_dtype == B200_F32) reinterpret_cast<float*>(p.c)[o] = v;
      else if (p.out_dtype == B200_BF16) reinterpret_cast<__nv_bfloat16*>(p.c)[o] = __float2bfloat16_rn(v);
      else reinterpret_cast<__half*>(p.c)[o] = __float2half_rn(v);
    }
  }
}

// split-K second pass: C = act(scale * sum over splits of the fp32 partial tiles), one rounding
template <int VEC>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(GemmParams p) {
  // one thread per VEC consecutive columns of a row (blockIdx.y strides over the rows), no division
  // per element.  VEC = 4 (16-byte loads) for large outputs, VEC = 1 for small ones, where more
  // threads hide more latency.  Four loads are in flight and are added in split order, so the sum
  // does not depend on timing.
  const long long total = (long long)p.M * p.N;
  float scale = 1.f;
  if (p.scale_a) scale *= __ldg(p.scale_a);
  if (p.scale_b) scale *= __ldg(p.scale_b);
  const int col = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (col >= p.N) return;
  for (int row = blockIdx.y; row < p.M; row += gridDim.y) {
    const long long i = (long long)row * p.N + col;
    float v[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) v[j] = 0.f;
    for (int sp = 0; sp < p.splits; sp += 4) {
      float t[4][VEC];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float* src = p.ws + (long long)(sp + u) * total + i;
        if (sp + u < p.splits) {
          if constexpr (VEC == 4) {
            const float4 q = *reinterpret_cast<const float4*>(src);
            t[u][0] = q.x; t[u][1] = q.y; t[u][2] = q.z; t[u][3] = q.w;
          } else {
            t[u][0] = *src;
          }
        } else {
#pragma unroll
          for (int j = 0; j < VEC; ++j) t[u][j] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < VEC; ++j) v[j] += t[u][j];
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float r = p.bias_mode ? finish<true>(p, v[j], scale, row, col + j) : finish<false>(p, v[j], scale, 0, 0);
      const long long o = (long long)row * p.ldc + col + j;
      if (p.out_dtype == B200_E4M3) reinterpret_cast<uint8_t*>(p.c)[o] = (uint8_t)__nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E4M3);
      else if (p.out_dtype == B200_F32) reinterpret_cast<float*>(p.c)[o] = r;
      else if (p.out_dtype == B200_BF16) reinterpret_cast<__nv_bfloat16*>(p.c)[o] = __float2bfloat16_rn(r);
      else reinterpret_cast<__half*>(p.c)[o] = __float2half_rn(r);
    }
  }
}

// ------------------------------------------------------------------------------------- grouped
// Grouped matmul (python/tutorials/08-grouped-gemm.py:64-141): several independent problems in one
// persistent launch.  The reference walks the groups on the device with a running tile count and
// reads pointers and sizes from device tensors; here each group has a descriptor in device memory
// (written by the host for this call) that also carries the group's three tensor maps, and every
// role warp walks the same tile sequence: tile t belongs to the group whose [tile_start,
// tile_start + num_tiles) contains it, tiles of a group in row-major order as in the reference.
// 128 x 128 tiles, two accumulators, so a group's epilogue overlaps the next tile's main loop even
// across a group boundary.  Partial tiles are zero-filled on load and clipped on store (the
// reference assumes full tiles).
struct alignas(128) GroupDesc {
  CUtensorMap ta, tb, tc;
  void* c;
  long long ldc;
  int M, N, num_k, num_pid_n, tile_start, num_tiles, c_tma, pad_;
};
static_assert(sizeof(GroupDesc) == 512, "GroupDesc is 512 bytes");

__device__ __forceinline__ int find_group(const GroupDesc* groups, int g, int tile) {
  while (tile >= groups[g].tile_start + groups[g].num_tiles) ++g;  // tiles only move forward
  return g;
}

template <int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_grouped_kernel(const GroupDesc* __restrict__ groups, int total_tiles, const GemmParams p) {
  constexpr int BM = 128, BN = 128;
  constexpr uint32_t A_BYTES = BM * KBYTES, B_BYTES = BN * KBYTES, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  uint8_t* staging = smem + STAGES * STAGE_BYTES;  // one 4 KiB buffer per epilogue warp
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + (BM / 32) * STG_BYTES);
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
      mbar_init(&tmem_empty[i], BM);
    }
    fence_barrier_init();
    cta_wait_flag_clear();
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
    // converged warp, one lane per TMA box of a stage (see gemm_kernel)
    const uint32_t n_a = p.ga.mn_major ? p.ga.nbox : 1u, n_b = p.gb.mn_major ? p.gb.nbox : 1u;
    const bool has_box = (uint32_t)lane < n_a + n_b, is_b = (uint32_t)lane >= n_a;
    const uint32_t box = is_b ? lane - n_a : lane;
    const uint32_t mn_major = is_b ? p.gb.mn_major : p.ga.mn_major;
    const uint32_t dst_off = (is_b ? A_BYTES : 0u) + (mn_major ? box * (is_b ? p.gb.box_bytes : p.ga.box_bytes) : 0u);
    const int mn_off = mn_major ? (int)(box * (is_b ? p.gb.box_mn : p.ga.box_mn)) : 0;
    uint32_t s = 0, ph = 0;
    int g = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      g = find_group(groups, g, tile);
      const GroupDesc* gd = groups + g;
      const int t = tile - gd->tile_start;
      const int mn0 = (is_b ? (t % gd->num_pid_n) * BN : (t / gd->num_pid_n) * BM) + mn_off;
      const CUtensorMap* map = is_b ? &gd->tb : &gd->ta;
      const int num_k = gd->num_k;
      for (int kb = 0; kb < num_k; ++kb) {
        mbar_wait(&empty[s], ph ^ 1u, p.status, SITE_GEMM_EMPTY);
        if (lane == 0) mbar_expect_tx(&full[s], STAGE_BYTES);
        if (has_box) {
          const int k0 = kb * p.bk_elems;
          tma_load_2d(smem + s * STAGE_BYTES + dst_off, map, &full[s], mn_major ? mn0 : k0, mn_major ? k0 : mn0);
        }
        if (++s == STAGES) { s = 0; ph ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    const uint64_t da0 = smem_desc_sw128(smem_u32(smem), p.ga.lbo, p.ga.sbo);
    const uint64_t db0 = smem_desc_sw128(smem_u32(smem) + A_BYTES, p.gb.lbo, p.gb.sbo);
    const uint32_t ka = p.ga.kstep_bytes >> 4, kb16 = p.gb.kstep_bytes >> 4;
    const uint32_t idesc = p.idesc;
    uint32_t s = 0, ph = 0, ti = 0;
    int g = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++ti) {
      g = find_group(groups, g, tile);
      const int num_k = groups[g].num_k;
      const uint32_t acc = ti & 1u;
      mbar_wait(&tmem_empty[acc], ((ti >> 1) & 1u) ^ 1u, p.status, SITE_GEMM_TMEM_EMPTY);
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      uint32_t accum = 0;
      for (int kb = 0; kb < num_k; ++kb) {
        mbar_wait(&full[s], ph, p.status, SITE_GEMM_FULL);
        const uint64_t das = da0 + s * (STAGE_BYTES >> 4), dbs = db0 + s * (STAGE_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < KBYTES / 32; ++k) {
          umma_ss_elect<false>(d_tmem, das + k * ka, dbs + k * kb16, idesc, accum);
          accum = 1;
        }
        tc_commit_elect(&empty[s]);
        if (++s == STAGES) { s = 0; ph ^= 1u; }
      }
      tc_commit_elect(&tmem_full[acc]);
    }
    __syncwarp();
  } else {
    const uint32_t quarter = warp & 3u;
    const int esize = (p.out_dtype == B200_F32) ? 4 : 2;
    uint32_t ti = 0;
    int g = 0;
    bool any_tma = false;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++ti) {
      g = find_group(groups, g, tile);
      const GroupDesc* gd = groups + g;
      const int t = tile - gd->tile_start;
      GemmParams q = p;  // the group's output replaces the common parameters' placeholders
      q.c = gd->c; q.ldc = gd->ldc; q.M = gd->M; q.N = gd->N; q.c_tma = gd->c_tma;
      any_tma |= q.c_tma != 0;
      const bool vec_ok = ((reinterpret_cast<uintptr_t>(q.c) & 15) == 0) && (((q.ldc * esize) & 15) == 0);
      const uint32_t acc = ti & 1u;
      mbar_wait(&tmem_full[acc], (ti >> 1) & 1u, p.status, SITE_GEMM_TMEM_FULL);
      tc_fence_after();
      drain_accumulator<false>(q, &gd->tc, staging + (warp - 2) * STG_BYTES,
                               tmem_base + ((quarter * 32u) << 16) + acc * BN, BN,
                               (t / gd->num_pid_n) * BM + quarter * 32, (t % gd->num_pid_n) * BN, lane, 1.f, vec_ok, [&]() {
                                 tc_fence_before();
                                 mbar_arrive(&tmem_empty[acc]);
                               });
    }
    if (any_tma && lane == 0) tma_store_wait_read<0>();
  }

  cta_linger_after_failure();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------- host
int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return v && *v ? atoi(v) : dflt;
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

constexpr size_t smem_bytes(int stages, int stage_bytes, int epilogue_warps) {
  return (size_t)stages * stage_bytes + (size_t)epilogue_warps * STG_BYTES + (2 * stages + 4) * 8 + 16 + 1024;
}

template <int BM, int BN, int STAGES, bool EXT>
int launch_tile_t(DeviceCtx* ctx, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb_, const CUtensorMap& tc,
                GemmParams& p) {
  static std::atomic<bool> attr_done[64];
  constexpr size_t smem = smem_bytes(STAGES, (BM + BN) * KBYTES, BM / 32);
  if (int rc = ensure_dynamic_smem(gemm_kernel<BM, BN, STAGES, EXT>, smem, ctx->device, attr_done, "gemm")) return rc;
  const int work = p.num_tiles * p.splits;
  const int grid = work < ctx->sm_count ? work : ctx->sm_count;
  gemm_kernel<BM, BN, STAGES, EXT><<<grid, 64 + BM + (BM == 256 ? 32 : 0), smem, stream>>>(ta, tb_, tc, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "gemm launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

template <int STAGES, int NB, bool EXT>
int launch_pair_t(DeviceCtx* ctx, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb_, const CUtensorMap& tc,
                GemmParams& p) {
  static std::atomic<bool> attr_done[64];
  constexpr size_t smem = smem_bytes(STAGES, (128 + 128 * NB) * KBYTES, pair_staging_warps(STAGES, NB));
  if (pair_staging_warps(STAGES, NB) == 0) p.c_tma = 0;
  if (int rc = ensure_dynamic_smem(gemm_pair_kernel<STAGES, NB, EXT>, smem, ctx->device, attr_done, "gemm pair")) return rc;
  int pairs = ctx->sm_count / 2;
  if (p.num_tiles < pairs) pairs = p.num_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<STAGES, NB, EXT>, ta, tb_, tc, p);
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "gemm pair launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

// the kernels with the bias and 8-bit-output epilogues are separate instantiations
template <int BM, int BN, int STAGES>
int launch_tile(DeviceCtx* ctx, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb_,
                const CUtensorMap& tc, GemmParams& p) {
  if (p.bias_mode || p.out_dtype == B200_E4M3 || p.activation == B200_ACT_SOFTMAX)
    return launch_tile_t<BM, BN, STAGES, true>(ctx, stream, ta, tb_, tc, p);
  return launch_tile_t<BM, BN, STAGES, false>(ctx, stream, ta, tb_, tc, p);
}
template <int STAGES, int NB>
int launch_pair(DeviceCtx* ctx, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb_,
                const CUtensorMap& tc, GemmParams& p) {
  if (p.bias_mode || p.out_dtype == B200_E4M3) return launch_pair_t<STAGES, NB, true>(ctx, stream, ta, tb_, tc, p);
  return launch_pair_t<STAGES, NB, false>(ctx, stream, ta, tb_, tc, p);
}

}  // namespace

// Split-K plan for skinny problems: when the chosen tile shape gives fewer than half as many tiles as
// there are SMs and K is long, the K range is cut so that about one wave of work items exists.
int gemm_plan_splits(DeviceCtx* ctx, int M, int N, int K, int in_dtype) {
  const int forced = env_int("B200_GEMM_SPLITK", -1);  // 0 or 1: never split; n > 1: that many splits
  if (forced >= 0) return forced < 1 ? 1 : (forced > 64 ? 64 : forced);
  const int bk_elems = KBYTES / dtype_bytes(in_dtype);
  const int num_k = (K + bk_elems - 1) / bk_elems;
  // skinny problems always end up on the 128 x 64 tile (most tiles)
  const long long tiles = (long long)((M + 127) / 128) * ((N + 63) / 64);
  // a second kernel and the workspace round trip cost a few microseconds: only long K loops pay
  if (tiles * 2 > ctx->sm_count || num_k < 32) return 1;
  long long s = ctx->sm_count / tiles;
  if (s > num_k / 8) s = num_k / 8;
  if (s > 16) s = 16;
  return s < 1 ? 1 : (int)s;
}

int launch_gemm(DeviceCtx* ctx, cudaStream_t stream, const void* a, const void* b, void* c, int M, int N, int K,
                int64_t sam, int64_t sak, int64_t sbk, int64_t sbn, int64_t scm, int in_dtype, int out_dtype,
                int activation, const float* scale_a, const float* scale_b, const void* bias, int bias_mode,
                int64_t bias_sm, int64_t bias_sn, int splits, float* ws) {
  const int elt = dtype_bytes(in_dtype);
  const int bk_elems = KBYTES / elt;
  const bool a_mn = !(sak == 1 || K == 1);  // K contiguous preferred
  const bool b_mn = !(sbk == 1 || K == 1);

  // Can TMA address A and B?  (C is written with plain stores and has no such limit.)
  // a single row (or column) has no row stride to speak of, but its base must still be aligned
  auto tma_ok = [&](const void* base, int64_t row_stride, int64_t rows) {
    return (reinterpret_cast<uintptr_t>(base) & 15) == 0 && (rows == 1 || ((row_stride * elt) & 15) == 0);
  };
  const bool a_ok = tma_ok(a, a_mn ? sak : sam, a_mn ? K : M);
  const bool b_ok = tma_ok(b, b_mn ? sbk : sbn, b_mn ? K : N);
  if (!a_ok || !b_ok || (a_mn && sam != 1) || (b_mn && sbn != 1) || env_int("B200_GEMM_PLAIN", 0)) {
    if (activation == B200_ACT_SOFTMAX)
      return fail(B200_ERR_UNSUPPORTED, "the softmax epilogue needs operands that TMA can address");
    GemmParams q{};
    q.c = c; q.M = M; q.N = N; q.K = K; q.ldc = scm;
    q.out_dtype = out_dtype; q.activation = activation;
    q.scale_a = scale_a; q.scale_b = scale_b;
    q.bias = bias; q.bias_mode = bias_mode; q.bias_sm = bias_sm; q.bias_sn = bias_sn;
    dim3 grid((N + 63) / 64, (M + 63) / 64, 1);
    gemm_plain_kernel<<<grid, 256, 0, stream>>>(a, b, q, sam, sak, sbk, sbn, in_dtype);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(B200_ERR_CUDA, "plain gemm launch: %s", cudaGetErrorString(e));
    return B200_OK;
  }

  // Tile shape.  B200_GEMM_TILE forces one: 128064, 128128, 128192, 128256, 256192, 256256, or 2256 / 2512 for the CTA pair
  // (256 x 256 / 256 x 512).
  auto tiles = [&](int bm_, int bn_) { return (long long)((M + bm_ - 1) / bm_) * ((N + bn_ - 1) / bn_); };
  int bm = 128, bn = 64;
  bool pair = false;
  const int force = env_int("B200_GEMM_TILE", 0);
  int pair_nb = 1;  // 256-column MMAs per pair tile
  if (activation == B200_ACT_SOFTMAX) {
    bm = 128; bn = N <= 64 ? 64 : (N <= 128 ? 128 : 256);  // one tile spans the row
  } else if (splits > 1) {
    bm = 128; bn = 64;  // split-K serves skinny problems: the shape with the most tiles
  } else if (force == 2256 || force == 2512) {
    pair = true;
    pair_nb = force == 2512 ? 2 : 1;
  } else if (force) {
    bm = force / 1000;
    bn = force % 1000;
  } else {
    // Pick the shape with the smallest estimated time: waves x (K blocks x time per K block + time
    // per tile).  The per-K-block times (us, one 128-byte K block, any operand type) are measured on
    // square fp16 problems from 1024 to 8192: the 128-row shapes are bound by the issue loops and,
    // with every SM busy, by the L2 -> shared-memory fill (a 128 x 256 tile draws 96 B/clk/SM), the
    // 256 x 256 shape by the tensor pipe; the per-tile time is the part of the epilogue and tile
    // turn-around that the next tile's main loop does not cover.  The model reproduces the measured
    // order of the shapes at every size of that sweep (e.g. 2304: 128 x 128 in three waves before
    // 256 x 256 in a 55 % wave; 3584: 128 x 256).  The pair shapes (`cta_group::2`) never won a size:
    // 256 x 256 on a pair has the fill traffic per flop of a 128 x 256 tile, 256 x 512 has no second
    // accumulator; they stay selectable through B200_GEMM_TILE.
    // (The 192-column shapes exist for the wave count: 2560^3 is 100 tiles of 256 x 256 - two thirds
    // of the SMs - or 400 of 128 x 128 - 2.7 waves - but 140 of 256 x 192, one full wave.  They need
    // 64-element TMA boxes of B to divide 192: not with an 8-bit N-major B.)
    struct Cand { int bm, bn; double kb_us, tile_us; };
    const bool wide_ok = !(elt == 1 && b_mn);
    const Cand cands[6] = {{256, 256, 0.68, 1.0}, {256, 192, 0.52, 0.9}, {128, 256, 0.36, 0.3},
                           {128, 192, 0.29, 0.3}, {128, 128, 0.21, 0.3}, {128, 64, 0.20, 0.3}};
    const int num_k_est = (int)(((long long)K * elt + KBYTES - 1) / KBYTES);
    double best = 1e300;
    for (const Cand& cd : cands) {
      if (cd.bn == 192 && !wide_ok) continue;
      const long long t = tiles(cd.bm, cd.bn);
      const long long waves = (t + ctx->sm_count - 1) / ctx->sm_count;
      const double est = (double)waves * (num_k_est * cd.kb_us + cd.tile_us);
      if (est < best) { best = est; bm = cd.bm; bn = cd.bn; }
    }
  }
  if (pair) { bm = 256; bn = 256 * pair_nb; }
  if (elt == 1 && b_mn && bn < 128) bn = 128;  // an MN-major box is 128 columns of 1-byte elements
  if (!pair && bn == 192 && elt == 1 && b_mn)
    return fail(B200_ERR_ARG, "B200_GEMM_TILE=%d: a 192-column tile cannot take an 8-bit N-major B", force);
  if (!pair && !((bm == 128 && (bn == 64 || bn == 128 || bn == 192 || bn == 256)) || (bm == 256 && (bn == 192 || bn == 256))))
    return fail(B200_ERR_ARG, "B200_GEMM_TILE=%d is not a tile shape of this library", force);
  const int a_rows = pair ? 128 : bm;  // rows of A / columns of B that one CTA stages
  const int b_rows = pair ? 128 : bn;

  GemmParams p{};
  p.c = c; p.M = M; p.N = N; p.K = K; p.ldc = scm;
  p.out_dtype = out_dtype; p.activation = activation; p.fp8 = (in_dtype == B200_E4M3);
  p.scale_a = scale_a; p.scale_b = scale_b; p.status = ctx->status;
  p.num_pid_m = (M + bm - 1) / bm; p.num_pid_n = (N + bn - 1) / bn;
  p.num_tiles = p.num_pid_m * p.num_pid_n;
  p.num_k = (K + bk_elems - 1) / bk_elems;
  p.bk_elems = bk_elems;
  p.kb_per_split = (p.num_k + splits - 1) / splits;
  p.splits = (p.num_k + p.kb_per_split - 1) / p.kb_per_split;  // no empty split
  p.ws = ws;
  p.bias = bias; p.bias_mode = bias_mode; p.bias_sm = bias_sm; p.bias_sn = bias_sn;
  p.group_m = env_int("B200_GEMM_GROUP_M", 8);
  if (p.group_m < 1) p.group_m = 1;
  const int fmt = (in_dtype == B200_BF16) ? 1 : 0;  // kind::f16: f16 = 0, bf16 = 1; kind::f8f6f4: e4m3 = 0
  p.idesc = make_idesc(fmt, fmt, a_mn, b_mn, pair ? 256 : 128, pair ? 256 : bn);
  p.ga = make_geom(a_mn, a_rows, elt, bk_elems);
  p.gb = make_geom(b_mn, b_rows, elt, bk_elems);

  CUtensorMap ta, tbm;
  {
    uint64_t dims[2], strides[1];
    uint32_t box[2];
    if (!a_mn) { dims[0] = K; dims[1] = M; strides[0] = (uint64_t)sam * elt; box[0] = bk_elems; box[1] = a_rows; }
    else       { dims[0] = M; dims[1] = K; strides[0] = (uint64_t)sak * elt; box[0] = p.ga.box_mn; box[1] = bk_elems; }
    if (!encode_tmap(&ta, in_dtype, 2, a, dims, strides, box, true)) return B200_ERR_UNSUPPORTED;
    if (!b_mn) { dims[0] = K; dims[1] = N; strides[0] = (uint64_t)sbn * elt; box[0] = bk_elems; box[1] = b_rows; }
    else       { dims[0] = N; dims[1] = K; strides[0] = (uint64_t)sbk * elt; box[0] = p.gb.box_mn; box[1] = bk_elems; }
    if (!encode_tmap(&tbm, in_dtype, 2, b, dims, strides, box, true)) return B200_ERR_UNSUPPORTED;
  }
  // C through TMA stores when it is a 16-bit output that a tensor map can describe
  CUtensorMap tcm = ta;  // a valid map even when unused
  p.c_tma = 0;
  if (activation != B200_ACT_SOFTMAX && (out_dtype == B200_F16 || out_dtype == B200_BF16) &&
      (reinterpret_cast<uintptr_t>(c) & 15) == 0 && ((scm * 2) & 15) == 0 && !env_int("B200_GEMM_DIRECT_STORE", 0)) {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)M}, strides[1] = {(uint64_t)scm * 2};
    uint32_t box[2] = {64, 32};
    if (encode_tmap(&tcm, out_dtype, 2, c, dims, strides, box, true)) p.c_tma = 1;
  }
  if (pair) {
    if (pair_nb == 2) return launch_pair<4, 2>(ctx, stream, ta, tbm, tcm, p);
    switch (env_int("B200_GEMM_PAIR_STAGES", 6)) {
      case 4: return launch_pair<4, 1>(ctx, stream, ta, tbm, tcm, p);
      case 5: return launch_pair<5, 1>(ctx, stream, ta, tbm, tcm, p);
      case 7: return launch_pair<7, 1>(ctx, stream, ta, tbm, tcm, p);
      default: return launch_pair<6, 1>(ctx, stream, ta, tbm, tcm, p);
    }
  }
  int rc;
  switch (bn) {
    case 256:
      rc = (bm == 256) ? launch_tile<256, 256, 3>(ctx, stream, ta, tbm, tcm, p)
                       : launch_tile<128, 256, 4>(ctx, stream, ta, tbm, tcm, p);
      break;
    case 192:
      rc = (bm == 256) ? launch_tile<256, 192, 3>(ctx, stream, ta, tbm, tcm, p)
                       : launch_tile<128, 192, 5>(ctx, stream, ta, tbm, tcm, p);
      break;
    case 128: rc = launch_tile<128, 128, 6>(ctx, stream, ta, tbm, tcm, p); break;
    default: rc = launch_tile<128, 64, 7>(ctx, stream, ta, tbm, tcm, p); break;
  }
  if (rc || p.splits == 1) return rc;
  const bool vec4 = (N & 3) == 0 && (long long)M * N > (1 << 20);  // 16-byte loads only pay on large outputs
  const int col_threads = vec4 ? N / 4 : N;
  const int tpb = col_threads >= 256 ? 256 : ((col_threads + 31) / 32) * 32;
  dim3 rgrid((col_threads + tpb - 1) / tpb, M < 65535 ? M : 65535, 1);
  if (vec4) splitk_reduce_kernel<4><<<rgrid, tpb, 0, stream>>>(p);
  else splitk_reduce_kernel<1><<<rgrid, tpb, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "split-K reduce launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

// C[M,N2] = out_type( in_type(out_type(A[M,K] B[K,N])) W[N,N2] ) in one launch (gemm_chain_kernel).
// 16-bit inputs, N and N2 at most 128, operands that TMA can address.
int launch_gemm_chain(DeviceCtx* ctx, cudaStream_t stream, const void* a, const void* b, const void* w, void* c, int M,
                      int N, int K, int N2, int64_t sam, int64_t sak, int64_t sbk, int64_t sbn, int64_t swk, int64_t swn,
                      int64_t scm, int in_dtype, int out_dtype) {
  const int elt = 2, bk_elems = KBYTES / elt;
  const bool a_mn = !(sak == 1 || K == 1), b_mn = !(sbk == 1 || K == 1), w_mn = !(swk == 1 || N == 1);
  auto tma_ok = [&](const void* base, int64_t row_stride, int64_t rows) {
    return (reinterpret_cast<uintptr_t>(base) & 15) == 0 && (rows == 1 || ((row_stride * elt) & 15) == 0);
  };
  if (!tma_ok(a, a_mn ? sak : sam, a_mn ? K : M) || !tma_ok(b, b_mn ? sbk : sbn, b_mn ? K : N) ||
      !tma_ok(w, w_mn ? swk : swn, w_mn ? N : N2) || (a_mn && sam != 1) || (b_mn && sbn != 1) || (w_mn && swn != 1))
    return fail(B200_ERR_UNSUPPORTED, "chain-dot needs A, B and W that TMA can address (16-byte aligned base and rows)");
  GemmParams p{};
  p.c = c; p.M = M; p.N = N2; p.K = K; p.ldc = scm;
  p.out_dtype = out_dtype; p.activation = B200_ACT_NONE; p.status = ctx->status;
  p.num_k = (K + bk_elems - 1) / bk_elems;
  p.bk_elems = bk_elems;
  p.splits = 1; p.kb_per_split = p.num_k;
  p.in_bf16 = (in_dtype == B200_BF16);
  const int fmt = p.in_bf16 ? 1 : 0;
  p.idesc = make_idesc(fmt, fmt, a_mn, b_mn, 128, 128);
  p.idesc2 = make_idesc(fmt, fmt, 0, w_mn, 128, 128);
  p.ga = make_geom(a_mn, 128, elt, bk_elems);
  p.gb = make_geom(b_mn, 128, elt, bk_elems);
  p.gw = make_geom(w_mn, 128, elt, bk_elems);
  CUtensorMap ta, tbm, tw;
  {
    uint64_t dims[2], strides[1];
    uint32_t box[2];
    if (!a_mn) { dims[0] = K; dims[1] = M; strides[0] = (uint64_t)sam * elt; box[0] = bk_elems; box[1] = 128; }
    else       { dims[0] = M; dims[1] = K; strides[0] = (uint64_t)sak * elt; box[0] = p.ga.box_mn; box[1] = bk_elems; }
    if (!encode_tmap(&ta, in_dtype, 2, a, dims, strides, box, true)) return B200_ERR_UNSUPPORTED;
    if (!b_mn) { dims[0] = K; dims[1] = N; strides[0] = (uint64_t)sbn * elt; box[0] = bk_elems; box[1] = 128; }
    else       { dims[0] = N; dims[1] = K; strides[0] = (uint64_t)sbk * elt; box[0] = p.gb.box_mn; box[1] = bk_elems; }
    if (!encode_tmap(&tbm, in_dtype, 2, b, dims, strides, box, true)) return B200_ERR_UNSUPPORTED;
    // W as the B operand of the second product: its "K" is N, its "N" is N2
    if (!w_mn) { dims[0] = N; dims[1] = N2; strides[0] = (uint64_t)swn * elt; box[0] = bk_elems; box[1] = 128; }
    else       { dims[0] = N2; dims[1] = N; strides[0] = (uint64_t)swk * elt; box[0] = p.gw.box_mn; box[1] = bk_elems; }
    if (!encode_tmap(&tw, in_dtype, 2, w, dims, strides, box, true)) return B200_ERR_UNSUPPORTED;
  }
  CUtensorMap tcm = ta;
  p.c_tma = 0;
  if ((out_dtype == B200_F16 || out_dtype == B200_BF16) && (reinterpret_cast<uintptr_t>(c) & 15) == 0 &&
      ((scm * 2) & 15) == 0) {
    uint64_t dims[2] = {(uint64_t)N2, (uint64_t)M}, strides[1] = {(uint64_t)scm * 2};
    uint32_t box[2] = {64, 32};
    if (encode_tmap(&tcm, out_dtype, 2, c, dims, strides, box, true)) p.c_tma = 1;
  }
  constexpr int STAGES = 4;
  constexpr size_t smem = (size_t)STAGES * 256 * KBYTES + 2 * 128 * KBYTES + 4 * STG_BYTES + (2 * STAGES + 6) * 8 + 16 + 1024;
  static std::atomic<bool> attr_done[64];
  if (int rc = ensure_dynamic_smem(gemm_chain_kernel<STAGES>, smem, ctx->device, attr_done, "chain gemm")) return rc;
  gemm_chain_kernel<STAGES><<<(M + 127) / 128, 192, smem, stream>>>(ta, tbm, tw, tcm, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "chain gemm launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

size_t gemm_grouped_workspace_bytes(int group_count) { return (size_t)(group_count > 0 ? group_count : 0) * sizeof(GroupDesc); }

// Writes the groups' descriptors to `workspace` (asynchronously on `stream`) and returns the number of tiles.
int prepare_gemm_grouped(DeviceCtx* ctx, cudaStream_t stream, int group_count, const void* const* a,
                         const void* const* b, void* const* c, const int* sizes, const int* lds, int in_dtype,
                         int out_dtype, void* workspace, int* total_tiles_out) {
  (void)ctx;
  constexpr int BM = 128, BN = 128;
  const int elt = dtype_bytes(in_dtype);  // 2
  const int bk_elems = KBYTES / elt;
  std::vector<GroupDesc> descs;
  descs.reserve(group_count);
  int total_tiles = 0;
  for (int g = 0; g < group_count; ++g) {
    const int M = sizes[3 * g], N = sizes[3 * g + 1], K = sizes[3 * g + 2];
    const long long lda = lds[3 * g], ldb = lds[3 * g + 1], ldc = lds[3 * g + 2];
    if (M < 0 || N < 0 || K < 0) return fail(B200_ERR_ARG, "group %d: negative dimension", g);
    if (M == 0 || N == 0) continue;
    if (!c[g] || (K > 0 && (!a[g] || !b[g]))) return fail(B200_ERR_ARG, "group %d: null pointer", g);
    if (K == 0) {  // an empty sum
      cudaError_t e = cudaMemset2DAsync(c[g], (size_t)ldc * dtype_bytes(out_dtype), 0, (size_t)N * dtype_bytes(out_dtype),
                                        (size_t)M, stream);
      if (e != cudaSuccess) return fail(B200_ERR_CUDA, "memset: %s", cudaGetErrorString(e));
      continue;
    }
    GroupDesc d{};
    uint64_t dims[2], strides[1];
    uint32_t box[2];
    // A [M, K] row-major: K-major operand; B [K, N] row-major: N-major operand (as in the reference)
    dims[0] = K; dims[1] = M; strides[0] = (uint64_t)lda * elt; box[0] = bk_elems; box[1] = BM;
    if (!encode_tmap(&d.ta, in_dtype, 2, a[g], dims, strides, box, true)) return B200_ERR_UNSUPPORTED;
    dims[0] = N; dims[1] = K; strides[0] = (uint64_t)ldb * elt; box[0] = 128 / elt; box[1] = bk_elems;
    if (!encode_tmap(&d.tb, in_dtype, 2, b[g], dims, strides, box, true)) return B200_ERR_UNSUPPORTED;
    d.tc = d.ta;
    d.c_tma = 0;
    if ((out_dtype == B200_F16 || out_dtype == B200_BF16) && (reinterpret_cast<uintptr_t>(c[g]) & 15) == 0 &&
        ((ldc * 2) & 15) == 0) {
      uint64_t cd[2] = {(uint64_t)N, (uint64_t)M}, cs[1] = {(uint64_t)ldc * 2};
      uint32_t cb[2] = {64, 32};
      if (encode_tmap(&d.tc, out_dtype, 2, c[g], cd, cs, cb, true)) d.c_tma = 1;
    }
    d.c = c[g]; d.ldc = ldc; d.M = M; d.N = N;
    d.num_k = (K + bk_elems - 1) / bk_elems;
    d.num_pid_n = (N + BN - 1) / BN;
    d.tile_start = total_tiles;
    d.num_tiles = ((M + BM - 1) / BM) * d.num_pid_n;
    total_tiles += d.num_tiles;
    descs.push_back(d);
  }
  *total_tiles_out = total_tiles;
  if (descs.empty()) return B200_OK;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 127))
    return fail(B200_ERR_ARG, "grouped matmul needs a 128-byte aligned device workspace (b200_grouped_matmul_workspace)");
  // pageable host memory: the copy has left the vector when the call returns
  cudaError_t e = cudaMemcpyAsync(workspace, descs.data(), descs.size() * sizeof(GroupDesc), cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "descriptor copy: %s", cudaGetErrorString(e));
  return B200_OK;
}

// One persistent launch over the tiles described in `workspace` (prepare_gemm_grouped).
int launch_gemm_grouped(DeviceCtx* ctx, cudaStream_t stream, const void* workspace, int total_tiles, int in_dtype,
                        int out_dtype) {
  constexpr int BM = 128, BN = 128, STAGES = 6;
  if (total_tiles <= 0) return B200_OK;
  const int elt = dtype_bytes(in_dtype);
  const int bk_elems = KBYTES / elt;
  cudaError_t e;
  GemmParams p{};
  p.out_dtype = out_dtype; p.activation = B200_ACT_NONE; p.status = ctx->status;
  p.bk_elems = bk_elems; p.splits = 1;
  const int fmt = (in_dtype == B200_BF16) ? 1 : 0;
  p.idesc = make_idesc(fmt, fmt, 0, 1, BM, BN);
  p.ga = make_geom(false, BM, elt, bk_elems);
  p.gb = make_geom(true, BN, elt, bk_elems);
  static std::atomic<bool> attr_done[64];
  constexpr size_t smem = smem_bytes(STAGES, (BM + BN) * KBYTES, BM / 32);
  if (int rc = ensure_dynamic_smem(gemm_grouped_kernel<STAGES>, smem, ctx->device, attr_done, "grouped gemm")) return rc;
  const int grid = total_tiles < ctx->sm_count ? total_tiles : ctx->sm_count;
  gemm_grouped_kernel<STAGES><<<grid, 192, smem, stream>>>(reinterpret_cast<const GroupDesc*>(workspace), total_tiles, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "grouped gemm launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

}  // namespace tb
