// Flash-attention forward for sm_100a.
//
// Computes what the reference's _attn_fwd / _attn_fwd_inner compute
// (python/tutorials/06-fused-attention.py:25-187): O = softmax(Q K^T * sm_scale [causal]) V with
// an online softmax in base 2 (scores scaled by sm_scale * log2 e, :160-161), fp32 statistics,
// P rounded to the storage type before the second product (:66-69), O = acc / l rounded once,
// and M = m + log2(l) per row (:183-187).  Masked scores contribute exactly 0.
//
// One CTA owns 256 query rows of one (batch, head): two 128-row tiles that ping-pong so that the
// tensor pipe works on one tile while the other tile's softmax runs (one 128-row tile at head dim
// 256, where a tile's accumulator alone takes half of TMEM).  Sixteen warps:
//   warps 0-3 / 4-7   softmax of tile 0 / 1, one thread per query row (no cross-thread reduction):
//                     tcgen05.ld S, running max and sum, exp2, P packed to 16 bit and written back over S in TMEM
//                     (tcgen05.st) as the A operand of the second MMA.  The accumulator O is
//                     rescaled lazily: only when the running max grew by more than 2^8 does the
//                     warp multiply its O rows in TMEM (the reference rescales every step; the
//                     result is the same up to fp32 rounding since P and l carry the same factor).
//                     At the end: O / l -> storage type -> global, M -> global.
//   warp 8            MMA issuer (one elected lane): S_i = Q_i K_j^T (operands in shared memory) and
//                     O_i += P_i V_j (P from TMEM, V from shared memory, N-major).  MMAs of one
//                     thread execute in issue order, which is what lets P alias S.
//   warp 9            TMA producer: Q tiles once, then K_0, V_0, K_1, V_1 ... through a ring.
//   warps 10-15       lend their registers: the CTA's 64K registers are re-divided at run time
//                     (setmaxnreg) so that a softmax thread can hold a whole 128-column score row
//                     without spilling (216 registers; with ten warps the limit was 168 and the
//                     row spilled to local memory, an L2 round trip per value).
// The kernel is persistent: one CTA per SM takes work items (256 query rows of one head) from an
// atomic counter, head-major and heavy-first, so a head's K/V stay in L2, causal work balances, and
// the epilogue of one item overlaps the loads and first MMAs of the next.
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [384,384+D); P_i = first 64 columns of S_i
// at head dim 128, and columns [320,384) / [448,512) at head dim 64 (16-bit), where S_i of the next
// block is then issued before P_i V of this one.  Head dim 256: S [0,128), O [256,512).
#include <cmath>
#include <cstdlib>

#define B200_INLINE_WAIT_SLOW  // this kernel re-divides registers between its warpgroups
#include "common.cuh"
#include "host.h"

namespace tb {

namespace {

constexpr int BLK = 128;           // rows of a Q tile and of a K/V block
constexpr int FWD_THREADS = 512;   // 8 softmax warps, MMA warp, TMA warp, 6 warps that only lend their registers
// registers per thread after the re-division; one warp of each warpgroup shares a scheduler's 16K
// registers: (2 * 216 + 56 + 24) * 32 lanes = 16384
constexpr int REGS_SOFTMAX = 216, REGS_MMA_TMA = 56, REGS_IDLE = 24;
// Lazy rescale: the accumulator and the row sum keep their reference point m_ref until the running
// maximum has grown past it by more than this many log2 units, so P may reach 2^threshold: 15 for an
// fp16 P (largest finite value 65504), 60 for bf16 (fp32 range; the row sum of 2^14 such values and the
// accumulator stay far below the fp32 limit).  The rounding of P is relative, so its bits do not
// depend on the reference point as long as it stays in range.
template <bool BF16> constexpr float kRescaleThreshold = BF16 ? 60.0f : 15.0f;

// Column pairs out of every 8 whose exp2 is computed by a cubic on the FMA pipe (0: all on the
// special-function unit).
#ifndef B200_FWD_POLY
#define B200_FWD_POLY 2
#endif
constexpr int kPolyStride = 3;  // spreads the chosen pairs over a group of 8 (3 is coprime to 8)

struct FwdParams {
  void* o;
  float* m;  // [Z*H, N] base-2 log-sum-exp of the scaled scores
  float* row_max;  // optional [Z*H, N]: base-2 row maximum of the scaled scores (the old-style kernels' M / ln 2)
  long long o_sz, o_sh, o_sn;  // element strides of O
  int Z, H, N;
  int causal;
  float scale_log2;  // sm_scale * log2(e)
  int num_qb;        // query blocks (one work item each: 256 rows, 128 at head dim 256) per head
  int total_items;   // num_qb * Z * H
  int* sched_counter;  // work counter of this launch: zero at launch, put back to zero by the last CTA
  int o_tma;           // O is written through shared-memory staging and TMA stores
  unsigned* status;
};

// FP8: Q, K, V, P and O are 8-bit (e5m2, the reference's fp8 forward, 06-fused-attention.py:38-40,
// 66-69, 127): both products use kind::f8f6f4 MMAs with K = 32 per instruction; V is read with its
// key dimension contiguous (the layout the reference gives an fp8 V), i.e. as a K-major operand.
template <int D, bool FP8 = false>
struct FwdCfg {
  static constexpr int TILE_BYTES = BLK * D * (FP8 ? 1 : 2);   // one Q tile or one K / V block
  static constexpr int TILES = (D == 256) ? 1 : 2;             // 128-row query tiles per work item
  static constexpr int KV_STAGES = (D == 256) ? 2 : ((D == 128 && !FP8) ? 4 : 8);
  // tiles + barriers + TMEM slot + scheduler slots + alignment slack
  static constexpr int STG_BYTES = 32 * 128;  // epilogue staging of one softmax warp: 32 rows x 64 columns
  static constexpr size_t SMEM = (size_t)TILES * TILE_BYTES + (size_t)KV_STAGES * TILE_BYTES + 4 * TILES * STG_BYTES + (2 * KV_STAGES + 22) * 8 + 32 + 1024;
};

// one Q tile or K / V block of 128 rows: boxes of 128 bytes x 128 rows.  `along_rows`: the 8-bit V,
// whose map is [D rows][N keys]: the block is 128 keys wide and starts at key row0.
template <int D, bool FP8>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int row0, int h, int z,
                                          bool along_rows = false) {
  if constexpr (FP8) {
    if (along_rows) tma_load_4d(dst, map, bar, row0, 0, h, z);
    else tma_load_4d(dst, map, bar, 0, row0, h, z);
  } else {
#pragma unroll
    for (int b = 0; b < D / 64; ++b) tma_load_4d(dst + b * (BLK * 128), map, bar, b * 64, row0, h, z);
  }
}

// One work item = TILES * 128 query rows of one (batch, head).  Items are numbered head-major, heavy
// (late, long) query blocks first inside a head, and handed out through an atomic counter.
struct Item {
  int qb, zh, z, h, n0, n1, nmax;  // n_i: K/V blocks tile i visits; nmax: blocks the item streams
};
template <int TILES>
__device__ __forceinline__ Item decode_item(const FwdParams& p, int w) {
  Item it;
  it.zh = w / p.num_qb;
  it.qb = p.num_qb - 1 - (w % p.num_qb);
  it.z = it.zh / p.H;
  it.h = it.zh % p.H;
  const int nkv_all = (p.N + BLK - 1) / BLK;
  // K/V blocks per tile: up to and including the block that holds the tile's diagonal when causal
  it.n0 = p.causal ? min(TILES * it.qb + 1, nkv_all) : nkv_all;
  it.n1 = (TILES == 2) ? (p.causal ? min(2 * it.qb + 2, nkv_all) : nkv_all) : 0;  // n0 <= n1 <= n0 + 1 with two tiles
  it.nmax = (TILES == 2) ? it.n1 : it.n0;
  return it;
}

template <int D, bool BF16, bool FP8>
__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o_map,
                const FwdParams p) {
  using Cfg = FwdCfg<D, FP8>;
  constexpr int TILE = Cfg::TILE_BYTES, NST = Cfg::KV_STAGES, TILES = Cfg::TILES;
  constexpr int ITEM_ROWS = TILES * BLK;
  constexpr int MMA_WARP = 8, TMA_WARP = 9;
  constexpr bool WAIT_PAUSE = (D != 64);  // see mbar_wait_slow

  extern __shared__ uint8_t smem_raw[];
  const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  uint8_t* sq = smem;                    // Q tiles
  uint8_t* skv = smem + TILES * TILE;    // ring
  uint8_t* sstage = skv + NST * TILE;  // one 4 KiB buffer per softmax warp, 128-byte swizzled
  uint64_t* bars = reinterpret_cast<uint64_t*>(sstage + 4 * TILES * Cfg::STG_BYTES);
  uint64_t* q_full = bars;             // [2]
  uint64_t* kv_full = bars + 2;        // [NST]
  uint64_t* kv_empty = kv_full + NST;  // [NST]
  uint64_t* s_full = kv_empty + NST;   // [2] S_i(j) is in TMEM
  uint64_t* p_full = s_full + 2;       // [2 tiles][2 halves] columns [64h, 64h+64) of P_i(j) are in TMEM (and O_i rescaled if it had to be)
  uint64_t* o_full = p_full + 4;       // [2] last P V of tile i done
  uint64_t* q_empty = o_full + 2;      // [1] every S MMA of the item has read the Q tiles
  uint64_t* sched_full = q_empty + 1;  // [2] an item id was published
  uint64_t* sched_empty = sched_full + 2;  // [2] all 9 readers have taken it
  uint64_t* s_free = sched_empty + 2;      // [2] (head dim 64) the softmax warps of tile i hold S_i(j) in registers
  uint64_t* pv_done = s_free + 2;          // [2] (head dim 64) P_i(j) V_j is complete: O_i and the P buffer may be touched
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  volatile int* sched_item = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  B200_TRACE_DECL;  // trace builds: regions 0 / 1 = first softmax warp of tile 0 / 1, region 2 = MMA warp

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[2 * i], 128);
      mbar_init(&p_full[2 * i + 1], 128);
      mbar_init(&o_full[i], 1);
      mbar_init(&s_free[i], 4);  // one arrival per softmax warp of the tile
      mbar_init(&pv_done[i], 1);
      mbar_init(&sched_full[i], 1);
      mbar_init(&sched_empty[i], 1 + 4 * TILES);  // MMA warp + one lane of each softmax warp
    }
    mbar_init(q_empty, 1);
    for (int s = 0; s < NST; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    fence_barrier_init();
    cta_wait_flag_clear();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_o_map);
  }
  if (warp == MMA_WARP) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const uint32_t tm_s[2] = {tmem_base, tmem_base + 128};
  const uint32_t tm_o[2] = {tmem_base + 256, tmem_base + 384};
  // At head dim 64 the O accumulators leave 2 x 64 columns free, which hold P: with P out of the
  // S buffer, S_i(j+1) is issued as soon as the softmax warps have S_i(j) in registers instead of
  // after P_i(j) V_j, so the scores of the next block are ready when a tile's softmax comes back
  // for them.  (At head dim 128 TMEM is full and P overwrites S.)
  constexpr bool SEP_P = (D == 64) && !FP8;
  auto tm_p = [&](int i) { return SEP_P ? tmem_base + (i ? 448u : 320u) : tm_s[i]; };

  // Every role ends with its own copy of the teardown and returns: no code is shared after the
  // register budgets have diverged (values live across a join would have to sit in registers that
  // every budget has).
  auto teardown = [&](bool owner) {
    // after a recorded failure give copies in flight time to land before the CTA exits
    cta_linger_after_failure();
    tc_fence_before();
    __syncthreads();
    if (owner) {
      tc_fence_after();
      tmem_dealloc(tmem_base, 512);
    }
  };
  if (warp >= 12 || (TILES == 1 && warp >= 4 && warp < 8)) {
    // nothing else: these warps only lend registers and take part in the barriers at both ends
    // (at head dim 256 the second tile's softmax warpgroup has no tile)
    reg_dec<REGS_IDLE>();
    teardown(false);
    return;
  } else if (warp >= 10) {
    reg_dec<REGS_MMA_TMA>();
    teardown(false);
    return;
  } else if (warp == TMA_WARP) {
    reg_dec<REGS_MMA_TMA>();
    // ------------------------------------------------------------------ scheduler + TMA producer
    if (lane == 0) {
      uint32_t s = 0, ph = 0;  // K/V ring position, runs on across items
      for (uint32_t n = 0;; ++n) {
        const int w = atomicAdd(p.sched_counter, 1);
        const uint32_t slot = n & 1u, sph = (n >> 1) & 1u;
        mbar_wait<WAIT_PAUSE>(&sched_empty[slot], sph ^ 1u, p.status, SITE_FWD_SCHED);
        sched_item[slot] = w;
        mbar_arrive(&sched_full[slot]);
        // every CTA draws exactly one ticket past the end: the last of them puts the zero back for the
        // next launch that is handed this counter
        if (w == p.total_items + (int)gridDim.x - 1) atomicExch(p.sched_counter, 0);
        if (w >= p.total_items) break;
        const Item it = decode_item<TILES>(p, w);
        mbar_wait<WAIT_PAUSE>(q_empty, (n & 1u) ^ 1u, p.status, SITE_FWD_Q);  // previous item's S MMAs are done with Q
        for (int i = 0; i < TILES; ++i) {
          mbar_expect_tx(&q_full[i], TILE);
          load_tile<D, FP8>(sq + i * TILE, &tm_q, &q_full[i], it.qb * ITEM_ROWS + i * BLK, it.h, it.z);
        }
        for (int j = 0; j < it.nmax; ++j) {
          for (int kv = 0; kv < 2; ++kv) {  // K_j then V_j
            mbar_wait<WAIT_PAUSE>(&kv_empty[s], ph ^ 1u, p.status, SITE_FWD_KV_EMPTY);
            mbar_expect_tx(&kv_full[s], TILE);
            load_tile<D, FP8>(skv + s * TILE, kv == 0 ? &tm_k : &tm_v, &kv_full[s], j * BLK, it.h, it.z, kv == 1);
            if (++s == NST) { s = 0; ph ^= 1u; }
          }
        }
      }
    }
    __syncwarp();
    teardown(false);
    return;
  } else if (warp == MMA_WARP) {
    reg_dec<REGS_MMA_TMA>();
    // ------------------------------------------------------------------ MMA issuer
    // The warp stays converged and an elected lane issues, for both tiles.  (Two issuing threads,
    // one per tile, were measured 20 % slower: MMAs of different threads interleave in the pipe
    // at a cost.)
    {
      constexpr int FMT = (BF16 || FP8) ? 1 : 0;  // kind::f16: bf16 = 1; kind::f8f6f4: e5m2 = 1
      constexpr uint32_t IDESC_S = make_idesc(FMT, FMT, 0, 0, 128, BLK);  // Q (K-major) x K (K-major)
      constexpr uint32_t IDESC_O = make_idesc(FMT, FMT, 0, FP8 ? 0 : 1, 128, D);  // P (TMEM) x V (N-major; K-major when 8-bit)
      // Q and K: rows of 128 bytes (64 16-bit or 128 8-bit elements per box), 128-byte swizzle; the
      // 8-bit forward at head dim 64 has rows of 64 bytes, 64-byte swizzle (8-row groups 512 B apart)
      constexpr bool ROW64 = FP8 && D == 64;
      const uint64_t dq0 = ROW64 ? smem_desc_sw64(smem_u32(sq), 0, 512) : smem_desc_sw128(smem_u32(sq), 0, 1024);
      const uint64_t dk0 = ROW64 ? smem_desc_sw64(smem_u32(skv), 0, 512) : smem_desc_sw128(smem_u32(skv), 0, 1024);
      const uint64_t dv0 = smem_desc_sw128(smem_u32(skv), FP8 ? 0 : BLK * 128, 1024);  // LBO: next 64-column box
      uint32_t s = 0, ph = 0;        // ring position of the next unconsumed K / V block
      uint32_t pcnt[2] = {0, 0};     // blocks of tile i whose P has been consumed (parity of p_full)
      [[maybe_unused]] uint32_t fcnt[2] = {0, 0};  // (head dim 64) blocks of tile i so far, across items (parity of s_free)

      auto issue_s = [&](int i, uint32_t stage) {  // S_i = Q_i K^T, D/16 MMAs
        const uint64_t dq = dq0 + i * (TILE >> 4), dk = dk0 + stage * (TILE >> 4);
        if constexpr (FP8) {
#pragma unroll
          for (int kk = 0; kk < D / 32; ++kk)  // one 128-byte box: 32 B (32 elements) per step
            umma_ss_elect<true>(tm_s[i], dq + kk * 2, dk + kk * 2, IDESC_S, kk != 0);
        } else {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * ((BLK * 128) >> 4) + (kk & 3) * 2;  // 64-col box, 32 B per step
            umma_ss_elect<false>(tm_s[i], dq + off, dk + off, IDESC_S, kk != 0);
          }
        }
        tc_commit_elect(&s_full[i]);
        if (lane == 0) B200_TRACE_EVENT(p.status, 2, 0x40 | i);
      };
      // O_i (+)= P_i V: 8 MMAs of 16 kv rows; the second four wait for the second half of P
      auto issue_pv = [&](int i, uint32_t stage, uint32_t accum, uint32_t parity) {
        const uint64_t dv = dv0 + stage * (TILE >> 4);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (lane == 0) B200_TRACE_EVENT(p.status, 2, 0x10 | (i << 1) | h);
          mbar_wait<WAIT_PAUSE>(&p_full[2 * i + h], parity, p.status, SITE_FWD_P_FULL);
          if (lane == 0) B200_TRACE_EVENT(p.status, 2, 0x20 | (i << 1) | h);
          tc_fence_after();
          if constexpr (FP8) {
#pragma unroll
            for (int kk = 2 * h; kk < 2 * h + 2; ++kk)  // 32 keys per MMA: 8 TMEM columns of P, 32 B of the V rows
              umma_ts_f8_elect(tm_o[i], tm_p(i) + kk * 8, dv + kk * 2, IDESC_O, (accum | kk) != 0);
          } else {
#pragma unroll
            for (int kk = 4 * h; kk < 4 * h + 4; ++kk)
              umma_ts_f16_elect(tm_o[i], tm_p(i) + kk * 8, dv + kk * ((16 * 128) >> 4), IDESC_O, (accum | kk) != 0);
          }
        }
      };
      auto advance = [&]() { if (++s == NST) { s = 0; ph ^= 1u; } };

      for (uint32_t n = 0;; ++n) {
        const uint32_t slot = n & 1u, sph = (n >> 1) & 1u;
        mbar_wait<WAIT_PAUSE>(&sched_full[slot], sph, p.status, SITE_FWD_SCHED);
        const int w = sched_item[slot];
        __syncwarp();
        if (lane == 0) mbar_arrive(&sched_empty[slot]);
        if (w >= p.total_items) break;
        const Item it = decode_item<TILES>(p, w);
        const int n0 = it.n0, n1 = it.n1, nmax = it.nmax;

        // prologue: S_0(0), S_1(0) on K_0
        mbar_wait<WAIT_PAUSE>(&kv_full[s], ph, p.status, SITE_FWD_KV_FULL);
        mbar_wait<WAIT_PAUSE>(&q_full[0], n & 1u, p.status, SITE_FWD_Q);
        issue_s(0, s);
        if constexpr (TILES == 2) {
          mbar_wait<WAIT_PAUSE>(&q_full[1], n & 1u, p.status, SITE_FWD_Q);
          issue_s(1, s);
        }
        tc_commit_elect(&kv_empty[s]);
        if (nmax == 1) tc_commit_elect(q_empty);
        advance();
        for (int j = 0; j < nmax; ++j) {
          const uint32_t vs = s, vph = ph;  // V_j
          advance();
          const uint32_t ks = s, kph = ph;  // K_{j+1} (if any)
          const bool more1 = (TILES == 2) && (j + 1 < n1), more0 = (j + 1 < n0);
          if constexpr (SEP_P) {
            // the next scores first: S_i(j+1) only needs the S buffer, which is free once the
            // softmax warps have loaded S_i(j)
            if (more0) {
              mbar_wait<WAIT_PAUSE>(&s_free[0], fcnt[0]++ & 1u, p.status, SITE_FWD_S_EMPTY);
              tc_fence_after();
              mbar_wait<WAIT_PAUSE>(&kv_full[ks], kph, p.status, SITE_FWD_KV_FULL);
              issue_s(0, ks);
            } else if (j < n0) {
              ++fcnt[0];  // the tile's last block: its arrival is not waited for, the count goes on
            }
            if (more1) {
              mbar_wait<WAIT_PAUSE>(&s_free[1], fcnt[1]++ & 1u, p.status, SITE_FWD_S_EMPTY);
              tc_fence_after();
              mbar_wait<WAIT_PAUSE>(&kv_full[ks], kph, p.status, SITE_FWD_KV_FULL);
              issue_s(1, ks);
              tc_commit_elect(&kv_empty[ks]);
              if (j + 2 == n1) tc_commit_elect(q_empty);  // that was the item's last S: the Q tiles may be replaced
            } else {
              ++fcnt[1];
            }
            if (lane == 0) B200_TRACE_EVENT(p.status, 2, 0x50);
            mbar_wait<WAIT_PAUSE>(&kv_full[vs], vph, p.status, SITE_FWD_KV_FULL);
            if (lane == 0) B200_TRACE_EVENT(p.status, 2, 0x60);
            if (j < n0) {
              issue_pv(0, vs, j > 0, pcnt[0]++ & 1u);
              tc_commit_elect(&pv_done[0]);
              if (j == n0 - 1) tc_commit_elect(&o_full[0]);
            }
            issue_pv(1, vs, j > 0, pcnt[1]++ & 1u);
            tc_commit_elect(&kv_empty[vs]);
            tc_commit_elect(&pv_done[1]);
            if (j == n1 - 1) tc_commit_elect(&o_full[1]);
            if (more1) advance();
          } else {
            if (lane == 0) B200_TRACE_EVENT(p.status, 2, 0x50);
            mbar_wait<WAIT_PAUSE>(&kv_full[vs], vph, p.status, SITE_FWD_KV_FULL);
            if (lane == 0) B200_TRACE_EVENT(p.status, 2, 0x60);
            if (j < n0) {
              issue_pv(0, vs, j > 0, pcnt[0]++ & 1u);
              if (TILES == 1) tc_commit_elect(&kv_empty[vs]);
              if (j == n0 - 1) tc_commit_elect(&o_full[0]);
              if (more0) {
                mbar_wait<WAIT_PAUSE>(&kv_full[ks], kph, p.status, SITE_FWD_KV_FULL);
                issue_s(0, ks);
                if (TILES == 1) {
                  tc_commit_elect(&kv_empty[ks]);
                  if (j + 2 == n0) tc_commit_elect(q_empty);
                  advance();
                }
              }
            }
            if constexpr (TILES == 2) {
              issue_pv(1, vs, j > 0, pcnt[1]++ & 1u);
              tc_commit_elect(&kv_empty[vs]);
              if (j == n1 - 1) tc_commit_elect(&o_full[1]);
              if (more1) {
                mbar_wait<WAIT_PAUSE>(&kv_full[ks], kph, p.status, SITE_FWD_KV_FULL);
                issue_s(1, ks);
                tc_commit_elect(&kv_empty[ks]);
                if (j + 2 == n1) tc_commit_elect(q_empty);  // that was the item's last S: the Q tiles may be replaced
                advance();
              }
            }
          }
        }
      }
    }
    __syncwarp();
    teardown(true);
    return;
  } else {
    reg_inc<REGS_SOFTMAX>();
    // ------------------------------------------------------------------ softmax + epilogue
    // 4 warps per tile, one thread per query row.
    const int i = warp >> 2;                 // tile
    const uint32_t quarter = warp & 3u;      // TMEM lanes [32*quarter, +32)
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = (quarter * 32u) << 16;
    const float scale = p.scale_log2;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.o) & 15) == 0) && ((p.o_sn & 7) == 0) && ((p.o_sh & 7) == 0) &&
                        ((p.o_sz & 7) == 0);
    uint32_t scnt = 0;  // blocks of this tile seen so far, across items (parity of s_full)

    for (uint32_t n = 0;; ++n) {
      const uint32_t slot = n & 1u, sph = (n >> 1) & 1u;
      int w = 0;
      if (lane == 0) {
        mbar_wait<WAIT_PAUSE>(&sched_full[slot], sph, p.status, SITE_FWD_SCHED);
        w = sched_item[slot];
        mbar_arrive(&sched_empty[slot]);
      }
      w = __shfl_sync(0xffffffffu, w, 0);
      if (w >= p.total_items) break;
      const Item it = decode_item<TILES>(p, w);
      const int qb = it.qb;
      const int row = qb * ITEM_ROWS + i * BLK + row_in_tile;  // query index
      const int nb = i ? it.n1 : it.n0;
      float m_ref = -INFINITY, l = 0.f;
      float m_true = -INFINITY;  // the exact running maximum (m_ref lags it by up to the rescale threshold)
      const bool traced = quarter == 0 && lane == 0;  // used by trace builds only
      if (traced) B200_TRACE_EVENT(p.status, i, 0x100 | nb);

      for (int j = 0; j < nb; ++j, ++scnt) {
        mbar_wait<WAIT_PAUSE>(&s_full[i], scnt & 1u, p.status, SITE_FWD_S_FULL);
        if (traced) B200_TRACE_EVENT(p.status, i, 1);
        tc_fence_after();
        const int col0 = j * BLK;
        const bool need_mask = (p.causal && col0 + BLK - 1 > qb * ITEM_ROWS + i * BLK) || (col0 + BLK > p.N);
        // load 32 columns at a time; the row maximum of a chunk is taken while the next chunk loads
        uint32_t r[BLK];
        float mx4[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) mx4[u] = -INFINITY;
        tmem_ld32(tm_s[i] + lane_addr, r);
        tmem_ld_wait32(r);
#pragma unroll
        for (int c = 0; c < BLK; c += 32) {
          if (c + 32 < BLK) tmem_ld32(tm_s[i] + lane_addr + c + 32, r + c + 32);
          if (need_mask) {
            // columns of this chunk that the row may see: below N and, when causal, up to the row itself
            const int lim = min(p.N, p.causal ? row + 1 : p.N) - (col0 + c);
#pragma unroll
            for (int k = 0; k < 32; ++k)
              if (k >= lim) r[c + k] = __float_as_uint(-INFINITY);
          }
#pragma unroll
          for (int u = 0; u < 16; ++u)  // three-input maximum: one instruction per column pair
            mx4[u] = max3(mx4[u], __uint_as_float(r[c + 2 * u]), __uint_as_float(r[c + 2 * u + 1]));
          if (c + 32 < BLK) tmem_ld_wait32(r + c + 32);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) mx4[u] = fmaxf(max3(mx4[u], mx4[u + 4], mx4[u + 8]), mx4[u + 12]);
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        if constexpr (SEP_P) {
          // S_i(j) is in registers: the S buffer may take S_i(j+1)
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s_free[i]);
        }
        // (head dim 64) before O_i or the P buffer is touched, P_i(j-1) V must be complete; on an
        // item's first block the epilogue's wait for the last P V of the previous item has seen to that
        auto wait_pv = [&]() {
          if (SEP_P && j > 0) {
            mbar_wait<WAIT_PAUSE>(&pv_done[i], (scnt - 1u) & 1u, p.status, SITE_FWD_O_READY);
            tc_fence_after();
          }
        };
        if (traced) B200_TRACE_EVENT(p.status, i, 2);
        // mx is finite: every row sees at least one valid column in every block it visits
        const float m_new = fmaxf(m_ref, mx * scale);
        m_true = fmaxf(m_true, mx * scale);
        // lazy rescale of the accumulator (the ld/st below are warp collectives, so the warp
        // rescales if any of its rows has to)
        // true on the first block (m_ref = -inf).  The 8-bit forward follows the exact running maximum,
        // as the reference does: the 2-bit mantissa of P makes its rounding depend on the scale
        const bool grow = FP8 ? (m_new > m_ref) : ((m_new - m_ref) > kRescaleThreshold<BF16>);
        if (__any_sync(0xffffffffu, grow)) {
          // every row of the warp moves its reference point to its exact running maximum (this block
          // included): the pass over O is paid for by the row that had to move, and the others start
          // their next window from zero lag.  (Leaving 6 log2 units of headroom above the maximum as
          // well bought another 2-3 % on sharply peaked scores; not taken: it costs P 6 bits of range.)
          const float m_to = FP8 ? m_new : m_true;
          const float alpha = (FP8 && !grow) ? 1.f : ex2(m_ref - m_to);  // 0 on the first block
          if (!FP8 || grow) { m_ref = m_to; l *= alpha; }
          if (j > 0) {
            wait_pv();
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
              uint32_t o[32];
              tmem_ld32(tm_o[i] + lane_addr + c, o);
              tmem_ld_wait();
#pragma unroll
              for (int k = 0; k < 32; ++k) o[k] = __float_as_uint(__uint_as_float(o[k]) * alpha);
              tmem_st32(tm_o[i] + lane_addr + c, o);
            }
          }
        }
        if (traced) B200_TRACE_EVENT(p.status, i, 3);
        wait_pv();  // (head dim 64) before the exponential loop, not inside it: a wait in the unrolled loop keeps the compiler from interleaving its chunks
        const float neg_m = -m_ref;
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        [[maybe_unused]] uint64_t sum2[2] = {pk2(0.f, 0.f), pk2(0.f, 0.f)};
        [[maybe_unused]] const uint64_t scale2 = pk2(scale, scale), neg_m2 = pk2(neg_m, neg_m);
#pragma unroll
        for (int c = 0; c < BLK; c += 32) {
          uint32_t wv[16];
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            float p0, p1;
            if constexpr (SEP_P) {
              // head dim 64 is bound by instruction issue: packed fp32 arithmetic for the scaling
              // and the row sum (one issue slot per column pair)
              float x0, x1;
              upk2(fma2(pk2(__uint_as_float(r[c + 2 * k]), __uint_as_float(r[c + 2 * k + 1])), scale2, neg_m2), x0, x1);
              p0 = ex2(x0);
              p1 = ex2(x1);
              sum2[k & 1] = add2(sum2[k & 1], pk2(p0, p1));
            } else if (!FP8 && ((k * kPolyStride) & 7) < B200_FWD_POLY) {
              // some of the exponentials on the FMA pipe: the special-function unit is the
              // busiest unit of this loop
              float x0, x1;
              upk2(fma2(pk2(__uint_as_float(r[c + 2 * k]), __uint_as_float(r[c + 2 * k + 1])), scale2, neg_m2), x0, x1);
              ex2_cubic2(x0, x1, p0, p1);
              sum4[k & 3] += p0 + p1;
            } else {
              p0 = ex2(fmaf(__uint_as_float(r[c + 2 * k]), scale, neg_m));
              p1 = ex2(fmaf(__uint_as_float(r[c + 2 * k + 1]), scale, neg_m));
              sum4[k & 3] += p0 + p1;
            }
            if constexpr (FP8) {  // keep the values; four are packed into one column below
              r[c + 2 * k] = __float_as_uint(p0);
              r[c + 2 * k + 1] = __float_as_uint(p1);
            } else {
              wv[k] = pack2<BF16>(p0, p1);
            }
          }
          if constexpr (FP8) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
              wv[k] = pack4_e5m2(__uint_as_float(r[c + 4 * k]), __uint_as_float(r[c + 4 * k + 1]),
                                 __uint_as_float(r[c + 4 * k + 2]), __uint_as_float(r[c + 4 * k + 3]));
            tmem_st8(tm_s[i] + lane_addr + (c >> 2), wv);
          } else {
            tmem_st16(tm_p(i) + lane_addr + (c >> 1), wv);
          }
          if (c == 32 || c == 96) {  // a half of P is complete: its four P V MMAs may start
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&p_full[2 * i + (c >> 6)]);
          }
        }
        if constexpr (SEP_P) {
          float a0, a1, b0, b1;
          upk2(sum2[0], a0, a1);
          upk2(sum2[1], b0, b1);
          l += (a0 + a1) + (b0 + b1);
        } else {
          l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        }
        if (traced) B200_TRACE_EVENT(p.status, i, 4);
      }

      // epilogue: O / l and M.  It overlaps the next item's Q / K loads and first S MMAs; the next
      // item's first P V (which overwrites O) needs this tile's next P, i.e. comes after these
      // reads in program order.
      mbar_wait<WAIT_PAUSE>(&o_full[i], n & 1u, p.status, SITE_FWD_O_FULL);
      if (traced) B200_TRACE_EVENT(p.status, i, 8);
      tc_fence_after();
      const float inv_l = 1.f / l;
      const bool valid = row < p.N;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + (long long)it.z * p.o_sz + (long long)it.h * p.o_sh +
                       (long long)row * p.o_sn;
      if (p.o_tma) {
        // 64 columns at a time: scaled, packed, written to this warp's swizzled staging buffer and
        // stored by TMA (full 128-byte lines; rows past N are clipped by the hardware).  A warp-wide
        // store of one row per lane touches 32 lines per instruction and made this epilogue cost
        // 5200 clk per item at D = 128.
        uint8_t* stg = sstage + warp * Cfg::STG_BYTES;
        const int warp_row0 = qb * ITEM_ROWS + i * BLK + quarter * 32;
        if constexpr (FP8) {
          // 8-bit O: the D columns of a row are one line of the staging buffer
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t o[32];
            tmem_ld32(tm_o[i] + lane_addr + c, o);
            tmem_ld_wait();
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
              uint32_t wv[4];
#pragma unroll
              for (int k = 0; k < 4; ++k)
                wv[k] = pack4_e5m2(__uint_as_float(o[16 * ch + 4 * k]) * inv_l, __uint_as_float(o[16 * ch + 4 * k + 1]) * inv_l,
                                   __uint_as_float(o[16 * ch + 4 * k + 2]) * inv_l, __uint_as_float(o[16 * ch + 4 * k + 3]) * inv_l);
              // one line of the staging buffer per row: 128 bytes (128-byte swizzle) or, at head dim 64, 64 bytes
              const uint32_t off = (D == 64) ? sw64_offset(lane, (c >> 4) + ch) : sw128_offset(lane, (c >> 4) + ch);
              *reinterpret_cast<uint4*>(stg + off) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && warp_row0 < p.N) {
            tma_store_4d(&tm_o_map, stg, 0, warp_row0, it.h, it.z);
            tma_store_commit();
          }
        } else
#pragma unroll 1
        for (int c = 0; c < D; c += 64) {
          uint32_t o[64];
          tmem_ld32(tm_o[i] + lane_addr + c, o);
          tmem_ld32(tm_o[i] + lane_addr + c + 32, o + 32);
          tmem_ld_wait();
          if (traced) B200_TRACE_EVENT(p.status, i, 0xA);
          if (lane == 0) tma_store_wait_read<0>();  // the previous store has read the staging buffer
          __syncwarp();
          if (traced) B200_TRACE_EVENT(p.status, i, 0xB);
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            uint32_t wv[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
              wv[k] = pack2<BF16>(__uint_as_float(o[8 * ch + 2 * k]) * inv_l, __uint_as_float(o[8 * ch + 2 * k + 1]) * inv_l);
            *reinterpret_cast<uint4*>(stg + sw128_offset(lane, ch)) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (traced) B200_TRACE_EVENT(p.status, i, 0xC);
          if (lane == 0 && warp_row0 < p.N) {
            tma_store_4d(&tm_o_map, stg, c, warp_row0, it.h, it.z);
            tma_store_commit();
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_ld32(tm_o[i] + lane_addr + c, o);
          tmem_ld_wait();
          if (valid && FP8) {
            uint8_t* brow = reinterpret_cast<uint8_t*>(p.o) + (long long)it.z * p.o_sz + (long long)it.h * p.o_sh +
                            (long long)row * p.o_sn + c;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const uint32_t wq = pack4_e5m2(__uint_as_float(o[4 * k]) * inv_l, __uint_as_float(o[4 * k + 1]) * inv_l,
                                             __uint_as_float(o[4 * k + 2]) * inv_l, __uint_as_float(o[4 * k + 3]) * inv_l);
              for (int b = 0; b < 4; ++b) brow[4 * k + b] = (uint8_t)(wq >> (8 * b));
            }
          } else if (valid) {
            uint32_t wv[16];
#pragma unroll
            for (int k = 0; k < 16; ++k)
              wv[k] = pack2<BF16>(__uint_as_float(o[2 * k]) * inv_l, __uint_as_float(o[2 * k + 1]) * inv_l);
            if (vec_ok) {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                reinterpret_cast<uint4*>(orow + c)[k] = make_uint4(wv[4 * k], wv[4 * k + 1], wv[4 * k + 2], wv[4 * k + 3]);
            } else {
#pragma unroll
              for (int k = 0; k < 16; ++k) {
                orow[c + 2 * k] = (uint16_t)(wv[k] & 0xFFFFu);
                orow[c + 2 * k + 1] = (uint16_t)(wv[k] >> 16);
              }
            }
          }
        }
      }
      if (valid) p.m[(long long)it.zh * p.N + row] = m_ref + log2f(l);
      if (valid && p.row_max) p.row_max[(long long)it.zh * p.N + row] = m_true;
      if (traced) B200_TRACE_EVENT(p.status, i, 9);
    }
    if (p.o_tma && lane == 0) tma_store_wait_read<0>();  // the staging buffer has been read: the CTA may exit, the writes land on their own
    teardown(false);
  }
}

template <int D, bool BF16, bool FP8 = false>
int launch_fwd_t(DeviceCtx* ctx, cudaStream_t stream, const CUtensorMap& tq, const CUtensorMap& tk,
                 const CUtensorMap& tv, const CUtensorMap& to, const FwdParams& p) {
  static std::atomic<bool> attr_done[64];
  constexpr size_t smem = FwdCfg<D, FP8>::SMEM;
  if (int rc = ensure_dynamic_smem(attn_fwd_kernel<D, BF16, FP8>, smem, ctx->device, attr_done, "attn fwd")) return rc;
  const int grid = p.total_items < ctx->sm_count ? p.total_items : ctx->sm_count;
  attn_fwd_kernel<D, BF16, FP8><<<grid, FWD_THREADS, smem, stream>>>(tq, tk, tv, to, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "attn fwd launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

}  // namespace

bool encode_rows_map(CUtensorMap* out, int dtype, const void* base, int Z, int H, int N, int D, int64_t sz, int64_t sh,
                     int64_t sn, int box_cols, int box_rows, int swizzle) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)N, (uint64_t)H, (uint64_t)Z};
  const uint64_t eb = (uint64_t)dtype_bytes(dtype);
  uint64_t strides[3] = {(uint64_t)sn * eb, (uint64_t)sh * eb, (uint64_t)sz * eb};
  uint32_t box[4] = {(uint32_t)box_cols, (uint32_t)box_rows, 1, 1};
  return encode_tmap(out, dtype, 4, base, dims, strides, box, swizzle);
}

// the operand maps: boxes of 64 columns (128 bytes, swizzled) x box_rows rows
bool encode_qkv_map(CUtensorMap* out, int dtype, const void* base, int Z, int H, int N, int D, int64_t sz, int64_t sh,
                    int64_t sn, int box_rows) {
  return encode_rows_map(out, dtype, base, Z, H, N, D, sz, sh, sn, 64, box_rows, true);
}

int launch_attn_fwd(DeviceCtx* ctx, cudaStream_t stream, const void* q, const void* k, const void* v, void* o,
                    float* m, float* row_max, int Z, int H, int N, int D, const int64_t* sq, const int64_t* sk, const int64_t* sv,
                    const int64_t* so, float sm_scale, int causal, int dtype) {
  if (dtype == B200_E5M2) {
    // 8-bit forward: rows of 128 bytes; V is addressed as [D rows][N keys] (keys contiguous)
    if (D != 128 && D != 64) return fail(B200_ERR_UNSUPPORTED, "the 8-bit forward has kernels for head dims 64 and 128");
    const int sw = (D == 64) ? 2 : 1;  // rows of 64 bytes take the 64-byte swizzle
    if (sq[3] != 1 || sk[3] != 1 || so[3] != 1) return fail(B200_ERR_UNSUPPORTED, "8-bit q, k, o need a contiguous head dimension");
    if (sv[2] != 1 && N != 1) return fail(B200_ERR_UNSUPPORTED, "an 8-bit v needs its key dimension contiguous (stride_v[2] == 1)");
    CUtensorMap tq8, tk8, tv8, to8;
    if (!encode_rows_map(&tq8, dtype, q, Z, H, N, D, sq[0], sq[1], sq[2], D, BLK, sw)) return B200_ERR_UNSUPPORTED;
    if (!encode_rows_map(&tk8, dtype, k, Z, H, N, D, sk[0], sk[1], sk[2], D, BLK, sw)) return B200_ERR_UNSUPPORTED;
    // "rows" of the V map are head-dim indices, "columns" are keys: a block is D rows of 128 keys
    if (!encode_rows_map(&tv8, dtype, v, Z, H, D, N, sv[0], sv[1], sv[3], 128, D, 1)) return B200_ERR_UNSUPPORTED;
    FwdParams p8{};
    p8.o_tma = encode_rows_map(&to8, dtype, o, Z, H, N, D, so[0], so[1], so[2], D, 32, sw) ? 1 : 0;
    if (!p8.o_tma) to8 = tq8;
    p8.o = o; p8.m = m; p8.row_max = row_max;
    p8.o_sz = so[0]; p8.o_sh = so[1]; p8.o_sn = so[2];
    p8.Z = Z; p8.H = H; p8.N = N; p8.causal = causal;
    p8.scale_log2 = sm_scale * 1.44269504f;
    p8.num_qb = (N + 255) / 256;
    p8.total_items = p8.num_qb * Z * H;
    p8.status = ctx->status;
    p8.sched_counter = next_sched_counter(ctx, stream);
    if (!p8.sched_counter) return B200_ERR_CUDA;
    return D == 64 ? launch_fwd_t<64, false, true>(ctx, stream, tq8, tk8, tv8, to8, p8)
                   : launch_fwd_t<128, false, true>(ctx, stream, tq8, tk8, tv8, to8, p8);
  }
  CUtensorMap tq, tk, tv;
  if (!encode_qkv_map(&tq, dtype, q, Z, H, N, D, sq[0], sq[1], sq[2], BLK)) return B200_ERR_UNSUPPORTED;
  if (!encode_qkv_map(&tk, dtype, k, Z, H, N, D, sk[0], sk[1], sk[2], BLK)) return B200_ERR_UNSUPPORTED;
  if (!encode_qkv_map(&tv, dtype, v, Z, H, N, D, sv[0], sv[1], sv[2], BLK)) return B200_ERR_UNSUPPORTED;
  CUtensorMap to;
  FwdParams p{};
  // O through TMA stores (boxes of 32 rows x 64 columns) when its layout allows, else direct stores
  p.o_tma = encode_qkv_map(&to, dtype, o, Z, H, N, D, so[0], so[1], so[2], 32) ? 1 : 0;
  if (!p.o_tma) to = tq;
  p.o = o; p.m = m; p.row_max = row_max;
  p.o_sz = so[0]; p.o_sh = so[1]; p.o_sn = so[2];
  p.Z = Z; p.H = H; p.N = N; p.causal = causal;
  p.scale_log2 = sm_scale * 1.44269504f;  // the reference's constant (06-fused-attention.py:161)
  const int item_rows = (D == 256) ? BLK : 2 * BLK;  // one 128-row tile per work item at head dim 256, two otherwise
  p.num_qb = (N + item_rows - 1) / item_rows;
  p.total_items = p.num_qb * Z * H;
  p.status = ctx->status;
  p.sched_counter = next_sched_counter(ctx, stream);
  if (!p.sched_counter) return B200_ERR_CUDA;
  const bool bf16 = dtype == B200_BF16;
  if (D == 256) return bf16 ? launch_fwd_t<256, true>(ctx, stream, tq, tk, tv, to, p) : launch_fwd_t<256, false>(ctx, stream, tq, tk, tv, to, p);
  if (D == 128) return bf16 ? launch_fwd_t<128, true>(ctx, stream, tq, tk, tv, to, p) : launch_fwd_t<128, false>(ctx, stream, tq, tk, tv, to, p);
  if (D == 64) return bf16 ? launch_fwd_t<64, true>(ctx, stream, tq, tk, tv, to, p) : launch_fwd_t<64, false>(ctx, stream, tq, tk, tv, to, p);
  return fail(B200_ERR_UNSUPPORTED, "head dim %d: the forward has kernels for 64, 128 and 256", D);
}

}  // namespace tb
