// Flash-attention backward for sm_100a.
//
// Computes what the reference's backward computes (python/tutorials/06-fused-attention.py:190-435,
// 478-517), with its decomposition: a pre-pass delta = rowsum(O * dO) (_attn_bwd_preprocess), then
// per 128-row K/V block dK and dV from a loop over Q blocks (_attn_bwd_dkdv), and per 128-row Q
// block dQ from a loop over K/V blocks (_attn_bwd_dq).  No atomics: every output element has one
// writer, results are deterministic.  P and dS are rounded to the storage type before the second
// products (:244, :251, :297), everything else is fp32.  The reference folds sm_scale/ln2 into a
// 16-bit copy of K on the host (:491-492); here the fp32 scores are scaled instead, which saves
// the extra pass over K and one rounding.
//
// Both main kernels are one pipeline (template parameter DQ):
//   resident operands R1, R2 (128 x D each) stay in shared memory, the other side streams through
//   a ring as pairs (U1, U2) of 128 x D tiles.  Per step
//       T1 = R1 U1^T        (scores: S^T = K Q^T, or S = Q K^T)
//       T2 = R2 U2^T        (dP^T = V dO^T, or dP = dO V^T)
//       P  = exp2(T1 * scale - M) masked;   dS = P * (T2 - delta)       (fp32, two threads per row)
//       accB += P  U2       (dV += P^T dO; dK/dV kernel only)
//       accA += dS U1       (dK += dS^T Q, or dQ += dS K)
//   T1/T2 live in TMEM (at head dim 64 there are two T1 buffers used in turn, so T1 of the next
//   step is computed during this step) and P/dS overwrite them as 16-bit A operands of the last two MMAs (each
//   thread over the first 32 of its own 64 columns), which read U1/U2 through an N-major view of
//   the same shared-memory tiles.  Gradients leave through staging buffers and TMA stores.
// Warps 0-7 compute (two threads per row, splitting the columns), warp 8 issues MMAs, warp 9 runs TMA.
#include <cmath>
#include <mutex>

#include "common.cuh"
#include "host.h"

namespace tb {

namespace {

constexpr int BLK = 128;
constexpr int BWD_THREADS = 320;  // 8 compute warps + MMA warp + TMA warp

struct BwdParams {
  const float* m;      // [Z*H, N] base-2 LSE from the forward
  const float* delta;  // [Z*H, N]
  void* out_a;         // dK (dK/dV kernel) or dQ (dQ kernel)
  void* out_b;         // dV (dK/dV kernel)
  long long oa_sz, oa_sh, oa_sn, ob_sz, ob_sh, ob_sn;
  int Z, H, N;
  int causal;
  float scale_log2;  // sm_scale * log2(e)
  float sm_scale;
  int total_items;     // (N / 128) * Z * H
  int* sched_counter;  // work counter of this launch: zero at launch, put back to zero by the last CTA
  int out_tma;         // gradients are written through shared-memory staging and TMA stores
  unsigned* status;
};

template <int D>
struct BwdCfg {
  static constexpr int TILE = BLK * D * 2;
  static constexpr int NST = (D == 128) ? 2 : 3;
  static constexpr int STAGE = 2 * TILE + 1024;  // U1, U2, column statistics (M, delta of the streamed rows)
  static constexpr int STG_BYTES = 32 * 64;  // epilogue staging of one compute warp: 32 rows x 32 columns
  static constexpr size_t SMEM = 2 * TILE + (size_t)NST * STAGE + 8 * STG_BYTES + (2 * NST + 16) * 8 + 32 + 1024;
};

template <int D>
__device__ __forceinline__ void load_tile_b(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int row0, int h, int z) {
#pragma unroll
  for (int b = 0; b < D / 64; ++b) tma_load_4d(dst + b * (BLK * 128), map, bar, b * 64, row0, h, z);
}

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// DQ = false: block = K/V block, R1 = K, R2 = V, stream (Q_i, dO_i), outputs dK (A), dV (B)
// DQ = true : block = Q block,  R1 = Q, R2 = dO, stream (K_j, V_j), output dQ (A)
// Persistent: one CTA per SM takes (block, head) items from an atomic counter, head-major and
// heavy-first; the epilogue of an item overlaps the loads and first MMAs of the next one.
template <bool DQ>
struct BwdItem {
  int blk, zh, z, h, t_lo, t_hi;
  __device__ BwdItem(const BwdParams& p, int w) {
    const int nblk = p.N / BLK;
    zh = w / nblk;
    const int pos = w % nblk;
    // the dK/dV kernel's early K/V blocks and the dQ kernel's late Q blocks see the most steps
    blk = DQ ? (nblk - 1 - pos) : pos;
    z = zh / p.H;
    h = zh % p.H;
    t_lo = DQ ? 0 : (p.causal ? blk : 0);        // streamed block range [t_lo, t_hi)
    t_hi = DQ ? (p.causal ? blk + 1 : nblk) : nblk;
  }
};

template <int D, bool BF16, bool DQ>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_r1, const __grid_constant__ CUtensorMap tm_r2,
                const __grid_constant__ CUtensorMap tm_u1, const __grid_constant__ CUtensorMap tm_u2,
                const __grid_constant__ CUtensorMap tm_oa, const __grid_constant__ CUtensorMap tm_ob,
                const BwdParams p) {
  using Cfg = BwdCfg<D>;
  constexpr int TILE = Cfg::TILE, NST = Cfg::NST, STAGE = Cfg::STAGE;
  constexpr int MMA_WARP = 8, TMA_WARP = 9;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  uint8_t* sres = smem;                 // R1, R2
  uint8_t* sring = smem + 2 * TILE;     // stages
  uint8_t* sstage = sring + NST * STAGE;  // 8 x 2 KiB epilogue staging, rows of 64 bytes, not swizzled
  uint64_t* bars = reinterpret_cast<uint64_t*>(sstage + 8 * Cfg::STG_BYTES);
  uint64_t* r_full = bars;              // resident tiles of the item loaded
  uint64_t* r_empty = bars + 1;         // every T MMA of the item has read them
  uint64_t* full = bars + 2;            // [NST]
  uint64_t* empty = full + NST;         // [NST]
  uint64_t* t1_full = empty + NST;      // [2] T1(t) in TMEM (head dim 64: two T1 buffers used in turn, one barrier each)
  uint64_t* t2_full = t1_full + 2;      // T2(t) in TMEM
  uint64_t* p_full = t2_full + 1;       // P(t) written (dK/dV kernel)
  uint64_t* ds_full = p_full + 1;       // dS(t) written
  uint64_t* acc_full = ds_full + 1;     // accumulators of the item final
  uint64_t* sched_full = acc_full + 1;  // [2] an item id was published
  uint64_t* sched_empty = sched_full + 2;  // [2] all 9 readers have taken it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sched_empty + 2);
  volatile int* sched_item = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  B200_TRACE_DECL;  // trace builds: region 0 / 1 = first compute warp of the dK/dV / dQ kernel

  if (threadIdx.x == 0) {
    mbar_init(r_full, 1);
    mbar_init(r_empty, 1);
    for (int s = 0; s < NST; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&t1_full[0], 1);
    mbar_init(&t1_full[1], 1);
    mbar_init(t2_full, 1);
    mbar_init(p_full, 256);
    mbar_init(ds_full, 256);
    mbar_init(acc_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sched_full[i], 1);
      mbar_init(&sched_empty[i], 9);  // MMA thread + one lane of each compute warp
    }
    fence_barrier_init();
    cta_wait_flag_clear();
    tma_prefetch_desc(&tm_r1);
    tma_prefetch_desc(&tm_r2);
    tma_prefetch_desc(&tm_u1);
    tma_prefetch_desc(&tm_u2);
  }
  if (warp == MMA_WARP) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const uint32_t tm_t2 = tmem_base + 128, tm_a = tmem_base + 256, tm_b = tmem_base + 256 + D;
  // At head dim 64, and in the dQ kernel (one accumulator) at either head dim, the accumulators
  // leave 128 TMEM columns free: a second T1 buffer, so that the scores of step t+1 are computed
  // while the compute warps still work on step t (P / dS overwrite T1 / T2 in place, so with one
  // buffer T1(t+1) has to wait until P(t) has been consumed).
  constexpr bool DB = (D == 64) || DQ;
  auto t1_addr = [&](uint32_t step) { return tmem_base + ((DB && (step & 1u)) ? 384u : 0u); };
  auto t1_bar = [&](uint32_t step) { return &t1_full[DB ? (step & 1u) : 0u]; };
  auto t1_parity = [&](uint32_t step) { return DB ? ((step >> 1) & 1u) : (step & 1u); };

  if (warp == TMA_WARP) {
    // ------------------------------------------------------------------ scheduler + TMA producer
    if (lane == 0) {
      uint32_t s = 0, ph = 0;  // ring position, runs on across items
      for (uint32_t n = 0;; ++n) {
        const int w = atomicAdd(p.sched_counter, 1);
        const uint32_t slot = n & 1u, sph = (n >> 1) & 1u;
        mbar_wait(&sched_empty[slot], sph ^ 1u, p.status, SITE_BWD_SCHED);
        sched_item[slot] = w;
        mbar_arrive(&sched_full[slot]);
        // every CTA draws exactly one ticket past the end: the last of them puts the zero back for the
        // next launch that is handed this counter
        if (w == p.total_items + (int)gridDim.x - 1) atomicExch(p.sched_counter, 0);
        if (w >= p.total_items) break;
        const BwdItem<DQ> it(p, w);
        mbar_wait(r_empty, (n & 1u) ^ 1u, p.status, SITE_BWD_KV);  // the previous item no longer reads R1, R2
        mbar_expect_tx(r_full, 2 * TILE);
        load_tile_b<D>(sres, &tm_r1, r_full, it.blk * BLK, it.h, it.z);
        load_tile_b<D>(sres + TILE, &tm_r2, r_full, it.blk * BLK, it.h, it.z);
        for (int t = it.t_lo; t < it.t_hi; ++t) {
          mbar_wait(&empty[s], ph ^ 1u, p.status, SITE_BWD_LOAD_EMPTY);
          uint8_t* st = sring + s * STAGE;
          mbar_expect_tx(&full[s], 2 * TILE + (DQ ? 0 : 1024));
          load_tile_b<D>(st, &tm_u1, &full[s], t * BLK, it.h, it.z);
          load_tile_b<D>(st + TILE, &tm_u2, &full[s], t * BLK, it.h, it.z);
          if (!DQ) {  // statistics of the streamed Q rows: M then delta, 128 floats each
            bulk_load(st + 2 * TILE, p.m + (long long)it.zh * p.N + t * BLK, 512, &full[s]);
            bulk_load(st + 2 * TILE + 512, p.delta + (long long)it.zh * p.N + t * BLK, 512, &full[s]);
          }
          if (++s == NST) { s = 0; ph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    {  // the warp stays converged; an elected lane issues (descriptor arithmetic stays warp-uniform)
      constexpr int FMT = BF16 ? 1 : 0;
      constexpr uint32_t IDESC_T = make_idesc(FMT, FMT, 0, 0, 128, BLK);  // R (K-major) x U (K-major)
      constexpr uint32_t IDESC_ACC = make_idesc(FMT, FMT, 0, 1, 128, D);  // P/dS (TMEM) x U (N-major)
      const uint64_t dr0 = smem_desc_sw128(smem_u32(sres), 0, 1024);
      const uint64_t du0 = smem_desc_sw128(smem_u32(sring), 0, 1024);
      const uint64_t dun0 = smem_desc_sw128(smem_u32(sring), BLK * 128, 1024);  // N-major view of a streamed tile

      auto issue_t = [&](uint32_t tm, uint64_t dr, uint64_t du) {  // T = R U^T, D/16 MMAs
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * ((BLK * 128) >> 4) + (kk & 3) * 2;
          umma_ss_elect<false>(tm, dr + off, du + off, IDESC_T, kk != 0);
        }
      };
      auto issue_acc = [&](uint32_t tm_acc, uint32_t tm_opnd, uint64_t dun, uint32_t accum) {  // acc (+)= X U, 8 MMAs
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk)
          umma_ts_f16_elect(tm_acc, tm_opnd + (kk >> 2) * 64 + (kk & 3) * 8, dun + kk * ((16 * 128) >> 4), IDESC_ACC,
                            (accum | kk) != 0);
      };

      uint32_t s = 0, ph = 0;  // ring position
      uint32_t cnt = 0;        // steps done so far, across items (parity of p_full / ds_full)
      for (uint32_t n = 0;; ++n) {
        const uint32_t slot = n & 1u, sph = (n >> 1) & 1u;
        mbar_wait(&sched_full[slot], sph, p.status, SITE_BWD_SCHED);
        const int w = sched_item[slot];
        __syncwarp();
        if (lane == 0) mbar_arrive(&sched_empty[slot]);
        if (w >= p.total_items) break;
        const BwdItem<DQ> item(p, w);
        const int steps = item.t_hi - item.t_lo;  // >= 1

        mbar_wait(r_full, n & 1u, p.status, SITE_BWD_KV);
        mbar_wait(&full[s], ph, p.status, SITE_BWD_LOAD_FULL);
        issue_t(t1_addr(cnt), dr0, du0 + s * (STAGE >> 4));
        tc_commit_elect(t1_bar(cnt));
        issue_t(tm_t2, dr0 + (TILE >> 4), du0 + s * (STAGE >> 4) + (TILE >> 4));
        tc_commit_elect(t2_full);
        if (steps == 1) tc_commit_elect(r_empty);
        for (int it = 0; it < steps; ++it, ++cnt) {
          const uint32_t cs = s;
          uint32_t ns = s + 1, nph = ph;
          if (ns == NST) { ns = 0; nph ^= 1u; }
          const uint64_t dun1 = dun0 + cs * (STAGE >> 4), dun2 = dun1 + (TILE >> 4);
          const bool more = it + 1 < steps;
          if (DB && more) {
            // two T1 buffers: the other one was last read two steps ago (its P by the dV MMAs issued
            // in that step, or by the compute warps before that step's ds_full)
            mbar_wait(&full[ns], nph, p.status, SITE_BWD_LOAD_FULL);
            issue_t(t1_addr(cnt + 1), dr0, du0 + ns * (STAGE >> 4));
            tc_commit_elect(t1_bar(cnt + 1));
          }
          if (!DQ) {
            mbar_wait(p_full, cnt & 1u, p.status, SITE_BWD_P_FULL);
            tc_fence_after();
            issue_acc(tm_b, t1_addr(cnt), dun2, it > 0);  // dV += P^T dO
          }
          if (!DB && more) {
            mbar_wait(&full[ns], nph, p.status, SITE_BWD_LOAD_FULL);
            if (!DQ) {  // T1 of the next step may start as soon as P was consumed (in-order pipe)
              issue_t(t1_addr(cnt + 1), dr0, du0 + ns * (STAGE >> 4));
              tc_commit_elect(t1_bar(cnt + 1));
            }
          }
          mbar_wait(ds_full, cnt & 1u, p.status, SITE_BWD_DS_FULL);
          tc_fence_after();
          issue_acc(tm_a, tm_t2, dun1, it > 0);  // dK += dS^T Q   /   dQ += dS K
          tc_commit_elect(&empty[cs]);
          if (more) {
            if (DQ && !DB) {  // no MMA consumes P here: T1 is free once the compute warps have read it (ds_full)
              issue_t(t1_addr(cnt + 1), dr0, du0 + ns * (STAGE >> 4));
              tc_commit_elect(t1_bar(cnt + 1));
            }
            issue_t(tm_t2, dr0 + (TILE >> 4), du0 + ns * (STAGE >> 4) + (TILE >> 4));
            tc_commit_elect(t2_full);
            if (it + 2 == steps) tc_commit_elect(r_empty);  // those were the item's last reads of R1, R2
          }
          s = ns; ph = nph;
        }
        tc_commit_elect(acc_full);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ compute
    // Two threads per row: warps w and w+4 own the same TMEM lanes and split the 128 columns of
    // T1 / T2 (and, in the epilogue, of the accumulators) in halves.  Each thread packs its P and
    // dS over the first 32 of its OWN 64 columns (the MMA reads its A operand from columns
    // [0, 32) and [64, 96)), so the two halves never touch each other's columns and need no
    // barrier between them: they may drift apart, and one half's exponentials overlap the other
    // half's dS arithmetic on the same scheduler.
    const uint32_t quarter = warp & 3u;
    const int half = warp >> 2;
    constexpr int HC = BLK / 2, HD = D / 2;
    const int r = quarter * 32 + lane;       // row inside the block
    const uint32_t lane_addr = (quarter * 32u) << 16;
    const float scale = p.scale_log2;
    uint32_t s = 0;    // ring position
    uint32_t cnt = 0;  // steps done so far, across items (parity of t1_full / t2_full)

    for (uint32_t n = 0;; ++n) {
      const uint32_t slot = n & 1u, sph = (n >> 1) & 1u;
      int w = 0;
      if (lane == 0) {
        mbar_wait(&sched_full[slot], sph, p.status, SITE_BWD_SCHED);
        w = sched_item[slot];
        mbar_arrive(&sched_empty[slot]);
      }
      w = __shfl_sync(0xffffffffu, w, 0);
      if (w >= p.total_items) break;
      const BwdItem<DQ> item(p, w);
      const int blk = item.blk, zh = item.zh;
      const int grow = blk * BLK + r;  // kv index (dK/dV kernel) or q index (dQ kernel)
      float m_row = 0.f, d_row = 0.f;
      if (DQ) {
        m_row = p.m[(long long)zh * p.N + grow];
        d_row = p.delta[(long long)zh * p.N + grow];
      }
      const int steps = item.t_hi - item.t_lo;
      for (int it = 0; it < steps; ++it, ++cnt) {
        const int t = item.t_lo + it;
        const float* sm = reinterpret_cast<const float*>(sring + s * STAGE + 2 * TILE) + half * HC;  // column M
        const float* sd = sm + 128;                                                                  // column delta
        // the diagonal block is the only one that needs the causal mask
        const bool diag = p.causal && (t == blk);
        const bool traced = warp == 0 && lane == 0;  // used by trace builds only
        if (traced) B200_TRACE_EVENT(p.status, DQ ? 1 : 0, 0x100 | steps);
        const uint32_t tm_t1 = t1_addr(cnt);
        mbar_wait(t1_bar(cnt), t1_parity(cnt), p.status, SITE_BWD_S_FULL);
        if (traced) B200_TRACE_EVENT(p.status, DQ ? 1 : 0, 1);
        tc_fence_after();
        uint32_t pr[HC];  // P as fp32 bits
#pragma unroll
        for (int c = 0; c < HC; c += 32) tmem_ld32(tm_t1 + lane_addr + half * HC + c, pr + c);
        tmem_ld_wait();
#pragma unroll
        for (int c4 = 0; c4 < HC; c4 += 4) {
          // column statistics: one 16-byte broadcast load for four columns
          const float4 m4 = DQ ? make_float4(m_row, m_row, m_row, m_row) : *reinterpret_cast<const float4*>(sm + c4);
          const float mq[4] = {m4.x, m4.y, m4.z, m4.w};
          // packed fp32 arithmetic (one issue slot per column pair) for the scaling
          float xs[4];
          upk2(fma2(pk2(__uint_as_float(pr[c4]), __uint_as_float(pr[c4 + 1])), pk2(scale, scale), pk2(-mq[0], -mq[1])), xs[0], xs[1]);
          upk2(fma2(pk2(__uint_as_float(pr[c4 + 2]), __uint_as_float(pr[c4 + 3])), pk2(scale, scale), pk2(-mq[2], -mq[3])), xs[2], xs[3]);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int c = c4 + u;
            float pv = ex2(xs[u]);
            // dK/dV kernel: row = kv, column = q, keep q >= kv.   dQ kernel: row = q, column = kv, keep kv <= q.
            const int cc = half * HC + c;
            if (diag && (DQ ? (cc > r) : (cc < r))) pv = 0.f;
            pr[c] = __float_as_uint(pv);
          }
        }
        if (!DQ) {
#pragma unroll
          for (int c = 0; c < HC; c += 32) {
            uint32_t wv[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) wv[k] = pack2<BF16>(__uint_as_float(pr[c + 2 * k]), __uint_as_float(pr[c + 2 * k + 1]));
            tmem_st16(tm_t1 + lane_addr + half * HC + (c >> 1), wv);  // over the first 32 of the own 64 columns
          }
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive(p_full);
        }
        if (traced) B200_TRACE_EVENT(p.status, DQ ? 1 : 0, 2);
        mbar_wait(t2_full, cnt & 1u, p.status, SITE_BWD_DP_FULL);
        if (traced) B200_TRACE_EVENT(p.status, DQ ? 1 : 0, 3);
        tc_fence_after();
        uint32_t dsw[HC / 2];  // dS packed to 16 bit
#pragma unroll
        for (int c = 0; c < HC; c += 32) {
          uint32_t dp[32];
          tmem_ld32(tm_t2 + lane_addr + half * HC + c, dp);
          tmem_ld_wait();
#pragma unroll
          for (int k4 = 0; k4 < 32; k4 += 4) {
            const float4 d4 = DQ ? make_float4(d_row, d_row, d_row, d_row) : *reinterpret_cast<const float4*>(sd + c + k4);
            float ds0, ds1, ds2, ds3;  // dS = P (dP - delta), two columns per instruction
            upk2(mul2(pk2(__uint_as_float(pr[c + k4]), __uint_as_float(pr[c + k4 + 1])),
                      sub2(pk2(__uint_as_float(dp[k4]), __uint_as_float(dp[k4 + 1])), pk2(d4.x, d4.y))), ds0, ds1);
            upk2(mul2(pk2(__uint_as_float(pr[c + k4 + 2]), __uint_as_float(pr[c + k4 + 3])),
                      sub2(pk2(__uint_as_float(dp[k4 + 2]), __uint_as_float(dp[k4 + 3])), pk2(d4.z, d4.w))), ds2, ds3);
            dsw[((c + k4) >> 1)] = pack2<BF16>(ds0, ds1);
            dsw[((c + k4) >> 1) + 1] = pack2<BF16>(ds2, ds3);
          }
        }
#pragma unroll
        for (int c = 0; c < HC / 2; c += 16) tmem_st16(tm_t2 + lane_addr + half * HC + c, dsw + c);  // own columns
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(ds_full);
        if (traced) B200_TRACE_EVENT(p.status, DQ ? 1 : 0, 4);
        if (++s == NST) s = 0;
      }

      // epilogue: each thread stores its half of the accumulator columns.  It overlaps the next
      // item's loads and first T MMAs; the next item's first accumulate MMA needs this warp's next
      // P / dS, i.e. comes after these reads in program order.
      mbar_wait(acc_full, n & 1u, p.status, SITE_BWD_ACC_FULL);
      if (warp == 0 && lane == 0) B200_TRACE_EVENT(p.status, DQ ? 1 : 0, 8);
      tc_fence_after();
      auto store_rows = [&](uint32_t tm_acc, const CUtensorMap* map, void* out, long long sz, long long sh,
                            long long sn, float mul) {
        if (p.out_tma) {
          // 32 columns at a time through this warp's staging buffer and a TMA store (a warp-wide
          // store of one row per lane touches 32 lines per instruction); rows past N are clipped
          uint8_t* stg = sstage + warp * Cfg::STG_BYTES;
          const int warp_row0 = blk * BLK + quarter * 32;
#pragma unroll 1
          for (int c = 0; c < HD; c += 32) {
            uint32_t o[32];
            tmem_ld32(tm_acc + lane_addr + half * HD + c, o);
            tmem_ld_wait();
            if (lane == 0) tma_store_wait_read<0>();  // the previous store has read the staging buffer
            __syncwarp();
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              uint32_t wv[4];
#pragma unroll
              for (int k = 0; k < 4; ++k)
                wv[k] = pack2<BF16>(__uint_as_float(o[8 * ch + 2 * k]) * mul, __uint_as_float(o[8 * ch + 2 * k + 1]) * mul);
              *reinterpret_cast<uint4*>(stg + lane * 64 + ch * 16) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && warp_row0 < p.N) {
              tma_store_4d(map, stg, half * HD + c, warp_row0, item.h, item.z);
              tma_store_commit();
            }
          }
          return;
        }
        uint16_t* orow = reinterpret_cast<uint16_t*>(out) + (long long)item.z * sz + (long long)item.h * sh +
                         (long long)grow * sn + half * HD;
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(out) & 15) == 0) && ((sn & 7) == 0) && ((sh & 7) == 0) && ((sz & 7) == 0);
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
          uint32_t o[32];
          tmem_ld32(tm_acc + lane_addr + half * HD + c, o);
          tmem_ld_wait();
          uint32_t wv[16];
#pragma unroll
          for (int k = 0; k < 16; ++k) wv[k] = pack2<BF16>(__uint_as_float(o[2 * k]) * mul, __uint_as_float(o[2 * k + 1]) * mul);
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
      };
      store_rows(tm_a, &tm_oa, p.out_a, p.oa_sz, p.oa_sh, p.oa_sn, p.sm_scale);  // dK or dQ carry sm_scale
      if (!DQ) store_rows(tm_b, &tm_ob, p.out_b, p.ob_sz, p.ob_sh, p.ob_sn, 1.0f);
      if (warp == 0 && lane == 0) B200_TRACE_EVENT(p.status, DQ ? 1 : 0, 9);
    }
    if (p.out_tma && lane == 0) tma_store_wait_read<0>();  // the staging buffer has been read: the CTA may exit, the writes land on their own
  }

  cta_linger_after_failure();
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[zh, n] = sum_d O * dO in fp32 (_attn_bwd_preprocess, 06-fused-attention.py:190-204).
// HBM-bound: each thread reads 8 elements (16 bytes) of O and of dO for four rows at a time (eight
// independent loads in flight), D/8 threads per row, a shuffle reduction per row.
template <int D, bool BF16>
__global__ void __launch_bounds__(256)
attn_bwd_delta_kernel(const uint16_t* __restrict__ o, const uint16_t* __restrict__ dout, float* __restrict__ delta,
                      long long o_sz, long long o_sh, long long o_sn, long long d_sz, long long d_sh, long long d_sn,
                      unsigned H, unsigned N, unsigned rows_total, float* __restrict__ zero_rows) {
  constexpr int TPR = D / 8;           // threads per row
  constexpr unsigned RPB = 256 / TPR;  // rows per block and step
  constexpr int U = 4;                 // rows per thread in flight (independent 16-byte loads)
  const unsigned part = threadIdx.x % TPR, rib = threadIdx.x / TPR;
  // 32-bit index arithmetic: 64-bit divisions per row made this kernel ALU-bound
  for (unsigned base = blockIdx.x * (RPB * U); base < rows_total; base += gridDim.x * (RPB * U)) {
    uint4 ov[U], dv[U];
    unsigned rows[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned row = base + u * RPB + rib;
      rows[u] = row;
      ov[u] = dv[u] = make_uint4(0, 0, 0, 0);
      if (row < rows_total) {
        const unsigned n = row % N, zh = row / N, hh = zh % H, zz = zh / H;
        ov[u] = *reinterpret_cast<const uint4*>(o + zz * o_sz + hh * o_sh + (long long)n * o_sn + part * 8);
        dv[u] = *reinterpret_cast<const uint4*>(dout + zz * d_sz + hh * d_sh + (long long)n * d_sn + part * 8);
        if (zero_rows) {  // the one-pass backward's fp32 dQ accumulator, [rows][D]: cleared on the way
          float4* z = reinterpret_cast<float4*>(zero_rows + (long long)row * D + part * 8);
          z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
          z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t ow[4] = {ov[u].x, ov[u].y, ov[u].z, ov[u].w}, dw[4] = {dv[u].x, dv[u].y, dv[u].z, dv[u].w};
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 a, b;
        if (BF16) {
          a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ow[k]));
          b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dw[k]));
        } else {
          a = __half22float2(*reinterpret_cast<const __half2*>(&ow[k]));
          b = __half22float2(*reinterpret_cast<const __half2*>(&dw[k]));
        }
        acc = fmaf(a.x, b.x, acc);
        acc = fmaf(a.y, b.y, acc);
      }
#pragma unroll
      for (int off = TPR / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (rows[u] < rows_total && part == 0) delta[rows[u]] = acc;
    }
  }
}

template <int D, bool BF16>
int launch_delta_t(DeviceCtx* ctx, cudaStream_t stream, const void* o, const void* dout, float* delta, const int64_t* so,
                   const int64_t* sdo, int Z, int H, int N, float* zero_rows = nullptr) {
  const long long rows = (long long)Z * H * N;
  if (rows >= (1ll << 32)) return fail(B200_ERR_UNSUPPORTED, "more than 2^32 rows");
  const long long rows_per_block = (256 / (D / 8)) * 4;
  long long blocks = (rows + rows_per_block - 1) / rows_per_block;
  if (blocks > (long long)ctx->sm_count * 16) blocks = (long long)ctx->sm_count * 16;
  attn_bwd_delta_kernel<D, BF16><<<(unsigned)blocks, 256, 0, stream>>>(
      reinterpret_cast<const uint16_t*>(o), reinterpret_cast<const uint16_t*>(dout), delta, so[0], so[1], so[2],
      sdo[0], sdo[1], sdo[2], (unsigned)H, (unsigned)N, (unsigned)rows, zero_rows);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "attn bwd delta launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

template <int D, bool BF16, bool DQ>
int launch_bwd_t(DeviceCtx* ctx, cudaStream_t stream, const CUtensorMap& r1, const CUtensorMap& r2,
                 const CUtensorMap& u1, const CUtensorMap& u2, const CUtensorMap& oa, const CUtensorMap& ob,
                 const BwdParams& p) {
  static std::atomic<bool> attr_done[64];
  constexpr size_t smem = BwdCfg<D>::SMEM;
  if (int rc = ensure_dynamic_smem(attn_bwd_kernel<D, BF16, DQ>, smem, ctx->device, attr_done, "attn bwd")) return rc;
  BwdParams q = p;
  q.total_items = (p.N / BLK) * p.Z * p.H;
  q.sched_counter = next_sched_counter(ctx, stream);
  if (!q.sched_counter) return B200_ERR_CUDA;
  const int grid = q.total_items < ctx->sm_count ? q.total_items : ctx->sm_count;
  attn_bwd_kernel<D, BF16, DQ><<<grid, BWD_THREADS, smem, stream>>>(r1, r2, u1, u2, oa, ob, q);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "attn bwd launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

template <int D, bool BF16>
int launch_bwd_all(DeviceCtx* ctx, cudaStream_t stream, const void* o, const void* dout, float* delta,
                   const int64_t* so, const int64_t* sdo, const CUtensorMap& tq, const CUtensorMap& tk,
                   const CUtensorMap& tv, const CUtensorMap& tdo, BwdParams p, void* dq, void* dk, void* dv,
                   const int64_t* sdq, const int64_t* sdk, const int64_t* sdv) {
  if (int rc = launch_delta_t<D, BF16>(ctx, stream, o, dout, delta, so, sdo, p.Z, p.H, p.N)) return rc;
  p.delta = delta;
  // gradients through TMA stores (boxes of 32 rows x 32 columns) when all three layouts allow
  CUtensorMap mdq, mdk, mdv;
  const int dt = BF16 ? B200_BF16 : B200_F16;
  p.out_tma = encode_rows_map(&mdq, dt, dq, p.Z, p.H, p.N, D, sdq[0], sdq[1], sdq[2], 32, 32, false) &&
              encode_rows_map(&mdk, dt, dk, p.Z, p.H, p.N, D, sdk[0], sdk[1], sdk[2], 32, 32, false) &&
              encode_rows_map(&mdv, dt, dv, p.Z, p.H, p.N, D, sdv[0], sdv[1], sdv[2], 32, 32, false);
  if (!p.out_tma) mdq = mdk = mdv = tq;
  // dK, dV: resident (K, V), streamed (Q, dO)
  p.out_a = dk; p.oa_sz = sdk[0]; p.oa_sh = sdk[1]; p.oa_sn = sdk[2];
  p.out_b = dv; p.ob_sz = sdv[0]; p.ob_sh = sdv[1]; p.ob_sn = sdv[2];
  int rc = launch_bwd_t<D, BF16, false>(ctx, stream, tk, tv, tq, tdo, mdk, mdv, p);
  if (rc) return rc;
  // dQ: resident (Q, dO), streamed (K, V)
  p.out_a = dq; p.oa_sz = sdq[0]; p.oa_sh = sdq[1]; p.oa_sn = sdq[2];
  p.out_b = nullptr;
  return launch_bwd_t<D, BF16, true>(ctx, stream, tq, tdo, tk, tv, mdq, mdq, p);
}

}  // namespace

// delta = rowsum(O * dO) for any head dim of the library (the pre-pass on its own); zero_rows: optional
// contiguous fp32 [Z*H*N][D] buffer that the same pass clears (head dim 64 only)
int launch_attn_bwd_delta(DeviceCtx* ctx, cudaStream_t stream, const void* o, const void* dout, float* delta, int Z,
                          int H, int N, int D, const int64_t* so, const int64_t* sdo, int dtype, float* zero_rows) {
  const bool bf16 = dtype == B200_BF16;
  if (zero_rows && D != 64) return fail(B200_ERR_ARG, "the pre-pass clears an accumulator at head dim 64 only");
  switch (D) {
    case 64: return bf16 ? launch_delta_t<64, true>(ctx, stream, o, dout, delta, so, sdo, Z, H, N, zero_rows)
                         : launch_delta_t<64, false>(ctx, stream, o, dout, delta, so, sdo, Z, H, N, zero_rows);
    case 128: return bf16 ? launch_delta_t<128, true>(ctx, stream, o, dout, delta, so, sdo, Z, H, N)
                          : launch_delta_t<128, false>(ctx, stream, o, dout, delta, so, sdo, Z, H, N);
    case 256: return bf16 ? launch_delta_t<256, true>(ctx, stream, o, dout, delta, so, sdo, Z, H, N)
                          : launch_delta_t<256, false>(ctx, stream, o, dout, delta, so, sdo, Z, H, N);
    default: return fail(B200_ERR_UNSUPPORTED, "head dim %d", D);
  }
}

// ---------------------------------------------------------------------------------------------
// Built-in scratch for b200_attention_bwd_noalloc: the delta vector lives in this fixed device
// array instead of caller memory.  Every GPU that loads the library holds these 4 MiB until the
// process exits.  In host code the name below is only a host-side stand-in for the symbol, not a
// device address, so the address is looked up once per device with cudaGetSymbolAddress.
constexpr long long kScratchFloats = 1ll << 20;  // rows (Z*H*N) one call may use
static __device__ __align__(256) float g_delta_scratch[kScratchFloats];

long long attn_bwd_scratch_capacity() { return kScratchFloats; }

// Device address of the scratch array on the CURRENT device (looked up on first use per device).
float* attn_bwd_scratch(DeviceCtx* ctx) {
  static std::mutex mu;
  static float* ptr[64] = {};
  std::lock_guard<std::mutex> lk(mu);
  if (!ptr[ctx->device]) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_delta_scratch);
    if (e != cudaSuccess || !p) {
      fail(B200_ERR_CUDA, "cudaGetSymbolAddress(delta scratch): %s", cudaGetErrorString(e));
      return nullptr;
    }
    ptr[ctx->device] = p;
  }
  return ptr[ctx->device];
}

int launch_attn_bwd(DeviceCtx* ctx, cudaStream_t stream, const void* q, const void* k, const void* v, const void* o,
                    const void* dout, const float* m, float* delta, void* dq, void* dk, void* dv, int Z, int H, int N,
                    int D, const int64_t* sq, const int64_t* sk, const int64_t* sv, const int64_t* so,
                    const int64_t* sdo, const int64_t* sdq, const int64_t* sdk, const int64_t* sdv, float sm_scale,
                    int causal, int dtype) {
  CUtensorMap tq, tk, tv, tdo;
  if (!encode_qkv_map(&tq, dtype, q, Z, H, N, D, sq[0], sq[1], sq[2], BLK)) return B200_ERR_UNSUPPORTED;
  if (!encode_qkv_map(&tk, dtype, k, Z, H, N, D, sk[0], sk[1], sk[2], BLK)) return B200_ERR_UNSUPPORTED;
  if (!encode_qkv_map(&tv, dtype, v, Z, H, N, D, sv[0], sv[1], sv[2], BLK)) return B200_ERR_UNSUPPORTED;
  if (!encode_qkv_map(&tdo, dtype, dout, Z, H, N, D, sdo[0], sdo[1], sdo[2], BLK)) return B200_ERR_UNSUPPORTED;
  for (const int64_t* s : {so, sdo}) {
    if ((s[0] & 7) || (s[1] & 7) || (s[2] & 7)) return fail(B200_ERR_UNSUPPORTED, "O / dO strides must be multiples of 8 elements");
  }
  if ((reinterpret_cast<uintptr_t>(o) & 15) || (reinterpret_cast<uintptr_t>(dout) & 15))
    return fail(B200_ERR_UNSUPPORTED, "O / dO must be 16-byte aligned");
  BwdParams p{};
  p.m = m;
  p.Z = Z; p.H = H; p.N = N; p.causal = causal;
  p.scale_log2 = sm_scale * 1.44269504f;
  p.sm_scale = sm_scale;
  p.status = ctx->status;
  const bool bf16 = dtype == B200_BF16;
  if (D == 128) {
    return bf16 ? launch_bwd_all<128, true>(ctx, stream, o, dout, delta, so, sdo, tq, tk, tv, tdo, p, dq, dk, dv, sdq, sdk, sdv)
                : launch_bwd_all<128, false>(ctx, stream, o, dout, delta, so, sdo, tq, tk, tv, tdo, p, dq, dk, dv, sdq, sdk, sdv);
  }
  if (D == 64) {
    return bf16 ? launch_bwd_all<64, true>(ctx, stream, o, dout, delta, so, sdo, tq, tk, tv, tdo, p, dq, dk, dv, sdq, sdk, sdv)
                : launch_bwd_all<64, false>(ctx, stream, o, dout, delta, so, sdo, tq, tk, tv, tdo, p, dq, dk, dv, sdq, sdk, sdv);
  }
  return fail(B200_ERR_UNSUPPORTED, "head dim %d: this library has kernels for 64 and 128", D);
}

}  // namespace tb
