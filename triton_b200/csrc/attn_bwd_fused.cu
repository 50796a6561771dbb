// Flash-attention backward at head dim 64 in ONE pass over the (K/V block, Q block) pairs.
//
// Same arithmetic as the two kernels of attn_bwd.cu (python/tutorials/06-fused-attention.py:190-435):
// per 128-row K/V block (K, V resident in shared memory) and per streamed 128-row Q block
//     T1 = K Q^T (scores, transposed)          T2 = V dO^T (dP, transposed)
//     P  = exp2(T1 * scale - M) masked         dS = P * (T2 - delta)          (fp32, two threads per K/V row)
//     dV += P dO        dK += dS Q             dQ_part = dS^T K               (P, dS rounded to the storage type)
// but the scores, the exponentials and dS are computed once instead of once per kernel: the dS block
// is also written to shared memory (as an M-major A operand) and multiplied with the resident K, and
// that 128 x 64 partial of dQ is added into an fp32 [Z, H, N, 64] buffer by TMA reduce-add
// (cp.reduce.async.bulk.tensor ... add, this GPU's own memory).  This is the reference's older
// "sequence parallel" backward (python/test/regression/test_performance.py:174, 194): partial dQ per
// K/V block, summed afterwards - here summed on the fly by the memory system.  A last element-wise
// kernel scales the sum by sm_scale and rounds it to the storage type.  The order in which the
// partials of one Q block arrive is not fixed, so dQ may differ in its last bit from run to run; dK
// and dV have one writer per element as before.  The two-kernel path stays available
// (deterministic) and serves head dim 128.
//
// Sixteen warps: 0-7 compute (two threads per K/V row, splitting the Q columns), 8-11 drain the dQ
// partial from TMEM into staging buffers and issue the reduce-adds and, at the end of an item, write
// dK and dV (so that the compute warps go straight on to the next item), 12 issues MMAs, 13 runs
// TMA, 14-15 lend registers (setmaxnreg).  K and V are double-buffered: the next item's pair is
// loaded while this item runs.
// TMEM columns: T1 [0,128) T2 [128,256) dK [256,320) dV [320,384) dQ partial [384,448).
#include <cmath>

#define B200_INLINE_WAIT_SLOW  // this kernel re-divides registers between its warpgroups
#include "common.cuh"
#include "host.h"

namespace tb {

namespace {

constexpr int BLK = 128, D = 64;
constexpr int FB_THREADS = 512;
// registers per thread after the re-division; one warp of each warpgroup shares a scheduler's 16K
// registers: (2 * 176 + 88 + 72) * 32 lanes = 16384
constexpr int REGS_COMPUTE = 176, REGS_DRAIN = 88, REGS_OTHER = 72;

struct FusedParams {
  const float* m;      // [Z*H, N] base-2 LSE from the forward
  const float* delta;  // [Z*H, N]
  int Z, H, N;
  int causal;
  float scale_log2;  // sm_scale * log2(e)
  float sm_scale;
  int total_items;     // (N / 128) * Z * H
  int* sched_counter;  // work counter of this launch: zero at launch, put back to zero by the last CTA
  unsigned* status;
};

constexpr int TILE = BLK * D * 2;            // one 128 x 64 tile of 16-bit values
constexpr int NST = 2;                       // stages of the (Q, dO) ring
constexpr int STAGE = 2 * TILE + 1024;       // Q_t, dO_t, M and delta of the streamed rows
constexpr int DS_BYTES = BLK * BLK * 2;      // dS as an M-major operand: two blocks of 64 q x 128 kv rows
constexpr int DQ_STG = 2 * 32 * 128;         // staging of one drain warp: two boxes of 32 rows x 128 bytes (dQ: 32 fp32 columns each; dK, dV: 64 16-bit columns)
constexpr size_t FUSED_SMEM = 4 * TILE + (size_t)NST * STAGE + DS_BYTES + 4 * DQ_STG + (2 * NST + 22) * 8 + 32 + 1024;

__device__ __forceinline__ void load_tile_f(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int row0, int h, int z) {
  tma_load_4d(dst, map, bar, 0, row0, h, z);  // head dim 64: one box of 64 columns x 128 rows
}

__device__ __forceinline__ void bulk_load_f(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// fp32 add of a shared-memory box into global memory (this GPU's own), by the TMA unit
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, const void* src, int x, int y, int z, int w) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(m),
               "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}

// One work item = one 128-row K/V block of one (batch, head); early blocks see the most Q blocks
// under the causal mask and are handed out first.
struct FusedItem {
  int blk, zh, z, h, t_lo, t_hi;
  __device__ FusedItem(const FusedParams& p, int w) {
    const int nblk = p.N / BLK;
    zh = w / nblk;
    blk = w % nblk;
    z = zh / p.H;
    h = zh % p.H;
    t_lo = p.causal ? blk : 0;  // streamed Q blocks [t_lo, t_hi)
    t_hi = nblk;
  }
};

template <bool BF16>
__global__ void __launch_bounds__(FB_THREADS, 1)
attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap map_dk, const __grid_constant__ CUtensorMap map_dv,
                      const __grid_constant__ CUtensorMap map_dqacc, const FusedParams p) {
  constexpr int DRAIN_WARP0 = 8, MMA_WARP = 12, TMA_WARP = 13;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  uint8_t* sres = smem;                   // (K, V) of even items, (K, V) of odd items
  uint8_t* sring = smem + 4 * TILE;       // stages
  uint8_t* sds = sring + NST * STAGE;     // dS, M-major
  uint8_t* sdq = sds + DS_BYTES;          // 4 x 8 KiB, 128-byte swizzled
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdq + 4 * DQ_STG);
  uint64_t* r_full = bars;              // [2] K, V of an item loaded (buffer = item parity)
  uint64_t* r_empty = bars + 2;         // [2] every MMA of the item has read them
  uint64_t* full = bars + 4;            // [NST]
  uint64_t* empty = full + NST;         // [NST]
  uint64_t* t1_full = empty + NST;      // T1(t) in TMEM
  uint64_t* t2_full = t1_full + 1;      // T2(t) in TMEM
  uint64_t* p_full = t2_full + 1;       // P(t) written over T1
  uint64_t* ds_full = p_full + 1;       // dS(t) written over T2 and to shared memory
  uint64_t* ds_free = ds_full + 1;      // the dQ MMAs of step t have read the shared-memory dS
  uint64_t* dq_full = ds_free + 1;      // the dQ partial of step t is in TMEM
  uint64_t* dq_free = dq_full + 1;      // the drain warps have read it
  uint64_t* acc_full = dq_free + 1;     // dK, dV of the item final
  uint64_t* acc_free = acc_full + 1;    // the drain warps have read them: the next item may overwrite
  uint64_t* sched_full = acc_free + 1;  // [2] an item id was published
  uint64_t* sched_empty = sched_full + 2;  // [2] all 13 readers have taken it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sched_empty + 2);
  volatile int* sched_item = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  B200_TRACE_DECL;  // trace builds: region 0 = first compute warp, 2 = MMA warp, 3 = first drain warp

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&r_full[i], 1);
      mbar_init(&r_empty[i], 1);
    }
    for (int s = 0; s < NST; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(t1_full, 1);
    mbar_init(t2_full, 1);
    mbar_init(p_full, 256);
    mbar_init(ds_full, 256);
    mbar_init(ds_free, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, 4);  // one arrival per drain warp
    mbar_init(acc_full, 1);
    mbar_init(acc_free, 4);  // one arrival per drain warp
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sched_full[i], 1);
      mbar_init(&sched_empty[i], 13);  // MMA warp + one lane of each compute and drain warp
    }
    fence_barrier_init();
    cta_wait_flag_clear();
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&map_dqacc);
    tma_prefetch_desc(&map_dk);
    tma_prefetch_desc(&map_dv);
  }
  if (warp == MMA_WARP) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const uint32_t tm_t1 = tmem_base, tm_t2 = tmem_base + 128, tm_dk = tmem_base + 256, tm_dv = tmem_base + 320,
                 tm_dq = tmem_base + 384;

  // Every role ends with its own copy of the teardown and returns: nothing is shared after the
  // register budgets have diverged.
  auto teardown = [&](bool owner) {
    cta_linger_after_failure();
    tc_fence_before();
    __syncthreads();
    if (owner) {
      tc_fence_after();
      tmem_dealloc(tmem_base, 512);
    }
  };

  if (warp >= 14) {
    reg_dec<REGS_OTHER>();
    teardown(false);
    return;
  } else if (warp == TMA_WARP) {
    reg_dec<REGS_OTHER>();
    // ------------------------------------------------------------------ scheduler + TMA producer
    if (lane == 0) {
      uint32_t s = 0, ph = 0;  // ring position, runs on across items
      // draws the n-th ticket, publishes it and, if it is an item, starts the load of its K and V
      // into buffer n & 1 (free once the item two back has finished)
      auto next_item = [&](uint32_t n) {
        const int w = atomicAdd(p.sched_counter, 1);
        const uint32_t slot = n & 1u, sph = (n >> 1) & 1u;
        mbar_wait(&sched_empty[slot], sph ^ 1u, p.status, SITE_BWD_SCHED);
        sched_item[slot] = w;
        mbar_arrive(&sched_full[slot]);
        if (w == p.total_items + (int)gridDim.x - 1) atomicExch(p.sched_counter, 0);  // the last ticket of the launch
        if (w < p.total_items) {
          const FusedItem it(p, w);
          mbar_wait(&r_empty[slot], sph ^ 1u, p.status, SITE_BWD_KV);
          mbar_expect_tx(&r_full[slot], 2 * TILE);
          load_tile_f(sres + slot * 2 * TILE, &tm_k, &r_full[slot], it.blk * BLK, it.h, it.z);
          load_tile_f(sres + slot * 2 * TILE + TILE, &tm_v, &r_full[slot], it.blk * BLK, it.h, it.z);
        }
        return w;
      };
      int w = next_item(0);
      for (uint32_t n = 0; w < p.total_items; ++n) {
        const FusedItem it(p, w);
        for (int t = it.t_lo; t < it.t_hi; ++t) {
          mbar_wait(&empty[s], ph ^ 1u, p.status, SITE_BWD_LOAD_EMPTY);
          uint8_t* st = sring + s * STAGE;
          mbar_expect_tx(&full[s], 2 * TILE + 1024);
          load_tile_f(st, &tm_q, &full[s], t * BLK, it.h, it.z);
          load_tile_f(st + TILE, &tm_do, &full[s], t * BLK, it.h, it.z);
          // statistics of the streamed Q rows: M then delta, 128 floats each
          bulk_load_f(st + 2 * TILE, p.m + (long long)it.zh * p.N + t * BLK, 512, &full[s]);
          bulk_load_f(st + 2 * TILE + 512, p.delta + (long long)it.zh * p.N + t * BLK, 512, &full[s]);
          if (++s == NST) { s = 0; ph ^= 1u; }
        }
        w = next_item(n + 1);  // the next item's K and V travel while this item's last steps run
      }
    }
    __syncwarp();
    teardown(false);
    return;
  } else if (warp == MMA_WARP) {
    reg_dec<REGS_OTHER>();
    // ------------------------------------------------------------------ MMA issuer
    {  // the warp stays converged; an elected lane issues (descriptor arithmetic stays warp-uniform)
      constexpr int FMT = BF16 ? 1 : 0;
      constexpr uint32_t IDESC_T = make_idesc(FMT, FMT, 0, 0, 128, BLK);   // K or V (K-major) x Q or dO (K-major)
      constexpr uint32_t IDESC_ACC = make_idesc(FMT, FMT, 0, 1, 128, D);   // P / dS (TMEM) x dO / Q (N-major)
      constexpr uint32_t IDESC_DQ = make_idesc(FMT, FMT, 1, 1, 128, D);    // dS (shared memory, M-major) x K (N-major)
      const uint64_t dres = smem_desc_sw128(smem_u32(sres), 0, 1024);
      const uint64_t du0 = smem_desc_sw128(smem_u32(sring), 0, 1024);
      const uint64_t dun0 = smem_desc_sw128(smem_u32(sring), BLK * 128, 1024);  // N-major view of a streamed tile
      const uint64_t dkn0 = smem_desc_sw128(smem_u32(sres), BLK * 128, 1024);   // N-major view of K
      const uint64_t dds = smem_desc_sw128(smem_u32(sds), BLK * 128, 1024);     // dS: 64-row M blocks 16 KiB apart

      auto issue_t = [&](uint32_t tm, uint64_t dr, uint64_t du) {  // T = R U^T, D/16 MMAs
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) umma_ss_elect<false>(tm, dr + kk * 2, du + kk * 2, IDESC_T, kk != 0);
      };
      auto issue_acc = [&](uint32_t tm_acc, uint32_t tm_opnd, uint64_t dun, uint32_t accum) {  // acc (+)= X U, 8 MMAs
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk)
          umma_ts_f16_elect(tm_acc, tm_opnd + (kk >> 2) * 64 + (kk & 3) * 8, dun + kk * ((16 * 128) >> 4), IDESC_ACC,
                            (accum | kk) != 0);
      };

      uint32_t s = 0, ph = 0;  // ring position
      uint32_t cnt = 0;        // steps done so far, across items (parity of the per-step barriers)
      for (uint32_t n = 0;; ++n) {
        const uint32_t slot = n & 1u, sph = (n >> 1) & 1u;
        mbar_wait(&sched_full[slot], sph, p.status, SITE_BWD_SCHED);
        const int w = sched_item[slot];
        __syncwarp();
        if (lane == 0) mbar_arrive(&sched_empty[slot]);
        if (w >= p.total_items) break;
        const FusedItem item(p, w);
        const int steps = item.t_hi - item.t_lo;  // >= 1

        const uint64_t dr0 = dres + slot * ((2 * TILE) >> 4), dkn = dkn0 + slot * ((2 * TILE) >> 4);  // this item's K, V
        mbar_wait(&r_full[slot], sph, p.status, SITE_BWD_KV);
        mbar_wait(&full[s], ph, p.status, SITE_BWD_LOAD_FULL);
        issue_t(tm_t1, dr0, du0 + s * (STAGE >> 4));
        tc_commit_elect(t1_full);
        issue_t(tm_t2, dr0 + (TILE >> 4), du0 + s * (STAGE >> 4) + (TILE >> 4));
        tc_commit_elect(t2_full);
        for (int it = 0; it < steps; ++it, ++cnt) {
          const uint32_t cs = s;
          uint32_t ns = s + 1, nph = ph;
          if (ns == NST) { ns = 0; nph ^= 1u; }
          const uint64_t dun_q = dun0 + cs * (STAGE >> 4), dun_do = dun_q + (TILE >> 4);
          const bool more = it + 1 < steps;
          if (lane == 0) B200_TRACE_EVENT(p.status, 2, 0x10);
          mbar_wait(p_full, cnt & 1u, p.status, SITE_BWD_P_FULL);
          if (lane == 0) B200_TRACE_EVENT(p.status, 2, 0x20);
          if (it == 0) mbar_wait(acc_free, (n & 1u) ^ 1u, p.status, SITE_BWD_FREE);  // the previous item's dK, dV have left TMEM
          tc_fence_after();
          issue_acc(tm_dv, tm_t1, dun_do, it > 0);  // dV += P dO
          if (more) {  // the next scores: T1 is free once the dV MMAs have consumed P (in-order pipe)
            mbar_wait(&full[ns], nph, p.status, SITE_BWD_LOAD_FULL);
            issue_t(tm_t1, dr0, du0 + ns * (STAGE >> 4));
            tc_commit_elect(t1_full);
          }
          if (lane == 0) B200_TRACE_EVENT(p.status, 2, 0x30);
          mbar_wait(ds_full, cnt & 1u, p.status, SITE_BWD_DS_FULL);
          if (lane == 0) B200_TRACE_EVENT(p.status, 2, 0x40);
          tc_fence_after();
          issue_acc(tm_dk, tm_t2, dun_q, it > 0);  // dK += dS Q
          tc_commit_elect(&empty[cs]);  // that was the last read of Q_t and dO_t: the stage refills while dQ runs
          if (!more) tc_commit_elect(acc_full);  // dK and dV of the item are final: they leave TMEM while the last dQ product runs
          // dQ partial = dS^T K: the previous partial must have left TMEM
          mbar_wait(dq_free, (cnt & 1u) ^ 1u, p.status, SITE_BWD_FREE);
          if (lane == 0) B200_TRACE_EVENT(p.status, 2, 0x50);
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < BLK / 16; ++kk)
            umma_ss_elect<false>(tm_dq, dds + kk * ((16 * 128) >> 4), dkn + kk * ((16 * 128) >> 4), IDESC_DQ, kk != 0);
          tc_commit_elect(dq_full);
          tc_commit_elect(ds_free);
          if (more) {  // the next dP: T2 is free once the dK MMAs have consumed dS
            issue_t(tm_t2, dr0 + (TILE >> 4), du0 + ns * (STAGE >> 4) + (TILE >> 4));
            tc_commit_elect(t2_full);
          }
          s = ns; ph = nph;
        }
        tc_commit_elect(&r_empty[slot]);  // the item's last MMAs (dQ reads K) are behind this
      }
    }
    __syncwarp();
    teardown(true);
    return;
  } else if (warp >= DRAIN_WARP0) {
    reg_dec<REGS_DRAIN>();
    // ------------------------------------------------------------------ dQ partials: TMEM -> staging -> reduce-add
    const uint32_t quarter = warp & 3u;
    const uint32_t lane_addr = (quarter * 32u) << 16;
    uint8_t* stg = sdq + quarter * DQ_STG;
    uint32_t cnt = 0;
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
      const FusedItem item(p, w);
      // the item's dK and dV: this warp's 32 rows, 64 columns each = one box of 128-byte lines per
      // gradient, through the same two staging boxes as the dQ partials
      auto write_dk_dv = [&]() {
        mbar_wait(acc_full, n & 1u, p.status, SITE_BWD_ACC_FULL);
        tc_fence_after();
        if (lane == 0) tma_store_wait_read<0>();  // the last reduce-adds have read the staging boxes
        __syncwarp();
#pragma unroll 1
        for (int g = 0; g < 2; ++g) {  // 0: dK (carries sm_scale), 1: dV
          const float mul = g ? 1.0f : p.sm_scale;
          uint8_t* box = stg + g * 4096;
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t o[32];
            tmem_ld32((g ? tm_dv : tm_dk) + lane_addr + c, o);
            tmem_ld_wait();
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              uint32_t wv[4];
#pragma unroll
              for (int k = 0; k < 4; ++k)
                wv[k] = pack2<BF16>(__uint_as_float(o[8 * ch + 2 * k]) * mul, __uint_as_float(o[8 * ch + 2 * k + 1]) * mul);
              *reinterpret_cast<uint4*>(box + sw128_offset(lane, (c >> 3) + ch)) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
            }
          }
        }
        tc_fence_before();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(acc_free);
          const int row0 = item.blk * BLK + quarter * 32;
          tma_store_4d(&map_dk, stg, 0, row0, item.h, item.z);
          tma_store_4d(&map_dv, stg + 4096, 0, row0, item.h, item.z);
          tma_store_commit();
        }
      };
      for (int t = item.t_lo; t < item.t_hi; ++t, ++cnt) {
        // dK and dV are final once the last step's dK product is done, before its dQ product: they
        // go first, so that the next item's first dV product (issued as soon as its P is there) does
        // not wait for the accumulators
        if (t == item.t_hi - 1) write_dk_dv();
        mbar_wait(dq_full, cnt & 1u, p.status, SITE_BWD_ACC_FULL);
        if (quarter == 0 && lane == 0) B200_TRACE_EVENT(p.status, 3, 7);
        tc_fence_after();
        uint32_t r[D];
        tmem_ld32(tm_dq + lane_addr, r);
        tmem_ld32(tm_dq + lane_addr + 32, r + 32);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(dq_free);
          tma_store_wait_read<0>();  // the previous reduce-adds (or the dK / dV stores) have read the staging buffer
        }
        __syncwarp();
#pragma unroll
        for (int b = 0; b < 2; ++b)
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(stg + b * 4096 + sw128_offset(lane, ch)) =
                make_uint4(r[32 * b + 4 * ch], r[32 * b + 4 * ch + 1], r[32 * b + 4 * ch + 2], r[32 * b + 4 * ch + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int row0 = t * BLK + quarter * 32;
          tma_reduce_add_4d(&map_dqacc, stg, 0, row0, item.h, item.z);
          tma_reduce_add_4d(&map_dqacc, stg + 4096, 32, row0, item.h, item.z);
          tma_store_commit();
        }
        if (quarter == 0 && lane == 0) B200_TRACE_EVENT(p.status, 3, 8);
      }
    }
    if (lane == 0) tma_store_wait_read<0>();  // the staging buffers have been read: the CTA may exit, the writes land on their own
    __syncwarp();
    teardown(false);
    return;
  } else {
    reg_inc<REGS_COMPUTE>();
    // ------------------------------------------------------------------ compute
    // Two threads per K/V row: warps w and w+4 own the same TMEM lanes and split the 128 Q columns
    // of T1 / T2 in halves.  Each thread packs its
    // P and dS over the first 32 of its OWN 64 columns, so the halves never touch each other's
    // columns and need no barrier between them.
    const uint32_t quarter = warp & 3u;
    const int half = warp >> 2;
    constexpr int HC = BLK / 2;
    const int r = quarter * 32 + lane;       // K/V row inside the block
    const uint32_t lane_addr = (quarter * 32u) << 16;
    const float scale = p.scale_log2;
    uint32_t s = 0;    // ring position
    uint32_t cnt = 0;  // steps done so far, across items

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
      const FusedItem item(p, w);
      const int blk = item.blk;
      const int steps = item.t_hi - item.t_lo;
      const bool traced = warp == 0 && lane == 0;  // used by trace builds only
      if (traced) B200_TRACE_EVENT(p.status, 0, 0x100 | steps);
      uint32_t pr[HC];  // P of the step in hand, fp32 bits (phase A writes it, phase B reads it)
      // phase A of step `it`: scores -> P (exp2), packed over T1 as the dV product's operand
      auto phase_a = [&](int it, uint32_t c_, uint32_t s_) {
        const int t = item.t_lo + it;
        const float* sm = reinterpret_cast<const float*>(sring + s_ * STAGE + 2 * TILE) + half * HC;  // column M
        const bool diag = p.causal && (t == blk);  // the only block that needs the causal mask
        mbar_wait(t1_full, c_ & 1u, p.status, SITE_BWD_S_FULL);
        if (traced) B200_TRACE_EVENT(p.status, 0, 1);
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HC; c += 32) tmem_ld32(tm_t1 + lane_addr + half * HC + c, pr + c);
        tmem_ld_wait();
#pragma unroll
        for (int c4 = 0; c4 < HC; c4 += 4) {
          const float4 m4 = *reinterpret_cast<const float4*>(sm + c4);  // one 16-byte broadcast load for four columns
          float xs[4];
          upk2(fma2(pk2(__uint_as_float(pr[c4]), __uint_as_float(pr[c4 + 1])), pk2(scale, scale), pk2(-m4.x, -m4.y)), xs[0], xs[1]);
          upk2(fma2(pk2(__uint_as_float(pr[c4 + 2]), __uint_as_float(pr[c4 + 3])), pk2(scale, scale), pk2(-m4.z, -m4.w)), xs[2], xs[3]);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float pv = ex2(xs[u]);
            if (diag && (half * HC + c4 + u < r)) pv = 0.f;  // row = kv, column = q: keep q >= kv
            pr[c4 + u] = __float_as_uint(pv);
          }
        }
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
        if (traced) B200_TRACE_EVENT(p.status, 0, 2);
      };
      // phase B of step `it`: dS = P (dP - delta), packed over T2 (dK product) and to shared memory (dQ product)
      auto phase_b = [&](uint32_t c_, uint32_t s_) {
        const float* sd = reinterpret_cast<const float*>(sring + s_ * STAGE + 2 * TILE) + 128 + half * HC;  // column delta
        mbar_wait(t2_full, c_ & 1u, p.status, SITE_BWD_DP_FULL);
        if (traced) B200_TRACE_EVENT(p.status, 0, 3);
        tc_fence_after();
        uint32_t dsw[HC / 2];  // dS packed to 16 bit
#pragma unroll
        for (int c = 0; c < HC; c += 32) {
          uint32_t dp[32];
          tmem_ld32(tm_t2 + lane_addr + half * HC + c, dp);
          tmem_ld_wait();
#pragma unroll
          for (int k4 = 0; k4 < 32; k4 += 4) {
            const float4 d4 = *reinterpret_cast<const float4*>(sd + c + k4);
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
        // the same dS as the A operand of the dQ product: row r (kv) of the M-major tile, this
        // thread's 64 q columns = one 128-byte line of block `half`, 16-byte chunks swizzled
        if (traced) B200_TRACE_EVENT(p.status, 0, 5);
        mbar_wait(ds_free, (c_ & 1u) ^ 1u, p.status, SITE_BWD_FREE);  // the previous step's dQ MMAs have read the tile
        if (traced) B200_TRACE_EVENT(p.status, 0, 6);
        {
          uint8_t* line = sds + half * (BLK * 128);
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(line + sw128_offset(r, ch)) = make_uint4(dsw[4 * ch], dsw[4 * ch + 1], dsw[4 * ch + 2], dsw[4 * ch + 3]);
        }
        fence_proxy_async_smem();
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(ds_full);
        if (traced) B200_TRACE_EVENT(p.status, 0, 4);
      };
      // Both warps of a scheduler (the halves of a row) run A(t) B(t) in step.  (Skewing them - half 1
      // doing B(t-1) A(t), so that one half's exponentials overlap the other's dS arithmetic - was
      // measured 25 % slower: T1 of the next step needs both halves' P, so the early half only waits.)
      for (int it = 0; it < steps; ++it, ++cnt) {
        phase_a(it, cnt, s);
        phase_b(cnt, s);
        if (++s == NST) s = 0;
      }
      // dK and dV of the item are written by the drain warps: straight on to the next item
    }
    teardown(false);
  }
}

// dq = storage type( sum of the partials * sm_scale ); eight columns per thread
template <bool BF16>
__global__ void __launch_bounds__(256)
attn_bwd_dq_convert_kernel(const float* __restrict__ acc, uint16_t* __restrict__ dq, long long sz, long long sh,
                           long long sn, unsigned H, unsigned N, unsigned rows_total, float mul) {
  constexpr unsigned TPR = D / 8;  // threads per row
  const unsigned idx = blockIdx.x * 256 + threadIdx.x;
  const unsigned row = idx / TPR, part = idx % TPR;
  if (row >= rows_total) return;
  const float4 a = *reinterpret_cast<const float4*>(acc + (long long)row * D + part * 8);
  const float4 b = *reinterpret_cast<const float4*>(acc + (long long)row * D + part * 8 + 4);
  const unsigned n = row % N, zh = row / N, hh = zh % H, zz = zh / H;
  uint4 out;
  out.x = pack2<BF16>(a.x * mul, a.y * mul);
  out.y = pack2<BF16>(a.z * mul, a.w * mul);
  out.z = pack2<BF16>(b.x * mul, b.y * mul);
  out.w = pack2<BF16>(b.z * mul, b.w * mul);
  *reinterpret_cast<uint4*>(dq + zz * sz + hh * sh + (long long)n * sn + part * 8) = out;
}

template <bool BF16>
int launch_fused_t(DeviceCtx* ctx, cudaStream_t stream, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tq,
                   const CUtensorMap& tdo, const CUtensorMap& mdk, const CUtensorMap& mdv, const CUtensorMap& macc,
                   FusedParams p, float* dq_acc, void* dq, const int64_t* sdq) {
  static std::atomic<bool> attr_done[64];
  if (int rc = ensure_dynamic_smem(attn_bwd_fused_kernel<BF16>, FUSED_SMEM, ctx->device, attr_done, "attn bwd fused")) return rc;
  p.sched_counter = next_sched_counter(ctx, stream);
  if (!p.sched_counter) return B200_ERR_CUDA;
  const int grid = p.total_items < ctx->sm_count ? p.total_items : ctx->sm_count;
  attn_bwd_fused_kernel<BF16><<<grid, FB_THREADS, FUSED_SMEM, stream>>>(tk, tv, tq, tdo, mdk, mdv, macc, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "attn bwd fused launch: %s", cudaGetErrorString(e));
  const long long rows = (long long)p.Z * p.H * p.N;
  const unsigned blocks = (unsigned)((rows * (D / 8) + 255) / 256);
  attn_bwd_dq_convert_kernel<BF16><<<blocks, 256, 0, stream>>>(dq_acc, reinterpret_cast<uint16_t*>(dq), sdq[0], sdq[1], sdq[2],
                                                               (unsigned)p.H, (unsigned)p.N, (unsigned)rows, p.sm_scale);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "attn bwd dq convert launch: %s", cudaGetErrorString(e));
  return B200_OK;
}

}  // namespace

size_t attn_bwd_fused_workspace_bytes(int Z, int H, int N, int Dh) { return (size_t)Z * H * N * Dh * sizeof(float); }

// Returns B200_OK after launching, B200_ERR_UNSUPPORTED (with a message) when the fused path does
// not apply: head dim other than 64, or a dK / dV / dQ layout that TMA stores cannot address.
int launch_attn_bwd_fused(DeviceCtx* ctx, cudaStream_t stream, const void* q, const void* k, const void* v, const void* o,
                          const void* dout, const float* m, float* delta, float* dq_acc, void* dq, void* dk, void* dv, int Z,
                          int H, int N, int Dh, const int64_t* sq, const int64_t* sk, const int64_t* sv, const int64_t* so,
                          const int64_t* sdo, const int64_t* sdq, const int64_t* sdk, const int64_t* sdv, float sm_scale,
                          int causal, int dtype) {
  if (Dh != D) return fail(B200_ERR_UNSUPPORTED, "the one-pass backward has a kernel for head dim 64 only");
  const long long rows = (long long)Z * H * N;
  if (rows >= (1ll << 32) / (D / 8)) return fail(B200_ERR_UNSUPPORTED, "too many rows for the one-pass backward");
  CUtensorMap tq, tk, tv, tdo, mdk, mdv, macc;
  if (!encode_qkv_map(&tq, dtype, q, Z, H, N, D, sq[0], sq[1], sq[2], BLK)) return B200_ERR_UNSUPPORTED;
  if (!encode_qkv_map(&tk, dtype, k, Z, H, N, D, sk[0], sk[1], sk[2], BLK)) return B200_ERR_UNSUPPORTED;
  if (!encode_qkv_map(&tv, dtype, v, Z, H, N, D, sv[0], sv[1], sv[2], BLK)) return B200_ERR_UNSUPPORTED;
  if (!encode_qkv_map(&tdo, dtype, dout, Z, H, N, D, sdo[0], sdo[1], sdo[2], BLK)) return B200_ERR_UNSUPPORTED;
  // dK, dV leave through boxes of 32 rows x 64 columns (128-byte lines, swizzled)
  if (!encode_qkv_map(&mdk, dtype, dk, Z, H, N, D, sdk[0], sdk[1], sdk[2], 32)) return B200_ERR_UNSUPPORTED;
  if (!encode_qkv_map(&mdv, dtype, dv, Z, H, N, D, sdv[0], sdv[1], sdv[2], 32)) return B200_ERR_UNSUPPORTED;
  // the fp32 accumulator of dQ: contiguous [Z, H, N, 64], boxes of 32 columns (128 bytes, swizzled) x 32 rows
  if (!encode_rows_map(&macc, B200_F32, dq_acc, Z, H, N, D, (int64_t)H * N * D, (int64_t)N * D, D, 32, 32, true))
    return B200_ERR_UNSUPPORTED;
  if ((sdq[0] & 7) || (sdq[1] & 7) || (sdq[2] & 7) || (reinterpret_cast<uintptr_t>(dq) & 15))
    return fail(B200_ERR_UNSUPPORTED, "dQ must be 16-byte aligned with strides that are multiples of 8 elements");
  // the pre-pass also clears the dQ accumulator (one launch, one pass over the rows)
  if (int rc = launch_attn_bwd_delta(ctx, stream, o, dout, delta, Z, H, N, D, so, sdo, dtype, dq_acc)) return rc;
  FusedParams p{};
  p.m = m; p.delta = delta;
  p.Z = Z; p.H = H; p.N = N; p.causal = causal;
  p.scale_log2 = sm_scale * 1.44269504f;
  p.sm_scale = sm_scale;
  p.total_items = (N / BLK) * Z * H;
  p.status = ctx->status;
  return dtype == B200_BF16 ? launch_fused_t<true>(ctx, stream, tk, tv, tq, tdo, mdk, mdv, macc, p, dq_acc, dq, sdq)
                            : launch_fused_t<false>(ctx, stream, tk, tv, tq, tdo, mdk, mdv, macc, p, dq_acc, dq, sdq);
}

}  // namespace tb
