// FlashAttention backward for sm_100a.
//
// Three launches:
//   1. bwd_preprocess: softmax_d[b,h,i] = p_keep * sum_d dO*O and zero-fill of the fp32 dQ
//      accumulator (HBM bound).
//   2. bwd_main: one CTA per 128-row key/value tile of one (batch, head) pair; it keeps K and V in
//      shared memory and walks the 128-row query tiles.  Per tile pair it recomputes
//      S = Q K^T and dP = dO V^T on the tensor cores (accumulators in tensor memory), forms
//      P = exp2(scale*log2e*S - LSE*log2e), regenerates the dropout mask, forms
//      dS = P*(dP - D) (kept) or -P*D (dropped), writes the 16-bit P~ and dS to shared memory
//      and issues dV += P~^T dO, dK += dS^T Q, dQ = dS K.  dQ tiles are added into the fp32
//      accumulator with TMA reduce-adds; dK and dV stay in tensor memory until the end.
//   3. bwd_postprocess: dq = accumulator * scale / p_keep in the 16-bit output type.
//
// The formulas are those of the reference backward
// (csrc/flash_attn/src/fmha_dgrad_kernel_1xN_loop.h:304-661): P recomputed from the saved LSE
// (:333), dropped entries contribute -P*D (:402-418), dQ and dK scaled by scale/p_keep (:583,
// :628), dV by 1/p_keep (:613-619), P~ and dS rounded to the 16-bit type before their products.
//
// Warp roles in bwd_main (512 threads):
//   warps 0-3   compute group 0: key columns 0-63 of the tile, S, dP -> P~, dS (one thread per
//               query row; at d = 64 with dropout the 16x256b quad layout, in which one Philox call
//               is private to a thread, and stmatrix stores); dV epilogue
//   warps 4-7   compute group 1: key columns 64-127; dK epilogue
//   warps 8-11  dQ group: tensor memory -> global reductions
//   warp 12     TMA producer     warp 13  MMA issuer (S, dP, dQ; everything at d = 128)
//   warp 14, 15 second and third MMA issuer (dV | dK) at d = 64
//
// Schedules.  d = 64: Q and dO travel together through a three-stage ring; S and dP of tile t + 1
// are issued as soon as the compute groups have read tile t into registers.  d = 128: shared
// memory holds one stage of Q and one of dO, each with its own barriers.  The compute groups work
// in two phases, P~ from S and then dS from dP; dV(t) is issued after phase one and releases dO
// for its refill, dK(t) and dQ(t) follow phase two and dK releases Q; S(t + 1) is issued when Q
// has landed and dP(t + 1) when dO has landed and the dQ group has read dQ(t) out of the
// tensor-memory columns it shares with dP.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "fa_kernels.h"
#include "fa_math.cuh"
#include "sm100_prims.cuh"

namespace fa {

namespace {

constexpr int kBM = 128;  // query rows per tile
constexpr int kBN = 128;  // key rows per tile
constexpr int kBwdThreads = 512;
constexpr int kMaxSparseTiles = 1024;  // query tiles of 128 per sequence in block-sparse mode

// BS: block-sparse variant (its tile list takes shared memory that the third Q / dO stage would need)
template <int D, bool BS = false>
struct BwdCfg {
  // d = 128 runs a different schedule: shared memory holds a single stage of Q and of dO, each
  // with its own barriers, and the compute groups work in two phases (P~ from S, then dS from dP)
  // so that dV can be issued - and dO released for its refill - before dP is even needed.
  static constexpr bool kTwoPhase = (D == 128);
  // Q / dO ring.  d = 64: a stage is released when the dK product of its tile has finished and
  // the refill takes about 1500 clk to land, so with two stages the S / dP products of the next
  // tile start late and the compute groups wait; the third stage lets the load run a whole tile
  // ahead.
  static constexpr int kQStages = (D == 64) ? (BS ? 2 : 3) : 1;
  static constexpr bool kAliasDq = kTwoPhase;     // dQ shares tensor-memory columns with dP
  static constexpr bool kDualIssue = !kTwoPhase;  // second MMA-issuing warp for dV, dK
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kPdsBytes = 128 * 128 * 2;
  static constexpr int kDqStageBytes = 2 * 16384;  // two [128 rows x 32 fp32] boxes
  // K, V, (Q, dO) x stages, P~, dS, dQ staging
  static constexpr int kSmemBytes = (2 + 2 * kQStages) * kTileBytes + 2 * kPdsBytes + kDqStageBytes + 1024;
  static constexpr uint32_t kTmemS = 0, kTmemDP = 128, kTmemDV = 256, kTmemDK = 256 + D;
  static constexpr uint32_t kTmemDQ = kAliasDq ? 128 : 256 + 2 * D;
  // d = 64 leaves 64 tensor-memory columns free: a second copy of the 16-bit dS can go there and feed
  // dQ = dS K as the A operand (its M dimension is the query row, like the lanes of S), so that
  // product does not read dS from shared memory; dK = dS^T Q still takes the shared-memory copy.
  // Used without dropout, where shared-memory bandwidth is the bound (8 x 12 x 4096: 1.49 -> 1.39 ms);
  // with dropout the compute groups are the bound and the extra stores cost 2 %.
  static constexpr bool kDsInTmemCapable = !kTwoPhase;
  static constexpr uint32_t kTmemDS = 256 + 3 * D;
};

struct BwdShared {
  uint64_t kv_full;
  uint64_t q_full[3], q_empty[3];
  uint64_t do_full, do_empty;  // dO ring of the two-phase schedule (one stage)
  // d = 64: S and dP together / P~ and dS together.  Two-phase schedule: sdp_full = dP landed,
  // sdp_consumed = S read into registers, pds_ready = dS stored, pds_free = dV has read P~.
  uint64_t sdp_full, sdp_consumed, pds_ready, pds_free, dq_full, dq_consumed;
  uint64_t s_full;    // two-phase: S landed
  uint64_t p_ready;   // two-phase: P~ stored
  uint64_t ds_free;   // two-phase: dK and dQ have finished reading the dS buffer
  uint64_t dq_group;  // rendezvous of the 128 threads of the dQ group (bounded, unlike bar.sync)
  uint32_t tmem_base;
  int abort_flag;
};

template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// Optional cycle accounting (build with -DFA_PROFILE): one thread of each role of CTA (0,0,0)
// accumulates the cycles it spends per phase into status[8..].
#ifdef FA_PROFILE
#define FA_PROF_DECL long long prof_t = clock64(); long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
// time stamps (low 32 bits of the SM clock) of one tile's events, for a timeline across the roles
#define FA_STAMP(tile, idx) if ((tile) >= 5 && (tile) <= 7 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && ka.status) { \
    ka.status[64 + ((tile) - 5) * 20 + (idx)] = static_cast<int32_t>(clock64()); }
#define FA_PROF(slot) { const long long now_ = clock64(); prof_acc[slot] += now_ - prof_t; prof_t = now_; }
#define FA_PROF_FLUSH(base, n) if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && ka.status) { \
    for (int i_ = 0; i_ < 8; ++i_) ka.status[(base) + i_] = static_cast<int32_t>(prof_acc[i_] / ((n) > 0 ? (n) : 1)); }
#else
#define FA_PROF_DECL
#define FA_STAMP(tile, idx)
#define FA_PROF(slot)
#define FA_PROF_FLUSH(base, n)
#endif

template <int N>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// ------------------------------------------------------------------------------------------------
template <int D, bool BF16, bool CAUSAL, bool DROPOUT, bool BLOCKSPARSE>
__global__ void __launch_bounds__(kBwdThreads, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
              const __grid_constant__ CUtensorMap tm_dq, const BwdArgs a) {
  using Cfg = BwdCfg<D, BLOCKSPARSE>;
  constexpr bool kDsInTmem = Cfg::kDsInTmemCapable && !DROPOUT;
  extern __shared__ uint8_t smem_raw[];
  __shared__ BwdShared sh;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int b = blockIdx.z;
  const int h = blockIdx.y;
  const int nt = blockIdx.x;  // key tile
  const KernelArgs& ka = a.k;

  const int q_start = ka.cu_seqlens_q[b];
  const int sq = ka.cu_seqlens_q[b + 1] - q_start;
  const int k_start = ka.cu_seqlens_k[b];
  const int sk = ka.cu_seqlens_k[b + 1] - k_start;
  const int n0 = nt * kBN;
  if (n0 >= sk) return;
  // fail fast: once a CTA of this launch has abandoned a wait, the remaining CTAs do not start
  if (ka.status && *reinterpret_cast<volatile int32_t*>(ka.status) == ka.launch_id) return;

  const int m_tiles = (sq + kBM - 1) / kBM;
  const int m_begin = CAUSAL ? min(m_tiles, n0 / kBM) : 0;
  int nm = m_tiles - m_begin;
  // block-sparse: query tiles that have at least one 16-row block in this key block's list
  __shared__ uint16_t qtile_list[BLOCKSPARSE ? kMaxSparseTiles : 1];
  // deterministic mode: how many key tiles before this one add into the same query tile
  __shared__ uint16_t qtile_order[BLOCKSPARSE ? kMaxSparseTiles : 1];
  __shared__ int qtile_count;
  if constexpr (BLOCKSPARSE) {
    uint8_t* flags = reinterpret_cast<uint8_t*>(smem_raw);
    const int32_t* brow = ka.bs_iter + (static_cast<int64_t>(b) * ka.bs_kblocks + (n0 >> 8)) * ka.bs_rows16;
    const int rb_end = min(ka.bs_rows16, (sq + 15) >> 4);
    const int mt = min(m_tiles, kMaxSparseTiles);
    uint16_t* order_all = reinterpret_cast<uint16_t*>(smem_raw + kMaxSparseTiles);
    for (int m = threadIdx.x; m < mt; m += kBwdThreads) {
      bool any = false;
      for (int rb = m * (kBM / 16); rb < min((m + 1) * (kBM / 16), rb_end); ++rb) any = any || (brow[rb] >= 0);
      if (CAUSAL && m < m_begin) any = false;  // query tiles entirely before this key tile see none of it
      flags[m] = any ? 1 : 0;
      if (a.dq_tickets != nullptr && any) {
        // the two 128-row key tiles of a 256-row key block visit the same query tiles
        int before = 0;
        for (int kb = 0; kb < (n0 >> 8); ++kb) {
          const int32_t* prow = ka.bs_iter + (static_cast<int64_t>(b) * ka.bs_kblocks + kb) * ka.bs_rows16;
          bool hit = false;
          for (int rb = m * (kBM / 16); rb < min((m + 1) * (kBM / 16), rb_end); ++rb) hit = hit || (prow[rb] >= 0);
          before += hit ? 2 : 0;
        }
        order_all[m] = static_cast<uint16_t>(before + ((nt & 1) ? 1 : 0));
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int n = 0;
      for (int m = 0; m < mt; ++m)
        if (flags[m]) {
          if (a.dq_tickets != nullptr) qtile_order[n] = order_all[m];
          qtile_list[n++] = static_cast<uint16_t>(m);
        }
      qtile_count = n;
    }
    __syncthreads();
    nm = qtile_count;
    __syncthreads();
  }
  // Deterministic mode: the key tiles of one (batch, head) add into a query tile in ascending
  // key-tile order.  Dense causal grids then walk the query tiles from the last one down, so that
  // every key tile starts on a query tile its predecessors start on too (walking up, key tile n
  // would idle until tile n - 1 arrives at its first query tile).
  const bool deterministic = a.dq_tickets != nullptr;
  const bool walk_down = CAUSAL && !BLOCKSPARSE && deterministic;
  auto q_tile = [&](int t) -> int {
    if constexpr (BLOCKSPARSE) return qtile_list[t];
    else return walk_down ? (m_tiles - 1 - t) : (m_begin + t);
  };

  uint16_t* dk_base = reinterpret_cast<uint16_t*>(a.dk);
  uint16_t* dv_base = reinterpret_cast<uint16_t*>(a.dv);

  if (nm <= 0) {
    // no query row sees these keys: their gradients are zero
    for (int idx = tid; idx < kBN * (ka.head_dim / 8); idx += kBwdThreads) {
      const int r = idx / (ka.head_dim / 8), c = (idx % (ka.head_dim / 8)) * 8;
      if (n0 + r < sk) {
        const int64_t row = k_start + n0 + r;
        *reinterpret_cast<uint4*>(dk_base + row * a.dk_row_stride + h * a.dk_head_stride + c) =
            make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(dv_base + row * a.dv_row_stride + h * a.dv_head_stride + c) =
            make_uint4(0, 0, 0, 0);
      }
    }
    return;
  }

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t smem_k = smem_u32(smem);
  const uint32_t smem_v = smem_k + Cfg::kTileBytes;
  const uint32_t smem_q = smem_v + Cfg::kTileBytes;                       // stages of Q
  const uint32_t smem_do = smem_q + Cfg::kQStages * Cfg::kTileBytes;      // stages of dO
  const uint32_t smem_p = smem_do + Cfg::kQStages * Cfg::kTileBytes;
  const uint32_t smem_ds = smem_p + Cfg::kPdsBytes;
  uint8_t* p_ptr = smem + (2 + 2 * Cfg::kQStages) * Cfg::kTileBytes;
  uint8_t* ds_ptr = p_ptr + Cfg::kPdsBytes;
  uint8_t* dq_stage = ds_ptr + Cfg::kPdsBytes;

  if (tid == 0) {
    sh.abort_flag = 0;
    mbar_init(smem_u32(&sh.kv_full), 1);
    for (int i = 0; i < 3; ++i) {
      mbar_init(smem_u32(&sh.q_full[i]), 1);
      mbar_init(smem_u32(&sh.q_empty[i]), Cfg::kDualIssue ? 2 : 1);  // d = 64: dV (reads dO) and dK (reads Q)
    }
    mbar_init(smem_u32(&sh.do_full), 1);
    mbar_init(smem_u32(&sh.do_empty), 1);
    mbar_init(smem_u32(&sh.sdp_full), 1);
    mbar_init(smem_u32(&sh.sdp_consumed), 2 * kBM);
    mbar_init(smem_u32(&sh.pds_ready), 2 * kBM);
    mbar_init(smem_u32(&sh.pds_free), Cfg::kDualIssue ? 3 : 1);  // d = 64: dQ, dV and dK each commit
    mbar_init(smem_u32(&sh.dq_full), 1);
    mbar_init(smem_u32(&sh.dq_consumed), kBM);
    mbar_init(smem_u32(&sh.dq_group), kBM);
    mbar_init(smem_u32(&sh.s_full), 1);
    mbar_init(smem_u32(&sh.p_ready), 2 * kBM);
    mbar_init(smem_u32(&sh.ds_free), 1);
    fence_mbar_init();
  }
  if (warp == 12) tmem_alloc(smem_u32(&sh.tmem_base), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh.tmem_base;
  volatile int* abort_flag = &sh.abort_flag;

  const float rp_keep = ka.rp_keep;

  // operand descriptors of the five products
  constexpr uint32_t idesc_s = make_idesc(BF16, false, false, 128, 128);   // Q K^T, dO V^T
  constexpr uint32_t idesc_tt = make_idesc(BF16, true, true, 128, D);      // P~^T dO, dS^T Q
  constexpr uint32_t idesc_dq = make_idesc(BF16, false, true, 128, D);     // dS K
  auto issue_kk = [&](uint32_t dst, uint32_t a_base, uint32_t b_base) {  // both K-major, K = D
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
      mma_ss(dst, make_smem_desc(a_base + off, 16, 1024), make_smem_desc(b_base + off, 16, 1024),
             idesc_s, ks > 0);
    }
  };
  auto issue_tt = [&](uint32_t dst, uint32_t a_base, uint32_t b_base, bool acc) {
    // A = [q][kv] read as M = kv (MN-major); B = [q][d] read as N = d (MN-major); K = q rows
#pragma unroll
    for (int ks = 0; ks < kBM / 16; ++ks) {
      mma_ss(dst, make_smem_desc(a_base + ks * 2048, 16384, 1024),
             make_smem_desc(b_base + ks * 2048, 16384, 1024), idesc_tt, acc || ks > 0);
    }
  };
  auto issue_dq = [&](uint32_t dst, uint32_t a_base, uint32_t b_base) {
    // A = dS [q][kv] K-major; B = K [kv][d] read as N = d (MN-major); K = kv
#pragma unroll
    for (int ks = 0; ks < kBN / 16; ++ks) {
      const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
      mma_ss(dst, make_smem_desc(a_base + off, 16, 1024),
             make_smem_desc(b_base + ks * 2048, 16384, 1024), idesc_dq, ks > 0);
    }
  };
  const uint32_t tS_ = tmem + Cfg::kTmemS, tDP_ = tmem + Cfg::kTmemDP;
  const uint32_t tDV_ = tmem + Cfg::kTmemDV, tDK_ = tmem + Cfg::kTmemDK, tDQ_ = tmem + Cfg::kTmemDQ;
  const uint32_t tDS_ = tmem + Cfg::kTmemDS;
  auto issue_dq_t = [&](uint32_t dst, uint32_t a_tmem, uint32_t b_base) {
    // A = dS from tensor memory (16 keys = 8 columns per step); B = K [kv][d] read as N = d; K = kv
#pragma unroll
    for (int ks = 0; ks < kBN / 16; ++ks)
      mma_ts(dst, a_tmem + ks * 8, make_smem_desc(b_base + ks * 2048, 16384, 1024), idesc_dq, ks > 0);
  };

  if (warp >= 12) {
    // register split (per thread): d = 64: 192 compute / 72 dQ / 56 here; d = 128: 176 / 88 / 72
    if constexpr (D == 64) reg_dealloc<56>(); else reg_dealloc<72>();
    if (warp == 12 && lane == 0) {
      // -------------------------------------------------------------- TMA producer
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_do);
      tma_prefetch_desc(&tm_dq);
      {
        const uint32_t bar = smem_u32(&sh.kv_full);
        mbar_expect_tx(bar, 2 * Cfg::kTileBytes);
        for (int p = 0; p < D / 64; ++p) {
          tma_load_3d(smem_k + p * 16384, &tm_k, bar, p * 64, k_start + n0, h);
          tma_load_3d(smem_v + p * 16384, &tm_v, bar, p * 64, k_start + n0, h);
        }
      }
      bool ok = true;
      for (int t = 0; t < nm && ok; ++t) {
        const int s = t % Cfg::kQStages;
        if (!Cfg::kTwoPhase && t >= Cfg::kQStages)
          ok = mbar_wait(smem_u32(&sh.q_empty[s]), ((t / Cfg::kQStages) & 1) ^ 1, abort_flag);
        if (!ok) break;
        if (!Cfg::kTwoPhase) { FA_STAMP(t - 1, 16) }
        const int row = q_start + q_tile(t) * kBM;
        if constexpr (Cfg::kTwoPhase) {
          // dO(t) follows dV(t - 1), Q(t) follows dK(t - 1): the order in which they finish
          if (t >= 1) ok = mbar_wait(smem_u32(&sh.do_empty), (t & 1) ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t bar_do = smem_u32(&sh.do_full);
          mbar_expect_tx(bar_do, Cfg::kTileBytes);
          for (int p = 0; p < D / 64; ++p) tma_load_3d(smem_do + p * 16384, &tm_do, bar_do, p * 64, row, h);
          if (t >= 1) ok = mbar_wait(smem_u32(&sh.q_empty[0]), (t & 1) ^ 1, abort_flag);
          if (!ok) break;
          FA_STAMP(t - 1, 16)
          const uint32_t bar = smem_u32(&sh.q_full[0]);
          mbar_expect_tx(bar, Cfg::kTileBytes);
          for (int p = 0; p < D / 64; ++p) tma_load_3d(smem_q + p * 16384, &tm_q, bar, p * 64, row, h);
        } else {
          const uint32_t bar = smem_u32(&sh.q_full[s]);
          mbar_expect_tx(bar, 2 * Cfg::kTileBytes);
          for (int p = 0; p < D / 64; ++p) {
            tma_load_3d(smem_q + s * Cfg::kTileBytes + p * 16384, &tm_q, bar, p * 64, row, h);
            tma_load_3d(smem_do + s * Cfg::kTileBytes + p * 16384, &tm_do, bar, p * 64, row, h);
          }
        }
      }
    } else if (warp == 13 && lane == 0) {
      // -------------------------------------------------------------- MMA issuer 1
      bool ok = mbar_wait(smem_u32(&sh.kv_full), 0, abort_flag);
      if (ok) ok = mbar_wait(smem_u32(&sh.q_full[0]), 0, abort_flag);
      if constexpr (Cfg::kTwoPhase) {
        // d = 128: every product, issued by this thread in the order
        //   dV(t) | dK(t), dQ(t) | S(t+1) | dP(t+1)
        // dV(t) follows P~ (end of phase one of the compute groups) and releases dO for its
        // refill while phase two is still running.  dK, dQ follow dS; dK releases Q.  S(t+1) is
        // issued when Q has landed, dP(t+1) when dO has landed and the dQ group has read dQ(t)
        // out of the columns it shares with dP.
        if (ok) {
          tc_fence_after();
          issue_kk(tS_, smem_q, smem_k);
          mma_commit(smem_u32(&sh.s_full));
          ok = mbar_wait(smem_u32(&sh.do_full), 0, abort_flag);
        }
        if (ok) {
          tc_fence_after();
          issue_kk(tDP_, smem_do, smem_v);
          mma_commit(smem_u32(&sh.sdp_full));
        }
        FA_PROF_DECL
        for (int t = 0; t < nm && ok; ++t) {
          const bool has_next = t + 1 < nm;
          FA_PROF(0)
          ok = mbar_wait(smem_u32(&sh.p_ready), t & 1, abort_flag);
          if (!ok) break;
          FA_PROF(1)
          tc_fence_after();
          issue_tt(tDV_, smem_p, smem_do, t > 0);
          mma_commit(smem_u32(&sh.pds_free));
          mma_commit(smem_u32(&sh.do_empty));
          FA_STAMP(t, 11)
          ok = mbar_wait(smem_u32(&sh.pds_ready), t & 1, abort_flag);
          if (!ok) break;
          FA_PROF(2)
          FA_STAMP(t, 9)
          tc_fence_after();
          issue_tt(tDK_, smem_ds, smem_q, t > 0);
          mma_commit(smem_u32(&sh.q_empty[0]));
          issue_dq(tDQ_, smem_ds, smem_k);
          mma_commit(smem_u32(&sh.dq_full));
          mma_commit(smem_u32(&sh.ds_free));
          FA_STAMP(t, 10)
          FA_PROF(3)
          if (has_next) {
            FA_STAMP(t, 5)
            ok = mbar_wait(smem_u32(&sh.q_full[0]), (t + 1) & 1, abort_flag);
            FA_STAMP(t, 6)
            if (ok) ok = mbar_wait(smem_u32(&sh.sdp_consumed), t & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            issue_kk(tS_, smem_q, smem_k);
            mma_commit(smem_u32(&sh.s_full));
            FA_STAMP(t, 12)
            FA_PROF(4)
            ok = mbar_wait(smem_u32(&sh.do_full), (t + 1) & 1, abort_flag);
            if (ok) ok = mbar_wait(smem_u32(&sh.dq_consumed), t & 1, abort_flag);
            if (!ok) break;
            FA_STAMP(t, 7)
            tc_fence_after();
            issue_kk(tDP_, smem_do, smem_v);
            mma_commit(smem_u32(&sh.sdp_full));
            FA_STAMP(t, 8)
            FA_PROF(5)
          }
        }
        FA_PROF_FLUSH(16, nm)
      } else {
        // d = 64: S, dP and dQ (dV, dK go through issuer 2)
        if (ok) {
          tc_fence_after();
          issue_kk(tS_, smem_q, smem_k);
          issue_kk(tDP_, smem_do, smem_v);
          mma_commit(smem_u32(&sh.sdp_full));
        }
        FA_PROF_DECL
        for (int t = 0; t < nm && ok; ++t) {
          const bool has_next = t + 1 < nm;
          const int sn = (t + 1) % Cfg::kQStages;
          FA_PROF(0)
          if (has_next) {
            FA_STAMP(t, 5)
            ok = mbar_wait(smem_u32(&sh.q_full[sn]), ((t + 1) / Cfg::kQStages) & 1, abort_flag);
            FA_STAMP(t, 6)
            if (ok) ok = mbar_wait(smem_u32(&sh.sdp_consumed), t & 1, abort_flag);
            FA_STAMP(t, 7)
            if (!ok) break;
            FA_PROF(1)
            tc_fence_after();
            issue_kk(tS_, smem_q + sn * Cfg::kTileBytes, smem_k);
            issue_kk(tDP_, smem_do + sn * Cfg::kTileBytes, smem_v);
            mma_commit(smem_u32(&sh.sdp_full));
            FA_PROF(2)
            FA_STAMP(t, 8)
          }
          ok = mbar_wait(smem_u32(&sh.pds_ready), t & 1, abort_flag);
          if (!ok) break;
          FA_PROF(3)
          FA_STAMP(t, 9)
          tc_fence_after();
          if (t > 0) {
            ok = mbar_wait(smem_u32(&sh.dq_consumed), (t - 1) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
          }
          FA_PROF(4)
          // its tile is read out of tensor memory while dV / dK are still running
          if constexpr (kDsInTmem) issue_dq_t(tDQ_, tDS_, smem_k);
          else issue_dq(tDQ_, smem_ds, smem_k);
          mma_commit(smem_u32(&sh.dq_full));
          FA_STAMP(t, 10)
          mma_commit(smem_u32(&sh.pds_free));
          FA_PROF(5)
        }
        FA_PROF_FLUSH(16, nm)
      }
    } else if (warp == 14 && lane == 0 && Cfg::kDualIssue) {
      // -------------------------------------------------------------- MMA issuer 2: dV
      // dV and dK have a thread each: an issuing thread gets an instruction out every ~130 clk
      // (it shares its scheduler with two compute warps), so the 16 instructions of the two products
      // took longer to issue than to execute and the compute groups waited for the buffers.
      bool ok = true;
      FA_PROF_DECL
      for (int t = 0; t < nm && ok; ++t) {
        const int s = t % Cfg::kQStages;
        FA_PROF(0)
        ok = mbar_wait(smem_u32(&sh.pds_ready), t & 1, abort_flag);
        if (!ok) break;
        FA_PROF(1)
        FA_STAMP(t, 11)
        tc_fence_after();
        issue_tt(tDV_, smem_p, smem_do + s * Cfg::kTileBytes, t > 0);
        FA_STAMP(t, 12)
        mma_commit(smem_u32(&sh.pds_free));
        mma_commit(smem_u32(&sh.q_empty[s]));
        FA_PROF(2)
      }
      FA_PROF_FLUSH(24, nm)
    } else if (warp == 15 && lane == 0 && Cfg::kDualIssue) {
      // -------------------------------------------------------------- MMA issuer 3: dK
      bool ok = true;
      for (int t = 0; t < nm && ok; ++t) {
        const int s = t % Cfg::kQStages;
        ok = mbar_wait(smem_u32(&sh.pds_ready), t & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        issue_tt(tDK_, smem_ds, smem_q + s * Cfg::kTileBytes, t > 0);
        FA_STAMP(t, 13)
        mma_commit(smem_u32(&sh.pds_free));
        mma_commit(smem_u32(&sh.q_empty[s]));
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ compute groups
    // group w (0 / 1) owns key columns [64 w, 64 w + 64) of the tile; one thread per query row
    if constexpr (D == 64) reg_alloc<192>(); else reg_alloc<176>();
    const int w = warp >> 2;
    const int row = tid & 127;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tS_ + lane_sel + w * 64;
    const uint32_t tDP = tDP_ + lane_sel + w * 64;
    const int64_t bh_sub =
        (static_cast<int64_t>(b) * ka.drop.heads_total + ka.drop.head_offset + h) * 256;
    const int L16 = (sq + 15) >> 4;
    const float* lse_row = ka.lse + (static_cast<int64_t>(b) * ka.heads + h) * ka.lse_stride;
    const float* d_row = a.softmax_d + (static_cast<int64_t>(b) * ka.heads + h) * ka.lse_stride;
    const uint64_t c2 = pack_f2(ka.scale_log2, ka.scale_log2);
    // dropout: per-lane generator state (lanes l and l ^ 8 share every Philox call)
    LanePhilox lp;
    float thr_term = 0.f;
    if constexpr (DROPOUT) {
      lp.init(ka.drop, bh_sub, row);
      thr_term = fa_keep_thr_term(ka.drop.threshold);
    }
    const int cbase = n0 + w * 64;  // first key column of this thread
    bool ok = true;
    FA_PROF_DECL
    constexpr bool kQuad = DROPOUT && !Cfg::kTwoPhase;
    if constexpr (kQuad) {
      // ---- d = 64 with dropout: quad layout.  A warp reads its 32 query rows as two 16-row blocks
      // (hh) with the 16x256b shape: a thread holds rows r8 and r8 + 8 of a block and two adjacent
      // columns of every 8-column unit, which is the ownership pattern of the reference's mask
      // generator (one Philox call = one thread's part of a 16 x 16 patch, QuadPhilox).  The packed
      // pairs go to the swizzled P~ / dS tiles with stmatrix (8 x 8 matrices = 16-byte row chunks).
      const int wq = warp & 3, lane = tid & 31;
      const int r8 = lane >> 2, q4 = lane & 3;
      constexpr uint32_t kHalf = 16u << 16;
      QuadPhilox<4> qp;
      qp.init(ka.drop, bh_sub, lane, w * 4);
      // stmatrix row address of this lane: matrix k = lane / 8 is (row half k & 1, unit k >> 1)
      const int st_row = wq * 32 + ((lane >> 3) & 1) * 8 + (lane & 7);   // + 16 * hh
      const int st_unit = lane >> 4;                                     // + first unit of the quadruple
      // per-row statistics (ri = hh * 2 + u) of the first tile; those of tile t + 1 are fetched while
      // tile t is processed
      float lse_nx[4], d_nx[4];
      int32_t bs_nx[2] = {0, 0};
      auto fetch_stats = [&](int t) {
#pragma unroll
        for (int ri = 0; ri < 4; ++ri) {
          const int ig_n = q_tile(t) * kBM + wq * 32 + (ri >> 1) * 16 + (ri & 1) * 8 + r8;
          const bool valid = ig_n < sq;
          lse_nx[ri] = valid ? lse_row[ig_n] : INFINITY;
          d_nx[ri] = valid ? d_row[ig_n] : 0.f;
        }
        if constexpr (BLOCKSPARSE) {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int i16 = (q_tile(t) * kBM + wq * 32 + hh * 16) >> 4;
            bs_nx[hh] = i16 < ka.bs_rows16
                            ? ka.bs_iter[(static_cast<int64_t>(b) * ka.bs_kblocks + (n0 >> 8)) * ka.bs_rows16 + i16]
                            : -1;
          }
        }
      };
      fetch_stats(0);
      for (int t = 0; t < nm && ok; ++t) {
        FA_PROF(0)
        const int m0 = q_tile(t) * kBM;
        const int row0 = m0 + wq * 32 + r8;  // + 16 * hh + 8 * u
        float lse2[4], d_i[4];
#pragma unroll
        for (int ri = 0; ri < 4; ++ri) { lse2[ri] = lse_nx[ri] * 1.4426950408889634f; d_i[ri] = d_nx[ri]; }
        const int32_t bs_it[2] = {bs_nx[0], bs_nx[1]};
        if (t + 1 < nm) fetch_stats(t + 1);

        // keep words of the thread's 2 x 4 patches (they do not depend on the scores: drawn before
        // the wait).  kw[hh * 4 + grp][2 * u + half]: row u, columns 16 grp + 8 half + 2 q4 (+1 high)
        uint32_t kw[8][4];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          int64_t it_tile;
          if constexpr (BLOCKSPARSE) it_tile = bs_it[hh];
          else it_tile = fa_iter_index(CAUSAL, n0 >> ka.drop.n_shift, (m0 + wq * 32 + hh * 16) >> 4, L16, ka.drop.n_shift);
          qp.set_tile(ka.drop, it_tile, n0);
#pragma unroll
          for (int g4 = 0; g4 < 4; ++g4) qp.start(g4, kw[hh * 4 + g4]);
        }
#pragma unroll
        for (int r = 2; r < 7; ++r)
#pragma unroll
          for (int k8 = 0; k8 < 8; ++k8) QuadPhilox<4>::round(ka.drop, kw[k8], r);

        const bool need_mask = (n0 + kBN > sk) || (CAUSAL && (n0 + kBN - 1 > m0));
        FA_PROF(1)
        if (w == 0 && row == 0) { FA_STAMP(t, 0) }
        ok = mbar_wait(smem_u32(&sh.sdp_full), t & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        FA_PROF(2)
        if (w == 0 && row == 0) { FA_STAMP(t, 1) }
        tc_fence_after();
        // everything goes to registers at once, so that the next tile's S and dP products can overwrite
        // tensor memory while this tile is still being processed
        uint32_t sr[2][32], dr[2][32];  // [hh][4 * unit + 2 * u + c]
        tmem_ld_quad32(tS, sr[0]);
        tmem_ld_quad32(tS + kHalf, sr[1]);
        tmem_ld_quad32(tDP, dr[0]);
        tmem_ld_quad32(tDP + kHalf, dr[1]);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(smem_u32(&sh.sdp_consumed));
        if (w == 0 && row == 0) { FA_STAMP(t, 2) }

#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t pp[16], pds[16];  // [2 * unit + u]: the stmatrix register order
          const bool blk_in_layout = !BLOCKSPARSE || bs_it[hh] >= 0;
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int ri = hh * 2 + u;
            const int ig = row0 + hh * 16 + u * 8;
            const uint64_t nlse2 = pack_f2(-lse2[ri], -lse2[ri]);
            const uint64_t nd2 = pack_f2(-d_i[ri], -d_i[ri]);
#pragma unroll
            for (int unit = 0; unit < 8; ++unit) {
              const int i = 4 * unit + 2 * u;
              float p0, p1;
              unpack_f2(fma2(pack_f2(__uint_as_float(sr[hh][i]), __uint_as_float(sr[hh][i + 1])), c2, nlse2), p0, p1);
              p0 = ex2f(p0);
              p1 = ex2f(p1);
              if (need_mask) {
                const int col = cbase + unit * 8 + 2 * q4;
                bool v0 = col < sk, v1 = col + 1 < sk;
                if (CAUSAL) { v0 = v0 && (col <= ig); v1 = v1 && (col + 1 <= ig); }
                if (!v0) p0 = 0.f;
                if (!v1) p1 = 0.f;
              }
              if (BLOCKSPARSE && !blk_in_layout) { p0 = 0.f; p1 = 0.f; }
              const uint32_t word = kw[hh * 4 + (unit >> 1)][2 * u + (unit & 1)];
              const uint64_t p01 = pack_f2(p0, p1);
              const uint64_t k01 = mul2(p01, pack_f2(fa_keep_factor_lo(word, thr_term), fa_keep_factor_hi(word, thr_term)));
              float k0, k1, s0, s1;
              unpack_f2(k01, k0, k1);
              // dS = P~ * dP - P * D  (P~ = P where kept, 0 where dropped)
              unpack_f2(fma2(k01, pack_f2(__uint_as_float(dr[hh][i]), __uint_as_float(dr[hh][i + 1])), mul2(p01, nd2)), s0, s1);
              pp[2 * unit + u] = pack_lowp<BF16>(k0, k1);
              pds[2 * unit + u] = pack_lowp<BF16>(s0, s1);
            }
          }
          // the previous tile's products must have finished reading the P~ / dS buffers
          if (hh == 0) { FA_PROF(3) }
          if (hh == 0 && t > 0) {
            ok = mbar_wait(smem_u32(&sh.pds_free), (t - 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
          }
          if (hh == 0) { FA_PROF(4) }
          if (hh == 0 && w == 0 && row == 0) { FA_STAMP(t, 3) }
          // four 8 x 8 matrices per instruction: (u = 0, 1) x (units a, a + 1) of the 64-column panel w
          const int srow = st_row + hh * 16;
#pragma unroll
          for (int a2 = 0; a2 < 8; a2 += 2) {
            const uint32_t off = w * 16384 + srow * 128 + (((a2 + st_unit) ^ (srow & 7)) << 4);
            stmatrix_x4(smem_u32(p_ptr + off), pp[2 * a2], pp[2 * a2 + 1], pp[2 * a2 + 2], pp[2 * a2 + 3]);
            stmatrix_x4(smem_u32(ds_ptr + off), pds[2 * a2], pds[2 * a2 + 1], pds[2 * a2 + 2], pds[2 * a2 + 3]);
          }
        }
        if (!ok) break;
        FA_PROF(5)
        fence_async_smem();
        mbar_arrive(smem_u32(&sh.pds_ready));
        FA_PROF(7)
        if (w == 0 && row == 0) { FA_STAMP(t, 4) }
      }
      if (w == 0 && row == 0) { FA_PROF_FLUSH(8, nm) }
    } else {

    // per-row statistics of the first tile; those of tile t + 1 are fetched while tile t is processed
    float lse_next = INFINITY, d_next = 0.f;
    int32_t bs_next = 0;
    auto fetch_row_stats = [&](int t) {
      const int ig_n = q_tile(t) * kBM + row;
      const bool valid = ig_n < sq;
      lse_next = valid ? lse_row[ig_n] : INFINITY;  // scaled at its first use, one tile later
      d_next = valid ? d_row[ig_n] : 0.f;
      if constexpr (BLOCKSPARSE) {
        bs_next = (ig_n >> 4) < ka.bs_rows16
                      ? ka.bs_iter[(static_cast<int64_t>(b) * ka.bs_kblocks + (n0 >> 8)) * ka.bs_rows16 + (ig_n >> 4)]
                      : -1;
      }
    };
    fetch_row_stats(0);

    for (int t = 0; t < nm && ok; ++t) {
      FA_PROF(0)
      const int m0 = q_tile(t) * kBM;
      const int ig = m0 + row;
      const float lse2 = lse_next * 1.4426950408889634f;
      const float d_i = d_next;
      const uint64_t nlse2 = pack_f2(-lse2, -lse2);
      const uint64_t nd2 = pack_f2(-d_i, -d_i);
      const int32_t bs_it = bs_next;
      const bool row_in_layout = !BLOCKSPARSE || bs_it >= 0;
      if (t + 1 < nm) fetch_row_stats(t + 1);

      // Keep words of this thread's 64 columns (wd[p] covers columns 2p, 2p + 1).  They do not depend
      // on the scores, so they are drawn before the wait for S and dP: eight independent Philox
      // calls (4 column groups x 2 quarters) with their rounds interleaved.
      uint32_t wd[DROPOUT ? 32 : 1];
      if constexpr (DROPOUT) {
        // one Philox iteration index per tile: a 128-column tile lies inside one key block
        int64_t it_tile;
        if constexpr (BLOCKSPARSE) it_tile = bs_it;
        else it_tile = fa_iter_index(CAUSAL, n0 >> ka.drop.n_shift, ig >> 4, L16, ka.drop.n_shift);
        lp.set_tile(ka.drop, it_tile, n0);
        uint32_t st[8][4];
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) {
          lp.start(w * 4 + g4, 0, st[2 * g4]);
          lp.start(w * 4 + g4, 1, st[2 * g4 + 1]);
        }
#pragma unroll
        for (int r = 0; r < 7; ++r)
#pragma unroll
          for (int k8 = 0; k8 < 8; ++k8) lp.round(st[k8], r);
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) lp.finish(st[2 * g4], st[2 * g4 + 1], wd + g4 * 8);
      }

      const bool need_mask = (n0 + kBN > sk) || (CAUSAL && (n0 + kBN - 1 > m0));
      if constexpr (Cfg::kTwoPhase) {
        // ---- phase one: P from S.  P~ goes to shared memory (dV can start), P stays in registers.
        FA_PROF(1)
        if (w == 0 && row == 0) { FA_STAMP(t, 0) }
        ok = mbar_wait(smem_u32(&sh.s_full), t & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        FA_PROF(2)
        if (w == 0 && row == 0) { FA_STAMP(t, 1) }
        tc_fence_after();
        uint32_t pf[2][32];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t sr[32];
          tmem_ld32(tS + c * 32, sr);
          tmem_wait_ld();
          if (c == 1) {
            tc_fence_before();
            mbar_arrive(smem_u32(&sh.sdp_consumed));
            if (w == 0 && row == 0) { FA_STAMP(t, 2) }
          }
          uint32_t pp[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0, p1;
            unpack_f2(fma2(pack_f2(__uint_as_float(sr[i]), __uint_as_float(sr[i + 1])), c2, nlse2), p0, p1);
            p0 = ex2f(p0);
            p1 = ex2f(p1);
            if (need_mask) {
              const int col = cbase + c * 32 + i;
              bool v0 = col < sk, v1 = col + 1 < sk;
              if (CAUSAL) { v0 = v0 && (col <= ig); v1 = v1 && (col + 1 <= ig); }
              if (!v0) p0 = 0.f;
              if (!v1) p1 = 0.f;
            }
            if (BLOCKSPARSE && !row_in_layout) { p0 = 0.f; p1 = 0.f; }
            pf[c][i] = __float_as_uint(p0);
            pf[c][i + 1] = __float_as_uint(p1);
            float k0 = p0, k1 = p1;
            if constexpr (DROPOUT) {
              const uint32_t word = wd[c * 16 + (i >> 1)];
              unpack_f2(mul2(pack_f2(p0, p1),
                             pack_f2(fa_keep_factor_lo(word, thr_term), fa_keep_factor_hi(word, thr_term))), k0, k1);
            }
            pp[i >> 1] = pack_lowp<BF16>(k0, k1);
          }
          // dV of the previous tile must have finished reading the P~ buffer
          if (c == 0 && t > 0) {
            ok = mbar_wait(smem_u32(&sh.pds_free), (t - 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
          }
#pragma unroll
          for (int ch4 = 0; ch4 < 4; ++ch4) {
            const int ch = c * 4 + ch4;
            const uint32_t off = w * 16384 + row * 128 + ((ch ^ (row & 7)) << 4);
            *reinterpret_cast<uint4*>(p_ptr + off) =
                make_uint4(pp[4 * ch4], pp[4 * ch4 + 1], pp[4 * ch4 + 2], pp[4 * ch4 + 3]);
          }
        }
        if (!ok) break;
        fence_async_smem();
        mbar_arrive(smem_u32(&sh.p_ready));
        FA_PROF(3)
        if (w == 0 && row == 0) { FA_STAMP(t, 3) }

        // ---- phase two: dS = P~ * dP - P * D from dP
        ok = mbar_wait(smem_u32(&sh.sdp_full), t & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        FA_PROF(4)
        if (w == 0 && row == 0) { FA_STAMP(t, 13) }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t dr[32];
          tmem_ld32(tDP + c * 32, dr);
          tmem_wait_ld();
          uint32_t pds[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const uint64_t p01 = pack_f2(__uint_as_float(pf[c][i]), __uint_as_float(pf[c][i + 1]));
            uint64_t k01 = p01;
            if constexpr (DROPOUT) {
              const uint32_t word = wd[c * 16 + (i >> 1)];
              k01 = mul2(p01, pack_f2(fa_keep_factor_lo(word, thr_term), fa_keep_factor_hi(word, thr_term)));
            }
            float s0, s1;
            unpack_f2(fma2(k01, pack_f2(__uint_as_float(dr[i]), __uint_as_float(dr[i + 1])), mul2(p01, nd2)), s0, s1);
            pds[i >> 1] = pack_lowp<BF16>(s0, s1);
          }
          // dK, dQ of the previous tile must have finished reading the dS buffer
          if (c == 0 && t > 0) {
            ok = mbar_wait(smem_u32(&sh.ds_free), (t - 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
          }
#pragma unroll
          for (int ch4 = 0; ch4 < 4; ++ch4) {
            const int ch = c * 4 + ch4;
            const uint32_t off = w * 16384 + row * 128 + ((ch ^ (row & 7)) << 4);
            *reinterpret_cast<uint4*>(ds_ptr + off) =
                make_uint4(pds[4 * ch4], pds[4 * ch4 + 1], pds[4 * ch4 + 2], pds[4 * ch4 + 3]);
          }
        }
        tc_fence_before();  // the dP columns are about to be overwritten by dQ
      } else {
      FA_PROF(1)
      if (w == 0 && row == 0) { FA_STAMP(t, 0) }
      ok = mbar_wait(smem_u32(&sh.sdp_full), t & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      FA_PROF(2)
      if (w == 0 && row == 0) { FA_STAMP(t, 1) }
      tc_fence_after();

      // This thread's 64 scores and 64 dP values go to registers at once, so that the next tile's
      // S and dP products can overwrite tensor memory while this tile is still being processed.
      // (d = 64 only: at d = 128 the next dP waits for the dQ read-out anyway, and the registers
      // are better spent elsewhere, so there the values are loaded 32 columns at a time.)
      constexpr bool kEarly = (D == 64);
      uint32_t sr_all[kEarly ? 2 : 1][32], dr_all[kEarly ? 2 : 1][32];
      if constexpr (kEarly) {
        tmem_ld32(tS, sr_all[0]);
        tmem_ld32(tS + 32, sr_all[1]);
        tmem_ld32(tDP, dr_all[0]);
        tmem_ld32(tDP + 32, dr_all[1]);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(smem_u32(&sh.sdp_consumed));
        if (w == 0 && row == 0) { FA_STAMP(t, 2) }
      }
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t(&sr)[32] = sr_all[kEarly ? c : 0];
        uint32_t(&dr)[32] = dr_all[kEarly ? c : 0];
        if constexpr (!kEarly) {
          tmem_ld32(tS + c * 32, sr);
          tmem_ld32(tDP + c * 32, dr);
        }

        uint32_t pp[16], pds[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0, p1;
          unpack_f2(fma2(pack_f2(__uint_as_float(sr[i]), __uint_as_float(sr[i + 1])), c2, nlse2), p0, p1);
          p0 = ex2f(p0);
          p1 = ex2f(p1);
          if (need_mask) {
            const int col = cbase + c * 32 + i;
            bool v0 = col < sk, v1 = col + 1 < sk;
            if (CAUSAL) { v0 = v0 && (col <= ig); v1 = v1 && (col + 1 <= ig); }
            if (!v0) p0 = 0.f;
            if (!v1) p1 = 0.f;
          }
          if (BLOCKSPARSE && !row_in_layout) { p0 = 0.f; p1 = 0.f; }
          float k0 = p0, k1 = p1;
          uint64_t k01 = pack_f2(p0, p1);
          if constexpr (DROPOUT) {
            const uint32_t word = wd[c * 16 + (i >> 1)];
            k01 = mul2(k01, pack_f2(fa_keep_factor_lo(word, thr_term), fa_keep_factor_hi(word, thr_term)));
            unpack_f2(k01, k0, k1);
          }
          // dS = P~ * dP - P * D  (P~ = P where kept, 0 where dropped)
          float s0, s1;
          unpack_f2(fma2(k01, pack_f2(__uint_as_float(dr[i]), __uint_as_float(dr[i + 1])),
                         mul2(pack_f2(p0, p1), nd2)), s0, s1);
          pp[i >> 1] = pack_lowp<BF16>(k0, k1);
          pds[i >> 1] = pack_lowp<BF16>(s0, s1);
        }
        // the previous tile's products must have finished reading the P~ / dS buffers
        if (c == 0) { FA_PROF(3) }
        if (c == 0 && t > 0) {
          ok = mbar_wait(smem_u32(&sh.pds_free), (t - 1) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
        }
        if (c == 0) { FA_PROF(4) }
        if (c == 0 && w == 0 && row == 0) { FA_STAMP(t, 3) }
        // 32 16-bit values = 4 chunks of 16 bytes of this row in the 64-column panel w
#pragma unroll
        for (int ch4 = 0; ch4 < 4; ++ch4) {
          const int ch = c * 4 + ch4;
          const uint32_t off = w * 16384 + row * 128 + ((ch ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(p_ptr + off) =
              make_uint4(pp[4 * ch4], pp[4 * ch4 + 1], pp[4 * ch4 + 2], pp[4 * ch4 + 3]);
          *reinterpret_cast<uint4*>(ds_ptr + off) =
              make_uint4(pds[4 * ch4], pds[4 * ch4 + 1], pds[4 * ch4 + 2], pds[4 * ch4 + 3]);
        }
        // second copy of dS for the dQ product (32 keys = 16 packed columns of this half)
        if constexpr (kDsInTmem) tmem_st16(tDS_ + lane_sel + w * 32 + c * 16, pds);
      }
      }
      if (!ok) break;
      FA_PROF(6)
      if constexpr (kDsInTmem) {
        tmem_wait_st();
        tc_fence_before();
      }
      fence_async_smem();
      mbar_arrive(smem_u32(&sh.pds_ready));
      FA_PROF(7)
      if (w == 0 && row == 0) { FA_STAMP(t, 4) }
    }
    if (w == 0 && row == 0) { FA_PROF_FLUSH(8, nm) }
    }  // row-per-thread layout

    // ---------------- epilogue: group 0 writes dV = acc / p_keep, group 1 writes dK = acc * scale / p_keep
    if (ok) {
      ok = mbar_wait(smem_u32(&sh.pds_free), (nm - 1) & 1, abort_flag);
      if constexpr (Cfg::kTwoPhase) {
        if (ok) ok = mbar_wait(smem_u32(&sh.ds_free), (nm - 1) & 1, abort_flag);
      }
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const uint32_t tAcc = (w == 0 ? tDV_ : tDK_) + lane_sel;
      const float f = (w == 0) ? rp_keep : ka.scale * rp_keep;
      const int kr = n0 + row;
      uint16_t* dst_row = (w == 0)
          ? dv_base + static_cast<int64_t>(k_start + kr) * a.dv_row_stride + static_cast<int64_t>(h) * a.dv_head_stride
          : dk_base + static_cast<int64_t>(k_start + kr) * a.dk_row_stride + static_cast<int64_t>(h) * a.dk_head_stride;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tAcc + c * 32, r);
        tmem_wait_ld();
        if (kr < sk && c * 32 < ka.head_dim) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            pk[i] = pack_lowp<BF16>(__uint_as_float(r[2 * i]) * f, __uint_as_float(r[2 * i + 1]) * f);
          uint4* dst = reinterpret_cast<uint4*>(dst_row + c * 32);
          const int nvec = min(4, (ka.head_dim - c * 32) / 8);
#pragma unroll
          for (int v = 0; v < 4; ++v)
            if (v < nvec) dst[v] = make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ dQ group (warps 8-11)
    // dQ tile: tensor memory -> registers -> swizzled fp32 staging in shared memory -> one TMA
    // reduce-add per [128 rows x 32 columns] box into the fp32 accumulator.  Rows past the end of
    // the sequence hold exact zeros (their P is zero), rows past the tensor are clipped by TMA.
    if constexpr (D == 64) reg_dealloc<72>(); else reg_dealloc<88>();
    const int row = tid - 256;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tDQ = tDQ_ + lane_sel;
    const uint32_t stage_addr = smem_u32(dq_stage);
    bool ok = true;
    bool pending = false;  // thread `row == 0`: a reduce group of this CTA may still read the staging
    uint32_t sync_phase = 0;
    auto group_sync = [&]() -> bool {
      mbar_arrive(smem_u32(&sh.dq_group));
      const bool done = mbar_wait(smem_u32(&sh.dq_group), sync_phase & 1, abort_flag);
      ++sync_phase;
      return done;
    };
    // Deterministic mode (thread `row == 0` only): wait until the key tiles before this one have
    // added their share of the query tile, add, wait for the adds to complete and pass the turn on.
    int32_t* ticket_row = deterministic
        ? a.dq_tickets + (static_cast<int64_t>(b) * ka.heads + h) * a.ticket_stride : nullptr;
    auto ticket_wait = [&](int t) -> bool {
      int32_t want;
      if constexpr (BLOCKSPARSE) want = qtile_order[t];
      else want = nt;
      const volatile int32_t* tk = ticket_row + q_tile(t);
      if (*abort_flag) return false;
      const long long t0 = clock64();
      while (true) {
        int32_t cur;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(cur) : "l"(tk) : "memory");
        if (cur >= want) break;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) { *abort_flag = 1; return false; }
      }
      // the adds below go through the async proxy
      asm volatile("fence.proxy.async.global;" ::: "memory");
      return true;
    };
    bool my_turn = true;
    auto ticket_pass = [&](int t) {
      bulk_wait_all();
      asm volatile("fence.proxy.async.global;" ::: "memory");
      __threadfence();
      int32_t* tk = ticket_row + q_tile(t);
      asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(tk) : "memory");
    };
    FA_PROF_DECL
    for (int t = 0; t < nm && ok; ++t) {
      const int m0 = q_tile(t) * kBM;
      FA_PROF(0)
      ok = mbar_wait(smem_u32(&sh.dq_full), t & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      FA_PROF(1)
      if (row == 0) { FA_STAMP(t, 14) }
      tc_fence_after();
      if constexpr (Cfg::kAliasDq) {
        // dQ shares its columns with the next dP, so the columns are released as early as possible:
        // both boxes of a 64-column half go to registers before anything waits for the staging
        // buffer, and the release follows the loads of the second half.
#pragma unroll
        for (int half = 0; half < D / 64; ++half) {
          uint32_t r0[32], r1[32];
          tmem_ld32(tDQ + half * 64, r0);
          tmem_ld32(tDQ + half * 64 + 32, r1);
          tmem_wait_ld();
          if (half == D / 64 - 1) {
            tc_fence_before();
            mbar_arrive(smem_u32(&sh.dq_consumed));
          }
          // the staging buffer is free once the previous reduce has read it
          if (row == 0 && pending) bulk_wait_read();
          ok = group_sync();
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            const uint32_t off = row * 128 + ((ch ^ (row & 7)) << 4);
            *reinterpret_cast<uint4*>(dq_stage + off) = make_uint4(r0[4 * ch], r0[4 * ch + 1], r0[4 * ch + 2], r0[4 * ch + 3]);
            *reinterpret_cast<uint4*>(dq_stage + 16384 + off) = make_uint4(r1[4 * ch], r1[4 * ch + 1], r1[4 * ch + 2], r1[4 * ch + 3]);
          }
          fence_async_smem();
          ok = group_sync();
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (row == 0) {
            // on expiry the abort flag is set, this tile's add is skipped and every role leaves
            // at its next wait
            if (deterministic && half == 0) my_turn = ticket_wait(t);
            if (my_turn) {
              tma_reduce_add_3d(&tm_dq, stage_addr, half * 64, q_start + m0, h);
              tma_reduce_add_3d(&tm_dq, stage_addr + 16384, half * 64 + 32, q_start + m0, h);
              bulk_commit();
              pending = true;
              if (deterministic && half == D / 64 - 1) { ticket_pass(t); pending = false; }
            }
          }
        }

      } else {
#pragma unroll
      for (int half = 0; half < D / 64; ++half) {
#pragma unroll
        for (int bx = 0; bx < 2; ++bx) {
          uint32_t r[32];
          tmem_ld32(tDQ + half * 64 + bx * 32, r);
          tmem_wait_ld();
          if (half == D / 64 - 1 && bx == 1) {
            tc_fence_before();
            mbar_arrive(smem_u32(&sh.dq_consumed));
          }
          if (bx == 0) {
            // the staging buffer is free once the previous reduce has read it
            if (row == 0 && pending) bulk_wait_read();
            ok = group_sync();
            ok = __all_sync(0xffffffffu, ok);
          }
          if (ok) {
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
              const uint32_t off = bx * 16384 + row * 128 + ((ch ^ (row & 7)) << 4);
              *reinterpret_cast<uint4*>(dq_stage + off) = make_uint4(r[4 * ch], r[4 * ch + 1], r[4 * ch + 2], r[4 * ch + 3]);
            }
          }
        }
        if (!ok) break;
        fence_async_smem();
        ok = group_sync();
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (row == 0) {
          if (deterministic && half == 0) my_turn = ticket_wait(t);
          if (my_turn) {
            tma_reduce_add_3d(&tm_dq, stage_addr, half * 64, q_start + m0, h);
            tma_reduce_add_3d(&tm_dq, stage_addr + 16384, half * 64 + 32, q_start + m0, h);
            bulk_commit();
            pending = true;
            if (deterministic && half == D / 64 - 1) { ticket_pass(t); pending = false; }
          }
        }
      }
      }
      FA_PROF(2)
      if (row == 0) { FA_STAMP(t, 15) }
    }
    if (row == 0 && pending) bulk_wait_all();
    if (row == 0) { FA_PROF_FLUSH(32, nm) }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 12) {
    tmem_dealloc(tmem, 512);
    if (lane == 0 && sh.abort_flag && ka.status) {
      atomicExch(ka.status, ka.launch_id);  // stops the CTAs of this launch that have not started yet
      atomicExch(ka.status + 3, 1);  // sticky: read by the host
    }
  }
}

// ------------------------------------------------------------------------------------------------
// softmax_d = p_keep * rowsum(dO * O); zero the dQ accumulator.  One thread per 8 elements.
template <bool BF16>
__global__ void bwd_preprocess_kernel(const BwdArgs a, int dpad) {
  const KernelArgs& ka = a.k;
  const int b = blockIdx.z, h = blockIdx.y;
  const int q_start = ka.cu_seqlens_q[b];
  const int sq = ka.cu_seqlens_q[b + 1] - q_start;
  const int d = ka.head_dim;
  const int tpr = d / 8;                      // threads per row: 2, 4, 8 or 16
  const int rows_per_block = blockDim.x / tpr;
  const int r = threadIdx.x / tpr, c = (threadIdx.x % tpr) * 8;
  const int i = blockIdx.x * rows_per_block + r;
  if (a.dq_tickets != nullptr && blockIdx.x == 0) {
    int32_t* tk = a.dq_tickets + (static_cast<int64_t>(b) * ka.heads + h) * a.ticket_stride;
    for (int t = threadIdx.x; t < a.ticket_stride; t += blockDim.x) tk[t] = 0;
  }
  float acc = 0.f;
  if (i < sq) {
    const int64_t row = q_start + i;
    const uint16_t* o = reinterpret_cast<const uint16_t*>(a.o_in) + row * ka.o_row_stride + h * ka.o_head_stride + c;
    const uint16_t* g = reinterpret_cast<const uint16_t*>(a.dout) + row * a.do_row_stride + h * a.do_head_stride + c;
    const uint4 ov = *reinterpret_cast<const uint4*>(o);
    const uint4 gv = *reinterpret_cast<const uint4*>(g);
    const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 of, gf;
      if constexpr (BF16) {
        of = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ow[k]));
        gf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[k]));
      } else {
        of = __half22float2(*reinterpret_cast<const __half2*>(&ow[k]));
        gf = __half22float2(*reinterpret_cast<const __half2*>(&gw[k]));
      }
      acc += of.x * gf.x + of.y * gf.y;
    }
    // zero this thread's share of the fp32 dQ accumulator row (dpad floats per (row, head))
    float* zr = a.dq_accum + (row * ka.heads + h) * dpad;
    for (int z = (threadIdx.x % tpr) * 4; z < dpad; z += tpr * 4)
      *reinterpret_cast<float4*>(zr + z) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int off = tpr / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (i < sq && (threadIdx.x % tpr) == 0)
    a.softmax_d[(static_cast<int64_t>(b) * ka.heads + h) * ka.lse_stride + i] = acc * a.p_keep;
}

// dq = accumulator * scale / p_keep.  One thread per 8 elements.
template <bool BF16>
__global__ void bwd_postprocess_kernel(const BwdArgs a, int dpad) {
  const KernelArgs& ka = a.k;
  const int d = ka.head_dim;
  const int tpr = d / 8;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = static_cast<int64_t>(a.total_q) * ka.heads * tpr;
  if (idx >= total) return;
  const int c = static_cast<int>(idx % tpr) * 8;
  const int64_t rh = idx / tpr;
  const int h = static_cast<int>(rh % ka.heads);
  const int64_t row = rh / ka.heads;
  // Rows behind the last sequence (a token buffer larger than cu_seqlens_q[batch]) belong to nobody:
  // the accumulator was not cleared there and dq keeps what the caller put in it, as in the
  // reference, which only ever writes rows of a sequence.
  if (row >= ka.cu_seqlens_q[ka.batch]) return;
  const float* src = a.dq_accum + rh * dpad + c;
  const float4 x = *reinterpret_cast<const float4*>(src);
  const float4 y = *reinterpret_cast<const float4*>(src + 4);
  const float f = ka.scale * ka.rp_keep;
  uint4 out;
  out.x = pack16<BF16>(x.x * f, x.y * f);
  out.y = pack16<BF16>(x.z * f, x.w * f);
  out.z = pack16<BF16>(y.x * f, y.y * f);
  out.w = pack16<BF16>(y.z * f, y.w * f);
  uint16_t* dst = reinterpret_cast<uint16_t*>(a.dq) + row * a.dq_row_stride + h * a.dq_head_stride + c;
  *reinterpret_cast<uint4*>(dst) = out;
}

template <int D, bool BF16, bool CAUSAL, bool DROPOUT, bool BS>
cudaError_t launch_main(const BwdLaunch& l, cudaStream_t stream) {
  auto kernel = fa_bwd_kernel<D, BF16, CAUSAL, DROPOUT, BS>;
  constexpr int smem = BwdCfg<D, BS>::kSmemBytes;
  static SmemLimitFlags smem_limit_set;  // one per template instantiation of this function
  cudaError_t e = set_smem_limit_once(kernel, smem, smem_limit_set);
  if (e != cudaSuccess) return e;
  dim3 grid((l.args.max_seqlen_k + kBN - 1) / kBN, l.args.k.heads, l.args.k.batch);
  kernel<<<grid, kBwdThreads, smem, stream>>>(l.tm_q, l.tm_k, l.tm_v, l.tm_do, l.tm_dq, l.args);
  return cudaGetLastError();
}

template <int D, bool BF16, bool CAUSAL>
cudaError_t launch_dd(const BwdLaunch& l, cudaStream_t stream) {
  return l.is_dropout ? launch_main<D, BF16, CAUSAL, true, false>(l, stream)
                      : launch_main<D, BF16, CAUSAL, false, false>(l, stream);
}

template <int D>
cudaError_t launch_d(const BwdLaunch& l, cudaStream_t stream) {
  if (l.is_bf16) {
    return l.is_causal ? launch_dd<D, true, true>(l, stream) : launch_dd<D, true, false>(l, stream);
  }
  return l.is_causal ? launch_dd<D, false, true>(l, stream) : launch_dd<D, false, false>(l, stream);
}

}  // namespace

cudaError_t launch_bwd(const BwdLaunch& l, cudaStream_t stream) {
  const BwdArgs& a = l.args;
  const int d = a.k.head_dim;
  const int stages = l.stage_mask == 0 ? 7 : l.stage_mask;
  // 1. preprocess
  if (stages & 1) {
    const int tpr = d / 8;
    const int threads = 256;
    const int rows_per_block = threads / tpr;
    dim3 grid((a.max_seqlen_q + rows_per_block - 1) / rows_per_block, a.k.heads, a.k.batch);
    if (l.is_bf16) bwd_preprocess_kernel<true><<<grid, threads, 0, stream>>>(a, l.dpad);
    else bwd_preprocess_kernel<false><<<grid, threads, 0, stream>>>(a, l.dpad);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  // 2. main
  if (stages & 2) {
    cudaError_t e;
    if (a.k.bs_iter != nullptr) {
      // block-sparse exists for fp16 and head_dim <= 64 (checked by the C ABI)
      if (l.is_causal)
        e = l.is_dropout ? launch_main<64, false, true, true, true>(l, stream)
                         : launch_main<64, false, true, false, true>(l, stream);
      else
        e = l.is_dropout ? launch_main<64, false, false, true, true>(l, stream)
                         : launch_main<64, false, false, false, true>(l, stream);
    } else {
      e = l.dpad == 64 ? launch_d<64>(l, stream) : launch_d<128>(l, stream);
    }
    if (e != cudaSuccess) return e;
  }
  // 3. postprocess
  if (stages & 4) {
    const int64_t total = static_cast<int64_t>(a.total_q) * a.k.heads * (d / 8);
    if (total > 0) {
      const int threads = 256;
      const int blocks = static_cast<int>((total + threads - 1) / threads);
      if (l.is_bf16) bwd_postprocess_kernel<true><<<blocks, threads, 0, stream>>>(a, l.dpad);
      else bwd_postprocess_kernel<false><<<blocks, threads, 0, stream>>>(a, l.dpad);
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return e;
    }
  }
  return cudaSuccess;
}

}  // namespace fa
