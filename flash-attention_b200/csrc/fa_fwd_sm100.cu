// FlashAttention forward for sm_100a.
//
// One CTA owns two consecutive 128-row query tiles of one (batch, head) pair and walks the key /
// value sequence in 128-row tiles.  Warp roles:
//   warps 0-3   softmax group 0 (query tile 0): one thread per query row; with dropout a thread
//               holds two rows of each of the warp's two 16-row blocks and a quarter of their
//               columns (the ownership pattern of the reference's mask generator)
//   warps 4-7   softmax group 1 (query tile 1)
//   warp  8     TMA producer (Q once, K/V ring)
//   warp  9     tcgen05.mma issuer (d = 128: every product; d = 64: S = Q K^T only)
//   warp 10     d = 64: second issuer, O += P V (an issuing thread shares its scheduler with two
//               softmax warps and gets an instruction out every 77-110 clk; two issuers keep S ahead)
//   warp 11     idle
// Tensor memory (512 columns): S0 [0,128) S1 [128,256) fp32 scores, O0 / O1 fp32 outputs behind
// them.  The 16-bit probabilities P feed the P*V product straight from tensor memory; at d = 128
// they overwrite the first 64 columns of their S buffer, at d = 64 they have columns of their own,
// so the next score product can start as soon as the group has read its scores into registers.
// The softmax groups are the bottleneck at every head size: their run time follows the sum of their
// instruction costs (exponentials on the special-function unit, the dropout generator on the wide
// integer multiplies, packed fp32 arithmetic), about 12 clk per score element and scheduler without
// dropout and 25 with, against 4 (d = 64) or 8 (d = 128) clk of tensor-core time.
//
// Numerics follow the reference forward (csrc/flash_attn/src/fmha_fprop_kernel_1xN.h:365-638):
// scores in fp32, p = exp2(scale*log2e*(s - max)), row sum of the un-dropped p, P rounded to the
// 16-bit input type before P*V, O accumulated in fp32 and scaled by 1/(sum * p_keep) at the end,
// LSE = max*scale + ln(sum), -inf for a row without any valid key.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "fa_kernels.h"
#include "fa_math.cuh"
#include "sm100_prims.cuh"

namespace fa {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kFwdThreads = 384;  // 2 softmax warpgroups + 1 (producer, MMA issuers, idle)

template <int D>
struct FwdCfg {
  static constexpr int kStages = (D == 64) ? 3 : 2;
  static constexpr int kPanels = D / 64;
  static constexpr int kTileBytes = kBlockM * D * 2;
  static constexpr int kSmemBytes = (2 + 2 * kStages) * kTileBytes + 1024;
  static constexpr uint32_t kTmemS0 = 0, kTmemS1 = 128, kTmemO0 = 256, kTmemO1 = 256 + D;
  // d = 64 leaves 128 tensor-memory columns free: P gets its own columns there, so the next
  // S = Q K^T can be issued as soon as the softmax group has read the current S into registers.
  // At d = 128 the 512 columns are full and P overwrites the first 64 columns of its S buffer.
  static constexpr bool kSeparateP = (D == 64);
  static constexpr uint32_t kTmemP0 = kSeparateP ? 384 : kTmemS0, kTmemP1 = kSeparateP ? 448 : kTmemS1;
};

constexpr int kMaxSparseTiles = 1024;  // key tiles of 128 per sequence in block-sparse mode

struct FwdShared {
  uint64_t q_full[2];
  uint64_t k_full[3], k_empty[3], v_full[3], v_empty[3];
  uint64_t s_full[2], s_free[2], p_full[2], o_full[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Optional cycle accounting (build with -DFA_PROFILE): thread 0 of softmax group 0 and the MMA
// thread of CTA (0,0,0) accumulate the cycles they spend in each phase into status[8..].
#ifdef FA_PROFILE
#define FA_PROF_DECL long long prof_t = clock64(); long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define FA_PROF(slot) { const long long now_ = clock64(); prof_acc[slot] += now_ - prof_t; prof_t = now_; }
#define FA_PROF_FLUSH(base, n) if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && a.status) { \
    for (int i_ = 0; i_ < 8; ++i_) a.status[(base) + i_] = static_cast<int32_t>(prof_acc[i_] / ((n) > 0 ? (n) : 1)); }
// time stamps (low 32 bits of the SM clock) of the events of kv steps 5, 6 of CTA (0,0,0): slot =
// 64 + (step - 5) * 24 + idx, for a timeline across the roles
#define FA_STAMP(step, idx) if ((step) >= 5 && (step) <= 6 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && a.status) { \
    a.status[64 + ((step) - 5) * 24 + (idx)] = static_cast<int32_t>(clock64()); }
#else
#define FA_PROF_DECL
#define FA_PROF(slot)
#define FA_PROF_FLUSH(base, n)
#define FA_STAMP(step, idx)
#endif

template <int N>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// Epilogue of one query row (thread = row, 32x32b shape): O = acc / (sum * p_keep) in the 16-bit
// type, LSE = max * scale + ln(sum); a row without any valid key gets zeros and -inf.
template <int D, bool BF16>
__device__ __forceinline__ void store_rows(const KernelArgs& a, uint32_t tO, bool have_acc, bool ok, int ig,
                                           int sq, int q_start, int b, int h, float m_run, float l_run) {
  const bool bad_sum = (l_run == 0.f) || (l_run != l_run);
  const float inv = bad_sum ? 1.f : (1.f / l_run) * a.rp_keep;
  const bool store_row = ok && (ig < sq);
  uint16_t* orow = reinterpret_cast<uint16_t*>(a.o) + static_cast<int64_t>(q_start + ig) * a.o_row_stride +
                   static_cast<int64_t>(h) * a.o_head_stride;
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    uint32_t orr[32];
    if (have_acc) {
      tmem_ld32(tO + c * 32, orr);
      tmem_wait_ld();
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) orr[i] = 0u;
    }
    if (store_row && c * 32 < a.head_dim) {
      uint32_t pko[16];
#pragma unroll
      for (int i = 0; i < 16; ++i)
        pko[i] = pack_lowp<BF16>(__uint_as_float(orr[2 * i]) * inv, __uint_as_float(orr[2 * i + 1]) * inv);
      uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
      const int nvec = min(4, (a.head_dim - c * 32) / 8);
#pragma unroll
      for (int v = 0; v < 4; ++v)
        if (v < nvec) dst[v] = make_uint4(pko[4 * v], pko[4 * v + 1], pko[4 * v + 2], pko[4 * v + 3]);
    }
  }
  if (store_row) {
    const float lse = bad_sum ? -INFINITY : (m_run * a.scale + __logf(l_run));
    a.lse[(static_cast<int64_t>(b) * a.heads + h) * a.lse_stride + ig] = lse;
  }
}

template <int D, bool BF16, bool CAUSAL, bool DROPOUT, bool BLOCKSPARSE>
__global__ void __launch_bounds__(kFwdThreads, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const KernelArgs a) {
  using Cfg = FwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ FwdShared sh;
  // block-sparse: key tiles this CTA visits (ascending), built from the layout table
  __shared__ uint16_t tile_list[BLOCKSPARSE ? kMaxSparseTiles : 1];
  __shared__ int tile_count;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  const int b = blockIdx.z;
  const int h = blockIdx.y;
  const int mp = CAUSAL ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;  // heavy tiles first
  const int q_start = a.cu_seqlens_q[b];
  const int sq = a.cu_seqlens_q[b + 1] - q_start;
  const int k_start = a.cu_seqlens_k[b];
  const int sk = a.cu_seqlens_k[b + 1] - k_start;
  if (mp * 2 * kBlockM >= sq) return;
  // fail fast: once a CTA of this launch has abandoned a wait, the remaining CTAs do not start
  if (a.status && *reinterpret_cast<volatile int32_t*>(a.status) == a.launch_id) return;

  int n_kv_total = (sk + kBlockN - 1) / kBlockN;
  if constexpr (BLOCKSPARSE) {
    // A key tile is visited when any 16-row block of this CTA's 256 query rows has its 256-column
    // key block in the layout; rows whose block is absent are masked inside the tile.
    uint8_t* flags = reinterpret_cast<uint8_t*>(smem_raw);
    const int rb0 = mp * (2 * kBlockM / 16);
    const int rb1 = min(min(rb0 + 2 * kBlockM / 16, a.bs_rows16), (sq + 15) >> 4);
    n_kv_total = min(n_kv_total, kMaxSparseTiles);
    for (int j = tid; j < n_kv_total; j += kFwdThreads) {
      const int32_t* row = a.bs_iter + (static_cast<int64_t>(b) * a.bs_kblocks + (j >> 1)) * a.bs_rows16;
      bool any = false;
      for (int rb = rb0; rb < rb1; ++rb) any = any || (row[rb] >= 0);
      // causal: a key tile that starts behind the CTA's last query row is masked entirely
      if (CAUSAL && j * kBlockN > mp * 2 * kBlockM + 2 * kBlockM - 1) any = false;
      flags[j] = any ? 1 : 0;
    }
    __syncthreads();
    if (tid == 0) {
      int n = 0;
      for (int j = 0; j < n_kv_total; ++j)
        if (flags[j]) tile_list[n++] = static_cast<uint16_t>(j);
      tile_count = n;
    }
    __syncthreads();
    n_kv_total = tile_count;
    __syncthreads();  // flags live in the tile buffers: finish reading before TMA may overwrite
  }
  auto kv_tile = [&](int j) -> int {
    if constexpr (BLOCKSPARSE) return tile_list[j];
    else return j;
  };
  int m0[2], n_tiles[2];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    m0[g] = (mp * 2 + g) * kBlockM;
    const bool active = m0[g] < sq;
    int n = n_kv_total;
    if constexpr (CAUSAL && BLOCKSPARSE) {
      // listed key tiles (ascending) up to the one that holds this query tile's diagonal
      n = 0;
      while (n < n_kv_total && tile_list[n] <= m0[g] / kBlockN) ++n;
    } else if (CAUSAL) {
      n = min(n, m0[g] / kBlockN + 1);
    }
    n_tiles[g] = active ? n : 0;
  }
  const int n_max = max(n_tiles[0], n_tiles[1]);

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t smem_q = smem_u32(smem);
  const uint32_t smem_k = smem_q + 2 * Cfg::kTileBytes;
  const uint32_t smem_v = smem_k + Cfg::kStages * Cfg::kTileBytes;

  if (tid == 0) {
    sh.abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sh.q_full[i]), 1);
      mbar_init(smem_u32(&sh.s_full[i]), 1);
      mbar_init(smem_u32(&sh.s_free[i]), kBlockM);
      mbar_init(smem_u32(&sh.p_full[i]), kBlockM);
      mbar_init(smem_u32(&sh.o_full[i]), 1);
    }
    for (int i = 0; i < 3; ++i) {
      mbar_init(smem_u32(&sh.k_full[i]), 1);
      mbar_init(smem_u32(&sh.k_empty[i]), 1);
      mbar_init(smem_u32(&sh.v_full[i]), 1);
      mbar_init(smem_u32(&sh.v_empty[i]), 1);
    }
    fence_mbar_init();
  }
  if (warp == 8) tmem_alloc(smem_u32(&sh.tmem_base), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh.tmem_base;
  volatile int* abort_flag = &sh.abort_flag;

  if (warp >= 8) reg_dealloc<56>();
  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      for (int g = 0; g < 2; ++g) {
        if (n_tiles[g] > 0) {
          const uint32_t bar = smem_u32(&sh.q_full[g]);
          mbar_expect_tx(bar, Cfg::kTileBytes);
          for (int p = 0; p < Cfg::kPanels; ++p)
            tma_load_3d(smem_q + g * Cfg::kTileBytes + p * 16384, &tm_q, bar, p * 64,
                        q_start + m0[g], h);
        }
      }
      bool ok = true;
      for (int j = 0; j < n_max && ok; ++j) {
        const int s = j % Cfg::kStages;
        const uint32_t ph = ((j / Cfg::kStages) & 1) ^ 1;
        if (j >= Cfg::kStages) ok = mbar_wait(smem_u32(&sh.k_empty[s]), ph, abort_flag);
        if (!ok) break;
        {
          const uint32_t bar = smem_u32(&sh.k_full[s]);
          mbar_expect_tx(bar, Cfg::kTileBytes);
          for (int p = 0; p < Cfg::kPanels; ++p)
            tma_load_3d(smem_k + s * Cfg::kTileBytes + p * 16384, &tm_k, bar, p * 64,
                        k_start + kv_tile(j) * kBlockN, h);
        }
        if (j >= Cfg::kStages) ok = mbar_wait(smem_u32(&sh.v_empty[s]), ph, abort_flag);
        if (!ok) break;
        {
          const uint32_t bar = smem_u32(&sh.v_full[s]);
          mbar_expect_tx(bar, Cfg::kTileBytes);
          for (int p = 0; p < Cfg::kPanels; ++p)
            tma_load_3d(smem_v + s * Cfg::kTileBytes + p * 16384, &tm_v, bar, p * 64,
                        k_start + kv_tile(j) * kBlockN, h);
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(BF16, false, false, kBlockM, kBlockN);
      constexpr uint32_t idesc_pv = make_idesc(BF16, false, true, kBlockM, D);
      const uint32_t tS[2] = {tmem + Cfg::kTmemS0, tmem + Cfg::kTmemS1};
      const uint32_t tO[2] = {tmem + Cfg::kTmemO0, tmem + Cfg::kTmemO1};
      const uint32_t tP[2] = {tmem + Cfg::kTmemP0, tmem + Cfg::kTmemP1};
      auto issue_qk = [&](int g, int stage) {
        const uint32_t qa = smem_q + g * Cfg::kTileBytes;
        const uint32_t ka = smem_k + stage * Cfg::kTileBytes;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
          mma_ss(tS[g], make_smem_desc(qa + off, 16, 1024), make_smem_desc(ka + off, 16, 1024),
                 idesc_qk, ks > 0);
        }
        mma_commit(smem_u32(&sh.s_full[g]));
      };
      auto issue_pv = [&](int g, int stage, bool accumulate) {
        const uint32_t va = smem_v + stage * Cfg::kTileBytes;
#pragma unroll
        for (int ks = 0; ks < kBlockN / 16; ++ks) {
          mma_ts(tO[g], tP[g] + ks * 8, make_smem_desc(va + ks * 2048, 16384, 1024), idesc_pv,
                 accumulate || ks > 0);
        }
        mma_commit(smem_u32(&sh.o_full[g]));
      };

      bool ok = true;
      for (int g = 0; g < 2 && ok; ++g)
        if (n_tiles[g] > 0) ok = mbar_wait(smem_u32(&sh.q_full[g]), 0, abort_flag);
      if (ok && n_max > 0) {
        ok = mbar_wait(smem_u32(&sh.k_full[0]), 0, abort_flag);
        if (ok) {
          tc_fence_after();
          for (int g = 0; g < 2; ++g)
            if (n_tiles[g] > 0) issue_qk(g, 0);
          mma_commit(smem_u32(&sh.k_empty[0]));
        }
      }
      FA_PROF_DECL
      for (int j = 0; j < n_max && ok; ++j) {
        const int s = j % Cfg::kStages;
        const int sn = (j + 1) % Cfg::kStages;
        const bool has_next = j + 1 < n_max;
        FA_PROF(0)
        if (!Cfg::kSeparateP) ok = mbar_wait(smem_u32(&sh.v_full[s]), (j / Cfg::kStages) & 1, abort_flag);
        if (ok && has_next)
          ok = mbar_wait(smem_u32(&sh.k_full[sn]), ((j + 1) / Cfg::kStages) & 1, abort_flag);
        if (!ok) break;
        FA_PROF(1)
        if constexpr (Cfg::kSeparateP) {
          // this warp issues only the score products; warp 10 issues P*V
          for (int g = 0; g < 2; ++g) {
            if (j + 1 < n_tiles[g]) {
              ok = mbar_wait(smem_u32(&sh.s_free[g]), j & 1, abort_flag);
              if (!ok) break;
              tc_fence_after();
              FA_STAMP(j, 16 + g * 2)
              issue_qk(g, sn);
              FA_STAMP(j, 17 + g * 2)
            }
          }
          if (!ok) break;
          FA_PROF(5)
        } else {
          for (int g = 0; g < 2; ++g) {
            if (j < n_tiles[g]) {
              ok = mbar_wait(smem_u32(&sh.p_full[g]), j & 1, abort_flag);
              if (!ok) break;
              FA_PROF(2 + g)
              tc_fence_after();
              issue_pv(g, s, j > 0);
              FA_PROF(4)
              if (j + 1 < n_tiles[g]) issue_qk(g, sn);
              FA_PROF(5)
            }
          }
        }
        if (!ok) break;
        if (!Cfg::kSeparateP) mma_commit(smem_u32(&sh.v_empty[s]));
        if (has_next) mma_commit(smem_u32(&sh.k_empty[sn]));
      }
      FA_PROF_FLUSH(16, n_max)
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------------ second MMA issuer (d = 64): P*V
    if (Cfg::kSeparateP && lane == 0) {
      constexpr uint32_t idesc_pv = make_idesc(BF16, false, true, kBlockM, D);
      const uint32_t tO[2] = {tmem + Cfg::kTmemO0, tmem + Cfg::kTmemO1};
      const uint32_t tP[2] = {tmem + Cfg::kTmemP0, tmem + Cfg::kTmemP1};
      bool ok = true;
      for (int j = 0; j < n_max && ok; ++j) {
        const int s = j % Cfg::kStages;
        ok = mbar_wait(smem_u32(&sh.v_full[s]), (j / Cfg::kStages) & 1, abort_flag);
        if (!ok) break;
        for (int g = 0; g < 2; ++g) {
          if (j < n_tiles[g]) {
            ok = mbar_wait(smem_u32(&sh.p_full[g]), j & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            FA_STAMP(j, 20 + g * 2)
            const uint32_t va = smem_v + s * Cfg::kTileBytes;
#pragma unroll
            for (int ks = 0; ks < kBlockN / 16; ++ks)
              mma_ts(tO[g], tP[g] + ks * 8, make_smem_desc(va + ks * 2048, 16384, 1024), idesc_pv,
                     j > 0 || ks > 0);
            mma_commit(smem_u32(&sh.o_full[g]));
            FA_STAMP(j, 21 + g * 2)
          }
        }
        if (!ok) break;
        mma_commit(smem_u32(&sh.v_empty[s]));
      }
    }
  } else if (warp < 8 && DROPOUT) {
    // ------------------------------------------------------------------ softmax groups, dropout
    // Quad layout: a warp reads its 32 rows as two 16-row blocks (hh) with the 16x256b shape, so a
    // thread holds rows r8 and r8 + 8 of each block and, of every 8-column unit, two adjacent columns.
    // That is the ownership pattern of the reference's mask generator: one Philox call covers exactly
    // one thread's part of a 16 x 16 patch (QuadPhilox).  Row statistics are reduced over the four
    // lanes of a quad.  Row index ri = hh * 2 + u for row r8 + 16 * hh + 8 * u of the warp.
    reg_alloc<224>();
    const int g = warp >> 2;
    const int wq = warp & 3;
    const int r8 = lane >> 2, q4 = lane & 3;
    const int row_base = m0[g] + wq * 32 + r8;  // + 16 * hh + 8 * u: query index within the sequence
    const uint32_t lane_sel = static_cast<uint32_t>(wq * 32) << 16;
    constexpr uint32_t kHalf = 16u << 16;  // second 16-row block of the warp
    const uint32_t tS = tmem + (g == 0 ? Cfg::kTmemS0 : Cfg::kTmemS1) + lane_sel;
    const uint32_t tO = tmem + (g == 0 ? Cfg::kTmemO0 : Cfg::kTmemO1) + lane_sel;
    const uint32_t tP = tmem + (g == 0 ? Cfg::kTmemP0 : Cfg::kTmemP1) + lane_sel;
    const int n = n_tiles[g];
    const bool active = m0[g] < sq;

    float m_run[4], l_run[4];  // l_run: this thread's share of the row sum (its 32 columns per tile)
#pragma unroll
    for (int ri = 0; ri < 4; ++ri) { m_run[ri] = -INFINITY; l_run[ri] = 0.f; }
    bool ok = true;
    const uint64_t c2 = pack_f2(a.scale_log2, a.scale_log2);

    const int64_t bh_sub =
        (static_cast<int64_t>(b) * a.drop.heads_total + a.drop.head_offset + h) * 256;
    const int L16 = (sq + 15) >> 4;
    const int i16_base = (m0[g] + wq * 32) >> 4;  // 16-row block index of hh = 0
    QuadPhilox<8> qp;
    qp.init(a.drop, bh_sub, lane);
    const float thr_term = fa_keep_thr_term(a.drop.threshold);

    for (int j = 0; j < n && ok; ++j) {
      const int col0 = kv_tile(j) * kBlockN;
      int32_t bs_it[2] = {0, 0};
      if constexpr (BLOCKSPARSE) {
        const int kb = col0 >> 8;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
          bs_it[hh] = (i16_base + hh) < a.bs_rows16
                          ? a.bs_iter[(static_cast<int64_t>(b) * a.bs_kblocks + kb) * a.bs_rows16 + i16_base + hh]
                          : -1;
      }
      bool need_mask = (col0 + kBlockN > sk);
      if (CAUSAL) need_mask = need_mask || (col0 + kBlockN - 1 > m0[g]);
      float alpha[4];
      bool grow_any = false;
      // pk[hh][2 * unit + u]: the 16x128b register of (row u, packed column pair 4 * unit + q4)
      uint32_t pk[2][32];
      // The two 16-row blocks of the warp one after the other (their rows are independent), which
      // keeps the live registers at one block of keep words, scores and packed probabilities.
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        // Keep words of the block: 8 calls (one per 16-column group), rounds interleaved so that their
        // multiply chains overlap.  kw[grp][2 * u + half]: row u, columns 16 grp + 8 half + 2 q4 (+1 in
        // the high 16 bits).  One iteration index per tile: a 128-column tile lies inside one key block.
        uint32_t kw[8][4];
        {
          int64_t it_index;
          if constexpr (BLOCKSPARSE) it_index = bs_it[hh];
          else it_index = fa_iter_index(CAUSAL, col0 >> a.drop.n_shift, i16_base + hh, L16, a.drop.n_shift);
          qp.set_tile(a.drop, it_index, col0);
#pragma unroll
          for (int grp = 0; grp < 8; ++grp) qp.start(grp, kw[grp]);
#pragma unroll
          for (int r = 2; r < 7; ++r)
#pragma unroll
            for (int k = 0; k < 8; ++k) QuadPhilox<8>::round(a.drop, kw[k], r);
        }
        if (hh == 0) {
          ok = mbar_wait(smem_u32(&sh.s_full[g]), j & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
        }
        // sr[4 * unit + 2 * u + c]: row u of the block, column 8 * unit + 2 * q4 + c of the tile
        uint32_t sr[64];
        tmem_ld_quad64(tS + hh * kHalf, sr);
        tmem_wait_ld();
        if constexpr (Cfg::kSeparateP) {
          if (hh == 1) {
            tc_fence_before();
            mbar_arrive(smem_u32(&sh.s_free[g]));
          }
        }
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const int col = col0 + (i >> 2) * 8 + 2 * q4 + (i & 1);
            const int ig = row_base + hh * 16 + ((i >> 1) & 1) * 8;
            bool valid = col < sk;
            if (CAUSAL) valid = valid && (col <= ig);
            if (!valid) sr[i] = __float_as_uint(-INFINITY);
          }
        }
        if constexpr (BLOCKSPARSE) {
          // a 16-row block that is not in the layout for this 256-column key block sees -inf
          if (bs_it[hh] < 0) {
#pragma unroll
            for (int i = 0; i < 64; ++i) sr[i] = __float_as_uint(-INFINITY);
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int ri = hh * 2 + u;
          // row maximum: 32 own columns, then the quad
          float mxa = -INFINITY, mxb = -INFINITY;
#pragma unroll
          for (int unit = 0; unit < 16; unit += 2) {
            mxa = max3(mxa, __uint_as_float(sr[4 * unit + 2 * u]), __uint_as_float(sr[4 * unit + 2 * u + 1]));
            mxb = max3(mxb, __uint_as_float(sr[4 * unit + 4 + 2 * u]), __uint_as_float(sr[4 * unit + 5 + 2 * u]));
          }
          float mx = fmaxf(mxa, mxb);
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
          const float m_new = fmaxf(m_run[ri], mx);
          // The running max is only raised when it would grow by more than 2^8 in the exponent:
          // until then the stale max keeps every p below 256 and saves rescaling O.
          const bool grow = (m_new - m_run[ri]) * a.scale_log2 > 8.f;
          const float m_next = grow ? m_new : m_run[ri];
          alpha[ri] = (!grow || m_run[ri] == -INFINITY) ? (grow ? 0.f : 1.f)
                                                        : ex2f((m_run[ri] - m_new) * a.scale_log2);
          m_run[ri] = m_next;
          const float mc = (m_next == -INFINITY) ? 0.f : m_next * a.scale_log2;
          grow_any = grow_any || grow;

          // p = exp2(s * c - m * c): packed fma, one ex2 per element, packed row sum; the row sum
          // takes the un-dropped p, P*V takes p times the keep factor (1 or 0), rounded to 16 bits
          const uint64_t nmc2 = pack_f2(-mc, -mc);
          uint64_t sum_a = 0ull, sum_b = 0ull;
#pragma unroll
          for (int unit = 0; unit < 16; unit += 2) {
            float p0, p1, p2, p3;
            unpack_f2(fma2(pack_f2(__uint_as_float(sr[4 * unit + 2 * u]), __uint_as_float(sr[4 * unit + 2 * u + 1])), c2, nmc2), p0, p1);
            unpack_f2(fma2(pack_f2(__uint_as_float(sr[4 * unit + 4 + 2 * u]), __uint_as_float(sr[4 * unit + 5 + 2 * u])), c2, nmc2), p2, p3);
            p0 = ex2f(p0); p1 = ex2f(p1); p2 = ex2f(p2); p3 = ex2f(p3);
            const uint64_t p01 = pack_f2(p0, p1), p23 = pack_f2(p2, p3);
            sum_a = add2(sum_a, p01);
            sum_b = add2(sum_b, p23);
            const uint32_t w01 = kw[unit / 2][2 * u], w23 = kw[unit / 2][2 * u + 1];
            unpack_f2(mul2(p01, pack_f2(fa_keep_factor_lo(w01, thr_term), fa_keep_factor_hi(w01, thr_term))), p0, p1);
            unpack_f2(mul2(p23, pack_f2(fa_keep_factor_lo(w23, thr_term), fa_keep_factor_hi(w23, thr_term))), p2, p3);
            pk[hh][2 * unit + u] = pack_lowp<BF16>(p0, p1);
            pk[hh][2 * unit + 2 + u] = pack_lowp<BF16>(p2, p3);
          }
          float s0, s1;
          unpack_f2(add2(sum_a, sum_b), s0, s1);
          l_run[ri] = l_run[ri] * alpha[ri] + (s0 + s1);
        }
      }
      if (!ok) break;

      // P*V of the previous tile must have finished before O is rescaled or its P buffer reused
      if (j > 0) {
        ok = mbar_wait(smem_u32(&sh.o_full[g]), (j - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, grow_any)) {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const uint64_t al0 = pack_f2(alpha[hh * 2], alpha[hh * 2]);
            const uint64_t al1 = pack_f2(alpha[hh * 2 + 1], alpha[hh * 2 + 1]);
#pragma unroll
            for (int c = 0; c < D / 64; ++c) {
              uint32_t orr[32];
              tmem_ld_quad32(tO + hh * kHalf + c * 64, orr);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                float lo, hi;
                unpack_f2(mul2(pack_f2(__uint_as_float(orr[i]), __uint_as_float(orr[i + 1])), (i & 2) ? al1 : al0), lo, hi);
                orr[i] = __float_as_uint(lo);
                orr[i + 1] = __float_as_uint(hi);
              }
              tmem_st_quad32(tO + hh * kHalf + c * 64, orr);
            }
          }
        }
      }
      // hand P to the tensor core through tensor memory
      tmem_st_pair32(tP, pk[0]);
      tmem_st_pair32(tP + kHalf, pk[1]);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(smem_u32(&sh.p_full[g]));
    }

    // ---------------- epilogue: O = acc / (sum * p_keep), LSE, one thread per query row again
    if (active) {
      if (n > 0 && ok) {
        ok = mbar_wait(smem_u32(&sh.o_full[g]), (n - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
      }
      // row lane (0..31 of the warp) = 16 * hh + 8 * u + r8: its statistics sit in the quad r8 under ri = lane / 8
      float m_row = -INFINITY, l_row = 0.f;
#pragma unroll
      for (int ri = 0; ri < 4; ++ri) {
        float l = l_run[ri];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const float l_src = __shfl_sync(0xffffffffu, l, (lane & 7) * 4);
        const float m_src = __shfl_sync(0xffffffffu, m_run[ri], (lane & 7) * 4);
        if ((lane >> 3) == ri) { l_row = l_src; m_row = m_src; }
      }
      store_rows<D, BF16>(a, tO, n > 0 && ok, ok, m0[g] + wq * 32 + lane, sq, q_start, b, h, m_row, l_row);
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ softmax groups, no dropout
    reg_alloc<224>();
    const int g = warp >> 2;
    const int row = tid & 127;
    const int ig = m0[g] + row;  // query index within the sequence
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + (g == 0 ? Cfg::kTmemS0 : Cfg::kTmemS1) + lane_sel;
    const uint32_t tO = tmem + (g == 0 ? Cfg::kTmemO0 : Cfg::kTmemO1) + lane_sel;
    const uint32_t tP = tmem + (g == 0 ? Cfg::kTmemP0 : Cfg::kTmemP1) + lane_sel;
    const int n = n_tiles[g];
    const bool active = m0[g] < sq;

    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    const uint64_t c2 = pack_f2(a.scale_log2, a.scale_log2);

#ifdef FA_FWD_OFFSET
    // experiment: start query tile 1 half a tile period behind query tile 0
    if (g == 1) {
      const long long t_start = clock64();
      while (clock64() - t_start < FA_FWD_OFFSET) {}
    }
#endif
    FA_PROF_DECL
    for (int j = 0; j < n && ok; ++j) {
      const int col0 = kv_tile(j) * kBlockN;
      int32_t bs_it = 0;
      if constexpr (BLOCKSPARSE) {
        const int kb = col0 >> 8;
        bs_it = (ig >> 4) < a.bs_rows16
                    ? a.bs_iter[(static_cast<int64_t>(b) * a.bs_kblocks + kb) * a.bs_rows16 + (ig >> 4)]
                    : -1;
      }
      FA_PROF(0)
      if (row == 0) { FA_STAMP(j, g * 8 + 0) }
      ok = mbar_wait(smem_u32(&sh.s_full[g]), j & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      FA_PROF(1)
      if (row == 0) { FA_STAMP(j, g * 8 + 1) }
      tc_fence_after();
      uint32_t sr[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, sr[c]);
      tmem_wait_ld();
      if constexpr (Cfg::kSeparateP) {
        tc_fence_before();
        mbar_arrive(smem_u32(&sh.s_free[g]));
      }
      FA_PROF(2)
      if (row == 0) { FA_STAMP(j, g * 8 + 2) }

      bool need_mask = (col0 + kBlockN > sk);
      if (CAUSAL) need_mask = need_mask || (col0 + kBlockN - 1 > m0[g]);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = col0 + c * 32 + i;
            bool valid = col < sk;
            if (CAUSAL) valid = valid && (col <= ig);
            if (!valid) sr[c][i] = __float_as_uint(-INFINITY);
          }
      }
      if constexpr (BLOCKSPARSE) {
        // a 16-row block that is not in the layout for this 256-column key block sees -inf
        if (bs_it < 0) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) sr[c][i] = __float_as_uint(-INFINITY);
        }
      }

      float mxa = -INFINITY, mxb = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          mxa = max3(mxa, __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
          mxb = max3(mxb, __uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3]));
        }
      const float m_new = max3(m_run, mxa, mxb);
      FA_PROF(3)
      if (row == 0) { FA_STAMP(j, g * 8 + 3) }

      // The running max is only raised when it would grow by more than 2^8 in the exponent:
      // until then the stale max keeps every p below 256 and saves rescaling O.
      const bool grow = (m_new - m_run) * a.scale_log2 > 8.f;
      const float m_next = grow ? m_new : m_run;
      const float alpha = (!grow || m_run == -INFINITY) ? (grow ? 0.f : 1.f) : ex2f((m_run - m_new) * a.scale_log2);
      m_run = m_next;
      FA_PROF(4)
      const float mc = (m_next == -INFINITY) ? 0.f : m_next * a.scale_log2;
      const uint64_t nmc2 = pack_f2(-mc, -mc);

      // p = exp2(s * c - m * c): packed fma, one ex2 per element, packed row sum, 16-bit pack
      uint32_t pk[64];
      uint64_t sum_a = 0ull, sum_b = 0ull;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float p0, p1, p2, p3;
          unpack_f2(fma2(pack_f2(__uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1])), c2, nmc2), p0, p1);
          unpack_f2(fma2(pack_f2(__uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3])), c2, nmc2), p2, p3);
          p0 = ex2f(p0); p1 = ex2f(p1); p2 = ex2f(p2); p3 = ex2f(p3);
          const uint64_t p01 = pack_f2(p0, p1), p23 = pack_f2(p2, p3);
          sum_a = add2(sum_a, p01);
          sum_b = add2(sum_b, p23);
          pk[c * 16 + i / 2] = pack_lowp<BF16>(p0, p1);
          pk[c * 16 + i / 2 + 1] = pack_lowp<BF16>(p2, p3);
        }
      {
        float s0, s1;
        unpack_f2(add2(sum_a, sum_b), s0, s1);
        l_run = l_run * alpha + (s0 + s1);
      }

      FA_PROF(5)
      if (row == 0) { FA_STAMP(j, g * 8 + 4) }
      // P*V of the previous tile must have finished before O is rescaled or its P buffer reused
      if (j > 0) {
        ok = mbar_wait(smem_u32(&sh.o_full[g]), (j - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (row == 0) { FA_STAMP(j, g * 8 + 5) }
        tc_fence_after();
        if (__any_sync(0xffffffffu, grow)) {
          const uint64_t alpha2 = pack_f2(alpha, alpha);
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t orr[32];
            tmem_ld32(tO + c * 32, orr);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float lo, hi;
              unpack_f2(mul2(pack_f2(__uint_as_float(orr[i]), __uint_as_float(orr[i + 1])), alpha2), lo, hi);
              orr[i] = __float_as_uint(lo);
              orr[i + 1] = __float_as_uint(hi);
            }
            tmem_st32(tO + c * 32, orr);
          }
        }
      }
      // hand P to the tensor core through tensor memory
      tmem_st32(tP, reinterpret_cast<uint32_t(&)[32]>(pk[0]));
      tmem_st32(tP + 32, reinterpret_cast<uint32_t(&)[32]>(pk[32]));
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(smem_u32(&sh.p_full[g]));
      FA_PROF(7)
      if (row == 0) { FA_STAMP(j, g * 8 + 6) }
    }
    if (g == 0 && row == 0) { FA_PROF_FLUSH(8, n) }

    // ---------------- epilogue: O = acc / (sum * p_keep), LSE
    if (active) {
      if (n > 0 && ok) {
        ok = mbar_wait(smem_u32(&sh.o_full[g]), (n - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
      }
      store_rows<D, BF16>(a, tO, n > 0 && ok, ok, ig, sq, q_start, b, h, m_run, l_run);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tmem_dealloc(tmem, 512);
    if (lane == 0 && sh.abort_flag && a.status) {
      atomicExch(a.status, a.launch_id);  // stops the CTAs of this launch that have not started yet
      atomicExch(a.status + 2, 1);  // sticky: read by the host
    }
  }
}

template <int D, bool BF16, bool CAUSAL, bool DROPOUT, bool BS>
cudaError_t launch_one(const FwdLaunch& l, cudaStream_t stream) {
  auto kernel = fa_fwd_kernel<D, BF16, CAUSAL, DROPOUT, BS>;
  constexpr int smem = FwdCfg<D>::kSmemBytes;
  static SmemLimitFlags smem_limit_set;  // one per template instantiation of this function
  cudaError_t e = set_smem_limit_once(kernel, smem, smem_limit_set);
  if (e != cudaSuccess) return e;
  dim3 grid((l.max_seqlen_q + 2 * kBlockM - 1) / (2 * kBlockM), l.args.heads, l.args.batch);
  kernel<<<grid, kFwdThreads, smem, stream>>>(l.tm_q, l.tm_k, l.tm_v, l.args);
  return cudaGetLastError();
}

template <int D, bool BF16, bool CAUSAL>
cudaError_t launch_dd(const FwdLaunch& l, cudaStream_t stream) {
  return l.is_dropout ? launch_one<D, BF16, CAUSAL, true, false>(l, stream)
                      : launch_one<D, BF16, CAUSAL, false, false>(l, stream);
}

template <int D>
cudaError_t launch_d(const FwdLaunch& l, cudaStream_t stream) {
  if (l.is_bf16) {
    return l.is_causal ? launch_dd<D, true, true>(l, stream) : launch_dd<D, true, false>(l, stream);
  }
  return l.is_causal ? launch_dd<D, false, true>(l, stream) : launch_dd<D, false, false>(l, stream);
}

}  // namespace

cudaError_t launch_fwd(const FwdLaunch& l, cudaStream_t stream) {
  if (l.args.bs_iter != nullptr) {
    // block-sparse exists for fp16 and head_dim <= 64 (checked by the C ABI)
    if (l.is_causal)
      return l.is_dropout ? launch_one<64, false, true, true, true>(l, stream)
                          : launch_one<64, false, true, false, true>(l, stream);
    return l.is_dropout ? launch_one<64, false, false, true, true>(l, stream)
                        : launch_one<64, false, false, false, true>(l, stream);
  }
  return l.dpad == 64 ? launch_d<64>(l, stream) : launch_d<128>(l, stream);
}

}  // namespace fa
