// Dropout mask of the reference, reproduced bit for bit.
//
// The reference draws its keep/drop decisions from a 7-round Philox4x32 generator
// (csrc/flash_attn/src/philox.cuh:7-136) whose counter and subsequence are tied to the thread and
// iteration structure of its sm80 kernels (fmha_fprop_kernel_1xN.h:653-670,
// fmha/softmax.h:375-414).  Because those are pure functions of (batch, head, row, column), any
// tiling can regenerate the same bits.  For query row i and key column j of one sequence:
//
//   N       key-block size of the reference kernel (128 or 256)
//   s       = j / N            c16 = (j % N) / 16       o = j % 16       r = i % 16
//   subsequence = (b*H + h)*256 + (c16 % 8)*32 + (r % 8)*4 + (o % 8)/2
//   counter     = offset/4 + iter_index(s, i/16) * (N/128) + c16/8
//   the 128-bit output, read as eight little-endian uint16, is indexed by
//   slot = (r/8)*4 + (o >= 8 ? 2 : 0) + (o & 1);  keep <=> u16[slot] <= floor(p_keep * 65535)
//
// iter_index counts the (key block, 16-row tile) iterations the reference CTA ran before this
// one, key-block major (see fa_iter_index below).
#pragma once
#include <cstdint>

namespace fa {

struct DropoutParams {
  uint32_t key0, key1;     // seed low / high
  uint64_t counter_base;   // offset / 4
  uint32_t threshold;      // floor(p_keep * 65535)
  int32_t n_shift;         // log2(N): 7 or 8
  int32_t heads_total;     // H used in the subsequence
  int32_t head_offset;
  uint32_t rk0[7], rk1[7]; // round keys key + r * (0x9E3779B9, 0xBB67AE85), r = 0..6 (kernel constants)
};

__host__ __device__ __forceinline__ uint64_t mul_wide_u32(uint32_t a, uint32_t b) {
#ifdef __CUDA_ARCH__
  uint64_t r;
  asm("mul.wide.u32 %0, %1, %2;" : "=l"(r) : "r"(a), "r"(b));
  return r;
#else
  return static_cast<uint64_t>(a) * b;
#endif
}

__host__ __device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint64_t p0 = mul_wide_u32(0xD2511F53u, c[0]);
  const uint64_t p1 = mul_wide_u32(0xCD9E8D57u, c[2]);
  const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c[1] ^ k0;
  const uint32_t n1 = static_cast<uint32_t>(p1);
  const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c[3] ^ k1;
  const uint32_t n3 = static_cast<uint32_t>(p0);
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

// Seven rounds: six with a key bump after each, then a final one (philox.cuh:30-42).
__host__ __device__ __forceinline__ void philox7(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int i = 0; i < 6; ++i) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  philox_round(c, k0, k1);
}

// Number of (key block, 16-row tile) iterations the reference ran before (s, i16) for a dense
// sequence with L = ceil(seqlen_q / 16) row tiles.  Non-causal: every key block walks all L row
// tiles (fmha_fprop_kernel_1xN.h:365-366).  Causal: key block s starts at row tile s*N/16
// (:270-272), so the blocks before it ran L, L-u, L-2u ... tiles with u = N/16.
__host__ __device__ __forceinline__ int64_t fa_iter_index(bool causal, int32_t s, int32_t i16,
                                                          int32_t L, int32_t n_shift) {
  if (!causal) return static_cast<int64_t>(s) * L + i16;
  const int64_t u = static_cast<int64_t>(1) << (n_shift - 4);
  return static_cast<int64_t>(s) * L - u * (static_cast<int64_t>(s) * (s - 1) / 2) + (i16 - s * u);
}

// The four keep bits of row i for columns {2q, 2q+1, 2q+8, 2q+9} of the 16-column group that
// starts at column jg0 (a multiple of 16): one Philox call.  Returned as two 32-bit words, each
// holding two uint16 random values: w0 -> columns 2q (low half) and 2q+1 (high half),
// w1 -> columns 2q+8 and 2q+9.
__host__ __device__ __forceinline__ void fa_dropout_words(const DropoutParams& dp, int64_t bh_sub,
                                                          int32_t i, int32_t jg0, int32_t q,
                                                          int64_t iter_index, uint32_t& w0,
                                                          uint32_t& w1) {
  const int32_t n_mask = (1 << dp.n_shift) - 1;
  const int32_t c16 = (jg0 & n_mask) >> 4;
  const int32_t r = i & 15;
  const uint64_t subseq = static_cast<uint64_t>(bh_sub) + (c16 & 7) * 32 + (r & 7) * 4 + q;
  const uint64_t ctr = dp.counter_base + static_cast<uint64_t>(iter_index << (dp.n_shift - 7)) +
                       static_cast<uint64_t>(c16 >> 3);
  uint32_t c[4] = {static_cast<uint32_t>(ctr), static_cast<uint32_t>(ctr >> 32),
                   static_cast<uint32_t>(subseq), static_cast<uint32_t>(subseq >> 32)};
  philox7(c, dp.key0, dp.key1);
  if (r >= 8) { w0 = c[2]; w1 = c[3]; } else { w0 = c[0]; w1 = c[1]; }
}

// 16 keep bits (bit o = column jg0 + o) for row i.
__host__ __device__ __forceinline__ uint32_t fa_dropout_keep16(const DropoutParams& dp,
                                                               int64_t bh_sub, int32_t i,
                                                               int32_t jg0, int64_t iter_index) {
  uint32_t bits = 0;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t w0, w1;
    fa_dropout_words(dp, bh_sub, i, jg0, q, iter_index, w0, w1);
    bits |= ((w0 & 0xFFFFu) <= dp.threshold ? 1u : 0u) << (2 * q);
    bits |= ((w0 >> 16) <= dp.threshold ? 1u : 0u) << (2 * q + 1);
    bits |= ((w1 & 0xFFFFu) <= dp.threshold ? 1u : 0u) << (2 * q + 8);
    bits |= ((w1 >> 16) <= dp.threshold ? 1u : 0u) << (2 * q + 9);
  }
  return bits;
}

}  // namespace fa

namespace fa {

#ifdef __CUDACC__
// ---------------------------------------------------------------------------------------------
// Row-per-thread mask generation (the layout of the attention kernels: lane = query row).
//
// Rows r and r + 8 of a 16-row block share every Philox call: output words 0, 1 belong to the row
// with (r % 16) < 8 and words 2, 3 to the row 8 below.  A lane and its partner 8 lanes away each run
// two of the four calls (quarters) of a 16-column group and exchange the half they do not need.
// So that both lanes send the same registers, the lane of the lower row runs the generator on the
// state (c0, c1, c2, c3) and the lane of the upper row on the mirrored state (c2, c3, c0, c1): one
// round maps the mirrored state to the mirror of the next state when the two multipliers and the
// two round keys trade places, which makes them per-lane registers.  Either way words 0, 1 of the
// state are the lane's own and words 2, 3 go to the partner.
struct LanePhilox {
  uint32_t mul_a, mul_b;       // multiplier of state word 0 / of state word 2
  uint32_t key_a[7], key_b[7];  // round keys folded into the new word 0 / the new word 2
  uint32_t base[4];             // state before the per-call subsequence offset is added
  uint32_t step_a, step_b;      // 1 on the state word that holds the subsequence's low word
  bool upper;                   // this lane owns the row with (r % 16) >= 8

  // i: query row of this lane.  The subsequence's low byte is (column group % 8) * 32 + (i % 8) * 4
  // + quarter; a lane runs quarters 0, 1 (lower row) or 2, 3 (upper row).
  __device__ __forceinline__ void init(const DropoutParams& dp, int64_t bh_sub, int32_t i) {
    upper = (i & 8) != 0;
    mul_a = upper ? 0xCD9E8D57u : 0xD2511F53u;
    mul_b = upper ? 0xD2511F53u : 0xCD9E8D57u;
#pragma unroll
    for (int r = 0; r < 7; ++r) {
      const uint32_t k0 = dp.key0 + static_cast<uint32_t>(r) * 0x9E3779B9u;
      const uint32_t k1 = dp.key1 + static_cast<uint32_t>(r) * 0xBB67AE85u;
      key_a[r] = upper ? k1 : k0;
      key_b[r] = upper ? k0 : k1;
    }
    const uint64_t sub = static_cast<uint64_t>(bh_sub) + (i & 7) * 4 + (upper ? 2 : 0);
    base[upper ? 0 : 2] = static_cast<uint32_t>(sub);
    base[upper ? 1 : 3] = static_cast<uint32_t>(sub >> 32);
    step_a = upper ? 1u : 0u;
    step_b = upper ? 0u : 1u;
  }
  // Counter of the calls of one 128-column tile: iteration index of (key block, 16-row block) and the
  // 128-column half of the key block the tile is (fa_dropout_words above).
  __device__ __forceinline__ void set_tile(const DropoutParams& dp, int64_t iter_index, int32_t col0) {
    const int32_t n_mask = (1 << dp.n_shift) - 1;
    const uint64_t ctr = dp.counter_base + static_cast<uint64_t>(iter_index << (dp.n_shift - 7)) +
                         static_cast<uint64_t>((col0 & n_mask) >> 7);
    base[upper ? 2 : 0] = static_cast<uint32_t>(ctr);
    base[upper ? 3 : 1] = static_cast<uint32_t>(ctr >> 32);
  }
  // State of the call for 16-column group `grp` (0..7 within the tile) and quarter offset qq (0 / 1).
  // The offset never carries: the low byte of the subsequence base is below 32.
  __device__ __forceinline__ void start(int grp, int qq, uint32_t (&s)[4]) const {
    const uint32_t off = static_cast<uint32_t>(grp * 32 + qq);
    s[0] = base[0] + off * step_a;
    s[1] = base[1];
    s[2] = base[2] + off * step_b;
    s[3] = base[3];
  }
  __device__ __forceinline__ void round(uint32_t (&s)[4], int r) const {
    const uint64_t p0 = mul_wide_u32(mul_a, s[0]);
    const uint64_t p1 = mul_wide_u32(mul_b, s[2]);
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ s[1] ^ key_a[r];
    const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ s[3] ^ key_b[r];
    s[1] = static_cast<uint32_t>(p1);
    s[3] = static_cast<uint32_t>(p0);
    s[0] = n0;
    s[2] = n2;
  }
  // After seven rounds of the calls (grp, 0) and (grp, 1): the eight keep words of the lane's row
  // for that group, wd[p] covering columns 2p, 2p + 1 (low half = even column).
  __device__ __forceinline__ void finish(const uint32_t (&sa)[4], const uint32_t (&sb)[4],
                                         uint32_t* wd) const {
    const uint32_t ra0 = __shfl_xor_sync(0xffffffffu, sa[2], 8);
    const uint32_t ra1 = __shfl_xor_sync(0xffffffffu, sa[3], 8);
    const uint32_t rb0 = __shfl_xor_sync(0xffffffffu, sb[2], 8);
    const uint32_t rb1 = __shfl_xor_sync(0xffffffffu, sb[3], 8);
    // quarter q: first word -> pair q (columns 2q, 2q+1), second word -> pair q + 4 (columns 2q+8, 2q+9)
    wd[0] = upper ? ra0 : sa[0]; wd[4] = upper ? ra1 : sa[1];
    wd[1] = upper ? rb0 : sb[0]; wd[5] = upper ? rb1 : sb[1];
    wd[2] = upper ? sa[0] : ra0; wd[6] = upper ? sa[1] : ra1;
    wd[3] = upper ? sb[0] : rb0; wd[7] = upper ? sb[1] : rb1;
  }
};

// ---------------------------------------------------------------------------------------------
// Quad-per-thread mask generation (the layout of the tcgen05.ld 16x256b shape: thread t of a warp
// working on a 16-row block holds rows t/4 and t/4 + 8 and, of every 16-column group, columns 2q,
// 2q+1, 2q+8, 2q+9 with q = t % 4).  Those eight values are the eight 16-bit outputs of ONE Philox
// call whose subsequence ends in (group % 8) * 32 + t: a thread runs whole calls, nothing is
// exchanged, and the multipliers stay immediates.
//
// Two of the fourteen wide multiplies of a call do not depend on the call.  With the state
// (c0, c1, c2, c3) = (counter low, counter high, subsequence low, subsequence high):
//   round 0   M1 * c2 depends on the subsequence only (computed once per kernel and group),
//             M0 * c0 on the counter only (once per tile);
//   round 1   its word-2 input hi(M0 * c0) ^ c3 ^ key1 is the same for every call of a tile
//             (the subsequence's high word is per (batch, head)), so M1 * that is per tile too.
// A call therefore starts at round 1 with one multiply, then runs rounds 2..6: 11 multiplies.
// NG: 16-column groups a thread covers per tile (8 = all 128 columns, 4 = one 64-column half).
template <int NG>
struct QuadPhilox {
  uint32_t a_hi[NG], b_lo[NG];  // per 16-column group: hi(M1 * sub) ^ key0[0], lo(M1 * sub)
  uint32_t sub_hi;
  // per (tile, 16-row block)
  uint32_t c1, n3k, w_hi, w_lo;

  // grp0: first 16-column group (of the 8 of a tile) this thread covers
  __device__ __forceinline__ void init(const DropoutParams& dp, int64_t bh_sub, int lane, int grp0 = 0) {
    // bh_sub is a multiple of 256 and group * 32 + lane < 256: the sum never carries
    const uint32_t sub_lo = static_cast<uint32_t>(bh_sub) + static_cast<uint32_t>(grp0 * 32 + lane);
    sub_hi = static_cast<uint32_t>(static_cast<uint64_t>(bh_sub) >> 32);
#pragma unroll
    for (int grp = 0; grp < NG; ++grp) {
      const uint64_t v = mul_wide_u32(0xCD9E8D57u, sub_lo + grp * 32);
      a_hi[grp] = static_cast<uint32_t>(v >> 32) ^ dp.rk0[0];
      b_lo[grp] = static_cast<uint32_t>(v);
    }
  }
  // Counter of the calls of one 128-column tile for one 16-row block (see fa_dropout_words).
  __device__ __forceinline__ void set_tile(const DropoutParams& dp, int64_t iter_index, int32_t col0) {
    const int32_t n_mask = (1 << dp.n_shift) - 1;
    const uint64_t ctr = dp.counter_base + static_cast<uint64_t>(iter_index << (dp.n_shift - 7)) +
                         static_cast<uint64_t>((col0 & n_mask) >> 7);
    c1 = static_cast<uint32_t>(ctr >> 32);
    const uint64_t u = mul_wide_u32(0xD2511F53u, static_cast<uint32_t>(ctr));
    const uint32_t n2 = static_cast<uint32_t>(u >> 32) ^ sub_hi ^ dp.rk1[0];
    n3k = static_cast<uint32_t>(u) ^ dp.rk1[1];
    const uint64_t w = mul_wide_u32(0xCD9E8D57u, n2);
    w_hi = static_cast<uint32_t>(w >> 32) ^ dp.rk0[1];
    w_lo = static_cast<uint32_t>(w);
  }
  // State after rounds 0 and 1 of the call for the thread's 16-column group `grp` (0 .. NG-1).
  __device__ __forceinline__ void start(int grp, uint32_t (&s)[4]) const {
    const uint64_t p = mul_wide_u32(0xD2511F53u, a_hi[grp] ^ c1);
    s[0] = w_hi ^ b_lo[grp];
    s[1] = w_lo;
    s[2] = static_cast<uint32_t>(p >> 32) ^ n3k;
    s[3] = static_cast<uint32_t>(p);
  }
  // Rounds 2..6; afterwards s[0], s[1] are the keep words of row t/4 (columns 2q, 2q+1 and 2q+8,
  // 2q+9; low half = even column) and s[2], s[3] those of row t/4 + 8.
  static __device__ __forceinline__ void round(const DropoutParams& dp, uint32_t (&s)[4], int r) {
    philox_round(s, dp.rk0[r], dp.rk1[r]);
  }
};

// Keep factors (1.0f kept / 0.0f dropped) of the two 16-bit values of a keep word, without integer
// compares: the 16 bits become the top mantissa bits of a float in [0.5, 2) (bytes 0x3F | hi | lo |
// filler, a monotone map), and a saturating fma against the threshold mapped the same way gives
// sat((T - x) * 2^24), which is exactly 1 when x < T and 0 otherwise (both are multiples of 2^-24).
//   thr_term = float(0x3F000000 + ((threshold + 1) << 8)) * 2^24
__device__ __forceinline__ float fa_keep_thr_term(uint32_t threshold) {
  return __uint_as_float(0x3F000000u + ((threshold + 1u) << 8)) * 16777216.f;
}
__device__ __forceinline__ float fa_keep_factor_lo(uint32_t w, float thr_term) {
  uint32_t f;
  float k;
  asm("prmt.b32 %0, %1, %2, 0x7104;" : "=r"(f) : "r"(w), "r"(0x3F000000u));
  asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(k) : "f"(__uint_as_float(f)), "f"(-16777216.f), "f"(thr_term));
  return k;
}
__device__ __forceinline__ float fa_keep_factor_hi(uint32_t w, float thr_term) {
  uint32_t f;
  float k;
  asm("prmt.b32 %0, %1, %2, 0x7321;" : "=r"(f) : "r"(w), "r"(0x3F000000u));
  asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(k) : "f"(__uint_as_float(f)), "f"(-16777216.f), "f"(thr_term));
  return k;
}
#endif  // __CUDACC__

}  // namespace fa
