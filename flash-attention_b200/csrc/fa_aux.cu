// Small helper kernels: dropout-mask dump (test hook), block-sparse iteration table.
#include <curand_kernel.h>
#include "fa_kernels.h"

namespace fa {

namespace {

// One thread per (row, 16-column group).
__global__ void dropout_mask_kernel(uint8_t* out, int b, int h, DropoutParams dp, bool causal,
                                    int sq, int sk, const int32_t* bs_iter, int bs_kblocks,
                                    int bs_rows16) {
  const int groups = (sk + 15) / 16;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(sq) * groups) return;
  const int i = static_cast<int>(idx / groups);
  const int jg0 = static_cast<int>(idx % groups) * 16;
  const int64_t bh_sub = (static_cast<int64_t>(b) * dp.heads_total + dp.head_offset + h) * 256;
  int64_t it;
  if (bs_iter) {
    it = bs_iter[(static_cast<int64_t>(b) * bs_kblocks + (jg0 >> 8)) * bs_rows16 + (i >> 4)];
  } else {
    it = fa_iter_index(causal, jg0 >> dp.n_shift, i >> 4, (sq + 15) >> 4, dp.n_shift);
  }
  const uint32_t keep = fa_dropout_keep16(dp, bh_sub, i, jg0, it);
  for (int o = 0; o < 16 && jg0 + o < sk; ++o)
    out[static_cast<int64_t>(i) * sk + jg0 + o] = (keep >> o) & 1u;
}

// Block-sparse iteration table.  The converted block mask lists, for each 256-column key block,
// the 16-row query blocks to visit in ascending order (value = 4 * row_block + flags, -1 ends the
// list).  The reference walks key blocks in order and, inside one, the list until it ends or
// reaches a row block at or beyond the sequence's query length
// (csrc/flash_attn/src/fmha_block_fprop_kernel_1xN.h:90-100, :209, :486); key blocks at or beyond
// the key length are not visited at all (:88).  table[b][kb][rb] = number of blocks visited
// before (kb, rb), or -1 when (kb, rb) is not visited.  One CTA per batch entry.
__global__ void bs_table_kernel(int32_t* table, const int32_t* blockmask, const int32_t* cu_q,
                                const int32_t* cu_k, int nk, int nr) {
  extern __shared__ int32_t cnt[];  // nk + 1 entries
  const int b = blockIdx.x;
  const int sq = cu_q[b + 1] - cu_q[b];
  const int sk = cu_k[b + 1] - cu_k[b];
  int32_t* tb = table + static_cast<int64_t>(b) * nk * nr;
  for (int i = threadIdx.x; i < nk * nr; i += blockDim.x) tb[i] = -1;
  for (int kb = threadIdx.x; kb < nk; kb += blockDim.x) {
    int c = 0;
    if (kb * 256 < sk) {
      const int32_t* row = blockmask + static_cast<int64_t>(kb) * nr;
      while (c < nr) {
        const int32_t v = row[c];
        if (v < 0 || (v >> 2) * 16 >= sq) break;
        ++c;
      }
    }
    cnt[kb + 1] = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    cnt[0] = 0;
    for (int kb = 0; kb < nk; ++kb) cnt[kb + 1] += cnt[kb];
  }
  __syncthreads();
  for (int kb = threadIdx.x; kb < nk; kb += blockDim.x) {
    const int32_t* row = blockmask + static_cast<int64_t>(kb) * nr;
    const int n = cnt[kb + 1] - cnt[kb];
    for (int c = 0; c < n; ++c) {
      const int rb = row[c] >> 2;
      if (rb >= 0 && rb < nr) tb[static_cast<int64_t>(kb) * nr + rb] = cnt[kb] + c;
    }
  }
}

// Philox self-check: thread i writes the four output words for (seed, subsequence i, offset).
// mode 0: this library's round function run `rounds` times with the counter layout of the
// attention kernels; mode 1: cuRAND's Philox4_32_10 device generator (10 rounds) as an
// independent implementation of the same generator.
__global__ void philox_probe_kernel(uint32_t* out, int n, unsigned long long seed,
                                    unsigned long long offset, int rounds, int mode) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint32_t c[4];
  if (mode == 1) {
    curandStatePhilox4_32_10_t st;
    curand_init(seed, static_cast<unsigned long long>(i), offset, &st);
    const uint4 r = curand4(&st);
    c[0] = r.x; c[1] = r.y; c[2] = r.z; c[3] = r.w;
  } else {
    const unsigned long long ctr = offset / 4;
    c[0] = static_cast<uint32_t>(ctr);
    c[1] = static_cast<uint32_t>(ctr >> 32);
    c[2] = static_cast<uint32_t>(i);
    c[3] = 0u;
    uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
    for (int r = 0; r < rounds; ++r) {
      philox_round(c, k0, k1);
      k0 += 0x9E3779B9u;
      k1 += 0xBB67AE85u;
    }
  }
  for (int k = 0; k < 4; ++k) out[4 * i + k] = c[k];
}

}  // namespace

cudaError_t launch_philox_probe(uint32_t* out, int n, unsigned long long seed, unsigned long long offset,
                                int rounds, int mode, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  philox_probe_kernel<<<(n + 127) / 128, 128, 0, stream>>>(out, n, seed, offset, rounds, mode);
  return cudaGetLastError();
}

cudaError_t launch_bs_table(int32_t* table, const int32_t* blockmask, const int32_t* cu_q,
                            const int32_t* cu_k, int batch, int nk, int nr, cudaStream_t stream) {
  bs_table_kernel<<<batch, 256, (nk + 1) * sizeof(int32_t), stream>>>(table, blockmask, cu_q, cu_k, nk, nr);
  return cudaGetLastError();
}

cudaError_t launch_dropout_mask(uint8_t* out, int b, int h, const DropoutParams& dp, bool causal,
                                int sq, int sk, const int32_t* bs_iter, int bs_kblocks,
                                int bs_rows16, cudaStream_t stream) {
  const int64_t n = static_cast<int64_t>(sq) * ((sk + 15) / 16);
  if (n == 0) return cudaSuccess;
  const int threads = 256;
  const int blocks = static_cast<int>((n + threads - 1) / threads);
  dropout_mask_kernel<<<blocks, threads, 0, stream>>>(out, b, h, dp, causal, sq, sk, bs_iter,
                                                      bs_kblocks, bs_rows16);
  return cudaGetLastError();
}

}  // namespace fa
