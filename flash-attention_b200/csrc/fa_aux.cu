// Small helper kernels: dropout-mask dump (test hook), block-sparse iteration table.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
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

// return_softmax output (test aid): s[b, h, i, j] = softmax probability of key j for query i,
// recomputed from q, k and the saved LSE on the CUDA cores, with the sign bit set where dropout
// dropped the entry.  The reference stores un-normalised values in its MMA fragment order
// (csrc/flash_attn/src/fmha/gmem_tile.h:289-405); this writes the documented (batch, heads,
// seqlen_q, seqlen_k) layout with normalised values.  One thread per (query, 16-key group).
template <bool BF16>
__global__ void sdmask_kernel(void* s_out, int64_t s_rows, int64_t s_cols, const void* q, const void* k,
                              int64_t q_row_stride, int64_t q_head_stride, int64_t k_row_stride,
                              int64_t k_head_stride, const KernelArgs a, bool causal, bool dropout) {
  const int b = blockIdx.z, h = blockIdx.y;
  const int q_start = a.cu_seqlens_q[b], sq = a.cu_seqlens_q[b + 1] - q_start;
  const int k_start = a.cu_seqlens_k[b], sk = a.cu_seqlens_k[b + 1] - k_start;
  const int groups = (sk + 15) / 16;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(sq) * groups) return;
  const int i = static_cast<int>(idx / groups);
  const int jg0 = static_cast<int>(idx % groups) * 16;
  const int d = a.head_dim;
  const uint16_t* qrow = reinterpret_cast<const uint16_t*>(q) + (q_start + i) * q_row_stride + h * q_head_stride;
  const float lse = a.lse[(static_cast<int64_t>(b) * a.heads + h) * a.lse_stride + i];
  int64_t it = 0;
  bool in_layout = true;
  if (a.bs_iter) {
    it = (i >> 4) < a.bs_rows16
             ? a.bs_iter[(static_cast<int64_t>(b) * a.bs_kblocks + (jg0 >> 8)) * a.bs_rows16 + (i >> 4)] : -1;
    in_layout = it >= 0;
  } else {
    it = fa_iter_index(causal, jg0 >> a.drop.n_shift, i >> 4, (sq + 15) >> 4, a.drop.n_shift);
  }
  uint32_t keep = 0xffffu;
  if (dropout) {
    const int64_t bh_sub = (static_cast<int64_t>(b) * a.drop.heads_total + a.drop.head_offset + h) * 256;
    keep = fa_dropout_keep16(a.drop, bh_sub, i, jg0, it < 0 ? 0 : it);
  }
  uint16_t* out = reinterpret_cast<uint16_t*>(s_out) + ((static_cast<int64_t>(b) * a.heads + h) * s_rows + i) * s_cols;
  for (int o = 0; o < 16 && jg0 + o < sk; ++o) {
    const int j = jg0 + o;
    const uint16_t* krow = reinterpret_cast<const uint16_t*>(k) + (k_start + j) * k_row_stride + h * k_head_stride;
    float acc = 0.f;
    for (int c = 0; c < d; ++c) {
      float qv, kv;
      if constexpr (BF16) {
        qv = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(qrow)[c]);
        kv = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(krow)[c]);
      } else {
        qv = __half2float(reinterpret_cast<const __half*>(qrow)[c]);
        kv = __half2float(reinterpret_cast<const __half*>(krow)[c]);
      }
      acc += qv * kv;
    }
    const bool visible = in_layout && (!causal || j <= i);
    float p = visible ? __expf(acc * a.scale - lse) : 0.f;
    if (!((keep >> o) & 1u)) p = -p;
    if (j < s_cols) {
      if constexpr (BF16) reinterpret_cast<__nv_bfloat16*>(out)[j] = __float2bfloat16(p);
      else reinterpret_cast<__half*>(out)[j] = __float2half(p);
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

cudaError_t launch_sdmask(void* s_out, int64_t s_rows, int64_t s_cols, const void* q, const void* k,
                          int64_t q_row_stride, int64_t q_head_stride, int64_t k_row_stride,
                          int64_t k_head_stride, const KernelArgs& a, int max_seqlen_q, int max_seqlen_k,
                          bool bf16, bool causal, bool dropout, cudaStream_t stream) {
  const int64_t n = static_cast<int64_t>(max_seqlen_q) * ((max_seqlen_k + 15) / 16);
  if (n == 0) return cudaSuccess;
  dim3 grid(static_cast<unsigned>((n + 127) / 128), a.heads, a.batch);
  if (bf16)
    sdmask_kernel<true><<<grid, 128, 0, stream>>>(s_out, s_rows, s_cols, q, k, q_row_stride, q_head_stride,
                                                  k_row_stride, k_head_stride, a, causal, dropout);
  else
    sdmask_kernel<false><<<grid, 128, 0, stream>>>(s_out, s_rows, s_cols, q, k, q_row_stride, q_head_stride,
                                                   k_row_stride, k_head_stride, a, causal, dropout);
  return cudaGetLastError();
}

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
