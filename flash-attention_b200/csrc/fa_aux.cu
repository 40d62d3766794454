// Small helper kernels: dropout-mask dump (test hook), block-sparse iteration table.
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

}  // namespace

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
