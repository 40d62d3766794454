// Row gather / scatter for the padding helpers (unpad_input / pad_input): the packed layout the
// attention kernels take is built by gathering the valid token rows of a padded (batch * seqlen,
// dim) tensor, and undone by scattering them back over zeros (flash_attn/bert_padding.py:9-95 in
// the reference, which leaves both to framework indexing).  HBM-bound copies: every byte is read
// once and written once with 16-byte accesses; rows are contiguous, so a warp moves 512 bytes per
// instruction.
#include <cstdint>
#include "fa_kernels.h"

namespace fa {

namespace {

constexpr int kRowThreads = 256;

constexpr int kRowsPerStep = 4;  // rows a CTA moves together: four independent 16-byte loads per thread in flight

// dst[r, :] = src[indices[r], :] (zeros when the index is out of range); vec = 16-byte units per row
__global__ void __launch_bounds__(kRowThreads)
gather_rows_kernel(const uint4* __restrict__ src, const int64_t* __restrict__ indices,
                   uint4* __restrict__ dst, int64_t n_rows, int64_t src_rows, int vec) {
  for (int64_t r0 = static_cast<int64_t>(blockIdx.x) * kRowsPerStep; r0 < n_rows;
       r0 += static_cast<int64_t>(gridDim.x) * kRowsPerStep) {
    const uint4* from[kRowsPerStep];
    bool ok[kRowsPerStep];
#pragma unroll
    for (int j = 0; j < kRowsPerStep; ++j) {
      const int64_t s = (r0 + j < n_rows) ? indices[r0 + j] : -1;
      ok[j] = s >= 0 && s < src_rows;
      from[j] = src + (ok[j] ? s : 0) * vec;
    }
    for (int c = threadIdx.x; c < vec; c += kRowThreads) {
      uint4 v[kRowsPerStep];
#pragma unroll
      for (int j = 0; j < kRowsPerStep; ++j) v[j] = ok[j] ? __ldg(from[j] + c) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int j = 0; j < kRowsPerStep; ++j)
        if (r0 + j < n_rows) dst[(r0 + j) * vec + c] = v[j];
    }
  }
}

__global__ void fill_i32_kernel(int32_t* p, int64_t n, int32_t value) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) p[i] = value;
}

// inverse[indices[r]] = r
__global__ void invert_indices_kernel(const int64_t* __restrict__ indices, int32_t* inverse,
                                      int64_t n_src_rows, int64_t n_dst_rows) {
  const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r < n_src_rows) {
    const int64_t d = indices[r];
    if (d >= 0 && d < n_dst_rows) inverse[d] = static_cast<int32_t>(r);
  }
}

// one pass over the destination: a row is either copied from its source row or zero-filled
__global__ void __launch_bounds__(kRowThreads)
scatter_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ inverse,
                    uint4* __restrict__ dst, int64_t n_dst_rows, int vec) {
  for (int64_t d0 = static_cast<int64_t>(blockIdx.x) * kRowsPerStep; d0 < n_dst_rows;
       d0 += static_cast<int64_t>(gridDim.x) * kRowsPerStep) {
    const uint4* from[kRowsPerStep];
    bool ok[kRowsPerStep];
#pragma unroll
    for (int j = 0; j < kRowsPerStep; ++j) {
      const int32_t s = (d0 + j < n_dst_rows) ? inverse[d0 + j] : -1;
      ok[j] = s >= 0;
      from[j] = src + static_cast<int64_t>(ok[j] ? s : 0) * vec;
    }
    for (int c = threadIdx.x; c < vec; c += kRowThreads) {
      uint4 v[kRowsPerStep];
#pragma unroll
      for (int j = 0; j < kRowsPerStep; ++j) v[j] = ok[j] ? __ldg(from[j] + c) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int j = 0; j < kRowsPerStep; ++j)
        if (d0 + j < n_dst_rows) dst[(d0 + j) * vec + c] = v[j];
    }
  }
}

// a few CTAs per SM, rows handed out in a grid-stride loop
int row_grid(int64_t rows) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t cap = static_cast<int64_t>(sms) * 8;
  const int64_t steps = (rows + kRowsPerStep - 1) / kRowsPerStep;
  return static_cast<int>(steps < cap ? steps : cap);
}

}  // namespace

cudaError_t launch_gather_rows(const void* src, const int64_t* indices, void* dst, int64_t n_rows,
                               int64_t src_rows, int64_t row_bytes, cudaStream_t stream) {
  if (n_rows <= 0 || row_bytes <= 0) return cudaSuccess;
  gather_rows_kernel<<<row_grid(n_rows), kRowThreads, 0, stream>>>(
      static_cast<const uint4*>(src), indices, static_cast<uint4*>(dst), n_rows, src_rows,
      static_cast<int>(row_bytes / 16));
  return cudaGetLastError();
}

cudaError_t launch_scatter_rows(const void* src, const int64_t* indices, void* dst, int64_t n_src_rows,
                                int64_t n_dst_rows, int64_t row_bytes, int32_t* inverse,
                                cudaStream_t stream) {
  if (n_dst_rows <= 0 || row_bytes <= 0) return cudaSuccess;
  fill_i32_kernel<<<static_cast<unsigned>((n_dst_rows + 255) / 256), 256, 0, stream>>>(inverse, n_dst_rows, -1);
  if (n_src_rows > 0)
    invert_indices_kernel<<<static_cast<unsigned>((n_src_rows + 255) / 256), 256, 0, stream>>>(
        indices, inverse, n_src_rows, n_dst_rows);
  scatter_rows_kernel<<<row_grid(n_dst_rows), kRowThreads, 0, stream>>>(
      static_cast<const uint4*>(src), inverse, static_cast<uint4*>(dst), n_dst_rows,
      static_cast<int>(row_bytes / 16));
  return cudaGetLastError();
}

}  // namespace fa
