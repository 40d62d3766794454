// Memory-bound helpers around the attention kernels.
//
// Row gather / scatter for the padding helpers (unpad_input / pad_input): the packed layout the
// attention kernels take is built by gathering the valid token rows of a padded (batch * seqlen,
// dim) tensor, and undone by scattering them back over zeros (flash_attn/bert_padding.py:9-95 in
// the reference, which leaves both to framework indexing).  HBM-bound copies: every byte is read
// once and written once with 16-byte accesses; rows are contiguous, so a warp moves 512 bytes per
// instruction.
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
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

// ------------------------------------------------------------------------------------------------
// Rotary position embedding applied to the q and k parts of a packed (rows, 3, heads, d) qkv tensor
// in one pass (v is copied): channel pairs (2i, 2i+1) of token position p are rotated by the angle
// whose cosine / sine are cos[p][i], sin[p][i] (fp32 tables, d / 2 entries per position).  The
// reference does this with framework elementwise ops on q and k followed by a re-stack of q, k, v
// (flash_attn/rotary.py:33-43, flash_attn/flash_attention.py:102-105).  HBM bound: qkv is read
// once and written once, 16 bytes (four pairs) per thread.  conj = rotate by the negative angle
// (the gradient of the rotation).
namespace fa {
namespace {

template <bool BF16>
__device__ __forceinline__ void rotate8(const uint4& in, const float4& c, const float4& s, uint4& out) {
  const uint32_t w[4] = {in.x, in.y, in.z, in.w};
  const float cs[4] = {c.x, c.y, c.z, c.w}, sn[4] = {s.x, s.y, s.z, s.w};
  uint32_t r[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float a, b;
    if constexpr (BF16) {
      a = __uint_as_float(w[j] << 16);
      b = __uint_as_float(w[j] & 0xffff0000u);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
      a = __low2float(h);
      b = __high2float(h);
    }
    const float ra = a * cs[j] - b * sn[j];
    const float rb = b * cs[j] + a * sn[j];
    if constexpr (BF16) {
      __nv_bfloat162 v = __floats2bfloat162_rn(ra, rb);
      r[j] = *reinterpret_cast<uint32_t*>(&v);
    } else {
      __half2 v = __floats2half2_rn(ra, rb);
      r[j] = *reinterpret_cast<uint32_t*>(&v);
    }
  }
  out = make_uint4(r[0], r[1], r[2], r[3]);
}

template <bool BF16>
__global__ void __launch_bounds__(256)
rotary_qkv_kernel(const uint4* __restrict__ qkv, uint4* __restrict__ out, const float* __restrict__ cos_t,
                  const float* __restrict__ sin_t, int64_t n_vec, int seqlen, int heads, int d, float sin_sign) {
  const int vec_per_head = d / 8;
  const int vec_per_part = heads * vec_per_head;   // one of q / k / v of one token
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t tok_part = i / vec_per_part;      // token * 3 + part
    const int part = static_cast<int>(tok_part % 3);
    uint4 v = __ldg(qkv + i);
    if (part < 2) {
      const int pos = static_cast<int>((tok_part / 3) % seqlen);
      const int pair0 = static_cast<int>(i % vec_per_head) * 4;   // first of the four channel pairs
      const float4 c = __ldg(reinterpret_cast<const float4*>(cos_t + static_cast<int64_t>(pos) * (d / 2) + pair0));
      float4 s = __ldg(reinterpret_cast<const float4*>(sin_t + static_cast<int64_t>(pos) * (d / 2) + pair0));
      s.x *= sin_sign; s.y *= sin_sign; s.z *= sin_sign; s.w *= sin_sign;
      uint4 r;
      rotate8<BF16>(v, c, s, r);
      v = r;
    }
    out[i] = v;
  }
}

}  // namespace

cudaError_t launch_rotary_qkv(const void* qkv, void* out, const float* cos_t, const float* sin_t,
                              int64_t rows, int seqlen, int heads, int d, bool bf16, bool conj,
                              cudaStream_t stream) {
  const int64_t n_vec = rows * 3 * heads * (d / 8);
  if (n_vec <= 0) return cudaSuccess;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t want = (n_vec + 255) / 256;
  const int grid = static_cast<int>(want < static_cast<int64_t>(sms) * 16 ? want : static_cast<int64_t>(sms) * 16);
  const float sign = conj ? -1.f : 1.f;
  if (bf16)
    rotary_qkv_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint4*>(qkv), static_cast<uint4*>(out),
                                                      cos_t, sin_t, n_vec, seqlen, heads, d, sign);
  else
    rotary_qkv_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint4*>(qkv), static_cast<uint4*>(out),
                                                       cos_t, sin_t, n_vec, seqlen, heads, d, sign);
  return cudaGetLastError();
}

}  // namespace fa
