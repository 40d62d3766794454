// Host-side launch interface between the C ABI (fa_api.cu) and the kernel translation units.
#pragma once
#include <atomic>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#include "fa_dropout.cuh"

namespace fa {

// Arguments shared by the forward and backward kernels (device pointers, sizes in elements).
struct KernelArgs {
  const int32_t* cu_seqlens_q;
  const int32_t* cu_seqlens_k;
  // Block-sparse: per (batch, key block of 256, 16-row block) iteration index of the reference
  // kernel, or -1 when the block is not in the layout; nullptr for dense attention.
  const int32_t* bs_iter;
  int32_t bs_rows16;   // row length of bs_iter: 16-row blocks per key block
  int32_t bs_kblocks;  // key blocks (of 256) per batch entry in bs_iter
  void* o;
  float* lse;
  int64_t o_row_stride, o_head_stride;
  int64_t lse_stride;
  int32_t batch, heads, head_dim;
  float scale;        // softmax_scale
  float scale_log2;   // softmax_scale * log2(e)
  float rp_keep;      // 1 / p_keep
  DropoutParams drop;
  int32_t* status;
  int32_t launch_id;  // non-zero serial number of this call: what an aborting CTA leaves in status[0]
};

struct BwdArgs {
  KernelArgs k;
  const void* q; const void* kk; const void* v;       // raw pointers for the plain-load paths
  const void* o_in; const void* dout;
  int64_t q_row_stride, q_head_stride;
  int64_t do_row_stride, do_head_stride;
  void* dq; void* dk; void* dv;
  int64_t dq_row_stride, dq_head_stride, dk_row_stride, dk_head_stride, dv_row_stride, dv_head_stride;
  float* softmax_d;
  float* dq_accum;    // fp32 [total_q, heads, Dpad]
  // Deterministic mode: one ticket per (batch, head, 128-row query tile) = number of key tiles
  // that have added their dQ tile so far; nullptr = add in arrival order.
  int32_t* dq_tickets;
  int32_t ticket_stride;  // tickets per (batch, head): ceil(max_seqlen_q / 128)
  int32_t total_q, total_k, max_seqlen_q, max_seqlen_k;
  float p_keep;
};

struct FwdLaunch {
  CUtensorMap tm_q, tm_k, tm_v;
  KernelArgs args;
  int32_t max_seqlen_q, max_seqlen_k;
  bool is_bf16, is_causal, is_dropout;
  int32_t dpad;  // 64 or 128
};

struct BwdLaunch {
  CUtensorMap tm_q, tm_k, tm_v, tm_do;
  CUtensorMap tm_dq;  // fp32 dQ accumulator [total_q, heads, dpad], 32-column boxes
  BwdArgs args;
  bool is_bf16, is_causal, is_dropout;
  int32_t dpad;  // 64 or 128
  int32_t stage_mask;  // 0 = all; 1 preprocess, 2 main, 4 postprocess
  bool deterministic;
};

cudaError_t launch_fwd(const FwdLaunch& l, cudaStream_t stream);
cudaError_t launch_bwd(const BwdLaunch& l, cudaStream_t stream);
cudaError_t launch_sdmask(void* s_out, int64_t s_rows, int64_t s_cols, const void* q, const void* k,
                          int64_t q_row_stride, int64_t q_head_stride, int64_t k_row_stride,
                          int64_t k_head_stride, const KernelArgs& a, int max_seqlen_q, int max_seqlen_k,
                          bool bf16, bool causal, bool dropout, cudaStream_t stream);
cudaError_t launch_philox_probe(uint32_t* out, int n, unsigned long long seed, unsigned long long offset,
                                int rounds, int mode, cudaStream_t stream);
cudaError_t launch_bs_table(int32_t* table, const int32_t* blockmask, const int32_t* cu_q,
                            const int32_t* cu_k, int batch, int nk, int nr, cudaStream_t stream);
cudaError_t launch_dropout_mask(uint8_t* out, int b, int h, const DropoutParams& dp, bool causal,
                                int sq, int sk, const int32_t* bs_iter, int bs_kblocks,
                                int bs_rows16, cudaStream_t stream);

cudaError_t launch_gather_rows(const void* src, const int64_t* indices, void* dst, int64_t n_rows,
                               int64_t src_rows, int64_t row_bytes, cudaStream_t stream);
cudaError_t launch_scatter_rows(const void* src, const int64_t* indices, void* dst, int64_t n_src_rows,
                                int64_t n_dst_rows, int64_t row_bytes, int32_t* inverse,
                                cudaStream_t stream);

cudaError_t launch_rotary_qkv(const void* qkv, void* out, const float* cos_t, const float* sin_t,
                              int64_t rows, int seqlen, int heads, int d, bool bf16, bool conj,
                              cudaStream_t stream);

// Raises the dynamic shared-memory limit of `kernel` the first time it is launched on a device
// (the attribute belongs to the device's context; setting it on every launch costs microseconds).
// `done` is the caller's per-kernel flag array, one entry per device: kernels that differ only in
// template arguments have the same function type, so the flags cannot live in this template.
constexpr int kMaxDevices = 64;
using SmemLimitFlags = std::atomic<unsigned char>[kMaxDevices];
template <typename Kernel>
inline cudaError_t set_smem_limit_once(Kernel kernel, int bytes, SmemLimitFlags& done) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < kMaxDevices && done[dev].load(std::memory_order_acquire)) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && dev >= 0 && dev < kMaxDevices) done[dev].store(1, std::memory_order_release);
  return e;
}

}  // namespace fa
