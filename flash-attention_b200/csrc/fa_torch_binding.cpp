// Compiled binding of the attention entry points: the reference's extension module
// (csrc/flash_attn/fmha_api.cpp: mha_fwd :173-299, mha_bwd :302-449, mha_fwd_block :451-573,
// mha_bwd_block :575-718) written against the C ABI of libfa_b200.so.  Same argument checks, output
// allocation and Philox protocol as the Python (ctypes) binding in flash_attn_b200/flash_attn_cuda.py,
// which remains for installations that did not build this file; what this one buys is host time: a
// call costs a few microseconds instead of 20-30, which is the whole run time at short sequences.
// The block-sparse entry points are the dense ones with a converted block mask (the Python module
// unpacks the reference's two call forms before it gets here).
//
// Things the reference's positional lists have no slot for arrive as trailing arguments from the
// Python wrapper: the status buffer of the device, the head-shard pair of the dropout mask, the
// deterministic-dQ switch, an explicit Philox pair for the backward.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAGeneratorImpl.h>
#include <c10/cuda/CUDAGuard.h>

#include <mutex>
#include <string>

#include "fa_b200.h"

namespace {

struct Dims {
  int64_t batch, total_q, total_k, heads, d;
};

void require(bool cond, const char* msg) {
  if (!cond) throw std::runtime_error(msg);
}

void check_rc(int rc) {
  if (rc != FA_OK)
    throw std::runtime_error(std::string("fa_b200: ") + fa_status_string(rc) + ": " + fa_last_error());
}

// Argument checks of mha_fwd / mha_bwd (fmha_api.cpp:199-230), same messages as the Python binding.
Dims check_qkv(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& cu_q,
               const at::Tensor& cu_k) {
  require(q.is_cuda() && k.is_cuda() && v.is_cuda(), "q, k, v must be CUDA tensors");
  const auto dt = q.scalar_type();
  require(dt == at::kHalf || dt == at::kBFloat16, "q must be fp16 or bf16");
  require(k.scalar_type() == dt && v.scalar_type() == dt, "q, k, v must have the same dtype");
  require(cu_q.scalar_type() == at::kInt && cu_k.scalar_type() == at::kInt, "cu_seqlens must be int32");
  require(cu_q.is_cuda() && cu_k.is_cuda(), "cu_seqlens must be CUDA tensors");
  require(cu_q.is_contiguous() && cu_k.is_contiguous(), "cu_seqlens must be contiguous");
  require(q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "q, k, v must be (total, heads, d)");
  require(q.stride(2) == 1 && k.stride(2) == 1 && v.stride(2) == 1,
          "q, k, v must have a contiguous last dimension");
  Dims s;
  s.batch = cu_q.size(0) - 1;
  require(s.batch > 0, "batch size must be positive");
  require(cu_k.size(0) == s.batch + 1, "cu_seqlens_q / cu_seqlens_k size mismatch");
  s.total_q = q.size(0);
  s.heads = q.size(1);
  s.d = q.size(2);
  s.total_k = k.size(0);
  require(s.d == 16 || s.d == 32 || s.d == 64 || s.d == 128, "head_dim must be 16, 32, 64 or 128");
  require(k.size(1) == s.heads && k.size(2) == s.d, "k has the wrong shape");
  require(v.size(0) == s.total_k && v.size(1) == s.heads && v.size(2) == s.d, "v has the wrong shape");
  return s;
}

void fill_fwd(fa_fwd_params& p, const Dims& s, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
              const at::Tensor& o, const at::Tensor& lse, const at::Tensor& cu_q, const at::Tensor& cu_k,
              int64_t max_q, int64_t max_k, double p_dropout, double scale, bool causal, uint64_t seed,
              uint64_t offset, int64_t mask_heads_total, int64_t mask_head_offset, int64_t status_ptr) {
  p = fa_fwd_params{};
  p.q = q.data_ptr();
  p.k = k.data_ptr();
  p.v = v.data_ptr();
  p.o = o.data_ptr();
  p.softmax_lse = static_cast<float*>(lse.data_ptr());
  p.cu_seqlens_q = static_cast<const int32_t*>(cu_q.data_ptr());
  p.cu_seqlens_k = static_cast<const int32_t*>(cu_k.data_ptr());
  p.q_row_stride = q.stride(0); p.q_head_stride = q.stride(1);
  p.k_row_stride = k.stride(0); p.k_head_stride = k.stride(1);
  p.v_row_stride = v.stride(0); p.v_head_stride = v.stride(1);
  p.o_row_stride = o.stride(0); p.o_head_stride = o.stride(1);
  p.lse_stride = lse.size(2);
  p.batch = static_cast<int32_t>(s.batch);
  p.heads = static_cast<int32_t>(s.heads);
  p.head_dim = static_cast<int32_t>(s.d);
  p.total_q = static_cast<int32_t>(s.total_q);
  p.total_k = static_cast<int32_t>(s.total_k);
  p.max_seqlen_q = static_cast<int32_t>(max_q);
  p.max_seqlen_k = static_cast<int32_t>(max_k);
  p.p_dropout = static_cast<float>(p_dropout);
  p.softmax_scale = static_cast<float>(scale);
  p.is_causal = causal ? 1 : 0;
  p.is_bf16 = q.scalar_type() == at::kBFloat16 ? 1 : 0;
  p.philox_seed = seed;
  p.philox_offset = offset;
  if (mask_heads_total != 0 || mask_head_offset != 0) {
    require(mask_heads_total >= mask_head_offset + s.heads && mask_head_offset >= 0,
            "head_shard: heads_total must cover head_offset + heads of this call");
    p.mask_heads_total = static_cast<int32_t>(mask_heads_total);
    p.mask_head_offset = static_cast<int32_t>(mask_head_offset);
  }
  p.status = reinterpret_cast<int32_t*>(static_cast<intptr_t>(status_ptr));
}

// (seed, offset) of the generator, then advance it by `increment` rounded up to a multiple of 4: what
// CUDAGeneratorImpl::philox_cuda_state(increment) does in the reference (fmha_api.cpp:288-292).
void philox_state(const c10::optional<at::Generator>& gen_, uint64_t increment, uint64_t& seed, uint64_t& offset) {
  auto gen = at::get_generator_or_default<at::CUDAGeneratorImpl>(gen_, at::cuda::detail::getDefaultCUDAGenerator());
  std::lock_guard<std::mutex> lock(gen->mutex_);
  seed = gen->current_seed();
  offset = gen->get_offset();
  gen->set_offset(offset + (increment + 3) / 4 * 4);
}

int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

// Block-sparse calls (fmha_api.cpp:451-573): checks of the converted mask and the scratch for the
// per-sequence block-visit table.  The reference checks for exactly (ceil(max_k / 256), ceil16(max_q) /
// 16) (:515); its own module passes a mask cut at a multiple of 256 rows' worth of slots, so a larger
// mask is accepted and its real row length is used.
void check_blockmask(const at::Tensor& blockmask, const at::Tensor& q, int64_t max_q, int64_t max_k) {
  require(blockmask.is_cuda() && blockmask.scalar_type() == at::kInt && blockmask.is_contiguous(),
          "blockmask must be a contiguous int32 CUDA tensor");
  const int64_t want0 = round_up(max_k, 256) / 256, want1 = round_up(max_q, 16) / 16;
  if (!(blockmask.dim() == 2 && blockmask.size(0) >= want0 && blockmask.size(1) >= want1)) {
    std::string got = "(";
    for (int64_t i = 0; i < blockmask.dim(); ++i) got += (i ? ", " : "") + std::to_string(blockmask.size(i));
    if (blockmask.dim() == 1) got += ",";
    throw std::runtime_error("blockmask must have at least shape (" + std::to_string(want0) + ", " +
                             std::to_string(want1) + "), got " + got + ")");
  }
  require(q.scalar_type() == at::kHalf, "block-sparse attention is fp16 only");
  require(q.size(2) == 16 || q.size(2) == 32 || q.size(2) == 64, "block-sparse attention supports head_dim 16, 32, 64");
}

at::Tensor attach_blockmask(fa_fwd_params& p, const at::Tensor& blockmask, const at::Tensor& q, int64_t batch) {
  const size_t nbytes = fa_blocksparse_workspace_bytes(static_cast<int32_t>(batch), static_cast<int32_t>(blockmask.size(0)),
                                                       static_cast<int32_t>(blockmask.size(1)));
  at::Tensor ws = at::empty({static_cast<int64_t>(nbytes < 4 ? 4 : nbytes)}, q.options().dtype(at::kByte));
  p.blockmask = static_cast<const int32_t*>(blockmask.data_ptr());
  p.blockmask_rows = static_cast<int32_t>(blockmask.size(0));
  p.blockmask_cols = static_cast<int32_t>(blockmask.size(1));
  p.bs_workspace = ws.data_ptr();
  p.bs_workspace_bytes = static_cast<size_t>(ws.numel());
  return ws;
}

py::list fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& cu_q,
             const at::Tensor& cu_k, int64_t max_q, int64_t max_k, double p_dropout, double scale,
             bool zero_tensors, bool causal, bool return_softmax, c10::optional<at::Generator> gen,
             c10::optional<at::Tensor> blockmask, bool return_philox, int64_t mask_heads_total,
             int64_t mask_head_offset, int64_t status_ptr) {
  const Dims s = check_qkv(q, k, v, cu_q, cu_k);
  require(p_dropout < 1.0, "p_dropout must be < 1");
  const bool sparse = blockmask.has_value();
  if (sparse) check_blockmask(*blockmask, q, max_q, max_k);
  c10::cuda::CUDAGuard guard(q.device());
  const auto opts = q.options();
  const int64_t lse_len = round_up(max_q, 16);
  // the block-sparse entry always starts from o = 0 (:519)
  at::Tensor o = (zero_tensors || sparse) ? at::zeros({s.total_q, s.heads, s.d}, opts)
                                          : at::empty({s.total_q, s.heads, s.d}, opts);
  at::Tensor lse = zero_tensors
                       ? at::full({s.batch, s.heads, lse_len}, -std::numeric_limits<float>::infinity(), opts.dtype(at::kFloat))
                       : at::empty({s.batch, s.heads, lse_len}, opts.dtype(at::kFloat));
  uint64_t seed = 0, offset = 0;
  if (p_dropout > 0)
    philox_state(gen, fa_philox_increment(static_cast<int32_t>(s.d), static_cast<int32_t>(max_q),
                                          static_cast<int32_t>(max_k), sparse ? 1 : 0), seed, offset);
  fa_fwd_params p;
  fill_fwd(p, s, q, k, v, o, lse, cu_q, cu_k, max_q, max_k, p_dropout, scale, causal, seed, offset,
           mask_heads_total, mask_head_offset, status_ptr);
  at::Tensor s_dmask, bs_ws;
  if (return_softmax) {
    // (batch, heads, seqlen_q rounded to 16, seqlen_k rounded as the reference does, :232-240, :253);
    // zero outside the sequences
    const int64_t base = sparse ? 256 : ((s.d == 128 && p_dropout > 0) ? 128 : 256);
    const int64_t sk_r = (max_k <= 128 && !sparse) ? 128 : (max_k <= 256 ? 256 : round_up(max_k, base));
    s_dmask = at::zeros({s.batch, s.heads, lse_len, sk_r}, opts);
    p.s_dmask = s_dmask.data_ptr();
    p.s_rows = lse_len;
    p.s_cols = sk_r;
  }
  if (sparse) bs_ws = attach_blockmask(p, *blockmask, q, s.batch);
  check_rc(fa_fwd(&p, at::cuda::getCurrentCUDAStream().stream()));
  py::list res;
  res.append(o);
  res.append(lse);
  if (return_softmax) res.append(s_dmask);
  if (return_philox) {
    res.append(py::int_(seed));
    res.append(py::int_(offset));
  }
  return res;
}

py::list bwd(const at::Tensor& dout, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
             const at::Tensor& out, const at::Tensor& lse, at::Tensor& dq, at::Tensor& dk, at::Tensor& dv,
             const at::Tensor& cu_q, const at::Tensor& cu_k, int64_t max_q, int64_t max_k, double p_dropout,
             double scale, bool zero_tensors, bool causal, c10::optional<at::Generator> gen,
             c10::optional<at::Tensor> blockmask, int64_t stage_mask, bool has_philox, uint64_t philox_seed,
             uint64_t philox_offset, bool deterministic,
             int64_t mask_heads_total, int64_t mask_head_offset, int64_t status_ptr) {
  const Dims s = check_qkv(q, k, v, cu_q, cu_k);
  const auto dt = q.scalar_type();
  require(dout.scalar_type() == dt && out.scalar_type() == dt, "dout / out dtype mismatch");
  require(dq.scalar_type() == dt && dk.scalar_type() == dt && dv.scalar_type() == dt, "dq / dk / dv dtype mismatch");
  require(out.is_contiguous() && dout.is_contiguous(), "out and dout must be contiguous");
  require(out.sizes() == q.sizes() && dout.sizes() == q.sizes(), "out / dout have the wrong shape");
  require(dq.sizes() == q.sizes(), "dq has the wrong shape");
  require(dk.sizes() == k.sizes() && dv.sizes() == k.sizes(), "dk / dv have the wrong shape");
  require(dq.stride(2) == 1 && dk.stride(2) == 1 && dv.stride(2) == 1,
          "dq, dk, dv must have a contiguous last dimension");
  require(lse.scalar_type() == at::kFloat && lse.dim() == 3 && lse.size(0) == s.batch && lse.size(1) == s.heads &&
              lse.size(2) >= max_q && lse.is_contiguous(),
          "softmax_lse must be a contiguous fp32 (batch, heads, >= max_seqlen_q) tensor");
  require(p_dropout < 1.0, "p_dropout must be < 1");
  c10::cuda::CUDAGuard guard(q.device());
  if (zero_tensors) {
    dq.zero_();
    dk.zero_();
    dv.zero_();
  }
  at::Tensor softmax_d = at::empty_like(lse);
  uint64_t seed = 0, offset = 0;
  if (p_dropout > 0) {
    // The caller restores the generator state saved before the forward, so reading the state here
    // yields the forward's pair; the reference then advances it by a dummy amount (:437-445).
    if (has_philox) {
      seed = philox_seed;
      offset = philox_offset;
    } else {
      philox_state(gen, 4, seed, offset);
    }
  }
  // fp32 dQ accumulator (and the ticket words of the deterministic mode) from the caching allocator,
  // per call, like the reference's dq_tmp (:402-404)
  const size_t nbytes = fa_bwd_workspace_bytes_ex(static_cast<int32_t>(s.total_q), static_cast<int32_t>(s.heads),
                                                  static_cast<int32_t>(s.d), static_cast<int32_t>(s.batch),
                                                  static_cast<int32_t>(max_q), deterministic ? 1 : 0);
  at::Tensor ws = at::empty({static_cast<int64_t>(nbytes < 16 ? 16 : nbytes)}, q.options().dtype(at::kByte));
  fa_bwd_params p = {};
  fill_fwd(p.fwd, s, q, k, v, out, lse, cu_q, cu_k, max_q, max_k, p_dropout, scale, causal, seed, offset,
           mask_heads_total, mask_head_offset, status_ptr);
  p.dout = dout.data_ptr();
  p.dq = dq.data_ptr();
  p.dk = dk.data_ptr();
  p.dv = dv.data_ptr();
  p.softmax_d = static_cast<float*>(softmax_d.data_ptr());
  p.dq_row_stride = dq.stride(0); p.dq_head_stride = dq.stride(1);
  p.dk_row_stride = dk.stride(0); p.dk_head_stride = dk.stride(1);
  p.dv_row_stride = dv.stride(0); p.dv_head_stride = dv.stride(1);
  p.workspace = ws.data_ptr();
  p.workspace_bytes = static_cast<size_t>(ws.numel());
  p.stage_mask = static_cast<int32_t>(stage_mask);
  p.deterministic = deterministic ? 1 : 0;
  at::Tensor bs_ws;
  if (blockmask.has_value()) {
    check_blockmask(*blockmask, q, max_q, max_k);
    bs_ws = attach_blockmask(p.fwd, *blockmask, q, s.batch);
  }
  check_rc(fa_bwd(&p, at::cuda::getCurrentCUDAStream().stream()));
  py::list res;
  res.append(dq);
  res.append(dk);
  res.append(dv);
  res.append(softmax_d);
  return res;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "compiled binding of libfa_b200.so: fwd / bwd with the reference extension's argument lists (+ optional block mask)";
  m.def("fwd", &fwd);
  m.def("bwd", &bwd);
}
