// C ABI of libfa_b200.so (declared in include/fa_b200.h): argument validation, TMA descriptor
// construction and kernel launches.  Mirrors the checks of the reference host API
// (csrc/flash_attn/fmha_api.cpp:173-299, :302-449) but reports errors through return codes
// instead of exceptions or exit().
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include "../../include/fa_b200.h"
#include "fa_kernels.h"

namespace {

thread_local std::string g_last_error;

int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

#define FA_REQUIRE(cond, msg)                                   \
  do {                                                          \
    if (!(cond)) return fail(FA_ERR_INVALID_ARGUMENT, (msg));   \
  } while (0)

#define FA_CUDA(expr)                                                                      \
  do {                                                                                     \
    cudaError_t e_ = (expr);                                                               \
    if (e_ != cudaSuccess)                                                                 \
      return fail(FA_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e_));        \
  } while (0)

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so that the library has no link-time
// dependency on libcuda and can be loaded (for symbol checks) on a machine without a driver.
EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 3-D map over a [rows, heads, head_dim] tensor with arbitrary row / head strides:
// dim0 = head_dim, dim1 = rows, dim2 = heads; box = 64 columns x box_rows rows x 1 head, stored
// with the 128-byte swizzle.  Columns beyond head_dim and rows beyond `rows` read as zero.
// `bind_context`: a thread that has only used the runtime API lazily (an autograd worker, for
// instance) may not have the primary context bound yet and the driver call below needs it;
// cudaFree(nullptr) binds it.  The entry point that must not touch the allocator passes false
// (it has bound the context with cudaSetDevice already).
int make_tile_map(CUtensorMap* tm, const void* base, bool bf16, int64_t rows, int heads, int head_dim,
                  int64_t row_stride, int64_t head_stride, int box_rows, bool bind_context = true) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return fail(FA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  static thread_local bool context_bound = false;
  if (bind_context && !context_bound) {
    FA_CUDA(cudaFree(nullptr));
    context_bound = true;
  }
  FA_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor base must be 16-byte aligned");
  FA_REQUIRE((row_stride * 2) % 16 == 0 && (head_stride * 2) % 16 == 0,
             "row and head strides must be multiples of 8 elements");
  // A descriptor is a pure function of these eight values, and a training loop presents the same
  // ones again and again (the caching allocator hands back the same blocks): a small per-thread
  // cache saves the driver call, which is a large share of the host time of a short-sequence call.
  struct Entry {
    const void* base; int64_t rows, row_stride, head_stride; int32_t heads, head_dim, box_rows, bf16;
    CUtensorMap map;
  };
  constexpr int kCacheSize = 32;
  static thread_local Entry cache[kCacheSize];
  static thread_local int cache_used = 0, cache_next = 0;
  for (int i = 0; i < cache_used; ++i) {
    const Entry& e = cache[i];
    if (e.base == base && e.rows == rows && e.row_stride == row_stride && e.head_stride == head_stride &&
        e.heads == heads && e.head_dim == head_dim && e.box_rows == box_rows && e.bf16 == (bf16 ? 1 : 0)) {
      *tm = e.map;
      return FA_OK;
    }
  }
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(rows),
                        static_cast<cuuint64_t>(heads)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(row_stride) * 2,
                           static_cast<cuuint64_t>(head_stride) * 2};
  cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(FA_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  Entry& slot = cache[cache_next];
  slot = Entry{base, rows, row_stride, head_stride, heads, head_dim, box_rows, bf16 ? 1 : 0, *tm};
  cache_next = (cache_next + 1) % kCacheSize;
  if (cache_used < kCacheSize) ++cache_used;
  return FA_OK;
}

// fp32 dQ accumulator [rows, heads, dpad]: box = 32 columns x 128 rows x 1 head, 128-byte swizzle
// (the layout the backward kernel stages dQ tiles in before its TMA reduce-add).
int make_accum_map(CUtensorMap* tm, float* base, int64_t rows, int heads, int dpad) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return fail(FA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(dpad), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(heads)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(heads) * dpad * 4, static_cast<cuuint64_t>(dpad) * 4};
  cuuint32_t box[3] = {32, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(FA_ERR_CUDA, "cuTensorMapEncodeTiled (accumulator) failed with code " + std::to_string((int)r));
  return FA_OK;
}

int round_up(int x, int m) { return (x + m - 1) / m * m; }

// Serial number of a call (never 0).  The kernels compare status[0] with it instead of having the
// word cleared before every launch: one stream operation less per call.
int32_t next_launch_id() {
  static std::atomic<uint32_t> counter{0};
  uint32_t id = counter.fetch_add(1, std::memory_order_relaxed) + 1;
  if ((id & 0x7fffffffu) == 0) id = counter.fetch_add(1, std::memory_order_relaxed) + 1;
  return static_cast<int32_t>(id & 0x7fffffffu);
}

int validate_common(const fa_fwd_params* p) {
  FA_REQUIRE(p != nullptr, "params is null");
  FA_REQUIRE(p->q && p->k && p->v, "q, k, v must be non-null");
  FA_REQUIRE(p->cu_seqlens_q && p->cu_seqlens_k, "cu_seqlens must be non-null");
  FA_REQUIRE(p->batch > 0, "batch must be positive");
  FA_REQUIRE(p->heads > 0, "heads must be positive");
  FA_REQUIRE(p->head_dim == 16 || p->head_dim == 32 || p->head_dim == 64 || p->head_dim == 128,
             "head_dim must be 16, 32, 64 or 128");
  FA_REQUIRE(p->total_q >= 0 && p->total_k >= 0, "negative token count");
  FA_REQUIRE(p->max_seqlen_q > 0 && p->max_seqlen_k > 0, "max_seqlen must be positive");
  FA_REQUIRE(p->p_dropout >= 0.f && p->p_dropout < 1.f, "p_dropout must be in [0, 1)");
  FA_REQUIRE(p->lse_stride >= p->max_seqlen_q, "softmax_lse rows are shorter than max_seqlen_q");
  if (p->blockmask) {
    FA_REQUIRE(!p->is_bf16, "block-sparse attention is fp16 only");
    FA_REQUIRE(p->head_dim <= 64, "block-sparse attention supports head_dim 16, 32, 64");
  }
  return FA_OK;
}

void fill_dropout(const fa_fwd_params* p, fa::KernelArgs* a) {
  const float p_keep = 1.f - p->p_dropout;
  a->rp_keep = 1.f / p_keep;
  a->drop.key0 = static_cast<uint32_t>(p->philox_seed);
  a->drop.key1 = static_cast<uint32_t>(p->philox_seed >> 32);
  a->drop.counter_base = p->philox_offset / 4;
  for (int r = 0; r < 7; ++r) {
    a->drop.rk0[r] = a->drop.key0 + static_cast<uint32_t>(r) * 0x9E3779B9u;
    a->drop.rk1[r] = a->drop.key1 + static_cast<uint32_t>(r) * 0xBB67AE85u;
  }
  a->drop.threshold = static_cast<uint32_t>(
      static_cast<uint16_t>(std::floor(static_cast<double>(p_keep) * 65535.0)));
  a->drop.n_shift = fa_mask_block_n(p->head_dim, p->max_seqlen_k, p->blockmask != nullptr) == 128 ? 7 : 8;
  a->drop.heads_total = p->mask_heads_total > 0 ? p->mask_heads_total : p->heads;
  a->drop.head_offset = p->mask_heads_total > 0 ? p->mask_head_offset : 0;
}

// Block-sparse: check the scratch, build the block-visit table on the stream, point the kernel
// arguments at it.
int setup_blocksparse(const fa_fwd_params* p, fa::KernelArgs* a, cudaStream_t stream) {
  const int nk = p->blockmask_rows;
  const int nr = p->blockmask_cols;
  FA_REQUIRE(nk >= round_up(p->max_seqlen_k, 256) / 256, "blockmask has too few key-block rows");
  FA_REQUIRE(nr >= round_up(p->max_seqlen_q, 16) / 16, "blockmask rows are too short for max_seqlen_q");
  // the kernels keep a per-CTA list of visited 128-row tiles in shared memory (1024 entries)
  FA_REQUIRE(p->max_seqlen_q <= 131072 && p->max_seqlen_k <= 131072,
             "block-sparse attention supports sequences up to 131072");
  const size_t need = fa_blocksparse_workspace_bytes(p->batch, nk, nr);
  if (p->bs_workspace == nullptr || p->bs_workspace_bytes < need)
    return fail(FA_ERR_WORKSPACE, "bs_workspace must hold " + std::to_string(need) + " bytes");
  FA_REQUIRE(nk <= 4096, "block-sparse attention supports at most 4096 key blocks");
  int32_t* table = static_cast<int32_t*>(p->bs_workspace);
  FA_CUDA(fa::launch_bs_table(table, p->blockmask, p->cu_seqlens_q, p->cu_seqlens_k, p->batch, nk, nr, stream));
  a->bs_iter = table;
  a->bs_kblocks = nk;
  a->bs_rows16 = nr;
  return FA_OK;
}

void fill_args(const fa_fwd_params* p, fa::KernelArgs* a) {
  std::memset(a, 0, sizeof(*a));
  a->cu_seqlens_q = p->cu_seqlens_q;
  a->cu_seqlens_k = p->cu_seqlens_k;
  a->o = p->o;
  a->lse = p->softmax_lse;
  a->o_row_stride = p->o_row_stride;
  a->o_head_stride = p->o_head_stride;
  a->lse_stride = p->lse_stride;
  a->batch = p->batch;
  a->heads = p->heads;
  a->head_dim = p->head_dim;
  a->scale = p->softmax_scale;
  a->scale_log2 = p->softmax_scale * 1.4426950408889634f;
  a->status = p->status;
  a->launch_id = next_launch_id();
  fill_dropout(p, a);
}

}  // namespace

extern "C" {

int fa_gather_rows(const void* src, const int64_t* indices, void* dst, int64_t n_rows,
                   int64_t src_rows, int64_t row_bytes, void* cuda_stream) {
  FA_REQUIRE(n_rows >= 0 && src_rows >= 0 && row_bytes >= 0, "negative size");
  if (n_rows == 0 || row_bytes == 0) return FA_OK;
  FA_REQUIRE(src && indices && dst, "src, indices and dst must be non-null");
  FA_REQUIRE(row_bytes % 16 == 0, "row_bytes must be a multiple of 16");
  FA_REQUIRE(((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0,
             "src and dst must be 16-byte aligned");
  FA_CUDA(fa::launch_gather_rows(src, indices, dst, n_rows, src_rows, row_bytes,
                                 static_cast<cudaStream_t>(cuda_stream)));
  return FA_OK;
}

int fa_scatter_rows(const void* src, const int64_t* indices, void* dst, int64_t n_src_rows,
                    int64_t n_dst_rows, int64_t row_bytes, int32_t* workspace, void* cuda_stream) {
  FA_REQUIRE(n_src_rows >= 0 && n_dst_rows >= 0 && row_bytes >= 0, "negative size");
  if (n_dst_rows == 0 || row_bytes == 0) return FA_OK;
  FA_REQUIRE(dst && workspace, "dst and workspace must be non-null");
  FA_REQUIRE(n_src_rows == 0 || (src && indices), "src and indices must be non-null");
  FA_REQUIRE(n_src_rows <= 0x7fffffffLL, "too many source rows");
  FA_REQUIRE(row_bytes % 16 == 0, "row_bytes must be a multiple of 16");
  FA_REQUIRE(((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0,
             "src and dst must be 16-byte aligned");
  FA_CUDA(fa::launch_scatter_rows(src, indices, dst, n_src_rows, n_dst_rows, row_bytes, workspace,
                                  static_cast<cudaStream_t>(cuda_stream)));
  return FA_OK;
}

int fa_rotary_qkv(const void* qkv, void* out, const float* cos_table, const float* sin_table,
                  int64_t rows, int32_t seqlen, int32_t heads, int32_t head_dim, int32_t is_bf16,
                  int32_t conjugate, void* cuda_stream) {
  FA_REQUIRE(rows >= 0 && seqlen > 0 && heads > 0 && head_dim > 0, "sizes must be positive");
  if (rows == 0) return FA_OK;
  FA_REQUIRE(qkv && out && cos_table && sin_table, "null pointer");
  FA_REQUIRE(qkv != out, "out may not alias qkv");
  FA_REQUIRE(head_dim % 8 == 0, "head_dim must be a multiple of 8");
  FA_REQUIRE(rows % seqlen == 0, "rows must be a multiple of seqlen");
  FA_REQUIRE(((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(out) |
               reinterpret_cast<uintptr_t>(cos_table) | reinterpret_cast<uintptr_t>(sin_table)) & 15) == 0,
             "qkv, out and the tables must be 16-byte aligned");
  FA_CUDA(fa::launch_rotary_qkv(qkv, out, cos_table, sin_table, rows, seqlen, heads, head_dim,
                                is_bf16 != 0, conjugate != 0, static_cast<cudaStream_t>(cuda_stream)));
  return FA_OK;
}

const char* fa_status_string(int status) {
  switch (status) {
    case FA_OK: return "ok";
    case FA_ERR_INVALID_ARGUMENT: return "invalid argument";
    case FA_ERR_CUDA: return "CUDA error";
    case FA_ERR_UNSUPPORTED: return "unsupported configuration";
    case FA_ERR_WORKSPACE: return "workspace missing or too small";
    default: return "unknown status";
  }
}

const char* fa_last_error(void) { return g_last_error.c_str(); }

int fa_device_supported(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fail(FA_ERR_CUDA, "no CUDA device");
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
    return fail(FA_ERR_CUDA, "cannot query the device");
  if (major != 10) return fail(FA_ERR_UNSUPPORTED, "this library only runs on sm_100 devices");
  return FA_OK;
}

int32_t fa_mask_block_n(int32_t head_dim, int32_t max_seqlen_k, int32_t is_blocksparse) {
  if (is_blocksparse) return 256;
  if (max_seqlen_k <= 128) return 128;
  return head_dim == 128 ? 128 : 256;
}

uint64_t fa_philox_increment(int32_t head_dim, int32_t max_seqlen_q, int32_t max_seqlen_k,
                             int32_t is_blocksparse) {
  const int n = fa_mask_block_n(head_dim, max_seqlen_k, is_blocksparse);
  const int base = is_blocksparse ? 256 : (head_dim == 128 ? 128 : 256);
  int sk = round_up(max_seqlen_k, base);
  if (!is_blocksparse) {
    if (max_seqlen_k <= 128) sk = 128;
    else if (max_seqlen_k <= 256) sk = 256;
  }
  const int sq = round_up(max_seqlen_q, 16);
  const uint64_t steps = static_cast<uint64_t>(sq / 16);
  const uint64_t mmas_n = static_cast<uint64_t>(n / 64);
  const uint64_t loop_steps = static_cast<uint64_t>((sk + n - 1) / n);
  return steps * mmas_n * 8 * loop_steps;
}

int fa_fwd(const fa_fwd_params* p, void* cuda_stream) {
  if (int rc = validate_common(p)) return rc;
  FA_REQUIRE(p->o && p->softmax_lse, "o and softmax_lse must be non-null");
  FA_REQUIRE((reinterpret_cast<uintptr_t>(p->o) & 15) == 0, "o must be 16-byte aligned");
  FA_REQUIRE(p->o_row_stride % 8 == 0 && p->o_head_stride % 8 == 0,
             "o strides must be multiples of 8 elements");
  if (p->s_dmask) FA_REQUIRE(p->s_rows >= p->max_seqlen_q && p->s_cols >= p->max_seqlen_k,
                             "s_dmask must be at least (max_seqlen_q, max_seqlen_k) per (batch, head)");

  fa::FwdLaunch l;
  std::memset(&l, 0, sizeof(l));
  fill_args(p, &l.args);
  if (p->blockmask)
    if (int rc = setup_blocksparse(p, &l.args, static_cast<cudaStream_t>(cuda_stream))) return rc;
  l.dpad = p->head_dim <= 64 ? 64 : 128;
  l.is_bf16 = p->is_bf16 != 0;
  l.is_causal = p->is_causal != 0;
  l.is_dropout = p->p_dropout > 0.f;
  l.max_seqlen_q = p->max_seqlen_q;
  l.max_seqlen_k = p->max_seqlen_k;
  if (int rc = make_tile_map(&l.tm_q, p->q, l.is_bf16, p->total_q, p->heads, p->head_dim,
                             p->q_row_stride, p->q_head_stride, 128)) return rc;
  if (int rc = make_tile_map(&l.tm_k, p->k, l.is_bf16, p->total_k, p->heads, p->head_dim,
                             p->k_row_stride, p->k_head_stride, 128)) return rc;
  if (int rc = make_tile_map(&l.tm_v, p->v, l.is_bf16, p->total_k, p->heads, p->head_dim,
                             p->v_row_stride, p->v_head_stride, 128)) return rc;
  FA_CUDA(fa::launch_fwd(l, static_cast<cudaStream_t>(cuda_stream)));
  if (p->s_dmask)
    FA_CUDA(fa::launch_sdmask(p->s_dmask, p->s_rows, p->s_cols, p->q, p->k, p->q_row_stride, p->q_head_stride,
                              p->k_row_stride, p->k_head_stride, l.args, p->max_seqlen_q, p->max_seqlen_k,
                              l.is_bf16, l.is_causal, l.is_dropout, static_cast<cudaStream_t>(cuda_stream)));
  return FA_OK;
}

int fa_debug_dropout_mask(uint8_t* mask_out, int32_t batch_idx, int32_t head_idx,
                          const fa_fwd_params* p, int32_t seqlen_q, int32_t seqlen_k,
                          void* cuda_stream) {
  FA_REQUIRE(p != nullptr && mask_out != nullptr, "null argument");
  fa::KernelArgs a;
  std::memset(&a, 0, sizeof(a));
  fill_dropout(p, &a);
  if (p->blockmask)
    if (int rc = setup_blocksparse(p, &a, static_cast<cudaStream_t>(cuda_stream))) return rc;
  FA_CUDA(fa::launch_dropout_mask(mask_out, batch_idx, head_idx, a.drop, p->is_causal != 0, seqlen_q,
                                  seqlen_k, a.bs_iter, a.bs_kblocks, a.bs_rows16,
                                  static_cast<cudaStream_t>(cuda_stream)));
  return FA_OK;
}

int fa_debug_philox(uint32_t* out, int32_t n, uint64_t seed, uint64_t offset, int32_t rounds,
                    int32_t use_curand, void* cuda_stream) {
  FA_REQUIRE(out != nullptr && n >= 0, "bad arguments");
  FA_REQUIRE(use_curand || (rounds >= 1 && rounds <= 16), "rounds must be in [1, 16]");
  FA_CUDA(fa::launch_philox_probe(out, n, seed, offset, rounds, use_curand ? 1 : 0,
                                  static_cast<cudaStream_t>(cuda_stream)));
  return FA_OK;
}

size_t fa_blocksparse_workspace_bytes(int32_t batch, int32_t blockmask_rows, int32_t blockmask_cols) {
  return static_cast<size_t>(batch) * static_cast<size_t>(blockmask_rows) *
         static_cast<size_t>(blockmask_cols) * sizeof(int32_t);
}

size_t fa_bwd_workspace_bytes(int32_t total_q, int32_t heads, int32_t head_dim) {
  const size_t dpad = head_dim <= 64 ? 64 : 128;
  return static_cast<size_t>(total_q) * static_cast<size_t>(heads) * dpad * sizeof(float);
}

namespace {

// Body shared by fa_bwd and fa_bwd_static_scratch: validation, kernel arguments, the five tensor
// maps and the launches.  `accum` is the fp32 dQ accumulator (already checked to be large enough).
int run_bwd(const fa_bwd_params* p, float* accum, int stage_mask, bool bind_context, cudaStream_t stream) {
  const fa_fwd_params* f = &p->fwd;
  if (int rc = validate_common(f)) return rc;
  FA_REQUIRE(f->o && f->softmax_lse, "out and softmax_lse must be non-null");
  FA_REQUIRE(p->dout && p->dq && p->dk && p->dv && p->softmax_d, "dout, dq, dk, dv, softmax_d must be non-null");
  FA_REQUIRE(((reinterpret_cast<uintptr_t>(p->dq) | reinterpret_cast<uintptr_t>(p->dk) |
               reinterpret_cast<uintptr_t>(p->dv) | reinterpret_cast<uintptr_t>(f->o)) & 15) == 0,
             "o, dq, dk, dv must be 16-byte aligned");
  FA_REQUIRE(p->dq_row_stride % 8 == 0 && p->dq_head_stride % 8 == 0 && p->dk_row_stride % 8 == 0 &&
                 p->dk_head_stride % 8 == 0 && p->dv_row_stride % 8 == 0 && p->dv_head_stride % 8 == 0 &&
                 f->o_row_stride % 8 == 0 && f->o_head_stride % 8 == 0,
             "gradient strides must be multiples of 8 elements");
  FA_REQUIRE((reinterpret_cast<uintptr_t>(accum) & 15) == 0, "workspace must be 16-byte aligned");

  fa::BwdLaunch l;
  std::memset(&l, 0, sizeof(l));
  fill_args(f, &l.args.k);
  if (f->blockmask)
    if (int rc = setup_blocksparse(f, &l.args.k, stream)) return rc;
  l.dpad = f->head_dim <= 64 ? 64 : 128;
  l.is_bf16 = f->is_bf16 != 0;
  l.is_causal = f->is_causal != 0;
  l.is_dropout = f->p_dropout > 0.f;
  l.stage_mask = stage_mask;
  l.deterministic = p->deterministic != 0;
  fa::BwdArgs& a = l.args;
  a.o_in = f->o;
  a.dout = p->dout;
  a.do_row_stride = static_cast<int64_t>(f->heads) * f->head_dim;
  a.do_head_stride = f->head_dim;
  a.dq = p->dq; a.dk = p->dk; a.dv = p->dv;
  a.dq_row_stride = p->dq_row_stride; a.dq_head_stride = p->dq_head_stride;
  a.dk_row_stride = p->dk_row_stride; a.dk_head_stride = p->dk_head_stride;
  a.dv_row_stride = p->dv_row_stride; a.dv_head_stride = p->dv_head_stride;
  a.softmax_d = p->softmax_d;
  a.dq_accum = accum;
  if (l.deterministic) {
    // ticket words sit behind the accumulator (fa_bwd_workspace_bytes_ex)
    const size_t off = fa_bwd_workspace_bytes(f->total_q, f->heads, f->head_dim);
    a.dq_tickets = reinterpret_cast<int32_t*>(reinterpret_cast<char*>(accum) + ((off + 255) & ~size_t(255)));
    a.ticket_stride = (f->max_seqlen_q + 127) / 128;
  }
  a.total_q = f->total_q; a.total_k = f->total_k;
  a.max_seqlen_q = f->max_seqlen_q; a.max_seqlen_k = f->max_seqlen_k;
  a.p_keep = 1.f - f->p_dropout;
  if (int rc = make_tile_map(&l.tm_q, f->q, l.is_bf16, f->total_q, f->heads, f->head_dim,
                             f->q_row_stride, f->q_head_stride, 128, bind_context)) return rc;
  if (int rc = make_tile_map(&l.tm_k, f->k, l.is_bf16, f->total_k, f->heads, f->head_dim,
                             f->k_row_stride, f->k_head_stride, 128, bind_context)) return rc;
  if (int rc = make_tile_map(&l.tm_v, f->v, l.is_bf16, f->total_k, f->heads, f->head_dim,
                             f->v_row_stride, f->v_head_stride, 128, bind_context)) return rc;
  if (int rc = make_tile_map(&l.tm_do, p->dout, l.is_bf16, f->total_q, f->heads, f->head_dim,
                             a.do_row_stride, a.do_head_stride, 128, bind_context)) return rc;
  if (int rc = make_accum_map(&l.tm_dq, a.dq_accum, f->total_q, f->heads, l.dpad)) return rc;
  FA_CUDA(fa::launch_bwd(l, stream));
  return FA_OK;
}

}  // namespace

size_t fa_bwd_workspace_bytes_ex(int32_t total_q, int32_t heads, int32_t head_dim, int32_t batch,
                                 int32_t max_seqlen_q, int32_t deterministic) {
  const size_t accum = fa_bwd_workspace_bytes(total_q, heads, head_dim);
  if (!deterministic) return accum;
  const size_t tickets = static_cast<size_t>(batch) * static_cast<size_t>(heads) *
                         static_cast<size_t>((max_seqlen_q + 127) / 128) * sizeof(int32_t);
  return ((accum + 255) & ~size_t(255)) + tickets;
}

int fa_bwd(const fa_bwd_params* p, void* cuda_stream) {
  FA_REQUIRE(p != nullptr, "params is null");
  const fa_fwd_params* f = &p->fwd;
  FA_REQUIRE(f->total_q >= 0 && f->heads > 0 && f->batch > 0 && f->max_seqlen_q > 0, "bad sizes");
  const size_t need = fa_bwd_workspace_bytes_ex(f->total_q, f->heads, f->head_dim, f->batch,
                                                f->max_seqlen_q, p->deterministic);
  if (p->workspace == nullptr || p->workspace_bytes < need)
    return fail(FA_ERR_WORKSPACE, "workspace must hold " + std::to_string(need) + " bytes");
  return run_bwd(p, static_cast<float*>(p->workspace), p->stage_mask, true,
                 static_cast<cudaStream_t>(cuda_stream));
}

// ---------------------------------------------------------------------------------------------
// Backward without a caller-supplied workspace.
//
// The fp32 dQ accumulator of the backward pass normally lives in scratch the caller allocates
// (fa_bwd_params.workspace).  Some callers have nothing to allocate it from: a serving process
// whose device memory was carved up at start-up and that must stay away from the CUDA allocator
// afterwards (cudaMalloc may fail once another pool owns the memory, and it synchronises the
// device), or a plain C / Go / Java binding that holds tensors but no caching allocator to borrow
// scratch from.  For them the accumulator below is part of the library image: every GPU that
// loads the library holds these FA_STATIC_SCRATCH_BYTES until the process exits.
static __device__ __align__(256) float g_static_dq_accum[FA_STATIC_SCRATCH_BYTES / sizeof(float)];

namespace {

constexpr int kMaxDevices = 64;
float* g_static_dq_ptr[kMaxDevices] = {};

// Device address of g_static_dq_accum on the current device.  The array's name is only a
// host-side handle here; the kernels need the address cudaGetSymbolAddress reports, which differs
// per device.  Looked up once per device (with that device current) and cached.
int static_scratch_address(float** out) {
  int dev = 0;
  FA_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(FA_ERR_UNSUPPORTED, "device ordinal out of range");
  // Binds the primary context to this thread without allocating anything.
  FA_CUDA(cudaSetDevice(dev));
  float* ptr = __atomic_load_n(&g_static_dq_ptr[dev], __ATOMIC_ACQUIRE);
  if (ptr == nullptr) {
    void* sym = nullptr;
    FA_CUDA(cudaGetSymbolAddress(&sym, g_static_dq_accum));
    if (sym == nullptr) return fail(FA_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    ptr = static_cast<float*>(sym);
    __atomic_store_n(&g_static_dq_ptr[dev], ptr, __ATOMIC_RELEASE);
  }
  *out = ptr;
  return FA_OK;
}

}  // namespace

int fa_bwd_static_scratch(const fa_bwd_params* p, void* cuda_stream) {
  FA_REQUIRE(p != nullptr, "params is null");
  const fa_fwd_params* f = &p->fwd;
  FA_REQUIRE(f->total_q >= 0 && f->heads > 0 && f->batch > 0 && f->max_seqlen_q > 0, "bad sizes");
  const size_t need = fa_bwd_workspace_bytes_ex(f->total_q, f->heads, f->head_dim, f->batch,
                                                f->max_seqlen_q, p->deterministic);
  if (need > FA_STATIC_SCRATCH_BYTES)
    return fail(FA_ERR_WORKSPACE,
                "fa_bwd_static_scratch: this call needs " + std::to_string(need) +
                    " bytes of dQ accumulator but the built-in scratch holds " +
                    std::to_string(static_cast<size_t>(FA_STATIC_SCRATCH_BYTES)) +
                    " (total_q * heads * padded head_dim * 4); use fa_bwd with a workspace");
  float* accum = nullptr;
  if (int rc = static_scratch_address(&accum)) return rc;
  // all three stages: the preprocess stage clears the rows of the shared scratch this call uses
  return run_bwd(p, accum, 0, false, static_cast<cudaStream_t>(cuda_stream));
}

}  // extern "C"
