"""ctypes view of libfa_b200.so: structures and prototypes of include/fa_b200.h.

There is no fallback: if the shared library is missing, or cannot be loaded, importing this
module raises and every public function of the package is unusable.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfa_b200.so")

FA_OK = 0
FA_ERR_INVALID_ARGUMENT = -1
FA_ERR_CUDA = -2
FA_ERR_UNSUPPORTED = -3
FA_ERR_WORKSPACE = -4
FA_STATIC_SCRATCH_BYTES = 8 << 20

EXPORTED_SYMBOLS = (
    "fa_fwd",
    "fa_bwd",
    "fa_bwd_static_scratch",
    "fa_bwd_workspace_bytes",
    "fa_bwd_workspace_bytes_ex",
    "fa_blocksparse_workspace_bytes",
    "fa_philox_increment",
    "fa_mask_block_n",
    "fa_debug_dropout_mask",
    "fa_debug_philox",
    "fa_gather_rows",
    "fa_scatter_rows",
    "fa_rotary_qkv",
    "fa_status_string",
    "fa_last_error",
    "fa_device_supported",
)


class FwdParams(ctypes.Structure):
    """struct fa_fwd_params"""
    _fields_ = [
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("o", ctypes.c_void_p),
        ("softmax_lse", ctypes.c_void_p),
        ("cu_seqlens_q", ctypes.c_void_p),
        ("cu_seqlens_k", ctypes.c_void_p),
        ("blockmask", ctypes.c_void_p),
        ("s_dmask", ctypes.c_void_p),
        ("s_rows", ctypes.c_int64),
        ("s_cols", ctypes.c_int64),
        ("q_row_stride", ctypes.c_int64),
        ("q_head_stride", ctypes.c_int64),
        ("k_row_stride", ctypes.c_int64),
        ("k_head_stride", ctypes.c_int64),
        ("v_row_stride", ctypes.c_int64),
        ("v_head_stride", ctypes.c_int64),
        ("o_row_stride", ctypes.c_int64),
        ("o_head_stride", ctypes.c_int64),
        ("lse_stride", ctypes.c_int64),
        ("batch", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("total_q", ctypes.c_int32),
        ("total_k", ctypes.c_int32),
        ("max_seqlen_q", ctypes.c_int32),
        ("max_seqlen_k", ctypes.c_int32),
        ("p_dropout", ctypes.c_float),
        ("softmax_scale", ctypes.c_float),
        ("is_causal", ctypes.c_int32),
        ("is_bf16", ctypes.c_int32),
        ("philox_seed", ctypes.c_uint64),
        ("philox_offset", ctypes.c_uint64),
        ("mask_heads_total", ctypes.c_int32),
        ("mask_head_offset", ctypes.c_int32),
        ("status", ctypes.c_void_p),
        ("bs_workspace", ctypes.c_void_p),
        ("bs_workspace_bytes", ctypes.c_size_t),
        ("blockmask_rows", ctypes.c_int32),
        ("blockmask_cols", ctypes.c_int32),
    ]


class BwdParams(ctypes.Structure):
    """struct fa_bwd_params"""
    _fields_ = [
        ("fwd", FwdParams),
        ("dout", ctypes.c_void_p),
        ("dq", ctypes.c_void_p),
        ("dk", ctypes.c_void_p),
        ("dv", ctypes.c_void_p),
        ("softmax_d", ctypes.c_void_p),
        ("dq_row_stride", ctypes.c_int64),
        ("dq_head_stride", ctypes.c_int64),
        ("dk_row_stride", ctypes.c_int64),
        ("dk_head_stride", ctypes.c_int64),
        ("dv_row_stride", ctypes.c_int64),
        ("dv_head_stride", ctypes.c_int64),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("stage_mask", ctypes.c_int32),
        ("deterministic", ctypes.c_int32),
    ]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libfa_b200.so is not built: run `python flash-attention_b200/build.py` "
            "(there is no fallback implementation)")
    lib = ctypes.CDLL(LIB_PATH)
    lib.fa_fwd.argtypes = [ctypes.POINTER(FwdParams), ctypes.c_void_p]
    lib.fa_fwd.restype = ctypes.c_int
    lib.fa_bwd.argtypes = [ctypes.POINTER(BwdParams), ctypes.c_void_p]
    lib.fa_bwd.restype = ctypes.c_int
    lib.fa_bwd_static_scratch.argtypes = [ctypes.POINTER(BwdParams), ctypes.c_void_p]
    lib.fa_bwd_static_scratch.restype = ctypes.c_int
    lib.fa_bwd_workspace_bytes.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
    lib.fa_bwd_workspace_bytes.restype = ctypes.c_size_t
    lib.fa_bwd_workspace_bytes_ex.argtypes = [ctypes.c_int32] * 6
    lib.fa_bwd_workspace_bytes_ex.restype = ctypes.c_size_t
    lib.fa_blocksparse_workspace_bytes.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
    lib.fa_blocksparse_workspace_bytes.restype = ctypes.c_size_t
    lib.fa_philox_increment.argtypes = [ctypes.c_int32] * 4
    lib.fa_philox_increment.restype = ctypes.c_uint64
    lib.fa_mask_block_n.argtypes = [ctypes.c_int32] * 3
    lib.fa_mask_block_n.restype = ctypes.c_int32
    lib.fa_debug_dropout_mask.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32,
                                          ctypes.POINTER(FwdParams), ctypes.c_int32,
                                          ctypes.c_int32, ctypes.c_void_p]
    lib.fa_debug_dropout_mask.restype = ctypes.c_int
    lib.fa_debug_philox.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_uint64, ctypes.c_uint64,
                                    ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
    lib.fa_debug_philox.restype = ctypes.c_int
    lib.fa_gather_rows.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                   ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
    lib.fa_gather_rows.restype = ctypes.c_int
    lib.fa_scatter_rows.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                    ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
    lib.fa_scatter_rows.restype = ctypes.c_int
    lib.fa_rotary_qkv.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                  ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                  ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
    lib.fa_rotary_qkv.restype = ctypes.c_int
    lib.fa_status_string.argtypes = [ctypes.c_int]
    lib.fa_status_string.restype = ctypes.c_char_p
    lib.fa_last_error.argtypes = []
    lib.fa_last_error.restype = ctypes.c_char_p
    lib.fa_device_supported.argtypes = []
    lib.fa_device_supported.restype = ctypes.c_int
    return lib


lib = _load()


def check(rc):
    """Turn a non-zero status into RuntimeError, like TORCH_CHECK does in the reference
    (csrc/flash_attn/fmha_api.cpp:192)."""
    if rc != FA_OK:
        raise RuntimeError("fa_b200: %s: %s" % (lib.fa_status_string(rc).decode(),
                                                lib.fa_last_error().decode()))
