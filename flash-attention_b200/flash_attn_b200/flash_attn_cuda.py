"""Drop-in for the reference's compiled extension module `flash_attn_cuda`
(csrc/flash_attn/fmha_api.cpp:721-727): `fwd`, `bwd`, `fwd_block`, `bwd_block` with the reference's
argument lists, implemented as a thin binding over the C ABI of libfa_b200.so.

PyTorch is used here only for device memory (output / scratch allocation through the caching
allocator), the current stream and the default CUDA generator's Philox state.

Two routes into the library.  The ctypes route below is complete (every entry point and option).
When the compiled binding `_fa_binding` (csrc/fa_torch_binding.cpp, built by build.py) is present,
the calls go through it instead: same checks, allocation and Philox protocol in C++, a few
microseconds of host time per call instead of 20-30.  Set
FA_B200_BINDING=ctypes to keep everything on the ctypes route.
"""
import ctypes
import os
import struct

import torch

from . import _lib
from ._lib import BwdParams, FwdParams, check, lib

_binding = None
if os.environ.get("FA_B200_BINDING", "") != "ctypes":
    try:
        from . import _fa_binding as _binding   # noqa: F401
    except ImportError:
        _binding = None


def binding_in_use():
    """'compiled' when calls go through the C++ binding, else 'ctypes'."""
    return "compiled" if _binding is not None else "ctypes"


_status = {}
_status_ptr = {}


class _Options:
    """Process-wide switches of the binding that have no counterpart in the reference's argument
    lists (the four entry points keep the reference's positional contract).

    deterministic  backward passes add their dQ tiles in key-tile order, so dq is bit-for-bit
                   reproducible (fa_bwd_params.deterministic); slower.
    mask_heads     (heads_total, head_offset) or None: a rank that holds heads
                   [head_offset, head_offset + heads) of a model with heads_total heads draws the
                   dropout mask of the unsharded call (fa_fwd_params.mask_heads_total / _offset).
    """
    __slots__ = ("deterministic", "mask_heads")

    def __init__(self):
        self.deterministic = False
        self.mask_heads = None


options = _Options()


class head_shard:
    """Context manager: inside it every forward / backward on this process draws the dropout mask
    of heads [head_offset, head_offset + heads) of an unsharded call with `heads_total` heads."""

    def __init__(self, heads_total, head_offset):
        self.value = (int(heads_total), int(head_offset))
        self.prev = None

    def __enter__(self):
        self.prev = options.mask_heads
        options.mask_heads = self.value
        return self

    def __exit__(self, *exc):
        options.mask_heads = self.prev
        return False


def _status_buffer(device):
    """Per-device int32[4] the kernels write to when they abandon a bounded wait."""
    buf = _status.get(device)
    if buf is None:
        buf = torch.zeros(128, dtype=torch.int32, device=device)
        _status[device] = buf
        _status_ptr[device] = buf.data_ptr()
    return buf


def check_device_status(device=None):
    """Synchronises and raises if any kernel on `device` reported an abandoned wait."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    buf = _status.get(device)
    if buf is None:
        return
    val = buf[:4].cpu().tolist()
    if val[2] or val[3]:
        buf.zero_()
        raise RuntimeError("fa_b200: a kernel abandoned a bounded wait (status %s)" % val)


def _require(cond, msg):
    if not cond:
        raise RuntimeError(msg)


class _on_device:
    """`torch.cuda.device(dev)` that costs nothing when `dev` is already current (the usual case;
    the stock context manager resolves the device twice on every entry)."""
    __slots__ = ("idx", "prev")

    def __init__(self, device):
        self.idx = device.index
        self.prev = -1

    def __enter__(self):
        cur = torch._C._cuda_getDevice()
        if self.idx is not None and cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


def _raw_stream():
    """Handle (cudaStream_t as an integer) of the current stream of the current device."""
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


def _philox_state(gen, increment):
    """(seed, offset) of the generator, then advance it by `increment` -- what
    CUDAGeneratorImpl::philox_cuda_state(increment) does in the reference
    (csrc/flash_attn/fmha_api.cpp:288-292)."""
    if gen is None:
        gen = torch.cuda.default_generators[torch.cuda.current_device()]
    seed = gen.initial_seed()
    offset = gen.get_offset()
    # the generator keeps its offset a multiple of 4, like the reference's PhiloxCudaState
    gen.set_offset(offset + ((int(increment) + 3) // 4) * 4)
    return seed, offset


_DIMS_OK = (16, 32, 64, 128)


def _check_qkv(q, k, v, cu_seqlens_q, cu_seqlens_k):
    """Argument checks of mha_fwd / mha_bwd (csrc/flash_attn/fmha_api.cpp:199-230).  The usual, valid
    call is decided by one expression; only a call that fails it is taken apart for its message."""
    qs, ks, vs = q.shape, k.shape, v.shape
    dt = q.dtype
    nb = cu_seqlens_q.shape[0]
    if (len(qs) == 3 and ks[1:] == qs[1:] and vs == ks and q.is_cuda and k.is_cuda and v.is_cuda
            and (dt is torch.float16 or dt is torch.bfloat16) and k.dtype is dt and v.dtype is dt
            and cu_seqlens_q.dtype is torch.int32 and cu_seqlens_k.dtype is torch.int32
            and cu_seqlens_q.is_cuda and cu_seqlens_k.is_cuda and nb > 1 and cu_seqlens_k.shape[0] == nb
            and qs[2] in _DIMS_OK and q.stride(2) == 1 and k.stride(2) == 1 and v.stride(2) == 1
            and cu_seqlens_q.is_contiguous() and cu_seqlens_k.is_contiguous()):
        return nb - 1, qs[0], ks[0], qs[1], qs[2]
    _require(q.is_cuda and k.is_cuda and v.is_cuda, "q, k, v must be CUDA tensors")
    _require(dt is torch.float16 or dt is torch.bfloat16, "q must be fp16 or bf16")
    _require(k.dtype is dt and v.dtype is dt, "q, k, v must have the same dtype")
    _require(cu_seqlens_q.dtype is torch.int32 and cu_seqlens_k.dtype is torch.int32,
             "cu_seqlens must be int32")
    _require(cu_seqlens_q.is_cuda and cu_seqlens_k.is_cuda, "cu_seqlens must be CUDA tensors")
    _require(cu_seqlens_q.is_contiguous() and cu_seqlens_k.is_contiguous(),
             "cu_seqlens must be contiguous")
    _require(len(qs) == 3 and len(ks) == 3 and len(vs) == 3, "q, k, v must be (total, heads, d)")
    _require(q.stride(2) == 1 and k.stride(2) == 1 and v.stride(2) == 1,
             "q, k, v must have a contiguous last dimension")
    batch = nb - 1
    _require(batch > 0, "batch size must be positive")
    _require(cu_seqlens_k.shape[0] == batch + 1, "cu_seqlens_q / cu_seqlens_k size mismatch")
    total_q, heads, d = qs
    total_k = ks[0]
    _require(d in _DIMS_OK, "head_dim must be 16, 32, 64 or 128")
    _require(ks[1] == heads and ks[2] == d, "k has the wrong shape")
    _require(vs[0] == total_k and vs[1] == heads and vs[2] == d, "v has the wrong shape")
    return batch, total_q, total_k, heads, d


# struct fa_fwd_params / fa_bwd_params as `struct` formats (native alignment): packing forty values into
# a buffer in one call costs a third of the ctypes constructor, and the per-call host time of
# short-sequence workloads is mostly this binding.
_FWD_FMT = "9P 2q 9q 7i 2f 2i 2Q 2i P P N 2i"
_FWD_PACK = struct.Struct("@" + _FWD_FMT)
_BWD_PACK = struct.Struct("@" + _FWD_FMT + " 5P 6q P N 2i")
assert _FWD_PACK.size == ctypes.sizeof(FwdParams), (_FWD_PACK.size, ctypes.sizeof(FwdParams))
assert _BWD_PACK.size == ctypes.sizeof(BwdParams), (_BWD_PACK.size, ctypes.sizeof(BwdParams))


def _fwd_values(dims, q, k, v, o, lse, cu_q, cu_k, max_q, max_k, p_dropout, scale, causal, seed, offset):
    batch, total_q, total_k, heads, d = dims
    qs, ks, vs, os_ = q.stride(), k.stride(), v.stride(), o.stride()
    mh = options.mask_heads
    if mh is not None:
        _require(mh[0] >= mh[1] + heads and mh[1] >= 0,
                 "head_shard: heads_total must cover head_offset + heads of this call")
        mh_total, mh_offset = mh
    else:
        mh_total = mh_offset = 0
    return (q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
            cu_q.data_ptr(), cu_k.data_ptr(), 0, 0, 0, 0,
            qs[0], qs[1], ks[0], ks[1], vs[0], vs[1], os_[0], os_[1], lse.shape[-1],
            batch, heads, d, total_q, total_k, int(max_q), int(max_k),
            float(p_dropout), float(scale), 1 if causal else 0,
            1 if q.dtype is torch.bfloat16 else 0, seed, offset, mh_total, mh_offset,
            _status_buffer(q.device).data_ptr(), 0, 0, 0, 0)


def _make_fwd(dims, q, k, v, o, lse, cu_q, cu_k, max_q, max_k, p_dropout, scale, causal, seed, offset):
    """A filled FwdParams (a view of one packed buffer)."""
    buf = bytearray(_FWD_PACK.size)
    _FWD_PACK.pack_into(buf, 0, *_fwd_values(dims, q, k, v, o, lse, cu_q, cu_k, max_q, max_k, p_dropout,
                                             scale, causal, seed, offset))
    return FwdParams.from_buffer(buf)


def _make_bwd(fwd_values, dout, dq, dk, dv, softmax_d, ws, stage_mask, deterministic):
    """A filled BwdParams: the forward block followed by the gradient pointers and strides."""
    dqs, dks, dvs = dq.stride(), dk.stride(), dv.stride()
    buf = bytearray(_BWD_PACK.size)
    _BWD_PACK.pack_into(buf, 0, *fwd_values, dout.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                        softmax_d.data_ptr(), dqs[0], dqs[1], dks[0], dks[1], dvs[0], dvs[1],
                        ws.data_ptr(), ws.numel(), stage_mask, deterministic)
    return BwdParams.from_buffer(buf)


def _fill_fwd(p, dims, q, k, v, o, lse, cu_q, cu_k, max_q, max_k, p_dropout, scale, causal, seed, offset):
    """Same as _make_fwd, into an existing FwdParams (for instance the `fwd` member of a BwdParams)."""
    src = _make_fwd(dims, q, k, v, o, lse, cu_q, cu_k, max_q, max_k, p_dropout, scale, causal, seed, offset)
    ctypes.memmove(ctypes.addressof(p), ctypes.addressof(src), ctypes.sizeof(FwdParams))


def _round_up(x, m):
    return (x + m - 1) // m * m


def _bs_workspace(device, batch, blockmask):
    nbytes = lib.fa_blocksparse_workspace_bytes(batch, blockmask.shape[0], blockmask.shape[1])
    return torch.empty(max(nbytes, 4), dtype=torch.uint8, device=device)


def _check_blockmask(blockmask, max_seqlen_q, max_seqlen_k, q):
    _require(blockmask.is_cuda and blockmask.dtype == torch.int32 and blockmask.is_contiguous(),
             "blockmask must be a contiguous int32 CUDA tensor")
    # The reference checks for exactly (ceil(max_k / 256), ceil16(max_q) / 16)
    # (csrc/flash_attn/fmha_api.cpp:515); its own module passes a mask cut at a multiple of 256
    # rows' worth of slots, so a larger mask is accepted here and its real row length is used.
    want = (_round_up(int(max_seqlen_k), 256) // 256, _round_up(int(max_seqlen_q), 16) // 16)
    _require(blockmask.dim() == 2 and blockmask.shape[0] >= want[0] and blockmask.shape[1] >= want[1],
             "blockmask must have at least shape %s, got %s" % (want, tuple(blockmask.shape)))
    _require(q.dtype == torch.float16, "block-sparse attention is fp16 only")
    _require(q.shape[-1] in (16, 32, 64), "block-sparse attention supports head_dim 16, 32, 64")


def _run_fwd(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, p_dropout,
             softmax_scale, zero_tensors, is_causal, return_softmax, gen, blockmask=None,
             return_philox=False):
    if _binding is not None:
        dev = q.device
        sp = _status_ptr.get(dev)
        if sp is None:
            sp = _status_buffer(dev).data_ptr()
        mh = options.mask_heads or (0, 0)
        return _binding.fwd(q, k, v, cu_seqlens_q, cu_seqlens_k, int(max_seqlen_q), int(max_seqlen_k),
                            float(p_dropout), float(softmax_scale), bool(zero_tensors), bool(is_causal),
                            bool(return_softmax), gen, blockmask, return_philox, mh[0], mh[1], sp)
    batch, total_q, total_k, heads, d = _check_qkv(q, k, v, cu_seqlens_q, cu_seqlens_k)
    _require(p_dropout < 1.0, "p_dropout must be < 1")
    sparse = blockmask is not None
    if sparse:
        _check_blockmask(blockmask, max_seqlen_q, max_seqlen_k, q)
    with _on_device(q.device):
        lse_len = _round_up(int(max_seqlen_q), 16)
        if zero_tensors or sparse:  # the block-sparse entry always starts from o = 0 (:519)
            o = torch.zeros((total_q, heads, d), dtype=q.dtype, device=q.device)
        else:
            o = torch.empty((total_q, heads, d), dtype=q.dtype, device=q.device)
        if zero_tensors:
            lse = torch.full((batch, heads, lse_len), float("-inf"), dtype=torch.float32,
                             device=q.device)
        else:
            lse = torch.empty((batch, heads, lse_len), dtype=torch.float32, device=q.device)
        seed, offset = 0, 0
        if p_dropout > 0:
            inc = lib.fa_philox_increment(d, int(max_seqlen_q), int(max_seqlen_k), int(sparse))
            seed, offset = _philox_state(gen, inc)
        p = _make_fwd((batch, total_q, total_k, heads, d), q, k, v, o, lse, cu_seqlens_q,
                      cu_seqlens_k, max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale, is_causal,
                      seed, offset)
        s_dmask = None
        if return_softmax:
            # (batch, heads, seqlen_q rounded to 16, seqlen_k rounded as the reference does,
            # csrc/flash_attn/fmha_api.cpp:232-240, :253); zero outside the sequences
            base = 256 if sparse else (128 if (d == 128 and p_dropout > 0) else 256)
            sk_r = 128 if (max_seqlen_k <= 128 and not sparse) else (256 if max_seqlen_k <= 256 else _round_up(int(max_seqlen_k), base))
            s_dmask = torch.zeros((batch, heads, lse_len, sk_r), dtype=q.dtype, device=q.device)
            p.s_dmask, p.s_rows, p.s_cols = s_dmask.data_ptr(), lse_len, sk_r
        if sparse:
            ws = _bs_workspace(q.device, batch, blockmask)
            p.blockmask = blockmask.data_ptr()
            p.blockmask_rows, p.blockmask_cols = blockmask.shape
            p.bs_workspace, p.bs_workspace_bytes = ws.data_ptr(), ws.numel()
        check(lib.fa_fwd(ctypes.byref(p), _raw_stream()))
    res = [o, lse, s_dmask] if return_softmax else [o, lse]
    if return_philox:
        res += [seed, offset]
    return res


def fwd(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale,
        zero_tensors, is_causal, return_softmax, gen=None, return_philox=False):
    """mha_fwd (csrc/flash_attn/fmha_api.cpp:173-299): returns [o, softmax_lse(, s)].

    return_philox (keyword, not in the reference): append the Philox (seed, offset) the dropout
    mask of this call was drawn from -- the pair the reference takes from the generator under its
    mutex (:288-292) and keeps to itself -- as two Python ints behind the tensors.  They are what
    fa_fwd_params.philox_seed / philox_offset received; the generator has been advanced by
    fa_philox_increment() past them.  Both are 0 when p_dropout == 0."""
    return _run_fwd(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, p_dropout,
                    softmax_scale, zero_tensors, is_causal, return_softmax, gen,
                    return_philox=return_philox)


def fwd_block(*args, return_philox=False):
    """mha_fwd_block.  Two call forms are accepted because the reference's Python call site and its
    C++ signature disagree:
      * 13 arguments, the C++ signature (csrc/flash_attn/fmha_api.cpp:451-464):
        (q, k, v, cu_seqlens_q, cu_seqlens_k, blockmask, max_seqlen_q, max_seqlen_k, p_dropout,
         softmax_scale, is_causal, return_softmax, gen) -> [o, softmax_lse]
      * 9 arguments, the Python call site (flash_attn/flash_blocksparse_attn_interface.py:45-47):
        (qkv, cu_seqlens, blockmask, dropout_p, max_s, softmax_scale, causal, return_softmax, gen)
        with qkv (total, 3, heads, d) -> [context, softmax_lse]"""
    if len(args) == 13:
        (q, k, v, cu_q, cu_k, blockmask, max_q, max_k, p_dropout, scale, causal, ret_sm, gen) = args
        return _run_fwd(q, k, v, cu_q, cu_k, max_q, max_k, p_dropout, scale, False, causal, ret_sm,
                        gen, blockmask=blockmask, return_philox=return_philox)
    if len(args) == 9:
        (qkv, cu, blockmask, p_dropout, max_s, scale, causal, ret_sm, gen) = args
        _require(qkv.dim() == 4 and qkv.shape[1] == 3, "qkv must be (total, 3, heads, head_dim)")
        return _run_fwd(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, cu, max_s, max_s, p_dropout, scale,
                        False, causal, ret_sm, gen, blockmask=blockmask, return_philox=return_philox)
    raise TypeError("fwd_block takes 9 or 13 positional arguments, got %d" % len(args))


fwd_block.accepted_arities = (9, 13)


def bwd(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
        max_seqlen_k, p_dropout, softmax_scale, zero_tensors, is_causal, gen=None, _stage_mask=0,
        _blockmask=None, philox=None):
    """mha_bwd (csrc/flash_attn/fmha_api.cpp:302-449): writes dq, dk, dv in place and returns
    [dq, dk, dv, softmax_d].

    philox (keyword, not in the reference): the (seed, offset) pair `fwd(..., return_philox=True)`
    handed back; the mask is then regenerated from it and the generator is left alone (the
    reference's callers restore the generator state around this call instead)."""
    if _binding is not None:
        dev = q.device
        sp = _status_ptr.get(dev)
        if sp is None:
            sp = _status_buffer(dev).data_ptr()
        mh = options.mask_heads or (0, 0)
        has_philox = philox is not None
        return _binding.bwd(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k,
                            int(max_seqlen_q), int(max_seqlen_k), float(p_dropout), float(softmax_scale),
                            bool(zero_tensors), bool(is_causal), gen, _blockmask, int(_stage_mask), has_philox,
                            int(philox[0]) if has_philox else 0, int(philox[1]) if has_philox else 0,
                            bool(options.deterministic), mh[0], mh[1], sp)
    batch, total_q, total_k, heads, d = _check_qkv(q, k, v, cu_seqlens_q, cu_seqlens_k)
    dt, qshape, kshape = q.dtype, q.shape, k.shape
    _require(dout.dtype is dt and out.dtype is dt, "dout / out dtype mismatch")
    _require(dq.dtype is dt and dk.dtype is dt and dv.dtype is dt, "dq / dk / dv dtype mismatch")
    _require(out.is_contiguous() and dout.is_contiguous(), "out and dout must be contiguous")
    _require(out.shape == qshape and dout.shape == qshape, "out / dout have the wrong shape")
    _require(dq.shape == qshape, "dq has the wrong shape")
    _require(dk.shape == kshape and dv.shape == kshape, "dk / dv have the wrong shape")
    _require(dq.stride(2) == 1 and dk.stride(2) == 1 and dv.stride(2) == 1,
             "dq, dk, dv must have a contiguous last dimension")
    lshape = softmax_lse.shape
    _require(softmax_lse.dtype is torch.float32 and len(lshape) == 3 and lshape[0] == batch
             and lshape[1] == heads and lshape[2] >= max_seqlen_q and softmax_lse.is_contiguous(),
             "softmax_lse must be a contiguous fp32 (batch, heads, >= max_seqlen_q) tensor")
    _require(p_dropout < 1.0, "p_dropout must be < 1")
    with _on_device(q.device):
        if zero_tensors:
            dq.zero_()
            dk.zero_()
            dv.zero_()
        softmax_d = torch.empty_like(softmax_lse)
        seed, offset = 0, 0
        if p_dropout > 0:
            # The caller restores the generator state saved before the forward, so reading the
            # state here yields the forward's (seed, offset); the reference then advances it by a
            # dummy amount (csrc/flash_attn/fmha_api.cpp:437-445).
            seed, offset = philox if philox is not None else _philox_state(gen, 4)
        # fp32 dQ accumulator (and the ticket words of the deterministic mode): allocated per call
        # from the caching allocator like the reference's dq_tmp (csrc/flash_attn/fmha_api.cpp:
        # 402-404), so backward passes on different streams or threads never share scratch
        det = 1 if options.deterministic else 0
        nbytes = lib.fa_bwd_workspace_bytes_ex(total_q, heads, d, batch, int(max_seqlen_q), det)
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
        p = _make_bwd(_fwd_values((batch, total_q, total_k, heads, d), q, k, v, out, softmax_lse,
                                  cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, p_dropout,
                                  softmax_scale, is_causal, seed, offset),
                      dout, dq, dk, dv, softmax_d, ws, _stage_mask, det)
        if _blockmask is not None:
            _check_blockmask(_blockmask, max_seqlen_q, max_seqlen_k, q)
            bws = _bs_workspace(q.device, batch, _blockmask)
            p.fwd.blockmask = _blockmask.data_ptr()
            p.fwd.blockmask_rows, p.fwd.blockmask_cols = _blockmask.shape
            p.fwd.bs_workspace, p.fwd.bs_workspace_bytes = bws.data_ptr(), bws.numel()
        check(lib.fa_bwd(ctypes.byref(p), _raw_stream()))
    return [dq, dk, dv, softmax_d]


def bwd_block(*args, philox=None):
    """mha_bwd_block.  Accepts the C++ signature (18 arguments,
    csrc/flash_attn/fmha_api.cpp:575-594):
        (dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k, blockmask,
         max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale, is_causal, gen)
        -> [dq, dk, dv, softmax_d]
    and the Python call site's form (12 arguments,
    flash_attn/flash_blocksparse_attn_interface.py:56-58):
        (dout, qkv, out, S_dmask, softmax_lse, cu_seqlens, blockmask, dropout_p, softmax_scale,
         max_s, causal, gen) -> (dqkv, dp, softmax_d)
    where S_dmask is ignored (the call site passes a placeholder) and dp is None."""
    if len(args) == 18:
        (dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, blockmask, max_q, max_k, p_dropout, scale,
         causal, gen) = args
        return bwd(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, max_q, max_k, p_dropout, scale,
                   False, causal, gen, _blockmask=blockmask, philox=philox)
    if len(args) == 12:
        (dout, qkv, out, _s_dmask, lse, cu, blockmask, p_dropout, scale, max_s, causal, gen) = args
        _require(qkv.dim() == 4 and qkv.shape[1] == 3, "qkv must be (total, 3, heads, head_dim)")
        dqkv = torch.empty_like(qkv)
        res = bwd(dout.contiguous(), qkv[:, 0], qkv[:, 1], qkv[:, 2], out, lse, dqkv[:, 0],
                  dqkv[:, 1], dqkv[:, 2], cu, cu, max_s, max_s, p_dropout, scale, False, causal, gen,
                  _blockmask=blockmask, philox=philox)
        return dqkv, None, res[3]
    raise TypeError("bwd_block takes 12 or 18 positional arguments, got %d" % len(args))


bwd_block.accepted_arities = (12, 18)
