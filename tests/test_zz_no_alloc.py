"""fa_bwd_static_scratch: the backward entry point for callers that cannot allocate device memory
at call time (the dQ accumulator is an array inside the library instead of caller scratch).

Called through the C ABI twice in a row and compared with fa_bwd on the same inputs.  The second
call uses a smaller problem, so it also shows that what the first call left in the shared array
does not leak into the next result.  Collected last on purpose (file name): a failure here cannot
hide the result of any other test in a run that stops at the first failure."""
import ctypes

import pytest
import torch

from tests import _util as U

pytestmark = pytest.mark.gpu


def _bwd_params(fc, _lib, q, k, v, out, lse, dout, grads, softmax_d, cu_q, cu_k, max_q, max_k, scale, causal,
                p_dropout=0.0, philox=(0, 0)):
    p = _lib.BwdParams()
    dims = fc._check_qkv(q, k, v, cu_q, cu_k)
    fc._fill_fwd(p.fwd, dims, q, k, v, out, lse, cu_q, cu_k, max_q, max_k, p_dropout, scale, causal,
                 philox[0], philox[1])
    p.dout = dout.data_ptr()
    p.dq, p.dk, p.dv = (g.data_ptr() for g in grads)
    p.softmax_d = softmax_d.data_ptr()
    p.dq_row_stride, p.dq_head_stride = grads[0].stride(0), grads[0].stride(1)
    p.dk_row_stride, p.dk_head_stride = grads[1].stride(0), grads[1].stride(1)
    p.dv_row_stride, p.dv_head_stride = grads[2].stride(0), grads[2].stride(1)
    return p


def _attach_blockmask(_lib, p, blockmask, batch):
    """Block-sparse calls still bring their own block-visit table scratch (caller memory)."""
    ws = torch.empty(_lib.lib.fa_blocksparse_workspace_bytes(batch, blockmask.shape[0], blockmask.shape[1]),
                     dtype=torch.uint8, device="cuda")
    p.fwd.blockmask = blockmask.data_ptr()
    p.fwd.blockmask_rows, p.fwd.blockmask_cols = blockmask.shape
    p.fwd.bs_workspace, p.fwd.bs_workspace_bytes = ws.data_ptr(), ws.numel()
    return ws


def _one_call(seqlens_q, seqlens_k, heads, d, dtype, causal, seed, p_dropout=0.0, blockmask=None):
    from flash_attn_b200 import _lib
    from flash_attn_b200 import flash_attn_cuda as fc
    q, k, v, dout, cu_q, cu_k = U.make_varlen(seqlens_q, seqlens_k, heads, d, dtype, seed=seed)
    max_q, max_k = max(seqlens_q), max(seqlens_k)
    scale = d ** -0.5
    if blockmask is None:
        out, lse, ph_seed, ph_off = fc.fwd(q, k, v, cu_q, cu_k, max_q, max_k, p_dropout, scale, False, causal,
                                           False, None, return_philox=True)
    else:
        out, lse, ph_seed, ph_off = fc.fwd_block(q, k, v, cu_q, cu_k, blockmask, max_q, max_k, p_dropout, scale,
                                                 causal, False, None, return_philox=True)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    philox = (ph_seed, ph_off)
    keep_alive = []

    # existing entry point, caller-allocated workspace
    ref = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]
    d_ref = torch.empty_like(lse)
    p = _bwd_params(fc, _lib, q, k, v, out, lse, dout, ref, d_ref, cu_q, cu_k, max_q, max_k, scale, causal,
                    p_dropout, philox)
    if blockmask is not None:
        keep_alive.append(_attach_blockmask(_lib, p, blockmask, len(seqlens_q)))
    ws = torch.empty(_lib.lib.fa_bwd_workspace_bytes(q.shape[0], heads, d), dtype=torch.uint8, device="cuda")
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    _lib.check(_lib.lib.fa_bwd(ctypes.byref(p), stream))

    # new entry point: no workspace passed, nothing allocated by the call
    got = [torch.full_like(q, float("nan")), torch.full_like(k, float("nan")), torch.full_like(v, float("nan"))]
    d_got = torch.empty_like(lse)
    p2 = _bwd_params(fc, _lib, q, k, v, out, lse, dout, got, d_got, cu_q, cu_k, max_q, max_k, scale, causal,
                     p_dropout, philox)
    if blockmask is not None:
        keep_alive.append(_attach_blockmask(_lib, p2, blockmask, len(seqlens_q)))
    p2.workspace, p2.workspace_bytes = None, 0
    # one call first: it loads the kernels' module and looks up the address of the built-in array
    _lib.check(_lib.lib.fa_bwd_static_scratch(ctypes.byref(p2), stream))
    torch.cuda.synchronize()
    # the property in the entry point's name: a call moves neither the framework's allocator
    # counters nor the device's free memory
    stats0 = torch.cuda.memory_stats()
    free0 = torch.cuda.mem_get_info()[0]
    _lib.check(_lib.lib.fa_bwd_static_scratch(ctypes.byref(p2), stream))
    torch.cuda.synchronize()
    stats1 = torch.cuda.memory_stats()
    free1 = torch.cuda.mem_get_info()[0]
    for key in ("allocation.all.allocated", "allocation.all.freed", "segment.all.allocated",
                "reserved_bytes.all.current", "allocated_bytes.all.current"):
        assert stats0.get(key) == stats1.get(key), key
    assert free0 == free1
    fc.check_device_status()

    # dk, dv are computed in a fixed order: identical.  dq is summed with fp32 atomics whose order
    # varies from run to run: same tolerance as the dense-vs-sparse comparison of the other tests.
    assert torch.equal(got[1], ref[1]) and torch.equal(got[2], ref[2])
    assert U.max_err(got[0], ref[0]) < 2e-3
    assert not torch.isnan(got[0].float()).any()
    for b, n in enumerate(seqlens_q):
        assert torch.equal(d_got[b, :, :n], d_ref[b, :, :n])
    # and both agree with the oracle
    if p_dropout == 0.0 and blockmask is None:
        o32, dq32, dk32, dv32 = U.oracle_cpu(q, k, v, dout, cu_q, cu_k, scale, causal)
        o16, dq16, dk16, dv16 = U.oracle_cpu(q, k, v, dout, cu_q, cu_k, scale, causal, dtype=dtype)
        U.assert_within_2x("dq", got[0], dq32, dq16)
        U.assert_within_2x("dk", got[1], dk32, dk16)
        U.assert_within_2x("dv", got[2], dv32, dv16)


def test_static_scratch_backward_two_calls_in_a_row():
    _one_call([700, 300], [700, 300], 4, 64, torch.float16, True, seed=61)
    _one_call([130], [257], 2, 128, torch.bfloat16, False, seed=62)


def test_static_scratch_backward_with_dropout_and_blocksparse():
    """The same two paths that regenerate a dropout mask or walk a block-sparse layout, through the
    built-in array (compared with fa_bwd on the same Philox pair)."""
    from flash_attn_b200.flash_blocksparse_attn_interface import convert_blockmask
    _one_call([600, 450], [600, 450], 4, 64, torch.float16, False, seed=63, p_dropout=0.2)
    torch.manual_seed(1)
    S = 768
    blocks = (torch.rand(S // 256, S // 256) < 0.5) | torch.eye(S // 256, dtype=torch.bool)
    conv = convert_blockmask(blocks.repeat_interleave(16, dim=0).to(torch.int32).cuda(), False)
    _one_call([S, 500], [S, 500], 2, 64, torch.float16, False, seed=64, p_dropout=0.1, blockmask=conv)


def test_static_scratch_leaves_rows_behind_the_sequences_alone():
    """After a larger call has dirtied the shared array, a call whose dq buffer is longer than its
    sequences must not write the stale contents into the rows that belong to no sequence."""
    from flash_attn_b200 import _lib
    from flash_attn_b200 import flash_attn_cuda as fc
    _one_call([900, 800], [900, 800], 4, 64, torch.float16, False, seed=65)   # dirties ~1700 rows
    lens, extra = [100, 160], 300
    q, k, v, dout, cu, _ = U.make_varlen(lens + [extra], lens + [extra], 4, 64, torch.float16, seed=66)
    cu = cu[:3].contiguous()
    out, lse = fc.fwd(q, k, v, cu, cu, 160, 160, 0.0, 0.125, False, False, False, None)
    grads = [torch.full_like(q, 7.0), torch.full_like(k, 7.0), torch.full_like(v, 7.0)]
    p = _bwd_params(fc, _lib, q, k, v, out, lse, dout, grads, torch.empty_like(lse), cu, cu, 160, 160, 0.125, False)
    p.workspace, p.workspace_bytes = None, 0
    _lib.check(_lib.lib.fa_bwd_static_scratch(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    fc.check_device_status()
    assert torch.all(grads[0][260:] == 7.0)
    o32, dq32, dk32, dv32 = U.oracle_cpu(q[:260], k[:260], v[:260], dout[:260], cu, cu, 0.125, False)
    assert U.max_err(grads[0][:260], dq32) < 4e-3


def test_static_scratch_rejects_oversized_calls():
    from flash_attn_b200 import _lib
    from flash_attn_b200 import flash_attn_cuda as fc
    heads, d = 16, 64
    total = _lib.FA_STATIC_SCRATCH_BYTES // (heads * d * 4) + 1
    q = torch.zeros(total, heads, d, device="cuda", dtype=torch.float16)
    cu = torch.tensor([0, total], dtype=torch.int32, device="cuda")
    lse = torch.zeros(1, heads, (total + 15) // 16 * 16, device="cuda")
    grads = [torch.empty_like(q) for _ in range(3)]
    p = _bwd_params(fc, _lib, q, q, q, q, lse, q, grads, torch.empty_like(lse), cu, cu, total, total, 0.125, False)
    rc = _lib.lib.fa_bwd_static_scratch(ctypes.byref(p), None)
    assert rc == _lib.FA_ERR_WORKSPACE
    assert b"built-in scratch" in _lib.lib.fa_last_error()
