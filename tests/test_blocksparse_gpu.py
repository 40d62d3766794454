"""Block-sparse attention through the blocksparse interface and the extension-module contract
(fwd_block / bwd_block, both call forms), against the CPU oracle with the layout applied as a
score mask."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from tests import _util as U

pytestmark = pytest.mark.gpu


def _layout(seed, seqlen, density):
    """Random 0/1 layout over 256 x 256 blocks with the diagonal kept, expanded to 16-row blocks."""
    nb = (seqlen + 255) // 256
    g = torch.Generator().manual_seed(seed)
    blocks = (torch.rand(nb, nb, generator=g) < density) | torch.eye(nb, dtype=torch.bool)
    return blocks.repeat_interleave(16, dim=0).to(torch.int32)  # (nb * 16, nb)


def _allowed(blockmask_conv, sq_list, sk_list):
    return [torch.from_numpy(orc.blocksparse_allowed(blockmask_conv, sq, sk)) for sq, sk in zip(sq_list, sk_list)]


@pytest.mark.parametrize("d,seqlens,density,p", [
    (64, [512], 0.5, 0.0),
    (64, [1024, 700], 0.3, 0.0),
    (32, [300, 513], 0.5, 0.0),
    (64, [1024], 0.3, 0.1),
    (16, [600, 256], 0.4, 0.2),
])
def test_blocksparse_forward_backward_parity(d, seqlens, density, p):
    from flash_attn_b200.flash_blocksparse_attn_interface import convert_blockmask, flash_blocksparse_attn_func
    heads = 2
    max_s = max(seqlens)
    layout = _layout(3, max_s, density).cuda()
    q, k, v, dout, cu, _ = U.make_varlen(seqlens, seqlens, heads, d, torch.float16, seed=23)
    qkv = torch.stack([q, k, v], dim=1).contiguous().requires_grad_()
    seed = 31
    torch.cuda.manual_seed(seed)
    out = flash_blocksparse_attn_func(qkv, cu, layout, p, max_s)
    out.backward(dout)
    torch.cuda.synchronize()
    from flash_attn_b200 import flash_attn_cuda
    flash_attn_cuda.check_device_status()

    conv = convert_blockmask(layout, False).cpu().numpy()
    np.testing.assert_array_equal(conv, orc.convert_blockmask_loops(layout.cpu().numpy()))
    allowed = _allowed(conv, seqlens, seqlens)
    masks = None
    if p > 0:
        masks = []
        for b, n in enumerate(seqlens):
            it = orc.blocksparse_walk(conv, n, n)
            masks.append(torch.from_numpy(np.stack([
                orc.dropout_keep_mask(seed, 0, b, h, heads, n, n, p, 256, False, bs_iter=it)
                for h in range(heads)])))
    scale = d ** -0.5
    o32, dq32, dk32, dv32 = U.oracle_cpu(q, k, v, dout, cu, cu, scale, False, p, masks, allowed)
    o16, dq16, dk16, dv16 = U.oracle_cpu(q, k, v, dout, cu, cu, scale, False, p, masks, allowed, dtype=torch.float16)
    g = qkv.grad
    U.assert_within_2x("out", out.detach(), o32, o16)
    U.assert_within_2x("dq", g[:, 0], dq32, dq16)
    U.assert_within_2x("dk", g[:, 1], dk32, dk16)
    U.assert_within_2x("dv", g[:, 2], dv32, dv16)


def test_blocksparse_equals_dense_for_full_layout():
    """A layout of all ones computes exactly what the dense entry computes."""
    from flash_attn_b200 import flash_attn_cuda as fc
    from flash_attn_b200.flash_blocksparse_attn_interface import convert_blockmask
    seqlens = [512, 300]
    q, k, v, dout, cu, _ = U.make_varlen(seqlens, seqlens, 3, 64, torch.float16, seed=4)
    layout = torch.ones(32, 2, dtype=torch.int32, device="cuda")
    conv = convert_blockmask(layout, False)
    o_bs, lse_bs = fc.fwd_block(q, k, v, cu, cu, conv, 512, 512, 0.0, 0.125, False, False, None)
    o_d, lse_d = fc.fwd(q, k, v, cu, cu, 512, 512, 0.0, 0.125, False, False, False, None)
    assert torch.equal(o_bs, o_d)
    assert torch.equal(lse_bs[0, :, :512], lse_d[0, :, :512]) and torch.equal(lse_bs[1, :, :300], lse_d[1, :, :300])
    g_bs = [torch.empty_like(q) for _ in range(3)]
    g_d = [torch.empty_like(q) for _ in range(3)]
    fc.bwd_block(dout, q, k, v, o_bs, lse_bs, g_bs[0], g_bs[1], g_bs[2], cu, cu, conv, 512, 512, 0.0, 0.125, False, None)
    fc.bwd(dout, q, k, v, o_d, lse_d, g_d[0], g_d[1], g_d[2], cu, cu, 512, 512, 0.0, 0.125, False, False, None)
    torch.cuda.synchronize()
    fc.check_device_status()
    assert torch.equal(g_bs[1], g_d[1]) and torch.equal(g_bs[2], g_d[2])
    assert U.max_err(g_bs[0], g_d[0]) < 2e-3   # dq is summed with atomics in a run-dependent order


def test_rows_without_any_block_give_zero():
    from flash_attn_b200 import flash_attn_cuda as fc
    from flash_attn_b200.flash_blocksparse_attn_interface import convert_blockmask
    q, k, v, dout, cu, _ = U.make_varlen([512], [512], 2, 64, torch.float16, seed=8)
    layout = torch.ones(32, 2, dtype=torch.int32, device="cuda")
    layout[4:7, :] = 0  # query rows 64..111 attend to nothing
    conv = convert_blockmask(layout, False)
    out, lse = fc.fwd_block(q, k, v, cu, cu, conv, 512, 512, 0.0, 0.125, False, False, None)
    torch.cuda.synchronize()
    assert torch.all(out[64:112] == 0)
    assert torch.all(out[:64].float().abs().sum(-1) > 0)


def test_blocksparse_dropout_mask_dump_is_bit_exact():
    from flash_attn_b200 import _lib
    from flash_attn_b200.flash_blocksparse_attn_interface import convert_blockmask
    sq = sk = 700
    heads, p = 3, 0.15
    layout = _layout(5, 768, 0.4).cuda()
    conv = convert_blockmask(layout, False)
    cu = torch.tensor([0, 100, 100 + sq], dtype=torch.int32, device="cuda")  # batch entry 1 is the one dumped
    prm = _lib.FwdParams()
    prm.batch, prm.heads, prm.head_dim = 2, heads, 64
    prm.max_seqlen_q = prm.max_seqlen_k = 768
    prm.p_dropout = p
    prm.philox_seed, prm.philox_offset = 2024, 16
    prm.cu_seqlens_q = prm.cu_seqlens_k = cu.data_ptr()
    prm.blockmask = conv.data_ptr()
    prm.blockmask_rows, prm.blockmask_cols = conv.shape
    ws = torch.empty(_lib.lib.fa_blocksparse_workspace_bytes(2, conv.shape[0], conv.shape[1]), dtype=torch.uint8,
                     device="cuda")
    prm.bs_workspace, prm.bs_workspace_bytes = ws.data_ptr(), ws.numel()
    out = torch.zeros(sq, sk, dtype=torch.uint8, device="cuda")
    _lib.check(_lib.lib.fa_debug_dropout_mask(out.data_ptr(), 1, 2, ctypes.byref(prm), sq, sk,
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    conv_np = conv.cpu().numpy()
    it = orc.blocksparse_walk(conv_np, sq, sk)
    want = orc.dropout_keep_mask(2024, 16, 1, 2, heads, sq, sk, p, 256, False, bs_iter=it)
    vis = orc.blocksparse_allowed(conv_np, sq, sk)
    np.testing.assert_array_equal(out.cpu().numpy().astype(bool)[vis], want[vis])


def test_blocksparse_module_paths():
    from flash_attn_b200.flash_blocksparse_attention import FlashBlocksparseAttention, FlashBlocksparseMHA
    torch.manual_seed(0)
    layout = _layout(9, 512, 0.5)
    attn = FlashBlocksparseAttention(layout, attention_dropout=0.0, max_seq_length=512).cuda().eval()
    qkv = torch.randn(2, 512, 3, 2, 64, device="cuda", dtype=torch.float16)
    out, _ = attn(qkv)
    assert out.shape == (2, 512, 2, 64)
    cu = torch.tensor([0, 512, 1024], dtype=torch.int32, device="cuda")
    out2, _ = attn(qkv.reshape(1024, 3, 2, 64), cu_seqlens=cu, max_s=512)
    out3, _ = attn(qkv.reshape(1024, 3, 2, 64), cu_seqlens=cu, max_s=512, convert_mask=False)
    assert torch.equal(out.reshape(1024, 2, 64), out2) and torch.equal(out2, out3)
    mask = torch.ones(2, 512, dtype=torch.bool, device="cuda")
    mask[1, 300:] = False
    out4, _ = attn(qkv, key_padding_mask=mask)
    assert torch.equal(out4[0], out[0]) and torch.all(out4[1, 300:] == 0)
    mha = FlashBlocksparseMHA(128, 2, layout, max_seq_length=512, device="cuda", dtype=torch.float16)
    y, _ = mha(torch.randn(2, 512, 128, device="cuda", dtype=torch.float16))
    assert y.shape == (2, 512, 128) and not torch.isnan(y).any()


@pytest.mark.parametrize("p,lens", [(0.0, [1024, 700]), (0.15, [768, 300])])
def test_causal_blocksparse_parity(p, lens):
    """Causal + layout (not available in the reference, which asserts `not causal`): the result is
    standard attention under (layout AND key <= query), with the dropout mask of the block-sparse
    walk over the layout that convert_blockmask(causal=True) leaves."""
    from flash_attn_b200.flash_blocksparse_attn_interface import convert_blockmask
    from flash_attn_b200.sparsity_layouts import RandomLayout
    from flash_attn_b200 import flash_attn_cuda as fc
    S, heads = 1024, 2
    layout = RandomLayout(0.4, seed=7).make_layout(S).cuda()
    conv = convert_blockmask(layout, True)
    q, k, v, dout, cu, _ = U.make_varlen(lens, lens, heads, 64, torch.float16, seed=23)
    torch.cuda.manual_seed(3)
    out, lse, seed, offset = fc.fwd_block(q, k, v, cu, cu, conv, S, S, p, 0.125, True, False, None,
                                          return_philox=True)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    fc.bwd_block(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, conv, S, S, p, 0.125, True, None,
                 philox=(seed, offset))
    torch.cuda.synchronize()
    fc.check_device_status()
    conv_np = conv.cpu().numpy()
    allowed, keep = [], []
    for b, n in enumerate(lens):
        a = orc.blocksparse_allowed(conv_np, n, n)
        allowed.append(torch.from_numpy(a))
        if p > 0:
            it = orc.blocksparse_walk(conv_np, n, n)
            keep.append(torch.from_numpy(np.stack([
                orc.dropout_keep_mask(seed, offset, b, h, heads, n, n, p, 256, False, bs_iter=it)
                for h in range(heads)])))
    kw = dict(dropout_p=p, keep_masks=keep if p > 0 else None, allowed=allowed)
    o32, dq32, dk32, dv32 = U.oracle_cpu(q, k, v, dout, cu, cu, 0.125, True, **kw)
    o16, dq16, dk16, dv16 = U.oracle_cpu(q, k, v, dout, cu, cu, 0.125, True, dtype=torch.float16, **kw)
    U.assert_within_2x("out", out, o32, o16)
    U.assert_within_2x("dq", dq, dq32, dq16)
    U.assert_within_2x("dk", dk, dk32, dk16)
    U.assert_within_2x("dv", dv, dv32, dv16)
    # a mask converted without the causal pruning gives the same numbers when dropout is off
    if p == 0.0:
        conv_full = convert_blockmask(layout, False)
        out2, lse2 = fc.fwd_block(q, k, v, cu, cu, conv_full, S, S, 0.0, 0.125, True, False, None)
        torch.cuda.synchronize()
        assert torch.equal(out2, out)
        for b, n in enumerate(lens):
            assert torch.equal(lse2[b, :, :n], lse[b, :, :n])


def test_blocksparse_module_with_a_layout_generator_and_causal():
    from flash_attn_b200.flash_blocksparse_attention import FlashBlocksparseAttention
    from flash_attn_b200.sparsity_layouts import DenseLayout, SlidingWindowLayout
    from flash_attn_b200.flash_attention import FlashAttention
    torch.manual_seed(0)
    qkv = torch.randn(2, 512, 3, 2, 64, device="cuda", dtype=torch.float16)
    dense = FlashAttention().cuda().eval()
    sparse = FlashBlocksparseAttention(DenseLayout(), max_seq_length=512).cuda().eval()
    for causal in (False, True):
        a, _ = dense(qkv, causal=causal)
        b, _ = sparse(qkv, causal=causal)
        assert U.max_err(a, b) < 2e-3
    win = FlashBlocksparseAttention(SlidingWindowLayout(0, 0), max_seq_length=512).cuda().eval()
    c, _ = win(qkv)   # block-diagonal: the second 256 tokens do not see the first
    d, _ = dense(qkv[:, 256:].contiguous())
    assert U.max_err(c[:, 256:], d) < 2e-3
