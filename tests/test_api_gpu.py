"""The public functional API and modules (same names and arguments as the reference's flash_attn
package), exercised through autograd."""
import math

import pytest
import torch

from oracle import attention_oracle as orc
from tests import _util as U

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("causal", [False, True])
def test_three_layouts_agree_and_match_oracle(causal):
    from flash_attn_b200.flash_attn_interface import (flash_attn_func, flash_attn_unpadded_func,
                                                      flash_attn_unpadded_kvpacked_func,
                                                      flash_attn_unpadded_qkvpacked_func)
    seqlens = [257, 100]
    q, k, v, dout, cu, _ = U.make_varlen(seqlens, seqlens, 3, 64, torch.bfloat16, seed=41)
    qkv = torch.stack([q, k, v], 1).requires_grad_()
    out1 = flash_attn_unpadded_qkvpacked_func(qkv, cu, 257, 0.0, causal=causal)
    out1.backward(dout)
    q2 = q.clone().requires_grad_()
    kv2 = torch.stack([k, v], 1).requires_grad_()
    out2 = flash_attn_unpadded_kvpacked_func(q2, kv2, cu, cu, 257, 257, 0.0, causal=causal)
    out2.backward(dout)
    q3, k3, v3 = (t.clone().requires_grad_() for t in (q, k, v))
    out3 = flash_attn_unpadded_func(q3, k3, v3, cu, cu, 257, 257, 0.0, causal=causal)
    out3.backward(dout)
    out4 = flash_attn_func(qkv.detach(), cu, 0.0, 257, causal=causal)
    torch.cuda.synchronize()
    assert torch.equal(out1, out2) and torch.equal(out1, out3) and torch.equal(out1, out4)
    assert torch.equal(qkv.grad[:, 1], kv2.grad[:, 0]) and torch.equal(qkv.grad[:, 2], v3.grad)
    assert U.max_err(qkv.grad[:, 0], q3.grad) < 5e-3
    o32, dq32, dk32, dv32 = U.oracle_cpu(q, k, v, dout, cu, cu, 64 ** -0.5, causal)
    o16, dq16, dk16, dv16 = U.oracle_cpu(q, k, v, dout, cu, cu, 64 ** -0.5, causal, dtype=torch.bfloat16)
    U.assert_within_2x("out", out1.detach(), o32, o16)
    U.assert_within_2x("dq", qkv.grad[:, 0], dq32, dq16)
    U.assert_within_2x("dk", qkv.grad[:, 1], dk32, dk16)
    U.assert_within_2x("dv", qkv.grad[:, 2], dv32, dv16)


def test_cross_attention_with_different_lengths():
    from flash_attn_b200.flash_attn_interface import flash_attn_unpadded_kvpacked_func
    sq, sk = [60, 200], [333, 90]
    q, k, v, dout, cu_q, cu_k = U.make_varlen(sq, sk, 2, 128, torch.float16, seed=43)
    qg = q.clone().requires_grad_()
    kv = torch.stack([k, v], 1).requires_grad_()
    out, lse, _ = flash_attn_unpadded_kvpacked_func(qg, kv, cu_q, cu_k, 200, 333, 0.0, softmax_scale=0.07,
                                                    return_attn_probs=False), None, None
    out.backward(dout)
    torch.cuda.synchronize()
    o32, dq32, dk32, dv32 = U.oracle_cpu(q, k, v, dout, cu_q, cu_k, 0.07, False)
    o16, dq16, dk16, dv16 = U.oracle_cpu(q, k, v, dout, cu_q, cu_k, 0.07, False, dtype=torch.float16)
    U.assert_within_2x("out", out.detach(), o32, o16)
    U.assert_within_2x("dq", qg.grad, dq32, dq16)
    U.assert_within_2x("dk", kv.grad[:, 0], dk32, dk16)
    U.assert_within_2x("dv", kv.grad[:, 1], dv32, dv16)


def test_dropout_autograd_regenerates_the_forward_mask():
    """The functions save the generator state in forward and restore it around backward, so the
    gradients correspond to the mask of the forward, and the generator ends up advanced once."""
    from flash_attn_b200.flash_attn_interface import flash_attn_unpadded_qkvpacked_func
    seqlens = [300, 180]
    heads, d, p = 2, 64, 0.1
    q, k, v, dout, cu, _ = U.make_varlen(seqlens, seqlens, heads, d, torch.float16, seed=47)
    qkv = torch.stack([q, k, v], 1).requires_grad_()
    seed = 2025
    torch.cuda.manual_seed(seed)
    gen = torch.cuda.default_generators[torch.cuda.current_device()]
    out = flash_attn_unpadded_qkvpacked_func(qkv, cu, 300, p)
    off_after_fwd = gen.get_offset()
    _ = torch.rand(10, device="cuda")  # other random work between forward and backward
    off_before_bwd = gen.get_offset()
    out.backward(dout)
    torch.cuda.synchronize()
    assert off_after_fwd == orc.philox_increment(d, 300, 300)
    assert gen.get_offset() == off_before_bwd  # backward leaves the generator where it found it
    n = orc.mask_block_n(d, 300)
    masks = []
    import numpy as np
    for b, s in enumerate(seqlens):
        masks.append(torch.from_numpy(np.stack([orc.dropout_keep_mask(seed, 0, b, h, heads, s, s, p, n)
                                                for h in range(heads)])))
    o32, dq32, dk32, dv32 = U.oracle_cpu(q, k, v, dout, cu, cu, d ** -0.5, False, p, masks)
    o16, dq16, dk16, dv16 = U.oracle_cpu(q, k, v, dout, cu, cu, d ** -0.5, False, p, masks, dtype=torch.float16)
    U.assert_within_2x("out", out.detach(), o32, o16)
    U.assert_within_2x("dq", qkv.grad[:, 0], dq32, dq16)
    U.assert_within_2x("dk", qkv.grad[:, 1], dk32, dk16)
    U.assert_within_2x("dv", qkv.grad[:, 2], dv32, dv16)


def test_flash_attention_module_three_input_paths():
    from flash_attn_b200.flash_attention import FlashAttention, FlashMHA
    torch.manual_seed(1)
    attn = FlashAttention(attention_dropout=0.1).cuda().eval()  # eval: dropout off
    qkv = torch.randn(3, 200, 3, 4, 32, device="cuda", dtype=torch.float16)
    out, w = attn(qkv, causal=True)
    assert w is None and out.shape == (3, 200, 4, 32)
    cu = torch.arange(0, 4 * 200, 200, dtype=torch.int32, device="cuda")
    out2, _ = attn(qkv.reshape(600, 3, 4, 32), cu_seqlens=cu, max_s=200, causal=True)
    assert torch.equal(out.reshape(600, 4, 32), out2)
    lengths = torch.tensor([200, 57, 130], device="cuda")
    mask = torch.arange(200, device="cuda")[None, :] < lengths[:, None]
    out3, _ = attn(qkv, key_padding_mask=mask, causal=True)
    assert torch.equal(out3[0], out[0]) and torch.all(out3[1, 57:] == 0)
    ref = orc.attention_ref(qkv.cpu(), mask.cpu(), 0.0, upcast=True, causal=True)
    assert U.max_err(out3[mask], ref[mask.cpu()]) < 3e-3
    with pytest.raises(AssertionError):
        attn(qkv.bfloat16())
    mha = FlashMHA(256, 4, use_rotary_emb="1d", causal=True, device="cuda", dtype=torch.float16)
    y, _ = mha(torch.randn(2, 64, 256, device="cuda", dtype=torch.float16), key_padding_mask=None)
    assert y.shape == (2, 64, 256) and not torch.isnan(y).any()


@pytest.mark.parametrize("causal,p", [(False, 0.0), (True, 0.2)])
def test_return_attn_probs_gives_probabilities_and_dropout_signs(causal, p):
    """return_attn_probs=True: S_dmask holds the softmax probabilities in (batch, heads, seqlen_q,
    seqlen_k) order with a negative sign where dropout dropped the entry."""
    import numpy as np
    from flash_attn_b200.flash_attn_interface import flash_attn_unpadded_qkvpacked_func
    seqlens = [150, 260]
    heads, d = 2, 64
    q, k, v, dout, cu, _ = U.make_varlen(seqlens, seqlens, heads, d, torch.float16, seed=53)
    qkv = torch.stack([q, k, v], 1)
    seed = 77
    torch.cuda.manual_seed(seed)
    out, lse, s_dmask = flash_attn_unpadded_qkvpacked_func(qkv, cu, 260, p, causal=causal, return_attn_probs=True)
    torch.cuda.synchronize()
    assert s_dmask.shape == (2, heads, 272, 512) and lse.shape == (2, heads, 272)
    n = orc.mask_block_n(d, 260)
    start = 0
    for b, s in enumerate(seqlens):
        qb, kb = q[start:start + s].float().cpu(), k[start:start + s].float().cpu()
        scores = torch.einsum("thd,shd->hts", qb, kb) * d ** -0.5
        if causal:
            scores = scores.masked_fill(torch.triu(torch.ones(s, s, dtype=torch.bool), 1), float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        got = s_dmask[b, :, :s, :s].float().cpu()
        assert (got.abs() - probs).abs().max().item() < 2e-3
        if p > 0:
            keep = np.stack([orc.dropout_keep_mask(seed, 0, b, h, heads, s, s, p, n, causal) for h in range(heads)])
            visible = probs.numpy() > 1e-6
            np.testing.assert_array_equal((got.numpy() >= 0)[visible], keep[visible])
        else:
            assert (got >= 0).all()
        start += s
