"""CPU tests of the oracle against the golden fixtures produced from the reference's own Python
code (tests/golden/make_golden.py), plus self-consistency checks of the Philox restatement."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_golden as mg  # noqa: E402  (only its pure helpers and case tables are used here)


@pytest.mark.parametrize("name", list(mg.ATTENTION_CASES))
def test_attention_ref_matches_reference_outputs(golden_dir, name):
    gold = np.load(os.path.join(golden_dir, "attention_ref.npz"))
    seed, b, s, h, d, lengths, causal = mg.ATTENTION_CASES[name]
    qkv, dout, mask = mg.attention_inputs(seed, b, s, h, d, lengths)
    qkv = qkv.clone().requires_grad_()
    out = orc.attention_ref(qkv, mask, 0.0, upcast=True, causal=causal)
    (out * dout).sum().backward()
    o_np, g_np = out.detach().numpy(), qkv.grad.numpy()
    if name + "/out" in gold:
        np.testing.assert_allclose(o_np, gold[name + "/out"], rtol=0, atol=2e-6)
        np.testing.assert_allclose(g_np, gold[name + "/dqkv"], rtol=0, atol=2e-5)
    else:
        np.testing.assert_allclose(o_np.reshape(-1)[::37], gold[name + "/out_stride37"], rtol=0, atol=2e-6)
        np.testing.assert_allclose(g_np.reshape(-1)[::37], gold[name + "/dqkv_stride37"], rtol=0, atol=2e-5)
        assert abs(o_np.astype(np.float64).sum() - float(gold[name + "/out_sum"])) < 1e-2
        assert abs(np.abs(g_np.astype(np.float64)).sum() - float(gold[name + "/dqkv_abs_sum"])) < 1e-1


@pytest.mark.parametrize("name", list(mg.ATTENTION_CASES))
def test_varlen_oracle_agrees_with_padded_oracle(name):
    """The packed (varlen) oracle used by the GPU parity tests equals the padded attention_ref on
    the valid tokens: outputs, LSE and gradients."""
    seed, b, s, h, d, lengths, causal = mg.ATTENTION_CASES[name]
    qkv, dout, mask = mg.attention_inputs(seed, b, s, h, d, lengths)
    lengths = lengths or [s] * b
    qkv_p = qkv.clone().requires_grad_()
    out_p = orc.attention_ref(qkv_p, mask, 0.0, upcast=True, causal=causal)
    (out_p * dout * mask[:, :, None, None]).sum().backward()
    idx = mask.flatten().nonzero().flatten()
    packed = qkv.reshape(b * s, 3, h, d)[idx]
    cu = np.concatenate([[0], np.cumsum(lengths)]).tolist()
    out, dq, dk, dv = orc.attention_varlen_grads(
        packed[:, 0], packed[:, 1], packed[:, 2], dout.reshape(b * s, h, d)[idx], cu, cu,
        d ** -0.5, causal=causal)
    torch.testing.assert_close(out, out_p.detach().reshape(b * s, h, d)[idx], rtol=0, atol=3e-6)
    gp = qkv_p.grad.reshape(b * s, 3, h, d)[idx]
    torch.testing.assert_close(dq, gp[:, 0], rtol=0, atol=3e-5)
    torch.testing.assert_close(dk, gp[:, 1], rtol=0, atol=3e-5)
    torch.testing.assert_close(dv, gp[:, 2], rtol=0, atol=3e-5)


@pytest.mark.parametrize("name", list(mg.BLOCKMASK_CASES))
def test_convert_blockmask_restatement(golden_dir, name):
    gold = np.load(os.path.join(golden_dir, "convert_blockmask.npz"))
    layout = mg.blockmask_layout(*mg.BLOCKMASK_CASES[name]).numpy()
    np.testing.assert_array_equal(orc.convert_blockmask_loops(layout), gold[name])


def test_blocksparse_walk_covers_layout(golden_dir):
    gold = np.load(os.path.join(golden_dir, "convert_blockmask.npz"))
    layout = mg.blockmask_layout(*mg.BLOCKMASK_CASES["bm_16x4"]).numpy()
    it = orc.blocksparse_walk(gold["bm_16x4"], 16 * 16)
    np.testing.assert_array_equal(it >= 0, layout.T != 0)
    # iteration numbers are a permutation of 0..nnz-1 in key-block-major, row-ascending order
    visited = it[it >= 0]
    assert sorted(visited.tolist()) == list(range(int((layout != 0).sum())))
    assert np.all(np.diff(it[0][it[0] >= 0]) > 0)
    # a shorter sequence stops at the first row block beyond it
    it_short = orc.blocksparse_walk(gold["bm_16x4"], 40)
    assert np.all(it_short[:, 3:] == -1)


def test_philox_counter_and_key_sensitivity():
    """Bijection-style sanity checks of the Philox restatement: distinct counters / keys give
    distinct outputs, the function is deterministic, and 7 and 10 rounds differ."""
    ctr = np.zeros((64, 4), dtype=np.uint64)
    ctr[:, 0] = np.arange(64)
    a = orc.philox4x32(ctr, (123, 456), rounds=7)
    b = orc.philox4x32(ctr, (123, 456), rounds=7)
    np.testing.assert_array_equal(a, b)
    assert len({tuple(x) for x in a.tolist()}) == 64
    c = orc.philox4x32(ctr, (124, 456), rounds=7)
    assert not np.array_equal(a, c)
    d = orc.philox4x32(ctr, (123, 456), rounds=10)
    assert not np.array_equal(a, d)
    # output words are roughly uniform
    big = np.zeros((1 << 14, 4), dtype=np.uint64)
    big[:, 2] = np.arange(1 << 14)
    out = orc.philox4x32(big, (1, 2), rounds=7).astype(np.float64) / 2 ** 32
    assert abs(out.mean() - 0.5) < 0.01


def test_philox_single_round_by_hand():
    """One round, computed independently with Python integers."""
    c = [0x01234567, 0x89ABCDEF, 0x0F1E2D3C, 0x4B5A6978]
    k = (0xDEADBEEF, 0x0BADF00D)
    p0 = 0xD2511F53 * c[0]
    p1 = 0xCD9E8D57 * c[2]
    want = [(p1 >> 32) ^ c[1] ^ k[0], p1 & 0xFFFFFFFF, (p0 >> 32) ^ c[3] ^ k[1], p0 & 0xFFFFFFFF]
    got = orc.philox4x32(np.array([c], dtype=np.uint64), k, rounds=1)[0]
    assert [int(x) for x in got] == want


@pytest.mark.parametrize("p", [0.1, 0.17, 0.5])
def test_dropout_mask_rate_and_structure(p):
    m = orc.dropout_keep_mask(seed=42, offset=8, batch_idx=1, head_idx=2, heads=4, seqlen_q=256,
                              seqlen_k=512, dropout_p=p, block_n=256)
    assert m.shape == (256, 512)
    assert abs(m.mean() - (1 - p)) < 0.01
    # head / batch / offset all change the mask
    m2 = orc.dropout_keep_mask(42, 8, 1, 3, 4, 256, 512, p, 256)
    m3 = orc.dropout_keep_mask(42, 12, 1, 2, 4, 256, 512, p, 256)
    assert (m != m2).mean() > 0.05 and (m != m3).mean() > 0.05
    # N = 128 and N = 256 layouts agree on the first 128 keys of the first row tile only
    m128 = orc.dropout_keep_mask(42, 8, 1, 2, 4, 256, 512, p, 128)
    np.testing.assert_array_equal(m128[:16, :128], m[:16, :128])


def test_dropout_mask_causal_iteration_count():
    """Causal walks skip row tiles above the diagonal, so the counter of a given (key block, row
    tile) differs from the non-causal one except in the first key block."""
    a = orc.dropout_keep_mask(7, 0, 0, 0, 1, 512, 512, 0.2, 256, causal=False)
    c = orc.dropout_keep_mask(7, 0, 0, 0, 1, 512, 512, 0.2, 256, causal=True)
    np.testing.assert_array_equal(a[:, :256], c[:, :256])
    assert (a[256:, 256:] != c[256:, 256:]).mean() > 0.05


def test_block_size_rule_and_increment():
    assert orc.mask_block_n(64, 128) == 128
    assert orc.mask_block_n(64, 129) == 256
    assert orc.mask_block_n(128, 4096) == 128
    assert orc.mask_block_n(32, 512) == 256
    assert orc.mask_block_n(64, 100, blocksparse=True) == 256
    # STEPS * MMAS_N * 8 * loop_steps
    assert orc.philox_increment(64, 128, 128) == 8 * 2 * 8 * 1
    assert orc.philox_increment(64, 512, 512) == 32 * 4 * 8 * 2
    assert orc.philox_increment(128, 1000, 1000) == 63 * 2 * 8 * 8
    assert orc.dropout_threshold(0.1) == int(np.floor(float(np.float32(1) - np.float32(0.1)) * 65535.0))


def test_bert_padding_matches_reference(golden_dir):
    from flash_attn_b200 import bert_padding as bp
    gold = np.load(os.path.join(golden_dir, "bert_padding.npz"))
    g = torch.Generator().manual_seed(21)
    x = torch.randn(4, 12, 8, generator=g)
    mask = torch.arange(12)[None, :] < torch.tensor([12, 5, 1, 9])[:, None]
    x_unpad, indices, cu, max_s = bp.unpad_input(x, mask)
    np.testing.assert_array_equal(x_unpad.numpy(), gold["x_unpad"])
    np.testing.assert_array_equal(indices.numpy(), gold["indices"])
    np.testing.assert_array_equal(cu.numpy(), gold["cu_seqlens"])
    assert cu.dtype == torch.int32 and max_s == int(gold["max_s"])
    np.testing.assert_array_equal(bp.pad_input(x_unpad, indices, 4, 12).numpy(), gold["x_pad"])
    # gradients flow back to the valid tokens only
    xg = x.clone().requires_grad_()
    u, idx, _, _ = bp.unpad_input(xg, mask)
    bp.pad_input(u * 2.0, idx, 4, 12).sum().backward()
    np.testing.assert_array_equal(xg.grad.numpy(), 2.0 * mask[:, :, None].expand_as(x).numpy())


def test_attention_flops_convention():
    f = orc.attention_flops([128, 128], [128, 128], 12, 64)
    assert f == 4 * 2 * 12 * 128 * 128 * 64
    assert orc.attention_flops([128], [128], 1, 64, causal=True) == 4 * 128 * 128 * 64 / 2
    assert orc.attention_flops([128], [128], 1, 64, mode="fwd_bwd") == 3.5 * 4 * 128 * 128 * 64
