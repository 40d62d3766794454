"""Row gather / scatter kernels behind unpad_input / pad_input (fa_gather_rows / fa_scatter_rows)
against framework indexing: copies must be bit-exact, padded rows exactly zero, gradients equal to
those of the indexing formulation (flash_attn/bert_padding.py:9-95 in the reference)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mask(batch, seqlen, seed):
    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(1, seqlen + 1, (batch,), generator=g)
    lengths[0] = seqlen
    return (torch.arange(seqlen)[None, :] < lengths[:, None]).cuda()


@pytest.mark.parametrize("dtype,dim", [(torch.float16, 768), (torch.bfloat16, 2304), (torch.float32, 4),
                                       (torch.float16, 8), (torch.float16, 520)])
def test_gather_scatter_match_indexing(dtype, dim):
    from flash_attn_b200 import bert_padding as bp
    batch, seqlen = 5, 67
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(batch * seqlen, dim, device="cuda", dtype=torch.float32, generator=g).to(dtype)
    mask = _mask(batch, seqlen, 11)
    idx = torch.nonzero(mask.flatten(), as_tuple=False).flatten()
    assert bp._kernel_path(x, idx)
    got = bp.gather_rows(x, idx)
    assert torch.equal(got, x.index_select(0, idx))
    back = bp.scatter_rows(got, idx, batch * seqlen)
    want = torch.zeros_like(x)
    want.index_copy_(0, idx, got)
    assert torch.equal(back, want)
    # unsorted indices are legal for the scatter
    perm = torch.randperm(idx.numel(), device="cuda", generator=g)
    back2 = bp.scatter_rows(got[perm], idx[perm], batch * seqlen)
    assert torch.equal(back2, want)


def test_rows_that_do_not_fit_the_kernels_use_indexing():
    from flash_attn_b200 import bert_padding as bp
    x = torch.randn(40, 5, device="cuda", dtype=torch.float16)   # 10-byte rows
    idx = torch.tensor([3, 7, 39], device="cuda")
    assert not bp._kernel_path(x, idx)
    assert torch.equal(bp.gather_rows(x, idx), x[idx])
    out = bp.scatter_rows(x[idx], idx, 40)
    assert torch.equal(out[idx], x[idx]) and float(out.abs().sum()) == float(x[idx].abs().sum())


def test_empty_and_out_of_range():
    from flash_attn_b200 import bert_padding as bp
    x = torch.randn(16, 64, device="cuda", dtype=torch.float16)
    none = torch.empty(0, dtype=torch.int64, device="cuda")
    assert bp.gather_rows(x, none).shape == (0, 64)
    assert float(bp.scatter_rows(x[:0], none, 16).abs().sum()) == 0.0
    # the C ABI tolerates a bad index: zero row on gather, skipped on scatter
    bad = torch.tensor([2, 99, -1, 5], device="cuda")
    got = bp.gather_rows(x, bad)
    assert torch.equal(got[0], x[2]) and torch.equal(got[3], x[5])
    assert float(got[1].abs().sum()) == 0.0 and float(got[2].abs().sum()) == 0.0
    out = bp.scatter_rows(x[:4].contiguous(), bad, 16)
    assert torch.equal(out[2], x[0]) and torch.equal(out[5], x[3])
    assert float(out.abs().sum()) == float(x[0].abs().sum() + x[3].abs().sum())


def test_unpad_pad_round_trip_and_gradients():
    from flash_attn_b200.bert_padding import pad_input, unpad_input
    batch, seqlen, dim = 4, 50, 96
    mask = _mask(batch, seqlen, 5)
    x = torch.randn(batch, seqlen, dim, device="cuda", dtype=torch.float16, requires_grad=True)
    packed, idx, cu, max_s = unpad_input(x, mask)
    assert cu.dtype == torch.int32 and int(cu[-1]) == int(mask.sum()) and max_s == seqlen
    y = pad_input(packed * 2, idx, batch, seqlen)
    want = torch.where(mask[..., None], x.detach() * 2, torch.zeros_like(x))
    assert torch.equal(y.detach(), want)
    w = torch.randn_like(y)
    (y * w).sum().backward()
    assert torch.equal(x.grad, torch.where(mask[..., None], 2 * w, torch.zeros_like(w)))
