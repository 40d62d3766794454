"""Layout generators (flash_attn_b200/sparsity_layouts.py) and convert_blockmask with causal=True,
checked on CPU against the loop restatement of the reference's convert_blockmask."""
import numpy as np
import pytest
import torch

from oracle import attention_oracle as ao


def _layouts():
    from flash_attn_b200 import sparsity_layouts as sl
    return [sl.DenseLayout(), sl.FixedLayout(4, 1), sl.FixedLayout(2, 2), sl.SlidingWindowLayout(1, 1),
            sl.SlidingWindowLayout(2, 0), sl.RandomLayout(0.25, seed=3)]


@pytest.mark.parametrize("seq_len", [256, 1024, 2048])
def test_layout_shapes_and_diagonal(seq_len):
    for gen in _layouts():
        layout = gen.make_layout(seq_len)
        assert layout.shape == (seq_len // 16, seq_len // 256) and layout.dtype == torch.int32
        assert set(layout.unique().tolist()) <= {0, 1}
        blocks = layout.reshape(seq_len // 256, 16, seq_len // 256)
        assert (blocks == blocks[:, :1]).all(), "a 256-row block is 16 identical layout rows"
        assert bool(torch.diagonal(blocks[:, 0]).all()), "the diagonal is kept"
    with pytest.raises(ValueError):
        _layouts()[0].make_layout(300)


def test_layout_patterns():
    from flash_attn_b200 import sparsity_layouts as sl
    n = 8
    dense = sl.DenseLayout().make_layout(256 * n)
    assert int(dense.sum()) == 16 * n * n
    win = sl.SlidingWindowLayout(1, 0).make_layout(256 * n)[::16]
    i = torch.arange(n)
    assert torch.equal(win.bool(), (i[:, None] - i[None, :]).abs() <= 1)
    fixed = sl.FixedLayout(4, 1).make_layout(256 * n)[::16].bool()
    assert fixed[5, 4] and fixed[5, 7] and fixed[5, 3] and not fixed[5, 2]   # window {4..7}, global columns 3 and 7
    a, b = sl.RandomLayout(0.3, seed=1).make_layout(2048), sl.RandomLayout(0.3, seed=1).make_layout(2048)
    assert torch.equal(a, b)


@pytest.mark.parametrize("causal", [False, True])
def test_convert_blockmask_matches_the_loop_restatement(causal):
    from flash_attn_b200.flash_blocksparse_attn_interface import convert_blockmask
    for gen in _layouts():
        layout = gen.make_layout(1024)
        got = convert_blockmask(layout, causal).numpy()
        ref_layout = layout.numpy().copy()
        if causal:
            r = np.arange(ref_layout.shape[0])[:, None]
            c = np.arange(ref_layout.shape[1])[None, :]
            ref_layout[256 * c > 16 * r + 15] = 0
        np.testing.assert_array_equal(got, ao.convert_blockmask_loops(ref_layout))
