"""The closed-form dropout mask (oracle/attention_oracle.py:dropout_keep_mask, the formula the CUDA
kernels implement) against a literal walk of the reference's thread / loop structure
(oracle/dropout_layout_sim.py): forward enumeration (128 threads, two streams), backward enumeration
(256 threads, one stream), key blocks of 128 and 256, causal or not, ragged lengths, block-sparse."""
import numpy as np
import pytest

from oracle import attention_oracle as ao
from oracle.dropout_layout_sim import simulate_keep_mask

SEED = 0x1234_5678_9ABC_DEF1
OFFSET = 4 * 977


def _rounded_k(max_k, n, sparse=False):
    """params.seqlen_k as the reference's host entries round it (csrc/flash_attn/fmha_api.cpp:232-241,
    :499-500)."""
    if not sparse:
        if max_k <= 128:
            return 128
        if max_k <= 256:
            return 256
    base = 256 if sparse else n
    return (max_k + base - 1) // base * base


def _compare(sim, closed, sq, sk):
    got = sim[:sq, :sk]
    assert (got != 255).all(), "the walk left entries of the sequence without a decision"
    np.testing.assert_array_equal(got.astype(bool), closed)


@pytest.mark.parametrize("backward", [False, True])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("n,sq,sk,max_q,max_k", [
    (128, 128, 128, 128, 128),     # single key block (the seqlen_k == N branch)
    (128, 100, 77, 128, 128),      # ragged inside one block
    (128, 300, 513, 320, 520),     # head_dim 128 rule: N = 128, several key blocks
    (256, 256, 256, 256, 256),
    (256, 513, 1000, 600, 1024),   # ragged, actual < max (a shorter sequence of a batch)
    (256, 1000, 333, 1000, 1000),  # more queries than keys
    (256, 31, 700, 64, 700),
])
def test_dense_walk_equals_closed_form(backward, causal, n, sq, sk, max_q, max_k):
    thr = ao.dropout_threshold(0.17)
    heads, b, h = 5, 2, 3
    sim = simulate_keep_mask(SEED, OFFSET, b, h, heads, sq, sk, max_q, _rounded_k(max_k, n), thr, n,
                             causal=causal, backward=backward)
    closed = ao.dropout_keep_mask(SEED, OFFSET, b, h, heads, sq, sk, 0.17, n, causal=causal)
    if causal:
        # tiles above the diagonal are never visited (their probabilities are zero anyway):
        # compare where the walk drew, and require that it drew everything at or below the diagonal
        got = sim[:sq, :sk]
        i, j = np.arange(sq)[:, None], np.arange(sk)[None, :]
        assert (got[j <= i + 0 * j] != 255).all()
        drawn = got != 255
        np.testing.assert_array_equal(got[drawn].astype(bool), closed[drawn])
    else:
        _compare(sim, closed, sq, sk)


@pytest.mark.parametrize("backward", [False, True])
@pytest.mark.parametrize("sq,sk,max_s,density,seed", [
    (512, 512, 512, 0.5, 0),
    (1024, 1024, 1024, 0.25, 1),
    (700, 700, 768, 0.4, 2),     # ragged: the walk stops at the first row block past the sequence
    (200, 900, 1024, 0.6, 3),
])
def test_blocksparse_walk_equals_closed_form(backward, sq, sk, max_s, density, seed):
    rng = np.random.default_rng(seed)
    nk, nr = max_s // 256, max_s // 16
    blocks = rng.random((max_s // 256, nk)) < density
    blocks |= np.eye(max_s // 256, nk, dtype=bool)
    layout = np.repeat(blocks, 16, axis=0)              # (16-row blocks, key blocks)
    blockmask = ao.convert_blockmask_loops(layout)      # (key blocks, slots)
    assert blockmask.shape == (nk, nr)
    thr = ao.dropout_threshold(0.1)
    heads, b, h = 3, 1, 2
    sim = simulate_keep_mask(SEED, OFFSET, b, h, heads, sq, sk, max_s, max_s, thr, 256,
                             backward=backward, blockmask=blockmask)
    it = ao.blocksparse_walk(blockmask, sq, sk)
    closed = ao.dropout_keep_mask(SEED, OFFSET, b, h, heads, sq, sk, 0.1, 256, bs_iter=it)
    allowed = ao.blocksparse_allowed(blockmask, sq, sk)
    got = sim[:sq, :sk]
    # the walk draws exactly the blocks the layout keeps ...
    np.testing.assert_array_equal(got != 255, allowed)
    # ... and draws what the closed form says
    np.testing.assert_array_equal(got[allowed].astype(bool), closed[allowed])


def test_forward_and_backward_enumerations_agree():
    thr = ao.dropout_threshold(0.3)
    for n, sq, sk in [(128, 200, 300), (256, 300, 600)]:
        f = simulate_keep_mask(SEED, 0, 0, 1, 2, sq, sk, sq, _rounded_k(sk, n), thr, n)
        g = simulate_keep_mask(SEED, 0, 0, 1, 2, sq, sk, sq, _rounded_k(sk, n), thr, n, backward=True)
        np.testing.assert_array_equal(f, g)
