"""Dropout: the mask the kernels apply is bit-exact with the CPU restatement of the reference's
Philox layout, and outputs / gradients with dropout match the oracle with that mask injected."""
import ctypes
import math

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from tests import _util as U

pytestmark = pytest.mark.gpu


def _fc():
    from flash_attn_b200 import flash_attn_cuda
    return flash_attn_cuda


def _oracle_masks(seed, offset, sq_list, sk_list, heads, d, p, causal, max_sk):
    n = orc.mask_block_n(d, max_sk)
    masks = []
    for b, (sq, sk) in enumerate(zip(sq_list, sk_list)):
        m = np.stack([orc.dropout_keep_mask(seed, offset, b, h, heads, sq, sk, p, n, causal)
                      for h in range(heads)])
        masks.append(torch.from_numpy(m))
    return masks


@pytest.mark.parametrize("d,sq,sk,p,causal", [
    (64, 128, 128, 0.1, False),
    (64, 300, 300, 0.17, False),
    (64, 520, 700, 0.1, True),
    (128, 260, 390, 0.5, False),
    (32, 77, 129, 0.25, True),
])
def test_mask_dump_is_bit_exact(d, sq, sk, p, causal):
    """The device code that generates keep bits (shared by the attention kernels) against the
    CPU restatement, for one (batch, head) pair."""
    from flash_attn_b200 import _lib
    heads, b_idx, h_idx = 5, 2, 3
    seed, offset = 0x1234567890AB, 40
    out = torch.zeros(sq, sk, dtype=torch.uint8, device="cuda")
    prm = _lib.FwdParams()
    prm.heads, prm.head_dim, prm.max_seqlen_k = heads, d, sk
    prm.p_dropout, prm.is_causal = p, int(causal)
    prm.philox_seed, prm.philox_offset = seed, offset
    _lib.check(_lib.lib.fa_debug_dropout_mask(out.data_ptr(), b_idx, h_idx, ctypes.byref(prm), sq, sk,
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    want = orc.dropout_keep_mask(seed, offset, b_idx, h_idx, heads, sq, sk, p, orc.mask_block_n(d, sk), causal)
    np.testing.assert_array_equal(out.cpu().numpy().astype(bool), want)


@pytest.mark.parametrize("d,dtype,causal,sq,sk,p", [
    (64, torch.float16, False, [128], [128], 0.1),
    (64, torch.float16, False, [300, 200], [300, 200], 0.1),
    (64, torch.bfloat16, True, [384], [384], 0.2),
    (128, torch.bfloat16, False, [260], [390], 0.1),
    (32, torch.float16, False, [100], [260], 0.3),
])
def test_forward_mask_seen_through_one_hot_values(d, dtype, causal, sq, sk, p):
    """Bit-exactness of the mask inside the forward kernel: with V one-hot on a window of `d`
    keys, O[i, c] is the dropped-out probability of key window_start + c, so O != 0 exactly where
    the key was kept (and visible)."""
    fc = _fc()
    heads = 2
    q, k, v, dout, cu_q, cu_k = U.make_varlen(sq, sk, heads, d, dtype, seed=11)
    q, k = q * 0.1, k * 0.1  # keep probabilities far from underflow
    seed = 777
    for win in range(0, max(sk), d):
        v.zero_()
        start = 0
        for n in sk:
            for c in range(d):
                if win + c < n:
                    v[start + win + c, :, c] = 1.0
            start += n
        torch.cuda.manual_seed(seed)
        out, _ = fc.fwd(q, k, v, cu_q, cu_k, max(sq), max(sk), p, d ** -0.5, False, causal, False, None)
        masks = _oracle_masks(seed, 0, sq, sk, heads, d, p, causal, max(sk))
        qs = 0
        for b, (nq, nk) in enumerate(zip(sq, sk)):
            w = min(d, max(0, nk - win))
            if w > 0:
                got = (out[qs:qs + nq, :, :w] != 0).permute(1, 0, 2).cpu()  # heads, nq, w
                want = masks[b][:, :, win:win + w].clone()
                if causal:
                    vis = torch.arange(win, win + w)[None, :] <= torch.arange(nq)[:, None]
                    want &= vis[None]
                assert torch.equal(got, want), "window %d of batch %d" % (win, b)
            qs += nq
    fc.check_device_status()


@pytest.mark.parametrize("d,dtype,causal,sq,sk,p", [
    (64, torch.float16, False, [128], [128], 0.1),
    (64, torch.float16, True, [300, 200], [300, 200], 0.1),
    (128, torch.bfloat16, False, [260], [390], 0.1),
])
def test_backward_mask_seen_through_one_hot_grads(d, dtype, causal, sq, sk, p):
    """Same idea for the backward kernel: with dO one-hot on a window of `d` queries,
    dV[j, c] = P~[window_start + c, j] / p_keep, non-zero exactly where (query, key) was kept."""
    fc = _fc()
    heads = 2
    q, k, v, dout, cu_q, cu_k = U.make_varlen(sq, sk, heads, d, dtype, seed=13)
    q, k = q * 0.1, k * 0.1
    seed = 4242
    torch.cuda.manual_seed(seed)
    out, lse = fc.fwd(q, k, v, cu_q, cu_k, max(sq), max(sk), p, d ** -0.5, False, causal, False, None)
    masks = _oracle_masks(seed, 0, sq, sk, heads, d, p, causal, max(sk))
    for win in range(0, max(sq), d):
        dout.zero_()
        start = 0
        for n in sq:
            for c in range(d):
                if win + c < n:
                    dout[start + win + c, :, c] = 1.0
            start += n
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        torch.cuda.manual_seed(seed)  # the backward reads (seed, offset) of the forward
        fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, max(sq), max(sk), p, d ** -0.5, False,
               causal, None)
        ks = 0
        for b, (nq, nk) in enumerate(zip(sq, sk)):
            w = min(d, max(0, nq - win))
            if w > 0:
                got = (dv[ks:ks + nk, :, :w] != 0).permute(1, 2, 0).cpu()  # heads, w (queries), nk
                want = masks[b][:, win:win + w, :].clone()
                if causal:
                    vis = torch.arange(nk)[None, :] <= torch.arange(win, win + w)[:, None]
                    want &= vis[None]
                assert torch.equal(got, want), "window %d of batch %d" % (win, b)
            ks += nk
    fc.check_device_status()


@pytest.mark.parametrize("d,dtype,causal,sq,sk,p", [
    (64, torch.float16, False, [300, 77], [300, 77], 0.1),
    (64, torch.bfloat16, True, [513], [513], 0.1),
    (128, torch.bfloat16, False, [260], [390], 0.25),
    (32, torch.float16, True, [200, 130], [100, 513], 0.1),
])
def test_dropout_numerics_with_injected_mask(d, dtype, causal, sq, sk, p):
    fc = _fc()
    heads = 2
    q, k, v, dout, cu_q, cu_k = U.make_varlen(sq, sk, heads, d, dtype, seed=17)
    scale = d ** -0.5
    seed = 99
    torch.cuda.manual_seed(seed)
    gen = torch.cuda.default_generators[torch.cuda.current_device()]
    out, lse = fc.fwd(q, k, v, cu_q, cu_k, max(sq), max(sk), p, scale, False, causal, False, None)
    assert gen.get_offset() == orc.philox_increment(d, max(sq), max(sk))
    torch.cuda.manual_seed(seed)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, max(sq), max(sk), p, scale, False, causal, None)
    torch.cuda.synchronize()
    fc.check_device_status()
    masks = _oracle_masks(seed, 0, sq, sk, heads, d, p, causal, max(sk))
    o32, dq32, dk32, dv32 = U.oracle_cpu(q, k, v, dout, cu_q, cu_k, scale, causal, p, masks)
    o16, dq16, dk16, dv16 = U.oracle_cpu(q, k, v, dout, cu_q, cu_k, scale, causal, p, masks, dtype=dtype)
    U.assert_within_2x("out", out, o32, o16)
    U.assert_within_2x("dq", dq, dq32, dq16)
    U.assert_within_2x("dk", dk, dk32, dk16)
    U.assert_within_2x("dv", dv, dv32, dv16)
    # LSE is that of the un-dropped softmax
    lses = U.oracle_lse(q, k, v, cu_q, cu_k, scale, causal)
    for b, n in enumerate(sq):
        assert U.max_err(lse[b, :, :n], lses[b]) < 2e-4


@pytest.mark.parametrize("seed,offset", [(0, 0), (0x9E3779B97F4A7C15, 4096), (12345, 2 ** 34 + 8)])
def test_philox_generator_against_curand(seed, offset):
    """Pins the round function, key schedule and counter / key layout: at 10 rounds both this
    library's device code and the numpy restatement in the oracle equal cuRAND's Philox4_32_10;
    at the 7 rounds the attention kernels use, device code and restatement agree."""
    from flash_attn_b200 import _lib
    n = 1000
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def run(rounds, use_curand):
        out = torch.zeros(n, 4, dtype=torch.int32, device="cuda")
        _lib.check(_lib.lib.fa_debug_philox(out.data_ptr(), n, seed, offset, rounds, use_curand, stream))
        return out.cpu().numpy().view(np.uint32)

    counter = np.zeros((n, 4), dtype=np.uint64)
    counter[:, 0] = (offset // 4) & 0xFFFFFFFF
    counter[:, 1] = (offset // 4) >> 32
    counter[:, 2] = np.arange(n)
    key = (seed & 0xFFFFFFFF, seed >> 32)
    cur = run(10, 1)
    np.testing.assert_array_equal(run(10, 0), cur)
    np.testing.assert_array_equal(orc.philox4x32(counter, key, rounds=10), cur)
    np.testing.assert_array_equal(orc.philox4x32(counter, key, rounds=7), run(7, 0))
    assert not np.array_equal(run(7, 0), cur)


@pytest.mark.parametrize("d,dtype,offset", [(64, torch.float16, 2 ** 34 + 8), (128, torch.bfloat16, 2 ** 34 + 8),
                                            (64, torch.float16, 2 ** 34 - 16), (128, torch.bfloat16, 2 ** 34 - 16)])
def test_mask_with_high_counter_and_subsequence_words(d, dtype, offset):
    """Philox state words that are zero in everyday calls: an offset beyond 2^34 (counter high word
    1), an offset just below it (the high word changes from 0 to 1 between the tiles of one launch)
    and, through the head-shard option, a (batch, head) index beyond 2^24 (subsequence high word
    1 and 2).  Forward mask through one-hot V, backward mask through one-hot dO, against the oracle."""
    fc = _fc()
    heads, p, causal = 2, 0.2, False
    sq, sk = [150, 90], [150, 90]
    seed = 0x9E3779B97F4A7C15 & 0x7FFFFFFFFFFFFFFF
    heads_total, head_offset = 2 ** 24 + 16, 2 ** 24 + 3
    q, k, v, dout, cu_q, cu_k = U.make_varlen(sq, sk, heads, d, dtype, seed=17)
    q, k = q * 0.1, k * 0.1
    n = orc.mask_block_n(d, max(sk))
    masks = [torch.from_numpy(np.stack([orc.dropout_keep_mask(seed, offset, b, head_offset + h, heads_total,
                                                              sq[b], sk[b], p, n, causal) for h in range(heads)]))
             for b in range(2)]
    gen = torch.cuda.default_generators[torch.cuda.current_device()]

    def rewind():
        gen.manual_seed(seed)
        gen.set_offset(offset)

    with fc.head_shard(heads_total, head_offset):
        for win in range(0, max(sk), d):
            v.zero_()
            start = 0
            for nk in sk:
                for c in range(d):
                    if win + c < nk:
                        v[start + win + c, :, c] = 1.0
                start += nk
            rewind()
            out, lse = fc.fwd(q, k, v, cu_q, cu_k, max(sq), max(sk), p, d ** -0.5, False, causal, False, None)
            qs = 0
            for b, (nq, nk) in enumerate(zip(sq, sk)):
                w = min(d, max(0, nk - win))
                if w > 0:
                    got = (out[qs:qs + nq, :, :w] != 0).permute(1, 0, 2).cpu()
                    assert torch.equal(got, masks[b][:, :, win:win + w]), "forward, window %d of batch %d" % (win, b)
                qs += nq
        v.normal_()
        rewind()
        out, lse = fc.fwd(q, k, v, cu_q, cu_k, max(sq), max(sk), p, d ** -0.5, False, causal, False, None)
        for win in range(0, max(sq), d):
            dout.zero_()
            start = 0
            for nq in sq:
                for c in range(d):
                    if win + c < nq:
                        dout[start + win + c, :, c] = 1.0
                start += nq
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, max(sq), max(sk), p, d ** -0.5, False,
                   causal, None, philox=(seed, offset))
            ks = 0
            for b, (nq, nk) in enumerate(zip(sq, sk)):
                w = min(d, max(0, nq - win))
                if w > 0:
                    got = (dv[ks:ks + nk, :, :w] != 0).permute(1, 2, 0).cpu()
                    assert torch.equal(got, masks[b][:, win:win + w, :]), "backward, window %d of batch %d" % (win, b)
                ks += nk
    fc.check_device_status()


@pytest.mark.parametrize("dtype,p", [(torch.float16, 0.05), (torch.bfloat16, 0.25)])
def test_rows_with_a_single_key_leave_only_the_rounding_of_o_in_dq(dtype, p):
    """Where a query sees one key its softmax is 1, dS is 0 and so is dq in exact arithmetic (and in
    the oracle, whose softmax backward computes g - sum(g * a) = 0).  A FlashAttention backward takes
    D = rowsum(dO * O) from the 16-bit O (csrc/flash_attn/src/fmha_dgrad_kernel_1xN_loop.h:16-28,
    :225), so dP - D keeps the rounding of O: |dq| <= eps * sum_c |dO_c O_c| * |k| * scale with eps one
    unit in the last place of the 16-bit type.  The '2 x the 16-bit program's error' rule cannot hold
    against an error of exactly zero; this is the bound that does."""
    fc = _fc()
    d, heads, nq = 64, 2, 63
    q, k, v, dout, cu_q, cu_k = U.make_varlen([nq], [1], heads, d, dtype, seed=23)
    scale = d ** -0.5
    torch.cuda.manual_seed(4)
    out, lse, seed, offset = fc.fwd(q, k, v, cu_q, cu_k, nq, 1, p, scale, False, False, False, None,
                                    return_philox=True)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, nq, 1, p, scale, False, False, None,
           philox=(seed, offset))
    fc.check_device_status()
    eps = 2.0 ** (-10 if dtype is torch.float16 else -7)
    bound = eps * (dout.float() * out.float()).abs().sum(-1).max() * k.float().abs().max() * scale
    err = dq.float().abs().max()
    assert 0 < err <= bound, (float(err), float(bound))
    # kept rows hold v / p_keep, dropped rows zero: the forward is exact up to that rounding
    kept = (out.float().abs().sum(-1) > 0)
    want = (v.float() / (1 - p)).expand_as(out.float())
    assert U.max_err(out[kept], want[kept]) <= eps * want.abs().max()
