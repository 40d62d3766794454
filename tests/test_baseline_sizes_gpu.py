"""Parity at the sizes the benchmark reports: the four GPU configurations of the workload list run
at full batch x heads on the GPU and are compared with the oracle on one or two (batch, head)
pairs at sampled rows (oracle/sampled_oracle.py: O, LSE, dQ at sampled query rows, dK, dV at
sampled key rows; first / middle / last tile and rows on either side of the 128- and 256-row
boundaries).  Same rule as the small cases: max|x - ref32| <= 2 * max|16-bit - ref32| + 1e-4,
LSE within 2e-4.  With dropout the kernel's Philox (seed, offset) is read back and the oracle
applies the mask of oracle/attention_oracle.py:dropout_keep_mask."""
import math

import numpy as np
import pytest
import torch

from oracle import attention_oracle as ao
from oracle.sampled_oracle import sampled_attention_grads
from tests import _util as U

pytestmark = pytest.mark.gpu


def _fc():
    from flash_attn_b200 import flash_attn_cuda
    return flash_attn_cuda


def _sample_rows(n):
    """First, middle and last 128-row tile, and both sides of the 128 / 256 boundaries."""
    mid = (n // 2) // 256 * 256
    cand = [0, 1, 15, 16, 127, 128, 129, 255, 256, 257, mid - 129, mid - 1, mid, mid + 1, mid + 127, mid + 128,
            n - 257, n - 256, n - 129, n - 128, n - 17, n - 2, n - 1]
    return sorted(set(r for r in cand if 0 <= r < n))


def _check_pair(name, dtype, q, k, v, dout, out, lse, dq, dk, dv, q0, k0, sq, sk, b, h, scale, causal,
                dropout_p=0.0, keep_fn=None, allowed_fn=None):
    """Oracle on (batch b, head h) of a packed problem; q0 / k0 = first token of the sequence."""
    cpu = lambda t, s0, n: t[s0:s0 + n, h].float().cpu()
    qc, kc, vc, gc = cpu(q, q0, sq), cpu(k, k0, sk), cpu(v, k0, sk), cpu(dout, q0, sq)
    q_rows, k_rows = _sample_rows(sq), _sample_rows(sk)
    masks = {}

    def cached(fn, tag):
        if fn is None:
            return None

        def inner(r0, r1):
            key = (tag, r0, r1)
            if key not in masks:
                masks[key] = fn(r0, r1)
            return masks[key]
        return inner

    keep_c, allow_c = cached(keep_fn, "keep"), cached(allowed_fn, "allowed")
    ref = sampled_attention_grads(qc, kc, vc, gc, scale, causal, q_rows, k_rows, dropout_p, keep_c, allow_c, None)
    low = sampled_attention_grads(qc, kc, vc, gc, scale, causal, q_rows, k_rows, dropout_p, keep_c, allow_c, dtype)
    qi = torch.tensor(q_rows, device=q.device) + q0
    ki = torch.tensor(k_rows, device=q.device) + k0
    U.assert_within_2x(name + " out", out[qi, h], ref["out"], low["out"])
    U.assert_within_2x(name + " dq", dq[qi, h], ref["dq"], low["dq"])
    U.assert_within_2x(name + " dk", dk[ki, h], ref["dk"], low["dk"])
    U.assert_within_2x(name + " dv", dv[ki, h], ref["dv"], low["dv"])
    got_lse = lse[b, h, torch.tensor(q_rows, device=q.device)].cpu()
    finite = torch.isfinite(ref["lse"])
    assert (got_lse[finite] - ref["lse"][finite]).abs().max().item() < 2e-4, name + " lse"


def _run(fc, q, k, v, dout, cu, max_s, p, scale, causal, blockmask=None):
    if blockmask is None:
        res = fc.fwd(q, k, v, cu, cu, max_s, max_s, p, scale, False, causal, False, None, return_philox=True)
    else:
        res = fc.fwd_block(q, k, v, cu, cu, blockmask, max_s, max_s, p, scale, causal, False, None,
                           return_philox=True)
    out, lse, seed, offset = res
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    if blockmask is None:
        fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, max_s, max_s, p, scale, False, causal, None,
               philox=(seed, offset))
    else:
        fc.bwd_block(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, blockmask, max_s, max_s, p, scale, causal, None,
                     philox=(seed, offset))
    torch.cuda.synchronize()
    fc.check_device_status()
    return out, lse, dq, dk, dv, seed, offset


def test_bert_varlen_fp16_dropout_max_seqlen_4096():
    """Workload 2: batch 8 x 12 heads x d 64, lengths uniform in [2048, 4096], fp16, dropout 0.1."""
    fc = _fc()
    rng = np.random.default_rng(0)
    lens = [int(x) for x in rng.integers(2048, 4097, size=8)]
    heads, d, p = 12, 64, 0.1
    q, k, v, dout, cu, _ = U.make_varlen(lens, lens, heads, d, torch.float16, seed=2)
    scale = 1.0 / math.sqrt(d)
    torch.cuda.manual_seed(1234)
    out, lse, dq, dk, dv, seed, offset = _run(fc, q, k, v, dout, cu, 4096, p, scale, False)
    starts = np.concatenate([[0], np.cumsum(lens)])
    longest, shortest = int(np.argmax(lens)), int(np.argmin(lens))
    for b, h in ((longest, 7), (shortest, 0)):
        n = lens[b]
        keep_fn = lambda r0, r1, b=b, h=h, n=n: torch.from_numpy(
            ao.dropout_keep_mask(seed, offset, b, h, heads, n, n, p, 256, False, row_range=(r0, r1)))
        _check_pair("bert b%d h%d" % (b, h), torch.float16, q, k, v, dout, out, lse, dq, dk, dv,
                    int(starts[b]), int(starts[b]), n, n, b, h, scale, False, p, keep_fn)


def test_causal_lm_bf16_d128_seqlen_8192():
    """Workload 3: batch 16 x 12 heads x d 128, 8192 tokens each, bf16, causal."""
    fc = _fc()
    B, H, d, S = 16, 12, 128, 8192
    g = torch.Generator(device="cuda").manual_seed(5)
    mk = lambda: torch.randn(B * S, H, d, device="cuda", dtype=torch.bfloat16, generator=g)
    q, k, v, dout = mk(), mk(), mk(), mk()
    cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(d)
    out, lse, dq, dk, dv, _, _ = _run(fc, q, k, v, dout, cu, S, 0.0, scale, True)
    for b, h in ((11, 5),):
        _check_pair("causal_lm b%d h%d" % (b, h), torch.bfloat16, q, k, v, dout, out, lse, dq, dk, dv,
                    b * S, b * S, S, S, b, h, scale, True)


def test_blocksparse_fp16_dropout_seqlen_4096():
    """Workload 4: batch 4 x 16 heads x d 64 x 4096, random 25 % layout of 256 x 256 blocks with the
    diagonal kept, dropout 0.1."""
    fc = _fc()
    from flash_attn_b200.flash_blocksparse_attn_interface import convert_blockmask
    B, H, d, S, p = 4, 16, 64, 4096, 0.1
    rng = np.random.default_rng(4)
    blocks = (rng.random((S // 256, S // 256)) < 0.25) | np.eye(S // 256, dtype=bool)
    layout = torch.from_numpy(np.repeat(blocks, 16, axis=0).astype(np.int32)).cuda()   # (S/16, S/256)
    blockmask = convert_blockmask(layout, False)
    np.testing.assert_array_equal(blockmask.cpu().numpy(), ao.convert_blockmask_loops(layout.cpu().numpy()))
    g = torch.Generator(device="cuda").manual_seed(6)
    mk = lambda: torch.randn(B * S, H, d, device="cuda", dtype=torch.float16, generator=g)
    q, k, v, dout = mk(), mk(), mk(), mk()
    cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(d)
    torch.cuda.manual_seed(77)
    out, lse, dq, dk, dv, seed, offset = _run(fc, q, k, v, dout, cu, S, p, scale, False, blockmask)
    bm = blockmask.cpu().numpy()
    it = ao.blocksparse_walk(bm, S, S)
    allowed = torch.from_numpy(ao.blocksparse_allowed(bm, S, S))
    b, h = 2, 9
    keep_fn = lambda r0, r1: torch.from_numpy(
        ao.dropout_keep_mask(seed, offset, b, h, H, S, S, p, 256, False, bs_iter=it, row_range=(r0, r1)))
    _check_pair("blocksparse b%d h%d" % (b, h), torch.float16, q, k, v, dout, out, lse, dq, dk, dv,
                b * S, b * S, S, S, b, h, scale, False, p, keep_fn, lambda r0, r1: allowed[r0:r1])


def test_long_context_bf16_d64_seqlen_65536():
    """Workload 5 on one GPU: batch 2 x 32 heads x d 64 x 65536 tokens, bf16, causal."""
    fc = _fc()
    B, H, d, S = 2, 32, 64, 65536
    g = torch.Generator(device="cuda").manual_seed(7)
    mk = lambda: torch.randn(B * S, H, d, device="cuda", dtype=torch.bfloat16, generator=g)
    q, k, v, dout = mk(), mk(), mk(), mk()
    cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(d)
    out, lse, dq, dk, dv, _, _ = _run(fc, q, k, v, dout, cu, S, 0.0, scale, True)
    b, h = 1, 17
    _check_pair("long_context b%d h%d" % (b, h), torch.bfloat16, q, k, v, dout, out, lse, dq, dk, dv,
                b * S, b * S, S, S, b, h, scale, True)
