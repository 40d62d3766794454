"""GPU parity tests of the forward and backward kernels, called through the extension-module
contract (flash_attn_cuda.fwd / bwd, i.e. the C ABI), against the fp32 CPU oracle.

Floating-point bar: max|x - ref32| <= 2 * max|lowp - ref32| (+1e-4), where lowp is the oracle run
in the 16-bit input type; LSE within 2e-4 absolute."""
import math

import pytest
import torch

from tests import _util as U

pytestmark = pytest.mark.gpu


def _fc():
    from flash_attn_b200 import flash_attn_cuda
    return flash_attn_cuda


CASES = [
    # d, dtype, causal, seqlens_q, seqlens_k, heads
    (64, torch.float16, False, [128], [128], 2),
    (64, torch.bfloat16, False, [256, 256], [256, 256], 3),
    (64, torch.float16, True, [300, 77, 1], [300, 77, 1], 3),
    (64, torch.float16, False, [1, 15, 16, 17, 97], [1, 15, 16, 17, 97], 2),
    (64, torch.bfloat16, True, [129, 255, 256, 257], [129, 255, 256, 257], 2),
    (64, torch.float16, False, [513], [1000], 2),
    (64, torch.float16, True, [700], [333], 2),
    (128, torch.bfloat16, True, [512], [512], 2),
    (128, torch.bfloat16, False, [1000, 333], [1000, 333], 2),
    (128, torch.float16, False, [130], [257], 1),
    (32, torch.float16, False, [200, 130], [100, 513], 2),
    (16, torch.float16, True, [200, 130], [100, 513], 2),
    (32, torch.bfloat16, True, [384], [384], 1),
]


@pytest.mark.parametrize("d,dtype,causal,sq,sk,heads", CASES)
def test_forward_backward_parity(d, dtype, causal, sq, sk, heads):
    fc = _fc()
    q, k, v, dout, cu_q, cu_k = U.make_varlen(sq, sk, heads, d, dtype, seed=d + len(sq))
    scale = 1.0 / math.sqrt(d)
    out, lse = fc.fwd(q, k, v, cu_q, cu_k, max(sq), max(sk), 0.0, scale, False, causal, False, None)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    _, _, _, softmax_d = fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, max(sq), max(sk),
                                0.0, scale, False, causal, None)
    torch.cuda.synchronize()
    fc.check_device_status()

    o32, dq32, dk32, dv32 = U.oracle_cpu(q, k, v, dout, cu_q, cu_k, scale, causal)
    o16, dq16, dk16, dv16 = U.oracle_cpu(q, k, v, dout, cu_q, cu_k, scale, causal, dtype=dtype)
    U.assert_within_2x("out", out, o32, o16)
    U.assert_within_2x("dq", dq, dq32, dq16)
    U.assert_within_2x("dk", dk, dk32, dk16)
    U.assert_within_2x("dv", dv, dv32, dv16)
    lses = U.oracle_lse(q, k, v, cu_q, cu_k, scale, causal)
    for b, n in enumerate(sq):
        assert U.max_err(lse[b, :, :n], lses[b]) < 2e-4
    # softmax_d = rowsum(dO * O)
    o_cpu, do_cpu = out.float().cpu(), dout.float().cpu()
    start = 0
    for b, n in enumerate(sq):
        want = (o_cpu[start:start + n] * do_cpu[start:start + n]).sum(-1).transpose(0, 1)
        assert U.max_err(softmax_d[b, :, :n], want) < 1e-3
        start += n


def test_packed_qkv_views_and_gradient_views():
    """The normal calling pattern: q, k, v are strided views of one packed tensor and the
    gradients are written into views of one packed gradient tensor."""
    fc = _fc()
    torch.manual_seed(3)
    seqlens = [100, 260]
    total, heads, d = sum(seqlens), 4, 64
    qkv = torch.randn(total, 3, heads, d, device="cuda", dtype=torch.float16)
    dout = torch.randn(total, heads, d, device="cuda", dtype=torch.float16)
    cu = torch.tensor([0, 100, 360], dtype=torch.int32, device="cuda")
    out, lse = fc.fwd(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, cu, 260, 260, 0.0, 0.125, False, True, False, None)
    dqkv = torch.full_like(qkv, float("nan"))
    fc.bwd(dout, qkv[:, 0], qkv[:, 1], qkv[:, 2], out, lse, dqkv[:, 0], dqkv[:, 1], dqkv[:, 2], cu, cu,
           260, 260, 0.0, 0.125, False, True, None)
    torch.cuda.synchronize()
    fc.check_device_status()
    o32, dq32, dk32, dv32 = U.oracle_cpu(qkv[:, 0], qkv[:, 1], qkv[:, 2], dout, cu, cu, 0.125, True)
    o16, dq16, dk16, dv16 = U.oracle_cpu(qkv[:, 0], qkv[:, 1], qkv[:, 2], dout, cu, cu, 0.125, True,
                                         dtype=torch.float16)
    U.assert_within_2x("out", out, o32, o16)
    U.assert_within_2x("dq", dqkv[:, 0], dq32, dq16)
    U.assert_within_2x("dk", dqkv[:, 1], dk32, dk16)
    U.assert_within_2x("dv", dqkv[:, 2], dv32, dv16)


def test_empty_sequences_and_zero_tensors():
    """A batch entry with no keys gives O = 0 and LSE = -inf; one with no queries writes nothing
    for its queries and zero gradients for its keys."""
    fc = _fc()
    sq, sk = [64, 0, 40], [0, 50, 40]
    q, k, v, dout, cu_q, cu_k = U.make_varlen(sq, sk, 2, 64, torch.float16, seed=5)
    out, lse = fc.fwd(q, k, v, cu_q, cu_k, 64, 50, 0.0, 0.125, True, False, False, None)
    dq = torch.full_like(q, float("nan"))
    dk = torch.full_like(k, float("nan"))
    dv = torch.full_like(v, float("nan"))
    fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, 64, 50, 0.0, 0.125, False, False, None)
    torch.cuda.synchronize()
    fc.check_device_status()
    assert torch.all(out[:64] == 0) and torch.all(torch.isinf(lse[0, :, :64]))
    assert torch.all(dq[:64] == 0)
    assert torch.all(dk[:50] == 0) and torch.all(dv[:50] == 0)
    o32, dq32, dk32, dv32 = U.oracle_cpu(q[64:], k[50:], v[50:], dout[64:], [0, 40], [0, 40], 0.125, False)
    assert U.max_err(out[64:], o32) < 2e-3
    assert U.max_err(dq[64:], dq32) < 4e-3 and U.max_err(dk[50:], dk32) < 4e-3 and U.max_err(dv[50:], dv32) < 4e-3
    assert not torch.isnan(dq).any() and not torch.isnan(dk).any() and not torch.isnan(dv).any()


def test_no_out_of_bounds_writes():
    """Gradient and output rows next to the ones a call owns keep their sentinel values."""
    fc = _fc()
    sq = [200, 57]
    q, k, v, dout, cu_q, cu_k = U.make_varlen(sq, sq, 2, 64, torch.bfloat16, seed=9)
    total = sum(sq)
    pad = 8
    bufs = [torch.full((total + 2 * pad, 2, 64), 7.0, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    dq, dk, dv = (b[pad:pad + total] for b in bufs)
    out, lse = fc.fwd(q, k, v, cu_q, cu_k, 200, 200, 0.0, 0.125, False, True, False, None)
    fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, 200, 200, 0.0, 0.125, False, True, None)
    torch.cuda.synchronize()
    for b in bufs:
        assert torch.all(b[:pad] == 7.0) and torch.all(b[pad + total:] == 7.0)
    assert not torch.isnan(dq.float()).any()


def test_forward_is_deterministic_and_dkdv_too():
    fc = _fc()
    q, k, v, dout, cu_q, cu_k = U.make_varlen([640], [640], 3, 128, torch.bfloat16, seed=1)
    res = []
    for _ in range(2):
        out, lse = fc.fwd(q, k, v, cu_q, cu_k, 640, 640, 0.0, 0.09, False, True, False, None)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, 640, 640, 0.0, 0.09, False, True, None)
        res.append((out.clone(), lse.clone(), dk.clone(), dv.clone()))
    torch.cuda.synchronize()
    for a, b in zip(*res):
        assert torch.equal(a, b)


def test_argument_checks_raise():
    fc = _fc()
    q, k, v, dout, cu_q, cu_k = U.make_varlen([32], [32], 1, 64, torch.float16, seed=2)
    with pytest.raises(RuntimeError):
        fc.fwd(q.float(), k.float(), v.float(), cu_q, cu_k, 32, 32, 0.0, 0.125, False, False, False, None)
    with pytest.raises(RuntimeError):
        fc.fwd(q, k, v, cu_q.long(), cu_k, 32, 32, 0.0, 0.125, False, False, False, None)
    with pytest.raises(RuntimeError):
        fc.fwd(q[:, :, :48], k[:, :, :48], v[:, :, :48], cu_q, cu_k, 32, 32, 0.0, 0.125, False, False, False, None)
    with pytest.raises(RuntimeError):
        fc.fwd(q, k, v, cu_q, cu_k, 32, 32, 1.0, 0.125, False, False, False, None)


@pytest.mark.parametrize("batch,heads,d,seqlen,causal,dtype", [
    (8, 12, 64, 2048, False, torch.float16),      # BERT-base shape of the headline sweep
    (16, 12, 128, 2048, True, torch.bfloat16),    # causal LM shape
])
def test_full_size_properties(batch, heads, d, seqlen, causal, dtype):
    """Size-independent properties at benchmark sizes (the CPU oracle would take minutes there):
    softmax rows sum to one, so constant V gives constant O, sum_j dV_j = sum_i dO_i, and with
    all keys equal every dS row sums to zero, so dQ = 0; attention is linear in V."""
    fc = _fc()
    total = batch * seqlen
    g = torch.Generator(device="cuda").manual_seed(0)
    cu = torch.arange(0, (batch + 1) * seqlen, seqlen, dtype=torch.int32, device="cuda")
    q = torch.randn(total, heads, d, device="cuda", dtype=dtype, generator=g)
    k = torch.randn(total, heads, d, device="cuda", dtype=dtype, generator=g)
    v1 = torch.randn(total, heads, d, device="cuda", dtype=dtype, generator=g)
    dout = torch.randn(total, heads, d, device="cuda", dtype=dtype, generator=g)
    scale = d ** -0.5
    ones = torch.full_like(v1, 0.5)
    out_c, lse = fc.fwd(q, k, ones, cu, cu, seqlen, seqlen, 0.0, scale, False, causal, False, None)
    assert (out_c.float() - 0.5).abs().max().item() < 4e-3
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v1)
    fc.bwd(dout, q, k, ones, out_c, lse, dq, dk, dv, cu, cu, seqlen, seqlen, 0.0, scale, False, causal, None)
    sum_dv = dv.float().reshape(batch, seqlen, heads, d).sum(1)
    sum_do = dout.float().reshape(batch, seqlen, heads, d).sum(1)
    assert (sum_dv - sum_do).abs().max().item() < 0.5  # sums of 2048 16-bit values of magnitude ~1
    # all keys equal -> uniform attention, dQ = 0
    k_same = k[:1].expand_as(k).contiguous()
    out_u, lse_u = fc.fwd(q, k_same, v1, cu, cu, seqlen, seqlen, 0.0, scale, False, causal, False, None)
    fc.bwd(dout, q, k_same, v1, out_u, lse_u, dq, dk, dv, cu, cu, seqlen, seqlen, 0.0, scale, False, causal, None)
    assert dq.float().abs().max().item() < 2e-2
    # linearity in V
    v2 = torch.randn(total, heads, d, device="cuda", dtype=dtype, generator=g)
    o1, _ = fc.fwd(q, k, v1, cu, cu, seqlen, seqlen, 0.0, scale, False, causal, False, None)
    o2, _ = fc.fwd(q, k, v2, cu, cu, seqlen, seqlen, 0.0, scale, False, causal, False, None)
    o12, _ = fc.fwd(q, k, (v1.float() * 0.5 + v2.float() * 0.25).to(dtype), cu, cu, seqlen, seqlen, 0.0, scale,
                    False, causal, False, None)
    torch.cuda.synchronize()
    fc.check_device_status()
    assert (o12.float() - (0.5 * o1.float() + 0.25 * o2.float())).abs().max().item() < 3e-2


@pytest.mark.parametrize("d,dtype,causal,gain", [
    (64, torch.float16, False, 6.0),
    (64, torch.bfloat16, True, 8.0),
    (128, torch.bfloat16, False, 5.0),
])
def test_large_scores_and_growing_maxima(d, dtype, causal, gain):
    """Scores tens of units apart (peaked softmax rows) and keys sorted so that the row maximum keeps
    growing from key tile to key tile: exercises the deferred rescaling of the running maximum (the
    kernel keeps a stale maximum while it lags by less than 2^8) without overflow or loss."""
    fc = _fc()
    sq, sk, heads = [384, 200], [640, 257], 2
    q, k, v, dout, cu_q, cu_k = U.make_varlen(sq, sk, heads, d, dtype, seed=77)
    # later keys align more and more with a common direction of the queries
    direction = torch.randn(d, device="cuda").to(dtype)
    ramp = torch.cat([torch.linspace(0.0, 1.0, n, device="cuda") for n in sk]).to(dtype)
    k = (k + gain * ramp[:, None, None] * direction[None, None, :]).contiguous()
    q = (q + 0.5 * direction[None, None, :]).contiguous()
    scale = 1.0 / math.sqrt(d)
    out, lse = fc.fwd(q, k, v, cu_q, cu_k, max(sq), max(sk), 0.0, scale, False, causal, False, None)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, max(sq), max(sk), 0.0, scale, False, causal, None)
    torch.cuda.synchronize()
    fc.check_device_status()
    for name, x in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv), ("lse", lse)):
        assert torch.isfinite(x.float()).all() or name == "lse", name
    o32, dq32, dk32, dv32 = U.oracle_cpu(q, k, v, dout, cu_q, cu_k, scale, causal)
    o16, dq16, dk16, dv16 = U.oracle_cpu(q, k, v, dout, cu_q, cu_k, scale, causal, dtype=dtype)
    U.assert_within_2x("out", out, o32, o16)
    U.assert_within_2x("dq", dq, dq32, dq16)
    U.assert_within_2x("dk", dk, dk32, dk16)
    U.assert_within_2x("dv", dv, dv32, dv16)
    lses = U.oracle_lse(q, k, v, cu_q, cu_k, scale, causal)
    for b, n in enumerate(sq):
        assert U.max_err(lse[b, :, :n], lses[b]) < 2e-3   # LSE values reach the hundreds here
