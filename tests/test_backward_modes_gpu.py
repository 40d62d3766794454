"""Backward-pass behaviour beyond plain parity: the deterministic (ticketed) dQ mode, backward
calls on two streams at once, token buffers longer than the sequences, and the Philox (seed,
offset) pair handed back by the forward."""
import ctypes
import math

import pytest
import torch

from tests import _util as U

pytestmark = pytest.mark.gpu


def _fc():
    from flash_attn_b200 import flash_attn_cuda
    return flash_attn_cuda


@pytest.fixture
def deterministic():
    fc = _fc()
    fc.options.deterministic = True
    yield fc
    fc.options.deterministic = False


DET_CASES = [
    # d, dtype, causal, seqlens, heads, dropout
    (64, torch.float16, False, [1500, 700, 333], 3, 0.0),
    (64, torch.float16, False, [1100, 1300], 2, 0.1),
    (64, torch.bfloat16, True, [2048, 1000, 129], 2, 0.0),
    (128, torch.bfloat16, True, [1024, 600], 2, 0.0),
    (128, torch.float16, False, [900], 2, 0.0),
    (32, torch.float16, True, [300, 77, 1], 2, 0.0),
]


@pytest.mark.parametrize("d,dtype,causal,lens,heads,p", DET_CASES)
def test_deterministic_dq_is_reproducible_and_correct(deterministic, d, dtype, causal, lens, heads, p):
    fc = deterministic
    q, k, v, dout, cu, _ = U.make_varlen(lens, lens, heads, d, dtype, seed=31 + d)
    scale = 1.0 / math.sqrt(d)
    out, lse, seed, offset = fc.fwd(q, k, v, cu, cu, max(lens), max(lens), p, scale, False, causal, False, None,
                                    return_philox=True)
    runs = []
    for _ in range(3):
        dq, dk, dv = torch.full_like(q, float("nan")), torch.empty_like(k), torch.empty_like(v)
        fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, max(lens), max(lens), p, scale, False, causal, None,
               philox=(seed, offset))
        runs.append((dq, dk, dv))
    torch.cuda.synchronize()
    fc.check_device_status()
    for dq, dk, dv in runs[1:]:
        assert torch.equal(dq, runs[0][0]) and torch.equal(dk, runs[0][1]) and torch.equal(dv, runs[0][2])
    if p == 0.0:
        o32, dq32, dk32, dv32 = U.oracle_cpu(q, k, v, dout, cu, cu, scale, causal)
        o16, dq16, dk16, dv16 = U.oracle_cpu(q, k, v, dout, cu, cu, scale, causal, dtype=dtype)
        U.assert_within_2x("dq", runs[0][0], dq32, dq16)
        U.assert_within_2x("dk", runs[0][1], dk32, dk16)
        U.assert_within_2x("dv", runs[0][2], dv32, dv16)
    # the arrival-order mode computes the same sums in another order
    fc.options.deterministic = False
    dq2, dk2, dv2 = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    fc.bwd(dout, q, k, v, out, lse, dq2, dk2, dv2, cu, cu, max(lens), max(lens), p, scale, False, causal, None,
           philox=(seed, offset))
    torch.cuda.synchronize()
    if causal:
        # the deterministic mode walks the query tiles of a causal problem from the last one down,
        # so dK / dV are summed in the opposite order
        assert U.max_err(dk2, runs[0][1]) < 4e-3 and U.max_err(dv2, runs[0][2]) < 4e-3
    else:
        assert torch.equal(dk2, runs[0][1]) and torch.equal(dv2, runs[0][2])
    assert U.max_err(dq2, runs[0][0]) < 4e-3


def test_deterministic_blocksparse(deterministic):
    fc = deterministic
    from flash_attn_b200.flash_blocksparse_attn_interface import convert_blockmask
    torch.manual_seed(0)
    S, heads = 1024, 2
    blocks = (torch.rand(S // 256, S // 256) < 0.4) | torch.eye(S // 256, dtype=torch.bool)
    layout = blocks.repeat_interleave(16, dim=0).to(torch.int32).cuda()
    conv = convert_blockmask(layout, False)
    q, k, v, dout, cu, _ = U.make_varlen([S, 700], [S, 700], heads, 64, torch.float16, seed=12)
    out, lse = fc.fwd_block(q, k, v, cu, cu, conv, S, S, 0.0, 0.125, False, False, None)
    res = []
    for _ in range(2):
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        fc.bwd_block(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, conv, S, S, 0.0, 0.125, False, None)
        res.append(dq)
    torch.cuda.synchronize()
    fc.check_device_status()
    assert torch.equal(res[0], res[1])
    fc.options.deterministic = False
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    fc.bwd_block(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, conv, S, S, 0.0, 0.125, False, None)
    torch.cuda.synchronize()
    assert U.max_err(dq, res[0]) < 4e-3


def test_backward_calls_on_two_streams_do_not_share_scratch():
    """Two backward passes in flight on different streams (each call owns its dQ accumulator)."""
    fc = _fc()
    lens = [2000, 1500]
    probs = []
    for seed in (1, 2):
        q, k, v, dout, cu, _ = U.make_varlen(lens, lens, 4, 64, torch.float16, seed=seed)
        out, lse = fc.fwd(q, k, v, cu, cu, 2000, 2000, 0.0, 0.125, False, False, False, None)
        probs.append((q, k, v, dout, cu, out, lse))
    torch.cuda.synchronize()
    want = []
    for q, k, v, dout, cu, out, lse in probs:
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, 2000, 2000, 0.0, 0.125, False, False, None)
        want.append(dq)
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    got = []
    for _ in range(3):
        got = []
        for s, (q, k, v, dout, cu, out, lse) in zip(streams, probs):
            with torch.cuda.stream(s):
                dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
                fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, 2000, 2000, 0.0, 0.125, False, False, None)
                got.append(dq)
    torch.cuda.synchronize()
    fc.check_device_status()
    for a, b in zip(got, want):
        assert U.max_err(a, b) < 4e-3


@pytest.mark.parametrize("zero_tensors", [False, True])
def test_rows_behind_the_last_sequence_are_left_alone(zero_tensors):
    """q / dq buffers longer than cu_seqlens[-1] (a preallocated token buffer): dq rows that belong
    to no sequence keep the caller's contents, or zero with zero_tensors, and never receive
    accumulator garbage."""
    fc = _fc()
    lens, extra = [100, 160], 75
    q, k, v, dout, cu, _ = U.make_varlen(lens + [extra], lens + [extra], 2, 64, torch.float16, seed=4)
    cu = cu[:3].contiguous()   # the last `extra` rows belong to no sequence
    out, lse = fc.fwd(q, k, v, cu, cu, 160, 160, 0.0, 0.125, False, False, False, None)
    # dirty the allocator's blocks so that a fresh accumulator holds garbage
    junk = torch.full((q.shape[0] * 2 * 64,), float("nan"), device="cuda")
    del junk
    dq, dk, dv = (torch.full_like(t, 7.0) for t in (q, k, v))
    fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, 160, 160, 0.0, 0.125, zero_tensors, False, None)
    torch.cuda.synchronize()
    fc.check_device_status()
    tail = dq[260:]
    assert torch.all(tail == (0.0 if zero_tensors else 7.0))
    o32, dq32, dk32, dv32 = U.oracle_cpu(q[:260], k[:260], v[:260], dout[:260], cu, cu, 0.125, False)
    assert U.max_err(dq[:260], dq32) < 4e-3


def test_forward_hands_back_the_philox_pair():
    fc = _fc()
    q, k, v, dout, cu, _ = U.make_varlen([300, 200], [300, 200], 2, 64, torch.float16, seed=6)
    gen = torch.cuda.default_generators[torch.cuda.current_device()]
    torch.cuda.manual_seed(99)
    off0 = gen.get_offset()
    res = fc.fwd(q, k, v, cu, cu, 300, 300, 0.2, 0.125, False, False, False, None, return_philox=True)
    assert len(res) == 4 and res[2] == 99 and res[3] == off0
    from flash_attn_b200 import _lib
    assert gen.get_offset() == off0 + _lib.lib.fa_philox_increment(64, 300, 300, 0)
    # a forward given that state again reproduces the output; the pair alone drives the backward
    gen.set_offset(off0)
    again = fc.fwd(q, k, v, cu, cu, 300, 300, 0.2, 0.125, False, False, False, None)
    assert torch.equal(again[0], res[0])
    plain = fc.fwd(q, k, v, cu, cu, 300, 300, 0.0, 0.125, False, False, False, None, return_philox=True)
    assert plain[2:] == [0, 0]
