"""The compiled binding (csrc/fa_torch_binding.cpp) and the ctypes binding are two routes to the
same C ABI: same outputs bit for bit, same Philox protocol, same options, same errors."""
import pytest
import torch

from tests import _util as U

pytestmark = pytest.mark.gpu


def _fc():
    from flash_attn_b200 import flash_attn_cuda
    return flash_attn_cuda


class _ctypes_route:
    """Temporarily send dense calls through the ctypes route."""

    def __enter__(self):
        self.fc = _fc()
        self.saved = self.fc._binding
        self.fc._binding = None

    def __exit__(self, *exc):
        self.fc._binding = self.saved
        return False


def _require_compiled():
    if _fc().binding_in_use() != "compiled":
        pytest.skip("compiled binding not built (or disabled by FA_B200_BINDING=ctypes)")


@pytest.mark.parametrize("d,dtype,causal,p", [(64, torch.float16, False, 0.1), (128, torch.bfloat16, True, 0.0),
                                              (32, torch.float16, True, 0.2)])
def test_both_routes_give_the_same_tensors(d, dtype, causal, p):
    _require_compiled()
    fc = _fc()
    sq, sk = [200, 77], [260, 77]
    q, k, v, dout, cu_q, cu_k = U.make_varlen(sq, sk, 3, d, dtype, seed=31)
    gen = torch.cuda.default_generators[torch.cuda.current_device()]

    def run():
        gen.manual_seed(99)
        gen.set_offset(40)
        res = fc.fwd(q, k, v, cu_q, cu_k, max(sq), max(sk), p, d ** -0.5, False, causal, False, None,
                     return_philox=True)
        out, lse, seed, offset = res
        after_fwd = gen.get_offset()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        fc.options.deterministic = True   # so that dq is comparable bit for bit
        try:
            r = fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, max(sq), max(sk), p, d ** -0.5, False,
                       causal, None, philox=(seed, offset))
        finally:
            fc.options.deterministic = False
        return out, lse, seed, offset, after_fwd, r[0], r[1], r[2], r[3]

    a = run()
    with _ctypes_route():
        b = run()
    assert a[2:5] == b[2:5]                    # Philox pair and generator advance
    for x, y, n in zip(a[0:2] + a[5:], b[0:2] + b[5:], ("out", "lse", "dq", "dk", "dv", "softmax_d")):
        if n in ("lse", "softmax_d"):          # rows past a sequence's end are never written
            for bi, nq in enumerate(sq):
                assert torch.equal(x[bi, :, :nq], y[bi, :, :nq]), n
        else:
            assert torch.equal(x, y), n
    fc.check_device_status()


def test_generator_protocol_without_explicit_pair():
    """The reference's protocol: the caller restores the generator state saved before the forward,
    the backward reads the pair from the generator (and advances it by a dummy amount)."""
    _require_compiled()
    fc = _fc()
    q, k, v, dout, cu_q, cu_k = U.make_varlen([150], [150], 2, 64, torch.float16, seed=32)
    gen = torch.cuda.default_generators[torch.cuda.current_device()]

    def run():
        gen.manual_seed(5)
        state = gen.get_state()
        out, lse = fc.fwd(q, k, v, cu_q, cu_k, 150, 150, 0.3, 0.125, False, False, False, None)
        gen.set_state(state)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, 150, 150, 0.3, 0.125, False, False, None)
        return out, dk, dv, gen.get_offset()

    a = run()
    with _ctypes_route():
        b = run()
    assert a[3] == b[3]
    for x, y in zip(a[:3], b[:3]):
        assert torch.equal(x, y)


def test_zero_tensors_head_shard_and_errors():
    _require_compiled()
    fc = _fc()
    q, k, v, dout, cu_q, cu_k = U.make_varlen([100, 60], [100, 60], 2, 64, torch.float16, seed=33)
    # zero_tensors: rows of lse that belong to no query hold -inf
    out, lse = fc.fwd(q, k, v, cu_q, cu_k, 100, 100, 0.0, 0.125, True, False, False, None)
    assert torch.isinf(lse[1, :, 60:100]).all() and (lse[1, :, 60:100] < 0).all()
    # head-shard option reaches the C ABI through both routes
    torch.cuda.manual_seed(3)
    with fc.head_shard(8, 4):
        a = fc.fwd(q, k, v, cu_q, cu_k, 100, 100, 0.5, 0.125, False, False, False, None)[0]
    torch.cuda.manual_seed(3)
    with _ctypes_route(), fc.head_shard(8, 4):
        b = fc.fwd(q, k, v, cu_q, cu_k, 100, 100, 0.5, 0.125, False, False, False, None)[0]
    assert torch.equal(a, b)
    torch.cuda.manual_seed(3)
    c = fc.fwd(q, k, v, cu_q, cu_k, 100, 100, 0.5, 0.125, False, False, False, None)[0]
    assert not torch.equal(a, c)
    # same exception type and message as the ctypes route
    for bad in (lambda: fc.fwd(q.float(), k, v, cu_q, cu_k, 100, 100, 0.0, 0.125, False, False, False, None),
                lambda: fc.fwd(q, k[:, :1], v, cu_q, cu_k, 100, 100, 0.0, 0.125, False, False, False, None),
                lambda: fc.fwd(q, k, v, cu_q, cu_k, 100, 100, 1.0, 0.125, False, False, False, None)):
        with pytest.raises(RuntimeError) as e1:
            bad()
        with _ctypes_route(), pytest.raises(RuntimeError) as e2:
            bad()
        assert str(e1.value).splitlines()[0] == str(e2.value).splitlines()[0]


def test_block_sparse_and_return_softmax_through_both_routes():
    _require_compiled()
    fc = _fc()
    from flash_attn_b200.flash_blocksparse_attn_interface import convert_blockmask
    S = 512
    torch.manual_seed(2)
    blocks = (torch.rand(S // 256, S // 256) < 0.5) | torch.eye(S // 256, dtype=torch.bool)
    conv = convert_blockmask(blocks.repeat_interleave(16, dim=0).to(torch.int32).cuda(), False)
    q, k, v, dout, cu_q, cu_k = U.make_varlen([S, 300], [S, 300], 2, 64, torch.float16, seed=34)

    def run():
        torch.cuda.manual_seed(8)
        out, lse, seed, offset = fc.fwd_block(q, k, v, cu_q, cu_k, conv, S, S, 0.1, 0.125, False, False, None,
                                              return_philox=True)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        fc.bwd_block(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, conv, S, S, 0.1, 0.125, False, None,
                     philox=(seed, offset))
        torch.cuda.manual_seed(8)
        o2, _, s_dmask = fc.fwd(q, k, v, cu_q, cu_k, S, S, 0.1, 0.125, False, True, True, None)
        return out, dk, dv, o2, s_dmask

    a = run()
    with _ctypes_route():
        b = run()
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    # the messages of the block-mask checks agree too
    for bad in (lambda: fc.fwd_block(q, k, v, cu_q, cu_k, conv[:1], S, S, 0.0, 0.125, False, False, None),
                lambda: fc.fwd_block(q, k, v, cu_q, cu_k, conv.long(), S, S, 0.0, 0.125, False, False, None)):
        with pytest.raises(RuntimeError) as e1:
            bad()
        with _ctypes_route(), pytest.raises(RuntimeError) as e2:
            bad()
        assert str(e1.value).splitlines()[0] == str(e2.value).splitlines()[0]
