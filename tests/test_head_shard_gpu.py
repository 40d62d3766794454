"""Head-sharded execution equals the unsharded call: the shards of a batch x heads problem run one
after another on one GPU (each the way a rank of a multi-GPU job would run its share, with the
dropout mask of the unsharded call selected through head_shard) and their concatenation is
compared bit for bit with the single call -- O, LSE, dK, dV, the dropout mask, and dQ in the
deterministic mode.  This is the independence the multi-GPU path relies on (every (batch, head)
pair is its own problem, csrc/flash_attn/src/fmha_fprop_fp16_kernel.sm80.cu:77)."""
import math

import pytest
import torch

from tests import _util as U

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("d,dtype,causal,p,world", [
    (64, torch.float16, False, 0.1, 2),
    (64, torch.bfloat16, True, 0.1, 4),
    (128, torch.bfloat16, True, 0.0, 2),
])
def test_head_shards_concatenate_to_the_unsharded_result(d, dtype, causal, p, world):
    from flash_attn_b200 import flash_attn_cuda as fc
    heads, lens = 8, [700, 300, 1025]
    q, k, v, dout, cu, _ = U.make_varlen(lens, lens, heads, d, dtype, seed=17)
    scale, max_s = 1.0 / math.sqrt(d), max(lens)
    fc.options.deterministic = True
    try:
        torch.cuda.manual_seed(5)
        out, lse, s_full, seed, offset = fc.fwd(q, k, v, cu, cu, max_s, max_s, p, scale, False, causal, True, None,
                                                return_philox=True)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, max_s, max_s, p, scale, False, causal, None,
               philox=(seed, offset))
        hs = heads // world
        gen = torch.cuda.default_generators[torch.cuda.current_device()]
        for r in range(world):
            sl = slice(r * hs, (r + 1) * hs)
            qs, ks, vs, gs = (t[:, sl].contiguous() for t in (q, k, v, dout))
            with fc.head_shard(heads, r * hs):
                gen.set_offset(offset)   # every rank starts from the generator state of the unsharded call
                o_s, lse_s, s_s = fc.fwd(qs, ks, vs, cu, cu, max_s, max_s, p, scale, False, causal, True, None)
                dq_s, dk_s, dv_s = torch.empty_like(qs), torch.empty_like(ks), torch.empty_like(vs)
                fc.bwd(gs, qs, ks, vs, o_s, lse_s, dq_s, dk_s, dv_s, cu, cu, max_s, max_s, p, scale, False, causal,
                       None, philox=(seed, offset))
            torch.cuda.synchronize()
            assert torch.equal(o_s, out[:, sl])
            for b, n in enumerate(lens):   # LSE entries past a sequence's length are never written
                assert torch.equal(lse_s[b, :, :n], lse[b, sl, :n])
            assert torch.equal(dk_s, dk[:, sl]) and torch.equal(dv_s, dv[:, sl]) and torch.equal(dq_s, dq[:, sl])
            # sign bit of the returned probabilities = dropped: the masks agree bit for bit
            assert torch.equal(torch.signbit(s_s), torch.signbit(s_full[:, sl]))
        fc.check_device_status()
        if p > 0:
            # without head_shard a shard draws the mask of a `hs`-head call, which differs
            qs, ks, vs = (t[:, hs:2 * hs].contiguous() for t in (q, k, v))
            gen.set_offset(offset)
            o_plain = fc.fwd(qs, ks, vs, cu, cu, max_s, max_s, p, scale, False, causal, False, None)[0]
            assert not torch.equal(o_plain, out[:, hs:2 * hs])
    finally:
        fc.options.deterministic = False
