"""oracle/sampled_oracle.py (one (batch, head) pair, chunked, results only at sampled rows) against
the dense oracle oracle/attention_oracle.py:attention_varlen_grads on sizes the dense one handles:
fp32 mode and the 16-bit emulation, causal, dropout mask, block-sparse layout."""
import numpy as np
import pytest
import torch

from oracle import attention_oracle as ao
from oracle.sampled_oracle import sampled_attention_grads


def _inputs(sq, sk, d, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    mk = lambda n: torch.randn(n, 1, d, generator=g).to(dtype)
    return mk(sq), mk(sk), mk(sk), mk(sq)


@pytest.mark.parametrize("mode_dtype", [None, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal,drop,sparse,sq,sk", [
    (False, 0.0, False, 300, 517),
    (True, 0.0, False, 521, 521),
    (False, 0.2, False, 384, 300),
    (False, 0.1, True, 512, 512),
    (True, 0.0, False, 200, 90),     # more queries than keys
])
def test_sampled_equals_dense(mode_dtype, causal, drop, sparse, sq, sk):
    d, scale = 32, 0.2
    in_dtype = mode_dtype or torch.float16
    q, k, v, do = _inputs(sq, sk, d, in_dtype, seed=sq + sk)
    keep = allowed = None
    rng = np.random.default_rng(3)
    if drop > 0:
        keep = torch.from_numpy(rng.random((1, sq, sk)) >= drop)
    if sparse:
        blocks = rng.random((sq // 256, sk // 256)) < 0.5
        blocks |= np.eye(sq // 256, sk // 256, dtype=bool)
        allowed = torch.from_numpy(np.kron(blocks, np.ones((256, 256), dtype=bool)))
    cdt = mode_dtype or torch.float32
    o, dq, dk, dv = ao.attention_varlen_grads(q, k, v, do, [0, sq], [0, sk], scale, causal, drop,
                                              None if keep is None else [keep],
                                              None if allowed is None else [allowed], cdt)
    q_rows = sorted(set(r for r in [0, 1, 127, 128, 129, sq // 2, sq - 2, sq - 1] if r < sq))
    k_rows = sorted(set(r for r in [0, 5, 127, 128, sk // 2, sk - 1] if r < sk))
    got = sampled_attention_grads(
        q[:, 0].float(), k[:, 0].float(), v[:, 0].float(), do[:, 0].float(), scale, causal, q_rows, k_rows,
        dropout_p=drop, keep_fn=None if keep is None else (lambda r0, r1: keep[0, r0:r1]),
        allowed_fn=None if allowed is None else (lambda r0, r1: allowed[r0:r1]),
        lowp_dtype=mode_dtype, chunk=128)
    # fp32: identical mathematics, summation order differs; 16-bit: each rounding can flip one ulp
    tol = 2e-5 if mode_dtype is None else (3e-2 if mode_dtype is torch.bfloat16 else 4e-3)
    for name, dense, rows in (("out", o, q_rows), ("dq", dq, q_rows), ("dk", dk, k_rows), ("dv", dv, k_rows)):
        want = dense[rows, 0].float()
        err = (got[name] - want).abs().max().item()
        assert err <= tol * max(1.0, want.abs().max().item()), (name, err)
    _, lses = ao.attention_varlen_ref(q, k, v, [0, sq], [0, sk], scale, causal,
                                      allowed=None if allowed is None else [allowed], compute_dtype=cdt)
    want_lse = lses[0][0, q_rows]
    finite = torch.isfinite(want_lse)
    assert torch.equal(torch.isfinite(got["lse"]), finite)
    assert (got["lse"][finite] - want_lse[finite]).abs().max().item() < 1e-4
