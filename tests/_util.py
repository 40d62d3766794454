"""Shared helpers of the GPU parity tests."""
import numpy as np
import torch

from oracle import attention_oracle as orc


def make_varlen(seqlens_q, seqlens_k, heads, d, dtype, seed, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    tq, tk = sum(seqlens_q), sum(seqlens_k)
    q = torch.randn(tq, heads, d, generator=g).to(dtype).to(device)
    k = torch.randn(tk, heads, d, generator=g).to(dtype).to(device)
    v = torch.randn(tk, heads, d, generator=g).to(dtype).to(device)
    dout = torch.randn(tq, heads, d, generator=g).to(dtype).to(device)
    cu_q = torch.tensor(np.concatenate([[0], np.cumsum(seqlens_q)]), dtype=torch.int32, device=device)
    cu_k = torch.tensor(np.concatenate([[0], np.cumsum(seqlens_k)]), dtype=torch.int32, device=device)
    return q, k, v, dout, cu_q, cu_k


def max_err(a, b):
    return (a.float().cpu() - b.float().cpu()).abs().max().item()


def assert_within_2x(name, got, ref32, lowp, atol=1e-4):
    """The parity rule for floating-point results: the kernel's max-abs error against the fp32
    oracle is at most twice that of the same math done in the 16-bit type, plus `atol`."""
    e_kernel = max_err(got, ref32)
    e_lowp = max_err(lowp, ref32)
    assert not torch.isnan(got.float()).any(), name + " has NaN"
    assert e_kernel <= 2.0 * e_lowp + atol, "%s: kernel error %.3e > 2 x %.3e" % (name, e_kernel, e_lowp)
    return e_kernel, e_lowp


def _as_list(cu):
    return cu.cpu().tolist() if torch.is_tensor(cu) else list(cu)


def oracle_cpu(q, k, v, dout, cu_q, cu_k, scale, causal, dropout_p=0.0, keep_masks=None, allowed=None,
               dtype=torch.float32):
    """fp32 (or low-precision) oracle forward + backward on CPU copies of the inputs."""
    args = [t.detach().cpu() for t in (q, k, v, dout)]
    return orc.attention_varlen_grads(args[0], args[1], args[2], args[3], _as_list(cu_q),
                                      _as_list(cu_k), scale, causal, dropout_p, keep_masks,
                                      allowed, dtype)


def oracle_lse(q, k, v, cu_q, cu_k, scale, causal, allowed=None):
    _, lses = orc.attention_varlen_ref(q.detach().cpu(), k.detach().cpu(), v.detach().cpu(),
                                       _as_list(cu_q), _as_list(cu_k), scale, causal,
                                       allowed=allowed)
    return lses
