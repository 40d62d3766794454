"""Standard attention of ONE (batch, head) pair at full benchmark size, evaluated only where a
test looks -- TEST INFRASTRUCTURE ONLY (imported by tests/, never by the product).

The parity tests at the benchmark shapes (sequences of 4096 ... 65536) cannot afford the dense
oracle for every (batch, head).  This module runs the same mathematics as
`attention_oracle.attention_varlen_grads` -- the reference's `attention_ref`
(benchmarks/benchmark_flash_attention.py:14-36) plus its autograd backward -- for one pair, in
chunks of query rows, and returns

    O, LSE, dQ  at a list of sampled query rows   (each needs its whole row of scores),
    dK, dV      at a list of sampled key rows     (each needs its whole column, i.e. every query).

Two modes in one pass: fp32, and an emulation of the same PyTorch program run in the 16-bit input
type (every operator reads 16-bit tensors, accumulates in fp32 and rounds its output to 16 bits,
which is what the framework's fp16 / bf16 CPU and GPU kernels do).  The second is the "same math in
the 16-bit type" comparator of the parity rule: max|kernel - fp32| <= 2 * max|16-bit - fp32|.
"""
import torch


def _round_to(dtype):
    if dtype is None or dtype == torch.float32:
        return lambda x: x
    return lambda x: x.to(dtype).to(torch.float32)


def sampled_attention_grads(q, k, v, dout, softmax_scale, causal, q_rows, k_rows, dropout_p=0.0,
                            keep_fn=None, allowed_fn=None, lowp_dtype=None, chunk=1024):
    """q, dout (sq, d); k, v (sk, d): fp32 CPU tensors holding the kernel's 16-bit inputs.

    q_rows / k_rows   sorted lists of sampled query / key indices
    keep_fn(r0, r1)   -> bool (r1 - r0, sk) dropout keep mask of query rows [r0, r1), or None
    allowed_fn(r0,r1) -> bool (r1 - r0, sk) block-sparse layout mask of those rows, or None
    lowp_dtype        None: fp32 mathematics; torch.float16 / bfloat16: the 16-bit emulation

    Returns dict(out (nq, d), lse (nq,), dq (nq, d), dk (nk, d), dv (nk, d)), fp32 tensors.
    """
    rnd = _round_to(lowp_dtype)
    sq, d = q.shape
    sk = k.shape[0]
    qf, kf, vf, gf = (t.to(torch.float32) for t in (q, k, v, dout))
    ks = rnd(kf * softmax_scale)                       # `k * softmax_scale` (attention_ref: k / sqrt(d))
    q_rows_t = torch.as_tensor(q_rows, dtype=torch.long)
    k_rows_t = torch.as_tensor(k_rows, dtype=torch.long)
    inv_keep = 1.0 / (1.0 - dropout_p)
    nq, nk = len(q_rows), len(k_rows)
    out = torch.zeros(nq, d)
    lse = torch.full((nq,), float("-inf"))
    dq = torch.zeros(nq, d)
    dks = torch.zeros(nk, d)                           # gradient of (k * scale), fp32 accumulation
    dv = torch.zeros(nk, d)

    for r0 in range(0, sq, chunk):
        r1 = min(sq, r0 + chunk)
        kmax = min(sk, r1) if causal else sk           # keys beyond the chunk's last row are masked anyway
        if kmax == 0:
            continue
        s = rnd(qf[r0:r1] @ ks[:kmax].T)               # scores
        if causal:
            i = torch.arange(r0, r1)[:, None]
            j = torch.arange(kmax)[None, :]
            s.masked_fill_(j > i, float("-inf"))
        if allowed_fn is not None:
            s.masked_fill_(~allowed_fn(r0, r1)[:, :kmax], float("-inf"))
        row_lse = torch.logsumexp(s, dim=-1)           # from the (possibly rounded) scores, in fp32
        a = torch.softmax(s, dim=-1)
        a = rnd(torch.nan_to_num(a, nan=0.0))          # rows without any valid key
        del s
        if keep_fn is not None:
            keep = keep_fn(r0, r1)[:, :kmax].to(torch.float32)
            ad = rnd(rnd(a * keep) * inv_keep)         # attention * mask / (1 - p)
        else:
            keep = None
            ad = a
        # backward of this chunk: d(attention_drop) = dout v^T
        g = rnd(gf[r0:r1] @ vf[:kmax].T)
        if keep is not None:
            g = rnd(rnd(g * inv_keep) * keep)
        rs = (g * a).sum(dim=-1, keepdim=True)         # softmax backward accumulates in fp32
        ds = rnd((g - rs) * a)
        del g
        # sampled key rows: whole-column sums accumulate over the chunks
        cols = k_rows_t < kmax
        if cols.any():
            idx = k_rows_t[cols]
            dks[cols] += ds[:, idx].T @ qf[r0:r1]
            dv[cols] += ad[:, idx].T @ gf[r0:r1]
        # sampled query rows inside this chunk
        sel = (q_rows_t >= r0) & (q_rows_t < r1)
        if sel.any():
            loc = q_rows_t[sel] - r0
            out[sel] = rnd(ad[loc] @ vf[:kmax])
            lse[sel] = row_lse[loc]
            dq[sel] = rnd(ds[loc] @ ks[:kmax])
        del a, ad, ds
    return {"out": out, "lse": lse, "dq": dq, "dk": rnd(rnd(dks) * softmax_scale), "dv": rnd(dv)}
