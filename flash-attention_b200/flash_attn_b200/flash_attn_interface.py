"""Functional API with autograd: the counterpart of flash_attn/flash_attn_interface.py in the
reference (functions at :151-252, autograd classes at :39-148).

The three tensor layouts (packed qkv, q + packed kv, separate q/k/v) share one forward and one
backward helper; the autograd classes only differ in how they slice their inputs and in which
gradient buffers they allocate, so gradients of packed inputs are written straight into one
packed tensor through strided views, as the reference does (:64-68, :100-106).
"""
import torch

from . import flash_attn_cuda


def _get_block_size(device, head_dim, is_dropout):
    """Key-block size that fixes the dropout-mask layout (reference :7-14, evaluated for the A100
    branch, which is the layout this library reproduces)."""
    assert head_dim in (16, 32, 64, 128)
    if head_dim == 128:
        return 128 if is_dropout else 256
    return 256


def _flash_attn_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p,
                        softmax_scale, causal, return_softmax):
    res = flash_attn_cuda.fwd(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                              dropout_p, softmax_scale, False, causal, return_softmax, None)
    out, softmax_lse = res[0], res[1]
    return out, softmax_lse, (res[2] if return_softmax else None)


def _flash_attn_backward(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k,
                         max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale, causal):
    res = flash_attn_cuda.bwd(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q,
                              cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale,
                              False, causal, None)
    return dq, dk, dv, res[3]


class _VarlenAttnBase(torch.autograd.Function):
    """Shared forward / backward.  Subclasses define `_split(*packed)` -> (q, k, v) views and
    `_grad_buffers(*packed)` -> (packed gradient tensors, (dq, dk, dv) views into them)."""

    N_PACKED = 0

    @classmethod
    def _run_forward(cls, ctx, packed, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                     dropout_p, softmax_scale, causal, return_softmax):
        q, k, v = cls._split(*packed)
        # The backward pass regenerates the dropout mask from the generator state saved here.
        rng_state = torch.cuda.get_rng_state(q.device) if dropout_p > 0 else None
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        out, softmax_lse, s_dmask = _flash_attn_forward(
            q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p,
            softmax_scale, causal, return_softmax)
        ctx.save_for_backward(*packed, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, rng_state)
        ctx.dropout_p = dropout_p
        ctx.max_seqlen_q = max_seqlen_q
        ctx.max_seqlen_k = max_seqlen_k
        ctx.softmax_scale = softmax_scale
        ctx.causal = causal
        return out if not return_softmax else (out, softmax_lse, s_dmask)

    @classmethod
    def _run_backward(cls, ctx, dout):
        saved = ctx.saved_tensors
        packed = saved[:cls.N_PACKED]
        out, softmax_lse, cu_seqlens_q, cu_seqlens_k, rng_state = saved[cls.N_PACKED:]
        q, k, v = cls._split(*packed)
        device = q.device
        if rng_state is not None:
            cur_rng_state = torch.cuda.get_rng_state(device)
            torch.cuda.set_rng_state(rng_state, device)
        grads, (dq, dk, dv) = cls._grad_buffers(*packed)
        _flash_attn_backward(dout.contiguous(), q, k, v, out, softmax_lse, dq, dk, dv,
                             cu_seqlens_q, cu_seqlens_k, ctx.max_seqlen_q, ctx.max_seqlen_k,
                             ctx.dropout_p, ctx.softmax_scale, ctx.causal)
        if rng_state is not None:
            torch.cuda.set_rng_state(cur_rng_state, device)
        return grads


class FlashAttnQKVPackedFunc(_VarlenAttnBase):
    """Self-attention on qkv (total, 3, heads, d) (reference :39-72)."""
    N_PACKED = 1

    @staticmethod
    def _split(qkv):
        return qkv[:, 0], qkv[:, 1], qkv[:, 2]

    @staticmethod
    def _grad_buffers(qkv):
        dqkv = torch.empty_like(qkv)
        return (dqkv,), (dqkv[:, 0], dqkv[:, 1], dqkv[:, 2])

    @staticmethod
    def forward(ctx, qkv, cu_seqlens, max_seqlen, dropout_p, softmax_scale, causal, return_softmax):
        return FlashAttnQKVPackedFunc._run_forward(
            ctx, (qkv,), cu_seqlens, cu_seqlens, max_seqlen, max_seqlen, dropout_p, softmax_scale,
            causal, return_softmax)

    @staticmethod
    def backward(ctx, dout, *args):
        (dqkv,) = FlashAttnQKVPackedFunc._run_backward(ctx, dout)
        return dqkv, None, None, None, None, None, None


class FlashAttnKVPackedFunc(_VarlenAttnBase):
    """Cross-attention on q (total_q, heads, d) and kv (total_k, 2, heads, d) (reference :75-111)."""
    N_PACKED = 2

    @staticmethod
    def _split(q, kv):
        return q, kv[:, 0], kv[:, 1]

    @staticmethod
    def _grad_buffers(q, kv):
        dq, dkv = torch.empty_like(q), torch.empty_like(kv)
        return (dq, dkv), (dq, dkv[:, 0], dkv[:, 1])

    @staticmethod
    def forward(ctx, q, kv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p,
                softmax_scale, causal, return_softmax):
        return FlashAttnKVPackedFunc._run_forward(
            ctx, (q, kv), cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p,
            softmax_scale, causal, return_softmax)

    @staticmethod
    def backward(ctx, dout, *args):
        dq, dkv = FlashAttnKVPackedFunc._run_backward(ctx, dout)
        return dq, dkv, None, None, None, None, None, None, None, None


class FlashAttnFunc(_VarlenAttnBase):
    """Separate q, k, v (reference :114-148)."""
    N_PACKED = 3

    @staticmethod
    def _split(q, k, v):
        return q, k, v

    @staticmethod
    def _grad_buffers(q, k, v):
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        return (dq, dk, dv), (dq, dk, dv)

    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p,
                softmax_scale, causal, return_softmax):
        return FlashAttnFunc._run_forward(
            ctx, (q, k, v), cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p,
            softmax_scale, causal, return_softmax)

    @staticmethod
    def backward(ctx, dout, *args):
        dq, dk, dv = FlashAttnFunc._run_backward(ctx, dout)
        return dq, dk, dv, None, None, None, None, None, None, None, None


def flash_attn_unpadded_qkvpacked_func(qkv, cu_seqlens, max_seqlen, dropout_p, softmax_scale=None,
                                       causal=False, return_attn_probs=False):
    """Variable-length self-attention on packed tokens.

    qkv          (total, 3, heads, head_dim) fp16 / bf16, `total` = sum of sequence lengths
    cu_seqlens   (batch + 1,) int32 cumulative sequence lengths indexing into `total`
    max_seqlen   longest sequence in the batch
    dropout_p    dropout probability on the attention probabilities; use 0.0 for evaluation
    softmax_scale  multiplier of Q K^T, default 1 / sqrt(head_dim)
    causal       each query attends only to keys at or before its own position
    return_attn_probs  also return (softmax_lse, S_dmask), a testing aid

    Returns out (total, heads, head_dim); with return_attn_probs also softmax_lse
    (batch, heads, seqlen) fp32 = log-sum-exp of each row of softmax_scale * Q K^T, and S_dmask.
    """
    return FlashAttnQKVPackedFunc.apply(qkv, cu_seqlens, max_seqlen, dropout_p, softmax_scale,
                                        causal, return_attn_probs)


def flash_attn_unpadded_kvpacked_func(q, kv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                      dropout_p, softmax_scale=None, causal=False,
                                      return_attn_probs=False):
    """Variable-length cross-attention: q (total_q, heads, d) attends to kv (total_k, 2, heads, d).
    Query and key sequences have their own cu_seqlens / max_seqlen; other arguments and returns as
    in flash_attn_unpadded_qkvpacked_func.  With `causal`, key j is visible to query i when
    j <= i (both counted from the start of their sequence)."""
    return FlashAttnKVPackedFunc.apply(q, kv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                                       max_seqlen_k, dropout_p, softmax_scale, causal,
                                       return_attn_probs)


def flash_attn_unpadded_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                             dropout_p, softmax_scale=None, causal=False, return_attn_probs=False):
    """Variable-length attention with separate q (total_q, heads, d) and k, v (total_k, heads, d).
    Arguments and returns as in flash_attn_unpadded_kvpacked_func."""
    return FlashAttnFunc.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                               dropout_p, softmax_scale, causal, return_attn_probs)


def flash_attn_func(qkv, cu_seqlens, dropout_p, max_s, softmax_scale=None, causal=False,
                    return_attn_probs=False):
    """Older argument order of flash_attn_unpadded_qkvpacked_func, kept for callers of the
    reference's compatibility alias (:246-252)."""
    return flash_attn_unpadded_qkvpacked_func(qkv, cu_seqlens, max_s, dropout_p, softmax_scale,
                                              causal, return_attn_probs)
