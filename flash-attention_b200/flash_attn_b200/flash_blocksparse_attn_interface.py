"""Block-sparse attention, functional API: the counterpart of
flash_attn/flash_blocksparse_attn_interface.py in the reference.

The sparsity layout is a 0/1 matrix over (16-row query blocks, 256-column key blocks).
`convert_blockmask` turns it into the per-key-block visit lists the kernels consume.
"""
import torch

from . import flash_attn_cuda


def convert_blockmask(blockmask, causal):
    """0/1 layout (rows, cols) -> int32 (cols, rows): row c lists, in ascending order, 4 * r for
    every non-zero (r, c), plus 1 when c is the first non-zero column of row r and plus 2 when it
    is the last; the rest of the row is -1.  Same output as the reference function (:8-40).

    causal=True (the reference asserts `not causal`, :21): blocks that lie entirely above the
    diagonal -- first key column 256 * c behind the last query row 16 * r + 15 -- are removed
    from the layout first, so they are neither visited nor counted; inside the remaining blocks
    the kernels apply the causal mask element by element.  The dropout mask of a causal call is
    the block-sparse one of the reduced layout: as in the reference's block kernels, the Philox
    iteration index follows the visit lists alone (csrc/flash_attn/src/
    fmha_block_fprop_kernel_1xN.h:205-232 takes its loop bounds from the block mask, with no
    causal start row)."""
    mask = blockmask != 0
    nrow, ncol = mask.shape
    device = mask.device
    cols = torch.arange(ncol, device=device)
    if causal:
        last_query = 16 * torch.arange(nrow, device=device)[:, None] + 15
        mask = mask & (256 * cols[None, :] <= last_query)
    # first / last non-zero column of each row (ncol / -1 when the row is empty)
    first = torch.where(mask, cols[None, :], torch.full_like(cols, ncol)[None, :]).min(dim=1).values
    last = torch.where(mask, cols[None, :], torch.full_like(cols, -1)[None, :]).max(dim=1).values
    rows = torch.arange(nrow, device=device)[:, None]
    value = 4 * rows + (cols[None, :] == first[:, None]).long() + 2 * (cols[None, :] == last[:, None]).long()
    value = torch.where(mask, value, torch.full_like(value, -1))
    # move the non-zero entries of every column to the front, keeping row order
    order = torch.sort((~mask).to(torch.uint8), dim=0, stable=True).indices
    return torch.gather(value, 0, order).t().contiguous().to(torch.int32)


def _flash_blocksparse_attn_forward(qkv, cu_seqlens, blockmask, dropout_p, max_s, softmax_scale,
                                    causal, return_softmax):
    res = flash_attn_cuda.fwd_block(qkv, cu_seqlens, blockmask, dropout_p, max_s, softmax_scale,
                                    causal, return_softmax, None)
    return res[0], res[1], (res[2] if return_softmax else None)


def _flash_blocksparse_attn_backward(dout, qkv, out, S_dmask, softmax_lse, cu_seqlens, blockmask,
                                     dropout_p, max_s, softmax_scale, causal):
    dqkv, _, _ = flash_attn_cuda.bwd_block(dout, qkv, out, S_dmask, softmax_lse, cu_seqlens,
                                           blockmask, dropout_p, softmax_scale, max_s, causal, None)
    return dqkv


class FlashBlocksparseAttnFun(torch.autograd.Function):
    """Block-sparse self-attention on packed qkv (reference :64-96)."""

    RETURN_SOFTMAX = False

    @classmethod
    def _fwd(cls, ctx, qkv, cu_seqlens, blockmask, dropout_p, max_s, softmax_scale, causal):
        rng_state = torch.cuda.get_rng_state(qkv.device) if dropout_p > 0 else None
        if softmax_scale is None:
            softmax_scale = qkv.shape[-1] ** (-0.5)
        context, softmax_lse, s_dmask = _flash_blocksparse_attn_forward(
            qkv, cu_seqlens, blockmask, dropout_p, max_s, softmax_scale, causal, cls.RETURN_SOFTMAX)
        ctx.save_for_backward(qkv, context, softmax_lse, cu_seqlens, blockmask, rng_state)
        ctx.dropout_p, ctx.max_s, ctx.softmax_scale, ctx.causal = dropout_p, max_s, softmax_scale, causal
        return context, s_dmask, softmax_lse

    @staticmethod
    def _bwd(ctx, dout):
        qkv, context, softmax_lse, cu_seqlens, blockmask, rng_state = ctx.saved_tensors
        if rng_state is not None:
            cur_rng_state = torch.cuda.get_rng_state(qkv.device)
            torch.cuda.set_rng_state(rng_state, qkv.device)
        dqkv = _flash_blocksparse_attn_backward(dout, qkv, context, context, softmax_lse, cu_seqlens,
                                                blockmask, ctx.dropout_p, ctx.max_s,
                                                ctx.softmax_scale, ctx.causal)
        if rng_state is not None:
            torch.cuda.set_rng_state(cur_rng_state, qkv.device)
        return dqkv

    @staticmethod
    def forward(ctx, qkv, cu_seqlens, blockmask, dropout_p, max_s, softmax_scale, causal):
        return FlashBlocksparseAttnFun._fwd(ctx, qkv, cu_seqlens, blockmask, dropout_p, max_s,
                                            softmax_scale, causal)[0]

    @staticmethod
    def backward(ctx, dout):
        return FlashBlocksparseAttnFun._bwd(ctx, dout), None, None, None, None, None, None


class FlashBlocksparseAttnFunWithS(FlashBlocksparseAttnFun):
    """Variant that also returns (S_dmask, softmax_lse), for testing (reference :101-132)."""

    RETURN_SOFTMAX = True

    @staticmethod
    def forward(ctx, qkv, cu_seqlens, blockmask, dropout_p, max_s, softmax_scale, causal):
        return FlashBlocksparseAttnFunWithS._fwd(ctx, qkv, cu_seqlens, blockmask, dropout_p, max_s,
                                                 softmax_scale, causal)

    @staticmethod
    def backward(ctx, dout, _ds_dmask_ignored, _dlse_ignored):
        return FlashBlocksparseAttnFun._bwd(ctx, dout), None, None, None, None, None, None


def flash_blocksparse_attn_func(qkv, cu_seqlens, blockmask, dropout_p, max_s, softmax_scale=None,
                                causal=False, return_attn_probs=False, convert_mask=True):
    """Block-sparse variable-length self-attention.  qkv (total, 3, heads, d) fp16, blockmask a 0/1
    layout of shape (ceil(max_s / 256) * 16, ceil(max_s / 256)) (or an already converted mask with
    convert_mask=False).  dropout_p should be 0.0 for evaluation."""
    func = FlashBlocksparseAttnFunWithS if return_attn_probs else FlashBlocksparseAttnFun
    if convert_mask:
        blockmask = convert_blockmask(blockmask, causal=causal)
    return func.apply(qkv, cu_seqlens, blockmask, dropout_p, max_s, softmax_scale, causal)
