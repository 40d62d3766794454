"""Padding helpers: the counterpart of flash_attn/bert_padding.py in the reference.

`unpad_input` turns a padded (batch, seqlen, dim) tensor plus a validity mask into the packed
(total, dim) layout with int32 cu_seqlens that the attention functions take; `pad_input` is its
inverse.  Both are differentiable.
"""
import torch
import torch.nn.functional as F


class IndexFirstAxis(torch.autograd.Function):
    """rows = input[indices] on a 2-D input (reference :9-29)."""

    @staticmethod
    def forward(ctx, input, indices):
        assert input.ndim == 2
        ctx.save_for_backward(indices)
        ctx.first_axis_dim = input.shape[0]
        return input.index_select(0, indices)

    @staticmethod
    def backward(ctx, grad_output):
        (indices,) = ctx.saved_tensors
        grad_input = grad_output.new_zeros((ctx.first_axis_dim,) + tuple(grad_output.shape[1:]))
        grad_input.index_copy_(0, indices, grad_output)
        return grad_input, None


index_first_axis = IndexFirstAxis.apply


class IndexPutFirstAxis(torch.autograd.Function):
    """output[indices] = values on a zero (first_axis_dim, dim) tensor (reference :35-54)."""

    @staticmethod
    def forward(ctx, values, indices, first_axis_dim):
        assert indices.ndim == 1 and values.ndim == 2
        ctx.save_for_backward(indices)
        output = values.new_zeros((first_axis_dim, values.shape[1]))
        output.index_copy_(0, indices, values)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        (indices,) = ctx.saved_tensors
        return grad_output.index_select(0, indices), None, None


index_put_first_axis = IndexPutFirstAxis.apply


def unpad_input(hidden_states, attention_mask):
    """hidden_states (batch, seqlen, dim); attention_mask (batch, seqlen) bool / int, non-zero =
    valid token.  Returns (packed (total, dim), indices (total,), cu_seqlens (batch + 1,) int32,
    max_seqlen_in_batch int) (reference :60-80)."""
    seqlens_in_batch = attention_mask.sum(dim=-1, dtype=torch.int32)
    indices = torch.nonzero(attention_mask.flatten(), as_tuple=False).flatten()
    max_seqlen_in_batch = int(seqlens_in_batch.max().item())
    cu_seqlens = F.pad(torch.cumsum(seqlens_in_batch, dim=0, dtype=torch.int32), (1, 0))
    flat = hidden_states.reshape(-1, hidden_states.shape[-1])
    return index_first_axis(flat, indices), indices, cu_seqlens, max_seqlen_in_batch


def pad_input(hidden_states, indices, batch, seqlen):
    """Inverse of unpad_input: (total, dim) -> (batch, seqlen, dim), zeros at padded positions
    (reference :83-95)."""
    output = index_put_first_axis(hidden_states, indices, batch * seqlen)
    return output.reshape(batch, seqlen, hidden_states.shape[-1])
