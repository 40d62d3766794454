"""Padding helpers: the counterpart of flash_attn/bert_padding.py in the reference.

`unpad_input` turns a padded (batch, seqlen, dim) tensor plus a validity mask into the packed
(total, dim) layout with int32 cu_seqlens that the attention functions take; `pad_input` is its
inverse.  Both are differentiable.  On CUDA tensors the row gather / scatter behind them runs as
one HBM-bound pass of the library's own kernels (fa_gather_rows / fa_scatter_rows).
"""
import ctypes

import torch
import torch.nn.functional as F

from ._lib import check, lib


def _kernel_path(values, indices):
    """The row kernels of the library take CUDA tensors with contiguous rows of a multiple of 16
    bytes and int64 indices; anything else (CPU tensors in particular) goes through framework
    indexing, which is what the reference always does."""
    return (values.is_cuda and indices.is_cuda and indices.dtype is torch.int64
            and values.dim() == 2 and values.is_contiguous() and indices.is_contiguous()
            and (values.shape[1] * values.element_size()) % 16 == 0 and values.data_ptr() % 16 == 0)


def _stream(device):
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(device.index))


def gather_rows(values, indices):
    """values[indices] for a 2-D `values`: one pass, 16-byte accesses."""
    if not _kernel_path(values, indices):
        return values.index_select(0, indices)
    out = torch.empty((indices.shape[0], values.shape[1]), dtype=values.dtype, device=values.device)
    with torch.cuda.device(values.device):
        check(lib.fa_gather_rows(values.data_ptr(), indices.data_ptr(), out.data_ptr(), indices.shape[0],
                                 values.shape[0], values.shape[1] * values.element_size(),
                                 _stream(values.device)))
    return out


def scatter_rows(values, indices, first_axis_dim):
    """(first_axis_dim, dim) tensor of zeros with rows `indices` set to `values`: the zero fill and
    the copy are one pass over the output."""
    if not _kernel_path(values, indices):
        out = values.new_zeros((first_axis_dim, values.shape[1]))
        out.index_copy_(0, indices, values)
        return out
    out = torch.empty((first_axis_dim, values.shape[1]), dtype=values.dtype, device=values.device)
    inverse = torch.empty(max(first_axis_dim, 1), dtype=torch.int32, device=values.device)
    with torch.cuda.device(values.device):
        check(lib.fa_scatter_rows(values.data_ptr(), indices.data_ptr(), out.data_ptr(), values.shape[0],
                                  first_axis_dim, values.shape[1] * values.element_size(),
                                  inverse.data_ptr(), _stream(values.device)))
    return out


class IndexFirstAxis(torch.autograd.Function):
    """rows = input[indices] on a 2-D input (reference :9-29)."""

    @staticmethod
    def forward(ctx, input, indices):
        assert input.ndim == 2
        ctx.save_for_backward(indices)
        ctx.first_axis_dim = input.shape[0]
        return gather_rows(input, indices)

    @staticmethod
    def backward(ctx, grad_output):
        (indices,) = ctx.saved_tensors
        return scatter_rows(grad_output.contiguous(), indices, ctx.first_axis_dim), None


index_first_axis = IndexFirstAxis.apply


class IndexPutFirstAxis(torch.autograd.Function):
    """output[indices] = values on a zero (first_axis_dim, dim) tensor (reference :35-54)."""

    @staticmethod
    def forward(ctx, values, indices, first_axis_dim):
        assert indices.ndim == 1 and values.ndim == 2
        ctx.save_for_backward(indices)
        return scatter_rows(values, indices, first_axis_dim)

    @staticmethod
    def backward(ctx, grad_output):
        (indices,) = ctx.saved_tensors
        return gather_rows(grad_output.contiguous(), indices), None, None


index_put_first_axis = IndexPutFirstAxis.apply


def unpad_input(hidden_states, attention_mask):
    """hidden_states (batch, seqlen, dim); attention_mask (batch, seqlen) bool / int, non-zero =
    valid token.  Returns (packed (total, dim), indices (total,), cu_seqlens (batch + 1,) int32,
    max_seqlen_in_batch int) (reference :60-80)."""
    seqlens_in_batch = attention_mask.sum(dim=-1, dtype=torch.int32)
    # One synchronisation, which the API cannot avoid (the packed size and max_seqlen are host values):
    # the lengths come to the host once and both are read from them; the index list is then built
    # with a known size, which does not synchronise again (the reference pays one for `nonzero` and
    # one for `.item()`, :70-72).
    seqlens_host = seqlens_in_batch.cpu()
    total = int(seqlens_host.sum())
    max_seqlen_in_batch = int(seqlens_host.max()) if seqlens_host.numel() else 0
    indices = torch.nonzero_static(attention_mask.flatten(), size=total).flatten()
    cu_seqlens = F.pad(torch.cumsum(seqlens_in_batch, dim=0, dtype=torch.int32), (1, 0))
    flat = hidden_states.reshape(-1, hidden_states.shape[-1])
    return index_first_axis(flat, indices), indices, cu_seqlens, max_seqlen_in_batch


def pad_input(hidden_states, indices, batch, seqlen):
    """Inverse of unpad_input: (total, dim) -> (batch, seqlen, dim), zeros at padded positions
    (reference :83-95)."""
    output = index_put_first_axis(hidden_states, indices, batch * seqlen)
    return output.reshape(batch, seqlen, hidden_states.shape[-1])
