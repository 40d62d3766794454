"""Rotary position embeddings used by FlashMHA(use_rotary_emb=...): same results as
flash_attn/rotary.py in the reference (consecutive channel pairs (2i, 2i+1) are rotated by
position * 10000^(-2i/dim)), written as a complex multiplication."""
import ctypes
import math

import torch

from ._lib import check, lib


def _rotate(x, angles):
    """x (..., seqlen-broadcastable, dim); angles broadcastable to (..., dim/2)."""
    xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
    rot = torch.polar(torch.ones_like(angles), angles)
    return torch.view_as_real(xc * rot).flatten(-2).to(x.dtype)


class _RotaryQKV(torch.autograd.Function):
    """Rotation of the q and k parts of a packed (batch, seqlen, 3, heads, d) tensor by the library's
    one-pass kernel (fa_rotary_qkv); the gradient is the rotation by the negative angles."""

    @staticmethod
    def _run(qkv, cos, sin, conjugate):
        batch, seqlen, _, heads, d = qkv.shape
        out = torch.empty_like(qkv)
        with torch.cuda.device(qkv.device):
            stream = ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(qkv.device.index))
            check(lib.fa_rotary_qkv(qkv.data_ptr(), out.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                    batch * seqlen, seqlen, heads, d,
                                    1 if qkv.dtype is torch.bfloat16 else 0, 1 if conjugate else 0, stream))
        return out

    @staticmethod
    def forward(ctx, qkv, cos, sin):
        ctx.save_for_backward(cos, sin)
        return _RotaryQKV._run(qkv, cos, sin, False)

    @staticmethod
    def backward(ctx, grad):
        cos, sin = ctx.saved_tensors
        return _RotaryQKV._run(grad.contiguous(), cos, sin, True), None, None


class RotaryEmbedding(torch.nn.Module):
    def __init__(self, dim_model, *_, **__):
        super().__init__()
        inv_freq = 1.0 / (10000 ** (torch.arange(0, dim_model, 2).float() / dim_model))
        self.register_buffer("inv_freq", inv_freq)

    def _angles(self, x, seq_dimension):
        seqlen = x.shape[seq_dimension]
        t = torch.arange(seqlen, device=x.device, dtype=self.inv_freq.dtype)
        ang = torch.outer(t, self.inv_freq.to(x.device))      # (seqlen, dim/2)
        return ang[:, None, :] if seq_dimension == -3 else ang

    def forward(self, q, k, seq_dimension=-2):
        """q, k: (..., seqlen, dim) for seq_dimension -2 or (..., seqlen, heads, dim) for -3."""
        assert seq_dimension in (-2, -3)
        ang = self._angles(k, seq_dimension)
        return (_rotate(q, ang[:q.shape[seq_dimension]]), _rotate(k, ang))

    @staticmethod
    def fused_path(qkv):
        """The one-pass kernel takes a contiguous 16-bit CUDA tensor (batch, seqlen, 3, heads, d) with
        d a multiple of 8."""
        return (qkv.is_cuda and qkv.dim() == 5 and qkv.shape[2] == 3 and qkv.is_contiguous()
                and qkv.dtype in (torch.float16, torch.bfloat16) and qkv.shape[-1] % 8 == 0
                and qkv.data_ptr() % 16 == 0)

    def apply_qkv(self, qkv):
        """(batch, seqlen, 3, heads, d) -> the same layout with q and k rotated, v unchanged: what
        forward(q, k, seq_dimension=-3) followed by a re-stack computes, in one pass over qkv."""
        if not self.fused_path(qkv):
            q, k, v = qkv.unbind(dim=2)
            q, k = self.forward(q, k, seq_dimension=-3)
            return torch.stack([q, k, v], dim=2)
        seqlen = qkv.shape[1]
        key = (seqlen, qkv.device)
        if getattr(self, "_table_key", None) != key:
            # fp32 tables, kept until the sequence length or the device changes (the reference
            # caches its tables the same way, flash_attn/rotary.py:72-88)
            t = torch.arange(seqlen, device=qkv.device, dtype=self.inv_freq.dtype)
            ang = torch.outer(t, self.inv_freq.to(qkv.device))        # (seqlen, d / 2)
            self._cos_table, self._sin_table = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
            self._table_key = key
        return _RotaryQKV.apply(qkv, self._cos_table, self._sin_table)


class RotaryEmbedding2D(torch.nn.Module):
    """For sequences that are flattened h x w grids: the first half of the channels is rotated by
    the column index, the second half by the row index."""

    def __init__(self, dim):
        super().__init__()
        assert dim % 4 == 0
        self.rotary_emb1d = RotaryEmbedding(dim // 2)

    def forward(self, q, k, seq_dimension=-2):
        assert seq_dimension in (-2, -3)
        seqlen = q.shape[seq_dimension]
        side = int(math.sqrt(seqlen))
        assert side * side == seqlen
        if seq_dimension == -3:
            q, k = q.transpose(1, 2), k.transpose(1, 2)       # (b, heads, s, d)

        def grid(x):
            return x.reshape(*x.shape[:2], side, side, x.shape[-1])

        q0, q1 = q.chunk(2, dim=-1)
        k0, k1 = k.chunk(2, dim=-1)
        q0e, k0e = self.rotary_emb1d(grid(q0), grid(k0), seq_dimension=-2)   # column index
        q1e, k1e = self.rotary_emb1d(grid(q1), grid(k1), seq_dimension=-3)   # row index
        qe = torch.cat([q0e.flatten(2, 3), q1e.flatten(2, 3)], dim=-1)
        ke = torch.cat([k0e.flatten(2, 3), k1e.flatten(2, 3)], dim=-1)
        if seq_dimension == -3:
            qe, ke = qe.transpose(1, 2), ke.transpose(1, 2)
        return qe, ke

    def apply_qkv(self, qkv):
        """(batch, seqlen, 3, heads, d) with seqlen = side * side -> q and k rotated, v unchanged,
        in one pass of the same kernel the 1-D embedding uses: the 2-D scheme is a per-position
        angle table like any other -- token p = row * side + col turns the channel pairs of the
        first half of d by col * f_i and those of the second half by row * f_i, f_i the
        frequencies of a (d / 2)-wide 1-D embedding (reference flash_attn/rotary.py:103-135)."""
        if not RotaryEmbedding.fused_path(qkv):
            q, k, v = qkv.unbind(dim=2)
            q, k = self.forward(q, k, seq_dimension=-3)
            return torch.stack([q, k, v], dim=2)
        seqlen = qkv.shape[1]
        side = int(math.sqrt(seqlen))
        assert side * side == seqlen
        key = (seqlen, qkv.device)
        if getattr(self, "_table_key", None) != key:
            inv_freq = self.rotary_emb1d.inv_freq.to(qkv.device)          # d / 4 frequencies
            pos = torch.arange(seqlen, device=qkv.device)
            col = (pos % side).to(inv_freq.dtype)
            row = torch.div(pos, side, rounding_mode="floor").to(inv_freq.dtype)
            ang = torch.cat([torch.outer(col, inv_freq), torch.outer(row, inv_freq)], dim=-1)   # (seqlen, d / 2)
            self._cos_table, self._sin_table = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
            self._table_key = key
        return _RotaryQKV.apply(qkv, self._cos_table, self._sin_table)
