"""Rotary position embeddings used by FlashMHA(use_rotary_emb=...): same results as
flash_attn/rotary.py in the reference (consecutive channel pairs (2i, 2i+1) are rotated by
position * 10000^(-2i/dim)), written as a complex multiplication."""
import math

import torch


def _rotate(x, angles):
    """x (..., seqlen-broadcastable, dim); angles broadcastable to (..., dim/2)."""
    xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
    rot = torch.polar(torch.ones_like(angles), angles)
    return torch.view_as_real(xc * rot).flatten(-2).to(x.dtype)


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
