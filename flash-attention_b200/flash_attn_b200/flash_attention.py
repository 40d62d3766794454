"""nn.Module wrappers: the counterpart of flash_attn/flash_attention.py in the reference
(FlashAttention :12-77, FlashMHA :80-118)."""
import torch
import torch.nn as nn

from .bert_padding import pad_input, unpad_input
from .flash_attn_interface import flash_attn_unpadded_qkvpacked_func
from .rotary import RotaryEmbedding, RotaryEmbedding2D


def _mask_matrix(key_padding_mask):
    """The reference expects an object with a `bool_matrix` attribute (:58); a plain bool / int
    tensor is accepted here as well."""
    return getattr(key_padding_mask, "bool_matrix", key_padding_mask)


class FlashAttention(nn.Module):
    """Scaled dot-product attention with softmax on a packed qkv tensor.

    softmax_scale      multiplier of Q K^T (default 1 / sqrt(head_dim), resolved per call)
    attention_dropout  dropout probability, applied in training mode only
    """

    def __init__(self, softmax_scale=None, attention_dropout=0.0, device=None, dtype=None):
        super().__init__()
        self.softmax_scale = softmax_scale
        self.dropout_p = attention_dropout

    def forward(self, qkv, attn_mask=None, key_padding_mask=None, causal=False, cu_seqlens=None,
                max_s=None, need_weights=False):
        """qkv is (batch, seqlen, 3, heads, d) when `cu_seqlens` is None, else already packed as
        (total, 3, heads, d) with `cu_seqlens` / `max_s` describing the sequences.
        key_padding_mask marks the valid tokens of a padded batch.  Returns (output, None);
        output has the layout of the input without the `3` axis."""
        assert not need_weights
        assert attn_mask is None
        assert qkv.dtype == torch.float16
        assert qkv.is_cuda
        p = self.dropout_p if self.training else 0.0

        if cu_seqlens is not None:
            assert max_s is not None
            out = flash_attn_unpadded_qkvpacked_func(qkv, cu_seqlens, max_s, p,
                                                     softmax_scale=self.softmax_scale, causal=causal)
            return out, None

        batch, seqlen, three, heads, d = qkv.shape
        if key_padding_mask is None:
            packed = qkv.reshape(batch * seqlen, three, heads, d)
            cu = torch.arange(0, (batch + 1) * seqlen, step=seqlen, dtype=torch.int32,
                              device=qkv.device)
            out = flash_attn_unpadded_qkvpacked_func(packed, cu, seqlen, p,
                                                     softmax_scale=self.softmax_scale, causal=causal)
            return out.reshape(batch, seqlen, heads, d), None

        mask = _mask_matrix(key_padding_mask)
        x_unpad, indices, cu, max_len = unpad_input(qkv.reshape(batch, seqlen, three * heads * d), mask)
        out_unpad = flash_attn_unpadded_qkvpacked_func(
            x_unpad.reshape(-1, three, heads, d), cu, max_len, p,
            softmax_scale=self.softmax_scale, causal=causal)
        out = pad_input(out_unpad.reshape(-1, heads * d), indices, batch, seqlen)
        return out.reshape(batch, seqlen, heads, d), None


class FlashMHA(nn.Module):
    """Multi-head self-attention block: Wqkv projection, optional rotary embedding, FlashAttention,
    output projection.  The projections are ordinary nn.Linear layers."""

    def __init__(self, embed_dim, num_heads, bias=True, batch_first=True, attention_dropout=0.0,
                 causal=False, use_rotary_emb=None, device=None, dtype=None, **kwargs):
        assert batch_first
        factory_kwargs = {"device": device, "dtype": dtype}
        super().__init__()
        self.embed_dim = embed_dim
        self.causal = causal
        self.num_heads = num_heads
        assert embed_dim % num_heads == 0, "embed_dim must be divisible by num_heads"
        self.head_dim = embed_dim // num_heads
        assert self.head_dim in (16, 32, 64, 128), "head_dim must be 16, 32, 64 or 128"
        assert use_rotary_emb in (None, "1d", "2d")
        self.use_rotary_emb = use_rotary_emb
        if use_rotary_emb == "1d":
            self.rotary_emb = RotaryEmbedding(self.head_dim)
        elif use_rotary_emb == "2d":
            self.rotary_emb = RotaryEmbedding2D(self.head_dim)
        self.Wqkv = nn.Linear(embed_dim, 3 * embed_dim, bias=bias, **factory_kwargs)
        self.inner_attn = FlashAttention(attention_dropout=attention_dropout, **factory_kwargs)
        self.out_proj = nn.Linear(embed_dim, embed_dim, bias=bias, **factory_kwargs)

    def forward(self, x, x_ignored_=None, x_ignored_1_=None, attn_mask=None, key_padding_mask=None,
                need_weights=False):
        batch, seqlen, _ = x.shape
        qkv = self.Wqkv(x).reshape(batch, seqlen, 3, self.num_heads, self.head_dim)
        if self.use_rotary_emb:
            qkv = self.rotary_emb.apply_qkv(qkv)   # one pass over qkv on CUDA, 1-D or 2-D angle table
        context, attn_weights = self.inner_attn(qkv, key_padding_mask=key_padding_mask,
                                                need_weights=need_weights, causal=self.causal)
        return self.out_proj(context.reshape(batch, seqlen, self.embed_dim)), attn_weights
