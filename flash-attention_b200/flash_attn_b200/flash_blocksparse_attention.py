"""nn.Module wrappers for block-sparse attention: the counterpart of
flash_attn/flash_blocksparse_attention.py in the reference (FlashBlocksparseAttention :14-104,
FlashBlocksparseMHA :107-136)."""
import torch
import torch.nn as nn

from .bert_padding import pad_input, unpad_input
from .flash_blocksparse_attn_interface import convert_blockmask, flash_blocksparse_attn_func


def _make_layout(sparsity_config, max_seq_length):
    """`sparsity_config` may be a ready 0/1 layout tensor of shape (seq/16, seq/256), an object with
    a make_layout(seq_len) method (sparsity_layouts.py has several), or a hydra config describing
    such an object (the reference's only form, :27-33; hydra is imported only in that case)."""
    if torch.is_tensor(sparsity_config):
        return sparsity_config
    if not hasattr(sparsity_config, "make_layout"):
        import hydra  # optional dependency, as in the reference
        sparsity_config = hydra.utils.instantiate(sparsity_config)
    return sparsity_config.make_layout(max_seq_length)


class FlashBlocksparseAttention(nn.Module):
    """Block-sparse scaled dot-product attention.

    softmax_temp        multiplier of Q K^T (default 1 / sqrt(head_dim))
    attention_dropout   dropout probability, applied in training mode only
    max_seq_length      rounded up to a multiple of 256; the layout covers that length
    """

    def __init__(self, sparsity_config, softmax_temp=None, attention_dropout=0.0,
                 max_seq_length=2048, device=None, dtype=None):
        super().__init__()
        self.softmax_temp = softmax_temp
        self.dropout_p = attention_dropout
        max_seq_length = ((max_seq_length + 255) // 256) * 256
        layout = _make_layout(sparsity_config, max_seq_length)
        if device is not None:
            layout = layout.to(device)
        self.register_buffer("layout", layout)
        self.register_buffer("blockmask_converted", convert_blockmask(self.layout, causal=False))
        self.register_buffer("blockmask_converted_causal", convert_blockmask(self.layout, causal=True))

    def _layout_for(self, seqlen):
        rounded = ((seqlen + 255) // 256) * 256
        assert rounded // 16 <= self.layout.shape[0] and rounded // 256 <= self.layout.shape[1]
        return self.layout[:rounded // 16, :rounded // 256]

    def forward(self, qkv, attn_mask=None, key_padding_mask=None, causal=False, cu_seqlens=None,
                max_s=None, need_weights=False, convert_mask=True):
        """qkv (batch, seqlen, 3, heads, d) when cu_seqlens is None, else packed (total, 3, heads, d).
        Returns (output, None)."""
        assert not need_weights
        assert attn_mask is None
        assert qkv.dtype == torch.float16
        assert qkv.is_cuda
        p = self.dropout_p if self.training else 0.0

        if cu_seqlens is not None:
            assert max_s is not None
            if convert_mask:
                out = flash_blocksparse_attn_func(qkv, cu_seqlens, self._layout_for(max_s), p, max_s,
                                                  softmax_scale=self.softmax_temp, causal=causal)
            else:
                converted = self.blockmask_converted_causal if causal else self.blockmask_converted
                out = flash_blocksparse_attn_func(qkv, cu_seqlens, converted, p, max_s,
                                                  softmax_scale=self.softmax_temp, causal=causal,
                                                  convert_mask=False)
            return out, None

        batch, seqlen, three, heads, d = qkv.shape
        blockmask = self._layout_for(seqlen)
        if key_padding_mask is None:
            cu = torch.arange(0, (batch + 1) * seqlen, step=seqlen, dtype=torch.int32, device=qkv.device)
            out = flash_blocksparse_attn_func(qkv.reshape(batch * seqlen, three, heads, d), cu, blockmask,
                                              p, seqlen, softmax_scale=self.softmax_temp, causal=causal)
            return out.reshape(batch, seqlen, heads, d), None
        mask = getattr(key_padding_mask, "bool_matrix", key_padding_mask)
        x_unpad, indices, cu, max_len = unpad_input(qkv.reshape(batch, seqlen, three * heads * d), mask)
        # the layout must cover max_len rounded up to 256, which may be shorter than seqlen
        out_unpad = flash_blocksparse_attn_func(x_unpad.reshape(-1, three, heads, d), cu,
                                                self._layout_for(max_len), p, max_len,
                                                softmax_scale=self.softmax_temp, causal=causal)
        out = pad_input(out_unpad.reshape(-1, heads * d), indices, batch, seqlen)
        return out.reshape(batch, seqlen, heads, d), None


class FlashBlocksparseMHA(nn.Module):
    """Multi-head self-attention block around FlashBlocksparseAttention."""

    def __init__(self, embed_dim, num_heads, sparsity_config, bias=True, batch_first=True,
                 attention_dropout=0.0, causal=False, max_seq_length=2048, device=None, dtype=None,
                 **kwargs):
        assert batch_first
        factory_kwargs = {"device": device, "dtype": dtype}
        super().__init__()
        self.embed_dim = embed_dim
        self.causal = causal
        self.num_heads = num_heads
        assert embed_dim % num_heads == 0, "embed_dim must be divisible by num_heads"
        self.head_dim = embed_dim // num_heads
        assert self.head_dim in (16, 32, 64), "head_dim must be 16, 32 or 64"
        self.Wqkv = nn.Linear(embed_dim, 3 * embed_dim, bias=bias, **factory_kwargs)
        self.inner_attn = FlashBlocksparseAttention(sparsity_config, attention_dropout=attention_dropout,
                                                    max_seq_length=max_seq_length, **factory_kwargs)
        self.out_proj = nn.Linear(embed_dim, embed_dim, bias=bias, **factory_kwargs)

    def forward(self, x, x_ignored_=None, x_ignored_1_=None, attn_mask=None, key_padding_mask=None,
                need_weights=False):
        batch, seqlen, _ = x.shape
        qkv = self.Wqkv(x).reshape(batch, seqlen, 3, self.num_heads, self.head_dim)
        context, attn_weights = self.inner_attn(qkv, key_padding_mask=key_padding_mask,
                                                need_weights=need_weights, causal=self.causal)
        return self.out_proj(context.reshape(batch, seqlen, self.embed_dim)), attn_weights
