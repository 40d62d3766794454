"""flash_attn_b200: FlashAttention for NVIDIA B200 (sm_100a) behind the Python API of
lw921014/flash-attention.

Public surface (same names and argument meaning as the reference's `flash_attn` package):

    flash_attn_interface              flash_attn_unpadded_func, flash_attn_unpadded_qkvpacked_func,
                                      flash_attn_unpadded_kvpacked_func, flash_attn_func
    flash_blocksparse_attn_interface  flash_blocksparse_attn_func, convert_blockmask
    flash_attention                   FlashAttention, FlashMHA
    flash_blocksparse_attention       FlashBlocksparseAttention, FlashBlocksparseMHA
    bert_padding                      unpad_input, pad_input, index_first_axis
    flash_attn_cuda                   fwd, bwd, fwd_block, bwd_block (extension-module contract)

Everything runs on hand-written sm_100a kernels in libfa_b200.so; there is no fallback path.
"""
__version__ = "0.1.0"
