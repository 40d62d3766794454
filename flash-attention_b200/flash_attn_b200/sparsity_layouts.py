"""Sparsity layouts for FlashBlocksparseAttention.

The reference builds its layout with `hydra.utils.instantiate(sparsity_config).make_layout(seqlen)`
(flash_attn/flash_blocksparse_attention.py:27-33) from configuration classes that are not part
of its tree.  The classes here provide that `make_layout` interface directly, so the module works
without hydra: each returns the 0/1 int32 matrix over (16-row query blocks, 256-column key blocks)
that `convert_blockmask` consumes, of shape (seq_len / 16, seq_len / 256) for a seq_len that is a
multiple of 256.  Patterns are defined on 256 x 256 blocks (every 256-row block is 16 identical
layout rows) and always keep the diagonal, so no query row is left without a key.
"""
import torch


class _BlockLayout:
    block = 256

    def block_pattern(self, n):
        """bool (n, n): which 256 x 256 blocks are kept, before the diagonal is added."""
        raise NotImplementedError

    def make_layout(self, seq_len):
        if seq_len % self.block != 0:
            raise ValueError("seq_len must be a multiple of %d, got %d" % (self.block, seq_len))
        n = seq_len // self.block
        pattern = self.block_pattern(n).to(torch.bool) | torch.eye(n, dtype=torch.bool)
        return pattern.repeat_interleave(self.block // 16, dim=0).to(torch.int32)


class DenseLayout(_BlockLayout):
    """Every block: block-sparse attention that equals dense attention."""

    def block_pattern(self, n):
        return torch.ones(n, n, dtype=torch.bool)


class FixedLayout(_BlockLayout):
    """The "fixed" pattern of sparse transformers: blocks attend within their local window of
    `local_blocks` consecutive blocks, and to the last `global_blocks` blocks of every window."""

    def __init__(self, local_blocks=4, global_blocks=1):
        self.local_blocks, self.global_blocks = int(local_blocks), int(global_blocks)

    def block_pattern(self, n):
        idx = torch.arange(n)
        same_window = (idx[:, None] // self.local_blocks) == (idx[None, :] // self.local_blocks)
        is_global = (idx % self.local_blocks) >= self.local_blocks - self.global_blocks
        return same_window | is_global[None, :]


class SlidingWindowLayout(_BlockLayout):
    """A band of `window_blocks` blocks on either side of the diagonal plus `global_blocks` leading
    blocks that every query sees and that see every key (the long-document pattern)."""

    def __init__(self, window_blocks=1, global_blocks=1):
        self.window_blocks, self.global_blocks = int(window_blocks), int(global_blocks)

    def block_pattern(self, n):
        idx = torch.arange(n)
        band = (idx[:, None] - idx[None, :]).abs() <= self.window_blocks
        glob = (idx[None, :] < self.global_blocks) | (idx[:, None] < self.global_blocks)
        return band | glob


class RandomLayout(_BlockLayout):
    """Each block kept with probability `density` from a seeded generator (plus the diagonal)."""

    def __init__(self, density=0.25, seed=0):
        self.density, self.seed = float(density), int(seed)

    def block_pattern(self, n):
        g = torch.Generator().manual_seed(self.seed)
        return torch.rand(n, n, generator=g) < self.density
