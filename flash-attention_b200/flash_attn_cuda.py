"""`import flash_attn_cuda` -- the module name the reference's Python files import
(flash_attn/flash_attn_interface.py:4, flash_attn/flash_blocksparse_attn_interface.py:5) and
that its build produces as a compiled extension (setup.py:117-150,
csrc/flash_attn/fmha_api.cpp:721-727).

With this directory on sys.path ahead of any compiled extension of that name, the reference's
own `flash_attn/*.py` run unmodified on top of libfa_b200.so: the four entry points below take
the positional argument lists of the reference's call sites.
"""
from flash_attn_b200.flash_attn_cuda import bwd, bwd_block, fwd, fwd_block  # noqa: F401

__all__ = ["fwd", "bwd", "fwd_block", "bwd_block"]
