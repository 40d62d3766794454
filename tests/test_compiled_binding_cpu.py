"""The compiled binding loads without a GPU, exposes the two dense entry points, and rejects bad
arguments with the ctypes route's messages (no compute calls here)."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "flash-attention_b200"))


def test_binding_module_loads_and_checks_arguments():
    from flash_attn_b200 import flash_attn_cuda as fc
    if fc.binding_in_use() != "compiled":
        pytest.skip("compiled binding not built (python flash-attention_b200/build.py builds it)")
    from flash_attn_b200 import _fa_binding
    assert callable(_fa_binding.fwd) and callable(_fa_binding.bwd)
    x = torch.zeros(4, 2, 64, dtype=torch.float16)
    cu = torch.zeros(2, dtype=torch.int32)

    def call():
        fc.fwd(x, x, x, cu, cu, 4, 4, 0.0, 0.125, False, False, False, None)

    with pytest.raises(RuntimeError) as compiled:
        call()
    saved, fc._binding = fc._binding, None
    try:
        with pytest.raises(RuntimeError) as by_ctypes:
            call()
    finally:
        fc._binding = saved
    assert str(compiled.value).splitlines()[0] == str(by_ctypes.value) == "q, k, v must be CUDA tensors"
