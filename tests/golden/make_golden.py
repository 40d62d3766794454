"""Generates the golden fixtures in this directory from the reference's own Python code.

Run once where a checkout of the reference (lw921014/flash-attention) is available:

    python tests/golden/make_golden.py /path/to/reference      (or FA_REFERENCE_ROOT=... in the environment)

* attention_ref      is cut out of benchmarks/benchmark_flash_attention.py with `ast` (the script
                     itself cannot be imported: it imports the CUDA extension and runs GPU code at
                     import time) and executed on CPU.
* convert_blockmask  is cut out of flash_attn/flash_blocksparse_attn_interface.py the same way.
* unpad_input / pad_input are imported from flash_attn/bert_padding.py (pure PyTorch).

Inputs are regenerated in the tests from the recorded seeds; only outputs are stored.
"""
import ast
import importlib.util
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = None  # root of the reference checkout; set by the command line below


def extract_function(path, name, extra_globals):
    src = open(path).read()
    tree = ast.parse(src)
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            code = compile(ast.Module(body=[node], type_ignores=[]), path, "exec")
            ns = dict(extra_globals)
            exec(code, ns)
            return ns[name]
    raise KeyError(name)


def attention_inputs(seed, batch, seqlen, heads, d, lengths=None):
    """Seeded inputs shared by this script and tests/test_oracle.py."""
    g = torch.Generator().manual_seed(seed)
    qkv = torch.randn(batch, seqlen, 3, heads, d, generator=g)
    dout = torch.randn(batch, seqlen, heads, d, generator=g)
    if lengths is None:
        mask = torch.ones(batch, seqlen, dtype=torch.bool)
    else:
        mask = torch.arange(seqlen)[None, :] < torch.tensor(lengths)[:, None]
    return qkv, dout, mask


ATTENTION_CASES = {
    # name: (seed, batch, seqlen, heads, d, lengths, causal)
    "c1_b2_h12_s128_d64": (1234, 2, 128, 12, 64, None, False),
    "small_padded": (7, 3, 48, 2, 32, [48, 17, 33], False),
    "small_causal": (11, 2, 40, 3, 16, [40, 25], True),
}

BLOCKMASK_CASES = {
    # name: (seed, rows, cols, density)
    "bm_16x4": (3, 16, 4, 0.5),
    "bm_32x2": (5, 32, 2, 0.3),
    "bm_256x16_c4": (0, 256, 16, 0.25),
}


def blockmask_layout(seed, rows, cols, density):
    g = torch.Generator().manual_seed(seed)
    layout = (torch.rand(rows, cols, generator=g) < density)
    # every row and every column keeps at least one block, like a layout with its diagonal kept
    for r in range(rows):
        layout[r, (r * cols) // rows] = True
    return layout.to(torch.int32)


def main():
    from einops import rearrange
    import torch.nn.functional as F
    attention_ref = extract_function(
        os.path.join(REF, "benchmarks", "benchmark_flash_attention.py"), "attention_ref",
        {"torch": torch, "math": math, "rearrange": rearrange, "F": F})
    out = {}
    for name, (seed, b, s, h, d, lengths, causal) in ATTENTION_CASES.items():
        qkv, dout, mask = attention_inputs(seed, b, s, h, d, lengths)
        qkv = qkv.clone().requires_grad_()
        o = attention_ref(qkv, mask, 0.0, upcast=True, causal=causal)
        # padded query rows hold attention over valid keys too; the tests compare valid rows only
        (o * dout).sum().backward()
        o_np = o.detach().numpy().astype(np.float32)
        g_np = qkv.grad.numpy().astype(np.float32)
        if o_np.size > 40000:  # keep the fixture small: every 37th element plus the full sums
            out[name + "/out_stride37"] = o_np.reshape(-1)[::37].copy()
            out[name + "/dqkv_stride37"] = g_np.reshape(-1)[::37].copy()
            out[name + "/out_sum"] = np.float64(o_np.astype(np.float64).sum())
            out[name + "/dqkv_abs_sum"] = np.float64(np.abs(g_np.astype(np.float64)).sum())
        else:
            out[name + "/out"] = o_np
            out[name + "/dqkv"] = g_np
    np.savez_compressed(os.path.join(HERE, "attention_ref.npz"), **out)

    convert_blockmask = extract_function(
        os.path.join(REF, "flash_attn", "flash_blocksparse_attn_interface.py"), "convert_blockmask",
        {"torch": torch})
    bm = {}
    for name, (seed, rows, cols, density) in BLOCKMASK_CASES.items():
        layout = blockmask_layout(seed, rows, cols, density)
        bm[name] = convert_blockmask(layout, causal=False).numpy().astype(np.int32)
    np.savez_compressed(os.path.join(HERE, "convert_blockmask.npz"), **bm)

    spec = importlib.util.spec_from_file_location(
        "ref_bert_padding", os.path.join(REF, "flash_attn", "bert_padding.py"))
    bp = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bp)
    g = torch.Generator().manual_seed(21)
    x = torch.randn(4, 12, 8, generator=g)
    mask = torch.arange(12)[None, :] < torch.tensor([12, 5, 1, 9])[:, None]
    x_unpad, indices, cu_seqlens, max_s = bp.unpad_input(x, mask)
    x_pad = bp.pad_input(x_unpad, indices, 4, 12)
    np.savez_compressed(os.path.join(HERE, "bert_padding.npz"), x_unpad=x_unpad.numpy(),
                        indices=indices.numpy(), cu_seqlens=cu_seqlens.numpy(),
                        max_s=np.int64(max_s), x_pad=x_pad.numpy())
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FA_REFERENCE_ROOT")
    if not REF or not os.path.isdir(os.path.join(REF, "flash_attn")):
        sys.exit("usage: make_golden.py /path/to/reference (a checkout of lw921014/flash-attention)")
    main()
