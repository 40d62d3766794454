"""CPU tests of the C-ABI library: it loads without a GPU driver, exports every function that
include/fa_b200.h declares, and its host-only entry points and argument checks behave."""
import ctypes
import os
import re

import pytest

from oracle import attention_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "fa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fa_[a-z0-9_]+)\s*\(", text)))


def test_header_functions_are_exported():
    from flash_attn_b200 import _lib
    names = _declared_functions()
    assert "fa_fwd" in names and "fa_bwd" in names
    assert sorted(_lib.EXPORTED_SYMBOLS) == names
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in names:
        assert getattr(raw, name) is not None


def test_struct_layout_matches_header():
    """Field order of the ctypes mirrors equals the order of the members in the header."""
    from flash_attn_b200 import _lib
    text = open(os.path.join(ROOT, "include", "fa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)

    def members(struct):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (struct, struct), text, flags=re.S).group(1)
        out = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            names = decl.split(",")
            first = names[0].split()[-1].lstrip("*")
            out.append(first)
            out.extend(n.strip().lstrip("*") for n in names[1:])
        return out

    assert members("fa_fwd_params") == [f[0] for f in _lib.FwdParams._fields_]
    assert members("fa_bwd_params") == [f[0] for f in _lib.BwdParams._fields_]


def test_status_strings():
    from flash_attn_b200 import _lib
    assert _lib.lib.fa_status_string(0) == b"ok"
    for code in (-1, -2, -3, -4):
        assert _lib.lib.fa_status_string(code) not in (b"ok", b"unknown status")


@pytest.mark.parametrize("d,sq,sk", [(64, 128, 128), (64, 512, 512), (128, 1000, 1000), (32, 77, 300),
                                     (16, 4096, 4096), (128, 128, 129)])
def test_host_rules_match_oracle(d, sq, sk):
    from flash_attn_b200 import _lib
    assert _lib.lib.fa_mask_block_n(d, sk, 0) == orc.mask_block_n(d, sk)
    assert _lib.lib.fa_philox_increment(d, sq, sk, 0) == orc.philox_increment(d, sq, sk)
    assert _lib.lib.fa_mask_block_n(d, sk, 1) == 256


def test_workspace_size():
    from flash_attn_b200 import _lib
    assert _lib.lib.fa_bwd_workspace_bytes(1000, 12, 64) == 1000 * 12 * 64 * 4
    assert _lib.lib.fa_bwd_workspace_bytes(10, 2, 32) == 10 * 2 * 64 * 4
    assert _lib.lib.fa_bwd_workspace_bytes(10, 2, 128) == 10 * 2 * 128 * 4


def test_argument_errors_are_reported_without_a_gpu():
    from flash_attn_b200 import _lib
    p = _lib.FwdParams()
    rc = _lib.lib.fa_fwd(ctypes.byref(p), None)
    assert rc == _lib.FA_ERR_INVALID_ARGUMENT
    assert b"non-null" in _lib.lib.fa_last_error()
    with pytest.raises(RuntimeError, match="invalid argument"):
        _lib.check(rc)
    # bad head_dim
    p.q = p.k = p.v = p.o = p.softmax_lse = p.cu_seqlens_q = p.cu_seqlens_k = 256
    p.batch, p.heads, p.head_dim = 1, 1, 48
    assert _lib.lib.fa_fwd(ctypes.byref(p), None) == _lib.FA_ERR_INVALID_ARGUMENT
    assert b"head_dim" in _lib.lib.fa_last_error()
    bp = _lib.BwdParams()
    assert _lib.lib.fa_bwd(ctypes.byref(bp), None) == _lib.FA_ERR_INVALID_ARGUMENT


def test_packed_parameter_buffers_match_the_structures():
    """The binding fills fa_fwd_params / fa_bwd_params by packing all values into a buffer in one call;
    every value must land in the field the ctypes structure (and so the header) gives it."""
    from flash_attn_b200 import _lib
    from flash_attn_b200 import flash_attn_cuda as fc
    vals = list(range(1, 41))
    vals[27], vals[28] = 0.5, 0.25          # p_dropout, softmax_scale
    buf = bytearray(fc._FWD_PACK.size)
    fc._FWD_PACK.pack_into(buf, 0, *vals)
    p = _lib.FwdParams.from_buffer(buf)
    assert [(getattr(p, name) or 0) for name, _ in _lib.FwdParams._fields_] == vals
    tail = list(range(41, 56))
    buf = bytearray(fc._BWD_PACK.size)
    fc._BWD_PACK.pack_into(buf, 0, *(vals + tail))
    pb = _lib.BwdParams.from_buffer(buf)
    assert [(getattr(pb, name) or 0) for name, _ in _lib.BwdParams._fields_[1:]] == tail
    assert pb.fwd.blockmask_cols == 40 and pb.fwd.q == 1
