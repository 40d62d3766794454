"""The drop-in boundary by its module name: `import flash_attn_cuda` must give the four entry
points with the positional argument lists the reference's Python call sites pass
(flash_attn/flash_attn_interface.py:19-22, :31-33; flash_attn/flash_blocksparse_attn_interface.py:
45-47, :56-58).  The expected arities below are those of the cited lines; when the environment
variable FA_REFERENCE_ROOT points at a checkout of the reference they are re-read from its source."""
import ast
import inspect
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "flash-attention_b200")

# entry point -> number of positional arguments at the reference's call site
CALL_SITE_ARITY = {"fwd": 13, "bwd": 18, "fwd_block": 9, "bwd_block": 12}


def _import_by_name():
    if PKG_DIR not in sys.path:
        sys.path.insert(0, PKG_DIR)
    sys.modules.pop("flash_attn_cuda", None)
    import flash_attn_cuda
    return flash_attn_cuda


def _accepts(fn, n):
    arities = getattr(fn, "accepted_arities", None)
    if arities is not None:
        return n in arities
    try:
        inspect.signature(fn).bind(*([None] * n))
        return True
    except TypeError:
        return False


def test_module_name_and_entry_points():
    mod = _import_by_name()
    assert os.path.dirname(os.path.abspath(mod.__file__)) == PKG_DIR
    for name, n in CALL_SITE_ARITY.items():
        fn = getattr(mod, name)
        assert callable(fn)
        assert _accepts(fn, n), "%s does not take the %d arguments of the reference's call site" % (name, n)
    # the C++ signatures of the block-sparse entries (csrc/flash_attn/fmha_api.cpp:451-464, :575-594)
    assert _accepts(mod.fwd_block, 13) and _accepts(mod.bwd_block, 18)
    # one argument less or more is an error, as with the compiled extension
    assert not _accepts(mod.fwd, 14 + 1) and not _accepts(mod.fwd_block, 10)
    with pytest.raises(TypeError):
        mod.fwd_block(*([None] * 10))
    with pytest.raises(TypeError):
        mod.bwd_block(*([None] * 13))


def _call_site_arities(path):
    found = {}
    for node in ast.walk(ast.parse(open(path).read())):
        if (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute)
                and isinstance(node.func.value, ast.Name) and node.func.value.id == "flash_attn_cuda"):
            assert not node.keywords, "the reference passes positional arguments only"
            found[node.func.attr] = len(node.args)
    return found


def test_arities_against_the_reference_source():
    ref = os.environ.get("FA_REFERENCE_ROOT")
    if not ref or not os.path.isdir(os.path.join(ref, "flash_attn")):
        pytest.skip("FA_REFERENCE_ROOT does not point at a checkout of the reference")
    found = {}
    found.update(_call_site_arities(os.path.join(ref, "flash_attn", "flash_attn_interface.py")))
    found.update(_call_site_arities(os.path.join(ref, "flash_attn", "flash_blocksparse_attn_interface.py")))
    assert found == CALL_SITE_ARITY
