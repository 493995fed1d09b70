"""CPU checks of the boundary: the C-ABI library loads without a GPU and exports every function the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    for header, prefix in (("kata_attn.h", "kata_attn_"), ("kata_draft.h", "kata_draft_")):
        src = open(os.path.join(ROOT, "include", header)).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        names |= set(re.findall(r"\b(" + prefix + r"[a-z0-9_]+)\s*\(", src))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    from kata_b200 import build
    path = build.build()
    lib = ctypes.CDLL(path)
    names = _declared()
    assert len(names) >= 29
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ but not exported"


def test_binding_lists_the_same_symbols():
    from kata_b200 import capi
    assert sorted(capi.EXPORTS) == [n for n in _declared() if n != "kata_attn_ctx"]


def test_null_arguments_are_rejected_without_a_device():
    from kata_b200 import build
    lib = ctypes.CDLL(build.build())
    assert lib.kata_attn_create(None, None) == 1          # KATA_ERR_ARG
    assert lib.kata_attn_destroy(None) == 1
    assert lib.kata_attn_kv_planes(None) == 0
    lib.kata_attn_last_error.restype = ctypes.c_char_p
    assert lib.kata_attn_last_error(None) == b"null context"
    assert lib.kata_draft_create(None, None) == 1 and lib.kata_draft_destroy(None) == 1 and lib.kata_draft_attn(None, 0, None, None, 0, 1, None) == 1
