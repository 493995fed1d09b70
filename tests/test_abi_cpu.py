"""CPU checks of the boundary: the C-ABI library loads without a GPU and exports every function the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


HEADERS = (("kata_attn.h", "kata_attn_"), ("kata_draft.h", "kata_draft_"))
ALL_HEADERS = HEADERS + (("kata_ckpt.h", "kata_ckpt_"), ("kata_engine.h", "kata_engine_"))


def _declared(HEADERS=HEADERS):
    names = set()
    for header, prefix in HEADERS:
        src = open(os.path.join(ROOT, "include", header)).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        names |= set(re.findall(r"\b(" + prefix + r"[a-z0-9_]+)\s*\(", src))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    from kata_b200 import build
    path = build.build()
    lib = ctypes.CDLL(path)
    names = _declared(ALL_HEADERS)
    assert len(names) >= 60 and "kata_ckpt_publish" in names and "kata_engine_mtp_rows_attn" in names
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
    assert lib.kata_engine_step_attn(None, 0, 0, None, None, None, None, None, None, None, None, None) == 1 and lib.kata_engine_kv_planes(None) == 0
    assert lib.kata_ckpt_publish(None) == 1 and lib.kata_attn_mark_rows_written(None, 0, 0) == 1 and lib.kata_attn_peer_resync(None, 1) == 1
    assert lib.kata_draft_create(None, None) == 1 and lib.kata_draft_destroy(None) == 1 and lib.kata_draft_attn(None, 0, None, None, 0, 1, None) == 1
