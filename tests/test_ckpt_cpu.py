"""CPU tests of the checkpoint-file logic (include/kata_ckpt.h): segment layout, prefix hashes, and the acceptance checks
on files built here byte by byte from the format the reference documents in src/ckpt.cpp:16-34 (header fields, 4 KiB
alignment) - including the reference's own regression cases: a truncated file and a file of another numerics tag are ignored."""
import ctypes as C
import os
import struct

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ALIGN, VOCAB = 4096, 248320


def _lib():
    from kata_b200 import build
    L = C.CDLL(build.build())
    return L


def _up(x):
    return (x + ALIGN - 1) // ALIGN * ALIGN


def _fnv(tokens):
    a, b = 1469598103934665603, 0x9E3779B97F4A7C15
    for byte in np.asarray(tokens, np.int32).tobytes():
        a = ((a ^ byte) * 1099511628211) & (2**64 - 1)
        b = ((b ^ byte ^ 0x5bd1e995) * 0x100000001b3) & (2**64 - 1)
    return a, b


def _make_file(path, tokens, fp, tag, n_attn, kv_row, gdn, conv, mtp, truncate=0):
    n = len(tokens)
    t_off = ALIGN; g_off = _up(t_off + 4 * n); c_off = _up(g_off + gdn); k_off = _up(c_off + conv)
    m_off = _up(k_off + n_attn * n * kv_row); h_off = _up(m_off + (2 * n * 2048 if mtp else 0)); l_off = _up(h_off + (20480 if mtp else 0)); total = l_off + VOCAB * 4
    h0, h1 = _fnv(tokens)
    hdr = struct.pack("<8sIIQ64sIIIIQQQQii8Q", b"BNSCKPT1", 2, n, fp, tag.encode(), int(mtp), n_attn, kv_row, 0, gdn, conv, h0, h1, 7, 0, t_off, g_off, c_off, k_off, m_off, h_off, l_off, total)
    with open(path, "wb") as f:
        f.write(hdr); f.seek(t_off); f.write(np.asarray(tokens, np.int32).tobytes()); f.truncate(total - truncate)
    return [t_off, g_off, c_off, k_off, m_off, h_off, l_off, total]


def test_layout_and_hashes_match_the_documented_format():
    L = _lib()
    out = (C.c_uint64 * 8)()
    n, gdn, conv, n_attn, kv_row = 3600, 48 * 48 * 128 * 128 * 4, 48 * 3 * 10240 * 4, 16, 4096
    L.kata_ckpt_layout(n, C.c_uint64(gdn), C.c_uint64(conv), n_attn, kv_row, 1, out)
    t_off = ALIGN; g_off = _up(t_off + 4 * n); c_off = _up(g_off + gdn); k_off = _up(c_off + conv); m_off = _up(k_off + n_attn * n * kv_row)
    h_off = _up(m_off + 2 * n * 2048); l_off = _up(h_off + 20480)
    assert list(out) == [t_off, g_off, c_off, k_off, m_off, h_off, l_off, l_off + VOCAB * 4]
    toks = np.arange(100, 100 + 57, dtype=np.int32)
    h = (C.c_uint64 * 2)(); L.kata_ckpt_prefix_hash(toks.ctypes.data_as(C.c_void_p), 57, h)
    assert (h[0], h[1]) == _fnv(toks)


def test_probe_accepts_complete_and_rejects_truncated_or_foreign(tmp_path):
    L = _lib()
    toks = np.arange(5, 5 + 300, dtype=np.int32); prompt = np.concatenate([toks, np.arange(9000, 9050, dtype=np.int32)])
    path = str(tmp_path / "a.ckpt").encode()
    _make_file(path, toks, 0xABCDEF, "fp16", 16, 4096, 1000, 2000, True)
    n = C.c_uint32()
    probe = lambda p, tk, fp=0xABCDEF, tag=b"fp16", kvr=4096: L.kata_ckpt_probe(p, tk.ctypes.data_as(C.c_void_p), len(tk), C.c_uint64(fp), tag, 16, kvr, C.c_uint64(1000), C.c_uint64(2000), 1, C.byref(n))
    assert probe(path, prompt) == 0 and n.value == 300
    assert probe(path, prompt, tag=b"fp16+kv8") == 2          # another numerics mode never reuses the file
    assert probe(path, prompt, fp=1) == 2 and probe(path, prompt, kvr=2064) == 2
    other = prompt.copy(); other[10] += 1
    assert probe(path, other) == 2                            # not a prefix of this prompt
    assert probe(path, toks[:200]) == 2                       # checkpoint longer than the prompt
    p2 = str(tmp_path / "b.ckpt").encode()
    _make_file(p2, toks, 0xABCDEF, "fp16", 16, 4096, 1000, 2000, True, truncate=1)
    assert probe(p2, prompt) == 2                             # truncated file: ignored (tools/test_cache.sh:22-24)
    assert probe(str(tmp_path / "missing.ckpt").encode(), prompt) == 1
