"""Front end of ``oracle/_ref/libprobe_ref.so``: the reference's own CPU check of the attention path
(tools/probe_flash.cpp: input recipe lines 16-19, NaN poison and fp64 comparison lines 26-34) compiled here from the
reference's own lines by ``make -C oracle ref``.

TEST INFRASTRUCTURE ONLY (used by ``tests/``). The library is built when the reference checkout is present; the built
file is what other machines use. ``run(kernel)`` executes the reference's procedure with ``kernel`` standing in for the
Metal dispatch: the reference's loop compares what ``kernel`` wrote with its fp64 formula and reports the worst
difference, and the fp64 values themselves are read back through the recorder described in ``probe_ref_shim.h``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libprobe_ref.so")
MAX_CTX, PB, M = 8448, 300, 70          # tools/probe_flash.cpp:13, 26
T_STEP, H_STEP = 3, 5                   # tools/probe_flash.cpp:29


def reference_root() -> str:
    return os.environ.get("REF", os.path.abspath(os.path.join(_HERE, "..", "..", "reference")))


def build() -> str | None:
    """Builds the library if the reference checkout is there; returns its path, or None when neither exists."""
    src = os.path.join(reference_root(), "tools", "probe_flash.cpp")
    if os.path.exists(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "ref", f"REF={reference_root()}"])
    return LIB_PATH if os.path.exists(LIB_PATH) else None


_KERNEL = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p)


class ProbeResult:
    def __init__(self, worst, mx, bad, ref, q16, k, v, gate):
        self.worst, self.max_ref, self.non_finite = worst, mx, bad   # what the reference's printf reports (line 35)
        self.ref = ref                                               # fp64 reference values [24 tokens][5 heads][256]
        self.q16, self.k, self.v, self.gate = q16, k, v, gate        # the reference's inputs (fp16 bit patterns / fp32)


def run(kernel) -> ProbeResult:
    """kernel(q16 [1024][6144] u16, k, v [8448][1024] u16, gate [1024][6144] f32, pos_base, M) -> out [M][6144] f32."""
    path = build()
    if path is None:
        raise FileNotFoundError("oracle/_ref/libprobe_ref.so is missing and there is no reference checkout to build it from")
    L = C.CDLL(path)
    L.probe_ref_buffer.restype = C.c_void_p
    L.probe_ref_taps.restype = C.c_uint64

    def view(i, n, dt):
        return np.ctypeslib.as_array(C.cast(L.probe_ref_buffer(i), C.POINTER(C.c_uint8)), shape=(n * np.dtype(dt).itemsize,)).view(dt)

    def cb(q, kc, vc, gate, out, pos_base, m, _user):
        k = view(0, MAX_CTX * 1024, np.uint16).reshape(MAX_CTX, 1024); v = view(1, MAX_CTX * 1024, np.uint16).reshape(MAX_CTX, 1024)
        q16 = view(2, 1024 * 6144, np.uint16).reshape(1024, 6144); g = view(3, 1024 * 6144, np.float32).reshape(1024, 6144)
        o = view(4, 1024 * 6144, np.float32).reshape(1024, 6144)
        o[:m] = 0.0 if kernel is None else np.asarray(kernel(q16, k, v, g, int(pos_base), int(m)), np.float32).reshape(m, 6144)

    stats = (C.c_double * 3)()
    fn = _KERNEL(cb)
    L.probe_ref_run(fn, None, stats)
    p = C.POINTER(C.c_double)()
    n = int(L.probe_ref_taps(C.byref(p)))
    taps = np.ctypeslib.as_array(p, shape=(n,)).copy()
    nt, nh = (M + T_STEP - 1) // T_STEP, (24 + H_STEP - 1) // H_STEP
    assert n == 3 * nt * nh * 256, n
    diff = taps.reshape(nt, nh, 256, 3)[..., 0]                      # g - a, with g the float the kernel wrote
    o = view(4, 1024 * 6144, np.float32).reshape(1024, 6144)[:M].reshape(M, 24, 256)[::T_STEP, ::H_STEP].astype(np.float64)
    ref = o - diff                                                   # exact when the kernel wrote zeros (kernel=None)
    return ProbeResult(float(stats[0]), float(stats[1]), int(stats[2]), ref,
                       view(2, 1024 * 6144, np.uint16).reshape(1024, 6144)[:M].copy(), view(0, MAX_CTX * 1024, np.uint16).reshape(MAX_CTX, 1024).copy(),
                       view(1, MAX_CTX * 1024, np.uint16).reshape(MAX_CTX, 1024).copy(), view(3, 1024 * 6144, np.float32).reshape(1024, 6144)[:M].copy())
