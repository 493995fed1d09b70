"""ctypes binding of ``libkata_attn.so`` (the C ABI in ``include/kata_attn.h``) for the tests and the benchmark.

torch is used only to own device memory and streams; every attention computation goes through the C ABI into the
hand-written CUDA kernels. There is no CPU or PyTorch fallback: if the library is missing, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkata_attn.so")

OK = 0
KV_FP16, KV_INT8, KV_INT8V, KV_INT8G = 0, 1, 2, 3
_KV_MODES = {"fp16": KV_FP16, "int8": KV_INT8, "int8v": KV_INT8V, "int8g": KV_INT8G}   # the reference's KATA_KV values (src/engine.cpp:54)
ROUND_RINT, ROUND_HALF_AWAY = 0, 1
ACT_F32, ACT_BF16, ACT_F16 = 0, 1, 2
_ACT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}   # KATA_ACT_*
QD, KVD, QFULL, MAX_BATCH = 6144, 1024, 12288, 64

EXPORTS = [
    "kata_attn_create", "kata_attn_destroy", "kata_attn_reset", "kata_attn_numerics_tag", "kata_attn_last_error", "kata_attn_check",
    "kata_attn_prep", "kata_attn_kv_quant", "kata_attn_decode", "kata_attn_decode_scalar", "kata_attn_prefill",
    "kata_attn_decode_partial", "kata_attn_merge_parts", "kata_attn_kv_planes", "kata_attn_kv_plane_row_bytes",
    "kata_attn_kv_plane_read", "kata_attn_kv_plane_write", "kata_attn_kv_plane_ptr", "kata_attn_mark_rows_written", "kata_attn_launch_count", "kata_attn_decode_static", "kata_attn_decode_static_check", "kata_attn_set_position_offset", "kata_attn_set_kv_heads", "kata_attn_out_fwht",
    "kata_attn_layers_step", "kata_attn_layers_decode", "kata_attn_prefill_plan", "kata_attn_decode_plan", "kata_attn_host_step_create", "kata_attn_host_step_destroy", "kata_attn_host_step_run",
    "kata_attn_peer_create", "kata_attn_peer_open", "kata_attn_peer_open_pointers", "kata_attn_peer_buffer", "kata_attn_peer_set_wait_polls", "kata_attn_peer_exchange_merge", "kata_attn_peer_decode", "kata_attn_peer_layers_step",
    "kata_attn_peer_check", "kata_attn_peer_resync", "kata_attn_peer_last_error", "kata_attn_peer_destroy",
    "kata_draft_create", "kata_draft_destroy", "kata_draft_reset", "kata_draft_last_error", "kata_draft_qk", "kata_draft_attn", "kata_draft_ring_ptr",
    "kata_draft_ring_read", "kata_draft_ring_write", "kata_draft_launch_count",
]


class Config(C.Structure):
    _fields_ = [("device", C.c_int32), ("n_layers", C.c_int32), ("n_seqs", C.c_int32), ("max_ctx", C.POINTER(C.c_int32)),
                ("kv_mode", C.c_int32), ("quant_round", C.c_int32), ("dec_chunk", C.c_int32), ("flags", C.c_int32)]


class KataError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"kata_attn error {code}: {msg}")
        self.code = code


_lib = None


def lib() -> C.CDLL:
    """Loads the library; raises if it has not been built (``python -m kata_b200.build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m kata_b200.build` (there is no fallback path)")
        L = C.CDLL(LIB_PATH)
        L.kata_attn_numerics_tag.restype = C.c_char_p
        L.kata_attn_last_error.restype = C.c_char_p
        L.kata_attn_kv_plane_row_bytes.restype = C.c_size_t
        L.kata_attn_kv_plane_ptr.restype = C.c_void_p
        L.kata_attn_launch_count.restype = C.c_uint64
        for name in EXPORTS:
            getattr(L, name)
        _lib = L
    return _lib


def _i32(xs):
    """ctypes int32 array of a list / numpy vector of small integers (about 1 us; the numpy route costs three times that per call)."""
    if isinstance(xs, np.ndarray):
        xs = xs.reshape(-1).tolist()
    a = (C.c_int32 * len(xs))(*[int(x) for x in xs])
    return a, a


def _dp(t):
    if t is None:
        return C.c_void_p(0)
    assert t.is_cuda and t.is_contiguous()
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def out_fwht(x, sign, out=None):
    """The engine's attention output transform (sign, 1024-point Walsh-Hadamard per block, 1/32): x [rows][width] fp32 on the GPU."""
    out = torch.empty_like(x) if out is None else out
    assert x.dtype == torch.float32 and sign.dtype == torch.float32 and x.dim() == 2
    rc = lib().kata_attn_out_fwht(_dp(x), _dp(sign), _dp(out), C.c_int64(x.shape[0]), C.c_int32(x.shape[1]), _stream())
    if rc != OK:
        raise KataError(rc, "kata_attn_out_fwht")
    return out


class AttnContext:
    """One context per GPU: the KV caches of ``len(max_ctx)`` sequences x ``n_layers`` layers plus all scratch."""

    def __init__(self, n_layers: int, max_ctx, kv_mode: str = "fp16", quant_round: str = "rint", device: int | None = None, dec_chunk: int = 0, legacy_prefill: bool = False, flags: int = 0):
        self.L = lib()
        self.device = torch.cuda.current_device() if device is None else device
        self.max_ctx, mp = _i32(max_ctx)
        self.n_layers, self.n_seqs = n_layers, len(self.max_ctx)
        if kv_mode not in _KV_MODES:
            raise ValueError(f"kv_mode {kv_mode!r}: one of {sorted(_KV_MODES)}")
        self.int8, self.kv_mode = kv_mode == "int8", kv_mode
        cfg = Config(self.device, n_layers, self.n_seqs, mp, _KV_MODES[kv_mode], ROUND_HALF_AWAY if quant_round == "half_away" else ROUND_RINT, dec_chunk, (1 if legacy_prefill else 0) | int(flags))
        self.h = C.c_void_p()
        rc = self.L.kata_attn_create(C.byref(cfg), C.byref(self.h))
        if rc != OK:
            raise KataError(rc, "kata_attn_create failed")

    def close(self):
        if self.h:
            self.L.kata_attn_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, rc):
        if rc != OK:
            raise KataError(rc, self.L.kata_attn_last_error(self.h).decode())

    def tag(self) -> str:
        return self.L.kata_attn_numerics_tag(self.h).decode()

    def reset(self):
        self._ck(self.L.kata_attn_reset(self.h, _stream()))

    def check(self):
        self._ck(self.L.kata_attn_check(self.h, _stream()))

    def set_position_offset(self, seq: int, first_position: int):
        self._ck(self.L.kata_attn_set_position_offset(self.h, seq, first_position))

    def set_kv_heads(self, kv_head_lo: int, kv_head_n: int):
        """This context computes KV heads [lo, lo + n) only (a rank of a head-sharded group)."""
        self._ck(self.L.kata_attn_set_kv_heads(self.h, kv_head_lo, kv_head_n))

    def launches(self) -> int:
        return int(self.L.kata_attn_launch_count(self.h))

    def prep(self, layer, seq_ids, pos0, T, qfull, kproj, vproj, qnorm, knorm, h0=0, nh=32, q16=None, q32=None, gate=None, want_q32=False):
        """Returns (q16, q32 or None, gate). qfull [n][T][12288], kproj/vproj [n][T][1024] in fp32 or bf16."""
        sa, sp = _i32(seq_ids)
        pa, pp = _i32(pos0)
        n = len(sa)
        ref = kproj if kproj is not None else qfull
        act = _ACT[ref.dtype]
        dev = ref.device
        if h0 < 24:
            q16 = torch.empty((n, T, QD), dtype=torch.float16, device=dev) if q16 is None else q16
            gate = torch.empty((n, T, QD), dtype=torch.float32, device=dev) if gate is None else gate
            if want_q32 and q32 is None:
                q32 = torch.empty((n, T, QD), dtype=torch.float32, device=dev)
        self._ck(self.L.kata_attn_prep(self.h, layer, n, sp, pp, T, _dp(qfull), _dp(kproj), _dp(vproj), act, _dp(qnorm), _dp(knorm),
                                       _dp(q16), _dp(q32), _dp(gate), h0, nh, _stream()))
        return q16, q32, gate

    def layers_step(self, n_layers, seq_ids, pos0, T, qfull, kproj, vproj, qnorm, knorm, q16, gate, out, first_pos=0):
        """prep + decode of layers 0..n_layers-1 in one call; every tensor is [n_layers][...] on the device."""
        sa, sp = _i32(seq_ids); pa, pp = _i32(pos0)
        self._ck(self.L.kata_attn_layers_step(self.h, n_layers, len(sa), sp, pp, T, first_pos, _dp(qfull), _dp(kproj), _dp(vproj), _ACT[qfull.dtype], _dp(qnorm), _dp(knorm),
                                              _dp(q16), _dp(gate), _dp(out), _ACT[out.dtype], _stream()))
        return out

    def layers_decode(self, n_layers, seq_ids, pos_base, T, q16, gate, out, first_pos=0):
        """kata_attn_decode of layers 0..n_layers-1 in one call (the attention kernels by themselves); tensors are [n_layers][...]."""
        sa, sp = _i32(seq_ids); pa, pp = _i32(pos_base)
        self._ck(self.L.kata_attn_layers_decode(self.h, n_layers, len(sa), sp, pp, T, first_pos, _dp(q16), _dp(gate), _dp(out), _ACT[out.dtype], _stream()))
        return out

    def kv_quant(self, layer, seq, ks, vs, pos0):
        self._ck(self.L.kata_attn_kv_quant(self.h, layer, seq, _dp(ks), _dp(vs), vs.shape[0], pos0, _stream()))   # ks may be None on an int8v context

    def decode(self, layer, seq_ids, pos_base, T, q16, gate, first_pos=0, out=None, out_dtype=torch.float32):
        sa, sp = _i32(seq_ids)
        pa, pp = _i32(pos_base)
        n = len(sa)
        out = torch.empty((n, T, QD), dtype=out_dtype, device=q16.device) if out is None else out
        self._ck(self.L.kata_attn_decode(self.h, layer, n, sp, pp, T, first_pos, _dp(q16), _dp(gate), _dp(out), _ACT[out.dtype], _stream()))
        return out

    def decode_scalar(self, layer, seq_ids, pos_base, T, q32, gate, first_pos=0, out=None):
        sa, sp = _i32(seq_ids)
        pa, pp = _i32(pos_base)
        n = len(sa)
        out = torch.empty((n, T, QD), dtype=torch.float32, device=q32.device) if out is None else out
        self._ck(self.L.kata_attn_decode_scalar(self.h, layer, n, sp, pp, T, first_pos, _dp(q32), _dp(gate), _dp(out), _stream()))
        return out

    def prefill(self, layer, seq_ids, pos_base, M, q16, gate, out=None, out_dtype=torch.float32):
        sa, sp = _i32(seq_ids)
        pa, pp = _i32(pos_base)
        n = len(sa)
        out = torch.empty((n, M, QD), dtype=out_dtype, device=q16.device) if out is None else out
        self._ck(self.L.kata_attn_prefill(self.h, layer, n, sp, pp, M, _dp(q16), _dp(gate), _dp(out), _ACT[out.dtype], _stream()))
        return out

    def decode_partial(self, layer, seq, pos_base, T, key_lo, key_hi, q16, part=None):
        part = torch.empty((T * 24, 258), dtype=torch.float32, device=q16.device) if part is None else part
        self._ck(self.L.kata_attn_decode_partial(self.h, layer, seq, pos_base, T, key_lo, key_hi, _dp(q16), _dp(part), _stream()))
        return part

    def merge_parts(self, parts, T, gate, out=None, out_dtype=torch.float32):
        n_parts = parts.shape[0]
        out = torch.empty((T, QD), dtype=out_dtype, device=parts.device) if out is None else out
        self._ck(self.L.kata_attn_merge_parts(self.h, _dp(parts), n_parts, T, _dp(gate), _dp(out), _ACT[out.dtype], _stream()))
        return out

    # ---- KV planes (prefix-cache contract) ----
    def kv_planes(self) -> int:
        return int(self.L.kata_attn_kv_planes(self.h))

    def plane_row_bytes(self, plane: int) -> int:
        return int(self.L.kata_attn_kv_plane_row_bytes(self.h, plane))

    def plane_read(self, layer, seq, plane, row0, nrows) -> np.ndarray:
        buf = np.empty(nrows * self.plane_row_bytes(plane), np.uint8)
        self._ck(self.L.kata_attn_kv_plane_read(self.h, layer, seq, plane, row0, nrows, buf.ctypes.data_as(C.c_void_p)))
        return buf

    def plane_write(self, layer, seq, plane, row0, data: np.ndarray):
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        rb = self.plane_row_bytes(plane)
        assert rb and data.size % rb == 0
        self._ck(self.L.kata_attn_kv_plane_write(self.h, layer, seq, plane, row0, data.size // rb, data.ctypes.data_as(C.c_void_p)))

    def plane_ptr(self, layer, seq, plane) -> int:
        return int(self.L.kata_attn_kv_plane_ptr(self.h, layer, seq, plane) or 0)

    def mark_rows_written(self, seq: int, pos_lo: int):
        self._ck(self.L.kata_attn_mark_rows_written(self.h, seq, pos_lo))

    def plane_tensor(self, layer, seq, plane, nrows) -> torch.Tensor:
        """A uint8 CUDA tensor [nrows][row bytes] aliasing the plane's rows (through kata_attn_kv_plane_ptr): lets a test write rows with a
        device-side copy, as a device-resident restore would."""
        rb = self.plane_row_bytes(plane)

        class _Alias:
            __cuda_array_interface__ = {"shape": (nrows, rb), "typestr": "|u1", "data": (self.plane_ptr(layer, seq, plane), False), "version": 3, "strides": None}
        return torch.as_tensor(_Alias(), device=torch.device("cuda", self.device))


def decode_static(k_rows, v_rows, seq_row0, pos_base, T, q16, gate, first_pos=0, out=None, out_dtype=torch.float32):
    """kata_attn_decode_static: decode over caller-owned fp16 K/V rows ([rows][1024] tensors) with no context and no
    allocation inside the library. Returns (status code, out)."""
    L = lib()
    n = len(pos_base)
    rows0 = (C.c_int64 * n)(*[int(x) for x in seq_row0])
    pa, pp = _i32(pos_base)
    out = torch.empty((n, T, QD), dtype=out_dtype, device=q16.device) if out is None else out
    rc = L.kata_attn_decode_static(_dp(k_rows), _dp(v_rows), C.c_int64(k_rows.shape[0]), n, rows0, pp, T, first_pos, _dp(q16), _dp(gate), _dp(out),
                                   _ACT[out.dtype], _stream())
    return rc, out


class DraftConfig(C.Structure):
    _fields_ = [("device", C.c_int32), ("n_layers", C.c_int32), ("ring", C.c_int32), ("window", C.c_int32)]


class DraftContext:
    """The block drafter's K/V rings and attention (include/kata_draft.h; Draft::kbuf/vbuf, src/draft.h:36)."""

    def __init__(self, n_layers: int = 5, ring: int = 4096, window: int = 2048, device: int | None = None):
        self.L = lib()
        self.L.kata_draft_last_error.restype = C.c_char_p
        self.L.kata_draft_ring_ptr.restype = C.c_void_p
        self.L.kata_draft_launch_count.restype = C.c_uint64
        self.device = torch.cuda.current_device() if device is None else device
        self.n_layers, self.ring, self.window = n_layers, ring, window
        self.h = C.c_void_p()
        cfg = DraftConfig(self.device, n_layers, ring, window)
        rc = self.L.kata_draft_create(C.byref(cfg), C.byref(self.h))
        if rc != OK:
            raise KataError(rc, "kata_draft_create failed")

    def close(self):
        if self.h:
            self.L.kata_draft_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, rc):
        if rc != OK:
            raise KataError(rc, self.L.kata_draft_last_error(self.h).decode())

    def reset(self):
        self._ck(self.L.kata_draft_reset(self.h, _stream()))

    def launches(self) -> int:
        return int(self.L.kata_draft_launch_count(self.h))

    def qk(self, layer, qin, kin, vin, qnorm, knorm, pos0, out=None):
        """k_draft_qk (returns the fp32 query rows) or, with qin None, k_draft_ctx_kv."""
        T = kin.shape[0]
        qout = (torch.empty((T, 4096), dtype=torch.float32, device=kin.device) if out is None else out) if qin is not None else None
        self._ck(self.L.kata_draft_qk(self.h, layer, _dp(qin), _dp(kin), _dp(vin), _dp(qnorm), _dp(knorm), _dp(qout), pos0, T, _stream()))
        return qout

    def attn(self, layer, q, pos0, out=None):
        T = q.shape[0]
        out = torch.empty((T, 4096), dtype=torch.float32, device=q.device) if out is None else out
        self._ck(self.L.kata_draft_attn(self.h, layer, _dp(q), _dp(out), pos0, T, _stream()))
        return out

    def ring_read(self, layer, value: bool, row0: int = 0, nrows: int | None = None) -> np.ndarray:
        nrows = self.ring - row0 if nrows is None else nrows
        buf = np.empty((nrows, 1024), np.uint16)
        self._ck(self.L.kata_draft_ring_read(self.h, layer, int(value), row0, nrows, buf.ctypes.data_as(C.c_void_p)))
        return buf

    def ring_write(self, layer, value: bool, row0: int, data: np.ndarray):
        data = np.ascontiguousarray(data).view(np.uint16).reshape(-1, 1024)
        self._ck(self.L.kata_draft_ring_write(self.h, layer, int(value), row0, data.shape[0], data.ctypes.data_as(C.c_void_p)))


class HostStep:
    """A decode or verify step of all layers with the projections and the output rows in pinned host memory (kata_attn_host_step_*):
    the copies of the neighbouring layers run under the layer that computes."""

    def __init__(self, ctx: "AttnContext", max_n: int, max_T: int = 1, act_dtype=torch.float32):
        self.L = lib(); self.ctx = ctx; self.h = C.c_void_p(); self.act = act_dtype
        rc = self.L.kata_attn_host_step_create(ctx.h, ctx.device, max_n, max_T, _ACT[act_dtype], C.byref(self.h))
        if rc != OK:
            raise KataError(rc, "kata_attn_host_step_create failed")

    def run(self, n_layers, seq_ids, pos0, T, h_qfull, h_kproj, h_vproj, d_qnorm, d_knorm, h_out, first_pos=0):
        """h_*: pinned host tensors [n_layers][n][T][...]; d_qnorm, d_knorm: device [n_layers][256]. Enqueued on the current stream."""
        sa, sp = _i32(seq_ids); pa, pp = _i32(pos0)
        for t in (h_qfull, h_kproj, h_vproj, h_out):
            assert t.device.type == "cpu" and t.is_contiguous()
        rc = self.L.kata_attn_host_step_run(self.h, n_layers, len(sa), sp, pp, T, first_pos, C.c_void_p(h_qfull.data_ptr()), C.c_void_p(h_kproj.data_ptr()), C.c_void_p(h_vproj.data_ptr()),
                                            _dp(d_qnorm), _dp(d_knorm), C.c_void_p(h_out.data_ptr()), _stream())
        if rc != OK:
            raise KataError(rc, self.L.kata_attn_last_error(self.ctx.h).decode() or "kata_attn_host_step_run failed")
        return h_out

    def close(self):
        if self.h:
            self.L.kata_attn_host_step_destroy(self.h); self.h = C.c_void_p()


class PeerExchange:
    """Push-and-merge of the split-KV parts between the GPUs of one box (kata_attn_peer_*): one process per GPU, handles swapped
    through ``torch.distributed`` object collectives (host side, once); the per-layer exchange itself runs no library collective."""

    def __init__(self, rank: int, world: int, device: int | None = None, group=None, buffers=None):
        self.L = lib()
        self.L.kata_attn_peer_last_error.restype = C.c_char_p
        self.L.kata_attn_peer_buffer.restype = C.c_void_p
        self.rank, self.world = rank, world
        self.device = torch.cuda.current_device() if device is None else device
        self.h = C.c_void_p()
        handle = (C.c_ubyte * 64)()
        rc = self.L.kata_attn_peer_create(self.device, rank, world, C.byref(self.h), handle)
        if rc != OK:
            raise KataError(rc, "kata_attn_peer_create failed")
        if buffers is not None:       # same process: device addresses of every rank's buffer (tests)
            self.open_pointers(buffers)
        elif world > 1 and group is not False:
            import torch.distributed as dist
            got = [None] * world
            dist.all_gather_object(got, bytes(handle), group=group)
            blob = (C.c_ubyte * (64 * world)).from_buffer_copy(b"".join(got))
            self._ck(self.L.kata_attn_peer_open(self.h, blob))

    def buffer(self) -> int:
        return int(self.L.kata_attn_peer_buffer(self.h) or 0)

    def open_pointers(self, buffers):
        arr = (C.c_void_p * self.world)(*[C.c_void_p(int(b)) for b in buffers])
        self._ck(self.L.kata_attn_peer_open_pointers(self.h, arr))

    def set_wait_polls(self, polls: int):
        self._ck(self.L.kata_attn_peer_set_wait_polls(self.h, C.c_uint32(polls)))

    def _ck(self, rc):
        if rc != OK:
            raise KataError(rc, self.L.kata_attn_peer_last_error(self.h).decode())

    def exchange_merge(self, part, T, gate, out=None, out_dtype=torch.float32):
        out = torch.empty((T, QD), dtype=out_dtype, device=part.device) if out is None else out
        self._ck(self.L.kata_attn_peer_exchange_merge(self.h, _dp(part), T, _dp(gate), _dp(out), _ACT[out.dtype], _stream()))
        return out

    def decode(self, ctx, layer, seq, pos_base, T, key_lo, key_hi, q16, gate, out=None, out_dtype=torch.float32):
        """This rank's share of a decode whose keys are split across the ranks, exchange and merge included (kata_attn_peer_decode)."""
        out = torch.empty((T, QD), dtype=out_dtype, device=q16.device) if out is None else out
        self._ck(self.L.kata_attn_peer_decode(self.h, ctx.h, layer, seq, pos_base, T, key_lo, key_hi, _dp(q16), _dp(gate), _dp(out), _ACT[out.dtype], _stream()))
        return out

    def layers_step(self, ctx, n_layers, seq, pos, T, key_lo, key_hi, appends, qfull, kproj, vproj, qnorm, knorm, q16, gate, out):
        """prep + split-KV decode of layers 0..n_layers-1 in one call (kata_attn_peer_layers_step); every tensor is [n_layers][T][...] on the device."""
        self._ck(self.L.kata_attn_peer_layers_step(self.h, ctx.h, n_layers, seq, pos, T, key_lo, key_hi, 1 if appends else 0, _dp(qfull), _dp(kproj), _dp(vproj), _ACT[qfull.dtype],
                                                   _dp(qnorm), _dp(knorm), _dp(q16), _dp(gate), _dp(out), _ACT[out.dtype], _stream()))
        return out

    def check(self):
        self._ck(self.L.kata_attn_peer_check(self.h, _stream()))

    def resync(self, call_number: int):
        self._ck(self.L.kata_attn_peer_resync(self.h, C.c_uint32(call_number)))

    def close(self):
        if self.h:
            self.L.kata_attn_peer_destroy(self.h)
            self.h = C.c_void_p()
